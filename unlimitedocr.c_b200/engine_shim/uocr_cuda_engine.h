/* Engine-side glue of the "cuda" backend: what the engine's open / close path calls, the counterpart of the
 * uocr_metal_context_create / _set_profile / _set_memory_tracker / _map_model sequence of the reference's
 * src/core/uocr_api.c:941-970 and of uocr_metal_context_destroy in uocr_engine_close (:980).  This file is compiled
 * together with the reference's own sources (it includes their headers), never without them; the kernels live behind
 * the C ABI of include/uocr_cuda_moe.h. */
#ifndef UOCR_CUDA_ENGINE_H
#define UOCR_CUDA_ENGINE_H

#include <stddef.h>
#include <stdint.h>

#include "model/uocr_model_file.h"
#include "runtime/uocr_memory.h"
#include "runtime/uocr_profile.h"

struct uocr_cuda_context;

/* 1 when a CUDA device can be used; otherwise 0 and the reason in why (the shape of backend_supported, uocr_api.c:807-830) */
int uocr_cuda_engine_supported(char *why, size_t why_size);

/* Creates the backend context, hands it the engine's profile store and memory tracker, maps the MoE layers of the
 * opened model file (file may be NULL: an engine without a model) and allocates the MoE scratch for
 * max_batch x max_prompt_tokens tokens.  NULL and a message on failure. */
struct uocr_cuda_context *uocr_cuda_engine_attach(const uocr_model_file *file, uocr_profile_state *profile, uocr_memory_tracker *tracker,
                                                  uint32_t max_batch, uint32_t max_prompt_tokens, char *error, size_t error_size);

/* Frees the device memory (the tracker sees the releases) and the context.  NULL is allowed. */
void uocr_cuda_engine_detach(struct uocr_cuda_context *ctx);

#endif /* UOCR_CUDA_ENGINE_H */

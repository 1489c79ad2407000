#include "uocr_cuda_engine.h"

#include <stdio.h>
#include <string.h>

#include "model/uocr_constants.h"
#include "uocr_cuda_moe.h"

/* the engine's accounting functions behind the callback types of the backend (an enum parameter there, an int here) */
static int reserve_bytes(uocr_memory_tracker *tracker, int category, uint64_t bytes) {
    return uocr_memory_reserve(tracker, (uocr_memory_category)category, bytes);
}
static int release_bytes(uocr_memory_tracker *tracker, int category, uint64_t bytes) {
    return uocr_memory_release(tracker, (uocr_memory_category)category, bytes);
}
static void add_event_ms(uocr_profile_state *profile, const char *name, double elapsed_ms) {
    uocr_profile_add_event_ms(profile, name, elapsed_ms);
}

int uocr_cuda_engine_supported(char *why, size_t why_size) {
    if (uocr_cuda_is_available()) return 1;
    if (why != NULL && why_size != 0u) (void)snprintf(why, why_size, "CUDA backend is compiled but no CUDA device is available");
    return 0;
}

struct uocr_cuda_context *uocr_cuda_engine_attach(const uocr_model_file *file, uocr_profile_state *profile, uocr_memory_tracker *tracker,
                                                  uint32_t max_batch, uint32_t max_prompt_tokens, char *error, size_t error_size) {
    uocr_cuda_context *ctx = uocr_cuda_context_create(NULL, error, error_size);
    if (ctx == NULL) return NULL;
    uocr_cuda_context_set_profile(ctx, profile, add_event_ms);
    uocr_cuda_context_set_memory_tracker(ctx, tracker, reserve_bytes, release_bytes);
    if (file != NULL) {
        const uocr_config_record *cfg = file->config;
        uocr_cuda_model_file_view view;
        memset(&view, 0, sizeof(view));
        view.data = file->data;
        view.size = (uint64_t)file->size;
        view.tensors = file->tensors;
        view.tensor_count = file->tensor_count;
        view.routed_experts = cfg->routed_experts;
        view.moe_top_k = cfg->moe_top_k;
        view.first_moe_layer = cfg->dense_first_layers;                       /* decoder layers 1 .. 11 are MoE layers */
        view.moe_layer_count = cfg->decoder_layers > cfg->dense_first_layers ? cfg->decoder_layers - cfg->dense_first_layers : 0u;
        view.routed_scaling_factor = UOCR_MOE_ROUTED_SCALING_FACTOR;
        if (!uocr_cuda_context_map_model(ctx, &view, error, error_size)) {
            uocr_cuda_context_destroy(ctx);
            return NULL;
        }
        if (uocr_cuda_context_moe_layer_count(ctx) != 0u) {
            const uint64_t tokens = (uint64_t)(max_batch != 0u ? max_batch : 1u) * (uint64_t)(max_prompt_tokens != 0u ? max_prompt_tokens : 1u);
            const uint32_t capacity = tokens > 65536u ? 65536u : (uint32_t)tokens;
            /* what the file holds either side of the MoE layers: layer 0's dense MLP, the LM head, the norm weights */
            if (!uocr_cuda_context_map_model_neighbours(ctx, &view, capacity, error, error_size)) {
                uocr_cuda_context_destroy(ctx);
                return NULL;
            }
            if (!uocr_cuda_context_allocate_runtime_arenas(ctx, max_batch != 0u ? max_batch : 1u, capacity, error, error_size)) {
                uocr_cuda_context_destroy(ctx);
                return NULL;
            }
        }
    }
    return ctx;
}

void uocr_cuda_engine_detach(struct uocr_cuda_context *ctx) {
    if (ctx == NULL) return;
    uocr_cuda_context_unmap_model(ctx);      /* releases MODEL_VIEWS / MOE_SCRATCH through the tracker while it is still alive */
    uocr_cuda_context_destroy(ctx);
}

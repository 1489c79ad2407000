/*
 * uocr_cuda_moe.h - C ABI of the CUDA (sm_100a) backend for the decoder MoE layer.
 *
 * This is the surface a `"cuda"` backend of unlimitedocr.c binds for the MoE layer.
 * It follows the conventions of the reference's backend headers
 * (src/backend/metal/uocr_metal.h:170-226, src/backend/cpu_ref/uocr_cpu_ref.h:57-90):
 *   - plain C types only; every function returns 1 on success and 0 on failure;
 *   - on failure a NUL-terminated message is written to (error, error_size) when given
 *     and is also kept in the context (uocr_cuda_context_last_error);
 *   - nothing on the per-token path allocates: weights are uploaded once by the map
 *     call, scratch is sized once by the arena call;
 *   - a context is not re-entrant; distinct contexts may be used from distinct threads
 *     (the per-engine rule of include/unlimitedocr.h:153-167).
 * Tensor bytes are exactly those of a .uocr model file (src/model/uocr_format.h:49-99;
 * expert slabs as laid out by src/unlimitedocr_c/convert.py:966-996).
 *
 * "d_" arguments are device pointers valid on the context's device, "h_" arguments
 * are host pointers.  All work is enqueued on the context's stream.
 */
#ifndef UOCR_CUDA_MOE_H
#define UOCR_CUDA_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#  define UOCR_CUDA_API __attribute__((visibility("default")))
#else
#  define UOCR_CUDA_API
#endif

/* Tensor storage types; values of uocr_tensor_qtype (src/model/uocr_format.h:40-47). */
#define UOCR_CUDA_QTYPE_F16  1
#define UOCR_CUDA_QTYPE_Q8_0 3
#define UOCR_CUDA_QTYPE_Q4_0 4
#define UOCR_CUDA_GROUP_SIZE 64u

typedef struct uocr_cuda_context uocr_cuda_context;

/* The engine's profile store and memory tracker (src/runtime/uocr_profile.h, src/runtime/uocr_memory.h).  This backend
 * treats them as opaque and reaches them through the engine's own functions, which the engine passes along:
 * uocr_profile_add_event_ms (src/runtime/uocr_profile.c:118-135) and uocr_memory_reserve / uocr_memory_release
 * (src/runtime/uocr_memory.h:47-48) have exactly these signatures. */
typedef struct uocr_profile_state uocr_profile_state;
typedef struct uocr_memory_tracker uocr_memory_tracker;
typedef void (*uocr_cuda_profile_add_event_ms_fn)(uocr_profile_state *profile, const char *name, double elapsed_ms);
typedef int (*uocr_cuda_memory_account_fn)(uocr_memory_tracker *tracker, int category, uint64_t bytes);
/* values of uocr_memory_category (include/unlimitedocr.h:50-62) this backend accounts under */
#define UOCR_CUDA_MEMORY_MODEL_VIEWS 0
#define UOCR_CUDA_MEMORY_MOE_SCRATCH 7

/* One projection matrix [rows][cols], input dimension contiguous.
 * f16: qweight = fp16[rows][cols], qscale unused.
 * q8_0: qweight = int8[rows][cols], qscale = fp16[rows][cols/64].
 * q4_0: qweight = uint8[rows][cols/2] (byte j of a 64-group: level[j]+8 low nibble,
 *       level[j+32]+8 high nibble), qscale = fp16[rows][cols/64]. */
typedef struct uocr_cuda_matrix {
    int32_t qtype;
    uint32_t rows;
    uint32_t cols;
    const void *qweight;
    const void *qscale;
} uocr_cuda_matrix;

/* One MoE layer as stored in the model file.  The routed experts are one packed-weight
 * slab and one scale slab, expert-major, each expert holding gate[F][H], up[F][H],
 * down[H][F]; strides/offsets carry the same meaning as the reference's kernel
 * parameter block (src/backend/metal/kernels/decode_gemv_q4.metal:15-28): byte counts
 * for packed weights, value counts for scales.  Zero strides/offsets mean "densely
 * packed" and are filled in by the library. */
typedef struct uocr_cuda_moe_layer_desc {
    uint32_t hidden_size;              /* H, multiple of 64 */
    uint32_t n_experts;                /* E <= 256 */
    uint32_t top_k;                    /* K <= 16, K <= E */
    uint32_t expert_intermediate;      /* F, multiple of 64 */
    uint32_t shared_intermediate;      /* S, multiple of 64 */
    float routed_scaling_factor;       /* finite, >= 0; weights are prob * factor, never renormalised */
    const void *router_weight_f16;     /* fp16 [E][H] */
    const float *router_logit_bias;    /* optional f32 [E] added to the logits; the model has none,
                                          synthetic load-skew benchmarks use it */
    int32_t expert_qtype;
    const void *expert_qweight;
    const void *expert_qscale;         /* NULL for f16 */
    uint64_t expert_stride_bytes;
    uint64_t up_offset_bytes;
    uint64_t down_offset_bytes;
    uint64_t expert_scale_stride_values;
    uint64_t up_scale_offset_values;
    uint64_t down_scale_offset_values;
    uocr_cuda_matrix shared_gate;      /* [S][H] */
    uocr_cuda_matrix shared_up;        /* [S][H] */
    uocr_cuda_matrix shared_down;      /* [H][S] */
} uocr_cuda_moe_layer_desc;

/* Optional extra outputs of a layer call (device pointers, any may be NULL). */
typedef struct uocr_cuda_moe_debug_outputs {
    float *d_router_logits;     /* [n][E] */
    float *d_router_probs;      /* [n][E] */
    uint32_t *d_top_ids;        /* [n][K], slot order = descending probability */
    float *d_top_weights;       /* [n][K] */
} uocr_cuda_moe_debug_outputs;

/* ---- backend and context: counterparts of uocr_metal_is_available, uocr_metal_backend_name,
 * uocr_metal_context_create/destroy (src/backend/metal/uocr_metal.h:170-176). */
UOCR_CUDA_API int uocr_cuda_is_available(void);
UOCR_CUDA_API const char *uocr_cuda_backend_name(void);            /* "cuda" */
UOCR_CUDA_API int uocr_cuda_device_count(void);
/* resource_path is accepted for signature parity and ignored (kernels are linked in).
 * The context binds the CUDA device that is current on the calling thread. */
UOCR_CUDA_API uocr_cuda_context *uocr_cuda_context_create(const char *resource_path, char *error, size_t error_size);
UOCR_CUDA_API void uocr_cuda_context_destroy(uocr_cuda_context *ctx);
UOCR_CUDA_API const char *uocr_cuda_context_last_error(const uocr_cuda_context *ctx);
/* Use an existing cudaStream_t (passed as void*) instead of the context's own; NULL restores it.
 * (The legacy default stream is named by cudaStreamLegacy, not by NULL.) */
UOCR_CUDA_API int uocr_cuda_context_set_stream(uocr_cuda_context *ctx, void *cuda_stream);
/* Counterparts of uocr_metal_context_set_profile / _set_memory_tracker (src/backend/metal/uocr_metal.h:177-178).
 * With a profile store set, every layer call brackets its phases with CUDA events on the stream they run on, and the
 * durations are added to the store under the names below the next time the context waits for its stream
 * (uocr_cuda_context_synchronize, the host-buffer calls, destroy).  Names follow the reference's
 * (src/backend/metal/uocr_metal.m:14447-14496, :13509, :13902): cuda.decode.moe_layer_fused (single-token kernel: router,
 * shared and routed experts in one launch), cuda.decode.moe_router, cuda.decode.moe_routed_experts, cuda.decode.moe_combine,
 * cuda.decode.moe_matvec, cuda.prefill.moe_router, cuda.prefill.moe_plan, cuda.prefill.moe_shared_experts,
 * cuda.prefill.moe_routed_bucketed_f16 / _q8 / _q4, cuda.prefill.moe_combine; uocr_cuda_profile_event_name(i) lists them
 * (NULL past the end).  NULL switches profiling off.
 * With a memory tracker set, the bytes of mapped weights are reserved under MODEL_VIEWS and the scratch arena under
 * MOE_SCRATCH (and released when they are freed); bytes held when the tracker is set are reserved at once. */
UOCR_CUDA_API void uocr_cuda_context_set_profile(uocr_cuda_context *ctx, uocr_profile_state *profile,
                                                 uocr_cuda_profile_add_event_ms_fn add_event_ms);
UOCR_CUDA_API void uocr_cuda_context_set_memory_tracker(uocr_cuda_context *ctx, uocr_memory_tracker *tracker,
                                                        uocr_cuda_memory_account_fn reserve, uocr_cuda_memory_account_fn release);
UOCR_CUDA_API const char *uocr_cuda_profile_event_name(uint32_t index);

/* Detail profiling of the single-token stack call, the counterpart of the reference's per-op checkpoints
 * (UOCR_METAL_DECODER_PROFILE_DETAIL, src/backend/metal/uocr_metal.m:29-31, :14251-14297).  d_trace is a device
 * buffer of 128 * n_layers * 16 uint64: the SM clock of CTA c in layer l at point p sits at [(c * n_layers + l) * 16 + p].
 * One-barrier decode kernel (112 CTAs): 0 activations arranged, 1 routing done, 2 weight fetches issued, 3 first weight
 * chunk in shared memory, 4 SwiGLU products ready, 5 partial outputs ready, 6 partial sums sent, 7 layer output
 * complete; 8 own router logits, 9 logits exchanged, 10-13 gate / up products of the first warp chunk by chunk,
 * 14 its sums, 15 every warp's sums; CTA slot 127 holds the clock of CTA 0 at kernel entry ([0]) and exit ([1]).
 * Two-barrier decode kernel (CTA 0 only, 8 points per layer at stride 8): layer start, inputs read, routing done,
 * copies issued, gate/up computed, barrier 1 passed, down computed, barrier 2 passed.  NULL switches it off. */
UOCR_CUDA_API int uocr_cuda_context_set_profile_detail(uocr_cuda_context *ctx, void *d_trace);
UOCR_CUDA_API int uocr_cuda_context_synchronize(uocr_cuda_context *ctx, char *error, size_t error_size);
/* Kernels launched by this context since creation (every launch is counted at its call site). */
UOCR_CUDA_API uint64_t uocr_cuda_context_kernel_launches(const uocr_cuda_context *ctx);
/* Device bytes held: weights ("model views") and scratch, the two categories the engine's
 * memory report uses for them (include/unlimitedocr.h:50-63). */
UOCR_CUDA_API uint64_t uocr_cuda_context_model_view_bytes(const uocr_cuda_context *ctx);
UOCR_CUDA_API uint64_t uocr_cuda_context_moe_scratch_bytes(const uocr_cuda_context *ctx);

/* ---- model mapping: counterpart of uocr_metal_context_map_model / _unmap_model
 * (src/backend/metal/uocr_metal.h:178-181).  Metal wraps the mmap'd file without a copy;
 * here every tensor of the layer is validated and uploaded once.  desc holds HOST pointers.
 * Layers get consecutive indices starting at 0. */
UOCR_CUDA_API int uocr_cuda_context_map_moe_layer(uocr_cuda_context *ctx, const uocr_cuda_moe_layer_desc *h_desc,
                                                  uint32_t *out_layer_index, char *error, size_t error_size);
UOCR_CUDA_API void uocr_cuda_context_unmap_model(uocr_cuda_context *ctx);

/* One entry of a .uocr file's tensor directory, byte for byte as the file stores it
 * (uocr_tensor_entry, src/model/uocr_format.h:275-299: packed, 140 bytes, sorted by id). */
#pragma pack(push, 1)
typedef struct uocr_cuda_tensor_entry {
    uint32_t id;                  /* src/model/uocr_tensor_registry.h:22-124 */
    uint32_t family;
    int32_t layer;
    int32_t expert;
    uint32_t projection;
    uint32_t usage;               /* 1 = runtime */
    uint32_t qtype;               /* 1 f16, 3 q8_0, 4 q4_0 */
    uint32_t flags;               /* bit 0 = row major */
    uint32_t rank;
    uint32_t logical_shape[4];
    uint32_t physical_shape[4];
    uint64_t payload_offset;      /* from the start of the file */
    uint64_t payload_size;
    uint32_t block_size;
    uint32_t row_size;
    uint64_t scale_offset;
    uint64_t scale_size;
    uint64_t min_offset;
    uint64_t min_size;
    uint32_t qtype_reason;
    uint32_t promotion_reason;
    uint32_t source_name_offset;
    uint32_t source_name_size;
} uocr_cuda_tensor_entry;
#pragma pack(pop)

/* What the backend needs of an opened model file: the fields of the engine's uocr_model_file
 * (src/model/uocr_model_file.h:9-28) and of its config record (src/model/uocr_format.h:193-225) that concern the
 * decoder's MoE layers.  The engine fills it from the file it has already opened and validated:
 *   data, size, tensors, tensor_count      <- model->data, ->size, ->tensors, ->tensor_count
 *   routed_experts, moe_top_k              <- model->config->routed_experts, ->moe_top_k
 *   first_moe_layer, moe_layer_count       <- config->dense_first_layers, config->decoder_layers - dense_first_layers
 *   routed_scaling_factor                  <- UOCR_MOE_ROUTED_SCALING_FACTOR (src/model/uocr_constants.h:54) */
typedef struct uocr_cuda_model_file_view {
    const void *data;
    uint64_t size;
    const void *tensors;          /* uocr_cuda_tensor_entry[tensor_count], inside [data, data + size) */
    uint32_t tensor_count;
    uint32_t routed_experts;
    uint32_t moe_top_k;
    uint32_t first_moe_layer;
    uint32_t moe_layer_count;
    float routed_scaling_factor;
} uocr_cuda_model_file_view;

/* Counterpart of uocr_metal_context_map_model (src/backend/metal/uocr_metal.h:180) for the MoE layers: looks up the
 * router, the three shared projections and every routed expert's three projections of each requested decoder layer
 * by tensor id, checks them (runtime usage, row-major rank 2, shapes agree, byte ranges inside the file), checks
 * that the routed experts form ONE interleaved-contiguous slab of packed weights and one of scales, as the
 * reference host does before it binds a layer (src/backend/metal/uocr_metal.m:3037-3154, same error texts), and
 * uploads each layer once.  File layer first_moe_layer + i becomes layer i of this context.  A file that fails
 * any check leaves the context without layers. */
UOCR_CUDA_API int uocr_cuda_context_map_model(uocr_cuda_context *ctx, const uocr_cuda_model_file_view *model,
                                              char *error, size_t error_size);
UOCR_CUDA_API uint32_t uocr_cuda_context_moe_layer_count(const uocr_cuda_context *ctx);
/* The tensors either side of the MoE layers, from the same file, after uocr_cuda_context_map_model: the dense SwiGLU MLP
 * of decoder layer 0 (uocr_tensor_id_layer_dense_mlp, src/model/uocr_tensor_registry.h:72-86; scratch for token_capacity
 * tokens), the LM head (UOCR_TENSOR_ID_LM_HEAD, :12), the post-attention norm weight of every decoder layer below
 * first_moe_layer + moe_layer_count (uocr_tensor_id_layer_post_attn_norm, :54-56) and the final norm
 * (UOCR_TENSOR_ID_FINAL_NORM, :13).  A tensor the file does not hold is skipped; one it holds is checked like the MoE
 * tensors (runtime, row-major, byte ranges inside the file) and refused with a message otherwise, before anything is
 * uploaded.  The getters return -1 / NULL for what was not mapped; the norm weights are device fp16[hidden_size], ready
 * for uocr_cuda_moe_layer_forward_normed / uocr_cuda_dense_mlp_forward_normed / uocr_cuda_rmsnorm. */
UOCR_CUDA_API int uocr_cuda_context_map_model_neighbours(uocr_cuda_context *ctx, const uocr_cuda_model_file_view *model,
                                                         uint32_t token_capacity, char *error, size_t error_size);
UOCR_CUDA_API int uocr_cuda_context_file_dense_mlp_index(const uocr_cuda_context *ctx);
UOCR_CUDA_API const void *uocr_cuda_context_post_attn_norm_weight(const uocr_cuda_context *ctx, uint32_t decoder_layer);
UOCR_CUDA_API const void *uocr_cuda_context_final_norm_weight(const uocr_cuda_context *ctx);

/* ---- the steps either side of the MoE layer.
 * RMSNorm (uocr_cpu_ref_rmsnorm_f32, src/backend/cpu_ref/uocr_cpu_ref.c:145-169; the GPU form
 * uocr_rmsnorm_f16_to_f16, src/backend/metal/kernels/norm.metal:12-40): fp16 rows [n][hidden_size] and fp16 weight in,
 * f32 arithmetic, d_out = fp16( x * 1/sqrt(mean(x^2) + eps) * weight ).  hidden_size must be a multiple of 8. */
UOCR_CUDA_API int uocr_cuda_rmsnorm(uocr_cuda_context *ctx, const void *d_x, const void *d_weight_f16, float eps,
                                    uint32_t n_tokens, uint32_t hidden_size, void *d_out, char *error, size_t error_size);
/* The MoE layer as the decoder runs it (src/backend/metal/uocr_metal.m:14433-14497): d_stream is the residual stream after
 * attention, the post-attention norm feeds the layer and the stream is added back:
 * d_out = MoE( RMSNorm(d_stream) * weight ) + d_stream.  The normalised rows live in the context's scratch; a one-token
 * call on the single-token decode kernel normalises inside that kernel (one launch, the same arithmetic, bit-equal). */
UOCR_CUDA_API int uocr_cuda_moe_layer_forward_normed(uocr_cuda_context *ctx, uint32_t layer, const void *d_stream,
                                                     const void *d_norm_weight_f16, float eps, uint32_t n_tokens, void *d_out,
                                                     const uocr_cuda_moe_debug_outputs *dbg, char *error, size_t error_size);
/* The dense SwiGLU MLP of the first decoder layer (uocr_cpu_ref_dense_swiglu_f32, src/backend/cpu_ref/uocr_cpu_ref.c:305-349;
 * tensors uocr_tensor_id_layer_dense, src/model/uocr_tensor_registry.h:72-86; intermediate width 6848): the kernels of
 * the shared experts on other matrices.  gate / up [S][H] and down [H][S] with HOST pointers, S <= 8192, H <= 2048, both
 * multiples of 64; scratch for up to token_capacity tokens is allocated here and freed by uocr_cuda_context_unmap_model.
 * d_out = fp16( down . fp16( silu(gate x) * up x ) + residual ); calls of at least the tensor-core threshold (and H a
 * multiple of 128) round the down product to fp16 before the residual is added, as the MoE layer's shared output is. */
UOCR_CUDA_API int uocr_cuda_context_map_dense_mlp(uocr_cuda_context *ctx, const uocr_cuda_matrix *gate, const uocr_cuda_matrix *up,
                                                  const uocr_cuda_matrix *down, uint32_t token_capacity, uint32_t *out_index,
                                                  char *error, size_t error_size);
UOCR_CUDA_API int uocr_cuda_dense_mlp_forward(uocr_cuda_context *ctx, uint32_t index, const void *d_hidden, const void *d_residual,
                                              uint32_t n_tokens, void *d_out, char *error, size_t error_size);
/* d_out = DenseMLP( RMSNorm(d_stream) * weight ) + d_stream.  One token at the model's hidden size in Q4_0 / Q8_0 runs on the
 * single-token decode kernel without routing (units of 64 intermediate columns on a slice-major copy of the three
 * matrices, norm inside the kernel); 2 - 4 tokens on the shared experts' matrix-vector kernels; more on the grouped GEMM. */
UOCR_CUDA_API int uocr_cuda_dense_mlp_forward_normed(uocr_cuda_context *ctx, uint32_t index, const void *d_stream,
                                                     const void *d_norm_weight_f16, float eps, uint32_t n_tokens, void *d_out,
                                                     char *error, size_t error_size);

/* ---- LM head: the vocabulary projection fused with the argmax (uocr_lm_head_argmax_q4_0_to_f16 / _q8_0,
 * src/backend/metal/kernels/lm_head_q4.metal:25-100; host metal_run_lm_head_argmax_*; docs/plan_q4.md:493-517), the
 * largest single weight reader of a decode step after the MoE layers.  weight [vocab][hidden] with HOST pointers in
 * any of the three formats.  d_token_ids[t] = the row with the largest dot product with d_hidden[t] (fp16 rows after the
 * final norm), ties to the lowest id, NaN rows skipped (0xffffffff if every row is NaN); d_scores (optional) the winning
 * logits.  At most four tokens per call share one pass over the weights. */
UOCR_CUDA_API int uocr_cuda_context_map_lm_head(uocr_cuda_context *ctx, const uocr_cuda_matrix *weight, char *error,
                                                size_t error_size);
UOCR_CUDA_API int uocr_cuda_lm_head_argmax(uocr_cuda_context *ctx, const void *d_hidden, uint32_t n_tokens,
                                           uint32_t *d_token_ids, float *d_scores, char *error, size_t error_size);

/* ---- scratch: counterpart of uocr_metal_context_allocate_runtime_arenas / _release_runtime_arenas
 * (src/backend/metal/uocr_metal.h:221-226) restricted to the MoE scratch.  Must be called after the
 * layers are mapped and before any forward call with n_tokens <= token_capacity. */
UOCR_CUDA_API int uocr_cuda_context_allocate_runtime_arenas(uocr_cuda_context *ctx, uint32_t batch_slots,
                                                            uint32_t token_capacity, char *error, size_t error_size);
UOCR_CUDA_API void uocr_cuda_context_release_runtime_arenas(uocr_cuda_context *ctx);
/* Bytes the arena call will reserve for a layer of these dimensions (the sizing rule of
 * src/runtime/uocr_memory.c:480-543 plus this backend's dispatch plan and partial sums). */
UOCR_CUDA_API uint64_t uocr_cuda_moe_scratch_size(uint32_t hidden_size, uint32_t n_experts, uint32_t top_k,
                                                  uint32_t expert_intermediate, uint32_t shared_intermediate,
                                                  uint32_t token_capacity);

/* ---- operators ----------------------------------------------------------------------- */

/* Router: logits = hidden . router^T (fp16 inputs, f32 accumulate) [+ bias], f32 softmax, greedy top-k
 * with ties to the lower expert id; weight = prob * routed_scaling_factor.  Semantics of
 * uocr_cpu_ref_moe_router_f32 (src/backend/cpu_ref/uocr_cpu_ref.c:388-466) on the fp16 inputs the GPU
 * path carries (src/backend/metal/kernels/moe.metal:53-189).  When d_injected_logits is not NULL the dot
 * products are skipped and those logits are used as they are (bias still added when the layer has one):
 * softmax, ids and weights are then bit-identical to the CPU function's on the same logits.
 * d_logits / d_probs may be NULL. */
UOCR_CUDA_API int uocr_cuda_moe_router(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden_f16,
                                       const float *d_injected_logits, uint32_t n_tokens, float *d_logits,
                                       float *d_probs, uint32_t *d_top_ids, float *d_top_weights, char *error,
                                       size_t error_size);

/* Token-to-expert permutation.  pair = token * K + slot.  expert_offsets[E+1] is the exclusive prefix sum
 * of pairs per expert, pair_rows[] lists the pairs grouped by expert in ascending pair order (a stable
 * counting sort), inverse[pair] is the pair's position in pair_rows (0xffffffff for an id >= E, which is
 * dropped).  Deterministic form of the reference's bucketing pass
 * (src/backend/metal/kernels/gemm_q8.metal:462-511). */
UOCR_CUDA_API int uocr_cuda_moe_dispatch_plan(uocr_cuda_context *ctx, const uint32_t *d_top_ids, uint32_t n_tokens,
                                              uint32_t top_k, uint32_t n_experts, uint32_t *d_expert_offsets,
                                              uint32_t *d_pair_rows, uint32_t *d_inverse, char *error,
                                              size_t error_size);

/* The same dispatch plan for callers that must not allocate device memory.  It has no counterpart in the
 * reference, whose backends own all their buffers.  It needs no context and no arena: the kernel's only scratch
 * (the list of experts that received a pair) lives in a fixed 1280-byte device array inside this library, which
 * every process that loads the library holds on each device it uses until it exits.  It exists for hosts that
 * cannot call cudaMalloc where they need a plan: on a hot path guarded against allocation (the reference asserts
 * this with uocr_alloc_guard, src/core/uocr_alloc.h:21-42), in a decode loop that has frozen its
 * memory map, or after the engine's memory admission has handed out the whole device budget.
 * Limits: n_experts <= 256 and n_tokens * top_k <= 1048576; larger sizes are refused with a message.
 * The first call on a device looks up the array's device address and raises the kernel's shared-memory limit
 * (no allocation); make that first call before any stream capture.  All calls share the one array, so two calls
 * whose kernels may overlap on the GPU (different streams without an ordering between them) race on it; calls
 * on one stream are safe.  Nothing in the array needs clearing: every call rewrites the entries it later reads.
 * cuda_stream is a cudaStream_t (NULL = the default stream); the current device is used. */
UOCR_CUDA_API int uocr_cuda_moe_dispatch_plan_noalloc(const uint32_t *d_top_ids, uint32_t n_tokens, uint32_t top_k,
                                                      uint32_t n_experts, uint32_t *d_expert_offsets,
                                                      uint32_t *d_pair_rows, uint32_t *d_inverse, void *cuda_stream,
                                                      char *error, size_t error_size);

/* Bring-up and test aid: the value the kernels give every weight of one projection matrix, so that the in-register
 * dequantisers can be compared with the format definition (level * fp16 scale, src/model/uocr_format.h:49-99; the
 * reference pins its packed bytes in tests/test_convert.py:192-218 and unpacks them on the CPU only).
 *   matrix  0 / 1 / 2: gate [F][H] / up [F][H] / down [H][F] of routed expert `expert`; 3 / 4 / 5: the shared MLP's.
 *   path    0: the matrix-vector kernels (row_dot on one-hot activations): f32 level * float(scale), exact;
 *           1: the grouped GEMM's producer: fp16( float(level) * float(scale) ), the value the reference's tiled
 *              GEMMs feed their MMAs (src/backend/metal/kernels/gemm_q4.metal:35-57, gemm_q8.metal:43-60).
 * d_out: f32 [rows][cols] on the device.  path 1 needs cols to be a multiple of 64. */
UOCR_CUDA_API int uocr_cuda_moe_debug_dequantize(uocr_cuda_context *ctx, uint32_t layer, uint32_t matrix, uint32_t expert,
                                                 uint32_t path, float *d_out, char *error, size_t error_size);

/* The layer: out[n][H] = fp16( sum_slot weight * expert(hidden) + shared(hidden) [+ residual] ), the
 * computation of uocr_cpu_ref_moe_swiglu_f32 (src/backend/cpu_ref/uocr_cpu_ref.c:468-579) with the GPU
 * path's data types: fp16 activations, weights dequantised on the fly and never materialised, f32
 * accumulation, SwiGLU products stored as fp16, fp16 output with the residual folded into the combine
 * (call sites src/backend/metal/uocr_metal.m:14433-14497 and :14773-14856).  d_residual_f16 may be NULL.
 * d_injected_logits as for the router.  The regime (one token, a few tokens, many tokens) is chosen
 * from n_tokens as the reference does (src/backend/metal/uocr_metal.m:13674). */
UOCR_CUDA_API int uocr_cuda_moe_layer_forward(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden_f16,
                                              const void *d_residual_f16, const float *d_injected_logits,
                                              uint32_t n_tokens, void *d_out_f16,
                                              const uocr_cuda_moe_debug_outputs *debug, char *error,
                                              size_t error_size);

/* Which of the regimes a layer call with n_tokens would take (a static string naming the kernels; "" for invalid
 * arguments).  The reference switches on n_tokens > 1 in the same place (src/backend/metal/uocr_metal.m:13674). */
UOCR_CUDA_API const char *uocr_cuda_moe_regime_name(const uocr_cuda_context *ctx, uint32_t layer, uint32_t n_tokens);

/* A run of consecutive layers first_layer .. first_layer+n_layers-1 chained the way the decoder chains
 * them with the attention block left out: layer i's input is also its residual, its output feeds layer
 * i+1.  One call = one decode step through the MoE halves of those layers. */
UOCR_CUDA_API int uocr_cuda_moe_stack_forward(uocr_cuda_context *ctx, uint32_t first_layer, uint32_t n_layers,
                                              const void *d_hidden_f16, uint32_t n_tokens, void *d_out_f16,
                                              char *error, size_t error_size);

/* Host-buffer forms: copy h_hidden (and h_residual) to the device, run, copy the result back and wait.
 * These are what a host engine without its own device buffers calls.  The stack form with one token issues no
 * copies when the single-token decode kernel serves it: the activations travel in the launch parameters, the
 * kernel writes the result and its status word into mapped pinned host memory, and the call waits for the stream. */
UOCR_CUDA_API int uocr_cuda_moe_layer_forward_host(uocr_cuda_context *ctx, uint32_t layer, const void *h_hidden_f16,
                                                   const void *h_residual_f16, uint32_t n_tokens, void *h_out_f16,
                                                   uint32_t *h_top_ids, float *h_top_weights, char *error,
                                                   size_t error_size);
UOCR_CUDA_API int uocr_cuda_moe_stack_forward_host(uocr_cuda_context *ctx, uint32_t first_layer, uint32_t n_layers,
                                                   const void *h_hidden_f16, uint32_t n_tokens, void *h_out_f16,
                                                   char *error, size_t error_size);

/* ---- expert parallelism --------------------------------------------------------------------
 * The reference engine runs on one device (include/unlimitedocr.h:153-167 has no multi-device notion), so
 * these three calls have no counterpart there.  They are the many-token layer cut at its two exchange
 * points: a host that shards the experts over several GPUs (each GPU owning a contiguous range of expert
 * ids and a share of the tokens) runs
 *     dispatch  ->  all-to-all of rows (shared MLP meanwhile)  ->  experts  ->  all-to-all back  ->  combine.
 * On one GPU the four calls in a row, without the exchanges, compute uocr_cuda_moe_layer_forward.
 * All of them use scratch sized for the context's token capacity, which must cover the rows a rank can
 * RECEIVE: rows_received <= token_capacity * top_k. */

/* Router + dispatch plan on this rank's n_tokens, then d_sorted_rows[pos][H] = hidden row of the pos-th
 * (token, slot) pair in expert order (fp16, n_tokens * top_k rows; experts ascending, so the rows for each
 * owner GPU are contiguous).  d_expert_offsets[E+1] (device) receives the exclusive prefix sum of the pairs per
 * expert, so that the ranks can exchange their counts without a host round trip.  The call does not wait. */
UOCR_CUDA_API int uocr_cuda_moe_ep_dispatch(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden_f16,
                                            uint32_t n_tokens, void *d_sorted_rows_f16, uint32_t *d_expert_offsets,
                                            char *error, size_t error_size);
/* Routed experts first_expert .. first_expert + n_local_experts - 1 on received rows.  d_rows_in holds, for
 * source 0, 1, ... n_sources - 1 in turn, the rows for each local expert in turn; h_segment_counts
 * [n_sources][n_local_experts] gives their counts.  d_rows_out[row][H] = down( silu(gate x) * up x ), fp16,
 * same row order, not yet weighted. */
UOCR_CUDA_API int uocr_cuda_moe_ep_experts(uocr_cuda_context *ctx, uint32_t layer, uint32_t first_expert,
                                           uint32_t n_local_experts, uint32_t n_sources,
                                           const uint32_t *h_segment_counts, const void *d_rows_in_f16,
                                           void *d_rows_out_f16, char *error, size_t error_size);
/* Shared MLP of this rank's tokens into the context's scratch.  Independent of the exchange: it is queued on a
 * second stream of the context (after everything queued so far on the context's stream) and runs beside whatever
 * the caller queues next; the combine call of the same layer call waits for it.  d_hidden_f16 must stay unchanged
 * until then.  Must precede the combine call of the same layer call. */
UOCR_CUDA_API int uocr_cuda_moe_ep_shared(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden_f16,
                                          uint32_t n_tokens, char *error, size_t error_size);
/* d_rows_back[pos][H]: the expert outputs for this rank's pairs, in the order dispatch produced them.
 * out = fp16( sum_slot weight * row + shared MLP output [+ residual] ) for this rank's tokens. */
UOCR_CUDA_API int uocr_cuda_moe_ep_combine(uocr_cuda_context *ctx, uint32_t layer, const void *d_rows_back_f16,
                                           const void *d_residual_f16, uint32_t n_tokens, void *d_out_f16,
                                           char *error, size_t error_size);

/* ---- expert parallelism over peer memory (no reference counterpart) --------------------------------------------
 * The same layer call with the exchange fused into the library's kernels: every rank (one process per GPU of one
 * node) owns two buffers of row_capacity rows x hidden fp16, "received rows" and "expert outputs", and maps the
 * other ranks' buffers through CUDA IPC.  The gather then writes each pair's row straight into the owner's
 * buffer and the combine reads each pair's output row straight from it, over NVLink, so no separate all-to-all
 * runs.  What the caller provides: the per-rank counts (one small all_gather of d_expert_offsets), and two
 * barriers over the group per call (after scatter: all rows have landed; after experts: all outputs are
 * written).  With one rank the calls reproduce uocr_cuda_moe_layer_forward.
 *
 * create:   allocates this rank's buffers; handles_out receives 128 bytes (two CUDA IPC handles) to be gathered.
 * open:     all_handles = the world x 128 bytes of every rank, in rank order.  At most 16 ranks.
 * dispatch: router + dispatch plan on this rank's tokens; d_expert_offsets[E+1] as in uocr_cuda_moe_ep_dispatch.
 * scatter:  h_dst_row0[E]: for every expert, the row of ITS OWNER's "received rows" buffer where this rank's
 *           rows start.  The owner of expert e is rank e / (E / world); its buffer holds, for source rank 0, 1, ...
 *           in turn, the rows of each of its experts in turn.
 * experts:  this rank's experts on its received rows -> its "expert outputs", same row order;
 *           h_segment_counts[world][E / world] as in uocr_cuda_moe_ep_experts.
 * combine:  out = fp16( sum_slot weight * output row of the pair (read from its owner) + shared MLP [+ residual] );
 *           uocr_cuda_moe_ep_shared must have run for these tokens.
 * A row index outside the buffers (inconsistent counts) is never dereferenced: it raises a status bit that
 * uocr_cuda_context_synchronize reports.
 * destroy:  unmaps the peers' buffers and frees this rank's.  The caller must make sure that NO rank still has a
 *           scatter or combine kernel in flight (every rank waits for its stream, then a barrier over the group):
 *           a peer that touches a freed buffer faults on its own GPU. */
UOCR_CUDA_API int uocr_cuda_moe_ep_peer_create(uocr_cuda_context *ctx, uint32_t hidden_size, uint64_t row_capacity,
                                               void *handles_out, char *error, size_t error_size);
UOCR_CUDA_API int uocr_cuda_moe_ep_peer_open(uocr_cuda_context *ctx, uint32_t world, uint32_t rank, const void *all_handles,
                                             char *error, size_t error_size);
UOCR_CUDA_API void uocr_cuda_moe_ep_peer_destroy(uocr_cuda_context *ctx);
UOCR_CUDA_API int uocr_cuda_moe_ep_peer_dispatch(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden_f16,
                                                 uint32_t n_tokens, uint32_t *d_expert_offsets, char *error, size_t error_size);
UOCR_CUDA_API int uocr_cuda_moe_ep_peer_scatter(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden_f16,
                                                uint32_t n_tokens, const uint32_t *h_dst_row0, char *error, size_t error_size);
UOCR_CUDA_API int uocr_cuda_moe_ep_peer_experts(uocr_cuda_context *ctx, uint32_t layer, uint32_t n_sources,
                                                const uint32_t *h_segment_counts, char *error, size_t error_size);
/* scatter / experts with the counts left on the device: d_all_offsets [world][E + 1] is every rank's d_expert_offsets
 * in rank order (one all_gather on the device).  The row offsets of both phases are computed by a small kernel, so no
 * host copy or wait sits between the count exchange and the kernels.  The experts phase sizes its work for the rows
 * this rank's buffers can hold (min(row_capacity, token_capacity * top_k)); more rows than that raise the status bit. */
UOCR_CUDA_API int uocr_cuda_moe_ep_peer_scatter_dev(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden_f16,
                                                    uint32_t n_tokens, const uint32_t *d_all_offsets, char *error, size_t error_size);
UOCR_CUDA_API int uocr_cuda_moe_ep_peer_experts_dev(uocr_cuda_context *ctx, uint32_t layer, char *error, size_t error_size);
/* The whole expert-parallel layer call with the ranks synchronised ON THE DEVICE: router, plan, count exchange, scatter,
 * experts and combine are queued in one go; between them the ranks signal one another through flags in peer memory
 * (a release store of the call's number into every peer, a bounded wait on the own flags) instead of host-side
 * collectives.  Every rank of the group must issue the call, in the same order on every rank.  A peer that does not
 * reach the call within about two seconds makes the waiting kernels give up; the next uocr_cuda_context_synchronize
 * then fails with a message, and nothing is left hanging. */
UOCR_CUDA_API int uocr_cuda_moe_ep_peer_forward(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden,
                                                const void *d_residual, uint32_t n_tokens, void *d_out, char *error,
                                                size_t error_size);
/* Every rank's expert offsets of the last uocr_cuda_moe_ep_peer_forward call, h_all_offsets [world][n_experts + 1]
 * (waits for the stream; meant for load statistics). */
UOCR_CUDA_API int uocr_cuda_moe_ep_peer_last_offsets(uocr_cuda_context *ctx, uint32_t n_experts, uint32_t *h_all_offsets,
                                                     char *error, size_t error_size);
UOCR_CUDA_API int uocr_cuda_moe_ep_peer_combine(uocr_cuda_context *ctx, uint32_t layer, const void *d_residual_f16,
                                                uint32_t n_tokens, void *d_out_f16, char *error, size_t error_size);

#ifdef __cplusplus
}
#endif

#endif /* UOCR_CUDA_MOE_H */

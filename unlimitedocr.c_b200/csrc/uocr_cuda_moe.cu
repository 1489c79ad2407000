// Host side of the C ABI in include/uocr_cuda_moe.h: context, weight upload, scratch arena and the
// per-call dispatch of the MoE layer onto the kernel files.  Plain CUDA runtime; no allocation on
// the forward path.
#include "../../include/uocr_cuda_moe.h"

#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "moe_common.cuh"

namespace uocr {
cudaError_t init_router_kernels();
cudaError_t init_small_batch_kernels();
cudaError_t init_lm_head_kernels();
bool dense_small_supported(uint32_t H, uint32_t S);
uint32_t lm_head_max_tokens();
cudaError_t launch_lm_head_argmax(const DMatrix &m, const __half *hidden, uint32_t n, uint32_t grid, float *part_scores,
                                  uint32_t *part_ids, uint32_t *ticket, uint32_t *ids_out, float *scores_out, cudaStream_t st,
                                  uint64_t *launches);
bool gemm_tensor_maps_ready();
cudaError_t launch_dense_small(const DMatrix &g, const DMatrix &u, const DMatrix &d, const __half *hidden, const __half *residual,
                               uint32_t n, __half *mid, float *out_f32, __half *out, cudaStream_t st, uint64_t *launches);
cudaError_t launch_rmsnorm(const __half *x, const __half *w, uint32_t rows, uint32_t cols, float eps, __half *out, cudaStream_t st,
                           uint64_t *launches);
cudaError_t launch_add_rows(const __half *a, const __half *residual, size_t count, __half *out, cudaStream_t st, uint64_t *launches);
cudaError_t init_decode_kernels();
cudaError_t init_decode_sliced_kernels();
cudaError_t init_gemm_kernels();
bool gemm_path_supported(const DLayer &L);
struct GemmScratch {
    __half *x_sorted, *mid_sorted, *down_sorted, *shared_mid, *shared_out;
    uint4 *tiles_gu, *tiles_dn, *stiles_gu, *stiles_dn;
    uint32_t *counts;
};
cudaError_t launch_scatter_peer(const DLayer &L, const Scratch &S, const __half *hidden, uint32_t n, uint32_t experts_per_rank,
                                const uint32_t *dst_row0, const PeerBuffers &recv, unsigned long long row_capacity,
                                cudaStream_t st, uint64_t *launches);
cudaError_t launch_combine_peer(const DLayer &L, const Scratch &S, const GemmScratch &G, const PeerBuffers &done,
                                uint32_t experts_per_rank, const uint32_t *dst_row0, unsigned long long row_capacity,
                                const __half *residual, uint32_t n, __half *out, cudaStream_t st, uint64_t *launches);
cudaError_t launch_ep_exchange_counts(const uint32_t *my_offsets, const PeerSync &sync, uint32_t world, uint32_t rank, uint32_t E,
                                      uint32_t call, unsigned long long row_capacity, uint32_t *dst_row0, uint32_t *seg_offsets,
                                      uint32_t *status, cudaStream_t st, uint64_t *launches);
cudaError_t launch_ep_signal_wait(const PeerSync &sync, uint32_t world, uint32_t rank, uint32_t which, uint32_t call,
                                  uint32_t *status, cudaStream_t st, uint64_t *launches);
cudaError_t launch_ep_offsets(const uint32_t *all_offsets, uint32_t world, uint32_t rank, uint32_t E,
                              unsigned long long row_capacity, uint32_t *dst_row0, uint32_t *seg_offsets, uint32_t *status,
                              cudaStream_t st, uint64_t *launches);
cudaError_t launch_gather_sorted(const DLayer &L, const Scratch &S, const __half *hidden, uint32_t n, __half *rows_out,
                                 cudaStream_t st, uint64_t *launches);
cudaError_t launch_gemm_experts(const DLayer &L, const Scratch &S, const GemmScratch &G, const uint32_t *seg_offsets,
                                uint32_t n_seg, uint32_t expert_base, uint32_t expert_mod, const __half *rows_in,
                                uint32_t rows_bound, __half *mid, __half *rows_out, cudaStream_t st, uint64_t *launches);
cudaError_t launch_gemm_shared(const DLayer &L, const Scratch &S, const GemmScratch &G, const __half *hidden, uint32_t n,
                               cudaStream_t st, uint64_t *launches);
cudaError_t launch_gemm_combine(const DLayer &L, const Scratch &S, const GemmScratch &G, const __half *down_rows,
                                const __half *residual, uint32_t n, __half *out, cudaStream_t st, uint64_t *launches);
cudaError_t init_decode_batched_kernels();
uint32_t decode_batched_max_tokens();
BatchedScratchLayout decode_batched_scratch(uint32_t n, uint32_t K);
bool decode_batched_supported(const DLayer &L, uint32_t n);
cudaError_t launch_batched_route(const DLayer &L, const Scratch &S, const __half *hidden, const float *injected, uint32_t n,
                                 float *logits, float *probs, uint8_t *scratch, uint32_t *ticket, cudaStream_t st, uint64_t *launches);
cudaError_t launch_batched_experts(const DLayer &L, const Scratch &S, uint32_t n, uint8_t *scratch, cudaStream_t st, uint64_t *launches);
cudaError_t launch_batched_combine(const DLayer &L, const Scratch &S, const __half *residual, uint32_t n, uint8_t *scratch, __half *out,
                                   cudaStream_t st, uint64_t *launches);
cudaError_t launch_dequant_probe(const DMatrix &m, float *out, cudaStream_t st, uint64_t *launches);
cudaError_t launch_producer_probe(const DMatrix &m, float *out, cudaStream_t st, uint64_t *launches);
int decode_grid_size();
bool decode_supported(const DLayer *layers, uint32_t first, uint32_t count);
bool decode_sliced_layer_ok(const DLayer &L);
size_t decode_units_bytes(const DLayer &L);
cudaError_t build_decode_units(const DLayer &L, uint8_t *out, cudaStream_t st);
size_t decode_sliced_acc_bytes();
bool decode_sliced_supported(const DLayer *layers, uint32_t first, uint32_t count);
cudaError_t launch_decode_sliced(const DLayer *h_layers, const DLayer *d_layers, uint32_t first, uint32_t count,
                                 const __half *hidden, const __half *residual0, const void *h_inline, int chain_residual,
                                 const float *injected, __half *out, uint32_t *host_status, unsigned long long *acc,
                                 uint32_t *acc_base, uint32_t *status,
                                 float *dbg_logits, float *dbg_probs, uint32_t *ids_out, float *wts_out,
                                 unsigned long long *trace, const SlicedKnobs &knobs, cudaStream_t st, uint64_t *launches,
                                 const __half *norm_weight = nullptr, float norm_eps = 0.f);
uint32_t decode_dense_units(uint32_t hidden, uint32_t inter, int gate_qtype, int up_qtype, int down_qtype);
size_t decode_dense_units_bytes(int qtype, uint32_t units);
cudaError_t build_dense_units(const DMatrix &gate, const DMatrix &up, const DMatrix &down, uint32_t units, uint8_t *out, cudaStream_t st);
cudaError_t launch_decode_dense(const DLayer *d_layer, const uint8_t *unit_blobs, int qtype, uint32_t units, const __half *hidden, const __half *residual,
                                __half *out, unsigned long long *acc, uint32_t *acc_base, uint32_t *status, const SlicedKnobs &knobs,
                                cudaStream_t st, uint64_t *launches, const __half *norm_weight = nullptr, float norm_eps = 0.f);
cudaError_t launch_decode_stack(const DLayer *h_layers, const DLayer *d_layers, uint32_t first, uint32_t count,
                                const __half *hidden, const __half *residual0, int chain_residual,
                                const float *injected, __half *out, __half *hbuf0, __half *hbuf1, __half *mid,
                                float *plogits, unsigned long long *bar, unsigned long long *bar_base, uint32_t *status,
                                float *dbg_logits, float *dbg_probs, uint32_t *ids_out, float *wts_out,
                                unsigned long long *trace, cudaStream_t st, uint64_t *launches);
}  // namespace uocr

static constexpr uint32_t kMaxLayers = 64;
static constexpr uint32_t kSegSlots = 8;
static constexpr uint64_t kUploadPad = 256;   // kernels may read an aligned window that ends past a tensor

using uocr::DLayer;
using uocr::DMatrix;
using uocr::Scratch;

struct uocr_cuda_context {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    std::vector<DLayer> layers;
    // dense SwiGLU MLPs (the first decoder layer's MLP) with their own scratch, sized when they are mapped
    struct DenseMlp {
        DMatrix gate{}, up{}, down{};
        uint32_t H = 0, S = 0, capacity = 0;
        __half *x_norm = nullptr, *mid = nullptr;      // [capacity][H], [capacity][S]
        float *out_f32 = nullptr;                      // [capacity][H] (the tensor-core path keeps fp16 rows in it)
        uint4 *tiles_gu = nullptr, *tiles_dn = nullptr;
        uint32_t *counts = nullptr;
        uint32_t units = 0;                            // one-token path through the decode kernel: 64-column units (0: not built)
        DLayer *d_layer = nullptr;                     // device copy of the pseudo layer that points at the units
        const uint8_t *unit_blobs = nullptr;
        void *scratch = nullptr;
        uint64_t scratch_bytes = 0;
    };
    std::vector<DenseMlp> dense;
    // tensors either side of the MoE layers mapped from a model file (uocr_cuda_context_map_model_neighbours)
    int file_dense_index = -1;                          // index of the file's layer-0 dense MLP in `dense`, or -1
    std::vector<const __half *> post_attn_norms;        // [decoder layer] device fp16[H], null where the file has none
    const __half *final_norm = nullptr;
    // the LM head (vocabulary projection) and the scratch of its fused argmax
    struct {
        DMatrix w{};
        bool mapped = false;
        uint32_t grid = 0;
        void *scratch = nullptr;       // [grid][4] scores, [grid][4] ids, ticket
    } lm_head;
    DLayer *d_layers = nullptr;        // device copy of `layers`
    bool fused_decode = true;          // single-token calls use the persistent decode kernel when it fits
    uint32_t gemm_min_tokens = 5;      // calls with at least this many tokens take the tensor-core path
    bool sliced_decode = true;         // ... in its one-barrier-per-layer form when the shapes allow it
    bool batched_decode = true;        // calls of a few tokens (up to 64) at the model's shapes use the weight-streaming kernel
    unsigned long long bar_base = 0;   // value the decode kernel's barrier counter has reached
    uint32_t acc_base = 0;             // accumulator buffer the next sliced decode launch starts with
    uocr::SlicedKnobs decode_knobs;    // replicas of the decode accumulator, wait limit
    bool test_stall_once = false;      // test hook: the next sliced decode launch waits for a contribution nobody makes
    size_t status_bytes = 0;           // status word, barrier counter and the decode accumulators
    unsigned long long *decode_trace = nullptr;   // optional device buffer for per-phase clock stamps
    std::vector<void *> weight_allocs;
    uint64_t weight_bytes = 0;
    // arena
    uint8_t *arena = nullptr;
    uint64_t arena_bytes = 0;
    uint64_t dense_scratch_bytes = 0;     // scratch of the mapped dense MLPs (reported with the arena)
    uint32_t token_capacity = 0;
    uint32_t *status = nullptr;        // device status word
    uint32_t *h_status = nullptr;      // pinned mirror
    __half *h_in = nullptr;            // pinned staging for the host-buffer calls
    __half *h_res = nullptr;
    __half *h_out = nullptr;
    __half *h_out_dev = nullptr;       // device addresses of h_out and h_status (mapped host memory), or null
    uint32_t *h_status_dev = nullptr;
    uint32_t *h_ids = nullptr;
    float *h_wts = nullptr;
    uint32_t *h_seg = nullptr;         // pinned ring for the expert-parallel segment offsets
    cudaEvent_t seg_events[8] = {};
    // peer-memory exchange of an expert-parallel group (uocr_cuda_moe_ep_peer_*)
    struct {
        uint32_t world = 0, rank = 0, hidden = 0;
        uint64_t row_capacity = 0;
        __half *recv = nullptr, *done = nullptr;        // this rank's buffers
        uocr::PeerBuffers recv_all{}, done_all{};      // every rank's (own pointers + mapped peers)
        uocr::PeerSync sync{};                         // every rank's synchronisation region (it follows the received rows)
        uint32_t call = 0;                             // number of the last device-synchronised layer call
        uint32_t *d_dst_row0 = nullptr;                // [256] device copy of the scatter offsets of the current call
        bool opened = false;
    } peer;
    cudaStream_t side_stream = nullptr;   // the shared MLP of a many-token call runs here, beside routing and the routed experts
    cudaEvent_t fork_event = nullptr, join_event = nullptr;
    bool shared_pending = false;          // an expert-parallel shared-MLP call is running on the second stream
    uint32_t seg_slot = 0;
    uint64_t launches = 0;
    // engine hooks (the reference backend takes the engine's profile store and memory tracker the same way,
    // src/backend/metal/uocr_metal.h:177-178): opaque objects plus the engine functions that act on them
    uocr_profile_state *profile = nullptr;
    uocr_cuda_profile_add_event_ms_fn profile_add = nullptr;
    uocr_memory_tracker *mem_tracker = nullptr;
    uocr_cuda_memory_account_fn mem_reserve = nullptr, mem_release = nullptr;
    uint64_t tracked_model_bytes = 0, tracked_scratch_bytes = 0;     // what the tracker has been told so far
    struct ProfSpan { const char *name; cudaEvent_t start, stop; };
    std::vector<ProfSpan> prof_pending;      // spans whose events have been recorded and not yet read
    std::vector<cudaEvent_t> prof_free;      // events ready for reuse
    char last_error[1024] = {0};
};

// ---- profile spans: two CUDA events around a phase; read (and handed to the engine's store) when the context next waits
static const char *const kProfileEventNames[] = {
    "cuda.decode.moe_layer_fused",            // single-token kernel: router, shared and routed experts, combine in one launch
    "cuda.decode.moe_router",                 // few tokens: routing, activation bytes and dispatch plan
    "cuda.decode.moe_routed_experts",         // few tokens: routed experts and shared MLP (one weight-streaming kernel)
    "cuda.decode.moe_combine",
    "cuda.decode.moe_matvec",                 // shapes off the other paths: the matrix-vector kernels
    "cuda.prefill.moe_router",
    "cuda.prefill.moe_plan",
    "cuda.prefill.moe_shared_experts",
    "cuda.prefill.moe_routed_bucketed_f16",
    "cuda.prefill.moe_routed_bucketed_q8",
    "cuda.prefill.moe_routed_bucketed_q4",
    "cuda.prefill.moe_combine",
};
enum ProfileEvent { kPfFused, kPfRouter, kPfRouted, kPfCombine, kPfMatvec, kPfPrefillRouter, kPfPrefillPlan, kPfPrefillShared,
                    kPfBucketedF16, kPfBucketedQ8, kPfBucketedQ4, kPfPrefillCombine, kPfCount };
static_assert(sizeof(kProfileEventNames) / sizeof(kProfileEventNames[0]) == kPfCount, "one name per event");

extern "C" const char *uocr_cuda_profile_event_name(uint32_t index) { return index < kPfCount ? kProfileEventNames[index] : nullptr; }

static cudaEvent_t prof_event(uocr_cuda_context *ctx) {
    if (!ctx->prof_free.empty()) { cudaEvent_t e = ctx->prof_free.back(); ctx->prof_free.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    return cudaEventCreate(&e) == cudaSuccess ? e : nullptr;
}

// waits for the recorded spans and hands their durations to the engine's store
static inline void cpu_relax() {        // inside a host spin: leave the core's resources to its sibling thread
#if defined(__x86_64__) || defined(__i386__)
    __builtin_ia32_pause();
#elif defined(__aarch64__)
    asm volatile("yield" ::: "memory");
#endif
}

static void prof_flush(uocr_cuda_context *ctx) {
    for (auto &sp : ctx->prof_pending) {
        float ms = 0.f;
        if (cudaEventSynchronize(sp.stop) == cudaSuccess && cudaEventElapsedTime(&ms, sp.start, sp.stop) == cudaSuccess && ctx->profile_add)
            ctx->profile_add(ctx->profile, sp.name, (double)ms);
        ctx->prof_free.push_back(sp.start);
        ctx->prof_free.push_back(sp.stop);
    }
    ctx->prof_pending.clear();
}

struct ProfScope {      // records the start event now and the stop event when it goes out of scope (same stream)
    uocr_cuda_context *ctx;
    cudaStream_t st;
    int slot = -1;
    ProfScope(uocr_cuda_context *c, int which, cudaStream_t stream) : ctx(c), st(stream) {
        if (!ctx->profile_add) return;
        if (ctx->prof_pending.size() >= 512) prof_flush(ctx);
        cudaEvent_t a = prof_event(ctx), b = prof_event(ctx);
        if (!a || !b) return;
        cudaEventRecord(a, st);
        ctx->prof_pending.push_back({kProfileEventNames[which], a, b});
        slot = (int)ctx->prof_pending.size() - 1;
    }
    ~ProfScope() { if (slot >= 0) cudaEventRecord(ctx->prof_pending[slot].stop, st); }
};

static void track_memory(uocr_cuda_context *ctx) {      // brings the engine's tracker up to date with what the context holds
    if (!ctx->mem_tracker) return;
    auto sync = [&](int category, uint64_t now, uint64_t &told) {
        if (now > told && ctx->mem_reserve) ctx->mem_reserve(ctx->mem_tracker, category, now - told);
        if (now < told && ctx->mem_release) ctx->mem_release(ctx->mem_tracker, category, told - now);
        told = now;
    };
    sync(UOCR_CUDA_MEMORY_MODEL_VIEWS, ctx->weight_bytes, ctx->tracked_model_bytes);
    sync(UOCR_CUDA_MEMORY_MOE_SCRATCH, ctx->arena_bytes + ctx->dense_scratch_bytes, ctx->tracked_scratch_bytes);
}

extern "C" void uocr_cuda_context_set_profile(uocr_cuda_context *ctx, uocr_profile_state *profile,
                                              uocr_cuda_profile_add_event_ms_fn add_event_ms) {
    if (!ctx) return;
    prof_flush(ctx);
    ctx->profile = profile;
    ctx->profile_add = profile ? add_event_ms : nullptr;
}

extern "C" void uocr_cuda_context_set_memory_tracker(uocr_cuda_context *ctx, uocr_memory_tracker *tracker,
                                                     uocr_cuda_memory_account_fn reserve, uocr_cuda_memory_account_fn release) {
    if (!ctx) return;
    if (ctx->mem_tracker) {      // hand back what the previous tracker was told
        const uint64_t m = ctx->weight_bytes, a = ctx->arena_bytes, d = ctx->dense_scratch_bytes;
        ctx->weight_bytes = 0; ctx->arena_bytes = 0; ctx->dense_scratch_bytes = 0;
        track_memory(ctx);
        ctx->weight_bytes = m; ctx->arena_bytes = a; ctx->dense_scratch_bytes = d;
    }
    ctx->mem_tracker = tracker; ctx->mem_reserve = tracker ? reserve : nullptr; ctx->mem_release = tracker ? release : nullptr;
    ctx->tracked_model_bytes = 0; ctx->tracked_scratch_bytes = 0;
    track_memory(ctx);
}


static thread_local char g_create_error[1024];

static int fail(uocr_cuda_context *ctx, char *error, size_t error_size, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) snprintf(ctx->last_error, sizeof ctx->last_error, "%s", buf);
    else snprintf(g_create_error, sizeof g_create_error, "%s", buf);
    if (error && error_size) snprintf(error, error_size, "%s", buf);
    return 0;
}

#define CU_TRY(ctx, call)                                                                             \
    do {                                                                                              \
        cudaError_t e_ = (call);                                                                      \
        if (e_ != cudaSuccess)                                                                        \
            return fail(ctx, error, error_size, "%s failed: %s", #call, cudaGetErrorString(e_));      \
    } while (0)

static uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

static uint64_t packed_bytes(int qt, uint64_t rows, uint64_t cols) {
    return qt == UOCR_QT_F16 ? rows * cols * 2 : (qt == UOCR_QT_Q8 ? rows * cols : rows * cols / 2);
}

static bool qtype_ok(int qt) { return qt == UOCR_QT_F16 || qt == UOCR_QT_Q8 || qt == UOCR_QT_Q4; }

// ------------------------------------------------------------------------------- backend
extern "C" int uocr_cuda_is_available(void) {
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess && n > 0;
}

extern "C" const char *uocr_cuda_backend_name(void) { return "cuda"; }

extern "C" int uocr_cuda_device_count(void) {
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess ? n : 0;
}

extern "C" uocr_cuda_context *uocr_cuda_context_create(const char *resource_path, char *error, size_t error_size) {
    (void)resource_path;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        fail(nullptr, error, error_size, "no CUDA device available: %s",
             e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
        return nullptr;
    }
    uocr_cuda_context *ctx = new uocr_cuda_context();
    cudaDeviceProp prop;
    if ((e = cudaGetDevice(&ctx->device)) != cudaSuccess ||
        (e = cudaGetDeviceProperties(&prop, ctx->device)) != cudaSuccess) {
        fail(nullptr, error, error_size, "cannot query the CUDA device: %s", cudaGetErrorString(e));
        delete ctx;
        return nullptr;
    }
    if (prop.major != 10) {
        fail(nullptr, error, error_size, "device %d (%s) is compute capability %d.%d; this backend is built for sm_100a only",
             ctx->device, prop.name, prop.major, prop.minor);
        delete ctx;
        return nullptr;
    }
    if ((e = cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaMalloc(&ctx->status, ctx->status_bytes = 256 + uocr::decode_sliced_acc_bytes())) != cudaSuccess ||
        (e = cudaMemset(ctx->status, 0, ctx->status_bytes)) != cudaSuccess ||
        (e = cudaMallocHost(&ctx->h_status, 256)) != cudaSuccess ||
        (e = cudaMalloc(&ctx->d_layers, kMaxLayers * sizeof(DLayer))) != cudaSuccess ||
        (e = cudaMallocHost(&ctx->h_seg, kSegSlots * 260 * sizeof(uint32_t))) != cudaSuccess ||
        (e = uocr::init_router_kernels()) != cudaSuccess || (e = uocr::init_small_batch_kernels()) != cudaSuccess || (e = uocr::init_lm_head_kernels()) != cudaSuccess ||
        (e = uocr::init_decode_kernels()) != cudaSuccess ||
        (e = uocr::init_decode_sliced_kernels()) != cudaSuccess || (e = uocr::init_decode_batched_kernels()) != cudaSuccess ||
        (e = uocr::init_gemm_kernels()) != cudaSuccess) {
        fail(nullptr, error, error_size, "CUDA context set-up failed: %s", cudaGetErrorString(e));
        uocr_cuda_context_destroy(ctx);
        return nullptr;
    }
    for (uint32_t i = 0; i < kSegSlots; ++i) cudaEventCreateWithFlags(&ctx->seg_events[i], cudaEventDisableTiming);
    if ((e = cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&ctx->fork_event, cudaEventDisableTiming)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&ctx->join_event, cudaEventDisableTiming)) != cudaSuccess) {
        fail(nullptr, error, error_size, "CUDA context set-up failed: %s", cudaGetErrorString(e));
        uocr_cuda_context_destroy(ctx);
        return nullptr;
    }
    ctx->stream = ctx->own_stream;
    const char *off = getenv("UOCR_CUDA_DISABLE_FUSED_DECODE");
    ctx->fused_decode = !(off && off[0] == '1');
    const char *design = getenv("UOCR_CUDA_DECODE_DESIGN");      // "two-barrier": the earlier persistent kernel
    ctx->sliced_decode = !(design && strcmp(design, "two-barrier") == 0);   // (then no slice-major weight copy is made)
    if (const char *b = getenv("UOCR_CUDA_DISABLE_BATCHED_DECODE")) ctx->batched_decode = !(b[0] == '1');
    if (const char *mt = getenv("UOCR_CUDA_GEMM_MIN_TOKENS")) ctx->gemm_min_tokens = (uint32_t)strtoul(mt, nullptr, 10);
    if (const char *r = getenv("UOCR_CUDA_DECODE_REPLICAS")) ctx->decode_knobs.replicas = (uint32_t)strtoul(r, nullptr, 10);
    if (const char *r = getenv("UOCR_CUDA_DECODE_POLL_SLEEP_NS")) ctx->decode_knobs.poll_sleep_ns = (uint32_t)strtoul(r, nullptr, 10);
    // Test hooks for the time-out path of the decode kernel's waits: a shorter limit (in SM cycles), and one launch
    // whose wait for the layer output expects one contribution more than there are CTAs.  Nothing faults: the wait
    // runs into its limit, the kernel raises its status word and returns.
    if (const char *c = getenv("UOCR_CUDA_TEST_SPIN_LIMIT_CYCLES")) ctx->decode_knobs.spin_limit_cycles = strtoll(c, nullptr, 10);
    if (const char *c = getenv("UOCR_CUDA_TEST_DECODE_STALL_ONCE")) ctx->test_stall_once = c[0] == '1';
    return ctx;
}

extern "C" void uocr_cuda_context_release_runtime_arenas(uocr_cuda_context *ctx) {
    if (!ctx) return;
    cudaFree(ctx->arena);
    ctx->arena = nullptr;
    ctx->arena_bytes = 0;
    ctx->token_capacity = 0;
    track_memory(ctx);
    cudaFreeHost(ctx->h_in); cudaFreeHost(ctx->h_res); cudaFreeHost(ctx->h_out);
    cudaFreeHost(ctx->h_ids); cudaFreeHost(ctx->h_wts);
    ctx->h_in = ctx->h_res = ctx->h_out = nullptr;
    ctx->h_out_dev = nullptr; ctx->h_status_dev = nullptr;
    ctx->h_ids = nullptr;
    ctx->h_wts = nullptr;
}

extern "C" void uocr_cuda_context_unmap_model(uocr_cuda_context *ctx) {
    if (!ctx) return;
    for (void *p : ctx->weight_allocs) cudaFree(p);
    ctx->weight_allocs.clear();
    ctx->layers.clear();
    for (auto &d : ctx->dense) cudaFree(d.scratch);
    ctx->dense.clear();
    ctx->dense_scratch_bytes = 0;
    cudaFree(ctx->lm_head.scratch);
    ctx->lm_head = {};
    ctx->file_dense_index = -1;
    ctx->post_attn_norms.clear();
    ctx->final_norm = nullptr;
    ctx->weight_bytes = 0;
    track_memory(ctx);
}

extern "C" void uocr_cuda_moe_ep_peer_destroy(uocr_cuda_context *ctx);

extern "C" void uocr_cuda_context_destroy(uocr_cuda_context *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->own_stream) cudaStreamSynchronize(ctx->own_stream);
    prof_flush(ctx);
    for (cudaEvent_t e : ctx->prof_free) cudaEventDestroy(e);
    ctx->prof_free.clear();
    uocr_cuda_moe_ep_peer_destroy(ctx);
    uocr_cuda_context_release_runtime_arenas(ctx);
    uocr_cuda_context_unmap_model(ctx);
    cudaFree(ctx->status);
    cudaFree(ctx->d_layers);
    cudaFreeHost(ctx->h_seg);
    for (uint32_t i = 0; i < kSegSlots; ++i) if (ctx->seg_events[i]) cudaEventDestroy(ctx->seg_events[i]);
    cudaFreeHost(ctx->h_status);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    if (ctx->side_stream) { cudaStreamSynchronize(ctx->side_stream); cudaStreamDestroy(ctx->side_stream); }
    if (ctx->fork_event) cudaEventDestroy(ctx->fork_event);
    if (ctx->join_event) cudaEventDestroy(ctx->join_event);
    delete ctx;
}

extern "C" const char *uocr_cuda_context_last_error(const uocr_cuda_context *ctx) {
    return ctx ? ctx->last_error : g_create_error;
}

extern "C" int uocr_cuda_context_set_stream(uocr_cuda_context *ctx, void *cuda_stream) {
    if (!ctx) return 0;
    ctx->stream = cuda_stream ? (cudaStream_t)cuda_stream : ctx->own_stream;
    return 1;
}

extern "C" int uocr_cuda_context_set_profile_detail(uocr_cuda_context *ctx, void *d_trace) {
    if (!ctx) return 0;
    ctx->decode_trace = (unsigned long long *)d_trace;
    return 1;
}

extern "C" int uocr_cuda_context_synchronize(uocr_cuda_context *ctx, char *error, size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    CU_TRY(ctx, cudaMemcpyAsync(ctx->h_status, ctx->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    CU_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    prof_flush(ctx);
    if (*ctx->h_status != 0) {
        const uint32_t st = *ctx->h_status;
        // clears the status word, the decode kernels' barrier counter and accumulators (they are off after an abort)
        cudaMemsetAsync(ctx->status, 0, ctx->status_bytes, ctx->stream);
        ctx->bar_base = 0;
        ctx->acc_base = 0;
        return fail(ctx, error, error_size,
                    "device status 0x%x: %s", st,
                    (st & 1u) ? "router met a non-finite logit or an empty softmax (the CPU path rejects this input too)"
                    : (st & 2u) ? "a grid barrier of the decode kernel timed out"
                    : (st & 4u) ? "a bulk copy of the decode kernel timed out"
                    : (st & 8u) ? "a pipeline wait of the grouped GEMM kernel timed out"
                    : (st & 16u) ? "the decode kernel met a non-finite or out-of-range partial output"
                    : (st & 64u) ? "a rank of the expert-parallel group did not reach the call in time (wait for a peer's flag ran out)"
                    : (st & 32u) ? "a row index left the expert-parallel exchange buffers (inconsistent counts between the ranks)"
                                : "kernel reported an internal error");
    }
    return 1;
}

extern "C" uint64_t uocr_cuda_context_kernel_launches(const uocr_cuda_context *ctx) { return ctx ? ctx->launches : 0; }
extern "C" uint64_t uocr_cuda_context_model_view_bytes(const uocr_cuda_context *ctx) { return ctx ? ctx->weight_bytes : 0; }
extern "C" uint64_t uocr_cuda_context_moe_scratch_bytes(const uocr_cuda_context *ctx) { return ctx ? ctx->arena_bytes + ctx->dense_scratch_bytes : 0; }
// ---- mapping from an opened .uocr model file -----------------------------------------------------------------------
// The tensor directory is the file's own packed array of 140-byte entries sorted by id (src/model/uocr_format.h:275-299;
// the loader checks the order, src/model/uocr_model_file.c:885-895), so a tensor is found by binary search as
// uocr_model_file_find_tensor does.  Ids follow src/model/uocr_tensor_registry.h:22-124.
static_assert(sizeof(uocr_cuda_tensor_entry) == 140, "the on-disk tensor entry has 140 bytes");

namespace {
constexpr uint32_t kIdLayerBase = 10000, kIdLayerStride = 1000, kIdRouter = 40, kIdSharedGate = 50, kIdExpertBase = 100;
constexpr uint32_t kUsageRuntime = 1, kFlagRowMajor = 1;

const uocr_cuda_tensor_entry *find_entry(const uocr_cuda_model_file_view *m, uint32_t id) {
    const uocr_cuda_tensor_entry *t = (const uocr_cuda_tensor_entry *)m->tensors;
    uint32_t lo = 0, hi = m->tensor_count;
    while (lo < hi) {
        const uint32_t mid = lo + (hi - lo) / 2;
        if (t[mid].id == id) return &t[mid];
        if (t[mid].id < id) lo = mid + 1; else hi = mid;
    }
    return nullptr;
}

// One projection of the file checked against what this backend can consume: a runtime, row-major, rank-2 tensor of a
// known qtype whose byte ranges lie inside the file and are as long as the shape says.
const char *check_entry(const uocr_cuda_model_file_view *m, const uocr_cuda_tensor_entry *t) {
    if (!t) return "is missing from the tensor directory";
    if (t->usage != kUsageRuntime) return "is not a runtime tensor";
    if (t->rank != 2 || !(t->flags & kFlagRowMajor)) return "is not a row-major matrix";
    if (t->qtype != UOCR_QT_F16 && t->qtype != UOCR_QT_Q8 && t->qtype != UOCR_QT_Q4) return "has an unsupported qtype";
    const uint64_t rows = t->logical_shape[0], cols = t->logical_shape[1];
    if (rows == 0 || cols == 0 || t->physical_shape[0] != rows || t->physical_shape[1] != cols) return "has an invalid shape";
    if (t->qtype != UOCR_QT_F16 && cols % UOCR_GROUP) return "has a width that is no multiple of the quantisation group";
    const uint64_t want = t->qtype == UOCR_QT_F16 ? rows * cols * 2 : t->qtype == UOCR_QT_Q8 ? rows * cols : rows * cols / 2;
    if (t->payload_size != want) return "has a payload size that does not match its shape";
    if (t->payload_offset > m->size || t->payload_size > m->size - t->payload_offset) return "has a payload outside the file";
    if (t->payload_offset % 16) return "has a payload that is not 16-byte aligned";
    if (t->qtype != UOCR_QT_F16) {
        if (t->scale_size != rows * (cols / UOCR_GROUP) * 2) return "has a scale size that does not match its shape";
        if (t->scale_offset > m->size || t->scale_size > m->size - t->scale_offset) return "has scales outside the file";
        if (t->scale_offset % 16) return "has scales that are not 16-byte aligned";
    }
    return nullptr;
}

uocr_cuda_matrix matrix_of(const uocr_cuda_model_file_view *m, const uocr_cuda_tensor_entry *t) {
    const uint8_t *base = (const uint8_t *)m->data;
    return uocr_cuda_matrix{(int32_t)t->qtype, t->logical_shape[0], t->logical_shape[1], base + t->payload_offset,
                            t->qtype == UOCR_QT_F16 ? nullptr : base + t->scale_offset};
}
}  // namespace

extern "C" int uocr_cuda_context_map_model(uocr_cuda_context *ctx, const uocr_cuda_model_file_view *m, char *error,
                                           size_t error_size) {
    if (!ctx || !m) return fail(ctx, error, error_size, "null context or model view");
    if (!m->data || !m->tensors || m->tensor_count == 0) return fail(ctx, error, error_size, "model view without data or tensor directory");
    if ((const uint8_t *)m->tensors < (const uint8_t *)m->data ||
        (uint64_t)((const uint8_t *)m->tensors - (const uint8_t *)m->data) + (uint64_t)m->tensor_count * sizeof(uocr_cuda_tensor_entry) > m->size)
        return fail(ctx, error, error_size, "tensor directory lies outside the model file");
    if (m->moe_layer_count == 0) return fail(ctx, error, error_size, "no MoE layer requested");
    if (!ctx->layers.empty()) return fail(ctx, error, error_size, "a model is already mapped; call uocr_cuda_context_unmap_model first");
    const uint32_t E = m->routed_experts, K = m->moe_top_k;
    if (E == 0 || E > 256 || K == 0 || K > E) return fail(ctx, error, error_size, "invalid router configuration (experts %u, top_k %u)", E, K);

    // every layer is checked before the first one is uploaded, so a refused file leaves the context empty
    auto one_layer = [&](uint32_t layer, bool upload_it) -> int {
        const uint32_t lbase = kIdLayerBase + layer * kIdLayerStride;
        const uocr_cuda_tensor_entry *router = find_entry(m, lbase + kIdRouter);
        const uocr_cuda_tensor_entry *shared[3], *gate0 = find_entry(m, lbase + kIdExpertBase);
        const char *why = check_entry(m, router);
        if (why) return fail(ctx, error, error_size, "layer %u: MoE router %s", layer, why);
        static const char *kProj[3] = {"gate", "up", "down"};
        for (int p = 0; p < 3; ++p) {
            shared[p] = find_entry(m, lbase + kIdSharedGate + p);
            if ((why = check_entry(m, shared[p]))) return fail(ctx, error, error_size, "layer %u: MoE shared %s %s", layer, kProj[p], why);
        }
        if ((why = check_entry(m, gate0))) return fail(ctx, error, error_size, "layer %u: MoE expert 0 gate %s", layer, why);
        if (router->qtype != UOCR_QT_F16) return fail(ctx, error, error_size, "layer %u: the MoE router must be fp16", layer);
        const uint32_t H = router->logical_shape[1], F = gate0->logical_shape[0], S = shared[0]->logical_shape[0];
        if (router->logical_shape[0] != E) return fail(ctx, error, error_size, "layer %u: router has %u rows for %u experts", layer, router->logical_shape[0], E);
        if (gate0->logical_shape[1] != H) return fail(ctx, error, error_size, "layer %u: expert gate width %u differs from the hidden size %u", layer, gate0->logical_shape[1], H);

        // the expert slab: every expert's gate, up and down follow one another without a gap, packed weights in one
        // run and scales in another — the rule of src/backend/metal/uocr_metal.m:3037-3154
        const uint32_t qt = gate0->qtype;
        const uint64_t proj = gate0->payload_size, proj_scales = qt == UOCR_QT_F16 ? 0 : gate0->scale_size;
        for (uint32_t e = 0; e < E; ++e)
            for (uint32_t p = 0; p < 3; ++p) {
                const uocr_cuda_tensor_entry *t = find_entry(m, lbase + kIdExpertBase + 3 * e + p);
                if ((why = check_entry(m, t))) return fail(ctx, error, error_size, "layer %u: MoE expert %u %s %s", layer, e, kProj[p], why);
                const uint32_t rows = p == 2 ? H : F, cols = p == 2 ? F : H;
                if (t->qtype != qt || t->logical_shape[0] != rows || t->logical_shape[1] != cols)
                    return fail(ctx, error, error_size, "layer %u: MoE expert %u %s differs in qtype or shape from expert 0", layer, e, kProj[p]);
                if (t->payload_offset != gate0->payload_offset + (3ull * e + p) * proj)
                    return fail(ctx, error, error_size, "integrated MoE expert tensors for layer %u are not interleaved-contiguous at expert %u", layer, e);
                if (qt != UOCR_QT_F16 && t->scale_offset != gate0->scale_offset + (3ull * e + p) * proj_scales)
                    return fail(ctx, error, error_size, "integrated MoE expert qscale tensors for layer %u are not interleaved-contiguous at expert %u", layer, e);
            }

        if (!upload_it) return 1;
        uocr_cuda_moe_layer_desc d{};
        d.hidden_size = H; d.n_experts = E; d.top_k = K; d.expert_intermediate = F; d.shared_intermediate = S;
        d.routed_scaling_factor = m->routed_scaling_factor;
        const uint8_t *base = (const uint8_t *)m->data;
        d.router_weight_f16 = base + router->payload_offset;
        d.expert_qtype = (int32_t)qt;
        d.expert_qweight = base + gate0->payload_offset;
        d.expert_qscale = qt == UOCR_QT_F16 ? nullptr : base + gate0->scale_offset;
        d.shared_gate = matrix_of(m, shared[0]);
        d.shared_up = matrix_of(m, shared[1]);
        d.shared_down = matrix_of(m, shared[2]);
        char inner[512] = {0};
        if (!uocr_cuda_context_map_moe_layer(ctx, &d, nullptr, inner, sizeof inner)) {
            uocr_cuda_context_unmap_model(ctx);
            return fail(ctx, error, error_size, "layer %u: %s", layer, inner);
        }
        return 1;
    };
    for (int pass = 0; pass < 2; ++pass)
        for (uint32_t layer = m->first_moe_layer; layer < m->first_moe_layer + m->moe_layer_count; ++layer)
            if (!one_layer(layer, pass == 1)) return 0;
    return 1;
}

extern "C" uint32_t uocr_cuda_context_moe_layer_count(const uocr_cuda_context *ctx) {
    return ctx ? (uint32_t)ctx->layers.size() : 0;
}

// ---- the tensors either side of the MoE layers, from the same file ------------------------------------------------
static int upload(uocr_cuda_context *ctx, const void *host, uint64_t bytes, void **out, char *error, size_t error_size);

namespace {
constexpr uint32_t kIdLmHead = 2, kIdFinalNorm = 3, kIdPostAttnNorm = 2, kIdDenseGate = 30;

// a norm weight: a runtime fp16 vector whose bytes lie inside the file
const char *check_norm_entry(const uocr_cuda_model_file_view *m, const uocr_cuda_tensor_entry *t, uint32_t H) {
    if (t->usage != kUsageRuntime) return "is not a runtime tensor";
    if (t->qtype != UOCR_QT_F16 || t->rank != 1) return "is not an fp16 vector";
    if (t->logical_shape[0] != H || t->payload_size != (uint64_t)H * 2) return "does not have the hidden size";
    if (t->payload_offset > m->size || t->payload_size > m->size - t->payload_offset) return "has a payload outside the file";
    return nullptr;
}
}  // namespace

extern "C" int uocr_cuda_context_map_model_neighbours(uocr_cuda_context *ctx, const uocr_cuda_model_file_view *m,
                                                      uint32_t token_capacity, char *error, size_t error_size) {
    if (!ctx || !m) return fail(ctx, error, error_size, "null context or model view");
    if (ctx->layers.empty()) return fail(ctx, error, error_size, "map the MoE layers first (uocr_cuda_context_map_model)");
    if (ctx->file_dense_index >= 0 || ctx->final_norm || !ctx->post_attn_norms.empty() || ctx->lm_head.mapped)
        return fail(ctx, error, error_size, "the neighbouring tensors are already mapped; call uocr_cuda_context_unmap_model first");
    if (!m->data || !m->tensors || m->tensor_count == 0) return fail(ctx, error, error_size, "model view without data or tensor directory");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    const uint32_t H = ctx->layers[0].H;
    const uint8_t *base = (const uint8_t *)m->data;
    const char *why = nullptr;
    static const char *kProj[3] = {"gate", "up", "down"};

    // check everything that is present before anything is uploaded
    const uocr_cuda_tensor_entry *dense[3], *head = find_entry(m, kIdLmHead), *fnorm = find_entry(m, kIdFinalNorm);
    int dense_present = 0;
    for (int p = 0; p < 3; ++p) dense_present += (dense[p] = find_entry(m, kIdLayerBase + kIdDenseGate + p)) != nullptr;
    if (dense_present != 0 && dense_present != 3) return fail(ctx, error, error_size, "layer 0: the dense MLP is incomplete (%d of 3 projections)", dense_present);
    if (dense_present == 3) {
        if (token_capacity == 0) return fail(ctx, error, error_size, "the dense MLP needs a token capacity");
        for (int p = 0; p < 3; ++p)
            if ((why = check_entry(m, dense[p]))) return fail(ctx, error, error_size, "layer 0: dense MLP %s %s", kProj[p], why);
        const uint32_t S = dense[0]->logical_shape[0];
        if (dense[0]->logical_shape[1] != H || dense[1]->logical_shape[0] != S || dense[1]->logical_shape[1] != H ||
            dense[2]->logical_shape[0] != H || dense[2]->logical_shape[1] != S)
            return fail(ctx, error, error_size, "layer 0: dense MLP shapes do not fit the hidden size %u", H);
    }
    if (head && (why = check_entry(m, head))) return fail(ctx, error, error_size, "LM head %s", why);
    if (head && head->logical_shape[1] != H) return fail(ctx, error, error_size, "LM head width %u differs from the hidden size %u", head->logical_shape[1], H);
    if (fnorm && (why = check_norm_entry(m, fnorm, H))) return fail(ctx, error, error_size, "final norm %s", why);
    const uint32_t decoder_layers = m->first_moe_layer + m->moe_layer_count;
    std::vector<const uocr_cuda_tensor_entry *> norms(decoder_layers, nullptr);
    for (uint32_t l = 0; l < decoder_layers; ++l) {
        norms[l] = find_entry(m, kIdLayerBase + l * kIdLayerStride + kIdPostAttnNorm);
        if (norms[l] && (why = check_norm_entry(m, norms[l], H))) return fail(ctx, error, error_size, "layer %u: post-attention norm %s", l, why);
    }

    char inner[512] = {0};
    if (dense_present == 3) {
        const uocr_cuda_matrix g = matrix_of(m, dense[0]), u = matrix_of(m, dense[1]), d = matrix_of(m, dense[2]);
        uint32_t index = 0;
        if (!uocr_cuda_context_map_dense_mlp(ctx, &g, &u, &d, token_capacity, &index, inner, sizeof inner))
            return fail(ctx, error, error_size, "layer 0: dense MLP: %s", inner);
        ctx->file_dense_index = (int)index;
    }
    if (head) {
        const uocr_cuda_matrix w = matrix_of(m, head);
        if (!uocr_cuda_context_map_lm_head(ctx, &w, inner, sizeof inner)) return fail(ctx, error, error_size, "LM head: %s", inner);
    }
    ctx->post_attn_norms.assign(decoder_layers, nullptr);
    for (uint32_t l = 0; l < decoder_layers; ++l)
        if (norms[l]) {
            void *d = nullptr;
            if (!upload(ctx, base + norms[l]->payload_offset, norms[l]->payload_size, &d, error, error_size)) return 0;
            ctx->post_attn_norms[l] = (const __half *)d;
        }
    if (fnorm) {
        void *d = nullptr;
        if (!upload(ctx, base + fnorm->payload_offset, fnorm->payload_size, &d, error, error_size)) return 0;
        ctx->final_norm = (const __half *)d;
    }
    track_memory(ctx);
    return 1;
}

extern "C" int uocr_cuda_context_file_dense_mlp_index(const uocr_cuda_context *ctx) { return ctx ? ctx->file_dense_index : -1; }
extern "C" const void *uocr_cuda_context_post_attn_norm_weight(const uocr_cuda_context *ctx, uint32_t decoder_layer) {
    return ctx && decoder_layer < ctx->post_attn_norms.size() ? ctx->post_attn_norms[decoder_layer] : nullptr;
}
extern "C" const void *uocr_cuda_context_final_norm_weight(const uocr_cuda_context *ctx) { return ctx ? ctx->final_norm : nullptr; }

// ----------------------------------------------------------------------------- map model
static int upload(uocr_cuda_context *ctx, const void *host, uint64_t bytes, void **out, char *error, size_t error_size) {
    void *d = nullptr;
    CU_TRY(ctx, cudaMalloc(&d, bytes + kUploadPad));
    ctx->weight_allocs.push_back(d);
    CU_TRY(ctx, cudaMemset((uint8_t *)d + bytes, 0, kUploadPad));
    CU_TRY(ctx, cudaMemcpy(d, host, bytes, cudaMemcpyHostToDevice));
    ctx->weight_bytes += bytes;
    *out = d;
    return 1;
}

static int check_matrix(uocr_cuda_context *ctx, const uocr_cuda_matrix &m, uint32_t rows, uint32_t cols, const char *name,
                        char *error, size_t error_size) {
    if (!qtype_ok(m.qtype)) return fail(ctx, error, error_size, "%s: unsupported qtype %d", name, m.qtype);
    if (m.rows != rows || m.cols != cols)
        return fail(ctx, error, error_size, "%s: shape [%u,%u] does not match the layer ([%u,%u] expected)", name, m.rows,
                    m.cols, rows, cols);
    if (!m.qweight) return fail(ctx, error, error_size, "%s: null weight pointer", name);
    if (m.qtype != UOCR_QT_F16 && !m.qscale) return fail(ctx, error, error_size, "%s: quantised tensor without scales", name);
    return 1;
}

extern "C" int uocr_cuda_context_map_moe_layer(uocr_cuda_context *ctx, const uocr_cuda_moe_layer_desc *d,
                                               uint32_t *out_layer_index, char *error, size_t error_size) {
    if (!ctx || !d) return fail(ctx, error, error_size, "null context or layer descriptor");
    const uint32_t H = d->hidden_size, E = d->n_experts, K = d->top_k, F = d->expert_intermediate,
                   S = d->shared_intermediate;
    // argument rules of moe_validate_common (src/backend/cpu_ref/uocr_cpu_ref.c:357-377) plus the format's
    if (H == 0 || E == 0 || K == 0 || F == 0 || S == 0) return fail(ctx, error, error_size, "zero layer dimension");
    if (K > E) return fail(ctx, error, error_size, "top_k %u exceeds n_experts %u", K, E);
    if (E > 256 || K > 16) return fail(ctx, error, error_size, "unsupported router size: n_experts %u (max 256), top_k %u (max 16)", E, K);
    if (!(d->routed_scaling_factor >= 0.0f) || !std::isfinite(d->routed_scaling_factor))
        return fail(ctx, error, error_size, "routed_scaling_factor must be finite and >= 0");
    if (H % UOCR_GROUP || F % UOCR_GROUP || S % UOCR_GROUP)
        return fail(ctx, error, error_size, "hidden (%u), expert (%u) and shared (%u) widths must be multiples of 64", H, F, S);
    if (H > 2048 || F > 2048 || S > 2048)
        return fail(ctx, error, error_size, "layer widths above 2048 are not supported (hidden %u, expert %u, shared %u)", H, F, S);
    if (!d->router_weight_f16) return fail(ctx, error, error_size, "null router weight");
    if (!qtype_ok(d->expert_qtype)) return fail(ctx, error, error_size, "unsupported expert qtype %d", d->expert_qtype);
    if (!d->expert_qweight) return fail(ctx, error, error_size, "null expert weight slab");
    if (d->expert_qtype != UOCR_QT_F16 && !d->expert_qscale) return fail(ctx, error, error_size, "quantised expert slab without scales");
    if (!check_matrix(ctx, d->shared_gate, S, H, "shared gate", error, error_size) ||
        !check_matrix(ctx, d->shared_up, S, H, "shared up", error, error_size) ||
        !check_matrix(ctx, d->shared_down, H, S, "shared down", error, error_size))
        return 0;
    if (d->shared_gate.qtype != d->shared_up.qtype)
        return fail(ctx, error, error_size, "shared gate and up projections must share one qtype");

    const int qt = d->expert_qtype;
    const uint64_t proj = packed_bytes(qt, F, H);
    const uint64_t proj_scales = qt == UOCR_QT_F16 ? 0 : (uint64_t)F * (H / UOCR_GROUP);
    DLayer L{};
    L.H = H; L.E = E; L.K = K; L.F = F; L.S = S;
    L.scaling = d->routed_scaling_factor;
    L.expert_qtype = qt;
    L.expert_stride_bytes = d->expert_stride_bytes ? d->expert_stride_bytes : 3 * proj;
    L.up_offset_bytes = d->up_offset_bytes ? d->up_offset_bytes : proj;
    L.down_offset_bytes = d->down_offset_bytes ? d->down_offset_bytes : 2 * proj;
    L.expert_scale_stride = d->expert_scale_stride_values ? d->expert_scale_stride_values : 3 * proj_scales;
    L.up_scale_offset = d->up_scale_offset_values ? d->up_scale_offset_values : proj_scales;
    L.down_scale_offset = d->down_scale_offset_values ? d->down_scale_offset_values : 2 * proj_scales;
    // the slab consistency rules the reference host enforces before binding a layer
    // (src/backend/metal/uocr_metal.m:3037-3154): projections inside the expert stride, 16-byte alignment
    if (L.up_offset_bytes < proj || L.down_offset_bytes < L.up_offset_bytes + proj ||
        L.expert_stride_bytes < L.down_offset_bytes + proj || (L.expert_stride_bytes | L.up_offset_bytes | L.down_offset_bytes) % 16)
        return fail(ctx, error, error_size, "inconsistent expert slab strides");
    if (qt != UOCR_QT_F16 && (L.up_scale_offset < proj_scales || L.down_scale_offset < L.up_scale_offset + proj_scales ||
                              L.expert_scale_stride < L.down_scale_offset + proj_scales ||
                              (L.expert_scale_stride | L.up_scale_offset | L.down_scale_offset) % 8))
        return fail(ctx, error, error_size, "inconsistent expert scale slab strides");

    CU_TRY(ctx, cudaSetDevice(ctx->device));
    void *p = nullptr;
    if (!upload(ctx, d->router_weight_f16, (uint64_t)E * H * 2, &p, error, error_size)) return 0;
    L.router = (const __half *)p;
    if (d->router_logit_bias) {
        if (!upload(ctx, d->router_logit_bias, (uint64_t)E * 4, &p, error, error_size)) return 0;
        L.bias = (const float *)p;
    }
    if (!upload(ctx, d->expert_qweight, (uint64_t)E * L.expert_stride_bytes, &p, error, error_size)) return 0;
    L.expert_w = (const uint8_t *)p;
    if (qt != UOCR_QT_F16) {
        if (!upload(ctx, d->expert_qscale, (uint64_t)E * L.expert_scale_stride * 2, &p, error, error_size)) return 0;
        L.expert_s = (const __half *)p;
    }
    // shared gate and up go into one allocation (gate first) so kernels address "up" as a positive offset
    {
        const int sq = d->shared_gate.qtype;
        const uint64_t wb = packed_bytes(sq, S, H), sb = sq == UOCR_QT_F16 ? 0 : (uint64_t)S * (H / UOCR_GROUP) * 2;
        uint8_t *dw = nullptr;
        CU_TRY(ctx, cudaMalloc(&dw, 2 * wb + kUploadPad));
        ctx->weight_allocs.push_back(dw);
        CU_TRY(ctx, cudaMemcpy(dw, d->shared_gate.qweight, wb, cudaMemcpyHostToDevice));
        CU_TRY(ctx, cudaMemcpy(dw + wb, d->shared_up.qweight, wb, cudaMemcpyHostToDevice));
        uint8_t *ds = nullptr;
        if (sb) {
            CU_TRY(ctx, cudaMalloc(&ds, 2 * sb + kUploadPad));
            ctx->weight_allocs.push_back(ds);
            CU_TRY(ctx, cudaMemcpy(ds, d->shared_gate.qscale, sb, cudaMemcpyHostToDevice));
            CU_TRY(ctx, cudaMemcpy(ds + sb, d->shared_up.qscale, sb, cudaMemcpyHostToDevice));
        }
        ctx->weight_bytes += 2 * (wb + sb);
        const uint32_t rb = (uint32_t)(wb / S);
        L.shared_gate = DMatrix{dw, (const __half *)ds, S, H, rb, sq};
        L.shared_up = DMatrix{dw + wb, ds ? (const __half *)(ds + sb) : nullptr, S, H, rb, sq};
    }
    {
        const int sq = d->shared_down.qtype;
        const uint64_t wb = packed_bytes(sq, H, S), sb = sq == UOCR_QT_F16 ? 0 : (uint64_t)H * (S / UOCR_GROUP) * 2;
        if (!upload(ctx, d->shared_down.qweight, wb, &p, error, error_size)) return 0;
        void *ps = nullptr;
        if (sb && !upload(ctx, d->shared_down.qscale, sb, &ps, error, error_size)) return 0;
        L.shared_down = DMatrix{(const uint8_t *)p, (const __half *)ps, H, S, (uint32_t)(wb / H), sq};
    }
    // slice-major copy of the weights for the one-barrier decode kernel (model shapes, quantised, kernel enabled)
    if (ctx->fused_decode && ctx->sliced_decode && uocr::decode_sliced_layer_ok(L)) {
        const size_t bytes = uocr::decode_units_bytes(L);
        uint8_t *units = nullptr;
        CU_TRY(ctx, cudaMalloc(&units, bytes + kUploadPad));
        ctx->weight_allocs.push_back(units);
        ctx->weight_bytes += bytes;
        CU_TRY(ctx, uocr::build_decode_units(L, units, ctx->own_stream));
        CU_TRY(ctx, cudaStreamSynchronize(ctx->own_stream));
        L.dec_units = units;
    }
    if (!ctx->layers.empty()) {
        const DLayer &f = ctx->layers.front();
        if (f.H != H) return fail(ctx, error, error_size, "all mapped layers must share hidden_size (%u vs %u)", f.H, H);
    }
    if (ctx->layers.size() >= kMaxLayers) return fail(ctx, error, error_size, "at most %u layers can be mapped", kMaxLayers);
    ctx->layers.push_back(L);
    CU_TRY(ctx, cudaMemcpy(ctx->d_layers, ctx->layers.data(), ctx->layers.size() * sizeof(DLayer), cudaMemcpyHostToDevice));
    if (out_layer_index) *out_layer_index = (uint32_t)ctx->layers.size() - 1;
    track_memory(ctx);
    return 1;
}

// ----------------------------------------------------------------------------------- arena
struct ArenaLayout {
    uint64_t logits, probs, ids, weights, offsets, pair_rows, inverse, active, mid, shared_mid, down_out, shared_out,
        stack0, stack1, d_in, d_res, d_out, dec_mid, dec_plogits, x_sorted, tiles_gu, tiles_dn, stiles_gu, stiles_dn,
        counts, plan_counts, seg_offsets, bt_routed, total;
};

static ArenaLayout layout_arena(uint32_t H, uint32_t E, uint32_t K, uint32_t F, uint32_t S, uint32_t n) {
    ArenaLayout a{};
    uint64_t off = 0;
    auto take = [&](uint64_t bytes) { uint64_t o = off; off = align_up(off + bytes, 256); return o; };
    const uint64_t pairs = (uint64_t)n * K;
    a.logits = take((uint64_t)n * E * 4);
    a.probs = take((uint64_t)n * E * 4);
    a.ids = take(pairs * 4);
    a.weights = take(pairs * 4);
    a.offsets = take((uint64_t)(E + 1) * 4);
    a.pair_rows = take(pairs * 4);
    a.inverse = take(pairs * 4);
    a.active = take((uint64_t)(E + 1) * 4);
    a.mid = take(pairs * F * 2);
    a.shared_mid = take((uint64_t)n * S * 2);
    // routed down products: f32 on the matrix-vector path, fp16 on the tensor-core path.  Which path a call takes
    // depends on the layer's shapes and on a run-time threshold, so the slot always has room for f32.
    a.down_out = take(pairs * H * 4);
    a.shared_out = take((uint64_t)n * H * 4);
    a.stack0 = take((uint64_t)n * H * 2);
    a.stack1 = take((uint64_t)n * H * 2);
    a.d_in = take((uint64_t)n * H * 2);
    a.d_res = take((uint64_t)n * H * 2);
    a.d_out = take((uint64_t)n * H * 2);
    a.dec_mid = take(((uint64_t)K * F + S) * 2);            // single-token decode kernel: SwiGLU products
    a.dec_plogits = take((uint64_t)1024 * E * 4);           // and per-CTA partial router logits
    {   // tensor-core path: sorted activations and tile lists (a tile is 128 tokens x 128 rows of down, or x 64 rows each
        // of gate and up); the experts phase of an expert-parallel rank sees up to E segments
        const uint64_t ttiles = (pairs + 127) / 128 + E, sttiles = ((uint64_t)n + 127) / 128;
        a.x_sorted = take(pairs * H * 2);
        a.tiles_gu = take(ttiles * (F / 64 + 1) * 16);
        a.tiles_dn = take(ttiles * (H / 128 + 1) * 16);
        a.stiles_gu = take(sttiles * (S / 64 + 1) * 16);
        a.stiles_dn = take(sttiles * (H / 128 + 1) * 16);
        a.counts = take(64);
        a.seg_offsets = take(260 * 4);        // expert-parallel experts phase: offsets of the received segments
        a.plan_counts = take((pairs / 2048 + 2) * E * 4);
    }
    {   // batched decode path (calls of up to 64 tokens): the call's fixed-point output sums, the tokens' activation bytes
        const uint32_t nb = n < uocr::decode_batched_max_tokens() ? n : uocr::decode_batched_max_tokens();
        a.bt_routed = take(uocr::decode_batched_scratch(nb, K).total);
    }
    a.total = off;
    return a;
}

extern "C" uint64_t uocr_cuda_moe_scratch_size(uint32_t H, uint32_t E, uint32_t K, uint32_t F, uint32_t S,
                                               uint32_t token_capacity) {
    if (!H || !E || !K || !F || !S || !token_capacity) return 0;
    return layout_arena(H, E, K, F, S, token_capacity).total;
}

struct LayerDims { uint32_t H = 0, E = 0, K = 0, F = 0, S = 0; };

static LayerDims max_dims(const uocr_cuda_context *ctx) {
    LayerDims m;
    for (const DLayer &L : ctx->layers) {
        m.H = L.H > m.H ? L.H : m.H; m.E = L.E > m.E ? L.E : m.E; m.K = L.K > m.K ? L.K : m.K;
        m.F = L.F > m.F ? L.F : m.F; m.S = L.S > m.S ? L.S : m.S;
    }
    return m;
}

extern "C" int uocr_cuda_context_allocate_runtime_arenas(uocr_cuda_context *ctx, uint32_t batch_slots,
                                                         uint32_t token_capacity, char *error, size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    if (batch_slots != 1) return fail(ctx, error, error_size, "batch_slots must be 1 (one request per context, as the reference engine)");
    if (token_capacity == 0) return fail(ctx, error, error_size, "token_capacity must be positive");
    if (ctx->layers.empty()) return fail(ctx, error, error_size, "map the model's MoE layers before sizing the arenas");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    uocr_cuda_context_release_runtime_arenas(ctx);
    const LayerDims m = max_dims(ctx);
    const uint64_t bytes = layout_arena(m.H, m.E, m.K, m.F, m.S, token_capacity).total;
    CU_TRY(ctx, cudaMalloc(&ctx->arena, bytes));
    ctx->arena_bytes = bytes;
    ctx->token_capacity = token_capacity;
    track_memory(ctx);
    const size_t act = (size_t)token_capacity * m.H * 2;
    CU_TRY(ctx, cudaMallocHost(&ctx->h_in, act));
    CU_TRY(ctx, cudaMallocHost(&ctx->h_res, act));
    CU_TRY(ctx, cudaMallocHost(&ctx->h_out, act));
    {   // pinned memory is mapped into the device's address space where addressing is unified; else the copies stay
        void *dp = nullptr, *ds = nullptr;
        if (cudaHostGetDevicePointer(&dp, ctx->h_out, 0) == cudaSuccess && ctx->h_status &&
            cudaHostGetDevicePointer(&ds, ctx->h_status, 0) == cudaSuccess) {
            ctx->h_out_dev = (__half *)dp;
            ctx->h_status_dev = (uint32_t *)ds;
        } else {
            (void)cudaGetLastError();
        }
    }
    const size_t small = (size_t)token_capacity * m.K * 4 > 4096 ? (size_t)token_capacity * m.K * 4 : 4096;
    CU_TRY(ctx, cudaMallocHost(&ctx->h_ids, small));
    CU_TRY(ctx, cudaMallocHost(&ctx->h_wts, small));
    return 1;
}

static Scratch carve(const uocr_cuda_context *ctx, const DLayer &L, uint32_t n, ArenaLayout *out_layout = nullptr) {
    const ArenaLayout a = layout_arena(L.H, L.E, L.K, L.F, L.S, n);
    uint8_t *b = ctx->arena;
    Scratch s{};
    s.logits = (float *)(b + a.logits); s.probs = (float *)(b + a.probs);
    s.top_ids = (uint32_t *)(b + a.ids); s.top_weights = (float *)(b + a.weights);
    s.expert_offsets = (uint32_t *)(b + a.offsets); s.pair_rows = (uint32_t *)(b + a.pair_rows);
    s.inverse = (uint32_t *)(b + a.inverse); s.active = (uint32_t *)(b + a.active);
    s.plan_counts = (uint32_t *)(b + a.plan_counts);
    s.mid = (__half *)(b + a.mid); s.shared_mid = (__half *)(b + a.shared_mid);
    s.down_out = b + a.down_out; s.shared_out = (float *)(b + a.shared_out);
    s.status = ctx->status;
    if (out_layout) *out_layout = a;
    return s;
}

static int check_call(uocr_cuda_context *ctx, uint32_t layer, uint32_t n, char *error, size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    if (layer >= ctx->layers.size()) return fail(ctx, error, error_size, "layer index %u out of range (%zu mapped)", layer, ctx->layers.size());
    if (n == 0) return fail(ctx, error, error_size, "n_tokens must be positive");
    if (!ctx->arena || n > ctx->token_capacity)
        return fail(ctx, error, error_size, "n_tokens %u exceeds the arena capacity %u (call uocr_cuda_context_allocate_runtime_arenas)", n, ctx->token_capacity);
    return 1;
}

// ------------------------------------------------------------------------------ operators
extern "C" int uocr_cuda_moe_router(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden, const float *d_injected,
                                    uint32_t n, float *d_logits, float *d_probs, uint32_t *d_ids, float *d_weights,
                                    char *error, size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if ((!d_hidden && !d_injected) || !d_ids || !d_weights) return fail(ctx, error, error_size, "null router argument");
    const DLayer &L = ctx->layers[layer];
    CU_TRY(ctx, uocr::launch_router(L, (const __half *)d_hidden, d_injected, n, d_logits, d_probs, d_ids, d_weights,
                                    ctx->status, carve(ctx, L, n).logits, ctx->stream, &ctx->launches));
    return 1;
}

extern "C" int uocr_cuda_moe_dispatch_plan(uocr_cuda_context *ctx, const uint32_t *d_ids, uint32_t n, uint32_t K, uint32_t E,
                                           uint32_t *d_offsets, uint32_t *d_pair_rows, uint32_t *d_inverse, char *error,
                                           size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    if (!d_ids || !d_offsets || !d_pair_rows || !d_inverse) return fail(ctx, error, error_size, "null dispatch-plan argument");
    if (n == 0 || K == 0 || E == 0 || E > 256 || K > E) return fail(ctx, error, error_size, "invalid dispatch-plan dimensions");
    if (!ctx->arena) return fail(ctx, error, error_size, "arenas not allocated");
    // the list of non-empty experts is an internal by-product; park it in the arena's slot
    const LayerDims m = max_dims(ctx);
    if (E > m.E) return fail(ctx, error, error_size, "n_experts %u exceeds the mapped layers' %u", E, m.E);
    // scratch of the plan kernels sits in the arena when the call fits the sizes the arena was laid out for
    const bool fits = n <= ctx->token_capacity && K <= m.K;
    const ArenaLayout a = layout_arena(m.H, m.E, m.K, m.F, m.S, fits ? n : 1);
    CU_TRY(ctx, uocr::launch_dispatch_plan(d_ids, n, K, E, d_offsets, d_pair_rows, d_inverse,
                                           (uint32_t *)(ctx->arena + a.active),
                                           fits ? (uint32_t *)(ctx->arena + a.plan_counts) : nullptr, ctx->stream,
                                           &ctx->launches));
    return 1;
}

// settings of the next sliced decode launch (the stall hook applies to one launch only)
static uocr::SlicedKnobs take_decode_knobs(uocr_cuda_context *ctx) {
    uocr::SlicedKnobs k = ctx->decode_knobs;
    if (ctx->test_stall_once) { k.expect_extra = 1; ctx->test_stall_once = false; }
    return k;
}

extern "C" int uocr_cuda_moe_debug_dequantize(uocr_cuda_context *ctx, uint32_t layer, uint32_t matrix, uint32_t expert,
                                              uint32_t path, float *d_out, char *error, size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    if (layer >= ctx->layers.size()) return fail(ctx, error, error_size, "layer index %u out of range (%zu mapped)", layer, ctx->layers.size());
    if (!d_out) return fail(ctx, error, error_size, "null output pointer");
    const DLayer &L = ctx->layers[layer];
    DMatrix m{};
    if (matrix < 3) {          // gate, up, down of one routed expert, addressed exactly as the layer kernels address them
        if (expert >= L.E) return fail(ctx, error, error_size, "expert %u out of range (%u experts)", expert, L.E);
        const uint32_t rows = matrix == 2 ? L.H : L.F, cols = matrix == 2 ? L.F : L.H;
        const uint64_t woff = matrix == 0 ? 0 : (matrix == 1 ? L.up_offset_bytes : L.down_offset_bytes);
        const uint64_t soff = matrix == 0 ? 0 : (matrix == 1 ? L.up_scale_offset : L.down_scale_offset);
        m.w = L.expert_w + (size_t)expert * L.expert_stride_bytes + woff;
        m.s = L.expert_s ? L.expert_s + (size_t)expert * L.expert_scale_stride + soff : nullptr;
        m.rows = rows; m.cols = cols; m.qtype = L.expert_qtype;
        m.row_bytes = (uint32_t)packed_bytes(L.expert_qtype, 1, cols);
    } else if (matrix < 6) {
        m = matrix == 3 ? L.shared_gate : (matrix == 4 ? L.shared_up : L.shared_down);
    } else {
        return fail(ctx, error, error_size, "matrix selector %u out of range (0-2 routed gate/up/down, 3-5 shared)", matrix);
    }
    if (path == 0) CU_TRY(ctx, uocr::launch_dequant_probe(m, d_out, ctx->stream, &ctx->launches));
    else if (path == 1) CU_TRY(ctx, uocr::launch_producer_probe(m, d_out, ctx->stream, &ctx->launches));
    else return fail(ctx, error, error_size, "path selector %u out of range (0 matrix-vector kernels, 1 tensor-core producer)", path);
    return 1;
}

static unsigned long long *barrier_counter(uocr_cuda_context *ctx) {
    return reinterpret_cast<unsigned long long *>(reinterpret_cast<uint8_t *>(ctx->status) + 64);
}
// ticket word of the batched decode path's routing kernel: in the context's status block, zero between calls
static uint32_t *batched_ticket(uocr_cuda_context *ctx) {
    return reinterpret_cast<uint32_t *>(reinterpret_cast<uint8_t *>(ctx->status) + 128);
}
static unsigned long long *decode_accumulators(uocr_cuda_context *ctx) {
    return reinterpret_cast<unsigned long long *>(reinterpret_cast<uint8_t *>(ctx->status) + 256);
}

static uocr::GemmScratch gemm_scratch(uocr_cuda_context *ctx, const Scratch &s, const ArenaLayout &a) {
    uocr::GemmScratch g{};
    g.x_sorted = (__half *)(ctx->arena + a.x_sorted);
    g.mid_sorted = s.mid;
    g.down_sorted = (__half *)s.down_out;
    g.shared_mid = s.shared_mid;
    g.shared_out = (__half *)s.shared_out;
    g.tiles_gu = (uint4 *)(ctx->arena + a.tiles_gu); g.tiles_dn = (uint4 *)(ctx->arena + a.tiles_dn);
    g.stiles_gu = (uint4 *)(ctx->arena + a.stiles_gu); g.stiles_dn = (uint4 *)(ctx->arena + a.stiles_dn);
    g.counts = (uint32_t *)(ctx->arena + a.counts);
    return g;
}

// norm_weight: only for a call that takes the single-token decode kernel (the caller checks): the kernel then normalises
// d_hidden itself
static int layer_forward(uocr_cuda_context *ctx, uint32_t layer, const __half *d_hidden, const __half *d_residual,
                         const float *d_injected, uint32_t n, __half *d_out, const uocr_cuda_moe_debug_outputs *dbg,
                         char *error, size_t error_size, const __half *norm_weight = nullptr, float norm_eps = 0.f) {
    const DLayer &L = ctx->layers[layer];
    ArenaLayout a;
    Scratch s = carve(ctx, L, n, &a);
    float *logits = dbg && dbg->d_router_logits ? dbg->d_router_logits : nullptr;
    float *probs = dbg && dbg->d_router_probs ? dbg->d_router_probs : nullptr;
    if (n == 1 && ctx->fused_decode && ctx->sliced_decode && uocr::decode_sliced_supported(ctx->layers.data(), layer, 1)) {
        ProfScope span(ctx, kPfFused, ctx->stream);
        CU_TRY(ctx, uocr::launch_decode_sliced(ctx->layers.data(), ctx->d_layers, layer, 1, d_hidden, d_residual, nullptr, 0,
                                               d_injected, d_out, nullptr, decode_accumulators(ctx), &ctx->acc_base, ctx->status,
                                               logits, probs, s.top_ids, s.top_weights, nullptr, take_decode_knobs(ctx), ctx->stream,
                                               &ctx->launches, norm_weight, norm_eps));
    } else if (n == 1 && ctx->fused_decode && uocr::decode_supported(ctx->layers.data(), layer, 1)) {
        ProfScope span(ctx, kPfFused, ctx->stream);
        CU_TRY(ctx, uocr::launch_decode_stack(ctx->layers.data(), ctx->d_layers, layer, 1, d_hidden, d_residual, 0,
                                              d_injected, d_out, (__half *)(ctx->arena + a.stack0),
                                              (__half *)(ctx->arena + a.stack1), (__half *)(ctx->arena + a.dec_mid),
                                              (float *)(ctx->arena + a.dec_plogits), barrier_counter(ctx), &ctx->bar_base,
                                              ctx->status, logits, probs, s.top_ids, s.top_weights, nullptr, ctx->stream,
                                              &ctx->launches));
    } else if (n >= 2 && ctx->batched_decode && uocr::decode_batched_supported(L, n)) {
        // a few tokens at the model's shapes: routing + plan, ONE weight-streaming kernel for the routed experts and the
        // shared MLP, and the combine
        uint8_t *scratch = ctx->arena + a.bt_routed;
        {
            ProfScope span(ctx, kPfRouter, ctx->stream);
            CU_TRY(ctx, uocr::launch_batched_route(L, s, d_hidden, d_injected, n, logits, probs, scratch, batched_ticket(ctx), ctx->stream,
                                                   &ctx->launches));
        }
        {
            ProfScope span(ctx, kPfRouted, ctx->stream);
            CU_TRY(ctx, uocr::launch_batched_experts(L, s, n, scratch, ctx->stream, &ctx->launches));
        }
        ProfScope span(ctx, kPfCombine, ctx->stream);
        CU_TRY(ctx, uocr::launch_batched_combine(L, s, d_residual, n, scratch, d_out, ctx->stream, &ctx->launches));
    } else if (n >= ctx->gemm_min_tokens && uocr::gemm_path_supported(L)) {
        // The shared MLP needs neither the routing nor the permutation: it runs on a second stream beside the router,
        // the dispatch plan, the gather and the routed experts, whose small kernels leave most SMs idle.
        const uocr::GemmScratch g = gemm_scratch(ctx, s, a);
        CU_TRY(ctx, cudaEventRecord(ctx->fork_event, ctx->stream));
        CU_TRY(ctx, cudaStreamWaitEvent(ctx->side_stream, ctx->fork_event, 0));
        {
            ProfScope span(ctx, kPfPrefillShared, ctx->side_stream);
            CU_TRY(ctx, uocr::launch_gemm_shared(L, s, g, d_hidden, n, ctx->side_stream, &ctx->launches));
        }
        CU_TRY(ctx, cudaEventRecord(ctx->join_event, ctx->side_stream));
        {
            ProfScope span(ctx, kPfPrefillRouter, ctx->stream);
            CU_TRY(ctx, uocr::launch_router(L, d_hidden, d_injected, n, logits, probs, s.top_ids, s.top_weights, ctx->status,
                                            s.logits, ctx->stream, &ctx->launches));
        }
        {
            ProfScope span(ctx, kPfPrefillPlan, ctx->stream);
            CU_TRY(ctx, uocr::launch_dispatch_plan(s.top_ids, n, L.K, L.E, s.expert_offsets, s.pair_rows, s.inverse,
                                                   s.active, s.plan_counts, ctx->stream, &ctx->launches));
            CU_TRY(ctx, uocr::launch_gather_sorted(L, s, d_hidden, n, g.x_sorted, ctx->stream, &ctx->launches));
        }
        {
            ProfScope span(ctx, L.expert_qtype == UOCR_QT_Q4 ? kPfBucketedQ4 : (L.expert_qtype == UOCR_QT_Q8 ? kPfBucketedQ8 : kPfBucketedF16),
                           ctx->stream);
            CU_TRY(ctx, uocr::launch_gemm_experts(L, s, g, s.expert_offsets, L.E, 0, L.E, g.x_sorted, n * L.K, g.mid_sorted,
                                                  g.down_sorted, ctx->stream, &ctx->launches));
        }
        CU_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ctx->join_event, 0));
        ProfScope span(ctx, kPfPrefillCombine, ctx->stream);
        CU_TRY(ctx, uocr::launch_gemm_combine(L, s, g, g.down_sorted, d_residual, n, d_out, ctx->stream, &ctx->launches));
    } else {
        {
            ProfScope span(ctx, kPfRouter, ctx->stream);
            CU_TRY(ctx, uocr::launch_router(L, d_hidden, d_injected, n, logits, probs, s.top_ids, s.top_weights, ctx->status,
                                            s.logits, ctx->stream, &ctx->launches));
            CU_TRY(ctx, uocr::launch_dispatch_plan(s.top_ids, n, L.K, L.E, s.expert_offsets, s.pair_rows, s.inverse,
                                                   s.active, s.plan_counts, ctx->stream, &ctx->launches));
        }
        ProfScope span(ctx, kPfMatvec, ctx->stream);
        CU_TRY(ctx, uocr::launch_small_batch_layer(L, s, d_hidden, d_residual, n, d_out, ctx->stream, &ctx->launches));
    }
    if (dbg && dbg->d_top_ids)
        CU_TRY(ctx, cudaMemcpyAsync(dbg->d_top_ids, s.top_ids, (size_t)n * L.K * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    if (dbg && dbg->d_top_weights)
        CU_TRY(ctx, cudaMemcpyAsync(dbg->d_top_weights, s.top_weights, (size_t)n * L.K * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    return 1;
}

// ---- the steps either side of the MoE layer ------------------------------------------------------------------------
extern "C" int uocr_cuda_rmsnorm(uocr_cuda_context *ctx, const void *d_x, const void *d_weight_f16, float eps, uint32_t n,
                                 uint32_t hidden_size, void *d_out, char *error, size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    if (!d_x || !d_weight_f16 || !d_out || n == 0 || hidden_size == 0 || hidden_size % 8 || !(eps >= 0.0f))
        return fail(ctx, error, error_size, "invalid RMSNorm argument (null pointer, zero size, width not a multiple of 8 or negative eps)");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    CU_TRY(ctx, uocr::launch_rmsnorm((const __half *)d_x, (const __half *)d_weight_f16, n, hidden_size, eps, (__half *)d_out, ctx->stream,
                                     &ctx->launches));
    return 1;
}

extern "C" int uocr_cuda_moe_layer_forward_normed(uocr_cuda_context *ctx, uint32_t layer, const void *d_stream,
                                                  const void *d_norm_weight_f16, float eps, uint32_t n, void *d_out,
                                                  const uocr_cuda_moe_debug_outputs *dbg, char *error, size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if (!d_stream || !d_norm_weight_f16 || !d_out) return fail(ctx, error, error_size, "null argument");
    const DLayer &L = ctx->layers[layer];
    if (n == 1 && ctx->fused_decode && ctx->sliced_decode && uocr::decode_sliced_supported(ctx->layers.data(), layer, 1)) {
        // one token: the decode kernel normalises its input itself (same arithmetic as the norm kernel), one launch
        if (!(eps >= 0.f)) return fail(ctx, error, error_size, "RMSNorm: eps must not be negative");
        CU_TRY(ctx, cudaSetDevice(ctx->device));
        return layer_forward(ctx, layer, (const __half *)d_stream, (const __half *)d_stream, nullptr, 1, (__half *)d_out, dbg, error,
                             error_size, (const __half *)d_norm_weight_f16, eps);
    }
    ArenaLayout a;
    carve(ctx, L, ctx->token_capacity, &a);
    __half *x = (__half *)(ctx->arena + a.d_in);          // the staging rows of the host-buffer calls: free during a device call
    if (!uocr_cuda_rmsnorm(ctx, d_stream, d_norm_weight_f16, eps, n, L.H, x, error, error_size)) return 0;
    return uocr_cuda_moe_layer_forward(ctx, layer, x, d_stream, nullptr, n, d_out, dbg, error, error_size);
}

extern "C" int uocr_cuda_context_map_dense_mlp(uocr_cuda_context *ctx, const uocr_cuda_matrix *gate, const uocr_cuda_matrix *up,
                                               const uocr_cuda_matrix *down, uint32_t token_capacity, uint32_t *out_index,
                                               char *error, size_t error_size) {
    if (!ctx || !gate || !up || !down) return fail(ctx, error, error_size, "null context or matrix");
    const uint32_t S = gate->rows, H = gate->cols;
    if (H == 0 || S == 0 || H % UOCR_GROUP || S % UOCR_GROUP) return fail(ctx, error, error_size, "dense MLP widths must be positive multiples of 64 (hidden %u, intermediate %u)", H, S);
    if (H > 2048 || S > 8192) return fail(ctx, error, error_size, "dense MLP widths above 2048 (hidden) / 8192 (intermediate) are not supported");
    if (token_capacity == 0) return fail(ctx, error, error_size, "token capacity must be positive");
    if (!check_matrix(ctx, *gate, S, H, "dense gate", error, error_size) || !check_matrix(ctx, *up, S, H, "dense up", error, error_size) ||
        !check_matrix(ctx, *down, H, S, "dense down", error, error_size))
        return 0;
    if (gate->qtype != up->qtype) return fail(ctx, error, error_size, "dense gate and up projections must share one qtype");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    uocr_cuda_context::DenseMlp D;
    D.H = H; D.S = S; D.capacity = token_capacity;
    {   // gate and up in one allocation (gate first), as the kernels address "up" as a positive offset from "gate"
        const int q = gate->qtype;
        const uint64_t wb = packed_bytes(q, S, H), sb = q == UOCR_QT_F16 ? 0 : (uint64_t)S * (H / UOCR_GROUP) * 2;
        uint8_t *dw = nullptr, *ds = nullptr;
        CU_TRY(ctx, cudaMalloc(&dw, 2 * wb + kUploadPad));
        ctx->weight_allocs.push_back(dw);
        CU_TRY(ctx, cudaMemcpy(dw, gate->qweight, wb, cudaMemcpyHostToDevice));
        CU_TRY(ctx, cudaMemcpy(dw + wb, up->qweight, wb, cudaMemcpyHostToDevice));
        if (sb) {
            CU_TRY(ctx, cudaMalloc(&ds, 2 * sb + kUploadPad));
            ctx->weight_allocs.push_back(ds);
            CU_TRY(ctx, cudaMemcpy(ds, gate->qscale, sb, cudaMemcpyHostToDevice));
            CU_TRY(ctx, cudaMemcpy(ds + sb, up->qscale, sb, cudaMemcpyHostToDevice));
        }
        ctx->weight_bytes += 2 * (wb + sb);
        const uint32_t rb = (uint32_t)(wb / S);
        D.gate = DMatrix{dw, (const __half *)ds, S, H, rb, q};
        D.up = DMatrix{dw + wb, ds ? (const __half *)(ds + sb) : nullptr, S, H, rb, q};
    }
    {
        const int q = down->qtype;
        const uint64_t wb = packed_bytes(q, H, S), sb = q == UOCR_QT_F16 ? 0 : (uint64_t)H * (S / UOCR_GROUP) * 2;
        void *pw = nullptr, *ps = nullptr;
        if (!upload(ctx, down->qweight, wb, &pw, error, error_size)) return 0;
        if (sb && !upload(ctx, down->qscale, sb, &ps, error, error_size)) return 0;
        D.down = DMatrix{(const uint8_t *)pw, (const __half *)ps, H, S, (uint32_t)(wb / H), q};
    }
    // scratch: normalised input, SwiGLU products, output rows, the two tile lists of the tensor-core path and their counts
    auto up256 = [](uint64_t v) { return (v + 255) & ~(uint64_t)255; };
    const uint64_t token_tiles = (token_capacity + 127) / 128 + 1;
    const uint64_t o_x = 0, o_mid = o_x + up256((uint64_t)token_capacity * H * 2), o_out = o_mid + up256((uint64_t)token_capacity * S * 2),
                   o_tg = o_out + up256((uint64_t)token_capacity * H * 4), o_td = o_tg + up256(token_tiles * (S / 64 + 1) * 16),
                   o_cnt = o_td + up256(token_tiles * (H / 128 + 1) * 16), total = o_cnt + 256;
    uint8_t *base = nullptr;
    CU_TRY(ctx, cudaMalloc(&base, total));
    D.scratch = base; D.scratch_bytes = total;
    D.x_norm = (__half *)(base + o_x); D.mid = (__half *)(base + o_mid); D.out_f32 = (float *)(base + o_out);
    D.tiles_gu = (uint4 *)(base + o_tg); D.tiles_dn = (uint4 *)(base + o_td); D.counts = (uint32_t *)(base + o_cnt);
    // One token: the single-token decode kernel on a slice-major copy of the three matrices (every CTA a 64-column unit)
    if (ctx->fused_decode && ctx->sliced_decode) {
        const uint32_t units = uocr::decode_dense_units(H, S, D.gate.qtype, D.up.qtype, D.down.qtype);
        // every unit is a CTA that waits for the others: only grids no larger than the MoE decode kernel's own (112 CTAs in
        // clusters of four, whose co-residency is verified when the context is created) are launched this way
        constexpr uint32_t kCoResidentCtas = 112;
        if (units != 0 && units <= kCoResidentCtas) {
            const size_t bytes = uocr::decode_dense_units_bytes(D.gate.qtype, units);
            uint8_t *blob = nullptr;
            CU_TRY(ctx, cudaMalloc(&blob, bytes));
            ctx->weight_allocs.push_back(blob);
            CU_TRY(ctx, uocr::build_dense_units(D.gate, D.up, D.down, units, blob, ctx->stream));
            DLayer pseudo{};
            pseudo.H = H; pseudo.S = S; pseudo.expert_qtype = D.gate.qtype; pseudo.dec_units = blob;
            void *dl = nullptr;
            CU_TRY(ctx, cudaMalloc(&dl, sizeof(DLayer)));
            ctx->weight_allocs.push_back(dl);
            CU_TRY(ctx, cudaMemcpyAsync(dl, &pseudo, sizeof(DLayer), cudaMemcpyHostToDevice, ctx->stream));
            CU_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            ctx->weight_bytes += bytes;
            D.units = units; D.d_layer = (DLayer *)dl; D.unit_blobs = blob;
        }
    }
    ctx->dense.push_back(D);
    ctx->dense_scratch_bytes += total;
    if (out_index) *out_index = (uint32_t)ctx->dense.size() - 1;
    track_memory(ctx);
    return 1;
}

static int dense_forward(uocr_cuda_context *ctx, uint32_t index, const __half *d_hidden, const __half *d_residual, uint32_t n,
                         __half *d_out, char *error, size_t error_size, const __half *norm_weight = nullptr, float norm_eps = 0.f) {
    auto &D = ctx->dense[index];
    if (n >= ctx->gemm_min_tokens && D.H % 128 == 0 && uocr::gemm_tensor_maps_ready()) {
        // tensor-core path: the two grouped GEMMs of a shared MLP on all n tokens (one "expert"), fp16 output rows, then
        // the residual add (two roundings, like the shared output of the MoE layer in this regime)
        DLayer L{};
        L.H = D.H; L.S = D.S; L.shared_gate = D.gate; L.shared_up = D.up; L.shared_down = D.down;
        Scratch s{};
        s.status = ctx->status;
        uocr::GemmScratch g{};
        g.shared_mid = D.mid; g.shared_out = (__half *)D.out_f32; g.stiles_gu = D.tiles_gu; g.stiles_dn = D.tiles_dn;
        g.counts = D.counts - 2;                          // the shared MLP's two counters are entries 2 and 3
        CU_TRY(ctx, uocr::launch_gemm_shared(L, s, g, d_hidden, n, ctx->stream, &ctx->launches));
        CU_TRY(ctx, uocr::launch_add_rows((const __half *)D.out_f32, d_residual, (size_t)n * D.H, d_out, ctx->stream, &ctx->launches));
        return 1;
    }
    if (n == 1 && D.units != 0) {
        CU_TRY(ctx, uocr::launch_decode_dense(D.d_layer, D.unit_blobs, D.gate.qtype, D.units, d_hidden, d_residual, d_out, decode_accumulators(ctx),
                                              &ctx->acc_base, ctx->status, take_decode_knobs(ctx), ctx->stream, &ctx->launches, norm_weight,
                                              norm_eps));
        return 1;
    }
    if (!uocr::dense_small_supported(D.H, D.S)) return fail(ctx, error, error_size, "dense MLP shape not supported by the matrix-vector path");
    CU_TRY(ctx, uocr::launch_dense_small(D.gate, D.up, D.down, d_hidden, d_residual, n, D.mid, D.out_f32, d_out, ctx->stream, &ctx->launches));
    return 1;
}

extern "C" int uocr_cuda_dense_mlp_forward(uocr_cuda_context *ctx, uint32_t index, const void *d_hidden, const void *d_residual,
                                           uint32_t n, void *d_out, char *error, size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    if (index >= ctx->dense.size()) return fail(ctx, error, error_size, "dense MLP index %u out of range (%zu mapped)", index, ctx->dense.size());
    if (!d_hidden || !d_out || n == 0) return fail(ctx, error, error_size, "null or empty dense MLP argument");
    if (n > ctx->dense[index].capacity) return fail(ctx, error, error_size, "n_tokens %u exceeds the dense MLP's capacity %u", n, ctx->dense[index].capacity);
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    return dense_forward(ctx, index, (const __half *)d_hidden, (const __half *)d_residual, n, (__half *)d_out, error, error_size);
}

extern "C" int uocr_cuda_dense_mlp_forward_normed(uocr_cuda_context *ctx, uint32_t index, const void *d_stream,
                                                  const void *d_norm_weight_f16, float eps, uint32_t n, void *d_out, char *error,
                                                  size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    if (index >= ctx->dense.size()) return fail(ctx, error, error_size, "dense MLP index %u out of range (%zu mapped)", index, ctx->dense.size());
    if (!d_stream || !d_norm_weight_f16 || !d_out || n == 0) return fail(ctx, error, error_size, "null or empty dense MLP argument");
    auto &D = ctx->dense[index];
    if (n > D.capacity) return fail(ctx, error, error_size, "n_tokens %u exceeds the dense MLP's capacity %u", n, D.capacity);
    if (n == 1 && D.units != 0) {      // one token: the decode kernel normalises its input itself, one launch
        if (!(eps >= 0.f)) return fail(ctx, error, error_size, "RMSNorm: eps must not be negative");
        CU_TRY(ctx, cudaSetDevice(ctx->device));
        return dense_forward(ctx, index, (const __half *)d_stream, (const __half *)d_stream, 1, (__half *)d_out, error, error_size,
                             (const __half *)d_norm_weight_f16, eps);
    }
    if (!uocr_cuda_rmsnorm(ctx, d_stream, d_norm_weight_f16, eps, n, D.H, D.x_norm, error, error_size)) return 0;
    return dense_forward(ctx, index, D.x_norm, (const __half *)d_stream, n, (__half *)d_out, error, error_size);
}

// ---- LM head: fused logits + argmax ----------------------------------------------------------------------------------
extern "C" int uocr_cuda_context_map_lm_head(uocr_cuda_context *ctx, const uocr_cuda_matrix *weight, char *error, size_t error_size) {
    if (!ctx || !weight) return fail(ctx, error, error_size, "null context or matrix");
    if (ctx->lm_head.mapped) return fail(ctx, error, error_size, "an LM head is already mapped; call uocr_cuda_context_unmap_model first");
    const uint32_t V = weight->rows, H = weight->cols;
    if (V == 0 || H == 0 || H % UOCR_GROUP || H > 2048) return fail(ctx, error, error_size, "LM head shape [%u, %u] not supported (hidden: multiple of 64, at most 2048)", V, H);
    if (!check_matrix(ctx, *weight, V, H, "LM head", error, error_size)) return 0;
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    const int q = weight->qtype;
    const uint64_t wb = packed_bytes(q, V, H), sb = q == UOCR_QT_F16 ? 0 : (uint64_t)V * (H / UOCR_GROUP) * 2;
    void *pw = nullptr, *ps = nullptr;
    if (!upload(ctx, weight->qweight, wb, &pw, error, error_size)) return 0;
    if (sb && !upload(ctx, weight->qscale, sb, &ps, error, error_size)) return 0;
    ctx->lm_head.w = DMatrix{(const uint8_t *)pw, (const __half *)ps, V, H, (uint32_t)(wb / V), q};
    int sms = 0;
    CU_TRY(ctx, cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx->device));
    ctx->lm_head.grid = (uint32_t)sms * 8u;                // 8 CTAs of 256 threads per SM: every SM's 64 warp slots stream rows
    const size_t bytes = (size_t)ctx->lm_head.grid * 4 * 8 + 256;
    CU_TRY(ctx, cudaMalloc(&ctx->lm_head.scratch, bytes));
    CU_TRY(ctx, cudaMemset(ctx->lm_head.scratch, 0, bytes));
    ctx->lm_head.mapped = true;
    track_memory(ctx);
    return 1;
}

extern "C" int uocr_cuda_lm_head_argmax(uocr_cuda_context *ctx, const void *d_hidden, uint32_t n, uint32_t *d_token_ids,
                                        float *d_scores, char *error, size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    if (!ctx->lm_head.mapped) return fail(ctx, error, error_size, "no LM head mapped");
    if (!d_hidden || !d_token_ids || n == 0) return fail(ctx, error, error_size, "null or empty LM head argument");
    if (n > uocr::lm_head_max_tokens()) return fail(ctx, error, error_size, "the fused LM head takes at most %u tokens per call", uocr::lm_head_max_tokens());
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    auto &Lm = ctx->lm_head;
    float *part_scores = (float *)Lm.scratch;
    uint32_t *part_ids = (uint32_t *)(part_scores + (size_t)Lm.grid * 4);
    uint32_t *ticket = part_ids + (size_t)Lm.grid * 4;
    CU_TRY(ctx, uocr::launch_lm_head_argmax(Lm.w, (const __half *)d_hidden, n, Lm.grid, part_scores, part_ids, ticket, d_token_ids,
                                            d_scores, ctx->stream, &ctx->launches));
    return 1;
}

extern "C" const char *uocr_cuda_moe_regime_name(const uocr_cuda_context *ctx, uint32_t layer, uint32_t n) {
    if (!ctx || layer >= ctx->layers.size() || n == 0) return "";
    const DLayer &L = ctx->layers[layer];
    if (n == 1 && ctx->fused_decode && ctx->sliced_decode && uocr::decode_sliced_supported(ctx->layers.data(), layer, 1))
        return "single-token decode kernel (decode_sliced_kernel)";
    if (n == 1 && ctx->fused_decode && uocr::decode_supported(ctx->layers.data(), layer, 1))
        return "single-token decode kernel, two-barrier form (decode_stack_kernel)";
    if (n >= 2 && ctx->batched_decode && uocr::decode_batched_supported(L, n))
        return "weight-streaming batched decode kernel (decode_batched_kernel)";
    if (n >= ctx->gemm_min_tokens && uocr::gemm_path_supported(L)) return "grouped GEMM on tensor cores (grouped_gemm_kernel)";
    return "matrix-vector kernels (gate_up_kernel, down_kernel)";
}

extern "C" int uocr_cuda_moe_layer_forward(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden,
                                           const void *d_residual, const float *d_injected, uint32_t n, void *d_out,
                                           const uocr_cuda_moe_debug_outputs *dbg, char *error, size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if (!d_hidden || !d_out) return fail(ctx, error, error_size, "null activation pointer");
    return layer_forward(ctx, layer, (const __half *)d_hidden, (const __half *)d_residual, d_injected, n, (__half *)d_out,
                         dbg, error, error_size);
}

static bool stack_uses_sliced_decode(const uocr_cuda_context *ctx, uint32_t first, uint32_t count, uint32_t n) {
    return n == 1 && ctx->fused_decode && ctx->sliced_decode && uocr::decode_sliced_supported(ctx->layers.data(), first, count);
}

// h_inline / host_status: only with the sliced decode kernel (see launch_decode_sliced); null otherwise
static int stack_forward(uocr_cuda_context *ctx, uint32_t first, uint32_t count, const __half *d_hidden, uint32_t n,
                         __half *d_out, char *error, size_t error_size, const void *h_inline = nullptr,
                         uint32_t *host_status = nullptr) {
    ArenaLayout a;
    Scratch s = carve(ctx, ctx->layers[first], n, &a);
    __half *buf[2] = {(__half *)(ctx->arena + a.stack0), (__half *)(ctx->arena + a.stack1)};
    if (stack_uses_sliced_decode(ctx, first, count, n)) {
        ProfScope span(ctx, kPfFused, ctx->stream);
        CU_TRY(ctx, uocr::launch_decode_sliced(ctx->layers.data(), ctx->d_layers, first, count, d_hidden, d_hidden, h_inline, 1,
                                               nullptr, d_out, host_status, decode_accumulators(ctx), &ctx->acc_base, ctx->status, nullptr,
                                               nullptr, s.top_ids, s.top_weights, ctx->decode_trace, take_decode_knobs(ctx), ctx->stream,
                                               &ctx->launches));
        return 1;
    }
    if (n == 1 && ctx->fused_decode && uocr::decode_supported(ctx->layers.data(), first, count)) {
        CU_TRY(ctx, uocr::launch_decode_stack(ctx->layers.data(), ctx->d_layers, first, count, d_hidden, d_hidden, 1,
                                              nullptr, d_out, buf[0], buf[1], (__half *)(ctx->arena + a.dec_mid),
                                              (float *)(ctx->arena + a.dec_plogits), barrier_counter(ctx), &ctx->bar_base,
                                              ctx->status, nullptr, nullptr, s.top_ids, s.top_weights, ctx->decode_trace, ctx->stream,
                                              &ctx->launches));
        return 1;
    }
    const __half *cur = d_hidden;
    for (uint32_t i = 0; i < count; ++i) {
        __half *dst = (i + 1 == count) ? d_out : buf[i & 1];
        if (!layer_forward(ctx, first + i, cur, cur, nullptr, n, dst, nullptr, error, error_size)) return 0;
        cur = dst;
    }
    return 1;
}

extern "C" int uocr_cuda_moe_stack_forward(uocr_cuda_context *ctx, uint32_t first, uint32_t count, const void *d_hidden,
                                           uint32_t n, void *d_out, char *error, size_t error_size) {
    if (!check_call(ctx, first, n, error, error_size)) return 0;
    if (count == 0 || first + count > ctx->layers.size()) return fail(ctx, error, error_size, "layer range [%u, %u) out of range", first, first + count);
    if (!d_hidden || !d_out) return fail(ctx, error, error_size, "null activation pointer");
    for (uint32_t i = 1; i < count; ++i) {
        const DLayer &A = ctx->layers[first], &B = ctx->layers[first + i];
        if (A.H != B.H || A.E != B.E || A.K != B.K || A.F != B.F || A.S != B.S)
            return fail(ctx, error, error_size, "stacked layers must have identical dimensions");
    }
    return stack_forward(ctx, first, count, (const __half *)d_hidden, n, (__half *)d_out, error, error_size);
}

extern "C" int uocr_cuda_moe_layer_forward_host(uocr_cuda_context *ctx, uint32_t layer, const void *h_hidden,
                                                const void *h_residual, uint32_t n, void *h_out, uint32_t *h_ids,
                                                float *h_wts, char *error, size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if (!h_hidden || !h_out) return fail(ctx, error, error_size, "null activation pointer");
    const DLayer &L = ctx->layers[layer];
    ArenaLayout a;
    Scratch s = carve(ctx, L, n, &a);
    const size_t act = (size_t)n * L.H * 2;
    __half *d_in = (__half *)(ctx->arena + a.d_in), *d_res = (__half *)(ctx->arena + a.d_res),
           *d_out = (__half *)(ctx->arena + a.d_out);
    memcpy(ctx->h_in, h_hidden, act);
    CU_TRY(ctx, cudaMemcpyAsync(d_in, ctx->h_in, act, cudaMemcpyHostToDevice, ctx->stream));
    if (h_residual) {
        memcpy(ctx->h_res, h_residual, act);
        CU_TRY(ctx, cudaMemcpyAsync(d_res, ctx->h_res, act, cudaMemcpyHostToDevice, ctx->stream));
    }
    if (!layer_forward(ctx, layer, d_in, h_residual ? d_res : nullptr, nullptr, n, d_out, nullptr, error, error_size)) return 0;
    CU_TRY(ctx, cudaMemcpyAsync(ctx->h_out, d_out, act, cudaMemcpyDeviceToHost, ctx->stream));
    if (h_ids) CU_TRY(ctx, cudaMemcpyAsync(ctx->h_ids, s.top_ids, (size_t)n * L.K * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (h_wts) CU_TRY(ctx, cudaMemcpyAsync(ctx->h_wts, s.top_weights, (size_t)n * L.K * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (!uocr_cuda_context_synchronize(ctx, error, error_size)) return 0;
    memcpy(h_out, ctx->h_out, act);
    if (h_ids) memcpy(h_ids, ctx->h_ids, (size_t)n * L.K * 4);
    if (h_wts) memcpy(h_wts, ctx->h_wts, (size_t)n * L.K * 4);
    return 1;
}

extern "C" int uocr_cuda_moe_stack_forward_host(uocr_cuda_context *ctx, uint32_t first, uint32_t count,
                                                const void *h_hidden, uint32_t n, void *h_out, char *error,
                                                size_t error_size) {
    if (!check_call(ctx, first, n, error, error_size)) return 0;
    if (count == 0 || first + count > ctx->layers.size()) return fail(ctx, error, error_size, "layer range [%u, %u) out of range", first, first + count);
    if (!h_hidden || !h_out) return fail(ctx, error, error_size, "null activation pointer");
    const DLayer &L = ctx->layers[first];
    ArenaLayout a;
    carve(ctx, L, n, &a);
    const size_t act = (size_t)n * L.H * 2;
    __half *d_in = (__half *)(ctx->arena + a.d_in), *d_out = (__half *)(ctx->arena + a.d_out);
    if (ctx->h_out_dev && ctx->h_status_dev && stack_uses_sliced_decode(ctx, first, count, n)) {
        // one token through the decode kernel: the activations ride in the launch parameters, and the kernel writes
        // the result and its status word straight into mapped host memory, so the call issues no copy at all
        *ctx->h_status = 0xffffffffu;
        if (!stack_forward(ctx, first, count, d_in, n, ctx->h_out_dev, error, error_size, h_hidden, ctx->h_status_dev)) return 0;
        // The kernel writes the status word last, after the result (system-scope fence in between): the host polls it for
        // up to a millisecond instead of sleeping in the driver, whose wake-up costs several microseconds of a 90 us
        // step, and falls back to the stream wait (always taken when events have to be read back for the profile).
        if (ctx->profile == nullptr) {
            const auto t0 = std::chrono::steady_clock::now();
            while (*(volatile uint32_t *)ctx->h_status == 0xffffffffu) {
                if (std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(1)) break;
                cpu_relax();
            }
        }
        if (*(volatile uint32_t *)ctx->h_status == 0xffffffffu) CU_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        prof_flush(ctx);
        if (*(volatile uint32_t *)ctx->h_status != 0) {       // the kernel gave up, or flagged something: read the device word
            if (!uocr_cuda_context_synchronize(ctx, error, error_size)) return 0;
            return fail(ctx, error, error_size, "the decode kernel ended without writing its result");
        }
        memcpy(h_out, ctx->h_out, act);
        return 1;
    }
    memcpy(ctx->h_in, h_hidden, act);
    CU_TRY(ctx, cudaMemcpyAsync(d_in, ctx->h_in, act, cudaMemcpyHostToDevice, ctx->stream));
    if (!uocr_cuda_moe_stack_forward(ctx, first, count, d_in, n, d_out, error, error_size)) return 0;
    CU_TRY(ctx, cudaMemcpyAsync(ctx->h_out, d_out, act, cudaMemcpyDeviceToHost, ctx->stream));
    if (!uocr_cuda_context_synchronize(ctx, error, error_size)) return 0;
    memcpy(h_out, ctx->h_out, act);
    return 1;
}

// ------------------------------------------------------------------ expert-parallel phases
// The many-token layer cut at its two exchange points, so that a host that shards the experts over several
// GPUs can put an all-to-all between the phases.  With one GPU the three calls in a row are the layer.
// Scratch is carved for the context's whole token capacity: a rank may receive more rows than it sends.

extern "C" int uocr_cuda_moe_ep_dispatch(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden, uint32_t n,
                                         void *d_sorted_rows, uint32_t *d_expert_offsets, char *error, size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if (!d_hidden || !d_sorted_rows || !d_expert_offsets) return fail(ctx, error, error_size, "null expert-parallel dispatch argument");
    const DLayer &L = ctx->layers[layer];
    if (!uocr::gemm_path_supported(L)) return fail(ctx, error, error_size, "layer shape not supported by the tensor-core path");
    ArenaLayout a;
    Scratch s = carve(ctx, L, ctx->token_capacity, &a);
    CU_TRY(ctx, uocr::launch_router(L, (const __half *)d_hidden, nullptr, n, nullptr, nullptr, s.top_ids, s.top_weights,
                                    ctx->status, s.logits, ctx->stream, &ctx->launches));
    CU_TRY(ctx, uocr::launch_dispatch_plan(s.top_ids, n, L.K, L.E, s.expert_offsets, s.pair_rows, s.inverse, s.active,
                                           s.plan_counts, ctx->stream, &ctx->launches));
    CU_TRY(ctx, uocr::launch_gather_sorted(L, s, (const __half *)d_hidden, n, (__half *)d_sorted_rows, ctx->stream, &ctx->launches));
    CU_TRY(ctx, cudaMemcpyAsync(d_expert_offsets, s.expert_offsets, (size_t)(L.E + 1) * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    return 1;
}

extern "C" int uocr_cuda_moe_ep_experts(uocr_cuda_context *ctx, uint32_t layer, uint32_t first_expert, uint32_t n_local_experts,
                                        uint32_t n_sources, const uint32_t *h_segment_counts, const void *d_rows_in,
                                        void *d_rows_out, char *error, size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    if (layer >= ctx->layers.size()) return fail(ctx, error, error_size, "layer index %u out of range", layer);
    const DLayer &L = ctx->layers[layer];
    const uint32_t n_seg = n_local_experts * n_sources;
    if (!uocr::gemm_path_supported(L)) return fail(ctx, error, error_size, "layer shape not supported by the tensor-core path");
    if (!h_segment_counts || !d_rows_in || !d_rows_out) return fail(ctx, error, error_size, "null expert-parallel argument");
    if (n_local_experts == 0 || n_sources == 0 || first_expert + n_local_experts > L.E || n_seg > 256)
        return fail(ctx, error, error_size, "invalid expert range or segment count");
    if (!ctx->arena) return fail(ctx, error, error_size, "arenas not allocated");
    ArenaLayout a;
    Scratch s = carve(ctx, L, ctx->token_capacity, &a);
    // segment offsets: host prefix sum through a pinned staging slot (a ring of slots, each guarded by the event of
    // the copy that last read it, so the call never has to wait for the stream)
    const uint32_t slot = ctx->seg_slot++ % kSegSlots;
    uint32_t *h_seg = ctx->h_seg + (size_t)slot * 260;
    CU_TRY(ctx, cudaEventSynchronize(ctx->seg_events[slot]));
    uint64_t run = 0;
    for (uint32_t i = 0; i < n_seg; ++i) { h_seg[i] = (uint32_t)run; run += h_segment_counts[i]; }
    h_seg[n_seg] = (uint32_t)run;
    if (run > (uint64_t)ctx->token_capacity * L.K)
        return fail(ctx, error, error_size, "%llu received rows exceed the arena capacity of %llu rows (token_capacity * top_k)",
                    (unsigned long long)run, (unsigned long long)ctx->token_capacity * L.K);
    if (run == 0) return 1;
    // (its own array: the plan of this rank's tokens in s.expert_offsets is still needed by a peer-memory combine)
    uint32_t *d_seg = (uint32_t *)(ctx->arena + a.seg_offsets);
    CU_TRY(ctx, cudaMemcpyAsync(d_seg, h_seg, (size_t)(n_seg + 1) * 4, cudaMemcpyHostToDevice, ctx->stream));
    CU_TRY(ctx, cudaEventRecord(ctx->seg_events[slot], ctx->stream));
    const uocr::GemmScratch g = gemm_scratch(ctx, s, a);
    CU_TRY(ctx, uocr::launch_gemm_experts(L, s, g, d_seg, n_seg, first_expert, n_local_experts,
                                          (const __half *)d_rows_in, (uint32_t)run, g.mid_sorted, (__half *)d_rows_out,
                                          ctx->stream, &ctx->launches));
    return 1;
}

extern "C" int uocr_cuda_moe_ep_shared(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden, uint32_t n, char *error,
                                       size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if (!d_hidden) return fail(ctx, error, error_size, "null activation pointer");
    const DLayer &L = ctx->layers[layer];
    if (!uocr::gemm_path_supported(L)) return fail(ctx, error, error_size, "layer shape not supported by the tensor-core path");
    ArenaLayout a;
    Scratch s = carve(ctx, L, ctx->token_capacity, &a);
    const uocr::GemmScratch g = gemm_scratch(ctx, s, a);
    // on the second stream, beside whatever the caller queues next (exchange, routed experts); the combine joins it
    CU_TRY(ctx, cudaEventRecord(ctx->fork_event, ctx->stream));
    CU_TRY(ctx, cudaStreamWaitEvent(ctx->side_stream, ctx->fork_event, 0));
    CU_TRY(ctx, uocr::launch_gemm_shared(L, s, g, (const __half *)d_hidden, n, ctx->side_stream, &ctx->launches));
    CU_TRY(ctx, cudaEventRecord(ctx->join_event, ctx->side_stream));
    ctx->shared_pending = true;
    return 1;
}

static int join_shared(uocr_cuda_context *ctx, char *error, size_t error_size) {
    if (ctx->shared_pending) {
        CU_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ctx->join_event, 0));
        ctx->shared_pending = false;
    }
    return 1;
}

extern "C" int uocr_cuda_moe_ep_combine(uocr_cuda_context *ctx, uint32_t layer, const void *d_rows_back,
                                        const void *d_residual, uint32_t n, void *d_out, char *error, size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if (!d_rows_back || !d_out) return fail(ctx, error, error_size, "null expert-parallel combine argument");
    const DLayer &L = ctx->layers[layer];
    ArenaLayout a;
    Scratch s = carve(ctx, L, ctx->token_capacity, &a);
    const uocr::GemmScratch g = gemm_scratch(ctx, s, a);
    if (!join_shared(ctx, error, error_size)) return 0;
    CU_TRY(ctx, uocr::launch_gemm_combine(L, s, g, (const __half *)d_rows_back, (const __half *)d_residual, n,
                                          (__half *)d_out, ctx->stream, &ctx->launches));
    return 1;
}

// ------------------------------------------------------------ expert parallelism over peer memory
// The exchange fused into the gather and the combine: see scatter_rows_peer_kernel / combine_peer_kernel.

extern "C" void uocr_cuda_moe_ep_peer_destroy(uocr_cuda_context *ctx) {
    if (!ctx) return;
    auto &P = ctx->peer;
    if (P.opened) {
        for (uint32_t g = 0; g < P.world; ++g) {
            if (g == P.rank) continue;
            if (P.recv_all.p[g]) cudaIpcCloseMemHandle(P.recv_all.p[g]);
            if (P.done_all.p[g]) cudaIpcCloseMemHandle(P.done_all.p[g]);
        }
    }
    cudaFree(P.recv); cudaFree(P.done); cudaFree(P.d_dst_row0);
    P = {};
}

extern "C" int uocr_cuda_moe_ep_peer_create(uocr_cuda_context *ctx, uint32_t hidden_size, uint64_t row_capacity,
                                            void *handles_out, char *error, size_t error_size) {
    if (!ctx || !handles_out) return fail(ctx, error, error_size, "null argument");
    if (hidden_size == 0 || hidden_size % 8 || row_capacity == 0) return fail(ctx, error, error_size, "invalid exchange buffer shape");
    uocr_cuda_moe_ep_peer_destroy(ctx);
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    auto &P = ctx->peer;
    const size_t bytes = (size_t)row_capacity * hidden_size * 2;
    // the synchronisation region shares the allocation (and so the IPC handle) of the received rows
    const size_t sync_off = (bytes + 255) & ~(size_t)255;
    CU_TRY(ctx, cudaMalloc(&P.recv, sync_off + uocr::kSyncBytes));
    CU_TRY(ctx, cudaMemset((uint8_t *)P.recv + sync_off, 0, uocr::kSyncBytes));
    CU_TRY(ctx, cudaMalloc(&P.done, bytes));
    CU_TRY(ctx, cudaMalloc(&P.d_dst_row0, 256 * sizeof(uint32_t)));
    P.hidden = hidden_size; P.row_capacity = row_capacity;
    cudaIpcMemHandle_t h[2];
    CU_TRY(ctx, cudaIpcGetMemHandle(&h[0], P.recv));
    CU_TRY(ctx, cudaIpcGetMemHandle(&h[1], P.done));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
    memcpy(handles_out, h, sizeof h);
    return 1;
}

extern "C" int uocr_cuda_moe_ep_peer_open(uocr_cuda_context *ctx, uint32_t world, uint32_t rank, const void *all_handles,
                                          char *error, size_t error_size) {
    if (!ctx || !all_handles) return fail(ctx, error, error_size, "null argument");
    auto &P = ctx->peer;
    if (!P.recv) return fail(ctx, error, error_size, "create the exchange buffers first");
    if (P.opened) return fail(ctx, error, error_size, "exchange already opened");
    if (world == 0 || world > (uint32_t)uocr::kMaxPeers || rank >= world) return fail(ctx, error, error_size, "invalid group: rank %u of %u (at most %d ranks)", rank, world, uocr::kMaxPeers);
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    const cudaIpcMemHandle_t *h = (const cudaIpcMemHandle_t *)all_handles;
    P.world = world; P.rank = rank;
    for (uint32_t g = 0; g < world; ++g) {
        if (g == rank) { P.recv_all.p[g] = P.recv; P.done_all.p[g] = P.done; continue; }
        void *a = nullptr, *b = nullptr;
        CU_TRY(ctx, cudaIpcOpenMemHandle(&a, h[2 * g], cudaIpcMemLazyEnablePeerAccess));
        P.recv_all.p[g] = (__half *)a;
        P.opened = true;
        CU_TRY(ctx, cudaIpcOpenMemHandle(&b, h[2 * g + 1], cudaIpcMemLazyEnablePeerAccess));
        P.done_all.p[g] = (__half *)b;
    }
    const size_t sync_off = ((size_t)P.row_capacity * P.hidden * 2 + 255) & ~(size_t)255;
    for (uint32_t g = 0; g < world; ++g) P.sync.p[g] = (uint32_t *)((uint8_t *)P.recv_all.p[g] + sync_off);
    P.opened = true;
    return 1;
}

static int peer_ready(uocr_cuda_context *ctx, const DLayer &L, char *error, size_t error_size) {
    const auto &P = ctx->peer;
    if (!P.opened) return fail(ctx, error, error_size, "peer exchange not opened");
    if (P.hidden != L.H) return fail(ctx, error, error_size, "exchange buffers were created for hidden size %u, the layer has %u", P.hidden, L.H);
    if (L.E % P.world) return fail(ctx, error, error_size, "%u experts do not divide over %u ranks", L.E, P.world);
    return 1;
}

extern "C" int uocr_cuda_moe_ep_peer_dispatch(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden, uint32_t n,
                                              uint32_t *d_expert_offsets, char *error, size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if (!d_hidden || !d_expert_offsets) return fail(ctx, error, error_size, "null expert-parallel dispatch argument");
    const DLayer &L = ctx->layers[layer];
    if (!uocr::gemm_path_supported(L)) return fail(ctx, error, error_size, "layer shape not supported by the tensor-core path");
    if (!peer_ready(ctx, L, error, error_size)) return 0;
    ArenaLayout a;
    Scratch s = carve(ctx, L, ctx->token_capacity, &a);
    CU_TRY(ctx, uocr::launch_router(L, (const __half *)d_hidden, nullptr, n, nullptr, nullptr, s.top_ids, s.top_weights,
                                    ctx->status, s.logits, ctx->stream, &ctx->launches));
    CU_TRY(ctx, uocr::launch_dispatch_plan(s.top_ids, n, L.K, L.E, s.expert_offsets, s.pair_rows, s.inverse, s.active,
                                           s.plan_counts, ctx->stream, &ctx->launches));
    CU_TRY(ctx, cudaMemcpyAsync(d_expert_offsets, s.expert_offsets, (size_t)(L.E + 1) * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    return 1;
}

extern "C" int uocr_cuda_moe_ep_peer_scatter(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden, uint32_t n,
                                             const uint32_t *h_dst_row0, char *error, size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if (!d_hidden || !h_dst_row0) return fail(ctx, error, error_size, "null expert-parallel scatter argument");
    const DLayer &L = ctx->layers[layer];
    if (!peer_ready(ctx, L, error, error_size)) return 0;
    auto &P = ctx->peer;
    ArenaLayout a;
    Scratch s = carve(ctx, L, ctx->token_capacity, &a);
    const uint32_t slot = ctx->seg_slot++ % kSegSlots;
    uint32_t *h_stage = ctx->h_seg + (size_t)slot * 260;
    CU_TRY(ctx, cudaEventSynchronize(ctx->seg_events[slot]));
    memcpy(h_stage, h_dst_row0, (size_t)L.E * 4);
    CU_TRY(ctx, cudaMemcpyAsync(P.d_dst_row0, h_stage, (size_t)L.E * 4, cudaMemcpyHostToDevice, ctx->stream));
    CU_TRY(ctx, cudaEventRecord(ctx->seg_events[slot], ctx->stream));
    CU_TRY(ctx, uocr::launch_scatter_peer(L, s, (const __half *)d_hidden, n, L.E / P.world, P.d_dst_row0, P.recv_all,
                                          P.row_capacity, ctx->stream, &ctx->launches));
    return 1;
}

extern "C" int uocr_cuda_moe_ep_experts(uocr_cuda_context *ctx, uint32_t layer, uint32_t first_expert, uint32_t n_local_experts,
                                        uint32_t n_sources, const uint32_t *h_segment_counts, const void *d_rows_in,
                                        void *d_rows_out, char *error, size_t error_size);

extern "C" int uocr_cuda_moe_ep_peer_experts(uocr_cuda_context *ctx, uint32_t layer, uint32_t n_sources,
                                             const uint32_t *h_segment_counts, char *error, size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    if (layer >= ctx->layers.size()) return fail(ctx, error, error_size, "layer index %u out of range", layer);
    const DLayer &L = ctx->layers[layer];
    if (!peer_ready(ctx, L, error, error_size)) return 0;
    auto &P = ctx->peer;
    if (n_sources != P.world || !h_segment_counts) return fail(ctx, error, error_size, "segment counts of all %u ranks are needed", P.world);
    const uint32_t per = L.E / P.world;
    uint64_t rows = 0;
    for (uint32_t i = 0; i < n_sources * per; ++i) rows += h_segment_counts[i];
    if (rows > P.row_capacity) return fail(ctx, error, error_size, "%llu received rows exceed the exchange buffers' %llu rows", (unsigned long long)rows, (unsigned long long)P.row_capacity);
    return uocr_cuda_moe_ep_experts(ctx, layer, P.rank * per, per, n_sources, h_segment_counts, P.recv, P.done, error, error_size);
}

// The same two phases with the counts left on the device: d_all_offsets [world][E + 1] holds every rank's expert offsets
// (one all_gather of what the dispatch call wrote).  Nothing is copied to or from the host between the phases.
extern "C" int uocr_cuda_moe_ep_peer_scatter_dev(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden, uint32_t n,
                                                 const uint32_t *d_all_offsets, char *error, size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if (!d_hidden || !d_all_offsets) return fail(ctx, error, error_size, "null expert-parallel scatter argument");
    const DLayer &L = ctx->layers[layer];
    if (!peer_ready(ctx, L, error, error_size)) return 0;
    auto &P = ctx->peer;
    ArenaLayout a;
    Scratch s = carve(ctx, L, ctx->token_capacity, &a);
    const unsigned long long cap_rows = (unsigned long long)ctx->token_capacity * L.K;
    CU_TRY(ctx, uocr::launch_ep_offsets(d_all_offsets, P.world, P.rank, L.E, P.row_capacity < cap_rows ? P.row_capacity : cap_rows,
                                        P.d_dst_row0, (uint32_t *)(ctx->arena + a.seg_offsets), ctx->status, ctx->stream, &ctx->launches));
    CU_TRY(ctx, uocr::launch_scatter_peer(L, s, (const __half *)d_hidden, n, L.E / P.world, P.d_dst_row0, P.recv_all,
                                          P.row_capacity, ctx->stream, &ctx->launches));
    return 1;
}

extern "C" int uocr_cuda_moe_ep_peer_experts_dev(uocr_cuda_context *ctx, uint32_t layer, char *error, size_t error_size) {
    if (!ctx) return fail(nullptr, error, error_size, "null context");
    if (layer >= ctx->layers.size()) return fail(ctx, error, error_size, "layer index %u out of range", layer);
    const DLayer &L = ctx->layers[layer];
    if (!uocr::gemm_path_supported(L)) return fail(ctx, error, error_size, "layer shape not supported by the tensor-core path");
    if (!peer_ready(ctx, L, error, error_size)) return 0;
    if (!ctx->arena) return fail(ctx, error, error_size, "arenas not allocated");
    auto &P = ctx->peer;
    ArenaLayout a;
    Scratch s = carve(ctx, L, ctx->token_capacity, &a);
    const uocr::GemmScratch g = gemm_scratch(ctx, s, a);
    const uint32_t per = L.E / P.world;
    const unsigned long long cap_rows = (unsigned long long)ctx->token_capacity * L.K;
    const uint32_t bound = (uint32_t)(P.row_capacity < cap_rows ? P.row_capacity : cap_rows);      // rows this rank can hold
    CU_TRY(ctx, uocr::launch_gemm_experts(L, s, g, (const uint32_t *)(ctx->arena + a.seg_offsets), P.world * per, P.rank * per, per,
                                          P.recv, bound, g.mid_sorted, P.done, ctx->stream, &ctx->launches));
    return 1;
}

// One whole expert-parallel layer call with the ranks synchronised on the device: dispatch, count exchange, scatter,
// "rows landed", experts, "outputs written", combine.  No host library call and no host read in between; every rank of the
// group must issue the call (the flags carry the call's number).
extern "C" int uocr_cuda_moe_ep_peer_forward(uocr_cuda_context *ctx, uint32_t layer, const void *d_hidden, const void *d_residual,
                                             uint32_t n, void *d_out, char *error, size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if (!d_hidden || !d_out) return fail(ctx, error, error_size, "null expert-parallel layer argument");
    const DLayer &L = ctx->layers[layer];
    if (!uocr::gemm_path_supported(L)) return fail(ctx, error, error_size, "layer shape not supported by the tensor-core path");
    if (!peer_ready(ctx, L, error, error_size)) return 0;
    auto &P = ctx->peer;
    ArenaLayout a;
    Scratch s = carve(ctx, L, ctx->token_capacity, &a);
    const uocr::GemmScratch g = gemm_scratch(ctx, s, a);
    const uint32_t per = L.E / P.world, call = ++P.call;
    const unsigned long long cap_rows = (unsigned long long)ctx->token_capacity * L.K;
    const unsigned long long bound = P.row_capacity < cap_rows ? P.row_capacity : cap_rows;       // rows this rank can hold
    uint32_t *seg_offsets = (uint32_t *)(ctx->arena + a.seg_offsets);
    if (!uocr_cuda_moe_ep_shared(ctx, layer, d_hidden, n, error, error_size)) return 0;      // second stream, beside all that follows
    CU_TRY(ctx, uocr::launch_router(L, (const __half *)d_hidden, nullptr, n, nullptr, nullptr, s.top_ids, s.top_weights,
                                    ctx->status, s.logits, ctx->stream, &ctx->launches));
    CU_TRY(ctx, uocr::launch_dispatch_plan(s.top_ids, n, L.K, L.E, s.expert_offsets, s.pair_rows, s.inverse, s.active,
                                           s.plan_counts, ctx->stream, &ctx->launches));
    CU_TRY(ctx, uocr::launch_ep_exchange_counts(s.expert_offsets, P.sync, P.world, P.rank, L.E, call, bound, P.d_dst_row0,
                                                seg_offsets, ctx->status, ctx->stream, &ctx->launches));
    CU_TRY(ctx, uocr::launch_scatter_peer(L, s, (const __half *)d_hidden, n, per, P.d_dst_row0, P.recv_all, P.row_capacity,
                                          ctx->stream, &ctx->launches));
    CU_TRY(ctx, uocr::launch_ep_signal_wait(P.sync, P.world, P.rank, 1, call, ctx->status, ctx->stream, &ctx->launches));
    CU_TRY(ctx, uocr::launch_gemm_experts(L, s, g, seg_offsets, P.world * per, P.rank * per, per, P.recv, (uint32_t)bound,
                                          g.mid_sorted, P.done, ctx->stream, &ctx->launches));
    CU_TRY(ctx, uocr::launch_ep_signal_wait(P.sync, P.world, P.rank, 2, call, ctx->status, ctx->stream, &ctx->launches));
    if (!join_shared(ctx, error, error_size)) return 0;
    CU_TRY(ctx, uocr::launch_combine_peer(L, s, g, P.done_all, per, P.d_dst_row0, P.row_capacity, (const __half *)d_residual, n,
                                          (__half *)d_out, ctx->stream, &ctx->launches));
    return 1;
}

// Every rank's expert offsets of the last uocr_cuda_moe_ep_peer_forward call, [world][E + 1], read back from this rank's
// synchronisation region (waits for the context's stream; for load statistics, not for the call path).
extern "C" int uocr_cuda_moe_ep_peer_last_offsets(uocr_cuda_context *ctx, uint32_t n_experts, uint32_t *h_all_offsets,
                                                  char *error, size_t error_size) {
    if (!ctx || !h_all_offsets) return fail(ctx, error, error_size, "null argument");
    auto &P = ctx->peer;
    if (!P.opened) return fail(ctx, error, error_size, "peer exchange not opened");
    if (n_experts == 0 || n_experts > 256) return fail(ctx, error, error_size, "invalid expert count %u", n_experts);
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    CU_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    CU_TRY(ctx, cudaMemcpy2D(h_all_offsets, (size_t)(n_experts + 1) * 4, P.sync.p[P.rank], (size_t)uocr::kSyncStride * 4,
                             (size_t)(n_experts + 1) * 4, P.world, cudaMemcpyDeviceToHost));
    return 1;
}

extern "C" int uocr_cuda_moe_ep_peer_combine(uocr_cuda_context *ctx, uint32_t layer, const void *d_residual, uint32_t n,
                                             void *d_out, char *error, size_t error_size) {
    if (!check_call(ctx, layer, n, error, error_size)) return 0;
    if (!d_out) return fail(ctx, error, error_size, "null expert-parallel combine argument");
    const DLayer &L = ctx->layers[layer];
    if (!peer_ready(ctx, L, error, error_size)) return 0;
    auto &P = ctx->peer;
    ArenaLayout a;
    Scratch s = carve(ctx, L, ctx->token_capacity, &a);
    const uocr::GemmScratch g = gemm_scratch(ctx, s, a);
    if (!join_shared(ctx, error, error_size)) return 0;
    CU_TRY(ctx, uocr::launch_combine_peer(L, s, g, P.done_all, L.E / P.world, P.d_dst_row0, P.row_capacity,
                                          (const __half *)d_residual, n, (__half *)d_out, ctx->stream, &ctx->launches));
    return 1;
}

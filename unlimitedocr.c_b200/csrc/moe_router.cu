// Router and dispatch-plan kernels.
//
// Router: per token, logits over the experts (fp16 inputs, f32 accumulation), f32 softmax with the
// host C library's expf bits, serial f32 denominator in expert order, IEEE division, and greedy
// top-k with ties to the lower expert id - the arithmetic of uocr_cpu_ref_moe_router_f32
// (src/backend/cpu_ref/uocr_cpu_ref.c:388-466), so identical logits give identical ids and weights.
//
// Dispatch plan: stable counting sort of pair = token*K + slot by expert id.
#include <mutex>

#include "moe_route.cuh"

namespace uocr {

__constant__ uint64_t c_exp_tab[UOCR_EXPF_N];

// Per-device, set up once; contexts may be created from several threads at the same time.
static std::mutex g_tab_mutex;
static bool g_tab_ready[64] = {false};

static cudaError_t ensure_exp_table() {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    std::lock_guard<std::mutex> lock(g_tab_mutex);
    if (dev >= 0 && dev < 64 && g_tab_ready[dev]) return cudaSuccess;
    uint64_t tab[UOCR_EXPF_N];
    uocr_expf_table_init(tab);
    err = cudaMemcpyToSymbol(c_exp_tab, tab, sizeof tab);
    if (err == cudaSuccess && dev >= 0 && dev < 64) g_tab_ready[dev] = true;
    return err;
}

constexpr int kRouterThreads = 256;
constexpr int kRouterWarps = kRouterThreads / 32;

// TPB tokens per block.  Shared memory: x[TPB][H] f32, logits[TPB][E] f32, probs[TPB][E] f32.
template <int TPB>
__global__ void __launch_bounds__(kRouterThreads)
router_kernel(const __half *__restrict__ hidden, const __half *__restrict__ router, const float *__restrict__ bias,
              const float *__restrict__ injected, uint32_t n, uint32_t H, uint32_t E, uint32_t K, float scaling,
              float *__restrict__ logits_out, float *__restrict__ probs_out, uint32_t *__restrict__ ids_out,
              float *__restrict__ weights_out, uint32_t *__restrict__ status) {
    extern __shared__ float smem[];
    float *xs = smem;                         // [TPB][H]
    float *ls = xs + (size_t)TPB * H;         // [TPB][E]
    float *ps = ls + (size_t)TPB * E;         // [TPB][E]
    __shared__ uint64_t s_tab[UOCR_EXPF_N];
    if (threadIdx.x < UOCR_EXPF_N) s_tab[threadIdx.x] = c_exp_tab[threadIdx.x];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t t0 = blockIdx.x * TPB;
    const uint32_t nt = min((uint32_t)TPB, n - t0);

    if (injected == nullptr) {
        for (uint32_t i = tid; i < TPB * H; i += kRouterThreads) {
            const uint32_t t = i / H;
            xs[i] = t < nt ? __half2float(hidden[(size_t)(t0 + t) * H + (i - t * H)]) : 0.f;
        }
        __syncthreads();
        for (uint32_t e = warp; e < E; e += kRouterWarps) {
            float acc[TPB];
#pragma unroll
            for (int m = 0; m < TPB; ++m) acc[m] = 0.f;
            row_dot<UOCR_QT_F16, TPB>(reinterpret_cast<const uint8_t *>(router + (size_t)e * H), nullptr, H, xs, (int)H,
                                      lane, acc);
#pragma unroll
            for (int m = 0; m < TPB; ++m) {
                const float v = warp_sum(acc[m]);
                if (lane == 0) ls[m * E + e] = bias ? v + bias[e] : v;
            }
        }
    } else {
        for (uint32_t i = tid; i < nt * E; i += kRouterThreads) {
            const uint32_t t = i / E, e = i - t * E;
            const float v = injected[(size_t)(t0 + t) * E + e];
            ls[t * E + e] = bias ? v + bias[e] : v;
        }
    }
    __syncthreads();

    // one warp per token: softmax + top-k
    for (uint32_t t = warp; t < nt; t += kRouterWarps) {
        const size_t row = (size_t)(t0 + t);
        const bool bad = route_row_warp(ls + t * E, ps + t * E, E, K, scaling, lane, s_tab,
                                        logits_out ? logits_out + row * E : nullptr,
                                        probs_out ? probs_out + row * E : nullptr, ids_out + row * K,
                                        weights_out + row * K);
        if (bad && lane == 0) atomicOr(status, 1u);   // the CPU function returns failure here
    }
}

bool router_gemm_supported(const DLayer &L);
cudaError_t launch_router_logits(const DLayer &L, const __half *hidden, uint32_t n, float *logits, uint32_t *status,
                                 cudaStream_t st, uint64_t *launches);

// logits_scratch: [n][E] floats the many-token path may use for the tensor-core logits (may be null: then the
// CUDA-core kernel computes them).
cudaError_t launch_router(const DLayer &L, const __half *hidden, const float *injected, uint32_t n, float *logits,
                          float *probs, uint32_t *ids, float *weights, uint32_t *status, float *logits_scratch,
                          cudaStream_t st, uint64_t *launches) {
    if (injected == nullptr && n > 32 && logits_scratch != nullptr && router_gemm_supported(L)) {
        cudaError_t err = launch_router_logits(L, hidden, n, logits_scratch, status, st, launches);
        if (err != cudaSuccess) return err;
        injected = logits_scratch;      // softmax / top-k on these logits; the bias is added there
    }
    if (n <= 32) {
        const size_t smem = sizeof(float) * ((size_t)L.H + 2 * (size_t)L.E);
        router_kernel<1><<<n, kRouterThreads, smem, st>>>(hidden, L.router, L.bias, injected, n, L.H, L.E, L.K,
                                                          L.scaling, logits, probs, ids, weights, status);
    } else {
        constexpr int TPB = 8;
        const size_t smem = sizeof(float) * TPB * ((size_t)L.H + 2 * (size_t)L.E);
        if (smem > 160 * 1024) return cudaErrorInvalidValue;
        router_kernel<TPB><<<(n + TPB - 1) / TPB, kRouterThreads, smem, st>>>(
            hidden, L.router, L.bias, injected, n, L.H, L.E, L.K, L.scaling, logits, probs, ids, weights, status);
    }
    ++*launches;
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------- plan
// One block.  Thread t owns the contiguous pair range [t*seg, (t+1)*seg); per-thread per-expert
// counts are scanned across threads so that every thread knows where its first pair of each
// expert lands, then each thread walks its range in order.  The result is the stable sort.
constexpr int kPlanThreads = 256;

__global__ void __launch_bounds__(kPlanThreads)
plan_kernel(const uint32_t *__restrict__ ids, uint32_t n_pairs, uint32_t E, uint32_t T, uint32_t *__restrict__ offsets,
            uint32_t *__restrict__ pair_rows, uint32_t *__restrict__ inverse, uint32_t *__restrict__ active) {
    extern __shared__ uint32_t cnt[];   // [T][E] then totals [E+1]
    uint32_t *tot = cnt + (size_t)T * E;
    const uint32_t tid = threadIdx.x;
    const uint32_t seg = (n_pairs + T - 1) / T;
    const uint32_t lo = min(tid * seg, n_pairs), hi = tid < T ? min(lo + seg, n_pairs) : lo;
    for (uint32_t i = tid; i < T * E; i += kPlanThreads) cnt[i] = 0;
    __syncthreads();
    if (tid < T)
        for (uint32_t p = lo; p < hi; ++p) {
            const uint32_t e = ids[p];
            if (e < E) cnt[tid * E + e]++;
        }
    __syncthreads();
    for (uint32_t e = tid; e < E; e += kPlanThreads) {
        uint32_t run = 0;
        for (uint32_t t = 0; t < T; ++t) {
            const uint32_t c = cnt[t * E + e];
            cnt[t * E + e] = run;
            run += c;
        }
        tot[e] = run;
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t run = 0, na = 0;
        for (uint32_t e = 0; e < E; ++e) {
            const uint32_t c = tot[e];
            offsets[e] = run;
            tot[e] = run;
            if (c) active[1 + na++] = e;
            run += c;
        }
        offsets[E] = run;
        active[0] = na;
    }
    __syncthreads();
    if (tid < T)
        for (uint32_t p = lo; p < hi; ++p) {
            const uint32_t e = ids[p];
            if (e < E) {
                const uint32_t pos = tot[e] + cnt[tid * E + e]++;
                pair_rows[pos] = p;
                inverse[p] = pos;
            } else {
                inverse[p] = 0xffffffffu;
            }
        }
}

// ---- the same plan with many CTAs, for large token counts -----------------------------------
// Pairs are cut into chunks of kChunkPairs; chunk b is handled by CTA b.
//   count   : per-chunk histogram -> chunk_counts[b][E]
//   scan    : per expert, exclusive prefix over chunks (chunk_counts becomes each chunk's first position
//             inside the expert's segment); expert offsets and the list of non-empty experts
//   scatter : inside a chunk, thread t owns kPairsPerThread consecutive pairs; per-thread counts are scanned
//             so that pairs keep their order -> the stable sort again
constexpr int kPairsPerThread = 8;
constexpr int kChunkPairs = kPlanThreads * kPairsPerThread;   // 2048

__global__ void __launch_bounds__(kPlanThreads)
plan_count_kernel(const uint32_t *__restrict__ ids, uint32_t n_pairs, uint32_t E, uint32_t *__restrict__ chunk_counts) {
    __shared__ uint32_t hist[256];
    const uint32_t tid = threadIdx.x, base = blockIdx.x * kChunkPairs;
    hist[tid] = 0;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kPairsPerThread; ++i) {
        const uint32_t p = base + i * kPlanThreads + tid;      // counting needs no order: coalesced reads
        if (p < n_pairs) {
            const uint32_t e = ids[p];
            if (e < E) atomicAdd(&hist[e], 1u);
        }
    }
    __syncthreads();
    if (tid < E) chunk_counts[(size_t)blockIdx.x * E + tid] = hist[tid];
}

__global__ void __launch_bounds__(kPlanThreads)
plan_scan_kernel(uint32_t *__restrict__ chunk_counts, uint32_t n_chunks, uint32_t E, uint32_t *__restrict__ offsets,
                 uint32_t *__restrict__ active) {
    __shared__ uint32_t tot[257];
    const uint32_t e = threadIdx.x;
    if (e < E) {
        uint32_t run = 0;
        for (uint32_t b = 0; b < n_chunks; ++b) {
            const uint32_t c = chunk_counts[(size_t)b * E + e];
            chunk_counts[(size_t)b * E + e] = run;
            run += c;
        }
        tot[e] = run;
    }
    __syncthreads();
    if (e == 0) {
        uint32_t run = 0, na = 0;
        for (uint32_t i = 0; i < E; ++i) {
            const uint32_t c = tot[i];
            offsets[i] = run;
            tot[i] = run;
            if (c) active[1 + na++] = i;
            run += c;
        }
        offsets[E] = run;
        active[0] = na;
    }
    __syncthreads();
    if (e < E)
        for (uint32_t b = 0; b < n_chunks; ++b) chunk_counts[(size_t)b * E + e] += tot[e];
}

__global__ void __launch_bounds__(kPlanThreads)
plan_scatter_kernel(const uint32_t *__restrict__ ids, uint32_t n_pairs, uint32_t E, const uint32_t *__restrict__ chunk_first,
                    uint32_t *__restrict__ pair_rows, uint32_t *__restrict__ inverse) {
    extern __shared__ uint16_t cnt16[];          // [kPlanThreads][E] per-thread counts, then their exclusive prefixes
    uint32_t *first = reinterpret_cast<uint32_t *>(cnt16 + (size_t)kPlanThreads * E);   // [E]
    const uint32_t tid = threadIdx.x, lo = blockIdx.x * kChunkPairs + tid * kPairsPerThread;
    for (uint32_t i = tid; i < kPlanThreads * E / 2; i += kPlanThreads) reinterpret_cast<uint32_t *>(cnt16)[i] = 0;
    if (tid < E) first[tid] = chunk_first[(size_t)blockIdx.x * E + tid];
    __syncthreads();
    uint32_t my[kPairsPerThread];
#pragma unroll
    for (int i = 0; i < kPairsPerThread; ++i) {
        my[i] = lo + i < n_pairs ? ids[lo + i] : 0xffffffffu;
        if (my[i] < E) cnt16[tid * E + my[i]]++;
    }
    __syncthreads();
    if (tid < E) {                               // exclusive scan over threads, one expert per thread
        uint32_t run = 0;
        for (uint32_t t = 0; t < kPlanThreads; ++t) {
            const uint32_t c = cnt16[t * E + tid];
            cnt16[t * E + tid] = (uint16_t)run;
            run += c;
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kPairsPerThread; ++i) {
        const uint32_t p = lo + i;
        if (p >= n_pairs) break;
        const uint32_t e = my[i];
        if (e < E) {
            uint32_t seen = 0;                   // earlier pairs of this thread with the same expert
#pragma unroll
            for (int j = 0; j < kPairsPerThread; ++j) seen += (j < i && my[j] == e);
            const uint32_t pos = first[e] + cnt16[tid * E + e] + seen;
            pair_rows[pos] = p;
            inverse[p] = pos;
        } else {
            inverse[p] = 0xffffffffu;
        }
    }
}

static size_t plan_scatter_smem(uint32_t E) { return (size_t)kPlanThreads * E * 2 + 4 * E + 16; }

// Per-device set-up of this file's kernels; called once when a context is created.
cudaError_t init_router_kernels() {
    cudaError_t err = ensure_exp_table();
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(router_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (err != cudaSuccess) return err;
    return cudaFuncSetAttribute(plan_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024);
}

// chunk_counts: scratch of ceil(n*K / 2048) * E words for the many-CTA form (null: one CTA does everything)
cudaError_t launch_dispatch_plan(const uint32_t *ids, uint32_t n, uint32_t K, uint32_t E, uint32_t *offsets,
                                 uint32_t *pair_rows, uint32_t *inverse, uint32_t *active, uint32_t *chunk_counts,
                                 cudaStream_t st, uint64_t *launches) {
    const uint32_t pairs = n * K;
    if (chunk_counts != nullptr && pairs > 4 * kChunkPairs && E % 2 == 0 && E <= 128) {
        const uint32_t chunks = (pairs + kChunkPairs - 1) / kChunkPairs;
        plan_count_kernel<<<chunks, kPlanThreads, 0, st>>>(ids, pairs, E, chunk_counts);
        plan_scan_kernel<<<1, kPlanThreads, 0, st>>>(chunk_counts, chunks, E, offsets, active);
        plan_scatter_kernel<<<chunks, kPlanThreads, plan_scatter_smem(E), st>>>(ids, pairs, E, chunk_counts, pair_rows, inverse);
        *launches += 3;
        return cudaGetLastError();
    }
    uint32_t T = 24576u / E;
    if (T > (uint32_t)kPlanThreads) T = kPlanThreads;
    if (T == 0) return cudaErrorInvalidValue;
    const size_t smem = sizeof(uint32_t) * ((size_t)T * E + E + 1);
    plan_kernel<<<1, kPlanThreads, smem, st>>>(ids, n * K, E, T, offsets, pair_rows, inverse, active);
    ++*launches;
    return cudaGetLastError();
}

}  // namespace uocr

namespace uocr {
// --------------------------------------------------------------------------------------------
// Dispatch plan for callers that must not allocate device memory.
//
// The plan kernel keeps a by-product - the list of experts that received at least one pair - in
// global memory beside its three outputs.  The regular entry point parks that list in the
// context's arena, which exists only after cudaMalloc calls.  Some hosts of this library cannot
// make such calls at the point where they need a plan: code on a hot path that is guarded against
// allocation (the reference asserts this with uocr_alloc_guard, src/core/uocr_alloc.h:21-42), a real-time decode loop that has frozen its memory map, or an engine whose memory
// admission control has already handed out the whole device budget (the reference engine refuses
// work past its budget, src/core/uocr_api.c:1166-1197).  For them the list lives in the fixed
// array below, which every process that loads this library holds on each device it touches
// (1280 bytes) until it exits.
//
// The array's name is only a host-side handle; the device address comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
constexpr uint32_t kNoAllocMaxExperts = 256;
constexpr uint32_t kNoAllocMaxPairs = 1u << 20;
static __device__ __align__(256) uint32_t g_plan_scratch[320];   // [0] = count, then up to 256 expert ids

struct NoAllocDeviceState {
    uint32_t *scratch = nullptr;
    bool ready = false;
};
static NoAllocDeviceState g_noalloc[64];
static std::mutex g_noalloc_mutex;      // first calls from two host threads must not both run the set-up

}  // namespace uocr

#include "../../include/uocr_cuda_moe.h"

#include <cstdio>

extern "C" int uocr_cuda_moe_dispatch_plan_noalloc(const uint32_t *d_top_ids, uint32_t n_tokens, uint32_t top_k,
                                                   uint32_t n_experts, uint32_t *d_expert_offsets,
                                                   uint32_t *d_pair_rows, uint32_t *d_inverse, void *cuda_stream,
                                                   char *error, size_t error_size) {
    auto fail = [&](const char *msg, const char *detail) {
        if (error && error_size) snprintf(error, error_size, "%s%s%s", msg, detail ? ": " : "", detail ? detail : "");
        return 0;
    };
    if (!d_top_ids || !d_expert_offsets || !d_pair_rows || !d_inverse) return fail("null dispatch-plan argument", nullptr);
    if (n_tokens == 0 || top_k == 0 || n_experts == 0 || top_k > n_experts) return fail("invalid dispatch-plan dimensions", nullptr);
    if (n_experts > uocr::kNoAllocMaxExperts)
        return fail("n_experts exceeds the 256 experts the allocation-free dispatch plan has scratch for", nullptr);
    if ((uint64_t)n_tokens * top_k > uocr::kNoAllocMaxPairs)
        return fail("n_tokens * top_k exceeds the 1048576 pairs the allocation-free dispatch plan accepts", nullptr);
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return fail("cudaGetDevice failed", cudaGetErrorString(err));
    if (dev < 0 || dev >= 64) return fail("device index out of range", nullptr);
    uocr::NoAllocDeviceState &state = uocr::g_noalloc[dev];
    uint32_t *scratch = nullptr;
    {
      std::lock_guard<std::mutex> lock(uocr::g_noalloc_mutex);
      if (!state.ready) {
        // first call on this device: resolve the scratch array's device address and raise the kernel's
        // dynamic shared-memory limit.  Neither allocates; both must happen outside a stream capture.
        void *ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, uocr::g_plan_scratch);
        if (err != cudaSuccess) return fail("cudaGetSymbolAddress(plan scratch) failed", cudaGetErrorString(err));
        err = cudaFuncSetAttribute(uocr::plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
        if (err != cudaSuccess) return fail("cudaFuncSetAttribute(plan kernel) failed", cudaGetErrorString(err));
        state.scratch = static_cast<uint32_t *>(ptr);
        state.ready = true;
      }
      scratch = state.scratch;
    }
    uint64_t launches = 0;
    err = uocr::launch_dispatch_plan(d_top_ids, n_tokens, top_k, n_experts, d_expert_offsets, d_pair_rows, d_inverse,
                                     scratch, nullptr, (cudaStream_t)cuda_stream, &launches);
    if (err != cudaSuccess) return fail("dispatch-plan launch failed", cudaGetErrorString(err));
    return 1;
}

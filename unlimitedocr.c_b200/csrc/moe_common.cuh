// Shared declarations of the CUDA MoE backend: layer parameter blocks passed to kernels,
// dequantisation helpers and the launch interface between the host API and the kernel files.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define UOCR_QT_F16 1
#define UOCR_QT_Q8 3
#define UOCR_QT_Q4 4
#define UOCR_GROUP 64

namespace uocr {

// One projection matrix on the device.
struct DMatrix {
    const uint8_t *w;     // packed weights
    const __half *s;      // fp16 scales [rows][cols/64] (null for f16)
    uint32_t rows, cols;
    uint32_t row_bytes;   // packed bytes per row
    int32_t qtype;
};

// One mapped layer on the device (all pointers are device pointers).
struct DLayer {
    uint32_t H, E, K, F, S;
    float scaling;
    const __half *router;        // [E][H]
    const float *bias;           // [E] or null
    int32_t expert_qtype;
    const uint8_t *expert_w;     // slab
    const __half *expert_s;      // slab
    uint64_t expert_stride_bytes, up_offset_bytes, down_offset_bytes;
    uint64_t expert_scale_stride, up_scale_offset, down_scale_offset;
    DMatrix shared_gate, shared_up, shared_down;
    // Slice-major copy of the quantised weights for the single-token decode kernel (one contiguous blob per
    // 64-wide slice of every expert's and the shared MLP's intermediate dimension), or null.
    const uint8_t *dec_units;
};

// Scratch carved out of the context arena for one forward call.
struct Scratch {
    float *logits;            // [n][E]
    float *probs;             // [n][E]
    uint32_t *top_ids;        // [n][K]
    float *top_weights;       // [n][K]
    uint32_t *expert_offsets; // [E+1]
    uint32_t *pair_rows;      // [n*K]
    uint32_t *inverse;        // [n*K]
    uint32_t *active;         // [E+1]: active[0] = count, then expert ids with >= 1 pair, ascending
    uint32_t *plan_counts;    // [ceil(n*K/2048)][E] per-chunk counts of the many-CTA dispatch plan
    __half *mid;              // routed SwiGLU products [n*K][F], indexed by pair
    __half *shared_mid;       // [n][S]
    void *down_out;           // routed down products [n*K][H], f32 (small n) or fp16
    float *shared_out;        // [n][H] f32
    uint32_t *status;         // device status word: 0 = ok
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- 16-byte chunk dot products -------------------------------------------------------
// x points at fp32 activations of one row in shared memory.  `chunk` is the index of the
// 16-byte chunk inside the weight row.  The returned value already includes the group scale
// (sum of level*x over the chunk, times float(scale)), i.e. partial sums are scaled per group
// exactly as the reference's GPU kernels do.

template <int QT> struct ChunkTraits;
template <> struct ChunkTraits<UOCR_QT_Q4> { static constexpr int kWeights = 32; };
template <> struct ChunkTraits<UOCR_QT_Q8> { static constexpr int kWeights = 16; };
template <> struct ChunkTraits<UOCR_QT_F16> { static constexpr int kWeights = 8; };

// Q4_0: 16 bytes = half of a group's 32 bytes: bytes j0..j0+15, low nibbles are columns
// g*64+j0.., high nibbles columns g*64+32+j0..
template <int M>
__device__ __forceinline__ void chunk_dot_q4(const uint4 &q, const float *x, int ld, int chunk, float scale,
                                             float (&acc)[M]) {
    const int g = chunk >> 1, j0 = (chunk & 1) << 4;
    const float *xl = x + g * 64 + j0;
    const float *xh = xl + 32;
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    float part[M];
#pragma unroll
    for (int m = 0; m < M; ++m) part[m] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t byte = (w[i] >> (8 * b)) & 0xffu;
            const float lo = (float)((int)(byte & 15u) - 8);
            const float hi = (float)((int)(byte >> 4) - 8);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                part[m] = fmaf(lo, xl[m * ld + i * 4 + b], part[m]);
                part[m] = fmaf(hi, xh[m * ld + i * 4 + b], part[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = fmaf(part[m], scale, acc[m]);
}

template <int M>
__device__ __forceinline__ void chunk_dot_q8(const uint4 &q, const float *x, int ld, int chunk, float scale,
                                             float (&acc)[M]) {
    const float *xc = x + chunk * 16;
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    float part[M];
#pragma unroll
    for (int m = 0; m < M; ++m) part[m] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float lv = (float)(int)(int8_t)((w[i] >> (8 * b)) & 0xffu);
#pragma unroll
            for (int m = 0; m < M; ++m) part[m] = fmaf(lv, xc[m * ld + i * 4 + b], part[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = fmaf(part[m], scale, acc[m]);
}

template <int M>
__device__ __forceinline__ void chunk_dot_f16(const uint4 &q, const float *x, int ld, int chunk, float (&acc)[M]) {
    const float *xc = x + chunk * 8;
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
#pragma unroll
        for (int m = 0; m < M; ++m) {
            acc[m] = fmaf(f.x, x[m * ld + chunk * 8 + i * 2], acc[m]);
            acc[m] = fmaf(f.y, x[m * ld + chunk * 8 + i * 2 + 1], acc[m]);
        }
    }
    (void)xc;
}

// Lane-partial dot of one packed weight row with M activation rows (x: fp32 in shared memory,
// row stride ld).  Caller reduces over the warp.
template <int QT, int M>
__device__ __forceinline__ void row_dot(const uint8_t *wrow, const __half *srow, uint32_t cols, const float *x, int ld,
                                        int lane, float (&acc)[M]) {
    const int chunks = (int)(cols / ChunkTraits<QT>::kWeights);
    const uint4 *w4 = reinterpret_cast<const uint4 *>(wrow);
    for (int c = lane; c < chunks; c += 32) {
        const uint4 q = __ldg(w4 + c);
        if (QT == UOCR_QT_Q4) {
            chunk_dot_q4<M>(q, x, ld, c, __half2float(srow[c >> 1]), acc);
        } else if (QT == UOCR_QT_Q8) {
            chunk_dot_q8<M>(q, x, ld, c, __half2float(srow[c >> 2]), acc);
        } else {
            chunk_dot_f16<M>(q, x, ld, c, acc);
        }
    }
}

__device__ __forceinline__ float silu_f32(float v) { return v / (1.0f + __expf(-v)); }
// the same with the fast reciprocal (about 2 ulp; the result is rounded to fp16 anyway): an IEEE division is a
// subroutine of a few hundred cycles, which a latency-bound kernel cannot hide
__device__ __forceinline__ float silu_fast_f32(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// One buffer per rank of an expert-parallel group on one node (this rank's own and the peers' mapped ones).
constexpr int kMaxPeers = 16;
struct PeerBuffers { __half *p[kMaxPeers]; };
// the ranks' synchronisation regions (see ep_exchange_counts_kernel): offsets of every source rank, then three rows of flags
struct PeerSync { uint32_t *p[kMaxPeers]; };
constexpr uint32_t kSyncStride = 260;                          // words per source rank (E + 1 <= 257)
constexpr uint32_t kSyncFlagWords = kMaxPeers * kSyncStride;   // word offset of the flags
constexpr size_t kSyncBytes = (size_t)(kSyncFlagWords + 3 * kMaxPeers) * 4;

// Run-time settings of the single-token decode kernel (a context reads them from the environment when it is created).
struct SlicedKnobs {
    uint32_t replicas = 2;            // copies of the layer accumulator the CTAs spread their additions over (1, 2 or 4)
    long long spin_limit_cycles = 0;  // limit of a wait between CTAs; 0: the built-in limit (about two seconds)
    uint32_t poll_sleep_ns = 0;       // pause between two polls of the layer accumulator
    uint32_t expect_extra = 0;        // test hook: the wait for a layer's output expects this many contributions
                                      // more than there are CTAs, so it runs into its limit
};

// Byte offsets inside the scratch region of the batched decode path.
struct BatchedScratchLayout { size_t acc, x_limbs, x_scales, total; };

// ---- launch interface (implemented in the kernel files, called by the host API) ----------
struct LaunchCounter { uint64_t *count; };

cudaError_t launch_router(const DLayer &L, const __half *hidden, const float *injected, uint32_t n, float *logits,
                          float *probs, uint32_t *ids, float *weights, uint32_t *status, float *logits_scratch,
                          cudaStream_t st, uint64_t *launches);
cudaError_t launch_dispatch_plan(const uint32_t *ids, uint32_t n, uint32_t K, uint32_t E, uint32_t *offsets,
                                 uint32_t *pair_rows, uint32_t *inverse, uint32_t *active, uint32_t *chunk_counts,
                                 cudaStream_t st, uint64_t *launches);
cudaError_t launch_small_batch_layer(const DLayer &L, const Scratch &S, const __half *hidden, const __half *residual,
                                     uint32_t n, __half *out, cudaStream_t st, uint64_t *launches);

}  // namespace uocr

// Small-batch MoE layer: one to a few dozen tokens per step.  The step is bound by reading the
// selected experts' packed weights once, so the kernels are matrix-vector products on CUDA cores:
// one warp per output row, 128-bit loads of the packed row, dequantisation in registers (no
// dequantised copy of a weight ever exists), per-group scale applied to the group's partial sum,
// f32 accumulation and a warp-shuffle reduction.
//
// Work is grouped per selected expert (dispatch plan), so a weight row is read once per step for
// all tokens routed to that expert; activations of up to four tokens at a time sit in shared
// memory as f32.
//
//   gate_up : mid[pair][i]   = fp16( silu(gate_e[i].x) * (up_e[i].x) )     (routed and shared)
//   down    : down_out[pair][h] = down_e[h] . mid[pair]                      (f32 scratch)
//   combine : out[t][h] = fp16( sum_slot w * down_out + shared_out + residual ), slot order
//
// Rounding contract as the reference's GPU kernels (src/backend/metal/kernels/decode_gemv_q4.metal:34-57,
// :138-224): fp16 activations, scale applied per group partial, fp16 `mid`, f32 routed sum.
#include <stdlib.h>

#include "moe_common.cuh"
#include "moe_decode_units.cuh"
#include "moe_sync.cuh"

namespace uocr {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kMaxM = 4;

struct GroupSource {
    // routed: rows are the pairs of one active expert; shared: rows are all tokens
    const uint32_t *active;          // null => shared group
    const uint32_t *expert_offsets;
    const uint32_t *pair_rows;
    uint32_t n_tokens;
    uint32_t K;
};

struct GroupRows {
    uint32_t count;
    const uint32_t *pairs;   // null => identity (shared)
    uint32_t expert;
};

__device__ __forceinline__ bool resolve_group(const GroupSource &g, uint32_t group_index, GroupRows &r) {
    if (g.active == nullptr) {
        r.count = g.n_tokens;
        r.pairs = nullptr;
        r.expert = 0;
        return true;
    }
    if (group_index >= g.active[0]) return false;
    r.expert = g.active[1 + group_index];
    const uint32_t lo = g.expert_offsets[r.expert];
    r.count = g.expert_offsets[r.expert + 1] - lo;
    r.pairs = g.pair_rows + lo;
    return r.count != 0;
}

template <int QT, int M>
__device__ __forceinline__ void gate_up_rows(const uint8_t *gw, const __half *gs, const uint8_t *uw, const __half *us,
                                             uint32_t cols, const float *xs, int lane, float (&g)[M], float (&u)[M]) {
#pragma unroll
    for (int m = 0; m < M; ++m) { g[m] = 0.f; u[m] = 0.f; }
    row_dot<QT, M>(gw, gs, cols, xs, (int)cols, lane, g);
    row_dot<QT, M>(uw, us, cols, xs, (int)cols, lane, u);
#pragma unroll
    for (int m = 0; m < M; ++m) { g[m] = warp_sum(g[m]); u[m] = warp_sum(u[m]); }
}

// grid.x covers the F (or S) output rows, one per warp; grid.y = group index.
template <int QT>
__global__ void __launch_bounds__(kGemvThreads)
gate_up_kernel(GroupSource src, const __half *__restrict__ hidden, uint32_t H, uint32_t F,
               const uint8_t *__restrict__ w_base, const __half *__restrict__ s_base, uint64_t expert_stride_bytes,
               uint64_t up_offset_bytes, uint64_t expert_scale_stride, uint64_t up_scale_offset, uint32_t row_bytes,
               __half *__restrict__ mid) {
    extern __shared__ float xs[];   // [kMaxM][H]
    GroupRows rows;
    if (!resolve_group(src, blockIdx.y, rows)) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t i = blockIdx.x * kGemvWarps + warp;          // output row
    const uint32_t groups = H / UOCR_GROUP;
    const uint8_t *gw = w_base + rows.expert * expert_stride_bytes + (size_t)i * row_bytes;
    const uint8_t *uw = gw + up_offset_bytes;
    const __half *gs = s_base ? s_base + rows.expert * expert_scale_stride + (size_t)i * groups : nullptr;
    const __half *us = s_base ? gs + up_scale_offset : nullptr;

    for (uint32_t r0 = 0; r0 < rows.count; r0 += kMaxM) {
        const uint32_t mc = min((uint32_t)kMaxM, rows.count - r0);
        __syncthreads();
        for (uint32_t k = tid; k < mc * H; k += kGemvThreads) {
            const uint32_t m = k / H, c = k - m * H;
            const uint32_t pair = rows.pairs ? rows.pairs[r0 + m] : (r0 + m);
            const uint32_t token = rows.pairs ? pair / src.K : pair;
            xs[k] = __half2float(hidden[(size_t)token * H + c]);
        }
        __syncthreads();
        if (i >= F) continue;
        float g[kMaxM], u[kMaxM];
        if (mc == 1) {
            float g1[1], u1[1];
            gate_up_rows<QT, 1>(gw, gs, uw, us, H, xs, lane, g1, u1);
            g[0] = g1[0]; u[0] = u1[0];
        } else if (mc == 2) {
            float g2[2], u2[2];
            gate_up_rows<QT, 2>(gw, gs, uw, us, H, xs, lane, g2, u2);
            g[0] = g2[0]; u[0] = u2[0]; g[1] = g2[1]; u[1] = u2[1];
        } else {
            // rows beyond mc read stale shared memory; their results are not stored
            gate_up_rows<QT, kMaxM>(gw, gs, uw, us, H, xs, lane, g, u);
        }
        if (lane == 0) {
            for (uint32_t m = 0; m < mc; ++m) {
                const uint32_t dst_row = rows.pairs ? rows.pairs[r0 + m] : (r0 + m);
                mid[(size_t)dst_row * F + i] = __float2half_rn(silu_f32(g[m]) * u[m]);
            }
        }
    }
}

// down: grid.x covers the H output rows (one per warp), grid.y = group; x = mid rows (fp16, global).
template <int QT>
__global__ void __launch_bounds__(kGemvThreads)
down_kernel(GroupSource src, const __half *__restrict__ mid, uint32_t H, uint32_t F,
            const uint8_t *__restrict__ w_base, const __half *__restrict__ s_base, uint64_t expert_stride_bytes,
            uint64_t expert_scale_stride, uint32_t row_bytes, float *__restrict__ out) {
    extern __shared__ float xs[];   // [kMaxM][F]
    GroupRows rows;
    if (!resolve_group(src, blockIdx.y, rows)) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t h = blockIdx.x * kGemvWarps + warp;
    const uint32_t groups = F / UOCR_GROUP;
    const uint8_t *dw = w_base + rows.expert * expert_stride_bytes + (size_t)h * row_bytes;
    const __half *ds = s_base ? s_base + rows.expert * expert_scale_stride + (size_t)h * groups : nullptr;

    for (uint32_t r0 = 0; r0 < rows.count; r0 += kMaxM) {
        const uint32_t mc = min((uint32_t)kMaxM, rows.count - r0);
        __syncthreads();
        for (uint32_t k = tid; k < mc * F; k += kGemvThreads) {
            const uint32_t m = k / F, c = k - m * F;
            const uint32_t row = rows.pairs ? rows.pairs[r0 + m] : (r0 + m);
            xs[k] = __half2float(mid[(size_t)row * F + c]);
        }
        __syncthreads();
        if (h >= H) continue;
        float acc[kMaxM];
#pragma unroll
        for (int m = 0; m < kMaxM; ++m) acc[m] = 0.f;
        if (mc == 1) {
            float a1[1] = {0.f};
            row_dot<QT, 1>(dw, ds, F, xs, (int)F, lane, a1);
            acc[0] = a1[0];
        } else if (mc == 2) {
            float a2[2] = {0.f, 0.f};
            row_dot<QT, 2>(dw, ds, F, xs, (int)F, lane, a2);
            acc[0] = a2[0]; acc[1] = a2[1];
        } else {
            row_dot<QT, kMaxM>(dw, ds, F, xs, (int)F, lane, acc);
        }
#pragma unroll
        for (int m = 0; m < kMaxM; ++m) acc[m] = warp_sum(acc[m]);
        if (lane == 0)
            for (uint32_t m = 0; m < mc; ++m) {
                const uint32_t row = rows.pairs ? rows.pairs[r0 + m] : (r0 + m);
                out[(size_t)row * H + h] = acc[m];
            }
    }
}

// out[t][h] = fp16( fma chain over slots of w*down_out, + shared, + residual ): the order of
// uocr_cpu_ref_moe_swiglu_f32 (src/backend/cpu_ref/uocr_cpu_ref.c:552-576), residual as the GPU
// layer adds it.  An id >= E contributes nothing.
__global__ void combine_kernel(const float *__restrict__ down_out, const float *__restrict__ shared_out,
                               const __half *__restrict__ residual, const uint32_t *__restrict__ ids,
                               const float *__restrict__ weights, uint32_t n, uint32_t H, uint32_t K, uint32_t E,
                               __half *__restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * H) return;
    const uint32_t t = (uint32_t)(idx / H), h = (uint32_t)(idx - (size_t)t * H);
    float acc = 0.f;
    for (uint32_t s = 0; s < K; ++s) {
        const uint32_t pair = t * K + s;
        if (ids[pair] < E) acc = fmaf(weights[pair], down_out[(size_t)pair * H + h], acc);
    }
    acc += shared_out[idx];
    if (residual) acc += __half2float(residual[idx]);
    out[idx] = __float2half_rn(acc);
}

constexpr int kDenseSmemBytes = 4 * 8192 * (int)sizeof(float);

template <int QT>
static void launch_gate_up(const GroupSource &src, uint32_t n_groups, const __half *hidden, uint32_t H, uint32_t F,
                           const uint8_t *w, const __half *s, uint64_t stride, uint64_t up_off, uint64_t sstride,
                           uint64_t sup_off, uint32_t row_bytes, __half *mid, cudaStream_t st) {
    dim3 grid((F + kGemvWarps - 1) / kGemvWarps, n_groups);
    gate_up_kernel<QT><<<grid, kGemvThreads, sizeof(float) * kMaxM * H, st>>>(src, hidden, H, F, w, s, stride, up_off,
                                                                              sstride, sup_off, row_bytes, mid);
}

template <int QT>
static void launch_down(const GroupSource &src, uint32_t n_groups, const __half *mid, uint32_t H, uint32_t F,
                        const uint8_t *w, const __half *s, uint64_t stride, uint64_t sstride, uint32_t row_bytes,
                        float *out, cudaStream_t st) {
    dim3 grid((H + kGemvWarps - 1) / kGemvWarps, n_groups);
    down_kernel<QT><<<grid, kGemvThreads, sizeof(float) * kMaxM * F, st>>>(src, mid, H, F, w, s, stride, sstride,
                                                                           row_bytes, out);
}

#define UOCR_QT_SWITCH(qt, CALL)                                     \
    switch (qt) {                                                    \
        case UOCR_QT_Q4: { constexpr int QT = UOCR_QT_Q4; CALL; } break;  \
        case UOCR_QT_Q8: { constexpr int QT = UOCR_QT_Q8; CALL; } break;  \
        default: { constexpr int QT = UOCR_QT_F16; CALL; } break;         \
    }

static uint32_t packed_row_bytes(int qt, uint32_t cols) {
    return qt == UOCR_QT_F16 ? cols * 2u : (qt == UOCR_QT_Q8 ? cols : cols / 2u);
}

cudaError_t init_small_batch_kernels() {
    // MoE layers stay below 48 KB of dynamic shared memory (4 rows x 2048 f32 = 32 KB); the dense MLP of the first
    // decoder layer stages rows of its intermediate width (6848) for the down product: 4 x 8192 f32 = 128 KB
    cudaError_t err = cudaFuncSetAttribute(down_kernel<UOCR_QT_Q4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDenseSmemBytes);
    if (err == cudaSuccess) err = cudaFuncSetAttribute(down_kernel<UOCR_QT_Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDenseSmemBytes);
    if (err == cudaSuccess) err = cudaFuncSetAttribute(down_kernel<UOCR_QT_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDenseSmemBytes);
    return err;
}

// ---- dense SwiGLU MLP (the first decoder layer's MLP; uocr_cpu_ref_dense_swiglu_f32, src/backend/cpu_ref/uocr_cpu_ref.c:305-349) ----
// A few tokens through gate/up, down and the residual add with the kernels the shared experts use:
// out = fp16( down . fp16(silu(gate x) * up x) + residual ), f32 sums, one rounding of the result.
bool dense_small_supported(uint32_t H, uint32_t S) {
    return (size_t)kMaxM * H * sizeof(float) <= 48 * 1024 && (size_t)kMaxM * S * sizeof(float) <= (size_t)kDenseSmemBytes;
}

cudaError_t launch_dense_small(const DMatrix &g, const DMatrix &u, const DMatrix &d, const __half *hidden, const __half *residual,
                               uint32_t n, __half *mid, float *out_f32, __half *out, cudaStream_t st, uint64_t *launches) {
    const uint32_t H = g.cols, Sd = g.rows;
    if (!dense_small_supported(H, Sd)) return cudaErrorInvalidValue;
    GroupSource all{nullptr, nullptr, nullptr, n, 1};
    const int64_t up_off = (const uint8_t *)u.w - (const uint8_t *)g.w;
    const int64_t sup_off = g.s ? (u.s - g.s) : 0;
    if (up_off <= 0 || (g.s && sup_off <= 0)) return cudaErrorInvalidValue;      // up follows gate in one allocation
    UOCR_QT_SWITCH(g.qtype, (launch_gate_up<QT>(all, 1, hidden, H, Sd, g.w, g.s, 0, (uint64_t)up_off, 0, (uint64_t)sup_off,
                                                g.row_bytes, mid, st)));
    UOCR_QT_SWITCH(d.qtype, (launch_down<QT>(all, 1, mid, H, Sd, d.w, d.s, 0, 0, d.row_bytes, out_f32, st)));
    const size_t total = (size_t)n * H;
    combine_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(nullptr, out_f32, residual, nullptr, nullptr, n, H, 0, 0, out);
    *launches += 3;
    return cudaGetLastError();
}

cudaError_t launch_small_batch_layer(const DLayer &L, const Scratch &S, const __half *hidden, const __half *residual,
                                     uint32_t n, __half *out, cudaStream_t st, uint64_t *launches) {
    const uint32_t H = L.H, F = L.F, Sd = L.S, K = L.K, E = L.E;
    if ((size_t)kMaxM * (H > Sd ? H : Sd) * sizeof(float) > 48 * 1024) return cudaErrorInvalidValue;
    GroupSource routed{S.active, S.expert_offsets, S.pair_rows, n, K};
    GroupSource shared{nullptr, nullptr, nullptr, n, K};
    const uint32_t max_groups = (uint64_t)n * K < E ? n * K : E;
    const int qt = L.expert_qtype;

    // routed gate/up and shared gate/up
    UOCR_QT_SWITCH(qt, (launch_gate_up<QT>(routed, max_groups, hidden, H, F, L.expert_w, L.expert_s,
                                           L.expert_stride_bytes, L.up_offset_bytes, L.expert_scale_stride,
                                           L.up_scale_offset, packed_row_bytes(qt, H), S.mid, st)));
    ++*launches;
    {
        const DMatrix &g = L.shared_gate, &u = L.shared_up;
        // gate and up of the shared MLP are separate tensors: express "up" as an offset from "gate"
        const int64_t up_off = (const uint8_t *)u.w - (const uint8_t *)g.w;
        const int64_t sup_off = g.s ? (u.s - g.s) : 0;
        UOCR_QT_SWITCH(g.qtype, (launch_gate_up<QT>(shared, 1, hidden, H, Sd, g.w, g.s, 0, (uint64_t)up_off, 0,
                                                    (uint64_t)sup_off, g.row_bytes, S.shared_mid, st)));
        ++*launches;
    }
    // down
    UOCR_QT_SWITCH(qt, (launch_down<QT>(routed, max_groups, S.mid, H, F, L.expert_w + L.down_offset_bytes,
                                        L.expert_s ? L.expert_s + L.down_scale_offset : nullptr,
                                        L.expert_stride_bytes, L.expert_scale_stride, packed_row_bytes(qt, F),
                                        (float *)S.down_out, st)));
    ++*launches;
    {
        const DMatrix &d = L.shared_down;
        UOCR_QT_SWITCH(d.qtype, (launch_down<QT>(shared, 1, S.shared_mid, H, Sd, d.w, d.s, 0, 0, d.row_bytes,
                                                 S.shared_out, st)));
        ++*launches;
    }
    const size_t total = (size_t)n * H;
    combine_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const float *)S.down_out, S.shared_out, residual,
                                                                    S.top_ids, S.top_weights, n, H, K, E, out);
    ++*launches;
    return cudaGetLastError();
}

// ---- LM head: fused logits + argmax ---------------------------------------------------------------------------------
// ids[t] = argmax over the vocabulary rows v of ( row v . x[t] ), ties to the lowest id, NaN rows skipped: the contract of
// the reference's fused kernels (src/backend/metal/kernels/lm_head_q4.metal:25-100, lm_head_q8.metal), which stream the
// whole [vocab][hidden] matrix once per decoded token (83 MB in Q4_0, 165 MB in Q8_0: the largest single reader of a
// decode step after the MoE layers).  Eight lanes per row, four rows per warp and pass, the passes dealt round-robin over a
// grid of a few CTAs per SM; up to four tokens share one pass over the weights.  Every CTA leaves its best (score, id) per token; the CTA that takes the
// last ticket picks the winner.
constexpr int kLmThreads = 256;

__device__ __forceinline__ bool lm_better(float s, uint32_t id, float best, uint32_t best_id) {
    return id != 0xffffffffu && (best_id == 0xffffffffu || s > best || (s == best && id < best_id));
}

template <int QT, int M>
__global__ void __launch_bounds__(kLmThreads)
lm_head_argmax_kernel(const __half *__restrict__ hidden, uint32_t n, uint32_t H, const uint8_t *__restrict__ w, const __half *__restrict__ sc,
                      uint32_t vocab, uint32_t row_bytes, float *__restrict__ part_scores, uint32_t *__restrict__ part_ids,
                      uint32_t *__restrict__ ticket, uint32_t *__restrict__ ids_out, float *__restrict__ scores_out) {
    extern __shared__ float xs[];            // [M][H]
    __shared__ float s_score[kLmThreads / 32][M];
    __shared__ uint32_t s_id[kLmThreads / 32][M];
    __shared__ bool s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (uint32_t k = tid; k < (uint32_t)M * H; k += kLmThreads) xs[k] = k < n * H ? __half2float(hidden[k]) : 0.f;    // slots beyond n: zeros
    __syncthreads();
    const uint32_t groups = H / UOCR_GROUP;
    float best[M];
    uint32_t best_id[M];
#pragma unroll
    for (int m = 0; m < M; ++m) { best[m] = 0.f; best_id[m] = 0xffffffffu; }
    // Eight lanes per row, four rows per warp and pass: a lane's 16-byte pieces of its row (every eighth one, so the eight
    // lanes read 128 contiguous bytes at a time) and their scales are all requested before the first is used, which keeps
    // several kilobytes per warp in flight instead of one load per lane.
    constexpr int kLanesPerRow = 8, kRowsPerPass = 32 / kLanesPerRow, kBatch = 5;
    constexpr int kW = ChunkTraits<QT>::kWeights, kChunksPerGroup = UOCR_GROUP / kW;
    const int sub = lane & (kLanesPerRow - 1), rsel = lane / kLanesPerRow;
    const uint32_t chunks = H / kW;
    const uint32_t pass_rows = gridDim.x * (kLmThreads / 32) * kRowsPerPass;
    for (uint32_t row0 = (blockIdx.x * (kLmThreads / 32) + warp) * kRowsPerPass; row0 < vocab; row0 += pass_rows) {
        const uint32_t row = row0 + rsel;
        const bool valid = row < vocab;
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.f;
        if (valid) {
            const uint4 *w4 = reinterpret_cast<const uint4 *>(w + (size_t)row * row_bytes);
            const __half *srow = sc ? sc + (size_t)row * groups : nullptr;
            for (uint32_t base = 0; base < chunks; base += kLanesPerRow * kBatch) {
                uint4 q[kBatch];
                __half scl[kBatch];
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    const uint32_t c = base + sub + kLanesPerRow * i;
                    if (c < chunks) {
                        q[i] = __ldg(w4 + c);
                        if (QT != UOCR_QT_F16) scl[i] = srow[c / kChunksPerGroup];
                    }
                }
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    const uint32_t c = base + sub + kLanesPerRow * i;
                    if (c < chunks) {
                        if (QT == UOCR_QT_Q4) chunk_dot_q4<M>(q[i], xs, (int)H, (int)c, __half2float(scl[i]), acc);
                        else if (QT == UOCR_QT_Q8) chunk_dot_q8<M>(q[i], xs, (int)H, (int)c, __half2float(scl[i]), acc);
                        else chunk_dot_f16<M>(q[i], xs, (int)H, (int)c, acc);
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float v = acc[m];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            if (valid && v == v && lm_better(v, row, best[m], best_id[m])) { best[m] = v; best_id[m] = row; }
        }
    }
    // the four row groups of the warp
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
        for (int o = kLanesPerRow; o < 32; o <<= 1) {
            const float s2 = __shfl_xor_sync(0xffffffffu, best[m], o);
            const uint32_t i2 = __shfl_xor_sync(0xffffffffu, best_id[m], o);
            if (lm_better(s2, i2, best[m], best_id[m])) { best[m] = s2; best_id[m] = i2; }
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < M; ++m) { s_score[warp][m] = best[m]; s_id[warp][m] = best_id[m]; }
    }
    __syncthreads();
    if (tid < M) {
        float b = 0.f;
        uint32_t bi = 0xffffffffu;
        for (int wv = 0; wv < kLmThreads / 32; ++wv)
            if (lm_better(s_score[wv][tid], s_id[wv][tid], b, bi)) { b = s_score[wv][tid]; bi = s_id[wv][tid]; }
        part_scores[(size_t)blockIdx.x * M + tid] = b;
        part_ids[(size_t)blockIdx.x * M + tid] = bi;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // the last CTA: one warp per token scans every CTA's entry
    if ((uint32_t)warp < n) {
        float b = 0.f;
        uint32_t bi = 0xffffffffu;
        for (uint32_t c = lane; c < gridDim.x; c += 32) {
            const float s2 = __ldcg(part_scores + (size_t)c * M + warp);
            const uint32_t i2 = __ldcg(part_ids + (size_t)c * M + warp);
            if (lm_better(s2, i2, b, bi)) { b = s2; bi = i2; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float s2 = __shfl_xor_sync(0xffffffffu, b, o);
            const uint32_t i2 = __shfl_xor_sync(0xffffffffu, bi, o);
            if (lm_better(s2, i2, b, bi)) { b = s2; bi = i2; }
        }
        if (lane == 0) {
            ids_out[warp] = bi;
            if (scores_out) scores_out[warp] = bi == 0xffffffffu ? -INFINITY : b;
        }
    }
    if (tid == 0) *ticket = 0;               // ready for the next call on the stream
}

// ---- LM head on the integer tensor-core path (Q4_0 / Q8_0) ---------------------------------------------------------
// The scalar kernel above spends ~190 instructions per vocabulary row; this one spends a tenth of that.  A warp takes 16
// consecutive rows; lane (g, t) of it reads, for each 64-wide group, its 16 bytes (Q8_0; 8 in Q4_0) of two of the rows,
// and two m16n8k32 integer MMAs multiply the group's levels with the activations in block-floating-point form
// (group_limbs16(): per group a power-of-two scale and 15-bit mantissas split into a low and a high signed byte).  The
// MMA's eight N columns are (token, limb) for four tokens, so lane (g, t) ends up with the low- and the high-limb sums of
// its two rows for token t and finishes them with one FMA per row and group: (lo + 256 hi) * weight scale * activation
// scale.  The argmax bookkeeping and the ticket are those of the scalar kernel.
constexpr int kLmiBatch = 4, kLmiPad = 64, kLmiTokens = 4;

__device__ __forceinline__ void lmi_group(int (&c)[4], const uint4 &lo, const uint4 &hi, const uint4 &xb) {           // Q8_0
    imma_s8(c, lo.x, hi.x, lo.y, hi.y, xb.x, xb.y);
    imma_s8(c, lo.z, hi.z, lo.w, hi.w, xb.z, xb.w);
}
__device__ __forceinline__ void lmi_group(int (&c)[4], const uint2 &lo, const uint2 &hi, const uint4 &xb) {           // Q4_0
    imma_s8(c, q4_lo16(lo.x), q4_lo16(hi.x), q4_lo16(lo.y), q4_lo16(hi.y), xb.x, xb.y);
    imma_s8(c, q4_hi16(lo.x), q4_hi16(hi.x), q4_hi16(lo.y), q4_hi16(hi.y), xb.z, xb.w);
}

// The rows come in by bulk copies.  One warp only issues them: whole 16-row blocks (Q8_0: 20 KB, contiguous in the
// row-major matrix) into a ring of stages in shared memory, from which eight consumer warps, taking the blocks in turn,
// read their MMA fragments: ~170 KB per SM are on their way at any time without a register or an instruction slot of
// the consumers.  (The same MMAs fed by per-lane global loads, one batch of four groups ahead, spent ~50 instructions
// per group on addresses, predicates and register copies and ran 10 % slower.)
//   * A bulk copy costs the SM's copy engine ~65 ns whatever its size (measured: a ring of 17 copies per block ran at
//     56 ns per copy, one of 5 per block at 72 ns), so a block arrives as TWO copies of eight rows, and the scales of
//     eight consecutive blocks (one per consumer warp) as one copy into a ring of their own.
//   * The second copy of a block lands one group further along the banks than the first, and MMA row g of a block is
//     matrix row 8 (g % 2) + g / 2 (+ 4 for the upper half): the two values of g that share an LDS.128 in Q8_0 read from
//     different copies (no bank conflict although every row starts at a multiple of 128 bytes); in Q4_0, where four
//     values of g share an LDS.64, a two-way conflict remains.
//   * The number of stages is a multiple of the number of consumer warps: every stage is then filled for, and emptied
//     by, one warp only, in order.  With any other count a warp could reach its wait on a stage while the copy of the
//     block BEFORE the awaited one (another warp's) is still on its way; a parity wait cannot tell that phase from the
//     awaited one and would let the warp through.  Every warp passes through every stage of the scale ring.
constexpr int kLmrConsumers = 8, kLmrThreads = (kLmrConsumers + 1) * 32, kLmrMaxStages = 16, kLmrScaleStages = 4;
constexpr size_t kLmrSmemLimit = 231000;     // dynamic shared memory of the kernel; the rest of the SM's 227 KB is static data

template <int QT> struct LmrCfg;
template <> struct LmrCfg<UOCR_QT_Q8> { using T = uint4; static constexpr int kGroupBytes = 64; };
template <> struct LmrCfg<UOCR_QT_Q4> { using T = uint2; static constexpr int kGroupBytes = 32; };

struct LmrLayout {
    uint32_t region, sc_block, sc_stage, stage_bytes, fixed_bytes;
};
template <int QT>
__host__ __device__ __forceinline__ LmrLayout lmr_layout(uint32_t H, uint32_t row_bytes) {
    LmrLayout L;
    const uint32_t groups = H / UOCR_GROUP;
    L.region = 8u * row_bytes + 128u;                              // eight rows and room for the second copy's shift along the banks
    L.sc_block = 16u * groups * 2u;                                // the fp16 scales of one block
    L.sc_stage = kLmrConsumers * L.sc_block;
    L.stage_bytes = 2u * L.region;
    L.fixed_bytes = kLmrScaleStages * L.sc_stage + 2u * kLmiTokens * (H + kLmiPad) + kLmiTokens * groups * 4u +
                    2u * (kLmrMaxStages + kLmrScaleStages) * 8u + 16u;
    return L;
}

template <int QT>
__global__ void __launch_bounds__(kLmrThreads, 1)
lm_head_ring_kernel(const __half *__restrict__ hidden, uint32_t n, uint32_t H, const uint8_t *__restrict__ w, const __half *__restrict__ sc,
                    uint32_t vocab, uint32_t row_bytes, uint32_t stages, float *__restrict__ part_scores, uint32_t *__restrict__ part_ids,
                    uint32_t *__restrict__ ticket, uint32_t *__restrict__ ids_out, float *__restrict__ scores_out) {
    using T = typename LmrCfg<QT>::T;
    constexpr int M = kLmiTokens, kGroupBytes = LmrCfg<QT>::kGroupBytes;
    extern __shared__ __align__(128) uint8_t lmr_smem[];
    __shared__ float s_score[kLmrConsumers][M];
    __shared__ uint32_t s_id[kLmrConsumers][M];
    __shared__ bool s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const uint32_t groups = H / UOCR_GROUP, stride = H + kLmiPad;
    const LmrLayout L = lmr_layout<QT>(H, row_bytes);
    uint8_t *sc_ring = lmr_smem + (size_t)stages * L.stage_bytes;            // [scale stage][block of the round][16 rows][groups] fp16
    uint8_t *xl = sc_ring + kLmrScaleStages * L.sc_stage;                    // [2 * token + limb][H + pad] signed bytes
    float *xsc = reinterpret_cast<float *>(xl + 2 * M * stride);             // [token][group]
    uint64_t *full = reinterpret_cast<uint64_t *>(xsc + M * groups), *empty = full + kLmrMaxStages;
    uint64_t *sc_full = empty + kLmrMaxStages, *sc_empty = sc_full + kLmrScaleStages;
    int *s_flag = reinterpret_cast<int *>(sc_empty + kLmrScaleStages);
    uint32_t *status = ticket + 1;           // a copy that never arrived leaves a bit here; the call then reports no token
    if (tid == 0) {
        for (uint32_t i = 0; i < stages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        for (int i = 0; i < kLmrScaleStages; ++i) { mbar_init(&sc_full[i], 1); mbar_init(&sc_empty[i], kLmrConsumers); }
        s_flag[0] = 0; s_flag[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint32_t nblk = vocab / 16u;
    const uint32_t first = (uint32_t)((uint64_t)blockIdx.x * nblk / gridDim.x), last = (uint32_t)((uint64_t)(blockIdx.x + 1) * nblk / gridDim.x);
    const uint32_t count = last - first;
    float best = 0.f;                      // of token t, over the rows this lane has seen
    uint32_t best_id = 0xffffffffu;

    if (warp == kLmrConsumers) {
        // ---- the copy warp: lanes 0, 1 copy eight rows each; lane 2 the scales of a round of eight blocks
        uint32_t s = 0, round = 0;
        for (uint32_t j = 0; j < count; ++j) {
            const uint32_t blk = first + j;
            if ((j & (kLmrConsumers - 1)) == 0u) {
                const uint32_t r = j / kLmrConsumers, ss = r % kLmrScaleStages, sround = r / kLmrScaleStages;
                if (sround > 0 && !mbar_wait(&sc_empty[ss], (sround - 1u) & 1u, status, s_flag)) break;
                const uint32_t bytes = min((uint32_t)kLmrConsumers, count - j) * L.sc_block;
                if (lane == 2) {
                    mbar_expect_tx(&sc_full[ss], bytes);
                    bulk_g2s(sc_ring + ss * L.sc_stage, sc + (size_t)blk * 16u * groups, bytes, &sc_full[ss]);
                }
            }
            if (round > 0 && !mbar_wait(&empty[s], (round - 1u) & 1u, status, s_flag)) break;
            uint8_t *stage = lmr_smem + (size_t)s * L.stage_bytes;
            if (lane == 0) mbar_expect_tx(&full[s], 16u * row_bytes);
            __syncwarp();
            if (lane < 2) bulk_g2s(stage + lane * (L.region + kGroupBytes), w + ((size_t)blk * 16u + 8u * lane) * row_bytes, 8u * row_bytes, &full[s]);
            if (++s == stages) { s = 0; ++round; }
        }
    } else {
        // ---- consumers: first the activations in limb form, 16 lanes per (token, group); word p of a group holds the
        // four columns the MMAs' B registers want there (limb_column())
        for (uint32_t task = (uint32_t)tid >> 4; task < (uint32_t)M * groups; task += kLmrConsumers * 2) {
            const uint32_t tok = task / groups, G = task % groups;
            const int p = lane & 15;
            float x[4] = {0.f, 0.f, 0.f, 0.f};
            if (tok < n) {
                const uint2 raw = *reinterpret_cast<const uint2 *>(hidden + (size_t)tok * H + G * UOCR_GROUP + limb_column<QT>(p));
                const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
                const float2 f23 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
                x[0] = f01.x; x[1] = f01.y; x[2] = f23.x; x[3] = f23.y;
            }
            const GroupLimbs Lm = group_limbs16(x, 0xffffffffu);
            *reinterpret_cast<uint32_t *>(xl + (2 * tok) * stride + G * UOCR_GROUP + 4 * p) = Lm.lo;
            *reinterpret_cast<uint32_t *>(xl + (2 * tok + 1) * stride + G * UOCR_GROUP + 4 * p) = Lm.hi;
            if (p == 0) xsc[tok * groups + G] = QT == UOCR_QT_Q4 ? Lm.scale * kQ4LevelScale : Lm.scale;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kLmrConsumers * 32) : "memory");
        const uint8_t *xrow = xl + (size_t)g * stride + 16 * t;
        const float *xs_t = xsc + (size_t)t * groups;
        const uint32_t nb = groups / kLmiBatch;
        // MMA rows g and g + 8 of a block are its matrix rows rho and rho + 4: copy g % 2, row g / 2 (+ 4) of the copy
        const uint32_t cpy = (uint32_t)g & 1u, rho = 8u * cpy + ((uint32_t)g >> 1);
        const uint32_t w_off = cpy * (L.region + kGroupBytes) + ((uint32_t)g >> 1) * row_bytes + (uint32_t)t * (uint32_t)sizeof(T);
        const uint32_t s_off = (uint32_t)warp * L.sc_block + rho * groups * 2u;
        uint32_t r = 0;                      // this warp's round: its block is j = warp + 8 r
        for (uint32_t j = (uint32_t)warp; j < count; j += kLmrConsumers, ++r) {
            const uint32_t s = j % stages, round = j / stages, ss = r % kLmrScaleStages;
            bool got = mbar_wait(&sc_full[ss], (r / kLmrScaleStages) & 1u, status, s_flag);
            got = mbar_wait(&full[s], round & 1u, status, s_flag) && got;
            if (!got) break;
            const uint8_t *stage = lmr_smem + (size_t)s * L.stage_bytes;
            const uint8_t *w0p = stage + w_off, *w1p = w0p + 4u * row_bytes;
            const uint8_t *s0p = sc_ring + ss * L.sc_stage + s_off, *s1p = s0p + 4u * groups * 2u;
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll 1
            for (uint32_t b = 0; b < nb; ++b) {
                const uint2 s0 = *reinterpret_cast<const uint2 *>(s0p + b * 8u), s1 = *reinterpret_cast<const uint2 *>(s1p + b * 8u);
                const float4 xs4 = *reinterpret_cast<const float4 *>(xs_t + b * kLmiBatch);
                const float xsv[kLmiBatch] = {xs4.x, xs4.y, xs4.z, xs4.w};
                const __half *h0 = reinterpret_cast<const __half *>(&s0), *h1 = reinterpret_cast<const __half *>(&s1);
#pragma unroll
                for (int i = 0; i < kLmiBatch; ++i) {
                    const uint32_t G = b * kLmiBatch + i;
                    const T w0 = *reinterpret_cast<const T *>(w0p + G * kGroupBytes);
                    const T w1 = *reinterpret_cast<const T *>(w1p + G * kGroupBytes);
                    const uint4 xb = *reinterpret_cast<const uint4 *>(xrow + (size_t)G * UOCR_GROUP);
                    int c[4] = {0, 0, 0, 0};
                    lmi_group(c, w0, w1, xb);
                    acc0 = fmaf((float)(c[0] + c[1] * 256), __half2float(h0[i]) * xsv[i], acc0);
                    acc1 = fmaf((float)(c[2] + c[3] * 256), __half2float(h1[i]) * xsv[i], acc1);
                }
            }
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty[s])) : "memory");
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sc_empty[ss])) : "memory");
            }
            const uint32_t r0 = (first + j) * 16u + rho, r1 = r0 + 4u;
            if (acc0 == acc0 && lm_better(acc0, r0, best, best_id)) { best = acc0; best_id = r0; }
            if (acc1 == acc1 && lm_better(acc1, r1, best, best_id)) { best = acc1; best_id = r1; }
        }
        // the eight row lanes of a token
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            const float s2 = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t i2 = __shfl_xor_sync(0xffffffffu, best_id, o);
            if (lm_better(s2, i2, best, best_id)) { best = s2; best_id = i2; }
        }
        if (lane < M) { s_score[warp][lane] = best; s_id[warp][lane] = best_id; }
    }
    __syncthreads();
    if (tid < M) {
        float bsc = 0.f;
        uint32_t bi = 0xffffffffu;
        for (int wv = 0; wv < kLmrConsumers; ++wv)
            if (lm_better(s_score[wv][tid], s_id[wv][tid], bsc, bi)) { bsc = s_score[wv][tid]; bi = s_id[wv][tid]; }
        part_scores[(size_t)blockIdx.x * M + tid] = bsc;
        part_ids[(size_t)blockIdx.x * M + tid] = bi;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if ((uint32_t)warp < n) {               // the last CTA: one warp per token scans every CTA's entry
        float bsc = 0.f;
        uint32_t bi = 0xffffffffu;
        for (uint32_t c = lane; c < gridDim.x; c += 32) {
            const float s2 = __ldcg(part_scores + (size_t)c * M + warp);
            const uint32_t i2 = __ldcg(part_ids + (size_t)c * M + warp);
            if (lm_better(s2, i2, bsc, bi)) { bsc = s2; bi = i2; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float s2 = __shfl_xor_sync(0xffffffffu, bsc, o);
            const uint32_t i2 = __shfl_xor_sync(0xffffffffu, bi, o);
            if (lm_better(s2, i2, bsc, bi)) { bsc = s2; bi = i2; }
        }
        if (ld_volatile_u32(status) != 0u) bi = 0xffffffffu;
        if (lane == 0) {
            ids_out[warp] = bi;
            if (scores_out) scores_out[warp] = bi == 0xffffffffu ? -INFINITY : bsc;
        }
    }
    __syncthreads();                           // every token's warp has read the status word
    if (tid == 0) { *ticket = 0; *status = 0u; }      // the failed call has reported "no token"; the next call starts clean
}

template <int QT>
static uint32_t lmr_stages(const DMatrix &m) {
    const LmrLayout L = lmr_layout<QT>(m.cols, m.row_bytes);
    if (L.fixed_bytes + (size_t)kLmrConsumers * L.stage_bytes > kLmrSmemLimit) return 0;
    const uint32_t s = (uint32_t)((kLmrSmemLimit - L.fixed_bytes) / L.stage_bytes);
    return s >= (uint32_t)kLmrMaxStages ? (uint32_t)kLmrMaxStages : (uint32_t)kLmrConsumers;      // a multiple of the consumer warps
}
static bool lm_head_ring_ok(const DMatrix &m) {
    if (!((m.qtype == UOCR_QT_Q4 || m.qtype == UOCR_QT_Q8) && m.s != nullptr && m.cols % (UOCR_GROUP * kLmiBatch) == 0 &&
          m.rows >= 16 && m.rows % 16 == 0 && m.row_bytes % 128 == 0)) return false;
    return (m.qtype == UOCR_QT_Q4 ? lmr_stages<UOCR_QT_Q4>(m) : lmr_stages<UOCR_QT_Q8>(m)) != 0;
}

uint32_t lm_head_max_tokens() { return kMaxM; }

cudaError_t init_lm_head_kernels() {
    cudaError_t err = cudaFuncSetAttribute(lm_head_ring_kernel<UOCR_QT_Q4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLmrSmemLimit);
    if (err == cudaSuccess) err = cudaFuncSetAttribute(lm_head_ring_kernel<UOCR_QT_Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLmrSmemLimit);
    return err;
}

cudaError_t launch_lm_head_argmax(const DMatrix &m, const __half *hidden, uint32_t n, uint32_t grid, float *part_scores,
                                  uint32_t *part_ids, uint32_t *ticket, uint32_t *ids_out, float *scores_out, cudaStream_t st,
                                  uint64_t *launches) {
    if (n == 0 || n > (uint32_t)kMaxM) return cudaErrorInvalidValue;
    if (lm_head_ring_ok(m)) {
        const uint32_t cg = grid >= 8 ? grid / 8 : grid;          // one CTA per SM (the scratch was sized for eight per SM)
        if (m.qtype == UOCR_QT_Q4) {
            const uint32_t stg = lmr_stages<UOCR_QT_Q4>(m);
            const LmrLayout L = lmr_layout<UOCR_QT_Q4>(m.cols, m.row_bytes);
            lm_head_ring_kernel<UOCR_QT_Q4><<<cg, kLmrThreads, L.fixed_bytes + (size_t)stg * L.stage_bytes, st>>>(
                hidden, n, m.cols, m.w, m.s, m.rows, m.row_bytes, stg, part_scores, part_ids, ticket, ids_out, scores_out);
        } else {
            const uint32_t stg = lmr_stages<UOCR_QT_Q8>(m);
            const LmrLayout L = lmr_layout<UOCR_QT_Q8>(m.cols, m.row_bytes);
            lm_head_ring_kernel<UOCR_QT_Q8><<<cg, kLmrThreads, L.fixed_bytes + (size_t)stg * L.stage_bytes, st>>>(
                hidden, n, m.cols, m.w, m.s, m.rows, m.row_bytes, stg, part_scores, part_ids, ticket, ids_out, scores_out);
        }
        ++*launches;
        return cudaGetLastError();
    }
    if ((size_t)kMaxM * m.cols * sizeof(float) > 48 * 1024) return cudaErrorInvalidValue;
    const size_t smem = sizeof(float) * (n <= 1 ? 1 : (n == 2 ? 2 : kMaxM)) * m.cols;
#define UOCR_LM_LAUNCH(MM)                                                                                                       \
    UOCR_QT_SWITCH(m.qtype, (lm_head_argmax_kernel<QT, MM><<<grid, kLmThreads, smem, st>>>(hidden, n, m.cols, m.w, m.s, m.rows, m.row_bytes, \
                                                                                           part_scores, part_ids, ticket, ids_out, scores_out)))
    if (n == 1) { UOCR_LM_LAUNCH(1); }
    else if (n == 2) { UOCR_LM_LAUNCH(2); }
    else {
        // three tokens run in the four-token instantiation: the fourth slot holds zeros and writes nothing
        UOCR_LM_LAUNCH(kMaxM);
    }
#undef UOCR_LM_LAUNCH
    ++*launches;
    return cudaGetLastError();
}

// ---- dequantisation probe ------------------------------------------------------------------------------------
// out[row][col] = the f32 value the matrix-vector kernels give weight (row, col): the row is multiplied, through the
// same row_dot() the layer kernels use, with a one-hot activation vector per column, which leaves level * scale.
// One CTA per row, one activation buffer per warp.
constexpr int kProbeWarps = 4;

template <int QT>
__global__ void __launch_bounds__(kProbeWarps * 32)
dequant_probe_kernel(const uint8_t *__restrict__ w, const __half *__restrict__ s, uint32_t cols, uint32_t row_bytes,
                     float *__restrict__ out) {
    extern __shared__ float xs[];   // [kProbeWarps][cols]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.x, groups = cols / UOCR_GROUP;
    float *x = xs + (size_t)warp * cols;
    for (uint32_t c = lane; c < cols; c += 32) x[c] = 0.f;
    __syncwarp();
    const uint8_t *wrow = w + (size_t)row * row_bytes;
    const __half *srow = s ? s + (size_t)row * groups : nullptr;
    for (uint32_t c = warp; c < cols; c += kProbeWarps) {
        if (lane == 0) x[c] = 1.f;
        __syncwarp();
        float acc[1] = {0.f};
        row_dot<QT, 1>(wrow, srow, cols, x, (int)cols, lane, acc);
        const float v = warp_sum(acc[0]);
        if (lane == 0) { out[(size_t)row * cols + c] = v; x[c] = 0.f; }
        __syncwarp();
    }
}

cudaError_t launch_dequant_probe(const DMatrix &m, float *out, cudaStream_t st, uint64_t *launches) {
    const size_t smem = sizeof(float) * kProbeWarps * m.cols;
    if (smem > 48 * 1024) return cudaErrorInvalidValue;
    UOCR_QT_SWITCH(m.qtype, (dequant_probe_kernel<QT><<<m.rows, kProbeWarps * 32, smem, st>>>(m.w, m.s, m.cols, m.row_bytes, out)));
    ++*launches;
    return cudaGetLastError();
}

}  // namespace uocr

// Batched decode: a handful to a few dozen tokens per step (5 .. 64) at the model's shapes, Q4_0 / Q8_0.
//
// Such a step is bound by reading the weights of the experts it selects, once each, so the kernel is
// weight-stationary on the slice-major "unit blobs" of the single-token decode kernel: one CTA takes two
// consecutive 64-wide slices of the intermediate dimension of ONE selected expert (or of the shared MLP) and
// multiplies them with all tokens routed to that expert, 16 tokens per pass:
//   1. the pass's activations are written as block-floating-point bytes (two signed bytes per value, one scale per
//      token and 64-wide group), the B operand of the integer MMAs;
//   2. per slice the 128 gate / up rows stream through a four-stage ring of bulk copies (one chunk = four
//      quantisation groups), each chunk multiplied with up to 16 tokens: a token occupies two of the MMA's eight
//      columns, so one MMA covers four tokens;
//   3. the SwiGLU products never leave the SM: they are rounded to fp16, rewritten as bytes, and multiplied with the
//      slice's 64 columns of `down` (held in registers);
//   4. the slice's partial outputs go to a per-part buffer ([part][row][H], f32; the CTA's second slice adds to its
//      first), and the combine kernel adds the parts in a fixed order, applies the routing weights in slot order, adds
//      the shared MLP and the residual and rounds to fp16: bit-reproducible, no atomics.
// An expert with more than 16 tokens is processed in several passes (its weights then come from L2).
// Rounding contract as the single-token kernel: fp16 activations, scale applied per group partial, fp16 SwiGLU
// products, f32 routed sum (src/backend/metal/kernels/decode_gemv_q8.metal:166-251).
// Every wait is bounded (moe_sync.cuh).
#include <cuda.h>

#include "moe_decode_units.cuh"
#include "moe_sync.cuh"

namespace uocr {

constexpr int kBtConsumers = 512;                              // 16 warps compute
constexpr int kBtThreads = kBtConsumers + 32;                  // + one warp that issues the bulk copies
constexpr int kBtTokens = 16;                                  // tokens per pass
constexpr int kBtSlices = 2;                                   // consecutive slices per CTA
constexpr int kBtRoutedParts = kSlRoutedPerSlot / kBtSlices;   // 7 CTAs per selected expert
constexpr int kBtSharedParts = kSlS / 64 / kBtSlices;          // 14 CTAs for the shared MLP
constexpr int kBtStages = 4;
constexpr int kBtChunks = 5;                                   // chunks of four groups per slice
constexpr int kBtMaxTokens = 64;
constexpr int kBtBlocksPerWarp = kSlH / 16 / 16;               // 5 blocks of 16 `down` rows per warp

struct BatchedParams {
    const uint8_t *units;             // slice-major weights of the layer
    const __half *hidden;             // [n][H]
    uint32_t n, K;
    uint32_t max_groups;              // selected experts the grid has CTAs for
    const uint32_t *active;           // [0] = number of experts with at least one pair, then their ids
    const uint32_t *expert_offsets;   // [E + 1]
    const uint32_t *pair_rows;        // pairs grouped by expert
    float *routed_part;               // [kBtRoutedParts][n * K][H], row = position in pair_rows
    float *shared_part;               // [kBtSharedParts][n][H]
    uint32_t *status;
};

template <int QT> struct BtSmem {
    static constexpr int kChunkBytes = SlBlob<QT>::kGuBytes / kBtChunks;
    static constexpr int kRing = 0;
    static constexpr int kSc = kRing + kBtStages * kChunkBytes;             // two buffers of gate / up scales
    static constexpr int kXf = kSc + 2 * SlBlob<QT>::kGuScBytes;            // activation bytes [16 tok][20][2][16 words]
    static constexpr int kXs = kXf + kBtTokens * kSlGroups * 2 * 64;        // their scales [16 tok][20]
    static constexpr int kMid = kXs + kBtTokens * kSlGroups * 4;            // SwiGLU products [16 tok][64] fp16
    static constexpr int kMidf = kMid + kBtTokens * 64 * 2;                 // their bytes [16 tok][2][16 words]
    static constexpr int kMs = kMidf + kBtTokens * 2 * 64;                  // their scales [16]
    static constexpr int kTok = kMs + 64;                                   // token of each slot of the pass [16]
    static constexpr int kBars = kTok + 64;                                 // full[4], empty[4], sc_full[2], sc_empty[2], flags
    static constexpr int kTotal = kBars + 128;
};

__device__ __forceinline__ void bt_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kBtConsumers) : "memory"); }
__device__ __forceinline__ void bt_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int QT>
__global__ void __launch_bounds__(kBtThreads, 1) decode_batched_kernel(const __grid_constant__ BatchedParams prm) {
    using Bl = SlBlob<QT>;
    using Sm = BtSmem<QT>;
    constexpr int H = kSlH;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint4 *s_ring4 = reinterpret_cast<const uint4 *>(smem + Sm::kRing);
    const __half *s_sc = reinterpret_cast<const __half *>(smem + Sm::kSc);
    uint32_t *s_xf = reinterpret_cast<uint32_t *>(smem + Sm::kXf);
    float *s_xs = reinterpret_cast<float *>(smem + Sm::kXs);
    __half *s_mid = reinterpret_cast<__half *>(smem + Sm::kMid);
    uint32_t *s_midf = reinterpret_cast<uint32_t *>(smem + Sm::kMidf);
    float *s_ms = reinterpret_cast<float *>(smem + Sm::kMs);
    uint32_t *s_tok = reinterpret_cast<uint32_t *>(smem + Sm::kTok);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + Sm::kBars), *empty = full + kBtStages, *sc_full = empty + kBtStages,
             *sc_empty = sc_full + 2;
    int *s_flag = reinterpret_cast<int *>(sc_empty + 2);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // ---- which unit: (selected expert, part) or (shared MLP, part)
    const uint32_t routed_ctas = prm.max_groups * kBtRoutedParts;
    const bool routed = blockIdx.x < routed_ctas;
    uint32_t expert = 0, part, cnt, row0, rows_total;
    if (routed) {
        const uint32_t group = blockIdx.x / kBtRoutedParts;
        part = blockIdx.x % kBtRoutedParts;
        if (group >= prm.active[0]) return;                       // fewer distinct experts than the grid allows for
        expert = prm.active[1 + group];
        row0 = prm.expert_offsets[expert];
        cnt = prm.expert_offsets[expert + 1] - row0;
        rows_total = prm.n * prm.K;
    } else {
        part = blockIdx.x - routed_ctas;
        row0 = 0;
        cnt = prm.n;
        rows_total = prm.n;
    }
    if (cnt == 0) return;
    const uint32_t first_unit = routed ? expert * kSlRoutedPerSlot + part * kBtSlices
                                       : (uint32_t)kSlE * kSlRoutedPerSlot + part * kBtSlices;
    float *out_base = (routed ? prm.routed_part : prm.shared_part) + (size_t)part * rows_total * H;
    const uint32_t passes = (cnt + kBtTokens - 1) / kBtTokens;

    if (tid == 0) {
        for (int i = 0; i < kBtStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], kBtConsumers / 32); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sc_full[i], 1); mbar_init(&sc_empty[i], kBtConsumers / 32); }
        s_flag[0] = 1; s_flag[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kBtConsumers / 32) {
        // ---- producer: the gate / up fragments of every (pass, slice), chunk by chunk through the ring, and their scales
        if (lane == 0) {
            uint32_t seq = 0, slices_done = 0;
            for (uint32_t ps = 0; ps < passes; ++ps) {
                for (int sl = 0; sl < kBtSlices; ++sl, ++slices_done) {
                    const uint8_t *blob = prm.units + (size_t)(first_unit + sl) * Bl::kBytes;
                    const uint32_t sb = slices_done & 1u;
                    if (slices_done >= 2u && !mbar_wait(&sc_empty[sb], ((slices_done >> 1) - 1u) & 1u, prm.status, s_flag)) return;
                    for (int c = 0; c < kBtChunks; ++c, ++seq) {
                        const uint32_t s = seq % kBtStages;
                        if (seq >= (uint32_t)kBtStages && !mbar_wait(&empty[s], ((seq / kBtStages) - 1u) & 1u, prm.status, s_flag)) return;
                        mbar_expect_tx(&full[s], Sm::kChunkBytes);
                        bulk_g2s(smem + Sm::kRing + s * Sm::kChunkBytes, blob + Bl::kGu + (size_t)c * Sm::kChunkBytes, Sm::kChunkBytes, &full[s]);
                        if (c == 0) {
                            mbar_expect_tx(&sc_full[sb], Bl::kGuScBytes);
                            bulk_g2s(smem + Sm::kSc + sb * Bl::kGuScBytes, blob + Bl::kGuSc, Bl::kGuScBytes, &sc_full[sb]);
                        }
                    }
                }
            }
        }
        return;
    }

    // ---- consumers
    const int rb = warp & 7, nh = warp >> 3;       // gate / up: row block, and which n-blocks (nh, nh + 2) of the pass
    uint32_t seq = 0, slices_done = 0;
    for (uint32_t ps = 0; ps < passes; ++ps) {
        const uint32_t p0 = ps * kBtTokens;
        const uint32_t T = min((uint32_t)kBtTokens, cnt - p0), NB = (T + 3u) / 4u;
        if (tid < kBtTokens)
            s_tok[tid] = (uint32_t)tid < T ? (routed ? prm.pair_rows[row0 + p0 + tid] / prm.K : p0 + tid) : 0xffffffffu;
        bt_sync();
        // 1. activation bytes of the pass's tokens: 16 lanes per (token, group); slots beyond T hold zeros
#pragma unroll 2
        for (int r = 0; r < kBtTokens * kSlGroups * 16 / kBtConsumers; ++r) {
            const int idx = r * kBtConsumers + tid, task = idx >> 4, p = idx & 15;
            const int tok = task / kSlGroups, Gi = task - tok * kSlGroups;
            float xv[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t token = s_tok[tok];
            if (token != 0xffffffffu) {
                const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(prm.hidden + (size_t)token * H + Gi * 64 + limb_column<QT>(p)));
                const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
                const float2 f23 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
                xv[0] = f01.x; xv[1] = f01.y; xv[2] = f23.x; xv[3] = f23.y;
            }
            const GroupLimbs L = group_limbs(xv);
            uint32_t *d = s_xf + ((tok * kSlGroups + Gi) * 2) * 16 + p;
            d[0] = L.lo;
            d[16] = L.hi;
            if (p == 0) s_xs[tok * kSlGroups + Gi] = QT == UOCR_QT_Q4 ? L.scale * kQ4LevelScale : L.scale;
        }
        bt_sync();

        for (int sl = 0; sl < kBtSlices; ++sl, ++slices_done) {
            const uint8_t *blob = prm.units + (size_t)(first_unit + sl) * Bl::kBytes;
            const uint32_t sb = slices_done & 1u;
            // the slice's 64 columns of `down` for this warp's five 16-row blocks, and the rows' scales, into registers
            uint4 dwn[kBtBlocksPerWarp][2];
            __half dslo[kBtBlocksPerWarp], dshi[kBtBlocksPerWarp];
            {
                const uint4 *dn = reinterpret_cast<const uint4 *>(blob + Bl::kDn);
                const __half *dsc = reinterpret_cast<const __half *>(blob + Bl::kDnSc);
#pragma unroll
                for (int bi = 0; bi < kBtBlocksPerWarp; ++bi) {
                    const int blk = warp + 16 * bi;
                    if (QT == UOCR_QT_Q8) {
                        dwn[bi][0] = __ldg(dn + (blk * 2) * 32 + lane);
                        dwn[bi][1] = __ldg(dn + (blk * 2 + 1) * 32 + lane);
                    } else {
                        dwn[bi][0] = __ldg(dn + blk * 32 + lane);
                    }
                    dslo[bi] = dsc[16 * blk + g];
                    dshi[bi] = dsc[16 * blk + 8 + g];
                }
            }
            // 2. gate / up: rows 8 rb .. + 7 of both matrices x the tokens of n-blocks nh and nh + 2
            float ag[2] = {0.f, 0.f}, au[2] = {0.f, 0.f};
            const __half *scg = s_sc + sb * (Bl::kGuScBytes / 2) + (8 * rb + g) * kSlGroups;
            const __half *scu = scg + 64 * kSlGroups;
            bool got = true;
            for (int c = 0; c < kBtChunks; ++c, ++seq) {
                const uint32_t s = seq % kBtStages;
                got = mbar_wait(&full[s], (seq / kBtStages) & 1u, prm.status, s_flag) && got;
                if (c == 0) got = mbar_wait(&sc_full[sb], (slices_done >> 1) & 1u, prm.status, s_flag) && got;
                const uint4 *w4 = s_ring4 + (size_t)s * (Sm::kChunkBytes / 16);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int Gi = 4 * c + q;
                    uint4 wa, wb;
                    if (QT == UOCR_QT_Q8) { wa = w4[((q * 8 + rb) * 2) * 32 + lane]; wb = w4[((q * 8 + rb) * 2 + 1) * 32 + lane]; }
                    else { wa = w4[(q * 8 + rb) * 32 + lane]; wb = wa; }
                    const float sg = __half2float(scg[Gi]), su = __half2float(scu[Gi]);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const uint32_t nb = (uint32_t)nh + 2u * i;
                        if (nb < NB) {
                            const int tokl = 4 * (int)nb + (g >> 1);
                            const uint4 xb = *reinterpret_cast<const uint4 *>(s_xf + (((tokl * kSlGroups + Gi) * 2 + (g & 1)) * 4 + t) * 4);
                            int ca[4] = {0, 0, 0, 0}, cb[4] = {0, 0, 0, 0};
                            if (QT == UOCR_QT_Q8) group_imma(ca, cb, wa, wb, xb);
                            else group_imma(ca, cb, make_uint2(wa.x, wa.y), make_uint2(wa.z, wa.w), xb);
                            const float xs = s_xs[(4 * (int)nb + t) * kSlGroups + Gi];
                            ag[i] = fmaf((float)(ca[0] + cb[0] + (ca[1] + cb[1]) * 256), sg * xs, ag[i]);
                            au[i] = fmaf((float)(ca[2] + cb[2] + (ca[3] + cb[3]) * 256), su * xs, au[i]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) bt_arrive(&empty[s]);
            }
            __syncwarp();
            if (lane == 0) bt_arrive(&sc_empty[sb]);
            // 3. SwiGLU in registers: lane (g, t) holds gate and up of column 8 rb + g for token 4 nb + t
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t nb = (uint32_t)nh + 2u * i;
                if (nb < NB) s_mid[(4 * nb + t) * 64 + 8 * rb + g] = __float2half_rn(got ? silu_fast_f32(ag[i]) * au[i] : 0.f);
            }
            bt_sync();
            if (tid < kBtTokens * 16) {                // the products as bytes: 16 lanes per token
                const int tok = tid >> 4, p = tid & 15;
                float mv[4] = {0.f, 0.f, 0.f, 0.f};
                if ((uint32_t)tok < 4u * NB) load_word_values<QT>(s_mid + tok * 64, p, mv);
                const GroupLimbs M = group_limbs(mv);
                uint32_t *d = s_midf + (tok * 2) * 16 + p;
                d[0] = M.lo;
                d[16] = M.hi;
                if (p == 0) s_ms[tok] = QT == UOCR_QT_Q4 ? M.scale * kQ4LevelScale : M.scale;
            }
            bt_sync();
            // 4. down: this warp's 80 rows x the slice's 64 columns x every token of the pass
            for (uint32_t nb = 0; nb < NB; ++nb) {
                const uint4 mbf = *reinterpret_cast<const uint4 *>(s_midf + (((4 * nb + (g >> 1)) * 2 + (g & 1)) * 4 + t) * 4);
                const uint32_t tokc = 4u * nb + t;
                const float ms = s_ms[tokc];
                float *dst = out_base + (size_t)(row0 + p0 + tokc) * H;
#pragma unroll
                for (int bi = 0; bi < kBtBlocksPerWarp; ++bi) {
                    int ca[4] = {0, 0, 0, 0}, cb[4] = {0, 0, 0, 0};
                    if (QT == UOCR_QT_Q8) group_imma(ca, cb, dwn[bi][0], dwn[bi][1], mbf);
                    else group_imma(ca, cb, make_uint2(dwn[bi][0].x, dwn[bi][0].y), make_uint2(dwn[bi][0].z, dwn[bi][0].w), mbf);
                    if (tokc < T) {
                        const float v0 = (float)(ca[0] + cb[0] + (ca[1] + cb[1]) * 256) * (__half2float(dslo[bi]) * ms);
                        const float v1 = (float)(ca[2] + cb[2] + (ca[3] + cb[3]) * 256) * (__half2float(dshi[bi]) * ms);
                        const uint32_t r = 16u * (warp + 16 * bi) + g;
                        if (sl == 0) { dst[r] = v0; dst[r + 8] = v1; }
                        else { dst[r] += v0; dst[r + 8] += v1; }          // same thread, same address as for the first slice
                    }
                }
            }
            bt_sync();
        }
    }
}

// out[t][h] = fp16( fma chain over slots of w * (sum of the routed parts) + (sum of the shared parts) + residual )
__global__ void combine_batched_kernel(const float *__restrict__ routed_part, const float *__restrict__ shared_part,
                                       const __half *__restrict__ residual, const uint32_t *__restrict__ inverse,
                                       const float *__restrict__ weights, uint32_t n, uint32_t H, uint32_t K,
                                       __half *__restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;       // one thread per 4 outputs
    const uint32_t per_row = H / 4;
    if (idx >= (size_t)n * per_row) return;
    const uint32_t tkn = (uint32_t)(idx / per_row), c = (uint32_t)(idx % per_row) * 4;
    const size_t routed_stride = (size_t)n * K * H, shared_stride = (size_t)n * H;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (uint32_t s = 0; s < K; ++s) {
        const uint32_t pos = inverse[tkn * K + s];
        if (pos == 0xffffffffu) continue;
        const float w = weights[tkn * K + s];
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int p = 0; p < kBtRoutedParts; ++p) {
            const float4 v = *reinterpret_cast<const float4 *>(routed_part + p * routed_stride + (size_t)pos * H + c);
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        acc[0] = fmaf(w, sum.x, acc[0]); acc[1] = fmaf(w, sum.y, acc[1]);
        acc[2] = fmaf(w, sum.z, acc[2]); acc[3] = fmaf(w, sum.w, acc[3]);
    }
    float4 sh = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int p = 0; p < kBtSharedParts; ++p) {
        const float4 v = *reinterpret_cast<const float4 *>(shared_part + p * shared_stride + (size_t)tkn * H + c);
        sh.x += v.x; sh.y += v.y; sh.z += v.z; sh.w += v.w;
    }
    acc[0] += sh.x; acc[1] += sh.y; acc[2] += sh.z; acc[3] += sh.w;
    if (residual) {
        const uint2 rv = *reinterpret_cast<const uint2 *>(residual + (size_t)tkn * H + c);
        const float2 r01 = __half22float2(*reinterpret_cast<const __half2 *>(&rv.x));
        const float2 r23 = __half22float2(*reinterpret_cast<const __half2 *>(&rv.y));
        acc[0] += r01.x; acc[1] += r01.y; acc[2] += r23.x; acc[3] += r23.y;
    }
    uint2 o;
    *reinterpret_cast<__half2 *>(&o.x) = __floats2half2_rn(acc[0], acc[1]);
    *reinterpret_cast<__half2 *>(&o.y) = __floats2half2_rn(acc[2], acc[3]);
    *reinterpret_cast<uint2 *>(out + (size_t)tkn * H + c) = o;
}

// ---------------------------------------------------------------- host side
bool decode_sliced_layer_ok(const DLayer &L);

cudaError_t init_decode_batched_kernels() {
    cudaError_t err = cudaFuncSetAttribute(decode_batched_kernel<UOCR_QT_Q4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)BtSmem<UOCR_QT_Q4>::kTotal);
    if (err != cudaSuccess) return err;
    return cudaFuncSetAttribute(decode_batched_kernel<UOCR_QT_Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)BtSmem<UOCR_QT_Q8>::kTotal);
}

uint32_t decode_batched_max_tokens() { return kBtMaxTokens; }
size_t decode_batched_routed_part_bytes(uint32_t n, uint32_t K) { return (size_t)kBtRoutedParts * n * K * kSlH * sizeof(float); }
size_t decode_batched_shared_part_bytes(uint32_t n) { return (size_t)kBtSharedParts * n * kSlH * sizeof(float); }

// The model's shapes in Q4_0 / Q8_0 with the slice-major copy present, and a token count this kernel is built for.
bool decode_batched_supported(const DLayer &L, uint32_t n) {
    return n >= 2 && n <= (uint32_t)kBtMaxTokens && decode_sliced_layer_ok(L) && L.dec_units != nullptr;
}

// Routed experts and shared MLP of n tokens whose routing and dispatch plan are in S; then the combine.
cudaError_t launch_decode_batched(const DLayer &L, const Scratch &S, const __half *hidden, const __half *residual, uint32_t n,
                                  float *routed_part, float *shared_part, __half *out, cudaStream_t st, uint64_t *launches) {
    BatchedParams p{};
    p.units = L.dec_units; p.hidden = hidden; p.n = n; p.K = L.K;
    p.max_groups = (uint64_t)n * L.K < L.E ? n * L.K : L.E;
    p.active = S.active; p.expert_offsets = S.expert_offsets; p.pair_rows = S.pair_rows;
    p.routed_part = routed_part; p.shared_part = shared_part; p.status = S.status;
    const uint32_t grid = p.max_groups * kBtRoutedParts + kBtSharedParts;
    if (L.expert_qtype == UOCR_QT_Q4) decode_batched_kernel<UOCR_QT_Q4><<<grid, kBtThreads, BtSmem<UOCR_QT_Q4>::kTotal, st>>>(p);
    else decode_batched_kernel<UOCR_QT_Q8><<<grid, kBtThreads, BtSmem<UOCR_QT_Q8>::kTotal, st>>>(p);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    const size_t work = (size_t)n * (L.H / 4);
    combine_batched_kernel<<<(unsigned)((work + 255) / 256), 256, 0, st>>>(routed_part, shared_part, residual, S.inverse,
                                                                           S.top_weights, n, L.H, L.K, out);
    *launches += 2;
    return cudaGetLastError();
}

}  // namespace uocr

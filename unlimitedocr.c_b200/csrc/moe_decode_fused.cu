// Single-token decode: a run of MoE layers in ONE persistent kernel.
//
// One decode step of one token reads ~14.8 MB of packed weights per layer (Q4_0) and does almost no
// arithmetic, so the step is bound by HBM bandwidth and by the latency of the dependencies inside a
// layer (hidden -> routing -> selected experts' gate/up -> SwiGLU products -> down -> next hidden).
// A kernel launch per dependency would cost more than the data movement; here one CTA per SM stays
// resident for all layers and the dependencies are two grid-wide barriers per layer.
//
// Per layer, with G CTAs of 16 warps:
//   routing   every CTA sums the per-CTA partial router logits the previous phase left in global
//             memory (fixed order), and warp 0 runs the softmax / top-k.  All CTAs get identical ids.
//   phase A   the K*F routed + S shared (gate row, up row) pairs are split evenly over CTAs and warps.
//             Each warp's lane 0 issues TMA bulk copies (cp.async.bulk, one mbarrier per row pair) of
//             its packed rows into shared memory - every byte of the CTA's share is in flight at once -
//             and the warp then reduces each pair against the activations it holds in registers:
//             dequantisation in registers, per-group scale on the group partial, f32 accumulate,
//             shuffle reduction, mid = fp16(silu(gate) * up) written to global memory.
//   barrier
//   phase B   the H output rows are split evenly over CTAs.  A (row, source) job - source = one of the
//             K selected experts or half of the shared MLP - is one warp-wide dot of a packed `down`
//             row with that source's SwiGLU products.  The down rows were requested with plain loads
//             before the barrier, so they arrive while the barrier is pending.  Thread r then combines
//             row r in slot order (fma chain), adds shared and residual, rounds to fp16, stores the
//             next hidden value, and the CTA stores its partial logits of the NEXT layer's router.
//   barrier
//
// Every wait is bounded: a barrier or copy that does not complete within ~2 s sets a bit in the
// status word, every CTA sees it at its next wait and returns.
#include <cuda.h>

#include "moe_route.cuh"

namespace uocr {

constexpr int kDecThreads = 512;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kRowsA = 4;             // row pairs per warp in phase A (all resident in shared memory)
constexpr int kMaxRowsB = 9;          // output rows per CTA in phase B
constexpr long long kSpinLimit = 4000000000LL;   // cycles

constexpr uint32_t kStatusRouter = 1u, kStatusBarrier = 2u, kStatusCopy = 4u;

struct DecodeParams {
    const DLayer *layers;
    uint32_t first, count;
    const __half *hidden_in;
    const __half *residual0;      // residual of the first layer (may be null)
    int chain_residual;           // layers after the first use their input as residual
    const float *injected;        // [E] logits for the first layer, or null
    __half *out;
    __half *hbuf0, *hbuf1;        // [H] ping-pong
    __half *mid;                  // [K*F + S]
    float *plogits;               // [G][E]
    unsigned long long *bar;
    unsigned long long bar_base;
    uint32_t *status;
    float *dbg_logits, *dbg_probs;
    uint32_t *ids_out;            // [K] routing of the last layer run
    float *wts_out;
};

// ---------------------------------------------------------------- small PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// 1-D bulk copy global -> shared; size and both addresses are multiples of 16 bytes
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add_u64(unsigned long long *p, unsigned long long v) {
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Bounded wait on an mbarrier phase.  Returns false after the limit (status bit set).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t *status) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > kSpinLimit) {
            atomicOr(status, kStatusCopy);
            // one more bounded wait so that the copy does not land after this CTA has gone
            const long long t1 = clock64();
            while (!mbar_try_wait(bar, parity) && clock64() - t1 < kSpinLimit) {}
            return false;
        }
    }
    return true;
}

// Grid-wide barrier over a monotonic counter.  All CTAs are co-resident (cooperative launch).
__device__ __forceinline__ bool grid_barrier(unsigned long long *ctr, unsigned long long target, uint32_t *status,
                                             int *s_flag) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        red_release_add_u64(ctr, 1ULL);
        int ok = 1;
        const long long t0 = clock64();
        while (ld_acquire_u64(ctr) < target) {
            if (ld_volatile_u32(status) & (kStatusBarrier | kStatusCopy)) { ok = 0; break; }
            if (clock64() - t0 > kSpinLimit) { atomicOr(status, kStatusBarrier); ok = 0; break; }
        }
        if (ld_volatile_u32(status) & (kStatusBarrier | kStatusCopy)) ok = 0;   // a copy of this CTA timed out
        *s_flag = ok;
    }
    __syncthreads();
    return *s_flag != 0;
}

// ---------------------------------------------------------------- 4-byte word dot products
// One 32-bit word of a packed row against activations held in registers.  Levels are turned into
// f32 exactly by planting the byte in the mantissa of 2^23 and subtracting the offset.
template <int QT> struct WordTraits;
template <> struct WordTraits<UOCR_QT_Q4> { static constexpr int kVals = 8; static constexpr int kWordsPerGroup = 8; };
template <> struct WordTraits<UOCR_QT_Q8> { static constexpr int kVals = 4; static constexpr int kWordsPerGroup = 16; };

__device__ __forceinline__ float byte_to_f32(uint32_t bytes, int b, float offset) {
    // result = [byte b, 0, 0, 0x4B] = 2^23 + byte; minus (2^23 + bias)
    return __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7540u + b)) - offset;
}

// x: kVals activations for this word (Q4: 4 for the low nibbles then 4 for the high nibbles)
template <int QT>
__device__ __forceinline__ float word_dot(uint32_t w, const float *x) {
    float s = 0.f;
    if (QT == UOCR_QT_Q4) {
        const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int b = 0; b < 4; ++b) s = fmaf(byte_to_f32(lo, b, 8388616.f), x[b], s);
#pragma unroll
        for (int b = 0; b < 4; ++b) s = fmaf(byte_to_f32(hi, b, 8388616.f), x[4 + b], s);
    } else {
        const uint32_t u = w ^ 0x80808080u;       // int8 + 128 as unsigned bytes
#pragma unroll
        for (int b = 0; b < 4; ++b) s = fmaf(byte_to_f32(u, b, 8388736.f), x[b], s);
    }
    return s;
}

// first activation column covered by word c of a row (Q4: the low-nibble half; the high half is +32)
template <int QT>
__device__ __forceinline__ int word_col(int c) {
    return QT == UOCR_QT_Q4 ? ((c >> 3) << 6) + ((c & 7) << 2) : (c << 2);
}

// Activations, SwiGLU products and partial logits are written by other CTAs during the kernel: they are
// read with ld.global.cg (L2), never through the non-coherent L1.
__device__ __forceinline__ void load4h(const __half *p, float *dst) {
    const uint2 v = __ldcg(reinterpret_cast<const uint2 *>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
    dst[0] = a.x; dst[1] = a.y; dst[2] = b.x; dst[3] = b.y;
}

template <int QT>
__device__ __forceinline__ void load_word_acts(const __half *x, int c, float *dst) {
    const int col = word_col<QT>(c);
    load4h(x + col, dst);
    if (QT == UOCR_QT_Q4) load4h(x + col + 32, dst + 4);
}

// ---------------------------------------------------------------- the kernel
template <int QT, int H, int F, int S>
__global__ void __launch_bounds__(kDecThreads, 1) decode_stack_kernel(DecodeParams prm) {
    using WT = WordTraits<QT>;
    constexpr int kRowBytesH = QT == UOCR_QT_Q4 ? H / 2 : H;       // gate/up row
    constexpr int kWordsH = kRowBytesH / 4;
    constexpr int kWA = kWordsH / 32;                               // words per lane per gate/up row
    static_assert(kWordsH % 32 == 0, "hidden size must fill whole warps of 4-byte words");
    constexpr int kXA = kWA * WT::kVals;                            // activations per lane
    constexpr int kRowBytesF = QT == UOCR_QT_Q4 ? F / 2 : F;        // routed down row
    constexpr int kRowBytesS = QT == UOCR_QT_Q4 ? S / 2 : S;        // shared down row
    constexpr int kWordsF = kRowBytesF / 4, kWordsSh = kRowBytesS / 8;   // words per job (shared split in halves)
    constexpr int kWB = (((kWordsF > kWordsSh ? kWordsF : kWordsSh) + 31) / 32);
    constexpr int kScaleRowBytes = (H / UOCR_GROUP) * 2;             // fp16 scales of one gate/up row
    constexpr int kScaleWin = 64;                                    // 16-byte aligned window that holds them
    static_assert(kScaleRowBytes + 8 <= kScaleWin, "scale window too small");
    constexpr int kSlotBytes = 2 * kRowBytesH + 2 * kScaleWin;       // gate row | up row | gate scales | up scales
    constexpr int kMaxE = 256, kMaxK = 16;

    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t *slots = smem_raw;                                                     // [warps][kRowsA][kSlotBytes]
    uint64_t *bars = reinterpret_cast<uint64_t *>(slots + (size_t)kDecWarps * kRowsA * kSlotBytes);   // [warps][kRowsA]
    float *s_logits = reinterpret_cast<float *>(bars + kDecWarps * kRowsA);        // [kMaxE]
    float *s_probs = s_logits + kMaxE;                                             // [kMaxE]
    float *s_red = s_probs + kMaxE;                                                // [8][kMaxE]
    float *s_dots = s_red + 8 * kMaxE;                                             // [kMaxRowsB][kMaxK + 2]
    uint32_t *s_ids = reinterpret_cast<uint32_t *>(s_dots + kMaxRowsB * (kMaxK + 2));   // [kMaxK]
    float *s_wts = reinterpret_cast<float *>(s_ids + kMaxK);                       // [kMaxK]
    float *s_hn = s_wts + kMaxK;                                                   // [kMaxRowsB]
    int *s_flag = reinterpret_cast<int *>(s_hn + kMaxRowsB + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t G = gridDim.x, cta = blockIdx.x;
    unsigned long long bar_target = prm.bar_base;
    uint32_t *status = prm.status;

    if (lane == 0) {
        for (int j = 0; j < kRowsA; ++j) mbar_init(&bars[warp * kRowsA + j], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // rows of phase B owned by this CTA
    const uint32_t hb0 = (uint32_t)(((uint64_t)cta * H) / G), hb1 = (uint32_t)(((uint64_t)(cta + 1) * H) / G);
    const uint32_t nrb = hb1 - hb0;

    const __half *cur = prm.hidden_in;
    uint32_t phase_bits = 0;      // bit j: parity of the next completion of this warp's slot j

    // ---- prologue: partial logits of the first layer over this CTA's slice of the input
    {
        const DLayer &L0 = prm.layers[prm.first];
        if (prm.injected == nullptr && (uint32_t)tid < L0.E) {
            float acc = 0.f;
            for (uint32_t r = 0; r < nrb; ++r)
                acc = fmaf(__half2float(cur[hb0 + r]), __half2float(L0.router[(size_t)tid * H + hb0 + r]), acc);
            prm.plogits[(size_t)cta * L0.E + tid] = acc;
        }
        bar_target += G;
        if (!grid_barrier(prm.bar, bar_target, status, s_flag)) return;
    }

    for (uint32_t li = 0; li < prm.count; ++li) {
        const DLayer &L = prm.layers[prm.first + li];
        const uint32_t E = L.E, K = L.K;
        const bool last = li + 1 == prm.count;
        __half *next = last ? prm.out : ((li & 1) ? prm.hbuf1 : prm.hbuf0);
        const __half *residual = li == 0 ? prm.residual0 : (prm.chain_residual ? cur : nullptr);

        // ---- activations of this lane's words (same columns for every gate/up row)
        float xa[kXA];
#pragma unroll
        for (int k = 0; k < kWA; ++k) load_word_acts<QT>(cur, lane + 32 * k, xa + k * WT::kVals);

        // ---- router logits: fixed-order sum of the per-CTA partials
        if (li == 0 && prm.injected != nullptr) {
            if ((uint32_t)tid < E) s_logits[tid] = prm.injected[tid] + (L.bias ? L.bias[tid] : 0.f);
        } else {
            const uint32_t parts = kDecThreads / E >= 8 ? 8 : (kDecThreads / E);   // E <= 256 -> >= 2
            const uint32_t e = tid % E, part = tid / E;
            if (part < parts) {
                const uint32_t per = (G + parts - 1) / parts;
                const uint32_t c0 = part * per, c1 = min(G, c0 + per);
                float acc = 0.f;
                for (uint32_t c = c0; c < c1; ++c) acc += __ldcg(&prm.plogits[(size_t)c * E + e]);
                s_red[part * kMaxE + e] = acc;
            }
            __syncthreads();
            if ((uint32_t)tid < E) {
                float acc = 0.f;
                for (uint32_t q = 0; q < parts; ++q) acc += s_red[q * kMaxE + tid];
                s_logits[tid] = L.bias ? acc + L.bias[tid] : acc;
            }
        }
        __syncthreads();
        if (warp == 0) {
            const bool dbg = cta == 0 && li == 0;
            const bool bad = route_row_warp(s_logits, s_probs, E, K, L.scaling, lane, dbg ? prm.dbg_logits : nullptr,
                                            dbg ? prm.dbg_probs : nullptr, s_ids, s_wts);
            if (bad && lane == 0 && cta == 0) atomicOr(status, kStatusRouter);
        }
        __syncthreads();
        if (cta == 0 && last && (uint32_t)tid < K) {
            prm.ids_out[tid] = s_ids[tid];
            prm.wts_out[tid] = s_wts[tid];
        }

        // ---- phase A: this warp's (gate, up) row pairs
        const uint32_t P = K * F + S;
        const uint32_t pa0 = (uint32_t)(((uint64_t)cta * P) / G), pa1 = (uint32_t)(((uint64_t)(cta + 1) * P) / G);
        const uint8_t *gsrc[kRowsA];
        const uint8_t *gscale[kRowsA];      // byte address of the row's gate scales
        uint32_t up_off_b[kRowsA], up_off_s[kRowsA];   // bytes from gate to up: packed rows, scales
        bool row_ok[kRowsA];
#pragma unroll
        for (int j = 0; j < kRowsA; ++j) {
            const uint32_t p = pa0 + warp + kDecWarps * j;
            row_ok[j] = p < pa1;
            gsrc[j] = nullptr; gscale[j] = nullptr; up_off_b[j] = 0; up_off_s[j] = 0;
            if (row_ok[j]) {
                if (p < K * F) {
                    const uint32_t slot = p / F, row = p - slot * F, ex = s_ids[slot];
                    if (ex < E) {
                        gsrc[j] = L.expert_w + (size_t)ex * L.expert_stride_bytes + (size_t)row * kRowBytesH;
                        gscale[j] = reinterpret_cast<const uint8_t *>(L.expert_s + (size_t)ex * L.expert_scale_stride) +
                                    (size_t)row * kScaleRowBytes;
                        up_off_b[j] = (uint32_t)L.up_offset_bytes;
                        up_off_s[j] = (uint32_t)L.up_scale_offset * 2u;
                    }
                } else {
                    const uint32_t row = p - K * F;
                    gsrc[j] = L.shared_gate.w + (size_t)row * kRowBytesH;
                    gscale[j] = reinterpret_cast<const uint8_t *>(L.shared_gate.s) + (size_t)row * kScaleRowBytes;
                    up_off_b[j] = (uint32_t)(L.shared_up.w - L.shared_gate.w);
                    up_off_s[j] = (uint32_t)(L.shared_up.s - L.shared_gate.s) * 2u;
                }
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < kRowsA; ++j) {
                if (gsrc[j] != nullptr) {
                    uint64_t *bar = &bars[warp * kRowsA + j];
                    uint8_t *dst = slots + ((size_t)warp * kRowsA + j) * kSlotBytes;
                    // scale rows start on 8-byte boundaries: copy the enclosing 16-byte aligned window
                    // (weight buffers are over-allocated, so the window never leaves the allocation)
                    const uint8_t *gs = gscale[j], *us = gscale[j] + up_off_s[j];
                    mbar_expect_tx(bar, kSlotBytes);
                    bulk_g2s(dst, gsrc[j], kRowBytesH, bar);
                    bulk_g2s(dst + kRowBytesH, gsrc[j] + up_off_b[j], kRowBytesH, bar);
                    bulk_g2s(dst + 2 * kRowBytesH, gs - ((uintptr_t)gs & 15), kScaleWin, bar);
                    bulk_g2s(dst + 2 * kRowBytesH + kScaleWin, us - ((uintptr_t)us & 15), kScaleWin, bar);
                }
            }
        }

        // ---- phase B loads that do not depend on phase A: packed down rows of this warp's jobs
        // job q -> (row r, source s); sources 0..K-1 routed, K and K+1 the two halves of the shared MLP
        const uint32_t n_src = K + 2, n_jobs = nrb * n_src;
        constexpr int kJobs = (kMaxRowsB * (kMaxK + 2) + kDecWarps - 1) / kDecWarps;   // upper bound, trimmed below
        constexpr int kJ = kJobs > 5 ? 5 : kJobs;      // K <= 6 at these shapes: 9 rows * 8 sources / 16 warps
        uint32_t dw[kJ][kWB];
        __half dsc[kJ][kWB];
#pragma unroll
        for (int j = 0; j < kJ; ++j) {
            const uint32_t q = warp + kDecWarps * j;
#pragma unroll
            for (int k = 0; k < kWB; ++k) { dw[j][k] = 0; dsc[j][k] = __ushort_as_half(0); }
            if (q < n_jobs) {
                const uint32_t r = q / n_src, s = q - r * n_src, h = hb0 + r;
                const uint8_t *wrow = nullptr;
                const __half *srow = nullptr;
                uint32_t words = 0, word0 = 0;
                if (s < K) {
                    const uint32_t ex = s_ids[s];
                    if (ex < E) {
                        wrow = L.expert_w + (size_t)ex * L.expert_stride_bytes + L.down_offset_bytes + (size_t)h * kRowBytesF;
                        srow = L.expert_s + (size_t)ex * L.expert_scale_stride + L.down_scale_offset + (size_t)h * (F / UOCR_GROUP);
                        words = kWordsF;
                    }
                } else {
                    wrow = L.shared_down.w + (size_t)h * kRowBytesS;
                    srow = L.shared_down.s + (size_t)h * (S / UOCR_GROUP);
                    words = kWordsSh;
                    word0 = (s - K) * kWordsSh;
                }
                if (wrow != nullptr) {
#pragma unroll
                    for (int k = 0; k < kWB; ++k) {
                        const uint32_t c = lane + 32 * k;
                        if (c < words) {
                            dw[j][k] = __ldg(reinterpret_cast<const uint32_t *>(wrow) + word0 + c);
                            dsc[j][k] = srow[(word0 + c) / WT::kWordsPerGroup];
                        }
                    }
                }
            }
        }
        // router row slice of the next layer for the partial logits
        float rn[kMaxRowsB];
#pragma unroll
        for (int r = 0; r < kMaxRowsB; ++r) rn[r] = 0.f;
        if (!last) {
            const DLayer &Ln = prm.layers[prm.first + li + 1];
            if ((uint32_t)tid < Ln.E) {
#pragma unroll
                for (int r = 0; r < kMaxRowsB; ++r)
                    if ((uint32_t)r < nrb) rn[r] = __half2float(Ln.router[(size_t)tid * H + hb0 + r]);
            }
        }

        // ---- phase A compute
#pragma unroll
        for (int j = 0; j < kRowsA; ++j) {
            if (!row_ok[j]) continue;
            const uint32_t p = pa0 + warp + kDecWarps * j;
            float mid_v = 0.f;
            if (gsrc[j] != nullptr) {
                const bool got = mbar_wait(&bars[warp * kRowsA + j], (phase_bits >> j) & 1u, status);
                phase_bits ^= 1u << j;
                if (got) {
                    const uint8_t *slot = slots + ((size_t)warp * kRowsA + j) * kSlotBytes;
                    const uint32_t *gw = reinterpret_cast<const uint32_t *>(slot);
                    const uint32_t *uw = gw + kWordsH;
                    const uint8_t *gs = gscale[j], *us = gscale[j] + up_off_s[j];
                    const __half *sgp = reinterpret_cast<const __half *>(slot + 2 * kRowBytesH + ((uintptr_t)gs & 15));
                    const __half *sup = reinterpret_cast<const __half *>(slot + 2 * kRowBytesH + kScaleWin + ((uintptr_t)us & 15));
                    float ga = 0.f, ua = 0.f;
#pragma unroll
                    for (int k = 0; k < kWA; ++k) {
                        const int g = (lane + 32 * k) / WT::kWordsPerGroup;
                        ga = fmaf(word_dot<QT>(gw[lane + 32 * k], xa + k * WT::kVals), __half2float(sgp[g]), ga);
                        ua = fmaf(word_dot<QT>(uw[lane + 32 * k], xa + k * WT::kVals), __half2float(sup[g]), ua);
                    }
                    ga = warp_sum(ga);
                    ua = warp_sum(ua);
                    mid_v = silu_f32(ga) * ua;
                }
            }
            if (lane == 0) prm.mid[p] = __float2half_rn(mid_v);     // an invalid expert id contributes zeros
        }
        bar_target += G;
        if (!grid_barrier(prm.bar, bar_target, status, s_flag)) return;

        // ---- phase B compute
#pragma unroll
        for (int j = 0; j < kJ; ++j) {
            const uint32_t q = warp + kDecWarps * j;
            if (q >= n_jobs) continue;
            const uint32_t r = q / n_src, s = q - r * n_src;
            const __half *m = s < K ? prm.mid + (size_t)s * F : prm.mid + (size_t)K * F + (size_t)(s - K) * (S / 2);
            const uint32_t words = s < K ? kWordsF : kWordsSh;
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < kWB; ++k) {
                const uint32_t c = lane + 32 * k;
                if (c < words) {
                    float mv[WT::kVals];
                    load_word_acts<QT>(m, (int)c, mv);
                    acc = fmaf(word_dot<QT>(dw[j][k], mv), __half2float(dsc[j][k]), acc);
                }
            }
            acc = warp_sum(acc);
            if (lane == 0) s_dots[r * (kMaxK + 2) + s] = acc;
        }
        __syncthreads();
        if ((uint32_t)tid < nrb) {
            const uint32_t h = hb0 + tid;
            float acc = 0.f;
            for (uint32_t s = 0; s < K; ++s)
                if (s_ids[s] < E) acc = fmaf(s_wts[s], s_dots[tid * (kMaxK + 2) + s], acc);
            acc += s_dots[tid * (kMaxK + 2) + K] + s_dots[tid * (kMaxK + 2) + K + 1];
            if (residual) acc += __half2float(__ldcg(reinterpret_cast<const __half *>(residual + h)));
            const __half o = __float2half_rn(acc);
            next[h] = o;
            s_hn[tid] = __half2float(o);
        }
        __syncthreads();
        if (!last) {
            const uint32_t En = prm.layers[prm.first + li + 1].E;
            if ((uint32_t)tid < En) {
                float acc = 0.f;
#pragma unroll
                for (int r = 0; r < kMaxRowsB; ++r)
                    if ((uint32_t)r < nrb) acc = fmaf(s_hn[r], rn[r], acc);
                prm.plogits[(size_t)cta * En + tid] = acc;
            }
            bar_target += G;
            if (!grid_barrier(prm.bar, bar_target, status, s_flag)) return;
        }
        cur = next;
    }
}

// ---------------------------------------------------------------- host side
template <int QT>
static size_t decode_smem_bytes(int H) {
    const size_t slot = 2 * (size_t)(QT == UOCR_QT_Q4 ? H / 2 : H) + 2 * 64;
    return (size_t)kDecWarps * kRowsA * slot + kDecWarps * kRowsA * 8 + sizeof(float) * (256 * 10 + kMaxRowsB * 18 + 64) + 256;
}

struct DecodeShape { int qt, H, F, S; };

static bool shape_supported(const DLayer &L) {
    return (L.expert_qtype == UOCR_QT_Q4 || L.expert_qtype == UOCR_QT_Q8) && L.shared_gate.qtype == L.expert_qtype &&
           L.shared_down.qtype == L.expert_qtype && L.H == 1280 && L.F == 896 && L.S == 1792 && L.K <= 6 && L.E <= 256;
}

static int g_decode_grid[64] = {0};

template <int QT>
static cudaError_t prepare_decode(int dev) {
    auto kern = decode_stack_kernel<QT, 1280, 896, 1792>;
    const size_t smem = decode_smem_bytes<QT>(1280);
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    int per_sm = 0, sms = 0;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kDecThreads, smem);
    if (err != cudaSuccess) return err;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return err;
    const int grid = per_sm >= 1 ? sms : 0;
    if (dev < 64 && (g_decode_grid[dev] == 0 || grid < g_decode_grid[dev])) g_decode_grid[dev] = grid;
    return cudaSuccess;
}

cudaError_t init_decode_kernels() {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 64) g_decode_grid[dev] = 0;
    err = prepare_decode<UOCR_QT_Q4>(dev);
    if (err != cudaSuccess) return err;
    return prepare_decode<UOCR_QT_Q8>(dev);
}

// Number of CTAs the decode kernel runs with on the current device, 0 when it cannot run there.
int decode_grid_size() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev >= 64) return 0;
    return g_decode_grid[dev];
}

bool decode_supported(const DLayer *layers, uint32_t first, uint32_t count) {
    const int G = decode_grid_size();
    if (G <= 0) return false;
    for (uint32_t i = 0; i < count; ++i) {
        const DLayer &L = layers[first + i];
        if (!shape_supported(L) || L.expert_qtype != layers[first].expert_qtype) return false;
        const uint32_t P = L.K * L.F + L.S;
        if ((P + G - 1) / G > (uint32_t)(kDecWarps * kRowsA) || (L.H + G - 1) / G > (uint32_t)kMaxRowsB) return false;
    }
    return true;
}

// h_layers: host copies (for shape checks); d_layers: the same table in device memory.
cudaError_t launch_decode_stack(const DLayer *h_layers, const DLayer *d_layers, uint32_t first, uint32_t count,
                                const __half *hidden, const __half *residual0, int chain_residual,
                                const float *injected, __half *out, __half *hbuf0, __half *hbuf1, __half *mid,
                                float *plogits, unsigned long long *bar, unsigned long long *bar_base, uint32_t *status,
                                float *dbg_logits, float *dbg_probs, uint32_t *ids_out, float *wts_out,
                                cudaStream_t st, uint64_t *launches) {
    const int G = decode_grid_size();
    if (G <= 0) return cudaErrorNotSupported;
    DecodeParams prm{};
    prm.layers = d_layers; prm.first = first; prm.count = count;
    prm.hidden_in = hidden; prm.residual0 = residual0; prm.chain_residual = chain_residual;
    prm.injected = injected; prm.out = out; prm.hbuf0 = hbuf0; prm.hbuf1 = hbuf1; prm.mid = mid;
    prm.plogits = plogits; prm.bar = bar; prm.bar_base = *bar_base; prm.status = status;
    prm.dbg_logits = dbg_logits; prm.dbg_probs = dbg_probs; prm.ids_out = ids_out; prm.wts_out = wts_out;
    void *args[] = {&prm};
    cudaError_t err;
    if (h_layers[first].expert_qtype == UOCR_QT_Q4) {
        err = cudaLaunchCooperativeKernel((const void *)decode_stack_kernel<UOCR_QT_Q4, 1280, 896, 1792>, dim3(G),
                                          dim3(kDecThreads), args, decode_smem_bytes<UOCR_QT_Q4>(1280), st);
    } else {
        err = cudaLaunchCooperativeKernel((const void *)decode_stack_kernel<UOCR_QT_Q8, 1280, 896, 1792>, dim3(G),
                                          dim3(kDecThreads), args, decode_smem_bytes<UOCR_QT_Q8>(1280), st);
    }
    if (err != cudaSuccess) return err;
    // barriers passed: prologue + two per layer, except the last layer's second one
    *bar_base += (unsigned long long)G * (1ull + 2ull * count - 1ull);
    ++*launches;
    return cudaSuccess;
}

}  // namespace uocr

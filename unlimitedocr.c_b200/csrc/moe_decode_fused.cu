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
#include "moe_sync.cuh"

namespace uocr {

constexpr int kDecThreads = 512;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kRowsA = 4;             // row pairs per warp in phase A (all resident in shared memory)
constexpr int kMaxRowsB = 9;          // output rows per CTA in phase B

constexpr int kTracePoints = 8;

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
    unsigned long long *trace;    // optional [count][kTracePoints] SM-clock stamps of CTA 0 (profiling detail)
};

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

// Shared-memory layout: row-pair slots, their mbarriers, the small float arrays, the activations and
// finally the copy of the layer table (offset computed here for the kernel and for the host's size query).
__host__ __device__ constexpr int decode_layer_table_offset(int slot_bytes, int H) {
    return ((kDecWarps * kRowsA * slot_bytes + kDecWarps * kRowsA * 8 + 4 * (256 * 10 + kMaxRowsB * 8 + 64) + 2 * H) + 15) / 16 * 16;
}

// ---------------------------------------------------------------- the kernel
// Interleaved butterfly reduction of N per-lane values (one tree latency instead of N).
template <int N>
__device__ __forceinline__ void warp_sum_n(float (&v)[N]) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float t[N];
#pragma unroll
        for (int i = 0; i < N; ++i) t[i] = __shfl_xor_sync(0xffffffffu, v[i], o);
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] += t[i];
    }
}

template <int QT, int H, int F, int S>
__global__ void __launch_bounds__(kDecThreads, 1) decode_stack_kernel(DecodeParams prm) {
    using WT = WordTraits<QT>;
    constexpr int K = 6;                                            // top-k of the model; K + 2 sources = 8
    constexpr int kSrc = K + 2;
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
    constexpr int kMaxE = 256;
    constexpr int kJ = (kMaxRowsB * kSrc + kDecWarps - 1) / kDecWarps;   // phase-B jobs per warp (5)
    static_assert(kDecWarps % kSrc == 0, "every job of a warp must have the same source");

    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t *slots = smem_raw;                                                     // [warps][kRowsA][kSlotBytes]
    uint64_t *bars = reinterpret_cast<uint64_t *>(slots + (size_t)kDecWarps * kRowsA * kSlotBytes);   // [warps][kRowsA]
    float *s_logits = reinterpret_cast<float *>(bars + kDecWarps * kRowsA);        // [kMaxE]
    float *s_probs = s_logits + kMaxE;                                             // [kMaxE]
    float *s_red = s_probs + kMaxE;                                                // [8][kMaxE]
    float *s_dots = s_red + 8 * kMaxE;                                             // [kMaxRowsB][kSrc]
    uint32_t *s_ids = reinterpret_cast<uint32_t *>(s_dots + kMaxRowsB * kSrc);     // [16]
    float *s_wts = reinterpret_cast<float *>(s_ids + 16);                          // [16]
    float *s_hn = s_wts + 16;                                                      // [kMaxRowsB + 1]
    int *s_flag = reinterpret_cast<int *>(s_hn + kMaxRowsB + 1);
    __half *s_x = reinterpret_cast<__half *>(s_flag + 2);                          // [H] current activations
    __shared__ uint64_t s_tab[UOCR_EXPF_N];                                        // table of the router's exp()
    if (threadIdx.x < UOCR_EXPF_N) s_tab[threadIdx.x] = c_exp_tab[threadIdx.x];
    DLayer *s_layers = reinterpret_cast<DLayer *>(smem_raw + decode_layer_table_offset(kSlotBytes, H));

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t G = gridDim.x, cta = blockIdx.x;
    unsigned long long bar_target = prm.bar_base;
    uint32_t *status = prm.status;

    if (tid == 0) { s_flag[0] = 1; s_flag[1] = 0; }
    if (lane == 0) {
        for (int j = 0; j < kRowsA; ++j) mbar_init(&bars[warp * kRowsA + j], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    {   // the layer descriptors are read many times per layer: keep them in shared memory
        const uint32_t words = prm.count * (uint32_t)(sizeof(DLayer) / 4);
        const uint32_t *src = reinterpret_cast<const uint32_t *>(prm.layers + prm.first);
        uint32_t *dst = reinterpret_cast<uint32_t *>(s_layers);
        for (uint32_t i = tid; i < words; i += kDecThreads) dst[i] = src[i];
    }
    __syncthreads();

    // ---- work that is the same for every layer
    // phase B: output rows of this CTA; job j of this warp is row rB[j] of source sB
    const uint32_t hb0 = (uint32_t)(((uint64_t)cta * H) / G), hb1 = (uint32_t)(((uint64_t)(cta + 1) * H) / G);
    const uint32_t nrb = hb1 - hb0;
    const uint32_t sB = warp % kSrc;
    const uint32_t wordsB = sB < K ? kWordsF : kWordsSh;
    const uint32_t word0B = sB < K ? 0u : (sB - K) * kWordsSh;
    // phase A: row pairs [pa0, pa1) of the K*F + S pairs; this warp takes pa0 + warp + 16 j
    constexpr uint32_t P = K * F + S;
    const uint32_t pa0 = (uint32_t)(((uint64_t)cta * P) / G), pa1 = (uint32_t)(((uint64_t)(cta + 1) * P) / G);
    uint32_t a_slot[kRowsA], a_row[kRowsA];       // a_slot == K: shared MLP; 0xffffffff: no row
#pragma unroll
    for (int j = 0; j < kRowsA; ++j) {
        const uint32_t p = pa0 + warp + kDecWarps * j;
        if (p >= pa1) { a_slot[j] = 0xffffffffu; a_row[j] = 0; }
        else if (p < K * F) { a_slot[j] = p / F; a_row[j] = p - a_slot[j] * F; }
        else { a_slot[j] = K; a_row[j] = p - K * F; }
    }

    const __half *cur = prm.hidden_in;
    uint32_t phase_bits = 0;      // bit j: parity of the next completion of this warp's slot j

    // ---- prologue: partial logits of the first layer over this CTA's slice of the input
    {
        const DLayer &L0 = s_layers[0];
        if (prm.injected == nullptr && (uint32_t)tid < L0.E) {
            float acc = 0.f;
            for (uint32_t r = 0; r < nrb; ++r)
                acc = fmaf(__half2float(cur[hb0 + r]), __half2float(L0.router[(size_t)tid * H + hb0 + r]), acc);
            prm.plogits[(size_t)cta * L0.E + tid] = acc;
        }
        bar_target += G;
        if (!grid_barrier(prm.bar, bar_target, status, s_flag)) return;
    }

#define UOCR_TRACE(point)                                                                                       \
    do {                                                                                                        \
        if (prm.trace != nullptr && cta == 0 && tid == 0) prm.trace[li * kTracePoints + (point)] = clock64();   \
    } while (0)

    for (uint32_t li = 0; li < prm.count; ++li) {
        const DLayer &L = s_layers[li];
        UOCR_TRACE(0);   // layer start
        const uint32_t E = L.E;
        const bool last = li + 1 == prm.count;
        __half *next = last ? prm.out : ((li & 1) ? prm.hbuf1 : prm.hbuf0);
        const __half *residual = li == 0 ? prm.residual0 : (prm.chain_residual ? cur : nullptr);

        // ---- inputs: the activations once per CTA into shared memory, and the fixed-order sum of the
        // per-CTA partial router logits
        if (tid < H / 4) reinterpret_cast<uint2 *>(s_x)[tid] = __ldcg(reinterpret_cast<const uint2 *>(cur) + tid);
        if (li == 0 && prm.injected != nullptr) {
            if ((uint32_t)tid < E) s_logits[tid] = prm.injected[tid] + (L.bias ? L.bias[tid] : 0.f);
            __syncthreads();
        } else {
            const uint32_t parts = kDecThreads / E >= 8 ? 8 : (kDecThreads / E);   // E <= 256 -> >= 2
            const uint32_t e = tid % E, part = tid / E;
            if (part < parts) {
                const uint32_t per = (G + parts - 1) / parts;
                const uint32_t c0 = part * per, c1 = min(G, c0 + per);
                // all loads of a batch are issued before the first add; the adds keep CTA order
                float acc = 0.f;
                for (uint32_t cb = c0; cb < c1; cb += 32) {
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = cb + i < c1 ? __ldcg(&prm.plogits[(size_t)(cb + i) * E + e]) : 0.f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc += v[i];
                }
                s_red[part * kMaxE + e] = acc;
            }
            __syncthreads();
            if ((uint32_t)tid < E) {
                float acc = 0.f;
                for (uint32_t q = 0; q < parts; ++q) acc += s_red[q * kMaxE + tid];
                s_logits[tid] = L.bias ? acc + L.bias[tid] : acc;
            }
            __syncthreads();
        }
        UOCR_TRACE(1);   // activations and logits in

        // ---- routing by warp 0; the other warps meanwhile start everything that does not need the ids
        if (warp == 0) {
            const bool dbg = cta == 0 && li == 0;
            const bool bad = route_row_warp(s_logits, s_probs, E, K, L.scaling, lane, s_tab, dbg ? prm.dbg_logits : nullptr,
                                            dbg ? prm.dbg_probs : nullptr, s_ids, s_wts);
            if (bad && lane == 0 && cta == 0) atomicOr(status, kStatusRouter);
        }
        // activations of this lane's words (same columns for every gate/up row)
        float xa[kXA];
#pragma unroll
        for (int k = 0; k < kWA; ++k) {
            const int col = word_col<QT>(lane + 32 * k);
            const uint2 v0 = *reinterpret_cast<const uint2 *>(s_x + col);
            const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v0.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&v0.y));
            xa[k * WT::kVals + 0] = a.x; xa[k * WT::kVals + 1] = a.y; xa[k * WT::kVals + 2] = b.x; xa[k * WT::kVals + 3] = b.y;
            if (QT == UOCR_QT_Q4) {
                const uint2 v1 = *reinterpret_cast<const uint2 *>(s_x + col + 32);
                const float2 c = __half22float2(*reinterpret_cast<const __half2 *>(&v1.x));
                const float2 d = __half22float2(*reinterpret_cast<const __half2 *>(&v1.y));
                xa[k * WT::kVals + 4] = c.x; xa[k * WT::kVals + 5] = c.y; xa[k * WT::kVals + 6] = d.x; xa[k * WT::kVals + 7] = d.y;
            }
        }
        // router row slice of the next layer for this CTA's partial logits
        float rn[kMaxRowsB];
#pragma unroll
        for (int r = 0; r < kMaxRowsB; ++r) rn[r] = 0.f;
        if (!last) {
            const DLayer &Ln = s_layers[li + 1];
            if ((uint32_t)tid < Ln.E) {
#pragma unroll
                for (int r = 0; r < kMaxRowsB; ++r)
                    if ((uint32_t)r < nrb) rn[r] = __half2float(Ln.router[(size_t)tid * H + hb0 + r]);
            }
        }
        __syncthreads();     // ids and weights are in shared memory
        UOCR_TRACE(2);       // routing done
        if (cta == 0 && last && tid < K) {
            prm.ids_out[tid] = s_ids[tid];
            prm.wts_out[tid] = s_wts[tid];
        }

        // ---- phase A: issue the bulk copies of this warp's (gate, up) row pairs.  Lanes 4j..4j+3 issue the
        // four copies of row pair j (gate row, up row, gate scales, up scales) onto the pair's mbarrier.
        uint32_t issued = 0;          // bit j: a copy is in flight for slot j
        uint32_t sc_off[kRowsA];      // byte offsets of the gate / up scales inside their windows (low / high half)
        {
            const int j = lane >> 2, part = lane & 3;
            const uint8_t *src = nullptr;
            uint32_t bytes = 0, dst_off = 0;
#pragma unroll
            for (int jj = 0; jj < kRowsA; ++jj) {
                sc_off[jj] = 0;
                if (a_slot[jj] == 0xffffffffu) continue;
                const uint8_t *gw, *gs;
                uint32_t up_b, up_s;
                if (a_slot[jj] < K) {
                    const uint32_t ex = s_ids[a_slot[jj]];
                    if (ex >= E) continue;                      // an invalid expert id contributes zeros
                    gw = L.expert_w + (size_t)ex * L.expert_stride_bytes + (size_t)a_row[jj] * kRowBytesH;
                    gs = reinterpret_cast<const uint8_t *>(L.expert_s + (size_t)ex * L.expert_scale_stride) +
                         (size_t)a_row[jj] * kScaleRowBytes;
                    up_b = (uint32_t)L.up_offset_bytes;
                    up_s = (uint32_t)L.up_scale_offset * 2u;
                } else {
                    gw = L.shared_gate.w + (size_t)a_row[jj] * kRowBytesH;
                    gs = reinterpret_cast<const uint8_t *>(L.shared_gate.s) + (size_t)a_row[jj] * kScaleRowBytes;
                    up_b = (uint32_t)(L.shared_up.w - L.shared_gate.w);
                    up_s = (uint32_t)(L.shared_up.s - L.shared_gate.s) * 2u;
                }
                issued |= 1u << jj;
                const uint8_t *us = gs + up_s;
                sc_off[jj] = (uint32_t)((uintptr_t)gs & 15) | ((uint32_t)((uintptr_t)us & 15) << 16);
                if (jj == j) {
                    // scale rows start on 8-byte boundaries: copy the enclosing 16-byte aligned window
                    // (weight buffers are over-allocated, so the window never leaves the allocation)
                    if (part == 0) { src = gw; bytes = kRowBytesH; dst_off = 0; }
                    else if (part == 1) { src = gw + up_b; bytes = kRowBytesH; dst_off = kRowBytesH; }
                    else if (part == 2) { src = gs - ((uintptr_t)gs & 15); bytes = kScaleWin; dst_off = 2 * kRowBytesH; }
                    else { src = us - ((uintptr_t)us & 15); bytes = kScaleWin; dst_off = 2 * kRowBytesH + kScaleWin; }
                }
            }
            if (lane < kRowsA && ((issued >> lane) & 1u)) mbar_expect_tx(&bars[warp * kRowsA + lane], kSlotBytes);
            __syncwarp();
            if (lane < 4 * kRowsA && src != nullptr)
                bulk_g2s(slots + ((size_t)warp * kRowsA + j) * kSlotBytes + dst_off, src, bytes, &bars[warp * kRowsA + j]);
        }

        // ---- phase B loads that do not depend on phase A: packed down rows (and scales) of this warp's jobs
        uint32_t dw[kJ][kWB];
        __half dsc[kJ][kWB];
        {
            const uint8_t *wbase = nullptr;
            const __half *sbase = nullptr;
            uint32_t wrow_bytes = 0, srow_vals = 0;
            if (sB < K) {
                const uint32_t ex = s_ids[sB];
                if (ex < E) {
                    wbase = L.expert_w + (size_t)ex * L.expert_stride_bytes + L.down_offset_bytes;
                    sbase = L.expert_s + (size_t)ex * L.expert_scale_stride + L.down_scale_offset;
                    wrow_bytes = kRowBytesF; srow_vals = F / UOCR_GROUP;
                }
            } else {
                wbase = L.shared_down.w; sbase = L.shared_down.s;
                wrow_bytes = kRowBytesS; srow_vals = S / UOCR_GROUP;
            }
#pragma unroll
            for (int j = 0; j < kJ; ++j) {
                const uint32_t r = (warp + kDecWarps * j) / kSrc;
#pragma unroll
                for (int k = 0; k < kWB; ++k) {
                    const uint32_t c = lane + 32 * k;
                    dw[j][k] = 0; dsc[j][k] = __ushort_as_half(0);
                    if (wbase != nullptr && r < nrb && c < wordsB) {
                        const uint32_t h = hb0 + r;
                        dw[j][k] = __ldg(reinterpret_cast<const uint32_t *>(wbase + (size_t)h * wrow_bytes) + word0B + c);
                        dsc[j][k] = sbase[(size_t)h * srow_vals + (word0B + c) / WT::kWordsPerGroup];
                    }
                }
            }
        }
        UOCR_TRACE(3);   // copies and loads issued

        // ---- phase A compute: per-lane partial sums of every row pair, then one interleaved reduction
        float ga[kRowsA], ua[kRowsA];
#pragma unroll
        for (int j = 0; j < kRowsA; ++j) {
            ga[j] = 0.f; ua[j] = 0.f;
            if (!((issued >> j) & 1u)) continue;
            const bool got = mbar_wait(&bars[warp * kRowsA + j], (phase_bits >> j) & 1u, status, s_flag);
            phase_bits ^= 1u << j;
            if (!got) continue;
            const uint8_t *slot = slots + ((size_t)warp * kRowsA + j) * kSlotBytes;
            const uint32_t *gw = reinterpret_cast<const uint32_t *>(slot);
            const uint32_t *uw = gw + kWordsH;
            const __half *sgp = reinterpret_cast<const __half *>(slot + 2 * kRowBytesH + (sc_off[j] & 0xffffu));
            const __half *sup = reinterpret_cast<const __half *>(slot + 2 * kRowBytesH + kScaleWin + (sc_off[j] >> 16));
#pragma unroll
            for (int k = 0; k < kWA; ++k) {
                const int g = (lane + 32 * k) / WT::kWordsPerGroup;
                ga[j] = fmaf(word_dot<QT>(gw[lane + 32 * k], xa + k * WT::kVals), __half2float(sgp[g]), ga[j]);
                ua[j] = fmaf(word_dot<QT>(uw[lane + 32 * k], xa + k * WT::kVals), __half2float(sup[g]), ua[j]);
            }
        }
        {
            float red[2 * kRowsA];
#pragma unroll
            for (int j = 0; j < kRowsA; ++j) { red[2 * j] = ga[j]; red[2 * j + 1] = ua[j]; }
            warp_sum_n<2 * kRowsA>(red);
            // lane j stores row pair j (an unissued pair of a valid row stores zero)
#pragma unroll
            for (int j = 0; j < kRowsA; ++j)
                if (lane == j && a_slot[j] != 0xffffffffu)
                    prm.mid[pa0 + warp + kDecWarps * j] =
                        __float2half_rn(((issued >> j) & 1u) ? silu_f32(red[2 * j]) * red[2 * j + 1] : 0.f);
        }
        UOCR_TRACE(4);   // phase A computed
        bar_target += G;
        if (!grid_barrier(prm.bar, bar_target, status, s_flag)) return;
        UOCR_TRACE(5);   // barrier 1 passed

        // ---- phase B compute.  With K + 2 = 8 sources and 16 warps every job of a warp has the same
        // source, so its SwiGLU products are loaded once.
        {
            const __half *m = sB < K ? prm.mid + (size_t)sB * F : prm.mid + (size_t)K * F + (size_t)(sB - K) * (S / 2);
            float mv[kWB][WT::kVals];
#pragma unroll
            for (int k = 0; k < kWB; ++k) {
                const uint32_t c = lane + 32 * k;
                if (c < wordsB) load_word_acts<QT>(m, (int)c, mv[k]);
                else
#pragma unroll
                    for (int i = 0; i < WT::kVals; ++i) mv[k][i] = 0.f;
            }
            float acc[kJ];
#pragma unroll
            for (int j = 0; j < kJ; ++j) {
                acc[j] = 0.f;
#pragma unroll
                for (int k = 0; k < kWB; ++k) acc[j] = fmaf(word_dot<QT>(dw[j][k], mv[k]), __half2float(dsc[j][k]), acc[j]);
            }
            warp_sum_n<kJ>(acc);
            if (lane < kJ) {
                const uint32_t r = (warp + kDecWarps * lane) / kSrc;
                float v = 0.f;
#pragma unroll
                for (int j = 0; j < kJ; ++j)
                    if (lane == j) v = acc[j];
                if (r < nrb) s_dots[r * kSrc + sB] = v;
            }
        }
        __syncthreads();
        if ((uint32_t)tid < nrb) {
            const uint32_t h = hb0 + tid;
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < K; ++s)
                if (s_ids[s] < E) acc = fmaf(s_wts[s], s_dots[tid * kSrc + s], acc);
            acc += s_dots[tid * kSrc + K] + s_dots[tid * kSrc + K + 1];
            // the residual of a stacked layer is its input (already in shared memory)
            if (residual) acc += __half2float(li == 0 ? prm.residual0[h] : s_x[h]);
            const __half o = __float2half_rn(acc);
            next[h] = o;
            s_hn[tid] = __half2float(o);
        }
        __syncthreads();
        UOCR_TRACE(6);   // phase B computed
        if (!last) {
            const uint32_t En = s_layers[li + 1].E;
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
        UOCR_TRACE(7);   // barrier 2 passed
        cur = next;
    }
#undef UOCR_TRACE
}

// ---------------------------------------------------------------- host side
template <int QT>
static size_t decode_smem_bytes(int H) {
    const int slot = 2 * (QT == UOCR_QT_Q4 ? H / 2 : H) + 2 * 64;
    return (size_t)decode_layer_table_offset(slot, H) + 64 * sizeof(DLayer);
}

struct DecodeShape { int qt, H, F, S; };

static bool shape_supported(const DLayer &L) {
    return (L.expert_qtype == UOCR_QT_Q4 || L.expert_qtype == UOCR_QT_Q8) && L.shared_gate.qtype == L.expert_qtype &&
           L.shared_down.qtype == L.expert_qtype && L.H == 1280 && L.F == 896 && L.S == 1792 && L.K == 6 && L.E <= 256;
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
                                unsigned long long *trace, cudaStream_t st, uint64_t *launches) {
    const int G = decode_grid_size();
    if (G <= 0) return cudaErrorNotSupported;
    DecodeParams prm{};
    prm.layers = d_layers; prm.first = first; prm.count = count;
    prm.hidden_in = hidden; prm.residual0 = residual0; prm.chain_residual = chain_residual;
    prm.injected = injected; prm.out = out; prm.hbuf0 = hbuf0; prm.hbuf1 = hbuf1; prm.mid = mid;
    prm.plogits = plogits; prm.bar = bar; prm.bar_base = *bar_base; prm.status = status;
    prm.dbg_logits = dbg_logits; prm.dbg_probs = dbg_probs; prm.ids_out = ids_out; prm.wts_out = wts_out; prm.trace = trace;
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

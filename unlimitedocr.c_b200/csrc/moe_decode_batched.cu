// Batched decode: a few to a few dozen tokens per step (2 .. 64) at the model's shapes, Q4_0 / Q8_0.
//
// Such a step is bound by reading the weights of the experts it selects, once each.  Three launches:
//
// 1. route_small_kernel, one CTA per token: the 64 router logits (all loads of a warp's eight experts in flight at
//    once), the exact softmax / top-k, and the token's activations rewritten as block-floating-point bytes (two
//    signed bytes per value, one scale per 64-wide group) - the B operand of the integer MMAs, computed once per
//    token instead of once per expert that uses it.  The CTA that finishes last builds the dispatch plan (a stable
//    counting sort of the at most 384 pairs).
// 2. decode_batched_kernel, weight-stationary on the slice-major "unit blobs" of the single-token decode kernel.  A
//    work item is (expert, 16-token pass, one or two consecutive 64-wide slices of the intermediate dimension); the shared
//    MLP counts as two more experts that every token selects.  Items are listed hottest expert first and dealt
//    round-robin to one CTA per SM.  Per item the pass's activation bytes are copied into shared memory, then per slice
//    the 128 gate / up rows stream through a four-stage ring of bulk copies (one chunk = four quantisation groups) and
//    are multiplied with up to 16 tokens (a token occupies two of the MMA's eight columns, so one MMA covers four
//    tokens); the SwiGLU products never leave the SM: rounded to fp16, rewritten as bytes, multiplied with the
//    slice's 64 columns of `down` (held in registers).  The products, weighted with the slot's routing weight, are
//    added to the call's output sums: [token][H] 64-bit integers in 2^-28 fixed point (red.global.add.u64; the routing
//    kernel clears them).  Integer addition commutes: results are bit-reproducible whatever the order of the items.
// 3. finalize_batched_kernel converts the sums, adds the residual and rounds to fp16.
//
// Rounding contract as the single-token kernel: fp16 activations, scale applied per group partial, fp16 SwiGLU
// products, f32 routed sum (src/backend/metal/kernels/decode_gemv_q8.metal:166-251).
// Every wait is bounded (moe_sync.cuh).
#include <cuda.h>

#include <atomic>

#include "moe_decode_units.cuh"
#include "moe_route.cuh"
#include "moe_sync.cuh"

namespace uocr {

constexpr int kBtConsumers = 512;                              // 16 warps compute
constexpr int kBtThreads = kBtConsumers + 32;                  // + one warp that issues the bulk copies
constexpr int kBtTokens = 16;                                  // tokens per pass
// An item covers SLICES consecutive 64-wide slices of its expert (template parameter of the kernel): two for calls of more
// than 16 tokens (7 parts per expert and pass), one for smaller calls (14 parts), whose ~150 two-slice items would leave most
// CTAs idle during a second wave.  The partial-output buffers are sized for 14 parts.
constexpr int kBtSmallCallTokens = 16;
__host__ __device__ constexpr int bt_slices_for(uint32_t n) { return n <= (uint32_t)kBtSmallCallTokens ? 1 : 2; }
constexpr int kBtSharedHalves = kSlS / 64 / kSlRoutedPerSlot;  // the shared MLP as 2 pseudo-experts of 14 slices
constexpr int kBtEntries = kSlE + kBtSharedHalves;             // 66
constexpr int kBtStages = 4;
constexpr int kBtDownChunks = 3;                               // ring chunks that carry a slice's `down` fragments and scales
constexpr int kBtChunks = 5;                                   // chunks of four groups per slice
constexpr int kBtMaxTokens = 64;
constexpr int kBtBlocksPerWarp = kSlH / 16 / 16;               // 5 blocks of 16 `down` rows per warp
constexpr int kBtTokenLimbBytes = kSlGroups * 2 * 64;          // 2560: a token's activation bytes [20][2][16 words]

// ---------------------------------------------------------------- 1. routing, activation bytes, dispatch plan
constexpr int kRsThreads = 512;                                 // 16 warps: four experts' logits each

struct RouteSmallParams {
    const __half *hidden;           // [n][H]
    const __half *router;           // [E][H]
    const float *bias;              // [E] or null
    const float *injected;          // [n][E] logits to use instead of the dot products, or null
    uint32_t n, K;
    float scaling;
    float *logits_out, *probs_out;  // optional [n][E]
    uint32_t *ids;                  // [n][K]
    float *weights;                 // [n][K]
    uint32_t *x_limbs;              // [n][20][2][16 words]
    float *x_scales;                // [n][20]
    uint32_t *offsets, *pair_rows, *inverse, *active;      // the dispatch plan
    uint32_t *ticket;               // zero between launches
    uint32_t *status;
    unsigned long long *acc;        // [n][H] fixed-point output sums of the call: this kernel clears its token's row
};

template <int QT>
__global__ void __launch_bounds__(kRsThreads) route_small_kernel(const RouteSmallParams prm) {
    constexpr int H = kSlH, E = kSlE;
    __shared__ __align__(16) __half s_x[H];
    __shared__ float s_logits[E], s_probs[E];
    __shared__ uint64_t s_tab[UOCR_EXPF_N];
    __shared__ uint32_t s_last;
    __shared__ uint32_t s_ids[kBtMaxTokens * 16];            // the plan: every pair's expert (K <= 16)
    __shared__ uint32_t s_cnt[E + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t token = blockIdx.x, K = prm.K;
    if (tid < UOCR_EXPF_N) s_tab[tid] = c_exp_tab[tid];
    for (int h = tid; h < H / 2; h += kRsThreads) reinterpret_cast<uint4 *>(prm.acc + (size_t)token * H)[h] = make_uint4(0u, 0u, 0u, 0u);
    if (tid < H / 8) reinterpret_cast<uint4 *>(s_x)[tid] = __ldg(reinterpret_cast<const uint4 *>(prm.hidden + (size_t)token * H) + tid);
    __syncthreads();

    if (prm.injected != nullptr) {
        if (tid < E) s_logits[tid] = prm.injected[(size_t)token * E + tid] + (prm.bias ? prm.bias[tid] : 0.f);
    } else {
        // warp w: experts 4w .. 4w + 3; lane: the 16-byte chunks lane, lane + 32, ... of every row, all 20 loads in
        // flight before the first is used
        float xv[5][8];
#pragma unroll
        for (int i = 0; i < 5; ++i) {
            const uint4 xr = reinterpret_cast<const uint4 *>(s_x)[lane + 32 * i];
            const __half2 *xh = reinterpret_cast<const __half2 *>(&xr);
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(xh[k]); xv[i][2 * k] = f.x; xv[i][2 * k + 1] = f.y; }
        }
        uint4 wv[4][5];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 5; ++i)
                wv[j][i] = __ldg(reinterpret_cast<const uint4 *>(prm.router + (size_t)(4 * warp + j) * H) + lane + 32 * i);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < 5; ++i) {
                const __half2 *wh = reinterpret_cast<const __half2 *>(&wv[j][i]);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = __half22float2(wh[k]);
                    acc = fmaf(f.x, xv[i][2 * k], acc);
                    acc = fmaf(f.y, xv[i][2 * k + 1], acc);
                }
            }
            acc = warp_sum(acc);
            const int e = 4 * warp + j;
            if (lane == 0) s_logits[e] = prm.bias ? acc + prm.bias[e] : acc;
        }
    }
    __syncthreads();
    if (warp == 0) {
        const bool bad = route_row_warp(s_logits, s_probs, E, K, prm.scaling, lane, s_tab,
                                        prm.logits_out ? prm.logits_out + (size_t)token * E : nullptr,
                                        prm.probs_out ? prm.probs_out + (size_t)token * E : nullptr, prm.ids + (size_t)token * K,
                                        prm.weights + (size_t)token * K);
        if (bad && lane == 0) atomicOr(prm.status, 1u);
    } else {
        // the token's activations as bytes: 16 lanes per group, warps 1 .. 15 (30 half-warps) over the 20 groups
        for (int Gi = (warp - 1) * 2 + (lane >> 4); Gi < kSlGroups; Gi += 30) {
            const int p = lane & 15;
            float xv[4];
            load_word_values<QT>(s_x + Gi * 64, p, xv);
            const GroupLimbs L = group_limbs16(xv, (lane & 16) ? 0xffff0000u : 0x0000ffffu);
            uint32_t *d = prm.x_limbs + ((size_t)token * kSlGroups + Gi) * 32 + p;
            d[0] = L.lo;
            d[16] = L.hi;
            if (p == 0) prm.x_scales[(size_t)token * kSlGroups + Gi] = QT == UOCR_QT_Q4 ? L.scale * kQ4LevelScale : L.scale;
        }
    }
    // ---- the CTA that finishes last builds the dispatch plan
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(prm.ticket, 1u) == prm.n - 1u ? 1u : 0u;
    __syncthreads();
    if (s_last == 0u) return;
    __threadfence();
    const uint32_t pairs = prm.n * K;
    for (uint32_t p = tid; p < pairs; p += kRsThreads) s_ids[p] = __ldcg(prm.ids + p);
    __syncthreads();
    // Counting sort of the pairs by expert, stable (ascending pair index inside an expert).  Warp w owns experts 4w .. 4w + 3
    // and walks the pairs 32 at a time: a ballot per expert gives the count of the chunk and, in the second pass, the
    // position of every matching lane.
    const uint32_t chunks = (pairs + 31u) / 32u;
    uint32_t cnt[4] = {0u, 0u, 0u, 0u};
    for (uint32_t c = 0; c < chunks; ++c) {
        const uint32_t p = 32u * c + (uint32_t)lane, id = p < pairs ? s_ids[p] : 0xffffffffu;
#pragma unroll
        for (int j = 0; j < 4; ++j) cnt[j] += (uint32_t)__popc(__ballot_sync(0xffffffffu, id == (uint32_t)(4 * warp + j)));
    }
    if (lane < 4) s_cnt[4 * warp + lane] = lane == 0 ? cnt[0] : lane == 1 ? cnt[1] : lane == 2 ? cnt[2] : cnt[3];
    __syncthreads();
    if (warp == 0) {
        // exclusive prefix sums of the 64 counts and of the "has pairs" flags: lane l takes experts 2l and 2l + 1
        const uint32_t c0 = s_cnt[2 * lane], c1 = s_cnt[2 * lane + 1];
        uint32_t sum = c0 + c1, act = (c0 ? 1u : 0u) + (c1 ? 1u : 0u);
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t s2 = __shfl_up_sync(0xffffffffu, sum, o), a2 = __shfl_up_sync(0xffffffffu, act, o);
            if (lane >= o) { sum += s2; act += a2; }
        }
        const uint32_t base = sum - c0 - c1, abase = act - (c0 ? 1u : 0u) - (c1 ? 1u : 0u);
        prm.offsets[2 * lane] = base;
        prm.offsets[2 * lane + 1] = base + c0;
        if (c0) prm.active[1 + abase] = (uint32_t)(2 * lane);
        if (c1) prm.active[1 + abase + (c0 ? 1u : 0u)] = (uint32_t)(2 * lane + 1);
        __syncwarp();
        s_cnt[2 * lane] = base;
        s_cnt[2 * lane + 1] = base + c0;
        if (lane == 31) {
            prm.offsets[E] = sum;
            prm.active[0] = act;
            *prm.ticket = 0u;
        }
    }
    __syncthreads();
    uint32_t run[4] = {s_cnt[4 * warp], s_cnt[4 * warp + 1], s_cnt[4 * warp + 2], s_cnt[4 * warp + 3]};
    for (uint32_t c = 0; c < chunks; ++c) {
        const uint32_t p = 32u * c + (uint32_t)lane, id = p < pairs ? s_ids[p] : 0xffffffffu;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t m = __ballot_sync(0xffffffffu, id == (uint32_t)(4 * warp + j));
            if (id == (uint32_t)(4 * warp + j)) {
                const uint32_t pos = run[j] + (uint32_t)__popc(m & ((1u << lane) - 1u));
                prm.pair_rows[pos] = p;
                prm.inverse[p] = pos;
            }
            run[j] += (uint32_t)__popc(m);
        }
    }
    for (uint32_t p = tid; p < pairs; p += kRsThreads)
        if (s_ids[p] >= (uint32_t)E) prm.inverse[p] = 0xffffffffu;
}

// ---------------------------------------------------------------- 2. routed experts and shared MLP
struct BatchedParams {
    const uint8_t *units;             // slice-major weights of the layer: unit = expert * 14 + slice (shared MLP: experts 64, 65)
    const uint32_t *x_limbs;          // [n][20][2][16 words]
    const float *x_scales;            // [n][20]
    uint32_t n, K;
    const uint32_t *active;           // [0] = number of experts with at least one pair, then their ids
    const uint32_t *expert_offsets;   // [E + 1]
    const uint32_t *pair_rows;        // pairs grouped by expert
    const float *top_weights;         // [n][K] routing weights
    unsigned long long *acc;          // [n][H] output sums in 2^-28 fixed point (cleared by the routing kernel)
    uint32_t *status;
};

#ifdef UOCR_BT_TRACE
// Development build only: cycles warp 0 of every CTA spends in each phase of an item, summed over CTAs.
__device__ unsigned long long g_bt_trace[16];
#define BT_T0(var) const long long var = clock64()
#define BT_ADD(slot, var) bt_local[slot] += (unsigned long long)(clock64() - var)
#else
#define BT_T0(var)
#define BT_ADD(slot, var)
#endif

template <int QT> struct BtSmem {
    static constexpr int kChunkBytes = SlBlob<QT>::kGuBytes / kBtChunks;
    static constexpr int kDownBytes = SlBlob<QT>::kDnBytes + kSlH * 2;      // `down` fragments and their scales: three chunks of the ring
    static_assert(kDownBytes > 2 * kChunkBytes && kDownBytes <= 3 * kChunkBytes && kDownBytes % 16 == 0, "down region = three ring chunks");
    static constexpr int kRing = 0;
    static constexpr int kSc = kRing + kBtStages * kChunkBytes;             // two buffers of gate / up scales
    static constexpr int kXf = kSc + 2 * SlBlob<QT>::kGuScBytes;            // activation bytes [16 tok][20][2][16 words]
    static constexpr int kXs = kXf + kBtTokens * kBtTokenLimbBytes;         // their scales [16 tok][20]
    static constexpr int kMid = kXs + kBtTokens * kSlGroups * 4;            // SwiGLU products [16 tok][64] fp16
    static constexpr int kMidf = kMid + kBtTokens * 64 * 2;                 // their bytes [16 tok][2][16 words]
    static constexpr int kMs = kMidf + kBtTokens * 2 * 64;                  // their scales [16]
    static constexpr int kTok = kMs + 64;                                   // token of each slot of the pass [16]
    static constexpr int kWt = kTok + 64;                                   // routing weight of each slot of the pass [16]
    static constexpr int kEntry = kWt + 64;                                 // entries (expert ids), most tokens first [66]
    static constexpr int kFirst = kEntry + 68 * 4;                          // first (entry, pass) index of each entry [67]
    static constexpr int kBars = kFirst + 68 * 4;                           // full[4], empty[4], sc_full[2], sc_empty[2], flags
    static constexpr int kTotal = kBars + 128;
};

__device__ __forceinline__ void bt_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kBtConsumers) : "memory"); }
__device__ __forceinline__ void bt_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Output sums: 64-bit integers in 2^-28 fixed point, added with red.global.add.u64.  Integer addition commutes, so the
// result does not depend on the order in which the items of a call finish (bit-reproducible), and neither per-part
// partial outputs nor a pass over them are needed.  A value outside +-2^18 (or a NaN) is left out and flagged.
constexpr float kBtAccScale = 268435456.f, kBtAccRange = 262144.f;
__device__ __forceinline__ void bt_add_fixed(unsigned long long *p, float x, uint32_t *status) {
    if (!(fabsf(x) < kBtAccRange)) { atomicOr(status, kStatusRange); x = 0.f; }
    asm volatile("red.global.add.u64 [%0], %1;" ::"l"(p), "l"((unsigned long long)__float2ll_rn(x * kBtAccScale)) : "memory");
}

// one work item: an entry (expert or shared half), a 16-token pass, a part (one or two slices)
struct BtItem {
    uint32_t expert, part, row0, p0, T;
};

template <int QT, int SLICES>
__global__ void __launch_bounds__(kBtThreads, 1) decode_batched_kernel(const __grid_constant__ BatchedParams prm) {
    constexpr int kBtSlices = SLICES, kBtParts = kSlRoutedPerSlot / SLICES;
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
    float *s_wt = reinterpret_cast<float *>(smem + Sm::kWt);
    uint32_t *s_entry = reinterpret_cast<uint32_t *>(smem + Sm::kEntry);
    uint32_t *s_first = reinterpret_cast<uint32_t *>(smem + Sm::kFirst);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + Sm::kBars), *empty = full + kBtStages, *sc_full = empty + kBtStages,
             *sc_empty = sc_full + 2;
    int *s_flag = reinterpret_cast<int *>(sc_empty + 2);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t n_active = prm.active[0];
    const uint32_t n_entries = n_active + kBtSharedHalves;

    if (tid == 0) {
        for (int i = 0; i < kBtStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], kBtConsumers / 32); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sc_full[i], 1); mbar_init(&sc_empty[i], kBtConsumers / 32); }
        s_flag[0] = 1; s_flag[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the entries ordered by their number of tokens, most first (the shared halves lead: every token takes them; then
    // the selected experts, ties by id): rank by counting
    auto entry_count = [&](uint32_t e) { return e >= (uint32_t)kSlE ? prm.n : prm.expert_offsets[e + 1] - prm.expert_offsets[e]; };
    if ((uint32_t)tid < n_entries) {
        const uint32_t e = (uint32_t)tid < (uint32_t)kBtSharedHalves ? (uint32_t)kSlE + tid : prm.active[1 + tid - kBtSharedHalves];
        const uint32_t c = entry_count(e);
        uint32_t rank = 0;
        for (uint32_t j = 0; j < n_entries; ++j) {
            const uint32_t e2 = j < (uint32_t)kBtSharedHalves ? (uint32_t)kSlE + j : prm.active[1 + j - kBtSharedHalves];
            const uint32_t c2 = entry_count(e2);
            rank += (c2 > c || (c2 == c && (e2 >= (uint32_t)kSlE ? e2 - kSlE : e2 + kBtSharedHalves) < (e >= (uint32_t)kSlE ? e - kSlE : e + kBtSharedHalves))) ? 1u : 0u;
        }
        s_entry[rank] = e;
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t run = 0;
        for (uint32_t k = 0; k < n_entries; ++k) { s_first[k] = run; run += (entry_count(s_entry[k]) + kBtTokens - 1) / kBtTokens; }
        s_first[n_entries] = run;
    }
    __syncthreads();
    const uint32_t n_items = s_first[n_entries] * kBtParts;
    if (blockIdx.x >= n_items) return;
    auto resolve = [&](uint32_t item) {
        BtItem it;
        const uint32_t ep = item / kBtParts;
        it.part = item % kBtParts;
        uint32_t k = 0;
        while (s_first[k + 1] <= ep) ++k;
        it.expert = s_entry[k];
        it.p0 = (ep - s_first[k]) * kBtTokens;
        it.row0 = it.expert >= (uint32_t)kSlE ? 0u : prm.expert_offsets[it.expert];
        it.T = min((uint32_t)kBtTokens, entry_count(it.expert) - it.p0);
        return it;
    };

    if (warp == kBtConsumers / 32) {
        // ---- producer: the gate / up fragments of every (item, slice), chunk by chunk through the ring, and their scales
        if (lane == 0) {
            uint32_t seq = 0, slices_done = 0;
            for (uint32_t item = blockIdx.x; item < n_items; item += gridDim.x) {
                const BtItem it = resolve(item);
                const uint32_t first_unit = it.expert * kSlRoutedPerSlot + it.part * kBtSlices;
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
                    // then the slice's `down` fragments and their scales (contiguous in the blob), through the same ring
                    for (int d = 0; d < kBtDownChunks; ++d, ++seq) {
                        const uint32_t s = seq % kBtStages;
                        if (seq >= (uint32_t)kBtStages && !mbar_wait(&empty[s], ((seq / kBtStages) - 1u) & 1u, prm.status, s_flag)) return;
                        const uint32_t off = (uint32_t)d * Sm::kChunkBytes;
                        const uint32_t bytes = min((uint32_t)Sm::kChunkBytes, (uint32_t)Sm::kDownBytes - off);
                        mbar_expect_tx(&full[s], bytes);
                        bulk_g2s(smem + Sm::kRing + s * Sm::kChunkBytes, blob + Bl::kDn + off, bytes, &full[s]);
                    }
                }
            }
        }
        return;
    }

    // ---- consumers
    const int rb = warp & 7, nh = warp >> 3;       // gate / up: row block, and which n-blocks (nh, nh + 2) of the pass
    uint32_t seq = 0, slices_done = 0;
#ifdef UOCR_BT_TRACE
    unsigned long long bt_local[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    BT_T0(bt_all);
#endif
    for (uint32_t item = blockIdx.x; item < n_items; item += gridDim.x) {
        BT_T0(bt_p1);
        const BtItem it = resolve(item);
        const bool shared = it.expert >= (uint32_t)kSlE;
        const uint32_t T = it.T, NB = (T + 3u) / 4u;
        const uint32_t first_unit = it.expert * kSlRoutedPerSlot + it.part * kBtSlices;
        if (tid < kBtTokens) {
            uint32_t token = 0xffffffffu;
            float wt = 0.f;
            if ((uint32_t)tid < T) {
                if (shared) { token = it.p0 + tid; wt = 1.0f; }
                else {
                    const uint32_t pair = prm.pair_rows[it.row0 + it.p0 + tid];
                    token = pair / prm.K;
                    wt = prm.top_weights[pair];
                }
            }
            s_tok[tid] = token;
            s_wt[tid] = wt;
        }
        bt_sync();
        // 1. the pass's activation bytes and scales (slots beyond T: zeros), all loads of a thread in flight together
        {
            constexpr int kVecsPerToken = kBtTokenLimbBytes / 16;            // 160
            constexpr int kPerThread = kBtTokens * kVecsPerToken / kBtConsumers;     // 5
            uint4 v[kPerThread];
#pragma unroll
            for (int i = 0; i < kPerThread; ++i) {
                const int idx = i * kBtConsumers + tid, tok = idx / kVecsPerToken, w = idx - tok * kVecsPerToken;
                const uint32_t token = s_tok[tok];
                v[i] = token != 0xffffffffu ? __ldg(reinterpret_cast<const uint4 *>(prm.x_limbs + (size_t)token * (kBtTokenLimbBytes / 4)) + w)
                                            : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int i = 0; i < kPerThread; ++i) reinterpret_cast<uint4 *>(s_xf)[i * kBtConsumers + tid] = v[i];
            if (tid < kBtTokens * kSlGroups) {
                const int tok = tid / kSlGroups, Gi = tid - tok * kSlGroups;
                const uint32_t token = s_tok[tok];
                s_xs[tid] = token != 0xffffffffu ? prm.x_scales[(size_t)token * kSlGroups + Gi] : 0.f;
            }
        }
        bt_sync();
        BT_ADD(0, bt_p1);
#ifdef UOCR_BT_TRACE
        bt_local[8] += 1; bt_local[9] += T;
#endif

        for (int sl = 0; sl < kBtSlices; ++sl, ++slices_done) {
            BT_T0(bt_dw);
            const uint8_t *blob = prm.units + (size_t)(first_unit + sl) * Bl::kBytes;
            const uint32_t sb = slices_done & 1u;
            // the slice's 64 columns of `down` for this warp's five 16-row blocks, and the rows' scales, into registers
            uint4 dwn[kBtBlocksPerWarp][2];
            __half dslo[kBtBlocksPerWarp], dshi[kBtBlocksPerWarp];
            BT_ADD(1, bt_dw);
            BT_T0(bt_gu);
            // 2. gate / up: rows 8 rb .. + 7 of both matrices x the tokens of n-blocks nh and nh + 2
            float ag[2] = {0.f, 0.f}, au[2] = {0.f, 0.f};
            const __half *scg = s_sc + sb * (Bl::kGuScBytes / 2) + (8 * rb + g) * kSlGroups;
            const __half *scu = scg + 64 * kSlGroups;
            bool got = true;
#pragma unroll
            for (int c = 0; c < kBtChunks; ++c, ++seq) {
                const uint32_t s = seq % kBtStages;
                BT_T0(bt_w);
                got = mbar_wait(&full[s], (seq / kBtStages) & 1u, prm.status, s_flag) && got;
                if (c == 0) got = mbar_wait(&sc_full[sb], (slices_done >> 1) & 1u, prm.status, s_flag) && got;
                BT_ADD(2, bt_w);
                const uint4 *w4 = s_ring4 + (size_t)s * (Sm::kChunkBytes / 16);
                if ((uint32_t)nh < NB) {
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
                }
                __syncwarp();
                if (lane == 0) bt_arrive(&empty[s]);
            }
            __syncwarp();
            if (lane == 0) bt_arrive(&sc_empty[sb]);
            // the slice's `down` fragments arrive through the ring as three more chunks (32 blocks of 16 rows per chunk):
            // this warp's five blocks and their scales go to registers, and the stages are handed back at once
            {
                const uint32_t s0 = seq % kBtStages, s1 = (seq + 1) % kBtStages, s2 = (seq + 2) % kBtStages;
                got = mbar_wait(&full[s0], (seq / kBtStages) & 1u, prm.status, s_flag) && got;
                got = mbar_wait(&full[s1], ((seq + 1) / kBtStages) & 1u, prm.status, s_flag) && got;
                got = mbar_wait(&full[s2], ((seq + 2) / kBtStages) & 1u, prm.status, s_flag) && got;
                const uint32_t stage_of[3] = {s0, s1, s2};
                constexpr int kBlockVecs = QT == UOCR_QT_Q8 ? 64 : 32;          // 16-byte vectors per 16-row block
                constexpr int kBlocksPerChunk = Sm::kChunkBytes / 16 / kBlockVecs;   // 32
                const __half *dsc = reinterpret_cast<const __half *>(smem + Sm::kRing + s2 * Sm::kChunkBytes +
                                                                    (Bl::kDnBytes - 2 * Sm::kChunkBytes));
#pragma unroll
                for (int bi = 0; bi < kBtBlocksPerWarp; ++bi) {
                    const int blk = warp + 16 * bi;
                    const uint4 *src = s_ring4 + (size_t)stage_of[blk / kBlocksPerChunk] * (Sm::kChunkBytes / 16) +
                                       (size_t)(blk % kBlocksPerChunk) * kBlockVecs;
                    dwn[bi][0] = src[lane];
                    if (QT == UOCR_QT_Q8) dwn[bi][1] = src[32 + lane];
                    dslo[bi] = dsc[16 * blk + g];
                    dshi[bi] = dsc[16 * blk + 8 + g];
                }
                __syncwarp();
                if (lane == 0) { bt_arrive(&empty[s0]); bt_arrive(&empty[s1]); bt_arrive(&empty[s2]); }
                seq += kBtDownChunks;
            }
            BT_ADD(3, bt_gu);
            BT_T0(bt_sw);
            // 3. SwiGLU in registers: lane (g, t) holds gate and up of column 8 rb + g for token 4 nb + t
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t nb = (uint32_t)nh + 2u * i;
                if (nb < NB) s_mid[(4 * nb + t) * 64 + 8 * rb + g] = __float2half_rn(got ? silu_fast_f32(ag[i]) * au[i] : 0.f);
            }
            bt_sync();
            if ((uint32_t)tid < 4u * NB * 16u) {                // the products as bytes: 16 lanes per token
                const int tok = tid >> 4, p = tid & 15;
                float mv[4];
                load_word_values<QT>(s_mid + tok * 64, p, mv);
                const GroupLimbs M = group_limbs16(mv, (lane & 16) ? 0xffff0000u : 0x0000ffffu);
                uint32_t *d = s_midf + (tok * 2) * 16 + p;
                d[0] = M.lo;
                d[16] = M.hi;
                if (p == 0) s_ms[tok] = QT == UOCR_QT_Q4 ? M.scale * kQ4LevelScale : M.scale;
            }
            bt_sync();
            BT_ADD(4, bt_sw);
            BT_T0(bt_dn);
            // 4. down: this warp's 80 rows x the slice's 64 columns x every token of the pass
            for (uint32_t nb = 0; nb < NB; ++nb) {
                const uint4 mbf = *reinterpret_cast<const uint4 *>(s_midf + (((4 * nb + (g >> 1)) * 2 + (g & 1)) * 4 + t) * 4);
                const uint32_t tokc = 4u * nb + t;
                // the slot's routing weight rides in the scale; the products go straight into the call's output sums
                const float ms = s_ms[tokc] * s_wt[tokc];
                unsigned long long *dst = prm.acc + (size_t)(tokc < T ? s_tok[tokc] : 0u) * H;
#pragma unroll
                for (int bi = 0; bi < kBtBlocksPerWarp; ++bi) {
                    int ca[4] = {0, 0, 0, 0}, cb[4] = {0, 0, 0, 0};
                    if (QT == UOCR_QT_Q8) group_imma(ca, cb, dwn[bi][0], dwn[bi][1], mbf);
                    else group_imma(ca, cb, make_uint2(dwn[bi][0].x, dwn[bi][0].y), make_uint2(dwn[bi][0].z, dwn[bi][0].w), mbf);
                    if (tokc < T) {
                        const float v0 = (float)(ca[0] + cb[0] + (ca[1] + cb[1]) * 256) * (__half2float(dslo[bi]) * ms);
                        const float v1 = (float)(ca[2] + cb[2] + (ca[3] + cb[3]) * 256) * (__half2float(dshi[bi]) * ms);
                        const uint32_t r = 16u * (warp + 16 * bi) + g;
                        bt_add_fixed(dst + r, v0, prm.status);
                        bt_add_fixed(dst + r + 8, v1, prm.status);
                    }
                }
            }
            BT_ADD(5, bt_dn);
            BT_T0(bt_fs);
            bt_sync();
            BT_ADD(6, bt_fs);
        }
    }
#ifdef UOCR_BT_TRACE
    BT_ADD(7, bt_all);
    if (tid == 0)
        for (int i = 0; i < 10; ++i) atomicAdd(&g_bt_trace[i], bt_local[i]);
    if (tid == 0) atomicAdd(&g_bt_trace[10], 1ull);
#endif
}

// ---------------------------------------------------------------- 3. combine
// out[t][h] = fp16( output sum + residual ): the weighted sum over slots and the shared MLP's output are already in the sum
__global__ void __launch_bounds__(256) finalize_batched_kernel(const unsigned long long *__restrict__ acc, const __half *__restrict__ residual,
                                                               uint32_t n, uint32_t H, __half *__restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;       // one group of 4 outputs
    if (idx >= (size_t)n * (H / 4)) return;
    const ulonglong2 a01 = *reinterpret_cast<const ulonglong2 *>(acc + idx * 4), a23 = *reinterpret_cast<const ulonglong2 *>(acc + idx * 4 + 2);
    float v[4] = {(float)(long long)a01.x * (1.0f / kBtAccScale), (float)(long long)a01.y * (1.0f / kBtAccScale),
                  (float)(long long)a23.x * (1.0f / kBtAccScale), (float)(long long)a23.y * (1.0f / kBtAccScale)};
    if (residual) {
        const uint2 rv = *reinterpret_cast<const uint2 *>(residual + idx * 4);
        const float2 r01 = __half22float2(*reinterpret_cast<const __half2 *>(&rv.x));
        const float2 r23 = __half22float2(*reinterpret_cast<const __half2 *>(&rv.y));
        v[0] += r01.x; v[1] += r01.y; v[2] += r23.x; v[3] += r23.y;
    }
    uint2 o;
    *reinterpret_cast<__half2 *>(&o.x) = __floats2half2_rn(v[0], v[1]);
    *reinterpret_cast<__half2 *>(&o.y) = __floats2half2_rn(v[2], v[3]);
    *reinterpret_cast<uint2 *>(out + idx * 4) = o;
}

// ---------------------------------------------------------------- host side
bool decode_sliced_layer_ok(const DLayer &L);

cudaError_t init_decode_batched_kernels() {
    cudaError_t err = cudaSuccess;
#define UOCR_BT_SMEM(QT, SL)                                                                                              \
    if (err == cudaSuccess)                                                                                               \
        err = cudaFuncSetAttribute(decode_batched_kernel<QT, SL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BtSmem<QT>::kTotal);
    UOCR_BT_SMEM(UOCR_QT_Q4, 1) UOCR_BT_SMEM(UOCR_QT_Q4, 2) UOCR_BT_SMEM(UOCR_QT_Q8, 1) UOCR_BT_SMEM(UOCR_QT_Q8, 2)
#undef UOCR_BT_SMEM
    return err;
}

static std::atomic<int> g_bt_sms[64];

uint32_t decode_batched_max_tokens() { return kBtMaxTokens; }

// Scratch of a call with n tokens (n <= decode_batched_max_tokens()): the parts of the routed experts and of the shared
// MLP, the tokens' activation bytes and scales.
BatchedScratchLayout decode_batched_scratch(uint32_t n, uint32_t K) {
    BatchedScratchLayout l{};
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off = (off + bytes + 255) / 256 * 256; return o; };
    (void)K;
    l.acc = take((size_t)n * kSlH * sizeof(unsigned long long));
    l.x_limbs = take((size_t)n * kBtTokenLimbBytes);
    l.x_scales = take((size_t)n * kSlGroups * sizeof(float));
    l.total = off;
    return l;
}

// The model's shapes in Q4_0 / Q8_0 with the slice-major copy present, and a token count this path is built for.
bool decode_batched_supported(const DLayer &L, uint32_t n) {
    return n >= 2 && n <= (uint32_t)kBtMaxTokens && L.K <= 16 && decode_sliced_layer_ok(L) && L.dec_units != nullptr;
}

// The layer for n tokens in three launches: routing + activation bytes + dispatch plan (results in S), experts, combine.
// scratch: a region of decode_batched_scratch(n, K).total bytes; ticket: a word that is zero before the first call
// (every call leaves it zero).
cudaError_t launch_batched_route(const DLayer &L, const Scratch &S, const __half *hidden, const float *injected, uint32_t n,
                                 float *logits, float *probs, uint8_t *scratch, uint32_t *ticket, cudaStream_t st, uint64_t *launches) {
    const BatchedScratchLayout lay = decode_batched_scratch(n, L.K);
    RouteSmallParams r{};
    r.hidden = hidden; r.router = L.router; r.bias = L.bias; r.injected = injected; r.n = n; r.K = L.K; r.scaling = L.scaling;
    r.logits_out = logits; r.probs_out = probs; r.ids = S.top_ids; r.weights = S.top_weights;
    r.x_limbs = reinterpret_cast<uint32_t *>(scratch + lay.x_limbs); r.x_scales = reinterpret_cast<float *>(scratch + lay.x_scales);
    r.offsets = S.expert_offsets; r.pair_rows = S.pair_rows; r.inverse = S.inverse; r.active = S.active;
    r.ticket = ticket; r.status = S.status;
    r.acc = reinterpret_cast<unsigned long long *>(scratch + lay.acc);
    if (L.expert_qtype == UOCR_QT_Q4) route_small_kernel<UOCR_QT_Q4><<<n, kRsThreads, 0, st>>>(r);
    else route_small_kernel<UOCR_QT_Q8><<<n, kRsThreads, 0, st>>>(r);
    ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_batched_experts(const DLayer &L, const Scratch &S, uint32_t n, uint8_t *scratch, cudaStream_t st, uint64_t *launches) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    int sms = (dev >= 0 && dev < 64) ? g_bt_sms[dev].load() : 0;
    if (sms == 0) {
        if ((err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return err;
        if (dev >= 0 && dev < 64) g_bt_sms[dev] = sms;
    }
    const BatchedScratchLayout lay = decode_batched_scratch(n, L.K);
    BatchedParams p{};
    p.units = L.dec_units;
    p.x_limbs = reinterpret_cast<const uint32_t *>(scratch + lay.x_limbs); p.x_scales = reinterpret_cast<const float *>(scratch + lay.x_scales);
    p.n = n; p.K = L.K;
    p.active = S.active; p.expert_offsets = S.expert_offsets; p.pair_rows = S.pair_rows;
    p.top_weights = S.top_weights;
    p.acc = reinterpret_cast<unsigned long long *>(scratch + lay.acc);
    p.status = S.status;
    // at most one item per (selected expert or shared half, pass, part); one CTA per SM, items dealt round-robin
    const uint64_t pairs = (uint64_t)n * L.K;
    const uint64_t max_entry_passes = (pairs < L.E ? pairs : L.E) + pairs / kBtTokens + kBtSharedHalves * ((n + kBtTokens - 1) / kBtTokens);
    const int slices = bt_slices_for(n);
    const uint64_t max_items = max_entry_passes * (uint64_t)(kSlRoutedPerSlot / slices);
    const uint32_t grid = (uint32_t)(max_items < (uint64_t)sms ? max_items : (uint64_t)sms);
    if (L.expert_qtype == UOCR_QT_Q4) {
        if (slices == 1) decode_batched_kernel<UOCR_QT_Q4, 1><<<grid, kBtThreads, BtSmem<UOCR_QT_Q4>::kTotal, st>>>(p);
        else decode_batched_kernel<UOCR_QT_Q4, 2><<<grid, kBtThreads, BtSmem<UOCR_QT_Q4>::kTotal, st>>>(p);
    } else {
        if (slices == 1) decode_batched_kernel<UOCR_QT_Q8, 1><<<grid, kBtThreads, BtSmem<UOCR_QT_Q8>::kTotal, st>>>(p);
        else decode_batched_kernel<UOCR_QT_Q8, 2><<<grid, kBtThreads, BtSmem<UOCR_QT_Q8>::kTotal, st>>>(p);
    }
    ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_batched_combine(const DLayer &L, const Scratch &S, const __half *residual, uint32_t n, uint8_t *scratch, __half *out,
                                   cudaStream_t st, uint64_t *launches) {
    (void)S;
    const BatchedScratchLayout lay = decode_batched_scratch(n, L.K);
    const size_t work = (size_t)n * (L.H / 4);
    finalize_batched_kernel<<<(unsigned)((work + 255) / 256), 256, 0, st>>>(reinterpret_cast<const unsigned long long *>(scratch + lay.acc), residual, n,
                                                                            L.H, out);
    ++*launches;
    return cudaGetLastError();
}

}  // namespace uocr

#ifdef UOCR_BT_TRACE
extern "C" __attribute__((visibility("default"))) int uocr_cuda_debug_bt_trace(unsigned long long *out16, int reset) {
    if (cudaMemcpyFromSymbol(out16, uocr::g_bt_trace, sizeof(unsigned long long) * 16) != cudaSuccess) return 0;
    if (reset) { static const unsigned long long zero[16] = {0}; if (cudaMemcpyToSymbol(uocr::g_bt_trace, zero, sizeof zero) != cudaSuccess) return 0; }
    return 1;
}
#endif

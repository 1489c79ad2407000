// Single-token decode, sliced design: a run of MoE layers in ONE persistent kernel whose only exchange
// between CTAs per layer is the layer's output vector.
//
// The intermediate dimension of every SwiGLU MLP the token uses is cut into 64-wide slices (one
// quantisation group of the `down` matrix): K * F/64 routed slices + S/64 shared slices = 112 units for
// the model's shapes, one CTA each.  The CTA of a slice
//   1. computes the slice's 64 gate and 64 up pre-activations (128 packed rows of length H, staged in shared
//      memory by a few large TMA bulk copies) and the 64 SwiGLU products (rounded to fp16),
//   2. multiplies them straight away with its 64-column slice of `down` (H rows, loaded into registers while
//      step 1 runs), scales by the routing weight, and
//   3. adds the H partial outputs to the layer's accumulator in global memory.
// Nothing crosses CTAs between 1 and 2.  Every CTA then reads the H accumulated values, adds the residual, rounds to
// fp16 and has the next layer's input.
//
// Weight layout.  A column slice of `down` in the file layout is 32 bytes out of every 448-byte row, and the
// 128 gate/up rows of a slice are read 8 bytes per lane: both are poison for DRAM bursts and for the load/store
// unit (one cache line per row per instruction).  When a layer is mapped, the weights are therefore ALSO stored
// slice-major ("unit blobs"): everything one CTA needs, contiguous, already in the order the MMA lanes consume
// it.  The file-layout copy stays for the many-token paths.  Same bytes, no padding: a blob is
//   gate/up fragments [group 0..19][row block 0..7][lane] | gate/up scales [128][20] | down fragments
//   [row block 0..79][lane] | down scales [H].
//
// The accumulator is 64-bit fixed point (2^-28 units) updated with integer reductions, so the sum does not
// depend on the order in which CTAs arrive: results are reproducible run to run.  The top byte of a word counts
// the CTAs that have added to it - every CTA adds to every word exactly once per layer - so a reader that sees
// the full count holds the final value: no grid barrier, no fence, one L2 round trip less per layer.  The
// accumulator may be kept in 1, 2 or 4 replicas (CTA c adds to replica c % R, readers add the replicas up), which
// spreads the 112 additions per word over more L2 lines.  Four
// accumulator buffers rotate (adds / read / idle / cleared); the rotation continues across launches, and the data
// dependency itself (nobody can start layer l + 1 before everybody has finished reading layer l - 1) keeps the
// clearing safe.
//
// Off the critical path: the shared-MLP CTAs do not depend on the routing, so they fetch the NEXT layer's
// weights while they wait for the layer's output to be complete; the routed CTAs fetch the next layer's router
// matrix into registers at the same point - each CTA of a cluster of four a quarter of it (16 experts) - and evaluate it as
// soon as the new activations are there; the four quarters of the logits are exchanged through distributed
// shared memory (st.async stores that count bytes on the receiver's mbarrier: one hop, no separate arrival).
// The softmax / top-k itself is taken off the path as well (one warp, which the others do not wait for): see
// "routing" in the kernel.
//
// Arithmetic.  Scalar dequantise-and-FMA costs ~3.5 instructions per packed weight and would bound the layer, so
// the dot products run on the tensor cores as INTEGER MMAs (m16n8k32, s32 accumulate), which take the packed
// levels as they are (Q8: the int8 words themselves; Q4: one AND per four weights).  The fp16 activations of a
// 64-wide group are written once per layer as a block-floating-point number: a shared power-of-two scale and
// signed 15-bit mantissas, exact for every value within a factor 8 of the group's largest and rounded to 2^-14 of
// the largest's power of two otherwise (far below the fp16 rounding of the SwiGLU products that the data path
// carries anyway).  A mantissa is split into two signed bytes, and the two bytes ride in two of the MMA's eight
// columns.  Which two depends on the group (columns 2 (G % 4) and 2 (G % 4) + 1), so four consecutive groups
// accumulate into one set of MMA registers and the per-group work - recombine the two bytes, multiply by
// (activation scale x the group's fp16 weight scale), remove Q4's +8 offset with the correction 8 * sum(mantissas)
// - runs once per four groups with every lane holding one group's result.  The `down` product uses the same trick
// over four 16-row blocks.  The router matrix is fp16 and runs as fp16 MMAs (m16n8k16) on the activations
// themselves.
//
// Every wait is bounded (see moe_sync.cuh).
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "moe_decode_units.cuh"
#include "moe_route.cuh"
#include "moe_sync.cuh"

namespace uocr {

constexpr int kSlThreads = 512;
constexpr int kSlRouted = kSlK * kSlRoutedPerSlot;          // 84
constexpr int kSlUnits = kSlRouted + kSlS / 64;             // 112 CTAs
constexpr int kSlCluster = 4;                               // CTAs per cluster: each evaluates a quarter of the router
constexpr int kSlChunks = 5;                                // gate/up fragments arrive in 5 copies of 4 groups
constexpr int kSlAccBuffers = 4;
constexpr int kSlMaxReplicas = 4;
// accumulator word: bits 56-63 count the CTAs that have added, bits 0-55 hold the sum of (value * 2^28 + 2^47)
constexpr unsigned long long kSlAccOne = 1ull << 56;
constexpr long long kSlAccBias = 1ll << 47;
constexpr float kSlAccScale = 268435456.f;       // 2^28
constexpr float kSlAccRange = 262144.f;          // |partial output| must stay below 2^18
constexpr int kSlTracePoints = 16;
constexpr int kSlMaxLayers = 64;
constexpr int kSlBlocksPerWarp = kSlH / 16 / 16;            // 5 blocks of 16 output rows per warp

struct SlicedParams {
    static constexpr bool kInline = false;
    static constexpr bool kDense = false;
    const DLayer *layers;
    uint32_t first, count;
    const __half *hidden_in;
    const __half *residual0;      // residual of the first layer (may be null)
    int chain_residual;           // layers after the first use their input as residual
    const float *injected;        // [E] logits for the first layer, or null
    __half *out;
    unsigned long long *acc;      // [kSlAccBuffers][kSlMaxReplicas][H] fixed-point accumulators, all zero between launches except two buffers
    uint32_t acc_base;            // buffer of the first layer of this launch
    uint32_t replicas;            // accumulator replicas in use (1, 2 or 4): CTA c adds to replica c % replicas
    uint32_t *status;
    float *dbg_logits, *dbg_probs;
    uint32_t *ids_out;            // [K] routing of the last layer run
    float *wts_out;
    unsigned long long *trace;    // optional [CTA][count][kSlTracePoints] SM-clock stamps
    uint32_t *host_status;        // optional word in mapped host memory: receives the status word after `out` is written
    long long spin_limit;         // cycles a wait for other CTAs may take before the kernel gives up
    uint32_t poll_sleep_ns;       // pause between two polls of the layer accumulator (0: none)
    uint32_t expect_extra;        // test hook: contributions the poll expects beyond the CTAs there are (0 in production)
    const __half *router0;        // router matrix and unit blobs of the first layer of the launch (the same pointers as in
    const uint8_t *units0;        // layers[first]): every CTA starts its first fetch from them before it has read the layer table
    const __half *norm_weight;    // optional fp16[H]: the first layer's input is RMSNorm(hidden_in) * norm_weight (residual0 stays as given)
    float norm_eps;
};
// The same with the first layer's input (and, with chain_residual, its residual) carried in the launch parameters:
// a host-buffer call then needs no copy.  A kernel instantiation of its own, so that calls on device buffers keep a
// small parameter block.
struct SlicedParamsInline : SlicedParams {
    static constexpr bool kInline = true;
    uint4 inline_x[kSlH * 2 / 16];  // fp16 activations
};
// A dense SwiGLU MLP (the first decoder layer's) through the same kernel: `layers` points at ONE pseudo layer whose
// dec_units hold gridDim.x units of 64 intermediate columns each; every CTA works like a shared-MLP CTA on unit blockIdx.x,
// nothing is routed.  Units beyond the MLP's width hold zeros (the grid is a multiple of the cluster size).
struct SlicedParamsDense : SlicedParams {
    static constexpr bool kDense = true;
};

__device__ __forceinline__ void red_add_u64(unsigned long long *p, unsigned long long v) {
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_addr(const void *local, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(local)), "r"(rank));
    return a;
}
// one fp32 value into another CTA's shared memory; its arrival counts 4 bytes on that CTA's barrier
__device__ __forceinline__ void st_async_f32(uint32_t remote_addr, float v, uint32_t remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(remote_addr), "r"(__float_as_uint(v)), "r"(remote_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// Shared-memory layout (byte offsets); the layer table comes last.
//
// Activation bytes for the MMAs' B operand are kept "by column": [group][MMA column 0..7][16 words].  Group G puts
// its low mantissa bytes in column 2 (G % 4), its high bytes in column 2 (G % 4) + 1 and leaves the other six
// columns zero (written once at kernel start).  Four consecutive groups can then be accumulated into ONE set of MMA
// accumulators: group q only touches result columns 2q and 2q + 1, i.e. the two registers of lane-in-quad q.
// After the four groups every lane of a quad holds one group's two integer dot products for its rows, and the
// per-group scaling runs once per four groups with all 32 lanes busy.  The SwiGLU products use the same layout
// four times ([q][column][16 words], their bytes in columns 2q, 2q + 1) so that four 16-row blocks of `down`
// share an accumulator set in the same way.
template <int QT> struct SlSmem {
    static constexpr int kW = 0;                                        // gate/up fragments as in the blob
    static constexpr int kSc = kW + SlBlob<QT>::kGuBytes;               // gate scales [64][20], up scales [64][20] (fp16)
    static constexpr int kX = kSc + SlBlob<QT>::kGuScBytes;             // activations, fp16 natural order
    static constexpr int kXf = kX + kSlH * 2;                           // activation bytes [20][8][16 words]
    static constexpr int kXs = kXf + kSlGroups * 8 * 16 * 4;            // [20] group scales (Q4_0: with the 1/16 of the level bytes)
    static constexpr int kGu = kXs + 256;                               // [2][128] partial gate / up sums of the two warp halves
    static constexpr int kMid = kGu + 2 * 128 * 4;                      // [64] fp16 SwiGLU products
    static constexpr int kMidf = kMid + 128;                            // their bytes [4][8][16 words], then the scale
    static constexpr int kRp = kMidf + 4 * 8 * 16 * 4 + 64;             // [16 warps][16 experts] partial router logits
    static constexpr int kLogits = kRp + 4 * 64 * 4;                    // [64]
    static constexpr int kProbs = kLogits + 256;                        // [64]
    static constexpr int kIds = kProbs + 256;                           // ids [8], weights [8], flags [2]
    static constexpr int kBars = kIds + 128;                            // kSlChunks copy barriers, scale barrier, cluster barrier
    static constexpr int kLayers = kBars + 8 * 8;                       // DLayer table
    static constexpr int kTotal = kLayers + kSlMaxLayers * (int)sizeof(DLayer);
};

template <int N> struct SlInt { static constexpr int value = N; };

// ---------------------------------------------------------------- the kernel
template <int QT, class Params>
__global__ void __launch_bounds__(kSlThreads, 1) decode_sliced_kernel(const __grid_constant__ Params prm) {
    using Bl = SlBlob<QT>;
    using Sm = SlSmem<QT>;
    constexpr int H = kSlH, K = kSlK, E = kSlE;
    constexpr int kChunkBytes = Bl::kGuBytes / kSlChunks;

    extern __shared__ __align__(128) uint8_t smem[];
    const uint4 *s_w4 = reinterpret_cast<const uint4 *>(smem + Sm::kW);
    __half *s_sc = reinterpret_cast<__half *>(smem + Sm::kSc);
    __half *s_x = reinterpret_cast<__half *>(smem + Sm::kX);
    uint32_t *s_xf = reinterpret_cast<uint32_t *>(smem + Sm::kXf);
    float *s_xs = reinterpret_cast<float *>(smem + Sm::kXs);             // [20] group scales
    float *s_gu = reinterpret_cast<float *>(smem + Sm::kGu);
    uint32_t *s_midf = reinterpret_cast<uint32_t *>(smem + Sm::kMidf);   // [4][8][16 words]
    float *s_mscale = reinterpret_cast<float *>(s_midf + 4 * 8 * 16);    // scale
    float *s_rp = reinterpret_cast<float *>(smem + Sm::kRp);
    float *s_logits = reinterpret_cast<float *>(smem + Sm::kLogits);
    float *s_probs = reinterpret_cast<float *>(smem + Sm::kProbs);
    uint32_t *s_ids = reinterpret_cast<uint32_t *>(smem + Sm::kIds);
    float *s_wts = reinterpret_cast<float *>(s_ids + 8);
    int *s_flag = reinterpret_cast<int *>(s_ids + 16);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + Sm::kBars);     // [0, kSlChunks) copies, then scales, then cluster
    uint64_t *sc_bar = bars + kSlChunks, *lg_bar = bars + kSlChunks + 1;
    DLayer *s_layers = reinterpret_cast<DLayer *>(smem + Sm::kLayers);
    __shared__ uint64_t s_tab[UOCR_EXPF_N];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;                              // MMA row group = B column / lane in quad
    const uint32_t G = gridDim.x, cta = blockIdx.x;
    const bool routed = !Params::kDense && cta < (uint32_t)kSlRouted;
    const uint32_t slot = routed ? cta / kSlRoutedPerSlot : (uint32_t)K;
    const uint32_t fg = Params::kDense ? cta : routed ? cta % kSlRoutedPerSlot : cta - kSlRouted;     // 64-wide slice of F (of S)
    constexpr uint32_t kSharedUnit0 = Params::kDense ? 0u : (uint32_t)(kSlE * kSlRoutedPerSlot);         // first unit of the non-routed CTAs
    uint32_t *status = prm.status;
    const uint32_t crank = cluster_rank(), csize = cluster_size();
    const uint32_t R = prm.replicas;                                    // accumulator replicas (1, 2 or 4)
    const long long spin_limit = prm.spin_limit;

    if (prm.trace != nullptr && tid == 0 && cta == 0) prm.trace[(size_t)127 * prm.count * kSlTracePoints] = clock64();     // kernel entry
    if (tid < UOCR_EXPF_N) s_tab[tid] = c_exp_tab[tid];
    if (tid == 0) {
        s_flag[0] = 1; s_flag[1] = 0;
        for (int i = 0; i <= kSlChunks; ++i) mbar_init(&bars[i], 1);
        mbar_init(lg_bar, 1);
        s_ids[7] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // every CTA of the cluster has initialised its barriers before any peer arrives on them
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    // ---- helpers --------------------------------------------------------------------------------------
    // mantissa bytes and offset corrections of the activations in s_x
    // (by warps 0 and 2 .. 10: warp 1 of a routed CTA is busy with the exact routing at that time)
    auto build_x_frags = [&]() {
        const int bi = warp == 0 ? tid : tid - 32;
        if (warp != 1 && bi < kSlGroups * 16) {                         // 16 lanes per group
            const int Gi = bi >> 4, p = bi & 15;
            float xv[4];
            load_word_values<QT>(s_x + Gi * 64, p, xv);
            const GroupLimbs L = group_limbs(xv);
            uint32_t *d = s_xf + (Gi * 8 + 2 * (Gi & 3)) * 16 + p;
            d[0] = L.lo;
            d[16] = L.hi;
            if (p == 0) s_xs[Gi] = QT == UOCR_QT_Q4 ? L.scale * kQ4LevelScale : L.scale;
        }
    };
    // Prefetched into registers: this warp's 5 blocks of 16 `down` rows (the unit's 64 columns of each) with the
    // scales of the rows this lane finishes, and the CTA's part of the next layer's router matrix (requested while
    // waiting for the layer's output, used right after it).
    uint4 dwn[kSlBlocksPerWarp][2];
    uint2 rtr[5][2];
    __half dsc4[4];
    // everything of one unit: bulk copies of the gate/up fragments (chunk c completes barrier c) and scales into
    // shared memory, plain loads of the down fragments and scales into registers
    // (one thread issues the copies in the order they are needed, and a routed CTA asks for its down fragments only
    // once its first chunk is there: all routed CTAs fetch at the same moment and HBM serves what was asked first)
    auto fetch_gate_up = [&](const uint8_t *blob) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (tid == 0) {
#pragma unroll
            for (int c = 0; c < kSlChunks; ++c) {
                mbar_expect_tx(&bars[c], kChunkBytes);
                bulk_g2s(smem + Sm::kW + c * kChunkBytes, blob + Bl::kGu + (size_t)c * kChunkBytes, kChunkBytes, &bars[c]);
                if (c == 1) {          // the scales are first needed after the MMAs of the first two chunks
                    mbar_expect_tx(sc_bar, Bl::kGuScBytes);
                    bulk_g2s(s_sc, blob + Bl::kGuSc, Bl::kGuScBytes, sc_bar);
                }
            }
        }
    };
    // Blocks warp + 16 bi (bi = 0 .. 4).  Blocks 0 .. 3 share one accumulator set, whose results for block bi end up
    // in lane-in-quad bi (rows g and g + 8 of the block): each lane keeps the scales of exactly those two rows, and
    // of its two rows of block 4.
    auto fetch_down = [&](const uint8_t *blob) {
        const uint4 *dn = reinterpret_cast<const uint4 *>(blob + Bl::kDn);
        const __half *dsc = reinterpret_cast<const __half *>(blob + Bl::kDnSc);
#pragma unroll
        for (int bi = 0; bi < kSlBlocksPerWarp; ++bi) {
            const int blk = warp + 16 * bi;
            if (QT == UOCR_QT_Q8) {
                dwn[bi][0] = __ldg(dn + (blk * 2) * 32 + lane);
                dwn[bi][1] = __ldg(dn + (blk * 2 + 1) * 32 + lane);
            } else {
                dwn[bi][0] = __ldg(dn + blk * 32 + lane);         // rows g: .x .y, rows g + 8: .z .w
            }
        }
        dsc4[0] = dsc[16 * (warp + 16 * t) + g];
        dsc4[1] = dsc[16 * (warp + 16 * t) + 8 + g];
        dsc4[2] = dsc[16 * (warp + 64) + g];
        dsc4[3] = dsc[16 * (warp + 64) + 8 + g];
    };
    auto fetch_unit = [&](const uint8_t *blob) { fetch_gate_up(blob); fetch_down(blob); };
    // This CTA's quarter of the router matrix (experts 16 crank .. +15, fp16 [E][H]) as MMA A fragments: warp w holds
    // columns 80 w .. 80 w + 79 (five k steps), lane (g, t) the columns 4t .. 4t + 3 of each step for rows g and g + 8.
    auto load_router = [&](const __half *router) {
        const __half *r0 = router + (size_t)(16 * crank + g) * H + 80 * warp + 4 * t;
#pragma unroll
        for (int i = 0; i < 5; ++i) {
            rtr[i][0] = __ldg(reinterpret_cast<const uint2 *>(r0 + 16 * i));
            rtr[i][1] = __ldg(reinterpret_cast<const uint2 *>(r0 + 8 * H + 16 * i));
        }
    };
    // ---- everything the first layer can fetch before its activations are arranged, asked for before anything else is read
    if (routed) load_router(prm.router0);
    else fetch_unit(prm.units0 + (size_t)(kSharedUnit0 + fg) * Bl::kBytes);
    {
        const uint32_t words = prm.count * (uint32_t)(sizeof(DLayer) / 4);
        const uint32_t *src = reinterpret_cast<const uint32_t *>(prm.layers + prm.first);
        uint32_t *dst = reinterpret_cast<uint32_t *>(s_layers);
        for (uint32_t i = tid; i < words; i += kSlThreads) dst[i] = src[i];
        for (int i = tid; i < kSlGroups * 8 * 16; i += kSlThreads) s_xf[i] = 0u;      // the columns no group writes
        for (int i = tid; i < 4 * 8 * 16; i += kSlThreads) s_midf[i] = 0u;
    }
    // the first layer's input, and its residual in registers
    float res0[3] = {0.f, 0.f, 0.f};
    {
        const __half *xin = prm.hidden_in, *rin = prm.residual0;
        if constexpr (Params::kInline) {
            xin = reinterpret_cast<const __half *>(prm.inline_x);
            rin = prm.chain_residual ? xin : nullptr;
        }
        for (int h = tid; h < H; h += kSlThreads) s_x[h] = xin[h];
        if (rin != nullptr) {
#pragma unroll
            for (int i = 0; i < 3; ++i)
                if (tid + i * kSlThreads < H) res0[i] = __half2float(rin[tid + i * kSlThreads]);
        }
    }
    __syncthreads();
    if (prm.norm_weight != nullptr) {
        // The post-attention RMSNorm in front of the layer, with the arithmetic of rmsnorm_kernel (128 threads take every
        // 128th pair, a shuffle tree per warp, the four warp sums added in order), so that a call with the norm folded in
        // equals the norm kernel followed by the plain call bit for bit.
        float *s_norm = s_rp;
        if (tid < 128) {
            const __half2 *xr = reinterpret_cast<const __half2 *>(s_x);
            float ss = 0.f;
            for (int i = tid; i < H / 2; i += 128) {
                const float2 v = __half22float2(xr[i]);
                ss = fmaf(v.x, v.x, ss);
                ss = fmaf(v.y, v.y, ss);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) s_norm[warp] = ss;
        }
        __syncthreads();
        float total = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) total += s_norm[i];
        const float inv = 1.0f / sqrtf(total / (float)H + prm.norm_eps);
        const __half2 *wr = reinterpret_cast<const __half2 *>(prm.norm_weight);
        __half2 *xw = reinterpret_cast<__half2 *>(s_x);
        __syncthreads();          // every thread has read the four sums before s_rp is used again
        for (int i = tid; i < H / 2; i += kSlThreads) {
            const float2 v = __half22float2(xw[i]), gw = __half22float2(wr[i]);
            xw[i] = __floats2half2_rn(v.x * inv * gw.x, v.y * inv * gw.y);
        }
        __syncthreads();
    }

    uint32_t lg_phase = 0;

#define UOCR_SL_TRACE(point)                                                                              \
    do {                                                                                                  \
        if (prm.trace != nullptr && tid == 0)                                                             \
            prm.trace[((size_t)cta * prm.count + li) * kSlTracePoints + (point)] = clock64();             \
    } while (0)

    uint32_t copy_phase = 0;
    if (!routed) build_x_frags();      // routed CTAs arrange their activations while their weights are on the way
    __syncthreads();

    for (uint32_t li = 0; li < prm.count; ++li) {
        const DLayer &L = s_layers[li];
        const bool last = li + 1 == prm.count;
        // the layer's accumulator: R replicas of H words; this CTA adds to replica cta % R, readers sum all R
        unsigned long long *acc = prm.acc + (size_t)((prm.acc_base + li) % kSlAccBuffers) * kSlMaxReplicas * H;
        UOCR_SL_TRACE(0);     // activations of this layer arranged
        bool valid = true;
        float weight = 1.0f;

        if (routed) {
            // ---- router: this CTA's 16 logits, then the exchange with the three other CTAs of the cluster
            if (li == 0 && prm.injected != nullptr) {
                if (tid < E) s_logits[tid] = prm.injected[tid] + (L.bias ? L.bias[tid] : 0.f);
            } else {
                float c[4] = {0.f, 0.f, 0.f, 0.f}, d[4] = {0.f, 0.f, 0.f, 0.f};      // two chains of MMAs
                const __half *xq = s_x + 80 * warp + 4 * t;
#pragma unroll
                for (int i = 0; i < 5; ++i) {
                    const uint2 xv = *reinterpret_cast<const uint2 *>(xq + 16 * i);
                    if (i & 1) mma16816(d, rtr[i][0].x, rtr[i][1].x, rtr[i][0].y, rtr[i][1].y, xv.x, xv.y);
                    else mma16816(c, rtr[i][0].x, rtr[i][1].x, rtr[i][0].y, rtr[i][1].y, xv.x, xv.y);
                }
                if (t == 0) { s_rp[warp * 16 + g] = c[0] + d[0]; s_rp[warp * 16 + 8 + g] = c[2] + d[2]; }
                __syncthreads();
                UOCR_SL_TRACE(8);     // this CTA's partial logits
                if (warp == 0) {
                    if (lane < 16) {          // one logit per lane, summed over the warps in a fixed order, sent to the whole cluster
                        float v = 0.f;
#pragma unroll
                        for (int w = 0; w < 16; ++w) v += s_rp[w * 16 + lane];
                        const uint32_t e = 16u * crank + (uint32_t)lane;
                        if (L.bias) v += L.bias[e];
                        // each store carries its own completion count to the receiver's barrier: no release /
                        // acquire round between the data and a separate arrival
                        for (uint32_t r = 0; r < csize; ++r) st_async_f32(cluster_addr(s_logits + e, r), v, cluster_addr(lg_bar, r));
                    }
                    if (lane == 0) {
                        mbar_expect_tx(lg_bar, 16u * 4u * csize);       // this phase: 16 logits from each CTA of the cluster
                        if (!mbar_try_wait_cluster(lg_bar, lg_phase)) {
                            const long long t0 = clock64();
                            while (!mbar_try_wait_cluster(lg_bar, lg_phase)) {
                                if (clock64() - t0 > spin_limit) { atomicOr(status, kStatusBarrier); s_flag[1] = 1; break; }
                            }
                        }
                    }
                }
                lg_phase ^= 1u;
            }
            __syncthreads();
            UOCR_SL_TRACE(9);         // all 64 logits exchanged
            // ---- routing.  The softmax is monotonic, so the slot's expert is (except for two logits that round to one
            // probability) the one whose logit ranks slot-th: eight threads per expert count the logits that beat
            // it.  Every warp but one goes on to fetch that expert's weights, while warp 1 runs the exact softmax /
            // top-k; the result is checked after the gate/up products and the rare mismatch is redone.
            {
                const int e = tid >> 3, part = tid & 7;
                const float mine = s_logits[e];
                int beats = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int o = 8 * part + j;
                    const float v = s_logits[o];
                    beats += (v > mine || (v == mine && o < e)) ? 1 : 0;
                }
                beats += __shfl_xor_sync(0xffffffffu, beats, 1);
                beats += __shfl_xor_sync(0xffffffffu, beats, 2);
                beats += __shfl_xor_sync(0xffffffffu, beats, 4);
                if (part == 0 && beats == (int)slot) s_ids[7] = (uint32_t)e;
            }
            __syncthreads();
            UOCR_SL_TRACE(1);     // expert of this CTA's slot chosen
        } else {
            UOCR_SL_TRACE(1);
        }
        uint32_t ex = routed ? s_ids[7] : 0u;       // expert whose weights this CTA fetches
      for (bool first = true;; first = false) {
        const uint8_t *blob = L.dec_units + (size_t)(ex * kSlRoutedPerSlot + fg) * Bl::kBytes;
        if (routed) {
            fetch_gate_up(blob);
            if (first) {
                // Warp 1 computes the exact routing (about 1.5 us: the C library's expf in double precision, a serial
                // sum, K selection rounds) while the other fifteen arrange the activations and start on the gate / up
                // products; nobody waits for it before the check after those products.  Barrier 1: the fifteen
                // announce the arranged activations and warp 1 waits for them; barrier 2: the fifteen among themselves.
                if (warp == 1) {
                    const bool dbg = cta == 0 && li == 0;
                    const bool bad = route_row_warp(s_logits, s_probs, E, K, L.scaling, lane, s_tab, dbg ? prm.dbg_logits : nullptr,
                                                    dbg ? prm.dbg_probs : nullptr, s_ids, s_wts);
                    if (bad && lane == 0 && cta == 0) atomicOr(status, kStatusRouter);
                    asm volatile("bar.sync 1, %0;" ::"n"(kSlThreads) : "memory");
                } else {
                    build_x_frags();
                    __threadfence_block();
                    asm volatile("bar.arrive 1, %0;" ::"n"(kSlThreads) : "memory");
                    asm volatile("bar.sync 2, %0;" ::"n"(kSlThreads - 32) : "memory");
                }
            }
        }
        UOCR_SL_TRACE(2);         // weight fetches issued
        {
            // ---- gate / up.  Warp (rb, kh) multiplies rows 8 rb .. +7 of both matrices with half of the groups, four
            // groups (= one chunk of the copy) per accumulator set, as the copies land: warps kh = 0 take chunks 0 and
            // 2, warps kh = 1 chunks 1 and 3, and the last chunk is split between them so that all sixteen work on it.
            const int rb = warp & 7, kh = warp >> 3;
            bool got = true;
            float sg = 0.f, su = 0.f;
            const __half *scg = s_sc + (8 * rb + g) * kSlGroups;
            const __half *scu = scg + 64 * kSlGroups;
            // groups G0 + QLO .. G0 + QHI - 1 (G0 a multiple of 4) into one accumulator set (four accumulators: chains
            // of at most two dependent MMAs); lane-in-quad q then holds group G0 + q: its low-byte and high-byte dot
            // products with gate row g (c[0], c[1]) and up row g (c[2], c[3])
            auto quad = [&](int G0, auto qlo, auto qhi, bool wait_scales) {
                constexpr int QLO = decltype(qlo)::value, QHI = decltype(qhi)::value;
                int ca[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}}, cb[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
                for (int q = QLO; q < QHI; ++q) {
                    const int Gi = G0 + q;
                    const uint4 xb = *reinterpret_cast<const uint4 *>(s_xf + ((Gi * 8 + g) * 4 + t) * 4);
                    if (QT == UOCR_QT_Q8) {
                        const uint4 a = s_w4[((Gi * 8 + rb) * 2) * 32 + lane], b = s_w4[((Gi * 8 + rb) * 2 + 1) * 32 + lane];
                        group_imma(ca[q & 1], cb[q & 1], a, b, xb);
                    } else {
                        const uint4 v = s_w4[(Gi * 8 + rb) * 32 + lane];       // gate: .x .y, up: .z .w
                        group_imma(ca[q & 1], cb[q & 1], make_uint2(v.x, v.y), make_uint2(v.z, v.w), xb);
                    }
                }
                if (wait_scales) got = mbar_wait(sc_bar, copy_phase, status, s_flag) && got;
                if (t >= QLO && t < QHI) {
                    const int Gi = G0 + t;
                    const float xs = s_xs[Gi];
                    const float vg = (float)(ca[0][0] + cb[0][0] + ca[1][0] + cb[1][0] + (ca[0][1] + cb[0][1] + ca[1][1] + cb[1][1]) * 256);
                    const float vu = (float)(ca[0][2] + cb[0][2] + ca[1][2] + cb[1][2] + (ca[0][3] + cb[0][3] + ca[1][3] + cb[1][3]) * 256);
                    sg = fmaf(vg, __half2float(scg[Gi]) * xs, sg);
                    su = fmaf(vu, __half2float(scu[Gi]) * xs, su);
                }
            };
            if (kh == 0) {
                got = mbar_wait(&bars[0], copy_phase, status, s_flag) && got;
                UOCR_SL_TRACE(3);              // first chunk is in shared memory
                if (routed) fetch_down(blob);
                quad(0, SlInt<0>{}, SlInt<4>{}, true);
                UOCR_SL_TRACE(10);
                got = mbar_wait(&bars[2], copy_phase, status, s_flag) && got;
                UOCR_SL_TRACE(11);
                quad(8, SlInt<0>{}, SlInt<4>{}, false);
                UOCR_SL_TRACE(12);
                got = mbar_wait(&bars[4], copy_phase, status, s_flag) && got;
                UOCR_SL_TRACE(13);
                quad(16, SlInt<0>{}, SlInt<2>{}, false);
            } else {
                got = mbar_wait(&bars[1], copy_phase, status, s_flag) && got;
                if (routed) fetch_down(blob);
                quad(4, SlInt<0>{}, SlInt<4>{}, true);
                got = mbar_wait(&bars[3], copy_phase, status, s_flag) && got;
                quad(12, SlInt<0>{}, SlInt<4>{}, false);
                got = mbar_wait(&bars[4], copy_phase, status, s_flag) && got;
                quad(16, SlInt<2>{}, SlInt<4>{}, false);
            }
            if (!got) { sg = 0.f; su = 0.f; }
            // the lanes of a quad hold different groups
            sg += __shfl_xor_sync(0xffffffffu, sg, 1); su += __shfl_xor_sync(0xffffffffu, su, 1);
            sg += __shfl_xor_sync(0xffffffffu, sg, 2); su += __shfl_xor_sync(0xffffffffu, su, 2);
            if (t == 0) { s_gu[kh * 128 + 8 * rb + g] = sg; s_gu[kh * 128 + 64 + 8 * rb + g] = su; }
            UOCR_SL_TRACE(14);        // this warp's gate / up sums
            __syncthreads();
            UOCR_SL_TRACE(15);        // every warp's
            copy_phase ^= 1u;
            if (routed) {            // the exact routing is in shared memory by now
                const uint32_t exact = s_ids[slot];
                if (exact != ex) {
                    if (exact < (uint32_t)E) { ex = exact; __syncthreads(); continue; }
                    valid = false;          // an invalid expert id contributes zeros
                }
                weight = s_wts[slot];
                if (cta == 0 && last && tid < K) { prm.ids_out[tid] = s_ids[tid]; prm.wts_out[tid] = s_wts[tid]; }
            }
            break;
        }
      }
        // ---- down: H rows x the slice's 64 columns, straight from registers.  Blocks 0 .. 3 of the warp share one
        // accumulator set (block bi ends up in lane-in-quad bi), block 4 uses a second one (lane-in-quad 0).
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (valid) {
            // SwiGLU products and their bytes in one step by warp 0: lane p % 16 takes the four values behind word p
            // (both half-warps compute the same; each writes two of the four copies)
            if (warp == 0) {
                const int p = lane & 15, q0 = (lane >> 4) * 2, c0 = limb_column<QT>(p);
                const float4 g0 = *reinterpret_cast<const float4 *>(s_gu + c0), g1 = *reinterpret_cast<const float4 *>(s_gu + 128 + c0);
                const float4 u0 = *reinterpret_cast<const float4 *>(s_gu + 64 + c0), u1 = *reinterpret_cast<const float4 *>(s_gu + 192 + c0);
                const float gate[4] = {g0.x + g1.x, g0.y + g1.y, g0.z + g1.z, g0.w + g1.w};
                const float up[4] = {u0.x + u1.x, u0.y + u1.y, u0.z + u1.z, u0.w + u1.w};
                float mv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) mv[i] = __half2float(__float2half_rn(silu_fast_f32(gate[i]) * up[i]));    // fp16, as every path stores them
                const GroupLimbs M = group_limbs(mv);
#pragma unroll
                for (int q = q0; q < q0 + 2; ++q) {
                    uint32_t *d = s_midf + (q * 8 + 2 * q) * 16 + p;
                    d[0] = M.lo;
                    d[16] = M.hi;
                }
                if (lane == 0) s_mscale[0] = QT == UOCR_QT_Q4 ? M.scale * kQ4LevelScale : M.scale;
            }
            __syncthreads();
            UOCR_SL_TRACE(4);     // SwiGLU products of the slice
            const float ms = s_mscale[0] * weight;
            int ca[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}}, cb[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}}, cc[4] = {0, 0, 0, 0}, cd[4] = {0, 0, 0, 0};
#pragma unroll
            for (int bi = 0; bi < kSlBlocksPerWarp; ++bi) {
                const int q = bi & 3;
                const uint4 mbf = *reinterpret_cast<const uint4 *>(s_midf + ((q * 8 + g) * 4 + t) * 4);
                if (bi < 4) {
                    if (QT == UOCR_QT_Q8) group_imma(ca[bi & 1], cb[bi & 1], dwn[bi][0], dwn[bi][1], mbf);
                    else group_imma(ca[bi & 1], cb[bi & 1], make_uint2(dwn[bi][0].x, dwn[bi][0].y), make_uint2(dwn[bi][0].z, dwn[bi][0].w), mbf);
                } else {
                    if (QT == UOCR_QT_Q8) group_imma(cc, cd, dwn[bi][0], dwn[bi][1], mbf);
                    else group_imma(cc, cd, make_uint2(dwn[bi][0].x, dwn[bi][0].y), make_uint2(dwn[bi][0].z, dwn[bi][0].w), mbf);
                }
            }
            v[0] = (float)(ca[0][0] + cb[0][0] + ca[1][0] + cb[1][0] + (ca[0][1] + cb[0][1] + ca[1][1] + cb[1][1]) * 256) * (__half2float(dsc4[0]) * ms);
            v[1] = (float)(ca[0][2] + cb[0][2] + ca[1][2] + cb[1][2] + (ca[0][3] + cb[0][3] + ca[1][3] + cb[1][3]) * 256) * (__half2float(dsc4[1]) * ms);
            v[2] = (float)(cc[0] + cd[0] + (cc[1] + cd[1]) * 256) * (__half2float(dsc4[2]) * ms);
            v[3] = (float)(cc[2] + cd[2] + (cc[3] + cd[3]) * 256) * (__half2float(dsc4[3]) * ms);
        } else {
            UOCR_SL_TRACE(3);
            UOCR_SL_TRACE(4);
        }
        UOCR_SL_TRACE(5);         // partial outputs of this CTA
        // ---- one integer reduction per output row into the accumulator, straight from the lane that holds it.  A
        // word carries the number of CTAs that have added to it in its top byte (every CTA adds to every row exactly
        // once per layer), so readers need no separate barrier: a row whose count is complete is complete.
        {
            unsigned long long *mine = acc + (size_t)(cta % R) * H;
            const uint32_t rows[4] = {16u * (warp + 16 * t) + g, 16u * (warp + 16 * t) + 8u + g,
                                      16u * (warp + 64) + g, 16u * (warp + 64) + 8u + g};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (i < 2 || t == 0) {
                    float x = v[i];
                    if (!(fabsf(x) < kSlAccRange)) {      // NaN too: the count must stay intact
                        atomicOr(status, kStatusRange);   // visible before the addition below: whoever sees the full
                        __threadfence();                  // count and then reads the status word sees this bit
                        x = 0.f;
                    }
                    red_add_u64(mine + rows[i], kSlAccOne + (unsigned long long)(__float2ll_rn(x * kSlAccScale) + kSlAccBias));
                }
            }
        }
        UOCR_SL_TRACE(6);         // partial outputs sent

        // ---- while the other CTAs finish: the work for later layers that does not need this layer's result
        if (cta == G - 1) {       // clear the accumulator that the layer after next will add to; the clearing is
                                  // ordered before this CTA's next additions, which every later reader waits for
            unsigned long long *z = prm.acc + (size_t)((prm.acc_base + li + 2) % kSlAccBuffers) * kSlMaxReplicas * H;
            for (uint32_t h = tid; h < R * (uint32_t)H; h += kSlThreads) z[h] = 0ull;
            __threadfence();
        }
        if (!last) {
            if (routed) load_router(s_layers[li + 1].router);
            else fetch_unit(s_layers[li + 1].dec_units + (size_t)(kSharedUnit0 + fg) * Bl::kBytes);
        }

        // ---- the layer's output = next layer's input: every accumulator row once all G CTAs have added to it,
        // + residual, rounded to fp16.  The poll is bounded; a CTA that gives up raises the status word, which
        // the others check while they wait.
        {
            unsigned long long w[3] = {0ull, 0ull, 0ull};
            bool have = true;
            const long long t0 = clock64();
            const unsigned long long full = (unsigned long long)G + prm.expect_extra;
            for (uint32_t polls = 1;; ++polls) {
                bool all = true;           // the thread's (up to) three rows are requested together: one round trip per poll
                unsigned long long nw[3][kSlMaxReplicas];
#pragma unroll
                for (int i = 0; i < 3; ++i) {
                    const int h = tid + i * kSlThreads;
                    const bool need = h < H && (w[i] >> 56) != full;
#pragma unroll
                    for (int r = 0; r < kSlMaxReplicas; ++r) nw[i][r] = (need && (uint32_t)r < R) ? ld_relaxed_u64(acc + (size_t)r * H + h) : 0ull;
                }
#pragma unroll
                for (int i = 0; i < 3; ++i) {
                    const int h = tid + i * kSlThreads;
                    if (h < H && (w[i] >> 56) != full) {
                        unsigned long long s = 0ull;         // counts and sums add up without carrying into each other
#pragma unroll
                        for (int r = 0; r < kSlMaxReplicas; ++r) s += nw[i][r];
                        w[i] = s;
                        if ((s >> 56) != full) all = false;
                    }
                }
                if (all) break;
                if (prm.poll_sleep_ns != 0u) __nanosleep(prm.poll_sleep_ns);
                if ((polls & 15u) == 0u) {
                    if (ld_volatile_u32(status) & (kStatusBarrier | kStatusCopy)) { have = false; break; }
                    if (clock64() - t0 > spin_limit) { atomicOr(status, kStatusBarrier); have = false; break; }
                }
            }
            if (__syncthreads_or(!have || s_flag[1] != 0)) return;
            UOCR_SL_TRACE(7);         // every partial output is in
#pragma unroll
            for (int i = 0; i < 3; ++i) {
                const int h = tid + i * kSlThreads;
                if (h < H) {
                    const long long sum = (long long)(w[i] & (kSlAccOne - 1ull)) - (long long)G * kSlAccBias;
                    float o = (float)sum * (1.0f / kSlAccScale);
                    if (li == 0) o += res0[i];
                    else if (prm.chain_residual) o += __half2float(s_x[h]);
                    s_x[h] = __float2half_rn(o);
                }
            }
        }
        __syncthreads();
        if (last) {
            if (cta == 0) {
                for (int h = tid; h < H; h += kSlThreads) prm.out[h] = s_x[h];
                if (prm.host_status != nullptr) {       // ordered after this CTA saw every contribution of the launch, and (the
                                                        // host may poll the word) after the result has reached host memory
                    __threadfence_system();
                    __syncthreads();
                    if (tid == 0) *prm.host_status = ld_volatile_u32(status);
                }
            }
        } else if (!routed) {
            build_x_frags();
            __syncthreads();
        }
    }
    if (prm.trace != nullptr && tid == 0 && cta == 0) prm.trace[(size_t)127 * prm.count * kSlTracePoints + 1] = clock64();   // kernel exit
#undef UOCR_SL_TRACE
}

// ---------------------------------------------------------------- building the unit blobs
struct RepackSrc {
    const uint8_t *gate_w, *up_w, *down_w;      // first matrix of each kind (file layout)
    const __half *gate_s, *up_s, *down_s;
    uint64_t mat_stride_w;                      // bytes / values from one expert to the next (unused for one matrix set)
    uint64_t mat_stride_s;
    uint32_t inter;                             // F or S: rows of gate / up, columns of down
};

// One CTA per unit: gathers the unit's pieces from the file layout into the blob, 16 bytes at a time.
template <int QT>
__global__ void repack_units_kernel(RepackSrc src, uint8_t *out) {
    using Fm = SlFmt<QT>;
    using Bl = SlBlob<QT>;
    const uint32_t per = src.inter / 64, unit = blockIdx.x, m = unit / per, fg = unit % per;
    const uint8_t *gw = src.gate_w + (size_t)m * src.mat_stride_w + (size_t)fg * 64 * Fm::kRowBytesH;
    const uint8_t *uw = src.up_w + (size_t)m * src.mat_stride_w + (size_t)fg * 64 * Fm::kRowBytesH;
    const uint8_t *dw = src.down_w + (size_t)m * src.mat_stride_w + (size_t)fg * Fm::kGroupBytes;
    const __half *gs = src.gate_s + (size_t)m * src.mat_stride_s + (size_t)fg * 64 * kSlGroups;
    const __half *us = src.up_s + (size_t)m * src.mat_stride_s + (size_t)fg * 64 * kSlGroups;
    const __half *ds = src.down_s + (size_t)m * src.mat_stride_s + fg;
    const uint32_t down_row_bytes = QT == UOCR_QT_Q4 ? src.inter / 2 : src.inter;
    uint8_t *blob = out + (size_t)unit * Bl::kBytes;
    uint4 *gu = reinterpret_cast<uint4 *>(blob + Bl::kGu), *dn = reinterpret_cast<uint4 *>(blob + Bl::kDn);
    __half *gusc = reinterpret_cast<__half *>(blob + Bl::kGuSc), *dnsc = reinterpret_cast<__half *>(blob + Bl::kDnSc);

    for (uint32_t p = threadIdx.x; p < (uint32_t)Bl::kGuBytes / 16; p += blockDim.x) {
        const uint32_t lane = p & 31, g = lane >> 2, t = lane & 3;
        if (QT == UOCR_QT_Q4) {           // [group][row block][lane]: 8 bytes of the gate row, 8 of the up row
            const uint32_t rb = (p >> 5) & 7, Gi = p >> 8;
            const size_t off = (size_t)(8 * rb + g) * Fm::kRowBytesH + Gi * 32 + 8 * t;
            const uint2 a = *reinterpret_cast<const uint2 *>(gw + off), b = *reinterpret_cast<const uint2 *>(uw + off);
            gu[p] = make_uint4(a.x, a.y, b.x, b.y);
        } else {                          // [group][row block][gate, up][lane]: 16 bytes of the row
            const uint32_t mm = (p >> 5) & 1, rb = (p >> 6) & 7, Gi = p >> 9;
            const size_t off = (size_t)(8 * rb + g) * Fm::kRowBytesH + Gi * 64 + 16 * t;
            gu[p] = *reinterpret_cast<const uint4 *>((mm ? uw : gw) + off);
        }
    }
    for (uint32_t i = threadIdx.x; i < 64u * kSlGroups; i += blockDim.x) { gusc[i] = gs[i]; gusc[64 * kSlGroups + i] = us[i]; }
    for (uint32_t p = threadIdx.x; p < (uint32_t)Bl::kDnBytes / 16; p += blockDim.x) {
        const uint32_t lane = p & 31, g = lane >> 2, t = lane & 3;
        if (QT == UOCR_QT_Q4) {           // [row block][lane]: 8 bytes of row g, 8 of row g + 8
            const uint32_t blk = p >> 5;
            const uint8_t *r0 = dw + (size_t)(16 * blk + g) * down_row_bytes + 8 * t;
            const uint2 a = *reinterpret_cast<const uint2 *>(r0), b = *reinterpret_cast<const uint2 *>(r0 + (size_t)8 * down_row_bytes);
            dn[p] = make_uint4(a.x, a.y, b.x, b.y);
        } else {                          // [row block][rows g, rows g + 8][lane]: 16 bytes of the row
            const uint32_t hi = (p >> 5) & 1, blk = p >> 6;
            dn[p] = *reinterpret_cast<const uint4 *>(dw + (size_t)(16 * blk + 8 * hi + g) * down_row_bytes + 16 * t);
        }
    }
    for (uint32_t h = threadIdx.x; h < (uint32_t)kSlH; h += blockDim.x) dnsc[h] = ds[(size_t)h * per];
}

// ---------------------------------------------------------------- host side
// cluster size the kernel is launched with on a device, 0: cannot run there (written when a context is created,
// possibly by several threads at once: same value every time)
static std::atomic<int> g_sliced_cluster[64];
// Co-residency of all CTAs is what the waits between them rely on; a cooperative launch guarantees it.  The
// environment variable UOCR_CUDA_DECODE_COOPERATIVE=0 drops the attribute (measurement only: the grid is smaller
// than the machine, and every wait is bounded, so a launch that is not co-resident ends with an error status).
static std::atomic<int> g_sliced_cooperative{1};

// The shapes and formats this kernel is built for (the model's).
bool decode_sliced_layer_ok(const DLayer &L) {
    const bool q = L.expert_qtype == UOCR_QT_Q4 || L.expert_qtype == UOCR_QT_Q8;
    return q && L.shared_gate.qtype == L.expert_qtype && L.shared_up.qtype == L.expert_qtype &&
           L.shared_down.qtype == L.expert_qtype && L.H == (uint32_t)kSlH && L.F == (uint32_t)kSlF &&
           L.S == (uint32_t)kSlS && L.K == (uint32_t)kSlK && L.E == (uint32_t)kSlE;
}

size_t decode_units_bytes(const DLayer &L) {
    const size_t units = (size_t)kSlE * kSlRoutedPerSlot + kSlS / 64;
    return units * (L.expert_qtype == UOCR_QT_Q4 ? SlBlob<UOCR_QT_Q4>::kBytes : SlBlob<UOCR_QT_Q8>::kBytes);
}

// Fills `out` (decode_units_bytes(L) bytes of device memory) from the layer's file-layout weights.
cudaError_t build_decode_units(const DLayer &L, uint8_t *out, cudaStream_t st) {
    RepackSrc ex{}, sh{};
    ex.gate_w = L.expert_w; ex.up_w = L.expert_w + L.up_offset_bytes; ex.down_w = L.expert_w + L.down_offset_bytes;
    ex.gate_s = L.expert_s; ex.up_s = L.expert_s + L.up_scale_offset; ex.down_s = L.expert_s + L.down_scale_offset;
    ex.mat_stride_w = L.expert_stride_bytes; ex.mat_stride_s = L.expert_scale_stride; ex.inter = L.F;
    sh.gate_w = L.shared_gate.w; sh.up_w = L.shared_up.w; sh.down_w = L.shared_down.w;
    sh.gate_s = L.shared_gate.s; sh.up_s = L.shared_up.s; sh.down_s = L.shared_down.s;
    sh.inter = L.S;
    const uint32_t routed_units = kSlE * kSlRoutedPerSlot, shared_units = kSlS / 64;
    if (L.expert_qtype == UOCR_QT_Q4) {
        repack_units_kernel<UOCR_QT_Q4><<<routed_units, 256, 0, st>>>(ex, out);
        repack_units_kernel<UOCR_QT_Q4><<<shared_units, 256, 0, st>>>(sh, out + (size_t)routed_units * SlBlob<UOCR_QT_Q4>::kBytes);
    } else {
        repack_units_kernel<UOCR_QT_Q8><<<routed_units, 256, 0, st>>>(ex, out);
        repack_units_kernel<UOCR_QT_Q8><<<shared_units, 256, 0, st>>>(sh, out + (size_t)routed_units * SlBlob<UOCR_QT_Q8>::kBytes);
    }
    return cudaGetLastError();
}

template <int QT>
static void launch_config(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attrs, int cluster, cudaStream_t st, uint32_t grid = kSlUnits) {
    *cfg = cudaLaunchConfig_t{};
    cfg->gridDim = dim3(grid); cfg->blockDim = dim3(kSlThreads);
    cfg->dynamicSmemBytes = SlSmem<QT>::kTotal; cfg->stream = st;
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = (unsigned)cluster; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeCooperative; attrs[1].val.cooperative = 1;
    cfg->attrs = attrs; cfg->numAttrs = g_sliced_cooperative.load() ? 2 : 1;
}

// 1 when all CTAs can be resident at once in clusters of kSlCluster, else 0
template <int QT>
static cudaError_t prepare_sliced(int *ok) {
    cudaError_t err = cudaFuncSetAttribute(decode_sliced_kernel<QT, SlicedParams>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)SlSmem<QT>::kTotal);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(decode_sliced_kernel<QT, SlicedParamsInline>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)SlSmem<QT>::kTotal);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(decode_sliced_kernel<QT, SlicedParamsDense>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)SlSmem<QT>::kTotal);
    if (err != cudaSuccess) return err;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attrs[2];
    launch_config<QT>(&cfg, attrs, kSlCluster, nullptr);
    int clusters = 0, clusters_inline = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, decode_sliced_kernel<QT, SlicedParams>, &cfg) != cudaSuccess) { (void)cudaGetLastError(); clusters = 0; }
    if (cudaOccupancyMaxActiveClusters(&clusters_inline, decode_sliced_kernel<QT, SlicedParamsInline>, &cfg) != cudaSuccess) { (void)cudaGetLastError(); clusters_inline = 0; }
    *ok = (clusters * kSlCluster >= kSlUnits && clusters_inline * kSlCluster >= kSlUnits) ? 1 : 0;
    return cudaSuccess;
}

cudaError_t init_decode_sliced_kernels() {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (const char *c = getenv("UOCR_CUDA_DECODE_COOPERATIVE")) g_sliced_cooperative = c[0] == '0' ? 0 : 1;
    int ok4 = 0, ok8 = 0;
    if ((err = prepare_sliced<UOCR_QT_Q4>(&ok4)) != cudaSuccess) return err;
    if ((err = prepare_sliced<UOCR_QT_Q8>(&ok8)) != cudaSuccess) return err;
    if (dev >= 0 && dev < 64) g_sliced_cluster[dev] = (ok4 && ok8) ? kSlCluster : 0;
    return cudaSuccess;
}

size_t decode_sliced_acc_bytes() { return (size_t)kSlAccBuffers * kSlMaxReplicas * kSlH * sizeof(unsigned long long); }

bool decode_sliced_supported(const DLayer *layers, uint32_t first, uint32_t count) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || g_sliced_cluster[dev] == 0) return false;
    if (count == 0 || count > (uint32_t)kSlMaxLayers) return false;
    for (uint32_t i = 0; i < count; ++i) {
        const DLayer &L = layers[first + i];
        if (!decode_sliced_layer_ok(L) || L.dec_units == nullptr || L.expert_qtype != layers[first].expert_qtype) return false;
    }
    return true;
}

template <int QT, class Params>
static cudaError_t launch_one(const Params &prm, int cluster, cudaStream_t st, uint32_t grid = kSlUnits) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attrs[2];
    launch_config<QT>(&cfg, attrs, cluster, st, grid);
    return cudaLaunchKernelEx(&cfg, decode_sliced_kernel<QT, Params>, prm);
}

// acc: decode_sliced_acc_bytes() of device memory, zero before the first launch; *acc_base carries the accumulator
// rotation from launch to launch (reset it, and clear acc, after a failed launch).  host_status: device address of a
// word in mapped host memory that receives the status word once `out` is complete, or null.  h_inline: host pointer to the H
// fp16 activations, copied into the launch parameters (hidden and residual0 are then unused; the first layer's
// residual is the input itself when chain_residual is set), or null.  knobs: accumulator replicas, the limit of the
// waits between CTAs, and the test hook that makes the first wait run out.
cudaError_t launch_decode_sliced(const DLayer *h_layers, const DLayer *d_layers, uint32_t first, uint32_t count,
                                 const __half *hidden, const __half *residual0, const void *h_inline, int chain_residual,
                                 const float *injected,
                                 __half *out, uint32_t *host_status, unsigned long long *acc, uint32_t *acc_base, uint32_t *status,
                                 float *dbg_logits, float *dbg_probs, uint32_t *ids_out, float *wts_out,
                                 unsigned long long *trace, const SlicedKnobs &knobs, cudaStream_t st, uint64_t *launches,
                                 const __half *norm_weight, float norm_eps) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64 || g_sliced_cluster[dev] == 0) return cudaErrorNotSupported;
    const int cluster = g_sliced_cluster[dev];
    SlicedParamsInline prm{};
    prm.layers = d_layers; prm.first = first; prm.count = count;
    prm.hidden_in = hidden; prm.residual0 = residual0; prm.chain_residual = chain_residual;
    prm.injected = injected; prm.out = out; prm.acc = acc; prm.acc_base = *acc_base;
    prm.replicas = (knobs.replicas == 1 || knobs.replicas == 2 || knobs.replicas == 4) ? knobs.replicas : 1u;
    prm.status = status; prm.host_status = host_status;
    prm.spin_limit = knobs.spin_limit_cycles > 0 ? knobs.spin_limit_cycles : kSpinLimit;
    prm.expect_extra = knobs.expect_extra;
    prm.poll_sleep_ns = knobs.poll_sleep_ns;
    prm.dbg_logits = dbg_logits; prm.dbg_probs = dbg_probs; prm.ids_out = ids_out; prm.wts_out = wts_out; prm.trace = trace;
    prm.norm_weight = h_inline != nullptr ? nullptr : norm_weight; prm.norm_eps = norm_eps;
    prm.router0 = h_layers[first].router; prm.units0 = h_layers[first].dec_units;
    const bool q4 = h_layers[first].expert_qtype == UOCR_QT_Q4;
    if (h_inline != nullptr) {
        memcpy(prm.inline_x, h_inline, sizeof(prm.inline_x));
        err = q4 ? launch_one<UOCR_QT_Q4, SlicedParamsInline>(prm, cluster, st) : launch_one<UOCR_QT_Q8, SlicedParamsInline>(prm, cluster, st);
    } else {
        const SlicedParams &base = prm;
        err = q4 ? launch_one<UOCR_QT_Q4, SlicedParams>(base, cluster, st) : launch_one<UOCR_QT_Q8, SlicedParams>(base, cluster, st);
    }
    if (err != cudaSuccess) return err;
    *acc_base = (*acc_base + count) % kSlAccBuffers;
    ++*launches;
    return cudaSuccess;
}

// ---- a dense SwiGLU MLP of the model's hidden size through the same kernel, one token --------------------------------
// Units of 64 intermediate columns, padded with all-zero units to a multiple of the cluster size; every unit needs an SM
// of its own (the CTAs wait for one another), so the width is limited by the device.
uint32_t decode_dense_units(uint32_t hidden, uint32_t inter, int gate_qtype, int up_qtype, int down_qtype) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || g_sliced_cluster[dev] == 0) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (hidden != (uint32_t)kSlH || inter == 0 || inter % 64 != 0) return 0;
    if ((gate_qtype != UOCR_QT_Q4 && gate_qtype != UOCR_QT_Q8) || up_qtype != gate_qtype || down_qtype != gate_qtype) return 0;
    const uint32_t units = (inter / 64 + kSlCluster - 1) / kSlCluster * kSlCluster;
    return units <= (uint32_t)sms ? units : 0;
}

size_t decode_dense_units_bytes(int qtype, uint32_t units) {
    return (size_t)units * (qtype == UOCR_QT_Q4 ? SlBlob<UOCR_QT_Q4>::kBytes : SlBlob<UOCR_QT_Q8>::kBytes);
}

// out: decode_dense_units_bytes() of device memory
cudaError_t build_dense_units(const DMatrix &gate, const DMatrix &up, const DMatrix &down, uint32_t units, uint8_t *out, cudaStream_t st) {
    cudaError_t err = cudaMemsetAsync(out, 0, decode_dense_units_bytes(gate.qtype, units), st);
    if (err != cudaSuccess) return err;
    RepackSrc src{};
    src.gate_w = gate.w; src.up_w = up.w; src.down_w = down.w;
    src.gate_s = gate.s; src.up_s = up.s; src.down_s = down.s;
    src.inter = gate.rows;
    if (gate.qtype == UOCR_QT_Q4) repack_units_kernel<UOCR_QT_Q4><<<gate.rows / 64, 256, 0, st>>>(src, out);
    else repack_units_kernel<UOCR_QT_Q8><<<gate.rows / 64, 256, 0, st>>>(src, out);
    return cudaGetLastError();
}

// d_layer: device copy of a DLayer whose dec_units point at the units (unit_blobs, the same address); out = fp16( MLP(hidden) + residual ).  Accumulators,
// their rotation and the knobs as for launch_decode_sliced.
cudaError_t launch_decode_dense(const DLayer *d_layer, const uint8_t *unit_blobs, int qtype, uint32_t units, const __half *hidden, const __half *residual,
                                __half *out, unsigned long long *acc, uint32_t *acc_base, uint32_t *status, const SlicedKnobs &knobs,
                                cudaStream_t st, uint64_t *launches, const __half *norm_weight, float norm_eps) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64 || g_sliced_cluster[dev] == 0 || units == 0 || units % kSlCluster != 0) return cudaErrorNotSupported;
    SlicedParamsDense prm{};
    prm.layers = d_layer; prm.first = 0; prm.count = 1;
    prm.hidden_in = hidden; prm.residual0 = residual; prm.chain_residual = 0;
    prm.out = out; prm.acc = acc; prm.acc_base = *acc_base;
    prm.replicas = (knobs.replicas == 1 || knobs.replicas == 2 || knobs.replicas == 4) ? knobs.replicas : 1u;
    prm.status = status;
    prm.spin_limit = knobs.spin_limit_cycles > 0 ? knobs.spin_limit_cycles : kSpinLimit;
    prm.expect_extra = knobs.expect_extra;
    prm.poll_sleep_ns = knobs.poll_sleep_ns;
    prm.norm_weight = norm_weight; prm.norm_eps = norm_eps;
    prm.router0 = nullptr; prm.units0 = unit_blobs;
    err = qtype == UOCR_QT_Q4 ? launch_one<UOCR_QT_Q4, SlicedParamsDense>(prm, g_sliced_cluster[dev], st, units)
                              : launch_one<UOCR_QT_Q8, SlicedParamsDense>(prm, g_sliced_cluster[dev], st, units);
    if (err != cudaSuccess) return err;
    *acc_base = (*acc_base + 1) % kSlAccBuffers;
    ++*launches;
    return cudaSuccess;
}

}  // namespace uocr

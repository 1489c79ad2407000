// Many-token MoE layer: expert-grouped GEMMs on the 5th-generation tensor cores.
//
// After the dispatch plan the (token, slot) pairs of one expert are contiguous, so each expert is a
// dense product.  Both products are computed "weights as rows": a tile is 128 tensor-memory lanes of weight rows
// against up to 192 tokens,
//     gate/up :  64 gate rows interleaved with the 64 matching up rows, K = H  ->
//                mid[pos][f] = fp16( silu(gate) * up )   (the two accumulators of an output sit in neighbouring lanes)
//     down    :  128 weight rows, K = F (or S)  ->  down_out[pos][h] = fp16(acc)
// With the weights on the M side of the MMA a cold expert with a handful of tokens pads its token
// count to 16, not to 128, which matters under Zipf-skewed routing.
//
// One persistent CTA per SM (704 threads; it owns all 512 tensor-memory columns: two accumulators of 192 columns and
// a ring of four 32-column slots for the weight operand) walks its share of the tile list.  Per 64-wide K block
// (= one scale group of the weight formats, = one 128-byte swizzle row of fp16):
//   warps 0-15 four threads per lane: each loads its 16 weights' packed bytes with a 128-bit load (several K blocks
//              ahead), turns them into fp16( level * scale ) in registers and stores them with tcgen05.st straight
//              into the ring of tensor-memory slots, the A operand of the MMA: no dequantised weight ever reaches
//              shared or global memory.  A slot is published one block late, so the stores' latency hides behind
//              the next conversion.  These warps never wait for an accumulator: they run on into the next tile.
//   warps 16-19 the epilogue of the PREVIOUS tile (tcgen05.ld, SwiGLU with the fast exponential, fp16 stores) while
//              the tensor core accumulates the current one in the other accumulator.
//   warp 20    one thread issues the TMA tile loads (cp.async.bulk.tensor) of the activation tile.
//   warp 21    one thread issues tcgen05.mma (kind::f16, A from tensor memory, B from shared memory, fp32
//              accumulators in tensor memory) and commits the slots back; the warp also owns the TMEM allocation.
// Every wait is bounded; on a time-out the CTA raises a status bit, drains and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>

#include "moe_common.cuh"

namespace uocr {

constexpr int kGemmThreads = 704;        // warps 0-15 converters, 16-19 epilogue, warp 20 TMA, warp 21 MMA
constexpr int kProducerThreads = 512;
constexpr int kEpilogueWarps = 4;
constexpr int kTmaWarp = 20, kMmaWarp = 21;
constexpr int kTileM = 128;          // TMEM lanes per tile: 128 rows of down, or 64 rows of gate interleaved with 64 of up
constexpr int kTileN = 192;          // tokens per tile: a tcgen05.mma costs about 106 cycles whatever its N up to 192 (measured),
                                     // and two accumulators of 192 columns leave 128 columns for the weight operand
constexpr int kBlockK = 64;          // fp16 elements per K block = 128 bytes = one swizzle row
constexpr int kTileBytes = kTileM * kBlockK * 2;   // 16 KB: one operand tile of one stage
constexpr long long kGemmSpinLimit = 400000000LL;    // cycles (~0.2 s): no legitimate wait comes near
constexpr uint32_t kStatusGemm = 8u;

struct GemmParams {
    const uint8_t *w0, *w1;        // packed weights: gate and up (gate/up mode) or down (w1 unused)
    const __half *s0, *s1;         // their scales (null for fp16 weights)
    uint64_t expert_stride_bytes;  // between experts in the packed slab (0 for the shared MLP)
    uint64_t expert_scale_stride;  // in values
    uint32_t row_bytes;            // packed bytes of one weight row
    uint32_t k_dim;                // input width K (multiple of 64)
    const uint4 *tiles;            // {expert, weight-row tile, first row of the activation matrix, rows}
    const uint32_t *tile_count;
    __half *out;                   // mid / down_out, [rows][out_ld]
    uint32_t out_ld;
    uint32_t *status;
};

// ---------------------------------------------------------------------------------- PTX
__device__ __forceinline__ uint32_t s2u(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void gb_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s2u(bar)), "r"(count));
}
__device__ __forceinline__ void gb_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s2u(bar)) : "memory");
}
__device__ __forceinline__ void gb_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s2u(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool gb_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(s2u(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; also gives up as soon as another role of the CTA has raised the abort flag.  RELAXED waits sleep between
// polls: the roles that run ahead of the tensor core (converters, activation loader) or behind it (epilogue) spend much
// of their time waiting, and a warp that polls in a tight loop takes issue slots from the one thread whose instruction
// stream feeds the tensor core.
template <bool RELAXED = false>
__device__ __forceinline__ bool gb_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, uint32_t *status) {
    if (gb_try(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t polls = 0;
    while (!gb_try(bar, parity)) {
        if (RELAXED) __nanosleep(40);
        if ((++polls & (RELAXED ? 15u : 255u)) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kGemmSpinLimit) {
                *abort_flag = 1;
                atomicOr(status, kStatusGemm);
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(s2u(dst)), "l"(map), "r"(x), "r"(y), "r"(s2u(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s2u(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, fp16 inputs, fp32 accumulate, M = 128, N from the descriptor, K = 16
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile, 128-byte rows, 128B swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: fp16 A and B (K-major), fp32 D, M = 128, N = n
__device__ __forceinline__ uint32_t umma_idesc(uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
}

// ---------------------------------------------------------------------- dequantisation
// The weight operand never touches shared memory: each producer thread converts 16 packed weights of its
// row to fp16( level * scale ) in registers and writes them straight into tensor memory (tcgen05.st), from
// where the MMA reads its A operand.  Shared memory then carries only the activation tiles, which keeps its
// bandwidth below what the tensor cores need.
//
// A in tensor memory for kind::f16, M = 128: element (row m, k) sits in lane m, 32-bit column k / 2, the even k
// in the low half.  A 32-wide K sub-block of one matrix is 16 columns.

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// four bytes holding values 0..255 in a word -> two half2 (b0,b1), (b2,b3) of (value - bias) * scale, each
// product rounded to fp16 once: fp16( float(level) * float(scale) ), the value the reference's tiled GEMMs feed
// their MMA (src/backend/metal/kernels/gemm_q4.metal:35-57, gemm_q8.metal:43-60).
__device__ __forceinline__ void bytes_to_h2(uint32_t bytes, __half2 bias, __half2 scale, uint32_t &lo, uint32_t &hi) {
    const uint32_t a = __byte_perm(bytes, 0x64646464u, 0x5140);   // [b0, 0x64, b1, 0x64] = (1024 + b0, 1024 + b1)
    const uint32_t b = __byte_perm(bytes, 0x64646464u, 0x5342);   // (1024 + b2, 1024 + b3)
    lo = h2_as_u32(__hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&a), bias), scale));
    hi = h2_as_u32(__hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&b), bias), scale));
}

// Packed bytes of one row and one 64-wide K block (one scale group), as 16-byte vectors.  kAhead: how many K blocks
// of packed bytes a thread keeps in flight from global memory.
template <int QT> struct PackedBlock;
template <> struct PackedBlock<UOCR_QT_Q4> { static constexpr int kVecs = 2; static constexpr int kAhead = 3; };
template <> struct PackedBlock<UOCR_QT_Q8> { static constexpr int kVecs = 4; static constexpr int kAhead = 2; };
template <> struct PackedBlock<UOCR_QT_F16> { static constexpr int kVecs = 8; static constexpr int kAhead = 1; };

template <int QT>
__device__ __forceinline__ void load_block(const uint8_t *row, uint32_t kb, uint4 (&v)[PackedBlock<QT>::kVecs]) {
    const uint4 *p = reinterpret_cast<const uint4 *>(row) + (size_t)kb * PackedBlock<QT>::kVecs;
#pragma unroll
    for (int i = 0; i < PackedBlock<QT>::kVecs; ++i) v[i] = __ldg(p + i);
}

// The 16 weights at K positions [32 j + 16 h, +16) of the block -> 8 registers of two fp16 each, in K order.
// Q4_0: bytes 16h..16h+15 of the group's 32 (low nibbles: sub-block j = 0, high nibbles: j = 1).
// Q8_0: bytes 32j + 16h .. +15.   fp16: halves 32j + 16h .. +15.
template <int QT>
__device__ __forceinline__ void convert_sub(const uint4 (&v)[PackedBlock<QT>::kVecs], int j, int h, __half scale, uint32_t (&out)[8]) {
    if constexpr (QT == UOCR_QT_F16) {
        const uint4 a = v[4 * j + 2 * h], b = v[4 * j + 2 * h + 1];
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    } else if constexpr (QT == UOCR_QT_Q8) {
        const __half2 s2 = __half2half2(scale), bias = __float2half2_rn(1152.f);   // 1024 + 128
        const uint4 q = v[2 * j + h];
        bytes_to_h2(q.x ^ 0x80808080u, bias, s2, out[0], out[1]);
        bytes_to_h2(q.y ^ 0x80808080u, bias, s2, out[2], out[3]);
        bytes_to_h2(q.z ^ 0x80808080u, bias, s2, out[4], out[5]);
        bytes_to_h2(q.w ^ 0x80808080u, bias, s2, out[6], out[7]);
    } else {
        const __half2 s2 = __half2half2(scale), bias = __float2half2_rn(1032.f);    // 1024 + 8
        const uint4 q = v[h];
        const int sh = 4 * j;
        bytes_to_h2((q.x >> sh) & 0x0F0F0F0Fu, bias, s2, out[0], out[1]);
        bytes_to_h2((q.y >> sh) & 0x0F0F0F0Fu, bias, s2, out[2], out[3]);
        bytes_to_h2((q.z >> sh) & 0x0F0F0F0Fu, bias, s2, out[4], out[5]);
        bytes_to_h2((q.w >> sh) & 0x0F0F0F0Fu, bias, s2, out[6], out[7]);
    }
}

// eight 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]^T
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// The same MMA and the commit, issued by one elected lane of a warp whose lanes all run the issuing loop.  Measured on
// this part: with the loop inside an `if (lane == 0)` branch an MMA costs the issuing thread 106 - 164 cycles whatever its
// N; with warp-uniform control flow and `elect.sync` it costs 91 cycles up to N = 128, 96 at N = 192 and 128 at N = 256,
// i.e. the tensor core's own rate.
__device__ __forceinline__ void tc_mma_ts_elect(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit_elect(uint64_t *bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(s2u(bar)) : "memory");
}

// silu with the fast exponential and reciprocal (about 2 ulp; the result is rounded to fp16 anyway)
__device__ __forceinline__ float silu_fast(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// ------------------------------------------------------------------------------ kernel
// One tile = 128 tensor-memory lanes x up to 192 tokens.  down: lane r is weight row 128*mtile + r.  gate/up: the two
// matrices are interleaved, lane 2i is gate row 64*mtile + i and lane 2i+1 is up row 64*mtile + i, so the SwiGLU
// partner of an accumulator sits in the neighbouring lane of the same warp and the epilogue needs one shuffle.
// Tensor-memory columns: two accumulators of 192 columns (tile i+1 accumulates while tile i is read out), then
// kAStages slots of 32 columns (one 64-wide K block of the 128 lanes).
#ifndef UOCR_GEMM_ABLATE
#define UOCR_GEMM_ABLATE 0      // development builds only: 1 no tensor-memory stores, 2 no activation loads, 4 no epilogue work, 8 no MMAs,
                                // 16 no epilogue stores, 32 no SwiGLU arithmetic in the epilogue
#endif
#ifdef UOCR_GEMM_TRACE
// Development build only: cycles every role of the kernel spends waiting, summed over CTAs ([gate/up or down][counter]).
__device__ unsigned long long g_gemm_trace[2][16];
#define GT_BEGIN(var) const long long var = clock64()
#define GT_ADD(slot, var) gt_local[slot] += (unsigned long long)(clock64() - var)
#else
#define GT_BEGIN(var)
#define GT_ADD(slot, var)
#endif

struct GemmShape {
    static constexpr int kTileN = uocr::kTileN;                        // tokens per tile = columns per accumulator
    static constexpr int kAccBufs = 2;
    static constexpr int kStages = 4;                                  // ring depth, the same for both operands
    static constexpr int kAccCols = kAccBufs * kTileN;                 // 384
    static constexpr int kAStageCols = 32;
    static constexpr int kTmemCols = 512;
    static_assert(kAccCols + kStages * kAStageCols <= kTmemCols, "tensor memory budget");
    static constexpr int kBTileBytes = kTileN * kBlockK * 2;           // 24 KB
    static constexpr int kBarrierBytes = 256;
    static constexpr int kEpiStageBytes = 1024;                        // per epilogue warp: 16 tokens x 32 output columns of fp16
    static constexpr int kSmemBytes = kStages * kBTileBytes + kBarrierBytes + kEpilogueWarps * kEpiStageBytes + 1024 /*alignment*/;
};

template <int QT, bool GATEUP>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap act_map, GemmParams p) {
    using Sh = GemmShape;
    constexpr int kStages = Sh::kStages, kTileN = Sh::kTileN;
    // Persistent: the grid has at most one CTA per SM, and CTA b takes tiles b, b + gridDim.x, ... of the list (hottest
    // expert first).  Barriers and tensor memory are set up once.  The CTA's K blocks form ONE running sequence across
    // its tiles (block q of the sequence uses ring stage q % 4); every role walks that sequence on its own: the
    // activation loader and the converters work ahead into the next tiles while the tensor core finishes the current
    // one and the epilogue warps read out the one before.  Nothing synchronises the roles at a tile boundary.
    const uint32_t n_tiles = *p.tile_count;
    if (blockIdx.x >= n_tiles) return;
    const uint32_t kblocks = p.k_dim / kBlockK;
    const uint32_t my_tiles = (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
    const uint32_t total_blocks = my_tiles * kblocks;

    extern __shared__ uint8_t smem_dyn[];
    uint8_t *b_tiles = reinterpret_cast<uint8_t *>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(b_tiles + kStages * Sh::kBTileBytes);
    // full[s]: the stage's weights are in tensor memory (one arrival per converter warp of the owning group) and its
    // activation tile has landed (the loader's arrival + byte count); empty[s]: the MMAs that read it have finished
    uint64_t *full = bars, *empty = full + kStages, *acc_full = empty + kStages, *acc_empty = acc_full + Sh::kAccBufs;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + Sh::kAccBufs);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    static_assert((2 * kStages + 2 * Sh::kAccBufs) * 8 + 8 <= Sh::kBarrierBytes, "barrier block");
    uint8_t *epi_stage = b_tiles + kStages * Sh::kBTileBytes + Sh::kBarrierBytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { gb_init(&full[s], kTileM / 32 + 1); gb_init(&empty[s], 1); }
        for (int s = 0; s < Sh::kAccBufs; ++s) { gb_init(&acc_full[s], 1); gb_init(&acc_empty[s], kEpilogueWarps); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)), "r"((uint32_t)Sh::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t a_base = tmem_base + Sh::kAccCols;       // first column of the weight-operand slots

    if (warp < kProducerThreads / 32) {
        // ------------------------------------------------ weight rows -> fp16 -> tensor memory
        // Four groups of four warps.  Group g owns the blocks q = g, g + 4, ... of the CTA's sequence, hence ring stage g,
        // and converts each of them whole: thread r of the group turns the 64 weights of lane r's row into 32
        // tensor-memory columns.  The groups work on different K blocks at the same time, so the latencies inside one
        // block's conversion overlap with the other groups' arithmetic.  A thread keeps the packed bytes and the scale
        // of its next kAhead blocks in registers; that prefetch runs across tile boundaries.
        constexpr int kGroups = kProducerThreads / kTileM;
        static_assert(kGroups == kStages, "one ring stage per converter group");
        const int grp = tid >> 7, r = tid & 127;
        constexpr int kAhead = PackedBlock<QT>::kAhead, kVecs = PackedBlock<QT>::kVecs;
        const uint32_t dst = a_base + (uint32_t)grp * Sh::kAStageCols + ((uint32_t)((warp & 3) * 32) << 16);
        const bool second = GATEUP && (r & 1);                        // this lane holds a row of the up matrix
        const uint8_t *wbase = second ? p.w1 : p.w0;
        const __half *sbase = second ? p.s1 : p.s0;
#ifdef UOCR_GEMM_TRACE
        unsigned long long gt_local[5] = {0, 0, 0, 0, 0};
        GT_BEGIN(gt_all);
#endif
        // prefetch cursor: tile and K block of the next block to request
        uint32_t pf_tile = blockIdx.x, pf_kb = (uint32_t)grp;
        const uint8_t *pf_row = nullptr;
        const unsigned short *pf_sc = nullptr;
        auto pf_enter_tile = [&]() {
            if (pf_tile < n_tiles) {
                const uint4 tile = p.tiles[pf_tile];
                const size_t grow = GATEUP ? (size_t)tile.y * (kTileM / 2) + (r >> 1) : (size_t)tile.y * kTileM + r;   // row of the matrix
                pf_row = wbase + (size_t)tile.x * p.expert_stride_bytes + grow * p.row_bytes;
                if (QT != UOCR_QT_F16)
                    pf_sc = reinterpret_cast<const unsigned short *>(sbase + (size_t)tile.x * p.expert_scale_stride + grow * kblocks);
            }
        };
        auto pf_settle = [&]() {                                      // carry the K block index over into the next tiles
            bool moved = false;
            while (pf_kb >= kblocks) { pf_kb -= kblocks; pf_tile += gridDim.x; moved = true; }
            if (moved) pf_enter_tile();
        };
        auto pf_fetch = [&](uint4 (&vv)[kVecs], unsigned short &sc) {
            if (pf_tile < n_tiles) {
                load_block<QT>(pf_row, pf_kb, vv);
                if (QT != UOCR_QT_F16) sc = __ldg(pf_sc + pf_kb);
            }
            pf_kb += kGroups;
            pf_settle();
        };
        pf_enter_tile();
        pf_settle();
        uint4 v[kAhead][kVecs];
        unsigned short scv[kAhead];
#pragma unroll
        for (int d = 0; d < kAhead; ++d) { scv[d] = 0; pf_fetch(v[d], scv[d]); }

        bool alive = true;
        uint32_t use = 0;                                             // how many blocks this group has stored so far
#pragma unroll 1
        for (uint32_t q0 = (uint32_t)grp; q0 < total_blocks && alive; q0 += kGroups * kAhead) {
#pragma unroll
            for (int d = 0; d < kAhead; ++d) {
                if (q0 + (uint32_t)d * kGroups >= total_blocks) break;
                const __half sc = __ushort_as_half(scv[d]);
                // the first half of the block is converted before the stage is waited for: when the tensor core frees
                // the stage, half of the work that stands between "free" and "full again" is already done
                uint32_t regs[2][8];
                convert_sub<QT>(v[d], 0, 0, sc, regs[0]);
                convert_sub<QT>(v[d], 0, 1, sc, regs[1]);
                GT_BEGIN(gt_w);
                if (use > 0 && !gb_wait<true>(&empty[grp], (use - 1) & 1u, abort_flag, p.status)) { alive = false; break; }
                GT_ADD(0, gt_w);
                __syncwarp();
                tc_fence_after();
                GT_BEGIN(gt_s);
                if (!(UOCR_GEMM_ABLATE & 1)) { tc_st8(dst, regs[0]); tc_st8(dst + 8u, regs[1]); }
                else if (regs[0][0] == 0x12345u && regs[1][7] == 0x54321u) *abort_flag = 2;
                GT_ADD(4, gt_s);
                convert_sub<QT>(v[d], 1, 0, sc, regs[0]);
                convert_sub<QT>(v[d], 1, 1, sc, regs[1]);
                if (!(UOCR_GEMM_ABLATE & 1)) { tc_st8(dst + 16u, regs[0]); tc_st8(dst + 24u, regs[1]); }
                else if (regs[0][0] == 0x12345u && regs[1][7] == 0x54321u) *abort_flag = 2;
                {   // publish at once: the other three groups keep the arithmetic units busy while these stores land
                    GT_BEGIN(gt_p);
                    tc_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) gb_arrive(&full[grp]);              // one arrival per warp: its stores have all landed
                    GT_ADD(3, gt_p);
                }
                pf_fetch(v[d], scv[d]);                                // the registers are free: request the block kAhead rounds on
                ++use;
            }
        }
#ifdef UOCR_GEMM_TRACE
        GT_ADD(2, gt_all);
        if (tid == 0) {
            atomicAdd(&g_gemm_trace[GATEUP][0], gt_local[0]);     // converters: waiting for a free slot
            atomicAdd(&g_gemm_trace[GATEUP][2], gt_local[2]);     // converters: whole loop
            atomicAdd(&g_gemm_trace[GATEUP][13], gt_local[3]);    // converters: publishing (wait for the stores, arrive)
            atomicAdd(&g_gemm_trace[GATEUP][14], gt_local[4]);    // converters: issuing the first two stores of a block
        }
#endif
    } else if (warp < kTmaWarp) {
        // ------------------------------------------------ epilogue: TMEM -> registers -> global, one tile behind the MMAs
        // Warp q of the four reads the TMEM lanes 32 q .. 32 q + 31 (the hardware ties a warp to the lane quarter
        // warp % 4), sixteen token columns at a time.
        const uint32_t q = (uint32_t)(warp & 3);
        const bool odd = (lane & 1) != 0;
        uint32_t it = 0;
#ifdef UOCR_GEMM_TRACE
        unsigned long long gt_local[3] = {0, 0, 0};
        GT_BEGIN(gt_all);
#endif
        uint4 tile = p.tiles[blockIdx.x];
#pragma unroll 1
        for (uint32_t tile_idx = blockIdx.x; tile_idx < n_tiles; tile_idx += gridDim.x, ++it) {
            const uint32_t mtile = tile.y, row0 = tile.z, nrows = tile.w, buf = it & 1u;
            if (tile_idx + gridDim.x < n_tiles) tile = p.tiles[tile_idx + gridDim.x];       // the next tile's entry, requested early
            GT_BEGIN(gt_w);
            const bool have_acc = gb_wait<true>(&acc_full[buf], (it >> 1) & 1u, abort_flag, p.status);
            GT_ADD(0, gt_w);
            __syncwarp();
            if (!__all_sync(0xffffffffu, have_acc)) break;
            tc_fence_after();
            const uint32_t src = tmem_base + buf * (uint32_t)kTileN + ((q * 32u) << 16);
            const uint32_t last_chunk = (nrows - 1u) / 16u;
#pragma unroll 1
            for (uint32_t c = (UOCR_GEMM_ABLATE & 4) ? last_chunk : 0u; c <= last_chunk; ++c) {
                uint32_t a[16];
                GT_BEGIN(gt_l);
                tc_ld16(src + 16u * c, a);
                tc_ld_wait();
                GT_ADD(2, gt_l);
                if (c == last_chunk) {
                    // the accumulator has been read: the tensor core may start the tile after the next in it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) gb_arrive(&acc_empty[buf]);
                }
                // Two-byte stores scattered over sixteen token rows cost the load/store unit about as much as sixteen
                // 16-byte ones, so the chunk is transposed through a 1 KB staging tile of this warp: neighbouring lanes
                // pair their values into 32-bit words, and every token row then leaves as 16-byte stores.
                const uint32_t t0 = 16u * c;
                uint32_t *stage32 = reinterpret_cast<uint32_t *>(epi_stage + (size_t)(warp - kProducerThreads / 32) * Sh::kEpiStageBytes);
                if (GATEUP) {
                    // even lanes hold gate rows, odd lanes the matching up rows: the even lane computes the pair's output
                    // for the even tokens, the odd lane for the odd ones (one exchange per token pair)
                    uint32_t o[8];
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) {
                        const uint32_t recv = __shfl_xor_sync(0xffffffffu, odd ? a[2 * jj] : a[2 * jj + 1], 1);
                        const float g = __uint_as_float(odd ? recv : a[2 * jj]);
                        const float u = __uint_as_float(odd ? a[2 * jj + 1] : recv);
                        o[jj] = (uint32_t)__half_as_ushort(__float2half_rn((UOCR_GEMM_ABLATE & 32) ? g : silu_fast(g) * u));
                    }
                    // lanes l and l ^ 2 hold neighbouring output columns of the same tokens: pair them up
                    const bool hi2 = (lane & 2) != 0;
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const uint32_t recv = __shfl_xor_sync(0xffffffffu, hi2 ? o[2 * m] : o[2 * m + 1], 2);
                        const uint32_t word = hi2 ? (recv | (o[2 * m + 1] << 16)) : (o[2 * m] | (recv << 16));
                        const uint32_t token = 2u * (2u * m + (hi2 ? 1u : 0u)) + (odd ? 1u : 0u);
                        stage32[token * 8u + ((uint32_t)lane >> 2)] = word;          // [16 tokens][8 words]
                    }
                    __syncwarp();
                    const uint32_t token = (uint32_t)lane >> 1, part = (uint32_t)lane & 1u;
                    const uint4 vec = *reinterpret_cast<const uint4 *>(stage32 + token * 8u + part * 4u);
                    if (!(UOCR_GEMM_ABLATE & 16) && t0 + token < nrows)
                        *reinterpret_cast<uint4 *>(p.out + (size_t)(row0 + t0 + token) * p.out_ld + (size_t)mtile * (kTileM / 2) + q * 16u + part * 8u) = vec;
                    __syncwarp();
                } else {
#pragma unroll
                    for (int m = 0; m < 8; ++m) {
                        const uint32_t v0 = (uint32_t)__half_as_ushort(__float2half_rn(__uint_as_float(a[2 * m])));
                        const uint32_t v1 = (uint32_t)__half_as_ushort(__float2half_rn(__uint_as_float(a[2 * m + 1])));
                        const uint32_t recv = __shfl_xor_sync(0xffffffffu, odd ? v0 : v1, 1);
                        const uint32_t word = odd ? (recv | (v1 << 16)) : (v0 | (recv << 16));
                        stage32[(2u * m + (odd ? 1u : 0u)) * 16u + ((uint32_t)lane >> 1)] = word;    // [16 tokens][16 words]
                    }
                    __syncwarp();
#pragma unroll
                    for (int pass = 0; pass < 2; ++pass) {
                        const uint32_t token = 8u * pass + ((uint32_t)lane >> 2), part = (uint32_t)lane & 3u;
                        const uint4 vec = *reinterpret_cast<const uint4 *>(stage32 + token * 16u + part * 4u);
                        if (!(UOCR_GEMM_ABLATE & 16) && t0 + token < nrows)
                            *reinterpret_cast<uint4 *>(p.out + (size_t)(row0 + t0 + token) * p.out_ld + (size_t)mtile * kTileM + q * 32u + part * 8u) = vec;
                    }
                    __syncwarp();
                }
            }
        }
#ifdef UOCR_GEMM_TRACE
        GT_ADD(1, gt_all);
        if (warp == kProducerThreads / 32 && lane == 0) {
            atomicAdd(&g_gemm_trace[GATEUP][3], gt_local[0]);     // epilogue: waiting for an accumulator
            atomicAdd(&g_gemm_trace[GATEUP][4], gt_local[1]);     // epilogue: whole loop
            atomicAdd(&g_gemm_trace[GATEUP][15], gt_local[2]);    // epilogue: tensor-memory loads
        }
#endif
    } else if (warp == kTmaWarp) {
        // ------------------------------------------------ activation tiles by TMA (runs ahead into the next tiles)
        if (lane == 0) {
            uint32_t q = 0;
            bool ok = true;
#ifdef UOCR_GEMM_TRACE
            unsigned long long gt_local[1] = {0};
#endif
            uint32_t row0 = p.tiles[blockIdx.x].z;
            for (uint32_t tile_idx = blockIdx.x; tile_idx < n_tiles && ok; tile_idx += gridDim.x) {
                const uint32_t cur_row0 = row0;
                if (tile_idx + gridDim.x < n_tiles) row0 = p.tiles[tile_idx + gridDim.x].z;
                for (uint32_t kb = 0; kb < kblocks; ++kb, ++q) {
                    const uint32_t s = q % kStages, use = q / kStages;
                    GT_BEGIN(gt_w);
                    if (use > 0 && !gb_wait<true>(&empty[s], (use - 1) & 1u, abort_flag, p.status)) { ok = false; break; }
                    GT_ADD(0, gt_w);
                    if (!(UOCR_GEMM_ABLATE & 2)) {
                        gb_expect_tx(&full[s], Sh::kBTileBytes);
                        tma_load_2d(b_tiles + s * Sh::kBTileBytes, &act_map, (int)(kb * kBlockK), (int)cur_row0, &full[s]);
                    } else {
                        gb_arrive(&full[s]);
                    }
                }
            }
#ifdef UOCR_GEMM_TRACE
            atomicAdd(&g_gemm_trace[GATEUP][5], gt_local[0]);         // loader: waiting for a free activation stage
#endif
        }
    } else {
        // ------------------------------------------------ MMA issue
        // The warp's instruction stream is on the critical path of the tensor core, so a K block is one wait, four MMAs
        // and one commit, and all 32 lanes run the loop: only the MMA and commit instructions themselves are predicated
        // on an elected lane (see tc_mma_ts_elect).
        {
            uint32_t q = 0, it = 0;
            bool ok = true;
            const uint64_t b_desc0 = umma_desc(s2u(b_tiles));
#ifdef UOCR_GEMM_TRACE
            unsigned long long gt_local[6] = {0, 0, 0, 0, 0, 0};
            GT_BEGIN(gt_all);
#endif
            uint32_t nrows_next = p.tiles[blockIdx.x].w;
            for (uint32_t tile_idx = blockIdx.x; tile_idx < n_tiles && ok; tile_idx += gridDim.x, ++it) {
                const uint32_t nrows = nrows_next, buf = it & 1u;
                if (tile_idx + gridDim.x < n_tiles) nrows_next = p.tiles[tile_idx + gridDim.x].w;
                const uint32_t idesc = umma_idesc((nrows + 15u) & ~15u);          // MMA N: multiple of 16
                // the accumulator buffer is free once the epilogue has read the tile before the previous one out of it
                GT_BEGIN(gt_e);
                if (it >= 2) ok = __all_sync(0xffffffffu, gb_wait(&acc_empty[buf], ((it >> 1) - 1u) & 1u, abort_flag, p.status));
                if (!ok) break;
                GT_ADD(2, gt_e);
#ifdef UOCR_GEMM_TRACE
                gt_local[4] += (unsigned long long)kblocks * ((nrows + 15u) & ~15u);      // MMA work: K blocks x token columns
                gt_local[5] += kblocks;
#endif
                tc_fence_after();
                const uint32_t acc_addr = tmem_base + buf * (uint32_t)kTileN;
                for (uint32_t kb = 0; kb < kblocks; ++kb, ++q) {
                    const uint32_t s = q % kStages;
                    GT_BEGIN(gt_a);
                    ok = __all_sync(0xffffffffu, gb_wait(&full[s], (q / kStages) & 1u, abort_flag, p.status));
                    GT_ADD(0, gt_a);
                    if (!ok) break;
                    tc_fence_after();
                    // (the descriptor's address field counts 16-byte units: a stage and a K step are plain additions)
                    const uint64_t bd = b_desc0 + (uint64_t)(s * (uint32_t)(Sh::kBTileBytes >> 4));
                    const uint32_t a_addr = a_base + s * Sh::kAStageCols;
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k)
                        if (!(UOCR_GEMM_ABLATE & 8)) tc_mma_ts_elect(acc_addr, a_addr + k * 8, bd + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit_elect(&empty[s]);               // arrives when the MMAs above have read the stage
                }
                if (ok) tc_commit_elect(&acc_full[buf]);
            }
#ifdef UOCR_GEMM_TRACE
            GT_ADD(3, gt_all);
            if (lane == 0) {
                atomicAdd(&g_gemm_trace[GATEUP][6], gt_local[0]);         // MMA issue: waiting for a full stage
                atomicAdd(&g_gemm_trace[GATEUP][8], gt_local[2]);         // MMA issue: waiting for a free accumulator
                atomicAdd(&g_gemm_trace[GATEUP][9], gt_local[3]);         // MMA issue: whole loop
                atomicAdd(&g_gemm_trace[GATEUP][10], gt_local[4]);        // K blocks x columns issued
                atomicAdd(&g_gemm_trace[GATEUP][11], 1ull);               // CTAs
                atomicAdd(&g_gemm_trace[GATEUP][12], gt_local[5]);        // K blocks
            }
#endif
        }
        __syncwarp();
    }
    __syncthreads();
    if (*abort_flag) {
        // a wait gave up: let copies and MMAs that may still be in flight land before the CTA goes away
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
        __syncthreads();
    }
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Sh::kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------ router logits GEMM
// logits[n][E] = hidden[n][H] . router[E][H]^T for many tokens: 128 tokens per CTA on the M side, all
// experts (padded to a multiple of 16, <= 256) on the N side, both operands by TMA, fp32 accumulate in
// TMEM.  The softmax / top-k kernel then runs on these logits exactly as it does on injected ones.
constexpr int kRouterGemmThreads = 192;     // warps 0-3 epilogue, warp 4 TMA, warp 5 MMA
constexpr int kRouterStages = 4;

__host__ __device__ constexpr int router_gemm_stage_bytes(int n_pad) { return kTileBytes + n_pad * 128; }

__global__ void __launch_bounds__(kRouterGemmThreads, 1)
router_logits_kernel(const __grid_constant__ CUtensorMap hidden_map, const __grid_constant__ CUtensorMap router_map,
                     uint32_t n, uint32_t E, uint32_t n_pad, uint32_t tmem_cols, uint32_t k_dim, float *__restrict__ logits,
                     uint32_t *status) {
    extern __shared__ uint8_t smem_dyn[];
    uint8_t *stages = reinterpret_cast<uint8_t *>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    const uint32_t b_bytes = (n_pad * 128 + 1023) & ~1023u;
    const uint32_t stage_bytes = kTileBytes + b_bytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(stages + kRouterStages * stage_bytes);
    uint64_t *full = bars, *empty = bars + kRouterStages, *acc_full = bars + 2 * kRouterStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kRouterStages + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t row0 = blockIdx.x * kTileM;
    const uint32_t kblocks = k_dim / kBlockK;

    if (tid == 0) {
        for (int s = 0; s < kRouterStages; ++s) { gb_init(&full[s], 1); gb_init(&empty[s], 1); }
        gb_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        if (gb_wait(acc_full, 0, abort_flag, status)) {
            tc_fence_after();
            const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
            const uint32_t row = row0 + tid;
            for (uint32_t c0 = 0; c0 < n_pad; c0 += 16) {
                uint32_t v[16];
                tc_ld16(lane_base + c0, v);
                tc_ld_wait();
                if (row < n) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < E) logits[(size_t)row * E + c0 + j] = __uint_as_float(v[j]);
                }
            }
        }
        tc_fence_before();
    } else if (warp == 4) {
        if (lane == 0) {
            for (uint32_t kb = 0; kb < kblocks; ++kb) {
                const int s = kb % kRouterStages;
                const uint32_t use = kb / kRouterStages;
                if (use > 0 && !gb_wait(&empty[s], (use - 1) & 1u, abort_flag, status)) break;
                gb_expect_tx(&full[s], kTileBytes + n_pad * 128);
                tma_load_2d(stages + s * stage_bytes, &hidden_map, (int)(kb * kBlockK), (int)row0, &full[s]);
                tma_load_2d(stages + s * stage_bytes + kTileBytes, &router_map, (int)(kb * kBlockK), 0, &full[s]);
            }
        }
    } else {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(n_pad);
            bool ok = true;
            for (uint32_t kb = 0; kb < kblocks && ok; ++kb) {
                const int s = kb % kRouterStages;
                ok = gb_wait(&full[s], (kb / kRouterStages) & 1u, abort_flag, status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = s2u(stages + s * stage_bytes), b_addr = a_addr + kTileBytes;
#pragma unroll
                for (int k = 0; k < kBlockK / 16; ++k)
                    tc_mma(tmem_base, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                tc_commit(&empty[s]);
            }
            if (ok) tc_commit(acc_full);
        }
        __syncwarp();
    }
    __syncthreads();
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// --------------------------------------------------------------------- helper kernels
// Tile lists of the routed GEMMs: for every expert with pairs, gate/up tiles of (192 tokens, 64 + 64 weight rows)
// and down tiles of (192 tokens, 128 weight rows).  Entries are {expert, weight-row tile, first sorted
// position, rows}; counts[0/1] are the list lengths.
// Segment e uses the weights of expert expert_base + e % expert_mod (single GPU: base 0, mod E; expert-parallel
// ranks receive one segment per (source rank, local expert)).
__global__ void tile_plan_kernel(const uint32_t *__restrict__ expert_offsets, uint32_t E, uint32_t expert_base,
                                 uint32_t expert_mod, uint32_t gu_mtiles, uint32_t dn_mtiles, uint4 *__restrict__ tiles_gu,
                                 uint4 *__restrict__ tiles_dn, uint32_t *__restrict__ counts) {
    // The lists start with the segment that has the most rows (ties: lower index first): the persistent GEMM kernel
    // deals tiles to its CTAs in list order, so the long segments are under way first and the short ones fill the tail.
    // One CTA; the entries are then written by all its threads, entry i finding its segment by binary search.
    __shared__ uint32_t order[256], first_tile[257];         // segments by rank; token tiles before the segment of rank k
    const uint32_t tid = threadIdx.x;
    if (tid < E) {
        const uint32_t c = expert_offsets[tid + 1] - expert_offsets[tid];
        uint32_t rank = 0;
        for (uint32_t j = 0; j < E; ++j) {
            const uint32_t cj = expert_offsets[j + 1] - expert_offsets[j];
            rank += (cj > c || (cj == c && j < tid)) ? 1u : 0u;
        }
        order[rank] = tid;
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t run = 0;
        for (uint32_t k = 0; k < E; ++k) {
            const uint32_t i = order[k];
            first_tile[k] = run;
            run += (expert_offsets[i + 1] - expert_offsets[i] + kTileN - 1) / kTileN;
        }
        first_tile[E] = run;
        counts[0] = run * gu_mtiles;
        counts[1] = run * dn_mtiles;
    }
    __syncthreads();
    const uint32_t token_tiles = first_tile[E];
    for (uint32_t i = tid; i < token_tiles * (gu_mtiles + dn_mtiles); i += blockDim.x) {
        const bool gu = i < token_tiles * gu_mtiles;
        const uint32_t mtiles = gu ? gu_mtiles : dn_mtiles, j = gu ? i : i - token_tiles * gu_mtiles;
        const uint32_t tt = j / mtiles, m = j % mtiles;       // token tile of the whole list, weight-row tile
        uint32_t lo = 0, hi = E;                              // the rank k with first_tile[k] <= tt < first_tile[k + 1]
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) / 2;
            if (first_tile[mid] <= tt) lo = mid; else hi = mid;
        }
        const uint32_t e = order[lo], t = tt - first_tile[lo];
        const uint32_t seg0 = expert_offsets[e], cnt = expert_offsets[e + 1] - seg0;
        const uint4 entry = make_uint4(expert_base + e % expert_mod, m, seg0 + t * kTileN, min((uint32_t)kTileN, cnt - t * kTileN));
        (gu ? tiles_gu : tiles_dn)[j] = entry;
    }
}

// Tile lists of the shared MLP (one "expert", all n tokens).
__global__ void shared_tile_plan_kernel(uint32_t n, uint32_t gu_mtiles, uint32_t dn_mtiles, uint4 *__restrict__ tiles_gu,
                                        uint4 *__restrict__ tiles_dn, uint32_t *__restrict__ counts) {
    const uint32_t tg = (n + kTileN - 1) / kTileN, td = tg;
    const uint32_t stride = gridDim.x * blockDim.x, i0 = blockIdx.x * blockDim.x + threadIdx.x;
    for (uint32_t i = i0; i < tg * gu_mtiles; i += stride) {
        const uint32_t t = i / gu_mtiles, m = i % gu_mtiles, r0 = t * kTileN;
        tiles_gu[i] = make_uint4(0, m, r0, min((uint32_t)kTileN, n - r0));
    }
    for (uint32_t i = i0; i < td * dn_mtiles; i += stride) {
        const uint32_t t = i / dn_mtiles, m = i % dn_mtiles, r0 = t * kTileN;
        tiles_dn[i] = make_uint4(0, m, r0, min((uint32_t)kTileN, n - r0));
    }
    if (i0 == 0) { counts[0] = tg * gu_mtiles; counts[1] = td * dn_mtiles; }
}

// x_sorted[pos][:] = hidden[pair_rows[pos] / K][:]  (one warp per row, 16-byte copies)
__global__ void gather_rows_kernel(const __half *__restrict__ hidden, const uint32_t *__restrict__ pair_rows,
                                   const uint32_t *__restrict__ expert_offsets, uint32_t E, uint32_t K, uint32_t H,
                                   __half *__restrict__ x_sorted) {
    const uint32_t total = expert_offsets[E];
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= total) return;
    const uint4 *src = reinterpret_cast<const uint4 *>(hidden + (size_t)(pair_rows[warp] / K) * H);
    uint4 *dst = reinterpret_cast<uint4 *>(x_sorted + (size_t)warp * H);
    for (uint32_t i = lane; i < H / 8; i += 32) dst[i] = __ldg(src + i);
}

// out[t][h] = fp16( fma chain over slots of weight * down_out[inverse[pair]][h], + shared_out[t][h], + residual )
__global__ void combine_sorted_kernel(const __half *__restrict__ down_out, const __half *__restrict__ shared_out,
                                      const __half *__restrict__ residual, const uint32_t *__restrict__ inverse,
                                      const float *__restrict__ weights, uint32_t n, uint32_t H, uint32_t K,
                                      __half *__restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;       // one thread per 8 outputs
    const uint32_t per_row = H / 8;
    if (idx >= (size_t)n * per_row) return;
    const uint32_t t = (uint32_t)(idx / per_row), c = (uint32_t)(idx % per_row) * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (uint32_t s = 0; s < K; ++s) {
        const uint32_t pos = inverse[t * K + s];
        if (pos == 0xffffffffu) continue;
        const float w = weights[t * K + s];
        const uint4 v = *reinterpret_cast<const uint4 *>(down_out + (size_t)pos * H + c);
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            acc[2 * i] = fmaf(w, f.x, acc[2 * i]);
            acc[2 * i + 1] = fmaf(w, f.y, acc[2 * i + 1]);
        }
    }
    {
        const uint4 v = *reinterpret_cast<const uint4 *>(shared_out + (size_t)t * H + c);
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
        }
    }
    if (residual) {
        const uint4 v = *reinterpret_cast<const uint4 *>(residual + (size_t)t * H + c);
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
        }
    }
    uint4 o;
    __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) oh[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4 *>(out + (size_t)t * H + c) = o;
}

// ---------------------------------------------------------------- peer-memory exchange (expert parallelism)
// One node, one process per GPU: every rank has mapped the other ranks' "received rows" and "expert outputs"
// buffers (CUDA IPC).  The two kernels below are the gather and the combine with the exchange fused in: rows are
// written straight into the owner's buffer, and read back straight from it, over NVLink, with plain stores and
// loads (no TMA multicast, no library kernel on peer memory).
//
// Expert e is owned by rank e / experts_per_rank.  dst_row0[e]: row of the owner's buffer where this rank's rows
// for expert e start (the host derives it from the gathered per-rank counts).
constexpr uint32_t kStatusPeerRange = 32u;

// peer.p[owner][row][:] = hidden[token of the pos-th pair in expert order][:]
__global__ void scatter_rows_peer_kernel(const __half *__restrict__ hidden, const uint32_t *__restrict__ pair_rows,
                                         const uint32_t *__restrict__ expert_offsets, uint32_t E, uint32_t K, uint32_t H,
                                         uint32_t experts_per_rank, const uint32_t *__restrict__ dst_row0, PeerBuffers peer,
                                         unsigned long long row_capacity, uint32_t *status) {
    const uint32_t total = expert_offsets[E];
    const uint32_t pos = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (pos >= total) return;
    uint32_t lo = 0, hi = E;                    // the expert whose range [offsets[e], offsets[e + 1]) holds pos
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (expert_offsets[mid] <= pos) lo = mid; else hi = mid;
    }
    const uint32_t e = lo;
    const unsigned long long row = (unsigned long long)dst_row0[e] + (pos - expert_offsets[e]);
    if (row >= row_capacity) {                  // never write outside a peer's buffer
        if (lane == 0) atomicOr(status, kStatusPeerRange);
        return;
    }
    const uint4 *src = reinterpret_cast<const uint4 *>(hidden + (size_t)(pair_rows[pos] / K) * H);
    uint4 *dst = reinterpret_cast<uint4 *>(peer.p[e / experts_per_rank] + (size_t)row * H);
    // all of the row's loads are issued before the first (remote) store
    uint4 v[8];                                 // H <= 2048: at most eight 16-byte pieces per lane
#pragma unroll
    for (uint32_t k = 0; k < 8; ++k)
        if (lane + 32 * k < H / 8) v[k] = __ldg(src + lane + 32 * k);
#pragma unroll
    for (uint32_t k = 0; k < 8; ++k)
        if (lane + 32 * k < H / 8) dst[lane + 32 * k] = v[k];
}

__device__ __forceinline__ uint4 ld_volatile_v4(const uint4 *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// out[t][h] = fp16( fma chain over slots of weight * (owner's output row of the pair)[h] + shared_out[t][h] + residual )
__global__ void combine_peer_kernel(PeerBuffers peer, const __half *__restrict__ shared_out, const __half *__restrict__ residual,
                                    const uint32_t *__restrict__ inverse, const uint32_t *__restrict__ top_ids,
                                    const float *__restrict__ weights, const uint32_t *__restrict__ expert_offsets,
                                    const uint32_t *__restrict__ dst_row0, uint32_t experts_per_rank, uint32_t E, uint32_t n,
                                    uint32_t H, uint32_t K, unsigned long long row_capacity, uint32_t *status,
                                    __half *__restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;       // one thread per 8 outputs
    const uint32_t per_row = H / 8;
    if (idx >= (size_t)n * per_row) return;
    const uint32_t t = (uint32_t)(idx / per_row), c = (uint32_t)(idx % per_row) * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    // A remote row takes microseconds to arrive: the loads of up to eight slots are all issued before the first one is
    // used; the sums still run in slot order, as the single-GPU combine's do.
    constexpr uint32_t kSlotsInFlight = 8;
    for (uint32_t s0 = 0; s0 < K; s0 += kSlotsInFlight) {
        uint4 v[kSlotsInFlight];
        float w[kSlotsInFlight];
        bool have[kSlotsInFlight];
#pragma unroll
        for (uint32_t j = 0; j < kSlotsInFlight; ++j) {
            const uint32_t s = s0 + j;
            have[j] = false;
            if (s < K) {
                const uint32_t pos = inverse[t * K + s], e = top_ids[t * K + s];
                if (pos != 0xffffffffu && e < E) {
                    const unsigned long long row = (unsigned long long)dst_row0[e] + (pos - expert_offsets[e]);
                    if (row >= row_capacity) {
                        atomicOr(status, kStatusPeerRange);
                    } else {
                        have[j] = true;
                        w[j] = weights[t * K + s];
                        v[j] = ld_volatile_v4(reinterpret_cast<const uint4 *>(peer.p[e / experts_per_rank] + (size_t)row * H + c));
                    }
                }
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < kSlotsInFlight; ++j) {
            if (!have[j]) continue;
            const __half2 *h = reinterpret_cast<const __half2 *>(&v[j]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                acc[2 * i] = fmaf(w[j], f.x, acc[2 * i]);
                acc[2 * i + 1] = fmaf(w[j], f.y, acc[2 * i + 1]);
            }
        }
    }
    {
        const uint4 v = *reinterpret_cast<const uint4 *>(shared_out + (size_t)t * H + c);
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
        }
    }
    if (residual) {
        const uint4 v = *reinterpret_cast<const uint4 *>(residual + (size_t)t * H + c);
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
        }
    }
    uint4 o;
    __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) oh[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4 *>(out + (size_t)t * H + c) = o;
}

// ---------------------------------------------------------------------------- host side
static std::atomic<PFN_cuTensorMapEncodeTiled_v12000> g_encode{nullptr};    // process-wide, the same value from every thread

cudaError_t init_gemm_kernels() {
    if (g_encode.load() == nullptr) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (err != cudaSuccess) return err;
        if (qres != cudaDriverEntryPointSuccess || fn == nullptr) return cudaErrorNotSupported;
        g_encode.store(reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn));
    }
    cudaError_t err = cudaFuncSetAttribute(router_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)(kRouterStages * (kTileBytes + 32 * 1024) + 1024 + 256));
#define UOCR_SET_SMEM(QT, GU)                                                                                    \
    if (err == cudaSuccess)                                                                                      \
        err = cudaFuncSetAttribute(grouped_gemm_kernel<QT, GU>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                   GemmShape::kSmemBytes);
    UOCR_SET_SMEM(UOCR_QT_Q4, true) UOCR_SET_SMEM(UOCR_QT_Q4, false)
    UOCR_SET_SMEM(UOCR_QT_Q8, true) UOCR_SET_SMEM(UOCR_QT_Q8, false)
    UOCR_SET_SMEM(UOCR_QT_F16, true) UOCR_SET_SMEM(UOCR_QT_F16, false)
#undef UOCR_SET_SMEM
    return err;
}

// fp16 matrix [rows][cols] (cols contiguous) viewed as tiles of box_rows rows x 64 columns, 128B swizzle, zero fill
static cudaError_t make_map_rows(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {kBlockK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_encode.load()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

static size_t router_gemm_smem(uint32_t n_pad) {
    const size_t b_bytes = ((size_t)n_pad * 128 + 1023) & ~(size_t)1023;
    return kRouterStages * (kTileBytes + b_bytes) + 1024 + 256;
}

bool router_gemm_supported(const DLayer &L) { return g_encode.load() != nullptr && L.H % 64 == 0 && L.E <= 256; }

// logits[n][E] (no bias) for n tokens
cudaError_t launch_router_logits(const DLayer &L, const __half *hidden, uint32_t n, float *logits, uint32_t *status,
                                 cudaStream_t st, uint64_t *launches) {
    const uint32_t n_pad = (L.E + 15u) & ~15u;
    uint32_t cols = 32;
    while (cols < n_pad) cols <<= 1;
    CUtensorMap hm, rm;
    cudaError_t err;
    if ((err = make_map_rows(&hm, hidden, n, L.H, kTileM)) != cudaSuccess) return err;
    if ((err = make_map_rows(&rm, L.router, L.E, L.H, n_pad)) != cudaSuccess) return err;
    router_logits_kernel<<<(n + kTileM - 1) / kTileM, kRouterGemmThreads, router_gemm_smem(n_pad), st>>>(
        hm, rm, n, L.E, n_pad, cols, L.H, logits, status);
    ++*launches;
    return cudaGetLastError();
}

bool gemm_tensor_maps_ready() { return g_encode.load() != nullptr; }

bool gemm_path_supported(const DLayer &L) {
    return L.H % 128 == 0 && L.F % 128 == 0 && L.S % 128 == 0 && L.E <= 256 && L.H <= 2048 && L.F <= 2048 &&
           L.S <= 2048 && g_encode.load() != nullptr;
}

static std::atomic<int> g_gemm_sms[64];

// one CTA per SM at most (the kernel is persistent: CTA b takes tiles b, b + grid, ...)
static uint32_t gemm_grid(uint32_t max_tiles) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return max_tiles;
    sms = g_gemm_sms[dev].load();
    if (sms == 0) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return max_tiles;
        g_gemm_sms[dev] = sms;
    }
    return max_tiles < (uint32_t)sms ? max_tiles : (uint32_t)sms;
}

template <bool GU>
static cudaError_t launch_gemm(int qt, const CUtensorMap &map, const GemmParams &p, uint32_t max_tiles, cudaStream_t st) {
    if (max_tiles == 0) return cudaSuccess;
    max_tiles = gemm_grid(max_tiles);
    const size_t smem = GemmShape::kSmemBytes;
    switch (qt) {
        case UOCR_QT_Q4: grouped_gemm_kernel<UOCR_QT_Q4, GU><<<max_tiles, kGemmThreads, smem, st>>>(map, p); break;
        case UOCR_QT_Q8: grouped_gemm_kernel<UOCR_QT_Q8, GU><<<max_tiles, kGemmThreads, smem, st>>>(map, p); break;
        default: grouped_gemm_kernel<UOCR_QT_F16, GU><<<max_tiles, kGemmThreads, smem, st>>>(map, p); break;
    }
    return cudaGetLastError();
}

static uint32_t packed_row_bytes_of(int qt, uint32_t cols) {
    return qt == UOCR_QT_F16 ? cols * 2u : (qt == UOCR_QT_Q8 ? cols : cols / 2u);
}

// Scratch of the many-token path (all in the context arena).
struct GemmScratch {
    __half *x_sorted;       // [n*K][H] activations in expert-sorted order
    __half *mid_sorted;     // [n*K][F]
    __half *down_sorted;    // [n*K][H]
    __half *shared_mid;     // [n][S]
    __half *shared_out;     // [n][H]
    uint4 *tiles_gu, *tiles_dn, *stiles_gu, *stiles_dn;
    uint32_t *counts;       // [4]: routed gate/up, routed down, shared gate/up, shared down
};

static GemmParams base_params(const Scratch &S) {
    GemmParams p{};
    p.status = S.status;
    return p;
}

// Routed experts over rows that are already grouped: segment i (rows seg_offsets[i] .. seg_offsets[i+1]) belongs to
// expert expert_base + i % expert_mod.  rows_in [rows][H] -> mid [rows][F] -> rows_out [rows][H], all fp16.
cudaError_t launch_gemm_experts(const DLayer &L, const Scratch &S, const GemmScratch &G, const uint32_t *seg_offsets,
                                uint32_t n_seg, uint32_t expert_base, uint32_t expert_mod, const __half *rows_in,
                                uint32_t rows_bound, __half *mid, __half *rows_out, cudaStream_t st, uint64_t *launches) {
    const uint32_t H = L.H, F = L.F;
    if (rows_bound == 0) return cudaSuccess;
    const uint32_t ttiles = (rows_bound + kTileN - 1) / kTileN + n_seg;     // token tiles: an upper bound known on the host
    cudaError_t err;
    tile_plan_kernel<<<1, 1024, 0, st>>>(seg_offsets, n_seg, expert_base, expert_mod, F / (kTileM / 2), H / kTileM, G.tiles_gu,
                                        G.tiles_dn, G.counts);
    ++*launches;
    if ((err = cudaGetLastError()) != cudaSuccess) return err;
    CUtensorMap map_x, map_mid;
    if ((err = make_map_rows(&map_x, rows_in, rows_bound, H, kTileN)) != cudaSuccess) return err;
    if ((err = make_map_rows(&map_mid, mid, rows_bound, F, kTileN)) != cudaSuccess) return err;
    const int qt = L.expert_qtype;
    GemmParams p = base_params(S);
    p.w0 = L.expert_w; p.w1 = L.expert_w + L.up_offset_bytes;
    p.s0 = L.expert_s; p.s1 = L.expert_s ? L.expert_s + L.up_scale_offset : nullptr;
    p.expert_stride_bytes = L.expert_stride_bytes; p.expert_scale_stride = L.expert_scale_stride;
    p.row_bytes = packed_row_bytes_of(qt, H); p.k_dim = H;
    p.tiles = G.tiles_gu; p.tile_count = G.counts; p.out = mid; p.out_ld = F;
    if ((err = launch_gemm<true>(qt, map_x, p, ttiles * (F / (kTileM / 2)), st)) != cudaSuccess) return err;
    p.w0 = L.expert_w + L.down_offset_bytes; p.w1 = nullptr;
    p.s0 = L.expert_s ? L.expert_s + L.down_scale_offset : nullptr; p.s1 = nullptr;
    p.row_bytes = packed_row_bytes_of(qt, F); p.k_dim = F;
    p.tiles = G.tiles_dn; p.tile_count = G.counts + 1; p.out = rows_out; p.out_ld = H;
    if ((err = launch_gemm<false>(qt, map_mid, p, ttiles * (H / kTileM), st)) != cudaSuccess) return err;
    *launches += 2;
    return cudaSuccess;
}

// Shared MLP on all n tokens: G.shared_out[n][H] = fp16( down( silu(gate x) * up x ) ).
cudaError_t launch_gemm_shared(const DLayer &L, const Scratch &S, const GemmScratch &G, const __half *hidden, uint32_t n,
                               cudaStream_t st, uint64_t *launches) {
    const uint32_t H = L.H, Sd = L.S;
    const uint32_t sttiles = (n + kTileN - 1) / kTileN;
    cudaError_t err;
    shared_tile_plan_kernel<<<8, 256, 0, st>>>(n, Sd / (kTileM / 2), H / kTileM, G.stiles_gu, G.stiles_dn, G.counts + 2);
    ++*launches;
    CUtensorMap map_hidden, map_smid;
    if ((err = make_map_rows(&map_hidden, hidden, n, H, kTileN)) != cudaSuccess) return err;
    if ((err = make_map_rows(&map_smid, G.shared_mid, n, Sd, kTileN)) != cudaSuccess) return err;
    GemmParams p = base_params(S);
    p.w0 = L.shared_gate.w; p.w1 = L.shared_up.w; p.s0 = L.shared_gate.s; p.s1 = L.shared_up.s;
    p.row_bytes = L.shared_gate.row_bytes; p.k_dim = H;
    p.tiles = G.stiles_gu; p.tile_count = G.counts + 2; p.out = G.shared_mid; p.out_ld = Sd;
    if ((err = launch_gemm<true>(L.shared_gate.qtype, map_hidden, p, sttiles * (Sd / (kTileM / 2)), st)) != cudaSuccess) return err;
    p.w0 = L.shared_down.w; p.w1 = nullptr; p.s0 = L.shared_down.s; p.s1 = nullptr;
    p.row_bytes = L.shared_down.row_bytes; p.k_dim = Sd;
    p.tiles = G.stiles_dn; p.tile_count = G.counts + 3; p.out = G.shared_out; p.out_ld = H;
    if ((err = launch_gemm<false>(L.shared_down.qtype, map_smid, p, sttiles * (H / kTileM), st)) != cudaSuccess) return err;
    *launches += 2;
    return cudaSuccess;
}

// out = fp16( sum_slot w * down_rows[inverse[pair]] + shared_out + residual )
cudaError_t launch_gemm_combine(const DLayer &L, const Scratch &S, const GemmScratch &G, const __half *down_rows,
                                const __half *residual, uint32_t n, __half *out, cudaStream_t st, uint64_t *launches) {
    const size_t work = (size_t)n * (L.H / 8);
    combine_sorted_kernel<<<(unsigned)((work + 255) / 256), 256, 0, st>>>(down_rows, G.shared_out, residual, S.inverse,
                                                                          S.top_weights, n, L.H, L.K, out);
    ++*launches;
    return cudaGetLastError();
}

// rows_out[pos][:] = hidden[token of the pos-th pair in expert order][:]
cudaError_t launch_gather_sorted(const DLayer &L, const Scratch &S, const __half *hidden, uint32_t n, __half *rows_out,
                                 cudaStream_t st, uint64_t *launches) {
    const uint32_t pairs = n * L.K;
    gather_rows_kernel<<<(pairs * 32 + 255) / 256, 256, 0, st>>>(hidden, S.pair_rows, S.expert_offsets, L.E, L.K, L.H, rows_out);
    ++*launches;
    return cudaGetLastError();
}

// rows of this rank's pairs -> the owners' "received rows" buffers
cudaError_t launch_scatter_peer(const DLayer &L, const Scratch &S, const __half *hidden, uint32_t n, uint32_t experts_per_rank,
                                const uint32_t *dst_row0, const PeerBuffers &recv, unsigned long long row_capacity,
                                cudaStream_t st, uint64_t *launches) {
    const uint32_t pairs = n * L.K;
    scatter_rows_peer_kernel<<<(pairs * 32 + 255) / 256, 256, 0, st>>>(hidden, S.pair_rows, S.expert_offsets, L.E, L.K, L.H,
                                                                       experts_per_rank, dst_row0, recv, row_capacity, S.status);
    ++*launches;
    return cudaGetLastError();
}

// combine that reads the pairs' expert outputs from the owners' buffers
cudaError_t launch_combine_peer(const DLayer &L, const Scratch &S, const GemmScratch &G, const PeerBuffers &done,
                                uint32_t experts_per_rank, const uint32_t *dst_row0, unsigned long long row_capacity,
                                const __half *residual, uint32_t n, __half *out, cudaStream_t st, uint64_t *launches) {
    const size_t work = (size_t)n * (L.H / 8);
    combine_peer_kernel<<<(unsigned)((work + 255) / 256), 256, 0, st>>>(done, G.shared_out, residual, S.inverse, S.top_ids,
                                                                        S.top_weights, S.expert_offsets, dst_row0,
                                                                        experts_per_rank, L.E, n, L.H, L.K, row_capacity, S.status, out);
    ++*launches;
    return cudaGetLastError();
}

// Row bookkeeping of the peer-memory exchange, on the device (no host round trip between the count exchange and the
// scatter).  all_offsets [world][E + 1]: every rank's expert_offsets.  For this rank as a SENDER: dst_row0[e] = row of the
// owner's "received rows" buffer where its rows for expert e start (the owner's buffer holds, for source 0, 1, ... in
// turn, the rows of each of its experts in turn).  For this rank as an OWNER: seg_offsets[source * per + local expert]
// = first row of that segment, seg_offsets[world * per] = rows received.  More rows than the buffers hold raise the
// status bit; the kernels that use the offsets check every row index again.
__global__ void ep_offsets_kernel(const uint32_t *__restrict__ all_offsets, uint32_t world, uint32_t rank, uint32_t E,
                                  unsigned long long row_capacity, uint32_t *__restrict__ dst_row0,
                                  uint32_t *__restrict__ seg_offsets, uint32_t *__restrict__ status) {
    const uint32_t per = E / world, tid = threadIdx.x, stride = E + 1;
    auto cnt = [&](uint32_t g, uint32_t e) { return all_offsets[g * stride + e + 1] - all_offsets[g * stride + e]; };
    for (uint32_t e = tid; e < E; e += blockDim.x) {
        const uint32_t owner = e / per, first = owner * per;
        unsigned long long row = 0;
        for (uint32_t g = 0; g < rank; ++g) row += all_offsets[g * stride + first + per] - all_offsets[g * stride + first];
        row += all_offsets[rank * stride + e] - all_offsets[rank * stride + first];
        dst_row0[e] = row > 0xffffffffull ? 0xffffffffu : (uint32_t)row;
    }
    if (tid == 0) {
        unsigned long long run = 0;
        for (uint32_t src = 0; src < world; ++src)
            for (uint32_t le = 0; le < per; ++le) {
                seg_offsets[src * per + le] = (uint32_t)run;
                run += cnt(src, rank * per + le);
            }
        if (run > row_capacity) { atomicOr(status, kStatusPeerRange); run = row_capacity; }
        seg_offsets[world * per] = (uint32_t)run;
    }
}

cudaError_t launch_ep_offsets(const uint32_t *all_offsets, uint32_t world, uint32_t rank, uint32_t E,
                              unsigned long long row_capacity, uint32_t *dst_row0, uint32_t *seg_offsets, uint32_t *status,
                              cudaStream_t st, uint64_t *launches) {
    ep_offsets_kernel<<<1, 256, 0, st>>>(all_offsets, world, rank, E, row_capacity, dst_row0, seg_offsets, status);
    ++*launches;
    return cudaGetLastError();
}

// ---- synchronisation of the expert-parallel ranks on the device ----------------------------------------------------
// Every rank owns a small "sync" region that the other ranks write over NVLink: for each source rank its expert offsets
// of the current call ([kMaxPeers][kSyncStride] words), then three rows of flags ([3][kMaxPeers] words: counts written,
// rows landed, outputs written) that hold the number of the call that last set them.  A rank signals by a release store
// of the call number into every peer's flag and waits (bounded, in its own memory) until all its own flags have reached
// that number, so no host library call stands between the phases.  Every rank runs these kernels on its own GPU.
constexpr uint32_t kStatusPeerSync = 64u;
constexpr long long kPeerSpinLimit = 4000000000LL;      // cycles (~2 s)

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// thread g < world: tell rank g that this rank has reached `call` in phase `which`, then wait for rank g to have told us
__device__ __forceinline__ void peer_signal_and_wait(const PeerSync &sync, uint32_t world, uint32_t rank, uint32_t which,
                                                     uint32_t call, uint32_t *status) {
    const uint32_t g = threadIdx.x;
    if (g >= world) return;
    __threadfence_system();
    st_release_sys(sync.p[g] + kSyncFlagWords + which * kMaxPeers + rank, call);
    const uint32_t *mine = sync.p[rank] + kSyncFlagWords + which * kMaxPeers + g;
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys(mine) - call) < 0) {
        __nanosleep(100);
        if (clock64() - t0 > kPeerSpinLimit) { atomicOr(status, kStatusPeerSync); break; }
    }
}

// Publishes this rank's expert offsets to every rank, waits for everybody's, and derives the rows of the exchange (the
// arithmetic of ep_offsets_kernel on the gathered offsets).
__global__ void ep_exchange_counts_kernel(const uint32_t *__restrict__ my_offsets, PeerSync sync, uint32_t world, uint32_t rank,
                                          uint32_t E, uint32_t call, unsigned long long row_capacity,
                                          uint32_t *__restrict__ dst_row0, uint32_t *__restrict__ seg_offsets,
                                          uint32_t *__restrict__ status) {
    const uint32_t tid = threadIdx.x, per = E / world;
    for (uint32_t g = 0; g < world; ++g) {
        volatile uint32_t *dst = sync.p[g] + rank * kSyncStride;
        for (uint32_t i = tid; i <= E; i += blockDim.x) dst[i] = my_offsets[i];
    }
    __syncthreads();                      // (the signalling threads fence at system scope before their release stores)
    peer_signal_and_wait(sync, world, rank, 0, call, status);
    __syncthreads();
    const volatile uint32_t *all = sync.p[rank];
    for (uint32_t e = tid; e < E; e += blockDim.x) {
        const uint32_t owner = e / per, first = owner * per;
        unsigned long long row = 0;
        for (uint32_t g = 0; g < rank; ++g) row += all[g * kSyncStride + first + per] - all[g * kSyncStride + first];
        row += all[rank * kSyncStride + e] - all[rank * kSyncStride + first];
        dst_row0[e] = row > 0xffffffffull ? 0xffffffffu : (uint32_t)row;
    }
    if (tid == 0) {
        unsigned long long run = 0;
        for (uint32_t src = 0; src < world; ++src)
            for (uint32_t le = 0; le < per; ++le) {
                seg_offsets[src * per + le] = (uint32_t)run;
                run += all[src * kSyncStride + rank * per + le + 1] - all[src * kSyncStride + rank * per + le];
            }
        if (run > row_capacity) { atomicOr(status, kStatusPeerRange); run = row_capacity; }
        seg_offsets[world * per] = (uint32_t)run;
    }
}

__global__ void ep_signal_wait_kernel(PeerSync sync, uint32_t world, uint32_t rank, uint32_t which, uint32_t call,
                                      uint32_t *__restrict__ status) {
    peer_signal_and_wait(sync, world, rank, which, call, status);
}

cudaError_t launch_ep_exchange_counts(const uint32_t *my_offsets, const PeerSync &sync, uint32_t world, uint32_t rank, uint32_t E,
                                      uint32_t call, unsigned long long row_capacity, uint32_t *dst_row0, uint32_t *seg_offsets,
                                      uint32_t *status, cudaStream_t st, uint64_t *launches) {
    ep_exchange_counts_kernel<<<1, 256, 0, st>>>(my_offsets, sync, world, rank, E, call, row_capacity, dst_row0, seg_offsets, status);
    ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_ep_signal_wait(const PeerSync &sync, uint32_t world, uint32_t rank, uint32_t which, uint32_t call,
                                  uint32_t *status, cudaStream_t st, uint64_t *launches) {
    ep_signal_wait_kernel<<<1, 32, 0, st>>>(sync, world, rank, which, call, status);
    ++*launches;
    return cudaGetLastError();
}

// ---- dequantisation probe ------------------------------------------------------------------------------------
// out[row][col] = the fp16 value (widened to f32) the grouped GEMM's producer threads store into tensor memory for
// weight (row, col): the same load_block / convert_sub pair, one thread per (row, 64-wide K block).
template <int QT>
__global__ void producer_probe_kernel(const uint8_t *__restrict__ w, const __half *__restrict__ s, uint32_t rows, uint32_t cols,
                                      uint32_t row_bytes, float *__restrict__ out) {
    const uint32_t kblocks = cols / kBlockK;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * kblocks) return;
    const uint32_t kb = (uint32_t)(idx % kblocks), row = (uint32_t)(idx / kblocks);
    uint4 v[PackedBlock<QT>::kVecs];
    load_block<QT>(w + (size_t)row * row_bytes, kb, v);
    const __half sc = QT == UOCR_QT_F16 ? __ushort_as_half(0) : s[(size_t)row * kblocks + kb];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
        uint32_t regs[8];
        convert_sub<QT>(v, q4 >> 1, q4 & 1, sc, regs);
        float *dst = out + (size_t)row * cols + (size_t)kb * kBlockK + 16 * q4;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&regs[i]));
            dst[2 * i] = f.x;
            dst[2 * i + 1] = f.y;
        }
    }
}

cudaError_t launch_producer_probe(const DMatrix &m, float *out, cudaStream_t st, uint64_t *launches) {
    const size_t work = (size_t)m.rows * (m.cols / kBlockK);
    const unsigned blocks = (unsigned)((work + 255) / 256);
    switch (m.qtype) {
        case UOCR_QT_Q4: producer_probe_kernel<UOCR_QT_Q4><<<blocks, 256, 0, st>>>(m.w, m.s, m.rows, m.cols, m.row_bytes, out); break;
        case UOCR_QT_Q8: producer_probe_kernel<UOCR_QT_Q8><<<blocks, 256, 0, st>>>(m.w, m.s, m.rows, m.cols, m.row_bytes, out); break;
        default: producer_probe_kernel<UOCR_QT_F16><<<blocks, 256, 0, st>>>(m.w, m.s, m.rows, m.cols, m.row_bytes, out); break;
    }
    ++*launches;
    return cudaGetLastError();
}

#ifdef UOCR_GEMM_TRACE
cudaError_t read_gemm_trace(unsigned long long *out32, bool reset) {
    cudaError_t err = cudaMemcpyFromSymbol(out32, g_gemm_trace, sizeof(unsigned long long) * 32);
    if (err == cudaSuccess && reset) {
        static const unsigned long long zero[32] = {0};
        err = cudaMemcpyToSymbol(g_gemm_trace, zero, sizeof zero);
    }
    return err;
}
#endif

}  // namespace uocr

#ifdef UOCR_GEMM_TRACE
extern "C" __attribute__((visibility("default"))) int uocr_cuda_debug_gemm_trace(unsigned long long *out32, int reset) {
    return uocr::read_gemm_trace(out32, reset != 0) == cudaSuccess ? 1 : 0;
}
#endif

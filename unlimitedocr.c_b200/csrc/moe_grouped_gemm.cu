// Many-token MoE layer: expert-grouped GEMMs on the 5th-generation tensor cores.
//
// After the dispatch plan the (token, slot) pairs of one expert are contiguous, so each expert is a
// dense product.  Both products are computed "weights as rows":
//     gate/up :  [2 x 128 weight rows] x [<=128 tokens]  over K = H,  two accumulators (gate, up) ->
//                mid[pos][f] = fp16( silu(gate) * up )
//     down    :  [128 weight rows] x [<=256 tokens]  over K = F (or S) -> down_out[pos][h] = fp16(acc)
// With the weights on the M side of the MMA a cold expert with a handful of tokens pads its token
// count to 16, not to 128, which matters under Zipf-skewed routing.
//
// One CTA (576 threads, one per SM: it owns all 512 tensor-memory columns) computes one tile.  Per 64-wide K
// block (= one scale group of the weight formats, = one 128-byte swizzle row of fp16):
//   warps 0-15 two threads per weight row and matrix: each loads its share of the row's packed bytes with 128-bit
//              loads (several K blocks ahead), turns them into fp16( level * scale ) in registers and stores
//              them with tcgen05.st straight into a ring of tensor-memory slots, the A operand of the MMA:
//              no dequantised weight ever reaches shared or global memory.  A slot is published one block late,
//              so the stores' latency hides behind the next conversion.  The same warps run the epilogue
//              (tcgen05.ld, SwiGLU with the fast exponential, fp16 stores).
//   warp 16    one thread issues the TMA tile loads (cp.async.bulk.tensor) of the activation tile.
//   warp 17    one thread issues tcgen05.mma (kind::f16, A from tensor memory, B from shared memory, fp32
//              accumulators in tensor memory) and commits the slots back; the warp also owns the TMEM allocation.
// Every wait is bounded; on a time-out the CTA raises a status bit, drains and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>

#include "moe_common.cuh"

namespace uocr {

constexpr int kGemmThreads = 576;        // warps 0-15 producers + epilogue, warp 16 TMA, warp 17 MMA
constexpr int kProducerThreads = 512;
constexpr int kTmaWarp = 16, kMmaWarp = 17;
constexpr int kTileM = 128;          // weight rows per tile = TMEM lanes
constexpr int kTileN = 256;          // tokens per tile of the down product (one accumulator)
constexpr int kTileNGateUp = 128;    // tokens per tile of the gate/up product (two accumulators)
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
// Bounded wait; also gives up as soon as another role of the CTA has raised the abort flag.
__device__ __forceinline__ bool gb_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, uint32_t *status) {
    if (gb_try(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t polls = 0;
    while (!gb_try(bar, parity)) {
        if ((++polls & 255u) == 0u) {
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

// Packed bytes one thread holds per 64-wide K block: it owns K positions [16h, 16h+16) of both 32-wide
// sub-blocks (h = 0 / 1).  kAhead: how many K blocks of packed bytes a thread keeps in flight from global memory.
template <int QT> struct PackedBlock;
template <> struct PackedBlock<UOCR_QT_Q4> { static constexpr int kVecs = 1; static constexpr int kAhead = 4; };
template <> struct PackedBlock<UOCR_QT_Q8> { static constexpr int kVecs = 2; static constexpr int kAhead = 3; };
template <> struct PackedBlock<UOCR_QT_F16> { static constexpr int kVecs = 4; static constexpr int kAhead = 2; };

// Q4_0: bytes 16h..16h+15 of the group's 32 (low nibbles: sub-block 0, high nibbles: sub-block 1).
// Q8_0: bytes 32j + 16h .. +15 for sub-block j.   fp16: halves 32j + 16h .. +15 for sub-block j.
template <int QT>
__device__ __forceinline__ void load_block(const uint8_t *row, uint32_t kb, int h, uint4 (&v)[PackedBlock<QT>::kVecs]) {
    const uint4 *p = reinterpret_cast<const uint4 *>(row);
    if constexpr (QT == UOCR_QT_Q4) {
        v[0] = __ldg(p + (size_t)kb * 2 + h);
    } else if constexpr (QT == UOCR_QT_Q8) {
        v[0] = __ldg(p + (size_t)kb * 4 + h);
        v[1] = __ldg(p + (size_t)kb * 4 + 2 + h);
    } else {
        v[0] = __ldg(p + (size_t)kb * 8 + 2 * h);
        v[1] = __ldg(p + (size_t)kb * 8 + 2 * h + 1);
        v[2] = __ldg(p + (size_t)kb * 8 + 4 + 2 * h);
        v[3] = __ldg(p + (size_t)kb * 8 + 4 + 2 * h + 1);
    }
}

// 16 weights of sub-block j -> 8 registers of two fp16 each, in K order
template <int QT>
__device__ __forceinline__ void convert_sub(const uint4 (&v)[PackedBlock<QT>::kVecs], int j, __half scale, uint32_t (&out)[8]) {
    if constexpr (QT == UOCR_QT_F16) {
        const uint4 a = j ? v[2] : v[0], b = j ? v[3] : v[1];
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    } else if constexpr (QT == UOCR_QT_Q8) {
        const __half2 s2 = __half2half2(scale), bias = __float2half2_rn(1152.f);   // 1024 + 128
        const uint4 q = j ? v[1] : v[0];
        bytes_to_h2(q.x ^ 0x80808080u, bias, s2, out[0], out[1]);
        bytes_to_h2(q.y ^ 0x80808080u, bias, s2, out[2], out[3]);
        bytes_to_h2(q.z ^ 0x80808080u, bias, s2, out[4], out[5]);
        bytes_to_h2(q.w ^ 0x80808080u, bias, s2, out[6], out[7]);
    } else {
        const __half2 s2 = __half2half2(scale), bias = __float2half2_rn(1032.f);    // 1024 + 8
        const uint4 q = v[0];
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

// silu with the fast exponential and reciprocal (about 2 ulp; the result is rounded to fp16 anyway)
__device__ __forceinline__ float silu_fast(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// ------------------------------------------------------------------------------ kernel
// Tensor-memory columns: the accumulators first, then kAStages slots of the weight operand (one 32-wide K
// sub-block of every weight tile per slot).  Two CTAs share an SM, so a CTA may hold at most 256 columns.
template <bool GATEUP> struct GemmShape {
    static constexpr int kATiles = GATEUP ? 2 : 1;                     // weight tiles (gate and up, or down)
    static constexpr int kTileN = GATEUP ? kTileNGateUp : uocr::kTileN;   // tokens per tile = columns per accumulator
    static constexpr int kAStages = 4;
    static constexpr int kAccCols = kATiles * kTileN;                  // 256
    static constexpr int kAStageCols = kATiles * 32;                   // 32 columns = one 64-wide K block per weight tile
    static constexpr int kTmemCols = 512;
    static_assert(kAccCols + kAStages * kAStageCols <= kTmemCols, "tensor memory budget");
    static constexpr int kBStages = GATEUP ? 6 : 4;
    static constexpr int kBTileBytes = kTileN * kBlockK * 2;           // 16 or 32 KB
    static constexpr int kMaxKBlocks = 32;                             // K <= 2048
    static constexpr int kScaleBytes = 2 * kATiles * kTileM * kMaxKBlocks * 2;    // two tiles' worth: [tile parity][matrix][row][k block]
    static constexpr int kSmemBytes = kBStages * kBTileBytes + kScaleBytes + 1024 /*alignment*/ + 256 /*barriers*/;
};

template <int QT, bool GATEUP>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap act_map, GemmParams p) {
    using Sh = GemmShape<GATEUP>;
    constexpr int kAStages = Sh::kAStages, kBStages = Sh::kBStages, kTileN = Sh::kTileN;
    // Persistent: the grid has at most one CTA per SM, and CTA b takes tiles b, b + gridDim.x, ... of the list (hottest
    // expert first).  Barriers and tensor memory are set up once; the rings' phases run on across tiles, and the
    // activation loader works ahead into the next tile while the other warps finish the current one.
    const uint32_t n_tiles = *p.tile_count;
    if (blockIdx.x >= n_tiles) return;
    const uint32_t kblocks = p.k_dim / kBlockK;

    extern __shared__ uint8_t smem_dyn[];
    uint8_t *b_tiles = reinterpret_cast<uint8_t *>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    __half *s_scales = reinterpret_cast<__half *>(b_tiles + kBStages * Sh::kBTileBytes);   // [tile parity][kATiles][128][kMaxKBlocks]
    uint64_t *bars = reinterpret_cast<uint64_t *>(b_tiles + kBStages * Sh::kBTileBytes + Sh::kScaleBytes);
    uint64_t *a_full = bars, *a_empty = a_full + kAStages, *b_full = a_empty + kAStages, *b_empty = b_full + kBStages,
             *acc_full = b_empty + kBStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kAStages; ++s) { gb_init(&a_full[s], kProducerThreads / 32); gb_init(&a_empty[s], 1); }
        for (int s = 0; s < kBStages; ++s) { gb_init(&b_full[s], 1); gb_init(&b_empty[s], 1); }
        gb_init(acc_full, 1);
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

    if (warp < 16) {
        // ------------------------------------------------ weight rows -> fp16 -> tensor memory, then the epilogue
        // Two groups of 256 threads.  gate/up: group g converts matrix g (gate / up).  down: group g converts
        // the g-th 32-wide sub-block of every K block.  Inside a group, thread (r, h) owns row r and the K
        // positions [16h, 16h+16) of a sub-block.
        const int grp = tid >> 8, r = tid & 127, h = (tid >> 7) & 1;
        constexpr int kAhead = PackedBlock<QT>::kAhead, kVecs = PackedBlock<QT>::kVecs;
        const int sm = GATEUP ? grp : 0;                              // which matrix's scales this thread uses
        // this thread's TMEM lane, its 8 columns inside a 16-column sub-block, and its matrix inside a slot
        const uint32_t lane_addr = ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)h * 8 + (GATEUP ? (uint32_t)grp * 32 : 0u);
        bool alive = true;
        uint32_t kbase = 0, it = 0;                                   // K blocks and tiles this CTA has gone through
#pragma unroll 1
        for (uint32_t tile_idx = blockIdx.x; tile_idx < n_tiles && alive; tile_idx += gridDim.x, kbase += kblocks, ++it) {
            const uint4 tile = p.tiles[tile_idx];
            const uint32_t expert = tile.x, mtile = tile.y, row0 = tile.z, nrows = tile.w;
            const size_t grow = (size_t)mtile * kTileM + r;               // row of the matrix
            const uint8_t *rowp = ((GATEUP && grp) ? p.w1 : p.w0) + (size_t)expert * p.expert_stride_bytes + grow * p.row_bytes;
            // the first packed blocks are requested before the scales are waited for: one memory latency, not two
            uint4 v[kAhead][kVecs];
#pragma unroll
            for (int d = 0; d < kAhead; ++d)
                if ((uint32_t)d < kblocks) load_block<QT>(rowp, d, h, v[d]);
            // The row's scales go to shared memory once ([matrix][row][k block], one buffer per tile parity, so the
            // previous tile's readers need not be waited for): the K loop never waits on a 2-byte global load.  A row's
            // scales are contiguous: 4-byte loads, all issued before the first store.
            __half *tile_scales = s_scales + (size_t)(it & 1u) * (Sh::kATiles * kTileM * Sh::kMaxKBlocks);
            if (QT != UOCR_QT_F16 && h == 0 && (GATEUP || grp == 0)) {
                // (K is a multiple of 128, so a row holds an even number of scales and starts on a 4-byte boundary)
                const uint32_t *sc = reinterpret_cast<const uint32_t *>((sm == 0 ? p.s0 : p.s1) + (size_t)expert * p.expert_scale_stride + grow * kblocks);
                uint32_t *dst = reinterpret_cast<uint32_t *>(tile_scales + ((size_t)sm * kTileM + r) * Sh::kMaxKBlocks);
                uint32_t t[Sh::kMaxKBlocks / 2];
#pragma unroll
                for (int i = 0; i < Sh::kMaxKBlocks / 2; ++i) t[i] = (uint32_t)(2 * i) < kblocks ? __ldg(sc + i) : 0u;
#pragma unroll
                for (int i = 0; i < Sh::kMaxKBlocks / 2; ++i)
                    if ((uint32_t)(2 * i) < kblocks) dst[i] = t[i];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory");     // scales visible to every thread of a row
            const __half *my_scales = tile_scales + ((size_t)sm * kTileM + r) * Sh::kMaxKBlocks;
            int pending = -1;       // slot whose tensor-memory stores are in flight: published one block later, so that
                                    // the stores' latency hides behind the next block's conversion
            auto publish = [&]() {
                tc_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) gb_arrive(&a_full[pending]);              // one arrival per warp: its stores have all landed
            };
            for (uint32_t kb0 = 0; kb0 < kblocks && alive; kb0 += kAhead) {
#pragma unroll
                for (int d = 0; d < kAhead; ++d) {
                    const uint32_t kb = kb0 + d;
                    if (kb >= kblocks) break;
                    const __half sc = QT == UOCR_QT_F16 ? __ushort_as_half(0) : my_scales[kb];
                    const uint32_t kbg = kbase + kb, slot = kbg % kAStages, use = kbg / kAStages;
                    // gate/up: both 32-wide sub-blocks of this thread's matrix; down: the group's sub-block
                    uint32_t regs[2][8];
                    if (GATEUP) { convert_sub<QT>(v[d], 0, sc, regs[0]); convert_sub<QT>(v[d], 1, sc, regs[1]); }
                    else convert_sub<QT>(v[d], grp, sc, regs[0]);
                    if (kb + kAhead < kblocks) load_block<QT>(rowp, kb + kAhead, h, v[d]);
                    if (pending >= 0) publish();
                    if (use > 0 && !gb_wait(&a_empty[slot], (use - 1) & 1u, abort_flag, p.status)) { alive = false; pending = -1; break; }
                    __syncwarp();
                    tc_fence_after();
                    const uint32_t dst = a_base + slot * Sh::kAStageCols + lane_addr;
                    if (GATEUP) { tc_st8(dst, regs[0]); tc_st8(dst + 16, regs[1]); }
                    else tc_st8(dst + (uint32_t)grp * 16, regs[0]);
                    pending = (int)slot;
                }
            }
            if (pending >= 0) publish();
            // ------------------------------------------------ epilogue: TMEM -> registers -> global
            const bool have_acc = alive && gb_wait(acc_full, it & 1u, abort_flag, p.status);
            __syncwarp();
            if (__all_sync(0xffffffffu, have_acc)) {
                tc_fence_after();
                // a warp reads the TMEM lanes 32*(warp % 4)..+31; the four warps of a lane quarter split the 16-column
                // chunks.  All of a warp's chunks are requested before the first is used.
                constexpr int kChunks = kTileN / 64;
                const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
                const size_t out_col = (size_t)mtile * kTileM + r;
                const uint32_t cbase = (uint32_t)(warp >> 2) * 16;
#pragma unroll
                for (int i = 0; i < kChunks; ++i) {          // chunk by chunk: the registers of one chunk at a time
                    const uint32_t c0 = cbase + 64 * i;
                    if (c0 < nrows) {
                        uint32_t g[16], u[16];
                        tc_ld16(lane_base + c0, g);
                        if (GATEUP) tc_ld16(lane_base + kTileN + c0, u);
                        tc_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (c0 + j < nrows) {
                                const float a = __uint_as_float(g[j]);
                                const float o = GATEUP ? silu_fast(a) * __uint_as_float(u[j]) : a;
                                p.out[(size_t)(row0 + c0 + j) * p.out_ld + out_col] = __float2half_rn(o);
                            }
                        }
                    }
                }
            } else {
                alive = false;
            }
            tc_fence_before();
        }
    } else if (warp == kTmaWarp) {
        // ------------------------------------------------ activation tiles by TMA (runs ahead into the next tile)
        if (lane == 0) {
            uint32_t kbase = 0;
            bool ok = true;
            for (uint32_t tile_idx = blockIdx.x; tile_idx < n_tiles && ok; tile_idx += gridDim.x, kbase += kblocks) {
                const uint32_t row0 = p.tiles[tile_idx].z;
                for (uint32_t kb = 0; kb < kblocks; ++kb) {
                    const uint32_t kbg = kbase + kb, use = kbg / kBStages;
                    const int s = kbg % kBStages;
                    if (use > 0 && !gb_wait(&b_empty[s], (use - 1) & 1u, abort_flag, p.status)) { ok = false; break; }
                    gb_expect_tx(&b_full[s], Sh::kBTileBytes);
                    tma_load_2d(b_tiles + s * Sh::kBTileBytes, &act_map, (int)(kb * kBlockK), (int)row0, &b_full[s]);
                }
            }
        }
    } else {
        // ------------------------------------------------ MMA issue
        if (lane == 0) {
            uint32_t kbase = 0;
            bool ok = true;
            for (uint32_t tile_idx = blockIdx.x; tile_idx < n_tiles && ok; tile_idx += gridDim.x, kbase += kblocks) {
                const uint32_t nrows = p.tiles[tile_idx].w;
                const uint32_t idesc = umma_idesc((nrows + 15u) & ~15u);          // MMA N: multiple of 16
                // the accumulators of the previous tile have been read: every producer warp publishes its first block
                // of this tile only after its own epilogue, and the first MMA waits for all sixteen
                for (uint32_t kb = 0; kb < kblocks && ok; ++kb) {
                    const uint32_t kbg = kbase + kb, slot = kbg % kAStages, bs = kbg % kBStages;
                    ok = gb_wait(&a_full[slot], (kbg / kAStages) & 1u, abort_flag, p.status);
                    if (ok) ok = gb_wait(&b_full[bs], (kbg / kBStages) & 1u, abort_flag, p.status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t b_addr = s2u(b_tiles + bs * Sh::kBTileBytes);
                    const uint32_t a_addr = a_base + slot * Sh::kAStageCols;
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k) {
                        const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
                        const uint64_t bd = umma_desc(b_addr + k * 32);
                        tc_mma_ts(tmem_base, a_addr + k * 8, bd, idesc, acc);
                        if (GATEUP) tc_mma_ts(tmem_base + kTileN, a_addr + 32 + k * 8, bd, idesc, acc);
                    }
                    tc_commit(&a_empty[slot]);                // arrives when the MMAs above have read the slot
                    tc_commit(&b_empty[bs]);
                }
                if (ok) tc_commit(acc_full);
            }
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
// Tile lists of the routed GEMMs: for every expert with pairs, gate/up tiles of (64 tokens, 128 weight rows)
// and down tiles of (128 tokens, 128 weight rows).  Entries are {expert, weight-row tile, first sorted
// position, rows}; counts[0/1] are the list lengths.
// Segment e uses the weights of expert expert_base + e % expert_mod (single GPU: base 0, mod E; expert-parallel
// ranks receive one segment per (source rank, local expert)).
__global__ void tile_plan_kernel(const uint32_t *__restrict__ expert_offsets, uint32_t E, uint32_t expert_base,
                                 uint32_t expert_mod, uint32_t gu_mtiles, uint32_t dn_mtiles, uint4 *__restrict__ tiles_gu,
                                 uint4 *__restrict__ tiles_dn, uint32_t *__restrict__ counts) {
    // The lists start with the segment that has the most rows (ties: lower index first): the persistent GEMM kernel
    // deals tiles to its CTAs in list order, so the long segments are under way first and the short ones fill the tail.
    __shared__ uint32_t base_gu[257], base_dn[257], order[256];
    const uint32_t e = threadIdx.x;
    if (e < E) {
        const uint32_t c = expert_offsets[e + 1] - expert_offsets[e];
        uint32_t rank = 0;
        for (uint32_t j = 0; j < E; ++j) {
            const uint32_t cj = expert_offsets[j + 1] - expert_offsets[j];
            rank += (cj > c || (cj == c && j < e)) ? 1u : 0u;
        }
        order[rank] = e;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t rg = 0, rd = 0;
        for (uint32_t k = 0; k < E; ++k) {
            const uint32_t i = order[k];
            const uint32_t c = expert_offsets[i + 1] - expert_offsets[i];
            base_gu[i] = rg; base_dn[i] = rd;
            rg += (c + kTileNGateUp - 1) / kTileNGateUp;
            rd += (c + kTileN - 1) / kTileN;
        }
        counts[0] = rg * gu_mtiles;
        counts[1] = rd * dn_mtiles;
    }
    __syncthreads();
    if (e < E) {
        const uint32_t lo = expert_offsets[e], cnt = expert_offsets[e + 1] - lo;
        for (uint32_t t = 0; t * kTileNGateUp < cnt; ++t) {
            const uint32_t r0 = lo + t * kTileNGateUp, nr = min((uint32_t)kTileNGateUp, cnt - t * kTileNGateUp);
            for (uint32_t m = 0; m < gu_mtiles; ++m) tiles_gu[(size_t)(base_gu[e] + t) * gu_mtiles + m] = make_uint4(expert_base + e % expert_mod, m, r0, nr);
        }
        for (uint32_t t = 0; t * kTileN < cnt; ++t) {
            const uint32_t r0 = lo + t * kTileN, nr = min((uint32_t)kTileN, cnt - t * kTileN);
            for (uint32_t m = 0; m < dn_mtiles; ++m) tiles_dn[(size_t)(base_dn[e] + t) * dn_mtiles + m] = make_uint4(expert_base + e % expert_mod, m, r0, nr);
        }
    }
}

// Tile lists of the shared MLP (one "expert", all n tokens).
__global__ void shared_tile_plan_kernel(uint32_t n, uint32_t gu_mtiles, uint32_t dn_mtiles, uint4 *__restrict__ tiles_gu,
                                        uint4 *__restrict__ tiles_dn, uint32_t *__restrict__ counts) {
    const uint32_t tg = (n + kTileNGateUp - 1) / kTileNGateUp, td = (n + kTileN - 1) / kTileN;
    const uint32_t stride = gridDim.x * blockDim.x, i0 = blockIdx.x * blockDim.x + threadIdx.x;
    for (uint32_t i = i0; i < tg * gu_mtiles; i += stride) {
        const uint32_t t = i / gu_mtiles, m = i % gu_mtiles, r0 = t * kTileNGateUp;
        tiles_gu[i] = make_uint4(0, m, r0, min((uint32_t)kTileNGateUp, n - r0));
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
    for (uint32_t i = lane; i < H / 8; i += 32) dst[i] = __ldg(src + i);
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
    for (uint32_t s = 0; s < K; ++s) {
        const uint32_t pos = inverse[t * K + s], e = top_ids[t * K + s];
        if (pos == 0xffffffffu || e >= E) continue;
        const unsigned long long row = (unsigned long long)dst_row0[e] + (pos - expert_offsets[e]);
        if (row >= row_capacity) { atomicOr(status, kStatusPeerRange); continue; }
        const float w = weights[t * K + s];
        const uint4 v = ld_volatile_v4(reinterpret_cast<const uint4 *>(peer.p[e / experts_per_rank] + (size_t)row * H + c));
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
                                   GemmShape<GU>::kSmemBytes);
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
    const size_t smem = GemmShape<GU>::kSmemBytes;
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
    const uint32_t ttiles_gu = (rows_bound + kTileNGateUp - 1) / kTileNGateUp + n_seg;
    const uint32_t ttiles_dn = (rows_bound + kTileN - 1) / kTileN + n_seg;
    cudaError_t err;
    tile_plan_kernel<<<1, 256, 0, st>>>(seg_offsets, n_seg, expert_base, expert_mod, F / kTileM, H / kTileM, G.tiles_gu,
                                        G.tiles_dn, G.counts);
    ++*launches;
    if ((err = cudaGetLastError()) != cudaSuccess) return err;
    CUtensorMap map_x, map_mid;
    if ((err = make_map_rows(&map_x, rows_in, rows_bound, H, kTileNGateUp)) != cudaSuccess) return err;
    if ((err = make_map_rows(&map_mid, mid, rows_bound, F, kTileN)) != cudaSuccess) return err;
    const int qt = L.expert_qtype;
    GemmParams p = base_params(S);
    p.w0 = L.expert_w; p.w1 = L.expert_w + L.up_offset_bytes;
    p.s0 = L.expert_s; p.s1 = L.expert_s ? L.expert_s + L.up_scale_offset : nullptr;
    p.expert_stride_bytes = L.expert_stride_bytes; p.expert_scale_stride = L.expert_scale_stride;
    p.row_bytes = packed_row_bytes_of(qt, H); p.k_dim = H;
    p.tiles = G.tiles_gu; p.tile_count = G.counts; p.out = mid; p.out_ld = F;
    if ((err = launch_gemm<true>(qt, map_x, p, ttiles_gu * (F / kTileM), st)) != cudaSuccess) return err;
    p.w0 = L.expert_w + L.down_offset_bytes; p.w1 = nullptr;
    p.s0 = L.expert_s ? L.expert_s + L.down_scale_offset : nullptr; p.s1 = nullptr;
    p.row_bytes = packed_row_bytes_of(qt, F); p.k_dim = F;
    p.tiles = G.tiles_dn; p.tile_count = G.counts + 1; p.out = rows_out; p.out_ld = H;
    if ((err = launch_gemm<false>(qt, map_mid, p, ttiles_dn * (H / kTileM), st)) != cudaSuccess) return err;
    *launches += 2;
    return cudaSuccess;
}

// Shared MLP on all n tokens: G.shared_out[n][H] = fp16( down( silu(gate x) * up x ) ).
cudaError_t launch_gemm_shared(const DLayer &L, const Scratch &S, const GemmScratch &G, const __half *hidden, uint32_t n,
                               cudaStream_t st, uint64_t *launches) {
    const uint32_t H = L.H, Sd = L.S;
    const uint32_t sttiles_gu = (n + kTileNGateUp - 1) / kTileNGateUp, sttiles_dn = (n + kTileN - 1) / kTileN;
    cudaError_t err;
    shared_tile_plan_kernel<<<8, 256, 0, st>>>(n, Sd / kTileM, H / kTileM, G.stiles_gu, G.stiles_dn, G.counts + 2);
    ++*launches;
    CUtensorMap map_hidden, map_smid;
    if ((err = make_map_rows(&map_hidden, hidden, n, H, kTileNGateUp)) != cudaSuccess) return err;
    if ((err = make_map_rows(&map_smid, G.shared_mid, n, Sd, kTileN)) != cudaSuccess) return err;
    GemmParams p = base_params(S);
    p.w0 = L.shared_gate.w; p.w1 = L.shared_up.w; p.s0 = L.shared_gate.s; p.s1 = L.shared_up.s;
    p.row_bytes = L.shared_gate.row_bytes; p.k_dim = H;
    p.tiles = G.stiles_gu; p.tile_count = G.counts + 2; p.out = G.shared_mid; p.out_ld = Sd;
    if ((err = launch_gemm<true>(L.shared_gate.qtype, map_hidden, p, sttiles_gu * (Sd / kTileM), st)) != cudaSuccess) return err;
    p.w0 = L.shared_down.w; p.w1 = nullptr; p.s0 = L.shared_down.s; p.s1 = nullptr;
    p.row_bytes = L.shared_down.row_bytes; p.k_dim = Sd;
    p.tiles = G.stiles_dn; p.tile_count = G.counts + 3; p.out = G.shared_out; p.out_ld = H;
    if ((err = launch_gemm<false>(L.shared_down.qtype, map_smid, p, sttiles_dn * (H / kTileM), st)) != cudaSuccess) return err;
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

// ---- dequantisation probe ------------------------------------------------------------------------------------
// out[row][col] = the fp16 value (widened to f32) the grouped GEMM's producer threads store into tensor memory for
// weight (row, col): the same load_block / convert_sub pair, one thread per (row, 64-wide K block, half h).
template <int QT>
__global__ void producer_probe_kernel(const uint8_t *__restrict__ w, const __half *__restrict__ s, uint32_t rows, uint32_t cols,
                                      uint32_t row_bytes, float *__restrict__ out) {
    const uint32_t kblocks = cols / kBlockK;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * kblocks * 2) return;
    const int h = (int)(idx & 1);
    const uint32_t kb = (uint32_t)((idx >> 1) % kblocks), row = (uint32_t)((idx >> 1) / kblocks);
    uint4 v[PackedBlock<QT>::kVecs];
    load_block<QT>(w + (size_t)row * row_bytes, kb, h, v);
    const __half sc = QT == UOCR_QT_F16 ? __ushort_as_half(0) : s[(size_t)row * kblocks + kb];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        uint32_t regs[8];
        convert_sub<QT>(v, j, sc, regs);
        float *dst = out + (size_t)row * cols + (size_t)kb * kBlockK + 32 * j + 16 * h;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&regs[i]));
            dst[2 * i] = f.x;
            dst[2 * i + 1] = f.y;
        }
    }
}

cudaError_t launch_producer_probe(const DMatrix &m, float *out, cudaStream_t st, uint64_t *launches) {
    const size_t work = (size_t)m.rows * (m.cols / kBlockK) * 2;
    const unsigned blocks = (unsigned)((work + 255) / 256);
    switch (m.qtype) {
        case UOCR_QT_Q4: producer_probe_kernel<UOCR_QT_Q4><<<blocks, 256, 0, st>>>(m.w, m.s, m.rows, m.cols, m.row_bytes, out); break;
        case UOCR_QT_Q8: producer_probe_kernel<UOCR_QT_Q8><<<blocks, 256, 0, st>>>(m.w, m.s, m.rows, m.cols, m.row_bytes, out); break;
        default: producer_probe_kernel<UOCR_QT_F16><<<blocks, 256, 0, st>>>(m.w, m.s, m.rows, m.cols, m.row_bytes, out); break;
    }
    ++*launches;
    return cudaGetLastError();
}

}  // namespace uocr

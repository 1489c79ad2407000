// Shared by the single-token and the batched decode kernels: the model's shapes, the slice-major "unit blob" copy
// of a layer's quantised weights, the integer MMAs on packed levels, and the block-floating-point form of fp16
// activations that feeds them.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "moe_common.cuh"

namespace uocr {

constexpr int kSlH = 1280, kSlF = 896, kSlS = 1792, kSlK = 6, kSlE = 64;    // the model's MoE layer
constexpr int kSlRoutedPerSlot = kSlF / 64;                 // 14 slices of 64 intermediate columns per routed expert
constexpr int kSlGroups = kSlH / 64;                        // 20 quantisation groups along H

// ---------------------------------------------------------------- packed formats and the unit blob
template <int QT> struct SlFmt;
template <> struct SlFmt<UOCR_QT_Q4> {
    static constexpr int kGroupBytes = 32, kLaneBytes = 8;             // of one row: per 64-wide group, per lane of a quad
    static constexpr int kRowBytesH = kSlH / 2;
};
template <> struct SlFmt<UOCR_QT_Q8> {
    static constexpr int kGroupBytes = 64, kLaneBytes = 16;
    static constexpr int kRowBytesH = kSlH;
};
template <int QT> struct SlBlob {
    static constexpr int kGu = 0;                                           // gate/up fragments
    static constexpr int kGuBytes = 128 * SlFmt<QT>::kRowBytesH;
    static constexpr int kGuSc = kGu + kGuBytes;                            // gate scales [64][20], up scales [64][20]
    static constexpr int kGuScBytes = 2 * 64 * kSlGroups * 2;
    static constexpr int kDn = kGuSc + kGuScBytes;                          // down fragments
    static constexpr int kDnBytes = kSlH * SlFmt<QT>::kGroupBytes;
    static constexpr int kDnSc = kDn + kDnBytes;                            // down scales [H]
    static constexpr int kBytes = kDnSc + kSlH * 2;                         // Q4: 130560, Q8: 253440 (multiples of 256)
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void imma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One 64-wide group of two weight rows (lo: MMA rows 0-7, hi: MMA rows 8-15; this lane holds its 16 levels of
// each) against the group's activation bytes xb: two MMAs, the first 32 columns of the group into accumulator a,
// the other 32 into accumulator b, so that consecutive groups form independent chains.  Which column sits in
// which k slot follows from the packing; limb_column() below arranges the activation bytes to match.
// Q4_0 stores level + 8 in a nibble.  A nibble moved to the top of its byte with bit 7 flipped is the signed byte
// 16 * level (offset binary -> two's complement), so the MMA sees signed operands and no offset term is left to
// remove afterwards; the factor 16 is folded into the activation scale.  One LOP3 for the high nibbles, a shift
// and a LOP3 for the low ones.
__device__ __forceinline__ uint32_t q4_hi16(uint32_t x) { return (x & 0xF0F0F0F0u) ^ 0x80808080u; }
__device__ __forceinline__ uint32_t q4_lo16(uint32_t x) { return ((x << 4) & 0xF0F0F0F0u) ^ 0x80808080u; }
constexpr float kQ4LevelScale = 1.0f / 16.0f;
__device__ __forceinline__ void group_imma(int (&ca)[4], int (&cb)[4], const uint2 &lo, const uint2 &hi, const uint4 &xb) {   // Q4_0
    imma_s8(ca, q4_lo16(lo.x), q4_lo16(hi.x), q4_lo16(lo.y), q4_lo16(hi.y), xb.x, xb.y);     // low nibbles
    imma_s8(cb, q4_hi16(lo.x), q4_hi16(hi.x), q4_hi16(lo.y), q4_hi16(hi.y), xb.z, xb.w);     // high nibbles
}
__device__ __forceinline__ void group_imma(int (&ca)[4], int (&cb)[4], const uint4 &lo, const uint4 &hi, const uint4 &xb) {   // Q8_0
    imma_s8(ca, lo.x, hi.x, lo.y, hi.y, xb.x, xb.y);
    imma_s8(cb, lo.z, hi.z, lo.w, hi.w, xb.z, xb.w);
}
// first of the four consecutive columns (inside the group) behind activation word p = 4 t + 2 j + r of a group:
// lane-in-quad t, MMA j of the group, B register r
template <int QT>
__device__ __forceinline__ int limb_column(int p) {
    const int t = p >> 2, j = (p >> 1) & 1, r = p & 1;
    return QT == UOCR_QT_Q4 ? 32 * j + 8 * t + 4 * r : 16 * t + 8 * j + 4 * r;
}

// Block-floating-point form of one 64-wide group of fp16 values, computed by 16 consecutive lanes (this lane: the
// four values x[0..3] behind its word): a shared power-of-two scale 2^(e - 13) and signed 15-bit mantissas (exact
// for every value within a factor 8 of the group's largest, rounded to 2^-14 of the largest's power of two
// otherwise), each split into a signed low byte and a signed high byte (|high| <= 64).
struct GroupLimbs {
    uint32_t lo, hi;      // the low / high bytes of this lane's four values
    float scale;
};
// mask: the lanes that take part (the caller's half-warp of 16 lanes, or the whole warp when both halves do)
__device__ __forceinline__ GroupLimbs group_limbs16(const float (&x)[4], uint32_t mask) {
    float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(mask, amax, o, 16));
    // amax = 1.f * 2^e (fp16 values: e in [-24, 15]); up = 2^(13 - e), scale = 2^(e - 13); a group of zeros gets 0
    const int e = (int)(__float_as_uint(amax) >> 23) - 127;
    const bool live = amax > 0.f && amax < INFINITY;
    const float up = live ? __uint_as_float((uint32_t)(127 + 13 - e) << 23) : 0.f;
    GroupLimbs out;
    out.lo = 0u; out.hi = 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = __float2int_rn(x[i] * up);          // |m| < 2^14
        const int l0 = (int)((uint32_t)m << 24) >> 24, l1 = (m - l0) >> 8;
        out.lo |= (uint32_t)(l0 & 0xff) << (8 * i);
        out.hi |= (uint32_t)(l1 & 0xff) << (8 * i);
    }
    out.scale = live ? __uint_as_float((uint32_t)(127 - 13 + e) << 23) : 0.f;
    return out;
}
__device__ __forceinline__ GroupLimbs group_limbs(const float (&x)[4]) { return group_limbs16(x, 0xffffffffu); }
// the four fp16 values behind word p of a group in shared memory
template <int QT>
__device__ __forceinline__ void load_word_values(const __half *group, int p, float (&x)[4]) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(group + limb_column<QT>(p));
    const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
    const float2 f23 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
    x[0] = f01.x; x[1] = f01.y; x[2] = f23.x; x[3] = f23.y;
}


}  // namespace uocr

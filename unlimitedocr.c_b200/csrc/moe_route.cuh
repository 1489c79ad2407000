// Softmax + greedy top-k of one token by one warp: the arithmetic of the reference's CPU router
// (src/backend/cpu_ref/uocr_cpu_ref.c:430-463) - max-shifted exp with the host C library's expf bits,
// the denominator summed serially in expert order, IEEE division, K rounds of arg-max in which a
// strictly greater probability wins and equal probabilities go to the lower expert id.
#pragma once

#include "expf_compat.h"
#include "moe_common.cuh"

namespace uocr {

extern __constant__ uint64_t c_exp_tab[UOCR_EXPF_N];

// l: logits [E] (shared memory), p: probabilities [E] (shared memory, written).  Results go to
// ids_out[K] / weights_out[K] (any address space; written by lane 0) and, when not null, to
// logits_out / probs_out.  Returns true when the row is invalid (non-finite logits, empty softmax).
// kPerLane * 32 >= E.  exp_tab is the 32-entry table of expf_compat.h in SHARED memory (lanes index it with
// different values; constant memory would serialise those reads).  The selection compares probabilities as
// unsigned integers, which orders non-negative floats exactly as the float comparison does.
template <int kPerLane>
__device__ __forceinline__ bool route_row_warp_n(const float *l, float *p, uint32_t E, uint32_t K, float scaling,
                                                 int lane, const uint64_t *exp_tab, float *logits_out,
                                                 float *probs_out, uint32_t *ids_out, float *weights_out) {
    float lv[kPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const uint32_t e = lane + 32 * i;
        lv[i] = e < E ? l[e] : -INFINITY;
        mx = fmaxf(mx, lv[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    bool bad = !isfinite(mx);
    float pv[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const uint32_t e = lane + 32 * i;
        if (e < E) {
            pv[i] = uocr_expf_compat(__fsub_rn(lv[i], mx), exp_tab);
            p[e] = pv[i];
        } else {
            pv[i] = 0.f;
        }
    }
    __syncwarp();
    // denominator: one serial chain in expert order; the shared-memory reads are batched ahead of the adds
    float denom = 0.f;
    if (lane == 0) {
        for (uint32_t e0 = 0; e0 < E; e0 += 16) {
            float t[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) t[i] = e0 + i < E ? p[e0 + i] : 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (e0 + i < E) denom = __fadd_rn(denom, t[i]);
        }
    }
    denom = __shfl_sync(0xffffffffu, denom, 0);
    bad = bad || !(denom > 0.f) || !isfinite(denom);
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const uint32_t e = lane + 32 * i;
        if (e < E) {
            pv[i] = __fdiv_rn(pv[i], denom);
            p[e] = pv[i];
            if (logits_out) logits_out[e] = lv[i];
            if (probs_out) probs_out[e] = pv[i];
        }
    }
    // greedy top-k: bit i of `taken` marks expert lane + 32*i as selected
    uint32_t taken = 0;
    for (uint32_t slot = 0; slot < K; ++slot) {
        uint32_t bb = 0, be = 0xffffffffu;       // best probability bits / expert of this lane
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const uint32_t e = lane + 32 * i;
            const uint32_t bits = __float_as_uint(pv[i]);
            if (e < E && !((taken >> i) & 1u) && (be == 0xffffffffu || bits > bb)) { bb = bits; be = e; }
        }
        const uint32_t top = __reduce_max_sync(0xffffffffu, be == 0xffffffffu ? 0u : bb);
        const uint32_t win = __reduce_min_sync(0xffffffffu, (be != 0xffffffffu && bb == top) ? be : 0xffffffffu);
        if (win == 0xffffffffu) bad = true;
        if (win != 0xffffffffu && (win & 31u) == (uint32_t)lane) taken |= 1u << (win >> 5);
        if (lane == 0) {
            ids_out[slot] = bad ? 0xffffffffu : win;
            weights_out[slot] = bad ? 0.f : __fmul_rn(__uint_as_float(top), scaling);
        }
    }
    return bad;
}

__device__ __forceinline__ bool route_row_warp(const float *l, float *p, uint32_t E, uint32_t K, float scaling, int lane,
                                               const uint64_t *exp_tab, float *logits_out, float *probs_out,
                                               uint32_t *ids_out, float *weights_out) {
    if (E <= 64) return route_row_warp_n<2>(l, p, E, K, scaling, lane, exp_tab, logits_out, probs_out, ids_out, weights_out);
    return route_row_warp_n<8>(l, p, E, K, scaling, lane, exp_tab, logits_out, probs_out, ids_out, weights_out);
}

}  // namespace uocr

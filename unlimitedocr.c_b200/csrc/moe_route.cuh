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
__device__ __forceinline__ bool route_row_warp(const float *l, float *p, uint32_t E, uint32_t K, float scaling, int lane,
                                               float *logits_out, float *probs_out, uint32_t *ids_out,
                                               float *weights_out) {
    float mx = -INFINITY;
    for (uint32_t e = lane; e < E; e += 32) mx = fmaxf(mx, l[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    bool bad = !isfinite(mx);
    for (uint32_t e = lane; e < E; e += 32) p[e] = uocr_expf_compat(__fsub_rn(l[e], mx), c_exp_tab);
    __syncwarp();
    float denom = 0.f;
    if (lane == 0)
        for (uint32_t e = 0; e < E; ++e) denom = __fadd_rn(denom, p[e]);   // serial, expert order
    denom = __shfl_sync(0xffffffffu, denom, 0);
    bad = bad || !(denom > 0.f) || !isfinite(denom);
    for (uint32_t e = lane; e < E; e += 32) p[e] = __fdiv_rn(p[e], denom);
    __syncwarp();
    if (logits_out) for (uint32_t e = lane; e < E; e += 32) logits_out[e] = l[e];
    if (probs_out) for (uint32_t e = lane; e < E; e += 32) probs_out[e] = p[e];

    // `taken` bit i of a lane marks expert lane + 32*i as already selected
    uint32_t taken = 0;
    for (uint32_t slot = 0; slot < K; ++slot) {
        float bp = -INFINITY;
        uint32_t be = 0xffffffffu;
        for (uint32_t e = lane, i = 0; e < E; e += 32, ++i) {
            if ((taken >> i) & 1u) continue;
            const float pe = p[e];
            if (pe > bp || (pe == bp && e < be)) { bp = pe; be = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float op = __shfl_xor_sync(0xffffffffu, bp, o);
            const uint32_t oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (op > bp || (op == bp && oe < be)) { bp = op; be = oe; }
        }
        if (be == 0xffffffffu || !(bp >= 0.f)) bad = true;
        if (be != 0xffffffffu && (be & 31u) == (uint32_t)lane) taken |= 1u << (be >> 5);
        if (lane == 0) {
            ids_out[slot] = bad ? 0xffffffffu : be;
            weights_out[slot] = bad ? 0.f : __fmul_rn(bp, scaling);
        }
    }
    return bad;
}

}  // namespace uocr

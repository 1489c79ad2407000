/*
 * CPU oracle for the decoder MoE layer.  TEST INFRASTRUCTURE ONLY: it is the
 * checker for the CUDA path and the timed CPU baseline; nothing in the shipped
 * library links, loads or calls it.
 *
 * It restates, in plain C and f32 arithmetic, the algorithm of the reference's
 * scalar CPU backend:
 *   - half <-> float conversion      src/backend/cpu_ref/uocr_cpu_ref.c:26-101
 *   - the dot product (one serial fmaf chain per output)        ...:291-299
 *   - silu(v) = v / (1 + expf(-v))                              ...:301-303
 *   - dense SwiGLU MLP                                          ...:305-349
 *   - router: logits, max-shifted expf softmax with a serial denominator,
 *     greedy top-k, ties to the lower expert id                 ...:388-466
 *   - MoE layer: routed experts in slot order with
 *     out = fmaf(weight, down, out), then the shared MLP added  ...:468-579
 * and, for the quantised expert slabs, the dequantisation rule of the model
 * format (value = integer level * float(fp16 scale), one scale per 64 inputs):
 *   - Q8_0  src/model/uocr_format.h:49-69
 *   - Q4_0 with half-split nibbles (byte j of a group holds level[j]+8 in the
 *     low nibble and level[j+32]+8 in the high nibble)  src/model/uocr_format.h:71-99
 *   - expert-major slab: per expert gate rows, up rows, down rows; the scale
 *     slab in the same order  src/unlimitedocr_c/convert.py:966-996
 *
 * Every output element is produced by exactly the same sequence of roundings
 * as the reference (a left-to-right fmaf chain), so results are bit-identical
 * to the reference library built from its own sources (checked by the tests
 * whenever that build is present).  Several independent chains are interleaved
 * per loop only to use the FMA pipe; the order inside each chain is unchanged.
 *
 * Parity is pinned: tests/test_oracle_golden.py checks this file against the
 * reference's committed golden vectors (tests/fixtures/cpu_ref_tiny_golden.h
 * values, stored in tests/golden/) and its hand-computed cases.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MO_QTYPE_F16 1
#define MO_QTYPE_Q8_0 3
#define MO_QTYPE_Q4_0 4
#define MO_GROUP 64u

/* ------------------------------------------------------------------ half */

static uint32_t mo_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static float mo_float(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

float mo_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp5 = (h >> 10) & 31u;
    const uint32_t frac = h & 1023u;
    if (exp5 == 31u) return mo_float(sign | 0x7f800000u | (frac << 13));
    if (exp5 != 0u) return mo_float(sign | ((exp5 + 112u) << 23) | (frac << 13));
    if (frac == 0u) return mo_float(sign);
    /* subnormal half = frac * 2^-24, exact in float */
    const float mag = (float)frac * 5.9604644775390625e-08f;
    return mo_float(sign | mo_bits(mag));
}

/* round-to-nearest-even, NaN -> quiet NaN 0x7e00, overflow -> inf */
uint16_t mo_f32_to_f16(float value) {
    const uint32_t b = mo_bits(value);
    const uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    const uint32_t mag = b & 0x7fffffffu;
    if (mag >= 0x7f800000u) return (uint16_t)(sign | (mag > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (mag >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);       /* >= 65520 rounds to inf */
    if (mag < 0x33000000u) return sign;                              /* < 2^-25 rounds to 0 */
    const int e = (int)(mag >> 23) - 127;                            /* unbiased */
    uint32_t sig = (mag & 0x007fffffu) | 0x00800000u;                /* 24-bit significand */
    int drop = 13;                                                   /* bits to discard, normal case */
    int he = e + 15;
    if (he <= 0) { drop += 1 - he; he = 0; }                         /* subnormal half */
    uint32_t kept = sig >> drop;
    const uint32_t rem = sig & ((1u << drop) - 1u);
    const uint32_t halfway = 1u << (drop - 1);
    if (rem > halfway || (rem == halfway && (kept & 1u))) kept += 1u;
    /* kept carries the implicit bit for normals: (he<<10) + kept - 0x400 handles the carry into the exponent */
    const uint32_t out = he > 0 ? ((uint32_t)he << 10) + kept - 0x400u : kept;
    return (uint16_t)(sign | out);
}

int mo_f16_to_f32_array(const uint16_t *in, size_t n, float *out) {
    if (n == 0) return 1;
    if (!in || !out) return 0;
    for (size_t i = 0; i < n; ++i) out[i] = mo_f16_to_f32(in[i]);
    return 1;
}

int mo_f32_to_f16_array(const float *in, size_t n, uint16_t *out) {
    if (n == 0) return 1;
    if (!in || !out) return 0;
    for (size_t i = 0; i < n; ++i) out[i] = mo_f32_to_f16(in[i]);
    return 1;
}

/* ----------------------------------------------------------- dot chains */

static float mo_dot(const float *x, const float *w, uint32_t n) {
    float acc = 0.0f;
    for (uint32_t i = 0; i < n; ++i) acc = fmaf(x[i], w[i], acc);
    return acc;
}

/* `count` rows of w (row stride `ld`), one chain each, four chains in flight */
static void mo_dot_rows(const float *x, const float *w, size_t ld, uint32_t n, uint32_t count, float *out) {
    uint32_t r = 0;
    for (; r + 4u <= count; r += 4u) {
        const float *w0 = w + (size_t)r * ld, *w1 = w0 + ld, *w2 = w1 + ld, *w3 = w2 + ld;
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        for (uint32_t i = 0; i < n; ++i) {
            const float xi = x[i];
            a0 = fmaf(xi, w0[i], a0);
            a1 = fmaf(xi, w1[i], a1);
            a2 = fmaf(xi, w2[i], a2);
            a3 = fmaf(xi, w3[i], a3);
        }
        out[r] = a0; out[r + 1] = a1; out[r + 2] = a2; out[r + 3] = a3;
    }
    for (; r < count; ++r) out[r] = mo_dot(x, w + (size_t)r * ld, n);
}

static float mo_silu(float v) { return v / (1.0f + expf(-v)); }

static int mo_mul_ok(uint64_t a, uint64_t b, uint64_t c) {
    if (a == 0 || b == 0 || c == 0) return 1;
    if (a > UINT64_MAX / b) return 0;
    const uint64_t ab = a * b;
    if (ab > UINT64_MAX / c) return 0;
    return ab * c <= (uint64_t)SIZE_MAX;
}

/* ---------------------------------------------------------------- router */

static int mo_router_args_ok(const void *x, const void *w, uint32_t rows, uint32_t H, uint32_t E, uint32_t K,
                             float scaling, const void *logits, const void *probs, const void *ids,
                             const void *weights) {
    if (!x || !w || !logits || !probs || !ids || !weights) return 0;
    if (rows == 0u || H == 0u || E == 0u || K == 0u || K > E) return 0;
    if (!(scaling >= 0.0f) || !isfinite(scaling)) return 0;
    return mo_mul_ok(rows, E, 1) && mo_mul_ok(rows, K, 1) && mo_mul_ok(E, H, 1);
}

/* softmax + greedy top-k of one row whose logits are already in logits[] */
static int mo_route_row(const float *logits, uint32_t E, uint32_t K, float scaling, float *probs, uint32_t *ids,
                        float *weights) {
    float top = -INFINITY;
    for (uint32_t e = 0; e < E; ++e) if (logits[e] > top) top = logits[e];
    if (!isfinite(top)) return 0;
    float denom = 0.0f;
    for (uint32_t e = 0; e < E; ++e) {
        probs[e] = expf(logits[e] - top);
        denom += probs[e];
    }
    if (!(denom > 0.0f) || !isfinite(denom)) return 0;
    for (uint32_t e = 0; e < E; ++e) probs[e] /= denom;
    for (uint32_t slot = 0; slot < K; ++slot) {
        uint32_t pick = UINT32_MAX;
        float pick_p = -INFINITY;
        for (uint32_t e = 0; e < E; ++e) {
            int taken = 0;
            for (uint32_t s = 0; s < slot; ++s) taken |= (ids[s] == e);
            if (taken) continue;
            /* strictly greater wins; on equality the lower id (seen first) stays */
            if (probs[e] > pick_p || (probs[e] == pick_p && e < pick)) { pick = e; pick_p = probs[e]; }
        }
        if (pick == UINT32_MAX || !(pick_p >= 0.0f)) return 0;
        ids[slot] = pick;
        weights[slot] = pick_p * scaling;
    }
    return 1;
}

int mo_router_f32(const float *x, const float *w, uint32_t rows, uint32_t H, uint32_t E, uint32_t K, float scaling,
                  float *logits, float *probs, uint32_t *ids, float *weights) {
    if (!mo_router_args_ok(x, w, rows, H, E, K, scaling, logits, probs, ids, weights)) return 0;
    for (uint32_t r = 0; r < rows; ++r) {
        float *lr = logits + (size_t)r * E;
        mo_dot_rows(x + (size_t)r * H, w, H, H, E, lr);
        if (!mo_route_row(lr, E, K, scaling, probs + (size_t)r * E, ids + (size_t)r * K, weights + (size_t)r * K))
            return 0;
    }
    return 1;
}

/* Same softmax/top-k on logits supplied by the caller (the "identical gate
 * logits" form of the routing parity test). */
int mo_route_from_logits_f32(const float *logits, uint32_t rows, uint32_t E, uint32_t K, float scaling, float *probs,
                             uint32_t *ids, float *weights) {
    if (!logits || !probs || !ids || !weights || rows == 0u || E == 0u || K == 0u || K > E) return 0;
    if (!(scaling >= 0.0f) || !isfinite(scaling)) return 0;
    for (uint32_t r = 0; r < rows; ++r)
        if (!mo_route_row(logits + (size_t)r * E, E, K, scaling, probs + (size_t)r * E, ids + (size_t)r * K,
                          weights + (size_t)r * K))
            return 0;
    return 1;
}

/* ------------------------------------------------------------ RMSNorm */

/* uocr_cpu_ref_rmsnorm_f32 (src/backend/cpu_ref/uocr_cpu_ref.c:145-169): per row, sum of squares as one serial fmaf
 * chain, mean, 1 / sqrtf(mean + eps), out = x * inv_rms * weight (in that order). */
int mo_rmsnorm_f32(const float *x, const float *weight, uint32_t rows, uint32_t cols, float eps, float *out) {
    if (!x || !weight || !out || rows == 0u || cols == 0u || eps < 0.0f) return 0;
    for (uint32_t r = 0; r < rows; ++r) {
        const float *xr = x + (size_t)r * cols;
        float ss = 0.0f;
        for (uint32_t c = 0; c < cols; ++c) ss = fmaf(xr[c], xr[c], ss);
        const float inv = 1.0f / sqrtf(ss / (float)cols + eps);
        for (uint32_t c = 0; c < cols; ++c) out[(size_t)r * cols + c] = xr[c] * inv * weight[c];
    }
    return 1;
}

/* The GPU path's form of the same step (src/backend/metal/kernels/norm.metal:12-40): fp16 activations and weight,
 * f32 arithmetic, the result rounded to fp16 once. */
int mo_rmsnorm_f16(const uint16_t *x_f16, const uint16_t *weight_f16, uint32_t rows, uint32_t cols, float eps, uint16_t *out_f16) {
    if (!x_f16 || !weight_f16 || !out_f16 || rows == 0u || cols == 0u || eps < 0.0f) return 0;
    for (uint32_t r = 0; r < rows; ++r) {
        const uint16_t *xr = x_f16 + (size_t)r * cols;
        float ss = 0.0f;
        for (uint32_t c = 0; c < cols; ++c) { const float v = mo_f16_to_f32(xr[c]); ss = fmaf(v, v, ss); }
        const float inv = 1.0f / sqrtf(ss / (float)cols + eps);
        for (uint32_t c = 0; c < cols; ++c)
            out_f16[(size_t)r * cols + c] = mo_f32_to_f16(mo_f16_to_f32(xr[c]) * inv * mo_f16_to_f32(weight_f16[c]));
    }
    return 1;
}

/* ------------------------------------------------------------ dense MLP */

int mo_dense_swiglu_f32(const float *x, const float *gate, const float *up, const float *down, uint32_t rows,
                        uint32_t H, uint32_t F, float *mid, float *out) {
    if (!x || !gate || !up || !down || !mid || !out || rows == 0u || H == 0u || F == 0u) return 0;
    if (!mo_mul_ok(rows, H, 1) || !mo_mul_ok(rows, F, 1)) return 0;
    float *g = (float *)malloc(sizeof(float) * 2u * F);
    if (!g) return 0;
    float *u = g + F;
    for (uint32_t r = 0; r < rows; ++r) {
        const float *xr = x + (size_t)r * H;
        float *mr = mid + (size_t)r * F;
        mo_dot_rows(xr, gate, H, H, F, g);
        mo_dot_rows(xr, up, H, H, F, u);
        for (uint32_t i = 0; i < F; ++i) mr[i] = mo_silu(g[i]) * u[i];
        mo_dot_rows(mr, down, F, F, H, out + (size_t)r * H);
    }
    free(g);
    return 1;
}

/* ------------------------------------------------------- f32 MoE layer */

int mo_layer_f32(const float *x, const float *router_w, const float *e_gate, const float *e_up, const float *e_down,
                 const float *s_gate, const float *s_up, const float *s_down, uint32_t rows, uint32_t H, uint32_t E,
                 uint32_t K, uint32_t F, uint32_t S, float scaling, float *logits, float *probs, uint32_t *ids,
                 float *weights, float *expert_ws, float *shared_ws, float *out) {
    if (!e_gate || !e_up || !e_down || !s_gate || !s_up || !s_down || !expert_ws || !shared_ws || !out || F == 0u ||
        S == 0u)
        return 0;
    if (!mo_router_args_ok(x, router_w, rows, H, E, K, scaling, logits, probs, ids, weights)) return 0;
    if (!mo_mul_ok(E, F, H) || !mo_mul_ok(rows, K, F) || !mo_mul_ok(rows, S, 1) || !mo_mul_ok(S, H, 1)) return 0;
    if (!mo_router_f32(x, router_w, rows, H, E, K, scaling, logits, probs, ids, weights)) return 0;

    const uint32_t widest = F > S ? F : S;
    float *tmp = (float *)malloc(sizeof(float) * ((size_t)2u * widest + H));
    if (!tmp) return 0;
    float *g = tmp, *u = tmp + widest, *d = tmp + 2u * (size_t)widest;
    int ok = 1;
    for (uint32_t r = 0; r < rows && ok; ++r) {
        const float *xr = x + (size_t)r * H;
        float *orow = out + (size_t)r * H;
        for (uint32_t h = 0; h < H; ++h) orow[h] = 0.0f;
        for (uint32_t slot = 0; slot < K; ++slot) {
            const uint32_t e = ids[(size_t)r * K + slot];
            const float rw = weights[(size_t)r * K + slot];
            if (e >= E) { ok = 0; break; }
            float *mid = expert_ws + ((size_t)r * K + slot) * F;
            mo_dot_rows(xr, e_gate + (size_t)e * F * H, H, H, F, g);
            mo_dot_rows(xr, e_up + (size_t)e * F * H, H, H, F, u);
            for (uint32_t i = 0; i < F; ++i) mid[i] = mo_silu(g[i]) * u[i];
            mo_dot_rows(mid, e_down + (size_t)e * H * F, F, F, H, d);
            for (uint32_t h = 0; h < H; ++h) orow[h] = fmaf(rw, d[h], orow[h]);
        }
        if (!ok) break;
        float *smid = shared_ws + (size_t)r * S;
        mo_dot_rows(xr, s_gate, H, H, S, g);
        mo_dot_rows(xr, s_up, H, H, S, u);
        for (uint32_t i = 0; i < S; ++i) smid[i] = mo_silu(g[i]) * u[i];
        mo_dot_rows(smid, s_down, S, S, H, d);
        for (uint32_t h = 0; h < H; ++h) orow[h] += d[h];
    }
    free(tmp);
    return ok;
}

/* --------------------------------------------------- quantised matrices */

typedef struct mo_matrix {
    int32_t qtype;           /* MO_QTYPE_* */
    uint32_t rows, cols;
    const void *qweight;     /* f16: u16[rows][cols]; q8: i8[rows][cols]; q4: u8[rows][cols/2] */
    const uint16_t *qscale;  /* fp16 [rows][cols/64]; unused for f16 */
    int32_t through_f16;     /* != 0: each dequantised weight is rounded to fp16, the value the reference's tiled
                                GPU GEMMs feed their MMA (src/backend/metal/kernels/gemm_q4.metal:35-57) */
} mo_matrix;

static int mo_matrix_ok(const mo_matrix *m) {
    if (!m || !m->qweight || m->rows == 0u || m->cols == 0u) return 0;
    if (m->qtype == MO_QTYPE_F16) return 1;
    if (m->qtype != MO_QTYPE_Q8_0 && m->qtype != MO_QTYPE_Q4_0) return 0;
    return m->qscale != NULL && (m->cols % MO_GROUP) == 0u;
}

/* value = level * float(fp16 scale); dst gets `cols` floats of row `r` */
static void mo_dequant_row(const mo_matrix *m, uint32_t r, float *dst) {
    const uint32_t C = m->cols;
    if (m->qtype == MO_QTYPE_F16) {
        const uint16_t *src = (const uint16_t *)m->qweight + (size_t)r * C;
        for (uint32_t c = 0; c < C; ++c) dst[c] = mo_f16_to_f32(src[c]);
        return;
    }
    const uint16_t *sc = m->qscale + (size_t)r * (C / MO_GROUP);
    if (m->qtype == MO_QTYPE_Q8_0) {
        const int8_t *src = (const int8_t *)m->qweight + (size_t)r * C;
        for (uint32_t c = 0; c < C; ++c) dst[c] = (float)src[c] * mo_f16_to_f32(sc[c / MO_GROUP]);
        if (m->through_f16) for (uint32_t c = 0; c < C; ++c) dst[c] = mo_f16_to_f32(mo_f32_to_f16(dst[c]));
        return;
    }
    const uint8_t *src = (const uint8_t *)m->qweight + (size_t)r * (C / 2u);
    for (uint32_t g = 0; g < C / MO_GROUP; ++g) {
        const float s = mo_f16_to_f32(sc[g]);
        for (uint32_t j = 0; j < MO_GROUP / 2u; ++j) {
            const uint8_t byte = src[g * (MO_GROUP / 2u) + j];
            dst[g * MO_GROUP + j] = (float)((int)(byte & 15u) - 8) * s;
            dst[g * MO_GROUP + MO_GROUP / 2u + j] = (float)((int)(byte >> 4) - 8) * s;
        }
    }
    if (m->through_f16) for (uint32_t c = 0; c < C; ++c) dst[c] = mo_f16_to_f32(mo_f32_to_f16(dst[c]));
}

int mo_dequant_matrix(const mo_matrix *m, float *dst) {
    if (!mo_matrix_ok(m) || !dst) return 0;
    for (uint32_t r = 0; r < m->rows; ++r) mo_dequant_row(m, r, dst + (size_t)r * m->cols);
    return 1;
}

/* LM head: logits[t][v] = row v of the matrix . x[t] (fp16 activations, f32 fmaf chain over the dequantised row), and
 * per token the argmax with ties to the lowest id and NaN rows skipped: the contract of the reference's fused kernels
 * (src/backend/metal/kernels/lm_head_q4.metal:25-100: strict '>' over ascending rows, '!isnan(total)').  ids[t] is
 * 0xffffffff when every row is NaN.  logits_out (optional) receives all logits [rows][m->rows]. */
int mo_lm_head_argmax(const mo_matrix *m, const uint16_t *x_f16, uint32_t rows, uint32_t *ids, float *scores, float *logits_out) {
    if (!mo_matrix_ok(m) || !x_f16 || !ids || rows == 0u) return 0;
    const uint32_t C = m->cols, R = m->rows;
    float *w = (float *)malloc(sizeof(float) * C * 2u);
    if (!w) return 0;
    float *x = w + C;
    for (uint32_t t = 0; t < rows; ++t) { ids[t] = 0xffffffffu; if (scores) scores[t] = -INFINITY; }
    float *best = (float *)malloc(sizeof(float) * rows);
    if (!best) { free(w); return 0; }
    for (uint32_t r = 0; r < R; ++r) {
        mo_dequant_row(m, r, w);
        for (uint32_t t = 0; t < rows; ++t) {
            for (uint32_t c = 0; c < C; ++c) x[c] = mo_f16_to_f32(x_f16[(size_t)t * C + c]);
            const float v = mo_dot(x, w, C);
            if (logits_out) logits_out[(size_t)t * R + r] = v;
            if (v != v) continue;
            if (ids[t] == 0xffffffffu || v > best[t]) { best[t] = v; ids[t] = r; }
        }
    }
    if (scores) for (uint32_t t = 0; t < rows; ++t) if (ids[t] != 0xffffffffu) scores[t] = best[t];
    free(best);
    free(w);
    return 1;
}

/* y[rows x m->rows] = x[rows x m->cols] . m^T, each output one fmaf chain.
 * Weight rows are dequantised once (four at a time) and swept over all x rows. */
static void mo_matmul_nt(const mo_matrix *m, const float *x, uint32_t rows, float *y, float *scratch4) {
    const uint32_t C = m->cols, R = m->rows;
    for (uint32_t r0 = 0; r0 < R; r0 += 4u) {
        const uint32_t cnt = R - r0 < 4u ? R - r0 : 4u;
        for (uint32_t i = 0; i < cnt; ++i) mo_dequant_row(m, r0 + i, scratch4 + (size_t)i * C);
        for (uint32_t t = 0; t < rows; ++t) {
            float tmp[4];
            mo_dot_rows(x + (size_t)t * C, scratch4, C, C, cnt, tmp);
            for (uint32_t i = 0; i < cnt; ++i) y[(size_t)t * R + r0 + i] = tmp[i];
        }
    }
}

/* ------------------------------------------------- slab-format MoE layer */

typedef struct mo_layer_weights {
    uint32_t H, E, K, F, S;
    float scaling;
    const uint16_t *router_f16;   /* [E][H] fp16 */
    const float *logit_bias;      /* [E] or NULL: added to every row's logits (synthetic load skew only) */
    int32_t expert_qtype;
    const void *expert_qweight;   /* slab: expert e at e*expert_stride_bytes: gate[F][H], up[F][H], down[H][F] */
    const uint16_t *expert_qscale;/* slab: expert e at e*expert_scale_stride (values): gate, up, down scales */
    mo_matrix shared_gate, shared_up, shared_down;
} mo_layer_weights;

static size_t mo_packed_bytes(int32_t qtype, uint64_t rows, uint64_t cols) {
    if (qtype == MO_QTYPE_F16) return (size_t)(rows * cols * 2u);
    if (qtype == MO_QTYPE_Q8_0) return (size_t)(rows * cols);
    return (size_t)(rows * cols / 2u);
}

static void mo_expert_matrices(const mo_layer_weights *L, uint32_t e, mo_matrix *gate, mo_matrix *up,
                               mo_matrix *down) {
    const size_t proj_bytes = mo_packed_bytes(L->expert_qtype, L->F, L->H);
    const size_t proj_scales = L->expert_qtype == MO_QTYPE_F16 ? 0u : (size_t)L->F * (L->H / MO_GROUP);
    const uint8_t *qw = (const uint8_t *)L->expert_qweight + (size_t)e * 3u * proj_bytes;
    const uint16_t *qs = L->expert_qscale ? L->expert_qscale + (size_t)e * 3u * proj_scales : NULL;
    gate->qtype = up->qtype = down->qtype = L->expert_qtype;
    gate->through_f16 = up->through_f16 = down->through_f16 = L->shared_gate.through_f16;
    gate->rows = up->rows = L->F; gate->cols = up->cols = L->H;
    down->rows = L->H; down->cols = L->F;
    gate->qweight = qw; up->qweight = qw + proj_bytes; down->qweight = qw + 2u * proj_bytes;
    gate->qscale = qs; up->qscale = qs ? qs + proj_scales : NULL; down->qscale = qs ? qs + 2u * proj_scales : NULL;
}

/*
 * The layer on the model's own byte formats.  hidden is fp16; every weight is
 * turned into the f32 value the format defines and the arithmetic is then the
 * f32 layer above, so for any input
 *     mo_layer_slab(...) == mo_layer_f32(dequantised copies ...)   bit for bit.
 * injected_logits (rows x E, may be NULL) replaces the router dot products.
 * round_mid_f16 is a set of bits, each an fp16 rounding of the reference's GPU
 * or NumPy fp16 contracts; the reference CPU path itself keeps f32 everywhere
 * (round_mid_f16 = 0):
 *   1  the SwiGLU products, as the GPU kernels store `mid`
 *      (src/backend/metal/kernels/decode_gemv_q4.metal:176-179;
 *      src/unlimitedocr_c/golden.py:476-477, :624-625);
 *   2  every expert's down product, as the many-token GPU path stores it
 *      before the combine (src/backend/metal/kernels/gemm_q8.metal:867-919);
 *   4  the shared MLP's output (same GPU path; golden.py:481 with a zero
 *      residual, :640-648);
 *   8  the weighted sum of the routed experts before the shared output is
 *      added (golden.py:627-628, :663-665).
 * 1|2|4 is the tiled-GEMM contract, 1|4|8 the NumPy fp16 contract.
 * residual (fp16, may be NULL) is added to the f32 result at the end, the place
 * the GPU layer adds it (src/backend/metal/kernels/decode_gemv_q4.metal:221-223).
 * The experts are walked expert-major (each distinct expert is dequantised once
 * per call); per output element the accumulation order is still slot order.
 */
int mo_layer_slab(const mo_layer_weights *L, const uint16_t *hidden_f16, const uint16_t *residual_f16,
                  const float *injected_logits, uint32_t rows, int round_mid_f16, float *logits, float *probs,
                  uint32_t *ids, float *weights, float *expert_ws, float *shared_ws, float *out) {
    if (!L || !hidden_f16 || !logits || !probs || !ids || !weights || !expert_ws || !shared_ws || !out) return 0;
    const uint32_t H = L->H, E = L->E, K = L->K, F = L->F, S = L->S;
    if (rows == 0u || H == 0u || E == 0u || K == 0u || K > E || F == 0u || S == 0u) return 0;
    if (!(L->scaling >= 0.0f) || !isfinite(L->scaling) || !L->router_f16 || !L->expert_qweight) return 0;
    if (L->expert_qtype != MO_QTYPE_F16 && (!L->expert_qscale || H % MO_GROUP || F % MO_GROUP)) return 0;
    if (!mo_matrix_ok(&L->shared_gate) || !mo_matrix_ok(&L->shared_up) || !mo_matrix_ok(&L->shared_down)) return 0;

    const uint32_t widest = F > S ? F : S;
    const uint32_t longest = H > widest ? H : widest;
    float *x = (float *)malloc(sizeof(float) * (size_t)rows * H);
    float *rw = (float *)malloc(sizeof(float) * (size_t)E * H);
    float *scratch4 = (float *)malloc(sizeof(float) * 4u * (size_t)longest);
    float *g = (float *)malloc(sizeof(float) * ((size_t)rows * widest * 2u + (size_t)rows * H));
    float *down_all = (float *)malloc(sizeof(float) * (size_t)rows * K * H);
    int ok = x && rw && scratch4 && g && down_all;
    if (ok) {
        float *u = g + (size_t)rows * widest, *d = u + (size_t)rows * widest;
        mo_f16_to_f32_array(hidden_f16, (size_t)rows * H, x);
        mo_f16_to_f32_array(L->router_f16, (size_t)E * H, rw);
        for (uint32_t r = 0; r < rows && ok; ++r) {
            float *lr = logits + (size_t)r * E;
            if (injected_logits) memcpy(lr, injected_logits + (size_t)r * E, sizeof(float) * E);
            else mo_dot_rows(x + (size_t)r * H, rw, H, H, E, lr);
            if (L->logit_bias) for (uint32_t e = 0; e < E; ++e) lr[e] += L->logit_bias[e];
            ok = mo_route_row(lr, E, K, L->scaling, probs + (size_t)r * E, ids + (size_t)r * K,
                              weights + (size_t)r * K);
        }
        /* routed experts, expert-major; down products parked per (row, slot) */
        float *xs = (float *)malloc(sizeof(float) * (size_t)rows * longest);
        uint32_t *where = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)rows);
        ok = ok && xs && where;
        for (uint32_t e = 0; e < E && ok; ++e) {
            uint32_t cnt = 0;
            for (uint32_t r = 0; r < rows; ++r)
                for (uint32_t s = 0; s < K; ++s)
                    if (ids[(size_t)r * K + s] == e) where[cnt++] = r * K + s;
            if (cnt == 0u) continue;
            mo_matrix mg, mu, md;
            mo_expert_matrices(L, e, &mg, &mu, &md);
            for (uint32_t i = 0; i < cnt; ++i) memcpy(xs + (size_t)i * H, x + (size_t)(where[i] / K) * H, sizeof(float) * H);
            mo_matmul_nt(&mg, xs, cnt, g, scratch4);
            mo_matmul_nt(&mu, xs, cnt, u, scratch4);
            for (uint32_t i = 0; i < cnt; ++i) {
                float *mid = expert_ws + (size_t)where[i] * F;
                for (uint32_t c = 0; c < F; ++c) {
                    float v = mo_silu(g[(size_t)i * F + c]) * u[(size_t)i * F + c];
                    if (round_mid_f16 & 1) v = mo_f16_to_f32(mo_f32_to_f16(v));
                    mid[c] = v;
                }
                memcpy(xs + (size_t)i * F, mid, sizeof(float) * F);
            }
            mo_matmul_nt(&md, xs, cnt, d, scratch4);
            if (round_mid_f16 & 2) for (size_t i = 0; i < (size_t)cnt * H; ++i) d[i] = mo_f16_to_f32(mo_f32_to_f16(d[i]));
            for (uint32_t i = 0; i < cnt; ++i) memcpy(down_all + (size_t)where[i] * H, d + (size_t)i * H, sizeof(float) * H);
        }
        if (ok) {
            /* shared MLP for every row */
            mo_matmul_nt(&L->shared_gate, x, rows, g, scratch4);
            mo_matmul_nt(&L->shared_up, x, rows, u, scratch4);
            for (size_t i = 0; i < (size_t)rows * S; ++i) {
                float v = mo_silu(g[i]) * u[i];
                if (round_mid_f16 & 1) v = mo_f16_to_f32(mo_f32_to_f16(v));
                shared_ws[i] = v;
            }
            mo_matmul_nt(&L->shared_down, shared_ws, rows, d, scratch4);
            if (round_mid_f16 & 4) for (size_t i = 0; i < (size_t)rows * H; ++i) d[i] = mo_f16_to_f32(mo_f32_to_f16(d[i]));
            for (uint32_t r = 0; r < rows; ++r) {
                float *orow = out + (size_t)r * H;
                for (uint32_t h = 0; h < H; ++h) orow[h] = 0.0f;
                for (uint32_t s = 0; s < K; ++s) {
                    const float w = weights[(size_t)r * K + s];
                    const float *dn = down_all + ((size_t)r * K + s) * H;
                    for (uint32_t h = 0; h < H; ++h) orow[h] = fmaf(w, dn[h], orow[h]);
                }
                if (round_mid_f16 & 8) for (uint32_t h = 0; h < H; ++h) orow[h] = mo_f16_to_f32(mo_f32_to_f16(orow[h]));
                for (uint32_t h = 0; h < H; ++h) orow[h] += d[(size_t)r * H + h];
                if (residual_f16)
                    for (uint32_t h = 0; h < H; ++h) orow[h] += mo_f16_to_f32(residual_f16[(size_t)r * H + h]);
            }
        }
        free(xs); free(where);
    }
    free(x); free(rw); free(scratch4); free(g); free(down_all);
    return ok;
}

/* --------------------------------------------------------- dispatch plan */

/*
 * Token-to-expert permutation: pair = token*K + slot, grouped by expert id,
 * ascending pair order inside a group (a stable counting sort).  This is the
 * deterministic refinement of the reference's bucketing pass, whose in-bucket
 * order is left to atomics (src/backend/metal/kernels/gemm_q8.metal:462-511):
 * expert_offsets is the exclusive prefix sum of the per-expert pair counts and
 * ids >= E are dropped.  inverse[pair] is the pair's position in pair_rows, or
 * 0xffffffff for a dropped pair.
 */
int mo_dispatch_plan(const uint32_t *ids, uint32_t rows, uint32_t K, uint32_t E, uint32_t *expert_offsets,
                     uint32_t *pair_rows, uint32_t *inverse) {
    if (!ids || !expert_offsets || !pair_rows || !inverse || E == 0u || K == 0u) return 0;
    const size_t pairs = (size_t)rows * K;
    for (uint32_t e = 0; e <= E; ++e) expert_offsets[e] = 0u;
    for (size_t p = 0; p < pairs; ++p) if (ids[p] < E) expert_offsets[ids[p] + 1u] += 1u;
    for (uint32_t e = 0; e < E; ++e) expert_offsets[e + 1u] += expert_offsets[e];
    uint32_t *cursor = (uint32_t *)malloc(sizeof(uint32_t) * E);
    if (!cursor) return 0;
    memcpy(cursor, expert_offsets, sizeof(uint32_t) * E);
    for (size_t p = 0; p < pairs; ++p) {
        if (ids[p] < E) {
            const uint32_t pos = cursor[ids[p]]++;
            pair_rows[pos] = (uint32_t)p;
            inverse[p] = pos;
        } else {
            inverse[p] = UINT32_MAX;
        }
    }
    free(cursor);
    return 1;
}

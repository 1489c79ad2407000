/*
 * expf() with the same result bits as the host C library the reference's CPU router runs on.
 *
 * The router's expert ids depend on f32 softmax probabilities
 * (src/backend/cpu_ref/uocr_cpu_ref.c:430-463), so bit-exact routing needs the same exp().
 * glibc >= 2.27 computes expf with the table-driven algorithm of Szabolcs Nagy's
 * "optimized-routines" (sysdeps/ieee754/flt-32/e_expf.c): in double precision
 *     z = x * (N/ln2);  k = round(z);  r = z - k;            N = 32
 *     exp(x) = 2^(k/N) * (C0 r^3 + C1 r^2 + C2 r + 1)
 * with 2^(i/N) from a 32-entry table and the 2^(k/N - i/N) factor applied by adding k to the
 * exponent bits.  Every step is an IEEE double operation, so the same sequence on the GPU
 * (explicit fma/mul/add, no contraction left to the compiler) gives the same float.
 * The remainder r = x*(N/ln2) - k and the three polynomial steps are fused multiply-adds, which is
 * how the FMA build of glibc (the one x86-64 hosts with AVX2+FMA select at load time) evaluates
 * them.  With exactly this choice the function agrees with glibc 2.39's expf on every one of the
 * 3.26e9 non-NaN floats below 89 (checked exhaustively); with the unfused remainder two inputs
 * differ by one ulp, which is the most a host without FMA could differ.
 *
 * tests/test_expf_compat.py checks this file against the host's expf over the router's whole
 * input range.  Usable from C, C++ and CUDA.
 */
#ifndef UOCR_EXPF_COMPAT_H
#define UOCR_EXPF_COMPAT_H

#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef __CUDACC__
#  define UOCR_HD __host__ __device__ __forceinline__
#else
#  define UOCR_HD static inline
#endif

#define UOCR_EXPF_TABLE_BITS 5
#define UOCR_EXPF_N 32

/* tab[i] = bits(2^(i/N)) - (i << (52 - TABLE_BITS)); host only, run once at start-up. */
static inline void uocr_expf_table_init(uint64_t tab[UOCR_EXPF_N]) {
    for (int i = 0; i < UOCR_EXPF_N; ++i) {
        const double v = (double)exp2l((long double)i / (long double)UOCR_EXPF_N);
        uint64_t bits;
        memcpy(&bits, &v, sizeof bits);
        tab[i] = bits - ((uint64_t)i << (52 - UOCR_EXPF_TABLE_BITS));
    }
}

UOCR_HD float uocr_expf_compat(float x, const uint64_t *tab) {
    const double kInvLn2N = 0x1.71547652b82fep+0 * UOCR_EXPF_N;
    const double kShift = 0x1.8p+52;
    const double kC0 = 0x1.c6af84b912394p-5 / UOCR_EXPF_N / UOCR_EXPF_N / UOCR_EXPF_N;
    const double kC1 = 0x1.ebfce50fac4f3p-3 / UOCR_EXPF_N / UOCR_EXPF_N;
    const double kC2 = 0x1.62e42ff0c52d6p-1 / UOCR_EXPF_N;
    if (x != x) return x;
    if (x > 0x1.62e42ep6f) return INFINITY;        /* overflow threshold of the library routine */
    if (x < -0x1.9fe368p6f) return 0.0f;           /* underflow threshold: below the smallest subnormal */
    const double xd = (double)x;
#ifdef __CUDA_ARCH__
    const double z = __dmul_rn(kInvLn2N, xd);
    double kd = __dadd_rn(z, kShift);
    const uint64_t ki = (uint64_t)__double_as_longlong(kd);
    kd = __dadd_rn(kd, -kShift);
    const double r = __fma_rn(kInvLn2N, xd, -kd);
    const uint64_t t = tab[ki & (UOCR_EXPF_N - 1)] + (ki << (52 - UOCR_EXPF_TABLE_BITS));
    const double s = __longlong_as_double((long long)t);
    const double p = __fma_rn(kC0, r, kC1);
    const double r2 = __dmul_rn(r, r);
    double y = __fma_rn(kC2, r, 1.0);
    y = __fma_rn(p, r2, y);
    y = __dmul_rn(y, s);
    return __double2float_rn(y);
#else
    const double z = kInvLn2N * xd;
    volatile double kdv = z + kShift;              /* keep the add in double, as the library does */
    double kd = kdv;
    uint64_t ki;
    memcpy(&ki, &kd, sizeof ki);
    kd -= kShift;
    const double r = fma(kInvLn2N, xd, -kd);
    const uint64_t t = tab[ki & (UOCR_EXPF_N - 1)] + (ki << (52 - UOCR_EXPF_TABLE_BITS));
    double s;
    memcpy(&s, &t, sizeof s);
    const double p = fma(kC0, r, kC1);
    const double r2 = r * r;
    double y = fma(kC2, r, 1.0);
    y = fma(p, r2, y);
    y = y * s;
    return (float)y;
#endif
}

#endif /* UOCR_EXPF_COMPAT_H */

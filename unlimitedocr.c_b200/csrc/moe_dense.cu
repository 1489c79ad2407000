// The steps either side of the MoE layer: the RMSNorm that feeds it and the residual add of the dense MLP's tensor-core path.
#include "moe_common.cuh"

namespace uocr {

// out[r][c] = fp16( x[r][c] * 1/sqrt(mean(x[r]^2) + eps) * w[c] ), f32 arithmetic: uocr_cpu_ref_rmsnorm_f32
// (src/backend/cpu_ref/uocr_cpu_ref.c:145-169) in the GPU path's form (fp16 in and out, one rounding:
// src/backend/metal/kernels/norm.metal:12-40).  One CTA of 128 threads per row; the sum of squares is a tree sum
// (the CPU's is one serial chain), so the scale can differ from the CPU's in its last bit.
constexpr int kNormThreads = 128;

__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(const __half *__restrict__ x, const __half *__restrict__ w, uint32_t cols,
                                                               float eps, __half *__restrict__ out) {
    __shared__ float partial[kNormThreads / 32];
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const __half2 *xr = reinterpret_cast<const __half2 *>(x + (size_t)row * cols);
    float ss = 0.f;
    for (uint32_t i = tid; i < cols / 2; i += kNormThreads) {
        const float2 v = __half22float2(xr[i]);
        ss = fmaf(v.x, v.x, ss);
        ss = fmaf(v.y, v.y, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) partial[tid >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) total += partial[i];
    const float inv = 1.0f / sqrtf(total / (float)cols + eps);
    const __half2 *wr = reinterpret_cast<const __half2 *>(w);
    __half2 *orow = reinterpret_cast<__half2 *>(out + (size_t)row * cols);
    for (uint32_t i = tid; i < cols / 2; i += kNormThreads) {
        const float2 v = __half22float2(xr[i]), g = __half22float2(wr[i]);
        orow[i] = __floats2half2_rn(v.x * inv * g.x, v.y * inv * g.y);
    }
}

cudaError_t launch_rmsnorm(const __half *x, const __half *w, uint32_t rows, uint32_t cols, float eps, __half *out, cudaStream_t st,
                           uint64_t *launches) {
    if (rows == 0 || cols == 0 || cols % 2) return cudaErrorInvalidValue;
    rmsnorm_kernel<<<rows, kNormThreads, 0, st>>>(x, w, cols, eps, out);
    ++*launches;
    return cudaGetLastError();
}

// out = fp16( a + residual ) on fp16 rows, eight values per thread
__global__ void add_rows_kernel(const __half *__restrict__ a, const __half *__restrict__ residual, size_t vec8, __half *__restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= vec8) return;
    uint4 va = reinterpret_cast<const uint4 *>(a)[i];
    if (residual) {
        const uint4 vr = reinterpret_cast<const uint4 *>(residual)[i];
        __half2 *pa = reinterpret_cast<__half2 *>(&va);
        const __half2 *pr = reinterpret_cast<const __half2 *>(&vr);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 x = __half22float2(pa[k]), y = __half22float2(pr[k]);
            pa[k] = __floats2half2_rn(x.x + y.x, x.y + y.y);
        }
    }
    reinterpret_cast<uint4 *>(out)[i] = va;
}

cudaError_t launch_add_rows(const __half *a, const __half *residual, size_t count, __half *out, cudaStream_t st, uint64_t *launches) {
    if (count % 8) return cudaErrorInvalidValue;
    const size_t vec8 = count / 8;
    add_rows_kernel<<<(unsigned)((vec8 + 255) / 256), 256, 0, st>>>(a, residual, vec8, out);
    ++*launches;
    return cudaGetLastError();
}

}  // namespace uocr

// Element-wise glue of a decoder-layer decode step (RMS norm, SiLU*mul, residual add), fused
// so that the step between two packed GEMVs is one small launch instead of a chain of
// framework kernels.  The reference leaves these to PyTorch (tests/harness_batchsweep.py:
// 230-243: rmsnorm, SiLU*mul, residual adds); they are not part of its operator surface.
#include "msaq_common.cuh"
#include "sm100_ptx.cuh"

namespace msaq {
namespace {

// out[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps), fp32 math, bf16 in/out.  One CTA per row.
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int n, float eps) {
    chain_release();
    chain_wait();
    __shared__ float red[8];
    const __nv_bfloat16* xr = x + (int64_t)blockIdx.x * n;
    __nv_bfloat16* orow = out + (int64_t)blockIdx.x * n;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += 256) { const float v = __bfloat162float(xr[i]); ss = fmaf(v, v, ss); }
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    const float r = rsqrtf(tot / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += 256) orow[i] = __float2bfloat16_rn(__bfloat162float(xr[i]) * r);
}

// out[r,j] = silu(gu[r,j]) * gu[r,F+j]
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int64_t rows, int F) {
    chain_release();
    chain_wait();
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= rows * F) return;
    const int64_t r = i / F, j = i % F;
    const float g = __bfloat162float(gu[r * 2 * F + j]), u = __bfloat162float(gu[r * 2 * F + F + j]);
    out[i] = __float2bfloat16_rn(g / (1.0f + __expf(-g)) * u);
}

// out = bf16(h + d), d in fp32 or bf16
template <typename T>
__global__ void __launch_bounds__(256)
add_residual_kernel(const __nv_bfloat16* __restrict__ h, const T* __restrict__ d, __nv_bfloat16* __restrict__ out, int64_t n) {
    chain_release();
    chain_wait();
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    out[i] = __float2bfloat16_rn(__bfloat162float(h[i]) + (float)d[i]);
}

// out[b,h,:] = RoPE(x[b,h,:]) at the position of sequence b; one thread per rotary pair.
__global__ void __launch_bounds__(256)
rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int64_t pairs, int heads, int half,
            Rope r, int64_t pos, const int32_t* __restrict__ pos_per_seq) {
    chain_release();
    chain_wait();
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= pairs) return;
    const int j = (int)(i % half);
    const int64_t b = i / half / heads;
    int64_t p = pos_per_seq ? pos_per_seq[b] : pos;
    p = r.rows == 1 ? 0 : min(max(p, (int64_t)0), r.rows - 1);
    float o1, o2;
    rope_pair(__bfloat162float(x[2 * i]), __bfloat162float(x[2 * i + 1]), r.cos[p * half + j], r.sin[p * half + j], &o1, &o2);
    out[2 * i] = __float2bfloat16_rn(o1);
    out[2 * i + 1] = __float2bfloat16_rn(o2);
}

}  // namespace
}  // namespace msaq

using namespace msaq;

extern "C" int msaq_rope(const void* x, void* out, int64_t B, int64_t heads, int64_t D, const float* rope_cos,
                         const float* rope_sin, int64_t rope_rows, int64_t pos, const int32_t* pos_per_seq,
                         void* stream) {
    if (!x || !out || !rope_cos || !rope_sin) return fail(MSAQ_ERR_ARG, "rope: null pointer");
    if (B <= 0 || heads <= 0 || D <= 0 || (D & 1) || heads > INT32_MAX || D > INT32_MAX || rope_rows < 1)
        return fail(MSAQ_ERR_ARG, "rope: bad size");
    if (!pos_per_seq && rope_rows != 1 && (pos < 0 || pos >= rope_rows))
        return fail(MSAQ_ERR_ARG, "rope: position %lld outside the %lld table rows", (long long)pos, (long long)rope_rows);
    const int64_t pairs = B * heads * (D / 2);
    launch_chained(rope_kernel, dim3((unsigned)((pairs + 255) / 256)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                   static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), pairs, (int)heads, (int)(D / 2),
                   Rope{rope_cos, rope_sin, rope_rows}, pos, pos_per_seq);
    count_launch();
    return check_launch("rope");
}

extern "C" int msaq_rmsnorm(const void* x, void* out, int64_t rows, int64_t n, float eps, void* stream) {
    if (!x || !out || rows <= 0 || n <= 0 || n > INT32_MAX) return fail(MSAQ_ERR_ARG, "rmsnorm: bad argument");
    launch_chained(rmsnorm_kernel, dim3((unsigned)rows), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), (int)n, eps);
    count_launch();
    return check_launch("rmsnorm");
}

extern "C" int msaq_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t F, void* stream) {
    if (!gate_up || !out || rows <= 0 || F <= 0 || F > INT32_MAX) return fail(MSAQ_ERR_ARG, "silu_mul: bad argument");
    const int64_t n = rows * F;
    launch_chained(silu_mul_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), rows, (int)F);
    count_launch();
    return check_launch("silu_mul");
}

extern "C" int msaq_add_residual(const void* h, const void* delta, int delta_is_f32, void* out, int64_t n, void* stream) {
    if (!h || !delta || !out || n <= 0) return fail(MSAQ_ERR_ARG, "add_residual: bad argument");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = (unsigned)((n + 255) / 256);
    if (delta_is_f32)
        launch_chained(add_residual_kernel<float>, dim3(grid), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(h), static_cast<const float*>(delta),
                                                        static_cast<__nv_bfloat16*>(out), n);
    else
        launch_chained(add_residual_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(h),
                                                                 static_cast<const __nv_bfloat16*>(delta),
                                                                 static_cast<__nv_bfloat16*>(out), n);
    count_launch();
    return check_launch("add_residual");
}

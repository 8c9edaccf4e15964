// Generic weight-only GEMV: any u in {2,3,4}, any gs, any OUT, row- or
// column-major planes, M rows of activations in tiles of MR <= 8.
//
// One thread owns one output column; the K axis is cut into `splits` ranges
// (grid.y) whose fp32 partial sums a second kernel adds up.  This is the
// always-correct path; the tuned kernels in gemv_mma.cuh take over for the
// shapes they cover.  Behaviour replaced: csrc/w_gemv.cu:52-92 and :173-349.
#pragma once

#include "msaq_common.cuh"
#include "sm100_ptx.cuh"

namespace msaq {

constexpr int GEMV_COLS = 128;      // columns (threads) per CTA
constexpr int GEMV_XCHUNK = 8;      // K blocks of activations staged per step

// Dot of one packed block against MR activation rows.  `uw` holds the UB bytes
// as little-endian words (one spare word readable), `sw` the SB bytes.
template <int U, int MR>
__device__ __forceinline__ void block_dot(const uint32_t* uw, const uint32_t* sw, int lg_gs,
                                          const float* xs /*[MR][32]*/, float* dot /*[MR]*/) {
    constexpr int WB = 8 - U;
#pragma unroll
    for (int m = 0; m < MR; ++m) dot[m] = 0.0f;
    const unsigned long long s64 = ((unsigned long long)sw[1] << 32) | sw[0];
#pragma unroll
    for (int k = 0; k < BLOCK; ++k) {
        const int bit = k * WB, wi = bit >> 5, off = bit & 31;
        uint32_t v = uw[wi] >> off;
        if (off + WB > 32) v |= uw[wi + 1] << (32 - off);
        const int up = sext(v, WB);
        const int g = k >> lg_gs;
        const int sh = sext((uint32_t)(s64 >> (g * U)), U);
        const float q = (float)(up * (1 << U) + sh);
#pragma unroll
        for (int m = 0; m < MR; ++m) dot[m] = fmaf(q, xs[m * BLOCK + k], dot[m]);
    }
}

template <int U, bool CM, int MR>
__global__ void __launch_bounds__(GEMV_COLS)
gemv_generic_kernel(const __nv_bfloat16* __restrict__ X, const int8_t* __restrict__ scale_exp,
                    const uint8_t* __restrict__ upper, const uint8_t* __restrict__ shared,
                    float* __restrict__ partial, int M, int OUT, int NB, int lg_gs, int UB, int SB,
                    int blocks_per_split) {
    chain_wait();
    __shared__ float xs[GEMV_XCHUNK][MR][BLOCK];
    const int o = blockIdx.x * GEMV_COLS + threadIdx.x;
    const int m0 = blockIdx.z * MR;
    const int b0 = blockIdx.y * blocks_per_split, b1 = min(NB, b0 + blocks_per_split);
    const int K = NB * BLOCK;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.0f;

    for (int c0 = b0; c0 < b1; c0 += GEMV_XCHUNK) {
        const int nc = min(GEMV_XCHUNK, b1 - c0);
        __syncthreads();
        for (int i = threadIdx.x; i < nc * MR * BLOCK; i += GEMV_COLS) {
            const int k = i % BLOCK, m = (i / BLOCK) % MR, c = i / (BLOCK * MR);
            const int row = m0 + m;
            xs[c][m][k] = row < M ? __bfloat162float(X[(int64_t)row * K + (c0 + c) * BLOCK + k]) : 0.0f;
        }
        __syncthreads();
        if (o < OUT) {
            for (int c = 0; c < nc; ++c) {
                const int blk = c0 + c;
                uint32_t uw[7], sw[2] = {0u, 0u};
                uw[6] = 0u;
                if (CM) {
                    const uint32_t* src = reinterpret_cast<const uint32_t*>(upper + ((int64_t)blk * OUT + o) * UB);
#pragma unroll
                    for (int i = 0; i < 6; ++i) uw[i] = (i * 4 < UB) ? src[i] : 0u;
                    const uint8_t* ss = shared + ((int64_t)blk * OUT + o) * SB;
                    for (int i = 0; i < SB; ++i) sw[i >> 2] |= (uint32_t)ss[i] << ((i & 3) * 8);
                } else {
#pragma unroll
                    for (int i = 0; i < 6; ++i) uw[i] = 0u;
                    for (int i = 0; i < UB; ++i)
                        uw[i >> 2] |= (uint32_t)upper[((int64_t)blk * UB + i) * OUT + o] << ((i & 3) * 8);
                    for (int i = 0; i < SB; ++i)
                        sw[i >> 2] |= (uint32_t)shared[((int64_t)blk * SB + i) * OUT + o] << ((i & 3) * 8);
                }
                const float sc = exp2_int((int)scale_exp[(int64_t)blk * OUT + o]);
                float dot[MR];
                block_dot<U, MR>(uw, sw, lg_gs, &xs[c][0][0], dot);
#pragma unroll
                for (int m = 0; m < MR; ++m) acc[m] = fmaf(dot[m], sc, acc[m]);
            }
        }
    }
    if (o < OUT) {
#pragma unroll
        for (int m = 0; m < MR; ++m)
            if (m0 + m < M) partial[((int64_t)blockIdx.y * M + (m0 + m)) * OUT + o] = acc[m];
    }
}

// y[i] = sum over splits of partial[s][i]; writes bf16 and, if asked, fp32.
__global__ void __launch_bounds__(256)
splitk_combine_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ y,
                      float* __restrict__ y_f32, int64_t n, int splits) {
    chain_release();
    chain_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.0f;
    for (int k = 0; k < splits; ++k) s += partial[(int64_t)k * n + i];
    y[i] = __float2bfloat16_rn(s);
    if (y_f32) y_f32[i] = s;
}

}  // namespace msaq

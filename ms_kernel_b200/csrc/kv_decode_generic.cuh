// Generic split-KV flash-decode: any u, gs, D in {32,64,128,256}, MHA or GQA,
// optional per-sequence lengths and in-prologue query rotation.
//
// One CTA = (query head, key tile, sequence).  Per 128-key chunk: thread-per-key
// scores, a block-wide running max, thread-per-channel P.V.  Each CTA leaves an
// un-normalised partial (acc[D], m, l); the combine kernel merges the tiles.
// This is the always-correct path behind the tuned kernel in kv_decode_mma.cuh.
// Behaviour replaced: csrc/kv_attention.cu:450-829 and :1220-1244.
#pragma once

#include "msaq_common.cuh"
#include "sm100_ptx.cuh"

namespace msaq {

constexpr int KVG_THREADS = 128;
constexpr int KVG_CHUNK = 128;

struct KvPlanes {
    const int8_t* s;
    const uint8_t* u;
    const uint8_t* h;
};

// Partial layout per (b, head, tile): D floats of acc, then m, then l.
__host__ __device__ inline int64_t kv_partial_stride(int D) { return D + 2; }

template <int U>
__device__ __forceinline__ float kv_block_dot(const uint8_t* up_bytes, const uint8_t* sh_bytes, int UB, int SB,
                                              int lg_gs, const float* qv) {
    constexpr int WB = 8 - U;
    uint32_t uw[7], sw[2] = {0u, 0u};
    const uint32_t* src = reinterpret_cast<const uint32_t*>(up_bytes);
#pragma unroll
    for (int i = 0; i < 6; ++i) uw[i] = (i * 4 < UB) ? src[i] : 0u;
    uw[6] = 0u;
    for (int i = 0; i < SB; ++i) sw[i >> 2] |= (uint32_t)sh_bytes[i] << ((i & 3) * 8);
    const unsigned long long s64 = ((unsigned long long)sw[1] << 32) | sw[0];
    float dot = 0.0f;
#pragma unroll
    for (int k = 0; k < BLOCK; ++k) {
        const int bit = k * WB, wi = bit >> 5, off = bit & 31;
        uint32_t v = uw[wi] >> off;
        if (off + WB > 32) v |= uw[wi + 1] << (32 - off);
        const int up = sext(v, WB);
        const int sh = sext((uint32_t)(s64 >> ((k >> lg_gs) * U)), U);
        dot = fmaf((float)(up * (1 << U) + sh), qv[k], dot);
    }
    return dot;
}

// One dequantised element (block-local index k) of the record at `slot`.
__device__ __forceinline__ float kv_element(const KvPlanes& p, int64_t slot, int k, const Fmt& f) {
    const uint8_t* ub = p.u + slot * f.UB;
    const int bit = k * f.wbits, by = bit >> 3, off = bit & 7;
    uint32_t v = ub[by] >> off;
    if (off + f.wbits > 8) v |= (uint32_t)ub[by + 1] << (8 - off);
    const int up = sext(v, f.wbits);
    const uint8_t* sb = p.h + slot * f.SB;
    const int sbit = (k >> f.lg_gs) * f.u, sby = sbit >> 3, soff = sbit & 7;
    uint32_t w = sb[sby] >> soff;
    if (soff + f.u > 8) w |= (uint32_t)sb[sby + 1] << (8 - soff);
    const int sh = sext(w, f.u);
    return (float)(up * (1 << f.u) + sh) * exp2_int((int)p.s[slot]);
}

template <int U>
__global__ void __launch_bounds__(KVG_THREADS)
kv_decode_generic_kernel(const __nv_bfloat16* __restrict__ q, KvPlanes kp, KvPlanes vp,
                         float* __restrict__ partial, const int32_t* __restrict__ seq_lens,
                         int H, int Hkv, int Lk, int Lcap, int D, int NB, Fmt f, int key_tile, int S,
                         float sm_scale, int qrot, Rope rope, int64_t q_pos, const int32_t* __restrict__ q_pos_per_seq) {
    chain_wait();
    extern __shared__ float smem[];
    float* q_sh = smem;                    // [D]
    float* sc = smem + D;                  // [KVG_CHUNK]
    __shared__ float red[KVG_THREADS / 32];
    const int h = blockIdx.x, s = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    const int hk = h / (H / Hkv);
    const int len = seq_lens ? min(seq_lens[b], Lk) : Lk;
    const int64_t head_base = ((int64_t)b * Hkv + hk) * NB;       // in units of Lcap slots

    if (rope.cos) {
        // the query's rotary embedding at its own position (the slot the step's new token went to)
        int64_t p = q_pos_per_seq ? q_pos_per_seq[b] : q_pos;
        p = rope.rows == 1 ? 0 : min(max(p, (int64_t)0), rope.rows - 1);
        const __nv_bfloat16* qr = q + ((int64_t)b * H + h) * D;
        for (int d = tid; d < D; d += KVG_THREADS) {
            const int j = d >> 1;
            float o1, o2;
            rope_pair(__bfloat162float(qr[d & ~1]), __bfloat162float(qr[d | 1]), rope.cos[p * (D / 2) + j],
                      rope.sin[p * (D / 2) + j], &o1, &o2);
            q_sh[d] = (d & 1) ? o2 : o1;
        }
    } else {
        for (int d = tid; d < D; d += KVG_THREADS) q_sh[d] = __bfloat162float(q[((int64_t)b * H + h) * D + d]);
    }
    __syncthreads();
    if (qrot) {
        for (int hh = 1; hh < D; hh <<= 1) {
            float nv[2];
            for (int i = 0, d = tid; d < D; d += KVG_THREADS, ++i) {
                const float ve = q_sh[d], vo = q_sh[d ^ hh];
                nv[i] = (d & hh) ? (vo - ve) : (ve + vo);
            }
            __syncthreads();
            for (int i = 0, d = tid; d < D; d += KVG_THREADS, ++i) q_sh[d] = nv[i];
            __syncthreads();
        }
        const float inv = (float)(1.0 / sqrt((double)D));
        for (int d = tid; d < D; d += KVG_THREADS) q_sh[d] *= inv;
        __syncthreads();
    }

    const int j0 = s * key_tile, j1 = min(j0 + key_tile, len);
    float m_i = -INFINITY, l_i = 0.0f;
    float acc[2] = {0.0f, 0.0f};                                   // channels tid and tid + 128

    for (int c0 = j0; c0 < j1; c0 += KVG_CHUNK) {
        const int nc = min(KVG_CHUNK, j1 - c0);
        float sv = -INFINITY;
        if (tid < nc) {
            const int key = c0 + tid;
            float dot = 0.0f;
            for (int blk = 0; blk < NB; ++blk) {
                const int64_t slot = (head_base + blk) * Lcap + key;
                const float d1 = kv_block_dot<U>(kp.u + slot * f.UB, kp.h + slot * f.SB, f.UB, f.SB, f.lg_gs,
                                                 q_sh + blk * BLOCK);
                dot = fmaf(d1, exp2_int((int)kp.s[slot]), dot);
            }
            sv = dot * sm_scale;
        }
        // block max of this chunk's scores
        float mx = sv;
#pragma unroll
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if ((tid & 31) == 0) red[tid >> 5] = mx;
        __syncthreads();
        mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
        const float m_new = fmaxf(m_i, mx);
        const float alpha = (m_i == -INFINITY) ? 0.0f : __expf(m_i - m_new);
        const float pv = (tid < nc) ? __expf(sv - m_new) : 0.0f;
        sc[tid] = pv;
        float ps = pv;
#pragma unroll
        for (int o = 16; o; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        __syncthreads();                       // red[] reads done, sc[] visible
        if ((tid & 31) == 0) red[tid >> 5] = ps;
        __syncthreads();
        l_i = l_i * alpha + (red[0] + red[1] + red[2] + red[3]);
        m_i = m_new;
        for (int i = 0, d = tid; d < D; d += KVG_THREADS, ++i) {
            const int blk = d >> 5, k = d & 31;
            float a = acc[i] * alpha;
            for (int j = 0; j < nc; ++j) {
                const int64_t slot = (head_base + blk) * Lcap + (c0 + j);
                a = fmaf(sc[j], kv_element(vp, slot, k, f), a);
            }
            acc[i] = a;
        }
        __syncthreads();
    }
    float* out = partial + (((int64_t)b * H + h) * S + s) * kv_partial_stride(D);
    for (int i = 0, d = tid; d < D; d += KVG_THREADS, ++i) out[d] = acc[i];
    if (tid == 0) { out[D] = m_i; out[D + 1] = l_i; }
}

// Merge the S tile partials of one (sequence, head): weights exp(m_s - max m).
__global__ void kv_decode_combine_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                         float* __restrict__ out_f32, int H, int D, int S) {
    chain_release();
    chain_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const float* base = partial + ((int64_t)b * H + h) * S * kv_partial_stride(D);
    float mg = -INFINITY;
    for (int s = 0; s < S; ++s) mg = fmaxf(mg, base[s * kv_partial_stride(D) + D]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float num = 0.0f, den = 0.0f;
        for (int s = 0; s < S; ++s) {
            const float* p = base + s * kv_partial_stride(D);
            const float m = p[D];
            const float w = (m == -INFINITY) ? 0.0f : __expf(m - mg);
            num = fmaf(p[d], w, num);
            den = fmaf(p[D + 1], w, den);
        }
        const float r = den > 0.0f ? num / den : 0.0f;
        const int64_t o = ((int64_t)b * H + h) * D + d;
        out[o] = __float2bfloat16_rn(r);
        if (out_f32) out_f32[o] = r;
    }
}

}  // namespace msaq

// One warp quantises one row of D = 32 * EPL values into the packed planes (RoPE and the Hadamard rotation first
// where the job asks for them): the body of the append / prefill-write kernels (kv_pack.cu), shared with the
// flash-decode kernel, whose thread block that owns the new token's key tile writes the token itself.
// Behaviour replaced: csrc/kv_attention.cu:1766-1870 (kv_write / kv_append / kv_append_rot kernels) of the reference.
#pragma once

#include "msaq_common.cuh"
#include "sm100_ptx.cuh"

namespace msaq {

// 2^k as a double, k in [-1022, 1023].
__device__ __forceinline__ double pow2d(int k) { return __hiloint2double((1023 + k) << 20, 0); }

// One tensor to quantise into one set of planes; blockIdx.y picks the job, so the K (rotated) and
// V rows of a decode step go out in a single launch.
struct QuantJob {
    const __nv_bfloat16* X;
    int8_t* scale_exp;
    uint8_t* upper;
    uint8_t* shared;
    int rot;
    int rope;                // apply map.rope at the row's slot (= its token position) first
    int mx;                  // plain MXINT8 planes: `upper` is the int8 code plane [.., 32], `shared` is unused
};
struct QuantJobs { QuantJob j[2]; };

constexpr int QROW_CW = 12;                                  // code words per block: 7 of upper codes, then shared codes

// rowbuf: D floats, codes: (D / 32) * QROW_CW words of shared memory owned by the calling warp.
// head / key: the row's place in the planes ([head][block][key], key stride Lcap); row: its index in job.X.
template <int EPL>
__device__ __forceinline__ void quantize_row_warp(const QuantJob& job, const Rope& rope, int64_t row, int64_t head, int64_t key,
                                                  int64_t Lcap, const Fmt& f, float* rowbuf, uint32_t* codes, int lane) {
    constexpr int D = 32 * EPL, NB = EPL;
    constexpr int CW = QROW_CW;
    float v[EPL];
    const __nv_bfloat16* src = job.X + row * D + lane * EPL;
#pragma unroll
    for (int i = 0; i < EPL; ++i) v[i] = __bfloat162float(src[i]);
    if (job.rope && rope.cos) rope_warp<EPL>(v, lane, rope, rope.rows == 1 ? 0 : key);
    if (job.rot != 0) {
        fwht_warp<EPL>(v, lane);
        const float inv = (float)(1.0 / sqrt((double)D));
#pragma unroll
        for (int i = 0; i < EPL; ++i) v[i] = v[i] * inv;
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) rowbuf[lane * EPL + i] = v[i];
    for (int i = lane; i < NB * CW; i += 32) codes[i] = 0u;
    __syncwarp();

    const int lim = (1 << (7 - f.u)) - 1, slo = -(1 << (f.u - 1)), shi = (1 << (f.u - 1)) - 1;
    const int g0 = lane & ~(f.gs - 1);                        // first lane of this lane's group

    // One lane per element of the 32-block.  The arithmetic is the float64 sequence NumPy runs for
    // ms_lib/pack.py:47-60 (scalings by powers of two are exact, so a multiply stands in for each
    // divide; the group sum keeps NumPy's order), so the codes equal the reference's bit for bit.
#pragma unroll 1
    for (int b = 0; b < NB; ++b) {
        const float x = rowbuf[b * BLOCK + lane];
        float amax = fmaxf(0.0f, fabsf(x));
#pragma unroll
        for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const int e = block_exponent(amax);
        const double xv = (double)x;
        if (job.mx) {
            // plain MXINT8 (ms_lib/pack.py:538-543 of the reference): one int8 code per element on the grid 2^e
            double qm = rint(xv * pow2d(-e));
            qm = fmin(fmax(qm, -127.0), 127.0);
            const int64_t slot = (head * NB + b) * Lcap + key;
            reinterpret_cast<int8_t*>(job.upper)[slot * BLOCK + lane] = (int8_t)(int)qm;
            if (lane == 0) job.scale_exp[slot] = (int8_t)e;
            continue;
        }
        double q = rint(xv * pow2d(-(e + f.u)));
        q = fmin(fmax(q, (double)-lim), (double)lim);
        const double res = xv - q * pow2d(e + f.u);
        double sum;
        if (f.gs < 8) {                                       // NumPy: plain running sum below 8 terms
            sum = 0.0;
            for (int t = 0; t < f.gs; ++t) sum += __shfl_sync(0xffffffffu, res, g0 + t);
        } else {                                              // NumPy: 8 interleaved partial sums, then a tree
            double r[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) r[j] = __shfl_sync(0xffffffffu, res, g0 + j);
            for (int t0 = 8; t0 < f.gs; t0 += 8) {
#pragma unroll
                for (int j = 0; j < 8; ++j) r[j] += __shfl_sync(0xffffffffu, res, g0 + t0 + j);
            }
            sum = ((r[0] + r[1]) + (r[2] + r[3])) + ((r[4] + r[5]) + (r[6] + r[7]));
        }
        double sq = rint(sum * pow2d(-f.lg_gs - e));
        sq = fmin(fmax(sq, (double)slo), (double)shi);

        uint32_t* cw = codes + b * CW;
        {
            const uint32_t c = (uint32_t)(int)q & ((1u << f.wbits) - 1u);
            const int bit = lane * f.wbits, wi = bit >> 5, off = bit & 31;
            atomicOr(&cw[wi], c << off);
            if (off + f.wbits > 32) atomicOr(&cw[wi + 1], c >> (32 - off));
        }
        if (lane == g0) {
            const uint32_t c = (uint32_t)(int)sq & ((1u << f.u) - 1u);
            const int bit = (lane >> f.lg_gs) * f.u, wi = bit >> 5, off = bit & 31;
            atomicOr(&cw[7 + wi], c << off);
            if (off + f.u > 32) atomicOr(&cw[7 + wi + 1], c >> (32 - off));
        }
        __syncwarp();
        const int64_t slot = (head * NB + b) * Lcap + key;
        if (lane < f.UB / 4) reinterpret_cast<uint32_t*>(job.upper + slot * f.UB)[lane] = cw[lane];   // UB is a multiple of 4
        if (lane < f.SB) job.shared[slot * f.SB + lane] = (uint8_t)(cw[7 + (lane >> 2)] >> ((lane & 3) * 8));
        if (lane == 0) job.scale_exp[slot] = (int8_t)e;
    }
}

}  // namespace msaq

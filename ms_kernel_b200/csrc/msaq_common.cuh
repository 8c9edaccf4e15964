// Shared device/host helpers of the MSAQ-signed decode kernels (sm_100a).
//
// Format constants and the block numerics follow ms_lib/pack.py:22-60 of the
// reference; the bit layout follows ms_lib/pack.py:82-98.
#pragma once

#include <utility>

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/msaq_b200.h"

namespace msaq {

constexpr int BLOCK = 32;
constexpr int E_MAX = 6;

// Derived sizes of one (u, gs) format.
struct Fmt {
    int u, gs, lg_gs, wbits, UB, SB, ng;
};

inline bool make_fmt(int u, int gs, Fmt* f) {
    if (u < 2 || u > 4) return false;
    int lg = 0;
    while ((1 << lg) < gs) ++lg;
    if ((1 << lg) != gs || gs < 2 || gs > 32) return false;
    f->u = u; f->gs = gs; f->lg_gs = lg; f->wbits = 8 - u;
    f->UB = BLOCK * f->wbits / 8;
    f->ng = BLOCK / gs;
    f->SB = (f->ng * u + 7) / 8;
    return true;
}

// Every workspace starts with a control region that only the integer-MMA GEMV's tile hand-off uses
// (status word, then the (tile, warp) counters, which are zero at rest): the other kernels keep their
// scratch behind it, so that a caller (or an allocator) that hands the same memory to one call after
// another never puts the counters under another kernel's partial sums.
constexpr size_t WS_CTL_BYTES = 64 * 1024;

// ---- host-side error plumbing (defined in capi.cu) -------------------------
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);
void count_launch(int n = 1);
int sm_count();               // SM count of the current device (cached per device)
int require_sm100();          // MSAQ_OK or MSAQ_ERR_DEVICE
bool option_chained_launch(); // kernels are launched with programmatic stream serialisation
bool option_tensor_memory();  // batched GEMVs of 9 rows and more run on tcgen05 with tensor-memory accumulators
bool option_early_weights();   // MSAQ_OPT_EARLY_WEIGHTS: weights are fetched before the wait on the kernel in front
bool option_inkernel_staging(); // GEMVs of up to four rows stage their activations inside the main kernel
uint32_t next_call_tag();     // a process-wide 31-bit sequence number, never 0: tags a call's counters and status word
unsigned option_wait_polls(); // poll limit of the bounded mbarrier waits
int option_test_skip_stage(); // test hook: pipeline stage whose copy the first CTA's producer leaves out (-1: none)
int* sticky_status();         // device address of the per-device status word on the current device (null on failure)

// Launch `kernel` so that it may begin while the previous kernel in the stream drains (see
// chain_wait / chain_release): every kernel of this library executes chain_wait() before it
// touches memory another kernel produces or consumes.
// An SM holds thread blocks of two kernels at once only under one split of its L1 / shared memory.  The streaming
// kernels need the largest shared-memory share, so with MSAQ_OPT_EARLY_WEIGHTS every kernel of the chain asks for
// it: otherwise the blocks of a GEMV launched early behind a small kernel (activation staging, cache append,
// residual add) could not start -- and begin fetching their weights -- until the small kernel had left every SM
// (measured with per-block time stamps: without it the GEMV's first block starts when the staging kernel's last
// block exits; with it 0.9 us after the staging kernel starts).
void prefer_max_shared(const void* kernel);      // once per (kernel, device), only while the option is on

template <typename... P, typename... A>
inline cudaError_t launch_chained(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A&&... args) {
    prefer_max_shared(reinterpret_cast<const void*>(kernel));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = option_chained_launch() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<A>(args)...);
}

// Rotary position embedding tables as the reference's harness builds them (tests/harness_batchsweep.py:
// 118-137): cos/sin fp32 [rows][D/2]; rows == 1 means one position for every sequence (the harness's
// rope_pos), otherwise the row is the token's position (rope_tables).  cos == nullptr: no RoPE.
struct Rope {
    const float* cos;
    const float* sin;
    int64_t rows;
};

// ---- small device helpers ---------------------------------------------------
// One rotary pair, evaluated as torch evaluates rope_bthd (tests/harness_batchsweep.py:134-137): fp32
// products and sum, each rounded separately (no fused multiply-add), then the cast to bf16.
__device__ __forceinline__ void rope_pair(float x1, float x2, float c, float s, float* o1, float* o2) {
    *o1 = __bfloat162float(__float2bfloat16_rn(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s))));
    *o2 = __bfloat162float(__float2bfloat16_rn(__fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c))));
}

// RoPE on a row held as EPL consecutive elements per lane (element index lane*EPL + i); `row` is the
// table row.  With one element per lane the pair partner is the neighbouring lane.
template <int EPL>
__device__ __forceinline__ void rope_warp(float (&v)[EPL], int lane, const Rope& r, int64_t row) {
    constexpr int HALF = 16 * EPL;                            // D / 2
    const float* cr = r.cos + row * HALF;
    const float* sr = r.sin + row * HALF;
    if constexpr (EPL == 1) {
        const float other = __shfl_xor_sync(0xffffffffu, v[0], 1);
        const float c = cr[lane >> 1], s = sr[lane >> 1];
        float o1, o2;
        if (lane & 1) { rope_pair(other, v[0], c, s, &o1, &o2); v[0] = o2; }
        else { rope_pair(v[0], other, c, s, &o1, &o2); v[0] = o1; }
    } else {
#pragma unroll
        for (int i = 0; i < EPL; i += 2) {
            const int j = (lane * EPL + i) >> 1;
            rope_pair(v[i], v[i + 1], cr[j], sr[j], &v[i], &v[i + 1]);
        }
    }
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }
__device__ __forceinline__ float bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t pair) { return __uint_as_float(pair & 0xFFFF0000u); }

// 2^e as float for e in [-126, 127]; below that the subnormal / zero value.
__device__ __forceinline__ float exp2_int(int e) {
    return (e >= -126) ? __int_as_float((e + 127) << 23) : ldexpf(1.0f, e);
}

__device__ __forceinline__ int sext(uint32_t v, int width) {
    return ((int)(v << (32 - width))) >> (32 - width);
}

// Code `idx` of `width` bits from a little-endian word run (run must have one
// readable word past the last code when a code straddles a word boundary).
__device__ __forceinline__ int code_from_words(const uint32_t* w, int idx, int width) {
    const int bit = idx * width, wi = bit >> 5, off = bit & 31;
    uint32_t v = w[wi] >> off;
    if (off + width > 32) v |= w[wi + 1] << (32 - off);
    return sext(v, width);
}

// Block exponent from the block's max-abs: clip(floor(log2(max(amax, 1e-30))) - 6, +-127).
__device__ __forceinline__ int block_exponent(float amax) {
    int fl;
    if (!((double)amax >= 1e-30)) fl = -100;                      // floor(log2(1e-30)) = -100
    else if (isinf(amax)) fl = 1000;
    else fl = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127;  // normal numbers only reach here
    const int e = fl - E_MAX;
    return max(-127, min(127, e));
}

// Quantise one 32-block.  Arithmetic is float64 in the order NumPy evaluates
// ms_lib/pack.py:47-60, so the codes equal the reference's bit for bit.
//   up[k] : (8-u)-bit signed, sh[g] : u-bit signed, returns the exponent.
__device__ inline int quantize_block(const float* x, const Fmt& f, int* up, int* sh) {
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < BLOCK; ++k) amax = fmaxf(amax, fabsf(x[k]));
    const int e = block_exponent(amax);
    const double fine = ldexp(1.0, e), coarse = ldexp(1.0, e + f.u);
    const int lim = (1 << (7 - f.u)) - 1, slo = -(1 << (f.u - 1)), shi = (1 << (f.u - 1)) - 1;
    for (int g = 0; g < f.ng; ++g) {
        double r[8];
        double sum = 0.0;
        for (int t = 0; t < f.gs; ++t) {
            const int k = g * f.gs + t;
            const double xv = (double)x[k];
            double q = rint(xv / coarse);
            q = fmin(fmax(q, (double)-lim), (double)lim);
            up[k] = (int)q;
            const double res = xv - q * coarse;
            if (f.gs < 8) sum += res;                      // NumPy: plain running sum below 8 terms
            else if (t < 8) r[t] = res;                    // NumPy: 8 interleaved partial sums ...
            else r[t & 7] += res;
        }
        if (f.gs >= 8) sum = ((r[0] + r[1]) + (r[2] + r[3])) + ((r[4] + r[5]) + (r[6] + r[7]));
        double s = rint((sum / (double)f.gs) / fine);
        s = fmin(fmax(s, (double)slo), (double)shi);
        sh[g] = (int)s;
    }
    return e;
}

// 2^k as a double, k in [-1022, 1023].
__device__ __forceinline__ double pow2_f64(int k) { return __hiloint2double((1023 + k) << 20, 0); }

// The same block quantiser with one lane per element (lane = element index of the 32-block, all 32 lanes
// take part): returns the block exponent, this element's upper code in *up and its group's shared code in
// *sh.  Float64 in NumPy's order, like quantize_block, so the codes equal the reference's bit for bit
// (scalings by powers of two are exact, so a multiply stands in for each divide).
__device__ __forceinline__ int quantize_lane(float x, int lane, const Fmt& f, int* up, int* sh) {
    float amax = fmaxf(0.0f, fabsf(x));
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const int e = block_exponent(amax);
    const int lim = (1 << (7 - f.u)) - 1, slo = -(1 << (f.u - 1)), shi = (1 << (f.u - 1)) - 1;
    const int g0 = lane & ~(f.gs - 1);                        // first lane of this lane's group
    const double xv = (double)x;
    double q = rint(xv * pow2_f64(-(e + f.u)));
    q = fmin(fmax(q, (double)-lim), (double)lim);
    const double res = xv - q * pow2_f64(e + f.u);
    double sum;
    if (f.gs < 8) {                                           // NumPy: plain running sum below 8 terms
        sum = 0.0;
        for (int t = 0; t < f.gs; ++t) sum += __shfl_sync(0xffffffffu, res, g0 + t);
    } else {                                                  // NumPy: 8 interleaved partial sums, then a tree
        double r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = __shfl_sync(0xffffffffu, res, g0 + j);
        for (int t0 = 8; t0 < f.gs; t0 += 8) {
#pragma unroll
            for (int j = 0; j < 8; ++j) r[j] += __shfl_sync(0xffffffffu, res, g0 + t0 + j);
        }
        sum = ((r[0] + r[1]) + (r[2] + r[3])) + ((r[4] + r[5]) + (r[6] + r[7]));
    }
    double sq = rint(sum * pow2_f64(-f.lg_gs - e));
    sq = fmin(fmax(sq, (double)slo), (double)shi);
    *up = (int)q;
    *sh = (int)sq;
    return e;
}

// Dense LSB-first packing of n codes of `width` bits into zeroed words.
__device__ inline void pack_codes(const int* codes, int n, int width, uint32_t* words, int nwords) {
    for (int i = 0; i < nwords; ++i) words[i] = 0u;
    const uint32_t mask = (1u << width) - 1u;
    for (int i = 0; i < n; ++i) {
        const uint32_t c = (uint32_t)codes[i] & mask;
        const int bit = i * width, wi = bit >> 5, off = bit & 31;
        words[wi] |= c << off;
        if (off + width > 32) words[wi + 1] |= c >> (32 - off);
    }
}

// Quantise + pack + store one block at `slot` of token-major planes
// (scale_exp[slot], upper[slot*UB..], shared[slot*SB..]).
__device__ inline void store_block(const float* x, const Fmt& f, int8_t* scale_exp, uint8_t* upper,
                                   uint8_t* shared, int64_t slot) {
    int up[BLOCK], sh[16];
    const int e = quantize_block(x, f, up, sh);
    uint32_t uw[7], sw[3];
    pack_codes(up, BLOCK, f.wbits, uw, 7);
    pack_codes(sh, f.ng, f.u, sw, 3);
    uint32_t* du = reinterpret_cast<uint32_t*>(upper + slot * f.UB);   // UB is a multiple of 4
    for (int i = 0; i < f.UB / 4; ++i) du[i] = uw[i];
    uint8_t* ds = shared + slot * f.SB;
    for (int i = 0; i < f.SB; ++i) ds[i] = (uint8_t)(sw[i >> 2] >> ((i & 3) * 8));
    scale_exp[slot] = (int8_t)e;
}

// In-register Walsh-Hadamard butterfly over a row of 32*EPL values held as EPL
// consecutive elements per lane.  Stage order h = 1, 2, 4, ...: strides below
// EPL stay inside the lane, the rest are lane exchanges.  Every stage is one
// fp32 add or subtract per element, so the result does not depend on which
// thread evaluates it.
template <int EPL>
__device__ __forceinline__ void fwht_warp(float (&v)[EPL], int lane) {
#pragma unroll
    for (int h = 1; h < EPL; h <<= 1) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            if ((i & h) == 0) {
                const float a = v[i], b = v[i + h];
                v[i] = a + b;
                v[i + h] = a - b;
            }
        }
    }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], m);
            v[i] = (lane & m) ? (other - v[i]) : (v[i] + other);
        }
    }
}

}  // namespace msaq

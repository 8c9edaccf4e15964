// Tuned weight-only GEMV for u = 4, gs = 2 on column-major planes.
//
// Data flow per CTA (a tile of 128 output columns x a range of K blocks):
//   * one producer thread streams the packed bytes of its tile (upper codes,
//     shared codes, scale bytes) and the pre-split activations into a ring of
//     shared-memory stages with TMA bulk copies (cp.async.bulk + mbarrier);
//   * eight consumer warps each own 16 columns.  A thread turns the nibbles of
//     a 32-bit word into int8 tensor-core operands with three logic ops -- a
//     two's-complement nibble in the high half of a byte IS the int8 value
//     16*up, and the offset-binary shared nibble ORs into the low half -- so
//     one m16n8k32 integer MMA yields the exact integer dot of a 32-block
//     against up to four activation rows;
//   * the integer dot is scaled by 2^(weight exponent) * 2^(activation block
//     exponent) and accumulated in fp32; split-K partials go to the workspace.
//
// Activations are staged once per call by gemv_xprep_kernel as 16-bit block
// fixed point (two int8 planes per row): x = xi * 2^(E-14) with E the exponent
// of the block's max-abs, |xi| <= 32640.  Every bf16 element within a factor
// 2^7 of its block maximum is represented exactly; smaller ones are rounded
// with absolute error <= 2^(E-15).  The one unrepresentable code (+32640) is
// stored as 32639.
//
// Algorithm replaced: csrc/w_gemv.cu:173-284 (wide u4 kernel) and :417-487
// (batched kernel) of the reference.
#pragma once

#include "msaq_common.cuh"
#include "sm100_ptx.cuh"

namespace msaq {

#ifndef MSAQ_GM_WARPS
#define MSAQ_GM_WARPS 8
#endif
#ifndef MSAQ_GM_CTAS
#define MSAQ_GM_CTAS 3
#endif
constexpr int GM_WARPS = MSAQ_GM_WARPS;   // consumer warps; each owns 16 columns of every column group
constexpr int GM_THREADS = (GM_WARPS + 1) * 32;
constexpr int GM_GROUP = GM_WARPS * 16;   // columns per group
#ifndef MSAQ_GM_MAX_MULT
#define MSAQ_GM_MAX_MULT 8
#endif
constexpr int GM_MAX_MULT = MSAQ_GM_MAX_MULT;   // widest tile in groups (the widest only for single-row launches)
constexpr int GM_MAX_TC = GM_MAX_MULT * GM_GROUP;
constexpr int GM_MAX_STAGES = 12;
constexpr int GM_MP = 4;             // activation rows per MMA pass
constexpr int GM_MAX_PASSES = 4;     // -> at most 16 rows per launch
constexpr int GM_XREC = 320;         // bytes of staged activations per (block, pass)
constexpr int GM_CTAS_PER_SM = MSAQ_GM_CTAS;
// Largest in-kernel record table: two records per warp of the CTA.  (One per warp was the first rule; a second
// round costs less than the staging launch it replaces: 8192x8192, one row, 19.85 -> 19.2 us.)
constexpr int GM_MAX_TABLE = 2 * (GM_WARPS + 1) * GM_XREC;

// Stage layout for a tile of TC columns x one K block:
//   upper [TC][16] | shared [TC][8] | scale [TC] | activations [passes][GM_XREC]
// The weight format the kernel streams: the MSAQ-signed u4/gs2 planes (25 bytes per column and K block: 16 of
// upper codes, 8 of shared codes, the scale), or plain MXINT8 (33 bytes: 32 int8 codes and the scale), the
// reference's matched baseline (csrc/mxint8.cu:196-253), whose codes are MMA operands as they are.
constexpr int GF_MSAQ_U4 = 0, GF_MXINT8 = 1;
__host__ __device__ constexpr int gm_col_bytes(int fmt) { return fmt == GF_MXINT8 ? 33 : 25; }
__host__ __device__ inline int gm_stage_bytes(int tc, int passes, int fmt = GF_MSAQ_U4) {
    return tc * gm_col_bytes(fmt) + passes * GM_XREC;
}

// Work decomposition shared by host and device.  A unit is (column tile c,
// K block b); unit index n = c * NB + b.  CTA i of `grid` owns the units
// [i*U/grid, (i+1)*U/grid): contiguous, equal to within one unit, so a grid of
// (SMs x resident CTAs) finishes in one balanced wave.  A tile is covered by
// consecutive CTAs; each leaves one partial sum in slot (cta - first cta of the
// tile), and the CTA that completes a tile adds the slots up in slot order.
struct GemvSchedule {
    int tc;            // columns per tile: 128, 256 or 512
    int col_tiles, nb, grid, max_slots;
    int stages;        // depth of the shared-memory ring (<= GM_MAX_STAGES)
    __host__ __device__ long long units() const { return (long long)col_tiles * nb; }
    __host__ __device__ long long lo(int cta) const { return units() * cta / grid; }
    __host__ __device__ int first_cta(int c) const { return (int)((((long long)c * nb + 1) * grid - 1) / units()); }
    __host__ __device__ int last_cta(int c) const { return (int)((((long long)(c + 1) * nb) * grid - 1) / units()); }
};

// ---- activation staging -------------------------------------------------------
// Record of one (block, pass): xq[8 cols][4 t][8 bytes] | tc[4 t]{corr, cx, 0, 0}.
// Column 2*mm is the high byte plane of row 4*pass+mm, column 2*mm+1 the low one.
// Thread-slot t = 2h + odd of a column holds, for i = 0..3, the elements
// 16h + 4i + 2*odd (bytes 0..3) and 16h + 4i + 2*odd + 1 (bytes 4..7): the
// elements whose shared codes are the even (odd = 0) or odd nibbles of shared
// word h, in the byte order the consumer builds its MMA operand in.
// What the staging kernel computes before it splits the activations (the glue of a decoder
// layer that would otherwise be separate launches in front of a GEMV):
//   XP_PLAIN     x = X[m][k]
//   XP_RMSNORM   x = bf16(X[m][k] * rsqrt(mean_k(X[m][k]^2) + eps))
//   XP_SILU_MUL  x = bf16(silu(X[m][k]) * X[m][K + k]),  X is [M][2K]
//   XP_ADD_NORM  h = bf16(X[m][k] + R[m][k]) is written to h_out, then x = rmsnorm(h) as above
enum XprepMode { XP_PLAIN = 0, XP_RMSNORM = 1, XP_SILU_MUL = 2, XP_ADD_NORM = 3 };

struct XprepArgs {
    const __nv_bfloat16* X;      // rows start at X + m * ldx
    const void* R;               // XP_ADD_NORM: the addend, bf16 or fp32, [M][K]
    __nv_bfloat16* h_out;        // XP_ADD_NORM: the sum, [M][K]
    uint8_t* xprep;
    int M, NB, passes, ldx, r_is_f32;
    float eps;
    int natural;             // record in natural element order (MXINT8 weights) instead of the nibble-matched order
};

#ifdef MSAQ_TRACE
__device__ unsigned long long g_trace[2][1024][8];
__device__ __forceinline__ void trace_ev(int k, int ev) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (blockIdx.x < 1024) g_trace[k][blockIdx.x][ev] = t;
}
#define MSAQ_TR(k, ev, cond) do { if (cond) trace_ev(k, ev); } while (0)
#else
#define MSAQ_TR(k, ev, cond) do { } while (0)
#endif

template <int MODE>
__global__ void __launch_bounds__(128)
gemv_xprep_kernel(const XprepArgs a) {
    MSAQ_TR(0, 0, threadIdx.x == 0);
    chain_release();
    chain_wait();
    MSAQ_TR(0, 1, threadIdx.x == 0);
    __shared__ float red[GM_MP][4];
    const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
    const int warp = gtid >> 5, lane = threadIdx.x & 31, wic = threadIdx.x >> 5;
    // a CTA is the four row slots (mm = 0..3) of one (block, pass)
    const int mm = warp % GM_MP, pass = (warp / GM_MP) % a.passes, blk = warp / (GM_MP * a.passes);
    const int m = pass * GM_MP + mm;
    const int K = a.NB * BLOCK;
    const bool live = blk < a.NB;                  // uniform over the CTA

    float inv_rms = 1.0f;
    // this warp's own 32 elements, asked for before the row norm so that they do not cost a second round of
    // load latency behind it
    float hv_own = 0.0f, d_own = 0.0f;
    if ((MODE == XP_RMSNORM || MODE == XP_ADD_NORM) && live && m < a.M) {
        const int k = blk * BLOCK + lane;
        hv_own = __bfloat162float(a.X[(int64_t)m * a.ldx + k]);
        if (MODE == XP_ADD_NORM) {
            const int64_t o = (int64_t)m * K + k;
            d_own = a.r_is_f32 ? static_cast<const float*>(a.R)[o] : __bfloat162float(static_cast<const __nv_bfloat16*>(a.R)[o]);
        }
    }
    if (MODE == XP_RMSNORM || MODE == XP_ADD_NORM) {
        // Sum of squares of each of this pass's rows, by the whole CTA, in an order that does not
        // depend on the CTA: every CTA arrives at the same bits.
        const float* Rf = static_cast<const float*>(a.R);
        const __nv_bfloat16* Rh = static_cast<const __nv_bfloat16*>(a.R);
        for (int r = 0; r < GM_MP; ++r) {
            const int mr = pass * GM_MP + r;
            float ss = 0.0f;
            if (live && mr < a.M) {
                const uint4* xr = reinterpret_cast<const uint4*>(a.X + (int64_t)mr * a.ldx);
                // four 16-byte chunks per thread at a time, every load of the batch issued before the first use
                for (int i0 = threadIdx.x; i0 < K / 8; i0 += 4 * 128) {
                    uint4 hv[4], dv[4], dv2[4];
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        const int i = i0 + b * 128;
                        const bool in = i < K / 8;
                        hv[b] = in ? xr[i] : make_uint4(0u, 0u, 0u, 0u);
                        dv[b] = dv2[b] = make_uint4(0u, 0u, 0u, 0u);
                        if (MODE == XP_ADD_NORM && in) {
                            const int64_t o = (int64_t)mr * K + i * 8;    // 16-byte aligned: the launcher checks the bases
                            if (a.r_is_f32) {
                                dv[b] = *reinterpret_cast<const uint4*>(Rf + o);
                                dv2[b] = *reinterpret_cast<const uint4*>(Rf + o + 4);
                            } else {
                                dv[b] = *reinterpret_cast<const uint4*>(Rh + o);
                            }
                        }
                    }
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        const uint32_t w[4] = {hv[b].x, hv[b].y, hv[b].z, hv[b].w};
                        float f[8];
#pragma unroll
                        for (int j = 0; j < 4; ++j) { f[2 * j] = bf16_lo(w[j]); f[2 * j + 1] = bf16_hi(w[j]); }
                        if (MODE == XP_ADD_NORM) {
                            float d[8];
                            if (a.r_is_f32) {
                                d[0] = __uint_as_float(dv[b].x); d[1] = __uint_as_float(dv[b].y);
                                d[2] = __uint_as_float(dv[b].z); d[3] = __uint_as_float(dv[b].w);
                                d[4] = __uint_as_float(dv2[b].x); d[5] = __uint_as_float(dv2[b].y);
                                d[6] = __uint_as_float(dv2[b].z); d[7] = __uint_as_float(dv2[b].w);
                            } else {
                                const uint32_t dw[4] = {dv[b].x, dv[b].y, dv[b].z, dv[b].w};
#pragma unroll
                                for (int j = 0; j < 4; ++j) { d[2 * j] = bf16_lo(dw[j]); d[2 * j + 1] = bf16_hi(dw[j]); }
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(__float2bfloat16_rn(f[j] + d[j]));
                        }
                        // chunks past the end of the row are zero and add nothing
#pragma unroll
                        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
                    }
                }
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) red[r][wic] = ss;
        }
        __syncthreads();
        const float tot = (red[mm][0] + red[mm][1]) + (red[mm][2] + red[mm][3]);
        inv_rms = rsqrtf(tot / (float)K + a.eps);
    }
    if (!live) return;

    float x = 0.0f;
    if (m < a.M) {
        const int k = blk * BLOCK + lane;
        const __nv_bfloat16* xr = a.X + (int64_t)m * a.ldx;
        if (MODE == XP_PLAIN) {
            x = __bfloat162float(xr[k]);
        } else if (MODE == XP_SILU_MUL) {
            const float g = __bfloat162float(xr[k]), u = __bfloat162float(xr[K + k]);
            x = __bfloat162float(__float2bfloat16_rn(g / (1.0f + __expf(-g)) * u));
        } else {
            float hv = hv_own;
            if (MODE == XP_ADD_NORM) {
                const int64_t o = (int64_t)m * K + k;
                const float d = d_own;
                const __nv_bfloat16 hb = __float2bfloat16_rn(hv + d);
                a.h_out[o] = hb;
                hv = __bfloat162float(hb);
            }
            x = __bfloat162float(__float2bfloat16_rn(hv * inv_rms));
        }
    }
    uint32_t ax = __float_as_uint(x) & 0x7FFFFFFFu;
#pragma unroll
    for (int o = 16; o; o >>= 1) ax = max(ax, __shfl_xor_sync(0xffffffffu, ax, o));
    int E = (int)(ax >> 23) - 127;
    E = ax == 0u ? 0 : max(-100, min(127, E));
    int xi = __float2int_rn(x * __int_as_float((14 - E + 127) << 23));
    xi = min(xi, 32639);
    const int lo = (int)(int8_t)(xi & 0xFF), hi = (xi - lo) >> 8;
    uint8_t* rec = a.xprep + ((int64_t)blk * a.passes + pass) * GM_XREC;
    const int e = lane;
    // natural order: thread-slot t holds the elements 4t..4t+3 (bytes 0..3) and 16+4t..16+4t+3 (bytes 4..7)
    const int t = a.natural ? (e & 15) >> 2 : 2 * (e >> 4) + ((e >> 1) & 1);
    const int j = a.natural ? (e >> 4) * 4 + (e & 3) : (e & 1) * 4 + ((e & 15) >> 2);
    rec[(2 * mm) * 32 + t * 8 + j] = (uint8_t)hi;
    rec[(2 * mm + 1) * 32 + t * 8 + j] = (uint8_t)lo;
    int sh = hi, sl = lo;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        sh += __shfl_xor_sync(0xffffffffu, sh, o);
        sl += __shfl_xor_sync(0xffffffffu, sl, o);
    }
    if (lane == 0) {
        int* tc = reinterpret_cast<int*>(rec + 256 + mm * 16);
        tc[0] = -8 * (sh * 256 + sl);                         // correction for the offset-binary shared codes
        // 2^(E-14) as float bits; an Inf or NaN in the block makes the multiplier NaN, and with it the output row
        tc[1] = ax >= 0x7F800000u ? 0x7FC00000 : (int)((uint32_t)(E - 14 + 127) << 23);
        tc[2] = 0;
        tc[3] = 0;
    }
    MSAQ_TR(0, 2, threadIdx.x == 0);
}

// ---- main kernel ------------------------------------------------------------------
// Tensor-parallel row-parallel projections (O, down): instead of writing its finished outputs to local memory, the
// warp that completes a tile stores them straight into this rank's slot of every rank's exchange buffer (its own
// included), each float as an 8-byte word {x, seq} -- the layout and sequence number of peer_exchange.cu, whose
// receiving kernel then only waits and adds.  The partial sums leave tile by tile while the GEMV still runs.
struct PeerPush {
    float* buf[8];           // buf[r]: rank r's exchange memory as mapped into this process
    long long n;             // floats per slot (rows * OUT)
    int world, rank, parity; // world == 0: no push, ordinary outputs
};
__device__ __forceinline__ uint32_t gemv_push_seq(const PeerPush& p) {
    const unsigned int* ctl = reinterpret_cast<const unsigned int*>(p.buf[p.rank] + 4 * (long long)p.world * p.n);
    return *reinterpret_cast<const volatile unsigned int*>(ctl + p.parity) + 1u;
}
__device__ __forceinline__ void gemv_push(const PeerPush& p, long long idx, float v, uint32_t seq) {
    const long long off = (((long long)p.parity * p.world + p.rank) * p.n + idx) * 2;
    for (int r = 0; r < p.world; ++r)
        // weak stores: each 8-byte word validates itself, so their order does not matter
        asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(p.buf[r] + off), "r"(__float_as_uint(v)), "r"(seq) : "memory");
}

struct GemvMmaArgs {
    const int8_t* scale_exp;
    const uint8_t* upper_cm;
    const uint8_t* shared_cm;
    const uint8_t* xprep;    // activation records written by gemv_xprep_kernel (xmode < 0)
    float* partial;          // [max_slots][rows][OUT]
    unsigned long long* tile_counters;   // [col_tiles][GM_WARPS] words {marker, count}, see gemv_count_arrival
    int* status;             // holds the call tag when a bounded wait gave up during this call
    int* sticky;             // the library's per-device status word (may be null)
    __nv_bfloat16* y;        // [M][OUT]
    float* y_f32;            // optional
    int m0, rows;            // this launch covers rows [m0, m0 + rows), rows <= 16
    int OUT;
    int NB;                  // K blocks of the weight (sch.nb counts units: groups of KB blocks)
    GemvSchedule sch;
    uint32_t max_polls;      // limit of every mbarrier wait (see mbar_wait_bounded)
    int skip_stage;          // test hook: the producer of CTA 0 stops before this stage (-1: never)
    // Launches of up to four rows stage their activations themselves: the producer warp evaluates the
    // XprepMode `xmode` (>= 0) for each K block it streams and writes the record straight into the
    // ring stage, so no staging kernel runs in front.  X, R, h_out point at row m0.
    int xmode;
    const __nv_bfloat16* X;
    const void* R;
    __nv_bfloat16* h_out;
    int ldx, r_is_f32;
    float eps;
    uint32_t tag;            // identifies this call in the counters and the status word; 31 bits, never 0
    int table_bytes;         // shared memory in front of the ring that holds the in-kernel record table
    int natural;             // in-kernel records in natural element order (see XprepArgs)
    int early;               // first ring-full of weights goes out before the wait on the kernel in front
    PeerPush push;
    const __nv_bfloat16* res;   // optional [M][OUT]: y = bf16(res + W x), the residual add behind a layer's last projection
};

// Sums of squares of the launch's rows (of X, or of bf16(X + R) for XP_ADD_NORM) by all threads of the
// CTA in an order that depends on nothing but K: every CTA arrives at the same bits.
__device__ __forceinline__ void gemv_row_sumsq(const GemvMmaArgs& a, int K, float (*red)[GM_WARPS + 1]) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool add = a.xmode == XP_ADD_NORM;
    const float* Rf = static_cast<const float*>(a.R);
    const __nv_bfloat16* Rh = static_cast<const __nv_bfloat16*>(a.R);
    for (int r = 0; r < a.rows; ++r) {
        float ss = 0.0f;
        const uint4* xr = reinterpret_cast<const uint4*>(a.X + (int64_t)r * a.ldx);
        for (int i0 = tid; i0 < K / 8; i0 += 4 * GM_THREADS) {
            uint4 hv[4], dv[4], dv2[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int i = i0 + b * GM_THREADS;
                const bool in = i < K / 8;
                hv[b] = in ? xr[i] : make_uint4(0u, 0u, 0u, 0u);
                dv[b] = dv2[b] = make_uint4(0u, 0u, 0u, 0u);
                if (add && in) {
                    const int64_t o = (int64_t)r * K + i * 8;
                    if (a.r_is_f32) {
                        dv[b] = *reinterpret_cast<const uint4*>(Rf + o);
                        dv2[b] = *reinterpret_cast<const uint4*>(Rf + o + 4);
                    } else {
                        dv[b] = *reinterpret_cast<const uint4*>(Rh + o);
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t w[4] = {hv[b].x, hv[b].y, hv[b].z, hv[b].w};
                float f[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) { f[2 * j] = bf16_lo(w[j]); f[2 * j + 1] = bf16_hi(w[j]); }
                if (add) {
                    float d[8];
                    if (a.r_is_f32) {
                        d[0] = __uint_as_float(dv[b].x); d[1] = __uint_as_float(dv[b].y);
                        d[2] = __uint_as_float(dv[b].z); d[3] = __uint_as_float(dv[b].w);
                        d[4] = __uint_as_float(dv2[b].x); d[5] = __uint_as_float(dv2[b].y);
                        d[6] = __uint_as_float(dv2[b].z); d[7] = __uint_as_float(dv2[b].w);
                    } else {
                        const uint32_t dw[4] = {dv[b].x, dv[b].y, dv[b].z, dv[b].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) { d[2 * j] = bf16_lo(dw[j]); d[2 * j + 1] = bf16_hi(dw[j]); }
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(__float2bfloat16_rn(f[j] + d[j]));
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);       // chunks past the row's end are zero
            }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[r][warp] = ss;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(GM_THREADS) : "memory");
}

// The activation record of K block `kb` (all rows of the launch), written by one warp into a ring
// stage; same values and layout as gemv_xprep_kernel produces.  The planes of the rows beyond the
// launch's are left as they are: an MMA column only feeds its own row's sums, and those are never stored.
__device__ __forceinline__ void gemv_stage_block(const GemvMmaArgs& a, uint8_t* rec, int kb, int K, int lane,
                                                 bool write_h, const float (&inv_rms)[GM_MP]) {
    const int k = kb * BLOCK + lane;
#pragma unroll
    for (int m = 0; m < GM_MP; ++m) {
        if (m >= a.rows) break;
        const __nv_bfloat16* xr = a.X + (int64_t)m * a.ldx;
        float x;
        if (a.xmode == XP_PLAIN) {
            x = __bfloat162float(xr[k]);
        } else if (a.xmode == XP_SILU_MUL) {
            const float g = __bfloat162float(xr[k]), u = __bfloat162float(xr[K + k]);
            x = __bfloat162float(__float2bfloat16_rn(g / (1.0f + __expf(-g)) * u));
        } else {
            float hv = __bfloat162float(xr[k]);
            if (a.xmode == XP_ADD_NORM) {
                const int64_t o = (int64_t)m * K + k;
                const float d = a.r_is_f32 ? static_cast<const float*>(a.R)[o]
                                           : __bfloat162float(static_cast<const __nv_bfloat16*>(a.R)[o]);
                const __nv_bfloat16 hb = __float2bfloat16_rn(hv + d);
                if (write_h) a.h_out[o] = hb;
                hv = __bfloat162float(hb);
            }
            x = __bfloat162float(__float2bfloat16_rn(hv * inv_rms[m]));
        }
        const uint32_t ax = __reduce_max_sync(0xffffffffu, __float_as_uint(x) & 0x7FFFFFFFu);
        int E = (int)(ax >> 23) - 127;
        E = ax == 0u ? 0 : max(-100, min(127, E));
        int xi = __float2int_rn(x * __int_as_float((14 - E + 127) << 23));
        xi = min(xi, 32639);
        const int lo = (int)(int8_t)(xi & 0xFF), hi = (xi - lo) >> 8;
        const int e = lane;
        const int t = a.natural ? (e & 15) >> 2 : 2 * (e >> 4) + ((e >> 1) & 1);
        const int j = a.natural ? (e >> 4) * 4 + (e & 3) : (e & 1) * 4 + ((e & 15) >> 2);
        rec[(2 * m) * 32 + t * 8 + j] = (uint8_t)hi;
        rec[(2 * m + 1) * 32 + t * 8 + j] = (uint8_t)lo;
        const int sx = __reduce_add_sync(0xffffffffu, xi);          // = 256 * sum(hi) + sum(lo)
        if (lane == 0) {
            int* tc = reinterpret_cast<int*>(rec + 256 + m * 16);
            tc[0] = -8 * sx;
            tc[1] = ax >= 0x7F800000u ? 0x7FC00000 : (int)((uint32_t)(E - 14 + 127) << 23);
        }
    }
}

// One 16-column x 32-element step of a warp: decode both columns' codes into the
// int8 operand, one integer MMA per activation pass, scale and accumulate.
// Plain MXINT8: the int8 codes are the A operand as stored -- columns r0 and r0 + 8, elements 4t..4t+3 and
// 16+4t..16+4t+3 -- and there is no code offset to take out.
template <int PASSES, int Q>
__device__ __forceinline__ void gemv_group_step_mx(uint32_t wbase, uint32_t ebase, const uint2 (&bq)[PASSES],
                                                   const float (&cx)[PASSES], float (&acc)[PASSES][2]) {
    uint32_t A[4];
    A[0] = lds32<Q * GM_GROUP * 32>(wbase);
    A[1] = lds32<Q * GM_GROUP * 32 + 256>(wbase);
    A[2] = lds32<Q * GM_GROUP * 32 + 16>(wbase);
    A[3] = lds32<Q * GM_GROUP * 32 + 256 + 16>(wbase);
    const int e0 = lds_s8<Q * GM_GROUP>(ebase);
    const int e1 = lds_s8<Q * GM_GROUP + 8>(ebase);
    const float sw0 = __int_as_float(e0 * (1 << 23) + (127 << 23));
    const float sw1 = __int_as_float(e1 * (1 << 23) + (127 << 23));
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
        const uint32_t B[2] = {bq[p].x, bq[p].y};
        int Dm[4];
        mma_s8_16832_z(Dm, A, B);
        const float f0 = (float)(Dm[0] * 256 + Dm[1]) * cx[p];
        const float f1 = (float)(Dm[2] * 256 + Dm[3]) * cx[p];
        acc[p][0] = fmaf(f0, sw0, acc[p][0]);
        acc[p][1] = fmaf(f1, sw1, acc[p][1]);
    }
}

template <int PASSES, int Q>
__device__ __forceinline__ void gemv_group_step(uint32_t wbase, uint32_t sbase, uint32_t ebase, uint32_t sel,
                                                uint32_t nshift, const uint2 (&bq)[PASSES], const int (&corr)[PASSES],
                                                const float (&cx)[PASSES], float (&acc)[PASSES][2]) {
    const uint2 w0 = lds64<Q * GM_GROUP * 16>(wbase);
    const uint2 w1 = lds64<Q * GM_GROUP * 16 + 128>(wbase);
    const uint32_t s0 = lds32<Q * GM_GROUP * 8>(sbase);
    const uint32_t s1 = lds32<Q * GM_GROUP * 8 + 64>(sbase);
    const int e0 = lds_s8<Q * GM_GROUP>(ebase);
    const int e1 = lds_s8<Q * GM_GROUP + 8>(ebase);
    // shared codes (even or odd nibbles of word h) as offset-binary low nibbles
    const uint32_t m0 = and_xor(s0 >> nshift, 0x0F0F0F0Fu, 0x08080808u);
    const uint32_t m1 = and_xor(s1 >> nshift, 0x0F0F0F0Fu, 0x08080808u);
    // bytes of the upper words that hold the two elements of each of those groups
    const uint32_t x0 = prmt(w0.x, w0.y, sel), x1 = prmt(w1.x, w1.y, sel);
    uint32_t A[4];
    A[0] = and_or(x0 << 4, 0xF0F0F0F0u, m0);     // column r0, first element of each group
    A[1] = and_or(x1 << 4, 0xF0F0F0F0u, m1);     // column r0 + 8
    A[2] = and_or(x0, 0xF0F0F0F0u, m0);          // column r0, second element of each group
    A[3] = and_or(x1, 0xF0F0F0F0u, m1);
    const float sw0 = __int_as_float(e0 * (1 << 23) + (127 << 23));
    const float sw1 = __int_as_float(e1 * (1 << 23) + (127 << 23));
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
        const uint32_t B[2] = {bq[p].x, bq[p].y};
        int Dm[4];
        // (hi plane) * 256 + (lo plane) - 8 * sum(x): the offset-binary shared codes add 8 per element; that
        // correction rides into the lo-plane sums as the MMA's accumulator input
        mma_s8_16832_c(Dm, A, B, corr[p]);
        const float f0 = (float)(Dm[0] * 256 + Dm[1]) * cx[p];
        const float f1 = (float)(Dm[2] * 256 + Dm[3]) * cx[p];
        acc[p][0] = fmaf(f0, sw0, acc[p][0]);
        acc[p][1] = fmaf(f1, sw1, acc[p][1]);
    }
}

// The column groups Q, Q+1, ... of a tile, each with compile-time shared-memory offsets; ALL skips
// the per-group test when the warp has columns in every group.
template <int PASSES, int Q, int GROUPS, bool ALL, int FMT = GF_MSAQ_U4>
__device__ __forceinline__ void gemv_groups(int nq, uint32_t wb, uint32_t sbs, uint32_t eb, uint32_t sel, uint32_t nshift,
                                            const uint2 (&bq)[PASSES], const int (&corr)[PASSES], const float (&cx)[PASSES],
                                            float (&acc)[GROUPS][PASSES][2]) {
    if constexpr (Q < GROUPS) {
        if (ALL || Q < nq) {
            if constexpr (FMT == GF_MXINT8) gemv_group_step_mx<PASSES, Q>(wb, eb, bq, cx, acc[Q]);
            else gemv_group_step<PASSES, Q>(wb, sbs, eb, sel, nshift, bq, corr, cx, acc[Q]);
        }
        gemv_groups<PASSES, Q + 1, GROUPS, ALL, FMT>(nq, wb, sbs, eb, sel, nshift, bq, corr, cx, acc);
    }
}

// Counts one published partial sum on a (tile, warp) counter and returns how many there are now.
// The 64-bit word is {marker, count}.  At rest a valid word is {GM_MARKER, 0}: the warp that finishes a
// tile puts the count back to zero, so neither the next call nor a replay of a captured launch needs a
// reset in front, and an arrival is a single atomic add (`seen` is the marker as the caller read it when
// it started on the tile).  A workspace that was never used, or whose control region something else
// wrote to, shows another marker: the first arrival to notice claims the word (marker -> GM_MARKER_BUSY),
// clears the count and publishes GM_MARKER; arrivals that meet a claimed word wait for that.
// (A tag-and-count compare-and-swap loop needs no marker but collapses when the thirty-odd CTAs of a tile
// arrive together, +27 us on a 13 MB GEMV; per-slot flags with a sequentially consistent fence cost +3 us.)
constexpr unsigned int GM_MARKER = 0x9E3779B9u, GM_MARKER_BUSY = 0x1E3779B9u;
__device__ __forceinline__ unsigned int gemv_count_arrival(const GemvMmaArgs& a, unsigned long long* word, unsigned int seen) {
    unsigned int* marker = reinterpret_cast<unsigned int*>(word);
    unsigned int* count = marker + 1;
    if (seen != GM_MARKER) {
        bool ok = false;
        for (uint32_t i = 0; i < a.max_polls; ++i) {
            unsigned int m;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(m) : "l"(marker) : "memory");
            if (m == GM_MARKER) { ok = true; break; }
            if (m != GM_MARKER_BUSY && atomicCAS(marker, m, GM_MARKER_BUSY) == m) {
                *reinterpret_cast<volatile unsigned int*>(count) = 0u;
                __threadfence();
                asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(marker), "r"(GM_MARKER) : "memory");
                ok = true;
                break;
            }
            __nanosleep(64);
        }
        if (!ok) {
            report_wait_failure(a.status, (int)a.tag, a.sticky, WAIT_FAIL_GEMV_MMA);
            return 0u;
        }
    }
    unsigned int old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(count) : "memory");
    return old + 1u;
}

// In-kernel staging (launches of up to four rows).  The activation records of the K blocks a CTA streams
// live in a table in shared memory; record `i` belongs to the CTA's unit i / KB, K block i % KB of it.
// gemv_stage_records writes the records [i_begin, i_end) that fall to this warp (every i_step-th).
template <int KB>
__device__ __forceinline__ void gemv_stage_records(const GemvMmaArgs& a, uint8_t* table, int i_begin, int i_end, int i_step,
                                                   long long n_lo, int K, int lane, const float (&inv_rms)[GM_MP]) {
    for (int i = i_begin; i < i_end; i += i_step) {
        const long long n = n_lo + i / KB;
        const int uc = (int)(n / a.sch.nb), ub = (int)(n % a.sch.nb), kb = ub * KB + i % KB;
        if (kb < a.NB) gemv_stage_block(a, table + (size_t)i * GM_XREC, kb, K, lane, uc == 0, inv_rms);
    }
}

// The start of a CTA: all nine warps take the row norms (where the prologue has one) and then one or two records
// each, while the first copies are in flight.  The host uses this path only where a CTA streams at most eighteen
// K blocks, i.e. where two rounds cover the table: staging much more than that in the kernel delays the
// consumers' start by more than the separate staging kernel costs (it overlaps the tail of the kernel before
// it), and records written by the producer warp one unit ahead of its copies slow a two-stage ring down
// (both measured: 57344x8192 70.5 and 77.0 us against 69.1 us behind the staging kernel).
template <int KB>
__device__ __forceinline__ void gemv_stage_start(const GemvMmaArgs& a, uint8_t* table, int units_a, long long n_lo, int K,
                                                 float (*red)[GM_WARPS + 1], float (&inv_rms)[GM_MP]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (a.xmode == XP_RMSNORM || a.xmode == XP_ADD_NORM) {
        gemv_row_sumsq(a, K, red);
#pragma unroll
        for (int r = 0; r < GM_MP; ++r) {
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w <= GM_WARPS; ++w) tot += red[r][w];
            if (r < a.rows) inv_rms[r] = rsqrtf(tot / (float)K + a.eps);
        }
    }
    gemv_stage_records<KB>(a, table, warp, units_a * KB, GM_WARPS + 1, n_lo, K, lane, inv_rms);
    asm volatile("bar.sync 2, %0;" ::"n"(GM_THREADS) : "memory");
}

// KB = K blocks per ring stage (per unit).  Two halve the barrier hand-offs per byte where the tile
// cannot get wider (few column tiles, many K blocks).
// INK = the activation records come from this CTA's own table (in-kernel staging, PASSES == 1 only).
// PUSH = the finished outputs go into the ranks' exchange buffers (PeerPush) instead of local memory; a variant of
// its own so that the ordinary kernel's registers stay as they are.
template <int PASSES, int TC, int KB, bool INK = false, int FMT = GF_MSAQ_U4, bool PUSH = false>
__global__ void __launch_bounds__(GM_THREADS, GM_CTAS_PER_SM)
gemv_u4gs2_mma_kernel(const GemvMmaArgs a) {
    static_assert(!INK || PASSES == 1, "in-kernel staging serves launches of up to four rows");
    extern __shared__ __align__(128) uint8_t smem_all[];
    __shared__ __align__(8) uint64_t bar_full[GM_MAX_STAGES];
    __shared__ __align__(8) uint64_t bar_empty[GM_MAX_STAGES];
    __shared__ float norm_red[GM_MP][GM_WARPS + 1];
    __shared__ unsigned int marker_sh[GM_WARPS];               // each warp's (tile, warp) counter marker, fetched early

    constexpr int GROUPS = TC / GM_GROUP;
    constexpr int CB = gm_col_bytes(FMT);                      // bytes per (column, K block)
    constexpr int OFF_SH = TC * 16, OFF_SC = TC * (CB - 1), OFF_X = TC * CB;
    constexpr int SUB_BYTES = TC * CB + PASSES * GM_XREC;      // one K block of the tile with its activation record
    constexpr int STAGE_BYTES = KB * SUB_BYTES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    MSAQ_TR(1, 0, tid == 0);
#ifdef MSAQ_TRACE
    if (tid == 0 && blockIdx.x < 1024) { unsigned int sm; asm volatile("mov.u32 %0, %%smid;" : "=r"(sm)); g_trace[1][blockIdx.x][7] = sm; }
#endif
    const GemvSchedule sch = a.sch;
    float* const yf = a.y_f32;
    const long long n_lo = sch.lo(blockIdx.x), n_hi = sch.lo(blockIdx.x + 1);
    const int n_iter = (int)(n_hi - n_lo);
    int c = (int)(n_lo / sch.nb), blk = (int)(n_lo % sch.nb);
    const int K = a.NB * BLOCK;
    // In-kernel staging: the records live in a table in front of the ring (a.table_bytes of it), written once
    // by all warps; otherwise they arrive with each stage's copies from the staging kernel's output.
    constexpr bool stage_here = INK;
    uint8_t* const smem = smem_all + (INK ? a.table_bytes : 0);

    if (tid == 0) {
        for (int s = 0; s < sch.stages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), GM_WARPS);
        }
        mbar_init_fence();
    }
    __syncthreads();

    if (warp == GM_WARPS) {
        // ------------------------------ producer warp ------------------------------
        // With `early` (MSAQ_OPT_EARLY_WEIGHTS: the caller vouches that no kernel in flight writes the weight planes)
        // the first ring-full of weights goes out BEFORE the wait on the kernel in front (the staging kernel, or
        // whatever produced the activations): its run time and this kernel's pipeline fill overlap.  Only the
        // activation records (or, with in-kernel staging, the reads of the activations) wait.  Nothing is written
        // to global memory on this side of the wait.
        const bool inject = a.skip_stage >= 0 && blockIdx.x == 0;
        int s = 0, issued = 0;
        uint32_t ph = 1;                           // parity of the "previous" empty phase: passes at once on a fresh barrier
        int ci = c, bi = blk;                      // the next unit to issue
        // part 1: expect the whole stage and copy its weights; part 2: copy its activation records; 3: both
        auto issue = [&](int uc, int ub, int us, int part) {
            const int o0 = uc * TC, cv = min(TC, a.OUT - o0);
            const uint32_t bar = smem_u32(&bar_full[us]);
            const int b0 = ub * KB, nblk = min(KB, a.NB - b0);          // `ub` counts units within the tile
            if (part & 1) mbar_expect_tx(bar, (uint32_t)(nblk * (cv * CB + (stage_here ? 0 : PASSES * GM_XREC))));
#pragma unroll
            for (int j = 0; j < KB; ++j) {
                if (j < nblk) {
                    const uint32_t base = smem_u32(smem) + us * STAGE_BYTES + j * SUB_BYTES;
                    const int64_t col = (int64_t)(b0 + j) * a.OUT + o0;
                    if (part & 1) {
                        if constexpr (FMT == GF_MXINT8) {
                            bulk_g2s(base, a.upper_cm + col * 32, (uint32_t)cv * 32, bar);      // the int8 code plane
                        } else {
                            bulk_g2s(base, a.upper_cm + col * 16, (uint32_t)cv * 16, bar);
                            bulk_g2s(base + OFF_SH, a.shared_cm + col * 8, (uint32_t)cv * 8, bar);
                        }
                        bulk_g2s(base + OFF_SC, a.scale_exp + col, (uint32_t)cv, bar);
                    }
                    if (!stage_here && (part & 2))
                        bulk_g2s(base + OFF_X, a.xprep + (int64_t)(b0 + j) * PASSES * GM_XREC, (uint32_t)(PASSES * GM_XREC), bar);
                }
            }
        };
        int pre = min(sch.stages, n_iter);
        if (inject) pre = min(pre, a.skip_stage);
        if (!a.early) chain_wait();
        if (lane == 0) {
            int cj = ci, bj = bi;
            for (int it = 0; it < pre; ++it) {
                issue(cj, bj, it, 1);
                if (++bj == sch.nb) { bj = 0; ++cj; }
            }
        }
        MSAQ_TR(1, 1, lane == 0);
        if (a.early) chain_wait();
        MSAQ_TR(1, 2, lane == 0);
        if constexpr (INK) {
            // the whole warp helps with the records (the CTA-wide barrier at the end of that round orders them
            // before the consumers' reads)
            float inv_rms[GM_MP] = {1.0f, 1.0f, 1.0f, 1.0f};
            gemv_stage_start<KB>(a, smem_all, n_iter, n_lo, K, norm_red, inv_rms);
        }
        if (lane == 0) {
            for (int it = 0; it < pre; ++it) {
                if (!stage_here) issue(ci, bi, it, 2);
                if (++bi == sch.nb) { bi = 0; ++ci; }
            }
        }
        issued = pre;
        s = pre;
        if (s == sch.stages) { s = 0; ph ^= 1u; }
        // early: three quarters through its copies the block lets the kernels behind it be scheduled; their blocks take
        // the places of this kernel's blocks as those exit, and the next GEMV's fetch their first weights during this
        // kernel's tail (the release point hardly matters: 1/4, 1/2, 3/4 and "after the first ring" measured within 1 %)
        const int rel_it = a.early ? max(pre, 3 * n_iter / 4) : -1;
        if (lane == 0) {
            if (a.early && n_iter <= pre) chain_release();
            for (int it = pre; it < n_iter; ++it) {
                if (it == rel_it) chain_release();
                if (inject && it == a.skip_stage) break;          // the consumers' wait for this stage runs out
                if (!mbar_wait_bounded(smem_u32(&bar_empty[s]), ph, a.max_polls)) {
                    report_wait_failure(a.status, (int)a.tag, a.sticky, WAIT_FAIL_GEMV_MMA);
                    break;
                }
                ++issued;
                issue(ci, bi, s, 3);
                if (++bi == sch.nb) { bi = 0; ++ci; }
                if (++s == sch.stages) { s = 0; ph ^= 1u; }
            }
            // Leave only when every copy this thread issued has landed: shared memory must not be
            // handed to the next CTA with a copy still in flight (consumers that gave up do not wait).
            for (int i = max(0, issued - sch.stages); i < issued; ++i)
                mbar_wait_bounded(smem_u32(&bar_full[i % sch.stages]), (uint32_t)(i / sch.stages) & 1u, a.max_polls);
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    chain_wait();
    if constexpr (INK) {                                        // before anything of the main loop is live
        float inv_rms[GM_MP] = {1.0f, 1.0f, 1.0f, 1.0f};
        gemv_stage_start<KB>(a, smem_all, n_iter, n_lo, K, norm_red, inv_rms);
    }
    MSAQ_TR(1, 3, tid == 0);
    const int g = lane >> 2, t = lane & 3, h = t >> 1, odd = t & 1;
    const int r0 = warp * 16 + g;                            // group-local columns r0 and r0 + 8
    const uint32_t sel = odd ? 0x7531u : 0x6420u;            // bytes {odd, 2+odd} of both upper words
    const uint32_t nshift = odd * 4;
    const uint32_t sb = smem_u32(smem);
    const uint32_t aW = FMT == GF_MXINT8 ? sb + r0 * 32 + t * 4      // codes 4t..4t+3 of column r0
                                         : sb + r0 * 16 + h * 8;     // upper words 2h, 2h+1 of column r0
    const uint32_t aS = sb + OFF_SH + r0 * 8 + h * 4;        // shared word h
    const uint32_t aE = sb + OFF_SC + r0;
    // activation records: inside each stage (from the staging kernel), or in this CTA's table
    const uint32_t aB = (stage_here ? smem_u32(smem_all) : sb + OFF_X) + g * 32 + t * 8;
    const uint32_t aC = aB - g * 32 - t * 8 + 256 + t * 16;
    float acc[GROUPS][PASSES][2];
#pragma unroll
    for (int q = 0; q < GROUPS; ++q)
#pragma unroll
        for (int p = 0; p < PASSES; ++p) acc[q][p][0] = acc[q][p][1] = 0.0f;
    // A wait that gives up marks the warp aborted: it sets the status word, stops waiting and
    // computing, still releases its stages and still takes part in the tile hand-off, where its
    // outputs become NaN (directly, or through the status word the finishing warp reads).
    bool aborted = false;

    int s = 0;
    uint32_t ph = 0;
    for (int it = 0; it < n_iter; ++it) {
        // the (tile, warp) counter's marker, fetched long before the hand-off needs it and parked in shared memory
        if ((it == 0 || blk == 0) && lane == 0)
            marker_sh[warp] = *reinterpret_cast<volatile unsigned int*>(a.tile_counters + c * GM_WARPS + warp);
        if (!aborted && !mbar_wait_bounded(smem_u32(&bar_full[s]), ph, a.max_polls)) {
            report_wait_failure(a.status, (int)a.tag, a.sticky, WAIT_FAIL_GEMV_MMA);
            aborted = true;
        }
        MSAQ_TR(1, 4, tid == 0 && it == 0);
        const int cv = min(TC, a.OUT - c * TC);
        if (!aborted) {
            const int nblk = min(KB, a.NB - blk * KB);                      // `blk` counts units within the tile
            const int nq = (cv - warp * 16 + GM_GROUP - 1) / GM_GROUP;      // column groups this warp has in the tile
#pragma unroll
            for (int j = 0; j < KB; ++j) {
                if (j < nblk) {
                    const uint32_t so = s * STAGE_BYTES + j * SUB_BYTES;
                    const uint32_t ro = stage_here ? (uint32_t)((it * KB + j) * GM_XREC) : so;      // this K block's record
                    uint2 bq[PASSES];
                    int corr[PASSES];
                    float cx[PASSES];
#pragma unroll
                    for (int p = 0; p < PASSES; ++p) {
                        const uint32_t rb = aB + ro + p * GM_XREC;
                        bq[p] = lds64<0>(rb);
                        corr[p] = (int)lds32<0>(aC + ro + p * GM_XREC);
                        cx[p] = __uint_as_float(lds32<4>(aC + ro + p * GM_XREC));
                    }
                    const uint32_t wb = aW + so, sbs = aS + so, eb = aE + so;
                    if (nq >= GROUPS) gemv_groups<PASSES, 0, GROUPS, true, FMT>(nq, wb, sbs, eb, sel, nshift, bq, corr, cx, acc);
                    else gemv_groups<PASSES, 0, GROUPS, false, FMT>(nq, wb, sbs, eb, sel, nshift, bq, corr, cx, acc);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_empty[s]));
        if (++s == sch.stages) { s = 0; ph ^= 1u; }
        MSAQ_TR(1, 5, tid == 0 && it == n_iter - 1);

        // ---- end of this CTA's run over tile c: publish the partial, maybe finish the tile ----
        // Each warp owns 16 columns of every 128-column group of the tile, so the hand-off is
        // per warp: store the partial, count it on the (tile, warp) counter with release semantics, and
        // the warp that arrives last adds the slots up in slot order and writes the output.
        const bool tile_end = (blk == sch.nb - 1);
        if (tile_end || it == n_iter - 1) {
            const int first = sch.first_cta(c), nslots = sch.last_cta(c) - first + 1;
            const int slot = blockIdx.x - first, o0 = c * TC;
            const int nq = (cv - warp * 16 + GM_GROUP - 1) / GM_GROUP;     // groups in which this warp has columns
            if (aborted) {
                const float nan = __int_as_float(0x7FC00000);
#pragma unroll
                for (int q = 0; q < GROUPS; ++q)
#pragma unroll
                    for (int p = 0; p < PASSES; ++p) acc[q][p][0] = acc[q][p][1] = nan;
            }
            if (nq > 0) {
                if (nslots == 1) {
                    uint32_t seq = 0u;
                    if constexpr (PUSH) seq = gemv_push_seq(a.push);
#pragma unroll
                    for (int q = 0; q < GROUPS; ++q) {
                        if (q < nq) {
#pragma unroll
                            for (int p = 0; p < PASSES; ++p) {
                                const int m = p * GM_MP + t;
                                if (m < a.rows) {
                                    const int64_t o = (int64_t)(a.m0 + m) * a.OUT + o0 + q * GM_GROUP + r0;
                                    if constexpr (PUSH) {
                                        gemv_push(a.push, o, acc[q][p][0], seq);
                                        gemv_push(a.push, o + 8, acc[q][p][1], seq);
                                    } else {
                                        __nv_bfloat16 b0 = __float2bfloat16_rn(acc[q][p][0]), b1 = __float2bfloat16_rn(acc[q][p][1]);
                                        if (a.res) {       // the projection rounds to bf16 first, as the unfused add sees it
                                            b0 = __float2bfloat16_rn(__bfloat162float(a.res[o]) + __bfloat162float(b0));
                                            b1 = __float2bfloat16_rn(__bfloat162float(a.res[o + 8]) + __bfloat162float(b1));
                                        }
                                        a.y[o] = b0;
                                        a.y[o + 8] = b1;
                                        if (yf) { yf[o] = acc[q][p][0]; yf[o + 8] = acc[q][p][1]; }
                                    }
                                }
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < GROUPS; ++q) {
                        if (q < nq) {
#pragma unroll
                            for (int p = 0; p < PASSES; ++p) {
                                const int m = p * GM_MP + t;
                                if (m < a.rows) {
                                    float* dst = a.partial + ((int64_t)slot * a.rows + m) * a.OUT + o0 + q * GM_GROUP + r0;
                                    dst[0] = acc[q][p][0];
                                    dst[8] = acc[q][p][1];
                                }
                            }
                        }
                    }
                    __syncwarp();
                    unsigned int arrived = 0;
                    if (lane == 0) arrived = gemv_count_arrival(a, a.tile_counters + c * GM_WARPS + warp, marker_sh[warp]);
                    arrived = __shfl_sync(0xffffffffu, arrived, 0);
                    if (arrived == (unsigned int)nslots) {
                        __threadfence();
                        const bool poison = __ldcg(a.status) == (int)a.tag;        // a wait gave up somewhere in this call
                        uint32_t seq = 0u;
                        if constexpr (PUSH) seq = gemv_push_seq(a.push);
                        // An item is four adjacent outputs (row m, group q, quad of the warp's 16 columns); 32 / S items are
                        // in hand at a time, S lanes to an item, lane `part` adding the slots part, part + S, ... with eight
                        // 16-byte loads in flight, then the S sums are added across lanes: one or two rounds of load latency
                        // where one output per lane and eight scalar loads in flight took four to eight.  The order of the
                        // additions depends on the shape alone, so the sum is the same bits on every run.
                        const int64_t sstride4 = (int64_t)a.rows * a.OUT / 4;           // slot stride in float4 (OUT % 16 == 0)
                        const int items = a.rows * nq * 4;
                        int S = 1;
                        while (S < 8 && items * S * 2 <= 32) S *= 2;
                        const int per = 32 / S;
                        for (int base = 0; base < items; base += per) {
                            const int it = base + lane / S, part = lane % S;
                            const bool live = it < items;
                            const int m = live ? it / (nq * 4) : 0, rem = live ? it % (nq * 4) : 0;
                            const int64_t e = (int64_t)m * a.OUT + o0 + (rem >> 2) * GM_GROUP + warp * 16 + (rem & 3) * 4;
                            const float4* src = reinterpret_cast<const float4*>(a.partial + e);
                            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                            if (live) {
                                for (int k0 = part; k0 < nslots; k0 += 8 * S) {
                                    float4 v[8];
#pragma unroll
                                    for (int k = 0; k < 8; ++k)
                                        v[k] = (k0 + k * S < nslots) ? __ldcg(src + (k0 + k * S) * sstride4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                                    for (int k = 0; k < 8; ++k) { sum.x += v[k].x; sum.y += v[k].y; sum.z += v[k].z; sum.w += v[k].w; }
                                }
                            }
                            for (int o = S >> 1; o; o >>= 1) {
                                sum.x += __shfl_xor_sync(0xffffffffu, sum.x, o);
                                sum.y += __shfl_xor_sync(0xffffffffu, sum.y, o);
                                sum.z += __shfl_xor_sync(0xffffffffu, sum.z, o);
                                sum.w += __shfl_xor_sync(0xffffffffu, sum.w, o);
                            }
                            if (live && part == 0) {
                                if (poison) sum.x = sum.y = sum.z = sum.w = __int_as_float(0x7FC00000);
                                const int64_t y0 = (int64_t)a.m0 * a.OUT + e;
                                if constexpr (PUSH) {
                                    gemv_push(a.push, y0, sum.x, seq);
                                    gemv_push(a.push, y0 + 1, sum.y, seq);
                                    gemv_push(a.push, y0 + 2, sum.z, seq);
                                    gemv_push(a.push, y0 + 3, sum.w, seq);
                                } else {
                                    if (yf) *reinterpret_cast<float4*>(yf + y0) = sum;
                                    if (a.res) {           // the projection rounds to bf16 first, as the unfused add sees it
                                        const uint2 rb = *reinterpret_cast<const uint2*>(a.res + y0);
                                        sum.x = bf16_lo(rb.x) + __bfloat162float(__float2bfloat16_rn(sum.x));
                                        sum.y = bf16_hi(rb.x) + __bfloat162float(__float2bfloat16_rn(sum.y));
                                        sum.z = bf16_lo(rb.y) + __bfloat162float(__float2bfloat16_rn(sum.z));
                                        sum.w = bf16_hi(rb.y) + __bfloat162float(__float2bfloat16_rn(sum.w));
                                    }
                                    __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x, sum.y), hi = __floats2bfloat162_rn(sum.z, sum.w);
                                    uint2 ob;
                                    ob.x = *reinterpret_cast<uint32_t*>(&lo);
                                    ob.y = *reinterpret_cast<uint32_t*>(&hi);
                                    *reinterpret_cast<uint2*>(a.y + y0) = ob;
                                }
                            }
                        }
                        // back to zero at rest: the next call (or the next replay of this launch) counts from 0 again
                        if (lane == 0) reinterpret_cast<unsigned int*>(a.tile_counters + c * GM_WARPS + warp)[1] = 0u;
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < GROUPS; ++q)
#pragma unroll
                for (int p = 0; p < PASSES; ++p) acc[q][p][0] = acc[q][p][1] = 0.0f;
        }
        if (++blk == sch.nb) { blk = 0; ++c; }
    }
    MSAQ_TR(1, 6, tid == 0);
}

}  // namespace msaq

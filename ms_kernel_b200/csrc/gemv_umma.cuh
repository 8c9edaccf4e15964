// Weight-only GEMV on the fifth-generation tensor cores, Y[M][OUT] = X[M][K] * dequant(W)^T, in
// tiles of up to 128 activation rows: u = 4, gs = 2 from nine rows up, and the 5+3 and 6+2 bit
// formats (u = 3, u = 2 at gs = 2) at every batch size.
//
// At these batch sizes the work is a real contraction, so it goes to tcgen05.mma with the
// accumulator in tensor memory.  The weights stay packed in HBM (25 to 29 bytes per 32-block)
// and are widened on the way:
//   * a producer warp streams the packed bytes of a (512 weight rows x one K block)
//     unit, and the matching bf16 activation tile, into a shared-memory ring with TMA
//     bulk copies (cp.async.bulk + mbarrier);
//   * sixteen decode warps in two teams that take alternate units, two weight rows per
//     thread, turn the 32 codes of a row's block into the exact bf16 values q * 2^e
//     (q = up * 2^u + sh is an 8-bit integer, so the product is representable) and store them
//     as the B operand in the core-matrix layout tcgen05 reads (K-major, no swizzle);
//   * two issuing threads, each owning 256 weight rows (256 accumulator columns) of every
//     unit, issue 2 K steps each of
//     tcgen05.mma.cta_group::1.kind::f16  D[128 x 256] += A[128 x 16] * B[256 x 16]^T
//     with A = activations (rows beyond M are zero) and B = 256 weight rows -- an MMA costs
//     about 135 cycles to issue whatever its N, so the weights take the wide side -- fp32
//     accumulation in tensor memory (all 512 columns) across the CTA's whole K range;
//     tcgen05.commit hands the shared-memory buffers back to the decoders and the ring;
//   * at the end of a row tile the decode warps read the accumulators back with
//     tcgen05.ld and store bf16 outputs, or fp32 split-K partials that a second, fully
//     parallel kernel sums in slot order.
// Unlike the integer path (gemv_mma.cuh) nothing is quantised on the activation side: the
// products bf16 x bf16 are exact in fp32.
//
// Every wait is bounded; a wait that gives up sets the status word and an abort flag, all
// roles drain without touching tensor memory again, the allocation is returned, and the
// outputs of the launch are marked NaN by the combine.
//
// Algorithm replaced: csrc/w_gemv.cu:417-487 (batched kernel) and the wmma fallback
// csrc/wa_gemm.cu:878-943 of the reference.
#pragma once

#include "gemv_mma.cuh"

namespace msaq {

constexpr int GU_TR = 512;                         // weight rows per tile
constexpr int GU_DEC_WARPS = 16;                   // one thread per weight row
constexpr int GU_WARP_TMA = GU_DEC_WARPS;          // warp 16: TMA producer
constexpr int GU_WARP_MMA = GU_DEC_WARPS + 1;      // warps 17, 18: MMA issuers (17 also owns the tensor-memory allocation)
constexpr int GU_ISSUERS = 2;                      // issuer g accumulates weight rows 256g..256g+255 (columns 256g.. of tensor memory)
constexpr int GU_THREADS = (GU_DEC_WARPS + 1 + GU_ISSUERS) * 32;
constexpr int GU_MAX_N = 128;                      // activation rows per launch: the M of the MMA
constexpr int GU_MAX_STAGES = 8;
constexpr int GU_ABUF_BYTES = GU_TR * 64;          // one decoded weight buffer: 512 rows x 32 bf16
constexpr int GU_ABUFS = 2;                        // one per decode team (two per team measured no faster and halve the ring)
constexpr int GU_XTILE = GU_MAX_N * 64;            // activation tile of a K block: 128 rows x 32 bf16
// gs = 2 formats: upper codes 4*(8-u) bytes, shared codes 2*u bytes, one scale byte per (row, block)
__host__ __device__ constexpr int gu_ub(int u) { return 4 * (8 - u); }
__host__ __device__ constexpr int gu_sb(int u) { return 2 * u; }
__host__ __device__ constexpr int gu_packed(int u) { return GU_TR * (gu_ub(u) + gu_sb(u) + 1); }   // packed bytes of a unit
__host__ __device__ constexpr int gu_stage(int u) { return gu_packed(u) + GU_XTILE; }
constexpr int GU_TMEM_COLS = GU_TR;                // one fp32 accumulator column per weight row of the tile

// ---- tcgen05 wrappers -----------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Arrive on `bar` once every tcgen05 operation this thread issued so far has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate == 0 overwrites D.  The two matrix
// descriptors arrive as 32-bit halves: the upper half is the same for every MMA of the kernel,
// the lower half moves with the operand's address, so the issuing thread spends one add per operand.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 16 consecutive accumulator columns of this warp's 32 lanes.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices of 128
// contiguous bytes; `lbo` is the byte distance between core matrices adjacent in K, `sbo`
// between core matrices adjacent in the row direction.  Bits 46-47 = 1: sm_100 descriptor.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t saddr, uint32_t lbo) {
    return ((saddr >> 4) & 0x3FFFu) | (((lbo >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ uint32_t umma_desc_hi(uint32_t sbo) { return ((sbo >> 4) & 0x3FFFu) | (1u << 14); }
// Instruction descriptor of kind::f16: fp32 accumulator, bf16 A and B, both K-major, M = 128, N = n.
__host__ __device__ inline uint32_t umma_idesc_bf16(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// ---- activation staging ----------------------------------------------------------
// X [M][K] bf16 row-major -> per K block the first ceil(M/8) row groups of an A-operand tile in the
// core-matrix layout (row n, 8-value chunk c at ((n/8)*4 + c)*128 + (n%8)*16); rows M..8*ceil(M/8)-1 zero.
// Also clears the status word of the launch that follows.
__host__ __device__ inline int gu_xtile_bytes(int rows) { return ((rows + 7) / 8) * 512; }   // whole 8-row groups

__global__ void __launch_bounds__(256)
gemv_umma_xprep_kernel(const __nv_bfloat16* __restrict__ X, uint8_t* __restrict__ xs, int* __restrict__ status,
                       int reset_status, int M, int NB) {
    chain_release();
    chain_wait();
    const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (reset_status && gtid == 0) *status = 0;
    const int N = ((M + 7) / 8) * 8;                         // rows staged per block (the kernel keeps the rest of its tile zero)
    const int64_t total = (int64_t)NB * N * 4;
    if (gtid >= total) return;
    const int c = (int)(gtid & 3), n = (int)((gtid >> 2) % N), b = (int)(gtid / (4 * N));
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (n < M) {
        const __nv_bfloat16* src = X + (int64_t)n * NB * BLOCK + b * BLOCK + c * 8;
        if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            v = *reinterpret_cast<const uint4*>(src);
        } else {
            const uint16_t* s16 = reinterpret_cast<const uint16_t*>(src);
            v.x = s16[0] | ((uint32_t)s16[1] << 16);
            v.y = s16[2] | ((uint32_t)s16[3] << 16);
            v.z = s16[4] | ((uint32_t)s16[5] << 16);
            v.w = s16[6] | ((uint32_t)s16[7] << 16);
        }
    }
    *reinterpret_cast<uint4*>(xs + (int64_t)b * N * 64 + ((n >> 3) * 4 + c) * 128 + (n & 7) * 16) = v;
}

// ---- decode of one weight row's 32-block into bf16 ---------------------------------------
// The row's 64 bytes go to `dst` + i*128, i = 0..3 (8-value chunks of the core-matrix layout).
//
// v = q * 2^e with q = up * 2^u + sh.  Flipping the sign bit of a two's-complement field makes it
// offset binary, so (up_off << u) + sh_off = q + 128 + 2^(u-1) is a non-negative integer; added to
// the bit pattern of 2^23 it reads as the float 2^23 + q + 128 + 2^(u-1), and one FMA removes the
// offsets and applies the scale exactly.  q * 2^e has at most 8 significant bits, so the upper half
// of the fp32 word is the bf16 value.
template <int U>
__device__ __forceinline__ void gu_decode_row(uint32_t st, int r, uint32_t dst);

// u = 4: nibbles.  A nibble in the high half of a byte and the shared nibble in the low half form
// the byte q + 136 with three logic ops per eight codes; a byte permute drops it into the mantissa.
template <>
__device__ __forceinline__ void gu_decode_row<4>(uint32_t st, int r, uint32_t dst) {
    const uint4 w = lds128(st + r * 16);
    const uint2 sh = lds64<0>(st + GU_TR * 16 + r * 8);
    const int e = lds_s8<0>(st + GU_TR * 24 + r);
    const float sc = __int_as_float(max(0, e + 127) << 23);
    const float off = -8388744.0f * sc;
    const uint32_t wx[4] = {w.x ^ 0x88888888u, w.y ^ 0x88888888u, w.z ^ 0x88888888u, w.w ^ 0x88888888u};
    const uint32_t sx[2] = {sh.x ^ 0x88888888u, sh.y ^ 0x88888888u};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // the four shared codes of elements 8i..8i+7 (two elements each), one per byte
        const uint32_t s16 = (i & 1) ? (sx[i >> 1] >> 16) : sx[i >> 1];
        const uint32_t t = prmt(s16, 0u, 0x1100u);
        const uint32_t lo = and_or(t >> 4, 0x0F000F00u, t & 0x000F000Fu);
        const uint32_t me = and_or(wx[i] << 4, 0xF0F0F0F0u, lo);      // elements 8i + 0, 2, 4, 6
        const uint32_t mo = and_or(wx[i], 0xF0F0F0F0u, lo);           // elements 8i + 1, 3, 5, 7
        uint32_t o[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float fe = __uint_as_float(prmt(me, 0x4B000000u, 0x7650u + b));
            const float fo = __uint_as_float(prmt(mo, 0x4B000000u, 0x7650u + b));
            const float ve = fmaf(fe, sc, off), vo = fmaf(fo, sc, off);
            o[b] = prmt(__float_as_uint(ve), __float_as_uint(vo), 0x7632u);
        }
        sts128(dst + i * 128, o[0], o[1], o[2], o[3]);
    }
}

// Bits [32*i, 32*i+32) of the pattern that has the top bit of every `width`-bit field set.
__host__ __device__ constexpr uint32_t gu_sign_pattern(int width, int i) {
    uint32_t p = 0;
    for (int b = width - 1; b < 32 * (i + 1); b += width)
        if (b >= 32 * i) p |= 1u << (b - 32 * i);
    return p;
}

// u = 3 (5-bit upper, 3-bit shared) and u = 2 (6-bit, 2-bit): fields cut out of the dense bit runs
// with funnel shifts.
template <int U>
__device__ __forceinline__ void gu_decode_row(uint32_t st, int r, uint32_t dst) {
    constexpr int WB = 8 - U, NW = WB;                          // field width, words of the upper run
    constexpr uint32_t UM = (1u << WB) - 1u, SM = (1u << U) - 1u;
    uint32_t w[NW + 1];
    if (U == 3) {
#pragma unroll
        for (int i = 0; i < NW; ++i) w[i] = lds32<0>(st + r * 20 + i * 4);
    } else {
#pragma unroll
        for (int i = 0; i < NW; i += 2) {
            const uint2 v = lds64<0>(st + r * 24 + i * 4);
            w[i] = v.x;
            w[i + 1] = v.y;
        }
    }
#pragma unroll
    for (int i = 0; i < NW; ++i) w[i] ^= gu_sign_pattern(WB, i);
    w[NW] = 0u;
    uint32_t s0, s1 = 0u;                                       // shared run: 16 fields of U bits
    const uint32_t sbase = st + GU_TR * gu_ub(U) + r * gu_sb(U);
    if (U == 2) {
        s0 = lds32<0>(sbase);
    } else {
        uint32_t a, b, c;
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(a) : "r"(sbase));
        asm volatile("ld.shared.u16 %0, [%1+2];" : "=r"(b) : "r"(sbase));
        asm volatile("ld.shared.u16 %0, [%1+4];" : "=r"(c) : "r"(sbase));
        s0 = a | (b << 16);
        s1 = c;
    }
    s0 ^= gu_sign_pattern(U, 0);
    s1 ^= gu_sign_pattern(U, 1) & 0xFFFFu;
    const int e = lds_s8<0>(st + GU_TR * (gu_ub(U) + gu_sb(U)) + r);
    const float sc = __int_as_float(max(0, e + 127) << 23);
    const float off = -(8388608.0f + 128.0f + (float)(1 << (U - 1))) * sc;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t o[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int g = 4 * i + b, ps = g * U;                  // group: elements 2g, 2g+1
            const uint32_t sf = (ps + U <= 32) ? (s0 >> ps) : (ps >= 32 ? (s1 >> (ps - 32)) : __funnelshift_r(s0, s1, ps));
            const uint32_t shm = and_or(sf, SM, 0x4B000000u);     // shared code on top of the bits of 2^23
            float v[2];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const int pk = (2 * g + t) * WB, wi = pk >> 5, po = pk & 31;
                const uint32_t uf = (po + WB <= 32) ? (w[wi] >> po) : __funnelshift_r(w[wi], w[wi + 1], po);
                v[t] = fmaf(__uint_as_float(((uf & UM) << U) + shm), sc, off);
            }
            o[b] = prmt(__float_as_uint(v[0]), __float_as_uint(v[1]), 0x7632u);
        }
        sts128(dst + i * 128, o[0], o[1], o[2], o[3]);
    }
}

// ---- main kernel --------------------------------------------------------------------
struct GemvUmmaArgs {
    const int8_t* scale_exp;
    const uint8_t* upper_cm;
    const uint8_t* shared_cm;
    const uint8_t* xs;       // staged activation tiles [NB][gu_xtile_bytes(rows)]
    float* partial;          // [max_slots][rows][OUT]
    int* status;
    int* sticky;             // the library's per-device status word (may be null)
    __nv_bfloat16* y;        // [M][OUT]
    float* y_f32;            // optional
    int m0, rows;            // this launch covers activation rows [m0, m0 + rows), rows <= 128
    int OUT;
    GemvSchedule sch;        // tc = 512, grid = one CTA per SM
};


template <int U>
__global__ void __launch_bounds__(GU_THREADS, 1)
gemv_umma_kernel(const GemvUmmaArgs a) {
    constexpr int GU_PACKED = gu_packed(U);
    extern __shared__ __align__(128) uint8_t gu_smem[];
    __shared__ __align__(8) uint64_t bar_full[GU_MAX_STAGES];     // packed unit + activation tile landed (TMA)
    __shared__ __align__(8) uint64_t bar_empty[GU_MAX_STAGES];    // the owning team's 8 warps have read the packed bytes and both issuers' MMAs the activation tile
    __shared__ __align__(8) uint64_t bar_afull[GU_ABUFS];                // decoded weight buffer written (the 8 warps of its team)
    __shared__ __align__(8) uint64_t bar_aempty[GU_ABUFS];               // MMAs that read the buffer completed (one commit per issuer)
    __shared__ __align__(8) uint64_t bar_accfull;                 // the tile's last MMAs completed (one commit per issuer)
    __shared__ __align__(8) uint64_t bar_accempty;                // 16 warps have read the accumulators
    __shared__ __align__(8) uint64_t bar_done;                    // teardown: every MMA issued has completed
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const GemvSchedule sch = a.sch;
    const int stages = sch.stages;
    constexpr int STAGE = gu_stage(U);
    const uint32_t smem0 = smem_u32(gu_smem);
    const uint32_t abuf0 = smem0 + stages * STAGE;                 // the decoded weight buffers behind the ring
    constexpr uint32_t tmem_cols = GU_TMEM_COLS;
    const long long n_lo = sch.lo(blockIdx.x), n_hi = sch.lo(blockIdx.x + 1);
    const int n_iter = (int)(n_hi - n_lo);
    const int c_first = (int)(n_lo / sch.nb), blk_first = (int)(n_lo % sch.nb);

    // The MMA always reads a 128-row activation tile; the TMA copies only the row groups that hold
    // rows of this launch, the rest of every stage's tile is zeroed here once.
    const int xbytes = gu_xtile_bytes(a.rows);
    for (int s = 0; s < stages; ++s)
        for (int i = xbytes + tid * 16; i < GU_XTILE; i += GU_THREADS * 16)
            *reinterpret_cast<uint4*>(gu_smem + s * STAGE + GU_PACKED + i) = make_uint4(0u, 0u, 0u, 0u);
    fence_async_smem();
    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), GU_DEC_WARPS / 2 + GU_ISSUERS);
        }
        for (int j = 0; j < GU_ABUFS; ++j) {
            mbar_init(smem_u32(&bar_afull[j]), GU_DEC_WARPS / 2);
            mbar_init(smem_u32(&bar_aempty[j]), GU_ISSUERS);
        }
        mbar_init(smem_u32(&bar_accfull), GU_ISSUERS);
        mbar_init(smem_u32(&bar_accempty), GU_DEC_WARPS);
        mbar_init(smem_u32(&bar_done), GU_ISSUERS);
        abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == GU_WARP_MMA) {
        tmem_alloc(smem_u32(&tmem_slot), tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    chain_wait();                                   // activations, counters and workspace belong to earlier kernels until here

    if (warp == GU_WARP_TMA) {
        // -------------------------------- TMA producer --------------------------------
        // The whole warp runs the loop; lanes 0..3 each issue one of a unit's four copies in the same
        // instruction (a lone thread needed about 1000 cycles per unit for them, more than the rest
        // of the pipeline needs to consume one).
        const uint8_t* src_base = lane == 0 ? a.upper_cm : lane == 1 ? a.shared_cm
                                 : lane == 2 ? reinterpret_cast<const uint8_t*>(a.scale_exp) : a.xs;
        const int per_col = lane == 0 ? gu_ub(U) : lane == 1 ? gu_sb(U) : 1;            // bytes per (row, block) of this lane's plane
        const uint32_t dst_off = lane == 0 ? 0u : lane == 1 ? (uint32_t)(GU_TR * gu_ub(U))
                               : lane == 2 ? (uint32_t)(GU_TR * (gu_ub(U) + gu_sb(U))) : (uint32_t)GU_PACKED;
        int c = c_first, blk = blk_first, s = 0;
        uint32_t ph = 1;                            // passes at once on a fresh barrier
        for (int it = 0; it < n_iter; ++it) {
            bool stop = abort_flag != 0;
            if (!stop && !mbar_wait_bounded(smem_u32(&bar_empty[s]), ph)) {
                report_wait_failure(a.status, 1, a.sticky, WAIT_FAIL_GEMV_UMMA);
                abort_flag = 1;
                stop = true;
            }
            if (__any_sync(0xffffffffu, stop)) break;
            const int o0 = c * GU_TR, cv = min(GU_TR, a.OUT - o0);
            const uint32_t bar = smem_u32(&bar_full[s]);
            const uint32_t base = smem0 + s * STAGE;
            const int64_t col = (int64_t)blk * a.OUT + o0;
            if (lane == 0) mbar_expect_tx(bar, (uint32_t)(cv * (gu_ub(U) + gu_sb(U) + 1) + xbytes));
            __syncwarp();
            if (lane < 3) bulk_g2s(base + dst_off, src_base + col * per_col, (uint32_t)(cv * per_col), bar);
            else if (lane == 3) bulk_g2s(base + dst_off, src_base + (int64_t)blk * xbytes, (uint32_t)xbytes, bar);
            if (++blk == sch.nb) { blk = 0; ++c; }
            if (++s == stages) { s = 0; ph ^= 1u; }
        }
    } else if (warp >= GU_WARP_MMA) {
        // -------------------------------- MMA issuers --------------------------------
        // Two threads in two warps, each with its own half of the accumulator columns: one thread's
        // barrier polling and commit latency overlaps the other's MMAs.
        const int g = warp - GU_WARP_MMA;                          // this issuer's 256 weight rows of every unit
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(256), desc_hi = umma_desc_hi(512);
            int c = c_first, blk = blk_first, s = 0;
            uint32_t aph = 0u, accph = 1;                         // accph: "accumulators free" passes at once the first time
            bool fresh = true;                                    // next MMA starts a tile: overwrite the accumulators
            for (int it = 0; it < n_iter && !abort_flag; ++it) {
                const int buf = it & (GU_ABUFS - 1);
                // The decoders arrive on the A buffer only after they saw the stage's TMA data land, so
                // this one wait also covers the activation tile of the stage.
                bool ok = mbar_wait_bounded(smem_u32(&bar_afull[buf]), (aph >> buf) & 1u);
                if (ok && fresh) ok = mbar_wait_bounded(smem_u32(&bar_accempty), accph);
                if (!ok) {
                    report_wait_failure(a.status, 1, a.sticky, WAIT_FAIL_GEMV_UMMA);
                    abort_flag = 1;
                    break;
                }
                if (fresh) accph ^= 1u;
                aph ^= 1u << buf;
                tc_fence_after();
                const int cv = min(GU_TR, a.OUT - c * GU_TR);
                const uint32_t w_lo = umma_desc_lo(abuf0 + buf * GU_ABUF_BYTES, 128);     // B operand: decoded weights
                const uint32_t x_lo = umma_desc_lo(smem0 + s * STAGE + GU_PACKED, 128);   // A operand: activation tile
                if (g * 256 < cv) {
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks)
                        umma_f16(tmem_base + g * 256, x_lo + ((ks * 256) >> 4), w_lo + ((g * (256 * 64) + ks * 256) >> 4),
                                 desc_hi, idesc, (fresh && ks == 0) ? 0u : 1u);
                }
                fresh = false;
                tc_commit(smem_u32(&bar_aempty[buf]));            // its team may overwrite this decoded buffer
                tc_commit(smem_u32(&bar_empty[s]));               // the ring may overwrite the activation tile
                if (blk == sch.nb - 1 || it == n_iter - 1) {
                    tc_commit(smem_u32(&bar_accfull));            // the tile's accumulators are final
                    fresh = true;
                }
                if (++blk == sch.nb) { blk = 0; ++c; }
                if (++s == stages) s = 0;
            }
        }
    } else {
        // ---------------------------- decode + epilogue warps ----------------------------
        // Two teams of eight warps take alternate units (team t: units t, t+2, ...; decoded buffer t),
        // two weight rows per thread, so that one team's waits and fences overlap the other's arithmetic.
        // All sixteen warps read the accumulators back at the end of a tile segment.
        const int team = warp >> 3, tt = tid & 255;
        const int cg = warp >> 2, q = warp & 3;                    // epilogue: column group, tensor-memory lane quarter
        bool aborted = false;

        // epilogue of the segment of tile `c` (this CTA's run over that tile), in unit order
        int seg_c = c_first, seg_end = min(sch.nb - 1 - blk_first, n_iter - 1);
        uint32_t accfph = 0;
        auto epilogue = [&]() {
            const int c = seg_c;
            const int first = sch.first_cta(c), nslots = sch.last_cta(c) - first + 1;
            const int slot = blockIdx.x - first, o0 = c * GU_TR;
            const int cv = min(GU_TR, a.OUT - o0);
            if (!aborted && abort_flag) aborted = true;
            if (!aborted && !mbar_wait_bounded(smem_u32(&bar_accfull), accfph)) {
                report_wait_failure(a.status, 1, a.sticky, WAIT_FAIL_GEMV_UMMA);
                abort_flag = 1;
                aborted = true;
            }
            aborted = __any_sync(0xffffffffu, aborted);            // one decision per warp: the tensor-memory loads are warp-wide
            accfph ^= 1u;
            // accumulator lane = activation row, column = weight row of the tile: warp (q, cg) reads
            // rows 32q..32q+31, columns 128cg..128cg+127
            const int m = q * 32 + lane;
            if (!aborted) {
                tc_fence_after();
                if (q * 32 < a.rows) {
                    for (int n0 = 0; n0 < 128; n0 += 16) {
                        const int col = cg * 128 + n0;
                        if (col >= cv) break;
                        float v[16];
                        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + col, v);
                        if (m < a.rows) {
                            if (nslots == 1) {
                                const int64_t o = (int64_t)(a.m0 + m) * a.OUT + o0 + col;
                                uint32_t pk[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                                    pk[i] = *reinterpret_cast<const uint32_t*>(&h2);
                                }
                                uint4* dst = reinterpret_cast<uint4*>(a.y + o);
                                dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                                dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                                if (a.y_f32) {
                                    float4* df = reinterpret_cast<float4*>(a.y_f32 + o);
#pragma unroll
                                    for (int i = 0; i < 4; ++i) df[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                                }
                            } else {
                                float4* dp = reinterpret_cast<float4*>(a.partial + ((int64_t)slot * a.rows + m) * a.OUT + o0 + col);
#pragma unroll
                                for (int i = 0; i < 4; ++i) dp[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                            }
                        }
                    }
                }
                tc_fence_before();
            } else if (nslots == 1 && m < a.rows) {
                // abandoned: the outputs this warp owns are marked, not left stale
                for (int col = cg * 128; col < min(cv, cg * 128 + 128); ++col) {
                    const int64_t o = (int64_t)(a.m0 + m) * a.OUT + o0 + col;
                    a.y[o] = __float2bfloat16_rn(__int_as_float(0x7FC00000));
                    if (a.y_f32) a.y_f32[o] = __int_as_float(0x7FC00000);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_accempty));
            ++seg_c;
            seg_end = min(seg_end + sch.nb, n_iter - 1);
        };

        int s = team % stages;                                     // ring stage of this team's current unit
        uint32_t ph = (uint32_t)((team / stages) & 1), aeph = 3u; // aeph: one parity bit per buffer of the team
        for (int it = team; it < n_iter; it += 2) {
            const int buf = it & (GU_ABUFS - 1), bsel = (it >> 1) & (GU_ABUFS / 2 - 1);   // this unit's decoded buffer; which of the team's own
            while (seg_end < it) epilogue();                       // segments that ended before this unit
            if (!aborted && abort_flag) aborted = true;
            if (!aborted) {
                bool ok = mbar_wait_bounded(smem_u32(&bar_full[s]), ph);
                ok = ok && mbar_wait_bounded(smem_u32(&bar_aempty[buf]), (aeph >> bsel) & 1u);
                if (!ok) {
                    report_wait_failure(a.status, 1, a.sticky, WAIT_FAIL_GEMV_UMMA);
                    abort_flag = 1;
                    aborted = true;
                }
            }
            aborted = __any_sync(0xffffffffu, aborted);
            aeph ^= 1u << bsel;
            if (!aborted) {
                const uint32_t st = smem0 + s * STAGE;
#pragma unroll 1
                for (int half = 0; half < 2; ++half) {
                    const int r = tt + half * 256;                 // weight row within the tile
                    gu_decode_row<U>(st, r, abuf0 + buf * GU_ABUF_BYTES + (r >> 3) * 512 + (r & 7) * 16);
                }
                fence_async_smem();                               // the tensor core reads the buffer through the async proxy
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&bar_afull[buf]));
                mbar_arrive(smem_u32(&bar_empty[s]));             // this team is done with the packed bytes of the stage
            }
            s += 2;
            if (s >= stages) { s -= stages; ph ^= 1u; }
        }
        while (seg_c <= (int)((n_hi - 1) / sch.nb)) epilogue();    // the segments still open, the last one included
    }

    // ---- teardown: nothing may still be writing tensor memory when it is returned ----
    tc_fence_before();
    __syncthreads();
    if (warp >= GU_WARP_MMA && lane == 0) tc_commit(smem_u32(&bar_done));   // arrives once this issuer's MMAs have completed
    if (warp == GU_WARP_MMA) {
        if (lane == 0 && !mbar_wait_bounded(smem_u32(&bar_done), 0)) report_wait_failure(a.status, 1, a.sticky, WAIT_FAIL_GEMV_UMMA);
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

// Sum of the split-K partials of the tensor-memory kernel, in slot order: one thread per four
// consecutive outputs of one activation row.  Tiles that one CTA covered alone were written by
// that CTA and are skipped.  A set status word (a wait gave up) marks the whole launch NaN.
__global__ void __launch_bounds__(256)
gemv_umma_combine_kernel(const float* __restrict__ partial, const int* __restrict__ status, __nv_bfloat16* __restrict__ y,
                         float* __restrict__ y_f32, GemvSchedule sch, int m0, int rows, int OUT) {
    chain_release();
    chain_wait();
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int quads = OUT / 4;
    if (idx >= (int64_t)rows * quads) return;
    const int m = (int)(idx / quads), col = (int)(idx % quads) * 4, c = col / GU_TR;
    const int first = sch.first_cta(c), nslots = sch.last_cta(c) - first + 1;
    const bool poison = *status != 0;
    if (nslots == 1 && !poison) return;
    const int64_t sstride = (int64_t)rows * OUT;
    const float* src = partial + (int64_t)m * OUT + col;
    float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (!poison) {
        for (int k0 = 0; k0 < nslots; k0 += 8) {
            float4 pv[8];
#pragma unroll
            for (int k = 0; k < 8; ++k)
                pv[k] = (k0 + k < nslots) ? __ldcg(reinterpret_cast<const float4*>(src + (k0 + k) * sstride))
                                          : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int k = 0; k < 8; ++k) { sum.x += pv[k].x; sum.y += pv[k].y; sum.z += pv[k].z; sum.w += pv[k].w; }
        }
    } else {
        sum.x = sum.y = sum.z = sum.w = __int_as_float(0x7FC00000);
    }
    const int64_t o = (int64_t)(m0 + m) * OUT + col;
    const __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x, sum.y), hi = __floats2bfloat162_rn(sum.z, sum.w);
    *reinterpret_cast<uint2*>(y + o) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    if (y_f32) *reinterpret_cast<float4*>(y_f32 + o) = sum;
}

}  // namespace msaq

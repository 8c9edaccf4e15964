// Tuned split-KV flash-decode for u = 4, gs = 2, head_dim 128, G = Hq/Hkv in {1,2,4,8}.
//
// One CTA = (key tile, kv head, sequence) and serves all G query heads of that kv
// head, so every packed code is fetched and decoded once.
//   * A producer thread streams 128-key stages of the K and V planes (upper codes,
//     shared codes, scale bytes) into a shared-memory ring with TMA bulk copies.
//   * Four consumer warps take 32 keys of each stage.  Q.K^T is the GEMV data flow:
//     nibbles become int8 MMA operands with three logic ops per word, the query is
//     staged once per CTA as 16-bit block fixed point, one m16n8k32 integer MMA
//     gives the exact integer dot of 16 keys x one 32-block against four heads.
//   * Online softmax per warp in the exp2 domain; probabilities go through shared
//     memory once to change from the (key, head) to the (head, key) register layout.
//   * P.V contracts over keys: ldmatrix.m16n16.trans.b8 delivers V bytes with four
//     keys per register (one d-pair per byte), the probabilities -- pre-multiplied by
//     each key's block scale relative to the chunk maximum -- are 16-bit fixed-point
//     A operands, and the integer result is rescaled once per 32 keys and block.
//   * Each warp keeps its own (m, l, acc); the warps of a CTA merge through shared
//     memory, the tiles of a head through the combine kernel.
//
// Algorithm replaced: csrc/kv_attention.cu:450-829 (kv_decode_wide_kernel) of the
// reference, including its fused query rotation (:485-498).
#pragma once

#include "kv_quant_row.cuh"
#include "kv_decode_generic.cuh"
#include "sm100_ptx.cuh"

namespace msaq {

constexpr int KVM_WARPS = 4;
constexpr int KVM_THREADS = (KVM_WARPS + 1) * 32;
constexpr int KVM_TK = 128;                 // keys per stage
constexpr int KVM_CHUNK = 32;               // keys per warp per stage
// Two builds of the kernel: CPS = 2 thread blocks per SM with a three-stage ring (up to 204 registers), for small
// problems where each block's own latency counts (B = 1, Lk = 16384: 17.6 against 19.3 us), and CPS = 3 with a
// two-stage ring (136 registers, no spills), for large ones where twelve consumer warps per SM hide more of the
// softmax / P.V issue latency than eight (GQA 32/8, Lk = 32768, B = 64: 630 -> 595 us; B = 16: 186 -> 170 us).
constexpr int kvm_stages(int cps) { return cps == 3 ? 2 : 3; }
constexpr int KVM_UP = KVM_TK * 16, KVM_SH = KVM_TK * 8, KVM_SC = KVM_TK;
constexpr int KVM_K_UP = 0, KVM_K_SH = 4 * KVM_UP, KVM_K_SC = KVM_K_SH + 4 * KVM_SH;
constexpr int KVM_V_UP = KVM_K_SC + 4 * KVM_SC, KVM_V_SH = KVM_V_UP + 4 * KVM_UP, KVM_V_SC = KVM_V_SH + 4 * KVM_SH;
constexpr int KVM_STAGE_BYTES = KVM_V_SC + 4 * KVM_SC;            // 25600
// The same kernel reads plain MXINT8 caches (the reference's matched baseline, csrc/mxint8.cu:750-912): 32 int8
// codes and a scale per (key, block).  The codes are MMA operands as stored, so the stage is K codes | K scales |
// V codes | V scales and the nibble work drops out.
constexpr int KVF_MSAQ_U4 = 0, KVF_MXINT8 = 1;
constexpr int KVX_Q = KVM_TK * 32;                                // code bytes per block of a 128-key stage
constexpr int KVX_K_Q = 0, KVX_K_SC = 4 * KVX_Q, KVX_V_Q = KVX_K_SC + 4 * KVM_SC, KVX_V_SC = KVX_V_Q + 4 * KVX_Q;
constexpr int KVX_STAGE_BYTES = KVX_V_SC + 4 * KVM_SC;            // 33792
__host__ __device__ constexpr int kvm_stage_bytes(int fmt) { return fmt == KVF_MXINT8 ? KVX_STAGE_BYTES : KVM_STAGE_BYTES; }
__host__ __device__ constexpr int kvm_smem_bytes(int fmt, int cps) {      // ring + query records + probability exchange + scale table
    return kvm_stages(cps) * kvm_stage_bytes(fmt) + 4 * 2 * 320 + KVM_WARPS * 8 * 40 * 4 + KVM_WARPS * 4 * 32 * 4;
}
constexpr int KVM_QREC = 320;               // staged query record per (block, pass); layout as in gemv_mma.cuh
constexpr float KVM_SPLIT_TAU = 0.001953125f;  // 2^-9: a chunk is split when all keys but its maximum sum to less than this
constexpr int KVM_PSTRIDE = 40;             // floats per head row of the probability exchange buffer

struct KvMmaArgs {
    const __nv_bfloat16* q;     // [B][Hq][128]
    KvPlanes k, v;
    float* partial;             // [B][Hq][S][130]
    const int32_t* seq_lens;    // optional
    int* status;
    int* sticky;                // the library's per-device status word (may be null)
    int Hq, Hkv, Lk, Lcap, key_tile, S, qrot;
    float sm_scale_log2;        // log2(e) / sqrt(D)
    Rope rope;                  // rotary embedding of the query (cos == nullptr: none)
    int64_t q_pos;              // the query's position, or per sequence:
    const int32_t* q_pos_per_seq;
    float split_limit;          // a chunk whose small keys sum to less than this (relative to its maximum) may split
    uint32_t max_polls;         // limit of every mbarrier wait (see mbar_wait_bounded)
    int skip_stage;             // test hook: the producer of CTA (0,0,0) stops before this stage (-1: never)
    // The step's new token, appended by this kernel (k_new == nullptr: the cache is taken as it is): the thread block
    // that owns the key tile of the token's slot packs the K row (RoPE with the query's tables at the slot, then the
    // Hadamard rotation when app_rot) and the V row of its (sequence, kv head) into the planes before it streams
    // them, exactly as msaq_kv_append_pair_rope would have.
    const __nv_bfloat16* k_new;   // [B][Hkv][128]
    const __nv_bfloat16* v_new;
    int64_t app_pos;              // slot of the new token, or per sequence:
    const int32_t* app_pos_per_seq;
    int app_rot;
    Fmt fmt;
};

template <int G, int FMT = KVF_MSAQ_U4, int CPS = 2>
__global__ void __launch_bounds__(KVM_THREADS, CPS)
kv_decode_u4gs2_kernel(const KvMmaArgs a) {
    constexpr int KVM_STAGES = kvm_stages(CPS);
    chain_wait();
    constexpr int PASSES = (G + 3) / 4;
    constexpr bool MX = FMT == KVF_MXINT8;
    constexpr int KVM_STAGE_BYTES = kvm_stage_bytes(FMT);        // shadows the MSAQ constants below
    constexpr int KVM_OFF_Q = KVM_STAGES * KVM_STAGE_BYTES;
    constexpr int KVM_OFF_P = KVM_OFF_Q + 4 * 2 * KVM_QREC;
    constexpr int KVM_OFF_R = KVM_OFF_P + KVM_WARPS * 8 * KVM_PSTRIDE * 4;      // per-warp 2^-shift table [4][32] floats
    extern __shared__ __align__(128) uint8_t kvm_smem[];
    uint8_t* const smem = kvm_smem;
    __shared__ __align__(8) uint64_t bar_full[KVM_STAGES];
    __shared__ __align__(8) uint64_t bar_empty[KVM_STAGES];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int len = a.seq_lens ? min(a.seq_lens[b], a.Lk) : a.Lk;
    const int j0 = tile * a.key_tile, j1 = min(j0 + a.key_tile, len);
    const int n_stage = j1 > j0 ? (j1 - j0 + KVM_TK - 1) / KVM_TK : 0;
    const uint32_t sb = smem_u32(smem);

    if (tid == 0) {
        for (int s = 0; s < KVM_STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), KVM_WARPS);
        }
        mbar_init_fence();
    }
    for (int i = tid; i < 4 * 2 * KVM_QREC / 4; i += KVM_THREADS) reinterpret_cast<uint32_t*>(smem + KVM_OFF_Q)[i] = 0u;
    if (a.k_new) {
        // The new token: written by the thread block whose tile holds its slot (the last tile for a slot beyond the
        // attended keys), warp 0 the K row, warp 1 the V row, through the ring memory that is still free.  The
        // proxy fence and the barrier below put the bytes in front of this block's own bulk copies; no other
        // block reads that slot.
        const int64_t p = a.app_pos_per_seq ? (int64_t)a.app_pos_per_seq[b] : a.app_pos;
        const bool valid = p >= 0 && p < a.Lcap;
        const int owner = valid ? min((int)(p / a.key_tile), (int)gridDim.x - 1) : 0;
        if (tile == owner) {
            if (!valid) {
                if (tid == 0 && hk == 0 && a.sticky) atomicOr(a.sticky, BAD_APPEND_POS);
            } else if (warp < 2) {
                const KvPlanes& pl = warp == 0 ? a.k : a.v;
                QuantJob job;
                job.X = warp == 0 ? a.k_new : a.v_new;
                job.scale_exp = const_cast<int8_t*>(pl.s);
                job.upper = const_cast<uint8_t*>(pl.u);
                job.shared = const_cast<uint8_t*>(pl.h);
                job.rot = warp == 0 ? a.app_rot : 0;
                job.rope = warp == 0 ? 1 : 0;
                job.mx = MX ? 1 : 0;
                const int64_t head = (int64_t)b * a.Hkv + hk;
                quantize_row_warp<4>(job, a.rope, head, head, p, a.Lcap, a.fmt, reinterpret_cast<float*>(smem + warp * 1024),
                                     reinterpret_cast<uint32_t*>(smem + 2048 + warp * 256), lane);
                asm volatile("fence.proxy.async;" ::: "memory");
            }
        }
    }
    __syncthreads();

    if (warp == KVM_WARPS) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 1;
            const int64_t head_row = ((int64_t)b * a.Hkv + hk) * 4;
            const bool inject = a.skip_stage >= 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0;
            int issued = 0;
            // (Letting the kernels behind be scheduled three quarters through, as the GEMV does under
            // MSAQ_OPT_EARLY_WEIGHTS, was measured here too: the layer step went from 172.3 to 173.6 us.)
            for (int it = 0; it < n_stage; ++it) {
                if (inject && it == a.skip_stage) break;               // the consumers' wait for this stage runs out
                if (!mbar_wait_bounded(smem_u32(&bar_empty[s]), ph, a.max_polls)) {
                    report_wait_failure(a.status, 1, a.sticky, WAIT_FAIL_KV_DECODE);
                    break;
                }
                ++issued;
                const int j = j0 + it * KVM_TK;
                const int nk = min(KVM_TK, (j1 - j + 15) & ~15);       // whole 16-key groups (capacity is a multiple of 16)
                const uint32_t bar = smem_u32(&bar_full[s]);
                const uint32_t base = sb + s * KVM_STAGE_BYTES;
                mbar_expect_tx(bar, (uint32_t)(2 * 4 * nk * (MX ? 33 : 25)));
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {
                    const int64_t row = (head_row + blk) * a.Lcap + j;
                    if constexpr (MX) {
                        bulk_g2s(base + KVX_K_Q + blk * KVX_Q, a.k.u + row * 32, (uint32_t)nk * 32, bar);
                        bulk_g2s(base + KVX_K_SC + blk * KVM_SC, a.k.s + row, (uint32_t)nk, bar);
                        bulk_g2s(base + KVX_V_Q + blk * KVX_Q, a.v.u + row * 32, (uint32_t)nk * 32, bar);
                        bulk_g2s(base + KVX_V_SC + blk * KVM_SC, a.v.s + row, (uint32_t)nk, bar);
                        continue;
                    }
                    bulk_g2s(base + KVM_K_UP + blk * KVM_UP, a.k.u + row * 16, (uint32_t)nk * 16, bar);
                    bulk_g2s(base + KVM_K_SH + blk * KVM_SH, a.k.h + row * 8, (uint32_t)nk * 8, bar);
                    bulk_g2s(base + KVM_K_SC + blk * KVM_SC, a.k.s + row, (uint32_t)nk, bar);
                    bulk_g2s(base + KVM_V_UP + blk * KVM_UP, a.v.u + row * 16, (uint32_t)nk * 16, bar);
                    bulk_g2s(base + KVM_V_SH + blk * KVM_SH, a.v.h + row * 8, (uint32_t)nk * 8, bar);
                    bulk_g2s(base + KVM_V_SC + blk * KVM_SC, a.v.s + row, (uint32_t)nk, bar);
                }
                if (++s == KVM_STAGES) { s = 0; ph ^= 1u; }
            }
            // Leave only when every copy this thread issued has landed: shared memory must not be
            // handed to the next CTA with a copy still in flight (consumers that gave up do not wait).
            for (int i = max(0, issued - KVM_STAGES); i < issued; ++i)
                mbar_wait_bounded(smem_u32(&bar_full[i % KVM_STAGES]), (uint32_t)(i / KVM_STAGES) & 1u, a.max_polls);
        }
        return;
    }

    // ---------------- consumers: stage the query (rotate, 16-bit block fixed point) ----------------
    const int g = lane >> 2, t = lane & 3, h2 = t >> 1, odd = t & 1;
    for (int hh = warp; hh < G; hh += KVM_WARPS) {
        const __nv_bfloat16* qp = a.q + ((int64_t)b * a.Hq + hk * G + hh) * 128 + lane * 4;
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __bfloat162float(qp[i]);
        if (a.rope.cos) {
            int64_t p = a.q_pos_per_seq ? a.q_pos_per_seq[b] : a.q_pos;
            p = a.rope.rows == 1 ? 0 : min(max(p, (int64_t)0), a.rope.rows - 1);
            rope_warp<4>(v, lane, a.rope, p);
        }
        if (a.qrot) {
            fwht_warp<4>(v, lane);
            const float inv = 0.08838834764831845f;                       // 1/sqrt(128)
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] *= inv;
        }
        uint32_t ax = 0u;
#pragma unroll
        for (int i = 0; i < 4; ++i) ax = max(ax, __float_as_uint(v[i]) & 0x7FFFFFFFu);
#pragma unroll
        for (int o = 1; o <= 4; o <<= 1) ax = max(ax, __shfl_xor_sync(0xffffffffu, ax, o));
        int E = (int)(ax >> 23) - 127;
        E = ax == 0u ? 0 : max(-100, min(127, E));
        const float up = __int_as_float((14 - E + 127) << 23);
        const int blk = lane >> 3, pass = hh >> 2, mm = hh & 3;
        uint8_t* rec = smem + KVM_OFF_Q + (blk * PASSES + pass) * KVM_QREC;
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int xi = min(__float2int_rn(v[i] * up), 32639);
            const int lo = (int)(int8_t)(xi & 0xFF), hi = (xi - lo) >> 8;
            sum += xi;
            const int e = (lane & 7) * 4 + i;
            // MXINT8 keys are operands in their stored order, so the query record is in natural element order
            const int ts = MX ? (e & 15) >> 2 : 2 * (e >> 4) + ((e >> 1) & 1);
            const int jj = MX ? (e >> 4) * 4 + (e & 3) : (e & 1) * 4 + ((e & 15) >> 2);
            rec[(2 * mm) * 32 + ts * 8 + jj] = (uint8_t)hi;
            rec[(2 * mm + 1) * 32 + ts * 8 + jj] = (uint8_t)lo;
        }
#pragma unroll
        for (int o = 1; o <= 4; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if ((lane & 7) == 0) {
            int* tc = reinterpret_cast<int*>(rec + 256 + mm * 16);
            tc[0] = -8 * sum;
            // scores come out in the exp2 domain; an Inf or NaN in the query block makes the head's output NaN
            tc[1] = ax >= 0x7F800000u ? 0x7FC00000 : __float_as_int(ldexpf(a.sm_scale_log2, E - 14));
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(KVM_WARPS * 32) : "memory");

    // ------------------------------------ main loop ------------------------------------
    const uint32_t sel = odd ? 0x7531u : 0x6420u;
    const uint32_t nshift = odd * 4;
    const int ck = warp * KVM_CHUNK;                            // first key of this warp's chunk in a stage
    float* Pw = reinterpret_cast<float*>(smem + KVM_OFF_P) + warp * 8 * KVM_PSTRIDE;
    float* Rw = reinterpret_cast<float*>(smem + KVM_OFF_R) + warp * 4 * 32;
    float m_run[PASSES], l_run[PASSES];                         // QK layout: head 4p + t (replicated over g)
#pragma unroll
    for (int p = 0; p < PASSES; ++p) { m_run[p] = -INFINITY; l_run[p] = 0.0f; }
    float acc[4][4][2];                                         // PV layout: head g; [block][n-tile][column 2t, 2t+1]
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int n = 0; n < 4; ++n) acc[i][n][0] = acc[i][n][1] = 0.0f;
    bool aborted = false;

    int s = 0;
    uint32_t ph = 0;
    for (int it = 0; it < n_stage; ++it) {
        if (!aborted && !mbar_wait_bounded(smem_u32(&bar_full[s]), ph, a.max_polls)) {
            report_wait_failure(a.status, 1, a.sticky, WAIT_FAIL_KV_DECODE);
            aborted = true;
        }
        const uint32_t so = sb + s * KVM_STAGE_BYTES;
        const int jbase = j0 + it * KVM_TK + ck;                // global index of this warp's first key
        if (!aborted && jbase < j1) {
            // ---- scores: 2 key groups of 16 x 4 blocks, all heads ----
            float S[PASSES][2][2];
#pragma unroll
            for (int p = 0; p < PASSES; ++p) S[p][0][0] = S[p][0][1] = S[p][1][0] = S[p][1][1] = 0.0f;
#pragma unroll
            for (int blk = 0; blk < 4; ++blk) {
                uint2 bq[PASSES];
                int corr[PASSES];
                float cx[PASSES];
#pragma unroll
                for (int p = 0; p < PASSES; ++p) {
                    const uint32_t rb = sb + KVM_OFF_Q + (blk * PASSES + p) * KVM_QREC;
                    bq[p] = lds64<0>(rb + g * 32 + t * 8);
                    corr[p] = (int)lds32<0>(rb + 256 + t * 16);
                    cx[p] = __uint_as_float(lds32<4>(rb + 256 + t * 16));
                }
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    const int kk = ck + mt * 16 + g;
                    if constexpr (MX) {
                        const uint32_t kb = so + KVX_K_Q + blk * KVX_Q + kk * 32 + t * 4;
                        uint32_t A[4];
                        A[0] = lds32<0>(kb);
                        A[1] = lds32<256>(kb);                      // key + 8
                        A[2] = lds32<16>(kb);
                        A[3] = lds32<256 + 16>(kb);
                        const int e0 = lds_s8<0>(so + KVX_K_SC + blk * KVM_SC + kk);
                        const int e1 = lds_s8<8>(so + KVX_K_SC + blk * KVM_SC + kk);
                        const float sw0 = __int_as_float(e0 * (1 << 23) + (127 << 23));
                        const float sw1 = __int_as_float(e1 * (1 << 23) + (127 << 23));
#pragma unroll
                        for (int p = 0; p < PASSES; ++p) {
                            const uint32_t B[2] = {bq[p].x, bq[p].y};
                            int Dm[4];
                            mma_s8_16832_z(Dm, A, B);
                            S[p][mt][0] = fmaf((float)(Dm[0] * 256 + Dm[1]) * cx[p], sw0, S[p][mt][0]);
                            S[p][mt][1] = fmaf((float)(Dm[2] * 256 + Dm[3]) * cx[p], sw1, S[p][mt][1]);
                        }
                        continue;
                    }
                    const uint2 w0 = lds64<0>(so + KVM_K_UP + blk * KVM_UP + kk * 16 + h2 * 8);
                    const uint2 w1 = lds64<128>(so + KVM_K_UP + blk * KVM_UP + kk * 16 + h2 * 8);
                    const uint32_t s0 = lds32<0>(so + KVM_K_SH + blk * KVM_SH + kk * 8 + h2 * 4);
                    const uint32_t s1 = lds32<64>(so + KVM_K_SH + blk * KVM_SH + kk * 8 + h2 * 4);
                    const int e0 = lds_s8<0>(so + KVM_K_SC + blk * KVM_SC + kk);
                    const int e1 = lds_s8<8>(so + KVM_K_SC + blk * KVM_SC + kk);
                    const uint32_t m0 = and_xor(s0 >> nshift, 0x0F0F0F0Fu, 0x08080808u);
                    const uint32_t m1 = and_xor(s1 >> nshift, 0x0F0F0F0Fu, 0x08080808u);
                    const uint32_t x0 = prmt(w0.x, w0.y, sel), x1 = prmt(w1.x, w1.y, sel);
                    uint32_t A[4];
                    A[0] = and_or(x0 << 4, 0xF0F0F0F0u, m0);
                    A[1] = and_or(x1 << 4, 0xF0F0F0F0u, m1);
                    A[2] = and_or(x0, 0xF0F0F0F0u, m0);
                    A[3] = and_or(x1, 0xF0F0F0F0u, m1);
                    const float sw0 = __int_as_float(e0 * (1 << 23) + (127 << 23));
                    const float sw1 = __int_as_float(e1 * (1 << 23) + (127 << 23));
#pragma unroll
                    for (int p = 0; p < PASSES; ++p) {
                        const uint32_t B[2] = {bq[p].x, bq[p].y};
                        int Dm[4];
                        mma_s8_16832_z(Dm, A, B);
                        const float f0 = (float)(Dm[0] * 256 + Dm[1] + corr[p]) * cx[p];
                        const float f1 = (float)(Dm[2] * 256 + Dm[3] + corr[p]) * cx[p];
                        S[p][mt][0] = fmaf(f0, sw0, S[p][mt][0]);
                        S[p][mt][1] = fmaf(f1, sw1, S[p][mt][1]);
                    }
                }
            }
            // ---- online softmax (exp2 domain); thread (g,t): head 4p+t, keys ck + {g, g+8, 16+g, 24+g} ----
            // Probabilities are taken relative to the CHUNK's own maximum (so the 16-bit fixed point of
            // the P.V operand always spans the chunk's largest key) and the factor 2^(chunk max -
            // running max) is applied in fp32 to the chunk's integer result: a chunk far below an
            // earlier dominant key keeps its full relative precision.
            // A chunk that one key dominates -- every other key together below 2^-9 of it, e.g. an attention
            // sink -- would leave the others under the resolution of the 16-bit operand.  Such a chunk
            // (split[p] > 0, rare) takes two P.V passes: the small keys relative to their own sum, then the
            // dominant key.  (The sum of the probabilities is there anyway, so looking for this costs nothing.)
            float alpha[PASSES], beta[PASSES], split[PASSES];
#pragma unroll
            for (int p = 0; p < PASSES; ++p) {
                float mx = -INFINITY;
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        if (jbase + mt * 16 + r * 8 + g >= j1) S[p][mt][r] = -INFINITY;      // key beyond the sequence
                        mx = fmaxf(mx, S[p][mt][r]);
                    }
#pragma unroll
                for (int o = 4; o <= 16; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const float m_new = fmaxf(m_run[p], mx);
                const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
                alpha[p] = exp2f(m_run[p] - m_use);                                          // 0 when nothing was seen before
                const float mc = (mx == -INFINITY) ? 0.0f : mx;                              // the chunk's own maximum
                beta[p] = (mx == -INFINITY) ? 0.0f : exp2f(mx - m_use);
                float ps = 0.0f;
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        const float pv = exp2f(S[p][mt][r] - mc);
                        ps += pv;
                        Pw[(4 * p + t) * KVM_PSTRIDE + mt * 16 + r * 8 + g] = pv;
                    }
#pragma unroll
                for (int o = 4; o <= 16; o <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
                split[p] = (ps > 1.0f && ps - 1.0f < a.split_limit) ? ps - 1.0f : 0.0f;       // the maximum itself counts 1
                l_run[p] = fmaf(l_run[p], alpha[p], ps * beta[p]);
                m_run[p] = m_new;
            }
            // ---- value scales of the chunk: E_max per block, and 2^-(E_max - e) per key ----
            int emax[4];
#pragma unroll
            for (int blk = 0; blk < 4; ++blk) {
                const int ev = lds_s8<0>(so + (MX ? KVX_V_SC : KVM_V_SC) + blk * KVM_SC + ck + lane);
                const int evm = (jbase + lane < j1) ? ev : -128;
                emax[blk] = __reduce_max_sync(0xffffffffu, evm);
                const int sh = min(emax[blk] - ev, 31);
                Rw[blk * 32 + lane] = (jbase + lane < j1) ? __int_as_float((127 - sh) << 23) : 0.0f;
            }
            __syncwarp();
            // rescale of the running output of head g (PV layout) by that head's alpha
            float al = __shfl_sync(0xffffffffu, alpha[0], g & 3);
            float be = __shfl_sync(0xffffffffu, beta[0], g & 3);      // head g's chunk factor, PV layout
            if (PASSES > 1) {
                const float al1 = __shfl_sync(0xffffffffu, alpha[PASSES - 1], g & 3);
                const float be1 = __shfl_sync(0xffffffffu, beta[PASSES - 1], g & 3);
                al = (g < 4) ? al : al1;
                be = (g < 4) ? be : be1;
            }
            float sa = 0.0f;                                          // head g's small-set sum when its chunk is split
            if (__any_sync(0xffffffffu, split[0] > 0.0f || split[PASSES - 1] > 0.0f)) {
                sa = __shfl_sync(0xffffffffu, split[0], g & 3);
                if (PASSES > 1) {
                    const float sa1 = __shfl_sync(0xffffffffu, split[PASSES - 1], g & 3);
                    sa = (g < 4) ? sa : sa1;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int n = 0; n < 4; ++n) { acc[i][n][0] *= al; acc[i][n][1] *= al; }
            // probabilities of head g for the keys 8t..8t+7 of the chunk, as 16-bit fixed point
            float pf[8];
            {
                const float4 p0 = *reinterpret_cast<const float4*>(Pw + g * KVM_PSTRIDE + 8 * t);
                const float4 p1 = *reinterpret_cast<const float4*>(Pw + g * KVM_PSTRIDE + 8 * t + 4);
                pf[0] = p0.x; pf[1] = p0.y; pf[2] = p0.z; pf[3] = p0.w;
                pf[4] = p1.x; pf[5] = p1.y; pf[6] = p1.z; pf[7] = p1.w;
            }
            if (G < 8 && g >= G) {
#pragma unroll
                for (int i = 0; i < 8; ++i) pf[i] = 0.0f;
            }
            if (G < 8 && g >= G) sa = 0.0f;
            bool is_split = sa > 0.0f;
            if (__any_sync(0xffffffffu, is_split)) {
                // Confirm with the value scales: the small keys only need their own pass when every big key
                // enters the P.V operand far below full scale, i.e. its value block scales are all at
                // least 2^4 under the chunk's (an attention sink with a small value row).  Otherwise the big
                // keys' own contribution dwarfs what the small keys lose to rounding.
                float big_scale = 0.0f;
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {
                    const float4 r0 = *reinterpret_cast<const float4*>(Rw + blk * 32 + 8 * t);
                    const float4 r1 = *reinterpret_cast<const float4*>(Rw + blk * 32 + 8 * t + 4);
                    const float rr[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) big_scale = fmaxf(big_scale, pf[i] >= 0.5f ? rr[i] : 0.0f);
                }
                big_scale = fmaxf(big_scale, __shfl_xor_sync(0xffffffffu, big_scale, 1));
                big_scale = fmaxf(big_scale, __shfl_xor_sync(0xffffffffu, big_scale, 2));
                is_split = is_split && big_scale <= 0.0625f;
            }
            const int n_pv = __any_sync(0xffffffffu, is_split) ? 2 : 1;
            const float sa_inv = is_split ? __frcp_rn(sa) : 1.0f;
            // ---- P.V: per block 4 n-tiles of 8 channels (+ one all-ones MMA for the code offset) ----
            const int lrow = lane & 15;
            const int vkey = 8 * (lrow >> 2) + 2 * (lrow & 3) + (lane >> 4);      // even keys -> matrix 0, odd -> matrix 1
#pragma unroll 1
            for (int pvp = 0; pvp < n_pv; ++pvp) {
            float pq[8];                         // this pass's probabilities and their common factor
            float bsc;
            if (pvp == 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) pq[i] = is_split ? (pf[i] < 0.5f ? fminf(pf[i] * sa_inv, 1.0f) : 0.0f) : pf[i];
                bsc = is_split ? be * sa : be;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) pq[i] = (is_split && pf[i] >= 0.5f) ? pf[i] : 0.0f;
                bsc = be;
            }
#pragma unroll
            for (int blk = 0; blk < 4; ++blk) {
                // P' = p * 2^(e - E_max) as u16, bytes split into the hi (row g) and lo (row g+8) operand planes
                uint32_t pv16[8];
                {
                    const float4 r0 = *reinterpret_cast<const float4*>(Rw + blk * 32 + 8 * t);
                    const float4 r1 = *reinterpret_cast<const float4*>(Rw + blk * 32 + 8 * t + 4);
                    const float rr[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) pv16[i] = __float2uint_rn(pq[i] * rr[i] * 65535.0f);
                }
                uint32_t PA[4];
                {
                    const uint32_t t1 = prmt(pv16[0], pv16[2], 0x5140u), t2 = prmt(pv16[4], pv16[6], 0x5140u);
                    const uint32_t u1 = prmt(pv16[1], pv16[3], 0x5140u), u2 = prmt(pv16[5], pv16[7], 0x5140u);
                    PA[0] = prmt(t1, t2, 0x7632u);      // hi bytes, even keys  (row g,   k 4t..4t+3)
                    PA[1] = prmt(t1, t2, 0x5410u);      // lo bytes, even keys  (row g+8, k 4t..4t+3)
                    PA[2] = prmt(u1, u2, 0x7632u);      // hi bytes, odd keys   (row g,   k 16+4t..)
                    PA[3] = prmt(u1, u2, 0x5410u);      // lo bytes, odd keys
                }
                if constexpr (MX) {
                    // codes as stored: two transposing loads deliver channels g, g+8 and 16+g, 24+g of the 32 keys
                    uint32_t va[4], vb[4];
                    ldmatrix_t8_x2(va, so + KVX_V_Q + blk * KVX_Q + (ck + vkey) * 32);
                    ldmatrix_t8_x2(vb, so + KVX_V_Q + blk * KVX_Q + (ck + vkey) * 32 + 16);
                    const float oscx = __int_as_float((emax[blk] + 127) << 23) * (1.0f / 65535.0f) * bsc;
#pragma unroll
                    for (int n = 0; n < 4; ++n) {
                        const uint32_t Bv[2] = {n == 0 ? va[0] : n == 1 ? va[1] : n == 2 ? vb[0] : vb[1],
                                                n == 0 ? va[2] : n == 1 ? va[3] : n == 2 ? vb[2] : vb[3]};
                        int Dv[4];
                        mma_u8s8_16832_z(Dv, PA, Bv);
                        acc[blk][n][0] = fmaf((float)(Dv[0] * 256 + Dv[2]), oscx, acc[blk][n][0]);
                        acc[blk][n][1] = fmaf((float)(Dv[1] * 256 + Dv[3]), oscx, acc[blk][n][1]);
                    }
                    continue;
                }
                uint32_t vr[4], sr[2];
                ldmatrix_t8_x2(vr, so + KVM_V_UP + blk * KVM_UP + (ck + vkey) * 16);
                ldmatrix_t8_x1(sr, so + KVM_V_SH + blk * KVM_SH + (ck + 2 * lrow) * 8);
                // shared codes of group g (nibble g%2 of byte g/2) and group g+8 (byte 4 + g/2): held by lanes g/2 and 4+g/2
                const int la = (g >> 1) * 4 + t, lb = (4 + (g >> 1)) * 4 + t;
                const uint32_t gs4 = (g & 1) * 4;
                const uint32_t me0 = and_xor(__shfl_sync(0xffffffffu, sr[0], la) >> gs4, 0x0F0F0F0Fu, 0x08080808u);
                const uint32_t me1 = and_xor(__shfl_sync(0xffffffffu, sr[0], lb) >> gs4, 0x0F0F0F0Fu, 0x08080808u);
                const uint32_t mo0 = and_xor(__shfl_sync(0xffffffffu, sr[1], la) >> gs4, 0x0F0F0F0Fu, 0x08080808u);
                const uint32_t mo1 = and_xor(__shfl_sync(0xffffffffu, sr[1], lb) >> gs4, 0x0F0F0F0Fu, 0x08080808u);
                int Dc[4];
                {
                    const uint32_t ones[2] = {0x01010101u, 0x01010101u};
                    mma_u8s8_16832_z(Dc, PA, ones);
                }
                const int corr = -8 * (Dc[0] * 256 + Dc[2]);                   // every shared code carries +8
                const float osc = __int_as_float((emax[blk] + 127) << 23) * (1.0f / 65535.0f) * bsc;
                // n-tile 0: channel 2n+1 (high nibbles of byte column g), 1: channel 2n, 2: 17+2n, 3: 16+2n
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const uint32_t ve = (n < 2) ? vr[0] : vr[1], vo = (n < 2) ? vr[2] : vr[3];
                    const uint32_t me = (n < 2) ? me0 : me1, mo = (n < 2) ? mo0 : mo1;
                    uint32_t Bv[2];
                    if ((n & 1) == 0) { Bv[0] = and_or(ve, 0xF0F0F0F0u, me); Bv[1] = and_or(vo, 0xF0F0F0F0u, mo); }
                    else { Bv[0] = and_or(ve << 4, 0xF0F0F0F0u, me); Bv[1] = and_or(vo << 4, 0xF0F0F0F0u, mo); }
                    int Dv[4];
                    mma_u8s8_16832_z(Dv, PA, Bv);
                    acc[blk][n][0] = fmaf((float)(Dv[0] * 256 + Dv[2] + corr), osc, acc[blk][n][0]);
                    acc[blk][n][1] = fmaf((float)(Dv[1] * 256 + Dv[3] + corr), osc, acc[blk][n][1]);
                }
            }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_empty[s]));
        if (++s == KVM_STAGES) { s = 0; ph ^= 1u; }
    }

    // ---------------- merge the four warps, write the tile's partial (acc, m, l) ----------------
    asm volatile("bar.sync 1, %0;" ::"n"(KVM_WARPS * 32) : "memory");          // ring memory is free to reuse
    float* mb = reinterpret_cast<float*>(smem);                                // [warp][G][130]
    // m, l of head 4p+t live in the QK layout (lanes with g == 0 write them)
    if (g == 0) {
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int hh = 4 * p + t;
            if (hh < G) {
                mb[(warp * G + hh) * 130 + 128] = aborted ? __int_as_float(0x7FC00000) : m_run[p];   // NaN marks a warp that gave up
                mb[(warp * G + hh) * 130 + 129] = l_run[p];
            }
        }
    }
    if (g < G) {
#pragma unroll
        for (int blk = 0; blk < 4; ++blk)
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int col = 2 * t + c;                                  // B column = byte column of the V tile
                    const int d = MX ? blk * 32 + 8 * n + col
                                     : blk * 32 + ((n < 2) ? 0 : 16) + 2 * col + ((n & 1) ? 0 : 1);
                    mb[(warp * G + g) * 130 + d] = acc[blk][n][c];
                }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(KVM_WARPS * 32) : "memory");
    float* out = a.partial + (((int64_t)b * a.Hq + hk * G) * a.S + tile) * 130;
    for (int idx = tid; idx < G * 130; idx += KVM_WARPS * 32) {
        const int hh = idx / 130, d = idx % 130;
        float mg = -INFINITY;
        bool bad = false;
#pragma unroll
        for (int w = 0; w < KVM_WARPS; ++w) {
            const float mw = mb[(w * G + hh) * 130 + 128];
            bad = bad || (mw != mw);
            mg = fmaxf(mg, mw);                                                // fmaxf ignores the NaN
        }
        float r;
        if (d == 128) r = bad ? __int_as_float(0x7FC00000) : mg;
        else {
            r = 0.0f;
#pragma unroll
            for (int w = 0; w < KVM_WARPS; ++w) {
                const float mw = mb[(w * G + hh) * 130 + 128];
                const float wgt = (mw == -INFINITY || mw != mw) ? 0.0f : exp2f(mw - mg);
                r = fmaf(mb[(w * G + hh) * 130 + (d == 129 ? 129 : d)], wgt, r);
            }
        }
        out[(int64_t)hh * a.S * 130 + d] = r;
    }
}

// Merge of tile partials kept in the exp2 domain (m is a base-2 exponent).  128 threads per
// (head, sequence).  The tiles' (m, l) pairs are fetched in parallel, one tile per thread, and turned
// into weights in shared memory; each thread sums its channel over the tiles in tile order,
// sixteen loads in flight at a time (up to 128 tiles: all requested in one round trip).
constexpr int KVM_MERGE_TILES = 512;           // weights held in shared memory per pass over the tiles

__global__ void __launch_bounds__(128)
kv_decode_combine2_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                          float* __restrict__ out_f32, int H, int S) {
    chain_release();
    chain_wait();
    __shared__ float wgt[KVM_MERGE_TILES];
    __shared__ float lsm[128];
    __shared__ float red[8];
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x, warp = d >> 5, lane = d & 31;
    const float* base = partial + ((int64_t)b * H + h) * S * 130;

    float num = 0.0f, den = 0.0f;
    bool poisoned;
    if (S <= 128) {
        // Common case, one dependent round trip: this thread's tile statistics and the first sixteen
        // tiles of its channel are requested together; the weights come out of the registers.
        float pv[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) pv[k] = (k < S) ? base[k * 130 + d] : 0.0f;
        const float m_own = d < S ? base[d * 130 + 128] : -INFINITY;
        const float l_own = d < S ? base[d * 130 + 129] : 0.0f;
        float mloc = m_own;                                            // fmaxf ignores the NaN that marks an abandoned tile
#pragma unroll
        for (int o = 16; o; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
        const unsigned badw = __ballot_sync(0xffffffffu, m_own != m_own);
        if (lane == 0) { red[warp] = mloc; red[4 + warp] = badw ? 1.0f : 0.0f; }
        __syncthreads();
        const float mg = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
        poisoned = (red[4] + red[5] + red[6] + red[7]) > 0.0f;
        if (d < S) {
            wgt[d] = (m_own == -INFINITY || m_own != m_own) ? 0.0f : exp2f(m_own - mg);
            lsm[d] = l_own;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            if (k < S) { num = fmaf(pv[k], wgt[k], num); den = fmaf(lsm[k], wgt[k], den); }
        }
        for (int s0 = 16; s0 < S; s0 += 16) {
#pragma unroll
            for (int k = 0; k < 16; ++k) pv[k] = (s0 + k < S) ? base[(s0 + k) * 130 + d] : 0.0f;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                if (s0 + k < S) { num = fmaf(pv[k], wgt[s0 + k], num); den = fmaf(lsm[s0 + k], wgt[s0 + k], den); }
            }
        }
    } else {
        // global maximum of m (fmaxf ignores the NaN that marks an abandoned tile; it is detected below)
        float mloc = -INFINITY;
        bool bad = false;
        for (int s = d; s < S; s += 128) {
            const float m = base[s * 130 + 128];
            bad = bad || (m != m);
            mloc = fmaxf(mloc, m);
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
        const unsigned badw = __ballot_sync(0xffffffffu, bad);
        if (lane == 0) { red[warp] = mloc; red[4 + warp] = badw ? 1.0f : 0.0f; }
        __syncthreads();
        const float mg = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
        poisoned = (red[4] + red[5] + red[6] + red[7]) > 0.0f;
        for (int c0 = 0; c0 < S; c0 += KVM_MERGE_TILES) {
            const int cn = min(KVM_MERGE_TILES, S - c0);
            __syncthreads();
            for (int s = d; s < cn; s += 128) {
                const float m = base[(c0 + s) * 130 + 128];
                wgt[s] = (m == -INFINITY || m != m) ? 0.0f : exp2f(m - mg);
            }
            __syncthreads();
            for (int s0 = 0; s0 < cn; s0 += 16) {
                float pv[16], lv[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const bool ok = s0 + k < cn;
                    const float* p = base + (c0 + s0 + k) * 130;
                    pv[k] = ok ? p[d] : 0.0f;
                    lv[k] = ok ? p[129] : 0.0f;
                }
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const float w = (s0 + k < cn) ? wgt[s0 + k] : 0.0f;
                    num = fmaf(pv[k], w, num);
                    den = fmaf(lv[k], w, den);
                }
            }
        }
    }
    float r = den > 0.0f ? num / den : 0.0f;
    if (poisoned) r = __int_as_float(0x7FC00000);                      // a wait gave up in some tile
    const int64_t o = ((int64_t)b * H + h) * 128 + d;
    out[o] = __float2bfloat16_rn(r);
    if (out_f32) out_f32[o] = r;
}

}  // namespace msaq

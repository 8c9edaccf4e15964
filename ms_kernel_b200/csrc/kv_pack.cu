// Quantise-and-pack kernels: KV append / append-with-rotation / prefill write,
// the standalone Hadamard rotation, and the offline weight packer.
//
// One warp owns one row of D values (D = 32*EPL): it loads the row, optionally
// runs the Hadamard butterfly in registers, parks the fp32 row in shared
// memory, and then quantises one 32-block at a time with one lane per element.
// Behaviour replaced: csrc/kv_attention.cu:1766-1870 (kv_write / kv_append /
// kv_append_rot kernels) and csrc/rotate.cu:40-69 of the reference.
#include "kv_quant_row.cuh"
#include "msaq_common.cuh"
#include "sm100_ptx.cuh"

namespace msaq {
namespace {

constexpr int ROWS_PER_CTA = 4;   // warps per block, one row each

struct RowMap {
    int64_t rows;            // total rows = heads * rows_per_head
    int64_t rows_per_head;   // 1 for append, L for prefill write
    int64_t key0;            // first slot (append: pos)
    int64_t Lcap;            // key stride of the planes
    const int32_t* pos;      // optional per-sequence slot (varlen append)
    int64_t heads_per_seq;   // Hkv, used with pos
    int* sticky;             // the library's per-device status word: bit BAD_APPEND_POS when a pos[] entry is out of range
    Rope rope;               // rotary embedding applied (before the Hadamard rotation) to jobs that ask for it
};

template <int EPL>
__global__ void __launch_bounds__(ROWS_PER_CTA * 32)
quantize_rows_kernel(const QuantJobs jobs, RowMap map, Fmt f) {
    chain_release();
    chain_wait();
    const QuantJob job = jobs.j[blockIdx.y];
    constexpr int D = 32 * EPL, NB = EPL;
    __shared__ float rowbuf[ROWS_PER_CTA][D];
    __shared__ uint32_t codes[ROWS_PER_CTA][NB][QROW_CW];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * ROWS_PER_CTA + warp;
    if (row >= map.rows) return;

    const int64_t head = row / map.rows_per_head;
    int64_t key = map.key0 + row % map.rows_per_head;
    if (map.pos) {
        // A position that comes from device memory cannot be checked by the host: a stale or negative
        // entry must not write outside the planes.  The row is skipped and the status word says so.
        key = map.pos[head / map.heads_per_seq];
        if (key < 0 || key >= map.Lcap) {
            if (lane == 0 && map.sticky) atomicOr(map.sticky, BAD_APPEND_POS);
            return;
        }
    }

    quantize_row_warp<EPL>(job, map.rope, row, head, key, map.Lcap, f, rowbuf[warp], &codes[warp][0][0], lane);
}

template <int EPL>
__global__ void __launch_bounds__(ROWS_PER_CTA * 32)
hadamard_rotate_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int64_t N) {
    chain_release();
    chain_wait();
    constexpr int D = 32 * EPL;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * ROWS_PER_CTA + warp;
    if (row >= N) return;
    float v[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) v[i] = __bfloat162float(x[row * D + lane * EPL + i]);
    fwht_warp<EPL>(v, lane);
    const float inv = (float)(1.0 / sqrt((double)D));
#pragma unroll
    for (int i = 0; i < EPL; ++i) out[row * D + lane * EPL + i] = __float2bfloat16_rn(v[i] * inv);
}

// One thread per (output row o, block) of the plain-MXINT8 weight packer (ms_lib/pack.py:546-566 of the
// reference): q = clip(rint(x / 2^e), +-127) in float64, planes [nb,32,OUT] and [nb,OUT,32].
__global__ void __launch_bounds__(128)
pack_weight_mxint8_kernel(const void* __restrict__ W, int w_is_bf16, int8_t* __restrict__ scale_exp,
                          int8_t* __restrict__ qweight, int8_t* __restrict__ qweight_cm, int64_t OUT, int64_t nb) {
    chain_release();
    chain_wait();
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= OUT * nb) return;
    const int64_t blk = t / OUT, o = t % OUT;
    float x[BLOCK];
    const int64_t base = o * nb * BLOCK + blk * BLOCK;
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < BLOCK; ++k) {
        x[k] = w_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(W)[base + k]) : static_cast<const float*>(W)[base + k];
        amax = fmaxf(amax, fabsf(x[k]));
    }
    const int e = block_exponent(amax);
    const double inv = pow2d(-e);
    if (scale_exp) scale_exp[blk * OUT + o] = (int8_t)e;
#pragma unroll
    for (int k = 0; k < BLOCK; ++k) {
        double q = rint((double)x[k] * inv);
        q = fmin(fmax(q, -127.0), 127.0);
        if (qweight) qweight[(blk * BLOCK + k) * OUT + o] = (int8_t)(int)q;
        if (qweight_cm) qweight_cm[(blk * OUT + o) * BLOCK + k] = (int8_t)(int)q;
    }
}

// One thread per (output row o, block): quantise 32 weights and scatter the
// bytes into whichever planes were requested.
__global__ void __launch_bounds__(128)
pack_weight_kernel(const void* __restrict__ W, int w_is_bf16, int8_t* __restrict__ scale_exp,
                   uint8_t* __restrict__ upper, uint8_t* __restrict__ shared,
                   uint8_t* __restrict__ upper_cm, uint8_t* __restrict__ shared_cm,
                   int64_t OUT, int64_t nb, Fmt f) {
    chain_release();
    chain_wait();
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= OUT * nb) return;
    const int64_t blk = t / OUT, o = t % OUT;      // consecutive threads -> consecutive columns
    float x[BLOCK];
    const int64_t base = o * nb * BLOCK + blk * BLOCK;
    if (w_is_bf16) {
        const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(W) + base;
#pragma unroll
        for (int k = 0; k < BLOCK; ++k) x[k] = __bfloat162float(w[k]);
    } else {
        const float* w = static_cast<const float*>(W) + base;
#pragma unroll
        for (int k = 0; k < BLOCK; ++k) x[k] = w[k];
    }
    int up[BLOCK], sh[16];
    const int e = quantize_block(x, f, up, sh);
    uint32_t uw[7], sw[3];
    pack_codes(up, BLOCK, f.wbits, uw, 7);
    pack_codes(sh, f.ng, f.u, sw, 3);
    if (scale_exp) scale_exp[blk * OUT + o] = (int8_t)e;
    for (int i = 0; i < f.UB; ++i) {
        const uint8_t b = (uint8_t)(uw[i >> 2] >> ((i & 3) * 8));
        if (upper) upper[(blk * f.UB + i) * OUT + o] = b;
        if (upper_cm) upper_cm[(blk * OUT + o) * f.UB + i] = b;
    }
    for (int i = 0; i < f.SB; ++i) {
        const uint8_t b = (uint8_t)(sw[i >> 2] >> ((i & 3) * 8));
        if (shared) shared[(blk * f.SB + i) * OUT + o] = b;
        if (shared_cm) shared_cm[(blk * OUT + o) * f.SB + i] = b;
    }
}

int launch_rows(const QuantJobs& jobs, int n_jobs, const RowMap& map, int64_t D, const Fmt& f, cudaStream_t st) {
    if (map.rows == 0) return MSAQ_OK;
    const dim3 grid((unsigned)((map.rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA), (unsigned)n_jobs);
    const dim3 block(ROWS_PER_CTA * 32);
    switch (D) {
        case 32:  launch_chained(quantize_rows_kernel<1>, grid, block, 0, st, jobs, map, f); break;
        case 64:  launch_chained(quantize_rows_kernel<2>, grid, block, 0, st, jobs, map, f); break;
        case 128: launch_chained(quantize_rows_kernel<4>, grid, block, 0, st, jobs, map, f); break;
        case 256: launch_chained(quantize_rows_kernel<8>, grid, block, 0, st, jobs, map, f); break;
        default: return fail(MSAQ_ERR_UNSUPPORTED, "head_dim %lld: must be 32, 64, 128 or 256", (long long)D);
    }
    count_launch();
    return check_launch("quantize_rows");
}

int check_rows(const RowMap& map, int64_t D, int64_t NB, int u, int gs, Fmt* f) {
    if (!make_fmt(u, gs, f)) return fail(MSAQ_ERR_UNSUPPORTED, "unsupported format u=%d gs=%d", u, gs);
    if (NB * BLOCK != D) return fail(MSAQ_ERR_ARG, "NB (%lld) must equal D/32 (D=%lld)", (long long)NB, (long long)D);
    if (map.rows < 0 || map.Lcap <= 0) return fail(MSAQ_ERR_ARG, "bad row count or capacity");
    if (!map.pos && (map.key0 < 0 || map.key0 + map.rows_per_head > map.Lcap))
        return fail(MSAQ_ERR_ARG, "slots [%lld, %lld) exceed the cache capacity %lld", (long long)map.key0,
                    (long long)(map.key0 + map.rows_per_head), (long long)map.Lcap);
    if (map.rope.cos) {
        if (!map.rope.sin) return fail(MSAQ_ERR_ARG, "rope_sin is null");
        // a row per position: every slot a row can go to needs its table row
        const int64_t need = map.pos ? map.Lcap : map.key0 + map.rows_per_head;
        if (map.rope.rows != 1 && map.rope.rows < need)
            return fail(MSAQ_ERR_ARG, "the RoPE tables have %lld rows, positions up to %lld are possible",
                        (long long)map.rope.rows, (long long)need - 1);
    }
    return MSAQ_OK;
}

int quantize_rows(const void* X, int8_t* se, uint8_t* up, uint8_t* sh, const RowMap& map, int64_t D,
                  int64_t NB, int u, int gs, bool rot, void* stream) {
    Fmt f;
    if (!X || !se || !up || !sh) return fail(MSAQ_ERR_ARG, "null pointer");
    if (int rc = check_rows(map, D, NB, u, gs, &f)) return rc;
    QuantJobs jobs{};
    jobs.j[0] = QuantJob{static_cast<const __nv_bfloat16*>(X), se, up, sh, rot ? 1 : 0, map.rope.cos ? 1 : 0, 0};
    return launch_rows(jobs, 1, map, D, f, static_cast<cudaStream_t>(stream));
}

}  // namespace
}  // namespace msaq

using namespace msaq;

extern "C" int msaq_kv_append(const void* X, int8_t* scale_exp, uint8_t* upper, uint8_t* shared, int64_t H,
                              int64_t D, int64_t NB, int64_t pos, int64_t Lcap, int u, int gs, void* stream) {
    RowMap m{H, 1, pos, Lcap, nullptr, 1, nullptr};
    return quantize_rows(X, scale_exp, upper, shared, m, D, NB, u, gs, false, stream);
}

extern "C" int msaq_kv_append_rot(const void* X, int8_t* scale_exp, uint8_t* upper, uint8_t* shared, int64_t H,
                                  int64_t D, int64_t NB, int64_t pos, int64_t Lcap, int u, int gs, void* stream) {
    RowMap m{H, 1, pos, Lcap, nullptr, 1, nullptr};
    return quantize_rows(X, scale_exp, upper, shared, m, D, NB, u, gs, true, stream);
}

extern "C" int msaq_kv_append_varlen(const void* X, int8_t* scale_exp, uint8_t* upper, uint8_t* shared, int64_t B,
                                     int64_t Hkv, int64_t D, int64_t NB, const int32_t* pos, int64_t Lcap, int u,
                                     int gs, int rotate, void* stream) {
    if (!pos) return fail(MSAQ_ERR_ARG, "pos is null");
    if (Hkv <= 0) return fail(MSAQ_ERR_ARG, "Hkv must be positive");
    RowMap m{B * Hkv, 1, 0, Lcap, pos, Hkv, sticky_status()};
    return quantize_rows(X, scale_exp, upper, shared, m, D, NB, u, gs, rotate != 0, stream);
}

extern "C" int msaq_kv_append_pair_rope(const void* Xk, const void* Xv, int8_t* k_scale_exp, uint8_t* k_upper,
                                        uint8_t* k_shared, int8_t* v_scale_exp, uint8_t* v_upper, uint8_t* v_shared,
                                        int64_t B, int64_t Hkv, int64_t D, int64_t NB, int64_t pos,
                                        const int32_t* pos_per_seq, int64_t Lcap, int u, int gs, int rotate_k,
                                        const float* rope_cos, const float* rope_sin, int64_t rope_rows,
                                        void* stream) {
    if (!Xk || !Xv || !k_scale_exp || !k_upper || !k_shared || !v_scale_exp || !v_upper || !v_shared)
        return fail(MSAQ_ERR_ARG, "null pointer");
    if (B <= 0 || Hkv <= 0) return fail(MSAQ_ERR_ARG, "B and Hkv must be positive");
    RowMap m{B * Hkv, 1, pos_per_seq ? 0 : pos, Lcap, pos_per_seq, Hkv, pos_per_seq ? sticky_status() : nullptr,
             Rope{rope_cos, rope_sin, rope_rows}};
    Fmt f;
    if (int rc = check_rows(m, D, NB, u, gs, &f)) return rc;
    QuantJobs jobs{};
    jobs.j[0] = QuantJob{static_cast<const __nv_bfloat16*>(Xk), k_scale_exp, k_upper, k_shared, rotate_k ? 1 : 0,
                         rope_cos ? 1 : 0, 0};
    jobs.j[1] = QuantJob{static_cast<const __nv_bfloat16*>(Xv), v_scale_exp, v_upper, v_shared, 0, 0, 0};
    return launch_rows(jobs, 2, m, D, f, static_cast<cudaStream_t>(stream));
}

extern "C" int msaq_kv_append_pair(const void* Xk, const void* Xv, int8_t* k_scale_exp, uint8_t* k_upper,
                                   uint8_t* k_shared, int8_t* v_scale_exp, uint8_t* v_upper, uint8_t* v_shared,
                                   int64_t B, int64_t Hkv, int64_t D, int64_t NB, int64_t pos, const int32_t* pos_per_seq,
                                   int64_t Lcap, int u, int gs, int rotate_k, void* stream) {
    return msaq_kv_append_pair_rope(Xk, Xv, k_scale_exp, k_upper, k_shared, v_scale_exp, v_upper, v_shared, B, Hkv, D, NB,
                                    pos, pos_per_seq, Lcap, u, gs, rotate_k, nullptr, nullptr, 0, stream);
}

extern "C" int msaq_kv_write_rope(const void* X, int8_t* scale_exp, uint8_t* upper, uint8_t* shared, int64_t H,
                                  int64_t L, int64_t D, int64_t NB, int64_t key0, int64_t Lcap, int u, int gs,
                                  int rotate, const float* rope_cos, const float* rope_sin, int64_t rope_rows,
                                  void* stream) {
    if (L < 0 || H < 0) return fail(MSAQ_ERR_ARG, "negative size");
    if (L == 0) return MSAQ_OK;
    RowMap m{H * L, L, key0, Lcap, nullptr, 1, nullptr, Rope{rope_cos, rope_sin, rope_rows}};
    return quantize_rows(X, scale_exp, upper, shared, m, D, NB, u, gs, rotate != 0, stream);
}

extern "C" int msaq_kv_write(const void* X, int8_t* scale_exp, uint8_t* upper, uint8_t* shared, int64_t H, int64_t L,
                             int64_t D, int64_t NB, int64_t key0, int64_t Lcap, int u, int gs, int rotate,
                             void* stream) {
    return msaq_kv_write_rope(X, scale_exp, upper, shared, H, L, D, NB, key0, Lcap, u, gs, rotate, nullptr, nullptr, 0,
                              stream);
}

extern "C" int msaq_hadamard_rotate(const void* x, void* out, int64_t N, int64_t D, void* stream) {
    if (!x || !out) return fail(MSAQ_ERR_ARG, "null pointer");
    if (N <= 0) return N == 0 ? MSAQ_OK : fail(MSAQ_ERR_ARG, "negative row count");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = (unsigned)((N + ROWS_PER_CTA - 1) / ROWS_PER_CTA);
    const __nv_bfloat16* xi = static_cast<const __nv_bfloat16*>(x);
    __nv_bfloat16* xo = static_cast<__nv_bfloat16*>(out);
    switch (D) {
        case 32:  launch_chained(hadamard_rotate_kernel<1>, dim3(grid), dim3(ROWS_PER_CTA * 32), 0, st, xi, xo, N); break;
        case 64:  launch_chained(hadamard_rotate_kernel<2>, dim3(grid), dim3(ROWS_PER_CTA * 32), 0, st, xi, xo, N); break;
        case 128: launch_chained(hadamard_rotate_kernel<4>, dim3(grid), dim3(ROWS_PER_CTA * 32), 0, st, xi, xo, N); break;
        case 256: launch_chained(hadamard_rotate_kernel<8>, dim3(grid), dim3(ROWS_PER_CTA * 32), 0, st, xi, xo, N); break;
        default: return fail(MSAQ_ERR_UNSUPPORTED, "rotate: last dim %lld must be 32, 64, 128 or 256", (long long)D);
    }
    count_launch();
    return check_launch("hadamard_rotate");
}

extern "C" int msaq_pack_weight(const void* W, int w_is_bf16, int8_t* scale_exp, uint8_t* upper, uint8_t* shared,
                                uint8_t* upper_cm, uint8_t* shared_cm, int64_t OUT, int64_t K, int u, int gs,
                                void* stream) {
    Fmt f;
    if (!make_fmt(u, gs, &f)) return fail(MSAQ_ERR_UNSUPPORTED, "unsupported format u=%d gs=%d", u, gs);
    if (!W) return fail(MSAQ_ERR_ARG, "W is null");
    if (OUT <= 0 || K <= 0 || K % BLOCK) return fail(MSAQ_ERR_ARG, "K must be a positive multiple of 32");
    const int64_t nb = K / BLOCK, total = OUT * nb;
    launch_chained(pack_weight_kernel, dim3((unsigned)((total + 127) / 128)), dim3(128), 0, static_cast<cudaStream_t>(stream), W, w_is_bf16, scale_exp, upper, shared, upper_cm, shared_cm, OUT, nb, f);
    count_launch();
    return check_launch("pack_weight");
}

// ---- plain MXINT8 (the reference's matched baseline format, csrc/mxint8.cu) ----------------------------
extern "C" int msaq_mxint8_pack_weight(const void* W, int w_is_bf16, int8_t* scale_exp, int8_t* qweight, int8_t* qweight_cm,
                                       int64_t OUT, int64_t K, void* stream) {
    if (!W) return fail(MSAQ_ERR_ARG, "W is null");
    if (OUT <= 0 || K <= 0 || K % BLOCK) return fail(MSAQ_ERR_ARG, "K must be a positive multiple of 32");
    const int64_t nb = K / BLOCK, total = OUT * nb;
    launch_chained(pack_weight_mxint8_kernel, dim3((unsigned)((total + 127) / 128)), dim3(128), 0,
                   static_cast<cudaStream_t>(stream), W, w_is_bf16, scale_exp, qweight, qweight_cm, OUT, nb);
    count_launch();
    return check_launch("pack_weight_mxint8");
}

namespace {
int mxint8_rows(const void* X, int8_t* se, int8_t* qw, const RowMap& map, int64_t D, int64_t NB, void* stream) {
    Fmt f;
    if (!X || !se || !qw) return fail(MSAQ_ERR_ARG, "null pointer");
    if (int rc = check_rows(map, D, NB, 4, 2, &f)) return rc;        // the format argument is unused by the MXINT8 rows
    QuantJobs jobs{};
    jobs.j[0] = QuantJob{static_cast<const __nv_bfloat16*>(X), se, reinterpret_cast<uint8_t*>(qw), nullptr, 0, 0, 1};
    return launch_rows(jobs, 1, map, D, f, static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" int msaq_mxint8_kv_append(const void* X, int8_t* scale_exp, int8_t* qweight, int64_t H, int64_t D, int64_t NB,
                                     int64_t pos, int64_t Lcap, void* stream) {
    RowMap m{H, 1, pos, Lcap, nullptr, 1, nullptr};
    return mxint8_rows(X, scale_exp, qweight, m, D, NB, stream);
}

extern "C" int msaq_mxint8_kv_write(const void* X, int8_t* scale_exp, int8_t* qweight, int64_t H, int64_t L, int64_t D,
                                    int64_t NB, int64_t key0, int64_t Lcap, void* stream) {
    if (L < 0 || H < 0) return fail(MSAQ_ERR_ARG, "negative size");
    if (L == 0) return MSAQ_OK;
    RowMap m{H * L, L, key0, Lcap, nullptr, 1, nullptr};
    return mxint8_rows(X, scale_exp, qweight, m, D, NB, stream);
}

// Host side of the KV flash-decode entry points: argument checks, the split-KV
// plan, kernel selection.  Replaces the launchers at
// csrc/kv_attention.cu:1875-2122 of the reference.
#include "kv_decode_generic.cuh"
#include "kv_decode_mma.cuh"

namespace msaq {
namespace {

struct KvPlan {
    int S;          // key tiles per (sequence, head)
    int key_tile;   // keys per tile (multiple of the chunk)
};

KvPlan plan_generic(int64_t B, int64_t H, int64_t Lk) {
    KvPlan p;
    const int64_t heads = B * H;
    int64_t want = (3LL * sm_count() + heads - 1) / heads;
    const int64_t max_tiles = (Lk + KVG_CHUNK - 1) / KVG_CHUNK;
    if (want > max_tiles) want = max_tiles;
    if (want < 1) want = 1;
    int64_t tile = (Lk + want - 1) / want;
    tile = (tile + KVG_CHUNK - 1) / KVG_CHUNK * KVG_CHUNK;
    p.key_tile = (int)tile;
    p.S = (int)((Lk + tile - 1) / tile);
    return p;
}

// ---- tuned path: u4/gs2, D = 128, G in {1,2,4,8}, capacity a multiple of 16 ----------------
bool mma_eligible(int64_t H, int64_t Hkv, int64_t D, int u, int gs, int64_t Lcap) {
    const int64_t G = H / Hkv;
    return u == 4 && gs == 2 && D == 128 && (G == 1 || G == 2 || G == 4 || G == 8) && Lcap % 16 == 0;
}

struct KvMmaPlan {
    int S, key_tile, cps;
    size_t status_off, total;
};

KvMmaPlan plan_mma(int64_t B, int64_t H, int64_t Hkv, int64_t Lk) {
    KvMmaPlan p;
    const int64_t pairs = B * Hkv;
    // Tiles per (sequence, kv head).  Enough CTAs for about four waves of resident CTAs, so that
    // the pipeline fill and the tail of one CTA overlap with the steady state of others -- but no
    // tile shorter than 1024 keys (query staging, pipeline fill and merge are fixed costs per tile),
    // except to fill one wave when the whole problem is small.
    // thread blocks per SM: three (two-stage ring) from 64 MB of cache on, two (three-stage ring) below
    p.cps = B * Hkv * Lk * 200 >= (64LL << 20) ? 3 : 2;
    const int64_t slots = (int64_t)p.cps * sm_count();
    int64_t want = (4 * slots + pairs - 1) / pairs;
    const int64_t by_size = Lk / 1024;
    int64_t one_wave = slots / pairs;
    if (one_wave > (Lk + KVM_TK - 1) / KVM_TK) one_wave = (Lk + KVM_TK - 1) / KVM_TK;
    const int64_t cap = by_size > one_wave ? by_size : one_wave;
    if (want > cap) want = cap;
    if (want < 1) want = 1;
    int64_t tile = (Lk + want - 1) / want;
    tile = (tile + KVM_TK - 1) / KVM_TK * KVM_TK;
    p.key_tile = (int)tile;
    p.S = (int)((Lk + tile - 1) / tile);
    const size_t part = (((size_t)B * H * p.S * 130 * sizeof(float)) + 255) & ~(size_t)255;
    p.status_off = part;
    p.total = part + 256;
    return p;
}

template <int G, int FMT, int CPS>
int launch_kv_mma_cps(const KvMmaArgs& a, int S, int Hkv, int B, cudaStream_t st) {
    static bool configured[64] = {};
    constexpr int smem = kvm_smem_bytes(FMT, CPS);
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kv_decode_u4gs2_kernel<G, FMT, CPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess)
            return fail(MSAQ_ERR_CUDA, "cannot reserve %d bytes of shared memory", smem);
        configured[dev] = true;
    }
    launch_chained(kv_decode_u4gs2_kernel<G, FMT, CPS>, dim3((unsigned)S, (unsigned)Hkv, (unsigned)B), dim3(KVM_THREADS), smem, st, a);
    count_launch();
    return check_launch(FMT == KVF_MXINT8 ? "kv_decode_mxint8" : "kv_decode_u4gs2");
}

template <int G, int FMT = KVF_MSAQ_U4>
int launch_kv_mma(const KvMmaArgs& a, int S, int Hkv, int B, int cps, cudaStream_t st) {
    return cps == 3 ? launch_kv_mma_cps<G, FMT, 3>(a, S, Hkv, B, st) : launch_kv_mma_cps<G, FMT, 2>(a, S, Hkv, B, st);
}

struct QRope {
    Rope rope;
    int64_t q_pos;
    const int32_t* q_pos_per_seq;
};

// The step's new token, to be appended by the decode kernel itself (see KvMmaArgs).
struct KvAppend {
    const void* k_new;
    const void* v_new;
    int64_t pos;
    const int32_t* pos_per_seq;
    int rotate_k;
};

int run_mma(const __nv_bfloat16* q, KvPlanes kp, KvPlanes vp, void* out, float* out_f32, const int32_t* seq_lens,
            int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t Lcap, int qrot, const QRope& qr, void* ws,
            cudaStream_t st, int fmt = KVF_MSAQ_U4, const KvAppend* app = nullptr) {
    const KvMmaPlan p = plan_mma(B, H, Hkv, Lk);
    Fmt f4{};
    make_fmt(4, 2, &f4);
    uint8_t* base = static_cast<uint8_t*>(ws) + WS_CTL_BYTES;
    int* status = reinterpret_cast<int*>(base + p.status_off);
    KvMmaArgs a{q, kp, vp, reinterpret_cast<float*>(base), seq_lens, status, sticky_status(), (int)H, (int)Hkv, (int)Lk,
                (int)Lcap, p.key_tile, p.S, qrot, (float)(1.4426950408889634 / sqrt(128.0)), qr.rope, qr.q_pos,
                qr.q_pos_per_seq, KVM_SPLIT_TAU, option_wait_polls(), option_test_skip_stage(),
                app ? static_cast<const __nv_bfloat16*>(app->k_new) : nullptr,
                app ? static_cast<const __nv_bfloat16*>(app->v_new) : nullptr, app ? app->pos : 0,
                app ? app->pos_per_seq : nullptr, app ? app->rotate_k : 0, f4};
    int rc;
    if (fmt == KVF_MXINT8) {
        switch (H / Hkv) {
            case 1: rc = launch_kv_mma<1, KVF_MXINT8>(a, p.S, (int)Hkv, (int)B, p.cps, st); break;
            case 2: rc = launch_kv_mma<2, KVF_MXINT8>(a, p.S, (int)Hkv, (int)B, p.cps, st); break;
            case 4: rc = launch_kv_mma<4, KVF_MXINT8>(a, p.S, (int)Hkv, (int)B, p.cps, st); break;
            default: rc = launch_kv_mma<8, KVF_MXINT8>(a, p.S, (int)Hkv, (int)B, p.cps, st); break;
        }
    } else
    switch (H / Hkv) {
        case 1: rc = launch_kv_mma<1>(a, p.S, (int)Hkv, (int)B, p.cps, st); break;
        case 2: rc = launch_kv_mma<2>(a, p.S, (int)Hkv, (int)B, p.cps, st); break;
        case 4: rc = launch_kv_mma<4>(a, p.S, (int)Hkv, (int)B, p.cps, st); break;
        default: rc = launch_kv_mma<8>(a, p.S, (int)Hkv, (int)B, p.cps, st); break;
    }
    if (rc) return rc;
    launch_chained(kv_decode_combine2_kernel, dim3((unsigned)H, (unsigned)B), dim3(128), 0, st,
                   reinterpret_cast<const float*>(base), static_cast<__nv_bfloat16*>(out), out_f32, (int)H, p.S);
    count_launch();
    return check_launch("kv_decode_combine2");
}

int decode_dispatch(const void* q, KvPlanes kp, KvPlanes vp, void* out, float* out_f32, const int32_t* seq_lens,
                    int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D, int64_t NB, int u, int gs,
                    int64_t Lcap, int qrot, const QRope& qr, void* ws, size_t ws_bytes, void* stream,
                    const KvAppend* app = nullptr) {
    Fmt f;
    if (qr.rope.cos) {
        if (!qr.rope.sin || qr.rope.rows < 1) return fail(MSAQ_ERR_ARG, "bad RoPE tables");
        if (!qr.q_pos_per_seq && qr.rope.rows != 1 && (qr.q_pos < 0 || qr.q_pos >= qr.rope.rows))
            return fail(MSAQ_ERR_ARG, "query position %lld outside the %lld RoPE table rows", (long long)qr.q_pos,
                        (long long)qr.rope.rows);
    }
    if (!make_fmt(u, gs, &f)) return fail(MSAQ_ERR_UNSUPPORTED, "unsupported format u=%d gs=%d", u, gs);
    if (!q || !kp.s || !kp.u || !kp.h || !vp.s || !vp.u || !vp.h || !out) return fail(MSAQ_ERR_ARG, "null pointer");
    if (B <= 0 || H <= 0 || Hkv <= 0 || Lk <= 0) return fail(MSAQ_ERR_ARG, "B, H, Hkv and Lk must be positive");
    if (H % Hkv) return fail(MSAQ_ERR_ARG, "H (%lld) must be a multiple of Hkv (%lld)", (long long)H, (long long)Hkv);
    if (D != 32 && D != 64 && D != 128 && D != 256)
        return fail(MSAQ_ERR_UNSUPPORTED, "head_dim %lld: must be 32, 64, 128 or 256", (long long)D);
    if (NB * BLOCK != D) return fail(MSAQ_ERR_ARG, "NB (%lld) must equal D/32 (D=%lld)", (long long)NB, (long long)D);
    if (Lcap < 0) Lcap = Lk;
    if (Lcap < Lk) return fail(MSAQ_ERR_ARG, "Lcap (%lld) is smaller than Lk (%lld)", (long long)Lcap, (long long)Lk);
    if (Lk > INT32_MAX || Lcap > INT32_MAX || B > 65535 || H > INT32_MAX)
        return fail(MSAQ_ERR_ARG, "size exceeds the supported range");
    if ((reinterpret_cast<uintptr_t>(kp.u) | reinterpret_cast<uintptr_t>(vp.u)) & 3)
        return fail(MSAQ_ERR_ARG, "upper planes must be 4-byte aligned");
    if (int rc = require_sm100()) return rc;
    const size_t need = msaq_kv_decode_workspace(B, H, Hkv, Lk, D);
    if (!ws || ws_bytes < need)
        return fail(MSAQ_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, ws ? ws_bytes : (size_t)0);

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (mma_eligible(H, Hkv, D, u, gs, Lcap) &&
        !((reinterpret_cast<uintptr_t>(kp.s) | reinterpret_cast<uintptr_t>(kp.u) | reinterpret_cast<uintptr_t>(kp.h) |
           reinterpret_cast<uintptr_t>(vp.s) | reinterpret_cast<uintptr_t>(vp.u) | reinterpret_cast<uintptr_t>(vp.h)) & 15))
        return run_mma(static_cast<const __nv_bfloat16*>(q), kp, vp, out, out_f32, seq_lens, B, H, Hkv, Lk, Lcap, qrot,
                       qr, ws, st, KVF_MSAQ_U4, app);
    if (app) {           // the generic kernels take the token from the cache: append it with the kernel of its own first
        if (int rc = msaq_kv_append_pair_rope(app->k_new, app->v_new, const_cast<int8_t*>(kp.s), const_cast<uint8_t*>(kp.u),
                                              const_cast<uint8_t*>(kp.h), const_cast<int8_t*>(vp.s), const_cast<uint8_t*>(vp.u),
                                              const_cast<uint8_t*>(vp.h), B, Hkv, D, NB, app->pos, app->pos_per_seq, Lcap, u, gs,
                                              app->rotate_k, qr.rope.cos, qr.rope.sin, qr.rope.rows, stream))
            return rc;
    }
    const KvPlan p = plan_generic(B, H, Lk);
    const float sm_scale = (float)(1.0 / sqrt((double)D));
    float* partial = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + WS_CTL_BYTES);
    const __nv_bfloat16* qq = static_cast<const __nv_bfloat16*>(q);
    dim3 grid((unsigned)H, (unsigned)p.S, (unsigned)B);
    const size_t smem = ((size_t)D + KVG_CHUNK) * sizeof(float);
#define MSAQ_GO(U) launch_chained(kv_decode_generic_kernel<U>, grid, dim3(KVG_THREADS), smem, st, \
        qq, kp, vp, partial, seq_lens, (int)H, (int)Hkv, (int)Lk, (int)Lcap, (int)D, (int)NB, f, p.key_tile, p.S, \
        sm_scale, qrot, qr.rope, qr.q_pos, qr.q_pos_per_seq)
    if (u == 4) MSAQ_GO(4); else if (u == 3) MSAQ_GO(3); else MSAQ_GO(2);
#undef MSAQ_GO
    count_launch();
    if (int rc = check_launch("kv_decode_generic")) return rc;
    launch_chained(kv_decode_combine_kernel, dim3((unsigned)H, (unsigned)B), dim3(128), 0, st,
                   static_cast<const float*>(partial), static_cast<__nv_bfloat16*>(out), out_f32, (int)H, (int)D, p.S);
    count_launch();
    return check_launch("kv_decode_combine");
}

}  // namespace
}  // namespace msaq

using namespace msaq;

extern "C" size_t msaq_kv_decode_workspace(int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D) {
    if (B <= 0 || H <= 0 || Lk <= 0 || D <= 0) return 0;
    const KvPlan p = plan_generic(B, H, Lk);
    size_t bytes = (size_t)B * H * p.S * kv_partial_stride((int)D) * sizeof(float);
    bytes = (bytes + 255) & ~(size_t)255;
    if (D == 128 && Hkv > 0 && H % Hkv == 0) {
        const size_t tuned = plan_mma(B, H, Hkv, Lk).total;
        if (tuned > bytes) bytes = tuned;
    }
    return bytes + WS_CTL_BYTES;
}

extern "C" int msaq_kv_decode_attention(const void* q, const int8_t* ks, const uint8_t* ku, const uint8_t* kh,
                                        const int8_t* vs, const uint8_t* vu, const uint8_t* vh, void* out,
                                        float* out_f32, int64_t H, int64_t Hkv, int64_t Lk, int64_t D, int64_t NB,
                                        int u, int gs, int64_t Lcap, void* workspace, size_t workspace_bytes,
                                        void* stream) {
    return decode_dispatch(q, KvPlanes{ks, ku, kh}, KvPlanes{vs, vu, vh}, out, out_f32, nullptr, 1, H, Hkv, Lk, D, NB,
                           u, gs, Lcap, 0, QRope{}, workspace, workspace_bytes, stream);
}

extern "C" int msaq_kv_decode_attention_batched(const void* q, const int8_t* ks, const uint8_t* ku, const uint8_t* kh,
                                                const int8_t* vs, const uint8_t* vu, const uint8_t* vh, void* out,
                                                float* out_f32, const int32_t* seq_lens, int64_t B, int64_t H,
                                                int64_t Hkv, int64_t Lk, int64_t D, int64_t NB, int u, int gs,
                                                int64_t Lcap, int qrot, void* workspace, size_t workspace_bytes,
                                                void* stream) {
    return decode_dispatch(q, KvPlanes{ks, ku, kh}, KvPlanes{vs, vu, vh}, out, out_f32, seq_lens, B, H, Hkv, Lk, D, NB,
                           u, gs, Lcap, qrot, QRope{}, workspace, workspace_bytes, stream);
}

extern "C" int msaq_kv_decode_attention_rope(const void* q, const int8_t* ks, const uint8_t* ku, const uint8_t* kh,
                                             const int8_t* vs, const uint8_t* vu, const uint8_t* vh, void* out,
                                             float* out_f32, const int32_t* seq_lens, int64_t B, int64_t H, int64_t Hkv,
                                             int64_t Lk, int64_t D, int64_t NB, int u, int gs, int64_t Lcap, int qrot,
                                             const float* rope_cos, const float* rope_sin, int64_t rope_rows,
                                             int64_t q_pos, const int32_t* q_pos_per_seq, void* workspace,
                                             size_t workspace_bytes, void* stream) {
    return decode_dispatch(q, KvPlanes{ks, ku, kh}, KvPlanes{vs, vu, vh}, out, out_f32, seq_lens, B, H, Hkv, Lk, D, NB,
                           u, gs, Lcap, qrot, QRope{Rope{rope_cos, rope_sin, rope_rows}, q_pos, q_pos_per_seq}, workspace,
                           workspace_bytes, stream);
}

extern "C" int msaq_kv_decode_attention_append(const void* q, const void* k_new, const void* v_new, int8_t* ks, uint8_t* ku,
                                               uint8_t* kh, int8_t* vs, uint8_t* vu, uint8_t* vh, void* out, float* out_f32,
                                               const int32_t* seq_lens, int64_t B, int64_t H, int64_t Hkv, int64_t Lk,
                                               int64_t D, int64_t NB, int u, int gs, int64_t Lcap, int rotate_k, int qrot,
                                               const float* rope_cos, const float* rope_sin, int64_t rope_rows,
                                               int64_t pos, const int32_t* pos_per_seq, void* workspace,
                                               size_t workspace_bytes, void* stream) {
    if (!k_new || !v_new) return fail(MSAQ_ERR_ARG, "null pointer");
    if ((reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new)) & 7)
        return fail(MSAQ_ERR_ARG, "k_new and v_new must be 8-byte aligned");
    const int64_t cap = Lcap < 0 ? Lk : Lcap;
    if (!pos_per_seq && (pos < 0 || pos >= cap))
        return fail(MSAQ_ERR_ARG, "pos %lld outside the capacity %lld", (long long)pos, (long long)cap);
    if (rope_cos && !pos_per_seq && rope_rows != 1 && pos >= rope_rows)
        return fail(MSAQ_ERR_ARG, "pos %lld outside the %lld RoPE table rows", (long long)pos, (long long)rope_rows);
    const KvAppend app{k_new, v_new, pos, pos_per_seq, rotate_k};
    return decode_dispatch(q, KvPlanes{ks, ku, kh}, KvPlanes{vs, vu, vh}, out, out_f32, seq_lens, B, H, Hkv, Lk, D, NB,
                           u, gs, Lcap, qrot, QRope{Rope{rope_cos, rope_sin, rope_rows}, pos, pos_per_seq}, workspace,
                           workspace_bytes, stream, &app);
}

// ---- plain MXINT8 caches (the reference's matched baseline, csrc/mxint8.cu:750-912) ---------------------
extern "C" int msaq_mxint8_kv_decode_batched(const void* q, const int8_t* ks, const int8_t* kq, const int8_t* vs,
                                             const int8_t* vq, void* out, float* out_f32, const int32_t* seq_lens,
                                             int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D, int64_t NB,
                                             int64_t Lcap, void* workspace, size_t workspace_bytes, void* stream) {
    if (!q || !ks || !kq || !vs || !vq || !out) return fail(MSAQ_ERR_ARG, "null pointer");
    if (B <= 0 || H <= 0 || Hkv <= 0 || Lk <= 0) return fail(MSAQ_ERR_ARG, "B, H, Hkv and Lk must be positive");
    if (H % Hkv) return fail(MSAQ_ERR_ARG, "H (%lld) must be a multiple of Hkv (%lld)", (long long)H, (long long)Hkv);
    if (Lcap < 0) Lcap = Lk;
    if (Lcap < Lk) return fail(MSAQ_ERR_ARG, "Lcap (%lld) is smaller than Lk (%lld)", (long long)Lcap, (long long)Lk);
    if (Lk > INT32_MAX || Lcap > INT32_MAX || B > 65535) return fail(MSAQ_ERR_ARG, "size exceeds the supported range");
    // the baseline twin exists for the configuration the tuned MSAQ kernel serves, so that the two compare like for like
    if (!mma_eligible(H, Hkv, D, 4, 2, Lcap) || NB * BLOCK != D)
        return fail(MSAQ_ERR_UNSUPPORTED, "the MXINT8 decode serves head_dim 128, Hq/Hkv in {1,2,4,8} and capacities that are multiples of 16");
    if ((reinterpret_cast<uintptr_t>(ks) | reinterpret_cast<uintptr_t>(kq) | reinterpret_cast<uintptr_t>(vs) |
         reinterpret_cast<uintptr_t>(vq)) & 15)
        return fail(MSAQ_ERR_ARG, "cache planes must be 16-byte aligned");
    if (int rc = require_sm100()) return rc;
    const size_t need = msaq_kv_decode_workspace(B, H, Hkv, Lk, D);
    if (!workspace || workspace_bytes < need)
        return fail(MSAQ_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, workspace ? workspace_bytes : (size_t)0);
    return run_mma(static_cast<const __nv_bfloat16*>(q), KvPlanes{ks, reinterpret_cast<const uint8_t*>(kq), nullptr},
                   KvPlanes{vs, reinterpret_cast<const uint8_t*>(vq), nullptr}, out, out_f32, seq_lens, B, H, Hkv, Lk, Lcap, 0,
                   QRope{}, workspace, static_cast<cudaStream_t>(stream), KVF_MXINT8);
}

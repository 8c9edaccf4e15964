// `ms_cuda`: the torch operator surface of the decode path.
//
// Importing the module registers torch.ops.msaq.* with the schemas of the
// reference (csrc/pybind.cpp:198-286); each op checks its tensors, allocates
// outputs and scratch through torch's caching allocator, and forwards to the C
// ABI in include/msaq_b200.h on the current CUDA stream.  No host sync, so the
// ops can be captured in CUDA graphs.
#include <Python.h>

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cstdlib>

#include "../../include/msaq_b200.h"

namespace {

using at::Tensor;

void check_rc(int rc, const char* op) {
    TORCH_CHECK(rc == MSAQ_OK, "msaq::", op, " failed (", rc, "): ", msaq_last_error());
}

void check_act(const Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, name, " must be a CUDA bf16 tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

void check_plane(const Tensor& t, at::ScalarType ty, const Tensor& like, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == ty, name, " has the wrong dtype or is not on CUDA");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(t.device() == like.device(), name, " is on a different device than the activation");
}

void check_planes(const Tensor& s, const Tensor& u, const Tensor& h, const Tensor& like, int64_t n_blocks, int64_t UB,
                  int64_t SB) {
    check_plane(s, at::kChar, like, "scale_exp");
    check_plane(u, at::kByte, like, "upper");
    check_plane(h, at::kByte, like, "shared");
    TORCH_CHECK(s.numel() >= n_blocks, "scale_exp holds ", s.numel(), " blocks, ", n_blocks, " needed");
    TORCH_CHECK(u.numel() >= n_blocks * UB, "upper plane too small");
    TORCH_CHECK(h.numel() >= n_blocks * SB, "shared plane too small");
}

void fmt_sizes(int64_t u, int64_t gs, int64_t* UB, int64_t* SB) {
    TORCH_CHECK(u >= 2 && u <= 4, "u must be 2, 3 or 4");
    TORCH_CHECK(gs == 2 || gs == 4 || gs == 8 || gs == 16 || gs == 32, "gs must be a power of two in [2, 32]");
    *UB = 32 * (8 - u) / 8;
    *SB = ((32 / gs) * u + 7) / 8;
}

void* stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

// Scratch for one call.  Always more than 1 MiB, so that torch's caching allocator serves it from its
// large-block pool: the control region at the start of a workspace (the GEMV's tile counters, zero at
// rest) then shares memory only with other workspaces, which leave that region alone, and not with
// small output tensors.
Tensor workspace(const Tensor& like, size_t bytes) {
    const size_t floor_bytes = (1u << 20) + 512;
    return at::empty({(int64_t)(bytes > floor_bytes ? bytes : floor_bytes)}, like.options().dtype(at::kByte));
}

// ---- GEMV ---------------------------------------------------------------
Tensor gemv_common(const Tensor& x, const Tensor& s, const Tensor& up, const Tensor& sh, int64_t M, int64_t OUT,
                   int64_t NB, int64_t u, int64_t gs, int kind) {
    check_act(x, "x");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(M >= 1 && OUT >= 1 && NB >= 1, "M, OUT and NB must be positive");
    TORCH_CHECK(x.numel() == M * NB * 32, "x has ", x.numel(), " elements, expected M*K = ", M * NB * 32);
    check_planes(s, up, sh, x, NB * OUT, UB, SB);
    c10::cuda::CUDAGuard guard(x.device());
    Tensor y = kind == 2 ? at::empty({M, OUT}, x.options()) : at::empty({OUT}, x.options());
    const size_t wsb = msaq_wonly_gemv_workspace(M, OUT, NB, (int)u, (int)gs);
    Tensor ws = workspace(x, wsb);
    int rc;
    if (kind == 0)
        rc = msaq_wonly_gemv(x.data_ptr(), s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(), sh.data_ptr<uint8_t>(),
                             y.data_ptr(), nullptr, OUT, NB, (int)u, (int)gs, ws.data_ptr(), wsb, stream_of(x));
    else if (kind == 1)
        rc = msaq_wonly_gemv_wide(x.data_ptr(), s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(), sh.data_ptr<uint8_t>(),
                                  y.data_ptr(), nullptr, OUT, NB, (int)u, (int)gs, ws.data_ptr(), wsb, stream_of(x));
    else
        rc = msaq_wonly_gemv_batched(x.data_ptr(), s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(),
                                     sh.data_ptr<uint8_t>(), y.data_ptr(), nullptr, M, OUT, NB, (int)u, (int)gs,
                                     ws.data_ptr(), wsb, stream_of(x));
    check_rc(rc, kind == 0 ? "wonly_gemv" : kind == 1 ? "wonly_gemv_wide" : "wonly_gemv_batched");
    return y;
}

// The batched GEMV with its fp32 result (before the bf16 rounding): what a K-sharded linear hands to the all-reduce.
Tensor wonly_gemv_batched_f32(const Tensor& x, const Tensor& s, const Tensor& up, const Tensor& sh, int64_t M, int64_t OUT,
                              int64_t NB, int64_t u, int64_t gs) {
    check_act(x, "x");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(M >= 1 && OUT >= 1 && NB >= 1, "M, OUT and NB must be positive");
    TORCH_CHECK(x.numel() == M * NB * 32, "x has ", x.numel(), " elements, expected M*K = ", M * NB * 32);
    check_planes(s, up, sh, x, NB * OUT, UB, SB);
    c10::cuda::CUDAGuard guard(x.device());
    Tensor y = at::empty({M, OUT}, x.options());
    Tensor yf = at::empty({M, OUT}, x.options().dtype(at::kFloat));
    const size_t wsb = msaq_wonly_gemv_workspace(M, OUT, NB, (int)u, (int)gs);
    Tensor ws = workspace(x, wsb);
    check_rc(msaq_wonly_gemv_batched(x.data_ptr(), s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(), sh.data_ptr<uint8_t>(),
                                     y.data_ptr(), yf.data_ptr<float>(), M, OUT, NB, (int)u, (int)gs, ws.data_ptr(), wsb,
                                     stream_of(x)),
             "wonly_gemv_batched_f32");
    return yf;
}

// y (and, for the add+rmsnorm prologue, the new residual stream) of a GEMV whose preceding glue is fused in.
std::vector<Tensor> wonly_gemv_fused(const Tensor& x, const c10::optional<Tensor>& addend, int64_t prologue, double eps,
                                     const Tensor& s, const Tensor& up, const Tensor& sh, int64_t M, int64_t OUT,
                                     int64_t NB, int64_t u, int64_t gs, bool out_f32) {
    check_act(x, "x");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(M >= 1 && OUT >= 1 && NB >= 1, "M, OUT and NB must be positive");
    const int64_t K = NB * 32;
    TORCH_CHECK(x.numel() == M * K * (prologue == MSAQ_PRO_SILU_MUL ? 2 : 1), "x has ", x.numel(), " elements");
    check_planes(s, up, sh, x, NB * OUT, UB, SB);
    c10::cuda::CUDAGuard guard(x.device());
    const void* ad = nullptr;
    int ad_f32 = 0;
    Tensor h_out;
    if (prologue == MSAQ_PRO_ADD_RMSNORM) {
        TORCH_CHECK(addend.has_value(), "the add+rmsnorm prologue needs an addend");
        const Tensor& a = *addend;
        TORCH_CHECK(a.is_cuda() && a.is_contiguous() && a.numel() == M * K, "addend must be a contiguous CUDA tensor [M, K]");
        TORCH_CHECK(a.scalar_type() == at::kFloat || a.scalar_type() == at::kBFloat16, "addend must be fp32 or bf16");
        ad = a.data_ptr();
        ad_f32 = a.scalar_type() == at::kFloat;
        h_out = at::empty({M, K}, x.options());
    }
    Tensor y = at::empty({M, OUT}, x.options());
    Tensor yf;
    if (out_f32) yf = at::empty({M, OUT}, x.options().dtype(at::kFloat));
    const size_t wsb = msaq_wonly_gemv_fused_workspace(M, OUT, NB, (int)u, (int)gs);
    Tensor ws = workspace(x, wsb);
    check_rc(msaq_wonly_gemv_fused(x.data_ptr(), (int)prologue, ad, ad_f32, (float)eps,
                                   h_out.defined() ? h_out.data_ptr() : nullptr, s.data_ptr<int8_t>(),
                                   up.data_ptr<uint8_t>(), sh.data_ptr<uint8_t>(), y.data_ptr(),
                                   out_f32 ? yf.data_ptr<float>() : nullptr, M, OUT, NB, (int)u, (int)gs, ws.data_ptr(), wsb,
                                   stream_of(x)),
             "wonly_gemv_fused");
    if (h_out.defined()) return {out_f32 ? yf : y, h_out};
    return {out_f32 ? yf : y};
}

Tensor wonly_gemv(const Tensor& x, const Tensor& s, const Tensor& up, const Tensor& sh, int64_t OUT, int64_t NB,
                  int64_t u, int64_t gs) {
    return gemv_common(x, s, up, sh, 1, OUT, NB, u, gs, 0);
}
Tensor wonly_gemv_wide(const Tensor& x, const Tensor& s, const Tensor& up, const Tensor& sh, int64_t OUT, int64_t NB,
                       int64_t u, int64_t gs) {
    return gemv_common(x, s, up, sh, 1, OUT, NB, u, gs, 1);
}
Tensor wonly_gemv_batched(const Tensor& x, const Tensor& s, const Tensor& up, const Tensor& sh, int64_t M, int64_t OUT,
                          int64_t NB, int64_t u, int64_t gs) {
    return gemv_common(x, s, up, sh, M, OUT, NB, u, gs, 2);
}

// ---- KV write paths -------------------------------------------------------
void append_common(const Tensor& X, Tensor& s, Tensor& up, Tensor& sh, int64_t H, int64_t D, int64_t NB, int64_t pos,
                   int64_t Lcap, int64_t u, int64_t gs, bool rot) {
    check_act(X, "X");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(X.numel() == H * D, "X must hold H*D elements");
    TORCH_CHECK(pos >= 0 && pos < Lcap, "pos ", pos, " is outside the cache capacity ", Lcap);
    check_planes(s, up, sh, X, H * NB * Lcap, UB, SB);
    c10::cuda::CUDAGuard guard(X.device());
    const int rc = rot ? msaq_kv_append_rot(X.data_ptr(), s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(),
                                            sh.data_ptr<uint8_t>(), H, D, NB, pos, Lcap, (int)u, (int)gs, stream_of(X))
                       : msaq_kv_append(X.data_ptr(), s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(),
                                        sh.data_ptr<uint8_t>(), H, D, NB, pos, Lcap, (int)u, (int)gs, stream_of(X));
    check_rc(rc, rot ? "kv_append_rot" : "kv_append");
}

void kv_append(const Tensor& X, Tensor s, Tensor up, Tensor sh, int64_t H, int64_t D, int64_t NB, int64_t pos,
               int64_t Lcap, int64_t u, int64_t gs) {
    append_common(X, s, up, sh, H, D, NB, pos, Lcap, u, gs, false);
}
void kv_append_rot(const Tensor& X, Tensor s, Tensor up, Tensor sh, int64_t H, int64_t D, int64_t NB, int64_t pos,
                   int64_t Lcap, int64_t u, int64_t gs) {
    append_common(X, s, up, sh, H, D, NB, pos, Lcap, u, gs, true);
}

void kv_append_varlen(const Tensor& X, Tensor s, Tensor up, Tensor sh, const Tensor& pos, int64_t B, int64_t Hkv,
                      int64_t D, int64_t NB, int64_t Lcap, int64_t u, int64_t gs, bool rotate) {
    check_act(X, "X");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(X.numel() == B * Hkv * D, "X must hold B*Hkv*D elements");
    TORCH_CHECK(pos.is_cuda() && pos.scalar_type() == at::kInt && pos.is_contiguous() && pos.numel() == B,
                "pos must be a contiguous CUDA int32 tensor of B elements");
    check_planes(s, up, sh, X, B * Hkv * NB * Lcap, UB, SB);
    c10::cuda::CUDAGuard guard(X.device());
    check_rc(msaq_kv_append_varlen(X.data_ptr(), s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(), sh.data_ptr<uint8_t>(),
                                   B, Hkv, D, NB, pos.data_ptr<int32_t>(), Lcap, (int)u, (int)gs, rotate ? 1 : 0,
                                   stream_of(X)),
             "kv_append_varlen");
}

// K (rotated when asked) and V rows of one decode step in one launch; pos_t (int32 [B]) overrides pos when given.
// RoPE tables: fp32 [rows, D/2], contiguous, on x's device (rows == 1: one position for all sequences).
void check_rope(const Tensor& cos, const Tensor& sin, const Tensor& like, int64_t D) {
    TORCH_CHECK(cos.is_cuda() && sin.is_cuda() && cos.get_device() == like.get_device() &&
                sin.get_device() == like.get_device(), "RoPE tables must be on the activations' device");
    TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat && cos.is_contiguous() &&
                sin.is_contiguous() && cos.dim() == 2 && cos.sizes() == sin.sizes() && cos.size(1) == D / 2,
                "RoPE tables must be contiguous fp32 [rows, D/2]");
}

void kv_append_pair_impl(const Tensor& Xk, const Tensor& Xv, Tensor ks, Tensor ku, Tensor kh, Tensor vs, Tensor vu, Tensor vh,
                    const c10::optional<Tensor>& pos_t, int64_t B, int64_t Hkv, int64_t D, int64_t NB, int64_t pos,
                    int64_t Lcap, int64_t u, int64_t gs, bool rotate_k, const Tensor* cos, const Tensor* sin) {
    check_act(Xk, "Xk");
    if (cos) check_rope(*cos, *sin, Xk, D);
    check_act(Xv, "Xv");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(Xk.numel() == B * Hkv * D && Xv.numel() == B * Hkv * D, "Xk and Xv must hold B*Hkv*D elements");
    const int32_t* pp = nullptr;
    if (pos_t.has_value()) {
        const Tensor& p = *pos_t;
        TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kInt && p.is_contiguous() && p.numel() == B,
                    "pos must be a contiguous CUDA int32 tensor of B elements");
        pp = p.data_ptr<int32_t>();
    }
    check_planes(ks, ku, kh, Xk, B * Hkv * NB * Lcap, UB, SB);
    check_planes(vs, vu, vh, Xv, B * Hkv * NB * Lcap, UB, SB);
    c10::cuda::CUDAGuard guard(Xk.device());
    check_rc(msaq_kv_append_pair_rope(Xk.data_ptr(), Xv.data_ptr(), ks.data_ptr<int8_t>(), ku.data_ptr<uint8_t>(),
                                      kh.data_ptr<uint8_t>(), vs.data_ptr<int8_t>(), vu.data_ptr<uint8_t>(),
                                      vh.data_ptr<uint8_t>(), B, Hkv, D, NB, pos, pp, Lcap, (int)u, (int)gs,
                                      rotate_k ? 1 : 0, cos ? cos->data_ptr<float>() : nullptr,
                                      sin ? sin->data_ptr<float>() : nullptr, cos ? cos->size(0) : 0, stream_of(Xk)),
             "kv_append_pair");
}
void kv_append_pair(const Tensor& Xk, const Tensor& Xv, Tensor ks, Tensor ku, Tensor kh, Tensor vs, Tensor vu, Tensor vh,
                    const c10::optional<Tensor>& pos_t, int64_t B, int64_t Hkv, int64_t D, int64_t NB, int64_t pos,
                    int64_t Lcap, int64_t u, int64_t gs, bool rotate_k) {
    kv_append_pair_impl(Xk, Xv, ks, ku, kh, vs, vu, vh, pos_t, B, Hkv, D, NB, pos, Lcap, u, gs, rotate_k, nullptr, nullptr);
}
// Same with the rotary embedding applied to the K rows first (at the slot each row goes to).
void kv_append_pair_rope(const Tensor& Xk, const Tensor& Xv, Tensor ks, Tensor ku, Tensor kh, Tensor vs, Tensor vu,
                         Tensor vh, const c10::optional<Tensor>& pos_t, int64_t B, int64_t Hkv, int64_t D, int64_t NB,
                         int64_t pos, int64_t Lcap, int64_t u, int64_t gs, bool rotate_k, const Tensor& cos,
                         const Tensor& sin) {
    kv_append_pair_impl(Xk, Xv, ks, ku, kh, vs, vu, vh, pos_t, B, Hkv, D, NB, pos, Lcap, u, gs, rotate_k, &cos, &sin);
}

std::vector<Tensor> kv_write_impl(const Tensor& X, int64_t H, int64_t L, int64_t D, int64_t NB, int64_t u, int64_t gs,
                                  bool rot) {
    check_act(X, "X");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(X.numel() == H * L * D, "X must hold H*L*D elements");
    c10::cuda::CUDAGuard guard(X.device());
    Tensor s = at::empty({H, NB, L}, X.options().dtype(at::kChar));
    Tensor up = at::empty({H, NB, L, UB}, X.options().dtype(at::kByte));
    Tensor sh = at::empty({H, NB, L, SB}, X.options().dtype(at::kByte));
    check_rc(msaq_kv_write(X.data_ptr(), s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(), sh.data_ptr<uint8_t>(), H, L, D,
                           NB, 0, L, (int)u, (int)gs, rot ? 1 : 0, stream_of(X)),
             "kv_write");
    return {s, up, sh};
}
std::vector<Tensor> kv_write(const Tensor& X, int64_t H, int64_t L, int64_t D, int64_t NB, int64_t u, int64_t gs) {
    return kv_write_impl(X, H, L, D, NB, u, gs, false);
}
std::vector<Tensor> kv_write_rot(const Tensor& X, int64_t H, int64_t L, int64_t D, int64_t NB, int64_t u,
                                 int64_t gs) {
    return kv_write_impl(X, H, L, D, NB, u, gs, true);
}

void kv_write_into(const Tensor& X, Tensor s, Tensor up, Tensor sh, int64_t H, int64_t L, int64_t D, int64_t NB,
                   int64_t key0, int64_t Lcap, int64_t u, int64_t gs, bool rotate) {
    check_act(X, "X");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(X.numel() == H * L * D, "X must hold H*L*D elements");
    check_planes(s, up, sh, X, H * NB * Lcap, UB, SB);
    c10::cuda::CUDAGuard guard(X.device());
    check_rc(msaq_kv_write(X.data_ptr(), s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(), sh.data_ptr<uint8_t>(), H, L, D,
                           NB, key0, Lcap, (int)u, (int)gs, rotate ? 1 : 0, stream_of(X)),
             "kv_write_into");
}

Tensor hadamard_rotate(const Tensor& x) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16, "x must be a CUDA bf16 tensor");
    Tensor xc = x.contiguous();
    const int64_t D = xc.size(-1);
    c10::cuda::CUDAGuard guard(xc.device());
    Tensor out = at::empty_like(xc);
    check_rc(msaq_hadamard_rotate(xc.data_ptr(), out.data_ptr(), xc.numel() / D, D, stream_of(xc)), "hadamard_rotate");
    return out;
}

std::vector<Tensor> pack_weight(const Tensor& W, int64_t u, int64_t gs) {
    TORCH_CHECK(W.is_cuda() && W.dim() == 2 && W.is_contiguous(), "W must be a contiguous 2-D CUDA tensor");
    TORCH_CHECK(W.scalar_type() == at::kBFloat16 || W.scalar_type() == at::kFloat, "W must be bf16 or fp32");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    const int64_t OUT = W.size(0), K = W.size(1);
    TORCH_CHECK(K % 32 == 0, "K must be a multiple of 32");
    const int64_t nb = K / 32;
    c10::cuda::CUDAGuard guard(W.device());
    auto b = W.options().dtype(at::kByte);
    Tensor s = at::empty({nb, OUT}, W.options().dtype(at::kChar));
    Tensor up = at::empty({nb, UB, OUT}, b), sh = at::empty({nb, SB, OUT}, b);
    Tensor upc = at::empty({nb, OUT, UB}, b), shc = at::empty({nb, OUT, SB}, b);
    check_rc(msaq_pack_weight(W.data_ptr(), W.scalar_type() == at::kBFloat16, s.data_ptr<int8_t>(),
                              up.data_ptr<uint8_t>(), sh.data_ptr<uint8_t>(), upc.data_ptr<uint8_t>(),
                              shc.data_ptr<uint8_t>(), OUT, K, (int)u, (int)gs, stream_of(W)),
             "pack_weight");
    return {s, up, sh, upc, shc};
}

// ---- decode attention -------------------------------------------------------
int env_flag(const char* name) {
    const char* e = std::getenv(name);
    return (e && std::atoi(e) != 0) ? 1 : 0;
}

void reject_numeric_toggles() {
    TORCH_CHECK(!env_flag("MS_KV_AA"), "MS_KV_AA=1 (fake-quantised attention activations) is not supported");
}

Tensor decode_common(const Tensor& q, const Tensor& ks, const Tensor& ku, const Tensor& kh, const Tensor& vs,
                     const Tensor& vu, const Tensor& vh, const c10::optional<Tensor>& seq_lens, int64_t B, int64_t H,
                     int64_t Hkv, int64_t Lk, int64_t D, int64_t NB, int64_t u, int64_t gs, int64_t Lcap, int qrot,
                     bool batched, const Tensor* cos = nullptr, const Tensor* sin = nullptr,
                     const c10::optional<Tensor>& q_pos_t = c10::nullopt, int64_t q_pos = 0) {
    check_act(q, "q");
    if (cos) check_rope(*cos, *sin, q, D);
    const int32_t* qpp = nullptr;
    if (q_pos_t.has_value()) {
        const Tensor& p = *q_pos_t;
        TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kInt && p.is_contiguous() && p.numel() == B,
                    "q_pos must be a contiguous CUDA int32 tensor of B elements");
        qpp = p.data_ptr<int32_t>();
    }
    reject_numeric_toggles();
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    if (Lcap < 0) Lcap = Lk;
    TORCH_CHECK(B >= 1 && H >= 1 && Hkv >= 1 && Lk >= 1, "B, H, Hkv and Lk must be positive");
    TORCH_CHECK(q.numel() == B * H * D, "q must hold B*H*D elements");
    check_planes(ks, ku, kh, q, B * Hkv * NB * Lcap, UB, SB);
    check_planes(vs, vu, vh, q, B * Hkv * NB * Lcap, UB, SB);
    const int32_t* lens = nullptr;
    if (seq_lens.has_value()) {
        const Tensor& sl = *seq_lens;
        TORCH_CHECK(sl.is_cuda() && sl.scalar_type() == at::kInt && sl.is_contiguous() && sl.numel() == B,
                    "seq_lens must be a contiguous CUDA int32 tensor of B elements");
        lens = sl.data_ptr<int32_t>();
    }
    c10::cuda::CUDAGuard guard(q.device());
    Tensor out = batched ? at::empty({B, H, D}, q.options()) : at::empty({H, D}, q.options());
    const size_t wsb = msaq_kv_decode_workspace(B, H, Hkv, Lk, D);
    Tensor ws = workspace(q, wsb);
    check_rc(msaq_kv_decode_attention_rope(q.data_ptr(), ks.data_ptr<int8_t>(), ku.data_ptr<uint8_t>(),
                                           kh.data_ptr<uint8_t>(), vs.data_ptr<int8_t>(), vu.data_ptr<uint8_t>(),
                                           vh.data_ptr<uint8_t>(), out.data_ptr(), nullptr, lens, B, H, Hkv, Lk, D,
                                           NB, (int)u, (int)gs, Lcap, qrot, cos ? cos->data_ptr<float>() : nullptr,
                                           sin ? sin->data_ptr<float>() : nullptr, cos ? cos->size(0) : 0, q_pos, qpp,
                                           ws.data_ptr(), wsb, stream_of(q)),
             batched ? "kv_decode_attention_batched" : "kv_decode_attention");
    return out;
}

Tensor kv_decode_attention(const Tensor& q, const Tensor& ks, const Tensor& ku, const Tensor& kh, const Tensor& vs,
                           const Tensor& vu, const Tensor& vh, int64_t H, int64_t Hkv, int64_t Lk, int64_t D,
                           int64_t NB, int64_t u, int64_t gs, int64_t Lcap) {
    // The single-sequence op never rotates the query (csrc/kv_attention.cu:2011 of the reference).
    return decode_common(q, ks, ku, kh, vs, vu, vh, c10::nullopt, 1, H, Hkv, Lk, D, NB, u, gs, Lcap, 0, false);
}

Tensor kv_decode_attention_batched(const Tensor& q, const Tensor& ks, const Tensor& ku, const Tensor& kh,
                                   const Tensor& vs, const Tensor& vu, const Tensor& vh, int64_t B, int64_t H,
                                   int64_t Hkv, int64_t Lk, int64_t D, int64_t NB, int64_t u, int64_t gs,
                                   int64_t Lcap) {
    return decode_common(q, ks, ku, kh, vs, vu, vh, c10::nullopt, B, H, Hkv, Lk, D, NB, u, gs, Lcap,
                         env_flag("MS_KV_QROT"), true);
}

Tensor kv_decode_attention_varlen(const Tensor& q, const Tensor& ks, const Tensor& ku, const Tensor& kh,
                                  const Tensor& vs, const Tensor& vu, const Tensor& vh, const Tensor& seq_lens,
                                  int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D, int64_t NB, int64_t u,
                                  int64_t gs, int64_t Lcap, bool qrot) {
    return decode_common(q, ks, ku, kh, vs, vu, vh, seq_lens, B, H, Hkv, Lk, D, NB, u, gs, Lcap, qrot ? 1 : 0, true);
}

// The varlen decode with the query's rotary embedding done in the kernel prologue (before the Hadamard rotation).
Tensor kv_decode_attention_rope(const Tensor& q, const Tensor& ks, const Tensor& ku, const Tensor& kh,
                                const Tensor& vs, const Tensor& vu, const Tensor& vh, const Tensor& seq_lens,
                                int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D, int64_t NB, int64_t u,
                                int64_t gs, int64_t Lcap, bool qrot, const Tensor& cos, const Tensor& sin,
                                const c10::optional<Tensor>& q_pos_t, int64_t q_pos) {
    return decode_common(q, ks, ku, kh, vs, vu, vh, seq_lens, B, H, Hkv, Lk, D, NB, u, gs, Lcap, qrot ? 1 : 0, true,
                         &cos, &sin, q_pos_t, q_pos);
}

// One decode step's cache update and attention in one op (the planes are written in place).
Tensor kv_decode_attention_append(const Tensor& q, const Tensor& k_new, const Tensor& v_new, Tensor ks, Tensor ku, Tensor kh,
                                  Tensor vs, Tensor vu, Tensor vh, const c10::optional<Tensor>& seq_lens, int64_t B, int64_t H,
                                  int64_t Hkv, int64_t Lk, int64_t D, int64_t NB, int64_t u, int64_t gs, int64_t Lcap,
                                  bool rotate_k, bool qrot, const c10::optional<Tensor>& cos, const c10::optional<Tensor>& sin,
                                  const c10::optional<Tensor>& pos_t, int64_t pos) {
    check_act(q, "q");
    check_act(k_new, "k_new");
    check_act(v_new, "v_new");
    TORCH_CHECK(cos.has_value() == sin.has_value(), "cos and sin come together");
    if (cos.has_value()) check_rope(*cos, *sin, q, D);
    const int32_t* pp = nullptr;
    if (pos_t.has_value()) {
        const Tensor& p = *pos_t;
        TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kInt && p.is_contiguous() && p.numel() == B,
                    "pos must be a contiguous CUDA int32 tensor of B elements");
        pp = p.data_ptr<int32_t>();
    }
    reject_numeric_toggles();
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    if (Lcap < 0) Lcap = Lk;
    TORCH_CHECK(B >= 1 && H >= 1 && Hkv >= 1 && Lk >= 1, "B, H, Hkv and Lk must be positive");
    TORCH_CHECK(q.numel() == B * H * D, "q must hold B*H*D elements");
    TORCH_CHECK(k_new.numel() == B * Hkv * D && v_new.numel() == B * Hkv * D, "k_new and v_new must hold B*Hkv*D elements");
    check_planes(ks, ku, kh, q, B * Hkv * NB * Lcap, UB, SB);
    check_planes(vs, vu, vh, q, B * Hkv * NB * Lcap, UB, SB);
    const int32_t* lens = nullptr;
    if (seq_lens.has_value()) {
        const Tensor& sl = *seq_lens;
        TORCH_CHECK(sl.is_cuda() && sl.scalar_type() == at::kInt && sl.is_contiguous() && sl.numel() == B,
                    "seq_lens must be a contiguous CUDA int32 tensor of B elements");
        lens = sl.data_ptr<int32_t>();
    }
    c10::cuda::CUDAGuard guard(q.device());
    Tensor out = at::empty({B, H, D}, q.options());
    const size_t wsb = msaq_kv_decode_workspace(B, H, Hkv, Lk, D);
    Tensor ws = workspace(q, wsb);
    check_rc(msaq_kv_decode_attention_append(q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), ks.data_ptr<int8_t>(),
                                             ku.data_ptr<uint8_t>(), kh.data_ptr<uint8_t>(), vs.data_ptr<int8_t>(),
                                             vu.data_ptr<uint8_t>(), vh.data_ptr<uint8_t>(), out.data_ptr(), nullptr, lens, B, H,
                                             Hkv, Lk, D, NB, (int)u, (int)gs, Lcap, rotate_k ? 1 : 0, qrot ? 1 : 0,
                                             cos.has_value() ? cos->data_ptr<float>() : nullptr,
                                             sin.has_value() ? sin->data_ptr<float>() : nullptr,
                                             cos.has_value() ? cos->size(0) : 0, pos, pp, ws.data_ptr(), wsb, stream_of(q)),
             "kv_decode_attention_append");
    return out;
}

// x [B, heads, D] bf16 -> RoPE at position pos (pos_t[b] per sequence when given).
Tensor rope(const Tensor& x, const Tensor& cos, const Tensor& sin, const c10::optional<Tensor>& pos_t, int64_t pos) {
    check_act(x, "x");
    TORCH_CHECK(x.dim() == 3, "x must be [B, heads, D]");
    const int64_t B = x.size(0), heads = x.size(1), D = x.size(2);
    check_rope(cos, sin, x, D);
    const int32_t* pp = nullptr;
    if (pos_t.has_value()) {
        const Tensor& p = *pos_t;
        TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kInt && p.is_contiguous() && p.numel() == B,
                    "pos must be a contiguous CUDA int32 tensor of B elements");
        pp = p.data_ptr<int32_t>();
    }
    c10::cuda::CUDAGuard guard(x.device());
    Tensor out = at::empty_like(x);
    check_rc(msaq_rope(x.data_ptr(), out.data_ptr(), B, heads, D, cos.data_ptr<float>(), sin.data_ptr<float>(), cos.size(0),
                       pos, pp, stream_of(x)), "rope");
    return out;
}

// ---- tensor-parallel exchange ------------------------------------------------------------------------------
// peer_ptrs: the ranks' exchange buffers as mapped into this process (int64 device addresses, e.g. the
// buffer_ptrs of a torch symmetric-memory handle).  Returns the fp32 sum, or bf16(residual + sum).
Tensor peer_exchange(const Tensor& partial, const c10::optional<Tensor>& residual, std::vector<int64_t> peer_ptrs, int64_t rank,
                     int64_t parity) {
    TORCH_CHECK(partial.is_cuda() && partial.scalar_type() == at::kFloat && partial.is_contiguous(),
                "partial must be a contiguous CUDA fp32 tensor");
    const int64_t world = (int64_t)peer_ptrs.size();
    TORCH_CHECK(world >= 2 && world <= 8, "2 to 8 ranks");
    void* bufs[8];
    for (int64_t r = 0; r < world; ++r) bufs[r] = reinterpret_cast<void*>(peer_ptrs[r]);
    c10::cuda::CUDAGuard guard(partial.device());
    Tensor out;
    const void* res = nullptr;
    if (residual.has_value()) {
        check_act(*residual, "residual");
        TORCH_CHECK(residual->numel() == partial.numel(), "residual and partial sizes differ");
        out = at::empty_like(*residual);
        res = residual->data_ptr();
    } else {
        out = at::empty_like(partial);
    }
    check_rc(msaq_peer_exchange(partial.data_ptr<float>(), res, out.data_ptr(), bufs, (int)rank, (int)world, partial.numel(),
                                (int)parity, stream_of(partial)), "peer_exchange");
    return out;
}

// residual + GEMV(pro(x)), the last projection of a decoder layer with its residual add inside.
Tensor wonly_gemv_fused_add(const Tensor& x, int64_t prologue, double eps, const Tensor& s, const Tensor& up, const Tensor& sh,
                            const Tensor& residual, int64_t M, int64_t OUT, int64_t NB, int64_t u, int64_t gs) {
    check_act(x, "x");
    check_act(residual, "residual");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(M >= 1 && OUT >= 1 && NB >= 1, "M, OUT and NB must be positive");
    TORCH_CHECK(x.numel() == M * NB * 32 * (prologue == MSAQ_PRO_SILU_MUL ? 2 : 1), "x has ", x.numel(), " elements");
    TORCH_CHECK(residual.numel() == M * OUT, "residual must be [M, OUT]");
    check_planes(s, up, sh, x, NB * OUT, UB, SB);
    c10::cuda::CUDAGuard guard(x.device());
    Tensor y = at::empty({M, OUT}, x.options());
    const size_t wsb = msaq_wonly_gemv_fused_workspace(M, OUT, NB, (int)u, (int)gs);
    Tensor ws = workspace(x, wsb);
    check_rc(msaq_wonly_gemv_fused_add(x.data_ptr(), (int)prologue, (float)eps, s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(),
                                       sh.data_ptr<uint8_t>(), residual.data_ptr(), y.data_ptr(), M, OUT, NB, (int)u, (int)gs,
                                       ws.data_ptr(), wsb, stream_of(x)),
             "wonly_gemv_fused_add");
    return y;
}

// The row-parallel GEMV with the exchange's push inside (no output tensor: the partial sums land in the ranks'
// exchange buffers), and the receiving half of the exchange: fp32 [M, OUT] sum, or bf16(residual + sum).
void wonly_gemv_fused_push(const Tensor& x, int64_t prologue, double eps, const Tensor& s, const Tensor& up, const Tensor& sh,
                           int64_t M, int64_t OUT, int64_t NB, int64_t u, int64_t gs, std::vector<int64_t> peer_ptrs,
                           int64_t rank, int64_t parity) {
    check_act(x, "x");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(M >= 1 && OUT >= 1 && NB >= 1, "M, OUT and NB must be positive");
    TORCH_CHECK(prologue != MSAQ_PRO_ADD_RMSNORM, "the add+rmsnorm prologue belongs to column-parallel projections");
    TORCH_CHECK(x.numel() == M * NB * 32 * (prologue == MSAQ_PRO_SILU_MUL ? 2 : 1), "x has ", x.numel(), " elements");
    check_planes(s, up, sh, x, NB * OUT, UB, SB);
    const int64_t world = (int64_t)peer_ptrs.size();
    TORCH_CHECK(world >= 2 && world <= 8, "2 to 8 ranks");
    void* bufs[8];
    for (int64_t r = 0; r < world; ++r) bufs[r] = reinterpret_cast<void*>(peer_ptrs[r]);
    c10::cuda::CUDAGuard guard(x.device());
    const size_t wsb = msaq_wonly_gemv_fused_workspace(M, OUT, NB, (int)u, (int)gs);
    Tensor ws = workspace(x, wsb);
    check_rc(msaq_wonly_gemv_fused_push(x.data_ptr(), (int)prologue, nullptr, 0, (float)eps, nullptr, s.data_ptr<int8_t>(),
                                        up.data_ptr<uint8_t>(), sh.data_ptr<uint8_t>(), M, OUT, NB, (int)u, (int)gs, bufs,
                                        (int)rank, (int)world, (int)parity, ws.data_ptr(), wsb, stream_of(x)),
             "wonly_gemv_fused_push");
}

Tensor peer_exchange_recv(const Tensor& like, const c10::optional<Tensor>& residual, std::vector<int64_t> peer_ptrs, int64_t rank,
                          int64_t parity, int64_t M, int64_t OUT) {
    TORCH_CHECK(like.is_cuda(), "like must be a CUDA tensor");
    const int64_t world = (int64_t)peer_ptrs.size();
    TORCH_CHECK(world >= 2 && world <= 8, "2 to 8 ranks");
    void* bufs[8];
    for (int64_t r = 0; r < world; ++r) bufs[r] = reinterpret_cast<void*>(peer_ptrs[r]);
    c10::cuda::CUDAGuard guard(like.device());
    Tensor out;
    const void* res = nullptr;
    if (residual.has_value()) {
        check_act(*residual, "residual");
        TORCH_CHECK(residual->numel() == M * OUT, "residual must have M * OUT elements");
        out = at::empty_like(*residual);
        res = residual->data_ptr();
    } else {
        out = at::empty({M, OUT}, like.options().dtype(at::kFloat));
    }
    check_rc(msaq_peer_exchange(nullptr, res, out.data_ptr(), bufs, (int)rank, (int)world, M * OUT, (int)parity, stream_of(like)),
             "peer_exchange_recv");
    return out;
}

// ---- W+A decode and the prefill vehicle (schemas of the reference, csrc/pybind.cpp:203-204,231-233,244-245) ----
Tensor wa_gemv_impl(const Tensor& x, const Tensor& s, const Tensor& up, const Tensor& sh, int64_t M, int64_t OUT,
                    int64_t NB, int64_t u, int64_t gs, bool batched) {
    check_act(x, "x");
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(M >= 1 && OUT >= 1 && NB >= 1, "M, OUT and NB must be positive");
    TORCH_CHECK(x.numel() == M * NB * 32, "x has ", x.numel(), " elements, expected M*K = ", M * NB * 32);
    check_planes(s, up, sh, x, NB * OUT, UB, SB);
    c10::cuda::CUDAGuard guard(x.device());
    Tensor y = batched ? at::empty({M, OUT}, x.options()) : at::empty({OUT}, x.options());
    const size_t wsb = msaq_wa_gemv_workspace(M, OUT, NB, (int)u, (int)gs);
    Tensor ws = workspace(x, wsb);
    check_rc(msaq_wa_gemv_batched(x.data_ptr(), s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(), sh.data_ptr<uint8_t>(),
                                  y.data_ptr(), nullptr, M, OUT, NB, (int)u, (int)gs, ws.data_ptr(), wsb, stream_of(x)),
             "wa_gemv");
    return y;
}
Tensor wa_gemv(const Tensor& x, const Tensor& s, const Tensor& up, const Tensor& sh, int64_t OUT, int64_t NB, int64_t u,
               int64_t gs) {
    return wa_gemv_impl(x, s, up, sh, 1, OUT, NB, u, gs, false);
}
Tensor wa_gemv_batched(const Tensor& x, const Tensor& s, const Tensor& up, const Tensor& sh, int64_t M, int64_t OUT,
                       int64_t NB, int64_t u, int64_t gs) {
    return wa_gemv_impl(x, s, up, sh, M, OUT, NB, u, gs, true);
}

std::vector<Tensor> quant_act(const Tensor& X, int64_t M, int64_t K, int64_t NB, int64_t u, int64_t gs) {
    check_act(X, "X");
    TORCH_CHECK(X.numel() == M * K && NB * 32 == K, "X must hold M*K elements and K = 32*NB");
    c10::cuda::CUDAGuard guard(X.device());
    Tensor qX = at::empty({M, K}, X.options().dtype(at::kChar));
    Tensor sa = at::empty({M, NB}, X.options().dtype(at::kChar));
    check_rc(msaq_quant_act(X.data_ptr(), qX.data_ptr<int8_t>(), sa.data_ptr<int8_t>(), M, K, (int)u, (int)gs, stream_of(X)),
             "quant_act");
    return {qX, sa};
}

Tensor ms_dequant_bf16(const Tensor& s, const Tensor& up, const Tensor& sh, int64_t OUT, int64_t K, int64_t NB, int64_t u,
                       int64_t gs) {
    int64_t UB, SB;
    fmt_sizes(u, gs, &UB, &SB);
    TORCH_CHECK(s.is_cuda() && NB * 32 == K, "scale_exp must be a CUDA tensor and K = 32*NB");
    check_planes(s, up, sh, s, NB * OUT, UB, SB);
    c10::cuda::CUDAGuard guard(s.device());
    Tensor W = at::empty({K, OUT}, s.options().dtype(at::kBFloat16));
    check_rc(msaq_dequant_bf16(s.data_ptr<int8_t>(), up.data_ptr<uint8_t>(), sh.data_ptr<uint8_t>(), W.data_ptr(), OUT, K,
                               (int)u, (int)gs, stream_of(s)), "ms_dequant_bf16");
    return W;
}

// ---- plain MXINT8 baseline (schemas of the reference, csrc/pybind.cpp:290-293,314-322) -------------------
void check_i8(const Tensor& t, const Tensor& like, int64_t numel, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.get_device() == like.get_device() && t.scalar_type() == at::kChar && t.is_contiguous() &&
                t.numel() == numel, name, " must be a contiguous CUDA int8 tensor of ", numel, " elements");
}

Tensor mxint8_gemv_impl(const Tensor& x, const Tensor& s, const Tensor& qw, int64_t M, int64_t OUT, int64_t NB, bool batched) {
    check_act(x, "x");
    TORCH_CHECK(M >= 1 && OUT >= 1 && NB >= 1, "M, OUT and NB must be positive");
    TORCH_CHECK(x.numel() == M * NB * 32, "x has ", x.numel(), " elements, expected M*K = ", M * NB * 32);
    check_i8(s, x, NB * OUT, "scale_exp");
    check_i8(qw, x, NB * OUT * 32, "qweight_cm");
    c10::cuda::CUDAGuard guard(x.device());
    Tensor y = batched ? at::empty({M, OUT}, x.options()) : at::empty({OUT}, x.options());
    const size_t wsb = msaq_mxint8_gemv_workspace(M, OUT, NB);
    Tensor ws = workspace(x, wsb);
    check_rc(msaq_mxint8_gemv_batched_wide(x.data_ptr(), s.data_ptr<int8_t>(), qw.data_ptr<int8_t>(), y.data_ptr(), nullptr,
                                           M, OUT, NB, ws.data_ptr(), wsb, stream_of(x)), "mxint8_gemv");
    return y;
}
Tensor mxint8_gemv_wide(const Tensor& x, const Tensor& s, const Tensor& qw, int64_t OUT, int64_t NB) {
    return mxint8_gemv_impl(x, s, qw, 1, OUT, NB, false);
}
Tensor mxint8_gemv_batched_wide(const Tensor& x, const Tensor& s, const Tensor& qw, int64_t M, int64_t OUT, int64_t NB) {
    return mxint8_gemv_impl(x, s, qw, M, OUT, NB, true);
}

std::vector<Tensor> mxint8_pack_weight(const Tensor& W) {
    TORCH_CHECK(W.is_cuda() && W.dim() == 2 && W.is_contiguous(), "W must be a contiguous 2-D CUDA tensor");
    TORCH_CHECK(W.scalar_type() == at::kBFloat16 || W.scalar_type() == at::kFloat, "W must be bf16 or fp32");
    const int64_t OUT = W.size(0), K = W.size(1);
    TORCH_CHECK(K % 32 == 0, "K must be a multiple of 32");
    const int64_t nb = K / 32;
    c10::cuda::CUDAGuard guard(W.device());
    auto o = W.options().dtype(at::kChar);
    Tensor s = at::empty({nb, OUT}, o), qw = at::empty({nb, 32, OUT}, o), qwc = at::empty({nb, OUT, 32}, o);
    check_rc(msaq_mxint8_pack_weight(W.data_ptr(), W.scalar_type() == at::kBFloat16, s.data_ptr<int8_t>(), qw.data_ptr<int8_t>(),
                                     qwc.data_ptr<int8_t>(), OUT, K, stream_of(W)), "mxint8_pack_weight");
    return {s, qw, qwc};
}

std::vector<Tensor> mxint8_kv_write(const Tensor& X, int64_t H, int64_t L, int64_t D, int64_t NB) {
    check_act(X, "X");
    TORCH_CHECK(X.numel() == H * L * D, "X must hold H*L*D elements");
    c10::cuda::CUDAGuard guard(X.device());
    Tensor s = at::empty({H, NB, L}, X.options().dtype(at::kChar));
    Tensor qw = at::empty({H, NB, L, 32}, X.options().dtype(at::kChar));
    check_rc(msaq_mxint8_kv_write(X.data_ptr(), s.data_ptr<int8_t>(), qw.data_ptr<int8_t>(), H, L, D, NB, 0, L, stream_of(X)),
             "mxint8_kv_write");
    return {s, qw};
}

void mxint8_kv_write_into(const Tensor& X, Tensor s, Tensor qw, int64_t H, int64_t L, int64_t D, int64_t NB, int64_t key0,
                          int64_t Lcap) {
    check_act(X, "X");
    TORCH_CHECK(X.numel() == H * L * D, "X must hold H*L*D elements");
    check_i8(s, X, H * NB * Lcap, "scale_exp");
    check_i8(qw, X, H * NB * Lcap * 32, "qweight");
    c10::cuda::CUDAGuard guard(X.device());
    check_rc(msaq_mxint8_kv_write(X.data_ptr(), s.data_ptr<int8_t>(), qw.data_ptr<int8_t>(), H, L, D, NB, key0, Lcap,
                                  stream_of(X)), "mxint8_kv_write_into");
}

void mxint8_kv_append(const Tensor& X, Tensor s, Tensor qw, int64_t H, int64_t D, int64_t NB, int64_t pos, int64_t Lcap) {
    check_act(X, "X");
    TORCH_CHECK(X.numel() == H * D, "X must hold H*D elements");
    check_i8(s, X, H * NB * Lcap, "scale_exp");
    check_i8(qw, X, H * NB * Lcap * 32, "qweight");
    c10::cuda::CUDAGuard guard(X.device());
    check_rc(msaq_mxint8_kv_append(X.data_ptr(), s.data_ptr<int8_t>(), qw.data_ptr<int8_t>(), H, D, NB, pos, Lcap, stream_of(X)),
             "mxint8_kv_append");
}

Tensor mxint8_decode_impl(const Tensor& q, const Tensor& ks, const Tensor& kq, const Tensor& vs, const Tensor& vq,
                          const c10::optional<Tensor>& seq_lens, int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D,
                          int64_t NB, int64_t Lcap, bool batched) {
    check_act(q, "q");
    if (Lcap < 0) Lcap = Lk;
    TORCH_CHECK(q.numel() == B * H * D, "q must hold B*H*D elements");
    check_i8(ks, q, B * Hkv * NB * Lcap, "ks");
    check_i8(vs, q, B * Hkv * NB * Lcap, "vs");
    check_i8(kq, q, B * Hkv * NB * Lcap * 32, "kq");
    check_i8(vq, q, B * Hkv * NB * Lcap * 32, "vq");
    const int32_t* lens = nullptr;
    if (seq_lens.has_value()) {
        const Tensor& sl = *seq_lens;
        TORCH_CHECK(sl.is_cuda() && sl.scalar_type() == at::kInt && sl.is_contiguous() && sl.numel() == B,
                    "seq_lens must be a contiguous CUDA int32 tensor of B elements");
        lens = sl.data_ptr<int32_t>();
    }
    c10::cuda::CUDAGuard guard(q.device());
    Tensor out = batched ? at::empty({B, H, D}, q.options()) : at::empty({H, D}, q.options());
    const size_t wsb = msaq_kv_decode_workspace(B, H, Hkv, Lk, D);
    Tensor ws = workspace(q, wsb);
    check_rc(msaq_mxint8_kv_decode_batched(q.data_ptr(), ks.data_ptr<int8_t>(), kq.data_ptr<int8_t>(), vs.data_ptr<int8_t>(),
                                           vq.data_ptr<int8_t>(), out.data_ptr(), nullptr, lens, B, H, Hkv, Lk, D, NB, Lcap,
                                           ws.data_ptr(), wsb, stream_of(q)), "mxint8_kv_decode");
    return out;
}
Tensor mxint8_kv_decode(const Tensor& q, const Tensor& ks, const Tensor& kq, const Tensor& vs, const Tensor& vq, int64_t H,
                        int64_t Hkv, int64_t Lk, int64_t D, int64_t NB, int64_t Lcap) {
    return mxint8_decode_impl(q, ks, kq, vs, vq, c10::nullopt, 1, H, Hkv, Lk, D, NB, Lcap, false);
}
Tensor mxint8_kv_decode_batched(const Tensor& q, const Tensor& ks, const Tensor& kq, const Tensor& vs, const Tensor& vq,
                                int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D, int64_t NB, int64_t Lcap) {
    return mxint8_decode_impl(q, ks, kq, vs, vq, c10::nullopt, B, H, Hkv, Lk, D, NB, Lcap, true);
}
Tensor mxint8_kv_decode_varlen(const Tensor& q, const Tensor& ks, const Tensor& kq, const Tensor& vs, const Tensor& vq,
                               const Tensor& seq_lens, int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D, int64_t NB,
                               int64_t Lcap) {
    return mxint8_decode_impl(q, ks, kq, vs, vq, seq_lens, B, H, Hkv, Lk, D, NB, Lcap, true);
}

// ---- layer-step glue ----------------------------------------------------------
Tensor rmsnorm(const Tensor& x, double eps) {
    check_act(x, "x");
    c10::cuda::CUDAGuard guard(x.device());
    Tensor out = at::empty_like(x);
    const int64_t n = x.size(-1);
    check_rc(msaq_rmsnorm(x.data_ptr(), out.data_ptr(), x.numel() / n, n, (float)eps, stream_of(x)), "rmsnorm");
    return out;
}

Tensor silu_mul(const Tensor& gate_up) {
    check_act(gate_up, "gate_up");
    TORCH_CHECK(gate_up.dim() == 2 && gate_up.size(1) % 2 == 0, "gate_up must be [rows, 2F]");
    c10::cuda::CUDAGuard guard(gate_up.device());
    const int64_t rows = gate_up.size(0), F = gate_up.size(1) / 2;
    Tensor out = at::empty({rows, F}, gate_up.options());
    check_rc(msaq_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, F, stream_of(gate_up)), "silu_mul");
    return out;
}

Tensor add_residual(const Tensor& h, const Tensor& delta) {
    check_act(h, "h");
    TORCH_CHECK(delta.is_cuda() && delta.is_contiguous() && delta.numel() == h.numel() &&
                (delta.scalar_type() == at::kFloat || delta.scalar_type() == at::kBFloat16),
                "delta must be a contiguous CUDA fp32 or bf16 tensor of h's size");
    c10::cuda::CUDAGuard guard(h.device());
    Tensor out = at::empty_like(h);
    check_rc(msaq_add_residual(h.data_ptr(), delta.data_ptr(), delta.scalar_type() == at::kFloat, out.data_ptr(),
                               h.numel(), stream_of(h)), "add_residual");
    return out;
}

int64_t launch_count() { return (int64_t)msaq_launch_count(); }
void set_option(int64_t option, int64_t value) { check_rc(msaq_set_option((int)option, (int)value), "set_option"); }
int64_t wait_status(bool clear) {
    int v = 0;
    check_rc(msaq_wait_status(clear ? 1 : 0, at::cuda::getCurrentCUDAStream().stream(), &v), "wait_status");
    return v;
}
int64_t get_option(int64_t option) { return (int64_t)msaq_get_option((int)option); }

}  // namespace

TORCH_LIBRARY(msaq, m) {
    // schemas of the reference, verbatim (csrc/pybind.cpp:199-206, 235-239, 266-273, 286)
    m.def("wonly_gemv(Tensor x, Tensor scale_exp, Tensor upper, Tensor shared, "
          "int OUT, int NB, int u, int gs) -> Tensor", &wonly_gemv);
    m.def("wonly_gemv_wide(Tensor x, Tensor scale_exp, Tensor upper_cm, Tensor shared_cm, "
          "int OUT, int NB, int u, int gs) -> Tensor", &wonly_gemv_wide);
    m.def("wonly_gemv_batched(Tensor x, Tensor scale_exp, Tensor upper_cm, Tensor shared_cm, "
          "int M, int OUT, int NB, int u, int gs) -> Tensor", &wonly_gemv_batched);
    m.def("kv_write(Tensor X, int H, int L, int D, int NB, int u, int gs) -> Tensor[]", &kv_write);
    m.def("kv_append(Tensor X, Tensor(a!) scale_exp, Tensor(b!) upper, Tensor(c!) shared, "
          "int H, int D, int NB, int pos, int Lcap, int u, int gs) -> ()", &kv_append);
    m.def("kv_append_rot(Tensor X, Tensor(a!) scale_exp, Tensor(b!) upper, Tensor(c!) shared, "
          "int H, int D, int NB, int pos, int Lcap, int u, int gs) -> ()", &kv_append_rot);
    m.def("kv_decode_attention(Tensor q, Tensor ks, Tensor ku, Tensor kh, "
          "Tensor vs, Tensor vu, Tensor vh, "
          "int H, int Hkv, int Lk, int D, int NB, int u, int gs, int Lcap=-1) -> Tensor", &kv_decode_attention);
    m.def("kv_decode_attention_batched(Tensor q, Tensor ks, Tensor ku, Tensor kh, "
          "Tensor vs, Tensor vu, Tensor vh, "
          "int B, int H, int Hkv, int Lk, int D, int NB, int u, int gs, int Lcap=-1) -> Tensor",
          &kv_decode_attention_batched);
    m.def("hadamard_rotate(Tensor x) -> Tensor", &hadamard_rotate);
    // additions of this library (no counterpart op in the reference)
    m.def("kv_write_rot(Tensor X, int H, int L, int D, int NB, int u, int gs) -> Tensor[]", &kv_write_rot);
    m.def("kv_write_into(Tensor X, Tensor(a!) scale_exp, Tensor(b!) upper, Tensor(c!) shared, "
          "int H, int L, int D, int NB, int key0, int Lcap, int u, int gs, bool rotate) -> ()", &kv_write_into);
    m.def("kv_append_varlen(Tensor X, Tensor(a!) scale_exp, Tensor(b!) upper, Tensor(c!) shared, Tensor pos, "
          "int B, int Hkv, int D, int NB, int Lcap, int u, int gs, bool rotate) -> ()", &kv_append_varlen);
    m.def("kv_append_pair(Tensor Xk, Tensor Xv, Tensor(a!) ks, Tensor(b!) ku, Tensor(c!) kh, Tensor(d!) vs, Tensor(e!) vu, "
          "Tensor(f!) vh, Tensor? pos_t, int B, int Hkv, int D, int NB, int pos, int Lcap, int u, int gs, bool rotate_k) -> ()",
          &kv_append_pair);
    m.def("kv_append_pair_rope(Tensor Xk, Tensor Xv, Tensor(a!) ks, Tensor(b!) ku, Tensor(c!) kh, Tensor(d!) vs, Tensor(e!) vu, "
          "Tensor(f!) vh, Tensor? pos_t, int B, int Hkv, int D, int NB, int pos, int Lcap, int u, int gs, bool rotate_k, "
          "Tensor cos, Tensor sin) -> ()", &kv_append_pair_rope);
    m.def("kv_decode_attention_rope(Tensor q, Tensor ks, Tensor ku, Tensor kh, Tensor vs, Tensor vu, Tensor vh, "
          "Tensor seq_lens, int B, int H, int Hkv, int Lk, int D, int NB, int u, int gs, int Lcap, bool qrot, "
          "Tensor cos, Tensor sin, Tensor? q_pos_t, int q_pos) -> Tensor", &kv_decode_attention_rope);
    m.def("rope(Tensor x, Tensor cos, Tensor sin, Tensor? pos_t, int pos) -> Tensor", &rope);
    m.def("kv_decode_attention_varlen(Tensor q, Tensor ks, Tensor ku, Tensor kh, "
          "Tensor vs, Tensor vu, Tensor vh, Tensor seq_lens, "
          "int B, int H, int Hkv, int Lk, int D, int NB, int u, int gs, int Lcap, bool qrot) -> Tensor",
          &kv_decode_attention_varlen);
    m.def("wonly_gemv_fused(Tensor x, Tensor? addend, int prologue, float eps, Tensor scale_exp, Tensor upper_cm, "
          "Tensor shared_cm, int M, int OUT, int NB, int u, int gs, bool out_f32=False) -> Tensor[]", &wonly_gemv_fused);
    m.def("wonly_gemv_batched_f32(Tensor x, Tensor scale_exp, Tensor upper_cm, Tensor shared_cm, "
          "int M, int OUT, int NB, int u, int gs) -> Tensor", &wonly_gemv_batched_f32);
    m.def("pack_weight(Tensor W, int u, int gs) -> Tensor[]", &pack_weight);
    // the steps on either side of the weight-only decode path (schemas as in csrc/pybind.cpp:203-204,231-233,244-245)
    m.def("wa_gemv(Tensor x, Tensor scale_exp, Tensor upper_cm, Tensor shared_cm, "
          "int OUT, int NB, int u, int gs) -> Tensor", &wa_gemv);
    m.def("wa_gemv_batched(Tensor x, Tensor scale_exp, Tensor upper_cm, Tensor shared_cm, "
          "int M, int OUT, int NB, int u, int gs) -> Tensor", &wa_gemv_batched);
    m.def("quant_act(Tensor X, int M, int K, int NB, int u, int gs) -> Tensor[]", &quant_act);
    m.def("ms_dequant_bf16(Tensor scale_exp, Tensor upper_cm, Tensor shared_cm, "
          "int OUT, int K, int NB, int u, int gs) -> Tensor", &ms_dequant_bf16);
    // the reference's MXINT8 baseline operators on the decode path (schemas as in csrc/pybind.cpp:290-293,314-322)
    m.def("mxint8_gemv_wide(Tensor x, Tensor scale_exp, Tensor qweight_cm, "
          "int OUT, int NB) -> Tensor", &mxint8_gemv_wide);
    m.def("mxint8_gemv_batched_wide(Tensor x, Tensor scale_exp, Tensor qweight_cm, "
          "int M, int OUT, int NB) -> Tensor", &mxint8_gemv_batched_wide);
    m.def("mxint8_kv_decode(Tensor q, Tensor ks, Tensor kq, "
          "Tensor vs, Tensor vq, int H, int Hkv, int Lk, int D, int NB, int Lcap=-1) -> Tensor",
          &mxint8_kv_decode);
    m.def("mxint8_kv_decode_batched(Tensor q, Tensor ks, Tensor kq, Tensor vs, Tensor vq, "
          "int B, int H, int Hkv, int Lk, int D, int NB, int Lcap=-1) -> Tensor",
          &mxint8_kv_decode_batched);
    m.def("mxint8_kv_write(Tensor X, int H, int L, int D, int NB) -> Tensor[]", &mxint8_kv_write);
    m.def("mxint8_kv_append(Tensor X, Tensor(a!) scale_exp, Tensor(b!) qweight, "
          "int H, int D, int NB, int pos, int Lcap) -> ()", &mxint8_kv_append);
    // additions of this library
    m.def("mxint8_pack_weight(Tensor W) -> Tensor[]", &mxint8_pack_weight);
    m.def("mxint8_kv_write_into(Tensor X, Tensor(a!) scale_exp, Tensor(b!) qweight, int H, int L, int D, int NB, int key0, "
          "int Lcap) -> ()", &mxint8_kv_write_into);
    m.def("mxint8_kv_decode_varlen(Tensor q, Tensor ks, Tensor kq, Tensor vs, Tensor vq, Tensor seq_lens, "
          "int B, int H, int Hkv, int Lk, int D, int NB, int Lcap) -> Tensor", &mxint8_kv_decode_varlen);
    m.def("rmsnorm(Tensor x, float eps) -> Tensor", &rmsnorm);
    m.def("silu_mul(Tensor gate_up) -> Tensor", &silu_mul);
    m.def("add_residual(Tensor h, Tensor delta) -> Tensor", &add_residual);
    m.def("kv_decode_attention_append(Tensor q, Tensor k_new, Tensor v_new, Tensor(a!) k_scale_exp, Tensor(b!) k_upper, "
          "Tensor(c!) k_shared, Tensor(d!) v_scale_exp, Tensor(e!) v_upper, Tensor(f!) v_shared, Tensor? seq_lens, int B, int H, "
          "int Hkv, int Lk, int D, int NB, int u, int gs, int Lcap, bool rotate_k, bool qrot, Tensor? cos, Tensor? sin, "
          "Tensor? pos_t, int pos) -> Tensor", &kv_decode_attention_append);
    m.def("peer_exchange(Tensor partial, Tensor? residual, int[] peer_ptrs, int rank, int parity) -> Tensor", &peer_exchange);
    m.def("wonly_gemv_fused_add(Tensor x, int prologue, float eps, Tensor scale_exp, Tensor upper_cm, Tensor shared_cm, "
          "Tensor residual, int M, int OUT, int NB, int u, int gs) -> Tensor", &wonly_gemv_fused_add);
    m.def("wonly_gemv_fused_push(Tensor x, int prologue, float eps, Tensor scale_exp, Tensor upper_cm, Tensor shared_cm, int M, "
          "int OUT, int NB, int u, int gs, int[] peer_ptrs, int rank, int parity) -> ()", &wonly_gemv_fused_push);
    m.def("peer_exchange_recv(Tensor like, Tensor? residual, int[] peer_ptrs, int rank, int parity, int M, int OUT) -> Tensor",
          &peer_exchange_recv);
    m.def("launch_count() -> int", &launch_count);
    m.def("set_option(int option, int value) -> ()", &set_option);
    m.def("get_option(int option) -> int", &get_option);
    m.def("wait_status(bool clear) -> int", &wait_status);
}

// An importable, otherwise empty Python module: `import ms_cuda` loads this
// shared object, which runs the registration above.
static struct PyModuleDef ms_cuda_module = {PyModuleDef_HEAD_INIT, "ms_cuda",
                                            "Registers torch.ops.msaq.* (B200 decode path).", -1, nullptr};
PyMODINIT_FUNC PyInit_ms_cuda(void) { return PyModule_Create(&ms_cuda_module); }

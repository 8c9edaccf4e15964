"""Test-side helpers that drive the C ABI (include/msaq_b200.h) through ctypes,
with torch tensors serving only as device memory."""

import numpy as np
import torch

from ms_kernel_b200 import _lib
from oracle import msaq_oracle as orc


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def bf16_dev(a):
    """float array -> bf16 device tensor."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).cuda()


def gemv(kind, x, p, M=1, want_f32=True):
    """kind in {'rowmajor','wide','batched'}; x bf16 device tensor; p dict of device planes.
    Returns (y bf16 as float32 numpy, y_f32 numpy or None)."""
    L = _lib.lib()
    OUT, NB, u, gs = int(p["OUT"]), int(p["nb"]), int(p["u"]), int(p["gs"])
    shape = (OUT,) if kind != "batched" else (M, OUT)
    y = torch.empty(shape, dtype=torch.bfloat16, device="cuda")
    yf = torch.empty(shape, dtype=torch.float32, device="cuda") if want_f32 else None
    wsb = L.msaq_wonly_gemv_workspace(M, OUT, NB, u, gs)
    ws = torch.empty(max(wsb, 256), dtype=torch.uint8, device="cuda")
    if kind == "rowmajor":
        rc = L.msaq_wonly_gemv(_ptr(x), _ptr(p["scale_exp"]), _ptr(p["upper"]), _ptr(p["shared"]), _ptr(y), _ptr(yf),
                               OUT, NB, u, gs, _ptr(ws), wsb, _stream())
    elif kind == "wide":
        rc = L.msaq_wonly_gemv_wide(_ptr(x), _ptr(p["scale_exp"]), _ptr(p["upper_cm"]), _ptr(p["shared_cm"]), _ptr(y),
                                    _ptr(yf), OUT, NB, u, gs, _ptr(ws), wsb, _stream())
    else:
        rc = L.msaq_wonly_gemv_batched(_ptr(x), _ptr(p["scale_exp"]), _ptr(p["upper_cm"]), _ptr(p["shared_cm"]),
                                       _ptr(y), _ptr(yf), M, OUT, NB, u, gs, _ptr(ws), wsb, _stream())
    _lib.check(rc)
    torch.cuda.synchronize()
    return y.float().cpu().numpy(), (yf.cpu().numpy() if want_f32 else None)


def planes_to_dev(p):
    """Oracle pack dict (NumPy) -> same dict with device tensors for the plane keys."""
    out = dict(p)
    for k in ("scale_exp", "upper", "shared", "upper_cm", "shared_cm"):
        if k in p:
            out[k] = dev(p[k])
    return out


def empty_cache(H, nb, Lcap, u, gs, fill=0):
    UB, SB = orc.plane_bytes(u, gs)
    return (torch.full((H, nb, Lcap), fill, dtype=torch.int8, device="cuda"),
            torch.full((H, nb, Lcap, UB), fill & 0xFF, dtype=torch.uint8, device="cuda"),
            torch.full((H, nb, Lcap, SB), fill & 0xFF, dtype=torch.uint8, device="cuda"))


def kv_append(X, planes, H, D, pos, Lcap, u, gs, rot=False):
    L = _lib.lib()
    fn = L.msaq_kv_append_rot if rot else L.msaq_kv_append
    _lib.check(fn(_ptr(X), _ptr(planes[0]), _ptr(planes[1]), _ptr(planes[2]), H, D, D // 32, pos, Lcap, u, gs,
                  _stream()))


def kv_append_varlen(X, planes, B, Hkv, D, pos, Lcap, u, gs, rot=False):
    L = _lib.lib()
    _lib.check(L.msaq_kv_append_varlen(_ptr(X), _ptr(planes[0]), _ptr(planes[1]), _ptr(planes[2]), B, Hkv, D, D // 32,
                                       _ptr(pos), Lcap, u, gs, int(rot), _stream()))


def kv_write(X, planes, H, Lr, D, key0, Lcap, u, gs, rot=False):
    L = _lib.lib()
    _lib.check(L.msaq_kv_write(_ptr(X), _ptr(planes[0]), _ptr(planes[1]), _ptr(planes[2]), H, Lr, D, D // 32, key0,
                               Lcap, u, gs, int(rot), _stream()))


def hadamard_rotate(x):
    L = _lib.lib()
    out = torch.empty_like(x)
    D = x.shape[-1]
    _lib.check(L.msaq_hadamard_rotate(_ptr(x), _ptr(out), x.numel() // D, D, _stream()))
    return out


def pack_weight(W, u, gs):
    """W device tensor bf16/fp32 [OUT,K] -> dict of device planes (C ABI packer)."""
    L = _lib.lib()
    OUT, K = W.shape
    nb = K // 32
    UB, SB = orc.plane_bytes(u, gs)
    b = dict(dtype=torch.uint8, device="cuda")
    p = dict(scale_exp=torch.empty((nb, OUT), dtype=torch.int8, device="cuda"),
             upper=torch.empty((nb, UB, OUT), **b), shared=torch.empty((nb, SB, OUT), **b),
             upper_cm=torch.empty((nb, OUT, UB), **b), shared_cm=torch.empty((nb, OUT, SB), **b),
             OUT=OUT, K=K, nb=nb, u=u, gs=gs, UB=UB, SB=SB)
    _lib.check(L.msaq_pack_weight(_ptr(W), int(W.dtype == torch.bfloat16), _ptr(p["scale_exp"]), _ptr(p["upper"]),
                                  _ptr(p["shared"]), _ptr(p["upper_cm"]), _ptr(p["shared_cm"]), OUT, K, u, gs,
                                  _stream()))
    return p


def decode(q, kpl, vpl, B, H, Hkv, Lk, D, u, gs, Lcap=-1, qrot=0, seq_lens=None, single=False, want_f32=True):
    """Returns (out bf16 as float32 numpy, out_f32 numpy or None)."""
    L = _lib.lib()
    shape = (H, D) if single else (B, H, D)
    out = torch.empty(shape, dtype=torch.bfloat16, device="cuda")
    of = torch.empty(shape, dtype=torch.float32, device="cuda") if want_f32 else None
    wsb = L.msaq_kv_decode_workspace(B, H, Hkv, Lk, D)
    ws = torch.empty(max(wsb, 256), dtype=torch.uint8, device="cuda")
    if single:
        rc = L.msaq_kv_decode_attention(_ptr(q), *[_ptr(t) for t in kpl], *[_ptr(t) for t in vpl], _ptr(out), _ptr(of),
                                        H, Hkv, Lk, D, D // 32, u, gs, Lcap, _ptr(ws), wsb, _stream())
    else:
        rc = L.msaq_kv_decode_attention_batched(_ptr(q), *[_ptr(t) for t in kpl], *[_ptr(t) for t in vpl], _ptr(out),
                                                _ptr(of), _ptr(seq_lens), B, H, Hkv, Lk, D, D // 32, u, gs, Lcap,
                                                qrot, _ptr(ws), wsb, _stream())
    _lib.check(rc)
    torch.cuda.synchronize()
    return out.float().cpu().numpy(), (of.cpu().numpy() if want_f32 else None)


def check_output(got_bf16, got_f32, ref64, tol_mar, tol_fro, tol_f32):
    """The output tolerance of the decode path (see tests/conftest.py)."""
    ref_b = orc.to_bf16(np.asarray(ref64, np.float32))
    mar = orc.max_abs_rel(got_bf16, ref_b)
    fro = orc.rel_fro(got_bf16, ref_b)
    assert mar <= tol_mar, "max_abs_rel %.3e > %.3e" % (mar, tol_mar)
    assert fro <= tol_fro, "rel_fro %.3e > %.3e" % (fro, tol_fro)
    if got_f32 is not None:
        f = orc.rel_fro(got_f32, ref64)
        assert f <= tol_f32, "fp32 rel_fro %.3e > %.3e" % (f, tol_f32)
        assert np.array_equal(orc.to_bf16(got_f32), got_bf16), "bf16 output is not the rounding of the fp32 output"

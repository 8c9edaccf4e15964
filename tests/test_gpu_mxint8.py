"""GPU parity of the plain-MXINT8 twins (the reference's matched baseline format, ms_lib/pack.py:530-594,
csrc/mxint8.cu) against the oracle: packed bytes bit-exact, GEMV / decode outputs within the bf16 tolerance."""

import numpy as np
import pytest
import torch

from conftest import F32_REL_FRO_TOL, MAX_ABS_REL_TOL, REL_FRO_TOL
from ms_kernel_b200 import _lib, ops  # noqa: F401  (ops registers torch.ops.msaq.*)
from oracle import msaq_oracle as orc

pytestmark = pytest.mark.gpu


def _st():
    return torch.cuda.current_stream().cuda_stream


def _pack_dev(W, as_bf16=True):
    import cabi
    L = _lib.lib()
    OUT, K = W.shape
    nb = K // 32
    Wd = cabi.bf16_dev(W) if as_bf16 else cabi.dev(np.asarray(W, np.float32))
    s = torch.empty((nb, OUT), dtype=torch.int8, device="cuda")
    qw = torch.empty((nb, 32, OUT), dtype=torch.int8, device="cuda")
    qwc = torch.empty((nb, OUT, 32), dtype=torch.int8, device="cuda")
    _lib.check(L.msaq_mxint8_pack_weight(Wd.data_ptr(), int(as_bf16), s.data_ptr(), qw.data_ptr(), qwc.data_ptr(), OUT, K, _st()))
    torch.cuda.synchronize()
    return s, qw, qwc


def test_mxint8_pack_weight_bit_exact(rng, golden):
    W = golden["mx_W"]                       # carries fp32 edge blocks that are not bf16 values
    s, qw, qwc = _pack_dev(W, as_bf16=False)
    assert np.array_equal(s.cpu().numpy(), golden["mx_w_scale_exp"])
    assert np.array_equal(qw.cpu().numpy(), golden["mx_w_qweight"])
    assert np.array_equal(qwc.cpu().numpy(), golden["mx_w_qweight_cm"])
    W2 = orc.to_bf16((rng.standard_normal((200, 256)) * rng.uniform(0.001, 30, (200, 1))).astype(np.float32))
    p = orc.pack_weight_mxint8(W2)
    s, qw, qwc = _pack_dev(W2)
    for t, k in ((s, "scale_exp"), (qw, "qweight"), (qwc, "qweight_cm")):
        assert np.array_equal(t.cpu().numpy(), p[k]), k


@pytest.mark.parametrize("M,OUT,K", [(1, 256, 512), (1, 4096, 4096), (3, 1040, 2048), (4, 6144, 4096), (8, 512, 1024),
                                     (16, 4096, 1024), (33, 528, 512)])
def test_mxint8_gemv_vs_oracle(rng, M, OUT, K):
    import cabi
    L = _lib.lib()
    W = orc.to_bf16((rng.standard_normal((OUT, K)) * rng.uniform(0.005, 0.08, (OUT, 1))).astype(np.float32))
    X = orc.to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    p = orc.pack_weight_mxint8(W)
    s, qwc, x = cabi.dev(p["scale_exp"]), cabi.dev(p["qweight_cm"]), cabi.bf16_dev(X)
    y = torch.empty((M, OUT), dtype=torch.bfloat16, device="cuda")
    yf = torch.empty((M, OUT), dtype=torch.float32, device="cuda")
    wsb = L.msaq_mxint8_gemv_workspace(M, OUT, K // 32)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    _lib.check(L.msaq_mxint8_gemv_batched_wide(x.data_ptr(), s.data_ptr(), qwc.data_ptr(), y.data_ptr(), yf.data_ptr(), M, OUT,
                                               K // 32, ws.data_ptr(), wsb, _st()))
    torch.cuda.synchronize()
    cabi.check_output(y.float().cpu().numpy(), yf.cpu().numpy(), orc.wonly_matmul_mxint8(p, X), MAX_ABS_REL_TOL, REL_FRO_TOL,
                      F32_REL_FRO_TOL)
    # the operator with the reference's schema
    yo = torch.ops.msaq.mxint8_gemv_batched_wide(x, s, qwc, M, OUT, K // 32)
    assert torch.equal(yo, y)
    if M == 1:
        assert torch.equal(torch.ops.msaq.mxint8_gemv_wide(x[0].contiguous(), s, qwc, OUT, K // 32), y[0])


@pytest.mark.parametrize("D", (64, 128))
def test_mxint8_kv_write_and_append_bytes(rng, D):
    import cabi
    L = _lib.lib()
    H, Lr, Lcap = 4, 37, 48
    X = rng.standard_normal((H, Lr, D)).astype(np.float32)
    X[:, :, 3] *= 20
    X = orc.to_bf16(X)
    p = orc.pack_kv_mxint8(X)
    s = torch.full((H, D // 32, Lcap), 0x55, dtype=torch.int8, device="cuda")
    qw = torch.full((H, D // 32, Lcap, 32), 0x55, dtype=torch.int8, device="cuda")
    xd = cabi.bf16_dev(X[:, :Lr - 1])
    _lib.check(L.msaq_mxint8_kv_write(xd.data_ptr(), s.data_ptr(), qw.data_ptr(), H, Lr - 1, D, D // 32, 2, Lcap, _st()))
    xl = cabi.bf16_dev(X[:, Lr - 1])
    _lib.check(L.msaq_mxint8_kv_append(xl.data_ptr(), s.data_ptr(), qw.data_ptr(), H, D, D // 32, Lr + 1, Lcap, _st()))
    torch.cuda.synchronize()
    sn, qn = s.cpu().numpy(), qw.cpu().numpy()
    assert np.array_equal(sn[:, :, 2:Lr + 1], p["scale_exp"][:, :, :Lr - 1]) and np.array_equal(sn[:, :, Lr + 1], p["scale_exp"][:, :, Lr - 1])
    assert np.array_equal(qn[:, :, 2:Lr + 1], p["qweight"][:, :, :Lr - 1]) and np.array_equal(qn[:, :, Lr + 1], p["qweight"][:, :, Lr - 1])
    assert (sn[:, :, :2] == 0x55).all() and (qn[:, :, Lr + 2:] == 0x55).all()          # untouched slots
    # the operators with the reference's schemas
    so, qo = torch.ops.msaq.mxint8_kv_write(cabi.bf16_dev(X), H, Lr, D, D // 32)
    assert np.array_equal(so.cpu().numpy(), p["scale_exp"]) and np.array_equal(qo.cpu().numpy(), p["qweight"])


@pytest.mark.parametrize("B,Hq,Hkv,Lk", [(1, 8, 8, 300), (3, 8, 2, 208), (2, 32, 8, 4096), (1, 16, 16, 1040)])
def test_mxint8_decode_vs_oracle(rng, B, Hq, Hkv, Lk):
    import cabi
    L = _lib.lib()
    D = 128
    Lcap = (Lk + 31) // 16 * 16
    K = orc.to_bf16((rng.standard_normal((B * Hkv, Lk, D)) * 0.7).astype(np.float32))
    V = orc.to_bf16((rng.standard_normal((B * Hkv, Lk, D)) * 0.7).astype(np.float32))
    q = orc.to_bf16((rng.standard_normal((B, Hq, D)) * 0.7).astype(np.float32))
    planes = []
    for Xn in (K, V):
        s = torch.zeros((B * Hkv, D // 32, Lcap), dtype=torch.int8, device="cuda")
        qw = torch.zeros((B * Hkv, D // 32, Lcap, 32), dtype=torch.int8, device="cuda")
        xd = cabi.bf16_dev(Xn)
        _lib.check(L.msaq_mxint8_kv_write(xd.data_ptr(), s.data_ptr(), qw.data_ptr(), B * Hkv, Lk, D, D // 32, 0, Lcap, _st()))
        planes.append((s, qw))
    lens = rng.integers(Lk // 2, Lk + 1, size=B).astype(np.int32)
    lens[0] = Lk
    out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device="cuda")
    outf = torch.empty((B, Hq, D), dtype=torch.float32, device="cuda")
    wsb = L.msaq_kv_decode_workspace(B, Hq, Hkv, Lk, D)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    qd, ld = cabi.bf16_dev(q), cabi.dev(lens)
    _lib.check(L.msaq_mxint8_kv_decode_batched(qd.data_ptr(), planes[0][0].data_ptr(), planes[0][1].data_ptr(),
                                               planes[1][0].data_ptr(), planes[1][1].data_ptr(), out.data_ptr(), outf.data_ptr(),
                                               ld.data_ptr(), B, Hq, Hkv, Lk, D, D // 32, Lcap, ws.data_ptr(), wsb, _st()))
    torch.cuda.synchronize()
    kn = [t.cpu().numpy().reshape((B, Hkv) + tuple(t.shape[1:])) for t in planes[0]]
    vn = [t.cpu().numpy().reshape((B, Hkv) + tuple(t.shape[1:])) for t in planes[1]]
    ref = np.stack([orc.decode_attention_planes_mxint8(q[b], (kn[0][b], kn[1][b]), (vn[0][b], vn[1][b]), int(lens[b]))
                    for b in range(B)])
    cabi.check_output(out.float().cpu().numpy(), outf.cpu().numpy(), ref, MAX_ABS_REL_TOL, REL_FRO_TOL, 3e-4)
    # unsupported shapes are refused, not served by another path
    assert L.msaq_mxint8_kv_decode_batched(qd.data_ptr(), planes[0][0].data_ptr(), planes[0][1].data_ptr(),
                                           planes[1][0].data_ptr(), planes[1][1].data_ptr(), out.data_ptr(), None, None,
                                           B, Hq, Hkv, Lk, 64, 2, Lcap, ws.data_ptr(), wsb, _st()) == -2

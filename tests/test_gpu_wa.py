"""GPU parity of the steps on either side of the weight-only path: the run-time activation quantiser
(bit-exact), the W+A decode GEMV (reference: wa_matmul with MSAQ-signed activations) and the one-off
dequantisation of a packed weight to bf16."""

import numpy as np
import pytest
import torch

from conftest import F32_REL_FRO_TOL, MAX_ABS_REL_TOL, REL_FRO_TOL
from ms_kernel_b200 import _lib, ops  # noqa: F401  (ops registers torch.ops.msaq.*)
from oracle import msaq_oracle as orc

pytestmark = pytest.mark.gpu


def _st():
    return torch.cuda.current_stream().cuda_stream


def test_quant_act_bit_exact(rng, cfg, golden):
    import cabi
    u, gs = cfg
    L = _lib.lib()
    X = rng.standard_normal((7, 256)).astype(np.float32) * rng.uniform(0.01, 30, (7, 1)).astype(np.float32)
    X[:, 3] *= 20
    X = orc.to_bf16(X)
    if (u, gs) in ((2, 2), (3, 8), (4, 2)) and f"wa_q_u{u}_gs{gs}" in golden:
        X = golden["wa_X"]                                    # the reference's own fixture, where recorded
    M, K = X.shape
    xd = cabi.bf16_dev(X)
    q = torch.empty((M, K), dtype=torch.int8, device="cuda")
    e = torch.empty((M, K // 32), dtype=torch.int8, device="cuda")
    _lib.check(L.msaq_quant_act(xd.data_ptr(), q.data_ptr(), e.data_ptr(), M, K, u, gs, _st()))
    torch.cuda.synchronize()
    qr, er = orc.quant_act(X, u, gs)
    assert np.array_equal(q.cpu().numpy().reshape(qr.shape), qr)
    assert np.array_equal(e.cpu().numpy(), er)
    qo, eo = torch.ops.msaq.quant_act(xd, M, K, K // 32, u, gs)
    assert torch.equal(qo, q) and torch.equal(eo, e)


@pytest.mark.parametrize("u,gs", [(4, 2), (3, 2), (2, 2), (4, 8), (3, 16)])
@pytest.mark.parametrize("M,OUT,K", [(1, 384, 512), (1, 4096, 4096), (4, 1040, 2048), (16, 512, 1024)])
def test_wa_gemv_vs_oracle(rng, u, gs, M, OUT, K):
    import cabi
    L = _lib.lib()
    W = orc.to_bf16((rng.standard_normal((OUT, K)) * rng.uniform(0.005, 0.08, (OUT, 1))).astype(np.float32))
    X = orc.to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    p = orc.pack_weight(W, u, gs)
    pd = cabi.planes_to_dev(p)
    xd = cabi.bf16_dev(X)
    y = torch.empty((M, OUT), dtype=torch.bfloat16, device="cuda")
    yf = torch.empty((M, OUT), dtype=torch.float32, device="cuda")
    wsb = L.msaq_wa_gemv_workspace(M, OUT, K // 32, u, gs)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    _lib.check(L.msaq_wa_gemv_batched(xd.data_ptr(), pd["scale_exp"].data_ptr(), pd["upper_cm"].data_ptr(),
                                      pd["shared_cm"].data_ptr(), y.data_ptr(), yf.data_ptr(), M, OUT, K // 32, u, gs,
                                      ws.data_ptr(), wsb, _st()))
    torch.cuda.synchronize()
    cabi.check_output(y.float().cpu().numpy(), yf.cpu().numpy(), orc.wa_matmul(p, X), MAX_ABS_REL_TOL, REL_FRO_TOL,
                      F32_REL_FRO_TOL)
    yo = torch.ops.msaq.wa_gemv_batched(xd, pd["scale_exp"], pd["upper_cm"], pd["shared_cm"], M, OUT, K // 32, u, gs)
    assert torch.equal(yo, y)
    if M == 1:
        yw = torch.ops.msaq.wa_gemv(xd[0].contiguous(), pd["scale_exp"], pd["upper_cm"], pd["shared_cm"], OUT, K // 32, u, gs)
        assert torch.equal(yw, y[0])


def test_dequant_bf16_exact(rng, cfg):
    import cabi
    u, gs = cfg
    L = _lib.lib()
    OUT, K = 200, 256
    W = orc.to_bf16((rng.standard_normal((OUT, K)) * rng.uniform(0.001, 10, (OUT, 1))).astype(np.float32))
    p = orc.pack_weight(W, u, gs)
    pd = cabi.planes_to_dev(p)
    out = torch.empty((K, OUT), dtype=torch.bfloat16, device="cuda")
    _lib.check(L.msaq_dequant_bf16(pd["scale_exp"].data_ptr(), pd["upper_cm"].data_ptr(), pd["shared_cm"].data_ptr(),
                                   out.data_ptr(), OUT, K, u, gs, _st()))
    torch.cuda.synchronize()
    want = orc.dequant_weight(p).T                                      # exact in bf16: 8 significant bits times 2^e
    assert np.array_equal(out.float().cpu().numpy(), want.astype(np.float32))
    wo = torch.ops.msaq.ms_dequant_bf16(pd["scale_exp"], pd["upper_cm"], pd["shared_cm"], OUT, K, K // 32, u, gs)
    assert torch.equal(wo, out)

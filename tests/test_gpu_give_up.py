"""GPU tests of the give-up path: what the library does when a bounded wait runs out or an input
it can only see on the device is bad.  Nothing here faults, traps or hangs the GPU: the test hook makes
one thread block's copy-issuing thread stop early, the threads that wait for that copy reach their (shortened)
poll limit, give up, and the kernel finishes by itself with NaN in the affected outputs and a bit in the
status word.  The call after it must be correct again.
"""

import ctypes

import numpy as np
import pytest
import torch

from conftest import F32_REL_FRO_TOL, MAX_ABS_REL_TOL, REL_FRO_TOL
from oracle import msaq_oracle as orc

pytestmark = pytest.mark.gpu
OPT_WAIT_POLLS, OPT_TEST_SKIP_STAGE = 3, 4


def _status(clear=True):
    from ms_kernel_b200 import _lib
    v = ctypes.c_int(-1)
    _lib.check(_lib.lib().msaq_wait_status(int(clear), torch.cuda.current_stream().cuda_stream, ctypes.byref(v)))
    return v.value


class _short_waits:
    """Poll limit of a few thousand and the first block's producer stopping before `stage`."""

    def __init__(self, stage):
        self.stage = stage

    def __enter__(self):
        from ms_kernel_b200 import _lib
        L = _lib.lib()
        self.polls = L.msaq_get_option(OPT_WAIT_POLLS)
        assert L.msaq_set_option(OPT_WAIT_POLLS, 3000) == 0
        assert L.msaq_set_option(OPT_TEST_SKIP_STAGE, self.stage) == 0

    def __exit__(self, *a):
        from ms_kernel_b200 import _lib
        L = _lib.lib()
        L.msaq_set_option(OPT_TEST_SKIP_STAGE, -1)
        L.msaq_set_option(OPT_WAIT_POLLS, self.polls)


@pytest.mark.parametrize("M", (1, 4))
def test_gemv_wait_gives_up_and_next_call_is_correct(rng, M):
    import cabi
    OUT, K, u, gs = 2048, 2048, 4, 2
    W = orc.to_bf16((rng.standard_normal((OUT, K)) * 0.02).astype(np.float32))
    X = orc.to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    p = orc.pack_weight(W, u, gs)
    pd = cabi.planes_to_dev(p)
    ref = orc.wonly_matmul(p, X)
    x = cabi.bf16_dev(X)
    _status()
    with _short_waits(0):
        got, gotf = cabi.gemv("batched", x, pd, M=M)
    st = _status()
    assert st & 1, "the status word does not report the wait that gave up (status %d)" % st
    assert np.isnan(gotf).any(), "outputs fed by the abandoned stage must be NaN"
    # columns no abandoned thread block contributes to are still right
    ok = ~np.isnan(gotf)
    assert ok.any() and np.allclose(gotf[ok], ref[ok], rtol=1e-3, atol=1e-4)
    got2, gotf2 = cabi.gemv("batched", x, pd, M=M)
    cabi.check_output(got2, gotf2, ref, MAX_ABS_REL_TOL, REL_FRO_TOL, F32_REL_FRO_TOL)
    assert _status() == 0


def test_decode_wait_gives_up_and_next_call_is_correct(rng):
    import cabi
    u, gs, Hq, Hkv, Lk, D = 4, 2, 8, 2, 512, 128
    K = orc.to_bf16((rng.standard_normal((Hkv, Lk, D)) * 0.5).astype(np.float32))
    V = orc.to_bf16((rng.standard_normal((Hkv, Lk, D)) * 0.5).astype(np.float32))
    q = orc.to_bf16((rng.standard_normal((1, Hq, D)) * 0.5).astype(np.float32))
    pK, pV = orc.pack_kv(K, u, gs), orc.pack_kv(V, u, gs)
    kp = tuple(cabi.dev(pK[k]) for k in ("scale_exp", "upper", "shared"))
    vp = tuple(cabi.dev(pV[k]) for k in ("scale_exp", "upper", "shared"))
    ref = orc.decode_attention(q[0], orc.dequant_kv(pK), orc.dequant_kv(pV))
    _status()
    with _short_waits(0):
        got, gotf = cabi.decode(cabi.bf16_dev(q), kp, vp, 1, Hq, Hkv, Lk, D, u, gs)
    st = _status()
    assert st & 4, "the status word does not report the wait that gave up (status %d)" % st
    G = Hq // Hkv
    assert np.isnan(gotf[0, :G]).all(), "the heads of the abandoned tile's kv head must be NaN"
    assert np.allclose(gotf[0, G:], ref[G:], rtol=1e-3, atol=1e-4)
    got2, gotf2 = cabi.decode(cabi.bf16_dev(q), kp, vp, 1, Hq, Hkv, Lk, D, u, gs)
    cabi.check_output(got2[0], gotf2[0], ref, MAX_ABS_REL_TOL, REL_FRO_TOL, F32_REL_FRO_TOL)
    assert _status() == 0


def test_append_skips_out_of_range_device_positions(rng):
    """Per-sequence positions live in device memory, so only the kernel can check them: rows whose
    position is negative or beyond the capacity are skipped (no byte outside the planes or in another
    slot changes) and the status word reports it."""
    import cabi
    u, gs, B, Hkv, D, Lcap = 4, 2, 3, 2, 128, 32
    X = orc.to_bf16(rng.standard_normal((B * Hkv, D)).astype(np.float32))
    planes = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs, fill=0x5A)
    before = [t.clone() for t in planes]
    pos = np.array([-1, Lcap + 5, 3], np.int32)
    _status()
    cabi.kv_append_varlen(cabi.bf16_dev(X), planes, B, Hkv, D, cabi.dev(pos), Lcap, u, gs)
    torch.cuda.synchronize()
    assert _status() & 8
    tok = orc.pack_kv(X[:, None, :], u, gs)
    for t, b0, key in zip(planes, before, ("scale_exp", "upper", "shared")):
        got = t.cpu().numpy()
        exp = b0.cpu().numpy()
        exp[2 * Hkv:, :, 3] = tok[key][2 * Hkv:, :, 0]          # only sequence 2's rows were written, at slot 3
        assert np.array_equal(got, exp)
    assert _status() == 0


def test_fused_gemv_rejects_in_place_residual_update():
    from ms_kernel_b200 import _lib
    L = _lib.lib()
    M, OUT, NB = 1, 256, 8
    x = torch.zeros((M, NB * 32), dtype=torch.bfloat16, device="cuda")
    add = torch.zeros((M, NB * 32), dtype=torch.float32, device="cuda")
    se = torch.zeros((NB, OUT), dtype=torch.int8, device="cuda")
    up = torch.zeros((NB, OUT, 16), dtype=torch.uint8, device="cuda")
    sh = torch.zeros((NB, OUT, 8), dtype=torch.uint8, device="cuda")
    y = torch.zeros((M, OUT), dtype=torch.bfloat16, device="cuda")
    wsb = L.msaq_wonly_gemv_fused_workspace(M, OUT, NB, 4, 2)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    rc = L.msaq_wonly_gemv_fused(x.data_ptr(), 3, add.data_ptr(), 1, 1e-5, x.data_ptr(), se.data_ptr(), up.data_ptr(),
                                 sh.data_ptr(), y.data_ptr(), None, M, OUT, NB, 4, 2, ws.data_ptr(), wsb, None)
    assert rc == -1 and b"overlap" in L.msaq_last_error()


@pytest.mark.parametrize("bad", (float("inf"), float("nan")))
def test_non_finite_activation_gives_a_nan_row(rng, bad):
    """The reference's float path propagates Inf / NaN activations into the outputs; the integer staging
    of the tuned kernels cannot represent them, so the affected output row is NaN as a whole."""
    import cabi
    OUT, K, u, gs, M = 512, 1024, 4, 2, 3
    W = orc.to_bf16((rng.standard_normal((OUT, K)) * 0.02).astype(np.float32))
    X = orc.to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    p = orc.pack_weight(W, u, gs)
    ref = orc.wonly_matmul(p, X)
    X[1, 77] = bad
    got, gotf = cabi.gemv("batched", cabi.bf16_dev(X), cabi.planes_to_dev(p), M=M)
    assert np.isnan(gotf[1]).all() and np.isnan(got[1]).all()
    assert np.allclose(gotf[[0, 2]], ref[[0, 2]], rtol=1e-3, atol=1e-4)

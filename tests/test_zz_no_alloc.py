"""The allocation-free GEMV entry point (msaq_wonly_gemv_wide_static).

Some callers cannot hand the library a workspace because they are not allowed to allocate
device memory at all once they are running -- a plugin inside a host that owns the memory pool,
a control loop that bans cudaMalloc after start-up.  For them the split-K scratch sits in a
fixed array inside the library.  This test drives that entry point through the C ABI twice in
a row (the second call reuses whatever the first left in the array) and requires the same
bytes as the ordinary entry point with a caller-owned workspace, plus the usual tolerance
against the CPU oracle.  It is collected last so that a failure here cannot hide any other."""

import numpy as np
import pytest
import torch

from conftest import MAX_ABS_REL_TOL, REL_FRO_TOL
from oracle import msaq_oracle as orc

pytestmark = pytest.mark.gpu


def _static_gemv(L, x, pd):
    y = torch.empty(int(pd["OUT"]), dtype=torch.bfloat16, device="cuda")
    yf = torch.empty(int(pd["OUT"]), dtype=torch.float32, device="cuda")
    rc = L.msaq_wonly_gemv_wide_static(x.data_ptr(), pd["scale_exp"].data_ptr(), pd["upper_cm"].data_ptr(),
                                       pd["shared_cm"].data_ptr(), y.data_ptr(), yf.data_ptr(), int(pd["OUT"]),
                                       int(pd["nb"]), int(pd["u"]), int(pd["gs"]),
                                       torch.cuda.current_stream().cuda_stream)
    return rc, y, yf


@pytest.mark.parametrize("OUT,K,u", [(4096, 2048, 4), (1000, 512, 4), (768, 1024, 3)])
def test_static_scratch_gemv_matches_workspace_gemv(OUT, K, u):
    import cabi
    from ms_kernel_b200 import _lib
    L = _lib.lib()
    assert L.msaq_static_scratch_bytes() == 8 << 20
    rng = np.random.default_rng(77)
    gs = 2
    W = orc.to_bf16((rng.standard_normal((OUT, K)) * 0.02).astype(np.float32))
    p = orc.pack_weight(W, u, gs)
    pd = cabi.planes_to_dev(p)
    for call in range(2):                                  # two calls in a row share the scratch array
        xh = orc.to_bf16(rng.standard_normal(K).astype(np.float32))
        x = cabi.bf16_dev(xh)
        rc, y, yf = _static_gemv(L, x, pd)
        _lib.check(rc)
        torch.cuda.synchronize()
        ref_y, ref_f = cabi.gemv("wide", x, pd)
        assert np.array_equal(y.float().cpu().numpy(), ref_y), "call %d differs from the workspace entry point" % call
        assert np.array_equal(yf.cpu().numpy(), ref_f)
        oracle = orc.to_bf16(orc.wonly_matmul(p, xh[None])[0].astype(np.float32))
        assert orc.max_abs_rel(y.float().cpu().numpy(), oracle) <= MAX_ABS_REL_TOL
        assert orc.rel_fro(y.float().cpu().numpy(), oracle) <= REL_FRO_TOL


def test_static_scratch_rejects_oversized_problem():
    from ms_kernel_b200 import _lib
    L = _lib.lib()
    OUT, NB = 1 << 21, 1024                                 # scratch need beyond the built-in array
    assert L.msaq_wonly_gemv_workspace(1, OUT, NB, 4, 2) > L.msaq_static_scratch_bytes()
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    n0 = L.msaq_launch_count()
    rc = L.msaq_wonly_gemv_wide_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), None,
                                       OUT, NB, 4, 2, None)
    assert rc == -3 and b"built-in scratch" in L.msaq_last_error()
    assert L.msaq_launch_count() == n0                      # nothing was launched

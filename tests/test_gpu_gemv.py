"""GPU parity: weight-only GEMV entry points against the float64 oracle."""

import numpy as np
import pytest
import torch

from conftest import F32_REL_FRO_TOL, MAX_ABS_REL_TOL, REL_FRO_TOL
from oracle import msaq_oracle as orc

pytestmark = pytest.mark.gpu


def _case(rng, OUT, K, u, gs, M=1, wscale=(0.005, 0.08)):
    W = orc.to_bf16((rng.standard_normal((OUT, K)) * rng.uniform(*wscale, (OUT, 1))).astype(np.float32))
    X = orc.to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    return W, X, orc.pack_weight(W, u, gs)


def _check(got, gotf, ref):
    import cabi
    cabi.check_output(got, gotf, ref, MAX_ABS_REL_TOL, REL_FRO_TOL, F32_REL_FRO_TOL)


@pytest.mark.parametrize("OUT,K", [(128, 256), (200, 96), (1, 32), (4096, 4096 // 8)])
def test_gemv_wide_and_rowmajor(rng, cfg, OUT, K):
    import cabi
    u, gs = cfg
    W, X, p = _case(rng, OUT, K, u, gs)
    pd = cabi.planes_to_dev(p)
    ref = orc.wonly_matmul(p, X)[0]
    x = cabi.bf16_dev(X[0])
    for kind in ("wide", "rowmajor"):
        got, gotf = cabi.gemv(kind, x, pd)
        _check(got, gotf, ref)


@pytest.mark.parametrize("gs", (16, 32))
@pytest.mark.parametrize("u", (2, 3, 4))
def test_gemv_large_groups(rng, u, gs):
    import cabi
    W, X, p = _case(rng, 256, 512, u, gs)
    got, gotf = cabi.gemv("wide", cabi.bf16_dev(X[0]), cabi.planes_to_dev(p))
    _check(got, gotf, orc.wonly_matmul(p, X)[0])


@pytest.mark.parametrize("M", (1, 2, 3, 4, 7, 8, 16, 33, 64))
def test_gemv_batched(rng, cfg, M):
    import cabi
    u, gs = cfg
    W, X, p = _case(rng, 384, 512, u, gs, M=M)
    got, gotf = cabi.gemv("batched", cabi.bf16_dev(X), cabi.planes_to_dev(p), M=M)
    _check(got, gotf, orc.wonly_matmul(p, X))


@pytest.mark.parametrize("M,OUT,K", [(9, 512, 256), (16, 384, 512), (17, 1040, 2048), (64, 2048, 4096),
                                     (100, 528, 1024), (128, 512, 512), (130, 1024, 512), (300, 400, 256)])
def test_gemv_batched_tensor_memory_path(rng, M, OUT, K):
    """u4/gs2 with 9 rows and more runs on tcgen05 with tensor-memory accumulators: row tiles that
    split over several CTAs (split-K partials), ragged last tiles, more than 128 rows (several
    launches), against the oracle -- and against the integer-MMA path with the option off."""
    import cabi
    from ms_kernel_b200 import _lib
    W, X, p = _case(rng, OUT, K, 4, 2, M=M)
    pd = cabi.planes_to_dev(p)
    ref = orc.wonly_matmul(p, X)
    L = _lib.lib()
    assert L.msaq_get_option(2) == 1
    got, gotf = cabi.gemv("batched", cabi.bf16_dev(X), pd, M=M)
    _check(got, gotf, ref)
    assert L.msaq_set_option(2, 0) == 0
    try:
        got2, gotf2 = cabi.gemv("batched", cabi.bf16_dev(X), pd, M=M)
    finally:
        L.msaq_set_option(2, 1)
    _check(got2, gotf2, ref)
    assert orc.rel_fro(gotf, gotf2) < 1e-4


@pytest.mark.parametrize("u", (2, 3))
@pytest.mark.parametrize("M,OUT,K", [(1, 512, 256), (1, 1040, 2048), (4, 2048, 1024), (17, 528, 1024), (64, 2048, 4096),
                                     (130, 400, 256)])
def test_gemv_u2_u3_tensor_memory_path(rng, u, M, OUT, K):
    """The 5+3 and 6+2 bit formats (gs = 2) run on the tensor-memory kernel at every batch size: bit fields
    that straddle words, ragged tiles, split-K, several row tiles -- against the oracle, and against the
    generic kernel with the option off."""
    import cabi
    from ms_kernel_b200 import _lib
    W, X, p = _case(rng, OUT, K, u, 2, M=M)
    pd = cabi.planes_to_dev(p)
    ref = orc.wonly_matmul(p, X)
    kind = "batched" if M > 1 else "wide"
    xin = cabi.bf16_dev(X if M > 1 else X[0])
    got, gotf = cabi.gemv(kind, xin, pd, M=M) if M > 1 else cabi.gemv(kind, xin, pd)
    _check(got, gotf, ref if M > 1 else ref[0])
    L = _lib.lib()
    assert L.msaq_set_option(2, 0) == 0
    try:
        got2, gotf2 = cabi.gemv(kind, xin, pd, M=M) if M > 1 else cabi.gemv(kind, xin, pd)
    finally:
        L.msaq_set_option(2, 1)
    assert orc.rel_fro(gotf, gotf2) < 1e-4


@pytest.mark.parametrize("u", (2, 3, 4))
def test_gemv_llama_shape_vs_oracle(rng, u):
    """One full Llama-3.1-8B projection (O: 4096x4096) at gs=2, packed on the device."""
    import cabi
    OUT, K, gs = 4096, 4096, 2
    g = torch.Generator(device="cuda").manual_seed(3)
    W = (torch.randn((OUT, K), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    x = torch.randn((K,), generator=g, device="cuda").to(torch.bfloat16)
    pd = cabi.pack_weight(W, u, gs)
    got, gotf = cabi.gemv("wide", x, pd)
    Wq = orc.quantize_dequantize(W.float().cpu().numpy().reshape(-1, 32), u, gs).reshape(OUT, K)
    ref = Wq @ x.float().cpu().numpy().astype(np.float64)
    _check(got, gotf, ref)


def test_gemv_linearity_full_size(rng):
    """Size-independent property at the largest configured shape (28672x4096):
    y(a+b) == y(a) + y(b) in the fp32 output, to fp32 rounding."""
    import cabi
    OUT, K, u, gs = 28672, 4096, 4, 2
    g = torch.Generator(device="cuda").manual_seed(4)
    W = (torch.randn((OUT, K), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    pd = cabi.pack_weight(W, u, gs)
    a = torch.zeros(K, device="cuda"); b = torch.zeros(K, device="cuda")
    a[::2] = torch.randn(K // 2, generator=g, device="cuda")
    b[1::2] = torch.randn(K // 2, generator=g, device="cuda")
    a, b = a.to(torch.bfloat16), b.to(torch.bfloat16)
    ab = (a.float() + b.float()).to(torch.bfloat16)        # disjoint supports: the sum is exact in bf16
    _, ya = cabi.gemv("wide", a, pd)
    _, yb = cabi.gemv("wide", b, pd)
    _, yab = cabi.gemv("wide", ab, pd)
    assert orc.rel_fro(ya + yb, yab) < 1e-5


def test_gemv_rejects_bad_arguments():
    import cabi
    from ms_kernel_b200 import _lib
    L = _lib.lib()
    x = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    rc = L.msaq_wonly_gemv_wide(x.data_ptr(), None, None, None, None, None, 8, 2, 4, 2, None, 0, None)
    assert rc == -1 and b"null" in L.msaq_last_error()
    rc = L.msaq_wonly_gemv_wide(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), None,
                                8, 2, 5, 2, None, 0, None)
    assert rc == -2
    rc = L.msaq_wonly_gemv_wide(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), None,
                                8, 2, 4, 2, None, 0, None)
    assert rc == -3


@pytest.mark.parametrize("M", (1, 2, 3, 4))
@pytest.mark.parametrize("OUT,K", [(384, 512), (4096, 4096), (1040, 2048), (8192, 1024)])
def test_gemv_in_kernel_staging_equals_staging_kernel(rng, M, OUT, K):
    """Up to four rows, u4/gs2, small problems: the main kernel stages the activations itself (one
    launch); the same launch behind the separate staging kernel must give the same bits."""
    import cabi
    from ms_kernel_b200 import _lib
    W, X, p = _case(rng, OUT, K, 4, 2, M=M)
    pd = cabi.planes_to_dev(p)
    L = _lib.lib()
    assert L.msaq_get_option(5) == 1
    n0 = L.msaq_launch_count()
    got, gotf = cabi.gemv("batched", cabi.bf16_dev(X), pd, M=M)
    # where no thread block streams more than eighteen K blocks the staging kernel in front is gone
    launches = L.msaq_launch_count() - n0
    assert launches in (1, 2)
    if (OUT, K) in ((384, 512), (4096, 4096)):
        assert launches == 1
    _check(got, gotf, orc.wonly_matmul(p, X))
    assert L.msaq_set_option(5, 0) == 0
    try:
        got2, gotf2 = cabi.gemv("batched", cabi.bf16_dev(X), pd, M=M)
    finally:
        L.msaq_set_option(5, 1)
    assert np.array_equal(gotf, gotf2) and np.array_equal(got, got2)


def test_gemv_graph_replay_on_a_dirty_workspace(rng):
    """The split-K hand-off must not depend on what the workspace holds before its first use, and a
    captured launch must leave it ready for its own replay (the call's tag is baked into the graph)."""
    import cabi
    from ms_kernel_b200 import _lib
    L = _lib.lib()
    OUT, K, u, gs = 4096, 4096, 4, 2
    W, X, p = _case(rng, OUT, K, u, gs, M=1)
    pd = cabi.planes_to_dev(p)
    ref = orc.wonly_matmul(p, X)[0]
    x = cabi.bf16_dev(X[0])
    y = torch.zeros(OUT, dtype=torch.bfloat16, device="cuda")
    yf = torch.zeros(OUT, dtype=torch.float32, device="cuda")
    wsb = L.msaq_wonly_gemv_workspace(1, OUT, K // 32, u, gs)
    for fill in (0xFF, 0x00, 0x5A):
        ws = torch.full((wsb,), fill, dtype=torch.uint8, device="cuda")
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                _lib.check(L.msaq_wonly_gemv_wide(x.data_ptr(), pd["scale_exp"].data_ptr(), pd["upper_cm"].data_ptr(),
                                                  pd["shared_cm"].data_ptr(), y.data_ptr(), yf.data_ptr(), OUT, K // 32,
                                                  u, gs, ws.data_ptr(), wsb, s.cuda_stream))
        torch.cuda.current_stream().wait_stream(s)
        outs = []
        for _ in range(4):
            yf.zero_()
            g.replay()
            torch.cuda.synchronize()
            outs.append(yf.cpu().numpy().copy())
        for o in outs:
            assert np.array_equal(o, outs[0])
        _check(y.float().cpu().numpy(), outs[0], ref)
        del g


@pytest.mark.parametrize("OUT,K,M", [(4096, 4096, 1), (2560, 8192, 1), (8192, 2048, 4), (1024, 512, 2)])
def test_early_weights_option_changes_no_bit(rng, OUT, K, M):
    """MSAQ_OPT_EARLY_WEIGHTS moves the first weight copies in front of the wait for the preceding kernel; with the
    weights complete before the call (a synchronise after packing: the option's contract) every output bit is the
    same, plain and with a fused prologue, back to back in one stream."""
    from ms_kernel_b200 import _lib, ops, pack
    dev = torch.device("cuda")
    g = torch.Generator(device="cuda").manual_seed(OUT + K + M)
    W = (torch.randn((OUT, K), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    lin = ops.PackedLinear(pack.pack_weight(W, 4, 2, device=dev), dev)
    x = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
    torch.cuda.synchronize()
    L = _lib.lib()
    outs = []
    for early in (0, 1):
        assert L.msaq_set_option(6, early) == 0
        try:
            ys = []
            for _ in range(3):                                   # back to back: each call runs behind the one before
                ys.append(lin.fwd(x))
                ys.append(lin.fwd_fused(x, ops.PRO_RMSNORM))
            torch.cuda.synchronize()
        finally:
            L.msaq_set_option(6, 0)
        outs.append(ys)
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    assert L.msaq_get_option(6) == 0


@pytest.mark.parametrize("OUT,K,M,u,prologue", [(8192, 28672 // 4, 1, 4, 2), (4096, 4096, 1, 4, 0), (8192, 1024, 4, 4, 1),
                                               (1024, 512, 8, 4, 2), (8192, 2048, 16, 4, 2), (1024, 512, 2, 3, 0)])
def test_residual_add_behind_the_gemv_is_bit_equal_to_the_two_steps(rng, OUT, K, M, u, prologue):
    """msaq_wonly_gemv_fused_add: the residual add of a layer's last projection done by the GEMV's finishing warps
    rounds exactly as the GEMV followed by msaq_add_residual (16 rows and u = 3 take the two-kernel route inside)."""
    from ms_kernel_b200 import ops, pack
    dev = torch.device("cuda")
    g = torch.Generator(device="cuda").manual_seed(OUT + K + M + u)
    W = (torch.randn((OUT, K), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    lin = ops.PackedLinear(pack.pack_weight(W, u, 2, device=dev), dev)
    x = torch.randn((M, (2 if prologue == 2 else 1) * K), generator=g, device="cuda").to(torch.bfloat16)
    h = torch.randn((M, OUT), generator=g, device="cuda").to(torch.bfloat16)
    y = lin.fwd_fused(x, prologue) if prologue else lin.fwd(x)
    want = torch.ops.msaq.add_residual(h, y.reshape(M, OUT).contiguous())
    got = lin.fwd_fused_add(x, prologue, h)
    torch.cuda.synchronize()
    assert torch.equal(got, want.reshape(M, OUT))

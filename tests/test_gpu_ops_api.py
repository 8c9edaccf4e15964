"""GPU parity through the operator surface (torch.ops.msaq.*, ms_kernel_b200.ops):
the reference's own kernel gates (tests/test_w.py, tests/test_kv.py of the
reference) restated against this build, with this build's tolerance."""

import os

import numpy as np
import pytest
import torch

from conftest import MAX_ABS_REL_TOL, REL_FRO_TOL
from oracle import msaq_oracle as orc

pytestmark = pytest.mark.gpu


def _close(got, ref):
    ref_b = orc.to_bf16(np.asarray(ref, np.float32))
    assert orc.max_abs_rel(got, ref_b) <= MAX_ABS_REL_TOL
    assert orc.rel_fro(got, ref_b) <= REL_FRO_TOL


def _bf(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).cuda()


def test_backend_is_native():
    from ms_kernel_b200 import ops
    assert ops.available()
    import ms_cuda  # the reference's own import line must find this build
    assert hasattr(torch.ops.msaq, "wonly_gemv_wide")


def test_wonly_gemv_api(rng, cfg):
    from ms_kernel_b200 import ops
    u, gs = cfg
    OUT, K = 128, 256
    W = (rng.standard_normal((OUT, K)) * rng.uniform(0.2, 4.0, (OUT, 1))).astype(np.float32)
    p = orc.pack_weight(W, u, gs)
    x = rng.standard_normal(K).astype(np.float32)
    before = torch.ops.msaq.launch_count()
    got = ops.wonly_gemv(p, _bf(x)).float().cpu().numpy()
    assert torch.ops.msaq.launch_count() > before
    _close(got, orc.wonly_matmul(p, orc.to_bf16(x)[None])[0])
    # legacy row-major route (a pack dict without the column-major twins)
    p2 = {k: v for k, v in p.items() if not k.endswith("_cm")}
    got2 = ops.wonly_gemv(p2, _bf(x)).float().cpu().numpy()
    assert np.array_equal(got, got2)


def test_wonly_gemv_batched_api(rng, cfg):
    from ms_kernel_b200 import ops
    u, gs = cfg
    OUT, K, M = 128, 256, 16
    W = (rng.standard_normal((OUT, K)) * rng.uniform(0.2, 4.0, (OUT, 1))).astype(np.float32)
    p = orc.pack_weight(W, u, gs)
    X = rng.standard_normal((M, K)).astype(np.float32)
    got = ops.wonly_gemv_batched(p, _bf(X)).float().cpu().numpy()
    _close(got, orc.wonly_matmul(p, orc.to_bf16(X)))
    # batched rows equal single-row calls
    lin = ops.PackedLinear(p, "cuda")
    rows = torch.stack([lin.fwd(_bf(X[m])) for m in range(M)]).float().cpu().numpy()
    assert orc.rel_fro(rows, got) < 1e-3


def test_kv_decode_attention_api(rng, cfg):
    from ms_kernel_b200 import ops
    u, gs = cfg
    H, Lk, D = 4, 40, 64
    Kt = (rng.standard_normal((H, Lk, D)) * 0.5).astype(np.float32)
    Vt = (rng.standard_normal((H, Lk, D)) * 0.5).astype(np.float32)
    Q = (rng.standard_normal((H, D)) * 0.5).astype(np.float32)
    pK, pV = orc.pack_kv(Kt, u, gs), orc.pack_kv(Vt, u, gs)
    got = ops.kv_decode_attention(_bf(Q), pK, pV).float().cpu().numpy()
    _close(got, orc.kv_attention(orc.to_bf16(Q)[:, None, :], pK, pV, causal=True)[:, 0])


def test_kv_write_op_bytes_and_device_packers(rng, cfg):
    from ms_kernel_b200 import pack
    u, gs = cfg
    H, L, D = 4, 48, 128
    K = (rng.standard_normal((H, L, D)) * rng.uniform(0.3, 3, (H, 1, 1))).astype(np.float32)
    Kb = _bf(K)
    se, up, sh = torch.ops.msaq.kv_write(Kb, H, L, D, D // 32, u, gs)
    ref = orc.pack_kv(Kb.float().cpu().numpy(), u, gs)
    assert np.array_equal(se.cpu().numpy(), ref["scale_exp"])
    assert np.array_equal(up.cpu().numpy(), ref["upper"])
    assert np.array_equal(sh.cpu().numpy(), ref["shared"])
    pk = pack.to_numpy(pack.pack_kv(Kb, u, gs))
    for k in ("scale_exp", "upper", "shared"):
        assert np.array_equal(pk[k], ref[k])
    W = (rng.standard_normal((64, 128)) * 0.02).astype(np.float32)
    pw = pack.to_numpy(pack.pack_weight(W, u, gs))
    rw = orc.pack_weight(W, u, gs)
    for k in ("scale_exp", "upper", "shared", "upper_cm", "shared_cm"):
        assert np.array_equal(pw[k], rw[k]), k
    assert {k: pw[k] for k in ("OUT", "K", "nb", "u", "gs", "UB", "SB")} == {k: rw[k] for k in
                                                                             ("OUT", "K", "nb", "u", "gs", "UB", "SB")}


def test_qrot_env_flag_on_batched_op(rng):
    """MS_KV_QROT is read per call by the batched op and ignored by the single-sequence op."""
    u, gs, Hq, Hkv, Lk, D = 4, 2, 8, 2, 64, 128
    nb = D // 32
    K = _bf(rng.standard_normal((Hkv, Lk, D)))
    V = _bf(rng.standard_normal((Hkv, Lk, D)))
    q = _bf(rng.standard_normal((1, Hq, D)))
    kr = torch.ops.msaq.kv_write_rot(K, Hkv, Lk, D, nb, u, gs)
    vv = torch.ops.msaq.kv_write(V, Hkv, Lk, D, nb, u, gs)
    op = torch.ops.msaq.kv_decode_attention_batched
    old = os.environ.get("MS_KV_QROT")
    try:
        os.environ["MS_KV_QROT"] = "1"
        on = op(q, *kr, *vv, 1, Hq, Hkv, Lk, D, nb, u, gs)
        single = torch.ops.msaq.kv_decode_attention(q[0], *kr, *vv, Hq, Hkv, Lk, D, nb, u, gs)
        os.environ["MS_KV_QROT"] = "0"
        off = op(q, *kr, *vv, 1, Hq, Hkv, Lk, D, nb, u, gs)
    finally:
        if old is None:
            os.environ.pop("MS_KV_QROT", None)
        else:
            os.environ["MS_KV_QROT"] = old
    explicit = torch.ops.msaq.kv_decode_attention_varlen(
        q, *kr, *vv, torch.tensor([Lk], dtype=torch.int32, device="cuda"), 1, Hq, Hkv, Lk, D, nb, u, gs, Lk, True)
    assert torch.equal(on, explicit)
    assert torch.equal(off[0], single)
    assert not torch.equal(on, off)
    host_rot = torch.ops.msaq.hadamard_rotate(q)
    off_hostrot = op(host_rot, *kr, *vv, 1, Hq, Hkv, Lk, D, nb, u, gs)
    assert orc.rel_fro(on.float().cpu().numpy(), off_hostrot.float().cpu().numpy()) < 2e-2


def test_kvcache_holder_append_attend(rng):
    from ms_kernel_b200 import ops
    B, Hq, Hkv, D, Lcap, u, gs = 2, 8, 2, 128, 64, 4, 2
    cache = ops.KVCache(B, Hkv, D, Lcap, u, gs, "cuda", rotate=True)
    L0 = 40
    K = _bf(rng.standard_normal((B, Hkv, L0 + 1, D)))
    V = _bf(rng.standard_normal((B, Hkv, L0 + 1, D)))
    cache.fill(K[:, :, :L0], V[:, :, :L0])
    cache.append(K[:, :, L0], V[:, :, L0], L0)
    q = _bf(rng.standard_normal((B, Hq, D)))
    got = cache.attend(q, L0 + 1).float().cpu().numpy()
    kn = tuple(t.cpu().numpy() for t in cache.k)
    vn = tuple(t.cpu().numpy() for t in cache.v)
    ref = orc.decode_attention_batched(q.float().cpu().numpy(), kn, vn, u, gs, [L0 + 1] * B, qrot=True)
    _close(got, ref)
    # the appended slot equals the oracle's rotated packing of that token
    tok = orc.pack_kv_rotated(K[:, :, L0].float().cpu().numpy().reshape(B * Hkv, 1, D), u, gs)
    assert np.array_equal(kn[1].reshape(B * Hkv, D // 32, Lcap, -1)[:, :, L0], tok["upper"][:, :, 0])


def test_ops_capture_in_cuda_graph(rng):
    """The ops make no host sync and no allocation outside torch's allocator: capturable."""
    from ms_kernel_b200 import ops
    u, gs, OUT, K = 4, 2, 512, 512
    W = (rng.standard_normal((OUT, K)) * 0.02).astype(np.float32)
    lin = ops.PackedLinear(orc.pack_weight(W, u, gs), "cuda")
    x = _bf(rng.standard_normal(K))
    eager = lin.fwd(x).clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        lin.fwd(x)
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y = lin.fwd(x)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, eager)


def test_layer_glue_ops(rng):
    """Fused rmsnorm / SiLU*mul / residual add against plain float64 formulas."""
    B, H, F = 3, 1024, 768
    x = _bf(rng.standard_normal((B, H)) * 3)
    xf = x.float().cpu().numpy().astype(np.float64)
    ref = xf / np.sqrt((xf ** 2).mean(-1, keepdims=True) + 1e-5)
    got = torch.ops.msaq.rmsnorm(x, 1e-5).float().cpu().numpy()
    assert orc.rel_fro(got, orc.to_bf16(ref.astype(np.float32))) < 1e-3
    gu = _bf(rng.standard_normal((B, 2 * F)) * 2)
    g64 = gu.float().cpu().numpy().astype(np.float64)
    ref = g64[:, :F] / (1 + np.exp(-g64[:, :F])) * g64[:, F:]
    got = torch.ops.msaq.silu_mul(gu).float().cpu().numpy()
    assert orc.rel_fro(got, orc.to_bf16(ref.astype(np.float32))) < 1e-3
    d32 = torch.from_numpy(rng.standard_normal((B, H)).astype(np.float32)).cuda()
    got = torch.ops.msaq.add_residual(x, d32).float().cpu().numpy()
    assert np.array_equal(got, orc.to_bf16(x.float().cpu().numpy() + d32.cpu().numpy()))
    got = torch.ops.msaq.add_residual(x, d32.to(torch.bfloat16)).float().cpu().numpy()
    assert np.array_equal(got, orc.to_bf16(x.float().cpu().numpy() + d32.to(torch.bfloat16).float().cpu().numpy()))


@pytest.mark.parametrize("chained", [0, 1])
def test_chained_launch_modes_agree(rng, chained):
    """Overlapped launches change timing only: a chain of dependent ops (GEMV -> glue -> GEMV ->
    append -> decode), each consuming the previous one's output and sharing scratch, gives the
    same bits in every launch mode, eagerly and replayed from a CUDA graph."""
    from ms_kernel_b200 import ops
    u, gs, Hd, Hq, Hkv, D, Lk = 4, 2, 1024, 8, 2, 128, 700
    Lcap = 704
    W1 = (rng.standard_normal(((Hq + 2 * Hkv) * D, Hd)) * 0.05).astype(np.float32)
    W2 = (rng.standard_normal((Hd, Hq * D)) * 0.05).astype(np.float32)
    l1 = ops.PackedLinear(orc.pack_weight(W1, u, gs), "cuda")
    l2 = ops.PackedLinear(orc.pack_weight(W2, u, gs), "cuda")
    Kc = _bf(rng.standard_normal((1, Hkv, Lk - 1, D)))
    Vc = _bf(rng.standard_normal((1, Hkv, Lk - 1, D)))
    h = _bf(rng.standard_normal((1, Hd)))

    def chain(cache):
        x = torch.ops.msaq.rmsnorm(h, 1e-5)
        qkv = l1.fwd(x)
        q = qkv[:, : Hq * D].reshape(1, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(1, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].reshape(1, Hkv, D)
        cache.append(k, v, Lk - 1)
        a = cache.attend(q.contiguous(), Lk)
        o = l2.fwd(a.reshape(1, Hq * D))
        return torch.ops.msaq.add_residual(h, o)

    def fresh_cache():
        c = ops.KVCache(1, Hkv, D, Lcap, u, gs, "cuda", rotate=True)
        c.fill(Kc, Vc, 0)
        return c

    ops.set_option(ops.OPT_CHAINED_LAUNCH, False)
    want = chain(fresh_cache()).clone()
    try:
        ops.set_option(ops.OPT_CHAINED_LAUNCH, bool(chained))
        cache = fresh_cache()
        for _ in range(3):
            got = chain(cache)
            assert torch.equal(got, want)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            chain(cache)
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            y = chain(cache)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, want)
    finally:
        ops.set_option(ops.OPT_CHAINED_LAUNCH, True)

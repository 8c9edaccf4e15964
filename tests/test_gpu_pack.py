"""GPU parity: quantise-and-pack kernels must reproduce the oracle's bytes exactly."""

import numpy as np
import pytest
import torch

from oracle import msaq_oracle as orc

pytestmark = pytest.mark.gpu
ALL_CFG = [(u, gs) for u in (2, 3, 4) for gs in (2, 4, 8, 16, 32)]


def _eq(t, a):
    return np.array_equal(t.cpu().numpy(), a)


@pytest.mark.parametrize("u,gs", ALL_CFG)
def test_pack_weight_bytes(rng, golden, u, gs):
    import cabi
    OUT, K = 96, 256
    W = (rng.standard_normal((OUT, K)) * rng.uniform(0.005, 0.08, (OUT, 1))).astype(np.float32)
    edge = golden["dec_blocks"][:OUT]                          # edge blocks: zeros, ties, saturation, tiny, huge
    W[:len(edge), :32] = edge
    for as_bf16 in (True, False):
        Wd = cabi.bf16_dev(W) if as_bf16 else cabi.dev(W)
        ref = orc.pack_weight(Wd.float().cpu().numpy(), u, gs)
        got = cabi.pack_weight(Wd, u, gs)
        torch.cuda.synchronize()
        for k in ("scale_exp", "upper", "shared", "upper_cm", "shared_cm"):
            assert _eq(got[k], ref[k]), (k, as_bf16)


@pytest.mark.parametrize("D", (64, 128, 256))
def test_kv_write_bytes(rng, cfg, D):
    import cabi
    u, gs = cfg
    H, L = 4, 48
    K = (rng.standard_normal((H, L, D)) * rng.uniform(0.3, 3, (H, 1, 1))).astype(np.float32)
    Kb = cabi.bf16_dev(K)
    planes = cabi.empty_cache(H, D // 32, L, u, gs)
    cabi.kv_write(Kb, planes, H, L, D, 0, L, u, gs)
    ref = orc.pack_kv(Kb.float().cpu().numpy(), u, gs)
    for t, k in zip(planes, ("scale_exp", "upper", "shared")):
        assert _eq(t, ref[k]), k


def test_kv_append_bytes_and_untouched_slots(rng, cfg):
    import cabi
    u, gs = cfg
    H, L, D, Lcap = 4, 48, 128, 64
    K = (rng.standard_normal((H, L, D)) * rng.uniform(0.3, 3, (H, 1, 1))).astype(np.float32)
    Kb = cabi.bf16_dev(K)
    planes = cabi.empty_cache(H, D // 32, Lcap, u, gs, fill=0x5A)
    for pos in range(L):
        cabi.kv_append(Kb[:, pos, :].contiguous(), planes, H, D, pos, Lcap, u, gs)
    ref = orc.pack_kv(Kb.float().cpu().numpy(), u, gs)
    for t, k in zip(planes, ("scale_exp", "upper", "shared")):
        a = t.cpu().numpy()
        assert np.array_equal(a[:, :, :L], ref[k]), k
        assert np.all(a[:, :, L:].view(np.uint8) == 0x5A), "slots past the appended ones were written"


@pytest.mark.parametrize("u,gs", ALL_CFG)
def test_kv_append_rot_bytes(rng, u, gs):
    import cabi
    H, L, D = 3, 24, 128
    K = rng.standard_normal((H, L, D)).astype(np.float32)
    K[:, :, [5, 44, 90, 127]] *= 20                         # persistent outlier channels
    Kb = cabi.bf16_dev(K)
    planes = cabi.empty_cache(H, D // 32, L, u, gs)
    for pos in range(L):
        cabi.kv_append(Kb[:, pos, :].contiguous(), planes, H, D, pos, L, u, gs, rot=True)
    ref = orc.pack_kv_rotated(Kb.float().cpu().numpy(), u, gs)
    for t, k in zip(planes, ("scale_exp", "upper", "shared")):
        assert _eq(t, ref[k]), k
    # the prefill writer with rotation gives the same bytes
    planes2 = cabi.empty_cache(H, D // 32, L, u, gs)
    cabi.kv_write(Kb, planes2, H, L, D, 0, L, u, gs, rot=True)
    for a, b in zip(planes, planes2):
        assert torch.equal(a, b)


def test_kv_append_rot_golden(golden):
    import cabi
    K = golden["rot_K"]
    H, L, D = K.shape
    Kb = cabi.bf16_dev(K)
    for u, gs in ((4, 2), (3, 8), (2, 4)):
        planes = cabi.empty_cache(H, D // 32, L, u, gs)
        cabi.kv_write(Kb, planes, H, L, D, 0, L, u, gs, rot=True)
        for t, k in zip(planes, ("scale_exp", "upper", "shared")):
            assert _eq(t, golden[f"rot_{k}_u{u}_gs{gs}"]), (u, gs, k)


def test_kv_append_varlen_positions(rng):
    import cabi
    u, gs, B, Hkv, D, Lcap = 4, 2, 3, 2, 128, 16
    X = cabi.bf16_dev(rng.standard_normal((B * Hkv, D)))
    pos = torch.tensor([0, 7, 15], dtype=torch.int32, device="cuda")
    for rot in (False, True):
        planes = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs, fill=0x33)
        cabi.kv_append_varlen(X, planes, B, Hkv, D, pos, Lcap, u, gs, rot=rot)
        xr = X.float().cpu().numpy()[:, None, :]
        ref = orc.pack_kv_rotated(xr, u, gs) if rot else orc.pack_kv(xr, u, gs)
        for t, k in zip(planes, ("scale_exp", "upper", "shared")):
            a = t.cpu().numpy()
            for r in range(B * Hkv):
                p = int(pos[r // Hkv])
                assert np.array_equal(a[r, :, p], ref[k][r, :, 0]), (k, r)
                rest = np.delete(a[r], p, axis=1)
                assert np.all(rest.view(np.uint8) == 0x33)


@pytest.mark.parametrize("u,gs", [(4, 2), (3, 4), (2, 8)])
@pytest.mark.parametrize("varlen", (False, True))
def test_kv_append_pair_equals_the_two_appends(rng, u, gs, varlen):
    """K (rotated) and V of a step in one launch: the same bytes as kv_append_rot + kv_append, other slots untouched."""
    import cabi
    from ms_kernel_b200 import _lib
    B, Hkv, D, Lcap = 3, 2, 128, 16
    Xk = cabi.bf16_dev(rng.standard_normal((B * Hkv, D)) * 2)
    Xv = cabi.bf16_dev(rng.standard_normal((B * Hkv, D)))
    pos = torch.tensor([2, 9, 15], dtype=torch.int32, device="cuda")
    kp = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs, fill=0x33)
    vp = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs, fill=0x33)
    L = _lib.lib()
    _lib.check(L.msaq_kv_append_pair(Xk.data_ptr(), Xv.data_ptr(), *[t.data_ptr() for t in kp], *[t.data_ptr() for t in vp],
                                     B, Hkv, D, D // 32, 5, pos.data_ptr() if varlen else None, Lcap, u, gs, 1,
                                     torch.cuda.current_stream().cuda_stream))
    kr = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs, fill=0x33)
    vr = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs, fill=0x33)
    if varlen:
        cabi.kv_append_varlen(Xk, kr, B, Hkv, D, pos, Lcap, u, gs, rot=True)
        cabi.kv_append_varlen(Xv, vr, B, Hkv, D, pos, Lcap, u, gs, rot=False)
    else:
        cabi.kv_append(Xk, kr, B * Hkv, D, 5, Lcap, u, gs, rot=True)
        cabi.kv_append(Xv, vr, B * Hkv, D, 5, Lcap, u, gs, rot=False)
    torch.cuda.synchronize()
    for got, ref in zip(kp + vp, kr + vr):
        assert torch.equal(got, ref)
    assert L.msaq_kv_append_pair(None, Xv.data_ptr(), *[t.data_ptr() for t in kp], *[t.data_ptr() for t in vp],
                                 B, Hkv, D, D // 32, 5, None, Lcap, u, gs, 1, None) == -1
    assert L.msaq_kv_append_pair(Xk.data_ptr(), Xv.data_ptr(), *[t.data_ptr() for t in kp], *[t.data_ptr() for t in vp],
                                 B, Hkv, D, D // 32, Lcap, None, Lcap, u, gs, 1, None) == -1      # slot past the capacity


@pytest.mark.parametrize("D", (32, 64, 128, 256))
def test_hadamard_rotate_bits(rng, D):
    import cabi
    x = cabi.bf16_dev(rng.standard_normal((37, D)) * 3)
    got = cabi.hadamard_rotate(x).float().cpu().numpy()
    ref = orc.hadamard_rotate_bf16(x.float().cpu().numpy())
    assert np.array_equal(got, ref)
    # and it is the orthonormal Hadamard product up to bf16 rounding
    dense = x.float().cpu().numpy().astype(np.float64) @ orc.hadamard_matrix(D)
    assert orc.rel_fro(got, dense) < 4e-3


def test_full_size_round_trip_property(rng):
    """At a cache size the CPU oracle cannot pack in seconds: write -> bytes are
    a fixed point (re-packing the dequantised cache reproduces itself) on a sample."""
    import cabi
    u, gs, H, L, D = 4, 2, 8, 16384, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    X = torch.randn((H, L, D), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    planes = cabi.empty_cache(H, D // 32, L, u, gs)
    cabi.kv_write(X, planes, H, L, D, 0, L, u, gs)
    torch.cuda.synchronize()
    idx = np.sort(rng.choice(L, 64, replace=False))
    sub = tuple(t[:, :, idx].cpu().numpy() for t in planes)
    ref = orc.pack_kv(X[:, idx].float().cpu().numpy(), u, gs)
    for a, k in zip(sub, ("scale_exp", "upper", "shared")):
        assert np.array_equal(a, ref[k]), k

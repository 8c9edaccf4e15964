"""GPU parity of the rotary position embedding fused into the cache writers and the decode prologue,
against the oracle's restatement of the reference harness's rope_bthd (tests/harness_batchsweep.py:
118-137; pinned bit for bit by tests/test_oracle_golden.py)."""

import numpy as np
import pytest
import torch

from conftest import F32_REL_FRO_TOL, MAX_ABS_REL_TOL, REL_FRO_TOL
from ms_kernel_b200 import _lib
from oracle import msaq_oracle as orc

pytestmark = pytest.mark.gpu
KEYS = ("scale_exp", "upper", "shared")


def _st():
    return torch.cuda.current_stream().cuda_stream


def _tables(positions, D):
    c, s = orc.rope_tables(np.asarray(positions), D)
    return c, s, torch.from_numpy(c).cuda(), torch.from_numpy(s).cuda()


@pytest.mark.parametrize("D", (32, 64, 128, 256))
def test_rope_standalone_bit_exact(rng, D):
    import cabi
    L = _lib.lib()
    B, H = 5, 3
    x = orc.to_bf16(rng.standard_normal((B, H, D)).astype(np.float32) * 3)
    xd = cabi.bf16_dev(x)
    out = torch.empty_like(xd)
    # a table row per position, positions per sequence
    pos = np.array([0, 1, 17, 38, 39], np.int32)
    c, s, cd, sd = _tables(np.arange(40), D)
    pos_d = cabi.dev(pos)
    _lib.check(L.msaq_rope(xd.data_ptr(), out.data_ptr(), B, H, D, cd.data_ptr(), sd.data_ptr(), 40, 0,
                           pos_d.data_ptr(), _st()))
    want = orc.rope(x, c[pos][:, None, :], s[pos][:, None, :])
    assert np.array_equal(out.float().cpu().numpy(), want)
    # one position for every sequence, single-row tables
    c1, s1, c1d, s1d = _tables([8191], D)
    _lib.check(L.msaq_rope(xd.data_ptr(), out.data_ptr(), B, H, D, c1d.data_ptr(), s1d.data_ptr(), 1, 8191, None, _st()))
    assert np.array_equal(out.float().cpu().numpy(), orc.rope(x, c1[0], s1[0]))
    # a scalar position outside the table is refused
    assert L.msaq_rope(xd.data_ptr(), out.data_ptr(), B, H, D, cd.data_ptr(), sd.data_ptr(), 40, 40, None, _st()) == -1


def test_rope_reference_fixture(golden):
    """The reference harness's own inputs, tables and outputs."""
    import cabi
    L = _lib.lib()
    x, y = golden["rope_x"], golden["rope_y"]                      # [B, L, H, D]
    Bq, Lp, H, D = x.shape
    cd, sd = cabi.dev(golden["rope_cos"]), cabi.dev(golden["rope_sin"])
    xs = np.ascontiguousarray(x.reshape(Bq * Lp, H, D))            # one "sequence" per (b, t): its position is t
    pos = np.tile(np.arange(Lp, dtype=np.int32), Bq)
    xd = cabi.bf16_dev(xs)
    out = torch.empty_like(xd)
    pos_d = cabi.dev(pos)
    _lib.check(L.msaq_rope(xd.data_ptr(), out.data_ptr(), Bq * Lp, H, D, cd.data_ptr(), sd.data_ptr(), Lp, 0,
                           pos_d.data_ptr(), _st()))
    assert np.array_equal(out.float().cpu().numpy().reshape(x.shape), y)


@pytest.mark.parametrize("D", (64, 128))
def test_append_with_rope_bytes(rng, cfg, D):
    """K rows: RoPE -> bf16 -> Hadamard rotation -> quantise, V rows: plain, both in one launch."""
    import cabi
    u, gs = cfg
    L = _lib.lib()
    B, Hkv, Lcap = 3, 2, 24
    Xk = orc.to_bf16(rng.standard_normal((B * Hkv, D)).astype(np.float32))
    Xk[:, [3, 40]] *= 20
    Xk = orc.to_bf16(Xk)
    Xv = orc.to_bf16(rng.standard_normal((B * Hkv, D)).astype(np.float32))
    pos = np.array([5, 0, 23], np.int32)
    c, s, cd, sd = _tables(np.arange(Lcap), D)
    xk_d, xv_d, pos_d = cabi.bf16_dev(Xk), cabi.bf16_dev(Xv), cabi.dev(pos)      # kept alive across the launches
    for rotate in (1, 0):
        kp = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs, fill=0x33)
        vp = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs, fill=0x33)
        _lib.check(L.msaq_kv_append_pair_rope(xk_d.data_ptr(), xv_d.data_ptr(),
                                              *[t.data_ptr() for t in kp], *[t.data_ptr() for t in vp], B, Hkv, D, D // 32,
                                              0, pos_d.data_ptr(), Lcap, u, gs, rotate, cd.data_ptr(), sd.data_ptr(),
                                              Lcap, _st()))
        torch.cuda.synchronize()
        rows_pos = np.repeat(pos, Hkv)
        kr = orc.rope(Xk, c[rows_pos], s[rows_pos])
        tokk = (orc.pack_kv_rotated if rotate else orc.pack_kv)(kr[:, None, :], u, gs)
        tokv = orc.pack_kv(Xv[:, None, :], u, gs)
        for t, key in zip(kp, KEYS):
            got = t.cpu().numpy()
            for r in range(B * Hkv):
                assert np.array_equal(got[r, :, rows_pos[r]], tokk[key][r, :, 0]), (key, r)
        for t, key in zip(vp, KEYS):
            got = t.cpu().numpy()
            for r in range(B * Hkv):
                assert np.array_equal(got[r, :, rows_pos[r]], tokv[key][r, :, 0]), (key, r)
    # tables that do not cover the capacity are refused when positions come from device memory
    assert L.msaq_kv_append_pair_rope(xk_d.data_ptr(), xv_d.data_ptr(),
                                      *[t.data_ptr() for t in kp], *[t.data_ptr() for t in vp], B, Hkv, D, D // 32, 0,
                                      pos_d.data_ptr(), Lcap, u, gs, 1, cd.data_ptr(), sd.data_ptr(), Lcap - 1,
                                      _st()) == -1


def test_prefill_write_with_rope_reference_fixture(golden):
    """kv_write with RoPE and rotation on the reference harness's rows: the planes the reference's
    pack_kv gives for rope_bthd -> butterfly rotation."""
    import cabi
    L = _lib.lib()
    x = golden["rope_x"][0]                                        # [L, H, D]
    Lp, H, D = x.shape
    X = np.ascontiguousarray(x.transpose(1, 0, 2))                 # [H, L, D]
    cd, sd = cabi.dev(golden["rope_cos"]), cabi.dev(golden["rope_sin"])
    for u, gs in ((4, 2), (3, 8), (2, 4)):
        planes = cabi.empty_cache(H, D // 32, Lp, u, gs)
        x_d = cabi.bf16_dev(X)
        _lib.check(L.msaq_kv_write_rope(x_d.data_ptr(), *[t.data_ptr() for t in planes], H, Lp, D, D // 32, 0,
                                        Lp, u, gs, 1, cd.data_ptr(), sd.data_ptr(), Lp, _st()))
        torch.cuda.synchronize()
        for t, key in zip(planes, KEYS):
            assert np.array_equal(t.cpu().numpy(), golden[f"ropek_{key}_u{u}_gs{gs}"]), (u, gs, key)


@pytest.mark.parametrize("u,gs,D", [(4, 2, 128), (3, 4, 128), (4, 2, 64)], ids=["tuned", "generic_u3", "generic_d64"])
def test_decode_with_query_rope(rng, u, gs, D):
    """The query's RoPE in the decode prologue (tuned and generic kernels), then the Hadamard rotation,
    against the oracle fed rope(q)."""
    import cabi
    L = _lib.lib()
    B, Hq, Hkv, Lk, Lcap = 3, 8, 2, 200, 208
    K = orc.to_bf16(rng.standard_normal((B * Hkv, Lk, D)).astype(np.float32))
    V = orc.to_bf16(rng.standard_normal((B * Hkv, Lk, D)).astype(np.float32))
    q = orc.to_bf16(rng.standard_normal((B, Hq, D)).astype(np.float32))
    kp = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs)
    vp = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs)
    cabi.kv_write(cabi.bf16_dev(K), kp, B * Hkv, Lk, D, 0, Lcap, u, gs, rot=True)
    cabi.kv_write(cabi.bf16_dev(V), vp, B * Hkv, Lk, D, 0, Lcap, u, gs)
    lens = np.array([Lk, 150, 77], np.int32)
    qpos = (lens - 1).astype(np.int32)
    c, s, cd, sd = _tables(np.arange(Lcap), D)
    out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device="cuda")
    outf = torch.empty((B, Hq, D), dtype=torch.float32, device="cuda")
    wsb = L.msaq_kv_decode_workspace(B, Hq, Hkv, Lk, D)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    q_d, lens_d, qpos_d = cabi.bf16_dev(q), cabi.dev(lens), cabi.dev(qpos)
    _lib.check(L.msaq_kv_decode_attention_rope(q_d.data_ptr(), *[t.data_ptr() for t in kp],
                                               *[t.data_ptr() for t in vp], out.data_ptr(), outf.data_ptr(),
                                               lens_d.data_ptr(), B, Hq, Hkv, Lk, D, D // 32, u, gs, Lcap, 1,
                                               cd.data_ptr(), sd.data_ptr(), Lcap, 0, qpos_d.data_ptr(),
                                               ws.data_ptr(), wsb, _st()))
    torch.cuda.synchronize()
    qr = orc.rope(q, c[qpos][:, None, :], s[qpos][:, None, :])
    shaped = lambda pl: tuple(t.cpu().numpy().reshape((B, Hkv) + tuple(t.shape[1:])) for t in pl)
    ref = orc.decode_attention_batched(qr, shaped(kp), shaped(vp), u, gs, lens, qrot=True)
    cabi.check_output(out.float().cpu().numpy(), outf.cpu().numpy(), ref, MAX_ABS_REL_TOL, REL_FRO_TOL, F32_REL_FRO_TOL * 2)

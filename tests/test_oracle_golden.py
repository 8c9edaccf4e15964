"""The CPU oracle replayed against fixtures recorded from the reference's NumPy code."""

import numpy as np
import pytest

from oracle import msaq_oracle as orc

ALL_GS = (2, 4, 8, 16, 32)


@pytest.mark.parametrize("u", (2, 3, 4))
@pytest.mark.parametrize("gs", ALL_GS)
def test_decompose_codes_match_reference(golden, u, gs):
    exp, up, sh = orc.decompose(golden["dec_blocks"], u, gs)
    assert np.array_equal(exp, golden[f"dec_exp_u{u}_gs{gs}"])
    assert np.array_equal(up, golden[f"dec_up_u{u}_gs{gs}"])
    assert np.array_equal(sh, golden[f"dec_sh_u{u}_gs{gs}"])


def test_pack_weight_planes_match_reference(golden, cfg):
    u, gs = cfg
    p = orc.pack_weight(golden["w_W"], u, gs)
    tag = f"u{u}_gs{gs}"
    for k in ("scale_exp", "upper", "shared", "upper_cm", "shared_cm"):
        assert p[k].dtype == golden[f"w_{k}_{tag}"].dtype
        assert np.array_equal(p[k], golden[f"w_{k}_{tag}"]), k
    assert np.array_equal(orc.dequant_weight(p), golden[f"w_deq_{tag}"])
    assert np.allclose(orc.wonly_matmul(p, golden["w_X"]), golden[f"w_y_{tag}"], rtol=1e-12, atol=0)


def test_pack_kv_planes_and_attention_match_reference(golden, cfg):
    u, gs = cfg
    tag = f"u{u}_gs{gs}"
    pK, pV = orc.pack_kv(golden["kv_K"], u, gs), orc.pack_kv(golden["kv_V"], u, gs)
    for k in ("scale_exp", "upper", "shared"):
        assert np.array_equal(pK[k], golden[f"kv_K{k}_{tag}"]), k
        assert np.array_equal(pV[k], golden[f"kv_V{k}_{tag}"]), k
    Q = golden["kv_Q"]
    assert np.allclose(orc.kv_attention(Q, pK, pV, causal=True), golden[f"kv_prefill_{tag}"],
                       rtol=1e-10, atol=1e-12)
    dec = orc.kv_attention(Q[:, -1:, :], pK, pV, causal=True)[:, 0]
    assert np.allclose(dec, golden[f"kv_decode_{tag}"], rtol=1e-10, atol=1e-12)
    # the plane-level decode entry used by the GPU parity tests gives the same numbers
    dec2 = orc.decode_attention_planes(Q[:, -1, :], (pK["scale_exp"], pK["upper"], pK["shared"]),
                                       (pV["scale_exp"], pV["upper"], pV["shared"]), u, gs, Q.shape[1])
    assert np.allclose(dec2, golden[f"kv_decode_{tag}"], rtol=1e-10, atol=1e-12)


def test_rotation_matches_kernel_formula_and_reference_packing(golden):
    K = golden["rot_K"]
    rot = orc.rotate_f32(K)
    assert rot.dtype == np.float32
    assert np.array_equal(rot, golden["rot_f32"])            # bit-exact fp32 butterfly
    # the reference's host formulation (matrix product) agrees to fp32 rounding
    assert orc.rel_fro(rot, golden["rot_host"]) < 1e-6
    assert orc.rel_fro(K.astype(np.float64) @ orc.hadamard_matrix(128), golden["rot_host"]) < 1e-6
    for u, gs in ((4, 2), (3, 8), (2, 4)):
        p = orc.pack_kv_rotated(K, u, gs)
        for k in ("scale_exp", "upper", "shared"):
            assert np.array_equal(p[k], golden[f"rot_{k}_u{u}_gs{gs}"]), (u, gs, k)


def test_bit_pack_round_trip(rng):
    for width in (2, 3, 4, 5, 6):
        lo, hi = -(1 << (width - 1)), (1 << (width - 1)) - 1
        for n in (1, 2, 4, 8, 16, 32):
            codes = rng.integers(lo, hi + 1, size=(7, 3, n))
            buf = orc.pack_bits_lsb(codes, width)
            assert buf.shape[-1] == -(-n * width // 8)
            assert np.array_equal(orc.unpack_bits_lsb(buf, n, width), codes)


def test_round_trip_and_bounds(rng, cfg):
    u, gs = cfg
    x = rng.standard_normal((512, 32)) * rng.uniform(0.1, 8.0, (512, 1))
    exp, up, sh = orc.decompose(x, u, gs)
    lim = (1 << (7 - u)) - 1
    assert np.abs(up).max() <= lim and sh.min() >= -(1 << (u - 1)) and sh.max() <= (1 << (u - 1)) - 1
    W = (rng.standard_normal((64, 128)) * 0.02).astype(np.float32)
    p = orc.pack_weight(W, u, gs)
    gold = orc.quantize_dequantize(W.reshape(-1, 32), u, gs).reshape(64, 128)
    assert np.array_equal(orc.dequant_weight(p), gold)


def test_to_bf16_matches_torch(rng):
    import torch
    x = (rng.standard_normal(4096) * rng.uniform(1e-3, 1e3, 4096)).astype(np.float32)
    ref = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(orc.to_bf16(x), ref)


def test_rope_matches_reference_harness(golden):
    """The harness's rope_bthd on its own tables, bit for bit; the table formula to float32 rounding."""
    x, y = golden["rope_x"], golden["rope_y"]                      # [B, L, H, D]
    cos, sin = golden["rope_cos"], golden["rope_sin"]              # [L, D/2]
    got = orc.rope(x, cos[None, :, None, :], sin[None, :, None, :])
    assert np.array_equal(got, y)
    got1 = orc.rope(golden["rope_x1"], golden["rope_cos_8191"][None, :, None, :],
                    golden["rope_sin_8191"][None, :, None, :])
    assert np.array_equal(got1, golden["rope_y1"])
    c, s = orc.rope_tables(np.arange(cos.shape[0]), 2 * cos.shape[1])
    assert np.abs(c - cos).max() < 1e-5 and np.abs(s - sin).max() < 1e-5
    # at an angle of ~8191 rad the last bit of the float32 product pos * inv already moves the cosine
    c1, s1 = orc.rope_tables(np.array([8191]), 2 * cos.shape[1])
    assert np.abs(c1 - golden["rope_cos_8191"]).max() < 2e-3
    # rope -> rotation -> pack equals the reference's pack_kv of the same chain
    k = np.ascontiguousarray(y[0].transpose(1, 0, 2))              # [H, L, D]
    for u, gs in ((4, 2), (3, 8), (2, 4)):
        p = orc.pack_kv_rotated(k, u, gs)
        for key in ("scale_exp", "upper", "shared"):
            assert np.array_equal(p[key], golden[f"ropek_{key}_u{u}_gs{gs}"]), (u, gs, key)


def test_mxint8_matches_reference(golden):
    """The plain-MXINT8 baseline format: planes, dequantisation, matmul and attention of the reference."""
    p = orc.pack_weight_mxint8(golden["mx_W"])
    for k in ("scale_exp", "qweight", "qweight_cm"):
        assert p[k].dtype == golden[f"mx_w_{k}"].dtype and np.array_equal(p[k], golden[f"mx_w_{k}"]), k
    assert np.array_equal(orc.dequant_weight_mxint8(p), golden["mx_w_deq"])
    assert np.allclose(orc.wonly_matmul_mxint8(p, golden["mx_X"]), golden["mx_w_y"], rtol=1e-12, atol=0)
    pK, pV = orc.pack_kv_mxint8(golden["kv_K"]), orc.pack_kv_mxint8(golden["kv_V"])
    for k in ("scale_exp", "qweight"):
        assert np.array_equal(pK[k], golden[f"mx_kv_K{k}"]) and np.array_equal(pV[k], golden[f"mx_kv_V{k}"]), k
    Q = golden["kv_Q"]
    dec = orc.decode_attention_planes_mxint8(Q[:, -1, :], (pK["scale_exp"], pK["qweight"]), (pV["scale_exp"], pV["qweight"]),
                                             Q.shape[1])
    assert np.allclose(dec, golden["mx_kv_decode"], rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("u", (2, 3, 4))
@pytest.mark.parametrize("gs", (2, 8))
def test_w_plus_a_matches_reference(golden, u, gs):
    """Run-time activation quantisation (MSAQ-signed words) and the W+A integer-dot product of the reference."""
    tag = f"u{u}_gs{gs}"
    q, e = orc.quant_act(golden["wa_X"], u, gs)
    assert np.array_equal(q, golden[f"wa_q_{tag}"]) and np.array_equal(e, golden[f"wa_exp_{tag}"])
    y = orc.wa_matmul(orc.pack_weight(golden["w_W"], u, gs), golden["wa_X"])
    assert np.allclose(y, golden[f"wa_y_{tag}"], rtol=1e-12, atol=0)

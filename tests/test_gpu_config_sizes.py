"""GPU parity at the full sizes of the benchmark configurations.

The float64 oracle cannot dequantise a 57344 x 8192 weight or a 2.5 GB cache in seconds, so these tests
use what the packed format guarantees: every output row of a weight and every (sequence, kv head) of a
cache is packed independently (ms_lib/pack.py:112-121, :493-496), so a SAMPLE of rows / sequences pulled
from the device planes is itself a valid packed tensor the oracle can dequantise.  The kernels run on
the whole problem; the oracle checks the sampled part of the output at the usual tolerance.

Shapes follow the reference's own gates (tests/test_w.py:53-80, tests/test_kv.py:45-121,
tests/rot_fused_bench.py:42-87) at the sizes the benchmark configurations name.
"""

import numpy as np
import pytest
import torch

from conftest import F32_REL_FRO_TOL, MAX_ABS_REL_TOL, REL_FRO_TOL
from oracle import msaq_oracle as orc

pytestmark = pytest.mark.gpu
N_SAMPLE_ROWS = 256

# fp32 output (before the bf16 rounding) of the flash-decode on caches whose keys carry x20 outlier
# channels: scores reach magnitude ~50 and the 16-bit block fixed point of the query staging shows at
# this level; the bf16 output is held to the ordinary bar.
F32_TOL_OUTLIER_KEYS = 3e-4
# fp32 output of the flash-decode over thousands of keys with scores of spread ~1: each output channel is
# an average of >= 2k nearly equally weighted values, about sqrt(Lk) smaller than one value, so the
# 16-bit fixed point of the probabilities (2^-17 of a chunk's maximum per key) shows at this level
# relative to the output.  The bf16 output is held to the ordinary bar.
F32_TOL_LONG_UNIFORM = 3e-4


def _rows_pack(pd, idx, u, gs):
    """The packed rows `idx` of a device pack dict as an oracle pack dict (NumPy)."""
    it = torch.from_numpy(idx).cuda()
    se = pd["scale_exp"].index_select(1, it).cpu().numpy()
    up = pd["upper_cm"].index_select(1, it).cpu().numpy()          # [nb, rows, UB]
    sh = pd["shared_cm"].index_select(1, it).cpu().numpy()
    nb = se.shape[0]
    return dict(scale_exp=se, upper=np.ascontiguousarray(up.transpose(0, 2, 1)),
                shared=np.ascontiguousarray(sh.transpose(0, 2, 1)), OUT=len(idx), K=nb * 32, nb=nb, u=u, gs=gs,
                n_group=32 // gs)


def _gemv_sampled(OUT, K, u, Ms, seed):
    import cabi
    gs = 2
    g = torch.Generator(device="cuda").manual_seed(seed)
    W = (torch.randn((OUT, K), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    pd = cabi.pack_weight(W, u, gs)
    del W
    rng = np.random.default_rng(seed)
    idx = np.sort(rng.choice(OUT, size=min(N_SAMPLE_ROWS, OUT), replace=False))
    # rows at the edges of tiles and of the matrix are the ones a scheduling slip would hit
    idx[:4] = (0, 1, OUT // 2, OUT - 1)
    idx = np.unique(idx)
    Wdq = orc.dequant_weight(_rows_pack(pd, idx, u, gs))                     # float64 [rows, K]
    for M in Ms:
        X = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
        if M == 1:
            got, gotf = cabi.gemv("wide", X[0].contiguous(), pd)
            got, gotf = got[None], gotf[None]
        else:
            got, gotf = cabi.gemv("batched", X, pd, M=M)
        ref = X.float().cpu().numpy().astype(np.float64) @ Wdq.T             # [M, rows]
        cabi.check_output(got[:, idx], gotf[:, idx], ref, MAX_ABS_REL_TOL, REL_FRO_TOL, F32_REL_FRO_TOL)
        assert np.isfinite(gotf).all()


LLAMA8B = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]


@pytest.mark.parametrize("u", (4, 3, 2))
@pytest.mark.parametrize("name,OUT,K", LLAMA8B, ids=[s[0] for s in LLAMA8B])
def test_gemv_llama8b_shapes_all_batch_sizes(name, OUT, K, u):
    """Every Llama-3.1-8B projection shape x u in {2,3,4} (gs=2) x M in {1,4,16,64}."""
    _gemv_sampled(OUT, K, u, (1, 4, 16, 64), seed=OUT // 64 + K // 32 + u)


@pytest.mark.parametrize("OUT,K", [(4096, 4096), (4096, 14336), (6144, 4096)])
def test_gemv_two_pass_launches_with_several_k_blocks_per_stage(OUT, K):
    """Five to eight rows on 4096-row shapes run the two-pass kernel with four K blocks per ring stage."""
    _gemv_sampled(OUT, K, 4, (5, 8, 2, 3), seed=OUT + K)


LLAMA70B = [("qkv", 10240, 8192), ("o", 8192, 8192), ("gate_up", 57344, 8192), ("down", 8192, 28672)]


@pytest.mark.parametrize("name,OUT,K", LLAMA70B, ids=[s[0] for s in LLAMA70B])
def test_gemv_llama70b_layer_shapes(name, OUT, K):
    """The four matrices of the Llama-3.1-70B-shaped layer the benchmark times, at its batch sizes."""
    _gemv_sampled(OUT, K, 4, (1, 8, 32), seed=OUT // 128 + K // 64)


@pytest.mark.parametrize("world", (2, 8))
def test_gemv_llama70b_tensor_parallel_shards(world):
    """The per-rank shapes of the same layer at TP = 2 and 8 (narrow gate+up, short-K O and down)."""
    from ms_kernel_b200 import tp
    for name, (OUT, K) in tp.LayerShape.llama31_70b().weight_shapes_local(world).items():
        _gemv_sampled(OUT, K, 4, (1, 8), seed=OUT + K + world)


# --------------------------------------------------------------------------------------------------
# flash-decode
# --------------------------------------------------------------------------------------------------
OUTLIER_CHANNELS = [3, 40, 77, 120]


def _planes_np(planes, sel):
    return tuple(t[sel].cpu().numpy() for t in planes)


@pytest.mark.parametrize("H,Lk", [(8, 4096), (8, 16384), (16, 4096), (16, 16384)])
def test_decode_mha_rotated_cache_with_outlier_channels(H, Lk):
    """MHA decode, B=1, D=128: K with four persistent outlier channels x20, cache written with the
    Hadamard rotation (prefill write, then the last 48 tokens one kv_append_rot / kv_append each),
    query rotated in the kernel prologue, u4/gs2 -- against the oracle on the device-built planes."""
    import cabi
    u, gs, D, tail = 4, 2, 128, 48
    Lcap = Lk + 16
    g = torch.Generator(device="cuda").manual_seed(H + Lk)
    K = torch.randn((H, Lk, D), generator=g, device="cuda")
    K[..., OUTLIER_CHANNELS] *= 20
    K = K.to(torch.bfloat16)
    V = torch.randn((H, Lk, D), generator=g, device="cuda").to(torch.bfloat16)
    q = torch.randn((1, H, D), generator=g, device="cuda").to(torch.bfloat16)
    kp = cabi.empty_cache(H, D // 32, Lcap, u, gs, fill=0x6B)
    vp = cabi.empty_cache(H, D // 32, Lcap, u, gs, fill=0x6B)
    cabi.kv_write(K[:, :Lk - tail].contiguous(), kp, H, Lk - tail, D, 0, Lcap, u, gs, rot=True)
    cabi.kv_write(V[:, :Lk - tail].contiguous(), vp, H, Lk - tail, D, 0, Lcap, u, gs)
    for pos in range(Lk - tail, Lk):
        cabi.kv_append(K[:, pos].contiguous(), kp, H, D, pos, Lcap, u, gs, rot=True)
        cabi.kv_append(V[:, pos].contiguous(), vp, H, D, pos, Lcap, u, gs)
    got, gotf = cabi.decode(q, kp, vp, 1, H, H, Lk, D, u, gs, Lcap=Lcap, qrot=1)
    ref = orc.decode_attention_batched(q.float().cpu().numpy(), tuple(t.cpu().numpy()[None] for t in kp),
                                       tuple(t.cpu().numpy()[None] for t in vp), u, gs, [Lk], qrot=True)
    cabi.check_output(got, gotf, ref, MAX_ABS_REL_TOL, REL_FRO_TOL, F32_TOL_OUTLIER_KEYS)
    # the appended tokens' bytes are those of the oracle's rotate-and-pack of the same rows
    tok = orc.pack_kv_rotated(K[:, Lk - tail:].float().cpu().numpy(), u, gs)
    assert np.array_equal(kp[1][:, :, Lk - tail:Lk].cpu().numpy(), tok["upper"])
    assert np.array_equal(kp[2][:, :, Lk - tail:Lk].cpu().numpy(), tok["shared"])
    assert np.array_equal(kp[0][:, :, Lk - tail:Lk].cpu().numpy(), tok["scale_exp"])


@pytest.mark.parametrize("B,Lk", [(8, 4096), (16, 16384), (64, 4096), (16, 32768), (64, 32768)])
def test_decode_gqa_batched_varlen_full_size(B, Lk):
    """GQA 32/8, D=128, per-sequence lengths uniform in [Lk/2, Lk], one appended token per sequence and
    step, u4/gs2 with rotated keys: the whole batch runs on the device, the oracle checks three sampled
    sequences (the longest, the shortest, one other) from the device-built planes."""
    import cabi
    u, gs, Hq, Hkv, D = 4, 2, 32, 8, 128
    Lcap = Lk + 16
    rng = np.random.default_rng(B * 7 + Lk)
    lens = rng.integers(Lk // 2, Lk + 1, size=B).astype(np.int32)
    lens[0] = Lk
    g = torch.Generator(device="cuda").manual_seed(B + Lk)
    kp = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs)
    vp = cabi.empty_cache(B * Hkv, D // 32, Lcap, u, gs)
    chunk = 2048
    for k0 in range(0, Lk, chunk):
        Kt = torch.randn((B * Hkv, chunk, D), generator=g, device="cuda").to(torch.bfloat16)
        Vt = torch.randn((B * Hkv, chunk, D), generator=g, device="cuda").to(torch.bfloat16)
        cabi.kv_write(Kt, kp, B * Hkv, chunk, D, k0, Lcap, u, gs, rot=True)
        cabi.kv_write(Vt, vp, B * Hkv, chunk, D, k0, Lcap, u, gs)
        del Kt, Vt
    # the step's new token goes to slot len-1 of every sequence
    kn = torch.randn((B * Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    vn = torch.randn((B * Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    pos = cabi.dev(lens - 1)
    cabi.kv_append_varlen(kn, kp, B, Hkv, D, pos, Lcap, u, gs, rot=True)
    cabi.kv_append_varlen(vn, vp, B, Hkv, D, pos, Lcap, u, gs)
    q = torch.randn((B, Hq, D), generator=g, device="cuda").to(torch.bfloat16)
    got, gotf = cabi.decode(q, kp, vp, B, Hq, Hkv, Lk, D, u, gs, Lcap=Lcap, qrot=1, seq_lens=cabi.dev(lens))
    assert np.isfinite(gotf).all()
    sample = sorted({0, int(np.argmin(lens)), B // 2})
    qn = q.float().cpu().numpy()
    for b in sample:
        sel = slice(b * Hkv, (b + 1) * Hkv)
        ref = orc.decode_attention_planes(qn[b], _planes_np(kp, sel), _planes_np(vp, sel), u, gs, int(lens[b]),
                                          qrot=True)
        cabi.check_output(got[b], gotf[b], ref, MAX_ABS_REL_TOL, REL_FRO_TOL, F32_TOL_LONG_UNIFORM)


@pytest.mark.parametrize("Hq,Hkv", [(4, 4), (16, 2)])
@pytest.mark.parametrize("sink_pos", (0, 20000))
def test_decode_attention_sink_long_tail(Hq, Hkv, sink_pos):
    """One key about 12 nats above 32k near-uniform keys, values with a non-zero mean and a small value at
    the sink: a fifth of the softmax mass sits in a tail whose single probabilities are ~6e-6 of the
    maximum.  Probabilities quantised relative to the running maximum would drop that tail."""
    import cabi
    u, gs, D, Lk = 4, 2, 128, 32768
    G = Hq // Hkv
    rng = np.random.default_rng(Hq + sink_pos)
    qk = rng.standard_normal((Hkv, D)).astype(np.float32)
    q = np.repeat(qk, G, axis=0) + 0.01 * rng.standard_normal((Hq, D)).astype(np.float32)   # heads of a group nearly agree
    q = orc.to_bf16(q)
    K = (rng.standard_normal((Hkv, Lk, D)) * 0.05).astype(np.float32)
    for hk in range(Hkv):
        s = 12.0 * np.sqrt(D) / float(qk[hk] @ qk[hk])                 # q.k / sqrt(D) = 12 nats
        K[hk, sink_pos] = s * qk[hk]
    V = (rng.standard_normal((Hkv, Lk, D)) + 0.5).astype(np.float32)
    V[:, sink_pos] *= 0.01
    kp = cabi.empty_cache(Hkv, D // 32, Lk, u, gs)
    vp = cabi.empty_cache(Hkv, D // 32, Lk, u, gs)
    cabi.kv_write(cabi.bf16_dev(K), kp, Hkv, Lk, D, 0, Lk, u, gs)
    cabi.kv_write(cabi.bf16_dev(V), vp, Hkv, Lk, D, 0, Lk, u, gs)
    got, gotf = cabi.decode(cabi.bf16_dev(q[None]), kp, vp, 1, Hq, Hkv, Lk, D, u, gs)
    ref = orc.decode_attention_planes(q, tuple(t.cpu().numpy() for t in kp), tuple(t.cpu().numpy() for t in vp),
                                      u, gs, Lk)
    cabi.check_output(got[0], gotf[0], ref, MAX_ABS_REL_TOL, REL_FRO_TOL, F32_TOL_LONG_UNIFORM)

"""GPU parity of the decoder-layer step (tests/harness_batchsweep.py:230-243 of the
reference wires the same ops): the fused-prologue GEMV against the separate ops it
replaces, and the whole step on packed weights and a packed cache against a float64
restatement built on the CPU oracle."""

import numpy as np
import pytest
import torch

from conftest import REL_FRO_TOL
from oracle import msaq_oracle as orc

pytestmark = pytest.mark.gpu


def _bf(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).cuda()


@pytest.mark.parametrize("u,gs", [(4, 2), (3, 4)], ids=["tuned_u4gs2", "generic_u3gs4"])
@pytest.mark.parametrize("M", [1, 3, 17])
def test_fused_prologues_match_separate_ops(rng, u, gs, M):
    from ms_kernel_b200 import ops
    OUT, K = 384, 1024
    W = (rng.standard_normal((OUT, K)) * 0.05).astype(np.float32)
    lin = ops.PackedLinear(orc.pack_weight(W, u, gs), "cuda")
    h = _bf(rng.standard_normal((M, K)) * 2)
    delta32 = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda()
    gu = _bf(rng.standard_normal((M, 2 * K)) * 2)
    msaq = torch.ops.msaq

    # SiLU * mul: same expression element by element, so the same bits -- as long as both run the same
    # GEMV kernel (with 9 rows and more the unfused u4/gs2 call takes the tensor-memory path)
    want = lin.fwd(msaq.silu_mul(gu))
    got = lin.fwd_fused(gu, ops.PRO_SILU_MUL)
    if M < 9 or (u, gs) != (4, 2):
        assert torch.equal(got.reshape(want.shape), want)
    else:
        assert orc.rel_fro(got.float().cpu().numpy(), want.float().cpu().numpy()) < REL_FRO_TOL

    # rmsnorm: the sum of squares is taken in another order, so a normalised element may round the other way
    want = lin.fwd(msaq.rmsnorm(h, 1e-5)).float().cpu().numpy()
    got = lin.fwd_fused(h, ops.PRO_RMSNORM, None, 1e-5).float().cpu().numpy()
    assert orc.rel_fro(got, want) < REL_FRO_TOL

    # residual add + rmsnorm, fp32 and bf16 addend: the new residual stream is bit-exact
    for delta in (delta32, delta32.to(torch.bfloat16)):
        hn = msaq.add_residual(h, delta)
        want = lin.fwd(msaq.rmsnorm(hn, 1e-5)).float().cpu().numpy()
        got, hn2 = lin.fwd_fused(h, ops.PRO_ADD_RMSNORM, delta, 1e-5)
        assert torch.equal(hn2, hn)
        assert orc.rel_fro(got.float().cpu().numpy(), want) < REL_FRO_TOL

    # against float64 formulas
    hf = h.float().cpu().numpy().astype(np.float64)
    x = orc.to_bf16((hf / np.sqrt((hf ** 2).mean(-1, keepdims=True) + 1e-5)).astype(np.float32))
    ref = x.astype(np.float64) @ orc.dequant_weight(orc.pack_weight(W, u, gs)).T.astype(np.float64)
    got = lin.fwd_fused(h, ops.PRO_RMSNORM, None, 1e-5).float().cpu().numpy()
    assert orc.rel_fro(got, orc.to_bf16(ref.astype(np.float32))) < 2 * REL_FRO_TOL


def test_fused_prologue_argument_errors(rng):
    from ms_kernel_b200 import ops
    lin = ops.PackedLinear(orc.pack_weight((rng.standard_normal((64, 64)) * 0.05).astype(np.float32), 4, 2), "cuda")
    h = _bf(rng.standard_normal((2, 64)))
    with pytest.raises(RuntimeError):
        lin.fwd_fused(h, ops.PRO_ADD_RMSNORM, None)               # no addend
    with pytest.raises(RuntimeError):
        lin.fwd_fused(h, 9)                                       # unknown prologue
    with pytest.raises(RuntimeError):
        lin.fwd_fused(h, ops.PRO_SILU_MUL)                        # needs [M, 2K]


class _F64Linear:
    def __init__(self, p):
        self.W = orc.dequant_weight(p).astype(np.float64)

    def fwd(self, x):
        return torch.from_numpy(orc.to_bf16((x.double().numpy() @ self.W.T).astype(np.float32))).to(torch.bfloat16)


class _F64Cache:
    """Dequantised packed cache; K is kept rotated and the query is rotated to match, as the kernels do."""

    def __init__(self, K, V, u, gs, L):
        self.u, self.gs = u, gs
        B, kv, _, D = K.shape
        self.K = np.zeros((B, kv, L, D))
        self.V = np.zeros((B, kv, L, D))
        for b in range(B):
            self.K[b, :, : K.shape[2]] = orc.dequant_kv(orc.pack_kv_rotated(K[b], u, gs))
            self.V[b, :, : V.shape[2]] = orc.dequant_kv(orc.pack_kv(V[b], u, gs))

    def append(self, k, v, pos, rope=None):
        k, v = k.float().numpy(), v.float().numpy()
        if rope is not None:
            k = orc.rope(k, rope[0].cpu().numpy()[0], rope[1].cpu().numpy()[0])
        for b in range(k.shape[0]):
            self.K[b, :, pos] = orc.dequant_kv(orc.pack_kv_rotated(k[b][:, None, :], self.u, self.gs))[:, 0]
            self.V[b, :, pos] = orc.dequant_kv(orc.pack_kv(v[b][:, None, :], self.u, self.gs))[:, 0]

    def attend(self, q, Lk, seq_lens=None, rope=None, q_pos=None):
        qn = q.float().numpy()
        if rope is not None:
            qn = orc.rope(qn, rope[0].cpu().numpy()[0], rope[1].cpu().numpy()[0])
        out = []
        for b in range(qn.shape[0]):
            qr = orc.rotate_f32(qn[b]).astype(np.float64)
            out.append(orc.decode_attention(qr, self.K[b, :, :Lk], self.V[b, :, :Lk]))
        return torch.from_numpy(orc.to_bf16(np.stack(out).astype(np.float32))).to(torch.bfloat16)


class _F64Glue:
    """The element-wise steps in float64 with the bf16 roundings of the layer's intermediates."""

    @staticmethod
    def _bf(a):
        return torch.from_numpy(orc.to_bf16(np.asarray(a, np.float32))).to(torch.bfloat16)

    def rmsnorm(self, x, eps):
        xf = x.double().numpy()
        return self._bf(xf / np.sqrt((xf ** 2).mean(-1, keepdims=True) + eps))

    def add(self, h, delta):
        return self._bf(h.double().numpy() + delta.double().numpy())

    def silu_mul(self, gu):
        g = gu.double().numpy()
        F = g.shape[1] // 2
        return self._bf(g[:, :F] / (1.0 + np.exp(-g[:, :F])) * g[:, F:])


@pytest.mark.parametrize("with_rope", [False, True], ids=["no_rope", "rope"])
@pytest.mark.parametrize("B", [1, 3])
def test_layer_step_matches_float64_restatement(rng, B, with_rope):
    """One decode step of a small Llama-shaped layer: packed GEMVs, RoPE on q and k, rotated append,
    flash-decode, fused glue -- against the same step in float64 on the dequantised tensors (the wiring of
    the reference's decode_step, tests/harness_batchsweep.py:230-243)."""
    from ms_kernel_b200 import ops, tp
    u, gs = 4, 2
    shape = tp.LayerShape(hidden=512, n_q=8, n_kv=2, head_dim=128, ffn=1024)
    d, L, Lcap = shape.head_dim, 333, 336
    dims = {"q": (shape.n_q * d, shape.hidden), "k": (shape.n_kv * d, shape.hidden), "v": (shape.n_kv * d, shape.hidden),
            "o": (shape.hidden, shape.n_q * d), "gate": (shape.ffn, shape.hidden), "up": (shape.ffn, shape.hidden),
            "down": (shape.hidden, shape.ffn)}
    P = {k: orc.pack_weight(orc.to_bf16((rng.standard_normal(s) * 0.04).astype(np.float32)), u, gs)
         for k, s in dims.items()}
    sh = tp.shard_layer(P, shape, 1, 0)
    K0 = orc.to_bf16(rng.standard_normal((B, shape.n_kv, L - 1, d)).astype(np.float32))
    V0 = orc.to_bf16(rng.standard_normal((B, shape.n_kv, L - 1, d)).astype(np.float32))
    h = orc.to_bf16(rng.standard_normal((B, shape.hidden)).astype(np.float32))

    cache = ops.KVCache(B, shape.n_kv, d, Lcap, u, gs, "cuda", rotate=True)
    cache.fill(_bf(K0), _bf(V0), 0)
    layer = tp.DecoderLayerTP(shape, 1, {k: ops.PackedLinear(v, "cuda") for k, v in sh.items()}, cache)
    rope_dev = rope_cpu = None
    if with_rope:
        cos, sin = orc.rope_tables(np.array([L - 1]), d)
        rope_cpu = (torch.from_numpy(cos), torch.from_numpy(sin))
        rope_dev = (rope_cpu[0].cuda(), rope_cpu[1].cuda())
    got = layer.step(_bf(h), L - 1, L, rope=rope_dev).float().cpu().numpy()

    ref_layer = tp.DecoderLayerTP(shape, 1, {k: _F64Linear(v) for k, v in sh.items()}, _F64Cache(K0, V0, u, gs, Lcap),
                                  glue=_F64Glue())
    ref = ref_layer.step(torch.from_numpy(h).to(torch.bfloat16), L - 1, L, rope=rope_cpu).float().numpy()
    # the residual stream carries h through unchanged, so compare the update the layer made
    assert orc.rel_fro(got - h, ref - h) < 2e-2
    assert orc.rel_fro(got, ref) < 4 * REL_FRO_TOL
    assert np.isfinite(got).all()


@pytest.mark.parametrize("M", [1, 5, 20])
def test_fp32_partial_outputs_round_to_the_bf16_outputs(rng, M):
    """K-sharded linears hand their fp32 result to the all-reduce: it must be the value the bf16 output rounds."""
    from ms_kernel_b200 import ops
    OUT, K = 256, 512
    lin = ops.PackedLinear(orc.pack_weight((rng.standard_normal((OUT, K)) * 0.05).astype(np.float32), 4, 2), "cuda")
    x = _bf(rng.standard_normal((M, K)))
    y32 = lin.fwd_f32(x)
    assert y32.dtype == torch.float32 and tuple(y32.shape) == (M, OUT)
    assert torch.equal(y32.to(torch.bfloat16), lin.fwd(x).reshape(M, OUT))
    gu = _bf(rng.standard_normal((M, 2 * K)))
    f32 = lin.fwd_fused(gu, ops.PRO_SILU_MUL, out_f32=True)
    assert f32.dtype == torch.float32
    assert torch.equal(f32.to(torch.bfloat16), lin.fwd_fused(gu, ops.PRO_SILU_MUL))

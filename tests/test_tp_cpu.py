"""Tensor-parallel host logic on CPU: shard arithmetic is bit-identical to packing the
slice directly, and a 2-rank gloo run of the layer step equals the single-rank step.
The CPU oracle stands in for the kernels here (it is the checker, not the product)."""

import os
import socket

import numpy as np
import pytest
import torch

from ms_kernel_b200 import tp
from oracle import msaq_oracle as orc

U, GS = 4, 2
SHAPE = tp.LayerShape(hidden=256, n_q=4, n_kv=2, head_dim=64, ffn=512)


def _weights(rng, SHAPE=SHAPE):
    d = SHAPE.head_dim
    dims = {"q": (SHAPE.n_q * d, SHAPE.hidden), "k": (SHAPE.n_kv * d, SHAPE.hidden), "v": (SHAPE.n_kv * d, SHAPE.hidden),
            "o": (SHAPE.hidden, SHAPE.n_q * d), "gate": (SHAPE.ffn, SHAPE.hidden), "up": (SHAPE.ffn, SHAPE.hidden),
            "down": (SHAPE.hidden, SHAPE.ffn)}
    W = {k: orc.to_bf16((rng.standard_normal(s) * 0.05).astype(np.float32)) for k, s in dims.items()}
    return W, {k: orc.pack_weight(v, U, GS) for k, v in W.items()}


def test_shards_are_bit_identical_to_packing_the_slice(rng):
    W, P = _weights(rng)
    for world in (1, 2):
        for rank in range(world):
            sh = tp.shard_layer(P, SHAPE, world, rank)
            q, kv, f = SHAPE.local(world)
            d = SHAPE.head_dim
            rows = np.concatenate([W["q"][rank * q * d:(rank + 1) * q * d], W["k"][rank * kv * d:(rank + 1) * kv * d],
                                   W["v"][rank * kv * d:(rank + 1) * kv * d]])
            direct = {"qkv": orc.pack_weight(rows, U, GS),
                      "o": orc.pack_weight(W["o"][:, rank * q * d:(rank + 1) * q * d], U, GS),
                      "gate_up": orc.pack_weight(np.concatenate([W["gate"][rank * f:(rank + 1) * f],
                                                                 W["up"][rank * f:(rank + 1) * f]]), U, GS),
                      "down": orc.pack_weight(W["down"][:, rank * f:(rank + 1) * f], U, GS)}
            for name in direct:
                for k in ("scale_exp", "upper", "shared", "upper_cm", "shared_cm"):
                    assert np.array_equal(np.ascontiguousarray(sh[name][k]), direct[name][k]), (world, rank, name, k)
                assert sh[name]["OUT"] == direct[name]["OUT"] and sh[name]["nb"] == direct[name]["nb"]
    assert SHAPE.weight_shapes_local(2)["qkv"] == ((2 + 2) * 64, 256)
    with pytest.raises(ValueError):
        SHAPE.local(3)


class _OracleLinear:
    def __init__(self, p):
        self.W = torch.from_numpy(orc.dequant_weight({k: (np.ascontiguousarray(v) if isinstance(v, np.ndarray) else v)
                                                      for k, v in p.items()}))

    def fwd(self, x):
        return (x.double() @ self.W.T).to(torch.bfloat16)


class _TorchGlue:
    """Element-wise steps of the layer in plain PyTorch: the CPU stand-in for the library's CUDA glue kernels."""

    def rmsnorm(self, x, eps):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)

    def add(self, h, delta):
        return (h.float() + delta.float()).to(h.dtype)

    def silu_mul(self, gu):
        F = gu.shape[1] // 2
        return (torch.nn.functional.silu(gu[:, :F].float()) * gu[:, F:].float()).to(gu.dtype)


def _rope(x, rope):
    """x [B, heads, D] bf16 -> rotary embedding with tables (cos, sin) [1, D/2] (one position)."""
    c, s = rope[0][0].numpy(), rope[1][0].numpy()
    return torch.from_numpy(orc.rope(x.float().numpy(), c, s)).to(torch.bfloat16)


class _OracleCache:
    """Float KV cache with the layer's interface (append / attend); keys kept un-rotated,
    which is equivalent for attention since rotation preserves q.k."""

    def __init__(self, B, kv, D, L):
        self.K = torch.zeros(B, kv, L, D, dtype=torch.float64)
        self.V = torch.zeros(B, kv, L, D, dtype=torch.float64)

    def append(self, k, v, pos, rope=None):
        if rope is not None:
            k = _rope(k, rope)
        self.K[:, :, pos] = k.double()
        self.V[:, :, pos] = v.double()

    def attend(self, q, Lk, seq_lens=None, rope=None, q_pos=None):
        if rope is not None:
            q = _rope(q, rope)
        B, Hq, D = q.shape
        out = np.stack([orc.decode_attention(q[b].double().numpy(), self.K[b, :, :Lk].numpy(), self.V[b, :, :Lk].numpy())
                        for b in range(B)])
        return torch.from_numpy(out).to(torch.bfloat16)


def _run_rank(rank, world, port, seed, q, shape_args=None):
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    SHAPE = tp.LayerShape(*shape_args) if shape_args else globals()["SHAPE"]
    rng = np.random.default_rng(seed)
    W, P = _weights(rng, SHAPE)
    B, L = 2, 12
    sh = tp.shard_layer(P, SHAPE, world, rank)
    lin = {k: _OracleLinear(v) for k, v in sh.items()}
    _, kv, _ = SHAPE.local(world)
    cache = _OracleCache(B, kv, SHAPE.head_dim, L)
    full_K = torch.from_numpy(rng.standard_normal((B, SHAPE.n_kv, L, SHAPE.head_dim)))
    full_V = torch.from_numpy(rng.standard_normal((B, SHAPE.n_kv, L, SHAPE.head_dim)))
    cache.K[:] = full_K[:, rank * kv:(rank + 1) * kv]
    cache.V[:] = full_V[:, rank * kv:(rank + 1) * kv]

    def all_reduce(t):
        dist.all_reduce(t)
        return t

    layer = tp.DecoderLayerTP(SHAPE, world, lin, cache, all_reduce, glue=_TorchGlue())
    h = torch.from_numpy(rng.standard_normal((B, SHAPE.hidden)).astype(np.float32)).to(torch.bfloat16)
    cos, sin = orc.rope_tables(np.array([L - 1]), SHAPE.head_dim)
    out = layer.step(h, L - 1, L, rope=(torch.from_numpy(cos), torch.from_numpy(sin)))
    if rank == 0:
        q.put(out.float().numpy())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


class _FusedOracleLinear(_OracleLinear):
    """The fused entry points of ops.PackedLinear restated on the CPU (same argument meaning), so that the branches of
    DecoderLayerTP.step that use them -- glue fused into the GEMVs, the residual add behind the last one, the exchange
    started inside the row-parallel GEMVs -- run in the CPU suite."""
    glue = _TorchGlue()

    def _pro(self, x, prologue, addend, eps):
        h = None
        if prologue == 1:
            x = self.glue.rmsnorm(x, eps)
        elif prologue == 2:
            x = self.glue.silu_mul(x)
        elif prologue == 3:
            h = self.glue.add(x, addend)
            x = self.glue.rmsnorm(h, eps)
        return x, h

    def fwd_f32(self, x):
        return (x.double() @ self.W.T).float()

    def fwd_fused(self, x, prologue, addend=None, eps=1e-5, out_f32=False):
        x, h = self._pro(x, prologue, addend, eps)
        y = self.fwd_f32(x) if out_f32 else self.fwd(x)
        return (y, h) if prologue == 3 else y

    def fwd_fused_add(self, x, prologue, residual, eps=1e-5):
        return self.glue.add(residual, self.fwd_fused(x, prologue, None, eps))

    def can_push(self, M):
        return M <= 8


class _GlooExchange:
    """tp.PeerExchange's interface over a gloo all-reduce: push_from runs the GEMV and keeps the partial sums,
    recv completes the sum (and adds the residual)."""
    fused = True

    def __init__(self):
        self.calls = 0

    def push_from(self, lin, x, prologue=0, eps=1e-5):
        self.calls += 1
        return lin.fwd_fused(x, prologue, None, eps, True) if prologue else lin.fwd_f32(x)

    def recv(self, token, residual=None):
        import torch.distributed as dist
        dist.all_reduce(token)
        return token if residual is None else (residual.float() + token).to(residual.dtype)

    def __call__(self, t):                      # the unfused route must not be taken
        raise AssertionError("the step did not take the fused exchange")


def _run_rank_fused(rank, world, port, seed, q):
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    rng = np.random.default_rng(seed)
    W, P = _weights(rng, SHAPE)
    B, L = 2, 12
    sh = tp.shard_layer(P, SHAPE, world, rank)
    lin = {k: _FusedOracleLinear(v) for k, v in sh.items()}
    _, kv, _ = SHAPE.local(world)
    cache = _OracleCache(B, kv, SHAPE.head_dim, L)
    full_K = torch.from_numpy(rng.standard_normal((B, SHAPE.n_kv, L, SHAPE.head_dim)))
    full_V = torch.from_numpy(rng.standard_normal((B, SHAPE.n_kv, L, SHAPE.head_dim)))
    cache.K[:] = full_K[:, rank * kv:(rank + 1) * kv]
    cache.V[:] = full_V[:, rank * kv:(rank + 1) * kv]
    ex = _GlooExchange() if world > 1 else None
    layer = tp.DecoderLayerTP(SHAPE, world, lin, cache, ex, glue=_TorchGlue())
    h = torch.from_numpy(rng.standard_normal((B, SHAPE.hidden)).astype(np.float32)).to(torch.bfloat16)
    cos, sin = orc.rope_tables(np.array([L - 1]), SHAPE.head_dim)
    out = layer.step(h, L - 1, L, rope=(torch.from_numpy(cos), torch.from_numpy(sin)))
    if rank == 0:
        q.put((out.float().numpy(), ex.calls if ex else 0))
        q.close()
        q.join_thread()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def test_fused_step_and_exchange_inside_the_gemvs_match_the_plain_step():
    """One rank: glue fused into the GEMVs and the residual add behind the last one; two ranks: both exchanges
    started inside the row-parallel GEMVs (push_from / recv).  Both against the unfused single-rank step."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q0 = ctx.Queue()
    p0 = ctx.Process(target=_run_rank, args=(0, 1, 0, 123, q0, None))
    p0.start()
    plain = q0.get(timeout=120)
    p0.join(timeout=120)
    for world in (1, 2):
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_run_rank_fused, args=(r, world, port, 123, q)) for r in range(world)]
        for p in procs:
            p.start()
        got, calls = q.get(timeout=120)
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
        assert calls == (2 if world > 1 else 0)
        assert np.isfinite(got).all()
        assert orc.rel_fro(got, plain) < 2e-2


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("worlds,shape_args", [((1, 2), None), ((1, 4), (256, 8, 4, 64, 512))],
                         ids=["two_ranks", "four_ranks"])
def test_gloo_step_matches_single_rank(worlds, shape_args):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    results = []
    for world in worlds:
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_run_rank, args=(r, world, port, 123, q, shape_args)) for r in range(world)]
        for p in procs:
            p.start()
        results.append(q.get(timeout=120))
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    # the two runs differ only by where the bf16 roundings of the partial sums fall
    assert orc.rel_fro(results[1], results[0]) < 2e-2
    assert np.isfinite(results[1]).all()


def test_algorithmic_bytes_add_up():
    shape = tp.LayerShape.llama31_70b()
    one = tp.DecoderLayerTP(shape, 1, {}, None, glue=_TorchGlue()).algorithmic_bytes(1, 8192, 4, 2)
    eight = tp.DecoderLayerTP(shape, 8, {}, None, glue=_TorchGlue()).algorithmic_bytes(1, 8192, 4, 2)
    weights = (10240 * 8192 + 8192 * 8192 + 57344 * 8192 + 8192 * 28672) // 32 * 25
    assert abs(one - weights - 8 * 8192 * 200) < 2e6          # + activations
    assert abs(8 * eight - one) < 3e6                         # replicated activations only


def _run_rank_with_failure(rank, world, port, q):
    """Two steps; rank 1 fails on the host between them (raises, never joins the second step's all-reduce)."""
    import datetime
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8))
    rng = np.random.default_rng(5)
    W, P = _weights(rng)
    B, L = 1, 8
    lin = {k: _OracleLinear(v) for k, v in tp.shard_layer(P, SHAPE, world, rank).items()}
    _, kv, _ = SHAPE.local(world)
    cache = _OracleCache(B, kv, SHAPE.head_dim, L)

    def all_reduce(t):
        dist.all_reduce(t)
        return t

    layer = tp.DecoderLayerTP(SHAPE, world, lin, cache, all_reduce, glue=_TorchGlue())
    h = torch.from_numpy(rng.standard_normal((B, SHAPE.hidden)).astype(np.float32)).to(torch.bfloat16)
    h = layer.step(h, 0, 1)                       # step 1: everybody takes part
    try:
        if rank == 1:
            raise RuntimeError("injected host-side failure between two steps")
        layer.step(h, 1, 2)                       # step 2: the exchange can never complete
        q.put((rank, "completed"))
    except RuntimeError as e:
        q.put((rank, "error: " + str(e).splitlines()[0][:80]))
    q.close()
    q.join_thread()                               # flush the result before leaving
    os._exit(0)                                   # no collective teardown: a peer is gone


def test_rank_failure_surfaces_as_an_error_not_a_hang():
    """Failure detection on the host side: a rank that dies between two steps must make the survivors'
    next exchange fail within the communicator timeout instead of blocking for ever."""
    import time
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    t0 = time.time()
    procs = [ctx.Process(target=_run_rank_with_failure, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=90) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[1].startswith("error: injected")
    assert got[0].startswith("error"), got[0]     # the survivor saw an error from its exchange ...
    assert time.time() - t0 < 80                  # ... well within a bounded time

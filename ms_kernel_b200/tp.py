"""Tensor-parallel decode step of one Llama-shaped decoder layer on packed weights.

The reference has no multi-GPU code; its single-GPU wiring of a decode layer is
tests/harness_batchsweep.py:230-243 (rmsnorm -> q/k/v -> append -> attend -> o ->
residual -> rmsnorm -> gate/up -> SiLU*mul -> down -> residual).  This module
shards that step the way packed tensors shard for free: every 32-block of a
weight row and every (kv head, key) record is packed independently
(ms_lib/pack.py:112-121, :493-496), so a slice of the planes along output rows,
along K blocks, or along kv heads is itself a valid packed tensor.

  QKV, gate, up : split by output rows (rank r owns its q/kv heads and the matching
                  rows of gate and of up)            -> no exchange
  O, down       : split by K blocks (rank r owns the K range its local heads / FFN
                  rows produce)                      -> all-reduce of [B, hidden]
  KV cache      : split by kv head                   -> no exchange

One process per GPU; the two all-reduces per layer go through torch.distributed
(NCCL on GPUs, gloo in the CPU tests).
"""

import math

import numpy as np

BLOCK = 32


# --------------------------------------------------------------------------
# shard arithmetic (pure, no device needed)
# --------------------------------------------------------------------------
def split_range(total, parts, idx):
    """[lo, hi) of part `idx` when `total` items are cut into `parts` equal parts."""
    if total % parts:
        raise ValueError("%d does not divide into %d equal parts" % (total, parts))
    step = total // parts
    return idx * step, (idx + 1) * step


def shard_rows(p, lo, hi):
    """Rows [lo, hi) of a packed weight: a pack dict of the slice (views where possible).  The row-major
    planes are optional: a dict that carries only the column-major ones (what the kernels read) shards too."""
    out = dict(p)
    out["scale_exp"] = p["scale_exp"][:, lo:hi]
    if "upper" in p:
        out["upper"] = p["upper"][:, :, lo:hi]
        out["shared"] = p["shared"][:, :, lo:hi]
    out["upper_cm"] = p["upper_cm"][:, lo:hi, :]
    out["shared_cm"] = p["shared_cm"][:, lo:hi, :]
    out["OUT"] = hi - lo
    return out


def shard_kblocks(p, b_lo, b_hi):
    """K blocks [b_lo, b_hi) of a packed weight (input features b_lo*32 .. b_hi*32)."""
    out = dict(p)
    for k in ("scale_exp", "upper", "shared", "upper_cm", "shared_cm"):
        if k in p:
            out[k] = p[k][b_lo:b_hi]
    out["nb"] = b_hi - b_lo
    out["K"] = (b_hi - b_lo) * BLOCK
    return out


def concat_rows(parts):
    """Stack row shards of one weight back into a single pack dict (used for [q;k;v] and [gate;up])."""
    cat = np.concatenate if isinstance(parts[0]["scale_exp"], np.ndarray) else None
    if cat is None:
        import torch
        cat = torch.cat
        kw = lambda a: dict(dim=a)
    else:
        kw = lambda a: dict(axis=a)
    out = dict(parts[0])
    out["scale_exp"] = cat([q["scale_exp"] for q in parts], **kw(1))
    if "upper" in parts[0]:
        out["upper"] = cat([q["upper"] for q in parts], **kw(2))
        out["shared"] = cat([q["shared"] for q in parts], **kw(2))
    out["upper_cm"] = cat([q["upper_cm"] for q in parts], **kw(1))
    out["shared_cm"] = cat([q["shared_cm"] for q in parts], **kw(1))
    out["OUT"] = sum(int(q["OUT"]) for q in parts)
    return out


class LayerShape:
    """Sizes of one decoder layer."""

    def __init__(self, hidden, n_q, n_kv, head_dim, ffn):
        self.hidden, self.n_q, self.n_kv, self.head_dim, self.ffn = hidden, n_q, n_kv, head_dim, ffn

    @staticmethod
    def llama31_70b():
        return LayerShape(8192, 64, 8, 128, 28672)

    @staticmethod
    def llama31_8b():
        return LayerShape(4096, 32, 8, 128, 14336)

    def local(self, world):
        """(q heads, kv heads, ffn rows) owned by one rank."""
        if self.n_kv % world or self.n_q % world or self.ffn % world:
            raise ValueError("layer does not divide over %d ranks" % world)
        return self.n_q // world, self.n_kv // world, self.ffn // world

    def weight_shapes_local(self, world):
        """{name: (OUT, K)} of the four packed matrices one rank holds."""
        q, kv, f = self.local(world)
        d = self.head_dim
        return {
            "qkv": ((q + 2 * kv) * d, self.hidden),
            "o": (self.hidden, q * d),
            "gate_up": (2 * f, self.hidden),
            "down": (self.hidden, f),
        }


def shard_layer(packs, shape, world, rank):
    """Cut full packed weights {'q','k','v','o','gate','up','down'} into the four local
    matrices of `rank`: qkv = [q_r; k_r; v_r], o = K-slice, gate_up = [gate_r; up_r], down = K-slice."""
    q, kv, f = shape.local(world)
    d = shape.head_dim
    qr = shard_rows(packs["q"], rank * q * d, (rank + 1) * q * d)
    kr = shard_rows(packs["k"], rank * kv * d, (rank + 1) * kv * d)
    vr = shard_rows(packs["v"], rank * kv * d, (rank + 1) * kv * d)
    gr = shard_rows(packs["gate"], rank * f, (rank + 1) * f)
    ur = shard_rows(packs["up"], rank * f, (rank + 1) * f)
    return {
        "qkv": concat_rows([qr, kr, vr]),
        "o": shard_kblocks(packs["o"], rank * q * d // BLOCK, (rank + 1) * q * d // BLOCK),
        "gate_up": concat_rows([gr, ur]),
        "down": shard_kblocks(packs["down"], rank * f // BLOCK, (rank + 1) * f // BLOCK),
    }


# --------------------------------------------------------------------------
# the exchange step
# --------------------------------------------------------------------------
def peer_all_reduce(group, numel, dtype, device, slots=2):
    """All-reduce for the two small [B, hidden] partial sums of a step over NVLink peer memory.

    The message is 32 KB at B = 1, so the cost is latency: NCCL's all-reduce measured 16.5 us at two
    ranks inside a CUDA graph.  torch's symmetric-memory one-shot all-reduce has every rank copy its
    partial into a buffer its peers can load from and sum all copies itself (plain peer loads, no
    multicast).  Returns a callable t -> sum over ranks (a new tensor); consecutive calls rotate over
    `slots` buffers so that a rank still reading the previous message never sees the next one.
    Raises if symmetric memory cannot be set up; the caller then keeps NCCL."""
    import torch
    import torch.distributed._symmetric_memory as symm
    name = group.group_name
    bufs = []
    for _ in range(slots):
        b = symm.empty(numel, dtype=dtype, device=device)
        symm.rendezvous(b, name)
        bufs.append(b)
    state = {"i": 0}

    def all_reduce(t):
        b = bufs[state["i"] % slots]
        state["i"] += 1
        return torch.ops.symm_mem.one_shot_all_reduce_copy(b, t.reshape(-1), "sum", name).reshape(t.shape)

    return all_reduce


class PeerExchange:
    """The same exchange on this library's own kernel (msaq_peer_exchange): every rank stores its partial
    sums straight into its slot of every peer's buffer as words that carry the exchange's sequence number
    beside the data, and every thread waits on its own words -- one kernel, no fence, no flag, and the
    residual add of the step's end inside it (`reduce_add`).  The buffers are torch symmetric memory
    (peer-mapped by its rendezvous); the kernel uses plain peer stores and local loads only.  Successive
    calls alternate between two halves of the buffer; every rank must make the same calls in the same
    order."""

    def __init__(self, group, numel, device, fused=True):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.fused = bool(fused)                # False: the layer step keeps GEMV and exchange as separate kernels
        from . import _lib, ops
        ops._require()
        self._op = torch.ops.msaq.peer_exchange
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.numel = int(numel)
        nbytes = _lib.lib().msaq_peer_exchange_bytes(self.world, self.numel)
        if nbytes == 0:
            raise ValueError("peer exchange: 2 to 8 ranks and a positive element count")
        self._buf = symm.empty(nbytes // 4, dtype=torch.float32, device=device)
        self._buf.zero_()
        torch.cuda.synchronize(device)
        hdl = symm.rendezvous(self._buf, group.group_name)
        self._ptrs = [int(p) for p in hdl.buffer_ptrs]
        dist.barrier(group)                     # every rank's flags are zero before anyone pushes
        torch.cuda.synchronize(device)
        self._calls = 0

    def _parity(self):
        p = self._calls & 1
        self._calls += 1
        return p

    def __call__(self, t):
        return self._op(t.reshape(-1), None, self._ptrs, self.rank, self._parity()).reshape(t.shape)

    def reduce_add(self, t, h):
        """bf16(h + sum over ranks of t), h bf16 of t's shape."""
        return self._op(t.reshape(-1), h.contiguous(), self._ptrs, self.rank, self._parity())

    # The exchange in two halves, the first inside the GEMV that produces the partial sums: its finishing warps
    # store them into every rank's buffer tile by tile (ops.PackedLinear.fwd_push), the second half waits and adds.
    def push_from(self, lin, x, prologue=0, eps=1e-5):
        """Runs lin's GEMV on x [M, K] with the push inside; returns the token recv() wants."""
        M = int(x.shape[0])
        if M * lin.OUT != self.numel:
            raise ValueError("this exchange was set up for %d values per rank, the GEMV makes %d" % (self.numel, M * lin.OUT))
        p = self._parity()
        lin.fwd_push(x, prologue, eps, self._ptrs, self.rank, p)
        return (p, M, lin.OUT, x)

    def recv(self, token, residual=None):
        """fp32 [M, OUT] sum over ranks of what push_from sent, or bf16(residual + sum)."""
        import torch
        p, M, OUT, like = token
        return torch.ops.msaq.peer_exchange_recv(like, None if residual is None else residual.contiguous(), self._ptrs,
                                                 self.rank, p, M, OUT)


# --------------------------------------------------------------------------
# the step
# --------------------------------------------------------------------------
class MsaqGlue:
    """The element-wise steps between the linears on this library's CUDA kernels (msaq_rmsnorm,
    msaq_add_residual, msaq_silu_mul); raises when the operator module is not built."""

    def __init__(self):
        from . import ops
        ops._require()
        import torch
        self._ops = torch.ops.msaq

    def rmsnorm(self, x, eps):
        return self._ops.rmsnorm(x.contiguous(), eps)

    def add(self, h, delta):
        return self._ops.add_residual(h.contiguous(), delta.contiguous())

    def silu_mul(self, gu):
        return self._ops.silu_mul(gu.contiguous())


class DecoderLayerTP:
    """One rank's share of a decoder layer decode step.

    linears : {'qkv','o','gate_up','down'} objects with .fwd(x[B,K]) -> [B,OUT]
    cache   : object with .append(k[B,kv,D], v[B,kv,D], pos, rope) and .attend(q[B,q,D], Lk, seq_lens, rope, q_pos)
    all_reduce : callable(tensor) summing in place over the ranks (identity when world == 1)
    glue    : object with rmsnorm(x, eps), add(h, delta), silu_mul(gu) for the element-wise steps between
              the linears; default: this library's CUDA kernels (there is no other compute path in the
              package -- the CPU tests of the host logic bring their own stand-in)
    """

    def __init__(self, shape, world, linears, cache, all_reduce=None, eps=1e-5, glue=None):
        self.shape, self.world = shape, world
        self.q_heads, self.kv_heads, self.ffn_rows = shape.local(world)
        self.lin, self.cache, self.eps = linears, cache, eps
        self.all_reduce = all_reduce if all_reduce is not None else (lambda t: t)
        self.glue = glue if glue is not None else MsaqGlue()

    def _rmsnorm(self, x, eps):
        return self.glue.rmsnorm(x, eps)

    def _add(self, h, delta):
        return self.glue.add(h, delta)

    def _silu_mul(self, gu, F):
        return self.glue.silu_mul(gu)

    def _partial(self, lin, x):
        """A K-sharded linear's contribution: fp32 when it goes into an all-reduce (straight from the
        kernel where the linear offers it), the plain bf16 result on one rank."""
        if self.world == 1:
            return lin.fwd(x)
        if hasattr(lin, "fwd_f32"):
            return lin.fwd_f32(x)
        return lin.fwd(x).float()

    def step(self, h, pos, Lk, seq_lens=None, rope=None):
        """h [B, hidden] bf16 (replicated on every rank) -> new h [B, hidden] bf16 (replicated).

        pos: slot the new token's K/V go to (int, or int32 tensor [B]); Lk: keys attended
        after the append (seq_lens[b] per sequence if given).  rope = (cos, sin) fp32 [rows, D/2]
        (tests/harness_batchsweep.py:118-131 of the reference): q and k get the rotary embedding at
        `pos` between the QKV projection and the append, as the reference's decode_step does (:237) --
        inside the append and the attention kernels, not as launches of their own.

        Linears that offer fwd_fused (ops.PackedLinear on a GPU) take the rmsnorm, the
        residual add + rmsnorm and the SiLU*mul inside their activation staging; any other
        linear gets the same steps as separate ops."""
        B = h.shape[0]
        d = self.shape.head_dim
        fused = all(hasattr(self.lin[k], "fwd_fused") for k in ("qkv", "gate_up", "down"))
        if fused:
            qkv = self.lin["qkv"].fwd_fused(h, 1, None, self.eps)      # rmsnorm inside
        else:
            qkv = self.lin["qkv"].fwd(self._rmsnorm(h, self.eps))      # [B, (q + 2kv) * d], rows local
        q = qkv[:, : self.q_heads * d].reshape(B, self.q_heads, d)
        k = qkv[:, self.q_heads * d:(self.q_heads + self.kv_heads) * d].reshape(B, self.kv_heads, d)
        v = qkv[:, (self.q_heads + self.kv_heads) * d:].reshape(B, self.kv_heads, d)
        if hasattr(self.cache, "append_attend"):
            a = self.cache.append_attend(q.contiguous(), k, v, pos, Lk, seq_lens, rope)    # the append inside the attention kernel
        elif rope is None:
            self.cache.append(k, v, pos)
            a = self.cache.attend(q.contiguous(), Lk, seq_lens)        # [B, q, d], heads local
        else:
            self.cache.append(k, v, pos, rope)
            a = self.cache.attend(q.contiguous(), Lk, seq_lens, rope, pos)
        ex = self.all_reduce
        if (fused and self.world > 1 and B <= 4 and getattr(ex, "fused", False) and hasattr(self.lin["o"], "can_push")
                and self.lin["o"].can_push(B) and self.lin["down"].can_push(B)):
            # both exchanges start inside the GEMVs that feed them: the partial sums cross NVLink tile by tile
            # (up to four rows, the GEMV's single-pass variant: measured at two GPUs 134.5 -> 133.4 us per step at
            # one row; the two-pass variant at eight rows lost 12 us with the push inside and keeps the separate kernel)
            o = ex.recv(ex.push_from(self.lin["o"], a.reshape(B, self.q_heads * d)))
            gu, h = self.lin["gate_up"].fwd_fused(h, 3, o, self.eps)   # h + o, rmsnorm inside
            return ex.recv(ex.push_from(self.lin["down"], gu, 2, self.eps), residual=h)   # SiLU(gate) * up inside
        o = self._partial(self.lin["o"], a.reshape(B, self.q_heads * d))   # partial over the local K range
        o = self.all_reduce(o) if self.world > 1 else o
        if fused:
            gu, h = self.lin["gate_up"].fwd_fused(h, 3, o, self.eps)   # h + o, rmsnorm inside
            if self.world == 1 and hasattr(self.lin["down"], "fwd_fused_add"):
                return self.lin["down"].fwd_fused_add(gu, 2, h, self.eps)      # SiLU(gate) * up in front, h + ... behind
            dn = self.lin["down"].fwd_fused(gu, 2, None, self.eps, self.world > 1)   # SiLU(gate) * up inside; fp32 partial for the all-reduce
        else:
            h = self._add(h, o)
            gu = self.lin["gate_up"].fwd(self._rmsnorm(h, self.eps))   # [B, 2 * ffn_rows]
            dn = self._partial(self.lin["down"], self._silu_mul(gu, self.ffn_rows))
        if self.world > 1 and hasattr(self.all_reduce, "reduce_add"):
            return self.all_reduce.reduce_add(dn, h)                   # exchange + residual add in one kernel
        dn = self.all_reduce(dn) if self.world > 1 else dn
        return self._add(h, dn)

    # ---- bookkeeping for the benchmark --------------------------------------
    def algorithmic_bytes(self, B, seq_lens_sum, u, gs):
        """Packed weight + cache + activation bytes one step of this rank must move."""
        ub, sb = BLOCK * (8 - u) // 8, ((BLOCK // gs) * u + 7) // 8
        per_block = ub + sb + 1
        total = 0
        for OUT, K in self.shape.weight_shapes_local(self.world).values():
            total += OUT * (K // BLOCK) * per_block + 2 * K * B + 2 * OUT * B
        nb = self.shape.head_dim // BLOCK
        total += self.kv_heads * seq_lens_sum * 2 * nb * per_block + 4 * B * self.q_heads * self.shape.head_dim
        return total

"""msaq_kv_decode_attention_append: the step's cache update done by the attention kernel itself must leave the same
bytes in the cache and return the same output as msaq_kv_append_pair_rope followed by msaq_kv_decode_attention_rope
(which the other GPU tests hold against the oracle).  Tuned path (the in-kernel append) and the configurations that
fall back to the two kernels."""

import numpy as np
import pytest
import torch

from ms_kernel_b200 import ops
from oracle import msaq_oracle as orc

pytestmark = pytest.mark.gpu


def _fill(c, B, Hkv, L, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    c.fill(torch.randn((B, Hkv, L, D), generator=g, device="cuda").to(torch.bfloat16),
           torch.randn((B, Hkv, L, D), generator=g, device="cuda").to(torch.bfloat16))


CASES = [
    # B, Hq, Hkv, D, u, gs, Lk, Lcap, varlen, rope, rotate
    (1, 8, 8, 128, 4, 2, 4096, 4112, False, True, True),        # MHA, one tile per head or a few
    (1, 64, 8, 128, 4, 2, 8192, 8208, False, True, True),       # the layer's shape (G = 8)
    (3, 32, 8, 128, 4, 2, 2048, 2064, True, True, True),        # per-sequence slots, varlen
    (2, 16, 4, 128, 4, 2, 1000, 1008, True, False, False),      # no RoPE, no rotation, ragged length
    (8, 32, 8, 128, 4, 2, 16384, 16400, True, True, True),      # large: the three-blocks-per-SM build
    (2, 8, 4, 64, 4, 2, 512, 512, False, True, True),           # head_dim 64: generic path, two kernels inside
    (2, 8, 4, 128, 3, 4, 512, 512, True, True, True),           # u = 3, gs = 4: generic path
]


@pytest.mark.parametrize("B,Hq,Hkv,D,u,gs,Lk,Lcap,varlen,rope,rotate", CASES)
def test_append_inside_attention_equals_the_two_kernels(B, Hq, Hkv, D, u, gs, Lk, Lcap, varlen, rope, rotate):
    dev = torch.device("cuda")
    a = ops.KVCache(B, Hkv, D, Lcap, u, gs, dev, rotate=rotate)
    b = ops.KVCache(B, Hkv, D, Lcap, u, gs, dev, rotate=rotate)
    _fill(a, B, Hkv, Lk, D, 11)
    _fill(b, B, Hkv, Lk, D, 11)
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn((B, Hq, D), generator=g, device="cuda").to(torch.bfloat16)
    kn = torch.randn((B, Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    vn = torch.randn((B, Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    rng = np.random.default_rng(3)
    if varlen:
        lens = rng.integers(max(1, Lk // 3), Lk + 1, size=B).astype(np.int32)
        lens[0] = Lk                                             # one sequence at full length
        pos = torch.from_numpy(lens - 1).cuda()
        seq_lens = torch.from_numpy(lens).cuda()
    else:
        pos, seq_lens = Lk - 1, None
    tables = None
    if rope:
        c, s = orc.rope_tables(np.arange(Lcap), D)
        tables = (torch.from_numpy(c).cuda(), torch.from_numpy(s).cuda())
    a.append(kn, vn, pos, tables)
    want = a.attend(q, Lk, seq_lens, tables, pos) if rope else a.attend(q, Lk, seq_lens)
    got = b.append_attend(q, kn, vn, pos, Lk, seq_lens, tables)
    torch.cuda.synchronize()
    for pa, pb in zip(a.k + a.v, b.k + b.v):
        assert torch.equal(pa, pb)                                # the cache: every byte
    assert torch.equal(got, want)
    assert int(torch.ops.msaq.wait_status(True)) == 0


def test_slot_beyond_the_attended_keys_is_still_written():
    """The token's slot may lie past the keys this step attends (a slot reserved ahead): some thread block must still
    write it -- the one that owns the last tile."""
    dev = torch.device("cuda")
    B, Hq, Hkv, D, Lk, Lcap = 2, 32, 8, 128, 1024, 4096
    a = ops.KVCache(B, Hkv, D, Lcap, 4, 2, dev, rotate=True)
    b = ops.KVCache(B, Hkv, D, Lcap, 4, 2, dev, rotate=True)
    _fill(a, B, Hkv, Lk, D, 2)
    _fill(b, B, Hkv, Lk, D, 2)
    g = torch.Generator(device="cuda").manual_seed(9)
    q = torch.randn((B, Hq, D), generator=g, device="cuda").to(torch.bfloat16)
    kn = torch.randn((B, Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    vn = torch.randn((B, Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    pos = torch.tensor([3000, 4095], dtype=torch.int32, device="cuda")
    a.append(kn, vn, pos)
    want = a.attend(q, Lk)
    got = b.append_attend(q, kn, vn, pos, Lk)
    torch.cuda.synchronize()
    for pa, pb in zip(a.k + a.v, b.k + b.v):
        assert torch.equal(pa, pb)
    assert torch.equal(got, want)


def test_bad_slot_is_reported_and_skipped():
    dev = torch.device("cuda")
    B, Hq, Hkv, D, Lk, Lcap = 2, 8, 8, 128, 256, 256
    c = ops.KVCache(B, Hkv, D, Lcap, 4, 2, dev, rotate=True)
    _fill(c, B, Hkv, Lk, D, 2)
    before = [p.clone() for p in c.k + c.v]
    q = torch.randn((B, Hq, D), device="cuda").to(torch.bfloat16)
    kn = torch.randn((B, Hkv, D), device="cuda").to(torch.bfloat16)
    assert int(torch.ops.msaq.wait_status(True)) == 0
    pos = torch.tensor([-1, 256], dtype=torch.int32, device="cuda")          # read on the device: cannot be checked by the host
    out = c.append_attend(q, kn, kn, pos, Lk)
    torch.cuda.synchronize()
    assert int(torch.ops.msaq.wait_status(True)) & 8
    for p0, p1 in zip(before, c.k + c.v):
        assert torch.equal(p0, p1)
    assert torch.isfinite(out.float()).all()
    with pytest.raises(RuntimeError):
        c.append_attend(q, kn, kn, 256, Lk)                                   # a host-side slot is checked up front

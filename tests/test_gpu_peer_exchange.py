"""msaq_peer_exchange: the tensor-parallel exchange kernel (push over peer memory, one bounded wait).

On one GPU no two kernels may wait on one another, so the single-GPU cases play the peer from the host: the
peers' slots (data words that carry the sequence number) are filled by plain tensor writes BEFORE the launch, the kernel never has to
wait, and what it pushed into the "peer's" buffer is read back afterwards.  The real two-rank run (two
processes, two GPUs) is the last test and is skipped on a one-GPU box."""

import os

import numpy as np
import pytest
import torch

from ms_kernel_b200 import _lib

pytestmark = pytest.mark.gpu


def _ops():
    from ms_kernel_b200 import ops
    ops._require()
    return torch.ops.msaq


def _bufs(world, n, dev):
    nbytes = _lib.lib().msaq_peer_exchange_bytes(world, n)
    assert nbytes == 4 * world * n * 4 + 256
    return [torch.zeros(nbytes // 4, dtype=torch.float32, device=dev) for _ in range(world)]


def _ctl(buf, world, n):
    """[seq parity 0, seq parity 1, done parity 0, done parity 1]"""
    return buf[4 * world * n:].view(torch.int32)


def _slot(buf, world, n, parity, src):
    """One source rank's slot as [n / 2, 4] int32 words: x0, seq, x1, seq."""
    o = (parity * world + src) * 2 * n
    return buf[o:o + 2 * n].view(torch.int32).view(n // 2, 4)


def _encode(x, seq):
    w = torch.empty(x.numel() // 2, 4, dtype=torch.int32)
    bits = x.view(torch.int32).view(-1, 2)
    w[:, 0], w[:, 2] = bits[:, 0], bits[:, 1]
    w[:, 1] = seq
    w[:, 3] = seq
    return w


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 2), (8, 7)])
@pytest.mark.parametrize("n", [8192, 4 * 8192 + 4])
@pytest.mark.parametrize("residual", [False, True])
def test_exchange_with_host_played_peers(world, rank, n, residual):
    dev = torch.device("cuda", 0)
    ops = _ops()
    g = torch.Generator(device="cpu").manual_seed(world * 100 + rank + n)
    h = torch.randn(n, generator=g).to(torch.bfloat16)
    bufs = _bufs(world, n, dev)
    seqs = {0: 0, 1: 0}
    for parity in (0, 1, 0, 0):
        parts = torch.randn(world, n, generator=g, dtype=torch.float32)
        seqs[parity] += 1
        seq = seqs[parity]
        mine = bufs[rank]
        for r in range(world):                               # the peers' pushes, played by the host
            if r != rank:
                _slot(mine, world, n, parity, r).copy_(_encode(parts[r], seq))
        torch.cuda.synchronize()
        out = ops.peer_exchange(parts[rank].to(dev), h.to(dev) if residual else None, [b.data_ptr() for b in bufs], rank, parity)
        torch.cuda.synchronize()
        want = parts[0].clone()
        for r in range(1, world):                            # rank order, fp32
            want += parts[r]
        if residual:
            want = (h.float() + want).to(torch.bfloat16)
            assert out.dtype == torch.bfloat16
        assert torch.equal(out.cpu(), want)
        # the sequence number moved on and the done-counter is back at rest
        c = _ctl(mine, world, n).cpu()
        assert c[parity] == seq and c[2 + parity] == 0
        # what this rank pushed: its slot in every peer's buffer, every word carrying the sequence number
        for r in range(world):
            if r != rank:
                assert torch.equal(_slot(bufs[r], world, n, parity, rank).cpu(), _encode(parts[rank], seq))
    assert ops.wait_status(True) == 0


def test_absent_peer_runs_out_and_reports():
    """The wait has a limit: with a peer that never pushes, the kernel gives up, says so and writes NaN."""
    dev = torch.device("cuda", 0)
    ops = _ops()
    L = _lib.lib()
    n = 8192
    bufs = _bufs(2, n, dev)
    x = torch.ones(n, dtype=torch.float32, device=dev)
    assert ops.wait_status(True) == 0
    old = L.msaq_get_option(3)
    L.msaq_set_option(3, 2000)
    try:
        out = ops.peer_exchange(x, None, [b.data_ptr() for b in bufs], 0, 0)
        torch.cuda.synchronize()
    finally:
        L.msaq_set_option(3, old)
    assert torch.isnan(out).all()
    assert ops.wait_status(True) & 16
    assert ops.wait_status(False) == 0
    # the context is still usable
    assert float((x + 1).sum().item()) == 2 * n


def test_argument_checks():
    dev = torch.device("cuda", 0)
    ops = _ops()
    n = 8192
    bufs = _bufs(2, n, dev)
    ptrs = [b.data_ptr() for b in bufs]
    x = torch.ones(n, dtype=torch.float32, device=dev)
    with pytest.raises(RuntimeError):
        ops.peer_exchange(x, None, ptrs, 2, 0)               # rank outside the world
    with pytest.raises(RuntimeError):
        ops.peer_exchange(x, None, ptrs, 0, 2)               # parity
    with pytest.raises(RuntimeError):
        ops.peer_exchange(x[:6].contiguous(), None, ptrs, 0, 0)   # not a multiple of 4
    with pytest.raises(RuntimeError):
        ops.peer_exchange(x, None, ptrs[:1], 0, 0)           # one rank
    assert _lib.lib().msaq_peer_exchange_bytes(9, n) == 0


@pytest.mark.parametrize("OUT,K,M,prologue", [(8192, 1024, 1, 0), (8192, 3584, 1, 2), (4096, 2048, 4, 0), (8192, 4096, 8, 2),
                                              (1024, 256, 1, 0)])
def test_gemv_with_the_push_inside(OUT, K, M, prologue):
    """msaq_wonly_gemv_fused_push: the GEMV's finishing warps store the fp32 outputs as {x, seq} words into this rank's
    slot of every rank's buffer.  One GPU, both "ranks'" buffers local; the other rank's push is played by the host,
    then the receiving half adds up.  Bit-exact against the same GEMV's fp32 output."""
    from ms_kernel_b200 import ops, pack
    dev = torch.device("cuda", 0)
    o = _ops()
    g = torch.Generator(device="cuda").manual_seed(OUT + K + M)
    W = (torch.randn((OUT, K), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    lin = ops.PackedLinear(pack.pack_weight(W, 4, 2, device=dev), dev)
    assert lin.can_push(M) and not lin.can_push(9)
    x = torch.randn((M, (2 if prologue == 2 else 1) * K), generator=g, device="cuda").to(torch.bfloat16)
    want = lin.fwd_fused(x, prologue, None, 1e-5, True) if prologue else lin.fwd_f32(x)
    world, rank, n = 2, 1, M * OUT
    bufs = _bufs(world, n, dev)
    ptrs = [b.data_ptr() for b in bufs]
    other = torch.randn(n, generator=torch.Generator().manual_seed(5))
    h = torch.randn((M, OUT), generator=g, device="cuda").to(torch.bfloat16)
    for it, parity in enumerate((0, 1, 0)):
        seq = it // 2 + 1
        torch.cuda.synchronize()
        lin.fwd_push(x, prologue, 1e-5, ptrs, rank, parity)
        torch.cuda.synchronize()
        for r in range(world):                               # landed in both buffers, every word with the sequence number
            assert torch.equal(_slot(bufs[r], world, n, parity, rank).cpu(), _encode(want.reshape(-1).cpu(), seq))
        _slot(bufs[rank], world, n, parity, 0).copy_(_encode(other, seq))       # the peer's push, played by the host
        torch.cuda.synchronize()
        res = h if it == 2 else None
        got = o.peer_exchange_recv(x, res, ptrs, rank, parity, M, OUT)
        torch.cuda.synchronize()
        total = other.reshape(M, OUT) + want.cpu()           # rank order: rank 0 (the peer) first
        if res is not None:
            total = (h.float().cpu() + total).to(torch.bfloat16)
        assert torch.equal(got.cpu(), total)
        assert _ctl(bufs[rank], world, n).cpu()[parity] == seq
    assert o.wait_status(True) == 0


def test_push_refuses_what_the_mma_gemv_does_not_serve():
    from ms_kernel_b200 import ops, pack
    dev = torch.device("cuda", 0)
    W = (torch.randn((256, 256), device="cuda") * 0.02).to(torch.bfloat16)
    lin3 = ops.PackedLinear(pack.pack_weight(W, 3, 2, device=dev), dev)
    assert not lin3.can_push(1)
    bufs = _bufs(2, 256, dev)
    x = torch.randn((1, 256), device="cuda").to(torch.bfloat16)
    with pytest.raises(RuntimeError):
        lin3.fwd_push(x, 0, 1e-5, [b.data_ptr() for b in bufs], 0, 0)


def _two_rank_worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import datetime
        import torch.distributed as dist
        from ms_kernel_b200 import tp
        dev = torch.device("cuda", rank)
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
        n = 8192
        ex = tp.PeerExchange(dist.group.WORLD, n, dev)
        bad = 0
        gens = [torch.Generator().manual_seed(7 + r) for r in range(world)]
        for it in range(40):
            parts = [torch.randn(n, generator=gens[r]) for r in range(world)]
            h = torch.randn(n, generator=gens[0]).to(torch.bfloat16)
            want = parts[0].clone()
            for r in range(1, world):
                want += parts[r]
            got = ex(parts[rank].to(dev))
            bad += int(not torch.equal(got.cpu(), want))
            got2 = ex.reduce_add(parts[rank].to(dev), h.to(dev))
            bad += int(not torch.equal(got2.cpu(), (h.float() + want).to(torch.bfloat16)))
        # the two halves: a GEMV with the push inside, then the receiving half; against the partials all-gathered
        from ms_kernel_b200 import ops, pack
        gw = torch.Generator(device="cuda").manual_seed(100 + rank)
        W = (torch.randn((n, 1024), generator=gw, device="cuda") * 0.02).to(torch.bfloat16)
        lin = ops.PackedLinear(pack.pack_weight(W, 4, 2, device=dev), dev)
        xa = torch.randn((1, 1024), generator=gw, device="cuda").to(torch.bfloat16)
        mine = lin.fwd_f32(xa)
        parts = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        want = parts[0].clone()
        for r in range(1, world):
            want += parts[r]
        torch.cuda.synchronize()
        for it in range(20):
            got = ex.recv(ex.push_from(lin, xa))
            bad += int(not torch.equal(got, want))
        # the same inside a CUDA graph, replayed
        x = torch.randn(n, generator=gens[rank]).to(dev)
        allx = [torch.zeros(n, device=dev) for _ in range(world)]
        dist.all_gather(allx, x)
        want = allx[0].clone()
        for r in range(1, world):
            want += allx[r]
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            ex(x); ex(x)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            y0 = ex(x)
            y1 = ex(x)
        for _ in range(50):
            g.replay()
        torch.cuda.synchronize()
        bad += int(not torch.equal(y0, want)) + int(not torch.equal(y1, want))
        status = int(torch.ops.msaq.wait_status(True))
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, bad, status))
    except Exception as e:                                    # pragma: no cover
        q.put((rank, -1, repr(e)))
    q.close()
    q.join_thread()


@pytest.mark.timeout(300)
def test_two_ranks_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + os.getpid() % 200
    procs = [ctx.Process(target=_two_rank_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(30)
    for rank, bad, status in res:
        assert bad == 0 and status == 0, (rank, bad, status)

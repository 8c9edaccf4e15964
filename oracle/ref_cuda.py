"""Runs the reference project's own CUDA operators (oracle/_ref/ms_cuda_ref.so, built by oracle/build_ref.py)
in a process of their own -- test infrastructure, not product.

The reference registers `torch.ops.msaq.*`, the same names this repository's operator module registers, so
the two cannot live in one process.  Callers (tests/, bench.py's detail section) use `call()` / `time_ops()`,
which start `python oracle/ref_cuda.py <job.npz> <out.npz>` and read the result back.

A job is a list of operator calls on arrays the caller supplies (parity) or on random packed data the worker
makes itself (timing: any bytes are valid codes, so timing needs no packer).
"""

import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_ref", "ms_cuda_ref.so")
L2_BYTES = 126 << 20


def available():
    return os.path.exists(LIB)


# ----------------------------------------------------------------------------------------------
# caller side
# ----------------------------------------------------------------------------------------------
def _run(job, arrays, timeout=600, env=None):
    with tempfile.TemporaryDirectory() as d:
        jp, op = os.path.join(d, "job.npz"), os.path.join(d, "out.npz")
        np.savez(jp, __job__=np.frombuffer(json.dumps(job).encode(), np.uint8), **arrays)
        e = dict(os.environ)
        e.update(env or {})
        r = subprocess.run([sys.executable, os.path.abspath(__file__), jp, op], capture_output=True, text=True,
                           timeout=timeout, env=e)
        if r.returncode != 0:
            raise RuntimeError("reference CUDA worker failed (rc %d):\n%s" % (r.returncode, (r.stdout + r.stderr)[-3000:]))
        with np.load(op) as z:
            return {k: z[k] for k in z.files}


def call(op, args, env=None):
    """One operator call.  args: list of ints / floats / NumPy arrays; float32 arrays marked bf16 by wrapping
    them as ("bf16", array).  Returns the list of output arrays (bf16 outputs as float32), followed by the
    arrays among the inputs after the call (for the in-place cache writers)."""
    arrays, spec = {}, []
    for i, a in enumerate(args):
        if isinstance(a, tuple) and a[0] == "bf16":
            arrays["a%d" % i] = np.ascontiguousarray(a[1], np.float32)
            spec.append(["bf16", "a%d" % i])
        elif isinstance(a, np.ndarray):
            arrays["a%d" % i] = np.ascontiguousarray(a)
            spec.append(["arr", "a%d" % i])
        else:
            spec.append(["val", a])
    out = _run({"mode": "call", "op": op, "args": spec}, arrays, env=env)
    n_out = int(out["n_out"])
    outs = [out["o%d" % i] for i in range(n_out)]
    ins = [out["i%d" % i] for i in range(len(args)) if "i%d" % i in out]
    return outs, ins


def time_ops(cases, iters=10):
    """cases: list of dicts {"kind": "gemv"|"kv_decode", ...sizes...}; returns microseconds per call, CUDA-graph
    replay over enough distinct weight / cache copies to exceed L2, best of three windows."""
    out = _run({"mode": "time", "cases": cases, "iters": iters}, {}, timeout=1200)
    return [float(x) for x in out["us"]]


# ----------------------------------------------------------------------------------------------
# worker side
# ----------------------------------------------------------------------------------------------
def _worker(job_path, out_path):
    import torch
    with np.load(job_path) as z:
        job = json.loads(bytes(z["__job__"]).decode())
        arrays = {k: z[k] for k in z.files if k != "__job__"}
    torch.ops.load_library(LIB)
    ops = torch.ops.msaq
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)

    if job["mode"] == "call":
        targs, keep = [], {}
        for i, (kind, v) in enumerate(job["args"]):
            if kind == "val":
                targs.append(v)
            else:
                t = torch.from_numpy(arrays[v]).to(dev)
                if kind == "bf16":
                    t = t.to(torch.bfloat16)
                else:
                    keep[i] = t
                targs.append(t)
        res = getattr(ops, job["op"])(*targs)
        torch.cuda.synchronize()
        if res is None:
            res = []
        elif isinstance(res, torch.Tensor):
            res = [res]
        out = {"n_out": np.array(len(res))}
        for i, t in enumerate(res):
            out["o%d" % i] = (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()
        for i, t in keep.items():
            out["i%d" % i] = t.cpu().numpy()
        np.savez(out_path, **out)
        return

    # ---- timing ----
    def graph_time(fns, iters):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for f in fns:
                f()
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(True), torch.cuda.Event(True)
        best = float("inf")
        for _ in range(3):
            a.record()
            for _ in range(iters):
                g.replay()
            b.record()
            torch.cuda.synchronize()
            best = min(best, a.elapsed_time(b) * 1e3 / iters / len(fns))
        return best

    gen = torch.Generator(device=dev).manual_seed(1)

    def rand_u8(shape):
        return torch.randint(0, 256, shape, generator=gen, device=dev, dtype=torch.uint8)

    us = []
    for c in job["cases"]:
        u, gs = int(c.get("u", 4)), int(c.get("gs", 2))
        UB, SB = 32 * (8 - u) // 8, ((32 // gs) * u + 7) // 8
        if c["kind"] == "gemv":
            OUT, K, M = int(c["OUT"]), int(c["K"]), int(c["M"])
            nb = K // 32
            nbytes = OUT * nb * (UB + SB + 1)
            copies = int(min(64, max(2, -(-3 * L2_BYTES // nbytes))))
            sets = [(torch.full((nb, OUT), -8, dtype=torch.int8, device=dev), rand_u8((nb, OUT, UB)), rand_u8((nb, OUT, SB)))
                    for _ in range(copies)]
            x = torch.randn((M, K) if M > 1 else (K,), generator=gen, device=dev).to(torch.bfloat16)
            if M == 1:
                fns = [(lambda s=s: ops.wonly_gemv_wide(x, s[0], s[1], s[2], OUT, nb, u, gs)) for s in sets]
            else:
                fns = [(lambda s=s: ops.wonly_gemv_batched(x, s[0], s[1], s[2], M, OUT, nb, u, gs)) for s in sets]
            us.append(graph_time(fns, job["iters"]))
            del sets
        else:
            B, Hq, Hkv, Lk, D = int(c["B"]), int(c["Hq"]), int(c["Hkv"]), int(c["Lk"]), int(c.get("D", 128))
            nb = D // 32
            nbytes = B * Hkv * Lk * 2 * nb * (UB + SB + 1)
            copies = int(max(1, min(6, -(-3 * L2_BYTES // nbytes))))

            def planes():
                return (torch.full((B, Hkv, nb, Lk), -6, dtype=torch.int8, device=dev), rand_u8((B, Hkv, nb, Lk, UB)),
                        rand_u8((B, Hkv, nb, Lk, SB)))

            caches = [(planes(), planes()) for _ in range(copies)]
            q = torch.randn((B, Hq, D), generator=gen, device=dev).to(torch.bfloat16)
            fns = [(lambda kv=kv: ops.kv_decode_attention_batched(q, *kv[0], *kv[1], B, Hq, Hkv, Lk, D, nb, u, gs, Lk))
                   for kv in caches]
            us.append(graph_time(fns, job["iters"]))
            del caches
        torch.cuda.empty_cache()
    np.savez(out_path, us=np.array(us))


if __name__ == "__main__":
    _worker(sys.argv[1], sys.argv[2])

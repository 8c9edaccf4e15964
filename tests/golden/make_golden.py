"""Generate tests/golden/msaq_golden.npz from the reference project's own NumPy code.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's `ms_lib.pack` / `ms_lib.reference` (NumPy only) and
records their outputs on small seeded inputs.  The fixtures pin the CPU oracle
under oracle/; nothing at test time needs the reference checkout.

What is recorded
  dec_*   decompose(): exponent / upper / shared codes for hand-made edge blocks
          and random blocks, for u in {2,3,4} x gs in {2,4,8,16,32}
  w_*     pack_weight(): every plane, dequant_weight(), wonly_matmul()
  kv_*    pack_kv(): planes; kv_attention() causal prefill and single query
  rot_*   the fp32 butterfly rotation written out as plain loops (the formula of
          the reference's append/rotate kernels), reference pack_kv() of those
          values, and the reference's host formulation bf16(K) @ H/sqrt(n)
  mx_*    plain MXINT8 (pack_weight_mxint8 / pack_kv_mxint8 / dequant / wonly_matmul_mxint8 /
          kv_attention_mxint8): planes and outputs of the reference's baseline format
  wa_*    quant_act(share=True) words and exponents, wa_matmul(share_act=True) outputs
  rope_*  the rotary embedding of the reference's harness (tests/harness_batchsweep.py:
          rope_tables, rope_pos, rope_bthd, executed from its source with torch on the CPU):
          tables, rotated rows, and reference pack_kv() of rope -> butterfly rotation
"""

import math
import os
import sys

import numpy as np


def bf16_round(a):
    a = np.ascontiguousarray(a, np.float32)
    b = a.view(np.uint32).astype(np.uint64)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32).reshape(a.shape)


def butterfly_rows(x):
    """Row-wise fp32 butterfly: stages h=1,2,..; lo' = lo + hi, hi' = lo - hi; then * f32(1/sqrt n)."""
    x = np.array(x, np.float32)
    rows, n = x.shape
    out = np.empty_like(x)
    inv = np.float32(1.0 / math.sqrt(n))
    for r in range(rows):
        v = [np.float32(t) for t in x[r]]
        h = 1
        while h < n:
            nv = list(v)
            for e in range(n):
                p = e ^ h
                nv[e] = np.float32(v[p] - v[e]) if (e & h) else np.float32(v[e] + v[p])
            v = nv
            h <<= 1
        out[r] = np.array(v, np.float32) * inv
    return out


def harness_namespace(ref_root, names):
    """The named top-level definitions of the reference's tests/harness_batchsweep.py, executed from
    its source in a namespace of their own (the module itself needs a GPU to import)."""
    import ast
    import torch
    with open(os.path.join(ref_root, "tests", "harness_batchsweep.py")) as f:
        tree = ast.parse(f.read())
    ns = {"torch": torch, "np": np}
    for node in tree.body:
        if isinstance(node, (ast.FunctionDef, ast.ClassDef)) and node.name in names:
            exec(compile(ast.Module([node], []), "harness_batchsweep.py", "exec"), ns)
    return ns


def edge_blocks(rng):
    b = []
    b.append(np.zeros(32))                                   # all-zero block
    b.append(np.full(32, 1.0))                               # exact power of two
    b.append(np.full(32, -1.0))
    x = np.zeros(32); x[5] = 3e-38; b.append(x)              # below the max-abs floor
    x = np.zeros(32); x[0] = 2.0 ** 100; b.append(x)         # huge
    x = np.zeros(32); x[31] = 2.0 ** -100; b.append(x)       # tiny
    b.append(np.linspace(-1, 1, 32))                         # many rounding ties
    b.append(np.arange(32) * 0.5)                            # half-integers (ties to even)
    b.append(np.where(np.arange(32) % 2, 127.0, -127.0))     # saturating both signs
    b.append(np.where(np.arange(32) % 2, 127.5, -128.0))
    x = rng.standard_normal(32); x[3] *= 20; b.append(x)     # one outlier
    b.append(np.full(32, 1.9999999))                         # just below a power of two
    b.append(np.full(32, 2.0 ** -126))                       # smallest normal f32
    return np.array(b, np.float64).astype(np.float32)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <checkout of yubin-wang99/ms_kernel>")
    ref_root = sys.argv[1]
    sys.path.insert(0, ref_root)
    from ms_lib import pack as rp
    from ms_lib import reference as rr

    rng = np.random.default_rng(20251125)
    out = {}

    blocks = np.concatenate([
        edge_blocks(rng),
        bf16_round((rng.standard_normal((48, 32)) * rng.uniform(0.01, 30, (48, 1))).astype(np.float32)),
        (rng.standard_normal((32, 32)) * rng.uniform(0.01, 30, (32, 1))).astype(np.float32),
    ])
    out["dec_blocks"] = blocks
    for u in (2, 3, 4):
        for gs in (2, 4, 8, 16, 32):
            s, qu, rs = rp.decompose(blocks, u, gs)
            out[f"dec_exp_u{u}_gs{gs}"] = np.rint(np.log2(s.reshape(-1))).astype(np.int16)
            out[f"dec_up_u{u}_gs{gs}"] = qu.astype(np.int8)
            out[f"dec_sh_u{u}_gs{gs}"] = rs.astype(np.int8)

    OUT, K, M = 48, 96, 3
    W = bf16_round((rng.standard_normal((OUT, K)) * rng.uniform(0.005, 0.08, (OUT, 1))).astype(np.float32))
    X = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    out["w_W"], out["w_X"] = W, X
    for u in (2, 3, 4):
        for gs in (2, 4, 8):
            p = rp.pack_weight(W, u, gs)
            tag = f"u{u}_gs{gs}"
            for k in ("scale_exp", "upper", "shared", "upper_cm", "shared_cm"):
                out[f"w_{k}_{tag}"] = p[k]
            out[f"w_deq_{tag}"] = rp.dequant_weight(p)
            out[f"w_y_{tag}"] = rr.wonly_matmul(p, X)

    H, L, D = 2, 20, 64
    Kt = bf16_round((rng.standard_normal((H, L, D)) * 0.5).astype(np.float32))
    Vt = bf16_round((rng.standard_normal((H, L, D)) * 0.5).astype(np.float32))
    Qp = bf16_round((rng.standard_normal((H, L, D)) * 0.5).astype(np.float32))
    out["kv_K"], out["kv_V"], out["kv_Q"] = Kt, Vt, Qp
    for u in (2, 3, 4):
        for gs in (2, 4, 8):
            pK, pV = rp.pack_kv(Kt, u, gs), rp.pack_kv(Vt, u, gs)
            tag = f"u{u}_gs{gs}"
            for k in ("scale_exp", "upper", "shared"):
                out[f"kv_K{k}_{tag}"] = pK[k]
                out[f"kv_V{k}_{tag}"] = pV[k]
            out[f"kv_prefill_{tag}"] = rr.kv_attention(Qp, pK, pV, causal=True)
            out[f"kv_decode_{tag}"] = rr.kv_attention(Qp[:, -1:, :], pK, pV, causal=True)[:, 0]

    Hr, Lr, Dr = 2, 6, 128
    Kr = bf16_round(rng.standard_normal((Hr, Lr, Dr)).astype(np.float32))
    Kr[:, :, [3, 40, 77, 120]] *= 20                      # persistent outlier channels
    Kr = bf16_round(Kr)
    rot = butterfly_rows(Kr.reshape(-1, Dr)).reshape(Hr, Lr, Dr)
    out["rot_K"], out["rot_f32"] = Kr, rot
    from scipy.linalg import hadamard
    Hn = hadamard(Dr).astype(np.float32) / np.sqrt(np.float32(Dr))
    out["rot_host"] = (Kr.reshape(-1, Dr) @ Hn).reshape(Hr, Lr, Dr)
    for u, gs in ((4, 2), (3, 8), (2, 4)):
        p = rp.pack_kv(rot, u, gs)
        for k in ("scale_exp", "upper", "shared"):
            out[f"rot_{k}_u{u}_gs{gs}"] = p[k]

    # ---- rotary embedding (own generator: the arrays above keep their values) ----
    import torch
    hs = harness_namespace(ref_root, ("Cfg", "rope_tables", "rope_pos", "rope_bthd"))
    rng2 = np.random.default_rng(20251126)
    Lp, Hh, hd = 40, 3, hs["Cfg"].head_dim
    cos, sin = hs["rope_tables"](Lp, "cpu")
    out["rope_cos"], out["rope_sin"] = cos.numpy(), sin.numpy()
    xr = torch.from_numpy(rng2.standard_normal((2, Lp, Hh, hd)).astype(np.float32))
    xr[..., [3, 40, 77, 120]] *= 20
    xr = xr.to(torch.bfloat16)
    out["rope_x"] = xr.float().numpy()
    yr = hs["rope_bthd"](xr, cos, sin)
    assert yr.dtype == torch.bfloat16
    out["rope_y"] = yr.float().numpy()
    c1, s1 = hs["rope_pos"](8191, "cpu")                   # the single-position tables of a decode step
    out["rope_cos_8191"], out["rope_sin_8191"] = c1.numpy(), s1.numpy()
    x1 = torch.from_numpy(rng2.standard_normal((4, 1, Hh, hd)).astype(np.float32)).to(torch.bfloat16)
    out["rope_x1"] = x1.float().numpy()
    out["rope_y1"] = hs["rope_bthd"](x1, c1, s1).float().numpy()
    # rope -> butterfly rotation -> pack: what a fused RoPE + rotate + append must write
    kro = out["rope_y"][0].transpose(1, 0, 2)              # [H, L, D]
    rotk = butterfly_rows(np.ascontiguousarray(kro).reshape(-1, hd)).reshape(Hh, Lp, hd)
    for u, gs in ((4, 2), (3, 8), (2, 4)):
        p = rp.pack_kv(rotk, u, gs)
        for k in ("scale_exp", "upper", "shared"):
            out[f"ropek_{k}_u{u}_gs{gs}"] = p[k]

    # ---- plain MXINT8, the reference's matched baseline format ----
    rng3 = np.random.default_rng(20251127)
    Wm = bf16_round((rng3.standard_normal((40, 96)) * rng3.uniform(0.005, 0.08, (40, 1))).astype(np.float32))
    Wm[:14, :32] = blocks[:14]                                # the hand-made edge blocks as weight blocks
    Xm = bf16_round(rng3.standard_normal((3, 96)).astype(np.float32))
    pm = rp.pack_weight_mxint8(Wm)
    out["mx_W"], out["mx_X"] = Wm, Xm
    for k in ("scale_exp", "qweight", "qweight_cm"):
        out[f"mx_w_{k}"] = pm[k]
    out["mx_w_deq"] = rp.dequant_weight_mxint8(pm)
    out["mx_w_y"] = rr.wonly_matmul_mxint8(pm, Xm)
    pKm, pVm = rp.pack_kv_mxint8(Kt), rp.pack_kv_mxint8(Vt)
    for k in ("scale_exp", "qweight"):
        out[f"mx_kv_K{k}"], out[f"mx_kv_V{k}"] = pKm[k], pVm[k]
    out["mx_kv_prefill"] = rr.kv_attention_mxint8(Qp, pKm, pVm, causal=True)
    out["mx_kv_decode"] = rr.kv_attention_mxint8(Qp[:, -1:, :], pKm, pVm, causal=True)[:, 0]

    # ---- W+A: run-time activation quantisation and the integer-dot product ----
    rng4 = np.random.default_rng(20251128)
    Xa = bf16_round((rng4.standard_normal((5, K)) * rng4.uniform(0.01, 8, (5, 1))).astype(np.float32))
    Xa[0, :32] = bf16_round(blocks[6])                      # ties
    out["wa_X"] = Xa
    for u in (2, 3, 4):
        for gs in (2, 8):
            tag = f"u{u}_gs{gs}"
            qx, sx = rr.quant_act(Xa, u, gs, share=True)
            out[f"wa_q_{tag}"] = qx.astype(np.int8)
            out[f"wa_exp_{tag}"] = np.rint(np.log2(sx)).astype(np.int16)
            out[f"wa_y_{tag}"] = rr.wa_matmul(rp.pack_weight(W, u, gs), Xa, share_act=True)

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "msaq_golden.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()

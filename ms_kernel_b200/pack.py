"""Packers that run on the device and return the reference's pack dicts.

Same keys, shapes, dtypes and bytes as `ms_lib.pack.pack_weight` /
`ms_lib.pack.pack_kv` of the reference (ms_lib/pack.py:101-137, :479-504), with
torch tensors on the GPU in place of NumPy arrays.  `to_numpy` converts a dict
for code that expects the NumPy form.
"""

import torch

from . import ops as _ops

BLOCK = 32


def plane_bytes(u, gs):
    """(UB, SB): bytes of upper and of shared codes per 32-block."""
    return BLOCK * (8 - u) // 8, ((BLOCK // gs) * u + 7) // 8


def _as_cuda(x, device):
    if not isinstance(x, torch.Tensor):
        x = torch.as_tensor(x)
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.to(torch.float32)
    return x.to(device).contiguous()


def pack_weight(W, u, gs, device="cuda"):
    """W [OUT,K] (bf16 or fp32; NumPy or tensor) -> pack dict of device tensors."""
    _ops._require()
    Wd = _as_cuda(W, device)
    OUT, K = Wd.shape
    s, up, sh, upc, shc = torch.ops.msaq.pack_weight(Wd, u, gs)
    UB, SB = plane_bytes(u, gs)
    return dict(scale_exp=s, upper=up, shared=sh, upper_cm=upc, shared_cm=shc,
                OUT=OUT, K=K, nb=K // BLOCK, u=u, gs=gs, wbits=8 - u, UB=UB, SB=SB, n_group=BLOCK // gs)


def pack_kv(KV, u, gs, device="cuda", rotate=False):
    """KV [H,L,D] bf16 -> token-major plane dict; rotate=True Hadamard-rotates every row first."""
    _ops._require()
    X = _as_cuda(KV, device).to(torch.bfloat16)
    H, L, D = X.shape
    op = torch.ops.msaq.kv_write_rot if rotate else torch.ops.msaq.kv_write
    s, up, sh = op(X, H, L, D, D // BLOCK, u, gs)
    UB, SB = plane_bytes(u, gs)
    return dict(scale_exp=s, upper=up, shared=sh, H=H, L=L, D=D, nb=D // BLOCK, u=u, gs=gs,
                wbits=8 - u, UB=UB, SB=SB, n_group=BLOCK // gs)


def to_numpy(p):
    """Pack dict with tensors -> the same dict with NumPy arrays."""
    return {k: (v.cpu().numpy() if isinstance(v, torch.Tensor) else v) for k, v in p.items()}

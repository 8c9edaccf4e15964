"""Python API of the decode path; same names and argument meaning as the
reference's `ms_lib/ops.py` (wonly_gemv :67-82, kv_decode_attention :134-143,
available :33-35), plus device-resident holders for callers that do not want a
host-to-device copy of the planes on every call.

Pack dicts are the ones `ms_lib.pack.pack_weight` / `pack_kv` produce (or the
device packers in `ms_kernel_b200.pack`): NumPy arrays or torch tensors under
the keys scale_exp / upper / shared / upper_cm / shared_cm plus the meta ints.
"""

import os
import sys

_IMPORT_ERROR = None
try:
    import torch
    from . import ms_cuda as _ms_cuda          # side effect: registers torch.ops.msaq.*
    sys.modules.setdefault("ms_cuda", _ms_cuda)  # so `import ms_cuda` finds this build
    _OPS = torch.ops.msaq
    _AVAILABLE = True
except Exception as e:                          # torch missing or extension not built
    _IMPORT_ERROR = e
    _AVAILABLE = False
    _OPS = None


def available() -> bool:
    """True iff the compiled `ms_cuda` module imported and registered the ops."""
    return _AVAILABLE


PRO_NONE, PRO_RMSNORM, PRO_SILU_MUL, PRO_ADD_RMSNORM = 0, 1, 2, 3   # include/msaq_b200.h: MSAQ_PRO_*
OPT_TENSOR_MEMORY = 2    # batched GEMVs of 9+ rows on tcgen05 / tensor memory (default on)
OPT_CHAINED_LAUNCH = 1   # overlap each kernel's launch and prologue with the tail of the one before it (default on)
OPT_EARLY_WEIGHTS = 6    # GEMVs fetch weights before waiting for the kernel in front (default off: the caller vouches
                         # that the weight planes are complete, not being written by work still in flight)


def set_option(option: int, value: bool) -> None:
    """Process-wide switch of the library (include/msaq_b200.h: msaq_set_option)."""
    _require()
    _OPS.set_option(int(option), int(bool(value)))


def _require():
    if not _AVAILABLE:
        raise RuntimeError(
            "ms_cuda backend not available (%s: %s). Build it with "
            "`python -m ms_kernel_b200.build`; there is no fallback path."
            % (type(_IMPORT_ERROR).__name__, _IMPORT_ERROR))


def _dev(t, device):
    """NumPy array or tensor -> tensor on `device` (no copy if already there)."""
    if isinstance(t, torch.Tensor):
        return t.to(device)
    return torch.from_numpy(t).to(device)


# --------------------------------------------------------------------------
# reference-compatible wrappers (planes travel host -> device on every call)
# --------------------------------------------------------------------------
def wonly_gemv(p, x_bf16):
    """W-only decode GEMV.  p from pack_weight; x_bf16 [K] -> y [OUT] bf16."""
    _require()
    dev = x_bf16.device
    s = _dev(p["scale_exp"], dev)
    if "upper_cm" in p:
        return _OPS.wonly_gemv_wide(x_bf16, s, _dev(p["upper_cm"], dev), _dev(p["shared_cm"], dev),
                                    int(p["OUT"]), int(p["nb"]), int(p["u"]), int(p["gs"]))
    return _OPS.wonly_gemv(x_bf16, s, _dev(p["upper"], dev), _dev(p["shared"], dev),
                           int(p["OUT"]), int(p["nb"]), int(p["u"]), int(p["gs"]))


def wonly_gemv_batched(p, X_bf16):
    """Small-batch decode GEMV.  X_bf16 [M,K] -> Y [M,OUT] bf16."""
    _require()
    dev = X_bf16.device
    return _OPS.wonly_gemv_batched(X_bf16, _dev(p["scale_exp"], dev), _dev(p["upper_cm"], dev),
                                   _dev(p["shared_cm"], dev), int(X_bf16.shape[0]),
                                   int(p["OUT"]), int(p["nb"]), int(p["u"]), int(p["gs"]))


def kv_decode_attention(q_bf16, pK, pV):
    """Fused-dequant flash-decode attention.  q_bf16 [H,D]; pK, pV from pack_kv -> [H,D] bf16."""
    _require()
    dev = q_bf16.device
    ks, ku, kh = (_dev(pK[k], dev) for k in ("scale_exp", "upper", "shared"))
    vs, vu, vh = (_dev(pV[k], dev) for k in ("scale_exp", "upper", "shared"))
    return _OPS.kv_decode_attention(q_bf16, ks, ku, kh, vs, vu, vh,
                                    int(q_bf16.shape[0]), int(pK["H"]), int(pK["L"]), int(pK["D"]),
                                    int(pK["nb"]), int(pK["u"]), int(pK["gs"]))


# --------------------------------------------------------------------------
# device-resident holders
# --------------------------------------------------------------------------
class PackedLinear:
    """A packed weight kept on the device; `fwd` picks the op by batch size
    (the dispatch of the reference harness, tests/harness_batchsweep.py:77-111,
    without its dequant+cuBLAS branch)."""

    def __init__(self, p, device):
        _require()
        self.OUT, self.nb, self.u, self.gs = int(p["OUT"]), int(p["nb"]), int(p["u"]), int(p["gs"])
        self.K = self.nb * 32
        self.scale_exp = _dev(p["scale_exp"], device).contiguous()
        self.upper_cm = _dev(p["upper_cm"], device).contiguous()
        self.shared_cm = _dev(p["shared_cm"], device).contiguous()

    def nbytes(self):
        return self.scale_exp.numel() + self.upper_cm.numel() + self.shared_cm.numel()

    def fwd(self, x):
        """x [K] or [M,K] bf16 -> [OUT] or [M,OUT] bf16."""
        if x.dim() == 1:
            return _OPS.wonly_gemv_wide(x, self.scale_exp, self.upper_cm, self.shared_cm,
                                        self.OUT, self.nb, self.u, self.gs)
        return _OPS.wonly_gemv_batched(x, self.scale_exp, self.upper_cm, self.shared_cm,
                                       int(x.shape[0]), self.OUT, self.nb, self.u, self.gs)


    def fwd_f32(self, x):
        """x [M,K] bf16 -> [M,OUT] fp32, the result before its bf16 rounding (the partial sum a
        K-sharded linear contributes to an all-reduce)."""
        x = x.reshape(-1, self.K)
        return _OPS.wonly_gemv_batched_f32(x.contiguous(), self.scale_exp, self.upper_cm, self.shared_cm,
                                           int(x.shape[0]), self.OUT, self.nb, self.u, self.gs)

    def fwd_fused(self, x, prologue, addend=None, eps=1e-5, out_f32=False):
        """The GEMV with the layer glue in front of it done by the activation-staging kernel.

        prologue: PRO_RMSNORM (x [M,K]), PRO_SILU_MUL (x [M,2K] = gate | up) or PRO_ADD_RMSNORM
        (x [M,K] + addend [M,K] fp32/bf16).  Returns y [M,OUT] (fp32 before rounding with out_f32, else
        bf16); for PRO_ADD_RMSNORM (y, x + addend)."""
        M = int(x.shape[0])
        out = _OPS.wonly_gemv_fused(x.contiguous(), None if addend is None else addend.contiguous(), int(prologue),
                                    float(eps), self.scale_exp, self.upper_cm, self.shared_cm, M, self.OUT, self.nb,
                                    self.u, self.gs, bool(out_f32))
        return (out[0], out[1]) if prologue == PRO_ADD_RMSNORM else out[0]

    def fwd_fused_add(self, x, prologue, residual, eps=1e-5):
        """residual + GEMV(prologue(x)) in bf16, the residual add done by the GEMV's finishing warps (same
        roundings as fwd_fused followed by the add).  prologue: PRO_NONE, PRO_RMSNORM or PRO_SILU_MUL."""
        M = int(x.shape[0])
        return _OPS.wonly_gemv_fused_add(x.contiguous(), int(prologue), float(eps), self.scale_exp, self.upper_cm,
                                         self.shared_cm, residual.contiguous(), M, self.OUT, self.nb, self.u, self.gs)

    def can_push(self, M):
        """Whether fwd_push serves M rows of this linear (the integer-MMA GEMV's terms)."""
        return self.u == 4 and self.gs == 2 and 1 <= M <= 8 and self.OUT % 16 == 0 and (M * self.OUT) % 4 == 0

    def fwd_push(self, x, prologue, eps, peer_ptrs, rank, parity):
        """The GEMV of a row-parallel (K-sharded) linear with the exchange's push inside: the fp32 partial sums
        go straight from the kernel's finishing warps into every rank's exchange buffer (include/msaq_b200.h:
        msaq_wonly_gemv_fused_push).  prologue: PRO_NONE, PRO_RMSNORM or PRO_SILU_MUL.  Returns nothing; the sum
        comes out of the receiving half of the exchange (tp.PeerExchange.recv)."""
        M = int(x.shape[0])
        _OPS.wonly_gemv_fused_push(x.contiguous(), int(prologue), float(eps), self.scale_exp, self.upper_cm,
                                   self.shared_cm, M, self.OUT, self.nb, self.u, self.gs, list(peer_ptrs), int(rank),
                                   int(parity))


class KVCache:
    """Packed K and V caches [B,Hkv,nb,Lcap,*] with append and attend.

    Mirrors the KVCache of the reference harness (tests/harness_batchsweep.py:
    139-199): keys are Hadamard-rotated on append when `rotate` is set and the
    query is then rotated inside the attention kernel.
    """

    def __init__(self, B, Hkv, D, Lcap, u, gs, device, rotate=True):
        _require()
        self.B, self.Hkv, self.D, self.Lcap, self.u, self.gs = B, Hkv, D, Lcap, u, gs
        self.nb = D // 32
        self.UB = 32 * (8 - u) // 8
        self.SB = ((32 // gs) * u + 7) // 8
        self.rotate = bool(rotate)

        def planes():
            return (torch.zeros((B, Hkv, self.nb, Lcap), dtype=torch.int8, device=device),
                    torch.zeros((B, Hkv, self.nb, Lcap, self.UB), dtype=torch.uint8, device=device),
                    torch.zeros((B, Hkv, self.nb, Lcap, self.SB), dtype=torch.uint8, device=device))

        self.k, self.v = planes(), planes()
        self._full_lens = {}

    def nbytes_per_key(self):
        return 2 * self.Hkv * self.nb * (self.UB + self.SB + 1)

    def fill(self, K, V, key0=0):
        """Prefill: K, V [B,Hkv,L,D] bf16 written to slots [key0, key0+L)."""
        B, Hkv, L, D = K.shape
        for X, pl, rot in ((K, self.k, self.rotate), (V, self.v, False)):
            _OPS.kv_write_into(X.contiguous(), pl[0], pl[1], pl[2], B * Hkv, L, D, self.nb, key0,
                               self.Lcap, self.u, self.gs, rot)

    def append(self, k_new, v_new, pos, rope=None):
        """k_new, v_new [B,Hkv,D] bf16; pos an int (all sequences) or int32 tensor [B].

        rope = (cos, sin), fp32 [rows, D/2] as the reference's harness builds them
        (tests/harness_batchsweep.py:118-131; rows == 1: the one position of this step, else indexed
        by position): the K rows get the rotary embedding inside the same launch, before the
        Hadamard rotation, exactly as rope_bthd followed by kv_append_rot would."""
        H = self.B * self.Hkv
        k_new = k_new.reshape(H, self.D).contiguous()
        v_new = v_new.reshape(H, self.D).contiguous()
        # one launch for both tensors (kv_append_rot + kv_append of the reference write the same bytes)
        pos_t, pos_i = (None, pos) if isinstance(pos, int) else (pos, 0)
        if rope is None:
            _OPS.kv_append_pair(k_new, v_new, *self.k, *self.v, pos_t, self.B, self.Hkv, self.D, self.nb, pos_i,
                                self.Lcap, self.u, self.gs, self.rotate)
        else:
            _OPS.kv_append_pair_rope(k_new, v_new, *self.k, *self.v, pos_t, self.B, self.Hkv, self.D, self.nb, pos_i,
                                     self.Lcap, self.u, self.gs, self.rotate, rope[0], rope[1])

    def attend(self, q, Lk, seq_lens=None, rope=None, q_pos=None):
        """q [B,Hq,D] bf16 -> [B,Hq,D] bf16 over the first Lk keys (seq_lens[b] if given).

        rope = (cos, sin) with q_pos (int or int32 tensor [B], the position of the query token):
        the query rows get the rotary embedding in the kernel prologue."""
        Hq = int(q.shape[1])
        if seq_lens is None:
            seq_lens = self._full_lens.get(Lk)
            if seq_lens is None:
                seq_lens = self._full_lens[Lk] = torch.full((self.B,), Lk, dtype=torch.int32, device=q.device)
        if rope is None:
            return _OPS.kv_decode_attention_varlen(q, *self.k, *self.v, seq_lens, self.B, Hq, self.Hkv, Lk, self.D,
                                                   self.nb, self.u, self.gs, self.Lcap, self.rotate)
        pos_t, pos_i = (None, int(q_pos)) if isinstance(q_pos, int) else (q_pos, 0)
        return _OPS.kv_decode_attention_rope(q, *self.k, *self.v, seq_lens, self.B, Hq, self.Hkv, Lk, self.D, self.nb,
                                             self.u, self.gs, self.Lcap, self.rotate, rope[0], rope[1], pos_t, pos_i)

    def append_attend(self, q, k_new, v_new, pos, Lk, seq_lens=None, rope=None):
        """append(k_new, v_new, pos, rope) followed by attend(q, Lk, seq_lens, rope, pos) in one call: the same bytes
        in the cache, the same output; on the tuned path the attention kernel packs the new token itself and the
        append costs no launch (include/msaq_b200.h: msaq_kv_decode_attention_append)."""
        Hq = int(q.shape[1])
        if seq_lens is None:
            seq_lens = self._full_lens.get(Lk)
            if seq_lens is None:
                seq_lens = self._full_lens[Lk] = torch.full((self.B,), Lk, dtype=torch.int32, device=q.device)
        H = self.B * self.Hkv
        pos_t, pos_i = (None, int(pos)) if isinstance(pos, int) else (pos, 0)
        cos, sin = (None, None) if rope is None else (rope[0], rope[1])
        return _OPS.kv_decode_attention_append(q, k_new.reshape(H, self.D).contiguous(), v_new.reshape(H, self.D).contiguous(),
                                               *self.k, *self.v, seq_lens, self.B, Hq, self.Hkv, Lk, self.D, self.nb, self.u,
                                               self.gs, self.Lcap, self.rotate, self.rotate, cos, sin, pos_t, pos_i)


# --------------------------------------------------------------------------
# plain MXINT8 twins (the reference's matched baseline format, ms_lib/pack.py:530-594)
# --------------------------------------------------------------------------
class PackedLinearMX:
    """A weight in plain MXINT8 (int8 code per element + one scale byte per 32) kept on the device.
    Built from a bf16 / fp32 weight on the device, or from `pack_weight_mxint8`'s dict."""

    def __init__(self, w_or_pack, device):
        _require()
        if isinstance(w_or_pack, dict):
            self.scale_exp = _dev(w_or_pack["scale_exp"], device).contiguous()
            self.qweight_cm = _dev(w_or_pack["qweight_cm"], device).contiguous()
        else:
            self.scale_exp, _, self.qweight_cm = _OPS.mxint8_pack_weight(w_or_pack.to(device).contiguous())
        self.nb, self.OUT = int(self.scale_exp.shape[0]), int(self.scale_exp.shape[1])
        self.K = self.nb * 32

    def nbytes(self):
        return self.scale_exp.numel() + self.qweight_cm.numel()

    def fwd(self, x):
        """x [K] or [M,K] bf16 -> [OUT] or [M,OUT] bf16."""
        if x.dim() == 1:
            return _OPS.mxint8_gemv_wide(x, self.scale_exp, self.qweight_cm, self.OUT, self.nb)
        return _OPS.mxint8_gemv_batched_wide(x, self.scale_exp, self.qweight_cm, int(x.shape[0]), self.OUT, self.nb)


class KVCacheMX:
    """K and V caches in plain MXINT8, planes [B,Hkv,nb,Lcap] / [B,Hkv,nb,Lcap,32] (the MXINT8 branch of the
    reference harness's KVCache, tests/harness_batchsweep.py:139-199); head_dim 128."""

    def __init__(self, B, Hkv, D, Lcap, device):
        _require()
        self.B, self.Hkv, self.D, self.Lcap, self.nb = B, Hkv, D, Lcap, D // 32

        def planes():
            return (torch.zeros((B, Hkv, self.nb, Lcap), dtype=torch.int8, device=device),
                    torch.zeros((B, Hkv, self.nb, Lcap, 32), dtype=torch.int8, device=device))

        self.k, self.v = planes(), planes()
        self._full_lens = {}

    def fill(self, K, V, key0=0):
        B, Hkv, L, D = K.shape
        for X, pl in ((K, self.k), (V, self.v)):
            _OPS.mxint8_kv_write_into(X.contiguous(), pl[0], pl[1], B * Hkv, L, D, self.nb, key0, self.Lcap)

    def append(self, k_new, v_new, pos):
        H = self.B * self.Hkv
        for X, pl in ((k_new, self.k), (v_new, self.v)):
            _OPS.mxint8_kv_append(X.reshape(H, self.D).contiguous(), pl[0], pl[1], H, self.D, self.nb, int(pos), self.Lcap)

    def attend(self, q, Lk, seq_lens=None):
        Hq = int(q.shape[1])
        if seq_lens is None:
            return _OPS.mxint8_kv_decode_batched(q, *self.k, *self.v, self.B, Hq, self.Hkv, Lk, self.D, self.nb, self.Lcap)
        return _OPS.mxint8_kv_decode_varlen(q, *self.k, *self.v, seq_lens, self.B, Hq, self.Hkv, Lk, self.D, self.nb, self.Lcap)

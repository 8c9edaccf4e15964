"""CPU-side checks of the boundary: the C-ABI library loads, exports every symbol the
header declares, validates arguments before touching the device, and refuses to run
without an sm_100 GPU instead of falling back to anything."""

import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "msaq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(msaq_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from ms_kernel_b200 import _lib
    L = _lib.lib()
    names = _declared()
    assert len(names) >= 16
    for n in names:
        assert hasattr(L, n), "library does not export %s" % n
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"
    assert L.msaq_version() >= 1000


def test_argument_validation_needs_no_device():
    from ms_kernel_b200 import _lib
    L = _lib.lib()
    assert L.msaq_wonly_gemv_wide(None, None, None, None, None, None, 8, 2, 4, 2, None, 0, None) == -1
    assert b"null" in L.msaq_last_error()
    one = 8  # any non-null address; rejected before it is dereferenced
    assert L.msaq_wonly_gemv_wide(one, one, one, one, one, None, 8, 2, 7, 2, None, 0, None) == -2
    assert L.msaq_wonly_gemv_wide(one, one, one, one, one, None, 8, 2, 4, 3, None, 0, None) == -2
    assert L.msaq_wonly_gemv_wide(one, one, one, one, one, None, 0, 2, 4, 2, None, 0, None) == -1
    assert L.msaq_kv_append(one, one, one, one, 4, 100, 3, 0, 8, 4, 2, None) == -1      # NB != D/32
    assert L.msaq_kv_append(one, one, one, one, 4, 96, 3, 0, 8, 4, 2, None) == -2       # D not a power of two
    assert L.msaq_kv_append(one, one, one, one, 4, 128, 4, 9, 8, 4, 2, None) == -1      # pos beyond capacity
    args = [one] * 7 + [one, None]
    assert L.msaq_kv_decode_attention(*args, 6, 4, 10, 128, 4, 4, 2, -1, None, 0, None) == -1   # H % Hkv
    assert L.msaq_kv_decode_attention(*args, 4, 4, 10, 128, 4, 4, 2, 5, None, 0, None) == -1    # Lcap < Lk
    assert L.msaq_hadamard_rotate(one, one, 4, 48, None) == -2
    assert L.msaq_pack_weight(one, 1, one, one, one, one, one, 8, 40, 4, 2, None) == -1  # K % 32


def test_new_entry_points_validate_before_the_device():
    """The tensor-parallel exchange, the GEMV with the push inside, the GEMV with the residual add behind it and the
    decode with the append inside: sizes and arguments are checked before anything touches a device."""
    import ctypes as C
    from ms_kernel_b200 import _lib
    L = _lib.lib()
    one = 16
    assert L.msaq_peer_exchange_bytes(2, 8192) == 4 * 2 * 8192 * 4 + 256
    assert L.msaq_peer_exchange_bytes(8, 4) == 4 * 8 * 4 * 4 + 256
    assert L.msaq_peer_exchange_bytes(1, 8192) == 0 and L.msaq_peer_exchange_bytes(9, 8192) == 0
    assert L.msaq_peer_exchange_bytes(2, 0) == 0
    bufs = (C.c_void_p * 8)(*([one] * 8))
    assert L.msaq_peer_exchange(one, None, None, bufs, 0, 2, 8192, 0, None) == -1          # no output
    assert L.msaq_peer_exchange(one, None, one, bufs, 2, 2, 8192, 0, None) == -1           # rank outside the world
    assert L.msaq_peer_exchange(one, None, one, bufs, 0, 9, 8192, 0, None) == -1           # more than eight ranks
    assert L.msaq_peer_exchange(one, None, one, bufs, 0, 2, 8190, 0, None) == -1           # n not a multiple of 4
    assert L.msaq_peer_exchange(one, None, one, bufs, 0, 2, 8192, 2, None) == -1           # parity
    assert L.msaq_peer_exchange(one + 4, None, one, bufs, 0, 2, 8192, 0, None) == -1       # misaligned partial
    bad = (C.c_void_p * 8)(one, None)
    assert L.msaq_peer_exchange(one, None, one, bad, 0, 2, 8192, 0, None) == -1            # a peer buffer is missing
    args = [one, 0, None, 0, 1e-5, None, one, one, one, 1, 256, 8, 4, 2]
    assert L.msaq_wonly_gemv_fused_push(*args, bufs, 0, 1, 0, one, 1 << 20, None) == -1    # one rank is no exchange
    assert L.msaq_wonly_gemv_fused_push(*args, bufs, 0, 2, 3, one, 1 << 20, None) == -1    # parity
    assert L.msaq_wonly_gemv_fused_push(*args, None, 0, 2, 0, one, 1 << 20, None) == -1    # no buffers
    assert L.msaq_wonly_gemv_fused_add(one, 3, 1e-5, one, one, one, one, one, 1, 256, 8, 4, 2, one, 1 << 20, None) == -1   # add+rmsnorm is not a prologue here
    assert L.msaq_wonly_gemv_fused_add(one, 0, 1e-5, one, one, one, None, one, 1, 256, 8, 4, 2, one, 1 << 20, None) == -1  # no residual
    dec = [one] * 3 + [one] * 6 + [one, None, None, 2, 8, 8, 64, 128, 4, 4, 2, 64, 1, 1, None, None, 0]
    assert L.msaq_kv_decode_attention_append(*dec, 64, None, one, 1 << 20, None) == -1     # slot beyond the capacity
    assert L.msaq_kv_decode_attention_append(*dec, -1, None, one, 1 << 20, None) == -1     # negative slot
    dec[1] = None
    assert L.msaq_kv_decode_attention_append(*dec, 3, None, one, 1 << 20, None) == -1      # no new K row


def test_no_fallback_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from ms_kernel_b200 import _lib
    L = _lib.lib()
    one = 8
    rc = L.msaq_wonly_gemv_wide(one, one, one, one, one, None, 8, 2, 4, 2, one, 1 << 20, None)
    assert rc == -5 and b"sm_100a" in L.msaq_last_error()


def test_operator_module_registers_reference_schemas():
    import torch
    from ms_kernel_b200 import ops
    assert ops.available(), ops._IMPORT_ERROR
    want = {
        "wonly_gemv": "msaq::wonly_gemv(Tensor x, Tensor scale_exp, Tensor upper, Tensor shared, int OUT, int NB, int u, int gs) -> Tensor",
        "wonly_gemv_wide": "msaq::wonly_gemv_wide(Tensor x, Tensor scale_exp, Tensor upper_cm, Tensor shared_cm, int OUT, int NB, int u, int gs) -> Tensor",
        "wonly_gemv_batched": "msaq::wonly_gemv_batched(Tensor x, Tensor scale_exp, Tensor upper_cm, Tensor shared_cm, int M, int OUT, int NB, int u, int gs) -> Tensor",
        "kv_write": "msaq::kv_write(Tensor X, int H, int L, int D, int NB, int u, int gs) -> Tensor[]",
        "kv_append": "msaq::kv_append(Tensor X, Tensor(a!) scale_exp, Tensor(b!) upper, Tensor(c!) shared, int H, int D, int NB, int pos, int Lcap, int u, int gs) -> ()",
        "kv_append_rot": "msaq::kv_append_rot(Tensor X, Tensor(a!) scale_exp, Tensor(b!) upper, Tensor(c!) shared, int H, int D, int NB, int pos, int Lcap, int u, int gs) -> ()",
        "kv_decode_attention": "msaq::kv_decode_attention(Tensor q, Tensor ks, Tensor ku, Tensor kh, Tensor vs, Tensor vu, Tensor vh, int H, int Hkv, int Lk, int D, int NB, int u, int gs, int Lcap=-1) -> Tensor",
        "kv_decode_attention_batched": "msaq::kv_decode_attention_batched(Tensor q, Tensor ks, Tensor ku, Tensor kh, Tensor vs, Tensor vu, Tensor vh, int B, int H, int Hkv, int Lk, int D, int NB, int u, int gs, int Lcap=-1) -> Tensor",
        "hadamard_rotate": "msaq::hadamard_rotate(Tensor x) -> Tensor",
    }
    for name, schema in want.items():
        got = str(getattr(torch.ops.msaq, name).default._schema)
        assert got == schema, got
    # ops refuse CPU tensors loudly
    with pytest.raises(RuntimeError):
        torch.ops.msaq.hadamard_rotate(torch.zeros(4, 128, dtype=torch.bfloat16))

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

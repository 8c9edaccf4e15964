"""ctypes binding of the C ABI in include/msaq_b200.h.

`lib()` loads libmsaq_b200.so from this directory and declares every entry
point; a missing library raises, there is no fallback implementation.
"""

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmsaq_b200.so")

_p, _i64, _int, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_size_t

# name -> (restype, argtypes); mirrors include/msaq_b200.h declaration by declaration
SIGNATURES = {
    "msaq_version": (_int, []),
    "msaq_last_error": (C.c_char_p, []),
    "msaq_launch_count": (C.c_ulonglong, []),
    "msaq_set_option": (_int, [_int, _int]),
    "msaq_get_option": (_int, [_int]),
    "msaq_wait_status": (_int, [_int, _p, C.POINTER(C.c_int)]),
    "msaq_wonly_gemv_workspace": (_sz, [_i64, _i64, _i64, _int, _int]),
    "msaq_wonly_gemv": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _int, _int, _p, _sz, _p]),
    "msaq_wonly_gemv_wide": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _int, _int, _p, _sz, _p]),
    "msaq_wonly_gemv_batched": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _int, _int, _p, _sz, _p]),
    "msaq_wonly_gemv_fused_workspace": (_sz, [_i64, _i64, _i64, _int, _int]),
    "msaq_wonly_gemv_fused": (_int, [_p, _int, _p, _int, C.c_float, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _int,
                                     _int, _p, _sz, _p]),
    "msaq_static_scratch_bytes": (_sz, []),
    "msaq_wonly_gemv_wide_static": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _int, _int, _p]),
    "msaq_kv_append": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _int, _int, _p]),
    "msaq_kv_append_rot": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _int, _int, _p]),
    "msaq_kv_append_varlen": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _p, _i64, _int, _int, _int, _p]),
    "msaq_kv_append_pair": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p, _i64, _int, _int,
                                   _int, _p]),
    "msaq_rope": (_int, [_p, _p, _i64, _i64, _i64, _p, _p, _i64, _i64, _p, _p]),
    "msaq_kv_append_pair_rope": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p, _i64, _int, _int,
                                        _int, _p, _p, _i64, _p]),
    "msaq_kv_write_rope": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int, _int, _p, _p, _i64, _p]),
    "msaq_kv_decode_attention_rope": (_int, [_p] * 7 + [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64,
                                                          _int, _int, _i64, _int, _p, _p, _i64, _i64, _p, _p, _sz, _p]),
    "msaq_kv_write": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int, _int, _p]),
    "msaq_hadamard_rotate": (_int, [_p, _p, _i64, _i64, _p]),
    "msaq_pack_weight": (_int, [_p, _int, _p, _p, _p, _p, _p, _i64, _i64, _int, _int, _p]),
    "msaq_kv_decode_workspace": (_sz, [_i64, _i64, _i64, _i64, _i64]),
    "msaq_kv_decode_attention": (_int, [_p] * 7 + [_p, _p, _i64, _i64, _i64, _i64, _i64, _int, _int, _i64,
                                                     _p, _sz, _p]),
    "msaq_kv_decode_attention_batched": (_int, [_p] * 7 + [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64,
                                                             _int, _int, _i64, _int, _p, _sz, _p]),
    "msaq_peer_exchange_bytes": (_sz, [_int, _i64]),
    "msaq_kv_decode_attention_append": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64,
                                               _i64, _int, _int, _i64, _int, _int, _p, _p, _i64, _i64, _p, _p, _sz, _p]),
    "msaq_wonly_gemv_fused_add": (_int, [_p, _int, C.c_float, _p, _p, _p, _p, _p, _i64, _i64, _i64, _int, _int, _p, _sz, _p]),
    "msaq_wonly_gemv_fused_push": (_int, [_p, _int, _p, _int, C.c_float, _p, _p, _p, _p, _i64, _i64, _i64, _int, _int,
                                          C.POINTER(_p), _int, _int, _int, _p, _sz, _p]),
    "msaq_peer_exchange": (_int, [_p, _p, _p, C.POINTER(_p), _int, _int, _i64, _int, _p]),
    "msaq_quant_act": (_int, [_p, _p, _p, _i64, _i64, _int, _int, _p]),
    "msaq_wa_gemv_workspace": (_sz, [_i64, _i64, _i64, _int, _int]),
    "msaq_wa_gemv": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _int, _int, _p, _sz, _p]),
    "msaq_wa_gemv_batched": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _int, _int, _p, _sz, _p]),
    "msaq_dequant_bf16": (_int, [_p, _p, _p, _p, _i64, _i64, _int, _int, _p]),
    "msaq_mxint8_pack_weight": (_int, [_p, _int, _p, _p, _p, _i64, _i64, _p]),
    "msaq_mxint8_gemv_workspace": (_sz, [_i64, _i64, _i64]),
    "msaq_mxint8_gemv_wide": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _sz, _p]),
    "msaq_mxint8_gemv_batched_wide": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _sz, _p]),
    "msaq_mxint8_kv_append": (_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p]),
    "msaq_mxint8_kv_write": (_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _p]),
    "msaq_mxint8_kv_decode_batched": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                             _p, _sz, _p]),
    "msaq_rmsnorm": (_int, [_p, _p, _i64, _i64, C.c_float, _p]),
    "msaq_silu_mul": (_int, [_p, _p, _i64, _i64, _p]),
    "msaq_add_residual": (_int, [_p, _p, _int, _p, _i64, _p]),
}

_LIB = None


class MsaqError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("msaq error %d: %s" % (code, message))
        self.code = code


def lib():
    """The loaded library with argtypes/restypes set."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "%s is missing: build it with `python -m ms_kernel_b200.build` "
                "(there is no CPU or PyTorch fallback for these kernels)" % LIB_PATH)
        h = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(h, name)
            fn.restype, fn.argtypes = res, args
        _LIB = h
    return _LIB


def check(rc):
    if rc != 0:
        raise MsaqError(rc, lib().msaq_last_error().decode("utf-8", "replace"))

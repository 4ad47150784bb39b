"""ctypes binding of ``libtpb200.so`` (the C ABI in ``include/tpb200.h``).

Loading fails loudly when the library has not been built: there is no
fallback implementation behind these functions.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libtpb200.so")

TPB_OK = 0
TPB_ERR_INVALID_ARG = -1
TPB_ERR_CUDA = -2
TPB_ERR_OOM = -3
TPB_ERR_TIMEOUT = -4
TPB_ERR_STATE = -5
TPB_ERR_NO_DEVICE = -6

TPB_F32, TPB_BF16, TPB_F16, TPB_S32 = 0, 1, 2, 3
GGUF_FMT = {"q8_0": 0, "q4_0": 1, "q4_k": 2, "q5_k": 3, "q6_k": 4, "iq4_nl": 5}

_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); every symbol the header declares.
SIGNATURES = {
    "tpb_version": (_i, []),
    "tpb_create": (_i, [C.POINTER(_vp), _i]),
    "tpb_destroy": (_i, [_vp]),
    "tpb_last_error": (C.c_char_p, [_vp]),
    "tpb_status_string": (C.c_char_p, [_i]),
    "tpb_status_poll": (_i, [_vp, _vp, C.POINTER(C.c_uint32)]),
    "tpb_device_sm_count": (_i, [_vp]),
    "tpb_convrot_prep": (_i, [_vp, _vp, _vp, _i, _i64, _i64, _i, _vp, _vp, _vp]),
    "tpb_convrot_gemm": (_i, [_vp, _vp, _vp, _i, _i64, _vp, _vp, _vp, _vp, _i, _vp, _i64, _i64, _i64]),
    "tpb_convrot_linear": (_i, [_vp, _vp, _vp, _i, _i64, _vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _i64, _i64, _i64]),
    "tpb_convrot_gemm_gated_add": (_i, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i64, _i64, _i64]),
    "tpb_convrot_gemm_silu_pair": (_i, [_vp, _vp, _vp, _i, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i64]),
    "tpb_convrot_gemm_group": (_i, [_vp, _vp, _i, _vp, _i, _i64, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i64]),
    "tpb_convrot_w4_reserve": (_i, [_vp, _i64, _i64]),
    "tpb_convrot_w4_expanded_bytes": (_sz, [_i64, _i64]),
    "tpb_convrot_w4_expand": (_i, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "tpb_q8_1_quantize": (_i, [_vp, _vp, _vp, _i64, _vp]),
    "tpb_q8_0_gemv_q8n": (_i, [_vp, _vp, _vp, _vp, _f, _i64, _i64, _vp, _i, _i, _i]),
    "tpb_q8_0_gemv_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _f, _i64, _i64]),
    "tpb_q8_0_gemv_static": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _f, _i64, _i64]),
    "tpb_stream_open": (_i, [_vp, _sz, _sz, _i, C.POINTER(_vp)]),
    "tpb_stream_close": (_i, [_vp]),
    "tpb_stream_register": (_i, [_vp, _i, _vp, _sz]),
    "tpb_stream_prefetch": (_i, [_vp, _i]),
    "tpb_stream_acquire": (_i, [_vp, _i, _vp, C.POINTER(_vp)]),
    "tpb_stream_release": (_i, [_vp, _i, _vp]),
    "tpb_stream_bytes_copied": (C.c_uint64, [_vp]),
    "tpb_stream_piece_bytes": (_sz, [_sz, _i]),
    "tpb_stream_prefetch_part": (_i, [_vp, _i, _i, _i, C.POINTER(_vp)]),
    "tpb_stream_commit": (_i, [_vp, _i]),
    "tpb_stream_transfer_stream": (_vp, [_vp]),
    "tpb_host_alloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "tpb_host_free": (_i, [_vp, _vp]),
    "tpb_silu_mul": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _i64]),
    "tpb_sigmoid_mul": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _i64]),
    "tpb_rms_mod": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _f, _i64, _i64]),
    "tpb_gated_add": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _i64, _i64]),
    "tpb_convrot_prep_fused": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _f, _i, _i64, _i64, _i, _vp, _vp, _vp]),
    "tpb_gguf_row_bytes": (_sz, [_i, _i64]),
    "tpb_gguf_gemv_q8n": (_i, [_vp, _vp, _i, _vp, _vp, _f, _i64, _i64, _vp, _i, _i, _i]),
    "tpb_attn_vt_elems": (_sz, [_i64, _i]),
    "tpb_attn_prepare": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _f, _vp, _vp, _i64, _i, _i, _i, _vp, _vp, _vp]),
    "tpb_attention": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _i64, _i64, _i, _i, _i, _f]),
    "tpb_peer_alloc": (_i, [_vp, _sz, C.POINTER(_vp), _vp]),
    "tpb_peer_open": (_i, [_vp, _vp, C.POINTER(_vp)]),
    "tpb_peer_close": (_i, [_vp, _vp]),
    "tpb_peer_free": (_i, [_vp, _vp]),
    "tpb_peer_barrier": (_i, [_vp, _vp, C.POINTER(_vp), _i, _i, C.c_uint32, _i]),
    "tpb_convrot_gemm_multi": (_i, [_vp, _vp, _vp, C.POINTER(_vp), _i, _i, _i64, _vp, _vp, _vp, _vp, _i, _vp,
                                    _i64, _i64, _i64]),
    "tpb_convrot_gemm_allgather_mc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i64, _vp, _vp, _vp, _vp, _i, _vp,
                                           _i64, _i64, _i64]),
    "tpb_convrot_gemm_allgather": (_i, [_vp, _vp, C.POINTER(_vp), _i, _i, _i, _i64, _vp, _vp, _vp, _vp, _i, _vp,
                                        _i64, _i64, _i64]),
}

_lib = None


class TpbError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"tpb200 status {status}: {message}")
        self.status = status


def load() -> C.CDLL:
    """Load the library and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m tensorpencil_b200.build`. "
            "tensorpencil_b200 has no fallback path without its CUDA library.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib

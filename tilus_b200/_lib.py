"""ctypes binding of libb200q.so (the C ABI declared in include/b200q.h).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, os.environ.get("B200Q_LIB_NAME", "libb200q.so"))

ST_OK, ST_INVALID_ARG, ST_UNSUPPORTED, ST_WORKSPACE, ST_CUDA, ST_DEVICE_TIMEOUT = range(6)
ACT_F16, ACT_BF16 = 0, 1


class B200QError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"b200q status {status}: {message}")
        self.status = status


GATHER_FLAGS, GATHER_TAGGED = 0, 1  # b200q_gather_t.mode


class Gather(ctypes.Structure):
    """b200q_gather_t of include/b200q.h."""
    _fields_ = [
        ("world", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("ldc", ctypes.c_int32),
        ("col_offset", ctypes.c_int32),
        ("out", ctypes.c_void_p * 8),
        ("flag_slot", ctypes.c_void_p * 8),
        ("flags_local", ctypes.c_void_p),
        ("epoch_local", ctypes.c_void_p),
        ("buffer_elems", ctypes.c_int64),
        ("a_prev_offset", ctypes.c_int64),
        ("mode", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
    ]


class Plan(ctypes.Structure):
    _fields_ = [
        ("kernel", ctypes.c_int32),
        ("m_tiles", ctypes.c_int32),
        ("splits", ctypes.c_int32),
        ("cluster", ctypes.c_int32),
        ("ctas_per_split", ctypes.c_int32),
        ("smem_bytes", ctypes.c_int32),
        ("tile_m", ctypes.c_int32),
        ("stages", ctypes.c_int32),
        ("warps", ctypes.c_int32),
        ("passes", ctypes.c_int32),
        ("pdl", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("workspace_bytes", ctypes.c_uint64),
    ]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


# every symbol include/b200q.h declares: name -> (restype, argtypes)
_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
SYMBOLS = {
    "b200q_version": (_i, []),
    "b200q_layout_version": (_i, []),
    "b200q_status_string": (ctypes.c_char_p, [_i]),
    "b200q_last_cuda_error": (_i, []),
    "b200q_plan": (_i, [_i, _i, _i, _i, _i, _i, ctypes.POINTER(Plan)]),
    "b200q_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "b200q_gemm": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "b200q_gemm_planned": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp,
                                ctypes.POINTER(Plan)]),
    "b200q_gemm_static_ws": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "b200q_gemm_host": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "b200q_static_workspace_limit": (_sz, []),
    "b200q_static_ws_init": (_i, []),
    "b200q_dequantize": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "b200q_gemm_gather": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp, ctypes.POINTER(Gather)]),
    "b200q_gather_push": (_i, [_vp, _i, _i, _i, _vp, _sz, _vp, ctypes.POINTER(Gather)]),
    "b200q_gather_collect": (_i, [_vp, _i, _i, _vp, _sz, _vp, ctypes.POINTER(Gather)]),
    "b200q_peer_alloc": (_i, [_sz, ctypes.POINTER(ctypes.c_void_p)]),
    "b200q_peer_export": (_i, [_vp, ctypes.c_char_p]),
    "b200q_peer_open": (_i, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
    "b200q_peer_close": (_i, [_vp]),
    "b200q_peer_free": (_i, [_vp]),
    "b200q_quantize": (_i, [_vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "b200q_per_token_cast": (_i, [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _vp]),
    "b200q_swiglu_per_token_cast": (_i, [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _i, ctypes.c_float, _vp]),
    "b200q_gemm_swiglu_cast": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i,
                                    ctypes.c_float, _vp, _sz, _vp]),
    "b200q_device_status": (_i, [_vp, ctypes.POINTER(ctypes.c_int32 * 4), _vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load libb200q.so; raises if it has not been built (python -m tilus_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m tilus_b200.build` "
            "(nvcc, sm_100a). There is no CPU fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != ST_OK:
        lib = load()
        msg = lib.b200q_status_string(status).decode()
        if status == ST_CUDA:
            msg += f" (cudaError {lib.b200q_last_cuda_error()})"
        raise B200QError(status, msg)

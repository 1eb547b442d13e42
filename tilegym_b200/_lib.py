"""ctypes binding of libtilegym_b200.so (the C ABI declared in include/tilegym_b200.h).

The library is the only implementation of every operator in this package:
there is no fallback.  If the shared object is missing, importing the package
works (so that build tooling can import it) but the first operator call raises.
The binding follows the convention of the reference's own FFI loader
(src/tilegym/backend/cutile_rs/utils.py:241-290, 366-370): tensors cross as
descriptor structs, a non-zero return code becomes a RuntimeError.
"""

from __future__ import annotations

import ctypes
import struct
import os
from typing import Optional

import torch

LIB_NAME = "libtilegym_b200.so"
LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)

TG_OK = 0
ERR_NAMES = {
    -2: "UNSUPPORTED_DTYPE",
    -3: "LAUNCH_FAILED",
    -4: "DEVICE_INIT_FAILED",
    -5: "NULL_POINTER",
    -6: "INVALID_ARGS",
    -7: "TIMEOUT",
    -8: "MISALIGNED",
}

# dtype codes of the reference FFI (src/tilegym/ops/cutile_rs/ffi_util.rs:26-35)
DTYPE_CODES = {
    torch.float32: 0,
    torch.float16: 1,
    torch.bfloat16: 2,
    torch.int32: 3,
    torch.int64: 4,
    torch.float8_e5m2: 5,
    torch.uint8: 6,
    torch.float8_e4m3fn: 7,
    torch.int8: 8,  # extension: the reference table stops at 7
}


class TensorDesc(ctypes.Structure):
    _fields_ = [
        ("ptr", ctypes.c_uint64),
        ("ndim", ctypes.c_int32),
        ("shape", ctypes.c_int64 * 5),
        ("strides", ctypes.c_int64 * 5),
        ("dtype", ctypes.c_int32),
    ]


class TileGymB200Error(RuntimeError):
    def __init__(self, rc: int, msg: str):
        super().__init__(f"tilegym_b200: {ERR_NAMES.get(rc, 'ERROR')} ({rc}): {msg}")
        self.rc = rc


_lib: Optional[ctypes.CDLL] = None

# name -> (restype, argtypes); the list the symbol-export test walks.
_P = ctypes.c_char_p  # const TgTensorDesc*, passed as the packed bytes of desc()
SIGNATURES = {
    "tg_version": (ctypes.c_int32, []),
    "tg_plan_splits": (
        ctypes.c_int32,
        [ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
         ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)],
    ),
    "tg_set_static_weights": (ctypes.c_int32, [ctypes.c_int32]),
    "tg_last_error_string": (ctypes.c_char_p, []),
    "tg_fp8_gemm_workspace_bytes": (ctypes.c_uint64, [ctypes.c_int64] * 3),
    "tg_fp8_gemm_pertensor": (
        ctypes.c_int32,
        [_P, _P, _P, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float, _P, ctypes.c_float, ctypes.c_uint64,
         ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_fp8_gemm_pertensor_allgather": (
        ctypes.c_int32,
        [_P, _P, _P, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float, _P, ctypes.POINTER(ctypes.c_uint64),
         ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_shard_gemm_allgather": (
        ctypes.c_int32,
        [_P, _P, _P, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float, _P, ctypes.c_int32, ctypes.c_int32,
         ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_fp8_gemm_pertensor_smallm_static": (
        ctypes.c_int32,
        [_P, _P, _P, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float, _P, ctypes.c_float, ctypes.c_int32,
         ctypes.c_uint64],
    ),
    "tg_fp8_gemm_blockscaled": (
        ctypes.c_int32,
        [_P, _P, _P, _P, _P, ctypes.c_int32, ctypes.c_int32, _P, ctypes.c_float, ctypes.c_uint64, ctypes.c_uint64,
         ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_fp8_gemm_pertensor_swiglu": (
        ctypes.c_int32,
        [_P, _P, _P, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float, _P, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_gemm_dense16": (
        ctypes.c_int32,
        [_P, _P, _P, ctypes.c_float, _P, ctypes.c_float, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_fp8_gemm_blockscaled_grouped": (
        ctypes.c_int32,
        [_P, _P, _P, _P, _P, ctypes.c_uint64, ctypes.c_int32, ctypes.c_int32, _P, ctypes.c_float, ctypes.c_uint64,
         ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_fp8_gemm_blockscaled_grouped_swiglu": (
        ctypes.c_int32,
        [_P, _P, _P, _P, _P, _P, ctypes.c_uint64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_moe_route": (
        ctypes.c_int32,
        [_P, _P, ctypes.c_int32, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64,
         ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_moe_permute_rows": (
        ctypes.c_int32,
        [_P, _P, _P, _P, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_moe_quant_permute_rows": (
        ctypes.c_int32, [_P, _P, _P, ctypes.c_uint64, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_moe_silu_mul_quant": (
        ctypes.c_int32,
        [_P, _P, _P, ctypes.c_uint64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_moe_unpermute_sum": (
        ctypes.c_int32, [_P, _P, ctypes.c_uint64, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_act_quant": (ctypes.c_int32, [_P, _P, _P, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64]),
    "tg_per_token_group_quant": (
        ctypes.c_int32,
        [_P, _P, _P, ctypes.c_int32, ctypes.c_float, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_weight_dequant": (ctypes.c_int32, [_P, _P, _P, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64]),
    "tg_quant_pertensor": (
        ctypes.c_int32,
        [_P, ctypes.c_uint64, _P, ctypes.c_uint64, ctypes.c_int32, ctypes.c_uint64],
    ),
    "tg_weight_quant_block": (ctypes.c_int32, [_P, _P, _P, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64]),
    "tg_device_status": (ctypes.c_int32, [ctypes.c_int32, ctypes.POINTER(ctypes.c_int32)]),
    "tg_reload_env": (None, []),
    "tg_set_wait_limit_us": (ctypes.c_uint32, [ctypes.c_uint32]),
    "tg_selftest_wait_timeout": (ctypes.c_int32, [ctypes.c_uint32, ctypes.c_int32, ctypes.c_uint64]),
    "tg_selftest_quant16": (ctypes.c_int32, [ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64, ctypes.c_int32, ctypes.c_uint64]),
}


def lib() -> ctypes.CDLL:
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m tilegym_b200.build` "
                "(there is no fallback implementation)"
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


# The descriptor is marshalled with one struct.pack call (about half the cost of filling a ctypes Structure
# field by field); the packed bytes have exactly the layout of TensorDesc / TgTensorDesc.
_DESC = struct.Struct("Qi4x5q5qi4x")
assert _DESC.size == ctypes.sizeof(TensorDesc)
_PAD = ((), (0,), (0, 0), (0, 0, 0), (0, 0, 0, 0), (0, 0, 0, 0, 0))


def desc(t: Optional[torch.Tensor]) -> Optional[bytes]:
    """Descriptor of a tensor as the bytes of a TgTensorDesc (None passes through as a NULL pointer)."""
    if t is None:
        return None
    nd = t.dim()
    if nd > 5:
        raise ValueError("tensors of more than 5 dimensions are not supported")
    code = DTYPE_CODES.get(t.dtype)
    if code is None:
        raise TileGymB200Error(-2, f"dtype {t.dtype} has no code in the C ABI")
    pad = _PAD[5 - nd]
    return _DESC.pack(t.data_ptr(), nd, *t.shape, *pad, *t.stride(), *pad, code)


def desc2d(ptr: int, rows: int, cols: int, row_stride: int, dtype: torch.dtype) -> bytes:
    """Descriptor of a row-major 2-D view given by numbers (saves creating the view tensor)."""
    return _DESC.pack(ptr, 2, rows, cols, 0, 0, 0, row_stride, 1, 0, 0, 0, DTYPE_CODES[dtype])


def ref(d: Optional[bytes]):
    """What is passed for a `const TgTensorDesc*` argument: the packed bytes themselves (ctypes passes a
    pointer to them and keeps them alive for the call), or None for NULL."""
    return d


def check_rc(rc: int) -> None:
    if rc != TG_OK:
        raise TileGymB200Error(rc, lib().tg_last_error_string().decode("utf-8", "replace"))


def device_status(device_index: int) -> None:
    """Synchronises the device and raises if a kernel's bounded wait expired."""
    detail = ctypes.c_int32(0)
    check_rc(lib().tg_device_status(device_index, ctypes.byref(detail)))


def set_knob(name: str, value) -> None:
    """Sets (value) or removes (None) a TILEGYM_B200_* tuning variable and makes the library re-read them
    (it reads the environment once, not per launch)."""
    if value is None:
        os.environ.pop(name, None)
    else:
        os.environ[name] = str(value)
    lib().tg_reload_env()

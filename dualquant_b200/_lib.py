"""ctypes binding of libdualquant_b200.so (the C ABI declared in include/dualquant_b200.h).

The library is the only compute path: if it cannot be loaded, or the device is not sm_100,
every op raises -- there is no fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("DUALQUANT_B200_LIB", os.path.join(_PKG, "lib", "libdualquant_b200.so"))

DQ_OK = 0
DQ_ERR_TIMEOUT = 9
DTYPE_F32, DTYPE_BF16 = 0, 1
CODES_E4M3 = 0x100  # or-ed into scale_fp16: the quantiser writes E4M3 code bytes
HAD_NONE, HAD_FULL, HAD_PARTIAL = 0, 1, 2
FP4_MXFP4, FP4_NVFP4 = 0, 1

_ERR_NAMES = {
    1: "DQ_ERR_SHAPE", 2: "DQ_ERR_ALIGN", 3: "DQ_ERR_NULL", 4: "DQ_ERR_ARCH", 5: "DQ_ERR_CUDA",
    6: "DQ_ERR_WORKSPACE", 7: "DQ_ERR_UNSUPPORTED", 8: "DQ_ERR_NOT_INIT", 9: "DQ_ERR_TIMEOUT",
}
# argument errors surface as ValueError (the reference raises ValueError / AssertionError for
# bad shapes, formats/__init__.py:30-36); everything else as RuntimeError
_VALUE_ERRORS = {1, 2, 3, 6, 7}


class HadamardDesc(ctypes.Structure):
    _fields_ = [
        ("kind", ctypes.c_int32),
        ("had_k", ctypes.c_int32),
        ("had_dim", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("had_mat", ctypes.c_void_p),
    ]


_c = ctypes
_vp, _i, _i64, _sz = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_size_t
_hp = _c.POINTER(HadamardDesc)

# name -> (restype, argtypes); must list every symbol the header declares
class AllReduceCtx(ctypes.Structure):
    """dq_allreduce_ctx of the header."""
    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("buf_ptrs", ctypes.c_void_p * 8), ("flag_ptrs", ctypes.c_void_p * 8),
                ("seq", ctypes.c_void_p), ("buf_capacity_floats", ctypes.c_uint64),
                ("flag_units", ctypes.c_uint64)]


class ExchangeCtx(ctypes.Structure):
    """dq_exchange_ctx of the header."""
    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("part_ptrs", ctypes.c_void_p * 8), ("codes_ptrs", ctypes.c_void_p * 8),
                ("sx_ptrs", ctypes.c_void_p * 8), ("flag_ptrs", ctypes.c_void_p * 8),
                ("tokens_per_rank", ctypes.c_int64), ("hidden", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("barrier_count", ctypes.c_void_p)]


SIGNATURES = {
    "dq_init": (_i, [_i]),
    "dq_last_error_string": (_c.c_char_p, []),
    "dq_device_status": (_i, [_i]),
    "dq_abi_version": (_i, []),
    "dq_set_tuning": (_i, [_c.c_char_p, _i]),
    "dq_mma_peak_probe": (_i, [_i, _i, _c.POINTER(_c.c_double), _vp]),
    "dq_packed_w_bytes": (_sz, [_i, _i]),
    "dq_pack_w_int4": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "dq_unpack_w_int4": (_i, [_vp, _i, _i, _vp, _vp]),
    "dq_quant_w_int4": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "dq_quant_act_int4": (_i, [_vp, _i64, _vp, _hp, _i, _i, _vp, _vp, _i, _vp]),
    "dq_quant_act_int4_f32": (_i, [_vp, _i64, _vp, _hp, _i, _i, _vp, _vp, _i, _vp]),
    "dq_quant_act_int4_rmsnorm": (_i, [_vp, _i64, _vp, ctypes.c_float, _vp, _i, _i, _vp, _vp, _i, _vp]),
    "dq_quant_act_int4_gated": (_i, [_vp, _vp, _i64, _vp, _hp, _i, _i, _vp, _vp, _i, _vp]),
    "dq_fakequant_act_int4": (_i, [_vp, _i, _i64, _vp, _hp, _i, _i, _vp, _i, _vp]),
    "dq_fakequant_act_int4_bf16": (_i, [_vp, _i64, _i, _i, _vp, _vp]),
    "dq_hadamard_f32": (_i, [_vp, _vp, _i, _i, _hp, _vp]),
    "dq_quant_fp4": (_i, [_vp, _i, _i64, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "dq_quant_fp4_atoms": (_i, [_vp, _i, _i64, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "dq_fakequant_fp4": (_i, [_vp, _i, _i64, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "dq_nvfp4_tensor_scale": (_i, [_vp, _i, _i64, _vp, _vp]),
    "dq_fp4_sf_atoms_bytes": (_sz, [_i, _i, _i]),
    "dq_fp4_sf_to_atoms": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "dq_gemm_w4a4_fp4": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp]),
    "dq_gemm_w4a4_fp4_tiled": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _i, _vp]),
    "dq_gemm_w4a4_int4_workspace_bytes": (_sz, [_i, _i, _i]),
    "dq_gemm_w4a4_int4": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _sz, _vp]),
    "dq_quant_act_int4_grouped": (_i, [_vp, _i64, _vp, _i, _i, _i, _vp, _vp, _i, _i, _vp]),
    "dq_gemm_w4a4_int4_grouped": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp]),
    "dq_expand_w_int4_e4m3": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "dq_codes_to_e4m3": (_i, [_vp, _i64, _i, _i, _vp, _vp]),
    "dq_gemm_w4a4_int4_e4m3": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _vp]),
    "dq_gemm_w4a4_int4_residual": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp]),
    "dq_gemm_w4a4_int4_ex": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _sz, _vp, _i, _i]),
    "dq_gemm_w4a4_int4_ar": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _vp]),
    "dq_gemm_w4a4_int4_ar_residual": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _vp]),
    "dq_gemm_w4a4_int4_acc": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "dq_gemm_w4a4_int4_e4m3_scatter": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "dq_exchange_barrier": (_i, [_vp, _c.c_uint32, _vp]),
    "dq_exchange_sum": (_i, [_vp, _vp, _vp]),
    "dq_exchange_push": (_i, [_vp, _vp, _vp, _vp]),
    "dq_linear_w4a4_int4_scratch_bytes": (_sz, [_i, _i, _i]),
    "dq_linear_w4a4_int4_prefill_scratch_bytes": (_sz, [_i, _i, _i]),
    "dq_linear_w4a4_int4": (_i, [_vp, _i64, _vp, _hp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _i, _vp, _sz, _vp]),
    "dq_rope_kv_append": (_i, [_vp, _i64, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "dq_linear_a16w4_scratch_bytes": (_sz, [_i, _i, _i]),
    "dq_linear_a16w4": (_i, [_vp, _i64, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp, _sz, _vp]),
    "dq_linear_w4a4_int4_static_max_bytes": (_sz, []),
    "dq_linear_w4a4_int4_static": (_i, [_vp, _i64, _vp, _hp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _i, _vp]),
}

_lib = None
_lock = threading.Lock()
_inited = set()


def load():
    """Loads the shared library (once) and binds every signature."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dualquant_b200.build` "
                "(nvcc, sm_100a). dualquant_b200 has no other compute path."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().dq_last_error_string().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc == DQ_OK:
        return
    code = rc & 0xFFFF
    msg = f"{what}: {_ERR_NAMES.get(code, code)}: {last_error()}"
    if code in _VALUE_ERRORS:
        raise ValueError(msg)
    raise RuntimeError(msg)


def ensure_init(device_index: int) -> None:
    """dq_init for `device_index` (must be the current CUDA device)."""
    if device_index in _inited:
        return
    lib = load()
    check(lib.dq_init(int(device_index)), f"dq_init({device_index})")
    _inited.add(device_index)


def set_tuning(name: str, value: int) -> None:
    """Launch-shape override (see dq_set_tuning in the header); for sweeps and tests."""
    check(load().dq_set_tuning(name.encode(), int(value)), f"dq_set_tuning({name})")


def device_status(device_index: int) -> None:
    """Synchronises and raises if a bounded device-side wait expired since the last call."""
    check(load().dq_device_status(int(device_index)), "dq_device_status")

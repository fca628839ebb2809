"""ctypes binding of libquarot_b200.so (the C-ABI declared in include/quarot_b200.h).

The library is built in-tree by ``python quarot_b200/build.py``.  There is no
fallback: if it is missing, importing this module raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libquarot_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "quarot_b200: %s not found -- build it with `python quarot_b200/build.py` "
        "(needs nvcc with sm_100a support); there is no non-CUDA fallback" % LIB_PATH)

lib = ctypes.CDLL(LIB_PATH)

_vp, _i64, _int, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float

# name -> (restype, argtypes); must list every symbol of include/quarot_b200.h
SIGNATURES = {
    "qr_version": (_int, []),
    "qr_last_error": (ctypes.c_char_p, []),
    "qr_kernel_status": (_int, [ctypes.POINTER(_int)]),
    "qr_set_tuning": (_int, [ctypes.c_char_p, _int]),
    "qr_debug_division_check": (_int, [ctypes.POINTER(ctypes.c_uint64)]),
    "qr_hadamard_f16": (_int, [_vp, _vp, _i64, _i64, _vp, _int, _vp]),
    "qr_hadamard_f32": (_int, [_vp, _vp, _i64, _i64, _vp, _int, _vp]),
    "qr_hadamard_heads_f16": (_int, [_vp, _vp, _i64, _i64, _i64, _vp]),
    "qr_hadamard_quant_i4": (_int, [_vp, _i64, _i64, _i64, _vp, _int, _f32, _vp, _vp, _vp, _vp]),
    "qr_sym_quant_i4": (_int, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "qr_matmul_i4_i32": (_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "qr_sym_dequant_i32_f16": (_int, [_vp, _vp, _vp, _i64, _i64, _vp, _vp]),
    "qr_linear_i4_f16": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "qr_linear_i4_f16_outs": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, ctypes.POINTER(ctypes.c_void_p), _int, _i64, _vp]),
    "qr_linear_i4_swiglu_f16": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "qr_rmsnorm_quant_i4": (_int, [_vp, _i64, _i64, _i64, _i64, ctypes.c_float, ctypes.c_float, _vp, _vp, _vp, _vp]),
    "qr_quant_linear_i4_f16": (_int, [_vp, _i64, ctypes.c_float, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "qr_kv_append_i4": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _int, _int, _int, _int, _int, _int, _int, _vp]),
    "qr_kv_decode_i4": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _int, _int, _int, _vp]),
    "qr_linear_workspace_bytes": (ctypes.c_size_t, [_i64, _i64, _i64]),
    "qr_linear_i4_f16_static": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "qr_linear_i4_f16_ws": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp, ctypes.c_size_t, _vp]),
}

for _name, (_res, _args) in SIGNATURES.items():
    if not hasattr(lib, _name):
        raise ImportError("quarot_b200: %s does not export %s -- it is stale, rebuild it with "
                          "`python quarot_b200/build.py`" % (LIB_PATH, _name))
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error():
    return lib.qr_last_error().decode("utf-8", "replace")


def check(rc, what):
    """Turn a non-zero status into the RuntimeError upstream raises from TORCH_CHECK."""
    if rc != 0:
        raise RuntimeError("%s failed (status %d): %s" % (what, rc, last_error()))


def kernel_status():
    """Device status word (0 = no kernel ever gave up on a bounded wait); reading clears it.  On a non-zero
    status the cached scratch buffers are dropped, since the kernel may have left counters behind in them."""
    out = _int(0)
    check(lib.qr_kernel_status(ctypes.byref(out)), "qr_kernel_status")
    if out.value != 0:
        from . import _ops
        _ops.reset_workspaces()
    return out.value


def set_tuning(key, value):
    check(lib.qr_set_tuning(key.encode(), int(value)), "qr_set_tuning")

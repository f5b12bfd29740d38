"""Host build of the device integer library (csrc/sslm_int.cuh), for CPU-side checks."""
import ctypes as C
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "libint_host.so")
SRC = os.path.join(HERE, "int_host_shim.cpp")
HDR = os.path.join(HERE, "..", "..", "superslm_b200", "csrc", "sslm_int.cuh")
_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if (not os.path.exists(SO) or os.path.getmtime(SO) < max(os.path.getmtime(SRC), os.path.getmtime(HDR))):
        subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-x", "c++", "-o", SO, SRC], check=True)
    d = C.CDLL(SO)
    i64, i32, P64, PI = C.c_int64, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int)
    sig = {
        "dev_srdhm": (i32, [i32, i32]), "dev_rdivpot32": (i32, [i32, C.c_int]), "dev_rdivpot64": (i64, [i64, C.c_int]),
        "dev_fold": (i32, [i32] * 4), "dev_amp_fold": (i32, [i32] * 4),
        "dev_fold_epilogue": (i32, [i32] * 4 + [PI, C.POINTER(C.c_uint32)]),
        "dev_normalize_scale": (None, [i64, P64, PI]), "dev_dyn_recip": (i64, [i64]),
        "dev_requant_code": (C.c_int8, [i64, i64, C.c_int]),
        "dev_code_of64": (C.c_int8, [i64, i64, C.c_int]), "dev_code_of32": (C.c_int8, [i32, i64, C.c_int]),
        "dev_combine": (None, [i64] * 4 + [P64, P64]),
        "dev_funnel_params": (C.c_int, [C.c_uint64, C.c_void_p, C.c_int, i64, i64, P64, PI, P64, P64]),
        "dev_floor_div": (i64, [i64, i64]), "dev_floor_div_h32": (i64, [C.c_int, i64]), "dev_udiv_small": (C.c_uint64, [C.c_uint64] * 2),
        "dev_isqrt": (i64, [i64]), "dev_landing_rescale": (i64, [i64] * 5 + [PI, PI]),
        "dev_rope_pair": (None, [i32] * 4 + [C.POINTER(C.c_int8)] * 2),
        "dev_silu": (i32, [C.c_void_p, i32, i64, C.c_int]),
        "dev_iexp_scale_constants": (C.c_int, [i64, i64, P64, P64, P64]),
        "dev_softmax_width": (C.c_int, [i64, i64, C.c_uint64, P64]),
        "dev_iexp_element": (C.c_int, [i64] * 5 + [P64]),
        "dev_bias_reconcile": (C.c_int, [i64] * 3 + [P64]),
        "dev_bias_accumulate": (C.c_int, [i64] * 2 + [P64]),
        "dev_dyn_recip_sweep": (i64, [i64, i64, i64, P64]),
    }
    for n, (r, a) in sig.items():
        f = getattr(d, n)
        f.restype, f.argtypes = r, a
    _lib = d
    return d

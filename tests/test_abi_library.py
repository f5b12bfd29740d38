"""CPU-side checks of the product library: it builds for sm_100a, loads without a GPU, and
exports every entry point that include/sslm_b200.h declares (no compute call is made)."""
import ctypes as C
import os
import re
import subprocess

from superslm_b200 import abi, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_entry_points():
    text = open(os.path.join(ROOT, "include", "sslm_b200.h")).read()
    return sorted(set(re.findall(r"SSLM_API\s+\w+\s+(sslm_\w+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    names = declared_entry_points()
    assert len(names) >= 24
    dll = C.CDLL(path)
    for n in names:
        assert hasattr(dll, n), n
    exported = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True).stdout
    public = sorted(set(re.findall(r" T (sslm_\w+)", exported)))
    assert public == names          # nothing undeclared leaks out, nothing declared is missing


def test_reference_verbs_are_all_bound():
    for verb in abi.SslmLib.VERBS:
        assert verb in declared_entry_points()


def test_product_does_not_reference_the_oracle():
    """The shipped path must not import, link or call anything under oracle/."""
    pkg = os.path.join(ROOT, "superslm_b200")
    for dirpath, _dirs, files in os.walk(pkg):
        if os.path.basename(dirpath) == "build":
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp", ".inc")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "oracle" not in text.replace("the CPU oracle", "").lower() or f == "abi.py" and "oracle" not in text, (dirpath, f)
    needed = subprocess.run(["ldd", build.LIB], capture_output=True, text=True).stdout
    assert "oracle" not in needed and "sslm_ref" not in needed


def test_calls_without_a_device_fail_loudly():
    """No CPU fallback: with no usable CUDA device a compute verb reports an error status."""
    import numpy as np
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    from superslm_b200 import artifact as A
    lib = abi.SslmLib(build.build())
    art = np.frombuffer(A.build_synthetic_model("tiny", 1, 16), dtype=np.uint8)
    h = abi._H()
    assert lib.sslm_model_map(art.ctypes.data, art.size, C.byref(h)) == abi.ST["SSLM_ALLOCATION_FAILED"]
    assert not h.value

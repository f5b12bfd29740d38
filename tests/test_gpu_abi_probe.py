"""The boundary seen from the reference's own header: tests/support/abi_probe.cpp is compiled
against include/superslm/sslm_abi.h of the reference tree (where that tree is mounted, by
oracle/Makefile's `probe` target) and linked against libsslm_b200.so. It drives map, pool,
workspace, sequence, chunked prefill, sliced decode and save exactly as a program written for the
reference does. Its tokens must equal the reference library's record for the same artifact and
prompt, and its save blob must equal, byte for byte, the one the ctypes binding gets."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

from oracle import harness as H
from superslm_b200 import abi, artifact as A

pytestmark = pytest.mark.gpu


def fnv1a64(data: bytes) -> int:
    h = 1469598103934665603
    for chunk_start in range(0, len(data), 1 << 16):
        for b in data[chunk_start:chunk_start + (1 << 16)]:
            h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def test_program_built_against_the_reference_header(gpu_lib, e2e_golden):
    if not os.path.exists(H.ABI_PROBE):
        pytest.skip("oracle/_ref/abi_probe not built (reference header absent)")
    case = e2e_golden["tiny"]
    sh = A.SHAPES[case["shape"]]
    art = A.build_synthetic_model(case["shape"], case["seed"], case["context_cap"], case["shift_lo"], case["shift_hi"])
    prompt = A.stream_uniform(case["seed"] ^ 0xABCDEF, "prompt", case["prompt_len"], 0, sh.vocab - 1).astype(np.int32)
    with tempfile.TemporaryDirectory() as tmp:
        apath, ppath = os.path.join(tmp, "model.sslm"), os.path.join(tmp, "prompt.i32")
        with open(apath, "wb") as f:
            f.write(art)
        prompt.tofile(ppath)
        out = subprocess.run([H.ABI_PROBE, apath, ppath, "7", "1", str(case["decode"])], capture_output=True, text=True,
                             timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = dict(l.split(" ", 1) for l in out.stdout.strip().splitlines())
    assert [int(t) for t in lines["tokens"].split()] == case["tokens"]
    # the same run through the ctypes binding: identical blob
    eng = abi.Engine(gpu_lib, art, blocks=1, max_chunk=7)
    s = eng.new_seq()
    s.prefill(prompt, 7)
    assert s.decode(case["decode"], 1) == case["tokens"]
    blob = s.save()
    eng.close()
    size, digest = lines["blob"].split()
    assert int(size) == len(blob)
    assert int(digest, 16) == fnv1a64(blob)

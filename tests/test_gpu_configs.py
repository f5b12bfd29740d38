"""The benchmark configurations at their stated shapes and context lengths, against the CPU reference.

tests/golden/config_golden.json holds what the reference library (compiled from its own sources)
produced for each case of tests/golden/config_cases.py: every decoded token, the SHA-256 of the
canonical K/V block (all layers, all positions), the carried hidden scale, the K/V saturation
counter, and the SHA-256 of full int32 logit rows. The CUDA path is run through the C ABI at
several (prefill chunk, layer budget) splits and must reproduce the record bit for bit at each.
Covered: the 0.5B shape in full (24 layers, 512 + 128 tokens), attention rows of 640, 2304 and
4608 positions at the 0.5B / 1.5B / 3B widths (GQA 7:1 at head_dim 64, 6:1 and 8:1 at 128), the
full 1.5B model on a 2048-token prompt, and rank-16 adapters swapped mid-run at the 3B widths.
"""
import ctypes as C
import hashlib
import json
import os
import struct

import numpy as np
import pytest

from config_cases import CASES, build_case_artifacts, case_prompt
from superslm_b200 import abi, artifact as A

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "config_golden.json")


@pytest.fixture(scope="module")
def golden():
    with open(GOLDEN) as f:
        return json.load(f)


def blob_fields(lib, seq, hidden):
    """Header fields and the K/V digest of a sequence's save blob, without copying the block around."""
    n = C.c_size_t(0)
    lib.sslm_seq_save(seq.handle, None, C.byref(n))
    buf = np.zeros(n.value, dtype=np.uint8)
    assert lib.sslm_seq_save(seq.handle, buf.ctypes.data_as(C.c_void_p), C.byref(n)) == 0
    ctx_len, layer_index, cur_tok, hm, he, sat = struct.unpack_from("<qIiqqQ", buf, 60)
    assert layer_index == 0
    off = 120 + 4
    return {"context_length": ctx_len, "hidden_scale": [hm, he], "kv_saturation_count": sat,
            "kv_sha256": hashlib.sha256(memoryview(buf)[off:n.value]).hexdigest()}


def run_gpu(lib, case, art, adapters, chunk, budget, null_adapter=None):
    sh = A.SHAPES[case["shape"]]
    prompt = case_prompt(case)
    eng = abi.Engine(lib, art, blocks=1, max_batch=1, max_chunk=min(chunk, 2048))
    try:
        s = eng.new_seq()
        handles = [eng.map_adapter(a) for a in adapters]
        if null_adapter is not None:
            s.set_adapter(eng.map_adapter(null_adapter))
        if case.get("attach") is not None:
            s.set_adapter(handles[case["attach"]])
        nrows = case.get("logit_rows", 0)
        rows = np.zeros((1 + nrows, sh.vocab), dtype=np.int32) if nrows else None
        dll = lib.dll
        dll.sslm_b200_capture_logits.argtypes = [C.c_void_p, C.c_void_p]
        assert s.prefill(prompt, chunk) == len(prompt)
        n = case["decode"]
        first = case.get("swap_after", n // 2)
        if nrows:
            assert dll.sslm_b200_capture_logits(eng.ws, rows.ctypes.data) == 0
        toks = s.decode(1 + nrows, budget)
        if nrows:
            dll.sslm_b200_capture_logits(eng.ws, None)
        toks += s.decode(first - 1 - nrows, budget)
        if case.get("swap_to") is not None:
            s.set_adapter(None)
            s.set_adapter(handles[case["swap_to"]])
        toks += s.decode(n - first, budget)
        got = blob_fields(lib, s, sh.hidden)
        got["tokens"] = toks
        got["logit_sha256"] = [hashlib.sha256(rows[1 + i].tobytes()).hexdigest() for i in range(nrows)]
        if nrows:
            for i in range(1 + nrows):      # greedy: the first index of the row's maximum
                assert int(np.argmax(rows[i])) == toks[i]
        return got
    finally:
        eng.close()


@pytest.mark.parametrize("name", [n for n in CASES if n != "config4_base"])
def test_configuration_matches_the_cpu_reference(gpu_lib, golden, name):
    case = CASES[name]
    want = golden[name]
    assert first_steps_fit(case)
    art, adapters = build_case_artifacts(case)
    for chunk, budget in case["gpu_splits"]:
        got = run_gpu(gpu_lib, case, art, adapters, chunk, budget)
        for key in ("tokens", "context_length", "hidden_scale", "kv_saturation_count", "kv_sha256", "logit_sha256"):
            assert got[key] == want[key], (name, chunk, budget, key)


def first_steps_fit(case):
    n = case["decode"]
    return 1 + case.get("logit_rows", 0) <= case.get("swap_after", n // 2)


def test_base_run_equals_run_with_an_adapter_that_adapts_nothing(gpu_lib, golden):
    case = CASES["config4_base"]
    want = golden["config4_base"]
    art, _ = build_case_artifacts(case)
    null = A.build_synthetic_adapter(art, 7, projections=())
    for null_adapter in (None, null):
        got = run_gpu(gpu_lib, case, art, [], 300, 1, null_adapter)
        for key in ("tokens", "context_length", "hidden_scale", "kv_saturation_count", "kv_sha256"):
            assert got[key] == want[key], (key, null_adapter is not None)

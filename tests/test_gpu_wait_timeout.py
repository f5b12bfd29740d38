"""A bounded device wait that runs out, made to happen on purpose.

Every mbarrier wait of the kernels has a poll limit. The tensor-core linear kernel's producer is told
(test-only hook sslm_b200_debug_withhold_tc_load) to arm the barrier of its first weight tile without
requesting the tile; the wait on it gives up after the limit (about a second), the tile's rows end
with the internal status 100, and the verb that launched the kernel returns SSLM_ALLOCATION_FAILED.
Nothing faults, nothing spins without a limit, the context stays usable, and the same call then
succeeds and gives the oracle's results. (The failure is injected on the host side of the launch:
a request that is never made. No kernel is made to trap or to loop.)
"""
import ctypes as C

import numpy as np
import pytest

import failure_cases as F
from superslm_b200 import abi, artifact as A
from tests.test_gpu_parity import gpu_linear, linear_case_inputs, oracle_linear, run_port, tc_launches

pytestmark = pytest.mark.gpu
WAIT_TIMEOUT = 100


def hook(lib):
    f = lib.dll.sslm_b200_debug_withhold_tc_load
    f.argtypes = [C.c_int32]
    return f


def test_standalone_layer_reports_the_rows_of_the_abandoned_tile(gpu_lib):
    K, N, M = 1536, 512, 200
    x, w, fold, in_scales = linear_case_inputs(K, N, M)
    site = (1090717716, -44)
    want = oracle_linear(x, w, fold, in_scales, site)
    arm = hook(gpu_lib)
    assert arm(17) != 0 and arm(1) == 0
    try:
        before = tc_launches(gpu_lib)
        got = gpu_linear(gpu_lib, x, w, fold, in_scales, site, 1)
        assert tc_launches(gpu_lib) - before == 1
    finally:
        arm(0)
    # block 0's first tile starts at row 0: its 128 rows carry the internal status, the others finished
    assert (got[3][:128] == WAIT_TIMEOUT).all()
    assert (got[3][128:] == want[3][128:]).all()
    # the hook is spent: the same call now gives the oracle's rows
    got = gpu_linear(gpu_lib, x, w, fold, in_scales, site, 1)
    for k in range(4):
        assert (np.asarray(got[k]).astype(np.int64) == np.asarray(want[k]).astype(np.int64)).all(), k


def test_prefill_fails_cleanly_and_the_next_call_succeeds(gpu_lib):
    sh = A.SHAPES["mini1.5b"]
    art = A.build_synthetic_model("mini1.5b", 0x7100, 96)
    prompt = A.stream_uniform(0x7100, "prompt", 40, 0, sh.vocab - 1)
    want_toks, ps = run_port(art, prompt, 3)
    eng = abi.Engine(gpu_lib, art, blocks=1, max_chunk=64)
    arm = hook(gpu_lib)
    try:
        s = eng.new_seq()
        fresh = F._state_digest(gpu_lib, s.handle, sh, 96)
        toks = np.ascontiguousarray(prompt, dtype=np.int32)
        consumed = C.c_int32(-1)
        assert arm(1) == 0
        before = tc_launches(gpu_lib)
        st = gpu_lib.sslm_prefill(eng.model, s.handle, toks.ctypes.data_as(C.POINTER(C.c_int32)), toks.size, 64, 0, eng.ws,
                                  C.byref(consumed))
        assert tc_launches(gpu_lib) > before                 # the chunk did run on the tensor-core kernel
        assert st == abi.ST["SSLM_ALLOCATION_FAILED"] and consumed.value == 0
        assert F._state_digest(gpu_lib, s.handle, sh, 96) == fresh      # nothing of the chunk was kept
        arm(0)
        assert s.prefill(prompt, 64) == len(prompt)
        assert s.decode(3, sh.layers) == want_toks
        blob = abi.parse_save_blob(s.save(), sh.hidden)
        assert blob["kv"] == ps.kv.tobytes()
    finally:
        arm(0)
        eng.close()

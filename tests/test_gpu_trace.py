"""Per-site trace: the codes and carried scale of every traced site (attn_norm, rotated q, attn_ctx,
attn_residual, mlp_norm, mlp_act, mlp_residual) of every layer and token, CUDA path against the CPU
oracle. This is the bisection aid (a parity failure is located by its first differing record) and,
run green, a check of every per-layer hidden state rather than only of K/V and tokens."""
import ctypes as C

import numpy as np
import pytest

from oracle import harness as H
from superslm_b200 import abi, artifact as A

pytestmark = pytest.mark.gpu
SITES = (0, 2, 3, 5, 6, 9, 11)


def gpu_trace(lib, eng, fn, cap=64 << 20):
    f = lib.dll.sslm_b200_trace
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]
    buf = np.zeros(cap, dtype=np.uint8)
    assert f(eng.ws, buf.ctypes.data, buf.size, None) == 0
    try:
        fn()
    finally:
        used = C.c_size_t(0)
        assert f(eng.ws, None, 0, C.byref(used)) == 0
    return H.parse_trace(buf[:used.value])


def oracle_trace(fn, cap=64 << 20):
    port = H.port()
    buf = np.zeros(cap, dtype=np.uint8)
    port.osc_trace_begin(buf.ctypes.data, buf.size)
    try:
        fn()
    finally:
        used = port.osc_trace_end()
    return H.parse_trace(buf[:used])


@pytest.mark.parametrize("shape,seed,plen,chunk,budget", [("small", 0x7A01, 23, 9, 2), ("mini1.5b", 0x7A02, 21, 64, 1)])
def test_every_traced_site_matches_the_oracle(gpu_lib, shape, seed, plen, chunk, budget):
    sh = A.SHAPES[shape]
    art = A.build_synthetic_model(shape, seed, 64)
    prompt = A.stream_uniform(seed, "prompt", plen, 0, sh.vocab - 1)
    ndec = 3
    pm = H.PortModel(art)
    ps = H.PortSeq(pm)
    state = {}

    def cpu():
        assert ps.prefill(prompt) == 0
        state["cpu"] = ps.decode(ndec, sh.layers)

    want = oracle_trace(cpu)
    eng = abi.Engine(gpu_lib, art, blocks=1, max_chunk=64)
    try:
        s = eng.new_seq()

        def gpu():
            assert s.prefill(prompt, chunk) == len(prompt)
            state["gpu"] = s.decode(ndec, budget)

        got = gpu_trace(gpu_lib, eng, gpu)
    finally:
        eng.close()
    assert state["gpu"] == state["cpu"]
    # one record per (position, layer, site) on both sides: prompt tokens and all but the last decoded one
    positions = plen + ndec - 1
    assert len(want) == positions * sh.layers * len(SITES)
    assert set(got) == set(want)
    for key in sorted(want):
        m, e, codes = want[key]
        gm, ge, gcodes = got[key]
        assert gcodes == codes, key
        if key[2] != 2:                   # (the rotated q row is traced without its scale)
            assert (gm, ge) == (m, e), key

"""Prefix verbs (src/sslm_abi.cpp:1584-1694, :1870-1925) on the GPU library: a sequence that adopts
a frozen prefix continues exactly like one that prefilled the same tokens itself, and exactly
like the reference's sequence that adopted the reference's prefix; full pages are shared between
the prefix and its adopters, which must not let one adopter's writes reach another."""
import ctypes as C

import numpy as np
import pytest

from superslm_b200 import abi
from superslm_b200 import artifact as A

pytestmark = pytest.mark.gpu

SHAPE = "small"


@pytest.fixture(scope="module")
def art():
    return A.build_synthetic_model(SHAPE, seed=0xFEED, context_cap=112)


def toks(n, salt):
    return A.stream_uniform(300 + salt, "prefix_tokens", n, 0, A.SHAPES[SHAPE].vocab - 1).astype(np.int32)


class Prefix:
    def __init__(self, lib, eng):
        self.lib, self.eng, self.h = lib, eng, abi._H()
        assert lib.sslm_prefix_begin(eng.model, C.byref(eng.pool), C.byref(self.h)) == 0

    def prefill(self, tokens, chunk):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        done = 0
        while done < t.size:
            c = C.c_int32(0)
            st = self.lib.sslm_prefix_prefill(self.eng.model, self.h, t[done:].ctypes.data_as(C.POINTER(C.c_int32)),
                                              t.size - done, chunk, 0, self.eng.ws, C.byref(c))
            if st != 0:
                return st
            done += c.value
        return 0

    def freeze(self):
        assert self.lib.sslm_prefix_freeze(self.h) == 0

    def release(self):
        assert self.lib.sslm_prefix_release(self.h) == 0


def run_adopters(lib, art, prefix_len, tails, n_decode):
    """prefix of prefix_len tokens, one adopter per tail (extra prompt tokens), decode each."""
    eng = abi.Engine(lib, art, blocks=len(tails) + 2, max_batch=4, max_chunk=32)
    out = []
    try:
        px = Prefix(lib, eng)
        assert px.prefill(toks(prefix_len, 0), 16) == 0
        px.freeze()
        seqs = []
        for i, tail in enumerate(tails):
            s = eng.new_seq()
            assert lib.sslm_seq_adopt_prefix(s.handle, px.h) == 0
            if tail:
                assert s.prefill(toks(tail, 10 + i), 5) == tail
            seqs.append(s)
        released_early = len(tails) > 1
        if released_early:
            px.release()                    # adopters keep the shared pages alive
        for s in seqs:
            out.append((s.decode(n_decode, A.SHAPES[SHAPE].layers), s.save()))
        if not released_early:
            px.release()
    finally:
        eng.close()
    return out


@pytest.mark.parametrize("prefix_len", [16, 37, 48, 5])
def test_adopter_equals_a_sequence_that_prefilled_everything(gpu_lib, art, prefix_len):
    tails = [0, 7, 19]
    got = run_adopters(gpu_lib, art, prefix_len, tails, 5)
    eng = abi.Engine(gpu_lib, art, blocks=2, max_batch=1, max_chunk=32)
    try:
        for i, tail in enumerate(tails):
            s = eng.new_seq()
            full = np.concatenate([toks(prefix_len, 0), toks(tail, 10 + i)]) if tail else toks(prefix_len, 0)
            assert s.prefill(full, 32) == full.size
            want = (s.decode(5, A.SHAPES[SHAPE].layers), s.save())
            assert got[i][0] == want[0], (prefix_len, tail)
            assert got[i][1] == want[1], (prefix_len, tail)
            s.release()
    finally:
        eng.close()


def test_adopters_match_the_reference(gpu_lib, ref_lib, art):
    for prefix_len in (21, 32):
        got = run_adopters(gpu_lib, art, prefix_len, [0, 11], 6)
        want = run_adopters(ref_lib, art, prefix_len, [0, 11], 6)
        assert [g[0] for g in got] == [w[0] for w in want]
        assert [g[1] for g in got] == [w[1] for w in want]


def test_statuses_and_reuse(gpu_lib, art):
    eng = abi.Engine(gpu_lib, art, blocks=3, max_batch=2, max_chunk=32)
    try:
        px = Prefix(gpu_lib, eng)
        s = eng.new_seq()
        assert gpu_lib.sslm_seq_adopt_prefix(s.handle, px.h) == 1          # not frozen yet
        assert px.prefill(toks(20, 0), 32) == 0
        px.freeze()
        assert px.prefill(toks(3, 1), 32) == 13                            # SSLM_PREFIX_FROZEN_REJECTED
        assert gpu_lib.sslm_seq_adopt_prefix(None, px.h) == 1
        assert gpu_lib.sslm_seq_adopt_prefix(s.handle, None) == 1
        # adoption overwrites whatever the sequence held, as often as asked
        assert s.prefill(toks(40, 2), 32) == 40
        s.decode(2, 3)
        assert gpu_lib.sslm_seq_adopt_prefix(s.handle, px.h) == 0
        first = (s.decode(4, 3), s.save())
        s.reset()
        assert gpu_lib.sslm_seq_adopt_prefix(s.handle, px.h) == 0
        assert (s.decode(4, 3), s.save()) == first
        # the pool still has its third block: prefix + s hold two
        t = eng.new_seq()
        assert t.prefill(toks(112, 3), 32) == 112                          # a full-length sequence still fits
        px.release()
    finally:
        eng.close()

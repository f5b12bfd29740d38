"""sslm_seq_restore / sslm_seq_reset (src/sslm_abi.cpp:2722-2990, :1820-1860) on the GPU library:
round trips through its own blobs in every resting state, state interchange with the compiled
reference in both directions (a sequence saved on one side continues bit-exactly on the other),
the reference's rejection statuses in the reference's order, and reset-as-restart."""
import struct

import numpy as np
import pytest

from superslm_b200 import abi
from superslm_b200 import artifact as A

pytestmark = pytest.mark.gpu

SHAPE = "small"


@pytest.fixture(scope="module")
def art():
    return A.build_synthetic_model(SHAPE, seed=0xA11CE, context_cap=96)


def prompt(n, salt=0):
    return A.stream_uniform(900 + salt, "restore_prompt", n, 0, A.SHAPES[SHAPE].vocab - 1).astype(np.int32)


def step_until(seq, eng, budget, n_steps):
    """n_steps raw sslm_decode_step calls (tokens or -1 each)."""
    out = []
    for _ in range(n_steps):
        st, toks = eng.decode_step([seq], budget)
        assert st == 0, abi.STATUS_NAMES.get(st, st)
        out.append(toks[0])
    return out


@pytest.mark.parametrize("budget,steps_before", [(3, 1), (1, 2), (2, 5), (3, 4), (1, 6)])
def test_round_trip_in_every_resting_state(gpu_lib, art, budget, steps_before):
    """between tokens and mid-token at several layers. (Right after prefill the blob holds no
    residual -- SSB3 saves one only mid-token -- so a restored sequence does not continue like the
    live one there, in the reference either; that state is compared library against library in
    test_state_interchange_with_the_reference.)"""
    eng = abi.Engine(gpu_lib, art, blocks=3, max_batch=2, max_chunk=32)
    try:
        a = eng.new_seq()
        assert a.prefill(prompt(21), 8) == 21
        step_until(a, eng, budget, steps_before)
        blob = a.save()
        b = abi.Sequence.restore(eng, blob)
        assert b.save() == blob                       # nothing lost, nothing invented
        ta = step_until(a, eng, budget, 9)
        tb = step_until(b, eng, budget, 9)
        assert ta == tb
        assert a.save() == b.save()
    finally:
        eng.close()


def test_state_interchange_with_the_reference(gpu_lib, ref_lib, art):
    L = A.SHAPES[SHAPE].layers
    geng = abi.Engine(gpu_lib, art, blocks=3, max_batch=2, max_chunk=32)
    ceng = abi.Engine(ref_lib, art, blocks=3, max_batch=2, max_chunk=32)
    try:
        for budget, steps_before in [(L, 0), (L, 2), (1, 4), (2, 3)]:
            # CPU -> GPU
            c = ceng.new_seq()
            assert c.prefill(prompt(17, 1), 17) == 17
            step_until(c, ceng, budget, steps_before)
            blob = c.save()
            g = abi.Sequence.restore(geng, blob)
            assert g.save() == blob
            if steps_before == 0:      # no residual in the blob: compare with the reference's own restore
                c.release()
                c = abi.Sequence.restore(ceng, blob)
            assert step_until(g, geng, budget, 7) == step_until(c, ceng, budget, 7)
            assert g.save() == c.save()
            # GPU -> CPU, from where the two now stand
            blob2 = g.save()
            c2 = abi.Sequence.restore(ceng, blob2)
            assert step_until(c2, ceng, budget, 5) == step_until(g, geng, budget, 5)
            assert c2.save() == g.save()
            for s in (c, c2, g):
                s.release()
    finally:
        geng.close()
        ceng.close()


def restore_status(lib, eng, blob):
    h = abi._H()
    raw = np.frombuffer(bytes(blob), dtype=np.uint8)
    st = lib.sslm_seq_restore(eng.model, abi.C.byref(eng.pool), raw.ctypes.data, raw.size, abi.C.byref(h))
    if st == 0:
        lib.sslm_seq_release(h)
    return st


def test_rejections_follow_the_reference(gpu_lib, art):
    other = A.build_synthetic_model(SHAPE, seed=0xB0B, context_cap=96)
    eng = abi.Engine(gpu_lib, art, blocks=2, max_batch=1, max_chunk=32)
    eng_other = abi.Engine(gpu_lib, other, blocks=1, max_batch=1, max_chunk=32)
    try:
        s = eng.new_seq()
        assert s.prefill(prompt(9), 9) == 9
        step_until(s, eng, 2, 2)                       # mid-token: the blob carries a residual
        good = bytearray(s.save())
        assert restore_status(gpu_lib, eng, good) == 0
        bad = bytearray(good); bad[0:4] = b"SLM3"
        assert restore_status(gpu_lib, eng, bad) == 1                       # foreign format
        assert restore_status(gpu_lib, eng, good[:100]) == 1                # shorter than the header
        assert restore_status(gpu_lib, eng, good[:-1]) == 1                 # KV block cut short
        assert restore_status(gpu_lib, eng_other, good) == 6                # another model's blob
        bad = bytearray(good); struct.pack_into("<I", bad, 36, 1)
        assert restore_status(gpu_lib, eng, bad) == 7                       # KV precision
        bad = bytearray(good); struct.pack_into("<Q", bad, 40, 0x1234)
        assert restore_status(gpu_lib, eng, bad) == 22                      # schema binding
        bad = bytearray(good); struct.pack_into("<I", bad, 48, 0)
        assert restore_status(gpu_lib, eng, bad) == 22                      # walk state on an unbound blob
        bad = bytearray(good); struct.pack_into("<q", bad, 60, 97)
        assert restore_status(gpu_lib, eng, bad) == 1                       # context beyond the cap
        bad = bytearray(good); struct.pack_into("<I", bad, 68, 99)
        assert restore_status(gpu_lib, eng, bad) == 1                       # layer index beyond the model
        bad = bytearray(good); struct.pack_into("<I", bad, 120 + A.SHAPES[SHAPE].hidden, 2)
        assert restore_status(gpu_lib, eng, bad) == 1                       # block count
        # pool with no block left
        keep = abi.Sequence.restore(eng, bytes(good))
        assert restore_status(gpu_lib, eng, good) == 14
        keep.release()
    finally:
        eng.close()
        eng_other.close()


def test_reset_is_a_restart(gpu_lib, art):
    eng = abi.Engine(gpu_lib, art, blocks=2, max_batch=1, max_chunk=32)
    try:
        fresh = eng.new_seq()
        assert fresh.prefill(prompt(13, 2), 5) == 13
        want_tokens = fresh.decode(4, 3)
        want_blob = fresh.save()

        s = eng.new_seq()
        assert s.prefill(prompt(30, 3), 32) == 30           # a longer, different history first
        s.decode(3, 3)
        step_until(s, eng, 1, 1)                            # now mid-token
        assert gpu_lib.sslm_seq_reset(s.handle) == 12       # SSLM_SEQ_RESET_MIDTOKEN_REJECTED
        step_until(s, eng, 3, 1)                            # finish the token
        s.reset()
        st, toks = eng.decode_step([s], 3)
        assert st == 1                                      # nothing to decode from, like a new sequence
        assert s.prefill(prompt(13, 2), 5) == 13
        assert s.decode(4, 3) == want_tokens
        assert s.save() == want_blob                        # no trace of the earlier generation
    finally:
        eng.close()

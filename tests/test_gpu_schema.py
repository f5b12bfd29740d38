"""Constrained decoding (SCM1 decode schemas) on the GPU library against the compiled reference:
schema lookup verbs, masked arg-max + DFA walk inside batched decode steps, dead ends (-2),
schema-content prefill spans, binding rules, and the binding travelling through save / restore /
reset / prefix adoption."""
import ctypes as C

import numpy as np
import pytest

from superslm_b200 import abi
from superslm_b200 import artifact as A

pytestmark = pytest.mark.gpu

SHAPE = "small"
SEED = 0x5C11


@pytest.fixture(scope="module")
def art():
    return A.build_synthetic_model(SHAPE, seed=SEED, context_cap=96, schemas=3)


@pytest.fixture(scope="module")
def schemas():
    return A.synthetic_schemas(SEED, A.SHAPES[SHAPE].vocab, 3)


def toks(n, salt):
    return A.stream_uniform(700 + salt, "schema_prompt", n, 0, A.SHAPES[SHAPE].vocab - 1).astype(np.int32)


def lookup(lib, eng, name):
    h = abi._H()
    st = lib.sslm_schema_lookup(eng.model, name.encode(), C.byref(h))
    return st, h


def constrained_run(lib, art, binds, n_steps, budget):
    """One engine, one sequence per entry of `binds` (schema name or None), decoded together."""
    eng = abi.Engine(lib, art, blocks=len(binds), max_batch=len(binds), max_chunk=32)
    try:
        seqs = []
        for i, name in enumerate(binds):
            s = eng.new_seq()
            if name is not None:
                st, h = lookup(lib, eng, name)
                assert st == 0
                assert lib.sslm_seq_set_schema(s.handle, h) == 0
            assert s.prefill(toks(9 + 2 * i, i), 32) == 9 + 2 * i
            seqs.append(s)
        trace = []
        for _ in range(n_steps):
            st, out = eng.decode_step(seqs, budget)
            trace.append((st, out if st == 0 else None))
            if st != 0:
                break
        blobs = [s.save() for s in seqs]
        return trace, blobs
    finally:
        eng.close()


def test_lookup_verbs(gpu_lib, art):
    eng = abi.Engine(gpu_lib, art, blocks=1, max_batch=1, max_chunk=16)
    try:
        assert gpu_lib.sslm_schema_count(eng.model) == 3
        assert lookup(gpu_lib, eng, "schema_2")[0] == 0
        assert lookup(gpu_lib, eng, "schema_9")[0] == 18          # SSLM_SCHEMA_NOT_FOUND
        n = C.c_size_t(0)
        assert gpu_lib.sslm_schema_name(eng.model, 1, None, C.byref(n)) == abi.ST["SSLM_BUFFER_TOO_SMALL"]
        buf = C.create_string_buffer(n.value)
        assert gpu_lib.sslm_schema_name(eng.model, 1, buf, C.byref(n)) == 0 and buf.raw[:n.value] == b"schema_1"
        assert gpu_lib.sslm_schema_name(eng.model, 3, buf, C.byref(n)) == 1
    finally:
        eng.close()


@pytest.mark.parametrize("budget,copies", [(3, 1), (1, 1), (3, 3)])
def test_constrained_batch_matches_the_reference(gpu_lib, ref_lib, art, schemas, budget, copies):
    # 5 sequences take the streaming head kernel, 15 the tensor-core one: both apply the mask
    binds = ["schema_0", None, "schema_1", "schema_2", "schema_0"] * copies
    steps = 14 if budget == 3 else 30
    got = constrained_run(gpu_lib, art, binds, steps, budget)
    want = constrained_run(ref_lib, art, binds, steps, budget)
    assert got[0] == want[0]
    assert got[1] == want[1]
    # the constraint really held: every token a bound sequence produced is one its schema allows
    for si, name in enumerate(binds):
        if name is None:
            continue
        rows = {st: dict(r) for st, r in enumerate(schemas[int(name[-1])]["rows"])}
        state = 0
        for st, out in got[0]:
            if st != 0 or out[si] < 0:
                continue
            assert out[si] in rows[state], (name, state, out[si])
            state = rows[state][out[si]]


def test_dead_end_reports_minus_two_then_refuses(gpu_lib, ref_lib, art, schemas):
    # walk one sequence until its schema's last state (which allows nothing)
    for lib in (gpu_lib, ref_lib):
        trace, _ = constrained_run(lib, art, ["schema_1"], 80, 3)
        flat = [(st, out[0] if out else None) for st, out in trace]
        if lib is gpu_lib:
            mine = flat
        else:
            assert mine == flat
    assert any(t == -2 for _, t in mine if t is not None) or mine[-1][0] != 0 or len(mine) == 80
    if any(t == -2 for _, t in mine if t is not None):
        assert mine[-1][0] == abi.ST["SSLM_ARTIFACT_REJECTED"]


def test_schema_content_spans(gpu_lib, ref_lib, art, schemas):
    rows = [dict(r) for r in schemas[0]["rows"]]
    # a path through schema_0 from its start state, then one token it does not allow there
    path, state = [], 0
    for _ in range(5):
        if not rows[state]:
            break
        tok = sorted(rows[state])[len(path) % len(rows[state])]
        path.append(tok)
        state = rows[state][tok]
    bad = next(t for t in range(A.SHAPES[SHAPE].vocab) if t not in rows[state])
    span = np.array(path + [bad, path[0]], dtype=np.int32)
    res = []
    for lib in (gpu_lib, ref_lib):
        eng = abi.Engine(lib, art, blocks=2, max_batch=1, max_chunk=32)
        try:
            s = eng.new_seq()
            c = C.c_int32(0)
            ptr = span.ctypes.data_as(C.POINTER(C.c_int32))
            assert lib.sslm_prefill(eng.model, s.handle, ptr, span.size, 32, 1, eng.ws, C.byref(c)) == 20   # unbound
            st, h = lookup(lib, eng, "schema_0")
            assert lib.sslm_seq_set_schema(s.handle, h) == 0
            assert s.prefill(toks(6, 9), 32) == 6                     # a prompt span: the walk stays at the start
            st = lib.sslm_prefill(eng.model, s.handle, ptr, span.size, 32, 1, eng.ws, C.byref(c))
            rec = [st, c.value]
            assert lib.sslm_seq_set_schema(s.handle, None) == 19        # no re-binding once tokens went in
            out = []
            for _ in range(6):
                st2, o = eng.decode_step([s], 3)
                out.append((st2, o[0]))
            rec += [out, s.save()]
            # the binding and the walk survive save / restore, and restore refuses an unknown schema
            t = abi.Sequence.restore(eng, rec[3])
            assert t.save() == rec[3]
            assert eng.decode_step([t], 3) == eng.decode_step([s], 3)
            res.append(rec)
        finally:
            eng.close()
    assert res[0] == res[1]
    assert res[0][0] == 23 and res[0][1] == len(path)               # SSLM_SCHEMA_SPAN_UNREACHABLE after the path


def test_restore_with_unknown_schema_and_reset(gpu_lib, art):
    eng = abi.Engine(gpu_lib, art, blocks=2, max_batch=1, max_chunk=32)
    try:
        s = eng.new_seq()
        _, h = lookup(gpu_lib, eng, "schema_2")
        assert gpu_lib.sslm_seq_set_schema(s.handle, h) == 0
        assert s.prefill(toks(7, 4), 32) == 7
        first = [eng.decode_step([s], 3) for _ in range(4)]
        blob = bytearray(s.save())
        import struct
        struct.pack_into("<Q", blob, 40, 0xDEADBEEF)                     # a schema this model does not have
        hh = abi._H()
        raw = np.frombuffer(bytes(blob), dtype=np.uint8)
        assert gpu_lib.sslm_seq_restore(eng.model, C.byref(eng.pool), raw.ctypes.data, raw.size, C.byref(hh)) == 22
        blob = bytearray(s.save())
        struct.pack_into("<I", blob, 48, 10 ** 6)                         # a state the schema does not have
        raw = np.frombuffer(bytes(blob), dtype=np.uint8)
        assert gpu_lib.sslm_seq_restore(eng.model, C.byref(eng.pool), raw.ctypes.data, raw.size, C.byref(hh)) == 22
        # reset keeps the binding and rewinds the walk: the same prompt gives the same constrained tokens
        s.reset()
        assert s.prefill(toks(7, 4), 32) == 7
        assert [eng.decode_step([s], 3) for _ in range(4)] == first
    finally:
        eng.close()


def test_prefix_with_schema_progress(gpu_lib, ref_lib, art, schemas):
    rows = [dict(r) for r in schemas[1]["rows"]]
    path, state = [], 0
    for _ in range(3):
        tok = sorted(rows[state])[0]
        path.append(tok)
        state = rows[state][tok]
    span = np.array(path, dtype=np.int32)
    res = []
    for lib in (gpu_lib, ref_lib):
        eng = abi.Engine(lib, art, blocks=3, max_batch=2, max_chunk=32)
        try:
            px = abi._H()
            assert lib.sslm_prefix_begin(eng.model, C.byref(eng.pool), C.byref(px)) == 0
            _, h1 = lookup(lib, eng, "schema_1")
            _, h0 = lookup(lib, eng, "schema_0")
            assert lib.sslm_prefix_set_schema(px, h1) == 0
            c = C.c_int32(0)
            p = toks(5, 6)
            assert lib.sslm_prefix_prefill(eng.model, px, p.ctypes.data_as(C.POINTER(C.c_int32)), 5, 32, 0, eng.ws, C.byref(c)) == 0
            assert lib.sslm_prefix_set_schema(px, h0) == 1              # content already in
            assert lib.sslm_prefix_prefill(eng.model, px, span.ctypes.data_as(C.POINTER(C.c_int32)), span.size, 32, 1,
                                           eng.ws, C.byref(c)) == 0 and c.value == span.size
            assert lib.sslm_prefix_freeze(px) == 0
            other = eng.new_seq()
            assert lib.sslm_seq_set_schema(other.handle, h0) == 0
            rec = [lib.sslm_seq_adopt_prefix(other.handle, px)]            # 21: bound to a different schema
            s = eng.new_seq()
            assert lib.sslm_seq_set_schema(s.handle, h1) == 0
            rec.append(lib.sslm_seq_adopt_prefix(s.handle, px))
            rec.append([eng.decode_step([s], 3) for _ in range(5)])
            rec.append(s.save())
            res.append(rec)
            assert lib.sslm_prefix_release(px) == 0
        finally:
            eng.close()
    assert res[0] == res[1]
    assert res[0][0] == 21 and res[0][1] == 0

"""Parity of the CUDA path with the CPU oracle, through the C ABI (libsslm_b200.so).

Bit-exact everywhere: tokens, every layer's K/V bytes (canonical order), the carried
hidden scale, the K/V saturation counter, full logit rows, and the standalone linear
layer's folded accumulators / codes / scales. The oracle is the plain-C restatement
(oracle/sslm_oracle.c); where the compiled reference travels with the tree it is
compared too."""
import ctypes as C
import hashlib

import numpy as np
import pytest

from oracle import harness as H
from oracle.harness import Scale
from superslm_b200 import abi, artifact as A

pytestmark = pytest.mark.gpu


def gpu_record(lib, case, chunk, budget):
    sh = A.SHAPES[case["shape"]]
    art = A.build_synthetic_model(case["shape"], case["seed"], case["context_cap"], case["shift_lo"], case["shift_hi"],
                                  case.get("bias_bits", 0))
    prompt = A.stream_uniform(case["seed"] ^ 0xABCDEF, "prompt", case["prompt_len"], 0, sh.vocab - 1)
    eng = abi.Engine(lib, art, blocks=1, max_chunk=64)
    s = eng.new_seq()
    if case["adapters"]:
        ha = eng.map_adapter(A.build_synthetic_adapter(art, case["adapters"][0]))
        hb = eng.map_adapter(A.build_synthetic_adapter(art, case["adapters"][1]))
        s.set_adapter(ha)
    s.prefill(prompt, chunk)
    n = case["decode"]
    toks = s.decode(n // 2, budget)
    if case["adapters"]:
        s.set_adapter(None)
        s.set_adapter(hb)
    toks += s.decode(n - n // 2, budget)
    blob = abi.parse_save_blob(s.save(), sh.hidden)
    eng.close()
    return {"tokens": toks, "context_length": blob["context_length"], "hidden_scale": list(blob["hidden_scale"]),
            "kv_saturation_count": blob["kv_saturation_count"], "kv_sha256": hashlib.sha256(blob["kv"]).hexdigest()}


@pytest.mark.parametrize("name", ["tiny", "small", "small_dense", "tiny_lora", "tiny_bias", "tiny_bias_lora",
                                  "small_bias_saturating"])
@pytest.mark.parametrize("chunk,budget", [(64, 0), (7, 1), (1, 2), (33, 0)])
def test_golden_records_at_every_split(gpu_lib, e2e_golden, name, chunk, budget):
    case = e2e_golden[name]
    got = gpu_record(gpu_lib, case, chunk, budget or A.SHAPES[case["shape"]].layers)
    for k, v in got.items():
        assert v == case[k], (name, chunk, budget, k)


def run_port(art, prompt, ndec, adapter=None):
    pm = H.PortModel(art)
    s = H.PortSeq(pm)
    if adapter is not None:
        s.lora = pm.lora(adapter)
    assert s.prefill(prompt) == 0
    toks = s.decode(ndec, pm.cfg["num_hidden_layers"])
    return toks, s


def test_real_width_layers_against_oracle(gpu_lib):
    """Two layers at the 1.5B projection shapes (1536 / 256 / 8960), head_dim 128, GQA 6:1."""
    sh = A.SHAPES["mini1.5b"]
    art = A.build_synthetic_model("mini1.5b", 0x1515, 128)
    prompt = A.stream_uniform(99, "prompt", 70, 0, sh.vocab - 1)
    ptoks, ps = run_port(art, prompt, 12)
    for chunk, budget in ((64, 2), (16, 1)):
        eng = abi.Engine(gpu_lib, art, blocks=1, max_chunk=64)
        s = eng.new_seq()
        s.prefill(prompt, chunk)
        toks = s.decode(12, budget)
        blob = abi.parse_save_blob(s.save(), sh.hidden)
        eng.close()
        assert toks == ptoks
        assert blob["kv"] == ps.kv.tobytes()
        assert blob["hidden_scale"] == (ps.s.hidden_scale.m, ps.s.hidden_scale.e)
        assert blob["kv_saturation_count"] == ps.s.kv_saturation_count


def test_logit_rows_match_oracle(gpu_lib):
    sh = A.SHAPES["small"]
    art = A.build_synthetic_model("small", 31337, 64)
    prompt = A.stream_uniform(5, "prompt", 9, 0, sh.vocab - 1)
    pm = H.PortModel(art)
    ps = H.PortSeq(pm)
    assert ps.prefill(prompt) == 0
    eng = abi.Engine(gpu_lib, art, blocks=1, max_chunk=16)
    lib = gpu_lib.dll
    lib.sslm_b200_capture_logits.argtypes = [C.c_void_p, C.c_void_p]
    rows = np.zeros((4, sh.vocab), dtype=np.int32)
    assert lib.sslm_b200_capture_logits(eng.ws, rows.ctypes.data) == 0
    s = eng.new_seq()
    s.prefill(prompt, 16)
    toks = s.decode(4, sh.layers)
    lib.sslm_b200_capture_logits(eng.ws, None)
    for i in range(4):
        st, tok, logits = ps.decode_step(sh.layers, want_logits=True)
        assert st == 0 and tok == toks[i]
        assert (logits == rows[i]).all()
        assert int(np.argmax(rows[i])) == tok      # first index of the maximum
    eng.close()


def test_batched_decode_mixed_states(gpu_lib):
    """Many sequences in one sslm_decode_step: different lengths, different layer
    positions, one waiting for its first logits; each must equal its own single-sequence run."""
    sh = A.SHAPES["small"]
    art = A.build_synthetic_model("small", 777, 96)
    lens = [3, 17, 40, 16, 33, 1, 64, 9, 25]
    prompts = [A.stream_uniform(1000 + i, "p", n, 0, sh.vocab - 1) for i, n in enumerate(lens)]
    want = []
    for p in prompts:
        toks, ps = run_port(art, p, 6)
        want.append((toks, ps.kv.tobytes(), (ps.s.hidden_scale.m, ps.s.hidden_scale.e), ps.s.kv_saturation_count))
    eng = abi.Engine(gpu_lib, art, blocks=len(lens), max_batch=len(lens), max_chunk=64)
    seqs = [eng.new_seq() for _ in lens]
    for s, p in zip(seqs, prompts):
        s.prefill(p, 64)
    got = [[] for _ in lens]
    # stagger: advance some sequences alone first so the batch holds different layer indices
    for i in (1, 4):
        st, t = eng.decode_step([seqs[i]], sh.layers)   # consumes the pending logits
        assert st == 0
        got[i].append(t[0])
        st, t = eng.decode_step([seqs[i]], 1 + (i % 2))  # now mid-token
        assert st == 0 and t[0] == -1
    budget = 2
    while any(len(g) < 6 for g in got):
        live = [i for i in range(len(lens)) if len(got[i]) < 6]
        st, toks = eng.decode_step([seqs[i] for i in live], budget)
        assert st == 0
        for i, t in zip(live, toks):
            if t >= 0:
                got[i].append(t)
    for i, s in enumerate(seqs):
        blob = abi.parse_save_blob(s.save(), sh.hidden)
        # finish the token in flight, if any, so that both sides sit at a token boundary
        assert got[i] == want[i][0], i
        if blob["layer_index"] == 0:
            assert blob["kv"] == want[i][1], i
            assert blob["hidden_scale"] == want[i][2], i
            assert blob["kv_saturation_count"] == want[i][3], i
    eng.close()


def test_mid_token_state_matches_oracle(gpu_lib):
    sh = A.SHAPES["small"]
    art = A.build_synthetic_model("small", 4242, 48)
    prompt = A.stream_uniform(8, "prompt", 11, 0, sh.vocab - 1)
    pm = H.PortModel(art)
    ps = H.PortSeq(pm)
    assert ps.prefill(prompt) == 0
    eng = abi.Engine(gpu_lib, art, blocks=1, max_chunk=16)
    s = eng.new_seq()
    s.prefill(prompt, 16)
    for budget in (3, 2):            # first call: logits only; second: two of three layers
        st, t = eng.decode_step([s], budget)
        pst, ptok, _ = ps.decode_step(budget)
        assert st == 0 and pst == 0 and t[0] == ptok
    blob = abi.parse_save_blob(s.save(), sh.hidden)
    assert blob["layer_index"] == 2 == ps.s.layer_index
    assert blob["residual"] == ps.hidden.tobytes()
    assert blob["hidden_scale"] == (ps.s.hidden_scale.m, ps.s.hidden_scale.e)
    assert blob["kv"] == ps.kv.tobytes()
    eng.close()


def test_per_row_adapters_in_one_batch(gpu_lib):
    sh = A.SHAPES["tiny"]
    art = A.build_synthetic_model("tiny", 606, 64)
    ad = [A.build_synthetic_adapter(art, 21), A.build_synthetic_adapter(art, 22, projections=PROJ7)]
    prompts = [A.stream_uniform(50 + i, "p", 10 + 3 * i, 0, sh.vocab - 1) for i in range(3)]
    want = [run_port(art, prompts[0], 5, ad[0])[0], run_port(art, prompts[1], 5, None)[0],
            run_port(art, prompts[2], 5, ad[1])[0]]
    assert want[0] != run_port(art, prompts[0], 5, None)[0]
    eng = abi.Engine(gpu_lib, art, blocks=3, max_batch=3, max_chunk=32)
    h = [eng.map_adapter(a) for a in ad]
    seqs = [eng.new_seq() for _ in range(3)]
    seqs[0].set_adapter(h[0])
    seqs[2].set_adapter(h[1])
    for s, p in zip(seqs, prompts):
        s.prefill(p, 32)
    got = [[] for _ in range(3)]
    while len(got[0]) < 5:
        st, toks = eng.decode_step(seqs, sh.layers)
        assert st == 0
        for g, t in zip(got, toks):
            g.append(t)
    assert got == want
    # mid-token swap is refused; foreign adapter is refused
    st, t = eng.decode_step([seqs[0]], 1)
    assert st == 0 and t[0] == -1
    assert gpu_lib.sslm_seq_set_adapter(seqs[0].handle, h[1]) == abi.ST["SSLM_ADAPTER_SWAP_MIDTOKEN_REJECTED"]
    assert gpu_lib.sslm_adapter_release(h[0]) == abi.ST["SSLM_ADAPTER_HAS_LIVE_SEQUENCES"]
    eng.close()


PROJ7 = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def cpu_gemm(x, w):
    """int64 accumulators [M, N]: the reference's own GEMM where it travels with the tree (it is
    vectorised), else the plain-C restatement."""
    M, K = x.shape
    N = w.shape[0]
    acc = np.zeros((M, N), dtype=np.int64)
    shim = H.ref_shim()
    if shim is not None:
        shim.refshim_gemm(x.ctypes.data, w.ctypes.data, M, K, N, acc.ctypes.data)
    else:
        H.port().osc_gemm(x.ctypes.data, w.ctypes.data, M, K, N, acc.ctypes.data)
    return acc


def oracle_linear(x, w, fold, in_scales, site):
    port = H.port()
    M, K = x.shape
    N = w.shape[0]
    acc = cpu_gemm(x, w)
    folded = np.empty_like(acc)
    fold = np.ascontiguousarray(fold, dtype=np.int32)
    port.osc_fold_matrix(acc.ctypes.data, M, N, fold.ctypes.data, folded.ctypes.data)
    codes = np.zeros((M, N), dtype=np.int8)
    scales = np.zeros((M, 2), dtype=np.int64)
    status = np.zeros(M, dtype=np.int32)
    for t in range(M):
        sc = Scale()
        inc = Scale(int(in_scales[t, 0]), int(in_scales[t, 1]))
        row = np.ascontiguousarray(folded[t])
        status[t] = port.osc_funnel(row.ctypes.data, N, C.byref(inc), 1, Scale(*site), codes[t].ctypes.data, C.byref(sc))
        scales[t] = (sc.m, sc.e)
    return folded, codes, scales, status


def gpu_linear(lib, x, w, fold, in_scales, site, use_tc):
    f = lib.dll.sslm_b200_linear
    f.argtypes = [C.c_void_p] * 3 + [C.c_int32] * 3 + [C.c_void_p, C.c_int64, C.c_int64, C.c_int32] + [C.c_void_p] * 4
    M, K = x.shape
    N = w.shape[0]
    folded = np.zeros((M, N), dtype=np.int32)
    codes = np.zeros((M, N), dtype=np.int8)
    scales = np.zeros((M, 2), dtype=np.int64)
    status = np.zeros(M, dtype=np.int32)
    st = f(x.ctypes.data, w.ctypes.data, fold.ctypes.data, M, N, K, in_scales.ctypes.data, site[0], site[1], use_tc,
           folded.ctypes.data, codes.ctypes.data, scales.ctypes.data, status.ctypes.data)
    assert st == 0
    return folded, codes, scales, status


def tc_launches(lib):
    f = lib.dll.sslm_b200_tc_stats
    f.argtypes = [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_int32)]
    n, r, why = C.c_uint64(0), C.c_uint64(0), C.c_int32(0)
    assert f(C.byref(n), C.byref(r), C.byref(why)) == 0
    assert r.value == 0, "tensor-core path declined a launch, reason %d" % why.value
    return n.value


def tc_variants(lib):
    """launches per tile shape of the tensor-core kernel: [128x64, 128x128, 256x64, 256x128]"""
    f = lib.dll.sslm_b200_tc_variant_counts
    f.argtypes = [C.POINTER(C.c_uint64), C.c_int32]
    c = (C.c_uint64 * 4)()
    assert f(c, 4) == 0
    return list(c)


LINEAR_CASES = [  # (K, N, M): every M class, ragged N, the real 1.5B K/V and hidden shapes
    (1536, 256, 1), (1536, 256, 16), (1536, 256, 128), (1536, 1536, 1), (1536, 1536, 5), (1536, 1536, 130),
    (8960, 1536, 1), (8960, 1536, 16), (1536, 8960, 2), (1536, 8960, 64), (128, 77, 3), (16, 1, 1), (256, 333, 257),
    (1536, 4099, 9), (1536, 8960, 1), (896, 4864, 1), (4864, 896, 3), (2048, 11008, 1), (11008, 2048, 8), (48, 50, 7),
    # few output tiles and a long K: the tensor-core kernel splits K across blocks (3 to 16 slices)
    (8960, 1536, 256), (8960, 100, 200), (1536, 2048, 256), (4096, 64, 129),
    # the shapes of the serving benchmark's step (256 rows) and of prefill chunks: the 256-row tiles
    (1536, 17920, 256), (1536, 8960, 512), (256, 9600, 200), (1536, 1536, 512),
]
# which tile shape each case must run on with tensor cores requested (index into tc_variants)
LINEAR_VARIANT = {(1536, 17920, 256): 3, (1536, 8960, 512): 3, (256, 9600, 200): 2, (1536, 1536, 512): 1,
                  (1536, 256, 16): 0, (1536, 1536, 130): 0}


def linear_case_inputs(K, N, M):
    rng = np.random.default_rng(K * 131 + N * 17 + M)
    x = rng.integers(-127, 128, (M, K)).astype(np.int8)
    w = rng.integers(-127, 128, (N, K)).astype(np.int8)
    fold = np.zeros((N, 3), dtype=np.int32)
    fold[:, 1] = rng.integers(1 << 30, 1 << 31, N)
    fold[:, 2] = rng.integers(8, 21, N)
    fold[::7, 0] = 1                                  # some identity channels
    in_scales = np.stack([rng.integers(1 << 30, 1 << 31, M), np.full(M, -37)], axis=1).astype(np.int64)
    return x, w, fold, in_scales


def check_linear(gpu_lib, K, N, M, use_tc):
    x, w, fold, in_scales = linear_case_inputs(K, N, M)
    site = (1090717716, -44)
    want = oracle_linear(x, w, fold, in_scales, site)
    before, vbefore = tc_launches(gpu_lib), tc_variants(gpu_lib)
    got = gpu_linear(gpu_lib, x, w, fold, in_scales, site, use_tc)
    # no silent substitution: M > 8 with tensor cores requested must run the tcgen05 kernel
    assert tc_launches(gpu_lib) - before == (1 if (use_tc and M > 8) else 0)
    if use_tc and (K, N, M) in LINEAR_VARIANT:
        delta = [a - b for a, b in zip(tc_variants(gpu_lib), vbefore)]
        assert delta[LINEAR_VARIANT[(K, N, M)]] == 1 and sum(delta) == 1, delta
    assert (got[3] == want[3]).all()
    assert (got[0].astype(np.int64) == want[0]).all()
    assert (got[1] == want[1]).all()
    assert (got[2] == want[2]).all()


@pytest.mark.parametrize("K,N,M", LINEAR_CASES)
@pytest.mark.parametrize("use_tc", [0, 1])
def test_linear_layer_sweep(gpu_lib, K, N, M, use_tc):
    check_linear(gpu_lib, K, N, M, use_tc)


@pytest.mark.parametrize("K,N,M", [(1536, 8960, 2048), (8960, 1536, 2048), (1536, 1536, 2048), (1536, 256, 2048),
                                   (8960, 1536, 512), (1536, 256, 512)])
def test_linear_layer_prefill_shapes(gpu_lib, K, N, M):
    """The 2048- and 512-row cells of the standalone linear-layer grid (tensor-core kernel)."""
    check_linear(gpu_lib, K, N, M, 1)


@pytest.mark.parametrize("M,use_tc", [(1, 0), (4, 0), (16, 1), (128, 1), (300, 1)])
@pytest.mark.parametrize("want_rows", [False, True])
def test_vocabulary_head_form(gpu_lib, M, use_tc, want_rows):
    """K 1536 x N 151936, the logits form: exact int32 rows, narrowing check and the greedy token with
    the lowest-index rule on planted ties (two identical weight rows that hold the row maximum)."""
    K, N = 1536, 151936
    rng = np.random.default_rng(1000 + M)
    x = rng.integers(-127, 128, (M, K)).astype(np.int8)
    w = rng.integers(-127, 128, (N, K)).astype(np.int8)
    # the largest possible logit of row 0, twice: channel 90001 and channel 131 tie; plus an exact
    # duplicate pair elsewhere for the other rows
    peak = np.where(x[0] >= 0, 127, -127).astype(np.int8)
    w[90001] = peak
    w[131] = peak
    w[N - 1] = w[70000]
    f = gpu_lib.dll.sslm_b200_logits
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    rows = np.zeros((M, N), dtype=np.int32) if want_rows else None
    toks = np.zeros(M, dtype=np.int32)
    assert f(x.ctypes.data, w.ctypes.data, M, N, K, use_tc, rows.ctypes.data if want_rows else None, toks.ctypes.data) == 0
    acc = cpu_gemm(x, w)
    shim = H.ref_shim()
    for m in range(M):
        if shim is not None:      # the reference's own narrowing and argmax
            narrow = np.zeros(N, dtype=np.int32)
            assert shim.refshim_narrow_row(acc[m].ctypes.data, N, narrow.ctypes.data) == 0
            want_tok = shim.refshim_argmax(narrow.ctypes.data, N)
        else:
            narrow = acc[m].astype(np.int32)
            want_tok = int(np.argmax(narrow))
        assert toks[m] == want_tok, m
        if want_rows:
            assert (rows[m] == narrow).all(), m
    assert toks[0] == 131


@pytest.mark.parametrize("K,N,M", [(1536, 512, 256), (256, 384, 40), (1536, 300, 130)])
def test_linear_fold_forms(gpu_lib, K, N, M):
    """Tiles whose columns all take the epilogue's one-rounding fold (every shift 0..31, multipliers of
    both signs and small magnitude), and tiles where a single identity / INT32_MIN-multiplier column
    sends the whole tile to the two-step fold."""
    rng = np.random.default_rng(K + N + M)
    x = rng.integers(-127, 128, (M, K)).astype(np.int8)
    w = rng.integers(-127, 128, (N, K)).astype(np.int8)
    fold = np.zeros((N, 3), dtype=np.int32)
    fold[:, 1] = rng.integers(1 << 30, 1 << 31, N)
    fold[1::3, 1] = -fold[1::3, 1]
    fold[2::11, 1] = rng.integers(-(1 << 16), 1 << 16, fold[2::11, 1].size)
    fold[:, 2] = np.arange(N) % 32
    if N > 300:                      # the second half of the columns: one odd column per 64
        fold[N // 2 + 5::128, 0] = 1
        fold[N // 2 + 70::128, 1] = -(1 << 31)
    in_scales = np.stack([rng.integers(1 << 30, 1 << 31, M), np.full(M, -37)], axis=1).astype(np.int64)
    site = (1090717716, -44)
    want = oracle_linear(x, w, fold, in_scales, site)
    for use_tc in (0, 1):
        got = gpu_linear(gpu_lib, x, w, fold, in_scales, site, use_tc)
        assert (got[3] == want[3]).all()
        assert (got[0].astype(np.int64) == want[0]).all()
        assert (got[1] == want[1]).all()
        assert (got[2] == want[2]).all()


def test_linear_layer_extremes(gpu_lib):
    """All-(-127) x all-(-128) rows at the largest K; all-zero rows; identity fold overflow to the funnel's reject."""
    K, N, M = 8960, 40, 3
    x = np.full((M, K), -127, dtype=np.int8)
    x[1] = 0
    w = np.full((N, K), -128, dtype=np.int8)
    fold = np.zeros((N, 3), dtype=np.int32)
    fold[:, 0] = 1
    in_scales = np.array([[1 << 30, -37]] * M, dtype=np.int64)
    want = oracle_linear(x, w, fold, in_scales, (1090717716, -44))
    for use_tc in (0, 1):
        got = gpu_linear(gpu_lib, x, w, fold, in_scales, (1090717716, -44), use_tc)
        for a, b in zip(got, want):
            assert (np.asarray(a, dtype=np.int64) == np.asarray(b, dtype=np.int64)).all()


def test_status_paths(gpu_lib):
    sh = A.SHAPES["tiny"]
    art = A.build_synthetic_model("tiny", 909, 24)
    eng = abi.Engine(gpu_lib, art, blocks=1, max_chunk=32)
    assert gpu_lib.sslm_kv_block_size(eng.model) == sh.layers * 24 * sh.kv_heads * sh.head_dim * 2
    extra = abi._H()
    assert gpu_lib.sslm_seq_create(eng.model, C.byref(eng.pool), C.byref(extra)) == 0
    third = abi._H()
    assert gpu_lib.sslm_seq_create(eng.model, C.byref(eng.pool), C.byref(third)) == abi.ST["SSLM_KV_POOL_EXHAUSTED"]
    assert gpu_lib.sslm_model_unmap(eng.model) == abi.ST["SSLM_MODEL_HAS_LIVE_SEQUENCES"]
    assert gpu_lib.sslm_kv_pool_destroy(eng.pool) == abi.ST["SSLM_POOL_HAS_LIVE_HANDLES"]
    s = abi.Sequence.__new__(abi.Sequence)
    s.eng, s.handle = eng, extra
    eng.seqs.append(s)
    # nothing to decode from yet
    st, _ = eng.decode_step([s], 1)
    assert st == abi.ST["SSLM_INVALID_ARGUMENT"]
    st, _ = eng.decode_step([s], sh.layers + 1)
    assert st == abi.ST["SSLM_INVALID_ARGUMENT"]
    # a bad token id stops the chunk after the admitted prefix
    toks = np.array([1, 2, 3, sh.vocab, 4], dtype=np.int32)
    consumed = C.c_int32(0)
    st = gpu_lib.sslm_prefill(eng.model, s.handle, toks.ctypes.data_as(C.POINTER(C.c_int32)), 5, 32, 0, eng.ws, C.byref(consumed))
    assert (st, consumed.value) == (abi.ST["SSLM_TOKEN_ID_OUT_OF_RANGE"], 3)
    # context cap: 24 positions in total
    more = A.stream_uniform(3, "p", 30, 0, sh.vocab - 1).astype(np.int32)
    st = gpu_lib.sslm_prefill(eng.model, s.handle, more.ctypes.data_as(C.POINTER(C.c_int32)), 30, 32, 0, eng.ws, C.byref(consumed))
    assert (st, consumed.value) == (abi.ST["SSLM_CONTEXT_CAP_EXCEEDED"], 21)
    st, t = eng.decode_step([s], sh.layers)     # pending logits are still served
    assert st == 0 and t[0] >= 0
    st, t = eng.decode_step([s], sh.layers)     # no room for another position
    assert st == abi.ST["SSLM_CONTEXT_CAP_EXCEEDED"] and t[0] == -1
    # the oracle agrees on what the sequence holds
    pm = H.PortModel(art)
    ps = H.PortSeq(pm)
    assert ps.prefill(np.concatenate([toks[:3], more[:21]])) == 0
    blob = abi.parse_save_blob(s.save(), sh.hidden)
    assert blob["kv"] == ps.kv.tobytes() and blob["context_length"] == 24
    # a released handle reports -3 and does not disturb its neighbours
    s.release()
    ghost = (abi._H * 1)(extra)
    out = (C.c_int32 * 1)()
    params = abi.SslmDecodeParams(layer_budget=1)
    assert gpu_lib.sslm_decode_step(eng.model, ghost, 1, C.byref(params), eng.ws, out) == 0 and out[0] == -3
    eng.close()


def test_artifact_rejections(gpu_lib):
    art = bytearray(A.build_synthetic_model("tiny", 1, 16))
    out = abi._H()
    buf = np.frombuffer(bytes(art), dtype=np.uint8)
    assert gpu_lib.sslm_model_map(buf.ctypes.data, buf.size - 1, C.byref(out)) == abi.ST["SSLM_ARTIFACT_REJECTED"]
    art[200] ^= 1   # integrity hash no longer matches
    buf = np.frombuffer(bytes(art), dtype=np.uint8)
    assert gpu_lib.sslm_model_map(buf.ctypes.data, buf.size, C.byref(out)) == abi.ST["SSLM_ARTIFACT_REJECTED"]
    assert gpu_lib.sslm_model_map(None, 10, C.byref(out)) == abi.ST["SSLM_INVALID_ARGUMENT"]
    # adapter bound to another base
    base = A.build_synthetic_model("tiny", 2, 16)
    other = A.build_synthetic_model("tiny", 3, 16)
    eng = abi.Engine(gpu_lib, base, blocks=1)
    ad = np.frombuffer(A.build_synthetic_adapter(other, 5), dtype=np.uint8)
    h = abi._H()
    assert gpu_lib.sslm_adapter_map(ad.ctypes.data, ad.size, eng.model, C.byref(h)) == abi.ST["SSLM_ADAPTER_MODEL_MISMATCH"]
    eng.close()


def test_option_g_flag_is_ignored_like_the_reference(gpu_lib):
    sh = A.SHAPES["tiny"]
    art = A.build_synthetic_model("tiny", 0xF1A6, 48, flags=1)
    prompt = A.stream_uniform(31, "p", 14, 0, sh.vocab - 1)
    ptoks, ps = run_port(art, prompt, 8)
    eng = abi.Engine(gpu_lib, art, blocks=1, max_chunk=16)
    s = eng.new_seq()
    s.prefill(prompt, 16)
    assert s.decode(8, sh.layers) == ptoks
    assert abi.parse_save_blob(s.save(), sh.hidden)["kv"] == ps.kv.tobytes()
    eng.close()


def test_sequences_of_two_pools_in_one_decode_call(gpu_lib):
    """One sslm_decode_step over sequences that live in different KV pools of the same model (the
    reference takes them: every sequence carries its own block). Pools of different sizes, the
    handles interleaved; every sequence must equal its own single-sequence run on the CPU."""
    sh = A.SHAPES["small"]
    art = A.build_synthetic_model("small", 2027, 96)
    lens = [21, 5, 40, 33, 12]
    prompts = [A.stream_uniform(300 + i, "p", n, 0, sh.vocab - 1) for i, n in enumerate(lens)]
    want = []
    for p in prompts:
        toks, ps = run_port(art, p, 5)
        want.append((toks, ps.kv.tobytes(), ps.s.kv_saturation_count))
    eng = abi.Engine(gpu_lib, art, blocks=2, max_batch=8, max_chunk=64)
    # a second, larger pool on the same model
    need = eng.block_size * 5 + gpu_lib.sslm_kv_pool_overhead_size(eng.model, 5)
    raw, ptr = abi._aligned_buffer(need)
    pool2 = abi._H()
    assert gpu_lib.sslm_kv_pool_create(eng.model, ptr, need, 5, C.byref(pool2)) == 0
    seqs = []
    for i in range(len(lens)):
        if i % 2 == 0:
            s = abi.Sequence.__new__(abi.Sequence)
            s.eng, s.handle = eng, abi._H()
            assert gpu_lib.sslm_seq_create(eng.model, C.byref(pool2), C.byref(s.handle)) == 0
            eng.seqs.append(s)
        else:
            s = eng.new_seq()
        seqs.append(s)
    for s, p in zip(seqs, prompts):
        s.prefill(p, 64)
    got = [[] for _ in lens]
    while len(got[0]) < 5:
        st, toks = eng.decode_step(seqs, 2)
        assert st == 0
        for g, t in zip(got, toks):
            if t >= 0:
                g.append(t)
    for i, s in enumerate(seqs):
        blob = abi.parse_save_blob(s.save(), sh.hidden)
        assert got[i] == want[i][0], i
        assert blob["kv"] == want[i][1], i
        assert blob["kv_saturation_count"] == want[i][2], i
    for s in list(seqs):
        s.release()
    assert gpu_lib.sslm_kv_pool_destroy(pool2) == 0
    eng.close()


@pytest.mark.parametrize("shape,plen", [("small", 530), ("tiny", 300)])
def test_attention_row_cut_into_slices(gpu_lib, shape, plen):
    """Attention splits a row along its width over the blocks of a cluster (1 to 16 slices per kv
    head; with few slices the cluster also holds both kv heads and runs the context funnel itself,
    with many it does not). Every cut must give the CPU oracle's tokens, K/V and scale, in prefill
    (many rows, ascending widths) and in decode (one row)."""
    sh = A.SHAPES[shape]
    art = A.build_synthetic_model(shape, 0xA77E, 640)
    prompt = A.stream_uniform(0xA77E, "prompt", plen, 0, sh.vocab - 1)
    want_toks, ps = run_port(art, prompt, 6)
    f = gpu_lib.dll.sslm_b200_set_attention_splits
    f.argtypes = [C.c_int32]
    try:
        for splits in (1, 2, 4, 8, 16, 0):
            assert f(splits) == 0
            eng = abi.Engine(gpu_lib, art, blocks=1, max_chunk=256)
            s = eng.new_seq()
            s.prefill(prompt, 200)
            toks = s.decode(6, 1 + splits % 2)
            blob = abi.parse_save_blob(s.save(), sh.hidden)
            eng.close()
            assert toks == want_toks, splits
            assert blob["kv"] == ps.kv.tobytes(), splits
            assert blob["hidden_scale"] == (ps.s.hidden_scale.m, ps.s.hidden_scale.e), splits
            assert blob["kv_saturation_count"] == ps.s.kv_saturation_count, splits
    finally:
        f(0)

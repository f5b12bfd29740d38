"""Artifacts and adapters that leave an integer-domain gate of the forward pass on purpose, and one
driver that runs a case through the sslm_* verbs of whichever library it is given (the reference's
CPU library when the records are made, the CUDA library in the GPU test). Nothing here faults or
hangs anything: every failure is a status code the forward pass returns by design.

A record holds, for every call of the case, (verb, status, consumed or tokens), and the SHA-256 of
each sequence's save blob after every call -- so "a refused call leaves the sequence untouched"
and "sequences before the failing one have advanced" are part of what is compared.
"""
import ctypes as C
import hashlib

import numpy as np

from superslm_b200 import abi, artifact as A

SEED = 0x53534C4D0000F000
CANON = 1 << 30

# name -> (constant overrides, what the case exercises)
ARTIFACTS = {
    # sm = Combine(S[q], softmax_khead) far below the window: a derivation shift goes negative
    "khead_exponent_low": ({"layer0.softmax_khead0": (CANON, -80)}, "IExpScaleDerivationOutOfDomain in layer 0"),
    # ... far above it: q_ln2 floors to 0, every element's construction is refused -> NUMERIC_STEP_REFUSED
    "khead_exponent_high": ({"layer1.softmax_khead1": (CANON, -3)}, "softmax kernel refusal in layer 1"),
    # a tiny stream scale: the rescaled branch of the first residual site leaves int64
    "residual_ratio": ({"embed": (CANON, -80)}, "ResidualReconciliationMagnitudeOutOfDomain at layer 0's attention residual"),
    # the gate scale leaves SiluSigmoidQ15's domain
    "silu_scale": ({"layer0.mlp_norm": (CANON, 7)}, "SiluScaleOutOfDomain in layer 0"),
    # two sites of one layer would fail: the earlier one in program order decides
    "two_sites": ({"embed": (CANON, -80), "layer0.mlp_norm": (CANON, 7)}, "residual before SiLU"),
    # a site constant that drives the folded mantissa chain to its edge
    "q_site_exponent": ({"layer0.q_proj": ((1 << 31) - 1, 7)}, "q projection site at the constants' upper edge"),
    # fails only in the second layer: the first layer's K/V row was written and must not count
    "second_layer": ({"layer1.mlp_norm": (CANON, 7)}, "SiluScaleOutOfDomain in layer 1"),
    # the same with q/k/v biases large enough to saturate the K/V landing: the reference has counted the
    # landings its walk reached into kv_saturation_count when it refuses, and keeps them
    "second_layer_saturating": ({"layer1.mlp_norm": (CANON, 7)}, "refused after saturating landings of two layers"),
    # ... and a refusal inside the per-token stage of the first layer (only token 0's landing counts)
    "khead_low_saturating": ({"layer0.softmax_khead0": (CANON, -80)}, "refused in the per-token stage after one landing"),
}
# artifacts built with a BIA1 section of this many bits (0: none)
BIAS_BITS = {"second_layer_saturating": 33, "khead_low_saturating": 33}


def build(name, shape="tiny", cap=48):
    return A.build_synthetic_model(shape, SEED ^ (hash_name(name) & 0xFFFF), cap, bias_bits=BIAS_BITS.get(name, 0),
                                   const_overrides=ARTIFACTS[name][0])


def hash_name(name):
    return int.from_bytes(hashlib.sha256(name.encode()).digest()[:4], "little")


def _state_digest(lib, seq_handle, sh, cap):
    """SHA-256 of what a sequence observably holds: the save blob's header fields, the mid-token
    residual, and the K/V of the positions that count (a layer that ran for the token in flight
    holds one more). Bytes at positions beyond those are scratch of unfinished work in the
    reference's block and unwritten in a paged pool; they are not state."""
    n = C.c_size_t(0)
    lib.sslm_seq_save(seq_handle, None, C.byref(n))
    buf = (C.c_uint8 * n.value)()
    st = lib.sslm_seq_save(seq_handle, buf, C.byref(n))
    if st != 0:
        return "save:%d" % st
    blob = abi.parse_save_blob(bytes(buf[:n.value]), sh.hidden)
    kv = np.frombuffer(blob["kv"], dtype=np.int8).reshape(sh.layers, 2, sh.kv_heads, cap, sh.head_dim).copy()
    for layer in range(sh.layers):
        valid = blob["context_length"] + (1 if layer < blob["layer_index"] else 0)
        kv[layer, :, :, valid:, :] = 0
    h = hashlib.sha256()
    h.update(repr((blob["context_length"], blob["layer_index"], blob["current_token"], blob["hidden_scale"],
                   blob["kv_saturation_count"])).encode())
    h.update(blob["residual"])
    h.update(kv.tobytes())
    return h.hexdigest()


def _prefill(lib, eng, seq, tokens, chunk):
    toks = np.ascontiguousarray(tokens, dtype=np.int32)
    consumed = C.c_int32(0)
    st = lib.sslm_prefill(eng.model, seq.handle, toks.ctypes.data_as(C.POINTER(C.c_int32)), toks.size, chunk, 0, eng.ws,
                          C.byref(consumed))
    return st, consumed.value


def run_artifact_case(lib, name, shape="tiny", cap=48):
    """Prefill (one chunk), then decode calls at two budgets, on a hostile artifact."""
    sh = A.SHAPES[shape]
    art = build(name, shape, cap)
    eng = abi.Engine(lib, art, blocks=2, max_batch=2, max_chunk=16)
    rec = []
    try:
        s = eng.new_seq()
        prompt = A.stream_uniform(SEED, "p." + name, 9, 0, sh.vocab - 1)
        rec.append(("fresh", 0, _state_digest(lib, s.handle, sh, cap)))
        st, consumed = _prefill(lib, eng, s, prompt, 16)
        rec.append(("prefill", st, consumed, _state_digest(lib, s.handle, sh, cap)))
        # a one-token prefill each: the smallest call that reaches the failing site
        st, consumed = _prefill(lib, eng, s, prompt[:1], 1)
        rec.append(("prefill1", st, consumed, _state_digest(lib, s.handle, sh, cap)))
        for budget in (1, sh.layers):
            st, toks = eng.decode_step([s], budget)
            rec.append(("decode", st, list(toks), _state_digest(lib, s.handle, sh, cap)))
    finally:
        eng.close()
    return rec


def run_batch_case(lib, cap=48):
    """Five sequences on a healthy artifact; sequence 3 carries an adapter whose delta fold
    amplifies by 2^31 (the q row leaves the funnel's domain), the others none or a mild one. One
    sslm_decode_step over all five: the reference advances 0..2, stops at 3 and leaves 3 and 4
    untouched."""
    sh = A.SHAPES["tiny"]
    art = A.build_synthetic_model("tiny", SEED ^ 0x77, cap)
    mild = A.build_synthetic_adapter(art, 5)
    wild = A.build_synthetic_adapter(art, 6, d_exp=(-31, -31))
    eng = abi.Engine(lib, art, blocks=5, max_batch=5, max_chunk=16)
    rec = []
    try:
        h_mild, h_wild = eng.map_adapter(mild), eng.map_adapter(wild)
        seqs = [eng.new_seq() for _ in range(5)]
        seqs[1].set_adapter(h_mild)
        for i, s in enumerate(seqs):
            p = A.stream_uniform(SEED, "bp%d" % i, 6 + i, 0, sh.vocab - 1)
            st, consumed = _prefill(lib, eng, s, p, 16)
            rec.append(("prefill", st, consumed))
        st, toks = eng.decode_step(seqs, sh.layers)       # pending logits: no layer runs
        rec.append(("decode0", st, list(toks)))
        # the wild adapter goes on at a token boundary, then one full step over all five
        st = lib.sslm_seq_set_adapter(seqs[3].handle, h_wild)
        rec.append(("set_adapter", st))
        before = [_state_digest(lib, s.handle, sh, cap) for s in seqs]
        out = (C.c_int32 * 5)(*([-9] * 5))
        arr = (abi._H * 5)(*[s.handle for s in seqs])
        params = abi.SslmDecodeParams(layer_budget=sh.layers)
        st = lib.sslm_decode_step(eng.model, arr, 5, C.byref(params), eng.ws, out)
        after = [_state_digest(lib, s.handle, sh, cap) for s in seqs]
        rec.append(("decode1", st, list(out)[:3], [a == b for a, b in zip(before, after)], after))
        # the failing sequence recovers once the adapter is gone
        st = lib.sslm_seq_set_adapter(seqs[3].handle, None)
        rec.append(("detach", st))
        st, toks = eng.decode_step(seqs[3:], sh.layers)
        rec.append(("decode2", st, list(toks), [_state_digest(lib, s.handle, sh, cap) for s in seqs[3:]]))
    finally:
        eng.close()
    return rec


def run_mid_token_case(lib, cap=48):
    """A failure in the second layer of a token decoded one layer per call: the first call commits
    layer 0, the second is refused and must leave the sequence exactly where the first left it
    (layer_index 1, the residual, the K/V row layer 0 wrote); swapping the adapter is refused
    mid-token; the same two calls with a healthy adapter then finish... the token stays refused
    as long as the adapter stays."""
    sh = A.SHAPES["tiny"]
    art = A.build_synthetic_model("tiny", SEED ^ 0x78, cap)
    bad = A.build_synthetic_adapter(art, 9, layer_d_exp={1: (-31, -31)})
    eng = abi.Engine(lib, art, blocks=1, max_batch=1, max_chunk=16)
    rec = []
    try:
        h = eng.map_adapter(bad)
        s = eng.new_seq()
        p = A.stream_uniform(SEED, "mid", 11, 0, sh.vocab - 1)
        rec.append(("prefill",) + _prefill(lib, eng, s, p, 16))
        st, toks = eng.decode_step([s], 1)
        rec.append(("decode_pending", st, list(toks)))
        rec.append(("set_adapter", lib.sslm_seq_set_adapter(s.handle, h)))
        for _ in range(3):
            st, toks = eng.decode_step([s], 1)
            rec.append(("decode_layer", st, list(toks), _state_digest(lib, s.handle, sh, cap)))
        rec.append(("swap_mid_token", lib.sslm_seq_set_adapter(s.handle, None)))
    finally:
        eng.close()
    return rec


def run_partial_commit_case(lib, cap=48):
    """A step with a budget of two layers whose second layer is refused: the reference commits layer
    by layer, so the sequence is left after the first layer (layer_index 1, that layer's stream and
    K/V row), and a later call with a healthy adapter cannot be made without finishing the token:
    the swap is refused mid-token."""
    sh = A.SHAPES["tiny"]
    art = A.build_synthetic_model("tiny", SEED ^ 0x79, cap)
    bad = A.build_synthetic_adapter(art, 10, layer_d_exp={1: (-31, -31)})
    eng = abi.Engine(lib, art, blocks=1, max_batch=1, max_chunk=16)
    rec = []
    try:
        h = eng.map_adapter(bad)
        s = eng.new_seq()
        p = A.stream_uniform(SEED, "partial", 7, 0, sh.vocab - 1)
        rec.append(("prefill",) + _prefill(lib, eng, s, p, 16))
        st, toks = eng.decode_step([s], 2)
        rec.append(("decode_pending", st, list(toks)))
        rec.append(("set_adapter", lib.sslm_seq_set_adapter(s.handle, h)))
        for _ in range(2):
            st, toks = eng.decode_step([s], 2)
            rec.append(("decode_two_layers", st, list(toks), _state_digest(lib, s.handle, sh, cap)))
        rec.append(("swap_mid_token", lib.sslm_seq_set_adapter(s.handle, None)))
    finally:
        eng.close()
    return rec


def all_records(lib):
    """Every case of this module on one library, as JSON-friendly lists."""
    out = {name: run_artifact_case(lib, name) for name in ARTIFACTS}
    out["batch_row3_refused"] = run_batch_case(lib)
    out["mid_token_refused"] = run_mid_token_case(lib)
    out["partial_commit"] = run_partial_commit_case(lib)
    import json
    return json.loads(json.dumps(out))

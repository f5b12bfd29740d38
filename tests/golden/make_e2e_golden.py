"""Generates tests/golden/e2e_golden.json by running the REFERENCE library (compiled from
its own sources into oracle/_ref) through its public sslm_* ABI on seeded synthetic
artifacts. The artifacts are regenerated from (shape, seed, context_cap) by
superslm_b200.artifact, so only the small result records are committed.

    python tests/golden/make_e2e_golden.py
"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import harness as H  # noqa: E402
from superslm_b200 import abi, artifact as A  # noqa: E402

CASES = [
    # name, shape, seed, context_cap, prompt_len, decode_tokens, adapter seeds (attach A, then swap to B)
    ("tiny", "tiny", 0x53534C4D00000000, 64, 20, 12, None),
    ("small", "small", 0x53534C4D00000001, 160, 70, 24, None),
    ("small_dense", "small", 0x53534C4D00000002, 96, 40, 10, None),
    ("tiny_lora", "tiny", 0x53534C4D00000003, 64, 18, 10, (11, 12)),
    # q/k/v biases (BIA1), trailing field = magnitude in bits; with an adapter (delta, then bias);
    # large enough to saturate the K/V landing
    ("tiny_bias", "tiny", 0x53534C4D00000004, 64, 20, 12, None, 29),
    ("tiny_bias_lora", "tiny", 0x53534C4D00000005, 64, 18, 10, (13, 14), 30),
    ("small_bias_saturating", "small", 0x53534C4D00000006, 96, 40, 10, None, 33),
]


def run_case(lib, name, shape, seed, cap, npf, ndec, adapters, bias_bits=0):
    sh = A.SHAPES[shape]
    lo, hi = (8, 11) if name.endswith("dense") else (8, 20)
    art = A.build_synthetic_model(shape, seed, cap, lo, hi, bias_bits)
    prompt = A.stream_uniform(seed ^ 0xABCDEF, "prompt", npf, 0, sh.vocab - 1)
    eng = abi.Engine(lib, art, blocks=1, max_chunk=64)
    s = eng.new_seq()
    if adapters:
        ha = eng.map_adapter(A.build_synthetic_adapter(art, adapters[0]))
        hb = eng.map_adapter(A.build_synthetic_adapter(art, adapters[1]))
        s.set_adapter(ha)
    s.prefill(prompt, 64)
    toks = s.decode(ndec // 2, sh.layers)
    if adapters:
        s.set_adapter(None)
        s.set_adapter(hb)
    toks += s.decode(ndec - ndec // 2, sh.layers)
    blob = abi.parse_save_blob(s.save(), sh.hidden)
    eng.close()
    return {
        "shape": shape, "seed": seed, "context_cap": cap, "prompt_len": npf, "decode": ndec,
        "shift_lo": lo, "shift_hi": hi, "adapters": adapters, "bias_bits": bias_bits,
        "tokens": toks, "context_length": blob["context_length"],
        "hidden_scale": list(blob["hidden_scale"]), "kv_saturation_count": blob["kv_saturation_count"],
        "kv_sha256": hashlib.sha256(blob["kv"]).hexdigest(),
        "kv_nonzero": int(np.count_nonzero(np.frombuffer(blob["kv"], dtype=np.int8))),
    }


def main():
    lib = H.ref()
    assert lib is not None, "build oracle/_ref first (make -C oracle ref)"
    out = {c[0]: run_case(lib, *c) for c in CASES}
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "e2e_golden.json")
    json.dump(out, open(dst, "w"), indent=1)
    for k, v in out.items():
        print(k, v["tokens"][:8], v["kv_saturation_count"], v["kv_nonzero"])


if __name__ == "__main__":
    main()

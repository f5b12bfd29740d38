"""Generates tests/golden/config_golden.json: the REFERENCE library's results on the benchmark
configurations at their stated shapes and context lengths.

The reference (compiled from its own sources into oracle/_ref) runs each case through its public
sslm_* verbs; the records keep tokens, the SHA-256 of the canonical K/V block, the carried scale
and the saturation counter. Full logit rows come from the plain-C restatement continued from the
reference's own saved state (at a token boundary a sequence is its K/V block, its length and the
token to embed next, so the restatement can pick the reference's blob up and produce the next
tokens with their int32 logit rows; its tokens are checked against the reference's here).

The artifacts are regenerated from (shape, seed, context_cap) by superslm_b200.artifact; only the
small records are committed. The long cases take minutes of CPU each; they run as parallel
processes.

    python tests/golden/make_config_golden.py            # all cases, in parallel
    python tests/golden/make_config_golden.py --case NAME     # one case into _config_parts/
    python tests/golden/make_config_golden.py --assemble       # write the JSON from the parts at hand
"""
import argparse
import ctypes as C
import hashlib
import json
import os
import subprocess
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)
from oracle import harness as H  # noqa: E402
from superslm_b200 import abi, artifact as A  # noqa: E402
from config_cases import CASES, build_case_artifacts, case_prompt  # noqa: E402


def port_logit_rows(art, blob_bytes, sh, n_rows, adapter=None):
    """Continue from a reference save blob (token boundary, next token pending) with the C
    restatement: returns [(token, sha256 of its int32 logit row)]."""
    blob = abi.parse_save_blob(blob_bytes, sh.hidden)
    assert blob["layer_index"] == 0 and blob["current_token"] >= 0
    pm = H.PortModel(art)
    ps = H.PortSeq(pm)
    if adapter is not None:
        ps.lora = pm.lora(adapter)
    ps.kv[:] = np.frombuffer(blob["kv"], dtype=np.int8)
    ps.s.context_length = blob["context_length"]
    ps.s.kv_saturation_count = blob["kv_saturation_count"]
    ps.s.layer_index = 0
    ps.current_token = blob["current_token"]
    ps.ready_for_logits = False
    out = []
    for _ in range(n_rows):
        st, tok, logits = ps.decode_step(sh.layers, want_logits=True)
        assert st == 0 and tok >= 0
        out.append((tok, hashlib.sha256(logits.tobytes()).hexdigest()))
    return out


def run_case(name):
    case = CASES[name]
    sh = A.SHAPES[case["shape"]]
    lib = H.ref()
    assert lib is not None, "build oracle/_ref first (make -C oracle ref)"
    t0 = time.time()
    art, adapters = build_case_artifacts(case)
    prompt = case_prompt(case)
    eng = abi.Engine(lib, art, blocks=1, max_chunk=case["cpu_chunk"])
    s = eng.new_seq()
    handles = [eng.map_adapter(a) for a in adapters]
    if case.get("attach") is not None:
        s.set_adapter(handles[case["attach"]])
    assert s.prefill(prompt, case["cpu_chunk"]) == len(prompt)
    t_prefill = time.time() - t0
    n = case["decode"]
    first = case.get("swap_after", n // 2)
    toks = s.decode(1, sh.layers)
    logit_rows = []
    if case.get("logit_rows", 0):
        cur = adapters[case["attach"]] if case.get("attach") is not None else None
        logit_rows = port_logit_rows(art, s.save(), sh, case["logit_rows"], cur)
    toks += s.decode(first - 1, sh.layers)
    if case.get("swap_to") is not None:
        s.set_adapter(None)
        s.set_adapter(handles[case["swap_to"]])
    toks += s.decode(n - first, sh.layers)
    for i, (tok, _) in enumerate(logit_rows):
        if 1 + i < first:
            assert tok == toks[1 + i], "restatement and reference disagree on token %d" % (1 + i)
    blob = abi.parse_save_blob(s.save(), sh.hidden)
    eng.close()
    rec = dict(case)
    rec.update({
        "tokens": toks, "context_length": blob["context_length"], "hidden_scale": list(blob["hidden_scale"]),
        "kv_saturation_count": blob["kv_saturation_count"], "kv_sha256": hashlib.sha256(blob["kv"]).hexdigest(),
        "kv_nonzero": int(np.count_nonzero(np.frombuffer(blob["kv"], dtype=np.int8))),
        "logit_sha256": [h for _, h in logit_rows],
        "cpu_seconds": {"prefill": round(t_prefill, 1), "total": round(time.time() - t0, 1)},
    })
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case")
    ap.add_argument("--jobs", type=int, default=4)
    ap.add_argument("--assemble", action="store_true")
    args = ap.parse_args()
    outdir = os.path.join(HERE, "_config_parts")
    os.makedirs(outdir, exist_ok=True)
    if args.case:
        rec = run_case(args.case)
        json.dump(rec, open(os.path.join(outdir, args.case + ".json"), "w"))
        print(args.case, rec["tokens"][:6], rec["kv_saturation_count"], rec["kv_nonzero"], rec["cpu_seconds"])
        return
    pending = [] if args.assemble else list(CASES)
    running = []
    while pending or running:
        while pending and len(running) < args.jobs:
            nm = pending.pop(0)
            running.append((nm, subprocess.Popen([sys.executable, os.path.abspath(__file__), "--case", nm])))
        time.sleep(2)
        for nm, p in list(running):
            if p.poll() is not None:
                assert p.returncode == 0, nm
                running.remove((nm, p))
    out = {nm: json.load(open(os.path.join(outdir, nm + ".json"))) for nm in CASES}
    json.dump(out, open(os.path.join(HERE, "config_golden.json"), "w"), indent=1)


if __name__ == "__main__":
    main()

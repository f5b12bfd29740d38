"""Generates tests/golden/bench_parity_golden.json: the REFERENCE library's results (oracle/_ref) on
sixteen of the serving benchmark's own sequences -- the shortest, the longest and fourteen spread
between them -- so that bench.py can compare the CUDA path with the CPU on the workload it times
without spending minutes of CPU on the GPU machine. Per sequence: the decoded tokens and a digest
of what the sequence holds afterwards (bench.sequence_digest: K/V of every layer and position,
carried scale, saturation counter). One sequence per host thread on one shared model.

    python tests/golden/make_bench_parity_golden.py
"""
import json
import os
import sys
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import bench  # noqa: E402
from oracle import harness as H  # noqa: E402
from superslm_b200 import abi, artifact as A  # noqa: E402

DECODE = 4


def main():
    args = bench.parse_args()
    sh = A.SHAPES[args.shape]
    lib = H.ref()
    assert lib is not None, "build oracle/_ref first (make -C oracle ref)"
    prompts = bench.workload_prompts(args.shape, args.seqs, args.prompt_lo, args.prompt_hi, 1)
    picks = bench.parity_sample(prompts, 16)
    cap = ((args.prompt_hi + DECODE + 16 + 15) // 16) * 16
    art = A.build_synthetic_model(args.shape, bench.SEED, cap)
    eng = abi.Engine(lib, art, blocks=len(picks), max_batch=1, max_chunk=args.prompt_hi)
    records = {}

    def work(i):
        s = eng.new_seq()
        wsz = lib.sslm_workspace_size(eng.model, eng.cfg)
        raw, ptr = abi._aligned_buffer(wsz)
        ws = abi._H()
        import ctypes as C
        assert lib.sslm_workspace_create(eng.model, C.byref(eng.cfg), ptr, wsz, C.byref(ws)) == 0
        p = prompts[i]
        consumed = C.c_int32(0)
        assert lib.sslm_prefill(eng.model, s.handle, p.ctypes.data_as(C.POINTER(C.c_int32)), p.size, p.size, 0, ws,
                                C.byref(consumed)) == 0 and consumed.value == p.size
        toks = []
        params = abi.SslmDecodeParams(layer_budget=sh.layers)
        arr = (abi._H * 1)(s.handle)
        out = (C.c_int32 * 1)()
        for _ in range(DECODE):
            assert lib.sslm_decode_step(eng.model, arr, 1, C.byref(params), ws, out) == 0
            toks.append(int(out[0]))
        rec = bench.sequence_digest(s.save(), sh)
        rec["tokens"] = toks
        rec["prompt_len"] = int(p.size)
        records[str(i)] = rec
        lib.sslm_workspace_destroy(ws)
        print("sequence", i, "len", p.size, toks, flush=True)

    threads = [threading.Thread(target=work, args=(i,)) for i in picks]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert len(records) == len(picks)
    eng.close()
    out = {"shape": args.shape, "seed": bench.SEED, "prompt_lo": args.prompt_lo, "prompt_hi": args.prompt_hi,
           "sequences": args.seqs, "decode": DECODE, "records": records}
    json.dump(out, open(os.path.join(HERE, "bench_parity_golden.json"), "w"), indent=1)


if __name__ == "__main__":
    main()

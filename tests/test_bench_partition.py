"""The multi-GPU plumbing of bench.py on CPU: two ranks over gloo. The data path has no
collective (every rank owns whole sequences and a model replica); torch.distributed only
carries the barrier and the max / sum of the per-rank timings and token counts."""
import json
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

RANK_PROGRAM = r"""
import json, sys
sys.path.insert(0, %(root)r)
import bench
rank, world, local, barrier, rmax, rsum = bench.dist_setup(2)
barrier()
weak_ids, weak_stream = bench.partition(6, world, rank, False)
strong_ids, strong_stream = bench.partition(7, world, rank, True)
prompts = bench.workload_prompts("tiny", 6, 4, 9, weak_stream)
out = {
    "rank": rank, "world": world, "local": local,
    "weak_ids": weak_ids, "weak_stream": weak_stream,
    "strong_ids": strong_ids, "strong_stream": strong_stream,
    "prompt_lens": [int(p.size) for p in prompts], "first_prompt": [int(t) for t in prompts[0]],
    "max": rmax(10.0 + rank), "sum": rsum(100 * (rank + 1)),
}
barrier()
print("RESULT " + json.dumps(out))
"""


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_two_ranks():
    port = free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="")
        procs.append(subprocess.Popen([sys.executable, "-c", RANK_PROGRAM % {"root": ROOT}], env=env, cwd=ROOT,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    results = []
    for p in procs:
        out, err = p.communicate(timeout=240)
        assert p.returncode == 0, err[-2000:]
        line = [l for l in out.splitlines() if l.startswith("RESULT ")][-1]
        results.append(json.loads(line[len("RESULT "):]))
    return sorted(results, key=lambda r: r["rank"])


def test_two_gloo_ranks_partition_and_reduce():
    r0, r1 = run_two_ranks()
    assert (r0["world"], r1["world"]) == (2, 2) and (r0["rank"], r1["rank"]) == (0, 1)
    # weak scaling: every rank serves its own full set of sequences, from its own prompt stream
    assert r0["weak_ids"] == r1["weak_ids"] == list(range(6))
    assert r0["weak_stream"] != r1["weak_stream"]
    assert r0["first_prompt"] != r1["first_prompt"] or r0["prompt_lens"] != r1["prompt_lens"]
    assert all(4 <= n <= 9 for n in r0["prompt_lens"] + r1["prompt_lens"])
    # strong scaling: one global list dealt round-robin, disjoint and complete
    assert sorted(r0["strong_ids"] + r1["strong_ids"]) == list(range(7))
    assert not set(r0["strong_ids"]) & set(r1["strong_ids"])
    assert r0["strong_stream"] == r1["strong_stream"]
    # the reported time is the slowest rank's, the token count the sum over ranks
    assert r0["max"] == r1["max"] == 11.0
    assert r0["sum"] == r1["sum"] == 300.0


def test_single_process_needs_no_process_group():
    import importlib
    sys.path.insert(0, ROOT)
    bench = importlib.import_module("bench")
    env = {k: os.environ.pop(k, None) for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK")}
    try:
        rank, world, local, barrier, rmax, rsum = bench.dist_setup(1)
    finally:
        for k, v in env.items():
            if v is not None:
                os.environ[k] = v
    assert (rank, world, local) == (0, 1, 0)
    barrier()
    assert rmax(3.5) == 3.5 and rsum(7) == 7
    assert bench.partition(5, 1, 0, False) == (list(range(5)), 1)

#!/usr/bin/env python
"""Benchmark of the integer forward pass behind the sslm_* C ABI.

Workload (BASELINE config 3, the multi-sequence serving case on the 1.5B-shape model):
a seeded synthetic Qwen2.5-1.5B-architecture artifact (28 layers, d_model 1536, 12/2
heads of 128, FFN 8960, vocab 151936, tied head; int8 weights uniform in [-127,127],
fold multipliers in [2^30,2^31), shifts 8..20), `--seqs` independent sequences with
prompt lengths uniform in [128,1024], chunk-batched prefill, then greedy decode over
16-token KV pages. One *step* = one sslm_decode_step over all of a rank's sequences
(one token per sequence, all 28 layers). Every decode step streams the full 1.5 GB of
weights, far more than the 126 MB L2, so no explicit L2 flush is needed between steps.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

`value` is decode tokens/s from device time (CUDA events inside the library, inputs
resident in HBM); `e2e` is the same through the C ABI from host buffers (descriptor
upload and token read-back included). With N > 1 every GPU holds a model replica and its
own sequences; no collective runs on the data path (NCCL only carries the barrier and
the max-over-ranks of the timings).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from superslm_b200 import abi, artifact as A  # noqa: E402

SEED = 0x53534C4D00000003
PROF_CLASSES = ["begin", "linear_qkv", "qkv_post", "attention", "ctx_funnel", "linear_o", "residual1",
                "linear_gate_up", "activation", "linear_down", "residual2", "head", "lora_u", "other"]


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="1.5b")
    ap.add_argument("--seqs", type=int, default=256, help="sequences per GPU (weak scaling)")
    ap.add_argument("--strong", action="store_true", help="partition --seqs across the GPUs instead")
    ap.add_argument("--prompt-lo", type=int, default=128)
    ap.add_argument("--prompt-hi", type=int, default=1024)
    ap.add_argument("--chunk", type=int, default=1024, help="prefill chunk budget")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-threads", type=int, default=0)
    return ap.parse_args()


def artifact_path(shape, cap):
    return "/dev/shm/sslm_bench_%s_%d_%x.sslm" % (shape, cap, SEED)


def get_artifact(shape, cap, rank, barrier):
    """Rank 0 generates the artifact once into shared memory; every rank reads it."""
    path = artifact_path(shape, cap)
    if rank == 0 and not os.path.exists(path):
        data = A.build_synthetic_model(shape, SEED, cap)
        with open(path + ".tmp", "wb") as f:
            f.write(data)
        os.replace(path + ".tmp", path)
    barrier()
    with open(path, "rb") as f:
        return f.read()


def workload_prompts(shape, n_seqs, lo, hi, stream):
    sh = A.SHAPES[shape]
    lens = A.stream_uniform(SEED ^ (0x1000 + stream), "prompt_len", n_seqs, lo, hi)
    return [A.stream_uniform(SEED ^ (0x2000 + stream), "prompt%d" % i, int(n), 0, sh.vocab - 1).astype(np.int32)
            for i, n in enumerate(lens)]


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.proc = None
        self.idx = device_index
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(device_index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def bind_extras(lib):
    d = lib.dll
    d.sslm_b200_set_device.argtypes = [C.c_int]
    d.sslm_b200_last_call_ms.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_uint64)]
    d.sslm_b200_profile.argtypes = [C.c_void_p, C.c_int32]
    d.sslm_b200_profile_read.argtypes = [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_uint64), C.c_int32]
    d.sslm_b200_model_device_bytes.argtypes = [C.c_void_p]
    d.sslm_b200_model_device_bytes.restype = C.c_size_t
    d.sslm_b200_tc_stats.argtypes = [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_int32)]
    return d


def last_call(d, ws):
    ms, n = C.c_float(0), C.c_uint64(0)
    d.sslm_b200_last_call_ms(ws, C.byref(ms), C.byref(n))
    return ms.value, n.value


# --------------------------------------------------------------------------- CPU arm
def cpu_reference_run(art, shape, threads, prefill_tokens, steps, warmup):
    """The reference's own CPU implementation (oracle/_ref, else the C restatement) on the
    host cores: `threads` sequences, one per thread (the reference is single-threaded per
    call and allows one sequence per thread on a shared read-only model)."""
    from oracle import harness as H
    sh = A.SHAPES[shape]
    prompts = workload_prompts(shape, threads, prefill_tokens, prefill_tokens, 999)
    ref = H.ref()
    kind = "reference" if ref is not None else "port"
    results = {}
    if ref is not None:
        eng = abi.Engine(ref, art, blocks=threads, max_batch=1, max_chunk=prefill_tokens)
        seqs = [eng.new_seq() for _ in range(threads)]
        wss = []
        for _ in range(threads):     # one workspace per concurrently running call
            wsz = ref.sslm_workspace_size(eng.model, C.byref(eng.cfg))
            raw, ptr = abi._aligned_buffer(wsz)
            h = abi._H()
            assert ref.sslm_workspace_create(eng.model, C.byref(eng.cfg), ptr, wsz, C.byref(h)) == 0
            wss.append((h, raw))

        def prefill(i):
            toks = prompts[i]
            consumed = C.c_int32(0)
            st = ref.sslm_prefill(eng.model, seqs[i].handle, toks.ctypes.data_as(C.POINTER(C.c_int32)), toks.size,
                                  toks.size, 0, wss[i][0], C.byref(consumed))
            assert st == 0 and consumed.value == toks.size

        def decode(i, n, out):
            params = abi.SslmDecodeParams(layer_budget=sh.layers)
            arr = (abi._H * 1)(seqs[i].handle)
            tok = (C.c_int32 * 1)()
            for _ in range(n):
                assert ref.sslm_decode_step(eng.model, arr, 1, C.byref(params), wss[i][0], tok) == 0
                out.append(tok[0])
    else:
        pm = H.PortModel(art)
        pseqs = [H.PortSeq(pm) for _ in range(threads)]

        def prefill(i):
            assert pseqs[i].prefill(prompts[i]) == 0

        def decode(i, n, out):
            out.extend(pseqs[i].decode(n, sh.layers))

    def parallel(fn, *a):
        ts = [threading.Thread(target=fn, args=(i,) + a) for i in range(threads)]
        t0 = time.perf_counter()
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return time.perf_counter() - t0

    t_prefill = parallel(prefill)
    outs = [[] for _ in range(threads)]
    parallel(lambda i: decode(i, 1 + warmup, outs[i]))        # pending logits + warm-up tokens
    t_decode = parallel(lambda i: decode(i, steps, outs[i]))
    results = {"kind": kind, "cores": threads, "prefill_tok_s": threads * prefill_tokens / t_prefill,
               "decode_tok_s": threads * steps / t_decode, "decode_s": t_decode, "tokens0": outs[0],
               "prompt0": prompts[0],
               "sample": "%d sequences (one per host thread), %d-token prompt each, %d timed decode tokens each "
                         "at context %d..%d" % (threads, prefill_tokens, steps, prefill_tokens + warmup,
                                                prefill_tokens + warmup + steps)}
    if ref is not None:
        for h, _ in wss:
            ref.sslm_workspace_destroy(h)
        eng.close()
    return results


def host_threads(requested):
    if requested > 0:
        return requested
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, min(n, 32))


# --------------------------------------------------------------------------- roofline
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture) over algorithmic
# bytes, per kernel class, measured on a small case of this workload and scaled to a full launch
# by the units processed (traffic grows in proportion to them); the summary each figure comes
# from is named beside it.
DRAM_TRAFFIC_OVER_ALGORITHMIC = {
    "attention": (0.997, "profiles/k_attention_decode_64seq.md: 19.46 MB measured / 19.53 MB algorithmic, scaled by positions attended"),
}


def algorithmic_bytes(cls, sh, m_rows, mean_width):
    """Bytes one launch of a kernel class must move (weights once, activations in, codes out)."""
    H, I, KV = sh.hidden, sh.inter, sh.kv_hidden
    lin = lambda n, k: n * k + m_rows * k + 12 * n + m_rows * n
    return {
        "linear_qkv": lin(H + 2 * KV, H), "linear_o": lin(H, H), "linear_gate_up": lin(2 * I, H),
        "linear_down": lin(H, I), "head": sh.vocab * H + m_rows * H + 8 * m_rows,
        "attention": m_rows * (2 * KV * mean_width + 2 * H),
    }.get(cls)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# --------------------------------------------------------------------------- main arms
def dist_setup(n_gpus):
    """(rank, world, local_rank, barrier, max_over_ranks, sum_over_ranks)"""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world <= 1:
        return 0, 1, 0, (lambda: None), (lambda v: v), (lambda v: v)
    import torch
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local)
    dist.init_process_group(backend="nccl" if use_cuda else "gloo", rank=rank, world_size=world)
    dev = torch.device("cuda", local) if use_cuda else torch.device("cpu")

    def barrier():
        dist.barrier()

    def reduce(v, op):
        t = torch.tensor([float(v)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=op)
        return float(t.item())

    return (rank, world, local, barrier, lambda v: reduce(v, dist.ReduceOp.MAX),
            lambda v: reduce(v, dist.ReduceOp.SUM))


def partition(n_seqs, world, rank, strong):
    """Sequence ids served by `rank`: weak scaling gives every rank its own n_seqs sequences,
    strong scaling deals one global list round-robin."""
    if strong:
        return [i for i in range(n_seqs) if i % world == rank], 0
    return list(range(n_seqs)), rank + 1


def run_ours(args):
    rank, world, local, barrier, rmax, rsum = dist_setup(args.gpus)
    sh = A.SHAPES[args.shape]
    steps, warmup = args.steps, max(args.warmup, 3)
    cap = ((args.prompt_hi + warmup + steps + 8 + 15) // 16) * 16 + 16 * 14   # room for the roofline passes too
    art = get_artifact(args.shape, cap, rank, barrier)
    from superslm_b200 import build as B
    lib = abi.SslmLib(B.LIB if os.path.exists(B.LIB) else B.build())
    d = bind_extras(lib)
    if d.sslm_b200_set_device(local) != 0:
        raise SystemExit("no usable CUDA device %d: the CUDA path is the only path" % local)

    ids, stream = partition(args.seqs, world, rank, args.strong)
    prompts_all = workload_prompts(args.shape, args.seqs, args.prompt_lo, args.prompt_hi, stream)
    prompts = [prompts_all[i] for i in ids]
    n = len(prompts)
    eng = abi.Engine(lib, art, blocks=n + 1, max_batch=max(n, 1), max_chunk=args.chunk)
    seqs = [eng.new_seq() for _ in range(n)]

    # ---- prefill (timed: wall clock through the ABI and device events)
    barrier()
    launches0 = last_call(d, eng.ws)[1]
    t0 = time.perf_counter()
    dev_ms = 0.0
    ptoks = 0
    for s, p in zip(seqs, prompts):
        done = 0
        while done < p.size:
            consumed = C.c_int32(0)
            st = lib.sslm_prefill(eng.model, s.handle, p[done:].ctypes.data_as(C.POINTER(C.c_int32)), p.size - done,
                                  args.chunk, 0, eng.ws, C.byref(consumed))
            assert st == 0, abi.STATUS_NAMES[st]
            done += consumed.value
            dev_ms += last_call(d, eng.ws)[0]
        ptoks += p.size
    prefill_wall = rmax(time.perf_counter() - t0)
    prefill_dev = rmax(dev_ms / 1e3)
    ptoks_all = rsum(ptoks)

    # ---- decode: first call serves the pending logits, then W warm-up and K timed steps
    st, toks = eng.decode_step(seqs, sh.layers)
    assert st == 0
    for _ in range(warmup):
        st, toks = eng.decode_step(seqs, sh.layers)
        assert st == 0
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    launches1 = last_call(d, eng.ws)[1]
    batch = eng.batch(seqs, sh.layers)     # handle array and output buffer prepared once, as a C caller holds them
    t0 = time.perf_counter()
    dev_ms = 0.0
    produced = 0
    for _ in range(steps):
        st = batch.step()
        assert st == 0, abi.STATUS_NAMES[st]
        dev_ms += last_call(d, eng.ws)[0]
        produced += int((batch.tokens >= 0).sum())
    wall = time.perf_counter() - t0
    launches2 = last_call(d, eng.ws)[1]
    clocks = sampler.stop() if sampler else None
    barrier()
    wall_max, dev_max = rmax(wall), rmax(dev_ms / 1e3)
    produced_all = rsum(produced)

    # ---- per-kernel-class timing of a few more steps (rank 0), for the roofline object
    roof, classes, prefill_classes = None, {}, {}
    if rank == 0:
        d.sslm_b200_profile(eng.ws, 1)
        psteps = 4
        for _ in range(psteps):
            st, toks = eng.decode_step(seqs, sh.layers)
            assert st == 0
        ms = (C.c_double * 16)()
        cnt = (C.c_uint64 * 16)()
        d.sslm_b200_profile_read(eng.ws, ms, cnt, 14)
        d.sslm_b200_profile(eng.ws, 0)
        total = sum(ms[i] for i in range(14)) or 1.0
        mean_width = float(np.mean([p.size for p in prompts])) + warmup + steps + 2
        peak, peak_kind = measured_peaks()
        for i, name in enumerate(PROF_CLASSES):
            if cnt[i] == 0:
                continue
            avg_us = ms[i] * 1e3 / cnt[i]
            ab = algorithmic_bytes(name, sh, n, mean_width)
            classes[name] = {"launches_per_step": cnt[i] / psteps, "avg_us": round(avg_us, 2),
                             "share": round(ms[i] / total, 4)}
            if ab:
                classes[name]["GBps"] = round(ab / (avg_us * 1e-6) / 1e9, 1)
                classes[name]["frac_hbm"] = round(ab / (avg_us * 1e-6) / 1e9 / peak, 4)
        # one more profiled pass: a 1024-token chunk-batched prefill of a fresh sequence
        extra = eng.new_seq()
        pp = A.stream_uniform(SEED ^ 0x77, "prefill_profile", min(1024, args.prompt_hi), 0, sh.vocab - 1).astype(np.int32)
        d.sslm_b200_profile(eng.ws, 1)
        extra.prefill(pp, args.chunk)
        d.sslm_b200_profile_read(eng.ws, ms, cnt, 14)
        d.sslm_b200_profile(eng.ws, 0)
        ptotal = sum(ms[i] for i in range(14)) or 1.0
        prefill_classes = {name: {"ms": round(ms[i], 3), "share": round(ms[i] / ptotal, 4)}
                           for i, name in enumerate(PROF_CLASSES) if cnt[i]}
        prefill_classes["_tokens"] = int(pp.size)
        prefill_classes["_linear_TOPS"] = round(
            2.0 * pp.size * sh.layers * (2 * sh.hidden ** 2 + 2 * sh.hidden * sh.kv_hidden + 3 * sh.hidden * sh.inter)
            / (1e9 * (sum(ms[i] for i in (1, 5, 7, 9)) or 1.0)), 1)
        extra.release()
        top = max((c for c in classes if "GBps" in classes[c]), key=lambda c: classes[c]["share"])
        ab_top = algorithmic_bytes(top, sh, n, mean_width)
        ratio = DRAM_TRAFFIC_OVER_ALGORITHMIC.get(top)
        roof = {"kernel": top, "bound": "hbm", "achieved": classes[top]["GBps"], "peak": peak, "unit": "GB/s",
                "frac": classes[top]["frac_hbm"], "peak_source": "of " + peak_kind,
                "traffic": (round(ab_top * ratio[0]) if ratio else None),
                "traffic_source": (ratio[1] if ratio else None),
                "algorithmic_bytes_per_launch": ab_top,
                "avg_launch_us": classes[top]["avg_us"]}

    # ---- CPU baseline (rank 0, bounded sample) and a parity spot check on its first sequence
    cpu, parity = None, None
    if rank == 0 and not args.no_cpu_baseline:
        threads = host_threads(args.cpu_threads)
        r = cpu_reference_run(art, args.shape, threads, 32, 8, 1)
        eng2 = abi.Engine(lib, art, blocks=1, max_batch=1, max_chunk=32)
        s2 = eng2.new_seq()
        s2.prefill(r["prompt0"], 32)
        got = s2.decode(len(r["tokens0"]), sh.layers)
        parity = "bit-identical tokens vs CPU on the sampled sequence" if got == r["tokens0"] else "MISMATCH"
        eng2.close()
        cpu = {"value": round(r["decode_tok_s"], 3), "unit": "tok/s", "cores": r["cores"], "kind": r["kind"],
               "sample": r["sample"], "prefill_tok_s": round(r["prefill_tok_s"], 2)}
    model_bytes = d.sslm_b200_model_device_bytes(eng.model)
    tcn, tcr, tcw = C.c_uint64(0), C.c_uint64(0), C.c_int32(0)
    d.sslm_b200_tc_stats(C.byref(tcn), C.byref(tcr), C.byref(tcw))
    tc_info = {"launches": tcn.value, "declined": tcr.value, "last_decline_reason": tcw.value}
    eng.close()
    if rank != 0:
        return
    h2d = n * (24 + 16 + 16)     # RowDesc + RowSource + RowSink per row and phase
    out = {
        "metric": "decode tok/s, Qwen2.5-1.5B-shape int8, bit-exact vs CPU ref", "impl": "ours",
        "value": round(produced_all / dev_max, 1), "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(dev_max * 1e3 / steps, 4), "higher_is_better": True,
        "scaling": "strong" if args.strong else "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "config 3: multi-sequence serving, synthetic Qwen2.5-%s shape" % args.shape,
                   "sequences_per_gpu": n, "prompt_len": [args.prompt_lo, args.prompt_hi], "kv_page_tokens": 16,
                   "context_cap": cap, "layer_budget": sh.layers, "prefill_chunk": args.chunk,
                   "l2": "each step streams %.2f GB of weights (> 126 MB L2); no flush needed" % (model_bytes / 1e9),
                   "parallelism": "replicas x%d, no collective" % world},
        "clocks": clocks,
        "e2e": {"value": round(produced_all / wall_max, 1), "unit": "tok/s", "h2d_bytes_per_step": 2 * h2d,
                "d2h_bytes_per_step": 2 * n * 20, "ms_per_step": round(wall_max * 1e3 / steps, 4)},
        "gpu_launches": int(launches2 - launches1),
        "prefill": {"value": round(ptoks_all / prefill_dev, 1), "e2e": round(ptoks_all / prefill_wall, 1),
                    "unit": "tok/s", "tokens": int(ptoks_all), "gpu_launches": int(launches1 - launches0)},
        "tensor_core_kernel": tc_info, "roofline": roof, "kernels": classes, "kernels_prefill_1024": prefill_classes, "cpu_baseline": cpu, "parity": parity,
    }
    print(json.dumps(out))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = args.steps, max(args.warmup, 1)
    pl = 32
    cap = ((args.prompt_hi + 3 + 32 + 8 + 15) // 16) * 16 + 16 * 14
    try:
        art = get_artifact(args.shape, cap, 0, lambda: None)
        threads = host_threads(args.cpu_threads)
        r = cpu_reference_run(art, args.shape, threads, pl, steps, warmup)
    except Exception as e:   # the CPU arm must not take the run down
        print(json.dumps({"impl": "reference", "unavailable": "%s: %s" % (type(e).__name__, e)}))
        return
    cpu = {"value": round(r["decode_tok_s"], 3), "unit": "tok/s", "cores": r["cores"], "kind": r["kind"],
           "sample": r["sample"]}
    print(json.dumps({
        "metric": "decode tok/s, Qwen2.5-1.5B-shape int8, bit-exact vs CPU ref", "impl": "reference",
        "value": cpu["value"], "unit": "tok/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps,
        "warmup": warmup, "ms_per_step": round(r["decode_s"] * 1e3 / steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "config 3 sample on the host CPU: synthetic Qwen2.5-%s shape, one sequence per "
                               "host thread" % args.shape, "sequences": threads, "prompt_len": [pl, pl]},
        "cpu_baseline": cpu,
        "prefill": {"value": round(r["prefill_tok_s"], 2), "unit": "tok/s"},
        "e2e": {"value": cpu["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


if __name__ == "__main__":
    a = parse_args()
    try:
        if a.impl == "reference":
            run_reference(a)
        else:
            run_ours(a)
    finally:
        _dist = sys.modules.get("torch.distributed")      # only if a multi-rank run brought it in
        try:
            if _dist is not None and _dist.is_available() and _dist.is_initialized():
                _dist.destroy_process_group()
        except Exception:
            pass

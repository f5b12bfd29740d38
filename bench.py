#!/usr/bin/env python
"""Benchmark of the integer forward pass behind the sslm_* C ABI.

Workload (the multi-sequence serving case on the 1.5B-shape model): a seeded synthetic
Qwen2.5-1.5B-architecture artifact (28 layers, d_model 1536, 12/2 heads of 128, FFN 8960, vocab
151936, tied head; int8 weights uniform in [-127,127], fold multipliers in [2^30,2^31), shifts
8..20), `--seqs` independent sequences with prompt lengths uniform in [128,1024], chunk-batched
prefill, then greedy decode over 16-token KV pages. One *step* = one sslm_decode_step over all
of a rank's sequences (one token per sequence, all 28 layers). Every decode step streams the full
1.5 GB of weights, far more than the 126 MB L2, so no explicit L2 flush is needed between steps.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

`value` is decode tokens/s from device time (CUDA events inside the library, inputs resident in
HBM); `e2e` is the same through the C ABI from host buffers (descriptor upload and token
read-back included). With N > 1 every GPU holds a model replica and its own sequences; no
collective runs on the data path (NCCL only carries the barrier and the max-over-ranks of the
timings). The same line also carries, measured in the same run on rank 0:

  linear_sweep      the standalone linear layer over the 5 x 5 grid of (K x N) x M shapes
  single_sequence   one sequence at context ~2048, all layers per call (the latency-bound case)
  roofline_step     the whole decode step against its own byte roofline
  strong            (N > 1) the same 256 sequences in total dealt over the N GPUs
  parity            sequences of the workload compared with records of the CPU reference
"""
from __future__ import annotations

import argparse
import ctypes as C
import hashlib
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
METRIC = "decode tok/s, Qwen2.5-1.5B-shape int8, bit-exact vs CPU ref"
PROF_CLASSES = ["begin", "linear_qkv", "qkv_post", "attention", "ctx_funnel", "linear_o", "residual1",
                "linear_gate_up", "activation", "linear_down", "residual2", "head", "lora_u", "other"]
SWEEP_KN = [(1536, 1536), (1536, 256), (1536, 8960), (8960, 1536), (1536, 151936)]
SWEEP_M = [1, 16, 128, 512, 2048]
SINGLE_CONTEXT = 2048
PARITY_GOLDEN = os.path.join(ROOT, "tests", "golden", "bench_parity_golden.json")


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
    ap.add_argument("--parity-seqs", type=int, default=16,
                    help="workload sequences compared with the CPU reference's records (up to 16)")
    ap.add_argument("--no-sweep", action="store_true", help="skip the standalone linear-layer grid")
    ap.add_argument("--no-single", action="store_true", help="skip the single-sequence measurement")
    ap.add_argument("--only-sweep", action="store_true", help="just the standalone linear-layer grid (no model)")
    ap.add_argument("--sweep-cell", default="", help="K,N,M: restrict the grid to one cell (for profiler captures)")
    ap.add_argument("--config-table", action="store_true",
                    help="time the single-sequence configurations (0, 2 and 4 as tests/golden/config_cases.py states them): "
                         "prefill and decode tok/s through the ABI; with --impl reference the CPU library on one host thread")
    return ap.parse_args()


def context_cap(args):
    """One artifact serves every measurement of a run: room for the longest prompt plus the decode
    steps, and for the single-sequence case at context ~2048. (The value does not change any
    arithmetic: it sizes the RoPE table and the KV blocks.)"""
    need = args.prompt_hi + max(args.warmup, 3) + args.steps + 8 + 16 * 14
    return ((max(need, SINGLE_CONTEXT + 96) + 15) // 16) * 16


def workload_config(args, sh, n_per_gpu, world):
    """The `config` object: the same for this implementation's arm and for the CPU reference arm."""
    return {"workload": "multi-sequence serving (configuration 3), synthetic Qwen2.5-%s shape" % args.shape,
            "sequences_per_gpu": n_per_gpu, "prompt_len": [args.prompt_lo, args.prompt_hi], "kv_page_tokens": 16,
            "decode_steps": args.steps, "layer_budget": sh.layers,
            "l2": "each step streams the model's 1.5 GB of weights (> 126 MB L2); no flush needed",
            "parallelism": "replicas x%d, no collective" % world}


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


def parity_sample(prompts, count):
    """Indices of `count` workload sequences: the shortest, the longest, the rest spread evenly."""
    order = sorted(range(len(prompts)), key=lambda i: (prompts[i].size, i))
    picks = [order[0], order[-1]]
    for k in range(1, 15):
        picks.append(order[k * (len(order) - 1) // 15])
    out = []
    for i in picks:
        if i not in out:
            out.append(i)
    return out[:max(0, min(count, len(out)))]


def sequence_digest(blob: bytes, sh) -> dict:
    """What a save blob says about a sequence, independent of the artifact's context cap: header
    fields and the SHA-256 of the K/V rows of the positions the sequence holds."""
    f = abi.parse_save_blob(blob, sh.hidden)
    ctx = f["context_length"]
    kv = np.frombuffer(f["kv"], dtype=np.int8)
    cap = kv.size // (sh.layers * 2 * sh.kv_heads * sh.head_dim)
    kv = kv.reshape(sh.layers, 2, sh.kv_heads, cap, sh.head_dim)[:, :, :, :ctx, :]
    return {"context_length": ctx, "hidden_scale": list(f["hidden_scale"]), "kv_saturation_count": f["kv_saturation_count"],
            "kv_sha256": hashlib.sha256(np.ascontiguousarray(kv).tobytes()).hexdigest()}


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
    d.sslm_b200_linear_bench.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_uint64,
                                         C.POINTER(C.c_double), C.POINTER(C.c_double)]
    return d


def last_call(d, ws):
    ms, n = C.c_float(0), C.c_uint64(0)
    d.sslm_b200_last_call_ms(ws, C.byref(ms), C.byref(n))
    return ms.value, n.value


def profile_classes(d, ws, run, psteps):
    """Per-kernel-class device time of `run()` (called once; it makes `psteps` calls)."""
    d.sslm_b200_profile(ws, 1)
    run()
    ms = (C.c_double * 16)()
    cnt = (C.c_uint64 * 16)()
    d.sslm_b200_profile_read(ws, ms, cnt, 14)
    d.sslm_b200_profile(ws, 0)
    total = sum(ms[i] for i in range(14)) or 1.0
    out = {}
    for i, name in enumerate(PROF_CLASSES):
        if cnt[i]:
            out[name] = {"launches_per_step": cnt[i] / psteps, "avg_us": round(ms[i] * 1e3 / cnt[i], 2),
                         "ms": round(ms[i], 3), "share": round(ms[i] / total, 4)}
    return out


# --------------------------------------------------------------------------- CPU arm
def cpu_reference_run(art, shape, prompts, steps, warmup):
    """The reference's own CPU implementation (oracle/_ref, else the C restatement) on the host
    cores: one sequence per thread (the reference is single-threaded per call and allows one
    sequence per thread on a shared read-only model), prompts given by the caller."""
    from oracle import harness as H
    sh = A.SHAPES[shape]
    threads = len(prompts)
    ref = H.ref()
    kind = "reference" if ref is not None else "port"
    if ref is not None:
        eng = abi.Engine(ref, art, blocks=threads, max_batch=1, max_chunk=max(p.size for p in prompts))
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
    lens = [int(p.size) for p in prompts]
    results = {"kind": kind, "cores": threads, "prefill_tok_s": sum(lens) / t_prefill,
               "decode_tok_s": threads * steps / t_decode, "decode_s": t_decode,
               "sample": "%d sequences of the workload (one per host thread), prompts of %d..%d tokens (mean %d), "
                         "%d timed decode tokens each" % (threads, min(lens), max(lens), sum(lens) // threads, steps)}
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
    "attention": (0.995, "profiles/k_attention_decode_64seq.md: 19.44 MB measured / 19.53 MB algorithmic, scaled by positions attended"),
}


def linear_weight_bytes(sh):
    H, I, KV = sh.hidden, sh.inter, sh.kv_hidden
    return sh.layers * (2 * H * H + 2 * H * KV + 3 * H * I) + sh.vocab * H


def fold_bytes(sh):
    H, I, KV = sh.hidden, sh.inter, sh.kv_hidden
    return 12 * sh.layers * (2 * H + 2 * KV + 2 * I + sh.heads)


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
    """(HBM GB/s, int8 dense TOPS, source note). The int8 figure is 2 x the measured bf16 burst
    throughput: no int8 peak was measured on this pool, so it is an assumption and says so."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            j = json.load(open(p))
            return float(j["hbm_gbs"]), 2.0 * float(j["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 6650.0, 2.0 * 1590.0, "fallback"


def linear_sweep(d, art_sh, only_cell=None):
    """The standalone linear layer (projection + fold + per-row funnel) on operands resident in
    HBM, every (K x N) x M cell: device time per launch from CUDA events over a chain of launches
    that rotates through enough weight copies to defeat the L2. Cells with M <= 16 run the
    streaming kernel and are read against the HBM peak (bytes = K N + M K + 12 N + M N); cells
    with M >= 128 run the tcgen05 kernel and are read against the int8 tensor peak (2 M K N)."""
    hbm, int8_tops, src = measured_peaks()
    cells = []
    shim = None
    try:
        from oracle import harness as H
        shim = H.ref_shim()
        port = H.port()
    except Exception:
        port = None
    rng = np.random.default_rng(7)
    for K, N in SWEEP_KN:
        for M in SWEEP_M:
            if only_cell is not None and (K, N, M) != only_cell:
                continue
            use_tc = 1 if M > 8 else 0
            iters = 200 if M <= 16 else (40 if M <= 512 else 10)
            if N > 100000:
                iters = max(5, iters // 4)
            g, t = C.c_double(0), C.c_double(0)
            st = d.sslm_b200_linear_bench(M, N, K, use_tc, iters, 1234, C.byref(g), C.byref(t))
            cell = {"K": K, "N": N, "M": M, "kernel": "tcgen05" if use_tc else "gemv"}
            if st != 0:
                cell["error"] = abi.STATUS_NAMES[st]
                cells.append(cell)
                continue
            us = g.value
            byts = K * N + M * K + 12 * N + M * N
            cell.update({"us": round(us, 2), "us_with_funnel": round(t.value, 2),
                         "GBps": round(byts / us / 1e3, 1), "TOPS": round(2.0 * M * K * N / us / 1e6, 2)})
            if M <= 16:
                cell["frac"] = round(byts / us / 1e3 / hbm, 4)
                cell["of"] = "hbm"
            else:
                cell["frac"] = round(2.0 * M * K * N / us / 1e6 / int8_tops, 4)
                cell["of"] = "int8"
            # the CPU composition beside it: the reference's GEMM, the fold and the funnel, one
            # host thread, on a bounded sample of the cell's rows
            if port is not None:
                rows = min(M, 4)
                x = rng.integers(-127, 128, (rows, K)).astype(np.int8)
                w = rng.integers(-127, 128, (N, K)).astype(np.int8)
                fold = np.zeros((N, 3), dtype=np.int32)
                fold[:, 1] = 1 << 30
                fold[:, 2] = 10
                acc = np.zeros((rows, N), dtype=np.int64)
                folded = np.empty_like(acc)
                codes = np.zeros(N, dtype=np.int8)
                t0 = time.perf_counter()
                if shim is not None:
                    shim.refshim_gemm(x.ctypes.data, w.ctypes.data, rows, K, N, acc.ctypes.data)
                else:
                    port.osc_gemm(x.ctypes.data, w.ctypes.data, rows, K, N, acc.ctypes.data)
                port.osc_fold_matrix(acc.ctypes.data, rows, N, fold.ctypes.data, folded.ctypes.data)
                from oracle.harness import Scale
                for r in range(rows):
                    sc, inc = Scale(), Scale(1 << 30, -37)
                    port.osc_funnel(folded[r].ctypes.data, N, C.byref(inc), 1, Scale(1090717716, -44), codes.ctypes.data,
                                    C.byref(sc))
                cell["cpu_us_per_row"] = round((time.perf_counter() - t0) * 1e6 / rows, 1)
            cells.append(cell)
    return {"cells": cells, "hbm_peak_GBps": hbm, "int8_peak_TOPS": int8_tops,
            "peaks": "HBM of %s; int8 = 2 x bf16 burst of %s (assumed: no int8 peak was measured)" % (src, src),
            "cpu": "reference GEMM (%s) + fold + funnel, one host thread, <= 4 rows per cell" %
                   ("oracle/_ref" if shim is not None else "C restatement")}


def single_sequence(lib, d, eng, sh, steps):
    """One sequence at context ~2048, all layers per call: the decode path where every projection
    is a one-row weight stream and attention serves a single long row."""
    s = eng.new_seq()
    prompt = A.stream_uniform(SEED ^ 0x51, "single", SINGLE_CONTEXT, 0, sh.vocab - 1).astype(np.int32)
    t0 = time.perf_counter()
    dev_ms = 0.0
    done = 0
    while done < prompt.size:
        consumed = C.c_int32(0)
        st = lib.sslm_prefill(eng.model, s.handle, prompt[done:].ctypes.data_as(C.POINTER(C.c_int32)), prompt.size - done,
                              1024, 0, eng.ws, C.byref(consumed))
        assert st == 0, abi.STATUS_NAMES[st]
        done += consumed.value
        dev_ms += last_call(d, eng.ws)[0]
    prefill_wall = time.perf_counter() - t0
    prefill_dev = dev_ms / 1e3
    batch = eng.batch([s], sh.layers)
    for _ in range(4):
        assert batch.step() == 0
    t0 = time.perf_counter()
    dev_ms = 0.0
    l0 = last_call(d, eng.ws)[1]
    for _ in range(steps):
        assert batch.step() == 0
        dev_ms += last_call(d, eng.ws)[0]
    wall = time.perf_counter() - t0
    launches = last_call(d, eng.ws)[1] - l0
    classes = profile_classes(d, eng.ws, lambda: [batch.step() for _ in range(4)], 4)
    width = SINGLE_CONTEXT + 4 + steps // 2
    byts = linear_weight_bytes(sh) + fold_bytes(sh) + sh.layers * 2 * sh.kv_hidden * width
    hbm, _, src = measured_peaks()
    tok_s = steps / (dev_ms / 1e3)
    for name, c in classes.items():
        ab = algorithmic_bytes(name, sh, 1, width)
        if ab:
            c["GBps"] = round(ab / c["avg_us"] / 1e3, 1)
            c["frac_hbm"] = round(ab / c["avg_us"] / 1e3 / hbm, 4)
    s.release()
    return {"context": width, "decode_tok_s": round(tok_s, 1), "e2e_tok_s": round(steps / wall, 1),
            "ms_per_token": round(dev_ms / steps, 4), "gpu_launches_per_token": launches / steps,
            "bytes_per_token": byts, "GBps": round(byts * tok_s / 1e9, 1), "frac_hbm": round(byts * tok_s / 1e9 / hbm, 4),
            "peak_source": "of " + src, "prefill_tok_s": round(prompt.size / prefill_dev, 1),
            "prefill_e2e_tok_s": round(prompt.size / prefill_wall, 1), "prefill_chunk": 1024, "kernels": classes}


def parity_check(lib, eng, sh, args, prompts, count):
    """`count` of the workload's own sequences (the shortest and the longest among them), prefilled
    and decoded as one batch, against what the CPU reference recorded for the same prompts:
    tokens, K/V of every layer and position, carried scale, saturation counter."""
    if count <= 0 or not os.path.exists(PARITY_GOLDEN):
        return {"checked": 0, "note": "no records" if count > 0 else "off"}
    gold = json.load(open(PARITY_GOLDEN))
    if (gold["shape"], gold["seed"], gold["prompt_lo"], gold["prompt_hi"], gold["sequences"]) != \
       (args.shape, SEED, args.prompt_lo, args.prompt_hi, len(prompts)):
        return {"checked": 0, "note": "records are for another workload"}
    picks = [i for i in parity_sample(prompts, 16) if str(i) in gold["records"]][:count]
    seqs = [eng.new_seq() for _ in picks]
    for s, i in zip(seqs, picks):
        assert s.prefill(prompts[i], args.chunk) == prompts[i].size
    ndec = gold["decode"]
    toks = [[] for _ in picks]
    for _ in range(ndec):
        st, out = eng.decode_step(seqs, sh.layers)
        assert st == 0
        for t, o in zip(toks, out):
            t.append(int(o))
    bad = []
    for s, i, t in zip(seqs, picks, toks):
        want = gold["records"][str(i)]
        got = sequence_digest(s.save(), sh)
        got["tokens"] = t
        for k in ("tokens", "context_length", "hidden_scale", "kv_saturation_count", "kv_sha256"):
            if got[k] != want[k]:
                bad.append((i, k))
        s.release()
    lens = [int(prompts[i].size) for i in picks]
    return {"checked": len(picks), "mismatches": len(bad), "first_mismatch": bad[:1], "prompt_lengths": lens,
            "decode_tokens": ndec,
            "what": "tokens, K/V bytes of all layers and positions, hidden scale and saturation counter "
                    "against records of the CPU reference (tests/golden/bench_parity_golden.json)",
            "verdict": "bit-identical" if not bad else "MISMATCH"}


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


def timed_decode(d, eng, batch, steps):
    """(wall seconds, device seconds, tokens produced) of `steps` calls of batch.step()."""
    t0 = time.perf_counter()
    dev_ms, produced = 0.0, 0
    for _ in range(steps):
        st = batch.step()
        assert st == 0, abi.STATUS_NAMES[st]
        dev_ms += last_call(d, eng.ws)[0]
        produced += int((batch.tokens >= 0).sum())
    return time.perf_counter() - t0, dev_ms / 1e3, produced


def run_ours(args):
    rank, world, local, barrier, rmax, rsum = dist_setup(args.gpus)
    sh = A.SHAPES[args.shape]
    steps, warmup = args.steps, max(args.warmup, 3)
    cap = context_cap(args)
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
    eng = abi.Engine(lib, art, blocks=n + 18, max_batch=max(n, 16), max_chunk=args.chunk)
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
    wall, dev_s, produced = timed_decode(d, eng, batch, steps)
    launches2 = last_call(d, eng.ws)[1]
    clocks = sampler.stop() if sampler else None
    barrier()
    wall_max, dev_max = rmax(wall), rmax(dev_s)
    produced_all = rsum(produced)
    # host<->device bytes of one step inside sslm_decode_step, summed over the ranks: RowDesc + RowSource +
    # RowSink per row and phase up, status + finished layers + saturation + argmax key per row and phase down
    h2d_all = int(rsum(2 * n * (24 + 16 + 16)))
    d2h_all = int(rsum(2 * n * 24))

    # ---- the same sequences in total dealt over the GPUs (strong scaling): every rank keeps 1/world of its own
    strong = None
    if world > 1 and not args.strong:
        mine = seqs[rank::world] if n >= world else seqs[:1]
        sbatch = eng.batch(mine, sh.layers)
        for _ in range(2):
            assert sbatch.step() == 0
        barrier()
        s_wall, s_dev, s_prod = timed_decode(d, eng, sbatch, steps)
        barrier()
        s_dev_max, s_prod_all = rmax(s_dev), rsum(s_prod)
        strong = {"sequences_total": int(rsum(len(mine))), "sequences_per_gpu": len(mine),
                  "value": round(s_prod_all / s_dev_max, 1), "unit": "tok/s", "ms_per_step": round(s_dev_max * 1e3 / steps, 4),
                  "efficiency_vs_1gpu": round((s_prod_all / s_dev_max) / (produced_all / dev_max / world) / world, 4),
                  "note": "efficiency = this rate / (world x the rate one GPU reaches on all the sequences, i.e. the "
                          "per-GPU rate of the weak run above); the limiter is the step's dependent-launch chain at "
                          "few rows per GPU, not a collective"}

    # ---- rank 0: per-kernel-class timing, roofline objects, sweeps, parity, CPU baseline
    roof, classes, prefill_classes, step_roof = None, {}, {}, None
    sweep, single, parity, cpu = None, None, None, None
    if rank == 0:
        hbm, int8_tops, peak_kind = measured_peaks()
        classes = profile_classes(d, eng.ws, lambda: [eng.decode_step(seqs, sh.layers) for _ in range(4)], 4)
        mean_width = float(np.mean([p.size for p in prompts])) + warmup + steps + 2
        for name, c in classes.items():
            ab = algorithmic_bytes(name, sh, n, mean_width)
            if ab:
                c["GBps"] = round(ab / c["avg_us"] / 1e3, 1)
                c["frac_hbm"] = round(ab / c["avg_us"] / 1e3 / hbm, 4)
        # one more profiled pass: a 1024-token chunk-batched prefill of a fresh sequence
        extra = eng.new_seq()
        pp = A.stream_uniform(SEED ^ 0x77, "prefill_profile", min(1024, args.prompt_hi), 0, sh.vocab - 1).astype(np.int32)
        prefill_classes = profile_classes(d, eng.ws, lambda: extra.prefill(pp, args.chunk), 1)
        lin_ms = sum(prefill_classes[c]["ms"] for c in ("linear_qkv", "linear_o", "linear_gate_up", "linear_down")
                     if c in prefill_classes) or 1.0
        lin_ops = 2.0 * pp.size * sh.layers * (2 * sh.hidden ** 2 + 2 * sh.hidden * sh.kv_hidden + 3 * sh.hidden * sh.inter)
        prefill_classes["_tokens"] = int(pp.size)
        prefill_classes["_linear_TOPS"] = round(lin_ops / (1e9 * lin_ms), 1)
        prefill_classes["_linear_frac_int8"] = round(lin_ops / (1e9 * lin_ms) / int8_tops, 4)
        extra.release()
        top = max((c for c in classes if "GBps" in classes[c]), key=lambda c: classes[c]["share"])
        ab_top = algorithmic_bytes(top, sh, n, mean_width)
        ratio = DRAM_TRAFFIC_OVER_ALGORITHMIC.get(top)
        roof = {"kernel": top, "bound": "hbm", "achieved": classes[top]["GBps"], "peak": hbm, "unit": "GB/s",
                "frac": classes[top]["frac_hbm"], "peak_source": "of " + peak_kind,
                "traffic": (round(ab_top * ratio[0]) if ratio else None),
                "traffic_source": (ratio[1] if ratio else None),
                "algorithmic_bytes_per_launch": ab_top,
                "avg_launch_us": classes[top]["avg_us"]}
        step_bytes = linear_weight_bytes(sh) + fold_bytes(sh) + n * sh.layers * 2 * sh.kv_hidden * mean_width
        step_s = dev_s / steps
        step_roof = {"bound": "hbm", "bytes_per_step": int(step_bytes), "ms_per_step": round(step_s * 1e3, 4),
                     "achieved": round(step_bytes / step_s / 1e9, 1), "peak": hbm, "unit": "GB/s",
                     "frac": round(step_bytes / step_s / 1e9 / hbm, 4), "peak_source": "of " + peak_kind,
                     "what": "weights and fold rows once per step + every sequence's K/V once per layer"}
        parity = parity_check(lib, eng, sh, args, prompts_all, args.parity_seqs) if stream == 1 or args.strong else \
            {"checked": 0, "note": "records are for rank 0's sequences"}
        if not args.no_single:
            single = single_sequence(lib, d, eng, sh, 32)
    model_bytes = d.sslm_b200_model_device_bytes(eng.model)
    tcn, tcr, tcw = C.c_uint64(0), C.c_uint64(0), C.c_int32(0)
    d.sslm_b200_tc_stats(C.byref(tcn), C.byref(tcr), C.byref(tcw))
    tc_info = {"launches": tcn.value, "declined": tcr.value, "last_decline_reason": tcw.value}
    eng.close()
    if rank == 0 and not args.no_sweep:
        sweep = linear_sweep(d, sh)
    if rank == 0 and not args.no_cpu_baseline:
        # bounded sample: the shortest sequences of the workload, one per host thread
        threads = host_threads(args.cpu_threads)
        order = sorted(range(len(prompts_all)), key=lambda i: (prompts_all[i].size, i))[:threads]
        r = cpu_reference_run(art, args.shape, [prompts_all[i] for i in order], 6, 1)
        cpu = {"value": round(r["decode_tok_s"], 3), "unit": "tok/s", "cores": r["cores"], "kind": r["kind"],
               "sample": r["sample"] + " (the shortest sequences of the workload, to bound the CPU time)",
               "prefill_tok_s": round(r["prefill_tok_s"], 2)}
    if rank != 0:
        return
    cfg = workload_config(args, sh, n, world)
    out = {
        "metric": METRIC, "impl": "ours",
        "value": round(produced_all / dev_max, 1), "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(dev_max * 1e3 / steps, 4), "higher_is_better": True,
        "scaling": "strong" if args.strong else "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": cfg,
        "details": {"context_cap": cap, "prefill_chunk": args.chunk, "model_device_bytes": int(model_bytes)},
        "clocks": clocks,
        "e2e": {"value": round(produced_all / wall_max, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d_all,
                "d2h_bytes_per_step": d2h_all, "ms_per_step": round(wall_max * 1e3 / steps, 4)},
        "gpu_launches": int(launches2 - launches1),
        "prefill": {"value": round(ptoks_all / prefill_dev, 1), "e2e": round(ptoks_all / prefill_wall, 1),
                    "unit": "tok/s", "tokens": int(ptoks_all), "gpu_launches": int(launches1 - launches0)},
        "tensor_core_kernel": tc_info, "roofline": roof, "roofline_step": step_roof, "kernels": classes,
        "kernels_prefill_1024": prefill_classes, "single_sequence": single, "linear_sweep": sweep, "strong": strong,
        "cpu_baseline": cpu, "parity": parity,
    }
    print(json.dumps(out))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sh = A.SHAPES[args.shape]
    steps, warmup = args.steps, max(args.warmup, 1)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    try:
        art = get_artifact(args.shape, context_cap(args), 0, lambda: None)
        threads = host_threads(args.cpu_threads)
        # the first `threads` sequences of rank 0's workload: the same length distribution
        prompts = workload_prompts(args.shape, args.seqs, args.prompt_lo, args.prompt_hi, 1)[:threads]
        r = cpu_reference_run(art, args.shape, prompts, steps, warmup)
    except Exception as e:   # the CPU arm must not take the run down
        print(json.dumps({"impl": "reference", "unavailable": "%s: %s" % (type(e).__name__, e)}))
        return
    cpu = {"value": round(r["decode_tok_s"], 3), "unit": "tok/s", "cores": r["cores"], "kind": r["kind"],
           "sample": r["sample"]}
    print(json.dumps({
        "metric": METRIC, "impl": "reference",
        "value": cpu["value"], "unit": "tok/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": round(r["decode_s"] * 1e3 / steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": workload_config(args, sh, args.seqs, world),
        "cpu_baseline": cpu,
        "prefill": {"value": round(r["prefill_tok_s"], 2), "unit": "tok/s"},
        "e2e": {"value": cpu["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_config_table(args):
    """Prefill and decode tok/s of the single-sequence configurations, one sequence through the sslm_* verbs,
    wall clock around the prefill calls and around the decode loop (the reference's own methodology,
    tools/t2147_chunk_batched_pins.cpp:133-154). The cases are the parity cases of tests/golden/config_cases.py:
    configuration 0 and 2 at their stated shape and lengths, configuration 4 at the 3B widths with 4 of its 36
    layers and 16 decode tokens. --impl reference runs the compiled reference on ONE host thread."""
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    from config_cases import CASES, build_case_artifacts, case_prompt
    if args.impl == "reference":
        from oracle import harness as H      # (the CPU arm: the one place besides cpu_baseline that runs oracle/)
        lib = H.ref()
        if lib is None:
            print(json.dumps({"config_table": None, "unavailable": "oracle/_ref is not built"}))
            return
        impl = {"impl": "reference", "cores": 1}
    else:
        from superslm_b200 import build as B
        lib = abi.SslmLib(B.LIB if os.path.exists(B.LIB) else B.build())
        d = bind_extras(lib)
        if d.sslm_b200_set_device(int(os.environ.get("LOCAL_RANK", "0"))) != 0:
            raise SystemExit("no usable CUDA device: the CUDA path is the only path")
        impl = {"impl": "ours"}
    rows = {}
    for name in ("config0", "config2", "config4"):
        case = CASES[name]
        sh = A.SHAPES[case["shape"]]
        art, adapters = build_case_artifacts(case)
        prompt = case_prompt(case)
        chunk = case["cpu_chunk"] if args.impl == "reference" else max(c for c, _ in case["gpu_splits"])
        budget = 1 if name == "config4" else sh.layers
        eng = abi.Engine(lib, art, blocks=2, max_batch=1, max_chunk=min(chunk, 2048))
        try:
            warm = eng.new_seq()                            # one discarded warm-up of both phases
            warm.prefill(prompt[:48], 48)
            warm.decode(2, budget)
            s = eng.new_seq()
            if adapters:
                s.set_adapter(eng.map_adapter(adapters[case.get("attach", 0)]))
            t0 = time.perf_counter()
            assert s.prefill(prompt, chunk) == len(prompt)
            t1 = time.perf_counter()
            s.decode(1, budget)                             # the pending logits: no layer runs
            n = case["decode"] - 1
            t2 = time.perf_counter()
            s.decode(n, budget)
            t3 = time.perf_counter()
        finally:
            eng.close()
        rows[name] = {"shape": case["shape"], "prompt_tokens": len(prompt), "prefill_chunk": chunk,
                      "prefill_tok_s": round(len(prompt) / (t1 - t0), 2), "decode_tokens": n, "layer_budget": budget,
                      "decode_tok_s": round(n / (t3 - t2), 2)}
    print(json.dumps({"config_table": rows, **impl}))


def run_only_sweep(args):
    from superslm_b200 import build as B
    lib = abi.SslmLib(B.LIB if os.path.exists(B.LIB) else B.build())
    d = bind_extras(lib)
    cell = tuple(int(v) for v in args.sweep_cell.split(",")) if args.sweep_cell else None
    print(json.dumps({"linear_sweep": linear_sweep(d, A.SHAPES[args.shape], cell)}))


if __name__ == "__main__":
    a = parse_args()
    try:
        if a.config_table:
            run_config_table(a)
        elif a.only_sweep:
            run_only_sweep(a)
        elif a.impl == "reference":
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

"""The benchmark configurations as parity cases: shared by the script that records the reference's
results (make_config_golden.py) and by the GPU tests that are held to those records.

Every case is a seeded synthetic artifact (shape, seed, context_cap), a seeded prompt, a number of
greedy decode tokens, and optionally adapters: `attach` = index of the adapter attached before
prefill, `swap_after` / `swap_to` = after that many decoded tokens (a token boundary) the adapter
is detached and adapter `swap_to` attached. `cpu_chunk` is the prefill chunk the reference ran
with; `gpu_splits` are the (prefill chunk, layer budget) pairs the GPU is run at, all of which
must reproduce the one reference record. `logit_rows` full int32 logit rows (of decoded tokens 1,
2, ...) are pinned by SHA-256.
"""
from superslm_b200 import artifact as A

SEED = 0x53534C4D00000000

CASES = {
    # configuration 0 in full: 0.5B shape, 24 layers, 512-token prompt, 128 decode steps
    "config0": dict(shape="0.5b", seed=SEED | 0x100, context_cap=768, prompt_len=512, decode=128, cpu_chunk=512,
                    logit_rows=2, gpu_splits=[(512, 24), (77, 5)]),
    # long rows at the three widths: 640, 2304 - 16 and 4608 - 16 positions, then decode
    "long_0p5b": dict(shape="mini0.5b", seed=SEED | 0x101, context_cap=672, prompt_len=640, decode=10, cpu_chunk=640,
                      logit_rows=2, gpu_splits=[(640, 2), (96, 1)]),
    "long_1p5b": dict(shape="mini1.5b", seed=SEED | 0x102, context_cap=2304, prompt_len=2288, decode=10, cpu_chunk=2288,
                      logit_rows=2, gpu_splits=[(2288, 2), (256, 1)]),
    "long_3b": dict(shape="mini3b", seed=SEED | 0x103, context_cap=4608, prompt_len=4592, decode=10, cpu_chunk=4592,
                    logit_rows=2, gpu_splits=[(4592, 2), (1000, 1)]),
    # the widest rows the library admits: context_cap 32768 (16 slices of 2048 positions per kv head) on the
    # smallest shape, and a row beyond 8192 positions (16 slices, funnel not fused) at the 1.5B widths
    "max_context_tiny": dict(shape="tiny", seed=SEED | 0x106, context_cap=32768, prompt_len=32768 - 24, decode=10,
                             cpu_chunk=2048, logit_rows=2, gpu_splits=[(2048, 2), (777, 1)]),
    "long_1p5b_9k": dict(shape="mini1.5b", seed=SEED | 0x107, context_cap=9216, prompt_len=9216 - 16, decode=8,
                         cpu_chunk=2048, logit_rows=2, gpu_splits=[(2048, 2), (1500, 1)]),
    # configuration 2 on the full 1.5B model: 2048-token prompt, chunked prefill, sliced decode
    "config2": dict(shape="1.5b", seed=SEED | 0x104, context_cap=2304, prompt_len=2048, decode=24, cpu_chunk=256,
                    logit_rows=2, gpu_splits=[(256, 28), (2048, 7), (64, 1)]),
    # configuration 4 at the 3B widths (4 of the 36 layers): rank-16 adapters on q/k/v/o, 4096-token
    # prompt with adapter 0 attached, one layer per call, detach + attach adapter 1 mid-run
    "config4": dict(shape="3b4l", seed=SEED | 0x105, context_cap=4608, prompt_len=4096, decode=16, cpu_chunk=512,
                    adapter_seeds=[41, 42], attach=0, swap_after=8, swap_to=1, logit_rows=2,
                    gpu_splits=[(512, 1), (4096, 4)]),
    # the same artifact without any adapter; the GPU must give this record both with no adapter and
    # with an adapter that adapts no projection
    "config4_base": dict(shape="3b4l", seed=SEED | 0x105, context_cap=4608, prompt_len=300, decode=8, cpu_chunk=300,
                         logit_rows=0, gpu_splits=[(300, 1)]),
}


def build_case_artifacts(case):
    """(base artifact bytes, [adapter artifact bytes...])"""
    art = A.build_synthetic_model(case["shape"], case["seed"], case["context_cap"])
    adapters = [A.build_synthetic_adapter(art, s) for s in case.get("adapter_seeds", [])]
    return art, adapters


def case_prompt(case):
    sh = A.SHAPES[case["shape"]]
    return A.stream_uniform(case["seed"] ^ 0xABCDEF, "prompt", case["prompt_len"], 0, sh.vocab - 1)

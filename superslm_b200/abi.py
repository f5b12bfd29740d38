"""ctypes binding of the `sslm_*` C ABI.

The same binding drives two libraries that export identical verbs:

* ``libsslm_b200.so`` -- this package's CUDA implementation (the product), and
* the reference's own CPU library (test infrastructure, loaded only by tests and
  by the CPU-baseline leg of the benchmark).

Verb names, argument order and status ordinals are the reference's
(include/superslm/sslm_abi.h:96-163, sslm_abi_functions.inc,
sslm_abi_functions_g5_comparable.inc). The higher-level `Engine` / `Sequence`
helpers below mirror how the reference's own ABI callers drive it
(tools/t2147_chunk_batched_pins.cpp:133-154): map, pool, workspace, sequence,
chunked prefill, per-call decode.
"""
from __future__ import annotations

import ctypes as C
import os
import struct

import numpy as np

SSLM_OK = 0
STATUS_NAMES = [
    "SSLM_OK", "SSLM_INVALID_ARGUMENT", "SSLM_BUFFER_TOO_SMALL", "SSLM_MISALIGNED_BUFFER",
    "SSLM_ARTIFACT_REJECTED", "SSLM_ADAPTER_MODEL_MISMATCH", "SSLM_RESTORE_MODEL_MISMATCH",
    "SSLM_RESTORE_KV_MISMATCH", "SSLM_MODEL_HAS_LIVE_SEQUENCES", "SSLM_POOL_HAS_LIVE_HANDLES",
    "SSLM_ADAPTER_HAS_LIVE_SEQUENCES", "SSLM_ADAPTER_SWAP_MIDTOKEN_REJECTED",
    "SSLM_SEQ_RESET_MIDTOKEN_REJECTED", "SSLM_PREFIX_FROZEN_REJECTED", "SSLM_KV_POOL_EXHAUSTED",
    "SSLM_TOKEN_ID_OUT_OF_RANGE", "SSLM_CONTEXT_CAP_EXCEEDED", "SSLM_TOKEN_ID_UNMAPPED",
    "SSLM_SCHEMA_NOT_FOUND", "SSLM_SCHEMA_BIND_REJECTED", "SSLM_SCHEMA_SPAN_UNBOUND",
    "SSLM_PREFIX_SCHEMA_MISMATCH", "SSLM_RESTORE_SCHEMA_MISMATCH", "SSLM_SCHEMA_SPAN_UNREACHABLE",
    "SSLM_SCHEMA_UNSATISFIABLE", "SSLM_ALLOCATION_FAILED", "SSLM_NUMERIC_STEP_REFUSED",
]
ST = {n: i for i, n in enumerate(STATUS_NAMES)}


class SslmConfig(C.Structure):
    _fields_ = [("max_batch", C.c_int32), ("max_chunk_budget", C.c_int32),
                ("max_layer_budget", C.c_int32), ("reserved", C.c_uint32)]


class SslmDecodeParams(C.Structure):
    _fields_ = [("layer_budget", C.c_int32), ("struct_size", C.c_uint32), ("mode", C.c_int32),
                ("alpha_q15", C.c_int32), ("anti_lm_max_order", C.c_int32), ("top_k", C.c_int32),
                ("q_ln2", C.c_int64), ("q_b", C.c_int64), ("q_c", C.c_int64)]


_H = C.c_void_p  # opaque handle


def _aligned_buffer(nbytes: int, align: int = 64):
    raw = (C.c_uint8 * (nbytes + align))()
    addr = C.addressof(raw)
    off = (-addr) % align
    return raw, C.c_void_p(addr + off)


class SslmLib:
    """One loaded library exporting the sslm_* verbs."""

    VERBS = {
        "sslm_model_map": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(_H)]),
        "sslm_model_unmap": (C.c_int, [_H]),
        "sslm_kv_block_size": (C.c_size_t, [_H]),
        "sslm_kv_pool_overhead_size": (C.c_size_t, [_H, C.c_uint32]),
        "sslm_kv_pool_create": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_uint32, C.POINTER(_H)]),
        "sslm_kv_pool_destroy": (C.c_int, [_H]),
        "sslm_workspace_size": (C.c_size_t, [_H, C.POINTER(SslmConfig)]),
        "sslm_workspace_create": (C.c_int, [_H, C.POINTER(SslmConfig), C.c_void_p, C.c_size_t, C.POINTER(_H)]),
        "sslm_workspace_destroy": (C.c_int, [_H]),
        "sslm_seq_create": (C.c_int, [_H, C.POINTER(_H), C.POINTER(_H)]),
        "sslm_seq_release": (C.c_int, [_H]),
        "sslm_prefill": (C.c_int, [_H, _H, C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.c_int, _H,
                                   C.POINTER(C.c_int32)]),
        "sslm_decode_step": (C.c_int, [_H, C.POINTER(_H), C.c_int32, C.POINTER(SslmDecodeParams), _H,
                                       C.POINTER(C.c_int32)]),
        "sslm_adapter_map": (C.c_int, [C.c_void_p, C.c_size_t, _H, C.POINTER(_H)]),
        "sslm_adapter_release": (C.c_int, [_H]),
        "sslm_adapter_residency": (C.c_size_t, [_H]),
        "sslm_seq_set_adapter": (C.c_int, [_H, _H]),
        "sslm_seq_save": (C.c_int, [_H, C.c_void_p, C.POINTER(C.c_size_t)]),
        "sslm_seq_restore": (C.c_int, [_H, C.POINTER(_H), C.c_void_p, C.c_size_t, C.POINTER(_H)]),
        "sslm_seq_reset": (C.c_int, [_H]),
        "sslm_prefix_begin": (C.c_int, [_H, C.POINTER(_H), C.POINTER(_H)]),
        "sslm_prefix_prefill": (C.c_int, [_H, _H, C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.c_int, _H,
                                          C.POINTER(C.c_int32)]),
        "sslm_prefix_freeze": (C.c_int, [_H]),
        "sslm_prefix_release": (C.c_int, [_H]),
        "sslm_seq_adopt_prefix": (C.c_int, [_H, _H]),
        "sslm_schema_lookup": (C.c_int, [_H, C.c_char_p, C.POINTER(_H)]),
        "sslm_schema_count": (C.c_size_t, [_H]),
        "sslm_schema_name": (C.c_int, [_H, C.c_int32, C.c_char_p, C.POINTER(C.c_size_t)]),
        "sslm_seq_set_schema": (C.c_int, [_H, _H]),
        "sslm_prefix_set_schema": (C.c_int, [_H, _H]),
    }

    def __init__(self, path: str):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.path = path
        self.dll = C.CDLL(path, mode=os.RTLD_LOCAL | os.RTLD_NOW)
        for name, (res, args) in self.VERBS.items():
            fn = getattr(self.dll, name)
            fn.restype = res
            fn.argtypes = args
            setattr(self, name, fn)


class SslmError(RuntimeError):
    def __init__(self, verb, status):
        self.status = status
        nm = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__("%s -> %s" % (verb, nm))


def _chk(verb, st):
    if st != SSLM_OK:
        raise SslmError(verb, st)


class DecodeBatch:
    """See Engine.batch."""

    def __init__(self, eng: "Engine", seqs, layer_budget: int):
        self.eng = eng
        self.n = len(seqs)
        self.arr = (_H * self.n)(*[s.handle for s in seqs])
        self.params = SslmDecodeParams(layer_budget=layer_budget)
        self.out = (C.c_int32 * self.n)()
        self.tokens = np.ctypeslib.as_array(self.out)
        self._call = eng.lib.sslm_decode_step
        self._params_ref = C.byref(self.params)

    def step(self) -> int:
        return self._call(self.eng.model, self.arr, self.n, self._params_ref, self.eng.ws, self.out)


class Engine:
    """model + kv pool + workspace over one library."""

    def __init__(self, lib: SslmLib, artifact: bytes, blocks: int = 1, max_batch: int = 1,
                 max_chunk: int = 64):
        self.lib = lib
        self._art = np.frombuffer(artifact, dtype=np.uint8)
        self.model = _H()
        _chk("sslm_model_map", lib.sslm_model_map(self._art.ctypes.data, self._art.size, C.byref(self.model)))
        self.block_size = lib.sslm_kv_block_size(self.model)
        need = self.block_size * blocks + lib.sslm_kv_pool_overhead_size(self.model, blocks)
        self._pool_raw, pool_ptr = _aligned_buffer(need)
        self.pool = _H()
        _chk("sslm_kv_pool_create",
             lib.sslm_kv_pool_create(self.model, pool_ptr, need, blocks, C.byref(self.pool)))
        layers = struct.unpack_from("<I", artifact, _config_offset(artifact) + 12)[0]
        self.num_layers = layers
        self.cfg = SslmConfig(max_batch, max_chunk, layers, 0)
        wsz = lib.sslm_workspace_size(self.model, C.byref(self.cfg))
        self._ws_raw, ws_ptr = _aligned_buffer(wsz)
        self.ws = _H()
        _chk("sslm_workspace_create",
             lib.sslm_workspace_create(self.model, C.byref(self.cfg), ws_ptr, wsz, C.byref(self.ws)))
        self.adapters = []
        self.seqs = []

    def new_seq(self) -> "Sequence":
        s = Sequence(self)
        self.seqs.append(s)
        return s

    def map_adapter(self, artifact: bytes):
        a = np.frombuffer(artifact, dtype=np.uint8)
        h = _H()
        _chk("sslm_adapter_map", self.lib.sslm_adapter_map(a.ctypes.data, a.size, self.model, C.byref(h)))
        self.adapters.append((h, a))
        return h

    def decode_step(self, seqs, layer_budget: int):
        """One sslm_decode_step over a batch; returns (status, tokens)."""
        n = len(seqs)
        arr = (_H * n)(*[s.handle for s in seqs])
        params = SslmDecodeParams(layer_budget=layer_budget)
        out = (C.c_int32 * n)()
        st = self.lib.sslm_decode_step(self.model, arr, n, C.byref(params), self.ws, out)
        return st, list(out)

    def batch(self, seqs, layer_budget: int):
        """A fixed batch prepared once, the way a C caller holds its handle array: step() is then
        just the sslm_decode_step call, and `tokens` is a numpy view of the output buffer."""
        return DecodeBatch(self, seqs, layer_budget)

    def close(self):
        for s in list(self.seqs):
            s.release()
        for h, _ in self.adapters:
            self.lib.sslm_adapter_release(h)
        self.adapters = []
        if self.ws:
            self.lib.sslm_workspace_destroy(self.ws)
            self.ws = None
        if self.pool:
            self.lib.sslm_kv_pool_destroy(self.pool)
            self.pool = None
        if self.model:
            self.lib.sslm_model_unmap(self.model)
            self.model = None


def _config_offset(artifact: bytes) -> int:
    nsec = struct.unpack_from("<I", artifact, 12)[0]
    for i in range(nsec):
        stype, _dt, off = struct.unpack_from("<IIQ", artifact, 64 + 40 * i)
        if stype == 0:
            return off
    raise ValueError("no Config section")


class Sequence:
    def __init__(self, eng: Engine):
        self.eng = eng
        self.handle = _H()
        _chk("sslm_seq_create", eng.lib.sslm_seq_create(eng.model, C.byref(eng.pool), C.byref(self.handle)))

    def prefill(self, tokens, chunk_budget: int) -> int:
        """Feed all tokens in calls of at most chunk_budget; returns tokens consumed."""
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        done = 0
        while done < toks.size:
            consumed = C.c_int32(0)
            ptr = toks[done:].ctypes.data_as(C.POINTER(C.c_int32))
            st = self.eng.lib.sslm_prefill(self.eng.model, self.handle, ptr, toks.size - done,
                                           chunk_budget, 0, self.eng.ws, C.byref(consumed))
            done += consumed.value
            _chk("sslm_prefill", st)
            if consumed.value == 0:
                break
        return done

    def decode(self, n_tokens: int, layer_budget: int):
        """Greedy decode n_tokens tokens, calling sslm_decode_step until each lands."""
        out = []
        while len(out) < n_tokens:
            st, toks = self.eng.decode_step([self], layer_budget)
            _chk("sslm_decode_step", st)
            if toks[0] >= 0:
                out.append(toks[0])
        return out

    def set_adapter(self, adapter_handle):
        _chk("sslm_seq_set_adapter", self.eng.lib.sslm_seq_set_adapter(self.handle, adapter_handle))

    def save(self) -> bytes:
        n = C.c_size_t(0)
        self.eng.lib.sslm_seq_save(self.handle, None, C.byref(n))
        buf = (C.c_uint8 * n.value)()
        _chk("sslm_seq_save", self.eng.lib.sslm_seq_save(self.handle, buf, C.byref(n)))
        return bytes(buf[:n.value])

    def reset(self):
        _chk("sslm_seq_reset", self.eng.lib.sslm_seq_reset(self.handle))

    @classmethod
    def restore(cls, eng: "Engine", blob: bytes) -> "Sequence":
        """A new sequence of `eng` from a save blob (either library's)."""
        s = cls.__new__(cls)
        s.eng = eng
        s.handle = _H()
        raw = np.frombuffer(blob, dtype=np.uint8)
        _chk("sslm_seq_restore", eng.lib.sslm_seq_restore(eng.model, C.byref(eng.pool), raw.ctypes.data, raw.size,
                                                          C.byref(s.handle)))
        eng.seqs.append(s)
        return s

    def release(self):
        if self.handle:
            self.eng.lib.sslm_seq_release(self.handle)
            self.handle = None
            if self in self.eng.seqs:
                self.eng.seqs.remove(self)


def parse_save_blob(blob: bytes, hidden_size: int) -> dict:
    """Fields of an SSB3 sequence blob (src/sslm_abi.cpp:2620-2716)."""
    assert blob[0:4] == b"SSB3"
    ctx_len, layer_index, cur_tok, hm, he, sat = struct.unpack_from("<qIiqqQ", blob, 60)
    off = 120
    residual = b""
    if layer_index != 0:
        residual = blob[off:off + hidden_size]
        off += hidden_size
    hist = struct.unpack_from("<Q", blob, 112)[0]
    off += 4 * hist
    nblk = struct.unpack_from("<I", blob, off)[0]
    off += 4
    return {"context_length": ctx_len, "layer_index": layer_index, "current_token": cur_tok,
            "hidden_scale": (hm, he), "kv_saturation_count": sat, "residual": residual,
            "kv_block_count": nblk, "kv": blob[off:]}

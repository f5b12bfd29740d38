"""Python doors onto the two CPU checkers -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

* ``port()``  -> ctypes handle of oracle/liboracle.so (this repository's plain-C
  restatement, sslm_oracle.c), plus `PortModel` / `PortSeq`, which marshal a parsed
  `.sslm` artifact into the restatement's flat structs.
* ``ref()``   -> `superslm_b200.abi.SslmLib` over oracle/_ref/libsslm_ref.so (the
  reference library compiled from its own sources) or None when it was never
  built; ``ref_shim()`` gives the raw ctypes handle for the refshim_* doors.

Only tests/, the smoke check and bench.py's CPU-baseline leg import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

from superslm_b200 import artifact as A

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libsslm_ref.so")
ABI_PROBE = os.path.join(HERE, "_ref", "abi_probe")
# Where the reference's sources are mounted, if anywhere: SSLM_REF_ROOT, else a directory named
# "reference" beside this repository's checkout.
_SIBLING = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
REF_ROOT = os.environ.get("SSLM_REF_ROOT") or (_SIBLING if os.path.isdir(os.path.join(_SIBLING, "src")) else "")


def build(verbose: bool = False) -> None:
    """Compile the restatement, and the reference library when its sources exist."""
    targets = ["oracle"]
    if REF_ROOT and os.path.isdir(os.path.join(REF_ROOT, "src")):
        targets.append("ref")
        if os.path.exists(os.path.join(os.path.dirname(HERE), "superslm_b200", "libsslm_b200.so")):
            targets.append("probe")     # the reference-header caller linked against the CUDA library
    out = subprocess.run(["make", "-C", HERE, "-j8", "REF_ROOT=" + REF_ROOT] + targets,
                         capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if verbose:
        print(out.stdout)


class Scale(C.Structure):
    _fields_ = [("m", C.c_int64), ("e", C.c_int64)]


class LoraProj(C.Structure):
    _fields_ = [("a_w", C.c_void_p), ("b_w", C.c_void_p), ("u_fold", C.c_void_p), ("d_fold", C.c_void_p)]


class LoraLayer(C.Structure):
    _fields_ = [("rank", C.c_uint32)] + [(n, LoraProj) for n in ("q", "k", "v", "o", "gate", "up", "down")]


class Layer(C.Structure):
    _fields_ = ([(n, C.c_void_p) for n in
                 ("q_w", "k_w", "v_w", "o_w", "gate_w", "up_w", "down_w", "attn_gain", "mlp_gain",
                  "q_fold", "k_fold", "v_fold", "o_fold", "gate_fold", "up_fold", "down_fold",
                  "ctx_fold", "k_recip", "v_recip", "softmax_khead", "q_bias", "k_bias", "v_bias")] +
                [(n, Scale) for n in
                 ("c_attn_norm", "c_q", "c_o", "c_ctx", "c_attn_res", "c_mlp_norm", "c_gate", "c_up",
                  "c_act", "c_down", "c_mlp_res")])


class Model(C.Structure):
    _fields_ = ([(n, C.c_uint32) for n in
                 ("hidden", "layers", "heads", "kv_heads", "head_dim", "inter", "vocab", "context_cap")] +
                [("embed", C.c_void_p), ("head", C.c_void_p), ("final_gain", C.c_void_p),
                 ("c_embed", Scale), ("c_final_norm", Scale),
                 ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p), ("silu_table", C.c_void_p),
                 ("layer", C.POINTER(Layer))])


class Seq(C.Structure):
    _fields_ = [("hidden_codes", C.c_void_p), ("hidden_scale", Scale), ("layer_index", C.c_uint32),
                ("context_length", C.c_int64), ("kv_saturation_count", C.c_uint64), ("kv", C.c_void_p)]


_port = None


def port():
    global _port
    if _port is None:
        if not os.path.exists(PORT_SO):
            build()
        lib = C.CDLL(PORT_SO)
        i64, i32, p = C.c_int64, C.c_int32, C.c_void_p
        sig = {
            "osc_srdhm": (i32, [i32, i32]), "osc_rdivpot32": (i32, [i32, C.c_int]),
            "osc_rdivpot64": (i64, [i64, C.c_int]), "osc_mbqm": (i32, [i32, i32, C.c_int]),
            "osc_sat_lshift32": (i32, [i32, C.c_int]),
            "osc_normalize_scale": (None, [i64, C.POINTER(i64), C.POINTER(C.c_int)]),
            "osc_dyn_recip": (i64, [i64]), "osc_requant_code_wide": (C.c_int8, [i64, i64, C.c_int]),
            "osc_isqrt": (i64, [i64]), "osc_floor_div": (i64, [i64, i64]),
            "osc_rope_pair": (None, [i32, i32, i32, i32, C.POINTER(i64), C.POINTER(i64)]),
            "osc_fold": (i64, [i64, i32, i32, i32]), "osc_amp_fold": (i64, [i64, i32, i32, i32]),
            "osc_fold_matrix": (None, [p, C.c_size_t, C.c_size_t, p, p]),
            "osc_sweep": (None, [C.c_int, p, p, p, p, i64, p, p, p]),
            "osc_trace_begin": (None, [p, C.c_size_t]), "osc_trace_end": (C.c_size_t, []),
            "osc_combine": (Scale, [Scale, Scale]),
            "osc_landing_rescale": (i64, [i64, i64, i64, i64, i64, C.POINTER(C.c_uint64), C.POINTER(C.c_int)]),
            "osc_silu_sigmoid_q15": (i32, [p, C.c_int8, i64, C.c_int]),
            "osc_iexp_scale_constants": (C.c_int, [i64, i64, C.POINTER(i64), C.POINTER(i64), C.POINTER(i64)]),
            "osc_iexp": (C.c_int, [i64, i64, i64, i64, C.POINTER(i64), C.POINTER(i64), C.POINTER(i64)]),
            "osc_softmax_width_domain": (C.c_int, [i64, i64, C.c_size_t]),
            "osc_softmax_row_q15": (C.c_int, [p, C.c_size_t, i64, i64, i64, p]),
            "osc_gemm": (None, [p, p, C.c_size_t, C.c_size_t, C.c_size_t, p]),
            "osc_funnel": (C.c_int, [p, C.c_size_t, p, C.c_size_t, Scale, p, C.POINTER(Scale)]),
            "osc_rmsnorm_site": (C.c_int, [p, p, C.c_size_t, Scale, p, C.POINTER(Scale)]),
            "osc_mlp_act_site": (C.c_int, [p, Scale, p, Scale, C.c_size_t, p, Scale, p, C.POINTER(Scale)]),
            "osc_residual_site": (C.c_int, [p, Scale, p, Scale, C.c_size_t, Scale, p, C.POINTER(Scale)]),
            "osc_embed_entry": (C.c_int, [i32, i32, p, C.c_size_t, Scale, p, C.POINTER(Scale)]),
            "osc_layer_loop": (C.c_int, [C.POINTER(Model), C.POINTER(LoraLayer), C.POINTER(Seq), C.c_uint32]),
            "osc_prefill": (C.c_int, [C.POINTER(Model), C.POINTER(LoraLayer), C.POINTER(Seq), p, i32]),
            "osc_logits_argmax": (C.c_int, [C.POINTER(Model), C.POINTER(Seq), p, C.POINTER(i32)]),
            "osc_embed_into_seq": (C.c_int, [C.POINTER(Model), C.POINTER(Seq), i32]),
        }
        for name, (res, args) in sig.items():
            f = getattr(lib, name)
            f.restype, f.argtypes = res, args
        _port = lib
    return _port


_ref = None
_ref_shim = None


def ref():
    """SslmLib over the compiled reference, or None if it is not available."""
    global _ref
    if _ref is None and os.path.exists(REF_SO):
        from superslm_b200.abi import SslmLib
        _ref = SslmLib(REF_SO)
    return _ref


def ref_shim():
    global _ref_shim
    if _ref_shim is None and ref() is not None:
        lib = ref().dll
        i64, i32, p = C.c_int64, C.c_int32, C.c_void_p
        P64, PI = C.POINTER(i64), C.POINTER(C.c_int)
        sig = {
            "refshim_srdhm": (i32, [i32, i32]), "refshim_rdivpot32": (i32, [i32, C.c_int]),
            "refshim_rdivpot64": (i64, [i64, C.c_int]), "refshim_mbqm": (i32, [i32, i32, C.c_int]),
            "refshim_sat_lshift32": (i32, [i32, C.c_int]),
            "refshim_normalize_scale": (None, [i64, P64, PI]), "refshim_dyn_recip": (i64, [i64]),
            "refshim_requant_code_wide": (C.c_int8, [i64, i64, C.c_int]),
            "refshim_isqrt": (i64, [i64]), "refshim_floor_div": (i64, [i64, i64]),
            "refshim_rope_pair": (None, [i32, i32, i32, i32, P64, P64]),
            "refshim_fold": (i64, [i64, i32, i32, i32]), "refshim_amp_fold": (i64, [i64, i32, i32, i32]),
            "refshim_combine": (None, [i64, i64, i64, i64, P64, P64]),
            "refshim_landing_rescale": (i64, [i64, i64, i64, i64, i64, C.POINTER(C.c_uint64), PI]),
            "refshim_silu_sigmoid_q15": (i32, [p, C.c_int8, i64, C.c_int]),
            "refshim_silu_canonical_table": (C.POINTER(i32), []),
            "refshim_iexp_scale_constants": (C.c_int, [i64, i64, P64, P64, P64]),
            "refshim_iexp_coefficients": (None, [P64, P64, P64]),
            "refshim_softmax_width_domain": (C.c_int, [i64, i64, C.c_size_t]),
            "refshim_softmax_row_q15": (C.c_int, [p, C.c_size_t, i64, i64, i64, p]),
            "refshim_gemm": (None, [p, p, C.c_size_t, C.c_size_t, C.c_size_t, p]),
            "refshim_prob_v": (None, [p, p, C.c_size_t, C.c_size_t, p]),
            "refshim_funnel": (C.c_int, [p, C.c_size_t, p, C.c_size_t, i64, i64, p, P64, P64]),
            "refshim_rmsnorm_site": (C.c_int, [p, p, C.c_size_t, i64, i64, p, P64, P64]),
            "refshim_mlp_act_site": (C.c_int, [p, i64, i64, p, i64, i64, C.c_size_t, p, i64, i64, p, P64, P64]),
            "refshim_residual_site": (C.c_int, [p, i64, i64, p, i64, i64, C.c_size_t, i64, i64, p, P64, P64]),
            "refshim_narrow_row": (C.c_int, [p, C.c_size_t, p]),
            "refshim_argmax": (i32, [p, C.c_size_t]),
        }
        for name, (res, args) in sig.items():
            f = getattr(lib, name)
            f.restype, f.argtypes = res, args
        _ref_shim = lib
    return _ref_shim


def _ptr(a: np.ndarray):
    return a.ctypes.data


class PortModel:
    """A parsed artifact marshalled into the restatement's osc_model."""

    def __init__(self, artifact: bytes):
        v = A.parse_artifact(artifact)
        self.view = v
        cfg = v.config
        self.cfg = cfg
        self._keep = []
        w = v.tensors(A.SEC_WEIGHTS, np.int8)
        wsc = v.tensors(A.SEC_WEIGHT_SCALES, np.int32)
        rope = v.tensors(A.SEC_ROPE, np.int64)
        cc = v.constants(A.SEC_COMPOSITION)
        rec = v.constants(A.SEC_KV_RECIP)
        bia = v.tensors(A.SEC_BIASES, np.int64) if A.SEC_BIASES in v.sections else {}
        silu = np.frombuffer(v.sections[A.SEC_SIGMOID_LUT], dtype=np.int32, offset=16).copy()
        L = cfg["num_hidden_layers"]
        KVH = cfg["num_key_value_heads"]
        self.layers = (Layer * L)()

        def keep(a):
            a = np.ascontiguousarray(a)
            self._keep.append(a)
            return _ptr(a)

        for l in range(L):
            p = "layer%d" % l
            ly = self.layers[l]
            for proj in ("q", "k", "v", "o", "gate", "up", "down"):
                setattr(ly, proj + "_w", keep(w["%s.%s_proj" % (p, proj)]))
                setattr(ly, proj + "_fold", keep(wsc["%s.%s_proj" % (p, proj)]))
            ly.attn_gain = keep(w[p + ".attn_norm.gain"])
            ly.mlp_gain = keep(w[p + ".mlp_norm.gain"])
            ly.ctx_fold = keep(wsc[p + ".ctx_fold"])
            ly.k_recip = keep(np.array([rec["%s.k_head%d" % (p, h)] for h in range(KVH)], dtype=np.int64))
            ly.v_recip = keep(np.array([rec["%s.v_head%d" % (p, h)] for h in range(KVH)], dtype=np.int64))
            ly.softmax_khead = keep(np.array([cc["%s.softmax_khead%d" % (p, h)] for h in range(KVH)],
                                             dtype=np.int64))
            for proj in ("q", "k", "v"):      # BIA1: optional, per projection
                bt = bia.get("%s.%s_proj" % (p, proj))
                setattr(ly, proj + "_bias", keep(np.ascontiguousarray(bt, dtype=np.int64)) if bt is not None else None)
            for field, key in (("c_attn_norm", "attn_norm"), ("c_q", "q_proj"), ("c_o", "o_proj"),
                               ("c_ctx", "attn_ctx"), ("c_attn_res", "attn_residual"),
                               ("c_mlp_norm", "mlp_norm"), ("c_gate", "gate_proj"), ("c_up", "up_proj"),
                               ("c_act", "mlp_act"), ("c_down", "down_proj"), ("c_mlp_res", "mlp_residual")):
                setattr(ly, field, Scale(*cc["%s.%s" % (p, key)]))
        m = Model()
        m.hidden, m.layers, m.heads = cfg["hidden_size"], L, cfg["num_attention_heads"]
        m.kv_heads, m.head_dim, m.inter = KVH, cfg["head_dim"], cfg["intermediate_size"]
        m.vocab, m.context_cap = cfg["vocab_size"], cfg["context_cap"]
        m.embed = keep(w["embed"])
        m.head = keep(w["embed"] if cfg["tie_word_embeddings"] else w["lm_head"])
        m.final_gain = keep(w["final_norm.gain"])
        m.c_embed = Scale(*cc["embed"])
        m.c_final_norm = Scale(*cc["final_norm"])
        m.rope_cos, m.rope_sin = keep(rope["cos"]), keep(rope["sin"])
        m.silu_table = keep(silu)
        m.layer = C.cast(self.layers, C.POINTER(Layer))
        self.m = m
        self.kv_block_bytes = L * 2 * KVH * cfg["head_dim"] * cfg["context_cap"]

    def lora(self, adapter_artifact: bytes):
        """osc_lora_layer[] for an adapter artifact (returned object keeps arrays alive)."""
        v = A.parse_artifact(adapter_artifact)
        w = v.tensors(A.SEC_WEIGHTS, np.int8)
        dfs = v.tensors(A.SEC_DELTA_FOLD, np.int32)
        ufs = v.tensors(A.SEC_U_FOLD, np.int32)
        rank = int.from_bytes(bytes(v.sections[A.SEC_PROVENANCE][8:12]), "little")
        L = self.cfg["num_hidden_layers"]
        arr = (LoraLayer * L)()
        keepl = []
        for l in range(L):
            arr[l].rank = rank
            for proj in ("q", "k", "v", "o", "gate", "up", "down"):
                nm = "layer%d.%s_proj" % (l, proj)
                if nm in dfs:
                    lp = getattr(arr[l], proj)
                    for f, a in (("a_w", w[nm + ".lora_A"]), ("b_w", w[nm + ".lora_B"]),
                                 ("u_fold", ufs[nm]), ("d_fold", dfs[nm])):
                        a = np.ascontiguousarray(a)
                        keepl.append(a)
                        setattr(lp, f, _ptr(a))
        arr._keep = keepl
        return arr


class PortSeq:
    """One sequence driven through the restatement with sslm_prefill / sslm_decode_step semantics."""

    def __init__(self, model: PortModel):
        self.pm = model
        self.hidden = np.zeros(model.cfg["hidden_size"], dtype=np.int8)
        self.kv = np.zeros(model.kv_block_bytes, dtype=np.int8)
        self.s = Seq(_ptr(self.hidden), Scale(0, 0), 0, 0, 0, _ptr(self.kv))
        self.current_token = -1
        self.ready_for_logits = False
        self.lora = None

    def prefill(self, tokens):
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        st = port().osc_prefill(C.byref(self.pm.m), self.lora, C.byref(self.s), _ptr(toks), toks.size)
        if st == 0 and toks.size:
            self.current_token = int(toks[-1])
            self.ready_for_logits = True
        return st

    def decode_step(self, layer_budget: int, want_logits: bool = False):
        """(status, token or -1, logits or None) with the semantics of one sslm_decode_step call."""
        lib = port()
        if self.ready_for_logits:
            self.ready_for_logits = False
        else:
            if self.s.layer_index == 0:
                st = lib.osc_embed_into_seq(C.byref(self.pm.m), C.byref(self.s), self.current_token)
                if st:
                    return st, -1, None
            st = lib.osc_layer_loop(C.byref(self.pm.m), self.lora, C.byref(self.s), layer_budget)
            if st:
                return st, -1, None
            if self.s.layer_index < self.pm.cfg["num_hidden_layers"]:
                return 0, -1, None
        logits = np.empty(self.pm.cfg["vocab_size"], dtype=np.int32) if want_logits else None
        tok = C.c_int32(-1)
        st = lib.osc_logits_argmax(C.byref(self.pm.m), C.byref(self.s),
                                   _ptr(logits) if want_logits else None, C.byref(tok))
        if st:
            return st, -1, None
        self.current_token = tok.value
        self.s.layer_index = 0
        return 0, tok.value, logits

    def decode(self, n_tokens: int, layer_budget: int):
        out = []
        while len(out) < n_tokens:
            st, tok, _ = self.decode_step(layer_budget)
            assert st == 0, st
            if tok >= 0:
                out.append(tok)
        return out


def parse_trace(buf) -> dict:
    """Per-site trace records (osc_trace_begin / sslm_b200_trace write the same layout) as
    {(position, layer, site): (m, e, codes bytes)}."""
    import struct
    raw = bytes(buf)
    out, off = {}, 0
    while off + 40 <= len(raw):
        position, layer, site, m, e, n, row = struct.unpack_from("<qiiqqii", raw, off)
        if n <= 0:
            break
        out[(position, layer, site)] = (m, e, raw[off + 40:off + 40 + n])
        off += 40 + ((n + 7) & ~7)
    return out

"""`.sslm` v2 artifact reader/writer and seeded synthetic Qwen2.5-shape models.

Host-side tooling for the forward-pass hot path: the engine only ever sees
artifact bytes (``sslm_model_map`` / ``sslm_adapter_map``), so synthetic base and
adapter artifacts are produced here, byte-compatible with the reference loader.

Layout facts follow the reference's format description (docs/sslm_format.md:47-77
header and section table, :200-238 tensor manifests, :242-288 KVC1 keyed constants,
:292-327 CFG1, :340-365 SIL1) and the tensor/constant *names* the reference's
marshal resolves (include/superslm/layer_marshal.h:141-322,
src/sslm_abi.cpp:637-663, include/superslm/adapter_marshal.h:262-451).

Synthetic values: int8 weights/gains uniform in [-127,127]; WSC1 fold rows
``(0, mult in [2^30,2^31), shift in [shift_lo, shift_hi])``; site constants from a
closed-form scale-balancing recipe (each carried scale read as a real "value per
code"), so that a random model stays inside every integer-domain gate of the
forward pass. Every stream derives from one 64-bit seed through a 64-bit LCG
(x <- x*6364136223846793005 + 1442695040888963407), with one sub-stream per
tensor name, so artifacts are regenerated anywhere and never committed.
"""
from __future__ import annotations

import hashlib
import math
import struct
from dataclasses import dataclass, field
from fractions import Fraction

import numpy as np

MASK64 = (1 << 64) - 1
LCG_A = 6364136223846793005
LCG_C = 1442695040888963407

# section types / dtypes (docs/sslm_format.md:86-130)
SEC_CONFIG, SEC_PROVENANCE, SEC_WEIGHTS, SEC_BIASES, SEC_ROPE = 0, 1, 2, 3, 4
SEC_WEIGHT_SCALES, SEC_COMPOSITION, SEC_KV_SCALES, SEC_KV_RECIP = 6, 7, 8, 9
SEC_SIGMOID_LUT, SEC_DELTA_FOLD, SEC_U_FOLD = 12, 40, 41
DT_RAW, DT_INT8, DT_INT32, DT_INT64 = 0, 1, 2, 3
_DT_SIZE = {DT_RAW: 1, DT_INT8: 1, DT_INT32: 4, DT_INT64: 8}
_SEC_DTYPE = {SEC_WEIGHTS: DT_INT8, SEC_BIASES: DT_INT64, SEC_ROPE: DT_INT64,
              SEC_WEIGHT_SCALES: DT_INT32, SEC_SIGMOID_LUT: DT_INT32,
              SEC_DELTA_FOLD: DT_INT32, SEC_U_FOLD: DT_INT32}

# bit positions of the adaptable projections inside ADP1.target_modules_mask
# (include/superslm/model.h:439-441)
PEFT_ORDER = ("q_proj", "o_proj", "gate_proj", "up_proj", "down_proj", "k_proj", "v_proj")


# --------------------------------------------------------------------------
# seeded streams
# --------------------------------------------------------------------------
def _name_seed(seed: int, name: str) -> int:
    h = 0xCBF29CE484222325 ^ (seed & MASK64)
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & MASK64
    # one LCG step so that nearby names do not start on nearby states
    return (h * LCG_A + LCG_C) & MASK64


def lcg_stream(x0: int, n: int) -> np.ndarray:
    """The n LCG states following x0 (x1..xn), vectorised by block doubling."""
    if n <= 0:
        return np.zeros(0, dtype=np.uint64)
    out = np.empty(n, dtype=np.uint64)
    out[0] = (x0 * LCG_A + LCG_C) & MASK64
    have = 1
    a_k, c_k = LCG_A, LCG_C  # k-step jump: x_{i+k} = a_k x_i + c_k
    with np.errstate(over="ignore"):
        while have < n:
            take = min(have, n - have)
            out[have:have + take] = out[:take] * np.uint64(a_k) + np.uint64(c_k)
            have += take
            c_k = (a_k * c_k + c_k) & MASK64
            a_k = (a_k * a_k) & MASK64
    return out


def stream_uniform(seed: int, name: str, n: int, lo: int, hi: int) -> np.ndarray:
    """n integers uniform in [lo, hi] from the (seed, name) sub-stream (int64)."""
    span = hi - lo + 1
    out = np.empty(n, dtype=np.int64)
    x0 = _name_seed(seed, name)
    step = 1 << 24
    done = 0
    while done < n:
        take = min(step, n - done)
        s = lcg_stream(x0, take)
        x0 = int(s[-1])
        out[done:done + take] = ((s >> np.uint64(32)) % np.uint64(span)).astype(np.int64) + lo
        done += take
    return out


def stream_int8(seed: int, name: str, n: int) -> np.ndarray:
    return stream_uniform(seed, name, n, -127, 127).astype(np.int8)


# --------------------------------------------------------------------------
# integer helpers (Python big-int restatements used only to *derive constants*)
# --------------------------------------------------------------------------
def dynamic_scale_reciprocal(dn: int) -> int:
    """round_half_up(2^62/dn) by seed + 3 Newton + 2 corrections, the sequence the
    reference runs at load/run time (src/intmath.cpp:303-333); Python's >> is a
    floor shift like the reference's arithmetic shift."""
    kc32 = (2 * (48 << 31) + 17) // 34
    kc32_2 = (2 * (32 << 31) + 17) // 34
    y = kc32 - ((kc32_2 * dn) >> 31)
    for _ in range(3):
        dn_y = (dn * y) >> 31
        y = (y * ((1 << 32) - dn_y)) >> 31
    for _ in range(2):
        r2 = 2 * ((1 << 62) - y * dn)
        if r2 >= dn:
            y += 1
        elif r2 < -dn:
            y -= 1
    return y


def canonical_scale(x) -> tuple[int, int]:
    """(m, e), m in [2^30, 2^31), x ~= m * 2^e, round-half-even."""
    fx = Fraction(x)
    assert fx > 0
    e = math.floor(math.log2(float(fx))) - 30
    while True:
        q = fx / (Fraction(2) ** e)
        m = round(q)  # Fraction rounds half to even
        if m >= (1 << 31):
            e += 1
            continue
        if m < (1 << 30):
            e -= 1
            continue
        return int(m), int(e)


# --------------------------------------------------------------------------
# container + sub-format writers
# --------------------------------------------------------------------------
def _align_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def build_container(sections: list[tuple[int, bytes]], flags: int = 0, alignment: int = 64) -> bytes:
    """sections: list of (section_type, payload). Returns the file bytes."""
    table_end = 64 + 40 * len(sections)
    placed = []
    cur = table_end
    for stype, data in sections:
        off = _align_up(cur, alignment)
        placed.append((stype, off, data))
        cur = off + len(data)
    buf = bytearray(cur)
    buf[0:4] = b"SSLM"
    struct.pack_into("<IIIII", buf, 4, 2, 64, len(sections), flags, 0)
    struct.pack_into("<Q", buf, 24, cur)
    for i, (stype, off, data) in enumerate(placed):
        dt = _SEC_DTYPE.get(stype, DT_RAW)
        row = 64 + 40 * i
        struct.pack_into("<IIQQQII", buf, row, stype, dt, off, len(data),
                         len(data) // _DT_SIZE[dt], alignment, 0)
        buf[off:off + len(data)] = data
    digest = hashlib.sha256(buf).digest()
    buf[32:64] = digest
    return bytes(buf)


def tensor_manifest(magic: bytes, elem_size: int, tensors: list[tuple[str, np.ndarray]]) -> bytes:
    n = len(tensors)
    names = b"".join(t[0].encode() for t in tensors)
    data_floor = _align_up(16 + 48 * n + len(names), 8)
    descs = bytearray()
    name_off = 0
    data_off = data_floor
    chunks = []
    for name, arr in tensors:
        arr = np.ascontiguousarray(arr)
        assert arr.dtype.itemsize == elem_size, (name, arr.dtype)
        shape = list(arr.shape) + [0] * (4 - arr.ndim)
        nb = name.encode()
        descs += struct.pack("<III4IQQI", name_off, len(nb), arr.ndim, *shape, data_off, arr.size, 0)
        name_off += len(nb)
        chunks.append((data_off, arr))
        data_off = _align_up(data_off + arr.nbytes, 8)
    out = bytearray(data_off)
    out[0:4] = magic
    struct.pack_into("<III", out, 4, 1, n, len(names))
    out[16:16 + len(descs)] = descs
    out[16 + len(descs):16 + len(descs) + len(names)] = names
    mv = memoryview(out)
    for off, arr in chunks:
        mv[off:off + arr.nbytes] = arr.view(np.uint8).reshape(-1).data
    return bytes(out)


def keyed_constants(entries: list[tuple[str, tuple[int, ...]]], words: int) -> bytes:
    n = len(entries)
    names = b"".join(k.encode() for k, _ in entries)
    out = bytearray(24 + 8 * n + 8 * words * n + len(names))
    out[0:4] = b"KVC1"
    struct.pack_into("<IIIII", out, 4, 1, n, words, len(names), 0)
    off = 0
    for i, (k, _) in enumerate(entries):
        struct.pack_into("<II", out, 24 + 8 * i, off, len(k.encode()))
        off += len(k.encode())
    vbase = 24 + 8 * n
    for i, (_, v) in enumerate(entries):
        assert len(v) == words
        struct.pack_into("<%dq" % words, out, vbase + 8 * words * i, *v)
    out[vbase + 8 * words * n:] = names
    return bytes(out)


def cfg1(hidden, layers, heads, kv_heads, head_dim, inter, vocab, context_cap,
         tie=1, kv_block=16, rope_theta=1e6, eps=1e-6) -> bytes:
    return struct.pack("<4s16Idd", b"CFG1", 1, hidden, layers, heads, kv_heads, head_dim, inter,
                       vocab, context_cap, tie, 0, kv_block, 15, 1, 0, 0, rope_theta, eps)


def sigmoid_lut_table() -> np.ndarray:
    """1025 Q15 nodes of sigmoid over [-16,16] (docs/sslm_format.md:340-365):
    entry i = round_half_even(sigmoid(-16 + i/32) * 2^15)."""
    out = np.empty(1025, dtype=np.int32)
    for i in range(1025):
        x = -16.0 + i * (32.0 / 1024.0)
        out[i] = int(round(32768.0 / (1.0 + math.exp(-x))))
    return out


def sil1() -> bytes:
    return struct.pack("<4sIII", b"SIL1", 1, 1025, 0) + sigmoid_lut_table().tobytes()


def rope_tables(context_cap: int, head_dim: int, theta: float) -> tuple[np.ndarray, np.ndarray]:
    pos = np.arange(context_cap, dtype=np.float64)[:, None]
    i = np.arange(head_dim // 2, dtype=np.float64)[None, :]
    ang = pos * np.power(theta, -2.0 * i / head_dim)
    cos = np.rint(np.cos(ang) * (1 << 30)).astype(np.int64)
    sin = np.rint(np.sin(ang) * (1 << 30)).astype(np.int64)
    return cos, sin


# --------------------------------------------------------------------------
# synthetic models
# --------------------------------------------------------------------------
@dataclass
class Shape:
    name: str
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    inter: int
    vocab: int

    @property
    def kv_hidden(self):
        return self.kv_heads * self.head_dim


SHAPES = {
    # Qwen2.5 architectures named by the benchmark configs
    "0.5b": Shape("0.5b", 896, 24, 14, 2, 64, 4864, 151936),
    "1.5b": Shape("1.5b", 1536, 28, 12, 2, 128, 8960, 151936),
    "3b": Shape("3b", 2048, 36, 16, 2, 128, 11008, 151936),
    # small geometries for tests (same structure: GQA, SwiGLU, tied head)
    "tiny": Shape("tiny", 128, 2, 4, 2, 32, 256, 512),
    "small": Shape("small", 256, 3, 4, 2, 64, 768, 1024),
    "mini1.5b": Shape("mini1.5b", 1536, 2, 12, 2, 128, 8960, 4096),
    # two layers at the 0.5B and 3B widths (GQA 7:1 with head_dim 64; GQA 8:1), and four layers at
    # the 3B widths for the adapter-swap workload: long rows at real widths that a CPU still
    # finishes in minutes
    "mini0.5b": Shape("mini0.5b", 896, 2, 14, 2, 64, 4864, 4096),
    "mini3b": Shape("mini3b", 2048, 2, 16, 2, 128, 11008, 4096),
    "3b4l": Shape("3b4l", 2048, 4, 16, 2, 128, 11008, 8192),
}

_W_RMS = 73.3  # rms of a uniform integer in [-127,127]


def _s_ref(k_in: int, in_rms: float) -> float:
    return 2.0 ** 8.5 / (_W_RMS * math.sqrt(k_in) * in_rms)


def _fold_rows(seed, name, n, shift_lo, shift_hi) -> np.ndarray:
    mult = stream_uniform(seed, name + ".mult", n, 1 << 30, (1 << 31) - 1)
    shift = stream_uniform(seed, name + ".shift", n, shift_lo, shift_hi)
    rows = np.zeros((n, 3), dtype=np.int32)
    rows[:, 1] = mult.astype(np.int32)
    rows[:, 2] = shift.astype(np.int32)
    return rows


SEC_SCHEMA_MASKS = 30


def schema_masks(vocab: int, schemas: list[dict]) -> bytes:
    """SCM1 section (include/superslm/schema_masks.h): 24-byte header, 56-byte descriptors, name
    blob, then per schema one vocab-bit mask page per DFA state, the (states + 1) row offsets,
    the ascending accepting states and the (token, next state) transitions sorted by token
    inside each state's row. schemas: [{"name": str, "accepting": [state...],
    "rows": [[(token, next_state), ...] per state]}]. A state's mask page has exactly the bits
    of its row's tokens (the loader checks that)."""
    names = b"".join(s["name"].encode() for s in schemas)
    manifest_end = 24 + 56 * len(schemas) + len(names)
    page = (vocab + 7) // 8
    body = bytearray()
    descs = bytearray()
    name_off = 0

    def place(chunk: bytes) -> int:
        off = manifest_end + len(body)
        body.extend(chunk)
        body.extend(b"\0" * ((-len(body)) % 8))
        return off

    for s in schemas:
        rows = [sorted(r) for r in s["rows"]]
        n_states = len(rows)
        pages = np.zeros((n_states, page), dtype=np.uint8)
        offsets = [0]
        trans = []
        for st, row in enumerate(rows):
            for tok, nxt in row:
                pages[st, tok >> 3] |= np.uint8(1 << (tok & 7))
                trans.append((tok, nxt))
            offsets.append(len(trans))
        acc = sorted(s["accepting"])
        nb = s["name"].encode()
        o_pages = place(pages.tobytes())
        o_offs = place(np.asarray(offsets, dtype="<u4").tobytes())
        o_acc = place(np.asarray(acc, dtype="<u4").tobytes())
        o_tr = place(np.asarray(trans, dtype="<u4").reshape(-1, 2).tobytes() if trans else b"")
        descs += struct.pack("<IIIIIIQQQQ", name_off, len(nb), n_states, len(acc), len(trans), 0,
                             o_pages, o_offs, o_acc, o_tr)
        name_off += len(nb)
    head = struct.pack("<4sIIIII", b"SCM1", 1, len(schemas), vocab, len(names), 0)
    return bytes(head + descs + names + body)


def synthetic_schemas(seed: int, vocab: int, count: int, states: int = 6, fanout: int = 40) -> list[dict]:
    """`count` seeded DFAs over the vocabulary: every state but the last allows `fanout` tokens,
    each leading to a seeded next state; the last state allows nothing (a dead end)."""
    out = []
    for k in range(count):
        rows = []
        for st in range(states):
            if st == states - 1:
                rows.append([])
                continue
            toks = np.unique(stream_uniform(seed, "schema%d.s%d.tok" % (k, st), fanout, 0, vocab - 1))
            nxt = stream_uniform(seed, "schema%d.s%d.next" % (k, st), toks.size, 0, states - 1)
            rows.append([(int(t), int(n)) for t, n in zip(toks, nxt)])
        out.append({"name": "schema_%d" % k, "accepting": [states - 2, states - 1], "rows": rows})
    return out


def build_synthetic_model(shape: Shape | str, seed: int, context_cap: int,
                          shift_lo: int = 8, shift_hi: int = 20, bias_bits: int = 0,
                          flags: int = 0, schemas: int = 0, const_overrides: dict | None = None) -> bytes:
    """A loadable base artifact of the given architecture (header flags 0). bias_bits > 0 adds a
    BIA1 section: int64 q/k/v bias codes (Q30 against the projection's input scale, as the
    converter writes them for Qwen2.5's q/k/v biases), uniform in +-2^bias_bits. schemas > 0 adds
    an SCM1 section with that many seeded decode schemas (synthetic_schemas). const_overrides
    replaces composition constants by name ("layer0.mlp_norm" -> (m, e)): the way tests build
    artifacts that leave an integer-domain gate of the forward pass on purpose."""
    sh = SHAPES[shape] if isinstance(shape, str) else shape
    H, L, I, KV = sh.hidden, sh.layers, sh.inter, sh.kv_hidden
    weights: list[tuple[str, np.ndarray]] = []
    wsc: list[tuple[str, np.ndarray]] = []
    consts: list[tuple[str, tuple[int, ...]]] = []
    kv_scales: list[tuple[str, tuple[int, ...]]] = []
    kv_recips: list[tuple[str, tuple[int, ...]]] = []
    biases: list[tuple[str, np.ndarray]] = []

    weights.append(("embed", stream_int8(seed, "embed", sh.vocab * H).reshape(sh.vocab, H)))
    weights.append(("final_norm.gain", stream_int8(seed, "final_norm.gain", H)))
    inv127 = Fraction(1, 127)
    norm_c = canonical_scale(inv127 / (1 << 16) / 127)
    consts.append(("embed", canonical_scale(inv127 / 127)))
    consts.append(("final_norm", norm_c))
    s_kh = Fraction(1, 30)
    for l in range(L):
        p = "layer%d" % l
        dims = {"q_proj": (H, H), "k_proj": (KV, H), "v_proj": (KV, H), "o_proj": (H, H),
                "gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I)}
        for proj, (n_out, k_in) in dims.items():
            nm = "%s.%s" % (p, proj)
            weights.append((nm, stream_int8(seed, nm, n_out * k_in).reshape(n_out, k_in)))
            wsc.append((nm, _fold_rows(seed, nm, n_out, shift_lo, shift_hi)))
        weights.append((p + ".attn_norm.gain", stream_int8(seed, p + ".attn_norm.gain", H)))
        weights.append((p + ".mlp_norm.gain", stream_int8(seed, p + ".mlp_norm.gain", H)))
        ctx = np.zeros((sh.heads, 3), dtype=np.int32)
        ctx[:, 0] = 1
        wsc.append((p + ".ctx_fold", ctx))
        if bias_bits > 0:
            for proj, n_out in (("q_proj", H), ("k_proj", KV), ("v_proj", KV)):
                nm = "%s.%s" % (p, proj)
                lo_bits = max(bias_bits - 20, 0)
                hi = stream_uniform(seed, nm + ".bias_hi", n_out, -(1 << min(bias_bits, 20)), 1 << min(bias_bits, 20))
                lo = stream_uniform(seed, nm + ".bias_lo", n_out, 0, (1 << lo_bits) - 1) if lo_bits else 0
                biases.append((nm, (hi * (1 << lo_bits) + lo).astype(np.int64)))

        s_norm_in = _s_ref(H, 0.58)
        consts.append((p + ".attn_norm", norm_c))
        consts.append((p + ".mlp_norm", norm_c))
        for proj in ("q_proj", "gate_proj", "up_proj"):
            consts.append(("%s.%s" % (p, proj), canonical_scale(Fraction(s_norm_in) / 127)))
        consts.append((p + ".o_proj", canonical_scale(Fraction(_s_ref(H, 0.35)) / 127)))
        consts.append((p + ".down_proj", canonical_scale(Fraction(_s_ref(I, 0.35)) / 127)))
        consts.append((p + ".attn_ctx", canonical_scale(s_kh / (1 << 15) / 127)))
        consts.append((p + ".mlp_act", canonical_scale(Fraction(1, (1 << 15) * 127))))
        consts.append((p + ".attn_residual", canonical_scale(inv127)))
        consts.append((p + ".mlp_residual", canonical_scale(inv127)))
        for h in range(sh.kv_heads):
            consts.append(("%s.softmax_khead%d" % (p, h),
                           canonical_scale(Fraction(float(s_kh) / math.sqrt(sh.head_dim)))))
            m_t, e_t = canonical_scale(s_kh / Fraction(s_norm_in))
            r_t = dynamic_scale_reciprocal(m_t)
            for kv in ("k", "v"):
                kv_scales.append(("%s.%s_head%d" % (p, kv, h), canonical_scale(s_kh)))
                kv_recips.append(("%s.%s_head%d" % (p, kv, h), (m_t, e_t, r_t)))

    if const_overrides:
        left = dict(const_overrides)
        consts = [(k, tuple(left.pop(k))) if k in left else (k, v) for k, v in consts]
        assert not left, "unknown constants: %s" % sorted(left)
    cos, sin = rope_tables(context_cap, sh.head_dim, 1e6)
    sections = [
        (SEC_CONFIG, cfg1(H, L, sh.heads, sh.kv_heads, sh.head_dim, I, sh.vocab, context_cap)),
        (SEC_SIGMOID_LUT, sil1()),
        (SEC_WEIGHTS, tensor_manifest(b"WGT1", 1, weights)),
        (SEC_WEIGHT_SCALES, tensor_manifest(b"WSC1", 4, wsc)),
        (SEC_ROPE, tensor_manifest(b"ROP1", 8, [("cos", cos), ("sin", sin)])),
        (SEC_COMPOSITION, keyed_constants(consts, 2)),
        (SEC_KV_SCALES, keyed_constants(kv_scales, 2)),
        (SEC_KV_RECIP, keyed_constants(kv_recips, 3)),
    ]
    if biases:
        sections.insert(3, (SEC_BIASES, tensor_manifest(b"BIA1", 8, biases)))
    if schemas > 0:
        sections.append((SEC_SCHEMA_MASKS, schema_masks(sh.vocab, synthetic_schemas(seed, sh.vocab, schemas))))
    return build_container(sections, flags)


def build_synthetic_adapter(base: bytes, seed: int, rank: int = 16,
                            projections=("q_proj", "k_proj", "v_proj", "o_proj"),
                            u_exp=(8, 9), d_exp=(8, 10), name: str = "synthetic",
                            layer_d_exp: dict | None = None) -> bytes:
    """A rank-`rank` runtime-additive LoRA adapter bound to `base` (ADP1 + lora_A/B +
    DFS1/UFS1). Layout: include/superslm/adapter_marshal.h:38-53, :266-307. layer_d_exp gives
    single layers their own delta-fold exponent range (tests use it to make one layer's delta
    leave the funnel's domain)."""
    view = parse_artifact(base)
    cfg = view.config
    H, I, KV, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["kv_hidden"], cfg["num_hidden_layers"]
    mask = 0
    for pr in projections:
        mask |= 1 << PEFT_ORDER.index(pr)
    nb = name.encode()
    adp1 = struct.pack("<4sIII32sdIII", b"ADP1", 1, rank, mask, base[32:64], 16.0, 0, 0, len(nb)) + nb
    weights, dfs, ufs = [], [], []
    for l in range(L):
        for pr in projections:
            n_out = {"q_proj": H, "o_proj": H, "down_proj": H, "k_proj": KV, "v_proj": KV,
                     "gate_proj": I, "up_proj": I}[pr]
            k_in = I if pr == "down_proj" else H
            nm = "layer%d.%s" % (l, pr)
            weights.append((nm + ".lora_A", stream_int8(seed, nm + ".A", rank * k_in).reshape(rank, k_in)))
            weights.append((nm + ".lora_B", stream_int8(seed, nm + ".B", n_out * rank).reshape(n_out, rank)))
            ufs.append((nm, _fold_rows(seed, nm + ".ufs", rank, u_exp[0], u_exp[1])))
            de = (layer_d_exp or {}).get(l, d_exp)
            dfs.append((nm, _fold_rows(seed, nm + ".dfs", n_out, de[0], de[1])))
    cfg_bytes = view.sections[SEC_CONFIG]
    sections = [
        (SEC_CONFIG, bytes(cfg_bytes)),
        (SEC_SIGMOID_LUT, sil1()),
        (SEC_PROVENANCE, adp1),
        (SEC_WEIGHTS, tensor_manifest(b"WGT1", 1, weights)),
        (SEC_DELTA_FOLD, tensor_manifest(b"DFS1", 4, dfs)),
        (SEC_U_FOLD, tensor_manifest(b"UFS1", 4, ufs)),
    ]
    return build_container(sections)


# --------------------------------------------------------------------------
# reader (used by the test harness to feed the CPU oracle port)
# --------------------------------------------------------------------------
@dataclass
class ArtifactView:
    raw: bytes
    sections: dict = field(default_factory=dict)   # type -> memoryview of payload
    config: dict = field(default_factory=dict)

    def tensors(self, stype: int, dtype) -> dict:
        sec = self.sections[stype]
        base = np.frombuffer(sec, dtype=np.uint8)
        _, n, name_len = struct.unpack_from("<III", sec, 4)
        names_off = 16 + 48 * n
        out = {}
        for i in range(n):
            (no, nl, rank, s0, s1, s2, s3, doff, cnt, _r) = struct.unpack_from("<III4IQQI", sec, 16 + 48 * i)
            nm = bytes(sec[names_off + no:names_off + no + nl]).decode()
            shp = [s0, s1, s2, s3][:rank]
            isz = np.dtype(dtype).itemsize
            out[nm] = base[doff:doff + cnt * isz].view(dtype).reshape(shp)
        return out

    def constants(self, stype: int) -> dict:
        sec = self.sections[stype]
        _, n, words, name_len, _r = struct.unpack_from("<IIIII", sec, 4)
        vbase = 24 + 8 * n
        nbase = vbase + 8 * words * n
        out = {}
        for i in range(n):
            no, nl = struct.unpack_from("<II", sec, 24 + 8 * i)
            nm = bytes(sec[nbase + no:nbase + no + nl]).decode()
            out[nm] = struct.unpack_from("<%dq" % words, sec, vbase + 8 * words * i)
        return out


def parse_artifact(raw: bytes) -> ArtifactView:
    assert raw[0:4] == b"SSLM"
    _ver, _hb, nsec, _flags, _r0 = struct.unpack_from("<IIIII", raw, 4)
    v = ArtifactView(raw=raw)
    mv = memoryview(raw)
    for i in range(nsec):
        stype, _dt, off, size, _cnt, _al, _rs = struct.unpack_from("<IIQQQII", raw, 64 + 40 * i)
        v.sections[stype] = mv[off:off + size]
    c = struct.unpack_from("<4s16Idd", v.sections[SEC_CONFIG], 0)
    keys = ["hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
            "head_dim", "intermediate_size", "vocab_size", "context_cap", "tie_word_embeddings",
            "kv_precision", "kv_block_size"]
    v.config = dict(zip(keys, c[2:13]))
    v.config["kv_hidden"] = v.config["num_key_value_heads"] * v.config["head_dim"]
    return v

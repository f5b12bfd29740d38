"""Transcribes the golden vectors of the reference's own test fixtures into JSON.

The reference keeps its known-answer vectors for the integer primitives as generated
C++ headers (tests/sslm_*_fixtures.h; produced by its arbitrary-precision Python
generators, never by the C++ under test). This script reads those headers AS TEXT --
struct definitions and constexpr array initialisers -- and writes the values to
tests/golden/reference_fixtures.json so that the oracle and the CUDA kernels can be
checked against them on machines where the reference tree is absent.

Run where the reference is mounted:
    python tests/golden/transcribe_reference_fixtures.py [<reference root>]
"""
from __future__ import annotations

import json
import os
import re
import sys

HEADERS = [
    "tests/sslm_intmath_fixtures.h",
    "tests/sslm_s3_1_wide_intmath_fixtures.h",
    "tests/sslm_iexp_domain_fixtures.h",
    "tests/sslm_s3_1_c30_iexp_domain_sweep_fixtures.h",
    "tests/sslm_c32_softmax_row_width_gate_fixtures.h",
    "tests/sslm_s3_2_fixtures.h",
    "tests/sslm_s3_3_fixtures.h",
    "tests/sslm_s3_3_rope_application_site_fixtures.h",
    "tests/sslm_matmul_fixtures.h",
]

CONSTS = {
    "superslm::kInt32Max": "2147483647", "superslm::kInt32Min": "(-2147483648)",
    "INT32_MAX": "2147483647", "INT32_MIN": "(-2147483648)",
    "INT64_MAX": "9223372036854775807", "INT64_MIN": "(-9223372036854775808)",
    "UINT64_MAX": "18446744073709551615", "true": "1", "false": "0", "nullptr": "0",
}


def strip_comments(s: str) -> str:
    s = re.sub(r"/\*.*?\*/", "", s, flags=re.S)
    out = []
    for line in s.splitlines():
        # keep string literals intact: cut at // only outside quotes
        q = False
        cut = len(line)
        i = 0
        while i < len(line) - 1:
            c = line[i]
            if c == '"' and (i == 0 or line[i - 1] != "\\"):
                q = not q
            elif not q and c == "/" and line[i + 1] == "/":
                cut = i
                break
            i += 1
        out.append(line[:cut])
    return "\n".join(out)


def split_top(s: str) -> list[str]:
    parts, depth, cur, q = [], 0, [], False
    for i, c in enumerate(s):
        if c == '"' and (i == 0 or s[i - 1] != "\\"):
            q = not q
        if not q:
            if c in "{(":
                depth += 1
            elif c in "})":
                depth -= 1
            elif c == "," and depth == 0:
                parts.append("".join(cur).strip())
                cur = []
                continue
        cur.append(c)
    tail = "".join(cur).strip()
    if tail:
        parts.append(tail)
    return parts


def leaf(tok: str):
    tok = tok.strip()
    if tok.startswith('"'):
        return "".join(re.findall(r'"((?:[^"\\]|\\.)*)"', tok))
    t = tok
    for k, v in CONSTS.items():
        t = re.sub(r"(?<![A-Za-z0-9_:])" + re.escape(k) + r"(?![A-Za-z0-9_])", v, t)
    t = re.sub(r"U?INT(?:8|16|32|64)_C\(", "(", t)
    t = re.sub(r"static_cast<[^>]+>\(", "(", t)
    t = re.sub(r"(?:int64_t|int32_t|uint64_t|size_t)\{([^}]*)\}", r"(\1)", t)
    t = re.sub(r"(?<=[0-9a-fA-F])(?:ULL|ull|LL|ll|UL|ul|U|u|L|l)\b", "", t)
    if re.fullmatch(r"[0-9xXa-fA-F\s()+\-*<>|&~/]+", t):
        try:
            return int(eval(t.replace("/", "//"), {"__builtins__": {}}, {}))
        except Exception:
            pass
    if re.fullmatch(r"&?[A-Za-z_][A-Za-z0-9_:]*(\[[0-9]+\])?", tok):
        return "@" + tok.lstrip("&")
    return {"expr": tok}


def parse_init(s: str):
    s = s.strip()
    if s.startswith("{") and s.endswith("}"):
        return [parse_init(p) for p in split_top(s[1:-1])]
    return leaf(s)


def transcribe(path: str) -> dict:
    text = strip_comments(open(path, encoding="utf-8").read())
    structs = {}
    for m in re.finditer(r"struct\s+(\w+)\s*\{(.*?)\};", text, flags=re.S):
        fields = []
        for decl in m.group(2).split(";"):
            decl = decl.strip()
            if not decl or "(" in decl:
                continue
            ty, _, names = decl.rpartition(" ")
            if "," in decl:   # "int32_t x, y, cos_q30, sin_q30"
                first, *rest = [p.strip() for p in decl.split(",")]
                ty, _, n0 = first.rpartition(" ")
                names_list = [n0] + rest
            else:
                names_list = [names]
            for n in names_list:
                fields.append(re.sub(r"\[.*\]", "", n.lstrip("*")))
        structs[m.group(1)] = fields
    arrays = {}
    pat = re.compile(r"(?:inline\s+|static\s+)?constexpr\s+([\w:]+(?:\s*\*)?)\s+(\w+)\s*(\[[^\]]*\])?\s*=\s*", re.S)
    for m in pat.finditer(text):
        i = m.end()
        if i >= len(text):
            continue
        if text[i] == "{":
            depth, j = 0, i
            while True:
                if text[j] == "{":
                    depth += 1
                elif text[j] == "}":
                    depth -= 1
                    if depth == 0:
                        break
                j += 1
            init = text[i:j + 1]
        else:
            j = text.index(";", i)
            init = text[i:j]
        arrays[m.group(2)] = {"type": m.group(1).strip(), "value": parse_init(init)}
    return {"structs": structs, "arrays": arrays}


def main():
    from oracle import harness
    root = sys.argv[1] if len(sys.argv) > 1 else harness.REF_ROOT
    out = {}
    for h in HEADERS:
        out[os.path.basename(h)] = transcribe(os.path.join(root, h))
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_fixtures.json")
    with open(dst, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    n = sum(len(v["arrays"]) for v in out.values())
    print("wrote", dst, os.path.getsize(dst), "bytes,", n, "arrays")


if __name__ == "__main__":
    main()

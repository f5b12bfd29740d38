"""Pins the CPU oracle (oracle/sslm_oracle.c) and the host build of the device integer
library (csrc/sslm_int.cuh) against the reference's own golden vectors, transcribed from
its fixture headers into tests/golden/reference_fixtures.json."""
import ctypes as C

import numpy as np
import pytest

from oracle.harness import Scale
from tests.support import devint

I64 = C.c_int64


def arr(fx, header, name):
    return fx[header]["arrays"][name]["value"]


def deref(fx, header, v):
    return arr(fx, header, v[1:]) if isinstance(v, str) and v.startswith("@") else v


INT = "sslm_intmath_fixtures.h"


def test_srdhm(fixtures_json, port):
    d = devint.lib()
    for _label, a, b, exp in arr(fixtures_json, INT, "kC2Cases"):
        assert port.osc_srdhm(a, b) == exp
        assert d.dev_srdhm(a, b) == exp


def test_rounding_divide_by_pot(fixtures_json, port):
    d = devint.lib()
    for _label, x, e, exp in arr(fixtures_json, INT, "kC1C3Cases"):
        assert port.osc_rdivpot32(x, e) == exp
        assert d.dev_rdivpot32(x, e) == exp
        assert port.osc_rdivpot64(x, e) == exp  # same tie rule at int64 width


def test_multiply_by_quantized_multiplier(fixtures_json, port):
    d = devint.lib()
    for _label, x, m, s, exp in arr(fixtures_json, INT, "kMbqmCases"):
        assert port.osc_mbqm(x, m, s) == exp
        assert d.dev_fold(x, 0, m, s) == exp
        assert port.osc_fold(x, 0, m, s) == exp
        assert port.osc_fold(x, 1, m, s) == x


def test_normalize_scale(fixtures_json, port):
    d = devint.lib()
    for _label, dp, dn, s in arr(fixtures_json, INT, "kNormalizeScaleCases"):
        for f in (port.osc_normalize_scale, d.dev_normalize_scale):
            odn, os_ = I64(), C.c_int()
            f(dp, C.byref(odn), C.byref(os_))
            assert (odn.value, os_.value) == (dn, s)


def test_dynamic_scale_reciprocal(fixtures_json, port):
    d = devint.lib()
    named = [(c[1], c[2]) for c in arr(fixtures_json, INT, "kDynRecipNamedCases")]
    dense = [tuple(c) for c in arr(fixtures_json, INT, "kDynRecipDenseCases")]
    assert len(dense) == 3000
    for dn, r in named + dense:
        assert port.osc_dyn_recip(dn) == r
        assert d.dev_dyn_recip(dn) == r


def test_requant_token_code(fixtures_json, port):
    d = devint.lib()
    cases = [c[1:] for c in arr(fixtures_json, INT, "kRequantCases")]
    cases += [c[1:] for c in arr(fixtures_json, "sslm_s3_1_wide_intmath_fixtures.h", "kRequantWideCases")]
    for x, r, s, exp in cases:
        assert port.osc_requant_code_wide(x, r, s) == exp
        assert d.dev_requant_code(x, r, s) == exp


def test_isqrt(fixtures_json, port):
    d = devint.lib()
    for c in arr(fixtures_json, INT, "kISqrtCases"):
        assert port.osc_isqrt(c[1]) == c[2]
        assert d.dev_isqrt(c[1]) == c[2]


def test_iexp_cases(fixtures_json, port):
    for _label, q, ln2, qb, qc, exp in arr(fixtures_json, INT, "kIExpCases"):
        v = I64()
        assert port.osc_iexp(q, ln2, qb, qc, None, None, C.byref(v)) == 0
        assert v.value == exp
    names = {"kOk": 0, "kBadQ": 1, "kBadQLn2": 2, "kBadQB": 3, "kNotRepresentable": 4}
    for c in arr(fixtures_json, "sslm_iexp_domain_fixtures.h", "kIExpConstructCases"):
        _label, q, ln2, qb, qc, dom, z, base, val = c
        dom = dom[1:] if dom.startswith("@") else dom
        dom = dom.split("::")[-1]
        zo, bo, v = I64(), I64(), I64()
        got = port.osc_iexp(q, ln2, qb, qc, C.byref(zo), C.byref(bo), C.byref(v))
        assert got == names[dom], c
        if got in (0, 4):
            assert (zo.value, bo.value, v.value) == (z, base, val), c
    for _label, q, ln2, qb, qc, ok in arr(fixtures_json, "sslm_iexp_domain_fixtures.h", "kIExpDomainCases"):
        v = I64()
        assert (port.osc_iexp(q, ln2, qb, qc, None, None, C.byref(v)) == 0) == bool(ok)


def test_rope_pairs(fixtures_json, port):
    d = devint.lib()
    for _label, x, y, c, s, ex, ey in arr(fixtures_json, INT, "kRopeCases"):
        ox, oy = I64(), I64()
        port.osc_rope_pair(x, y, c, s, C.byref(ox), C.byref(oy))
        assert (ox.value, oy.value) == (ex, ey)
        if abs(x) <= 127 and abs(y) <= 127:
            a, b = C.c_int8(), C.c_int8()
            d.dev_rope_pair(x, y, c, s, C.byref(a), C.byref(b))
            assert (a.value, b.value) == (max(-127, min(127, ex)), max(-127, min(127, ey)))


def test_requant_pipeline_rows(fixtures_json, port):
    """MaxAbs -> NormalizeScale -> reciprocal -> codes, through the funnel."""
    d = devint.lib()
    for label, xs, codes, n, d_prime, dn, s, r in arr(fixtures_json, INT, "kPipelineCases"):
        xs = np.array(deref(fixtures_json, INT, xs), dtype=np.int64)
        exp = np.array(deref(fixtures_json, INT, codes), dtype=np.int8)
        out = np.zeros(n, dtype=np.int8)
        sc = Scale()
        st = port.osc_funnel(xs.ctypes.data, n, None, 0, Scale(1 << 30, 0), out.ctypes.data, C.byref(sc))
        assert st == 0, label
        assert (out == exp).all(), label
        rr, ss, om, oe = I64(), C.c_int(), I64(), I64()
        assert d.dev_funnel_params(d_prime, None, 0, 1 << 30, 0, C.byref(rr), C.byref(ss), C.byref(om), C.byref(oe)) == 0
        assert (rr.value, ss.value) == (r, s), label
        assert (om.value, oe.value) == (sc.m, sc.e), label


def test_funnel_domain_witnesses(fixtures_json, port):
    h = "sslm_s3_1_wide_intmath_fixtures.h"
    for label, row, n, codes, _narrowed in arr(fixtures_json, h, "kFunnelWitnessRows"):
        row = np.array(deref(fixtures_json, h, row), dtype=np.int64)
        out = np.zeros(len(row), dtype=np.int8)
        sc = Scale()
        assert port.osc_funnel(row.ctypes.data, len(row), None, 0, Scale(1 << 30, 0), out.ctypes.data, C.byref(sc)) == 0
        assert list(out) == codes, label
    over = np.array(arr(fixtures_json, h, "kWideOverC29DomainRow"), dtype=np.int64)
    out = np.zeros(1, dtype=np.int8)
    assert port.osc_funnel(over.ctypes.data, 1, None, 0, Scale(1 << 30, 0), out.ctypes.data, C.byref(Scale())) == 1


def test_floor_division(fixtures_json, port):
    d = devint.lib()
    for hidden, roots, floor_q, trunc_q, _differs in arr(fixtures_json, "sslm_s3_2_fixtures.h", "kC31UnitCases"):
        num = hidden << 32
        assert port.osc_floor_div(num, roots) == floor_q
        assert d.dev_floor_div(num, roots) == floor_q
        assert int(num / roots) in (floor_q, trunc_q) or True


def test_c30_scale_constants_sweep(fixtures_json, port):
    d = devint.lib()
    rows = arr(fixtures_json, "sslm_s3_1_c30_iexp_domain_sweep_fixtures.h", "kC30IExpDomainSweepCases")
    assert len(rows) == 198
    for m, e, ok, ln2, qb, qc, *_ in rows:
        for f in (port.osc_iexp_scale_constants, d.dev_iexp_scale_constants):
            a, b, c = I64(), I64(), I64()
            st = f(m, e, C.byref(a), C.byref(b), C.byref(c))
            assert (st == 0) == bool(ok), (m, e)
            if ok:
                assert (a.value, b.value, c.value) == (ln2, qb, qc), (m, e)


def test_softmax_width_gate(fixtures_json, port):
    d = devint.lib()
    h = "sslm_s3_3_fixtures.h"
    for c in arr(fixtures_json, h, "kC32WidthDomainCases"):
        _label, m, e, ln2, qb, qc, row_max, width, shipped_ok, _ok48, ok47 = c
        a, b, cc = I64(), I64(), I64()
        assert port.osc_iexp_scale_constants(m, e, C.byref(a), C.byref(b), C.byref(cc)) == 0
        assert (a.value, b.value, cc.value) == (ln2, qb, qc)
        assert qb * qb + qc == row_max
        v = I64()
        assert (port.osc_iexp(0, ln2, qb, qc, None, None, C.byref(v)) == 0) == bool(shipped_ok)
        # the gate (CheckSoftmaxRowWidthDomain) is the 2^47 peak ceiling AND width * peak <= INT64_MAX
        expect = bool(ok47) and width * row_max <= (1 << 63) - 1
        pk = I64()
        assert (port.osc_softmax_width_domain(qb, qc, width) == 0) == expect
        assert bool(d.dev_softmax_width(qb, qc, width, C.byref(pk))) == expect


def test_landing_composite(fixtures_json, port):
    d = devint.lib()
    for c in arr(fixtures_json, "sslm_s3_3_fixtures.h", "kLandingCompositeCases"):
        _label, code, m_b, r_h, e_b, e_h, raw = c[:7]
        assert port.osc_landing_rescale(code, m_b, r_h, e_b, e_h, None, None) == raw
        s, x = C.c_int(), C.c_int()
        assert d.dev_landing_rescale(code, m_b, r_h, e_b, e_h, C.byref(s), C.byref(x)) == raw


def test_gemm_rows_and_composition(fixtures_json, port):
    h = "sslm_matmul_fixtures.h"
    for name in ("kRowCases", "kTailSweepCases"):
        for _label, k, n, acts, wgts, exp in arr(fixtures_json, h, name):
            a = np.array(deref(fixtures_json, h, acts), dtype=np.int8)
            w = np.array(deref(fixtures_json, h, wgts), dtype=np.int8)
            out = np.zeros(n, dtype=np.int64)
            port.osc_gemm(a.ctypes.data, w.ctypes.data, 1, k, n, out.ctypes.data)
            assert list(out) == deref(fixtures_json, h, exp)
    for _label, t, k, n, wgts, acts, exp in arr(fixtures_json, h, "kMultiRowCases"):
        a = np.array(deref(fixtures_json, h, acts), dtype=np.int8)
        w = np.array(deref(fixtures_json, h, wgts), dtype=np.int8)
        out = np.zeros(t * n, dtype=np.int64)
        port.osc_gemm(a.ctypes.data, w.ctypes.data, t, k, n, out.ctypes.data)
        assert list(out) == deref(fixtures_json, h, exp)
    # GEMM composed with the requant chain at real hidden sizes (1536, 8960, ...)
    for c in arr(fixtures_json, h, "kCompositionCases"):
        label, k, n, acts, wgts, gold, d_prime, dn, s, r, codes = c
        a = np.array(deref(fixtures_json, h, acts), dtype=np.int8)
        w = np.array(deref(fixtures_json, h, wgts), dtype=np.int8)
        out = np.zeros(n, dtype=np.int64)
        port.osc_gemm(a.ctypes.data, w.ctypes.data, 1, k, n, out.ctypes.data)
        assert list(out) == deref(fixtures_json, h, gold), label
        cod = np.zeros(n, dtype=np.int8)
        assert port.osc_funnel(out.ctypes.data, n, None, 0, Scale(1 << 30, 0), cod.ctypes.data, C.byref(Scale())) == 0
        assert list(cod) == deref(fixtures_json, h, codes), label
        assert port.osc_dyn_recip(dn) == r

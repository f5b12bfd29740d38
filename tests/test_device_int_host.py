"""The device integer library (csrc/sslm_int.cuh), compiled for the host, against the CPU
oracle on seeded sweeps: every function the kernels call, on operands that take the 64-bit
fast paths and on operands that force the general 128-bit routes."""
import ctypes as C
import random

from tests.support import devint

I64 = C.c_int64


def ri(rnd, bits):
    return rnd.randrange(-(1 << bits), 1 << bits)


def test_reciprocal_and_requant(port):
    d = devint.lib()
    rnd = random.Random(1)
    for _ in range(40000):
        x = rnd.choice([rnd.randrange(1 << 30, 1 << 31), ri(rnd, 31), ri(rnd, 40), ri(rnd, 62), rnd.randrange(1, 1000)])
        assert d.dev_dyn_recip(x) == port.osc_dyn_recip(x)
    for _ in range(60000):
        s = rnd.randrange(-1, 31)
        dn = rnd.randrange(1 << 30, 1 << 31)
        r = port.osc_dyn_recip(dn) if rnd.random() < 0.9 else rnd.randrange(1, 1 << 40)
        x = rnd.choice([ri(rnd, 31), ri(rnd, 33), ri(rnd, 10), 1 << 31, -(1 << 31), (1 << 31) + 1, 0, 1, -1])
        assert d.dev_requant_code(x, r, s) == port.osc_requant_code_wide(x, r, s), (x, r, s)


def test_narrow_coder_equals_the_wide_one(port):
    # the per-row coder's 32-bit path against RequantTokenCodeWide, with the edges of its
    # window: R = 2^32 and R just below, exponent 32/33/63, |x| = 2^31 and 2^31 + 1, rounding ties
    d = devint.lib()
    rnd = random.Random(11)
    for i in range(150000):
        s = rnd.choice([rnd.randrange(-1, 31), -1, 0, 29, 30])
        dn = rnd.choice([rnd.randrange(1 << 30, 1 << 31), 1 << 30, (1 << 30) + 1, (1 << 31) - 1])
        r = port.osc_dyn_recip(dn) if i % 10 else rnd.choice([1 << 32, (1 << 32) - 1, (1 << 31) + 1, rnd.randrange(1, 1 << 34)])
        x = rnd.choice([ri(rnd, 31), ri(rnd, 31), ri(rnd, 20), ri(rnd, 8), 1 << 31, -(1 << 31), (1 << 31) + 1,
                        -(1 << 31) - 1, (1 << 31) - 1, 0, 1, -1, ri(rnd, 40)])
        if i % 5 == 0 and 62 - s >= 33:
            # a value whose scaled magnitude sits next to a rounding tie
            k = rnd.randrange(0, 128)
            x = ((2 * k + 1) << (62 - s - 1)) // (r * 127) + rnd.choice([-1, 0, 1])
            x = rnd.choice([x, -x])
        want = port.osc_requant_code_wide(x, r, s)
        assert d.dev_code_of64(x, r, s) == want, (x, r, s)
        if -(1 << 31) <= x < (1 << 31):
            assert d.dev_code_of32(x, r, s) == want, (x, r, s)


def test_landing_rescale_fast_and_general(port):
    d = devint.lib()
    rnd = random.Random(2)
    for i in range(120000):
        code = rnd.choice([ri(rnd, 7), ri(rnd, 31), ri(rnd, 33), ri(rnd, 62), 1 << 31, -(1 << 31)])
        m = rnd.choice([rnd.randrange(1 << 30, 1 << 31), ri(rnd, 31), (1 << 31) - 1, -(1 << 31)])
        rt = rnd.choice([rnd.randrange((1 << 31) + 1, (1 << 32) + 1), 1 << 32, ri(rnd, 40), ri(rnd, 63), 0])
        ea, et = rnd.randrange(-90, 45), rnd.randrange(-70, 20)
        if i % 50 == 0:
            ea, et = ri(rnd, 63), ri(rnd, 63)
        if i % 7 == 0:      # pin the composed exponent to the edges of the fast window
            et = ea - 62 + rnd.choice([32, 33, 34, 93, 94, 95, 0, -1, 127, 128])
        s1, x1 = C.c_int(), C.c_int()
        sat, x2 = C.c_uint64(0), C.c_int()
        a = d.dev_landing_rescale(code, m, rt, ea, et, C.byref(s1), C.byref(x1))
        b = port.osc_landing_rescale(code, m, rt, ea, et, C.byref(sat), C.byref(x2))
        assert (a, s1.value, x1.value) == (b, sat.value, x2.value), (code, m, rt, ea, et)


def test_floor_div_and_isqrt(port):
    d = devint.lib()
    rnd = random.Random(3)
    for _ in range(60000):
        h = rnd.randrange(-127, 128)
        root = rnd.choice([1, 2, 3, rnd.randrange(1, 1 << 24), rnd.randrange(1, 1 << 12), 127 << 16])
        assert d.dev_floor_div_h32(h, root) == port.osc_floor_div(h * (1 << 32), root), (h, root)
        a, b = ri(rnd, 50), rnd.randrange(1, 1 << 30)
        assert d.dev_floor_div(a, b) == port.osc_floor_div(a, b)
        n = rnd.choice([rnd.randrange(0, 1 << 62), rnd.randrange(0, 1 << 40), rnd.randrange(0, 100)])
        assert d.dev_isqrt(n) == port.osc_isqrt(n)
    for _ in range(20000):      # perfect squares and their neighbours, up to the int64 ceiling
        k = rnd.choice([rnd.randrange(0, 3037000500), rnd.randrange(3037000000, 3037000500), rnd.randrange(0, 1 << 16)])
        for n in (k * k - 1, k * k, k * k + 1, k * k + k, k * k + 2 * k):
            if 0 <= n < (1 << 63):
                assert d.dev_isqrt(n) == port.osc_isqrt(n), n
    for n in ((1 << 63) - 1, (1 << 62), (1 << 62) - 1, 0, 1, 2, 3, -1, -(1 << 40)):
        assert d.dev_isqrt(n) == port.osc_isqrt(n), n
    for dn in ((1 << 30), (1 << 30) + 1, (1 << 31) - 1, (1 << 31), (1 << 30) - 1, 3 << 29, (3 << 29) + 1):
        assert d.dev_dyn_recip(dn) == port.osc_dyn_recip(dn), dn
    for den in (1, 2, 3, 1 << 40, (1 << 62) - 1):
        for q in (0, 1, 2, 32767, 32768, 65535):
            for rem in (0, 1, den - 1):
                num = min(q * den + min(rem, den - 1), (1 << 63) - 1)
                assert d.dev_udiv_small(num, den) == num // den


def test_folds_and_scale_algebra(port):
    d = devint.lib()
    rnd = random.Random(4)
    from oracle.harness import Scale
    for _ in range(60000):
        acc = ri(rnd, 31)
        mult = rnd.randrange(1 << 30, 1 << 31) if rnd.random() < 0.8 else ri(rnd, 31)
        sh, ex, idn = rnd.randrange(0, 32), rnd.randrange(-31, 32), int(rnd.random() < 0.1)
        assert d.dev_fold(acc, idn, mult, sh) == port.osc_fold(acc, idn, mult, sh)
        assert d.dev_amp_fold(acc, idn, mult, ex) == port.osc_amp_fold(acc, idn, mult, ex)
        am, bm = ri(rnd, 31), ri(rnd, 31)
        ae, be = rnd.choice([rnd.randrange(-80, 8), ri(rnd, 63)]), rnd.choice([rnd.randrange(-80, 8), ri(rnd, 63)])
        om, oe = I64(), I64()
        d.dev_combine(am, ae, bm, be, C.byref(om), C.byref(oe))
        c = port.osc_combine(Scale(am, ae), Scale(bm, be))
        assert (om.value, oe.value) == (c.m, c.e)


def test_epilogue_fold_equals_the_two_step_fold(port):
    # the GEMM epilogue's one-rounding form against ApplyWeightScaleFold: ties at every shift,
    # both signs, the int32 edges, and the operands that must stay on the two-step form
    d = devint.lib()
    rnd = random.Random(12)
    lo, hi = -(1 << 31), (1 << 31) - 1
    plain_seen = other_seen = 0
    for i in range(200000):
        sh = rnd.randrange(0, 32)
        mult = rnd.choice([rnd.randrange(1 << 30, 1 << 31), ri(rnd, 31), lo, hi, 1 << 30, -(1 << 30), 0, 1, -1])
        mult = max(lo, min(hi, mult))
        acc = rnd.choice([ri(rnd, 31), ri(rnd, 20), ri(rnd, 8), lo, hi, lo + 1, 0])
        acc = max(lo, min(hi, acc))
        if i % 3 == 0 and mult not in (0,):
            # an accumulator whose doubled high product lands next to a rounding tie of the shift
            k = rnd.randrange(-(1 << 20), 1 << 20)
            t = (2 * k + 1) << sh >> 1
            acc = max(lo, min(hi, (t << 31) // mult + rnd.choice([-1, 0, 1])))
        idn = int(i % 17 == 0)
        plain, mag = C.c_int(), C.c_uint32()
        got = d.dev_fold_epilogue(acc, idn, mult, sh, C.byref(plain), C.byref(mag))
        want = port.osc_fold(acc, idn, mult, sh)
        assert got == want, (acc, idn, mult, sh)
        if plain.value:
            plain_seen += 1
            assert mag.value == abs(want)
        else:
            other_seen += 1
            assert idn or mult == lo
    assert plain_seen > 100000 and other_seen > 1000


def test_bias_reconcile(port):
    d = devint.lib()
    rnd = random.Random(6)
    port.osc_bias_reconcile.argtypes = [I64, I64, I64, C.POINTER(I64)]
    port.osc_bias_reconcile.restype = C.c_int
    for i in range(60000):
        b = rnd.choice([ri(rnd, 47), ri(rnd, 30), ri(rnd, 62), 0, 1, -1, (1 << 63) - 1, -(1 << 63)])
        r_a = rnd.choice([rnd.randrange(1 << 31, (1 << 32) + 1), ri(rnd, 40), ri(rnd, 63), 0])
        e_a = rnd.choice([rnd.randrange(-60, -30), rnd.randrange(-95, -25), -92, -29, -93, -28, ri(rnd, 63)])
        v1, v2 = I64(), I64()
        ok1 = d.dev_bias_reconcile(b, r_a, e_a, C.byref(v1))
        ok2 = port.osc_bias_reconcile(b, r_a, e_a, C.byref(v2))
        assert ok1 == ok2, (b, r_a, e_a)
        if -92 <= e_a <= -29:
            assert v1.value == v2.value, (b, r_a, e_a)
    for acc, term in [(1, 2), ((1 << 63) - 1, 1), (-(1 << 63), -1), ((1 << 63) - 1, -(1 << 63)), (-5, 5),
                      ((1 << 62), (1 << 62)), (-(1 << 62), -(1 << 62)), (-(1 << 62) - 1, -(1 << 62))]:
        out = I64()
        fits = -(1 << 63) <= acc + term < (1 << 63)
        assert bool(d.dev_bias_accumulate(acc, term, C.byref(out))) == fits, (acc, term)
        if fits:
            assert out.value == acc + term


def test_iexp_constants_and_elements(port):
    d = devint.lib()
    rnd = random.Random(5)
    for _ in range(40000):
        m = rnd.choice([rnd.randrange(1 << 30, 1 << 31), ri(rnd, 31)])
        e = rnd.choice([rnd.randrange(-60, -25), rnd.randrange(-200, 100), ri(rnd, 63)])
        a3, b3 = [I64() for _ in range(3)], [I64() for _ in range(3)]
        sa = d.dev_iexp_scale_constants(m, e, *[C.byref(v) for v in a3])
        sb = port.osc_iexp_scale_constants(m, e, *[C.byref(v) for v in b3])
        assert (sa == 0) == (sb == 0)
        if sa == 0:
            assert [v.value for v in a3] == [v.value for v in b3]
    # elements: constants that pass the width gate, shifted scores over the whole clip range
    for _ in range(4000):
        m, e = rnd.randrange(1 << 30, 1 << 31), rnd.randrange(-53, -30)
        k = [I64() for _ in range(3)]
        if port.osc_iexp_scale_constants(m, e, *[C.byref(v) for v in k]) != 0:
            continue
        ln2, qb, qc = [v.value for v in k]
        pk = I64()
        if not d.dev_softmax_width(qb, qc, 1, C.byref(pk)) or ln2 < 1:
            continue
        assert port.osc_softmax_width_domain(qb, qc, 1) == 0
        for q in (0, -1, -ln2, -ln2 - 1, -29 * ln2, -30 * ln2, -30 * ln2 - 5, -(1 << 21), -rnd.randrange(0, 1 << 22)):
            v1, v2 = I64(), I64()
            ok = d.dev_iexp_element(q, ln2, qb, qc, pk.value, C.byref(v1))
            dom = port.osc_iexp(q, ln2, qb, qc, None, None, C.byref(v2))
            assert dom in (0, 4)
            assert v1.value == v2.value
            assert bool(ok) == (0 <= v2.value <= pk.value)


def test_single_division_reciprocal_equals_the_newton_sequence(port):
    """dyn_recip replaces DynamicScaleReciprocal's seed / Newton / correction sequence by one
    rounded division on normalised divisors [2^30, 2^31). Checked against the sequence (itself
    held to the oracle above) on every 1021st divisor plus both ends; SSLM_EXHAUSTIVE=1 walks
    all 2^30 of them (about a minute)."""
    import os
    d = devint.lib()
    first = I64(0)
    lo, hi = 1 << 30, 1 << 31
    if os.environ.get("SSLM_EXHAUSTIVE") == "1":
        assert d.dev_dyn_recip_sweep(lo, 1, hi - lo, C.byref(first)) == 0, first.value
    else:
        assert d.dev_dyn_recip_sweep(lo, 1021, (hi - lo) // 1021 + 1, C.byref(first)) == 0, first.value
        assert d.dev_dyn_recip_sweep(lo, 1, 1 << 16, C.byref(first)) == 0, first.value
        assert d.dev_dyn_recip_sweep(hi - (1 << 16), 1, 1 << 16, C.byref(first)) == 0, first.value
    for dn in (lo, lo + 1, hi - 1, 1090717716, 1156622235):
        assert d.dev_dyn_recip(dn) == port.osc_dyn_recip(dn)

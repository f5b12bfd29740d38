"""The device integer library evaluated ON THE DEVICE against the CPU oracle: a million seeded
operand tuples per primitive. The host build of the same header (tests/test_device_int_host.py)
cannot execute the device-only halves -- the rcp.approx / rsqrt.approx estimates behind the exact
divisions and roots, and the attention kernels' 32-bit softmax element -- so they are swept here.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import harness as H

pytestmark = pytest.mark.gpu

N = 1 << 20
I64 = np.int64


def device_sweep(lib, which, a, b, c, e):
    f = lib.dll.sslm_b200_int_sweep
    f.argtypes = [C.c_int32] + [C.c_void_p] * 4 + [C.c_int64] + [C.c_void_p] * 3
    outs = [np.zeros(a.size, dtype=I64) for _ in range(3)]
    assert f(which, a.ctypes.data, b.ctypes.data, c.ctypes.data, e.ctypes.data, a.size, *[o.ctypes.data for o in outs]) == 0
    return outs


def oracle_sweep(which, a, b, c, e):
    outs = [np.zeros(a.size, dtype=I64) for _ in range(3)]
    H.port().osc_sweep(which, a.ctypes.data, b.ctypes.data, c.ctypes.data, e.ctypes.data, a.size, *[o.ctypes.data for o in outs])
    return outs


def pack(hi, lo):
    return ((hi.astype(I64) << 32) | (lo.astype(I64) & 0xFFFFFFFF)).astype(I64)


def canonical(rng, n):
    return rng.integers(1 << 30, 1 << 31, n, dtype=I64)


def zeros():
    return np.zeros(N, dtype=I64)


def test_reciprocal_on_the_device(gpu_lib):
    rng = np.random.default_rng(1)
    a = canonical(rng, N)
    a[::9] = rng.integers(-(1 << 40), 1 << 40, a[::9].size, dtype=I64)     # non-canonical mantissas take the reference's sequence
    a[::11] = rng.integers(1, 1 << 20, a[::11].size, dtype=I64)
    a[:4] = [1 << 30, (1 << 31) - 1, (1 << 30) + 1, 1090717716]
    got, want = device_sweep(gpu_lib, 0, a, zeros(), zeros(), zeros()), oracle_sweep(0, a, zeros(), zeros(), zeros())
    assert (got[0] == want[0]).all()


def test_square_root_and_floor_divisions_on_the_device(gpu_lib):
    rng = np.random.default_rng(2)
    bits = rng.integers(0, 62, N)
    a = (rng.integers(0, 1 << 62, N, dtype=I64) >> (61 - bits)).astype(I64)
    a[:6] = [0, 1, 2, 3, (1 << 62) - 1, (1 << 32)]
    sq = rng.integers(1, 1 << 31, N // 4, dtype=I64)
    a[1000:1000 + sq.size] = sq * sq - rng.integers(0, 2, sq.size)          # perfect squares and their predecessors
    got, want = device_sweep(gpu_lib, 1, a, zeros(), zeros(), zeros()), oracle_sweep(1, a, zeros(), zeros(), zeros())
    assert (got[0] == want[0]).all()
    h = rng.integers(-127, 128, N, dtype=I64)
    root = (rng.integers(1, 1 << 39, N, dtype=I64) >> rng.integers(0, 38, N)).astype(I64)
    root[root < 1] = 1
    got, want = device_sweep(gpu_lib, 2, h, root, zeros(), zeros()), oracle_sweep(2, h, root, zeros(), zeros())
    assert (got[0] == want[0]).all()
    den = (rng.integers(1, 1 << 40, N, dtype=I64) >> rng.integers(0, 39, N)).astype(I64)
    den[den < 1] = 1
    q = rng.integers(0, 1 << 20, N, dtype=I64)
    num = q * den + (rng.integers(0, 1 << 40, N, dtype=I64) % den)
    got, want = device_sweep(gpu_lib, 5, num, den, zeros(), zeros()), oracle_sweep(5, num, den, zeros(), zeros())
    assert (got[0] == want[0]).all()


def test_requant_codes_and_funnel_scalars_on_the_device(gpu_lib):
    rng = np.random.default_rng(3)
    dn = canonical(rng, N)
    dn[::13] = 1 << 30                                                      # R = 2^32: the coders' edge
    r = oracle_sweep(0, dn, zeros(), zeros(), zeros())[0]
    s = rng.integers(-1, 31, N, dtype=I64)
    x = rng.integers(-(1 << 31), (1 << 31) + 1, N, dtype=I64)
    x[::7] = rng.integers(-(1 << 33), 1 << 33, x[::7].size, dtype=I64)
    x[:4] = [1 << 31, -(1 << 31), (1 << 31) + 1, 0]
    got, want = device_sweep(gpu_lib, 3, x, r, s, zeros()), oracle_sweep(3, x, r, s, zeros())
    for k in range(3):                   # the general composite and both per-row coders
        assert (got[k] == want[0]).all(), k
    mx = rng.integers(0, (1 << 31) + 3, N, dtype=I64)
    mx[::5] = (rng.integers(1, 1 << 31, mx[::5].size, dtype=I64) >> rng.integers(0, 30, mx[::5].size)).astype(I64)
    inc_m, inc_e = canonical(rng, N), rng.integers(-60, -20, N, dtype=I64)
    site = pack(canonical(rng, N), rng.integers(-60, -30, N, dtype=I64))
    got, want = device_sweep(gpu_lib, 6, mx, inc_m, inc_e, site), oracle_sweep(6, mx, inc_m, inc_e, site)
    assert (got[2] == want[2]).all()
    ok = want[2] == 0
    assert ok.sum() > N // 2
    assert (got[0][ok] == want[0][ok]).all() and (got[1][ok] == want[1][ok]).all()


def test_landing_rescale_on_the_device(gpu_lib):
    rng = np.random.default_rng(4)
    code = rng.integers(-(1 << 31), 1 << 31, N, dtype=I64)
    code[::3] = rng.integers(-127, 128, code[::3].size, dtype=I64)
    m_a = canonical(rng, N) * rng.choice(np.array([1, 1, 1, -1], dtype=I64), N)
    r_t = rng.integers((1 << 31) + 1, (1 << 32) + 1, N, dtype=I64)
    e = pack(rng.integers(-90, 40, N, dtype=I64), rng.integers(-70, 20, N, dtype=I64))
    got, want = device_sweep(gpu_lib, 4, code, m_a, r_t, e), oracle_sweep(4, code, m_a, r_t, e)
    exceeded = (want[1] & 2) != 0
    assert (got[1] == want[1]).all()
    assert (got[0][~exceeded] == want[0][~exceeded]).all()


def test_softmax_element_and_probability_on_the_device(gpu_lib):
    rng = np.random.default_rng(5)
    port = H.port()
    # constant triples of scales inside the softmax window, as k_qkv_post derives them
    sets = []
    for i in range(64):
        m, e = int(rng.integers(1 << 30, 1 << 31)), int(rng.integers(-51, -33))
        ln2, qb, qc = C.c_int64(0), C.c_int64(0), C.c_int64(0)
        if port.osc_iexp_scale_constants(m, e, C.byref(ln2), C.byref(qb), C.byref(qc)) == 0 and ln2.value >= 1 and \
           qb.value * qb.value + qc.value <= (1 << 47):
            sets.append((ln2.value, qb.value, qc.value))
    assert len(sets) >= 16
    pick = rng.integers(0, len(sets), N)
    ln2 = np.array([sets[i][0] for i in pick], dtype=I64)
    qb = np.array([sets[i][1] for i in pick], dtype=I64)
    qc = np.array([sets[i][2] for i in pick], dtype=I64)
    peak16 = ((qb * qb + qc) >> 16) + 1                                     # peak rounded up to a multiple of 2^16
    dq = (rng.integers(0, 34, N) * ln2 + rng.integers(-3, 4, N)).clip(0, (1 << 32) - 1).astype(I64)
    dq[::17] = rng.integers(0, 1 << 32, dq[::17].size, dtype=I64)
    e = pack(qc, peak16)
    got, want = device_sweep(gpu_lib, 7, dq, ln2, qb, e), oracle_sweep(7, dq, ln2, qb, e)
    assert (want[1] == 0).all()
    assert (got[0] == want[0]).all() and (got[2] == want[0]).all()
    bound = peak16 << 16
    assert (got[1] == ((want[0] < 0) | (want[0] > bound)).astype(I64)).all()
    tot = (rng.integers(1, 1 << 62, N, dtype=I64) >> rng.integers(0, 61, N)).astype(I64)
    tot[tot < 1] = 1
    ev = (rng.integers(0, 1 << 47, N, dtype=I64) % (np.minimum(tot, (1 << 47) - 1) + 1)).astype(I64)
    got = device_sweep(gpu_lib, 8, ev, tot, zeros(), zeros())
    want = ((ev.astype(np.uint64) << np.uint64(15)) // tot.astype(np.uint64)).astype(I64)
    assert (got[0] == want).all()

"""sslm_b200_linear_resident: the linear layer on device-resident operands with its scratch in
a fixed device array. Checked against sslm_b200_linear (the existing entry point, which stages
host buffers and allocates) on two calls in a row, so that a scratch slot left non-zero by the
first call would show in the second. Named to be collected last; passes alone too."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SITE = (1090717716, -44)


def reference_entry(lib, x, w, fold, in_scales):
    f = lib.dll.sslm_b200_linear
    f.argtypes = [C.c_void_p] * 3 + [C.c_int32] * 3 + [C.c_void_p, C.c_int64, C.c_int64, C.c_int32] + [C.c_void_p] * 4
    M, K = x.shape
    N = w.shape[0]
    folded = np.zeros((M, N), dtype=np.int32)
    codes = np.zeros((M, N), dtype=np.int8)
    scales = np.zeros((M, 2), dtype=np.int64)
    status = np.zeros(M, dtype=np.int32)
    assert f(x.ctypes.data, w.ctypes.data, fold.ctypes.data, M, N, K, in_scales.ctypes.data, SITE[0], SITE[1], 0,
             folded.ctypes.data, codes.ctypes.data, scales.ctypes.data, status.ctypes.data) == 0
    return folded, codes, scales, status


def resident_entry(lib, torch, x, w, fold, in_scales):
    f = lib.dll.sslm_b200_linear_resident
    f.restype = C.c_int32
    f.argtypes = [C.c_void_p] * 3 + [C.c_int32] * 3 + [C.c_void_p, C.c_int64, C.c_int64] + [C.c_void_p] * 5
    M, K = x.shape
    N = w.shape[0]
    dev = torch.device("cuda:0")
    dx, dw = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    dfold, dsc = torch.from_numpy(fold).to(dev), torch.from_numpy(in_scales).to(dev)
    # outputs pre-filled with junk: the entry must write every element it reports
    folded = torch.full((M, N), 0x5A5A5A5A, dtype=torch.int32, device=dev)
    codes = torch.full((M, N), 0x5A, dtype=torch.int8, device=dev)
    scales = torch.full((M, 2), -1, dtype=torch.int64, device=dev)
    status = torch.full((M,), 77, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    st = f(dx.data_ptr(), dw.data_ptr(), dfold.data_ptr(), M, N, K, dsc.data_ptr(), SITE[0], SITE[1],
           folded.data_ptr(), codes.data_ptr(), scales.data_ptr(), status.data_ptr(), None)
    assert st == 0
    torch.cuda.synchronize()
    return folded.cpu().numpy(), codes.cpu().numpy(), scales.cpu().numpy(), status.cpu().numpy()


def make_case(seed, M, N, K, amplitude):
    rng = np.random.default_rng(seed)
    x = rng.integers(-amplitude, amplitude + 1, (M, K)).astype(np.int8)
    w = rng.integers(-127, 128, (N, K)).astype(np.int8)
    fold = np.zeros((N, 3), dtype=np.int32)
    fold[:, 1] = rng.integers(1 << 30, 1 << 31, N)
    fold[:, 2] = rng.integers(8, 21, N)
    fold[::5, 0] = 1
    in_scales = np.stack([rng.integers(1 << 30, 1 << 31, M), np.full(M, -37)], axis=1).astype(np.int64)
    return x, w, fold, in_scales


def test_resident_linear_matches_the_allocating_entry_twice_in_a_row(gpu_lib):
    torch = pytest.importorskip("torch")
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    # the second call has fewer rows and much smaller magnitudes than the first: a row peak
    # surviving from call one would change its scales and codes
    for seed, (M, N, K, amp) in enumerate([(37, 777, 1536, 127), (21, 300, 512, 3)]):
        x, w, fold, in_scales = make_case(seed, M, N, K, amp)
        want = reference_entry(gpu_lib, x, w, fold, in_scales)
        got = resident_entry(gpu_lib, torch, x, w, fold, in_scales)
        for a, b, what in zip(got, want, ("folded", "codes", "scales", "status")):
            assert (a == b).all(), (what, seed)
        # both entry points run the same projection kernel, so the CPU oracle is asked as well
        from tests.test_gpu_parity import oracle_linear
        cpu = oracle_linear(x, w, fold, in_scales, SITE)
        for a, b, what in zip(got, cpu, ("folded", "codes", "scales", "status")):
            assert (np.asarray(a, dtype=np.int64) == np.asarray(b, dtype=np.int64)).all(), ("oracle", what, seed)


def test_resident_linear_refuses_more_rows_than_its_scratch_holds(gpu_lib):
    torch = pytest.importorskip("torch")
    torch.cuda.set_device(0)
    f = gpu_lib.dll.sslm_b200_linear_resident
    f.restype = C.c_int32
    f.argtypes = [C.c_void_p] * 3 + [C.c_int32] * 3 + [C.c_void_p, C.c_int64, C.c_int64] + [C.c_void_p] * 5
    buf = torch.zeros(1 << 16, dtype=torch.int32, device="cuda:0")
    p = buf.data_ptr()
    assert f(p, p, p, 257, 16, 16, p, SITE[0], SITE[1], p, None, None, None, None) == 1     # SSLM_INVALID_ARGUMENT
    assert f(p, p, p, 4, 16, 16400, p, SITE[0], SITE[1], p, None, None, None, None) == 1
    torch.cuda.synchronize()

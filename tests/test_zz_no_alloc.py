"""GPU test of gl_matmul_static, the allocation-free variant of the tensor-core product.

Some callers of this library cannot allocate device memory (the GPU belongs to their own arena, or
their loop must not hit cudaMalloc's device-wide synchronisation), so this entry point keeps its
scratch in a fixed array inside the library.  The test calls it through the C ABI twice in a row --
the second product is smaller and has a different layout, so stale scratch contents of the first call
would show -- and checks each result against the allocating entry point gl_matmul on the same
inputs (same kernels, so the outputs must be identical, and both within the product tolerance of a
float64 reference).  It lives in a file that pytest collects last, and it does not depend on any
earlier test: it passes alone in a fresh process and after the rest of the suite.
"""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(L, a):
    p = C.c_void_p()
    assert L.gl_device_alloc(C.byref(p), a.nbytes + 64, 0) == 0
    assert L.gl_memcpy_h2d(p, a.ctypes.data_as(C.c_void_p), a.nbytes, 0) == 0
    return p


def _product(L, g, A, B, a_mn, b_mn, static):
    M, K = A.shape
    N = B.shape[0]
    A_mem = np.ascontiguousarray(A.T) if a_mn else A
    B_mem = np.ascontiguousarray(B.T) if b_mn else B
    a_sm, a_sk = (1, M) if a_mn else (K, 1)
    b_sn, b_sk = (1, N) if b_mn else (K, 1)
    dA, dB = _dev(L, A_mem), _dev(L, B_mem)
    out = np.full((M, N), np.nan, np.float32)
    dC = _dev(L, out)
    if static:
        st = L.gl_matmul_static(dA, a_sm, a_sk, dB, b_sn, b_sk, dC, N, M, N, K, 0)
        assert st == 0, L.gl_matmul_static_error()
    else:
        st = L.gl_matmul(dA, a_sm, a_sk, dB, b_sn, b_sk, dC, N, M, N, K, g.GEMM_TCGEN05, 0)
        assert st == 0, L.gl_last_error()
    assert L.gl_memcpy_d2h(out.ctypes.data_as(C.c_void_p), dC, out.nbytes, 0) == 0
    for p in (dA, dB, dC):
        L.gl_device_free(p, 0)
    return out


def test_static_scratch_product_matches_allocating_product_twice(g):
    if g.device_count() < 1:
        pytest.fail("no sm_100 device visible")
    L = g.lib()
    rng = np.random.default_rng(2024)
    # two calls in a row: a large K-major product first, then a smaller MN-major one
    for (M, N, K, a_mn, b_mn) in [(512, 768, 1024, 0, 0), (128, 256, 96, 1, 1)]:
        A = rng.standard_normal((M, K)).astype(np.float32)
        B = rng.standard_normal((N, K)).astype(np.float32)
        got = _product(L, g, A, B, a_mn, b_mn, static=True)
        want = _product(L, g, A, B, a_mn, b_mn, static=False)
        ref = A.astype(np.float64) @ B.astype(np.float64).T
        bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64).T
        assert float(np.max(np.abs(got - ref) / bound)) <= 4e-6
        assert float(np.max(np.abs(got.astype(np.float64) - want) / bound)) <= 4e-6
        # The allocating entry point may split its last wave of tiles along k through a workspace it allocates
        # (another order of the same partial sums); with that switched off both run the same kernels in the same
        # order, so the outputs must then be identical bit for bit.
        os.environ["GLADES_TC_SPLITK"] = "0"
        try:
            same = _product(L, g, A, B, a_mn, b_mn, static=False)
        finally:
            del os.environ["GLADES_TC_SPLITK"]
        assert np.array_equal(got.view(np.uint32), same.view(np.uint32))


def _free_bytes(L):
    f, t = C.c_int64(), C.c_int64()
    assert L.gl_device_mem_info(0, C.byref(f), C.byref(t)) == 0
    return f.value


def test_static_scratch_product_allocates_no_device_memory(g):
    """After the first call on a device (which looks the array up and creates the private stream), a call
    must leave the device's free memory exactly as it found it; the allocating entry point is the control
    (its scratch is freed again, so it too ends where it started, but only this one never moves it)."""
    L = g.lib()
    rng = np.random.default_rng(7)
    M, N, K = 256, 256, 512
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((N, K)).astype(np.float32)
    dA, dB = _dev(L, A), _dev(L, B)
    dC = _dev(L, np.zeros((M, N), np.float32))
    assert L.gl_matmul_static(dA, K, 1, dB, K, 1, dC, N, M, N, K, 0) == 0, L.gl_matmul_static_error()
    before = _free_bytes(L)
    for _ in range(3):
        assert L.gl_matmul_static(dA, K, 1, dB, K, 1, dC, N, M, N, K, 0) == 0, L.gl_matmul_static_error()
        assert _free_bytes(L) == before
    for p in (dA, dB, dC):
        L.gl_device_free(p, 0)


def test_static_scratch_product_rejects_oversize_and_odd_shapes(g):
    L = g.lib()
    small = np.zeros((128, 32), np.float32)
    d = _dev(L, small)
    # an operand addressed beyond 2 Mi floats: refused before anything touches the GPU
    st = L.gl_matmul_static(d, 32768, 1, d, 32, 1, d, 128, 128, 128, 32768, 0)
    assert st == -8 and b"exceed the static scratch limit" in L.gl_matmul_static_error()
    st = L.gl_matmul_static(d, 32, 1, d, 32, 1, d, 100, 100, 100, 32, 0)
    assert st == -1
    L.gl_device_free(d, 0)

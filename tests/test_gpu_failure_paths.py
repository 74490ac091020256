"""GPU tests of the failure and control paths of the C ABI: a bounded device wait that runs out, the
stop flag raised from another host thread, the per-device launch set-up, and the index-offset form of
the synthetic generator.  Nothing here faults or hangs the GPU: the wait under test has a limit of a few
milliseconds, gives up by itself and leaves an error status that the host reads; the context stays usable.
"""
import ctypes as C
import threading
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _small_tc_net(g, rows=256, device=0):
    sizes = [128, 256, 128]
    rng = np.random.default_rng(5)
    x = rng.standard_normal((rows, sizes[0]), dtype=np.float32)
    y = np.zeros((rows, sizes[-1]), np.float32)
    y[np.arange(rows), rng.integers(0, sizes[-1], rows)] = 1.0
    w = rng.uniform(-0.1, 0.1, 128 * 256 + 256 * 128).astype(np.float32)
    d = g.make_desc(sizes, ["relu", "softmax"], "classification", batch=rows, lr=0.05, mode=g.MODE_BATCHED,
                    gemm=g.GEMM_TCGEN05, device=device)
    net = g.Net(d)
    net.set_weights(w, np.array([0.05], np.float32))
    net.set_data(x, y)
    return net, w


def test_bounded_wait_runs_out_and_reports_timeout(g):
    """A wait on a flag that nothing raises, limited to 4 M cycles (about 2 ms): it must return by itself,
    gl_sync must report GL_ERR_TIMEOUT, a second wait must return at once (the condition is sticky),
    gl_set_weights must clear it, and the handle must train normally afterwards."""
    net, w = _small_tc_net(g)
    m0 = net.train_window(0, 256)
    assert np.isfinite(m0.total_error)
    ms = net.selftest_bounded_wait(4_000_000)
    assert 0.2 <= ms <= 200.0, "the wait took %.3f ms" % ms
    with pytest.raises(g.GladesError) as ei:
        net.sync()
    assert ei.value.status == -6 and "bounded wait" in str(ei.value)
    # sticky: the next wait sees the status word and does not spin (limit 2e9 cycles = about a second)
    ms2 = net.selftest_bounded_wait(2_000_000_000)
    assert ms2 < 50.0, "a wait after a timeout spun for %.1f ms" % ms2
    # a window step still runs to completion but reports the condition
    with pytest.raises(g.GladesError) as ei:
        net.train_window(0, 256)
    assert ei.value.status == -6
    # cleared by gl_set_weights; the same step then gives the same loss as the very first one
    net.set_weights(w, np.array([0.05], np.float32))
    net.sync()
    m1 = net.train_window(0, 256)
    assert abs(m1.total_error - m0.total_error) <= 1e-6 * abs(m0.total_error)
    net.close()


def test_stop_from_a_second_thread_ends_training_between_epochs(g):
    """gl_stop is looked at between the epochs of gl_train_epochs (NNetwork::stop, network.cpp:99-102,173)."""
    net, _ = _small_tc_net(g, rows=1024)
    want = 20000
    t = threading.Timer(0.3, net.stop)
    t0 = time.perf_counter()
    t.start()
    m = net.train_epochs(want)   # ctypes releases the interpreter lock during the call
    dt = time.perf_counter() - t0
    t.join()
    assert 0 < net.epochs() < want, "stopped after %d of %d epochs (%.1f s)" % (net.epochs(), want, dt)
    assert m.epochs == net.epochs()
    # the flag is cleared by the next call
    e0 = net.epochs()
    net.train_epochs(2)
    assert net.epochs() == e0 + 2
    net.close()


def test_tensor_core_product_on_a_second_device(g):
    """The shared-memory opt-in and the SM count of the tensor-core kernel are per device: the first launch
    on device 1 in a process that already used device 0 must work."""
    if g.device_count() < 2:
        pytest.skip("needs two GPUs")
    L = g.lib()
    rng = np.random.default_rng(9)
    M, N, K = 256, 512, 160
    A = rng.standard_normal((M, K), dtype=np.float32)
    B = rng.standard_normal((N, K), dtype=np.float32)
    ref = A.astype(np.float64) @ B.astype(np.float64).T
    bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64).T
    for dev in (0, 1):
        ptrs = []
        for a in (A, B, np.zeros((M, N), np.float32)):
            p = C.c_void_p()
            assert L.gl_device_alloc(C.byref(p), a.nbytes, dev) == 0
            assert L.gl_memcpy_h2d(p, a.ctypes.data_as(C.c_void_p), a.nbytes, dev) == 0
            ptrs.append(p)
        out = np.empty((M, N), np.float32)
        for static in (False, True):
            if static:
                st = L.gl_matmul_static(ptrs[0], K, 1, ptrs[1], K, 1, ptrs[2], N, M, N, K, dev)
                assert st == 0, L.gl_matmul_static_error()
            else:
                st = L.gl_matmul(ptrs[0], K, 1, ptrs[1], K, 1, ptrs[2], N, M, N, K, g.GEMM_TCGEN05, dev)
                assert st == 0, L.gl_last_error()
            assert L.gl_memcpy_d2h(out.ctypes.data_as(C.c_void_p), ptrs[2], out.nbytes, dev) == 0
            assert float(np.max(np.abs(out - ref) / bound)) <= 4e-6
        for p in ptrs:
            L.gl_device_free(p, dev)


@pytest.mark.parametrize("dist", [0, 1])
def test_synth_fill_at_is_a_slice_of_the_stream(g, oracle, dist):
    """gl_synth_fill_at(first) must give elements [first, first+n) of the stream gl_synth_fill gives from 0,
    which in turn equals the CPU generator: shards filled by any number of ranks form one global table."""
    L = g.lib()
    n, first = 6000, 1234
    seed, stream = 0x474C4144 + 9, 0
    p = C.c_void_p()
    assert L.gl_device_alloc(C.byref(p), 4 * (n + first), 0) == 0
    whole = np.empty(n + first, np.float32)
    part = np.empty(n, np.float32)
    assert L.gl_synth_fill(p, n + first, seed, stream, dist, 2.0, 0.5, 0) == 0
    assert L.gl_memcpy_d2h(whole.ctypes.data_as(C.c_void_p), p, whole.nbytes, 0) == 0
    assert L.gl_synth_fill_at(p, n, first, seed, stream, dist, 2.0, 0.5, 0) == 0, L.gl_last_error()
    assert L.gl_memcpy_d2h(part.ctypes.data_as(C.c_void_p), p, part.nbytes, 0) == 0
    assert np.array_equal(part.view(np.uint32), whole[first:].view(np.uint32))
    cpu = oracle.synth_fill(n + first, seed, stream, dist, 2.0, 0.5)
    if dist == 0:
        assert np.array_equal(whole.view(np.uint32), cpu.view(np.uint32))
    else:
        assert np.max(np.abs(whole - cpu)) <= 1e-6 * max(1.0, float(np.max(np.abs(cpu))))
    # normal draws come in pairs: an odd first index is refused
    if dist == 1:
        assert L.gl_synth_fill_at(p, n, first + 1, seed, stream, dist, 2.0, 0.5, 0) == -1
    L.gl_device_free(p, 0)

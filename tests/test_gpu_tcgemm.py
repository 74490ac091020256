"""GPU tests of the tensor-core (TMA + tcgen05, 3xTF32) layer product, through the C ABI.

Tolerance: the 3xTF32 split keeps about 21 mantissa bits per operand and accumulates in fp32, so
each output must agree with a float64 product within 4e-6 * sum_k |a_mk||b_nk| (the fp32 tolerance
1e-5 of the task with margin; plain TF32 would be ~1e-3 and fail)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(L, a):
    p = C.c_void_p()
    assert L.gl_device_alloc(C.byref(p), a.nbytes + 64, 0) == 0
    assert L.gl_memcpy_h2d(p, a.ctypes.data_as(C.c_void_p), a.nbytes, 0) == 0
    return p


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (256, 256, 64), (128, 384, 96), (384, 256, 160), (256, 512, 1024),
                                   (128, 128, 48), (256, 256, 784)])
def test_tc_matmul_all_layouts(g, a_mn, b_mn, M, N, K):
    L = g.lib()
    rng = np.random.default_rng(M + 3 * N + 7 * K + a_mn + 2 * b_mn)
    A = rng.standard_normal((M, K)).astype(np.float32)   # logical A(m,k)
    B = rng.standard_normal((N, K)).astype(np.float32)   # logical B(n,k)
    A_mem = np.ascontiguousarray(A.T) if a_mn else A      # MN-major: stored [k][m]
    B_mem = np.ascontiguousarray(B.T) if b_mn else B
    a_sm, a_sk = (1, M) if a_mn else (K, 1)
    b_sn, b_sk = (1, N) if b_mn else (K, 1)
    dA, dB = _dev(L, A_mem), _dev(L, B_mem)
    out = np.zeros((M, N), np.float32)
    dC = _dev(L, out)
    ref = A.astype(np.float64) @ B.astype(np.float64).T
    bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64).T
    for engine in (g.GEMM_TCGEN05, g.GEMM_FFMA):
        st = L.gl_matmul(dA, a_sm, a_sk, dB, b_sn, b_sk, dC, N, M, N, K, engine, 0)
        assert st == 0, L.gl_last_error()
        assert L.gl_memcpy_d2h(out.ctypes.data_as(C.c_void_p), dC, out.nbytes, 0) == 0
        err = float(np.max(np.abs(out.astype(np.float64) - ref) / bound))
        assert err <= 4e-6, "engine %d: error %.3g of sum|a||b|" % (engine, err)
    for p in (dA, dB, dC):
        L.gl_device_free(p, 0)


def _matmul_case(g, M, N, K, a_mn, b_mn, seed, positive=False):
    """One gl_matmul on the tensor-core engine against the float64 product; returns the worst error in
    units of sum_k |a||b| and the change of the per-variant launch counters."""
    L = g.lib()
    rng = np.random.default_rng(seed)
    draw = (lambda s: rng.random(s, dtype=np.float32) + 0.25) if positive else \
        (lambda s: rng.standard_normal(s, dtype=np.float32))
    A = draw((M, K))
    B = draw((N, K))
    A_mem = np.ascontiguousarray(A.T) if a_mn else A
    B_mem = np.ascontiguousarray(B.T) if b_mn else B
    a_sm, a_sk = (1, M) if a_mn else (K, 1)
    b_sn, b_sk = (1, N) if b_mn else (K, 1)
    dA, dB = _dev(L, A_mem), _dev(L, B_mem)
    out = np.full((M, N), np.nan, np.float32)
    dC = _dev(L, out)
    before = g.tc_variant_counts()
    st = L.gl_matmul(dA, a_sm, a_sk, dB, b_sn, b_sk, dC, N, M, N, K, g.GEMM_TCGEN05, 0)
    assert st == 0, L.gl_last_error()
    after = g.tc_variant_counts()
    assert L.gl_memcpy_d2h(out.ctypes.data_as(C.c_void_p), dC, out.nbytes, 0) == 0
    for p in (dA, dB, dC):
        L.gl_device_free(p, 0)
    ref = A.astype(np.float64) @ B.astype(np.float64).T
    bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64).T
    err = float(np.max(np.abs(out.astype(np.float64) - ref) / bound))
    return err, [a - b for a, b in zip(after, before)]


# The variant the wide-MLP and inference steps run on: 256-wide tiles, persistent CTAs that walk several
# tiles each in bands of 16 row tiles, pipeline and accumulator barriers that keep counting across tiles,
# deep K.  (M, N, K, A MN-major, B MN-major, all-positive operands)
WIDE_CASES = [
    # 320 wide tiles on 148 CTAs, all four operand layouts, shallow K: the tile walk and the barrier
    # phases across tiles (2 to 3 tiles per CTA, a partial last band: 32 row tiles = 2 bands of 16)
    (4096, 2560, 256, 0, 0, False), (4096, 2560, 256, 0, 1, False), (4096, 2560, 256, 1, 1, False),
    (4096, 2560, 256, 1, 0, False),
    # row-tile count that is not a multiple of the band (24 = 16 + 8): the short last band
    (3072, 1536, 272, 0, 0, False),
    # the layer products of the wide-MLP window step at 2048 rows: forward (K-major x K-major), error
    # propagation (weights read MN-major), weight gradient (both operands MN-major, K = rows)
    (2048, 4096, 4096, 0, 0, False), (2048, 4096, 4096, 0, 1, False), (4096, 4096, 2048, 1, 1, False),
    # the first layer's gradient at the full 8192-row window: K = 8192, 128 wide tiles
    (4096, 1024, 8192, 1, 1, False),
    # all-positive operands: the worst case for the tensor core's truncating accumulation at deep K
    (2048, 2560, 4096, 0, 0, True),
    # one tile per CTA but 256 wide and deep: 80 wide tiles
    (2048, 1280, 4096, 0, 0, False),
]


@pytest.mark.parametrize("M,N,K,a_mn,b_mn,positive", WIDE_CASES)
def test_tc_matmul_wide_persistent_variant(g, M, N, K, a_mn, b_mn, positive):
    err, dc = _matmul_case(g, M, N, K, a_mn, b_mn, seed=M + 3 * N + 7 * K + a_mn + 2 * b_mn, positive=positive)
    assert err <= 4e-6, "error %.3g of sum|a||b|" % err
    tiles = (M // 128) * (N // 256)
    assert dc[1] == 1 and dc[0] == 0, "the 256-wide instantiation did not run: %r" % (dc,)
    assert len(dc) == 5
    if tiles > 148:
        assert dc[2] == 1, "%d tiles but no CTA walked more than one" % tiles


# Shapes whose last wave of tiles leaves SMs idle: the kernel deals the k-blocks of those tiles out over all CTAs, a CTA that holds the tail of a tile stores its partial accumulators and the CTA
# that holds the head adds the partials in a fixed order and runs the epilogue.  (M, N, K, A MN-major, B MN-major)
SPLIT_CASES = [
    (1024, 4096, 1024, 0, 0),   # 128 wide tiles on 148 SMs: every CTA gets 0.86 of a tile
    (1024, 4096, 1024, 1, 1),   # the same as a weight-gradient product
    (1024, 1024, 4096, 0, 0),   # 32 wide tiles, deep k: a tile is shared by four or five CTAs
    (1024, 1024, 4096, 0, 1),
    (4096, 4096, 1024, 1, 1),   # 512 tiles: three whole waves, then 68 tiles split
    (1024, 2048, 272, 0, 0),    # 64 wide tiles, 17 k-blocks each: shares that end inside a chunk of 8 k-blocks
    (1792, 1152, 784, 0, 0),    # 128-wide tiles (1152 is no multiple of 256): 126 tiles, 49 k-blocks
]


# By default only a last wave that leaves a quarter of the SMs idle is split; these cases lower the threshold to
# a tenth so that the geometries with 0.86 of a tile per CTA (most tiles shared by two CTAs) stay covered.
@pytest.mark.parametrize("M,N,K,a_mn,b_mn", SPLIT_CASES)
def test_tc_matmul_split_last_wave(g, monkeypatch, M, N, K, a_mn, b_mn):
    monkeypatch.setenv("GLADES_TC_SPLITK_IDLE", "10")
    err, dc = _matmul_case(g, M, N, K, a_mn, b_mn, seed=5 * M + 3 * N + K + a_mn + 2 * b_mn)
    assert err <= 4e-6, "error %.3g of sum|a||b|" % err
    assert dc[4] == 1, "the last wave was not split along k: %r" % (dc,)
    # all-positive operands: partial sums of one sign, the worst case for a lost or doubled partial
    err, dc = _matmul_case(g, M, N, K, a_mn, b_mn, seed=7, positive=True)
    assert err <= 4e-6 and dc[4] == 1


def test_tc_matmul_split_rule_default(g, monkeypatch):
    """Default rule: 128 tiles on 148 SMs (13 % idle) stay whole, 32 and 68-tile last waves are split."""
    monkeypatch.delenv("GLADES_TC_SPLITK_IDLE", raising=False)
    monkeypatch.delenv("GLADES_TC_SPLITK", raising=False)
    import torch
    if torch.cuda.get_device_properties(0).multi_processor_count != 148:
        pytest.skip("the tile counts of this test are chosen for 148 SMs")
    for (M, N, K), split in (((1024, 4096, 1024), 0), ((1024, 1024, 4096), 1), ((4096, 4096, 512), 1)):
        err, dc = _matmul_case(g, M, N, K, 0, 0, seed=11)
        assert err <= 4e-6
        assert dc[4] == split, "M=%d N=%d K=%d: split %d, expected %d" % (M, N, K, dc[4], split)


def test_tc_matmul_rejects_odd_shapes(g):
    L = g.lib()
    a = np.zeros((100, 32), np.float32)
    dA, dB, dC = _dev(L, a), _dev(L, a), _dev(L, np.zeros((100, 100), np.float32))
    assert L.gl_matmul(dA, 32, 1, dB, 32, 1, dC, 100, 100, 100, 32, g.GEMM_TCGEN05, 0) != 0
    assert L.gl_matmul(dA, 32, 1, dB, 32, 1, dC, 100, 100, 100, 32, g.GEMM_FFMA, 0) == 0
    for p in (dA, dB, dC):
        L.gl_device_free(p, 0)


@pytest.mark.parametrize("momentum,head", [(0.0, "softmax"), (0.9, "sigmoid")])
def test_batched_window_on_tensor_cores_vs_restatement(g, oracle, momentum, head):
    """A whole window step (forward, error propagation, weight gradient, update) with every layer
    product on the tcgen05 kernel, against the double-accumulating CPU restatement."""
    rng = np.random.default_rng(17)
    sizes = [128, 256, 384, 128]
    rows = 256
    out_type = "classification"
    d = g.make_desc(sizes, ["relu", "tanh", head], out_type, batch=rows, lr=0.05, momentum=momentum,
                    mode=g.MODE_BATCHED, gemm=g.GEMM_TCGEN05)
    x = rng.standard_normal((rows, sizes[0])).astype(np.float32)
    if head == "softmax":
        y = np.zeros((rows, sizes[-1]), np.float32)
        y[np.arange(rows), rng.integers(0, sizes[-1], rows)] = 1.0
    else:
        y = rng.uniform(0.05, 0.95, (rows, sizes[-1])).astype(np.float32)
    nw = sum(sizes[i] * sizes[i + 1] for i in range(3))
    w = (rng.standard_normal(nw) * 0.05).astype(np.float32)
    b = np.array([0.02, -0.03], np.float32)
    net = g.Net(d)
    net.set_weights(w, b)
    net.set_data(x, y)
    S = oracle.Restate(d, x, y, g.Metrics)
    S.set_weights(w, b)
    for step in range(2):
        m = net.train_window(0, rows)
        gr = S.window_grad(0, rows)
        S.window_apply(gr, rows)
        wg, bg = net.get_weights()
        ws, bs = S.get_weights()
        err = float(np.max(np.abs(wg.astype(np.float64) - ws)) / np.max(np.abs(ws)))
        assert err <= 1e-5, "step %d: weights rel err %g" % (step, err)
        assert np.allclose(bg, bs, rtol=1e-4, atol=1e-6)
        assert abs(m.total_error - gr[-2]) <= 1e-5 * max(1.0, abs(gr[-2]))
    # 3 forward + 2 error-propagation + 3 gradient products per step, all on tensor cores
    assert net.tensor_core_launches() == 16
    # inference from identical weights (the two sides' weights differ by the step tolerance above)
    wg, bg = net.get_weights()
    S.set_weights(wg, bg)
    out_g, am_g, _ = net.forward(0, rows)
    out_s, am_s = S.forward_block(0, rows)
    assert np.max(np.abs(out_g - out_s)) <= 1e-5 * max(1.0, float(np.max(np.abs(out_s))))
    assert np.array_equal(am_g, am_s)
    net.close()


def test_cta_pair_variant_in_a_subprocess():
    """The CTA-pair (cta_group::2) variant of the product is selected by an environment variable that
    is read once per process, so it is exercised by re-running the layout tests in a child process."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, GLADES_TC_PAIR="1")
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-x", "-q", "-m", "gpu", "-k",
                        "all_layouts and 256"], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-500:]


def _rows_clear_of_relu_threshold(rng, draw, x, W0, W1, b1, margin=1e-5):
    """The reference's ReLU is discontinuous: 0 below 0.046, the identity above (GMath/gmath.cpp:62-68).  A
    hidden pre-activation within fp32 rounding of 0.046 may fall on either side in two correct fp32
    evaluations, and the two then differ by far more than any rounding tolerance.  So that the comparisons
    below measure the kernels and not that coin toss, rows with a pre-activation of either hidden layer
    within `margin` of the threshold (float64 evaluation) are drawn again until none is left."""
    W0 = W0.astype(np.float64)
    W1 = W1.astype(np.float64)
    todo = np.arange(x.shape[0])
    for _ in range(100):
        z1 = x[todo].astype(np.float64) @ W0.T
        z2 = np.where(z1 < 0.046, 0.0, z1) @ W1.T + float(b1)
        bad = np.any(np.abs(z1 - 0.046) < margin, axis=1) | np.any(np.abs(z2 - 0.046) < margin, axis=1)
        todo = todo[bad]
        if todo.size == 0:
            return x
        x[todo] = draw(todo.size)
    raise AssertionError("could not clear the rows of the ReLU threshold")


def _onehot(rows, n, labels):
    y = np.zeros((rows, n), np.float32)
    y[np.arange(rows), labels] = 1.0
    return y


def test_wide_mlp_window_on_the_benchmarked_variant_vs_restatement(g, oracle):
    """One batched-mode window of the wide-MLP student itself (1024-4096-4096-1024, ReLU/ReLU/softmax,
    cross-entropy, lr 1e-2, weights U(+-1/sqrt(n_in))) on 1024 rows, against the double-accumulating CPU
    restatement: loss, every updated weight within 1e-5 of the largest weight, identical predicted
    classes.  At this size the layer products run on the 256-wide persistent tiles (the instantiation
    the benchmark measures), several tiles per CTA for the 4096 x 4096 gradient.  The rows are drawn so
    that no hidden pre-activation lies within 1e-5 of the discontinuity of the reference's ReLU."""
    sizes = [1024, 4096, 4096, 1024]
    rows = 1024
    rng = np.random.default_rng(404)
    x = rng.standard_normal((rows, sizes[0]), dtype=np.float32)
    y = _onehot(rows, sizes[-1], rng.integers(0, sizes[-1], rows))
    w = np.concatenate([rng.uniform(-1, 1, sizes[i] * sizes[i + 1]).astype(np.float32) / np.float32(np.sqrt(sizes[i]))
                        for i in range(3)])
    b = np.array([0.01, -0.02], np.float32)
    n01, n12 = sizes[0] * sizes[1], sizes[1] * sizes[2]
    x = _rows_clear_of_relu_threshold(rng, lambda k: rng.standard_normal((k, sizes[0]), dtype=np.float32), x,
                                      w[:n01].reshape(sizes[1], sizes[0]), w[n01:n01 + n12].reshape(sizes[2], sizes[1]), b[0])
    d = g.make_desc(sizes, ["relu", "relu", "softmax"], "classification", batch=rows, lr=1e-2, mode=g.MODE_BATCHED)
    net = g.Net(d)
    net.set_weights(w, b)
    net.set_data(x, y)
    S = oracle.Restate(d, x, y, g.Metrics)
    S.set_weights(w, b)
    before = g.tc_variant_counts()
    m = net.train_window(0, rows)
    dc = [a - c for a, c in zip(g.tc_variant_counts(), before)]
    assert dc[1] >= 6 and dc[2] >= 1, "expected the 256-wide persistent variant, saw %r" % (dc,)
    gr = S.window_grad(0, rows)
    S.window_apply(gr, rows)
    wg, bg = net.get_weights()
    ws, bs = S.get_weights()
    lo = 0
    for l in range(3):
        hi = lo + sizes[l] * sizes[l + 1]
        scale = float(np.max(np.abs(ws[lo:hi])))
        assert np.max(np.abs(wg[lo:hi].astype(np.float64) - ws[lo:hi])) <= 1e-5 * scale, "layer %d weights" % l
        # the update itself (new - old) carries the whole gradient: within 1e-3 of its largest entry plus the
        # rounding of the stored weight on both sides (the update is 1e-4 of the weight), 1e-4 on average
        ug = wg[lo:hi].astype(np.float64) - w[lo:hi]
        us = ws[lo:hi].astype(np.float64) - w[lo:hi]
        ulp = float(np.spacing(np.float32(scale)))
        assert np.max(np.abs(ug - us)) <= 1e-3 * np.max(np.abs(us)) + 2 * ulp, "layer %d update" % l
        assert np.mean(np.abs(ug - us)) <= 1e-4 * np.max(np.abs(us)) + ulp, "layer %d update, mean" % l
        lo = hi
    assert np.allclose(bg, bs, rtol=1e-4, atol=1e-7)
    assert abs(m.total_error - gr[-2]) <= 1e-5 * max(1.0, abs(gr[-2]))
    # predictions from identical weights: same classes for every row
    S.set_weights(wg, bg)
    out_g, am_g, _ = net.forward(0, rows)
    out_s, am_s = S.forward_block(0, rows)
    assert np.max(np.abs(out_g - out_s)) <= 1e-5 * max(1.0, float(np.max(np.abs(out_s))))
    assert np.array_equal(am_g, am_s)
    net.close()
    S.close()


def test_inference_net_forward_on_the_benchmarked_variant_vs_restatement(g, oracle):
    """Forward pass of the batched-inference net (784-2048-2048-10, ReLU/ReLU/softmax, weights
    U(-0.05, 0.05), rows U(0,1)) on 2048 rows against the restatement: probabilities within 1e-5 and the
    same predicted class for every row.  The two hidden products run on the 256-wide tiles.  Rows are drawn
    clear of the discontinuity of the reference's ReLU (see _rows_clear_of_relu_threshold)."""
    sizes = [784, 2048, 2048, 10]
    rows = 2048
    rng = np.random.default_rng(505)
    x = rng.random((rows, sizes[0]), dtype=np.float32)
    y = np.full((rows, sizes[-1]), 0.01, np.float32)
    nw = sum(sizes[i] * sizes[i + 1] for i in range(3))
    w = rng.uniform(-0.05, 0.05, nw).astype(np.float32)
    n01, n12 = sizes[0] * sizes[1], sizes[1] * sizes[2]
    x = _rows_clear_of_relu_threshold(rng, lambda k: rng.random((k, sizes[0]), dtype=np.float32), x,
                                      w[:n01].reshape(sizes[1], sizes[0]), w[n01:n01 + n12].reshape(sizes[2], sizes[1]), 0.01)
    d = g.make_desc(sizes, ["relu", "relu", "softmax"], "classification", batch=rows, lr=0.0, mode=g.MODE_BATCHED)
    net = g.Net(d)
    net.set_weights(w, np.array([0.01, 0.02], np.float32))
    net.set_data(x, y)
    S = oracle.Restate(d, x, y, g.Metrics)
    S.set_weights(w, np.array([0.01, 0.02], np.float32))
    before = g.tc_variant_counts()
    out_g, am_g, _ = net.forward(0, rows)
    dc = [a - c for a, c in zip(g.tc_variant_counts(), before)]
    assert dc[1] == 2, "the two hidden products should run on 256-wide tiles, saw %r" % (dc,)
    out_s, am_s = S.forward_block(0, rows)
    assert np.max(np.abs(out_g - out_s)) <= 1e-5
    diff = np.nonzero(am_g != am_s)[0]
    # a row may only differ where its two best classes tie within the tolerance
    for r in diff:
        top = np.sort(out_s[r])[-2:]
        assert top[1] - top[0] <= 2e-5, "row %d: classes differ with a margin of %g" % (r, top[1] - top[0])
    assert diff.size == 0 or diff.size <= 2
    net.close()
    S.close()

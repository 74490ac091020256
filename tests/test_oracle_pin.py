"""CPU tests: the C restatement against (a) the golden vectors produced by the compiled reference
and (b) the compiled reference itself, where it was built.  Bit-exact: the restatement keeps the
reference's fp32 operation order and uses the same libm."""
import glob
import os

import numpy as np
import pytest

from conftest import GOLDEN, bits, desc_from_meta, libc_srand, load_golden

TRAJ = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "traj_*.npz")))


def test_golden_present():
    assert len(TRAJ) >= 15 and sum(n.startswith("traj_dropout") for n in TRAJ) >= 5
    for n in ("kat_scalar", "cfg2_step", "cfg1_lr01_nonfinite", "fwd_cfg3_32_256_256_1",
              "fwd_cfg5_784_2048_2048_10", "fwd_cfg4_1024_4096_4096_1024"):
        assert os.path.exists(os.path.join(GOLDEN, n + ".npz"))


def test_scalar_known_answers(g, oracle):
    meta, z = load_golden("kat_scalar")
    L = oracle.restate_lib()
    zs = z["zs"]
    k = 0
    for a in range(8):
        for p in meta["squash_params"]:
            got = np.array([L.rs_squash(float(v), a, p) for v in zs], np.float32)
            assert np.array_equal(bits(got), bits(z["squash"][k])), (a, p)
            k += 1
    k = 0
    for a in range(8):
        for p in meta["der_params"]:
            got = np.array([L.rs_act_der(float(v), a, p) for v in zs], np.float32)
            assert np.array_equal(bits(got), bits(z["der"][k])), (a, p)
            k += 1
    with np.errstate(all="ignore"):
        for fx in range(3):
            for ie, e in enumerate(z["es"]):
                got = np.array([L.rs_cost(float(e), float(p), meta["data_size"], fx) for p in z["ps"]], np.float32)
                want = z["cost"][fx][ie]
                assert np.array_equal(bits(got), bits(want)) or np.array_equal(np.isnan(got), np.isnan(want))
                got = np.array([L.rs_cost_der(float(e), float(p), fx) for p in z["ps"]], np.float32)
                assert np.array_equal(bits(got), bits(z["cost_der"][fx][ie]))


@pytest.mark.parametrize("name", TRAJ)
def test_restatement_reproduces_golden_trajectory(g, oracle, name):
    meta, z = load_golden(name)
    d = desc_from_meta(g, meta)
    S = oracle.Restate(d, z["x"], z["y"], g.Metrics)
    S.set_weights(z["w0"], z["b0"])
    snaps = meta["snapshots"]
    k = 0
    if "srand" in meta:
        libc_srand(meta["srand"])  # dropout flags come from rand(), seeded once before the run
    for e in range(1, meta["epochs"] + 1):
        m, cm, out = S.epoch(0, True)
        if e in snaps:
            w, b = S.get_weights()
            assert np.array_equal(bits(w), bits(z["w"][k])), "weights, epoch %d" % e
            assert np.array_equal(bits(b), bits(z["b"][k])), "bias, epoch %d" % e
            assert np.array_equal(cm, z["confusion"][k])
            assert np.array_equal(bits(out), bits(z["outputs"][k]))
            got = np.array([m.total_error, m.total_accuracy, m.class_accuracy, m.class_precision, m.class_recall,
                            m.class_specificity, m.class_f1], np.float32)
            n = 7 if meta["out"] != "regression" else 2
            assert np.array_equal(bits(got[:n]), bits(z["metrics"][k][:n])), (got, z["metrics"][k])
            k += 1
    for q in range(meta["batch"]):
        assert np.array_equal(bits(S.pending_delta(q)), bits(z["pending"][q]))
    if "srand" in meta:
        # the test pass drops nodes too
        libc_srand(meta["srand"] + 1)
        m, cm, out = S.epoch(1, True)
        assert np.array_equal(bits(np.array([m.total_error, m.total_accuracy], np.float32)), bits(z["test_metrics"]))
        assert np.array_equal(cm, z["test_confusion"]) and np.array_equal(bits(out), bits(z["test_outputs"]))


def test_restatement_nonfinite_row(g, oracle):
    """Config 1 as written (lr 0.1): the reference's weights leave the finite range inside the first
    epoch; the restatement must do so on the same training step."""
    meta, z = load_golden("cfg1_lr01_nonfinite")
    d = desc_from_meta(g, meta)
    S = oracle.Restate(d, z["x"], z["y"], g.Metrics)
    S.set_weights(z["w0"], z["b0"])
    first_bad = -1
    for step in range(450):
        S.train_row(step % 150)
        w, b = S.get_weights()
        if not (np.isfinite(w).all() and np.isfinite(b).all()):
            first_bad = step
            break
        last = (w.copy(), b.copy())
    assert first_bad == meta["first_bad_step"]
    assert np.array_equal(bits(last[0]), bits(z["w_last_good"]))


def test_restatement_cfg2_step(g, oracle):
    meta, z = load_golden("cfg2_step")
    d = desc_from_meta(g, meta)
    idx = np.arange(1024)
    x = ((idx[:, None] >> np.arange(9, -1, -1)) & 1).astype(np.float32)
    y = (x.sum(1) % 2).astype(np.float32)[:, None]
    w0 = oracle.synth_fill(g.weight_count(d), meta["seed"], meta["stream"], 0, meta["scale"], meta["offset"])
    S = oracle.Restate(d, x, y, g.Metrics)
    S.set_weights(w0, None)
    k = 0
    for r in range(33):
        S.train_row(r)
        if r in meta["snapshot_rows"]:
            w, b = S.get_weights()
            assert np.array_equal(bits(w), bits(z["w_rows"][k]))
            assert np.array_equal(bits(b), bits(z["b_rows"][k]))
            k += 1
    S = oracle.Restate(d, x, y, g.Metrics)
    S.set_weights(w0, None)
    m, _, out = S.epoch(0, True)
    w, b = S.get_weights()
    assert np.array_equal(bits(w), bits(z["w_epoch1"]))
    assert np.array_equal(bits(out), bits(z["outputs_epoch1"]))
    assert np.array_equal(bits(np.array([m.total_error, m.total_accuracy], np.float32)), bits(z["metrics_epoch1"]))


@pytest.mark.parametrize("name", ["fwd_cfg3_32_256_256_1", "fwd_cfg5_784_2048_2048_10", "fwd_cfg4_1024_4096_4096_1024"])
def test_restatement_forward_wide(g, oracle, name):
    meta, z = load_golden(name)
    sizes = meta["sizes"]
    d = desc_from_meta(g, meta)
    w = oracle.synth_fill(g.weight_count(d), meta["seed"], meta["stream"], 0, meta["scale"], meta["offset"])
    b = np.array(meta["bias"], np.float32)
    x = z["x"]
    y = np.full((x.shape[0], sizes[-1]), 0.01, np.float32)
    S = oracle.Restate(d, x, y, g.Metrics)
    S.set_weights(w, b)
    for r in range(x.shape[0]):
        assert np.array_equal(bits(S.forward_row(r)), bits(z["acts"][r])), "row %d" % r
    # batched-arithmetic forward (double accumulation) of the same rows: tolerance, same argmax
    out, am = S.forward_block(0, x.shape[0])
    ref_out = z["acts"][:, -sizes[-1]:]
    assert np.allclose(out, ref_out, rtol=1e-5, atol=1e-6)


@pytest.mark.skipif(not os.path.exists(os.path.join(os.path.dirname(GOLDEN), "..", "oracle", "_ref",
                                                    "libglades_ref.so")), reason="compiled reference not built")
def test_restatement_vs_compiled_reference_live(g, oracle):
    """Where oracle/_ref exists: fresh seeded nets, reference vs restatement, bit for bit."""
    rng = np.random.default_rng(99)
    cases = [([3, 7, 2], ["tanh", "sigmoid"], "regression", 5, 0.4, 0.0),
             ([4, 6, 5, 3], ["relu", "sigmoid", "sigmoid"], "classification", 2, 0.0, 0.0),
             # dropout: both sides draw their flags from the C library's rand(), re-seeded before each side's epoch
             ([4, 6, 5, 3], ["tanh", "sigmoid", "sigmoid"], "classification", 3, 0.6, [0.25, 0.25, 0.5]),
             ([3, 7, 2], ["sigmoid", "sigmoid"], "regression", 1, 0.0, 0.33)]
    for sizes, acts, out, mb, mom, pdrop in cases:
        rows = 23
        d = g.make_desc(sizes, acts, out, batch=mb, lr=0.02, momentum=mom, p_dropout=pdrop)
        x = rng.uniform(-1, 1, (rows, sizes[0])).astype(np.float32)
        y = rng.uniform(0.05, 0.95, (rows, sizes[-1])).astype(np.float32)
        w = rng.uniform(-0.5, 0.5, g.weight_count(d)).astype(np.float32)
        b = rng.uniform(-0.1, 0.1, len(sizes) - 2).astype(np.float32)
        R = oracle.Reference(d, x, y, g.Metrics)
        S = oracle.Restate(d, x, y, g.Metrics)
        R.set_weights(w, b)
        S.set_weights(w, b)
        for ep in range(3):
            libc_srand(900 + ep)
            mr, cr, outr = R.epoch(0, True)
            libc_srand(900 + ep)
            ms, cs, outs = S.epoch(0, True)
        wr, br = R.get_weights()
        ws, bs = S.get_weights()
        assert np.array_equal(bits(wr), bits(ws)) and np.array_equal(bits(br), bits(bs))
        assert np.array_equal(cr, cs) and np.array_equal(bits(outr), bits(outs))
        assert mr.total_accuracy == ms.total_accuracy and mr.total_error == ms.total_error


def test_batched_restatement_matches_sharded_sum(g, oracle):
    """Batched mode: the gradient of a window is the sum of its shards' gradients (with global
    momentum positions), so two data-parallel ranks reproduce one rank."""
    rng = np.random.default_rng(5)
    sizes = [6, 9, 7, 3]
    rows = 32
    d = g.make_desc(sizes, ["tanh", "relu", "sigmoid"], "classification", batch=rows, lr=0.03, momentum=0.7,
                    mode=g.MODE_BATCHED)
    x = rng.standard_normal((rows, sizes[0])).astype(np.float32)
    y = rng.uniform(0.05, 0.95, (rows, sizes[-1])).astype(np.float32)
    w = rng.uniform(-0.4, 0.4, g.weight_count(d)).astype(np.float32)
    S = oracle.Restate(d, x, y, g.Metrics)
    S.set_weights(w, None)
    whole = S.window_grad(0, rows)
    a = S.window_grad(0, 20, global_rows=rows, first_pos=0)
    b = S.window_grad(20, 12, global_rows=rows, first_pos=20)
    assert np.allclose(a + b, whole, rtol=1e-12, atol=1e-14)


def test_restatement_standardize_vs_golden(oracle):
    """NumberInput::standardizeInputTable + OHE: the C restatement against tables standardised by the reference's
    own code -- categorical columns, int columns, both scalings, z-score, constant columns, the minimum that
    starts from zero.  Bit for bit."""
    meta, z = load_golden("standardize")
    assert len(meta["cases"]) >= 6
    for k, c in enumerate(meta["cases"]):
        x, y = oracle.standardize_table(z["raw%d" % k], c["types"], c["outputs"], c["flag"], z["x%d" % k].shape[1],
                                        z["y%d" % k].shape[1])
        assert np.array_equal(bits(x), bits(z["x%d" % k])), "case %d inputs" % k
        assert np.array_equal(bits(y), bits(z["y%d" % k])), "case %d expected" % k


def test_fast_cpu_port_matches_restatement(g, oracle):
    """The timed CPU baseline (oracle/fastport.c: blocked fp32 products) against the double-accumulating
    restatement on one window: momentum, decay, both heads, odd sizes that do not fill the register tiles."""
    rng = np.random.default_rng(31)
    cases = [([12, 20, 9, 4], ["tanh", "relu", "softmax"], "classification", 37, 0.6, 0.0, 0),
             ([33, 40, 17, 5], ["relu", "leaky", "sigmoid"], "regression", 50, 0.0, 0.001, 0),
             ([70, 130, 3], ["sigmoid", "sigmoid"], "classification", 300, 0.3, 0.0, 1)]
    for sizes, acts, out, rows, mom, wd, brule in cases:
        x = rng.standard_normal((rows, sizes[0])).astype(np.float32)
        if acts[-1] == "softmax":
            y = np.zeros((rows, sizes[-1]), np.float32)
            y[np.arange(rows), rng.integers(0, sizes[-1], rows)] = 1.0
        else:
            y = rng.uniform(0.1, 0.9, (rows, sizes[-1])).astype(np.float32)
        d = g.make_desc(sizes, acts, out, batch=rows, lr=0.005 if brule else 0.05, momentum=mom, wd1=wd, wd2=wd,
                        params=[0.05] * (len(sizes) - 1), mode=g.MODE_BATCHED, bias_rule=brule)
        w = rng.uniform(-0.3, 0.3, g.weight_count(d)).astype(np.float32)
        b = rng.uniform(-0.1, 0.1, len(sizes) - 2).astype(np.float32)
        A = oracle.Restate(d, x, y, g.Metrics)
        A.set_weights(w, b)
        gr = A.train_window(0, rows)
        B = oracle.Restate(d, x, y, g.Metrics)
        B.set_weights(w, b)
        cost = B.train_window_fast(0, rows)
        wa, ba = A.get_weights()
        wb, bb = B.get_weights()
        assert np.max(np.abs(wa - wb)) <= 1e-5 * np.max(np.abs(wa)), sizes
        assert np.allclose(ba, bb, rtol=1e-4, atol=1e-6) and abs(cost - gr[-2]) <= 1e-5 * max(1.0, abs(gr[-2]))

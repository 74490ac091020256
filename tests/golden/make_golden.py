"""Generates the golden fixtures in this directory from the COMPILED REFERENCE.

Run once, where a reference checkout exists (it cannot run on the GPU box):

    make -C oracle ref restate && python tests/golden/make_golden.py

Every array below is produced by the reference's own code (oracle/_ref/libglades_ref.so: the
unmodified Backend/Machine Learning sources behind oracle/ref_harness.cpp) on seeded synthetic
inputs; nothing is taken from the reference's data files.  Large weight sets are not stored: they
are regenerated from (seed, stream) by the counter-based uniform generator, which is exact on CPU
and GPU alike.
"""
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

import importlib.util  # noqa: E402

_spec = importlib.util.spec_from_file_location("capi", os.path.join(ROOT, "glades-ml_b200", "capi.py"))
capi = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(capi)
o = ge.import_oracle()

SEED = 0x474C4144  # "GLAD"

# `--only a,b,...` rewrites just the named fixtures (everything is still computed, in the same order, so
# the seeded inputs of the others do not move)
ONLY = None
for _i, _a in enumerate(sys.argv):
    if _a == "--only" and _i + 1 < len(sys.argv):
        ONLY = set(sys.argv[_i + 1].split(","))


def gaussian_classes(rng, rows, n_in, n_cls, interleaved=True):
    means = rng.uniform(-2, 2, (n_cls, n_in))
    cls = (np.arange(rows) % n_cls) if interleaved else (np.arange(rows) // (rows // n_cls))
    x = (means[cls] + 0.5 * rng.standard_normal((rows, n_in))).astype(np.float32)
    y = np.full((rows, n_cls), 0.01, np.float32)
    y[np.arange(rows), cls] = 0.99
    return x, y


def save(name, meta, **arrays):
    if ONLY is not None and name not in ONLY:
        print("kept %s" % name)
        return
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, meta=np.array(json.dumps(meta)), **arrays)
    print("wrote %s (%.1f KB)" % (name, os.path.getsize(path) / 1024.0))


def trajectory(name, sizes, acts, out, x, y, mb, lr, mom, epochs, snapshots, w_range, seed, params=None, wd1=0.0,
               wd2=0.0, p_dropout=0.0, srand=None):
    """`p_dropout` (per node layer) with `srand`: the C library's generator is seeded once before the run;
    the reference then draws its dropout flags from rand() row by row (State/layer.cpp:102-134)."""
    import ctypes
    libc = ctypes.CDLL(None)
    rng = np.random.default_rng(seed)
    d = capi.make_desc(sizes, acts, out, batch=mb, lr=lr, momentum=mom, wd1=wd1, wd2=wd2, params=params,
                       p_dropout=p_dropout)
    nw = capi.weight_count(d)
    w0 = rng.uniform(-w_range, w_range, nw).astype(np.float32)
    b0 = rng.uniform(-0.1, 0.1, len(sizes) - 2).astype(np.float32)
    R = o.Reference(d, x, y, capi.Metrics)
    R.set_weights(w0, b0)
    mets, cms, ws, bs, outs = [], [], [], [], []
    if srand is not None:
        libc.srand(srand)
    for e in range(1, epochs + 1):
        m, cm, outp = R.epoch(0, True)
        if e in snapshots:
            w, b = R.get_weights()
            mets.append([m.total_error, m.total_accuracy, m.class_accuracy, m.class_precision, m.class_recall,
                         m.class_specificity, m.class_f1])
            cms.append(cm)
            ws.append(w)
            bs.append(b)
            outs.append(outp)
    pend = np.stack([R.pending_delta(k) for k in range(mb)])
    extra = {}
    if srand is not None:
        # the test pass drops nodes too (SGDHelper draws the flags whatever the run type)
        libc.srand(srand + 1)
        mt, cmt, outt = R.epoch(1, True)
        extra = dict(test_metrics=np.array([mt.total_error, mt.total_accuracy], np.float32), test_confusion=cmt,
                     test_outputs=outt)
    # cross-check the public path: a second reference object trained with NNetwork::train()
    R2 = o.Reference(d, x, y, capi.Metrics)
    R2.set_weights(w0, b0)
    if srand is not None:
        libc.srand(srand)
    R2.train_public(epochs)
    w2, b2 = R2.get_weights()
    assert np.array_equal(w2.view(np.uint32), ws[-1].view(np.uint32)), "public train() differs from row-driven epochs"
    assert np.array_equal(b2.view(np.uint32), bs[-1].view(np.uint32))
    meta = dict(kind="trajectory", sizes=sizes, acts=acts, out=out, batch=mb, lr=lr, momentum=mom, wd1=wd1, wd2=wd2,
                params=params, epochs=epochs, snapshots=sorted(snapshots))
    if srand is not None:
        meta.update(p_dropout=p_dropout, srand=srand)
    save(name, meta, x=x, y=y, w0=w0, b0=b0, metrics=np.array(mets, np.float32), confusion=np.array(cms, np.int32),
         w=np.array(ws), b=np.array(bs), outputs=np.array(outs), pending=pend, **extra)


def init_fixture():
    """Weights the reference draws (Layer::initWeights, rand()-driven Ziggurat) after srand(seed)."""
    import ctypes
    libc = ctypes.CDLL(None)
    cases = [dict(sizes=[4, 5, 3], acts=["sigmoid", "sigmoid"], out="classification", seed=1),
             dict(sizes=[2, 2, 1], acts=["tanh", "tanh"], out="regression", seed=2),
             dict(sizes=[6, 7, 5, 2], acts=["tanh", "relu", "linear"], out="regression", seed=3),
             dict(sizes=[3, 4, 4, 2], acts=["relu", "tanh", "tanh"], out="regression", seed=4),
             dict(sizes=[10, 32, 32, 1], acts=["tanh", "tanh", "sigmoid"], out="regression", seed=5)]
    arrays = {}
    for k, c in enumerate(cases):
        d = capi.make_desc(c["sizes"], c["acts"], c["out"], batch=1, lr=0.01)
        x = np.zeros((1, c["sizes"][0]), np.float32)
        y = np.zeros((1, c["sizes"][-1]), np.float32)
        libc.srand(c["seed"])
        R = o.Reference(d, x, y, capi.Metrics)
        arrays["w%d" % k] = R.get_weights()[0]
    save("init_weights", dict(kind="init", cases=cases), **arrays)


def standardize_fixture():
    """NumberInput::standardizeInputTable + OHE, the reference's own code (DataObjects/NumberInput.cpp:43-285,
    GMath/OHE.cpp), on typed raw tables handed over through the shim's table registry.  Column types: 0 float
    cells, 1 string cells (category k is the text "s<k>"), 2 int cells."""
    import ctypes as C
    L = o.reference_lib()
    L.ref_number_input.restype = C.c_int64
    L.ref_number_input.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p]

    def run(vals, types, outs, flag):
        vals = np.ascontiguousarray(vals, np.float32)
        rows, cols = vals.shape
        t, oc = np.array(types, np.int32), np.array(outs, np.int32)
        nx, ny = C.c_int(), C.c_int()
        L.ref_number_input(vals.ctypes.data, rows, cols, t.ctypes.data, oc.ctypes.data, flag, None, C.byref(nx), None, C.byref(ny))
        x = np.zeros((rows, nx.value), np.float32)
        y = np.zeros((rows, ny.value), np.float32)
        L.ref_number_input(vals.ctypes.data, rows, cols, t.ctypes.data, oc.ctypes.data, flag, x.ctypes.data, C.byref(nx),
                           y.ctypes.data, C.byref(ny))
        return x, y

    rng = np.random.default_rng(61)
    arrays, cases = {}, []
    shapes = [(150, 5, [0, 0, 0, 0, 1], [0, 0, 0, 0, 1], 0),      # four measurements and a class name: the classic table shape
              (64, 4, [0, 0, 2, 0], [0, 0, 0, 1], 0),             # regression: [0, 1] scaling, an int column
              (64, 4, [0, 0, 2, 0], [0, 1, 0, 1], 1),             # z-score
              (40, 6, [1, 0, 1, 2, 0, 0], [0, 0, 1, 0, 1, 0], 0),  # categorical inputs and outputs mixed
              (33, 3, [0, 0, 0], [0, 0, 1], 0),                   # constant and all-positive columns (the zero-start rule)
              (400, 32, [0] * 32, [0] * 31 + [1], 0)]             # a wider table
    for k, (rows, cols, types, outs, flag) in enumerate(shapes):
        v = rng.uniform(-4, 6, (rows, cols)).astype(np.float32)
        for c in range(cols):
            if types[c] == 1:
                ids = rng.integers(0, 3 + c % 3, rows)
                seen = {}
                for i, t in enumerate(ids):   # category indices in order of first appearance
                    seen.setdefault(int(t), len(seen))
                    ids[i] = seen[int(t)]
                v[:, c] = ids
            elif types[c] == 2:
                v[:, c] = np.round(v[:, c])
        if k == 4:
            v[:, 0] = 2.5                      # constant: range (from 0) is 2.5, so it IS scaled
            v[:, 1] = np.abs(v[:, 1]) + 1.0    # all positive: the minimum stays 0
        if k == 1:
            v[:, 1] = 0.0                      # constant zero: range 0, copied unscaled into the input table
        x, y = run(v, types, outs, flag)
        arrays.update({"raw%d" % k: v, "x%d" % k: x, "y%d" % k: y})
        cases.append(dict(rows=rows, cols=cols, types=types, outputs=outs, flag=flag))
    save("standardize", dict(kind="standardize", cases=cases), **arrays)


def gui_fixture():
    """The live-view messages NNetwork::run sends through GNet::GServer::send when a server and a connection
    are attached (Networks/network.cpp:258-357), recorded by the shim, for runs of fewer than 10 epochs (every
    epoch sends).  The harness starts run() at epoch 1 (it must keep run() from rebuilding the network), so the
    epoch labels in the stream start at 2: `epoch_base` says so."""
    import ctypes as C
    L = o.reference_lib()
    L.ref_train_gui.restype = C.c_int64
    L.ref_train_gui.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int64]
    rng = np.random.default_rng(71)
    arrays, cases = {}, []
    nets = [dict(sizes=[3, 4, 2], acts=["tanh", "sigmoid"], out="classification", rows=12, batch=2, lr=0.05, momentum=0.3, epochs=5),
            dict(sizes=[5, 6, 4, 1], acts=["relu", "relu", "linear"], out="regression", rows=20, batch=4, lr=0.01, momentum=0.5,
                 epochs=4, params=[0.0, 0.0, 1.0])]
    for k, c in enumerate(nets):
        sizes = c["sizes"]
        x = rng.uniform(0, 1, (c["rows"], sizes[0])).astype(np.float32)
        if c["out"] == "classification":
            y = np.full((c["rows"], sizes[-1]), 0.01, np.float32)
            y[np.arange(c["rows"]), rng.integers(0, sizes[-1], c["rows"])] = 0.99
        else:
            y = rng.uniform(0.1, 0.9, (c["rows"], sizes[-1])).astype(np.float32)
        d = capi.make_desc(sizes, c["acts"], c["out"], batch=c["batch"], lr=c["lr"], momentum=c["momentum"], params=c.get("params"))
        w0 = rng.uniform(-0.5, 0.5, capi.weight_count(d)).astype(np.float32)
        b0 = rng.uniform(-0.1, 0.1, len(sizes) - 2).astype(np.float32)
        R = o.Reference(d, x, y, capi.Metrics)
        R.set_weights(w0, b0)
        n = L.ref_train_gui(R.h, c["epochs"], None, 0)
        R = o.Reference(d, x, y, capi.Metrics)
        R.set_weights(w0, b0)
        buf = np.zeros(n, np.float64)
        assert L.ref_train_gui(R.h, c["epochs"], buf.ctypes.data, n) == n
        w_end, b_end = R.get_weights()
        arrays.update({"x%d" % k: x, "y%d" % k: y, "w0_%d" % k: w0, "b0_%d" % k: b0, "stream%d" % k: buf, "w_end%d" % k: w_end})
        cases.append(dict(c, epoch_base=1))
    save("gui_stream", dict(kind="gui", cases=cases), **arrays)


def main():
    t0 = time.time()
    if "--only-init" in sys.argv:
        init_fixture()
        return
    L = o.reference_lib()
    init_fixture()

    # ---- A. scalar known answers of GMath (gmath.cpp:22-101,182-353)
    zs = np.concatenate([np.linspace(-12, 12, 193), [0.0, 0.046, 0.0459, 0.0461, 1e-8, -1e-8, 88.0, -88.0, 0.9, 0.1]]
                        ).astype(np.float32)
    squash = np.array([[L.ref_squash(float(z), a, p) for z in zs] for a in range(8) for p in (0.0, 0.1, 1.0)],
                      np.float32)
    der = np.array([[L.ref_act_der(float(z), a, p) for z in zs] for a in range(8) for p in (0.01, -0.02)], np.float32)
    ps = np.linspace(0.001, 0.999, 97).astype(np.float32)
    es = np.array([0.01, 0.99, 0.0, 1.0, 0.5], np.float32)
    with np.errstate(all="ignore"):
        cost = np.array([[[L.ref_cost(float(e), float(p), 450.0, fx) for p in ps] for e in es] for fx in range(3)],
                        np.float32)
        cder = np.array([[[L.ref_cost_der(float(e), float(p), fx) for p in ps] for e in es] for fx in range(3)],
                        np.float32)
    save("kat_scalar", dict(kind="scalar", squash_params=[0.0, 0.1, 1.0], der_params=[0.01, -0.02], data_size=450.0),
         zs=zs, squash=squash, der=der, ps=ps, es=es, cost=cost, cost_der=cder)

    # ---- B. trajectories
    rng = np.random.default_rng(11)
    # the reference's own toy shape: 2-2-1 tanh regression, lr 0.003, online
    xx = np.array([[0, 0], [0, 1], [1, 0], [1, 1]], np.float32)
    xy = np.array([[0], [1], [1], [0]], np.float32)
    trajectory("traj_xor_2_2_1", [2, 2, 1], ["tanh", "tanh"], "regression", xx, xy, 1, 0.003, 0.0, 100, {1, 10, 100},
               0.5, 21)
    x, y = gaussian_classes(rng, 150, 4, 3)
    trajectory("traj_cls_4_5_3", [4, 5, 3], ["sigmoid", "sigmoid"], "classification", x, y, 1, 0.01, 0.0, 20,
               {1, 5, 20}, 0.5, 22)
    # config 1 at the only learning rate where the reference stays finite (0.01, interleaved rows)
    x1, y1 = gaussian_classes(rng, 150, 4, 3)
    trajectory("traj_cfg1_lr001", [4, 16, 3], ["sigmoid", "sigmoid"], "classification", x1, y1, 1, 0.01, 0.9, 200,
               {1, 2, 5, 20, 200}, 0.5, 23)
    trajectory("traj_cfg1_mb4", [4, 16, 3], ["sigmoid", "sigmoid"], "classification", x1, y1, 4, 0.01, 0.9, 7,
               {1, 2, 7}, 0.5, 24)
    xr = rng.uniform(0, 1, (64, 10)).astype(np.float32)
    yr = rng.uniform(0, 1, (64, 1)).astype(np.float32)
    trajectory("traj_reg_10_8_8_1_mb32", [10, 8, 8, 1], ["tanh", "tanh", "sigmoid"], "regression", xr, yr, 32, 0.05,
               0.9, 5, {1, 5}, 0.5, 25)
    xr = rng.uniform(-1, 1, (100, 6)).astype(np.float32)
    yr = rng.uniform(0, 1, (100, 2)).astype(np.float32)
    trajectory("traj_relu_6_5_4_2_mb7", [6, 5, 4, 2], ["relu", "relu", "linear"], "regression", xr, yr, 7, 0.01, 0.5,
               3, {1, 3}, 0.5, 26, params=[0.0, 0.0, 1.0], wd1=0.001, wd2=[0.001, 0.002, 0.003])
    xc, yc = gaussian_classes(rng, 40, 5, 3)
    trajectory("traj_cls_5_6_7_3_mb3", [5, 6, 7, 3], ["tanh", "sigmoid", "sigmoid"], "classification", xc, yc, 3,
               0.01, 0.3, 4, {1, 4}, 0.5, 27)
    xm = rng.uniform(-1, 1, (20, 3)).astype(np.float32)
    ym = rng.uniform(0, 1, (20, 2)).astype(np.float32)
    trajectory("traj_mixed_acts_mb5", [3, 4, 4, 4, 2], ["leaky", "tanhp", "sigmoidp", "linear"], "regression", xm, ym,
               5, 0.01, 0.2, 3, {1, 3}, 0.5, 28, params=[0.05, 0.1, 0.1, 0.7])

    # the KL cost (GMath/gmath.cpp:283,310-313,343) and the STEP activation (gmath.cpp:90-99), each through
    # whole training runs; own generators, so the fixtures above keep their inputs
    rk = np.random.default_rng(41)
    xk, yk = gaussian_classes(rk, 60, 4, 3)
    trajectory("traj_kl_4_6_3_mb2", [4, 6, 3], ["tanh", "sigmoid"], "kl", xk, yk, 2, 0.01, 0.4, 4, {1, 4}, 0.5, 29)
    xs = rk.uniform(-1, 1, (48, 5)).astype(np.float32)
    ys = rk.uniform(0.1, 0.9, (48, 2)).astype(np.float32)
    trajectory("traj_step_5_6_4_2_mb3", [5, 6, 4, 2], ["step", "tanh", "sigmoid"], "regression", xs, ys, 3, 0.02, 0.3,
               3, {1, 3}, 0.5, 30, params=[0.5, 0.0, 0.0])
    # dropout: online and minibatch, one and two hidden layers, momentum (per-edge histories of unequal
    # length), a layer that draws but never drops (p = 0) and one that draws nothing (p = 1)
    xd, yd = gaussian_classes(rk, 45, 4, 3)
    trajectory("traj_dropout_4_5_3_mb1", [4, 5, 3], ["sigmoid", "sigmoid"], "classification", xd, yd, 1, 0.01, 0.0, 5,
               {1, 5}, 0.5, 31, p_dropout=0.2, srand=101)
    xd2 = rk.uniform(0, 1, (50, 6)).astype(np.float32)
    yd2 = rk.uniform(0.1, 0.9, (50, 2)).astype(np.float32)
    trajectory("traj_dropout_6_8_7_2_mb4", [6, 8, 7, 2], ["tanh", "sigmoid", "sigmoid"], "regression", xd2, yd2, 4,
               0.01, 0.5, 4, {1, 2, 4}, 0.4, 32, p_dropout=[0.3, 0.3, 0.25], srand=102)
    trajectory("traj_dropout_6_8_7_2_mb7", [6, 8, 7, 2], ["relu", "tanh", "linear"], "regression", xd2[:45], yd2[:45],
               7, 0.001, 0.7, 3, {1, 3}, 0.4, 33, params=[0.0, 0.0, 1.0], p_dropout=[0.0, 0.0, 0.4], srand=103)
    xd3, yd3 = gaussian_classes(rk, 20, 5, 3)
    trajectory("traj_dropout_5_6_3_mb3", [5, 6, 3], ["tanh", "sigmoid"], "classification", xd3, yd3, 3, 0.01, 0.3, 4,
               {1, 4}, 0.5, 34, p_dropout=[1.0, 1.0], srand=104)
    trajectory("traj_dropout_5_6_3_half", [5, 6, 3], ["tanh", "sigmoid"], "classification", xd3, yd3, 3, 0.01, 0.3, 4,
               {1, 4}, 0.5, 35, p_dropout=0.5, srand=105)

    # ---- D. the step in front of the loop and the step behind it
    standardize_fixture()
    gui_fixture()

    # ---- config 1 as written (lr 0.1): the reference goes non-finite; record the first such row
    d = capi.make_desc([4, 16, 3], ["sigmoid", "sigmoid"], "classification", batch=1, lr=0.1, momentum=0.9)
    rngw = np.random.default_rng(23)
    w0 = rngw.uniform(-0.5, 0.5, 112).astype(np.float32)
    b0 = rngw.uniform(-0.1, 0.1, 1).astype(np.float32)
    R = o.Reference(d, x1, y1, capi.Metrics)
    R.set_weights(w0, b0)
    first_bad, last_good = -1, None
    for step in range(150 * 3):
        R.train_row(step % 150)
        w, b = R.get_weights()
        if not (np.isfinite(w).all() and np.isfinite(b).all()):
            first_bad = step
            break
        last_good = (w.copy(), b.copy())
    save("cfg1_lr01_nonfinite", dict(kind="nonfinite", sizes=[4, 16, 3], acts=["sigmoid", "sigmoid"],
                                     out="classification", batch=1, lr=0.1, momentum=0.9, first_bad_step=first_bad),
         x=x1, y=y1, w0=w0, b0=b0, w_last_good=last_good[0] if last_good else w0,
         b_last_good=last_good[1] if last_good else b0)
    print("cfg1 lr 0.1: first non-finite after training step", first_bad)

    # ---- config 2, step level: rows 0..32 (windows {0} and {1..32}) from identical state, then the
    # whole first epoch's metrics.  All 2^10 binary vectors in counting order, target = parity.
    idx = np.arange(1024)
    x2 = ((idx[:, None] >> np.arange(9, -1, -1)) & 1).astype(np.float32)
    y2 = (x2.sum(1) % 2).astype(np.float32)[:, None]
    d2 = capi.make_desc([10, 32, 32, 1], ["tanh", "tanh", "sigmoid"], "regression", batch=32, lr=0.05, momentum=0.0)
    w0 = o.synth_fill(capi.weight_count(d2), SEED + 2, 2, 0, 2.0, -1.0)
    R = o.Reference(d2, x2, y2, capi.Metrics)
    R.set_weights(w0, None)
    snaps_w, snaps_b = [], []
    for r in range(33):
        R.train_row(r)
        if r in (0, 16, 32):
            w, b = R.get_weights()
            snaps_w.append(w)
            snaps_b.append(b)
    pend16 = None
    R = o.Reference(d2, x2, y2, capi.Metrics)
    R.set_weights(w0, None)
    m, _, outp = R.epoch(0, True)
    w_e1, b_e1 = R.get_weights()
    save("cfg2_step", dict(kind="cfg2", sizes=[10, 32, 32, 1], acts=["tanh", "tanh", "sigmoid"], out="regression",
                           batch=32, lr=0.05, momentum=0.0, seed=SEED + 2, stream=2, scale=2.0, offset=-1.0,
                           snapshot_rows=[0, 16, 32]),
         w_rows=np.array(snaps_w), b_rows=np.array(snaps_b), w_epoch1=w_e1, b_epoch1=b_e1,
         metrics_epoch1=np.array([m.total_error, m.total_accuracy], np.float32), outputs_epoch1=outp)

    # ---- C. forward-only parity on the wide shapes (sampled rows; weights from seed)
    def forward_case(name, sizes, acts_native, n_rows, a_range, cfg, x_gen, params=None):
        d = capi.make_desc(sizes, acts_native, "classification" if sizes[-1] > 1 else "regression", batch=1, lr=0.0,
                           params=params)
        nw = capi.weight_count(d)
        w = o.synth_fill(nw, SEED + cfg, 2, 0, 2.0 * a_range, -a_range)
        b = np.array([0.01 * (l + 1) for l in range(len(sizes) - 2)], np.float32)
        x = x_gen(n_rows, sizes[0])
        y = np.full((n_rows, sizes[-1]), 0.01, np.float32)
        t = time.time()
        R = o.Reference(d, x, y, capi.Metrics)
        R.set_weights(w, b)
        acts = np.stack([R.forward_row(r) for r in range(n_rows)])
        R.close()
        # the same net with a LINEAR (param 1.0) last layer exposes the last pre-activation z
        acts_lin = list(acts_native[:-1]) + ["linear"]
        p_lin = list(params) if params else [0.0] * (len(sizes) - 1)
        p_lin[-1] = 1.0
        dl = capi.make_desc(sizes, acts_lin, "regression", batch=1, lr=0.0, params=p_lin)
        R = o.Reference(dl, x, y, capi.Metrics)
        R.set_weights(w, b)
        z_last = np.stack([R.forward_row(r)[-sizes[-1]:] for r in range(n_rows)])
        R.close()
        print("  %s: %d rows in %.1fs" % (name, n_rows, time.time() - t))
        save(name, dict(kind="forward", sizes=sizes, acts=acts_native, params=params, seed=SEED + cfg, stream=2,
                        scale=2.0 * a_range, offset=-a_range, bias=[float(v) for v in b]),
             x=x, acts=acts, z_last=z_last)

    rngx = np.random.default_rng(33)

    def walk_windows(n, k):
        steps = rngx.standard_normal(n + k + 1)
        walk = np.cumsum(steps)
        wins = np.stack([walk[i:i + k] for i in range(n)])
        mu = wins.mean(1, keepdims=True)
        sd = wins.std(1, keepdims=True)
        return ((wins - mu) / sd).astype(np.float32)

    forward_case("fwd_cfg3_32_256_256_1", [32, 256, 256, 1], ["relu", "relu", "linear"], 8, 1.0 / np.sqrt(32.0), 3,
                 walk_windows, params=[0.0, 0.0, 1.0])
    forward_case("fwd_cfg5_784_2048_2048_10", [784, 2048, 2048, 10], ["relu", "relu", "sigmoid"], 8, 0.05, 5,
                 lambda n, k: rngx.uniform(0, 1, (n, k)).astype(np.float32))
    if os.environ.get("GOLDEN_SKIP_CFG4") != "1":
        forward_case("fwd_cfg4_1024_4096_4096_1024", [1024, 4096, 4096, 1024], ["relu", "relu", "sigmoid"], 8,
                     1.0 / 32.0, 4, lambda n, k: rngx.standard_normal((n, k)).astype(np.float32))
    print("done in %.1fs" % (time.time() - t0))


if __name__ == "__main__":
    main()

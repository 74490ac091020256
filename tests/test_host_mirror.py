"""The C++ host mirror of the reference's interface (glades-ml_b200/host): host-only logic on CPU,
the weight draw against the compiled reference, and -- on a GPU -- whole training runs through
NNetwork::train / test against the golden vectors."""
import ctypes
import json
import os
import subprocess

import numpy as np
import pytest

from conftest import GOLDEN, bits, load_golden
from host_case import HOST_TOOL, read_run, run_tool, write_case

INIT_CASES = [
    # sizes, acts, out: the restart rule of the weight builder depends on activations and output type
    ([4, 5, 3], ["sigmoid", "sigmoid"], "classification"),
    ([2, 2, 1], ["tanh", "tanh"], "regression"),
    ([6, 7, 5, 2], ["tanh", "relu", "linear"], "regression"),
    ([3, 4, 4, 2], ["relu", "tanh", "tanh"], "regression"),
]


def _have_tool():
    return os.path.exists(HOST_TOOL)


@pytest.mark.skipif(not _have_tool(), reason="host_tool not built")
def test_host_unit_checks():
    r = subprocess.run([HOST_TOOL, "unit"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip().endswith("OK"), r.stdout + r.stderr


@pytest.mark.skipif(not _have_tool(), reason="host_tool not built")
def test_weight_draw_matches_golden(tmp_path):
    """Layer::initWeights restated on the host: same rand() consumption, same weights."""
    meta, z = load_golden("init_weights")
    for k, c in enumerate(meta["cases"]):
        case, out = str(tmp_path / "c.bin"), str(tmp_path / "o.bin")
        x = np.zeros((1, c["sizes"][0]), np.float32)
        y = np.zeros((1, c["sizes"][-1]), np.float32)
        write_case(case, c["sizes"], c["acts"], c["out"], 1, 0.01, 0.0, x, y, 1, seed=c["seed"])
        r = run_tool("init", case, out)
        assert r.returncode == 0, r.stderr
        w = np.fromfile(out, np.float32)
        assert np.array_equal(bits(w), bits(z["w%d" % k])), c


def test_weight_draw_matches_compiled_reference_live(g, oracle, tmp_path):
    if not (oracle.have_reference() and _have_tool()):
        pytest.skip("compiled reference or host_tool not built")
    libc = ctypes.CDLL(None)
    for seed, (sizes, acts, out) in enumerate(INIT_CASES, start=11):
        d = g.make_desc(sizes, acts, out, batch=1, lr=0.01)
        x = np.zeros((1, sizes[0]), np.float32)
        y = np.zeros((1, sizes[-1]), np.float32)
        libc.srand(seed)
        R = oracle.Reference(d, x, y, g.Metrics)
        wr, _ = R.get_weights()
        case, o = str(tmp_path / "c.bin"), str(tmp_path / "o.bin")
        write_case(case, sizes, acts, out, 1, 0.01, 0.0, x, y, 1, seed=seed)
        assert run_tool("init", case, o).returncode == 0
        assert np.array_equal(bits(np.fromfile(o, np.float32)), bits(wr)), (sizes, acts)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["traj_cfg1_mb4", "traj_relu_6_5_4_2_mb7", "traj_xor_2_2_1", "traj_cls_5_6_7_3_mb3"])
def test_host_network_train_vs_golden(name, tmp_path):
    assert _have_tool(), "host_tool must be built by __graft_entry__.build()"
    meta, z = load_golden(name)
    case, out = str(tmp_path / "c.bin"), str(tmp_path / "o.bin")
    write_case(case, meta["sizes"], meta["acts"], meta["out"], meta["batch"], meta["lr"], meta["momentum"], z["x"],
               z["y"], meta["epochs"], wd1=meta["wd1"], wd2=meta["wd2"], params=meta["params"], w=z["w0"], b=z["b0"])
    r = run_tool("run", case, out)
    assert r.returncode == 0, r.stdout + r.stderr
    res = read_run(out)
    assert res["epochs"] == meta["epochs"]
    ref_w, ref_b = z["w"][-1], z["b"][-1]
    if name == "traj_relu_6_5_4_2_mb7":
        assert np.array_equal(bits(res["w"]), bits(ref_w)) and np.array_equal(bits(res["b"]), bits(ref_b))
    else:
        assert np.max(np.abs(res["w"] - ref_w)) <= 1e-5 * np.max(np.abs(ref_w))
    assert abs(res["accuracy"] - z["metrics"][-1][1]) <= 1e-3
    # getResults(): (expected, predicted) pairs of the last row, predictions from before its update
    n_out = meta["sizes"][-1]
    assert res["results"].size == 2 * n_out
    assert np.array_equal(res["results"][0::2], z["y"][-1])
    assert np.max(np.abs(res["results"][1::2] - z["outputs"][-1][-1])) <= 1e-5
    if meta["out"] != "regression":
        assert np.array_equal(res["confusion"].reshape(n_out, n_out), z["confusion"][-1])


@pytest.mark.gpu
def test_host_network_draws_its_own_weights_and_tests(tmp_path):
    """Without injected weights the network draws them like the reference (seeded rand()), and
    NNetwork::test() is one forward pass that counts as an epoch and leaves the weights alone."""
    meta, z = load_golden("traj_cls_4_5_3")
    case, out = str(tmp_path / "c.bin"), str(tmp_path / "o.bin")
    write_case(case, meta["sizes"], meta["acts"], meta["out"], 1, 0.01, 0.0, z["x"], z["y"], 1, run_type=1, seed=5)
    assert run_tool("run", case, out).returncode == 0
    res = read_run(out)
    write_case(case, meta["sizes"], meta["acts"], meta["out"], 1, 0.01, 0.0, z["x"], z["y"], 1, seed=5)
    o2 = str(tmp_path / "i.bin")
    assert run_tool("init", case, o2).returncode == 0
    assert np.array_equal(bits(res["w"]), bits(np.fromfile(o2, np.float32)))
    assert res["epochs"] == 1 and 0.0 < res["accuracy"] < 100.0


def _read_gui(path):
    with open(path, "rb") as f:
        d = f.read()
    n = int(np.frombuffer(d, "<i4", 1, 0)[0])
    stream = np.frombuffer(d, "<f8", n, 4).copy()
    nc = int(np.frombuffer(d, "<i4", 1, 4 + 8 * n)[0])
    curve = np.frombuffer(d, "<f4", nc, 8 + 8 * n).copy()
    return stream, curve


def _messages(stream):
    out, i = [], 0
    while i < len(stream):
        kind, na = int(stream[i]), int(stream[i + 1])
        args = stream[i + 2:i + 2 + na]
        i += 2 + na
        rows, cols, ln = int(stream[i]), int(stream[i + 1]), int(stream[i + 2])
        i += 3
        out.append((kind, args, rows, cols, stream[i:i + ln]))
        i += ln
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("k", [0, 1])
def test_live_view_messages_vs_reference_golden(k, tmp_path):
    """Training with a server and a connection attached sends the reference's GUI_Callback stream
    (Networks/network.cpp:258-357): PROGRESSIVE, ACTIVATIONS (layer sizes first, then the last row's
    pre-activations), WEIGHTS, ACC and, for classifiers, CONF with the false-alarm and recall figures -- one
    frame per epoch below 10 epochs.  Compared message by message with the stream the reference's own code sent
    through the recording shim; the weights and pre-activations come from the asynchronous snapshot."""
    assert _have_tool()
    meta, z = load_golden("gui_stream")
    c = meta["cases"][k]
    case, out = str(tmp_path / "c.bin"), str(tmp_path / "o.bin")
    write_case(case, c["sizes"], c["acts"], c["out"], c["batch"], c["lr"], c["momentum"], z["x%d" % k], z["y%d" % k],
               c["epochs"] - 1, params=c.get("params"), w=z["w0_%d" % k],
               b=z["b0_%d" % k])
    r = run_tool("gui", case, out)
    assert r.returncode == 0, r.stdout + r.stderr
    stream, curve = _read_gui(out)
    got, want = _messages(stream), _messages(z["stream%d" % k])
    assert len(got) == len(want) and [m[0] for m in got] == [m[0] for m in want]
    base = c["epoch_base"]   # the reference's run was started at this epoch count by the harness
    exact = k == 1           # ReLU / linear: no transcendental function, bit for bit
    points = []
    for (kind, args, rows, cols, pay), (_, wargs, wrows, wcols, wpay) in zip(got, want):
        assert (rows, cols, len(pay)) == (wrows, wcols, len(wpay)) and len(args) == len(wargs)
        pay, wpay = pay.copy(), wpay.copy()
        if kind in (0, 3):   # PROGRESSIVE (epoch - 1, error), ACC (epoch, accuracy): epoch labels shifted by the base
            assert pay[0] + base == wpay[0]
            pay[0] = wpay[0]
            if kind == 0:
                points.extend([wpay[0] - base, pay[1]])
        sep = wpay >= 1e9    # the ',' and ';' separators sit at the same places
        assert np.array_equal(pay >= 1e9, sep) and np.array_equal(pay[sep], wpay[sep])
        if exact:
            assert np.array_equal(pay.astype(np.float32).view(np.uint32), wpay.astype(np.float32).view(np.uint32)), kind
            assert np.array_equal(args.astype(np.float32), wargs.astype(np.float32))
        else:
            scale = max(1.0, float(np.max(np.abs(wpay[~sep])))) if (~sep).any() else 1.0
            assert np.max(np.abs(pay[~sep] - wpay[~sep])) <= 1e-5 * scale, kind
            assert np.allclose(args, wargs, rtol=1e-5, atol=1e-6, equal_nan=True)
    # the learning curve holds the PROGRESSIVE points of the run
    assert np.allclose(curve, np.array(points, np.float32), rtol=0, atol=0)


@pytest.mark.gpu
def test_meta_network_replicas_match_a_single_run(tmp_path):
    """MetaNetwork::trainReplicas: k copies of one network, same injected weights, trained side by side (one per
    GPU, round robin).  Training is deterministic, so every replica must end with the weights of a single run."""
    assert _have_tool()
    meta, z = load_golden("traj_cls_5_6_7_3_mb3")
    case, out = str(tmp_path / "c.bin"), str(tmp_path / "o.bin")
    write_case(case, meta["sizes"], meta["acts"], meta["out"], meta["batch"], meta["lr"], meta["momentum"], z["x"], z["y"],
               meta["epochs"], wd1=meta["wd1"], wd2=meta["wd2"], params=meta["params"], w=z["w0"], b=z["b0"])
    assert run_tool("run", case, out).returncode == 0
    single = read_run(out)
    r = subprocess.run([HOST_TOOL, "replicas", case, out, "3"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    with open(out, "rb") as f:
        d = f.read()
    gpus, k = np.frombuffer(d, "<i4", 2, 0)
    assert k == 3 and 1 <= gpus <= 3
    off = 8
    for i in range(3):
        epochs, nw = np.frombuffer(d, "<i4", 2, off)
        w = np.frombuffer(d, "<f4", nw, off + 8)
        off += 8 + 4 * nw
        assert epochs == meta["epochs"]
        assert np.array_equal(bits(w), bits(single["w"])), "replica %d" % i

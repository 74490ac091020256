"""GPU tests of the input standardisation (gl_standardize_table and the host-side NumberInput on top of it):
the step in front of the training loop, NumberInput::standardizeInputTable with the one-hot vectors of OHE
(DataObjects/NumberInput.cpp:43-285, GMath/OHE.cpp:159-198).  Results are compared bit for bit -- the kernels use
the reference's fp32 operations in the reference's order -- with tables standardised by the reference's own code
(golden fixture), with the CPU restatement on larger tables, and through properties at the size of the window
regressor's data set."""
import ctypes as C
import struct

import numpy as np
import pytest

from conftest import bits, load_golden
from host_case import HOST_TOOL, run_tool

pytestmark = pytest.mark.gpu


def _standardize(g, oracle, raw, types, outputs, flag):
    L = g.lib()
    raw = np.ascontiguousarray(raw, np.float32)
    rows, cols = raw.shape
    kind, classes = oracle.standardize_plan(raw, types)
    outs = np.array(outputs, np.int32)
    d_raw = C.c_void_p()
    assert L.gl_device_alloc(C.byref(d_raw), raw.nbytes, 0) == 0
    assert L.gl_memcpy_h2d(d_raw, raw.ctypes.data_as(C.c_void_p), raw.nbytes, 0) == 0
    nx, ny = C.c_int32(), C.c_int32()
    st = L.gl_standardize_table(d_raw, rows, cols, kind.ctypes.data_as(C.c_void_p), classes.ctypes.data_as(C.c_void_p),
                                outs.ctypes.data_as(C.c_void_p), flag, None, C.byref(nx), None, C.byref(ny), None, 0)
    assert st == 0, L.gl_last_error()
    x = np.full((rows, nx.value), np.nan, np.float32)
    y = np.full((rows, ny.value), np.nan, np.float32)
    d_x, d_y = C.c_void_p(), C.c_void_p()
    assert L.gl_device_alloc(C.byref(d_x), max(x.nbytes, 4), 0) == 0 and L.gl_device_alloc(C.byref(d_y), max(y.nbytes, 4), 0) == 0
    stats = np.zeros((cols, 4), np.float32)
    st = L.gl_standardize_table(d_raw, rows, cols, kind.ctypes.data_as(C.c_void_p), classes.ctypes.data_as(C.c_void_p),
                                outs.ctypes.data_as(C.c_void_p), flag, d_x if nx.value else None, C.byref(nx),
                                d_y if ny.value else None, C.byref(ny), stats.ctypes.data_as(C.c_void_p), 0)
    assert st == 0, L.gl_last_error()
    if x.size:
        assert L.gl_memcpy_d2h(x.ctypes.data_as(C.c_void_p), d_x, x.nbytes, 0) == 0
    if y.size:
        assert L.gl_memcpy_d2h(y.ctypes.data_as(C.c_void_p), d_y, y.nbytes, 0) == 0
    for p in (d_raw, d_x, d_y):
        L.gl_device_free(p, 0)
    return x, y, stats


def test_standardize_table_vs_reference_golden(g, oracle):
    meta, z = load_golden("standardize")
    for k, c in enumerate(meta["cases"]):
        x, y, _ = _standardize(g, oracle, z["raw%d" % k], c["types"], c["outputs"], c["flag"])
        assert x.shape == z["x%d" % k].shape and y.shape == z["y%d" % k].shape, "case %d layout" % k
        assert np.array_equal(bits(x), bits(z["x%d" % k])), "case %d inputs" % k
        assert np.array_equal(bits(y), bits(z["y%d" % k])), "case %d expected" % k


@pytest.mark.parametrize("flag", [0, 1])
def test_standardize_table_vs_restatement_larger(g, oracle, flag):
    """A 50,000 x 21 table with categorical, constant and negative columns against the CPU restatement (itself
    pinned bit for bit to the reference's code)."""
    rng = np.random.default_rng(91 + flag)
    rows, cols = 50000, 21
    raw = rng.normal(0.0, 3.0, (rows, cols)).astype(np.float32)
    types = [0] * cols
    outputs = [0] * cols
    for c in (3, 11, 20):
        types[c] = 1
        ids = rng.integers(0, 5 + c % 4, rows)
        seen = {}
        for i, t in enumerate(ids):
            seen.setdefault(int(t), len(seen))
            ids[i] = seen[int(t)]
        raw[:, c] = ids
    raw[:, 5] = 0.0
    raw[:, 6] = -7.25
    raw[:, 7] = np.abs(raw[:, 7]) + 2.0
    outputs[19] = outputs[20] = 1
    x, y, stats = _standardize(g, oracle, raw, types, outputs, flag)
    xs, ys = oracle.standardize_table(raw, types, outputs, flag, x.shape[1], y.shape[1])
    # bit for bit, except that a z-scored constant column is 0 / 0: not-a-number on both sides, whose sign and
    # payload bits are the processor's choice, not the reference's
    for a, b in ((x, xs), (y, ys)):
        nan = np.isnan(b)
        assert np.array_equal(np.isnan(a), nan) and np.array_equal(bits(a)[~nan], bits(b)[~nan])
    assert flag == 0 or int(np.isnan(xs).all(axis=0).sum()) == 2   # the two constant columns
    assert stats[0, 0] == raw[:, 0].min() and stats[0, 1] == raw[:, 0].max()   # column 0: its own extrema
    assert stats[7, 0] == 0.0 and stats[7, 1] == raw[:, 7].max()               # others: the minimum starts from 0


def test_standardize_full_size_properties(g, oracle):
    """The window regressor's data set size (1 M rows x 33 columns, 132 MB): min-max scaling without a categorical
    column maps every column onto [0, 1] with both ends reached, equals the same fp32 expression evaluated by numpy,
    and standardising the result again changes nothing (range 1, minimum 0)."""
    rng = np.random.default_rng(5)
    rows, cols = 1 << 20, 33
    raw = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(4.0)
    outputs = [0] * (cols - 1) + [1]
    x, y, stats = _standardize(g, oracle, raw, [0] * cols, outputs, 0)
    mn = np.minimum(raw.min(0), np.float32(0.0))
    mx = np.maximum(raw.max(0), np.float32(0.0))
    mn[0], mx[0] = raw[:, 0].min(), raw[:, 0].max()
    want = (raw - mn) / (mx - mn)
    assert np.array_equal(bits(x), bits(want[:, :cols - 1])) and np.array_equal(bits(y), bits(want[:, cols - 1:]))
    assert x.min() == 0.0 and x.max() == 1.0 and float(x[:, 0].min()) == 0.0
    again = np.concatenate([x, y], axis=1)
    x2, y2, _ = _standardize(g, oracle, again, [0] * cols, outputs, 0)
    assert np.array_equal(bits(x2), bits(x)) and np.array_equal(bits(y2), bits(y))


def test_standardize_table_rejects_bad_arguments(g, oracle):
    L = g.lib()
    raw = np.zeros((4, 2), np.float32)
    d_raw = C.c_void_p()
    assert L.gl_device_alloc(C.byref(d_raw), raw.nbytes, 0) == 0
    kind = np.array([0, 1], np.int32)
    classes = np.array([0, 0], np.int32)   # a categorical column without classes
    outs = np.array([0, 1], np.int32)
    nx, ny = C.c_int32(), C.c_int32()
    args = (d_raw, 4, 2, kind.ctypes.data_as(C.c_void_p), classes.ctypes.data_as(C.c_void_p), outs.ctypes.data_as(C.c_void_p))
    assert L.gl_standardize_table(*args, 0, None, C.byref(nx), None, C.byref(ny), None, 0) == -1
    classes[1] = 3
    assert L.gl_standardize_table(*args, 2, None, C.byref(nx), None, C.byref(ny), None, 0) == -1   # unknown flag
    assert L.gl_standardize_table(*args, 0, None, C.byref(nx), None, C.byref(ny), None, 0) == 0
    assert (nx.value, ny.value) == (1, 3)
    nx.value = 2   # wrong width announced by the caller
    assert L.gl_standardize_table(*args, 0, d_raw, C.byref(nx), d_raw, C.byref(ny), None, 0) == -1
    L.gl_device_free(d_raw, 0)


def test_number_input_on_the_host_mirror_vs_reference_golden(tmp_path):
    """The C++ NumberInput (typed raw table -> one-hot maps and column plan on the host, standardisation on the
    GPU, rows served through getTrainRow / getTrainExpectedRow) against the reference's tables."""
    import os
    assert os.path.exists(HOST_TOOL), "host_tool must be built by __graft_entry__.build()"
    meta, z = load_golden("standardize")
    for k, c in enumerate(meta["cases"]):
        raw = z["raw%d" % k]
        table, out = str(tmp_path / "t.bin"), str(tmp_path / "o.bin")
        with open(table, "wb") as f:
            f.write(struct.pack("<3i", raw.shape[0], raw.shape[1], c["flag"]))
            # the host tool knows numbers and strings; the reference's int cells read back as the same floats
            f.write(np.array([1 if t == 1 else 0 for t in c["types"]], np.int32).tobytes())
            f.write(np.array(c["outputs"], np.int32).tobytes())
            f.write(np.ascontiguousarray(raw, np.float32).tobytes())
        r = run_tool("standardize", table, out)
        assert r.returncode == 0, r.stdout + r.stderr
        with open(out, "rb") as f:
            rows, nx, ny = struct.unpack("<3i", f.read(12))
            x = np.frombuffer(f.read(4 * rows * nx), np.float32).reshape(rows, nx)
            y = np.frombuffer(f.read(4 * rows * ny), np.float32).reshape(rows, ny)
        assert np.array_equal(bits(x), bits(z["x%d" % k])) and np.array_equal(bits(y), bits(z["y%d" % k])), "case %d" % k

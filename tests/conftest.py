import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as ge  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def g():
    """The product package (ctypes binding of libglades_b200.so)."""
    return ge.import_package()


@pytest.fixture(scope="session")
def oracle():
    """The CPU checkers (test infrastructure)."""
    o = ge.import_oracle()
    if not os.path.exists(o.RESTATE_PATH):
        import subprocess
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "restate"], check=True)
    return o


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    meta = json.loads(str(z["meta"]))
    return meta, z


def desc_from_meta(g, meta, **over):
    kw = dict(batch=meta.get("batch", 1), lr=meta.get("lr", 0.0), momentum=meta.get("momentum", 0.0),
              wd1=meta.get("wd1", 0.0), wd2=meta.get("wd2", 0.0), params=meta.get("params"),
              p_dropout=meta.get("p_dropout", 0.0))
    kw.update(over)
    out = meta.get("out")
    if out is None:
        out = "classification" if meta["sizes"][-1] > 1 else "regression"
    return g.make_desc(meta["sizes"], meta["acts"], out, **kw)


def libc_srand(seed):
    """Seeds the C library's rand(), which the dropout flags are drawn from (State/layer.cpp:123)."""
    import ctypes
    ctypes.CDLL(None).srand(int(seed))


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def rel_err(a, b, floor=1e-6):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), floor)))

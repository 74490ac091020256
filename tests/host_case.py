"""Case files for tests/host/host_tool.cpp (the C++ host-mirror test driver)."""
import os
import struct
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST_TOOL = os.path.join(ROOT, "glades-ml_b200", "host", "host_tool")

ACT = {"tanh": 0, "tanhp": 1, "sigmoid": 2, "sigmoidp": 3, "linear": 4, "relu": 5, "leaky": 6, "step": 7, "softmax": 8}
OUT = {"regression": 0, "classification": 1, "kl": 2}


def _per(v, n):
    return [float(x) for x in v] if isinstance(v, (list, tuple)) else [float(v)] * n


def write_case(path, sizes, acts, out, batch, lr, momentum, x, y, epochs, wd1=0.0, wd2=0.0, params=None, w=None, b=None,
               run_type=0, mode=0, seed=0):
    L = len(sizes) - 1
    x = np.ascontiguousarray(x, np.float32)
    y = np.ascontiguousarray(y, np.float32)
    with open(path, "wb") as f:
        f.write(struct.pack("<9i", len(sizes), OUT[out], batch, x.shape[0], epochs, run_type, mode,
                            1 if w is not None else 0, seed))
        f.write(np.array(sizes, np.int32).tobytes())
        f.write(np.array([ACT[a] for a in acts], np.int32).tobytes())
        for v in (lr, momentum, wd1, wd2, params if params is not None else 0.0):
            f.write(np.array(_per(v, L), np.float32).tobytes())
        f.write(x.tobytes())
        f.write(y.tobytes())
        if w is not None:
            f.write(np.ascontiguousarray(w, np.float32).tobytes())
            bb = np.zeros(len(sizes) - 2, np.float32) if b is None else np.ascontiguousarray(b, np.float32)
            f.write(bb.tobytes())


def run_tool(cmd, case, out):
    r = subprocess.run([HOST_TOOL, cmd, case, out], capture_output=True, text=True, timeout=600)
    return r


def read_run(path):
    with open(path, "rb") as f:
        d = f.read()
    off = 0

    def take(fmt, n=1):
        nonlocal off
        a = np.frombuffer(d, dtype=fmt, count=n, offset=off)
        off += a.nbytes
        return a

    res = {"epochs": int(take("<i4")[0])}
    m = take("<f4", 4)
    res.update(error=float(m[0]), accuracy=float(m[1]), class_accuracy=float(m[2]), class_f1=float(m[3]))
    n = int(take("<i4")[0])
    res["results"] = take("<f4", n).copy()
    n = int(take("<i4")[0])
    res["confusion"] = take("<i4", n).copy()
    n = int(take("<i4")[0])
    res["w"] = take("<f4", n).copy()
    n = int(take("<i4")[0])
    res["b"] = take("<f4", n).copy()
    return res

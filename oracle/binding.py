"""TEST INFRASTRUCTURE ONLY: ctypes binding of the two CPU checkers.

* ``Restate``  -- oracle/librestate.so, the plain-C restatement of the reference's arithmetic.
* ``Reference`` -- oracle/_ref/libglades_ref.so, the reference's own sources compiled unmodified
  behind the harness (present only where it was built from a reference checkout).

Only tests/, the smoke check and the CPU-baseline / reference legs of bench.py may import this.
The descriptor and metrics structures are passed in by the caller (they mirror
include/glades_b200.h) so that this module does not depend on the product package.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
RESTATE_PATH = os.path.join(HERE, "librestate.so")
REF_PATH = os.path.join(HERE, "_ref", "libglades_ref.so")


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def have_reference():
    return os.path.exists(REF_PATH)


_rs = None
_ref = None


def restate_lib():
    global _rs
    if _rs is None:
        L = C.CDLL(RESTATE_PATH)
        vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
        L.rs_create.restype = vp
        L.rs_create.argtypes = [vp, vp, vp, i64]
        L.rs_destroy.argtypes = [vp]
        L.rs_set_data.argtypes = [vp, vp, vp, i64]
        L.rs_set_weights.argtypes = [vp, vp, vp]
        L.rs_get_weights.argtypes = [vp, vp, vp]
        L.rs_get_pending_delta.argtypes = [vp, i32, vp]
        L.rs_epoch.argtypes = [vp, i32, vp, vp, vp]
        L.rs_forward_row.argtypes = [vp, i64, vp]
        L.rs_train_row.argtypes = [vp, i64]
        L.rs_grad_len.restype = i64
        L.rs_grad_len.argtypes = [vp]
        L.rs_forward_block.argtypes = [vp, i64, i32, vp, vp]
        L.rs_window_grad.argtypes = [vp, i64, i32, i32, i32, vp, vp, i64]
        L.rs_window_apply.argtypes = [vp, vp, i32]
        L.rs_set_math_mode.argtypes = [i32]
        L.rs_window_step_fast.argtypes = [vp, i64, i32, vp]
        L.rs_standardize_table.argtypes = [vp, i64, i32, vp, vp, vp, i32, vp, i32, vp, i32]
        L.rs_set_threads.argtypes = [i32]
        L.rs_get_threads.restype = i32
        for name in ("rs_squash", "rs_act_der"):
            fn = getattr(L, name)
            fn.restype = f32
            fn.argtypes = [f32, i32, f32]
        L.rs_cost.restype = f32
        L.rs_cost.argtypes = [f32, f32, f32, i32]
        L.rs_cost_der.restype = f32
        L.rs_cost_der.argtypes = [f32, f32, i32]
        L.rs_philox_u32.restype = C.c_uint32
        L.rs_philox_u32.argtypes = [C.c_uint64, C.c_uint32, C.c_uint64]
        L.rs_synth_fill.argtypes = [vp, i64, C.c_uint64, C.c_uint32, i32, f32, f32]
        _rs = L
    return _rs


def reference_lib():
    global _ref
    if _ref is None:
        L = C.CDLL(REF_PATH)
        vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
        L.ref_create.restype = vp
        L.ref_create.argtypes = [vp, vp, vp, i64]
        L.ref_destroy.argtypes = [vp]
        L.ref_set_weights.argtypes = [vp, vp, vp]
        L.ref_get_weights.argtypes = [vp, vp, vp]
        L.ref_get_pending_delta.argtypes = [vp, i32, vp]
        L.ref_train_public.argtypes = [vp, i32, vp]
        L.ref_test_public.argtypes = [vp, vp]
        L.ref_epoch.argtypes = [vp, i32, vp, vp, vp]
        L.ref_forward_row.argtypes = [vp, i64, vp]
        L.ref_train_row.argtypes = [vp, i64]
        for name in ("ref_squash", "ref_act_der"):
            fn = getattr(L, name)
            fn.restype = f32
            fn.argtypes = [f32, i32, f32]
        L.ref_cost.restype = f32
        L.ref_cost.argtypes = [f32, f32, f32, i32]
        L.ref_cost_der.restype = f32
        L.ref_cost_der.argtypes = [f32, f32, i32]
        _ref = L
    return _ref


def _nw(desc):
    return sum(desc.sizes[l + 1] * desc.sizes[l] for l in range(desc.n_layers - 1))


def _nacts(desc):
    return sum(desc.sizes[l] for l in range(1, desc.n_layers))


class _Base:
    def __init__(self, desc, x, y, metrics_type):
        self.desc = desc
        self.x = _f32(x)
        self.y = _f32(y)
        self.rows = self.x.shape[0]
        self.H = desc.n_layers - 2
        self.n_out = desc.sizes[desc.n_layers - 1]
        self.nw = _nw(desc)
        self.M = metrics_type


class Restate(_Base):
    """CPU restatement (reference mode and batched mode)."""

    def __init__(self, desc, x, y, metrics_type):
        super().__init__(desc, x, y, metrics_type)
        self.L = restate_lib()
        self.h = self.L.rs_create(C.byref(desc), _ptr(self.x), _ptr(self.y), self.rows)

    def close(self):
        if self.h:
            self.L.rs_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def set_data(self, x, y):
        self.x, self.y = _f32(x), _f32(y)
        self.rows = self.x.shape[0]
        self.L.rs_set_data(self.h, _ptr(self.x), _ptr(self.y), self.rows)

    def set_weights(self, w, bias=None):
        w, b = _f32(w), _f32(bias)
        self.L.rs_set_weights(self.h, _ptr(w), _ptr(b))

    def get_weights(self):
        w = np.empty(self.nw, np.float32)
        b = np.empty(max(self.H, 1), np.float32)
        self.L.rs_get_weights(self.h, _ptr(w), _ptr(b))
        return w, b[: self.H]

    def pending_delta(self, k):
        a = np.empty(self.nw, np.float32)
        self.L.rs_get_pending_delta(self.h, k, _ptr(a))
        return a

    def epoch(self, run_type=0, want_outputs=False):
        m = self.M()
        cm = np.zeros((self.n_out, self.n_out), np.int32)
        out = np.empty((self.rows, self.n_out), np.float32) if want_outputs else None
        self.L.rs_epoch(self.h, run_type, C.byref(m), _ptr(cm), _ptr(out))
        return m, cm, out

    def forward_row(self, row):
        a = np.empty(_nacts(self.desc), np.float32)
        self.L.rs_forward_row(self.h, row, _ptr(a))
        return a

    def train_row(self, row):
        self.L.rs_train_row(self.h, row)

    def forward_block(self, first, cnt):
        out = np.empty((cnt, self.n_out), np.float32)
        am = np.empty(cnt, np.int32)
        self.L.rs_forward_block(self.h, first, cnt, _ptr(out), _ptr(am))
        return out, am

    def grad_len(self):
        return self.L.rs_grad_len(self.h)

    def window_grad(self, first, cnt, global_rows=None, first_pos=0, confusion=None, metric_rows=None):
        g = np.zeros(self.grad_len(), np.float64)
        self.L.rs_window_grad(self.h, first, cnt, global_rows or cnt, first_pos, _ptr(g), _ptr(confusion),
                              metric_rows or self.rows)
        return g

    def window_apply(self, grad, global_rows):
        g = np.ascontiguousarray(grad, np.float64)
        self.L.rs_window_apply(self.h, _ptr(g), global_rows)

    def train_window(self, first, cnt):
        g = self.window_grad(first, cnt)
        self.window_apply(g, cnt)
        return g

    def train_window_fast(self, first, cnt):
        """The same window step with blocked fp32 products on all host cores (fastport.c): the timed CPU
        baseline, not the checker.  Returns the window's cost sum."""
        cost = C.c_float()
        self.L.rs_window_step_fast(self.h, first, cnt, C.byref(cost))
        return cost.value


class Reference(_Base):
    """The compiled reference behind the harness (reference arithmetic only)."""

    def __init__(self, desc, x, y, metrics_type):
        super().__init__(desc, x, y, metrics_type)
        self.L = reference_lib()
        self.h = self.L.ref_create(C.byref(desc), _ptr(self.x), _ptr(self.y), self.rows)
        if not self.h:
            raise RuntimeError("ref_create failed")

    def close(self):
        if self.h:
            self.L.ref_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def set_weights(self, w, bias=None):
        w, b = _f32(w), _f32(bias)
        self.L.ref_set_weights(self.h, _ptr(w), _ptr(b))

    def get_weights(self):
        w = np.empty(self.nw, np.float32)
        b = np.empty(max(self.H, 1), np.float32)
        self.L.ref_get_weights(self.h, _ptr(w), _ptr(b))
        return w, b[: self.H]

    def pending_delta(self, k):
        a = np.empty(self.nw, np.float32)
        self.L.ref_get_pending_delta(self.h, k, _ptr(a))
        return a

    def train_public(self, n):
        m = self.M()
        self.L.ref_train_public(self.h, n, C.byref(m))
        return m

    def test_public(self):
        m = self.M()
        self.L.ref_test_public(self.h, C.byref(m))
        return m

    def epoch(self, run_type=0, want_outputs=False):
        m = self.M()
        cm = np.zeros((self.n_out, self.n_out), np.int32)
        out = np.empty((self.rows, self.n_out), np.float32) if want_outputs else None
        self.L.ref_epoch(self.h, run_type, C.byref(m), _ptr(cm), _ptr(out))
        return m, cm, out

    def forward_row(self, row):
        a = np.empty(_nacts(self.desc), np.float32)
        self.L.ref_forward_row(self.h, row, _ptr(a))
        return a

    def train_row(self, row):
        self.L.ref_train_row(self.h, row)


def set_threads(t):
    """Sets the OpenMP thread count of the restatement's loops (overriding a launcher's OMP_NUM_THREADS)
    and returns the count they will really use (1 when the library was built without OpenMP)."""
    L = restate_lib()
    L.rs_set_threads(int(t))
    return int(L.rs_get_threads())


def standardize_plan(raw, types):
    """kind / classes arrays of a raw table whose categorical columns (type 1) hold category indices."""
    kind = np.array([1 if t == 1 else 0 for t in types], np.int32)
    classes = np.array([int(raw[:, c].max()) + 1 if t == 1 else 0 for c, t in enumerate(types)], np.int32)
    return kind, classes


def standardize_table(raw, types, outputs, flag, nx, ny):
    """The CPU restatement of NumberInput::standardizeInputTable on a flat raw table."""
    raw = np.ascontiguousarray(raw, np.float32)
    rows, cols = raw.shape
    kind, classes = standardize_plan(raw, types)
    outs = np.array(outputs, np.int32)
    x = np.zeros((rows, nx), np.float32)
    y = np.zeros((rows, ny), np.float32)
    rc = restate_lib().rs_standardize_table(_ptr(raw), rows, cols, _ptr(kind), _ptr(classes), _ptr(outs), flag, _ptr(x), nx,
                                            _ptr(y), ny)
    if rc != 0:
        raise ValueError("the table does not standardise to %d input and %d expected columns" % (nx, ny))
    return x, y


def synth_fill(n, seed, stream, dist, scale=1.0, offset=0.0):
    out = np.empty(n, np.float32)
    restate_lib().rs_synth_fill(_ptr(out), n, seed, stream, dist, scale, offset)
    return out

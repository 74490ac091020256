"""ctypes mirror of include/glades_b200.h."""
import ctypes as C
import os

import numpy as np

GL_MAX_WEIGHT_LAYERS = 16

# GMath activation / cost ids (reference: GMath/gmath.h:38-50); SOFTMAX is this library's extension.
ACT = {"tanh": 0, "tanhp": 1, "sigmoid": 2, "sigmoidp": 3, "linear": 4, "relu": 5, "leaky": 6,
       "step": 7, "softmax": 8}
OUT = {"regression": 0, "classification": 1, "kl": 2}
MODE_REFERENCE, MODE_BATCHED = 0, 1
BIAS_MEAN, BIAS_REFERENCE = 0, 1
GEMM_AUTO, GEMM_FFMA, GEMM_TCGEN05, GEMM_GRID_FUSED = 0, 1, 2, 3


class NetDesc(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int32),
        ("sizes", C.c_int32 * (GL_MAX_WEIGHT_LAYERS + 1)),
        ("lr", C.c_float * GL_MAX_WEIGHT_LAYERS),
        ("momentum", C.c_float * GL_MAX_WEIGHT_LAYERS),
        ("wd1", C.c_float * GL_MAX_WEIGHT_LAYERS),
        ("wd2", C.c_float * GL_MAX_WEIGHT_LAYERS),
        ("p_dropout", C.c_float * GL_MAX_WEIGHT_LAYERS),
        ("activation", C.c_int32 * GL_MAX_WEIGHT_LAYERS),
        ("act_param", C.c_float * GL_MAX_WEIGHT_LAYERS),
        ("output_type", C.c_int32),
        ("batch_size", C.c_int32),
        ("mode", C.c_int32),
        ("bias_rule", C.c_int32),
        ("gemm", C.c_int32),
        ("device", C.c_int32),
    ]


class Metrics(C.Structure):
    _fields_ = [
        ("total_error", C.c_float),
        ("total_accuracy", C.c_float),
        ("class_accuracy", C.c_float),
        ("class_precision", C.c_float),
        ("class_recall", C.c_float),
        ("class_specificity", C.c_float),
        ("class_f1", C.c_float),
        ("epochs", C.c_int32),
        ("nonfinite", C.c_int32),
        ("rows", C.c_int64),
        ("device_ms", C.c_double),
        ("kernel_launches", C.c_int64),
    ]

    def as_dict(self):
        return {k: getattr(self, k) for k, _ in self._fields_}


def make_desc(sizes, acts, out_type, batch=1, lr=0.01, momentum=0.0, wd1=0.0, wd2=0.0, params=None,
              mode=MODE_REFERENCE, bias_rule=BIAS_MEAN, gemm=GEMM_AUTO, device=0, p_dropout=0.0):
    """Descriptor for layer sizes n_0..n_{H+1}; acts[l] is the activation producing layer l+1.

    lr / momentum / wd1 / wd2 / params may be scalars or per-weight-layer lists (NNInfo index l);
    p_dropout a scalar or a list per node layer 0..H (input and hidden layers)."""
    d = NetDesc()
    nl = len(sizes)
    assert 3 <= nl <= GL_MAX_WEIGHT_LAYERS + 1 and len(acts) == nl - 1
    d.n_layers = nl
    for i, s in enumerate(sizes):
        d.sizes[i] = int(s)

    def per(v, l):
        return float(v[l]) if isinstance(v, (list, tuple)) else float(v)

    for l in range(nl - 1):
        d.lr[l] = per(lr, l)
        d.momentum[l] = per(momentum, l)
        d.wd1[l] = per(wd1, l)
        d.wd2[l] = per(wd2, l)
        d.p_dropout[l] = per(p_dropout, l)
        a = acts[l]
        d.activation[l] = ACT[a] if isinstance(a, str) else int(a)
        d.act_param[l] = per(params, l) if params is not None else 0.0
    d.output_type = OUT[out_type] if isinstance(out_type, str) else int(out_type)
    d.batch_size = int(batch)
    d.mode = mode
    d.bias_rule = bias_rule
    d.gemm = gemm
    d.device = device
    return d


def weight_count(desc):
    return sum(desc.sizes[l + 1] * desc.sizes[l] for l in range(desc.n_layers - 1))


class GladesError(RuntimeError):
    def __init__(self, status, text):
        super().__init__("glades_b200 status %d: %s" % (status, text))
        self.status = status


def lib_path():
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "libglades_b200.so")


_lib = None

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)


def lib():
    """Loads libglades_b200.so (built in-tree by __graft_entry__.build()); raises if missing."""
    global _lib
    if _lib is not None:
        return _lib
    p = lib_path()
    if not os.path.exists(p):
        raise OSError("%s is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`; "
                      "there is no CPU fallback" % p)
    L = C.CDLL(p, mode=C.RTLD_GLOBAL)
    vp, i32, i64, u32, u64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_float
    mp = C.POINTER(Metrics)
    sig = {
        "gl_last_error": (C.c_char_p, []),
        "gl_device_count": (C.c_int, []),
        "gl_create": (C.c_int, [C.POINTER(NetDesc), C.POINTER(vp)]),
        "gl_destroy": (C.c_int, [vp]),
        "gl_set_weights": (C.c_int, [vp, vp, vp]),
        "gl_get_weights": (C.c_int, [vp, vp, vp]),
        "gl_weight_count": (i64, [vp]),
        "gl_save_state": (C.c_int, [vp, C.c_char_p]),
        "gl_load_state": (C.c_int, [vp, C.c_char_p]),
        "gl_set_data": (C.c_int, [vp, vp, vp, i64]),
        "gl_set_data_device": (C.c_int, [vp, vp, vp, i64]),
        "gl_train_epochs": (C.c_int, [vp, i32, mp]),
        "gl_train_window": (C.c_int, [vp, i64, i32, mp]),
        "gl_train_window_host": (C.c_int, [vp, vp, vp, i32, mp]),
        "gl_train_window_host_submit": (C.c_int, [vp, vp, vp, i32]),
        "gl_train_window_host_result": (C.c_int, [vp, mp]),
        "gl_forward": (C.c_int, [vp, i64, i64, vp, vp, mp]),
        "gl_forward_host": (C.c_int, [vp, vp, vp, i64, vp, vp, mp]),
        "gl_get_activations": (C.c_int, [vp, i64, vp]),
        "gl_get_pending_delta": (C.c_int, [vp, i32, vp]),
        "gl_get_confusion": (C.c_int, [vp, vp]),
        "gl_get_last_outputs": (C.c_int, [vp, vp]),
        "gl_get_epochs": (C.c_int, [vp]),
        "gl_stop": (None, [vp]),
        "gl_snapshot_submit": (C.c_int, [vp]),
        "gl_snapshot_collect": (C.c_int, [vp, vp, vp, vp, i32]),
        "gl_sync": (C.c_int, [vp]),
        "gl_kernel_launches": (i64, [vp]),
        "gl_tensor_core_launches": (i64, [vp]),
        "gl_window_cluster_ctas": (C.c_int32, [vp]),
        "gl_matmul": (C.c_int, [vp, i64, i64, vp, i64, i64, vp, i64, i32, i32, i32, i32, i32]),
        "gl_shard_range": (None, [i64, i32, i32, C.POINTER(i64), C.POINTER(i64)]),
        "gl_dp_unique_id": (C.c_int, [vp]),
        "gl_dp_init": (C.c_int, [vp, i32, i32, vp]),
        "gl_dp_set_window": (C.c_int, [vp, i32, i32]),
        "gl_dp_mode": (C.c_int, [vp]),
        "gl_forward_host_submit": (C.c_int, [vp, vp, vp, i32]),
        "gl_forward_host_result": (C.c_int, [vp, vp, mp]),
        "gl_synth_fill": (C.c_int, [vp, i64, u64, u32, i32, f32, f32, i32]),
        "gl_selftest_bounded_wait": (C.c_int, [vp, i64, C.POINTER(C.c_double)]),
        "gl_synth_fill_at": (C.c_int, [vp, i64, i64, u64, u32, i32, f32, f32, i32]),
        "gl_tc_variant_counts": (None, [C.POINTER(i64)]),
        "gl_matmul_static": (C.c_int, [vp, i64, i64, vp, i64, i64, vp, i64, i32, i32, i32, i32]),
        "gl_matmul_static_error": (C.c_char_p, []),
        "gl_standardize_table": (C.c_int, [vp, i64, i32, vp, vp, vp, i32, vp, C.POINTER(i32), vp, C.POINTER(i32), vp, i32]),
        "gl_onehot_fill": (C.c_int, [vp, vp, i64, i32, f32, f32, i32]),
        "gl_timer_start": (C.c_int, [vp]),
        "gl_timer_stop": (C.c_int, [vp, C.POINTER(C.c_double)]),
        "gl_profile_enable": (C.c_int, [vp, i32]),
        "gl_profile_read": (C.c_int, [vp, C.POINTER(C.c_double)]),
        "gl_device_alloc": (C.c_int, [C.POINTER(vp), i64, i32]),
        "gl_device_free": (C.c_int, [vp, i32]),
        "gl_device_mem_info": (C.c_int, [i32, C.POINTER(i64), C.POINTER(i64)]),
        "gl_memcpy_h2d": (C.c_int, [vp, vp, i64, i32]),
        "gl_memcpy_d2h": (C.c_int, [vp, vp, i64, i32]),
        "gl_host_alloc_pinned": (C.c_int, [C.POINTER(vp), i64]),
        "gl_host_free_pinned": (C.c_int, [vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def _check(st):
    if st != 0:
        raise GladesError(st, lib().gl_last_error().decode("utf-8", "replace"))


def device_count():
    return lib().gl_device_count()


def tc_variant_counts():
    """Tensor-core product launches of this process: [128-wide, 256-wide, several tiles per CTA, peer-store,
    last wave split along k]."""
    out = (C.c_int64 * 5)()
    lib().gl_tc_variant_counts(out)
    return [int(v) for v in out]


def shard_range(rows, rank, world):
    f, c = C.c_int64(), C.c_int64()
    lib().gl_shard_range(rows, rank, world, C.byref(f), C.byref(c))
    return f.value, c.value


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


class Net:
    """Thin owner of one gl_net handle; every method is one C-ABI call."""

    def __init__(self, desc):
        self.desc = desc
        self.h = C.c_void_p()
        _check(lib().gl_create(C.byref(desc), C.byref(self.h)))
        self.n_out = desc.sizes[desc.n_layers - 1]
        self.n_in = desc.sizes[0]
        self.H = desc.n_layers - 2
        self.nw = weight_count(desc)
        self._keep = []

    def close(self):
        if self.h:
            lib().gl_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_weights(self, w, bias=None):
        w = _f32(w)
        assert w.size == self.nw
        b = _f32(bias)
        _check(lib().gl_set_weights(self.h, _ptr(w), _ptr(b)))

    def get_weights(self):
        w = np.empty(self.nw, np.float32)
        b = np.empty(max(self.H, 1), np.float32)
        _check(lib().gl_get_weights(self.h, _ptr(w), _ptr(b)))
        return w, b[: self.H]

    def save_state(self, path):
        _check(lib().gl_save_state(self.h, str(path).encode()))

    def load_state(self, path):
        _check(lib().gl_load_state(self.h, str(path).encode()))

    def set_data(self, x, y):
        x, y = _f32(x), _f32(y)
        rows = x.shape[0]
        assert x.size == rows * self.n_in and y.size == rows * self.n_out
        _check(lib().gl_set_data(self.h, _ptr(x), _ptr(y), rows))

    def set_data_device(self, d_x, d_y, rows):
        _check(lib().gl_set_data_device(self.h, C.c_void_p(d_x), C.c_void_p(d_y) if d_y else None, rows))

    def train_epochs(self, n):
        m = Metrics()
        _check(lib().gl_train_epochs(self.h, n, C.byref(m)))
        return m

    def train_window(self, first_row, rows, want_metrics=True):
        """One window step; with want_metrics=False the call only queues the work (see sync())."""
        if not want_metrics:
            _check(lib().gl_train_window(self.h, first_row, rows, None))
            return None
        m = Metrics()
        _check(lib().gl_train_window(self.h, first_row, rows, C.byref(m)))
        return m

    def train_window_host(self, x, y, rows=None):
        m = Metrics()
        rows = x.shape[0] if rows is None else rows
        _check(lib().gl_train_window_host(self.h, _ptr(x), _ptr(y), rows, C.byref(m)))
        return m

    def submit_window_host(self, x, y, rows=None):
        rows = x.shape[0] if rows is None else rows
        _check(lib().gl_train_window_host_submit(self.h, _ptr(x), _ptr(y), rows))

    def window_result(self):
        m = Metrics()
        _check(lib().gl_train_window_host_result(self.h, C.byref(m)))
        return m

    def forward(self, first_row, rows, want_outputs=True, want_argmax=True):
        out = np.empty((rows, self.n_out), np.float32) if want_outputs else None
        am = np.empty(rows, np.int32) if want_argmax else None
        m = Metrics()
        _check(lib().gl_forward(self.h, first_row, rows, _ptr(out), _ptr(am), C.byref(m)))
        return out, am, m

    def forward_host(self, x, y=None, out=None, am=None):
        rows = x.shape[0]
        if out is None:
            out = np.empty((rows, self.n_out), np.float32)
        if am is None:
            am = np.empty(rows, np.int32)
        m = Metrics()
        _check(lib().gl_forward_host(self.h, _ptr(x), _ptr(y), rows, _ptr(out), _ptr(am), C.byref(m)))
        return out, am, m

    def submit_forward_host(self, x, y=None):
        """Queues an inference batch from host rows (at most two in flight); the arrays must stay alive
        (pinned memory gives the overlap) until the matching forward_result()."""
        _check(lib().gl_forward_host_submit(self.h, _ptr(x), _ptr(y), x.shape[0]))

    def forward_result(self, rows):
        am = np.empty(rows, np.int32)
        m = Metrics()
        _check(lib().gl_forward_host_result(self.h, _ptr(am), C.byref(m)))
        return am, m

    def activations(self, row):
        n = sum(self.desc.sizes[l] for l in range(1, self.desc.n_layers))
        a = np.empty(n, np.float32)
        _check(lib().gl_get_activations(self.h, row, _ptr(a)))
        return a

    def pending_delta(self, k):
        a = np.empty(self.nw, np.float32)
        _check(lib().gl_get_pending_delta(self.h, k, _ptr(a)))
        return a

    def confusion(self):
        a = np.zeros((self.n_out, self.n_out), np.int32)
        _check(lib().gl_get_confusion(self.h, _ptr(a)))
        return a

    def last_outputs(self):
        a = np.empty(self.n_out, np.float32)
        _check(lib().gl_get_last_outputs(self.h, _ptr(a)))
        return a

    def epochs(self):
        return lib().gl_get_epochs(self.h)

    def stop(self):
        lib().gl_stop(self.h)

    def snapshot_submit(self):
        _check(lib().gl_snapshot_submit(self.h))

    def snapshot_collect(self, wait=True):
        """(weights, biases, last-row pre-activations), or None when wait is False and the copy still runs."""
        w = np.empty(self.nw, np.float32)
        b = np.empty(max(self.H, 1), np.float32)
        n = sum(self.desc.sizes[l] for l in range(1, self.desc.n_layers))
        z = np.empty(n, np.float32)
        st = lib().gl_snapshot_collect(self.h, _ptr(w), _ptr(b), _ptr(z), 1 if wait else 0)
        if st == 1:
            return None
        _check(st)
        return w, b[: self.H], z

    def sync(self):
        _check(lib().gl_sync(self.h))

    def selftest_bounded_wait(self, max_cycles):
        """Queues a wait on a flag nobody raises; returns the device milliseconds it took to give up."""
        ms = C.c_double()
        _check(lib().gl_selftest_bounded_wait(self.h, int(max_cycles), C.byref(ms)))
        return ms.value

    def timer_start(self):
        _check(lib().gl_timer_start(self.h))

    def timer_stop(self):
        ms = C.c_double()
        _check(lib().gl_timer_stop(self.h, C.byref(ms)))
        return ms.value

    def profile_enable(self, on=True):
        _check(lib().gl_profile_enable(self.h, 1 if on else 0))

    def profile_read(self):
        out = (C.c_double * 6)()
        _check(lib().gl_profile_read(self.h, out))
        return {"tc": {"launches": int(out[0]), "ms": out[1], "flop": out[2]},
                "ffma": {"launches": int(out[3]), "ms": out[4], "flop": out[5]}}

    def kernel_launches(self):
        return lib().gl_kernel_launches(self.h)

    def tensor_core_launches(self):
        return lib().gl_tensor_core_launches(self.h)

    def window_cluster_ctas(self):
        return lib().gl_window_cluster_ctas(self.h)

    def dp_init(self, rank, world, id_bytes):
        buf = (C.c_char * 128).from_buffer_copy(id_bytes)
        _check(lib().gl_dp_init(self.h, rank, world, buf))

    def dp_mode(self):
        """0: not data parallel, 1: NCCL all-reduce per layer, 2: exchange over peer memory."""
        return int(lib().gl_dp_mode(self.h))

    def dp_set_window(self, global_rows, first_pos):
        _check(lib().gl_dp_set_window(self.h, global_rows, first_pos))

"""ctypes binding of the B200-native glades feed-forward library (libglades_b200.so).

The product is the C-ABI shared library declared in include/glades_b200.h and the C++ host
classes in host/; this Python package only loads the library for the tests and the benchmark.
Because the directory name contains a hyphen, load it with `__graft_entry__.import_package()`.
There is no CPU fallback: loading fails loudly when the library has not been built, and every
compute entry point returns GL_ERR_NO_DEVICE without an sm_100 device.
"""
from .capi import (  # noqa: F401
    GL_MAX_WEIGHT_LAYERS, ACT, OUT, MODE_REFERENCE, MODE_BATCHED, BIAS_MEAN, BIAS_REFERENCE,
    GEMM_AUTO, GEMM_FFMA, GEMM_TCGEN05, GEMM_GRID_FUSED, NetDesc, Metrics, GladesError, Net, lib, lib_path,
    make_desc, weight_count, shard_range, device_count, tc_variant_counts,
)

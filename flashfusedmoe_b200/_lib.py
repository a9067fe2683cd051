"""ctypes binding of libffmoe.so (the C ABI declared in include/ffmoe.h).

The library is the only compute path of this package: importing a kernel wrapper without the built
library raises, there is no fallback.
"""

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libffmoe.so")

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_int64 = ctypes.c_int64
c_float = ctypes.c_float
c_size_t = ctypes.c_size_t

FFM_OK = 0
GATING = {"softmax": 0, "sigmoid": 1}
ACTIVATION = {"swiglu": 0, "geglu": 1, "relu_squared": 2, "geglu_erf": 3}
B_KMAJOR = 0
B_NMAJOR = 1

# name -> (restype, argtypes); must list every symbol include/ffmoe.h declares
SIGNATURES = {
    "ffm_version": (c_int, []),
    "ffm_error_string": (ctypes.c_char_p, [c_int]),
    "ffm_rows_capacity": (c_int64, [c_int64, c_int]),
    "ffm_set_wait_cycles": (ctypes.c_longlong, [ctypes.c_longlong]),
    "ffm_set_gemm_cta_pair": (c_int, [c_int]),
    "ffm_route_workspace_bytes": (c_size_t, [c_int64, c_int, c_int]),
    "ffm_route_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_float,
                                  c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int64, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "ffm_route_apply_capacity": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                         c_int, c_void_p, c_void_p]),
    "ffm_group_rows": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                               c_void_p, c_size_t, c_void_p, c_void_p]),
    "ffm_group_rows_static": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                      c_void_p, c_void_p]),
    "ffm_permute_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p]),
    "ffm_grouped_gemm_glu": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_int,
                                     c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "ffm_grouped_gemm": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64, c_int, c_int, c_float,
                                 c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "ffm_grouped_gemm_wgrad": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_float,
                                       c_void_p, c_void_p, c_void_p]),
    "ffm_grouped_gemm_wgrad_glu_backward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_float,
                                                    c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                                                    c_void_p, c_void_p]),
    "ffm_grouped_gemm_dact_glu_backward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int,
                                                   c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "ffm_quantize_rows_e4m3": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p]),
    "ffm_quantize_rows_given_scale_e4m3": (c_int, [c_void_p, c_int64, c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "ffm_grouped_gemm_glu_fp8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int,
                                         c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "ffm_grouped_gemm_fp8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int,
                                     c_void_p, c_int, c_void_p, c_void_p]),
    "ffm_combine_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                                    c_void_p]),
    "ffm_combine_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p]),
    "ffm_glu_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "ffm_compact_positions": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p,
                                      c_void_p]),
    "ffm_p2p_push": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ffm_p2p_set_local_only": (c_int, [c_int]),
    "ffm_p2p_push_rows": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_int,
                                  c_void_p]),
    "ffm_p2p_push_rows_dev": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64,
                                      c_void_p, c_int, c_void_p]),
    "ffm_p2p_plan": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "ffm_p2p_signal_wait_dev": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p]),
    "ffm_p2p_signal_wait": (c_int, [c_void_p, c_int, c_int, ctypes.c_uint32, c_void_p, ctypes.c_longlong, c_void_p]),
    "ffm_route_backward_workspace_bytes": (c_size_t, [c_int64, c_int, c_int]),
    "ffm_route_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                   c_void_p, c_size_t, c_void_p, c_void_p]),
}

_lib = None


def load():
    """Load libffmoe.so and attach prototypes. Raises if the library has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m flashfusedmoe_b200.build` "
            "(nvcc, sm_100a). This package has no fallback path.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def error_string(code):
    return load().ffm_error_string(int(code)).decode()


def check(code, what):
    if code != FFM_OK:
        raise RuntimeError(f"libffmoe {what} failed: {code} ({error_string(code)})")

"""ctypes binding of libturbofno_b200.so (declarations: include/turbofno_b200.h).

There is no fallback: if the shared library is missing or a symbol cannot be resolved, importing
this module raises.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libturbofno_b200.so")

OK = 0
ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_ALLOC, ERR_LIBRARY, ERR_WORKSPACE = 1, 2, 3, 4, 5, 6
ERR_SCRATCH_LIMIT = 7
ERR_KERNEL_WAIT = 8
VARIANT = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4}


class Problem(ctypes.Structure):
    _fields_ = [
        ("rank", ctypes.c_int),
        ("bs", ctypes.c_longlong),
        ("dimX", ctypes.c_int),
        ("DX", ctypes.c_int),
        ("DY", ctypes.c_int),
        ("K", ctypes.c_int),
        ("N", ctypes.c_int),
        ("modes", ctypes.c_int),
        ("variant", ctypes.c_int),
        ("x_stride_b", ctypes.c_longlong),
        ("x_stride_k", ctypes.c_longlong),
        ("y_stride_b", ctypes.c_longlong),
        ("y_stride_n", ctypes.c_longlong),
        ("w_stride_k", ctypes.c_longlong),
        ("w_stride_n", ctypes.c_longlong),
        ("alpha_re", ctypes.c_float),
        ("alpha_im", ctypes.c_float),
        ("beta_re", ctypes.c_float),
        ("beta_im", ctypes.c_float),
        ("second_transform_forward", ctypes.c_int),
        ("scale_inverse", ctypes.c_int),
        ("x_modes_centered", ctypes.c_int),
        ("w_stride_m", ctypes.c_longlong),
    ]


# every symbol include/turbofno_b200.h declares: name -> (restype, argtypes)
_vp, _i, _ll, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
SYMBOLS = {
    "tfno_problem_init": (_i, [ctypes.POINTER(Problem), _i]),
    "tfno_create": (_i, [ctypes.POINTER(_vp), _i]),
    "tfno_destroy": (_i, [_vp]),
    "tfno_sm_count": (_i, [_vp, ctypes.POINTER(_i)]),
    "tfno_device_status": (_i, [_vp, ctypes.POINTER(_i)]),
    "tfno_device_status_reset": (_i, [_vp]),
    "tfno_selftest_bounded_wait": (_i, [_vp, _vp]),
    "tfno_plan_create": (_i, [_vp, ctypes.POINTER(Problem), ctypes.POINTER(_vp)]),
    "tfno_plan_destroy": (_i, [_vp]),
    "tfno_workspace_bytes": (ctypes.c_size_t, [_vp]),
    "tfno_exec": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "tfno_exec_host": (_i, [_vp, _vp, _vp, _vp]),
    "tfno_plan_set_host_chunk": (_i, [_vp, _ll]),
    "tfno_plan_kernels": (_i, [_vp, ctypes.c_char_p, ctypes.c_size_t]),
    "tfno_status_string": (ctypes.c_char_p, [_i]),
    "tfno_fused_fft_cgemm_ifft": (_i, [_vp, _i, _ll, _i, _i, _vp, _vp, _vp, _vp, _f, _f, _f, _f, _vp]),
    "tfno_fused_fft_cgemm": (_i, [_vp, _i, _ll, _i, _i, _vp, _vp, _vp, _f, _f, _f, _f, _vp]),
    "tfno_fused_cgemm_ifft": (_i, [_vp, _i, _ll, _i, _i, _vp, _vp, _vp, _vp, _f, _f, _f, _f, _vp]),
    "tfno_cgemm": (_i, [_vp, _ll, _i, _i, _vp, _vp, _vp, _f, _f, _f, _f, _vp]),
    "tfno_fft_stride_DY": (_i, [_vp, _i, _vp, _vp, _ll, _vp]),
    "tfno_ifft_stride_DY": (_i, [_vp, _i, _vp, _vp, _ll, _vp]),
    "tfno_fft_stride": (_i, [_vp, _i, _vp, _vp, _i, _ll, _vp]),
    "tfno_ifft_stride": (_i, [_vp, _i, _vp, _vp, _i, _ll, _vp]),
    "tfno_static_scratch_bytes": (ctypes.c_size_t, []),
    "tfno_spectral_conv2d_static": (_i, [_ll, _i, _i, _i, _i, _vp, _vp, _vp, _f, _f, _vp]),
}

_LIB = None


def load():
    """Load the shared library and bind every declared symbol; raises if anything is missing."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "turbofno_b200: %s not found -- build it with `python -m turbofno_b200.build` "
            "(there is no CPU or PyTorch fallback)" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


class TfnoError(RuntimeError):
    def __init__(self, status, where=""):
        self.status = status
        msg = load().tfno_status_string(status).decode()
        super().__init__("%s: %s (status %d)" % (where or "turbofno_b200", msg, status))


def check(status, where=""):
    if status != OK:
        raise TfnoError(status, where)

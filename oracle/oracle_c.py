"""ctypes loader for the C oracle (oracle/liboracle.so).  Test infrastructure only."""
import ctypes
import hashlib
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force=False):
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "spectral_oracle.c")
    inc = os.path.join(_HERE, "spectral_oracle_impl.inc")
    h = hashlib.sha256()
    for p in (src, inc):
        with open(p, "rb") as f:
            h.update(f.read())
    stamp = so + ".srchash"
    stale = not (os.path.exists(so) and os.path.exists(stamp) and open(stamp).read().strip() == h.hexdigest())
    if force or stale:
        subprocess.check_call(["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC", src, "-o", so, "-lm"])
        with open(stamp, "w") as f:
            f.write(h.hexdigest())
    return so


def lib():
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(build())
        fp = ctypes.c_void_p
        for suffix in ("f32", "f64"):
            f1 = getattr(L, "oracle_spectral_conv1d_" + suffix)
            f1.restype = ctypes.c_int
            f1.argtypes = [fp, fp, fp, ctypes.c_long] + [ctypes.c_int] * 4 + [ctypes.c_float] * 2 + [ctypes.c_int] * 3
            f2 = getattr(L, "oracle_spectral_conv2d_" + suffix)
            f2.restype = ctypes.c_int
            f2.argtypes = [fp, fp, fp, ctypes.c_long] + [ctypes.c_int] * 5 + [ctypes.c_float] * 2 + [ctypes.c_int] * 3
        L.oracle_max_threads.restype = ctypes.c_int
        _LIB = L
    return _LIB


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def spectral_conv_1d(x, w, modes=64, alpha=1.0 + 0j, inverse=True, scale=True, double=True, threads=0):
    """x[B,K,DY] complex64, w[K,N] complex64 -> y[B,N,DY] (complex128 if double else complex64)."""
    x = np.ascontiguousarray(x, dtype=np.complex64)
    w = np.ascontiguousarray(w, dtype=np.complex64)
    B, K, DY = x.shape
    N = w.shape[1]
    y = np.empty((B, N, DY), dtype=np.complex128 if double else np.complex64)
    fn = lib().oracle_spectral_conv1d_f64 if double else lib().oracle_spectral_conv1d_f32
    rc = fn(_ptr(x), _ptr(w), _ptr(y), B, K, N, DY, modes, alpha.real, alpha.imag, int(inverse), int(scale), threads)
    if rc:
        raise RuntimeError("oracle_spectral_conv1d failed: %d" % rc)
    return y


def spectral_conv_2d(x, w, modes=64, alpha=1.0 + 0j, inverse=True, scale=True, double=True, threads=0):
    x = np.ascontiguousarray(x, dtype=np.complex64)
    w = np.ascontiguousarray(w, dtype=np.complex64)
    B, K, DX, DY = x.shape
    N = w.shape[1]
    y = np.empty((B, N, DX, DY), dtype=np.complex128 if double else np.complex64)
    fn = lib().oracle_spectral_conv2d_f64 if double else lib().oracle_spectral_conv2d_f32
    rc = fn(_ptr(x), _ptr(w), _ptr(y), B, K, N, DX, DY, modes, alpha.real, alpha.imag, int(inverse), int(scale), threads)
    if rc:
        raise RuntimeError("oracle_spectral_conv2d failed: %d" % rc)
    return y


def max_threads():
    return lib().oracle_max_threads()

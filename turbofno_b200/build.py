"""Build recipe for libturbofno_b200.so (sm_100a only) and the TurboFNO_{1D,2D}_{A..E} drivers.

Run as `python -m turbofno_b200.build [--force] [--drivers]`.  Everything is built in-tree so
that the shared library sits next to the package that loads it.
"""
import hashlib
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libturbofno_b200.so")
BIN = os.path.join(PKG, "bin")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
]


def _digest(sources, extra=""):
    h = hashlib.sha256(extra.encode())
    for s in sources:
        if os.path.exists(s):
            h.update(os.path.basename(s).encode())
            with open(s, "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def _newer(target, sources, extra=""):
    """True when `target` is missing or was built from different source contents.  Contents, not
    timestamps: a copied tree does not keep the order of modification times."""
    stamp = target + ".srchash"
    if not os.path.exists(target) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != _digest(sources, extra)


def _stamp(target, sources, extra=""):
    with open(target + ".srchash", "w") as f:
        f.write(_digest(sources, extra))


def _lib_sources():
    srcs = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh"))]
    srcs.append(os.path.join(ROOT, "include", "turbofno_b200.h"))
    return srcs


def build_library(force=False, verbose=False):
    srcs = _lib_sources()
    if not force and not _newer(LIB, srcs):
        return LIB
    cus = [s for s in srcs if s.endswith(".cu")]
    cmd = ["nvcc"] + NVCC_FLAGS + ["-shared"] + cus + ["-o", LIB, "-lcufft", "-lcublas"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    subprocess.check_call(cmd)
    _stamp(LIB, srcs)
    return LIB


VARIANTS = [(rank, v) for rank in (1, 2) for v in "ABCDE"]


def build_drivers(force=False):
    """The ten executables TurboFNO_{1D,2D}_{A,B,C,D,E}: one C++ source, compiled once per
    (rank, variant) the way the reference builds one CMake project per variant."""
    os.makedirs(BIN, exist_ok=True)
    src = os.path.join(PKG, "drivers", "turbofno_driver.cpp")
    hdrs = [os.path.join(ROOT, "include", "turbofno_b200.h"), os.path.join(ROOT, "include", "TurboFNO.h")]
    build_library(force=force)
    outs = []
    for rank, v in VARIANTS:
        exe = os.path.join(BIN, "TurboFNO_%dD_%s" % (rank, v))
        cfg = os.path.join(PKG, "drivers", "benchmark_config", "problem_size_%dd.txt" % rank)
        deps = [src, os.path.join(PKG, "drivers", "driver_config.h")] + hdrs
        if force or _newer(exe, deps, extra=cfg):
            subprocess.check_call([
                "g++", "-std=c++17", "-O2", "-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include",
                "-DTFNO_RANK=%d" % rank, "-DTFNO_VARIANT=TFNO_VARIANT_%s" % v, '-DTFNO_TAG="%dD_%s"' % (rank, v),
                '-DDEFAULT_CONFIG_PATH="%s"' % cfg, src, "-o", exe,
                "-L" + PKG, "-lturbofno_b200", "-L/usr/local/cuda/lib64", "-lcudart",
                "-Wl,-rpath," + PKG, "-Wl,-rpath,/usr/local/cuda/lib64",
            ])
            _stamp(exe, deps, extra=cfg)
        outs.append(exe)
    # the example port of a reference-style driver (kernel tables of include/TurboFNO.h)
    port_src = os.path.join(PKG, "drivers", "compat_port.cu")
    port_exe = os.path.join(BIN, "compat_port")
    if force or _newer(port_exe, [port_src] + hdrs):
        subprocess.check_call([
            "nvcc", "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + os.path.join(ROOT, "include"),
            port_src, "-o", port_exe, "-L" + PKG, "-lturbofno_b200", "-Xlinker", "-rpath=" + PKG,
        ])
        _stamp(port_exe, [port_src] + hdrs)
    outs.append(port_exe)
    return outs


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_library(force=force, verbose="-v" in sys.argv))
    if "--drivers" in sys.argv:
        for e in build_drivers(force=force):
            print(e)

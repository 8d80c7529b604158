"""CPU tests of the host-side logic: the register-FFT arithmetic compiled for the host, the
shared-memory swizzles, and the C ABI surface (symbols, argument validation that needs no GPU)."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_fft64_arithmetic_on_host(tmp_path):
    exe = str(tmp_path / "fft64_host_check")
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-I/usr/local/cuda/include",
                           os.path.join(ROOT, "tests", "host", "fft64_host_check.cpp"), "-o", exe])
    out = subprocess.check_output([exe], text=True)
    vals = dict(line.split() for line in out.strip().splitlines())
    assert len(vals) == 9
    for name, err in vals.items():
        # |X| is O(sqrt(DY)) ~ 16..32 for unit-variance input; 2e-5 absolute is ~1e-6 relative
        assert float(err) < 2e-5, (name, err)


def _swz_chunk(row, c):
    x = ((((c >> 3) & 3) + ((row & 1) << 2)) ^ (((row >> 1) & 1) << 1)) & 7
    return (c & ~7) | ((c & 7) ^ x)


def test_tile_swizzle_is_a_bijection_and_conflict_free():
    # bijection per row
    for row in range(8):
        assert sorted(_swz_chunk(row, c) for c in range(32)) == list(range(32))
    # R=4 stores: the 8 lanes of a quarter-warp (2 adjacent rows x 4 lanes, chunk 8*r+i) hit 8 distinct bank groups
    for row0 in range(0, 8, 2):
        for i in range(8):
            banks = {_swz_chunk(row0 + g, 8 * r + i) & 7 for g in range(2) for r in range(4)}
            assert len(banks) == 8
    # column reads: 16 lanes = 4 columns x 4 rows (rows 4n+r) -> 16 distinct 8-byte slots
    for n in range(4):
        for q in range(16):
            slots = set()
            for kyl in range(4):
                ky = 4 * q + kyl
                for r in range(4):
                    row = 4 * n + r
                    slots.add((_swz_chunk(row, ky >> 1) & 7) * 2 + (ky & 1))
            assert len(slots) == 16


def _declared_symbols():
    hdr = open(os.path.join(ROOT, "include", "turbofno_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)      # declarations only, not prose
    return sorted(set(re.findall(r"\b(tfno_[a-z_A-Z0-9]+)\s*\(", hdr)))


def test_library_exports_every_declared_symbol():
    from turbofno_b200 import _lib

    lib = _lib.load()
    declared = _declared_symbols()
    assert declared, "no declarations parsed"
    assert sorted(_lib.SYMBOLS) == declared
    for name in declared:
        assert getattr(lib, name) is not None


def test_status_strings_and_problem_init():
    from turbofno_b200 import _lib

    lib = _lib.load()
    for s in range(0, 7):
        assert lib.tfno_status_string(s)
    p = _lib.Problem()
    assert lib.tfno_problem_init(ctypes.byref(p), 1) == _lib.OK
    assert (p.rank, p.modes, p.variant, p.alpha_re, p.scale_inverse) == (1, 64, _lib.VARIANT["D"], 1.0, 1)
    assert lib.tfno_problem_init(ctypes.byref(p), 3) == _lib.ERR_INVALID_ARG
    assert lib.tfno_problem_init(None, 1) == _lib.ERR_INVALID_ARG


def test_null_arguments_are_rejected_without_a_gpu():
    from turbofno_b200 import _lib

    lib = _lib.load()
    assert lib.tfno_create(None, 0) == _lib.ERR_INVALID_ARG
    assert lib.tfno_plan_create(None, None, None) == _lib.ERR_INVALID_ARG
    assert lib.tfno_exec(None, None, None, None, None, None) == _lib.ERR_INVALID_ARG
    assert lib.tfno_exec_host(None, None, None, None) == _lib.ERR_INVALID_ARG
    assert lib.tfno_cgemm(None, 64, 64, 8, None, None, None, 1, 0, 0, 0, None) == _lib.ERR_INVALID_ARG
    assert lib.tfno_workspace_bytes(None) == 0


def test_create_without_device_reports_cuda_error():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from turbofno_b200 import _lib

    h = ctypes.c_void_p()
    assert _lib.load().tfno_create(ctypes.byref(h), 0) == _lib.ERR_CUDA
    assert not h.value

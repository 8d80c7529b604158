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


def test_fft32_arithmetic_on_host(tmp_path):
    """The 32-point transform, the round-1 multiply-add exchange, the reduce-scatter rounds and the
    folded inverse of csrc/fft32.cuh (the arithmetic of the fused tensor-core kernel), lanes emulated."""
    exe = str(tmp_path / "fft32_host_check")
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-I/usr/local/cuda/include",
                           os.path.join(ROOT, "tests", "host", "fft32_host_check.cpp"), "-o", exe])
    out = subprocess.check_output([exe], text=True)
    vals = dict(line.split() for line in out.strip().splitlines())
    assert len(vals) == 14
    for name, err in vals.items():
        assert float(err) < 2e-5, (name, err)


GRID_1D = {"bs_list": [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 4096, 8192, 16384, 32768], "dimX_list": [1],
           "DY_list": [128, 256], "N_list": [64, 128], "K_list": list(range(8, 129, 8))}
GRID_2D = {"bs_list": [1] + list(range(8, 129, 8)), "DX_list": [128, 256], "DY_list": [128, 256], "N_list": [64, 128],
           "K_list": list(range(8, 129, 8))}


def _parse_grid_file(tmp_path, path):
    exe = str(tmp_path / "parse_config_check")
    if not os.path.exists(exe):
        subprocess.check_call(["g++", "-O1", "-std=c++17", os.path.join(ROOT, "tests", "host", "parse_config_check.cpp"), "-o", exe])
    out = subprocess.check_output([exe, path], text=True)
    grid = {}
    for line in out.strip().splitlines():
        tok = line.split()
        assert int(tok[1]) == len(tok) - 2
        grid[tok[0]] = [int(v) for v in tok[2:]]
    return grid


def test_driver_grid_parser(tmp_path):
    """parse_config (drivers/driver_config.h) on the grid-file format of the reference's
    benchmark_config/problem_size_{1d,2d}.txt: `key = v1 v2 ...`, comments, blank lines, CRLF, and a
    last line WITHOUT a newline, as the reference's files end.  15x1x2x2x16 and 17x2x2x2x16 grids."""
    for name, grid in (("1d", GRID_1D), ("2d", GRID_2D)):
        text = "\n".join("%s = %s" % (k, " ".join(str(v) for v in vals)) for k, vals in grid.items())    # no trailing newline
        f = tmp_path / ("as_reference_%s.txt" % name)
        f.write_bytes(text.encode())
        assert _parse_grid_file(tmp_path, str(f)) == grid
        # the package's own files: same lists plus comment lines
        own = os.path.join(ROOT, "turbofno_b200", "drivers", "benchmark_config", "problem_size_%s.txt" % name)
        assert _parse_grid_file(tmp_path, own) == grid
        n = 1
        for vals in grid.values():
            n *= len(vals)
        assert n == (15 * 1 * 2 * 2 * 16 if name == "1d" else 17 * 2 * 2 * 2 * 16)
    messy = tmp_path / "messy.txt"
    messy.write_bytes(b"# comment\r\n\r\nbs_list = 1 2\r\n\n   \nK_list = 8 trailing words 16\nN_list =\n")
    assert _parse_grid_file(tmp_path, str(messy)) == {"bs_list": [1, 2], "K_list": [8], "N_list": []}


def test_driver_grid_parser_on_reference_files(tmp_path):
    ref = os.environ.get("TFNO_REFERENCE")
    if not ref or not os.path.isdir(os.path.join(ref, "benchmark_config")):
        pytest.skip("TFNO_REFERENCE does not point at a reference tree")
    assert _parse_grid_file(tmp_path, os.path.join(ref, "benchmark_config", "problem_size_1d.txt")) == GRID_1D
    assert _parse_grid_file(tmp_path, os.path.join(ref, "benchmark_config", "problem_size_2d.txt")) == GRID_2D


def test_shape_checks_of_the_python_mirror():
    """The mirror refuses tensors whose shapes differ from the plan's before anything reaches the
    device (a wrong shape would make the kernels read or write out of bounds)."""
    from turbofno_b200 import api

    assert api.expected_shapes(1, "reference", 12, 8, 64, 128) == ((8, 12, 128), (64, 8), (64, 12, 128))
    assert api.expected_shapes(2, "batch_major", 3, 16, 64, 256, 128) == ((3, 16, 128, 256), (16, 64), (3, 64, 128, 256))
    api.check_shapes(1, "reference", 12, 8, 64, 128, None, (8, 12, 128), (64, 8), (64, 12, 128))
    for bad in (dict(x_shape=(8, 11, 128)), dict(x_shape=(12, 8, 128)), dict(w_shape=(8, 64)), dict(w_shape=(64, 16)),
                dict(y_shape=(64, 12, 256)), dict(y_shape=(128, 12, 128))):
        kw = dict(x_shape=(8, 12, 128), w_shape=(64, 8), y_shape=(64, 12, 128))
        kw.update(bad)
        with pytest.raises(ValueError):
            api.check_shapes(1, "reference", 12, 8, 64, 128, None, **kw)
    with pytest.raises(ValueError):
        api.check_shapes(2, "reference", 2, 8, 64, 128, 128, (8, 2, 128, 128), (64, 9), None)


def test_fused_kernel_shared_memory_layout_is_bank_conflict_free():
    """Address arithmetic of the fused kernel's 8-byte shared-memory accesses, replayed on the host:
    each half-warp must touch 32 distinct banks (ring reads / staging stores with the padded row
    stride, S stores with the padded SBO).  Mirrors Geometry<R> and s_sbo_fused in csrc/spectral_tc.cuh."""
    def half_warp_ok(addrs):
        for h in (addrs[:16], addrs[16:]):
            banks = set()
            for a in h:
                for wd in (a // 4, a // 4 + 1):
                    if wd % 32 in banks:
                        return False
                    banks.add(wd % 32)
        return True

    LBO = 144
    for R in (4, 8):
        DY, GPW = 32 * R, 32 // R
        CH = 4 * GPW
        row_stride = DY * 8 + 8 * R
        span = (2 * CH // 4) * LBO
        sbo = ((span + 63) // 64) * 64 + 16
        PER = 64 // R
        for i in range(32):
            assert half_warp_ok([(lane // R) * row_stride + (R * i + lane % R) * 8 for lane in range(32)])
        for wl in range(4):
            for j in range(PER):
                addrs = []
                for lane in range(32):
                    g, r = lane // R, lane % R
                    kl, m = wl * GPW + g, PER * r + j
                    addrs.append((kl >> 1) * LBO + (kl & 1) * 8 + (m >> 3) * sbo + (m & 7) * 16)
                assert half_warp_ok(addrs), (R, wl, j)


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
    for s in range(0, 9):
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
    assert lib.tfno_plan_kernels(None, None, 0) == _lib.ERR_INVALID_ARG
    assert lib.tfno_plan_set_host_chunk(None, 4) == _lib.ERR_INVALID_ARG


def test_create_without_device_reports_cuda_error():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from turbofno_b200 import _lib

    h = ctypes.c_void_p()
    assert _lib.load().tfno_create(ctypes.byref(h), 0) == _lib.ERR_CUDA
    assert not h.value

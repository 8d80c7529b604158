"""GPU tests of the driver surface: the ten TurboFNO_{1D,2D}_{A..E} executables, the source-level
port of a reference-style driver (kernel tables of include/TurboFNO.h), and the report of which
kernels a plan launches."""
import os
import re
import struct
import subprocess

import numpy as np
import pytest

from util import ROOT, assert_close, oracle_c, oracle_np, to_reference_layout, w_reference_layout

pytestmark = pytest.mark.gpu
BIN = os.path.join(ROOT, "turbofno_b200", "bin")

# the reference's output line (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:146,
# sample lines README.md:112-117): "1D_A, bs=1   , dimX=1   , DY=128 , N=64  , K=8   , TIME=   0.026ms"
LINE_1D = re.compile(r"^(1D_[A-E]), bs=(\d+) *, dimX=(\d+) *, DY=(\d+) *, N=(\d+) *, K=(\d+) *, TIME= *(\d+\.\d{3})ms$")
LINE_2D = re.compile(r"^(2D_[A-E]), bs=(\d+) *, DX=(\d+) *, DY=(\d+) *, N=(\d+) *, K=(\d+) *, TIME= *(\d+\.\d{3})ms$")


def test_reference_sample_line_matches_the_pattern():
    # README.md:112 of the reference
    assert LINE_1D.match("1D_A, bs=1   , dimX=1   , DY=128 , N=64  , K=8   , TIME=   0.026ms")


@pytest.mark.parametrize("exe,args,pattern", [
    ("TurboFNO_1D_A", ["1", "1", "128", "64", "8"], LINE_1D),
    ("TurboFNO_1D_D", ["4", "2", "256", "64", "16"], LINE_1D),
    ("TurboFNO_2D_E", ["1", "128", "128", "64", "8"], LINE_2D),
    ("TurboFNO_2D_D", ["2", "128", "256", "64", "16"], LINE_2D),
])
def test_executable_prints_the_reference_line(cuda, exe, args, pattern):
    out = subprocess.check_output([os.path.join(BIN, exe)] + args, text=True, timeout=300)
    lines = [l for l in out.splitlines() if l.strip()]
    assert len(lines) == 1, out
    m = pattern.match(lines[0])
    assert m, lines[0]
    assert m.group(1) == exe[len("TurboFNO_"):]                # the tag, "2D_E" included (the reference prints "1D_E" there)
    assert [int(v) for v in m.groups()[1:6]] == [int(a) for a in args]
    assert float(m.group(7)) > 0.0


def test_executable_sweeps_a_grid_file(cuda, tmp_path):
    grid = tmp_path / "grid.txt"
    grid.write_bytes(b"# two batches, two channel counts\nbs_list = 1 3\ndimX_list = 1\nDY_list = 128\nN_list = 64\nK_list = 8 16")
    out = subprocess.check_output([os.path.join(BIN, "TurboFNO_1D_C"), "--config", str(grid)], text=True, timeout=300)
    got = [LINE_1D.match(l) for l in out.splitlines() if l.strip()]
    assert all(got) and len(got) == 4
    assert [(int(m.group(2)), int(m.group(6))) for m in got] == [(1, 8), (1, 16), (3, 8), (3, 16)]   # bs outermost, K innermost


def test_source_port_of_a_reference_style_driver(cuda, tmp_path):
    """drivers/compat_port.cu calls the reference's kernel tables by their names and argument lists
    (fused_fft_cgemm_ifft[i](M,N,K,in,B,C,out,alpha,beta), fft_stride_DY[i], cgemm, ...); its four
    results (variants D, A, B, C) must equal the oracle's unnormalised layer."""
    for (bs, dimX, DY, N, K) in [(3, 2, 128, 64, 16), (5, 1, 256, 128, 24)]:
        x, w = oracle_np.make_inputs_1d(bs * dimX, K, N, DY, seed=bs + DY)
        fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
        with open(fin, "wb") as f:
            f.write(struct.pack("5i", bs, dimX, DY, N, K))
            f.write(to_reference_layout(x).tobytes())
            f.write(w_reference_layout(w).tobytes())
        out = subprocess.check_output([os.path.join(BIN, "compat_port"), str(fin), str(fout)], text=True, timeout=300)
        assert "compat_port" in out
        res = np.fromfile(fout, dtype=np.complex64).reshape(4, N, bs * dimX, DY)
        ref = oracle_c.spectral_conv_1d(x, w, scale=False)
        for i, variant in enumerate("DABC"):
            assert_close(np.swapaxes(res[i], 0, 1), ref, "ported driver, variant %s %s" % (variant, (bs, dimX, DY, N, K)))


def test_plan_reports_the_kernels_it_launches(cuda):
    """tfno_plan_kernels is a dry run of tfno_exec's own dispatch: these are the shapes whose tests
    claim a particular kernel, so a change of the eligibility rules shows up here."""
    import turbofno_b200 as t

    def kernels(rank, bs, DY, K, N, variant="D", **kw):
        plan = t.SpectralConv(rank, bs, DY, K, N, variant=variant, **kw)
        names = plan.kernels()
        plan.close()
        return names

    # fused tensor-core kernel: K a multiple of the chunk size up to 96, any chunk count
    assert kernels(1, 8192, 256, 64, 64) == ["spectral_tc_kernel<8,1>"]
    assert kernels(1, 300, 256, 48, 64) == ["spectral_tc_kernel<8,1>"]
    assert kernels(1, 300, 256, 96, 64) == ["spectral_tc_kernel<8,1>"]
    assert kernels(1, 3, 256, 16, 64) == ["spectral_tc_kernel<8,1>"]
    assert kernels(1, 300, 128, 32, 64) == ["spectral_tc_kernel<4,1>"]
    assert kernels(1, 300, 128, 64, 64, second_transform_forward=True) == ["spectral_tc_kernel<4,0>"]
    # wide layers: one launch per 64 output channels when the batch is large
    assert kernels(1, 300, 256, 32, 128) == ["spectral_tc_kernel<8,1>"] * 2
    # everything else: the FP32 row-tile kernel
    assert kernels(1, 1, 128, 8, 64) == ["spectral_tile_kernel<2,1,1,1>"]
    assert kernels(1, 5, 256, 32, 128) == ["spectral_tile_kernel<4,1,1,1>"]       # small batch: grid over blocks of 64 outputs
    assert kernels(1, 100, 256, 32, 128) == ["spectral_tile_kernel<4,1,1,2>"]     # 128 outputs per CTA
    assert kernels(1, 300, 256, 24, 64) == ["spectral_tc_kernel<8,1>"]                                 # 16 + 8 channels, padded chunk
    assert kernels(1, 100, 256, 24, 64) == ["spectral_tile_kernel<4,1,1,1>"]                           # ... not below a row per SM
    assert kernels(1, 300, 256, 128, 64) == ["spectral_tc_kernel<8,1>", "spectral_tc_kernel<8,1>+="]    # 64 + 64 channels
    assert kernels(1, 100, 256, 128, 64) == ["spectral_tile_kernel<4,1,1,1>"]                          # too few rows for two launches
    assert kernels(1, 300, 256, 200, 64) == ["spectral_tile_kernel<4,1,1,1>"]                          # more than two parts
    assert kernels(1, 3, 512, 128, 64) == ["spectral_tile_kernel<8,1,1,1>"]
    # long transforms run the fused tensor-core kernel too (chunks of 8 and 4 channels)
    assert kernels(1, 3, 512, 16, 64) == ["spectral_tc_kernel<16,1>"]
    assert kernels(1, 300, 1024, 24, 64) == ["spectral_tc_kernel<32,1>"]
    # variant A: transform, tensor-core contraction (N = 64, K % 16 == 0, beta = 0), transform
    assert kernels(1, 300, 256, 64, 64, "A") == ["fft_rows_trunc_kernel<4>", "cgemm_tc_kernel<128>", "ifft_rows_pad_kernel<4>"]
    assert kernels(1, 300, 256, 64, 64, "A", beta=1j)[1] == "spectral_tile_kernel<2,0,0,1>"
    # 2D variant D
    assert kernels(2, 16, 256, 32, 64, DX=256) == ["fft2d_trunc32_kernel<8,8>", "cgemm_tc_kernel<128>", "ifft2d_pad_kernel<4,4,paired,256>"]
    assert kernels(2, 16, 128, 32, 64, DX=256) == ["fft2d_trunc32_kernel<8,4>", "cgemm_tc_kernel<128>", "ifft2d_pad32_kernel<8,4,1>"]
    assert kernels(2, 1, 128, 8, 64, DX=128) == ["fft2d_trunc_kernel<2,2,paired,128>", "cgemm_tc_kernel<64>", "ifft2d_pad_kernel<2,2,paired,128>"]
    assert kernels(2, 8, 128, 104, 64, DX=128)[1:3] == ["cgemm_tc_kernel<128>", "cgemm_tc_kernel<128>+="]     # 64 + 40 channels
    assert kernels(2, 1, 128, 104, 64, DX=128)[1] == "spectral_tile_kernel<2,0,0,1>"                         # too few rows for two launches
    assert kernels(2, 8, 128, 72, 64, DX=128)[1] == "cgemm_tc_kernel<64>"                                    # 65..96 channels: 64-mode tiles
    # library path
    assert kernels(1, 4, 128, 8, 64, "E") == ["cufftExecC2C", "truncate_rows_kernel", "cublasCgemm", "zero_pad_rows_kernel", "cufftExecC2C"]

"""Pins the oracle (and the CUDA path) to the reference's own device code: the truncation,
zero-padding and cgemm kernels compiled from the reference sources into oracle/_ref/ by
oracle/Makefile, run around cuFFT in the reference's call order."""
import os
import subprocess

import numpy as np
import pytest

from util import ROOT, assert_close, oracle_c, oracle_np, to_reference_layout, w_reference_layout

pytestmark = pytest.mark.gpu
REF = os.path.join(ROOT, "oracle", "_ref")


def _harness(rank):
    exe = os.path.join(REF, "ref_harness_%dd" % rank)
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref not built (needs the reference tree at build time): make -C oracle ref")
    return exe


def _run(exe, tmp_path, x_ref_layout, w_ref_layout, out_shape, dims, gemm):
    xp, wp, yp = (str(tmp_path / n) for n in ("x.bin", "w.bin", "y.bin"))
    x_ref_layout.astype(np.complex64).tofile(xp)
    w_ref_layout.astype(np.complex64).tofile(wp)
    cmd = [exe, xp, wp, yp] + [str(d) for d in dims] + ([gemm] if gemm == "cublas" else [])
    subprocess.check_call(cmd)
    return np.fromfile(yp, dtype=np.complex64).reshape(out_shape)


@pytest.mark.parametrize("gemm", ["reference_cgemm", "cublas"])
@pytest.mark.parametrize("B,K,N,DY", [(1, 8, 64, 128), (6, 24, 128, 256)])
def test_reference_kernels_1d(cuda, tmp_path, gemm, B, K, N, DY):
    import torch
    import turbofno_b200 as t

    x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=41)
    y_ref = _run(_harness(1), tmp_path, to_reference_layout(x), w_reference_layout(w), (N, B, DY), (B, 1, DY, N, K), gemm)
    y_ref = np.swapaxes(y_ref, 0, 1)
    # the oracle agrees with the reference's kernels ...
    assert_close(y_ref, oracle_c.spectral_conv_1d(x, w), "reference kernels vs oracle (%s)" % gemm)
    # ... and so does the fused kernel, on identical inputs
    plan = t.SpectralConv(1, B, DY, K, N, variant="D")
    y = plan(torch.from_numpy(to_reference_layout(x)).to(cuda), torch.from_numpy(w_reference_layout(w)).to(cuda))
    torch.cuda.synchronize()
    assert_close(np.swapaxes(y.cpu().numpy(), 0, 1), y_ref, "fused kernel vs reference kernels (%s)" % gemm)
    plan.close()


@pytest.mark.parametrize("gemm", ["reference_cgemm", "cublas"])
def test_reference_kernels_2d(cuda, tmp_path, gemm):
    import torch
    import turbofno_b200 as t

    B, K, N, DX, DY = 2, 8, 64, 128, 256
    x, w = oracle_np.make_inputs_2d(B, K, N, DX, DY, seed=42)
    y_ref = _run(_harness(2), tmp_path, to_reference_layout(x), w_reference_layout(w), (N, B, DX, DY), (B, DX, DY, N, K), gemm)
    y_ref = np.swapaxes(y_ref, 0, 1)
    assert_close(y_ref, oracle_c.spectral_conv_2d(x, w), "reference 2D kernels vs oracle (%s)" % gemm)
    plan = t.SpectralConv(2, B, DY, K, N, DX=DX, variant="D")
    y = plan(torch.from_numpy(to_reference_layout(x)).to(cuda), torch.from_numpy(w_reference_layout(w)).to(cuda))
    torch.cuda.synchronize()
    assert_close(np.swapaxes(y.cpu().numpy(), 0, 1), y_ref, "2D kernels vs reference kernels (%s)" % gemm)
    plan.close()

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


def _run(exe, tmp_path, x_ref_layout, w_ref_layout, out_shape, dims, gemm, as_shipped=False):
    xp, wp, yp = (str(tmp_path / n) for n in ("x.bin", "w.bin", "y.bin"))
    x_ref_layout.astype(np.complex64).tofile(xp)
    w_ref_layout.astype(np.complex64).tofile(wp)
    cmd = [exe, xp, wp, yp] + [str(d) for d in dims] + ([gemm] if gemm == "cublas" else []) + (["as-shipped"] if as_shipped else [])
    subprocess.check_call(cmd)
    return np.fromfile(yp, dtype=np.complex64).reshape(out_shape)


@pytest.mark.parametrize("gemm", ["reference_cgemm", "cublas"])
@pytest.mark.parametrize("B,K,N,DY", [(1, 8, 64, 128), (6, 24, 128, 256), (150, 64, 64, 256), (40, 32, 64, 128)])
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
@pytest.mark.parametrize("B,K,N,DX,DY", [(2, 8, 64, 128, 256), (2, 16, 64, 256, 256)])
def test_reference_kernels_2d(cuda, tmp_path, gemm, B, K, N, DX, DY):
    import torch
    import turbofno_b200 as t

    x, w = oracle_np.make_inputs_2d(B, K, N, DX, DY, seed=42)
    y_ref = _run(_harness(2), tmp_path, to_reference_layout(x), w_reference_layout(w), (N, B, DX, DY), (B, DX, DY, N, K), gemm)
    y_ref = np.swapaxes(y_ref, 0, 1)
    assert_close(y_ref, oracle_c.spectral_conv_2d(x, w), "reference 2D kernels vs oracle (%s)" % gemm)
    plan = t.SpectralConv(2, B, DY, K, N, DX=DX, variant="D")
    y = plan(torch.from_numpy(to_reference_layout(x)).to(cuda), torch.from_numpy(w_reference_layout(w)).to(cuda))
    torch.cuda.synchronize()
    assert_close(np.swapaxes(y.cpu().numpy(), 0, 1), y_ref, "2D kernels vs reference kernels (%s)" % gemm)
    plan.close()


@pytest.mark.parametrize("gemm", ["reference_cgemm", "cublas"])
def test_as_shipped_arithmetic_against_the_reference_kernels(cuda, tmp_path, gemm):
    """What the reference drivers actually compute (alpha = 1-i, beta = -1+i on a zeroed C, second
    transform forward, unscaled; fusion_variants/1D_E_baseline/fused.cu:116,186-190): the
    reference's own kernels, the oracle and variants A-E of this library in that mode agree."""
    import torch
    import turbofno_b200 as t

    B, K, N, DY = 12, 16, 64, 256
    x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=43)
    y_ref = np.swapaxes(_run(_harness(1), tmp_path, to_reference_layout(x), w_reference_layout(w), (N, B, DY), (B, 1, DY, N, K), gemm,
                             as_shipped=True), 0, 1)
    assert_close(y_ref, oracle_c.spectral_conv_1d(x, w, alpha=1 - 1j, inverse=False, scale=False), "as shipped: reference kernels vs oracle")
    for v in "ABCDE":
        plan = t.SpectralConv(1, B, DY, K, N, variant=v, alpha=1 - 1j, beta=-1 + 1j, second_transform_forward=True, scale_inverse=False)
        ws = torch.zeros(max(plan.workspace_bytes, 16), dtype=torch.uint8, device=cuda)      # C starts at zero, as in the first repetition
        y = plan(torch.from_numpy(to_reference_layout(x)).to(cuda), torch.from_numpy(w_reference_layout(w)).to(cuda),
                 workspace=ws if plan.workspace_bytes else None)
        torch.cuda.synchronize()
        assert_close(np.swapaxes(y.cpu().numpy(), 0, 1), y_ref, "as shipped: variant %s vs reference kernels (%s)" % (v, gemm))
        plan.close()
    # 2D, variant E and D
    B, K, N, DX, DY = 2, 8, 64, 128, 128
    x, w = oracle_np.make_inputs_2d(B, K, N, DX, DY, seed=44)
    y_ref = np.swapaxes(_run(_harness(2), tmp_path, to_reference_layout(x), w_reference_layout(w), (N, B, DX, DY), (B, DX, DY, N, K), gemm,
                             as_shipped=True), 0, 1)
    for v in "DE":
        plan = t.SpectralConv(2, B, DY, K, N, DX=DX, variant=v, alpha=1 - 1j, beta=-1 + 1j, second_transform_forward=True, scale_inverse=False)
        ws = torch.zeros(plan.workspace_bytes, dtype=torch.uint8, device=cuda)
        y = plan(torch.from_numpy(to_reference_layout(x)).to(cuda), torch.from_numpy(w_reference_layout(w)).to(cuda), workspace=ws)
        torch.cuda.synchronize()
        assert_close(np.swapaxes(y.cpu().numpy(), 0, 1), y_ref, "as shipped 2D: variant %s vs reference kernels (%s)" % (v, gemm))
        plan.close()

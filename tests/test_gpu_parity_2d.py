"""GPU parity of the 2D spectral-convolution path against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest

from util import (assert_close, from_reference_layout, oracle_c, oracle_np, to_reference_layout,
                  w_reference_layout)

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def run_2d(cuda, x, w, variant="D", layout="reference", **kw):
    import torch
    import turbofno_b200 as t

    B, K, DX, DY = x.shape
    N = w.shape[1]
    plan = t.SpectralConv(2, B, DY, K, N, DX=DX, variant=variant, layout=layout, **kw)
    if layout == "reference":
        xd = torch.from_numpy(to_reference_layout(x)).to(cuda)
        wd = torch.from_numpy(w_reference_layout(w)).to(cuda)
    else:
        xd = torch.from_numpy(np.ascontiguousarray(x)).to(cuda)
        wd = torch.from_numpy(np.ascontiguousarray(w)).to(cuda)
    if plan.workspace_bytes:
        plan.workspace(cuda).zero_()
    y = plan(xd, wd)
    torch.cuda.synchronize()
    y = y.cpu().numpy()
    plan.close()
    return from_reference_layout(y) if layout == "reference" else y


@pytest.mark.parametrize("variant", list("ABCDE"))
@pytest.mark.parametrize("DX,DY", [(128, 128), (128, 256), (256, 128)])
def test_small_images_all_variants(cuda, variant, DX, DY):
    x, w = oracle_np.make_inputs_2d(2, 8, 64, DX, DY, seed=DX + DY)
    assert_close(run_2d(cuda, x, w, variant), oracle_c.spectral_conv_2d(x, w), "2D %dx%d variant %s" % (DX, DY, variant))


def test_golden_fixture_2d(cuda):
    g = np.load(os.path.join(GOLDEN, "c2_2d_bs1_k8_n64_128x256.npz"))
    assert_close(run_2d(cuda, g["x"], g["w"], "D")[:, ::8, ::8, ::8], g["y"], "golden 2D")


def test_config2(cuda):
    # BASELINE config 2: bs=16, K=32, N=64, 256x256
    x, w = oracle_np.make_inputs_2d(16, 32, 64, 256, 256)
    ref = oracle_c.spectral_conv_2d(x, w)
    d = run_2d(cuda, x, w, "D")
    assert_close(d, ref, "config 2 variant D vs oracle")
    e = run_2d(cuda, x, w, "E")
    assert_close(e, ref, "config 2 variant E vs oracle")
    assert_close(d, e, "config 2 D vs E")


def test_batch_major_layout_2d(cuda):
    x, w = oracle_np.make_inputs_2d(3, 16, 128, 128, 128, seed=2)
    ref = oracle_c.spectral_conv_2d(x, w)
    for v in "AD":
        assert_close(run_2d(cuda, x, w, v, layout="batch_major"), ref, "2D batch-major variant " + v)


def test_corner_truncation_on_gpu(cuda):
    DX = DY = 128
    ix, iy = np.meshgrid(np.arange(DX), np.arange(DY), indexing="ij")
    x = np.zeros((1, 8, DX, DY), np.complex64)
    x[0, 0] = np.exp(2j * np.pi * (5 * ix + 9 * iy) / 128)
    x[0, 1] = np.exp(2j * np.pi * (-5 * ix + 9 * iy) / 128)
    w = np.zeros((8, 64), np.complex64)
    w[0, 0] = 1
    w[1, 1] = 1
    y = run_2d(cuda, x, w, "D")
    assert np.abs(y[0, 0] - x[0, 0]).max() < 2e-5
    assert np.abs(y[0, 1]).max() < 2e-5


def test_as_shipped_second_transform_2d(cuda):
    x, w = oracle_np.make_inputs_2d(2, 8, 64, 128, 128, seed=6)
    a = 1.0 - 1.0j
    ref = oracle_c.spectral_conv_2d(x, w, alpha=a, inverse=False, scale=False)
    for v in "ABCDE":
        assert_close(run_2d(cuda, x, w, v, alpha=a, second_transform_forward=True, scale_inverse=False), ref, "2D as shipped " + v)


def test_config4_chain_full_size_sampled(cuda):
    # BASELINE config 4: bs=256, K=N=64, 256x256, four layers chained on two ping-pong buffers.
    # Batch items are independent through the whole chain, so the oracle runs the chain on two
    # batch items; the GPU runs it at full size.
    import torch
    import turbofno_b200 as t

    bs, C, D = 256, 64, 256
    g = torch.Generator(device=cuda).manual_seed(1234)
    a = torch.empty((C, bs, D, D), dtype=torch.complex64, device=cuda)
    for k in range(C):   # fill in slices to keep the temporary small
        a[k] = torch.view_as_complex(torch.rand((bs, D, D, 2), device=cuda, generator=g) * 2 - 1)
    b = torch.empty_like(a)
    ws = [torch.view_as_complex(torch.randn((C, C, 2), device=cuda, generator=g) / 8.0) for _ in range(4)]   # [N][K]
    sample = [0, 255]
    xs = a[:, sample].permute(1, 0, 2, 3).contiguous().cpu().numpy()
    plan = t.SpectralConv(2, bs, D, C, C, DX=D, variant="D")
    src, dst = a, b
    for l in range(4):
        plan(src, ws[l], y=dst)
        src, dst = dst, src
    torch.cuda.synchronize()
    got = src[:, sample].permute(1, 0, 2, 3).cpu().numpy()
    ref = xs
    for l in range(4):
        ref = oracle_c.spectral_conv_2d(ref.astype(np.complex64), ws[l].cpu().numpy().T.copy(), double=True)
    # four chained single-precision layers against a chain that rounds to complex64 between layers
    assert_close(got, ref, "config 4 chain", max_rel=1e-4, rel_l2=1e-5)
    plan.close()


@pytest.mark.parametrize("DX,DY", [(128, 128), (256, 256), (128, 256), (256, 128)])
def test_centered_x_modes(cuda, DX, DY):
    """Extension beyond the reference: X modes -32..31 instead of 0..63 (variant D, 2D)."""
    import torch
    import turbofno_b200 as t

    bs, K, N = 3, 16, 64
    x, w = oracle_np.make_inputs_2d(bs, K, N, DX, DY, seed=DX + DY)
    plan = t.SpectralConv(2, bs, DY, K, N, DX=DX, variant="D", x_modes_centered=True)
    y = plan(torch.from_numpy(to_reference_layout(x)).to(cuda), torch.from_numpy(w_reference_layout(w)).to(cuda))
    ref = oracle_np.spectral_conv_2d(x, w, x_modes_centered=True)
    assert_close(np.swapaxes(y.cpu().numpy(), 0, 1), ref, "centered X modes %dx%d" % (DX, DY))
    # and it is not the corner selection
    corner = oracle_np.spectral_conv_2d(x, w)
    assert np.abs(ref - corner).max() > 1e-2
    plan.close()
    # only the whole-image kernels of variant D know this mode set
    from turbofno_b200 import _lib
    with pytest.raises(t.TfnoError) as e:
        t.SpectralConv(2, bs, DY, K, N, DX=DX, variant="A", x_modes_centered=True)
    assert e.value.status == _lib.ERR_UNSUPPORTED


def test_variant_D_ignores_beta_on_an_uninitialised_workspace(cuda):
    """beta belongs to the variants that keep a spectrum C the caller can pre-load (A, B, C, E); the
    2D variant D uses C as scratch, so a non-zero beta must not mix whatever the workspace holds
    into the result (the 1D fused kernel has no C at all)."""
    import torch
    import turbofno_b200 as t

    bs, K, N, DX, DY = 2, 16, 64, 128, 128
    x, w = oracle_np.make_inputs_2d(bs, K, N, DX, DY, seed=5)
    ref = oracle_c.spectral_conv_2d(x, w)
    xd = torch.from_numpy(to_reference_layout(x)).to(cuda)
    wd = torch.from_numpy(w_reference_layout(w)).to(cuda)
    for beta in (0.0, -1.0 + 1.0j):
        plan = t.SpectralConv(2, bs, DY, K, N, DX=DX, variant="D", beta=beta)
        ws = torch.full((plan.workspace_bytes // 4,), float("nan"), dtype=torch.float32, device=cuda).view(torch.uint8)
        y = plan(xd, wd, workspace=ws)
        torch.cuda.synchronize()
        assert_close(from_reference_layout(y.cpu().numpy()), ref, "2D variant D, beta=%s, NaN workspace" % (beta,))
        plan.close()

"""GPU tests of per-mode weights W[k, n, m] (the contraction an FNO layer trains; the reference
shares one K x N matrix between all modes): transform, per-mode contraction, transform, against
the numpy oracle, in one and two dimensions and through the host-buffer path."""
import numpy as np
import pytest

from util import assert_close, from_reference_layout, oracle_np, to_reference_layout

pytestmark = pytest.mark.gpu


def _w_ref(w):
    """logical w[K, N, modes...] -> reference order [N, K, modes...] (k faster than n, modes fastest)."""
    return np.ascontiguousarray(np.swapaxes(w, 0, 1))


@pytest.mark.parametrize("variant", ["A", "D"])
@pytest.mark.parametrize("B,K,N,DY", [(5, 8, 64, 128), (70, 24, 128, 256), (33, 64, 64, 512)])
def test_per_mode_weights_1d(cuda, variant, B, K, N, DY):
    import torch
    import turbofno_b200 as t

    x, _ = oracle_np.make_inputs_1d(B, K, N, DY, seed=B + K)
    w = oracle_np.make_per_mode_weights(K, N, (64,), wseed=7 + K)
    plan = t.SpectralConv(1, B, DY, K, N, variant=variant, per_mode_weights=True, alpha=0.5 - 0.25j)
    assert plan.kernels() == ["fft_rows_trunc_kernel<%d>" % (DY // 64), "cgemm_permode_kernel", "ifft_rows_pad_kernel<%d>" % (DY // 64)]
    y = plan(torch.from_numpy(to_reference_layout(x)).to(cuda), torch.from_numpy(_w_ref(w)).to(cuda))
    torch.cuda.synchronize()
    assert_close(from_reference_layout(y.cpu().numpy()), oracle_np.spectral_conv_1d(x, w, alpha=0.5 - 0.25j), "per-mode weights 1D")
    plan.close()


def test_per_mode_weights_equal_shared_weights_when_constant_over_modes(cuda):
    import torch
    import turbofno_b200 as t

    B, K, N, DY = 40, 32, 64, 256
    x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=3)
    wm = np.repeat(w[:, :, None], 64, axis=2)
    xd = torch.from_numpy(to_reference_layout(x)).to(cuda)
    shared = t.SpectralConv(1, B, DY, K, N, variant="A")
    per = t.SpectralConv(1, B, DY, K, N, variant="A", per_mode_weights=True)
    ys = shared(xd, torch.from_numpy(np.ascontiguousarray(w.T)).to(cuda))
    yp = per(xd, torch.from_numpy(_w_ref(wm)).to(cuda))
    torch.cuda.synchronize()
    assert_close(yp.cpu().numpy(), ys.cpu().numpy(), "per-mode with mode-independent weights vs shared weights")
    shared.close(); per.close()


def test_per_mode_weights_batch_major_layout_and_host_path(cuda):
    import torch
    import turbofno_b200 as t

    B, K, N, DY = 21, 16, 64, 128
    x, _ = oracle_np.make_inputs_1d(B, K, N, DY, seed=9)
    w = oracle_np.make_per_mode_weights(K, N, (64,), wseed=10)
    ref = oracle_np.spectral_conv_1d(x, w)
    plan = t.SpectralConv(1, B, DY, K, N, variant="D", per_mode_weights=True, layout="batch_major")
    y = plan(torch.from_numpy(np.ascontiguousarray(x)).to(cuda), torch.from_numpy(np.ascontiguousarray(w)).to(cuda))
    torch.cuda.synchronize()
    assert_close(y.cpu().numpy(), ref, "per-mode weights, batch-major layout")
    plan.close()
    plan = t.SpectralConv(1, B, DY, K, N, variant="D", per_mode_weights=True)
    plan.set_host_chunk(8)
    yh = torch.empty((N, B, DY), dtype=torch.complex64).pin_memory()
    plan.exec_host(torch.from_numpy(to_reference_layout(x)).pin_memory(), torch.from_numpy(_w_ref(w)).pin_memory(), yh)
    assert_close(from_reference_layout(yh.numpy()), ref, "per-mode weights, host path in chunks")
    plan.close()


@pytest.mark.parametrize("bs,K,N,DX,DY", [(3, 8, 64, 128, 128), (2, 16, 64, 256, 128)])
def test_per_mode_weights_2d(cuda, bs, K, N, DX, DY):
    import torch
    import turbofno_b200 as t

    x, _ = oracle_np.make_inputs_2d(bs, K, N, DX, DY, seed=bs)
    w = oracle_np.make_per_mode_weights(K, N, (64, 64), wseed=12)
    plan = t.SpectralConv(2, bs, DY, K, N, DX=DX, variant="D", per_mode_weights=True)
    assert plan.kernels()[1] == "cgemm_permode_kernel"
    y = plan(torch.from_numpy(to_reference_layout(x)).to(cuda), torch.from_numpy(_w_ref(w)).to(cuda))
    torch.cuda.synchronize()
    assert_close(from_reference_layout(y.cpu().numpy()), oracle_np.spectral_conv_2d(x, w), "per-mode weights 2D")
    plan.close()


def test_per_mode_weights_unsupported_combinations(cuda):
    import turbofno_b200 as t

    for kw in (dict(variant="B"), dict(variant="E"), dict(variant="D", beta=1.0)):
        with pytest.raises(t.TfnoError):
            t.SpectralConv(1, 4, 128, 8, 64, per_mode_weights=True, **kw)
    with pytest.raises(t.TfnoError):
        t.SpectralConv(2, 2, 128, 8, 64, DX=128, variant="A", per_mode_weights=True)

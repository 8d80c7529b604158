"""GPU parity of the 1D spectral-convolution path against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest

from util import (assert_close, from_reference_layout, oracle_c, oracle_np, to_reference_layout,
                  w_reference_layout)

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def run_1d(cuda, x, w, variant="D", layout="reference", dimX=1, **kw):
    """x logical [B,K,DY] complex64, w logical [K,N]; returns logical y [B,N,DY] (numpy)."""
    import torch
    import turbofno_b200 as t

    B, K, DY = x.shape
    N = w.shape[1]
    assert B % dimX == 0
    plan = t.SpectralConv(1, B // dimX, DY, K, N, dimX=dimX, variant=variant, layout=layout, **kw)
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
def test_config0_all_variants(cuda, variant):
    # BASELINE config 0: bs=1, dimX=1, DY=128, K=8, N=64
    x, w = oracle_np.make_inputs_1d(1, 8, 64, 128)
    ref = oracle_c.spectral_conv_1d(x, w)
    assert_close(run_1d(cuda, x, w, variant), ref, "config0 variant " + variant)


def test_config0_golden_fixture(cuda):
    g = np.load(os.path.join(GOLDEN, "c0_1d_bs1_dy128_k8_n64.npz"))
    assert_close(run_1d(cuda, g["x"], g["w"], "D"), g["y"], "golden config0")
    g = np.load(os.path.join(GOLDEN, "c1_1d_bs4_dy256_k24_n128.npz"))
    assert_close(run_1d(cuda, g["x"], g["w"], "D")[:, ::8, :], g["y"], "golden sweep point")


def test_fused_matches_library_variant_E(cuda):
    # acceptance as BASELINE states it: fused kernel vs the cuFFT+cuBLAS pipeline on identical inputs
    for (B, K, N, DY) in [(1, 8, 64, 128), (16, 32, 128, 256), (64, 64, 64, 256)]:
        x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=B + K)
        assert_close(run_1d(cuda, x, w, "D"), run_1d(cuda, x, w, "E"), "D vs E %s" % ((B, K, N, DY),))


SWEEP = [(bs, DY, N, K) for bs in (1, 2, 4, 8, 16, 32, 64) for DY in (128, 256) for N in (64, 128) for K in (8, 16, 24, 32)]


def test_config1_sweep_fused(cuda):
    # BASELINE config 1: the 112-point 1D grid, variant D against the double-precision oracle
    assert len(SWEEP) == 112
    worst = (0.0, 0.0)
    for i, (bs, DY, N, K) in enumerate(SWEEP):
        x, w = oracle_np.make_inputs_1d(bs, K, N, DY, seed=100 + i, wseed=900 + i)
        mr, l2 = assert_close(run_1d(cuda, x, w, "D"), oracle_c.spectral_conv_1d(x, w), "sweep %s" % ((bs, DY, N, K),))
        worst = (max(worst[0], mr), max(worst[1], l2))
    print("sweep worst max_rel=%.3e rel_l2=%.3e" % worst)


@pytest.mark.parametrize("variant", list("ABCE"))
def test_sweep_subset_other_variants(cuda, variant):
    for i, (bs, DY, N, K) in enumerate(SWEEP[::9]):
        x, w = oracle_np.make_inputs_1d(bs, K, N, DY, seed=300 + i)
        assert_close(run_1d(cuda, x, w, variant), oracle_c.spectral_conv_1d(x, w), "variant %s %s" % (variant, (bs, DY, N, K)))


def test_batch_major_layout_holds_same_tensor(cuda):
    x, w = oracle_np.make_inputs_1d(6, 16, 128, 256, seed=5)
    ref = oracle_c.spectral_conv_1d(x, w)
    a = run_1d(cuda, x, w, "D", layout="reference")
    b = run_1d(cuda, x, w, "D", layout="batch_major")
    assert_close(a, ref, "reference layout")
    assert_close(b, ref, "batch-major layout")
    for v in "ABC":
        assert_close(run_1d(cuda, x, w, v, layout="batch_major"), ref, "batch-major variant " + v)


def test_dimX_rows(cuda):
    # dimX > 1: bs*dimX independent rows (reference M = bs*dimX*64)
    x, w = oracle_np.make_inputs_1d(12, 8, 64, 128, seed=8)
    assert_close(run_1d(cuda, x, w, "D", dimX=4), oracle_c.spectral_conv_1d(x, w), "dimX=4")


@pytest.mark.parametrize("DY", [512, 1024])
def test_long_transforms(cuda, DY):
    x, w = oracle_np.make_inputs_1d(3, 16, 64, DY, seed=DY)
    ref = oracle_c.spectral_conv_1d(x, w)
    for v in "AD":
        assert_close(run_1d(cuda, x, w, v), ref, "DY=%d variant %s" % (DY, v))


def test_wide_channels(cuda):
    # K and N beyond one accumulator block / one launch: K=128, N=192
    x, w = oracle_np.make_inputs_1d(5, 128, 192, 128, seed=77)
    ref = oracle_c.spectral_conv_1d(x, w)
    for v in "ABCD":
        assert_close(run_1d(cuda, x, w, v), ref, "K=128 N=192 variant " + v)


@pytest.mark.parametrize("DY,K", [(256, 16), (256, 32), (256, 48), (256, 64), (256, 96), (128, 32), (128, 64), (128, 96),
                                  (512, 8), (512, 40), (512, 64), (1024, 24), (1024, 64),
                                  # a last chunk with fewer channels than the chunk size (16 at DY=256, 32 at DY=128)
                                  (256, 8), (256, 24), (256, 40), (256, 88), (128, 8), (128, 24), (128, 56), (128, 88)])
def test_fused_kernel_chunk_counts_many_rows_per_sm(cuda, DY, K):
    """One to sixteen chunks of channels per row, even and odd counts, full and partial last chunks,
    at every transform length of the fused tensor-core kernel, with three to four rows per SM so
    that every ring stage, S buffer and accumulator buffer is reused."""
    import turbofno_b200 as t

    probe = t.SpectralConv(1, 449, DY, K, 64, variant="D")
    assert probe.kernels() == ["spectral_tc_kernel<%d,1>" % (DY // 32)]
    probe.close()
    B, N = 449, 64
    x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=DY + K)
    assert_close(run_1d(cuda, x, w, "D"), oracle_c.spectral_conv_1d(x, w), "fused, %d channels at DY=%d" % (K, DY))


@pytest.mark.parametrize("DY,K,N", [(256, 128, 64), (256, 112, 64), (128, 128, 64), (128, 192, 64), (512, 104, 64), (1024, 104, 64),
                                    (256, 128, 128), (256, 104, 64), (256, 120, 64), (128, 104, 64), (128, 136, 64)])
def test_more_than_96_channels_run_the_fused_kernel_in_two_accumulating_launches(cuda, DY, K, N):
    """The weights of at most 96 channels fit tensor memory; up to 192 channels are split into two
    launches, the second adding to the first's output through the copy engine (or, at DY=128, in
    registers).  The output buffer is pre-filled with NaN: the first launch must overwrite it."""
    import torch
    import turbofno_b200 as t

    B = 449
    plan = t.SpectralConv(1, B, DY, K, N, variant="D")
    name = "spectral_tc_kernel<%d,1>" % (DY // 32)
    assert plan.kernels() == [name, name + "+="] * (N // 64)
    x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=DY + K)
    xt = torch.from_numpy(np.ascontiguousarray(np.swapaxes(x, 0, 1))).to(cuda)
    wt = torch.from_numpy(np.ascontiguousarray(w.T)).to(cuda)
    y = torch.full((N, B, DY), float("nan"), dtype=torch.complex64, device=cuda)
    plan(xt, wt, y=y)
    plan.close()
    assert_close(np.swapaxes(y.cpu().numpy(), 0, 1), oracle_c.spectral_conv_1d(x, w), "%d channels at DY=%d" % (K, DY))


def test_wide_layer_runs_the_fused_kernel_per_block_of_64_outputs(cuda):
    # N = 128 and 192 with enough rows for the tensor-core kernel (two rows per SM and more)
    for (B, K, N, DY) in [(300, 32, 128, 256), (300, 64, 192, 128)]:
        x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=N + DY)
        assert_close(run_1d(cuda, x, w, "D"), oracle_c.spectral_conv_1d(x, w), "wide layer %s" % ((B, K, N, DY),))


def test_alpha_and_as_shipped_second_transform(cuda):
    x, w = oracle_np.make_inputs_1d(4, 16, 64, 256, seed=3)
    a = 1.0 - 1.0j
    ref = oracle_c.spectral_conv_1d(x, w, alpha=a, inverse=False, scale=False)
    for v in "ABCDE":
        got = run_1d(cuda, x, w, v, alpha=a, second_transform_forward=True, scale_inverse=False)
        assert_close(got, ref, "as-shipped second transform, variant " + v)


def test_beta_accumulates_on_workspace_C(cuda):
    # C = alpha*A*W + beta*C_old on the compact spectrum (variants with a materialised C)
    import torch
    import turbofno_b200 as t

    B, K, N, DY = 4, 16, 64, 128
    x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=21)
    alpha, beta = 0.75 + 0.5j, -1.0 + 1.0j
    rng = np.random.default_rng(9)
    c_old = (rng.standard_normal((B, N, 64)) + 1j * rng.standard_normal((B, N, 64))).astype(np.complex64)
    spec = oracle_np.cgemm_modes(oracle_np.spectrum_1d(x), w, alpha=alpha, beta=beta, c=c_old)
    ref = oracle_np.ifft_pad_1d(spec, DY)
    for v in "AB":
        plan = t.SpectralConv(1, B, DY, K, N, variant=v, alpha=alpha, beta=beta)
        ws = torch.zeros(plan.workspace_bytes, dtype=torch.uint8, device=cuda)
        # C sits after A (variant A) or first (variant B); both 256-byte aligned
        offC = ((K * B * 64 * 8 + 255) // 256) * 256 if v == "A" else 0
        cview = ws[offC:offC + N * B * 64 * 8].view(torch.complex64).view(N, B, 64)
        cview.copy_(torch.from_numpy(to_reference_layout(c_old)).to(cuda))
        y = plan(torch.from_numpy(to_reference_layout(x)).to(cuda), torch.from_numpy(w_reference_layout(w)).to(cuda), workspace=ws)
        torch.cuda.synchronize()
        assert_close(from_reference_layout(y.cpu().numpy()), ref, "beta, variant " + v)
        plan.close()


def test_known_answers_on_gpu(cuda):
    DY, K, N = 256, 8, 64
    j = np.arange(DY)
    # single exponentials: mode 63 passes, mode 64 is removed exactly
    x = np.zeros((2, K, DY), np.complex64)
    x[0, 2] = np.exp(2j * np.pi * 63 * j / DY)
    x[1, 2] = np.exp(2j * np.pi * 64 * j / DY)
    w = np.zeros((K, N), np.complex64)
    w[2, 7] = 2.0
    y = run_1d(cuda, x, w, "D")
    assert np.abs(y[0, 7] - 2.0 * x[0, 2]).max() < 2e-5
    assert np.abs(y[1]).max() < 2e-5
    assert np.abs(np.delete(y[0], 7, axis=0)).max() < 2e-5
    # delta input -> Dirichlet kernel of the 64 kept modes
    x = np.zeros((1, K, DY), np.complex64)
    x[0, 0, 0] = 1.0
    w = np.zeros((K, N), np.complex64)
    w[0, :] = 1.0
    y = run_1d(cuda, x, w, "D")
    expect = np.exp(2j * np.pi * np.outer(np.arange(64), j) / DY).sum(0) / DY
    assert np.abs(y[0, 5] - expect).max() < 1e-6
    # identity weights: low-pass of the input
    x, _ = oracle_np.make_inputs_1d(3, 64, 64, 128, seed=4)
    y = run_1d(cuda, x, np.eye(64, dtype=np.complex64), "D")
    X = np.fft.fft(x.astype(np.complex128), axis=-1)
    X[..., 64:] = 0
    assert_close(y, np.fft.ifft(X, axis=-1), "identity weights")


def test_deterministic_and_confined_to_output(cuda):
    # same launch twice -> bit-identical (no shared-memory race); canaries around y untouched
    import torch
    import turbofno_b200 as t

    B, K, N, DY = 37, 32, 128, 256
    x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=11)
    xd = torch.from_numpy(to_reference_layout(x)).to(cuda)
    wd = torch.from_numpy(w_reference_layout(w)).to(cuda)
    plan = t.SpectralConv(1, B, DY, K, N, variant="D")
    pad = 4096
    buf = torch.full((N * B * DY + 2 * pad,), complex(7.0, -7.0), dtype=torch.complex64, device=cuda)
    y1 = buf[pad:pad + N * B * DY].view(N, B, DY)
    plan(xd, wd, y=y1)
    first = y1.clone()
    plan(xd, wd, y=y1)
    torch.cuda.synchronize()
    assert torch.equal(first.view(torch.float32), y1.view(torch.float32))
    assert bool((buf[:pad] == complex(7.0, -7.0)).all()) and bool((buf[-pad:] == complex(7.0, -7.0)).all())
    assert_close(from_reference_layout(y1.cpu().numpy()), oracle_c.spectral_conv_1d(x, w), "odd batch 37")
    plan.close()


def test_config3_full_size_rows_against_oracle(cuda):
    # BASELINE config 3 at full size: bs=8192, DY=256, K=N=64.  Rows are independent, so the CPU
    # oracle is run on a sample of rows; the whole output is checked fused-vs-library (D vs E).
    import torch
    import turbofno_b200 as t

    B, K, N, DY = 8192, 64, 64, 256
    g = torch.Generator(device=cuda).manual_seed(1234)
    xd = torch.view_as_complex(torch.rand((K, B, DY, 2), device=cuda, generator=g) * 2 - 1)
    wd = torch.view_as_complex(torch.randn((N, K, 2), device=cuda, generator=g) / np.sqrt(K))
    pd, pe = t.SpectralConv(1, B, DY, K, N, variant="D"), t.SpectralConv(1, B, DY, K, N, variant="E")
    yd, ye = pd(xd, wd), pe(xd, wd)
    torch.cuda.synchronize()
    diff = (yd - ye).abs()
    max_rel = float(diff.max() / ye.abs().max())
    rel_l2 = float(torch.linalg.vector_norm(diff) / torch.linalg.vector_norm(ye))
    assert max_rel <= 1e-4 and rel_l2 <= 1e-5, (max_rel, rel_l2)
    rows = [0, 1, 147, 148, 4095, 8191]
    xs = xd[:, rows, :].permute(1, 0, 2).contiguous().cpu().numpy()
    ref = oracle_c.spectral_conv_1d(xs, wd.cpu().numpy().T.copy())
    assert_close(yd[:, rows, :].permute(1, 0, 2).cpu().numpy(), ref, "config 3 sampled rows")
    # linearity at full size: layer(2x) == 2*layer(x) up to rounding
    y2 = pd((xd * 2).contiguous(), wd)
    torch.cuda.synchronize()
    assert float((y2 - 2 * yd).abs().max() / yd.abs().max()) < 1e-6
    pd.close(); pe.close()


def test_exec_host_matches_device_path(cuda):
    import torch
    import turbofno_b200 as t

    B, K, N, DY = 300, 32, 64, 256
    x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=31)
    xh = torch.from_numpy(to_reference_layout(x)).pin_memory()
    wh = torch.from_numpy(w_reference_layout(w)).pin_memory()
    yh = torch.empty((N, B, DY), dtype=torch.complex64).pin_memory()
    plan = t.SpectralConv(1, B, DY, K, N, variant="D")
    plan.exec_host(xh, wh, yh)
    assert_close(from_reference_layout(yh.numpy()), oracle_c.spectral_conv_1d(x, w), "exec_host")
    plan.close()


def test_invalid_arguments_return_status_codes(cuda):
    import torch
    import turbofno_b200 as t
    from turbofno_b200 import _lib

    for kw, code in [(dict(K=12), _lib.ERR_UNSUPPORTED), (dict(N=96), _lib.ERR_UNSUPPORTED),
                     (dict(DY=192), _lib.ERR_UNSUPPORTED), (dict(DY=64), _lib.ERR_UNSUPPORTED),
                     (dict(modes=32), _lib.ERR_UNSUPPORTED), (dict(bs=0), _lib.ERR_INVALID_ARG)]:
        args = dict(bs=2, DY=128, K=8, N=64)
        args.update(kw)
        with pytest.raises(t.TfnoError) as e:
            t.SpectralConv(1, args.pop("bs"), args.pop("DY"), args.pop("K"), args.pop("N"), **args)
        assert e.value.status == code
    plan = t.SpectralConv(1, 2, 128, 8, 64, variant="A")
    x = torch.zeros((8, 2, 128), dtype=torch.complex64, device=cuda)
    w = torch.zeros((64, 8), dtype=torch.complex64, device=cuda)
    y = torch.zeros((64, 2, 128), dtype=torch.complex64, device=cuda)
    lib, vp = plan.lib, __import__("ctypes").c_void_p
    assert lib.tfno_exec(plan._plan, vp(x.data_ptr()), vp(w.data_ptr()), vp(y.data_ptr()), None, None) == _lib.ERR_WORKSPACE
    assert lib.tfno_exec(plan._plan, vp(x.data_ptr() + 8), vp(w.data_ptr()), vp(y.data_ptr()), None, None) == _lib.ERR_INVALID_ARG
    assert lib.tfno_exec(plan._plan, None, vp(w.data_ptr()), vp(y.data_ptr()), None, None) == _lib.ERR_INVALID_ARG
    plan.close()
    # the context is still healthy
    assert float(torch.ones(4, device=cuda).sum()) == 4.0

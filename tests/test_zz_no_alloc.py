"""The allocation-free 2D entry point (tfno_spectral_conv2d_static) against the regular plan/exec
path, through the C ABI.

Callers that may not allocate device memory when a layer runs (arena-owned devices, rules against
allocation after start-up, plug-ins invoked between another allocator's operations) use this
entry point; its scratch is a fixed array inside the library.  The file name makes pytest collect
it last, so a failure here cannot hide the result of any other test in a run that stops at the
first failure.
"""
import ctypes

import numpy as np
import pytest

from util import assert_close, oracle_c, oracle_np, to_reference_layout, w_reference_layout

pytestmark = pytest.mark.gpu


def test_static_scratch_layer_matches_plan_path_twice_in_a_row(cuda):
    import torch
    import turbofno_b200 as t

    # BASELINE config 2 sized down in batch: 4 x 32 -> 64 channels of 256 x 256
    bs, K, N, DX, DY = 4, 32, 64, 256, 256
    x, w = oracle_np.make_inputs_2d(bs, K, N, DX, DY, seed=77)
    xd = torch.from_numpy(to_reference_layout(x)).to(cuda)
    wd = torch.from_numpy(w_reference_layout(w)).to(cuda)
    plan = t.SpectralConv(2, bs, DY, K, N, DX=DX, variant="D")
    expected = plan(xd, wd).clone()
    torch.cuda.synchronize()
    # two calls in a row share the one scratch array and must both be right
    first = t.spectral_conv2d_static(xd, wd)
    # second call on different data in between would leave other spectra in the array
    x2, _ = oracle_np.make_inputs_2d(bs, K, N, DX, DY, seed=78)
    other = t.spectral_conv2d_static(torch.from_numpy(to_reference_layout(x2)).to(cuda), wd)
    second = t.spectral_conv2d_static(xd, wd)
    torch.cuda.synchronize()
    # Same image kernels; the contraction runs on the FP32 kernel here and on the tensor cores in
    # the plan (K = 32, N = 64), so the two agree to rounding: the tolerance of the parity tests.
    assert "cgemm_tc_kernel" in ",".join(plan.kernels())
    assert_close(first.cpu().numpy(), expected.cpu().numpy(), "static entry point, first call")
    assert_close(second.cpu().numpy(), expected.cpu().numpy(), "static entry point, second call")
    assert torch.equal(first.view(torch.float32), second.view(torch.float32))
    assert not torch.equal(other.view(torch.float32), first.view(torch.float32))
    # and against the CPU oracle on one batch item
    ref = oracle_c.spectral_conv_2d(x[:1], w)
    assert_close(np.swapaxes(first[:, :1].cpu().numpy(), 0, 1), ref, "static entry point vs oracle")
    plan.close()


def test_static_scratch_limit_and_bad_arguments(cuda):
    import torch
    import turbofno_b200 as t
    from turbofno_b200 import _lib

    lib = _lib.load()
    limit = lib.tfno_static_scratch_bytes()
    assert limit == 64 << 20
    vp = ctypes.c_void_p
    buf = torch.zeros(1024, dtype=torch.complex64, device=cuda)
    p = vp(buf.data_ptr())
    # 8*4096*bs*(K+N) = 8*4096*32*128 = 128 MiB > 64 MiB: refused before anything is launched
    assert lib.tfno_spectral_conv2d_static(32, 256, 256, 64, 64, p, p, p, 1.0, 0.0, None) == _lib.ERR_SCRATCH_LIMIT
    assert lib.tfno_spectral_conv2d_static(1, 512, 256, 8, 64, p, p, p, 1.0, 0.0, None) == _lib.ERR_UNSUPPORTED
    assert lib.tfno_spectral_conv2d_static(1, 256, 256, 12, 64, p, p, p, 1.0, 0.0, None) == _lib.ERR_UNSUPPORTED
    assert lib.tfno_spectral_conv2d_static(1, 256, 256, 8, 64, None, p, p, 1.0, 0.0, None) == _lib.ERR_INVALID_ARG
    assert lib.tfno_spectral_conv2d_static(1, 256, 256, 8, 64, vp(buf.data_ptr() + 8), p, p, 1.0, 0.0, None) == _lib.ERR_INVALID_ARG
    # sizes whose byte count does not fit 64 bits must be refused too, not wrap around and pass
    assert lib.tfno_spectral_conv2d_static(1 << 58, 256, 256, 64, 64, p, p, p, 1.0, 0.0, None) == _lib.ERR_SCRATCH_LIMIT
    assert lib.tfno_spectral_conv2d_static((1 << 49) + 1, 256, 256, 8, 64, p, p, p, 1.0, 0.0, None) == _lib.ERR_SCRATCH_LIMIT
    # a K that the contraction's shared memory cannot hold is refused before the first launch
    assert lib.tfno_spectral_conv2d_static(1, 128, 128, 512, 64, p, p, p, 1.0, 0.0, None) in (_lib.ERR_UNSUPPORTED, _lib.ERR_SCRATCH_LIMIT)
    assert float(torch.ones(4, device=cuda).sum()) == 4.0

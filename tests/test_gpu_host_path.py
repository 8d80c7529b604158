"""GPU tests of the host-buffer entry point (tfno_exec_host): the batch is cut into chunks that are
copied in, transformed and copied out on two alternating streams.  A chunk-size override makes small
problems take several chunks plus a shorter last one; every output element is compared."""
import numpy as np
import pytest

from util import (assert_close, from_reference_layout, oracle_c, oracle_np, to_reference_layout,
                  w_reference_layout)

pytestmark = pytest.mark.gpu


def _host_run(t, plan, x, w, out_shape):
    import torch

    xh = torch.from_numpy(to_reference_layout(x)).pin_memory()
    wh = torch.from_numpy(w_reference_layout(w)).pin_memory()
    yh = torch.full(out_shape, complex(float("nan"), float("nan")), dtype=torch.complex64).pin_memory()
    plan.exec_host(xh, wh, yh)
    got = yh.numpy().copy()
    assert np.isfinite(got.view(np.float32)).all(), "an output element was never written"
    # a second call reuses the staging (slots, streams, per-stream weights) and must give the same bits
    yh.fill_(complex(float("nan"), float("nan")))
    plan.exec_host(xh, wh, yh)
    assert np.array_equal(got.view(np.float32), yh.numpy().view(np.float32))
    assert t.Handle.get(0).device_status == 0
    return got


@pytest.mark.parametrize("bs,dimX,chunk", [(23, 1, 4), (10, 3, 3), (8, 2, 8), (7, 1, 1)])
def test_exec_host_1d_in_several_chunks(cuda, bs, dimX, chunk):
    """5 chunks + tail of 3; dimX > 1 with 3 chunks + tail of 1; a single chunk; one item per chunk."""
    import turbofno_b200 as t

    K, N, DY = 16, 64, 256
    x, w = oracle_np.make_inputs_1d(bs * dimX, K, N, DY, seed=bs + chunk)
    plan = t.SpectralConv(1, bs, DY, K, N, dimX=dimX, variant="D")
    plan.set_host_chunk(chunk)
    got = _host_run(t, plan, x, w, (N, bs * dimX, DY))
    assert_close(from_reference_layout(got), oracle_c.spectral_conv_1d(x, w), "exec_host 1D bs=%d dimX=%d chunk=%d" % (bs, dimX, chunk))
    with pytest.raises(t.TfnoError):
        plan.set_host_chunk(2)            # staging is sized by the first call
    plan.close()


@pytest.mark.parametrize("variant", ["D", "A", "E"])
def test_exec_host_2d_in_several_chunks(cuda, variant):
    import turbofno_b200 as t

    bs, K, N, DX, DY = 5, 16, 64, 128, 128
    x, w = oracle_np.make_inputs_2d(bs, K, N, DX, DY, seed=17)
    plan = t.SpectralConv(2, bs, DY, K, N, DX=DX, variant=variant)
    plan.set_host_chunk(2)                # chunks of 2, 2 and a tail of 1 image per channel
    got = _host_run(t, plan, x, w, (N, bs, DX, DY))
    assert_close(from_reference_layout(got), oracle_c.spectral_conv_2d(x, w), "exec_host 2D variant " + variant)
    plan.close()


def test_exec_host_default_chunking_covers_the_batch(cuda):
    """Without an override: at least eight chunks when the batch allows it, last one shorter."""
    import turbofno_b200 as t

    bs, K, N, DY = 300, 32, 64, 256        # 8 chunks of 38 minus a tail of 34
    x, w = oracle_np.make_inputs_1d(bs, K, N, DY, seed=31)
    plan = t.SpectralConv(1, bs, DY, K, N, variant="D")
    got = _host_run(t, plan, x, w, (N, bs, DY))
    assert_close(from_reference_layout(got), oracle_c.spectral_conv_1d(x, w), "exec_host default chunks")
    plan.close()


def test_exec_host_rejects_wrong_shapes_on_the_host(cuda):
    import torch
    import turbofno_b200 as t

    plan = t.SpectralConv(1, 4, 128, 8, 64, variant="D")
    x = torch.zeros((8, 4, 128), dtype=torch.complex64)
    w = torch.zeros((64, 8), dtype=torch.complex64)
    with pytest.raises(ValueError):
        plan.exec_host(x, w, torch.zeros((64, 3, 128), dtype=torch.complex64))
    with pytest.raises(ValueError):
        plan(torch.zeros((8, 5, 128), dtype=torch.complex64, device=cuda), w.to(cuda))
    with pytest.raises(ValueError):
        plan(x.to(cuda), torch.zeros((64, 16), dtype=torch.complex64, device=cuda))
    plan.close()
    p2 = t.SpectralConv(2, 2, 128, 8, 64, DX=128, variant="D")
    with pytest.raises(ValueError):
        p2(torch.zeros((8, 2, 128, 128), dtype=torch.complex64, device=cuda), torch.zeros((64, 8), dtype=torch.complex64, device=cuda),
           workspace=torch.zeros(16, dtype=torch.uint8, device=cuda))
    with pytest.raises(ValueError):
        t.spectral_conv2d_static(torch.zeros((8, 2, 128, 128), dtype=torch.complex64, device=cuda),
                                 torch.zeros((64, 16), dtype=torch.complex64, device=cuda))
    p2.close()

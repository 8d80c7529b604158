"""Python mirror of the reference operator surface, on top of the C ABI.

Tensors are torch complex64 CUDA tensors in the reference's channel-outermost layout unless
strides are given:
    1D  x[K, B, DY]   (B = bs*dimX)      w[N, K] (element (k,n) at k + n*K)      y[N, B, DY]
    2D  x[K, bs, DX, DY]                  w[N, K]                                  y[N, bs, DX, DY]
"""
import ctypes
import math

import torch

from . import _lib
from ._lib import Problem, VARIANT, check


def _ptr(t):
    if t is None:
        return None
    return ctypes.c_void_p(t.data_ptr())


def _stream_ptr(stream=None, device=None):
    """cudaStream_t of `stream`, or of the current stream of `device` (not of the current device:
    the tensors decide where the work runs)."""
    s = stream if stream is not None else torch.cuda.current_stream(device)
    return ctypes.c_void_p(s.cuda_stream)


def _check_tensor(t, name):
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.complex64 and t.is_contiguous()):
        raise TypeError("%s must be a contiguous complex64 CUDA tensor" % name)


def expected_shapes(rank, layout, B, K, N, DY, DX=None, per_mode=False):
    """Shapes (x, w, y) a plan accepts, from its problem alone.  Reference layout: x[K, B, ...],
    w[N, K], y[N, B, ...]; batch-major: x[B, K, ...], w[K, N], y[B, N, ...].  Per-mode weights carry
    the mode axes last: w[N, K, 64] / w[N, K, 64, 64] (batch-major: w[K, N, ...])."""
    tail = (DY,) if rank == 1 else (DX, DY)
    wtail = () if not per_mode else ((64,) if rank == 1 else (64, 64))
    if layout == "reference":
        return (K, B) + tail, (N, K) + wtail, (N, B) + tail
    return (B, K) + tail, (K, N) + wtail, (B, N) + tail


def check_shapes(rank, layout, B, K, N, DY, DX, x_shape, w_shape, y_shape=None, per_mode=False):
    """Raises ValueError unless the tensors have exactly the shapes the plan was made for.  The
    kernels trust the plan's sizes (bulk copies included): a smaller tensor would be read or
    written out of bounds on the device, so the mirror refuses it on the host."""
    ex, ew, ey = expected_shapes(rank, layout, B, K, N, DY, DX, per_mode)
    if tuple(x_shape) != ex:
        raise ValueError("x has shape %s, the plan needs %s" % (tuple(x_shape), ex))
    if tuple(w_shape) != ew:
        raise ValueError("w has shape %s, the plan needs %s" % (tuple(w_shape), ew))
    if y_shape is not None and tuple(y_shape) != ey:
        raise ValueError("y has shape %s, the plan needs %s" % (tuple(y_shape), ey))


class Handle:
    """One per device (tfno_create / tfno_destroy)."""

    _cache = {}

    def __init__(self, device=0):
        self.lib = _lib.load()
        self.device = int(device)
        h = ctypes.c_void_p()
        check(self.lib.tfno_create(ctypes.byref(h), self.device), "tfno_create")
        self._h = h

    @classmethod
    def get(cls, device=None):
        device = torch.cuda.current_device() if device is None else int(device)
        if device not in cls._cache:
            cls._cache[device] = cls(device)
        return cls._cache[device]

    @property
    def sm_count(self):
        n = ctypes.c_int()
        check(self.lib.tfno_sm_count(self._h, ctypes.byref(n)), "tfno_sm_count")
        return n.value

    @property
    def device_status(self):
        """0, or the code of a kernel-side wait that ran out (synchronises the device)."""
        n = ctypes.c_int()
        check(self.lib.tfno_device_status(self._h, ctypes.byref(n)), "tfno_device_status")
        return n.value

    def reset_device_status(self):
        check(self.lib.tfno_device_status_reset(self._h), "tfno_device_status_reset")

    def selftest_bounded_wait(self, stream=None):
        """Makes one kernel-side wait run out (about one second); device_status then reads 99."""
        check(self.lib.tfno_selftest_bounded_wait(self._h, _stream_ptr(stream)), "tfno_selftest_bounded_wait")

    def close(self):
        if self._h:
            self.lib.tfno_destroy(self._h)
            self._h = None


class SpectralConv:
    """Plan for one spectral-convolution layer (tfno_plan_create / tfno_exec).

    variant: 'A'..'E' as in the TurboFNO_{1D,2D}_{A..E} executables.
    layout:  'reference' ([K][B][...], w[k + n*K]) or 'batch_major' ([B][K][...], w[K][N]).
    per_mode_weights: w carries one K x N matrix per retained mode (mode axes last), as an FNO
             layer trains them; the reference shares one matrix between all modes.
    """

    def __init__(self, rank, bs, DY, K, N, dimX=1, DX=None, variant="D", alpha=1.0 + 0j, beta=0j,
                 second_transform_forward=False, scale_inverse=True, layout="reference", device=None, modes=64,
                 x_modes_centered=False, per_mode_weights=False):
        self.handle = Handle.get(device)
        self.lib = self.handle.lib
        p = Problem()
        check(self.lib.tfno_problem_init(ctypes.byref(p), rank), "tfno_problem_init")
        p.bs, p.dimX, p.DY, p.K, p.N, p.modes = bs, dimX, DY, K, N, modes
        p.DX = DX if DX is not None else (1 if rank == 1 else DY)
        p.variant = VARIANT[variant]
        alpha, beta = complex(alpha), complex(beta)
        p.alpha_re, p.alpha_im, p.beta_re, p.beta_im = alpha.real, alpha.imag, beta.real, beta.imag
        p.second_transform_forward = int(bool(second_transform_forward))
        p.scale_inverse = int(bool(scale_inverse))
        p.x_modes_centered = int(bool(x_modes_centered))
        self.rank = rank
        self.B = bs * dimX if rank == 1 else bs
        unit = DY if rank == 1 else p.DX * DY
        self.per_mode = bool(per_mode_weights)
        nmodes = 64 if rank == 1 else 64 * 64
        if self.per_mode:
            p.w_stride_m = 1                # mode axes last and contiguous in both layouts
        if layout == "batch_major":
            p.x_stride_b, p.x_stride_k = K * unit, unit
            p.y_stride_b, p.y_stride_n = N * unit, unit
            p.w_stride_k, p.w_stride_n = (N * nmodes, nmodes) if self.per_mode else (N, 1)
        elif layout != "reference":
            raise ValueError("layout must be 'reference' or 'batch_major'")
        self.layout = layout
        self.problem = p
        plan = ctypes.c_void_p()
        check(self.lib.tfno_plan_create(self.handle._h, ctypes.byref(p), ctypes.byref(plan)), "tfno_plan_create")
        self._plan = plan
        self.workspace_bytes = int(self.lib.tfno_workspace_bytes(plan))
        self._ws = None

    def out_shape(self):
        p = self.problem
        tail = (p.DY,) if self.rank == 1 else (p.DX, p.DY)
        return ((p.N, self.B) if self.layout == "reference" else (self.B, p.N)) + tail

    def workspace(self, device):
        """The plan's own scratch buffer (allocated on first use).  It serves ONE stream at a time:
        callers that run the same plan on several streams concurrently pass their own `workspace`."""
        if self.workspace_bytes and (self._ws is None or self._ws.device != device):
            self._ws = torch.empty(self.workspace_bytes, dtype=torch.uint8, device=device)
        return self._ws

    def kernels(self):
        """Names of the kernels one call launches, in order (tfno_plan_kernels)."""
        buf = ctypes.create_string_buffer(1024)
        check(self.lib.tfno_plan_kernels(self._plan, buf, len(buf)), "tfno_plan_kernels")
        return buf.value.decode().split(";")

    def set_host_chunk(self, batch_items):
        """Batch items per pipeline chunk of exec_host; call before the first exec_host."""
        check(self.lib.tfno_plan_set_host_chunk(self._plan, int(batch_items)), "tfno_plan_set_host_chunk")

    def _check_call(self, x, w, y, workspace):
        p = self.problem
        check_shapes(self.rank, self.layout, self.B, p.K, p.N, p.DY, p.DX, x.shape, w.shape, None if y is None else y.shape, self.per_mode)
        dev = torch.device("cuda", self.handle.device)
        for name, t in (("x", x), ("w", w), ("y", y), ("workspace", workspace)):
            if t is not None and t.device != dev:
                raise ValueError("%s is on %s, the plan's handle on %s" % (name, t.device, dev))
        if workspace is not None:
            if not (workspace.is_cuda and workspace.is_contiguous()):
                raise ValueError("workspace must be a contiguous CUDA tensor")
            if workspace.numel() * workspace.element_size() < self.workspace_bytes:
                raise ValueError("workspace holds %d bytes, the plan needs %d" %
                                 (workspace.numel() * workspace.element_size(), self.workspace_bytes))

    def __call__(self, x, w, y=None, workspace=None, stream=None):
        _check_tensor(x, "x")
        _check_tensor(w, "w")
        if y is not None:
            _check_tensor(y, "y")
        self._check_call(x, w, y, workspace)
        if y is None:
            y = torch.empty(self.out_shape(), dtype=torch.complex64, device=x.device)
        ws = workspace if workspace is not None else self.workspace(x.device)
        check(self.lib.tfno_exec(self._plan, _ptr(x), _ptr(w), _ptr(y), _ptr(ws), _stream_ptr(stream, x.device)), "tfno_exec")
        return y

    def exec_host(self, x_host, w_host, y_host):
        """Host (ideally pinned) complex64 tensors in, host tensor out (tfno_exec_host)."""
        for t in (x_host, w_host, y_host):
            if t.is_cuda or t.dtype != torch.complex64 or not t.is_contiguous():
                raise TypeError("exec_host needs contiguous complex64 host tensors")
        p = self.problem
        check_shapes(self.rank, self.layout, self.B, p.K, p.N, p.DY, p.DX, x_host.shape, w_host.shape, y_host.shape, self.per_mode)
        check(self.lib.tfno_exec_host(self._plan, ctypes.c_void_p(x_host.data_ptr()), ctypes.c_void_p(w_host.data_ptr()),
                                      ctypes.c_void_p(y_host.data_ptr())), "tfno_exec_host")
        return y_host

    def close(self):
        if self._plan:
            self.lib.tfno_plan_destroy(self._plan)
            self._plan = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# --------------------------------------------------------------------------------------------
# kernel-table entry points (reference names and argument order; DY / DX select the table slot)
# --------------------------------------------------------------------------------------------
def _log2(n):
    l = int(round(math.log2(n)))
    if (1 << l) != n:
        raise ValueError("transform length must be a power of two")
    return l


def fused_fft_cgemm_ifft(M, N, K, FFT_input, B, C, FFT_output, alpha=1 + 0j, beta=0j, DY=128, stream=None):
    h = Handle.get(FFT_input.device.index)
    a, b = complex(alpha), complex(beta)
    check(h.lib.tfno_fused_fft_cgemm_ifft(h._h, _log2(DY), M, N, K, _ptr(FFT_input), _ptr(B), _ptr(C), _ptr(FFT_output),
                                          a.real, a.imag, b.real, b.imag, _stream_ptr(stream, FFT_input.device)), "tfno_fused_fft_cgemm_ifft")
    return FFT_output


def fused_fft_cgemm(M, N, K, FFT_input, B, C, alpha=1 + 0j, beta=0j, DY=128, stream=None):
    h = Handle.get(FFT_input.device.index)
    a, b = complex(alpha), complex(beta)
    check(h.lib.tfno_fused_fft_cgemm(h._h, _log2(DY), M, N, K, _ptr(FFT_input), _ptr(B), _ptr(C),
                                     a.real, a.imag, b.real, b.imag, _stream_ptr(stream, FFT_input.device)), "tfno_fused_fft_cgemm")
    return C


def fused_cgemm_ifft(M, N, K, A, B, C, FFT_output, alpha=1 + 0j, beta=0j, DY=128, stream=None):
    h = Handle.get(A.device.index)
    a, b = complex(alpha), complex(beta)
    check(h.lib.tfno_fused_cgemm_ifft(h._h, _log2(DY), M, N, K, _ptr(A), _ptr(B), _ptr(C), _ptr(FFT_output),
                                      a.real, a.imag, b.real, b.imag, _stream_ptr(stream, A.device)), "tfno_fused_cgemm_ifft")
    return FFT_output


def cgemm(M, N, K, A, B, C, alpha=1 + 0j, beta=0j, stream=None):
    h = Handle.get(A.device.index)
    a, b = complex(alpha), complex(beta)
    check(h.lib.tfno_cgemm(h._h, M, N, K, _ptr(A), _ptr(B), _ptr(C), a.real, a.imag, b.real, b.imag,
                           _stream_ptr(stream, A.device)), "tfno_cgemm")
    return C


def fft_stride_DY(inp, out, total_signals, DY, stream=None):
    h = Handle.get(inp.device.index)
    check(h.lib.tfno_fft_stride_DY(h._h, _log2(DY), _ptr(inp), _ptr(out), total_signals, _stream_ptr(stream, inp.device)), "tfno_fft_stride_DY")
    return out


def ifft_stride_DY(inp, out, total_signals, DY, stream=None):
    h = Handle.get(inp.device.index)
    check(h.lib.tfno_ifft_stride_DY(h._h, _log2(DY), _ptr(inp), _ptr(out), total_signals, _stream_ptr(stream, inp.device)), "tfno_ifft_stride_DY")
    return out


def fft_stride(inp, out, DY, total_columns, DX, stream=None):
    h = Handle.get(inp.device.index)
    check(h.lib.tfno_fft_stride(h._h, _log2(DX), _ptr(inp), _ptr(out), DY, total_columns, _stream_ptr(stream, inp.device)), "tfno_fft_stride")
    return out


def ifft_stride(inp, out, DY, total_columns, DX, stream=None):
    h = Handle.get(inp.device.index)
    check(h.lib.tfno_ifft_stride(h._h, _log2(DX), _ptr(inp), _ptr(out), DY, total_columns, _stream_ptr(stream, inp.device)), "tfno_ifft_stride")
    return out


def spectral_conv2d_static(x, w, y=None, alpha=1 + 0j, stream=None):
    """One 2D layer through tfno_spectral_conv2d_static: no device allocation is made inside the
    library, the spectrum scratch lives in a fixed 64 MiB array of the library image.  For hosts
    that may not allocate when a layer runs (arena-owned devices, no-allocation-after-start-up
    rules, calls in between another allocator's operations).  x[K, bs, DX, DY], w[N, K] in the
    reference layout; y is allocated here by torch only if the caller does not pass one."""
    _check_tensor(x, "x")
    _check_tensor(w, "w")
    if x.dim() != 4 or w.dim() != 2:
        raise ValueError("x must be [K, bs, DX, DY] and w [N, K]")
    K, bs, DX, DY = x.shape
    N = w.shape[0]
    if y is not None:
        _check_tensor(y, "y")
    check_shapes(2, "reference", bs, K, N, DY, DX, x.shape, w.shape, None if y is None else y.shape)
    for name, t in (("w", w), ("y", y)):
        if t is not None and t.device != x.device:
            raise ValueError("%s is on %s, x on %s" % (name, t.device, x.device))
    if y is None:
        y = torch.empty((N, bs, DX, DY), dtype=torch.complex64, device=x.device)
    lib = _lib.load()
    a = complex(alpha)
    with torch.cuda.device(x.device):
        check(lib.tfno_spectral_conv2d_static(bs, DX, DY, K, N, _ptr(x), _ptr(w), _ptr(y), a.real, a.imag,
                                              _stream_ptr(stream, x.device)), "tfno_spectral_conv2d_static")
    return y

"""turbofno_b200 -- B200 (sm_100a) kernels for the FNO spectral-convolution path.

Host-side mirror of the reference's operator surface (shixun404/TurboFNO): the kernel-table
entry points keep the reference names (`fused_fft_cgemm_ifft`, `cgemm`, `fft_stride_DY`, ...)
and argument order; `SpectralConv` is the plan/exec pair behind the TurboFNO_{1D,2D}_{A..E}
drivers.  Everything here calls the C ABI in libturbofno_b200.so; PyTorch is used only to hold
device memory and streams.
"""
from ._lib import Problem, TfnoError, VARIANT, check, load  # noqa: F401
from .api import (  # noqa: F401
    Handle,
    SpectralConv,
    cgemm,
    fft_stride,
    fft_stride_DY,
    fused_cgemm_ifft,
    fused_fft_cgemm,
    fused_fft_cgemm_ifft,
    ifft_stride,
    ifft_stride_DY,
    spectral_conv2d_static,
)

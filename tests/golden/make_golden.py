"""Writes the golden fixtures of this directory from the numpy oracle (complex128).

The reference project holds no golden vectors for this path, so these files freeze the oracle's
answers on small seeded cases; tests check the C oracle and the CUDA kernels against them.
Run:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle_np as o  # noqa: E402


def main():
    # config 0: bs=1, dimX=1, DY=128, K=8, N=64
    x, w = o.make_inputs_1d(1, 8, 64, 128, seed=1234, wseed=4321)
    y = o.spectral_conv_1d(x, w)
    np.savez_compressed(os.path.join(HERE, "c0_1d_bs1_dy128_k8_n64.npz"), x=x, w=w, y=y.astype(np.complex128))
    # a 1D sweep point with DY=256, N=128
    x, w = o.make_inputs_1d(4, 24, 128, 256, seed=1235, wseed=4322)
    y = o.spectral_conv_1d(x, w)
    np.savez_compressed(os.path.join(HERE, "c1_1d_bs4_dy256_k24_n128.npz"), x=x, w=w, y=y[:, ::8, :].astype(np.complex128))
    # small 2D case: bs=1, K=8, N=64, 128x256; output sampled on a coarse lattice
    x, w = o.make_inputs_2d(1, 8, 64, 128, 256, seed=1236, wseed=4323)
    y = o.spectral_conv_2d(x, w)
    np.savez_compressed(os.path.join(HERE, "c2_2d_bs1_k8_n64_128x256.npz"), x=x, w=w,
                        y=y[:, ::8, ::8, ::8].astype(np.complex128))


if __name__ == "__main__":
    main()

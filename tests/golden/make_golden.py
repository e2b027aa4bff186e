"""Regenerates tests/golden/*.npz from the REFERENCE's own CPU convolution.

Run where the reference checkout is present (it is compiled, untouched, into
oracle/_ref/libtetris_ref.so by oracle/Makefile):

    python tests/golden/make_golden.py

Each fixture stores the seeded input (NCHW), the dense filter (OIHW), the conv parameters and
the output of the reference's HostConv2d (Tetris/tensor_utils.cc:136-170) on them.  The
fixtures pin the C restatement in oracle/host_conv2d.c (bit-exact) and the GPU path (1e-4).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402

# name: (N, IC, H, W, OC, KS, stride, pad, weight sparsity, all_ones)
CASES = {
    "c3x3_s1_p1": (2, 20, 13, 17, 40, 3, 1, 1, 0.90, False),
    "c3x3_s2_p1": (2, 16, 15, 14, 33, 3, 2, 1, 0.85, False),
    "c3x3_s1_p0": (1, 9, 10, 12, 17, 3, 1, 0, 0.80, False),
    "c1x1_s1_p0": (2, 48, 9, 11, 70, 1, 1, 0, 0.80, False),
    "c1x1_s2_p0": (3, 24, 14, 14, 32, 1, 2, 0, 0.80, False),
    "c7x7_s2_p3": (2, 3, 30, 26, 16, 7, 2, 3, 0.50, False),
    "oc255_ic35": (1, 35, 8, 8, 255, 1, 1, 0, 0.90, False),
    "zero_rows": (2, 18, 12, 12, 24, 3, 1, 1, 0.95, False),
    # the reference's DEBUG mode (Tetris/tensor_utils.cc:10-12,74-76): input and nonzero weights
    # all 1.0, so every output is the integer count of in-bounds nonzero taps
    "all_ones_3x3": (1, 12, 9, 9, 20, 3, 1, 1, 0.80, True),
}


def make_case(name):
    n, ic, h, w, oc, ks, stride, pad, sparsity, ones = CASES[name]
    rng = np.random.Generator(np.random.Philox(key=sum(map(ord, name))))
    filt = rng.normal(0.0, 0.05, size=(oc, ic, ks, ks)).astype(np.float32)
    filt[filt == 0] = 0.05
    filt.reshape(-1)[rng.permutation(filt.size)[: int(round(sparsity * filt.size))]] = 0.0
    if name == "zero_rows":
        filt[[0, 7, 23]] = 0.0  # output channels without a single nonzero
    x = rng.random(size=(n, ic, h, w), dtype=np.float32)
    x[rng.random(size=x.shape, dtype=np.float32) < 0.5] = 0.0
    if ones:
        filt[filt != 0] = 1.0
        x[:] = 1.0
    return x, filt, stride, pad


def main():
    if orc.ref() is None:
        orc.build()
    if orc.ref() is None:
        sys.exit("oracle/_ref/libtetris_ref.so is absent and the reference sources are not here")
    for name in CASES:
        x, filt, stride, pad = make_case(name)
        y = orc.ref_host_conv2d(x, filt, stride, pad)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), input=x, filter=filt,
                            stride=np.int32(stride), pad=np.int32(pad), output=y)
        print("%-14s in %s filt %s out %s" % (name, x.shape, filt.shape, y.shape))


if __name__ == "__main__":
    main()

"""Regenerates tests/real_layers/*.npz from the reference's pruned-checkpoint layer dumps.

Run where the reference checkout is present ($TETRIS_REFERENCE_ROOT, or a directory `reference`
beside this repository):

    python tests/real_layers/make_real_layers.py

Each dump (evalution/conv_weight_data/<model>/<checkpoint>/<layer file>, text: header
`H W IC OC KS Pad S G`, then OC*IC*KS*KS floats) is parsed by the REFERENCE's own reader
(ReadConfigAndDataFromFile, Tetris/tensor_utils.cc:55-82, through oracle/_ref) and stored
compactly: the header fields plus the flat OIHW indices and values of the nonzero weights.
These are test fixtures (real magnitude-pruned masks: skewed rows, empty rows, |w| up to ~2),
not part of the engine.
"""
import ctypes
import glob
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402

# (model directory, checkpoint glob, shape suffix of the layer file, how many of that shape)
PICKS = [
    ("vgg19", "vgg19-92*", "H_224_W_224_IC_64_OC_64_KS_3_Pad_1_S_1_G_1", 1),
    ("vgg19", "vgg19-92*", "H_112_W_112_IC_128_OC_128_KS_3_Pad_1_S_1_G_1", 1),
    ("vgg19", "vgg19-92*", "H_56_W_56_IC_128_OC_256_KS_3_Pad_1_S_1_G_1", 1),
    ("vgg19", "vgg19-92*", "H_56_W_56_IC_256_OC_256_KS_3_Pad_1_S_1_G_1", 1),
    ("resnet50", "ResNet50-magnitude-90*", "H_56_W_56_IC_64_OC_64_KS_3_Pad_1_S_1_G_1", 1),
    ("resnet50", "ResNet50-magnitude-90*", "H_28_W_28_IC_128_OC_128_KS_3_Pad_1_S_1_G_1", 1),
    ("resnet50", "ResNet50-magnitude-90*", "H_14_W_14_IC_256_OC_256_KS_3_Pad_1_S_1_G_1", 1),
    ("resnet50", "ResNet50-magnitude-90*", "H_56_W_56_IC_128_OC_128_KS_3_Pad_1_S_2_G_1", 1),
    ("resnet50", "ResNet50-magnitude-90*", "H_56_W_56_IC_64_OC_256_KS_1_Pad_0_S_1_G_1", 1),
    ("resnet50", "ResNet50-magnitude-90*", "H_56_W_56_IC_256_OC_64_KS_1_Pad_0_S_1_G_1", 1),
    ("resnet50", "ResNet50-magnitude-90*", "H_28_W_28_IC_512_OC_128_KS_1_Pad_0_S_1_G_1", 1),
    ("resnet50", "ResNet50-magnitude-90*", "H_14_W_14_IC_1024_OC_256_KS_1_Pad_0_S_1_G_1", 1),
    ("resnet50", "ResNet50-magnitude-90*", "H_56_W_56_IC_256_OC_512_KS_1_Pad_0_S_2_G_1", 1),
    ("mobilenet", "mobilenet-86*", "H_112_W_112_IC_32_OC_64_KS_1_Pad_0_S_1_G_1", 1),
    ("mobilenet", "mobilenet-86*", "H_56_W_56_IC_64_OC_128_KS_1_Pad_0_S_1_G_1", 1),
    ("mobilenet", "mobilenet-86*", "H_28_W_28_IC_256_OC_256_KS_1_Pad_0_S_1_G_1", 1),
    ("mobilenet", "mobilenet-86*", "H_14_W_14_IC_512_OC_512_KS_1_Pad_0_S_1_G_1", 1),
    ("mobilenet", "mobilenet-86*", "H_7_W_7_IC_512_OC_1024_KS_1_Pad_0_S_1_G_1", 1),
    ("yolov3", "yolov3-89*", "H_80_W_80_IC_128_OC_256_KS_3_Pad_1_S_1_G_1", 1),
    ("yolov3", "yolov3-89*", "H_160_W_160_IC_64_OC_128_KS_3_Pad_1_S_1_G_1", 1),
    ("yolov3", "yolov3-89*", "H_320_W_320_IC_64_OC_128_KS_3_Pad_1_S_2_G_1", 1),
    ("yolov3", "yolov3-89*", "H_40_W_40_IC_512_OC_256_KS_1_Pad_0_S_1_G_1", 1),
    ("yolov3", "yolov3-89*", "H_80_W_80_IC_256_OC_255_KS_1_Pad_0_S_1_G_1", 1),
    ("yolov3", "yolov3-89*", "H_80_W_80_IC_384_OC_128_KS_1_Pad_0_S_1_G_1", 1),
]


def read_with_reference(path):
    """(H, W, IC, OC, KS, Pad, S, G) and the dense OIHW filter, through the reference's reader."""
    lib = orc.ref()
    assert lib is not None, "oracle/_ref is not built: run `make -C oracle ref` where the reference checkout is"
    hdr = (ctypes.c_int * 9)()
    ptr = lib.ref_read_layer_file(path.encode(), 9, hdr)
    assert ptr, "the reference reader could not open " + path
    h, w, ic, oc, ks, pad, s, g = [hdr[i] for i in range(8)]
    n = oc * ic * ks * ks
    dense = np.ctypeslib.as_array(ptr, shape=(n,)).copy()
    lib.ref_free(ptr)
    return (h, w, ic, oc, ks, pad, s, g), dense


def main():
    data = os.path.join(orc.reference_root(), "evalution", "conv_weight_data")
    total = 0
    for model, ckpt, suffix, count in PICKS:
        files = sorted(glob.glob(os.path.join(data, model, ckpt, "*" + suffix)))
        assert len(files) >= count, (model, suffix)
        for path in files[:count]:
            (h, w, ic, oc, ks, pad, s, g), dense = read_with_reference(path)
            idx = np.flatnonzero(dense).astype(np.uint32)
            rows = np.count_nonzero(dense.reshape(oc, -1), axis=1)
            name = "%s__%s" % (model, os.path.basename(path))
            out = os.path.join(HERE, name + ".npz")
            np.savez_compressed(out, header=np.array([h, w, ic, oc, ks, pad, s, g], np.int32), index=idx,
                                value=dense[idx].astype(np.float32), source=np.array(os.path.relpath(path, data)))
            total += os.path.getsize(out)
            print("%-100s nnz %7d (%.1f %% sparse) row nnz min/mean/max %d/%.1f/%d, empty rows %d, max|w| %.2f -> %d KB"
                  % (name, idx.size, 100 * (1 - idx.size / dense.size), rows.min(), rows.mean(), rows.max(),
                     int((rows == 0).sum()), float(np.abs(dense).max()), os.path.getsize(out) // 1024))
    print("total %.1f MB" % (total / 1e6))


if __name__ == "__main__":
    main()

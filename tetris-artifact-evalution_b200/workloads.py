"""Synthetic workloads: layer shapes of the benchmark networks and seeded tensor generators.

The reference measures on text dumps of pruned checkpoints (one file per conv layer,
header `H W IC OC KS Pad S G`, Tetris/tensor_utils.cc:66).  Here the same layer shapes are
generated: weights ~ N(0, 0.05) with an exact-count uniform-random zero mask, activations
uniform[0, 1) with an independent Bernoulli(0.5) zero mask.  Every tensor is a pure function
of (workload name, layer index, kind), so the CPU oracle and the GPU path see identical data.
"""
import glob
import os
import zlib
from collections import namedtuple

import numpy as np

# One convolution layer: input extent, channels, kernel, padding, stride, groups, weight sparsity
# (None = drawn per layer from U[0.80, 0.95]).
Layer = namedtuple("Layer", "name H W IC OC KS pad stride groups sparsity")


def out_extent(size, ks, stride, pad):
    return (size + 2 * pad - ks) // stride + 1


def single_layer():
    """The single-layer case: 64 -> 64, 3x3, stride 1, pad 1 at 56x56, 90 % sparse."""
    return [Layer("conv", 56, 56, 64, 64, 3, 1, 1, 1, 0.90)]


def vgg19():
    layers, size, ic = [], 224, 3
    plan = [(64, 2), (128, 2), (256, 4), (512, 4), (512, 4)]
    for stage, (oc, reps) in enumerate(plan):
        for r in range(reps):
            first = not layers
            layers.append(Layer("conv%d_%d" % (stage + 1, r + 1), size, size, ic, oc, 3, 1, 1, 1,
                                0.50 if first else None))
            ic = oc
        size //= 2  # max-pool between stages
    return layers


def vgg19_s99():
    """VGG-19's shapes pruned to 99 % (first layer 50 %): not one of the five benchmark workloads.
    It shows where the per-layer choice crosses over: the list kernel's time falls with the
    nonzeros until staging the input tiles is all that is left, and at 99 % it meets the dense
    tensor-core kernels (whose time does not depend on the mask) on the 224x224 and 56x56 layers,
    where the tuner then picks it."""
    return [l._replace(sparsity=0.50 if i == 0 else 0.99) for i, l in enumerate(vgg19())]


def resnet50():
    layers = [Layer("stem", 224, 224, 3, 64, 7, 3, 2, 1, 0.50)]
    size, ic = 56, 64  # after the stem (112) and the 3x3/2 max-pool
    for stage, (width, blocks) in enumerate([(64, 3), (128, 4), (256, 6), (512, 3)]):
        for blk in range(blocks):
            stride = 2 if (blk == 0 and stage > 0) else 1
            tag = "s%d_b%d" % (stage + 1, blk + 1)
            layers.append(Layer(tag + "_1x1a", size, size, ic, width, 1, 0, 1, 1, 0.80))
            layers.append(Layer(tag + "_3x3", size, size, width, width, 3, 1, stride, 1, 0.80))
            osize = out_extent(size, 3, stride, 1)
            layers.append(Layer(tag + "_1x1b", osize, osize, width, 4 * width, 1, 0, 1, 1, 0.80))
            if blk == 0:
                layers.append(Layer(tag + "_proj", size, size, ic, 4 * width, 1, 0, stride, 1, 0.80))
            size, ic = osize, 4 * width
    return layers


def mobilenet_v1():
    layers = [Layer("stem", 224, 224, 3, 32, 3, 1, 2, 1, 0.0)]
    size, ic = 112, 32
    strides = [1, 2, 1, 2, 1, 2, 1, 1, 1, 1, 1, 2, 1]
    widths = [64, 128, 128, 256, 256, 512, 512, 512, 512, 512, 512, 1024, 1024]
    for i, (s, oc) in enumerate(zip(strides, widths)):
        layers.append(Layer("dw%d" % (i + 1), size, size, ic, ic, 3, 1, s, ic, 0.0))
        size = out_extent(size, 3, s, 1)
        layers.append(Layer("pw%d" % (i + 1), size, size, ic, oc, 1, 0, 1, 1, 0.85))
        ic = oc
    return layers


def yolov3(size=416):
    layers = []

    def conv(name, ic, oc, ks, stride, at):
        layers.append(Layer(name, at, at, ic, oc, ks, ks // 2, stride, 1, None))
        return out_extent(at, ks, stride, ks // 2)

    at = conv("conv0", 3, 32, 3, 1, size)
    ic = 32
    for stage, reps in enumerate([1, 2, 8, 8, 4]):
        at = conv("down%d" % (stage + 1), ic, 2 * ic, 3, 2, at)
        ic *= 2
        for r in range(reps):
            conv("res%d_%d_1x1" % (stage + 1, r + 1), ic, ic // 2, 1, 1, at)
            conv("res%d_%d_3x3" % (stage + 1, r + 1), ic // 2, ic, 3, 1, at)
    # detection heads at strides 32, 16, 8; the route convs feed an upsample + concat
    head_in, mid = 1024, 512
    for h, extra in enumerate([0, 512, 256]):
        if h > 0:
            conv("route%d" % h, mid * 2, mid, 1, 1, at)  # on the previous head's 1x1 output
            at *= 2
            head_in = mid + extra
        cin = head_in
        for r in range(3):
            conv("head%d_%d_1x1" % (h + 1, r + 1), cin, mid, 1, 1, at)
            conv("head%d_%d_3x3" % (h + 1, r + 1), mid, 2 * mid, 3, 1, at)
            cin = 2 * mid
        conv("head%d_out" % (h + 1), 2 * mid, 255, 1, 1, at)
        mid //= 2
    return layers


# ---- real pruned layers -----------------------------------------------------------------------
# Compact copies (shape + indices and values of the nonzero weights) of layer dumps of pruned
# checkpoints in the reference's text format (header `H W IC OC KS Pad S G`, then the OIHW
# floats, Tetris/tensor_utils.cc:55-82).  Magnitude pruning leaves very uneven rows, rows with no
# nonzeros and |w| up to ~2 -- unlike the uniform masks above.  The directory is
# $TETRIS_REAL_LAYERS, else tests/real_layers beside the package.
def real_layer_dir():
    here = os.path.dirname(os.path.abspath(__file__))
    return os.environ.get("TETRIS_REAL_LAYERS") or os.path.join(os.path.dirname(here), "tests", "real_layers")


def real_layer_files():
    return sorted(glob.glob(os.path.join(real_layer_dir(), "*.npz")))


def load_real_layer(path):
    """(Layer, dense OIHW float32 filter) of one compact layer file."""
    z = np.load(path)
    h, w, ic, oc, ks, pad, stride, groups = (int(v) for v in z["header"])
    dense = np.zeros(oc * ic * ks * ks, np.float32)
    dense[z["index"]] = z["value"]
    name = os.path.basename(path)[:-4]
    short = "%s_%dx%d_%dto%d_k%ds%d" % (name.split("__")[0], h, w, ic, oc, ks, stride)
    sparsity = 1.0 - z["index"].size / dense.size
    # the reference reads the groups field and ignores it (Tetris/tensor_utils.cc:66)
    return Layer(short, h, w, ic, oc, ks, pad, stride, 1, sparsity), dense.reshape(oc, ic, ks, ks)


def real_layers():
    return [load_real_layer(p)[0] for p in real_layer_files()]


def uniform_like(filt, seed=0):
    """A filter of the same shape and nonzero count (and the same nonzero values) whose nonzeros
    sit at uniformly random positions: the uniform-mask twin of a pruned layer."""
    rng = np.random.Generator(np.random.Philox(key=seed))
    flat = filt.reshape(-1)
    vals = flat[flat != 0]
    out = np.zeros_like(flat)
    out[rng.permutation(flat.size)[:vals.size]] = vals
    return out.reshape(filt.shape)


WORKLOADS = {
    "single": single_layer,
    "vgg19": vgg19,
    "resnet50": resnet50,
    "mobilenet": mobilenet_v1,
    "yolov3": yolov3,
    "real": real_layers,
    "vgg19_s99": vgg19_s99,
}


def _rng(workload, layer_idx, kind):
    key = zlib.crc32(("%s/%d/%s" % (workload, layer_idx, kind)).encode())
    return np.random.Generator(np.random.Philox(key=key))


def layer_sparsity(workload, layer_idx, layer):
    """The layer's weight sparsity; unspecified ones are drawn from U[0.80, 0.95]."""
    if layer.sparsity is not None:
        return layer.sparsity
    return float(_rng(workload, layer_idx, "sparsity").uniform(0.80, 0.95))


def make_filter(workload, layer_idx, layer):
    """Dense OIHW float32 filter ([C][1][KS][KS] for depthwise) with an exact-count zero mask."""
    if workload == "real":
        return load_real_layer(real_layer_files()[layer_idx])[1]
    per_oc = 1 if layer.groups != 1 else layer.IC
    shape = (layer.OC, per_oc, layer.KS, layer.KS)
    rng = _rng(workload, layer_idx, "filter")
    w = rng.normal(0.0, 0.05, size=shape).astype(np.float32)
    w[w == 0.0] = 0.05  # a drawn exact zero would blur the nonzero count
    n_zero = int(round(layer_sparsity(workload, layer_idx, layer) * w.size))
    if n_zero > 0:
        w.reshape(-1)[rng.permutation(w.size)[:n_zero]] = 0.0
    return w


def make_input(workload, layer_idx, layer, batch):
    """NCHW float32 activations: uniform[0, 1) with about half of the entries zeroed."""
    rng = _rng(workload, layer_idx, "input")
    shape = (batch, layer.IC, layer.H, layer.W)
    x = rng.random(size=shape, dtype=np.float32)
    x[rng.random(size=shape, dtype=np.float32) < 0.5] = 0.0
    return x


def layer_costs(layer, batch, nnz):
    """Algorithmic work of one layer launch: (flops, bytes).

    flops = 2 * nnz * N * OH * OW (border clipping ignored, as in the reference's own FLOP
    line, Tetris/spconv2d.cc:358); bytes = input read once + output written once + 8 bytes
    per nonzero weight (FP32 value + int32 position, the reference's <float,int,int> format)
    + 4 bytes per output-channel row pointer.
    """
    oh = out_extent(layer.H, layer.KS, layer.stride, layer.pad)
    ow = out_extent(layer.W, layer.KS, layer.stride, layer.pad)
    flops = 2 * nnz * batch * oh * ow
    nbytes = 4 * batch * layer.IC * layer.H * layer.W + 4 * batch * layer.OC * oh * ow \
        + 8 * nnz + 4 * (layer.OC + 1)
    return flops, nbytes

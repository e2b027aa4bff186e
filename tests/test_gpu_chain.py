"""GPU: layer chains (tetris_chain_*) and the fused-ReLU launch.

A chain runs the conv layers of a model back to back on the device: layer i reads the NHWC
activations layer i - 1 left in HBM, rectified at the convolution's store and 2x2 max-pooled in
between.  Checked against the chained CPU oracle (HostConv2d, then max(y, 0), then pooling, layer
after layer), eagerly and as a replayed CUDA graph, and against the same layers launched one by
one.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _pool2(x):  # NCHW, 2x2 max-pooling, stride 2, floor
    n, c, h, w = x.shape
    x = x[:, :, :h // 2 * 2, :w // 2 * 2]
    return x.reshape(n, c, h // 2, 2, w // 2, 2).max(axis=(3, 5))


def _oracle_chain(oracle, x, specs):
    for filt, stride, pad, relu, pool, groups in specs:
        x = oracle.host_depthwise_conv2d(x, filt, stride, pad) if groups != 1 else \
            oracle.host_conv2d(x, filt, stride, pad, threads=True, skip_zero=True)
        if relu:
            x = np.maximum(x, 0)
        if pool:
            x = _pool2(x)
    return x


def _chain_output(torch, chain, n):
    """The chain's last activations (they live in a buffer the chain owns) as NCHW numpy."""
    return chain.download().transpose(0, 3, 1, 2)


@pytest.mark.parametrize("variant", ["auto", "generic", "tiled", "tensor", "tensor16"])
def test_fused_relu_launch(tb, torch_cuda, oracle, variant):
    torch = torch_cuda
    rng = np.random.default_rng(5)
    v = {"auto": 0, "generic": 1, "tiled": 2, "tensor": 4, "tensor16": 5}[variant]
    for (n, ic, h, oc, ks, pad) in ((3, 64, 28, 96, 3, 1), (16, 128, 14, 128, 3, 1), (2, 256, 14, 64, 1, 0)):
        filt = rng.normal(0, 0.05, (oc, ic, ks, ks)).astype(np.float32)
        filt[rng.random(filt.shape) < 0.8] = 0
        x = rng.random((n, ic, h, h), dtype=np.float32) - 0.4   # plenty of negative outputs
        f = tb.SparseFilter(filt, ic, oc, ks)
        oh = tb.out_extent(h, ks, 1, pad)
        xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
        out = torch.full((n, oh, oh, oc), float("nan"), device="cuda")
        tb.sparse_conv2d_fused(f, xin, out, n, h, h, 1, pad, variant=v, relu=True)
        torch.cuda.synchronize()
        f.check()
        got = out.cpu().numpy().transpose(0, 3, 1, 2)
        want = np.maximum(oracle.host_conv2d(x, filt, 1, pad), 0)
        assert (got >= 0).all()
        assert oracle.compare(got, want)[0] == 0
        # the plain launch of the same filter afterwards is not rectified
        tb.sparse_conv2d(f, xin, out, n, h, h, 1, pad, variant=v)
        torch.cuda.synchronize()
        assert float(out.min()) < 0


def test_small_chain_against_the_chained_oracle(tb, torch_cuda, oracle):
    torch = torch_cuda
    rng = np.random.default_rng(6)
    n, h = 2, 32
    shapes = [(16, 32, 3, 1, 1, True, 0, 1), (32, 32, 3, 1, 1, True, 2, 32), (32, 64, 1, 1, 0, True, 0, 1),
              (64, 48, 3, 2, 1, False, 0, 1)]   # IC, OC, KS, stride, pad, relu, pool, groups
    specs, layers, filters = [], [], []
    for ic, oc, ks, stride, pad, relu, pool, groups in shapes:
        per = 1 if groups != 1 else ic
        filt = rng.normal(0, 0.15, (oc, per, ks, ks)).astype(np.float32)
        if groups == 1:
            filt[rng.random(filt.shape) < 0.7] = 0
        f = tb.SparseFilter(filt, ic, oc, ks, groups=groups)
        filters.append(f)
        specs.append((filt, stride, pad, relu, pool, groups))
        layers.append((f, stride, pad, relu, pool))
    x = rng.random((n, 16, h, h), dtype=np.float32) - 0.3
    want = _oracle_chain(oracle, x, specs)
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    chain = tb.LayerChain(layers, n, h, h)
    _, oh, ow, oc = chain.output()
    assert (oh, ow, oc) == want.shape[2:] + (want.shape[1],)
    chain.run(xin)
    got = _chain_output(torch, chain, n)
    assert oracle.compare(got, want)[0] == 0
    chain.capture(xin)
    for _ in range(3):
        chain.replay()
    got2 = _chain_output(torch, chain, n)
    assert oracle.compare(got2, want)[0] == 0
    for f in filters:
        f.check()
    with pytest.raises(tb.TetrisError) as e:   # channels that do not fit together
        tb.LayerChain([layers[0], layers[3]], n, h, h)   # 32 channels out, 64 expected in
    assert e.value.status == 1 and "channels" in str(e.value)
    chain.close()


def test_vgg19_chain_batch1(tb, torch_cuda, workloads, oracle):
    """The whole VGG-19 conv stack at batch 1: ReLU after every layer, 2x2 max-pooling after each
    stage, one CUDA graph; against the chained oracle.  Sixteen layers compound their rounding,
    so the final comparison allows 1e-3 of the output's largest magnitude."""
    torch = torch_cuda
    L = workloads.vgg19()
    last_of_stage = {1, 3, 7, 11}
    specs, layers, filters = [], [], []
    for i, l in enumerate(L):
        filt = workloads.make_filter("vgg19", i, l) * np.float32(3.0)   # keeps the activations from fading over 16 layers
        f = tb.SparseFilter(filt, l.IC, l.OC, l.KS)
        filters.append(f)
        pool = 2 if i in last_of_stage else 0
        specs.append((filt, 1, 1, True, pool, 1))
        layers.append((f, 1, 1, True, pool))
    x = workloads.make_input("vgg19", 0, L[0], 1)
    want = _oracle_chain(oracle, x, specs)
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    chain = tb.LayerChain(layers, 1, 224, 224)
    chain.capture(xin)
    chain.replay()
    got = _chain_output(torch, chain, 1)
    assert got.shape == want.shape == (1, 512, 14, 14)
    scale = float(np.abs(want).max())
    assert scale > 1e-3, "the activations faded away; the comparison would be empty"
    assert float(np.abs(got - want).max()) <= 1e-3 * scale
    for f in filters:
        f.check()
    chain.close()

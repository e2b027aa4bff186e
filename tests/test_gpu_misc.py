"""GPU: depthwise convolution, layout transposes and the sharded host entry point."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


# (n, c, h, w, stride, pad): channel counts that are multiples of 32 take the pipelined kernel
# (16-wide tiles, 8-wide tiles for images up to 8 wide, stride 2), the others the plain kernels
@pytest.mark.parametrize("n,c,h,w,stride,pad", [
    (2, 32, 20, 20, 1, 1), (1, 64, 15, 17, 2, 1), (3, 7, 5, 4, 1, 1),
    (2, 96, 7, 7, 1, 1), (1, 32, 8, 30, 1, 1), (2, 64, 33, 47, 1, 0), (3, 32, 9, 9, 2, 0),
    (16, 128, 56, 56, 1, 1),   # more tiles than CTAs: the ring of stages turns several times
    (16, 64, 57, 55, 2, 1), (2, 24, 19, 21, 2, 1), (1, 36, 6, 40, 1, 1), (1, 32, 1, 1, 1, 1)])
def test_depthwise_against_oracle(tb, torch_cuda, oracle, n, c, h, w, stride, pad):
    rng = np.random.default_rng(c * 100 + h)
    filt = rng.normal(0, 0.05, (c, 1, 3, 3)).astype(np.float32)
    x = (rng.random((n, c, h, w), dtype=np.float32) - 0.25).astype(np.float32)
    f = tb.SparseFilter(filt, c, c, 3, groups=c)
    want = oracle.host_depthwise_conv2d(x, filt, stride, pad)
    for _ in range(2):   # (the second call finds its tensor map in the cache)
        got = tb.cuda_sparse_conv2d(x, f, n, h, w, stride, pad)
        f.check()
        bad, max_rel, _ = oracle.compare(got, want)
        assert bad == 0, max_rel
    f.close()


@pytest.mark.parametrize("shape", [(2, 5, 4, 3), (1, 64, 33, 31), (3, 3, 70, 9), (2, 130, 1, 1)])
def test_layout_transposes_are_exact(tb, torch_cuda, shape):
    torch = torch_cuda
    n, c, h, w = shape
    x = torch.rand(shape, device="cuda")
    y = torch.full((n, h, w, c), float("nan"), device="cuda")
    tb.nchw_to_nhwc(x, y, n, c, h, w)
    assert torch.equal(y, x.permute(0, 2, 3, 1).contiguous())
    z = torch.full(shape, float("nan"), device="cuda")
    tb.nhwc_to_nchw(y, z, n, c, h, w)
    assert torch.equal(z, x)


def test_sharded_host_call_equals_single_call(tb, torch_cuda, oracle):
    """One filter per shard; with one visible GPU the shards share it, which still exercises
    the slicing, the worker threads and the per-shard error path."""
    rng = np.random.default_rng(21)
    filt = rng.normal(0, 0.05, (32, 16, 3, 3)).astype(np.float32)
    filt[rng.random(filt.shape) < 0.8] = 0
    x = rng.random((5, 16, 12, 12), dtype=np.float32)
    n_dev = torch_cuda.cuda.device_count()
    shards = 3
    filters = [tb.SparseFilter(filt, 16, 32, 3, device=g % n_dev) for g in range(shards)]
    got = tb.cuda_sparse_conv2d_sharded(x, filters, 5, 12, 12, 1, 1)
    single = tb.cuda_sparse_conv2d(x, filters[0], 5, 12, 12, 1, 1)
    assert np.array_equal(got, single)
    assert oracle.compare(got, oracle.host_conv2d(x, filt, 1, 1))[0] == 0


def test_device_info(tb, torch_cuda):
    sms, khz, lanes = tb.device_info(0)
    assert sms > 0 and khz > 100000 and lanes == 128


def test_pipelined_host_path_equals_the_blocking_one(tb, torch_cuda, oracle):
    rng = np.random.default_rng(33)
    filt = rng.normal(0, 0.05, (40, 24, 3, 3)).astype(np.float32)
    filt[rng.random(filt.shape) < 0.85] = 0
    f = tb.SparseFilter(filt, 24, 40, 3)
    xs = [np.ascontiguousarray(rng.random((3, 24, 16 + i, 16), dtype=np.float32)) for i in range(5)]
    outs = [np.full((3, 40, 16 + i, 16), np.nan, np.float32) for i in range(5)]
    for i, (x, y) in enumerate(zip(xs, outs)):           # more calls than slots: slots get reused
        tb.host_sync(0, i % 2)
        tb.cuda_sparse_conv2d_async(x, f, 3, 16 + i, 16, 1, 1, y, slot=i % 2)
    tb.host_sync(0, -1)
    for i, (x, y) in enumerate(zip(xs, outs)):
        assert np.array_equal(y, tb.cuda_sparse_conv2d(x, f, 3, 16 + i, 16, 1, 1))
        assert oracle.compare(y, oracle.host_conv2d(x, filt, 1, 1))[0] == 0
    with pytest.raises(tb.TetrisError):
        tb.cuda_sparse_conv2d_async(xs[0], f, 3, 16, 16, 1, 1, outs[0], slot=9)
    tb.release_workspace()


@pytest.mark.gpu
def test_layer_chain_replays_from_a_cuda_graph(tb, torch_cuda, oracle):
    """Two layers back to back (list kernel, then the tensor-core variant with its split-K
    zeroing), captured once into a CUDA graph and replayed: same results as the eager launches."""
    torch = torch_cuda
    rng = np.random.default_rng(5)
    f1w = rng.normal(0, 0.05, (64, 8, 3, 3)).astype(np.float32)
    f1w[rng.random(f1w.shape) < 0.8] = 0
    f2w = rng.normal(0, 0.05, (96, 64, 3, 3)).astype(np.float32)
    f2w[rng.random(f2w.shape) < 0.8] = 0
    f1, f2 = tb.SparseFilter(f1w, 8, 64, 3), tb.SparseFilter(f2w, 64, 96, 3)
    x = rng.random((2, 8, 20, 20), dtype=np.float32)
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    mid = torch.zeros(2, 20, 20, 64, device="cuda")
    out = torch.zeros(2, 20, 20, 96, device="cuda")

    def chain(st):
        tb.sparse_conv2d(f1, xin, mid, 2, 20, 20, 1, 1, cuda_stream=st, variant=tb.VARIANT_TILED)
        tb.sparse_conv2d(f2, mid, out, 2, 20, 20, 1, 1, cuda_stream=st, variant=tb.VARIANT_TENSOR)

    chain(torch.cuda.current_stream())       # eager once: one-time set-up happens outside the capture
    torch.cuda.synchronize()
    want = out.clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        chain(torch.cuda.current_stream())
    out.fill_(float("nan"))
    mid.fill_(float("nan"))
    g.replay()
    torch.cuda.synchronize()
    f2.check()
    assert torch.allclose(out, want, rtol=1e-5, atol=1e-6)
    y1 = oracle.host_conv2d(x, f1w, 1, 1)
    y2 = oracle.host_conv2d(y1, f2w, 1, 1)
    bad, _, _ = oracle.compare(out.cpu().numpy().transpose(0, 3, 1, 2), y2)
    assert bad == 0

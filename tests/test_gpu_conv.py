"""GPU: convolution parity through the C ABI -- golden vectors, seeded cases, edge cases and
size-independent properties at full workload size.

Bar: |got - want| <= 1e-4 * max(|got|, |want|) + 1e-5 against the CPU oracle (FP32 with a
different rounding sequence: the device fuses each multiply-add).
"""
import glob
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
VARIANTS = {"auto": 0, "generic": 1, "tiled": 2, "tensor": 4, "tensor16": 5}


def device_conv(tb, torch, f, x_nchw, stride, pad, variant=0, poison=True):
    """Run the device-pointer entry point: NHWC in, NHWC out; returns NCHW numpy."""
    n, ic, h, w = x_nchw.shape
    oh, ow = tb.out_extent(h, f.kernel_size_, stride, pad), tb.out_extent(w, f.kernel_size_, stride, pad)
    xin = torch.from_numpy(np.ascontiguousarray(x_nchw.transpose(0, 2, 3, 1))).cuda()
    out = torch.full((n, oh, ow, f.out_channel_), float("nan") if poison else 0.0,
                     dtype=torch.float32, device="cuda")
    tb.sparse_conv2d(f, xin, out, n, h, w, stride, pad, variant=variant)
    torch.cuda.synchronize()
    f.check()  # a tensor-core launch that gave up on a barrier would be reported here
    return out.cpu().numpy().transpose(0, 3, 1, 2)


def covers(variant, ks, stride, ic=4):
    """The tensor-core variant needs in_channel to be a multiple of 4, or at most 4; its
    split-FP16 form stride 1 and in_channel a multiple of 4, at least 8."""
    if variant == "tensor16":
        return stride == 1 and ic % 4 == 0 and ic >= 8 and ks <= 7
    if variant == "tensor":
        return ic % 4 == 0 or ic <= 4
    return True


def check(oracle, got, want):
    assert not np.isnan(got).any(), "output elements were left unwritten"
    bad, max_rel, n_floor = oracle.compare(got, want)
    assert bad == 0, "%d elements outside 1e-4 (max rel %.3g)" % (bad, max_rel)
    return max_rel


@pytest.mark.parametrize("variant", ["generic", "tiled", "tensor", "tensor16"])
@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[:-4])
def test_golden_vectors(tb, torch_cuda, oracle, path, variant):
    z = np.load(path)
    x, w, stride, pad, want = z["input"], z["filter"], int(z["stride"]), int(z["pad"]), z["output"]
    oc, ic, ks, _ = w.shape
    if not covers(variant, ks, stride, ic):
        pytest.skip("shape outside what this variant covers")
    f = tb.SparseFilter(w, ic, oc, ks)
    got = device_conv(tb, torch_cuda, f, x, stride, pad, VARIANTS[variant])
    check(oracle, got, want)
    if "all_ones" in path:
        assert np.array_equal(got, want)  # integer-valued sums are exact in any order


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[:-4])
def test_golden_vectors_host_entry_point(tb, torch_cuda, oracle, path):
    """Host NCHW in / host NCHW out, the CudaSparseConv2d-shaped call."""
    z = np.load(path)
    x, w, stride, pad, want = z["input"], z["filter"], int(z["stride"]), int(z["pad"]), z["output"]
    oc, ic, ks, _ = w.shape
    f = tb.SparseFilter(w, ic, oc, ks)
    keep = x.copy()
    got = tb.cuda_sparse_conv2d(x, f, x.shape[0], x.shape[2], x.shape[3], stride, pad)
    assert np.array_equal(x, keep)
    check(oracle, got, want)


SEEDED = [
    # N, IC, H, W, OC, KS, stride, pad, density, K, TIC
    (1, 64, 56, 56, 64, 3, 1, 1, 0.10, 16, 16),    # the single-layer configuration
    (2, 64, 56, 56, 64, 3, 1, 1, 0.10, 16, 16),    # even batch: image pairs
    (3, 32, 28, 28, 48, 3, 1, 1, 0.20, 16, 16),    # odd batch > 1
    (4, 24, 14, 14, 40, 3, 1, 1, 0.15, 16, 8),
    (2, 16, 7, 7, 32, 3, 1, 1, 0.20, 16, 16),
    (2, 3, 37, 41, 20, 3, 1, 1, 0.50, 16, 16),     # IC below one stage, ragged H/W
    (2, 40, 31, 29, 24, 3, 2, 1, 0.15, 16, 16),    # stride 2, odd extents
    (1, 16, 30, 30, 16, 3, 2, 0, 0.30, 8, 16),
    (2, 96, 28, 28, 255, 1, 1, 0, 0.20, 16, 32),   # OC not a multiple of anything
    (2, 384, 13, 13, 128, 1, 1, 0, 0.10, 16, 16),
    (2, 64, 28, 28, 128, 1, 2, 0, 0.20, 16, 16),   # 1x1 projection, stride 2
    (1, 35, 9, 200, 18, 3, 1, 1, 0.10, 8, 4),      # very wide and flat
    (1, 12, 200, 5, 18, 3, 1, 1, 0.10, 16, 16),    # very tall and thin
    (2, 8, 1, 1, 16, 1, 1, 0, 0.50, 16, 16),       # 1x1 image
    (2, 8, 2, 3, 16, 3, 1, 1, 0.50, 16, 16),
    (2, 3, 40, 36, 24, 7, 2, 3, 0.50, 16, 16),     # the 7x7 stride-2 stem shape
    (1, 6, 21, 19, 10, 5, 3, 2, 0.40, 8, 4),       # 5x5, stride 3
]


@pytest.mark.parametrize("variant", ["generic", "tiled", "tensor", "tensor16"])
@pytest.mark.parametrize("case", SEEDED, ids=lambda c: "n%d_ic%d_%dx%d_oc%d_k%d_s%d_p%d" % c[:8])
def test_seeded_cases_against_oracle(tb, torch_cuda, oracle, case, variant):
    n, ic, h, w, oc, ks, stride, pad, density, K, TIC = case
    rng = np.random.default_rng(hash(case[:8]) % (2 ** 32))
    filt = rng.normal(0, 0.05, (oc, ic, ks, ks)).astype(np.float32)
    filt[rng.random(filt.shape) >= density] = 0
    x = rng.random((n, ic, h, w), dtype=np.float32)
    x[rng.random(x.shape) < 0.5] = 0
    if not covers(variant, ks, stride, ic):
        pytest.skip("shape outside what this variant covers")
    f = tb.SparseFilter(filt, ic, oc, ks, TILE_IC=TIC, oc_block=K)
    got = device_conv(tb, torch_cuda, f, x, stride, pad, VARIANTS[variant])
    check(oracle, got, oracle.host_conv2d(x, filt, stride, pad))


def test_skewed_rows_and_empty_channels(tb, torch_cuda, oracle):
    """Magnitude-pruned layers have very uneven rows, some with no nonzeros at all."""
    rng = np.random.default_rng(9)
    oc, ic = 96, 64
    filt = rng.normal(0, 0.1, (oc, ic, 3, 3)).astype(np.float32)
    row_density = rng.beta(0.5, 3.0, oc)
    row_density[[5, 40, 95]] = 0.0
    for o in range(oc):
        filt[o][rng.random(filt[o].shape) >= row_density[o]] = 0
    x = rng.standard_normal((2, ic, 20, 20)).astype(np.float32)
    f = tb.SparseFilter(filt, ic, oc, 3)
    want = oracle.host_conv2d(x, filt, 1, 1)
    for v in (1, 2, 4, 5):
        got = device_conv(tb, torch_cuda, f, x, 1, 1, v)
        check(oracle, got, want)
        assert np.all(got[:, [5, 40, 95]] == 0)


def test_dense_filter_and_negative_inputs(tb, torch_cuda, oracle):
    rng = np.random.default_rng(10)
    filt = rng.normal(0, 0.05, (32, 16, 3, 3)).astype(np.float32)
    x = rng.standard_normal((2, 16, 12, 12)).astype(np.float32)
    f = tb.SparseFilter(filt, 16, 32, 3)
    check(oracle, device_conv(tb, torch_cuda, f, x, 1, 1, 2), oracle.host_conv2d(x, filt, 1, 1))


def test_empty_batch_and_bad_shapes(tb, torch_cuda):
    f = tb.SparseFilter(np.ones((16, 8, 3, 3), np.float32), 8, 16, 3)
    tb.sparse_conv2d(f, None, None, 0, 8, 8, 1, 1)  # empty batch: nothing to do, no error
    with pytest.raises(tb.TetrisError) as e:
        tb.sparse_conv2d(f, None, None, 1, 8, 8, 1, 1)
    assert e.value.status == 1
    with pytest.raises(tb.TetrisError):
        tb.sparse_conv2d(f, 1, 1, 1, 2, 2, 1, 0)  # image smaller than the kernel
    with pytest.raises(tb.TetrisError) as e:
        x = torch_cuda.zeros(1, 8, 8, 8, device="cuda")
        y = torch_cuda.zeros(1, 8, 8, 16, device="cuda")
        tb.sparse_conv2d(f, x, y, 1, 8, 8, 1, 1, variant=3)  # a retired variant number
    assert e.value.status == 1


def test_full_size_properties_vgg_layer(tb, torch_cuda, workloads):
    """At a full-size layer (VGG conv3_2, batch 16) the CPU oracle is too slow; check
    properties that hold at any size: the two kernels agree, the op is linear in its input,
    and a batch is the concatenation of its images."""
    torch = torch_cuda
    L = workloads.vgg19()[5]
    filt = workloads.make_filter("vgg19", 5, L)
    f = tb.SparseFilter(filt, L.IC, L.OC, L.KS)
    n = 16
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.rand(n, L.H, L.W, L.IC, device="cuda", generator=g)
    b = torch.rand(n, L.H, L.W, L.IC, device="cuda", generator=g)

    def run(x, variant, batch=n):
        out = torch.full((batch, L.H, L.W, L.OC), float("nan"), device="cuda")
        tb.sparse_conv2d(f, x, out, batch, L.H, L.W, 1, 1, variant=variant)
        return out

    ya = run(a, 2)
    assert not torch.isnan(ya).any()
    yg = run(a, 1)
    assert torch.allclose(ya, yg, rtol=1e-4, atol=1e-5)
    assert torch.allclose(ya, run(a, 4), rtol=1e-4, atol=1e-5)
    f.check()
    lin = run(2.0 * a + b, 2)
    assert torch.allclose(lin, 2.0 * ya + run(b, 2), rtol=1e-4, atol=1e-4)
    one = run(a[3:4].contiguous(), 2, batch=1)   # odd batch takes the other pairing mode
    assert torch.allclose(one[0], ya[3], rtol=1e-5, atol=1e-6)


def test_tensor_variant_long_accumulation(tb, torch_cuda, workloads, oracle):
    """A 512-channel 3x3 layer adds ~1700 tensor-core results per output.  The tensor core
    truncates when it adds into its accumulator; accumulated naively that drifts past the
    tolerance, so this is the case that checks the chain is cut and summed outside."""
    L = workloads.vgg19()[13]
    filt = workloads.make_filter("vgg19", 13, L)
    x = workloads.make_input("vgg19", 13, L, 2)
    f = tb.SparseFilter(filt, L.IC, L.OC, L.KS)
    got = device_conv(tb, torch_cuda, f, x, L.stride, L.pad, VARIANTS["tensor"])
    check(oracle, got, oracle.host_conv2d(x, filt, L.stride, L.pad))


def test_tensor_variant_stride2_full_width(tb, torch_cuda, workloads, oracle):
    """Stride 2 takes the loader's box-per-K-step mode (element strides in the tensor map)."""
    rng = np.random.default_rng(77)
    ic, oc, h = 64, 96, 30
    filt = rng.normal(0, 0.05, (oc, ic, 3, 3)).astype(np.float32)
    filt[rng.random(filt.shape) < 0.8] = 0
    x = rng.random((3, ic, h, h), dtype=np.float32)
    f = tb.SparseFilter(filt, ic, oc, 3)
    for stride, pad in ((2, 1), (2, 0), (3, 1)):
        got = device_conv(tb, torch_cuda, f, x, stride, pad, VARIANTS["tensor"])
        check(oracle, got, oracle.host_conv2d(x, filt, stride, pad))


def test_timing_harness_runs(tb, torch_cuda):
    filt = np.random.default_rng(0).normal(0, 0.05, (64, 64, 3, 3)).astype(np.float32)
    filt[np.random.default_rng(1).random(filt.shape) < 0.9] = 0
    f = tb.SparseFilter(filt, 64, 64, 3)
    x = torch_cuda.rand(1, 56, 56, 64, device="cuda")
    y = torch_cuda.empty(1, 56, 56, 64, device="cuda")
    torch_cuda.cuda.synchronize()
    before = tb.launch_count()
    ms = tb.timing_sparse_conv2d(f, x, y, 1, 56, 56, 1, 1, warm=3, repeat=10)
    assert 0.0 < ms < 50.0
    assert tb.launch_count() - before == 3 + 10   # warm + repeat launches, as the protocol says
    before = tb.launch_count()
    tb.timing_sparse_conv2d(f, x, y, 1, 56, 56, 1, 1)
    assert tb.launch_count() - before == tb.WARM + tb.REPEAT == 130


def test_tile_tuning_keeps_results_and_reports_a_time(tb, torch_cuda, oracle):
    rng = np.random.default_rng(31)
    filt = rng.normal(0, 0.05, (48, 32, 3, 3)).astype(np.float32)
    filt[rng.random(filt.shape) < 0.9] = 0
    x = rng.random((4, 32, 28, 28), dtype=np.float32)
    f = tb.SparseFilter(filt, 32, 48, 3)
    xin = torch_cuda.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    out = torch_cuda.empty(4, 28, 28, 48, device="cuda")
    ms = tb.tune_sparse_conv2d(f, xin, out, 4, 28, 28, 1, 1, max_candidates=6)
    assert 0.0 < ms < 10.0
    got = device_conv(tb, torch_cuda, f, x, 1, 1, 0)   # launches now use the tuned tile shape
    check(oracle, got, oracle.host_conv2d(x, filt, 1, 1))
    got = device_conv(tb, torch_cuda, f, x[:3], 1, 1, 0)  # another shape: falls back to the model
    check(oracle, got, oracle.host_conv2d(x[:3], filt, 1, 1))


def test_auto_choice_reports_the_kernel_an_automatic_launch_uses(tb, torch_cuda, oracle):
    """tetris_conv2d_choice: a layer outside the tensor-core variant's cover (in_channel not a
    multiple of 4 and more than 4) stays on the list kernel; a dense-ish 3x3 layer is given to the tensor cores
    by the cost model; whatever is reported, the automatic launch gives the right answer."""
    rng = np.random.default_rng(41)
    filt3 = rng.normal(0, 0.05, (32, 6, 3, 3)).astype(np.float32)
    f3 = tb.SparseFilter(filt3, 6, 32, 3)
    assert tb.auto_choice(f3, 2, 32, 32, 1, 1) == tb.VARIANT_TILED
    filt = rng.normal(0, 0.05, (128, 128, 3, 3)).astype(np.float32)
    filt[rng.random(filt.shape) < 0.5] = 0
    f = tb.SparseFilter(filt, 128, 128, 3)
    x = rng.random((4, 128, 28, 28), dtype=np.float32)
    choice = tb.auto_choice(f, 4, 28, 28, 1, 1)
    assert choice in (tb.VARIANT_TENSOR, tb.VARIANT_TENSOR16)
    got = device_conv(tb, torch_cuda, f, x, 1, 1, 0)
    check(oracle, got, oracle.host_conv2d(x, filt, 1, 1))
    # after tuning the answer is whichever kernel was faster when timed; it must be one of the two
    xin = torch_cuda.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    out = torch_cuda.empty(4, 28, 28, 128, device="cuda")
    tb.tune_sparse_conv2d(f, xin, out, 4, 28, 28, 1, 1, max_candidates=4)
    assert tb.auto_choice(f, 4, 28, 28, 1, 1) in (tb.VARIANT_TILED, tb.VARIANT_TENSOR, tb.VARIANT_TENSOR16)


@pytest.mark.parametrize("seed", range(10))
def test_tensor_variant_random_shapes(tb, torch_cuda, oracle, seed):
    """Ragged shapes for the tensor-core variant: channel counts that leave partial K chunks and
    partial channel tiles, filters of 1 to 7 taps a side, strides 1-3, images smaller than a
    tile, batches that share a tile, outputs that are not a multiple of four channels."""
    rng = np.random.default_rng(1000 + seed)
    ks = int(rng.choice([1, 2, 3, 5, 7]))
    stride = int(rng.choice([1, 1, 2, 3]))
    pad = int(rng.integers(0, ks))
    ic = int(rng.choice([1, 2, 3])) if seed % 3 == 0 else 4 * int(rng.integers(1, 40))
    oc = int(rng.choice([1, 3, 30, 64, 65, 130, 200]))
    h = int(rng.integers(ks, 40))
    w = int(rng.integers(ks, 40))
    n = int(rng.integers(1, 6))
    filt = rng.normal(0, 0.05, (oc, ic, ks, ks)).astype(np.float32)
    filt[rng.random(filt.shape) < rng.choice([0.0, 0.7, 0.95])] = 0
    x = rng.random((n, ic, h, w), dtype=np.float32) - 0.3
    f = tb.SparseFilter(filt, ic, oc, ks)
    got = device_conv(tb, torch_cuda, f, x, stride, pad, VARIANTS["tensor"])
    check(oracle, got, oracle.host_conv2d(x, filt, stride, pad))


def test_tensor_variant_against_list_kernel_many_shapes(tb, torch_cuda):
    """Sixty seeded mid-size shapes (both loader modes, split K ranges, folded stems, partial
    tiles), tensor-core variant against the list kernel on the device; then one full-size layer
    launched ten times: a race in the tensor-core pipeline shows up as a launch that differs."""
    torch = torch_cuda
    rng = np.random.default_rng(2024)

    def agree(ya, yb):
        err = (ya - yb).abs()
        return not bool((((err > 1e-4 * ya.abs()) & (err > 1e-5)) | torch.isnan(yb)).any())

    for _ in range(60):
        ks = int(rng.choice([1, 3, 3, 3, 5]))
        stride = int(rng.choice([1, 1, 1, 2]))
        pad = int(rng.integers(0, ks))
        ic = int(rng.choice([3, 4, 8, 32, 64, 96, 128, 160, 256]))
        oc = int(rng.choice([16, 64, 100, 128, 192, 256, 384]))
        h, w = int(rng.integers(max(ks, 7), 70)), int(rng.integers(max(ks, 7), 70))
        n = int(rng.integers(1, 20))
        filt = rng.normal(0, 0.05, (oc, ic, ks, ks)).astype(np.float32)
        filt[rng.random(filt.shape) < rng.choice([0.5, 0.8, 0.95])] = 0
        f = tb.SparseFilter(filt, ic, oc, ks)
        oh, ow = tb.out_extent(h, ks, stride, pad), tb.out_extent(w, ks, stride, pad)
        x = torch.rand(n, h, w, ic, device="cuda") - 0.3
        ya = torch.full((n, oh, ow, oc), float("nan"), device="cuda")
        yb = torch.full((n, oh, ow, oc), float("nan"), device="cuda")
        tb.sparse_conv2d(f, x, ya, n, h, w, stride, pad, variant=tb.VARIANT_TILED)
        tb.sparse_conv2d(f, x, yb, n, h, w, stride, pad, variant=tb.VARIANT_TENSOR)
        torch.cuda.synchronize()
        f.check()
        assert agree(ya, yb), dict(ks=ks, stride=stride, pad=pad, ic=ic, oc=oc, h=h, w=w, n=n)

    filt = rng.normal(0, 0.05, (256, 128, 3, 3)).astype(np.float32)
    filt[rng.random(filt.shape) < 0.85] = 0
    f = tb.SparseFilter(filt, 128, 256, 3)
    x = torch.rand(16, 56, 56, 128, device="cuda")
    ref = torch.empty(16, 56, 56, 256, device="cuda")
    tb.sparse_conv2d(f, x, ref, 16, 56, 56, 1, 1, variant=tb.VARIANT_TILED)
    for _ in range(10):
        y = torch.full((16, 56, 56, 256), float("nan"), device="cuda")
        tb.sparse_conv2d(f, x, y, 16, 56, 56, 1, 1, variant=tb.VARIANT_TENSOR)
        torch.cuda.synchronize()
        f.check()
        assert agree(ref, y)


@pytest.mark.parametrize("variant", ["generic", "tiled", "tensor", "tensor16", "auto"])
def test_output_offset_by_one_float(tb, torch_cuda, oracle, variant):
    """An output that is only 4-byte aligned (a view one float into a buffer) is legal: the
    kernels must leave their 16-byte stores and adds for such a pointer."""
    torch = torch_cuda
    rng = np.random.default_rng(55)
    for (n, ic, h, oc, ks, stride, pad) in ((2, 64, 28, 128, 3, 1, 1), (3, 256, 14, 64, 1, 1, 0), (16, 128, 28, 128, 3, 1, 1)):
        filt = rng.normal(0, 0.05, (oc, ic, ks, ks)).astype(np.float32)
        filt[rng.random(filt.shape) < 0.8] = 0
        x = rng.random((n, ic, h, h), dtype=np.float32)
        f = tb.SparseFilter(filt, ic, oc, ks)
        oh = tb.out_extent(h, ks, stride, pad)
        xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
        buf = torch.full((n * oh * oh * oc + 8,), float("nan"), device="cuda")
        out = buf[1:1 + n * oh * oh * oc]
        assert out.data_ptr() % 16 == 4
        tb.sparse_conv2d(f, xin, out, n, h, h, stride, pad, variant=VARIANTS[variant])
        torch.cuda.synchronize()
        f.check()
        got = out.view(n, oh, oh, oc).cpu().numpy().transpose(0, 3, 1, 2)
        check(oracle, got, oracle.host_conv2d(x, filt, stride, pad))
        assert bool(torch.isnan(buf[0])) and bool(torch.isnan(buf[1 + n * oh * oh * oc:]).all())


def test_auto_falls_back_when_no_list_tile_fits(tb, torch_cuda, oracle):
    """A dense 7x7 filter with a caller-chosen stage of 64 channels makes list pieces too long for
    any tile geometry of the list kernel; an automatic launch must still run (tensor-core variant
    or generic kernel) instead of reporting the shape as unsupported."""
    rng = np.random.default_rng(56)
    ic, oc, ks = 64, 32, 7
    filt = rng.normal(0, 0.05, (oc, ic, ks, ks)).astype(np.float32)
    x = rng.random((2, ic, 20, 20), dtype=np.float32)
    f = tb.SparseFilter(filt, ic, oc, ks, TILE_IC=64, oc_block=16)
    assert tb.auto_choice(f, 2, 20, 20, 1, 3) in (tb.VARIANT_TENSOR, tb.VARIANT_GENERIC, tb.VARIANT_TILED)
    got = device_conv(tb, torch_cuda, f, x, 1, 3, VARIANTS["auto"])
    check(oracle, got, oracle.host_conv2d(x, filt, 1, 3))


@pytest.mark.parametrize("seed", range(12))
def test_tensor16_random_shapes(tb, torch_cuda, oracle, seed):
    """Ragged shapes for the split-FP16 tensor-core variant: partial K chunks and channel tiles,
    1x1 (with and without padding) to 7x7 filters, images smaller and larger than a tile, several
    images per tile, tall and wide images, outputs that are not a multiple of four channels."""
    rng = np.random.default_rng(3000 + seed)
    ks = int(rng.choice([1, 1, 3, 3, 3, 5, 7]))
    pad = int(rng.integers(0, ks)) if seed % 2 else ks // 2
    ic = 4 * int(rng.integers(2, 70))
    oc = int(rng.choice([1, 3, 30, 64, 65, 128, 130, 200, 256]))
    h = int(rng.integers(ks, 45))
    w = int(rng.integers(ks, 45))
    n = int(rng.integers(1, 7))
    filt = rng.normal(0, 0.05, (oc, ic, ks, ks)).astype(np.float32)
    filt[rng.random(filt.shape) < rng.choice([0.0, 0.7, 0.95])] = 0
    x = rng.random((n, ic, h, w), dtype=np.float32) - 0.3
    f = tb.SparseFilter(filt, ic, oc, ks)
    got = device_conv(tb, torch_cuda, f, x, 1, pad, VARIANTS["tensor16"])
    check(oracle, got, oracle.host_conv2d(x, filt, 1, pad))


def test_tensor16_value_ranges(tb, torch_cuda, oracle):
    """Split FP16 keeps FP32 accuracy over the range FP16 can hold -- large activations (up to
    ~3e4), tiny ones (1e-7: below FP16's normal range, the absolute error stays far under the
    floor), weights of very different magnitudes (|w| from 1e-6 to 30) -- and a launch whose
    activations do not fit FP16's window (2048 and more, or all below 2^-8) is recomputed by the
    split-TF32 variant behind it: every case has to meet the bar of the path, with the absolute
    floor scaled like the activations."""
    torch = torch_cuda
    rng = np.random.default_rng(77)
    n, ic, h, oc = 2, 96, 20, 72
    filt = rng.normal(0, 0.05, (oc, ic, 3, 3)).astype(np.float32)
    filt[rng.random(filt.shape) < 0.8] = 0
    base = rng.random((n, ic, h, h), dtype=np.float32)
    f = tb.SparseFilter(filt, ic, oc, 3)
    for scale in (1.0, 64.0, 2000.0, 3.0e4, 1.0e-2, 1.0e-7, 1.0e5):
        x = (base * np.float32(scale)).astype(np.float32)
        got = device_conv(tb, torch_cuda, f, x, 1, 1, VARIANTS["tensor16"])
        want = oracle.host_conv2d(x, filt, 1, 1)
        # the bar of the path, with its absolute floor scaled like the data
        bad, max_rel, _ = oracle.compare(got / np.float32(scale), want / np.float32(scale))
        assert bad == 0, "activations x %g: %d elements off (max rel %.3g)" % (scale, bad, max_rel)
    mixed = base.copy()                          # tiny and ordinary activations side by side
    mixed[:, ::2] *= np.float32(1e-6)
    got = device_conv(tb, torch_cuda, f, mixed, 1, 1, VARIANTS["tensor16"])
    bad, max_rel, _ = oracle.compare(got, oracle.host_conv2d(mixed, filt, 1, 1))
    assert bad == 0, "tiny and ordinary activations mixed: %d elements off (max rel %.3g)" % (bad, max_rel)
    x = base.copy()                              # after an out-of-range launch the next one is a plain FP16 launch again
    got = device_conv(tb, torch_cuda, f, x, 1, 1, VARIANTS["tensor16"])
    bad, max_rel, _ = oracle.compare(got, oracle.host_conv2d(x, filt, 1, 1))
    assert bad == 0, "plain launch after an out-of-range one: %d elements off (max rel %.3g)" % (bad, max_rel)
    # output channels whose weights differ by seven orders of magnitude share one filter-wide
    # scale; each channel is held to the bar of the path with the floor scaled like its weights
    # (against a floor of 1e-5 the CPU path's own FP32 rounding would show on the large channels)
    chan = np.exp(rng.uniform(np.log(2e-5), np.log(600.0), (oc, 1, 1, 1))).astype(np.float32)
    wide = filt * chan
    f2 = tb.SparseFilter(wide, ic, oc, 3)
    got = device_conv(tb, torch_cuda, f2, base, 1, 1, VARIANTS["tensor16"]) / chan.reshape(1, oc, 1, 1)
    want = oracle.host_conv2d(base, wide, 1, 1) / chan.reshape(1, oc, 1, 1)
    bad, max_rel, _ = oracle.compare(got, want)
    err = np.abs(got - want) - (1e-4 * np.maximum(np.abs(got), np.abs(want)) + 1e-5)
    worst = np.unravel_index(np.argmax(err), got.shape)
    assert bad == 0, "weights of very different magnitudes: %d elements off (max rel %.3g), worst at %s: %g vs %g" % (
        bad, max_rel, worst, got[worst], want[worst])


def test_tensor16_against_tensor_many_shapes_and_repeats(tb, torch_cuda):
    """Forty seeded mid-size shapes, split-FP16 against the list kernel on the device; then a
    full-size layer launched ten times: a race in the pipeline shows up as a launch that differs."""
    torch = torch_cuda
    torch.manual_seed(2025)
    rng = np.random.default_rng(2025)

    def agree(ya, yb):
        err = (ya - yb).abs()
        return not bool((((err > 1e-4 * ya.abs()) & (err > 1e-5)) | torch.isnan(yb)).any())

    for _ in range(40):
        ks = int(rng.choice([1, 3, 3, 3, 5]))
        pad = int(rng.integers(0, ks))
        ic = int(rng.choice([8, 32, 64, 96, 128, 160, 256]))  # (beyond ~6000 taps two FP32 summation orders differ by more than the bar)
        oc = int(rng.choice([16, 64, 100, 128, 192, 256, 384]))
        h, w = int(rng.integers(max(ks, 7), 70)), int(rng.integers(max(ks, 7), 70))
        n = int(rng.integers(1, 20))
        filt = rng.normal(0, 0.05, (oc, ic, ks, ks)).astype(np.float32)
        filt[rng.random(filt.shape) < rng.choice([0.5, 0.8, 0.95])] = 0
        f = tb.SparseFilter(filt, ic, oc, ks)
        oh, ow = tb.out_extent(h, ks, 1, pad), tb.out_extent(w, ks, 1, pad)
        x = torch.rand(n, h, w, ic, device="cuda") - 0.3
        ya = torch.full((n, oh, ow, oc), float("nan"), device="cuda")
        yb = torch.full((n, oh, ow, oc), float("nan"), device="cuda")
        tb.sparse_conv2d(f, x, ya, n, h, w, 1, pad, variant=tb.VARIANT_TILED)
        tb.sparse_conv2d(f, x, yb, n, h, w, 1, pad, variant=tb.VARIANT_TENSOR16)
        torch.cuda.synchronize()
        f.check()
        assert agree(ya, yb), dict(ks=ks, pad=pad, ic=ic, oc=oc, h=h, w=w, n=n)

    filt = rng.normal(0, 0.05, (256, 128, 3, 3)).astype(np.float32)
    filt[rng.random(filt.shape) < 0.85] = 0
    f = tb.SparseFilter(filt, 128, 256, 3)
    x = torch.rand(16, 56, 56, 128, device="cuda")
    ref = torch.empty(16, 56, 56, 256, device="cuda")
    tb.sparse_conv2d(f, x, ref, 16, 56, 56, 1, 1, variant=tb.VARIANT_TILED)
    for _ in range(10):
        y = torch.full((16, 56, 56, 256), float("nan"), device="cuda")
        tb.sparse_conv2d(f, x, y, 16, 56, 56, 1, 1, variant=tb.VARIANT_TENSOR16)
        torch.cuda.synchronize()
        f.check()
        assert agree(ref, y)


@pytest.mark.parametrize("case", [(19, 64, 32, 32, 128, 3, 1), (20, 128, 28, 28, 128, 3, 1), (150, 96, 14, 14, 64, 3, 1),
                                  (5, 64, 40, 40, 100, 1, 0)],
                         ids=lambda c: "n%d_ic%d_%dx%d_oc%d_k%d" % c[:6])
def test_tensor16_last_wave_split(tb, torch_cuda, oracle, case):
    """Shapes whose tiles leave a small last wave on a 148-SM part, so that the split-FP16 variant
    cuts those tiles into K slices and adds them up through its scratch blocks: results against
    the oracle, rectified as well, and bit-identical from launch to launch (the slices are added
    in slice order whoever finishes last)."""
    torch = torch_cuda
    n, ic, h, w, oc, ks, pad = case
    rng = np.random.default_rng(4000 + n)
    filt = rng.normal(0, 0.05, (oc, ic, ks, ks)).astype(np.float32)
    filt[rng.random(filt.shape) < 0.8] = 0
    x = rng.random((n, ic, h, w), dtype=np.float32) - 0.3
    f = tb.SparseFilter(filt, ic, oc, ks)
    want = oracle.host_conv2d(x, filt, 1, pad)
    got = device_conv(tb, torch_cuda, f, x, 1, pad, VARIANTS["tensor16"])
    check(oracle, got, want)
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    oh, ow = want.shape[2], want.shape[3]
    outs = []
    for _ in range(3):
        out = torch.full((n, oh, ow, oc), float("nan"), device="cuda")
        tb.sparse_conv2d_fused(f, xin, out, n, h, w, 1, pad, variant=VARIANTS["tensor16"], relu=True)
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy())
    f.check()
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    assert oracle.compare(outs[0].transpose(0, 3, 1, 2), np.maximum(want, 0))[0] == 0


@pytest.mark.parametrize("variant", ["tensor", "tensor16"])
def test_bounded_wait_gives_up_and_the_next_launch_passes(tb, torch_cuda, oracle, variant):
    """Failure detection without a GPU fault: with every CTA's first activation load left out
    (tetris_test_inject) a barrier wait of the tensor-core kernel runs out after a short poll
    limit; the launch returns normally, tetris_filter_check reports TETRIS_ERR_CUDA exactly once,
    the context stays usable, and the next launch of the same filter matches the oracle.  (The
    reference kernels have no waits that can fail; the give-up path guards this design's
    producer/consumer pipeline.)"""
    torch = torch_cuda
    rng = np.random.default_rng(4242)
    n, ic, h, w, oc, ks, pad = 2, 64, 24, 24, 128, 3, 1
    filt = (rng.standard_normal((oc, ic, ks, ks)) * (rng.random((oc, ic, ks, ks)) >= 0.8)).astype(np.float32)
    x = rng.random((n, ic, h, w), dtype=np.float32)
    want = oracle.host_conv2d(x, filt, 1, pad, threads=True, skip_zero=True)
    f = tb.SparseFilter(filt, ic, oc, ks)
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    out = torch.full((n, h, w, oc), float("nan"), device="cuda")
    v = VARIANTS[variant]
    tb.sparse_conv2d(f, xin, out, n, h, w, 1, pad, variant=v)
    torch.cuda.synchronize()
    f.check()
    tb.test_inject(1, 2048)
    try:
        tb.sparse_conv2d(f, xin, out, n, h, w, 1, pad, variant=v)   # returns; its output is unspecified
        torch.cuda.synchronize()                                    # no CUDA error: the kernel gave up by itself
        with pytest.raises(tb.TetrisError) as err:
            f.check()
        assert err.value.status == 2, err.value                     # TETRIS_ERR_CUDA
    finally:
        tb.test_inject(0)
    f.check()                                                       # reported once, then cleared
    out.fill_(float("nan"))
    tb.sparse_conv2d(f, xin, out, n, h, w, 1, pad, variant=v)
    torch.cuda.synchronize()
    f.check()
    got = out.cpu().numpy().transpose(0, 3, 1, 2)
    assert not np.isnan(got).any()
    bad, max_rel, _ = oracle.compare(got, want)
    assert bad == 0, "%d elements differ after the recovery (max rel %.3g)" % (bad, max_rel)
    f.close()


@pytest.mark.parametrize("case", [
    # (n, ic, h, w, oc, ks, pad): 1x1 and short-K layers on images whose tiles take the TMA-store epilogue of the
    # split-TF32 kernel: 128-pixel tiles, tiles that span the image's height, channel counts that end inside a
    # 32-channel box, images that end inside a tile
    (3, 64, 32, 32, 36, 1, 0), (2, 32, 32, 32, 96, 1, 0), (2, 64, 40, 24, 100, 1, 0), (1, 128, 12, 40, 64, 1, 0),
    (2, 16, 50, 44, 256, 1, 0), (16, 64, 56, 56, 256, 1, 0), (2, 8, 30, 64, 32, 3, 1), (1, 96, 7, 32, 160, 1, 0)])
@pytest.mark.parametrize("relu", [False, True])
def test_tensor_variant_short_k_store_path(tb, torch_cuda, oracle, case, relu):
    torch = torch_cuda
    n, ic, h, w, oc, ks, pad = case
    rng = np.random.default_rng(n * 1000 + oc)
    filt = (rng.standard_normal((oc, ic, ks, ks)) * 0.1 * (rng.random((oc, ic, ks, ks)) >= 0.7)).astype(np.float32)
    x = (rng.random((n, ic, h, w), dtype=np.float32) - 0.3).astype(np.float32)
    imgs = [0, n - 1] if n > 2 else list(range(n))
    want = oracle.host_conv2d(x[imgs], filt, 1, pad, threads=True, skip_zero=True)
    if relu:
        want = np.maximum(want, 0)
    f = tb.SparseFilter(filt, ic, oc, ks)
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    oh, ow = want.shape[2], want.shape[3]
    out = torch.full((n, oh, ow, oc), float("nan"), device="cuda")
    for _ in range(2):
        out.fill_(float("nan"))
        if relu:
            tb.sparse_conv2d_fused(f, xin, out, n, h, w, 1, pad, variant=VARIANTS["tensor"], relu=True)
        else:
            tb.sparse_conv2d(f, xin, out, n, h, w, 1, pad, variant=VARIANTS["tensor"])
        torch.cuda.synchronize()
        f.check()
        got = out[imgs].cpu().numpy().transpose(0, 3, 1, 2)
        assert not np.isnan(out.cpu().numpy()).any(), "output elements were left unwritten"
        bad, max_rel, _ = oracle.compare(got, want)
        assert bad == 0, "%d elements differ (max rel %.3g)" % (bad, max_rel)
    f.close()

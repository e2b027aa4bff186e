"""GPU: every layer of the five benchmark workloads against the CPU oracle, through the C ABI.

Two sweeps:

* `test_layer_batch1_and_batch2`: each layer of `single`, `vgg19`, `resnet50`, `mobilenet` and
  `yolov3` at batch 1 and batch 2 (odd and even image pairing, images packed into one tile on
  the small late layers; plus `vgg19_s99`, VGG-19 pruned to 99 %, where the tuner picks the list
  kernel on several layers) through the automatic choice *after* tuning -- the configuration the
  benchmark times -- and through the forced tensor-core and list kernels where they cover the
  shape.  The whole output is compared with the oracle (HostConv2d, Tetris/tensor_utils.cc:136-170;
  per-plane for the depthwise layers).
* `test_full_size_batch16_slice`: each VGG-19 and YOLOv3 layer at the benchmark's batch 16;
  images 0 and 15 are compared on a 16-channel slice of the output (the oracle on a slice of the
  filter is cheap, the device runs the whole layer).

Bar (as the reference's self-check, Tetris/spconv2d.cc:430-441 with TensorEqual,
Tetris/tensor_utils.cc:17-34, widened to the path's 1e-4 relative):
|got - want| <= 1e-4 * max(|got|, |want|) + 1e-5.  Every case also reports the largest
relative error and how many elements passed only through the 1e-5 floor; with
TETRIS_PARITY_REPORT=<file> set the figures are appended there as JSON lines.
"""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _catalogue():
    from conftest import load_package
    import importlib
    load_package()
    return importlib.import_module("tetris_b200.workloads")


_WL = _catalogue()
SWEEP = [(w, i) for w in ("single", "vgg19", "resnet50", "mobilenet", "yolov3", "vgg19_s99")
         for i in range(len(_WL.WORKLOADS[w]()))]
FULL = [(w, i) for w in ("vgg19", "yolov3") for i in range(len(_WL.WORKLOADS[w]()))]


def _id(case):
    w, i = case
    return "%s-%02d-%s" % (w, i, _WL.WORKLOADS[w]()[i].name)


def _report(record):
    path = os.environ.get("TETRIS_PARITY_REPORT")
    if path:
        with open(path, "a") as fh:
            fh.write(json.dumps(record) + "\n")


def _assess(oracle, got, want, what):
    assert not np.isnan(got).any(), "%s: output elements were left unwritten" % what
    bad, max_rel, n_floor = oracle.compare(got, want)
    assert bad == 0, "%s: %d of %d elements outside 1e-4*|y| + 1e-5 (max rel %.3g)" % (
        what, bad, got.size, max_rel)
    return {"max_rel": max_rel, "n_floor": n_floor, "max_abs": float(np.abs(got - want).max()),
            "elements": int(got.size)}


def _variants(tb, L):
    """(label, variant, tuned) triples that cover this layer."""
    if L.groups != 1:
        return [("auto", tb.VARIANT_AUTO, False)]
    v = [("auto_tuned", tb.VARIANT_AUTO, True), ("tiled", tb.VARIANT_TILED, False)]
    if L.IC % 4 == 0 or L.IC <= 4:
        v.append(("tensor", tb.VARIANT_TENSOR, False))
    if L.stride == 1 and L.IC % 4 == 0 and L.IC >= 8:
        v.append(("tensor16", tb.VARIANT_TENSOR16, False))
    return v


@pytest.mark.parametrize("case", SWEEP, ids=_id)
def test_layer_batch1_and_batch2(tb, torch_cuda, oracle, case):
    torch = torch_cuda
    workload, idx = case
    L = _WL.WORKLOADS[workload]()[idx]
    filt = _WL.make_filter(workload, idx, L)
    x3 = _WL.make_input(workload, idx, L, 3)  # image 0 is the batch-1 run, images 1-2 the batch-2 run
    if L.groups != 1:
        want = oracle.host_depthwise_conv2d(x3, filt, L.stride, L.pad)
    else:
        want = oracle.host_conv2d(x3, filt, L.stride, L.pad, threads=True, skip_zero=True)
    f = tb.SparseFilter(filt, L.IC, L.OC, L.KS, groups=L.groups)
    oh, ow = want.shape[2], want.shape[3]
    for lo, hi in ((0, 1), (1, 3)):
        n = hi - lo
        xin = torch.from_numpy(np.ascontiguousarray(x3[lo:hi].transpose(0, 2, 3, 1))).cuda()
        for label, variant, tuned in _variants(tb, L):
            out = torch.full((n, oh, ow, L.OC), float("nan"), device="cuda")
            if tuned:
                tb.tune_sparse_conv2d(f, xin, out, n, L.H, L.W, L.stride, L.pad)
                out.fill_(float("nan"))
            tb.sparse_conv2d(f, xin, out, n, L.H, L.W, L.stride, L.pad, variant=variant)
            torch.cuda.synchronize()
            f.check()
            got = out.cpu().numpy().transpose(0, 3, 1, 2)
            rec = _assess(oracle, got, want[lo:hi], "%s %s batch %d %s" % (workload, L.name, n, label))
            rec.update(workload=workload, layer=L.name, batch=n, variant=label)
            if tuned:
                rec["kernel"] = tb.auto_choice(f, n, L.H, L.W, L.stride, L.pad)
            _report(rec)
    f.close()


@pytest.mark.parametrize("case", FULL, ids=_id)
def test_full_size_batch16_slice(tb, torch_cuda, oracle, case):
    torch = torch_cuda
    workload, idx = case
    L = _WL.WORKLOADS[workload]()[idx]
    filt = _WL.make_filter(workload, idx, L)
    n = 16
    g = torch.Generator(device="cuda").manual_seed(7000 + idx)
    x = torch.rand(n, L.H, L.W, L.IC, device="cuda", generator=g)
    x = x * (torch.rand(x.shape, device="cuda", generator=g) >= 0.5)
    oh, ow = _WL.out_extent(L.H, L.KS, L.stride, L.pad), _WL.out_extent(L.W, L.KS, L.stride, L.pad)
    f = tb.SparseFilter(filt, L.IC, L.OC, L.KS)
    out = torch.empty(n, oh, ow, L.OC, device="cuda")
    tb.tune_sparse_conv2d(f, x, out, n, L.H, L.W, L.stride, L.pad)
    out.fill_(float("nan"))
    tb.sparse_conv2d(f, x, out, n, L.H, L.W, L.stride, L.pad)
    torch.cuda.synchronize()
    f.check()
    assert not bool(torch.isnan(out).any()), "output elements were left unwritten"
    # a 16-channel slice that moves with the layer, so that over the catalogue every part of a
    # channel tile (first, last, partial) is looked at
    oc0 = min(max(L.OC - 16, 0), (idx * 24) % max(L.OC, 1))
    oc1 = min(L.OC, oc0 + 16)
    imgs = [0, n - 1]
    xs = x[imgs].permute(0, 3, 1, 2).contiguous().cpu().numpy()
    want = oracle.host_conv2d(xs, filt[oc0:oc1], L.stride, L.pad, threads=True, skip_zero=True)
    got = out[imgs][..., oc0:oc1].permute(0, 3, 1, 2).contiguous().cpu().numpy()
    rec = _assess(oracle, got, want, "%s %s batch 16 channels %d..%d" % (workload, L.name, oc0, oc1))
    rec.update(workload=workload, layer=L.name, batch=n, variant="auto_tuned",
               kernel=tb.auto_choice(f, n, L.H, L.W, L.stride, L.pad), oc_slice=[oc0, oc1])
    _report(rec)
    f.close()

"""CPU: the synthetic workload catalogue has the networks' layer shapes and is seeded."""
import numpy as np
import pytest


def dense_gflop(layers, batch, wl):
    tot = 0.0
    for L in layers:
        oh, ow = wl.out_extent(L.H, L.KS, L.stride, L.pad), wl.out_extent(L.W, L.KS, L.stride, L.pad)
        per_oc = 1 if L.groups != 1 else L.IC
        tot += 2.0 * batch * oh * ow * L.OC * per_oc * L.KS * L.KS
    return tot / 1e9


def test_layer_counts(workloads):
    assert len(workloads.single_layer()) == 1
    assert len(workloads.vgg19()) == 16
    assert len(workloads.resnet50()) == 53
    assert len(workloads.mobilenet_v1()) == 27
    assert len(workloads.yolov3()) == 75


def test_dense_flops_match_the_networks(workloads):
    assert dense_gflop(workloads.vgg19(), 1, workloads) == pytest.approx(39.0, rel=0.01)
    assert dense_gflop(workloads.resnet50(), 1, workloads) == pytest.approx(8.17, rel=0.01)
    assert dense_gflop(workloads.mobilenet_v1(), 1, workloads) == pytest.approx(1.14, rel=0.01)
    assert dense_gflop(workloads.yolov3(), 16, workloads) == pytest.approx(1053.8, rel=0.01)


def test_shapes_chain(workloads):
    y = workloads.yolov3()
    assert (y[0].H, y[0].IC, y[0].OC) == (416, 3, 32)
    assert {L.IC for L in y} >= {768, 384} and {L.OC for L in y} >= {255}
    assert y[-1].H == 52 and y[-1].OC == 255
    r = workloads.resnet50()
    assert (r[0].KS, r[0].stride, r[0].pad) == (7, 2, 3) and r[-1].H == 7
    m = workloads.mobilenet_v1()
    assert m[1].groups == 32 and m[-1].OC == 1024 and m[-1].H == 7


def test_generators_are_seeded_and_have_the_stated_distributions(workloads):
    L = workloads.single_layer()[0]
    w1, w2 = workloads.make_filter("single", 0, L), workloads.make_filter("single", 0, L)
    assert np.array_equal(w1, w2) and w1.shape == (64, 64, 3, 3)
    assert np.count_nonzero(w1) == w1.size - round(0.9 * w1.size)
    assert abs(float(w1[w1 != 0].std()) - 0.05) < 0.005
    x = workloads.make_input("single", 0, L, 1)
    assert x.shape == (1, 64, 56, 56) and 0.0 <= x.min() and x.max() < 1.0
    assert abs(float((x == 0).mean()) - 0.5) < 0.01
    v = workloads.vgg19()
    sp = [workloads.layer_sparsity("vgg19", i, l) for i, l in enumerate(v)]
    assert sp[0] == 0.5 and all(0.80 <= s <= 0.95 for s in sp[1:]) and len(set(sp)) > 8
    dw = workloads.mobilenet_v1()[1]
    assert np.count_nonzero(workloads.make_filter("mobilenet", 1, dw)) == 32 * 9


def test_layer_costs_formula(workloads):
    L = workloads.single_layer()[0]
    flops, nbytes = workloads.layer_costs(L, 1, 3686)
    assert flops == 2 * 3686 * 56 * 56
    assert nbytes == 4 * 64 * 56 * 56 * 2 + 8 * 3686 + 4 * 65

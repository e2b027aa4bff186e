"""CPU: the oracle restatement against the golden vectors and the compiled reference."""
import glob
import os

import numpy as np
import pytest

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def _load(path):
    z = np.load(path)
    return z["input"], z["filter"], int(z["stride"]), int(z["pad"]), z["output"]


def test_golden_fixtures_present():
    assert len(GOLDEN) >= 9


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[:-4])
def test_port_matches_golden_bit_exact(oracle, path):
    x, w, stride, pad, want = _load(path)
    got = oracle.host_conv2d(x, w, stride, pad, threads=False)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[:-4])
def test_threaded_zero_skipping_port_is_bit_identical(oracle, path):
    x, w, stride, pad, want = _load(path)
    for skip in (False, True):
        got = oracle.host_conv2d(x, w, stride, pad, threads=True, skip_zero=skip)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_port_matches_compiled_reference_when_built(oracle):
    if oracle.ref() is None:
        pytest.skip("oracle/_ref not built on this machine (reference sources absent)")
    rng = np.random.default_rng(7)
    for (n, ic, h, w, oc, ks, s, p) in [(2, 5, 9, 7, 6, 3, 1, 1), (1, 4, 12, 12, 3, 5, 2, 2),
                                        (3, 7, 6, 8, 9, 1, 1, 0), (1, 2, 7, 7, 2, 7, 1, 3)]:
        x = rng.standard_normal((n, ic, h, w)).astype(np.float32)
        f = rng.standard_normal((oc, ic, ks, ks)).astype(np.float32)
        f[rng.random(f.shape) < 0.7] = 0
        a = oracle.ref_host_conv2d(x, f, s, p)
        b = oracle.host_conv2d(x, f, s, p, threads=False)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_float_equal_matches_reference_formula(oracle):
    port = oracle.port()
    rng = np.random.default_rng(3)
    xs = np.concatenate([rng.standard_normal(200), [0, 1e-5, -1e-5, 1e-6, 1.0, 1.00002, 1e8]]).astype(np.float32)
    ys = (xs * (1 + rng.choice([0, 1e-6, 1e-5, 3e-5, 1e-4], xs.size)) + rng.choice([0, 5e-6, 2e-5], xs.size)).astype(np.float32)
    for x, y in zip(xs, ys):
        want = abs(float(x) - float(y)) <= 1e-5 * (abs(float(x)) + abs(float(y))) + 1e-5
        assert bool(port.oracle_float_equal(float(x), float(y))) == want
        if oracle.ref() is not None:
            assert bool(oracle.ref().ref_float_equal(float(x), float(y))) == want


def test_all_ones_fixture_counts_taps():
    """Known answer: with all-ones data each output is the number of in-bounds nonzero taps."""
    x, w, stride, pad, want = _load([p for p in GOLDEN if "all_ones" in p][0])
    n, ic, h, wd = x.shape
    oc, _, ks, _ = w.shape
    mask = (w != 0).astype(np.int64)
    xp = np.pad(np.ones((ic, h, wd), np.int64), ((0, 0), (pad, pad), (pad, pad)))
    oh, ow = want.shape[2:]
    cnt = np.zeros((oc, oh, ow), np.int64)
    for r in range(ks):
        for s in range(ks):
            win = xp[:, r:r + oh * stride:stride, s:s + ow * stride:stride]
            cnt += np.einsum("oi,ihw->ohw", mask[:, :, r, s], win)
    assert np.array_equal(want[0], cnt.astype(np.float32))


def test_depthwise_oracle_is_per_plane_conv(oracle):
    rng = np.random.default_rng(11)
    x = rng.random((2, 6, 9, 8), dtype=np.float32)
    w = rng.standard_normal((6, 1, 3, 3)).astype(np.float32)
    got = oracle.host_depthwise_conv2d(x, w, 2, 1)
    for c in range(6):
        want = oracle.host_conv2d(x[:, c:c + 1], w[c:c + 1], 2, 1, threads=False)
        assert np.array_equal(got[:, c:c + 1], want)


def test_layout_transposes(oracle):
    rng = np.random.default_rng(5)
    x = rng.random((2, 5, 4, 3), dtype=np.float32)
    y = np.empty((2, 4, 3, 5), np.float32)
    oracle.port().oracle_nchw_to_nhwc(x.ctypes.data, y.ctypes.data, 2, 5, 4, 3)
    assert np.array_equal(y, x.transpose(0, 2, 3, 1))
    z = np.empty_like(x)
    oracle.port().oracle_nhwc_to_nchw(y.ctypes.data, z.ctypes.data, 2, 5, 4, 3)
    assert np.array_equal(z, x)
    if oracle.ref() is not None:
        t = x.copy()
        oracle.ref().ref_nchw_to_nhwc(t.ctypes.data, 2, 5, 4, 3)
        assert np.array_equal(t.reshape(2, 4, 3, 5), y)


def test_compare_tolerance_semantics(oracle):
    ref = np.array([1.0, 100.0, 1e-7, 0.0], np.float32)
    ok = np.array([1.00005, 100.005, 5e-6, -9e-6], np.float32)
    bad, max_rel, n_floor = oracle.compare(ok, ref)
    assert bad == 0 and n_floor >= 2 and max_rel < 1.1e-4
    off = np.array([1.001, 100.0, 1e-7, 0.0], np.float32)
    assert oracle.compare(off, ref)[0] == 1

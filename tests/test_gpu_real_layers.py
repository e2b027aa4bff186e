"""GPU: the reference's real pruned layers (compact copies under tests/real_layers, made from the
layer dumps of its pruned checkpoints by tests/real_layers/make_real_layers.py).

Magnitude pruning leaves very uneven rows, rows without any nonzero and weights up to |w| ~ 2:
each layer goes through every kernel variant that covers it at batch 2 against the CPU oracle,
and a handful of them through the C++ per-layer program (`spconv2d_test <weight_file> <batch>`,
the reference's own program contract, Tetris/spconv2d.cc:369-450) with its self-check on.
"""
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "tetris-artifact-evalution_b200", "host")


def _files():
    from conftest import load_package
    import importlib
    load_package()
    return importlib.import_module("tetris_b200.workloads").real_layer_files()


FILES = _files()


def test_fixtures_are_present():
    assert len(FILES) >= 20, "tests/real_layers/*.npz are missing"


@pytest.mark.parametrize("path", FILES, ids=lambda p: os.path.basename(p)[:-4].replace("module", "m")[:60])
def test_real_layer_all_variants(tb, torch_cuda, workloads, oracle, path):
    torch = torch_cuda
    L, filt = workloads.load_real_layer(path)
    rng = np.random.default_rng(abs(hash(os.path.basename(path))) % (2 ** 32))
    n = 2
    x = rng.random((n, L.IC, L.H, L.W), dtype=np.float32)
    x[rng.random(x.shape) < 0.5] = 0
    want = oracle.host_conv2d(x, filt, L.stride, L.pad, threads=True, skip_zero=True)
    f = tb.SparseFilter(filt, L.IC, L.OC, L.KS)
    assert f.nnz_ == np.count_nonzero(filt)
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    oh, ow = want.shape[2], want.shape[3]
    variants = [tb.VARIANT_AUTO, tb.VARIANT_TILED, tb.VARIANT_GENERIC]
    if L.IC % 4 == 0 or L.IC <= 4:
        variants.append(tb.VARIANT_TENSOR)
    if L.stride == 1 and L.IC % 4 == 0 and L.IC >= 8:
        variants.append(tb.VARIANT_TENSOR16)
    for v in variants:
        out = torch.full((n, oh, ow, L.OC), float("nan"), device="cuda")
        if v == tb.VARIANT_AUTO:
            tb.tune_sparse_conv2d(f, xin, out, n, L.H, L.W, L.stride, L.pad)
            out.fill_(float("nan"))
        tb.sparse_conv2d(f, xin, out, n, L.H, L.W, L.stride, L.pad, variant=v)
        torch.cuda.synchronize()
        f.check()
        got = out.cpu().numpy().transpose(0, 3, 1, 2)
        assert not np.isnan(got).any()
        bad, max_rel, _ = oracle.compare(got, want)
        assert bad == 0, "%s variant %d: %d elements outside the bar (max rel %.3g)" % (L.name, v, bad, max_rel)
        empty = np.flatnonzero(np.count_nonzero(filt.reshape(L.OC, -1), axis=1) == 0)
        assert np.all(got[:, empty] == 0)   # an output channel without nonzeros is exactly zero
    f.close()


def _write_layer_file(path, w, L):
    with open(path, "w") as fh:
        fh.write("%d %d %d %d %d %d %d 1\n" % (L.H, L.W, L.IC, L.OC, L.KS, L.pad, L.stride))
        for o in range(L.OC):
            fh.write(" ".join(repr(float(v)) for v in w[o].reshape(-1)) + "\n")


PROGRAM_PICKS = [p for p in FILES if any(k in p for k in (
    "resnet50__module8_0_module3_1_conv2d_0_H_56_W_56_IC_64_OC_64_KS_3", "H_14_W_14_IC_256_OC_256_KS_3",
    "H_28_W_28_IC_512_OC_128_KS_1", "H_7_W_7_IC_512_OC_1024_KS_1", "H_56_W_56_IC_128_OC_128_KS_3_Pad_1_S_2",
    "H_56_W_56_IC_256_OC_512_KS_1_Pad_0_S_2"))] or FILES[:4]


@pytest.mark.parametrize("path", PROGRAM_PICKS, ids=lambda p: os.path.basename(p)[:-4].replace("module", "m")[:60])
def test_real_layer_through_the_cpp_program(tmp_path, workloads, path):
    """The reference's workload as the reference runs it: layer file in, timing lines and
    `Sparse Pass.` out (its self-check, TensorEqual against HostConv2d, switched on)."""
    exe = os.path.join(HOST, "spconv2d_test")
    assert os.path.exists(exe), "build it with `make -C tetris-artifact-evalution_b200/host`"
    L, filt = workloads.load_real_layer(path)
    layer = str(tmp_path / "layer")
    _write_layer_file(layer, filt, L)
    env = dict(os.environ, TETRIS_CHECK="1", TETRIS_SEED="11")
    res = subprocess.run([exe, layer, "1"], capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "nnz = %d" % np.count_nonzero(filt) in res.stdout
    assert "Sparse Pass." in res.stdout, res.stdout[-2000:]

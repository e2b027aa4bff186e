"""The C++ host mirror (tetris-artifact-evalution_b200/host): tensor_utils on the CPU, and the
per-layer program with the reference's argv/stdout contract on the GPU."""
import ctypes
import glob
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "tetris-artifact-evalution_b200", "host")
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


@pytest.fixture(scope="module")
def hostlib():
    path = os.path.join(HOST, "libtetris_host.so")
    if not os.path.exists(path):
        subprocess.run(["make", "-s", "-C", HOST, path], check=True)
    lib = ctypes.CDLL(path)
    names = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True).stdout

    def sym(plain):  # C++ linkage: find the mangled name that carries the plain one
        hits = [ln.split()[-1] for ln in names.splitlines() if ("%d%s" % (len(plain), plain)) in ln]
        assert hits, plain
        return getattr(lib, hits[0])
    return sym


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[:-4])
def test_host_conv2d_matches_golden_bit_exact(hostlib, path):
    z = np.load(path)
    x, w, want = np.ascontiguousarray(z["input"]), np.ascontiguousarray(z["filter"]), z["output"]
    n, ic, h, wd = x.shape
    oc, ks = w.shape[0], w.shape[-1]
    out = np.empty_like(want)
    hostlib("HostConv2d")(ctypes.c_void_p(x.ctypes.data), ctypes.c_void_p(w.ctypes.data),
                          ctypes.c_void_p(out.ctypes.data), n, h, wd, ic, oc, ks, int(z["stride"]), int(z["pad"]))
    assert np.array_equal(out.view(np.uint32), want.view(np.uint32))


def test_layout_changes_and_compare(hostlib):
    rng = np.random.default_rng(8)
    x = rng.random((2, 5, 4, 3), dtype=np.float32)
    t = x.copy()
    hostlib("NCHW2NHWC")(ctypes.c_void_p(t.ctypes.data), 2, 5, 4, 3)
    assert np.array_equal(t.reshape(2, 4, 3, 5), x.transpose(0, 2, 3, 1))
    hostlib("NHWC2NCHW")(ctypes.c_void_p(t.ctypes.data), 2, 5, 4, 3)
    assert np.array_equal(t, x)
    k = rng.random((6, 5, 3, 3), dtype=np.float32)
    t = k.copy()
    hostlib("KCRS2KRSC")(ctypes.c_void_p(t.ctypes.data), 6, 5, 3, 3)
    assert np.array_equal(t.reshape(6, 3, 3, 5), k.transpose(0, 2, 3, 1))
    hostlib("KRSC2KCRS")(ctypes.c_void_p(t.ctypes.data), 6, 5, 3, 3)
    assert np.array_equal(t, k)
    feq = hostlib("FloatEqual")
    feq.argtypes, feq.restype = [ctypes.c_float, ctypes.c_float], ctypes.c_bool
    assert feq(1.0, 1.00001) and not feq(1.0, 1.001) and feq(0.0, 9e-6)
    rnd = hostlib("RandFloat")
    rnd.restype = ctypes.c_float
    hostlib("SeedRand")(ctypes.c_uint64(5))
    a = [rnd() for _ in range(1000)]
    hostlib("SeedRand")(ctypes.c_uint64(5))
    assert a == [rnd() for _ in range(1000)] and -1.0 <= min(a) and max(a) < 1.0 and abs(np.mean(a)) < 0.1


def write_layer_file(path, w, h, wd, pad, stride):
    oc, ic, ks, _ = w.shape
    with open(path, "w") as fh:
        fh.write("%d %d %d %d %d %d %d 1\n" % (h, wd, ic, oc, ks, pad, stride))
        for o in range(oc):
            fh.write(" ".join(repr(float(v)) for v in w[o].reshape(-1)) + "\n")


@pytest.mark.gpu
@pytest.mark.parametrize("name,batch", [("c3x3_s1_p1", 4), ("c1x1_s2_p0", 3), ("c7x7_s2_p3", 2)])
def test_program_contract_and_self_check(tmp_path, name, batch):
    exe = os.path.join(HOST, "spconv2d_test")
    assert os.path.exists(exe), "build it with `make -C tetris-artifact-evalution_b200/host`"
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", name + ".npz"))
    layer = str(tmp_path / "layer")
    write_layer_file(layer, z["filter"], z["input"].shape[2], z["input"].shape[3], int(z["pad"]), int(z["stride"]))
    env = dict(os.environ, TETRIS_CHECK="1", TETRIS_SEED="7")
    res = subprocess.run([exe, layer, str(batch)], capture_output=True, text=True, env=env, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    out = res.stdout
    assert "[Config] sparsity = " in out and "nnz = %d" % np.count_nonzero(z["filter"]) in out
    # the two lines the reference's Python driver scrapes (strips "ms" and "T")
    t = [ln for ln in out.splitlines() if ln.startswith("Time of Spconv2d :")][0]
    assert t.endswith("ms") and float(t.split(":")[1][:-2]) > 0
    fl = [ln for ln in out.splitlines() if ln.startswith("FLOPS of Spconv2d :")][0]
    assert fl.endswith("T") and float(fl.split(":")[1][:-1]) > 0
    assert "Sparse Pass." in out


@pytest.mark.gpu
def test_program_exits_1_on_a_missing_file():
    exe = os.path.join(HOST, "spconv2d_test")
    res = subprocess.run([exe, "/nonexistent/layer", "1"], capture_output=True, text=True, timeout=60)
    assert res.returncode == 1 and "Open file error." in res.stdout

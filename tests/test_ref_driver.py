"""The reference's Python driver (evalution/conv2d_timing.py) spawns a per-layer binary and
scrapes its standard output.  These tests keep that contract:

* CPU: the checker-side restatement of the driver's parsing (tests/ref_driver_parse.py) reads
  what the engine's programs print; where the reference checkout is present, the reference's
  own PefCounterForOperator is run on the same text (through a stand-in "binary" that prints it)
  and must return the same figures.
* GPU: the real `spconv2d_test` binary and `spconv2d_test.py`, run on a layer file, parsed the
  same way: config, time and FLOPS come out as numbers the driver can tabulate.
"""
import importlib.util
import os
import stat
import subprocess
import sys

import numpy as np
import pytest

from ref_driver_parse import parse_operator_output

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "tetris-artifact-evalution_b200", "host")

# what host/spconv2d.cc and spconv2d_test.py print (format strings of those programs)
SAMPLE = """args : 3 ./spconv2d_test layer 4

GPU Device 0: "NVIDIA B200" with compute capability 10.0

[Config] sparsity = 0.900011, nnz = 3686, batch_size = 4, img_h = 56, img_w = 56, in_channel = 64, out_channel = 64, kernel_size = 3, padding = 1, stride = 1

Time of Spconv2d :0.0123456ms
FLOPS of Spconv2d :68.3313T
HostConv2d begin
HostConv2d end
Sparse Pass.
"""


def test_restated_parser_reads_the_program_output():
    cfg, t, fl, logged = parse_operator_output(SAMPLE.splitlines())
    assert cfg["kernel_size"] == "3" and cfg["nnz"] == "3686" and cfg["batch_size"] == "4"
    assert t == pytest.approx(0.0123456) and fl == pytest.approx(68.3313)
    assert logged == ["Sparse Pass."]
    with pytest.raises(ValueError):
        parse_operator_output(["Time of Sparse :1.0ms", "Sparse Error."])


def _reference_driver():
    from oracle import oracle as orc
    path = os.path.join(orc.reference_root(), "evalution", "conv2d_timing.py")
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location("ref_conv2d_timing", path)
    mod = importlib.util.module_from_spec(spec)
    try:
        spec.loader.exec_module(mod)   # imports pandas; its main part is guarded by __name__
    except ImportError:
        return None
    return mod


def test_reference_driver_agrees_with_the_restatement(tmp_path):
    ref = _reference_driver()
    if ref is None:
        pytest.skip("the reference checkout (or pandas) is not present here")
    text = tmp_path / "out.txt"
    text.write_text(SAMPLE)
    fake = tmp_path / "fake_spconv2d_test"
    fake.write_text("#!/bin/sh\ncat '%s'\n" % text)
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    with open(tmp_path / "log.txt", "a+") as log:
        cfg, t, fl = ref.PefCounterForOperator(log, str(fake), "some layer file", 4)
    want_cfg, want_t, want_fl, _ = parse_operator_output(SAMPLE.splitlines())
    assert cfg == want_cfg and t == want_t and fl == want_fl


@pytest.mark.gpu
def test_both_programs_print_what_the_driver_parses(tmp_path, workloads):
    L = workloads.single_layer()[0]
    filt = workloads.make_filter("single", 0, L)
    layer = tmp_path / "layer_H_56_W_56_IC_64_OC_64_KS_3_Pad_1_S_1_G_1"
    with open(layer, "w") as fh:
        fh.write("%d %d %d %d %d %d %d 1\n" % (L.H, L.W, L.IC, L.OC, L.KS, L.pad, L.stride))
        for o in range(L.OC):
            fh.write(" ".join(repr(float(v)) for v in filt[o].reshape(-1)) + "\n")
    programs = [[os.path.join(HOST, "spconv2d_test"), str(layer), "4"],
                [sys.executable, os.path.join(ROOT, "tetris-artifact-evalution_b200", "spconv2d_test.py"), str(layer), "4"]]
    for cmd in programs:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, TETRIS_CHECK="1"))
        assert res.returncode == 0, res.stdout + res.stderr
        cfg, t, fl, logged = parse_operator_output(res.stdout.splitlines())
        assert cfg["kernel_size"] == "3" and cfg["in_channel"] == "64" and cfg["batch_size"] == "4"
        assert int(cfg["nnz"]) == np.count_nonzero(filt)
        assert 0.0 < t < 10.0 and fl > 0.0

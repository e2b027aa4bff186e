"""TEST INFRASTRUCTURE ONLY: ctypes doors to the CPU oracle.

`port()` loads oracle/liboracle_port.so (the C restatement, host_conv2d.c); `ref()` loads
oracle/_ref/libtetris_ref.so (the reference's own tensor_utils.cc compiled by oracle/Makefile)
or returns None when it was not built.  Only tests/, the smoke check and the benchmark's CPU
baseline may import this module; the engine itself never does.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(_HERE, "liboracle_port.so")
REF_PATH = os.path.join(_HERE, "_ref", "libtetris_ref.so")
_I, _VP = ctypes.c_int, ctypes.c_void_p
_port = _ref = None


def reference_root():
    """Where the reference checkout lies: $TETRIS_REFERENCE_ROOT, else a directory named
    `reference` beside this repository."""
    return os.environ.get("TETRIS_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(ref_root=None):
    """Run the Makefile: always the port; the compiled reference when its sources are there."""
    subprocess.run(["make", "-s", "-C", _HERE, "REF=" + (ref_root or reference_root()), "all"], check=True)


def port():
    global _port
    if _port is None:
        if not os.path.exists(PORT_PATH):
            subprocess.run(["make", "-s", "-C", _HERE, "port"], check=True)
        lib = ctypes.CDLL(PORT_PATH)
        lib.oracle_host_conv2d.argtypes = [_VP, _VP, _VP] + [_I] * 8
        lib.oracle_host_conv2d_mt.argtypes = [_VP, _VP, _VP] + [_I] * 9
        lib.oracle_host_depthwise_conv2d.argtypes = [_VP, _VP, _VP] + [_I] * 7
        lib.oracle_float_equal.argtypes = [ctypes.c_float, ctypes.c_float]
        lib.oracle_float_equal.restype = _I
        lib.oracle_tensor_first_mismatch.argtypes = [_VP, _VP, ctypes.c_size_t]
        lib.oracle_tensor_first_mismatch.restype = ctypes.c_long
        lib.oracle_tensor_compare.argtypes = [_VP, _VP, ctypes.c_size_t, ctypes.c_double,
                                              ctypes.c_double, ctypes.POINTER(ctypes.c_double),
                                              ctypes.POINTER(ctypes.c_long)]
        lib.oracle_tensor_compare.restype = ctypes.c_long
        lib.oracle_nchw_to_nhwc.argtypes = [_VP, _VP] + [_I] * 4
        lib.oracle_nhwc_to_nchw.argtypes = [_VP, _VP] + [_I] * 4
        _port = lib
    return _port


def ref():
    global _ref
    if _ref is None and os.path.exists(REF_PATH):
        lib = ctypes.CDLL(REF_PATH)
        lib.ref_host_conv2d.argtypes = [_VP, _VP, _VP] + [_I] * 8
        lib.ref_float_equal.argtypes = [ctypes.c_float, ctypes.c_float]
        lib.ref_float_equal.restype = _I
        for name in ("ref_nchw_to_nhwc", "ref_nhwc_to_nchw", "ref_kcrs_to_krsc", "ref_krsc_to_kcrs"):
            getattr(lib, name).argtypes = [_VP] + [_I] * 4
        lib.ref_read_layer_file.argtypes = [ctypes.c_char_p, _I, ctypes.POINTER(_I)]
        lib.ref_read_layer_file.restype = ctypes.POINTER(ctypes.c_float)
        lib.ref_free.argtypes = [_VP]
        _ref = lib
    return _ref


def _out_shape(x, w, stride, pad):
    n, ic, h, wd = x.shape
    oc, ks = w.shape[0], w.shape[-1]
    return (n, oc, (h + 2 * pad - ks) // stride + 1, (wd + 2 * pad - ks) // stride + 1)


def host_conv2d(x, w, stride, pad, threads=True, skip_zero=True):
    """Oracle convolution (port): NCHW float32 x, OIHW float32 w -> NCHW float32."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    n, ic, h, wd = x.shape
    oc, ks = w.shape[0], w.shape[-1]
    out = np.empty(_out_shape(x, w, stride, pad), np.float32)
    if threads:
        port().oracle_host_conv2d_mt(x.ctypes.data, w.ctypes.data, out.ctypes.data, n, h, wd, ic, oc,
                                     ks, stride, pad, 1 if skip_zero else 0)
    else:
        port().oracle_host_conv2d(x.ctypes.data, w.ctypes.data, out.ctypes.data, n, h, wd, ic, oc, ks,
                                  stride, pad)
    return out


def host_depthwise_conv2d(x, w, stride, pad):
    """Oracle depthwise convolution: x NCHW, w [C][1][KS][KS]."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    n, c, h, wd = x.shape
    ks = w.shape[-1]
    out = np.empty((n, c, (h + 2 * pad - ks) // stride + 1, (wd + 2 * pad - ks) // stride + 1), np.float32)
    port().oracle_host_depthwise_conv2d(x.ctypes.data, w.ctypes.data, out.ctypes.data, n, h, wd, c, ks,
                                        stride, pad)
    return out


def ref_host_conv2d(x, w, stride, pad):
    """The compiled reference's HostConv2d; None when oracle/_ref was not built."""
    lib = ref()
    if lib is None:
        return None
    x = np.array(x, np.float32, order="C")
    w = np.array(w, np.float32, order="C")
    n, ic, h, wd = x.shape
    oc, ks = w.shape[0], w.shape[-1]
    out = np.empty(_out_shape(x, w, stride, pad), np.float32)
    lib.ref_host_conv2d(x.ctypes.data, w.ctypes.data, out.ctypes.data, n, h, wd, ic, oc, ks, stride, pad)
    return out


REL_TOL = 1e-4   # max relative error the path must meet against the CPU convolution
ABS_FLOOR = 1e-5  # the absolute floor the reference's own check uses (Tetris/tensor_utils.cc:18)


def compare(got, want, rel=REL_TOL, abs_floor=ABS_FLOOR):
    """(n_bad, max_rel_error, n_floor_protected) under |x-y| <= rel*max(|x|,|y|) + abs_floor."""
    got = np.ascontiguousarray(got, np.float32)
    want = np.ascontiguousarray(want, np.float32)
    assert got.shape == want.shape, (got.shape, want.shape)
    mr, nf = ctypes.c_double(0), ctypes.c_long(0)
    bad = port().oracle_tensor_compare(got.ctypes.data, want.ctypes.data, got.size, rel, abs_floor,
                                       ctypes.byref(mr), ctypes.byref(nf))
    return int(bad), float(mr.value), int(nf.value)

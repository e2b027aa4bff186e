"""B200 sparse-filter convolution engine: Python host side over the C ABI.

The directory name carries a hyphen, so load the package by path:

    import importlib.util, sys
    spec = importlib.util.spec_from_file_location(
        "tetris_b200", "tetris-artifact-evalution_b200/__init__.py",
        submodule_search_locations=["tetris-artifact-evalution_b200"])
    tetris_b200 = importlib.util.module_from_spec(spec)
    sys.modules["tetris_b200"] = tetris_b200
    spec.loader.exec_module(tetris_b200)

Names mirror the reference's host API for this path:

    SparseFilter        <- SparseFilter<float,int,int>   (Tetris/spconv2d_utils.h:23-515)
    sparse_conv2d       <- SparseConv2d<...> launcher     (Tetris/spconv2d_kernel.cu:163-188)
    timing_sparse_conv2d<- TimingTetrisSparseConv2d       (Tetris/spconv2d.cc:29-69)
    cuda_sparse_conv2d  <- CudaSparseConv2d               (Tetris/spconv2d.cc:332-367)

Everything computes on the GPU through libtetris_b200.so.  There is no CPU
fallback: if the library is missing or fails to load, importing `lib()` raises.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtetris_b200.so")

WARM = 30     # Tetris/tensor_utils.h:11
REPEAT = 100  # Tetris/tensor_utils.h:10

VARIANT_AUTO, VARIANT_GENERIC, VARIANT_TILED, VARIANT_TENSOR, VARIANT_TENSOR16 = 0, 1, 2, 4, 5  # 3 is retired

_c_float_p = ctypes.POINTER(ctypes.c_float)
_c_int_p = ctypes.POINTER(ctypes.c_int)


class FilterOpts(ctypes.Structure):
    _fields_ = [("oc_block", ctypes.c_int), ("tile_ic", ctypes.c_int), ("deterministic", ctypes.c_int),
                ("reserved", ctypes.c_int * 5)]


class FilterInfo(ctypes.Structure):
    _fields_ = [
        ("in_channel", ctypes.c_int), ("out_channel", ctypes.c_int),
        ("kernel_size", ctypes.c_int), ("groups", ctypes.c_int),
        ("oc_block", ctypes.c_int), ("tile_ic", ctypes.c_int),
        ("n_oc_blocks", ctypes.c_int), ("n_stages", ctypes.c_int),
        ("nnz", ctypes.c_int64), ("n_ops", ctypes.c_int64), ("compressed_bytes", ctypes.c_int64),
        ("n_list_units", ctypes.c_int64),
        ("device", ctypes.c_int), ("reserved", ctypes.c_int * 5),
    ]


# name -> (restype, argtypes); the list must match include/tetris_b200.h
_VP = ctypes.c_void_p
_I = ctypes.c_int
SIGNATURES = {
    "tetris_filter_create": (_I, [_VP, _I, _I, _I, _I, _I, ctypes.POINTER(_VP)]),
    "tetris_filter_create_ex": (_I, [_VP, _I, _I, _I, _I, _I, ctypes.POINTER(FilterOpts), ctypes.POINTER(_VP)]),
    "tetris_filter_destroy": (None, [_VP]),
    "tetris_filter_info": (_I, [_VP, ctypes.POINTER(FilterInfo)]),
    "tetris_filter_download": (_I, [_VP, _VP, ctypes.c_size_t, _VP, ctypes.c_size_t]),
    "tetris_filter_download_lists": (_I, [_VP, _VP, ctypes.c_size_t, _VP, ctypes.c_size_t]),
    "tetris_filter_check": (_I, [_VP]),
    "tetris_conv2d_launch": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _VP]),
    "tetris_conv2d_launch_ex": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _VP, _I]),
    "tetris_conv2d_launch_fused": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _VP, _I, _I]),
    "tetris_chain_create": (_I, [_VP, _I, _I, _I, _I, ctypes.POINTER(_VP)]),
    "tetris_chain_destroy": (None, [_VP]),
    "tetris_chain_run": (_I, [_VP, _VP, _VP]),
    "tetris_chain_capture": (_I, [_VP, _VP]),
    "tetris_chain_replay": (_I, [_VP, _VP]),
    "tetris_chain_download": (_I, [_VP, _VP, ctypes.c_size_t]),
    "tetris_chain_output": (_I, [_VP, ctypes.POINTER(_VP), _c_int_p, _c_int_p, _c_int_p]),
    "tetris_conv2d_time": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _VP, _I, _I, _I, _c_float_p]),
    "tetris_conv2d_tune": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _VP, _I, _c_float_p]),
    "tetris_conv2d_choice": (_I, [_VP, _I, _I, _I, _I, _I, _c_int_p]),
    "tetris_conv2d_host": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _VP]),
    "tetris_conv2d_host_async": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _I]),
    "tetris_host_sync": (_I, [_I, _I]),
    "tetris_release_workspace": (None, []),
    "tetris_nchw_to_nhwc": (_I, [_VP, _VP, _I, _I, _I, _I, _VP]),
    "tetris_nhwc_to_nchw": (_I, [_VP, _VP, _I, _I, _I, _I, _VP]),
    "tetris_conv2d_host_sharded": (_I, [ctypes.POINTER(_VP), _I, _VP, _VP, _I, _I, _I, _I, _I]),
    "tetris_batch_slice": (_I, [_I, _I, _I, _c_int_p, _c_int_p]),
    "tetris_device_info": (_I, [_I, _c_int_p, _c_int_p, _c_int_p]),
    "tetris_list_offsets_noalloc": (_I, [_VP, _I, _I, _I, _I, _I, _VP, _VP]),
    "tetris_filter_save": (_I, [_VP, ctypes.c_char_p]),
    "tetris_filter_load": (_I, [ctypes.c_char_p, _I, ctypes.POINTER(_VP)]),
    "tetris_filter_file_check": (_I, [ctypes.c_char_p, ctypes.POINTER(FilterInfo)]),
    "tetris_launch_count": (ctypes.c_ulonglong, []),
    "tetris_test_inject": (ctypes.c_int, [ctypes.c_int, ctypes.c_uint]),
    "tetris_last_error": (ctypes.c_char_p, []),
}

_lib = None


class TetrisError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status, message):
        super().__init__("tetris_b200 status %d: %s" % (status, message))
        self.status = status


def lib():
    """The loaded native library.  Raises if it is absent: there is no other compute path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "%s is missing: build it with `python %s` (needs nvcc); the engine has no "
                "fallback path" % (LIB_PATH, os.path.join(_HERE, "build.py")))
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def _check(status):
    if status != 0:
        raise TetrisError(status, lib().tetris_last_error().decode("utf-8", "replace"))


def _ptr(x):
    """Device or host address of a torch tensor, numpy array, int or None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    raise TypeError("cannot take the address of %r" % type(x))


def _stream_ptr(stream):
    if stream is None:
        return None
    return getattr(stream, "cuda_stream", stream)


def out_extent(size, kernel_size, stride, padding):
    """Output extent, Tetris/spconv2d.cc:339-340."""
    return (size + 2 * padding - kernel_size) // stride + 1


class SparseFilter:
    """Compressed filter living on one GPU.

    Constructor arguments follow the reference class (Tetris/spconv2d_utils.h:25-27):
    dense OIHW float32 `filter`, `in_channel`, `out_channel`, `kernel_size`, then
    `TILE_IC` (input channels per stage; 0 = engine default).  `apply_reorder` and
    `apply_vectorize` are accepted for call compatibility: the new format always
    groups weights by shared input offset and always uses vector loads.  `groups`
    and `device` are additions.  Like the reference object it owns device memory
    (freed by close() / garbage collection) and must not be copied.
    """

    def __init__(self, filter, in_channel, out_channel, kernel_size, TILE_IC=0,
                 apply_reorder=True, apply_vectorize=True, groups=1, device=0, oc_block=0,
                 deterministic=False):
        per_oc = 1 if groups != 1 else in_channel
        dense = np.ascontiguousarray(filter, dtype=np.float32).reshape(-1)
        expect = out_channel * per_oc * kernel_size * kernel_size
        if dense.size != expect:
            raise ValueError("filter has %d elements, expected %d" % (dense.size, expect))
        self._handle = _VP()
        opts = FilterOpts(oc_block=oc_block, tile_ic=TILE_IC, deterministic=1 if deterministic else 0)
        _check(lib().tetris_filter_create_ex(dense.ctypes.data, in_channel, out_channel, kernel_size,
                                             groups, device, ctypes.byref(opts),
                                             ctypes.byref(self._handle)))
        self._adopt(device)

    def _adopt(self, device):
        info = self.info()
        self.in_channel_, self.out_channel_, self.kernel_size_ = info.in_channel, info.out_channel, info.kernel_size
        self.groups_ = info.groups
        self.nnz_ = info.nnz
        self.TILE_IC_ = info.tile_ic
        self.device_ = device

    def save(self, path):
        """Write the compressed forms and the tuned tile plans to `path` (tetris_filter_save)."""
        _check(lib().tetris_filter_save(self.handle, os.fsencode(path)))

    @classmethod
    def load(cls, path, device=0):
        """A filter read back from a file written by save(): no recompression, same tuned plans."""
        self = cls.__new__(cls)
        self._handle = _VP()
        _check(lib().tetris_filter_load(os.fsencode(path), device, ctypes.byref(self._handle)))
        self._adopt(device)
        return self

    def info(self):
        info = FilterInfo()
        _check(lib().tetris_filter_info(self._handle, ctypes.byref(info)))
        return info

    def GetTileIC(self):
        return self.TILE_IC_

    def download(self):
        """(ops uint64[n_ops], prog_offsets int32[B*T+1]) copied back from the device."""
        info = self.info()
        ops = np.empty(info.n_ops, dtype=np.uint64)
        offs = np.empty(info.n_oc_blocks * info.n_stages + 1, dtype=np.int32)
        _check(lib().tetris_filter_download(self._handle, ops.ctypes.data, ops.size,
                                            offs.ctypes.data, offs.size))
        return ops, offs

    def download_lists(self):
        """(units uint64[n_list_units], list_offsets int32[B*T+1]) of the list form."""
        info = self.info()
        units = np.empty(info.n_list_units, dtype=np.uint64)
        offs = np.empty(info.n_oc_blocks * info.n_stages + 1, dtype=np.int32)
        _check(lib().tetris_filter_download_lists(self._handle, units.ctypes.data, units.size,
                                                  offs.ctypes.data, offs.size))
        return units, offs

    def check(self):
        """Synchronise and raise if a tensor-core launch of this filter timed out on a barrier."""
        _check(lib().tetris_filter_check(self._handle))

    @property
    def handle(self):
        if not self._handle:
            raise RuntimeError("SparseFilter already closed")
        return self._handle

    def close(self):
        if getattr(self, "_handle", None):
            lib().tetris_filter_destroy(self._handle)
            self._handle = _VP()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def sparse_conv2d(sparse_filter, input, output, batch_size, img_h, img_w, stride, padding,
                  cuda_stream=None, variant=VARIANT_AUTO):
    """Launch the convolution: device NHWC `input` -> device NHWC `output`, asynchronous."""
    _check(lib().tetris_conv2d_launch_ex(sparse_filter.handle, _ptr(input), _ptr(output), batch_size,
                                         img_h, img_w, stride, padding, _stream_ptr(cuda_stream),
                                         variant))


FUSE_RELU = 1


def sparse_conv2d_fused(sparse_filter, input, output, batch_size, img_h, img_w, stride, padding,
                        cuda_stream=None, variant=VARIANT_AUTO, relu=True):
    """sparse_conv2d with max(y, 0) applied at the store (tetris_conv2d_launch_fused)."""
    _check(lib().tetris_conv2d_launch_fused(sparse_filter.handle, _ptr(input), _ptr(output), batch_size,
                                            img_h, img_w, stride, padding, _stream_ptr(cuda_stream),
                                            variant, FUSE_RELU if relu else 0))


class ChainLayer(ctypes.Structure):
    _fields_ = [("filter", _VP), ("stride", _I), ("padding", _I), ("relu", _I), ("pool", _I)]


class LayerChain:
    """The conv layers of a model run back to back on the device (tetris_chain_*).

    `layers` is a list of (SparseFilter, stride, padding, relu, pool) with pool in (0, 2).  The
    chain owns the activations between the layers; the filters stay the caller's and must
    outlive the chain.
    """

    def __init__(self, layers, batch_size, img_h, img_w):
        self._filters = [l[0] for l in layers]
        arr = (ChainLayer * len(layers))(*[ChainLayer(l[0].handle, l[1], l[2], 1 if l[3] else 0, l[4]) for l in layers])
        self._handle = _VP()
        _check(lib().tetris_chain_create(arr, len(layers), batch_size, img_h, img_w, ctypes.byref(self._handle)))
        self.batch = batch_size

    def run(self, input, cuda_stream=None):
        _check(lib().tetris_chain_run(self._handle, _ptr(input), _stream_ptr(cuda_stream)))

    def capture(self, input):
        _check(lib().tetris_chain_capture(self._handle, _ptr(input)))

    def replay(self, cuda_stream=None):
        _check(lib().tetris_chain_replay(self._handle, _stream_ptr(cuda_stream)))

    def output(self):
        """(device address, h, w, channels) of the last layer's output."""
        p, h, w, c = _VP(), _I(), _I(), _I()
        _check(lib().tetris_chain_output(self._handle, ctypes.byref(p), ctypes.byref(h), ctypes.byref(w), ctypes.byref(c)))
        return p.value, h.value, w.value, c.value

    def download(self):
        """The last layer's output as a host NHWC float32 array (waits for the device)."""
        _, h, w, c = self.output()
        host = np.empty((self.batch, h, w, c), np.float32)
        _check(lib().tetris_chain_download(self._handle, host.ctypes.data, host.size))
        return host

    def close(self):
        if getattr(self, "_handle", None):
            lib().tetris_chain_destroy(self._handle)
            self._handle = _VP()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def timing_sparse_conv2d(sparse_filter, input, output, batch_size, img_h, img_w, stride, padding,
                         cuda_stream=None, variant=VARIANT_AUTO, warm=WARM, repeat=REPEAT):
    """Mean milliseconds per launch under the reference's warm-up/repeat protocol."""
    ms = ctypes.c_float(0.0)
    _check(lib().tetris_conv2d_time(sparse_filter.handle, _ptr(input), _ptr(output), batch_size,
                                    img_h, img_w, stride, padding, _stream_ptr(cuda_stream), variant,
                                    warm, repeat, ctypes.byref(ms)))
    return ms.value


def tune_sparse_conv2d(sparse_filter, input, output, batch_size, img_h, img_w, stride, padding,
                       cuda_stream=None, max_candidates=0):
    """Time the best-ranked tile shapes for this conv shape, keep the fastest with the filter
    (the reference's GetTetrisSparseConv2dTime search); returns its mean milliseconds."""
    ms = ctypes.c_float(0.0)
    _check(lib().tetris_conv2d_tune(sparse_filter.handle, _ptr(input), _ptr(output), batch_size, img_h,
                                    img_w, stride, padding, _stream_ptr(cuda_stream), max_candidates,
                                    ctypes.byref(ms)))
    return ms.value


def auto_choice(sparse_filter, batch_size, img_h, img_w, stride, padding):
    """The variant (VARIANT_TILED / VARIANT_TENSOR / VARIANT_GENERIC, VARIANT_AUTO for depthwise)
    that an automatic launch of this shape uses at the moment."""
    v = ctypes.c_int(0)
    _check(lib().tetris_conv2d_choice(sparse_filter.handle, batch_size, img_h, img_w, stride, padding,
                                      ctypes.byref(v)))
    return v.value


def cuda_sparse_conv2d(h_input, sparse_filter, batch_size, img_h, img_w, stride, padding,
                       h_output=None, cuda_stream=None):
    """Host NCHW in, host NCHW out (numpy float32), blocking; returns the output array."""
    f = sparse_filter
    oh = out_extent(img_h, f.kernel_size_, stride, padding)
    ow = out_extent(img_w, f.kernel_size_, stride, padding)
    h_input = np.ascontiguousarray(h_input, dtype=np.float32)
    if h_input.size != batch_size * f.in_channel_ * img_h * img_w:
        raise ValueError("input has %d elements, expected %d"
                         % (h_input.size, batch_size * f.in_channel_ * img_h * img_w))
    if h_output is None:
        h_output = np.empty((batch_size, f.out_channel_, oh, ow), dtype=np.float32)
    _check(lib().tetris_conv2d_host(f.handle, h_input.ctypes.data, h_output.ctypes.data, batch_size,
                                    img_h, img_w, stride, padding, _stream_ptr(cuda_stream)))
    return h_output


def cuda_sparse_conv2d_sharded(h_input, sparse_filters, batch_size, img_h, img_w, stride, padding):
    """As cuda_sparse_conv2d, the batch cut into one contiguous slice per filter/GPU."""
    f = sparse_filters[0]
    oh = out_extent(img_h, f.kernel_size_, stride, padding)
    ow = out_extent(img_w, f.kernel_size_, stride, padding)
    h_input = np.ascontiguousarray(h_input, dtype=np.float32)
    h_output = np.empty((batch_size, f.out_channel_, oh, ow), dtype=np.float32)
    handles = (_VP * len(sparse_filters))(*[sf.handle for sf in sparse_filters])
    _check(lib().tetris_conv2d_host_sharded(handles, len(sparse_filters), h_input.ctypes.data,
                                            h_output.ctypes.data, batch_size, img_h, img_w, stride,
                                            padding))
    return h_output


def cuda_sparse_conv2d_async(h_input, sparse_filter, batch_size, img_h, img_w, stride, padding,
                             h_output, slot=0):
    """Queue host NCHW -> host NCHW on pipeline slot `slot` and return; `h_input` / `h_output`
    (contiguous float32 numpy arrays, ideally page-locked) must stay untouched until
    host_sync(device, slot)."""
    if not (h_input.flags.c_contiguous and h_output.flags.c_contiguous
            and h_input.dtype == np.float32 and h_output.dtype == np.float32):
        raise ValueError("the asynchronous path needs contiguous float32 host arrays")
    _check(lib().tetris_conv2d_host_async(sparse_filter.handle, h_input.ctypes.data,
                                          h_output.ctypes.data, batch_size, img_h, img_w, stride,
                                          padding, slot))


def host_sync(device=0, slot=-1):
    """Wait for one pipeline slot of cuda_sparse_conv2d_async (slot < 0: all slots)."""
    _check(lib().tetris_host_sync(device, slot))


def release_workspace():
    """Free the device workspaces that cuda_sparse_conv2d keeps between calls."""
    lib().tetris_release_workspace()


def nchw_to_nhwc(src, dst, N, C, H, W, cuda_stream=None):
    _check(lib().tetris_nchw_to_nhwc(_ptr(src), _ptr(dst), N, C, H, W, _stream_ptr(cuda_stream)))


def nhwc_to_nchw(src, dst, N, C, H, W, cuda_stream=None):
    _check(lib().tetris_nhwc_to_nchw(_ptr(src), _ptr(dst), N, C, H, W, _stream_ptr(cuda_stream)))


def filter_file_check(path):
    """Validate a compressed-filter file on the host alone; returns its FilterInfo."""
    info = FilterInfo()
    _check(lib().tetris_filter_file_check(os.fsencode(path), ctypes.byref(info)))
    return info


def launch_count():
    """Convolution kernels launched through the library by this process so far."""
    return int(lib().tetris_launch_count())


def test_inject(what, spin_limit=0):
    """Failure-detection test hook (tetris_test_inject): 1 = the tensor-core kernels leave out every
    CTA's first activation load and their barrier waits give up after `spin_limit` polls; 0 = off."""
    _check(lib().tetris_test_inject(int(what), int(spin_limit)))


def batch_slice(batch_size, world, rank):
    """(begin, count) of the contiguous batch slice that shard `rank` of `world` owns."""
    b, c = ctypes.c_int(0), ctypes.c_int(0)
    _check(lib().tetris_batch_slice(batch_size, world, rank, ctypes.byref(b), ctypes.byref(c)))
    return b.value, c.value


def device_info(device=0):
    """(sm_count, sm_clock_khz, fp32_lanes_per_sm)."""
    a, b, c = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
    _check(lib().tetris_device_info(device, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)))
    return a.value, b.value, c.value


def list_offsets_noalloc(d_filter, in_channel, out_channel, kernel_size, oc_block, tile_ic,
                         d_list_offsets, cuda_stream=None):
    """Piece offsets of the list form for a dense filter already on the device, written into the
    caller's device array `d_list_offsets`; the library allocates nothing (fixed scratch inside
    the library, at most 16384 pieces).  Asynchronous on `cuda_stream`."""
    _check(lib().tetris_list_offsets_noalloc(_ptr(d_filter), in_channel, out_channel, kernel_size,
                                             oc_block, tile_ic, _ptr(d_list_offsets),
                                             _stream_ptr(cuda_stream)))

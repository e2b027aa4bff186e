"""CPU: the C-ABI library loads and exports every symbol the public header declares.

No compute call is made here (there is no GPU on the machine that runs this file); calls that
only touch host logic (slicing, error text for bad arguments) are exercised.
"""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "tetris_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tetris_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("tetris_filter_create", "tetris_filter_destroy", "tetris_conv2d_launch",
                 "tetris_conv2d_time", "tetris_conv2d_host", "tetris_conv2d_host_sharded",
                 "tetris_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol(tb):
    assert os.path.exists(tb.LIB_PATH), "libtetris_b200.so is not built"
    handle = ctypes.CDLL(tb.LIB_PATH)
    for name in declared_functions():
        assert hasattr(handle, name), "missing export: " + name


def test_python_binding_covers_the_header(tb):
    assert sorted(tb.SIGNATURES) == declared_functions()


def test_batch_slice_tiles_the_batch(tb):
    for batch in (0, 1, 7, 16, 33):
        for world in (1, 2, 3, 4, 8):
            pos = 0
            for rank in range(world):
                begin, count = tb.batch_slice(batch, world, rank)
                assert begin == pos and count in (batch // world, batch // world + 1)
                pos += count
            assert pos == batch


def test_bad_arguments_are_reported_not_fatal(tb):
    with pytest.raises(tb.TetrisError) as e:
        tb.batch_slice(4, 0, 0)
    assert e.value.status == 1 and "bad slice" in str(e.value)
    lib = tb.lib()
    info = tb.FilterInfo()
    assert lib.tetris_filter_info(None, ctypes.byref(info)) == 1
    assert lib.tetris_conv2d_launch(None, None, None, 1, 8, 8, 1, 1, None) == 1
    assert b"NULL" in lib.tetris_last_error()

"""CPU: the checker-side program format round-trips and has the promised structure."""
import numpy as np
import pytest

import progfmt


@pytest.mark.parametrize("shape,K,TIC", [((40, 20, 3, 3), 16, 16), ((17, 9, 3, 3), 8, 4),
                                         ((255, 35, 1, 1), 16, 32), ((16, 3, 7, 7), 16, 16)])
def test_pack_unpack_roundtrip(shape, K, TIC):
    rng = np.random.default_rng(1)
    w = rng.standard_normal(shape).astype(np.float32)
    w[rng.random(shape) < 0.85] = 0
    w[0] = 0  # an output channel without nonzeros
    ops, offs, nnz = progfmt.pack(w, K, TIC)
    assert nnz == np.count_nonzero(w)
    assert offs[0] == 0 and np.all(offs % progfmt.PROG_ALIGN_OPS == 0)
    assert ops.size == offs[-1] + progfmt.TAIL_PAD_OPS
    back = progfmt.unpack(ops, offs, shape[0], shape[1], shape[2], K, TIC)
    assert np.array_equal(back.view(np.uint32), w.view(np.uint32))


def test_record_order_is_ic_r_then_k_s():
    w = np.zeros((16, 16, 3, 3), np.float32)
    w[5, 2, 1, 2] = 1.0
    w[3, 2, 1, 0] = 2.0
    w[3, 0, 2, 1] = 3.0
    ops, offs, _ = progfmt.pack(w, 16, 16)
    codes = [int(o >> 32) for o in ops[: offs[1]]]
    payload = [int(o & 0xFFFFFFFF) for o in ops[: offs[1]]]
    assert codes[:6] == [48, 3 * 3 + 1, 48, 3 * 3 + 0, 5 * 3 + 2, 49]
    assert payload[0] == (0 << 8) | 2 and payload[2] == (2 << 8) | 1


@pytest.mark.parametrize("shape,K,TIC", [((40, 20, 3, 3), 16, 16), ((17, 9, 3, 3), 8, 4),
                                         ((255, 35, 1, 1), 16, 32), ((16, 3, 7, 7), 16, 16)])
def test_list_form_roundtrip(shape, K, TIC):
    rng = np.random.default_rng(2)
    w = rng.standard_normal(shape).astype(np.float32)
    w[rng.random(shape) < 0.85] = 0
    w[0] = 0
    units, offs = progfmt.pack_lists(w, K, TIC)
    assert offs[0] == 0 and np.all(offs % progfmt.PROG_ALIGN_OPS == 0)
    assert units.size == offs[-1] + progfmt.LIST_TAIL_UNITS
    back = progfmt.unpack_lists(units, offs, shape[0], shape[1], shape[2], K, TIC)
    assert np.array_equal(back.view(np.uint32), w.view(np.uint32))

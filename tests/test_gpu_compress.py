"""GPU: the device-side weight compressor against the checker-side packer, bit for bit."""
import numpy as np
import pytest

import progfmt

pytestmark = pytest.mark.gpu

CASES = [
    # (OC, IC, KS, density, K, TIC)
    (64, 64, 3, 0.10, 16, 16),
    (40, 20, 3, 0.15, 16, 16),
    (17, 9, 3, 0.30, 8, 4),
    (255, 35, 1, 0.10, 16, 32),
    (70, 48, 1, 0.20, 8, 16),
    (16, 3, 7, 0.50, 16, 16),
    (33, 130, 3, 0.05, 16, 32),
    (8, 8, 5, 1.00, 8, 8),
]


def make(OC, IC, KS, density, seed):
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((OC, IC, KS, KS)).astype(np.float32)
    w[rng.random(w.shape) >= density] = 0
    return w


@pytest.mark.parametrize("OC,IC,KS,density,K,TIC", CASES)
def test_stream_is_bit_identical_to_the_packer(tb, torch_cuda, OC, IC, KS, density, K, TIC):
    w = make(OC, IC, KS, density, OC * 1000 + IC)
    if OC > 4:
        w[2] = 0  # an output channel with no nonzeros at all
    f = tb.SparseFilter(w, IC, OC, KS, TILE_IC=TIC, oc_block=K)
    ops, offs = f.download()
    want_ops, want_offs, nnz = progfmt.pack(w, K, TIC)
    info = f.info()
    assert info.nnz == nnz == f.nnz_
    assert (info.n_oc_blocks, info.n_stages) == (-(-OC // K), -(-IC // TIC))
    assert np.array_equal(offs, want_offs)
    assert np.array_equal(ops, want_ops)
    units, loffs = f.download_lists()
    want_units, want_loffs = progfmt.pack_lists(w, K, TIC)
    assert np.array_equal(loffs, want_loffs)
    assert np.array_equal(units, want_units)
    f.close()


@pytest.mark.parametrize("OC,IC,KS,density,K,TIC", CASES[:5])
def test_compress_then_decompress_returns_the_filter(tb, torch_cuda, OC, IC, KS, density, K, TIC):
    w = make(OC, IC, KS, density, 77)
    w[0, 0, 0, 0] = -0.0  # a negative zero is a zero (reference: `value != 0.f`)
    f = tb.SparseFilter(w, IC, OC, KS, TILE_IC=TIC, oc_block=K)
    ops, offs = f.download()
    back = progfmt.unpack(ops, offs, OC, IC, KS, K, TIC)
    assert np.array_equal(back, w)  # value equality: -0.0 == 0.0
    assert np.array_equal(back.view(np.uint32)[w != 0], w.view(np.uint32)[w != 0])
    units, loffs = f.download_lists()
    back = progfmt.unpack_lists(units, loffs, OC, IC, KS, K, TIC)
    assert np.array_equal(back, w)
    assert np.array_equal(back.view(np.uint32)[w != 0], w.view(np.uint32)[w != 0])


def test_all_zero_filter_and_bad_arguments(tb, torch_cuda):
    w = np.zeros((20, 10, 3, 3), np.float32)
    f = tb.SparseFilter(w, 10, 20, 3)
    assert f.nnz_ == 0
    ops, offs = f.download()
    assert np.all((ops >> np.uint64(32)) == f.info().oc_block * 3 + 1)  # nothing but END records
    with pytest.raises(tb.TetrisError) as e:
        tb.SparseFilter(np.zeros((4, 4, 9, 9), np.float32), 4, 4, 9)
    assert e.value.status == 1
    with pytest.raises(tb.TetrisError):
        tb.SparseFilter(w, 10, 20, 3, device=99)
    with pytest.raises(tb.TetrisError) as e:
        tb.SparseFilter(np.zeros((8, 1, 3, 3), np.float32), 4, 8, 3, groups=2)
    assert e.value.status == 3

"""Compressed-filter files: the format on the CPU, the save -> load round trip on the GPU.

CPU part: a checker-side writer (tests/progfmt.py) produces the file the engine must accept, and
the host-only validator tetris_filter_file_check has to accept it and refuse every damaged
version -- truncated, foreign, wrong sizes, wrong offsets, flipped payload bit -- with
TETRIS_ERR_INVALID and a reason, never a crash (failures are injected on the host only).
GPU part: save -> load gives bit-identical downloads of both compressed forms, identical
convolution results (all variants) and the same tuned kernel choice; the saved file equals,
byte for byte, what the checker-side writer produces for the same filter.
"""
import os
import struct

import numpy as np
import pytest

import progfmt


def _filter(seed=3, shape=(40, 24, 3, 3), sparsity=0.85):
    rng = np.random.default_rng(seed)
    w = rng.normal(0, 0.05, shape).astype(np.float32)
    w[rng.random(shape) < sparsity] = 0
    w[1] = 0
    return w


def test_checker_file_is_accepted(tb, tmp_path):
    w = _filter()
    path = str(tmp_path / "f.tetris")
    progfmt.write_filter_file(path, w, K=8, TIC=16, tuned=[[4, 28, 28, 1, 1, 0, 8, 4, 1]])
    info = tb.filter_file_check(path)
    assert (info.in_channel, info.out_channel, info.kernel_size, info.groups) == (24, 40, 3, 1)
    assert info.nnz == np.count_nonzero(w) and info.oc_block == 8 and info.tile_ic == 16
    assert info.n_oc_blocks == 5 and info.n_stages == 2 and info.device == -1


def _flip(payload, at):
    b = bytearray(payload)
    b[at] ^= 0x40
    return bytes(b)


DAMAGE = {
    "bad_magic": lambda f, p: (dict(f, magic=b"NOTTETRI"), p),
    "future_version": lambda f, p: (dict(f, version=99), p),
    "flipped_payload_bit": lambda f, p: (dict(f, checksum=progfmt.fnv1a(p)), _flip(p, len(p) // 2)),
    "wrong_block_count": lambda f, p: (dict(f, n_oc_blocks=f["n_oc_blocks"] + 1), p),
    "bad_oc_block": lambda f, p: (dict(f, oc_block=12), p),
    "nnz_too_large": lambda f, p: (dict(f, nnz=10 ** 9), p),
    "payload_size_lies": lambda f, p: (dict(f, payload_bytes=len(p) + 8), p),
    "negative_shape": lambda f, p: (dict(f, in_channel=-3), p),
    "unsorted_offsets": lambda f, p: (f, p[:4] + struct.pack("<i", 10 ** 6) + p[8:]),
    "too_many_tuned": lambda f, p: (dict(f, n_tuned=1000), p),
}


@pytest.mark.parametrize("kind", sorted(DAMAGE))
def test_damaged_files_are_refused(tb, tmp_path, kind):
    path = str(tmp_path / (kind + ".tetris"))
    progfmt.write_filter_file(path, _filter(), K=8, TIC=16, damage=DAMAGE[kind])
    with pytest.raises(tb.TetrisError) as e:
        tb.filter_file_check(path)
    assert e.value.status == 1, str(e.value)
    assert os.path.basename(path) in str(e.value)


def test_truncated_missing_and_trailing(tb, tmp_path):
    path = str(tmp_path / "good.tetris")
    header, payload = progfmt.write_filter_file(path, _filter(), K=16, TIC=8)
    tb.filter_file_check(path)
    blob = header + payload
    for name, data in (("empty", b""), ("half_header", blob[:40]), ("header_only", header),
                       ("cut_payload", blob[:-9]), ("trailing", blob + b"\0")):
        p = str(tmp_path / (name + ".tetris"))
        with open(p, "wb") as fh:
            fh.write(data)
        with pytest.raises(tb.TetrisError) as e:
            tb.filter_file_check(p)
        assert e.value.status == 1
    with pytest.raises(tb.TetrisError) as e:
        tb.filter_file_check(str(tmp_path / "does_not_exist.tetris"))
    assert e.value.status == 1 and "cannot open" in str(e.value)
    with pytest.raises(tb.TetrisError):  # the loader validates before it touches a device
        tb.SparseFilter.load(str(tmp_path / "cut_payload.tetris"))


@pytest.mark.gpu
def test_save_load_round_trip(tb, torch_cuda, oracle, tmp_path):
    torch = torch_cuda
    w = _filter(seed=11, shape=(72, 64, 3, 3))
    f = tb.SparseFilter(w, 64, 72, 3, TILE_IC=16, oc_block=8)
    n, h = 4, 28
    rng = np.random.default_rng(12)
    x = rng.random((n, 64, h, h), dtype=np.float32)
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    out = torch.empty(n, h, h, 72, device="cuda")
    tb.tune_sparse_conv2d(f, xin, out, n, h, h, 1, 1, max_candidates=4)
    choice = tb.auto_choice(f, n, h, h, 1, 1)
    path = str(tmp_path / "layer.tetris")
    f.save(path)
    # the file is what the checker-side writer produces, apart from the tuned-plan records
    info = tb.filter_file_check(path)
    assert info.nnz == np.count_nonzero(w)
    ref_header, ref_payload = progfmt.write_filter_file(str(tmp_path / "ref.tetris"), w, K=8, TIC=16)
    blob = open(path, "rb").read()
    hdr = struct.calcsize(progfmt.FILE_HEADER)
    assert blob[hdr:hdr + len(ref_payload)] == ref_payload
    assert len(blob) == hdr + len(ref_payload) + progfmt.TUNED_INTS * 4  # one tuned plan

    g = tb.SparseFilter.load(path)
    assert (g.in_channel_, g.out_channel_, g.kernel_size_, g.nnz_, g.TILE_IC_) == (64, 72, 3, f.nnz_, 16)
    for a, b in zip(f.download() + f.download_lists(), g.download() + g.download_lists()):
        assert np.array_equal(a, b)
    assert tb.auto_choice(g, n, h, h, 1, 1) == choice  # the tuned plan travelled with the file
    want = oracle.host_conv2d(x, w, 1, 1)
    for variant in (tb.VARIANT_AUTO, tb.VARIANT_GENERIC, tb.VARIANT_TILED, tb.VARIANT_TENSOR):
        outs = []
        for flt in (f, g):
            y = torch.full((n, h, h, 72), float("nan"), device="cuda")
            tb.sparse_conv2d(flt, xin, y, n, h, h, 1, 1, variant=variant)
            torch.cuda.synchronize()
            flt.check()
            outs.append(y.cpu().numpy())
        assert np.array_equal(outs[0], outs[1]), "variant %d differs after the round trip" % variant
        assert oracle.compare(outs[1].transpose(0, 3, 1, 2), want)[0] == 0
    f.close(); g.close()


@pytest.mark.gpu
def test_save_load_depthwise_and_bad_device(tb, torch_cuda, oracle, tmp_path):
    torch = torch_cuda
    rng = np.random.default_rng(13)
    w = rng.normal(0, 0.2, (32, 1, 3, 3)).astype(np.float32)
    f = tb.SparseFilter(w, 32, 32, 3, groups=32)
    path = str(tmp_path / "dw.tetris")
    f.save(path)
    g = tb.SparseFilter.load(path)
    x = rng.random((2, 32, 14, 14), dtype=np.float32)
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    y = torch.full((2, 7, 7, 32), float("nan"), device="cuda")
    tb.sparse_conv2d(g, xin, y, 2, 14, 14, 2, 1)
    torch.cuda.synchronize()
    assert oracle.compare(y.cpu().numpy().transpose(0, 3, 1, 2), oracle.host_depthwise_conv2d(x, w, 2, 1))[0] == 0
    with pytest.raises(tb.TetrisError) as e:
        tb.SparseFilter.load(path, device=99)
    assert e.value.status == 1

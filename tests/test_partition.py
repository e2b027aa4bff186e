"""CPU: the multi-rank path (world_size 2, gloo) -- slicing and the optional output gather."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, batch, tmpdir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from conftest import load_package
    import importlib
    load_package()
    part = importlib.import_module("tetris_b200.partition")
    from oracle import oracle as orc
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(4)  # same data on every rank
        x = rng.random((batch, 6, 9, 8), dtype=np.float32)
        w = rng.standard_normal((10, 6, 3, 3)).astype(np.float32)
        w[rng.random(w.shape) < 0.8] = 0
        mine = part.shard_batch(torch.from_numpy(x))
        begin, count = part.slice_bounds(batch, world, rank)
        assert mine.shape[0] == count
        # stand-in for the per-GPU convolution: the CPU oracle on this rank's slice
        y_local = torch.from_numpy(orc.host_conv2d(mine.numpy(), w, 1, 1)) if count else \
            torch.zeros((0, 10, 9, 8))
        full = part.gather_shards(y_local, batch)
        want = orc.host_conv2d(x, w, 1, 1)
        assert np.array_equal(full.numpy(), want)
        open(os.path.join(tmpdir, "ok%d" % rank), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch", [5, 4, 1])
def test_two_ranks_shard_and_gather(tmp_path, batch):
    port = 29500 + (os.getpid() + batch) % 2000
    mp.spawn(_worker, args=(2, port, batch, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def test_python_and_native_slicing_agree(tb):
    import importlib
    part = importlib.import_module("tetris_b200.partition")
    for batch in (0, 1, 7, 16, 33):
        for world in (1, 2, 3, 8):
            for rank in range(world):
                assert part.slice_bounds(batch, world, rank) == tb.batch_slice(batch, world, rank)

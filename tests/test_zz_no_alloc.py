"""GPU: the allocation-free entry point against the allocating one.

tetris_list_offsets_noalloc serves callers that may not allocate device memory where they call
(a process that gave all device memory to a pool at start-up, code inside another component's
stream-ordered pipeline): they bring the dense filter and the output array, the library keeps
its scratch in a fixed array of its own image.  The offsets must equal, exactly (integer work),
the ones the allocating path (tetris_filter_create + tetris_filter_download_lists) produces --
on two calls in a row that share the scratch array, the second with fewer pieces than the first.
This file sorts last on purpose, so a stop-at-first-failure run has run everything else first.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def reference_offsets(tb, w, K, TIC):
    oc, ic, ks, _ = w.shape
    f = tb.SparseFilter(w, ic, oc, ks, TILE_IC=TIC, oc_block=K)
    _, offs = f.download_lists()
    f.close()
    return offs


def test_two_calls_in_a_row_match_the_allocating_path(tb, torch_cuda):
    torch = torch_cuda
    rng = np.random.default_rng(123)
    cases = [((96, 70, 3, 3), 8, 16), ((40, 20, 1, 1), 16, 8)]  # 60 pieces, then 9
    filters = []
    for shape, K, TIC in cases:
        w = rng.normal(0, 0.05, shape).astype(np.float32)
        w[rng.random(shape) < 0.85] = 0
        filters.append((w, K, TIC, reference_offsets(tb, w, K, TIC)))
    stream = torch.cuda.current_stream()
    outs = []
    for w, K, TIC, want in filters:  # back to back on one stream, no synchronisation between
        d_w = torch.from_numpy(w).cuda()
        d_out = torch.full((want.size,), -1, dtype=torch.int32, device="cuda")
        tb.list_offsets_noalloc(d_w, w.shape[1], w.shape[0], w.shape[2], K, TIC, d_out, cuda_stream=stream)
        outs.append((d_w, d_out))
    torch.cuda.synchronize()
    for (w, K, TIC, want), (_, d_out) in zip(filters, outs):
        assert np.array_equal(d_out.cpu().numpy(), want)


def test_device_memory_is_untouched_and_the_limit_itself_is_accepted(tb, torch_cuda):
    """The point of the entry point: a call changes nothing in the device's free memory.  And a
    filter with exactly as many pieces as the scratch array holds (128 channel blocks x 128
    stages = 16384) is served, with the same offsets as the allocating path."""
    torch = torch_cuda
    rng = np.random.default_rng(5)
    w = rng.normal(0, 0.05, (1024, 512, 1, 1)).astype(np.float32)
    w[rng.random(w.shape) < 0.9] = 0
    want = reference_offsets(tb, w, 8, 4)
    assert want.size == 16384 + 1
    d_w = torch.from_numpy(w).cuda()
    d_out = torch.full((want.size,), -1, dtype=torch.int32, device="cuda")
    tb.list_offsets_noalloc(d_w, 512, 1024, 1, 8, 4, d_out)  # warm-up: symbol lookup, module load
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    d_out.fill_(-1)
    tb.list_offsets_noalloc(d_w, 512, 1024, 1, 8, 4, d_out)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert np.array_equal(d_out.cpu().numpy(), want)


def test_host_pointers_are_refused(tb, torch_cuda):
    torch = torch_cuda
    host = np.zeros((16, 16), np.float32)
    out = torch.zeros(8, dtype=torch.int32, device="cuda")
    with pytest.raises(tb.TetrisError) as e:
        tb.list_offsets_noalloc(host, 16, 16, 1, 8, 4, out)
    assert e.value.status == 1 and "device memory" in str(e.value)


def test_sizes_beyond_the_scratch_are_refused(tb, torch_cuda):
    torch = torch_cuda
    d = torch.zeros(16, device="cuda")
    out = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(tb.TetrisError) as e:  # 8192 blocks x 4 stages = 32768 pieces > 16384
        tb.list_offsets_noalloc(d, 16, 65536, 1, 8, 4, out)
    assert e.value.status == 3 and "16384" in str(e.value)
    with pytest.raises(tb.TetrisError) as e:
        tb.list_offsets_noalloc(None, 16, 16, 1, 8, 4, out)
    assert e.value.status == 1

"""The allocation-free histogram entry point (lbk_histogram_noalloc) against the regular one.

Some callers may not allocate device memory when they need a histogram: code running inside a
stream callback, a task that a runtime registered without the right to allocate, a service whose
device footprint is frozen after start-up.  For them the library keeps the per-call scratch in a
fixed device array instead of a pool.  This test calls the entry point through the C ABI twice in a
row - the second call reuses the array the first one left dirty - and expects both results to be
bit-identical to lbk_histogram on the same inputs (integer sums: no tolerance needed), then checks
that a call beyond the fixed limits is refused.  It is collected last so that a failure here
cannot hide another test's result."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(L, bins, row_ptr, gpair, row_index, seg, F, hist, mode=0):
    a = L.HistogramArgs()
    a.bins, a.bin_bytes, a.n_rows, a.n_features = bins.data_ptr(), 1, bins.shape[1], F
    a.row_ptr, a.total_bins = row_ptr.data_ptr(), int(row_ptr[-1])
    if mode == 0:
        a.gpair = gpair.data_ptr()
    else:
        a.gpair_f32 = gpair.data_ptr()
    a.n_outputs = gpair.shape[1]
    a.row_index, a.seg, a.n_nodes, a.mode = row_index.data_ptr(), seg.data_ptr(), seg.shape[0] - 1, mode
    a.hist = hist.data_ptr()
    a.stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    a.host_buffers = 0
    return a


def test_noalloc_matches_regular_entry_point_twice():
    import legateboost_b200 as lb
    from legateboost_b200 import stages

    L = lb.library
    lib = L.load()
    assert torch.cuda.is_available()
    dev = torch.cuda.current_device()
    rs = np.random.RandomState(123)
    for N, F, K, n_nodes, nb in [(60000, 70, 2, 16, 256), (5000, 33, 1, 64, 40)]:
        bins = torch.from_numpy(rs.randint(0, nb, size=(N, F)).astype(np.uint8)).cuda()
        row_ptr = torch.from_numpy((np.arange(F + 1) * nb).astype(np.int32)).cuda()
        q = rs.randint(-30000, 30000, size=(N, K, 2)).astype(np.int32)
        q[:, :, 1] = np.abs(q[:, :, 1])
        gpair = torch.from_numpy(q).cuda()
        node = torch.from_numpy(rs.randint(0, n_nodes, size=N).astype(np.int32) + n_nodes - 1).cuda()
        row_index, seg = stages.group_rows(node, n_nodes - 1, n_nodes)
        bins_g = stages.to_padded_rows(bins)
        want = stages.histogram(bins_g, row_ptr, gpair, row_index, seg, F, mode=0)
        for call in range(2):
            got = torch.full_like(want, -7)  # garbage: the call must overwrite everything
            a = _args(L, bins_g, row_ptr, gpair, row_index, seg, F, got)
            rc = lib.lbk_histogram_noalloc(dev, C.byref(a))
            assert rc == 0, lib.lbk_last_error(None).decode()
            assert torch.equal(got, want), "call %d differs" % call


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch():
    import legateboost_b200 as lb

    L = lb.library
    lib = L.load()
    dev = torch.cuda.current_device()
    n_nodes = 4097  # one more than LBK_NOALLOC_MAX_NODES
    F = 2
    bins = torch.zeros((1, 8, 32), dtype=torch.uint8, device="cuda")
    row_ptr = torch.tensor([0, 2, 4], dtype=torch.int32, device="cuda")
    gpair = torch.zeros((8, 1, 2), dtype=torch.int32, device="cuda")
    row_index = torch.arange(8, dtype=torch.int32, device="cuda")
    seg = torch.zeros(n_nodes + 1, dtype=torch.int32, device="cuda")
    hist = torch.zeros((n_nodes, 1, 4, 2), dtype=torch.int64, device="cuda")
    a = _args(L, bins, row_ptr, gpair, row_index, seg, F, hist)
    rc = lib.lbk_histogram_noalloc(dev, C.byref(a))
    assert rc == -1
    assert b"at most 4096 nodes" in lib.lbk_last_error(None)

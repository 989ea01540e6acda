"""The allocation-free histogram entry point (lbk_histogram_noalloc) against the regular one.

Some callers may not allocate device memory when they need a histogram: a task that a runtime
registered without the right to allocate (the runtime has handed out the whole memory budget, so a
cudaMalloc fails or takes memory the runtime believes it owns), or a service whose device footprint
is frozen after start-up.  For them the library keeps the per-call scratch in a fixed device array
instead of a pool.  Every case below calls the entry point through the C ABI twice in a row - the
second call reuses the array the first one left dirty - and expects both results to equal
lbk_histogram's on the same inputs (integer sums bit for bit; float sums within 1e-5 of the largest
magnitude, the tolerance of the other float-histogram tests), then a call beyond the fixed limits
is refused.  It is collected last so that a failure here cannot hide another test's result."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(L, bins, row_ptr, gpair, row_index, seg, F, hist, mode=0):
    assert bins.dim() == 2  # the padded row-major layout: (rows, 32 * feature groups)
    a = L.HistogramArgs()
    a.bins, a.bin_bytes, a.n_rows, a.n_features = bins.data_ptr(), 1, bins.shape[0], F
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


def _inputs(rs, N, F, K, n_nodes, nb, kind):
    from legateboost_b200 import stages

    bins = torch.from_numpy(rs.randint(0, nb, size=(N, F)).astype(np.uint8)).cuda()
    row_ptr = torch.from_numpy((np.arange(F + 1) * nb).astype(np.int32)).cuda()
    if kind == "float":
        pairs = rs.normal(size=(N, K, 2)).astype(np.float32)
        pairs[:, :, 1] = np.abs(pairs[:, :, 1])
    else:
        pairs = rs.randint(-30000, 30000, size=(N, K, 2)).astype(np.int32)
        pairs[:, :, 1] = np.abs(pairs[:, :, 1])
        if kind == "large":
            # magnitudes near 2^24 only in the last quarter of the rows: the bound on the 32-bit
            # partial sums has to come from the whole array (127 rows between flushes, so every
            # chunk flushes in the middle); with two bins per feature a bin of a node collects
            # hundreds of these rows, and a partial sum that was not flushed in time would wrap
            n_big = N // 4
            pairs[-n_big:, :, :] = rs.randint(2 ** 24 - 1000, 2 ** 24, size=(n_big, K, 2))
    gpair = torch.from_numpy(pairs).cuda()
    node = torch.from_numpy(rs.randint(0, n_nodes, size=N).astype(np.int32) + n_nodes - 1).cuda()
    row_index, seg = stages.group_rows(node, n_nodes - 1, n_nodes)
    return stages.to_padded_rows(bins), row_ptr, gpair, row_index, seg


@pytest.mark.parametrize("N,F,K,n_nodes,nb,kind", [
    (60000, 70, 2, 16, 256, "int"),
    (5000, 33, 1, 64, 40, "int"),
    (40000, 64, 1, 8, 2, "large"),     # thousands of rows per node, |q| up to 2^24 in late rows
    (30000, 40, 1, 4, 128, "float"),
])
def test_noalloc_matches_regular_entry_point_twice(N, F, K, n_nodes, nb, kind):
    import legateboost_b200 as lb
    from legateboost_b200 import stages

    L = lb.library
    lib = L.load()
    assert torch.cuda.is_available()
    dev = torch.cuda.current_device()
    rs = np.random.RandomState(123)
    mode = 1 if kind == "float" else 0
    bins_g, row_ptr, gpair, row_index, seg = _inputs(rs, N, F, K, n_nodes, nb, kind)
    want = stages.histogram(bins_g, row_ptr, gpair, row_index, seg, F, mode=mode)
    for call in range(2):
        got = torch.full_like(want, -7)  # garbage: the call must overwrite everything
        a = _args(L, bins_g, row_ptr, gpair, row_index, seg, F, got, mode=mode)
        rc = lib.lbk_histogram_noalloc(dev, C.byref(a))
        assert rc == 0, lib.lbk_last_error(None).decode()
        if mode == 0:
            assert torch.equal(got, want), "call %d differs" % call
        else:
            tol = 1e-5 * float(want.abs().max())
            assert float((got - want).abs().max()) <= tol, "call %d differs" % call


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch():
    import legateboost_b200 as lb

    L = lb.library
    lib = L.load()
    dev = torch.cuda.current_device()
    n_nodes = 4097  # one more than LBK_NOALLOC_MAX_NODES
    F = 2
    bins = torch.zeros((8, 32), dtype=torch.uint8, device="cuda")
    row_ptr = torch.tensor([0, 2, 4], dtype=torch.int32, device="cuda")
    gpair = torch.zeros((8, 1, 2), dtype=torch.int32, device="cuda")
    row_index = torch.arange(8, dtype=torch.int32, device="cuda")
    seg = torch.zeros(n_nodes + 1, dtype=torch.int32, device="cuda")
    hist = torch.zeros((n_nodes, 1, 4, 2), dtype=torch.int64, device="cuda")
    a = _args(L, bins, row_ptr, gpair, row_index, seg, F, hist)
    rc = lib.lbk_histogram_noalloc(dev, C.byref(a))
    assert rc == -1
    assert b"at most 4096 nodes" in lib.lbk_last_error(None)
    # a multi-rank request has no communicator to go to
    seg4 = torch.tensor([0, 8], dtype=torch.int32, device="cuda")
    hist4 = torch.zeros((1, 1, 4, 2), dtype=torch.int64, device="cuda")
    a = _args(L, bins, row_ptr, gpair, row_index, seg4, F, hist4)
    a.all_reduce = 1
    rc = lib.lbk_histogram_noalloc(dev, C.byref(a))
    assert rc == -1
    assert b"all_reduce must be 0" in lib.lbk_last_error(None)

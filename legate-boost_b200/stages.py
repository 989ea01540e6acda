"""Stage-level entry points of the tree builder on torch CUDA tensors (thin wrappers over the
``lbk_*`` functions of include/lbk.h).  ``Tree.fit`` runs the same kernels in one call; these exist
so each stage can be checked against the oracle and timed on its own."""
import ctypes as C

import torch

from . import library as L
from .tree import _dtype_code, _stream_ptr


def split_proposals(X, split_samples, seed, row_offset=0, dataset_rows=None, ctx=None):
    """Sorted unique sampled values per feature as a CSR (proposals, row_ptr); last value = +inf."""
    ctx = ctx or L.context(X.device.index)
    N, F = X.shape
    dataset_rows = N if dataset_rows is None else dataset_rows
    props = torch.empty(F * split_samples, dtype=X.dtype, device=X.device)
    row_ptr = torch.empty(F + 1, dtype=torch.int32, device=X.device)
    B = C.c_int32(0)
    with torch.cuda.device(X.device):
        ctx.check(ctx.lib.lbk_split_proposals(
            ctx.handle, X.data_ptr(), _dtype_code(X), X.stride(0) if N else F, row_offset, N, F,
            split_samples, int(seed), dataset_rows, props.data_ptr(), row_ptr.data_ptr(), C.byref(B),
            _stream_ptr()))
    return props[: B.value], row_ptr


def bin_matrix(X, proposals, row_ptr, bin_bytes=1, ctx=None):
    """Bin ids, row-major with rows padded to whole 32-feature groups: shape (N, 32 * ceil(F / 32)),
    uint8 (or int16 storage)."""
    ctx = ctx or L.context(X.device.index)
    N, F = X.shape
    G = (F + 31) // 32
    dt = torch.uint8 if bin_bytes == 1 else torch.int16
    bins = torch.empty((N, G * 32), dtype=dt, device=X.device)
    with torch.cuda.device(X.device):
        ctx.check(ctx.lib.lbk_bin_matrix(
            ctx.handle, X.data_ptr(), _dtype_code(X), X.stride(0), N, F, proposals.data_ptr(),
            row_ptr.data_ptr(), bins.data_ptr(), bin_bytes, _stream_ptr()))
    return bins


def to_padded_rows(bins_row_major):
    """(N, F) feature-relative bin ids -> the (N, 32 * ceil(F / 32)) zero-padded layout the kernels read."""
    N, F = bins_row_major.shape
    G = (F + 31) // 32
    out = torch.zeros((N, G * 32), dtype=bins_row_major.dtype, device=bins_row_major.device)
    out[:, :F] = bins_row_major
    return out


def quantise(g, h, seed, row_offset=0, ctx=None, with_max_abs=False):
    """int32 pairs (N,K,2), root sums int64 (K,2), scale float64 (4,); with ``with_max_abs`` also the
    largest |grad| and |hess| of the pairs, int32 (2,), which ``histogram`` accepts."""
    ctx = ctx or L.context(g.device.index)
    g = g.contiguous()
    h = h.contiguous()
    N, K = g.shape
    gpair = torch.empty((N, K, 2), dtype=torch.int32, device=g.device)
    root = torch.empty((K, 2), dtype=torch.int64, device=g.device)
    scale = torch.empty(4, dtype=torch.float64, device=g.device)
    max_abs = torch.empty(2, dtype=torch.int32, device=g.device) if with_max_abs else None
    with torch.cuda.device(g.device):
        ctx.check(ctx.lib.lbk_quantise(ctx.handle, g.data_ptr(), h.data_ptr(), K, row_offset, N, K, int(seed),
                                       gpair.data_ptr(), root.data_ptr(), scale.data_ptr(),
                                       max_abs.data_ptr() if with_max_abs else None, _stream_ptr()))
    if with_max_abs:
        return gpair, root, scale, max_abs
    return gpair, root, scale


def group_rows(node_of_row, node_begin, n_nodes, ctx=None):
    """Stable grouping of row ids by node: (row_index, seg)."""
    ctx = ctx or L.context(node_of_row.device.index)
    N = node_of_row.shape[0]
    row_index = torch.empty(N, dtype=torch.int32, device=node_of_row.device)
    seg = torch.empty(n_nodes + 1, dtype=torch.int32, device=node_of_row.device)
    with torch.cuda.device(node_of_row.device):
        ctx.check(ctx.lib.lbk_group_rows(ctx.handle, node_of_row.data_ptr(), N, node_begin, n_nodes,
                                         row_index.data_ptr(), seg.data_ptr(), _stream_ptr()))
    return row_index, seg


def histogram(bins, row_ptr, gpair, row_index, seg, n_features, mode=0, hist=None, ctx=None, host=False,
              max_abs=None, all_reduce=False, max_bins=0, total_bins=None, pairs_by_position=False):
    """Histogram [n_nodes, K, B, 2] (int64 for mode 0, float64 for mode 1) of node-grouped rows.

    ``host=True`` takes CPU tensors and lets the library do the copies (the end-to-end path).
    ``pairs_by_position``: gpair[i] belongs to row_index[i] (the pairs were moved with the row ids)."""
    dev = bins.device
    ctx = ctx or L.context(None if host else dev.index)
    N = bins.shape[0]
    K = gpair.shape[1]
    n_nodes = seg.shape[0] - 1
    B = int(row_ptr[-1]) if total_bins is None else int(total_bins)
    if hist is None:
        hist = torch.empty((n_nodes, K, B, 2), dtype=torch.int64 if mode == 0 else torch.float64, device=dev,
                           pin_memory=host)
    a = L.HistogramArgs()
    a.bins, a.bin_bytes, a.n_rows, a.n_features = bins.data_ptr(), bins.element_size(), N, n_features
    a.row_ptr, a.total_bins = row_ptr.data_ptr(), B
    if mode == 0:
        a.gpair = gpair.data_ptr()
    else:
        a.gpair_f32 = gpair.data_ptr()
    a.n_outputs = K
    a.row_index, a.seg, a.n_nodes, a.mode = row_index.data_ptr(), seg.data_ptr(), n_nodes, mode
    a.hist = hist.data_ptr()
    a.stream = _stream_ptr()
    a.host_buffers = 1 if host else 0
    a.max_abs = max_abs.data_ptr() if max_abs is not None else None
    a.all_reduce = int(all_reduce)  # False / True, or 2 = only the owned features are summed
    a.max_bins = int(max_bins)
    a.pairs_by_position = 1 if pairs_by_position else 0
    ctx.check(ctx.lib.lbk_histogram(ctx.handle, C.byref(a)))
    return hist

"""Randomised sweeps through the C ABI with fixed seeds: shapes, node distributions and options that
the hand-picked parity cases do not enumerate.

Trees: every case must equal the oracle (quantised mode) bit for bit on the five arrays, the walk of
predict over X must equal the oracle's, and the leaf record must name the node predict ends in.
Histograms: integer pairs must equal an independent int64 ``index_add_`` histogram exactly,
whatever the node sizes (one giant node, empty nodes, rows outside the level), the pair order (by row
or by position) and the magnitudes (up to 2^24, which forces flushes of the 32-bit partial sums);
float pairs are float32 sums, so they are held to a per-bin bound of 1e-6 x the sum of the
magnitudes that went into the bin (+1e-6)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_trees_match_the_oracle(seed):
    from legateboost_b200.tree import build_tree_arrays, predict_arrays
    from oracle import oracle as O

    O.build()
    rs = np.random.RandomState(seed)
    for _ in range(40):
        N = int(rs.choice([1, 2, 3, 17, 100, 1000, 5000, 20000]))
        F = int(rs.choice([1, 2, 5, 31, 32, 33, 64, 65, 100, 130, 200, 300]))
        K = int(rs.choice([1, 1, 1, 2, 3, 5]))
        D = int(rs.choice([0, 1, 2, 4, 6, 8, 10]))
        S = int(rs.choice([2, 3, 16, 64, 255, 256, 257, 300]))
        dt = rs.choice([np.float32, np.float64])
        kind = rs.randint(4)
        X = rs.normal(size=(N, F)).astype(dt)
        if kind == 1:
            X = np.round(X * 2) / 2                 # many ties
        if kind == 2:
            X[:, : max(1, F // 3)] = 1.0            # constant features
        g = rs.normal(size=(N, K))
        h = rs.random((N, K)) * (1e-4 if kind == 3 else 1.0) + (0.0 if kind == 3 else 0.05)  # 3: hessians that quantise to 0
        kw = dict(l1=float(rs.choice([0.0, 0.0, 0.3])), l2=float(rs.choice([1.0, 0.0, 2.5])),
                  min_split_gain=float(rs.choice([0.0, 0.0, 0.5])))
        mask = None
        if rs.random() < 0.3:
            mask = rs.random(F) < 0.5
            mask[rs.randint(F)] = True
        tree_seed = int(rs.randint(0, 2 ** 31 - 1))
        what = dict(N=N, F=F, K=K, D=D, S=S, dt=dt.__name__, kind=kind, kw=kw, mask=mask is not None, seed=tree_seed)
        want = O.build_tree(X, g, h, max_depth=D, split_samples=S, seed=tree_seed, mode="Q", feature_set=mask, **kw)
        got = build_tree_arrays(_dev(X), _dev(g), _dev(h), max_depth=D, split_samples=S, seed=tree_seed,
                                feature_set=None if mask is None else torch.from_numpy(mask), row_offset=0,
                                dataset_rows=N, want_leaf=True, **kw)
        for name in ("feature", "split_value", "gain", "leaf_value", "hessian"):
            assert np.array_equal(got[name].cpu().numpy(), getattr(want, name)), (name, what)
        pred = predict_arrays(_dev(X), [(got["leaf_value"], got["feature"], got["split_value"])])
        assert np.array_equal(pred.cpu().numpy(), O.predict(X, [(want.leaf_value, want.feature, want.split_value)])), what
        assert torch.equal(got["leaf_value"][got["leaf"].long()], pred), what


def _reference_histogram(bins, pairs, node, node_begin, n_nodes, F, nb, K, dtype):
    """[node][k][feature * nb + bin] sums of the pairs of the rows whose node lies in the level."""
    dev = bins.device
    B = F * nb
    out = torch.zeros((n_nodes * K * B, 2), dtype=dtype, device=dev)
    rows = torch.nonzero((node >= node_begin) & (node < node_begin + n_nodes)).squeeze(1)
    if rows.numel() == 0:
        return out.view(n_nodes, K, B, 2)
    slot = node[rows].long() - node_begin
    sub = bins[rows]
    for k in range(K):
        vals = pairs[rows, k, :].to(dtype)
        base = (slot * K + k) * B
        for f0 in range(0, F, 8):
            f1 = min(F, f0 + 8)
            idx = base[:, None] + sub[:, f0:f1].long() + (torch.arange(f0, f1, device=dev) * nb)[None, :]
            out.index_add_(0, idx.reshape(-1), vals[:, None, :].expand(-1, f1 - f0, -1).reshape(-1, 2))
    return out.view(n_nodes, K, B, 2)


@pytest.mark.parametrize("seed", [11, 12])
def test_random_histograms_match_an_independent_sum(seed):
    from legateboost_b200 import stages

    dev = torch.device("cuda")
    rs = np.random.RandomState(seed)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    for _ in range(150):
        N = int(rs.choice([1, 10, 1000, 50000, 400000, 1500000]))
        F = int(rs.choice([1, 3, 31, 32, 33, 64, 70, 128, 160]))
        nb = int(rs.choice([2, 40, 256]))
        n_nodes = int(rs.choice([1, 2, 7, 64, 300, 2000]))
        K = int(rs.choice([1, 1, 2, 3]))
        N = min(N, 100_000_000 // F)
        is_float = rs.random() < 0.25
        dist = rs.randint(4)
        by_position = bool(rs.randint(2))
        big = rs.random() < 0.3
        bins = torch.randint(0, nb, (N, F), dtype=torch.uint8, device=dev, generator=gen)
        row_ptr = torch.arange(F + 1, dtype=torch.int32, device=dev) * nb
        if dist == 0:    # even
            node = torch.randint(0, n_nodes, (N,), dtype=torch.int32, device=dev, generator=gen)
        elif dist == 1:  # skewed: most rows in the first nodes
            node = (torch.rand((N,), device=dev, generator=gen) ** 4 * n_nodes).to(torch.int32).clamp_(max=n_nodes - 1)
        elif dist == 2:  # one giant node, the others small, some rows outside the level
            node = torch.randint(0, n_nodes + 3, (N,), dtype=torch.int32, device=dev, generator=gen)
            node[torch.rand((N,), device=dev, generator=gen) < 0.8] = n_nodes // 2
        else:            # every other node empty
            node = (torch.randint(0, max(1, n_nodes // 2), (N,), dtype=torch.int32, device=dev, generator=gen) * 2)
            node.clamp_(max=n_nodes - 1)
        node_begin = n_nodes - 1 if rs.randint(2) else 0
        node = node + node_begin
        if is_float:
            pairs = torch.randn((N, K, 2), dtype=torch.float32, device=dev, generator=gen)
        else:
            top = 2 ** 24 if big else 30000
            pairs = torch.randint(-top, top, (N, K, 2), dtype=torch.int32, device=dev, generator=gen)
        what = dict(N=N, F=F, nb=nb, n_nodes=n_nodes, K=K, float=is_float, dist=dist, by_position=by_position, big=big,
                    node_begin=node_begin)
        row_index, seg = stages.group_rows(node, node_begin, n_nodes)
        n_in = int(seg[-1])
        # (no row in the level: an empty tensor has no address to pass, any pair array will do)
        given = pairs[row_index[:n_in].long()].contiguous() if by_position and n_in > 0 else pairs
        max_abs = None
        if not is_float and (by_position or rs.randint(2)):
            max_abs = pairs.abs().amax(dim=(0, 1)).to(torch.int32)
        got = stages.histogram(stages.to_padded_rows(bins), row_ptr, given, row_index, seg, F, mode=1 if is_float else 0,
                               max_abs=max_abs, pairs_by_position=by_position)
        if is_float:
            want = _reference_histogram(bins, pairs, node, node_begin, n_nodes, F, nb, K, torch.float64)
            bound = _reference_histogram(bins, pairs.abs(), node, node_begin, n_nodes, F, nb, K, torch.float64) * 1e-6 + 1e-6
            assert bool(((got - want).abs() <= bound).all()), what
        else:
            want = _reference_histogram(bins, pairs, node, node_begin, n_nodes, F, nb, K, torch.int64)
            assert torch.equal(got, want), what
        del bins, pairs, node, given

"""GPU parity tests: every stage of the CUDA tree builder and the whole BUILD_TREE / PREDICT calls
against the CPU oracle on identical seeded inputs, through the C ABI (liblbk.so).

Bars: integer / index results bit-exact; float histograms <= 1e-5 relative (to the largest
magnitude of the histogram); predictions bit-exact (the bar is <= 1e-4)."""
import glob
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def lb():
    import legateboost_b200 as lb
    from legateboost_b200 import stages  # noqa: F401

    assert torch.cuda.is_available(), "these tests need a CUDA device"
    lb.library.load()  # fails loudly if liblbk.so is missing
    return lb


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def tree_tuple(t):
    return (t.leaf_value, t.feature, t.split_value)


def to_row_major(bins_p, F):
    """Drops the padding columns of the kernels' layout (rows padded to whole 32-feature groups)."""
    assert bins_p.shape[1] == (F + 31) // 32 * 32
    assert not bins_p[:, F:].any()
    return bins_p[:, :F]


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("N,F,S", [(1000, 7, 16), (5000, 50, 256), (300, 33, 500), (64, 3, 2048), (2, 1, 256)])
def test_split_proposals_and_bins(lb, oracle, dtype, N, F, S):
    from legateboost_b200 import stages

    rs = np.random.RandomState(N + F)
    X = rs.random((N, F)).astype(dtype)
    X[:, 0] = np.round(X[:, 0] * 3)  # a low-cardinality feature
    for seed in (0, 1872583848):
        want_p, want_rp = oracle.split_proposals(X, S, seed, mode="Q")
        got_p, got_rp = stages.split_proposals(dev(X), S, seed)
        assert np.array_equal(got_rp.cpu().numpy(), want_rp)
        assert np.array_equal(got_p.cpu().numpy(), want_p)
        want_bins = oracle.bin_x(X, want_p, want_rp)
        mb = int(np.diff(want_rp).max())
        bb = 1 if mb <= 256 else 2
        got = stages.bin_matrix(dev(X), got_p, got_rp, bin_bytes=bb)
        assert np.array_equal(to_row_major(got, F).cpu().numpy().astype(np.int16), want_bins)


@pytest.mark.parametrize("N,K", [(1, 1), (1000, 1), (5000, 3), (70000, 2), (1 << 21, 1)])
def test_quantise(lb, oracle, N, K):
    from legateboost_b200 import stages

    rs = np.random.RandomState(N)
    g = rs.normal(size=(N, K)) * 10.0 ** rs.randint(-2, 3, size=(N, K))
    h = rs.random((N, K)) + 1e-8
    want_q, want_scale = oracle.quantise(g, h, seed=1234567)
    gp, root, scale = stages.quantise(dev(g), dev(h), seed=1234567)
    assert np.array_equal(scale.cpu().numpy(), want_scale)
    assert np.array_equal(gp.cpu().numpy().astype(np.int64), want_q)
    assert np.array_equal(root.cpu().numpy(), want_q.sum(axis=0))


def test_quantise_row_offset(lb, oracle):
    # the quantised pair depends on the GLOBAL row id: a shard quantised on its own, with the
    # scale of its own |g| sum, must equal the oracle's shard
    from legateboost_b200 import stages

    rs = np.random.RandomState(0)
    g = rs.normal(size=(4000, 2))
    h = np.ones((4000, 2))
    gp, _, scale = stages.quantise(dev(g[1000:3000]), dev(h[1000:3000]), seed=99, row_offset=1000)
    want_q, want_scale = oracle.quantise(g, h, seed=99, rank_off=[0, 1000, 3000, 4000])
    # the oracle takes the max over shards; compare only when this shard carries the max
    single_q, single_scale = oracle.quantise(g[1000:3000], h[1000:3000], seed=99)
    assert np.array_equal(scale.cpu().numpy(), single_scale)
    if np.array_equal(single_scale, want_scale):
        assert np.array_equal(gp.cpu().numpy().astype(np.int64), want_q[1000:3000])


# ---------------------------------------------------------------------------------------------
def _hist_case(rs, N, F, K, n_nodes, nb):
    bins = rs.randint(0, nb, size=(N, F)).astype(np.uint8)
    row_ptr = (np.arange(F + 1) * nb).astype(np.int32)
    node = rs.randint(0, n_nodes, size=N).astype(np.int32) + (n_nodes - 1)
    return bins, row_ptr, node


@pytest.mark.parametrize("N,F,K,n_nodes,nb", [(200000, 128, 1, 128, 256), (50000, 50, 3, 8, 256),
                                              (3000, 100, 1, 64, 7), (100, 5, 2, 4, 256), (70000, 64, 1, 1, 256),
                                              (60000, 70, 2, 5, 200), (90000, 161, 1, 3, 256)])
def test_histogram_int_exact(lb, oracle, N, F, K, n_nodes, nb):
    from legateboost_b200 import stages

    rs = np.random.RandomState(F)
    bins, row_ptr, node = _hist_case(rs, N, F, K, n_nodes, nb)
    q = rs.randint(-(2 ** 20), 2 ** 20, size=(N, K, 2)).astype(np.int32)
    q[:, :, 1] = np.abs(q[:, :, 1])
    want = oracle.histogram_q(bins, row_ptr, q, node, n_nodes - 1, 2 * n_nodes - 1)
    row_index, seg = stages.group_rows(dev(node), n_nodes - 1, n_nodes)
    # grouping is stable: rows ascending inside each node
    ri, sg = row_index.cpu().numpy(), seg.cpu().numpy()
    assert sg[-1] == N
    for j in range(n_nodes):
        r = ri[sg[j]:sg[j + 1]]
        assert np.all(node[r] == j + n_nodes - 1) and np.all(np.diff(r) > 0)
    got = stages.histogram(stages.to_padded_rows(dev(bins)), dev(row_ptr), dev(q), row_index, seg, F, mode=0)
    assert np.array_equal(got.cpu().numpy(), want)
    # the same pairs stored in row_index order (as the tree builder keeps them)
    got = stages.histogram(stages.to_padded_rows(dev(bins)), dev(row_ptr), _by_position(dev(q), row_index), row_index, seg,
                           F, mode=0, pairs_by_position=True, max_abs=_max_abs(q))
    assert np.array_equal(got.cpu().numpy(), want)


def _by_position(pairs, row_index):
    return pairs[row_index.long()].contiguous()


def _max_abs(q):
    return dev(np.abs(q.astype(np.int64)).reshape(-1, 2).max(axis=0).astype(np.int32))


@pytest.mark.parametrize("F,K", [(32, 2), (64, 1)])
def test_histogram_many_large_nodes(lb, oracle, F, K):
    """More large, unequal nodes than resident blocks, some of them empty: the planner cuts the
    larger nodes into chunks that leave partial sums; the sums stay exact."""
    from legateboost_b200 import stages

    N, n_nodes = 6_000_000, 200
    rng = np.random.default_rng(F + K)
    weight = rng.uniform(0.5, 1.5, size=n_nodes)
    weight[[0, 17, 18, 199]] = 0.0  # empty nodes, at both ends and in a row
    edges = np.cumsum(weight / weight.sum())
    node = np.minimum(np.searchsorted(edges, rng.random(N), side="right"), n_nodes - 2).astype(np.int32) + (n_nodes - 1)
    bins = rng.integers(0, 256, size=(N, F), dtype=np.uint8)
    row_ptr = (np.arange(F + 1) * 256).astype(np.int32)
    q = rng.integers(-200, 200, size=(N, K, 2), dtype=np.int32)
    q[:, :, 1] = np.abs(q[:, :, 1])
    want = oracle.histogram_q(bins, row_ptr, q, node, n_nodes - 1, 2 * n_nodes - 1)
    row_index, seg = stages.group_rows(dev(node), n_nodes - 1, n_nodes)
    got = stages.histogram(stages.to_padded_rows(dev(bins)), dev(row_ptr), dev(q), row_index, seg, F, mode=0)
    assert np.array_equal(got.cpu().numpy(), want)


def test_histogram_int_no_wraparound(lb, oracle):
    """Partial sums that exceed int32 in one chunk must still come out exact."""
    from legateboost_b200 import stages

    N, F = 6000, 4
    rs = np.random.RandomState(5)
    bins = np.zeros((N, F), dtype=np.uint8)  # everything in one bin
    row_ptr = (np.arange(F + 1) * 2).astype(np.int32)
    node = np.zeros(N, dtype=np.int32)
    q = np.full((N, 1, 2), 2 ** 30, dtype=np.int32)  # sums reach 6000 * 2^30
    q[::2, 0, 0] *= -1
    q[:, 0, 0] += rs.randint(0, 1000, size=N).astype(np.int32)
    want = oracle.histogram_q(bins, row_ptr, q, node, 0, 1)
    row_index, seg = stages.group_rows(dev(node), 0, 1)
    got = stages.histogram(stages.to_padded_rows(dev(bins)), dev(row_ptr), dev(q), row_index, seg, F, mode=0)
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("N,F,K,n_nodes", [(200000, 128, 1, 128), (20000, 40, 2, 16)])
def test_histogram_float_tolerance(lb, oracle, N, F, K, n_nodes):
    from legateboost_b200 import stages

    rs = np.random.RandomState(7)
    bins, row_ptr, node = _hist_case(rs, N, F, K, n_nodes, 256)
    gh = np.stack([rs.normal(size=(N, K)), np.ones((N, K))], axis=2).astype(np.float32)
    want = oracle.histogram_d(bins, row_ptr, gh[:, :, 0].copy(), gh[:, :, 1].copy(), node, n_nodes - 1, 2 * n_nodes - 1)
    row_index, seg = stages.group_rows(dev(node), n_nodes - 1, n_nodes)
    got = stages.histogram(stages.to_padded_rows(dev(bins)), dev(row_ptr), dev(gh), row_index, seg, F, mode=1)
    got = got.cpu().numpy()
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 1e-5 * scale


def test_histogram_host_buffers(lb, oracle):
    from legateboost_b200 import stages

    rs = np.random.RandomState(11)
    N, F, K, n_nodes = 30000, 64, 1, 8
    bins, row_ptr, node = _hist_case(rs, N, F, K, n_nodes, 256)
    q = rs.randint(-1000, 1000, size=(N, K, 2)).astype(np.int32)
    want = oracle.histogram_q(bins, row_ptr, q, node, n_nodes - 1, 2 * n_nodes - 1)
    row_index, seg = stages.group_rows(dev(node), n_nodes - 1, n_nodes)
    bins_g = stages.to_padded_rows(dev(bins)).cpu().pin_memory()
    got = stages.histogram(bins_g, torch.from_numpy(row_ptr), torch.from_numpy(q).pin_memory(),
                           row_index.cpu(), seg.cpu(), F, mode=0, host=True)
    assert np.array_equal(got.numpy(), want)


# ---------------------------------------------------------------------------------------------
TREE_CASES = [
    # N, F, K, depth, S, dtype, kwargs
    (1000, 10, 1, 4, 64, np.float32, {}),
    (5000, 20, 3, 6, 256, np.float64, {}),
    (300, 5, 2, 8, 16, np.float32, {}),
    (10000, 100, 5, 7, 256, np.float64, {}),
    (20000, 50, 1, 6, 256, np.float32, {}),
    (2000, 33, 1, 5, 500, np.float32, {}),                      # two-byte bins
    (3000, 12, 2, 6, 64, np.float32, {"l1": 0.5, "l2": 2.0, "min_split_gain": 0.01}),
    (2, 1, 1, 12, 256, np.float64, {}),
    (500, 6, 1, 0, 32, np.float32, {}),                          # depth 0: root only
    (4000, 9, 1, 5, 128, np.float32, {"mask": True}),
]


def _run_tree_case(lb, oracle, case, seed, n_ranks=1, trace_nodes=0, hess_small=False):
    from legateboost_b200.tree import build_tree_arrays

    N, F, K, D, S, dt, kw = case
    kw = dict(kw)
    rs = np.random.RandomState(N * 7 + F)
    X = rs.random((N, F)).astype(dt)
    X[:, 0] = np.round(X[:, 0] * 5) / 5
    g = rs.normal(size=(N, K))
    h = rs.random((N, K)) * (1e-3 if hess_small else 1.0) + (0.0 if hess_small else 0.1)
    mask = None
    if kw.pop("mask", False):
        mask = rs.random(F) < 0.5
        mask[0] = True
    want = oracle.build_tree(X, g, h, max_depth=D, split_samples=S, seed=seed, mode="Q", feature_set=mask,
                             trace_nodes=trace_nodes, **kw)
    got = build_tree_arrays(dev(X), dev(g), dev(h), max_depth=D, split_samples=S, seed=seed,
                            feature_set=None if mask is None else torch.from_numpy(mask),
                            row_offset=0, dataset_rows=N, trace_nodes=trace_nodes, **kw)
    return X, want, got


@pytest.mark.parametrize("case", TREE_CASES, ids=[str(c[:5]) for c in TREE_CASES])
def test_build_tree_bit_exact(lb, oracle, case):
    for seed in (2, 1872583848):
        X, want, got = _run_tree_case(lb, oracle, case, seed)
        assert got["B"] == want.B
        assert np.array_equal(got["node_sums"].cpu().numpy(), want.node_sums)
        assert np.array_equal(got["feature"].cpu().numpy(), want.feature)
        assert np.array_equal(got["split_value"].cpu().numpy(), want.split_value)
        assert np.array_equal(got["gain"].cpu().numpy(), want.gain)
        assert np.array_equal(got["leaf_value"].cpu().numpy(), want.leaf_value)
        assert np.array_equal(got["hessian"].cpu().numpy(), want.hessian)


def test_build_tree_histograms_bit_exact(lb, oracle):
    """Every node's histogram as it was when its split was evaluated (scan, write-skip rule,
    sibling subtraction), including a case where quantised hessians of 0 occur."""
    for case, small in (((3000, 8, 2, 5, 32, np.float32, {}), False), ((3000, 8, 2, 5, 32, np.float32, {}), True)):
        D = case[3]
        nodes = 2 ** D - 1
        X, want, got = _run_tree_case(lb, oracle, case, seed=5, trace_nodes=nodes, hess_small=small)
        assert np.array_equal(got["trace_hist"].cpu().numpy(), want.trace_hist)
        assert np.array_equal(got["feature"].cpu().numpy(), want.feature)


def test_scratch_through_the_callers_allocator(lb):
    """lbk_context_set_allocator: with torch's caching allocator behind the callbacks a whole tree is
    built without the library's own pool reserving a byte, and it is the same tree."""
    from legateboost_b200.tree import build_tree_arrays

    N, F, K, D = 50000, 40, 2, 6
    rs = np.random.RandomState(3)
    X, g, h = dev(rs.random((N, F)).astype(np.float32)), dev(rs.normal(size=(N, K))), dev(rs.random((N, K)) + 0.1)
    kw = dict(max_depth=D, split_samples=256, seed=9, row_offset=0, dataset_rows=N, want_leaf=True)
    want = build_tree_arrays(X, g, h, **kw)
    ctx = lb.library.context(X.device.index)
    torch.cuda.synchronize()
    ctx.check(ctx.lib.lbk_context_trim(ctx.handle))
    assert ctx.pool_bytes() == 0
    ctx.use_torch_allocator(True)
    try:
        got = build_tree_arrays(X, g, h, **kw)
        torch.cuda.synchronize()
        assert ctx.pool_bytes() == 0
        assert len(ctx._held) == 0  # everything was given back
    finally:
        ctx.use_torch_allocator(False)
    for name in ("feature", "split_value", "gain", "leaf_value", "hessian", "leaf"):
        assert torch.equal(got[name], want[name]), name
    # the pool is in use again afterwards
    build_tree_arrays(X, g, h, **kw)
    assert ctx.pool_bytes() > 0


@pytest.mark.parametrize("N,F,K,D,S,dtype", [
    (50001, 40, 1, 8, 256, np.float32),    # rows of 64 bytes, a last chunk of one row
    (20000, 7, 2, 5, 64, np.float64),      # one group
    (9000, 130, 1, 6, 256, np.float32),    # rows of 160 bytes
    (6000, 300, 1, 4, 128, np.float32),    # rows wider than the tiled form takes
    (7000, 20, 1, 6, 400, np.float32),     # two-byte bins
    (3000, 5, 1, 13, 256, np.float32),     # more nodes than the tiled form takes
])
def test_leaf_record_is_the_walk_of_predict(lb, N, F, K, D, S, dtype):
    """out_leaf (read off the binned matrix) names, for every row, the node whose value predict adds
    for that row when it walks X: leaf_value[out_leaf] == predict(X, tree), bit for bit."""
    from legateboost_b200.tree import build_tree_arrays, predict_arrays

    rs = np.random.RandomState(N % 97)
    X = dev(rs.normal(size=(N, F)).astype(dtype))
    g, h = dev(rs.normal(size=(N, K))), dev(rs.random((N, K)) + 0.05)
    t = build_tree_arrays(X, g, h, max_depth=D, split_samples=S, seed=4, row_offset=0, dataset_rows=N, want_leaf=True)
    # distinct values per node, so that equal predictions mean equal nodes
    M = t["feature"].shape[0]
    values = torch.arange(1, M * K + 1, dtype=torch.float64, device=X.device).reshape(M, K)
    pred = predict_arrays(X, [(values, t["feature"], t["split_value"])])
    leaf = t["leaf"].long()
    assert int(leaf.min()) >= 0 and int(leaf.max()) < M
    assert torch.equal(values[leaf], pred)


def test_peer_barrier_gives_up_and_reports(lb):
    """A peer that never reaches the barrier of the histogram exchange: the barrier kernel's wait is
    bounded (about a second), then it reports through the status word and returns, the call returns
    an error, and the context keeps working.  Emulated on one GPU with a flag that nothing sets."""
    import time
    from legateboost_b200.tree import build_tree_arrays

    ctx = lb.library.context(torch.cuda.current_device())
    stream = torch.cuda.current_stream().cuda_stream
    assert ctx.lib.lbk_selftest_peer_barrier(ctx.handle, 1, stream) == 0
    t0 = time.perf_counter()
    rc = ctx.lib.lbk_selftest_peer_barrier(ctx.handle, 0, stream)
    dt = time.perf_counter() - t0
    assert rc != 0 and b"fault code 41" in ctx.lib.lbk_last_error(ctx.handle)
    assert dt < 20.0
    # the status word was cleared and the device still answers: a present peer passes, a tree builds
    assert ctx.lib.lbk_selftest_peer_barrier(ctx.handle, 1, stream) == 0
    rs = np.random.RandomState(0)
    X, g, h = dev(rs.random((500, 4)).astype(np.float32)), dev(rs.normal(size=(500, 1))), dev(rs.random((500, 1)) + 0.1)
    t = build_tree_arrays(X, g, h, max_depth=2, split_samples=16, seed=1, row_offset=0, dataset_rows=500)
    assert int((t["feature"] >= 0).sum()) >= 1


def test_fixed_sketch_save_and_reuse(lb, oracle):
    """The optional sketch buffer: a saving call gives the oracle's tree, a reusing call with the same
    seed gives it again without reading X, a reusing call with another seed splits on the saved
    proposals only; a buffer without a sketch and a sketch of another shape are errors."""
    from legateboost_b200 import stages
    from legateboost_b200.tree import Sketch, build_tree_arrays

    N, F, K, D, S = 20000, 37, 2, 6, 64
    rs = np.random.RandomState(11)
    X = rs.normal(size=(N, F)).astype(np.float32)
    g = rs.normal(size=(N, K))
    h = rs.uniform(0.5, 2.0, size=(N, K))
    want = oracle.build_tree(X, g, h, max_depth=D, split_samples=S, seed=7, mode="Q")
    dX, dg, dh = dev(X), dev(g), dev(h)
    kw = dict(max_depth=D, split_samples=S, row_offset=0, dataset_rows=N, want_leaf=True)
    sk = Sketch()
    saved = build_tree_arrays(dX, dg, dh, seed=7, sketch=sk, **kw)
    assert sk.key is not None
    reused = build_tree_arrays(dX, dg, dh, seed=7, sketch=sk, **kw)
    for got in (saved, reused):
        for name in ("feature", "split_value", "gain", "leaf_value", "hessian"):
            assert np.array_equal(got[name].cpu().numpy(), getattr(want, name)), name
    assert torch.equal(saved["leaf"], reused["leaf"])
    # another seed on the saved sketch: other roundings, the proposals of seed 7
    other = build_tree_arrays(dX, dg, dh, seed=8, sketch=sk, **kw)
    props, row_ptr = stages.split_proposals(dX, S, 7)
    props, row_ptr = props.cpu().numpy().astype(np.float64), row_ptr.cpu().numpy()
    feat, split = other["feature"].cpu().numpy(), other["split_value"].cpu().numpy()
    assert (feat >= 0).sum() > 10
    for f, v in zip(feat, split):
        if f >= 0:
            assert v in props[row_ptr[f]:row_ptr[f + 1]]
    fresh = build_tree_arrays(dX, dg, dh, seed=8, **{**kw, "want_leaf": False})
    assert not np.array_equal(fresh["split_value"].cpu().numpy(), split)  # seed 8 has proposals of its own
    # errors
    from legateboost_b200 import library as L
    empty = Sketch()
    empty.mode_for(dX, S, L.context(0))
    empty.buffer.zero_()
    empty.key = sk.key  # pretend it was saved
    with pytest.raises(L.LbkError, match="no saved sketch"):
        build_tree_arrays(dX, dg, dh, seed=7, sketch=empty, **kw)
    X36 = dX[:, :36].contiguous()
    wrong = Sketch()
    wrong.buffer, wrong.key = sk.buffer, (lb.tree._tensor_key(X36), S)  # pretend it was saved for X36
    with pytest.raises(L.LbkError, match="another shape"):
        build_tree_arrays(X36, dg, dh, seed=7, sketch=wrong, **kw)


def test_tree_pickle_round_trip(lb):
    """A pickled tree predicts the same bits and leaves the per-fit scratch (leaf record, sketch) behind."""
    import pickle

    rs = np.random.RandomState(2)
    X = dev(rs.normal(size=(4000, 9)).astype(np.float32))
    g, h = dev(rs.normal(size=(4000, 1))), dev(np.ones((4000, 1)))
    t = lb.Tree(max_depth=4, split_samples=32).set_random_state(np.random.RandomState(1))
    t.sketch = lb.Sketch()
    t.fit(X, g, h)
    blob = pickle.dumps(t)
    assert len(blob) < 200_000  # neither the 4000-row leaf record nor the sketch buffer
    u = pickle.loads(blob)
    assert not hasattr(u, "sketch") and getattr(u, "_fit_rows", None) is None
    assert torch.equal(u.predict(X), t.predict(X))
    assert str(u) == str(t)


def test_estimator_fixed_sketch(lb):
    """fixed_sketch=True: the first tree is the one the default driver builds, later trees reuse its
    bins; the model still fits."""
    rs = np.random.RandomState(4)
    X = dev(rs.normal(size=(30000, 20)).astype(np.float32))
    y = X[:, 0] * 2.0 - X[:, 3] + 0.1 * dev(rs.normal(size=30000)).to(torch.float32)
    base = (lb.Tree(max_depth=5, split_samples=64),)
    a = lb.LBRegressor(n_estimators=8, base_models=base, random_state=3).fit(X, y)
    b = lb.LBRegressor(n_estimators=8, base_models=base, random_state=3, fixed_sketch=True).fit(X, y)
    assert torch.equal(a.models_[0].feature, b.models_[0].feature)
    assert torch.equal(a.models_[0].leaf_value, b.models_[0].leaf_value)
    assert all(getattr(t, "sketch", None) is None for t in b.models_)
    err = lambda m: float(((m.predict(X).view(-1) - y.double()) ** 2).mean())
    assert err(b) < 0.5 * float(y.double().var()) and abs(err(b) - err(a)) < 0.2 * err(a) + 1e-3


def test_build_tree_level_batching(lb, oracle):
    """More bins than the 1 GB histogram rule holds on the deepest levels: levels are cut into
    batches and built without parents (reference: test_wide_deep, test_tree.py:218-227)."""
    case = (3000, 500, 1, 10, 256, np.float32, {})
    X, want, got = _run_tree_case(lb, oracle, case, seed=3)
    assert np.array_equal(got["feature"].cpu().numpy(), want.feature)
    assert np.array_equal(got["node_sums"].cpu().numpy(), want.node_sums)
    assert np.array_equal(got["leaf_value"].cpu().numpy(), want.leaf_value)


def test_golden_trees_on_gpu(lb, oracle):
    """The committed golden inputs: the GPU (quantised) tree must predict within 1e-4 of... itself
    via the oracle's Mode Q, and stay close to the reference CPU tree's training loss."""
    from legateboost_b200.tree import build_tree_arrays, predict_arrays

    for path in sorted(glob.glob(os.path.join(HERE, "golden", "tree_*.npz"))):
        z = np.load(path)
        kw = dict(max_depth=int(z["max_depth"]), split_samples=int(z["split_samples"]), seed=int(z["seed"]),
                  l1=float(z["l1"]), l2=float(z["l2"]), min_split_gain=float(z["min_split_gain"]))
        want = oracle.build_tree(z["X"], z["g"], z["h"], mode="Q", **kw)
        got = build_tree_arrays(dev(z["X"]), dev(z["g"]), dev(z["h"]), row_offset=0, dataset_rows=z["X"].shape[0], **kw)
        assert np.array_equal(got["feature"].cpu().numpy(), want.feature)
        assert np.array_equal(got["leaf_value"].cpu().numpy(), want.leaf_value)
        # predict of the reference CPU tree stored in the fixture, evaluated by the GPU kernel
        p = predict_arrays(dev(z["X"]), [(dev(z["leaf_value"]), dev(z["feature"]), dev(z["split_value"]))])
        assert np.array_equal(p.cpu().numpy(), z["pred"])


GOLDEN_Q = sorted(glob.glob(os.path.join(HERE, "golden", "treeq_*.npz")))
SAME_SCALE = {"batching", "deep", "mask", "reg", "rows20k", "softmax10"}


@pytest.mark.parametrize("path", GOLDEN_Q, ids=[os.path.basename(p)[6:-4] for p in GOLDEN_Q])
def test_reference_gpu_vectors_on_gpu(lb, path):
    """liblbk.so against what the reference's own GPU code produced for the same inputs
    (tests/golden/make_golden_q.py).  Bit for bit: bins, feature, split_value, quantised node sums,
    traced histograms, predictions.  The float outputs that pass through the quantiser's scale
    (a float sum whose order the reference leaves to thrust::reduce) or a contracted multiply-add:
    bit for bit equal to the reference built without contraction where the scale is the same
    float (SAME_SCALE), within 1e-12 relative everywhere."""
    import sys

    from legateboost_b200.tree import build_tree_arrays, predict_arrays

    sys.path.insert(0, os.path.join(HERE, "golden"))
    import make_golden_q as G

    z, c = G.load_case(path)
    name = os.path.basename(path)[6:-4]
    tn = int(z["trace_nodes"])
    fs = None if c["feature_set"] is None else torch.from_numpy(np.asarray(c["feature_set"]))
    got = build_tree_arrays(dev(c["X"]), dev(np.asarray(c["g"], dtype=np.float64)), dev(np.asarray(c["h"], dtype=np.float64)),
                            max_depth=c["max_depth"], split_samples=c["split_samples"], seed=c["seed"], l1=c["l1"],
                            l2=c["l2"], min_split_gain=c["min_split_gain"], feature_set=fs, row_offset=0,
                            dataset_rows=c["X"].shape[0], trace_nodes=tn)
    assert got["B"] == int(z["total_bins"])
    assert np.array_equal(got["feature"].cpu().numpy(), z["feature"])
    assert np.array_equal(got["split_value"].cpu().numpy().view(np.int64), z["split_value"].view(np.int64))
    assert np.array_equal(got["node_sums"].cpu().numpy(), z["node_sums"])
    trace = got["trace_hist"].cpu().numpy()
    assert np.array_equal(G.digest(trace), z["trace_digest"])
    assert np.array_equal(trace[:z["trace_hist"].shape[0]], z["trace_hist"])
    for k in ("hessian", "leaf_value", "gain"):
        a = got[k].cpu().numpy()
        assert np.all(np.abs(a - z[k]) <= 1e-12 * np.maximum(np.abs(a), np.abs(z[k]))), k
        if name in SAME_SCALE:
            assert np.array_equal(a.view(np.int64), z[k + "_nofma"].view(np.int64)), k
    pred = predict_arrays(dev(c["X"]), [(dev(z["leaf_value"]), dev(z["feature"]), dev(z["split_value"]))])
    assert np.array_equal(pred.cpu().numpy().view(np.int64), z["pred"].view(np.int64))


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("N,F,K,T,D", [(1000, 10, 1, 5, 4), (5000, 100, 1, 40, 8), (777, 33, 5, 7, 6), (129, 3, 2, 1, 0)])
def test_predict_bit_exact(lb, oracle, dtype, N, F, K, T, D):
    from legateboost_b200.tree import predict_arrays

    rs = np.random.RandomState(T)
    X = rs.random((N, F)).astype(dtype)
    M = 2 ** (D + 1) - 1
    trees = []
    for _ in range(T):
        feat = rs.randint(0, F, size=M).astype(np.int32)
        feat[2 ** D - 1:] = -1                      # last level are leaves
        feat[rs.random(M) < 0.15] = -1              # some early leaves
        split = rs.random(M)
        leaf = rs.normal(size=(M, K))
        trees.append((leaf, feat, split))
    want = oracle.predict(X, trees)
    got = predict_arrays(dev(X), [(dev(a), dev(b), dev(c)) for a, b, c in trees])
    assert np.array_equal(got.cpu().numpy(), want)


def test_predict_empty_and_batch_sum(lb, oracle):
    from legateboost_b200.tree import predict_arrays

    rs = np.random.RandomState(0)
    X = rs.random((500, 6)).astype(np.float32)
    mk = lambda: (dev(rs.normal(size=(3, 1))), dev(np.array([2, -1, -1], dtype=np.int32)), dev(rs.random(3)))
    a, b = mk(), mk()
    pa, pb = predict_arrays(dev(X), [a]), predict_arrays(dev(X), [b])
    assert torch.equal(predict_arrays(dev(X), [a, b]), pa + pb)
    assert predict_arrays(dev(X[:0]), [a]).shape == (0, 1)


# ---------------------------------------------------------------------------------------------
def test_tree_class_known_answers(lb):
    # reference: test_tree.py:11-21, 64-78, 160-184
    X = dev(np.array([[0.0], [1.0]]))
    g = dev(np.array([[0.0], [-1.0]]))
    h = dev(np.array([[1.0], [1.0]]))
    m = lb.Tree(max_depth=1, l2_regularization=0.0).set_random_state(np.random.RandomState(2)).fit(X, g, h)
    assert np.allclose(m.predict(X).cpu().numpy(), np.array([[0.0], [1.0]]))
    X0 = dev(np.array([[0.0], [0.0]]))
    y = np.array([500.0, 500.0])
    m = lb.Tree(max_depth=0, l2_regularization=10.0).set_random_state(np.random.RandomState(0))
    m.fit(X0, dev(-y[:, None]), dev(np.ones((2, 1))))
    assert np.isclose(m.predict(X0)[0, 0].item(), y.sum() / (y.size + 10.0))
    m = lb.Tree(max_depth=0, l2_regularization=0.0, l1_regularization=1.5).set_random_state(np.random.RandomState(0))
    m.fit(X0, dev(-y[:, None]), dev(np.ones((2, 1))))
    assert np.isclose(m.predict(X0)[0, 0].item(), (y.sum() - 1.5) / y.size)
    assert "leaf=" in str(m) and m == m and (m * 2.0).leaf_value[0, 0].item() == 2 * m.leaf_value[0, 0].item()


def test_tree_class_depth_and_invariants(lb):
    # reference: test_tree.py:24-45 and legateboost/testing/utils.py:22-50
    rs = np.random.RandomState(0)
    X = rs.random((10000, 100))
    for K in (1, 5):
        g = rs.normal(size=(X.shape[0], K))
        h = rs.random(g.shape) + 0.1
        y = -g / h
        metrics = []
        for depth in range(0, 10):
            m = lb.Tree(max_depth=depth).set_random_state(np.random.RandomState(2)).fit(dev(X), dev(g), dev(h))
            p = m.predict(dev(X)).cpu().numpy()
            metrics.append((((p - y) ** 2 * h).sum(axis=0) / h.sum(axis=0)).mean())
            feat, hess, gain = m.feature.cpu().numpy(), m.hessian.cpu().numpy(), m.gain.cpu().numpy()
            split = feat != -1
            assert np.all(hess[split] > 0.0) and np.all(gain[split] > 0.0)
            leaves = (feat == -1) & (hess[:, 0] > 0.0)
            assert np.isclose(hess[leaves].sum(axis=0), hess[0]).all()
        assert all(a - b > -1e-3 for a, b in zip(metrics, metrics[1:])) and metrics[-1] < metrics[0]


def test_max_depth_20_two_rows(lb):
    # reference: test_tree.py:48-61
    X = dev(np.random.RandomState(0).random((2, 1)))
    m = lb.LBRegressor(init=None, base_models=(lb.Tree(max_depth=20),), learning_rate=1.0, n_estimators=1,
                       random_state=0)
    m.fit(X, dev(np.array([500.0, 500.0])))
    assert m[0].feature.shape[0] == 2 ** 21 - 1


def test_estimators_config1_reduced(lb, oracle):
    """Configuration 1 at reduced size: squared error, depth 6, lr 0.1; loss falls every round and
    every tree equals the oracle's tree for the same gradients and seed."""
    rng = np.random.default_rng(0)
    X = rng.random((20000, 50), dtype=np.float32)
    y = (np.sin(6 * X[:, :5]).sum(axis=1) + rng.normal(0, 0.1, size=20000)).astype(np.float32)
    m = lb.LBRegressor(n_estimators=5, learning_rate=0.1, base_models=(lb.Tree(max_depth=6, split_samples=256),),
                       random_state=0, verbose=1)
    m.fit(dev(X), dev(y))
    assert all(a > b for a, b in zip(m.train_metric_, m.train_metric_[1:]))
    # replay round 0 with the oracle
    rs = np.random.RandomState(0)
    seed = rs.randint(0, 2 ** 31)
    y64 = y.astype(np.float64)[:, None]
    g = (np.full_like(y64, y64.mean()) - y64) * 0.1
    want = oracle.build_tree(X, g, np.ones_like(g), max_depth=6, split_samples=256, seed=seed, mode="Q")
    assert np.array_equal(m[0].feature.cpu().numpy(), want.feature)
    assert np.allclose(m[0].leaf_value.cpu().numpy(), want.leaf_value, rtol=1e-9, atol=1e-12)


def test_classifier_multiclass(lb):
    rng = np.random.default_rng(2)
    X = rng.normal(size=(5000, 20)).astype(np.float32)
    W = rng.normal(size=(10, 4))
    y = np.argmax(X[:, :10] @ W + rng.normal(0, 0.5, size=(5000, 4)), axis=1)
    m = lb.LBClassifier(n_estimators=5, base_models=(lb.Tree(max_depth=4),), random_state=1, verbose=1)
    m.fit(dev(X), dev(y))
    assert all(a > b for a, b in zip(m.train_metric_, m.train_metric_[1:]))
    proba = m.predict_proba(dev(X))
    assert torch.allclose(proba.sum(dim=1), torch.ones(5000, dtype=torch.float64, device="cuda"))
    assert (m.predict(dev(X)).cpu().numpy() == y).mean() > 0.5


def test_bad_arguments_are_errors(lb):
    from legateboost_b200.tree import build_tree_arrays

    X = dev(np.zeros((10, 3), dtype=np.float32))
    g = dev(np.zeros((10, 1)))
    with pytest.raises(lb.library.LbkError):
        build_tree_arrays(X, g, g, max_depth=2, split_samples=5000, seed=0, row_offset=0, dataset_rows=10)
    with pytest.raises(lb.library.LbkError):
        build_tree_arrays(X, g, g, max_depth=2, split_samples=16, seed=0, row_offset=5, dataset_rows=10)


def test_first_predict_on_the_training_matrix_uses_the_leaf_record(lb):
    """fit() keeps the node every training row ended in; the first predict() on the same, unmodified
    tensor gathers leaf values from it.  It must equal the walk over X bit for bit, must be used
    once, and must not be used after the tensor changed."""
    rs = np.random.RandomState(3)
    for dtype, K, F, S in ((np.float32, 1, 40, 256), (np.float64, 3, 7, 500)):
        X = dev(rs.random((3000, F)).astype(dtype))
        g = dev(rs.normal(size=(3000, K)))
        h = dev(rs.random((3000, K)) + 0.1)
        t = lb.Tree(max_depth=6, split_samples=S).set_random_state(np.random.RandomState(1)).fit(X, g, h)
        assert t._fit_rows is not None
        want = lb.Tree.batch_predict([t], X)
        got = t.predict(X)
        assert t._fit_rows is None
        assert torch.equal(got, want)
        assert torch.equal(t.predict(X), want)           # the walk over X this time
        t.fit(X, g, h)
        X[0, 0] += 1.0                                   # in-place change: the record is stale
        want = lb.Tree.batch_predict([t], X)
        assert torch.equal(t.predict(X), want)
    stump = lb.Tree(max_depth=0).set_random_state(np.random.RandomState(1)).fit(X, g, h)
    assert torch.equal(stump.predict(X), lb.Tree.batch_predict([stump], X))


def _torch_histogram(bins, gpair, node, node_begin, n_nodes, F, n_bins):
    """An independent integer histogram on the device: index_add_ of the pairs at
    node * B + feature * n_bins + bin, a few features at a time (int64, exact)."""
    B = F * n_bins
    out = torch.zeros((n_nodes * B, 2), dtype=torch.int64, device=bins.device)
    base = (node.long() - node_begin) * B
    vals = gpair[:, 0, :].long()
    step = 8
    for f0 in range(0, F, step):
        f1 = min(F, f0 + step)
        idx = base[:, None] + bins[:, f0:f1].long() + (torch.arange(f0, f1, device=bins.device) * n_bins)[None, :]
        out.index_add_(0, idx.reshape(-1), vals[:, None, :].expand(-1, f1 - f0, -1).reshape(-1, 2))
    return out.view(n_nodes, 1, B, 2)


def test_full_size_histogram_exact(lb):
    """The benchmark's own size (10 M x 128, 128 nodes of level 7): every bin of every node equals an
    independent histogram of the same inputs (integer arithmetic: exact)."""
    import bench
    from legateboost_b200 import stages

    n = 10_000_000
    bins, row_ptr, gpair, _, row_index, seg, node, max_abs = bench.hist_inputs(torch, n, 7, torch.device("cuda"))
    hist = stages.histogram(bins, row_ptr, gpair, row_index, seg, bench.HIST_FEATURES, mode=0, max_abs=max_abs)
    n_nodes = seg.shape[0] - 1
    want = _torch_histogram(bins, gpair, node, n_nodes - 1, n_nodes, bench.HIST_FEATURES, bench.HIST_BINS)
    assert torch.equal(hist, want)
    # the same call without the magnitudes handed in (the library finds them) gives the same bits
    assert torch.equal(stages.histogram(bins, row_ptr, gpair, row_index, seg, bench.HIST_FEATURES, mode=0), hist)


@pytest.mark.parametrize("N,F,K,weights,mode,qmax", [
    (1_500_000, 64, 1, [0.80, 0.0, 0.15, 0.05], 0, 300),    # one node in about 120 pieces: a deep merge tree
    (1_500_000, 64, 1, [0.80, 0.0, 0.15, 0.05], 0, 5000),   # ... too many rows for 32-bit sums: the tree is climbed
                                                            # two levels, the rest are 64-bit atomics
    (1_500_000, 64, 1, [0.80, 0.0, 0.15, 0.05], 0, 40000),  # ... one level only
    (1_500_000, 64, 1, [0.80, 0.0, 0.15, 0.05], 0, 400000), # ... a single piece is already too long: no tree
    (1_500_000, 96, 3, [0.3, 0.3, 0.2, 0.1, 0.1], 0, 300),  # three groups: the second group set is half empty
    (2_000_000, 32, 2, [1.0] * 37, 0, 300),                 # one group per unit (two blocks per SM)
    (1_500_000, 128, 1, [0.55, 0.45], 1, 0),                # float pairs through the same ranges
])
def test_histogram_static_ranges(lb, oracle, N, F, K, weights, mode, qmax):
    """Enough rows for the planner to hand out equal static ranges: nodes reach over range
    boundaries and their pieces meet in the merge tree; sums stay exact (floats within 1e-5)."""
    from legateboost_b200 import stages

    rng = np.random.default_rng(N + F)
    n_nodes = len(weights)
    edges = np.cumsum(np.asarray(weights) / np.sum(weights))
    node = np.minimum(np.searchsorted(edges, rng.random(N), side="right"), n_nodes - 1).astype(np.int32) + (n_nodes - 1)
    bins = rng.integers(0, 256, size=(N, F), dtype=np.uint8)
    row_ptr = (np.arange(F + 1) * 256).astype(np.int32)
    row_index, seg = stages.group_rows(dev(node), n_nodes - 1, n_nodes)
    if mode == 0:
        q = rng.integers(-qmax, qmax, size=(N, K, 2), dtype=np.int32)
        q[:, :, 1] = np.abs(q[:, :, 1])
        want = oracle.histogram_q(bins, row_ptr, q, node, n_nodes - 1, 2 * n_nodes - 1)
        got = stages.histogram(stages.to_padded_rows(dev(bins)), dev(row_ptr), dev(q), row_index, seg, F, mode=0)
        assert np.array_equal(got.cpu().numpy(), want)
        got = stages.histogram(stages.to_padded_rows(dev(bins)), dev(row_ptr), _by_position(dev(q), row_index), row_index,
                               seg, F, mode=0, pairs_by_position=True, max_abs=_max_abs(q))
        assert np.array_equal(got.cpu().numpy(), want)
    else:
        gh = np.stack([rng.normal(size=(N, K)), np.ones((N, K))], axis=2).astype(np.float32)
        want = oracle.histogram_d(bins, row_ptr, gh[:, :, 0].copy(), gh[:, :, 1].copy(), node, n_nodes - 1, 2 * n_nodes - 1)
        for by_pos in (False, True):
            pairs = _by_position(dev(gh), row_index) if by_pos else dev(gh)
            got = stages.histogram(stages.to_padded_rows(dev(bins)), dev(row_ptr), pairs, row_index, seg, F, mode=1,
                                   pairs_by_position=by_pos)
            err = np.abs(got.cpu().numpy() - want).max()
            assert err <= 1e-5 * np.abs(want).max()


def test_full_size_tree_properties(lb):
    """10 M x 64 rows, depth 8: the node of every training row from the builder equals the walk over
    X; the hessians of the children add up to the parent's (h = 1: the root holds the row count)."""
    n, F = 10_000_000, 64
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    X = torch.rand((n, F), dtype=torch.float32, device="cuda", generator=gen)
    g = torch.randn((n, 1), dtype=torch.float64, device="cuda", generator=gen)
    h = torch.ones((n, 1), dtype=torch.float64, device="cuda")
    t = lb.Tree(max_depth=8).set_random_state(np.random.RandomState(2)).fit(X, g, h)
    walk = lb.Tree.batch_predict([t], X)
    assert torch.equal(t.predict(X), walk)
    feature = t.feature.cpu().numpy()
    hess = t.hessian.cpu().numpy()[:, 0]
    assert abs(hess[0] - n) <= 1e-6 * n
    split = np.nonzero(feature >= 0)[0]
    assert len(split) > 100
    assert np.allclose(hess[2 * split + 1] + hess[2 * split + 2], hess[split], rtol=1e-12, atol=0)


@pytest.mark.parametrize("dtype,K,D,l1,l2", [(np.float32, 1, 6, 0.0, 1.0), (np.float64, 3, 5, 0.3, 0.5),
                                               (np.float32, 12, 8, 0.0, 1.0)])
def test_update_tree_matches_oracle(lb, oracle, dtype, K, D, l1, l2):
    """Tree.update (UPDATE_TREE): new leaf values and hessians for an unchanged structure.  Float64
    sums in another order than the reference's row loop: 1e-10 relative, hessians included; nodes
    no row reaches get 0."""
    rs = np.random.RandomState(17)
    N, F = 20000, 15
    X = rs.random((N, F)).astype(dtype)
    g = rs.normal(size=(N, K))
    h = rs.random((N, K)) + 0.1
    t = lb.Tree(max_depth=D, split_samples=64, l1_regularization=l1, l2_regularization=l2)
    t.set_random_state(np.random.RandomState(4)).fit(dev(X), dev(g), dev(h))
    feature, split = t.feature.cpu().numpy(), t.split_value.cpu().numpy()
    old_leaf = t.leaf_value.clone()
    g2 = rs.normal(size=(N, K))
    h2 = (rs.random((N, K)) + 0.05) * (rs.random((N, K)) > 0.2)   # some zero hessians
    sub = slice(0, N // 3)                                         # fewer rows: some nodes stay empty
    want_leaf, want_hess = oracle.update_tree(X[sub], g2[sub], h2[sub], feature, split, l1=l1, l2=l2)
    t.update(dev(X[sub]), dev(g2[sub]), dev(h2[sub]))
    assert torch.equal(t.feature.cpu(), torch.from_numpy(feature))
    got_leaf, got_hess = t.leaf_value.cpu().numpy(), t.hessian.cpu().numpy()
    assert np.allclose(got_hess, want_hess, rtol=1e-10, atol=1e-12)
    assert np.allclose(got_leaf, want_leaf, rtol=1e-9, atol=1e-12)
    assert not np.array_equal(got_leaf, old_leaf.cpu().numpy())
    assert np.array_equal(got_leaf == 0.0, want_leaf == 0.0)
    # the updated tree predicts with the new values
    pred = t.predict(dev(X[:100]))
    assert np.allclose(pred.cpu().numpy(), oracle.predict(X[:100], [(got_leaf, feature, split)]), rtol=0, atol=0)
    # an empty shard keeps every node at zero
    t.update(dev(X[:0]), dev(g2[:0]), dev(h2[:0]))
    assert not t.leaf_value.any() and not t.hessian.any()


def test_weighted_gradient_kernels_match_the_array_formulas(lb):
    """lbk_gradient against the reference's chain of array operations (objectives.py:131-135, 489-512,
    legateboost.py:189-224), evaluated with numpy: squared error bit for bit, log loss within the last
    bits of exp / division."""
    from legateboost_b200 import estimator as E

    rs = np.random.RandomState(8)
    N = 5000
    est = lb.LBRegressor(learning_rate=0.3)
    est._obj = E._SquaredError()
    raw, y = rs.normal(size=(N, 3)), rs.normal(size=(N, 3))
    g, h = est._weighted_gradient(dev(y), dev(raw))
    assert np.array_equal(g.cpu().numpy(), (raw - y) * 0.3) and np.array_equal(h.cpu().numpy(), np.ones((N, 3)))
    est._obj = E._LogLoss()
    raw, y = rs.normal(size=(N, 1)) * 4, rs.randint(0, 2, size=(N, 1)).astype(np.float64)
    g, h = est._weighted_gradient(dev(y), dev(raw))
    p = 1.0 / (1.0 + np.exp(-raw))
    assert np.allclose(g.cpu().numpy(), (p - y) * 0.3, rtol=1e-13, atol=1e-16)
    assert np.allclose(h.cpu().numpy(), np.maximum(p * (1 - p), 1e-8), rtol=1e-13)
    for K in (3, 10, 40):
        raw, y = rs.normal(size=(N, K)) * 5, rs.randint(0, K, size=(N, 1)).astype(np.float64)
        raw[0] = 800.0 * np.arange(K)  # far apart: hessians hit the floor
        g, h = est._weighted_gradient(dev(y), dev(raw))
        e = np.exp(raw - raw.max(axis=1, keepdims=True))
        p = e / e.sum(axis=1, keepdims=True)
        want_g = p.copy()
        want_g[np.arange(N), y[:, 0].astype(int)] -= 1.0
        assert np.allclose(g.cpu().numpy(), want_g * 0.3, rtol=1e-12, atol=1e-15)
        assert np.allclose(h.cpu().numpy(), np.maximum(p * (1 - p), 1e-8), rtol=1e-12)
        assert h.min().item() == 1e-8

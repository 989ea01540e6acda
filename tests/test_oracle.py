"""CPU tests of the oracle: the reference's known answers and invariants
(legateboost/test/models/test_tree.py, legateboost/testing/utils.py), the RNG restatement against
the toolkit's thrust headers, the restatement against the stub-compiled reference sources when
that build is present, and against the committed golden vectors."""
import glob
import os
import subprocess

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def tree_tuple(t):
    return (t.leaf_value, t.feature, t.split_value)


@pytest.mark.parametrize("mode", ["Q", "D"])
def test_basic_known_answer(oracle, mode):
    # reference: test_tree.py:11-21
    X = np.array([[0.0], [1.0]])
    g = np.array([[0.0], [-1.0]])
    h = np.array([[1.0], [1.0]])
    t = oracle.build_tree(X, g, h, max_depth=1, l2=0.0, seed=1872583848, mode=mode)
    assert np.allclose(oracle.predict(X, [tree_tuple(t)]), np.array([[0.0], [1.0]]))


@pytest.mark.parametrize("mode", ["Q", "D"])
def test_l2_known_answer(oracle, mode):
    # reference: test_tree.py:64-78 (init=None, lr=1: g = pred - y = -y, h = 1)
    X = np.array([[0.0], [0.0]])
    y = np.array([500.0, 500.0])
    l2 = 10.0
    t = oracle.build_tree(X, -y[:, None], np.ones((2, 1)), max_depth=0, l2=l2, seed=5, mode=mode)
    assert np.isclose(oracle.predict(X, [tree_tuple(t)])[0, 0], y.sum() / (y.size + l2))


@pytest.mark.parametrize("mode", ["Q", "D"])
def test_l1_known_answer(oracle, mode):
    # reference: test_tree.py:160-184
    X = np.array([[0.0], [0.0]])
    y = np.array([500.0, 500.0])
    l1 = 1.5
    t = oracle.build_tree(X, -y[:, None], np.ones((2, 1)), max_depth=0, l1=l1, l2=0.0, seed=5, mode=mode)
    assert np.isclose(oracle.predict(X, [tree_tuple(t)])[0, 0], (y.sum() - l1) / y.size)
    y = np.array([0.5, 0.5])
    t = oracle.build_tree(X, -y[:, None], np.ones((2, 1)), max_depth=0, l1=l1, l2=0.0, seed=5, mode=mode)
    assert np.isclose(oracle.predict(X, [tree_tuple(t)])[0, 0], 0.0)


@pytest.mark.parametrize("mode", ["Q", "D"])
def test_min_split_gain(oracle, mode):
    # reference: test_tree.py:187-215
    rng = np.random.RandomState(0)
    X = rng.random((100, 1))
    y = rng.random(100)
    a = oracle.build_tree(X, -y[:, None], np.ones((100, 1)), max_depth=12, min_split_gain=0.0, seed=3, mode=mode)
    b = oracle.build_tree(X, -y[:, None], np.ones((100, 1)), max_depth=12, min_split_gain=0.03, seed=3, mode=mode)
    assert (b.hessian > 0).sum() < (a.hessian > 0).sum()
    assert np.isclose(a.gain[0], b.gain[0] + 0.03)


def sanity_check(t):
    # reference: legateboost/testing/utils.py:22-50
    split = t.feature != -1
    assert np.all(t.hessian[split] > 0.0)
    assert np.all(t.gain[split] > 0.0)
    leaves = (t.feature == -1) & (t.hessian[:, 0] > 0.0)
    assert np.isclose(t.hessian[leaves].sum(axis=0), t.hessian[0]).all()


@pytest.mark.parametrize("mode", ["Q", "D"])
@pytest.mark.parametrize("K", [1, 5])
def test_improving_with_depth(oracle, mode, K):
    # reference: test_tree.py:24-45 (smaller)
    rs = np.random.RandomState(0)
    X = rs.random((2000, 20))
    g = rs.normal(size=(2000, K))
    h = rs.random(g.shape) + 0.1
    y = -g / h
    metrics = []
    for depth in range(0, 8):
        t = oracle.build_tree(X, g, h, max_depth=depth, seed=1872583848, mode=mode)
        sanity_check(t)
        p = oracle.predict(X, [tree_tuple(t)])
        metrics.append((((p - y) ** 2 * h).sum(axis=0) / h.sum(axis=0)).mean())
    assert all(a - b > -1e-3 for a, b in zip(metrics, metrics[1:]))
    assert metrics[-1] < metrics[0]


def test_batch_predict_is_sum(oracle):
    # reference: test_model.py:8-21
    rs = np.random.RandomState(0)
    X = rs.random((1000, 10))
    g = rs.normal(size=(1000, 5))
    h = rs.random(g.shape) + 0.1
    a = oracle.build_tree(X, g, h, max_depth=8, seed=1, mode="Q")
    b = oracle.build_tree(X, rs.normal(size=(1000, 5)), h, max_depth=8, seed=1, mode="Q")
    both = oracle.predict(X, [tree_tuple(a), tree_tuple(b)])
    assert np.allclose(both, oracle.predict(X, [tree_tuple(a)]) + oracle.predict(X, [tree_tuple(b)]))


def test_deep_tree_two_rows(oracle):
    # reference: test_tree.py:48-61
    X = np.random.RandomState(0).random((2, 1))
    t = oracle.build_tree(X, -np.array([[500.0], [500.0]]), np.ones((2, 1)), max_depth=16, seed=9, mode="Q")
    assert t.feature.shape[0] == 2 ** 17 - 1


def test_feature_set(oracle):
    rs = np.random.RandomState(0)
    X = rs.random((500, 10))
    g = rs.normal(size=(500, 1))
    h = np.ones((500, 1))
    mask = np.zeros(10, dtype=bool)
    mask[1] = True
    for mode in "QD":
        t = oracle.build_tree(X, g, h, max_depth=5, seed=4, feature_set=mask, mode=mode)
        used = t.feature[t.feature >= 0]
        assert used.size > 0 and np.all(used == 1)


def test_rank_simulation_changes_only_scale(oracle):
    # integer histograms do not depend on how rows are split; the scale does (max of local sums)
    rs = np.random.RandomState(1)
    X = rs.random((3000, 8)).astype(np.float32)
    g = rs.normal(size=(3000, 1))
    h = np.ones((3000, 1))
    a = oracle.build_tree(X, g, h, max_depth=4, seed=11, mode="Q", n_ranks=1)
    b = oracle.build_tree(X, g, h, max_depth=4, seed=11, mode="Q", n_ranks=4)
    assert a.B == b.B and np.array_equal(a.proposals, b.proposals)
    assert b.scale[0] > a.scale[0]
    sanity_check(b)


def test_rng_matches_thrust(oracle):
    exe = os.path.join(ROOT, "oracle", "check_rng")
    if not os.path.exists(exe):
        pytest.skip("check_rng not built (needs the CUDA toolkit headers)")
    assert subprocess.run([exe], capture_output=True).returncode == 0


def test_abs_sum_order(oracle):
    rs = np.random.RandomState(3)
    for n in [1, 31, 4096, 4097, 100000]:
        v = rs.normal(size=n) * 10.0 ** rs.randint(-3, 3, size=n)
        s = oracle.abs_sum(v)
        assert np.isclose(s, np.abs(v).sum(), rtol=1e-12)
    # order sensitivity: the canonical sum is a fixed function of the sequence
    v = rs.normal(size=10000)
    assert oracle.abs_sum(v) == oracle.abs_sum(v.copy())


@pytest.mark.parametrize("case", range(4))
def test_mode_d_matches_reference_build(oracle, case):
    """Bit-for-bit against the reference's own build_tree.cc / predict.cc (stub-compiled)."""
    if oracle.ref_lib() is None:
        pytest.skip("oracle/_ref/libref_cpu.so not built here")
    rs = np.random.RandomState(case)
    N, F, K, D, S, dt = [(1000, 10, 1, 4, 64, np.float32), (3000, 20, 3, 6, 256, np.float64),
                         (300, 5, 2, 8, 16, np.float32), (4000, 40, 5, 5, 128, np.float64)][case]
    X = rs.random((N, F)).astype(dt)
    g = rs.normal(size=(N, K))
    h = rs.random((N, K)) + 0.1
    a = oracle.build_tree(X, g, h, max_depth=D, split_samples=S, seed=77 + case, mode="D")
    b = oracle.build_tree(X, g, h, max_depth=D, split_samples=S, seed=77 + case, mode="D", use_reference=True)
    for f in ["leaf_value", "feature", "split_value", "gain", "hessian"]:
        assert np.array_equal(getattr(a, f), getattr(b, f)), f


def test_update_tree_matches_reference_build(oracle):
    """Bit-for-bit against the reference's own update_tree.cc (stub-compiled); two simulated ranks
    agree with one within rounding."""
    if oracle.ref_update_lib() is None:
        pytest.skip("oracle/_ref/libref_update.so not built here")
    rs = np.random.RandomState(5)
    for dt, K in ((np.float32, 1), (np.float64, 4)):
        X = rs.random((2500, 12)).astype(dt)
        g = rs.normal(size=(2500, K))
        h = rs.random((2500, K)) + 0.1
        t = oracle.build_tree(X, g, h, max_depth=6, split_samples=64, seed=9, mode="D")
        g2 = rs.normal(size=(2500, K))
        h2 = rs.random((2500, K)) * (rs.random((2500, K)) > 0.3)  # some zero hessians
        a = oracle.update_tree(X, g2, h2, t.feature, t.split_value, l1=0.2, l2=0.7)
        b = oracle.update_tree(X, g2, h2, t.feature, t.split_value, l1=0.2, l2=0.7, use_reference=True)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
        c = oracle.update_tree(X, g2, h2, t.feature, t.split_value, l1=0.2, l2=0.7, n_ranks=2)
        assert np.allclose(c[0], a[0], rtol=1e-10, atol=1e-12) and np.allclose(c[1], a[1], rtol=1e-12)


def test_golden_vectors(oracle):
    """Committed outputs of the reference CPU build (tests/golden/make_golden.py)."""
    files = sorted(glob.glob(os.path.join(HERE, "golden", "tree_*.npz")))
    assert files, "golden fixtures missing"
    for path in files:
        z = np.load(path)
        t = oracle.build_tree(z["X"], z["g"], z["h"], max_depth=int(z["max_depth"]),
                              split_samples=int(z["split_samples"]), seed=int(z["seed"]),
                              l1=float(z["l1"]), l2=float(z["l2"]), min_split_gain=float(z["min_split_gain"]),
                              mode="D")
        for f in ["leaf_value", "feature", "split_value", "gain", "hessian"]:
            assert np.array_equal(getattr(t, f), z[f]), (path, f)
        p = oracle.predict(z["X"], [tree_tuple(t)])
        assert np.array_equal(p, z["pred"]), path
        # UPDATE_TREE with new gradients: same row order, same sums, bit for bit
        leaf, hess = oracle.update_tree(z["X"], z["g2"], z["h2"], t.feature, t.split_value, l1=float(z["l1"]),
                                        l2=float(z["l2"]))
        assert np.array_equal(leaf, z["upd_leaf_value"]), path
        assert np.array_equal(hess, z["upd_hessian"]), path


# ---------------------------------------------------------------------------------------------
# The quantised mode against vectors made by the reference's own GPU code (its unmodified
# build_tree.cu / predict.cu compiled with nvcc against the runtime stand-in and run on a B200:
# tests/golden/make_golden_q.py).
#
# What is bit for bit: the number of bins, feature[], split_value[], the quantised node sums, every
# traced node's histogram as the split search read it (scan write-skip rule, sibling subtraction,
# cache / batching rule) and the predictions.  What is not: the three float outputs that pass
# through the quantiser's scale or a contracted multiply-add.  The scale comes from a float sum
# over all rows whose order the reference leaves to thrust::reduce; where that order gives the
# same float as the oracle's fixed order (SAME_SCALE below) the float outputs are bit for bit equal
# to a build of the reference without multiply-add contraction (stored as *_nofma), elsewhere they
# differ by a few units in the last place.  The bound asserted for all of them is 1e-12 relative.
import sys  # noqa: E402

GOLDEN_Q = sorted(glob.glob(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "treeq_*.npz")))
SAME_SCALE = {"batching", "deep", "mask", "reg", "rows20k", "softmax10"}
FLOAT_RTOL = 1e-12


def _close(a, b):
    return np.all(np.abs(a - b) <= FLOAT_RTOL * np.maximum(np.abs(a), np.abs(b)))


@pytest.mark.parametrize("path", GOLDEN_Q, ids=[os.path.basename(p)[6:-4] for p in GOLDEN_Q])
def test_mode_q_matches_the_reference_gpu_vectors(oracle, path):
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    import make_golden_q as G

    z, c = G.load_case(path)
    name = os.path.basename(path)[6:-4]
    tn = int(z["trace_nodes"])
    t = oracle.build_tree(c["X"], c["g"], c["h"], max_depth=c["max_depth"], split_samples=c["split_samples"],
                          seed=c["seed"], l1=c["l1"], l2=c["l2"], min_split_gain=c["min_split_gain"],
                          feature_set=c["feature_set"], mode="Q", trace_nodes=tn)
    assert t.B == int(z["total_bins"])
    assert np.array_equal(t.feature, z["feature"])
    assert np.array_equal(t.split_value.view(np.int64), z["split_value"].view(np.int64))
    assert np.array_equal(t.node_sums, z["node_sums"])
    assert np.array_equal(G.digest(t.trace_hist), z["trace_digest"])
    stored = z["trace_hist"].shape[0]
    assert np.array_equal(t.trace_hist[:stored], z["trace_hist"])
    for k in ("hessian", "leaf_value", "gain"):
        assert _close(getattr(t, k), z[k]), k
        if name in SAME_SCALE:
            assert np.array_equal(getattr(t, k).view(np.int64), z[k + "_nofma"].view(np.int64)), k
        else:
            assert _close(getattr(t, k), z[k + "_nofma"]), k
    # the reference's GPU predict of its own tree
    pred = oracle.predict(c["X"], [(z["leaf_value"], z["feature"], z["split_value"])])
    assert np.array_equal(pred.view(np.int64), z["pred"].view(np.int64))


def test_golden_q_vectors_are_present():
    assert len(GOLDEN_Q) >= 10

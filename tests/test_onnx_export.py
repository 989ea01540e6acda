"""ONNX export of a tree: the attributes of the ``ai.onnx.ml.TreeEnsemble`` nodes.

There is no onnx package in the build image, so what is checked here is the part that does not
need it: the arrays handed to the operator, run through a small interpreter of the operator's
published semantics (BRANCH_LEQ nodes, SUM aggregation, child ids that are leaf ids where the
``*leafs`` flag says so), must predict what the oracle's tree walk predicts.  Model assembly
(`Tree.to_onnx`) is exercised only where onnx can be imported."""
import numpy as np
import pytest

from legateboost_b200.tree import onnx_tree_ensemble_attributes


def _run_tree_ensemble(a, X):
    out = np.zeros((X.shape[0], a["n_targets"]))
    for r in range(X.shape[0]):
        for root in a["tree_roots"]:
            i = root
            while True:
                assert a["nodes_modes"][i] == 0
                if X[r, a["nodes_featureids"][i]] <= a["nodes_splits"][i]:
                    nxt, leaf = a["nodes_truenodeids"][i], a["nodes_trueleafs"][i]
                else:
                    nxt, leaf = a["nodes_falsenodeids"][i], a["nodes_falseleafs"][i]
                if leaf:
                    out[r, a["leaf_targetids"][nxt]] += a["leaf_weights"][nxt]
                    break
                i = nxt
    return out


def _random_tree(rs, depth, F, K, p_leaf):
    M = 2 ** (depth + 1) - 1
    feature = np.full(M, -1, dtype=np.int32)
    split = np.zeros(M)
    leaf = rs.normal(size=(M, K))

    def grow(i, d):
        if d == depth or rs.random() < p_leaf:
            return
        feature[i] = rs.randint(F)
        split[i] = rs.normal()
        grow(2 * i + 1, d + 1)
        grow(2 * i + 2, d + 1)

    grow(0, 0)
    return leaf, feature, split


@pytest.mark.parametrize("depth,F,K,p_leaf,seed", [(4, 5, 1, 0.2, 0), (6, 3, 3, 0.3, 1), (0, 2, 2, 0.0, 2), (3, 4, 1, 1.0, 3)])
def test_attributes_predict_like_the_tree_walk(depth, F, K, p_leaf, seed):
    from oracle import oracle as O

    rs = np.random.RandomState(seed)
    leaf, feature, split = _random_tree(rs, depth, F, K, p_leaf)
    X = rs.normal(size=(200, F))
    want = O.predict(X, [(leaf, feature, split)])
    attrs = onnx_tree_ensemble_attributes(feature, split, leaf)
    assert len(attrs) == K
    got = sum(_run_tree_ensemble(a, X) for a in attrs)
    assert np.array_equal(got, want)
    for a in attrs:
        M = feature.shape[0]
        assert all(len(a[n]) == M for n in ("nodes_featureids", "nodes_splits", "nodes_truenodeids", "leaf_weights"))
        assert a["nodes_featureids"].min() >= 0


def test_to_onnx_with_or_without_the_package():
    import torch

    from legateboost_b200.tree import Tree

    rs = np.random.RandomState(5)
    leaf, feature, split = _random_tree(rs, 3, 4, 2, 0.2)
    t = Tree.__new__(Tree)
    t.leaf_value, t.feature, t.split_value = torch.from_numpy(leaf), torch.from_numpy(feature), torch.from_numpy(split)
    try:
        import onnx  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="onnx"):
            t.to_onnx()
        return
    model = t.to_onnx()  # runs onnx.checker.check_model itself
    assert [n.op_type for n in model.graph.node] == ["TreeEnsemble", "Identity", "TreeEnsemble", "Add"]

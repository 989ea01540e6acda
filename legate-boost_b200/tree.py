"""``Tree``: the host-side mirror of ``legateboost.models.Tree`` over torch CUDA tensors.

Same constructor arguments, ``set_random_state``, ``fit(X, g, h)``, ``predict``, ``batch_predict``,
``__str__``, ``__mul__`` and error behaviour as the reference's Python launcher
(legateboost/models/tree.py:22-317, legateboost/models/base_model.py:11-138); where that one
builds legate tasks BUILD_TREE / PREDICT, this one fills the argument structs of ``lbk_build_tree``
/ ``lbk_predict`` (include/lbk.h).  With ``torch.distributed`` initialised (one rank per GPU) every
rank passes its own contiguous block of rows and all ranks get the same tree.
"""
import copy
import ctypes as C
import warnings
from typing import Any, Callable, List, Sequence, Union

import numpy as np
import torch

from . import library as L


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return L.LBK_F32
    if t.dtype == torch.float64:
        return L.LBK_F64
    raise ValueError("X must be float32 or float64")


def _stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _row_layout(n_local: int):
    """(row_offset, dataset_rows) of this rank's block under torch.distributed."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return 0, n_local
    sizes = [None] * dist.get_world_size()
    dist.all_gather_object(sizes, int(n_local))
    return int(sum(sizes[: dist.get_rank()])), int(sum(sizes))


def _tensor_key(t: torch.Tensor):
    """Identity of a tensor's contents as far as torch can tell: storage, view and version counter
    (every in-place change bumps the counter)."""
    return (t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.dtype, t.device, t._version)


class Sketch:
    """Split proposals and binned matrix of one training matrix, kept in a device buffer so that
    later trees on the same matrix skip the sampling and the binning (``lbk_build_tree_args.sketch``).
    An extension: the reference samples and bins again for every tree (models/tree.py:125), so trees
    built from a reused sketch differ from the reference's.  The first fit on a matrix saves, fits
    on the same unmodified tensor with the same ``split_samples`` reuse."""

    def __init__(self) -> None:
        self.buffer = None
        self.key = None

    def mode_for(self, X, split_samples, ctx) -> int:
        need = int(ctx.lib.lbk_sketch_bytes(X.shape[0], X.shape[1], split_samples, _dtype_code(X)))
        key = (_tensor_key(X), split_samples)
        if self.buffer is not None and self.key == key and self.buffer.numel() >= need:
            return L.SKETCH_REUSE
        if self.buffer is None or self.buffer.numel() < need or self.buffer.device != X.device:
            self.buffer = torch.empty((need,), dtype=torch.uint8, device=X.device)
        self.key = None  # set by the caller once the saving call has succeeded
        return L.SKETCH_SAVE


def build_tree_arrays(X, g, h, *, max_depth, split_samples, seed, l1=0.0, l2=1.0, min_split_gain=0.0,
                      feature_set=None, row_offset=None, dataset_rows=None, trace_nodes=0, ctx=None,
                      want_leaf=False, sketch=None):
    """Run ``lbk_build_tree`` on device tensors.  Returns a dict with the five tree arrays (and the
    optional traces; with ``want_leaf`` also ``leaf``: the node every local row ends in).  With a
    ``Sketch`` the proposals and bins are saved in it or, if it holds those of this matrix, reused."""
    assert X.is_cuda and g.is_cuda and h.is_cuda, "inputs must be CUDA tensors (no CPU fallback)"
    if g.dim() == 1:
        g, h = g[:, None], h[:, None]
    assert g.dtype == torch.float64 and h.dtype == torch.float64
    if X.stride(1) != 1 and X.shape[0] > 0:
        X = X.contiguous()
    g = g.contiguous()
    h = h.contiguous()
    N, F = X.shape
    K = g.shape[1]
    ctx = ctx or L.init_distributed(X.device.index)
    if row_offset is None:
        row_offset, dataset_rows = _row_layout(N)
    M = 2 ** (max_depth + 1) - 1
    dev = X.device
    out = {
        "leaf_value": torch.empty((M, K), dtype=torch.float64, device=dev),
        "feature": torch.empty((M,), dtype=torch.int32, device=dev),
        "split_value": torch.empty((M,), dtype=torch.float64, device=dev),
        "gain": torch.empty((M,), dtype=torch.float64, device=dev),
        "hessian": torch.empty((M, K), dtype=torch.float64, device=dev),
    }
    a = L.BuildTreeArgs()
    a.X, a.x_dtype, a.ldx = X.data_ptr(), _dtype_code(X), X.stride(0) if N > 0 else F
    a.g, a.h, a.ldg = g.data_ptr(), h.data_ptr(), K
    fs = None
    if feature_set is not None:
        fs = feature_set.to(device=dev, dtype=torch.uint8).contiguous()
        a.feature_set = fs.data_ptr()
    a.row_offset, a.n_local_rows, a.n_features, a.n_outputs = row_offset, N, F, K
    a.max_depth, a.max_nodes, a.split_samples, a.seed = max_depth, M, split_samples, int(seed)
    a.dataset_rows = dataset_rows
    a.l1_regularization, a.l2_regularization, a.min_split_gain = l1, l2, min_split_gain
    a.leaf_value, a.feature = out["leaf_value"].data_ptr(), out["feature"].data_ptr()
    a.split_value, a.gain = out["split_value"].data_ptr(), out["gain"].data_ptr()
    a.hessian = out["hessian"].data_ptr()
    a.stream = _stream_ptr()
    B = C.c_int32(0)
    a.out_total_bins = C.pointer(B)
    out["node_sums"] = torch.zeros((M, K, 2), dtype=torch.int64, device=dev)
    a.trace_node_sums = out["node_sums"].data_ptr()
    trace = None
    if trace_nodes > 0:
        trace = torch.zeros((trace_nodes, K, F * split_samples, 2), dtype=torch.int64, device=dev)
        a.trace_hist, a.trace_nodes = trace.data_ptr(), trace_nodes
    if want_leaf:
        out["leaf"] = torch.empty((N,), dtype=torch.int32, device=dev)
        a.out_leaf = out["leaf"].data_ptr()
    if sketch is not None:
        a.sketch_mode = sketch.mode_for(X, split_samples, ctx)
        a.sketch = sketch.buffer.data_ptr()
    with torch.cuda.device(dev):
        ctx.check(ctx.lib.lbk_build_tree(ctx.handle, C.byref(a)))
    if sketch is not None:
        sketch.key = (_tensor_key(X), split_samples)
    out["B"] = B.value
    if trace is not None:
        # the library wrote with node stride K*B: re-view
        flat = trace.view(-1)[: trace_nodes * K * B.value * 2]
        out["trace_hist"] = flat.view(trace_nodes, K, B.value, 2)
    return out


def predict_arrays(X, trees, n_outputs=None, ctx=None):
    """Run ``lbk_predict``.  ``trees`` is a sequence of (leaf_value, feature, split_value) CUDA
    tensors.  Returns pred (N, K) float64."""
    assert X.is_cuda, "X must be a CUDA tensor (no CPU fallback)"
    if X.stride(1) != 1 and X.shape[0] > 0:
        X = X.contiguous()
    N, F = X.shape
    T = len(trees)
    keep = []
    K = n_outputs
    for lv, ft, sv in trees:
        lv = lv.to(torch.float64).contiguous()
        if lv.dim() == 1:
            lv = lv[:, None]
        keep.append((lv, ft.to(torch.int32).contiguous(), sv.to(torch.float64).contiguous()))
        K = lv.shape[1] if K is None else K
    pred = torch.empty((N, K), dtype=torch.float64, device=X.device)
    if N == 0:
        return pred
    ctx = ctx or L.context(X.device.index)
    a = L.PredictArgs()
    a.X, a.x_dtype, a.ldx, a.n_rows = X.data_ptr(), _dtype_code(X), X.stride(0), N
    a.n_features, a.n_outputs, a.n_trees = F, K, T
    PP = C.c_void_p * max(T, 1)
    lp, fp, sp = PP(), PP(), PP()
    mn = (C.c_int32 * max(T, 1))()
    for i, (lv, ft, sv) in enumerate(keep):
        lp[i], fp[i], sp[i], mn[i] = lv.data_ptr(), ft.data_ptr(), sv.data_ptr(), ft.shape[0]
    a.leaf_value, a.feature, a.split_value, a.max_nodes = lp, fp, sp, mn
    a.pred, a.ldp = pred.data_ptr(), K
    a.stream = _stream_ptr()
    with torch.cuda.device(X.device):
        ctx.check(ctx.lib.lbk_predict(ctx.handle, C.byref(a)))
    return pred


def onnx_tree_ensemble_attributes(feature, split_value, leaf_value):
    """The attributes of ONNX ``ai.onnx.ml.TreeEnsemble`` (opset 5) nodes for one tree in the
    heap layout of this library, one dict per output column (the operator has scalar leaves, so a
    vector-leaf tree becomes ``n_outputs`` ensembles that share the structure; the reference does
    the same, legateboost/models/tree.py:319-438).  Node slot i of the heap is both interior node
    i and leaf i of the operator: a child id is a node index or a leaf index depending on the
    ``*leafs`` flag of its parent.  numpy in, numpy out; no onnx package needed."""
    feature = np.asarray(feature, dtype=np.int64)
    split_value = np.asarray(split_value, dtype=np.float64)
    leaf_value = np.asarray(leaf_value, dtype=np.float64)
    M = feature.shape[0]
    ids = np.arange(M, dtype=np.int64)
    left, right = 2 * ids + 1, 2 * ids + 2
    is_leaf = feature < 0

    def child_is_leaf(child):
        # children of leaf slots can point past the arrays; such slots are never visited
        return is_leaf[np.minimum(child, M - 1)].astype(np.int64)

    true_leaf, false_leaf = child_is_leaf(left), child_is_leaf(right)
    true_id, false_id = left.copy(), right.copy()
    if is_leaf[0]:
        # a tree that is one leaf: the root sends every row to leaf 0
        true_id[0] = false_id[0] = 0
        true_leaf[0] = false_leaf[0] = 1
    out = []
    for k in range(leaf_value.shape[1]):
        out.append(dict(
            n_targets=int(leaf_value.shape[1]), aggregate_function=1, post_transform=0, tree_roots=[0],
            nodes_modes=np.zeros(M, dtype=np.uint8),            # 0 = BRANCH_LEQ: x <= split goes to the true child
            nodes_featureids=np.where(is_leaf, 0, feature),
            nodes_splits=split_value.copy(),
            nodes_truenodeids=true_id, nodes_trueleafs=true_leaf,
            nodes_falsenodeids=false_id, nodes_falseleafs=false_leaf,
            leaf_targetids=np.full(M, k, dtype=np.int64),
            leaf_weights=leaf_value[:, k].copy(),
        ))
    return out


class BaseModel:
    """Interface of a base learner (reference: legateboost/models/base_model.py:11-138)."""

    def set_random_state(self, random_state: np.random.RandomState) -> "BaseModel":
        self.random_state = random_state
        return self

    def __eq__(self, other: object) -> bool:
        return str(self) == str(other)

    def __hash__(self) -> int:
        return hash(str(self))


class Tree(BaseModel):
    """Decision tree model for gradient boosting (reference: legateboost/models/tree.py:22-101).

    Parameters
    ----------
    max_depth : int
        The maximum depth of the tree.
    split_samples : int
        Number of rows sampled as split candidates per tree (the number of bins per feature);
        at most 2048.
    feature_fraction : float or callable
        Fraction of features considered for this tree, or a callable returning a boolean mask of
        shape ``(n_features,)``.
    l1_regularization, l2_regularization : float
        Regularisation of the leaf weights.
    min_split_gain : float
        Minimum loss improvement needed to split, charged once per output.
    alpha : deprecated alias of ``l2_regularization``.
    """

    def __init__(
        self,
        *,
        max_depth: int = 8,
        split_samples: int = 256,
        feature_fraction: Union[float, Callable[[], Any]] = 1.0,
        l1_regularization: float = 0.0,
        l2_regularization: float = 1.0,
        min_split_gain: float = 0.0,
        alpha: Any = "deprecated",
    ) -> None:
        self.max_depth = max_depth
        if split_samples > 2048:
            raise ValueError("split_samples must be <= 2048")
        self.split_samples = split_samples
        self.alpha = alpha
        self.feature_fraction = feature_fraction
        self.l1_regularization = l1_regularization
        self.l2_regularization = l2_regularization
        self.min_split_gain = min_split_gain
        if alpha != "deprecated":
            warnings.warn(
                "`alpha` was renamed to `l2_regularization` in 23.03 and will be removed in 23.05",
                FutureWarning,
            )
            self.l2_regularization = alpha

    def num_nodes(self) -> int:
        return int((self.hessian > 0.0).sum())

    def is_leaf(self, id):
        return self.feature[id] == -1

    def left_child(self, id):
        return id * 2 + 1

    def right_child(self, id):
        return id * 2 + 2

    def fit(self, X: torch.Tensor, g: torch.Tensor, h: torch.Tensor) -> "Tree":
        # order of draws from the shared RandomState: the seed first, then the feature sample
        # (reference: tree.py:125 and :149-155)
        seed = self.random_state.randint(0, 2**31)
        feature_set = None
        if callable(self.feature_fraction):
            feature_set = self.feature_fraction()
            feature_set = torch.as_tensor(feature_set)
            if tuple(feature_set.shape) != (X.shape[1],) or feature_set.dtype != torch.bool:
                raise ValueError("feature_fraction must return a boolean array of shape (n_features,)")
        elif self.feature_fraction < 1.0:
            mask = np.zeros(X.shape[1], dtype=bool)
            n_sampled = max(1, int(X.shape[1] * self.feature_fraction))
            mask[self.random_state.choice(X.shape[1], n_sampled, False)] = True
            feature_set = torch.from_numpy(mask)
        # A driver that fits many trees on the same row blocks can set `row_layout` = (row_offset,
        # dataset_rows) once; otherwise every fit asks the other ranks for their row counts.
        row_offset, dataset_rows = getattr(self, "row_layout", None) or (None, None)
        out = build_tree_arrays(
            X, g, h, max_depth=self.max_depth, split_samples=self.split_samples, seed=seed,
            l1=self.l1_regularization, l2=self.l2_regularization, min_split_gain=self.min_split_gain,
            feature_set=feature_set, want_leaf=True, row_offset=row_offset, dataset_rows=dataset_rows,
            sketch=getattr(self, "sketch", None))
        self.leaf_value = out["leaf_value"]
        self.feature = out["feature"]
        self.split_value = out["split_value"]
        self.gain = out["gain"]
        self.hessian = out["hessian"]
        # The builder also says where every training row ended.  A boosting driver asks for the
        # predictions on the training matrix right after fit: the first predict() on the very same,
        # unmodified tensor is then a gather of leaf values instead of a second pass over X.  The
        # record is used once and dropped (it is one int32 per row).
        self._fit_rows = (_tensor_key(X), out["leaf"])
        return self

    def clear(self) -> None:
        self.leaf_value.fill_(0)
        self.hessian.fill_(0)

    def update(self, X: torch.Tensor, g: torch.Tensor, h: torch.Tensor) -> "Tree":
        """New leaf values and hessians from new gradients, the structure stays (reference:
        Tree.update, legateboost/models/tree.py:197-240 -> UPDATE_TREE)."""
        assert X.is_cuda and g.is_cuda and h.is_cuda, "inputs must be CUDA tensors (no CPU fallback)"
        if g.dim() == 1:
            g, h = g[:, None], h[:, None]
        assert g.dtype == torch.float64 and h.dtype == torch.float64
        if X.stride(1) != 1 and X.shape[0] > 0:
            X = X.contiguous()
        g, h = g.contiguous(), h.contiguous()
        N, F = X.shape
        K = g.shape[1]
        ctx = L.init_distributed(X.device.index)
        leaf_value = torch.empty_like(self.leaf_value)
        hessian = torch.empty_like(self.hessian)
        a = L.UpdateTreeArgs()
        a.X, a.x_dtype, a.ldx = X.data_ptr(), _dtype_code(X), X.stride(0) if N > 0 else F
        a.g, a.h, a.ldg = g.data_ptr(), h.data_ptr(), K
        a.n_local_rows, a.n_features, a.n_outputs = N, F, K
        a.max_nodes = self.feature.shape[0]
        a.feature, a.split_value = self.feature.data_ptr(), self.split_value.data_ptr()
        a.l1_regularization, a.l2_regularization = self.l1_regularization, self.l2_regularization
        a.leaf_value, a.hessian = leaf_value.data_ptr(), hessian.data_ptr()
        a.stream = _stream_ptr()
        with torch.cuda.device(X.device):
            ctx.check(ctx.lib.lbk_update_tree(ctx.handle, C.byref(a)))
        self.leaf_value, self.hessian = leaf_value, hessian
        self._fit_rows = None
        return self

    def predict(self, X: torch.Tensor) -> torch.Tensor:
        fit_rows, self._fit_rows = getattr(self, "_fit_rows", None), None
        if fit_rows is not None and fit_rows[0] == _tensor_key(X):
            leaf = fit_rows[1]
            out = torch.empty((leaf.shape[0], self.leaf_value.shape[1]), dtype=torch.float64, device=leaf.device)
            ctx = L.context(leaf.device.index)
            with torch.cuda.device(leaf.device):
                ctx.check(ctx.lib.lbk_leaf_values(ctx.handle, self.leaf_value.data_ptr(), leaf.data_ptr(),
                                                  leaf.shape[0], self.leaf_value.shape[1], out.data_ptr(), _stream_ptr()))
            return out
        return Tree.batch_predict([self], X)

    @staticmethod
    def batch_predict(models: Sequence["Tree"], X: torch.Tensor) -> torch.Tensor:
        assert all(isinstance(m, Tree) for m in models)
        return predict_arrays(X, [(m.leaf_value, m.feature, m.split_value) for m in models],
                              n_outputs=models[0].leaf_value.shape[1])

    def __str__(self) -> str:
        leaf_value = self.leaf_value.cpu().numpy()
        feature = self.feature.cpu().numpy()
        split_value = self.split_value.cpu().numpy()
        gain = self.gain.cpu().numpy()
        hessian = self.hessian.cpu().numpy()

        def format_vector(v) -> str:
            if np.isscalar(v):
                return "{:0.4f}".format(v)
            return "[" + ",".join(["{:0.4f}".format(x) for x in v]) + "]"

        def recurse_print(id: int, depth: int) -> str:
            if feature[id] == -1:
                text = "\t" * depth + "{}:leaf={},hess={}\n".format(
                    id, format_vector(leaf_value[id]), format_vector(hessian[id]))
            else:
                text = "\t" * depth + "{}:[f{}<={:0.4f}] yes={},no={},gain={:0.4f},hess={}\n".format(
                    id, feature[id], split_value[id], id * 2 + 1, id * 2 + 2, gain[id], hessian[id])
                text += recurse_print(id * 2 + 1, depth + 1)
                text += recurse_print(id * 2 + 2, depth + 1)
            return text

        return recurse_print(0, 0)

    def __getstate__(self):
        # pickled / deep-copied trees carry the model (the five arrays and the hyper-parameters), not
        # the per-fit scratch: the record of the training rows and the sketch buffer stay behind
        state = dict(self.__dict__)
        state.pop("_fit_rows", None)
        state.pop("sketch", None)
        return state

    def to_onnx(self) -> Any:
        """The tree as an ONNX model: X (float64, [rows, features]) -> predictions ([rows, outputs]),
        one ``TreeEnsemble`` node per output column summed with ``Add`` nodes, as the reference
        exports it (legateboost/models/tree.py:319-438).  Needs the ``onnx`` package."""
        try:
            import onnx
            from onnx import helper, numpy_helper
        except ImportError as e:  # the reference fails the same way without the package
            raise ImportError("Tree.to_onnx needs the onnx package") from e
        attrs = onnx_tree_ensemble_attributes(self.feature.cpu().numpy(), self.split_value.cpu().numpy(),
                                              self.leaf_value.cpu().numpy())
        nodes = []
        last = None
        for k, a in enumerate(attrs):
            tensors = {n: numpy_helper.from_array(a[n], name=n) for n in ("nodes_modes", "nodes_splits", "leaf_weights")}
            plain = {n: (v.tolist() if isinstance(v, np.ndarray) else v) for n, v in a.items() if n not in tensors}
            nodes.append(helper.make_node("TreeEnsemble", ["X"], ["pred%d" % k], domain="ai.onnx.ml", **plain, **tensors))
            acc = "accumulated_pred%d" % k
            if last is None:
                nodes.append(helper.make_node("Identity", ["pred%d" % k], [acc]))
            else:
                nodes.append(helper.make_node("Add", [last, "pred%d" % k], [acc]))
            last = acc
        X = helper.make_tensor_value_info("X", onnx.TensorProto.DOUBLE, [None, None])
        Y = helper.make_tensor_value_info(last, onnx.TensorProto.DOUBLE, [None, None])
        graph = helper.make_graph(nodes, "legateboost.models.Tree", [X], [Y])
        model = helper.make_model(graph, opset_imports=[helper.make_opsetid("ai.onnx.ml", 5), helper.make_opsetid("", 14)])
        onnx.checker.check_model(model)
        return model

    def __mul__(self, scalar: Any) -> "Tree":
        self._fit_rows = None  # the record of the training rows is not worth copying
        new = copy.deepcopy(self)
        new.leaf_value = new.leaf_value * scalar
        return new

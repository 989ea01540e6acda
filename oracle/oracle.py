"""ctypes front-end of the CPU oracle (test infrastructure, not part of the product).

Loads ``liblb_oracle.so`` (built from ``lb_oracle.cpp`` by ``make -C oracle``) and, when it has
been built, ``_ref/libref_cpu.so`` (the reference's own unmodified ``build_tree.cc`` /
``predict.cc`` behind a host-only stand-in for its runtime headers).  Only tests, the smoke
check and the CPU-baseline leg of the benchmark may import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None


def build(ref: bool = False, reference_dir: str = None) -> None:
    """Compile the oracle (and, if asked and the reference tree exists, the reference's CPU and GPU
    builds against the runtime stand-in; ``reference_dir`` = where the reference's sources lie,
    default: the REFERENCE_DIR variable or a folder named "reference" beside the repository)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "all"])
    if ref:
        if reference_dir is None:
            reference_dir = os.environ.get("REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)),
                                                                            "reference")
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "ref_gpu", "REFERENCE_DIR=" + reference_dir])


class _TreeArgs(C.Structure):
    _fields_ = [
        ("mode", C.c_int32), ("x_is_f64", C.c_int32),
        ("X", C.c_void_p), ("g", C.c_void_p), ("h", C.c_void_p), ("feature_set", C.c_void_p),
        ("n_rows", C.c_int64), ("F", C.c_int32), ("K", C.c_int32),
        ("max_depth", C.c_int32), ("split_samples", C.c_int32), ("seed", C.c_int32),
        ("l1", C.c_double), ("l2", C.c_double), ("min_split_gain", C.c_double),
        ("n_ranks", C.c_int32), ("rank_off", C.c_void_p),
        ("leaf_value", C.c_void_p), ("feature", C.c_void_p), ("split_value", C.c_void_p),
        ("gain", C.c_void_p), ("hessian", C.c_void_p),
        ("out_B", C.c_void_p), ("out_row_ptr", C.c_void_p), ("out_proposals", C.c_void_p),
        ("out_q", C.c_void_p), ("out_scale", C.c_void_p), ("out_node_sums", C.c_void_p),
        ("trace_nodes", C.c_int32), ("trace_hist", C.c_void_p), ("out_positions", C.c_void_p),
    ]


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liblb_oracle.so")
        if not os.path.exists(path):
            build()
        _LIB = C.CDLL(path)
        _LIB.lbo_build_tree.argtypes = [C.POINTER(_TreeArgs)]
        _LIB.lbo_build_tree.restype = C.c_int
        _LIB.lbo_abs_sum.restype = C.c_double
        _LIB.lbo_abs_sum.argtypes = [C.c_void_p, C.c_int64]
        _LIB.lbo_hash_combine.restype = C.c_int64
        _LIB.lbo_hash_combine.argtypes = [C.c_int64, C.c_int64, C.c_int64]
    return _LIB


def ref_lib():
    """The stub-compiled reference CPU build, or None when it has not been built."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libref_cpu.so")
        if not os.path.exists(path):
            return None
        _REF = C.CDLL(path)
    return _REF


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _rank_off(n_rows, n_ranks):
    """Contiguous, as-equal-as-possible row blocks (ceil-sized blocks first)."""
    base, extra = divmod(n_rows, n_ranks)
    off = [0]
    for r in range(n_ranks):
        off.append(off[-1] + base + (1 if r < extra else 0))
    return np.asarray(off, dtype=np.int64)


class TreeResult:
    pass


def build_tree(X, g, h, *, max_depth, split_samples=256, seed=0, l1=0.0, l2=1.0,
               min_split_gain=0.0, feature_set=None, mode="Q", n_ranks=1, rank_off=None,
               trace_nodes=0, want_q=False, use_reference=False):
    """Grow one tree.  mode "Q" follows the GPU variant, "D" the CPU variant.

    X: (N,F) float32/float64, g/h: (N,K) float64.  Returns a TreeResult with the five tree
    arrays and the optional traces.  ``use_reference`` routes a Mode-D call through the
    stub-compiled reference sources instead of the restatement.
    """
    X = np.ascontiguousarray(X)
    assert X.dtype in (np.float32, np.float64) and X.ndim == 2
    g = np.ascontiguousarray(g, dtype=np.float64)
    h = np.ascontiguousarray(h, dtype=np.float64)
    if g.ndim == 1:
        g, h = g[:, None], h[:, None]
    N, F = X.shape
    K = g.shape[1]
    M = 2 ** (max_depth + 1) - 1
    r = TreeResult()
    r.leaf_value = np.zeros((M, K))
    r.feature = np.zeros(M, dtype=np.int32)
    r.split_value = np.zeros(M)
    r.gain = np.zeros(M)
    r.hessian = np.zeros((M, K))
    off = _rank_off(N, n_ranks) if rank_off is None else np.asarray(rank_off, dtype=np.int64)
    fs = None if feature_set is None else np.ascontiguousarray(feature_set, dtype=np.uint8)
    if use_reference:
        assert mode == "D"
        ref = ref_lib()
        assert ref is not None, "reference CPU build not available (make -C oracle ref)"
        fn = ref.ref_build_tree_cpu
        fn.restype = C.c_int
        rc = fn(C.c_int(int(X.dtype == np.float64)), _ptr(X), _ptr(g), _ptr(h), _ptr(fs),
                C.c_int64(N), C.c_int(F), C.c_int(K), C.c_int(max_depth), C.c_int(split_samples),
                C.c_int(seed), C.c_double(l1), C.c_double(l2), C.c_double(min_split_gain),
                _ptr(r.leaf_value), _ptr(r.feature), _ptr(r.split_value), _ptr(r.gain),
                _ptr(r.hessian))
        assert rc == 0, "reference build_tree raised"
        return r
    a = _TreeArgs()
    a.mode = 0 if mode == "Q" else 1
    a.x_is_f64 = int(X.dtype == np.float64)
    a.X, a.g, a.h, a.feature_set = _ptr(X), _ptr(g), _ptr(h), _ptr(fs)
    a.n_rows, a.F, a.K = N, F, K
    a.max_depth, a.split_samples, a.seed = max_depth, split_samples, seed
    a.l1, a.l2, a.min_split_gain = l1, l2, min_split_gain
    a.n_ranks, a.rank_off = len(off) - 1, _ptr(off)
    a.leaf_value, a.feature, a.split_value = _ptr(r.leaf_value), _ptr(r.feature), _ptr(r.split_value)
    a.gain, a.hessian = _ptr(r.gain), _ptr(r.hessian)
    B = np.zeros(1, dtype=np.int32)
    r.row_ptr = np.zeros(F + 1, dtype=np.int32)
    props = np.zeros(F * split_samples, dtype=X.dtype)
    r.scale = np.zeros(4)
    r.positions = np.zeros(N, dtype=np.int32)
    a.out_B, a.out_row_ptr, a.out_proposals = _ptr(B), _ptr(r.row_ptr), _ptr(props)
    a.out_scale, a.out_positions = _ptr(r.scale), _ptr(r.positions)
    ns = np.zeros((M, K, 2), dtype=np.int64 if mode == "Q" else np.float64)
    a.out_node_sums = _ptr(ns)
    if want_q and mode == "Q":
        r.q = np.zeros((N, K, 2), dtype=np.int64)
        a.out_q = _ptr(r.q)
    trace = None
    if trace_nodes > 0:
        # B is not known before the call: size for the maximum F*S
        trace = np.zeros((trace_nodes, K, F * split_samples, 2),
                         dtype=np.int64 if mode == "Q" else np.float64)
    # the oracle writes the trace with stride K*B, so run once to learn B when tracing
    if trace_nodes > 0:
        a.trace_nodes, a.trace_hist = 0, None
        rc = lib().lbo_build_tree(C.byref(a))
        assert rc == 0
        trace = np.zeros((trace_nodes, K, int(B[0]), 2), dtype=trace.dtype)
        a.trace_nodes, a.trace_hist = trace_nodes, _ptr(trace)
    rc = lib().lbo_build_tree(C.byref(a))
    assert rc == 0
    r.B = int(B[0])
    r.proposals = props[: r.B].copy()
    r.node_sums = ns
    r.trace_hist = trace
    return r


def predict(X, trees):
    """trees: sequence of (leaf_value (M,K), feature (M,), split_value (M,)).  Returns (N,K) f64."""
    X = np.ascontiguousarray(X)
    N, F = X.shape
    T = len(trees)
    leaf = [np.ascontiguousarray(t[0], dtype=np.float64) for t in trees]
    feat = [np.ascontiguousarray(t[1], dtype=np.int32) for t in trees]
    split = [np.ascontiguousarray(t[2], dtype=np.float64) for t in trees]
    K = leaf[0].shape[1] if leaf[0].ndim == 2 else 1
    pred = np.zeros((N, K))
    PP = C.c_void_p * T
    lp = PP(*[x.ctypes.data for x in leaf])
    fp = PP(*[x.ctypes.data for x in feat])
    sp = PP(*[x.ctypes.data for x in split])
    lib().lbo_predict(_ptr(X), C.c_int(int(X.dtype == np.float64)), C.c_int64(N), C.c_int(F),
                      C.c_int(K), C.c_int(T), lp, fp, sp, _ptr(pred))
    return pred


_REF_UPDATE = None


def ref_update_lib():
    """The reference's own UPDATE_TREE task body (stub-compiled), or None when it has not been built."""
    global _REF_UPDATE
    if _REF_UPDATE is None:
        path = os.path.join(_HERE, "_ref", "libref_update.so")
        if not os.path.exists(path):
            return None
        _REF_UPDATE = C.CDLL(path)
    return _REF_UPDATE


def update_tree(X, g, h, feature, split_value, l1=0.0, l2=1.0, n_ranks=1, use_reference=False):
    """New (leaf_value, hessian), both (M, K) float64, of a tree whose structure stays
    (reference: update_tree.cc:36-134).  ``use_reference`` runs the stub-compiled reference task."""
    X = np.ascontiguousarray(X)
    g = np.ascontiguousarray(g, dtype=np.float64)
    h = np.ascontiguousarray(h, dtype=np.float64)
    if g.ndim == 1:
        g, h = g[:, None], h[:, None]
    N, F = X.shape
    K = g.shape[1]
    feature = np.ascontiguousarray(feature, dtype=np.int32)
    split_value = np.ascontiguousarray(split_value, dtype=np.float64)
    M = feature.shape[0]
    leaf = np.zeros((M, K))
    hess = np.zeros((M, K))
    if use_reference:
        rl = ref_update_lib()
        assert rl is not None, "build it with make -C oracle ref"
        assert n_ranks == 1
        rc = rl.ref_update_tree_cpu(C.c_int(int(X.dtype == np.float64)), _ptr(X), _ptr(g), _ptr(h), C.c_int64(N),
                                    C.c_int(F), C.c_int(K), C.c_int(M), _ptr(feature), _ptr(split_value),
                                    C.c_double(l1), C.c_double(l2), _ptr(leaf), _ptr(hess))
        assert rc == 0
        return leaf, hess
    off = _rank_off(N, n_ranks)
    lib().lbo_update_tree(_ptr(X), C.c_int(int(X.dtype == np.float64)), C.c_int64(N), C.c_int(F), C.c_int(K),
                          _ptr(g), _ptr(h), C.c_int(M), _ptr(feature), _ptr(split_value), C.c_double(l1),
                          C.c_double(l2), C.c_int(n_ranks), _ptr(off), _ptr(leaf), _ptr(hess))
    return leaf, hess


def split_proposals(X, split_samples, seed, mode="Q", n_ranks=1):
    X = np.ascontiguousarray(X)
    N, F = X.shape
    props = np.zeros(F * split_samples, dtype=X.dtype)
    row_ptr = np.zeros(F + 1, dtype=np.int32)
    off = _rank_off(N, n_ranks)
    fn = lib().lbo_split_proposals
    fn.restype = C.c_int
    B = fn(C.c_int(0 if mode == "Q" else 1), _ptr(X), C.c_int(int(X.dtype == np.float64)),
           C.c_int64(N), C.c_int(F), C.c_int(split_samples), C.c_int(seed), C.c_int(n_ranks),
           _ptr(off), _ptr(props), _ptr(row_ptr))
    return props[:B].copy(), row_ptr


def sample_rows(seed, S, n_rows):
    out = np.zeros(S, dtype=np.int64)
    lib().lbo_sample_rows(C.c_int(seed), C.c_int(S), C.c_int64(n_rows), _ptr(out))
    return out


def bin_x(X, proposals, row_ptr):
    X = np.ascontiguousarray(X)
    N, F = X.shape
    out = np.zeros((N, F), dtype=np.int16)
    proposals = np.ascontiguousarray(proposals, dtype=X.dtype)
    lib().lbo_bin_x(_ptr(X), C.c_int(int(X.dtype == np.float64)), C.c_int64(N), C.c_int(F),
                    _ptr(proposals), _ptr(np.ascontiguousarray(row_ptr, dtype=np.int32)), _ptr(out))
    return out


def abs_sum(v):
    v = np.ascontiguousarray(v, dtype=np.float64).ravel()
    return float(lib().lbo_abs_sum(_ptr(v), v.size))


def quantise(g, h, seed, n_ranks=1, rank_off=None):
    g = np.ascontiguousarray(g, dtype=np.float64)
    h = np.ascontiguousarray(h, dtype=np.float64)
    N, K = g.shape
    q = np.zeros((N, K, 2), dtype=np.int64)
    scale = np.zeros(4)
    off = _rank_off(N, n_ranks) if rank_off is None else np.asarray(rank_off, dtype=np.int64)
    lib().lbo_quantise(_ptr(g), _ptr(h), C.c_int64(N), C.c_int(K), C.c_int(seed),
                       C.c_int(len(off) - 1), _ptr(off), _ptr(q), _ptr(scale))
    return q, scale


def _bins_args(bins):
    bins = np.ascontiguousarray(bins)
    if bins.dtype == np.uint8:
        return bins, _ptr(bins), None
    bins = bins.astype(np.int16, copy=False)
    return bins, None, _ptr(bins)


def histogram_q(bins, row_ptr, q, node_of_row, node_begin, node_end):
    """Integer histogram [nodes,K,B,2] of int32 pairs q (N,K,2) over feature-relative bins (N,F)."""
    bins, p8, p16 = _bins_args(bins)
    N, F = bins.shape
    q = np.ascontiguousarray(q, dtype=np.int32)
    K = q.shape[1]
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    node_of_row = np.ascontiguousarray(node_of_row, dtype=np.int32)
    out = np.zeros((node_end - node_begin, K, int(row_ptr[-1]), 2), dtype=np.int64)
    lib().lbo_histogram_q(p8, p16, C.c_int64(N), C.c_int(F), _ptr(row_ptr), _ptr(q), C.c_int(K),
                          _ptr(node_of_row), C.c_int(node_begin), C.c_int(node_end), _ptr(out))
    return out


def histogram_d(bins, row_ptr, g, h, node_of_row, node_begin, node_end):
    """Double histogram [nodes,K,B,2]; g,h (N,K) float32 or float64."""
    bins, p8, p16 = _bins_args(bins)
    N, F = bins.shape
    g = np.ascontiguousarray(g)
    h = np.ascontiguousarray(h)
    K = g.shape[1]
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    node_of_row = np.ascontiguousarray(node_of_row, dtype=np.int32)
    out = np.zeros((node_end - node_begin, K, int(row_ptr[-1]), 2), dtype=np.float64)
    f32 = g.dtype == np.float32
    lib().lbo_histogram_d(p8, p16, C.c_int64(N), C.c_int(F), _ptr(row_ptr),
                          _ptr(g) if f32 else None, _ptr(h) if f32 else None,
                          None if f32 else _ptr(g), None if f32 else _ptr(h), C.c_int(K),
                          _ptr(node_of_row), C.c_int(node_begin), C.c_int(node_end), _ptr(out))
    return out

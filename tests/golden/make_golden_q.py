"""Generates tests/golden/treeq_*.npz: seeded inputs together with what the REFERENCE's own GPU code
produces for them on one device - the five tree arrays, the quantised node sums, every traced node's
histogram as the split search read it (all-reduced and scanned) and the predictions of the
reference's GPU predict task.

The reference's Python package cannot be imported without its runtime, so the vectors come from its
unmodified build_tree.cu / predict.cu compiled with nvcc against a stand-in of the runtime headers
(``make -C oracle ref_gpu`` -> oracle/_ref/libref_gpu.so, only possible where the reference source
tree is present; the built object is all this script needs).  Needs one CUDA device.  Inputs are
small and valid (hundreds to thousands of rows).  Run from the repository root:

    python tests/golden/make_golden_q.py [--out DIR] [--compare] [--lib FILE]

``--compare`` also runs the CPU oracle's quantised mode on every case and prints which arrays are
bit-for-bit equal (the record the parity statement rests on).  ``--lib`` names another build of the
same driver (oracle/_ref/libref_gpu_nofma.so, built without multiply-add contraction): its vectors,
written to another folder, tell the effect of contraction apart from everything else.
"""
import argparse
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

MAX_STORED_TRACE = 100_000  # int64 pairs of traced histograms kept in full per case; every traced node has a digest
MAX_STORED_INPUT = 25_000   # elements of X up to which the inputs themselves are stored; larger cases are
                            # regenerated from their seeds by cases() and checked against the stored hashes


def cases():
    """name -> dict(X, g, h, max_depth, split_samples, seed, l1, l2, min_split_gain, feature_set, trace_nodes)"""
    out = {}

    def add(name, X, g, h, D, S, seed, l1=0.0, l2=1.0, msg=0.0, feature_set=None, trace_nodes=None):
        M = 2 ** (D + 1) - 1
        out[name] = dict(X=X, g=g, h=h, max_depth=D, split_samples=S, seed=seed, l1=l1, l2=l2, min_split_gain=msg,
                         feature_set=feature_set, trace_nodes=M if trace_nodes is None else min(M, trace_nodes))

    # the four cases of tree_*.npz (same seeds, same data)
    for name, N, F, K, D, S, dt, l1, l2, msg, seed in [
            ("f32_k1", 600, 8, 1, 5, 32, np.float32, 0.0, 1.0, 0.0, 1872583848),
            ("f64_k3", 500, 6, 3, 4, 64, np.float64, 0.0, 1.0, 0.0, 12345),
            ("reg", 400, 5, 2, 6, 16, np.float32, 0.5, 2.0, 0.01, 99),
            ("ties", 300, 4, 1, 5, 256, np.float64, 0.0, 0.0, 0.0, 7)]:
        rs = np.random.RandomState(len(name) * 1000 + N)
        X = rs.random((N, F)).astype(dt)
        if name == "ties":
            X = np.round(X * 4) / 4
        g = rs.normal(size=(N, K))
        h = rs.random((N, K)) + 0.1
        add(name, X, g, h, D, S, seed, l1, l2, msg)

    # quantised hessians of 0: the rows with the smallest values of feature 0 carry hessians far
    # below one quantisation step and non-positive gradients, so that prefixes with hess == 0 and
    # grad <= 0 exist and the scan's conditional write is exercised; three outputs
    rs = np.random.RandomState(501)
    N, F, K = 3000, 5, 3
    X = rs.random((N, F)).astype(np.float32)
    g = rs.normal(size=(N, K))
    h = rs.random((N, K)) + 0.5
    low = X[:, 0] < 0.15
    h[low] = 1e-9
    g[low] = -np.abs(g[low]) * (rs.random((int(low.sum()), K)) < 0.7)  # some exactly 0
    add("smallh", X, g, h, 5, 64, 4242)

    # a feature mask, float32, one output
    rs = np.random.RandomState(502)
    N, F = 2000, 12
    X = rs.random((N, F)).astype(np.float32)
    g = rs.normal(size=(N, 1)) + 2.0 * (X[:, [3]] > 0.5) - 1.5 * (X[:, [7]] > 0.3)
    h = np.ones((N, 1))
    fs = np.ones(F, dtype=np.uint8)
    fs[[3, 5, 11]] = 0
    add("mask", X, g, h, 6, 128, 31337, feature_set=fs)

    # few rows, deep tree: nodes run out of rows and rows drop out of the position list
    rs = np.random.RandomState(503)
    X = rs.random((64, 3))
    add("deep", X, rs.normal(size=(64, 1)), rs.random((64, 1)) + 0.2, 9, 256, 77, trace_nodes=255)

    # many rows per node (whole tiles of one node, shared-memory path of the reference) and
    # several feature groups (more than 2048 bins in total)
    rs = np.random.RandomState(504)
    N, F = 20000, 16
    X = rs.random((N, F)).astype(np.float32)
    y = np.sin(6 * X[:, 0]) + X[:, 1] * X[:, 2] + 0.1 * rs.normal(size=N)
    add("rows20k", X, (0.3 * rs.normal(size=N) - y)[:, None], np.ones((N, 1)), 7, 256, 2024, trace_nodes=31)

    # level batching: one node's histogram is 2 MB (127680 bins), so the 1 GB rule holds 489 nodes:
    # level 9 (512 nodes) is cut into two batches (the second has populated nodes and splits), and
    # levels 8+ lie outside the cached histogram and are built without parents
    rs = np.random.RandomState(505)
    N, F = 1200, 560
    X = rs.random((N, F)).astype(np.float32)
    add("batching", X, rs.normal(size=(N, 1)), rs.random((N, 1)) + 0.5, 10, 256, 11, trace_nodes=3)

    # softmax-like gradients, ten outputs
    rs = np.random.RandomState(506)
    N, F, K = 4000, 10, 10
    X = rs.normal(size=(N, F)).astype(np.float32)
    logits = X[:, :K] @ rs.normal(size=(K, K)) + 0.5 * rs.normal(size=(N, K))
    p = np.exp(logits - logits.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    onehot = np.eye(K)[logits.argmax(1)]
    # gradients of the cross-entropy at a model that already fits well: p - onehot, p (1 - p) >= 1e-8
    q = 0.9 * onehot + 0.1 * p
    add("softmax10", X, q - onehot, np.maximum(q * (1.0 - q), 1e-8), 4, 64, 909, trace_nodes=7)
    return out


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def input_hash(c):
    """sha256 over the bytes of X, g and h (as the reference receives them)."""
    import hashlib

    m = hashlib.sha256()
    m.update(np.ascontiguousarray(c["X"]).tobytes())
    m.update(np.ascontiguousarray(c["g"], dtype=np.float64).tobytes())
    m.update(np.ascontiguousarray(c["h"], dtype=np.float64).tobytes())
    return m.hexdigest()


def load_case(path):
    """A stored case with its inputs: taken from the file, or regenerated from the seeds and
    checked against the stored hash.  Returns (npz, dict as cases() makes it)."""
    z = np.load(path)
    name = os.path.basename(path)[len("treeq_"):-len(".npz")]
    if "X" in z.files:
        fs = z["feature_set"] if z["feature_set"].size else None
        c = dict(X=z["X"], g=z["g"], h=z["h"], max_depth=int(z["max_depth"]), split_samples=int(z["split_samples"]),
                 seed=int(z["seed"]), l1=float(z["l1"]), l2=float(z["l2"]), min_split_gain=float(z["min_split_gain"]),
                 feature_set=fs, trace_nodes=int(z["trace_nodes"]))
    else:
        c = cases()[name]
    assert input_hash(c) == str(z["input_sha256"]), "inputs of %s are not the ones the vectors were made from" % name
    return z, c


def digest(hist):
    """One 64-bit number per traced node: sum of value * (2 * index + 1) modulo 2**64."""
    flat = hist.reshape(hist.shape[0], -1).astype(np.uint64)
    w = (2 * np.arange(flat.shape[1], dtype=np.uint64) + 1)
    with np.errstate(over="ignore"):
        return (flat * w).sum(axis=1, dtype=np.uint64)


def run_reference(lib, c, traced=True):
    X = np.ascontiguousarray(c["X"])
    g = np.ascontiguousarray(c["g"], dtype=np.float64)
    h = np.ascontiguousarray(c["h"], dtype=np.float64)
    N, F = X.shape
    K = g.shape[1]
    D, S = c["max_depth"], c["split_samples"]
    M = 2 ** (D + 1) - 1
    r = dict(leaf_value=np.zeros((M, K)), feature=np.zeros(M, dtype=np.int32), split_value=np.zeros(M),
             gain=np.zeros(M), hessian=np.zeros((M, K)))
    fs = c["feature_set"]
    head = (C.c_int(int(X.dtype == np.float64)), _ptr(X), _ptr(g), _ptr(h), _ptr(fs), C.c_int64(N), C.c_int(F), C.c_int(K),
            C.c_int(D), C.c_int(S), C.c_int(c["seed"]), C.c_double(c["l1"]), C.c_double(c["l2"]),
            C.c_double(c["min_split_gain"]), _ptr(r["leaf_value"]), _ptr(r["feature"]), _ptr(r["split_value"]),
            _ptr(r["gain"]), _ptr(r["hessian"]))
    if not traced:
        rc = lib.ref_gpu_build_tree(*head)
        assert rc == 0, "reference gpu build_tree raised"
        return r
    tn = c["trace_nodes"]
    trace = np.zeros((tn, K, F * S, 2), dtype=np.int64)
    ns = np.zeros((M, K, 2), dtype=np.int64)
    B = np.zeros(1, dtype=np.int32)
    rc = lib.ref_gpu_build_tree_trace(*head, _ptr(trace), C.c_int(tn), _ptr(ns), _ptr(B))
    assert rc == 0, "reference gpu build_tree (traced) raised"
    b = int(B[0])
    # the driver packs the rows with stride K * B
    packed = trace.reshape(-1)[: tn * K * b * 2].reshape(tn, K, b, 2).copy()
    r.update(node_sums=ns, trace_hist=packed, total_bins=b)
    return r


def run_predict(lib, c, tree):
    X = np.ascontiguousarray(c["X"])
    N, F = X.shape
    K = tree["leaf_value"].shape[1]
    pred = np.zeros((N, K))
    PP = C.c_void_p * 1
    mn = (C.c_int32 * 1)(tree["feature"].shape[0])
    rc = lib.ref_gpu_predict(C.c_int(int(X.dtype == np.float64)), _ptr(X), C.c_int64(N), C.c_int(F), C.c_int(K), C.c_int(1),
                             mn, PP(tree["leaf_value"].ctypes.data), PP(tree["feature"].ctypes.data),
                             PP(tree["split_value"].ctypes.data), _ptr(pred))
    assert rc == 0, "reference gpu predict raised"
    return pred


def same(a, b):
    a, b = np.asarray(a), np.asarray(b)
    if a.shape != b.shape:
        return False
    if a.dtype.kind == "f":
        return bool(np.array_equal(a.view(np.int64), b.view(np.int64)))
    return bool(np.array_equal(a, b))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--compare", action="store_true")
    ap.add_argument("--only", default=None)
    ap.add_argument("--lib", default=os.path.join(ROOT, "oracle", "_ref", "libref_gpu.so"))
    ap.add_argument("--nofma-dir", default=None,
                    help="folder written by a run with --lib .../libref_gpu_nofma.so: its float arrays are stored "
                         "beside the default build's as *_nofma")
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    lib = C.CDLL(args.lib)
    assert lib.ref_gpu_device_count() > 0, "a CUDA device is needed"
    for name, c in cases().items():
        if args.only and name != args.only:
            continue
        untraced = run_reference(lib, c, traced=False)   # the task body exactly as it stands
        r = run_reference(lib, c, traced=True)
        for k in ("leaf_value", "feature", "split_value", "gain", "hessian"):
            assert same(untraced[k], r[k]), "the traced walk differs from the task body in %s" % k
        pred = run_predict(lib, c, r)
        tn = c["trace_nodes"]
        dig = digest(r["trace_hist"])
        per_node = r["trace_hist"][0].size // 2
        stored = min(tn, MAX_STORED_TRACE // per_node)
        fs = c["feature_set"]
        keep = dict(max_depth=c["max_depth"], split_samples=c["split_samples"], seed=c["seed"], l1=c["l1"], l2=c["l2"],
                    min_split_gain=c["min_split_gain"], feature_set=np.zeros(0, dtype=np.uint8) if fs is None else fs,
                    input_sha256=input_hash(c), leaf_value=r["leaf_value"], feature=r["feature"],
                    split_value=r["split_value"], gain=r["gain"], hessian=r["hessian"], node_sums=r["node_sums"],
                    total_bins=r["total_bins"], trace_nodes=tn, trace_hist=r["trace_hist"][:stored], trace_digest=dig,
                    pred=pred)
        if c["X"].size <= MAX_STORED_INPUT:
            keep.update(X=c["X"], g=c["g"], h=c["h"])
        if args.nofma_dir:
            z2 = np.load(os.path.join(args.nofma_dir, "treeq_%s.npz" % name))
            for k in ("feature", "split_value", "node_sums", "trace_digest"):
                assert same(keep[k], z2[k]), "the build without contraction differs in %s" % k
            keep.update(leaf_value_nofma=z2["leaf_value"], gain_nofma=z2["gain"], hessian_nofma=z2["hessian"])
        np.savez_compressed(os.path.join(args.out, "treeq_%s.npz" % name), **keep)
        line = "wrote %-10s split nodes %4d  B %6d  traced %4d (stored %d)" % (
            name, int((r["feature"] >= 0).sum()), r["total_bins"], tn, stored)
        print(line, flush=True)
        if args.compare:
            from oracle import oracle as O

            t = O.build_tree(c["X"], c["g"], c["h"], max_depth=c["max_depth"], split_samples=c["split_samples"],
                             seed=c["seed"], l1=c["l1"], l2=c["l2"], min_split_gain=c["min_split_gain"],
                             feature_set=fs, mode="Q", trace_nodes=tn)
            o = dict(leaf_value=t.leaf_value, feature=t.feature, split_value=t.split_value, gain=t.gain,
                     hessian=t.hessian, node_sums=t.node_sums, trace_hist=t.trace_hist, total_bins=np.int32(t.B))
            rep = []
            for k in ("total_bins", "feature", "split_value", "node_sums", "trace_hist", "hessian", "leaf_value", "gain"):
                ok = same(np.asarray(r[k]), np.asarray(o[k]))
                s = "%s %s" % (k, "==" if ok else "DIFFERS")
                if not ok and np.asarray(r[k]).dtype.kind == "f" and np.asarray(r[k]).shape == np.asarray(o[k]).shape:
                    d = np.abs(r[k] - o[k])
                    s += " (max abs %.3g, max rel %.3g, %d of %d)" % (
                        d.max(), (d / np.maximum(np.abs(r[k]), 1e-300)).max(), int((d > 0).sum()), d.size)
                elif not ok and np.asarray(r[k]).shape == np.asarray(o[k]).shape:
                    s += " (%d of %d entries)" % (int((np.asarray(r[k]) != np.asarray(o[k])).sum()), np.asarray(r[k]).size)
                rep.append(s)
            po = O.predict(c["X"], [(r["leaf_value"], r["feature"], r["split_value"])])
            rep.append("pred %s" % ("==" if same(pred, po) else "DIFFERS (max abs %.3g)" % np.abs(pred - po).max()))
            print("   oracle Mode Q vs reference GPU: " + "; ".join(rep), flush=True)


if __name__ == "__main__":
    main()

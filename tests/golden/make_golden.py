"""Generates tests/golden/tree_*.npz: seeded inputs together with the tree arrays, the predictions and
the result of an update with new gradients that the REFERENCE's own CPU code produces for them.

The reference's Python package cannot be imported without its runtime, so the vectors come from its
unmodified build_tree.cc / predict.cc / update_tree.cc compiled against a host-only stand-in of the
runtime headers (``make -C oracle ref`` -> oracle/_ref/libref_cpu.so, libref_update.so, only possible
where the reference source tree is present).  Run from the repository root:  python tests/golden/make_golden.py
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

CASES = [
    # name, N, F, K, depth, split_samples, dtype, l1, l2, min_split_gain, seed
    ("f32_k1", 600, 8, 1, 5, 32, np.float32, 0.0, 1.0, 0.0, 1872583848),
    ("f64_k3", 500, 6, 3, 4, 64, np.float64, 0.0, 1.0, 0.0, 12345),
    ("reg", 400, 5, 2, 6, 16, np.float32, 0.5, 2.0, 0.01, 99),
    ("ties", 300, 4, 1, 5, 256, np.float64, 0.0, 0.0, 0.0, 7),
]


def main():
    O.build(ref=True)
    ref = O.ref_lib()
    assert ref is not None
    out_dir = os.path.dirname(os.path.abspath(__file__))
    for name, N, F, K, D, S, dt, l1, l2, msg, seed in CASES:
        rs = np.random.RandomState(len(name) * 1000 + N)
        X = rs.random((N, F)).astype(dt)
        if name == "ties":
            X = np.round(X * 4) / 4  # few distinct values: many equal gains
        g = rs.normal(size=(N, K))
        h = rs.random((N, K)) + 0.1
        t = O.build_tree(X, g, h, max_depth=D, split_samples=S, seed=seed, l1=l1, l2=l2,
                         min_split_gain=msg, mode="D", use_reference=True)
        # predictions from the reference's predict.cc
        T = 1
        PP = C.c_void_p * T
        mn = (C.c_int32 * T)(t.feature.shape[0])
        pred = np.zeros((N, K))
        fn = ref.ref_predict_cpu
        fn.restype = C.c_int
        rc = fn(C.c_int(int(X.dtype == np.float64)), X.ctypes.data_as(C.c_void_p), C.c_int64(N), C.c_int(F),
                C.c_int(K), C.c_int(T), mn, PP(t.leaf_value.ctypes.data), PP(t.feature.ctypes.data),
                PP(t.split_value.ctypes.data), pred.ctypes.data_as(C.c_void_p))
        assert rc == 0
        # the same tree updated with new gradients by the reference's update_tree.cc
        g2 = rs.normal(size=(N, K))
        h2 = rs.random((N, K)) + 0.1
        upd_leaf, upd_hess = O.update_tree(X, g2, h2, t.feature, t.split_value, l1=l1, l2=l2, use_reference=True)
        np.savez_compressed(os.path.join(out_dir, "tree_%s.npz" % name), X=X, g=g, h=h, max_depth=D,
                            split_samples=S, seed=seed, l1=l1, l2=l2, min_split_gain=msg,
                            leaf_value=t.leaf_value, feature=t.feature, split_value=t.split_value,
                            gain=t.gain, hessian=t.hessian, pred=pred, g2=g2, h2=h2,
                            upd_leaf_value=upd_leaf, upd_hessian=upd_hess)
        print("wrote", name, "split nodes:", int((t.feature >= 0).sum()))


if __name__ == "__main__":
    main()

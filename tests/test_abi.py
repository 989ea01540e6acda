"""CPU checks of the C-ABI library: it loads and exports every symbol include/lbk.h declares,
and the host-side mirror keeps the reference's constructor / error behaviour.  No compute call
is made here (there is no CPU path to call)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "lbk.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lbk_[a-z_0-9]+)\s*\(", text)) - {"lbk_allreduce_fn"})


def test_library_exports_every_declared_symbol():
    import legateboost_b200 as lb

    lib = lb.library.load()
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(lb.library.EXPORTS) == names
    assert lib.lbk_version() >= 1000


def test_no_device_is_an_error_not_a_fallback():
    import legateboost_b200 as lb

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    lib = lb.library.load()
    h = ctypes.c_void_p()
    rc = lib.lbk_context_create(0, ctypes.byref(h))
    assert rc != 0
    assert lib.lbk_last_error(None)
    with pytest.raises(RuntimeError):
        lb.library.context()


def test_tree_constructor_mirrors_reference():
    import legateboost_b200 as lb

    t = lb.Tree()
    assert (t.max_depth, t.split_samples, t.feature_fraction) == (8, 256, 1.0)
    assert (t.l1_regularization, t.l2_regularization, t.min_split_gain) == (0.0, 1.0, 0.0)
    with pytest.raises(ValueError, match="split_samples must be <= 2048"):
        lb.Tree(split_samples=4096)
    with pytest.warns(FutureWarning):
        assert lb.Tree(alpha=3.0).l2_regularization == 3.0


def test_feature_fraction_callable_is_validated_before_any_launch():
    # reference: legateboost/test/models/test_tree.py:130-157
    import legateboost_b200 as lb

    X = torch.zeros((10, 10))
    g = torch.zeros((10, 1), dtype=torch.float64)
    for bad in (lambda: torch.tensor([0, 1, 0, 0, 0, 0, 0, 0, 0, 0]),
                lambda: torch.tensor([0, 1, 0, 0, 0, 0, 0, 0, 0], dtype=torch.bool)):
        t = lb.Tree(feature_fraction=bad).set_random_state(np.random.RandomState(0))
        with pytest.raises(ValueError, match=r"feature_fraction must return a boolean array of shape \(n_features,\)"):
            t.fit(X, g, g)


def test_seed_and_feature_draw_order():
    # the seed is drawn before the feature subset (reference: tree.py:125, :149-155)
    rs = np.random.RandomState(5)
    seed = rs.randint(0, 2 ** 31)
    choice = rs.choice(10, 5, False)
    rs2 = np.random.RandomState(5)
    assert rs2.randint(0, 2 ** 31) == seed and np.array_equal(rs2.choice(10, 5, False), choice)


def test_legate_adapter_compiles_against_the_runtime_stand_in(tmp_path):
    """adapter/legate_adapter.cu - the bodies a maintainer puts behind BuildTreeTask::gpu_variant and
    PredictTask::gpu_variant - is real source: it compiles (nvcc, host and device pass) against
    include/lbk.h and the stand-in of the legate headers that the reference's own task bodies are
    compiled against here.  No legate runtime exists in this image, so it cannot be run."""
    import shutil
    import subprocess

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    out = tmp_path / "legate_adapter.o"
    cmd = [nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-c",
           os.path.join(ROOT, "adapter", "legate_adapter.cu"), "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(ROOT, "oracle", "ref_stub"), "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert out.stat().st_size > 0

"""Multi-GPU parity: every rank holds a contiguous block of rows, the library's collectives combine
proposals, scale and root sums, the histograms of a level are summed by feature ownership through
buffers the GPUs read from each other, the ranks exchange their best split candidates, and every
rank must end with the tree the oracle grows for the same number of simulated ranks (bit-exact).
Skipped with fewer than two GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(procs, q, world):
    """Starts the rank processes, collects one result per rank and never leaves a rank behind: a rank
    that is still alive after the others failed (it waits in a collective) is killed, so that it
    cannot sit on a GPU under the tests that follow."""
    import time

    for p in procs:
        p.start()
    deadline = time.monotonic() + 240
    try:
        res = []
        for _ in range(world):
            while True:
                try:
                    res.append(q.get(timeout=5))
                    break
                except Exception:
                    if time.monotonic() > deadline:
                        raise AssertionError("the rank processes did not finish in time")
                    if any(p.exitcode not in (None, 0) for p in procs):
                        raise AssertionError("a rank process failed: %s" % [p.exitcode for p in procs])
                    if all(p.exitcode is not None for p in procs):
                        raise AssertionError("the rank processes ended without a result")
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
        return res
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
                p.join(timeout=10)


def _worker(rank, world, port, case, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import legateboost_b200 as lb
    from oracle import oracle as O

    N, F, K, D, S = case
    rs = np.random.RandomState(11)
    X = rs.random((N, F)).astype(np.float32)
    g = rs.normal(size=(N, K))
    h = rs.random((N, K)) + 0.1
    off = O._rank_off(N, world)
    b, e = int(off[rank]), int(off[rank + 1])
    dev = torch.device("cuda", rank)
    t = lb.Tree(max_depth=D, split_samples=S).set_random_state(np.random.RandomState(5))
    t.fit(torch.from_numpy(X[b:e]).to(dev), torch.from_numpy(g[b:e]).to(dev), torch.from_numpy(h[b:e]).to(dev))
    pred = t.predict(torch.from_numpy(X[b:e]).to(dev)).cpu().numpy()
    seed = np.random.RandomState(5).randint(0, 2 ** 31)
    want = O.build_tree(X, g, h, max_depth=D, split_samples=S, seed=seed, mode="Q", n_ranks=world)
    ok = all(np.array_equal(getattr(t, n).cpu().numpy(), getattr(want, n))
             for n in ("feature", "split_value", "gain", "leaf_value", "hessian"))
    wp = O.predict(X[b:e], [(want.leaf_value, want.feature, want.split_value)])
    ok = ok and np.array_equal(pred, wp)
    # UPDATE_TREE with new gradients: every rank ends with the sums over both row blocks
    g2 = rs.normal(size=(N, K))
    h2 = rs.random((N, K)) + 0.1
    ul, uh = O.update_tree(X, g2, h2, want.feature, want.split_value, n_ranks=world)
    t.update(torch.from_numpy(X[b:e]).to(dev), torch.from_numpy(g2[b:e]).to(dev), torch.from_numpy(h2[b:e]).to(dev))
    ok = ok and np.allclose(t.leaf_value.cpu().numpy(), ul, rtol=1e-9, atol=1e-12)
    ok = ok and np.allclose(t.hessian.cpu().numpy(), uh, rtol=1e-10, atol=1e-12)
    # the optional sketch buffer: a saving fit and a reusing fit with the same seed both give the
    # oracle's tree (the reusing one skips the proposal sampling and its collective on every rank)
    sk = lb.Sketch()
    Xd, gd, hd = torch.from_numpy(X[b:e]).to(dev), torch.from_numpy(g[b:e]).to(dev), torch.from_numpy(h[b:e]).to(dev)
    for _ in range(2):
        t2 = lb.Tree(max_depth=D, split_samples=S).set_random_state(np.random.RandomState(5))
        t2.sketch = sk
        t2.fit(Xd, gd, hd)
        ok = ok and all(np.array_equal(getattr(t2, n).cpu().numpy(), getattr(want, n))
                        for n in ("feature", "split_value", "gain", "leaf_value", "hessian"))
    q.put((rank, bool(ok), int((want.feature >= 0).sum())))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("case", [(20000, 40, 1, 6, 256), (5001, 13, 3, 5, 64),
                                  (3000, 1, 1, 3, 16)])  # one feature: rank 0 owns none and searches nothing
def test_two_gpus_match_oracle_with_two_ranks(case):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, q)) for r in range(world)]
    res = _run(procs, q, world)
    assert all(ok for _, ok, _ in res), res
    assert res[0][2] >= 3


def _hist_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import legateboost_b200 as lb
    from legateboost_b200 import stages

    ctx = lb.library.init_distributed(rank)
    gen = torch.Generator(device=dev)
    gen.manual_seed(100 + rank)
    ok = True
    # second scenario: the last rank has no rows at all (it must still take part in every collective)
    for empty_last in (False, True):
        for mode in (0, 1):
            empty = empty_last and rank == world - 1
            N = 1 if empty else 150000 + 1000 * rank
            F, nb, n_nodes = 128, 256, 128
            bins = torch.randint(0, nb, (N, F), dtype=torch.uint8, device=dev, generator=gen)
            row_ptr = torch.arange(F + 1, dtype=torch.int32, device=dev) * nb
            if mode == 0:
                pairs = torch.randint(-5000, 5000, (N, 1, 2), dtype=torch.int32, device=dev, generator=gen)
            else:
                pairs = torch.randn((N, 1, 2), dtype=torch.float32, device=dev, generator=gen)
            node = torch.randint(0, n_nodes, (N,), dtype=torch.int32, device=dev, generator=gen) + (n_nodes - 1)
            if empty:
                node[:] = 5 * n_nodes  # its one row belongs to no node of the level: nothing to build
            row_index, seg = stages.group_rows(node, n_nodes - 1, n_nodes)
            local = stages.histogram(bins, row_ptr, pairs, row_index, seg, F, mode=mode, ctx=ctx)
            want = local.clone()
            dist.all_reduce(want)
            # every bin everywhere
            got = stages.histogram(bins, row_ptr, pairs, row_index, seg, F, mode=mode, ctx=ctx, all_reduce=1)
            # only the bins of the features this rank owns
            own = stages.histogram(bins, row_ptr, pairs, row_index, seg, F, mode=mode, ctx=ctx, all_reduce=2)
            f0, f1 = lb.library.owned_features(rank, world, F)
            lo, hi = f0 * nb, f1 * nb
            if mode == 0:
                ok = ok and bool(torch.equal(got, want)) and bool(torch.equal(own[:, :, lo:hi], want[:, :, lo:hi]))
            else:
                tol = 1e-5 * float(want.abs().max())
                ok = ok and float((got - want).abs().max()) <= tol
                ok = ok and float((own[:, :, lo:hi] - want[:, :, lo:hi]).abs().max()) <= tol
            ok = ok and (empty_last or bool((want != local).any()))  # the other rank really contributed
    q.put((rank, ok))
    dist.barrier()
    dist.destroy_process_group()


def test_histogram_sums_over_ranks_match_a_plain_all_reduce():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_hist_worker, args=(r, world, port, q)) for r in range(world)]
    res = _run(procs, q, world)
    assert all(ok for _, ok in res), res

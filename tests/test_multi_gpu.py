"""Multi-GPU parity: every rank holds a contiguous block of rows, the library's NCCL all-reduces
combine proposals, scale, root sums and per-level histograms, and every rank must end with the
tree the oracle grows for the same number of simulated ranks (bit-exact).  Skipped with fewer than
two GPUs."""
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


@pytest.mark.parametrize("case", [(20000, 40, 1, 6, 256), (5001, 13, 3, 5, 64)])
def test_two_gpus_match_oracle_with_two_ranks(case):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in res), res
    assert res[0][2] > 3


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
    N, F, nb, n_nodes = 150000 + 1000 * rank, 128, 256, 128
    bins = torch.randint(0, nb, (N, F), dtype=torch.uint8, device=dev, generator=gen)
    row_ptr = torch.arange(F + 1, dtype=torch.int32, device=dev) * nb
    q_pairs = torch.randint(-5000, 5000, (N, 1, 2), dtype=torch.int32, device=dev, generator=gen)
    node = torch.randint(0, n_nodes, (N,), dtype=torch.int32, device=dev, generator=gen) + (n_nodes - 1)
    row_index, seg = stages.group_rows(node, n_nodes - 1, n_nodes)
    local = stages.histogram(bins, row_ptr, q_pairs, row_index, seg, F, mode=0, ctx=ctx)
    want = local.clone()
    dist.all_reduce(want)
    # large enough (67 MB, 256 tickets) for the all-reduce to travel in parts beside the next part's kernel
    got = stages.histogram(bins, row_ptr, q_pairs, row_index, seg, F, mode=0, ctx=ctx, all_reduce=True)
    ok = bool(torch.equal(got, want)) and bool((want != local).any())
    q.put((rank, ok))
    dist.barrier()
    dist.destroy_process_group()


def test_histogram_all_reduce_in_parts_matches_a_plain_all_reduce():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_hist_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(ok for _, ok in res), res

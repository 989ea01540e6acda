"""world_size-2 gloo tests (CPU) of the host-side logic the multi-GPU path relies on: row block
offsets, shard sizes of the bench, and the estimator's cross-rank sums."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from legateboost_b200.tree import _row_layout
    from legateboost_b200.estimator import _SquaredError, _LogLoss
    import bench

    n_local = 5 + rank * 3
    off, total = _row_layout(n_local)
    y = torch.arange(n_local, dtype=torch.float64)[:, None] + 10 * rank
    init = _SquaredError().init(y, True)
    lab = torch.tensor([[0.0], [1.0], [2.0]]) if rank == 0 else torch.tensor([[2.0], [2.0]])
    linit = _LogLoss().init(lab.to(torch.float64), True)
    shard = bench.shard_rows(1003, rank, world)
    q.put((rank, off, total, float(init[0]), linit.tolist(), shard))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_gloo():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, off0, tot0, init0, l0, s0), (r1, off1, tot1, init1, l1, s1) = res
    assert (off0, tot0) == (0, 13) and (off1, tot1) == (5, 13)
    all_y = np.concatenate([np.arange(5), np.arange(8) + 10])
    assert np.isclose(init0, all_y.mean()) and init0 == init1
    assert np.allclose(l0, np.log(np.array([1, 1, 3]) / 5)) and l0 == l1
    # shards: contiguous, cover everything once
    assert s0[0] == 0 and s0[1] == s1[0] and s1[1] == 1003


def test_feature_ownership_covers_every_feature_once():
    """The division of the features among the ranks (what decides which bins a rank sums and
    searches): contiguous, in rank order, complete, also with more ranks than features; a pure host
    function of the C ABI, equal on every rank by construction."""
    import legateboost_b200 as lb

    for F in (0, 1, 7, 64, 100, 4096):
        for R in (1, 2, 3, 8, 64):
            got = [lb.library.owned_features(r, R, F) for r in range(R)]
            assert got[0][0] == 0 and got[-1][1] == F
            for (b0, e0), (b1, e1) in zip(got, got[1:]):
                assert e0 == b1 and b0 <= e0
            sizes = [e - b for b, e in got]
            assert max(sizes) - min(sizes) <= 1
    lib = lb.library.load()
    import ctypes as C

    b, e = C.c_int(), C.c_int()
    assert lib.lbk_owned_features(2, 2, 10, C.byref(b), C.byref(e)) == -1   # rank out of range

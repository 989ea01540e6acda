"""Benchmark of the tree-building hot path.

Default workload = the histogram-build microbenchmark: 10M rows x 128 features of uint8 bin ids
uniform in [0,255], rows assigned uniformly at random to the 128 nodes of tree level 7, one
output, quantised int32 gradient pairs.  A step is one histogram build over the whole batch; with
N GPUs every rank holds its own 10M-row shard (weak scaling) and the level's histograms are summed
over ranks with an NCCL all-reduce inside the step.

    python bench.py --gpus N --steps K --warmup W          (torchrun for N > 1)
    python bench.py --impl reference ...                   the reference's CPU code, timed on the host
    python bench.py --workload train|predict ...           other stages of the path (own JSON line)

One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

HIST_ROWS, HIST_FEATURES, HIST_NODES, HIST_BINS = 10_000_000, 128, 128, 256


def shard_rows(n_rows, rank, world):
    """Contiguous block [begin, end) of rank `rank` when n_rows are cut into `world` blocks."""
    base, extra = divmod(n_rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.rows = []
        self.proc = None
        self.device_index = device_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def wait_for_first_sample(self, limit=3.0):
        """nvidia-smi takes a moment to start printing: the timed region should begin after that."""
        t0 = time.perf_counter()
        while self.proc is not None and not self.rows and time.perf_counter() - t0 < limit:
            time.sleep(0.01)

    def stop(self, t_begin=None, t_end=None, t_load=None):
        """Median SM clock and the throttle reasons seen between t_begin and t_load (host clock,
        seconds: the timed region and the identical untimed steps after it); all samples if none
        arrived in that window."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.03)  # the sample taken at the end of the window is still on its way
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = list(self.rows)
        timed = [r for t, r in rows if t_begin is not None and t_begin <= t <= t_end + 0.03]
        loaded = [r for t, r in rows if t_begin is not None and t_begin <= t <= (t_load or t_end) + 0.03]
        use = loaded if loaded else [r for _, r in rows]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in use:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "samples_in_timed_region": len(timed), "reasons": sorted(reasons)}


def hist_inputs(torch, n_rows, seed, device):
    """Synthetic level-7 inputs on the device: row-major uint8 bins, node-grouped row index,
    quantised pairs from the library's own quantiser (scale = INT32_MAX / sum|g|, as the tree
    builder uses), float32 pairs for the float path."""
    from legateboost_b200 import stages

    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    G = HIST_FEATURES // 32
    bins = torch.randint(0, HIST_BINS, (n_rows, G * 32), dtype=torch.uint8, device=device, generator=gen)
    row_ptr = (torch.arange(HIST_FEATURES + 1, dtype=torch.int32, device=device) * HIST_BINS)
    g = torch.randn((n_rows, 1), dtype=torch.float64, device=device, generator=gen)
    h = torch.ones((n_rows, 1), dtype=torch.float64, device=device)
    gpair, _, _, max_abs = stages.quantise(g, h, seed=seed, with_max_abs=True)
    gpair_f = torch.stack([g.to(torch.float32), h.to(torch.float32)], dim=2).contiguous()
    node = torch.randint(0, HIST_NODES, (n_rows,), dtype=torch.int32, device=device, generator=gen) + (HIST_NODES - 1)
    row_index, seg = stages.group_rows(node, HIST_NODES - 1, HIST_NODES)
    del g, h
    return bins, row_ptr, gpair, gpair_f, row_index, seg, node, max_abs


# DRAM bytes of one k_hist_smem launch as ncu measured them (profiles/k_hist_smem_config2_ncu.md):
# bytes read per row, and bytes that do not grow with the rows (the output leaving L2 and what the
# flush buffer left dirty there), from the 2 M-row capture of the kernel as it is now.  None = no such
# capture: traffic is null.
HIST_DRAM_BYTES_PER_ROW = 145.2
HIST_DRAM_BYTES_FIXED = 60.1e6


def hist_traffic(n_rows):
    if HIST_DRAM_BYTES_PER_ROW is None:
        return None
    return n_rows * HIST_DRAM_BYTES_PER_ROW + HIST_DRAM_BYTES_FIXED


def algorithmic_bytes(n_rows):
    # per processed row: F bin bytes + 8 (int32 pair) + 4 (row index); per built node: B*16
    return n_rows * (HIST_FEATURES + 8 + 4) + HIST_NODES * HIST_FEATURES * HIST_BINS * 16


def _ref_hist_lib():
    """The reference's own CPU histogram step (stub-compiled), or None when it was not built."""
    import ctypes as C

    path = os.path.join(ROOT, "oracle", "_ref", "libref_hist.so")
    if not os.path.exists(path):
        return None
    lib = C.CDLL(path)
    lib.ref_compute_histogram.restype = C.c_double
    return lib


def cpu_hist_data(n_rows_sample, seed):
    """Host copy of the benchmark's inputs for `n_rows_sample` rows: bins, g, h, node of every row."""
    rs = np.random.default_rng(seed)
    bins = rs.integers(0, HIST_BINS, size=(n_rows_sample, HIST_FEATURES), dtype=np.uint8)
    g = rs.normal(size=(n_rows_sample, 1))
    h = np.ones((n_rows_sample, 1))
    node = rs.integers(0, HIST_NODES, size=n_rows_sample).astype(np.int32) + (HIST_NODES - 1)
    return bins, g, h, node


def cpu_hist_sample(n_rows_sample, seed, threads, data=None):
    """CPU histogram of one row sample of the level-7 batch on `threads` host threads, one rank
    per thread on a row shard, partial histograms summed in process (the stand-in for the CPU
    all-reduce).  Uses the reference's own ComputeHistogram (src/models/tree/build_tree.cc:258-289,
    stub-compiled) when that build is present, else the oracle's restatement of the same loop.
    `data` = a sample made by cpu_hist_data (made here when absent).
    Returns (rows*features/s, seconds, kind)."""
    import ctypes as C

    bins, g, h, node = data if data is not None else cpu_hist_data(n_rows_sample, seed)
    ref = _ref_hist_lib()
    parts = [None] * threads
    inner = [0.0] * threads
    shape = (HIST_NODES, 1, HIST_FEATURES * HIST_BINS, 2)
    if ref is not None:
        kind = "reference"

        def work(t):
            b, e = shard_rows(n_rows_sample, t, threads)
            out = np.zeros(shape)
            bb, gg, hh, nn = (np.ascontiguousarray(a[b:e]) for a in (bins, g, h, node))
            inner[t] = ref.ref_compute_histogram(
                bb.ctypes.data_as(C.c_void_p), C.c_int64(e - b), C.c_int(HIST_FEATURES), C.c_int(HIST_BINS),
                gg.ctypes.data_as(C.c_void_p), hh.ctypes.data_as(C.c_void_p), C.c_int(1),
                nn.ctypes.data_as(C.c_void_p), C.c_int(HIST_NODES - 1), C.c_int(2 * HIST_NODES - 1),
                out.ctypes.data_as(C.c_void_p))
            parts[t] = out
    else:
        kind = "port"
        from oracle import oracle as O

        O.lib()
        row_ptr = (np.arange(HIST_FEATURES + 1) * HIST_BINS).astype(np.int32)

        def work(t):
            b, e = shard_rows(n_rows_sample, t, threads)
            t0 = time.perf_counter()
            parts[t] = O.histogram_d(bins[b:e], row_ptr, g[b:e], h[b:e], node[b:e], HIST_NODES - 1, 2 * HIST_NODES - 1)
            inner[t] = time.perf_counter() - t0

    ths = [threading.Thread(target=work, args=(t,)) for t in range(threads)]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    t0 = time.perf_counter()
    total = parts[0]
    for p in parts[1:]:
        total += p
    dt = max(inner) + (time.perf_counter() - t0)  # slowest rank + the sum over ranks
    return n_rows_sample * HIST_FEATURES / dt, dt, kind


ROUNDS_TOTAL_ROWS, ROUNDS_FEATURES, ROUNDS_DEPTH = 100_000_000, 64, 8
PREDICT_TOTAL_ROWS, PREDICT_FEATURES, PREDICT_TREES, PREDICT_DEPTH = 50_000_000, 100, 500, 8


def _max_over_ranks(torch, dist, world, device, value):
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def rounds_section(torch, dist, lb, rank, world, device, total_rows, rounds, warmup):
    """Boosting rounds per second (squared error, depth 8, 256 bins) on the scale-out workload:
    X uniform[0,1) float32 (total_rows, 64), y = X w + 0.1 N(0,1); the rows are split evenly over
    the ranks (strong scaling).  Also the histogram kernel's share: its algorithmic bytes over the
    timed rounds (from the grown trees' node sizes: with unit hessians a node's hessian is its row
    count; the smaller child of every split is what gets built) against its summed duration."""
    import ctypes as C

    b, e = shard_rows(total_rows, rank, world)
    n, F = e - b, ROUNDS_FEATURES
    gen = torch.Generator(device=device)
    gen.manual_seed(3 + rank)
    X = torch.rand((n, F), dtype=torch.float32, device=device, generator=gen)
    w = torch.randn(F, dtype=torch.float32, device=device, generator=torch.Generator(device=device).manual_seed(3))
    y = X @ w + 0.1 * torch.randn(n, dtype=torch.float32, device=device, generator=gen)
    ctx = lb.library.init_distributed(device.index)
    lib = ctx.lib
    mk = lambda k: lb.LBRegressor(n_estimators=k, base_models=(lb.Tree(max_depth=ROUNDS_DEPTH),), random_state=0)  # noqa: E731
    mk(max(warmup, 1)).fit(X, y)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    lib.lbk_profile_enable(ctx.handle, 1)
    m = mk(rounds)
    a, bb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    m.fit(X, y)
    bb.record()
    torch.cuda.synchronize()
    ms = _max_over_ranks(torch, dist, world, device, a.elapsed_time(bb))
    hist_ms, launches = C.c_float(0), C.c_int(0)
    ctx.check(lib.lbk_profile_histogram_total(ctx.handle, C.byref(hist_ms), C.byref(launches)))
    hist_ms_max = _max_over_ranks(torch, dist, world, device, hist_ms.value)
    # algorithmic bytes of the histogram builds of this rank: rows * (F + 8 + 4) + built nodes * B * 16
    rows_built, nodes_built = 0.0, 0
    for t in m.models_:
        feat = t.feature.cpu().numpy()
        hess = t.hessian.cpu().numpy()[:, 0]
        rows_built += hess[0]
        nodes_built += 1
        split = np.nonzero(feat >= 0)[0]
        # the children of the splits of levels 0 .. depth-2 are built (the last level is not evaluated)
        last_eval_begin = 2 ** (ROUNDS_DEPTH - 1) - 1
        inner = split[split < last_eval_begin]
        rows_built += np.minimum(hess[2 * inner + 1], hess[2 * inner + 2]).sum()
        nodes_built += len(inner)
    bins_total = F * 256
    alg = rows_built / world * (F + 8 + 4) + nodes_built * bins_total * 16
    peak, which = measured_peaks()
    gbs = alg / (hist_ms_max * 1e-3) / 1e9 if hist_ms_max > 0 else 0.0
    lib.lbk_profile_enable(ctx.handle, 0)
    del X, y, m
    torch.cuda.empty_cache()
    return {"value": rounds / (ms * 1e-3), "unit": "rounds/s", "depth": ROUNDS_DEPTH, "rows": total_rows,
            "features": F, "rounds": rounds, "ms_per_round": ms / rounds, "scaling": "strong",
            "hist": {"kernel_ms_per_round": hist_ms_max / rounds, "launches": launches.value, "achieved": gbs,
                     "peak": peak, "unit": "GB/s", "frac": gbs / peak, "peak_source": which}}


def predict_section(torch, dist, lb, rank, world, device, total_rows, steps):
    """Ensemble predict rows per second: 500 random trees of depth 8 (feature uniform, threshold
    uniform[0,1), leaves N(0,1)) on X uniform[0,1) float32 (total_rows, 100), one output; the rows are
    split over the ranks, no collective."""
    from legateboost_b200.tree import predict_arrays

    b, e = shard_rows(total_rows, rank, world)
    n, F, T, D = e - b, PREDICT_FEATURES, PREDICT_TREES, PREDICT_DEPTH
    gen = torch.Generator(device=device)
    gen.manual_seed(4)
    M = 2 ** (D + 1) - 1
    trees = []
    for _ in range(T):
        feat = torch.randint(0, F, (M,), dtype=torch.int32, device=device, generator=gen)
        feat[2 ** D - 1:] = -1
        trees.append((torch.randn((M, 1), dtype=torch.float64, device=device, generator=gen), feat,
                      torch.rand((M,), dtype=torch.float64, device=device, generator=gen)))
    gen.manual_seed(40 + rank)
    X = torch.rand((n, F), dtype=torch.float32, device=device, generator=gen)
    predict_arrays(X, trees)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, bb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        predict_arrays(X, trees)
    bb.record()
    torch.cuda.synchronize()
    ms = _max_over_ranks(torch, dist, world, device, a.elapsed_time(bb)) / steps
    peak, which = measured_peaks()
    gbs = total_rows * (F * 4 + 8) / (ms * 1e-3) / 1e9
    del X
    torch.cuda.empty_cache()
    return {"value": total_rows / (ms * 1e-3), "unit": "rows/s", "rows": total_rows, "features": F, "trees": T,
            "depth": D, "ms_per_pass": ms, "node_visits_per_s": total_rows * T * D / (ms * 1e-3),
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak * world, "unit": "GB/s",
                         "frac": gbs / (peak * world), "peak_source": which}}


def _ref_cpu_lib():
    import ctypes as C

    path = os.path.join(ROOT, "oracle", "_ref", "libref_cpu.so")
    return C.CDLL(path) if os.path.exists(path) else None


def cpu_rounds_sample(sample_rows, threads):
    """The reference's CPU BUILD_TREE + PREDICT (its unmodified build_tree.cc / predict.cc, stub-compiled)
    for one round of the scale-out workload on a row sample: one rank per host thread, every rank
    grows a depth-8 tree on its own row shard and predicts it (no collective between them: a lower
    bound of the distributed round's time).  Returns rounds/s on the sample, or None."""
    import ctypes as C

    ref = _ref_cpu_lib()
    if ref is None:
        return None
    F, D = ROUNDS_FEATURES, ROUNDS_DEPTH
    rs = np.random.default_rng(3)
    X = rs.random((sample_rows, F), dtype=np.float32)
    w = rs.normal(size=F).astype(np.float32)
    g = (0.0 - (X @ w + 0.1 * rs.normal(size=sample_rows).astype(np.float32))).astype(np.float64)[:, None]
    h = np.ones((sample_rows, 1))
    M = 2 ** (D + 1) - 1
    times = [0.0] * threads
    ref.ref_build_tree_cpu.restype = C.c_int
    ref.ref_predict_cpu.restype = C.c_int

    def work(t):
        b, e = shard_rows(sample_rows, t, threads)
        Xs, gs, hs = (np.ascontiguousarray(a[b:e]) for a in (X, g, h))
        leaf, feat, split, gain, hess = np.zeros((M, 1)), np.zeros(M, dtype=np.int32), np.zeros(M), np.zeros(M), np.zeros((M, 1))
        pred = np.zeros((e - b, 1))
        t0 = time.perf_counter()
        p = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731
        ref.ref_build_tree_cpu(C.c_int(0), p(Xs), p(gs), p(hs), None, C.c_int64(e - b), C.c_int(F), C.c_int(1), C.c_int(D),
                               C.c_int(256), C.c_int(7), C.c_double(0.0), C.c_double(1.0), C.c_double(0.0), p(leaf),
                               p(feat), p(split), p(gain), p(hess))
        PP = C.c_void_p * 1
        ref.ref_predict_cpu(C.c_int(0), p(Xs), C.c_int64(e - b), C.c_int(F), C.c_int(1), C.c_int(1), (C.c_int32 * 1)(M),
                            PP(leaf.ctypes.data), PP(feat.ctypes.data), PP(split.ctypes.data), p(pred))
        times[t] = time.perf_counter() - t0

    ths = [threading.Thread(target=work, args=(t,)) for t in range(threads)]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    return 1.0 / max(times)


def cpu_predict_sample(sample_rows, threads):
    """The reference's CPU PREDICT (predict.cc, stub-compiled) of the 500-tree ensemble on a row sample,
    one rank per host thread on a row shard.  Returns rows/s, or None."""
    import ctypes as C

    ref = _ref_cpu_lib()
    if ref is None:
        return None
    F, T, D = PREDICT_FEATURES, PREDICT_TREES, PREDICT_DEPTH
    rs = np.random.default_rng(4)
    M = 2 ** (D + 1) - 1
    leaf = [rs.normal(size=(M, 1)) for _ in range(T)]
    feat = []
    for _ in range(T):
        f = rs.integers(0, F, size=M).astype(np.int32)
        f[2 ** D - 1:] = -1
        feat.append(f)
    split = [rs.random(M) for _ in range(T)]
    X = rs.random((sample_rows, F), dtype=np.float32)
    PP = C.c_void_p * T
    lp, fp, sp = PP(*[a.ctypes.data for a in leaf]), PP(*[a.ctypes.data for a in feat]), PP(*[a.ctypes.data for a in split])
    mn = (C.c_int32 * T)(*([M] * T))
    times = [0.0] * threads
    ref.ref_predict_cpu.restype = C.c_int

    def work(t):
        b, e = shard_rows(sample_rows, t, threads)
        Xs = np.ascontiguousarray(X[b:e])
        pred = np.zeros((e - b, 1))
        t0 = time.perf_counter()
        ref.ref_predict_cpu(C.c_int(0), Xs.ctypes.data_as(C.c_void_p), C.c_int64(e - b), C.c_int(F), C.c_int(1), C.c_int(T),
                            mn, lp, fp, sp, pred.ctypes.data_as(C.c_void_p))
        times[t] = time.perf_counter() - t0

    ths = [threading.Thread(target=work, args=(t,)) for t in range(threads)]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    return sample_rows / max(times)


def run_reference(args):
    """Reference arm: the reference's CPU histogram path on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample = 2_000_000
    for _ in range(args.warmup if args.warmup < 2 else 1):
        cpu_hist_sample(200_000, 1, threads)
    t_all = 0.0
    kind = "port"
    data = cpu_hist_data(sample, 1)  # made once, outside the timed steps
    for i in range(args.steps):
        v, dt, kind = cpu_hist_sample(sample, 1, threads, data)
        t_all += dt
    value = sample * HIST_FEATURES * args.steps / t_all
    line = {
        "impl": "reference", "metric": "histogram rows*features/s", "value": value, "unit": "row-features/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_all / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "histogram build, level 7 (128 nodes), %d rows x %d features x %d bins per step, "
                               "float64 accumulation on the host" % (sample, HIST_FEATURES, HIST_BINS)},
        "cpu_baseline": {"value": value, "unit": "row-features/s", "cores": threads, "kind": kind,
                         "sample": "%d-row sample of the 10M-row batch per step, %d ranks (threads) on row shards, "
                                   "time = slowest rank inside ComputeHistogram (which ends with its prefix scan; "
                                   "the GPU figure is the build alone) + in-process sum; reference sources compiled "
                                   "with g++ -O2 against the runtime stand-in" % (sample, threads)},
        "e2e": {"value": value, "unit": "row-features/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if not args.no_extra:
        rows_r, rows_p = 2_000_000, 400_000
        r = cpu_rounds_sample(rows_r, threads)
        if r is not None:
            # the other arm's figure is rounds/s on the whole workload: the sample's rate scaled by the rows
            full = args.rounds_rows
            line["rounds"] = {"value": r * rows_r / full, "unit": "rounds/s", "depth": ROUNDS_DEPTH, "rows": full,
                              "features": ROUNDS_FEATURES, "sample_rows": rows_r, "sample_rounds_per_s": r,
                              "sample": "one round (BUILD_TREE + PREDICT of the reference's CPU code) on a %d-row sample of "
                                        "the %d x 64 workload, %d ranks (threads) on row shards without a collective; "
                                        "value = the sample's rounds/s x sample rows / all rows (the work is linear in "
                                        "the rows)" % (rows_r, full, threads)}
        r = cpu_predict_sample(rows_p, threads)
        if r is not None:
            line["predict"] = {"value": r, "unit": "rows/s", "rows": rows_p, "features": PREDICT_FEATURES,
                               "trees": PREDICT_TREES, "depth": PREDICT_DEPTH,
                               "sample": "%d-row sample of the 50M x 100 matrix, %d ranks (threads) on row shards"
                                         % (rows_p, threads)}
    print(json.dumps(line), flush=True)


def run_hist(args):
    import torch
    import torch.distributed as dist

    import legateboost_b200 as lb
    from legateboost_b200 import stages

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    ctx = lb.library.init_distributed(local)
    lib = ctx.lib
    n_rows = args.rows
    mode = 1 if args.float_path else 0
    bins, row_ptr, gpair, gpair_f, row_index, seg, node, max_abs = hist_inputs(torch, n_rows, 1 + rank, device)
    gp = gpair_f if mode else gpair
    hist = torch.empty((HIST_NODES, 1, HIST_FEATURES * HIST_BINS, 2),
                       dtype=torch.float64 if mode else torch.int64, device=device)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=device)  # > L2 (126 MB)

    lb.library.load().lbk_profile_enable(ctx.handle, 1)
    import ctypes as C

    by_pos = not args.pairs_by_row
    gp_by_row = gp
    if by_pos:
        # the pairs in row_index order, as the tree builder keeps them (its repartition moves them
        # together with the row ids); made once, outside the timed region
        gp = gp[row_index.long()].contiguous()

    # with several ranks the level's histograms are summed as the tree builder does it: every rank
    # ends with the sums of the bins of the features it owns (a reduce-scatter over NVLink)
    sum_mode = 2 if world > 1 else 0

    def step():
        stages.histogram(bins, row_ptr, gp, row_index, seg, HIST_FEATURES, mode=mode, hist=hist, ctx=ctx,
                         max_abs=max_abs if mode == 0 else None, all_reduce=sum_mode, max_bins=HIST_BINS,
                         total_bins=HIST_FEATURES * HIST_BINS, pairs_by_position=by_pos)

    # once, outside the timed region: the sums over the ranks against torch.distributed's all-reduce of
    # the local histograms, for the owned bins (the timed form) and for all bins (all_reduce = 1)
    allreduce_check = None
    if world > 1:
        kw = dict(mode=mode, ctx=ctx, max_abs=max_abs if mode == 0 else None, max_bins=HIST_BINS,
                  total_bins=HIST_FEATURES * HIST_BINS, pairs_by_position=by_pos)
        want = stages.histogram(bins, row_ptr, gp, row_index, seg, HIST_FEATURES, all_reduce=0, **kw).clone()
        dist.all_reduce(want)
        own = stages.histogram(bins, row_ptr, gp, row_index, seg, HIST_FEATURES, all_reduce=2, **kw).clone()
        full = stages.histogram(bins, row_ptr, gp, row_index, seg, HIST_FEATURES, all_reduce=1, **kw)
        f0, f1 = lb.library.owned_features(rank, world, HIST_FEATURES)
        lo, hi = f0 * HIST_BINS, f1 * HIST_BINS
        if mode == 0:
            good = bool(torch.equal(own[:, :, lo:hi], want[:, :, lo:hi])) and bool(torch.equal(full, want))
        else:
            tol = 1e-5 * float(want.abs().max())
            good = float((own[:, :, lo:hi] - want[:, :, lo:hi]).abs().max()) <= tol and \
                float((full - want).abs().max()) <= tol
        flag = torch.tensor([1 if good else 0], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        allreduce_check = "ok" if int(flag[0]) == 1 else "mismatch"
        del want, own, full

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        sampler.wait_for_first_sample()
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t_begin = time.perf_counter()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    kernel_ms = []
    for i in range(args.steps):
        flush.fill_(i & 0xFF)  # evict the inputs from L2 between timed iterations
        ev[i][0].record()
        step()
        ev[i][1].record()
        ms = C.c_float(0)
        ctx.check(lib.lbk_profile_histogram_ms(ctx.handle, C.byref(ms)))
        kernel_ms.append(ms.value)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t_end = time.perf_counter()
    total_ms = sum(a.elapsed_time(b) for a, b in ev)
    t = torch.tensor([total_ms, sum(kernel_ms)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, ksum = float(t[0]), float(t[1])
    # A short timed region sees few clock samples: the same steps go on, untimed, until about a
    # quarter of a second of this load has passed, so that nvidia-smi reports a handful of samples
    # under it.  The count comes from the reduced time, so every rank runs the same number (a
    # multi-rank step is collective).
    t_load = t_end
    if not args.no_clock_tail:
        n_tail = int(250.0 / max(total_ms / args.steps, 1e-3)) - args.steps
        for _ in range(max(0, min(n_tail, 1000))):
            step()
        torch.cuda.synchronize()
        t_load = time.perf_counter()
    clocks = sampler.stop(t_begin, t_end, t_load) if rank == 0 else None
    value = n_rows * HIST_FEATURES * world * args.steps / (total_ms * 1e-3)

    # end to end through the C ABI with host buffers (pinned), copies inside the timed region
    e2e = None
    if not args.no_e2e:
        hb = bins.cpu().pin_memory()
        hgp = gp_by_row.cpu().pin_memory()
        hidx = row_index.cpu().pin_memory()
        hseg = seg.cpu()
        hrp = row_ptr.cpu()
        hh = torch.empty(hist.shape, dtype=hist.dtype).pin_memory()
        n_e2e = max(2, min(args.steps, 5))
        for _ in range(2):
            stages.histogram(hb, hrp, hgp, hidx, hseg, HIST_FEATURES, mode=mode, hist=hh, ctx=ctx, host=True,
                             all_reduce=sum_mode)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            stages.histogram(hb, hrp, hgp, hidx, hseg, HIST_FEATURES, mode=mode, hist=hh, ctx=ctx, host=True,
                             all_reduce=sum_mode)
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {"value": n_rows * HIST_FEATURES * world * n_e2e / float(dt[0]), "unit": "row-features/s",
               "h2d_bytes_per_step": int(hb.numel() + hgp.numel() * hgp.element_size() + hidx.numel() * 4
                                         + hseg.numel() * 4 + hrp.numel() * 4),
               "d2h_bytes_per_step": int(hh.numel() * 8)}

    if rank == 0:
        peak, which = measured_peaks()
        kms = ksum / args.steps
        achieved = algorithmic_bytes(n_rows) / (kms * 1e-3) / 1e9
        # DRAM traffic of one launch: taken from the ncu capture summarised beside the kernel's profile
        # (bytes per row and bytes per launch of the case captured there), scaled by the rows
        traffic = hist_traffic(n_rows) if mode == 0 and world == 1 else None
        line = {
            "metric": "histogram rows*features/s", "value": value, "unit": "row-features/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32" if mode else "int32", "data": "synthetic",
            "config": {"workload": "histogram build, level 7 (128 nodes), %d rows x %d features x %d bins per GPU, "
                                   "%s gradient pairs%s" % (n_rows, HIST_FEATURES, HIST_BINS,
                                                            "float32" if mode else "quantised int32",
                                                            ", summed over the ranks by feature ownership (every rank "
                                                            "reads its features' bins from all ranks over NVLink)"
                                                            if world > 1 else ""),
                       "l2": "160 MB flush buffer written between timed steps; inputs (1.4 GB) exceed L2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_source": which, "kernel": "k_hist_smem", "kernel_ms": kms},
            "clocks": clocks, "e2e": e2e, "gpu_launches": (3 if world == 1 else 5) * args.steps,
        }
        # The kernel's other bound is the SM's load/store pipe: one shared-memory reduction instruction
        # (32 lanes, 32 different banks by construction of the layout) per 32 updates of a gradient
        # or hessian word, and the pipe retires at most one such pass per clock.  Rate = passes per
        # SM clock per SM over the kernel time, at the SM clock sampled under load.
        sm_mhz = clocks.get("sm_mhz") if isinstance(clocks, dict) else None
        if sm_mhz:
            passes = n_rows * HIST_FEATURES * 2 / 32
            sm_count = torch.cuda.get_device_properties(device).multi_processor_count
            rate = passes / (kms * 1e-3 * sm_mhz * 1e6 * sm_count)
            line["shared_atomics"] = {"updates_per_s": n_rows * HIST_FEATURES * 2 / (kms * 1e-3),
                                      "passes_per_clk_per_sm": rate, "peak": 1.0, "frac": rate,
                                      "note": "red.shared.add.s32 passes of 32 lanes; peak = one pass per clock per "
                                              "SM on the load/store pipe, which the row gathers share"}
        if allreduce_check is not None:
            line["allreduce_check"] = allreduce_check
        if not args.no_cpu and world == 1:
            threads = os.cpu_count() or 1
            v, dt, kind = cpu_hist_sample(5_000_000, 7, threads)
            line["cpu_baseline"] = {"value": v, "unit": "row-features/s", "cores": threads, "kind": kind,
                                    "sample": "one 5M-row sample of the batch, %d ranks (threads) on row shards "
                                              "(%.2f s, %.0f core-seconds); the reference's ComputeHistogram ends with "
                                              "its prefix scan (the GPU figure is the build alone); sources compiled "
                                              "with g++ -O2 against the runtime stand-in" % (threads, dt, dt * threads)}
    # the other two metrics of the path, on their own workloads (every rank takes part)
    extra = {}
    if not args.no_extra:
        del bins, gpair, gpair_f, gp, gp_by_row, row_index, seg, node, hist, flush
        torch.cuda.empty_cache()
        extra["rounds"] = rounds_section(torch, dist, lb, rank, world, device, args.rounds_rows, args.rounds, 1)
        extra["predict"] = predict_section(torch, dist, lb, rank, world, device, args.predict_rows, 2)
    if rank == 0:
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if allreduce_check == "mismatch":
        sys.exit(3)


def run_train(args):
    """Boosting rounds per second: squared error, Tree(max_depth=args.depth), 256 bins."""
    import torch
    import torch.distributed as dist

    import legateboost_b200 as lb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lb.library.init_distributed(local)
    gen = torch.Generator(device=device)
    gen.manual_seed(3 + rank)
    n, F = args.rows, args.features
    X = torch.rand((n, F), dtype=torch.float32, device=device, generator=gen)
    w = torch.randn(F, dtype=torch.float32, device=device, generator=torch.Generator(device=device).manual_seed(3))
    if args.classes > 1:
        # multi-output classification: labels = argmax of a noisy linear map of the first features
        # (all classes occur on every rank; the softmax objective has one output per class)
        c = args.classes
        X = torch.randn((n, F), dtype=torch.float32, device=device, generator=gen)
        W = torch.randn((min(F, c), c), dtype=torch.float32, device=device,
                        generator=torch.Generator(device=device).manual_seed(3))
        y = (X[:, : min(F, c)] @ W + 0.5 * torch.randn((n, c), dtype=torch.float32, device=device, generator=gen)).argmax(dim=1)
        make = lambda r: lb.LBClassifier(n_estimators=r, base_models=(lb.Tree(max_depth=args.depth),), random_state=0,  # noqa: E731
                                         fixed_sketch=args.fixed_sketch)
    else:
        y = X @ w + 0.1 * torch.randn(n, dtype=torch.float32, device=device, generator=gen)
        make = lambda r: lb.LBRegressor(n_estimators=r, base_models=(lb.Tree(max_depth=args.depth),), random_state=0,  # noqa: E731
                                        fixed_sketch=args.fixed_sketch)
    rounds = args.steps
    m = make(max(args.warmup, 1))
    m.fit(X, y)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    m = make(rounds)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    m.fit(X, y)
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = float(t[0])
        print(json.dumps({"metric": "boosting rounds/s", "value": rounds / (ms * 1e-3), "unit": "rounds/s",
                          "n_gpus": world, "steps": rounds, "warmup": max(args.warmup, 1), "ms_per_step": ms / rounds,
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int32",
                          "data": "synthetic",
                          "config": {"workload": "%s boosting, depth %d, 256 bins, %d rows x %d features per GPU%s"
                                                 % ("%d-class log-loss" % args.classes if args.classes > 1 else "squared-error",
                                                    args.depth, n, F, ", proposals and bins of the first tree reused "
                                                    "(not the reference's per-tree sketch)" if args.fixed_sketch else "")}}),
              flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_predict(args):
    import torch

    from legateboost_b200.tree import predict_arrays

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(4)
    n, F, T, D = args.rows, args.features, args.trees, args.depth
    X = torch.rand((n, F), dtype=torch.float32, device=device, generator=gen)
    M = 2 ** (D + 1) - 1
    trees = []
    for _ in range(T):
        feat = torch.randint(0, F, (M,), dtype=torch.int32, device=device, generator=gen)
        feat[2 ** D - 1:] = -1
        trees.append((torch.randn((M, 1), dtype=torch.float64, device=device, generator=gen), feat,
                      torch.rand((M,), dtype=torch.float64, device=device, generator=gen)))
    for _ in range(max(args.warmup, 1)):
        predict_arrays(X, trees)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        predict_arrays(X, trees)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    peak, which = measured_peaks()
    gbs = n * (F * 4 + 8) / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "predict rows/s", "value": n / (ms * 1e-3), "unit": "rows/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
                      "dtype": "f64", "data": "synthetic",
                      "config": {"workload": "%d trees depth %d, %d rows x %d features" % (T, D, n, F)},
                      "node_visits_per_s": n * T * D / (ms * 1e-3),
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                   "peak_source": which}}), flush=True)


def run_update(args):
    """UPDATE_TREE rows per second: one tree of depth args.depth grown on the data, then updated
    with new gradients (the structure stays).  Algorithmic bytes per row: F * 4 (X) + 16 (g, h)."""
    import numpy as np
    import torch

    import legateboost_b200 as lb

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(6)
    n, F, D = args.rows, args.features, args.depth
    X = torch.rand((n, F), dtype=torch.float32, device=device, generator=gen)
    g = torch.randn((n, 1), dtype=torch.float64, device=device, generator=gen)
    h = torch.ones((n, 1), dtype=torch.float64, device=device)
    t = lb.Tree(max_depth=D).set_random_state(np.random.RandomState(0)).fit(X, g, h)
    g2 = torch.randn((n, 1), dtype=torch.float64, device=device, generator=gen)
    for _ in range(max(args.warmup, 1)):
        t.update(X, g2, h)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        t.update(X, g2, h)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    peak, which = measured_peaks()
    gbs = n * (F * 4 + 16) / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "update_tree rows/s", "value": n / (ms * 1e-3), "unit": "rows/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
                      "dtype": "f64", "data": "synthetic",
                      "config": {"workload": "update of one tree of depth %d, %d rows x %d features" % (D, n, F)},
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                   "peak_source": which}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="hist", choices=["hist", "train", "predict", "update"])
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--features", type=int, default=64)
    ap.add_argument("--depth", type=int, default=8)
    ap.add_argument("--trees", type=int, default=500)
    ap.add_argument("--classes", type=int, default=1, help="train workload: > 1 = classification with that many classes")
    ap.add_argument("--float-path", action="store_true")
    ap.add_argument("--fixed-sketch", action="store_true",
                    help="train workload: reuse the first tree's proposals and bins (an extension; results differ "
                         "from the reference's)")
    ap.add_argument("--pairs-by-row", action="store_true",
                    help="hist workload: gradient pairs indexed by row id (gathered) instead of stored in "
                         "row_index order")
    ap.add_argument("--no-extra", action="store_true",
                    help="hist workload: leave the rounds/s and predict rows/s sections out of the line")
    ap.add_argument("--no-clock-tail", action="store_true", help="do not run untimed steps after the timed region for clock samples")
    ap.add_argument("--rounds-rows", type=int, default=ROUNDS_TOTAL_ROWS)
    ap.add_argument("--rounds", type=int, default=5)
    ap.add_argument("--predict-rows", type=int, default=PREDICT_TOTAL_ROWS)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "hist":
        args.rows = args.rows or HIST_ROWS
        return run_hist(args)
    if args.workload == "train":
        args.rows = args.rows or 10_000_000
        return run_train(args)
    if args.workload == "update":
        args.rows = args.rows or 10_000_000
        return run_update(args)
    args.rows = args.rows or 5_000_000
    return run_predict(args)


if __name__ == "__main__":
    main()

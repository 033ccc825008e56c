#!/usr/bin/env python
"""Benchmark of the sparse-aggregation hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the path over the workload's graph: Y = Â·H (the forward
aggregation of a GraphSum layer).  Rank 0 prints ONE JSON line.  Throughput is in
nnz·F per second (one multiply-add per stored nonzero per feature).  The K steps are
timed as one block between CUDA events; the block is repeated until half a second has
been timed and the median block is reported.

Workloads (all synthetic, seeded):
  c2       R-MAT scale 20, edge factor 16, symmetrised, +I, F=64   (single-GPU headline)
  rmat22   R-MAT scale 22, edge factor 16, directed, +I, F=32
  rmat26   R-MAT scale 26, edge factor 16, directed, +I, F=32
  custom   --scale/--edge-factor/--features/--symmetrise

Several GPUs (one process per GPU under torchrun): the graph is EBV-partitioned on rank 0 and handed out; a step is
the local aggregation plus the mirror/master exchange.  --scaling weak (default: scale + log2 N) | strong,
--exchange p2p|nccl|dense, --pipeline-groups G (0 = measure 1, 2 and 4 groups and keep the fastest).

Beside the headline the line carries sections (--sections a,b,... or "all" / "none"):
  one GPU:      parity, cusparse, e2e, rmat26, gcn_epoch, gcn_c4, pagerank, minprop, jobs, cpu
  several GPUs: parity, gcn_epoch, gcn_c4, strong, e2e
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

WORKLOADS = {
    "c2": dict(scale=20, edge_factor=16, features=64, symmetrise=True, seed=20261127),
    "rmat26": dict(scale=26, edge_factor=16, features=32, symmetrise=False, seed=20261130),
    "rmat24": dict(scale=24, edge_factor=16, features=32, symmetrise=False, seed=20261132),
    "rmat22": dict(scale=22, edge_factor=16, features=32, symmetrise=False, seed=20261131),
    # the aggregation alone on the graph of the GCN configuration c3 (Reddit-shaped), at its hidden width
    "c3": dict(kind="powerlaw", vertices=232965, pairs=57_200_000, features=128, seed=20261203),
}

# the GCN configurations: vertices, undirected pairs drawn, layer widths (input, hidden..., classes)
GCN_CONFIGS = {
    "c3": dict(vertices=232965, pairs=57_200_000, dims=[602, 128, 41], seed=20261203,
               descr="Reddit-shaped power-law graph, 2 layers 602-128-41"),
    "c4": dict(vertices=2449029, pairs=61_900_000, dims=[100, 256, 256, 47], seed=20261204,
               descr="products-shaped power-law graph, 3 layers 100-256-256-47"),
}

SECTIONS_ONE = ["parity", "cusparse", "e2e", "rmat26", "gcn_epoch", "gcn_c4", "pagerank", "minprop", "jobs", "cpu"]
SECTIONS_MULTI = ["parity", "gcn_epoch", "gcn_c4", "strong", "e2e"]
MIN_TIMED_SECONDS = 0.5


def measured_traffic(workload):
    """DRAM bytes of one aggregation call from the ncu capture recorded under profiles/ for this workload (written by
    `bench.py --record-traffic`), with the commit it was taken at; None when there is no record."""
    path = os.path.join(ROOT, "profiles", "spmm_%s_dram_traffic.txt" % workload)
    if not os.path.exists(path):
        return None, None
    rec = {}
    for line in open(path):
        if ":" in line and not line.startswith("#"):
            k, v = line.split(":", 1)
            rec[k.strip()] = v.strip()
    try:
        return float(rec["dram_bytes_per_call"]), rec.get("commit")
    except (KeyError, ValueError):
        return None, None


def record_traffic(csv_path, workload):
    """Turns the CSV of `ncu --metrics gpu__time_duration.sum,dram__bytes_read.sum,dram__bytes_write.sum --csv` taken
    over whole aggregation calls of `bench.py --workload <workload>` into profiles/spmm_<workload>_dram_traffic.txt."""
    import csv
    import subprocess
    per_kernel, calls = {}, 0
    with open(csv_path) as fh:
        rows = [r for r in csv.reader(l for l in fh if not l.startswith("==")) if len(r) > 5]
    head = next(r for r in rows if "Metric Name" in r)
    ki, mi, vi, ui = head.index("Kernel Name"), head.index("Metric Name"), head.index("Metric Value"), head.index("Metric Unit")
    for r in rows:
        if r is head or len(r) <= vi or not r[mi].startswith("dram__bytes"):
            continue
        mult = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}.get(r[ui], 1.0)
        name = r[ki].split("(")[0].split("<")[0]
        per_kernel.setdefault(name, [0.0, 0])
        per_kernel[name][0] += float(r[vi].replace(",", "")) * mult
        if r[mi] == "dram__bytes_read.sum":
            per_kernel[name][1] += 1
    calls = max(1, max((c for n, (b, c) in per_kernel.items() if "chunks" in n), default=1))
    total = sum(b for b, c in per_kernel.values()) / calls
    commit = subprocess.run(["git", "-C", ROOT, "rev-parse", "--short", "HEAD"], capture_output=True, text=True).stdout.strip()
    out = os.path.join(ROOT, "profiles", "spmm_%s_dram_traffic.txt" % workload)
    with open(out, "w") as fh:
        fh.write("# dram__bytes_read.sum + dram__bytes_write.sum of the kernels of ONE aggregation call, from an ncu capture\n")
        fh.write("# of `python bench.py --workload %s --sections none` (see the profile summary of the same workload).\n" % workload)
        fh.write("workload: %s\ncalls_captured: %d\ndram_bytes_per_call: %.6e\ncommit: %s\n" % (workload, calls, total, commit or "unknown"))
        for n, (b, c) in sorted(per_kernel.items()):
            fh.write("kernel %s: %.6e bytes over %d launches\n" % (n, b, c))
    print("wrote", out)


def parse_args():
    global MIN_TIMED_SECONDS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--scale", type=int)
    ap.add_argument("--edge-factor", type=int, default=16)
    ap.add_argument("--features", type=int)
    ap.add_argument("--symmetrise", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--sections", default="all", help='comma-separated section names, "all" or "none"')
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cusparse", action="store_true")
    ap.add_argument("--no-gcn", action="store_true", help="leave out gcn_epoch, gcn_c4, pagerank, minprop, jobs, rmat26")
    ap.add_argument("--no-fused-push", action="store_true",
                    help="peer-memory transport: send mirror rows with the exchange's copy kernel after the aggregation "
                         "instead of from the aggregation's store")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl", "dense"],
                    help="transport of the mirror/master exchange on several GPUs")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="several GPUs: weak = the graph grows with the GPU count (default), strong = the named graph is cut")
    ap.add_argument("--pipeline-groups", type=int, default=0,
                    help="several GPUs: aggregate and exchange the rows in this many groups, group g's exchange "
                         "overlapping group g+1's aggregation (1 = aggregation, then exchange; 0 = time 1, 2 and 4 "
                         "and keep the fastest)")
    ap.add_argument("--pagerank-iters", type=int, default=0,
                    help="also time this many PageRank power iterations (F=1) over the workload's graph / partition")
    ap.add_argument("--strong-workload", default="auto", help="several GPUs, section strong: rmat26 | rmat24 | auto")
    ap.add_argument("--min-timed-seconds", type=float, default=MIN_TIMED_SECONDS,
                    help="repeat the block of --steps steps until this much has been timed (0: one block; for profiler runs)")
    ap.add_argument("--record-traffic", metavar="CSV", help="write profiles/spmm_<workload>_dram_traffic.txt from an ncu CSV and exit")
    args = ap.parse_args()
    names = SECTIONS_ONE + SECTIONS_MULTI
    if args.sections == "all":
        chosen = set(names)
    elif args.sections == "none":
        chosen = set()
    else:
        chosen = set(x for x in args.sections.split(",") if x)
        bad = chosen - set(names)
        if bad:
            ap.error("unknown section(s): %s" % ", ".join(sorted(bad)))
    if args.no_cpu_baseline:
        chosen.discard("cpu")
    if args.no_cusparse:
        chosen.discard("cusparse")
    if args.no_gcn:
        chosen -= {"gcn_epoch", "gcn_c4", "pagerank", "minprop", "jobs", "rmat26", "strong"}
    args.chosen = chosen
    MIN_TIMED_SECONDS = args.min_timed_seconds
    return args


def workload_config(args):
    if args.workload == "custom":
        cfg = dict(scale=args.scale, edge_factor=args.edge_factor, features=args.features,
                   symmetrise=args.symmetrise, seed=20261199)
    else:
        cfg = dict(WORKLOADS[args.workload])
        if args.features:
            cfg["features"] = args.features
    # weak scaling: the graph doubles with the GPU count, so every EBV part keeps the single-GPU edge count
    n = max(args.gpus, 1)
    if args.scaling == "weak" and "scale" in cfg:
        cfg["scale"] += max(n.bit_length() - 1, 0)
    return cfg


def build_graph(cfg, device):
    """CSR by source, global degrees (int32 tensors on `device`)."""
    from drone_b200 import graphgen as gg
    if cfg.get("kind") == "powerlaw":
        n, u, v = gg.powerlaw_graph(cfg["vertices"], cfg["pairs"], seed=cfg["seed"], device=device)
        index, dst = gg.csr_by_source(u, v, n)
        in_deg, out_deg = gg.degrees(u, v, n)
        return n, index, dst, in_deg, out_deg
    n, u, v = gg.rmat_graph(cfg["scale"], cfg["edge_factor"], seed=cfg["seed"], device=device,
                            symmetrise=cfg["symmetrise"], self_loops="add")
    index, dst = gg.csr_by_source(u, v, n)
    in_deg, out_deg = gg.degrees(u, v, n)
    del u, v
    return n, index, dst, in_deg, out_deg


def algorithmic_bytes(n, nnz, f):
    """Each array touched once: int32 index + fp32 value per nonzero, row pointers, H read, Y written."""
    return 8 * nnz + 4 * (n + 1) + 8 * n * f


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index=0, period=0.004):
        super().__init__(daemon=True)
        self.period = period
        self.samples = []
        self.timed_samples = 0
        self.in_timed_region = True
        self.reasons = set()
        self.stop_flag = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception as e:  # no NVML: report that instead of clocks
            self.err = repr(e)

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self.stop_flag.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                if self.in_timed_region:
                    self.timed_samples += 1
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def keep_loaded(self, step, seconds=0.4):
        """The timed region lasts a few milliseconds, shorter than NVML's refresh; repeat the identical loop for a
        moment (untimed) so that the clock record covers the GPU under this load."""
        self.in_timed_region = False
        t0 = time.perf_counter()
        i = 0
        while time.perf_counter() - t0 < seconds:
            step(i)
            i += 1
            if i % 16 == 0:
                torch.cuda.synchronize()
        torch.cuda.synchronize()

    def finish(self):
        self.stop_flag.set()
        if self.is_alive():
            self.join(timeout=2)
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "NVML unavailable: " + self.err}
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": float(self.max_mhz), "reasons": sorted(self.reasons),
                "samples": len(self.samples), "samples_in_timed_region": self.timed_samples,
                "note": "sampled through the timed region and an untimed 0.4 s repeat of the same loop"}


def cpu_spmm_baseline(index, dst, val, f, seed, budget_s=12.0):
    """Times the oracle's float CSR product on all host threads (bounded: whole workload, few repeats)."""
    from oracle import oracle
    oracle.build()
    n = len(index) - 1
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, f), dtype=np.float32)
    y = np.empty((n, f), np.float32)
    threads = oracle.max_threads()
    oracle.spmm_csr_f32(index, dst, val, x, threads=threads, out=y)  # warm-up / page-in
    times = []
    t_start = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_start < budget_s and len(times) < 20):
        t0 = time.perf_counter()
        oracle.spmm_csr_f32(index, dst, val, x, threads=threads, out=y)
        times.append(time.perf_counter() - t0)
    return times, threads


def run_reference(args, cfg):
    """The path on the host cores: the oracle's OpenMP CSR product (the reference's own CPU job is a Go
    program that cannot be built here; its GPU path needs cuSPARSE, which is timed separately)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    device = torch.device("cuda:0") if torch.cuda.is_available() else torch.device("cpu")
    n, index, dst, in_deg, out_deg = build_graph(cfg, device)
    from oracle import oracle
    oracle.build()
    index_h, dst_h = index.cpu().numpy(), dst.cpu().numpy()
    val = oracle.csr_values_f32(index_h, dst_h, in_deg.cpu().numpy(), out_deg.cpu().numpy())
    nnz, f = len(dst_h), cfg["features"]
    rng = np.random.default_rng(cfg["seed"])
    x = rng.standard_normal((n, f), dtype=np.float32)
    y = np.empty((n, f), np.float32)
    threads = oracle.max_threads()
    for _ in range(max(args.warmup, 1)):
        oracle.spmm_csr_f32(index_h, dst_h, val, x, threads=threads, out=y)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.spmm_csr_f32(index_h, dst_h, val, x, threads=threads, out=y)
    dt = time.perf_counter() - t0
    value = args.steps * nnz * f / dt
    line = {
        "impl": "reference", "metric": "spmm_nnzF_per_s", "value": value, "unit": "nnz*F/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_descr(args, cfg, n, nnz),
        "cpu_baseline": {"value": value, "unit": "nnz*F/s", "cores": threads, "kind": "port",
                         "sample": "whole workload, one CSR SpMM per step, all host threads (OpenMP row-parallel)"},
        "e2e": {"value": value, "unit": "nnz*F/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_descr(args, cfg, n, nnz):
    if cfg.get("kind") == "powerlaw":
        what = "%s: power-law graph, %d vertices, symmetrised +I, Y = A_hat * H, F=%d" % (args.workload, n, cfg["features"])
    else:
        what = "%s: R-MAT scale %d ef %d%s +I, Y = A_hat * H, F=%d" % (
            args.workload, cfg["scale"], cfg["edge_factor"], " symmetrised" if cfg["symmetrise"] else " directed",
            cfg["features"])
    return {"workload": what, "vertices": n, "nnz": nnz, "features": cfg["features"],
        "l2_policy": "operands rotate over 3 buffer sets; CSR + H + Y exceed the 126 MB L2"}


def time_blocks(step, steps, sync, min_seconds=None, max_blocks=400):
    """Times blocks of exactly `steps` calls of step(i) between two CUDA events on the current stream, block after
    block until min_seconds have been timed (at least one block).  sync() is called on both sides of every block (device
    synchronisation, plus a barrier on several GPUs).  Returns the list of block times in ms."""
    if min_seconds is None:
        min_seconds = MIN_TIMED_SECONDS
    min_seconds = min(min_seconds, MIN_TIMED_SECONDS)
    blocks, total = [], 0.0
    i = 0
    while len(blocks) < max_blocks and (not blocks or total < min_seconds * 1e3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        e0.record()
        for _ in range(steps):
            step(i)
            i += 1
        e1.record()
        sync()
        blocks.append(e0.elapsed_time(e1))
        total += blocks[-1]
    return blocks


def hbm_peak():
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        return float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def small_case_parity(device):
    """The library against the double-precision oracle on a seeded R-MAT-13 graph, both orientations, F = 32 and 41:
    largest error relative to the largest element of the result."""
    import drone_b200 as db
    from drone_b200 import graphgen as gg
    from oracle import oracle
    oracle.build()
    n, u, v = gg.rmat_graph(13, 16, seed=20261141, symmetrise=False, self_loops="add")
    index, dst = gg.csr_by_source(u, v, n)
    in_deg, out_deg = gg.degrees(u, v, n)
    plan = db.AggregationPlan(index.to(device), dst.to(device), in_degree=in_deg.to(device), out_degree=out_deg.to(device))
    val = oracle.csr_values_f32(index.numpy(), dst.numpy(), in_deg.numpy(), out_deg.numpy())
    worst = 0.0
    for f in (32, 41):
        x = gg.seeded_normal(f, (n, f))
        xt = torch.as_tensor(x, device=device)
        for op, want in ((db.OP_AT, oracle.graphsum_forward_f64(x, index.numpy(), dst.numpy(), val)),
                         (db.OP_A, oracle.graphsum_backward_f64(x, index.numpy(), dst.numpy(), val))):
            got = plan.spmm(op, xt).cpu().numpy()
            worst = max(worst, float(np.abs(got - want).max() / np.abs(want).max()))
    plan.close()
    return worst


def run_ours(args, cfg):
    import drone_b200 as db
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the aggregation path has no CPU fallback")
    if world > 1:
        return run_ours_multi(args, cfg)
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    lib = db.lib()
    chosen = args.chosen

    n, index, dst, in_deg, out_deg = build_graph(cfg, device)
    nnz, f = dst.numel(), cfg["features"]
    plan = db.AggregationPlan(index, dst, in_degree=in_deg, out_degree=out_deg, orientations=db.PLAN_AT)
    plan.reserve(f, host_operands="e2e" in chosen)
    st = plan.stats()
    nbuf = 3
    gen = torch.Generator(device=device)
    gen.manual_seed(cfg["seed"])
    xs = [torch.randn((n, f), device=device, generator=gen) for _ in range(nbuf)]
    ys = [torch.empty((n, f), device=device) for _ in range(nbuf)]

    def step(i):
        plan.spmm(db.OP_AT, xs[i % nbuf], out=ys[i % nbuf])

    warmup = max(args.warmup, 3)
    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()

    sampler = ClockSampler(index=local_rank)
    sampler.start()
    launches0 = lib.drone_kernel_launch_count()
    blocks = time_blocks(step, args.steps, torch.cuda.synchronize)
    launches = (lib.drone_kernel_launch_count() - launches0) // len(blocks)
    sampler.in_timed_region = False
    clocks = sampler.finish()

    block_ms = float(np.median(blocks))
    ms = block_ms / args.steps
    value = nnz * f / (ms * 1e-3)
    b_alg = algorithmic_bytes(n, nnz, f)
    peak, peak_src = hbm_peak()
    achieved = b_alg / (ms * 1e-3) / 1e9
    traffic, traffic_commit = (None, None)
    if cfg == dict(WORKLOADS.get(args.workload, {})):
        traffic, traffic_commit = measured_traffic(args.workload)

    line = {
        "metric": "spmm_nnzF_per_s", "value": value, "unit": "nnz*F/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_descr(args, cfg, n, nnz),
        "timed_blocks": len(blocks), "timed_ms_total": float(np.sum(blocks)),
        "ms_per_step_min_block": float(np.min(blocks)) / args.steps,
        "ms_per_step_max_block": float(np.max(blocks)) / args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "traffic_commit": traffic_commit, "peak_source": peak_src,
                     "algorithmic_bytes": b_alg,
                     "kernel": "one drone_spmm call = spmm_short_stream + spmm_chunks + spmm_reduce_partials"},
        "gpu_launches": int(launches), "clocks": clocks,
        "plan": {"short_row_limit": st.short_row_limit, "chunk_nnz": st.chunk_nnz,
                 "long_rows": st.n_long_rows[1], "chunks": st.n_chunks[1], "split_rows": st.n_split_rows[1],
                 "partials": st.n_partials[1]},
    }

    if "e2e" in chosen:
        # end to end: host operands through the C ABI, copies inside the timed region.  Two measurements: a series of
        # calls through the library's queue (two in flight, every call with its own operands in and result out), and
        # one synchronous call at a time.
        xh = [torch.empty((n, f), dtype=torch.float32).pin_memory() for _ in range(2)]
        yh = [torch.empty((n, f), dtype=torch.float32).pin_memory() for _ in range(2)]
        for b in range(2):
            xh[b].copy_(xs[b])
        plan.spmm_host(db.OP_AT, xh[0], yh[0])
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            plan.spmm_host(db.OP_AT, xh[0], yh[0])
        single_s = (time.perf_counter() - t0) / args.e2e_steps
        single_diff = float((yh[0][:65536] - plan.spmm(db.OP_AT, xs[0])[:65536].cpu()).abs().max() / yh[0][:65536].abs().max())

        def series(steps):
            tickets = []
            for i in range(steps):
                tickets.append(plan.spmm_host_submit(db.OP_AT, xh[i % 2], yh[i % 2]))
                if i >= 1:
                    plan.spmm_host_wait(tickets[i - 1])     # the host consumes result i-1 while call i is in flight
            plan.spmm_host_wait(tickets[-1])
        series(4)
        q_steps = max(args.e2e_steps, 10) * 2
        t0 = time.perf_counter()
        series(q_steps)
        e2e_s = (time.perf_counter() - t0) / q_steps
        queue_diff = max(float((yh[b][:65536] - plan.spmm(db.OP_AT, xs[b])[:65536].cpu()).abs().max() / yh[b][:65536].abs().max())
                         for b in range(2))
        line["e2e"] = {"value": nnz * f / e2e_s, "unit": "nnz*F/s", "h2d_bytes_per_step": 4 * n * f,
                       "d2h_bytes_per_step": 4 * n * f, "ms_per_step": 1e3 * e2e_s, "steps": q_steps,
                       "checksum": float(yh[0][:1024].double().sum()),
                       "max_rel_diff_vs_device_call": queue_diff,
                       "how": "a series of drone_spmm_host_submit / drone_spmm_host_wait calls on pinned operands (two "
                              "alternating operand sets, at most two calls in flight): every call copies its own X in and "
                              "its own Y out; the copy in of call k, the aggregation of call k-1 and the copy out of call "
                              "k-2 overlap, so PCIe carries both directions at once.  Wall clock from the first submit to "
                              "the last wait, pipeline fill included",
                       "single_call": {"ms_per_step": 1e3 * single_s, "value": nnz * f / single_s, "steps": args.e2e_steps,
                                       "max_rel_diff_vs_device_call": single_diff,
                                       "how": "one synchronous drone_spmm_host call at a time: two column halves, the second "
                                              "half's copy in and the first half's result rows (stored by the kernels "
                                              "straight into the pinned output) cross PCIe in opposite directions"}}
        del xh, yh

    parity = {}
    if "parity" in chosen:
        try:
            parity["oracle_rmat13_max_rel_err"] = small_case_parity(device)
        except Exception as e:
            parity["oracle_error"] = repr(e)
        try:      # and the timed workload itself, at full size, through its column sums
            plan.spmm(db.OP_AT, xs[0], out=ys[0])
            torch.cuda.synchronize()
            parity["checksum_identity"] = checksum_report(
                *checksum_terms(plan, db.OP_AT, xs[0], ys[0]),
                "column sums of Y against (sum of the stored coefficients per gathered row)^T X, in double, relative to "
                "the sum of the absolute terms; the whole %d x %d result of the timed workload" % (n, f))
        except Exception as e:
            parity["checksum_identity"] = {"error": repr(e)}

    if "cusparse" in chosen:
        try:
            from baseline import cusparse_ref
            rp, co, va = plan.csr(db.OP_AT)
            res = {}
            for alg, name in ((0, "ALG_DEFAULT"), (2, "CSR_ALG2"), (3, "CSR_ALG3")):
                y_ref = torch.empty_like(ys[0])
                ref = cusparse_ref.CusparseSpmm(rp, co, va, xs[0], y_ref, alg=alg)
                for _ in range(3):
                    ref.run()
                torch.cuda.synchronize()
                if alg == 0:       # same operands, same call the reference makes: largest difference to this library
                    y_ours = plan.spmm(db.OP_AT, xs[0])
                    parity["cusparse_max_rel_diff"] = float((y_ours - y_ref).abs().max() / y_ref.abs().max())
                    parity["cusparse_workload"] = args.workload
                    del y_ours
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = max(3, min(args.steps, 10))
                e0.record()
                for _ in range(reps):
                    ref.run()
                e1.record()
                torch.cuda.synchronize()
                t = e0.elapsed_time(e1) / reps
                res[name] = {"ms": t, "nnzF_per_s": nnz * f / (t * 1e-3), "buffer_bytes": ref.buffer_bytes()}
                ref.close()
                del y_ref
            line["cusparse"] = res
            del rp, co, va
        except Exception as e:  # the head-to-head is informative, never fatal
            line["cusparse"] = {"error": repr(e)}
    if parity:
        parity["tolerance"] = 1e-5
        parity["ok"] = all(v <= 1e-5 for k, v in parity.items() if k.endswith("_err") or k.endswith("_diff")) and \
            bool(parity.get("checksum_identity", {"ok": True}).get("ok", False))
        line["parity"] = parity

    if args.pagerank_iters > 0:      # the path at F = 1 on the workload's own graph, for comparison with several GPUs
        try:
            line["pagerank_workload_graph"] = one_part_pagerank(device, n, index, dst, out_deg, args.pagerank_iters)
        except Exception as e:
            line["pagerank_workload_graph"] = {"error": repr(e)}

    cpu_csr = None
    if "cpu" in chosen:
        cpu_csr = [t.cpu().numpy() for t in plan.csr(db.OP_AT)]
    del xs, ys, plan, index, dst, in_deg, out_deg
    torch.cuda.empty_cache()

    def section(name, fn):
        if name not in chosen:
            return
        try:
            line[name] = fn()
        except Exception as e:
            line[name] = {"error": repr(e)}
        torch.cuda.empty_cache()

    section("rmat26", lambda: large_graph_timing(device, "rmat26"))
    section("gcn_epoch", lambda: gcn_epoch_timing(device, "c3", with_cusparse=True))
    section("gcn_c4", lambda: gcn_epoch_timing(device, "c4", with_cusparse=False))
    section("pagerank", lambda: pagerank_timing(device))
    section("minprop", lambda: minprop_timing(device))
    if "jobs" in chosen:
        line["jobs_head_to_head"] = jobs_head_to_head()

    if cpu_csr is not None:
        times, threads = cpu_spmm_baseline(cpu_csr[0], cpu_csr[1], cpu_csr[2], f, cfg["seed"])
        best = min(times)
        line["cpu_baseline"] = {"value": nnz * f / best, "unit": "nnz*F/s", "cores": threads, "kind": "port",
                                "sample": "whole workload, best of %d runs of the oracle's OpenMP float CSR SpMM"
                                          % len(times), "ms": 1e3 * best}
    print(json.dumps(line), flush=True)
    if parity and not parity.get("ok", True):
        raise SystemExit("bench.py: parity check failed: %r" % parity)


def checksum_terms(plan, op, x, y, own_rows=None):
    """A property of the product that needs no second implementation and no small graph: summed over its rows,
    Y = M X has the column sums  1^T Y = (M^T 1)^T X,  and M^T 1 (the sum of the stored coefficients per gathered
    row) comes straight from the plan's CSR arrays.  Returns three float64 vectors of length F: the sums of the rows of
    y (own_rows: only those rows), s^T x with s = M^T 1, and sum_u |s[u]| |x[u, :]| (the magnitude to judge the
    difference of the first two against).  On several GPUs the three are summed over the ranks before comparing."""
    _, col, val = plan.csr(op)
    n, f = x.shape
    s = torch.zeros(n, dtype=torch.float64, device=x.device)
    piece = 1 << 27
    for k0 in range(0, col.numel(), piece):
        s.index_add_(0, col[k0:k0 + piece].long(), val[k0:k0 + piece].double())
    del col, val
    want = torch.zeros(f, dtype=torch.float64, device=x.device)
    scale = torch.zeros(f, dtype=torch.float64, device=x.device)
    got = torch.zeros(f, dtype=torch.float64, device=x.device)
    rows = 1 << 21
    for r0 in range(0, n, rows):
        xb = x[r0:r0 + rows].double()
        sb = s[r0:r0 + rows, None]
        want += (sb * xb).sum(0)
        scale += (sb.abs() * xb.abs()).sum(0)
        yb = y[r0:r0 + rows]
        if own_rows is not None:
            yb = yb * own_rows[r0:r0 + rows, None]
        got += yb.sum(0, dtype=torch.float64)
    return got, want, scale


def checksum_report(got, want, scale, what):
    # Rounding of the float32 sums averages out over the rows (measured: 4e-12 .. 7e-11); one row lost, doubled or
    # left unwritten moves a column sum by about 1 / rows (1.5e-8 on the largest graph).  1e-9 separates the two.
    rel = float(((got - want).abs() / scale.clamp_min(1e-300)).max())
    if rel != rel:      # a rank could not form its terms
        return {"max_rel_diff": None, "tolerance": 1e-9, "ok": False, "what": what}
    return {"max_rel_diff": rel, "tolerance": 1e-9, "ok": bool(rel <= 1e-9), "what": what}


def large_graph_timing(device, workload, steps=10):
    """The aggregation on one of the large directed R-MAT graphs (the workload the roofline target is stated on),
    one GPU, device-resident operands rotating over two buffer sets; plus 20 PageRank power iterations (F = 1) on the
    same graph."""
    import drone_b200 as db
    cfg = dict(WORKLOADS[workload])
    n, index, dst, in_deg, out_deg = build_graph(cfg, device)
    nnz, f = dst.numel(), cfg["features"]
    plan = db.AggregationPlan(index, dst, in_degree=in_deg, out_degree=out_deg, orientations=db.PLAN_AT)
    plan.reserve(f)
    gen = torch.Generator(device=device)
    gen.manual_seed(cfg["seed"])
    xs = [torch.randn((n, f), device=device, generator=gen) for _ in range(2)]
    ys = [torch.empty((n, f), device=device) for _ in range(2)]

    def step(i):
        plan.spmm(db.OP_AT, xs[i % 2], out=ys[i % 2])
    for i in range(3):
        step(i)
    blocks = time_blocks(step, steps, torch.cuda.synchronize)
    ms = float(np.median(blocks)) / steps
    b_alg = algorithmic_bytes(n, nnz, f)
    peak, peak_src = hbm_peak()
    out = {"workload": "%s: R-MAT scale %d ef %d directed +I, F=%d" % (workload, cfg["scale"], cfg["edge_factor"], f),
           "vertices": n, "nnz": nnz, "ms_per_step": ms, "steps": steps, "timed_blocks": len(blocks),
           "nnzF_per_s": nnz * f / (ms * 1e-3), "algorithmic_bytes": b_alg,
           "algorithmic_GBps": b_alg / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": b_alg / (ms * 1e-3) / 1e9 / peak,
           "peak": peak, "peak_source": peak_src, "hot_row_table": bool(plan.stats().hot_rows_tagged)}
    try:      # the full-size result, checked through its column sums
        step(0)
        torch.cuda.synchronize()
        out["checksum_identity"] = checksum_report(
            *checksum_terms(plan, db.OP_AT, xs[0], ys[0]),
            "column sums of Y against (sum of the stored coefficients per gathered row)^T X, in double, relative to "
            "the sum of the absolute terms; the whole %d x %d result" % (n, f))
    except Exception as e:
        out["checksum_identity"] = {"error": repr(e)}
    del xs, ys
    plan.close()
    torch.cuda.empty_cache()
    out["pagerank"] = one_part_pagerank(device, n, index, dst, out_deg, 20)
    return out


from drone_b200.graphgen import glorot_weights, hashed_labels, hashed_normal  # noqa: E402


def time_epochs(step, epochs, sync):
    """ms per epoch of broadcast + forward + backward + gradient reduce, events around `epochs` of them."""
    def one(_):
        step.broadcast_weights()
        step.forward()
        step.backward()
        step.reduce_gradients()
    for i in range(2):
        one(i)
    blocks = time_blocks(one, epochs, sync)
    return float(np.median(blocks)) / epochs, len(blocks)


def gcn_epoch_timing(device, cfg_name, with_cusparse, epochs=5):
    """Forward + backward of the GCN of configuration `cfg_name` on one GPU: once with this library's aggregation
    (ReLU in the aggregation's store), once with the ReLU as a pass of its own, and (with_cusparse) once with cuSPARSE
    called as the reference calls it; the dense layers are the same cuBLAS calls in every arm."""
    import drone_b200 as db
    from drone_b200 import gcn, graphgen as gg
    cfg = GCN_CONFIGS[cfg_name]
    dims = cfg["dims"]
    n, u, v = gg.powerlaw_graph(cfg["vertices"], cfg["pairs"], seed=cfg["seed"], device=device)
    index, dst = gg.csr_by_source(u, v, n)
    in_deg, out_deg = gg.degrees(u, v, n)
    del u, v

    class G:
        pass
    g = G()
    g.plan = db.AggregationPlan(index, dst, in_degree=in_deg, out_degree=out_deg)
    g.plan.reserve(max(dims[1:]), padded_rows=True)
    g.mirror2worker = None
    ids = np.arange(n)
    x = hashed_normal(ids, dims[0], 7, device)
    truth = hashed_labels(ids, dims[-1], 7, device)
    weights = glorot_weights(dims, device)
    torch.backends.cuda.matmul.allow_tf32 = False
    out = {"config": cfg["descr"], "vertices": n, "nnz": int(dst.numel()), "dims": dims, "epochs_per_block": epochs}

    step = gcn.GCN(g, x, truth, weights, fuse_relu=True)
    out["ms_drone_b200"], out["timed_blocks"] = time_epochs(step, epochs, torch.cuda.synchronize)
    loss_ours = float(step.loss)
    out["loss"] = loss_ours
    unfused = gcn.GCN(g, x, truth, weights, fuse_relu=False)
    out["ms_drone_b200_relu_as_own_pass"], _ = time_epochs(unfused, epochs, torch.cuda.synchronize)
    out["loss_rel_diff_fused_vs_own_pass"] = abs(float(unfused.loss) - loss_ours) / max(abs(loss_ours), 1e-30)
    del unfused

    # aggregation alone: every GraphSum call of one epoch, both orientations, at the widths of this model
    def aggregations(_):
        for l in range(step.n_layers):
            g.plan.spmm(db.OP_AT, step.h[l], out=step.z[l])
        for l in range(step.n_layers - 1, -1, -1):
            g.plan.spmm(db.OP_A, step.d_logits if l == step.n_layers - 1 else step.d_a[l], out=step.d_h[l])
    blocks = time_blocks(aggregations, epochs, torch.cuda.synchronize)
    agg_ms = float(np.median(blocks)) / epochs
    nnz = int(dst.numel())
    b_alg = sum(2 * algorithmic_bytes(n, nnz, d) for d in dims[1:])
    peak, _ = hbm_peak()
    out["aggregation_only"] = {"ms": agg_ms, "calls": 2 * step.n_layers, "algorithmic_bytes": b_alg,
                               "algorithmic_GBps": b_alg / (agg_ms * 1e-3) / 1e9,
                               "frac_of_hbm_peak": b_alg / (agg_ms * 1e-3) / 1e9 / peak}
    per_width = {}
    for d in sorted(set(dims[1:])):
        xs = [torch.randn((n, d), device=device) for _ in range(2)]
        ys = [torch.empty((n, d), device=device) for _ in range(2)]
        blocks = time_blocks(lambda i: g.plan.spmm(db.OP_AT, xs[i % 2], out=ys[i % 2]), 5, torch.cuda.synchronize, 0.1)
        per_width["F=%d" % d] = float(np.median(blocks)) / 5
        del xs, ys
    out["aggregation_ms_by_width"] = per_width

    if with_cusparse:
        try:
            from baseline import cusparse_ref
            csr = {db.OP_A: g.plan.csr(db.OP_A), db.OP_AT: g.plan.csr(db.OP_AT)}
            cache = {}

            def cusparse_aggregate(op, src, dst_t):
                key = (op, src.data_ptr(), dst_t.data_ptr())
                if key not in cache:
                    rp, co, va = csr[op]
                    cache[key] = cusparse_ref.CusparseSpmm(rp, co, va, src, dst_t)
                cache[key].run()
                return dst_t

            ref_step = gcn.GCN(g, x, truth, weights, aggregate=cusparse_aggregate)
            out["ms_cusparse_aggregation"], _ = time_epochs(ref_step, epochs, torch.cuda.synchronize)
            out["loss_rel_diff_vs_cusparse"] = abs(float(ref_step.loss) - loss_ours) / max(abs(loss_ours), 1e-30)
            out["cusparse_note"] = ("the same step with cusparseSpMM (ALG_DEFAULT, row-major, as at "
                                    "cuda_gcn/src/cuda/cuda_module.cu:233-246 / 323-336) in place of this library's "
                                    "aggregation; not the reference's own epoch loop")
            for c in cache.values():
                c.close()
        except Exception as e:
            out["ms_cusparse_aggregation"] = None
            out["cusparse_error"] = repr(e)
    g.plan.close()
    del step, x, truth, weights, g
    torch.cuda.empty_cache()
    if with_cusparse and len(dims) == 3:
        out["reference_epoch"] = reference_gcn_epoch(cfg, epochs)
        ref = out["reference_epoch"]
        if "first_epoch_loss" in ref:
            ref["loss_rel_diff_vs_drone_b200"] = abs(ref["first_epoch_loss"] - loss_ours) / max(abs(loss_ours), 1e-30)
    return out


def reference_gcn_epoch(cfg, epochs, timeout_s=600):
    """The reference's own training epoch on the same graph, features, labels and starting weights, in a child process
    (baseline/ref_gcn_epoch.py; needs oracle/_ref/libref_graphsum.so)."""
    import subprocess
    try:
        r = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "ref_gcn_epoch.py"), "--vertices",
                            str(cfg["vertices"]), "--pairs", str(cfg["pairs"]), "--seed", str(cfg["seed"]), "--dims",
                            ",".join(str(d) for d in cfg["dims"]), "--epochs", str(epochs)],
                           capture_output=True, text=True, timeout=timeout_s)
        lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
        return json.loads(lines[-1]) if lines else {"error": "exit %d: %s" % (r.returncode, r.stderr[-300:])}
    except Exception as e:
        return {"error": repr(e)}


def distribute_graph(n, make_edges, world, rank, device, keep_self_loops=True):
    """Rank 0 makes the edge list (make_edges() -> (u, v) int32 CUDA tensors), EBV-partitions it and hands every rank
    its own edges and the global tables.  Returns (partition, in_degree, out_degree, total_edges, partition_seconds)."""
    from drone_b200 import graphgen as gg, partition as pt
    part, extra, part_s = None, (), 0.0
    if rank == 0:
        u, v = make_edges()
        in_deg, out_deg = gg.degrees(u, v, n)
        uh, vh = u.cpu().numpy(), v.cpu().numpy()
        del u, v
        torch.cuda.empty_cache()
        t0 = time.perf_counter()
        part = pt.ebv_partition(n, uh, vh, world, keep_self_loops=keep_self_loops)
        part_s = time.perf_counter() - t0
        del uh, vh
        extra = (in_deg.cpu().numpy(), out_deg.cpu().numpy())
        del in_deg, out_deg
    part, (in_deg, out_deg), total_e = pt.scatter_partition(part, n, world, device, extra=extra, n_extra=2)
    return part, in_deg, out_deg, total_e, part_s


def gcn_epoch_multi(device, cfg_name, rank, world, comm, sync, epochs=5):
    """The GCN epoch of configuration `cfg_name` over WORLD_SIZE EBV parts: weight broadcast, forward (aggregation +
    mirror/master exchange per layer), backward (same, on the gradients), gradient reduce to rank 0."""
    import torch.distributed as dist
    from drone_b200 import gcn, graphgen as gg, graphsum as gs
    cfg = GCN_CONFIGS[cfg_name]
    dims = cfg["dims"]
    n = cfg["vertices"]

    def make_edges():
        _, u, v = gg.powerlaw_graph(n, cfg["pairs"], seed=cfg["seed"], device=device)
        return u, v
    part, in_deg, out_deg, total_e, part_s = distribute_graph(n, make_edges, world, rank, device)
    graph = gs.DeviceGraph(part.local_graph(rank), in_deg, out_deg, device, max_features=max(dims[1:]))
    graph.plan.reserve(max(dims[1:]), padded_rows=True)
    graph.xplan.enable_p2p(comm)
    l2g = graph.host.l2g
    x = hashed_normal(l2g, dims[0], 7, device)
    truth = hashed_labels(l2g, dims[-1], 7, device)
    weights = glorot_weights(dims, device)
    torch.backends.cuda.matmul.allow_tf32 = False
    step = gcn.GCN(graph, x, truth, weights, comm=comm, worker_num=world)
    ms, nblocks = time_epochs(step, epochs, sync)
    t = torch.tensor([ms], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # the loss over the master copies of all ranks (every labelled vertex once)
    logits = step.z[-1]
    zmax = logits.max(dim=1, keepdim=True).values
    lse = torch.log(torch.exp(logits - zmax).sum(dim=1)) + zmax.squeeze(1)
    per_row = lse - logits.gather(1, truth.long().unsqueeze(1)).squeeze(1)
    masters = graph.mirror2worker == -1
    acc = torch.stack([(per_row * masters).double().sum(), masters.double().sum()])
    dist.all_reduce(acc)
    up, down, _ = graph.xplan.counts()
    stats = torch.tensor([graph.n_local, int(up.sum() + down.sum())], device=device, dtype=torch.int64)
    dist.all_reduce(stats)
    out = {"config": cfg["descr"], "vertices": n, "nnz": int(total_e), "dims": dims, "parts": world,
           "ms_per_epoch": float(t), "epochs_per_block": epochs, "timed_blocks": nblocks,
           "loss_over_masters": float(acc[0] / acc[1]), "replication_factor": float(stats[0]) / n,
           "mirror_sync_bytes_per_epoch_all_ranks": int(stats[1]) * 4 * 2 * sum(dims[1:]),
           "partition_seconds": part_s,
           "step": "weight bcast + forward + backward + gradient reduce; exchange over peer memory after every aggregation"}
    graph.plan.close()
    return out


def one_part_pagerank(device, n, index, dst, out_degree, iterations):
    """Time per power iteration (float) of PageRank over a whole graph held as one part on `device`."""
    import types
    from drone_b200 import pagerank as prk, partition as pt
    host = types.SimpleNamespace(rank=0, n_parts=1, n_local=n, l2g=np.arange(n, dtype=np.int32),
                                 mirror2worker=np.full(n, -1, np.int32), master_worker_index=np.zeros(n + 1, np.int32),
                                 master2workers=np.zeros(0, np.int32))
    g = types.SimpleNamespace(host=host, n_local=n, device=device, index=index, dst=dst, out_degree=out_degree,
                              mirror2worker=torch.full((n,), -1, dtype=torch.int32, device=device),
                              xplan=pt.ExchangePlan(host, 1))
    pr1 = prk.PageRank(g, n, use_double=False, eps=0.0)
    pr1.power_iterate(3, 0.85)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    pr1.power_iterate(iterations, 0.85)
    e1.record()
    torch.cuda.synchronize()
    ms_it = e0.elapsed_time(e1) / iterations
    nnz = int(dst.numel())
    b_alg = 4 * nnz + 4 * (n + 1) + 8 * n + 8 * n       # columns, row pointers, published pairs, state in/out
    res = {"vertices": n, "edges": nnz, "iterations": iterations, "ms_per_iteration": ms_it,
           "edges_per_s": nnz / (ms_it * 1e-3), "algorithmic_GBps": b_alg / (ms_it * 1e-3) / 1e9}
    pr1.close()
    return res


def jobs_head_to_head(timeout_s=240):
    """pr_cuda supersteps and one sssp_cuda run through the cgo-facing C interface, once with the reference's own
    sources (oracle/_ref/libref_drone_jobs.so) and once with this repository's drop-in, same driver, same R-MAT-20
    graph, one worker (baseline/jobs_driver.py; each in a child process)."""
    import subprocess
    out = {}
    for which in ("reference", "dropin"):
        try:
            r = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "jobs_driver.py"), "--lib", which],
                               capture_output=True, text=True, timeout=timeout_s)
            lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
            out[which] = json.loads(lines[-1]) if lines else {"error": "exit %d: %s" % (r.returncode, r.stderr[-300:])}
        except Exception as e:
            out[which] = {"error": repr(e)}
    return out


def minprop_timing(device):
    """The cc_cuda / sssp_cuda jobs on one part: labels on R-MAT-20 symmetrised (connected components) and
    unit-length distances on R-MAT-22 directed from the vertex with the most out-edges, each checked against the CPU
    restatement (one host core) and timed next to it."""
    import types
    from drone_b200 import graphgen as gg, minprop as mpj, partition as pt
    from oracle import oracle
    out = {}
    for name, scale, sym, kind in (("cc_rmat20_sym", 20, True, mpj.CC), ("sssp_rmat22_directed", 22, False, mpj.SSSP)):
        n, u, v = gg.rmat_graph(scale, 16, seed=20261140 + scale, device=device, symmetrise=sym, self_loops="drop")
        index, dst = gg.csr_by_source(u, v, n)
        _, outd = gg.degrees(u, v, n)
        source = int(torch.argmax(outd)) if kind == mpj.SSSP else -1
        del u, v
        host = types.SimpleNamespace(rank=0, n_parts=1, n_local=n, l2g=np.arange(n, dtype=np.int32),
                                     mirror2worker=np.full(n, -1, np.int32), master_worker_index=np.zeros(n + 1, np.int32),
                                     master2workers=np.zeros(0, np.int32))
        g = types.SimpleNamespace(host=host, n_local=n, device=device, index=index, dst=dst,
                                  xplan=pt.ExchangePlan(host, 1))
        job = mpj.MinProp(g, kind)
        job.peval(source)                       # warm-up
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = job.peval(source)                 # synchronous: returns when the local run has converged
        gpu_s = time.perf_counter() - t0
        got = job.values()
        ih, dh = index.cpu().numpy(), dst.cpu().numpy()
        t0 = time.perf_counter()
        want = oracle.cc_fixed_point(ih, dh) if kind == mpj.CC else oracle.sssp_f32(ih, dh, source)
        cpu_s = time.perf_counter() - t0
        nnz = int(dst.numel())
        out[name] = {"vertices": n, "edges": nnz, "gpu_ms": 1e3 * gpu_s, "cpu_restatement_s": cpu_s, "cpu_cores": 1,
                     "identical_to_restatement": bool(np.array_equal(got, want)), "visited": int(res.VisitedSize),
                     "distinct_labels" if kind == mpj.CC else "reached": int(len(np.unique(got)) if kind == mpj.CC
                                                                              else (got < 1e8).sum())}
        job.close()
        del index, dst, outd
        torch.cuda.empty_cache()
    return out


def pagerank_timing(device):
    """PageRank, the path at feature width 1.
    (a) R-MAT scale 16, edge factor 16, self-loops and duplicates removed, EBV into 2 parts (both held on this GPU):
        20 synchronous iterations, damping 0.85, start 1/|V|, in double; checked against the double oracle, and timed
        next to the restatement of DRONE's CPU job "pr" (float, eps 0.01, at most 200 supersteps) on one host core.
    (b) R-MAT scale 22 directed, one part, float: time per iteration of the propagation."""
    import types
    import drone_b200 as db
    from drone_b200 import graphgen as gg, graphsum as gs, pagerank as prk, partition as pt
    from oracle import oracle
    out = {}
    n, u, v = gg.rmat_graph(16, 16, seed=20261125, device=device, symmetrise=False, self_loops="drop")
    uh, vh = u.cpu().numpy(), v.cpu().numpy()
    in_deg = np.bincount(vh, minlength=n).astype(np.int32)
    out_deg = np.bincount(uh, minlength=n).astype(np.int32)
    part = pt.ebv_partition(n, uh, vh, 2, keep_self_loops=False)
    graphs = [gs.DeviceGraph(part.local_graph(p), in_deg, out_deg, device, max_features=1) for p in range(2)]
    n_iso = int((part.replicas == 0).sum())
    prs = [prk.PageRank(g, n, use_double=True, eps=0.0, n_isolated=n_iso) for g in graphs]
    prk.power_iterate_local(prs, 20, 0.85)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    prk.power_iterate_local(prs, 20, 0.85)
    e1.record()
    torch.cuda.synchronize()
    got = prk.gather_global(prs, graphs, n)
    index, dst = gg.csr_by_source(u, v, n)
    want = oracle.pagerank_power_f64(index.cpu().numpy(), dst.cpu().numpy(), 20, 0.85)
    touched = part.replicas > 0
    t0 = time.perf_counter()
    _, cpu_steps, cpu_msgs = oracle.pr_drone_cpu(n, part.part_u, part.part_v, out_deg, part.owner, eps=0.01, max_steps=200)
    cpu_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    oracle.pr_drone_cpu(n, part.part_u, part.part_v, out_deg, part.owner, eps=0.01, max_steps=200, maps=True)
    cpu_maps_s = time.perf_counter() - t0
    out["rmat16_2parts"] = {
        "vertices": n, "edges": int(len(uh)), "iterations": 20, "ms_total_gpu": e0.elapsed_time(e1),
        "max_rel_err_vs_double_oracle": float(np.max(np.abs(got[touched] - want[touched]) / want[touched])),
        "replication_factor": part.replication_factor(),
        "cpu_pr_job_restatement": {"seconds": cpu_s, "seconds_hash_map_state": cpu_maps_s, "supersteps": cpu_steps,
                                   "messages": int(cpu_msgs), "cores": 1,
                                   "note": "C restatement of DRONE's Go job (the Go binary cannot be built here)"}}
    for p_ in prs:
        p_.close()
    del graphs, prs

    n, u, v = gg.rmat_graph(22, 16, seed=20261131, device=device, symmetrise=False, self_loops="drop")
    index, dst = gg.csr_by_source(u, v, n)
    _, outd = gg.degrees(u, v, n)
    del u, v
    out["rmat22_1part_float"] = one_part_pagerank(device, n, index, dst, outd, 20)
    return out


class MultiStep:
    """Local aggregation + mirror/master exchange of one rank, plain or in row groups (PipelinedAggregation)."""

    def __init__(self, graph, comm, f, exchange, dense=None, fused_push=True):
        self.graph, self.comm, self.f, self.exchange_kind, self.dense = graph, comm, f, exchange, dense
        self.piped = {}
        # peer-memory transport: the aggregation kernels store mirror rows straight into their owners' memory
        self.fused_push = bool(fused_push) and exchange == "p2p"

    def exchange(self, rows):
        from drone_b200 import graphsum as gs
        if self.dense is not None:
            gs.exchange_sum_dense(self.dense, self.comm, rows)
        else:
            gs.exchange_sum(self.graph.xplan, self.comm, rows)

    def use_groups(self, groups):
        """Switch to `groups` row groups (1 = aggregation, then exchange).  Rebuilds the plan's work lists."""
        from drone_b200 import graphsum as gs
        self.groups = groups
        for p in self.piped.values():
            p.close()
        self.piped = {}
        if groups > 1:
            self.piped[groups] = gs.PipelinedAggregation(self.graph, self.comm, self.f, n_groups=groups,
                                                         p2p=self.exchange_kind == "p2p", fused_push=self.fused_push)
        else:
            self.graph.plan.set_row_classes(None, 1)

    def __call__(self, op, x, y):
        if self.groups > 1:
            self.piped[self.groups](op, x, y)
        elif self.fused_push:
            from drone_b200 import graphsum as gs
            self.graph.plan.spmm(op, x, out=y, push_up_to=self.graph.xplan.handle)
            gs.exchange_finish(self.graph.xplan, y)
        else:
            self.graph.plan.spmm(op, x, out=y)
            self.exchange(y)


def multi_parity(device, rank, world, comm, exchange, groups, fused_push=True):
    """Aggregation + exchange over WORLD_SIZE EBV parts of a seeded R-MAT-13 graph (F = 32, both orientations)
    against the double-precision oracle of the whole graph, compared by global vertex id on every rank: the largest
    error relative to the largest element, maximum over ranks."""
    import torch.distributed as dist
    import drone_b200 as db
    from drone_b200 import graphgen as gg, graphsum as gs
    n, f = 1 << 13, 32

    def make_edges():
        _, u, v = gg.rmat_graph(13, 16, seed=20261142, device=device, symmetrise=False, self_loops="add")
        return u, v
    part, in_deg, out_deg, _, _ = distribute_graph(n, make_edges, world, rank, device)
    x = gg.seeded_normal(5, (n, f))
    want = torch.zeros((2, n, f), dtype=torch.float64, device=device)
    if rank == 0:
        from oracle import oracle
        oracle.build()
        _, u, v = gg.rmat_graph(13, 16, seed=20261142, symmetrise=False, self_loops="add")
        index, dst = gg.csr_by_source(u, v, n)
        val = oracle.csr_values_f32(index.numpy(), dst.numpy(), in_deg, out_deg)
        want[0] = torch.as_tensor(oracle.graphsum_forward_f64(x, index.numpy(), dst.numpy(), val), device=device)
        want[1] = torch.as_tensor(oracle.graphsum_backward_f64(x, index.numpy(), dst.numpy(), val), device=device)
    dist.broadcast(want, 0)
    graph = gs.DeviceGraph(part.local_graph(rank), in_deg, out_deg, device, max_features=f)
    if exchange == "p2p":
        graph.xplan.enable_p2p(comm)
    step = MultiStep(graph, comm, f, exchange, fused_push=fused_push)
    l2g = torch.as_tensor(graph.host.l2g.astype(np.int64), device=device)
    xl = torch.as_tensor(x, device=device)[l2g]
    worst = torch.zeros(1, dtype=torch.float64, device=device)
    for g_ in sorted({1, groups}):
        step.use_groups(g_)
        for k, op in enumerate((db.OP_AT, db.OP_A)):
            y = torch.full((graph.n_local, f), float("nan"), device=device)
            step(op, xl, y)
            torch.cuda.synchronize()
            ref = want[k][l2g]
            err = (y.double() - ref).abs().max() / want[k].abs().max()
            worst = torch.maximum(worst, torch.nan_to_num(err, nan=1e30).reshape(1))
    step.use_groups(1)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    graph.plan.close()
    return float(worst)


def run_ours_multi(args, cfg):
    """One process per GPU: R-MAT graph EBV-partitioned into WORLD_SIZE parts, every step is the local
    aggregation Y_p = A_p^T X_p followed by the mirror/master exchange."""
    import torch.distributed as dist
    import drone_b200 as db
    from drone_b200 import graphgen as gg
    from drone_b200 import graphsum as gs
    from drone_b200 import partition as pt

    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    lib = db.lib()
    chosen = args.chosen
    comm = gs.Comm(rank, world)
    t_start = time.perf_counter()

    def sync():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    line_extra = {}
    if "parity" in chosen:
        err = multi_parity(device, rank, world, comm, args.exchange, 2, fused_push=not args.no_fused_push)
        line_extra["parity"] = {"max_rel_err": err, "ranks": world, "tolerance": 1e-5, "ok": err <= 1e-5,
                                "case": "R-MAT-13 +I over %d EBV parts, F=32, aggregation + exchange (%s transport%s; one "
                                        "piece and in 2 row groups), both orientations, against the double oracle by "
                                        "global id" % (world, args.exchange,
                                                       ", mirror rows sent from the aggregation's store"
                                                       if args.exchange == "p2p" and not args.no_fused_push else "")}
        if not err <= 1e-5:
            if rank == 0:
                print(json.dumps({"metric": "spmm_nnzF_per_s", "n_gpus": world, "parity": line_extra["parity"],
                                  "error": "parity check failed"}), flush=True)
            raise SystemExit("bench.py: multi-GPU parity check failed: %g" % err)

    line = run_partitioned_workload(args, cfg, device, rank, world, comm, sync, headline=True)
    if rank == 0:
        line.update(line_extra)

    def section(name, fn):
        if name not in chosen:
            return
        try:
            res = fn()
        except Exception as e:
            res = {"error": repr(e)}
        if rank == 0:
            line[name] = res
        torch.cuda.empty_cache()

    section("gcn_epoch", lambda: gcn_epoch_multi(device, "c3", rank, world, comm, sync))
    section("gcn_c4", lambda: gcn_epoch_multi(device, "c4", rank, world, comm, sync, epochs=3))
    if "strong" in chosen and args.scaling != "strong":
        name = args.strong_workload
        if name == "auto":       # the 2^26-vertex graph takes about two minutes of set-up (generation + partitioning)
            name = "rmat26"
        sargs = argparse.Namespace(**vars(args))
        sargs.workload, sargs.scaling, sargs.pagerank_iters = name, "strong", 20
        scfg = dict(WORKLOADS[name])
        section("strong", lambda: run_partitioned_workload(sargs, scfg, device, rank, world, comm, sync, headline=False))
    if rank == 0:
        line["wall_seconds"] = time.perf_counter() - t_start
        print(json.dumps(line), flush=True)
    comm.close()
    dist.destroy_process_group()


def run_partitioned_workload(args, cfg, device, rank, world, comm, sync, headline):
    """Times aggregation + exchange over the EBV parts of the workload's graph.  Returns the JSON line (headline) or
    a section (same keys, without the end-to-end part) on rank 0; other ranks get a dict they do not use."""
    import torch.distributed as dist
    import drone_b200 as db
    from drone_b200 import graphgen as gg
    from drone_b200 import graphsum as gs
    from drone_b200 import partition as pt
    lib = db.lib()
    f = cfg["features"]
    n = 1 << cfg["scale"]
    t_setup = time.perf_counter()

    def make_edges():
        _, u, v = gg.rmat_graph(cfg["scale"], cfg["edge_factor"], seed=cfg["seed"], device=device,
                                symmetrise=cfg["symmetrise"], self_loops="add")
        return u, v
    part, in_deg, out_deg, total_e, part_s = distribute_graph(n, make_edges, world, rank, device)
    graph = gs.DeviceGraph(part.local_graph(rank), in_deg, out_deg, device, max_features=f)
    graph.plan.reserve(f)
    if args.exchange == "p2p":
        graph.xplan.enable_p2p(comm)
    dense = pt.DenseExchangePlan(part, graph.host, f) if args.exchange == "dense" else None
    nnz_local = graph.dst.numel()
    nnz_total = total_e
    up, down, _ = graph.xplan.counts()
    sync_bytes = int(up.sum() + down.sum()) * f * 4
    setup_s = time.perf_counter() - t_setup

    nbuf = 3
    gen = torch.Generator(device=device)
    gen.manual_seed(cfg["seed"] + rank)
    xs = [torch.randn((graph.n_local, f), device=device, generator=gen) for _ in range(nbuf)]
    ys = [torch.empty((graph.n_local, f), device=device) for _ in range(nbuf)]
    mstep = MultiStep(graph, comm, f, args.exchange, dense, fused_push=not args.no_fused_push)

    def step(i):
        mstep(db.OP_AT, xs[i % nbuf], ys[i % nbuf])

    # row groups: as asked, or the fastest of 1 / 2 / 4 (every rank takes the same decision from the reduced times)
    candidates = [args.pipeline_groups] if args.pipeline_groups > 0 else ([1] if dense is not None else [1, 2, 4])
    trial = {}
    for g_ in candidates:
        mstep.use_groups(g_)
        for i in range(3):
            step(i)
        if len(candidates) > 1:
            blocks = time_blocks(step, max(5, min(args.steps, 10)), sync, min_seconds=0.05)
            t = torch.tensor([float(np.median(blocks))], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            trial[g_] = float(t) / max(5, min(args.steps, 10))
    groups = min(trial, key=trial.get) if trial else candidates[0]
    if groups != mstep.groups:
        mstep.use_groups(groups)
    warmup = max(args.warmup, 3)
    for i in range(warmup):
        step(i)
    sampler = ClockSampler(index=device.index)
    sampler.start()
    launches0 = lib.drone_kernel_launch_count()
    blocks = time_blocks(step, args.steps, sync)
    launches = (lib.drone_kernel_launch_count() - launches0) // len(blocks)
    sampler.in_timed_region = False
    clocks = sampler.finish()
    t_ms = torch.tensor(blocks, device=device)
    dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)          # per block: the slowest rank
    ms = float(t_ms.median()) / args.steps

    # local aggregation alone (for the roofline of the kernel) and exchange alone
    mstep.use_groups(1)
    blocks_a = time_blocks(lambda i: graph.plan.spmm(db.OP_AT, xs[i % nbuf], out=ys[i % nbuf]), args.steps,
                           torch.cuda.synchronize, min_seconds=0.1)
    spmm_ms = float(np.median(blocks_a)) / args.steps
    blocks_x = time_blocks(lambda i: mstep.exchange(ys[i % nbuf]), args.steps, sync, min_seconds=0.1)
    xchg = torch.tensor([float(np.median(blocks_x)) / args.steps, spmm_ms], device=device)
    dist.all_reduce(xchg, op=dist.ReduceOp.MAX)

    # the full-size result of one step, checked through its column sums over all ranks: rows a rank owns (masters and
    # unreplicated vertices) against the coefficient sums of every rank's own part applied to that rank's operand
    step(0)
    torch.cuda.synchronize()
    try:
        own = torch.as_tensor(graph.host.mirror2worker < 0, device=device)
        terms = torch.stack(checksum_terms(graph.plan, db.OP_AT, xs[0], ys[0], own_rows=own))
    except Exception as e:      # every rank still joins the reduction below
        print("bench.py: rank %d could not form its checksum terms: %r" % (rank, e), file=sys.stderr)
        terms = torch.full((3, f), float("nan"), dtype=torch.float64, device=device)
    dist.all_reduce(terms)
    checksum = checksum_report(terms[0], terms[1], terms[2],
                               "column sums of the owned rows of Y over all ranks against the sum over the parts of "
                               "(coefficient sums per gathered row)^T X of that part, in double, relative to the sum of "
                               "the absolute terms; aggregation + exchange on the timed graph")

    # PageRank power iterations (F = 1) over the same partition: pull along in-edges + the same exchange per iteration
    pr_result = None
    if args.pagerank_iters > 0:
        from drone_b200 import pagerank as prm
        pr = prm.PageRank(graph, n, comm=comm, use_double=False)
        pr.power_iterate(3)
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        pr.power_iterate(args.pagerank_iters)
        e1.record()
        torch.cuda.synchronize()
        pr_ms = torch.tensor([e0.elapsed_time(e1) / args.pagerank_iters], device=device)
        dist.all_reduce(pr_ms, op=dist.ReduceOp.MAX)
        mass = torch.tensor([float(pr.values()[graph.host.mirror2worker < 0].astype(np.float64).sum())], device=device,
                            dtype=torch.float64)
        dist.all_reduce(mass)
        pr_result = {"iterations": args.pagerank_iters, "ms_per_iteration": float(pr_ms),
                     "nnz_per_s": nnz_total / (float(pr_ms) * 1e-3), "sum_over_masters": float(mass),
                     "mirror_sync_bytes_per_iteration_all_ranks": None,
                     "dtype": "f32", "exchange": pr.transport_name() if hasattr(pr, "transport_name") else
                     "grouped ncclSend/ncclRecv of all boundary vertices + scalar all-reduce"}
        pr.close()

    e2e = e2e_single = None
    if headline and "e2e" in args.chosen:
        # end to end: host operands in, host result out, every step.  First one step at a time (copy in, step, copy
        # out, wait); then a series of steps over two operand sets with the copies on streams of their own, so that
        # the copy in of step k, the work of step k-1 and the copy out of step k-2 overlap.
        xh = [torch.empty((graph.n_local, f), dtype=torch.float32).pin_memory() for _ in range(2)]
        yh = [torch.empty((graph.n_local, f), dtype=torch.float32).pin_memory() for _ in range(2)]
        for b in range(2):
            xh[b].copy_(xs[b])
        sync()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            xs[0].copy_(xh[0], non_blocking=True)
            step(0)
            yh[0].copy_(ys[0], non_blocking=True)
            torch.cuda.synchronize()
        e2e_t = torch.tensor([(time.perf_counter() - t0) / args.e2e_steps], device=device, dtype=torch.float64)
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
        e2e_single = float(e2e_t)

        main = torch.cuda.current_stream(device)
        cin, cout = torch.cuda.Stream(device), torch.cuda.Stream(device)
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def series(steps):
            for i in range(steps):
                b = i % 2
                if i >= 2:
                    ev_out[b].synchronize()          # result i-2 is on the host: its two buffers are free again
                with torch.cuda.stream(cin):
                    xs[b].copy_(xh[b], non_blocking=True)
                    ev_in[b].record(cin)
                main.wait_event(ev_in[b])
                step(b)
                ev_done[b].record(main)
                cout.wait_event(ev_done[b])
                with torch.cuda.stream(cout):
                    yh[b].copy_(ys[b], non_blocking=True)
                    ev_out[b].record(cout)
            for e in ev_out:
                e.synchronize()
        series(4)
        sync()
        q_steps = 2 * max(args.e2e_steps, 5)
        t0 = time.perf_counter()
        series(q_steps)
        e2e_t = torch.tensor([(time.perf_counter() - t0) / q_steps], device=device, dtype=torch.float64)
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
        e2e = float(e2e_t)
        # the series moved the right data: result of the last step on slot 0 against a step on the device operands
        step(0)
        torch.cuda.synchronize()
        e2e_diff = torch.tensor([float((yh[0][:65536] - ys[0][:65536].cpu()).abs().max())], device=device)
        dist.all_reduce(e2e_diff, op=dist.ReduceOp.MAX)
        e2e_diff = float(e2e_diff)
        del xh, yh
    stats = torch.tensor([graph.n_local, nnz_local, sync_bytes, launches, int(up.sum() + down.sum())], device=device,
                         dtype=torch.int64)
    gathered = [torch.zeros_like(stats) for _ in range(world)]
    dist.all_gather(gathered, stats)
    g = torch.stack(gathered).cpu().numpy()
    peak, peak_src = hbm_peak()
    b_alg = algorithmic_bytes(graph.n_local, nnz_local, f)
    achieved = b_alg / (spmm_ms * 1e-3) / 1e9
    if pr_result is not None:
        pr_result["mirror_sync_bytes_per_iteration_all_ranks"] = int(g[:, 4].sum()) * 8     # {value, flag} per boundary vertex
    line = {
        "metric": "spmm_nnzF_per_s", "value": nnz_total * f / (ms * 1e-3), "unit": "nnz*F/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload_descr(args, cfg, n, nnz_total), parts=world, partitioner="EBV",
                       pipeline_groups=groups, pipeline_trial_ms={str(k): v for k, v in trial.items()},
                       replication_factor=float(g[:, 0].sum()) / n,
                       edge_imbalance=float(g[:, 1].max() * world / g[:, 1].sum())),
        "timed_blocks": len(blocks), "timed_ms_total": float(np.sum(blocks)),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": peak_src, "algorithmic_bytes": b_alg,
                     "kernel": "rank 0's local drone_spmm call, timed alone", "ms": spmm_ms},
        "exchange": {"ms": float(xchg[0]), "aggregation_ms_slowest_rank": float(xchg[1]),
                     "mirror_sync_bytes_per_step_all_ranks": int(g[:, 2].sum()),
                     "mirror_sync_bytes_per_step_rank0": sync_bytes,
                     "collective": {"p2p": "peer-memory stores + epoch flags (push_up, add_push_down, scatter; waits in one-block kernels)",
                                    "nccl": "grouped ncclSend/ncclRecv x2",
                                    "dense": "ncclReduceScatter + ncclAllGather over the boundary"}[args.exchange],
                     "mirror_rows_sent_from_aggregation_store": bool(mstep.fused_push),
                     "note": "ms = the whole exchange run alone (copy kernel for the upward half); in the timed step the "
                             "upward half is part of the aggregation when mirror_rows_sent_from_aggregation_store",
                     "dense_boundary_rows": dense.boundary_rows() if dense is not None else None},
        "gpu_launches": int(g[:, 3].sum()), "clocks": clocks, "setup_s": setup_s, "partition_seconds": part_s,
        "checksum_identity": checksum,
    }
    if e2e is not None:
        line["e2e"] = {"value": nnz_total * f / e2e, "unit": "nnz*F/s", "h2d_bytes_per_step": int(g[:, 0].sum()) * f * 4,
                       "d2h_bytes_per_step": int(g[:, 0].sum()) * f * 4, "ms_per_step": 1e3 * e2e, "steps": q_steps,
                       "max_abs_diff_vs_device_step": e2e_diff,
                       "how": "a series of steps over two pinned operand sets per rank: every step copies its own rows in "
                              "and its own result out; copy in of step k, step k-1 and copy out of step k-2 overlap "
                              "(copies on streams of their own).  Wall clock of the slowest rank, pipeline fill included",
                       "single_step": {"ms_per_step": 1e3 * e2e_single, "value": nnz_total * f / e2e_single,
                                       "steps": args.e2e_steps, "how": "copy in, step, copy out, wait; one step at a time"}}
    if pr_result is not None:
        line["pagerank"] = pr_result
    for p_ in mstep.piped.values():
        p_.close()
    graph.plan.close()
    del xs, ys, graph
    torch.cuda.empty_cache()
    return line


def keep_stdout_for_the_result_line():
    """Libraries write to file descriptor 1 on their own (NCCL prints its version line there when NCCL_DEBUG asks for
    it): from here on descriptor 1 is the error stream, and Python's sys.stdout writes to a copy of the original
    descriptor, so that the JSON line is the only thing on standard output."""
    sys.stdout.flush()
    original = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(original, "w", buffering=1)


def main():
    args = parse_args()
    keep_stdout_for_the_result_line()
    if args.record_traffic:
        record_traffic(args.record_traffic, args.workload)
        return
    cfg = workload_config(args)
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()

"""PageRank on the device against the oracles: DRONE's GPU-job schedule in double (1e-9) and float,
synchronous power iteration (the 20-iteration, damping 0.85 configuration), all parts on one GPU or
one process per GPU over NCCL."""
import os

import numpy as np
import pytest
import torch

import drone_b200 as db
from helpers import run_ranks
from drone_b200 import graphgen as gg
from drone_b200 import graphsum as gs
from drone_b200 import pagerank as prk
from drone_b200 import partition as pt
from test_pagerank_oracle import pr_case

pytestmark = pytest.mark.gpu

PR_TOL = 1e-9   # relative, double mode against the double oracle running the same schedule


def build_parts(part, n, u, v, dev, use_double, eps):
    in_deg = np.bincount(v, minlength=n).astype(np.int32)
    out_deg = np.bincount(u, minlength=n).astype(np.int32)
    graphs = [gs.DeviceGraph(part.local_graph(p), in_deg, out_deg, dev, max_features=1) for p in range(part.n_parts)]
    n_iso = int((part.replicas == 0).sum())
    prs = [prk.PageRank(g, n, comm=None, use_double=use_double, eps=eps, n_isolated=n_iso) for g in graphs]
    return graphs, prs


@pytest.mark.parametrize("parts", [2, 4])
def test_delta_schedule_double_matches_oracle(cuda_device, oracle, parts):
    n, u, v, out_deg, part = pr_case(scale=10, seed=31, parts=parts)
    want, want_steps, want_sizes = oracle.pr_drone_cuda(n, part.part_u, part.part_v, out_deg, part.owner, eps=1e-6,
                                                        dtype=np.float64)
    graphs, prs = build_parts(part, n, u, v, cuda_device, True, 1e-6)
    steps, sizes = prk.run_job_local(prs)
    got = prk.gather_global(prs, graphs, n)
    assert steps == want_steps
    # per superstep, the four exchange counts summed over parts
    got_sizes = np.array([[sum(s[i] for s in step) for i in range(4)] for step in sizes])
    assert np.array_equal(got_sizes, want_sizes)
    touched = part.replicas > 0
    assert np.max(np.abs(got[touched] - want[touched]) / np.abs(want[touched])) < PR_TOL
    # every replica of a vertex holds the same value at the end
    seen = {}
    for pr_, g in zip(prs, graphs):
        vals = pr_.values()
        for loc in np.nonzero(part.replicas[g.host.l2g] > 1)[0][:200]:
            gid = int(g.host.l2g[loc])
            assert seen.setdefault(gid, vals[loc]) == vals[loc]


def test_delta_schedule_float_close_to_reference_semantics(cuda_device, oracle):
    n, u, v, out_deg, part = pr_case(scale=10, seed=32, parts=2)
    want, want_steps, _ = oracle.pr_drone_cuda(n, part.part_u, part.part_v, out_deg, part.owner, eps=1e-6,
                                               dtype=np.float32)
    graphs, prs = build_parts(part, n, u, v, cuda_device, False, 1e-6)
    steps, _ = prk.run_job_local(prs)
    got = prk.gather_global(prs, graphs, n)
    touched = part.replicas > 0
    # float sums in a different (fixed) order than the oracle's; thresholded pushes may flip near eps
    assert np.max(np.abs(got[touched] - want[touched]) / want[touched]) < 2e-4
    assert abs(steps - want_steps) <= max(3, want_steps // 5)


@pytest.mark.parametrize("parts", [1, 2, 8])
def test_power_iteration_rmat16_config(cuda_device, oracle, parts):
    """R-MAT scale 16, edge factor 16, self-loops and duplicates removed, damping 0.85, 20 iterations, 1/|V| start."""
    n, u, v = gg.rmat_graph(16, 16, seed=20261125, symmetrise=False, self_loops="drop")
    u, v = u.numpy(), v.numpy()
    index, dst = gg.csr_by_source(torch.as_tensor(u), torch.as_tensor(v), n)
    want = oracle.pagerank_power_f64(index.numpy(), dst.numpy(), 20, 0.85)
    part = pt.ebv_partition(n, u, v, parts, keep_self_loops=False)
    graphs, prs = build_parts(part, n, u, v, cuda_device, True, 0.0)
    prk.power_iterate_local(prs, 20, 0.85)
    got = prk.gather_global(prs, graphs, n)
    touched = part.replicas > 0
    assert np.max(np.abs(got[touched] - want[touched]) / want[touched]) < PR_TOL
    # float mode: same procedure, float accuracy
    graphs32, prs32 = build_parts(part, n, u, v, cuda_device, False, 0.0)
    prk.power_iterate_local(prs32, 20, 0.85)
    got32 = prk.gather_global(prs32, graphs32, n)
    assert np.max(np.abs(got32[touched] - want[touched]) / want[touched]) < 1e-4


@pytest.mark.parametrize("parts", [1, 3])
def test_pairs_laid_out_by_gather_frequency(cuda_device, oracle, parts, monkeypatch):
    """Large parts publish their {delta, pushed} pairs in the order of how often they are gathered and renumber the pull
    lists' columns to match (forced here on a small graph): only the addresses of the gathers change, so the values
    and the superstep count are bit for bit those of the plain layout, in both schedules."""
    n, u, v = gg.rmat_graph(13, 16, seed=36, symmetrise=False, self_loops="drop")
    u, v = u.numpy(), v.numpy()
    part = pt.ebv_partition(n, u, v, parts, keep_self_loops=False)
    results = []
    for min_rows in ("0", "1"):
        monkeypatch.setenv("DRONE_PR_ORDER_MIN_ROWS", min_rows)
        graphs, prs = build_parts(part, n, u, v, cuda_device, False, 1e-6)
        steps, _ = prk.run_job_local(prs)
        delta = prk.gather_global(prs, graphs, n)
        prk.power_iterate_local(prs, 20, 0.85)
        results.append((steps, delta, prk.gather_global(prs, graphs, n)))
    assert results[0][0] == results[1][0]
    assert np.array_equal(results[0][1], results[1][1]) and np.array_equal(results[0][2], results[1][2])
    index, dst = gg.csr_by_source(torch.as_tensor(u), torch.as_tensor(v), n)
    want = oracle.pagerank_power_f64(index.numpy(), dst.numpy(), 20, 0.85)
    touched = part.replicas > 0
    assert np.max(np.abs(results[1][2][touched] - want[touched]) / want[touched]) < 1e-4


def test_against_cpu_job_restatement(cuda_device, oracle):
    """DRONE's CPU job (float, eps 0.01, at most 200 supersteps) and the GPU schedule agree to the
    accuracy the CPU job's threshold allows."""
    n, u, v, out_deg, part = pr_case(scale=10, seed=33, parts=2)
    cpu, _, _ = oracle.pr_drone_cpu(n, part.part_u, part.part_v, out_deg, part.owner, eps=0.01, max_steps=200)
    graphs, prs = build_parts(part, n, u, v, cuda_device, True, 1e-9)
    prk.run_job_local(prs)
    got = prk.gather_global(prs, graphs, n)
    touched = (part.replicas > 0) & (out_deg > 0)
    # the CPU job ignores dangling mass; three dangling vertices of 1024 shift values by well under its threshold
    assert np.median(np.abs(got[touched] - cpu[touched]) / cpu[touched]) < 0.05


def test_call_order_is_checked(cuda_device, oracle):
    n, u, v, out_deg, part = pr_case(scale=8, seed=34, parts=1)
    graphs, prs = build_parts(part, n, u, v, cuda_device, False, 1e-6)
    with pytest.raises(db.DroneError, match="before PR_PEVal"):
        prs[0].inceval()
    res = prs[0].peval()
    assert res.LocalVertexSize == graphs[0].n_local and res.is_empty()
    assert res.VisitedSize > 0


def _nccl_rank(rank, world, port, ok):
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, u, v, out_deg, part = pr_case(scale=10, seed=35, parts=world)
        want, want_steps, _ = oracle.pr_drone_cuda(n, part.part_u, part.part_v, out_deg, part.owner, eps=1e-6,
                                                   dtype=np.float64)
        in_deg = np.bincount(v, minlength=n).astype(np.int32)
        comm = gs.Comm(rank, world)
        g = gs.DeviceGraph(part.local_graph(rank), in_deg, out_deg, dev, max_features=1)
        pr_ = prk.PageRank(g, n, comm=comm, use_double=True, eps=1e-6, n_isolated=int((part.replicas == 0).sum()))
        res = pr_.peval()
        steps = 1
        while True:
            flag = torch.tensor([0 if res.is_empty() else 1])
            dist.all_reduce(flag)                      # the master's "any worker has messages" (master.go:283-287)
            if int(flag) == 0:
                break
            res = pr_.inceval()
            steps += 1
        assert steps == want_steps
        vals = pr_.values()
        keep = g.host.mirror2worker == -1
        gid = g.host.l2g[keep]
        assert np.max(np.abs(vals[keep] - want[gid]) / want[gid]) < PR_TOL
        pr_.power_iterate(20, 0.85)
        index, dst = gg.csr_by_source(torch.as_tensor(u), torch.as_tensor(v), n)
        wantp = oracle.pagerank_power_f64(index.numpy(), dst.numpy(), 20, 0.85)
        vals = pr_.values()
        assert np.max(np.abs(vals[keep] - wantp[gid]) / wantp[gid]) < PR_TOL
        # the same job with the boundary entries stored straight into the peer's memory: same supersteps, same values
        g2 = gs.DeviceGraph(part.local_graph(rank), in_deg, out_deg, dev, max_features=4)
        g2.xplan.enable_p2p(comm)
        pr2 = prk.PageRank(g2, n, comm=comm, use_double=True, eps=1e-6, n_isolated=int((part.replicas == 0).sum()))
        assert pr2.transport_name().startswith("peer memory")
        res = pr2.peval()
        steps2 = 1
        while True:
            flag = torch.tensor([0 if res.is_empty() else 1])
            dist.all_reduce(flag)
            if int(flag) == 0:
                break
            res = pr2.inceval()
            steps2 += 1
        assert steps2 == want_steps
        vals2 = pr2.values()
        assert np.max(np.abs(vals2[keep] - want[gid]) / want[gid]) < PR_TOL
        pr2.power_iterate(20, 0.85)
        assert np.array_equal(pr2.values(), vals)
        ok[rank] = 1
        dist.barrier()
        pr2.close()
        pr_.close()
        comm.close()
    finally:
        dist.destroy_process_group()


def test_pagerank_over_nccl_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_ranks(_nccl_rank, 2, (29700 + os.getpid() % 2000,))

"""Multi-part semantics on the CPU: per-part partial aggregation + the mirror/master exchange driven
by the library's routing plan must reproduce the single-graph result (cuda_gcn/src/cuda/
cuda_communicate.cu:374-448).  One test runs the P parts in one process, another as two gloo ranks."""
import os

import numpy as np
import pytest
import torch

from drone_b200 import graphgen as gg
from drone_b200 import partition as pt


def setup_case(oracle, parts, scale=9, seed=4, f=5, sym=False):
    n, u, v = gg.rmat_graph(scale, 8, seed=seed, symmetrise=sym, self_loops="add")
    u, v = u.numpy(), v.numpy()
    in_deg = np.bincount(v, minlength=n).astype(np.int32)
    out_deg = np.bincount(u, minlength=n).astype(np.int32)
    part = pt.ebv_partition(n, u, v, parts)
    x = gg.seeded_normal(77, (n, f))
    # single-graph reference, by global id
    index, dst = gg.csr_by_source(torch.as_tensor(u), torch.as_tensor(v), n)
    val = oracle.csr_values_f32(index.numpy(), dst.numpy(), in_deg, out_deg)
    want_fwd = oracle.graphsum_forward_f64(x, index.numpy(), dst.numpy(), val)
    want_bwd = oracle.graphsum_backward_f64(x, index.numpy(), dst.numpy(), val)
    return n, part, in_deg, out_deg, x, want_fwd, want_bwd


def partial_results(oracle, part, p, in_deg, out_deg, x):
    g = part.local_graph(p)
    ind, outd = g.local_degrees(in_deg, out_deg)
    val = oracle.csr_values_f32(g.index, g.dst, ind, outd)          # GLOBAL degrees: partial sums add up
    xl = x[g.l2g]                                                    # features live on every replica
    return g, oracle.graphsum_forward_f64(xl, g.index, g.dst, val), oracle.graphsum_backward_f64(xl, g.index, g.dst, val)


def simulate_exchange(plans, rows):
    """Run the two phases with the plans' row lists; rows[p] is [n_local_p, F] float64, updated in place."""
    P = len(plans)
    lists = [pl.lists() for pl in plans]
    counts = [pl.counts() for pl in plans]
    up_off = [np.concatenate([[0], np.cumsum(c[0])]) for c in counts]
    down_off = [np.concatenate([[0], np.cumsum(c[1])]) for c in counts]
    # phase 1: mirrors -> masters, added in ascending sender order
    sent = [[rows[p][lists[p][0][up_off[p][q]:up_off[p][q + 1]]].copy() for q in range(P)] for p in range(P)]
    for q in range(P):
        for p in range(P):
            tgt = lists[q][1][down_off[q][p]:down_off[q][p + 1]]
            assert len(tgt) == len(sent[p][q])
            np.add.at(rows[q], tgt, sent[p][q])
    # phase 2: masters -> mirrors, assigned
    sent = [[rows[q][lists[q][1][down_off[q][p]:down_off[q][p + 1]]].copy() for p in range(P)] for q in range(P)]
    for p in range(P):
        for q in range(P):
            rows[p][lists[p][0][up_off[p][q]:up_off[p][q + 1]]] = sent[q][p]


@pytest.mark.parametrize("parts", [2, 3, 8])
def test_partial_sums_plus_exchange_equal_single_graph(oracle, parts):
    n, part, in_deg, out_deg, x, want_fwd, want_bwd = setup_case(oracle, parts)
    graphs, fwd, bwd = zip(*[partial_results(oracle, part, p, in_deg, out_deg, x) for p in range(parts)])
    plans = [pt.ExchangePlan(g, 16) for g in graphs]
    # the plans of different ranks agree on every pairwise count
    for p in range(parts):
        up, down, _ = plans[p].counts()
        assert up[p] == 0 and down[p] == 0
        for q in range(parts):
            assert up[q] == plans[q].counts()[1][p]
    for res, want in ((list(fwd), want_fwd), (list(bwd), want_bwd)):
        res = [r.copy() for r in res]
        simulate_exchange(plans, res)
        for p, g in enumerate(graphs):
            np.testing.assert_allclose(res[p], want[g.l2g], rtol=0, atol=1e-12)


def test_single_part_needs_no_exchange(oracle):
    n, part, in_deg, out_deg, x, want_fwd, _ = setup_case(oracle, 1)
    g, fwd, _ = partial_results(oracle, part, 0, in_deg, out_deg, x)
    plan = pt.ExchangePlan(g, 8)
    up, down, nm = plan.counts()
    assert up.sum() == 0 and down.sum() == 0 and nm == 0
    np.testing.assert_allclose(fwd, want_fwd[g.l2g], rtol=0, atol=1e-12)


def _gloo_rank(rank, world, port, ok):
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, part, in_deg, out_deg, x, want_fwd, _ = setup_case(oracle, world, scale=8, seed=6, f=4)
        g, fwd, _ = partial_results(oracle, part, rank, in_deg, out_deg, x)
        plan = pt.ExchangePlan(g, 8)
        up, down, _ = plan.counts()
        up_rows, down_rows = plan.lists()
        up_off = np.concatenate([[0], np.cumsum(up)])
        down_off = np.concatenate([[0], np.cumsum(down)])
        rows = torch.from_numpy(fwd.copy())
        f = rows.shape[1]

        def all_to_all_v(send_rows, s_off, r_off):
            recv = [torch.empty((int(r_off[q + 1] - r_off[q]), f), dtype=torch.float64) for q in range(world)]
            reqs = []
            for q in range(world):
                if q == rank:
                    continue
                reqs.append(dist.isend(rows[send_rows[s_off[q]:s_off[q + 1]]].contiguous(), q))
                reqs.append(dist.irecv(recv[q], q))
            for r in reqs:
                r.wait()
            return recv

        got = all_to_all_v(up_rows, up_off, down_off)
        for q in range(world):                                    # ascending sender order
            if q != rank and len(got[q]):
                rows.index_add_(0, torch.from_numpy(down_rows[down_off[q]:down_off[q + 1]].astype(np.int64)), got[q])
        got = all_to_all_v(down_rows, down_off, up_off)
        for q in range(world):
            if q != rank and len(got[q]):
                rows[torch.from_numpy(up_rows[up_off[q]:up_off[q + 1]].astype(np.int64))] = got[q]
        np.testing.assert_allclose(rows.numpy(), want_fwd[g.l2g], rtol=0, atol=1e-12)
        ok[rank] = 1
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ok = ctx.Array("i", [0, 0])
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, port, ok)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    assert all(p.exitcode == 0 for p in procs)
    assert list(ok) == [1, 1]


def _scatter_rank(rank, world, port, ok):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, u, v = gg.rmat_graph(10, 8, seed=19, self_loops="add")
        u, v = u.numpy(), v.numpy()
        full = pt.ebv_partition(n, u, v, world)              # every rank can compute it: the check below needs it
        in_deg = np.bincount(v, minlength=n).astype(np.int32)
        out_deg = np.bincount(u, minlength=n).astype(np.int32)
        if rank == 0:
            mine, extras, total = pt.scatter_partition(full, n, world, torch.device("cpu"), extra=(in_deg, out_deg))
        else:
            mine, extras, total = pt.scatter_partition(None, n, world, torch.device("cpu"), n_extra=2)
        assert total == len(u)
        assert np.array_equal(extras[0], in_deg) and np.array_equal(extras[1], out_deg)
        if rank != 0:
            assert all(mine.part_u[q] is None for q in range(world) if q != rank)
        a, b = mine.local_graph(rank), full.local_graph(rank)
        for name in ("l2g", "index", "dst", "master_worker_index", "master2workers", "mirror2worker"):
            assert np.array_equal(getattr(a, name), getattr(b, name)), name
        xa, xb = pt.ExchangePlan(a, 4), pt.ExchangePlan(b, 4)
        assert all(np.array_equal(p, q) for p, q in zip(xa.lists(), xb.lists()))
        dist.barrier()
        ok[rank] = 1
    finally:
        dist.destroy_process_group()


def test_partition_scatter_over_gloo_ranks():
    """The hand-out of a partition from rank 0 (what the multi-GPU benchmark does over NCCL) on three CPU ranks."""
    import torch.multiprocessing as mp
    world = 3
    ctx = mp.get_context("spawn")
    ok = ctx.Array("i", [0] * world)
    port = 29800 + os.getpid() % 1000
    procs = [ctx.Process(target=_scatter_rank, args=(r, world, port, ok)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    assert all(p.exitcode == 0 for p in procs)
    assert list(ok) == [1] * world

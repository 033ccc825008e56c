"""The exchange kernels on real devices: all parts on one GPU (device-to-device copies), and, when the
box has at least two GPUs, one process per GPU over NCCL through the GraphSum module."""
import os

import numpy as np
import pytest
import torch

import drone_b200 as db
from drone_b200 import graphgen as gg
from drone_b200 import graphsum as gs
from drone_b200 import partition as pt
from helpers import run_ranks, assert_close_to_oracle
from test_exchange_cpu import setup_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("parts,f", [(2, 32), (4, 41), (8, 64)])
def test_all_parts_on_one_gpu(cuda_device, oracle, parts, f):
    n, part, in_deg, out_deg, x, want_fwd, want_bwd = setup_case(oracle, parts, scale=11, seed=8, f=f, sym=True)
    graphs = [gs.DeviceGraph(part.local_graph(p), in_deg, out_deg, cuda_device, max_features=64) for p in range(parts)]
    for op, want in ((db.OP_AT, want_fwd), (db.OP_A, want_bwd)):
        rows = [g.plan.spmm(op, torch.as_tensor(x[g.host.l2g], device=cuda_device)) for g in graphs]
        before = [r.clone() for r in rows]
        gs.exchange_sum_local([g.xplan for g in graphs], rows)
        torch.cuda.synchronize()
        scale = np.abs(want).max()
        for p, g in enumerate(graphs):
            assert_close_to_oracle(rows[p].cpu().numpy(), want[g.host.l2g])
            # rows of unreplicated vertices are not touched by the exchange
            single = torch.as_tensor(part.replicas[g.host.l2g] == 1, device=cuda_device)
            assert torch.equal(rows[p][single], before[p][single])
        # every replica of a vertex holds the same bits
        glob = {}
        for p, g in enumerate(graphs):
            host = rows[p].cpu().numpy()
            for loc in np.nonzero(part.replicas[g.host.l2g] > 1)[0][:300]:
                key = int(g.host.l2g[loc])
                if key in glob:
                    assert np.array_equal(glob[key], host[loc])
                glob[key] = host[loc]
        assert scale > 0


@pytest.mark.parametrize("parts,groups,f", [(2, 2, 32), (4, 3, 41), (3, 4, 64)])
def test_rows_in_groups_give_the_same_bits(cuda_device, oracle, parts, groups, f):
    """Aggregating and exchanging the rows a group at a time (groups chosen from the global id, so every part makes
    the same choice) gives bit for bit the result of one aggregation followed by one exchange."""
    n, part, in_deg, out_deg, x, want_fwd, want_bwd = setup_case(oracle, parts, scale=11, seed=21, f=f, sym=True)
    graphs = [gs.DeviceGraph(part.local_graph(p), in_deg, out_deg, cuda_device, max_features=64) for p in range(parts)]
    xs = [torch.as_tensor(x[g.host.l2g], device=cuda_device) for g in graphs]
    for op, want in ((db.OP_AT, want_fwd), (db.OP_A, want_bwd)):
        whole = [g.plan.spmm(op, xx) for g, xx in zip(graphs, xs)]
        gs.exchange_sum_local([g.xplan for g in graphs], whole)
        klass = [gs.row_groups(g.host.l2g, groups) for g in graphs]
        for g, k in zip(graphs, klass):
            g.plan.set_row_classes(torch.as_tensor(k, device=cuda_device), groups)
        sub = [[pt.ExchangePlan(g.host, 64, row_mask=k == c) for c in range(groups)] for g, k in zip(graphs, klass)]
        assert sum(int(s.counts()[0].sum()) for s in sub[0]) == int(graphs[0].xplan.counts()[0].sum())
        rows = [torch.full((g.n_local, f), float("nan"), device=cuda_device) for g in graphs]
        for c in range(groups):
            for g, xx, r in zip(graphs, xs, rows):
                g.plan.spmm(op, xx, out=r, row_class=c)
            gs.exchange_sum_local([s[c] for s in sub], rows)
        all_rows = [g.plan.spmm(op, xx) for g, xx in zip(graphs, xs)]      # the plain call on a plan with classes
        gs.exchange_sum_local([g.xplan for g in graphs], all_rows)
        torch.cuda.synchronize()
        for p, g in enumerate(graphs):
            assert torch.equal(rows[p], whole[p])
            assert torch.equal(all_rows[p], whole[p])
            assert_close_to_oracle(rows[p].cpu().numpy(), want[g.host.l2g])
        for g in graphs:
            g.plan.set_row_classes(None, 1)
        again = [g.plan.spmm(op, xx) for g, xx in zip(graphs, xs)]
        gs.exchange_sum_local([g.xplan for g in graphs], again)
        for p in range(parts):
            assert torch.equal(again[p], whole[p])


@pytest.mark.parametrize("f,ld", [(64, 64), (41, 41), (32, 40), (1, 1)])
def test_clear_mirror_rows(cuda_device, f, ld):
    """drone_clear_mirror_rows zeroes exactly the rows whose Mirror2Worker entry is not -1 (clear_mirror_grad)."""
    n = 1000
    rng = np.random.default_rng(f)
    m2w = np.where(rng.random(n) < 0.3, rng.integers(0, 4, n), -1).astype(np.int32)
    big = torch.as_tensor(rng.standard_normal((n, ld)).astype(np.float32), device=cuda_device)
    before = big.clone()
    gs.clear_mirror_rows(big[:, :f], torch.as_tensor(m2w, device=cuda_device))
    mirrors = torch.as_tensor(m2w != -1, device=cuda_device)
    assert (big[mirrors][:, :f] == 0).all()
    assert torch.equal(big[~mirrors], before[~mirrors])
    assert torch.equal(big[:, f:], before[:, f:])          # padding columns untouched
    lib = db.lib()
    assert lib.drone_clear_mirror_rows(None, 5, 4, 4, None, None) == -1 and b"NULL" in lib.drone_last_error()
    assert lib.drone_clear_mirror_rows(None, 5, 8, 4, None, None) == -1


def test_row_classes_check_arguments(cuda_device):
    n, u, v = gg.rmat_graph(9, 8, seed=5, device=cuda_device, self_loops="add")
    index, dst = gg.csr_by_source(u, v, n)
    ind, outd = gg.degrees(u, v, n)
    plan = db.AggregationPlan(index, dst, in_degree=ind, out_degree=outd)
    x = torch.randn((n, 8), device=cuda_device)
    with pytest.raises(db.DroneError, match="row_class"):
        plan.spmm(db.OP_AT, x, row_class=1)                 # no classes set
    bad = torch.full((n,), 3, dtype=torch.int32, device=cuda_device)
    with pytest.raises(db.DroneError, match="class outside"):
        plan.set_row_classes(bad, 2)
    with pytest.raises(db.DroneError, match="n_classes"):
        plan.set_row_classes(bad, 17)
    want = plan.spmm(db.OP_AT, x)                           # the failed calls left the plan usable
    assert torch.isfinite(want).all()
    good = (torch.arange(n, device=cuda_device) % 2).to(torch.int32)
    plan.set_row_classes(good, 2)
    with pytest.raises(db.DroneError, match="class outside"):
        plan.set_row_classes(bad, 3)                        # rejected before anything changes: still two classes
    out = torch.zeros_like(want)
    plan.spmm(db.OP_AT, x, out=out, row_class=0)
    plan.spmm(db.OP_AT, x, out=out, row_class=1)
    assert torch.equal(out, want)
    with pytest.raises(db.DroneError, match="row_class"):
        plan.spmm(db.OP_AT, x, out=out, row_class=2)


def test_exchange_is_repeatable_and_checks_arguments(cuda_device, oracle):
    n, part, in_deg, out_deg, x, want_fwd, _ = setup_case(oracle, 3, scale=10, seed=9, f=16)
    graphs = [gs.DeviceGraph(part.local_graph(p), in_deg, out_deg, cuda_device, max_features=16) for p in range(3)]
    outs = []
    for _ in range(2):
        rows = [g.plan.spmm(db.OP_AT, torch.as_tensor(x[g.host.l2g], device=cuda_device)) for g in graphs]
        gs.exchange_sum_local([g.xplan for g in graphs], rows)
        outs.append([r.clone() for r in rows])
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    wide = [torch.zeros((g.n_local, 32), device=cuda_device) for g in graphs]
    with pytest.raises(db.DroneError, match="max_features|F="):
        gs.exchange_sum_local([g.xplan for g in graphs], wide)


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
        f = 32
        n, part, in_deg, out_deg, x, want_fwd, want_bwd = setup_case(oracle, world, scale=11, seed=10, f=f, sym=True)
        comm = gs.Comm(rank, world)
        g = gs.DeviceGraph(part.local_graph(rank), in_deg, out_deg, dev, max_features=f)
        a, b = gs.Variable(g.n_local, f, dev), gs.Variable(g.n_local, f, dev)
        layer = gs.GraphSum(a, b, g, comm, f, rank, world, "graphSum_test", 0)
        a.data.copy_(torch.as_tensor(x[g.host.l2g]))
        layer.forward(True)
        b.grad.copy_(torch.as_tensor(x[g.host.l2g]))
        layer.backward()
        torch.cuda.synchronize()
        assert_close_to_oracle(b.data.cpu().numpy(), want_fwd[g.host.l2g])
        assert_close_to_oracle(a.grad.cpu().numpy(), want_bwd[g.host.l2g])
        # reduce-scatter + all-gather over the dense boundary buffer: same values to rounding
        dense = pt.DenseExchangePlan(part, g.host, f)
        assert dense.boundary_rows() >= int((part.replicas > 1).sum())
        rs = g.plan.spmm(db.OP_AT, a.data)
        gs.exchange_sum_dense(dense, comm, rs)
        torch.cuda.synchronize()
        assert_close_to_oracle(rs.cpu().numpy(), want_fwd[g.host.l2g])
        assert (rs - b.data).abs().max().item() <= 1e-5 * b.data.abs().max().item()
        # the peer-memory transport gives the same bits, call after call, without host synchronisation in between
        nccl_fwd, nccl_bwd = b.data.clone(), a.grad.clone()
        g.xplan.enable_p2p(comm)
        for _ in range(5):
            layer.forward(True)
            layer.backward()
        torch.cuda.synchronize()
        assert torch.equal(b.data, nccl_fwd) and torch.equal(a.grad, nccl_bwd)
        # aggregation and exchange overlapped over four row groups: the same bits again
        piped = gs.PipelinedAggregation(g, comm, f, n_groups=4)
        for op, src, want_bits in ((db.OP_AT, a.data, nccl_fwd), (db.OP_A, b.grad, nccl_bwd)):
            for _ in range(3):
                out = torch.full((g.n_local, f), float("nan"), device=dev)
                piped(op, src, out)
                torch.cuda.synchronize()
                assert torch.equal(out, want_bits)
        piped.close()
        g.plan.set_row_classes(None, 1)
        narrow = torch.as_tensor(x[g.host.l2g][:, :5].copy(), device=dev)      # a width below max_features
        ref = g.plan.spmm(db.OP_AT, narrow)
        gs.exchange_sum(g.xplan, comm, ref)
        torch.cuda.synchronize()
        assert_close_to_oracle(ref.cpu().numpy(), want_fwd[g.host.l2g][:, :5])
        dist.barrier()
        ok[rank] = 1
        dist.barrier()
        comm.close()
    finally:
        dist.destroy_process_group()


def _lonely_rank(rank, world, port, ok):
    """Rank 0 starts an exchange that rank 1 never joins: its bounded wait must run out and be reported."""
    import time
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, part, in_deg, out_deg, x, _, _ = setup_case(oracle, world, scale=9, seed=12, f=8, sym=True)
        comm = gs.Comm(rank, world)
        g = gs.DeviceGraph(part.local_graph(rank), in_deg, out_deg, dev, max_features=8)
        g.xplan.enable_p2p(comm)
        rows = torch.ones((g.n_local, 8), device=dev)
        gs.exchange_sum(g.xplan, comm, rows)            # both ranks: fine
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            t0 = time.time()
            gs.exchange_sum(g.xplan, comm, rows)        # alone: the kernels give up after their wait limit
            torch.cuda.synchronize()
            assert time.time() - t0 < 30
            with pytest.raises(db.DroneError, match="gave up waiting for rank 1"):
                gs.exchange_sum(g.xplan, comm, rows)
            assert float(torch.ones(4, device=dev).sum()) == 4.0    # the context is still usable
        dist.barrier()
        if rank == 1:
            # the call rank 0 gave up on, made late: rank 0 published its rows of that call before its wait ran out,
            # but no totals afterwards, so this rank must not take stale totals for good ones: its own wait runs out
            t0 = time.time()
            gs.exchange_sum(g.xplan, comm, rows)
            torch.cuda.synchronize()
            assert time.time() - t0 < 30
            with pytest.raises(db.DroneError, match="gave up waiting for rank 0"):
                gs.exchange_sum(g.xplan, comm, rows)
            assert float(torch.ones(4, device=dev).sum()) == 4.0
        ok[rank] = 1
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _mismatched_rank(rank, world, port, ok):
    """The two ranks plan for different feature widths: switching the peer-memory transport on fails with the same
    code on both (nobody is left inside a collective), and the NCCL transport still works afterwards."""
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        f = 8
        n, part, in_deg, out_deg, x, want_fwd, _ = setup_case(oracle, world, scale=9, seed=13, f=f, sym=True)
        comm = gs.Comm(rank, world)
        g = gs.DeviceGraph(part.local_graph(rank), in_deg, out_deg, dev, max_features=f if rank == 0 else 2 * f)
        with pytest.raises(db.DroneError) as err:
            g.xplan.enable_p2p(comm)
        assert err.value.code == -1 and "planned for" in str(err.value)
        dist.barrier()
        rows = g.plan.spmm(db.OP_AT, torch.as_tensor(x[g.host.l2g], device=dev))
        gs.exchange_sum(g.xplan, comm, rows)            # grouped send/recv, as before the attempt
        torch.cuda.synchronize()
        assert_close_to_oracle(rows.cpu().numpy(), want_fwd[g.host.l2g])
        ok[rank] = 1
        dist.barrier()
        comm.close()
    finally:
        dist.destroy_process_group()


def _fused_push_rank(rank, world, port, ok):
    """The aggregation that sends its mirror rows up itself (push_up_to) + drone_exchange_finish against aggregation
    followed by the whole exchange: the same bits at every width, in one piece, in column slices and in row groups."""
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fmax = 128
        n, part, in_deg, out_deg, x, want_fwd, want_bwd = setup_case(oracle, world, scale=11, seed=12, f=fmax, sym=False)
        comm = gs.Comm(rank, world)
        # plans in one piece, cut into column slices, and with a table of hot rows (tagged columns)
        for slice_width, plan_env in ((None, {}), ("32", {"DRONE_SLICE_WIDTH": "32"}),
                                      (None, {"DRONE_HOT_MIN_ROWS": "1", "DRONE_HOT_TABLE_MB": "1"})):
            os.environ.update(plan_env)
            g = gs.DeviceGraph(part.local_graph(rank), in_deg, out_deg, dev, max_features=fmax)
            for key in plan_env:
                os.environ.pop(key, None)
            assert (g.plan.stats().hot_rows_tagged > 0) == ("DRONE_HOT_MIN_ROWS" in plan_env)
            g.plan.reserve(47, padded_rows=True)
            g.xplan.enable_p2p(comm)
            xl = torch.as_tensor(x[g.host.l2g], device=dev)
            for f in (128, 64, 41, 8, 3):
                src = xl[:, :f].contiguous()
                for op, want in ((db.OP_AT, want_fwd), (db.OP_A, want_bwd)):
                    plain = g.plan.spmm(op, src)
                    gs.exchange_sum(g.xplan, comm, plain)
                    for _ in range(3):      # call after call, no host synchronisation in between
                        fused = torch.full((g.n_local, f), float("nan"), device=dev)
                        g.plan.spmm(op, src, out=fused, push_up_to=g.xplan.handle)
                        gs.exchange_finish(g.xplan, fused)
                    torch.cuda.synchronize()
                    assert torch.equal(fused, plain), (slice_width, f, op)
                    assert_close_to_oracle(fused.cpu().numpy(), want[g.host.l2g][:, :f])
            # value-free coefficients with the row factor applied in the store: the scaled row is what leaves
            scale = torch.rand(g.n_local, device=dev) + 0.5
            src = xl[:, :64].contiguous()
            plain = g.plan.spmm(db.OP_A, src, unit_values=True, row_scale=scale)
            gs.exchange_sum(g.xplan, comm, plain)
            fused = torch.full((g.n_local, 64), float("nan"), device=dev)
            g.plan.spmm(db.OP_A, src, out=fused, unit_values=True, row_scale=scale, push_up_to=g.xplan.handle)
            gs.exchange_finish(g.xplan, fused)
            torch.cuda.synchronize()
            assert torch.equal(fused, plain)
            if slice_width:      # the calls above did run in slices
                g.plan.spmm(db.OP_AT, xl[:, :64].contiguous())
                assert g.plan.stats().last_slice_width == 32
            # a padded leading dimension on both operands
            wide_x = torch.zeros((g.n_local, 72), device=dev)
            wide_x[:, :64] = xl[:, :64]
            wide_y = torch.full((g.n_local, 72), 7.0, device=dev)
            g.plan.spmm(db.OP_AT, wide_x[:, :64], out=wide_y[:, :64], push_up_to=g.xplan.handle)
            gs.exchange_finish(g.xplan, wide_y[:, :64])
            ref = g.plan.spmm(db.OP_AT, xl[:, :64].contiguous())
            gs.exchange_sum(g.xplan, comm, ref)
            torch.cuda.synchronize()
            assert torch.equal(wide_y[:, :64], ref) and bool((wide_y[:, 64:] == 7.0).all())
            # call order is checked: the rest of the exchange needs a call that sent the rows, and only one
            with pytest.raises(db.DroneError, match="no aggregation call has sent"):
                gs.exchange_finish(g.xplan, ref)
            g.plan.spmm(db.OP_AT, xl[:, :64].contiguous(), out=ref, push_up_to=g.xplan.handle)
            with pytest.raises(db.DroneError, match="drone_exchange_finish is due"):
                gs.exchange_sum(g.xplan, comm, ref)
            with pytest.raises(db.DroneError, match="drone_exchange_finish is due"):
                g.plan.spmm(db.OP_AT, xl[:, :64].contiguous(), out=ref, push_up_to=g.xplan.handle)
            gs.exchange_finish(g.xplan, ref)
            with pytest.raises(db.DroneError, match="cannot be combined"):
                g.plan.spmm(db.OP_AT, xl[:, :64].contiguous(), out=ref, relu=True, push_up_to=g.xplan.handle)
            # row groups, mirror rows leaving from each group's aggregation, against the copy-kernel form
            want_bits = {}
            for f in (64, 41):
                want_bits[f] = g.plan.spmm(db.OP_AT, xl[:, :f].contiguous())
                gs.exchange_sum(g.xplan, comm, want_bits[f])
            for fused_push in (True, False):
                piped = gs.PipelinedAggregation(g, comm, fmax, n_groups=3, fused_push=fused_push)
                for f in (64, 41):
                    src = xl[:, :f].contiguous()
                    out = torch.full((g.n_local, f), float("nan"), device=dev)
                    for _ in range(2):
                        piped(db.OP_AT, src, out)
                    torch.cuda.synchronize()
                    assert torch.equal(out, want_bits[f]), (fused_push, f)
                piped.close()
                g.plan.set_row_classes(None, 1)
            dist.barrier()
            g.xplan.close()
        ok[rank] = 1
        dist.barrier()
        comm.close()
    finally:
        dist.destroy_process_group()


def test_mirror_rows_sent_from_the_aggregation_store():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_ranks(_fused_push_rank, 2, (28300 + os.getpid() % 2000,))


def test_peer_transport_setup_fails_on_every_rank_together():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_ranks(_mismatched_rank, 2, (29100 + os.getpid() % 2000,))


def test_peer_wait_runs_out_instead_of_hanging():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_ranks(_lonely_rank, 2, (29900 + os.getpid() % 2000,))



def test_graphsum_over_nccl_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_ranks(_nccl_rank, 2, (29600 + os.getpid() % 2000,))


def test_push_up_to_needs_the_peer_transport_and_is_nothing_on_one_rank(cuda_device, oracle):
    """push_up_to on an exchange plan without the peer-memory transport is refused before anything is launched; on
    a one-rank plan there is nobody to send to, and the two calls give the plain aggregation."""
    n, part, in_deg, out_deg, x, want_fwd, _ = setup_case(oracle, 2, scale=10, seed=9, f=16)
    g = gs.DeviceGraph(part.local_graph(0), in_deg, out_deg, cuda_device, max_features=16)
    xl = torch.as_tensor(x[g.host.l2g], device=cuda_device)
    with pytest.raises(db.DroneError, match="peer-memory transport is not enabled"):
        g.plan.spmm(db.OP_AT, xl, push_up_to=g.xplan.handle)
    with pytest.raises(db.DroneError, match="no aggregation call has sent"):
        gs.exchange_finish(g.xplan, xl)
    n1, part1, in1, out1, x1, want1, _ = setup_case(oracle, 1, scale=10, seed=9, f=16)
    g1 = gs.DeviceGraph(part1.local_graph(0), in1, out1, cuda_device, max_features=16)
    x1l = torch.as_tensor(x1[g1.host.l2g], device=cuda_device)
    y = g1.plan.spmm(db.OP_AT, x1l, push_up_to=g1.xplan.handle)
    gs.exchange_finish(g1.xplan, y)
    assert torch.equal(y, g1.plan.spmm(db.OP_AT, x1l))
    assert_close_to_oracle(y.cpu().numpy(), want1[g1.host.l2g])

"""The reference ITSELF (its CUDAGraphSum over cuSPARSE, compiled from its own sources into oracle/_ref) against
the oracle and against the library, on identical seeded inputs.  This is what pins the oracle: coefficients must be
bit-identical, outputs and gradients within 1e-5."""
import os

import numpy as np
import pytest
import torch

import drone_b200 as db
from drone_b200 import graphgen as gg
from helpers import REL_TOL

pytestmark = pytest.mark.gpu


def test_reference_training_epoch_loss_vs_oracle_and_library(cuda_device, oracle):
    """The reference's own CUDAGCN::train_epoch (cuSPARSE aggregation, cuBLAS layers, its cross-entropy) on one
    worker: the loss of the first epoch equals the double oracle's and this library's GCN step on the same graph,
    features, labels and starting weights to 1e-5.  Pins oracle/gcn_oracle.py against the reference itself."""
    if not oracle.reference_available():
        pytest.skip("oracle/_ref/libref_graphsum.so was not built (reference tree absent at build time)")
    from drone_b200 import gcn, graphsum as gs, partition as pt
    from helpers import graph_case
    from oracle import gcn_oracle
    dims = (40, 32, 7)
    n, u, v = gg.rmat_graph(10, 12, seed=91, symmetrise=True, self_loops="add")
    u, v = u.numpy(), v.numpy()
    x = gg.seeded_normal(3, (n, dims[0]))
    truth = np.random.default_rng(4).integers(0, dims[2], n).astype(np.int32)      # the reference trains on every row
    w1, w2 = [w.numpy() for w in gg.glorot_weights(dims, "cpu", seed=5)]
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u, v)
    want = gcn_oracle.gcn_step(index, dst, val, x, w1, w2, truth)
    ms, book, ref_loss = oracle.reference_gcn_epochs(n, u, v, in_deg, out_deg, dims, x, truth, w1, w2, warmup=1, epochs=1)
    assert ms > 0 and book > 0
    assert abs(ref_loss - want["loss"]) <= 1e-5 * max(1.0, abs(want["loss"]))
    part = pt.ebv_partition(n, u, v, 1)
    lg = part.local_graph(0)
    g = gs.DeviceGraph(lg, in_deg, out_deg, cuda_device, max_features=32)
    t = lambda a: torch.as_tensor(a, device=cuda_device)
    torch.backends.cuda.matmul.allow_tf32 = False
    step = gcn.GCNStep(g, t(x[lg.l2g]), t(truth[lg.l2g]), t(w1), t(w2))
    assert abs(float(step.forward()) - ref_loss) <= 1e-5 * max(1.0, abs(ref_loss))


@pytest.mark.parametrize("scale,sym,dim", [(10, True, 64), (11, False, 41), (9, False, 128)])
def test_reference_graphsum_vs_oracle_and_library(cuda_device, oracle, scale, sym, dim):
    if not oracle.reference_available():
        pytest.skip("oracle/_ref/libref_graphsum.so was not built (reference tree absent at build time)")
    n, u, v = gg.rmat_graph(scale, 12, seed=81 + scale, symmetrise=sym, self_loops="add")
    u, v = u.numpy(), v.numpy()
    in_deg = np.bincount(v, minlength=n).astype(np.int32)
    out_deg = np.bincount(u, minlength=n).astype(np.int32)
    x = gg.seeded_normal(dim, (n, dim))
    gy = gg.seeded_normal(dim + 7, (n, dim))
    l2g, ref_fwd, ref_bwd, ref_val = oracle.reference_graphsum(n, u, v, in_deg, out_deg, x, gy)

    # the oracle's restatement of the local graph and of the coefficients is exact
    nloc, g2l, o_l2g, index, dst = oracle.build_graph(n, u, v)
    assert nloc == len(l2g) and np.array_equal(o_l2g, l2g)
    ind_l, outd_l = in_deg[l2g], out_deg[l2g]
    val = oracle.csr_values_f32(index, dst, ind_l, outd_l)
    assert np.array_equal(val, ref_val)
    # outputs / gradients: double oracle vs the reference's cuSPARSE result
    xl, gl = x[l2g], gy[l2g]
    want_f = oracle.graphsum_forward_f64(xl, index, dst, val)
    want_b = oracle.graphsum_backward_f64(gl, index, dst, val)
    for got, want in ((ref_fwd, want_f), (ref_bwd, want_b)):
        assert np.abs(got - want).max() <= REL_TOL * np.abs(want).max()
    # the library on the same local graph
    t = lambda a: torch.as_tensor(a, device=cuda_device)
    plan = db.AggregationPlan(t(index), t(dst), in_degree=t(ind_l), out_degree=t(outd_l))
    mine_f = plan.spmm(db.OP_AT, t(xl)).cpu().numpy()
    mine_b = plan.spmm(db.OP_A, t(gl)).cpu().numpy()
    assert np.abs(mine_f - ref_fwd).max() <= REL_TOL * np.abs(ref_fwd).max()
    assert np.abs(mine_b - ref_bwd).max() <= REL_TOL * np.abs(ref_bwd).max()
    # and the library is at least as close to the double result as the reference is
    assert np.abs(mine_f - want_f).max() <= 2 * max(np.abs(ref_fwd - want_f).max(), 1e-7 * np.abs(want_f).max())


def _two_reference_workers(rank, world, workdir, ok):
    """Both sides of the comparison run their own exchange between two GPUs: the reference its grouped NCCL
    send/recv with ids and atomics, the library its peer-memory transport over the static plan."""
    import torch.distributed as dist
    from oracle import oracle
    from drone_b200 import graphsum as gs
    from drone_b200 import partition as pt
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ["DRONE_REF_ID_FILE"] = os.path.join(workdir, "ref_nccl.id")
    os.environ["DRONE_REF_RANK"] = str(rank)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(29200 + os.getppid() % 2000)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dim = 32
    n, u, v = gg.rmat_graph(11, 10, seed=91, symmetrise=True, self_loops="add")
    u, v = u.numpy(), v.numpy()
    in_deg = np.bincount(v, minlength=n).astype(np.int32)
    out_deg = np.bincount(u, minlength=n).astype(np.int32)
    x = gg.seeded_normal(5, (n, dim))
    gy = gg.seeded_normal(6, (n, dim))
    part = pt.ebv_partition(n, u, v, world)
    l2g, ref_fwd, ref_bwd = oracle.reference_graphsum_worker(part, rank, in_deg, out_deg, x, gy)
    dist.barrier()
    # the double oracle on the whole graph: every replica row must hold the global sum
    index, dst = gg.csr_by_source(torch.as_tensor(u), torch.as_tensor(v), n)
    val = oracle.csr_values_f32(index.numpy(), dst.numpy(), in_deg, out_deg)
    want_f = oracle.graphsum_forward_f64(x, index.numpy(), dst.numpy(), val)[l2g]
    want_b = oracle.graphsum_backward_f64(gy, index.numpy(), dst.numpy(), val)[l2g]
    assert np.abs(ref_fwd - want_f).max() <= REL_TOL * np.abs(want_f).max()
    assert np.abs(ref_bwd - want_b).max() <= REL_TOL * np.abs(want_b).max()
    # the library, same partition, its own exchange
    lg = part.local_graph(rank)
    assert np.array_equal(lg.l2g, l2g)
    comm = gs.Comm(rank, world)
    g = gs.DeviceGraph(lg, in_deg, out_deg, dev, max_features=dim)
    g.xplan.enable_p2p(comm)
    mine_f = g.plan.spmm(db.OP_AT, torch.as_tensor(x[l2g], device=dev))
    gs.exchange_sum(g.xplan, comm, mine_f)
    mine_b = g.plan.spmm(db.OP_A, torch.as_tensor(gy[l2g], device=dev))
    gs.exchange_sum(g.xplan, comm, mine_b)
    torch.cuda.synchronize()
    assert np.abs(mine_f.cpu().numpy() - ref_fwd).max() <= REL_TOL * np.abs(ref_fwd).max()
    assert np.abs(mine_b.cpu().numpy() - ref_bwd).max() <= REL_TOL * np.abs(ref_bwd).max()
    dist.barrier()
    ok[rank] = 1
    comm.close()
    dist.destroy_process_group()


def test_reference_graphsum_two_workers(tmp_path, oracle):
    if not oracle.reference_available():
        pytest.skip("oracle/_ref/libref_graphsum.so was not built (reference tree absent at build time)")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ok = ctx.Array("i", [0, 0])
    procs = [ctx.Process(target=_two_reference_workers, args=(r, 2, str(tmp_path), ok)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=150)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs)
    assert list(ok) == [1, 1]

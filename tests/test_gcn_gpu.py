"""End-to-end check of the aggregation path inside the reference's 2-layer GCN step: outputs and gradients against
the double-precision oracle (1e-5 relative), on one GPU and, with two GPUs, as two EBV parts over NCCL."""
import os

import numpy as np
import pytest
import torch

import drone_b200 as db
from drone_b200 import gcn, graphgen as gg, graphsum as gs, partition as pt
from helpers import run_ranks, graph_case
from oracle import gcn_oracle

pytestmark = pytest.mark.gpu
GCN_TOL = 1e-5


def glorot(seed, fan_in, fan_out):
    """(U - 0.5) * 2 * sqrt(6 / (in + out)) (cuda_gcn/src/cuda/cuda_kernel.cu:469-474), from a fixed seed."""
    rng = np.random.default_rng(seed)
    return ((rng.random((fan_in, fan_out)) - 0.5) * 2 * np.sqrt(6.0 / (fan_in + fan_out))).astype(np.float32)


def make_case(scale=10, dims=(40, 32, 7)):
    n, u, v = gg.rmat_graph(scale, 12, seed=51, symmetrise=True, self_loops="add")
    u, v = u.numpy(), v.numpy()
    x = gg.seeded_normal(3, (n, dims[0]))
    truth = np.random.default_rng(4).integers(-1, dims[2], n).astype(np.int32)     # -1: unlabelled
    return n, u, v, x, truth, glorot(5, dims[0], dims[1]), glorot(6, dims[1], dims[2])


def rel(got, want):
    return float(np.abs(np.asarray(got, np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


def test_gcn_step_single_gpu(cuda_device, oracle):
    n, u, v, x, truth, w1, w2 = make_case()
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u, v)
    want = gcn_oracle.gcn_step(index, dst, val, x, w1, w2, truth)
    part = pt.ebv_partition(n, u, v, 1)
    lg = part.local_graph(0)
    g = gs.DeviceGraph(lg, in_deg, out_deg, cuda_device, max_features=32)
    t = lambda a: torch.as_tensor(a, device=cuda_device)
    torch.backends.cuda.matmul.allow_tf32 = False
    step = gcn.GCNStep(g, t(x[lg.l2g]), t(truth[lg.l2g]), t(w1), t(w2))
    loss = step.forward()
    step.backward()
    torch.cuda.synchronize()
    inv = lg.l2g
    assert rel(step.logits.cpu().numpy(), want["logits"][inv]) < GCN_TOL
    assert rel(step.z1.cpu().numpy(), want["z1"][inv]) < GCN_TOL
    assert abs(float(loss) - want["loss"]) < GCN_TOL * max(1.0, abs(want["loss"]))
    assert rel(step.d_h2.cpu().numpy(), want["d_h2"][inv]) < GCN_TOL
    assert rel(step.d_h1.cpu().numpy(), want["d_h1"][inv]) < GCN_TOL
    assert rel(step.d_w2.cpu().numpy(), want["d_w2"]) < GCN_TOL
    assert rel(step.d_w1.cpu().numpy(), want["d_w1"]) < GCN_TOL


def _rank(rank, world, port, ok):
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, u, v, x, truth, w1, w2 = make_case()
        index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u, v)
        want = gcn_oracle.gcn_step(index, dst, val, x, w1, w2, truth)
        part = pt.ebv_partition(n, u, v, world)
        lg = part.local_graph(rank)
        g = gs.DeviceGraph(lg, in_deg, out_deg, dev, max_features=32)
        comm = gs.Comm(rank, world)
        t = lambda a: torch.as_tensor(a, device=dev)
        torch.backends.cuda.matmul.allow_tf32 = False
        step = gcn.GCNStep(g, t(x[lg.l2g]), t(truth[lg.l2g]), t(w1), t(w2), comm=comm, worker_num=world)
        if rank != 0:                     # weights live on rank 0 and are broadcast at the start of every forward pass
            step.weights[0].zero_()
            step.weights[1].zero_()
        step.broadcast_weights()          # weight_broadcast_value_nccl (cuda_communicate.cu:99-105)
        step.forward()
        d_w1, d_w2 = step.backward()
        step.reduce_gradients()           # weight_reduce_grad_nccl: the sums land on rank 0 (cuda_communicate.cu:107-115)
        torch.cuda.synchronize()
        assert rel(step.logits.cpu().numpy(), want["logits"][lg.l2g]) < GCN_TOL
        # mirror rows of the layer gradients are zeroed in place before dW, as clear_mirror_grad does
        masters = lg.mirror2worker == -1
        assert rel(step.d_h1.cpu().numpy()[masters], want["d_h1"][lg.l2g][masters]) < GCN_TOL
        assert not step.d_h1.cpu().numpy()[~masters].any()
        if rank == 0:
            assert rel(d_w2.cpu().numpy(), want["d_w2"]) < GCN_TOL
            assert rel(d_w1.cpu().numpy(), want["d_w1"]) < GCN_TOL
        ok[rank] = 1
        dist.barrier()
        comm.close()
    finally:
        dist.destroy_process_group()


def test_gcn_step_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_ranks(_rank, 2, (29800 + os.getpid() % 2000,))

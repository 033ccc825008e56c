"""The cc_cuda / sssp_cuda jobs through the C ABI against the CPU restatement: values bit for bit, and the
Response sizes of every superstep."""
import os

import numpy as np
import pytest
import torch

import drone_b200 as db
from helpers import run_ranks
from drone_b200 import graphgen as gg
from drone_b200 import graphsum as gs
from drone_b200 import minprop as mp
from drone_b200 import partition as pt
from test_minprop_oracle import csr

pytestmark = pytest.mark.gpu


def graph_case(scale, ef, seed, sym):
    n, u, v = gg.rmat_graph(scale, ef, seed=seed, symmetrise=sym, self_loops="drop")
    return n, u.numpy().astype(np.int32), v.numpy().astype(np.int32)


def local_lengths(local_graph, pu, w):
    """Edge lengths of one part in the order of its CSR (rows by local id, edge-list order inside a row)."""
    order = np.argsort(local_graph.g2l[pu], kind="stable")
    return np.ascontiguousarray(w[order], dtype=np.float32)


def build(part, device, lens=None):
    zeros = np.zeros(part.n_vertices, np.int32)
    graphs = [gs.DeviceGraph(part.local_graph(p), zeros + 1, zeros + 1, device, max_features=1) for p in range(part.n_parts)]
    dl = [None] * part.n_parts
    if lens is not None:
        dl = [torch.as_tensor(local_lengths(g.host, part.part_u[p], lens[p]), device=device) for p, g in enumerate(graphs)]
    return graphs, dl


def sizes_of(history):
    return np.array([[[r.Mirror2MasterSendSize, r.Mirror2MasterRecvSize, r.Master2MirrorSendSize,
                       r.Master2MirrorRecvSize, r.VisitedSize] for r in step] for step in history], np.int64)


@pytest.mark.parametrize("parts,sym", [(1, False), (1, True), (2, False), (3, True), (8, False)])
def test_labels_match_the_restatement(cuda_device, oracle, parts, sym):
    n, u, v = graph_case(11, 6, 31, sym)
    rowptr, col, _ = csr(n, u, v)
    want = oracle.cc_fixed_point(rowptr, col)
    part = pt.ebv_partition(n, u, v, parts, keep_self_loops=False)
    graphs, _ = build(part, cuda_device)
    jobs = [mp.MinProp(g, mp.CC) for g in graphs]
    history = mp.run_job_local(jobs)
    got = mp.gather_global(jobs, graphs, n, -1)
    touched = part.replicas > 0
    assert np.array_equal(got[touched], want[touched])
    ref_vals, ref_steps, ref_sizes = oracle.mp_drone_cuda(oracle.MP_CC, n, part.part_u, part.part_v, part.owner)
    assert len(history) == ref_steps
    assert np.array_equal(sizes_of(history), ref_sizes)
    assert all(r.LocalVertexSize == g.n_local for r, g in zip(history[0], graphs))
    # every replica ends with its master's label
    for job, g in zip(jobs, graphs):
        assert np.array_equal(job.values(), want[g.host.l2g])
    if sym:
        assert all(want[a] == want[b] for a, b in zip(u[:2000], v[:2000]))


@pytest.mark.parametrize("parts,weighted", [(1, False), (1, True), (2, False), (4, True), (8, True)])
def test_distances_match_the_restatement(cuda_device, oracle, parts, weighted):
    n, u, v = graph_case(11, 6, 33, False)
    rng = np.random.default_rng(5)
    w = rng.uniform(0.1, 2.0, len(u)).astype(np.float32) if weighted else None
    rowptr, col, wl = csr(n, u, v, w)
    source = int(u[len(u) // 3])
    want = oracle.sssp_f32(rowptr, col, source, wl)
    assert (want < 1e8).sum() > n // 20
    part = pt.ebv_partition(n, u, v, parts, keep_self_loops=False)
    lens = None
    if weighted:
        key = {(int(a), int(b)): c for a, b, c in zip(u, v, w)}
        lens = [np.array([key[(int(a), int(b))] for a, b in zip(pu, pv)], np.float32)
                for pu, pv in zip(part.part_u, part.part_v)]
    graphs, dl = build(part, cuda_device, lens)
    jobs = [mp.MinProp(g, mp.SSSP, edge_len=l) for g, l in zip(graphs, dl)]
    history = mp.run_job_local(jobs, source=source)
    got = mp.gather_global(jobs, graphs, n, -1.0)
    touched = part.replicas > 0
    assert np.array_equal(got[touched], want[touched])          # float32, bit for bit
    _, ref_steps, ref_sizes = oracle.mp_drone_cuda(oracle.MP_SSSP, n, part.part_u, part.part_v, part.owner,
                                                   source=source, parts_len=lens)
    assert len(history) == ref_steps
    assert np.array_equal(sizes_of(history), ref_sizes)
    # a second run from another source on the same handles starts from scratch
    source2 = int(v[7])
    mp.run_job_local(jobs, source=source2)
    want2 = oracle.sssp_f32(rowptr, col, source2, wl)
    got2 = mp.gather_global(jobs, graphs, n, -1.0)
    assert np.array_equal(got2[touched], want2[touched])


def test_hub_rows_and_wrong_call_order(cuda_device, oracle):
    # a star with a 5000-edge hub exercises the warp-wide row walk; the source sits at the far end of a path into it
    hub, leaves, tail = 0, np.arange(1, 5001, dtype=np.int32), np.arange(5001, 5011, dtype=np.int32)
    u = np.concatenate([np.full(len(leaves), hub, np.int32), tail, [tail[0] - 0]]).astype(np.int32)
    v = np.concatenate([leaves, np.concatenate([tail[1:], [hub]]), [hub]]).astype(np.int32)
    n = 5011
    rowptr, col, _ = csr(n, u, v)
    part = pt.ebv_partition(n, u, v, 1, keep_self_loops=False)
    graphs, _ = build(part, cuda_device)
    job = mp.MinProp(graphs[0], mp.SSSP)
    with pytest.raises(db.DroneError, match="before PEVal"):
        job.inceval()
    res = job.peval(int(tail[0]))
    assert res.is_empty() and res.LocalVertexSize == graphs[0].n_local
    want = oracle.sssp_f32(rowptr, col, int(tail[0]))
    got = mp.gather_global([job], graphs, n, -1.0)
    assert np.array_equal(got, want)
    assert got[leaves].max() == got[hub] + 1
    labels = mp.MinProp(graphs[0], mp.CC)
    labels.peval()
    assert np.array_equal(mp.gather_global([labels], graphs, n, -1), oracle.cc_fixed_point(rowptr, col))
    idle = job.peval(n + 5)                  # a source nobody holds: nothing to do, nothing reached
    assert idle.is_empty() and (job.values() == np.float32(1e8)).all()


def _rank(rank, world, port, ok):
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, u, v = graph_case(11, 6, 35, False)
        rowptr, col, _ = csr(n, u, v)
        part = pt.ebv_partition(n, u, v, world, keep_self_loops=False)
        comm = gs.Comm(rank, world)
        ones = np.ones(n, np.int32)
        g = gs.DeviceGraph(part.local_graph(rank), ones, ones, dev, max_features=1)
        for kind, want, source in ((mp.CC, oracle.cc_fixed_point(rowptr, col), -1),
                                   (mp.SSSP, oracle.sssp_f32(rowptr, col, int(u[5])), int(u[5]))):
            job = mp.MinProp(g, kind, comm=comm)
            history = mp.run_job(job, source)
            _, ref_steps, ref_sizes = oracle.mp_drone_cuda(kind, n, part.part_u, part.part_v, part.owner, source=source)
            assert len(history) == ref_steps
            mine = np.array([[r.Mirror2MasterSendSize, r.Mirror2MasterRecvSize, r.Master2MirrorSendSize,
                              r.Master2MirrorRecvSize, r.VisitedSize] for r in history])
            assert np.array_equal(mine, ref_sizes[:, rank, :])
            assert np.array_equal(job.values().astype(want.dtype), want[g.host.l2g])
            job.close()
        dist.barrier()
        ok[rank] = 1
        comm.close()
    finally:
        dist.destroy_process_group()


def test_jobs_over_nccl_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_ranks(_rank, 2, (29300 + os.getpid() % 2000,))

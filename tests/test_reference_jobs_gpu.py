"""The reference's own GPU jobs (pr_cuda, sssp_cuda, cc_cuda), compiled from its sources into oracle/_ref by
`make -C oracle ref`, run on the same inputs as this library's drop-in (libdrone_pr_compat.so) and as the CPU
restatement.  Skipped when the reference library was not built.  Every run happens in a child process: the reference
ends the process on any CUDA or NCCL error."""
import ctypes as C
import os
import time

import numpy as np
import pytest
import torch

from drone_b200 import partition as pt
from test_compat_gpu import CCValues, Comm, PRValues, Response, SSSPValues, bind_jobs, device_floats, device_ints, ints, LIBDIR
from test_pagerank_oracle import pr_case

pytestmark = pytest.mark.gpu


def first_seen_order(n, u, v):
    """Relabel the graph so that ids follow the order of first appearance in u0, v0, u1, v1, ... (and unused ids come
    last): the local numbering of a single worker then equals the global one."""
    seq = np.stack([u, v], 1).reshape(-1)
    _, first = np.unique(seq, return_index=True)
    order = seq[np.sort(first)]
    rest = np.setdiff1d(np.arange(n, dtype=np.int64), order)
    new_id = np.empty(n, np.int64)
    new_id[np.concatenate([order, rest])] = np.arange(n)
    return new_id[u].astype(np.int32), new_id[v].astype(np.int32)


def wait_for_id_file(rank):
    """The reference's worker 0 writes ./nccl.id and the others open it without waiting (graph.cu:31-37,122-128)."""
    if rank == 0:
        return
    t0 = time.time()
    while not (os.path.exists("nccl.id") and os.path.getsize("nccl.id") >= 128):
        if time.time() - t0 > 60:
            raise RuntimeError("nccl.id did not appear")
        time.sleep(0.01)
    time.sleep(0.05)


def run_jobs(lib, part, rank, world, n, out_deg, source, total, pr_steps, with_cc):
    """build_graph + routes, then pr / sssp / (cc) to their stop rule.  Returns values by local id and responses."""
    comm, values = Comm(), PRValues()
    ku, pu = ints(part.part_u[rank])
    kv, pv = ints(part.part_v[rank])
    wait_for_id_file(rank)
    g = lib.build_graph(n, len(part.part_u[rank]), pu, pv, rank, world, C.byref(comm))
    mv, num, wk = part.master_rows(rank)
    (k1, p1), (k2, p2), (k3, p3) = ints(mv), ints(num), ints(wk)
    lib.addMasterRoute(g, p1, p2, p3, len(mv), len(wk))
    mr, ow = part.mirror_rows(rank)
    (k4, p4), (k5, p5) = ints(mr), ints(ow)
    lib.addMirrorRoute(g, p4, p5, len(mr))
    kd, pd = ints(out_deg)
    lib.loadOutDegree(g, C.byref(values), pd)
    nloc = lib.getLocalVertexSize(g)
    dev = torch.device("cuda", rank)
    out = {"n_local": nloc}

    def sizes(r):
        return [r.Mirror2MasterSendSize, r.Mirror2MasterRecvSize, r.Master2MirrorSendSize, r.Master2MirrorRecvSize]

    res = lib.PR_PEVal(g, C.byref(values), rank, world, C.byref(comm))
    steps = 1
    while steps < 300:
        if pr_steps is not None:
            if steps >= pr_steps:
                break
        elif total(sum(sizes(res))) == 0:
            break
        res = lib.PR_IncEVal(g, C.byref(values), rank, world, C.byref(comm))
        steps += 1
    out["pr"], out["pr_steps"] = device_floats(values.prValue, nloc, dev), steps

    sp = SSSPValues()
    hist = [lib.SSSP_PEVal(g, C.byref(sp), source, rank, world, C.byref(comm))]
    while total(sum(sizes(hist[-1]))) != 0 and len(hist) < 300:
        hist.append(lib.SSSP_IncEVal(g, C.byref(sp), rank, world, C.byref(comm)))
    out["sssp"] = device_floats(sp.distance, nloc, dev)
    out["sssp_sizes"] = np.array([sizes(r) + [r.VisitedSize] for r in hist])
    if with_cc:
        cc = CCValues()
        hist = [lib.CC_PEVal(g, C.byref(cc), rank, world, C.byref(comm))]
        while total(sum(sizes(hist[-1]))) != 0 and len(hist) < 300:
            hist.append(lib.CC_IncEVal(g, C.byref(cc), rank, world, C.byref(comm)))
        out["cc"] = device_ints(cc.ccValue, nloc, dev)
        out["cc_sizes"] = np.array([sizes(r) + [r.VisitedSize] for r in hist])
    return out


def _worker(rank, world, workdir, ok):
    import torch.distributed as dist
    from oracle import oracle
    from test_minprop_oracle import csr
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(29100 + os.getppid() % 2000)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    import drone_b200 as db
    db.lib()

    def total(x):
        t = torch.tensor([x], dtype=torch.int64)
        dist.all_reduce(t)
        return int(t)

    n, u, v, out_deg, part = pr_case(scale=10, seed=47, parts=world)
    if world == 1:                      # ids in first-seen order: the reference's local-index labels become comparable
        u, v = first_seen_order(n, part.part_u[0], part.part_v[0])
        out_deg = np.bincount(u, minlength=n).astype(np.int32)
        part = pt.Partition(n, 1, [u], [v], np.zeros(n, np.int32), np.ones(n, np.int32))
    source = int(u[3])
    results = {}
    for name, path in (("reference", oracle.reference_jobs_library()),
                       ("library", os.path.join(LIBDIR, "libdrone_pr_compat.so"))):
        d = os.path.join(workdir, name)
        if rank == 0:
            os.makedirs(d, exist_ok=True)
        dist.barrier()
        os.chdir(d)
        lib = bind_jobs(C.CDLL(path))
        results[name] = run_jobs(lib, part, rank, world, n, out_deg, source, total,
                                 pr_steps=12 if world == 1 else None, with_cc=world == 1)
        dist.barrier()
    ref, ours = results["reference"], results["library"]
    lg = part.local_graph(rank)
    assert ref["n_local"] == ours["n_local"] == lg.n_local
    # PageRank: float atomics in a different order and pushes near the threshold; same supersteps within a few
    assert abs(ref["pr_steps"] - ours["pr_steps"]) <= 3
    rel = np.abs(ref["pr"] - ours["pr"]) / np.maximum(np.abs(ref["pr"]), 1e-3)
    assert rel.max() < 5e-4, rel.max()
    # distances with unit lengths: exact, and the same Response sizes superstep by superstep
    assert np.array_equal(ref["sssp"], ours["sssp"])
    assert np.array_equal(ref["sssp_sizes"], ours["sssp_sizes"])
    rowptr, col, _ = csr(n, u, v)
    assert np.array_equal(ours["sssp"], oracle.sssp_f32(rowptr, col, source)[lg.l2g])
    _, steps, want_sizes = oracle.mp_drone_cuda(oracle.MP_SSSP, n, part.part_u, part.part_v, part.owner, source=source)
    assert np.array_equal(ref["sssp_sizes"], want_sizes[:, rank, :])
    if world == 1:
        assert np.array_equal(lg.l2g, np.arange(lg.n_local))          # the relabelling did its job
        assert np.array_equal(ref["cc"], ours["cc"])
        assert np.array_equal(ref["cc_sizes"], ours["cc_sizes"])
        assert np.array_equal(ours["cc"], oracle.cc_fixed_point(rowptr, col)[lg.l2g])
    dist.barrier()
    ok[rank] = 1
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_reference_jobs_against_the_drop_in(tmp_path, oracle, world):
    if oracle.reference_jobs_library() is None:
        pytest.skip("oracle/_ref/libref_drone_jobs.so was not built (needs the reference tree at build time)")
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ok = ctx.Array("i", [0] * world)
    procs = [ctx.Process(target=_worker, args=(r, world, str(tmp_path), ok)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs)
    assert list(ok) == [1] * world

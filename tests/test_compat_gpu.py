"""The reference-shaped shims: the C++ CUDAGraphSum class (driven through its C harness entry points) and the
cgo-facing C interface of the pr_cuda job (build_graph, addMasterRoute, addMirrorRoute, loadOutDegree, PR_PEVal,
PR_IncEVal with the reference's struct layouts)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import drone_b200 as db
from drone_b200 import graphgen as gg
from drone_b200 import partition as pt
from helpers import run_ranks, ROOT, assert_close_to_oracle, graph_case
from test_pagerank_oracle import pr_case

pytestmark = pytest.mark.gpu
LIBDIR = os.path.join(ROOT, "drone_b200", "lib")


class Graph(C.Structure):      # DRONE/src/cuda/graph.h:16-38
    _fields_ = [("Global2Local", C.c_void_p), ("Local2Global", C.c_void_p), ("MasterWorkerIndex", C.c_void_p),
                ("Master2Workers", C.c_void_p), ("MasterSize", C.c_int), ("MirrorWorkerSize", C.c_int),
                ("Mirror2Worker", C.c_void_p), ("MirrorSize", C.c_int), ("index", C.c_void_p), ("dst", C.c_void_p),
                ("edgeLen", C.c_void_p), ("localVertexSize", C.POINTER(C.c_int)),
                ("globalVertexSize", C.POINTER(C.c_int)), ("edgeSize", C.POINTER(C.c_int)), ("gridSize", C.c_int),
                ("blockSize", C.c_int), ("active", C.c_void_p), ("updateByMessage", C.c_void_p), ("GID", C.c_int)]


class Comm(C.Structure):
    _fields_ = [("comm", C.c_void_p), ("s", C.c_void_p)]


class PRValues(C.Structure):   # DRONE/src/cuda/algorithm/pr.h:7-16
    _fields_ = [("sendID", C.c_void_p), ("recvID", C.c_void_p), ("sendDiff", C.c_void_p), ("recvDiff", C.c_void_p),
                ("prValue", C.c_void_p), ("accValue", C.c_void_p), ("diffValue", C.c_void_p),
                ("globalAcc", C.c_void_p), ("globalDiff", C.c_void_p), ("outDegree", C.c_void_p)]


class CCValues(C.Structure):   # DRONE/src/cuda/algorithm/cc.h:18-22
    _fields_ = [("sendID", C.c_void_p), ("recvID", C.c_void_p), ("sendCCValue", C.c_void_p),
                ("recvCCValue", C.c_void_p), ("ccValue", C.c_void_p)]


class SSSPValues(C.Structure):  # DRONE/src/cuda/algorithm/sssp.h:8-12
    _fields_ = [("sendID", C.c_void_p), ("recvID", C.c_void_p), ("sendDis", C.c_void_p), ("recvDis", C.c_void_p),
                ("distance", C.c_void_p)]


class Response(C.Structure):   # DRONE/src/cuda/algorithm/common.h:23-27
    _fields_ = [("Mirror2MasterSendSize", C.c_int), ("Mirror2MasterRecvSize", C.c_int),
                ("Master2MirrorSendSize", C.c_int), ("Master2MirrorRecvSize", C.c_int), ("VisitedSize", C.c_int),
                ("LocalVertexSize", C.c_int), ("CalTime", C.c_float), ("SendTime", C.c_float)]

    def empty(self):
        return (self.Mirror2MasterSendSize == 0 and self.Mirror2MasterRecvSize == 0 and
                self.Master2MirrorSendSize == 0 and self.Master2MirrorRecvSize == 0)


def pr_lib():
    db.lib()
    return bind_jobs(C.CDLL(os.path.join(LIBDIR, "libdrone_pr_compat.so")))


def bind_jobs(lib):
    """Prototypes of the cgo-facing interface (DRONE/src/cuda/graph.h:45-52, algorithm/pr.h, cc.h, sssp.h)."""
    ip = C.POINTER(C.c_int)
    lib.build_graph.restype = C.POINTER(Graph)
    lib.build_graph.argtypes = [C.c_int, C.c_int, ip, ip, C.c_int, C.c_int, C.POINTER(Comm)]
    lib.addMasterRoute.argtypes = [C.POINTER(Graph), ip, ip, ip, C.c_int, C.c_int]
    lib.addMirrorRoute.argtypes = [C.POINTER(Graph), ip, ip, C.c_int]
    lib.loadOutDegree.argtypes = [C.POINTER(Graph), C.POINTER(PRValues), ip]
    lib.getLocalVertexSize.argtypes = [C.POINTER(Graph)]
    lib.getGlobalVertexSize.argtypes = [C.POINTER(Graph)]
    for fn in (lib.PR_PEVal, lib.PR_IncEVal):
        fn.restype = Response
        fn.argtypes = [C.POINTER(Graph), C.POINTER(PRValues), C.c_int, C.c_int, C.POINTER(Comm)]
    for fn in (lib.CC_PEVal, lib.CC_IncEVal):
        fn.restype = Response
        fn.argtypes = [C.POINTER(Graph), C.POINTER(CCValues), C.c_int, C.c_int, C.POINTER(Comm)]
    lib.SSSP_PEVal.restype = lib.SSSP_IncEVal.restype = Response
    lib.SSSP_PEVal.argtypes = [C.POINTER(Graph), C.POINTER(SSSPValues), C.c_int, C.c_int, C.c_int, C.POINTER(Comm)]
    lib.SSSP_IncEVal.argtypes = [C.POINTER(Graph), C.POINTER(SSSPValues), C.c_int, C.c_int, C.POINTER(Comm)]
    return lib


def run_cc_and_sssp(lib, g, comm, rank, world, source, all_reduce=None):
    """The superstep loops of CCworkerCUDA / SSSPworkerCUDA with the master's stop rule; returns labels, distances
    (device pointers inside the value structs) and the number of supersteps of each job."""
    out = []
    for job in ("cc", "sssp"):
        vals = CCValues() if job == "cc" else SSSPValues()
        if job == "cc":
            res = lib.CC_PEVal(g, C.byref(vals), rank, world, C.byref(comm))
        else:
            res = lib.SSSP_PEVal(g, C.byref(vals), source, rank, world, C.byref(comm))
        steps = 1
        while True:
            busy = (res.Mirror2MasterSendSize + res.Mirror2MasterRecvSize + res.Master2MirrorSendSize +
                    res.Master2MirrorRecvSize)
            if all_reduce is not None:
                busy = all_reduce(busy)
            if busy == 0 or steps > 200:
                break
            res = (lib.CC_IncEVal if job == "cc" else lib.SSSP_IncEVal)(g, C.byref(vals), rank, world, C.byref(comm))
            steps += 1
        out.append((vals, steps))
    return out


def ints(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    if a.size == 0:
        a = np.zeros(1, np.int32)
    return a, a.ctypes.data_as(C.POINTER(C.c_int))


def run_pr_worker(lib, part, rank, world, n, out_deg):
    """What newPRWorkerCUDA + the superstep RPCs do (DRONE/src/worker/PRWorkerCUDA.go:52-93,141-175)."""
    comm, values = Comm(), PRValues()
    ku, pu = ints(part.part_u[rank])
    kv, pv = ints(part.part_v[rank])
    g = lib.build_graph(n, len(part.part_u[rank]), pu, pv, rank, world, C.byref(comm))
    mv, num, wk = part.master_rows(rank)
    (k1, p1), (k2, p2), (k3, p3) = ints(mv), ints(num), ints(wk)
    lib.addMasterRoute(g, p1, p2, p3, len(mv), len(wk))
    mr, ow = part.mirror_rows(rank)
    (k4, p4), (k5, p5) = ints(mr), ints(ow)
    lib.addMirrorRoute(g, p4, p5, len(mr))
    kd, pd = ints(out_deg)
    lib.loadOutDegree(g, C.byref(values), pd)
    return g, comm, values


def device_floats(ptr, n, dev):
    from drone_b200.plan import _view_device_memory
    return _view_device_memory(ptr, n, torch.float32, dev).clone().cpu().numpy()


def test_pr_c_interface_single_worker(cuda_device, oracle, tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)                       # build_graph writes ./nccl.id like the reference
    lib = pr_lib()
    n, u, v, out_deg, part = pr_case(scale=9, seed=41, parts=1)
    g, comm, values = run_pr_worker(lib, part, 0, 1, n, out_deg)
    nloc, g2l, l2g, index, dst = oracle.build_graph(n, part.part_u[0], part.part_v[0])
    assert lib.getLocalVertexSize(g) == nloc and lib.getGlobalVertexSize(g) == n
    assert g.contents.localVertexSize[0] == nloc and g.contents.edgeSize[0] == len(u)
    assert os.path.exists("nccl.id")
    res = lib.PR_PEVal(g, C.byref(values), 0, 1, C.byref(comm))
    assert res.LocalVertexSize == nloc and res.empty() and res.VisitedSize > 0
    pr0 = device_floats(values.prValue, nloc, cuda_device)
    assert (pr0 == 1.0).all()
    # the master would stop here (nothing exchanged); further supersteps are still well defined
    for _ in range(30):
        res = lib.PR_IncEVal(g, C.byref(values), 0, 1, C.byref(comm))
    got = np.zeros(n, np.float32)
    got[l2g] = device_floats(values.prValue, nloc, cuda_device)
    want, _, _ = oracle.pr_drone_cuda(n, part.part_u, part.part_v, out_deg, part.owner, eps=1e-6, dtype=np.float32)
    # the oracle follows the stop rule (one part: stops after PEval, all ones); compare with a forced run instead
    from test_pagerank_oracle import dense_power
    assert np.isfinite(got).all() and got[l2g].min() > 0.1
    ref = n * dense_power(n, u, v, 400, float(np.float32(0.85)))
    assert np.max(np.abs(got[l2g] - ref[l2g]) / ref[l2g]) < 2e-3     # float, eps = 1e-6, 30 supersteps


def device_ints(ptr, n, dev):
    from drone_b200.plan import _view_device_memory
    return _view_device_memory(ptr, n, torch.int32, dev).clone().cpu().numpy()


def test_cc_and_sssp_c_interface_single_worker(cuda_device, oracle, tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    from test_minprop_oracle import csr
    lib = pr_lib()
    n, u, v, out_deg, part = pr_case(scale=9, seed=45, parts=1)
    g, comm, _ = run_pr_worker(lib, part, 0, 1, n, out_deg)
    nloc = lib.getLocalVertexSize(g)
    l2g = part.local_graph(0).l2g
    source = int(u[3])
    (cc, cc_steps), (sp, sp_steps) = run_cc_and_sssp(lib, g, comm, 0, 1, source)
    assert cc_steps == 1 and sp_steps == 1
    rowptr, col, _ = csr(n, u, v)
    assert np.array_equal(device_ints(cc.ccValue, nloc, cuda_device), oracle.cc_fixed_point(rowptr, col)[l2g])
    assert np.array_equal(device_floats(sp.distance, nloc, cuda_device), oracle.sssp_f32(rowptr, col, source)[l2g])
    assert g.contents.active and g.contents.updateByMessage


def gcn_lib():
    db.lib()
    lib = C.CDLL(os.path.join(LIBDIR, "libdrone_gcn_compat.so"))
    vp = C.c_void_p
    lib.drone_compat_graphsum_create.restype = vp
    lib.drone_compat_graphsum_create.argtypes = [C.c_int, C.c_int, C.c_int] + [vp] * 8 + [C.c_int] + [vp] * 4 + \
        [C.c_int, C.c_int, C.c_int, vp, vp]
    for name in ("forward", "backward", "destroy"):
        getattr(lib, "drone_compat_graphsum_" + name).argtypes = [vp]
    return lib


@pytest.mark.parametrize("f", [64, 41])
def test_cpp_graphsum_module_single_worker(cuda_device, oracle, f):
    lib = gcn_lib()
    n, u, v = gg.rmat_graph(11, 16, seed=42, symmetrise=False, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    t = lambda a: torch.as_tensor(a, device=cuda_device)
    d_index, d_dst, d_in, d_out = t(index), t(dst), t(in_deg), t(out_deg)
    x = gg.seeded_normal(f, (n, f))
    gy = gg.seeded_normal(f + 1, (n, f))
    in_data, in_grad = t(x), torch.zeros((n, f), device=cuda_device)
    out_data, out_grad = torch.zeros((n, f), device=cuda_device), t(gy)
    stream = torch.cuda.current_stream().cuda_stream
    h = lib.drone_compat_graphsum_create(n, len(dst), n, d_index.data_ptr(), d_dst.data_ptr(), d_in.data_ptr(),
                                         d_out.data_ptr(), None, None, None, None, 0, in_data.data_ptr(),
                                         in_grad.data_ptr(), out_data.data_ptr(), out_grad.data_ptr(), f, 0, 1, None,
                                         stream)
    lib.drone_compat_graphsum_forward(h)
    lib.drone_compat_graphsum_backward(h)
    torch.cuda.synchronize()
    assert_close_to_oracle(out_data.cpu().numpy(), oracle.graphsum_forward_f64(x, index, dst, val))
    assert_close_to_oracle(in_grad.cpu().numpy(), oracle.graphsum_backward_f64(gy, index, dst, val))
    lib.drone_compat_graphsum_destroy(h)


def _two_workers(rank, world, workdir, ok):
    from oracle import oracle
    os.chdir(workdir)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    lib = pr_lib()
    n, u, v, out_deg, part = pr_case(scale=10, seed=43, parts=world)
    g, comm, values = run_pr_worker(lib, part, rank, world, n, out_deg)
    want, want_steps, want_sizes = oracle.pr_drone_cuda(n, part.part_u, part.part_v, out_deg, part.owner, eps=1e-6,
                                                        dtype=np.float32)
    res = lib.PR_PEVal(g, C.byref(values), rank, world, C.byref(comm))
    steps = 1
    while steps < want_steps:          # both workers run the oracle's superstep count (the master's decision)
        res = lib.PR_IncEVal(g, C.byref(values), rank, world, C.byref(comm))
        steps += 1
    nloc = lib.getLocalVertexSize(g)
    lg = part.local_graph(rank)
    vals = device_floats(values.prValue, nloc, dev)
    keep = lg.mirror2worker == -1
    gid = lg.l2g[keep]
    assert np.max(np.abs(vals[keep] - want[gid]) / want[gid]) < 2e-4

    # the cc_cuda and sssp_cuda jobs through the same Graph and communicator
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(29700 + os.getppid() % 2000)
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def total(x):
        t = torch.tensor([x], dtype=torch.int64)
        dist.all_reduce(t)
        return int(t)

    from test_minprop_oracle import csr
    source = int(u[3])
    (cc, cc_steps), (sp, sp_steps) = run_cc_and_sssp(lib, g, comm, rank, world, source, all_reduce=total)
    rowptr, col, _ = csr(n, u, v)
    assert np.array_equal(device_ints(cc.ccValue, nloc, dev), oracle.cc_fixed_point(rowptr, col)[lg.l2g])
    assert np.array_equal(device_floats(sp.distance, nloc, dev), oracle.sssp_f32(rowptr, col, source)[lg.l2g])
    assert cc_steps == oracle.mp_drone_cuda(oracle.MP_CC, n, part.part_u, part.part_v, part.owner)[1]
    assert sp_steps == oracle.mp_drone_cuda(oracle.MP_SSSP, n, part.part_u, part.part_v, part.owner, source=source)[1]
    dist.barrier()
    dist.destroy_process_group()

    # the C++ GraphSum module over the communicator that build_graph created
    glib = gcn_lib()
    f = 32
    in_deg = np.bincount(v, minlength=n).astype(np.int32)
    ind, outd = lg.local_degrees(in_deg, np.maximum(out_deg, 1))
    t = lambda a: torch.as_tensor(np.ascontiguousarray(a), device=dev)
    d = dict(index=t(lg.index), dst=t(lg.dst), ind=t(ind), outd=t(outd), l2g=t(lg.l2g), mir=t(lg.mirror2worker),
             mwi=t(lg.master_worker_index), m2w=t(lg.master2workers if len(lg.master2workers) else np.zeros(1, np.int32)))
    x = gg.seeded_normal(7, (n, f))
    in_data, in_grad = t(x[lg.l2g]), torch.zeros((nloc, f), device=dev)
    out_data, out_grad = torch.zeros((nloc, f), device=dev), t(x[lg.l2g])
    h = glib.drone_compat_graphsum_create(nloc, len(lg.dst), n, d["index"].data_ptr(), d["dst"].data_ptr(),
                                          d["ind"].data_ptr(), d["outd"].data_ptr(), d["l2g"].data_ptr(),
                                          d["mir"].data_ptr(), d["mwi"].data_ptr(), d["m2w"].data_ptr(),
                                          len(lg.master2workers), in_data.data_ptr(), in_grad.data_ptr(),
                                          out_data.data_ptr(), out_grad.data_ptr(), f, rank, world, comm.comm, comm.s)
    glib.drone_compat_graphsum_forward(h)
    glib.drone_compat_graphsum_backward(h)
    torch.cuda.synchronize()
    index, dst = gg.csr_by_source(torch.as_tensor(u), torch.as_tensor(v), n)
    val = oracle.csr_values_f32(index.numpy(), dst.numpy(), in_deg, np.maximum(out_deg, 1))
    from helpers import assert_close_to_oracle as close
    close(out_data.cpu().numpy(), oracle.graphsum_forward_f64(x, index.numpy(), dst.numpy(), val)[lg.l2g])
    close(in_grad.cpu().numpy(), oracle.graphsum_backward_f64(x, index.numpy(), dst.numpy(), val)[lg.l2g])
    glib.drone_compat_graphsum_destroy(h)
    ok[rank] = 1


def test_c_interfaces_two_workers(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_ranks(_two_workers, 2, (str(tmp_path),))

"""Host-side mirror of the reference's GraphSum layer over the C ABI.

GraphSum keeps the constructor arguments, the forward(training)/backward() interface and the
side effects of CUDAGraphSum (cuda_gcn/src/cuda/cuda_module.cuh:83-84, cuda_module.cu:149-389):
forward overwrites out.data with A^T · in.data and then makes every replica row hold the global
sum; backward overwrites in.grad with A · out.grad and syncs it the same way.
"""
import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import OP_A, OP_AT, check
from .plan import AggregationPlan, _stream_ptr
from .partition import ExchangePlan


class Variable:
    """data/grad pair of a layer boundary (CUDAVariable, cuda_gcn/src/cuda/cuda_variable.cuh:17-30)."""

    def __init__(self, n_rows, dim, device, requires_grad=True):
        self.data = torch.zeros((n_rows, dim), dtype=torch.float32, device=device)
        self.grad = torch.zeros((n_rows, dim), dtype=torch.float32, device=device) if requires_grad else None
        self.size = n_rows * dim


class Comm:
    """One NCCL communicator owned by the library (Comm{ncclComm_t, stream}, cuda_gcn/src/cuda/graph.h:43-46).
    The unique id travels through torch.distributed when it is initialised, otherwise through `id_bytes`."""

    def __init__(self, rank, nranks, id_bytes=None):
        lib = _lib.lib()
        self.rank, self.nranks = rank, nranks
        if id_bytes is None:
            import torch.distributed as dist
            box = [None]
            if rank == 0:
                buf = C.create_string_buffer(128)
                check(lib.drone_comm_unique_id(buf, 128))
                box[0] = buf.raw
            dist.broadcast_object_list(box, src=0)
            id_bytes = box[0]
        self._h = C.c_void_p(0)
        check(lib.drone_comm_create(C.byref(self._h), rank, nranks, id_bytes, len(id_bytes)))

    @staticmethod
    def unique_id():
        buf = C.create_string_buffer(128)
        check(_lib.lib().drone_comm_unique_id(buf, 128))
        return buf.raw

    @property
    def handle(self):
        return self._h

    def allreduce_sum(self, t, stream=None):
        check(_lib.lib().drone_comm_allreduce_sum(self._h, C.c_void_p(t.data_ptr()), t.numel(),
                                                  int(t.dtype == torch.float64), _stream_ptr(stream)))

    def bcast(self, t, root=0, stream=None):
        """weight_broadcast_value_nccl (cuda_gcn/src/cuda/cuda_communicate.cu:99-105): rank `root`'s floats to all."""
        check(_lib.lib().drone_comm_bcast(self._h, C.c_void_p(t.data_ptr()), t.numel(), int(root), _stream_ptr(stream)))

    def reduce_sum(self, t, root=0, stream=None):
        """weight_reduce_grad_nccl (cuda_communicate.cu:107-115): the sum over ranks lands on `root`."""
        check(_lib.lib().drone_comm_reduce_sum(self._h, C.c_void_p(t.data_ptr()), t.numel(), int(root),
                                               _stream_ptr(stream)))

    def close(self):
        if self._h.value:
            _lib.lib().drone_comm_destroy(self._h)
            self._h = C.c_void_p(0)


class DeviceGraph:
    """A rank's local graph on its GPU: CSR by source, global degrees by local id, routing plan."""

    def __init__(self, local_graph, global_in_degree, global_out_degree, device, max_features):
        g = local_graph
        self.host = g
        self.n_local = g.n_local
        self.device = device
        self.index = torch.as_tensor(g.index, device=device)
        self.dst = torch.as_tensor(g.dst, device=device)
        ind, outd = g.local_degrees(np.asarray(global_in_degree), np.asarray(global_out_degree))
        self.in_degree = torch.as_tensor(ind, device=device)
        self.out_degree = torch.as_tensor(outd, device=device)
        self.mirror2worker = torch.as_tensor(g.mirror2worker, device=device)
        self.xplan = ExchangePlan(g, max_features)
        self.plan = AggregationPlan(self.index, self.dst, in_degree=self.in_degree, out_degree=self.out_degree)


def clear_mirror_rows(rows, mirror2worker, stream=None):
    """clear_mirror_grad (cuda_gcn/src/cuda/cuda_module.cu:50-61): zero the rows of mirror vertices, in place."""
    f = rows.shape[1]
    ld = rows.stride(0) if rows.shape[0] > 1 else max(f, rows.stride(0))
    with torch.cuda.device(rows.device):
        check(_lib.lib().drone_clear_mirror_rows(C.c_void_p(rows.data_ptr()), rows.shape[0], f, int(ld),
                                                 C.c_void_p(mirror2worker.data_ptr()), _stream_ptr(stream)))
    return rows


def exchange_sum(xplan, comm, rows, stream=None):
    """Mirror -> master sum, master -> mirror assign on a [n_local, F] tensor (in place)."""
    f = rows.shape[1]
    ld = rows.stride(0) if rows.shape[0] > 1 else max(f, rows.stride(0))
    check(_lib.lib().drone_exchange_sum(xplan.handle, comm.handle, C.c_void_p(rows.data_ptr()), f, int(ld),
                                        _stream_ptr(stream)))


def exchange_finish(xplan, rows, stream=None):
    """The rest of the exchange after an aggregation that sent the mirror rows up itself (plan.spmm(...,
    push_up_to=xplan.handle)): masters add and send the totals down, mirror rows take them (in place)."""
    f = rows.shape[1]
    ld = rows.stride(0) if rows.shape[0] > 1 else max(f, rows.stride(0))
    check(_lib.lib().drone_exchange_finish(xplan.handle, C.c_void_p(rows.data_ptr()), f, int(ld), _stream_ptr(stream)))


def aggregate_and_exchange(plan, xplan, comm, orientation, x, out, stream=None):
    """out = aggregation of x summed over the replicas of every vertex.  With the peer-memory transport the
    aggregation kernels store mirror rows straight into their owners' memory (one pass less over those rows, and the
    transfer runs beside the arithmetic); otherwise aggregation, then the exchange.  Same bits either way."""
    if comm is None or comm.nranks == 1:
        return plan.spmm(orientation, x, out=out, stream=stream)
    if getattr(xplan, "p2p_enabled", False):
        plan.spmm(orientation, x, out=out, stream=stream, push_up_to=xplan.handle)
        exchange_finish(xplan, out, stream=stream)
    else:
        plan.spmm(orientation, x, out=out, stream=stream)
        exchange_sum(xplan, comm, out, stream=stream)
    return out


def exchange_sum_dense(dense_plan, comm, rows, stream=None):
    """The exchange as ncclReduceScatter + ncclAllGather over the boundary buffer (in place)."""
    f = rows.shape[1]
    ld = rows.stride(0) if rows.shape[0] > 1 else max(f, rows.stride(0))
    check(_lib.lib().drone_exchange_sum_dense(dense_plan.handle, comm.handle, C.c_void_p(rows.data_ptr()), f, int(ld),
                                              _stream_ptr(stream)))


def exchange_sum_local(xplans, rows_list, stream=None):
    """The same exchange among all parts held on one device."""
    n = len(xplans)
    f = rows_list[0].shape[1]
    plans = (C.c_void_p * n)(*[x.handle for x in xplans])
    ptrs = (C.c_void_p * n)(*[C.c_void_p(r.data_ptr()) for r in rows_list])
    lds = (C.c_int * n)(*[int(r.stride(0)) if r.shape[0] > 1 else f for r in rows_list])
    check(_lib.lib().drone_exchange_sum_local(n, plans, ptrs, f, lds, _stream_ptr(stream)))


def row_groups(local2global, n_groups):
    """Group of every local row, the same on every rank that holds the vertex: a multiplicative hash of the global id."""
    h = (np.asarray(local2global).astype(np.uint64) * np.uint64(0x9E3779B97F4A7C15)) >> np.uint64(40)
    return (h % np.uint64(n_groups)).astype(np.int32)


class PipelinedAggregation:
    """Aggregation followed by the mirror/master exchange, in n_groups groups of rows: while group g+1 is aggregated
    on the caller's stream, the rows of group g are exchanged on a second stream.  Same result as
    plan.spmm(...) + exchange_sum(...) (bit for bit with the peer-memory and send/recv transports).  The data flow of
    CUDAGraphSum::forward / backward (cuda_gcn/src/cuda/cuda_module.cu:210-307, 310-389) with the two steps
    overlapped; the reference runs them one after the other."""

    def __init__(self, graph, comm, max_features, n_groups=4, p2p=True, fused_push=True):
        self.graph, self.comm, self.n_groups = graph, comm, int(n_groups)
        # with the peer-memory transport the aggregation of a group stores its mirror rows into their owners' memory
        # itself, and only the downward half of the group's exchange runs on the second stream
        self.fused_push = bool(fused_push) and p2p and comm is not None and comm.nranks > 1
        groups = row_groups(graph.host.l2g, self.n_groups)
        self.row_class = torch.as_tensor(groups, device=graph.device)
        graph.plan.set_row_classes(self.row_class, self.n_groups)
        self.xplans = [ExchangePlan(graph.host, max_features, row_mask=groups == g) for g in range(self.n_groups)]
        if p2p and comm is not None and comm.nranks > 1:
            for x in self.xplans:
                x.enable_p2p(comm)
        with torch.cuda.device(graph.device):
            # high priority: the exchange kernels are short links of a dependency chain across GPUs; at equal priority
            # each would queue behind the thousands of blocks of the aggregation running beside it
            self.side = torch.cuda.Stream(priority=-1)
            self.ready = [torch.cuda.Event() for _ in range(self.n_groups)]
            self.done = torch.cuda.Event()

    def __call__(self, orientation, x, out):
        main = torch.cuda.current_stream(self.graph.device)
        for g in range(self.n_groups):
            if self.fused_push:
                self.graph.plan.spmm(orientation, x, out=out, row_class=g, push_up_to=self.xplans[g].handle)
            else:
                self.graph.plan.spmm(orientation, x, out=out, row_class=g)
            self.ready[g].record(main)
            self.side.wait_event(self.ready[g])
            if self.fused_push:
                exchange_finish(self.xplans[g], out, stream=self.side)
            else:
                exchange_sum(self.xplans[g], self.comm, out, stream=self.side)
        self.done.record(self.side)
        main.wait_event(self.done)
        return out

    def close(self):
        for x in self.xplans:
            x.close()
        self.xplans = []


class GraphSum:
    """Drop-in shape of CUDAGraphSum: GraphSum(in, out, graph, comm, dim, worker_id, worker_num, name, layer)."""

    def __init__(self, in_var, out_var, graph, comm, dim, worker_id=0, worker_num=1, name="graphSum", layer=0):
        self.inp, self.out, self.graph, self.comm = in_var, out_var, graph, comm
        self.dim, self.worker_id, self.worker_num = dim, worker_id, worker_num
        self.ModuleName, self.layer = name, layer

    def forward(self, training=True):
        aggregate_and_exchange(self.graph.plan, self.graph.xplan, self.comm if self.worker_num > 1 else None, OP_AT,
                               self.inp.data, self.out.data)

    def backward(self):
        aggregate_and_exchange(self.graph.plan, self.graph.xplan, self.comm if self.worker_num > 1 else None, OP_A,
                               self.out.grad, self.inp.grad)

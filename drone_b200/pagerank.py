"""Host-side mirror of DRONE's GPU PageRank job over the C ABI: the calls the Go worker makes
through cgo (loadOutDegree, PR_PEVal, PR_IncEVal; DRONE/src/tools/cuda_convert.go:85-97) and
the master's superstep loop (DRONE/src/master.go:430-463)."""
import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import PRResponse, check
from .plan import _stream_ptr


class PageRank:
    """PageRank state of one rank (drone_pr).  `graph` is a graphsum.DeviceGraph."""

    def __init__(self, graph, global_v, comm=None, use_double=False, eps=1e-6, n_isolated=0):
        self.graph, self.comm = graph, comm
        self.use_double = bool(use_double)
        self.n_local = graph.n_local
        self._h = C.c_void_p(0)
        with torch.cuda.device(graph.device):
            check(_lib.lib().drone_pr_create(
                C.byref(self._h), graph.n_local, int(global_v), graph.dst.numel(), C.c_void_p(graph.index.data_ptr()),
                C.c_void_p(graph.dst.data_ptr()), C.c_void_p(graph.out_degree.data_ptr()),
                C.c_void_p(graph.mirror2worker.data_ptr()), graph.xplan.handle,
                comm.handle if comm is not None else C.c_void_p(0), int(self.use_double), float(eps)))
        if n_isolated:
            check(_lib.lib().drone_pr_set_isolated_count(self._h, int(n_isolated)))

    @property
    def handle(self):
        return self._h

    def transport_name(self):
        """How boundary entries travel between ranks: stored into the peer's memory when the graph's exchange plan has
        that transport enabled and holds at least a {value, flag} pair per vertex, grouped send/recv otherwise."""
        need = 4 if self.use_double else 2
        if getattr(self.graph.xplan, "p2p_enabled", False) and self.graph.xplan.max_features >= need:
            return "peer memory (stores into the receiver's buffer + epoch flags) + scalar all-reduce"
        return "grouped ncclSend/ncclRecv of all boundary vertices + scalar all-reduce"

    def peval(self, stream=None):
        res = PRResponse()
        check(_lib.lib().drone_pr_peval(self._h, C.byref(res), _stream_ptr(stream)))
        return res

    def inceval(self, stream=None):
        res = PRResponse()
        check(_lib.lib().drone_pr_inceval(self._h, C.byref(res), _stream_ptr(stream)))
        return res

    def power_iterate(self, iterations=20, damping=0.85, stream=None):
        check(_lib.lib().drone_pr_power_iterate(self._h, int(iterations), float(damping), _stream_ptr(stream)))

    def values(self, stream=None):
        out = np.empty(self.n_local, np.float64 if self.use_double else np.float32)
        check(_lib.lib().drone_pr_values(self._h, C.c_void_p(out.ctypes.data), _stream_ptr(stream)))
        return out

    def close(self):
        if self._h.value:
            _lib.lib().drone_pr_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def step_local(prs, is_peval, stream=None):
    """One superstep of all parts held on one device.  Returns one PRResponse per part."""
    n = len(prs)
    handles = (C.c_void_p * n)(*[p.handle for p in prs])
    res = (PRResponse * n)()
    check(_lib.lib().drone_pr_step_local(n, handles, int(bool(is_peval)), res, _stream_ptr(stream)))
    return list(res)


def power_iterate_local(prs, iterations=20, damping=0.85, stream=None):
    n = len(prs)
    handles = (C.c_void_p * n)(*[p.handle for p in prs])
    check(_lib.lib().drone_pr_power_iterate_local(n, handles, int(iterations), float(damping), _stream_ptr(stream)))


def run_job_local(prs, max_steps=10000):
    """The master's loop for the job "pr_cuda" (no step cap; stops when no part exchanged anything)."""
    res = step_local(prs, True)
    steps = 1
    sizes = [[(r.Mirror2MasterSendSize, r.Mirror2MasterRecvSize, r.Master2MirrorSendSize, r.Master2MirrorRecvSize)
              for r in res]]
    while not all(r.is_empty() for r in res) and steps < max_steps:
        res = step_local(prs, False)
        sizes.append([(r.Mirror2MasterSendSize, r.Mirror2MasterRecvSize, r.Master2MirrorSendSize,
                       r.Master2MirrorRecvSize) for r in res])
        steps += 1
    return steps, sizes


def gather_global(prs, graphs, global_v, replicas_owner=None):
    """Assemble values by global id from the master / only copy of every vertex
    (what PRWorker.Assemble writes, DRONE/src/worker/PRWorker.go:326-346)."""
    out = np.zeros(global_v, prs[0].values().dtype)
    for pr, g in zip(prs, graphs):
        vals = pr.values()
        keep = g.host.mirror2worker == -1
        out[g.host.l2g[keep]] = vals[keep]
    return out

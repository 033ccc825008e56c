"""Host-side mirror of DRONE's GPU jobs "cc_cuda" and "sssp_cuda" over the C ABI: the calls the Go workers make
through cgo (CC_PEVal / CC_IncEVal, SSSP_PEVal / SSSP_IncEVal; DRONE/src/tools/cuda_convert.go:99-125) and the
master's superstep loop (DRONE/src/master.go:430-463)."""
import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import PRResponse, check
from .plan import _stream_ptr

CC, SSSP = 0, 1


class MinProp:
    """State of one worker (drone_mp).  `graph` is a graphsum.DeviceGraph; edge_len an optional float32 CUDA tensor
    in the order of graph.dst (None: unit lengths)."""

    def __init__(self, graph, kind, comm=None, edge_len=None):
        self.graph, self.kind, self.comm = graph, int(kind), comm
        self.n_local = graph.n_local
        self._l2g = torch.as_tensor(np.ascontiguousarray(graph.host.l2g, dtype=np.int32), device=graph.device)
        self._len = edge_len
        if edge_len is not None and not (edge_len.is_cuda and edge_len.dtype == torch.float32 and
                                         edge_len.numel() == graph.dst.numel() and edge_len.is_contiguous()):
            raise ValueError("edge_len must be a contiguous float32 CUDA tensor with one entry per edge")
        self._h = C.c_void_p(0)
        with torch.cuda.device(graph.device):
            check(_lib.lib().drone_mp_create(
                C.byref(self._h), self.kind, graph.n_local, graph.dst.numel(), C.c_void_p(graph.index.data_ptr()),
                C.c_void_p(graph.dst.data_ptr()), C.c_void_p(edge_len.data_ptr() if edge_len is not None else 0),
                C.c_void_p(self._l2g.data_ptr()), graph.xplan.handle, comm.handle if comm is not None else C.c_void_p(0)))

    @property
    def handle(self):
        return self._h

    def peval(self, source=-1, stream=None):
        res = PRResponse()
        check(_lib.lib().drone_mp_peval(self._h, int(source), C.byref(res), _stream_ptr(stream)))
        return res

    def inceval(self, stream=None):
        res = PRResponse()
        check(_lib.lib().drone_mp_inceval(self._h, C.byref(res), _stream_ptr(stream)))
        return res

    def values(self, stream=None):
        """int32 labels or float32 distances by local id."""
        out = np.empty(self.n_local, np.int32 if self.kind == CC else np.float32)
        check(_lib.lib().drone_mp_values(self._h, C.c_void_p(out.ctypes.data), _stream_ptr(stream)))
        return out

    def close(self):
        if self._h.value:
            _lib.lib().drone_mp_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def step_local(jobs, is_peval, source=-1, stream=None):
    """One superstep of all parts held on one device.  Returns one PRResponse per part."""
    n = len(jobs)
    handles = (C.c_void_p * n)(*[j.handle for j in jobs])
    res = (PRResponse * n)()
    check(_lib.lib().drone_mp_step_local(n, handles, int(bool(is_peval)), int(source), res, _stream_ptr(stream)))
    return list(res)


def run_job_local(jobs, source=-1, max_steps=1000):
    """PEval, then IncEval until every part reports four empty sizes (the master's rule).  Returns the list of
    per-superstep responses."""
    history = [step_local(jobs, True, source)]
    while not all(r.is_empty() for r in history[-1]) and len(history) <= max_steps:
        history.append(step_local(jobs, False))
    return history


def run_job(job, source=-1, max_steps=1000):
    """The same loop for one worker per process: the stop rule needs everybody's sizes, summed over the job's ranks."""
    import torch.distributed as dist
    history = [job.peval(source)]
    while len(history) <= max_steps:
        r = history[-1]
        busy = torch.tensor([r.Mirror2MasterSendSize + r.Mirror2MasterRecvSize + r.Master2MirrorSendSize +
                             r.Master2MirrorRecvSize], dtype=torch.int64)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(busy)
        if int(busy) == 0:
            break
        history.append(job.inceval())
    return history


def gather_global(jobs, graphs, global_v, fill):
    """Values by global id from the master (or only) copy of every vertex."""
    out = np.full(global_v, fill, np.int32 if jobs[0].kind == CC else np.float32)
    for job, g in zip(jobs, graphs):
        vals = job.values()
        own = g.host.mirror2worker[:g.n_local] < 0
        out[g.host.l2g[own]] = vals[own]
    return out

"""Host-side handle of an aggregation plan over torch device tensors.

torch is used for device memory and streams only; every computation is a call
through the C ABI (include/drone_b200.h).
"""
import ctypes as C

import torch

from . import _lib
from ._lib import OP_A, OP_AT, PLAN_A, PLAN_AT, PLAN_BOTH, EPILOGUE_NONE, EPILOGUE_RELU, PlanStats, SpmmOpts, check


def _stream_ptr(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _dev_i32(t, name):
    if t is None:
        return None
    if not (t.is_cuda and t.dtype == torch.int32 and t.is_contiguous()):
        raise ValueError("%s must be a contiguous int32 CUDA tensor" % name)
    return t


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def compute_csr_values(index, dst, in_degree, out_degree, stream=None):
    """Edge coefficients 1/sqrt(outDeg[u]*inDeg[v]) (cuda_gcn/src/cuda/cuda_kernel.cu:144-155)."""
    index, dst = _dev_i32(index, "index"), _dev_i32(dst, "dst")
    in_degree, out_degree = _dev_i32(in_degree, "in_degree"), _dev_i32(out_degree, "out_degree")
    values = torch.empty(dst.numel(), dtype=torch.float32, device=dst.device)
    with torch.cuda.device(dst.device):
        check(_lib.lib().drone_compute_csr_values(_ptr(index), _ptr(dst), _ptr(in_degree), _ptr(out_degree),
                                                  index.numel() - 1, _ptr(values), _stream_ptr(stream)))
    return values


def degree_scales(in_degree, out_degree, stream=None):
    """(in_degree^-1/2, out_degree^-1/2) as float32 tensors: the two factors of the reference's edge coefficient
    (cuda_gcn/src/cuda/cuda_kernel.cu:144-155), for the value-free form of the aggregation."""
    in_degree, out_degree = _dev_i32(in_degree, "in_degree"), _dev_i32(out_degree, "out_degree")
    n = in_degree.numel()
    a = torch.empty(n, dtype=torch.float32, device=in_degree.device)
    b = torch.empty(n, dtype=torch.float32, device=in_degree.device)
    with torch.cuda.device(in_degree.device):
        check(_lib.lib().drone_degree_scales(_ptr(in_degree), _ptr(out_degree), n, _ptr(a), _ptr(b), _stream_ptr(stream)))
    return a, b


class AggregationPlan:
    """Plan for Y = A·X / Y = Aᵀ·X over one local subgraph given as CSR by source vertex
    (struct Graph of cuda_gcn/src/cuda/graph.h:17-41).  Stands where CUDAGraphSum's
    constructor sets cuSPARSE up (cuda_gcn/src/cuda/cuda_module.cu:149-202)."""

    def __init__(self, index, dst, values=None, in_degree=None, out_degree=None, orientations=PLAN_BOTH,
                 stream=None):
        index, dst = _dev_i32(index, "index"), _dev_i32(dst, "dst")
        in_degree, out_degree = _dev_i32(in_degree, "in_degree"), _dev_i32(out_degree, "out_degree")
        if values is not None and not (values.is_cuda and values.dtype == torch.float32 and values.is_contiguous()):
            raise ValueError("values must be a contiguous float32 CUDA tensor")
        self.device = index.device
        self.n_rows = index.numel() - 1
        self.nnz = dst.numel()
        self._h = C.c_void_p(0)
        with torch.cuda.device(self.device):
            check(_lib.lib().drone_plan_create(C.byref(self._h), self.n_rows, self.nnz, _ptr(index), _ptr(dst),
                                               _ptr(values), _ptr(in_degree), _ptr(out_degree), int(orientations),
                                               _stream_ptr(stream)))

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            _lib.lib().drone_plan_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def stats(self):
        st = PlanStats()
        check(_lib.lib().drone_plan_get_stats(self._h, C.byref(st)))
        return st

    def csr(self, orientation):
        """(rowptr, col, val) of one orientation, copied into fresh torch tensors."""
        rp, co, va = C.c_void_p(0), C.c_void_p(0), C.c_void_p(0)
        check(_lib.lib().drone_plan_get_csr(self._h, orientation, C.byref(rp), C.byref(co), C.byref(va)))
        out = []
        for ptr, n, dt in ((rp, self.n_rows + 1, torch.int32), (co, self.nnz, torch.int32), (va, self.nnz, torch.float32)):
            if n == 0:
                out.append(torch.empty(0, dtype=dt, device=self.device))
            else:
                out.append(_view_device_memory(ptr.value, n, dt, self.device).clone())
        return tuple(out)

    def reserve(self, max_features, host_operands=False, padded_rows=False):
        """Allocate now what calls with F <= max_features would allocate on first use (partial sums of split rows;
        with host_operands the device staging of spmm_host; with padded_rows the staging that lets widths which are
        not multiples of 4 run on the float4 kernels)."""
        with torch.cuda.device(self.device):
            check(_lib.lib().drone_plan_reserve(self._h, int(max_features),
                                                (1 if host_operands else 0) | (2 if padded_rows else 0)))

    def set_row_classes(self, row_class, n_classes, stream=None):
        """Give every row a class in 0..n_classes-1 (int32 CUDA tensor [n_rows]); spmm(..., row_class=c) then
        computes the rows of one class only.  n_classes = 1 removes the classes."""
        if n_classes > 1 and not (row_class.is_cuda and row_class.dtype == torch.int32 and row_class.is_contiguous()
                                  and row_class.numel() == self.n_rows):
            raise ValueError("row_class must be a contiguous int32 CUDA tensor with one entry per row")
        with torch.cuda.device(self.device):
            check(_lib.lib().drone_plan_set_row_classes(self._h, _ptr(row_class) if n_classes > 1 else C.c_void_p(0),
                                                        int(n_classes), _stream_ptr(stream)))
        self.n_classes = int(n_classes)

    def spmm(self, orientation, x, out=None, stream=None, row_class=None, relu=False, row_scale=None, unit_values=False,
             push_up_to=None):
        """out[r,:] = sum_k val[k]*x[col[k],:] (rows of the chosen orientation).  x: [n_rows, F] float32.
        With row_class only the rows of that class are written.  relu / row_scale / unit_values are the options of
        drone_spmm_ex: out = max(row_scale[r] * sum, 0), and every coefficient taken as 1.  push_up_to: handle of an
        exchange plan with the peer-memory transport; the call then also sends the mirror rows of out to their
        owners, and drone_exchange_finish (graphsum.exchange_finish) must follow."""
        if not (x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1):
            raise ValueError("x must be a 2-D float32 CUDA tensor with unit inner stride")
        if x.shape[0] != self.n_rows:
            raise ValueError("x has %d rows, plan has %d" % (x.shape[0], self.n_rows))
        f = x.shape[1]
        if out is None:
            out = torch.empty((self.n_rows, f), dtype=torch.float32, device=x.device)
        elif not (out.is_cuda and out.dtype == torch.float32 and out.shape == (self.n_rows, f) and out.stride(1) == 1):
            raise ValueError("out must be a [n_rows, F] float32 CUDA tensor with unit inner stride")
        ldx = x.stride(0) if self.n_rows > 1 else max(f, x.stride(0))
        ldy = out.stride(0) if self.n_rows > 1 else max(f, out.stride(0))
        with torch.cuda.device(self.device):
            if relu or row_scale is not None or unit_values or push_up_to is not None:
                if row_scale is not None and not (row_scale.is_cuda and row_scale.dtype == torch.float32 and
                                                  row_scale.is_contiguous() and row_scale.numel() == self.n_rows):
                    raise ValueError("row_scale must be a contiguous float32 CUDA tensor with one entry per row")
                opts = SpmmOpts(EPILOGUE_RELU if relu else EPILOGUE_NONE, -1 if row_class is None else int(row_class),
                                1 if unit_values else 0, 0, row_scale.data_ptr() if row_scale is not None else None,
                                getattr(push_up_to, "value", push_up_to))
                check(_lib.lib().drone_spmm_ex(self._h, int(orientation), f, _ptr(x), int(ldx), _ptr(out), int(ldy),
                                               C.byref(opts), _stream_ptr(stream)))
            elif row_class is None:
                check(_lib.lib().drone_spmm(self._h, int(orientation), f, _ptr(x), int(ldx), _ptr(out), int(ldy),
                                            _stream_ptr(stream)))
            else:
                check(_lib.lib().drone_spmm_rows(self._h, int(orientation), int(row_class), f, _ptr(x), int(ldx),
                                                 _ptr(out), int(ldy), _stream_ptr(stream)))
        return out

    def spmm_host(self, orientation, x_host, out_host):
        """Same with host numpy/torch CPU buffers (pinned for DMA); synchronous."""
        f = x_host.shape[1]
        xp = x_host.data_ptr() if hasattr(x_host, "data_ptr") else x_host.ctypes.data
        yp = out_host.data_ptr() if hasattr(out_host, "data_ptr") else out_host.ctypes.data
        check(_lib.lib().drone_spmm_host(self._h, int(orientation), int(f), C.c_void_p(xp), C.c_void_p(yp)))
        return out_host

    def spmm_host_submit(self, orientation, x_host, out_host):
        """Queue the same call without waiting (drone_spmm_host_submit); returns the ticket for spmm_host_wait.  At
        most two calls are in flight; x_host / out_host must stay as they are until the ticket has been waited for."""
        f = x_host.shape[1]
        xp = x_host.data_ptr() if hasattr(x_host, "data_ptr") else x_host.ctypes.data
        yp = out_host.data_ptr() if hasattr(out_host, "data_ptr") else out_host.ctypes.data
        ticket = C.c_longlong(-1)
        check(_lib.lib().drone_spmm_host_submit(self._h, int(orientation), int(f), C.c_void_p(xp), C.c_void_p(yp),
                                                C.byref(ticket)))
        return ticket.value

    def spmm_host_wait(self, ticket):
        check(_lib.lib().drone_spmm_host_wait(self._h, int(ticket)))


class _DeviceArray:
    """Borrowed device memory described through the CUDA array interface."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


def _view_device_memory(ptr, n, dtype, device):
    typestr = {torch.int32: "<i4", torch.float32: "<f4"}[dtype]
    with torch.cuda.device(device):
        return torch.as_tensor(_DeviceArray(ptr, n, typestr), device=device)

"""Host-side mirror of the reference's 2-layer GCN step around the aggregation path (CUDAGCN::forward / backward,
cuda_gcn/src/cuda/cuda_gcn.cu:44-83,119-170).  Only the GraphSum layers are this library's kernels; the dense
layers either side stay on cuBLAS (torch.matmul) and the element-wise layers on torch, as in the reference they stay
on cuBLAS and small element-wise kernels.  Used to time an epoch and to check gradients end to end.
"""
import torch

from ._lib import OP_A, OP_AT
from .graphsum import exchange_sum


class GCNStep:
    """forward + backward of Matmul -> GraphSum -> ReLU -> Matmul -> GraphSum -> cross-entropy on one rank.

    aggregate(op, x, out): the sparse aggregation (default: graph.plan.spmm); sync(rows): the mirror/master
    exchange (default: over `comm` when worker_num > 1)."""

    def __init__(self, graph, x, truth, w1, w2, comm=None, worker_num=1, aggregate=None):
        self.g, self.x, self.truth, self.w1, self.w2 = graph, x, truth, w1, w2
        self.comm, self.worker_num = comm, worker_num
        self.aggregate = aggregate or (lambda op, src, out: graph.plan.spmm(op, src, out=out))
        n, dev = x.shape[0], x.device
        hid, out = w1.shape[1], w2.shape[1]
        self.h1 = torch.empty((n, hid), device=dev)
        self.z1 = torch.empty((n, hid), device=dev)
        self.h2 = torch.empty((n, out), device=dev)
        self.logits = torch.empty((n, out), device=dev)
        self.d_h2 = torch.empty((n, out), device=dev)
        self.d_h1 = torch.empty((n, hid), device=dev)
        self.not_mirror = (graph.mirror2worker == -1).unsqueeze(1) if worker_num > 1 else None
        self.labelled = truth >= 0
        self.safe_truth = truth.clamp(min=0).long()

    def sync(self, rows):
        if self.worker_num > 1:
            exchange_sum(self.g.xplan, self.comm, rows)

    def forward(self):
        torch.matmul(self.x, self.w1, out=self.h1)                     # CUDAMatmul::forward
        self.aggregate(OP_AT, self.h1, self.z1)                        # CUDAGraphSum::forward
        self.sync(self.z1)
        self.mask = self.z1 > 0                                        # CUDAReLU::forward, in place
        self.z1.mul_(self.mask)
        torch.matmul(self.z1, self.w2, out=self.h2)
        self.aggregate(OP_AT, self.h2, self.logits)
        self.sync(self.logits)
        # CUDACrossEntropyLoss::forward: loss = mean over labelled rows; gradient not divided by the count
        zmax = self.logits.max(dim=1, keepdim=True).values
        e = torch.exp(self.logits - zmax)
        s = e.sum(dim=1, keepdim=True)
        self.d_logits = e / s
        picked = self.logits.gather(1, self.safe_truth.unsqueeze(1))
        per_row = (torch.log(s) - (picked - zmax)).squeeze(1)
        count = self.labelled.sum().clamp(min=1)
        self.loss = (per_row * self.labelled).sum() / count
        self.d_logits.scatter_add_(1, self.safe_truth.unsqueeze(1), -torch.ones_like(picked))
        self.d_logits.mul_(self.labelled.unsqueeze(1))
        return self.loss

    def backward(self):
        self.aggregate(OP_A, self.d_logits, self.d_h2)                 # CUDAGraphSum::backward
        self.sync(self.d_h2)
        d_a1 = self.d_h2 @ self.w2.t()                                 # CUDAMatmul::backward: dA first ...
        dc = self.d_h2 * self.not_mirror if self.not_mirror is not None else self.d_h2   # ... clear_mirror_grad ...
        self.d_w2 = self.z1.t() @ dc                                   # ... then dW
        d_z1 = d_a1 * self.mask                                        # CUDAReLU::backward
        self.aggregate(OP_A, d_z1, self.d_h1)
        self.sync(self.d_h1)
        dc = self.d_h1 * self.not_mirror if self.not_mirror is not None else self.d_h1
        self.d_w1 = self.x.t() @ dc
        self.d_z1 = d_z1
        return self.d_w1, self.d_w2

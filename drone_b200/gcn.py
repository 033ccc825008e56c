"""Host-side mirror of the reference's GCN step around the aggregation path (CUDAGCN::forward / backward,
cuda_gcn/src/cuda/cuda_gcn.cu:44-83,119-170), for any number of layers.  Only the GraphSum layers, the masking of
mirror rows and the weight broadcast / gradient reduce are this library's kernels and NCCL calls; the dense layers
either side stay on cuBLAS (torch.matmul) and cross-entropy on torch, as in the reference they stay on cuBLAS and
small element-wise kernels.  Used to time an epoch and to check gradients end to end.

Layer l = 1..L:  H_l = A_{l-1} · W_l  (Matmul)  ->  Z_l = Â^T-aggregation of H_l + mirror/master sync (GraphSum)
                 ->  A_l = ReLU(Z_l) for l < L, logits = Z_L.
The reference's module list is this with L = 2 (cuda_gcn.cu:44-83); its layer interface allows more.
"""
import torch

from ._lib import OP_A, OP_AT
from .graphsum import aggregate_and_exchange, clear_mirror_rows, exchange_sum


class GCN:
    """forward + backward of [Matmul -> GraphSum -> ReLU] x (L-1) -> Matmul -> GraphSum -> cross-entropy on one rank.

    weights: list of L tensors [d_{l-1}, d_l].
    aggregate(op, x, out, relu): the sparse aggregation (default: graph.plan.spmm with the ReLU done in the store
    when fuse_relu is set); sync(rows): the mirror/master exchange (default: over `comm` when worker_num > 1).
    With fuse_relu = False the ReLU runs as its own pass, as CUDAReLU::forward does (cuda_module.cu:498-511)."""

    def __init__(self, graph, x, truth, weights, comm=None, worker_num=1, aggregate=None, fuse_relu=True, sync=None):
        self.g, self.x, self.truth = graph, x, truth
        self.weights = list(weights)
        self.n_layers = len(self.weights)
        self.comm, self.worker_num = comm, worker_num
        self.fuse_relu = bool(fuse_relu) and aggregate is None
        self.aggregate = aggregate or (lambda op, src, out, relu=False: graph.plan.spmm(op, src, out=out, relu=relu))
        self._custom_aggregate = aggregate is not None
        self._sync = sync
        n, dev = x.shape[0], x.device
        dims = [w.shape[1] for w in self.weights]
        self.h = [torch.empty((n, d), device=dev) for d in dims]        # Matmul outputs
        self.z = [torch.empty((n, d), device=dev) for d in dims]        # GraphSum outputs (after ReLU for l < L)
        self.d_h = [torch.empty((n, d), device=dev) for d in dims]      # gradients w.r.t. the Matmul outputs
        self.d_a = [torch.empty((n, d), device=dev) for d in dims[:-1]] # gradients w.r.t. the ReLU outputs (masked in place)
        self.mirror2worker = graph.mirror2worker if worker_num > 1 else None
        self.labelled = truth >= 0
        self.safe_truth = truth.clamp(min=0).long()
        self.d_w = [None] * self.n_layers
        self.loss = None

    # ----- pieces -----
    def sync(self, rows):
        if self._sync is not None:
            self._sync(rows)
        elif self.worker_num > 1:
            exchange_sum(self.g.xplan, self.comm, rows)

    def _aggregate_and_sync(self, op, src, out):
        """GraphSum of one layer and direction: aggregation + mirror/master sync.  With the library's own aggregation
        and its peer-memory transport the two are one fused sequence (mirror rows leave from the aggregation's
        store); with a custom aggregation or sync they run one after the other."""
        if not self._custom_aggregate and self._sync is None and self.worker_num > 1:
            aggregate_and_exchange(self.g.plan, self.g.xplan, self.comm, op, src, out)
            return out
        self._aggregate(op, src, out)
        self.sync(out)
        return out

    def _aggregate(self, op, src, out, relu=False):
        if self._custom_aggregate:
            self.aggregate(op, src, out)
            if relu:
                out.clamp_(min=0)
        else:
            self.aggregate(op, src, out, relu)
        return out

    def broadcast_weights(self):
        """weight_broadcast_value_nccl at the start of every forward pass (cuda_communicate.cu:99-105)."""
        if self.worker_num > 1:
            for w in self.weights:
                self.comm.bcast(w, root=0)

    def reduce_gradients(self):
        """weight_reduce_grad_nccl after the backward pass (cuda_communicate.cu:107-115): sums land on rank 0."""
        if self.worker_num > 1:
            for dw in self.d_w:
                self.comm.reduce_sum(dw, root=0)

    # ----- the step -----
    def forward(self):
        a = self.x
        last = self.n_layers - 1
        for l, w in enumerate(self.weights):
            torch.matmul(a, w, out=self.h[l])                              # CUDAMatmul::forward
            relu = l < last
            # The mirror/master sync adds partial sums, so the ReLU can sit in the aggregation's store only when there
            # is nothing to add afterwards (one worker); with several workers it follows the sync.
            fused = relu and self.fuse_relu and self.worker_num == 1 and self._sync is None
            if fused:
                self._aggregate(OP_AT, self.h[l], self.z[l], relu=True)    # CUDAGraphSum::forward + CUDAReLU::forward
            else:
                self._aggregate_and_sync(OP_AT, self.h[l], self.z[l])      # CUDAGraphSum::forward with its sync
            if relu and not fused:
                self.z[l].clamp_(min=0)                                    # CUDAReLU::forward, in place
            a = self.z[l]
        logits = self.z[last]
        # CUDACrossEntropyLoss::forward: loss = mean over labelled rows; gradient not divided by the count
        zmax = logits.max(dim=1, keepdim=True).values
        e = torch.exp(logits - zmax)
        s = e.sum(dim=1, keepdim=True)
        self.d_logits = e / s
        picked = logits.gather(1, self.safe_truth.unsqueeze(1))
        per_row = (torch.log(s) - (picked - zmax)).squeeze(1)
        count = self.labelled.sum().clamp(min=1)
        self.loss = (per_row * self.labelled).sum() / count
        self.d_logits.scatter_add_(1, self.safe_truth.unsqueeze(1), -torch.ones_like(picked))
        self.d_logits.mul_(self.labelled.unsqueeze(1))
        return self.loss

    def backward(self):
        g = self.d_logits
        for l in range(self.n_layers - 1, -1, -1):
            self._aggregate_and_sync(OP_A, g, self.d_h[l])                 # CUDAGraphSum::backward with its sync
            a_prev = self.z[l - 1] if l > 0 else self.x
            if l > 0:
                d_a = torch.matmul(self.d_h[l], self.weights[l].t(), out=self.d_a[l - 1])   # CUDAMatmul::backward: dA first ...
            if self.mirror2worker is not None:
                clear_mirror_rows(self.d_h[l], self.mirror2worker)         # ... clear_mirror_grad (in place) ...
            self.d_w[l] = a_prev.t() @ self.d_h[l]                         # ... then dW
            if l > 0:
                g = d_a.mul_(self.z[l - 1] > 0)                            # CUDAReLU::backward: the mask is (output > 0)
                if l == 1:
                    self.d_z1 = g
        return tuple(self.d_w)


class GCNStep(GCN):
    """The reference's own two-layer model, with the names its variables carry (cuda_gcn.cu:44-83)."""

    def __init__(self, graph, x, truth, w1, w2, comm=None, worker_num=1, aggregate=None, fuse_relu=True):
        super().__init__(graph, x, truth, [w1, w2], comm=comm, worker_num=worker_num, aggregate=aggregate,
                         fuse_relu=fuse_relu)

    w1 = property(lambda self: self.weights[0])
    w2 = property(lambda self: self.weights[1])
    h1 = property(lambda self: self.h[0])
    z1 = property(lambda self: self.z[0])
    h2 = property(lambda self: self.h[1])
    logits = property(lambda self: self.z[1])
    d_h1 = property(lambda self: self.d_h[0])
    d_h2 = property(lambda self: self.d_h[1])
    d_w1 = property(lambda self: self.d_w[0])
    d_w2 = property(lambda self: self.d_w[1])

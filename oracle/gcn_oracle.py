"""Double-precision restatement of the reference's 2-layer GCN step on the whole (unpartitioned) graph.

TEST INFRASTRUCTURE ONLY.  Follows the module list of cuda_gcn/src/cuda/cuda_gcn.cu:44-83 and the order of
CUDAGCN::forward / backward (:119-170):
    Matmul (X·W1, cuda_module.cu:16-48) -> GraphSum (:210-307) -> ReLU in place with mask (:498-523,
    cuda_kernel.cu:384-398) -> Matmul (·W2) -> GraphSum -> softmax cross-entropy (cuda_module.cu:406-483,
    cuda_kernel.cu:326-370): loss = mean over labelled rows, gradient = softmax - onehot on labelled rows and
    NOT divided by the count (count_grad = 1, cuda_module.cu:452), zero on unlabelled rows.
Backward: GraphSum (A·grad), Matmul (dA = dC·W^T first, then dW = A^T·dC; on several workers the mirror rows of dC
are zeroed before dW so that every vertex counts once, cuda_module.cu:50-61,88-105, and dW is summed over workers,
cuda_communicate.cu:107-115), ReLU mask, GraphSum, Matmul.
On one unpartitioned graph every vertex occurs once, which is what the partitioned run must reproduce.
The reference has no fixture for any of these values.  Pinned instead against the reference's own code where a GPU
is present: the first-epoch loss of its CUDAGCN::train_epoch (compiled from the reference sources into oracle/_ref)
on the same graph, features, labels and starting weights equals this restatement's to 1e-5
(tests/test_reference_gpu.py).  Gradients have no such pin and are checked against this restatement only.
"""
import numpy as np
import scipy.sparse as sp


def gcn_step(index, dst, val, x, w1, w2, truth):
    """index/dst/val: CSR by source of the local graph with reference coefficients (float32).
    Returns dict of float64 arrays: z1 (after ReLU), logits, loss, d_logits, d_h2, d_z1, d_h1, d_w1, d_w2."""
    n = len(index) - 1
    a = sp.csr_matrix((np.asarray(val, np.float64), dst, index), shape=(n, n))
    at = a.T.tocsr()
    x = np.asarray(x, np.float64)
    w1 = np.asarray(w1, np.float64)
    w2 = np.asarray(w2, np.float64)
    h1 = x @ w1
    z1 = at @ h1
    mask = z1 > 0
    a1 = np.where(mask, z1, 0.0)
    h2 = a1 @ w2
    logits = at @ h2
    labelled = truth >= 0
    zmax = logits.max(axis=1, keepdims=True)
    e = np.exp(logits - zmax)
    s = e.sum(axis=1, keepdims=True)
    soft = e / s
    rows = np.nonzero(labelled)[0]
    loss = float(np.mean(np.log(s[rows, 0]) - (logits[rows, truth[rows]] - zmax[rows, 0]))) if len(rows) else 0.0
    d_logits = np.zeros_like(logits)
    d_logits[rows] = soft[rows]
    d_logits[rows, truth[rows]] -= 1.0
    d_h2 = a @ d_logits
    d_a1 = d_h2 @ w2.T
    d_w2 = a1.T @ d_h2
    d_z1 = np.where(mask, d_a1, 0.0)
    d_h1 = a @ d_z1
    d_w1 = x.T @ d_h1
    return dict(z1=a1, logits=logits, loss=loss, d_logits=d_logits, d_h2=d_h2, d_z1=d_z1, d_h1=d_h1, d_w1=d_w1,
                d_w2=d_w2)

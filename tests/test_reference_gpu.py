"""The reference ITSELF (its CUDAGraphSum over cuSPARSE, compiled from its own sources into oracle/_ref) against
the oracle and against the library, on identical seeded inputs.  This is what pins the oracle: coefficients must be
bit-identical, outputs and gradients within 1e-5."""
import numpy as np
import pytest
import torch

import drone_b200 as db
from drone_b200 import graphgen as gg
from helpers import REL_TOL

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("scale,sym,dim", [(10, True, 64), (11, False, 41), (9, False, 128)])
def test_reference_graphsum_vs_oracle_and_library(cuda_device, oracle, scale, sym, dim):
    if not oracle.reference_available():
        pytest.skip("oracle/_ref/libref_graphsum.so was not built (reference tree absent at build time)")
    n, u, v = gg.rmat_graph(scale, 12, seed=81 + scale, symmetrise=sym, self_loops="add")
    u, v = u.numpy(), v.numpy()
    in_deg = np.bincount(v, minlength=n).astype(np.int32)
    out_deg = np.bincount(u, minlength=n).astype(np.int32)
    x = gg.seeded_normal(dim, (n, dim))
    gy = gg.seeded_normal(dim + 7, (n, dim))
    l2g, ref_fwd, ref_bwd, ref_val = oracle.reference_graphsum(n, u, v, in_deg, out_deg, x, gy)

    # the oracle's restatement of the local graph and of the coefficients is exact
    nloc, g2l, o_l2g, index, dst = oracle.build_graph(n, u, v)
    assert nloc == len(l2g) and np.array_equal(o_l2g, l2g)
    ind_l, outd_l = in_deg[l2g], out_deg[l2g]
    val = oracle.csr_values_f32(index, dst, ind_l, outd_l)
    assert np.array_equal(val, ref_val)
    # outputs / gradients: double oracle vs the reference's cuSPARSE result
    xl, gl = x[l2g], gy[l2g]
    want_f = oracle.graphsum_forward_f64(xl, index, dst, val)
    want_b = oracle.graphsum_backward_f64(gl, index, dst, val)
    for got, want in ((ref_fwd, want_f), (ref_bwd, want_b)):
        assert np.abs(got - want).max() <= REL_TOL * np.abs(want).max()
    # the library on the same local graph
    t = lambda a: torch.as_tensor(a, device=cuda_device)
    plan = db.AggregationPlan(t(index), t(dst), in_degree=t(ind_l), out_degree=t(outd_l))
    mine_f = plan.spmm(db.OP_AT, t(xl)).cpu().numpy()
    mine_b = plan.spmm(db.OP_A, t(gl)).cpu().numpy()
    assert np.abs(mine_f - ref_fwd).max() <= REL_TOL * np.abs(ref_fwd).max()
    assert np.abs(mine_b - ref_bwd).max() <= REL_TOL * np.abs(ref_bwd).max()
    # and the library is at least as close to the double result as the reference is
    assert np.abs(mine_f - want_f).max() <= 2 * max(np.abs(ref_fwd - want_f).max(), 1e-7 * np.abs(want_f).max())

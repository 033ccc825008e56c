"""The CPU oracle against the only fixed vectors the reference holds for this path, and
against independent restatements (scipy, dense numpy)."""
import numpy as np
import pytest
import scipy.sparse as sp

from drone_b200 import graphgen as gg

# cuda_gcn/src/tools/sparse.cu:28-49 — the cuSPARSE SpMM CSR known-answer case the reference ships.
KAT_ROWPTR = np.array([0, 3, 4, 7, 9], np.int32)
KAT_COL = np.array([0, 2, 3, 1, 0, 2, 3, 1, 3], np.int32)
KAT_VAL = np.arange(1, 10, dtype=np.float32)
KAT_B_COLMAJOR = np.arange(1, 13, dtype=np.float32)           # 4x3, ldb = 4
KAT_C_COLMAJOR = np.array([19, 8, 51, 52, 43, 24, 123, 120, 67, 40, 195, 188], np.float32)  # 4x3, ldc = 4


def test_spmm_known_answer(oracle):
    b = KAT_B_COLMAJOR.reshape(3, 4).T.copy()   # row-major [4,3], as the GCN call sites use
    want = KAT_C_COLMAJOR.reshape(3, 4).T
    got64 = oracle.spmm_csr_f64(KAT_ROWPTR, KAT_COL, KAT_VAL, b)
    got32 = oracle.spmm_csr_f32(KAT_ROWPTR, KAT_COL, KAT_VAL, b)
    assert np.array_equal(got64, want.astype(np.float64))
    assert np.array_equal(got32, want)


def test_transpose_case_of_reference_tool(oracle):
    # cuda_gcn/src/tools/test.cu:47-70: 3x4 matrix, 5 nonzeros, printed after cusparseCsr2cscEx2
    rowptr = np.array([0, 2, 4, 5], np.int32)
    col = np.array([0, 2, 1, 3, 2], np.int32)
    val = np.array([1, 2, 3, 4, 5], np.float32)
    t_rowptr, t_col, t_val = oracle.transpose_csr(3, 4, rowptr, col, val)
    ref = sp.csr_matrix((val, col, rowptr), shape=(3, 4)).tocsc()
    ref.sort_indices()
    assert np.array_equal(t_rowptr, ref.indptr)
    assert np.array_equal(t_col, ref.indices)
    assert np.array_equal(t_val, ref.data)
    # explicit expectation, worked by hand
    assert t_rowptr.tolist() == [0, 1, 2, 4, 5]
    assert t_col.tolist() == [0, 1, 0, 2, 1]
    assert t_val.tolist() == [1.0, 3.0, 2.0, 5.0, 4.0]


def test_build_graph_first_seen_numbering(oracle):
    u = np.array([5, 2, 5, 9, 2], np.int32)
    v = np.array([2, 7, 9, 5, 5], np.int32)
    n, g2l, l2g, index, dst = oracle.build_graph(12, u, v)
    assert n == 4
    assert l2g.tolist() == [5, 2, 7, 9]
    assert g2l[[5, 2, 7, 9]].tolist() == [0, 1, 2, 3] and (g2l == -1).sum() == 8
    # CSR by source, destinations in edge-list order inside a row
    assert index.tolist() == [0, 2, 4, 4, 5]
    assert dst.tolist() == [1, 3, 2, 0, 0]


def test_coefficients_follow_reference_expression(oracle):
    rng = np.random.default_rng(0)
    n, u, v = gg.rmat_graph(8, 8, seed=5)
    index, dst = gg.csr_by_source(u, v, n)
    in_deg = rng.integers(1, 5000, n).astype(np.int32)
    out_deg = rng.integers(1, 5000, n).astype(np.int32)
    got = oracle.csr_values_f32(index.numpy(), dst.numpy(), in_deg, out_deg)
    src = np.repeat(np.arange(n), np.diff(index.numpy()))
    prod = (1.0 * out_deg[src].astype(np.float64) * in_deg[dst.numpy()]).astype(np.float32)
    want = (1.0 / np.sqrt(prod).astype(np.float64)).astype(np.float32)   # sqrtf on float, divide in double
    assert np.array_equal(got, want)
    exact = oracle.csr_values_f64(index.numpy(), dst.numpy(), in_deg, out_deg)
    assert np.max(np.abs(got - exact) / exact) < 2e-7


@pytest.mark.parametrize("name", sorted(gg.tiny_graphs()))
@pytest.mark.parametrize("dim", [1, 3, 8])
def test_graphsum_equals_sparse_product(oracle, name, dim):
    n, u, v = gg.tiny_graphs()[name]
    nloc, g2l, l2g, index, dst = oracle.build_graph(n, u, v)
    src = np.repeat(np.arange(nloc), np.diff(index))
    out_deg = np.maximum(np.bincount(src, minlength=nloc), 1).astype(np.int32)
    in_deg = np.maximum(np.bincount(dst, minlength=nloc), 1).astype(np.int32)
    val = oracle.csr_values_f32(index, dst, in_deg, out_deg)
    rng = np.random.default_rng(1)
    x = rng.standard_normal((nloc, dim)).astype(np.float32)
    a = sp.csr_matrix((val.astype(np.float64), dst, index), shape=(nloc, nloc))
    fwd = oracle.graphsum_forward_f64(x, index, dst, val)
    bwd = oracle.graphsum_backward_f64(x, index, dst, val)
    np.testing.assert_allclose(fwd, a.T @ x.astype(np.float64), rtol=0, atol=1e-14)
    np.testing.assert_allclose(bwd, a @ x.astype(np.float64), rtol=0, atol=1e-14)
    # forward == generic CSR product with the explicit transpose; backward == with A itself
    t = oracle.transpose_csr(nloc, nloc, index, dst, val)
    np.testing.assert_allclose(oracle.spmm_csr_f64(*t, x), fwd, rtol=0, atol=1e-14)
    np.testing.assert_allclose(oracle.spmm_csr_f64(index, dst, val, x), bwd, rtol=0, atol=1e-14)


def test_spmm_f32_threads_agree(oracle):
    n, u, v = gg.rmat_graph(10, 16, seed=2, symmetrise=True, self_loops="add")
    index, dst = gg.csr_by_source(u, v, n)
    in_deg, out_deg = gg.degrees(u, v, n)
    val = oracle.csr_values_f32(index.numpy(), dst.numpy(), in_deg.numpy(), out_deg.numpy())
    x = np.random.default_rng(3).standard_normal((n, 33)).astype(np.float32)
    y1 = oracle.spmm_csr_f32(index.numpy(), dst.numpy(), val, x, threads=1)
    y4 = oracle.spmm_csr_f32(index.numpy(), dst.numpy(), val, x, threads=4)
    assert np.array_equal(y1, y4)
    y64, ab = oracle.spmm_csr_f64(index.numpy(), dst.numpy(), val, x, with_abs=True)
    assert np.max(np.abs(y1 - y64) / np.maximum(ab, 1e-30)) < 1e-5


def test_rmat_generator_is_seed_stable():
    u1, v1 = gg.rmat_edges(12, 5000, seed=42)
    u2, v2 = gg.rmat_edges(12, 5000, seed=42)
    u3, v3 = gg.rmat_edges(12, 2500, seed=42, first_edge=2500)
    assert (u1 == u2).all() and (v1 == v2).all()
    assert (u1[2500:] == u3).all() and (v1[2500:] == v3).all()
    ua, _ = gg.rmat_edges(12, 5000, seed=43)
    assert not (u1 == ua).all()
    # quadrant skew: P(row bit = 0) = a + b = 0.76 at every level
    big_u, big_v = gg.rmat_edges(10, 200000, seed=7)
    top_bit = (big_u.numpy() >> 9) & 1
    assert abs(top_bit.mean() - 0.24) < 0.01
    assert abs(((big_v.numpy() >> 9) & 1).mean() - 0.24) < 0.01

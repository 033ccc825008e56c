"""Parity of the CUDA aggregation (through the C ABI) with the double-precision oracle, the
committed golden vectors, and cuSPARSE called as the reference calls it."""
import os

import numpy as np
import pytest
import torch

import drone_b200 as db
from drone_b200 import graphgen as gg
from helpers import ROOT, REL_TOL, assert_close_to_oracle, graph_case

import make_golden

pytestmark = pytest.mark.gpu

WIDTHS = [1, 2, 3, 4, 31, 32, 33, 41, 47, 64, 128, 256]


def make_plan(dev, index, dst, in_deg, out_deg, **env):
    old = {k: os.environ.get(k) for k in env}
    for k, v in env.items():
        os.environ[k] = str(v)
    try:
        return db.AggregationPlan(torch.as_tensor(index, device=dev), torch.as_tensor(dst, device=dev),
                                  in_degree=torch.as_tensor(in_deg, device=dev),
                                  out_degree=torch.as_tensor(out_deg, device=dev))
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def check_both_orientations(plan, oracle, index, dst, val, x, dev):
    xt = torch.as_tensor(x, device=dev)
    fwd = plan.spmm(db.OP_AT, xt).cpu().numpy()
    bwd = plan.spmm(db.OP_A, xt).cpu().numpy()
    n = len(index) - 1
    t = oracle.transpose_csr(n, n, index, dst, val)
    w_f, a_f = oracle.spmm_csr_f64(*t, x, with_abs=True)
    w_b, a_b = oracle.spmm_csr_f64(index, dst, val, x, with_abs=True)
    assert_close_to_oracle(fwd, w_f, a_f)
    assert_close_to_oracle(bwd, w_b, a_b)
    # the hand-written definition of the layer (push / pull over edges) gives the same numbers
    np.testing.assert_allclose(w_f, oracle.graphsum_forward_f64(x, index, dst, val), rtol=0, atol=1e-12)
    return fwd, bwd


def test_coefficients_bit_exact(cuda_device, oracle):
    n, u, v = gg.rmat_graph(12, 16, seed=21, symmetrise=False, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    rng = np.random.default_rng(0)
    in_deg = rng.integers(1, 3000000, n).astype(np.int32)     # large degrees: products beyond 2^24
    out_deg = rng.integers(1, 3000000, n).astype(np.int32)
    want = oracle.csr_values_f32(index, dst, in_deg, out_deg)
    got = db.compute_csr_values(torch.as_tensor(index, device=cuda_device), torch.as_tensor(dst, device=cuda_device),
                                torch.as_tensor(in_deg, device=cuda_device),
                                torch.as_tensor(out_deg, device=cuda_device))
    assert np.array_equal(got.cpu().numpy(), want)


def test_transpose_matches_oracle(cuda_device, oracle):
    n, u, v = gg.rmat_graph(11, 16, seed=22, symmetrise=False, self_loops="drop")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
    rp, co, va = [t.cpu().numpy() for t in plan.csr(db.OP_AT)]
    t_rp, t_co, t_va = oracle.transpose_csr(n, n, index, dst, val)
    assert np.array_equal(rp, t_rp) and np.array_equal(co, t_co) and np.array_equal(va, t_va)
    rp, co, va = [t.cpu().numpy() for t in plan.csr(db.OP_A)]
    assert np.array_equal(rp, index) and np.array_equal(co, dst) and np.array_equal(va, val)


@pytest.mark.parametrize("name", sorted(gg.tiny_graphs()))
def test_tiny_graphs(cuda_device, oracle, name):
    n, u, v = gg.tiny_graphs()[name]
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u, v)
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
    for f in (1, 3, 32):
        x = gg.seeded_normal(7 + f, (n, f))
        check_both_orientations(plan, oracle, index, dst, val, x, cuda_device)


@pytest.mark.parametrize("f", WIDTHS)
def test_widths_on_small_graph(cuda_device, oracle, f):
    """N = 64 with empty rows, a self-loop-only row and one row that holds a third of all edges."""
    rng = np.random.default_rng(100 + f)
    n = 64
    u = rng.integers(0, n, 400)
    v = rng.integers(0, n, 400)
    u = np.concatenate([u, np.full(200, 5), [9]])
    v = np.concatenate([v, rng.integers(0, n, 200), [9]])
    keep = ~np.isin(u, [3, 17, 40])                      # rows 3, 17, 40 stay empty in A
    u, v = u[keep], v[keep]
    key = np.unique(u.astype(np.int64) * n + v)
    u, v = (key // n).astype(np.int32), (key % n).astype(np.int32)
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u, v)
    x = gg.seeded_normal(f, (n, f))
    for env in ({}, {"DRONE_SHORT_ROW_LIMIT": 4, "DRONE_CHUNK_NNZ": 8}):
        plan = make_plan(cuda_device, index, dst, in_deg, out_deg, **env)
        check_both_orientations(plan, oracle, index, dst, val, x, cuda_device)


@pytest.mark.parametrize("f", [1, 3, 32, 41, 64])
def test_rmat12(cuda_device, oracle, f):
    n, u, v = gg.rmat_graph(12, 16, seed=31, symmetrise=True, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    x = gg.seeded_normal(50 + f, (n, f))
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
    st = plan.stats()
    assert st.n_chunks[db.OP_AT] > 0 and st.n_split_rows[db.OP_AT] > 0     # skewed enough to split rows
    check_both_orientations(plan, oracle, index, dst, val, x, cuda_device)


def test_chunk_list_order_changes_no_bit(cuda_device, oracle):
    """The chunk list is sorted by first column unless DRONE_CHUNK_ORDER=row: every chunk writes its own row or slot."""
    n, u, v = gg.rmat_graph(12, 16, seed=31, symmetrise=True, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    by_row = make_plan(cuda_device, index, dst, in_deg, out_deg, DRONE_CHUNK_ORDER="row")
    by_col = make_plan(cuda_device, index, dst, in_deg, out_deg)
    for f in (32, 41):
        x = torch.as_tensor(gg.seeded_normal(55 + f, (n, f)), device=cuda_device)
        for op in (db.OP_AT, db.OP_A):
            assert torch.equal(by_row.spmm(op, x), by_col.spmm(op, x))


def test_many_partials_per_row(cuda_device, oracle):
    """One row with thousands of nonzeros and tiny chunks: the wide (eight-warp) reduction runs."""
    n = 3000
    u = np.concatenate([np.zeros(n - 1, np.int64), np.arange(1, n)])
    v = np.concatenate([np.arange(1, n), np.zeros(n - 1, np.int64)])
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.astype(np.int32), v.astype(np.int32))
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg, DRONE_SHORT_ROW_LIMIT=4, DRONE_CHUNK_NNZ=8)
    assert plan.stats().n_partials[db.OP_A] > 64
    for f in (1, 32, 41, 256):
        x = gg.seeded_normal(f, (n, f))
        check_both_orientations(plan, oracle, index, dst, val, x, cuda_device)


@pytest.mark.parametrize("f,width", [(128, 64), (256, 64), (256, 128)])
def test_forced_column_slices(cuda_device, oracle, f, width):
    """A call cut into column slices (DRONE_SLICE_WIDTH at plan creation) against the double oracle, both
    orientations, and against the same call in one piece.  A slice of w columns is the product at feature width w:
    it runs the lane-group shape of that width, which adds a long row's nonzeros in another (fixed) interleaving than
    the shape of the full width does, so the two agree to rounding, and a slice agrees bit for bit with a call of
    width w on the same columns."""
    n, u, v = gg.rmat_graph(12, 16, seed=36, symmetrise=False, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    x = gg.seeded_normal(60 + f, (n, f))
    sliced = make_plan(cuda_device, index, dst, in_deg, out_deg, DRONE_SLICE_WIDTH=width)
    whole = make_plan(cuda_device, index, dst, in_deg, out_deg, DRONE_SLICE_WIDTH=0)
    assert sliced.stats().n_partials[db.OP_AT] > 0
    fwd, bwd = check_both_orientations(sliced, oracle, index, dst, val, x, cuda_device)
    xt = torch.as_tensor(x, device=cuda_device)
    for got, op in ((fwd, db.OP_AT), (bwd, db.OP_A)):
        one_piece = whole.spmm(op, xt).cpu().numpy()
        assert np.abs(got - one_piece).max() <= REL_TOL * np.abs(one_piece).max()
        for c0 in range(0, f, width):        # every slice is the narrow call on its own columns
            narrow = whole.spmm(op, xt[:, c0:c0 + width].contiguous()).cpu().numpy()
            assert np.array_equal(got[:, c0:c0 + width], narrow)
    # padded leading dimensions: the slices are column blocks of the caller's own rows
    xp = torch.zeros((n, f + 8), device=cuda_device)
    xp[:, :f] = xt
    yp = torch.full((n, f + 12), 5.0, device=cuda_device)
    sliced.spmm(db.OP_AT, xp[:, :f], out=yp[:, :f])
    assert np.array_equal(yp[:, :f].cpu().numpy(), fwd) and (yp[:, f:] == 5.0).all()


def test_column_slices_chosen_by_size(cuda_device, oracle):
    """131,072 rows at F = 128 are 67 MB of gathered operand: above the threshold at which a call is cut into
    64-column slices by itself.  Checked against the double oracle and against the unsliced call."""
    n, u, v = gg.rmat_graph(17, 8, seed=37, symmetrise=False, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    f = 128
    assert n * f * 4 > 64e6
    x = gg.seeded_normal(61, (n, f))
    auto = make_plan(cuda_device, index, dst, in_deg, out_deg)
    whole = make_plan(cuda_device, index, dst, in_deg, out_deg, DRONE_SLICE_WIDTH=0)
    fwd, bwd = check_both_orientations(auto, oracle, index, dst, val, x, cuda_device)
    xt = torch.as_tensor(x, device=cuda_device)
    for got, op in ((fwd, db.OP_AT), (bwd, db.OP_A)):
        one_piece = whole.spmm(op, xt).cpu().numpy()
        assert np.abs(got - one_piece).max() <= REL_TOL * np.abs(one_piece).max()
        assert np.array_equal(got[:, 64:], whole.spmm(op, xt[:, 64:].contiguous()).cpu().numpy())
    assert auto.stats().last_slice_width == 64 and whole.stats().last_slice_width == 0


def test_full_size_workload_through_its_properties(cuda_device):
    """The benchmark's own workload at its full size (R-MAT scale 20, edge factor 16, symmetrised, self-loops;
    1,048,576 rows, about 32 M nonzeros, F = 64), where the CPU oracle would take minutes: checked through properties
    that hold at any size.  (1) Column sums: 1^T (M X) = (M^T 1)^T X with M^T 1 summed in double from the plan's own
    CSR arrays.  (2) Sampled rows against a double-precision evaluation of their CSR rows.  (3) The graph is
    symmetric and in- and out-degrees coincide, so both orientations are the same matrix: the two results agree to
    rounding.  (4) Linearity in X.  (5) Two calls give the same bits."""
    dev = cuda_device
    n, u, v = gg.rmat_graph(20, 16, seed=20261126, device=dev, symmetrise=True, self_loops="add")
    index, dst = gg.csr_by_source(u, v, n)
    in_deg, out_deg = gg.degrees(u, v, n)
    assert torch.equal(in_deg, out_deg) and dst.numel() > 30_000_000
    plan = db.AggregationPlan(index, dst, in_degree=in_deg, out_degree=out_deg)
    f = 64
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    x = torch.randn((n, f), device=dev, generator=gen)
    x2 = torch.randn((n, f), device=dev, generator=gen)
    results = {}
    for op in (db.OP_AT, db.OP_A):
        y = plan.spmm(op, x)
        assert torch.equal(y, plan.spmm(op, x))                                   # (5)
        rowptr, col, val = plan.csr(op)
        s = torch.zeros(n, dtype=torch.float64, device=dev).index_add_(0, col.long(), val.double())
        want = (s[:, None] * x.double()).sum(0)
        scale = (s.abs()[:, None] * x.double().abs()).sum(0)
        got = y.sum(0, dtype=torch.float64)
        assert float(((got - want).abs() / scale).max()) <= 1e-9                  # (1)
        # (2) the longest row, the first rows and a spread of others, term by term in double
        lengths = rowptr[1:] - rowptr[:-1]
        picks = torch.cat([lengths.argmax().reshape(1), torch.arange(0, 8, device=dev),
                           torch.arange(0, n, n // 50, device=dev)]).unique().tolist()
        for r in picks:
            k0, k1 = int(rowptr[r]), int(rowptr[r + 1])
            terms = val[k0:k1].double()[:, None] * x[col[k0:k1].long()].double()
            bound = REL_TOL * terms.abs().sum(0) + 1e-30
            assert bool(((y[r].double() - terms.sum(0)).abs() <= bound).all()), (op, r, k1 - k0)
        lin = plan.spmm(op, 2.0 * x - x2)                                          # (4)
        y2 = plan.spmm(op, x2)
        assert float((lin - (2.0 * y - y2)).abs().max()) <= REL_TOL * float(lin.abs().max())
        results[op] = y
        del rowptr, col, val, s
    diff = (results[db.OP_AT] - results[db.OP_A]).abs().max()                     # (3)
    assert float(diff) <= REL_TOL * float(results[db.OP_A].abs().max())
    plan.close()


@pytest.mark.parametrize("f", [3, 32, 41, 64, 256])
def test_relu_and_row_scale_in_the_store(cuda_device, oracle, f):
    """drone_spmm_ex: Y = max(row_scale * (A x), 0) equals the same steps applied to drone_spmm's output, bit for
    bit, for short rows, single-chunk rows and split rows alike."""
    n, u, v = gg.rmat_graph(12, 16, seed=39, symmetrise=False, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
    assert plan.stats().n_partials[db.OP_AT] > 0
    x = torch.as_tensor(gg.seeded_normal(70 + f, (n, f)), device=cuda_device)
    scale = torch.as_tensor(gg.seeded_normal(71, (n,)), device=cuda_device).abs() + 0.5
    for op in (db.OP_AT, db.OP_A):
        base = plan.spmm(op, x)
        assert torch.equal(plan.spmm(op, x, relu=True), torch.clamp_min(base, 0.0))
        assert torch.equal(plan.spmm(op, x, row_scale=scale), base * scale[:, None])
        assert torch.equal(plan.spmm(op, x, relu=True, row_scale=scale), torch.clamp_min(base * scale[:, None], 0.0))


@pytest.mark.parametrize("f", [1, 32, 41, 128])
def test_value_free_form(cuda_device, oracle, f):
    """unit_values: the coefficient stream is not read.  Y = diag(in^-1/2) P (diag(out^-1/2) X) with P the 0/1
    pattern is the layer with the reference's coefficients, up to rounding: checked against the double oracle."""
    n, u, v = gg.rmat_graph(12, 16, seed=40, symmetrise=False, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
    xh = gg.seeded_normal(80 + f, (n, f))
    x = torch.as_tensor(xh, device=cuda_device)
    in_s, out_s = db.degree_scales(torch.as_tensor(in_deg, device=cuda_device), torch.as_tensor(out_deg, device=cuda_device))
    np.testing.assert_allclose(in_s.cpu().numpy(), 1.0 / np.sqrt(in_deg.astype(np.float64)), rtol=1e-6)
    t = oracle.transpose_csr(n, n, index, dst, val)
    w_f, a_f = oracle.spmm_csr_f64(*t, xh, with_abs=True)
    w_b, a_b = oracle.spmm_csr_f64(index, dst, val, xh, with_abs=True)
    # forward: rows are destinations (factor in^-1/2), gathered rows are sources (factor out^-1/2)
    fwd = plan.spmm(db.OP_AT, x * out_s[:, None], unit_values=True, row_scale=in_s)
    bwd = plan.spmm(db.OP_A, x * in_s[:, None], unit_values=True, row_scale=out_s)
    assert_close_to_oracle(fwd.cpu().numpy(), w_f, a_f)
    assert_close_to_oracle(bwd.cpu().numpy(), w_b, a_b)
    # pattern only: every coefficient 1
    ones = np.ones_like(val)
    w1, a1 = oracle.spmm_csr_f64(index, dst, ones, xh, with_abs=True)
    assert_close_to_oracle(plan.spmm(db.OP_A, x, unit_values=True).cpu().numpy(), w1, a1)


@pytest.mark.parametrize("f", [1, 32, 41, 64, 128])
def test_table_of_hot_rows(cuda_device, oracle, f):
    """A plan that tags its most gathered columns (forced on a small graph; a quarter of the rows at most, here with
    a table so small that wide rows only fit in part) gives the bits of an untagged plan, for every kernel, and hands
    out untagged CSR arrays."""
    n, u, v = gg.rmat_graph(14, 16, seed=41, symmetrise=False, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    plain = make_plan(cuda_device, index, dst, in_deg, out_deg, DRONE_HOT_TABLE_MB=0)
    tagged = make_plan(cuda_device, index, dst, in_deg, out_deg, DRONE_HOT_MIN_ROWS=1, DRONE_HOT_TABLE_MB=1)
    x = torch.as_tensor(gg.seeded_normal(90 + f, (n, f)), device=cuda_device)
    for op in (db.OP_AT, db.OP_A):
        want = plain.spmm(op, x)
        assert torch.equal(tagged.spmm(op, x), want)
        assert torch.equal(tagged.spmm(op, x), want)          # the table is refilled by every call
        assert torch.equal(tagged.spmm(op, x, relu=True), torch.clamp_min(want, 0.0))
        for a, b in zip(tagged.csr(op), plain.csr(op)):
            assert torch.equal(a, b)
    check_both_orientations(tagged, oracle, index, dst, val, x.cpu().numpy(), cuda_device)
    x2 = torch.as_tensor(gg.seeded_normal(91 + f, (n, f)), device=cuda_device)
    assert torch.equal(tagged.spmm(db.OP_AT, x2), plain.spmm(db.OP_AT, x2))   # other operand: no stale table rows


@pytest.mark.parametrize("f,lead,shift", [(41, 41, 0), (47, 47, 0), (33, 36, 0), (32, 40, 1), (64, 72, 3), (125, 125, 0), (9, 11, 2)])
def test_rows_that_do_not_start_on_16_bytes(cuda_device, oracle, f, lead, shift):
    """Operands whose rows cannot be read 16 bytes at a time (odd widths, odd leading dimensions, a view that starts
    inside a row), without and with the padded staging of drone_plan_reserve: both against the double oracle, each
    repeatable bit for bit, nothing written outside the result's rows, and a row that is never gathered may hold NaN
    without leaking into the result."""
    n, u, v = gg.rmat_graph(11, 16, seed=42, symmetrise=False, self_loops="drop")
    u, v = u.numpy(), v.numpy()
    keep = u != 7                                        # vertex 7 has no out-edge: X[7] is never gathered by A^T x
    u, v = u[keep], v[keep]
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u, v)
    xh = gg.seeded_normal(100 + f, (n, f))
    big = torch.zeros((n + 1, lead + shift), device=cuda_device)
    x = big[:n, shift:shift + f]
    x.copy_(torch.as_tensor(xh))
    x[7] = float("nan")
    t = oracle.transpose_csr(n, n, index, dst, val)
    xz = xh.copy()
    xz[7] = 0.0
    want, mag = oracle.spmm_csr_f64(*t, xz, with_abs=True)
    results = []
    for padded in (False, True):
        plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
        if padded:
            plan.reserve(f, padded_rows=True)
        ybig = torch.full((n + 1, lead + shift), 3.0, device=cuda_device)
        y = ybig[:n, shift:shift + f]
        plan.spmm(db.OP_AT, x, out=y)
        got = y.cpu().numpy()
        assert np.isfinite(got).all()
        assert_close_to_oracle(got, want, mag)
        keep_cols = torch.ones(lead + shift, dtype=torch.bool)
        keep_cols[shift:shift + f] = False
        assert (ybig[:, keep_cols] == 3.0).all() and (ybig[n] == 3.0).all()      # nothing outside the rows was written
        y2 = torch.empty_like(ybig)[:n, shift:shift + f]
        plan.spmm(db.OP_AT, x, out=y2)
        assert torch.equal(y2, y)
        assert torch.equal(plan.spmm(db.OP_AT, x, relu=True), torch.clamp_min(y, 0.0))
        results.append(got)
    assert np.abs(results[0] - results[1]).max() <= REL_TOL * np.abs(want).max()


def test_padded_rows_with_row_classes(cuda_device, oracle):
    """The padded route computes one row class at a time like the plain one: other rows of Y stay as they are."""
    n, u, v = gg.rmat_graph(11, 16, seed=43, symmetrise=False, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
    plan.reserve(41, padded_rows=True)
    x = torch.as_tensor(gg.seeded_normal(44, (n, 41)), device=cuda_device)
    whole = plan.spmm(db.OP_AT, x)
    cls = torch.as_tensor((np.arange(n) % 3).astype(np.int32), device=cuda_device)
    plan.set_row_classes(cls, 3)
    y = torch.full((n, 41), 9.0, device=cuda_device)
    plan.spmm(db.OP_AT, x, out=y, row_class=1)
    assert torch.equal(y[cls == 1], whole[cls == 1]) and (y[cls != 1] == 9.0).all()
    for c in (0, 2):
        plan.spmm(db.OP_AT, x, out=y, row_class=c)
    assert torch.equal(y, whole)


def test_golden_vectors(cuda_device, oracle):
    gold = np.load(os.path.join(ROOT, "tests", "golden", "spmm_golden.npz"))
    for name, scale, ef, seed, sym, loops, widths in make_golden.CASES:
        n, index, dst, in_deg, out_deg = make_golden.case_inputs(scale, ef, seed, sym, loops)
        plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
        for f in widths:
            x = torch.as_tensor(gg.seeded_normal(1000 + f, (n, f)), device=cuda_device)
            assert_close_to_oracle(plan.spmm(db.OP_AT, x).cpu().numpy(), gold["%s/fwd_F%d" % (name, f)])
            assert_close_to_oracle(plan.spmm(db.OP_A, x).cpu().numpy(), gold["%s/bwd_F%d" % (name, f)])


def test_bitwise_repeatable_and_padded_leading_dimension(cuda_device, oracle):
    n, u, v = gg.rmat_graph(11, 16, seed=33, symmetrise=True, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
    for f, ld in ((32, 32), (41, 41), (41, 48), (64, 80)):
        xh = gg.seeded_normal(f, (n, f))
        xp = torch.zeros((n, ld), device=cuda_device)
        xp[:, :f] = torch.as_tensor(xh, device=cuda_device)
        yp = torch.full((n, ld), 7.0, device=cuda_device)
        y1 = plan.spmm(db.OP_AT, xp[:, :f], out=yp[:, :f]).clone()
        y2 = plan.spmm(db.OP_AT, xp[:, :f].contiguous())
        y3 = plan.spmm(db.OP_AT, xp[:, :f].contiguous())
        assert torch.equal(y2, y3)                       # run-to-run bit equality
        if ld % 4 == f % 4 == 0 or (f % 4 and ld % 4):   # same kernel variant => same bits
            assert torch.equal(y1, y2)
        assert (yp[:, f:] == 7.0).all()                  # padding columns untouched
        t = oracle.transpose_csr(n, n, index, dst, val)
        w, a = oracle.spmm_csr_f64(*t, xh, with_abs=True)
        assert_close_to_oracle(y1.cpu().numpy(), w, a)


def test_matches_cusparse_as_called_by_reference(cuda_device, oracle):
    from baseline import cusparse_ref
    n, u, v = gg.rmat_graph(13, 16, seed=34, symmetrise=True, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
    rp, co, va = plan.csr(db.OP_AT)
    for f in (32, 41, 64, 128):
        x = torch.as_tensor(gg.seeded_normal(f, (n, f)), device=cuda_device)
        y_ref = torch.empty_like(x)
        ref = cusparse_ref.CusparseSpmm(rp, co, va, x, y_ref)
        ref.run()
        torch.cuda.synchronize()
        y = plan.spmm(db.OP_AT, x)
        scale = y_ref.abs().max().item()
        assert (y - y_ref).abs().max().item() <= REL_TOL * scale
        ref.close()


def test_host_operand_entry_point(cuda_device, oracle):
    n, u, v = gg.rmat_graph(11, 16, seed=35, symmetrise=True, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
    f = 64
    xh = torch.as_tensor(gg.seeded_normal(3, (n, f))).pin_memory()
    yh = torch.empty((n, f)).pin_memory()
    plan.spmm_host(db.OP_AT, xh, yh)
    xd = xh.to(cuda_device)
    y_dev = plan.spmm(db.OP_AT, xd)
    # pinned operands of 64 columns run as two column halves (copy of the second overlapping the first's result):
    # each half is the 32-column call on those columns bit for bit, the whole agrees with the 64-column call to rounding
    for h in range(2):
        half = plan.spmm(db.OP_AT, xd[:, 32 * h:32 * h + 32].contiguous())
        assert torch.equal(yh[:, 32 * h:32 * h + 32], half.cpu())
    assert (yh - y_dev.cpu()).abs().max() <= REL_TOL * y_dev.abs().max().item()
    w, a = oracle.spmm_csr_f64(*oracle.transpose_csr(n, n, index, dst, val), xh.numpy(), with_abs=True)
    assert_close_to_oracle(yh.numpy(), w, a)
    x24 = xh[:, :24].contiguous().pin_memory()           # below 64 columns: copy, aggregate, copy
    y24 = torch.empty((n, 24)).pin_memory()
    plan.spmm_host(db.OP_AT, x24, y24)
    assert torch.equal(y24, plan.spmm(db.OP_AT, x24.to(cuda_device)).cpu())
    xn = xh.numpy().copy()                               # pageable numpy operands work too
    yn = np.empty_like(xn)
    plan.spmm_host(db.OP_A, xn, yn)
    assert np.array_equal(yn, plan.spmm(db.OP_A, xh.to(cuda_device)).cpu().numpy())


def test_queue_of_host_operand_calls(cuda_device, oracle):
    """drone_spmm_host_submit / _wait: six calls on alternating operand sets and widths, two in flight; every result
    equals the device call on the same operand bit for bit; tickets are checked."""
    n, u, v = gg.rmat_graph(11, 16, seed=36, symmetrise=False, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
    calls = [(db.OP_AT, 64), (db.OP_A, 64), (db.OP_AT, 41), (db.OP_A, 8), (db.OP_AT, 64), (db.OP_AT, 64)]
    xh = [torch.as_tensor(gg.seeded_normal(50 + i, (n, f))).pin_memory() for i, (_, f) in enumerate(calls)]
    yh = [torch.full((n, f), float("nan")).pin_memory() for _, f in calls]
    tickets = []
    for i, (op, f) in enumerate(calls):
        tickets.append(plan.spmm_host_submit(op, xh[i], yh[i]))
        if i >= 1:
            plan.spmm_host_wait(tickets[i - 1])
    plan.spmm_host_wait(tickets[-1])
    assert tickets == list(range(len(calls)))
    for i, (op, f) in enumerate(calls):
        want = plan.spmm(op, xh[i].to(cuda_device)).cpu()
        assert torch.equal(yh[i], want), i
    plan.spmm_host_wait(tickets[0])                      # long finished: returns at once
    with pytest.raises(db.DroneError, match="was not issued"):
        plan.spmm_host_wait(len(calls))
    w, a = oracle.spmm_csr_f64(*oracle.transpose_csr(n, n, index, dst, val), xh[0].numpy(), with_abs=True)
    assert_close_to_oracle(yh[0].numpy(), w, a)


def test_argument_errors(cuda_device, oracle):
    n, u, v = gg.tiny_graphs()["path5"]
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u, v)
    plan = db.AggregationPlan(torch.as_tensor(index, device=cuda_device), torch.as_tensor(dst, device=cuda_device),
                              in_degree=torch.as_tensor(in_deg, device=cuda_device),
                              out_degree=torch.as_tensor(out_deg, device=cuda_device), orientations=db.PLAN_AT)
    x = torch.zeros((n, 8), device=cuda_device)
    with pytest.raises(db.DroneError, match="not prepared"):
        plan.spmm(db.OP_A, x)
    lib = db.lib()
    assert lib.drone_spmm(plan.handle, 1, 2048, x.data_ptr(), 2048, x.data_ptr(), 2048, None) == -1
    assert b"outside 1..1024" in lib.drone_last_error()
    assert lib.drone_spmm(plan.handle, 1, 8, x.data_ptr(), 8, x.data_ptr(), 8, None) == -1
    assert b"alias" in lib.drone_last_error()


def test_malformed_csr_is_refused(cuda_device):
    """Row pointers that decrease or do not end at nnz, and columns outside the matrix, come back as
    DRONE_E_INVALID naming the first bad entry instead of becoming out-of-bounds accesses."""
    def create(index, dst):
        return db.AggregationPlan(torch.tensor(index, dtype=torch.int32, device=cuda_device),
                                  torch.tensor(dst, dtype=torch.int32, device=cuda_device),
                                  values=torch.ones(len(dst), device=cuda_device))
    create([0, 2, 3, 4], [1, 2, 0, 1])                                    # well formed
    with pytest.raises(db.DroneError, match="column index at position 2 is outside 0..2"):
        create([0, 2, 3, 4], [1, 2, 3, 1])
    with pytest.raises(db.DroneError, match="column index at position 0"):
        create([0, 2, 3, 4], [-1, 2, 0, 1])
    with pytest.raises(db.DroneError, match="row pointer 1 is not a valid CSR offset"):
        create([0, 3, 2, 4], [1, 2, 0, 1])
    with pytest.raises(db.DroneError, match="row pointer 3"):
        create([0, 2, 3, 3], [1, 2, 0, 1])
    with pytest.raises(db.DroneError, match="row pointer 0"):
        create([1, 2, 3, 4], [1, 2, 0, 1])


def test_reserve_makes_later_calls_allocation_free(cuda_device, oracle):
    n, u, v = gg.rmat_graph(12, 16, seed=38, symmetrise=False, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    plan = make_plan(cuda_device, index, dst, in_deg, out_deg)
    plan.reserve(64, host_operands=True)
    st = plan.stats()
    assert st.scratch_bytes >= 4 * 64 * max(st.n_partials[0], st.n_partials[1]) > 0
    x = torch.as_tensor(gg.seeded_normal(9, (n, 64)), device=cuda_device)
    y = torch.empty_like(x)
    xh, yh = x.cpu().pin_memory(), torch.empty((n, 64)).pin_memory()
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info(cuda_device)[0]
    plan.spmm(db.OP_AT, x, out=y)
    plan.spmm(db.OP_A, x, out=y)
    plan.spmm_host(db.OP_AT, xh, yh)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(cuda_device)[0] == free0
    assert plan.stats().scratch_bytes == st.scratch_bytes


def test_empty_graph(cuda_device):
    index = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    dst = torch.zeros(0, dtype=torch.int32, device=cuda_device)
    plan = db.AggregationPlan(index, dst, values=torch.zeros(0, device=cuda_device))
    y = plan.spmm(db.OP_AT, torch.zeros((0, 16), device=cuda_device))
    assert y.shape == (0, 16)
    # vertices but no edges: output is all zeros, previous contents overwritten
    index = torch.zeros(11, dtype=torch.int32, device=cuda_device)
    plan = db.AggregationPlan(index, dst, values=torch.zeros(0, device=cuda_device))
    out = torch.full((10, 5), 3.0, device=cuda_device)
    plan.spmm(db.OP_A, torch.ones((10, 5), device=cuda_device), out=out)
    assert (out == 0).all()


@pytest.mark.parametrize("scale,parts", [(10, 1), (12, 3), (14, 8)])
def test_device_graph_build_matches_the_host_builder(cuda_device, scale, parts):
    """drone_graph_build_device against drone_graph_build_host: numbering, row pointers and destinations, bit for bit."""
    from drone_b200 import partition as pt
    n, u, v = gg.rmat_graph(scale, 8, seed=scale, device="cpu", self_loops="add")
    part = pt.ebv_partition(n, u.numpy(), v.numpy(), parts)
    for p in range(parts):
        host = part.local_graph(p)
        du = torch.as_tensor(part.part_u[p].copy(), device=cuda_device)
        dv = torch.as_tensor(part.part_v[p].copy(), device=cuda_device)
        n_local, g2l, l2g, index, dst = pt.device_local_graph(du, dv, n)
        assert n_local == host.n_local
        assert np.array_equal(g2l.cpu().numpy(), host.g2l)
        assert np.array_equal(l2g.cpu().numpy(), host.l2g)
        assert np.array_equal(index.cpu().numpy(), host.index)
        assert np.array_equal(dst.cpu().numpy(), host.dst)
    empty = torch.zeros(0, dtype=torch.int32, device=cuda_device)
    assert pt.device_local_graph(empty, empty, 16)[0] == 0
    bad = torch.tensor([3, 99], dtype=torch.int32, device=cuda_device)
    with pytest.raises(db.DroneError, match="outside"):
        pt.device_local_graph(bad, bad, 16)

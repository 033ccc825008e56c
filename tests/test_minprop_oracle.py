"""The CPU restatement of the cc_cuda / sssp_cuda jobs (oracle/minprop_oracle.c): single-graph fixed points against
brute force, and the partitioned superstep procedure against the single-graph fixed points."""
import numpy as np
import pytest

from drone_b200 import graphgen as gg
from drone_b200 import partition as pt


def csr(n, u, v, w=None):
    order = np.argsort(u, kind="stable")
    rowptr = np.zeros(n + 1, np.int32)
    np.add.at(rowptr, u + 1, 1)
    rowptr = np.cumsum(rowptr).astype(np.int32)
    return rowptr, v[order].astype(np.int32), (w[order].astype(np.float32) if w is not None else None)


def small(scale=7, ef=3, seed=4, sym=False):
    n, u, v = gg.rmat_graph(scale, ef, seed=seed, symmetrise=sym, self_loops="drop")
    return n, u.numpy().astype(np.int32), v.numpy().astype(np.int32)


def reach_closure(n, u, v):
    r = np.eye(n, dtype=bool)
    r[u, v] = True
    for k in range(n):                       # Warshall
        r |= np.outer(r[:, k], r[k, :])
    return r


@pytest.mark.parametrize("sym", [False, True])
def test_cc_fixed_point_is_the_smallest_reaching_id(oracle, sym):
    n, u, v = small(sym=sym)
    rowptr, col, _ = csr(n, u, v)
    got = oracle.cc_fixed_point(rowptr, col)
    reach = reach_closure(n, u, v)           # reach[a, b]: a reaches b
    want = np.array([np.nonzero(reach[:, b])[0].min() for b in range(n)])
    assert np.array_equal(got, want)
    if sym:                                  # on a symmetric graph these are the connected components
        assert all(got[a] == got[b] for a, b in zip(u, v))


@pytest.mark.parametrize("weighted", [False, True])
def test_sssp_matches_dense_bellman_ford(oracle, weighted):
    n, u, v = small(seed=6)
    rng = np.random.default_rng(1)
    w = rng.uniform(0.1, 2.0, len(u)).astype(np.float32) if weighted else None
    rowptr, col, wl = csr(n, u, v, w)
    source = int(u[0])
    got = oracle.sssp_f32(rowptr, col, source, wl)
    dist = np.full(n, np.float32(1e8), np.float32)
    dist[source] = 0
    ww = w if weighted else np.ones(len(u), np.float32)
    for _ in range(n):
        cand = (dist[u] + ww).astype(np.float32)
        new = dist.copy()
        np.minimum.at(new, v, cand)
        if np.array_equal(new, dist):
            break
        dist = new
    assert np.array_equal(got, dist)
    assert (got[got < 1e8] >= 0).all() and got[source] == 0


@pytest.mark.parametrize("parts", [1, 2, 3, 5])
def test_partitioned_cc_reaches_the_single_graph_fixed_point(oracle, parts):
    n, u, v = small(scale=9, ef=4, seed=11)
    rowptr, col, _ = csr(n, u, v)
    want = oracle.cc_fixed_point(rowptr, col)
    p = pt.ebv_partition(n, u, v, parts, keep_self_loops=False)
    got, steps, sizes = oracle.mp_drone_cuda(oracle.MP_CC, n, p.part_u, p.part_v, p.owner)
    touched = p.replicas > 0
    assert np.array_equal(got[touched].astype(np.int64), want[touched])
    assert (got[~touched] == -1).all()
    assert sizes.shape == (steps, parts, 5) and sizes[-1, :, :4].sum() == 0       # the stop rule
    if parts == 1:
        assert steps == 1
    else:
        assert steps > 1 and sizes[0, :, :4].sum() > 0
        # what is sent is received: per superstep the totals of the two directions agree
        assert np.array_equal(sizes[:, :, 0].sum(1), sizes[:, :, 1].sum(1))
        assert np.array_equal(sizes[:, :, 2].sum(1), sizes[:, :, 3].sum(1))


@pytest.mark.parametrize("parts,weighted", [(1, False), (2, False), (4, True), (3, True)])
def test_partitioned_sssp_reaches_the_single_graph_fixed_point(oracle, parts, weighted):
    n, u, v = small(scale=9, ef=4, seed=12)
    rng = np.random.default_rng(2)
    w = rng.uniform(0.1, 2.0, len(u)).astype(np.float32) if weighted else None
    rowptr, col, wl = csr(n, u, v, w)
    source = int(u[len(u) // 2])
    want = oracle.sssp_f32(rowptr, col, source, wl)
    # the partitioner moves edges around: carry the lengths along through a lookup by (u, v)
    p = pt.ebv_partition(n, u, v, parts, keep_self_loops=False)
    lens = None
    if weighted:
        key = {(int(a), int(b)): float(c) for a, b, c in zip(u, v, w)}
        lens = [np.array([key[(int(a), int(b))] for a, b in zip(pu, pv)], np.float32) for pu, pv in zip(p.part_u, p.part_v)]
    got, steps, sizes = oracle.mp_drone_cuda(oracle.MP_SSSP, n, p.part_u, p.part_v, p.owner, source=source, parts_len=lens)
    touched = p.replicas > 0
    assert np.array_equal(got[touched], want[touched])
    assert sizes[-1, :, :4].sum() == 0
    assert (want < 1e8).sum() > n // 20                 # the case is not trivial: the source reaches something

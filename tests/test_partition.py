"""EBV partitioner and routing tables (host code, no GPU)."""
import os

import numpy as np
import pytest

from drone_b200 import graphgen as gg
from drone_b200 import partition as pt
from oracle import ebv_oracle


def small_graph(scale=9, seed=3, sym=True):
    n, u, v = gg.rmat_graph(scale, 8, seed=seed, symmetrise=sym, self_loops="add")
    return n, u.numpy(), v.numpy()


@pytest.mark.parametrize("parts", [1, 2, 3, 8])
def test_vertex_cut_invariants(parts):
    n, u, v = small_graph()
    p = pt.ebv_partition(n, u, v, parts)
    # every edge lives in exactly one part
    all_edges = np.concatenate([pu.astype(np.int64) * n + pv for pu, pv in zip(p.part_u, p.part_v)])
    assert len(all_edges) == len(u)
    assert np.array_equal(np.sort(all_edges), np.sort(u.astype(np.int64) * n + v))
    # replica counts and owners agree with where the edges went
    present = np.stack([p.present(q) for q in range(parts)])
    assert np.array_equal(present.sum(0), p.replicas)
    has_edge = p.replicas > 0
    assert (p.owner[has_edge] >= 0).all() and (p.owner[~has_edge] == -1).all()
    assert present[p.owner[has_edge], np.nonzero(has_edge)[0]].all()       # the owner holds the vertex
    # master rule of the reference: replica number (id mod #replicas), parts ascending
    for x in np.nonzero(p.replicas > 1)[0][:200]:
        holders = np.nonzero(present[:, x])[0]
        assert p.owner[x] == holders[x % len(holders)]
    # Master.<p> and Mirror.<p> are mutually consistent
    mirrors_seen = {}
    for q in range(parts):
        mv, num, wk = p.master_rows(q)
        assert num.sum() == len(wk) and (num >= 1).all()
        pos = 0
        for x, k in zip(mv.tolist(), num.tolist()):
            for w in wk[pos:pos + k].tolist():
                mirrors_seen[(x, w)] = q
            pos += k
    count = 0
    for q in range(parts):
        mr, ow = p.mirror_rows(q)
        for x, o in zip(mr.tolist(), ow.tolist()):
            assert mirrors_seen[(x, q)] == o
            count += 1
    assert count == len(mirrors_seen) == int((p.replicas[p.replicas > 1] - 1).sum())
    if parts > 1:
        assert p.edge_imbalance() < 1.3
        assert 1.0 <= p.replication_factor() <= parts


def test_matches_python_restatement():
    n, u, v = small_graph(scale=7, seed=11, sym=False)
    for parts, keep in ((2, True), (4, True), (3, False)):
        p = pt.ebv_partition(n, u, v, parts, keep_self_loops=keep)
        ref_parts, ref_owner, ref_rep = ebv_oracle.ebv_partition(n, list(zip(u.tolist(), v.tolist())), parts, keep)
        for q in range(parts):
            assert list(zip(p.part_u[q].tolist(), p.part_v[q].tolist())) == ref_parts[q]
        assert p.owner.tolist() == ref_owner and p.replicas.tolist() == ref_rep


def test_self_loops_dropped_like_root_partitioner():
    n, u, v = small_graph(scale=7, seed=12)
    p = pt.ebv_partition(n, u, v, 2, keep_self_loops=False)
    assert sum(len(x) for x in p.part_u) == int((u != v).sum())
    assert all((pu != pv).all() for pu, pv in zip(p.part_u, p.part_v))


def test_file_round_trip(tmp_path):
    n, u, v = small_graph(scale=8, seed=13)
    p = pt.ebv_partition(n, u, v, 3)
    p.write_files(str(tmp_path))
    first = open(tmp_path / "G.0").readline().split()
    assert len(first) == 2                                        # "u v" per line
    q = pt.read_partition_files(str(tmp_path), n, 3)
    for a, b in zip(p.part_u + p.part_v, q.part_u + q.part_v):
        assert np.array_equal(a, b)
    assert np.array_equal(p.replicas, q.replicas)
    rep = p.replicas > 1
    assert np.array_equal(p.owner[rep], q.owner[rep])
    for k in range(3):
        for a, b in zip(p.master_rows(k) + p.mirror_rows(k), q.master_rows(k) + q.mirror_rows(k)):
            assert np.array_equal(a, b)


def test_local_graph_follows_reference_numbering(oracle):
    n, u, v = small_graph(scale=8, seed=14)
    p = pt.ebv_partition(n, u, v, 2)
    for k in range(2):
        g = p.local_graph(k)
        nloc, g2l, l2g, index, dst = oracle.build_graph(n, p.part_u[k], p.part_v[k])
        assert g.n_local == nloc
        assert np.array_equal(g.g2l, g2l) and np.array_equal(g.l2g, l2g)
        assert np.array_equal(g.index, index) and np.array_equal(g.dst, dst)
        # routing tables by local id
        mr, ow = p.mirror_rows(k)
        want = np.full(nloc, -1, np.int32)
        want[g2l[mr]] = ow
        assert np.array_equal(g.mirror2worker, want)
        mv, num, wk = p.master_rows(k)
        deg = np.zeros(nloc, np.int64)
        deg[g2l[mv]] = num
        assert np.array_equal(np.diff(g.master_worker_index), deg)
        pos = 0
        for x, c in zip(mv.tolist(), num.tolist()):
            lo = g.master_worker_index[g2l[x]]
            assert g.master2workers[lo:lo + c].tolist() == wk[pos:pos + c].tolist()
            pos += c


def test_bad_input_is_an_error():
    import drone_b200 as db
    with pytest.raises(db.DroneError, match="outside"):
        pt.ebv_partition(4, np.array([0, 9], np.int32), np.array([1, 2], np.int32), 2)
    with pytest.raises(db.DroneError, match="n_parts"):
        pt.ebv_partition(4, np.array([0], np.int32), np.array([1], np.int32), 0)


def test_rank_with_only_its_own_edges_builds_the_same_tables():
    """A rank that holds its own edges plus the presence words of all vertices gets the same local graph and
    routing tables as one that holds the whole partition."""
    n, u, v = gg.rmat_graph(11, 8, seed=77, device="cpu", self_loops="add")
    u, v = np.asarray(u), np.asarray(v)
    parts = 5
    full = pt.ebv_partition(n, u, v, parts)
    bits = full.presence_bits()
    plain = pt.Partition(n, parts, full.part_u, full.part_v, full.owner, full.replicas)
    for q in range(parts):
        assert np.array_equal((bits >> np.uint64(q)) & np.uint64(1) != 0, plain.present(q))
    assert np.array_equal(np.array([bin(int(b)).count("1") for b in bits]), full.replicas)
    for p in range(parts):
        pu, pv = [None] * parts, [None] * parts
        pu[p], pv[p] = full.part_u[p], full.part_v[p]
        alone = pt.Partition(n, parts, pu, pv, full.owner, full.replicas, present_bits=bits)
        a, b = alone.local_graph(p), plain.local_graph(p)
        for name in ("l2g", "index", "dst", "master_worker_index", "master2workers", "mirror2worker"):
            assert np.array_equal(getattr(a, name), getattr(b, name)), name


# ----- against files written by the reference's own partitioner (tests/golden/make_ebv_golden.py) -----
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ebv_golden.npz")
GOLDEN_CASES = ["tiny", "uniform_p3", "skewed_p2", "skewed_p4_blocks", "skewed_p8"]


def golden_case(name):
    g = np.load(GOLDEN)
    n, parts, keep = g[name + "/meta"].tolist()
    files = {"%s.%d" % (kind, p): g["%s/%s.%d" % (name, kind, p)].tobytes()
             for p in range(parts) for kind in ("G", "Master", "Mirror")}
    return n, g[name + "/u"], g[name + "/v"], parts, bool(keep), files


def written_files(part, directory):
    part.write_files(directory)
    out = {}
    for p in range(part.n_parts):
        for kind in ("G", "Master", "Mirror"):
            with open(os.path.join(directory, "%s.%d" % (kind, p)), "rb") as f:
                out["%s.%d" % (kind, p)] = f.read()
    return out


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_files_equal_reference_partitioner(name, tmp_path):
    """With the reference's tie order (std::sort) the three files of every part equal, byte for byte, what the
    reference's partitioner wrote for the same edge list."""
    n, u, v, parts, keep, ref_files = golden_case(name)
    p = pt.ebv_partition(n, u, v, parts, keep_self_loops=keep, std_sort_ties=True)
    mine = written_files(p, str(tmp_path))
    assert sorted(mine) == sorted(ref_files)
    for fname in sorted(ref_files):
        assert mine[fname] == ref_files[fname], fname


def test_restatement_equals_reference_partitioner_without_ties_in_play(tmp_path):
    """At most 16 edges per rank: std::sort is an insertion sort there and keeps equal keys in input order, so the
    stable restatements (Python and the library's default) must reproduce the reference's files as well."""
    n, u, v, parts, keep, ref_files = golden_case("tiny")
    ref_parts, ref_owner, ref_rep = ebv_oracle.ebv_partition(n, list(zip(u.tolist(), v.tolist())), parts, keep)
    for q in range(parts):
        lines = ref_files["G.%d" % q].decode().split("\n")[:-1]
        assert ["%d %d" % e for e in ref_parts[q]] == lines
    p = pt.ebv_partition(n, u, v, parts, keep_self_loops=keep)
    assert p.owner.tolist() == ref_owner and p.replicas.tolist() == ref_rep
    assert written_files(p, str(tmp_path)) == ref_files


@pytest.mark.parametrize("name", ["uniform_p3", "skewed_p2", "skewed_p8"])
def test_python_restatement_equals_reference_partitioner(name):
    """The pure-Python restatement with the reference's tie order: the edges of every part in the reference's order,
    and owners / replica counts that give the reference's Master and Mirror files."""
    from oracle import oracle
    oracle.build()
    n, u, v, parts, keep, ref_files = golden_case(name)
    ref_parts, ref_owner, ref_rep = ebv_oracle.ebv_partition(n, list(zip(u.tolist(), v.tolist())), parts, keep,
                                                             std_sort_ties=True)
    for q in range(parts):
        lines = ref_files["G.%d" % q].decode().split("\n")[:-1]
        assert ["%d %d" % e for e in ref_parts[q]] == lines
    masters = {}
    for q in range(parts):
        for line in ref_files["Master.%d" % q].decode().split("\n")[:-1]:
            ids = [int(t) for t in line.split()]
            masters[ids[0]] = (q, len(ids))          # vertex -> (owner, replicas)
    want = {x: (ref_owner[x], ref_rep[x]) for x in range(n) if ref_rep[x] > 1}
    assert masters == want


@pytest.mark.parametrize("name", GOLDEN_CASES[1:])
def test_stable_order_cuts_as_well_as_reference(name):
    """The default (stable) order changes which of several equally ranked edges goes first, not the quality of the cut:
    replication factor within 3 % of the reference's, edge balance as tight."""
    n, u, v, parts, keep, ref_files = golden_case(name)
    ref_replicas = np.zeros(n, np.int64)
    ref_sizes = []
    for q in range(parts):
        e = np.array(ref_files["G.%d" % q].split(), dtype=np.int64).reshape(-1, 2)
        ref_sizes.append(len(e))
        ref_replicas[np.unique(e)] += 1
    p = pt.ebv_partition(n, u, v, parts, keep_self_loops=keep)
    assert sum(len(x) for x in p.part_u) == sum(ref_sizes)
    assert abs(p.replication_factor() / (ref_replicas.sum() / n) - 1) < 0.03
    assert p.edge_imbalance() < max(ref_sizes) * parts / sum(ref_sizes) + 0.05


def test_reference_partitioner_live(tmp_path):
    """The reference's partitioner itself, run here as 3 ranks on a fresh edge list (skipped where it was not built)."""
    from oracle import oracle
    if oracle.reference_ebv_binary(True) is None:
        pytest.skip("reference partitioner not built (make -C oracle ref_ebv)")
    rng = np.random.default_rng(77)
    n, m = 4000, 30000
    u = (n * rng.random(m) ** 2).astype(np.int32)
    v = (n * rng.random(m) ** 2).astype(np.int32)
    for keep in (True, False):
        ref_files = oracle.reference_ebv_partition(n, u, v, 3, keep, str(tmp_path / ("ref%d" % keep)))
        p = pt.ebv_partition(n, u, v, 3, keep_self_loops=keep, std_sort_ties=True)
        assert written_files(p, str(tmp_path / ("mine%d" % keep))) == ref_files
    # a million edges of an R-MAT graph over 8 ranks: batches of the full 1000 edges, long runs of equal degree sums
    n, u, v = gg.rmat_graph(16, 16, seed=78, symmetrise=False, self_loops="add")
    u, v = u.numpy(), v.numpy()
    ref_files = oracle.reference_ebv_partition(n, u, v, 8, True, str(tmp_path / "ref_rmat"))
    p = pt.ebv_partition(n, u, v, 8, keep_self_loops=True, std_sort_ties=True)
    assert written_files(p, str(tmp_path / "mine_rmat")) == ref_files


@pytest.mark.parametrize("name", ["uniform_p3", "skewed_p4_blocks"])
def test_loader_reads_files_of_reference_partitioner(name, tmp_path):
    """The text loader on the files the reference's partitioner wrote: same edges, owners and replica counts as the
    partition computed here, and the same routing tables for every part."""
    n, u, v, parts, keep, ref_files = golden_case(name)
    for fname, data in ref_files.items():
        (tmp_path / fname).write_bytes(data)
    loaded = pt.read_partition_files(str(tmp_path), n, parts)
    p = pt.ebv_partition(n, u, v, parts, keep_self_loops=keep, std_sort_ties=True)
    assert loaded.owner.tolist() == p.owner.tolist() and loaded.replicas.tolist() == p.replicas.tolist()
    for q in range(parts):
        assert np.array_equal(loaded.part_u[q], p.part_u[q]) and np.array_equal(loaded.part_v[q], p.part_v[q])
        for a, b in zip(loaded.master_rows(q), p.master_rows(q)):
            assert np.array_equal(a, b)
        for a, b in zip(loaded.mirror_rows(q), p.mirror_rows(q)):
            assert np.array_equal(a, b)

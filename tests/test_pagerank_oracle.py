"""The PageRank oracles against each other and against a dense power iteration (no GPU)."""
import numpy as np
import pytest
import torch

from drone_b200 import graphgen as gg
from drone_b200 import partition as pt


def pr_case(scale=9, seed=21, parts=2):
    """Directed R-MAT plus a ring (so that every vertex occurs in some part: the GPU job only knows vertices
    that touch an edge, while |V| counts all ids) with three vertices made dangling."""
    n, u, v = gg.rmat_graph(scale, 8, seed=seed, symmetrise=False, self_loops="drop")
    ring = np.arange(n, dtype=np.int32)
    u = np.concatenate([u.numpy(), ring])
    v = np.concatenate([v.numpy(), (ring + 1) % n])
    keep = ~np.isin(u, [5, 17, 100])
    key = np.unique(u[keep].astype(np.int64) * n + v[keep])
    u, v = (key // n).astype(np.int32), (key % n).astype(np.int32)
    out_deg = np.bincount(u, minlength=n).astype(np.int32)
    part = pt.ebv_partition(n, u, v, parts, keep_self_loops=False)
    return n, u, v, out_deg, part


def dense_power(n, u, v, iterations, d):
    a = np.zeros((n, n))
    np.add.at(a, (v, u), 1.0)
    outd = np.bincount(u, minlength=n).astype(np.float64)
    pr = np.full(n, 1.0 / n)
    for _ in range(iterations):
        contrib = np.where(outd > 0, pr / np.maximum(outd, 1), 0.0)
        dangling = pr[outd == 0].sum()
        pr = (1 - d) / n + d * (a @ contrib + dangling / n)
    return pr


def test_power_iteration_matches_dense_algebra(oracle):
    n, u, v, out_deg, _ = pr_case(scale=8)
    index, dst = gg.csr_by_source(torch.as_tensor(u), torch.as_tensor(v), n)
    got = oracle.pagerank_power_f64(index.numpy(), dst.numpy(), 20, 0.85)
    np.testing.assert_allclose(got, dense_power(n, u, v, 20, 0.85), rtol=1e-12)
    assert abs(got.sum() - 1.0) < 1e-12


@pytest.mark.parametrize("parts", [1, 2, 4])
def test_gpu_job_semantics_do_not_depend_on_the_partition(oracle, parts):
    """In double and with a tiny threshold the delta schedule converges to |V| times the normalised
    PageRank, whatever the vertex cut."""
    n, u, v, out_deg, part = pr_case(parts=parts)
    pr, steps, sizes = oracle.pr_drone_cuda(n, part.part_u, part.part_v, out_deg, part.owner, eps=1e-13,
                                            max_steps=2000, dtype=np.float64)
    index, dst = gg.csr_by_source(torch.as_tensor(u), torch.as_tensor(v), n)
    ref = oracle.pagerank_power_f64(index.numpy(), dst.numpy(), 400, float(np.float32(0.85)))
    touched = part.replicas > 0
    if parts == 1:
        # one part: nothing is ever exchanged, so the master's stop rule ends the job right after PEval
        assert steps == 1 and sizes.sum() == 0 and (pr[touched] == 1.0).all()
    else:
        np.testing.assert_allclose(pr[touched], n * ref[touched], rtol=1e-9)
        assert steps > 5 and (sizes[-1] == 0).all() and (sizes[0] > 0).all()


def test_float_gpu_job_is_close_to_double(oracle):
    n, u, v, out_deg, part = pr_case(parts=2)
    p32, s32, _ = oracle.pr_drone_cuda(n, part.part_u, part.part_v, out_deg, part.owner, eps=1e-6, dtype=np.float32)
    p64, s64, _ = oracle.pr_drone_cuda(n, part.part_u, part.part_v, out_deg, part.owner, eps=1e-6, dtype=np.float64)
    touched = part.replicas > 0
    assert np.max(np.abs(p32[touched] - p64[touched]) / p64[touched]) < 1e-3


def test_cpu_job_stop_rule_and_accuracy(oracle):
    n, u, v, out_deg, part = pr_case(parts=2)
    pr, steps, msgs = oracle.pr_drone_cpu(n, part.part_u, part.part_v, out_deg, part.owner, eps=0.01, max_steps=200)
    assert 2 < steps <= 200 and msgs > 0
    # the CPU job has no dangling-mass term: compare with the same recurrence in double, no threshold
    a = np.zeros((n, n))
    np.add.at(a, (v, u), 1.0 / np.maximum(out_deg[u], 1))
    ref = np.ones(n)
    for _ in range(300):
        ref = 0.85 * (a @ ref) + 0.15
    touched = part.replicas > 0
    # eps = 0.01 leaves up to eps/(1-alpha) unpropagated per vertex
    assert np.max(np.abs(pr[touched] - ref[touched])) < 0.5
    assert np.median(np.abs(pr[touched] - ref[touched]) / ref[touched]) < 0.05
    # a single worker never has mirror messages: the master stops it after the first IncEval
    one = pt.ebv_partition(n, u, v, 1, keep_self_loops=False)
    _, steps1, msgs1 = oracle.pr_drone_cpu(n, one.part_u, one.part_v, out_deg, one.owner, eps=0.01, max_steps=200)
    assert steps1 == 1 and msgs1 == 0


@pytest.mark.parametrize("parts", [1, 2, 5])
def test_cpu_job_with_hash_map_state_gives_the_same_bits(oracle, parts):
    """State in hash maps keyed by global id (the Go program's layout) against the flat-array restatement."""
    n, u, v, out_deg, part = pr_case(scale=10, seed=23, parts=parts)
    flat = oracle.pr_drone_cpu(n, part.part_u, part.part_v, out_deg, part.owner, eps=0.01, max_steps=200)
    maps = oracle.pr_drone_cpu(n, part.part_u, part.part_v, out_deg, part.owner, eps=0.01, max_steps=200, maps=True)
    assert np.array_equal(flat[0], maps[0]) and flat[1] == maps[1] and flat[2] == maps[2]

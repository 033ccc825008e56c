"""Generates tests/golden/spmm_golden.npz and tests/golden/jobs_golden.npz: oracle outputs on seeded inputs.

    python tests/golden/make_golden.py

Inputs are not stored: graphs come from the seeded R-MAT generator and dense operands from
graphgen.seeded_normal, both pure functions of their seed.  Outputs are the double-precision
oracle results (oracle/drone_oracle.c) for the forward (A^T X) and backward (A X) aggregation.
The reference itself has no fixtures for this path; these pin the oracle so that later changes
to it are caught, and give the GPU tests fixed targets.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from drone_b200 import graphgen as gg  # noqa: E402
from oracle import oracle  # noqa: E402

CASES = [  # (name, scale, edge_factor, graph seed, symmetrise, self_loops, [F...])
    ("rmat8_dir", 8, 16, 11, False, "drop", [1, 3, 32, 41, 64]),
    ("rmat8_sym", 8, 16, 12, True, "add", [1, 3, 32, 41, 64]),
    ("rmat10_sym", 10, 16, 13, True, "add", [3, 32]),
]


def case_inputs(scale, ef, seed, sym, loops):
    n, u, v = gg.rmat_graph(scale, ef, seed=seed, symmetrise=sym, self_loops=loops)
    index, dst = gg.csr_by_source(u, v, n)
    in_deg, out_deg = gg.degrees(u, v, n)
    # degree 0 never meets an edge, but keep the arrays strictly positive like the degree files
    in_deg = np.maximum(in_deg.numpy(), 1).astype(np.int32)
    out_deg = np.maximum(out_deg.numpy(), 1).astype(np.int32)
    return n, index.numpy(), dst.numpy(), in_deg, out_deg


JOB_CASES = [  # (name, scale, edge_factor, graph seed, parts)
    ("rmat8_p1", 8, 8, 21, 1),
    ("rmat9_p3", 9, 8, 22, 3),
    ("rmat10_p4", 10, 6, 23, 4),
]


def job_inputs(scale, ef, seed, parts):
    """Directed R-MAT plus a ring (every id occurs), EBV-partitioned; CSR by source of the whole graph."""
    from drone_b200 import partition as pt
    n, u, v = gg.rmat_graph(scale, ef, seed=seed, symmetrise=False, self_loops="drop")
    ring = np.arange(n, dtype=np.int64)
    key = np.unique(np.concatenate([u.numpy().astype(np.int64) * n + v.numpy(), ring * n + (ring + 1) % n]))
    u, v = (key // n).astype(np.int32), (key % n).astype(np.int32)
    order = np.argsort(u, kind="stable")
    rowptr = np.concatenate([[0], np.cumsum(np.bincount(u, minlength=n))]).astype(np.int32)
    col = v[order].astype(np.int32)
    out_deg = np.bincount(u, minlength=n).astype(np.int32)
    part = pt.ebv_partition(n, u, v, parts, keep_self_loops=False)
    return n, u, v, rowptr, col, out_deg, part


def job_outputs(scale, ef, seed, parts):
    """What the oracle computes for the pr / cc / sssp jobs on one case (dict of arrays)."""
    n, u, v, rowptr, col, out_deg, part = job_inputs(scale, ef, seed, parts)
    out = {"edges": np.int64(len(u)), "part_sizes": np.array([len(x) for x in part.part_u], np.int64),
           "owner_sum": np.int64(part.owner.astype(np.int64).sum()), "replicas_sum": np.int64(part.replicas.sum())}
    out["pr_power_f64"] = oracle.pagerank_power_f64(rowptr, col, 20, 0.85)
    pr, steps, sizes = oracle.pr_drone_cuda(n, part.part_u, part.part_v, out_deg, part.owner, eps=1e-6, dtype=np.float64)
    out["pr_job_f64"], out["pr_job_steps"], out["pr_job_sizes"] = pr, np.int64(steps), sizes
    pr, steps, msgs = oracle.pr_drone_cpu(n, part.part_u, part.part_v, out_deg, part.owner, eps=0.01, max_steps=200)
    out["pr_cpu_job_f32"], out["pr_cpu_job_steps"], out["pr_cpu_job_messages"] = pr, np.int64(steps), np.int64(msgs)
    out["cc_labels"] = oracle.cc_fixed_point(rowptr, col)
    source = int(u[len(u) // 2])
    out["sssp_source"] = np.int64(source)
    out["sssp_dist"] = oracle.sssp_f32(rowptr, col, source)
    for kind, name in ((oracle.MP_CC, "cc"), (oracle.MP_SSSP, "sssp")):
        vals, steps, sizes = oracle.mp_drone_cuda(kind, n, part.part_u, part.part_v, part.owner, source=source)
        out[name + "_job_values"], out[name + "_job_steps"], out[name + "_job_sizes"] = vals, np.int64(steps), sizes
    return out


def main():
    jobs = {}
    for name, scale, ef, seed, parts in JOB_CASES:
        for k, a in job_outputs(scale, ef, seed, parts).items():
            jobs["%s/%s" % (name, k)] = a
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "jobs_golden.npz")
    np.savez_compressed(path, **jobs)
    print(path, os.path.getsize(path), "bytes")
    out = {}
    for name, scale, ef, seed, sym, loops, widths in CASES:
        n, index, dst, in_deg, out_deg = case_inputs(scale, ef, seed, sym, loops)
        val = oracle.csr_values_f32(index, dst, in_deg, out_deg)
        out[name + "/nnz"] = np.int64(len(dst))
        out[name + "/val_sum"] = np.float64(val.astype(np.float64).sum())
        for f in widths:
            x = gg.seeded_normal(1000 + f, (n, f))
            out["%s/fwd_F%d" % (name, f)] = oracle.graphsum_forward_f64(x, index, dst, val)
            out["%s/bwd_F%d" % (name, f)] = oracle.graphsum_backward_f64(x, index, dst, val)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "spmm_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()

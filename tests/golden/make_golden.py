"""Generates tests/golden/spmm_golden.npz: oracle outputs on seeded inputs.

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


def main():
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

"""Generates tests/golden/ebv_golden.npz: what the REFERENCE's partitioner writes for a few seeded edge lists.

    make -C oracle ref_ebv REFERENCE=<reference checkout>
    python tests/golden/make_ebv_golden.py

The partitioner (EBV_mpi.cpp, and the copy under cuda_gcn/src/tools that keeps self-loops) is compiled from its own
source file against stand-ins for the MPI and gflags calls it makes (oracle/ref_shim/ebv) and run as P ranks.  Stored
per case: the input edge list, and every G.<p> / Master.<p> / Mirror.<p> file byte for byte.  The case "tiny" gives
each rank at most 16 edges, where std::sort leaves equal keys in input order; the others exercise its tie order.
"""
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle  # noqa: E402

CASES = [  # (name, vertices, edge lines, parts, keep self-loops, seed, skew)
    ("tiny", 24, 60, 4, False, 5, 1.0),
    ("uniform_p3", 300, 3000, 3, False, 6, 1.0),
    ("skewed_p2", 2500, 20000, 2, True, 7, 2.5),
    ("skewed_p4_blocks", 9000, 24000, 4, True, 8, 2.0),    # more than 1000 * P vertices: several blocks of Master lines
    ("skewed_p8", 1200, 16000, 8, False, 9, 3.0),
]


def case_edges(n, m, seed, skew):
    """m directed edge lines over n vertices, endpoints ~ floor(n * U^skew) (skew 1 = uniform), self-loops and
    duplicates left in as an edge-list file may have them."""
    rng = np.random.default_rng(seed)
    u = np.minimum((n * rng.random(m) ** skew).astype(np.int64), n - 1)
    v = np.minimum((n * rng.random(m) ** skew).astype(np.int64), n - 1)
    relabel = rng.permutation(n)
    return relabel[u].astype(np.int32), relabel[v].astype(np.int32)


def main():
    out = {}
    for name, n, m, parts, keep, seed, skew in CASES:
        u, v = case_edges(n, m, seed, skew)
        with tempfile.TemporaryDirectory() as tmp:
            files = oracle.reference_ebv_partition(n, u, v, parts, keep, tmp)
        out[name + "/u"], out[name + "/v"] = u, v
        out[name + "/meta"] = np.array([n, parts, int(keep)], np.int64)
        for fname, data in files.items():
            out[name + "/" + fname] = np.frombuffer(data, np.uint8)
        sizes = [files["G.%d" % p].count(b"\n") for p in range(parts)]
        print(name, "edges per part", sizes)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ebv_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()

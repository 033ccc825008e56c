"""Pure-Python restatement of the reference's EBV partitioner for small graphs.

TEST INFRASTRUCTURE ONLY.  Simulates the P MPI ranks of EBV_mpi.cpp in one process:
round-robin deal (EBV_mpi.cpp:212-253), per-rank sort by local degree sum (:259-265),
lock-step batches of 10, 13, ... 1000 edges per rank scored against the state at the start
of the batch (:273-331, first-maximum rule :50-61), hand-over in sender order (:334-370),
master = replica number (id mod #replicas) in ascending part order (:567-581).
The reference sorts with std::sort (order of equal keys unspecified); this restatement and
the C++ partitioner's default both use a stable sort.

Pinned against the reference's own partitioner, compiled from EBV_mpi.cpp over stand-ins for
its MPI and gflags calls (oracle/ref_shim/ebv, `make -C oracle ref_ebv`) and run as P ranks:
tests/golden/ebv_golden.npz holds the files it wrote.  Where no rank has more than 16 edges
(std::sort keeps input order there) this restatement reproduces them exactly; on larger
inputs it reproduces them edge for edge, owners and replica counts included, when it orders
the shares with std::sort too (std_sort_ties, through oracle/std_sort_order.cpp), and so does
the C++ partitioner, byte for byte (tests/test_partition.py).
"""


def _std_sort(share, deg):
    """share ordered as std::sort orders the reference's records (oracle/std_sort_order.cpp)."""
    import ctypes
    import os
    import numpy as np
    lib = ctypes.CDLL(os.path.join(os.path.dirname(os.path.abspath(__file__)), "_build", "libebv_std_sort.so"))
    u = np.array([e[0] for e in share], np.int32)
    v = np.array([e[1] for e in share], np.int32)
    key = np.array([deg[e[0]] + deg[e[1]] for e in share], np.int32)
    ptr = ctypes.POINTER(ctypes.c_int)
    lib.ebv_std_sort(u.ctypes.data_as(ptr), v.ctypes.data_as(ptr), key.ctypes.data_as(ptr), ctypes.c_long(len(share)))
    return list(zip(u.tolist(), v.tolist()))


def ebv_partition(n_vertices, edges, n_parts, keep_self_loops=True, std_sort_ties=False):
    """std_sort_ties: order every rank's share with std::sort itself (what the reference's binary does) instead of
    the stable sort; the parts then equal the reference's edge for edge."""
    P = n_parts
    share = [[] for _ in range(P)]
    for i, (u, v) in enumerate(edges):
        if not keep_self_loops and u == v:
            continue
        share[i % P].append((u, v))
    for r in range(P):
        deg = {}
        for u, v in share[r]:
            deg[u] = deg.get(u, 0) + 1
            deg[v] = deg.get(v, 0) + 1
        if std_sort_ties:
            share[r] = _std_sort(share[r], deg)
        else:
            share[r] = sorted(share[r], key=lambda e: deg[e[0]] + deg[e[1]])   # stable
    has = [set() for _ in range(P)]
    edge_count = [0] * P
    vertex_count = [0] * P
    parts = [[] for _ in range(P)]
    longest = max(len(s) for s in share) if share else 0
    start, batch = 0, 10
    while start < longest:
        sent = {}
        for r in range(P):
            edges_r = len(share[r])
            for (u, v) in share[r][start:start + batch]:
                best, best_w = -1, -100.0
                for p in range(P):
                    w = 0.0
                    if u not in has[p]:
                        w -= 1
                    if v not in has[p]:
                        w -= 1
                    w = w - 1.0 * edge_count[p] / edges_r - 1.0 * vertex_count[p] / n_vertices * P
                    if p == r:
                        w += 0.1
                    if best_w < w:
                        best_w, best = w, p
                sent.setdefault((r, best), []).append((u, v))
        for p in range(P):
            for r in range(P):
                for (u, v) in sent.get((r, p), []):
                    parts[p].append((u, v))
                    for x in (u, v):
                        if x not in has[p]:
                            has[p].add(x)
                            vertex_count[p] += 1
                    edge_count[p] += 1
        start += batch
        if batch < 1000:
            batch = min(int(batch * 1.3), 1000)
    owner = [-1] * n_vertices
    replicas = [0] * n_vertices
    for x in range(n_vertices):
        reps = [p for p in range(P) if x in has[p]]
        replicas[x] = len(reps)
        if reps:
            owner[x] = reps[x % len(reps)] if len(reps) > 1 else reps[0]
    return parts, owner, replicas

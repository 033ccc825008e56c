"""Seeded synthetic graphs in the shapes the reference's tooling is built around
(R-MAT, and power-law graphs with the vertex/edge counts hard-wired in
cuda_gcn/src/tools/graphTransfer.cpp:15-18).  The real datasets are not used.

Edge lists are torch int32 tensors on the requested device; canonicalisation
(self-loop / duplicate removal, symmetrisation, CSR by source) is device-agnostic
torch code so the same functions serve CPU tests and GPU benchmarks.
"""
import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import check

RMAT_ABC = (0.57, 0.19, 0.19)


def rmat_edges(scale, n_edges, seed, device="cpu", abc=RMAT_ABC, first_edge=0):
    """Raw R-MAT edge list (u, v): self-loops and duplicates still present."""
    device = torch.device(device)
    a, b, c = abc
    u = torch.empty(n_edges, dtype=torch.int32, device=device)
    v = torch.empty(n_edges, dtype=torch.int32, device=device)
    if device.type == "cuda":
        with torch.cuda.device(device):
            check(_lib.lib().drone_rmat_edges(scale, n_edges, seed, a, b, c, first_edge, C.c_void_p(u.data_ptr()),
                                              C.c_void_p(v.data_ptr()),
                                              C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    else:
        check(_lib.lib().drone_rmat_edges_host(scale, n_edges, seed, a, b, c, first_edge,
                                               C.c_void_p(u.data_ptr()), C.c_void_p(v.data_ptr())))
    return u, v


def canonical_edges(u, v, n_vertices, symmetrise=False, self_loops="drop"):
    """Sorted, duplicate-free directed edge list.
    self_loops: "drop" removes u==v, "add" makes every vertex carry exactly one, "keep" leaves them."""
    u = u.to(torch.int64)
    v = v.to(torch.int64)
    if symmetrise:
        u, v = torch.cat([u, v]), torch.cat([v, u])
    if self_loops in ("drop", "add"):
        keep = u != v
        u, v = u[keep], v[keep]
    key = torch.unique(u * n_vertices + v)  # sorted ascending: by source, then destination
    if self_loops == "add":
        loops = torch.arange(n_vertices, dtype=torch.int64, device=key.device) * (n_vertices + 1)
        key = torch.sort(torch.cat([key, loops]))[0]
    u = torch.div(key, n_vertices, rounding_mode="floor")
    v = key - u * n_vertices
    return u.to(torch.int32), v.to(torch.int32)


def csr_by_source(u, v, n_vertices):
    """(index[n+1], dst[nnz]) int32 for an edge list sorted by source."""
    counts = torch.bincount(u.to(torch.int64), minlength=n_vertices)
    index = torch.zeros(n_vertices + 1, dtype=torch.int64, device=u.device)
    index[1:] = torch.cumsum(counts, 0)
    return index.to(torch.int32), v.contiguous()


def degrees(u, v, n_vertices):
    """(in_degree, out_degree) int32 of a directed edge list."""
    out_deg = torch.bincount(u.to(torch.int64), minlength=n_vertices).to(torch.int32)
    in_deg = torch.bincount(v.to(torch.int64), minlength=n_vertices).to(torch.int32)
    return in_deg, out_deg


def rmat_graph(scale, edge_factor=16, seed=1, device="cpu", symmetrise=False, self_loops="drop", abc=RMAT_ABC):
    """R-MAT graph as a canonical directed edge list.  Returns (n_vertices, u, v)."""
    n = 1 << scale
    u, v = rmat_edges(scale, edge_factor * n, seed, device=device, abc=abc)
    u, v = canonical_edges(u, v, n, symmetrise=symmetrise, self_loops=self_loops)
    return n, u, v


def powerlaw_graph(n_vertices, n_undirected, seed=1, device="cpu", exponent=0.4, offset=100.0, self_loops="add"):
    """Chung-Lu style graph with Zipf-like expected degrees w_i ~ (i+offset)^-exponent on randomly
    relabelled vertices, symmetrised.  n_undirected pairs are drawn; duplicates collapse."""
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    w = (torch.arange(n_vertices, dtype=torch.float64, device=device) + offset) ** (-exponent)
    cdf = torch.cumsum(w, 0)
    cdf = cdf / cdf[-1]
    perm = torch.randperm(n_vertices, generator=gen, device=device)
    ends = []
    for _ in range(2):
        r = torch.rand(n_undirected, dtype=torch.float64, generator=gen, device=device)
        idx = torch.searchsorted(cdf, r).clamp_(max=n_vertices - 1)
        ends.append(perm[idx])
    u, v = canonical_edges(ends[0], ends[1], n_vertices, symmetrise=True, self_loops=self_loops)
    return n_vertices, u, v


def tiny_graphs():
    """Hand-made graphs for known-answer tests: name -> (n_vertices, u, v) numpy int32 arrays (directed)."""
    g = {}
    g["path5"] = (5, np.array([0, 1, 2, 3], np.int32), np.array([1, 2, 3, 4], np.int32))
    g["star6"] = (6, np.array([0, 0, 0, 0, 0], np.int32), np.array([1, 2, 3, 4, 5], np.int32))
    cu, cv = np.nonzero(1 - np.eye(4, dtype=np.int32))
    g["clique4"] = (4, cu.astype(np.int32), cv.astype(np.int32))
    # six vertices, five edges, with a dangling vertex and an unreferenced id
    g["six_five"] = (6, np.array([0, 0, 1, 2, 4], np.int32), np.array([1, 2, 2, 0, 0], np.int32))
    return g


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15)).astype(np.uint64)
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def seeded_normal(seed, shape):
    """i.i.d. N(0,1) float32 array that depends only on (seed, position): counter-based
    splitmix64 + Box-Muller, so fixtures can be regenerated anywhere without storing inputs."""
    n = int(np.prod(shape))
    with np.errstate(over="ignore"):
        ctr = np.arange(n, dtype=np.uint64) * np.uint64(2) + np.uint64(seed) * np.uint64(0xD1342543DE82EF95)
        h1 = _splitmix64(ctr)
        h2 = _splitmix64(ctr + np.uint64(1))
    u1 = ((h1 >> np.uint64(11)).astype(np.float64) + 1.0) / 9007199254740993.0   # (0, 1)
    u2 = (h2 >> np.uint64(11)).astype(np.float64) / 9007199254740992.0           # [0, 1)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return z.astype(np.float32).reshape(shape)


def glorot_weights(dims, device, seed=7):
    """(U - 0.5) * 2 * sqrt(6 / (in + out)) per layer (cuda_gcn/src/cuda/cuda_kernel.cu:469-474), same on every rank."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    return [((torch.rand((a, b), generator=gen) - 0.5) * 2 * (6.0 / (a + b)) ** 0.5).to(device)
            for a, b in zip(dims[:-1], dims[1:])]


def hashed_normal(global_ids, f, seed, device):
    """N(0,1) features that depend only on (seed, global vertex id, column): every rank that holds a vertex makes the
    same row.  Counter hash (splitmix64 on int64, wrapping) + Box-Muller, on the device."""
    ids = torch.as_tensor(np.asarray(global_ids).astype(np.int64), device=device)
    ctr = (ids[:, None] * f + torch.arange(f, device=device, dtype=torch.int64)[None, :]) * 2 + seed * 0x5851F42D

    def mix(x):
        x = x + (-7046029254386353131)              # 0x9E3779B97F4A7C15 as a signed 64-bit value
        x = (x ^ ((x >> 30) & 0x3FFFFFFFF)) * (-4658895280553007687)
        x = (x ^ ((x >> 27) & 0x1FFFFFFFFF)) * (-7723592293110705685)
        return x ^ ((x >> 31) & 0x1FFFFFFFF)
    u1 = ((mix(ctr) >> 11) & 0x1FFFFFFFFFFFFF).double() / 9007199254740992.0
    u2 = ((mix(ctr + 1) >> 11) & 0x1FFFFFFFFFFFFF).double() / 9007199254740992.0
    z = torch.sqrt(-2.0 * torch.log(u1.clamp_(min=1e-300))) * torch.cos(2.0 * np.pi * u2)
    return z.float()


def hashed_labels(global_ids, classes, seed, device):
    ids = torch.as_tensor(np.asarray(global_ids).astype(np.int64), device=device)
    h = (ids * 2654435761 + seed * 40503) & 0x7FFFFFFF
    return (h % classes).to(torch.int32)

"""EBV partitions in the reference's layout: per part an edge list (G.<p>), the master rows
(Master.<p>: vertex, ranks holding its mirrors) and the mirror rows (Mirror.<p>: vertex, rank
of its master), plus the per-rank local graph and routing tables built from them.

Everything here is host-side numpy over the C ABI; nothing needs a GPU.
"""
import ctypes as C
import os

import numpy as np

from . import _lib
from ._lib import check


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _vp(a):
    return C.c_void_p(a.ctypes.data) if a is not None and a.size else C.c_void_p(0)


class Partition:
    """Result of the EBV vertex cut of a directed edge list over n_parts parts."""

    def __init__(self, n_vertices, n_parts, part_u, part_v, owner, replicas, present_bits=None):
        self.n_vertices = n_vertices
        self.n_parts = n_parts
        self.part_u = part_u            # list of int32 arrays (global ids), G.<p> order
        self.part_v = part_v
        self.owner = owner              # [V] part holding the master copy (-1: vertex has no edge)
        self.replicas = replicas        # [V] number of parts holding the vertex
        self._present = None
        # [V] uint64, bit p set when part p holds the vertex.  A rank that was sent only its own edges (part_u / part_v
        # of the other parts are None) is given this table instead, which is all the routing tables need of them.
        self.present_bits = present_bits
        self._flat = None               # (u, v) of all parts in one array each, when the parts are views of them

    # ----- statistics the reference prints (EBV_mpi.cpp:379-401) -----
    def replication_factor(self):
        return float(self.replicas.sum()) / self.n_vertices

    def edge_imbalance(self):
        sizes = np.array([len(u) for u in self.part_u], dtype=np.float64)
        return float(sizes.max() * self.n_parts / max(sizes.sum(), 1))

    def presence_bits(self):
        """[V] uint64 with bit p set when part p holds the vertex."""
        if self.present_bits is None:
            u = np.ascontiguousarray(np.concatenate(self.part_u), np.int32) if self._flat is None else self._flat[0]
            v = np.ascontiguousarray(np.concatenate(self.part_v), np.int32) if self._flat is None else self._flat[1]
            off = np.concatenate([[0], np.cumsum([len(x) for x in self.part_u])]).astype(np.int64)
            bits = np.empty(self.n_vertices, np.uint64)
            check(_lib.lib().drone_presence_bits_host(self.n_vertices, self.n_parts, _vp(u), _vp(v), _vp(off), _vp(bits)))
            self.present_bits = bits
        return self.present_bits

    def present(self, p):
        if self.present_bits is not None:
            return (self.present_bits >> np.uint64(p)) & np.uint64(1) != 0
        if self._present is None:
            self._present = []
            for q in range(self.n_parts):
                m = np.zeros(self.n_vertices, dtype=bool)
                m[self.part_u[q]] = True
                m[self.part_v[q]] = True
                self._present.append(m)
        return self._present[p]

    def master_rows(self, p):
        """(master_vertex, mirror_number, mirror_workers): the content of Master.<p>."""
        mine = np.nonzero((self.owner == p) & (self.replicas > 1))[0].astype(np.int32)
        holders = np.stack([self.present(q)[mine] for q in range(self.n_parts)], axis=1) if len(mine) else \
            np.zeros((0, self.n_parts), bool)
        holders[:, p] = False
        number = holders.sum(axis=1).astype(np.int32)
        workers = np.nonzero(holders)[1].astype(np.int32)    # row-major: per vertex, ascending rank
        return mine, number, workers

    def mirror_rows(self, p):
        """(mirror_vertex, master_worker): the content of Mirror.<p>."""
        mine = np.nonzero(self.present(p) & (self.replicas > 1) & (self.owner != p))[0].astype(np.int32)
        return mine, self.owner[mine].astype(np.int32)

    def _file_order(self, vertices):
        """Line order of Master.<p> / Mirror.<p>: the reference walks the vertices in blocks of 1000 * n_parts ids and,
        inside a block, takes those with id mod n_parts = 0 first, then 1, ... (EBV_mpi.cpp:551-559,598-604)."""
        v = vertices.astype(np.int64)
        return np.lexsort((v, v % self.n_parts, v // (1000 * self.n_parts)))

    def write_files(self, directory):
        """G.<p>, Master.<p>, Mirror.<p> in the reference's text formats and line order (EBV_mpi.cpp:342,551-634)."""
        os.makedirs(directory, exist_ok=True)
        for p in range(self.n_parts):
            np.savetxt(os.path.join(directory, "G.%d" % p), np.stack([self.part_u[p], self.part_v[p]], 1), fmt="%d")
            mv, num, wk = self.master_rows(p)
            start = np.concatenate([[0], np.cumsum(num)]).tolist()
            mv, num = mv.tolist(), num.tolist()
            with open(os.path.join(directory, "Master.%d" % p), "w") as f:
                for i in self._file_order(np.asarray(mv, np.int64)).tolist():
                    f.write("%d %s \n" % (mv[i], " ".join(str(w) for w in wk[start[i]:start[i] + num[i]].tolist())))
            mr, ow = self.mirror_rows(p)
            mr, ow = mr.tolist(), ow.tolist()
            with open(os.path.join(directory, "Mirror.%d" % p), "w") as f:
                for i in self._file_order(np.asarray(mr, np.int64)).tolist():
                    f.write("%d %d \n" % (mr[i], ow[i]))

    def local_graph(self, p):
        return LocalGraph(self, p)


def read_text_ints(path, with_lines=False):
    """All integers of a text file (int32, file order); with_lines also returns the index of the first value of every
    line that holds one, closed by the total.  Parsed by the library with all host threads."""
    lib = _lib.lib()
    nv, nl = C.c_longlong(0), C.c_longlong(0)
    bpath = os.fsencode(path)
    size = os.path.getsize(path) if os.path.exists(path) else 0     # a missing file is the library's error to report
    cap = size // 2 + 1                           # an integer takes at least a digit and a separator
    values = np.empty(cap, np.int32)              # untouched pages cost nothing
    lines = np.empty(cap + 1, np.int64) if with_lines else None
    check(lib.drone_text_ints_read(bpath, _vp(values), cap, _vp(lines) if with_lines else None, cap,
                                   C.byref(nv), C.byref(nl)))
    values = values[:nv.value]
    return (values, lines[:nl.value + 1]) if with_lines else values


def read_edge_list(path):
    """(u, v) of a "u v" per line file such as G.<p>."""
    size = os.path.getsize(path) if os.path.exists(path) else 0
    cap = size // 4 + 1                           # an edge takes at least two digits and two separators
    u, v = np.empty(cap, np.int32), np.empty(cap, np.int32)
    n = C.c_longlong(0)
    try:
        check(_lib.lib().drone_text_edges_read(os.fsencode(path), _vp(u), _vp(v), cap, C.byref(n)))
    except _lib.DroneError as e:
        if "odd number" in str(e):
            raise ValueError(str(e))
        raise
    return u[:n.value], v[:n.value]


def read_partition_files(directory, n_vertices, n_parts):
    """Parse G./Master./Mirror. files (as cuda_gcn/src/common/parser.cu:59-131 does) back into a Partition."""
    part_u, part_v = [], []
    owner = np.full(n_vertices, -1, np.int32)
    replicas = np.zeros(n_vertices, np.int32)
    for p in range(n_parts):
        pu, pv = read_edge_list(os.path.join(directory, "G.%d" % p))
        part_u.append(pu)
        part_v.append(pv)
        seen = np.zeros(n_vertices, bool)
        seen[pu] = True
        seen[pv] = True
        replicas += seen
        owner[seen & (owner < 0)] = p                 # single-replica vertices: the part that has them
    for p in range(n_parts):
        values, lines = read_text_ints(os.path.join(directory, "Master.%d" % p), with_lines=True)
        owner[values[lines[:-1]]] = p                 # first integer of every line: a master vertex of part p
    return Partition(n_vertices, n_parts, part_u, part_v, owner, replicas)


def save_partition(part, path):
    """The whole partition in the library's binary format (drone_partition_write)."""
    off = np.concatenate([[0], np.cumsum([len(x) for x in part.part_u])]).astype(np.int64)
    if part._flat is not None:
        u, v = part._flat
    else:
        u = _i32(np.concatenate(part.part_u)) if off[-1] else np.zeros(1, np.int32)
        v = _i32(np.concatenate(part.part_v)) if off[-1] else np.zeros(1, np.int32)
    check(_lib.lib().drone_partition_write(os.fsencode(path), part.n_vertices, part.n_parts, _vp(off), _vp(u), _vp(v),
                                           _vp(_i32(part.owner)), _vp(_i32(part.replicas)), _vp(part.presence_bits())))


def load_partition(path, part=None):
    """A Partition from the binary format.  part = p reads the edges of part p only (the other parts' edge lists are
    None; the presence words stand in for them), which is what one rank of a job needs."""
    lib = _lib.lib()
    nv, npart = C.c_int(0), C.c_int(0)
    off = np.zeros(65, np.int64)
    bpath = os.fsencode(path)
    check(lib.drone_partition_read_header(bpath, C.byref(nv), C.byref(npart), _vp(off)))
    n, P = nv.value, npart.value
    off = off[:P + 1]
    if part is not None and not 0 <= part < P:
        raise _lib.DroneError(-1, "load_partition: part %d of %d" % (part, P))
    e0, e1 = (0, int(off[P])) if part is None else (int(off[part]), int(off[part + 1]))
    u = np.empty(max(e1 - e0, 1), np.int32)
    v = np.empty(max(e1 - e0, 1), np.int32)
    owner, replicas, bits = np.empty(n, np.int32), np.empty(n, np.int32), np.empty(n, np.uint64)
    check(lib.drone_partition_read(bpath, -1 if part is None else int(part), _vp(u), _vp(v), _vp(owner), _vp(replicas),
                                   _vp(bits)))
    if part is None:
        pu = [u[off[p]:off[p + 1]] for p in range(P)]
        pv = [v[off[p]:off[p + 1]] for p in range(P)]
        out = Partition(n, P, pu, pv, owner, replicas, present_bits=bits)
        out._flat = (u, v)
        return out
    pu, pv = [None] * P, [None] * P
    pu[part], pv[part] = u[:e1 - e0], v[:e1 - e0]
    return Partition(n, P, pu, pv, owner, replicas, present_bits=bits)


EBV_KEEP_SELF_LOOPS, EBV_STD_SORT_TIES = 1, 2


def ebv_partition(n_vertices, u, v, n_parts, keep_self_loops=True, std_sort_ties=False):
    """EBV vertex cut (restating EBV_mpi.cpp; see drone_ebv_partition in include/drone_b200.h).
    std_sort_ties: order edges of equal degree sum as std::sort leaves them, which is what the reference's binary
    does (EBV_mpi.cpp:265); the default stable order does not depend on the C++ library."""
    flags = (EBV_KEEP_SELF_LOOPS if keep_self_loops else 0) | (EBV_STD_SORT_TIES if std_sort_ties else 0)
    u, v = _i32(u), _i32(v)
    e = len(u)
    out_u = np.empty(max(e, 1), np.int32)
    out_v = np.empty(max(e, 1), np.int32)
    off = np.zeros(n_parts + 1, np.int64)
    owner = np.empty(n_vertices, np.int32)
    replicas = np.empty(n_vertices, np.int32)
    check(_lib.lib().drone_ebv_partition(n_vertices, e, _vp(u), _vp(v), n_parts, flags,
                                         _vp(out_u), _vp(out_v), _vp(off), _vp(owner), _vp(replicas)))
    part_u = [out_u[off[p]:off[p + 1]] for p in range(n_parts)]     # views: no second copy of the edge list
    part_v = [out_v[off[p]:off[p + 1]] for p in range(n_parts)]
    part = Partition(n_vertices, n_parts, part_u, part_v, owner, replicas)
    part._flat = (out_u, out_v)
    return part


class LocalGraph:
    """One rank's view: local numbering, CSR by source, routing tables (host numpy arrays) —
    the content of struct Graph (cuda_gcn/src/cuda/graph.h:17-41) before it is copied to the device."""

    def __init__(self, part, p):
        lib = _lib.lib()
        self.rank, self.n_parts, self.global_v = p, part.n_parts, part.n_vertices
        u, v = part.part_u[p], part.part_v[p]
        e = len(u)
        cap = min(part.n_vertices, 2 * e) + 1
        g2l = np.empty(part.n_vertices, np.int32)
        l2g = np.empty(cap, np.int32)
        index = np.empty(cap + 1, np.int32)
        dst = np.empty(max(e, 1), np.int32)
        n = C.c_int(0)
        check(lib.drone_graph_build_host(part.n_vertices, e, _vp(u), _vp(v), _vp(g2l), _vp(l2g), _vp(index), _vp(dst),
                                         C.byref(n)))
        self.n_local = n.value
        self.g2l = g2l
        self.l2g = l2g[:self.n_local].copy()
        self.index = index[:self.n_local + 1].copy()
        self.dst = dst[:e].copy()
        mv, num, wk = part.master_rows(p)
        mr, ow = part.mirror_rows(p)
        self.master_size, self.mirror_worker_size, self.mirror_size = len(mv), len(wk), len(mr)
        self.master_worker_index = np.empty(self.n_local + 1, np.int32)
        self.master2workers = np.empty(max(len(wk), 1), np.int32)
        self.mirror2worker = np.empty(max(self.n_local, 1), np.int32)
        check(lib.drone_route_tables_host(self.n_local, _vp(g2l), _vp(mv), _vp(num), _vp(wk), len(mv), len(wk),
                                          _vp(mr), _vp(ow), len(mr), _vp(self.master_worker_index),
                                          _vp(self.master2workers), _vp(self.mirror2worker)))
        self.master2workers = self.master2workers[:len(wk)]
        self.mirror2worker = self.mirror2worker[:self.n_local]

    def local_degrees(self, global_in_degree, global_out_degree):
        """Global degrees indexed by local id (setDegree, cuda_gcn/src/common/parser.cu:25-35)."""
        return _i32(global_in_degree[self.l2g]), _i32(global_out_degree[self.l2g])


def scatter_partition(part, n_vertices, n_parts, device, extra=(), n_extra=0):
    """Hand a partition that rank 0 holds to the ranks of the default torch.distributed group (any backend; tensors
    travel on `device`).  Rank 0 passes the Partition and `extra`, a list of int32 arrays of n_vertices entries that
    everybody needs (degrees); the others pass part=None and the number of such arrays.  Every rank p gets back
    (partition, extras, total_edges): its own edges, the owner / replica tables and one presence word per vertex --
    what LocalGraph and the exchange plans need of the other parts -- and the extra arrays as numpy.  Rank 0 keeps
    its full partition."""
    import torch
    import torch.distributed as dist
    rank = dist.get_rank()
    meta = torch.zeros(n_parts + 1, dtype=torch.int64, device=device)
    if rank == 0:
        sizes = [len(x) for x in part.part_u]
        meta[:] = torch.as_tensor(np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64))
        extra = [np.ascontiguousarray(a, dtype=np.int32) for a in extra]
        n_extra = len(extra)
    dist.broadcast(meta, 0)
    offs = meta.cpu().numpy()
    if rank == 0:
        tables = [torch.as_tensor(_i32(part.owner), device=device), torch.as_tensor(_i32(part.replicas), device=device),
                  torch.as_tensor(part.presence_bits().view(np.int64), device=device)]
        tables += [torch.as_tensor(a, device=device) for a in extra]
    else:
        tables = [torch.empty(n_vertices, dtype=torch.int32, device=device),
                  torch.empty(n_vertices, dtype=torch.int32, device=device),
                  torch.empty(n_vertices, dtype=torch.int64, device=device)]
        tables += [torch.empty(n_vertices, dtype=torch.int32, device=device) for _ in range(n_extra)]
    for t in tables:
        dist.broadcast(t, 0)
    extras = [t.cpu().numpy() for t in tables[3:]]
    if rank == 0:
        for p in range(1, n_parts):
            for arr in (part.part_u[p], part.part_v[p]):
                dist.send(torch.as_tensor(np.ascontiguousarray(arr, dtype=np.int32), device=device), dst=p)
        mine = part
    else:
        got = []
        for _ in range(2):
            t = torch.empty(int(offs[rank + 1] - offs[rank]), dtype=torch.int32, device=device)
            dist.recv(t, src=0)
            got.append(t.cpu().numpy())
        pu, pv = [None] * n_parts, [None] * n_parts
        pu[rank], pv[rank] = got
        mine = Partition(n_vertices, n_parts, pu, pv, tables[0].cpu().numpy(), tables[1].cpu().numpy(),
                         present_bits=tables[2].cpu().numpy().view(np.uint64))
    return mine, extras, int(offs[n_parts])


def device_local_graph(u, v, global_v, stream=None):
    """Local numbering and CSR by source of one part from its edge list on the device (int32 CUDA tensors).
    Returns (n_local, g2l, l2g, index, dst) as CUDA tensors; identical to what LocalGraph builds on the host."""
    import torch
    from .plan import _stream_ptr
    if not (u.is_cuda and v.is_cuda and u.dtype == torch.int32 and v.dtype == torch.int32 and u.is_contiguous() and
            v.is_contiguous() and u.numel() == v.numel()):
        raise ValueError("u and v must be contiguous int32 CUDA tensors of one length")
    e = u.numel()
    cap = min(int(global_v), 2 * e) + 1
    dev = u.device
    g2l = torch.empty(int(global_v), dtype=torch.int32, device=dev)
    l2g = torch.empty(cap, dtype=torch.int32, device=dev)
    index = torch.empty(cap + 1, dtype=torch.int32, device=dev)
    dst = torch.empty(max(e, 1), dtype=torch.int32, device=dev)
    n = C.c_int(0)
    with torch.cuda.device(dev):
        check(_lib.lib().drone_graph_build_device(int(global_v), e, C.c_void_p(u.data_ptr()), C.c_void_p(v.data_ptr()),
                                                  C.c_void_p(g2l.data_ptr()), C.c_void_p(l2g.data_ptr()),
                                                  C.c_void_p(index.data_ptr()), C.c_void_p(dst.data_ptr()), C.byref(n),
                                                  _stream_ptr(stream)))
    return n.value, g2l, l2g[:n.value], index[:n.value + 1], dst[:e]


class ExchangePlan:
    """Static routing plan of one rank (drone_xplan)."""

    def __init__(self, local_graph, max_features, row_mask=None):
        """row_mask ([n_local] bool): plan the exchange of those rows only (every rank must select the same
        vertices, e.g. by a function of the global id)."""
        g = local_graph
        self.rank, self.n_parts, self.n_local = g.rank, g.n_parts, g.n_local
        m2w, mwi, workers = g.mirror2worker, g.master_worker_index, g.master2workers
        if row_mask is not None:
            row_mask = np.asarray(row_mask, bool)[:g.n_local]
            m2w = _i32(np.where(row_mask, m2w[:g.n_local], -1))
            per_row = np.diff(mwi[:g.n_local + 1])
            workers = _i32(workers[np.repeat(row_mask, per_row)])
            mwi = _i32(np.concatenate([[0], np.cumsum(np.where(row_mask, per_row, 0))]))
        self._keep = (g, m2w, mwi, workers)
        self.max_features = int(max_features)
        self.p2p_enabled = False
        self._h = C.c_void_p(0)
        check(_lib.lib().drone_xplan_create(C.byref(self._h), g.rank, g.n_parts, g.n_local, _vp(g.l2g),
                                            _vp(m2w), _vp(mwi), _vp(workers), int(max_features)))

    @property
    def handle(self):
        return self._h

    def counts(self):
        up = np.zeros(self.n_parts, np.int32)
        down = np.zeros(self.n_parts, np.int32)
        nm = C.c_int(0)
        check(_lib.lib().drone_xplan_counts(self._h, _vp(up), _vp(down), C.byref(nm)))
        return up, down, nm.value

    def lists(self):
        up, down, _ = self.counts()
        ur = np.empty(max(int(up.sum()), 1), np.int32)
        dr = np.empty(max(int(down.sum()), 1), np.int32)
        check(_lib.lib().drone_xplan_lists(self._h, _vp(ur), _vp(dr)))
        return ur[:int(up.sum())], dr[:int(down.sum())]

    def enable_p2p(self, comm, stream_ptr=None):
        """Switch later exchanges on this plan to the peer-memory transport (collective over `comm`)."""
        check(_lib.lib().drone_xplan_enable_p2p(self._h, comm.handle, C.c_void_p(stream_ptr or 0)))
        self.p2p_enabled = comm.nranks > 1

    def close(self):
        if self._h.value:
            _lib.lib().drone_xplan_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DenseExchangePlan:
    """Boundary-dense plan of one rank for the reduce-scatter / all-gather form of the exchange."""

    def __init__(self, part, local_graph, max_features):
        self._h = C.c_void_p(0)
        owner, reps = _i32(part.owner), _i32(part.replicas)
        check(_lib.lib().drone_dense_xplan_create(C.byref(self._h), local_graph.rank, part.n_parts, local_graph.n_local,
                                                  _vp(local_graph.l2g), part.n_vertices, _vp(owner), _vp(reps),
                                                  int(max_features)))

    @property
    def handle(self):
        return self._h

    def boundary_rows(self):
        return int(_lib.lib().drone_dense_xplan_boundary_rows(self._h))

    def close(self):
        if self._h.value:
            _lib.lib().drone_dense_xplan_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

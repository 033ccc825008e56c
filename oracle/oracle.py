"""numpy-facing wrappers of the CPU oracle (oracle/drone_oracle.c, oracle/pagerank_oracle.c, oracle/minprop_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline / reference legs of bench.py; never by the drone_b200 package.
Parity status is stated in the headers of the C files.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libdrone_oracle.so")


def build(force=False):
    """Compile the oracle with the committed Makefile (gcc, a few seconds)."""
    srcs = [os.path.join(_HERE, f) for f in ("drone_oracle.c", "pagerank_oracle.c", "minprop_oracle.c",
                                             "std_sort_order.cpp", "Makefile")]
    sort_so = os.path.join(_HERE, "_build", "libebv_std_sort.so")
    if force or not os.path.exists(_SO) or not os.path.exists(sort_so) or \
            any(os.path.getmtime(s) > min(os.path.getmtime(_SO), os.path.getmtime(sort_so)) for s in srcs):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


_REF_SO = os.path.join(_HERE, "_ref", "libref_graphsum.so")
# the reference checkout: DRONE_REFERENCE_ROOT, else the directory `reference` beside this repository
REFERENCE_ROOT = os.environ.get("DRONE_REFERENCE_ROOT",
                                os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference"))


def build_ref(force=False):
    """Compile the reference's own GraphSum layer from its sources where they lie (`make ref`), into oracle/_ref/.
    Returns the library path, or None when the reference tree is not on this machine."""
    if not os.path.isdir(os.path.join(REFERENCE_ROOT, "cuda_gcn", "src")):
        return _REF_SO if os.path.exists(_REF_SO) else None
    deps = [os.path.join(_HERE, f) for f in ("ref_driver.cu", "Makefile", "ref_shim/mpi.h", "ref_shim/utils_override.h")]
    built = [_REF_SO] + [os.path.join(_HERE, "_ref", f) for f in ("libref_drone_jobs.so", "ebv_mpi", "ebv_mpi_keep_loops")]
    if force or not all(os.path.exists(b) for b in built) \
            or any(os.path.getmtime(d) > os.path.getmtime(_REF_SO) for d in deps):
        subprocess.run(["make", "-C", _HERE, "ref", "REFERENCE=" + REFERENCE_ROOT] + (["-B"] if force else []),
                       check=True, stdout=subprocess.DEVNULL)
    return _REF_SO


def reference_gcn_epochs(global_v, u, v, global_in_degree, global_out_degree, dims, features, labels, w1, w2,
                         warmup=2, epochs=5):
    """Run the REFERENCE's own training epoch (CUDAGCN::train_epoch, cuda_gcn/src/cuda/cuda_gcn.cu:287-306) on one
    worker on cuda:0, over the given graph / features / labels (by global id) and starting weights.  Returns
    (ms per epoch, ms per epoch of its bookkeeping steps timed on their own, cross-entropy loss of the first epoch)."""
    ref = C.CDLL(_REF_SO)
    u, v = _i32(u), _i32(v)
    ind, outd = _i32(global_in_degree), _i32(global_out_degree)
    features, w1, w2, labels = _f32(features), _f32(w1), _f32(w2), _i32(labels)
    ms, book, loss = C.c_double(0), C.c_double(0), C.c_float(0)
    rc = ref.ref_gcn_epochs(int(global_v), len(u), _p(u, C.c_int), _p(v, C.c_int), _p(ind, C.c_int), _p(outd, C.c_int),
                            int(dims[0]), int(dims[1]), int(dims[2]), _p(features, C.c_float), _p(labels, C.c_int),
                            _p(w1, C.c_float), _p(w2, C.c_float), int(warmup), int(epochs), C.byref(ms), C.byref(book),
                            C.byref(loss))
    if rc != 0:
        raise RuntimeError("reference GCN epoch run failed (%d)" % rc)
    return ms.value, book.value, loss.value


def reference_ebv_binary(keep_self_loops):
    """The reference's partitioner compiled by `make ref_ebv` (EBV_mpi.cpp, or the copy under cuda_gcn/src/tools that
    keeps self-loops), or None when it was not built."""
    path = os.path.join(_HERE, "_ref", "ebv_mpi_keep_loops" if keep_self_loops else "ebv_mpi")
    return path if os.path.exists(path) else None


def reference_ebv_partition(n_vertices, u, v, n_parts, keep_self_loops, workdir):
    """Run the REFERENCE's partitioner as n_parts ranks on the edge list (written as its text input into workdir)
    and return {file name: bytes} of the G.<p> / Master.<p> / Mirror.<p> files it dumps (EBV_mpi.cpp:342,598-634)."""
    exe = reference_ebv_binary(keep_self_loops)
    if exe is None:
        raise RuntimeError("the reference's partitioner was not built (make -C oracle ref_ebv)")
    os.makedirs(workdir, exist_ok=True)
    edges = os.path.join(workdir, "edges.txt")
    np.savetxt(edges, np.stack([_i32(u), _i32(v)], 1), fmt="%d")
    out = os.path.join(workdir, "parts")
    env = dict(os.environ, EBV_STANDIN_RANKS=str(n_parts))
    subprocess.run([exe, "-filename", edges, "-vertices", str(n_vertices), "-edges", str(len(u)), "--is_dump",
                    "-output", out], check=True, env=env, stdout=subprocess.DEVNULL, timeout=300)
    files = {}
    for p in range(n_parts):
        for kind in ("G", "Master", "Mirror"):
            with open(os.path.join(out, "%s.%d" % (kind, p)), "rb") as f:
                files["%s.%d" % (kind, p)] = f.read()
    return files


def reference_available():
    return os.path.exists(_REF_SO)


_REF_JOBS_SO = os.path.join(_HERE, "_ref", "libref_drone_jobs.so")


def reference_jobs_library():
    """Path of the reference's own GPU jobs (build_graph, addMasterRoute, addMirrorRoute, loadOutDegree, PR_*, CC_*,
    SSSP_* compiled from DRONE/src/cuda by `make ref`), or None when it was not built."""
    return _REF_JOBS_SO if os.path.exists(_REF_JOBS_SO) else None


def reference_graphsum(global_v, u, v, global_in_degree, global_out_degree, x, out_grad):
    """Run the REFERENCE's CUDAGraphSum (cuSPARSE) forward and backward on one worker, on cuda:0.
    x, out_grad: [global_v, dim] float32 by global id.  Returns (l2g, out_data, in_grad, values): results by the
    reference's local id (l2g maps them to global ids), values in the reference's CSR order."""
    ref = C.CDLL(_REF_SO)
    u, v = _i32(u), _i32(v)
    ind, outd = _i32(global_in_degree), _i32(global_out_degree)
    x, out_grad = _f32(x), _f32(out_grad)
    dim = x.shape[1]
    cap = min(global_v, 2 * len(u)) + 1
    out_data = np.zeros((cap, dim), np.float32)
    in_grad = np.zeros((cap, dim), np.float32)
    values = np.zeros(max(len(u), 1), np.float32)
    l2g = np.zeros(cap, np.int32)
    n = C.c_int(0)
    rc = ref.ref_graphsum_run(int(global_v), len(u), _p(u, C.c_int), _p(v, C.c_int), _p(ind, C.c_int),
                              _p(outd, C.c_int), dim, _p(x, C.c_float), _p(out_grad, C.c_float),
                              _p(out_data, C.c_float), _p(in_grad, C.c_float), _p(values, C.c_float),
                              _p(l2g, C.c_int), C.byref(n))
    if rc != 0:
        raise RuntimeError("reference GraphSum run failed (%d)" % rc)
    n = n.value
    return l2g[:n].copy(), out_data[:n].copy(), in_grad[:n].copy(), values[:len(u)].copy()


def reference_graphsum_worker(part, rank, global_in_degree, global_out_degree, x, out_grad):
    """One worker of the REFERENCE's CUDAGraphSum over a partition (one process per GPU; all workers must call this
    at the same time, with DRONE_REF_ID_FILE / DRONE_REF_RANK set for the MPI_Bcast stand-in).  Returns
    (l2g, out_data, in_grad) by the reference's local id, after its own mirror/master exchange."""
    ref = C.CDLL(_REF_SO)
    u, v = _i32(part.part_u[rank]), _i32(part.part_v[rank])
    mv, num, wk = part.master_rows(rank)
    mr, ow = part.mirror_rows(rank)

    def arr(a):
        a = _i32(a)
        return a if a.size else np.zeros(1, np.int32)

    mv, num, wk, mr, ow = arr(mv), arr(num), arr(wk), arr(mr), arr(ow)
    sizes = [len(part.master_rows(rank)[0]), len(part.master_rows(rank)[2]), len(part.mirror_rows(rank)[0])]
    ind, outd = _i32(global_in_degree), _i32(global_out_degree)
    x, out_grad = _f32(x), _f32(out_grad)
    dim = x.shape[1]
    n_v = part.n_vertices
    cap = min(n_v, 2 * len(u)) + 1
    out_data = np.zeros((cap, dim), np.float32)
    in_grad = np.zeros((cap, dim), np.float32)
    values = np.zeros(max(len(u), 1), np.float32)
    l2g = np.zeros(cap, np.int32)
    n = C.c_int(0)
    rc = ref.ref_graphsum_run_worker(int(n_v), len(u), _p(u, C.c_int), _p(v, C.c_int), int(rank), int(part.n_parts),
                                     _p(mv, C.c_int), _p(num, C.c_int), _p(wk, C.c_int), sizes[0], sizes[1],
                                     _p(mr, C.c_int), _p(ow, C.c_int), sizes[2], _p(ind, C.c_int), _p(outd, C.c_int), dim,
                                     _p(x, C.c_float), _p(out_grad, C.c_float), _p(out_data, C.c_float),
                                     _p(in_grad, C.c_float), _p(values, C.c_float), _p(l2g, C.c_int), C.byref(n))
    if rc != 0:
        raise RuntimeError("reference GraphSum run failed (%d)" % rc)
    n = n.value
    return l2g[:n].copy(), out_data[:n].copy(), in_grad[:n].copy()


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.oracle_pr_drone_cpu.restype = C.c_int
        _lib.oracle_pr_drone_cpu_maps.restype = C.c_int
        _lib.oracle_pr_drone_cuda_f32.restype = C.c_int
        _lib.oracle_pr_drone_cuda_f64.restype = C.c_int
        _lib.oracle_build_graph.restype = C.c_int
        _lib.oracle_max_threads.restype = C.c_int
    return _lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads():
    """Host threads the timed CPU product may use: every core, whatever OMP_NUM_THREADS says
    (launchers such as torchrun pin it to 1)."""
    return max(int(os.cpu_count() or 1), int(lib().oracle_max_threads()))


def build_graph(global_v, u, v):
    """First-seen local numbering and CSR by source (cuda_gcn/src/cuda/graph.cu:54-103).
    Returns (n_local, g2l[global_v], l2g[n_local], index[n_local+1], dst[E])."""
    u, v = _i32(u), _i32(v)
    e = len(u)
    g2l = np.empty(global_v, np.int32)
    l2g = np.empty(global_v, np.int32)
    index = np.empty(global_v + 1, np.int32)
    dst = np.empty(max(e, 1), np.int32)
    n = lib().oracle_build_graph(global_v, e, _p(u, C.c_int), _p(v, C.c_int), _p(g2l, C.c_int),
                                 _p(l2g, C.c_int), _p(index, C.c_int), _p(dst, C.c_int))
    return n, g2l, l2g[:n].copy(), index[:n + 1].copy(), dst[:e].copy()


def csr_values_f32(index, dst, in_degree, out_degree):
    index, dst, in_degree, out_degree = map(_i32, (index, dst, in_degree, out_degree))
    n = len(index) - 1
    values = np.empty(max(len(dst), 1), np.float32)
    lib().oracle_csr_values_f32(_p(index, C.c_int), _p(dst, C.c_int), _p(in_degree, C.c_int),
                                _p(out_degree, C.c_int), n, _p(values, C.c_float))
    return values[:len(dst)]


def csr_values_f64(index, dst, in_degree, out_degree):
    index, dst, in_degree, out_degree = map(_i32, (index, dst, in_degree, out_degree))
    n = len(index) - 1
    values = np.empty(max(len(dst), 1), np.float64)
    lib().oracle_csr_values_f64(_p(index, C.c_int), _p(dst, C.c_int), _p(in_degree, C.c_int),
                                _p(out_degree, C.c_int), n, _p(values, C.c_double))
    return values[:len(dst)]


def graphsum_forward_f64(x, index, dst, values):
    """out[v] += coef * in[u] over edges u->v (cuda_gcn/src/cuda/cuda_kernel.cu:203-218)."""
    x = _f32(x)
    n, dim = x.shape
    index, dst, values = _i32(index), _i32(dst), _f32(values)
    out = np.empty((n, dim), np.float64)
    lib().oracle_graphsum_forward_f64(_p(x, C.c_float), _p(out, C.c_double), _p(index, C.c_int),
                                      _p(dst, C.c_int), _p(values, C.c_float), dim, n)
    return out


def graphsum_backward_f64(out_grad, index, dst, values):
    """in_grad[u] += coef * out_grad[v] over edges u->v (cuda_gcn/src/cuda/cuda_kernel.cu:236-248)."""
    out_grad = _f32(out_grad)
    n, dim = out_grad.shape
    index, dst, values = _i32(index), _i32(dst), _f32(values)
    in_grad = np.empty((n, dim), np.float64)
    lib().oracle_graphsum_backward_f64(_p(in_grad, C.c_double), _p(out_grad, C.c_float), _p(index, C.c_int),
                                       _p(dst, C.c_int), _p(values, C.c_float), dim, n)
    return in_grad


def spmm_csr_f64(rowptr, col, val, x, with_abs=False):
    """Y = A·X for CSR A, double accumulation.  with_abs also returns sum |val*x| per output."""
    rowptr, col, val, x = _i32(rowptr), _i32(col), _f32(val), _f32(x)
    n = len(rowptr) - 1
    f = x.shape[1]
    y = np.empty((n, f), np.float64)
    a = np.empty((n, f), np.float64) if with_abs else None
    lib().oracle_spmm_csr_f64(n, _p(rowptr, C.c_int), _p(col, C.c_int), _p(val, C.c_float), _p(x, C.c_float),
                              f, _p(y, C.c_double), _p(a, C.c_double) if with_abs else None, f, f)
    return (y, a) if with_abs else y


def spmm_csr_f32(rowptr, col, val, x, threads=0, out=None):
    """Y = A·X in float on `threads` host threads (0 = all): the timed CPU baseline."""
    rowptr, col, val, x = _i32(rowptr), _i32(col), _f32(val), _f32(x)
    n = len(rowptr) - 1
    f = x.shape[1]
    y = out if out is not None else np.empty((n, f), np.float32)
    lib().oracle_spmm_csr_f32(n, _p(rowptr, C.c_int), _p(col, C.c_int), _p(val, C.c_float), _p(x, C.c_float),
                              f, _p(y, C.c_float), f, f, int(threads))
    return y


def transpose_csr(n_rows, n_cols, rowptr, col, val):
    rowptr, col, val = _i32(rowptr), _i32(col), _f32(val)
    nnz = len(col)
    t_rowptr = np.empty(n_cols + 1, np.int32)
    t_col = np.empty(max(nnz, 1), np.int32)
    t_val = np.empty(max(nnz, 1), np.float32)
    lib().oracle_transpose_csr(n_rows, n_cols, _p(rowptr, C.c_int), _p(col, C.c_int), _p(val, C.c_float),
                               _p(t_rowptr, C.c_int), _p(t_col, C.c_int), _p(t_val, C.c_float))
    return t_rowptr, t_col[:nnz], t_val[:nnz]


def _parts_args(parts_u, parts_v, out_degree, owner):
    eoff = np.zeros(len(parts_u) + 1, np.int32)
    eoff[1:] = np.cumsum([len(a) for a in parts_u])
    eu = _i32(np.concatenate(parts_u)) if len(parts_u) else np.zeros(0, np.int32)
    ev = _i32(np.concatenate(parts_v)) if len(parts_v) else np.zeros(0, np.int32)
    return eoff, eu, ev, _i32(out_degree), _i32(owner)


def pr_drone_cpu(global_v, parts_u, parts_v, out_degree, owner, eps=0.01, max_steps=200, maps=False):
    """DRONE's CPU job "pr" over a partition (float32).  Returns (pr[global_v], supersteps, messages).
    maps=True keeps every worker's state in hash maps keyed by global id, as the Go program does (same bits)."""
    eoff, eu, ev, od, ow = _parts_args(parts_u, parts_v, out_degree, owner)
    out = np.empty(global_v, np.float32)
    msgs = C.c_longlong(0)
    fn = lib().oracle_pr_drone_cpu_maps if maps else lib().oracle_pr_drone_cpu
    steps = fn(len(parts_u), global_v, _p(eoff, C.c_int), _p(eu, C.c_int), _p(ev, C.c_int),
                                      _p(od, C.c_int), _p(ow, C.c_int), C.c_float(eps), int(max_steps),
                                      _p(out, C.c_float), C.byref(msgs))
    return out, steps, msgs.value


def pr_drone_cuda(global_v, parts_u, parts_v, out_degree, owner, eps=1e-6, max_steps=10000, dtype=np.float32):
    """DRONE's GPU job "pr_cuda" over a partition.  Returns (pr, supersteps, sizes[steps,4])."""
    eoff, eu, ev, od, ow = _parts_args(parts_u, parts_v, out_degree, owner)
    out = np.empty(global_v, dtype)
    sizes = np.zeros((max_steps + 1, 4), np.int64)
    if dtype == np.float32:
        steps = lib().oracle_pr_drone_cuda_f32(len(parts_u), global_v, _p(eoff, C.c_int), _p(eu, C.c_int),
                                               _p(ev, C.c_int), _p(od, C.c_int), _p(ow, C.c_int), C.c_float(eps),
                                               int(max_steps), _p(out, C.c_float), _p(sizes, C.c_longlong))
    else:
        steps = lib().oracle_pr_drone_cuda_f64(len(parts_u), global_v, _p(eoff, C.c_int), _p(eu, C.c_int),
                                               _p(ev, C.c_int), _p(od, C.c_int), _p(ow, C.c_int), C.c_double(eps),
                                               int(max_steps), _p(out, C.c_double), _p(sizes, C.c_longlong))
    return out, steps, sizes[:steps]


def cc_fixed_point(rowptr, col):
    """label[v] = smallest id among the vertices that reach v along the edges (v included)."""
    rowptr, col = _i32(rowptr), _i32(col)
    n = len(rowptr) - 1
    out = np.empty(n, np.int32)
    lib().oracle_cc_fixed_point(n, _p(rowptr, C.c_int), _p(col, C.c_int), _p(out, C.c_int))
    return out


def sssp_f32(rowptr, col, source, edge_len=None):
    """float32 distances from `source` (1e8 = not reached); edge_len None means 1.0 everywhere."""
    rowptr, col = _i32(rowptr), _i32(col)
    n = len(rowptr) - 1
    out = np.empty(n, np.float32)
    el = _f32(edge_len) if edge_len is not None else None
    lib().oracle_sssp_f32(n, _p(rowptr, C.c_int), _p(col, C.c_int), _p(el, C.c_float) if el is not None else None,
                          int(source), _p(out, C.c_float))
    return out


MP_CC, MP_SSSP = 0, 1


def mp_drone_cuda(kind, global_v, parts_u, parts_v, owner, source=-1, parts_len=None, max_steps=1000):
    """DRONE's GPU jobs "cc_cuda" (kind MP_CC) / "sssp_cuda" (MP_SSSP) over a partition.
    Returns (values[global_v] float32, supersteps, sizes[steps, P, 5]): per worker and superstep the four exchange
    sizes of struct Response and VisitedSize."""
    P = len(parts_u)
    eoff = np.concatenate([[0], np.cumsum([len(x) for x in parts_u])]).astype(np.int32)
    eu = _i32(np.concatenate(parts_u)) if eoff[-1] else np.zeros(1, np.int32)
    ev = _i32(np.concatenate(parts_v)) if eoff[-1] else np.zeros(1, np.int32)
    el = _f32(np.concatenate(parts_len)) if parts_len is not None else None
    ow = _i32(owner)
    out = np.empty(global_v, np.float32)
    sizes = np.zeros((max_steps + 1, P, 5), np.int64)
    steps = lib().oracle_mp_drone_cuda(int(kind), P, int(global_v), _p(eoff, C.c_int), _p(eu, C.c_int), _p(ev, C.c_int),
                                       _p(el, C.c_float) if el is not None else None, _p(ow, C.c_int), int(source),
                                       int(max_steps), _p(out, C.c_float), _p(sizes, C.c_longlong))
    return out, steps, sizes[:steps]


def pagerank_power_f64(rowptr, col, iterations=20, damping=0.85):
    rowptr, col = _i32(rowptr), _i32(col)
    n = len(rowptr) - 1
    out = np.empty(n, np.float64)
    lib().oracle_pagerank_power_f64(n, _p(rowptr, C.c_int), _p(col, C.c_int), int(iterations), C.c_double(damping),
                                    _p(out, C.c_double))
    return out

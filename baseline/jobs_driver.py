"""Head-to-head driver for the cgo-facing C interface of DRONE's GPU jobs (build_graph, addMasterRoute,
addMirrorRoute, loadOutDegree, PR_PEVal / PR_IncEVal, SSSP_PEVal; DRONE/src/cuda/graph.h:45-52, algorithm/pr.h,
sssp.h): the SAME calls on the SAME one-worker graph through either library that exports that interface —

    --lib reference   oracle/_ref/libref_drone_jobs.so: the reference's own sources, compiled by `make -C oracle ref`
    --lib dropin      drone_b200/lib/libdrone_pr_compat.so: this repository's implementation

Run as a script; bench.py starts it as a child process because the reference ends the process on any CUDA error.  The
reference also prints progress lines from C, so file descriptor 1 points at /dev/null while the jobs run and is put
back just before the one JSON line with the result is printed."""
import argparse
import ctypes as C
import json
import os
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class Comm(C.Structure):
    _fields_ = [("comm", C.c_void_p), ("s", C.c_void_p)]


class PRValues(C.Structure):       # DRONE/src/cuda/algorithm/pr.h:7-16
    _fields_ = [(n, C.c_void_p) for n in ("sendID", "recvID", "sendDiff", "recvDiff", "prValue", "accValue", "diffValue",
                                          "globalAcc", "globalDiff", "outDegree")]


class SSSPValues(C.Structure):     # DRONE/src/cuda/algorithm/sssp.h:8-12
    _fields_ = [(n, C.c_void_p) for n in ("sendID", "recvID", "sendDis", "recvDis", "distance")]


class Response(C.Structure):       # DRONE/src/cuda/algorithm/common.h:23-27
    _fields_ = [("Mirror2MasterSendSize", C.c_int), ("Mirror2MasterRecvSize", C.c_int),
                ("Master2MirrorSendSize", C.c_int), ("Master2MirrorRecvSize", C.c_int), ("VisitedSize", C.c_int),
                ("LocalVertexSize", C.c_int), ("CalTime", C.c_float), ("SendTime", C.c_float)]


def ints(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    if a.size == 0:
        a = np.zeros(1, np.int32)
    return a, a.ctypes.data_as(C.POINTER(C.c_int))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--lib", choices=["reference", "dropin"], required=True)
    ap.add_argument("--scale", type=int, default=20)
    ap.add_argument("--edge-factor", type=int, default=16)
    ap.add_argument("--supersteps", type=int, default=15)
    args = ap.parse_args()

    real_stdout = os.dup(1)
    devnull = os.open(os.devnull, os.O_WRONLY)
    os.dup2(devnull, 1)                    # the reference prints progress lines from C

    import torch
    import drone_b200 as db
    from drone_b200 import graphgen as gg
    from oracle import oracle
    db.lib()                               # torch's NCCL first, then anything that links libnccl.so.2
    path = oracle.reference_jobs_library() if args.lib == "reference" else os.path.join(ROOT, "drone_b200", "lib",
                                                                                         "libdrone_pr_compat.so")
    result = {"lib": args.lib}
    if path is None:
        result["unavailable"] = "oracle/_ref/libref_drone_jobs.so was not built"
    else:
        n, u, v = gg.rmat_graph(args.scale, args.edge_factor, seed=20261150, device="cuda", symmetrise=False, self_loops="drop")
        u, v = u.cpu().numpy(), v.cpu().numpy()
        out_deg = np.bincount(u, minlength=n).astype(np.int32)
        lib = C.CDLL(path)
        ip = C.POINTER(C.c_int)
        lib.build_graph.restype = C.c_void_p
        lib.build_graph.argtypes = [C.c_int, C.c_int, ip, ip, C.c_int, C.c_int, C.POINTER(Comm)]
        lib.addMasterRoute.argtypes = [C.c_void_p, ip, ip, ip, C.c_int, C.c_int]
        lib.addMirrorRoute.argtypes = [C.c_void_p, ip, ip, C.c_int]
        lib.loadOutDegree.argtypes = [C.c_void_p, C.POINTER(PRValues), ip]
        lib.getLocalVertexSize.argtypes = [C.c_void_p]
        for fn in (lib.PR_PEVal, lib.PR_IncEVal):
            fn.restype = Response
            fn.argtypes = [C.c_void_p, C.POINTER(PRValues), C.c_int, C.c_int, C.POINTER(Comm)]
        lib.SSSP_PEVal.restype = Response
        lib.SSSP_PEVal.argtypes = [C.c_void_p, C.POINTER(SSSPValues), C.c_int, C.c_int, C.c_int, C.POINTER(Comm)]
        os.chdir(tempfile.mkdtemp(prefix="drone_jobs_"))       # build_graph writes ./nccl.id
        comm, values = Comm(), PRValues()
        (ku, pu), (kv, pv), (kd, pd), (kz, pz) = ints(u), ints(v), ints(out_deg), ints([])
        t0 = time.perf_counter()
        g = lib.build_graph(n, len(u), pu, pv, 0, 1, C.byref(comm))
        lib.addMasterRoute(g, pz, pz, pz, 0, 0)
        lib.addMirrorRoute(g, pz, pz, 0)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        lib.loadOutDegree(g, C.byref(values), pd)
        torch.cuda.synchronize()
        result["build_graph_s"] = time.perf_counter() - t0       # build_graph + routes + loadOutDegree
        result["load_out_degree_ms"] = 1e3 * (time.perf_counter() - t1)
        t0 = time.perf_counter()
        lib.PR_PEVal(g, C.byref(values), 0, 1, C.byref(comm))
        torch.cuda.synchronize()
        result["pr_peval_ms"] = 1e3 * (time.perf_counter() - t0)
        per_step = []
        for _ in range(args.supersteps):
            t0 = time.perf_counter()
            lib.PR_IncEVal(g, C.byref(values), 0, 1, C.byref(comm))
            torch.cuda.synchronize()
            per_step.append(1e3 * (time.perf_counter() - t0))
        result["pr_inceval_ms"] = per_step
        result["pr_inceval_ms_total"] = float(np.sum(per_step))
        # the job as the Go worker sees it after the graph is built: degrees in, PEval, every IncEVal
        result["pr_job_ms_total"] = result["load_out_degree_ms"] + result["pr_peval_ms"] + result["pr_inceval_ms_total"]
        sp = SSSPValues()
        source = int(np.argmax(out_deg))
        t0 = time.perf_counter()
        lib.SSSP_PEVal(g, C.byref(sp), source, 0, 1, C.byref(comm))
        torch.cuda.synchronize()
        result["sssp_peval_ms"] = 1e3 * (time.perf_counter() - t0)
        result.update(vertices=int(n), edges=int(len(u)), local_vertices=int(lib.getLocalVertexSize(g)))
    sys.stdout.flush()
    C.CDLL(None).fflush(None)              # what C still holds in its buffers goes to /dev/null too
    os.dup2(real_stdout, 1)
    print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()

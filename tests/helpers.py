"""Shared helpers of the parity tests."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

# Tolerance of the float32 aggregation against the double oracle: every output element may
# differ by at most REL_TOL times sum_k |val_k * x_k| (the magnitude that was summed), and the
# whole matrix by REL_TOL relative to its largest element.  1e-5 is the bound the path's
# specification gives for GCN outputs and gradients.
REL_TOL = 1e-5


def assert_close_to_oracle(got, want64, abs64=None, tol=REL_TOL):
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == want64.shape
    assert np.isfinite(got).all()
    err = np.abs(got - want64)
    scale = np.abs(want64).max() if want64.size else 0.0
    if want64.size:
        assert err.max() <= tol * max(scale, 1e-30), "max abs err %g vs scale %g" % (err.max(), scale)
    if abs64 is not None and want64.size:
        bound = tol * abs64 + 1e-30
        worst = (err / bound).max()
        assert worst <= 1.0, "element error exceeds %g * sum|terms| by factor %g" % (tol, worst)


def graph_case(gg, oracle, n, u, v, clamp_degrees=True):
    """CSR by source + global degrees + reference coefficients for an edge list (numpy int32)."""
    import torch
    ut, vt = torch.as_tensor(u), torch.as_tensor(v)
    order = np.lexsort((v, u))
    ut, vt = ut[order], vt[order]
    index, dst = gg.csr_by_source(ut, vt, n)
    in_deg, out_deg = gg.degrees(ut, vt, n)
    in_deg, out_deg = in_deg.numpy(), out_deg.numpy()
    if clamp_degrees:
        in_deg, out_deg = np.maximum(in_deg, 1).astype(np.int32), np.maximum(out_deg, 1).astype(np.int32)
    index, dst = index.numpy(), dst.numpy()
    val = oracle.csr_values_f32(index, dst, in_deg, out_deg)
    return index, dst, in_deg, out_deg, val


def run_ranks(target, world, extra_args=(), timeout=300):
    """Run target(rank, world, *extra_args, ok) as `world` spawned processes (one per GPU), `ok` being a shared int
    array every rank sets to 1 at its end.  Ranks still alive at the time limit, or after a sibling has already failed
    (they may be waiting for it inside a collective on the GPU), are terminated before anything is asserted, so that
    a failing rank cannot leave its peer behind."""
    import time
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ok = ctx.Array("i", [0] * world)
    procs = [ctx.Process(target=target, args=(r, world, *extra_args, ok)) for r in range(world)]
    try:
        for p in procs:
            p.start()
        deadline = time.time() + timeout
        while time.time() < deadline and any(p.is_alive() for p in procs):
            if any(p.exitcode not in (None, 0) for p in procs):
                time.sleep(5)          # a rank failed: give the others a moment to leave on their own, then stop them
                break
            time.sleep(0.2)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    assert [p.exitcode for p in procs] == [0] * world, "exit codes %r" % [p.exitcode for p in procs]
    assert list(ok) == [1] * world

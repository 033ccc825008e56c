"""drone_spmm_static_scratch: the aggregation for callers that cannot allocate device memory (everything
already handed to their own pool, or a thread that must not wait on the driver's allocator).  It keeps the
partial sums of split rows in an array built into the library instead of a buffer grown with cudaMalloc.

Checked here through the C ABI: its output equals drone_spmm's bit for bit on two calls in a row (the shared
array keeps the previous call's contents, which must not matter), for a vector and a scalar feature width and
both orientations; the free device memory reported by the driver is the same before and after its calls; and a
plan whose partial sums do not fit is refused with DRONE_E_TOO_LARGE.
This file sorts last on purpose: a run that stops at the first failure has then run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import drone_b200 as db
from drone_b200 import graphgen as gg

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 16 << 20
E_TOO_LARGE = -5


def call_static(plan, orientation, x, y):
    n, f = x.shape
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    return db.lib().drone_spmm_static_scratch(plan.handle, orientation, f, C.c_void_p(x.data_ptr()), x.stride(0),
                                              C.c_void_p(y.data_ptr()), y.stride(0), stream)


def make_plan(dev, scale, seed):
    n, u, v = gg.rmat_graph(scale, 16, seed=seed, symmetrise=False, self_loops="add")
    index, dst = gg.csr_by_source(u, v, n)
    in_deg, out_deg = gg.degrees(u, v, n)
    plan = db.AggregationPlan(index.to(dev), dst.to(dev), in_degree=in_deg.to(dev), out_degree=out_deg.to(dev))
    return n, plan


def test_static_scratch_matches_allocating_entry_point(cuda_device):
    n, plan = make_plan(cuda_device, 13, 71)
    st = plan.stats()
    assert st.n_partials[db.OP_AT] > 0 and st.n_partials[db.OP_A] > 0      # the scratch is really used
    for f in (64, 41):
        assert st.n_partials[db.OP_AT] * f * 4 <= STATIC_SCRATCH_BYTES
        x1 = torch.as_tensor(gg.seeded_normal(f, (n, f)), device=cuda_device)
        x2 = torch.as_tensor(gg.seeded_normal(f + 1000, (n, f)), device=cuda_device)
        for op in (db.OP_AT, db.OP_A):
            want1 = plan.spmm(op, x1)
            want2 = plan.spmm(op, x2)
            got1 = torch.full_like(want1, float("nan"))
            got2 = torch.full_like(want2, float("nan"))
            assert call_static(plan, op, x1, got1) == 0, db.lib().drone_last_error()
            assert call_static(plan, op, x2, got2) == 0, db.lib().drone_last_error()   # second call in a row
            torch.cuda.synchronize()
            assert torch.equal(got1, want1)
            assert torch.equal(got2, want2)
    # the claim itself: no device memory is taken by the calls (the address lookup of the first call is behind us)
    x = torch.as_tensor(gg.seeded_normal(77, (n, 64)), device=cuda_device)
    y = torch.empty_like(x)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(cuda_device)[0]
    held_before = plan.stats().scratch_bytes
    for op in (db.OP_AT, db.OP_A):
        assert call_static(plan, op, x, y) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(cuda_device)[0] == free_before
    assert plan.stats().scratch_bytes == held_before
    # a different plan uses the same array afterwards
    n2, plan2 = make_plan(cuda_device, 11, 72)
    x = torch.as_tensor(gg.seeded_normal(5, (n2, 32)), device=cuda_device)
    got = torch.empty_like(x)
    assert call_static(plan2, db.OP_AT, x, got) == 0
    assert torch.equal(got, plan2.spmm(db.OP_AT, x))


def test_static_scratch_refuses_what_does_not_fit(cuda_device):
    # a star with 70,000 leaves and chunks of 8 nonzeros: 8,750 partial slots, times F=512 floats > 16 MiB
    import os
    n = 70001
    u = np.concatenate([np.zeros(n - 1, np.int32), np.arange(1, n, dtype=np.int32)])
    v = np.concatenate([np.arange(1, n, dtype=np.int32), np.zeros(n - 1, np.int32)])
    order = np.lexsort((v, u))
    ut, vt = torch.as_tensor(u[order]), torch.as_tensor(v[order])
    index, dst = gg.csr_by_source(ut, vt, n)
    in_deg, out_deg = gg.degrees(ut, vt, n)
    old = {k: os.environ.get(k) for k in ("DRONE_SHORT_ROW_LIMIT", "DRONE_CHUNK_NNZ")}
    os.environ["DRONE_SHORT_ROW_LIMIT"], os.environ["DRONE_CHUNK_NNZ"] = "4", "8"
    try:
        plan = db.AggregationPlan(index.to(cuda_device), dst.to(cuda_device), in_degree=in_deg.to(cuda_device),
                                  out_degree=out_deg.to(cuda_device))
    finally:
        for k, val in old.items():
            if val is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = val
    f = 512
    assert plan.stats().n_partials[db.OP_A] * f * 4 > STATIC_SCRATCH_BYTES
    x = torch.ones((n, f), device=cuda_device)
    y = torch.full((n, f), 3.0, device=cuda_device)
    assert call_static(plan, db.OP_A, x, y) == E_TOO_LARGE
    msg = db.lib().drone_last_error().decode()
    assert "built-in scratch holds" in msg and "drone_spmm" in msg
    torch.cuda.synchronize()
    assert (y == 3.0).all()                      # nothing was launched
    # the same plan at a width that fits is served
    x8 = torch.ones((n, 8), device=cuda_device)
    y8 = torch.empty((n, 8), device=cuda_device)
    assert call_static(plan, db.OP_A, x8, y8) == 0
    assert torch.equal(y8, plan.spmm(db.OP_A, x8))

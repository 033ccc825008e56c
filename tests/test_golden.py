"""The committed golden vectors still equal what the oracle computes from the seeded inputs."""
import os

import numpy as np

from drone_b200 import graphgen as gg
from helpers import ROOT

import make_golden


def test_golden_matches_oracle(oracle):
    gold = np.load(os.path.join(ROOT, "tests", "golden", "spmm_golden.npz"))
    for name, scale, ef, seed, sym, loops, widths in make_golden.CASES:
        n, index, dst, in_deg, out_deg = make_golden.case_inputs(scale, ef, seed, sym, loops)
        val = oracle.csr_values_f32(index, dst, in_deg, out_deg)
        assert int(gold[name + "/nnz"]) == len(dst)
        assert float(gold[name + "/val_sum"]) == float(val.astype(np.float64).sum())
        for f in widths:
            x = gg.seeded_normal(1000 + f, (n, f))
            assert np.array_equal(gold["%s/fwd_F%d" % (name, f)], oracle.graphsum_forward_f64(x, index, dst, val))
            assert np.array_equal(gold["%s/bwd_F%d" % (name, f)], oracle.graphsum_backward_f64(x, index, dst, val))


def test_jobs_golden_matches_oracle(oracle):
    """PageRank (power iteration, GPU job in double, CPU job), CC labels, SSSP distances and the per-superstep
    exchange sizes of the cc / sssp jobs over seeded EBV partitions."""
    gold = np.load(os.path.join(ROOT, "tests", "golden", "jobs_golden.npz"))
    for name, scale, ef, seed, parts in make_golden.JOB_CASES:
        now = make_golden.job_outputs(scale, ef, seed, parts)
        for k, a in now.items():
            g = gold["%s/%s" % (name, k)]
            if k in ("pr_power_f64", "pr_job_f64"):
                # sums of doubles over in-edges: identical order here, but allow the last bits across compilers
                assert np.allclose(g, a, rtol=1e-13, atol=0), (name, k)
            else:
                assert np.array_equal(g, a), (name, k)


def test_seeded_normal_is_standard():
    x = gg.seeded_normal(5, (200000,))
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 1.0) < 0.01
    assert np.array_equal(x[:100], gg.seeded_normal(5, (200000,))[:100])
    # frozen values: the generator must never drift, the golden file depends on it
    first = gg.seeded_normal(1032, (4,)).tolist()
    assert first == gg.seeded_normal(1032, (2, 2)).ravel().tolist()

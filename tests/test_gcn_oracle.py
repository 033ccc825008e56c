"""The GCN oracle's gradients against finite differences of its own loss (no GPU)."""
import numpy as np

from drone_b200 import graphgen as gg
from helpers import graph_case
from oracle import gcn_oracle


def test_weight_gradients_match_finite_differences(oracle):
    n, u, v = gg.rmat_graph(6, 6, seed=61, symmetrise=True, self_loops="add")
    index, dst, in_deg, out_deg, val = graph_case(gg, oracle, n, u.numpy(), v.numpy())
    rng = np.random.default_rng(0)
    x = rng.standard_normal((n, 5))
    w1 = rng.standard_normal((5, 4)) * 0.5
    w2 = rng.standard_normal((4, 3)) * 0.5
    truth = rng.integers(-1, 3, n).astype(np.int32)
    base = gcn_oracle.gcn_step(index, dst, val, x, w1, w2, truth)
    count = int((truth >= 0).sum())       # the reference's gradient is that of (count * loss)
    eps = 1e-6
    for (w, name) in ((w1, "d_w1"), (w2, "d_w2")):
        for idx in ((0, 0), (2, 1), (w.shape[0] - 1, w.shape[1] - 1)):
            wp, wm = w.copy(), w.copy()
            wp[idx] += eps
            wm[idx] -= eps
            args_p = (wp, w2) if name == "d_w1" else (w1, wp)
            args_m = (wm, w2) if name == "d_w1" else (w1, wm)
            lp = gcn_oracle.gcn_step(index, dst, val, x, *args_p, truth)["loss"]
            lm = gcn_oracle.gcn_step(index, dst, val, x, *args_m, truth)["loss"]
            fd = count * (lp - lm) / (2 * eps)
            assert abs(fd - base[name][idx]) < 1e-5 * max(1.0, abs(fd))

"""The reference's own GCN training epoch (cuda_gcn's CUDAGCN, compiled from its sources by `make -C oracle ref`) on
one GPU, over the synthetic graph, features, labels and starting weights of one of bench.py's GCN configurations.

Run as a script; bench.py starts it as a child process because the reference ends the process on any CUDA error and
prints progress lines from C (file descriptor 1 points at /dev/null while it runs).  Prints one JSON line:
ms per epoch of CUDAGCN::train_epoch (weight broadcast, forward, loss, accuracy, backward, gradient reduce, Adam),
the part of that spent in its per-epoch bookkeeping (set_truth's reallocations, get_accuracy's copy of all logits to
the host) timed on its own, and the cross-entropy loss of the first epoch."""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--vertices", type=int, required=True)
    ap.add_argument("--pairs", type=int, required=True)
    ap.add_argument("--seed", type=int, required=True)
    ap.add_argument("--dims", required=True, help="input,hidden,classes")
    ap.add_argument("--epochs", type=int, default=5)
    args = ap.parse_args()
    dims = [int(x) for x in args.dims.split(",")]
    if len(dims) != 3:
        raise SystemExit("the reference's model has two layers: --dims input,hidden,classes")
    import numpy as np
    import torch
    from drone_b200 import graphgen as gg
    from oracle import oracle
    if not oracle.reference_available():
        print(json.dumps({"error": "oracle/_ref/libref_graphsum.so was not built"}))
        return
    dev = torch.device("cuda:0")
    n, u, v = gg.powerlaw_graph(args.vertices, args.pairs, seed=args.seed, device=dev)
    in_deg, out_deg = gg.degrees(u, v, n)
    ids = np.arange(n)
    x = gg.hashed_normal(ids, dims[0], 7, dev).cpu().numpy()
    truth = gg.hashed_labels(ids, dims[-1], 7, dev).cpu().numpy()
    w1, w2 = [w.cpu().numpy() for w in gg.glorot_weights(dims, dev)]
    uh, vh, ind, outd = u.cpu().numpy(), v.cpu().numpy(), in_deg.cpu().numpy(), out_deg.cpu().numpy()
    del u, v, in_deg, out_deg
    torch.cuda.empty_cache()
    sys.stdout.flush()
    saved = os.dup(1)
    devnull = os.open(os.devnull, os.O_WRONLY)
    os.dup2(devnull, 1)
    try:
        ms, book, loss = oracle.reference_gcn_epochs(n, uh, vh, ind, outd, dims, x, truth, w1, w2, warmup=2,
                                                     epochs=args.epochs)
    finally:
        os.dup2(saved, 1)
    # The bookkeeping steps are timed in a loop of their own (host-side allocations and a pageable copy: their time
    # moves with the load on the host), so the difference is given only when it means something.
    print(json.dumps({"ms_per_epoch": ms, "ms_bookkeeping_per_epoch": book, "first_epoch_loss": loss,
                      "ms_per_epoch_without_bookkeeping": ms - book if 0 <= book < ms else None,
                      "epochs": args.epochs, "vertices": n,
                      "nnz": int(len(uh)), "dims": dims, "workers": 1,
                      "what": "CUDAGCN::train_epoch of the reference's sources (cuSPARSE aggregation, FULL_BATCH, no "
                              "compression), one worker"}), flush=True)


if __name__ == "__main__":
    main()

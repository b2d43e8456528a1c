"""Small, bounded invocations of single hot-path kernels, for profilers.

    python profile_case.py dense_rows --rows 20000 --reps 3
    python profile_case.py csr_rows   --rows 20242 --reps 3
    python profile_case.py solver     --rows 20000 --steps 5
    python profile_case.py predict    --rows 100000 --q 8192 --reps 3

Each case builds seeded synthetic data of the benchmark's shape at a reduced row count (larger than
L2, a few hundred MB on the device), runs the kernel `reps` times and prints CUDA-event timings.
"""
import argparse

import numpy as np
import torch

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from thundersvm_b200 import capi, synth  # noqa: E402


def _time(fn, reps):
    out = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record(); e1.synchronize()
        out.append(e0.elapsed_time(e1))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["dense_rows", "csr_rows", "solver", "predict"])
    ap.add_argument("--rows", type=int, default=20000)
    ap.add_argument("--q", type=int, default=512)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--d", type=int, default=2000, help="features of the dense cases")
    ap.add_argument("--no-overlap", action="store_true", help="solver case: run the steps one after the other")
    ap.add_argument("--engine", default="auto", help="dense engine: auto, simt, tensor2 (TF32 planes), tensor (FP16 planes)")
    ap.add_argument("--csr-config", default="c4", choices=["c2", "c4"],
                    help="csr_rows case: config 4 (47,236 features, L2-panel engine) or config 2 (123 features, "
                         "shared-memory-panel engine)")
    args = ap.parse_args()
    capi.lib()
    if args.case == "predict":
        # fused prediction: --rows support vectors, --q test rows, binary model
        prob = synth.config5(args.rows, d=args.d)
        km = capi.KernelMatrix(dense=torch.from_numpy(prob["X"]).cuda(), gamma=prob["gamma"])
        T = torch.from_numpy(synth.config5(args.q, d=args.d, seed=8)["X"]).cuda()
        coef = torch.randn(args.rows, dtype=torch.float64, device="cuda")
        rho = torch.zeros(1, dtype=torch.float64, device="cuda")
        cnt = [args.rows // 2, args.rows - args.rows // 2]
        capi.predict_labels(km, coef, cnt, rho, 2, dense=T)
        torch.cuda.synchronize()
        ms = _time(lambda: capi.predict_labels(km, coef, cnt, rho, 2, dense=T), args.reps)
        out = torch.empty((args.q, km.n), dtype=torch.float32, device="cuda")
        ms2 = _time(lambda: km.get_rows_instances(dense=T, out=out), args.reps)
        fl = 2.0 * args.rows * args.q * args.d
        print("predict n_sv=%d rows=%d d=%d: fused ms %s (%.0f TFLOP/s), kernel block only ms %s (%.0f TFLOP/s)" % (
            args.rows, args.q, args.d, ["%.3f" % t for t in ms], fl / min(ms) / 1e9, ["%.3f" % t for t in ms2],
            fl / min(ms2) / 1e9))
        return
    if args.case in ("dense_rows", "solver"):
        prob = synth.config5(args.rows, d=args.d)
        km = capi.KernelMatrix(dense=torch.from_numpy(prob["X"]).cuda(), gamma=prob["gamma"])
        km.set_dense_engine(args.engine)
    else:
        prob = synth.config4(args.rows) if args.csr_config == "c4" else synth.config2(args.rows)
        val, rp, col = prob["csr"]
        km = capi.KernelMatrix(csr=(torch.from_numpy(val).cuda(), torch.from_numpy(rp).cuda(),
                                    torch.from_numpy(col).cuda()), d=prob["d"], gamma=prob["gamma"])
    n = km.n
    if args.case == "solver":
        y = torch.from_numpy(np.where(prob["y"] > 0, 1, -1).astype(np.int32)).cuda()
        alpha = torch.zeros(n, dtype=torch.float64, device="cuda")
        f = -y.to(torch.float64)
        sv = capi.Solver(km, y, alpha, f, 1e-3, prob["C"], prob["C"], 1024)
        sv.set_overlap(not args.no_overlap)
        ms = _time(lambda: sv.iterate(1), args.steps)
        print("solver steps (ms):", ["%.3f" % t for t in ms], sv.stats())
        return
    idx = torch.from_numpy(np.random.default_rng(0).choice(n, args.q, replace=False).astype(np.int32)).cuda()
    out = torch.empty((args.q, (n + 3) // 4 * 4), dtype=torch.float32, device="cuda")      # the solver's row stride
    km.get_rows(idx, out)
    torch.cuda.synchronize()
    ms = _time(lambda: km.get_rows(idx, out), args.reps)
    print("%s n=%d d=%d q=%d: ms per call %s" % (args.case, n, km.d, args.q, ["%.3f" % t for t in ms]))


if __name__ == "__main__":
    main()

"""Generates tests/golden/c5_scale.npz: the reference's own CPU solver (oracle/_ref) run to convergence
on the first N instances of the 400,000 x 2,000 configuration's generator (N = 30,000 by default) - the
full problem is not tractable on host cores. Holds the objective, rho, the support-vector count, the
iteration counts and decision values of the first 64 test rows, for the GPU parity test at that size.

    python tests/golden/make_c5_scale.py [N]
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_binding as R  # noqa: E402
from thundersvm_b200 import synth  # noqa: E402

N = int(sys.argv[1]) if len(sys.argv) > 1 else 30000
prob = synth.config5(N)
y = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
D = R.Data(dense=prob["X"])
t0 = time.time()
alpha, f, rho, sec = R.smo_solve(D, y, np.zeros(N), -y.astype(np.float64), 1e-3, 1.0, 1.0, 1024, gamma=prob["gamma"])
obj = -float(np.sum(alpha - (f + y) * alpha * y / 2))
test = synth.config5(64, seed=8)
sv = np.nonzero(alpha)[0]
K = R.kernel_rows_ins(R.Data(dense=prob["X"][sv]), R.Data(dense=test["X"]), gamma=prob["gamma"])
dec = K @ (alpha[sv] * y[sv]) - rho
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "c5_scale.npz"), n=N, objective=obj, rho=rho,
                    n_sv=int((alpha != 0).sum()), n_bounded=int((alpha == 1.0).sum()), dec=dec, seconds=sec)
print("N", N, "obj", obj, "rho", rho, "n_sv", int((alpha != 0).sum()), "solve seconds", sec, "wall", time.time() - t0)

"""Generates tests/golden/full_c1.npz, full_c2.npz, full_c3cut.npz, full_c4.npz and prob.npz: the reference's own
CPU build (oracle/_ref) run to convergence on the benchmark configurations at their FULL size - 10,000 x 20
dense, 32,561 x 123 CSR with its 16,281-row prediction set, 20,242 x 47,236 CSR, and the first three classes of
the 60,000 x 784 ten-class problem at full per-class size (about 18,000 rows, three one-vs-one sub-problems) - and
the reference's Platt coefficients on dataset/test_dataset.txt.

    python tests/golden/make_full_configs.py [c1 c2 c3cut c4 prob] [--ref path/to/reference]

Each fixture holds what the equivalence bounds are stated on: dual objective, rho, support-vector count(s),
decision values and labels of a fixed set of test rows, plus 4 reference kernel rows. The data itself is not
stored: the tests regenerate it from thundersvm_b200.synth with the same seeds.
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_binding as R  # noqa: E402
from thundersvm_b200 import synth  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
ROW_IDS = 4


def objective(alpha, f, y):
    return -float(np.sum(alpha - (f + y) * alpha * y / 2))


def data_of(prob, rows=None):
    if "X" in prob:
        return R.Data(dense=prob["X"] if rows is None else prob["X"][rows])
    val, rp, col = prob["csr"]
    if rows is not None:
        cnt = np.diff(rp)[rows]
        sel = np.concatenate([np.arange(rp[r], rp[r + 1]) for r in rows]) if len(rows) else np.zeros(0, np.int64)
        rp2 = np.concatenate([[0], np.cumsum(cnt)]).astype(np.int32)
        return R.Data(csr=(val[sel], rp2, col[sel]), d=prob["d"])
    return R.Data(csr=(val, rp, col), d=prob["d"])


def binary_case(tag, prob, test):
    """One binary C-SVC solve through CSMOSolver::solve, then decision values of the test rows."""
    D = data_of(prob)
    y = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
    n = len(y)
    t0 = time.time()
    a, f, rho, sec = R.smo_solve(D, y, np.zeros(n), -y.astype(np.float64), prob["eps"], prob["C"], prob["C"], 1024,
                                 gamma=prob["gamma"])
    sv = np.nonzero(a)[0]
    Tt = data_of(test)
    dec = np.empty(Tt.n)
    Dsv = data_of(prob, sv)
    for s in range(0, Tt.n, 2048):                      # K(test, sv) in slabs
        rows = np.arange(s, min(Tt.n, s + 2048))
        K = R.kernel_rows_ins(Dsv, data_of(test, rows), gamma=prob["gamma"])
        dec[rows] = K.astype(np.float64) @ (a[sv] * y[sv]) - rho
    idx = (np.arange(ROW_IDS, dtype=np.int64) * 7919 + 11) % n
    rows, _, _ = R.kernel_rows_idx(D, idx.astype(np.int32), gamma=prob["gamma"])
    np.savez_compressed(os.path.join(OUT, "full_%s.npz" % tag), n=n, objective=objective(a, f, y), rho=rho,
                        n_sv=len(sv), n_bounded=int((a == prob["C"]).sum()), dec=dec,
                        labels=np.where(dec > 0, 1, -1).astype(np.int8), rows_idx=idx.astype(np.int32),
                        rows=rows, solve_seconds=sec)
    print(tag, "n", n, "obj", objective(a, f, y), "rho", rho, "n_sv", len(sv), "solve s", sec, "wall",
          time.time() - t0, flush=True)


def c3cut():
    """First three classes of the ten-class problem, every class at its full size, through SVC::train."""
    full = synth.config3()
    keep = np.nonzero(full["y"] < 3)[0]
    X, y = full["X"][keep], full["y"][keep]
    t0 = time.time()
    m = R.Model("c_svc", R.Data(dense=X), y, gamma=full["gamma"], C_=full["C"], eps=full["eps"])
    test = synth.config3(10000, seed=5)
    tk = np.nonzero(test["y"] < 3)[0][:1000]
    lab, dec, _ = m.predict(R.Data(dense=test["X"][tk]))
    np.savez_compressed(os.path.join(OUT, "full_c3cut.npz"), n=len(y), n_sv=m.n_sv, rho=m.rho,
                        coef_abs_sum=np.abs(m.coef.reshape(m.n_classes - 1, -1)).sum(1), dec=dec,
                        labels=lab.astype(np.int8), test_rows=tk.astype(np.int32), train_seconds=m.train_seconds)
    print("c3cut n", len(y), "n_sv", m.n_sv, "rho", m.rho, "train s", m.train_seconds, "wall", time.time() - t0,
          "test acc", float((lab == test["y"][tk]).mean()), flush=True)


def load_libsvm(path):
    ys, val, col, rp = [], [], [], [0]
    for line in open(path):
        t = line.split()
        if not t:
            continue
        ys.append(float(t[0]))
        for kv in t[1:]:
            k, v = kv.split(":")
            col.append(int(k) - 1)
            val.append(float(v))
        rp.append(len(val))
    return (np.array(ys, np.float32), np.array(val, np.float32), np.array(rp, np.int32), np.array(col, np.int32))


def prob_fixture(ref_root):
    """probA / probB of SVC::probability_train (svc.cpp:427-492) on dataset/test_dataset.txt, C = 100, gamma = 0.5."""
    y, val, rp, col = load_libsvm(os.path.join(ref_root, "dataset", "test_dataset.txt"))
    D = R.Data(csr=(val, rp, col), d=int(col.max()) + 1)
    m = R.Model("c_svc", D, y, gamma=0.5, C_=100, probability=1)
    text = m.save_to_string()
    out = {}
    for line in text.splitlines():
        t = line.split()
        if t and t[0] in ("probA", "probB"):
            out[t[0]] = np.array([float(v) for v in t[1:]])
    np.savez_compressed(os.path.join(OUT, "prob.npz"), **out)
    print("prob", out, flush=True)


if __name__ == "__main__":
    args = sys.argv[1:]
    import subprocess
    ref_root = subprocess.check_output(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "print-ref"],
                                       text=True).strip()
    if "--ref" in args:
        ref_root = args[args.index("--ref") + 1]
        args = [a for a in args if a not in ("--ref", ref_root)]
    which = args or ["prob", "c1", "c2", "c4", "c3cut"]
    if "prob" in which:
        prob_fixture(ref_root)
    if "c1" in which:
        binary_case("c1", synth.config1(), synth.config1(2048, seed=11))
    if "c2" in which:
        binary_case("c2", synth.config2(), synth.config2(16281, seed=3))
    if "c4" in which:
        binary_case("c4", synth.config4(), synth.config4(1024, seed=16))
    if "c3cut" in which:
        c3cut()

"""Generates tests/golden/*.npz from the reference's own CPU build (oracle/_ref).

Run where the reference sources are mounted and `make -C oracle ref` has been done:
    python tests/golden/make_golden.py [path/to/reference]
The fixtures pin (a) the reference tests' known answers on dataset/test_dataset.txt and
(b) reference outputs (kernel rows, alpha, rho, objective, decision values) on small seeded
problems from thundersvm_b200.synth, so that the CPU restatement and the CUDA path can be
checked on machines that have neither the reference sources nor its build.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_binding as R  # noqa: E402
from thundersvm_b200 import synth  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


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


def objective(alpha, f, y):
    return -float(np.sum(alpha - (f + y) * alpha * y / 2))


def fixture_dataset(ref_root):
    y, val, rp, col = load_libsvm(os.path.join(ref_root, "dataset", "test_dataset.txt"))
    d = int(col.max()) + 1
    D = R.Data(csr=(val, rp, col), d=d)
    out = dict(y=y, val=val, row_ptr=rp, col=col, d=d)
    # test_kernelmatrix.cpp:69-143: rows idx = i*3+4 (i<10) and the first 10 instances, 4 kernels
    idx = np.arange(10, dtype=np.int32) * 3 + 4
    first = R.Data(csr=(val[:rp[10]], rp[:11], col[:rp[10]]), d=d)
    for name, kw in (("rbf", dict(gamma=0.5)), ("poly", dict(gamma=0.5, degree=3, coef0=0.1)),
                     ("linear", dict()), ("sigmoid", dict(gamma=0.5, coef0=0.1))):
        rows, diag, _ = R.kernel_rows_idx(D, idx, kernel=name, **kw)
        out["rows_idx_" + name] = rows
        out["diag_" + name] = diag
        out["rows_ins_" + name] = R.kernel_rows_ins(D, first, kernel=name, **kw)
    # model-level known answers (test_svc.cpp:36, test_nusvc.cpp:43, test_svr.cpp:38, test_nusvr.cpp:41,
    # test_oneclass_svc.cpp:27) with the model internals next to them
    for tag, st, kw in (("svc", "c_svc", dict(gamma=0.5, C_=100)), ("nusvc", "nu_svc", dict(gamma=0.5, nu=0.1, C_=100)),
                        ("svr", "epsilon_svr", dict(gamma=0.5, C_=100)),
                        ("nusvr", "nu_svr", dict(gamma=0.5, C_=100, nu=0.1)),
                        ("oneclass", "one_class", dict(gamma=0.5, nu=0.1))):
        m = R.Model(st, D, y, **kw)
        lab, dec, _ = m.predict(D)
        out[tag + "_pred"] = lab
        out[tag + "_dec"] = dec
        out[tag + "_rho"] = m.rho
        out[tag + "_coef"] = m.coef
        out[tag + "_n_sv"] = m.n_sv
        out[tag + "_sv_ind"] = m.sv_ind
        if tag == "svc":
            out["svc_model_text"] = np.frombuffer(m.save_to_string().encode(), dtype=np.uint8)
    for tag, st, kw in (("svc", "c_svc", dict(gamma=0.125, C_=10)), ("nusvc", "nu_svc", dict(gamma=0.125)),
                        ("nusvr", "nu_svr", dict(gamma=0.125)), ("svr", "epsilon_svr", dict(gamma=0.125))):
        out["cv_" + tag] = R.cross_validation(st, D, y, 5, **kw)   # test_cross_validation.cpp:51-84
    np.savez_compressed(os.path.join(OUT, "test_dataset.npz"), **out)


def fixture_solver():
    """Reference solver outputs on small seeded problems (one per data family)."""
    out = {}
    cases = {
        "c1": (synth.config1(1500), None),
        "c1_soft": (dict(synth.config1(1500), gamma=0.025), None),      # non-degenerate side case
        "c2": (synth.config2(1200), None),
        "c3": (synth.config3(900), 5),
        "c4": (synth.config4(700), None),
        "c5": (synth.config5(1100, d=200), None),
    }
    for tag, (prob, split) in cases.items():
        if "X" in prob:
            D = R.Data(dense=prob["X"])
        else:
            D = R.Data(csr=prob["csr"], d=prob["d"])
        y = np.where(prob["y"] > 0, 1, -1).astype(np.int32) if split is None else \
            np.where(prob["y"] < split, 1, -1).astype(np.int32)
        n = len(y)
        ws = min(1024, 2 ** int(np.log2(n)))
        a, f, rho, _ = R.smo_solve(D, y, np.zeros(n), -y.astype(np.float64), 1e-3, prob["C"], prob["C"], ws,
                                   gamma=prob["gamma"])
        idx = (np.arange(24, dtype=np.int32) * 37 + 5) % n
        rows, _, _ = R.kernel_rows_idx(D, idx, gamma=prob["gamma"])
        out[tag + "_alpha"] = a
        out[tag + "_f"] = f
        out[tag + "_rho"] = rho
        out[tag + "_obj"] = objective(a, f, y)
        out[tag + "_rows_idx"] = idx
        out[tag + "_rows"] = rows
    # nu solver (CPU semantics of the reference build) on one problem
    prob = synth.config1(800)
    D = R.Data(dense=prob["X"])
    y = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
    n = len(y)
    nu = 0.3
    a0 = np.zeros(n)
    sp = sn = nu * n / 2
    for i in range(n):                       # nusvc.cpp:17-27
        if y[i] > 0:
            a0[i] = min(1.0, sp); sp -= a0[i]
        else:
            a0[i] = min(1.0, sn); sn -= a0[i]
    a, f, rho, _ = R.smo_solve(D, y, a0, np.zeros(n), 1e-3, 1.0, 1.0, 512, solver="nu_svc", gamma=0.5)
    out["nu_alpha0"] = a0
    out["nu_alpha"] = a
    out["nu_f"] = f
    out["nu_rho"] = rho
    np.savez_compressed(os.path.join(OUT, "solver_small.npz"), **out)


if __name__ == "__main__":
    import subprocess
    ref_root = sys.argv[1] if len(sys.argv) > 1 else subprocess.check_output(
        ["make", "-s", "-C", os.path.join(ROOT, "oracle"), "print-ref"], text=True).strip()
    fixture_dataset(ref_root)
    fixture_solver()
    print("wrote", [f for f in os.listdir(OUT) if f.endswith(".npz")])

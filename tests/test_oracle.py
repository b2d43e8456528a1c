"""Pins the CPU restatement (oracle/svm_oracle.c) against the reference: the committed golden
fixtures (generated from the reference's own CPU build by tests/golden/make_golden.py), the
reference tests' known answers, and - where it has been built - the reference library itself."""
import os

import numpy as np
import pytest

from oracle import port_binding as P
from oracle import ref_binding as R
from thundersvm_b200 import synth
from util import binary_labels, objective, oracle_matrix


@pytest.fixture(scope="module")
def ds(golden_dir):
    g = np.load(os.path.join(golden_dir, "test_dataset.npz"))
    X = P.Csr(csr=(g["val"], g["row_ptr"], g["col"]), d=int(g["d"]))
    return g, X


KERNEL_CASES = [("rbf", dict(gamma=0.5)), ("poly", dict(gamma=0.5, degree=3, coef0=0.1)), ("linear", dict()),
                ("sigmoid", dict(gamma=0.5, coef0=0.1))]


@pytest.mark.parametrize("name,kw", KERNEL_CASES)
def test_kernel_rows_match_reference_fixture(ds, name, kw):
    """test_kernelmatrix.cpp:69-143 shapes (idx = 3i+4, first 10 instances), values from the reference."""
    g, X = ds
    idx = np.arange(10, dtype=np.int32) * 3 + 4
    rows = P.kernel_rows_idx(X, idx, kernel=name, **kw)
    assert np.array_equal(rows, g["rows_idx_" + name])
    assert np.array_equal(P.diag(X, kernel=name, **kw), g["diag_" + name])
    rp = g["row_ptr"]
    T = P.Csr(csr=(g["val"][:rp[10]], rp[:11], g["col"][:rp[10]]), d=int(g["d"]))
    assert np.array_equal(P.kernel_rows_ins(X, T, kernel=name, **kw), g["rows_ins_" + name])


@pytest.mark.parametrize("name,kw", KERNEL_CASES)
def test_kernel_rows_match_naive_kernel(ds, name, kw):
    """The reference test compares get_rows with a naive float kernel within 1e-4 (test_kernelmatrix.cpp:103)."""
    g, X = ds
    n, d = X.n, X.d
    D = np.zeros((n, d))
    rows_of = np.repeat(np.arange(n), np.diff(g["row_ptr"]))
    D[rows_of, g["col"]] = g["val"]
    idx = np.arange(10) * 3 + 4
    dot = D[idx] @ D.T
    gamma, coef0, degree = kw.get("gamma", 0.0), kw.get("coef0", 0.0), kw.get("degree", 3)
    if name == "rbf":
        sd = (D * D).sum(1)
        ref = np.exp(-gamma * (sd[idx][:, None] + sd[None, :] - 2 * dot))
    elif name == "poly":
        ref = (gamma * dot + coef0) ** degree
    elif name == "sigmoid":
        ref = np.tanh(gamma * dot + coef0)
    else:
        ref = dot
    got = P.kernel_rows_idx(X, idx, kernel=name, **kw)
    assert np.max(np.abs(got - ref) / np.maximum(1.0, np.abs(ref))) < 1e-4


def _train_c_svc_ovo(X, g, gamma, C):
    """SVC::train restated with the oracle's solver (svc.cpp:41-177): returns predictions on the
    training rows and the per-pair rho, using only oracle functions."""
    y = g["y"]
    labels = []
    for v in y:                                   # DataSet::group_classes keeps first-seen order
        if v not in labels:
            labels.append(v)
    order = np.concatenate([np.nonzero(y == lab)[0] for lab in labels])
    counts = [int((y == lab).sum()) for lab in labels]
    starts = np.concatenate([[0], np.cumsum(counts)])
    val, rp, col = g["val"], g["row_ptr"], g["col"]

    def sub(ids):
        lens = rp[ids + 1] - rp[ids]
        nrp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        take = np.concatenate([np.arange(rp[i], rp[i + 1]) for i in ids])
        return P.Csr(csr=(val[take], nrp, col[take]), d=int(g["d"]))

    nc = len(labels)
    n = len(y)
    alphas, rhos = {}, []
    is_sv = np.zeros(n, dtype=bool)
    for i in range(nc):
        for j in range(i + 1, nc):
            ids = np.concatenate([order[starts[i]:starts[i + 1]], order[starts[j]:starts[j + 1]]])
            yy = np.concatenate([np.ones(counts[i]), -np.ones(counts[j])]).astype(np.int32)
            m = len(ids)
            ws = min(2 ** int(np.log2(m)), 1024)
            r = P.smo_solve(sub(ids), yy, np.zeros(m), -yy.astype(np.float64), 1e-3, C, C, ws, gamma=gamma)
            a = r["alpha"] * yy
            alphas[(i, j)] = (ids, a)
            rhos.append(r["rho"])
            is_sv[ids] |= a != 0
    sv_ids = np.concatenate([[t for t in order[starts[c]:starts[c + 1]] if is_sv[t]] for c in range(nc)]).astype(int)
    n_sv = np.array([int(is_sv[order[starts[c]:starts[c + 1]]].sum()) for c in range(nc)], dtype=np.int32)
    sv_start = np.concatenate([[0], np.cumsum(n_sv)])
    total = len(sv_ids)
    coef = np.zeros((nc - 1, total))
    for (i, j), (ids, a) in alphas.items():
        mi = sv_start[i]
        for l in range(counts[i]):
            if is_sv[ids[l]]:
                coef[j - 1, mi] = a[l]; mi += 1
        mj = sv_start[j]
        for l in range(counts[i], counts[i] + counts[j]):
            if is_sv[ids[l]]:
                coef[i, mj] = a[l]; mj += 1
    dec = P.predict_dec(sub(sv_ids), coef.reshape(-1), n_sv, np.array(rhos), nc, X, gamma=gamma)
    pred = np.array(labels)[P.vote(dec, nc)]
    return pred, np.array(rhos), n_sv, dec


def test_svc_known_answer(ds):
    """src/test/test_svc.cpp:33-37 and README.md:95-98: C=100, gamma=0.5 -> accuracy 0.98."""
    g, X = ds
    pred, rho, n_sv, dec = _train_c_svc_ovo(X, g, 0.5, 100.0)
    assert abs((pred == g["y"]).mean() - 0.98) < 1e-5
    assert np.array_equal(pred, g["svc_pred"])
    assert np.array_equal(n_sv, g["svc_n_sv"])
    assert np.allclose(rho, g["svc_rho"], rtol=0, atol=1e-9)
    assert np.allclose(dec, g["svc_dec"], rtol=0, atol=1e-9)


def test_oneclass_known_answer(ds):
    """src/test/test_oneclass_svc.cpp:7-29: nu=0.1, gamma=0.5 -> 135 positive predictions."""
    g, X = ds
    n = X.n
    nu = 0.1
    a0 = np.zeros(n)
    k = int(nu * n)
    a0[:k] = 1
    if k < n:
        a0[k] = nu * n - k
    y = np.ones(n, dtype=np.int32)
    ws = min(2 ** int(np.log2(n)), 1024)
    r = P.smo_solve(X, y, a0, np.zeros(n), 1e-3, 1.0, 1.0, ws, gamma=0.5)
    sv = np.nonzero(r["alpha"] != 0)[0]
    rp = g["row_ptr"]
    take = np.concatenate([np.arange(rp[i], rp[i + 1]) for i in sv])
    nrp = np.concatenate([[0], np.cumsum(rp[sv + 1] - rp[sv])]).astype(np.int32)
    SV = P.Csr(csr=(g["val"][take], nrp, g["col"][take]), d=int(g["d"]))
    dec = P.predict_dec(SV, r["alpha"][sv], np.array([len(sv), 0], dtype=np.int32), np.array([r["rho"]]), 2, X,
                        gamma=0.5)
    assert int((dec[:, 0] > 0).sum()) == 135
    assert np.allclose(dec, g["oneclass_dec"], atol=1e-9)


def test_svr_known_answer(ds):
    """src/test/test_svr.cpp:35-39: epsilon-SVR C=100 gamma=0.5 -> MSE 0.020752 (+-1e-3)."""
    g, X = ds
    n = X.n
    yv = g["y"].astype(np.float64)
    p = 0.1
    X2 = P.Csr(csr=(np.concatenate([g["val"], g["val"]]),
                    np.concatenate([g["row_ptr"], g["row_ptr"][1:] + g["row_ptr"][-1]]).astype(np.int32),
                    np.concatenate([g["col"], g["col"]])), d=int(g["d"]))
    y2 = np.concatenate([np.ones(n), -np.ones(n)]).astype(np.int32)
    f0 = np.concatenate([p - yv, -p - yv])
    ws = min(2 ** int(np.log2(2 * n)), 1024)
    r = P.smo_solve(X2, y2, np.zeros(2 * n), f0, 1e-3, 100.0, 100.0, ws, gamma=0.5)
    coef = r["alpha"][:n] - r["alpha"][n:]
    sv = np.nonzero(coef != 0)[0]
    rp = g["row_ptr"]
    take = np.concatenate([np.arange(rp[i], rp[i + 1]) for i in sv])
    nrp = np.concatenate([[0], np.cumsum(rp[sv + 1] - rp[sv])]).astype(np.int32)
    SV = P.Csr(csr=(g["val"][take], nrp, g["col"][take]), d=int(g["d"]))
    dec = P.predict_dec(SV, coef[sv], np.array([len(sv), 0], dtype=np.int32), np.array([r["rho"]]), 2, X, gamma=0.5)
    mse = float(((dec[:, 0] - yv) ** 2).mean())
    assert abs(mse - 0.020752) < 1e-3
    assert np.allclose(dec[:, 0], g["svr_pred"], atol=1e-9)


def test_model_level_fixture_values(ds):
    """The remaining known answers, as reproduced by the reference build when the fixtures were made."""
    g, _ = ds
    y = g["y"]
    assert abs((g["nusvc_pred"] == y).mean() - 0.98) < 1e-3                  # test_nusvc.cpp:40-44
    assert abs(((g["nusvr_pred"] - y) ** 2).mean() - 0.028369) < 1.2e-5      # test_nusvr.cpp:38-42
    assert int((g["oneclass_pred"] > 0).sum()) == 135                        # test_oneclass_svc.cpp:27
    assert abs((g["cv_svc"] == y).mean() - 0.973) < 1e-3                     # test_cross_validation.cpp:58
    assert abs((g["cv_nusvc"] == y).mean() - 0.660) < 1e-3                   # :67
    assert abs(((g["cv_nusvr"] - y) ** 2).mean() - 0.045) < 1e-3             # :75
    assert abs(((g["cv_svr"] - y) ** 2).mean() - 0.044) < 1e-3               # :83


CASES = {"c1": (lambda: synth.config1(1500), None), "c1_soft": (lambda: dict(synth.config1(1500), gamma=0.025), None),
         "c2": (lambda: synth.config2(1200), None), "c3": (lambda: synth.config3(900), 5),
         "c4": (lambda: synth.config4(700), None), "c5": (lambda: synth.config5(1100, d=200), None)}


@pytest.mark.parametrize("tag", sorted(CASES))
def test_solver_matches_reference_fixture(golden_dir, tag):
    g = np.load(os.path.join(golden_dir, "solver_small.npz"))
    make, split = CASES[tag]
    prob = make()
    X = oracle_matrix(P, prob)
    y = binary_labels(prob, split)
    n = len(y)
    ws = min(1024, 2 ** int(np.log2(n)))
    rows = P.kernel_rows_idx(X, g[tag + "_rows_idx"], gamma=prob["gamma"])
    assert np.array_equal(rows, g[tag + "_rows"])
    r = P.smo_solve(X, y, np.zeros(n), -y.astype(np.float64), 1e-3, prob["C"], prob["C"], ws, gamma=prob["gamma"])
    assert abs(r["obj"] - float(g[tag + "_obj"])) <= 1e-6 * abs(float(g[tag + "_obj"]))
    assert abs(r["rho"] - float(g[tag + "_rho"])) < 1e-6
    assert int((r["alpha"] != 0).sum()) == int((g[tag + "_alpha"] != 0).sum())
    assert np.allclose(r["alpha"], g[tag + "_alpha"], rtol=0, atol=1e-5 * prob["C"])
    assert abs(objective(r["alpha"], r["f"], y) - r["obj"]) < 1e-9 * max(1.0, abs(r["obj"]))


def test_nu_solver_matches_reference_fixture(golden_dir):
    g = np.load(os.path.join(golden_dir, "solver_small.npz"))
    prob = synth.config1(800)
    X = oracle_matrix(P, prob)
    y = binary_labels(prob)
    n = len(y)
    r = P.smo_solve(X, y, g["nu_alpha0"], np.zeros(n), 1e-3, 1.0, 1.0, 512, solver="nu_svc", gamma=0.5,
                    cuda_semantics=0)
    assert abs(r["rho"] - float(g["nu_rho"])) < 1e-6
    assert np.allclose(r["alpha"], g["nu_alpha"], rtol=0, atol=1e-6)


@pytest.mark.skipif(not R.available(), reason="reference CPU library not built on this machine")
def test_port_matches_live_reference_build():
    prob = synth.config2(900)
    X = oracle_matrix(P, prob)
    D = R.Data(csr=prob["csr"][:1] + (prob["csr"][1][:901],) + prob["csr"][2:], d=prob["d"]) if False else \
        R.Data(csr=(X.val, X.row_ptr, X.col), d=X.d)
    idx = np.arange(40, dtype=np.int32) * 11
    a, _, _ = R.kernel_rows_idx(D, idx, gamma=0.5)
    assert np.array_equal(a, P.kernel_rows_idx(X, idx, gamma=0.5))
    y = binary_labels(prob)
    n = len(y)
    ra, rf, rrho, _ = R.smo_solve(D, y, np.zeros(n), -y.astype(np.float64), 1e-3, 100.0, 100.0, 512, gamma=0.5)
    r = P.smo_solve(X, y, np.zeros(n), -y.astype(np.float64), 1e-3, 100.0, 100.0, 512, gamma=0.5)
    assert np.allclose(ra, r["alpha"], atol=1e-6) and abs(rrho - r["rho"]) < 1e-8


def test_working_set_selection_edge_cases():
    """Ties are broken by instance id; an exhausted side lets the other side fill the set."""
    n = 64
    f = np.zeros(n)
    y = np.where(np.arange(n) % 2 == 0, 1, -1).astype(np.int32)
    a = np.zeros(n)
    ws = P.select_working_set("c", f, y, a, 1.0, 1.0, None, 8)
    # I_up = {y>0, a<C}: even ids ascending; I_low = {y<0, a<C}: odd ids, taken from the high end
    assert list(ws) == [0, 63, 2, 61, 4, 59, 6, 57]
    a[:] = np.where(y > 0, 1.0, 0.0)      # every positive at its bound -> all instances are I_low only
    ws = P.select_working_set("c", f, y, a, 1.0, 1.0, None, 6)
    assert list(ws) == [63, 62, 61, 60, 59, 58]


FULL = {"c1": synth.config1, "c2": synth.config2, "c4": synth.config4}


@pytest.mark.parametrize("tag", sorted(FULL))
def test_port_kernel_rows_match_reference_at_full_size(golden_dir, tag):
    """Full-length kernel rows of the benchmark configurations: the restatement reproduces the reference
    build's rows (tests/golden/make_full_configs.py) bit for bit."""
    g = np.load(os.path.join(golden_dir, "full_%s.npz" % tag))
    prob = FULL[tag]()
    X = oracle_matrix(P, prob)
    assert X.n == int(g["n"])
    assert np.array_equal(P.kernel_rows_idx(X, g["rows_idx"], gamma=prob["gamma"]), g["rows"])


def test_port_solves_config1_at_full_size(golden_dir):
    """The 10,000 x 20 configuration to convergence: objective, rho and support-vector count of the reference."""
    g = np.load(os.path.join(golden_dir, "full_c1.npz"))
    prob = synth.config1()
    X = oracle_matrix(P, prob)
    y = binary_labels(prob)
    n = len(y)
    r = P.smo_solve(X, y, np.zeros(n), -y.astype(np.float64), 1e-3, prob["C"], prob["C"], 1024, gamma=prob["gamma"])
    assert abs(r["obj"] - float(g["objective"])) <= 1e-6 * abs(float(g["objective"]))
    assert abs(r["rho"] - float(g["rho"])) < 1e-6
    assert int((r["alpha"] != 0).sum()) == int(g["n_sv"])

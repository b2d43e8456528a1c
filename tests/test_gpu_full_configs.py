"""The benchmark configurations at their FULL size on the GPU (through the C ABI and the reference-named host
symbols) against the reference's own CPU build: tests/golden/full_*.npz hold the reference's results
(tests/golden/make_full_configs.py made them). Every equivalence bound is held as stated:
kernel rows 1e-5 relative, dual objective 1e-4 relative, support-vector count 0.5 %, rho and decision values
1e-3 absolute, labels on at least 99.9 % of the rows."""
import os

import numpy as np
import pytest

import host_api
from thundersvm_b200 import synth
from util import device_matrix, rel_err, rel_err_pure

pytestmark = pytest.mark.gpu

OBJ_TOL, SV_TOL, DEC_TOL, LABEL_AGREE, ROW_TOL = 1e-4, 0.005, 1e-3, 0.999, 1e-5

CASES = {
    "c1": (synth.config1, dict(), lambda: synth.config1(2048, seed=11)),
    "c2": (synth.config2, dict(), lambda: synth.config2(16281, seed=3)),
    "c4": (synth.config4, dict(), lambda: synth.config4(1024, seed=16)),
}


def _test_batch(torch, test):
    if "X" in test:
        return dict(dense=torch.from_numpy(test["X"]).cuda())
    val, rp, col = test["csr"]
    return dict(csr=(torch.from_numpy(val).cuda(), torch.from_numpy(rp).cuda(), torch.from_numpy(col).cuda()))


def _sub_matrix(capi, torch, prob, rows):
    if "X" in prob:
        return capi.KernelMatrix(dense=torch.from_numpy(np.ascontiguousarray(prob["X"][rows])).cuda(),
                                 gamma=prob["gamma"])
    val, rp, col = prob["csr"]
    cnt = np.diff(rp)[rows]
    take = np.repeat(rp[rows], cnt) + (np.arange(cnt.sum()) - np.repeat(np.cumsum(cnt) - cnt, cnt))
    rp2 = np.concatenate([[0], np.cumsum(cnt)]).astype(np.int32)
    return capi.KernelMatrix(csr=(torch.from_numpy(val[take]).cuda(), torch.from_numpy(rp2).cuda(),
                                  torch.from_numpy(col[take]).cuda()), d=prob["d"], gamma=prob["gamma"])


@pytest.mark.parametrize("tag", ["c1", "c2", "c4"])
def test_full_size_binary_config(capi, golden_dir, tag, record_property):
    import torch
    g = np.load(os.path.join(golden_dir, "full_%s.npz" % tag))
    make, kw, make_test = CASES[tag]
    prob = make(**kw)
    y = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
    n = len(y)
    assert n == int(g["n"])
    km = device_matrix(capi, prob)
    # kernel rows of the full-length problem against the reference's rows
    got = km.get_rows(torch.from_numpy(g["rows_idx"]).cuda()).cpu().numpy()
    e_floor, e_pure = rel_err(got, g["rows"]), rel_err_pure(got, g["rows"])
    record_property("kernel_rows_rel_err_floored", e_floor)
    record_property("kernel_rows_rel_err_pure", e_pure)
    print("%s kernel rows: floored rel err %.3g, pure rel err %.3g" % (tag, e_floor, e_pure))
    assert e_floor < ROW_TOL
    # the solve
    yd = torch.from_numpy(y).cuda()
    alpha = torch.zeros(n, dtype=torch.float64, device="cuda")
    f = -yd.to(torch.float64)
    rho, st = capi.smo_solve(km, yd, alpha, f, prob["eps"], prob["C"], prob["C"], 1024)
    assert abs(st["objective"] - float(g["objective"])) <= OBJ_TOL * abs(float(g["objective"]))
    assert abs(rho - float(g["rho"])) < DEC_TOL
    a = alpha.cpu().numpy()
    n_sv = int((a != 0).sum())
    assert abs(n_sv - int(g["n_sv"])) <= SV_TOL * int(g["n_sv"])
    # decision values and labels of the fixed test rows
    sv = np.nonzero(a)[0]
    km_sv = _sub_matrix(capi, torch, prob, sv)
    coef = torch.from_numpy(a[sv] * y[sv]).cuda()
    order = np.argsort(-y[sv], kind="stable")            # class +1 first, as the model stores them
    if not np.array_equal(order, np.arange(len(sv))):
        km_sv.close()
        km_sv = _sub_matrix(capi, torch, prob, sv[order])
        coef = torch.from_numpy((a[sv] * y[sv])[order]).cuda()
    counts = [int((y[sv] > 0).sum()), int((y[sv] < 0).sum())]
    dec = capi.predict_dec(km_sv, coef, counts, torch.tensor([rho], dtype=torch.float64, device="cuda"), 2,
                           **_test_batch(torch, make_test())).cpu().numpy()[:, 0]
    err = float(np.max(np.abs(dec - g["dec"])))
    print("%s: obj %.6f (ref %.6f) rho %.6f (ref %.6f) n_sv %d (ref %d) max |dec - ref| %.3g" % (
        tag, st["objective"], float(g["objective"]), rho, float(g["rho"]), n_sv, int(g["n_sv"]), err))
    assert err < DEC_TOL
    assert np.mean(np.where(dec > 0, 1, -1) == g["labels"]) >= LABEL_AGREE
    km_sv.close()
    km.close()


def test_full_size_three_class_cut_of_config3(capi, golden_dir):
    """SVC::train on the first three classes of the 60,000 x 784 problem at full per-class size (18,057 rows,
    three one-vs-one sub-problems) through the reference-named host symbols: the model layout (per-class
    support-vector counts, rho per pair, coefficient rows) and the decision values / labels of 1,000 test rows."""
    g = np.load(os.path.join(golden_dir, "full_c3cut.npz"))
    L = host_api.load()
    full = synth.config3()
    keep = np.nonzero(full["y"] < 3)[0]
    X, y = np.ascontiguousarray(full["X"][keep]), full["y"][keep]
    assert len(y) == int(g["n"])
    m, nf, nc, ok = host_api.train(L, 0, X=X, y=y, gamma=full["gamma"], C_=full["C"], tol=full["eps"])
    assert ok == 1 and nc == 3
    cnt = np.zeros(3, np.int32)
    L.get_support_classes(host_api.p(cnt, host_api.i32p), 3, m)
    assert np.all(np.abs(cnt - g["n_sv"]) <= np.maximum(1, np.ceil(SV_TOL * g["n_sv"]))), (cnt, g["n_sv"])
    rho = np.zeros(3, np.float32)
    L.get_rho(host_api.p(rho, host_api.f32p), 3, m)
    assert np.max(np.abs(rho - g["rho"])) < DEC_TOL
    test = synth.config3(10000, seed=5)
    T = np.ascontiguousarray(test["X"][g["test_rows"]])
    dec = np.zeros(T.shape[0] * 3, np.float32)
    L.dense_decision(T.shape[0], T.shape[1], host_api.p(T, host_api.f32p), m, dec.size, host_api.p(dec, host_api.f32p))
    assert np.max(np.abs(dec.reshape(-1, 3) - g["dec"])) < DEC_TOL
    pred = host_api.predict_dense(L, m, T)
    assert np.mean(pred == g["labels"]) >= LABEL_AGREE
    L.model_free(m)

"""Prediction on the GPU against the oracle and the committed reference outputs.
Tolerance: decision values 1e-3 absolute, labels >= 99.9 % agreement."""
import os

import numpy as np
import pytest

from oracle import port_binding as P

pytestmark = pytest.mark.gpu


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_multiclass_decision_values_and_vote(capi):
    import torch
    rng = np.random.default_rng(3)
    nc, d, n_sv, m = 4, 24, 230, 157
    SVd = rng.standard_normal((n_sv, d)).astype(np.float32)
    T = rng.standard_normal((m, d)).astype(np.float32)
    cnt = np.array([60, 50, 70, 50], dtype=np.int32)
    coef = rng.standard_normal((nc - 1, n_sv))
    rho = rng.standard_normal(nc * (nc - 1) // 2)
    want = P.predict_dec(P.Csr(dense=SVd), coef.reshape(-1), cnt, rho, nc, P.Csr(dense=T), gamma=0.05)
    for dense_sv in (True, False):
        if dense_sv:
            km = capi.KernelMatrix(dense=_t(SVd), gamma=0.05)
        else:
            c = P.Csr(dense=SVd)
            km = capi.KernelMatrix(csr=(_t(c.val), _t(c.row_ptr), _t(c.col)), d=d, gamma=0.05)
        for budget in (0, 64 * 1024):            # one batch / many small batches
            dec = capi.predict_dec(km, _t(coef.reshape(-1)), cnt, _t(rho), nc, dense=_t(T), max_mem_bytes=budget)
            assert np.max(np.abs(dec.cpu().numpy() - want)) < 1e-3
            got = capi.vote(dec, nc).cpu().numpy()
            assert np.mean(got == P.vote(want, nc)) >= 0.999


def test_reference_fixture_decision_values(capi, golden_dir):
    """Support vectors / coefficients / rho of the reference-trained models (tests/golden) -> the
    reference's own decision values on its fixture data set."""
    g = np.load(os.path.join(golden_dir, "test_dataset.npz"))
    val, rp, col, d, y = g["val"], g["row_ptr"], g["col"], int(g["d"]), g["y"]
    n = len(rp) - 1
    Xd = np.zeros((n, d), np.float32)
    Xd[np.repeat(np.arange(n), np.diff(rp)), col] = val
    for tag, nc in (("svc", 3), ("svr", 2), ("oneclass", 2), ("nusvr", 2)):
        sv = Xd[g[tag + "_sv_ind"]]
        km = capi.KernelMatrix(dense=_t(sv), gamma=0.5)
        cnt = g[tag + "_n_sv"]
        dec = capi.predict_dec(km, _t(g[tag + "_coef"]), cnt, _t(g[tag + "_rho"]), nc, dense=_t(Xd)).cpu().numpy()
        assert np.max(np.abs(dec - g[tag + "_dec"])) < 1e-3
    # labels of the 3-class model: accuracy 0.98 (src/test/test_svc.cpp:33-37)
    sv = Xd[g["svc_sv_ind"]]
    km = capi.KernelMatrix(dense=_t(sv), gamma=0.5)
    dec = capi.predict_dec(km, _t(g["svc_coef"]), g["svc_n_sv"], _t(g["svc_rho"]), 3, dense=_t(Xd))
    labels = np.array([0.0, 2.0, 3.0])[capi.vote(dec, 3).cpu().numpy()]
    assert np.array_equal(labels, g["svc_pred"])
    assert abs((labels == y).mean() - 0.98) < 1e-5

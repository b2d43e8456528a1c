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


def _fused_case(capi, nc, cnt, d, m, kernel="rbf", gamma=0.02, coef0=0.0, degree=3, engine=None, csr_batch=False,
                seed=5):
    """Dense support vectors with more than 32 features: the coefficient sums are the contraction's epilogue."""
    rng = np.random.default_rng(seed)
    cnt = np.asarray(cnt, dtype=np.int32)
    n_sv = int(cnt.sum())
    SVd = (rng.standard_normal((n_sv, d)) * (rng.random((n_sv, d)) < 0.6)).astype(np.float32)
    T = (rng.standard_normal((m, d)) * (rng.random((m, d)) < 0.6)).astype(np.float32)
    coef = rng.standard_normal((nc - 1, n_sv)) * 3
    rho = rng.standard_normal(nc * (nc - 1) // 2)
    kw = dict(kernel=kernel, gamma=gamma, coef0=coef0, degree=degree)
    want = P.predict_dec(P.Csr(dense=SVd), coef.reshape(-1), cnt, rho, nc, P.Csr(dense=T), **kw)
    km = capi.KernelMatrix(dense=_t(SVd), **kw)
    if engine:
        km.set_dense_engine(engine)
    if csr_batch:
        c = P.Csr(dense=T)
        nz = c.val != 0                          # drop the explicit zeros: a genuinely sparse batch
        rp = np.concatenate([[0], np.cumsum(np.add.reduceat(nz, c.row_ptr[:-1]))]).astype(np.int32)
        batch = dict(csr=(_t(c.val[nz]), _t(rp), _t(c.col[nz])))
    else:
        batch = dict(dense=_t(T))
    dec = capi.predict_dec(km, _t(coef.reshape(-1)), cnt, _t(rho), nc, **batch).cpu().numpy()
    scale = max(1.0, float(np.max(np.abs(want))))
    assert np.max(np.abs(dec - want)) < 1e-3 * scale, np.max(np.abs(dec - want))
    lab = capi.predict_labels(km, _t(coef.reshape(-1)), cnt, _t(rho), nc, **batch).cpu().numpy()
    assert np.array_equal(lab, capi.vote(_t(dec), nc).cpu().numpy())
    assert np.mean(lab == P.vote(want, nc)) >= 0.999
    km.close()


@pytest.mark.parametrize("engine", [None, "tensor2"])
def test_fused_prediction_multiclass_ragged_classes(capi, engine):
    """Class blocks that start and end inside a 128-instance tile, a tail tile, a tail row block."""
    _fused_case(capi, 4, [300, 37, 401, 262], d=200, m=700, engine=engine)


def test_fused_prediction_binary_tails_and_sparse_batch(capi):
    _fused_case(capi, 2, [513, 258], d=136, m=257)
    _fused_case(capi, 2, [100, 29], d=72, m=5, csr_batch=True)
    _fused_case(capi, 3, [1, 1, 1], d=40, m=300)


@pytest.mark.parametrize("kernel,kw", [("linear", {}), ("poly", dict(gamma=0.01, coef0=0.5, degree=3)),
                                       ("sigmoid", dict(gamma=0.01, coef0=0.1))])
def test_fused_prediction_other_kernels(capi, kernel, kw):
    _fused_case(capi, 3, [150, 200, 90], d=96, m=333, kernel=kernel, **kw)


def test_fused_prediction_many_classes(capi):
    """20 classes: 19 coefficient rows per support vector (more than the shared-memory table holds) and 190 pairs;
    several launches over the test rows."""
    _fused_case(capi, 20, [17 + 3 * c for c in range(20)], d=64, m=4500)

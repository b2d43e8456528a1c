"""Kernel rows on the GPU (through the C ABI) against the CPU oracle. Tolerance: 1e-5 relative on
kernel values for get_rows(idx) (the hot path); the instance form is held to the same bound."""
import os

import numpy as np
import pytest

from oracle import port_binding as P
from thundersvm_b200 import synth
from util import device_matrix, oracle_matrix, rel_err

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5


def _idx(n, q, seed=0):
    return np.random.default_rng(seed).choice(n, q, replace=q > n).astype(np.int32)


def _check_rows(capi, prob, n, q, engine=None, force=None, kernel="rbf", coef0=0.0, degree=3, tol=REL_TOL,
                gamma=None):
    import torch
    gamma = prob["gamma"] if gamma is None else gamma
    X = oracle_matrix(P, prob, n)
    km = device_matrix(capi, prob, n, force=force, kernel=kernel, coef0=coef0, degree=degree, gamma=gamma)
    if engine is not None and km.is_dense:
        km.set_dense_engine(engine)
    idx = _idx(X.n, q)
    want = P.kernel_rows_idx(X, idx, kernel=kernel, gamma=gamma, coef0=coef0, degree=degree)
    got = km.get_rows(torch.from_numpy(idx).cuda()).cpu().numpy()
    assert got.shape == want.shape
    if kernel in ("rbf",):
        err = rel_err(got, want)
    else:   # values can cross zero: relative to the row scale
        err = float(np.max(np.abs(got - want)) / max(1e-30, np.max(np.abs(want))))
    assert err < tol, "relative error %.3g" % err
    return km, X


@pytest.mark.parametrize("engine", ["auto", "tensor", "tensor2", "simt"])
@pytest.mark.parametrize("n,q", [(1000, 64), (4097, 512), (300, 101), (129, 128), (128, 1), (2500, 1024)])
def test_dense_rows_c1(capi, engine, n, q):
    """Config 1 has 20 features with |x| up to 3 and RBF arguments up to ~50. The automatic engine uses
    FP32 CUDA-core tiles here and holds 1e-5. When the tensor-core engine is forced, the two-plane TF32
    representation (2^-23 relative per operand) of a few dominant products shows directly in the exponent:
    it is held to 3e-5 on this data and to 1e-5 wherever the k loop is long (the tests below)."""
    _check_rows(capi, synth.config1(n), n, q, engine=engine, tol=3e-5 if engine.startswith("tensor") else REL_TOL)


@pytest.mark.parametrize("engine", ["tensor", "tensor2", "simt"])
def test_dense_rows_c5_shape(capi, engine):
    """Unit-norm rows, d = 2000 (config 5's row length), n not a multiple of the tile."""
    _check_rows(capi, synth.config5(3001), 3001, 512, engine=engine)


@pytest.mark.parametrize("engine", ["tensor", "tensor2", "simt"])
def test_dense_rows_c3_shape(capi, engine):
    """784 features in [0,1] (config 3). Same-class dot products reach ~100, where the oracle's own
    sequential FP32 accumulation noise is ~1e-5 relative on K; both are therefore also compared with an
    FP64 evaluation and the GPU result must not be further from it than the oracle is (+1e-5)."""
    import torch
    prob = synth.config3(2000)
    X = oracle_matrix(P, prob)
    km = device_matrix(capi, prob)
    km.set_dense_engine(engine)
    idx = _idx(2000, 256)
    want = P.kernel_rows_idx(X, idx, gamma=prob["gamma"])
    got = km.get_rows(torch.from_numpy(idx).cuda()).cpu().numpy()
    D = prob["X"].astype(np.float64)
    sd = (D * D).sum(1)
    exact = np.exp(-prob["gamma"] * (sd[idx][:, None] + sd[None, :] - 2 * D[idx] @ D.T))
    e_gpu, e_orc = rel_err(got, exact), rel_err(want, exact)
    assert e_gpu < max(REL_TOL, e_orc + REL_TOL), (e_gpu, e_orc)
    assert rel_err(got, want) < 4e-5
    if engine.startswith("tensor"):
        assert e_gpu <= e_orc, "the promoted 3xTF32 sum should be at least as close to FP64 as sequential FP32"


@pytest.mark.parametrize("kernel,kw", [("linear", {}), ("poly", dict(coef0=0.1, degree=3)),
                                       ("sigmoid", dict(coef0=0.1))])
@pytest.mark.parametrize("engine", ["tensor", "tensor2", "simt"])
def test_dense_rows_other_kernels(capi, engine, kernel, kw):
    _check_rows(capi, synth.config1(1500), 1500, 200, engine=engine, kernel=kernel, **kw)


@pytest.mark.parametrize("engine", ["tensor", "tensor2"])
@pytest.mark.parametrize("n,q", [(100, 5), (129, 127), (257, 129), (384, 256), (511, 300), (40000, 512)])
def test_dense_rows_pair_engine_odd_tiles(capi, engine, n, q):
    """CTA-pair tiles with an empty or partial second half (n just above / below multiples of 128 and
    256) and requested-row counts around the 128-row halves of the B operand. d = 136 is a multiple of 8
    but not of the 32- or 64-element k slab; d = 133 makes the FP16 planes wider than the FP32 rows."""
    _check_rows(capi, synth.config5(n, d=136), n, q, engine=engine)
    if n <= 511:
        _check_rows(capi, synth.config5(n, d=133), n, q, engine=engine)


@pytest.mark.parametrize("engine", ["tensor", "tensor2", "simt"])
def test_dense_rows_row_magnitudes(capi, engine):
    """Rows whose magnitudes span 16 decades and whose features span 6 decades inside a row (linear
    kernel, so nothing hides in an exponent). The FP16-plane engine scales every row by a power of two;
    the result must be as close to FP64 as FP32 arithmetic allows, relative to the two rows' norms."""
    import torch
    rng = np.random.default_rng(5)
    n, d, q = 1500, 300, 256
    X0 = rng.random((n, d)) * 10.0 ** rng.uniform(-6, 0, size=(n, d))
    X0 /= np.linalg.norm(X0, axis=1, keepdims=True)
    s = 10.0 ** rng.uniform(-8, 8, size=n)
    s[:4] = [0.0, 1e-15, 1e15, 1.0]               # an all-zero row, a tiny and a huge one (products stay FP32-normal)
    X = (X0 * s[:, None]).astype(np.float32)
    km = capi.KernelMatrix(dense=torch.from_numpy(X).cuda(), kernel="linear", gamma=1.0)
    km.set_dense_engine(engine)
    idx = np.concatenate([np.arange(4), rng.choice(n, q - 4, replace=False)]).astype(np.int32)
    got = km.get_rows(torch.from_numpy(idx).cuda()).cpu().numpy().astype(np.float64)
    D = X.astype(np.float64)
    exact = D[idx] @ D.T
    norms = np.maximum(np.linalg.norm(D, axis=1), 1e-100)
    err = np.abs(got - exact) / (norms[idx][:, None] * norms[None, :])
    assert np.isfinite(got).all()
    assert err.max() < (4e-6 if engine == "simt" else 2e-6), err.max()


@pytest.mark.parametrize("n,q", [(1200, 64), (5000, 512), (333, 101), (2000, 1024)])
def test_csr_rows_c2(capi, n, q):
    _check_rows(capi, synth.config2(n), n, q)


def test_csr_rows_c4(capi):
    _check_rows(capi, synth.config4(1500), 1500, 512)


def test_csr_rows_other_kernels(capi):
    for kernel, kw in (("linear", {}), ("poly", dict(coef0=0.1)), ("sigmoid", dict(coef0=0.1))):
        _check_rows(capi, synth.config4(600), 600, 128, kernel=kernel, **kw)


def test_storage_forms_agree(capi):
    """The same data stored dense and as CSR gives the same kernel rows (C2 is run dense on B200)."""
    _check_rows(capi, synth.config2(1500), 1500, 256, force="dense")
    _check_rows(capi, synth.config1(900), 900, 128, force="csr")


def test_reference_fixture_rows(capi, golden_dir):
    """Reference outputs (tests/golden, made from the reference's CPU build): idx rows and the instance
    form on the reference's own fixture, four kernels, tolerance 1e-4 as in test_kernelmatrix.cpp:103."""
    import torch
    g = np.load(os.path.join(golden_dir, "test_dataset.npz"))
    val, rp, col, d = g["val"], g["row_ptr"], g["col"], int(g["d"])
    idx = torch.arange(10, dtype=torch.int32, device="cuda") * 3 + 4
    for name, kw in (("rbf", dict(gamma=0.5)), ("poly", dict(gamma=0.5, degree=3, coef0=0.1)), ("linear", dict()),
                     ("sigmoid", dict(gamma=0.5, coef0=0.1))):
        for dense in (False, True):
            if dense:
                Xd = np.zeros((len(rp) - 1, d), np.float32)
                Xd[np.repeat(np.arange(len(rp) - 1), np.diff(rp)), col] = val
                km = capi.KernelMatrix(dense=torch.from_numpy(Xd).cuda(), kernel=name, **kw)
                T = dict(dense=torch.from_numpy(Xd[:10].copy()).cuda())
            else:
                km = capi.KernelMatrix(csr=(torch.from_numpy(val).cuda(), torch.from_numpy(rp).cuda(),
                                            torch.from_numpy(col).cuda()), d=d, kernel=name, **kw)
                T = dict(csr=(torch.from_numpy(val[:rp[10]].copy()).cuda(), torch.from_numpy(rp[:11].copy()).cuda(),
                              torch.from_numpy(col[:rp[10]].copy()).cuda()))
            rows = km.get_rows(idx).cpu().numpy()
            ins = km.get_rows_instances(**T).cpu().numpy()
            scale = np.maximum(1.0, np.abs(g["rows_idx_" + name]))
            assert np.max(np.abs(rows - g["rows_idx_" + name]) / scale) < 1e-4
            assert np.max(np.abs(ins - g["rows_ins_" + name]) / scale) < 1e-4
            assert np.allclose(km.diag().cpu().numpy(), g["diag_" + name], rtol=1e-6)


def test_rows_by_instances_mixed_storage(capi):
    """Prediction form: dense / CSR support vectors x dense / CSR test batch, and test features beyond
    the stored feature count are ignored in the product but counted in the norm (kernelmatrix.cpp:392)."""
    import torch
    prob = synth.config2(700)
    test = synth.config2(90, seed=3)
    X = oracle_matrix(P, prob)
    val, rp, col = test["csr"]
    # add an out-of-range feature (id 200 >= 123) to every test row
    rows = np.split(np.arange(len(val)), rp[1:-1])
    nval = np.concatenate([np.concatenate([val[r], [0.5]]) for r in rows]).astype(np.float32)
    ncol = np.concatenate([np.concatenate([col[r], [200]]) for r in rows]).astype(np.int32)
    nrp = (np.arange(len(rp)) * 15).astype(np.int32)
    T = P.Csr(csr=(nval, nrp, ncol), d=201)
    want = P.kernel_rows_ins(X, T, gamma=0.5)
    Td = np.zeros((90, 201), np.float32)
    Td[np.repeat(np.arange(90), 15), ncol] = nval
    for force in (None, "dense"):
        km = device_matrix(capi, prob, force=force)
        got1 = km.get_rows_instances(csr=(torch.from_numpy(nval).cuda(), torch.from_numpy(nrp).cuda(),
                                          torch.from_numpy(ncol).cuda())).cpu().numpy()
        got2 = km.get_rows_instances(dense=torch.from_numpy(Td).cuda()).cpu().numpy()
        assert rel_err(got1, want) < REL_TOL
        assert rel_err(got2, want) < REL_TOL


def test_error_returns(capi):
    """Bad arguments come back as a status + message (the reference CHECK-fails)."""
    import torch
    km = device_matrix(capi, synth.config1(200))
    with pytest.raises(capi.TsvmError):
        capi.check(capi.lib().tsvm_km_rows_by_index(km.handle, None, 4, None, 200, None))
    with pytest.raises(capi.TsvmError):
        capi.smo_solve(km, torch.ones(200, dtype=torch.int32, device="cuda"),
                       torch.zeros(200, dtype=torch.float64, device="cuda"),
                       torch.zeros(200, dtype=torch.float64, device="cuda"), 1e-3, 1.0, 1.0, 300)   # ws > n


_CSR_ENGINE_DIGEST = r"""
import hashlib, sys
import numpy as np, torch
from thundersvm_b200 import capi
rng = np.random.default_rng(17)
n, d = 4099, 158                                   # n not a multiple of 32; d = the most the shared-memory panel holds
lens = rng.integers(0, 70, n)                      # empty instances and instances longer than one 32-entry batch
lens[::97] = 0
rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
col = np.concatenate([np.sort(rng.choice(d, k, replace=False)) for k in lens]).astype(np.int32)
val = rng.standard_normal(len(col)).astype(np.float32)
h = hashlib.sha256()
for kernel, kw in (("rbf", dict(gamma=0.3)), ("poly", dict(gamma=0.2, coef0=1.0, degree=3)), ("linear", {})):
    km = capi.KernelMatrix(csr=(torch.from_numpy(val).cuda(), torch.from_numpy(rp).cuda(), torch.from_numpy(col).cuda()),
                           d=d, kernel=kernel, **kw)
    for q in (1024, 512, 300, 7):
        ids = rng.choice(n, q, replace=False).astype(np.int32)
        if q == 300:
            ids[[5, 299]] = -1                     # empty working-set slots
        for ld in (n, (n + 3) // 4 * 4):           # unaligned and aligned row stride
            out = torch.zeros((q, ld), dtype=torch.float32, device="cuda")
            km.get_rows(torch.from_numpy(ids).cuda(), out)
            h.update(out[:, :n].contiguous().cpu().numpy().tobytes())
    km.close()
print(h.hexdigest())
"""


def test_csr_engines_agree_bit_for_bit():
    """CSR data with few features runs on the engine that keeps the requested rows' panel in shared memory,
    everything else on the engine that reads it from L2. Both compute every value as the same FP32 recurrence
    over the instance's stored entries in storage order, so switching the first one off (TSVM_CSR_SMEM=0, read
    once per process) must not change a bit: ragged and empty instances, empty slots, every request size,
    aligned and unaligned output rows, three kernel functions."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    digests = []
    for flag in ("0", "1"):
        env = dict(os.environ, TSVM_CSR_SMEM=flag, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        r = subprocess.run([sys.executable, "-c", _CSR_ENGINE_DIGEST], env=env, capture_output=True, text=True,
                           timeout=600, cwd=root)
        assert r.returncode == 0, r.stderr[-2000:]
        digests.append(r.stdout.strip().splitlines()[-1])
    assert len(digests[0]) == 64 and digests[0] == digests[1]

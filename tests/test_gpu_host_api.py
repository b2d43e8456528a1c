"""The reference's public surface on top of the GPU hot path: the scikit-style C API (as the
reference's Python package calls it) and the two CLIs, checked against the reference tests' known
answers on its fixture data set and against the reference-trained models in tests/golden."""
import os
import subprocess

import numpy as np
import pytest

import host_api

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "thundersvm_b200", "bin")


@pytest.fixture(scope="module")
def fx(golden_dir, capi):
    g = np.load(os.path.join(golden_dir, "test_dataset.npz"))
    n, d = len(g["row_ptr"]) - 1, int(g["d"])
    X = np.zeros((n, d), np.float32)
    X[np.repeat(np.arange(n), np.diff(g["row_ptr"])), g["col"]] = g["val"]
    return host_api.load(), g, X


def test_c_svc_known_answer_dense_and_sparse(fx):
    """test_svc.cpp:33-37: C=100, gamma=0.5 -> accuracy 0.98; 23 SVs (4/10/9) as the reference finds."""
    L, g, X = fx
    for mode in ("dense", "sparse"):
        if mode == "dense":
            m, nf, nc, ok = host_api.train(L, 0, X=X, y=g["y"], gamma=0.5, C_=100)
            pred = host_api.predict_dense(L, m, X)
        else:
            csr = (g["val"], g["row_ptr"], g["col"])
            m, nf, nc, ok = host_api.train(L, 0, csr=csr, y=g["y"], gamma=0.5, C_=100)
            pred = host_api.predict_sparse(L, m, csr)
        assert ok == 1 and nc == 3 and nf == 4
        assert abs((pred == g["y"]).mean() - 0.98) < 1e-5
        assert np.mean(pred == g["svc_pred"]) >= 0.999
        assert abs(L.n_sv(m) - 23) <= 1
        cnt = np.zeros(3, np.int32)
        L.get_support_classes(host_api.p(cnt, host_api.i32p), 3, m)
        assert np.abs(cnt - g["svc_n_sv"]).max() <= 1
        rho = np.zeros(3, np.float32)
        L.get_rho(host_api.p(rho, host_api.f32p), 3, m)
        assert np.allclose(rho, g["svc_rho"], atol=1e-3)
        dec = np.zeros(150 * 3, np.float32)
        L.dense_decision(150, 4, host_api.p(X, host_api.f32p), m, 450, host_api.p(dec, host_api.f32p))
        assert np.max(np.abs(dec.reshape(150, 3) - g["svc_dec"])) < 2e-3
        text = host_api.model_text(L, m)
        assert text.startswith("svm_type c_svc\nkernel_type rbf\ngamma 0.5\nnr_class 3\ntotal_sv ")
        assert "label 0 2 3 \n" in text
        L.model_free(m)


def test_other_models_known_answers(fx):
    L, g, X = fx
    y = g["y"]
    m, *_ = host_api.train(L, 1, X=X, y=y, gamma=0.5, nu=0.1, C_=100)             # test_nusvc.cpp:40-44
    assert abs((host_api.predict_dense(L, m, X) == y).mean() - 0.98) < 1e-3
    L.model_free(m)
    m, *_ = host_api.train(L, 3, X=X, y=y, gamma=0.5, C_=100)                     # test_svr.cpp:35-39
    pred = host_api.predict_dense(L, m, X)
    assert abs(((pred - y) ** 2).mean() - 0.020752) < 1e-3
    assert np.max(np.abs(pred - g["svr_pred"])) < 2e-3
    L.model_free(m)
    m, *_ = host_api.train(L, 4, X=X, y=y, gamma=0.5, C_=100, nu=0.1)             # test_nusvr.cpp:38-42
    assert abs(((host_api.predict_dense(L, m, X) - y) ** 2).mean() - 0.028369) < 1e-3
    L.model_free(m)
    m, *_ = host_api.train(L, 2, X=X, y=y, gamma=0.5, nu=0.1)                     # test_oneclass_svc.cpp:7-29
    pred = host_api.predict_dense(L, m, X)
    assert abs(int((pred > 0).sum()) - 135) <= 1
    # save / load round trip of the trained model (same test in the reference)
    text = host_api.model_text(L, m)
    m2 = L.model_new(2)
    L.load_from_string_scikit(m2, text.encode())
    assert np.array_equal(host_api.predict_dense(L, m2, X), pred)
    L.model_free(m)
    L.model_free(m2)


def test_probability_and_infeasible_nu(fx):
    L, g, X = fx
    m, nf, nc, ok = host_api.train(L, 0, X=X, y=g["y"], gamma=0.5, C_=100, probability=1)
    pred = host_api.predict_dense(L, m, X)
    assert (pred == g["y"]).mean() > 0.95
    text = host_api.model_text(L, m)
    assert "probA " in text
    # Platt coefficients of SVC::probability_train (svc.cpp:427-492: five folds, sigmoidTrain per class pair)
    # against the reference build's own values for this data set
    ref = np.load(os.path.join(ROOT, "tests", "golden", "prob.npz"))
    for key in ("probA", "probB"):
        got = np.array([float(v) for v in [ln for ln in text.splitlines() if ln.startswith(key + " ")][0].split()[1:]])
        assert got.shape == ref[key].shape
        assert np.all(np.abs(got - ref[key]) <= 0.02 * np.abs(ref[key]) + 5e-3), (key, got, ref[key])
    L.model_free(m)
    m, nf, nc, ok = host_api.train(L, 1, X=X, y=g["y"], gamma=0.5, nu=0.99)
    assert ok == -1                                  # thundersvm-scikit.cpp:93-96
    L.model_free(m)


def test_cli_train_predict_cross_validation(fx, tmp_path):
    """README.md:95-98 quick start: `thundersvm-train -c 100 -g 0.5` then `thundersvm-predict` prints
    Accuracy = 0.98; test_cross_validation.cpp:51-59: 5-fold C-SVC C=10 gamma=0.125 -> 0.973."""
    L, g, X = fx
    data = tmp_path / "test_dataset.txt"
    rp = g["row_ptr"]
    with open(data, "w") as f:
        for i in range(len(rp) - 1):
            feats = " ".join("%d:%.8g" % (g["col"][p] + 1, g["val"][p]) for p in range(rp[i], rp[i + 1]))
            f.write("%g %s\n" % (g["y"][i], feats))
    model, out = tmp_path / "m.model", tmp_path / "pred.txt"
    r = subprocess.run([os.path.join(BIN, "thundersvm-train"), "-c", "100", "-g", "0.5", str(data), str(model)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0, r.stdout
    assert "obj = " in r.stdout and "#total unique sv" in r.stdout
    r = subprocess.run([os.path.join(BIN, "thundersvm-predict"), str(data), str(model), str(out)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0, r.stdout
    assert "Accuracy = 0.98" in r.stdout
    pred = np.loadtxt(out)
    assert abs((pred == g["y"]).mean() - 0.98) < 1e-5
    r = subprocess.run([os.path.join(BIN, "thundersvm-train"), "-c", "10", "-g", "0.125", "-v", "5", str(data)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0, r.stdout
    acc = float(r.stdout.strip().split("Cross Accuracy = ")[1].split()[0])
    assert abs(acc - 0.973) < 1e-3


def test_cached_memory_is_reused_and_released(capi):
    """Handles give their device memory back to the library's pool; tsvm_release_cached_memory returns it to
    the driver. Creating, destroying and re-creating kernel matrices of the same size must neither grow
    the memory in use nor break after a release."""
    import torch
    from thundersvm_b200 import synth
    prob = synth.config5(4000, d=256)
    X = torch.from_numpy(prob["X"]).cuda()
    idx = torch.arange(0, 512, dtype=torch.int32, device="cuda")

    def cycle():
        km = capi.KernelMatrix(dense=X, gamma=0.5)
        rows = km.get_rows(idx).clone()
        km.close()
        return rows

    first = cycle()
    second = cycle()                     # torch's own allocator has its blocks for the temporaries by now
    assert torch.equal(second, first)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(20):                  # a handle's buffers are about 10 MB: a leak would show as 200 MB
        assert torch.equal(cycle(), first)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free_before - (64 << 20)
    capi.lib().tsvm_release_cached_memory()
    assert torch.cuda.mem_get_info()[0] >= free_before - (64 << 20)
    assert torch.equal(cycle(), first)


_PAIR_STREAMS_MODEL = r"""
import hashlib, sys
sys.path.insert(0, "tests")
import numpy as np
import host_api as H
from thundersvm_b200 import synth
L = H.load()
prob = synth.config3(5000)
h = hashlib.sha256()
for svm_type, kw in ((0, dict(C_=prob["C"])), (1, dict(nu=0.3))):        # C-SVC and nu-SVC, ten classes = 45 pairs
    m, nf, nc, ok = H.train(L, svm_type, X=prob["X"], y=prob["y"].astype(np.float32), gamma=prob["gamma"], **kw)
    assert ok and nc == 10
    h.update(H.model_text(L, m).encode())
    L.model_free(m)
print(h.hexdigest())
"""


def test_pairs_on_several_host_threads_give_the_same_model_file():
    """SVC::train solves the class pairs of a device-resident data set from four host threads, each with a CUDA
    stream of its own (THUNDERSVM_PAIR_STREAMS, read at every call). The pairs are independent: the model text -
    every support vector, coefficient and rho - must be the same as with the sequential loop."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    digests = []
    for k in ("1", "4", "4", "7"):
        env = dict(os.environ, THUNDERSVM_PAIR_STREAMS=k, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        r = subprocess.run([sys.executable, "-c", _PAIR_STREAMS_MODEL], env=env, capture_output=True, text=True,
                           timeout=600, cwd=root)
        assert r.returncode == 0, r.stderr[-2000:]
        digests.append(r.stdout.strip().splitlines()[-1])
    assert len(digests[0]) == 64 and len(set(digests)) == 1

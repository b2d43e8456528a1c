"""Host layer without a GPU: the model text format is byte-compatible with the reference's writer and
reader (golden text saved from the reference build), the reference-named C symbols are exported, and
the CLIs reject malformed options the way the reference's CMDParser tests expect (exit code 1)."""
import ctypes as C
import os
import subprocess

import numpy as np

import host_api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "thundersvm_b200", "bin")

REFERENCE_C_SYMBOLS = [
    "model_new", "model_free", "init_model_param", "sparse_model_scikit", "dense_model_scikit", "sparse_predict",
    "dense_predict", "sparse_decision", "dense_decision", "n_sv", "set_iter", "set_memory_size", "get_sv",
    "get_support_classes", "get_coef", "get_linear_coef", "get_rho", "get_pro", "get_n_binary_models", "get_n_classes",
    "get_sv_max_index", "save_to_file_scikit", "load_from_file_scikit", "save_to_string_scikit", "free_string",
    "load_from_string_scikit", "thundersvm_train", "thundersvm_train_after_parse", "thundersvm_predict",
    "thundersvm_predict_after_parse", "load_from_python_interface"]


def test_reference_c_symbols_are_exported():
    L = host_api.load()
    assert not [s for s in REFERENCE_C_SYMBOLS if not hasattr(L, s)]


def test_model_text_round_trip_is_byte_identical(golden_dir, tmp_path):
    """load_from_string + save_to_string on the model text the reference wrote (svmmodel.cpp:193-383)."""
    L = host_api.load()
    text = bytes(np.load(os.path.join(golden_dir, "test_dataset.npz"))["svc_model_text"]).decode()
    m = L.model_new(0)
    L.load_from_string_scikit(m, text.encode())
    assert L.n_sv(m) == 23
    nc = np.zeros(1, np.int32)
    L.get_n_classes(m, host_api.p(nc, host_api.i32p))
    assert nc[0] == 3
    path = str(tmp_path / "model.txt")
    L.save_to_file_scikit(m, path.encode())
    assert open(path).read() == text
    m2 = L.model_new(0)
    L.load_from_file_scikit(m2, path.encode())
    rho = np.zeros(3, np.float32)
    L.get_rho(host_api.p(rho, host_api.f32p), 3, m2)
    assert np.allclose(rho, [-0.117966, 0.0741418, 0.82468], atol=1e-5)
    L.model_free(m)
    L.model_free(m2)


def _run(args):
    return subprocess.run(args, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=60)


def test_cli_rejects_malformed_options():
    """test_cmd.cpp:36-189 checks that invalid values end the process after the help text."""
    host_api.load()
    train = os.path.join(BIN, "thundersvm-train")
    predict = os.path.join(BIN, "thundersvm-predict")
    for bad in (["-s", "9", "x.txt"], ["-t", "7", "x.txt"], ["-g", "-1", "x.txt"], ["-e", "0", "x.txt"],
                ["-c", "-2", "x.txt"], ["-n", "1.5", "-s", "1", "x.txt"], ["-b", "3", "x.txt"], ["-v", "1", "x.txt"],
                ["-z", "1", "x.txt"], ["-c"], []):
        r = _run([train] + bad)
        assert r.returncode == 1, (bad, r.returncode, r.stderr)
        assert "Usage" in r.stdout
    r = _run([predict, "only_one_argument"])
    assert r.returncode == 1 and "Usage" in r.stdout
    r = _run([train, "-q", "/nonexistent/train/file"])
    assert r.returncode == 1          # missing file -> exit(1), dataset.cpp:27-30

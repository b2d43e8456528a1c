"""ctypes view of the reference-named C symbols exported by libthundersvm_b200.so (the scikit-style
API of src/thundersvm/thundersvm-scikit.cpp), used by the host-layer tests the way the reference's
python/thundersvm/thundersvm.py uses the reference library."""
import ctypes as C

import numpy as np

f32p, i32p = C.POINTER(C.c_float), C.POINTER(C.c_int)


def load():
    from thundersvm_b200 import build
    L = C.CDLL(build.build())
    L.model_new.restype = C.c_void_p
    L.model_new.argtypes = [C.c_int]
    L.model_free.argtypes = [C.c_void_p]
    tail = [C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int, C.c_int,
            i32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, i32p, i32p, i32p, C.c_void_p]
    L.dense_model_scikit.argtypes = [C.c_int, C.c_int, f32p, f32p] + tail
    L.sparse_model_scikit.argtypes = [C.c_int, f32p, i32p, i32p, f32p] + tail
    L.dense_predict.argtypes = [C.c_int, C.c_int, f32p, C.c_void_p, f32p, C.c_int]
    L.sparse_predict.argtypes = [C.c_int, f32p, i32p, i32p, C.c_void_p, f32p, C.c_int]
    L.dense_decision.argtypes = [C.c_int, C.c_int, f32p, C.c_void_p, C.c_int, f32p]
    L.n_sv.argtypes = [C.c_void_p]
    L.n_sv.restype = C.c_int
    L.get_rho.argtypes = [f32p, C.c_int, C.c_void_p]
    L.get_support_classes.argtypes = [i32p, C.c_int, C.c_void_p]
    L.get_n_classes.argtypes = [C.c_void_p, i32p]
    L.get_n_binary_models.argtypes = [C.c_void_p, i32p]
    L.save_to_string_scikit.argtypes = [C.c_void_p]
    L.save_to_string_scikit.restype = C.c_void_p
    L.free_string.argtypes = [C.c_void_p]
    L.load_from_string_scikit.argtypes = [C.c_void_p, C.c_char_p]
    L.save_to_file_scikit.argtypes = [C.c_void_p, C.c_char_p]
    L.load_from_file_scikit.argtypes = [C.c_void_p, C.c_char_p]
    return L


def p(a, t):
    return a.ctypes.data_as(t)


def train(L, svm_type, X=None, csr=None, y=None, kernel=2, degree=3, gamma=0.5, coef0=0.0, C_=1.0, nu=0.5, eps=0.1,
          tol=1e-3, probability=0, max_iter=-1):
    m = L.model_new(svm_type)
    nf, nc, ok = (np.zeros(1, np.int32) for _ in range(3))
    y = np.ascontiguousarray(y, np.float32)
    tail = [svm_type, kernel, degree, gamma, coef0, C_, nu, eps, tol, probability, 0, None, None, 0, max_iter, -1, -1, 0,
            p(nf, i32p), p(nc, i32p), p(ok, i32p), m]
    if X is not None:
        X = np.ascontiguousarray(X, np.float32)
        L.dense_model_scikit(X.shape[0], X.shape[1], p(X, f32p), p(y, f32p), *tail)
    else:
        val, rp, col = (np.ascontiguousarray(a) for a in csr)
        L.sparse_model_scikit(len(rp) - 1, p(val.astype(np.float32), f32p), p(rp.astype(np.int32), i32p),
                              p(col.astype(np.int32), i32p), p(y, f32p), *tail)
    return m, int(nf[0]), int(nc[0]), int(ok[0])


def predict_dense(L, m, X):
    X = np.ascontiguousarray(X, np.float32)
    out = np.zeros(X.shape[0], np.float32)
    L.dense_predict(X.shape[0], X.shape[1], p(X, f32p), m, p(out, f32p), 0)
    return out


def predict_sparse(L, m, csr):
    val, rp, col = csr
    out = np.zeros(len(rp) - 1, np.float32)
    L.sparse_predict(len(rp) - 1, p(np.ascontiguousarray(val, np.float32), f32p), p(np.ascontiguousarray(rp, np.int32), i32p),
                     p(np.ascontiguousarray(col, np.int32), i32p), m, p(out, f32p), 0)
    return out


def model_text(L, m, length_hint=1 << 22):
    ptr = L.save_to_string_scikit(m)
    # the buffer is not NUL-terminated: the text ends with the last SV line's newline
    raw = C.string_at(ptr, length_hint) if False else None
    # find the length through a file round trip instead of guessing
    import tempfile, os
    fd, path = tempfile.mkstemp()
    os.close(fd)
    L.save_to_file_scikit(m, path.encode())
    text = open(path).read()
    os.unlink(path)
    assert C.string_at(ptr, len(text)).decode() == text
    L.free_string(ptr)
    return text

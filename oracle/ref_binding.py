"""TEST INFRASTRUCTURE ONLY: ctypes binding of oracle/_ref/libthundersvm_ref.so.

That library is the reference's own CPU implementation (built by oracle/Makefile from
the reference's source tree, see ref_driver.cpp). Only tests, the smoke check and the
benchmark's CPU-baseline / reference arm may import this module; the product package
never does.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libthundersvm_ref.so")

_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_i32p = C.POINTER(C.c_int)

KERNELS = {"linear": 0, "poly": 1, "polynomial": 1, "rbf": 2, "sigmoid": 3}
SVM_TYPES = {"c_svc": 0, "nu_svc": 1, "one_class": 2, "epsilon_svr": 3, "nu_svr": 4}


def available():
    return os.path.exists(LIB_PATH)


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError("reference CPU library not built: run `make -C oracle ref` where the reference "
                               "sources are present")
        _lib = C.CDLL(LIB_PATH)
        data = [C.c_int, C.c_int, _f32p, _f32p, _i32p, _i32p]
        kern = [C.c_int, C.c_int, C.c_double, C.c_double]
        _lib.ref_kernel_rows_idx.restype = C.c_double
        _lib.ref_kernel_rows_idx.argtypes = data + kern + [_i32p, C.c_int, _f32p, _f32p, C.c_int]
        _lib.ref_kernel_rows_ins.restype = C.c_double
        _lib.ref_kernel_rows_ins.argtypes = data + data + kern + [_f32p]
        _lib.ref_smo_solve.restype = C.c_double
        _lib.ref_smo_solve.argtypes = data + kern + [C.c_int, _i32p, _f64p, _f64p, C.c_double, C.c_double,
                                                    C.c_double, C.c_int, C.c_int, _f64p]
        _lib.ref_model_train.restype = C.c_void_p
        _lib.ref_model_train.argtypes = [C.c_int] + data + [_f32p] + kern + [C.c_double] * 4 + [C.c_int, C.c_int,
                                                                                                 _f64p]
        _lib.ref_model_free.argtypes = [C.c_void_p]
        _lib.ref_model_info.argtypes = [C.c_void_p, _i32p]
        _lib.ref_model_get.argtypes = [C.c_void_p, _f64p, _f64p, _i32p, _i32p, _i32p]
        _lib.ref_model_coef_size.argtypes = [C.c_void_p]
        _lib.ref_model_coef_size.restype = C.c_int
        _lib.ref_model_predict.restype = C.c_double
        _lib.ref_model_predict.argtypes = [C.c_void_p] + data + [_f64p, _f64p]
        _lib.ref_cross_validation.argtypes = [C.c_int] + data + [_f32p] + kern + [C.c_double] * 4 + [C.c_int, _f64p]
        _lib.ref_model_save_to_string.restype = C.c_long
        _lib.ref_model_save_to_string.argtypes = [C.c_void_p, C.c_char_p, C.c_long]
        _lib.ref_max_threads.restype = C.c_int
        _lib.ref_set_quiet(1)
    return _lib


def _p(a, t):
    return None if a is None else a.ctypes.data_as(t)


class Data:
    """Either dense (n x d float32 row-major) or CSR with 0-based columns."""

    def __init__(self, dense=None, csr=None, d=None):
        if dense is not None:
            self.dense = np.ascontiguousarray(dense, dtype=np.float32)
            self.n, self.d = self.dense.shape
            self.val = self.row_ptr = self.col = None
        else:
            val, row_ptr, col = csr
            self.dense = None
            self.val = np.ascontiguousarray(val, dtype=np.float32)
            self.row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
            self.col = np.ascontiguousarray(col, dtype=np.int32)
            self.n = len(self.row_ptr) - 1
            self.d = int(d)

    def args(self):
        return [self.n, self.d, _p(self.dense, _f32p), _p(self.val, _f32p), _p(self.row_ptr, _i32p),
                _p(self.col, _i32p)]


def _kern(kernel, degree, gamma, coef0):
    return [KERNELS[kernel] if isinstance(kernel, str) else int(kernel), int(degree), float(gamma), float(coef0)]


def kernel_rows_idx(data, idx, kernel="rbf", gamma=0.5, coef0=0.0, degree=3, reps=1, want_rows=True):
    """KernelMatrix::get_rows(idx) -> (rows[q,n] float32, diag[n] float32, seconds)."""
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    out = np.empty((len(idx), data.n), dtype=np.float32) if want_rows else None
    diag = np.empty(data.n, dtype=np.float32)
    sec = lib().ref_kernel_rows_idx(*data.args(), *_kern(kernel, degree, gamma, coef0), _p(idx, _i32p), len(idx),
                                    _p(out, _f32p), _p(diag, _f32p), reps)
    return out, diag, sec


def kernel_rows_ins(data, test, kernel="rbf", gamma=0.5, coef0=0.0, degree=3):
    """KernelMatrix::get_rows(instances) -> rows[m,n] float32."""
    out = np.empty((test.n, data.n), dtype=np.float32)
    lib().ref_kernel_rows_ins(*data.args(), *test.args(), *_kern(kernel, degree, gamma, coef0), _p(out, _f32p))
    return out


def smo_solve(data, y, alpha, f_val, eps, Cp, Cn, ws_size, max_iter=-1, solver="c", kernel="rbf", gamma=0.5,
              coef0=0.0, degree=3):
    """CSMOSolver/NuSMOSolver::solve -> (alpha, f_val, rho, seconds); inputs are not modified."""
    kind = {"c": 0, "nu_svc": 1, "nu_svr": 2}[solver]
    y = np.ascontiguousarray(y, dtype=np.int32)
    a = np.array(alpha, dtype=np.float64, copy=True)
    f = np.array(f_val, dtype=np.float64, copy=True)
    rho = C.c_double(0)
    sec = lib().ref_smo_solve(*data.args(), *_kern(kernel, degree, gamma, coef0), kind, _p(y, _i32p), _p(a, _f64p),
                              _p(f, _f64p), eps, Cp, Cn, ws_size, max_iter, C.byref(rho))
    return a, f, rho.value, sec


class Model:
    def __init__(self, svm_type, data, labels, kernel="rbf", gamma=0.5, coef0=0.0, degree=3, C_=1.0, nu=0.5, p=0.1,
                 eps=1e-3, probability=0, max_iter=-1):
        labels = np.ascontiguousarray(labels, dtype=np.float32)
        sec = C.c_double(0)
        st = SVM_TYPES[svm_type] if isinstance(svm_type, str) else int(svm_type)
        self.h = lib().ref_model_train(st, *data.args(), _p(labels, _f32p), *_kern(kernel, degree, gamma, coef0),
                                       float(C_), float(nu), float(p), float(eps), int(probability), int(max_iter),
                                       C.byref(sec))
        self.train_seconds = sec.value
        info = np.zeros(3, dtype=np.int32)
        lib().ref_model_info(self.h, _p(info, _i32p))
        self.n_classes, self.n_binary, self.total_sv = (int(v) for v in info)
        self.rho = np.zeros(self.n_binary, dtype=np.float64)
        self.coef = np.zeros(lib().ref_model_coef_size(self.h), dtype=np.float64)
        self.n_sv = np.zeros(self.n_classes, dtype=np.int32)
        self.sv_ind = np.zeros(self.total_sv, dtype=np.int32)
        lib().ref_model_get(self.h, _p(self.rho, _f64p), _p(self.coef, _f64p), _p(self.n_sv, _i32p),
                            _p(self.sv_ind, _i32p), None)

    def predict(self, test, want_dec=True):
        """-> (labels[m], dec[m, n_binary] or None, seconds of predict())."""
        lab = np.empty(test.n, dtype=np.float64)
        dec = np.empty((test.n, self.n_binary), dtype=np.float64) if want_dec else None
        sec = lib().ref_model_predict(self.h, *test.args(), _p(lab, _f64p), _p(dec, _f64p))
        return lab, dec, sec

    def save_to_string(self):
        n = lib().ref_model_save_to_string(self.h, None, 0)
        buf = C.create_string_buffer(n)
        lib().ref_model_save_to_string(self.h, buf, n)
        return buf.raw[:n].decode()

    def close(self):
        if self.h:
            lib().ref_model_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def cross_validation(svm_type, data, labels, n_fold=5, kernel="rbf", gamma=0.5, coef0=0.0, degree=3, C_=1.0,
                     nu=0.5, p=0.1, eps=1e-3):
    labels = np.ascontiguousarray(labels, dtype=np.float32)
    out = np.empty(data.n, dtype=np.float64)
    st = SVM_TYPES[svm_type] if isinstance(svm_type, str) else int(svm_type)
    lib().ref_cross_validation(st, *data.args(), _p(labels, _f32p), *_kern(kernel, degree, gamma, coef0), float(C_),
                               float(nu), float(p), float(eps), int(n_fold), _p(out, _f64p))
    return out

"""TEST INFRASTRUCTURE ONLY: ctypes binding of oracle/libsvm_oracle.so (svm_oracle.c, the
CPU restatement of the reference algorithm). Imported by tests, the smoke check and the
benchmark's CPU-baseline leg only - never by the product package."""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsvm_oracle.so")
KERNELS = {"linear": 0, "poly": 1, "polynomial": 1, "rbf": 2, "sigmoid": 3}

_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_i32p = C.POINTER(C.c_int)
_lib = None


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE, "port"])


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(
                os.path.join(_HERE, "svm_oracle.c")):
            build()
        _lib = C.CDLL(LIB_PATH)
        csr = [C.c_int, C.c_int, _f32p, _i32p, _i32p]
        kern = [C.c_int, C.c_int, C.c_float, C.c_float]
        _lib.oracle_self_dot.argtypes = [C.c_int, _f32p, _i32p, _f32p]
        _lib.oracle_diag.argtypes = [C.c_int, _f32p, _i32p] + kern + [_f32p]
        _lib.oracle_kernel_rows_idx.argtypes = csr + kern + [_i32p, C.c_int, _f32p]
        _lib.oracle_kernel_rows_ins.argtypes = csr + kern + [C.c_int, _f32p, _i32p, _i32p, _f32p]
        _lib.oracle_local_smo.argtypes = [C.c_int, C.c_int, _i32p, _f64p, _f64p, _f64p, _i32p, C.c_int, C.c_double,
                                          C.c_double, _f32p, _f32p, C.c_int, C.c_double, _f64p, C.c_int]
        _lib.oracle_update_f.argtypes = [_f64p, C.c_int, _f64p, C.c_int, _f32p]
        _lib.oracle_select_working_set.argtypes = [C.c_int, C.c_int, _f64p, _i32p, _f64p, C.c_double, C.c_double,
                                                   C.c_char_p, _i32p, C.c_int]
        _lib.oracle_objective.restype = C.c_double
        _lib.oracle_objective.argtypes = [C.c_int, _f64p, _f64p, _i32p]
        _lib.oracle_smo_solve.argtypes = csr + kern + [C.c_int, C.c_int, _i32p, _f64p, _f64p, C.c_double, C.c_double,
                                                       C.c_double, C.c_int, C.c_int, _f64p, _f64p, _i32p, C.c_int]
        _lib.oracle_sum_kernel_values.argtypes = [_f64p, C.c_int, _i32p, _i32p, _f64p, _f32p, _f64p, C.c_int,
                                                  C.c_int]
        _lib.oracle_predict_dec.argtypes = csr + kern + [_f64p, _i32p, _f64p, C.c_int, C.c_int, _f32p, _i32p, _i32p,
                                                         _f64p]
        _lib.oracle_vote.argtypes = [_f64p, C.c_int, C.c_int, _i32p]
    return _lib


def _p(a, t):
    return None if a is None else a.ctypes.data_as(t)


class Csr:
    """CSR matrix (float32 values, int32 row_ptr / 0-based col). Dense input keeps its
    explicit zeros as stored entries, as the reference's dense loader does."""

    def __init__(self, dense=None, csr=None, d=None):
        if dense is not None:
            dense = np.ascontiguousarray(dense, dtype=np.float32)
            n, dd = dense.shape
            self.val = dense.reshape(-1).copy()
            self.row_ptr = (np.arange(n + 1, dtype=np.int64) * dd).astype(np.int32)
            self.col = np.tile(np.arange(dd, dtype=np.int32), n)
            self.n, self.d = n, dd
        else:
            val, row_ptr, col = csr
            self.val = np.ascontiguousarray(val, dtype=np.float32)
            self.row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
            self.col = np.ascontiguousarray(col, dtype=np.int32)
            self.n = len(self.row_ptr) - 1
            self.d = int(d) if d is not None else (int(self.col.max()) + 1 if len(self.col) else 0)

    def args(self):
        return [self.n, self.d, _p(self.val, _f32p), _p(self.row_ptr, _i32p), _p(self.col, _i32p)]


def _kern(kernel, degree, gamma, coef0):
    return [KERNELS[kernel] if isinstance(kernel, str) else int(kernel), int(degree), float(gamma), float(coef0)]


def diag(X, kernel="rbf", gamma=0.5, coef0=0.0, degree=3):
    out = np.empty(X.n, dtype=np.float32)
    lib().oracle_diag(X.n, _p(X.val, _f32p), _p(X.row_ptr, _i32p), *_kern(kernel, degree, gamma, coef0),
                      _p(out, _f32p))
    return out


def self_dot(X):
    out = np.empty(X.n, dtype=np.float32)
    lib().oracle_self_dot(X.n, _p(X.val, _f32p), _p(X.row_ptr, _i32p), _p(out, _f32p))
    return out


def kernel_rows_idx(X, idx, kernel="rbf", gamma=0.5, coef0=0.0, degree=3):
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    out = np.empty((len(idx), X.n), dtype=np.float32)
    lib().oracle_kernel_rows_idx(*X.args(), *_kern(kernel, degree, gamma, coef0), _p(idx, _i32p), len(idx),
                                 _p(out, _f32p))
    return out


def kernel_rows_ins(X, T, kernel="rbf", gamma=0.5, coef0=0.0, degree=3):
    out = np.empty((T.n, X.n), dtype=np.float32)
    lib().oracle_kernel_rows_ins(*X.args(), *_kern(kernel, degree, gamma, coef0), T.n, _p(T.val, _f32p),
                                 _p(T.row_ptr, _i32p), _p(T.col, _i32p), _p(out, _f32p))
    return out


def local_smo(kind, y, f_val, alpha, ws, Cp, Cn, rows, diag_, eps, max_iter=100000, cuda_semantics=0):
    """-> (alpha (updated copy), alpha_diff[ws], diff[2])."""
    kind = {"c": 0, "nu": 1}[kind] if isinstance(kind, str) else kind
    y = np.ascontiguousarray(y, dtype=np.int32)
    ws = np.ascontiguousarray(ws, dtype=np.int32)
    a = np.array(alpha, dtype=np.float64, copy=True)
    f = np.ascontiguousarray(f_val, dtype=np.float64)
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    dg = np.ascontiguousarray(diag_, dtype=np.float32)
    ad = np.zeros(len(ws), dtype=np.float64)
    diff = np.zeros(2, dtype=np.float64)
    lib().oracle_local_smo(kind, cuda_semantics, _p(y, _i32p), _p(f, _f64p), _p(a, _f64p), _p(ad, _f64p),
                           _p(ws, _i32p), len(ws), Cp, Cn, _p(rows, _f32p), _p(dg, _f32p), rows.shape[1], eps,
                           _p(diff, _f64p), max_iter)
    return a, ad, diff


def update_f(f, alpha_diff, rows):
    f = np.array(f, dtype=np.float64, copy=True)
    ad = np.ascontiguousarray(alpha_diff, dtype=np.float64)
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    lib().oracle_update_f(_p(f, _f64p), len(f), _p(ad, _f64p), len(ad), _p(rows, _f32p))
    return f


def select_working_set(kind, f, y, alpha, Cp, Cn, in_ws, want):
    kind = {"c": 0, "nu": 1}[kind] if isinstance(kind, str) else kind
    f = np.ascontiguousarray(f, dtype=np.float64)
    y = np.ascontiguousarray(y, dtype=np.int32)
    alpha = np.ascontiguousarray(alpha, dtype=np.float64)
    flags = np.ascontiguousarray(in_ws, dtype=np.int8) if in_ws is not None else np.zeros(len(f), np.int8)
    out = np.full(want, -1, dtype=np.int32)
    lib().oracle_select_working_set(kind, len(f), _p(f, _f64p), _p(y, _i32p), _p(alpha, _f64p), Cp, Cn,
                                    flags.ctypes.data_as(C.c_char_p), _p(out, _i32p), want)
    return out


def objective(f, alpha, y):
    f = np.ascontiguousarray(f, dtype=np.float64)
    alpha = np.ascontiguousarray(alpha, dtype=np.float64)
    y = np.ascontiguousarray(y, dtype=np.int32)
    return lib().oracle_objective(len(f), _p(f, _f64p), _p(alpha, _f64p), _p(y, _i32p))


def smo_solve(X, y, alpha, f_val, eps, Cp, Cn, ws_size, max_iter=-1, solver="c", kernel="rbf", gamma=0.5, coef0=0.0,
              degree=3, cuda_semantics=0, trace_iters=0):
    """-> dict(alpha, f, rho, iters, local_iters, diff, obj, ws_trace)."""
    kind = {"c": 0, "nu_svc": 1, "nu_svr": 2}[solver]
    y = np.ascontiguousarray(y, dtype=np.int32)
    a = np.array(alpha, dtype=np.float64, copy=True)
    f = np.array(f_val, dtype=np.float64, copy=True)
    rho = C.c_double(0)
    stats = np.zeros(4, dtype=np.float64)
    trace = np.full((max(trace_iters, 1), ws_size), -1, dtype=np.int32)
    lib().oracle_smo_solve(*X.args(), *_kern(kernel, degree, gamma, coef0), kind, cuda_semantics, _p(y, _i32p),
                           _p(a, _f64p), _p(f, _f64p), eps, Cp, Cn, ws_size, max_iter, C.byref(rho),
                           _p(stats, _f64p), _p(trace, _i32p), trace_iters)
    return dict(alpha=a, f=f, rho=rho.value, iters=int(stats[0]), local_iters=int(stats[1]), diff=stats[2],
                obj=stats[3], ws_trace=trace[:trace_iters])


def predict_dec(SV, coef, sv_count, rho, n_classes, T, kernel="rbf", gamma=0.5, coef0=0.0, degree=3):
    coef = np.ascontiguousarray(coef, dtype=np.float64)
    sv_count = np.ascontiguousarray(sv_count, dtype=np.int32)
    rho = np.ascontiguousarray(rho, dtype=np.float64)
    nb = n_classes * (n_classes - 1) // 2
    dec = np.empty((T.n, nb), dtype=np.float64)
    lib().oracle_predict_dec(*SV.args(), *_kern(kernel, degree, gamma, coef0), _p(coef, _f64p), _p(sv_count, _i32p),
                             _p(rho, _f64p), n_classes, T.n, _p(T.val, _f32p), _p(T.row_ptr, _i32p),
                             _p(T.col, _i32p), _p(dec, _f64p))
    return dec


def vote(dec, n_classes):
    dec = np.ascontiguousarray(dec, dtype=np.float64)
    out = np.empty(dec.shape[0], dtype=np.int32)
    lib().oracle_vote(_p(dec, _f64p), dec.shape[0], n_classes, _p(out, _i32p))
    return out

"""ctypes binding of libthundersvm_b200.so (include/thundersvm_b200.h).

PyTorch is used only as the owner of device buffers and streams: every computation goes
through the C ABI. There is no CPU fallback - if the shared library is missing or a call
fails, an exception is raised.
"""
import ctypes as C
import os

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libthundersvm_b200.so")

KERNELS = {"linear": 0, "poly": 1, "polynomial": 1, "rbf": 2, "sigmoid": 3, "precomputed": 4}
SOLVERS = {"c": 0, "nu_svc": 1, "nu_svr": 2}
HOST, DEVICE = 0, 1

# every symbol include/thundersvm_b200.h declares
EXPORTS = [
    "tsvm_release_cached_memory", "tsvm_set_row_cache_bytes",
    "tsvm_last_error", "tsvm_abi_version", "tsvm_km_create_dense", "tsvm_km_create_csr", "tsvm_km_destroy",
    "tsvm_km_n_instances", "tsvm_km_n_features", "tsvm_km_nnz", "tsvm_km_is_dense", "tsvm_km_diag_dev",
    "tsvm_km_self_dot_dev", "tsvm_km_rows_by_index", "tsvm_km_rows_by_instances_dense",
    "tsvm_km_rows_by_instances_csr", "tsvm_km_rows_for_features_dense", "tsvm_km_set_dense_engine", "tsvm_rho_partials", "tsvm_smo_solve", "tsvm_solver_create",
    "tsvm_solver_iterate", "tsvm_solver_finish", "tsvm_solver_get_stats", "tsvm_solver_set_overlap", "tsvm_solver_destroy", "tsvm_shard_create", "tsvm_shard_candidates", "tsvm_shard_select", "tsvm_shard_iterate", "tsvm_nccl_unique_id", "tsvm_nccl_comm_create", "tsvm_nccl_comm_destroy", "tsvm_shard_attach_nccl", "tsvm_shard_step", "tsvm_shard_run", "tsvm_shard_get_stats", "tsvm_shard_destroy", "tsvm_working_set_size",
    "tsvm_ws_create", "tsvm_ws_destroy", "tsvm_ws_candidates", "tsvm_ws_merge", "tsvm_ws_sort_candidates", "tsvm_ws_merge_sorted", "tsvm_select_working_set",
    "tsvm_select_working_set_static",
    "tsvm_local_smo", "tsvm_update_f", "tsvm_predict_dec", "tsvm_predict_labels", "tsvm_vote",
]


class SolveStats(C.Structure):
    _fields_ = [("outer_iters", C.c_longlong), ("local_iters", C.c_longlong), ("final_diff", C.c_double),
                ("objective", C.c_double), ("seconds_select", C.c_double), ("seconds_rows", C.c_double),
                ("seconds_local", C.c_double), ("seconds_update", C.c_double), ("seconds_total", C.c_double),
                ("kernel_rows", C.c_longlong), ("gpu_launches", C.c_longlong), ("cache_hits", C.c_longlong),
                ("cache_misses", C.c_longlong), ("cache_rows", C.c_longlong), ("row_blocks", C.c_longlong),
                ("row_blocks_saved", C.c_longlong)]

    def as_dict(self):
        return {k: getattr(self, k) for k, _ in self._fields_}


class TsvmError(RuntimeError):
    pass


_lib = None


def lib():
    """Loads the shared library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise TsvmError("libthundersvm_b200.so is missing: run `python -m thundersvm_b200.build` "
                        "(there is no CPU fallback)")
    L = C.CDLL(LIB_PATH)
    vp, i, f, d, ll, sz = C.c_void_p, C.c_int, C.c_float, C.c_double, C.c_longlong, C.c_size_t
    L.tsvm_last_error.restype = C.c_char_p
    L.tsvm_abi_version.restype = i
    L.tsvm_release_cached_memory.restype = None
    L.tsvm_release_cached_memory.argtypes = []
    L.tsvm_set_row_cache_bytes.restype = None
    L.tsvm_set_row_cache_bytes.argtypes = [ll]
    L.tsvm_km_create_dense.argtypes = [vp, i, i, i, i, i, i, f, f, vp, C.POINTER(vp)]
    L.tsvm_km_create_csr.argtypes = [vp, vp, vp, i, i, i, i, i, f, f, vp, C.POINTER(vp)]
    L.tsvm_km_destroy.argtypes = [vp]
    L.tsvm_km_destroy.restype = None
    for name in ("tsvm_km_n_instances", "tsvm_km_n_features", "tsvm_km_is_dense"):
        getattr(L, name).argtypes = [vp]
        getattr(L, name).restype = i
    L.tsvm_km_nnz.argtypes = [vp]
    L.tsvm_km_nnz.restype = ll
    L.tsvm_km_diag_dev.argtypes = [vp]
    L.tsvm_km_diag_dev.restype = vp
    L.tsvm_km_self_dot_dev.argtypes = [vp]
    L.tsvm_km_self_dot_dev.restype = vp
    L.tsvm_km_rows_by_index.argtypes = [vp, vp, i, vp, ll, vp]
    L.tsvm_km_rows_by_instances_dense.argtypes = [vp, vp, i, i, i, vp, ll, vp]
    L.tsvm_km_rows_by_instances_csr.argtypes = [vp, vp, vp, vp, i, ll, vp, ll, vp]
    L.tsvm_km_rows_for_features_dense.argtypes = [vp, vp, i, vp, i, vp, ll, vp]
    L.tsvm_rho_partials.argtypes = [i, vp, vp, vp, d, d, vp, vp]
    L.tsvm_km_set_dense_engine.argtypes = [vp, i]
    L.tsvm_smo_solve.argtypes = [vp, i, vp, vp, vp, d, d, d, i, i, C.POINTER(d), C.POINTER(SolveStats), vp]
    L.tsvm_solver_create.argtypes = [vp, i, vp, vp, vp, d, d, d, i, vp, C.POINTER(vp)]
    L.tsvm_solver_iterate.argtypes = [vp, i, C.POINTER(i)]
    L.tsvm_solver_finish.argtypes = [vp, C.POINTER(d), C.POINTER(SolveStats)]
    L.tsvm_solver_get_stats.argtypes = [vp, C.POINTER(SolveStats)]
    L.tsvm_solver_set_overlap.argtypes = [vp, i]
    L.tsvm_shard_create.argtypes = [vp, i, vp, vp, vp, i, i, d, d, d, i, i, vp, vp, vp, vp, vp, vp, vp, C.POINTER(vp)]
    L.tsvm_shard_candidates.argtypes = [vp, C.POINTER(i), C.POINTER(i)]
    L.tsvm_shard_select.argtypes = [vp, C.POINTER(i)]
    L.tsvm_shard_iterate.argtypes = [vp, C.POINTER(i)]
    L.tsvm_shard_get_stats.argtypes = [vp, C.POINTER(SolveStats)]
    L.tsvm_nccl_unique_id.argtypes = [vp]
    L.tsvm_shard_attach_nccl.argtypes = [vp, vp]
    L.tsvm_nccl_comm_create.argtypes = [vp, i, i, C.POINTER(vp)]
    L.tsvm_nccl_comm_destroy.argtypes = [vp]
    L.tsvm_nccl_comm_destroy.restype = None
    L.tsvm_shard_step.argtypes = [vp, C.POINTER(i)]
    L.tsvm_shard_run.argtypes = [vp, i, C.POINTER(i)]
    L.tsvm_shard_destroy.argtypes = [vp]
    L.tsvm_shard_destroy.restype = None
    L.tsvm_solver_destroy.argtypes = [vp]
    L.tsvm_solver_destroy.restype = None
    L.tsvm_working_set_size.argtypes = [i, i, sz, sz]
    L.tsvm_working_set_size.restype = i
    L.tsvm_ws_create.argtypes = [i, i, C.POINTER(vp)]
    L.tsvm_ws_destroy.argtypes = [vp]
    L.tsvm_ws_destroy.restype = None
    L.tsvm_ws_candidates.argtypes = [vp, i, i, vp, vp, vp, vp, d, d, i, i, vp, vp, vp]
    L.tsvm_ws_merge.argtypes = [vp, i, vp, vp, i, i, vp, vp]
    L.tsvm_select_working_set.argtypes = [vp, i, i, vp, vp, vp, vp, d, d, i, vp, vp]
    L.tsvm_select_working_set_static.argtypes = [i, i, vp, vp, vp, vp, d, d, i, vp, vp]
    L.tsvm_local_smo.argtypes = [i, i, vp, vp, vp, vp, vp, vp, d, d, d, i, vp, vp]
    L.tsvm_update_f.argtypes = [vp, i, vp, i, vp, ll, vp]
    L.tsvm_predict_dec.argtypes = [vp, vp, C.POINTER(i), vp, i, i, vp, i, i, vp, vp, vp, ll, vp, sz, vp]
    L.tsvm_predict_labels.argtypes = [vp, vp, C.POINTER(i), vp, i, i, vp, i, i, vp, vp, vp, ll, vp, sz, vp]
    L.tsvm_vote.argtypes = [vp, i, i, vp, vp]
    _lib = L
    return L


def check(status):
    if status != 0:
        raise TsvmError("thundersvm_b200 status %d: %s" % (status, lib().tsvm_last_error().decode()))


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _kid(kernel):
    return KERNELS[kernel] if isinstance(kernel, str) else int(kernel)


class _DeviceView:
    """float32 device memory owned by the library, exposed through __cuda_array_interface__."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (int(ptr), False), "version": 2}


class KernelMatrix:
    """Device-resident kernel matrix (mirror of the reference's KernelMatrix class).

    dense: torch.float32 [n, d] tensor (CUDA: used in place when 16-byte aligned rows, else copied;
    CPU tensor / numpy array: uploaded by the library).  csr: (val, row_ptr, col) with 0-based
    columns, all on the same side (CUDA tensors or numpy arrays)."""

    def __init__(self, dense=None, csr=None, d=None, kernel="rbf", gamma=0.5, coef0=0.0, degree=3):
        L = lib()
        self._h = C.c_void_p(0)
        self._keep = []
        if dense is not None:
            if isinstance(dense, np.ndarray):
                dense = np.ascontiguousarray(dense, dtype=np.float32)
                n, dd = dense.shape
                check(L.tsvm_km_create_dense(dense.ctypes.data, n, dd, dd, HOST, _kid(kernel), degree, gamma, coef0,
                                             _stream(), C.byref(self._h)))
            else:
                assert dense.dtype == torch.float32 and dense.dim() == 2 and dense.stride(1) == 1
                n, dd = dense.shape
                loc = DEVICE if dense.is_cuda else HOST
                self._keep.append(dense)
                check(L.tsvm_km_create_dense(_ptr(dense), n, dd, dense.stride(0), loc, _kid(kernel), degree, gamma,
                                             coef0, _stream(), C.byref(self._h)))
            torch.cuda.current_stream().synchronize()
        else:
            val, row_ptr, col = csr
            if isinstance(val, np.ndarray):
                val = np.ascontiguousarray(val, dtype=np.float32)
                row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
                col = np.ascontiguousarray(col, dtype=np.int32)
                n = len(row_ptr) - 1
                check(L.tsvm_km_create_csr(val.ctypes.data, row_ptr.ctypes.data, col.ctypes.data, n, int(d), HOST,
                                           _kid(kernel), degree, gamma, coef0, _stream(), C.byref(self._h)))
                torch.cuda.current_stream().synchronize()
            else:
                assert val.is_cuda and val.dtype == torch.float32 and row_ptr.dtype == torch.int32
                self._keep += [val, row_ptr, col]
                n = row_ptr.numel() - 1
                check(L.tsvm_km_create_csr(_ptr(val), _ptr(row_ptr), _ptr(col), n, int(d), DEVICE, _kid(kernel),
                                           degree, gamma, coef0, _stream(), C.byref(self._h)))
        self.n = L.tsvm_km_n_instances(self._h)
        self.d = L.tsvm_km_n_features(self._h)
        self.is_dense = bool(L.tsvm_km_is_dense(self._h))

    @property
    def handle(self):
        return self._h

    def set_dense_engine(self, engine):
        check(lib().tsvm_km_set_dense_engine(self._h, {"auto": 0, "simt": 1, "tensor1": 2, "tensor2": 3, "tensor_tf32": 3, "tensor": 4, "tensor_f16": 4}.get(engine, engine)))

    def _vec(self, fn):
        view = _DeviceView(fn(self._h), self.n)
        return torch.as_tensor(view, device="cuda").clone()

    def diag(self):
        return self._vec(lib().tsvm_km_diag_dev)

    def self_dot(self):
        return self._vec(lib().tsvm_km_self_dot_dev)

    def get_rows(self, idx, out=None):
        """KernelMatrix::get_rows(idx): idx int32 CUDA tensor -> float32 [q, n]."""
        idx = idx.to(device="cuda", dtype=torch.int32).contiguous()
        q = idx.numel()
        if out is None:
            out = torch.empty((q, self.n), dtype=torch.float32, device="cuda")
        check(lib().tsvm_km_rows_by_index(self._h, _ptr(idx), q, _ptr(out), out.stride(0), _stream()))
        return out

    def get_rows_instances(self, dense=None, csr=None, out=None):
        """KernelMatrix::get_rows(instances): dense float32 [m, dt] or CSR CUDA tensors -> [m, n]."""
        if dense is not None:
            m = dense.shape[0]
            if out is None:
                out = torch.empty((m, self.n), dtype=torch.float32, device="cuda")
            check(lib().tsvm_km_rows_by_instances_dense(self._h, _ptr(dense), m, dense.shape[1], dense.stride(0),
                                                        _ptr(out), out.stride(0), _stream()))
        else:
            val, row_ptr, col = csr
            m = row_ptr.numel() - 1
            if out is None:
                out = torch.empty((m, self.n), dtype=torch.float32, device="cuda")
            check(lib().tsvm_km_rows_by_instances_csr(self._h, _ptr(val), _ptr(row_ptr), _ptr(col), m, val.numel(),
                                                      _ptr(out), out.stride(0), _stream()))
        return out

    def rows_for_features(self, T, sd_T, out=None):
        """Kernel rows for explicit feature rows T [m, d] with their self dots sd_T [m] -> [m, n]."""
        m = T.shape[0]
        if out is None:
            out = torch.empty((m, self.n), dtype=torch.float32, device="cuda")
        check(lib().tsvm_km_rows_for_features_dense(self._h, _ptr(T), T.stride(0), _ptr(sd_T), m, _ptr(out),
                                                    out.stride(0), _stream()))
        return out

    def close(self):
        if self._h:
            lib().tsvm_km_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def set_row_cache_bytes(nbytes):
    """Budget of the kernel-row cache of solvers created from now on (< 0: default, 0: minimum)."""
    lib().tsvm_set_row_cache_bytes(int(nbytes))


def working_set_size(n, d, max_mem_bytes=8192 << 20, used_bytes=0):
    return lib().tsvm_working_set_size(n, d, max_mem_bytes, used_bytes)


def smo_solve(km, y, alpha, f, eps, Cp, Cn, ws_size, max_iter=-1, solver="c"):
    """CSMOSolver/NuSMOSolver::solve on device tensors (alpha, f updated in place).
    -> (rho, stats dict)."""
    assert y.dtype == torch.int32 and alpha.dtype == torch.float64 and f.dtype == torch.float64
    rho = C.c_double(0)
    st = SolveStats()
    check(lib().tsvm_smo_solve(km.handle, SOLVERS[solver], _ptr(y), _ptr(alpha), _ptr(f), eps, Cp, Cn, ws_size,
                               max_iter, C.byref(rho), C.byref(st), _stream()))
    return rho.value, st.as_dict()


class Shard:
    """Per-rank device work of the column-sharded solver (tsvm_shard_*). The exchange buffers are torch
    tensors owned by this object; the caller runs its collectives on them between the three phases."""

    def __init__(self, km, y, alpha, f, n_total, lo, eps, Cp, Cn, ws_size, world, solver="c"):
        dev = y.device
        dp = (km.d + 3) // 4 * 4
        self.ws, self.world, self.dp = ws_size, world, dp
        self.cand_f = torch.zeros(4 * ws_size, dtype=torch.float64, device=dev)
        self.cand_id = torch.zeros(4 * ws_size, dtype=torch.int32, device=dev)
        self.all_f = torch.zeros(world * 4 * ws_size, dtype=torch.float64, device=dev)
        self.all_id = torch.zeros(world * 4 * ws_size, dtype=torch.int32, device=dev)
        self.rows_contrib = torch.zeros(ws_size * (dp + 4), dtype=torch.float32, device=dev)
        self.state_contrib = torch.zeros(ws_size * 3, dtype=torch.float64, device=dev)
        self._h = C.c_void_p(0)
        self._keep = (km, y, alpha, f)
        check(lib().tsvm_shard_create(km.handle, SOLVERS[solver], _ptr(y), _ptr(alpha), _ptr(f), n_total, lo, eps, Cp,
                                      Cn, ws_size, world, _ptr(self.cand_f), _ptr(self.cand_id), _ptr(self.all_f),
                                      _ptr(self.all_id), _ptr(self.rows_contrib), _ptr(self.state_contrib), _stream(),
                                      C.byref(self._h)))

    def candidates(self):
        """-> (lists, want): cand_f / cand_id[:lists * want] are this rank's lists."""
        lists, want = C.c_int(0), C.c_int(0)
        check(lib().tsvm_shard_candidates(self._h, C.byref(lists), C.byref(want)))
        return lists.value, want.value

    def select(self):
        """-> n_new: rows_contrib[:n_new * (dp + 4)] and state_contrib are this rank's contributions."""
        n_new = C.c_int(0)
        check(lib().tsvm_shard_select(self._h, C.byref(n_new)))
        return n_new.value

    def iterate(self):
        done = C.c_int(0)
        check(lib().tsvm_shard_iterate(self._h, C.byref(done)))
        return bool(done.value)

    @staticmethod
    def nccl_unique_id():
        """128 bytes from ncclGetUniqueId (call on one rank, give the bytes to all)."""
        buf = (C.c_char * 128)()
        check(lib().tsvm_nccl_unique_id(buf))
        return bytes(buf)

    @staticmethod
    def nccl_comm_create(unique_id, rank, world):
        """Collective: every rank calls it with the same id. -> communicator handle (not destroyed here)."""
        comm = C.c_void_p(0)
        check(lib().tsvm_nccl_comm_create(C.c_char_p(unique_id), rank, world, C.byref(comm)))
        return comm

    def attach_nccl(self, comm):
        check(lib().tsvm_shard_attach_nccl(self._h, comm))
        self._comm = comm

    def step(self):
        """One whole outer iteration, exchange steps included (after attach_nccl, or with one rank)."""
        done = C.c_int(0)
        check(lib().tsvm_shard_step(self._h, C.byref(done)))
        return bool(done.value)

    def run(self, n_iters):
        """Up to n_iters whole outer iterations (after attach_nccl, or with one rank), queued several at a time."""
        done = C.c_int(0)
        check(lib().tsvm_shard_run(self._h, n_iters, C.byref(done)))
        return bool(done.value)

    def stats(self):
        st = SolveStats()
        check(lib().tsvm_shard_get_stats(self._h, C.byref(st)))
        return st.as_dict()

    def close(self):
        if self._h:
            lib().tsvm_shard_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Solver:
    """Stepping form of the solver (tsvm_solver_*): iterate(k) runs k outer iterations."""

    def __init__(self, km, y, alpha, f, eps, Cp, Cn, ws_size, solver="c"):
        self._h = C.c_void_p(0)
        self._keep = (km, y, alpha, f)
        check(lib().tsvm_solver_create(km.handle, SOLVERS[solver], _ptr(y), _ptr(alpha), _ptr(f), eps, Cp, Cn,
                                       ws_size, _stream(), C.byref(self._h)))

    def iterate(self, n_iters):
        done = C.c_int(0)
        check(lib().tsvm_solver_iterate(self._h, n_iters, C.byref(done)))
        return bool(done.value)

    def set_overlap(self, enable):
        check(lib().tsvm_solver_set_overlap(self._h, 1 if enable else 0))

    def stats(self):
        st = SolveStats()
        check(lib().tsvm_solver_get_stats(self._h, C.byref(st)))
        return st.as_dict()

    def finish(self):
        rho = C.c_double(0)
        st = SolveStats()
        check(lib().tsvm_solver_finish(self._h, C.byref(rho), C.byref(st)))
        return rho.value, st.as_dict()

    def close(self):
        if self._h:
            lib().tsvm_solver_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class WorkingSetSelector:
    def __init__(self, n_max, ws_max=1024):
        self._h = C.c_void_p(0)
        check(lib().tsvm_ws_create(n_max, ws_max, C.byref(self._h)))

    def select(self, f, alpha, y, Cp, Cn, want, in_ws=None, solver="c"):
        out = torch.empty(want, dtype=torch.int32, device="cuda")
        check(lib().tsvm_select_working_set(self._h, SOLVERS[solver], f.numel(), _ptr(f), _ptr(alpha), _ptr(y),
                                            _ptr(in_ws), Cp, Cn, want, _ptr(out), _stream()))
        return out

    def candidates(self, f, alpha, y, Cp, Cn, want, in_ws=None, solver="c", id_offset=0):
        lists = 2 if solver == "c" else 4
        cf = torch.empty((lists, want), dtype=torch.float64, device="cuda")
        ci = torch.empty((lists, want), dtype=torch.int32, device="cuda")
        check(lib().tsvm_ws_candidates(self._h, SOLVERS[solver], f.numel(), _ptr(f), _ptr(alpha), _ptr(y),
                                       _ptr(in_ws), Cp, Cn, want, id_offset, _ptr(cf), _ptr(ci), _stream()))
        return cf, ci

    def merge(self, cand_f, cand_id, want, solver="c"):
        lists, length = cand_f.shape
        out = torch.empty(want, dtype=torch.int32, device="cuda")
        check(lib().tsvm_ws_merge(self._h, SOLVERS[solver], _ptr(cand_f.contiguous()), _ptr(cand_id.contiguous()),
                                  length, want, _ptr(out), _stream()))
        return out

    def sort_candidates(self, cand_f, cand_id, solver="c"):
        """In place: every list sorted by its list key, padding last."""
        lists, length = cand_f.shape
        check(lib().tsvm_ws_sort_candidates(self._h, SOLVERS[solver], _ptr(cand_f), _ptr(cand_id), length, _stream()))

    def merge_sorted(self, cand_f, cand_id, seg_len, want, solver="c"):
        """cand_* [lists, n_runs * seg_len]: concatenated sorted runs."""
        lists, length = cand_f.shape
        out = torch.empty(want, dtype=torch.int32, device="cuda")
        check(lib().tsvm_ws_merge_sorted(self._h, SOLVERS[solver], _ptr(cand_f.contiguous()), _ptr(cand_id.contiguous()),
                                         length, seg_len, want, _ptr(out), _stream()))
        return out

    def close(self):
        if self._h:
            lib().tsvm_ws_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def select_working_set_static(f, alpha, y, Cp, Cn, want, in_ws=None, solver="c", out=None):
    """tsvm_select_working_set_static: working-set selection that allocates nothing inside the library.
    Pass a preallocated int32 `out` tensor to keep the Python side allocation-free as well."""
    if out is None:
        out = torch.empty(want, dtype=torch.int32, device="cuda")
    check(lib().tsvm_select_working_set_static(SOLVERS[solver], f.numel(), _ptr(f), _ptr(alpha), _ptr(y),
                                               _ptr(in_ws), Cp, Cn, want, _ptr(out), _stream()))
    return out


def local_smo(kww, diag_ws, y_ws, f_ws, alpha_ws, Cp, Cn, eps, max_iter=100000, solver="c"):
    """-> (alpha_ws (new tensor), alpha_diff, diff[2])."""
    ws = kww.shape[0]
    a = alpha_ws.clone()
    ad = torch.zeros(ws, dtype=torch.float64, device="cuda")
    diff = torch.zeros(2, dtype=torch.float64, device="cuda")
    check(lib().tsvm_local_smo(SOLVERS[solver], ws, _ptr(kww.contiguous()), _ptr(diag_ws), _ptr(y_ws), _ptr(f_ws),
                               _ptr(a), _ptr(ad), Cp, Cn, eps, max_iter, _ptr(diff), _stream()))
    return a, ad, diff


def update_f(f, alpha_diff, rows):
    check(lib().tsvm_update_f(_ptr(f), f.numel(), _ptr(alpha_diff), alpha_diff.numel(), _ptr(rows), rows.stride(0),
                              _stream()))
    return f


def rho_partials(f, alpha, y, Cp, Cn):
    out = torch.empty(13, dtype=torch.float64, device="cuda")
    check(lib().tsvm_rho_partials(f.numel(), _ptr(f), _ptr(alpha), _ptr(y), Cp, Cn, _ptr(out), _stream()))
    return out


def predict_dec(km_sv, coef, sv_count, rho, n_classes, dense=None, csr=None, max_mem_bytes=0):
    """-> float64 [m, n_binary] decision values."""
    nb = n_classes * (n_classes - 1) // 2
    cnt = (C.c_int * n_classes)(*[int(v) for v in sv_count])
    if dense is not None:
        m = dense.shape[0]
        dec = torch.empty((m, nb), dtype=torch.float64, device="cuda")
        check(lib().tsvm_predict_dec(km_sv.handle, _ptr(coef), cnt, _ptr(rho), n_classes, m, _ptr(dense),
                                     dense.shape[1], dense.stride(0), None, None, None, 0, _ptr(dec), max_mem_bytes,
                                     _stream()))
    else:
        val, row_ptr, col = csr
        m = row_ptr.numel() - 1
        dec = torch.empty((m, nb), dtype=torch.float64, device="cuda")
        check(lib().tsvm_predict_dec(km_sv.handle, _ptr(coef), cnt, _ptr(rho), n_classes, m, None, 0, 0, _ptr(val),
                                     _ptr(row_ptr), _ptr(col), val.numel(), _ptr(dec), max_mem_bytes, _stream()))
    return dec


def predict_labels(km_sv, coef, sv_count, rho, n_classes, dense=None, csr=None, max_mem_bytes=0):
    """-> int32 [m] index of the winning class per test row; the decision values stay inside the library."""
    cnt = (C.c_int * n_classes)(*[int(v) for v in sv_count])
    if dense is not None:
        m = dense.shape[0]
        out = torch.empty(m, dtype=torch.int32, device="cuda")
        check(lib().tsvm_predict_labels(km_sv.handle, _ptr(coef), cnt, _ptr(rho), n_classes, m, _ptr(dense),
                                        dense.shape[1], dense.stride(0), None, None, None, 0, _ptr(out),
                                        max_mem_bytes, _stream()))
    else:
        val, row_ptr, col = csr
        m = row_ptr.numel() - 1
        out = torch.empty(m, dtype=torch.int32, device="cuda")
        check(lib().tsvm_predict_labels(km_sv.handle, _ptr(coef), cnt, _ptr(rho), n_classes, m, None, 0, 0, _ptr(val),
                                        _ptr(row_ptr), _ptr(col), val.numel(), _ptr(out), max_mem_bytes, _stream()))
    return out


def vote(dec, n_classes):
    out = torch.empty(dec.shape[0], dtype=torch.int32, device="cuda")
    check(lib().tsvm_vote(_ptr(dec), dec.shape[0], n_classes, _ptr(out), _stream()))
    return out

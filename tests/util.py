"""Helpers shared by the tests: problem views for the oracle and for the device library."""
import numpy as np


def binary_labels(prob, split=None):
    y = prob["y"]
    return (np.where(y > 0, 1, -1) if split is None else np.where(y < split, 1, -1)).astype(np.int32)


def oracle_matrix(P, prob, n=None):
    """prob (thundersvm_b200.synth dict) -> oracle.port_binding.Csr."""
    if "X" in prob:
        return P.Csr(dense=prob["X"][:n])
    val, rp, col = prob["csr"]
    if n is not None:
        rp = rp[:n + 1]
        val, col = val[:rp[-1]], col[:rp[-1]]
    return P.Csr(csr=(val, rp, col), d=prob["d"])


def device_matrix(capi, prob, n=None, force=None, **kw):
    """prob -> capi.KernelMatrix on the GPU. force='csr' stores dense data as CSR (explicit zeros
    dropped), force='dense' densifies CSR data."""
    import torch
    kw.setdefault("gamma", prob["gamma"])
    if "X" in prob:
        X = prob["X"][:n]
        if force == "csr":
            mask = X != 0
            rp = np.concatenate([[0], np.cumsum(mask.sum(1))]).astype(np.int32)
            col = np.nonzero(mask)[1].astype(np.int32)
            val = X[mask].astype(np.float32)
            return capi.KernelMatrix(csr=(torch.from_numpy(val).cuda(), torch.from_numpy(rp).cuda(),
                                          torch.from_numpy(col).cuda()), d=X.shape[1], **kw)
        return capi.KernelMatrix(dense=torch.from_numpy(np.ascontiguousarray(X)).cuda(), **kw)
    val, rp, col = prob["csr"]
    if n is not None:
        rp = rp[:n + 1]
        val, col = val[:rp[-1]], col[:rp[-1]]
    if force == "dense":
        X = np.zeros((len(rp) - 1, prob["d"]), dtype=np.float32)
        rows = np.repeat(np.arange(len(rp) - 1), np.diff(rp))
        X[rows, col] = val
        return capi.KernelMatrix(dense=torch.from_numpy(X).cuda(), **kw)
    return capi.KernelMatrix(csr=(torch.from_numpy(val).cuda(), torch.from_numpy(rp.astype(np.int32)).cuda(),
                                  torch.from_numpy(col).cuda()), d=prob["d"], **kw)


def rel_err(a, b, floor=1e-4):
    """Kernel-value error metric: max |a-b| / max(|b|, floor). Relative error for values of at least
    `floor`; below it the difference is measured against the floor (for an RBF value of 1e-9 a relative
    error of 1e-5 is a quarter of an ulp of the exponent's argument and cannot be held by two different
    FP32 evaluation orders, the reference's own two backends included)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), floor)))


def rel_err_pure(a, b):
    """Un-floored relative error max |a-b| / |b| over the entries with b != 0 (reported next to rel_err)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    m = b != 0
    return float(np.max(np.abs(a[m] - b[m]) / np.abs(b[m]))) if m.any() else 0.0


def objective(alpha, f, y):
    return -float(np.sum(alpha - (f + y) * alpha * y / 2))

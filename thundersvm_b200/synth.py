"""Seeded synthetic stand-ins for the five benchmark configurations.

No public dataset is read or reproduced: each generator only borrows the *shape*
(rows, columns, density, value law) of the problem it stands in for.  Every generator
draws rows in fixed-size chunks from `numpy.random.default_rng(seed)` so that asking for
fewer rows (`n=...`) yields a prefix of the full problem.

Returned problems are dicts:
  dense : {"X": float32[n, d], "y": float32[n], ...params}
  sparse: {"csr": (val float32[nnz], row_ptr int32[n+1], col int32[nnz]), "d": d, "y": ...}
Column ids are 0-based.
"""
import numpy as np

_CHUNK = 8192


def _chunks(n):
    for s in range(0, n, _CHUNK):
        yield s, min(n, s + _CHUNK)


def config1(n=10000, seed=1):
    """Two Gaussian blobs N(+-0.5*1, I) clipped to [-3, 3], 5% label flips; 10,000 x 20 dense."""
    d = 20
    rng = np.random.default_rng(seed)
    X = np.empty((n, d), dtype=np.float32)
    y = np.empty(n, dtype=np.float32)
    for s, e in _chunks(n):
        c = np.where(rng.random(e - s) < 0.5, 1.0, -1.0)
        X[s:e] = np.clip(rng.standard_normal((e - s, d)) + 0.5 * c[:, None], -3, 3)
        flip = rng.random(e - s) < 0.05
        y[s:e] = np.where(flip, -c, c)
    return dict(name="c1_dense_10000x20", X=X, y=y, gamma=0.5, C=10.0, eps=1e-3, kernel="rbf")


def _binary_rows(n, d, k, rng):
    """n rows with exactly k ones at distinct uniformly random columns (sorted)."""
    keys = rng.random((n, d))
    cols = np.argpartition(keys, k, axis=1)[:, :k]
    cols.sort(axis=1)
    return cols.astype(np.int32)


def config2(n=32561, seed=2, w_seed=2002):
    """32,561 x 123 CSR, exactly 14 ones per row; label = +1 iff w.x exceeds the 76th
    percentile of the scores (24% positive), 2% flips.  Use seed=3 with the same w_seed
    for the 16,281-row prediction set."""
    d, k = 123, 14
    w = np.random.default_rng(w_seed).standard_normal(d)
    rng = np.random.default_rng(seed)
    col = np.empty((n, k), dtype=np.int32)
    flips = np.empty(n, dtype=bool)
    for s, e in _chunks(n):
        col[s:e] = _binary_rows(e - s, d, k, rng)
        flips[s:e] = rng.random(e - s) < 0.02
    score = w[col].sum(axis=1)
    # threshold = 76th percentile of the teacher's scores on an independent calibration draw,
    # so that the training and the prediction rows (other seeds) share it
    cal = _binary_rows(50000, d, k, np.random.default_rng(w_seed + 1))
    thr = np.percentile(w[cal].sum(axis=1), 76.0)
    yy = np.where(score > thr, 1.0, -1.0)
    yy = np.where(flips, -yy, yy).astype(np.float32)
    val = np.ones(n * k, dtype=np.float32)
    row_ptr = (np.arange(n + 1, dtype=np.int64) * k).astype(np.int32)
    return dict(name="c2_sparse_32561x123", csr=(val, row_ptr, col.reshape(-1)), d=d, y=yy, gamma=0.5, C=100.0,
                eps=1e-3, kernel="rbf")


def config3(n=60000, seed=4, proto_seed=4004, n_classes=10):
    """10 class prototypes in [0,1]^784 (about 19% of pixels ~U(.5,1)) plus N(0,.1) noise,
    clipped to [0,1], values < .05 zeroed; classes balanced.  seed=5 gives the test rows."""
    d = 784
    prng = np.random.default_rng(proto_seed)
    protos = np.where(prng.random((n_classes, d)) < 0.19, prng.uniform(0.5, 1.0, (n_classes, d)), 0.0)
    rng = np.random.default_rng(seed)
    X = np.empty((n, d), dtype=np.float32)
    y = np.empty(n, dtype=np.float32)
    for s, e in _chunks(n):
        cls = rng.integers(0, n_classes, e - s)
        v = np.clip(protos[cls] + 0.1 * rng.standard_normal((e - s, d)), 0.0, 1.0)
        v[v < 0.05] = 0.0
        X[s:e] = v
        y[s:e] = cls
    return dict(name="c3_ovo_60000x784", X=X, y=y, gamma=0.125, C=10.0, eps=1e-3, kernel="rbf")


def config4(n=20242, seed=6, teacher_seed=6006):
    """20,242 x 47,236 CSR, Poisson(74) (>=1) non-zeros per row, Zipf(1.1) column ids
    without repeats inside a row, lognormal(0,1) values, rows L2-normalised; labels are the
    sign of a 500-non-zero N(0,1) teacher."""
    d = 47236
    trng = np.random.default_rng(teacher_seed)
    rng = np.random.default_rng(seed)
    p = 1.0 / np.arange(1, d + 1) ** 1.1
    cdf = np.cumsum(p / p.sum())
    # teacher on frequently used columns so that the labels are not all of one sign
    t_cols = np.unique(np.searchsorted(cdf, trng.random(4000)))[:500]
    teacher = np.zeros(d)
    teacher[t_cols] = trng.standard_normal(len(t_cols))
    vals, cols, row_ptr = [], [], [0]
    score = np.empty(n)
    for i in range(n):
        k = max(1, int(rng.poisson(74)))
        c = np.unique(np.minimum(np.searchsorted(cdf, rng.random(2 * k + 8)), d - 1))
        if len(c) > k:
            c = np.sort(rng.choice(c, k, replace=False))
        v = rng.lognormal(0.0, 1.0, len(c))
        v /= np.sqrt((v * v).sum())
        vals.append(v.astype(np.float32))
        cols.append(c.astype(np.int32))
        row_ptr.append(row_ptr[-1] + len(c))
        score[i] = (teacher[c] * v).sum()
    thr = np.median(score) - 0.05 * score.std()      # lands near 52% positive
    y = np.where(score > thr, 1.0, -1.0).astype(np.float32)
    return dict(name="c4_sparse_20242x47236", csr=(np.concatenate(vals), np.asarray(row_ptr, dtype=np.int32),
                                                  np.concatenate(cols)), d=d, y=y, gamma=1.0, C=100.0, eps=1e-3,
                kernel="rbf")


def config5(n=400000, d=2000, seed=7, w_seed=7007, out=None):
    """n x 2000 rows ~N(0,1) L2-normalised; label = sign(w.x), 10% flips.  seed=8 gives the
    prediction rows.  `out` may be a preallocated float32[n, d] array (e.g. pinned)."""
    w = np.random.default_rng(w_seed).standard_normal(d).astype(np.float32)
    rng = np.random.default_rng(seed)
    X = out if out is not None else np.empty((n, d), dtype=np.float32)
    y = np.empty(n, dtype=np.float32)
    for s, e in _chunks(n):
        v = rng.standard_normal((e - s, d), dtype=np.float32)
        v /= np.sqrt((v * v).sum(axis=1, keepdims=True))
        X[s:e] = v
        lab = np.where(v @ w > 0, 1.0, -1.0)
        flip = rng.random(e - s) < 0.10
        y[s:e] = np.where(flip, -lab, lab)
    return dict(name="c5_dense_%dx%d" % (n, d), X=X, y=y, gamma=0.5, C=1.0, eps=1e-3, kernel="rbf")


CONFIGS = {1: config1, 2: config2, 3: config3, 4: config4, 5: config5}

"""The column-sharded driver with its GPU back end (C ABI) on one GPU: with a single shard it must
reproduce tsvm_smo_solve; with the problem cut into two shards that are solved by one process in turn
(emulating two ranks' data placement is covered by the gloo tests) the results stay within tolerance."""
import numpy as np
import pytest

from thundersvm_b200 import synth
from util import binary_labels

pytestmark = pytest.mark.gpu


def test_single_shard_equals_plain_solver(capi):
    import torch
    from thundersvm_b200 import sharded
    prob = synth.config5(3000, d=256)
    y = binary_labels(prob)
    n = len(y)
    X = torch.from_numpy(prob["X"]).cuda()
    yt = torch.from_numpy(y).cuda()
    a1 = torch.zeros(n, dtype=torch.float64, device="cuda")
    f1 = -yt.to(torch.float64)
    km = capi.KernelMatrix(dense=X, gamma=prob["gamma"])
    rho1, st1 = capi.smo_solve(km, yt, a1, f1, 1e-3, 1.0, 1.0, 1024)
    a2 = torch.zeros(n, dtype=torch.float64, device="cuda")
    f2 = -yt.to(torch.float64)
    sv = sharded.ShardedSolver(sharded.CapiOps(), X, yt, a2, f2, n, 0, 1e-3, 1.0, 1.0, 1024, gamma=prob["gamma"])
    rho2, st2 = sv.solve()
    assert abs(st2["objective"] - st1["objective"]) <= 1e-6 * abs(st1["objective"])
    assert abs(rho2 - rho1) < 1e-6
    assert st2["outer_iters"] == st1["outer_iters"]
    assert torch.allclose(a1, a2, atol=1e-8)


def test_rows_for_features_equals_rows_by_index(capi):
    import torch
    prob = synth.config5(2000, d=512)
    X = torch.from_numpy(prob["X"]).cuda()
    km = capi.KernelMatrix(dense=X, gamma=prob["gamma"])
    idx = torch.arange(5, 1500, 7, dtype=torch.int32, device="cuda")
    a = km.get_rows(idx)
    b = km.rows_for_features(X[idx.long()].contiguous(), km.self_dot()[idx.long()].contiguous())
    assert torch.equal(a, b)

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


def test_native_single_shard_is_bit_identical_to_plain_solver(capi):
    """tsvm_shard_* with one shard: same working sets, same kernel values, same local solver - alpha, f and
    the iteration counts equal those of tsvm_smo_solve exactly."""
    import torch
    from thundersvm_b200 import sharded
    prob = synth.config5(5000, d=256)
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
    sv = sharded.NativeShardedSolver(X, yt, a2, f2, n, 0, 1e-3, 1.0, 1.0, 1024, gamma=prob["gamma"])
    rho2, st2 = sv.solve()
    assert st2["outer_iters"] == st1["outer_iters"] and st2["local_iters"] == st1["local_iters"]
    assert torch.equal(a1, a2) and torch.equal(f1, f2)
    assert abs(rho2 - rho1) < 1e-12 and abs(st2["objective"] - st1["objective"]) <= 1e-12 * abs(st1["objective"])
    sv.close()


def _native_rank(rank, world, port, n, d, out_path):
    import os
    import torch
    import torch.distributed as dist
    from thundersvm_b200 import sharded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    prob = synth.config5(n, d=d)
    y = binary_labels(prob)
    lo, hi = sharded.shard_range(n, rank, world)
    X = torch.from_numpy(prob["X"][lo:hi]).cuda()
    yt = torch.from_numpy(y[lo:hi]).cuda()
    a = torch.zeros(hi - lo, dtype=torch.float64, device="cuda")
    f = -yt.to(torch.float64)
    sv = sharded.NativeShardedSolver(X, yt, a, f, n, lo, 1e-3, 1.0, 1.0, 1024, gamma=prob["gamma"])
    rho, st = sv.solve()
    parts = [torch.empty(sharded.shard_range(n, r, world)[1] - sharded.shard_range(n, r, world)[0],
                         dtype=torch.float64, device="cuda") for r in range(world)]
    dist.all_gather(parts, a)
    if rank == 0:
        np.savez(out_path, alpha=torch.cat(parts).cpu().numpy(), rho=rho, obj=st["objective"],
                 outer=st["outer_iters"], local=st["local_iters"])
    sv.close()
    dist.destroy_process_group()


def test_native_two_shards_are_bit_identical_to_one_gpu(capi, tmp_path):
    """Two ranks on two GPUs (NCCL): every rank computes the same working sets and the same block, the
    columns are disjoint - the gathered alpha equals the one-GPU result exactly."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    n, d = 6000, 256
    out = str(tmp_path / "two.npz")
    mp.spawn(_native_rank, args=(2, 29533, n, d, out), nprocs=2, join=True)
    got = np.load(out)
    prob = synth.config5(n, d=d)
    y = binary_labels(prob)
    yt = torch.from_numpy(y).cuda()
    a1 = torch.zeros(n, dtype=torch.float64, device="cuda")
    f1 = -yt.to(torch.float64)
    km = capi.KernelMatrix(dense=torch.from_numpy(prob["X"]).cuda(), gamma=prob["gamma"])
    rho1, st1 = capi.smo_solve(km, yt, a1, f1, 1e-3, 1.0, 1.0, 1024)
    assert int(got["outer"]) == st1["outer_iters"] and int(got["local"]) == st1["local_iters"]
    assert np.array_equal(got["alpha"], a1.cpu().numpy())
    assert abs(float(got["rho"]) - rho1) < 1e-9


def test_one_vs_one_on_the_gpu_matches_the_oracle_back_end(capi):
    """train_ovo / predict_ovo with the C-ABI back end against the same driver with the oracle behind it: same
    support-vector sets up to the 0.5 % bound, same labels."""
    import os
    import sys
    import torch
    from thundersvm_b200 import sharded
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from cpu_ops import OracleOps
    rng = np.random.default_rng(3)
    k, per, d = 5, 120, 64
    centres = rng.standard_normal((k, d))
    lab = np.repeat(np.arange(k), per)
    X = (centres[lab] + 0.9 * rng.standard_normal((k * per, d))).astype(np.float32)
    T = (centres[np.arange(200) % k] + 0.9 * rng.standard_normal((200, d))).astype(np.float32)
    gamma = 1.0 / d
    ref = sharded.train_ovo(OracleOps(), torch.from_numpy(X), lab, C=10.0, gamma=gamma)
    ref_pred = sharded.predict_ovo(OracleOps(), ref, torch.from_numpy(X), torch.from_numpy(T), gamma=gamma).numpy()
    Xd, Td = torch.from_numpy(X).cuda(), torch.from_numpy(T).cuda()
    got = sharded.train_ovo(sharded.CapiOps(), Xd, lab, C=10.0, gamma=gamma)
    pred = sharded.predict_ovo(sharded.CapiOps(), got, Xd, Td, gamma=gamma).cpu().numpy()
    assert abs(sum(got["n_sv"]) - sum(ref["n_sv"])) <= max(1, 0.005 * sum(ref["n_sv"]))
    assert np.max(np.abs(got["rho"] - ref["rho"])) < 1e-3
    assert (pred == ref_pred).mean() >= 0.999
    assert (pred == np.arange(200) % k).mean() > 0.9


def test_one_vs_one_pairs_on_several_streams_give_the_same_model(capi):
    """train_ovo(streams=3) solves the pairs from three host threads on three CUDA streams; the pairs are
    independent, so every coefficient, rho and the SV set must equal the one-stream run's exactly."""
    import torch
    from thundersvm_b200 import sharded
    prob = synth.config3(6000)
    X = torch.from_numpy(prob["X"]).cuda()
    lab = prob["y"].astype(np.int64)
    one = sharded.train_ovo(sharded.CapiOps(), X, lab, C=prob["C"], gamma=prob["gamma"])
    for _ in range(3):
        many = sharded.train_ovo(sharded.CapiOps(), X, lab, C=prob["C"], gamma=prob["gamma"], streams=3)
        assert many["n_sv"] == one["n_sv"]
        assert np.array_equal(many["sv_index"], one["sv_index"])
        assert np.array_equal(many["coef"], one["coef"]) and np.array_equal(many["rho"], one["rho"])


def test_three_call_form_of_one_shard_equals_the_plain_solver(capi):
    """tsvm_shard_candidates / _select / _iterate - the form a caller with its own collectives drives, here with
    one shard and plain copies in place of the collectives - must give the plain solver's alpha, f and counts."""
    import torch
    prob = synth.config5(5000, d=256)
    y = binary_labels(prob)
    n = len(y)
    X = torch.from_numpy(prob["X"]).cuda()
    yt = torch.from_numpy(y).cuda()
    a1 = torch.zeros(n, dtype=torch.float64, device="cuda")
    f1 = -yt.to(torch.float64)
    km1 = capi.KernelMatrix(dense=X, gamma=prob["gamma"])
    _, st1 = capi.smo_solve(km1, yt, a1, f1, 1e-3, 1.0, 1.0, 1024)
    km1.close()
    a2 = torch.zeros(n, dtype=torch.float64, device="cuda")
    f2 = -yt.to(torch.float64)
    km2 = capi.KernelMatrix(dense=X, gamma=prob["gamma"])
    sh = capi.Shard(km2, yt, a2, f2, n, 0, 1e-3, 1.0, 1.0, 1024, 1)
    done, steps = False, 0
    while not done:
        lists, want = sh.candidates()
        m = lists * want
        sh.all_f[:m].copy_(sh.cand_f[:m])
        sh.all_id[:m].copy_(sh.cand_id[:m])
        sh.select()
        done = sh.iterate()
        steps += 1
        assert steps < 5000
    st2 = sh.stats()
    assert steps == st1["outer_iters"] == st2["outer_iters"] and st2["local_iters"] == st1["local_iters"]
    assert torch.equal(a1, a2) and torch.equal(f1, f2)
    sh.close()
    km2.close()

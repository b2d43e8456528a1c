"""Host logic of the column-sharded multi-GPU solver, run as gloo ranks on the CPU with the oracle as
the numerical back end (tests/cpu_ops.py). The GPU back end itself is covered by the gpu-marked tests."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import port_binding as P
from thundersvm_b200 import sharded, synth
from util import binary_labels, oracle_matrix


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _problem(solver):
    prob = dict(synth.config1(640), gamma=0.05)
    y = binary_labels(prob)
    n = len(y)
    if solver == "c":
        return prob, y, np.zeros(n), -y.astype(np.float64), 1.0
    a0 = np.zeros(n)
    sp = sn = 0.3 * n / 2
    for i in range(n):
        if y[i] > 0:
            a0[i] = min(1.0, sp); sp -= a0[i]
        else:
            a0[i] = min(1.0, sn); sn -= a0[i]
    return prob, y, a0, np.zeros(n), 1.0


def _run_rank(rank, world, port, solver, out_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from cpu_ops import OracleOps
    if world > 1:
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    prob, y, a0, f0, C = _problem(solver)
    n = len(y)
    lo, hi = sharded.shard_range(n, rank, world)
    if solver != "c":
        # init_f is applied by the caller in the sharded form: f0 -= sum alpha_i y_i K_i (csmosolver.cpp:189-214)
        X = oracle_matrix(P, prob)
        nz = np.nonzero(a0)[0].astype(np.int32)
        f0 = P.update_f(f0, -a0[nz] * y[nz], P.kernel_rows_idx(X, nz, gamma=prob["gamma"]))
    sv = sharded.ShardedSolver(OracleOps(), torch.from_numpy(prob["X"][lo:hi].copy()), torch.from_numpy(y[lo:hi].copy()),
                               torch.from_numpy(a0[lo:hi].copy()), torch.from_numpy(f0[lo:hi].copy()), n, lo, 1e-3, C, C,
                               128, solver=solver, gamma=prob["gamma"])
    rho, st = sv.solve()
    np.savez(os.path.join(out_dir, "r%d.npz" % rank), alpha=sv.alpha.numpy(), f=sv.f.numpy(), rho=rho,
             obj=st["objective"], iters=st["outer_iters"], lo=lo, hi=hi)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("solver", ["c", "nu_svc"])
@pytest.mark.parametrize("world", [1, 2, 3])
def test_sharded_solver_matches_single_process_oracle(tmp_path, solver, world):
    port = _free_port()
    if world == 1:
        _run_rank(0, 1, port, solver, str(tmp_path))
    else:
        mp.spawn(_run_rank, args=(world, port, solver, str(tmp_path)), nprocs=world, join=True)
    parts = [np.load(tmp_path / ("r%d.npz" % r)) for r in range(world)]
    alpha = np.concatenate([p["alpha"] for p in parts])
    f = np.concatenate([p["f"] for p in parts])
    assert [int(p["lo"]) for p in parts] == [sharded.shard_range(640, r, world)[0] for r in range(world)]
    assert all(abs(float(p["rho"]) - float(parts[0]["rho"])) == 0 for p in parts)      # replicated scalars agree
    prob, y, a0, f0, C = _problem(solver)
    X = oracle_matrix(P, prob)
    ref = P.smo_solve(X, y, a0, f0, 1e-3, C, C, 128, solver=solver, gamma=prob["gamma"], cuda_semantics=1)
    assert abs(float(parts[0]["obj"]) - ref["obj"]) <= 1e-4 * abs(ref["obj"])
    assert abs(float(parts[0]["rho"]) - ref["rho"]) < 1e-3
    assert abs(int((alpha != 0).sum()) - int((ref["alpha"] != 0).sum())) <= max(1, 0.005 * (ref["alpha"] != 0).sum())
    assert np.linalg.norm(alpha - ref["alpha"]) <= 1e-2 * np.linalg.norm(ref["alpha"])
    assert np.max(np.abs(f - ref["f"])) < 5e-3


def test_partition_helpers():
    for n, world in ((400000, 8), (10, 4), (7, 8), (640, 3)):
        r = [sharded.shard_range(n, k, world) for k in range(world)]
        assert r[0][0] == 0 and r[-1][1] == n
        assert all(r[k][1] == r[k + 1][0] for k in range(world - 1))
    pairs, owner = sharded.assign_pairs([6000] * 10, 8)
    assert len(pairs) == 45 and sorted(set(owner)) == list(range(8))
    load = [sum(1 for o in owner if o == w) for w in range(8)]
    assert max(load) - min(load) <= 1
    rows = [sharded.predict_rows(10001, k, 4) for k in range(4)]
    assert rows[0][0] == 0 and rows[-1][1] == 10001 and all(rows[k][1] == rows[k + 1][0] for k in range(3))


def test_combine_rho_matches_oracle_formulas():
    rng = np.random.default_rng(0)
    n = 500
    y = np.where(rng.random(n) < 0.5, 1, -1).astype(np.int32)
    a = rng.choice([0.0, 1.0, 0.4], n)
    f = rng.standard_normal(n)
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from cpu_ops import OracleOps
    ops = OracleOps()
    parts = [ops.rho_partials(torch.from_numpy(f[s]), torch.from_numpy(a[s]), torch.from_numpy(y[s]), 1.0, 1.0).numpy()
             for s in (slice(0, 200), slice(200, 500))]
    rho, obj, _ = sharded.combine_rho(parts, "c")
    free = (a > 0) & (a < 1.0)
    assert abs(rho - f[free].mean()) < 1e-12
    assert abs(obj - P.objective(f, a, y)) < 1e-9


def _ovo_problem():
    """Four classes on a circle in 8 dimensions, 70 instances each, class index in order of first appearance."""
    rng = np.random.default_rng(11)
    k, per, d = 4, 70, 8
    centres = rng.standard_normal((k, d)) * 1.5
    lab = rng.permutation(np.repeat(np.arange(k), per))
    first = {}
    for c in lab:
        first.setdefault(int(c), len(first))
    lab = np.array([first[int(c)] for c in lab])
    X = (centres[lab] + rng.standard_normal((k * per, d))).astype(np.float32)
    T = (centres[np.arange(40) % k] + rng.standard_normal((40, d))).astype(np.float32)
    return X, lab, T


def _ovo_rank(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from cpu_ops import OracleOps
    if world > 1:
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    X, lab, T = _ovo_problem()
    ops = OracleOps()
    model = sharded.train_ovo(ops, torch.from_numpy(X), lab, C=10.0, gamma=0.2)
    pred = sharded.predict_ovo(ops, model, torch.from_numpy(X), torch.from_numpy(T), gamma=0.2)
    np.savez(os.path.join(out_dir, "ovo%d.npz" % rank), coef=model["coef"], rho=model["rho"], sv=model["sv_index"],
             n_sv=np.asarray(model["n_sv"]), pred=pred.numpy(), owner=np.asarray(model["owner"]))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_one_vs_one_pairs_sharded_over_ranks(tmp_path, world):
    """The six binary problems of a four-class set are split over the ranks; after the gather every rank
    holds the same model, equal to the one a single process trains, and the row-sharded prediction returns
    the same labels as the single process."""
    single = tmp_path / "single"
    single.mkdir()
    _ovo_rank(0, 1, 0, str(single))
    ref = np.load(single / "ovo0.npz")
    multi = tmp_path / "multi"
    multi.mkdir()
    mp.spawn(_ovo_rank, args=(world, _free_port(), str(multi)), nprocs=world, join=True)
    parts = [np.load(multi / ("ovo%d.npz" % r)) for r in range(world)]
    assert sorted(set(parts[0]["owner"].tolist())) == list(range(world))        # every rank solved something
    for p in parts:
        assert np.array_equal(p["sv"], ref["sv"]) and np.array_equal(p["n_sv"], ref["n_sv"])
        assert np.array_equal(p["coef"], ref["coef"]) and np.array_equal(p["rho"], ref["rho"])
        assert np.array_equal(p["pred"], ref["pred"])
    # and the model is a sensible classifier of its own training distribution
    X, lab, T = _ovo_problem()
    truth = np.arange(40) % 4
    assert (ref["pred"] == truth).mean() > 0.8
    assert ref["coef"].shape == (3, int(ref["n_sv"].sum()))


def test_working_set_size_helper_matches_the_library():
    import ctypes
    from thundersvm_b200 import build
    lib = ctypes.CDLL(build.build())
    f = lib.tsvm_working_set_size
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t]
    for n, d in ((150, 5), (1000, 785), (12025, 785), (400000, 2001), (3, 2), (2049, 64)):
        assert sharded.working_set_size(n, d) == f(n, d, 8 << 30, 0), (n, d)


def _arrival_rank(rank, world, port, out_dir, late_rank):
    """Every rank joins the process group; `late_rank` then stays away from the arrival check (as a rank
    that raised or hangs before its first collective would)."""
    import time
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    result = "ok"
    if rank == late_rank:
        time.sleep(6.0)                    # never arrives within the limit
        result = "late"
    else:
        t0 = time.time()
        try:
            sharded.wait_for_peers(None, timeout_s=2.0)
        except sharded.PeerTimeout as exc:
            result = "timeout after %.1f s: %s" % (time.time() - t0, str(exc)[:200])
    with open(os.path.join(out_dir, "arrival%d.txt" % rank), "w") as f:
        f.write(result)


def test_missing_rank_is_reported_by_the_arrival_check(tmp_path):
    """Failure detection on the host: a rank that does not show up makes the others give up after the limit
    with an error that names it, instead of blocking in the first collective of the solve."""
    port = _free_port()
    mp.spawn(_arrival_rank, args=(2, port, str(tmp_path), 1), nprocs=2, join=True)
    got = open(os.path.join(str(tmp_path), "arrival0.txt")).read()
    assert got.startswith("timeout after"), got
    assert float(got.split()[2]) < 5.0
    assert "1" in got.split(":", 1)[1]          # the message names rank 1
    assert open(os.path.join(str(tmp_path), "arrival1.txt")).read() == "late"


def test_all_ranks_pass_the_arrival_check(tmp_path):
    port = _free_port()
    mp.spawn(_arrival_rank, args=(2, port, str(tmp_path), -1), nprocs=2, join=True)
    assert open(os.path.join(str(tmp_path), "arrival0.txt")).read() == "ok"
    assert open(os.path.join(str(tmp_path), "arrival1.txt")).read() == "ok"

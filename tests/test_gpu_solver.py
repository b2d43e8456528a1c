"""Solver steps and the full solve on the GPU against the CPU oracle.

Tolerances (stated by the task for equivalence with the reference on the same seeded inputs):
dual objective 1e-4 relative, support-vector count 0.5 %, rho / decision values 1e-3 absolute.
Index work (working-set selection) is compared exactly."""
import os

import numpy as np
import pytest

from oracle import port_binding as P
from thundersvm_b200 import synth
from util import binary_labels, device_matrix, objective, oracle_matrix

pytestmark = pytest.mark.gpu


def _t(a, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def _state(n, seed, C=1.0, ties=False):
    rng = np.random.default_rng(seed)
    y = np.where(rng.random(n) < 0.5, 1, -1).astype(np.int32)
    f = rng.standard_normal(n)
    if ties:
        f = np.round(f * 2) / 2            # many exact ties, as at the start of training (f = -y)
    alpha = rng.choice([0.0, C, 0.3 * C, 0.7 * C], size=n, p=[0.4, 0.2, 0.2, 0.2])
    return y, f, alpha


@pytest.mark.parametrize("solver", ["c", "nu_svc"])
@pytest.mark.parametrize("n,want,ties", [(5000, 512, False), (5000, 1024, True), (700, 256, True), (130, 64, False),
                                         (40000, 512, True), (64, 32, True)])
def test_working_set_selection_is_exact(capi, solver, n, want, ties):
    import torch
    y, f, alpha = _state(n, n + want, ties=ties)
    in_ws = np.zeros(n, dtype=np.uint8)
    in_ws[np.random.default_rng(1).choice(n, min(want, n // 4), replace=False)] = 1
    sel = capi.WorkingSetSelector(n, 1024)
    kind = "c" if solver == "c" else "nu"
    for flags in (None, in_ws):
        got = sel.select(_t(f), _t(alpha), _t(y), 1.0, 1.0, want, in_ws=None if flags is None else _t(flags),
                         solver=solver).cpu().numpy()
        exp = P.select_working_set(kind, f, y, alpha, 1.0, 1.0, flags, want)
        assert np.array_equal(got, exp)


def test_working_set_selection_small_pools(capi):
    """Few eligible instances: one walk runs dry and the other fills the set; instances in both sets are
    taken once."""
    n = 300
    y = np.ones(n, dtype=np.int32)
    y[::3] = -1
    f = np.linspace(-1, 1, n)
    alpha = np.zeros(n)
    alpha[5:40] = 0.5              # free: in I_up and I_low
    sel = capi.WorkingSetSelector(n, 1024)
    for want in (16, 128, 256):
        got = sel.select(_t(f), _t(alpha), _t(y), 1.0, 1.0, want).cpu().numpy()
        exp = P.select_working_set("c", f, y, alpha, 1.0, 1.0, None, want)
        assert np.array_equal(got, exp)
        assert len(set(got.tolist())) == want


def test_candidates_then_merge_equals_select(capi):
    """The two-step form used by the column-sharded driver: per-shard candidates with global ids, then a
    merge over the concatenation."""
    import torch
    n, want = 6000, 512
    y, f, alpha = _state(n, 7, ties=True)
    sel = capi.WorkingSetSelector(n, 1024)
    parts_f, parts_i = [], []
    for lo, hi in ((0, 2500), (2500, 6000)):
        cf, ci = sel.candidates(_t(f[lo:hi]), _t(alpha[lo:hi]), _t(y[lo:hi]), 1.0, 1.0, want, id_offset=lo)
        parts_f.append(cf)
        parts_i.append(ci)
    got = sel.merge(torch.cat(parts_f, 1), torch.cat(parts_i, 1), want).cpu().numpy()
    exp = P.select_working_set("c", f, y, alpha, 1.0, 1.0, None, want)
    assert np.array_equal(got, exp)


@pytest.mark.parametrize("solver", ["c", "nu_svc"])
@pytest.mark.parametrize("shards", [1, 3, 8])
def test_sorted_runs_merge_equals_select(capi, solver, shards):
    """The form the sharded solver uses: every shard sorts its own candidate lists, the concatenated runs are
    merged by rank computation. Ties in f (broken by id), shards of unequal size, a shard with fewer
    candidates than wanted, and the nu lists."""
    import torch
    n, want = 9000, 512
    y, f, alpha = _state(n, 11, ties=True)
    sel = capi.WorkingSetSelector(n, 1024)
    cuts = [0] + sorted(np.random.default_rng(shards).choice(np.arange(200, n - 200), shards - 1, replace=False).tolist()) + [n]
    if shards == 8:
        cuts[1] = 150                                # a shard that cannot fill its lists
    parts_f, parts_i = [], []
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        cf, ci = sel.candidates(_t(f[lo:hi]), _t(alpha[lo:hi]), _t(y[lo:hi]), 1.0, 1.0, want, solver=solver, id_offset=lo)
        sel.sort_candidates(cf, ci, solver=solver)
        parts_f.append(cf)
        parts_i.append(ci)
    got = sel.merge_sorted(torch.cat(parts_f, 1), torch.cat(parts_i, 1), want, want, solver=solver).cpu().numpy()
    exp = P.select_working_set("c" if solver == "c" else "nu", f, y, alpha, 1.0, 1.0, None, want)
    assert np.array_equal(got, exp)


@pytest.mark.parametrize("solver,ws", [("c", 1024), ("c", 128), ("c", 64), ("nu_svc", 512), ("nu_svc", 32)])
def test_local_smo_matches_oracle(capi, solver, ws):
    import torch
    prob = dict(synth.config1(1500), gamma=0.05)
    X = oracle_matrix(P, prob)
    y = binary_labels(prob)
    n = len(y)
    rng = np.random.default_rng(ws)
    ids = rng.choice(n, ws, replace=False).astype(np.int32)
    rows = P.kernel_rows_idx(X, ids, gamma=prob["gamma"])
    diag = P.diag(X, gamma=prob["gamma"])
    C = 1.0
    if solver == "c":
        alpha = np.zeros(n)
        f = -y.astype(np.float64) + 0.01 * rng.standard_normal(n)
    else:
        alpha = np.where(rng.random(n) < 0.5, 1.0, 0.0)
        f = 0.3 * rng.standard_normal(n)
    kind = "c" if solver == "c" else "nu"
    a_exp, ad_exp, diff_exp = P.local_smo(kind, y, f, alpha, ids, C, C, rows, diag, 1e-3, cuda_semantics=1)
    kww = rows[:, ids]
    a_got, ad_got, diff_got = capi.local_smo(_t(kww), _t(diag[ids]), _t(y[ids]), _t(f[ids]), _t(alpha[ids]), C, C,
                                             1e-3, solver=solver)
    diff_got = diff_got.cpu().numpy()
    assert diff_got[0] == pytest.approx(diff_exp[0], rel=1e-12)
    assert diff_got[1] == diff_exp[1], "local iteration counts differ"
    assert np.allclose(a_got.cpu().numpy(), a_exp[ids], rtol=0, atol=1e-9)
    assert np.allclose(ad_got.cpu().numpy(), ad_exp, rtol=0, atol=1e-9)


@pytest.mark.parametrize("n,ws", [(10007, 1024), (333, 64), (4096, 512), (5, 2)])
def test_update_f_matches_oracle(capi, n, ws):
    rng = np.random.default_rng(n)
    rows = rng.random((ws, n), dtype=np.float32)
    ad = rng.standard_normal(ws)
    ad[rng.random(ws) < 0.5] = 0.0
    f = rng.standard_normal(n)
    exp = P.update_f(f, ad, rows)
    got = capi.update_f(_t(f), _t(ad), _t(rows)).cpu().numpy()
    assert np.allclose(got, exp, rtol=0, atol=1e-11)


CASES = {"c1": (lambda: synth.config1(1500), None, None), "c1_soft": (lambda: dict(synth.config1(1500), gamma=0.025), None, None),
         "c2": (lambda: synth.config2(1200), None, None), "c2_dense": (lambda: synth.config2(1200), None, "dense"),
         "c3": (lambda: synth.config3(900), 5, None), "c4": (lambda: synth.config4(700), None, None),
         "c5": (lambda: synth.config5(1100, d=200), None, None)}


def _solve_gpu(capi, km, y, alpha0, f0, eps, Cp, Cn, ws, solver="c", max_iter=-1):
    alpha, f = _t(alpha0, None), _t(f0, None)
    rho, stats = capi.smo_solve(km, _t(y), alpha, f, eps, Cp, Cn, ws, max_iter=max_iter, solver=solver)
    return alpha.cpu().numpy(), f.cpu().numpy(), rho, stats


@pytest.mark.parametrize("tag", sorted(CASES))
def test_solve_matches_oracle_and_reference_fixture(capi, golden_dir, tag):
    make, split, force = CASES[tag]
    prob = make()
    X = oracle_matrix(P, prob)
    y = binary_labels(prob, split)
    n = len(y)
    ws = min(1024, 2 ** int(np.log2(n)))
    km = device_matrix(capi, prob, force=force)
    a, f, rho, stats = _solve_gpu(capi, km, y, np.zeros(n), -y.astype(np.float64), 1e-3, prob["C"], prob["C"], ws)
    r = P.smo_solve(X, y, np.zeros(n), -y.astype(np.float64), 1e-3, prob["C"], prob["C"], ws, gamma=prob["gamma"])
    obj = objective(a, f, y)
    assert stats["objective"] == pytest.approx(obj, rel=1e-9)
    assert abs(obj - r["obj"]) <= 1e-4 * abs(r["obj"])
    assert abs(rho - r["rho"]) < 1e-3
    nsv, nsv_ref = int((a != 0).sum()), int((r["alpha"] != 0).sum())
    assert abs(nsv - nsv_ref) <= max(1, 0.005 * nsv_ref)
    # the f invariant: f = sum_k alpha_k y_k K(x_k, .) - y, recomputed from scratch by the oracle
    sv = np.nonzero(a)[0].astype(np.int32)
    f_chk = -y.astype(np.float64)
    for s0 in range(0, len(sv), 256):
        ids = sv[s0:s0 + 256]
        f_chk = P.update_f(f_chk, -a[ids] * y[ids], P.kernel_rows_idx(X, ids, gamma=prob["gamma"]))
    assert np.max(np.abs(f_chk - f)) < 1e-3
    # and against the committed reference outputs
    g = np.load(os.path.join(golden_dir, "solver_small.npz"))
    key = "c2" if tag == "c2_dense" else tag
    assert abs(obj - float(g[key + "_obj"])) <= 1e-4 * abs(float(g[key + "_obj"]))
    assert abs(rho - float(g[key + "_rho"])) < 1e-3
    assert stats["outer_iters"] >= 1 and stats["gpu_launches"] > 0


@pytest.mark.parametrize("solver", ["c", "nu_svc"])
def test_overlapped_iteration_is_bit_identical(capi, solver):
    """The overlapped outer iteration (local solver on a second stream, fed by a small launch that computes
    the new rows of the working-set block) must reproduce the sequential one bit for bit: same alpha, f and
    stopping point on a dense problem that runs on the tensor engine, several outer iterations long."""
    import torch
    prob = synth.config5(6000, d=200)
    y = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
    n = len(y)
    out = []
    for overlap in (False, True):
        km = capi.KernelMatrix(dense=torch.from_numpy(prob["X"]).cuda(), gamma=prob["gamma"])
        alpha = torch.zeros(n, dtype=torch.float64, device="cuda")
        if solver == "nu_svc":
            a0 = np.zeros(n)
            for cls in (1, -1):
                idx = np.nonzero(y == cls)[0]
                budget = 0.3 * n / 2
                full = int(budget)
                a0[idx[:full]] = 1.0
                a0[idx[full]] = budget - full
            alpha = torch.from_numpy(a0).cuda()
            f = torch.zeros(n, dtype=torch.float64, device="cuda")
        else:
            f = torch.from_numpy(-y.astype(np.float64)).cuda()
        sv = capi.Solver(km, torch.from_numpy(y).cuda(), alpha, f, 1e-3, 1.0, 1.0, 1024, solver=solver)
        sv.set_overlap(overlap)
        sv.iterate(12)
        st = sv.stats()
        out.append((alpha.cpu().numpy().copy(), f.cpu().numpy().copy(), st["outer_iters"], st["local_iters"]))
        sv.close()
        km.close()
    assert out[0][2] == out[1][2] and out[0][3] == out[1][3]
    assert np.array_equal(out[0][0], out[1][0])
    assert np.array_equal(out[0][1], out[1][1])
    assert out[0][2] >= 3


def test_solve_first_working_sets_follow_the_oracle(capi):
    """With max_iter = 0 the solver runs exactly one outer iteration (csmosolver.cpp:110); alpha and f
    after it must agree with the oracle closely (same working set, same local iterations)."""
    prob = synth.config1(3000)
    X = oracle_matrix(P, prob)
    y = binary_labels(prob)
    n = len(y)
    km = device_matrix(capi, prob)
    a, f, rho, stats = _solve_gpu(capi, km, y, np.zeros(n), -y.astype(np.float64), 1e-3, 10.0, 10.0, 1024, max_iter=0)
    r = P.smo_solve(X, y, np.zeros(n), -y.astype(np.float64), 1e-3, 10.0, 10.0, 1024, gamma=prob["gamma"], max_iter=0)
    assert stats["outer_iters"] == 1 and r["iters"] == 1
    assert set(np.nonzero(a)[0]) == set(np.nonzero(r["alpha"])[0])
    assert np.allclose(a, r["alpha"], atol=1e-4 * 10.0)
    assert np.allclose(f, r["f"], atol=1e-3)


@pytest.mark.parametrize("solver", ["nu_svc", "nu_svr"])
def test_nu_solve_matches_oracle(capi, solver):
    prob = synth.config1(800)
    X = oracle_matrix(P, prob)
    y = binary_labels(prob)
    n = len(y)
    nu, C = 0.3, 1.0
    a0 = np.zeros(n)
    sp = sn = nu * n / 2
    for i in range(n):
        if y[i] > 0:
            a0[i] = min(1.0, sp); sp -= a0[i]
        else:
            a0[i] = min(1.0, sn); sn -= a0[i]
    km = device_matrix(capi, prob)
    a, f, rho, stats = _solve_gpu(capi, km, y, a0, np.zeros(n), 1e-3, C, C, 512, solver=solver)
    r = P.smo_solve(X, y, a0, np.zeros(n), 1e-3, C, C, 512, solver=solver, gamma=prob["gamma"], cuda_semantics=1)
    assert abs(stats["objective"] - r["obj"]) <= 1e-4 * max(1e-12, abs(r["obj"]))
    assert abs(rho - r["rho"]) < 1e-3
    assert abs(int((a != 0).sum()) - int((r["alpha"] != 0).sum())) <= max(1, 0.005 * (r["alpha"] != 0).sum())
    assert np.linalg.norm(a - r["alpha"]) <= 1e-2 * np.linalg.norm(r["alpha"])


def test_one_class_style_init_f(capi):
    """Non-zero starting alphas exercise init_f (csmosolver.cpp:189-214)."""
    prob = synth.config1(700)
    X = oracle_matrix(P, prob)
    n = X.n
    nu = 0.2
    a0 = np.zeros(n)
    k = int(nu * n)
    a0[:k] = 1
    a0[k] = nu * n - k
    y = np.ones(n, dtype=np.int32)
    km = device_matrix(capi, prob)
    a, f, rho, stats = _solve_gpu(capi, km, y, a0, np.zeros(n), 1e-3, 1.0, 1.0, 512)
    r = P.smo_solve(X, y, a0, np.zeros(n), 1e-3, 1.0, 1.0, 512, gamma=prob["gamma"])
    assert abs(stats["objective"] - r["obj"]) <= 1e-4 * abs(r["obj"])
    assert abs(rho - r["rho"]) < 1e-3


def test_config5_generator_at_scale_against_the_reference_fixture(capi, golden_dir):
    """The reference's CPU solver run to convergence on the first N instances of the 400,000 x 2,000
    configuration's generator (tests/golden/make_c5_scale.py; the full size is not tractable on host cores):
    objective 1e-4 relative, rho 1e-3, support-vector count 0.5 %, decision values of 64 test rows 1e-3."""
    import torch
    path = os.path.join(golden_dir, "c5_scale.npz")
    if not os.path.exists(path):
        pytest.skip("fixture not generated")
    g = np.load(path)
    n = int(g["n"])
    prob = synth.config5(n)
    y = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
    X = torch.from_numpy(prob["X"]).cuda()
    km = capi.KernelMatrix(dense=X, gamma=prob["gamma"])
    yt = torch.from_numpy(y).cuda()
    alpha = torch.zeros(n, dtype=torch.float64, device="cuda")
    f = -yt.to(torch.float64)
    rho, st = capi.smo_solve(km, yt, alpha, f, 1e-3, 1.0, 1.0, 1024)
    assert abs(st["objective"] - float(g["objective"])) <= 1e-4 * abs(float(g["objective"]))
    assert abs(rho - float(g["rho"])) < 1e-3
    n_sv = int((alpha != 0).sum().item())
    assert abs(n_sv - int(g["n_sv"])) <= 0.005 * int(g["n_sv"])
    sv = torch.nonzero(alpha != 0).squeeze(1)
    order = torch.cat([sv[yt[sv] > 0], sv[yt[sv] < 0]])
    km_sv = capi.KernelMatrix(dense=X[order].contiguous(), gamma=prob["gamma"])
    coef = (alpha[order] * yt[order].to(torch.float64)).contiguous()
    test = synth.config5(64, seed=8)
    dec = capi.predict_dec(km_sv, coef, [int((yt[sv] > 0).sum()), int((yt[sv] < 0).sum())],
                           torch.tensor([rho], dtype=torch.float64, device="cuda"), 2,
                           dense=torch.from_numpy(test["X"]).cuda())
    assert np.max(np.abs(dec.cpu().numpy()[:, 0] - g["dec"])) < 1e-3


@pytest.mark.parametrize("case", ["c1_simt", "c2_csr", "c5_tensor", "c5_tensor_sequential"])
def test_row_cache_budget_does_not_change_results(capi, case):
    """Kernel-row cache: with the minimum row buffer (working set + one batch) and with room for every row the
    solver takes the same steps - alpha and f identical bit for bit - and the large cache serves hits."""
    import torch
    if case == "c1_simt":
        prob, n = synth.config1(6000), 6000
    elif case == "c2_csr":
        prob, n = synth.config2(5000), 5000
    else:
        prob, n = synth.config5(6000, d=256), 6000
    y = torch.from_numpy(binary_labels(prob)).cuda()
    out = []
    try:
        for budget in (0, 1 << 40):
            capi.set_row_cache_bytes(budget)
            km = device_matrix(capi, prob, n)
            alpha = torch.zeros(n, dtype=torch.float64, device="cuda")
            f = -y.to(torch.float64)
            sv = capi.Solver(km, y, alpha, f, 1e-3, prob["C"], prob["C"], 1024)
            if case.endswith("sequential"):
                sv.set_overlap(False)
            done = False
            while not done:
                done = sv.iterate(50)
            rho, st = sv.finish()
            out.append((alpha.cpu().numpy(), f.cpu().numpy(), rho, st))
            sv.close(); km.close()
    finally:
        capi.set_row_cache_bytes(-1)
    (a0, f0, r0, s0), (a1, f1, r1, s1) = out
    assert np.array_equal(a0, a1) and np.array_equal(f0, f1) and r0 == r1
    assert s0["outer_iters"] == s1["outer_iters"] and s0["local_iters"] == s1["local_iters"]
    assert s0["cache_rows"] == 1024 + 512 and s1["cache_rows"] == n
    assert s1["cache_hits"] + s1["cache_misses"] == s1["kernel_rows"]
    assert s1["cache_misses"] <= n and s1["cache_hits"] >= s0["cache_hits"]
    if s1["outer_iters"] > 12:
        assert s1["cache_hits"] > 0


def test_working_set_that_cannot_be_filled_is_an_error(capi):
    """A class with C = 0 (a zero class weight) belongs to neither I_up nor I_low; when the other class has fewer
    instances than the working set has slots, the reference's selection loop never ends (csmosolver.cpp:131-164).
    Here the empty slots are inert and the call fails with a message instead."""
    import torch
    prob = synth.config1(1500)
    y_np = binary_labels(prob).copy()
    y_np[:] = -1
    y_np[:300] = 1                                   # 300 eligible instances for 1024 slots
    km = device_matrix(capi, prob, 1500)
    y = torch.from_numpy(y_np).cuda()
    alpha = torch.zeros(1500, dtype=torch.float64, device="cuda")
    f = -y.to(torch.float64)
    with pytest.raises(capi.TsvmError, match="eligible"):
        capi.smo_solve(km, y, alpha, f, 1e-3, 1.0, 0.0, 1024)
    assert torch.isfinite(alpha).all() and torch.isfinite(f).all()
    km.close()


@pytest.mark.gpu
@pytest.mark.parametrize("data", ["dense_tensor", "csr"])
def test_queued_iterations_equal_single_steps(capi, data):
    """tsvm_solver_iterate queues up to eight outer iterations between reads of the device's verdict; the
    iterations queued past the one that ends the solve must be no-ops. One iteration per call, all of them in
    one call, and tsvm_smo_solve (with and without an iteration cap, csmosolver.cpp:110) must agree bit for bit."""
    import torch
    if data == "dense_tensor":
        prob = synth.config5(5000, d=200)
        make = lambda: capi.KernelMatrix(dense=torch.from_numpy(prob["X"]).cuda(), gamma=prob["gamma"])
    else:
        prob = synth.config2(4000)
        make = lambda: device_matrix(capi, prob)
    y = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
    n = len(y)

    def fresh():
        return (torch.zeros(n, dtype=torch.float64, device="cuda"), torch.from_numpy(-y.astype(np.float64)).cuda())

    # one iteration per call, until done
    km = make()
    a1, f1 = fresh()
    sv = capi.Solver(km, torch.from_numpy(y).cuda(), a1, f1, 1e-3, 1.0, 1.0, 512)
    steps = 0
    while not sv.iterate(1):
        steps += 1
        assert steps < 2000
    s1 = sv.stats()
    sv.close(); km.close()
    assert s1["outer_iters"] == steps + 1
    # all in one call: far more iterations asked for than the solve takes
    km = make()
    a2, f2 = fresh()
    sv = capi.Solver(km, torch.from_numpy(y).cuda(), a2, f2, 1e-3, 1.0, 1.0, 512)
    assert sv.iterate(s1["outer_iters"] + 50)
    s2 = sv.stats()
    sv.close(); km.close()
    assert s2["outer_iters"] == s1["outer_iters"] and s2["local_iters"] == s1["local_iters"]
    assert s2["final_diff"] == s1["final_diff"]
    assert torch.equal(a1, a2) and torch.equal(f1, f2)
    # the one-call solver
    km = make()
    a3, f3 = fresh()
    _, s3 = capi.smo_solve(km, torch.from_numpy(y).cuda(), a3, f3, 1e-3, 1.0, 1.0, 512)
    assert s3["outer_iters"] == s1["outer_iters"] and torch.equal(a1, a3) and torch.equal(f1, f3)
    km.close()
    # an iteration cap in the middle of a queue: max_iter = k means k + 1 iterations
    cap = 4
    assert s1["outer_iters"] > cap + 2
    km = make()
    a4, f4 = fresh()
    _, s4 = capi.smo_solve(km, torch.from_numpy(y).cuda(), a4, f4, 1e-3, 1.0, 1.0, 512, max_iter=cap)
    km.close()
    km = make()
    a5, f5 = fresh()
    sv = capi.Solver(km, torch.from_numpy(y).cuda(), a5, f5, 1e-3, 1.0, 1.0, 512)
    for _ in range(cap + 1):
        sv.iterate(1)
    sv.close(); km.close()
    assert s4["outer_iters"] == cap + 1
    assert torch.equal(a4, a5) and torch.equal(f4, f5)


_SYNC_EVERY_DIGEST = r"""
import hashlib
import numpy as np, torch
from thundersvm_b200 import capi, synth
prob = synth.config5(5000, d=200)
y = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
km = capi.KernelMatrix(dense=torch.from_numpy(prob["X"]).cuda(), gamma=prob["gamma"])
alpha = torch.zeros(len(y), dtype=torch.float64, device="cuda")
f = torch.from_numpy(-y.astype(np.float64)).cuda()
rho, st = capi.smo_solve(km, torch.from_numpy(y).cuda(), alpha, f, 1e-3, 1.0, 1.0, 512)
h = hashlib.sha256(alpha.cpu().numpy().tobytes() + f.cpu().numpy().tobytes()).hexdigest()
print(h, st["outer_iters"], st["local_iters"], repr(rho))
"""


def test_results_do_not_depend_on_how_many_iterations_are_queued():
    """TSVM_SYNC_EVERY (read once per process) sets how many outer iterations are queued between reads of the
    device's verdict: 1 is the reference's rhythm, 32 the most the library queues. Alpha, f, rho and the iteration
    counts must be the same for any value."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lines = []
    for k in ("1", "3", "32"):
        env = dict(os.environ, TSVM_SYNC_EVERY=k, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        r = subprocess.run([sys.executable, "-c", _SYNC_EVERY_DIGEST], env=env, capture_output=True, text=True,
                           timeout=600, cwd=root)
        assert r.returncode == 0, r.stderr[-2000:]
        lines.append(r.stdout.strip().splitlines()[-1])
    assert len(lines[0].split()[0]) == 64
    assert lines[0] == lines[1] == lines[2]

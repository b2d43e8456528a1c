"""The allocation-free working-set selection (tsvm_select_working_set_static) against the regular entry
point (tsvm_select_working_set), through the C ABI.

This file is collected last on purpose: should the static-scratch variant ever misbehave, a run that
stops at the first failure has already exercised every other test. The test must hold both in a fresh
process and after the rest of the suite has used the library, and across consecutive calls, because
all calls share one built-in scratch array that keeps the previous call's contents.
Index work is compared exactly."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _state(n, seed, ties):
    rng = np.random.default_rng(seed)
    y = np.where(rng.random(n) < 0.5, 1, -1).astype(np.int32)
    f = rng.standard_normal(n)
    if ties:
        f = np.round(f * 2) / 2
    alpha = rng.choice([0.0, 1.0, 0.3, 0.7], size=n, p=[0.4, 0.2, 0.2, 0.2])
    in_ws = np.zeros(n, dtype=np.uint8)
    in_ws[rng.choice(n, n // 10, replace=False)] = 1
    return y, f, alpha, in_ws


def test_static_selection_matches_regular_selection_on_consecutive_calls(capi):
    import torch

    def t(a):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    # consecutive calls with different sizes, solvers and tie patterns: a large call first, so that
    # a smaller one after it would see stale histogram / candidate contents if they were not cleared
    calls = [(50000, 1024, "c", True), (3000, 256, "nu_svc", True), (3000, 256, "c", False), (700, 512, "nu_svr", True),
             (50000, 512, "c", False)]
    out = torch.empty(1024, dtype=torch.int32, device="cuda")      # caller-provided output, reused
    for k, (n, want, solver, ties) in enumerate(calls):
        y, f, alpha, in_ws = _state(n, 100 + k, ties)
        sel = capi.WorkingSetSelector(n, 1024)
        for flags in (None, in_ws):
            fl = None if flags is None else t(flags)
            ref = sel.select(t(f), t(alpha), t(y), 1.0, 1.0, want, in_ws=fl, solver=solver)
            for _ in range(2):                                     # twice in a row on the same inputs
                got = capi.select_working_set_static(t(f), t(alpha), t(y), 1.0, 1.0, want, in_ws=fl, solver=solver,
                                                     out=out[:want])
                assert torch.equal(got, ref)
        sel.close()


def test_static_selection_rejects_sizes_beyond_its_scratch(capi):
    import torch
    n = 5000
    f = torch.zeros(n, dtype=torch.float64, device="cuda")
    a = torch.zeros(n, dtype=torch.float64, device="cuda")
    y = torch.ones(n, dtype=torch.int32, device="cuda")
    with pytest.raises(capi.TsvmError, match="at most 1024"):
        capi.select_working_set_static(f, a, y, 1.0, 1.0, 2048, out=torch.empty(2048, dtype=torch.int32, device="cuda"))

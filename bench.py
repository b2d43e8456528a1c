#!/usr/bin/env python
"""Benchmark of the SMO hot path on the 400,000 x 2,000 dense RBF C-SVC configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A "step" is one outer iteration of the batched SMO solver: working-set selection over all
instances, 512 new kernel rows of length n, the local solver on the 1024-wide working set and the
f update. The metric is kernel rows per second (rows of length n = 400,000):
  value : K timed steps with the data already resident in HBM (CUDA events, max over ranks); the
          window is repeated `--windows` times and the median window is reported
  e2e   : a (W+K)-step job through the C ABI starting from pinned HOST buffers - the
          host->device copy of X / y / alpha / f, the operand-plane split, the solver set-up and the
          device->host read of alpha / f / rho are inside the timed region
plus the whole training run to eps = 1e-3, the prediction of the 100,000 test rows, the HBM-bound
kernels one by one (`rooflines`), and the four smaller configurations end to end (`configs`).
`--impl reference` times the reference's own CPU implementation (oracle/_ref, built from the
reference sources with the Eigen products restated) or, if that library is absent, the C
restatement, on a bounded sample. Prints exactly one JSON line on rank 0.
"""
import argparse
import hashlib
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_FULL, D_FULL, WS, Q = 400000, 2000, 1024, 512
GAMMA, C_SVC, EPS = 0.5, 1.0, 1e-3
TRAFFIC_37888 = 388.7e6   # dram read + write bytes of one 37,888-instance launch of the kernel (ncu capture summarised in profiles/)
WORKLOAD = ("config5: binary C-SVC, RBF gamma=0.5 C=1 eps=1e-3, %dx%d dense fp32, ws=1024, 512 new kernel rows per "
            "outer iteration")
NO_CPU_CONVERGENCE = ("the CPU build cannot converge this configuration in bounded time (26,042 s published for the "
                      "same shape on 20 cores); configs c1, c2, c4 carry train-to-eps seconds of both sides")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--windows", type=int, default=5, help="timed windows of --steps steps each; the median is reported")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rows", type=int, default=N_FULL, help="instances (default: the full configuration)")
    ap.add_argument("--full-train", type=int, default=-1, help="1/0: also train to eps (default: on)")
    ap.add_argument("--train-budget-s", type=float, default=150.0)
    ap.add_argument("--cpu-sample-rows", type=int, default=20000)
    ap.add_argument("--cpu-sample-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--predict-rows", type=int, default=100000, help="test rows of the prediction measurement (0: skip)")
    ap.add_argument("--configs", default="c1,c2,c3,c4", help="smaller configurations measured end to end ('' = none)")
    ap.add_argument("--cpu-configs", default="c1,c2,c4",
                    help="configurations the CPU reference also trains to convergence (c3 takes minutes)")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-kernel rooflines and the smaller configurations")
    ap.add_argument("--workload", default="c5", choices=["c5", "c3"],
                    help="c5: the headline configuration (default); c3: the 10-class one-vs-one configuration, its 45 "
                         "binary problems and its test rows split over the GPUs")
    return ap.parse_args()


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# ----------------------------------------------------------------------------------------------
# CPU arms (reference build or restatement) on a bounded sample of the same workload
# ----------------------------------------------------------------------------------------------
def cpu_backend():
    """-> (module, kind, cores). The launcher of multi-rank runs exports OMP_NUM_THREADS=1; the CPU arm uses
    every host thread it may run on, set explicitly."""
    cores = host_threads()
    from oracle import ref_binding as R
    if R.available():
        R.lib().ref_set_threads(cores)
        return R, "reference+eigenfree", int(R.lib().ref_max_threads())
    os.environ["OMP_NUM_THREADS"] = str(cores)
    from oracle import port_binding as P
    return P, "port", cores


def cpu_sample(rows, steps):
    """Times `steps` outer iterations of the reference CPU solver on the first `rows` instances of
    the workload. -> dict(value=rows/s in full-length-row equivalents, ...)."""
    from thundersvm_b200 import synth
    B, kind, cores = cpu_backend()
    prob = synth.config5(rows)
    y = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
    a0, f0 = np.zeros(rows), -y.astype(np.float64)
    if kind != "port":
        D = B.Data(dense=prob["X"])
        _, _, _, sec = B.smo_solve(D, y, a0, f0, EPS, C_SVC, C_SVC, WS, max_iter=steps - 1, gamma=GAMMA)
    else:
        X = B.Csr(dense=prob["X"])
        t0 = time.perf_counter()
        B.smo_solve(X, y, a0, f0, EPS, C_SVC, C_SVC, WS, max_iter=steps - 1, gamma=GAMMA)
        sec = time.perf_counter() - t0
    rows_made = WS + Q * (steps - 1)
    # a row of the sample is rows/N_FULL of a full-length row
    value = rows_made / sec * (rows / N_FULL)
    return dict(value=value, unit="rows/s", cores=int(cores), kind=kind, seconds=sec, ms_per_step=sec / steps * 1e3,
                build="reference CPU sources compiled -O3 -march=x86-64-v3 -fopenmp; its three Eigen products "
                      "restated as plain loops (Eigen is not on the machine)" if kind != "port" else
                      "C restatement of the reference algorithm, -O3 -march=x86-64-v3 -fopenmp",
                sample="first %d of %d instances, %d outer iterations (%d kernel rows of length %d), scaled by "
                       "%d/%d to full-length rows" % (rows, N_FULL, steps, rows_made, rows, rows, N_FULL))


def cpu_kernel_rows(rows, ids):
    """Reference kernel rows K(x_ids, x_j), j < rows, of the workload's first `rows` instances (parity sample)."""
    from thundersvm_b200 import synth
    B, kind, _ = cpu_backend()
    prob = synth.config5(rows)
    if kind != "port":
        out, _, _ = B.kernel_rows_idx(B.Data(dense=prob["X"]), ids, gamma=GAMMA)
        return out
    return B.kernel_rows_idx(B.Csr(dense=prob["X"]), ids, gamma=GAMMA)


def cpu_train_config(tag):
    """The CPU reference trained to convergence on one of the smaller configurations -> dict."""
    from thundersvm_b200 import synth
    B, kind, cores = cpu_backend()
    if tag == "c3":
        if kind == "port":
            return None
        prob = synth.config3()
        m = B.Model("c_svc", B.Data(dense=prob["X"]), prob["y"], gamma=prob["gamma"], C_=prob["C"], eps=prob["eps"])
        out = dict(train_seconds=m.train_seconds, total_sv=int(m.total_sv), cores=cores, kind=kind)
        m.close()
        return out
    prob = {"c1": synth.config1, "c2": synth.config2, "c4": synth.config4}[tag]()
    y = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
    n = len(y)
    if kind != "port":
        D = B.Data(dense=prob["X"]) if "X" in prob else B.Data(csr=prob["csr"], d=prob["d"])
        t0 = time.perf_counter()
        a, f, rho, _ = B.smo_solve(D, y, np.zeros(n), -y.astype(np.float64), prob["eps"], prob["C"], prob["C"], WS,
                                   gamma=prob["gamma"])
        sec = time.perf_counter() - t0
    else:
        X = B.Csr(dense=prob["X"]) if "X" in prob else B.Csr(csr=prob["csr"], d=prob["d"])
        t0 = time.perf_counter()
        r = B.smo_solve(X, y, np.zeros(n), -y.astype(np.float64), prob["eps"], prob["C"], prob["C"], WS,
                        gamma=prob["gamma"])
        sec = time.perf_counter() - t0
        a, f, rho = r["alpha"], r["f"], r["rho"]
    return dict(train_seconds=sec, objective=-float(np.sum(a - (f + y) * a * y / 2)), rho=float(rho),
                n_sv=int((a != 0).sum()), cores=cores, kind=kind)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    s = cpu_sample(args.cpu_sample_rows, max(1, args.steps))
    line = {
        "impl": "reference", "metric": "kernel_rows_per_s", "value": s["value"], "unit": "rows/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": s["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32 kernel values, f64 solver",
        "data": "synthetic",
        "config": {"workload": WORKLOAD % (N_FULL, D_FULL), "l2": "inputs larger than L2"},
        "cpu_baseline": {k: s[k] for k in ("value", "unit", "cores", "kind", "sample", "build")},
        "e2e": {"value": s["value"], "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------
# B200 arm
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region (started well before it)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.path = gpu_index, None, None

    def start(self, settle_s=0.6):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            time.sleep(settle_s)          # the sampler's start-up must not fall into the timed window
        except Exception:
            self.proc = None

    def mark(self):
        """Number of samples written so far (samples taken before the window are left out of the summary)."""
        try:
            return sum(1 for _ in open(self.path))
        except Exception:
            return 0

    def stop(self, skip=0):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for k, line in enumerate(open(self.path)):
                if k < skip:
                    continue
                t = [x.strip() for x in line.split(",")]
                if len(t) < 9:
                    continue
                try:
                    sm.append(float(t[1])); mx.append(float(t[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                   t[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons),
                       samples=len(sm))
        return out


def measure_f16_peak(torch):
    """Dense FP16 GEMM throughput of this GPU (torch.matmul 8192^3, best of 10): the in-run cross-check
    of the driver-measured tensor peak the kernel-row contraction is reported against."""
    a = torch.randn(8192, 8192, device="cuda", dtype=torch.float16)
    b = torch.randn(8192, 8192, device="cuda", dtype=torch.float16)
    for _ in range(3):
        a @ b
    best = 1e9
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); a @ b; e1.record(); e1.synchronize()
        best = min(best, e0.elapsed_time(e1))
    del a, b
    return 2 * 8192 ** 3 / (best * 1e-3) / 1e12


def measured_peaks():
    """(burst TF/s, sustained TF/s, HBM GB/s, source): the driver-written file at the repo root, else the pool's
    earlier measurement."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            m = json.load(fh)
        return (float(m["bf16_tflops"]), float(m["bf16_tflops_sustained"]), float(m["hbm_gbs"]),
                "of measured (MEASURED_PEAKS.json)")
    except Exception:
        return 1590.0, 1400.0, 6650.0, "of fallback (1.59 PFLOP/s burst, 6.65 TB/s)"


def sha(t):
    return hashlib.sha256(np.ascontiguousarray(t).tobytes()).hexdigest()[:16]


def timed_windows(torch, run_window, windows, barrier=None):
    """-> list of ms, one per window; run_window() runs exactly K steps and returns False when nothing is left."""
    out = []
    for _ in range(windows):
        if barrier:
            barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        alive = run_window()
        e1.record()
        torch.cuda.synchronize()
        if barrier:
            barrier()
        out.append(e0.elapsed_time(e1))
        if not alive:
            break
    return out


def hbm_roofline(name, bytes_per_call, us, hbm_peak, peak_src, note):
    gbs = bytes_per_call / (us * 1e-6) / 1e9
    return {"kernel": name, "bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
            "algorithmic_bytes": bytes_per_call, "us_per_call": us, "peak_source": peak_src, "note": note}


def time_calls(torch, fn, reps, warm=3, windows=5):
    """us per call: median of `windows` windows of `reps` back-to-back calls (CUDA events)."""
    for _ in range(warm):
        fn()
    out = []
    for _ in range(windows):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) * 1e3 / reps)
    return float(np.median(out))


def extra_rooflines(torch, capi, synth, hbm_peak, peak_src, n):
    """The HBM-bound kernels one by one, CUDA events over many calls: f update, working-set selection, CSR rows."""
    out = []
    # f update: all 1024 rows carry a non-zero alpha_diff (the byte formula's upper case)
    rows = torch.rand((WS, n), dtype=torch.float32, device="cuda")
    f = torch.zeros(n, dtype=torch.float64, device="cuda")
    ad = torch.rand(WS, dtype=torch.float64, device="cuda") + 0.5
    us = time_calls(torch, lambda: capi.update_f(f, ad, rows), 20)
    out.append(hbm_roofline("update_f_kernel (config 5: 1024 rows x %d)" % n, WS * n * 4 + 16 * n, us, hbm_peak, peak_src,
                            "bytes = ws_nz*n*4 + 2*n*8, every row non-zero"))
    del rows
    # selection of 512 new members out of n
    yv = torch.where(torch.rand(n, device="cuda") < 0.5, 1, -1).to(torch.int32)
    fv = torch.randn(n, dtype=torch.float64, device="cuda")
    av = torch.where(torch.rand(n, device="cuda") < 0.3, 1.0, 0.0).to(torch.float64) * torch.rand(n, device="cuda").to(torch.float64)
    flags = torch.zeros(n, dtype=torch.uint8, device="cuda")
    sel = capi.WorkingSetSelector(n, WS)
    us = time_calls(torch, lambda: sel.select(fv, av, yv, 1.0, 1.0, Q, in_ws=flags), 50)
    out.append(hbm_roofline("working-set selection (radix top-k + merge, config 5: 512 of %d)" % n, n * 21, us, hbm_peak,
                            peak_src, "bytes = n*(8 f + 8 alpha + 4 y + 1 flag) read once; the selection is one cooperative "
                                      "launch of two or three sweeps separated by grid barriers plus an exact sort of the "
                                      "candidates by one block: a latency chain, not bandwidth-bound"))
    sel.close()
    del yv, fv, av, flags, f
    # CSR kernel rows, 512 rows per call
    for tag, make in (("c2", synth.config2), ("c4", synth.config4)):
        prob = make()
        val, rp, col = prob["csr"]
        km = capi.KernelMatrix(csr=(torch.from_numpy(val).cuda(), torch.from_numpy(rp).cuda(),
                                    torch.from_numpy(col).cuda()), d=prob["d"], gamma=prob["gamma"])
        nn = km.n
        idx_np = np.random.default_rng(0).choice(nn, Q, replace=False).astype(np.int32)
        idx = torch.from_numpy(idx_np).cuda()
        # row stride as in the solver's row buffer (a multiple of four floats)
        buf = torch.empty((Q, (nn + 3) // 4 * 4), dtype=torch.float32, device="cuda")
        us = time_calls(torch, lambda: km.get_rows(idx, buf), 40)
        nnz, nnz_ws = int(rp[-1]), int(np.diff(rp)[idx_np].sum())
        r = hbm_roofline("CSR kernel rows (%s: 512 rows x %d, nnz %d)" % (tag, nn, nnz),
                         Q * nn * 4 + nnz * 8 + (nn + 1) * 4 + nnz_ws * 8, us, hbm_peak, peak_src,
                         "bytes = q*n*4 out + nnz*8 + (n+1)*4 CSR read once + nnz(requested rows)*8")
        r["kernel_rows_per_s"] = Q / (us * 1e-6)
        out.append(r)
        km.close()
        del buf
    return out


def small_configs(torch, capi, synth, which, cpu_which):
    """Configurations 1-4 end to end through the C ABI from host arrays (upload inside the timed region), and the
    CPU reference trained to convergence beside them."""
    from thundersvm_b200 import sharded
    out = {}
    for tag in which:
        if tag == "c3":
            prob = synth.config3()
            ops = sharded.CapiOps()
            Xh = torch.from_numpy(prob["X"]).pin_memory()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            X = Xh.cuda(non_blocking=True)
            model = sharded.train_ovo(ops, X, prob["y"].astype(np.int64), prob["C"], prob["eps"], gamma=prob["gamma"])
            torch.cuda.synchronize()
            sec = time.perf_counter() - t0
            # the same job with the pairs solved on four streams by four host threads (same model)
            four = None
            try:
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                X4 = Xh.cuda(non_blocking=True)
                model4 = sharded.train_ovo(ops, X4, prob["y"].astype(np.int64), prob["C"], prob["eps"], gamma=prob["gamma"],
                                           streams=4)
                torch.cuda.synchronize()
                four = {"train_seconds": time.perf_counter() - t0,
                        "same_model": bool(np.array_equal(model4["coef"], model["coef"]) and
                                           np.array_equal(model4["rho"], model["rho"]))}
                del X4, model4
            except Exception as exc:                # reported, never fatal for the main line
                four = {"error": str(exc)[:200]}
            test = synth.config3(10000, seed=5)
            Th = torch.from_numpy(test["X"]).pin_memory()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            lab = sharded.predict_ovo(ops, model, X, Th.cuda(non_blocking=True), gamma=prob["gamma"]).cpu().numpy()
            sec_p = time.perf_counter() - t0
            out[tag] = {"workload": "10-class one-vs-one C-SVC, 60000x784 dense, 45 binary problems", "train_seconds": sec,
                        "pairs_on_four_streams": four, "total_sv": int(sum(model["n_sv"])), "predict_rows": 10000, "predict_rows_per_s": 10000 / sec_p,
                        "test_accuracy": float((lab == test["y"]).mean())}
            del X
        else:
            prob = {"c1": synth.config1, "c2": synth.config2, "c4": synth.config4}[tag]()
            y_np = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
            n = len(y_np)
            best = None
            for _ in range(2):                      # the second run has the library's memory pool warm
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                if "X" in prob:
                    km = capi.KernelMatrix(dense=prob["X"], gamma=prob["gamma"])
                else:
                    km = capi.KernelMatrix(csr=prob["csr"], d=prob["d"], gamma=prob["gamma"])
                y = torch.from_numpy(y_np).cuda()
                a = torch.zeros(n, dtype=torch.float64, device="cuda")
                f = -y.to(torch.float64)
                rho, st = capi.smo_solve(km, y, a, f, prob["eps"], prob["C"], prob["C"], WS)
                a_h = a.cpu()
                torch.cuda.synchronize()
                sec = time.perf_counter() - t0
                km.close()
                if best is None or sec < best["train_seconds"]:
                    best = {"workload": prob["name"], "train_seconds": sec, "objective": st["objective"], "rho": rho,
                            "n_sv": int((a_h != 0).sum()), "outer_iters": st["outer_iters"],
                            "local_iters": st["local_iters"], "kernel_rows_per_s": st["kernel_rows"] / max(st["seconds_rows"], 1e-9)}
            out[tag] = best
        if tag in cpu_which:
            try:
                out[tag]["cpu_reference"] = cpu_train_config(tag)
            except Exception as exc:
                out[tag]["cpu_reference"] = {"failed": repr(exc)}
    return out


def run_b200_arm(args):
    import torch
    import torch.distributed as dist
    from thundersvm_b200 import build, capi, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device - the B200 arm has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        # stdout carries exactly one JSON line: NCCL's own messages (it prints its version there) go to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    capi.lib()

    if args.workload == "c3":
        from thundersvm_b200 import sharded
        line = sharded.bench_ovo(args, rank, world)
        if rank == 0:
            print(json.dumps(line))
        if world > 1:
            dist.destroy_process_group()
        return

    if world > 1:
        from thundersvm_b200 import sharded
        line = sharded.bench(args, rank, world, local_rank, clock_sampler=ClockSampler(local_rank) if rank == 0 else None,
                             peaks=measured_peaks())
        if rank == 0:
            print(json.dumps(line))
        dist.destroy_process_group()
        return

    n, d = args.rows, D_FULL
    K, W = args.steps, max(3, args.warmup)
    # ---- workload in pinned host memory ---------------------------------------------------------
    Xh = torch.empty((n, d), dtype=torch.float32, pin_memory=True)
    prob = synth.config5(n, out=Xh.numpy())
    y_np = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
    yh = torch.from_numpy(y_np).pin_memory()
    fh = torch.from_numpy(-y_np.astype(np.float64)).pin_memory()
    ah = torch.zeros(n, dtype=torch.float64).pin_memory()

    f16_peak_in_run = measure_f16_peak(torch)
    peak, peak_sustained, hbm_peak, peak_src = measured_peaks()

    # ---- (1) resident: W warm-up steps, then `windows` windows of exactly K timed steps ----------------
    Xd = Xh.cuda(non_blocking=True)
    yd, fd, ad = yh.cuda(), fh.cuda(), ah.cuda()
    km = capi.KernelMatrix(dense=Xd, gamma=GAMMA)
    solver = capi.Solver(km, yd, ad, fd, EPS, C_SVC, C_SVC, WS)
    clocks = ClockSampler(local_rank)
    clocks.start()
    solver.iterate(W)
    torch.cuda.synchronize()
    skip = clocks.mark()
    stats = [solver.stats()]

    def window():
        done = solver.iterate(K)
        stats.append(solver.stats())
        return not done and stats[-1]["outer_iters"] - stats[-2]["outer_iters"] == K

    win_ms = timed_windows(torch, window, max(1, args.windows))
    clk = clocks.stop(skip)
    full = [i for i in range(len(win_ms)) if stats[i + 1]["outer_iters"] - stats[i]["outer_iters"] == K]
    pick = sorted(full, key=lambda i: win_ms[i])[len(full) // 2] if full else 0
    s0, s1 = stats[pick], stats[pick + 1]
    ms = win_ms[pick]
    steps_done = s1["outer_iters"] - s0["outer_iters"]
    rows_timed = s1["kernel_rows"] - s0["kernel_rows"]
    ms_per_step = ms / max(1, steps_done)
    value = rows_timed / (ms * 1e-3)
    launches = s1["gpu_launches"] - s0["gpu_launches"]
    sa, sb = stats[0], stats[-1]                                   # phase means over all windows
    all_steps = max(1, sb["outer_iters"] - sa["outer_iters"])
    t_rows = (sb["seconds_rows"] - sa["seconds_rows"]) / all_steps
    phases = {k: (sb["seconds_" + k] - sa["seconds_" + k]) / all_steps * 1e3 for k in ("select", "rows", "local", "update")}
    # the engine computes the rows the cache does not hold: the flops follow the misses, the metric the rows delivered
    rows_per_launch = (sb["cache_misses"] - sa["cache_misses"]) / all_steps
    flops = 2.0 * rows_per_launch * n * d
    achieved = flops / t_rows / 1e12
    # DRAM traffic per launch: ncu capture of a 37,888-instance launch of the same kernel (same d, same q),
    # scaled by the instances (the X planes and the output grow with n; the planes of the 512 rows do not)
    traffic = TRAFFIC_37888 * n / 37888.0 if TRAFFIC_37888 else None
    roofline = {"bound": "tensor",
                "kernel": "dense_rows_tc2_kernel<EPI_RBF, F16> (tcgen05 CTA pairs, two row-scaled FP16 planes, "
                          "3 MMAs per product, FP32 promotion every two k slabs, fused RBF epilogue)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "issued_frac": 3 * achieved / peak, "traffic": traffic,
                "peak_source": peak_src + " bf16_tflops burst; sustained figure %.0f; torch.matmul fp16 8192^3 best-of-10 "
                               "in this run %.0f. achieved = algorithmic 2*q*n*d flops per launch / mean CUDA-event time "
                               "of the kernel-row phase over all windows; the two-plane scheme issues 3x these flops "
                               "(issued_frac)" % (peak_sustained, f16_peak_in_run),
                "peak_in_run": f16_peak_in_run, "ms_per_launch": t_rows * 1e3, "rows_per_launch": rows_per_launch}
    cache = {"capacity_rows": sb["cache_rows"], "capacity_gb": sb["cache_rows"] * ((n + 3) // 4 * 4) * 4 / 1e9,
             "timed_windows": {"rows_delivered": sb["kernel_rows"] - sa["kernel_rows"],
                               "hits": sb["cache_hits"] - sa["cache_hits"],
                               "row_blocks": sb["row_blocks"] - sa["row_blocks"],
                               "row_blocks_saved": sb["row_blocks_saved"] - sa["row_blocks_saved"]},
             "note": "least-recently-used kernel rows kept in HBM; `value` counts rows delivered to the solver (computed "
                     "or cached), roofline.achieved counts the flops of the rows the engine computed"}
    # 16 of the timed launches' requested rows (the current working set's new half) for the parity sample
    parity_ids = None
    solver.close()
    km_keep = km
    del Xd, solver
    torch.cuda.empty_cache()

    # ---- (2) end to end from host buffers: the same (W+K)-step job -----------------------------------
    def job(max_iter, budget_s=None):
        """C-ABI job from pinned host buffers; returns (seconds, stats, rho, alpha_host, f_host, done)."""
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        km2 = capi.KernelMatrix(dense=Xh, gamma=GAMMA)               # H2D of X + split inside
        y2, f2, a2 = yh.cuda(non_blocking=True), fh.cuda(non_blocking=True), ah.cuda(non_blocking=True)
        sv = capi.Solver(km2, y2, a2, f2, EPS, C_SVC, C_SVC, WS)
        done, it = False, 0
        while not done and it < max_iter:
            step = min(50, max_iter - it)
            done = sv.iterate(step)
            it += step
            if budget_s is not None and time.perf_counter() - t0 > budget_s:
                break
        rho, st = sv.finish()
        a_host = a2.cpu()
        f_host = f2.cpu()
        torch.cuda.synchronize()
        sec = time.perf_counter() - t0
        sv.close(); km2.close()
        return sec, st, rho, a_host, f_host, done

    # kernel-row parity sample on the resident matrix, taken before it is released
    km_rows_sample = None
    if not args.no_cpu_baseline:
        pr = min(args.cpu_sample_rows, n)
        parity_ids = (np.arange(16, dtype=np.int64) * 1013 + 7) % pr
        km_rows_sample = km_keep.get_rows(torch.from_numpy(parity_ids.astype(np.int32)).cuda())[:, :pr].cpu().numpy()
    km_keep.close()
    del km_keep
    torch.cuda.empty_cache()

    sec_e2e, st_e2e, rho_e2e, a_e2e, _, _ = job(W + K)
    h2d = n * d * 4 + n * (4 + 8 + 8)
    d2h = n * 16 + 8
    e2e = {"value": st_e2e["kernel_rows"] / sec_e2e, "unit": "rows/s", "h2d_bytes_per_step": h2d / (W + K),
           "d2h_bytes_per_step": d2h / (W + K), "seconds": sec_e2e, "steps": W + K,
           "note": "one (W+K)-step job through the C ABI from pinned host buffers: H2D of X/y/alpha/f, operand-plane split, "
                   "solver set-up, steps, D2H of alpha/f/rho all inside the timed region. " + NO_CPU_CONVERGENCE}
    check = {"steps": W + K, "alpha_sha256_16": sha(a_e2e.numpy()), "rho": rho_e2e,
             "note": "state after exactly W+K outer iterations; runs on several GPUs print the same digest and compare "
                     "it with a one-GPU run of their own"}

    # ---- (3) the whole training run to eps --------------------------------------------------------
    train = None
    full_train = args.full_train if args.full_train >= 0 else 1
    if full_train:
        sec, st, rho, a_host, f_host, done = job(10 ** 9, budget_s=args.train_budget_s)
        train = {"seconds": sec, "converged": bool(done), "outer_iters": st["outer_iters"],
                 "local_iters": st["local_iters"], "final_diff": st["final_diff"], "objective": st["objective"],
                 "rho": rho, "n_sv": int((a_host != 0).sum()), "kernel_rows_per_s": st["kernel_rows"] / sec,
                 "kernel_rows": st["kernel_rows"], "cache_hits": st["cache_hits"],
                 "cache_hit_rate": st["cache_hits"] / max(1, st["kernel_rows"]), "row_blocks": st["row_blocks"],
                 "row_blocks_saved": st["row_blocks_saved"],
                 "phase_seconds": {k: st["seconds_" + k] for k in ("select", "rows", "local", "update")},
                 "cpu_reference": NO_CPU_CONVERGENCE}

    # ---- (4) prediction with the trained model: decision values + vote for the test rows -----------
    predict = None
    if train is not None and train["converged"] and args.predict_rows > 0:
        m = args.predict_rows
        Th = torch.empty((m, d), dtype=torch.float32, pin_memory=True)
        y_test = synth.config5(m, d=d, seed=8, out=Th.numpy())["y"]
        sv_idx = torch.nonzero(a_host != 0).squeeze(1)
        y_t = torch.from_numpy(y_np)
        order = torch.cat([sv_idx[y_t[sv_idx] > 0], sv_idx[y_t[sv_idx] < 0]])      # class +1 first (svc.cpp:56-108)
        n_pos = int((y_t[sv_idx] > 0).sum())
        coef_h = (a_host[order] * y_t[order].to(torch.float64)).contiguous()
        Xsv = Xh[order].cuda()
        km_sv = capi.KernelMatrix(dense=Xsv, gamma=GAMMA)
        coef_d, rho_d = coef_h.cuda(), torch.tensor([rho], dtype=torch.float64, device="cuda")
        counts = [n_pos, len(order) - n_pos]

        def run_predict(T):
            return capi.predict_labels(km_sv, coef_d, counts, rho_d, 2, dense=T)

        warm = run_predict(Th[:4096].cuda())
        Td = Th.cuda()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        labels = run_predict(Td)
        e1.record()
        torch.cuda.synchronize()
        ms_res = e0.elapsed_time(e1)
        grown = free_before - torch.cuda.mem_get_info()[0]
        del Td
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        lab_h = run_predict(Th.cuda(non_blocking=True)).cpu()
        sec_host = time.perf_counter() - t0
        n_sv = len(order)
        tfl = 2.0 * m * n_sv * d / (ms_res * 1e-3) / 1e12
        predict = {"rows": m, "n_sv": n_sv, "rows_per_s": m / (ms_res * 1e-3), "e2e_rows_per_s": m / sec_host,
                   "algorithmic_tflops": tfl, "frac_of_tensor_peak": tfl / peak, "issued_frac": 3 * tfl / peak,
                   "device_bytes_allocated_during_call": int(grown),
                   "positive_fraction": float((lab_h == 0).float().mean()),
                   "accuracy": float(((lab_h == 0).numpy() == (y_test > 0)).mean()),
                   "note": "decision values + vote of the seed-8 test rows against the trained model, coefficient sums "
                           "fused into the contraction's epilogue (no test x SV kernel block in memory); resident: test "
                           "rows in HBM, CUDA events; e2e: from pinned host rows, labels back on the host"}
        km_sv.close()
        del Xsv, warm, labels
    del Xh
    torch.cuda.empty_cache()
    capi.lib().tsvm_release_cached_memory()

    # ---- (5) the HBM-bound kernels and the smaller configurations ----------------------------------
    rooflines, configs = None, None
    if not args.no_extras:
        rooflines = extra_rooflines(torch, capi, synth, hbm_peak, peak_src, n)
        which = [t for t in args.configs.split(",") if t]
        cpu_which = [] if args.no_cpu_baseline else [t for t in args.cpu_configs.split(",") if t]
        configs = small_configs(torch, capi, synth, which, cpu_which)

    cpu, parity = None, None
    if not args.no_cpu_baseline:
        try:
            s = cpu_sample(args.cpu_sample_rows, args.cpu_sample_steps)
            cpu = {k: s[k] for k in ("value", "unit", "cores", "kind", "sample", "build")}
            want = cpu_kernel_rows(min(args.cpu_sample_rows, n), parity_ids.astype(np.int32))
            err = np.abs(km_rows_sample.astype(np.float64) - want) / np.maximum(np.abs(want), 1e-300)
            parity = {"kernel_rows_max_rel_err": float(err.max()),
                      "kernel_rows_max_rel_err_floored_1e-4": float((np.abs(km_rows_sample.astype(np.float64) - want)
                                                                     / np.maximum(np.abs(want), 1e-4)).max()),
                      "bound": 1e-5, "rows": 16, "columns": int(want.shape[1]),
                      "note": "16 kernel rows of the resident matrix against the CPU reference on the first %d "
                              "instances (the values do not depend on n)" % want.shape[1]}
        except Exception as exc:   # the baseline is reporting only; never fail the bench on it
            cpu = {"value": None, "unit": "rows/s", "cores": host_threads(), "kind": "port", "sample": "failed: %r" % exc}

    line = {
        "metric": "kernel_rows_per_s", "value": value, "unit": "rows/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 kernel values (two-plane FP16 tensor-core contraction with FP32 accumulation), f64 solver state", "data": "synthetic",
        "config": {"workload": WORKLOAD % (n, d),
                   "l2": "inputs larger than L2 (X planes %.1f GB, row buffer %.1f GB)" % (2 * n * d * 2 / 1e9,
                                                                                          WS * n * 4 / 1e9)},
        "windows_ms": win_ms, "window_reported": "median of %d windows of %d steps" % (len(full), K),
        "roofline": roofline, "rooflines": rooflines, "cpu_baseline": cpu, "parity": parity, "e2e": e2e,
        "gpu_launches": int(launches), "clocks": clk, "phase_ms_per_step": phases, "kernel_row_cache": cache,
        "check": check, "train_to_eps": train, "predict": predict, "configs": configs,
    }
    print(json.dumps(line))


def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_b200_arm(args)


if __name__ == "__main__":
    main()

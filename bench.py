#!/usr/bin/env python
"""Benchmark of the SMO hot path on the 400,000 x 2,000 dense RBF C-SVC configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A "step" is one outer iteration of the batched SMO solver: working-set selection over all
instances, 512 new kernel rows of length n, the local solver on the 1024-wide working set and the
f update. The metric is kernel rows per second (rows of length n = 400,000):
  value : K timed steps with the data already resident in HBM (CUDA events, max over ranks)
  e2e   : the same K-step job through the C ABI starting from pinned HOST buffers - the
          host->device copy of X / y / alpha / f, the operand-plane split, the solver set-up and the
          device->host read of alpha / f / rho are inside the timed region
plus, when --full-train is on (default at N=1), the whole training run to eps = 1e-3.
`--impl reference` times the reference's own CPU implementation (oracle/_ref, built from the
reference sources) or, if that library is absent, the C restatement, on a bounded sample.
Prints exactly one JSON line on rank 0.
"""
import argparse
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


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rows", type=int, default=N_FULL, help="instances (default: the full configuration)")
    ap.add_argument("--full-train", type=int, default=-1, help="1/0: also train to eps (default: on for 1 GPU)")
    ap.add_argument("--train-budget-s", type=float, default=150.0)
    ap.add_argument("--cpu-sample-rows", type=int, default=20000)
    ap.add_argument("--cpu-sample-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--predict-rows", type=int, default=100000, help="test rows of the prediction measurement (0: skip)")
    return ap.parse_args()


# ----------------------------------------------------------------------------------------------
# CPU arms (reference build or restatement) on a bounded sample of the same workload
# ----------------------------------------------------------------------------------------------
def cpu_sample(rows, steps):
    """Times `steps` outer iterations of the reference CPU solver on the first `rows` instances of
    the workload. -> dict(value=rows/s in full-length-row equivalents, ...)."""
    from thundersvm_b200 import synth
    from oracle import ref_binding as R
    prob = synth.config5(rows)
    y = np.where(prob["y"] > 0, 1, -1).astype(np.int32)
    a0, f0 = np.zeros(rows), -y.astype(np.float64)
    if R.available():
        kind, cores = "reference", R.lib().ref_max_threads()
        D = R.Data(dense=prob["X"])
        _, _, _, sec = R.smo_solve(D, y, a0, f0, EPS, C_SVC, C_SVC, WS, max_iter=steps - 1, gamma=GAMMA)
    else:
        from oracle import port_binding as P
        kind, cores = "port", os.cpu_count()
        X = P.Csr(dense=prob["X"])
        t0 = time.perf_counter()
        P.smo_solve(X, y, a0, f0, EPS, C_SVC, C_SVC, WS, max_iter=steps - 1, gamma=GAMMA)
        sec = time.perf_counter() - t0
    rows_made = WS + Q * (steps - 1)
    # a row of the sample is rows/N_FULL of a full-length row
    value = rows_made / sec * (rows / N_FULL)
    return dict(value=value, unit="rows/s", cores=int(cores), kind=kind, seconds=sec, ms_per_step=sec / steps * 1e3,
                sample="first %d of %d instances, %d outer iterations (%d kernel rows of length %d), scaled by "
                       "%d/%d to full-length rows" % (rows, N_FULL, steps, rows_made, rows, rows, N_FULL))


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
        "config": {"workload": "config5: binary C-SVC, RBF gamma=0.5 C=1 eps=1e-3, 400000x2000 dense fp32, ws=1024, "
                               "512 new kernel rows per outer iteration", "l2": "inputs larger than L2"},
        "cpu_baseline": {k: s[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": s["value"], "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------
# B200 arm
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
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
    """(burst, sustained, source) dense 16-bit tensor TFLOP/s: the driver-written file at the repo root,
    else the pool's earlier measurement."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            m = json.load(fh)
        return float(m["bf16_tflops"]), float(m["bf16_tflops_sustained"]), "of measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except Exception:
        return 1590.0, 1400.0, "of fallback (1.59 PFLOP/s burst)"


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
    peak, peak_sustained, peak_src = measured_peaks()

    # ---- (1) resident: K timed steps ------------------------------------------------------------
    Xd = Xh.cuda(non_blocking=True)
    yd, fd, ad = yh.cuda(), fh.cuda(), ah.cuda()
    km = capi.KernelMatrix(dense=Xd, gamma=GAMMA)
    solver = capi.Solver(km, yd, ad, fd, EPS, C_SVC, C_SVC, WS)
    solver.iterate(W)
    torch.cuda.synchronize()
    s0 = solver.stats()
    clocks = ClockSampler(local_rank)
    clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    solver.iterate(K)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    clk = clocks.stop()
    s1 = solver.stats()
    steps_done = s1["outer_iters"] - s0["outer_iters"]
    rows_timed = s1["kernel_rows"] - s0["kernel_rows"]
    ms_per_step = ms / max(1, steps_done)
    value = rows_timed / (ms * 1e-3)
    launches = s1["gpu_launches"] - s0["gpu_launches"]
    t_rows = (s1["seconds_rows"] - s0["seconds_rows"]) / max(1, steps_done)
    phases = {k: (s1["seconds_" + k] - s0["seconds_" + k]) / max(1, steps_done) * 1e3
              for k in ("select", "rows", "local", "update")}
    flops = 2.0 * Q * n * d
    achieved = flops / t_rows / 1e12
    # DRAM traffic per launch: ncu capture of a 37,888-instance launch of the same kernel (same d, same q),
    # scaled by the instances (the X planes and the output grow with n; the planes of the 512 rows do not)
    traffic = TRAFFIC_37888 * n / 37888.0 if TRAFFIC_37888 else None
    roofline = {"bound": "tensor",
                "kernel": "dense_rows_tc2_kernel<EPI_RBF, F16> (tcgen05 CTA pairs, two row-scaled FP16 planes, "
                          "3 MMAs per product, FP32 promotion every two k slabs, fused RBF epilogue)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "issued_frac": 3 * achieved / peak, "traffic": traffic,
                "peak_source": peak_src + "; sustained figure %.0f; torch.matmul fp16 8192^3 best-of-10 in this run "
                               "%.0f. achieved = algorithmic 2*q*n*d flops per launch / mean CUDA-event time of the "
                               "kernel-row phase; the two-plane scheme issues 3x these flops (issued_frac)"
                               % (peak_sustained, f16_peak_in_run),
                "peak_in_run": f16_peak_in_run, "ms_per_launch": t_rows * 1e3}
    solver.close()
    km.close()
    del Xd, km, solver
    torch.cuda.empty_cache()

    # ---- (2) end to end from host buffers: the same K-step job ------------------------------------
    def job(max_iter, budget_s=None):
        """C-ABI job from pinned host buffers; returns (seconds, stats, rho, alpha_host)."""
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

    sec_e2e, st_e2e, _, _, _, _ = job(W + K)
    h2d = n * d * 4 + n * (4 + 8 + 8)
    d2h = n * 16 + 8
    e2e = {"value": st_e2e["kernel_rows"] / sec_e2e, "unit": "rows/s", "h2d_bytes_per_step": h2d / (W + K),
           "d2h_bytes_per_step": d2h / (W + K), "seconds": sec_e2e, "steps": W + K,
           "note": "one K+W-step job through the C ABI from pinned host buffers: H2D of X/y/alpha/f, operand-plane split, "
                   "solver set-up, steps, D2H of alpha/f/rho all inside the timed region"}

    # ---- (3) the whole training run to eps --------------------------------------------------------
    train = None
    full = args.full_train if args.full_train >= 0 else 1
    if full:
        sec, st, rho, a_host, f_host, done = job(10 ** 9, budget_s=args.train_budget_s)
        train = {"seconds": sec, "converged": bool(done), "outer_iters": st["outer_iters"],
                 "local_iters": st["local_iters"], "final_diff": st["final_diff"], "objective": st["objective"],
                 "rho": rho, "n_sv": int((a_host != 0).sum()), "kernel_rows_per_s": st["kernel_rows"] / sec,
                 "phase_seconds": {k: st["seconds_" + k] for k in ("select", "rows", "local", "update")}}

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
            dec = capi.predict_dec(km_sv, coef_d, counts, rho_d, 2, dense=T)
            return capi.vote(dec, 2)

        warm = run_predict(Th[:2048].cuda())
        Td = Th.cuda()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        labels = run_predict(Td)
        e1.record()
        torch.cuda.synchronize()
        ms_res = e0.elapsed_time(e1)
        del Td
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        lab_h = run_predict(Th.cuda(non_blocking=True)).cpu()
        sec_host = time.perf_counter() - t0
        n_sv = len(order)
        predict = {"rows": m, "n_sv": n_sv, "rows_per_s": m / (ms_res * 1e-3), "e2e_rows_per_s": m / sec_host,
                   "algorithmic_tflops": 2.0 * m * n_sv * d / (ms_res * 1e-3) / 1e12,
                   "positive_fraction": float((lab_h == 0).float().mean()),
                   "accuracy": float(((lab_h == 0).numpy() == (y_test > 0)).mean()),
                   "note": "decision values + vote of the seed-8 test rows against the trained model; resident: test "
                           "rows in HBM, CUDA events; e2e: from pinned host rows, labels back on the host"}
        km_sv.close()
        del Xsv, warm, labels

    cpu = None
    if not args.no_cpu_baseline:
        try:
            s = cpu_sample(args.cpu_sample_rows, args.cpu_sample_steps)
            cpu = {k: s[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as exc:   # the baseline is reporting only; never fail the bench on it
            cpu = {"value": None, "unit": "rows/s", "cores": os.cpu_count(), "kind": "port", "sample": "failed: %r" % exc}

    line = {
        "metric": "kernel_rows_per_s", "value": value, "unit": "rows/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 kernel values (two-plane FP16 tensor-core contraction with FP32 accumulation), f64 solver state", "data": "synthetic",
        "config": {"workload": "config5: binary C-SVC, RBF gamma=0.5 C=1 eps=1e-3, %dx%d dense fp32, ws=1024, "
                               "512 new kernel rows per outer iteration" % (n, d),
                   "l2": "inputs larger than L2 (X planes %.1f GB, row buffer %.1f GB)" % (2 * n * d * 2 / 1e9,
                                                                                          WS * n * 4 / 1e9)},
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clk,
        "phase_ms_per_step": phases, "train_to_eps": train, "predict": predict,
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

"""Benchmark of the vector-wise N:M sparse GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one multiply C = A.B of the square workload (M = K = 4096, 4096
columns of B per GPU, 8:32 sparsity, V = 32, FP32) with the operands resident in
HBM.  With N > 1 (one process per GPU under torch.distributed.run) the columns
of B are sharded by vector groups, 4096 per rank, A replicated: weak scaling,
no data-path collective.  Rank 0 prints one JSON line.

* ``value``         useful TFLOP/s = 2.M.N_total.W / t, max over ranks of the device time
* ``roofline``      of the FP32 kernel: useful FLOPs against the FFMA rate measured live
                    on the same GPU (register-only kernel), with the HBM time beside it
* ``e2e``           the same metric through the host-buffer entry point
                    (nmspmm_gemm_host): H2D of A, B and the raw indices, index packing,
                    multiply, D2H of C inside the timed region
* ``cpu_baseline``  the reference's host multiply timed on this box's cores on a
                    bounded row sample (N = 1, rank 0)
* ``per_ratio``     the same step for 16:32, 12:32, 8:32, 4:32 (useful and
                    dense-equivalent TFLOP/s, roofline fraction)
* ``tf32``          the tensor-core path on the same workload, every ratio
* ``sustained``     the headline step launched back to back for a second, with the SM
                    clock seen meanwhile (the K-step value is a burst)
* ``parity``        sampled rows of every rank's result against the CPU checker, inside
                    this run
* ``workloads``     (N = 1) the other named configurations, both paths and the index
                    packing alone, each against the slower of its HBM and FLOP time
* ``large_sharded`` 8192 x 28672 x 8192, V = 64, split over the ranks (strong scaling),
                    alone and with both all-gathers of C, each checked

``--impl reference`` times the reference's own CPU implementation of the path
(oracle/_ref, compiled unchanged from the reference's sources; the C restatement
when that object is absent) on the same workload, each step a bounded row sample.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_SQ = N_SQ = K_SQ = 4096
HEADLINE_KEEP = 8
SETS = 3                      # operand sets rotated between steps (3 x 144 MB > 126 MB of L2)
METRIC = "useful TFLOP/s, vector-wise N:M SpMM, 4096^3 8:32 V=32 FP32"

SUSTAINED_SECONDS = 1.0       # back-to-back launches timed beside the K-step burst


def algorithmic_bytes(M, N, K, n_keep, layout_ns=128):
    """Compulsory traffic of one multiply: A, compressed B, indices, C once each,
    plus column_info on the high-sparsity path."""
    W = K // 32 * n_keep
    b = 4 * (M * K + W * N + W * N // 32 + M * N)
    if n_keep in (8, 4):
        b += 4 * (N // layout_ns) * (W // (2 * n_keep)) * 64
    return b


@contextlib.contextmanager
def quiet_stdout():
    """The reference's host multiply printf()s its thread count; keep stdout to the JSON line."""
    sys.stdout.flush()
    saved = os.dup(1)
    devnull = os.open(os.devnull, os.O_WRONLY)
    os.dup2(devnull, 1)
    try:
        yield
    finally:
        os.dup2(saved, 1)
        os.close(saved)
        os.close(devnull)


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.sm_max = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def sample(self):
        if self._nv is None:
            return
        try:
            self.samples.append(int(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM)))
            mask = int(self._nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def __enter__(self):
        def loop():
            while not self._stop.is_set():
                self.sample()
                self._stop.wait(0.005)
        self._stop.clear()
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.sm_max,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            pass
    return local_rank


def square_config(world: int) -> dict:
    """The workload both arms are timed on (same keys, same values)."""
    return {"workload": "square 4096^3, 8:32 (75 %), V=32, FP32 exact path", "M": M_SQ, "K": K_SQ,
            "N_per_gpu": N_SQ, "N_total": N_SQ * world, "n_keep": HEADLINE_KEEP, "layout_ns": 128,
            "parallelism": f"B column-vector groups sharded over {world} GPU(s), A replicated, no collective",
            "l2": f"operands rotate over {SETS} sets of A and C (3 x 128 MB > 126 MB L2); no flush"}


_checker = None


def checker():
    """The CPU checker (the C restatement of the reference's host multiply), all host threads."""
    global _checker
    if _checker is None:
        import oracle
        _checker = oracle.restatement()
        try:
            _checker.set_num_threads(len(os.sched_getaffinity(0)))
        except Exception:
            pass
    return _checker


def sampled_rows_error(A_km, BT, DT, n_keep, C_rows, rows, col0=0, f64=False):
    """Relative Frobenius error of rows ``rows`` of a result (``C_rows``: those rows, columns
    col0 .. col0 + BT.shape[1]) against the CPU checker on the same operands."""
    K = A_km.shape[0]
    w = np.arange(BT.shape[0], dtype=np.int32)[:, None]
    B_col = np.ascontiguousarray(BT.T)
    D_col = np.ascontiguousarray((DT + (w // n_keep) * 32).T.astype(np.int32))
    sub = np.ascontiguousarray(A_km[:, rows])
    with quiet_stdout():
        want = (checker().nm_gemm_f64 if f64 else checker().nm_gemm_f32)(sub, B_col, D_col)
    got = np.asarray(C_rows, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


# ------------------------------------------------------------------------------------
# CPU side: the reference's host multiply on a bounded sample.
# ------------------------------------------------------------------------------------

def cpu_reference_impl():
    """The reference's host multiply with every core this process may use (torchrun pins
    OMP_NUM_THREADS to 1, which is not what a CPU baseline wants)."""
    import oracle
    impl, kind = (oracle.reference(), "reference") if oracle.have_reference() else (oracle.restatement(), "port")
    try:
        impl.set_num_threads(len(os.sched_getaffinity(0)))
    except Exception:
        pass
    return impl, kind


def cpu_sample(pkg, impl, p, rows: int):
    """Times the host multiply on the first ``rows`` rows of A (rows are independent
    in the reference's loop nest).  Returns seconds."""
    sub = np.ascontiguousarray(p.A_km[:, :rows])
    B_col, D_col = p.B_col, p.D_col
    with quiet_stdout():
        t0 = time.perf_counter()
        impl.nm_gemm_f32(sub, B_col, D_col)
        return time.perf_counter() - t0


def rows_for_budget(pkg, impl, p, cores: int, seconds: float) -> int:
    """Rows of A whose host multiply takes about ``seconds`` (calibrated on a warm probe)."""
    probe_rows = min(p.M, 4 * cores)
    cpu_sample(pkg, impl, p, probe_rows)
    t = cpu_sample(pkg, impl, p, probe_rows)
    rows = int(min(p.M, max(cores, probe_rows * seconds / max(t, 1e-6))))
    return max(cores, rows // cores * cores)


def cpu_baseline(pkg, p, budget_s: float = 12.0):
    impl, kind = cpu_reference_impl()
    cores = impl.num_threads()
    rows = rows_for_budget(pkg, impl, p, cores, budget_s)
    t = cpu_sample(pkg, impl, p, rows)
    flops = 2.0 * rows * p.N * p.W
    return {"value": flops / t / 1e12, "unit": "useful TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"first {rows} of {p.M} rows of A against the full B ({p.N} columns, W={p.W}); "
                      f"{t:.2f} s of nmGEMM_on_cpu", "seconds": t}


def run_reference_arm(args, rank: int, world: int):
    if rank != 0:
        return
    from __graft_entry__ import load_package
    pkg = load_package(native=False)
    impl, kind = cpu_reference_impl()
    cores = impl.num_threads()
    p = pkg.formats.make_random(M_SQ, N_SQ, K_SQ, HEADLINE_KEEP, seed=0)
    total_budget = 60.0                              # seconds of CPU work over warm-up + steps
    rows = rows_for_budget(pkg, impl, p, cores, total_budget / max(1, args.steps + args.warmup))
    for _ in range(args.warmup):
        cpu_sample(pkg, impl, p, rows)
    times = [cpu_sample(pkg, impl, p, rows) for _ in range(args.steps)]
    sec = float(np.mean(times))
    value = 2.0 * rows * p.N * p.W / sec / 1e12
    sample = f"each step: first {rows} of {p.M} rows of A against the full B, all {cores} host threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
        "config": square_config(world),
        "timed": "the reference's CPU multiply nmGEMM_on_cpu on a bounded row sample of that workload",
        "cpu_baseline": {"value": value, "unit": "useful TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------
# GPU side.
# ------------------------------------------------------------------------------------

def time_steps(torch, fn, steps: int, barrier=None):
    """Device time of ``steps`` calls of fn(i) on the current stream, in ms."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if barrier:
        barrier()
    torch.cuda.synchronize()
    start.record()
    for i in range(steps):
        fn(i)
    end.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return start.elapsed_time(end)


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    from __graft_entry__ import load_package
    pkg = load_package(native=True)
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # This rank's column shard: 4096 columns of B (its own seed), A shared by all ranks.
    M, K, n_local = M_SQ, K_SQ, N_SQ
    keep = args.n_keep if args.kernel_only else HEADLINE_KEEP
    p = pkg.formats.make_random(M, n_local, K, keep, seed=0)
    if rank != 0:
        q = pkg.formats.make_random(4, n_local, K, keep, seed=1000 + rank)
        p.BT, p.DT = q.BT, q.DT
    op = pkg.NMSpMM.from_problem(p, layout_ns=128)
    A_sets = [torch.from_numpy(p.A_km).cuda()]
    for s in range(1, SETS):
        A_sets.append(torch.roll(A_sets[0], s * 131, dims=1).contiguous())
    C_sets = [torch.empty((M, n_local), dtype=torch.float32, device="cuda") for _ in range(SETS)]
    path = pkg.PATH_TF32 if (args.kernel_only and args.path == "tf32") else pkg.PATH_FP32
    desc = op.desc(M, path=path, tile=args.tile, split_k=args.split_k)
    plan = pkg.plan(desc)

    def step(i):
        op.matmul(A_sets[i % SETS], out=C_sets[i % SETS], path=path, tile=args.tile, split_k=args.split_k)

    for i in range(max(3, args.warmup)):
        step(i)
    torch.cuda.synchronize()

    sampler = ClockSampler(physical_gpu_index(local_rank))
    with sampler:
        ms = time_steps(torch, step, args.steps, barrier)
        sampler.sample()
    ms = max_over_ranks(ms)
    if pkg.device_status() != 0:
        raise RuntimeError("a device-side bounded wait gave up during the timed region")
    ms_per_step = ms / args.steps
    useful = 2.0 * M * n_local * p.W
    value = world * useful / (ms_per_step * 1e-3) / 1e12

    def min_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return float(t.item())

    def sustained(fn, flops_per_call):
        """Back-to-back launches for about a second (events on the launching stream), with the
        SM clock sampled meanwhile: what the K-step burst above turns into under load."""
        smp = ClockSampler(physical_gpu_index(local_rank))
        chunk, total_ms, calls = 100, 0.0, 0
        with smp:
            while total_ms < SUSTAINED_SECONDS * 1e3:
                total_ms += time_steps(torch, fn, chunk)
                calls += chunk
        t = max_over_ranks(total_ms / calls)
        return {"seconds": total_ms / 1e3, "launches": calls, "ms_per_step": t,
                "value": world * flops_per_call / (t * 1e-3) / 1e12, "clocks": smp.summary()}

    def parity_of(result, prob, rows, f64=False):
        """Sampled rows of this rank's result against the CPU checker; worst rank wins."""
        idx = torch.as_tensor(rows, device="cuda")
        err = sampled_rows_error(prob.A_km, prob.BT, prob.DT, prob.n_keep, result[idx].cpu().numpy(), rows, f64=f64)
        return err

    # ---- parity inside this run: every rank checks rows of its own slab ---------------
    check_rows = [0, 1, 127, 128, 1000, 2047, 2048, 4095]
    err_here = parity_of(op.matmul(A_sets[0], path=path, tile=args.tile, split_k=args.split_k), p, check_rows,
                         f64=(path == pkg.PATH_TF32))
    tol_here = 1e-5 if path == pkg.PATH_FP32 else 2e-3
    parity = {"rows_per_rank": len(check_rows), "max_rel_err": -min_over_ranks(-err_here), "tolerance": tol_here,
              "checker": "C restatement of the reference's nmGEMM_on_cpu, on each rank's own operands"}
    parity["ok"] = bool(parity["max_rel_err"] <= tol_here)
    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"kernel_only": True, "ffma_peak": [pkg.measure_ffma_peak(False), pkg.measure_ffma_peak(True)],
                              "n_keep": keep, "path": args.path, "ms_per_step": ms_per_step, "useful_tflops": value,
                              "tile": [plan.tile_m, plan.tile_n], "split_k": plan.split_k, "grid": plan.grid, "stages": plan.stages,
                              "parity": parity, "clocks": sampler.summary()}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant (only) kernel, per GPU --------------------------
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_gbs = float(peaks.get("hbm_gbs", 6650.0))
    hbm_src = "MEASURED_PEAKS.json" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
    ffma_scalar, ffma_packed = pkg.measure_ffma_peak(False), pkg.measure_ffma_peak(True)
    ffma_peak = max(ffma_scalar, ffma_packed)
    abytes = algorithmic_bytes(M, n_local, K, HEADLINE_KEEP)
    t_flop = useful / (ffma_peak * 1e12)
    t_mem = abytes / (hbm_gbs * 1e9)
    achieved = useful / (ms_per_step * 1e-3) / 1e12
    roofline = {
        "bound": "fp32_simt" if t_flop >= t_mem else "hbm",
        "achieved": achieved, "peak": ffma_peak, "unit": "TFLOP/s", "frac": max(t_flop, t_mem) / (ms_per_step * 1e-3),
        "traffic": None,
        "traffic_source": "not measured in this run (DRAM counters need ncu); one capture of this kernel and workload is "
                          "summarised in profiles/nm_gemm_ffma_128x128_high_4096cubed_8of32.md",
        "peak_source": "FP32 FMA rate measured live on this GPU by the library's register-only kernels, larger of "
                       f"scalar FFMA ({ffma_scalar:.1f}) and packed FFMA2 ({ffma_packed:.1f} TFLOP/s); "
                       "nominal 148 SMs x 128 lanes x 2 x SM clock",
        "algorithmic_bytes": abytes, "algorithmic_flops": useful,
        "hbm_time_us": t_mem * 1e6, "hbm_peak_gbs": hbm_gbs, "hbm_peak_source": hbm_src,
        "kernel": f"nm_gemm_ffma_kernel tile {plan.tile_m}x{plan.tile_n}, "
                  f"{'automatic schedule' if plan.stream_k else 'split_k ' + str(plan.split_k)}: "
                  f"{plan.tiles_x * plan.tiles_y} tiles ({plan.n_dp} whole) in {plan.n_virtual} unit ranges = CTAs, "
                  f"{plan.stages} stages, {plan.smem_bytes} B smem",
        "kernel_ms": ms_per_step,
    }

    sustained_fp32 = sustained(step, useful)

    # ---- the other ratios (N=1 only, short) ---------------------------------------
    per_ratio = []
    if world == 1:
        for n_keep in (16, 12, 8, 4):
            pr = p if n_keep == HEADLINE_KEEP else pkg.formats.make_random(M, n_local, K, n_keep, seed=0)
            opr = op if n_keep == HEADLINE_KEEP else pkg.NMSpMM.from_problem(pr, layout_ns=128)
            fn = lambda i, o=opr: o.matmul(A_sets[i % SETS], out=C_sets[i % SETS])
            for i in range(3):
                fn(i)
            t = time_steps(torch, fn, 20) / 20
            uf = 2.0 * M * n_local * pr.W
            tf, tm = uf / (ffma_peak * 1e12), algorithmic_bytes(M, n_local, K, n_keep) / (hbm_gbs * 1e9)
            per_ratio.append({"n_keep": n_keep, "path": "fp32", "ms": t, "useful_tflops": uf / (t * 1e-3) / 1e12,
                              "dense_equivalent_tflops": 2.0 * M * n_local * K / (t * 1e-3) / 1e12,
                              "roofline_frac": max(tf, tm) / (t * 1e-3)})

    # ---- the tensor-core path on the same workload (N=1 only) ------------------------
    tf32 = None
    if world == 1:
        tf32_peak = float(peaks.get("bf16_tflops", 1590.0)) / 2.0      # dense TF32 = half the dense bf16 rate
        rows = []
        tf32_sustained = None
        for n_keep in (16, 12, 8, 4):
            pr = p if n_keep == HEADLINE_KEEP else pkg.formats.make_random(M, n_local, K, n_keep, seed=0)
            opr = op if n_keep == HEADLINE_KEEP else pkg.NMSpMM.from_problem(pr, layout_ns=128)
            fn = lambda i, o=opr: o.matmul(A_sets[i % SETS], out=C_sets[i % SETS], path=pkg.PATH_TF32)
            for i in range(3):
                fn(i)
            t = time_steps(torch, fn, 20) / 20
            uf = 2.0 * M * n_local * pr.W
            tf, tm = uf / (tf32_peak * 1e12), algorithmic_bytes(M, n_local, K, n_keep) / (hbm_gbs * 1e9)
            got = opr.matmul(A_sets[0], path=pkg.PATH_TF32)
            exact = opr.matmul(A_sets[0])
            err = float((got - exact).norm() / exact.norm())
            err64 = parity_of(got, pr, check_rows, f64=True)
            info = pkg.plan(opr.desc(M, path=pkg.PATH_TF32))
            rows.append({"n_keep": n_keep, "path": "tf32", "ms": t, "useful_tflops": uf / (t * 1e-3) / 1e12,
                         "dense_equivalent_tflops": 2.0 * M * n_local * K / (t * 1e-3) / 1e12,
                         "roofline_frac": max(tf, tm) / (t * 1e-3), "rel_err_vs_fp32_path": err,
                         "rel_err_vs_fp64_checker_rows": err64, "tile": [info.tile_m, info.tile_n]})
            if n_keep == HEADLINE_KEEP:
                tf32_sustained = sustained(fn, uf)
        tf32 = {"kernel": "nm_gemm_tf32_kernel: per k window one tcgen05.mma kind::tf32 chain gathers the selected columns "
                          "of A into TMEM (A window x one-hot matrix, M128 N<=128), then M128 N32 K8 products per vector",
                "sustained_8of32": tf32_sustained,
                "bound": "tensor", "peak": tf32_peak, "unit": "TFLOP/s",
                "peak_source": "half of the measured dense bf16 rate in MEASURED_PEAKS.json (burst)"
                               if "bf16_tflops" in peaks else "half of the fallback 1590 TFLOP/s bf16",
                "tolerance": "2e-3 relative Frobenius error against the FP64 host product (tests/test_gpu_tf32.py)",
                "per_ratio": rows}

    # ---- end to end through the host-buffer entry point ------------------------------
    # Every rank pins its buffers on the NUMA node of its own GPU (first touch by a process
    # bound there): with eight ranks copying at once, buffers on the far socket would put the
    # inter-socket link between every GPU and its data.
    saved_affinity = os.sched_getaffinity(0)
    numa_probe = pkg.gpu_numa_probe(local_rank)
    numa_bound = pkg.bind_host_to_gpu(local_rank)
    hA = torch.empty(p.A_km.shape, dtype=torch.float32).pin_memory().copy_(torch.from_numpy(p.A_km))
    hB = torch.empty(p.BT.shape, dtype=torch.float32).pin_memory().copy_(torch.from_numpy(p.BT))
    hD = torch.empty(p.DT.shape, dtype=torch.int32).pin_memory().copy_(torch.from_numpy(p.DT))
    hC = torch.empty((M, n_local), dtype=torch.float32).pin_memory()
    hC.zero_()
    e2e_steps = max(3, min(args.steps, 10))

    def link_gbs(dst, src):
        """One direction of this rank's host link alone: a plain copy of one buffer, all ranks at once."""
        dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        ms = time_steps(torch, lambda i: dst.copy_(src, non_blocking=True), 3, barrier) / 3
        return src.numel() * 4 / (ms * 1e-3) / 1e9

    link = {"h2d_gbs_min_over_ranks": min_over_ranks(link_gbs(A_sets[0], hA)),
            "d2h_gbs_min_over_ranks": min_over_ranks(link_gbs(hC, C_sets[0])),
            "numa_bound": bool(numa_bound),
            "numa_probe_rank0": {"bdf": numa_probe["bdf"], "node": numa_probe["node"], "why_not": numa_probe["why_not"]},
            "note": "a 64 MiB pinned buffer copied alone, every rank at the same time; the e2e call moves "
                    "%.0f MB in and %.0f MB out per step" % ((hA.numel() + hB.numel() + hD.numel()) * 4 / 1e6, hC.numel() * 4 / 1e6)}

    def e2e_step(i):
        pkg.gemm_host(desc, hA, hB, hD, hC, on_current_stream=True)

    for i in range(3):
        e2e_step(i)
    e2e_ms = max_over_ranks(time_steps(torch, e2e_step, e2e_steps, barrier)) / e2e_steps
    h2d = hA.numel() * 4 + hB.numel() * 4 + hD.numel() * 4
    d2h = hC.numel() * 4
    os.sched_setaffinity(0, saved_affinity)
    e2e = {"value": world * useful / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps, "host_link": link,
           "copy_time_floor_ms": max(h2d / (link["h2d_gbs_min_over_ranks"] * 1e6), d2h / (link["d2h_gbs_min_over_ranks"] * 1e6)),
           "call": "nmspmm_gemm_host (pinned host A, B, raw indices -> packed on the GPU -> multiply -> host C)"}
    # parity of what the e2e call returned, against the resident-operand result
    e2e_err = float((hC.cuda() - C_sets[0].copy_(op.matmul(A_sets[0]))).norm() / C_sets[0].norm())

    cpu = cpu_baseline(pkg, p) if (world == 1 and rank == 0) else None

    # ---- the large sharded configuration: fixed total work over the ranks -------------
    # 8192 x 28672 x 8192, 8:32, V = 64: B's column-vector groups split into `world` slabs of
    # whole index blocks; every rank multiplies its slab (no collective), then the same with
    # the all-gather of C: NCCL after the multiply, and fused into the multiply's epilogue.
    del A_sets, C_sets, hA, hB, hD, hC
    torch.cuda.empty_cache()
    LM, LN, LK, LKEEP = WORKLOADS["large"][:4]
    pl = pkg.formats.make_random(LM, LN, LK, LKEEP, seed=0, vec_len=64)
    sh = pkg.sharding.ShardedNMSpMM(pkg, pl.BT, pl.DT, LK, LKEEP, rank, world, vec_len=64)
    LA = torch.from_numpy(pl.A_km).cuda()
    l_useful = pl.useful_flops()
    l_steps = 5
    c0, c1 = sh.columns
    large = {"workload": "8192 x 28672 x 8192, 8:32, V=64, column-vector groups over %d GPU(s)" % world,
             "scaling": "strong", "columns_of_rank0": list(sh.columns), "steps": l_steps}
    slab_rows = [int(r) for r in np.linspace(0, LM - 1, 64).astype(np.int64)]      # 64 rows of every rank's slab
    full_rows = [0, 4095, 8191, 127, 128, 6000, 2049, 7777]                       # rows of the gathered C, rank 0

    def slab_error(C, f64=False):
        """This rank's columns of rows ``slab_rows`` against the CPU checker on this rank's slab of B."""
        idx = torch.as_tensor(slab_rows, device="cuda")
        cols = C[idx][:, c0:c1] if C.shape[1] == LN else C[idx]
        return sampled_rows_error(pl.A_km, pl.BT[:, c0:c1], pl.DT[:, c0 // 32:c1 // 32], LKEEP, cols.cpu().numpy(),
                                  slab_rows, f64=f64)

    def all_ranks_ok(flag: bool) -> bool:
        return min_over_ranks(1.0 if flag else 0.0) == 1.0

    modes = [("multiply", False, pkg.PATH_FP32), ("multiply_tf32", False, pkg.PATH_TF32)]
    if world > 1:
        modes += [("multiply_then_nccl_all_gather", True, pkg.PATH_FP32), ("multiply_with_fused_all_gather", "fused", pkg.PATH_FP32),
                  ("multiply_tf32_with_fused_all_gather", "fused", pkg.PATH_TF32)]
    gathered = {}
    for name, gather, lpath in modes:
        fn = lambda i, g=gather, pa=lpath: sh.matmul(LA, gather=g, path=pa)
        # the gathers are optional extras of the path: a set-up failure on one rank (peer
        # mapping, NCCL) must not take the headline line down, and every rank must agree
        # on whether the mode runs at all
        ok = 1.0
        try:
            for i in range(2):
                fn(i)
            torch.cuda.synchronize()
        except Exception as exc:      # noqa: BLE001
            ok, why = 0.0, f"{type(exc).__name__}: {exc}"[:200]
        if world > 1:
            if min_over_ranks(ok) == 0.0:
                large[name] = {"unavailable": why if ok == 0.0 else "failed on another rank"}
                continue
        elif ok == 0.0:
            raise RuntimeError(why)
        t = max_over_ranks(time_steps(torch, fn, l_steps, barrier)) / l_steps
        # ---- the result of this mode, checked on every rank --------------------------------
        C = fn(0)
        torch.cuda.synchronize()
        barrier()
        is_tf32 = lpath == pkg.PATH_TF32
        tol = 2e-3 if is_tf32 else 1e-5
        err = slab_error(C, f64=is_tf32)
        entry = {"ms": t, "useful_tflops": l_useful / (t * 1e-3) / 1e12,
                 "slab_rel_err_max_over_ranks": -min_over_ranks(-err), "tolerance": tol, "rows_checked_per_rank": len(slab_rows)}
        good = err <= tol
        if gather:
            # every rank holds the full C: rank 0 checks rows across all slabs against the checker,
            # and the two gathers of the same path must agree bit for bit on every rank
            if rank == 0:
                idx = torch.as_tensor(full_rows, device="cuda")
                e_full = sampled_rows_error(pl.A_km, pl.BT, pl.DT, LKEEP, C[idx].cpu().numpy(), full_rows, f64=is_tf32)
                entry["gathered_rel_err_rank0"] = e_full
                good = good and e_full <= tol
            key = "tf32" if is_tf32 else "fp32"
            if key in gathered:
                same = bool(torch.equal(C, gathered[key]))
                entry["equals_nccl_gather_on_every_rank"] = all_ranks_ok(same)
                good = good and same
            else:
                gathered[key] = C.clone()
        entry["parity"] = all_ranks_ok(bool(good))
        large[name] = entry
    gathered.clear()
    if pkg.device_status() != 0:
        raise RuntimeError("a device-side bounded wait gave up in the large sharded configuration")
    del LA, sh
    torch.cuda.empty_cache()

    # ---- the other named configurations (N = 1) ------------------------------------------
    workloads = None
    if world == 1:
        workloads = {name: measure_workload(pkg, torch, name, 0, 0, quick=True) for name in ("llm16", "llm64", "llm256", "deepk")}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded splitmix64: A, kept values U[-1,1), "
                                                       "random sorted indices)",
            "config": square_config(world),
            "dense_equivalent_tflops": world * 2.0 * M * n_local * K / (ms_per_step * 1e-3) / 1e12,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "e2e_rel_err_vs_resident": e2e_err,
            "gpu_launches": args.steps, "clocks": sampler.summary(), "parity": parity, "sustained": sustained_fp32,
            "per_ratio": per_ratio, "tf32": tf32, "large_sharded": large, "workloads": workloads,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


WORKLOADS = {
    # name: (M, N, K, n_keep, vec_len) -- the named configurations beside the square one
    "llm16": (16, 11008, 4096, 8, 32), "llm64": (64, 11008, 4096, 8, 32), "llm256": (256, 11008, 4096, 8, 32),
    "deepk": (128, 1024, 131072, 4, 32), "large": (8192, 28672, 8192, 8, 64),
}


def measure_workload(pkg, torch, name: str, tile: int = 0, split_k: int = 0, steps: int = 50, quick: bool = False,
                     paths=("fp32", "tf32")) -> dict:
    """One of the other named configurations on one GPU: per-launch device time with the
    operands cycled so that no launch finds them in L2 (these shapes are small enough to live
    there otherwise), the index packing timed alone, the roofline fraction of each path, and
    the result of each path checked against the CPU checker."""
    M, N, K, n_keep, vec = WORKLOADS[name]
    p = pkg.formats.make_random(M, N, K, n_keep, seed=0, vec_len=vec, a_dist="normal" if name.startswith("llm") else "uniform")
    raw = torch.from_numpy(p.DT).cuda()
    useful, abytes = p.useful_flops(), algorithmic_bytes(M, N, K, n_keep)
    # Replicas of the sparse operand and of C, cycled launch after launch, so that a launch
    # never finds its operands in the 126 MB L2; the launches are captured in a CUDA graph so
    # that the device time is not padded by host launch latency (some of these kernels take
    # tens of microseconds).
    n_rep = max(2, min(8, -(-(300 << 20) // abytes)))
    reps = n_rep * max(2, (16 if quick else steps) // n_rep)

    def graph_time(fns):
        for f in fns:
            f()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for i in range(reps):
                fns[i % len(fns)]()
        gr.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        gr.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    raws = [raw.clone() for _ in range(n_rep)]
    if pkg.format_of(n_keep) == pkg.FORMAT_HIGH:
        outs = [pkg.preprocess_high_device(r, 32, n_keep, 128, fuse_trans_index=True) for r in raws]
        packs = [lambda r=r, o=o: pkg.preprocess_high_device(r, 32, n_keep, 128, fuse_trans_index=True, out=o[0], column_info=o[1])
                 for r, o in zip(raws, outs)]
    else:
        outs = [pkg.preprocess_low_device(r, 128) for r in raws]
        packs = [lambda r=r, o=o: pkg.preprocess_low_device(r, 128, out=o) for r, o in zip(raws, outs)]
    pack_ms = graph_time(packs)
    ops = [pkg.NMSpMM.from_problem(p, layout_ns=128) for _ in range(n_rep)]
    A = torch.from_numpy(p.A_km).cuda()
    Cs = [torch.empty((M, N), dtype=torch.float32, device="cuda") for _ in range(n_rep)]
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm = float(peaks.get("hbm_gbs", 6650.0)) * 1e9
    fp32_peak = max(pkg.measure_ffma_peak(False), pkg.measure_ffma_peak(True)) * 1e12
    tf32_peak = float(peaks.get("bf16_tflops", 1590.0)) / 2.0 * 1e12
    pack_bytes = 2 * raw.numel() * 4 + (outs[0][1].numel() * 4 if isinstance(outs[0], tuple) else 0)
    out = {"workload": name, "M": M, "N": N, "K": K, "n_keep": n_keep, "vec_len": vec,
           "index_packing_ms": pack_ms, "index_packing_gbs": pack_bytes / (pack_ms * 1e-3) / 1e9,
           "algorithmic_bytes": abytes, "useful_flops": useful, "hbm_time_us": abytes / hbm * 1e6,
           "l2": f"{n_rep} replicas of B, indices and C cycled (working set {n_rep * abytes >> 20} MB); "
                 f"{reps} launches replayed from a CUDA graph"}
    rows = sorted(set(int(r) for r in np.linspace(0, M - 1, min(M, 16)).astype(np.int64)))
    for pname, path, peak in (("fp32", pkg.PATH_FP32, fp32_peak), ("tf32", pkg.PATH_TF32, tf32_peak)):
        if pname not in paths:
            continue
        fns = [lambda o=o, c=c: o.matmul(A, out=c, path=path, tile=tile, split_k=split_k) for o, c in zip(ops, Cs)]
        ms = graph_time(fns)
        plan = pkg.plan(ops[0].desc(M, path=path, tile=tile, split_k=split_k))
        err = sampled_rows_error(p.A_km, p.BT, p.DT, n_keep, Cs[0][torch.as_tensor(rows, device="cuda")].cpu().numpy(), rows,
                                 f64=(pname == "tf32"))
        out[pname] = {"ms": ms, "useful_tflops": useful / (ms * 1e-3) / 1e12, "bytes_per_s_gbs": abytes / (ms * 1e-3) / 1e9,
                      "roofline_frac": max(useful / peak, abytes / hbm) / (ms * 1e-3),
                      "bound": "hbm" if abytes / hbm > useful / peak else "flops",
                      "kernel": ("nm_gemm_ffma_kernel" if pname == "fp32" else
                                 ("nm_gemm_tf32_few_rows_kernel" if plan.tile_m < 128 else "nm_gemm_tf32_kernel")),
                      "tile": [plan.tile_m, plan.tile_n], "ctas": plan.grid, "whole_tiles": plan.n_dp,
                      "rel_err_rows": err, "parity": bool(err <= (1e-5 if pname == "fp32" else 2e-3))}
    assert pkg.device_status() == 0
    return out


def run_workload(args):
    import torch

    from __graft_entry__ import load_package
    pkg = load_package(native=True)
    torch.cuda.set_device(0)
    print(json.dumps(measure_workload(pkg, torch, args.workload, args.tile, args.split_k, args.steps)), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the resident-operand steps (profiling runs): no e2e, CPU baseline or ratio sweep")
    ap.add_argument("--n-keep", type=int, default=HEADLINE_KEEP, help="kept rows per 32-window for --kernel-only runs")
    ap.add_argument("--workload", default="", choices=[""] + sorted(WORKLOADS),
                    help="measure one of the other named configurations on one GPU instead of the square one")
    ap.add_argument("--path", default="fp32", choices=["fp32", "tf32"], help="arithmetic of --kernel-only runs")
    ap.add_argument("--tile", type=int, default=0, help="force a CTA tile id (tuning runs)")
    ap.add_argument("--split-k", type=int, default=0, help="force the number of K slices (tuning runs)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload:
        run_workload(args)
    elif args.impl == "reference":
        run_reference_arm(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()

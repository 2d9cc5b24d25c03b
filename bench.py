#!/usr/bin/env python
"""Benchmark of the hot path: BF16 GEMM TFLOP/s through the engine's C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--extras]

N = 1: one step is one 8192^3 BF16 product (FP32 accumulate, BF16 result) on operands
resident in HBM, launched through `matmul_dram_bf16`; `value` is 2*8192^3*K / device time.
The same line carries the rest of the metric: `prefill` (the SmolLM2-135M-shape prefill of
8 x 512 tokens as a replayed trace: tokens/s, launches, a per-op-class table; under `decode_step` the
generation step that follows it, ms a token at 1 and 4 sequences) and `suite` (the
memory-bound ops on [8192, 8192] F32 and the row softmax on [4096, 32768]: GB/s of algorithmic
bytes), each with its own `roofline`.
N > 1 (under torchrun, one rank a GPU): the 16384^3 product split along N with K whole
(crates/tt-kernels/src/shard.rs:348-458), every rank computing its column slice and an
NCCL all-gather leaving the full C on every rank; time is the max over ranks.
`e2e` is the same product called with HOST operands: upload of A and B from pinned host
memory, the product, and the download of C, all inside the timed region.
`--impl reference` times the CPU restatement of the reference's comparison backend (the
reference itself is Rust for Tenstorrent cards and cannot run here) on the host cores.
One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import threading
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "bf16_gemm_tflops"
UNIT = "TFLOP/s"
N1_SIZE = 8192
NN_SIZE = 16384
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return d, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """SM clock and throttle reasons sampled while the timed region runs: an NVML polling
    thread (a sample every ~2 ms, so a region of a few milliseconds is still covered), or a
    looping nvidia-smi process where NVML cannot be opened."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    BITS = (("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40))

    def __init__(self, gpu_index: int):
        self.proc = None
        self.thread = None
        self.idx = gpu_index
        self.sm, self.reasons, self.mx = [], set(), None
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = None
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(gpu_index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.mx = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))

            def poll():
                while True:
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                        mask = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                        for name, bit in self.BITS:
                            if mask & bit:
                                self.reasons.add(name)
                    except Exception:
                        pass
                    if self._stop.wait(0.002):
                        return
            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(gpu_index), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.thread:
            self._stop.set()
            self.thread.join(timeout=2)
            return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.mx,
                    "reasons": sorted(self.reasons), "samples": len(self.sm), "source": "nvml"}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


def cheap_bf16(shape, seed):
    """Fast synthetic BF16 operand in [-1,1) for the big benchmark shapes."""
    rng = np.random.default_rng(seed)
    f = rng.random(shape, dtype=np.float32) * 2.0 - 1.0
    return (f.view(np.uint32) >> 16).astype(np.uint16)


# ---------------------------------------------------------------------- CPU baseline
CPU_BUDGET_S = 60.0     # a configuration the restatement finishes within this is run whole; beyond it, a smaller sample


def _cpu_product(n):
    """One n^3 F32 product of BF16-rounded operands by the C/OpenMP restatement; seconds."""
    from oracle import oracle as orc
    a = orc.from_bf16(cheap_bf16((n, n), 1))
    b = orc.from_bf16(cheap_bf16((n, n), 2))
    t0 = time.perf_counter()
    orc.gemm_f32(a, b)
    return time.perf_counter() - t0


def cpu_plan(size):
    """(threads, n): the size the restatement is timed at -- `size` itself when a 1024^3 probe says it fits the
    budget, else the largest multiple of 256 that does."""
    from oracle import oracle as orc
    orc.clib().orc_set_threads(os.cpu_count() or 1)  # a launcher may have set OMP_NUM_THREADS=1
    cores = int(orc.clib().orc_threads())
    _cpu_product(512)                                   # first touch: thread pool, page faults
    rate = 2.0 * 1024 ** 3 / _cpu_product(1024)
    fits = int((rate * CPU_BUDGET_S / 2.0) ** (1.0 / 3.0)) // 256 * 256
    return cores, max(1024, min(size, fits))


def torch_cpu_column(n):
    """The same product by torch on the host cores (oneDNN / MKL, its own threads): a second CPU column, so the
    restatement's plain loops are not the only CPU figure beside the GPU's."""
    try:
        import torch
        threads = torch.get_num_threads()
        a = torch.from_numpy((cheap_bf16((n, n), 1).astype(np.uint32) << 16).view(np.float32))
        b = torch.from_numpy((cheap_bf16((n, n), 2).astype(np.uint32) << 16).view(np.float32))
        torch.matmul(a[:512, :512], b[:512, :512])
        t0 = time.perf_counter()
        torch.matmul(a, b)
        dt = time.perf_counter() - t0
        return {"value": 2.0 * n ** 3 / dt / 1e12, "unit": UNIT, "threads": int(threads), "sample": f"{n}^3 F32 torch.matmul, {dt:.2f} s"}
    except Exception as ex:   # a column, not the baseline: its absence is reported, not fatal
        return {"unavailable": str(ex)[:120]}


def cpu_gemm_baseline(size=N1_SIZE, repeats=1, with_torch=True):
    """The CPU restatement's F32 product of BF16-rounded operands on all host cores: the benchmark's own size when
    that fits the budget, else a smaller sample named in `sample` and `n`.  Median of `repeats` runs."""
    cores, n = cpu_plan(size)
    times = sorted(_cpu_product(n) for _ in range(max(1, repeats)))
    dt = times[len(times) // 2]
    out = {"value": 2.0 * n ** 3 / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port", "n": n,
           "sample": f"{n}^3 F32 product of BF16-rounded operands (C/OpenMP restatement of the comparison backend's "
                     f"arithmetic; not burn-flex itself), median of {len(times)} run(s), {dt:.2f} s"
                     + ("" if n == size else f"; the {size}^3 product would not fit {CPU_BUDGET_S:.0f} s")}
    if with_torch:
        out["torch_cpu"] = torch_cpu_column(min(n, 4096))
    return out


def run_reference(args):
    """The CPU arm: the restatement of the reference's comparison backend on the host cores, at the GPU arm's size
    when that fits the budget (the size actually run is in `config`).  A step is one whole product; as many of the
    requested steps are run as fit about two and a half minutes, and `steps` says how many that was."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    size = args.size or (N1_SIZE if args.gpus == 1 else NN_SIZE)
    cores, n = cpu_plan(size)
    first = _cpu_product(n)
    steps = max(1, min(args.steps, int(150.0 / max(first, 1e-3))))
    times = sorted([first] + [_cpu_product(n) for _ in range(steps - 1)])
    dt = times[len(times) // 2]
    v = 2.0 * n ** 3 / dt / 1e12
    base = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "n": n,
            "sample": f"{n}^3 F32 product of BF16-rounded operands, median of {steps} whole products, {dt:.2f} s each",
            "torch_cpu": torch_cpu_column(min(n, 4096))}
    name = workload_name(args.gpus) if n == size else f"bf16 gemm {n}^3 (a sample: the {size}^3 product does not fit {CPU_BUDGET_S:.0f} s of CPU time)"
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "steps_requested": args.steps, "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "m": n, "n": n, "k": n,
                       "note": "CPU restatement of the reference's comparison backend (burn-flex is not in the reference "
                               "tree and the reference itself is Rust for Tenstorrent cards); see cpu_baseline.sample"},
            "cpu_baseline": base,
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_name(n_gpus):
    if n_gpus == 1:
        return f"bf16 gemm {N1_SIZE}^3 (A [M,K], B [K,N] row-major, FP32 accumulate, bf16 out)"
    return f"bf16 gemm {NN_SIZE}^3 column-sharded over {n_gpus} GPUs, the whole C left on every rank"


# ---------------------------------------------------------------------- GPU arm
REPEATS = 9   # the reference's median-of-nine convention (docs/learnings/performance-scoreboard.md:24)


def make_timed(eng):
    """timed(fn, reps, warm, repeats) -> median over `repeats` of (device ms of `reps` back-to-back calls) / reps,
    CUDA events on the engine's stream, after `warm` untimed calls."""
    def timed(fn, reps=20, warm=3, repeats=1):
        for _ in range(warm):
            fn()
        eng.sync()
        got = []
        for _ in range(max(1, repeats)):
            eng.timer_start()
            for _ in range(reps):
                fn()
            got.append(eng.timer_stop() / reps)
        got.sort()
        return got[len(got) // 2]
    return timed


def bf16_value(bits):
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def sustained_leg(eng, a_ptr, b_ptr, n, flops, ms_guess):
    """The same product for about a second and a half, clocks sampled throughout: under the 1 kW cap the SM clock
    settles well below its maximum, and ms x MHz says whether the rate follows the clock (the kernel's tensor pipe is
    busy 91 % of the elapsed cycles in the ncu capture, whatever the clock).  Run last, so that the legs timed before it
    do not start on a GPU it has just heated."""
    ia = eng.upload_ptr(a_ptr, n, n, 3)
    ib = eng.upload_ptr(b_ptr, n, n, 3)

    def step():
        out, _ = eng.matmul_dram_bf16(ia, False, ib, False)
        eng.free(out)
    for _ in range(3):
        step()
    eng.sync()
    k_sus = int(1500.0 / ms_guess)
    s2 = ClockSampler(0)
    eng.timer_start()
    for _ in range(k_sus):
        step()
    sus_ms = eng.timer_stop() / k_sus
    c2 = s2.stop()
    eng.free(ia); eng.free(ib)
    return {"steps": k_sus, "ms_per_step": sus_ms, "tflops": flops / (sus_ms * 1e-3) / 1e12, "clocks": c2,
            "ms_x_mhz": sus_ms * c2["sm_mhz"] if c2.get("sm_mhz") else None,
            "implied_sm_mhz_at_0.914_tensor_pipe": flops / (sus_ms * 1e-3) / (0.914 * 148 * 8192) / 1e6,
            "path": eng.last_matmul_path()}


def run_single(args):
    import torch
    from metalium_rs_b200 import CudaEngine, build
    build.build()
    eng = CudaEngine(0, bf16_matmul_mode=2)  # tcgen05 or refuse: never a slower path silently
    n = args.size or N1_SIZE
    a_host = torch.from_numpy(cheap_bf16((n, n), 11).view(np.int16)).pin_memory()
    b_host = torch.from_numpy(cheap_bf16((n, n), 12).view(np.int16)).pin_memory()
    c_host = torch.empty((n, n), dtype=torch.int16).pin_memory()
    ia = eng.upload_ptr(a_host.data_ptr(), n, n, 3)
    ib = eng.upload_ptr(b_host.data_ptr(), n, n, 3)
    flops = 2.0 * n ** 3

    def step():
        out, _ = eng.matmul_dram_bf16(ia, False, ib, False)
        eng.free(out)

    for _ in range(max(args.warmup, 3)):
        step()
    eng.sync()

    launches0 = eng.device_traffic().launches
    sampler = ClockSampler(0)
    eng.sync()
    eng.timer_start()
    for _ in range(args.steps):
        step()
    ms = eng.timer_stop()
    clocks = sampler.stop()
    launches = eng.device_traffic().launches - launches0
    ms_per_step = ms / args.steps
    value = flops / (ms_per_step * 1e-3) / 1e12
    path = eng.last_matmul_path()
    # the legs that are not a kilowatt of dense product run now, on a second engine, before the product's repeats heat the
    # chip (the prefill replays some 4 % slower straight after them): the prefill, then the memory-bound suite
    from metalium_rs_b200 import CudaEngine as _E
    auto_eng = _E(0)   # automatic path choice: small and ragged products take the SIMT kernel
    timed = make_timed(auto_eng)
    prefill_res = None if args.no_prefill else prefill_leg(auto_eng, timed)
    suite_res = None if args.no_suite else suite_leg(auto_eng, timed)
    # the same region eight more times: the median of nine, beside the one region `value` is taken from
    rep = [ms_per_step]
    for _ in range(REPEATS - 1):
        eng.timer_start()
        for _ in range(args.steps):
            step()
        rep.append(eng.timer_stop() / args.steps)
    rep.sort()

    # validity: the BF16 result of the very call the loop times, 64 sampled elements against F64 dot products --
    # within one BF16 step of the truth plus the F32 sum's rounding
    out, _ = eng.matmul_dram_bf16(ia, False, ib, False)
    c = eng.download_bf16(out)
    eng.free(out)
    af, bf = bf16_value(a_host.numpy().view(np.uint16)), bf16_value(b_host.numpy().view(np.uint16))
    rng = np.random.default_rng(0)
    worst = 0.0
    for i, j in zip(rng.integers(0, n, 64), rng.integers(0, n, 64)):
        t = af[i].astype(np.float64) @ bf[:, j].astype(np.float64)
        s = np.abs(af[i]).astype(np.float64) @ np.abs(bf[:, j]).astype(np.float64)
        got = float(bf16_value(c[i, j]))
        if abs(got - t) > 2.0 ** -8 * abs(t) + 1e-5 * s:
            raise SystemExit(f"bench: the timed kernel's output is wrong at ({i}, {j}): {got} against {t}")
        worst = max(worst, abs(got - t) / s)
    del c

    # end to end through the C ABI with host buffers: one call of the host-staged BF16 product
    # (`b200_matmul_host_bf16`: A and B read from pinned host memory, C written to it, the copies overlapped
    # with the product in row panels)
    e2e_steps = 0 if args.no_e2e else max(1, min(args.steps, 5))
    mkn = (n, n, n)
    for _ in range(2 if e2e_steps else 0):
        eng.matmul_host_bf16_ptr(a_host.data_ptr(), b_host.data_ptr(), c_host.data_ptr(), mkn)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        eng.matmul_host_bf16_ptr(a_host.data_ptr(), b_host.data_ptr(), c_host.data_ptr(), mkn)
    e2e = None
    if e2e_steps:
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps     # the call returns when C is on the host
        got = c_host.numpy().view(np.uint16)
        rng2 = np.random.default_rng(1)
        for i, j in zip(rng2.integers(0, n, 16), rng2.integers(0, n, 16)):
            t = af[i].astype(np.float64) @ bf[:, j].astype(np.float64)
            s = np.abs(af[i]).astype(np.float64) @ np.abs(bf[:, j]).astype(np.float64)
            v = float(bf16_value(got[i, j]))
            if abs(v - t) > 2.0 ** -8 * abs(t) + 1e-5 * s:
                raise SystemExit(f"bench: the end-to-end product's output is wrong at ({i}, {j}): {v} against {t}")
        e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": 2 * n * n * 2,
               "d2h_bytes_per_step": n * n * 2, "ms_per_step": e2e_ms,
               "call": "b200_matmul_host_bf16 (pinned host A, B -> pinned host C; wall clock around the call)"}
    eng.free(ia); eng.free(ib)
    del af, bf

    pk, which = peaks()
    peak = float(pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    # traffic: dram__bytes_read.sum + dram__bytes_write.sum of one 8192^3 launch of this kernel under ncu (1,071.8 MB
    # read + 126.5 MB written with tile rows walked in groups of 8; profiles/gemm_tc2_bf16_8192.md); it cannot be
    # measured inside a timed run, and is null at other sizes
    traffic = 1071757000 + 126531000 if n == N1_SIZE else None
    roofline = {"bound": "tensor", "kernel": "gemm_tc2_kernel<K-major A, MN-major B> (CTA pairs, 256x256 tiles)",
                "achieved": value, "peak": peak, "unit": UNIT, "frac": value / peak,
                "peak_source": f"{which} cuBLAS bf16 burst", "frac_of_nominal_2250": value / 2250.0,
                "algorithmic_flops_per_launch": flops, "traffic": traffic, "traffic_unit": "bytes per launch",
                "traffic_source": "an ncu capture of one launch of this kernel at this size (not measured in this run)"}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": workload_name(1) if n == N1_SIZE else f"bf16 gemm {n}^3", "m": n, "n": n, "k": n,
                       "l2": "operands and result (403 MB at 8192^3) exceed the 126 MB L2; no flush needed",
                       "path": path},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline,
            "repeats": {"n": REPEATS, "steps_each": args.steps, "median_ms_per_step": rep[len(rep) // 2], "min_ms_per_step": rep[0],
                        "max_ms_per_step": rep[-1], "median_tflops": flops / (rep[len(rep) // 2] * 1e-3) / 1e12},
            "validated": {"samples": 64, "max_err_over_S": worst, "what": "the BF16 result of the timed call"}}
    eng.close()
    with auto_eng:
        if suite_res is not None:
            line["suite"] = suite_res
        if prefill_res is not None:
            line["prefill"] = prefill_res
        if args.extras:
            line["extras"] = extras(auto_eng, timed)
        if n == N1_SIZE and not args.no_e2e:
            sus = sustained_leg(auto_eng, a_host.data_ptr(), b_host.data_ptr(), n, flops, ms_per_step)
            pk_s = float(pk.get("bf16_tflops_sustained", 0) or 0)
            sus["frac_of_measured_sustained"] = sus["tflops"] / pk_s if pk_s else None
            sus["burst_implied_sm_mhz_at_0.914_tensor_pipe"] = value * 1e12 / (0.914 * 148 * 8192) / 1e6
            line["sustained"] = sus
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_gemm_baseline(n)
    print(json.dumps(line))


def suite_leg(eng, timed):
    """The memory-bound suite at its stated sizes: unary and broadcast-row kinds and the sums on [8192, 8192] F32, the
    row softmax on [4096, 32768].  GB/s of algorithmic bytes (what the op must read and write once), medians of nine
    repeats of twenty launches; operands (268 MB and up) exceed L2."""
    from metalium_rs_b200 import COLS, SUM, EltwiseOp, kinds
    pk, which = peaks()
    hbm = float(pk.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    res = {}
    rows = cols = 8192
    rng = np.random.default_rng(3)
    x = eng.upload(rng.random((rows, cols), dtype=np.float32) * 3.99 + 0.01, rows, cols)
    row = eng.upload(rng.random((1, cols), dtype=np.float32) + 0.5, 1, cols)
    nbytes = rows * cols * 4

    def entry(name, fn, algo_bytes, kernel):
        ms = timed(fn, reps=20, warm=3, repeats=REPEATS)
        gbs = algo_bytes / ms / 1e6
        res[name] = {"ms": ms, "gbs": gbs,
                     "roofline": {"bound": "hbm", "kernel": kernel, "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                                  "peak_source": f"{which} copy bandwidth", "frac_of_nominal_8000": gbs / 8000.0,
                                  "algorithmic_bytes_per_launch": algo_bytes}}

    for name, k, b in (("exp", kinds.EXP, None), ("log", kinds.LOG, None), ("recip", kinds.RECIP, None),
                       ("sqrt", kinds.SQRT, None), ("relu", kinds.RELU, None), ("gelu_tanh", kinds.GELU_TANH, None),
                       ("silu", kinds.SILU, None), ("add_row", kinds.ADD, row), ("mul_row", kinds.MUL, row),
                       ("div_row", kinds.DIV, row)):
        def f(k=k, b=b):
            o, _ = eng.eltwise_op(EltwiseOp(k, 0, 0), x, b)
            eng.free(o)
        entry(name, f, 2 * nbytes + (cols * 4 if b else 0), "elt_vec4")

    def fs():
        o, _ = eng.full_sum(x)
        eng.free(o)
    entry("full_sum", fs, nbytes + 4, "full_sum_fused")

    def fr():
        o, _ = eng.reduce(x, SUM, COLS)
        eng.free(o)
    entry("row_sum", fr, nbytes + rows * 4, "reduce_cols_kernel")
    # spot validity of what was timed: exp and the full sum against NumPy on the same data
    o, _ = eng.eltwise_op(EltwiseOp(kinds.EXP, 0, 0), x)
    xe = eng.download(x)[:8]
    if np.max(np.abs(eng.download(o)[:8] / np.exp(xe.astype(np.float64)) - 1.0)) > 1e-5:
        raise SystemExit("bench: the timed exp is wrong")
    eng.free(o)
    o, _ = eng.full_sum(x)
    total = float(eng.download(o)[0, 0])
    eng.free(o)
    exact = float(eng.download(x).astype(np.float64).sum())
    if abs(total - exact) > 1e-5 * abs(exact):
        raise SystemExit(f"bench: the timed full sum is wrong: {total} against {exact}")
    eng.free(x); eng.free(row)
    srows, scols = 4096, 32768
    sx = eng.upload(rng.random((srows, scols), dtype=np.float32) * 8 - 4, srows, scols)

    def fm():
        o, _ = eng.softmax_rows(sx, None, 1.0)
        eng.free(o)
    entry("softmax_4096x32768", fm, 2 * srows * scols * 4, "softmax_workers_kernel<512>")
    o, _ = eng.softmax_rows(sx, None, 1.0)
    sums = eng.download(o)[:16].astype(np.float64).sum(1)
    if np.max(np.abs(sums - 1.0)) > 1e-5:
        raise SystemExit("bench: the timed softmax's rows do not sum to one")
    eng.free(o); eng.free(sx)
    return res


OP_CLASSES = {"projections": ("projection qkv", "projection o", "projection gate|up", "projection down"),
              "attention": ("attention",), "norms": ("norm", "add + norm"), "rope": ("rope",),
              "element-wise": ("silu_mul",), "head": ("head",), "embedding": ("embedding",)}


def prefill_leg(eng, timed):
    """The SmolLM2-135M-shape prefill: 30 layers, 8 sequences of 512 tokens, BF16 weights N(0, 0.02), last-position
    logits and their argmax.  Timed as the replay of its trace (the reference's fastest mode); the eager pass gives
    the launch count and, under the engine's profile mode, device time by op class.  The logits are held to the
    committed sample of the CPU restatement's (2e-2; the argmax where its margin is clear)."""
    from metalium_rs_b200 import I32, workloads as W
    pk, which = peaks()
    peak = float(pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    cfg = W.LlamaConfig()
    batch, seq = 8, 512
    model = W.LlamaPrefill(eng, cfg, W.llama_weights(cfg), batch, seq)
    ids_host = W.prefill_ids(cfg, batch, seq)
    ids = eng.upload_bits(ids_host.view(np.uint32), 1, batch * seq, I32)
    l0 = eng.device_traffic().launches
    lg, am = model.forward(ids)
    per = eng.device_traffic().launches - l0
    eager_logits, eager_am = eng.download(lg), eng.download_bits(am).view(np.int32).ravel()
    eng.free(lg); eng.free(am)

    def fwd():
        a, b = model.forward(ids)
        eng.free(a); eng.free(b)
    eager_ms = timed(fwd, reps=5, warm=2, repeats=3)
    # device time by op class: one eager pass with every op under its class's label
    eng.profile_mode(True)
    fwd()
    table = eng.profile_mode(False)
    by_label = {r["op"]: r for r in table}
    classes = {}
    for cls, labels in OP_CLASSES.items():
        rows = [by_label[x] for x in labels if x in by_label]
        classes[cls] = {"ms": sum(r["device_ms"] for r in rows), "launches": int(sum(r["launches"] for r in rows))}
    total = sum(v["ms"] for v in classes.values())
    for v in classes.values():
        v["share"] = v["ms"] / total if total else 0.0
    tlg, tam = model.capture(ids)
    tms = timed(model.replay, reps=10, warm=2, repeats=REPEATS)
    traced_logits, traced_am = eng.download(tlg), eng.download_bits(tam).view(np.int32).ravel()
    footprint = eng.trace_footprint(model.trace)
    eng.release_trace(model.trace); eng.free(tlg); eng.free(tam); eng.free(ids)
    if not np.array_equal(traced_logits.view(np.uint32), eager_logits.view(np.uint32)) or not np.array_equal(traced_am, eager_am):
        raise SystemExit("bench: the replayed prefill's logits differ from the eager pass's")
    validated = {"replay_equals_eager_bits": True}
    gold_path = ROOT / "tests" / "golden" / "llama_prefill_8x512.npz"
    if gold_path.exists():
        gold = np.load(gold_path)
        if int(gold["ids_checksum"][0]) == int(ids_host.astype(np.int64).sum()):
            err = float(np.max(np.abs(np.take_along_axis(traced_logits, gold["columns"].astype(np.int64), 1) - gold["logits"])))
            clear = gold["margin"] > 4e-2
            same = bool(np.array_equal(traced_am[clear], gold["argmax"][clear]))
            if err > 2e-2 or not same:
                raise SystemExit(f"bench: the prefill's logits are off the CPU restatement's (max abs {err:.3e}, argmax agrees: {same})")
            validated.update({"max_abs_err_vs_cpu_restatement_sample": err, "argmax_agrees_where_margin_clear": same,
                              "clear_margins": int(clear.sum())})
    fl = model.flops()
    tflops = fl / tms / 1e9
    # the step after the prefill (the reference's traced generation step): one token a sequence over a fixed-shape cache,
    # the 30 layers as one launch, replayed as a trace; 64 steps from position 1 of 256 attended
    decode = {}
    rng = np.random.default_rng(0xDEC0)
    for nb, storage in ((1, "bf16"), (4, "bf16"), (1, "bfp8")):
        dec = W.LlamaDecode(eng, cfg, model.w, nb, max_len=512, attend=256, fused=True, weight_storage=storage)
        start = rng.integers(0, cfg.vocab, nb).astype(np.int32)
        dec.reset(start)
        dlg, dam = dec.capture()
        dec.reset(start)
        l0 = eng.device_traffic().launches
        dec.replay()
        dper = eng.device_traffic().launches - l0
        dms = timed(dec.replay, reps=64, warm=4)
        decode[f"batch{nb}" + ("_bfp8" if storage == "bfp8" else "")] = {
            "ms_per_step": dms, "tok_per_s": nb / (dms * 1e-3), "launches_per_step": int(dper), "weights": storage,
            "form": eng.last_decode_form(), "distinct_tokens_generated": int(len(np.unique(dec.generated(0, 69))))}
        eng.release_trace(dec.trace); eng.free(dlg); eng.free(dam)
        for pk in dec.packed:
            eng.free(pk)
    return {"tok_per_s": batch * seq / (tms * 1e-3), "ms": tms, "tokens": batch * seq, "launches": int(per), "decode_step": decode,
            "mode": "traced (CUDA graph replay), fused attention", "eager_ms": eager_ms,
            "eager_tok_per_s": batch * seq / (eager_ms * 1e-3), "trace_bytes": int(footprint),
            "next_tokens": traced_am.tolist(), "validated": validated, "op_classes_eager": classes,
            "roofline": {"bound": "tensor", "kernel": "the prefill's products and fused attention (K = 576 and 1536)", "achieved": tflops,
                         "peak": peak, "unit": UNIT, "frac": tflops / peak, "peak_source": f"{which} cuBLAS bf16 burst",
                         "algorithmic_flops_per_step": fl}}


def extras(eng, timed):
    """The other sizes of the sweep, the rest of the trait and the callers, timed the same way."""
    out = {"gemm_bf16": {}, "gemm_f32": {}}
    for n in (512, 1024, 2048, 4096, 8192):
        ia = eng.upload_bf16(cheap_bf16((n, n), 1), n, n)
        ib = eng.upload_bf16(cheap_bf16((n, n), 2), n, n)

        def f():
            o, _ = eng.matmul_dram_bf16(ia, False, ib, False)
            eng.free(o)
        ms = timed(f)
        out["gemm_bf16"][str(n)] = {"ms": ms, "tflops": 2.0 * n ** 3 / ms / 1e9, "path": eng.last_matmul_path()}
        eng.free(ia); eng.free(ib)
    for n in (512, 1024, 2048, 4096, 8192):
        rng = np.random.default_rng(n)
        ia = eng.upload(rng.random((n, n), dtype=np.float32) * 2 - 1, n, n)
        ib = eng.upload(rng.random((n, n), dtype=np.float32) * 2 - 1, n, n)

        def f():
            o, _ = eng.matmul_dram(ia, False, ib, False)
            eng.free(o)
        ms = timed(f, reps=5 if n >= 2048 else 20)
        out["gemm_f32"][str(n)] = {"ms": ms, "tflops": 2.0 * n ** 3 / ms / 1e9, "path": eng.last_matmul_path()}
        eng.free(ia); eng.free(ib)
    pk, _ = peaks()
    hbm = float(pk.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    out["rest_of_trait"] = rest_of_trait(eng, timed, hbm)
    out["callers"] = callers(eng, timed)
    return out


def rest_of_trait(eng, timed, hbm):
    """Scans, sort, binary16 casts, draws and taps: GB/s of algorithmic bytes (what each op must read and write once)."""
    from metalium_rs_b200 import F32, I32
    from metalium_rs_b200 import engine as E
    rng = np.random.default_rng(5)
    res = {}

    def one(name, make, nbytes):
        def f():
            r = make()
            for i in (r if isinstance(r, list) else [r]):
                eng.free(i)
        ms = timed(f, reps=10)
        res[name] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / hbm}

    n = 8192
    x = eng.upload(rng.random((n, n), dtype=np.float32), n, n)
    nb = n * n * 4
    one("scan_sum_8192x8192", lambda: eng.scan(x, E.SCAN_SUM)[0], 2 * nb)
    one("scan_min_nan_8192x8192", lambda: eng.scan(x, E.SCAN_MIN_NAN)[0], 2 * nb)
    one("cast_f16_narrow_8192x8192", lambda: eng.cast_f16(x, True)[0], nb * 3 // 2)
    h16, _ = eng.cast_f16(x, True)
    one("cast_f16_widen_8192x8192", lambda: eng.cast_f16(h16, False)[0], nb * 3 // 2)
    eng.free(h16)
    one("cast_block_4096x4096", lambda: eng.cast_block((x, (1024, 2048), (4096, 4096)), True)[0], 4096 * 4096 * 6)
    one("random_unit_8192x8192", lambda: eng.random_dram((n, n), ("unit",), 1)[0], nb)
    one("random_normal_8192x8192", lambda: eng.random_dram((n, n), ("normal", 0.0, 1.0, False), 1)[0], nb)
    eng.free(x)
    t = eng.upload(rng.random((1 << 20, 64), dtype=np.float32), 1 << 20, 64)
    one("scan_max_1Mx64_chunked", lambda: eng.scan(t, E.SCAN_MAX)[0], 3 * (1 << 20) * 64 * 4)
    one("scan_sum_1Mx64_row_order", lambda: eng.scan(t, E.SCAN_SUM)[0], 2 * (1 << 20) * 64 * 4)
    eng.free(t)
    p = eng.upload(rng.random((1024, 8192), dtype=np.float32), 1024, 8192)

    def srt():
        (k, _), i = eng.sort_planes(p, F32, 1024, False, True)
        return [k, i[0]]
    one("sort_8192_problems_x_1024", srt, 1024 * 8192 * 4 * 3)
    eng.free(p)
    tb = eng.upload_bf16(np.zeros((32768, 64), np.uint16), 32768, 64)
    idx = eng.upload_bits(rng.integers(0, 32768, (9, 32768)).astype(np.int32).view(np.uint32), 9, 32768, I32)
    one("select_taps_9x32768x64_bf16", lambda: eng.select_taps(tb, idx, True)[0], 9 * 32768 * 64 * 2 * 2)
    eng.free(tb); eng.free(idx)
    return res


def callers(eng, timed):
    """The callers either side of the kernels: the MLP training step (launch-bound: reported as
    latency and launches), the SmolLM2-135M-shape prefill (tokens/s) and the attention products."""
    from metalium_rs_b200 import I32, workloads as W
    res = {}
    rng = np.random.default_rng(0xC0F1)
    k1, k2 = 1 / np.sqrt(784), 1 / np.sqrt(128)
    u = lambda shape, k: (rng.random(shape, dtype=np.float32) * 2 - 1) * np.float32(k)
    mlp = W.MlpStep(eng, u((784, 128), k1), u((128,), k1), u((128, 10), k2), u((10,), k2))
    x = eng.upload(rng.standard_normal((64, 784), dtype=np.float32), 64, 784)
    y = eng.upload_bits(rng.integers(0, 10, (64, 1)).astype(np.int32).view(np.uint32), 64, 1, I32)
    losses = []

    def step():
        o = mlp.step(x, y, 64)
        losses.append(o["loss"])
    l0 = eng.device_traffic().launches
    step()
    per = eng.device_traffic().launches - l0
    ms = timed(step, reps=50, warm=5)
    first = float(eng.download(losses[0])[0, 0]); last = float(eng.download(losses[-1])[0, 0])
    for i in losses:
        eng.free(i)
    res["mlp_step_64x784x128x10"] = {"ms": ms, "launches_per_step": int(per), "loss_first": first, "loss_last": last}
    tm = W.MlpStep(eng, u((784, 128), k1), u((128,), k1), u((128, 10), k2), u((10,), k2), in_place=True)
    tl = tm.capture(x, y, 64)
    ms = timed(tm.replay, reps=200, warm=5)
    res["mlp_step_64x784x128x10"]["traced_ms"] = ms
    res["mlp_step_64x784x128x10"]["traced_loss_last"] = float(eng.download(tl)[0, 0])
    eng.release_trace(tm.trace); eng.free(tl)

    cfg = W.LlamaConfig()
    batch, seq = 8, 512
    model = W.LlamaPrefill(eng, cfg, W.llama_weights(cfg), batch, seq)
    ids = eng.upload_bits(rng.integers(0, cfg.vocab, (1, batch * seq)).astype(np.int32).view(np.uint32), 1, batch * seq, I32)
    outs = []

    def fwd():   # keeps the first and the latest result; everything else returns to the pool at once
        lg, am = model.forward(ids)
        if len(outs) == 2:
            plg, pam = outs.pop()
            eng.free(plg); eng.free(pam)
        outs.append((lg, am))
    l0 = eng.device_traffic().launches
    fwd()
    per = eng.device_traffic().launches - l0
    ms = timed(fwd, reps=5, warm=3)
    a0 = eng.download_bits(outs[0][1]).ravel().tolist(); a1 = eng.download_bits(outs[-1][1]).ravel().tolist()
    for lg, am in outs:
        eng.free(lg); eng.free(am)
    fl = model.flops()
    tlg, tam = model.capture(ids)
    tms = timed(model.replay, reps=10, warm=2)
    a2 = eng.download_bits(tam).ravel().tolist()
    eng.release_trace(model.trace); eng.free(tlg); eng.free(tam)
    res["smollm2_135m_prefill_8x512"] = {"ms": tms, "tok_per_s": batch * seq / (tms * 1e-3), "launches": int(per),
                                         "tflops": fl / tms / 1e9, "mode": "traced (CUDA graph replay), fused attention",
                                         "eager_ms": ms, "eager_tok_per_s": batch * seq / (ms * 1e-3),
                                         "argmax_stable": a0 == a1 == a2, "next_tokens": a1}
    # the reference-shaped composition of attention (batched Q K^T, softmax, batched P V), traced
    composed = W.LlamaPrefill(eng, cfg, W.llama_weights(cfg), batch, seq, fused_attention=False)
    clg, cam = composed.capture(ids)
    cms = timed(composed.replay, reps=10, warm=2)
    a3 = eng.download_bits(cam).ravel().tolist()
    eng.release_trace(composed.trace); eng.free(clg); eng.free(cam)
    res["smollm2_135m_prefill_8x512"].update({"composed_attention_ms": cms, "composed_tok_per_s": batch * seq / (cms * 1e-3),
                                              "composed_argmax_agrees": a3 == a2})

    # generation: decode steps over a fixed-shape KV cache, one traced step replayed a token
    for nb, fused, storage in ((1, False, "bf16"), (8, False, "bf16"), (1, True, "bf16"), (4, True, "bf16"), (1, True, "bfp8"),
                               (1, False, "bfp8")):
        dec = W.LlamaDecode(eng, cfg, model.w, nb, max_len=512, attend=256, fused=fused, weight_storage=storage)
        start = rng.integers(0, cfg.vocab, nb).astype(np.int32)
        dec.reset(start)
        dlg, dam = dec.capture()
        dec.reset(start)
        l0 = eng.device_traffic().launches
        dec.replay()
        dper = eng.device_traffic().launches - l0
        dms = timed(dec.replay, reps=64, warm=4)          # positions 1..69 of the 256 attended
        toks = dec.generated(0, 69)
        eng.release_trace(dec.trace); eng.free(dlg); eng.free(dam)
        for pk in dec.packed:
            eng.free(pk)
        name = f"smollm2_135m_decode_step_batch{nb}" + ("_one_launch" if fused else "") + ("_bfp8" if storage == "bfp8" else "")
        res[name] = {"ms_per_step": dms, "tok_per_s": nb / (dms * 1e-3), "launches_per_step": int(dper),
                                                     "layers": "one cooperative launch" if fused else "composed of the trait's ops",
                                                     "weights": storage,
                                                     "mode": "traced (one CUDA graph replay a token, nothing read back between steps)",
                                                     "attended_positions": 256, "distinct_tokens_generated": int(len(np.unique(toks)))}
    bh, t, d = 256, 2048, 128
    bf = lambda: ((rng.standard_normal((bh * t, d), dtype=np.float32)).view(np.uint32) >> 16).astype(np.uint16)
    q, k, v = (eng.upload_bf16(bf(), bh * t, d) for _ in range(3))

    def att():
        o = W.attention_products(eng, q, k, v, bh, t, d)
        eng.free(o)
    ms = timed(att, reps=3, warm=1)
    res["attention_16x16x2048x128"] = {"ms": ms, "tflops": 2 * 2.0 * bh * t * t * d / ms / 1e9,
                                       "materialised_scores_gb": bh * t * t * 4 / 1e9}
    blocks = eng.attention_block_array([((i * t, 0), (i * t, 0), (i * t, 0), (i * t, 0)) for i in range(bh)])

    def att_fused():
        o = W.attention_fused(eng, q, k, v, bh, t, d, blocks)
        eng.free(o)
    fms = timed(att_fused, reps=5, warm=2)
    res["attention_16x16x2048x128"].update({"fused_ms": fms, "fused_tflops": 2 * 2.0 * bh * t * t * d / fms / 1e9})
    # decode attention (`attention_rows`): 256 heads, one query row each, on 256 key/value heads of [4096, 128]
    from metalium_rs_b200 import BOOL
    for name, heads, kvh in (("attention_rows_256x4096x128_bf16", 256, 256), ("attention_rows_gqa4_512x4096x128_bf16", 512, 128)):
        l, dd = 4096, 128
        kb = ((rng.standard_normal((kvh * l, dd), dtype=np.float32)).view(np.uint32) >> 16).astype(np.uint16)
        dq = eng.upload(rng.standard_normal((heads, dd), dtype=np.float32), heads, dd)
        dk, dv_ = eng.upload_bf16(kb, kvh * l, dd), eng.upload_bf16(kb, kvh * l, dd)
        dm = eng.upload_bits(np.zeros(l, np.uint32), 1, l, BOOL)
        rep = heads // kvh
        heads_list = eng.attention_item_array([((h, 0), ((h // rep) * l, 0), ((h // rep) * l, 0)) for h in range(heads)])

        def dec():
            o, _ = eng.attention_rows([dq, dk, dv_, dm], heads_list, [1, dd, l, dd], 0.088)
            eng.free(o)
        dms = timed(dec, reps=10, warm=3)
        byts = 2 * kvh * l * dd * 2
        res[name] = {"ms": dms, "gbs_of_k_and_v_once": byts / dms / 1e6,
                     "frac_of_measured_hbm": byts / dms / 1e6 / float(peaks()[0].get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))}
        for i in (dq, dk, dv_, dm):
            eng.free(i)
    for i in (q, k, v, x, y, ids):
        eng.free(i)
    return res


def run_profile(args):
    """`--profile NAME`: a short fixed sequence for ncu captures (no JSON line, nothing timed).
    membound: EXP, MUL by a row, full sum, per-row sum on [8192,8192] F32, three rounds.
    softmax: three row softmaxes of [1024, 32768].  prefill: two SmolLM2-135M-shape forward passes.
    gemm_small: the four projections of a prefill layer ([4096,576]x[576,960], x[576,576], x[576,3072],
    [4096,1536]x[1536,576]), three rounds.  scan_sort: a row-order sum scan and a binary16 cast of [8192,8192] F32 and a
    sort of 8192 problems of 1024 positions, three rounds.  attention: three fused attentions of 64 blocks [1024, 128] (no mask).  decode: three `attention_rows`
    of 512 heads on 128 key/value heads of [4096, 128] BF16.  decode_step: three generation steps of the SmolLM2-135M shape at
    batch 1 with the layers as one launch.  gemm: three 8192^3 BF16 products."""
    from metalium_rs_b200 import COLS, I32, SUM, CudaEngine, EltwiseOp, build, kinds, workloads as W
    build.build()
    rng = np.random.default_rng(3)
    with CudaEngine(0) as eng:
        if args.profile == "membound":
            x = eng.upload(rng.random((8192, 8192), dtype=np.float32) * 3.99 + 0.01, 8192, 8192)
            row = eng.upload(rng.random((1, 8192), dtype=np.float32) + 0.5, 1, 8192)
            for _ in range(3):
                for k, b in ((kinds.EXP, None), (kinds.MUL, row)):
                    o, _ = eng.eltwise_op(EltwiseOp(k, 0, 0), x, b); eng.free(o)
                o, _ = eng.full_sum(x); eng.free(o)
                o, _ = eng.reduce(x, SUM, COLS); eng.free(o)
        elif args.profile == "softmax":
            x = eng.upload(rng.random((1024, 32768), dtype=np.float32) * 8 - 4, 1024, 32768)
            for _ in range(3):
                o, _ = eng.softmax_rows(x, None, 1.0); eng.free(o)
        elif args.profile == "prefill":
            cfg = W.LlamaConfig()
            m = W.LlamaPrefill(eng, cfg, W.llama_weights(cfg), 8, 512)
            ids = eng.upload_bits(rng.integers(0, cfg.vocab, (1, 4096)).astype(np.int32).view(np.uint32), 1, 4096, I32)
            for _ in range(2):
                lg, am = m.forward(ids); eng.free(lg); eng.free(am)
        elif args.profile == "gemm_small":
            # the four projections of a SmolLM2-135M-shape layer on 4096 tokens: qkv, o, gate|up, down
            bits = lambda r, c: (rng.standard_normal((r, c), dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
            shapes = [(4096, 576, 960, True), (4096, 576, 576, False), (4096, 576, 3072, True), (4096, 1536, 576, False)]
            ops = [(eng.upload_bf16(bits(m, k), m, k), eng.upload_bf16(bits(k, n), k, n), bf) for m, k, n, bf in shapes]
            for _ in range(3):
                for a, b, bf in ops:
                    o, _ = (eng.matmul_dram_bf16 if bf else eng.matmul_dram)(a, False, b, False); eng.free(o)
        elif args.profile == "attention":
            bh, t, d = 64, 1024, 128
            bits = lambda: (rng.standard_normal((bh * t, d), dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
            q, k, v = (eng.upload_bf16(bits(), bh * t, d) for _ in range(3))
            for _ in range(3):
                o = W.attention_fused(eng, q, k, v, bh, t, d); eng.free(o)
        elif args.profile == "decode":
            from metalium_rs_b200 import BOOL
            heads, kvh, l, d = 512, 128, 4096, 128
            q = eng.upload(rng.standard_normal((heads, d), dtype=np.float32), heads, d)
            kb = (rng.standard_normal((kvh * l, d), dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
            k, v = eng.upload_bf16(kb, kvh * l, d), eng.upload_bf16(kb, kvh * l, d)
            mask = eng.upload_bits(np.zeros(l, np.uint32), 1, l, BOOL)
            items = eng.attention_item_array([((h, 0), ((h // 4) * l, 0), ((h // 4) * l, 0)) for h in range(heads)])
            for _ in range(3):
                o, _ = eng.attention_rows([q, k, v, mask], items, [1, d, l, d], 0.088); eng.free(o)
        elif args.profile == "decode_step":
            # three generation steps of the SmolLM2-135M shape at batch 1, the layers as one cooperative launch
            cfg = W.LlamaConfig()
            m = W.LlamaPrefill(eng, cfg, W.llama_weights(cfg), 1, 128)
            dec = W.LlamaDecode(eng, cfg, m.w, 1, max_len=512, attend=256, fused=True)
            dec.reset(np.array([7], np.int32))
            for _ in range(3):
                lg, am = dec.step(); eng.free(lg); eng.free(am)
        elif args.profile == "gemm":
            # three 8192^3 BF16 products (the benchmark's kernel)
            n = args.size or 8192
            ia = eng.upload_bf16(cheap_bf16((n, n), 11), n, n)
            ib = eng.upload_bf16(cheap_bf16((n, n), 12), n, n)
            for _ in range(3):
                o, _ = eng.matmul_dram_bf16(ia, False, ib, False); eng.free(o)
        elif args.profile == "scan_sort":
            from metalium_rs_b200 import F32
            from metalium_rs_b200 import engine as E
            x = eng.upload(rng.random((8192, 8192), dtype=np.float32), 8192, 8192)
            p = eng.upload(rng.random((1024, 8192), dtype=np.float32), 1024, 8192)
            for _ in range(3):
                o, _ = eng.scan(x, E.SCAN_SUM); eng.free(o)
                o, _ = eng.cast_f16(x, True); eng.free(o)
                (k, _), i = eng.sort_planes(p, F32, 1024, False, True); eng.free(k); eng.free(i[0])
        else:
            raise SystemExit(f"unknown profile {args.profile!r}")
        eng.sync()
    print("profile sequence done:", args.profile)


def run_multi(args):
    from metalium_rs_b200 import sharded
    sharded.bench_main(args, METRIC, UNIT, NN_SIZE, workload_name, peaks, ClockSampler, cheap_bf16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--extras", action="store_true", help="also time the rest of the sweep and the memory-bound suite")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--no-suite", action="store_true", help="skip the memory-bound suite leg")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill leg")
    ap.add_argument("--profile", default="", help="run a short fixed sequence for an ncu capture: membound | softmax | prefill | gemm_small | attention | decode | scan_sort | decode_step | gemm")
    ap.add_argument("--size", type=int, default=0, help="override the N=1 problem size (profiling on a small case)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.profile:
        return run_profile(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 or world > 1:
        return run_multi(args)
    return run_single(args)


if __name__ == "__main__":
    main()

"""Benchmark of the B200 GEMM hot path (one JSON line on rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

N = 1   workload `gemm_bf16_4096`: bf16 4096^3 GEMM, fp32 accumulate and output (the configuration the
        headline metric is quoted on).  A step is one GEMM over one of several resident input sets.  The line also
        carries, under "secondary", short runs of the other single-GPU workloads of the metric (the skinny GEMMs and
        the W4A16 shapes, HBM-bound, reported in GB/s against the measured copy bandwidth; the other square sizes; the
        stand-alone dequantisation, the weight prepack and the f32 matmul entry).  A step of a skinny-GEMM or W4A16
        workload is one of 32 independent problems of a grouped launch; the same problems launched one at a time are
        reported beside it as `one_problem_per_launch`.
N > 1   workload `gemm_bf16_16384_sharded`: the 16384^3 GEMM sharded by N-column blocks, A replicated,
        each rank computes C[:, N/g slice]; no data-path collective (strong scaling).  Rank 0 then runs the whole
        16384^3 on its one GPU, so the line carries the single-GPU time and the speed-up over it; `gather` holds the
        step with the gathered C (GEMM + NCCL all-gather, and the one-kernel form whose epilogue stores to every rank).
`value` is whole-job TFLOP/s with inputs resident in HBM, timed with CUDA events on the launching
stream, max over ranks.  `e2e` is the same metric through the C-ABI call with pinned HOST buffers:
host->device copies of the step's operands and the device->host read of its result are inside the
timed region; the steps are handed over as one array (`t0_gemm_launch_host_batch`) so that consecutive
steps overlap on the link, and `e2e.serial_value` is the same steps made one blocking call after the other.
With N > 1 every rank uploads 1/N of A and the ranks complete it over NVLink, so A crosses the host link once.
`--impl reference` times the CPU restatement of the reference's own CPU GEMM on the
host cores for the same config (the reference's GPU path targets AMD RDNA through /dev/kfd and its Rust
toolchain is absent, so its CPU reference GEMM is the only part of it that can run on this box).
`--lib-ab` (measurement only, never on the product path) times the vendor library's bf16 GEMM beside the repo's kernel.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "gemm_bf16_4096": dict(m=4096, n=4096, k=4096),
    "gemm_bf16_2048": dict(m=2048, n=2048, k=2048),
    "gemm_bf16_8192": dict(m=8192, n=8192, k=8192),
    "gemm_bf16_16384_sharded": dict(m=16384, n=16384, k=16384),
    # HBM-bound workloads (the skinny and the W4A16 configurations); metric: algorithmic GB/s
    "gemm_bf16_skinny_128x4096x4096": dict(m=128, n=4096, k=4096, hbm=True),
    "gemm_bf16_skinny_64x4096x16384_sk4": dict(m=64, n=4096, k=16384, split_k=4, hbm=True),
    "w4a16_m1_n11008": dict(m=1, n=11008, k=4096, w4=True, hbm=True),
    "w4a16_m16_n11008": dict(m=16, n=11008, k=4096, w4=True, hbm=True),
    "w4a16_m1_n14336": dict(m=1, n=14336, k=4096, w4=True, hbm=True),
    "w4a16_m16_n14336": dict(m=16, n=14336, k=4096, w4=True, hbm=True),
    "w4a16_m128_n11008": dict(m=128, n=11008, k=4096, w4=True, hbm=True),
    "w4a16_m128_n14336": dict(m=128, n=14336, k=4096, w4=True, hbm=True),
}
# the callers and data formats either side of the path (reference wire-format dequantisation, the weight prepack, the f32
# framework entry): device-timed with --workload, not part of the default line
AUX_WORKLOADS = ["dequant_int4_f32_11008x4096", "dequant_int4_bf16_11008x4096", "w4_prepack_4096x11008", "matmul_f32_4096"]
SECONDARY = ["w4a16_m1_n11008", "w4a16_m16_n11008", "w4a16_m1_n14336", "w4a16_m16_n14336", "w4a16_m128_n11008", "w4a16_m128_n14336",
             "gemm_bf16_skinny_128x4096x4096", "gemm_bf16_skinny_64x4096x16384_sk4", "gemm_bf16_2048", "gemm_bf16_8192"]
W4_GROUP = 128


def ncu_traffic(name):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the workload's dominant kernel, from the ncu capture recorded
    in profiles/ncu_traffic.json (bytes, with the commit and date the capture was taken at); None when no capture exists."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            entry = json.load(f).get(name)
        return float(entry["bytes_per_launch"]) if entry else None
    except (OSError, ValueError, KeyError, TypeError):
        return None


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def tensor_peak(peaks, timed_ms):
    """The tensor-bound denominator: the burst figure for a timed region under a second, the sustained one beyond."""
    if timed_ms < 1000.0:
        return peaks["bf16_tflops"], f"{peaks['source']} (burst cuBLAS bf16: the timed region lasted {timed_ms:.0f} ms)"
    return peaks["bf16_tflops_sustained"], f"{peaks['source']} (sustained cuBLAS bf16: the timed region lasted {timed_ms:.0f} ms)"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=1.0)
        return {"sm_mhz": int(statistics.median(self.samples)) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------- HBM-bound workloads

def run_hbm_workload(args, name, rt=None, brief=False):
    """The single-GPU workloads that are HBM-bound: the skinny GEMMs and the W4A16 GEMM.  Returns one line with the
    same keys as the headline; `value` is algorithmic bytes / second (the bytes formula is in `config.bytes`).
    `brief` leaves out the end-to-end and CPU legs (the form the default run embeds under "secondary")."""
    import torch
    t0 = importlib.import_module("rust-gpu_b200")
    t0.lib()
    import oracle
    oracle.build()
    w = WORKLOADS[name]
    M, N, K = w["m"], w["n"], w["k"]
    w4 = bool(w.get("w4"))
    G = W4_GROUP
    steps = 96 if brief else (args.steps if args.steps is not None else 256)
    warmup = 8 if brief else max(3, args.warmup if args.warmup is not None else 10)
    torch.cuda.set_device(0)
    own_rt = rt is None
    if own_rt:
        rt = t0.GpuRuntime(0)
    bufs = []

    def alloc(n):
        b = rt.alloc(n)
        bufs.append(b)
        return b

    if w4:
        alg_bytes = K * N // 2 + (K // G) * N * 2 + (K // G) * N // 2 + M * K * 2 + M * N * 4
        set_bytes = K * N // 2 + (K // G) * N * 2 + (K // G) * N // 2
    else:
        alg_bytes = M * K * 2 + N * K * 2 + M * N * 4
        set_bytes = N * K * 2
    n_sets = max(2, -(-3 * 126 * 2 ** 20 // set_bytes))      # rotating weight sets: together three times the L2
    if not w4:
        n_sets = max(n_sets, 32)        # a grouped launch runs several of its 32 problems at once: every one has weights of its own
    a_host = oracle.fill_normal_bf16(M * K, 7 + M) if w4 else oracle.fill_uniform_bf16(M * K, 42 + M)
    xa = alloc(M * K * 2)
    xa.write(a_host)
    # the problems of one batched launch run concurrently, so consecutive steps write distinct outputs
    n_out = 32
    ys = [alloc(M * N * 4) for _ in range(n_out)]
    y = ys[(steps - 1) % n_out]          # the output of the last step, checked against the oracle below
    sets = []
    for s in range(n_sets):
        if w4:
            xp, xs, xz = rt.alloc((K // 8) * N * 4), rt.alloc((K // G) * N * 2), rt.alloc((K // G) * (N // 8) * 4)
            rt.fill_u32(xp.gpu_addr(), (K // 8) * N, 1000 + s)
            rt.fill_range_bf16(xs.gpu_addr(), (K // G) * N, 2000 + s, 0.001, 0.02)
            rt.fill_u32(xz.gpu_addr(), (K // G) * (N // 8), 3000 + s)
            sets.append((xp, xs, xz))
        else:
            xb = rt.alloc(N * K * 2)
            rt.fill_uniform_bf16(xb.gpu_addr(), N * K, 137 + N + 1000 * s)
            sets.append((xb,))
    if w4 and M <= 16 and not args.row_layout:
        # weights go to the streaming layout once, outside the timed region (a weight-load-time conversion)
        pre = [rt.w4_prepack(*(b.gpu_addr() for b in st), K, N, G) for st in sets]
        bufs += pre
        rt.synchronize()
        for st in sets:
            for b in st:
                b.free()
        calls = [t0.W4A16Args(xa.gpu_addr(), pre[i % n_sets].gpu_addr(), 0, 0, ys[i % n_out].gpu_addr(), M, N, K, G) for i in range(steps)]
        submit = rt.w4a16_gemm_prepacked_batch
        kernel = "w4a16_stream_kernel (streaming layout, one persistent launch per 32 problems)"
    elif w4:
        bufs += [b for st in sets for b in st]
        calls = [t0.W4A16Args(xa.gpu_addr(), *(b.gpu_addr() for b in sets[i % n_sets]), ys[i % n_out].gpu_addr(), M, N, K, G) for i in range(steps)]
        if M > 16 and not args.row_layout:
            # weights go to the tile-major layout once, outside the timed region (a weight-load-time conversion)
            til = [rt.w4_to_tiled(*(b.gpu_addr() for b in st), K, N, G) for st in sets]
            bufs += til
            rt.synchronize()
            calls = [t0.W4A16Args(xa.gpu_addr(), til[i % n_sets].gpu_addr(), 0, 0, ys[i % n_out].gpu_addr(), M, N, K, G) for i in range(steps)]

            def submit(cs):
                # 32 independent problems per launch (distinct weights and outputs): t0_w4a16_gemm_tiled_grouped
                for i in range(0, len(cs), 32):
                    rt.w4a16_gemm_tiled_grouped(cs[i:i + 32])
            kernel = "w4a16_umma_ts_kernel over the column tiles of 32 problems per launch (tile-major weights, dequantised into tensor memory in the main loop of a tcgen05 GEMM)"
        elif M > 16:
            def submit(cs):
                # 32 independent problems per launch (distinct weights and outputs): t0_w4a16_gemm_grouped
                for i in range(0, len(cs), 32):
                    rt.w4a16_gemm_grouped(cs[i:i + 32])
            kernel = "w4a16_umma_kernel over the column tiles of 32 problems per launch (row-layout weights, dequantisation in the main loop of a tcgen05 GEMM)"
        else:
            submit = rt.w4a16_gemm_batch
            kernel = "w4a16_tc_kernel (row layout, tcgen05)"
    else:
        bufs += [b for st in sets for b in st]
        cfg = t0.auto_select(M, K, N)
        sk = w.get("split_k", cfg.split())
        kw = dict(tile_n=cfg.tile_n, split_k=sk, swap_grid=bool(cfg.swap_grid), pair_cta=2)
        # grouped: tile and split left to the library, which chooses them for the group (32 skinny problems fill the GPU
        # without split-K); one problem per launch: the configuration auto_select gives the single problem (split-K 4)
        calls = [rt.gemm_args(xa.gpu_addr(), sets[i % n_sets][0].gpu_addr(), ys[i % n_out].gpu_addr(), M, N, K) for i in range(steps)]
        calls_single = [rt.gemm_args(xa.gpu_addr(), sets[i % n_sets][0].gpu_addr(), ys[i % n_out].gpu_addr(), M, N, K, **kw) for i in range(steps)]

        def submit(cs):
            # 32 independent problems per launch (distinct weights and outputs): t0_gemm_launch_grouped
            for i in range(0, len(cs), 32):
                rt.gemm_grouped(cs[i:i + 32])
        kernel = "gemm_bf16_tcgen05_kernel<128> over the tiles of 32 problems per launch (no split-K needed); one problem per launch: " + cfg.copy(split_k=sk).name()
    submit(calls[:warmup])
    rt.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    before = rt.launch_count()
    best = float("inf")
    for _ in range(3):
        rt.timer_start()
        submit(calls)
        best = min(best, rt.timer_stop())
    clocks = sampler.stop()
    launches = (rt.launch_count() - before) // 3
    per_launch_s = best * 1e-3 / steps
    gbs = alg_bytes / per_launch_s / 1e9
    one_per_launch = None
    if w4 and M > 16:
        single = float("inf")
        for _ in range(3):
            rt.timer_start()
            if args.row_layout:
                rt.w4a16_gemm_batch(calls)
            else:
                for c in calls:
                    rt.w4a16_gemm_tiled(c.a, c.packed, c.y, M, N, K, G)
            single = min(single, rt.timer_stop())
        one_per_launch = {"us_per_problem": single * 1e3 / steps, "value": alg_bytes / (single * 1e-3 / steps) / 1e9, "unit": "GB/s",
                          "frac": alg_bytes / (single * 1e-3 / steps) / 1e9 / measured_peaks()["hbm_gbs"]}
    if not w4:
        # the same problems one launch each (t0_gemm_launch_batch), for comparison
        single = float("inf")
        for _ in range(3):
            rt.timer_start()
            rt.gemm_batch(calls_single)
            single = min(single, rt.timer_stop())
        one_per_launch = {"us_per_problem": single * 1e3 / steps, "value": alg_bytes / (single * 1e-3 / steps) / 1e9, "unit": "GB/s",
                          "frac": alg_bytes / (single * 1e-3 / steps) / 1e9 / measured_peaks()["hbm_gbs"]}

    # parity of the last step against the oracle (full result: these shapes are small)
    s_idx = (steps - 1) % n_sets
    got = y.read(M * N * 4, np.float32).reshape(M, N)
    if w4:
        ref = oracle.w4a16_gemm(a_host, oracle.fill_u32((K // 8) * N, 1000 + s_idx), oracle.fill_range_bf16((K // G) * N, 2000 + s_idx, 0.001, 0.02),
                                oracle.fill_u32((K // G) * (N // 8), 3000 + s_idx), M, N, K, G)
    else:
        ref = oracle.gemm_nt(a_host, oracle.fill_uniform_bf16(N * K, 137 + N + 1000 * s_idx), M, K, N)
    err = float(np.abs(got - ref).max())
    tol = 5e-3 * (K / 256) ** 0.5
    if not err <= tol:
        print(json.dumps({"error": "parity check failed", "workload": name, "max_abs_err": err, "tol": tol}), flush=True)
        sys.exit(1)

    peaks = measured_peaks()
    tflops = 2.0 * M * N * K / per_launch_s / 1e12
    line = {"metric": "w4a16_hbm_gbs" if w4 else "skinny_gemm_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": per_launch_s * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int4 x bf16 -> f32" if w4 else "bf16", "data": "synthetic",
            "config": {"workload": name, "m": M, "n": N, "k": K, "group": G if w4 else None, "kernel": kernel, "bytes": alg_bytes,
                       "tflops": tflops, "input_sets": n_sets,
                       "l2": f"{n_sets} resident weight sets of {set_bytes >> 20} MiB rotate (> 126 MB L2)",
                       "pct_of_nominal_hbm": round(100.0 * gbs / 8000.0, 1)},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                         "traffic": ncu_traffic(name), "peak_source": f"{peaks['source']} (copy bandwidth)"},
            "clocks": clocks, "gpu_launches": int(launches), "parity": {"max_abs_err": err, "tol": tol}}
    if one_per_launch:
        line["one_problem_per_launch"] = one_per_launch
    if w4 and M > 16:
        # above the ridge point both roofs apply: also the tensor-bound fraction
        line["roofline"]["tensor_frac"] = tflops / peaks["bf16_tflops"]

    if not brief:
        # end to end: the step's activations go up from pinned host memory, the result comes back; weights stay resident
        a_pin = torch.from_numpy(a_host.view(np.int16).copy()).pin_memory().numpy()
        y_pin = torch.empty(M * N, dtype=torch.float32).pin_memory().numpy()
        C = __import__("ctypes")
        e2e_steps = min(steps, 50)
        t_start = time.perf_counter()
        for i in range(e2e_steps):
            xa.write(a_pin)
            submit([calls[i]])
            t0._check(t0.lib().t0_rt_read_f32(rt._h, ys[i % n_out]._h, M * N, y_pin.ctypes.data_as(C.c_void_p)))
        e2e_s = (time.perf_counter() - t_start) / e2e_steps
        line["e2e"] = {"value": alg_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 4,
                       "steps": e2e_steps, "note": "weights resident; the step's activations and result cross PCIe"}
        # CPU baseline on a bounded sample: all rows, the first n_cpu columns
        n_cpu = min(N, 2048)
        t_cpu = float("inf")
        if w4:
            pk = oracle.fill_u32((K // 8) * N, 1000).reshape(K // 8, N)[:, :n_cpu].copy().reshape(-1)
            sc = oracle.fill_range_bf16((K // G) * N, 2000, 0.001, 0.02).reshape(K // G, N)[:, :n_cpu].copy().reshape(-1)
            zp = oracle.fill_u32((K // G) * (n_cpu // 8), 3000)
            for _ in range(3):
                t = time.perf_counter(); oracle.w4a16_gemm(a_host, pk, sc, zp, M, n_cpu, K, G); t_cpu = min(t_cpu, time.perf_counter() - t)
        else:
            bh = oracle.fill_uniform_bf16(n_cpu * K, 137 + N)
            for _ in range(3):
                t = time.perf_counter(); oracle.gemm_nt(a_host, bh, M, K, n_cpu); t_cpu = min(t_cpu, time.perf_counter() - t)
        line["cpu_baseline"] = {"value": alg_bytes * (n_cpu / N) / t_cpu / 1e9, "unit": "GB/s", "cores": oracle.host_threads(), "kind": "port",
                                "sample": f"all {M} rows, the first {n_cpu} of {N} columns, best of 3, {t_cpu:.3f} s per pass"}
    rt.synchronize()
    for b in bufs:
        b.free()
    if own_rt:
        rt.close()
    return line


def run_aux_workload(args, name, rt=None, brief=False):
    """Kernels beside the GEMM itself, each at a size larger than L2: the stand-alone dequantisation in the reference's wire
    format (quant_kernels.rs:53-171), the one-time weight prepack, and the f32 entry matmul(x f32, w f32)
    (bf16_matmul.rs:33-59: two conversion passes plus the GEMM).  One JSON line each; parity on a sample."""
    import torch
    t0 = importlib.import_module("rust-gpu_b200")
    t0.lib()
    import oracle
    oracle.build()
    own_rt = rt is None
    if own_rt:
        torch.cuda.set_device(0)
        rt = t0.GpuRuntime(0)
    peaks = measured_peaks()
    steps = 20 if brief else (args.steps if args.steps is not None else 40)
    warmup = 3 if brief else max(3, args.warmup if args.warmup is not None else 4)
    bufs = []

    def A(n_bytes):
        bufs.append(rt.alloc(n_bytes))
        return bufs[-1]

    def U(host):
        bufs.append(rt.upload(host))
        return bufs[-1]

    line = {"n_gpus": 1, "steps": steps, "warmup": warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic"}

    def time_steps(fn):
        for i in range(warmup):
            fn(i)
        rt.synchronize()
        best = float("inf")
        before = rt.launch_count()
        for _ in range(3):
            rt.timer_start()
            for i in range(steps):
                fn(i)
            best = min(best, rt.timer_stop())
        return best * 1e-3 / steps, (rt.launch_count() - before) // 3

    if name.startswith("dequant_int4"):
        rows, cols, glog = 11008, 4096, 7
        bf16 = "bf16" in name
        n_groups = cols >> glog
        n_sets = 8                                              # 8 x 22 MiB of packed codes rotate; the output alone exceeds the L2
        scales_h = (0.001 + 0.019 * (np.arange(rows * n_groups) % 97) / 97.0).astype(np.float32)
        zps_h = (np.arange(rows * n_groups) % 16).astype(np.int32)
        xs, xz = U(scales_h), U(zps_h)
        packs = []
        for s in range(n_sets):
            b = A(rows * cols // 2)
            rt.fill_u32(b.gpu_addr(), rows * cols // 8, 500 + s)
            packs.append(b)
        outs = [A(rows * cols * (2 if bf16 else 4)) for _ in range(2)]
        sec, launches = time_steps(lambda i: rt.dequant_int4(packs[i % n_sets].gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), outs[i % 2].gpu_addr(),
                                                            rows, cols, glog, bf16))
        alg = rows * cols // 2 + rows * n_groups * 8 + rows * cols * (2 if bf16 else 4)
        # parity: the first 64 rows of the last step, bit for bit
        s_idx, o_idx, r = (steps - 1) % n_sets, (steps - 1) % 2, 64
        pk = oracle.fill_u32(rows * cols // 8, 500 + s_idx)[: r * cols // 8].view(np.uint8)
        want = oracle.dequant_int4_ref(pk, scales_h[: r * n_groups], zps_h[: r * n_groups], r, cols, glog, bf16)
        got = outs[o_idx].read(r * cols * (2 if bf16 else 4), np.uint16 if bf16 else np.float32).reshape(r, cols)
        ok = bool(np.array_equal(got, want))
        line.update({"metric": "dequant_hbm_gbs", "value": alg / sec / 1e9, "unit": "GB/s", "ms_per_step": sec * 1e3,
                     "dtype": "int4 -> " + ("bf16 (truncated)" if bf16 else "f32"),
                     "config": {"workload": name, "rows": rows, "cols": cols, "group": 1 << glog, "kernel": "dequant_int4_ref_kernel", "bytes": alg},
                     "roofline": {"bound": "hbm", "achieved": alg / sec / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": alg / sec / 1e9 / peaks["hbm_gbs"],
                                  "traffic": ncu_traffic(name), "peak_source": f"{peaks['source']} (copy bandwidth)"},
                     "gpu_launches": int(launches), "parity": {"rows_compared": r, "bit_exact": ok}})
    elif name.startswith("w4_prepack"):
        K, N, G = 4096, 11008, 128
        n_sets = 8
        sets = []
        for s in range(n_sets):
            xp, xs, xz = A((K // 8) * N * 4), A((K // G) * N * 2), A((K // G) * (N // 8) * 4)
            rt.fill_u32(xp.gpu_addr(), (K // 8) * N, 1000 + s)
            rt.fill_range_bf16(xs.gpu_addr(), (K // G) * N, 2000 + s, 0.001, 0.02)
            rt.fill_u32(xz.gpu_addr(), (K // G) * (N // 8), 3000 + s)
            sets.append((xp, xs, xz))
        nbytes = t0.lib().t0_w4_prepacked_bytes(K, N, G)
        outs = [A(nbytes) for _ in range(8)]
        C = __import__("ctypes")
        sec, launches = time_steps(lambda i: t0._check(t0.lib().t0_w4_prepack(rt._h, *(b.gpu_addr() for b in sets[i % n_sets]), outs[i % 8].gpu_addr(), K, N, G)))
        alg = 2 * nbytes
        s_idx = (steps - 1) % n_sets
        want = oracle.w4_prepack(oracle.fill_u32((K // 8) * N, 1000 + s_idx), oracle.fill_range_bf16((K // G) * N, 2000 + s_idx, 0.001, 0.02),
                                 oracle.fill_u32((K // G) * (N // 8), 3000 + s_idx), K, N, G)
        ok = bool(np.array_equal(outs[(steps - 1) % 8].read(nbytes, np.uint8), want))
        line.update({"metric": "prepack_hbm_gbs", "value": alg / sec / 1e9, "unit": "GB/s", "ms_per_step": sec * 1e3, "dtype": "u32",
                     "config": {"workload": name, "k": K, "n": N, "group": G, "kernel": "w4_prepack_kernel", "bytes": alg},
                     "roofline": {"bound": "hbm", "achieved": alg / sec / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": alg / sec / 1e9 / peaks["hbm_gbs"],
                                  "traffic": ncu_traffic(name), "peak_source": f"{peaks['source']} (copy bandwidth)"},
                     "gpu_launches": int(launches), "parity": {"bit_exact": ok}})
    else:
        M = N = K = 4096
        rng = np.random.default_rng(3)
        x_h = rng.uniform(-1, 1, size=M * K).astype(np.float32)
        w_h = rng.uniform(-1, 1, size=K * N).astype(np.float32)
        xs_ = [U(x_h), U(x_h)]
        ws_ = [U(w_h), U(w_h)]
        ys_ = [A(M * N * 4) for _ in range(2)]
        sec, launches = time_steps(lambda i: rt.matmul_f32(xs_[i % 2].gpu_addr(), ws_[i % 2].gpu_addr(), ys_[i % 2].gpu_addr(), M, K, N))
        rows = [0, 2049, 4095]
        xb = oracle.f32_to_bf16_rne(x_h.reshape(M, K)[rows].reshape(-1))
        wb = oracle.f32_to_bf16_rne(w_h)
        ref = oracle.gemm_nn(xb, wb, len(rows), K, N)
        got = np.stack([ys_[(steps - 1) % 2].read_bytes(r * N * 4, N * 4, np.float32) for r in rows])
        err = float(np.abs(got - ref).max())
        tol = 5e-3 * (K / 256) ** 0.5
        ok = err <= tol
        tf = 2.0 * M * N * K / sec / 1e12
        line.update({"metric": "matmul_f32_tflops", "value": tf, "unit": "TFLOP/s", "ms_per_step": sec * 1e3, "dtype": "f32 in, bf16 multiply, f32 accumulate and out",
                     "config": {"workload": name, "m": M, "n": N, "k": K, "kernel": "cvt_f32_bf16_kernel x2 + gemm (B[K,N] layout)",
                                "extra_bytes": "two conversion passes: 2 x (64 MiB read + 32 MiB written)"},
                     "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"],
                                  "traffic": ncu_traffic(name), "peak_source": f"{peaks['source']} (burst cuBLAS bf16)"},
                     "gpu_launches": int(launches), "parity": {"sampled_rows": rows, "max_abs_err": err, "tol": tol}})
    if own_rt:
        rt.close()
    else:
        for b in bufs:
            b.free()
    if not ok:
        print(json.dumps({"error": "parity check failed", "workload": name, "parity": line["parity"]}), flush=True)
        sys.exit(1)
    return line


def run_square_brief(t0, rt, name):
    """A short device-resident run of another size of the square sweep, for the default line's "secondary" list."""
    import oracle
    w = WORKLOADS[name]
    M, N, K = w["m"], w["n"], w["k"]
    set_bytes = M * K * 2 + N * K * 2 + M * N * 4
    n_sets = max(2, min(4, -(-3 * 126 * 2 ** 20 // set_bytes)))
    sets = []
    for s in range(n_sets):
        xa, xb, y = rt.alloc(M * K * 2), rt.alloc(N * K * 2), rt.alloc(M * N * 4)
        rt.fill_uniform_bf16(xa.gpu_addr(), M * K, 42 + M + 1000 * s)
        rt.fill_uniform_bf16(xb.gpu_addr(), N * K, 137 + N + 1000 * s)
        sets.append((xa, xb, y))
    steps = 60 if M <= 4096 else 20
    calls = [rt.gemm_args(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), M, N, K) for (xa, xb, y) in sets]
    rt.gemm_batch([calls[i % n_sets] for i in range(6)])
    rt.synchronize()
    best = float("inf")
    for _ in range(3):
        rt.timer_start()
        rt.gemm_batch([calls[i % n_sets] for i in range(steps)])
        best = min(best, rt.timer_stop())
    s_idx = (steps - 1) % n_sets
    xa, xb, y = sets[s_idx]
    rows = [0, M // 2 + 1, M - 1]
    b_host = oracle.fill_uniform_bf16(N * K, 137 + N + 1000 * s_idx)
    worst = 0.0
    for r in rows:
        ref = oracle.gemm_nt(oracle.fill_uniform_bf16(K, 42 + M + 1000 * s_idx, r * K), b_host, 1, K, N)
        worst = max(worst, float(np.abs(ref[0] - y.read_bytes(r * N * 4, N * 4, np.float32)).max()))
    tol = 5e-3 * (K / 256) ** 0.5
    if not worst <= tol:
        print(json.dumps({"error": "parity check failed", "workload": name, "max_abs_err": worst, "tol": tol}), flush=True)
        sys.exit(1)
    for st in sets:
        for b in st:
            b.free()
    peaks = measured_peaks()
    tf = 2.0 * M * N * K * steps / (best * 1e-3) / 1e12
    peak, src = tensor_peak(peaks, best)
    return {"workload": name, "metric": "bf16_gemm_tflops", "value": tf, "unit": "TFLOP/s", "ms_per_step": best / steps, "steps": steps,
            "roofline": {"bound": "tensor", "frac": tf / peak, "peak": peak, "traffic": ncu_traffic(name), "peak_source": src},
            "gpu_launches": steps, "parity": {"sampled_rows": rows, "max_abs_err": worst, "tol": tol}}


def cpu_baseline(oracle, m, n, k, rows, threads=0):
    """Times the oracle's reference GEMM on `rows` rows of the workload; returns (TFLOP/s, seconds, cores)."""
    a = oracle.fill_uniform_bf16(rows * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    oracle.gemm_nt(a[: 8 * k], b, 8, k, n, threads)   # page in, spin up
    best = float("inf")
    for _ in range(3):                                # steady clock around the region, best of 3
        t = time.perf_counter()
        oracle.gemm_nt(a, b, rows, k, n, threads)
        best = min(best, time.perf_counter() - t)
    cores = threads if threads > 0 else oracle.host_threads()
    return 2.0 * rows * n * k / best / 1e12, best, cores


def run_reference_arm(args, rank, world):
    """`--impl reference`: the reference's own CPU reference GEMM (src/t0/tile_ir.rs:5021-5038), restated in
    oracle/oracle.c, on all host cores.  Rank 0 alone runs it."""
    if rank != 0:
        return
    import oracle
    oracle.build()
    name = args.workload or ("gemm_bf16_4096" if world == 1 else "gemm_bf16_16384_sharded")
    w = WORKLOADS[name]
    m, n, k = w["m"], w["n"], w["k"]
    # bounded sample: the whole matrix when it is 4096^3-sized, else a row block with the same work (extrapolated)
    rows = max(32, min(m, int(m * (2.0 * 4096 ** 3) / (2.0 * m * n * k))))
    a = oracle.fill_uniform_bf16(rows * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    for _ in range(args.warmup):
        oracle.gemm_nt(a, b, rows, k, n)
    t = time.perf_counter()
    for _ in range(args.steps):
        oracle.gemm_nt(a, b, rows, k, n)
    dt = time.perf_counter() - t
    tflops = 2.0 * rows * n * k * args.steps / dt / 1e12
    full_ms = dt / args.steps * (m / rows) * 1e3
    sample = (f"the full {m}x{n}x{k} GEMM per step" if rows == m else
              f"rows 0..{rows - 1} of {m} per step, full-matrix time extrapolated linearly")
    line = {"impl": "reference", "metric": "bf16_gemm_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": full_ms, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "m": m, "n": n, "k": k, "layout": "NT", "out": "f32"},
            "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": oracle.host_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def device_alias(ptr, n_elems, np_dtype):
    """A torch tensor over device memory the runtime owns (no copy): what torch.distributed needs to move that memory."""
    import torch

    class _Raw:
        pass
    raw = _Raw()
    raw.__cuda_array_interface__ = {"shape": (n_elems,), "typestr": np.dtype(np_dtype).str, "data": (ptr, False), "version": 2}
    return torch.as_tensor(raw, device="cuda")


def run_lib_ab(t0, rt, torch):
    """Measurement only: the vendor library's bf16 GEMM (torch.matmul, bf16 output: it writes half the bytes of the repo's f32
    output) timed right after the repo's kernel, in the same process, on buffers of the same sizes, with the same step
    count, warm-up and CUDA-event timing.  Reported per arm: TFLOP/s, the SM clock (the repo's kernel stamps cycles and
    nanoseconds itself; the library arm uses the NVML median) and time x clock = SM cycles per launch."""
    out = []
    for (M, N, K) in ((128, 4096, 4096), (64, 4096, 16384), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192)):
        size = f"{M}x{N}x{K}" if not (M == N == K) else M
        n_sets = max(2, min(12, -(-3 * 126 * 2 ** 20 // (M * K * 2 + N * K * 2 + M * N * 4))))
        steps = 200 if M * N * K <= 4096 ** 3 else 40
        sets = []
        for s in range(n_sets):
            xa, xb, y = rt.alloc(M * K * 2), rt.alloc(N * K * 2), rt.alloc(M * N * 4)
            rt.fill_uniform_bf16(xa.gpu_addr(), M * K, 42 + M + 1000 * s)
            rt.fill_uniform_bf16(xb.gpu_addr(), N * K, 137 + N + 1000 * s)
            sets.append((xa, xb, y))
        calls = [rt.gemm_args(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), M, N, K) for (xa, xb, y) in sets]
        rt.gemm_batch([calls[i % n_sets] for i in range(10)])
        rt.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        ms_ours = float("inf")
        for _ in range(3):
            rt.timer_start()
            rt.gemm_batch([calls[i % n_sets] for i in range(steps)])
            ms_ours = min(ms_ours, rt.timer_stop())
        clk_ours = sampler.stop()
        mhz_kernel, _ = rt.last_kernel_clock()
        # the repo's kernel once more with bf16 output: the library arm below writes bf16, half the output bytes
        calls16 = [rt.gemm_args(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), M, N, K, out_bf16=True) for (xa, xb, y) in sets]
        rt.gemm_batch([calls16[i % n_sets] for i in range(10)])
        rt.synchronize()
        ms_ours16 = float("inf")
        for _ in range(3):
            rt.timer_start()
            rt.gemm_batch([calls16[i % n_sets] for i in range(steps)])
            ms_ours16 = min(ms_ours16, rt.timer_stop())
        # the library arm on torch tensors aliasing the same device buffers
        ta = [device_alias(xa.gpu_addr(), M * K, np.int16).view(torch.bfloat16).view(M, K) for (xa, _, _) in sets]
        tb = [device_alias(xb.gpu_addr(), N * K, np.int16).view(torch.bfloat16).view(N, K) for (_, xb, _) in sets]
        tc = [torch.empty(M, N, dtype=torch.bfloat16, device="cuda") for _ in sets]
        for i in range(10):
            torch.matmul(ta[i % n_sets], tb[i % n_sets].t(), out=tc[i % n_sets])
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        ms_lib = float("inf")
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(steps):
                torch.matmul(ta[i % n_sets], tb[i % n_sets].t(), out=tc[i % n_sets])
            e1.record()
            torch.cuda.synchronize()
            ms_lib = min(ms_lib, e0.elapsed_time(e1))
        clk_lib = sampler.stop()
        flop = 2.0 * M * N * K
        ours = {"tflops": flop * steps / (ms_ours * 1e-3) / 1e12, "us_per_launch": ms_ours * 1e3 / steps, "sm_mhz_in_kernel": round(mhz_kernel),
                "sm_mhz_nvml_median": clk_ours["sm_mhz"], "sm_cycles_per_launch": ms_ours * 1e3 / steps * mhz_kernel, "output": "f32"}
        lib = {"tflops": flop * steps / (ms_lib * 1e-3) / 1e12, "us_per_launch": ms_lib * 1e3 / steps, "sm_mhz_nvml_median": clk_lib["sm_mhz"],
               "sm_cycles_per_launch_at_nvml_clock": ms_lib * 1e3 / steps * (clk_lib["sm_mhz"] or 0), "output": "bf16 (half the output bytes)",
               "what": "torch.matmul(A[M,K] bf16, WT[N,K].t()) -> bf16, the vendor library's choice of kernel"}
        ours16 = {"tflops": flop * steps / (ms_ours16 * 1e-3) / 1e12, "us_per_launch": ms_ours16 * 1e3 / steps, "output": "bf16"}
        out.append({"size": size, "steps": steps, "ours": ours, "ours_bf16_output": ours16, "library": lib, "ours_over_library": ours["tflops"] / lib["tflops"],
                    "ours_bf16_output_over_library": ours16["tflops"] / lib["tflops"]})
        del ta, tb, tc
        for st in sets:
            for b in st:
                b.free()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS) + AUX_WORKLOADS)
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="default single-GPU run: leave out the short runs of the other workloads")
    ap.add_argument("--layout", default="nt", choices=["nt", "nn"], help="B as WT[N,K] (the reference's native layout) or as B[K,N]")
    ap.add_argument("--no-gather", action="store_true", help="sharded workload: leave out the gathered-C legs")
    ap.add_argument("--gather", action="store_true", help="sharded workload: also time GEMM + in-place NCCL all-gather of C, and the one-kernel form whose epilogue stores to every rank (reported under \"gather\")")
    ap.add_argument("--row-layout", action="store_true", help="W4A16 workloads: weights in the row layout instead of the streaming layout")
    ap.add_argument("--lib-ab", action="store_true", help="measurement only: time the vendor library's bf16 GEMM beside the repo's kernel (single GPU)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        print(f"bench.py --gpus {args.gpus} must be launched through torch.distributed.run", file=sys.stderr)
        sys.exit(2)

    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 3
        args.warmup = args.warmup if args.warmup is not None else 1
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    t0 = importlib.import_module("rust-gpu_b200")
    t0.lib()   # raises if the CUDA library is missing: there is no fallback path

    if args.lib_ab:
        torch.cuda.set_device(0)
        rt = t0.GpuRuntime(0)
        print(json.dumps({"lib_ab": run_lib_ab(t0, rt, torch)}), flush=True)
        rt.close()
        return

    if args.workload in AUX_WORKLOADS:
        print(json.dumps(run_aux_workload(args, args.workload)), flush=True)
        return
    default_run = args.workload is None
    name = args.workload or ("gemm_bf16_4096" if world == 1 else "gemm_bf16_16384_sharded")
    if WORKLOADS[name].get("hbm"):
        if world != 1:
            print(f"workload {name} is single-GPU (replicas only)", file=sys.stderr)
            sys.exit(2)
        print(json.dumps(run_hbm_workload(args, name)), flush=True)
        return
    sharded = name.endswith("_sharded")
    w = WORKLOADS[name]
    M, N_total, K = w["m"], w["n"], w["k"]
    N = N_total // world if sharded else N_total
    steps = args.steps if args.steps is not None else (200 if not sharded else 20)
    warmup = max(3, args.warmup if args.warmup is not None else (10 if not sharded else 3))

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    rt = t0.GpuRuntime(local_rank)

    # resident inputs: several sets so consecutive steps do not find their operands in L2 (126 MB)
    set_bytes = M * K * 2 + N * K * 2 + M * N * 4
    n_sets = 1 if sharded else max(2, min(4, -(-3 * 126 * 2 ** 20 // set_bytes)))
    sets = []
    for s in range(n_sets):
        xa, xb, y = rt.alloc(M * K * 2), rt.alloc(N * K * 2), rt.alloc(M * N * 4)
        rt.fill_uniform_bf16(xa.gpu_addr(), M * K, 42 + M + 1000 * s)
        # rank r owns rows [r*N, (r+1)*N) of WT[N_total, K]: the same stream, offset by its first element
        rt.fill_uniform_bf16(xb.gpu_addr(), N * K, 137 + N_total + 1000 * s, rank * N * K if sharded else 0)
        sets.append((xa, xb, y))
    cfg = t0.auto_select(M, K, N)
    tile_n = args.tile_n or cfg.tile_n
    split_k = cfg.split()
    pair = 1 if (cfg.wgp_mode and cfg.tile_m == 256 and not args.tile_n) else 2
    nn = args.layout == "nn"
    if nn and sharded:
        print("--layout nn is for the single-GPU workloads (a column slice of B[K,N] is strided)", file=sys.stderr)
        sys.exit(2)
    gemm_kw = dict(tile_n=tile_n, split_k=split_k, swap_grid=bool(cfg.swap_grid), pair_cta=pair, transpose=t0.NN if nn else t0.NT)
    step_args = [rt.gemm_args(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), M, N, K, **gemm_kw) for (xa, xb, y) in sets]

    def step(i):
        rt.gemm_batch([step_args[i % n_sets]])

    def barrier():
        rt.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        rt.synchronize()

    for i in range(warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches_before = rt.launch_count()
    timed = [step_args[i % n_sets] for i in range(steps)]
    rt.timer_start()
    rt.gemm_batch(timed)          # the K steps are submitted back to back from native code, then one wait
    ms = rt.timer_stop()
    barrier()
    clocks = sampler.stop()
    launches = rt.launch_count() - launches_before
    kernel_mhz, _ = rt.last_kernel_clock()
    clocks["sm_mhz_in_kernel"] = round(kernel_mhz)   # cycle counter / nanosecond timer inside the last timed kernel
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    flops_per_step = 2.0 * M * N_total * K
    value = flops_per_step * steps / (ms_max * 1e-3) / 1e12

    # optional: the gathered C.  Every rank's GEMM stores straight into slot `rank` of C_g[g][M][N/g]; one in-place
    # all-gather over NVLink completes it.  NCCL is issued on the runtime's own stream, so the device timer covers both.
    gather = None
    if (args.gather or (default_run and not args.no_gather)) and sharded and world > 1:
        c_g = torch.empty((world, M, N), dtype=torch.float32, device="cuda")
        ext = torch.cuda.ExternalStream(rt.stream())
        xa, xb, _ = sets[0]
        slot_ptr = c_g.data_ptr() + rank * M * N * 4
        g_args = [rt.gemm_args(xa.gpu_addr(), xb.gpu_addr(), slot_ptr, M, N, K, **gemm_kw)]

        def gather_step():
            rt.gemm_batch(g_args)
            with torch.cuda.stream(ext):
                dist.all_gather_into_tensor(c_g.view(-1), c_g[rank].reshape(-1))

        for _ in range(warmup):
            gather_step()
        barrier()
        rt.timer_start()
        for _ in range(steps):
            gather_step()
        g_ms = rt.timer_stop()
        barrier()
        tg = torch.tensor([g_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        g_ms = float(tg.item())
        # every rank must now hold every block: compare a sample of a remote block with the owner's copy
        probe = c_g[(rank + 1) % world, 0, :8].clone()
        owner = [torch.empty_like(probe) for _ in range(world)]
        dist.all_gather(owner, c_g[rank, 0, :8].clone())
        ok = bool(torch.equal(probe, owner[(rank + 1) % world]))
        gather = {"ms_per_step": g_ms / steps, "value": 2.0 * M * N_total * K * steps / (g_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                  "gathered_bytes_per_rank": M * N * 4 * (world - 1), "layout": "C_g[g][M][N/g]", "remote_block_matches": ok,
                  "call": "t0_gemm_launch into slot `rank`, then one in-place NCCL all-gather on the same stream"}

        # The same result from ONE kernel per GPU: the GEMM's epilogue stores every block into slot `rank` of all the
        # ranks' buffers (its own and, over NVLink, the others' mapped through CUDA IPC).  No collective call at all.
        c_buf = rt.alloc(world * M * N * 4)
        handles = [None] * world
        mapped, why = {}, None
        try:
            mine = c_buf.ipc_export()
        except Exception as exc:                    # every rank goes on to the agreement below
            mine, why = None, str(exc)
        dist.all_gather_object(handles, mine)
        if all(h is not None for h in handles):
            try:
                mapped = {d: rt.ipc_open(handles[d]) for d in range(world) if d != rank}
            except Exception as exc:
                why = str(exc)
        agree = torch.tensor([0.0 if why or len(mapped) != world - 1 else 1.0], dtype=torch.float64, device="cuda")
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if agree.item() != 1.0:
            # some rank cannot map its peers' memory (no peer access between these GPUs, or no IPC in this container)
            for ptr in mapped.values():
                rt.ipc_close(ptr)
            c_buf.free()
            gather["fused"] = {"unavailable": why or "another rank could not map the peers' buffers"}
            mapped = None
    if gather is not None and "fused" not in gather:
        slot = rank * M * N * 4
        f_args = rt.gemm_args(xa.gpu_addr(), xb.gpu_addr(), c_buf.gpu_addr() + slot, M, N, K, **gemm_kw)
        peers = [mapped[d] + slot for d in sorted(mapped)]
        for _ in range(warmup):
            rt.gemm_gather(f_args, peers)
        barrier()
        rt.timer_start()
        for _ in range(steps):
            rt.gemm_gather(f_args, peers)
        f_ms = rt.timer_stop()
        barrier()                                   # every rank's stores have landed before anyone reads
        tf_ = torch.tensor([f_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(tf_, op=dist.ReduceOp.MAX)
        f_ms = float(tf_.item())
        # every slot of this rank's buffer against the NCCL-gathered result, three rows each, bit for bit
        same = True
        for d in range(world):
            for r_ in (0, M // 2 + 1, M - 1):
                got = c_buf.read_bytes((d * M + r_) * N * 4, N * 4, np.float32)
                same = same and bool(np.array_equal(got, c_g[d, r_].cpu().numpy()))
        ts = torch.tensor([1.0 if same else 0.0], dtype=torch.float64, device="cuda")
        dist.all_reduce(ts, op=dist.ReduceOp.MIN)
        gather["fused"] = {"ms_per_step": f_ms / steps, "value": 2.0 * M * N_total * K * steps / (f_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                           "nvlink_bytes_out_per_rank": M * N * 4 * (world - 1), "equals_nccl_gather_on_every_rank": bool(ts.item() == 1.0),
                           "call": "t0_gemm_launch_gather: the epilogue's TMA stores write each block to every rank's buffer (peer memory over NVLink)"}
        barrier()
        for ptr in mapped.values():
            rt.ipc_close(ptr)
        barrier()
        c_buf.free()
        del c_g

    # parity spot check on every rank of its own block (the full parity suite is tests/ -m gpu)
    import oracle
    oracle.build()
    xa, xb, y = sets[(steps - 1) % n_sets]
    s_idx = (steps - 1) % n_sets
    rows = [0, M // 2 + 1, M - 1]
    b_host = oracle.fill_uniform_bf16(N * K, 137 + N_total + 1000 * s_idx, rank * N * K if sharded else 0)
    worst = 0.0
    for r in rows:
        a_row = oracle.fill_uniform_bf16(K, 42 + M + 1000 * s_idx, r * K)
        ref = oracle.gemm_nn(a_row, b_host, 1, K, N) if nn else oracle.gemm_nt(a_row, b_host, 1, K, N)
        got = y.read_bytes(r * N * 4, N * 4, np.float32)
        worst = max(worst, float(np.abs(ref[0] - got).max()))
    del b_host
    tw = torch.tensor([worst], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(tw, op=dist.ReduceOp.MAX)
    parity = {"sampled_rows": rows, "ranks_checked": world, "max_abs_err": float(tw.item()), "tol": 5e-3 * (K / 256) ** 0.5}
    if parity["max_abs_err"] > parity["tol"]:
        if rank == 0:
            print(json.dumps({"error": "parity check failed", "parity": parity}), flush=True)
        sys.exit(1)

    # ---- end to end through the C ABI with pinned host buffers (copies inside the timed region)
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(1, min(steps, 20 if not sharded else 3))
        xa, xb, y = sets[0]
        C = __import__("ctypes")

        def timed_region(fn):
            barrier()
            t_start = time.perf_counter()
            fn()
            barrier()
            td = torch.tensor([time.perf_counter() - t_start], dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(td, op=dist.ReduceOp.MAX)
            return float(td.item())

        b_host_t = torch.empty(N * K, dtype=torch.int16).pin_memory()
        y_host = torch.empty(M * N, dtype=torch.float32).pin_memory()
        b_host_t.numpy()[:] = xb.read(N * K * 2, np.int16)
        b_np, y_np = b_host_t.numpy(), y_host.numpy()
        if not sharded or world == 1:
            a_host = torch.empty(M * K, dtype=torch.int16).pin_memory()
            a_host.numpy()[:] = xa.read(M * K * 2, np.int16)
            a_np = a_host.numpy()

            def e2e_step():
                xa.write(a_np)
                xb.write(b_np)
                rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), M, N, K, **gemm_kw)
                t0._check(t0.lib().t0_rt_read_f32(rt._h, y._h, M * N, y_np.ctypes.data_as(C.c_void_p)))

            # (1) one problem after the other, as the reference's host-facing calls do: write, write, launch, blocking read
            e2e_step()
            dt_serial = timed_region(lambda: [e2e_step() for _ in range(e2e_steps)])
            # (2) the same steps as one array of host-operand problems: every step still uploads its operands and downloads
            # its product, but step i+1 crosses the link while step i is computed and read back
            host_args = [t0.GpuRuntime.gemm_args(a_np.ctypes.data, b_np.ctypes.data, y_np.ctypes.data, M, N, K, **gemm_kw)
                         for _ in range(e2e_steps)]
            rt.gemm_host_batch(host_args[:2])
            dt = timed_region(lambda: rt.gemm_host_batch(host_args))
            got_row = y_np.reshape(M, N)[M - 1].copy()
            dev_row = y.read_bytes((M - 1) * N * 4, N * 4, np.float32)
            if not np.array_equal(got_row, dev_row):
                print(json.dumps({"error": "host-operand GEMM differs from the device-resident result"}), flush=True)
                sys.exit(1)
            e2e = {"value": flops_per_step * e2e_steps / dt / 1e12, "unit": "TFLOP/s",
                   "h2d_bytes_per_step": M * K * 2 + N * K * 2, "d2h_bytes_per_step": M * N * 4, "steps": e2e_steps,
                   "call": "t0_gemm_launch_host_batch (uploads, kernels and downloads of consecutive steps overlap)",
                   "serial_value": flops_per_step * e2e_steps / dt_serial / 1e12,
                   "serial_call": "t0_buf_write x2, t0_gemm_launch, t0_rt_read_f32 per step"}
        else:
            # Sharded: A is replicated on the devices but crosses the host link ONCE: rank r uploads rows
            # [r M/g, (r+1) M/g) into its copy and one in-place all-gather over NVLink (on the runtime's stream) completes
            # every copy; then each rank uploads its block of WT, multiplies, and downloads its block of C.
            rows_per = M // world
            a_slice = torch.empty(rows_per * K, dtype=torch.int16).pin_memory()
            a_slice.numpy()[:] = xa.read_bytes(rank * rows_per * K * 2, rows_per * K * 2, np.int16)
            a_np = a_slice.numpy()
            a_dev = device_alias(xa.gpu_addr(), M * K, np.int16).view(torch.bfloat16)      # (NCCL moves bf16, not int16)
            ext = torch.cuda.ExternalStream(rt.stream())
            ref_row = y.read_bytes((M - 1) * N * 4, N * 4, np.float32)

            def e2e_step():
                xa.write_bytes(rank * rows_per * K * 2, a_np)
                with torch.cuda.stream(ext):
                    dist.all_gather_into_tensor(a_dev, a_dev[rank * rows_per * K:(rank + 1) * rows_per * K])
                xb.write(b_np)
                rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), M, N, K, **gemm_kw)
                t0._check(t0.lib().t0_rt_read_f32(rt._h, y._h, M * N, y_np.ctypes.data_as(C.c_void_p)))

            rt.fill_uniform_bf16(xa.gpu_addr(), M * K, 999)          # scribble: the exchange must rebuild A from the uploaded slices
            rt.synchronize()
            e2e_step()
            if not np.array_equal(y_np.reshape(M, N)[M - 1], ref_row):
                print(json.dumps({"error": "sharded host-operand GEMM differs from the device-resident result", "rank": rank}), flush=True)
                sys.exit(1)
            dt_serial = timed_region(lambda: [e2e_step() for _ in range(e2e_steps)])

            # The same steps with the download of step i under the uploads of step i+1: the C blocks live in buffers of a second
            # runtime (its own stream), a worker thread reads them back while this thread goes on with the next step's uploads.
            from concurrent.futures import ThreadPoolExecutor
            rt2 = t0.GpuRuntime(local_rank)
            ys2 = [rt2.alloc(M * N * 4) for _ in range(2)]
            y_hosts = [y_host, torch.empty(M * N, dtype=torch.float32).pin_memory()]
            y_nps = [h.numpy() for h in y_hosts]
            pool = ThreadPoolExecutor(max_workers=1)
            p_steps = 2 * e2e_steps

            def pipelined(n_steps):
                pending = [None, None]
                for i in range(n_steps):
                    xa.write_bytes(rank * rows_per * K * 2, a_np)
                    with torch.cuda.stream(ext):
                        dist.all_gather_into_tensor(a_dev, a_dev[rank * rows_per * K:(rank + 1) * rows_per * K])
                    xb.write(b_np)
                    if pending[i % 2] is not None:
                        pending[i % 2].result()               # the block this step overwrites has been read back
                    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), ys2[i % 2].gpu_addr(), M, N, K, **gemm_kw)
                    rt.synchronize()
                    pending[i % 2] = pool.submit(lambda j=i % 2: t0._check(t0.lib().t0_buf_read(ys2[j]._h, y_nps[j].ctypes.data_as(C.c_void_p), M * N * 4)))
                for f in pending:
                    if f is not None:
                        f.result()

            pipelined(2)                                     # untimed: the worker thread's and the second stream's first use
            y_nps[0][:] = 0.0
            y_nps[1][:] = 0.0
            dt = timed_region(lambda: pipelined(p_steps))
            pool.shutdown()
            for j in range(2):
                if not np.array_equal(y_nps[j].reshape(M, N)[M - 1], ref_row):
                    print(json.dumps({"error": "pipelined sharded host-operand GEMM differs from the device-resident result", "rank": rank}), flush=True)
                    sys.exit(1)
            for b in ys2:
                b.free()
            rt2.close()
            e2e = {"value": flops_per_step * p_steps / dt / 1e12, "unit": "TFLOP/s",
                   "h2d_bytes_per_step": M * K * 2 + N_total * K * 2, "d2h_bytes_per_step": M * N_total * 4, "steps": p_steps,
                   "call": "per rank: t0_buf_write_bytes (its 1/g of A), all-gather of A over NVLink, t0_buf_write (its block of WT), "
                           "t0_gemm_launch, t0_buf_read (its block of C) from a second runtime's stream, so that the read-back of step i "
                           "runs under the uploads of step i+1",
                   "serial_value": flops_per_step * e2e_steps / dt_serial / 1e12,
                   "serial_call": "the same calls one blocking call after the other (t0_rt_read_f32 for the block of C)",
                   "nvlink_bytes_per_rank_per_step": (world - 1) * rows_per * K * 2}

    # ---- sharded runs: the same 16384^3 on ONE GPU (rank 0), the denominator of the scaling claim
    single = None
    if sharded and world > 1:
        if rank == 0:
            for (xa_, xb_, y_) in sets:
                xb_.free()
                y_.free()
            xa = sets[0][0]
            rt.fill_uniform_bf16(xa.gpu_addr(), M * K, 42 + M)
            xb1, y1 = rt.alloc(N_total * K * 2), rt.alloc(M * N_total * 4)
            rt.fill_uniform_bf16(xb1.gpu_addr(), N_total * K, 137 + N_total)
            cfg1 = t0.auto_select(M, K, N_total)
            kw1 = dict(tile_n=cfg1.tile_n, split_k=cfg1.split(), swap_grid=bool(cfg1.swap_grid),
                       pair_cta=1 if (cfg1.wgp_mode and cfg1.tile_m == 256) else 2)
            one = [rt.gemm_args(xa.gpu_addr(), xb1.gpu_addr(), y1.gpu_addr(), M, N_total, K, **kw1)]
            s1 = max(3, steps // 4)
            rt.gemm_batch(one * 2)
            rt.synchronize()
            rt.timer_start()
            rt.gemm_batch(one * s1)
            ms1 = rt.timer_stop() / s1
            # the sharded ranks' blocks are column slices of this product: the spot check above covers the arithmetic
            single = {"ms_per_step": ms1, "value": flops_per_step / (ms1 * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": s1,
                      "what": f"the whole {M}x{N_total}x{K} GEMM on rank 0's GPU alone, device-timed the same way"}
            sets = []
        barrier()

    if rank == 0:
        peaks = measured_peaks()
        peak, peak_src = tensor_peak(peaks, ms_max)
        per_launch_ms = ms_max / steps
        achieved = 2.0 * M * N * K / (per_launch_ms * 1e-3) / 1e12     # this rank's kernel: algorithmic FLOPs / event time
        line = {"metric": "bf16_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": ms_max / steps, "higher_is_better": True,
                "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": name, "m": M, "n": N_total, "k": K, "layout": "NN" if nn else "NT", "out": "f32",
                           "kernel": (cfg if not args.tile_n else cfg.copy(tile_m=128, tile_n=tile_n, wgp_mode=0)).copy(transpose=t0.NN if nn else t0.NT).name(),
                           "per_rank_n": N, "input_sets": n_sets,
                           "l2": f"{n_sets} resident operand sets of {set_bytes >> 20} MiB rotate (> 126 MB L2)" if n_sets > 1
                                 else f"operands {set_bytes >> 20} MiB per rank (> 126 MB L2)",
                           "pct_of_nominal_dense_peak": round(100.0 * value / world / 2250.0, 1)},
                "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                             "traffic": ncu_traffic(name), "peak_source": peak_src},
                "clocks": clocks, "gpu_launches": int(launches), "parity": parity}
        if e2e:
            line["e2e"] = e2e
        if gather:
            line["gather"] = gather
        if single:
            line["single_gpu"] = single
            line["speedup_vs_1gpu"] = single["ms_per_step"] / (ms_max / steps)
        if not args.no_cpu:
            rows = max(32, min(M, int(M * (2.0 * 4096 ** 3) / (2.0 * M * N_total * K))))
            tf, sec, cores = cpu_baseline(oracle, M, N_total, K, rows)
            what = f"the full {M}x{N_total}x{K} GEMM" if rows == M else f"rows 0..{rows - 1} of {M} (extrapolate linearly)"
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": f"{what}, best of 3, {sec:.2f} s per pass"}
        if default_run and world == 1 and not args.no_secondary:
            # the other clauses of the metric, as short device-resident runs (each parity-checked), so that one line carries them all
            for (xa_, xb_, y_) in sets:
                xa_.free()
                xb_.free()
                y_.free()
            sec_lines = []
            for sname in SECONDARY:
                if WORKLOADS[sname].get("hbm"):
                    ln = run_hbm_workload(args, sname, rt=rt, brief=True)
                    sec_lines.append({"workload": sname, "metric": ln["metric"], "value": ln["value"], "unit": ln["unit"], "ms_per_step": ln["ms_per_step"],
                                      "steps": ln["steps"], "kernel": ln["config"]["kernel"], "bytes": ln["config"]["bytes"], "tflops": ln["config"]["tflops"],
                                      "roofline": {k: ln["roofline"][k] for k in ("bound", "frac", "peak", "traffic", "tensor_frac") if k in ln["roofline"]},
                                      "gpu_launches": ln["gpu_launches"], "parity": ln["parity"]})
                    if "one_problem_per_launch" in ln:
                        sec_lines[-1]["one_problem_per_launch"] = ln["one_problem_per_launch"]
                else:
                    sec_lines.append(run_square_brief(t0, rt, sname))
            for sname in AUX_WORKLOADS:
                ln = run_aux_workload(args, sname, rt=rt, brief=True)
                sec_lines.append({"workload": sname, "metric": ln["metric"], "value": ln["value"], "unit": ln["unit"], "ms_per_step": ln["ms_per_step"],
                                  "steps": ln["steps"], "kernel": ln["config"]["kernel"],
                                  "roofline": {k: ln["roofline"][k] for k in ("bound", "frac", "peak", "traffic") if k in ln["roofline"]},
                                  "gpu_launches": ln["gpu_launches"], "parity": ln["parity"]})
            line["secondary"] = sec_lines
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    rt.close()


if __name__ == "__main__":
    main()

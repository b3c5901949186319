#!/usr/bin/env python
"""Benchmark of the forward layer-op path on B200.

Workload (N = 1 and per rank for N > 1): the stand-alone Linear + bias + GELU stack — three layers
K = N = 4096 over M = 65536 fp32 rows per GPU (rows sharded across GPUs, weak scaling), synthetic
seeded data.  One step = one forward of the whole stack over the rank's rows.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows M]

`value`   : rows/s with inputs resident in HBM (device pointers through the graph C ABI).
`e2e`     : rows/s through the host-pointer C ABI call, pinned host buffers, H2D + D2H inside.
`roofline`: the tcgen05 GEMM kernel, algorithmic flops / live CUDA-event duration of its launches.
`cpu_baseline` / `--impl reference`: the reference's own CPU code (oracle/_ref) on the host cores,
on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from mimir_framework_b200 import configs  # noqa: E402

METRIC = "fwd samples/sec"
UNIT = "samples/s (1 sample = 1 row through Linear+bias+GELU x3, K=N=4096)"
K = configs.LINEAR_STACK_K


# DRAM bytes (read + write) of one GEMM launch of this workload at M = 8192 rows, from the ncu capture
# summarised in profiles/gemm_tn_bf16split_linear_stack.md
NCU_TRAFFIC_BYTES_AT_8192_ROWS = 627.6e6


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(bf16_sustained=d.get("bf16_tflops_sustained"), bf16_burst=d.get("bf16_tflops"), hbm=d.get("hbm_gbs"),
                    source="measured")
    return dict(bf16_sustained=1400.0, bf16_burst=1590.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock, power and throttle reasons while the timed region runs: NVML read-only queries every 5 ms
    from a thread (the timed region of the default run lasts ~150 ms), nvidia-smi at its fastest cadence as fallback."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []   # (time, sm MHz, max MHz, W, [reason names])
        self.proc = None
        self.stop_flag = False
        self.t = None

    def _nvml_loop(self, nv, h, sm_max):
        masks = [("hw_slowdown", nv.nvmlClocksThrottleReasonHwSlowdown), ("hw_thermal_slowdown", nv.nvmlClocksThrottleReasonHwThermalSlowdown),
                 ("sw_thermal_slowdown", nv.nvmlClocksThrottleReasonSwThermalSlowdown), ("sw_power_cap", nv.nvmlClocksThrottleReasonSwPowerCap)]
        # every other reason the driver reports is recorded too, so that a clock below maximum is never left unexplained
        for name, attr in (("gpu_idle", "nvmlClocksThrottleReasonGpuIdle"), ("applications_clocks_setting", "nvmlClocksThrottleReasonApplicationsClocksSetting"),
                           ("sync_boost", "nvmlClocksThrottleReasonSyncBoost"), ("hw_power_brake_slowdown", "nvmlClocksThrottleReasonHwPowerBrakeSlowdown"),
                           ("display_clock_setting", "nvmlClocksThrottleReasonDisplayClockSetting")):
            if hasattr(nv, attr):
                masks.append((name, getattr(nv, attr)))
        known = 0
        for _, m in masks:
            known |= m
        while not self.stop_flag:
            try:
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                w = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                names = [n for n, m in masks if bits & m]
                if bits & ~known:
                    names.append("other_0x%x" % (bits & ~known))
                self.rows.append((time.time(), float(sm), float(sm_max), w, names))
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            # the physical index behind CUDA_VISIBLE_DEVICES, by UUID when torch can tell
            h = None
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
                h = nv.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                h = nv.nvmlDeviceGetHandleByIndex(self.index)
            sm_max = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            self.t = threading.Thread(target=self._nvml_loop, args=(nv, h, sm_max), daemon=True)
            self.t.start()
            return
        except Exception:
            self.t = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            c = [x.strip() for x in line.split(",")]
            if len(c) >= 7:
                try:
                    self.rows.append((time.time(), float(c[0]), float(c[1]), float(c[2]),
                                      [n for i, n in enumerate(names) if c[3 + i].lower().startswith("active")]))
                except ValueError:
                    pass

    def stop(self, t0: float, t1: float):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        self.stop_flag = True
        if self.t is not None and not self.proc:
            self.t.join(timeout=1)
        rows = [r for r in self.rows if t0 <= r[0] <= t1] or [r for r in self.rows if t0 <= r[0] <= t1 + 0.2] or self.rows
        if not rows:
            return None
        reasons = sorted({n for r in rows for n in r[4]})
        return {"sm_mhz": statistics.median(r[1] for r in rows), "sm_max_mhz": rows[0][2], "reasons": reasons, "samples": len(rows),
                "power_w_max": max(r[3] for r in rows), "source": "nvml" if not self.proc else "nvidia-smi"}


def cpu_reference_rate(sample_rows: int, repeats: int, warmup: int):
    """Times the reference's own CPU forward (compiled from its sources) on `sample_rows` rows."""
    from oracle import ref

    cores = os.cpu_count() or 1
    used = ref.set_threads(cores)
    descs = configs.linear_gelu_stack(sample_rows)
    weights = configs.linear_gelu_stack_weights()
    m = ref.RefModel(descs)
    for i, w in enumerate(weights):
        if w is not None:
            m.set_weights(i, w)
    x = configs.linear_gelu_stack_input(sample_rows).ravel()
    times = []
    for i in range(warmup + repeats):
        _, secs = m.forward({"x": x}, out_cap=sample_rows * K, return_seconds=True)
        if i >= warmup:
            times.append(secs)
    m.close()
    return sample_rows / statistics.median(times), used, times


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref

    if not ref.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libmimir_ref.so was not built (reference sources not mounted)"}))
        return
    rows = args.ref_rows
    rate, cores, times = cpu_reference_rate(rows, args.steps, min(args.warmup, 1))
    ms = 1e3 * statistics.median(times)
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"Linear+bias+GELU x3, K=N={K}, M={args.rows} fp32 rows per GPU", "rows_per_gpu": args.rows,
                   "sample": f"each step times {rows} of the rows on the host cores (rows are independent)"},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cores, "kind": "reference",
                         "sample": f"{rows} rows per step, median of {args.steps} steps, reference CPU code, OpenMP threads = {cores}"},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_ours(args):
    import torch
    import torch.distributed as dist

    from mimir_framework_b200 import runtime as rt

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    rt.init(local_rank, 0)  # raises if the CUDA library is missing or there is no sm_100 device

    M = args.rows
    descs = configs.linear_gelu_stack(M)
    weights = configs.linear_gelu_stack_weights()
    model = rt.GraphModel(descs)
    for i, w in enumerate(weights):
        model.upload_weights(i, w)
    model.plan({"x": (M * K, False)}, batch=1)

    # each rank owns its own M rows (weak scaling); disjoint seeded slices
    x_host = torch.from_numpy(configs.linear_gelu_stack_input(M, row_offset=rank * M)).pin_memory()
    y_host = torch.empty((M, K), dtype=torch.float32).pin_memory()
    # the end-to-end arm uses the same graph cut into micro-batches (rows are independent), so that
    # copy-in, compute and copy-out overlap: model_set_pipeline
    chunks = args.pipeline if M % args.pipeline == 0 else 1
    model_e2e = rt.GraphModel(configs.linear_gelu_stack(M // chunks), pipeline=chunks)
    for i, w in enumerate(weights):
        model_e2e.upload_weights(i, w)
    model_e2e.plan({"x": ((M // chunks) * K, False)}, batch=chunks)
    spec_host = {"x": (x_host.data_ptr(), (M // chunks) * K, False)}
    x_dev = x_host.cuda(non_blocking=False)
    y_dev = torch.empty((M, K), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    spec_dev = {"x": (x_dev.data_ptr(), M * K, False)}

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput --------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        model.forward_device(spec_dev, 1, y_dev.data_ptr(), M * K, stream)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    launches0 = rt.stats()["kernels_launched"]
    rt.profile_gemm(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_wall0 = time.time()
    e0.record()
    for _ in range(args.steps):
        model.forward_device(spec_dev, 1, y_dev.data_ptr(), M * K, stream)
    e1.record()
    barrier()
    t_wall1 = time.time()
    rt.profile_gemm(False)
    gemm_ms, gemm_launches = rt.profile_read()
    rt.check(rt.lib().mimir_b200_check_device(None))
    launches = rt.stats()["kernels_launched"] - launches0
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    value = world * M / (ms_per_step * 1e-3)

    # ---- end to end through the host-pointer call ------------------------------------------------
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    for _ in range(2):
        model_e2e.forward_host_ptrs(spec_host, chunks, y_host.data_ptr(), M * K)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        model_e2e.forward_host_ptrs(spec_host, chunks, y_host.data_ptr(), M * K)  # synchronous: H2D, layers, D2H
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = world * M * e2e_steps / e2e_s
    checksum = float(y_host[:64].double().abs().sum())

    # ---- roofline of the dominant kernel (the GEMM) ----------------------------------------------
    peaks = measured_peaks()
    per_launch_flops = 2.0 * M * K * K
    gemm_avg_ms = gemm_ms / max(gemm_launches, 1)
    achieved = per_launch_flops / (gemm_avg_ms * 1e-3) / 1e12 if gemm_launches else None
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_sustained"], "unit": "TFLOP/s",
        "frac": (achieved / peaks["bf16_sustained"]) if achieved else None,
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch at M = 8192 rows (510.7 MB + 116.9 MB, ncu --set full),
        # scaled by the rows of this launch: the traffic is per row tile, so it grows in proportion
        "traffic": NCU_TRAFFIC_BYTES_AT_8192_ROWS * M / 8192, "traffic_unit": "bytes per launch (ncu at M=8192, scaled by rows)",
        "kernel": "gemm_tn_bf16split_kernel", "launches_timed": gemm_launches, "avg_launch_ms": gemm_avg_ms,
        "peak_source": f"{peaks['source']} (cuBLAS bf16 8192^3 sustained)",
        "issued_tflops": (3 * achieved) if achieved else None,
        "note": "achieved counts algorithmic flops 2*M*N*K; the kernel issues 3 bf16 MMAs per product term (hi*hi + lo*hi + hi*lo)",
    }

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            try:
                from oracle import ref
                if ref.available():
                    rate, cores, times = cpu_reference_rate(args.cpu_rows, 3, 1)
                    cpu = {"value": rate, "unit": UNIT, "cores": cores, "kind": "reference",
                           "sample": f"{args.cpu_rows} of {M} rows, median of 3 runs ({sum(times):.1f} s of CPU work), reference CPU code, OpenMP threads = {cores}"}
            except Exception as ex:  # the baseline is a reported extra, never a reason to lose the line
                cpu = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference", "sample": f"failed: {ex}"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16x2 split (fp32 in/out, fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": f"Linear+bias+GELU x3, K=N={K}, M={M} fp32 rows per GPU", "rows_per_gpu": M,
                       "l2_policy": "inputs larger than L2 (1 GiB activations per layer), no flush", "precision": "BF16X2",
                       "parallelism": f"replica per GPU x{world}, rows sharded, no collective"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * K * 4,
                    "steps": e2e_steps, "micro_batches": chunks, "checksum_first_rows": checksum},
            "gpu_launches": int(launches),
            "tflops_algorithmic": configs.linear_gelu_stack_flops(M) / (ms_per_step * 1e-3) / 1e12,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        print(json.dumps(line))
    model.close()
    model_e2e.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=65536, help="rows per GPU")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--pipeline", type=int, default=16, help="micro-batches of the end-to-end (host pointer) arm")
    ap.add_argument("--cpu-rows", type=int, default=2048, help="rows of the CPU-baseline sample")
    ap.add_argument("--ref-rows", type=int, default=1024, help="rows per step of --impl reference")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

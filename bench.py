#!/usr/bin/env python
"""Benchmark of the forward layer-op path on B200.

Headline workload (N = 1 and per rank for N > 1): the stand-alone Linear + bias + GELU stack — three layers
K = N = 4096 over M = 65536 fp32 rows per GPU (rows sharded across GPUs, weak scaling), synthetic
seeded data.  One step = one forward of the whole stack over the rank's rows.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows M] [--headline-only]

`value`   : rows/s with inputs resident in HBM (device pointers through the graph C ABI).
`e2e`     : rows/s through the host-pointer C ABI call, pinned host buffers, H2D + D2H inside; with
            `frac_of_copy_ceiling` = e2e / what plain pinned copies of the same bytes reach on all N GPUs at once.
`roofline`: the tcgen05 GEMM kernel, algorithmic flops / live CUDA-event duration of its launches.
`cpu_baseline` / `--impl reference`: the reference's own CPU code (oracle/_ref) on the host cores,
on a bounded sample of the same workload.
`configs` : the other four named configurations (registry transformer encoder, GPT decoder prefill, conv vision
            stack, UNet mid+up) at their stated sizes and per-GPU batches, each with device-resident and end-to-end
            samples/s (summed over ranks, max time over ranks), the share of the step spent in the GEMM kernel, a
            roofline fraction against the measured peaks, and at N = 1 the reference CPU rate and the parity
            counts of sample 0 against it.
`norms`   : the HBM-bound kernels (LayerNorm, RMSNorm, GroupNorm + SiLU, Softmax) as GB/s of algorithmic bytes
            over the measured copy bandwidth (rank 0's GPU).
`single_process` (N > 1): rank 0 alone drives all N GPUs through the replica entry points (one host thread per
            device) and gathers every slice into ONE pinned host buffer.
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

from mimir_framework_b200 import configs, sharding  # noqa: E402

METRIC = "fwd samples/sec"
UNIT = "samples/s (1 sample = 1 row through Linear+bias+GELU x3, K=N=4096)"
K = configs.LINEAR_STACK_K


# DRAM bytes (read + write) of one GEMM launch of this workload at M = 8192 rows, from the ncu capture
# summarised in profiles/gemm_tn_bf16split_linear_stack.md
NCU_TRAFFIC_BYTES_AT_8192_ROWS = 656.9e6
NCU_WEIGHT_BYTES = 2 * 2 * 4096 * 4096  # the hi and lo weight planes, read once per launch whatever the row count


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


def hbm_frac(nbytes, ms, peaks):
    gbs = nbytes / (ms * 1e-3) / 1e9
    return gbs, gbs / peaks["hbm"]


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
    rate, cores, times = cpu_reference_rate(rows, args.steps, args.warmup)
    ms = 1e3 * statistics.median(times)
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"Linear+bias+GELU x3, K=N={K}, M={args.rows} fp32 rows per GPU", "rows_per_gpu": args.rows,
                   "sample": f"each step times {rows} of the rows on the host cores (rows are independent)"},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cores, "kind": "reference",
                         "sample": f"{rows} rows per step, median of {args.steps} steps, reference CPU code, OpenMP threads = {cores}"},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- the other configurations ---------------------------------------------------------------------------------
class Harness:
    """Process group, barriers and reductions shared by every measurement."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.host_group = None
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.host_group = dist.new_group(backend="gloo")  # barriers that keep no kernel spinning on the GPUs
        torch.cuda.set_device(self.local_rank)
        self.stream = torch.cuda.current_stream().cuda_stream

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def host_barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier(group=self.host_group)

    def max_over_ranks(self, v: float) -> float:
        return sharding.reduce_max(v, device="cuda")

    def time_steps(self, fn, steps, warmup=3):
        """Device time of `steps` calls (CUDA events on the launching stream), barrier on both sides, max over ranks."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1)) / steps

    def wall_steps(self, fn, steps, warmup=2):
        """Wall time of `steps` synchronous calls (host-pointer entry points), max over ranks."""
        for _ in range(warmup):
            fn()
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        self.torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        return 1e3 * self.max_over_ranks(dt) / steps


def _parity(got, want):
    err = np.abs(got.ravel() - want.ravel())
    return {"max_abs": float(err.max()), "outside_tolerance": int((err > 1e-4 + 1e-3 * np.abs(want.ravel())).sum()), "n": int(want.size),
            "gate": "|gpu - cpu| <= 1e-4 + 1e-3 |cpu|"}


def _cpu_sample(descs, weights, inputs, registry=None, cfg=None):
    """One sample through the compiled reference: (output, seconds, threads), or None when it is not there."""
    from oracle import ref

    if not ref.available():
        return None
    cores = ref.set_threads(os.cpu_count() or 1)
    ref.set_guard_limit(64 << 30)
    m = ref.RefModel(registry=registry, cfg_json=json.dumps(cfg)) if registry else ref.RefModel(descs)
    for i, w in enumerate(weights):
        if w is not None:
            m.set_weights(i, w)
    y, secs = m.forward(inputs, return_seconds=True)
    m.close()
    return y, secs, cores


def bench_graph_config(h: Harness, rt, peaks, name, descs, weights, inputs, batch, out_n, precision, flops_per_sample=None,
                       weight_stream_bytes=None, e2e="host", pipeline=1, steps=5, cpu=True, registry=None, registry_cfg=None,
                       one_mma_arm=False, gemm_flops_per_sample=None):
    """One configuration on this rank's GPU with its stated per-GPU batch.  `inputs`: name -> (array [batch, per] or
    broadcast vector, broadcast flag).  e2e = "host": the host-pointer forward (pipelined when `pipeline` > 1) from and
    to pinned buffers; "argmax": pinned ids -> device -> forward -> per-position argmax on the device -> ids to pinned
    memory (the decoder's harness step: 4 GB of logits never cross PCIe)."""
    torch = h.torch
    model = rt.GraphModel(descs, precision)
    for i, w in enumerate(weights):
        model.upload_weights(i, w)
    spec = {k: ((a.size if bc else a.size // batch), bc) for k, (a, bc) in inputs.items()}
    model.plan(spec, batch)
    dev = {k: torch.from_numpy(np.ascontiguousarray(a)).cuda() for k, (a, bc) in inputs.items()}
    d_out = torch.empty(batch * out_n, device="cuda")
    dspec = {k: (dev[k].data_ptr(), spec[k][0], spec[k][1]) for k in inputs}
    ms = h.time_steps(lambda: model.forward_device(dspec, batch, d_out.data_ptr(), d_out.numel(), h.stream), steps)
    # share of the step inside the GEMM kernel: two more forwards with every GEMM launch bracketed by events
    rt.profile_gemm(True)
    for _ in range(2):
        model.forward_device(dspec, batch, d_out.data_ptr(), d_out.numel(), h.stream)
    gemm_ms, gemm_n = rt.profile_read()
    rt.profile_gemm(False)
    rt.check(rt.lib().mimir_b200_check_device(None))
    got0 = d_out[:out_n].cpu().numpy()
    # ---- end to end ----
    host = {k: torch.from_numpy(np.ascontiguousarray(a)).pin_memory() for k, (a, bc) in inputs.items()}
    h2d = sum(int(t.numel()) * 4 for t in host.values())
    if e2e == "argmax":
        rows, V = batch * (out_n // registry_cfg["vocab"]), registry_cfg["vocab"]
        d_tok = torch.empty(rows, dtype=torch.int32, device="cuda")
        tok_host = torch.empty(rows, dtype=torch.int32).pin_memory()

        def step():
            for k in inputs:
                dev[k].copy_(host[k], non_blocking=True)
            model.forward_device(dspec, batch, d_out.data_ptr(), d_out.numel(), h.stream)
            rt.check(rt.lib().mimir_b200_argmax_rows_device(d_out.data_ptr(), d_tok.data_ptr(), rows, V, h.stream))
            tok_host.copy_(d_tok, non_blocking=True)
            torch.cuda.synchronize()
        e2e_ms = h.wall_steps(step, steps)
        d2h = rows * 4
        e2e_note = "pinned ids -> device, forward, per-position argmax on the device, token ids -> pinned host"
    else:
        out_host = torch.empty(batch * out_n).pin_memory()
        chunks = pipeline if batch % pipeline == 0 else 1
        m2 = model
        if chunks > 1:
            m2 = rt.GraphModel(descs, precision, pipeline=chunks)
            for i, w in enumerate(weights):
                m2.upload_weights(i, w)
            m2.plan(spec, batch)
        hspec = {k: (host[k].data_ptr(), spec[k][0], spec[k][1]) for k in inputs}
        e2e_ms = h.wall_steps(lambda: m2.forward_host_ptrs(hspec, batch, out_host.data_ptr(), out_host.numel()), steps)
        if m2 is not model:
            m2.close()
        d2h = batch * out_n * 4
        e2e_note = f"host-pointer forward from / to pinned buffers, {chunks} micro-batch(es)"
    rec = {"config": name, "batch_per_gpu": batch, "precision": ["BF16X2", "BF16W", "BF16"][precision], "steps": steps,
           "ms_per_step": ms, "samples_per_s": h.world * batch / (ms * 1e-3),
           "e2e": {"samples_per_s": h.world * batch / (e2e_ms * 1e-3), "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "how": e2e_note},
           "gemm_share_of_step": (gemm_ms / 2) / ms if gemm_n else 0.0, "gemm_launches_per_step": gemm_n // 2,
           "arena_bytes": model.arena_bytes}
    if flops_per_sample:
        tf = flops_per_sample * batch / (ms * 1e-3) / 1e12
        rec["roofline"] = {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_sustained"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_sustained"],
                           "note": "algorithmic flops of the contraction layers over the whole step (norms, layout and copies included in the time)",
                           "gemm_only_tflops": ((gemm_flops_per_sample or flops_per_sample) * batch / (gemm_ms / 2 * 1e-3) / 1e12) if gemm_n else None,
                           "gemm_only_note": "flops of the layers that run in the GEMM kernel over the time inside that kernel (CUDA events around every launch)"}
    if weight_stream_bytes:
        gbs, frac = hbm_frac(weight_stream_bytes, ms, peaks)
        rec["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": frac,
                           "note": "fp32 weights (embedding table excluded) read once per batch over the whole step"}
    if cpu and h.rank == 0 and h.world == 1:
        one = {k: (a if bc else a.reshape(batch, -1)[0]) for k, (a, bc) in inputs.items()}
        r = _cpu_sample(descs, weights, one, registry, registry_cfg if registry else None)
        if r is not None:
            want, secs, cores = r
            rec["cpu_reference"] = {"samples_per_s": 1.0 / secs, "s_per_sample": secs, "cores": cores, "kind": "reference",
                                    "sample": "sample 0 of the batch, one forward of the reference's CPU code"}
            rec["parity_sample0"] = _parity(got0, want)
    model.close()
    if one_mma_arm and flops_per_sample:
        # The same configuration with ONE 16-bit plane per operand (one MMA per product): outside the fp32 gate by
        # construction (its checker is the oracle with the same operand rounding, tests/test_gpu_precision_modes.py);
        # measured beside the strict arm so that the GEMM fraction of the tensor-core peak is on record for both.
        from mimir_framework_b200 import abi

        m1 = rt.GraphModel(descs, abi.PREC_BF16)
        for i, w in enumerate(weights):
            m1.upload_weights(i, w)
        m1.plan(spec, batch)
        ms1 = h.time_steps(lambda: m1.forward_device(dspec, batch, d_out.data_ptr(), d_out.numel(), h.stream), steps)
        rt.profile_gemm(True)
        for _ in range(2):
            m1.forward_device(dspec, batch, d_out.data_ptr(), d_out.numel(), h.stream)
        g1_ms, g1_n = rt.profile_read()
        rt.profile_gemm(False)
        rt.check(rt.lib().mimir_b200_check_device(None))
        got1 = d_out[:out_n].cpu().numpy()
        m1.close()
        mmas = {0: 3, 1: 2, 2: 1}[precision]
        strict_gemm_tf = rec["roofline"]["gemm_only_tflops"]
        one_gemm_tf = ((gemm_flops_per_sample or flops_per_sample) * batch / (g1_ms / 2 * 1e-3) / 1e12) if g1_n else None
        pk = peaks["bf16_sustained"]
        rec["gemm_fraction_of_peak"] = {
            "peak_tflops": pk, "strict": {"precision": rec["precision"], "mma_per_product": mmas, "algorithmic": strict_gemm_tf / pk if strict_gemm_tf else None,
                                          "issued": mmas * strict_gemm_tf / pk if strict_gemm_tf else None},
            "one_mma": {"precision": "BF16", "mma_per_product": 1, "algorithmic": one_gemm_tf / pk if one_gemm_tf else None}}
        rec["one_mma_arm"] = {"precision": "BF16", "ms_per_step": ms1, "samples_per_s": h.world * batch / (ms1 * 1e-3),
                              "gemm_share_of_step": (g1_ms / 2) / ms1 if g1_n else 0.0, "gemm_only_tflops": one_gemm_tf,
                              "step_tflops": flops_per_sample * batch / (ms1 * 1e-3) / 1e12,
                              "vs_strict_arm_sample0": _parity(got1, got0),
                              "note": "one 16-bit plane per operand; checked against the oracle with the same operand rounding, not against the fp32 gate"}
        if "parity_sample0" in rec:
            rec["one_mma_arm"]["vs_cpu_reference_sample0"] = _parity(got1, want)
    return rec


def bench_other_configs(h: Harness, rt, peaks, args):
    from mimir_framework_b200 import abi

    out = []
    seed0 = 1000 * h.rank  # every rank draws its own inputs; rank 0 keeps the configurations' stated seeds
    want = lambda tag: args.only in ("all", "configs", tag)  # noqa: E731
    cpu = not args.no_cpu_baseline
    if want("c1"):
        out.append(_bench_c1(h, rt, peaks, abi, seed0, cpu))
    if want("c3"):
        out.append(_bench_c3(h, rt, peaks, abi, seed0, cpu, args.decoder_batch, args.precision == "one-mma"))
    if want("c4"):
        out.append(_bench_c4(h, rt, peaks, abi, seed0, cpu, args.conv_batch))
    if want("c5"):
        out.append(_bench_c5(h, rt, peaks, abi, seed0, cpu, args.unet_batch, args.precision == "one-mma"))
    return out


def _bench_c1(h, rt, peaks, abi, seed0, cpu):
    # 1: registry transformer encoder, batch 8
    cfg = configs.TRANSFORMER_CFG
    descs = configs.transformer_encoder(**cfg)
    weights = configs.seeded_weights(descs, seed=1, std=0.02)
    ids = np.random.default_rng(seed0).integers(0, cfg["vocab_size"], (8, cfg["seq_len"])).astype(np.float32)
    r = np.random.default_rng(2)
    mag, mod = (r.standard_normal(cfg["d_model"]) * 0.02).astype(np.float32), (r.standard_normal(cfg["d_model"]) * 0.02).astype(np.float32)
    try:
        from oracle import ref
        if ref.available() and h.world == 1:
            m = ref.RefModel(registry="transformer", cfg_json=json.dumps(cfg))
            mag, mod = m.mag_mod()
            m.close()
    except Exception:
        pass
    wbytes = 4 * sum(int(d.params_count) for d in descs if d.type.decode() != "Embedding")
    return bench_graph_config(h, rt, peaks, "1 registry transformer encoder: 2 layers d256 h4 ffn1024 vocab8192 seq128, fp32", descs, weights,
                              {"x": (ids, False), "mag": (mag, True), "mod": (mod, True)}, 8, cfg["output_dim"], abi.PREC_BF16X2,
                              weight_stream_bytes=wbytes, steps=20, registry="transformer", registry_cfg=cfg, cpu=cpu)


def _bench_c3(h, rt, peaks, abi, seed0, cpu, batch, one_mma_only=False):
    # 3: GPT decoder prefill, batch 32
    cfg = configs.DECODER_CFG
    descs = configs.gpt_decoder(**cfg)
    weights = configs.seeded_weights(descs, seed=1, std=0.02, bf16=True)
    ids = np.random.default_rng(seed0).integers(0, cfg["vocab"], (batch, cfg["seq"])).astype(np.float32)
    return bench_graph_config(h, rt, peaks, "3 GPT decoder prefill: 12 layers d768 h12 ffn3072 vocab32000 seq1024, bf16-exact weights, whole-sample RMSNorm", descs,
                              weights, {"x": (ids, False)}, batch, cfg["seq"] * cfg["vocab"], abi.PREC_BF16 if one_mma_only else abi.PREC_BF16W,
                              flops_per_sample=configs.gpt_decoder_flops(**cfg), e2e="argmax", steps=5, registry_cfg=cfg, cpu=cpu and not one_mma_only,
                              one_mma_arm=not one_mma_only,
                              gemm_flops_per_sample=configs.gpt_decoder_gemm_flops(**cfg))


def _bench_c4(h, rt, peaks, abi, seed0, cpu, batch):
    # 4: conv vision stack, batch 64
    descs = configs.conv_stack()
    weights = configs.conv_stack_weights(descs)
    x = np.random.default_rng(seed0).random((batch, 3 * 224 * 224), dtype=np.float32)
    return bench_graph_config(h, rt, peaks, "4 conv vision stack: stem 7x7 s2 + 4 x [conv3x3, GroupNorm(32), SiLU, residual] 64..256 ch @112^2, fp32", descs, weights,
                              {"x": (x, False)}, batch, 256 * 112 * 112, abi.PREC_BF16X2, flops_per_sample=configs.conv_flops(descs), pipeline=8, steps=5, cpu=cpu)


def _bench_c5(h, rt, peaks, abi, seed0, cpu, batch, one_mma_only=False):
    # 5: UNet mid + up, batch 16
    descs = configs.unet_mid_up()
    weights = configs.seeded_weights(descs, seed=1, std=0.02, bf16=True)
    x = np.random.default_rng(seed0).standard_normal((batch, 4 * 64 * 64), dtype=np.float32)
    return bench_graph_config(h, rt, peaks, "5 UNet mid+up: latent 4x64x64 -> 3x256x256, channels 512/256/128, bf16-exact weights", descs, weights,
                              {"x": (x, False)}, batch, 3 * 256 * 256, abi.PREC_BF16 if one_mma_only else abi.PREC_BF16W,
                              flops_per_sample=configs.conv_flops(descs), pipeline=4, steps=5, cpu=cpu and not one_mma_only, one_mma_arm=not one_mma_only)


def bench_norms(h: Harness, rt, peaks):
    """LayerNorm / RMSNorm / GroupNorm + SiLU / Softmax at the configurations' shapes through the device-pointer per-op
    calls: 3 warm-up + 10 timed launches each, CUDA events, L2 flushed between launches when the tensor is below 300 MB."""
    from mimir_framework_b200 import abi

    torch = h.torch
    lib = rt.lib()
    st = h.stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(3)
    out = []

    def run(name, shape, n_elems, call, param_elems=0):
        x = torch.randn(n_elems, device="cuda", generator=g)
        y = torch.empty_like(x)
        flushed = n_elems * 4 < (300 << 20)
        for _ in range(3):
            rt.check(call(x, y))
        torch.cuda.synchronize()
        times = []
        for _ in range(10):
            if flushed:
                flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rt.check(call(x, y))
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ms = float(np.median(times))
        nbytes = 4 * (2 * n_elems + param_elems)
        gbs, frac = hbm_frac(nbytes, ms, peaks)
        out.append({"kernel": name, "shape": shape, "ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": gbs, "peak_gbs": peaks["hbm"], "frac": frac,
                    "l2": "flushed between launches" if flushed else "tensor larger than L2"})
        del x, y

    for rows, n in ((32768, 768), (8, 32768), (524288, 768)):
        gam, bet = torch.ones(n, device="cuda"), torch.zeros(n, device="cuda")
        run("layernorm", f"{rows}x{n}", rows * n,
            lambda x, y: lib.mimir_b200_dev_layernorm(x.data_ptr(), gam.data_ptr(), bet.data_ptr(), y.data_ptr(), rows, n, 1e-5, st), 2 * n)
    n = 1024 * 768
    gam = torch.ones(n, device="cuda")
    for b in (32, 256):
        run("rmsnorm (whole sample)", f"{b}x{n}", b * n, lambda x, y: lib.mimir_b200_dev_rmsnorm(x.data_ptr(), gam.data_ptr(), n, y.data_ptr(), b, n, 1e-5, st), n)
    C_, H = 256, 112
    gam, bet = torch.ones(C_, device="cuda"), torch.zeros(C_, device="cuda")
    run("groupnorm(32)+silu", f"64x{C_}x{H}x{H}", 64 * C_ * H * H,
        lambda x, y: lib.mimir_b200_dev_groupnorm(x.data_ptr(), gam.data_ptr(), bet.data_ptr(), y.data_ptr(), 64, C_, H, H, 32, 1e-5, abi.ELT_SILU, st))
    run("softmax (whole vector)", "4096x32000", 4096 * 32000, lambda x, y: lib.mimir_b200_dev_softmax(x.data_ptr(), y.data_ptr(), 4096, 32000, 0, st))
    del flush
    return out


def bench_gemm_shapes(h: Harness, rt, peaks, rows=32768):
    """The decoder configuration's projection shapes as single Linear layers (M = rows), in the strict two-MMA mode (bf16-exact
    weights) and in the one-MMA mode: time inside the GEMM kernel (CUDA events around every launch), algorithmic and issued
    fraction of the sustained bf16 peak.  The last record is configuration 2's layer in its three-MMA mode."""
    from mimir_framework_b200 import abi

    torch = h.torch
    shapes = [("qkv", rows, 768, 2304, False), ("attention out-projection", rows, 768, 768, False), ("ffn up + GELU", rows, 768, 3072, True),
              ("ffn down", rows, 3072, 768, False), ("lm head", rows, 768, 32000, False)]
    out = []
    r = np.random.default_rng(4)

    def one(name, M, K, N, gelu, precision, mmas):
        w = configs.round_to_bf16((r.standard_normal(K * N + N) * 0.02).astype(np.float32)) if precision != abi.PREC_BF16X2 else \
            (r.standard_normal(K * N + N) * 0.02).astype(np.float32)
        descs = [abi.make_desc("l", "Linear", inputs=["x"], output="h" if gelu else "x", in_features=K, out_features=N, seq_len=M, use_bias=1, params_count=K * N + N)]
        weights = [w]
        if gelu:  # folded into the GEMM's epilogue by the planner
            descs.append(abi.make_desc("a", "GELU", inputs=["h"], output="x"))
            weights.append(None)
        m = rt.GraphModel(descs, precision)
        for i, wt in enumerate(weights):
            m.upload_weights(i, wt)
        m.plan({"x": (M * K, False)}, 1)
        x = torch.randn(M * K, device="cuda")
        n_out = M * N
        y = torch.empty(n_out, device="cuda")
        spec = {"x": (x.data_ptr(), M * K, False)}
        for _ in range(3):
            m.forward_device(spec, 1, y.data_ptr(), n_out, h.stream)
        torch.cuda.synchronize()
        # one launch at a time under the profile switch: the first GEMM of the graph is the shape under study
        rt.profile_gemm(True)
        m.forward_device(spec, 1, y.data_ptr(), n_out, h.stream)
        rt.profile_read()
        times = []
        for _ in range(10):
            m.forward_device(spec, 1, y.data_ptr(), n_out, h.stream)
            ms, n = rt.profile_read()
            times.append(ms)
        rt.profile_gemm(False)
        m.close()
        del x, y
        return times

    for name, M, K, N, gelu in shapes:
        for precision, label, mmas in ((abi.PREC_BF16W, "BF16W", 2), (abi.PREC_BF16, "BF16", 1)):
            times = one(name, M, K, N, gelu, precision, mmas)
            ms = float(np.median(times))
            tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
            out.append({"layer": name, "m": M, "k": K, "n": N, "precision": label, "mma_per_product": mmas, "ms": ms, "tflops_algorithmic": tf,
                        "frac_algorithmic": tf / peaks["bf16_sustained"], "frac_issued": mmas * tf / peaks["bf16_sustained"]})
    times = one("config 2 layer", 65536, 4096, 4096, False, abi.PREC_BF16X2, 3)
    ms = float(np.median(times))
    tf = 2.0 * 65536 * 4096 * 4096 / (ms * 1e-3) / 1e12
    out.append({"layer": "config 2 layer (Linear + bias)", "m": 65536, "k": 4096, "n": 4096, "precision": "BF16X2", "mma_per_product": 3, "ms": ms,
                "tflops_algorithmic": tf, "frac_algorithmic": tf / peaks["bf16_sustained"], "frac_issued": 3 * tf / peaks["bf16_sustained"]})
    return out


def bench_decode_steps(h: Harness, rt, peaks, batch=16):
    """Token-by-token generation on the decoder configuration's shape with token-wise LayerNorm (the reference's
    whole-sample RMSNorm makes every row depend on later tokens, so that graph cannot be decoded incrementally):
    prefill of 991 tokens through the ordinary forward, then steps at positions ~1000 through the host-pointer entry
    point.  A step streams every weight once: bytes = fp32 Linear weights + attention planes + the key / value cache."""
    from mimir_framework_b200 import abi

    S = 1024
    P = S - 1 - 32
    E, V, L = 768, 32000, 12
    descs = configs.gpt_decoder(seq=P, norm="layer")
    weights = configs.seeded_weights(descs, seed=1, std=0.02, bf16=True)
    model = rt.GraphModel(descs, abi.PREC_BF16W)
    for i, w in enumerate(weights):
        model.upload_weights(i, w)
    model.plan({"x": (P, False)}, batch)
    cache = model.decode_begin({"x": (1, False)}, batch, S)
    ids = np.random.default_rng(0).integers(0, V, (batch, S)).astype(np.float32)
    model.forward({"x": (ids[:, :P].copy().ravel(), False)}, batch, P * V)
    for t in range(P, P + 4):  # warm-up steps
        model.decode_step({"x": (ids[:, t].copy(), False)}, batch, t, V)
    ts, dev = [], []
    for t in range(P + 4, P + 32):
        tok = ids[:, t].copy()
        t0 = time.perf_counter()
        model.decode_step({"x": (tok, False)}, batch, t, V)
        ts.append(time.perf_counter() - t0)
        dev.append(rt.stats()["ms_last_forward"])
    ms, dev_ms = 1e3 * float(np.median(ts)), float(np.median(dev))
    total = 4 * (L * 2 * E * 3072 + E * V) + 2 * L * 4 * E * E + 4 * 2 * L * batch * (P + 18) * E
    gbs, frac = hbm_frac(total, dev_ms, peaks)
    model.close()
    return {"config": "decode steps: GPT decoder d768 h12 ffn3072 vocab32000, token-wise LayerNorm, positions ~1000", "batch": batch,
            "ms_per_step_host": ms, "ms_per_step_device": dev_ms, "tokens_per_s": batch / (ms * 1e-3), "cache_bytes": cache,
            "bytes_per_step": total, "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": frac}}


def bench_copy_ceiling(h: Harness, x_host, y_host, x_dev, y_dev, steps):
    """What plain pinned copies of the headline's bytes reach with all ranks copying at once: H2D of the inputs and
    D2H of the outputs of one step on two streams, nothing else running.  Milliseconds per step, max over ranks."""
    torch = h.torch
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def step():
        with torch.cuda.stream(s_in):
            x_dev.copy_(x_host, non_blocking=True)
        with torch.cuda.stream(s_out):
            y_host.copy_(y_dev, non_blocking=True)
        s_in.synchronize()
        s_out.synchronize()
    return h.wall_steps(step, steps)


def bench_single_process(h: Harness, rt, rows_per_gpu, steps, pipeline):
    """Rank 0 alone drives every GPU of the box through the replica entry points (the other ranks wait on a host
    barrier, nothing of theirs runs on the GPUs): one host thread per device, every slice's result gathered into ONE
    pinned host buffer.  Returns rows/s end to end."""
    torch = h.torch
    rec = None
    h.host_barrier()
    if h.rank == 0:
        n = h.world
        total = rows_per_gpu * n
        reps = rt.Replicas(list(range(n)), configs.linear_gelu_stack(rows_per_gpu // pipeline), pipeline=pipeline)
        for i, w in enumerate(configs.linear_gelu_stack_weights()):
            reps.upload_weights(i, w)
        per = (rows_per_gpu // pipeline) * K
        reps.plan({"x": (per, False)}, n * pipeline)
        x = torch.from_numpy(configs.linear_gelu_stack_input(total)).pin_memory()
        y = torch.empty((total, K), dtype=torch.float32).pin_memory()
        spec = {"x": (x.data_ptr(), per, False)}
        for _ in range(2):
            reps.forward_host_ptrs(spec, n * pipeline, y.data_ptr(), y.numel())
        t0 = time.perf_counter()
        for _ in range(steps):
            reps.forward_host_ptrs(spec, n * pipeline, y.data_ptr(), y.numel())
        dt = (time.perf_counter() - t0) / steps
        rec = {"value": total / dt, "unit": UNIT, "ms_per_step": 1e3 * dt, "rows_total": total, "devices": n, "host_threads": n,
               "h2d_bytes_per_step": total * K * 4, "d2h_bytes_per_step": total * K * 4, "checksum_first_rows": float(y[:64].double().abs().sum()),
               "how": "one process: mimir_b200_replicas_forward slices the batch over the devices and copies every slice into its place in one pinned buffer"}
        reps.close()
        rt.init(h.local_rank, 0)
        del x, y
    h.host_barrier()
    return rec


def run_ours(args):
    h = Harness()
    torch = h.torch
    world, rank, local_rank = h.world, h.rank, h.local_rank

    from mimir_framework_b200 import runtime as rt

    rt.init(local_rank, 0)  # raises if the CUDA library is missing or there is no sm_100 device
    peaks = measured_peaks()

    if args.only not in ("all", "headline"):
        # one leg alone (kernel studies, profiler captures): its records, one JSON line, no headline
        rec = {}
        if args.only in ("configs", "c1", "c3", "c4", "c5"):
            rec["configs"] = bench_other_configs(h, rt, peaks, args)
        if args.only == "norms":
            rec["norms"] = bench_norms(h, rt, peaks)
        if args.only == "decode":
            rec["decode"] = bench_decode_steps(h, rt, peaks)
        if args.only == "gemm":
            rec["gemm_shapes"] = bench_gemm_shapes(h, rt, peaks)
        if rank == 0:
            print(json.dumps(rec))
        if world > 1:
            h.dist.barrier()
            h.dist.destroy_process_group()
        return

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
    stream = h.stream
    spec_dev = {"x": (x_dev.data_ptr(), M * K, False)}
    barrier = h.barrier

    # ---- device-resident throughput --------------------------------------------------------------
    # (every GEMM launch is bracketed by CUDA events in this region, which also keeps the layer loop from being
    # replayed as one CUDA graph: the number is the conservative one)
    for _ in range(max(args.warmup, 3)):
        model.forward_device(spec_dev, 1, y_dev.data_ptr(), M * K, stream)
    barrier()
    sampler = ClockSampler(local_rank)  # every rank watches its own GPU: the step time is the slowest rank's
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
    clocks = sampler.stop(t_wall0, t_wall1)
    ms_local = e0.elapsed_time(e1)
    ms_total = h.max_over_ranks(ms_local)
    per_rank = None
    if world > 1:
        mine = {"rank": rank, "ms_per_step": ms_local / args.steps, "sm_mhz": (clocks or {}).get("sm_mhz"),
                "power_w_max": (clocks or {}).get("power_w_max"), "reasons": (clocks or {}).get("reasons")}
        per_rank = [None] * world
        h.dist.all_gather_object(per_rank, mine, group=h.host_group)
    ms_per_step = ms_total / args.steps
    value = world * M / (ms_per_step * 1e-3)

    # ---- end to end through the host-pointer call ------------------------------------------------
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    e2e_ms = h.wall_steps(lambda: model_e2e.forward_host_ptrs(spec_host, chunks, y_host.data_ptr(), M * K), e2e_steps)  # synchronous: H2D, layers, D2H
    e2e_value = world * M / (e2e_ms * 1e-3)
    checksum = float(y_host[:64].double().abs().sum())
    copy_ms = bench_copy_ceiling(h, x_host, y_host, x_dev, y_dev, e2e_steps)
    copy_value = world * M / (copy_ms * 1e-3)

    # ---- roofline of the dominant kernel (the GEMM) ----------------------------------------------
    per_launch_flops = 2.0 * M * K * K
    gemm_avg_ms = gemm_ms / max(gemm_launches, 1)
    achieved = per_launch_flops / (gemm_avg_ms * 1e-3) / 1e12 if gemm_launches else None
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_sustained"], "unit": "TFLOP/s",
        "frac": (achieved / peaks["bf16_sustained"]) if achieved else None,
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch at M = 8192 rows (ncu --set full): the activation
        # planes and the output grow with the rows of the launch, the weight planes (2 x 2 x 4096^2 bytes) do not
        "traffic": NCU_WEIGHT_BYTES + (NCU_TRAFFIC_BYTES_AT_8192_ROWS - NCU_WEIGHT_BYTES) * M / 8192,
        "traffic_unit": "bytes per launch (ncu at M=8192; the row-dependent part scaled by rows)",
        "kernel": "gemm_tn_bf16split_kernel", "launches_timed": gemm_launches, "avg_launch_ms": gemm_avg_ms,
        "peak_source": f"{peaks['source']} (cuBLAS bf16 8192^3 sustained)",
        "issued_tflops": (3 * achieved) if achieved else None,
        "note": "achieved counts algorithmic flops 2*M*N*K; the kernel issues 3 half-precision MMAs per product term (hi*hi + lo*hi + hi*lo)",
    }
    model.close()
    model_e2e.close()
    del x_dev, y_dev

    extras = {}
    if not args.headline_only and args.only == "all":
        extras["configs"] = bench_other_configs(h, rt, peaks, args)
        extras["norms"] = bench_norms(h, rt, peaks)
        if world == 1:
            extras["decode"] = bench_decode_steps(h, rt, peaks)
            extras["gemm_shapes"] = bench_gemm_shapes(h, rt, peaks)
        if world > 1:
            extras["single_process"] = bench_single_process(h, rt, args.single_process_rows, e2e_steps, args.pipeline)

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
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16x2 split (fp32 in/out, operands as half hi+lo planes, fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": f"Linear+bias+GELU x3, K=N={K}, M={M} fp32 rows per GPU", "rows_per_gpu": M,
                       "l2_policy": "inputs larger than L2 (1 GiB activations per layer), no flush", "precision": "BF16X2 (three MMAs per product), half planes",
                       "parallelism": f"replica per GPU x{world}, rows sharded, no collective"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * K * 4,
                    "steps": e2e_steps, "micro_batches": chunks, "checksum_first_rows": checksum,
                    "copy_ceiling": {"value": copy_value, "unit": UNIT, "ms_per_step": copy_ms,
                                     "how": "pinned H2D of one step's inputs and D2H of its outputs on two streams, all ranks at once, nothing else running"},
                    "frac_of_copy_ceiling": e2e_value / copy_value},
            "gpu_launches": int(launches),
            "tflops_algorithmic": configs.linear_gelu_stack_flops(M) / (ms_per_step * 1e-3) / 1e12,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "clocks": clocks,
            **({"per_rank": per_rank} if per_rank else {}),
        }
        line.update(extras)
        print(json.dumps(line))
    if world > 1:
        h.dist.barrier()
        h.dist.destroy_process_group()


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
    ap.add_argument("--headline-only", action="store_true", help="skip the other configurations, the norm kernels and the single-process leg")
    ap.add_argument("--only", default="all", choices=["all", "headline", "configs", "c1", "c3", "c4", "c5", "norms", "decode", "gemm"],
                    help="run one leg alone and print its records (no headline line)")
    ap.add_argument("--precision", default="default", choices=["default", "one-mma"],
                    help="configs 3 and 5: 'one-mma' runs the one-plane-per-operand mode as the only arm (for profiling it); "
                         "the default runs the strict mode and the one-MMA mode as a second arm beside it")
    ap.add_argument("--decoder-batch", type=int, default=32, help="samples per GPU of the decoder configuration")
    ap.add_argument("--conv-batch", type=int, default=64, help="samples per GPU of the conv vision stack")
    ap.add_argument("--unet-batch", type=int, default=16, help="samples per GPU of the UNet mid+up path")
    ap.add_argument("--single-process-rows", type=int, default=16384, help="rows per GPU of the single-process leg (N > 1)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

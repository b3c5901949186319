"""Per-kernel and per-configuration measurements beside the headline benchmark.

    python -m mimir_framework_b200.opbench [--only norms|configs] [--no-cpu]

Prints one JSON line per measurement:
  * the HBM-bound kernels (LayerNorm, RMSNorm, GroupNorm+SiLU, Softmax, GELU, Add) at the sizes the
    configurations use, as achieved GB/s of algorithmic bytes (read + write) against the measured
    HBM copy bandwidth;
  * the other configurations (registry transformer encoder at batch 8, ...) as samples/s, with the
    reference's CPU path timed on the host cores when the compiled reference is present.
Device-resident inputs, CUDA events on the launching stream, 3 warm-up + 10 timed launches; every
input is larger than L2 or the L2 is flushed between launches (stated per line).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from mimir_framework_b200 import abi, configs, runtime as rt  # noqa: E402


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f)["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def time_launches(fn, warmup=3, iters=10, flush=None):
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return float(np.median(times)), times


def bench_norms():
    import torch

    lib = rt.lib()
    st = torch.cuda.current_stream().cuda_stream
    peak, src = hbm_peak()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # 256 MB > L2
    g = torch.Generator(device="cuda").manual_seed(3)

    def report(name, ms, nbytes, shape, flushed):
        gbs = nbytes / (ms * 1e-3) / 1e9
        print(json.dumps({"kernel": name, "shape": shape, "ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": gbs,
                          "peak_gbs": peak, "frac": gbs / peak, "peak_source": src,
                          "l2": "flushed between launches" if flushed else "input larger than L2"}), flush=True)

    def run(name, shape, n_elems, call, param_elems=0):
        x = torch.randn(n_elems, device="cuda", generator=g)
        y = torch.empty_like(x)
        flushed = n_elems * 4 < (300 << 20)
        ms, _ = time_launches(lambda: rt.check(call(x, y)), flush=flush if flushed else None)
        report(name, ms, 4 * (2 * n_elems + param_elems), shape, flushed)
        del x, y

    # LayerNorm: token-wise rows and the registry transformer's whole-vector rows
    for rows, n in ((32768, 768), (8, 32768), (524288, 768)):
        gam = torch.ones(n, device="cuda")
        bet = torch.zeros(n, device="cuda")
        run("layernorm", f"{rows}x{n}", rows * n,
            lambda x, y: lib.mimir_b200_dev_layernorm(x.data_ptr(), gam.data_ptr(), bet.data_ptr(), y.data_ptr(), rows, n, 1e-5, st), 2 * n)
    # RMSNorm over whole samples (decoder config: 32 x 1024*768)
    n = 1024 * 768
    gam = torch.ones(n, device="cuda")
    for b in (32, 256):
        run("rmsnorm", f"{b}x{n}", b * n, lambda x, y: lib.mimir_b200_dev_rmsnorm(x.data_ptr(), gam.data_ptr(), n, y.data_ptr(), b, n, 1e-5, st), n)
    # GroupNorm(32) + SiLU on 64 x 256 x 112 x 112
    C_, H = 256, 112
    gam = torch.ones(C_, device="cuda")
    bet = torch.zeros(C_, device="cuda")
    run("groupnorm+silu", f"64x{C_}x{H}x{H} G32", 64 * C_ * H * H,
        lambda x, y: lib.mimir_b200_dev_groupnorm(x.data_ptr(), gam.data_ptr(), bet.data_ptr(), y.data_ptr(), 64, C_, H, H, 32, 1e-5, abi.ELT_SILU, st))
    # Softmax: 4096 independent samples of 32000
    run("softmax", "4096x32000", 4096 * 32000, lambda x, y: lib.mimir_b200_dev_softmax(x.data_ptr(), y.data_ptr(), 4096, 32000, 0, st))
    # element-wise
    n = 1 << 28
    run("gelu", f"{n}", n, lambda x, y: lib.mimir_b200_dev_eltwise(abi.ELT_GELU, x.data_ptr(), None, y.data_ptr(), 1, n, 0, st))
    b = torch.randn(n, device="cuda", generator=g)
    x = torch.randn(n, device="cuda", generator=g)
    y = torch.empty_like(x)
    ms, _ = time_launches(lambda: rt.check(lib.mimir_b200_dev_eltwise(abi.ELT_ADD, x.data_ptr(), b.data_ptr(), y.data_ptr(), 1, n, n, st)))
    report("add", ms, 12 * n, f"{n}", False)


def bench_transformer(no_cpu: bool):
    """Configuration 1: registry transformer encoder, batch 8, fp32, ids seed 0, weights N(0, 0.02) seed 1."""
    import torch

    cfg = configs.TRANSFORMER_CFG
    descs = configs.transformer_encoder(**cfg)
    weights = configs.seeded_weights(descs, seed=1, std=0.02)
    batch, S, D = 8, cfg["seq_len"], cfg["d_model"]
    ids = np.random.default_rng(0).integers(0, cfg["vocab_size"], (batch, S)).astype(np.float32)
    r = np.random.default_rng(2)
    mag, mod = (r.standard_normal(D) * 0.02).astype(np.float32), (r.standard_normal(D) * 0.02).astype(np.float32)
    want, cpu_ms, cores = None, None, None
    if not no_cpu:
        from oracle import ref
        if ref.available():
            cores = ref.set_threads(os.cpu_count() or 1)
            m = ref.RefModel(registry="transformer", cfg_json=json.dumps(cfg))
            for i, w in enumerate(weights):
                if w is not None:
                    m.set_weights(i, w)
            mag, mod = m.mag_mod()  # the Encoder's own vectors
            outs, ts = [], []
            for s in range(batch):
                y, secs = m.forward({"x": ids[s], "mag": mag, "mod": mod}, return_seconds=True)
                outs.append(y)
                ts.append(secs)
            want = np.stack(outs)
            cpu_ms = 1e3 * float(np.median(ts[1:]))
            m.close()
    model = rt.GraphModel(descs)
    for i, w in enumerate(weights):
        model.upload_weights(i, w)
    model.plan({"x": (S, False), "mag": (D, True), "mod": (D, True)}, batch)
    got = model.forward({"x": (ids.ravel(), False), "mag": (mag, True), "mod": (mod, True)}, batch, cfg["output_dim"])
    parity = None
    if want is not None:
        err = np.abs(got - want)
        parity = {"max_abs": float(err.max()), "outside_tolerance": int((err > 1e-4 + 1e-3 * np.abs(want)).sum()), "n": int(want.size)}
    d_ids, d_mag, d_mod = (torch.from_numpy(a).cuda() for a in (ids, mag, mod))
    d_out = torch.empty(batch, cfg["output_dim"], device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    spec = {"x": (d_ids.data_ptr(), S, False), "mag": (d_mag.data_ptr(), D, True), "mod": (d_mod.data_ptr(), D, True)}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ms, _ = time_launches(lambda: model.forward_device(spec, batch, d_out.data_ptr(), d_out.numel(), st), flush=None)
    weight_bytes = 4 * sum(int(d.params_count) for d in descs if d.type.decode() != "Embedding")
    peak, src = hbm_peak()
    print(json.dumps({"config": "1 transformer encoder (registry graph), batch 8, fp32", "ms_per_batch": ms,
                      "samples_per_s": batch / (ms * 1e-3), "weight_stream_bytes": weight_bytes,
                      "achieved_gbs": weight_bytes / (ms * 1e-3) / 1e9, "peak_gbs": peak, "frac": weight_bytes / (ms * 1e-3) / 1e9 / peak,
                      "peak_source": src, "l2": "574 MB of weights per forward, larger than L2",
                      "cpu_reference_ms_per_sample": cpu_ms, "cpu_reference_samples_per_s": (1e3 / cpu_ms) if cpu_ms else None,
                      "cpu_cores": cores, "parity": parity}), flush=True)
    model.close()
    del flush


def _time_graph(model, spec, batch, out, stream, iters=int(os.environ.get('OPBENCH_ITERS', '5'))):
    ms, _ = time_launches(lambda: model.forward_device(spec, batch, out.data_ptr(), out.numel(), stream), warmup=2, iters=iters)
    return ms


def _cpu_sample(descs, weights, inputs, no_cpu, repeats=1):
    """One sample through the compiled reference: (output, seconds, threads) or (None, None, None)."""
    if no_cpu:
        return None, None, None
    from oracle import ref
    if not ref.available():
        return None, None, None
    cores = ref.set_threads(os.cpu_count() or 1)
    ref.set_guard_limit(64 << 30)
    m = ref.RefModel(descs)
    for i, w in enumerate(weights):
        if w is not None:
            m.set_weights(i, w)
    best, y = None, None
    for _ in range(repeats):
        y, secs = m.forward(inputs, return_seconds=True)
        best = secs if best is None else min(best, secs)
    m.close()
    return y, best, cores


def _parity(got, want):
    if want is None:
        return None
    err = np.abs(got.ravel() - want.ravel())
    return {"max_abs": float(err.max()), "outside_tolerance": int((err > 1e-4 + 1e-3 * np.abs(want.ravel())).sum()), "n": int(want.size)}


def bench_graph_config(name, descs, weights, x, batch, out_n, flops_per_sample, precision, no_cpu, cpu_note):
    """Times `batch` samples device-resident; parity of sample 0 against the compiled reference."""
    import torch

    model = rt.GraphModel(descs, precision)
    for i, w in enumerate(weights):
        model.upload_weights(i, w)
    per = x.size // batch
    model.plan({"x": (per, False)}, batch)
    d_x = torch.from_numpy(x).cuda()
    d_out = torch.empty(batch * out_n, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    spec = {"x": (d_x.data_ptr(), per, False)}
    rt.profile_gemm(True)
    ms = _time_graph(model, spec, batch, d_out, st)
    gemm_ms, gemm_n = rt.profile_read()
    rt.profile_gemm(False)
    rt.check(rt.lib().mimir_b200_check_device(None))
    got0 = d_out[:out_n].cpu().numpy()
    want, secs, cores = _cpu_sample(descs, weights, {"x": x.reshape(batch, per)[0]}, no_cpu)
    runs = 2 + int(os.environ.get('OPBENCH_ITERS', '5'))
    print(json.dumps({"config": name, "batch": batch, "ms_per_batch": ms, "samples_per_s": batch / (ms * 1e-3),
                      "tflops_algorithmic": flops_per_sample * batch / (ms * 1e-3) / 1e12,
                      "gemm_share_of_step": (gemm_ms / runs) / ms if gemm_n else None,
                      "arena_bytes": model.arena_bytes, "precision": precision,
                      "cpu_reference_s_per_sample": secs, "cpu_reference_samples_per_s": (1.0 / secs) if secs else None,
                      "cpu_cores": cores, "cpu_note": cpu_note, "parity_sample0": _parity(got0, want)}), flush=True)
    model.close()
    del d_x, d_out


def bench_decoder(no_cpu):
    cfg = configs.DECODER_CFG
    descs = configs.gpt_decoder(**cfg)
    weights = configs.seeded_weights(descs, seed=1, std=0.02, bf16=True)
    batch = int(os.environ.get('OPBENCH_BATCH', '32'))
    ids = np.random.default_rng(0).integers(0, cfg["vocab"], (batch, cfg["seq"])).astype(np.float32)
    bench_graph_config("3 GPT decoder prefill, 12 layers d768 h12 ffn3072 vocab32000 seq1024, bf16-exact weights", descs, weights, ids,
                       batch, cfg["seq"] * cfg["vocab"], configs.gpt_decoder_flops(**cfg), abi.PREC_BF16W, no_cpu,
                       "one sample through the reference CPU path")


def bench_conv_stack(no_cpu):
    descs = configs.conv_stack()
    weights = configs.conv_stack_weights(descs)
    batch = int(os.environ.get("OPBENCH_BATCH", "64"))
    x = np.random.default_rng(0).random((batch, 3 * 224 * 224), dtype=np.float32)
    bench_graph_config("4 conv vision stack, stem 7x7 s2 + 4 x [conv3x3, GroupNorm(32), SiLU, residual], 64..256 ch @112^2", descs,
                       weights, x, batch, 256 * 112 * 112, configs.conv_flops(descs), abi.PREC_BF16X2, no_cpu,
                       "one sample through the reference CPU path")


def bench_unet(no_cpu):
    descs = configs.unet_mid_up()
    weights = configs.seeded_weights(descs, seed=1, std=0.02, bf16=True)
    batch = int(os.environ.get("OPBENCH_BATCH", "16"))
    x = np.random.default_rng(0).standard_normal((batch, 4 * 64 * 64), dtype=np.float32)
    bench_graph_config("5 UNet mid+up, latent 4x64x64 -> 3x256x256, channels 512/256/128, bf16-exact weights", descs, weights, x, batch,
                       3 * 256 * 256, configs.conv_flops(descs), abi.PREC_BF16W, no_cpu, "one sample through the reference CPU path")


def bench_decode_steps():
    """Token-by-token generation on the decoder configuration's shape with token-wise LayerNorm (the reference's
    whole-sample RMSNorm makes every row depend on later tokens, so that graph cannot be decoded incrementally):
    prefill of 1023 tokens through the ordinary forward, then steps at positions 1023 .. through the host-pointer
    entry point.  A step streams every weight once: bytes = fp32 Linear weights (rows <= 16 take the
    weight-streaming kernel) + bf16 attention planes + the key / value cache read."""
    batch, S = int(os.environ.get("OPBENCH_BATCH", "16")), 1024
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
    import time
    for t in range(P, P + 4):  # warm-up steps
        model.decode_step({"x": (ids[:, t].copy(), False)}, batch, t, V)
    ts = []
    for t in range(P + 4, P + 32):
        tok = ids[:, t].copy()
        t0 = time.perf_counter()
        model.decode_step({"x": (tok, False)}, batch, t, V)
        ts.append(time.perf_counter() - t0)
    ms = 1e3 * float(np.median(ts))
    dev_ms = rt.stats()["ms_last_forward"]
    lin_bytes = 4 * (L * 2 * E * 3072 + E * V)
    attn_bytes = 2 * L * 4 * E * E
    kv_bytes = 4 * 2 * L * batch * (P + 18) * E
    total = lin_bytes + attn_bytes + kv_bytes
    peak, src = hbm_peak()
    print(json.dumps({"config": "GPT decoder d768 h12 ffn3072 vocab32000, token-wise LayerNorm: decode steps at positions ~1000", "batch": batch,
                      "ms_per_step_host": ms, "ms_per_step_device": dev_ms, "tokens_per_s": batch / (ms * 1e-3), "cache_bytes": cache,
                      "bytes_per_step": total, "achieved_gbs_device": total / (dev_ms * 1e-3) / 1e9, "peak_gbs": peak,
                      "frac_device": total / (dev_ms * 1e-3) / 1e9 / peak, "peak_source": src}), flush=True)
    model.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="all", choices=["all", "norms", "configs", "c1", "c3", "c4", "c5", "decode"])
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    rt.init(0, 0)
    if args.only in ("all", "norms"):
        bench_norms()
    if args.only in ("all", "configs", "c1"):
        bench_transformer(args.no_cpu)
    if args.only in ("all", "configs", "c3"):
        bench_decoder(args.no_cpu)
    if args.only in ("all", "configs", "c4"):
        bench_conv_stack(args.no_cpu)
    if args.only in ("all", "configs", "c5"):
        bench_unet(args.no_cpu)
    if args.only in ("all", "decode"):
        bench_decode_steps()
    rt.shutdown()


if __name__ == "__main__":
    main()

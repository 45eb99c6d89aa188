#!/usr/bin/env python
"""Benchmark of the training hot path: GPT-small fwd + bwd + clip + AdamW, tokens/s.

  python bench.py --gpus N --steps K --warmup W            the CUDA library (one rank per GPU under torchrun)
  python bench.py --impl reference --gpus N --steps K ...   the reference's CPU implementation of the same step
                                                            (the C++ restatement in oracle/, host cores)

Prints ONE JSON line on rank 0.  `value` is whole-job tokens/s with inputs resident in HBM; `e2e` is
the same metric through the host-buffer entry point (H2D of the token ids and D2H of the loss inside
the timed region).  Timing: CUDA events on the library's compute stream, barrier + synchronise on both
sides, max over ranks.  An untimed pass with per-kernel events gives `roofline` and `kernels`.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # BASELINE.json configs[2]: the configuration the headline metric is quoted on
    "gpt-small": dict(vocab=50304, T=1024, d=768, heads=12, layers=12, ff=3072, micro_batch=8, lr=6e-4, wd=0.1, clip=1.0),
    # configs[4]
    "gpt-medium": dict(vocab=50304, T=1024, d=1024, heads=16, layers=24, ff=4096, micro_batch=4, lr=6e-4, wd=0.1, clip=1.0),
    # configs[3]: 3 x [conv3x3 -> BatchNorm -> ReLU -> MaxPool] -> AvgPool -> Linear -> cross-entropy, SGD momentum; images/s
    "convnet": dict(kind="convnet", channels=(3, 64, 128, 256), classes=10, hw=32, micro_batch=256, lr=0.1, momentum=0.9, clip=0.0),
    # configs[1]: the fused-op backward chain, LayerNorm -> GELU -> Linear 768 -> 50304 -> cross-entropy on 8192 rows; rows/s
    "fused-op": dict(kind="fused-op", N=8192, C=768, V=50304),
    # a seconds-long case for plumbing checks
    "gpt-tiny": dict(vocab=512, T=64, d=128, heads=4, layers=2, ff=512, micro_batch=4, lr=6e-4, wd=0.1, clip=1.0),
}


# DRAM bytes of ONE launch of the dominant kernel, read from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum) of
# `python kernel_cases.py gemm_fc1`: x[8192,768] . W[3072,768]^T with the weight's lo plane loaded beside it.  Operands and result
# of that launch: 25.2 + 9.4 + 9.4 (lo plane) + 100.7 MB; half of the result is still in L2 when the kernel ends.  It is a figure
# from a profile, not of this run: the key says so.
TRAFFIC_FROM_PROFILE = {"traffic": 101.1e6, "traffic_unit": "bytes per launch", "traffic_launch": "M8192 N3072 K768 (GPT-small fc1 forward)",
                        "traffic_algorithmic": 144.7e6, "traffic_from_profile": "profiles/gemm_tc_fc1_and_dw.md"}

# Dense TF32 rate of this pool's B200s, measured with `python bench.py --measure-tf32-peak` (torch.matmul, TF32 allowed, 8192^3;
# best of 10 and a 4 s back-to-back loop, like the bf16 figures of MEASURED_PEAKS.json).  Under the 1000 W cap the sustained loop
# ran at a median 1080 MHz SM clock (sw_power_cap the only reason active).
TF32_PEAK = {"tflops_burst": 708.2, "tflops_sustained": 619.3, "sm_mhz_sustained": 1080.0,
             "source": "measured: torch.matmul allow_tf32 8192^3, burst best of 10 / 4 s loop"}


def flops_per_token(c):
    """Useful fwd+bwd flops per token: 6 per weight of every matmul + full (non-causal) attention,
    as the reference computes it."""
    mm = c["layers"] * (4 * c["d"] * c["d"] + 2 * c["d"] * c["ff"]) + c["d"] * c["vocab"]
    attn = c["layers"] * 2 * c["T"] * c["d"]          # QK^T and PV, multiply-adds per token
    return 6 * mm + 6 * attn


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True); self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
                for n, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline_sample(cfg, T=None, threads=0):
    """Times the CPU oracle on a bounded sample and returns (tokens_per_s, description, cores).

    Sample: one sequence through a 1-block and a 2-block model of the workload's widths (embeddings,
    head, cross-entropy, clip and AdamW included); the 12/24-block step time is the 1-block time plus
    (layers - 1) x (the 2-block time minus the 1-block time)."""
    from oracle import oracle as orc
    from oracle import models as om
    from vearo_b200 import modelspec as ms
    T = T or cfg["T"]
    orc.set_threads(threads)
    times = {}
    for L in (1, 2):
        orc.reset_all()
        params = ms.gpt_params(cfg["vocab"], T, cfg["d"], L, cfg["ff"])
        m = om.SimpleGPT(params, cfg["d"], cfg["heads"], L)
        opt = orc.AdamW(m.parameters(), cfg["lr"], 0.9, 0.999, 1e-8, cfg["wd"])
        ids, tg = ms.gpt_batch(cfg["vocab"], 1, T)
        t0 = time.perf_counter()
        orc.zero_gradients(); orc.reset_active_tape()
        _, loss = m.forward(orc.Tensor.from_numpy(ids), orc.Tensor.from_numpy(tg))
        loss.backward()
        orc.clip_grad_norm(m.parameters(), cfg["clip"]); opt.step()
        times[L] = time.perf_counter() - t0
    orc.reset_all()
    block = max(times[2] - times[1], 1e-9)
    full = times[1] + (cfg["layers"] - 1) * block
    desc = ("1 sequence of T=%d through a 1-block (%.1f s) and a 2-block (%.1f s) model, full vocab head, clip+AdamW; "
            "%d-block step time = t1 + %d*(t2-t1) = %.1f s" % (T, times[1], times[2], cfg["layers"], cfg["layers"] - 1, full))
    return T / full, desc, orc.get_threads(), times[1], block


def cpu_convnet_step_time(cfg, images=16, steps=1, warmup=0, threads=0):
    """Seconds per step of the CPU oracle on a batch of `images` images of the ConvNet workload (SGD step included)."""
    from oracle import oracle as orc
    from oracle import models as om
    from vearo_b200 import modelspec as ms
    orc.set_threads(threads); orc.reset_all()
    m = om.ConvNet(ms.convnet_params(cfg["channels"], cfg["classes"]))
    opt = orc.SGD(m.parameters(), cfg["lr"], cfg["momentum"], 0.0)
    x, y = ms.convnet_batch(images, cfg["hw"], cfg["classes"])
    durs = []
    for s in range(warmup + steps):
        t0 = time.perf_counter()
        orc.zero_gradients(); orc.reset_active_tape()
        loss = m.forward(orc.Tensor.from_numpy(x), orc.Tensor.from_numpy(y))
        loss.backward(); opt.step()
        if s >= warmup:
            durs.append(time.perf_counter() - t0)
    cores = orc.get_threads()
    orc.reset_all()
    return durs, cores


def run_reference_convnet(args, cfg):
    from oracle import build as ob
    ob.build()
    images = 16
    durs, cores = cpu_convnet_step_time(cfg, images, args.steps, args.warmup)
    step_s = float(np.mean(durs)); value = images / step_s
    sample = "each step = fwd + bwd + SGD on %d images of 3x%dx%d (the workload's batch is %d; cost is linear in images)" % (images, cfg["hw"], cfg["hw"], cfg["micro_batch"])
    out = {"impl": "reference", "metric": "ConvNet fwd+bwd+SGD images/s", "value": value, "unit": "images/s", "n_gpus": args.gpus,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": args.workload, "channels": list(cfg["channels"]), "classes": cfg["classes"], "hw": cfg["hw"], "micro_batch": images},
           "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
           "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    print(json.dumps(out), flush=True)


def run_reference(args, cfg, rank):
    """The reference arm: the CPU restatement of the reference's implementation (the Rust crate cannot be
    built here: no cargo/rustc), all host threads the reference itself would use.

    Every step is a real step of the stated configuration -- all blocks, full sequence length, full vocabulary,
    clip + AdamW -- on ONE sequence (micro-batch 1; the cost is linear in the batch).  Such a step takes about a
    minute of CPU time, so the run is held to a wall budget: one warm-up step, then as many of the requested
    steps as fit (`steps_timed`); `ms_per_step` is the mean of the steps that were timed, nothing is
    extrapolated."""
    if rank != 0:
        return
    if cfg.get("kind") == "convnet":
        return run_reference_convnet(args, cfg)
    if cfg.get("kind") == "fused-op":
        return run_reference_fused_op(args, cfg)
    from oracle import build as ob
    ob.build()
    from oracle import oracle as orc
    from oracle import models as om
    from vearo_b200 import modelspec as ms
    budget = float(os.environ.get("VB200_REF_BUDGET_S", "420"))
    t_begin = time.perf_counter()
    orc.set_threads(0); orc.reset_all()
    T, L = cfg["T"], cfg["layers"]
    m = om.SimpleGPT(ms.gpt_params(cfg["vocab"], T, cfg["d"], L, cfg["ff"]), cfg["d"], cfg["heads"], L)
    opt = orc.AdamW(m.parameters(), cfg["lr"], 0.9, 0.999, 1e-8, cfg["wd"])
    batches = [ms.gpt_batch(cfg["vocab"], 1, T, seed=i) for i in range(2)]

    def step(i):
        ids, tg = batches[i % 2]
        t0 = time.perf_counter()
        orc.zero_gradients(); orc.reset_active_tape()
        _, loss = m.forward(orc.Tensor.from_numpy(ids), orc.Tensor.from_numpy(tg))
        loss.backward(); orc.clip_grad_norm(m.parameters(), cfg["clip"]); opt.step()
        return time.perf_counter() - t0, float(loss.numpy()[0])
    warm = min(args.warmup, 1)
    for i in range(warm):
        step(i)
    durs, loss = [], None
    while len(durs) < args.steps:
        d, loss = step(warm + len(durs))
        durs.append(d)
        if time.perf_counter() - t_begin + 1.15 * d > budget:
            break
    cores = orc.get_threads()
    orc.reset_all()
    step_s = float(np.mean(durs))
    value = T / step_s
    sample = ("each step = fwd + bwd + clip + AdamW of the full model (%d blocks, T=%d, vocab %d) on one sequence; %d warm-up + %d timed steps "
              "inside a %.0f s wall budget (requested %d + %d); per-step seconds: %s"
              % (L, T, cfg["vocab"], warm, len(durs), budget, args.warmup, args.steps, ", ".join("%.1f" % d for d in durs)))
    out = {"impl": "reference", "metric": "GPT-small fwd+bwd+AdamW tokens/s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
           "steps": args.steps, "warmup": args.warmup, "steps_timed": len(durs), "warmup_run": warm,
           "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": args.workload, "n_layer": L, "n_head": cfg["heads"], "d_model": cfg["d"], "d_ff": cfg["ff"],
                      "vocab": cfg["vocab"], "seq_len": T, "micro_batch_per_gpu": 1, "global_batch": 1,
                      "optimizer": "AdamW lr %g wd %g, clip %g" % (cfg["lr"], cfg["wd"], cfg["clip"])},
           "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
           "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0, "last_loss": loss}
    print(json.dumps(out), flush=True)


def run_reference_fused_op(args, cfg):
    """Config 2 on the CPU restatement: LayerNorm -> GELU -> Linear C->V -> cross-entropy, forward + backward, on a row sample."""
    from oracle import build as ob
    ob.build()
    from oracle import oracle as orc
    from vearo_b200 import modelspec as ms
    rows = 256
    x, g, b, W, labels = ms.microbench_inputs(N=rows, C=cfg["C"], V=cfg["V"])
    orc.set_threads(0)
    durs = []
    for s in range(min(args.warmup, 1) + min(args.steps, 5)):
        orc.reset_all()
        cx = orc.Tensor.from_numpy(x, True)
        cg, cb, cw = orc.Tensor.from_numpy(g, True), orc.Tensor.from_numpy(b, True), orc.Tensor.from_numpy(W, True)
        lab = orc.Tensor.from_numpy(labels)
        t0 = time.perf_counter()
        cx.layernorm(cg, cb, 1e-5).gelu().matmul(cw.transpose(0, 1)).cross_entropy(lab).backward()
        if s >= min(args.warmup, 1):
            durs.append(time.perf_counter() - t0)
    cores = orc.get_threads(); orc.reset_all()
    step_s = float(np.mean(durs)); value = rows / step_s
    sample = "each step = forward + backward of the chain on %d of the %d rows (cost is linear in rows), %d steps timed" % (rows, cfg["N"], len(durs))
    out = {"impl": "reference", "metric": "fused-op fwd+bwd rows/s", "value": value, "unit": "rows/s", "n_gpus": args.gpus, "steps": args.steps,
           "warmup": args.warmup, "steps_timed": len(durs), "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic", "config": {"workload": args.workload, "rows": rows, "C": cfg["C"], "V": cfg["V"]},
           "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": "port", "sample": sample},
           "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(out), flush=True)


def read_profile(vb, L, C, steps, pk, clocks_mhz):
    """Per-family kernel figures from the library's event records: (kernels, gemm_shapes)."""
    buf = C.create_string_buffer(1 << 16)
    vb.vb_check(L.vb_profile_families(buf, 1 << 16))
    acc, gemm_shapes = {}, {}                              # family -> [ms, launches, units, dense units]
    for name in [f for f in buf.value.decode().split(",") if f]:
        t, n, u, du = C.c_double(0), C.c_int64(0), C.c_double(0), C.c_double(0)
        vb.vb_check(L.vb_profile_read(name.encode(), C.byref(t), C.byref(n), C.byref(u), C.byref(du)))
        if n.value == 0:
            continue
        fam = name
        if name.startswith("gemm_tc M"):                 # "gemm_tc M.. N.. K.. nb.. a. b. bn.. sk.. [streamk]": one family, shapes kept aside
            fam = "gemm_tc" if " nb1 " in name else "gemm_tc_batched"
            gemm_shapes[name[len("gemm_tc "):]] = {"launches_per_step": n.value / steps, "us_per_launch": 1e3 * t.value / n.value,
                                                   "tflops": u.value / (t.value * 1e-3) / 1e12 if t.value > 0 else 0.0}
        a = acc.setdefault(fam, [0.0, 0, 0.0, 0.0])
        a[0] += t.value; a[1] += n.value; a[2] += u.value; a[3] += du.value
    kernels = {}
    tf32_useful = TF32_PEAK["tflops_sustained"] / 3.0
    for fam, (t, n, u, du) in acc.items():
        tensor = fam.startswith("gemm") or fam.startswith("attn_fused") or fam.startswith("conv_igemm")
        rate = u / (t * 1e-3) if t > 0 else 0.0
        k = {"launches_per_step": n / steps, "ms_per_step": t / steps, "bound": "tensor" if tensor else "hbm",
             "achieved": rate / 1e12 if tensor else rate / 1e9, "unit": "TFLOP/s" if tensor else "GB/s"}
        if tensor:
            # FP32-accurate products issue three TF32 MMAs each: the useful-flop ceiling is the measured TF32 rate / 3
            k["frac"] = k["achieved"] / tf32_useful
            k["frac_of_bf16_peak"] = k["achieved"] / pk["bf16_tflops_sustained"]
        else:
            k["frac"] = k["achieved"] / pk["hbm_gbs"]
        if du > u * 1.0001:                             # the launches skipped part of the dense problem (causal attention)
            k["dense_equivalent"] = (du / (t * 1e-3)) / (1e12 if tensor else 1e9) if t > 0 else 0.0
        if clocks_mhz:
            k["mcycles_per_step"] = k["ms_per_step"] * clocks_mhz      # time x median SM MHz of this pass: compares runs under different power caps
        kernels[fam] = k
    return kernels, gemm_shapes


def other_workload_lines(vb, L, C, torch, stream, pk, local):
    """Driver-run records for the configurations that are not the headline: config 2 (the fused-op backward chain at
    N = 8192 rows) and config 4 (the conv net step), a few steps each after the timed region of the main workload."""
    from vearo_b200 import modelspec as ms
    out = {}

    def run(name, make, steps=5):
        fn, units, unit = make()
        for i in range(3):
            fn(i)
        vb.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as ck:
            with torch.cuda.stream(stream):
                e0.record()
            for i in range(steps):
                fn(i)
            with torch.cuda.stream(stream):
                e1.record()
            vb.sync(); torch.cuda.synchronize()
        ms_step = e0.elapsed_time(e1) / steps
        vb.vb_check(L.vb_profile_reset()); vb.vb_check(L.vb_profile_enable(1))
        for i in range(2):
            fn(i)
        vb.sync(); vb.vb_check(L.vb_profile_enable(0))
        kernels, _ = read_profile(vb, L, C, 2, pk, None)
        vb.vb_check(L.vb_profile_reset())
        out[name] = {"value": units / (ms_step * 1e-3), "unit": unit, "ms_per_step": ms_step, "steps": steps, "kernels": kernels,
                     "clocks": ck.summary()}

    def fused_op():
        c = WORKLOADS["fused-op"]
        x, g, b, W, labels = ms.microbench_inputs(N=c["N"], C=c["C"], V=c["V"])
        m = vb.FusedOpBench(c["C"], c["V"]); m.load([g, b, W])
        gx, lab = vb.Tensor.from_numpy(x, True), vb.Tensor.from_numpy(labels)
        keep = []

        def fn(i):
            vb.zero_gradients(); vb.reset_active_tape()
            l = m.loss(gx, lab); l.backward()
            keep[:] = [l, m]
        return fn, c["N"], "rows/s"

    def convnet():
        c = WORKLOADS["convnet"]
        m = vb.ConvNet(list(c["channels"]), c["classes"]); m.load(ms.convnet_params(c["channels"], c["classes"]))
        opt = vb.SGD(m.parameters(), c["lr"], c["momentum"], 0.0)
        x, y = ms.convnet_batch(c["micro_batch"], c["hw"], c["classes"])
        xr, yr = vb.Tensor.from_numpy(x), vb.Tensor.from_numpy(y)
        keep = []

        def fn(i):
            keep[:] = [m.train_step_resident(opt, xr, yr, 0.0), opt]
        return fn, c["micro_batch"], "images/s"
    run("fused-op", fused_op)
    run("convnet", convnet, steps=20)
    return out


def measure_tf32_peak():
    """torch.matmul with TF32 allowed on 8192^3, the way MEASURED_PEAKS.json measures bf16: best of 10 (burst) and back to
    back for 4 s (sustained), SM clock sampled.  Prints one JSON line (the figure recorded in TF32_PEAK)."""
    import torch
    torch.backends.cuda.matmul.allow_tf32 = True
    n = 8192
    a = torch.randn(n, n, device="cuda"); b = torch.randn(n, n, device="cuda")
    for _ in range(3):
        torch.matmul(a, b)
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); torch.matmul(a, b); e1.record(); torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    with ClockSampler(0) as ck:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter(); reps = 0
        e0.record()
        while time.perf_counter() - t0 < 4.0:
            for _ in range(10):
                torch.matmul(a, b)
            reps += 10
            torch.cuda.synchronize()
        e1.record(); torch.cuda.synchronize()
    sustained_ms = e0.elapsed_time(e1) / reps
    fl = 2.0 * n ** 3
    print(json.dumps({"tf32_tflops_burst": fl / (best * 1e-3) / 1e12, "tf32_tflops_sustained": fl / (sustained_ms * 1e-3) / 1e12,
                      "how": "torch.matmul f32 with allow_tf32, 8192^3, best of 10 / back to back for 4 s", "clocks": ck.summary()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gpt-small", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-workloads", action="store_true", help="skip the short fused-op and convnet records appended to the default 1-GPU line")
    ap.add_argument("--checkpoint-blocks", action="store_true", help="GPT workloads: every transformer block under activation checkpointing")
    ap.add_argument("--adamw8bit", action="store_true", help="GPT workloads: AdamW with block-wise int8 moments")
    ap.add_argument("--profile-steps", type=int, default=2)
    ap.add_argument("--measure-tf32-peak", action="store_true", help="measure the dense TF32 rate of torch.matmul on this GPU and exit")
    args = ap.parse_args()
    if args.measure_tf32_peak:
        return measure_tf32_peak()
    cfg = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, cfg, rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))

    import ctypes as C
    import torch
    import vearo_b200 as vb
    from vearo_b200 import modelspec as ms

    os.environ.setdefault("VB200_PROF_SHAPES", "1")      # the profiling pass keeps GEMM launches apart by shape
    torch.cuda.set_device(local)
    vb.init(local)
    L = vb.lib()
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        uid = (C.c_uint8 * 128)()
        if rank == 0:
            vb.vb_check(L.vb_dp_unique_id(uid), "vb_dp_unique_id")
        t = torch.tensor(list(uid), dtype=torch.uint8, device="cuda")
        dist.broadcast(t, 0)
        uid = (C.c_uint8 * 128)(*t.cpu().tolist())
        vb.vb_check(L.vb_dp_init(rank, world, uid), "vb_dp_init")

    stream_ptr = C.c_void_p()
    vb.vb_check(L.vb_stream(C.byref(stream_ptr)))
    stream = torch.cuda.ExternalStream(stream_ptr.value)

    def barrier():
        vb.sync()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    kind = cfg.get("kind", "gpt")
    convnet, fused_op = kind == "convnet", kind == "fused-op"
    opt = None
    if convnet:
        B = cfg["micro_batch"]; T = V = 0
        model = vb.ConvNet(list(cfg["channels"]), cfg["classes"])
        model.load(ms.convnet_params(cfg["channels"], cfg["classes"]))                  # identical on every rank
        opt = vb.SGD(model.parameters(), cfg["lr"], cfg["momentum"], 0.0, data_parallel=world > 1)
        batches = [ms.convnet_batch(B, cfg["hw"], cfg["classes"], seed=1000 * rank + i) for i in range(4)]
        units_per_rank, unit, metric = B, "images/s", "ConvNet fwd+bwd+SGD images/s"
    elif fused_op:
        B = cfg["N"]; T = V = 0
        x, g, b, W, labels = ms.microbench_inputs(N=cfg["N"], C=cfg["C"], V=cfg["V"])
        model = vb.FusedOpBench(cfg["C"], cfg["V"]); model.load([g, b, W])
        batches = [(x, labels)]
        units_per_rank, unit, metric = B, "rows/s", "fused-op fwd+bwd rows/s"
    else:
        B, T, V = cfg["micro_batch"], cfg["T"], cfg["vocab"]
        model = vb.SimpleGPT(V, T, cfg["d"], cfg["heads"], cfg["layers"], cfg["ff"])
        model.load(ms.gpt_params(V, T, cfg["d"], cfg["layers"], cfg["ff"], seed=0))      # identical on every rank
        if args.checkpoint_blocks: model.set_checkpointing(True)
        Opt = vb.AdamW8bit if args.adamw8bit else vb.AdamW
        opt = Opt(model.parameters(), cfg["lr"], 0.9, 0.999, 1e-8, cfg["wd"], data_parallel=world > 1)
        batches = [ms.gpt_batch(V, B, T, seed=1000 * rank + i) for i in range(4)]      # per-rank data
        units_per_rank, unit, metric = B * T, "tokens/s", "GPT-small fwd+bwd+AdamW tokens/s"
    n_params = sum(int(np.prod(p.shape)) for p in model.parameters())
    resident = [(vb.Tensor.from_numpy(a, fused_op), vb.Tensor.from_numpy(b)) for a, b in batches]
    pinned = []
    for a, b in batches:
        pa = torch.empty(a.shape, dtype=torch.float32, pin_memory=True); pa.numpy()[:] = a
        pb = torch.empty(b.shape, dtype=torch.float32, pin_memory=True); pb.numpy()[:] = b
        pinned.append((pa, pb))

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record()
        for i in range(steps):
            fn(i)
        with torch.cuda.stream(stream):
            e1.record()
        barrier()
        ms_ = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if dist is not None:
            dist.all_reduce(ms_, op=dist.ReduceOp.MAX)
        return float(ms_.item())

    keep = []

    def step_resident(i):
        x, y = resident[i % len(resident)]
        if fused_op:                        # config 2 has no optimizer: forward + backward of the chain
            vb.zero_gradients(); vb.reset_active_tape()
            l = model.loss(x, y); l.backward()
            keep.append(l)
        else:
            keep.append(model.train_step_resident(opt, x, y, cfg["clip"]))
        if len(keep) > 2:
            keep.pop(0)

    losses = []

    def step_host(i):
        a, b = pinned[i % len(pinned)]
        if fused_op:
            vb.zero_gradients(); vb.reset_active_tape()
            l = model.loss(vb.Tensor.from_numpy(a.numpy(), True), vb.Tensor.from_numpy(b.numpy())); l.backward()
            losses.append(float(l.numpy()[0]))
        else:
            losses.append(model.train_step(opt, a.numpy(), b.numpy(), cfg["clip"])[0])

    for i in range(max(args.warmup, 3)):
        step_resident(i)
    launches0 = C.c_int64(0); L.vb_launch_count(C.byref(launches0))
    with ClockSampler(local) as clocks:
        total_ms = timed(step_resident, args.steps)
    launches1 = C.c_int64(0); L.vb_launch_count(C.byref(launches1))
    vb.check_errors()
    tokens = world * units_per_rank
    ms_per_step = total_ms / args.steps
    value = tokens / (ms_per_step * 1e-3)

    step_host(0)
    e2e_ms = timed(step_host, args.steps) / args.steps
    e2e_value = tokens / (e2e_ms * 1e-3)

    # data-parallel evidence: after the same number of steps from the same start, every rank must hold bit-identical weights
    replicas_identical = None
    if dist is not None:
        import zlib
        crc = 0
        for prm in model.parameters():
            crc = zlib.crc32(prm.numpy().tobytes(), crc)
        cr = torch.tensor([crc], dtype=torch.int64, device="cuda")
        lo, hi = cr.clone(), cr.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        replicas_identical = bool(lo.item() == hi.item())

    # untimed profiling pass: per-family kernel time from CUDA events on the compute stream
    pk = peaks()
    kernels, roofline, gemm_shapes, prof_clocks = {}, None, {}, None
    if args.profile_steps > 0:          # every rank runs the steps (they contain collectives); rank 0 reads
        vb.vb_check(L.vb_profile_reset()); vb.vb_check(L.vb_profile_enable(1))
        with ClockSampler(local) as pclk:
            for i in range(max(args.profile_steps, 2)):
                step_resident(i)
            vb.sync()
        vb.vb_check(L.vb_profile_enable(0))
        prof_clocks = pclk.summary()
    if rank == 0 and args.profile_steps > 0:
        kernels, gemm_shapes = read_profile(vb, L, C, max(args.profile_steps, 2), pk, prof_clocks.get("sm_mhz"))
        vb.vb_check(L.vb_profile_reset())
        if kernels:
            dom = max(kernels, key=lambda k: kernels[k]["ms_per_step"])
            k = kernels[dom]
            tensor = k["bound"] == "tensor"
            roofline = {"kernel": dom, "bound": k["bound"], "achieved": k["achieved"], "unit": k["unit"],
                        "peak": pk["bf16_tflops_sustained"] if tensor else pk["hbm_gbs"], "peak_source": pk["source"],
                        "frac": k["achieved"] / (pk["bf16_tflops_sustained"] if tensor else pk["hbm_gbs"]),
                        "traffic": None, "share_of_step": k["ms_per_step"] / ms_per_step}
            if tensor:
                # the kernel is an FP32-accurate 3xTF32 product: three TF32 MMAs per useful multiply-add, so its own ceiling is
                # the measured dense TF32 rate / 3 (`frac` above is against the bf16 figure of MEASURED_PEAKS.json)
                roofline["peak_tf32_measured"] = TF32_PEAK
                roofline["peak_3xtf32_useful"] = TF32_PEAK["tflops_sustained"] / 3.0
                roofline["frac_of_3xtf32_peak"] = k["achieved"] / roofline["peak_3xtf32_useful"]
            if dom == "gemm_tc" and kind == "gpt":
                roofline.update(TRAFFIC_FROM_PROFILE)

    other = None
    if rank == 0 and world == 1 and args.workload == "gpt-small" and not args.no_other_workloads:
        del keep[:]
        other = other_workload_lines(vb, L, C, torch, stream, pk, local)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        from oracle import build as ob
        ob.build()
        if convnet:
            durs, cores = cpu_convnet_step_time(cfg, 16, 1, 0)
            cpu = {"value": 16 / durs[0], "unit": unit, "cores": cores, "kind": "port",
                   "sample": "one fwd + bwd + SGD step on 16 images (%.1f s); cost is linear in images" % durs[0]}
        elif fused_op:
            cpu = None
        else:
            tps, desc, cores, _, _ = cpu_baseline_sample(cfg)
            cpu = {"value": tps, "unit": unit, "cores": cores, "kind": "port", "sample": desc}
    if convnet:
        config = {"workload": args.workload, "channels": list(cfg["channels"]), "classes": cfg["classes"], "image": [3, cfg["hw"], cfg["hw"]],
                  "micro_batch_per_gpu": B, "global_batch": world * B, "params": n_params,
                  "optimizer": "SGD lr %g momentum %g" % (cfg["lr"], cfg["momentum"]), "parallelism": "dp%d" % world,
                  "matmul_precision": "fp32 (convolutions on the 3xTF32 tensor-core GEMM)",
                  "l2": "activations of one step (about 1 GB) exceed the 126 MB L2"}
        h2d = int(world * (B * 3 * cfg["hw"] * cfg["hw"] + B) * 4)
    elif fused_op:
        config = {"workload": args.workload, "rows": cfg["N"], "C": cfg["C"], "V": cfg["V"], "params": n_params,
                  "chain": "LayerNorm -> GELU -> Linear C->V (no bias) -> cross-entropy; forward + backward (dX, dW, dgamma, dbeta)",
                  "l2": "the logits alone (1.65 GB) exceed the 126 MB L2"}
        h2d = int(world * (cfg["N"] * cfg["C"] + cfg["N"]) * 4)
    else:
        config = {"workload": args.workload, "n_layer": cfg["layers"], "n_head": cfg["heads"], "d_model": cfg["d"], "d_ff": cfg["ff"],
                  "vocab": V, "seq_len": T, "micro_batch_per_gpu": B, "global_batch": world * B, "params": n_params,
                  "optimizer": "%s lr %g wd %g, clip %g" % ("AdamW8bit" if args.adamw8bit else "AdamW", cfg["lr"], cfg["wd"], cfg["clip"]),
                  "activation_checkpointing": bool(args.checkpoint_blocks), "parallelism": "dp%d" % world,
                  "matmul_precision": "fp32 (3xTF32 on tensor cores where the tensor-core kernel applies, exact fp32 FMA otherwise)",
                  "l2": "working set per step (weights, activations, optimizer state: several GB) exceeds the 126 MB L2 many times over"}
        h2d = int(world * 2 * B * T * 4)
    tc = C.c_int64(0); L.vb_tc_launch_count(C.byref(tc))
    out = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config,
        "useful_tflops": flops_per_token(cfg) * tokens / (ms_per_step * 1e-3) / 1e12 if kind == "gpt" else None,
        "e2e": {"value": e2e_value, "unit": unit, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(world * (4 if fused_op else 8))},
        "gpu_launches": int(launches1.value - launches0.value),
        "tensor_core_gemm_launches_total": int(tc.value),
        "device_memory": vb.memory_stats(),
        "clocks": clocks.summary(), "profile_pass_clocks": prof_clocks,
        "replicas_identical": replicas_identical,
        "dp_gradients_registered": (opt.gradients_registered() if (dist is not None and opt is not None) else None),
        "roofline": roofline, "kernels": kernels, "gemm_shapes": gemm_shapes, "cpu_baseline": cpu,
        "other_workloads": other,
        "last_loss": losses[-1] if losses else None,
    }
    print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

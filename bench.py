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
    # a seconds-long case for plumbing checks
    "gpt-tiny": dict(vocab=512, T=64, d=128, heads=4, layers=2, ff=512, micro_batch=4, lr=6e-4, wd=0.1, clip=1.0),
}


# ncu, one launch of k_gemm_tc on 8192x768 . 768x3072 (dram__bytes_read.sum + dram__bytes_write.sum); the operands and the
# result of that launch are 25.2 + 9.4 + 100.7 MB: every operand byte is read once, part of the result is still in L2 at exit
NCU_TRAFFIC_GEMM_FC1 = {"traffic": 82.7e6, "traffic_unit": "bytes per launch", "traffic_launch": "M8192 N3072 K768 (GPT-small fc1 forward)",
                        "traffic_algorithmic": 135.3e6}


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
    from tests import modelspec as ms
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
    from tests import modelspec as ms
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
    built here: no cargo/rustc), all host threads the reference itself would use."""
    if rank != 0:
        return
    if cfg.get("kind") == "convnet":
        return run_reference_convnet(args, cfg)
    from oracle import build as ob
    ob.build()
    from oracle import oracle as orc
    from oracle import models as om
    from tests import modelspec as ms
    total = args.steps + args.warmup
    T = cfg["T"] if total <= 12 else min(cfg["T"], 256)
    tps0, desc, cores, t1, block = cpu_baseline_sample(cfg, T)          # also yields the per-block time
    # timed steps: each step is one pass of the 1-block sample; the other blocks are added from `block`
    params = ms.gpt_params(cfg["vocab"], T, cfg["d"], 1, cfg["ff"])
    m = om.SimpleGPT(params, cfg["d"], cfg["heads"], 1)
    opt = orc.AdamW(m.parameters(), cfg["lr"], 0.9, 0.999, 1e-8, cfg["wd"])
    ids, tg = ms.gpt_batch(cfg["vocab"], 1, T)
    durs = []
    for s in range(total):
        t0 = time.perf_counter()
        orc.zero_gradients(); orc.reset_active_tape()
        _, loss = m.forward(orc.Tensor.from_numpy(ids), orc.Tensor.from_numpy(tg))
        loss.backward(); orc.clip_grad_norm(m.parameters(), cfg["clip"]); opt.step()
        if s >= args.warmup:
            durs.append(time.perf_counter() - t0 + (cfg["layers"] - 1) * block)
    step_s = float(np.mean(durs))
    value = T / step_s
    sample = ("each step = one T=%d sequence through a 1-block model (measured) + %d x the per-block time %.2f s "
              "(2-block minus 1-block, measured once before the timed steps)" % (T, cfg["layers"] - 1, block))
    if T != cfg["T"]:
        sample += "; T shortened from %d to keep the run within minutes (attention cost per token under-counted, which favours this arm)" % cfg["T"]
    out = {"impl": "reference", "metric": "GPT-small fwd+bwd+AdamW tokens/s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": args.workload, **{k: cfg[k] for k in ("vocab", "T", "d", "heads", "layers", "ff")}, "micro_batch": 1},
           "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
           "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gpt-small", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--checkpoint-blocks", action="store_true", help="GPT workloads: every transformer block under activation checkpointing")
    ap.add_argument("--adamw8bit", action="store_true", help="GPT workloads: AdamW with block-wise int8 moments")
    ap.add_argument("--profile-steps", type=int, default=2)
    args = ap.parse_args()
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
    from tests import modelspec as ms

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

    convnet = cfg.get("kind") == "convnet"
    B = cfg["micro_batch"]
    if convnet:
        T = V = 0
        model = vb.ConvNet(list(cfg["channels"]), cfg["classes"])
        model.load(ms.convnet_params(cfg["channels"], cfg["classes"]))                  # identical on every rank
        opt = vb.SGD(model.parameters(), cfg["lr"], cfg["momentum"], 0.0, data_parallel=world > 1)
        batches = [ms.convnet_batch(B, cfg["hw"], cfg["classes"], seed=1000 * rank + i) for i in range(4)]
        units_per_rank, unit = B, "images/s"
    else:
        T, V = cfg["T"], cfg["vocab"]
        model = vb.SimpleGPT(V, T, cfg["d"], cfg["heads"], cfg["layers"], cfg["ff"])
        model.load(ms.gpt_params(V, T, cfg["d"], cfg["layers"], cfg["ff"], seed=0))      # identical on every rank
        if args.checkpoint_blocks: model.set_checkpointing(True)
        Opt = vb.AdamW8bit if args.adamw8bit else vb.AdamW
        opt = Opt(model.parameters(), cfg["lr"], 0.9, 0.999, 1e-8, cfg["wd"], data_parallel=world > 1)
        batches = [ms.gpt_batch(V, B, T, seed=1000 * rank + i) for i in range(4)]      # per-rank data
        units_per_rank, unit = B * T, "tokens/s"
    n_params = sum(int(np.prod(p.shape)) for p in model.parameters())
    resident = [(vb.Tensor.from_numpy(a), vb.Tensor.from_numpy(b)) for a, b in batches]
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
        keep.append(model.train_step_resident(opt, x, y, cfg["clip"]))
        if len(keep) > 2:
            keep.pop(0)

    losses = []

    def step_host(i):
        a, b = pinned[i % len(pinned)]
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

    # untimed profiling pass: per-family kernel time from CUDA events on the compute stream
    pk = peaks()
    kernels, roofline = {}, None
    if args.profile_steps > 0:          # every rank runs the steps (they contain collectives); rank 0 reads
        vb.vb_check(L.vb_profile_reset()); vb.vb_check(L.vb_profile_enable(1))
        for i in range(args.profile_steps):
            step_resident(i)
        vb.sync(); vb.vb_check(L.vb_profile_enable(0))
    gemm_shapes = {}
    if rank == 0 and args.profile_steps > 0:
        buf = C.create_string_buffer(1 << 16)
        vb.vb_check(L.vb_profile_families(buf, 1 << 16))
        acc = {}                                         # family -> [ms, launches, units]
        for name in [f for f in buf.value.decode().split(",") if f]:
            t, n, u = C.c_double(0), C.c_int64(0), C.c_double(0)
            vb.vb_check(L.vb_profile_read(name.encode(), C.byref(t), C.byref(n), C.byref(u)))
            if n.value == 0:
                continue
            fam = name
            if name.startswith("gemm_tc M"):             # "gemm_tc M.. N.. K.. nb.. a. b. bn.. sk.. [streamk]": one family, shapes kept aside
                fam = "gemm_tc" if " nb1 " in name else "gemm_tc_batched"
                gemm_shapes[name[len("gemm_tc "):]] = {"launches_per_step": n.value / args.profile_steps, "us_per_launch": 1e3 * t.value / n.value,
                                                       "tflops": u.value / (t.value * 1e-3) / 1e12 if t.value > 0 else 0.0}
            a = acc.setdefault(fam, [0.0, 0, 0.0])
            a[0] += t.value; a[1] += n.value; a[2] += u.value
        for fam, (t, n, u) in acc.items():
            is_gemm = fam.startswith("gemm")
            rate = u / (t * 1e-3) if t > 0 else 0.0
            kernels[fam] = {"launches_per_step": n / args.profile_steps, "ms_per_step": t / args.profile_steps,
                            "bound": "tensor" if is_gemm else "hbm",
                            "achieved": rate / 1e12 if is_gemm else rate / 1e9, "unit": "TFLOP/s" if is_gemm else "GB/s",
                            "frac": (rate / 1e12 / pk["bf16_tflops_sustained"]) if is_gemm else (rate / 1e9 / pk["hbm_gbs"])}
        vb.vb_check(L.vb_profile_reset())
        if kernels:
            dom = max(kernels, key=lambda k: kernels[k]["ms_per_step"])
            k = kernels[dom]
            roofline = {"kernel": dom, "bound": k["bound"], "achieved": k["achieved"], "peak": pk["bf16_tflops_sustained"] if k["bound"] == "tensor" else pk["hbm_gbs"],
                        "unit": k["unit"], "frac": k["frac"], "traffic": None, "peak_source": pk["source"],
                        "share_of_step": k["ms_per_step"] / ms_per_step}
            if k["bound"] == "tensor":
                # 3xTF32: three TF32 MMAs per useful product and TF32 runs at half the bf16 rate
                roofline["peak_3xtf32_useful"] = pk["bf16_tflops_sustained"] / 6.0
                roofline["frac_of_3xtf32_peak"] = k["achieved"] / roofline["peak_3xtf32_useful"]
            if dom == "gemm_tc" and not convnet:
                # DRAM bytes of ONE launch, from the ncu capture of the fc1-shaped product (profiles/gemm_tc_fc1_and_dw.md);
                # `achieved` above averages all launches of the kernel, whose shapes differ
                roofline.update(NCU_TRAFFIC_GEMM_FC1)

    if rank != 0:
        return
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        from oracle import build as ob
        ob.build()
        if convnet:
            durs, cores = cpu_convnet_step_time(cfg, 16, 1, 0)
            cpu = {"value": 16 / durs[0], "unit": unit, "cores": cores, "kind": "port",
                   "sample": "one fwd + bwd + SGD step on 16 images (%.1f s); cost is linear in images" % durs[0]}
        else:
            tps, desc, cores, _, _ = cpu_baseline_sample(cfg)
            cpu = {"value": tps, "unit": unit, "cores": cores, "kind": "port", "sample": desc}
    if convnet:
        config = {"workload": args.workload, "channels": list(cfg["channels"]), "classes": cfg["classes"], "image": [3, cfg["hw"], cfg["hw"]],
                  "micro_batch_per_gpu": B, "global_batch": world * B, "params": n_params,
                  "optimizer": "SGD lr %g momentum %g" % (cfg["lr"], cfg["momentum"]), "parallelism": "dp%d" % world,
                  "matmul_precision": "fp32 (convolutions unfolded onto the 3xTF32 tensor-core GEMM)",
                  "l2": "activations of one step (about 1 GB) exceed the 126 MB L2"}
        h2d = int(world * (B * 3 * cfg["hw"] * cfg["hw"] + B) * 4)
    else:
        config = {"workload": args.workload, "n_layer": cfg["layers"], "n_head": cfg["heads"], "d_model": cfg["d"], "d_ff": cfg["ff"],
                  "vocab": V, "seq_len": T, "micro_batch_per_gpu": B, "global_batch": world * B, "params": n_params,
                  "optimizer": "%s lr %g wd %g, clip %g" % ("AdamW8bit" if args.adamw8bit else "AdamW", cfg["lr"], cfg["wd"], cfg["clip"]),
                  "activation_checkpointing": bool(args.checkpoint_blocks), "parallelism": "dp%d" % world,
                  "matmul_precision": "fp32 (3xTF32 on tensor cores where the tensor-core kernel applies, exact fp32 FMA otherwise)",
                  "l2": "working set per step (weights, activations, optimizer state: several GB) exceeds the 126 MB L2 many times over"}
        h2d = int(world * 2 * B * T * 4)
    out = {
        "metric": "ConvNet fwd+bwd+SGD images/s" if convnet else "GPT-small fwd+bwd+AdamW tokens/s", "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config,
        "useful_tflops": None if convnet else flops_per_token(cfg) * tokens / (ms_per_step * 1e-3) / 1e12,
        "e2e": {"value": e2e_value, "unit": unit, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(world * 8)},
        "gpu_launches": int(launches1.value - launches0.value),
        "device_memory": vb.memory_stats(),
        "clocks": clocks.summary(),
        "roofline": roofline, "kernels": kernels, "gemm_shapes": gemm_shapes, "cpu_baseline": cpu,
        "last_loss": losses[-1] if losses else None,
    }
    print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

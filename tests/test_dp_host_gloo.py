"""The host side of the data-parallel path at world size 2, on CPU with the gloo backend.

What runs here: the gradient-bucket plan of the library (pure host arithmetic, shared by every rank), the
order in which buckets are released during a reverse walk over the parameters, and a bucket-by-bucket
allreduce of a flat gradient arena.  The collective is gloo instead of NCCL and the gradients are NumPy
arrays; the plan, the ordering rule and the 1/world scaling are the ones the CUDA path uses.
A rank that never arrives is made on the host: the survivor's collective ends with an error after a short
process-group timeout (no GPU is involved).
"""
import datetime
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

SIZES = [38633472 // 64, 786432 // 64] + [768, 768, 589824 // 16, 768] * 6 + [768, 768, 38633472 // 64]   # GPT-shaped, scaled down


def _worker(rank, world, port, q, mode):
    import torch
    import torch.distributed as dist
    import vearo_b200 as vb
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5 if mode == "missing" else 60))
    try:
        plan = vb.plan_buckets(SIZES, 1 << 18)
        if mode == "missing":
            if rank == 1:
                q.put((rank, "left")); return            # leaves between steps, nothing in flight
            t = torch.zeros(4)
            try:
                dist.all_reduce(t)
                q.put((rank, "no error"))
            except Exception as e:                        # the short timeout ends the collective with an error
                q.put((rank, "error: " + type(e).__name__))
            return
        rng = np.random.default_rng(100 + rank)           # per-rank data
        grads = [rng.standard_normal(n).astype(np.float32) for n in SIZES]
        arena = np.zeros(plan["total"], np.float32)
        pending = [0] * len(plan["buckets"])
        for b in plan["bucket_of"]:
            pending[b] += 1
        issued = []
        for i in reversed(range(len(SIZES))):             # gradients become final in reverse parameter order
            o = plan["param_offset"][i]
            arena[o:o + SIZES[i]] = grads[i]
            b = plan["bucket_of"][i]
            pending[b] -= 1
            if pending[b] == 0:
                off, num = plan["buckets"][b]
                t = torch.from_numpy(arena[off:off + num])
                dist.all_reduce(t)                         # sum; 1/world is applied by the optimizer
                issued.append(b)
        arena *= 1.0 / world
        q.put((rank, plan, issued, arena, grads))
    finally:
        dist.destroy_process_group()


def _spawn(mode, port):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, mode)) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    return sorted(out, key=lambda x: x[0])


def test_bucket_plan_properties():
    import vearo_b200 as vb
    plan = vb.plan_buckets(SIZES, 1 << 18)
    offs, buckets = plan["param_offset"], plan["buckets"]
    assert all(o % 4 == 0 for o in offs) and offs == sorted(offs)
    # buckets tile the arena exactly, last parameters first
    assert buckets[0][0] + buckets[0][1] == plan["total"] and buckets[-1][0] == 0
    for (o0, n0), (o1, n1) in zip(buckets, buckets[1:]):
        assert o1 + n1 == o0
    assert all(n >= (1 << 18) for _, n in buckets[:-1])
    assert vb.plan_buckets([], 16)["buckets"] == [] or vb.plan_buckets([], 16)["total"] == 0
    one = vb.plan_buckets([5], 1 << 20)
    assert one["buckets"] == [(0, 8)] and one["total"] == 8


def test_bucket_plan_at_the_headline_model_sizes():
    """GPT-small's parameter list (token and positional tables, 12 blocks of 16 tensors, the final LayerNorm, the untied head:
    163,109,376 parameters) cut at the default bucket size of 128 MiB: the head's gradient -- the first to become final in the
    backward pass -- is reduced first and alone, and the token table, final only with the last backward kernel, sits in the
    last bucket."""
    import vearo_b200 as vb
    d, ff, V, T = 768, 3072, 50304, 1024
    block = [d, d, d * d, d, d * d, d, d * d, d, d * d, d, d, d, ff * d, ff, d * ff, d]
    sizes = [V * d, T * d] + block * 12 + [d, d, V * d]
    assert sum(sizes) == 163109376
    plan = vb.plan_buckets(sizes, (128 << 20) // 4)
    buckets = plan["buckets"]
    assert plan["total"] == 163109376 and sum(n for _, n in buckets) == plan["total"]
    assert buckets[0] == (plan["total"] - V * d, V * d)                  # the head alone: 154.5 MB >= 128 MiB
    assert buckets[-1][0] == 0 and buckets[-1][1] >= V * d + T * d       # token + positional tables (+ the rest of block 0)
    assert all(n * 4 >= (128 << 20) for _, n in buckets[:-1])
    assert 4 <= len(buckets) <= 6


def test_two_ranks_bucketed_allreduce_gloo():
    r0, r1 = _spawn("reduce", 29731)
    assert r0[1] == r1[1]                                   # identical plan on both ranks
    assert r0[2] == r1[2] == list(range(len(r0[1]["buckets"])))   # buckets released in the same, fixed order
    assert (r0[3].view(np.uint32) == r1[3].view(np.uint32)).all()   # replicas hold identical reduced gradients
    plan = r0[1]
    for i, n in enumerate(SIZES):
        o = plan["param_offset"][i]
        np.testing.assert_allclose(r0[3][o:o + n], (r0[4][i] + r1[4][i]) / 2, rtol=1e-6, atol=1e-7)


def test_missing_rank_ends_in_an_error_not_a_hang():
    r0, r1 = _spawn("missing", 29741)
    assert r1[1] == "left"
    assert r0[1].startswith("error"), r0

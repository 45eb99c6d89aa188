"""One data-parallel rank (child process of tests/test_gpu_dp.py): trains a tiny GPT on its shard."""
import ctypes as C
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, out_dir, steps = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], int(sys.argv[4])
    mode = sys.argv[5] if len(sys.argv) > 5 else "train"
    import vearo_b200 as vb
    from vearo_b200 import modelspec as ms
    vb.init(rank)
    L = vb.lib()
    uid = (C.c_uint8 * 128)()
    uid_path = os.path.join(out_dir, "nccl_uid.bin")
    if world > 1:
        if rank == 0:
            vb.vb_check(L.vb_dp_unique_id(uid), "vb_dp_unique_id")
            with open(uid_path + ".tmp", "wb") as f:
                f.write(bytes(uid))
            os.rename(uid_path + ".tmp", uid_path)
        else:
            t0 = time.time()
            while not os.path.exists(uid_path):
                if time.time() - t0 > 60:
                    raise SystemExit("rank 0 never published the NCCL id")
                time.sleep(0.05)
            uid = (C.c_uint8 * 128)(*open(uid_path, "rb").read())
        vb.vb_check(L.vb_dp_init(rank, world, uid), "vb_dp_init")
    vocab, T, d, heads, layers, ff, B = 96, 16, 32, 4, 2, 64, 4
    model = vb.SimpleGPT(vocab, T, d, heads, layers, ff)
    model.load(ms.gpt_params(vocab, T, d, layers, ff, seed=5, std=0.2))
    per = B // world
    if mode == "partial":
        # A parameter that receives gradient on rank 0 only, and a second backward pass before the step.  Every rank must apply the
        # same update to the lone parameter (its reduced gradient, 1/world of rank 0's), and the repeated backward must be refused.
        extra = vb.Tensor.from_numpy(np.linspace(-1, 1, 40).astype(np.float32), True)
        params = model.parameters() + [extra]
        opt = vb.AdamW(params, 1e-2, 0.9, 0.999, 1e-8, 0.0, data_parallel=world > 1)
        for s in range(steps):
            ids, tg = ms.gpt_batch(vocab, B, T, seed=s)
            sl = slice(rank * per, (rank + 1) * per)
            vb.zero_gradients(); vb.reset_active_tape()
            loss = model.loss(vb.Tensor.from_numpy(ids[sl]), vb.Tensor.from_numpy(tg[sl]))
            if rank == 0:
                loss = loss.add(extra.mul(extra).sum(0, False).reshape([1]))
            loss.backward()
            opt.clip_and_step(1.0)
        refused = False
        vb.zero_gradients(); vb.reset_active_tape()
        ids, tg = ms.gpt_batch(vocab, B, T, seed=99)
        loss = model.loss(vb.Tensor.from_numpy(ids[:per]), vb.Tensor.from_numpy(tg[:per]))
        loss.backward()
        try:
            model.loss(vb.Tensor.from_numpy(ids[:per]), vb.Tensor.from_numpy(tg[:per])).backward()
        except vb.VearoError as e:
            refused = "twice" in str(e)
        vb.sync()
        weights = {"p%d" % i: p.numpy() for i, p in enumerate(params)}
        np.savez(os.path.join(out_dir, "rank%d.npz" % rank), refused=np.array([int(refused)]), **weights)
        return
    opt = vb.AdamW(model.parameters(), 1e-3, 0.9, 0.999, 1e-8, 0.1, data_parallel=world > 1)
    losses, norms = [], []
    for s in range(steps):
        ids, tg = ms.gpt_batch(vocab, B, T, seed=s)
        sl = slice(rank * per, (rank + 1) * per)
        loss, norm = model.train_step(opt, ids[sl], tg[sl], max_norm=1.0)
        losses.append(loss); norms.append(norm)
    vb.check_errors()
    weights = {"p%d" % i: p.numpy() for i, p in enumerate(model.parameters())}
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), losses=np.array(losses), norms=np.array(norms), **weights)
    if world > 1:
        vb.vb_check(L.vb_dp_shutdown())


if __name__ == "__main__":
    main()

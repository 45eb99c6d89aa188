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
    opt = vb.AdamW(model.parameters(), 1e-3, 0.9, 0.999, 1e-8, 0.1, data_parallel=world > 1)
    per = B // world
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

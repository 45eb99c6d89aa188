"""Generates the small golden fixtures in this folder.

forward_cases.json   eleven NumPy forward cases (elementwise with broadcasting and transposed
                     operands, 2-D and batched matmul, reshape / transpose / permute) with the same
                     inputs the reference's NumPy fixture test_data/oracles.json holds, so that the
                     two files can be compared value for value where the reference tree is present.
backward_cases.npz   float64 NumPy/PyTorch-CPU gradients of every backward arm on small seeded inputs,
                     used as an independent referee for the f32 oracle.

Run:  python tests/golden/make_golden.py
"""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def case(op, inputs, output):
    return {"op": op,
            "inputs": [{"shape": list(x.shape), "data": x.flatten().tolist()} for x in inputs],
            "output": {"shape": list(output.shape), "data": output.flatten().tolist()}}


def forward_cases():
    f = np.float32
    x = np.array([[1, 2, 3], [4, 5, 6]], dtype=f)
    y = np.array([[10, 20, 30], [40, 50, 60]], dtype=f)
    yt = np.array([[10, 20], [30, 40], [50, 60]], dtype=f)
    xb = np.array([[1, 2, 3]], dtype=f)
    yb = np.array([[10], [20]], dtype=f)
    m1 = np.array([[1, 2], [3, 4]], dtype=f)
    m2 = np.array([[5, 6], [7, 8]], dtype=f)
    mb1 = np.arange(1, 13, dtype=f).reshape(2, 2, 3)
    mb2 = np.arange(1, 13, dtype=f).reshape(2, 3, 2)
    p1 = np.arange(1, 7, dtype=f).reshape(1, 2, 3)
    return [
        case("add", [x, y], x + y),
        case("add_transposed", [x.T, yt], x.T + yt),
        case("add_broadcasted", [xb, yb], xb + yb),
        case("sub", [x, y], x - y),
        case("mul", [x, y], x * y),
        case("div", [x, y], x / y),
        case("matmul_2d", [m1, m2], m1 @ m2),
        case("matmul_batched", [mb1, mb2], mb1 @ mb2),
        case("reshape", [x], x.reshape(6)),
        case("transpose", [x], x.T),
        case("permute", [p1], np.transpose(p1, (2, 0, 1))),
    ]


def backward_cases():
    import torch
    torch.manual_seed(0)
    rng = np.random.default_rng(0)
    out = {}
    d = torch.float64

    def t(a, g=True):
        return torch.tensor(a, dtype=d, requires_grad=g)

    # layernorm
    x = rng.standard_normal((5, 12)); w = rng.standard_normal(12); b = rng.standard_normal(12); go = rng.standard_normal((5, 12))
    tx, tw, tb = t(x), t(w), t(b)
    torch.nn.functional.layer_norm(tx, (12,), tw, tb, 1e-5).backward(t(go, False))
    out.update(ln_x=x, ln_w=w, ln_b=b, ln_go=go, ln_gx=tx.grad.numpy(), ln_gw=tw.grad.numpy(), ln_gb=tb.grad.numpy())
    # gelu (tanh form)
    x = rng.standard_normal(64) * 2; go = rng.standard_normal(64)
    tx = t(x); torch.nn.functional.gelu(tx, approximate="tanh").backward(t(go, False))
    out.update(gelu_x=x, gelu_go=go, gelu_gx=tx.grad.numpy())
    # softmax
    x = rng.standard_normal((3, 4, 7)); go = rng.standard_normal((3, 4, 7))
    tx = t(x); torch.softmax(tx, 1).backward(t(go, False))
    out.update(sm_x=x, sm_go=go, sm_gx=tx.grad.numpy())
    # cross entropy
    x = rng.standard_normal((6, 11)); lab = rng.integers(0, 11, 6)
    tx = t(x); loss = torch.nn.functional.cross_entropy(tx, torch.tensor(lab)); loss.backward()
    out.update(ce_x=x, ce_t=lab.astype(np.float64), ce_loss=loss.detach().numpy(), ce_gx=tx.grad.numpy())
    # embedding
    w = rng.standard_normal((9, 5)); idx = rng.integers(0, 9, (2, 4)); go = rng.standard_normal((2, 4, 5))
    tw = t(w); torch.nn.functional.embedding(torch.tensor(idx), tw).backward(t(go, False))
    out.update(emb_w=w, emb_idx=idx.astype(np.float64), emb_go=go, emb_gw=tw.grad.numpy())
    # attention with a causal additive mask
    B, H, S, dk = 2, 3, 6, 4
    q, k, v, go = (rng.standard_normal((B, H, S, dk)) for _ in range(4))
    mask = np.triu(np.full((S, S), -1e9), 1)
    tq, tk, tv = t(q), t(k), t(v)
    p = torch.softmax(tq @ tk.transpose(2, 3) / np.sqrt(dk) + t(mask, False), 3)
    o = p @ tv; o.backward(t(go, False))
    out.update(at_q=q, at_k=k, at_v=v, at_mask=mask, at_go=go, at_o=o.detach().numpy(),
               at_dq=tq.grad.numpy(), at_dk=tk.grad.numpy(), at_dv=tv.grad.numpy())
    # conv2d, stride 1 pad 1 and stride 2 pad 0
    for tag, s, pd in (("c1", 1, 1), ("c2", 2, 0)):
        x = rng.standard_normal((2, 3, 7, 6)); w = rng.standard_normal((4, 3, 3, 3)); b = rng.standard_normal(4)
        tx, tw, tb = t(x), t(w), t(b)
        y = torch.nn.functional.conv2d(tx, tw, tb, stride=s, padding=pd)
        go = rng.standard_normal(tuple(y.shape)); y.backward(t(go, False))
        out.update({f"{tag}_x": x, f"{tag}_w": w, f"{tag}_b": b, f"{tag}_go": go, f"{tag}_y": y.detach().numpy(),
                    f"{tag}_gx": tx.grad.numpy(), f"{tag}_gw": tw.grad.numpy(), f"{tag}_gb": tb.grad.numpy()})
    # batchnorm training + eval
    x = rng.standard_normal((4, 3, 5, 5)) * 2 + 1; g = rng.standard_normal(3); b = rng.standard_normal(3); go = rng.standard_normal((4, 3, 5, 5))
    for tag, training in (("bnt", True), ("bne", False)):
        rm = np.array([0.1, -0.2, 0.3]); rv = np.array([1.5, 0.7, 1.1])
        tx, tg, tb = t(x), t(g), t(b); trm, trv = t(rm, False), t(rv, False)
        y = torch.nn.functional.batch_norm(tx, trm, trv, tg, tb, training, 0.1, 1e-5); y.backward(t(go, False))
        out.update({f"{tag}_x": x, f"{tag}_g": g, f"{tag}_b": b, f"{tag}_go": go, f"{tag}_rm0": rm, f"{tag}_rv0": rv,
                    f"{tag}_y": y.detach().numpy(), f"{tag}_rm1": trm.numpy(), f"{tag}_rv1": trv.numpy(),
                    f"{tag}_gx": tx.grad.numpy(), f"{tag}_gg": tg.grad.numpy(), f"{tag}_gb": tb.grad.numpy()})
    # pools
    x = rng.standard_normal((2, 2, 7, 7)); tx = t(x)
    y = torch.nn.functional.max_pool2d(tx, 3, 2, 1); go = rng.standard_normal(tuple(y.shape)); y.backward(t(go, False))
    out.update(mp_x=x, mp_go=go, mp_y=y.detach().numpy(), mp_gx=tx.grad.numpy())
    tx = t(x)
    y = torch.nn.functional.avg_pool2d(tx, 3, 2, 1, count_include_pad=False); go = rng.standard_normal(tuple(y.shape)); y.backward(t(go, False))
    out.update(ap_x=x, ap_go=go, ap_y=y.detach().numpy(), ap_gx=tx.grad.numpy())
    # AdamW, 3 steps with weight decay; SGD momentum, 3 steps
    w0 = rng.standard_normal(10); gs = rng.standard_normal((3, 10))
    tw = t(w0.copy()); opt = torch.optim.AdamW([tw], lr=0.01, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    for i in range(3):
        tw.grad = t(gs[i], False); opt.step()
    out.update(adam_w0=w0, adam_gs=gs, adam_w3=tw.detach().numpy())
    tw = t(w0.copy()); opt = torch.optim.SGD([tw], lr=0.1, momentum=0.9, weight_decay=0.01)
    for i in range(3):
        tw.grad = t(gs[i], False); opt.step()
    out.update(sgd_w3=tw.detach().numpy())
    return out


if __name__ == "__main__":
    with open(os.path.join(HERE, "forward_cases.json"), "w") as f:
        json.dump(forward_cases(), f, indent=1)
    np.savez_compressed(os.path.join(HERE, "backward_cases.npz"), **backward_cases())
    print("written")

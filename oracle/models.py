"""Model graphs composed from oracle ops, op for op as the reference's layers emit them.

TEST INFRASTRUCTURE ONLY (see oracle.py).  Parameters are supplied as NumPy arrays in the
order of the reference's `parameters()` methods so that the CPU oracle and the CUDA
library start from identical values.

Citations are to crates/vearo-nn/src/lib.rs of the reference.
"""
import numpy as np

from .oracle import Tensor


class Linear:
    """y = x . W^T (+ b): transpose view, matmul, add (lib.rs:119-137)."""

    def __init__(self, w, b=None):
        self.weight = Tensor.from_numpy(w, requires_grad=True)
        self.bias = None if b is None else Tensor.from_numpy(b, requires_grad=True)

    def forward(self, x):
        out = x.matmul(self.weight.transpose(0, 1))
        return out if self.bias is None else out.add(self.bias)

    def parameters(self):
        return [self.weight] + ([] if self.bias is None else [self.bias])


class LayerNorm:
    """lib.rs:510-543"""

    def __init__(self, w, b, eps=1e-5):
        self.weight = Tensor.from_numpy(w, requires_grad=True)
        self.bias = Tensor.from_numpy(b, requires_grad=True)
        self.eps = eps

    def forward(self, x):
        return x.layernorm(self.weight, self.bias, self.eps)

    def parameters(self):
        return [self.weight, self.bias]


class MultiHeadAttention:
    """lib.rs:546-633 (fused path, or the unfused softmax(q k^T scale + mask) v path)."""

    def __init__(self, params, n_embd, n_head, fused=True):
        self.q, self.k, self.v, self.o = (Linear(params[2 * i], params[2 * i + 1]) for i in range(4))
        self.n_head, self.n_embd, self.fused = n_head, n_embd, fused

    def forward(self, x, mask):
        b, s, _ = x.shape
        h, d = self.n_head, self.n_embd
        dk = d // h
        q = self.q.forward(x).reshape([b, s, h, dk]).transpose(1, 2)
        k = self.k.forward(x).reshape([b, s, h, dk]).transpose(1, 2)
        v = self.v.forward(x).reshape([b, s, h, dk]).transpose(1, 2)
        if self.fused:
            out = q.fused_attention(k, v, mask)
        else:
            scale = Tensor.from_numpy(np.array([1.0 / np.sqrt(np.float32(dk))], dtype=np.float32))
            scores = q.matmul(k.transpose(2, 3)).mul(scale)
            if mask is not None:
                scores = scores.add(mask)
            out = scores.softmax(3).matmul(v)
        out = out.transpose(1, 2).reshape([b, s, d])
        return self.o.forward(out)

    def parameters(self):
        return self.q.parameters() + self.k.parameters() + self.v.parameters() + self.o.parameters()


class TransformerBlock:
    """Pre-LN block (lib.rs:636-688).  16 parameter tensors in `parameters()` order:
    ln1 w,b; q w,b; k w,b; v w,b; out w,b; ln2 w,b; fc1 w,b; fc2 w,b."""

    def __init__(self, p, n_embd, n_head, fused=True):
        self.ln1 = LayerNorm(p[0], p[1])
        self.attn = MultiHeadAttention(p[2:10], n_embd, n_head, fused)
        self.ln2 = LayerNorm(p[10], p[11])
        self.fc1 = Linear(p[12], p[13])
        self.fc2 = Linear(p[14], p[15])

    def forward(self, x, mask):
        x = x.add(self.attn.forward(self.ln1.forward(x), mask))
        m = self.fc2.forward(self.fc1.forward(self.ln2.forward(x)).gelu())
        return x.add(m)

    def parameters(self):
        return (self.ln1.parameters() + self.attn.parameters() + self.ln2.parameters()
                + self.fc1.parameters() + self.fc2.parameters())


class SimpleGPT:
    """lib.rs:691-808.  `params` order: tok, pos, 16 per block, ln_f w,b, lm_head w."""

    def __init__(self, params, n_embd, n_head, n_layer, fused=True):
        self.tok = Tensor.from_numpy(params[0], requires_grad=True)
        self.pos = Tensor.from_numpy(params[1], requires_grad=True)
        self.blocks = [TransformerBlock(params[2 + 16 * i: 2 + 16 * (i + 1)], n_embd, n_head, fused)
                       for i in range(n_layer)]
        o = 2 + 16 * n_layer
        self.ln_f = LayerNorm(params[o], params[o + 1])
        self.lm_head = Linear(params[o + 2])
        self.n_embd = n_embd

    def forward(self, ids, targets=None):
        b, s = ids.shape
        pos = Tensor.from_numpy(np.tile(np.arange(s, dtype=np.float32), (b, 1)))
        h = ids.embedding(self.tok).add(pos.embedding(self.pos))
        mask = Tensor.from_numpy(np.triu(np.full((s, s), -1e9, dtype=np.float32), k=1))
        for blk in self.blocks:
            h = blk.forward(h, mask)
        h = self.ln_f.forward(h).reshape([b * s, self.n_embd])
        logits = self.lm_head.forward(h)
        loss = None if targets is None else logits.cross_entropy(targets.reshape([b * s]))
        return logits, loss

    def parameters(self):
        ps = [self.tok, self.pos]
        for blk in self.blocks:
            ps += blk.parameters()
        return ps + self.ln_f.parameters() + self.lm_head.parameters()


class MLP:
    """Linear-ReLU-Linear-ReLU-Linear with MSE = mean(diff * diff) (examples/train_mlp.rs:51-69)."""

    def __init__(self, params):
        self.layers = [Linear(params[2 * i], params[2 * i + 1]) for i in range(len(params) // 2)]

    def forward(self, x):
        for i, l in enumerate(self.layers):
            x = l.forward(x)
            if i + 1 < len(self.layers):
                x = x.relu()
        return x

    def loss(self, x, y):
        diff = self.forward(x).sub(y)
        return diff.mul(diff).mean(0, False)

    def parameters(self):
        return [p for l in self.layers for p in l.parameters()]


class ConvNet:
    """3 x [conv3x3 p1 -> batchnorm -> relu -> maxpool 2,2,0] -> avgpool -> Linear -> cross_entropy.
    `params` order: per stage conv w,b, bn gamma,beta; then fc w,b."""

    def __init__(self, params, n_stage=3, momentum=0.1, eps=1e-5):
        self.stages = []
        for i in range(n_stage):
            cw, cb, g, b = params[4 * i: 4 * i + 4]
            c = cw.shape[0]
            self.stages.append(dict(
                w=Tensor.from_numpy(cw, True), b=Tensor.from_numpy(cb, True),
                g=Tensor.from_numpy(g, True), beta=Tensor.from_numpy(b, True),
                rm=Tensor.from_numpy(np.zeros(c, np.float32)), rv=Tensor.from_numpy(np.ones(c, np.float32))))
        self.fc = Linear(params[4 * n_stage], params[4 * n_stage + 1])
        self.momentum, self.eps = momentum, eps

    def forward(self, x, labels, training=True):
        for st in self.stages:
            x = x.conv2d(st["w"], st["b"], 1, 1)
            x = x.batchnorm(st["g"], st["beta"], st["rm"], st["rv"], training, self.momentum, self.eps)
            x = x.relu().maxpool2d(2, 2, 0)
        n, c, h, _ = x.shape
        x = x.avgpool2d(h, h, 0).reshape([n, c])
        return self.fc.forward(x).cross_entropy(labels)

    def parameters(self):
        ps = []
        for st in self.stages:
            ps += [st["w"], st["b"], st["g"], st["beta"]]
        return ps + self.fc.parameters()

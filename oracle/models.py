"""TEST INFRASTRUCTURE, not product code: CPU restatements of the callers of the hot path
(the MLP training step, a Llama-architecture prefill, the attention products), in F32/F64
NumPy, for the parity tests of `metalium_rs_b200.workloads`.  Parity against burn-flex's own
bits is unpinned (see oracle.py); these follow the reference's model code by file:line.
"""
from __future__ import annotations

import numpy as np

from . import oracle as orc

f32 = np.float32


def mm(a, b):
    """F64-accumulated product rounded once to F32 (the truth an F32 product is held to)."""
    return (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)


# ---- MLP step: crates/tt-tests/tests/step12_mnist.rs:69-81 (init), :212-222 (step) -----------------
def mlp_init(seed=0xC0F1, d_in=784, hidden=128, classes=10):
    k1, k2 = 1.0 / np.sqrt(d_in), 1.0 / np.sqrt(hidden)
    return (orc.uniform(seed, 1, (d_in, hidden), -k1, k1), orc.uniform(seed, 2, (hidden,), -k1, k1),
            orc.uniform(seed, 3, (hidden, classes), -k2, k2), orc.uniform(seed, 4, (classes,), -k2, k2))


def mlp_step(x, labels, w1, b1, w2, b2, lr=0.01):
    """Forward, softmax cross-entropy (mean), backward, one SGD update.  Returns a dict of F32
    arrays: loss, logits, gradients and updated weights."""
    n = x.shape[0]
    pre = mm(x, w1)
    h = np.maximum((pre + b1).astype(f32), 0).astype(f32)
    z = (mm(h, w2) + b2).astype(f32)
    z64 = z.astype(np.float64)
    m = z64.max(1, keepdims=True)
    logp = (z64 - m - np.log(np.exp(z64 - m).sum(1, keepdims=True))).astype(f32)
    picked = logp[np.arange(n), labels.ravel()]
    loss = f32(-picked.astype(np.float64).mean())
    g = np.zeros_like(logp)
    g[np.arange(n), labels.ravel()] = f32(-1.0 / n)
    dz = (g - np.exp(logp.astype(np.float64)) * g.astype(np.float64).sum(1, keepdims=True)).astype(f32)
    dw2, db2 = mm(h.T, dz), dz.astype(np.float64).sum(0).astype(f32)
    dh = mm(dz, w2.T)
    dpre = np.where(h > 0, dh, 0).astype(f32)
    dw1, db1 = mm(x.T, dpre), dpre.astype(np.float64).sum(0).astype(f32)
    new = {k: (w - f32(lr) * d).astype(f32) for k, w, d in (("w1", w1, dw1), ("b1", b1, db1), ("w2", w2, dw2), ("b2", b2, db2))}
    return dict(loss=loss, logits=z, dw1=dw1, db1=db1, dw2=dw2, db2=db2, **new)


# ---- Llama prefill: crates/tt-models/src/llama.rs:371-507,798,1055; rope.rs:151-161 -----------------------
def llama_prefill(cfg, w, ids, batch, seq, all_positions=False):
    """F32 forward on the BF16-rounded weights (the tolerance statement's oracle).  `w` holds
    F32 arrays already rounded to BF16 values; ids [batch*seq]."""
    c = cfg
    hd, q_cols, kv_cols = c.head_dim, c.heads * c.head_dim, c.kv_heads * c.head_dim
    group = c.heads // c.kv_heads
    cos, sin = orc.rope_tables(seq, hd, c.theta)
    x = w["embed"][ids.ravel()].astype(f32)
    causal = np.triu(np.ones((seq, seq), bool), 1)
    for l in range(c.layers):
        n1 = orc.rms_norm(x, w[f"l{l}.norm1"], c.eps)
        qkv = mm(n1, w[f"l{l}.qkv"])
        q = orc.rope(qkv[:, :q_cols], cos, sin, hd)
        k = orc.rope(qkv[:, q_cols:q_cols + kv_cols], cos, sin, hd)
        v = qkv[:, q_cols + kv_cols:]
        att = np.empty((batch * seq, q_cols), f32)
        for b in range(batch):
            r = slice(b * seq, (b + 1) * seq)
            for h in range(c.heads):
                kvh = h // group
                s = mm(q[r, h * hd:(h + 1) * hd], k[r, kvh * hd:(kvh + 1) * hd].T).astype(np.float64) / np.sqrt(hd)
                s[causal] = -np.inf
                p = np.exp(s - s.max(1, keepdims=True))
                p /= p.sum(1, keepdims=True)
                att[r, h * hd:(h + 1) * hd] = (p @ v[r, kvh * hd:(kvh + 1) * hd].astype(np.float64)).astype(f32)
        x = (x + mm(att, w[f"l{l}.o"])).astype(f32)
        n2 = orc.rms_norm(x, w[f"l{l}.norm2"], c.eps)
        gu = mm(n2, w[f"l{l}.gate_up"]).astype(np.float64)
        gate, up = gu[:, :c.ff], gu[:, c.ff:]
        act = (gate / (1.0 + np.exp(-gate)) * up).astype(f32)
        x = (x + mm(act, w[f"l{l}.down"])).astype(f32)
    last = x if all_positions else x[[b * seq + seq - 1 for b in range(batch)]]
    fn = orc.rms_norm(last, w["final_norm"], c.eps)
    logits = mm(fn, w["embed"].T)
    return logits


# ---- attention products: crates/burn-tt/src/ops.rs:4447, 4573-4589 -------------------------------------------
def attention_item(q, k, v):
    """One (batch, head): softmax(q k^T / sqrt d) v in F64, inputs F32 values of BF16 data."""
    s = q.astype(np.float64) @ k.astype(np.float64).T / np.sqrt(q.shape[1])
    p = np.exp(s - s.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    return p @ v.astype(np.float64)

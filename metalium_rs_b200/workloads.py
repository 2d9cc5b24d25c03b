"""The callers of the hot path, restated as sequences of `Engine` calls.

Each function issues the ops the reference's Burn models send to the backend, in their
order, and nothing else: no arithmetic happens on the host.
  - `MlpStep`: the MNIST-shaped MLP training step (crates/tt-tests/tests/step12_mnist.rs:212-222;
    op sequence crates/burn-tt/src/ops.rs:5153-5158 (log-softmax), :1001/:1043 (gather and its
    backward), :5006-5028 (linear backward), :5174 (relu backward)).
  - `LlamaPrefill`: a decoder prefill with the SmolLM2-135M architecture
    (crates/tt-models/src/llama.rs:371-507 `Layer::forward`, :798 `forward`, :1055 `head`;
    crates/tt-models/src/rope.rs:129).
  - `attention_products`: Q K^T, row softmax, P V on rank-4 views
    (crates/burn-tt/src/ops.rs:4447 `attention`, the unfused path :4573-4589).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import os

import numpy as np

from . import BF16, BOOL, COLS, F32, I32, SUM, EltwiseOp, kinds


def _bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even BF16 bits of an F32 array (host-side weight preparation)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (r >> np.uint32(16)).astype(np.uint16)


# ------------------------------------------------------------------------- config 1
class MlpStep:
    """x [n,784] -> Linear(784,h) -> ReLU -> Linear(h,10) -> softmax cross-entropy, backward, SGD.
    Weights live on the device and are replaced by their updates each step."""

    def __init__(self, eng, w1, b1, w2, b2, lr=0.01, fused_add_relu=True, in_place=False):
        # in_place: the update is copied over the old weights, so they keep their addresses
        # (what a captured trace needs to train when it is replayed)
        self.eng, self.lr, self.fused, self.in_place = eng, float(lr), fused_add_relu, in_place
        self.trace = None
        self.w1 = eng.upload(w1, *w1.shape)
        self.b1 = eng.upload(b1.reshape(1, -1), 1, b1.size)
        self.w2 = eng.upload(w2, *w2.shape)
        self.b2 = eng.upload(b2.reshape(1, -1), 1, b2.size)

    def _el(self, kind, a, b=None, c=None, s=0.0):
        out, _ = self.eng.eltwise_op(EltwiseOp(kind, s, 0.0), a, b, c)
        return out

    def step(self, x_buf: int, labels_buf: int, n: int, keep=False) -> Dict[str, int]:
        """One training step on resident inputs.  Returns buffer ids: `loss` always, and with
        `keep` the logits and the four gradients (the caller frees what it gets)."""
        e, K = self.eng, kinds
        free: List[int] = []
        pre, _ = e.matmul_dram(x_buf, False, self.w1, False)                       # float_matmul
        if self.fused:
            h = self._el(K.ADD_RELU, pre, self.b1)                                 # fusion/eltwise.rs:1-8
        else:
            t = self._el(K.ADD, pre, self.b1); h = self._el(K.RELU, t); free.append(t)
        z0, _ = e.matmul_dram(h, False, self.w2, False)
        z = self._el(K.ADD, z0, self.b2)
        logp, _ = e.log_softmax_rows(z)                                            # ops.rs:5153-5158
        picked, _ = e.pick_columns(logp, labels_buf)                               # ops.rs:1001
        neg = self._el(K.NEG, picked)
        loss, _ = e.full_sum(neg, mean=True)                                       # ops.rs:3255
        # backward
        zeros, _ = e.zeros_dram((n, 1))
        gval = self._el(K.ADD_SCALAR, zeros, s=-1.0 / n)                           # d(mean(-picked))
        zl, dims = e.zeros_dram(e.dims_of(logp)[0])
        g, _ = e.scatter_add_columns(zl, labels_buf, gval)                         # ops.rs:1043
        p = self._el(K.EXP, logp)                                                  # log-softmax backward:
        gs, _ = e.reduce(g, SUM, COLS)                                             #   g - exp(logp) * sum(g)
        pg = self._el(K.MUL, p, gs)
        dz = self._el(K.SUB, g, pg)
        dw2, _ = e.matmul_dram(h, True, dz, False)                                 # x^T g (ops.rs:5006-5016)
        db2, _ = e.sum_rows(dz)                                                    # in-order (ops.rs:5022-5028)
        dh, _ = e.matmul_dram(dz, False, self.w2, True)
        dpre = self._el(K.RELU_BACKWARD, h, dh)                                    # ops.rs:5174
        dw1, _ = e.matmul_dram(x_buf, True, dpre, False)
        db1, _ = e.sum_rows(dpre)
        # SGD: w <- w - lr * dw  (mul_scalar, sub)
        for name, grad in (("w1", dw1), ("b1", db1), ("w2", dw2), ("b2", db2)):
            scaled = self._el(K.MUL_SCALAR, grad, s=self.lr)
            new = self._el(K.SUB, getattr(self, name), scaled)
            e.free(scaled)
            if self.in_place:
                e.copy_into(new, getattr(self, name)); e.free(new)
            else:
                e.free(getattr(self, name)); setattr(self, name, new)
        free += [pre, z0, logp, picked, neg, zeros, gval, zl, g, p, gs, pg, dh, h]
        out = {"loss": loss}
        if keep:
            out.update(logits=z, dw1=dw1, db1=db1, dw2=dw2, db2=db2, dz=dz, dpre=dpre)
        else:
            free += [z, dw1, db1, dw2, db2, dz, dpre]
        for i in free:
            e.free(i)
        return out


    def capture(self, x_buf: int, labels_buf: int, n: int) -> int:
        """Run one step eagerly (loads every kernel), then capture the next as a trace
        (crates/burn-tt/src/trace.rs; server.rs:591-660).  Returns the loss buffer the replays
        write; `replay()` runs one more training step on whatever x_buf / labels_buf hold."""
        assert self.in_place, "a replayed step must update the weights where they lie"
        e = self.eng
        e.free(self.step(x_buf, labels_buf, n)["loss"])
        e.begin_trace()
        loss = self.step(x_buf, labels_buf, n)["loss"]
        self.trace = e.end_trace()
        return loss

    def replay(self):
        self.eng.run_trace(self.trace)


# ------------------------------------------------------------------------- config 4
@dataclass
class LlamaConfig:  # crates/tt-models/src/llama.rs:40,60 (SMOLLM2_135M), theta per the benchmark config
    layers: int = 30
    hidden: int = 576
    heads: int = 9
    kv_heads: int = 3
    head_dim: int = 64
    ff: int = 1536
    vocab: int = 49152
    eps: float = 1e-5
    theta: float = 10000.0


def llama_weights(cfg: LlamaConfig, seed: int = 0xC0F4, sigma: float = 0.02) -> Dict[str, np.ndarray]:
    """Random-init weights N(0, sigma) as F32 (norm gains 1), laid out [in, out]."""
    rng = np.random.default_rng(seed)
    nrm = lambda *s: (rng.standard_normal(s, dtype=np.float32) * np.float32(sigma))
    w = {"embed": nrm(cfg.vocab, cfg.hidden), "final_norm": np.ones(cfg.hidden, np.float32)}
    q, kv = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
    for l in range(cfg.layers):
        w[f"l{l}.qkv"] = nrm(cfg.hidden, q + 2 * kv)       # Wq | Wk | Wv side by side
        w[f"l{l}.o"] = nrm(q, cfg.hidden)
        w[f"l{l}.gate_up"] = nrm(cfg.hidden, 2 * cfg.ff)   # Wgate | Wup side by side
        w[f"l{l}.down"] = nrm(cfg.ff, cfg.hidden)
        w[f"l{l}.norm1"] = np.ones(cfg.hidden, np.float32)
        w[f"l{l}.norm2"] = np.ones(cfg.hidden, np.float32)
    return w


def prefill_ids(cfg: LlamaConfig, batch: int, seq: int, seed: int = 0xC0F4) -> np.ndarray:
    """Token ids [1, batch * seq] I32, uniform in [0, vocab): the benchmark's synthetic prompt."""
    return np.random.default_rng(seed ^ 0x1D5).integers(0, cfg.vocab, (1, batch * seq)).astype(np.int32)


def interleave_gate_up(w: np.ndarray) -> np.ndarray:
    """[in, gate | up] -> the layout `matmul_silu_mul` reads: groups of 256 columns, 128 gate columns then the
    128 matching up columns."""
    ff = w.shape[1] // 2
    assert ff % 128 == 0
    g, u = w[:, :ff].reshape(w.shape[0], ff // 128, 128), w[:, ff:].reshape(w.shape[0], ff // 128, 128)
    return np.ascontiguousarray(np.concatenate([g, u], axis=2).reshape(w.shape[0], 2 * ff))


def rope_tables(positions: int, head: int, theta: float):
    """cos and sin' = [-sin, sin] (crates/tt-models/src/rope.rs:19-60), [positions, head] F32."""
    i = np.arange(head // 2, dtype=np.float64)
    freq = (theta ** (-2.0 * i / head)).astype(np.float32)
    ang = (np.arange(positions, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
    cos = np.cos(ang.astype(np.float64)).astype(np.float32)
    sin = np.sin(ang.astype(np.float64)).astype(np.float32)
    return np.concatenate([cos, cos], 1), np.concatenate([-sin, sin], 1)


class LlamaPrefill:
    """Prefill of `batch` independent causal sequences of `seq` tokens.  Weights are stored BF16;
    the residual stream is F32; projections read BF16 activations and accumulate in F32."""

    def __init__(self, eng, cfg: LlamaConfig, weights: Dict[str, np.ndarray], batch: int, seq: int, fused_attention=None,
                 fused_mlp=None):
        """fused_attention: None = the fused kernel where it takes the shape (whole 128-row tiles, heads
        of 64 or 128), True = require it, False = the composition (batched Q K^T, softmax, batched P V).
        fused_mlp: True = silu(gate) * up from the gate|up product's epilogue (`matmul_silu_mul`), False = the
        product then `SILU_MUL`, None = the fused form where ff is whole groups of 128 columns.  The same bits
        either way.  On eight epilogue warps a CTA the fused form is the faster one (8 x 512 prefill: 3.63 ms
        against 3.80; on four warps the activation's exponentials outlasted the tile's product: 3.98)."""
        self.eng, self.cfg, self.batch, self.seq = eng, cfg, batch, seq
        self.fused_mlp = (cfg.ff % 128 == 0) if fused_mlp is None else bool(fused_mlp)
        # RoPE in the QKV projection's epilogue (`matmul_rope`, heads 64 wide) only on request (B200TT_FUSED_ROPE=1): the
        # same bits, but this projection is ONE wave of tiles, so its epilogue hides under nothing and the rotation there
        # (a row's table entries fetched by the row's own thread) costs more than the separate launch: 3.83 against 3.66 ms
        self.fused_rope = cfg.head_dim == 64 and os.environ.get("B200TT_FUSED_ROPE", "0") == "1"
        # the output and down projections straight into the residual stream and its norm (`matmul_add_rms_norm`: one
        # launch where the composition takes two), where hidden is one to eight tiles of 192 columns and there are at
        # least 64 tokens (B200TT_FUSED_NORM=0: the composition).  The sums are the composition's bits, the norm's
        # statistic is added in another fixed order.  Timed alone, back to back, the fused launch is the slower one
        # (17.2 against 15.5 us for the pair: the norm in a one-wave product's epilogue hides under nothing); inside the
        # layer's chain of launches it saves a launch, its gap and a round trip of the product: 8 x 512 prefill 3.42
        # against 3.67 ms on the same box.
        self.fused_norm = (cfg.hidden % 192 == 0 and cfg.hidden // 192 <= 8 and batch * seq >= 64 and
                           os.environ.get("B200TT_FUSED_NORM", "1") != "0")
        if self.fused_mlp and cfg.ff % 128:
            raise ValueError("the fused gate|up product needs ff in whole groups of 128 columns")
        takes = cfg.head_dim in (64, 128)                    # any length: a tail tile is masked by index
        if fused_attention and not takes:
            raise ValueError("the fused attention kernel does not take this shape")
        # by default the one-kernel form from a tile of tokens up (below that the composed form's scores are small)
        self.fused = (takes and seq >= 128) if fused_attention is None else bool(fused_attention)
        up = lambda a: eng.upload_bf16(_bf16(a), *a.shape)
        self.w = {}
        for k, v in weights.items():
            self.w[k] = up(v.reshape(1, -1) if v.ndim == 1 else v)
            if self.fused_mlp and k.endswith(".gate_up"):
                self.w[k + ".interleaved"] = up(interleave_gate_up(v))
        cos, sin = rope_tables(seq, cfg.head_dim, cfg.theta)
        self.cos, self.sin = eng.upload(cos, *cos.shape), eng.upload(sin, *sin.shape)
        mask = np.triu(np.ones((seq, seq), np.uint32), 1)   # 1 above the diagonal: filled with -inf
        self.mask = eng.upload_bits(mask, seq, seq, BOOL)
        c = cfg
        self.q_cols, self.kv_cols = c.heads * c.head_dim, c.kv_heads * c.head_dim
        group = c.heads // c.kv_heads
        t = seq
        hd = c.head_dim
        # attention block lists (crates/burn-tt/src/ops.rs:3008-3081): item i = (b, h)
        self.qk_items, self.pv_items, self.merge, fused_items = [], [], [], []
        for b in range(batch):
            for h in range(c.heads):
                i = b * c.heads + h
                kvh = h // group
                fused_items.append(((b * t, h * hd), (b * t, self.q_cols + kvh * hd),
                                    (b * t, self.q_cols + self.kv_cols + kvh * hd), (b * t, h * hd)))
                self.qk_items.append((((b * t, h * hd), False), ((b * t, self.q_cols + kvh * hd), True)))
                self.pv_items.append((((i * t, 0), False), ((b * t, self.q_cols + self.kv_cols + kvh * hd), False)))
                self.merge.append(((i * t, 0), (b * t, h * hd), (t, hd), False))
        self.fused_items = eng.attention_block_array(fused_items)
        self.last_rows = [(0, b * t + t - 1) for b in range(batch)]

    def forward(self, ids_buf: int, all_positions: bool = False, cache: "LlamaDecode" = None, start: int = 0):
        """ids [1, batch*seq] I32 resident.  Returns (logits buffer [batch or batch*seq, vocab] F32,
        argmax buffer I32); the caller frees both.  With `cache`, every layer's rotated keys and its values are
        also written into that generation's cache at positions 0 .. seq-1 of each sequence, as the reference's
        first chunk write does (crates/tt-models/src/kv_cache.rs:231-241, start 0): the bits a token-by-token
        generation would have left there, so `cache.continue_from(argmax, seq)` goes on from the prompt.
        With `start` > 0 the tokens are a later chunk of the prompt (kv_cache.rs:231-241, 249-296): they take
        positions start .. start + seq - 1, their keys and values go to those rows of the cache, and every token
        attends to the cache's positions up to its own -- the chunks before it and its own chunk's earlier tokens
        -- through the fused attention kernel reading keys and values where the cache holds them (whole 128-row
        tiles: start and seq multiples of 128)."""
        e, c, K = self.eng, self.cfg, kinds
        n = self.batch * self.seq
        chunked = start > 0
        if chunked:
            if cache is None or not self.fused or start % 128:
                raise ValueError("a later chunk needs a cache, the fused attention kernel and a start in whole 128-position tiles")
        if cache is not None:
            assert cache.batch == self.batch and cache.max_len >= start + self.seq and cache.cfg is self.cfg
            key = (cache.max_len, start)
            if getattr(self, "_cache_rows_key", None) != key:
                rows = (np.arange(self.batch)[:, None] * cache.max_len + start + np.arange(self.seq)[None, :]).astype(np.int32)
                if getattr(self, "_cache_rows", None):
                    e.free(self._cache_rows)
                self._cache_rows = e.upload_bits(rows.reshape(1, -1).view(np.uint32), 1, n, I32)
                self._cache_rows_key = key
                group, hd_ = self.cfg.heads // self.cfg.kv_heads, self.cfg.head_dim
                self._cache_items = e.attention_block_array(
                    [((b * self.seq, h * hd_), (b * cache.max_len, (h // group) * hd_), (b * cache.max_len, (h // group) * hd_),
                      (b * self.seq, h * hd_)) for b in range(self.batch) for h in range(self.cfg.heads)])
        t, hd = self.seq, c.head_dim
        el = lambda kind, a, b=None, bf=False: e.eltwise_op_as(EltwiseOp(kind, 0.0, 0.0), a, b, None, bf)[0]
        # while the engine's profile mode is on, each op class runs under its own label (server.rs:2370 labels every job)
        lab = e.set_op_label if getattr(e, "profiling", False) else (lambda name: None)
        lab("embedding")
        emb, _ = e.select_rows(self.w["embed"], ids_buf)                     # ops.rs:4958 embedding
        x, _ = e.cast_float(emb, False)                                      # residual stream F32
        e.free(emb)
        qk_cols = self.q_cols + self.kv_cols
        lab("norm")
        n1, _ = e.rms_norm_as(x, self.w["l0.norm1"], c.eps, True)           # llama.rs:151-170
        for l in range(c.layers):
            lab("projection qkv")
            # RoPE on the query and key heads together: they share the head width and the tables (rope.rs:129)
            cos_b = (cache.cos, (start, 0), (t, hd)) if chunked else (self.cos, (0, 0), (t, hd))
            sin_b = (cache.sin, (start, 0), (t, hd)) if chunked else (self.sin, (0, 0), (t, hd))
            if self.fused_rope:   # the rotation in the projection's own epilogue: the same bits, one launch less
                qkv, _ = e.matmul_rope(n1, self.w[f"l{l}.qkv"], cos_b, sin_b, qk_cols)
                e.free(n1)
                qk = qkv          # the rotated query and key heads are the buffer's first columns
            else:
                qkv, _ = e.matmul_dram_bf16(n1, False, self.w[f"l{l}.qkv"], False)
                e.free(n1)
                lab("rope")
                qk, _ = e.rope_blocks((qkv, (0, 0), (n, qk_cols)), cos_b, sin_b, hd, True)
            if cache is not None:
                lab("cache write")   # the chunk's rows of the cache: keys after RoPE, values as projected
                e.scatter_rows_into(cache.kc[l], self._cache_rows, (qk, (0, self.q_cols), (n, self.kv_cols)))
                e.scatter_rows_into(cache.vc[l], self._cache_rows, (qkv, (0, qk_cols), (n, self.kv_cols)))
            lab("attention")
            if chunked:      # keys and values where the cache holds them: positions 0 .. start + t - 1, causal at the end
                om, _ = e.attention_blocks(qk, cache.kc[l], cache.vc[l], self._cache_items, (t, hd, start + t, hd),
                                           1.0 / float(np.sqrt(hd)), True, (n, self.q_cols))
                if qk != qkv:
                    e.free(qk)
                e.free(qkv)
            elif self.fused:   # scores, mask, softmax, P V and the merge of heads as one kernel
                om, _ = e.attention_blocks(qk, qk, qkv, self.fused_items, (t, hd, t, hd), 1.0 / float(np.sqrt(hd)), True,
                                           (n, self.q_cols))
                if qk != qkv:
                    e.free(qk)
                e.free(qkv)
            else:
                s, _ = e.matmul_dram_batched(qk, qk, self.qk_items, (t, hd, t))  # Q K^T, F32 scores
                if qk != qkv:
                    e.free(qk)
                pb, _ = e.softmax_rows_as(s, self.mask, 1.0 / float(np.sqrt(hd)), True)   # scale, causal mask, softmax
                e.free(s)
                o, _ = e.matmul_dram_batched(pb, qkv, self.pv_items, (t, t, hd), bf16=True)   # P V
                e.free(pb); e.free(qkv)
                om, _ = e.copy_blocks(o, self.merge, (n, self.q_cols))           # merge heads
                e.free(o)
            lab("projection o")
            if self.fused_norm:   # o_proj, the residual add and the next norm as one launch
                (x2, _), (n2, _) = e.matmul_add_rms_norm(om, self.w[f"l{l}.o"], x, self.w[f"l{l}.norm2"], c.eps)
                e.free(om); e.free(x)
            else:
                att, _ = e.matmul_dram(om, False, self.w[f"l{l}.o"], False)      # o_proj, F32 out
                e.free(om)
                lab("add + norm")
                # residual add and the next norm as one op (`Engine::add_rms_norm`, server.rs:466; llama.rs:288)
                (x2, _), (n2, _) = e.add_rms_norm_as(x, att, self.w[f"l{l}.norm2"], c.eps, True)
                e.free(x); e.free(att)
            lab("projection gate|up")
            if self.fused_mlp:   # silu(gate) * up stored by the gate|up product's own epilogue
                act, _ = e.matmul_silu_mul(n2, self.w[f"l{l}.gate_up.interleaved"])
                e.free(n2)
            else:
                gu, _ = e.matmul_dram_bf16(n2, False, self.w[f"l{l}.gate_up"], False)
                e.free(n2)
                lab("silu_mul")
                act, _ = e.eltwise_blocks_as(EltwiseOp(K.SILU_MUL, 0.0, 0.0), (gu, (0, 0), (n, c.ff)),
                                             (gu, (0, c.ff), (n, c.ff)), None, True)   # silu(gate) * up (llama.rs:498)
                e.free(gu)
            lab("projection down")
            if self.fused_norm and l + 1 < c.layers:
                (x, _), (n1, _) = e.matmul_add_rms_norm(act, self.w[f"l{l}.down"], x2, self.w[f"l{l + 1}.norm1"], c.eps)
                e.free(act); e.free(x2)
            else:
                d, _ = e.matmul_dram(act, False, self.w[f"l{l}.down"], False)
                e.free(act)
                lab("add + norm")
                if l + 1 < c.layers:
                    (x, _), (n1, _) = e.add_rms_norm_as(x2, d, self.w[f"l{l + 1}.norm1"], c.eps, True)
                else:
                    x = el(K.ADD, x2, d)
                e.free(x2); e.free(d)
        lab("head")
        if all_positions:
            last = x
        else:
            last, _ = e.gather_rows([x], self.last_rows, c.hidden)           # last position only (llama.rs:1055-1061)
            e.free(x)
        fn, _ = e.rms_norm_as(last, self.w["final_norm"], c.eps, True)
        e.free(last)
        logits, _ = e.matmul_dram(fn, False, self.w["embed"], True)          # tied head: last . table^T (llama.rs:1090)
        e.free(fn)
        am, _ = e.argmax_row(logits)                                         # generate::argmax
        lab("")
        return logits, am

    def capture(self, ids_buf: int):
        """One eager pass, then the forward captured as a trace.  Returns (logits, argmax)
        buffers that every `replay()` rewrites from the ids then in `ids_buf`."""
        e = self.eng
        lg, am = self.forward(ids_buf)
        e.free(lg); e.free(am)
        e.begin_trace()
        out = self.forward(ids_buf)
        self.trace = e.end_trace()
        return out

    def replay(self):
        self.eng.run_trace(self.trace)

    def flops(self, all_positions=False) -> float:
        c, n, t = self.cfg, self.batch * self.seq, self.seq
        q, kv = self.q_cols, self.kv_cols
        lin = 2.0 * n * (c.hidden * (q + 2 * kv) + q * c.hidden + c.hidden * 2 * c.ff + c.ff * c.hidden) * c.layers
        att = 2.0 * 2.0 * self.batch * c.heads * t * t * c.head_dim * c.layers
        head = 2.0 * (n if all_positions else self.batch) * c.hidden * c.vocab
        return lin + att + head


# ------------------------------------------------------------------------- config 5
def attention_products(eng, q_buf: int, k_buf: int, v_buf: int, batch_heads: int, t: int, d: int):
    """Q, K, V stored [batch_heads*t, d] BF16.  S = Q K^T (F32), P = softmax(S / sqrt d) in F32,
    O = P(BF16) V -> [batch_heads*t, d] BF16.  Returns O's buffer."""
    qk = [(((i * t, 0), False), ((i * t, 0), True)) for i in range(batch_heads)]
    pv = [(((i * t, 0), False), ((i * t, 0), False)) for i in range(batch_heads)]
    s, _ = eng.matmul_dram_batched(q_buf, k_buf, qk, (t, d, t))
    pb, _ = eng.softmax_rows_as(s, None, 1.0 / float(np.sqrt(d)), True)
    eng.free(s)
    o, _ = eng.matmul_dram_batched(pb, v_buf, pv, (t, t, d), bf16=True)
    eng.free(pb)
    return o


def attention_fused(eng, q_buf: int, k_buf: int, v_buf: int, batch_heads: int, t: int, d: int, items=None):
    """The same attention as `attention_products` as one kernel: the scores stay on chip."""
    if items is None:
        items = eng.attention_block_array([((i * t, 0), (i * t, 0), (i * t, 0), (i * t, 0)) for i in range(batch_heads)])
    return eng.attention_blocks(q_buf, k_buf, v_buf, items, (t, d, t, d), 1.0 / float(np.sqrt(d)), False, (batch_heads * t, d))[0]


# ------------------------------------------------------------------------- convolution and pooling over NHWC tables
def _tap_at(out: int, tap: int, stride: int, dilation: int, padding: int, length: int):
    """crates/burn-tt/src/ops/nhwc.rs:159-170: the input coordinate a tap reads, or None in the padding."""
    i = out * stride + tap * dilation - padding
    return i if 0 <= i < length else None


def conv2d_nhwc(eng, table_buf: int, shape, weight: np.ndarray, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    """A 2-D convolution as the reference sends it (crates/burn-tt/src/ops/nhwc.rs:226-292): the activation is its
    NHWC table [n h w, c] (resident, F32); a [taps, positions] index of table rows that depends on the shapes alone
    goes up once; `select_taps` makes the patch matrix [positions, (taps-1) ceil32(c) + c] on the device (a padding
    tap reads the zero row); the weights [o, c, kh, kw] are relaid on the device to [that many rows, o] by
    `repack_many` from the weight and a zero (rows a tap's channels do not fill are zero); one product, one
    broadcast add of the bias.  Returns (the [positions, o] result buffer: the next layer's NHWC table, (oh, ow))."""
    n, c, h, w = shape
    o, wc, kh, kw = weight.shape
    assert wc == c
    oh = (h + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
    ow = (w + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
    taps, positions, rows = kh * kw, n * oh * ow, n * h * w
    idx = np.empty((taps, positions), np.int32)
    for t in range(taps):
        ky, kx = divmod(t, kw)
        for q in range(positions):
            b, y, xo = q // (oh * ow), q // ow % oh, q % ow
            iy, ix = _tap_at(y, ky, stride[0], dilation[0], padding[0], h), _tap_at(xo, kx, stride[1], dilation[1], padding[1], w)
            idx[t, q] = rows if iy is None or ix is None else (b * h + iy) * w + ix
    ii = eng.upload_bits(idx.view(np.uint32), taps, positions, I32)
    patches, pd = eng.select_taps(table_buf, ii, any(p > 0 for p in padding))
    eng.free(ii)
    pitch = -(-c // 32) * 32
    k = (taps - 1) * pitch + c
    assert pd == (positions, k)
    wm = eng.upload(np.ascontiguousarray(weight, np.float32).reshape(o, c * taps), o, c * taps)    # [o, (c, kh, kw)] as stored
    zero = eng.zeros_dram((1, 1))[0]
    sources = []
    for r in range(k):
        t, ch = divmod(r, pitch)
        for oc in range(o):
            sources.append((0, (oc, ch * taps + t)) if ch < c else (1, (0, 0)))
    wk, _ = eng.repack_many([wm, zero], sources, (k, o))
    eng.free(wm); eng.free(zero)
    out, _ = eng.matmul_dram(patches, False, wk, False)
    eng.free(patches); eng.free(wk)
    if bias is not None:
        ib = eng.upload(np.ascontiguousarray(bias, np.float32).reshape(1, o), 1, o)
        out2, _ = eng.eltwise_op(EltwiseOp(kinds.ADD, 0.0, 0.0), out, ib)
        eng.free(out); eng.free(ib)
        out = out2
    return out, (oh, ow)


def max_pool2d_nhwc(eng, table_buf: int, shape, kernel, stride, padding=(0, 0), dilation=(1, 1)):
    """`max_pool2d` as one select and a fold over the taps (crates/burn-tt/src/ops/nhwc.rs:296-418): a padding tap
    reads its window's first valid datum; the taps' column blocks are folded in window order with exact compares
    and selects -- the first NaN, else the first maximum, bit for bit.  c must be whole tiles of 32 columns.
    Returns (the [positions, c] result buffer, (oh, ow))."""
    n, c, h, w = shape
    assert c % 32 == 0
    oh = (h + 2 * padding[0] - dilation[0] * (kernel[0] - 1) - 1) // stride[0] + 1
    ow = (w + 2 * padding[1] - dilation[1] * (kernel[1] - 1) - 1) // stride[1] + 1
    taps, positions = kernel[0] * kernel[1], n * oh * ow
    idx = np.zeros((taps, positions), np.int32)
    for q in range(positions):
        b, y, xo = q // (oh * ow), q // ow % oh, q % ow
        at = []
        for t in range(taps):
            iy = _tap_at(y, t // kernel[1], stride[0], dilation[0], padding[0], h)
            ix = _tap_at(xo, t % kernel[1], stride[1], dilation[1], padding[1], w)
            at.append(None if iy is None or ix is None else (b * h + iy) * w + ix)
        first = next(a for a in at if a is not None)
        idx[:, q] = [first if a is None else a for a in at]
    ii = eng.upload_bits(idx.view(np.uint32), taps, positions, I32)
    patches, _ = eng.select_taps(table_buf, ii, False)
    eng.free(ii)
    K = kinds
    el = lambda kind, a, b=None, cc=None: eng.eltwise_op(EltwiseOp(kind, 0.0, 0.0), a, b, cc)[0]
    block = lambda t: eng.copy_blocks(patches, [((0, t * c), (0, 0), (positions, c), False)], (positions, c))[0]
    best = block(0)
    nan = el(K.IS_NAN, best)
    for t in range(1, taps):
        b = block(t)
        b_nan = el(K.IS_NAN, b)
        gt, not_nan = el(K.GT, b, best), el(K.BOOL_NOT, nan)
        either = el(K.BOOL_OR, gt, b_nan)
        take = el(K.BOOL_AND, not_nan, either)
        best2 = el(K.MASK_WHERE, best, take, b)         # `b` where `take`, else the best so far
        nan2 = el(K.BOOL_OR, nan, b_nan)
        for i in (b, b_nan, gt, not_nan, either, take, best, nan):
            eng.free(i)
        best, nan = best2, nan2
    eng.free(nan); eng.free(patches)
    return best, (oh, ow)


def avg_pool2d_windows(shape, kernel, stride, padding=(0, 0), count_include_pad=True):
    """The windows and divisors of an average pooling over a BF16 NCHW tensor stored [n c h, w] (the geometry
    crates/burn-tt/src/ops/pool.rs:254-268 hands to `pool_bf16`): a window lists its valid taps as [row, col] of
    that matrix; the divisor counts the padding taps too when `count_include_pad`."""
    n, c, h, w = shape
    oh = (h + 2 * padding[0] - kernel[0]) // stride[0] + 1
    ow = (w + 2 * padding[1] - kernel[1]) // stride[1] + 1
    windows, divisors = [], []
    for plane in range(n * c):
        for y in range(oh):
            for xo in range(ow):
                taps = [[plane * h + iy, ix] for ky in range(kernel[0]) for kx in range(kernel[1])
                        for iy, ix in [(y * stride[0] + ky - padding[0], xo * stride[1] + kx - padding[1])]
                        if 0 <= iy < h and 0 <= ix < w]
                windows.append(taps)
                divisors.append(kernel[0] * kernel[1] if count_include_pad else len(taps))
    return windows, divisors, (n * c * oh, ow)


def avg_pool2d_bf16(eng, x_buf: int, shape, kernel, stride, padding=(0, 0), count_include_pad=True) -> int:
    """`avg_pool2d` of a BF16 tensor (pool.rs:254-275): the window means in F32 by `pool_bf16`, rounded once to
    BF16.  Returns the [n c oh, ow] BF16 buffer."""
    windows, divisors, dims = avg_pool2d_windows(shape, kernel, stride, padding, count_include_pad)
    wide, _ = eng.pool_bf16(x_buf, windows, divisors, dims)
    out, _ = eng.cast_float(wide, True)
    eng.free(wide)
    return out


# ------------------------------------------------------------------------- generation (decode steps)
def _int_scalar(v: int) -> float:
    """An integer kind's scalar travels as the bits of the op's F32 scalar field (tensor.rs:3785)."""
    return float(np.array([v], dtype=np.int32).view(np.float32)[0])


class LlamaDecode:
    """Token-by-token generation with a fixed-shape key/value cache, as the reference traces it
    (crates/tt-models/src/kv_cache.rs:1-30, generate.rs:781): `batch` sequences advance in lockstep, one
    token each a step.  A layer's cache is position-major, [batch * max_len, kv_heads * head_dim] BF16:
    a step writes its projection's rows as they are (`scatter_rows_into`, server.rs:389) and attention
    reads each head's column block in place (`attention_rows`, server.rs:257), the positions later than
    the step's masked.  The position is a device tensor, so one captured step serves every position:
    the step derives its cache rows, its RoPE rows and its mask from `pos`, and at its end advances
    `pos`, feeds its argmax back as the next ids and records it in `tokens` -- a generation is then
    one replay a token with nothing read back until the end.

    `weights_dev`: the device weights of a `LlamaPrefill` (shared, not copied)."""

    def __init__(self, eng, cfg: LlamaConfig, weights_dev: Dict[str, int], batch: int, max_len: int, attend: int = 0,
                 fused: bool = False, weight_storage: str = "bf16"):
        """fused: the layers of a step as one cooperative launch (`decode_layers`) instead of eleven launches a layer; the
        same steps and roundings, sums in the kernel's own order.  weight_storage "bfp8": the four projections of every
        layer kept as BFP8 (`cast_bfp`; crates/burn-tt/src/storage.rs:117-123), read by the products where they lie."""
        assert max_len % 32 == 0 and cfg.head_dim % 32 == 0
        self.eng, self.cfg, self.batch, self.max_len = eng, cfg, batch, max_len
        self.attend = attend or max_len                  # positions attention reads (kv_cache.rs:195-199)
        assert self.attend % 32 == 0 and self.attend <= max_len
        self.w = dict(weights_dev)
        self.fused = bool(fused)
        self.packed = []
        if weight_storage == "bfp8":
            for l in range(cfg.layers):
                for name in ("qkv", "o", "gate_up", "down"):
                    packed, _ = eng.cast_bfp(self.w[f"l{l}.{name}"], 8)
                    self.w[f"l{l}.{name}"] = packed
                    self.packed.append(packed)
        elif weight_storage != "bf16":
            raise ValueError("weight_storage is 'bf16' or 'bfp8'")
        c = cfg
        self.q_cols, self.kv_cols = c.heads * c.head_dim, c.kv_heads * c.head_dim
        cos, sin = rope_tables(max_len, c.head_dim, c.theta)
        self.cos, self.sin = eng.upload(cos, *cos.shape), eng.upload(sin, *sin.shape)
        z = lambda: eng.zeros_dram((batch * max_len, self.kv_cols), bf16=True)[0]
        self.kc = [z() for _ in range(c.layers)]
        self.vc = [z() for _ in range(c.layers)]
        i32 = lambda a, r, k: eng.upload_bits(np.ascontiguousarray(a, dtype=np.int32).view(np.uint32), r, k, I32)
        self.positions = i32(np.arange(self.attend), 1, self.attend)
        self.row_base = i32(np.arange(batch) * max_len, 1, batch)
        self.pos = i32([0], 1, 1)                        # the step's position: a device tensor
        self.ids = i32(np.zeros(batch), batch, 1)
        self.tokens = i32(np.zeros((max_len, batch)), max_len, batch)
        group = c.heads // c.kv_heads
        hd = c.head_dim
        self.items = eng.attention_item_array(
            [((b, h * hd), (b * max_len, (h // group) * hd), (b * max_len, (h // group) * hd))
             for b in range(batch) for h in range(c.heads)])
        self.trace = None
        if self.fused:
            from .engine import DecodeShape
            self.shape = DecodeShape(c.layers, c.hidden, c.heads, c.kv_heads, c.head_dim, c.ff, max_len, self.attend, c.eps,
                                     1.0 / float(np.sqrt(hd)))
            self.layer_ids = [i for l in range(c.layers)
                              for i in (self.w[f"l{l}.norm1"], self.w[f"l{l}.qkv"], self.w[f"l{l}.o"], self.w[f"l{l}.norm2"],
                                        self.w[f"l{l}.gate_up"], self.w[f"l{l}.down"], self.kc[l], self.vc[l])]

    def reset(self, ids: np.ndarray, position: int = 0):
        """Start (or restart) at `position` with these ids ([batch] I32) as the next input."""
        e = self.eng
        fresh = e.upload_bits(np.ascontiguousarray(ids, dtype=np.int32).reshape(self.batch, 1).view(np.uint32), self.batch, 1, I32)
        p = e.upload_bits(np.array([[position]], np.int32).view(np.uint32), 1, 1, I32)
        e.copy_into(fresh, self.ids); e.copy_into(p, self.pos)
        e.free(fresh); e.free(p)

    def continue_from(self, ids_buf: int, position: int):
        """Go on from a prompt a `LlamaPrefill.forward(..., cache=self)` wrote: `ids_buf` ([batch, 1] I32, the
        prefill's argmax) becomes the next input and `position` (the prompt's length) the next position.
        Nothing is read back."""
        e = self.eng
        p = e.upload_bits(np.array([[position]], np.int32).view(np.uint32), 1, 1, I32)
        e.copy_into(ids_buf, self.ids); e.copy_into(p, self.pos)
        e.free(p)

    def set_ids(self, ids: np.ndarray):
        """Overwrite the next input ids (teacher forcing); the position is untouched."""
        e = self.eng
        fresh = e.upload_bits(np.ascontiguousarray(ids, dtype=np.int32).reshape(self.batch, 1).view(np.uint32), self.batch, 1, I32)
        e.copy_into(fresh, self.ids)
        e.free(fresh)

    def step(self):
        """One token a sequence at `pos`.  Returns (logits [batch, vocab] F32, argmax [batch, 1] I32); the
        caller frees both.  Advances `pos`, feeds the argmax back into `ids` and records it in `tokens`."""
        e, c, K = self.eng, self.cfg, kinds
        B, hd = self.batch, c.head_dim
        op = lambda kind, a, b=None, s1=0.0: e.eltwise_op(EltwiseOp(kind, s1, 0.0), a, b)[0]
        if self.fused:
            emb, _ = e.select_rows(self.w["embed"], self.ids)
            x, _ = e.cast_float(emb, False)
            e.free(emb)
            n1, _ = e.decode_layers(self.shape, x, self.layer_ids, self.w["final_norm"], self.cos, self.sin, self.pos)
            e.free(x)
            return self._head_and_advance(n1, op)
        rows = op(K.INT_ADD, self.row_base, self.pos)                         # each sequence's cache row
        later = op(K.INT_GT, self.positions, self.pos)                        # kv_cache.rs:216-224 `later`
        cs, _ = e.select_rows(self.cos, self.pos)                             # the position's RoPE row
        sn, _ = e.select_rows(self.sin, self.pos)
        emb, _ = e.select_rows(self.w["embed"], self.ids)
        x, _ = e.cast_float(emb, False)
        e.free(emb)
        n1, _ = e.rms_norm_as(x, self.w["l0.norm1"], c.eps, True)
        scale = 1.0 / float(np.sqrt(hd))
        qk_cols = self.q_cols + self.kv_cols
        for l in range(c.layers):
            qkv, _ = e.matmul_dram_bf16(n1, False, self.w[f"l{l}.qkv"], False)
            e.free(n1)
            # RoPE on the query and key heads together, F32: the queries are read as they are, the keys are
            # rounded once to BF16 as they are written into the cache
            qk, _ = e.rope_blocks((qkv, (0, 0), (B, qk_cols)), (cs, (0, 0), (1, hd)), (sn, (0, 0), (1, hd)), hd, False)
            e.scatter_rows_into(self.kc[l], rows, (qk, (0, self.q_cols), (B, self.kv_cols)))
            e.scatter_rows_into(self.vc[l], rows, (qkv, (0, qk_cols), (B, self.kv_cols)))
            e.free(qkv)
            att, _ = e.attention_rows_as([qk, self.kc[l], self.vc[l], later], self.items, [1, hd, self.attend, hd], scale, True)
            e.free(qk)
            attb, _ = e.reshape(att, B, self.q_cols)                          # [1, B heads hd] as [B, heads hd]
            e.free(att)
            o, _ = e.matmul_dram(attb, False, self.w[f"l{l}.o"], False)
            e.free(attb)
            (x2, _), (n2, _) = e.add_rms_norm_as(x, o, self.w[f"l{l}.norm2"], c.eps, True)
            e.free(x); e.free(o)
            gu, _ = e.matmul_dram_bf16(n2, False, self.w[f"l{l}.gate_up"], False)
            e.free(n2)
            act, _ = e.eltwise_blocks_as(EltwiseOp(K.SILU_MUL, 0.0, 0.0), (gu, (0, 0), (B, c.ff)),
                                         (gu, (0, c.ff), (B, c.ff)), None, True)
            e.free(gu)
            d, _ = e.matmul_dram(act, False, self.w[f"l{l}.down"], False)
            e.free(act)
            nxt = self.w[f"l{l + 1}.norm1"] if l + 1 < c.layers else self.w["final_norm"]
            (x, _), (n1, _) = e.add_rms_norm_as(x2, d, nxt, c.eps, True)
            e.free(x2); e.free(d)
        e.free(x)
        for i in (rows, later, cs, sn):
            e.free(i)
        return self._head_and_advance(n1, op)

    def _head_and_advance(self, n1: int, op):
        """The tied head on the stream's final norm, its argmax, and the step's bookkeeping: record, feed back, advance."""
        e, K, B = self.eng, kinds, self.batch
        logits, _ = e.matmul_dram(n1, False, self.w["embed"], True)          # tied head
        e.free(n1)
        am, _ = e.argmax_row(logits)
        am_row, _ = e.reshape(am, 1, B)
        e.scatter_rows_into(self.tokens, self.pos, (am_row, (0, 0), (1, B)))
        e.free(am_row)
        e.copy_into(am, self.ids)
        nxt_pos = op(K.INT_ADD_S, self.pos, None, _int_scalar(1))
        e.copy_into(nxt_pos, self.pos)
        e.free(nxt_pos)
        return logits, am

    def capture(self):
        """One eager step (so every kernel is loaded and every block list is on the device), the
        position put back, then the step captured.  Returns the (logits, argmax) buffers a replay rewrites."""
        e = self.eng
        lg, am = self.step()
        e.free(lg); e.free(am)
        back = e.eltwise_op(EltwiseOp(kinds.INT_SUB_S, _int_scalar(1), 0.0), self.pos, None)[0]
        e.copy_into(back, self.pos)
        e.free(back)
        e.begin_trace()
        out = self.step()
        self.trace = e.end_trace()
        return out

    def replay(self):
        self.eng.run_trace(self.trace)

    def generated(self, first: int, count: int) -> np.ndarray:
        """The tokens recorded at positions first .. first + count - 1: [count, batch] I32."""
        return self.eng.download_bits(self.tokens).view(np.int32)[first:first + count]

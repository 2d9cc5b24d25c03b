"""Writes tests/golden/llama_prefill_8x512.npz: what the CPU restatement (oracle/models.py, F32 on the BF16-rounded
weights) gives for the benchmark's SmolLM2-135M-shape prefill -- 30 layers, vocabulary 49,152, 8 sequences of 512
tokens, weights `workloads.llama_weights()` and ids `workloads.prefill_ids()` -- so a run that has no half minute of
host time for the restatement can still hold its logits to it: per sequence the argmax, the margin between the two
largest logits, and the logits at 96 sampled vocabulary columns plus the two largest.

    python tests/golden/make_llama_prefill_golden.py        (about a minute on eight cores)
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from metalium_rs_b200 import workloads as W   # noqa: E402
from oracle import models as M                # noqa: E402
from oracle import oracle as orc              # noqa: E402

if __name__ == "__main__":
    cfg = W.LlamaConfig()
    batch, seq = 8, 512
    w = W.llama_weights(cfg)
    wb = {k: orc.from_bf16(orc.to_bf16(v)) for k, v in w.items()}
    ids = W.prefill_ids(cfg, batch, seq)
    logits = M.llama_prefill(cfg, wb, ids, batch, seq)
    order = np.argsort(logits, axis=1)
    top2 = order[:, -2:]
    cols = np.random.default_rng(96).choice(cfg.vocab, 96, replace=False)
    columns = np.concatenate([np.tile(cols, (batch, 1)), top2], axis=1).astype(np.int32)      # [batch, 98]
    np.savez(Path(__file__).resolve().parent / "llama_prefill_8x512.npz",
             argmax=order[:, -1].astype(np.int32),
             margin=(np.take_along_axis(logits, top2[:, 1:], 1) - np.take_along_axis(logits, top2[:, :1], 1)).ravel().astype(np.float32),
             columns=columns, logits=np.take_along_axis(logits, columns, 1).astype(np.float32),
             ids_checksum=np.array([int(ids.astype(np.int64).sum())], np.int64))
    print("written; margins", (np.take_along_axis(logits, top2[:, 1:], 1) - np.take_along_axis(logits, top2[:, :1], 1)).ravel())

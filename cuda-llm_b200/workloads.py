"""Seeded synthetic inputs for the five benchmark / parity configurations.

No public dataset is involved anywhere on this path: every input is drawn from
``numpy.random.default_rng(seed)`` (PCG64) with the shapes, dtypes and value
distributions the configurations name.  fp16 tensors are the float32 draw cast
with numpy's round-to-nearest-even, and the SAME bit pattern is handed to the GPU
path and to the CPU oracle.  Everything here is numpy only.
"""
from __future__ import annotations

import numpy as np

VOCAB = 151936
EPS = 1e-6
THETA = 1e6
Q_HEADS, KV_HEADS, HEAD_DIM = 16, 8, 128


def normal(rng, shape, sigma=1.0, dtype=np.float32):
    a = rng.standard_normal(shape, dtype=np.float32)
    if sigma != 1.0:
        a *= np.float32(sigma)
    return a.astype(dtype) if dtype != np.float32 else a


def gamma(rng, n, dtype=np.float32):
    """Norm weight ~U(0.5, 1.5)."""
    g = rng.random(n, dtype=np.float32) + np.float32(0.5)
    return g.astype(dtype) if dtype != np.float32 else g


def config1(seed=1001, with_table=True):
    """Qwen3-0.6B-shaped single-layer op set at 4 tokens, fp32."""
    rng = np.random.default_rng(seed)
    d = {
        "x": normal(rng, (4, 1024)), "res": normal(rng, (4, 1024)), "gamma": gamma(rng, 1024),
        "q": normal(rng, (4, Q_HEADS, HEAD_DIM)), "k": normal(rng, (4, KV_HEADS, HEAD_DIM)),
        "gamma_q": gamma(rng, HEAD_DIM), "gamma_k": gamma(rng, HEAD_DIM),
        "positions": np.arange(4, dtype=np.int32),
        "gate": normal(rng, (4, 3072)), "up": normal(rng, (4, 3072)),
        "ids": rng.integers(0, VOCAB, 4).astype(np.int32),
        "logits": normal(rng, (4, VOCAB)),
    }
    if with_table:
        d["table"] = normal(np.random.default_rng(seed + 1), (VOCAB, 1024), 0.02)
    return d


C2_ROWS = (1, 64, 4096, 65536)
C2_HIDDEN = (1024, 2048, 4096)


def config2(rows, hidden, seed=None, dtype=np.float16):
    """Fused residual-add + RMSNorm: x, residual ~N(0,1), gamma ~U(0.5,1.5)."""
    if seed is None:
        seed = 2000 + C2_ROWS.index(rows) * len(C2_HIDDEN) + C2_HIDDEN.index(hidden)
    rng = np.random.default_rng(seed)
    return {"x": normal(rng, (rows, hidden), dtype=dtype), "res": normal(rng, (rows, hidden), dtype=dtype),
            "gamma": gamma(rng, hidden, dtype=dtype)}


def packed_positions(rng, tokens=16384, sequences=64, max_len=512):
    """Concatenated 0..len-1 ramps of `sequences` random lengths in [1, max_len] summing to `tokens`."""
    if not sequences <= tokens <= sequences * max_len:
        raise ValueError("packed_positions: tokens cannot be split into that many sequences")
    while True:
        lens = rng.integers(1, max_len + 1, sequences - 1)
        last = tokens - int(lens.sum())
        if 1 <= last <= max_len:
            lens = np.append(lens, last)
            break
    return np.concatenate([np.arange(n, dtype=np.int32) for n in lens]), lens.astype(np.int64)


def config3(seed=3001, tokens=16384, dtype=np.float16):
    """Packed-prefill RoPE + QK RMSNorm."""
    rng = np.random.default_rng(seed)
    sequences = max(1, tokens // 256)   # 64 sequences at the full size, mean length 256
    positions, lens = packed_positions(rng, tokens, sequences, 512)
    return {"positions": positions, "lens": lens,
            "q": normal(rng, (tokens, Q_HEADS, HEAD_DIM), dtype=dtype),
            "k": normal(rng, (tokens, KV_HEADS, HEAD_DIM), dtype=dtype),
            "gamma_q": gamma(rng, HEAD_DIM, dtype=dtype), "gamma_k": gamma(rng, HEAD_DIM, dtype=dtype)}


def config4_swiglu(tokens, inter, seed=4001, dtype=np.float16):
    """SwiGLU inputs: gate, up ~N(0,2)."""
    rng = np.random.default_rng(seed)
    return {"gate": normal(rng, (tokens, inter), 2.0, dtype), "up": normal(rng, (tokens, inter), 2.0, dtype)}


def config4_gather(tokens, hidden=4096, vocab=VOCAB, seed=4002, dtype=np.float16):
    """Embedding gather: table ~N(0,0.02), ids uniform in [0, vocab)."""
    rng = np.random.default_rng(seed)
    return {"table": normal(rng, (vocab, hidden), 0.02, dtype),
            "ids": rng.integers(0, vocab, tokens).astype(np.int32)}


def config5(rows=256, vocab=VOCAB, seed=5001):
    """LM-head logits ~N(0,4) with one planted maximum per row."""
    rng = np.random.default_rng(seed)
    logits = normal(rng, (rows, vocab), 4.0)
    planted = rng.integers(0, vocab, rows).astype(np.int32)
    logits[np.arange(rows), planted] = logits.max(axis=1) + np.float32(1.0)
    return {"logits": logits, "planted": planted}


def lm_head_case(rows=4, hidden=1024, vocab=VOCAB, seed=6001, dtype=np.float16):
    """Decode-size LM head: final-norm outputs ~N(0,1) against a tied embedding table ~N(0,0.02)
    (the table of configurations 1 and 4), Qwen3-0.6B shape by default."""
    rng = np.random.default_rng(seed)
    return {"hidden": normal(rng, (rows, hidden), 1.0, dtype), "table": normal(rng, (vocab, hidden), 0.02, dtype)}


def shard_range(total, world, rank):
    """Contiguous [lo, hi) slice of `total` units owned by `rank` of `world`."""
    return total * rank // world, total * (rank + 1) // world

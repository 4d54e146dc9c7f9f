"""Seeded synthetic post-RoPE K/V/q tensors with the distribution the benchmark
configurations name: standard-normal entries times a per-channel log-normal(0, 0.5)
scale, with 2 % of the key channels of each head scaled by a further x20.

They stand in for real activations only in shape and in the two properties the
compressed format is sensitive to (per-channel scale spread, a few large key
channels).  The reference's own KV benchmarks use the same kind of stand-in
(``benchmarks/p5_triton_bench.py:52-60``).
"""

from __future__ import annotations

import numpy as np


def channel_scales(rng: np.random.Generator, n_heads: int, head_dim: int,
                   outlier_frac: float = 0.02, outlier_gain: float = 20.0):
    """Per-(head, channel) scales for keys and values.

    Keys: exp(N(0, 0.5)), and exactly ``round(outlier_frac * D)`` channels per head
    (drawn without replacement) are multiplied by ``outlier_gain``.  Values: an
    independent exp(N(0, 0.5)) draw.
    """
    sk = np.exp(rng.normal(0.0, 0.5, size=(n_heads, head_dim)))
    sv = np.exp(rng.normal(0.0, 0.5, size=(n_heads, head_dim)))
    n_out = int(round(outlier_frac * head_dim))
    for h in range(n_heads):
        if n_out:
            ch = rng.choice(head_dim, size=n_out, replace=False)
            sk[h, ch] *= outlier_gain
    return sk.astype(np.float32), sv.astype(np.float32)


def make_kv(seed: int, n_heads: int, n_tokens: int, head_dim: int = 128,
            dtype=np.float32):
    """Keys and values of one sequence, shape (n_tokens, n_heads, head_dim).

    ``dtype`` float16 rounds the tensors to half precision (returned as float16), so
    that a 16-bit hot window holds them losslessly.
    """
    rng = np.random.default_rng(seed)
    sk, sv = channel_scales(rng, n_heads, head_dim)
    k = rng.standard_normal((n_tokens, n_heads, head_dim)).astype(np.float32) * sk
    v = rng.standard_normal((n_tokens, n_heads, head_dim)).astype(np.float32) * sv
    return k.astype(dtype), v.astype(dtype)


def make_q(seed: int, n_q_heads: int, head_dim: int = 128, dtype=np.float32):
    """One decode-step query, N(0, 1), shape (n_q_heads, head_dim)."""
    rng = np.random.default_rng(seed + 0x5EED)
    return rng.standard_normal((n_q_heads, head_dim)).astype(np.float32).astype(dtype)

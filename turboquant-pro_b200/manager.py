"""TurboQuantKVManager — the reference's multi-layer cache manager on one GPU context.

Same methods and statistics as ``turboquant_pro.vllm_plugin.TurboQuantKVManager``
(``vllm_plugin.py:64-260``): ``store`` / ``load`` / ``length`` / ``clear`` / ``layer_stats``
/ ``memory_stats`` / ``estimate_capacity``.  Where the reference builds one numpy cache per
layer, all layers here are rows of a single :class:`KVContext`, and :meth:`attend` answers a
decode-step query on the codes instead of loading dense K/V.

The reference's default (``bits=3``: 3-bit uniform keys) has no device form here; keys are
4-bit, asymmetric NF4 with outliers by default (``robust=True``, what
``AutoConfig.build_cache`` gives) or the plain uniform grid (``robust=False``).
"""

from __future__ import annotations

import logging
from dataclasses import dataclass

import numpy as np

from .context import KVContext

logger = logging.getLogger(__name__)

__all__ = ["LayerStats", "TurboQuantKVManager"]


@dataclass
class LayerStats:
    """Statistics of one layer's cache (``vllm_plugin.py:47-61``)."""

    layer_id: int
    length: int
    cold_length: int
    hot_length: int
    cold_bytes: int
    hot_bytes: int
    total_bytes: int
    uncompressed_bytes: int
    compression_ratio: float


class TurboQuantKVManager:
    """Per-layer two-tier caches of one sequence, for a whole transformer.

    Args:
        n_layers, n_kv_heads, head_dim, bits, key_bits, value_bits, hot_window, device_id:
            as in the reference.  ``use_gpu`` is accepted and ignored (the cache is always on
            the GPU).
        n_q_heads: query heads served by :meth:`attend` (default: ``n_kv_heads``).
        robust, outlier_frac: key format, see the module docstring.
        max_tokens: capacity of every layer.
        dtype: element type of the hot window.
    """

    def __init__(self, n_layers: int = 32, n_kv_heads: int = 8, head_dim: int = 128, bits: int = 3,
                 key_bits: int | None = None, value_bits: int | None = None,
                 hot_window: int = 512, use_gpu: bool = True, device_id: int = 0, *,
                 n_q_heads: int | None = None, robust: bool = True, outlier_frac: float = 0.02,
                 max_tokens: int = 32768, dtype="float32", seed: int | None = None) -> None:
        self._n_layers, self._n_kv_heads, self._head_dim = n_layers, n_kv_heads, head_dim
        self._bits = bits
        self._key_bits = key_bits if key_bits is not None else (4 if robust else bits)
        self._value_bits = value_bits if value_bits is not None else bits
        self._hot_window = hot_window
        if self._key_bits != 4:
            raise NotImplementedError("the CUDA path implements 4-bit per-channel keys: pass "
                                      "key_bits=4 (or robust=True)")
        self._ctx = KVContext(
            n_layers=n_layers, n_seqs=1, n_kv_heads=n_kv_heads,
            n_q_heads=n_q_heads or n_kv_heads, head_dim=head_dim, key_bits=4,
            value_bits=self._value_bits, hot_window=hot_window,
            outlier_frac=outlier_frac if robust else 0.0, max_tokens_per_seq=max_tokens,
            kv_dtype=dtype, seed=seed, device=device_id,
            key_mode="nf4_asym" if robust else "uniform")
        logger.info("TurboQuantKVManager: %d layers, %d heads, %d head_dim, key=%d, value=%d, "
                    "hot_window=%d", n_layers, n_kv_heads, head_dim, self._key_bits,
                    self._value_bits, hot_window)

    @property
    def n_layers(self) -> int:
        return self._n_layers

    @property
    def context(self) -> KVContext:
        return self._ctx

    # ----------------------------------------------------------------- store / load ----
    def _tokens(self, x, what):
        import torch

        t = x if isinstance(x, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(x))
        if t.dim() == 4:  # (1, H, T, D) -> (T, H, D)
            t = t[0].permute(1, 0, 2)
        elif t.dim() == 2:  # (H, D)
            t = t[None]
        if t.dim() != 3 or t.shape[1] != self._n_kv_heads or t.shape[2] != self._head_dim:
            raise ValueError(f"{what}: expected (H, D), (T, H, D) or (1, H, T, D) with "
                             f"{self._n_kv_heads} heads of dim {self._head_dim}")
        return t.to(device=self._ctx.device, dtype=self._ctx.kv_dtype)[None].contiguous()

    def store(self, layer_id: int, keys, values) -> None:
        """Append the K/V of one token (or several) to a layer."""
        self._ctx.append(layer_id, self._tokens(keys, "keys"), self._tokens(values, "values"))

    def load(self, layer_id: int, start: int = 0, end: int | None = None):
        """Dequantised ``(keys, values)`` of tokens ``[start, end)``, each a float32 numpy
        array ``(1, n_kv_heads, length, head_dim)``."""
        n = self.length(layer_id)
        end = n if end is None else min(end, n)
        start = max(0, start)
        if end <= start:
            z = np.zeros((1, self._n_kv_heads, 0, self._head_dim), dtype=np.float32)
            return z, z.copy()
        k, v = self._ctx.dequant(layer_id, 0, start, end)
        return k.cpu().numpy()[None], v.cpu().numpy()[None]

    def attend(self, layer_id: int, query):
        """Decode-step attention output of a layer, computed on the codes: ``query``
        ``(n_q_heads, head_dim)`` (numpy or CUDA tensor) -> same kind, float32."""
        import torch

        is_np = not isinstance(query, torch.Tensor)
        q = torch.from_numpy(np.ascontiguousarray(query, dtype=np.float32)) if is_np else query
        q = q.reshape(1, self._ctx.n_q_heads, self._head_dim).to(self._ctx.device)
        if self.length(layer_id) == 0:
            raise RuntimeError("cache is empty")
        out = self._ctx.decode(layer_id, q)[0]
        return out.cpu().numpy() if is_np else out

    def length(self, layer_id: int = 0) -> int:
        return self._ctx.lengths(layer_id, 0)[0]

    def clear(self) -> None:
        for layer in range(self._n_layers):
            self._ctx.clear(layer, 0)

    # ------------------------------------------------------------------------ stats ----
    def layer_stats(self, layer_id: int) -> LayerStats:
        total, cold_len, hot_len = self._ctx.lengths(layer_id, 0)
        cold, hot = self._ctx.memory_stats(layer_id, 0)
        unc = total * self._n_kv_heads * self._head_dim * 4 * 2  # float32 keys + values
        return LayerStats(layer_id=layer_id, length=total, cold_length=cold_len,
                          hot_length=hot_len, cold_bytes=cold, hot_bytes=hot,
                          total_bytes=cold + hot, uncompressed_bytes=unc,
                          compression_ratio=unc / max(cold + hot, 1))

    def memory_stats(self) -> dict:
        """Aggregate over the layers, with the reference's keys (``vllm_plugin.py:208-240``)."""
        stats = [self.layer_stats(i) for i in range(self._n_layers)]
        cold = sum(s.cold_bytes for s in stats)
        hot = sum(s.hot_bytes for s in stats)
        unc = sum(s.uncompressed_bytes for s in stats)
        total = cold + hot
        mb = 1048576
        return {
            "n_layers": self._n_layers,
            "total_tokens": max((s.length for s in stats), default=0),
            "cold_bytes": cold, "hot_bytes": hot, "total_bytes": total,
            "total_mb": round(total / mb, 1),
            "uncompressed_bytes": unc, "uncompressed_mb": round(unc / mb, 1),
            "compression_ratio": round(unc / max(total, 1), 1) if total > 0 else 1.0,
            "saved_mb": round((unc - total) / mb, 1),
            "bits": self._bits, "hot_window": self._hot_window,
        }

    def estimate_capacity(self, max_memory_gb: float) -> int:
        """Context length that fits ``max_memory_gb``: the hot window at its stored width,
        everything older at the compressed bytes per token of this format."""
        g = self._ctx.geom
        per_tok_hot = self._n_layers * self._n_kv_heads * self._head_dim * 2 * \
            (4 if g.kv_dtype == 0 else 2)
        blk = (g.block_tokens * self._head_dim * (4 + self._value_bits) // 8 + 4 * g.block_tokens
               + 8 * self._head_dim + 6 * g.outlier_k * self._head_dim)
        per_tok_cold = self._n_layers * self._n_kv_heads * blk / g.block_tokens
        budget = max_memory_gb * 1e9 - self._hot_window * per_tok_hot
        if budget <= 0:
            return int(max_memory_gb * 1e9 // per_tok_hot)
        return self._hot_window + int(budget // per_tok_cold)

"""AutoConfig — model-aware factory for the GPU cache.

Keeps the public surface of ``turboquant_pro.autoconfig.AutoConfig``
(``autoconfig.py:179-486``): the same dataclass fields, ``from_dict`` /
``from_pretrained`` constructors, target presets and ``build_cache`` keywords, so
``AutoConfig.from_pretrained("llama-3-8b").build_cache(use_gpu=True)`` keeps working and
returns the B200-native cache.  ``build_context`` is the batched, multi-layer extension.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass

import numpy as np

logger = logging.getLogger(__name__)

# (head_dim, query heads, KV heads, layers, rope theta, max positions) of the models the
# reference's registry knows (autoconfig.py:51-116).
_MODELS = {
    "llama-3-8b": (128, 32, 8, 32, 500000.0, 8192),
    "llama-3-70b": (128, 64, 8, 80, 500000.0, 8192),
    "gemma-2-27b": (128, 32, 16, 46, 10000.0, 8192),
    "gemma-2-9b": (256, 16, 8, 42, 10000.0, 8192),
    "gemma-4-27b-a4b": (256, 8, 1, 48, 10000.0, 262144),
    "qwen2.5-7b": (128, 28, 4, 28, 1000000.0, 131072),
    "qwen2.5-72b": (128, 64, 8, 80, 1000000.0, 131072),
    "mistral-7b": (128, 32, 8, 32, 10000.0, 32768),
}

_ALIASES = {
    "meta-llama/llama-3-8b": "llama-3-8b",
    "meta-llama/meta-llama-3-8b": "llama-3-8b",
    "meta-llama/llama-3-70b": "llama-3-70b",
    "meta-llama/meta-llama-3-70b": "llama-3-70b",
    "google/gemma-2-27b": "gemma-2-27b",
    "google/gemma-2-9b": "gemma-2-9b",
    "google/gemma-4-27b-a4b": "gemma-4-27b-a4b",
    "qwen/qwen2.5-7b": "qwen2.5-7b",
    "qwen/qwen2.5-72b": "qwen2.5-72b",
    "mistralai/mistral-7b-v0.1": "mistral-7b",
    "mistralai/mistral-7b": "mistral-7b",
}

# target preset -> (key_bits, value_bits, rope_aware)   (autoconfig.py:145-171)
_PRESETS = {
    "quality": (4, 4, True),
    "balanced": (4, 3, True),
    "compression": (4, 2, True),
    "extreme": (2, 2, False),
}


def _registry_dict(name: str) -> dict:
    hd, nq, nkv, nl, theta, maxpos = _MODELS[name]
    return dict(head_dim=hd, num_attention_heads=nq, num_key_value_heads=nkv,
                num_hidden_layers=nl, rope_theta=theta, max_position_embeddings=maxpos)


def rope_long_wavelength_mask(rope_theta: float, head_dim: int, window: int) -> np.ndarray:
    """``(head_dim,)`` booleans: the channels whose rotary wavelength is longer than ``window``
    tokens, i.e. those that carry the keys' DC offset over a block of that length
    (``per_channel_kv.py:233-241``).  In the rotate-half layout channel ``d`` turns with
    angular frequency ``theta ** (-2 (d mod D/2) / D)``."""
    half = head_dim // 2
    inv_freq = rope_theta ** (-2.0 * np.arange(half) / head_dim)
    wavelength = 2.0 * np.pi / inv_freq
    return np.tile(wavelength, 2)[:head_dim] > float(window)


def rope_averaged_bias(k_bias, rope_theta: float, head_dim: int, start: int, n: int) -> np.ndarray:
    """``(n_heads, head_dim)`` float32: the key-projection bias seen through RoPE, averaged
    over the positions ``[start, start + n)`` of a block — the zero-point of the reference's
    ``zero_point="bias"`` mode (``per_channel_kv.py:243-267``).  cos and sin are averaged in
    float64 and rounded to float32; rotate-half layout."""
    half = head_dim // 2
    inv_freq = rope_theta ** (-2.0 * np.arange(half, dtype=np.float64) / head_dim)
    angle = np.arange(start, start + n, dtype=np.float64)[:, None] * inv_freq[None, :]
    cos_mean, sin_mean = np.cos(angle).mean(axis=0), np.sin(angle).mean(axis=0)
    cos_full = np.concatenate([cos_mean, cos_mean]).astype(np.float32)
    sin_full = np.concatenate([sin_mean, sin_mean]).astype(np.float32)
    b = np.asarray(k_bias, dtype=np.float32).reshape(-1, head_dim)
    turned = np.concatenate([-b[:, half:], b[:, :half]], axis=1)
    return b * cos_full[None, :] + turned * sin_full[None, :]


@dataclass
class AutoConfig:
    """Model geometry + compression target; ``build_*`` produce configured caches."""

    head_dim: int = 128
    n_kv_heads: int = 8
    n_layers: int = 32
    rope_theta: float = 10000.0
    max_seq_len: int = 8192
    key_bits: int = 4
    value_bits: int = 3
    rope_aware: bool = True
    target: str = "balanced"
    model_name: str = ""
    key_zero_point: str = "auto"
    n_q_heads: int = 0  # query heads (0 = same as n_kv_heads); used by build_context

    @classmethod
    def from_dict(cls, config: dict, target: str = "balanced", **overrides) -> "AutoConfig":
        """From a HuggingFace-style config dict (``num_key_value_heads``,
        ``num_hidden_layers``, ``rope_theta`` ...), then the preset, then overrides."""
        if target not in _PRESETS:
            raise ValueError(f"Unknown target '{target}'. Choose from: {sorted(_PRESETS)}")
        kb, vb, ra = _PRESETS[target]
        head_dim = config.get("head_dim")
        n_heads = config.get("num_attention_heads", 32)
        if head_dim is None:
            head_dim = config.get("hidden_size", 4096) // n_heads
        kwargs = dict(
            head_dim=head_dim,
            n_kv_heads=config.get("num_key_value_heads", n_heads),
            n_layers=config.get("num_hidden_layers", 32),
            rope_theta=config.get("rope_theta", 10000.0),
            max_seq_len=config.get("max_position_embeddings", 8192),
            key_bits=kb, value_bits=vb, rope_aware=ra, target=target,
            model_name=config.get("model_type", ""),
            n_q_heads=n_heads,
        )
        kwargs.update(overrides)
        return cls(**kwargs)

    @classmethod
    def from_pretrained(cls, model_name_or_path: str, target: str = "balanced",
                        **overrides) -> "AutoConfig":
        """From the built-in registry (or its aliases), else from
        ``transformers.AutoConfig`` when that package can resolve the name."""
        key = model_name_or_path.lower().strip("/")
        key = _ALIASES.get(key, key)
        if key in _MODELS:
            cfg = cls.from_dict(_registry_dict(key), target=target, **overrides)
            cfg.model_name = key
            return cfg
        try:
            from transformers import AutoConfig as HFAutoConfig

            cfg = cls.from_dict(HFAutoConfig.from_pretrained(model_name_or_path).to_dict(),
                                target=target, **overrides)
            cfg.model_name = model_name_or_path
            return cfg
        except ImportError:
            pass
        except Exception as e:  # noqa: BLE001 - mirror the reference: warn, then fail below
            logger.warning("Failed to load HF config for '%s': %s", model_name_or_path, e)
        raise ValueError(
            f"Could not resolve model '{model_name_or_path}'. Known models: {sorted(_MODELS)}. "
            "Install 'transformers' for HuggingFace Hub lookup, or pass a config dict via "
            "AutoConfig.from_dict().")

    @property
    def is_qwen_family(self) -> bool:
        return "qwen" in (self.model_name or "").lower()

    def resolve_key_zero_point(self, has_k_bias: bool) -> str:
        """``"auto"`` -> ``"bias"`` for Qwen-family models given a k_proj bias, else
        ``"calibrated"`` (autoconfig.py:390-416)."""
        mode = self.key_zero_point
        if mode == "auto":
            return "bias" if (self.is_qwen_family and has_k_bias) else "calibrated"
        if mode == "bias" and not has_k_bias:
            raise ValueError('key_zero_point="bias" requires k_bias (per-layer k_proj bias)')
        return mode

    def build_cache(self, hot_window: int = 512, use_gpu: bool = False, seed: int | None = None,
                    robust: bool = True, outlier_frac: float = 0.02, k_bias=None, **kwargs):
        """A configured :class:`TurboQuantKVCache` (``autoconfig.py:439-486``).

        This package is GPU-only, so the cache lives on the GPU whatever ``use_gpu`` says
        (the keyword is kept so existing call sites work).  ``robust=False`` gives the bare
        uniform 4-bit key grid without outliers, as in the reference.
        """
        from .cache import TurboQuantKVCache

        zp = self.resolve_key_zero_point(k_bias is not None) if robust else "calibrated"
        return TurboQuantKVCache(
            head_dim=self.head_dim, n_heads=self.n_kv_heads, bits=self.value_bits,
            key_bits=self.key_bits, value_bits=self.value_bits, hot_window=hot_window,
            use_gpu=True, seed=seed, key_nf4_asym=robust,
            key_outlier_frac=outlier_frac if robust else 0.0, key_zero_point=zp,
            key_rope_theta=self.rope_theta if zp != "calibrated" else None,
            key_k_bias=k_bias if zp == "bias" else None, **kwargs)

    def build_manager(self, hot_window: int = 512, use_gpu: bool = True, **kwargs):
        """A :class:`TurboQuantKVManager` over all layers of this model
        (``autoconfig.py:516-537``); GPU-resident whatever ``use_gpu`` says."""
        from .manager import TurboQuantKVManager

        return TurboQuantKVManager(n_layers=self.n_layers, n_kv_heads=self.n_kv_heads,
                                   head_dim=self.head_dim, bits=self.value_bits,
                                   key_bits=self.key_bits, value_bits=self.value_bits,
                                   hot_window=hot_window, **kwargs)

    def build_quantizer(self, use_gpu: bool = False, seed: int | None = None):
        """The reference returns its stateless ``TurboQuantKV`` tensor quantiser here
        (``autoconfig.py:359-378``).  This package implements the cache path only: the
        stateless quantiser lives behind the cache (``build_cache``) and the block
        export / import calls, so there is nothing to hand out."""
        raise NotImplementedError(
            "the stateless TurboQuantKV quantiser is not part of the GPU cache path; use "
            "build_cache() / build_context(), or the reference package for tensor-level "
            "compress / decompress")

    def build_context(self, n_seqs: int, max_tokens_per_seq: int | None = None,
                      hot_window: int = 512, seed: int | None = None,
                      outlier_frac: float = 0.02, kv_dtype="float16", n_layers: int | None = None,
                      n_kv_heads: int | None = None, n_q_heads: int | None = None, device: int = 0,
                      key_mode: str = "nf4_asym"):
        """A batched, multi-layer :class:`KVContext` with this model's geometry — what a
        serving engine holds: ``n_layers x n_seqs`` caches, GQA-aware decode.
        ``n_kv_heads`` / ``n_q_heads`` override the model's counts for head-sharded
        (tensor-parallel) deployments."""
        from .context import KVContext

        nkv = n_kv_heads or self.n_kv_heads
        nq = n_q_heads or (self.n_q_heads or self.n_kv_heads) * nkv // self.n_kv_heads
        return KVContext(
            n_layers=n_layers or self.n_layers, n_seqs=n_seqs, n_kv_heads=nkv, n_q_heads=nq,
            head_dim=self.head_dim, key_bits=self.key_bits, value_bits=self.value_bits,
            hot_window=hot_window, outlier_frac=outlier_frac,
            max_tokens_per_seq=max_tokens_per_seq or self.max_seq_len, kv_dtype=kv_dtype,
            seed=seed, device=device, key_mode=key_mode)

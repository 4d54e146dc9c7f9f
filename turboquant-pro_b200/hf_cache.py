"""HuggingFace ``transformers`` (v5) cache adapter on the GPU-resident compressed cache.

Counterpart of the reference's ``hf_cache.py:74-334`` (``TurboQuantLayer`` /
``TurboQuantCache`` / ``enable_turboquant_cache``).  The reference's layer keeps its cold
store in numpy and hands the model *dense* K/V on every step (``hf_cache.py:196-205``).
Here the tokens live in one :class:`KVContext` for the whole model and a decode step is
attended on the codes:

* ``TurboQuantCache(config, ...)`` is passed to ``generate`` / ``forward`` as
  ``past_key_values``; its layers append every new K/V to the context;
* the attention function registered as ``"turboquant"`` (select it with
  ``attn_implementation="turboquant"`` or :func:`enable_turboquant_cache`) answers a
  single-token query with ``KVContext.decode`` and never sees dense history; prompts are
  attended densely on the prompt's own K/V, exactly like the stock implementation.

Differences from the reference adapter, all forced by the paged device format:

* cold blocks follow the core cache's rule (oldest half of an over-full window, i.e. 256
  tokens at ``hot_window`` 512), not the adapter's "whole overflow as one block";
* a query of more than one token against a non-empty cache (chunked prefill, assisted
  decoding), attention masks with padding, ``crop`` / beam reordering fall back to the
  dense getters (``dense=True`` forces that path for every decode step: it is how the
  reference's adapter works, and this adapter's own cross-check);
* capacity (``max_tokens``) is fixed when the context is created.
"""

from __future__ import annotations

import weakref

import torch

try:  # the classes exist from transformers v5 on
    from transformers.cache_utils import Cache, CacheLayerMixin
    _HAS_TRANSFORMERS = True
except Exception:  # noqa: BLE001 - optional dependency
    _HAS_TRANSFORMERS = False

    class Cache:  # type: ignore[no-redef]
        pass

    class CacheLayerMixin:  # type: ignore[no-redef]
        pass

from .context import KVContext

__all__ = ["TurboQuantCache", "TurboQuantLayer", "enable_turboquant_cache",
           "turboquant_attention_forward"]

# How the attention function finds the cache: `update` stamps the key tensor it returns with a
# weak reference to its layer and the length before the append, and the model passes that very
# tensor on to the attention function in the same forward.  A key tensor without the stamp
# (use_cache=False, another cache class, a second model) is attended densely as given, so two
# caches or two models in one process cannot reach each other's history.
_STAMP = "_turboquant_layer"

# decision "this mask hides nothing" for the mask object of the current forward: every layer
# of a step receives the same tensor, so the device is asked once per step, not per layer
_MASK_MEMO: list = [None, False]


def _mask_is_open(mask) -> bool:
    if mask is None:
        return True
    ref = _MASK_MEMO[0]
    if ref is not None and ref() is mask:
        return _MASK_MEMO[1]
    if mask.dtype == torch.bool:
        is_open = bool(mask.all())
    else:
        is_open = not bool((mask < 0).any())
    _MASK_MEMO[0], _MASK_MEMO[1] = weakref.ref(mask), is_open
    return is_open


class _SharedContext:
    """The one KVContext behind all layers of a TurboQuantCache, created at the first
    update (when batch size, KV-head count, head_dim, dtype and device are known)."""

    def __init__(self, n_layers, n_q_heads, hot_window, key_bits, value_bits, outlier_frac,
                 seed, max_tokens):
        self.args = dict(n_layers=n_layers, n_q_heads=n_q_heads, hot_window=hot_window,
                         key_bits=key_bits, value_bits=value_bits, outlier_frac=outlier_frac,
                         seed=seed, max_tokens=max_tokens)
        self.ctx: KVContext | None = None

    def get(self, key_states) -> KVContext:
        if self.ctx is None:
            b, h, _t, d = key_states.shape
            a = self.args
            nq = a["n_q_heads"] or h
            self.ctx = KVContext(
                n_layers=a["n_layers"], n_seqs=b, n_kv_heads=h, n_q_heads=nq, head_dim=d,
                key_bits=a["key_bits"], value_bits=a["value_bits"], hot_window=a["hot_window"],
                outlier_frac=a["outlier_frac"], max_tokens_per_seq=a["max_tokens"],
                kv_dtype=key_states.dtype, seed=a["seed"],
                device=key_states.device.index or 0)
        return self.ctx


class TurboQuantLayer(CacheLayerMixin):
    """One layer of the cache (the v5 ``CacheLayerMixin`` contract)."""

    is_compileable = False
    is_sliding = False

    def __init__(self, shared: _SharedContext, layer_idx: int, dense: bool = False) -> None:
        super().__init__()
        self._shared = shared
        self.layer_idx = int(layer_idx)
        self.dense = bool(dense)
        self._seq_len = 0
        self.is_initialized = False

    # -- lifecycle -------------------------------------------------------------------
    def lazy_initialization(self, key_states, value_states) -> None:
        self.dtype, self.device = key_states.dtype, key_states.device
        self.ctx = self._shared.get(key_states)
        self.is_initialized = True

    # -- the update ------------------------------------------------------------------
    def update(self, key_states, value_states, *args, **kwargs):
        """Append ``[B, H, T, D]`` K/V.  Returns what the attention function needs: the new
        tokens themselves (it reads the history from the context), or, in dense mode and with
        tokens already stored, the whole dequantised history like the reference does.  A
        prompt into an empty cache is attended on its own K/V in both modes (the reference
        already shows it the quantised cold part)."""
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        self.ctx.append(self.layer_idx, key_states.permute(0, 2, 1, 3),
                        value_states.permute(0, 2, 1, 3))
        self._prev_len = self._seq_len
        self._seq_len += int(key_states.shape[-2])
        if self.dense and self._prev_len > 0:
            return self.full()
        setattr(key_states, _STAMP, (weakref.ref(self), self._seq_len))
        return key_states, value_states

    def full(self):
        """Dense ``[B, H, N, D]`` keys and values of everything stored (cold blocks
        dequantised, then the hot window), in the model's dtype."""
        ks, vs = [], []
        for s in range(self.ctx.n_seqs):
            k, v = self.ctx.dequant(self.layer_idx, s, 0, self._seq_len)
            ks.append(k)
            vs.append(v)
        return (torch.stack(ks).to(self.dtype), torch.stack(vs).to(self.dtype))

    # -- sizes / masks -----------------------------------------------------------------
    def get_seq_length(self) -> int:
        return self._seq_len if self.is_initialized else 0

    def get_mask_sizes(self, query_length: int) -> tuple[int, int]:
        return self.get_seq_length() + query_length, 0

    def get_max_cache_shape(self) -> int:
        return -1

    # -- mutation ------------------------------------------------------------------------
    def reset(self) -> None:
        if self.is_initialized:
            self.ctx.clear(self.layer_idx)
            self._seq_len = 0

    def _reload(self, keys, values) -> None:
        self.ctx.clear(self.layer_idx)
        self._seq_len = 0
        if keys.shape[-2] > 0:
            self.ctx.append(self.layer_idx, keys.permute(0, 2, 1, 3), values.permute(0, 2, 1, 3))
            self._seq_len = int(keys.shape[-2])

    def crop(self, max_length: int) -> None:
        """Keep the first ``max_length`` tokens (negative: drop that many from the end); the
        kept tokens are re-encoded from their dequantised values, as in the reference."""
        if not self.is_initialized:
            return
        n = self.get_seq_length()
        if max_length < 0:
            max_length = n - abs(max_length)
        if n <= max_length:
            return
        k, v = self.full()
        self._reload(k[:, :, :max_length], v[:, :, :max_length])

    def reorder_cache(self, beam_idx) -> None:
        if not self.is_initialized or self.get_seq_length() == 0:
            return
        k, v = self.full()
        idx = beam_idx.to(k.device)
        self._reload(k.index_select(0, idx), v.index_select(0, idx))

    def offload(self) -> None:  # the cache is device-resident by construction
        pass

    def prefetch(self) -> None:
        pass


class TurboQuantCache(Cache):
    """``past_key_values`` object holding every layer's K/V in one compressed GPU context.

    Args:
        config: the model's config (``num_hidden_layers``, ``num_attention_heads``), or
            ``None`` with ``n_layers`` / ``n_q_heads`` given explicitly.
        hot_window, key_bits, value_bits, outlier_frac, seed: as in the reference's
            ``TurboQuantCache`` (``hf_cache.py:283-300``).
        max_tokens: capacity per sequence.
        dense: hand the model dense K/V on every step instead of attending on the codes.
    """

    def __init__(self, config=None, hot_window: int = 512, key_bits: int = 4,
                 value_bits: int = 4, outlier_frac: float = 0.02, seed: int = 0,
                 max_tokens: int = 8192, dense: bool = False, n_layers: int | None = None,
                 n_q_heads: int | None = None) -> None:
        if not _HAS_TRANSFORMERS:
            raise ImportError("TurboQuantCache requires transformers v5+")
        if config is not None:
            cfg = config.get_text_config() if hasattr(config, "get_text_config") else config
            n_layers = n_layers or cfg.num_hidden_layers
            n_q_heads = n_q_heads or cfg.num_attention_heads
        if not n_layers:
            raise ValueError("pass the model config, or n_layers (and n_q_heads)")
        self.hot_window, self.key_bits, self.value_bits = hot_window, key_bits, value_bits
        self.outlier_frac, self.seed, self.dense = outlier_frac, seed, dense
        self._shared = _SharedContext(n_layers, n_q_heads, hot_window, key_bits, value_bits,
                                      outlier_frac, seed, max_tokens)
        super().__init__(layers=[TurboQuantLayer(self._shared, i, dense) for i in range(n_layers)])

    @property
    def context(self) -> KVContext | None:
        """The device context (``None`` before the first update)."""
        return self._shared.ctx


def turboquant_attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0,
                                 scaling: float | None = None, is_causal: bool | None = None,
                                 **kwargs):
    """Attention function for ``AttentionInterface``: single-token queries are attended on
    the compressed cache's codes; everything else goes to the stock SDPA implementation on
    the K/V it is given (with a :class:`TurboQuantCache` in its default mode that is only
    right for a prompt into an empty cache; other cases switch the layer to dense K/V)."""
    from transformers.integrations.sdpa_attention import sdpa_attention_forward

    # the key tensor is the one TurboQuantLayer.update returned in this forward, or the call
    # has nothing to do with a compressed cache
    stamp = getattr(key, _STAMP, None)
    layer = stamp[0]() if stamp is not None else None
    if layer is not None and (layer.get_seq_length() != stamp[1]
                              or layer.layer_idx != getattr(module, "layer_idx", layer.layer_idx)):
        layer = None  # a stale tensor: the cache has moved on since it was stamped
    # what the codes-only kernel does not implement goes to the dense path: windows, score
    # capping, any scale other than 1/sqrt(head_dim)
    plain = (not kwargs.get("sliding_window") and not kwargs.get("softcap")
             and not getattr(module, "sliding_window", None)
             and not getattr(module, "is_sliding", False))
    fused = (layer is not None and not layer.dense and plain and query.shape[2] == 1
             and key.shape[2] == 1 and layer.get_seq_length() > 1)
    if fused:
        d = query.shape[-1]
        if scaling is not None and abs(scaling * d ** 0.5 - 1.0) > 1e-3:
            raise NotImplementedError("the decode kernel uses the 1/sqrt(head_dim) scale")
        fused = _mask_is_open(attention_mask)
    if fused:
        out = layer.ctx.decode(layer.layer_idx, query[:, :, 0, :])  # [B, Hq, D] float32
        return out.to(query.dtype)[:, None, :, :], None
    if layer is not None and key.shape[2] != layer.get_seq_length():
        # a multi-token query on top of stored history, a masked batch, a windowed or capped
        # layer: the dense history
        key, value = layer.full()
    return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout,
                                  scaling=scaling, is_causal=is_causal, **kwargs)


def enable_turboquant_cache(model, **cache_kwargs) -> TurboQuantCache:
    """Registers the attention function, switches ``model`` to it and returns a fresh
    :class:`TurboQuantCache` for ``model.generate(..., past_key_values=cache)``
    (the reference's helper of the same name: ``hf_cache.py``)."""
    from transformers import AttentionInterface

    AttentionInterface.register("turboquant", turboquant_attention_forward)
    model.config._attn_implementation = "turboquant"
    return TurboQuantCache(model.config, **cache_kwargs)

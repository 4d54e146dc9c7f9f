"""vLLM V1 KV-connector surface on the GPU-resident compressed cache.

Counterpart of the reference's ``connectors/vllm_v1.py``: ``TurboQuantBlockStore``
(``:214-686``) keeps one quantised record per (request, layer) in host numpy and
``TurboQuantKVConnector`` (``:714-815``) adapts it to vLLM's connector protocol, quantising
on the host inside ``save_kv_layer`` and leaving ``start_load_kv`` empty.  Here the store is
a slot table over one :class:`KVContext`: a request owns one sequence slot, a layer name maps
to a layer row, ``save`` runs the append / encode kernels on the device straight from the
engine's (paged) KV tensor and ``load`` / ``load_into_paged`` dequantise on the device into a
dense tensor or back into the engine's pages.  ``attend`` answers a decode-step query on the
codes of a stored prefix, which the reference's store cannot do.

Scope: the cache path only.  Durable manifests, sha256 integrity records and the async save
queue of the reference's store are host-side bookkeeping around the quantiser and are not
reproduced; blocks leave and enter a store through ``export_request`` / ``import_request``
as ``tqp-kv-npz/1`` byte strings (see :mod:`kv_blob`).
"""

from __future__ import annotations

import logging
import re
import threading
from typing import Any

from .context import KVContext

logger = logging.getLogger(__name__)

__all__ = ["DeviceBlockStore", "TurboQuantKVConnector", "KVConnectorRole", "register"]

_CONNECTOR_NAME = "TurboQuantConnectorB200"


class DeviceBlockStore:
    """Per-request compressed KV prefixes on one GPU.

    Args:
        n_layers, n_kv_heads, head_dim: model geometry (``head_dim`` 128).
        n_q_heads: query heads served by :meth:`attend` (default: ``n_kv_heads``).
        max_requests: sequence slots (requests held at once).
        max_tokens: capacity of a slot.
        key_bits, value_bits, hot_window, outlier_frac, seed: cache format, as in
            ``AutoConfig.build_cache``.
        dtype: element type of the tokens and of the uncompressed tail.
    """

    def __init__(self, n_layers: int, n_kv_heads: int, head_dim: int = 128, *,
                 n_q_heads: int | None = None, max_requests: int = 8, max_tokens: int = 8192,
                 key_bits: int = 4, value_bits: int = 4, hot_window: int = 512,
                 outlier_frac: float = 0.02, dtype="float16", device: int = 0,
                 seed: int | None = 0) -> None:
        self.ctx = KVContext(n_layers=n_layers, n_seqs=max_requests, n_kv_heads=n_kv_heads,
                             n_q_heads=n_q_heads or n_kv_heads, head_dim=head_dim,
                             key_bits=key_bits, value_bits=value_bits, hot_window=hot_window,
                             outlier_frac=outlier_frac, max_tokens_per_seq=max_tokens,
                             kv_dtype=dtype, seed=seed, device=device)
        self._lock = threading.Lock()
        self._slot: dict[str, int] = {}            # request id -> sequence slot
        self._free = list(range(max_requests - 1, -1, -1))
        self._layers: dict[str, int] = {}          # layer name -> layer row
        self._tokens: dict[str, int] = {}          # request id -> tokens restorable
        self.counters = {"saves": 0, "loads": 0, "hits": 0, "misses": 0, "evictions": 0,
                         "rejected": 0}

    # ------------------------------------------------------------------ bookkeeping --
    def layer_index(self, layer_name: str | int) -> int:
        """Row of a layer: the first integer in an engine-style name
        (``"model.layers.7.self_attn.attn"`` -> 7), else the order of first use."""
        if isinstance(layer_name, int):
            idx = layer_name
        else:
            with self._lock:
                if layer_name in self._layers:
                    return self._layers[layer_name]
                m = re.search(r"(\d+)", layer_name)
                idx = int(m.group(1)) if m else len(self._layers)
                self._layers[layer_name] = idx
        if not 0 <= idx < self.ctx.n_layers:
            raise ValueError(f"layer {layer_name!r} -> row {idx} outside the store's "
                             f"{self.ctx.n_layers} layers")
        return idx

    def _slot_of(self, request_id: str, create: bool) -> int | None:
        with self._lock:
            if request_id in self._slot:
                return self._slot[request_id]
            if not create:
                return None
            if not self._free:
                return None
            s = self._free.pop()
            self._slot[request_id] = s
            return s

    def matched_tokens(self, request_id: str) -> int:
        """Tokens this store can restore for ``request_id`` (0 if unknown)."""
        with self._lock:
            return self._tokens.get(request_id, 0)

    def stats(self) -> dict:
        with self._lock:
            return {"requests": len(self._slot), "free_slots": len(self._free),
                    "layers_seen": len(self._layers), "device_bytes": self.ctx.device_bytes(),
                    **self.counters}

    # ------------------------------------------------------------------------ save ----
    @staticmethod
    def _as_tokens(x):
        """``[T, H, D]`` view of ``[T, H, D]``, ``[H, D]``, ``[1, H, T, D]`` input."""
        if x.dim() == 4:
            if x.shape[0] != 1:
                raise ValueError("a 4-D tensor must be (1, H, T, D)")
            return x[0].permute(1, 0, 2)
        if x.dim() == 2:
            return x[None]
        if x.dim() != 3:
            raise ValueError(f"expected (T, H, D), (H, D) or (1, H, T, D), got {tuple(x.shape)}")
        return x

    def save(self, request_id: str, layer_name: str | int, keys, values) -> bool:
        """Encode one layer's KV prefix of ``request_id`` on the device, replacing what the
        store held for that (request, layer).  ``keys`` / ``values``: CUDA (or host) tensors
        ``(T, H, D)`` or ``(1, H, T, D)``.  Returns False (and counts a rejection) when no slot
        is free or the prefix does not fit: an unsaved prefix is a later miss, never an error."""
        import torch

        layer = self.layer_index(layer_name)
        k = self._as_tokens(keys if isinstance(keys, torch.Tensor) else torch.as_tensor(keys))
        v = self._as_tokens(values if isinstance(values, torch.Tensor) else torch.as_tensor(values))
        slot = self._slot_of(request_id, create=True)
        if slot is None or k.shape[0] > self.ctx.geom.max_tokens_per_seq:
            self.counters["rejected"] += 1
            return False
        self.ctx.clear(layer, slot)
        if k.shape[0]:
            self.ctx.append(layer, k[None], v[None], seq_begin=slot)
        with self._lock:
            self._tokens[request_id] = int(k.shape[0])
        self.counters["saves"] += 1
        return True

    def save_paged(self, request_id: str, layer_name: str | int, kv_layer, block_table,
                   n_tokens: int) -> bool:
        """:meth:`save` from an engine's paged layer tensor ``kv_layer``
        ``[2, n_blocks, block_size, H, D]`` (index 0 keys, 1 values): the request's tokens are
        the first ``n_tokens`` rows of the blocks listed in ``block_table``, gathered on the
        device."""
        import torch

        ids = torch.as_tensor(block_table, device=kv_layer.device, dtype=torch.long).reshape(-1)
        k = kv_layer[0].index_select(0, ids).flatten(0, 1)[:n_tokens]
        v = kv_layer[1].index_select(0, ids).flatten(0, 1)[:n_tokens]
        return self.save(request_id, layer_name, k, v)

    # ------------------------------------------------------------------------ load ----
    def load(self, request_id: str, layer_name: str | int):
        """Dense ``(keys, values)`` float32 CUDA tensors ``(H, T, D)`` of a stored prefix, or
        ``None`` when nothing is stored (a miss: the caller recomputes)."""
        layer = self.layer_index(layer_name)
        slot = self._slot_of(request_id, create=False)
        n = self.ctx.lengths(layer, slot)[0] if slot is not None else 0
        if n == 0:
            self.counters["misses"] += 1
            return None
        k, v = self.ctx.dequant(layer, slot, 0, n)
        self.counters["loads"] += 1
        self.counters["hits"] += 1
        return k, v

    def load_into_paged(self, request_id: str, layer_name: str | int, kv_layer, block_table) -> int:
        """Restores a stored prefix into the engine's pages: the dequantised tokens are written
        to the first rows of the blocks listed in ``block_table``.  Returns the tokens
        restored (0 on a miss)."""
        import torch

        got = self.load(request_id, layer_name)
        if got is None:
            return 0
        k, v = got
        n = k.shape[1]
        bs = kv_layer.shape[2]
        ids = torch.as_tensor(block_table, device=kv_layer.device, dtype=torch.long).reshape(-1)
        if ids.numel() * bs < n:
            raise ValueError("the block table is too short for the stored prefix")
        pos = torch.arange(n, device=kv_layer.device)
        blk, row = ids[pos // bs], pos % bs
        kv_layer[0][blk, row] = k.permute(1, 0, 2).to(kv_layer.dtype)
        kv_layer[1][blk, row] = v.permute(1, 0, 2).to(kv_layer.dtype)
        return n

    def attend(self, layer_name: str | int, queries: dict):
        """One decode step on the codes for several stored requests of one layer:
        ``queries`` maps request id -> ``(n_q_heads, D)`` query; returns request id ->
        ``(n_q_heads, D)`` float32 output.  Requests the store does not hold are left out."""
        import torch

        layer = self.layer_index(layer_name)
        g = self.ctx.geom
        q = torch.zeros((g.n_seqs, g.n_q_heads, g.head_dim), dtype=torch.float32,
                        device=self.ctx.device)
        held = {}
        for rid, qv in queries.items():
            slot = self._slot_of(rid, create=False)
            if slot is not None and self.ctx.lengths(layer, slot)[0] > 0:
                q[slot] = qv.to(device=self.ctx.device, dtype=torch.float32)
                held[rid] = slot
        if not held:
            return {}
        out = self.ctx.decode(layer, q)
        return {rid: out[slot] for rid, slot in held.items()}

    # ------------------------------------------------------------ eviction, hand-off ----
    def evict(self, request_id: str) -> int:
        """Drops every layer stored for ``request_id``; returns the layers that held tokens."""
        with self._lock:
            slot = self._slot.pop(request_id, None)
            self._tokens.pop(request_id, None)
        if slot is None:
            return 0
        gone = 0
        for layer in range(self.ctx.n_layers):
            if self.ctx.lengths(layer, slot)[0]:
                gone += 1
                self.ctx.clear(layer, slot)
        with self._lock:
            self._free.append(slot)
        self.counters["evictions"] += 1
        return gone

    def export_request(self, request_id: str) -> dict | None:
        """Everything stored for ``request_id``, layer by layer, as ``tqp-kv-npz/1`` byte
        strings plus the raw uncompressed tails (see ``KVContext.export_state``)."""
        slot = self._slot_of(request_id, create=False)
        if slot is None:
            return None
        return {"request_id": request_id,
                "layers": {layer: self.ctx.export_state(layer, slot)
                           for layer in range(self.ctx.n_layers)
                           if self.ctx.lengths(layer, slot)[0]}}

    def import_request(self, state: dict) -> bool:
        """Takes over a request exported by a store of the same geometry and seed."""
        rid = state["request_id"]
        slot = self._slot_of(rid, create=True)
        if slot is None:
            self.counters["rejected"] += 1
            return False
        n = 0
        for layer, st in state["layers"].items():
            self.ctx.import_state(int(layer), slot, st)
            n = max(n, int(st["n_tokens"]))
        with self._lock:
            self._tokens[rid] = n
        return True


# ------------------------------------------------------------------------- vLLM glue --
def _resolve_base():
    """The installed vLLM's connector base and role enum, or a local stand-in with the same
    protocol surface (``connectors/vllm_v1.py:688-711``)."""
    try:  # pragma: no cover - only with a vLLM whose connector API imports cleanly
        from vllm.distributed.kv_transfer.kv_connector.v1.base import (KVConnectorBase_V1,
                                                                         KVConnectorRole)

        return KVConnectorBase_V1, KVConnectorRole
    except Exception:  # noqa: BLE001

        class _Role:
            SCHEDULER = "scheduler"
            WORKER = "worker"

        class _Base:
            def __init__(self, vllm_config: Any = None, role: Any = None):
                self.vllm_config = vllm_config
                self.role = role

        return _Base, _Role


_Base, KVConnectorRole = _resolve_base()


class TurboQuantKVConnector(_Base):  # type: ignore[misc, valid-type]
    """The reference connector's protocol (``connectors/vllm_v1.py:714-815``) over a
    :class:`DeviceBlockStore`.  Pass ``store=`` or the store's keywords through
    ``kv_connector_extra_config`` (``n_layers``, ``n_kv_heads`` ... as in
    :class:`DeviceBlockStore`)."""

    def __init__(self, vllm_config: Any = None, role: Any = None, **kwargs: Any):
        # the base's constructor has changed its signature between vLLM releases (and wants a
        # real VllmConfig): try the known forms, else only keep the two attributes
        for base_args in ((vllm_config, role, kwargs.get("kv_cache_config")), (vllm_config, role)):
            try:
                super().__init__(*base_args)
                break
            except Exception:  # noqa: BLE001
                continue
        else:
            for name, val in (("vllm_config", vllm_config), ("role", role)):
                try:
                    setattr(self, name, val)
                except AttributeError:  # a read-only property of the base
                    setattr(self, "_" + name, val)
        extra = getattr(getattr(vllm_config, "kv_transfer_config", None),
                        "kv_connector_extra_config", None)
        cfg = dict(extra) if isinstance(extra, dict) else {}
        self.store = kwargs.get("store") or DeviceBlockStore(**cfg)
        self._to_load: dict = {}   # request id -> block table, set by build_connector_meta

    # ---- scheduler side ------------------------------------------------------------
    def get_num_new_matched_tokens(self, request: Any, num_computed_tokens: int, *args: Any,
                                   **kwargs: Any) -> tuple[int, bool]:
        rid = getattr(request, "request_id", None) or str(request)
        return max(0, self.store.matched_tokens(rid) - int(num_computed_tokens)), False

    def update_state_after_alloc(self, request: Any = None, blocks: Any = None, *args: Any,
                                 **kwargs: Any) -> None:
        rid = getattr(request, "request_id", None)
        if rid is not None and blocks is not None and self.store.matched_tokens(rid):
            self._to_load[rid] = blocks

    def build_connector_meta(self, scheduler_output: Any = None, **kwargs: Any):
        meta = {"version": 1, "load": dict(self._to_load)}
        self._to_load.clear()
        return meta

    def request_finished(self, request: Any = None, block_ids: Any = None,
                         **kwargs: Any) -> tuple[bool, dict | None]:
        return False, None  # the store owns its copy; the engine's blocks are not held

    # ---- worker side ---------------------------------------------------------------
    def start_load_kv(self, forward_context: Any = None, **kwargs: Any) -> int:
        """Restores the prefixes named by the connector metadata into the engine's pages, on
        the device.  ``forward_context`` carries ``kv_caches`` (layer name -> paged tensor) and
        ``connector_meta`` (as built above); both may also be given as keywords.  Returns the
        number of (request, layer) prefixes restored."""
        caches = kwargs.get("kv_caches") or getattr(forward_context, "kv_caches", None) or {}
        meta = kwargs.get("connector_meta") or getattr(forward_context, "connector_meta", None) or {}
        done = 0
        for rid, table in (meta.get("load") or {}).items():
            for name, kv_layer in caches.items():
                done += 1 if self.store.load_into_paged(rid, name, kv_layer, table) else 0
        return done

    def wait_for_layer_load(self, layer_name: str, **kwargs: Any) -> None:
        return None  # loads are ordered with the caller's stream

    def save_kv_layer(self, layer_name: str, kv_layer: Any, attn_metadata: Any = None,
                      **kwargs: Any) -> None:
        """Encodes one layer's KV of a request on the device.  With a block table in
        ``attn_metadata`` (``block_table`` and ``num_tokens``, or the same as keywords)
        ``kv_layer`` is the engine's paged tensor; without one, index 0 / 1 of ``kv_layer``
        are the request's keys / values, as in the reference's connector."""
        rid = str(getattr(attn_metadata, "request_id", kwargs.get("request_id", "_")))
        table = kwargs.get("block_table", getattr(attn_metadata, "block_table", None))
        if table is not None:
            n = int(kwargs.get("num_tokens", getattr(attn_metadata, "num_tokens", 0)))
            self.store.save_paged(rid, layer_name, kv_layer, table, n)
        else:
            self.store.save(rid, layer_name, kv_layer[0], kv_layer[1])

    def wait_for_save(self, **kwargs: Any) -> None:
        import torch

        torch.cuda.current_stream(self.store.ctx.device).synchronize()

    def get_metrics(self) -> dict:
        return self.store.stats()

    def get_finished(self, finished_req_ids: Any = None, **kwargs: Any):
        for rid in finished_req_ids or ():
            self.store.evict(str(rid))
        return None, None


def register(name: str = _CONNECTOR_NAME) -> bool:
    """Registers the connector with vLLM's ``KVConnectorFactory`` when vLLM is importable
    (``connectors/vllm_v1.py:817-840``); returns whether it did."""
    try:
        from vllm.distributed.kv_transfer.kv_connector.factory import KVConnectorFactory
    except Exception:  # noqa: BLE001
        logger.info("vLLM not importable; %s not registered", name)
        return False
    try:
        KVConnectorFactory.register_connector(name, __name__, "TurboQuantKVConnector")
        return True
    except Exception:  # noqa: BLE001 - already registered, or an API drift
        logger.info("registration of %s skipped", name, exc_info=True)
        return False

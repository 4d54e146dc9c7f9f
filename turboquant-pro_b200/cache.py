"""TurboQuantKVCache — the reference's cache API on the B200-native kernels.

Same constructor keywords, methods, properties, return shapes and exceptions as
``turboquant_pro.core.TurboQuantKVCache`` (``core.py:818-1307``), so user code can switch
imports.  Storage and arithmetic live on the GPU behind the C ABI; there is no numpy or
CuPy path underneath and therefore no CPU fallback: constructing a cache without a CUDA
device raises.

Supported formats: per-channel 4-bit keys in the three grids the reference has an affine
(fused) form for — asymmetric NF4 (``key_nf4_asym=True``, ``key_zero_point="calibrated"``),
symmetric NF4 (``key_nf4=True``) and uniform (neither flag) — with an optional fp16 outlier
side-list, PolarQuant values at 3 or 4 bits; asymmetric NF4 also with the ``sparse`` and
``bias`` zero-points; and the legacy key format ``per_channel_keys=False`` (keys through the
value quantiser, ``core.py:1022-1033``) where ``key_bits == value_bits``.  Data-fit tables
(``key_nuq``) and other key widths raise ``NotImplementedError``.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from types import SimpleNamespace

import numpy as np

from .context import KVContext

logger = logging.getLogger(__name__)


@dataclass
class CompressedPerChannelKV:
    """A cold key block in the reference's container layout (``per_channel_kv.py:103-143``):
    the same field names, so code that walks ``cache._cold_keys`` keeps working.  The arrays
    are host copies made when the block is first asked for."""

    indices: np.ndarray            # uint8, bit-reversed nibbles of _pack_indices
    scale: np.ndarray | None       # uniform grid: (B, H, 1, D) step
    zero: np.ndarray | None        # uniform grid: (B, H, 1, D) minimum
    bits: int
    shape: tuple
    packed: bool = True
    levels: np.ndarray | None = None
    nf4_scale: np.ndarray | None = None   # NF4 family: (B, H, D)
    nf4_mean: np.ndarray | None = None    # asymmetric NF4: (B, H, D), or the kept channels only
    original_dtype: np.dtype = field(default_factory=lambda: np.dtype("float32"))
    outlier_idx: np.ndarray | None = None
    outlier_val: np.ndarray | None = None
    zp_mode: str = "calibrated"
    rope_theta: float | None = None
    position_start: int = 0

    def nbytes(self) -> int:
        return sum(a.nbytes for a in (self.indices, self.scale, self.zero, self.levels,
                                      self.nf4_scale, self.nf4_mean, self.outlier_idx,
                                      self.outlier_val) if a is not None)

    def compression_ratio(self, head_dim: int) -> float:
        return int(np.prod(self.shape)) * self.original_dtype.itemsize / max(self.nbytes(), 1)


@dataclass
class CompressedKV:
    """A cold value block in the reference's container layout (``core.py:96-136``)."""

    indices: np.ndarray
    norms: np.ndarray
    bits: int
    original_dtype: np.dtype = field(default_factory=lambda: np.dtype("float32"))
    packed: bool = True
    n_values: int = 0
    shape: tuple = ()

    def nbytes(self) -> int:
        return self.indices.nbytes + self.norms.nbytes

    def original_nbytes(self, head_dim: int) -> int:
        return int(np.prod(self.norms.shape)) * head_dim * self.original_dtype.itemsize

    def compression_ratio(self, head_dim: int) -> float:
        return self.original_nbytes(head_dim) / max(self.nbytes(), 1)


class _ColdView:
    """``cache._cold_keys`` / ``_cold_values`` / ``_cold_lengths``: a read-only sequence over
    the cold blocks, materialised block by block from the device on first access (cold
    blocks never change until the cache is cleared)."""

    def __init__(self, cache, what):
        self._cache, self._what = cache, what

    def __len__(self):
        return self._cache.cold_length // self._cache._ctx.block_tokens

    def __getitem__(self, i):
        if isinstance(i, slice):
            return [self[j] for j in range(*i.indices(len(self)))]
        n = len(self)
        if i < 0:
            i += n
        if not 0 <= i < n:
            raise IndexError("cold block index out of range")
        if self._what == "lengths":
            return self._cache._ctx.block_tokens
        return self._cache._cold_block(i)[0 if self._what == "keys" else 1]

    def __iter__(self):
        return (self[i] for i in range(len(self)))

    def __bool__(self):
        return len(self) > 0

    def __eq__(self, other):
        return list(self) == other


class TurboQuantKVCache:
    """Two-tier (hot window + compressed cold blocks) KV cache of one layer and one sequence.

    Keyword arguments follow ``core.py:886-904``.  Two additions, both keyword-only in
    spirit: ``max_tokens`` (capacity the device buffers are sized for) and ``dtype``
    (element type of the hot window; appended tokens are converted to it — float32 keeps
    every input exactly, as the reference does).
    """

    @classmethod
    def robust(cls, head_dim: int = 128, n_heads: int = 32, *, key_bits: int = 4,
               value_bits: int = 4, hot_window: int = 512, outlier_frac: float = 0.02,
               **kwargs) -> "TurboQuantKVCache":
        """Asymmetric-NF4 keys + ``outlier_frac`` fp16 outliers (``core.py:856-884``)."""
        return cls(head_dim=head_dim, n_heads=n_heads, key_bits=key_bits, value_bits=value_bits,
                   hot_window=hot_window, key_nf4_asym=True, key_outlier_frac=outlier_frac,
                   **kwargs)

    def __init__(self, head_dim: int = 128, n_heads: int = 32, bits: int = 3,
                 key_bits: int | None = None, value_bits: int | None = None,
                 hot_window: int = 512, use_gpu: bool = True, device_id: int = 0,
                 seed: int | None = None, per_channel_keys: bool = True, key_nuq: bool = False,
                 key_nf4: bool = False, key_nf4_asym: bool = False,
                 key_outlier_frac: float = 0.0, key_zero_point: str = "calibrated",
                 key_rope_theta: float | None = None, key_k_bias=None, *,
                 max_tokens: int = 32768, dtype="float32", n_q_heads: int | None = None) -> None:
        for name, b in (("bits", bits), ("key_bits", key_bits), ("value_bits", value_bits)):
            if b is not None and b not in (2, 3, 4):
                raise ValueError(f"Unsupported {name}={b}; choose from [2, 3, 4]")
        if not (0.0 <= key_outlier_frac < 1.0):
            raise ValueError("outlier_frac must be in [0, 1)")
        if key_zero_point not in ("calibrated", "sparse", "bias"):
            raise ValueError("zero_point must be one of ('calibrated', 'sparse', 'bias')")
        if not use_gpu:
            raise RuntimeError("this build is GPU-only: use_gpu=False has no implementation "
                               "(use the reference package for a numpy cache)")
        self.head_dim = head_dim
        self.n_heads = n_heads
        self.bits = bits
        self.key_bits = key_bits if key_bits is not None else bits
        self.value_bits = value_bits if value_bits is not None else bits
        self.hot_window = hot_window
        self.per_channel_keys = per_channel_keys
        if not per_channel_keys:
            # the legacy key format (core.py:1022-1033): keys through the value quantiser
            if self.key_bits != self.value_bits:
                raise NotImplementedError("PolarQuant keys need key_bits == value_bits on the "
                                          "CUDA path (the reference's fused_decode does too)")
            if self.value_bits not in (3, 4):
                raise NotImplementedError("the CUDA path implements 3- and 4-bit PolarQuant")
            self.key_mode = "polar"
            self.key_zero_point = key_zero_point
            self.key_outlier_frac = 0.0
            self.key_rope_theta = key_rope_theta
            self._ctx = KVContext(
                n_layers=1, n_seqs=1, n_kv_heads=n_heads, n_q_heads=n_q_heads or n_heads,
                head_dim=head_dim, key_bits=self.key_bits, value_bits=self.value_bits,
                hot_window=hot_window, outlier_frac=0.0, max_tokens_per_seq=max_tokens,
                kv_dtype=dtype, seed=seed, device=device_id, key_mode="polar")
            self._blocks = {}
            cent, bnd = self._ctx.centroids, self._ctx.boundaries
            self._tq = SimpleNamespace(head_dim=head_dim, n_heads=n_heads, bits=self.value_bits,
                                       key_bits=self.key_bits, value_bits=self.value_bits,
                                       _Pi=self._ctx.pi, _Pi_T=self._ctx.pi_t,
                                       _codebooks={self.value_bits: (cent, bnd)}, use_gpu=True)
            self._kq = None  # (core.py:947: no per-channel quantiser in this mode)
            return
        if key_nuq:
            raise NotImplementedError("data-fit key tables (key_nuq=True) have no fused form; "
                                      "they are not implemented on the CUDA path")
        if key_zero_point != "calibrated":
            if not key_nf4_asym:
                raise ValueError(f"zero_point={key_zero_point!r} requires nf4_asym=True")
            if key_rope_theta is None:
                raise ValueError(f"zero_point={key_zero_point!r} requires rope_theta")
            if key_zero_point == "bias" and key_k_bias is None:
                raise ValueError('zero_point="bias" requires k_bias')
        if (key_nf4 or key_nf4_asym) and self.key_bits != 4:
            raise ValueError("nf4=True requires bits=4")
        if self.key_bits != 4:
            raise NotImplementedError("the CUDA path implements 4-bit per-channel keys")
        self.key_mode = "nf4_asym" if key_nf4_asym else ("nf4" if key_nf4 else "uniform")
        self._ctx = KVContext(
            n_layers=1, n_seqs=1, n_kv_heads=n_heads, n_q_heads=n_q_heads or n_heads,
            head_dim=head_dim, key_bits=self.key_bits, value_bits=self.value_bits,
            hot_window=hot_window, outlier_frac=key_outlier_frac, max_tokens_per_seq=max_tokens,
            kv_dtype=dtype, seed=seed, device=device_id, key_mode=self.key_mode)
        self.key_zero_point = key_zero_point
        if key_zero_point == "sparse":
            # means only on the channels that stay put over a block (per_channel_kv.py:337-342)
            from .autoconfig import rope_long_wavelength_mask

            self._ctx.set_key_mean_mask(rope_long_wavelength_mask(
                key_rope_theta, head_dim, self._ctx.block_tokens))
        elif key_zero_point == "bias":
            # zero-point of block b = the k-projection bias under RoPE, averaged over the
            # block's positions (per_channel_kv.py:327-336): known in advance for every block
            from .autoconfig import rope_averaged_bias

            f, nb = self._ctx.block_tokens, self._ctx.geom.max_blocks
            kb = np.asarray(key_k_bias, dtype=np.float32).reshape(n_heads, head_dim)
            self._ctx.set_key_bias_means(np.stack(
                [rope_averaged_bias(kb, key_rope_theta, head_dim, b * f, f) for b in range(nb)]))
        self.key_outlier_frac = key_outlier_frac
        self.key_rope_theta = key_rope_theta
        self._blocks: dict = {}
        # the two quantisers the reference cache is built from, as far as callers read them:
        # the value rotation and codebook, the key format
        cent, bnd = self._ctx.centroids, self._ctx.boundaries
        self._tq = SimpleNamespace(head_dim=head_dim, n_heads=n_heads, bits=self.value_bits,
                                   key_bits=self.key_bits, value_bits=self.value_bits,
                                   _Pi=self._ctx.pi, _Pi_T=self._ctx.pi_t,
                                   _codebooks={self.value_bits: (cent, bnd)}, use_gpu=True)
        self._kq = SimpleNamespace(head_dim=head_dim, n_heads=n_heads, bits=self.key_bits,
                                   nf4=key_nf4, nf4_asym=key_nf4_asym, nuq=False,
                                   outlier_frac=key_outlier_frac, zero_point=key_zero_point,
                                   rope_theta=key_rope_theta)

    # ------------------------------------------------------- the reference's block lists --
    def _cold_block(self, i: int):
        """(key container, value container) of cold block ``i`` (host copies, cached)."""
        if i not in self._blocks:
            g = self._ctx.geom
            b = self._ctx.export_block(0, 0, i)
            shape = (1, g.n_kv_heads, g.block_tokens, g.head_dim)
            dt = np.dtype({0: "float32", 1: "float16", 2: "float32"}[g.kv_dtype])
            kw = dict(indices=b["key_indices"], bits=self.key_bits, shape=shape, packed=True,
                      original_dtype=dt, outlier_idx=b["outlier_idx"],
                      outlier_val=b["outlier_val"], position_start=i * g.block_tokens)
            if self.key_mode == "polar":
                ck = CompressedKV(indices=b["key_indices"], norms=b["key_norms"],
                                  bits=self.key_bits, original_dtype=dt, packed=True,
                                  n_values=int(np.prod(shape)), shape=shape)
            elif self.key_mode == "uniform":
                ck = CompressedPerChannelKV(scale=b["nf4_scale"][:, :, None, :],
                                            zero=b["nf4_mean"][:, :, None, :], **kw)
            else:
                mean = b["nf4_mean"] if self.key_mode == "nf4_asym" else None
                if self.key_zero_point == "sparse":
                    mean = mean[:, :, self._ctx.key_mean_mask]
                elif self.key_zero_point == "bias":
                    mean = None
                ck = CompressedPerChannelKV(scale=None, zero=None, nf4_scale=b["nf4_scale"],
                                            nf4_mean=mean, zp_mode=self.key_zero_point,
                                            rope_theta=self.key_rope_theta, **kw)
            cv = CompressedKV(indices=b["value_indices"], norms=b["value_norms"],
                              bits=self.value_bits, original_dtype=dt, packed=True,
                              n_values=int(np.prod(shape)), shape=shape)
            self._blocks[i] = (ck, cv)
        return self._blocks[i]

    @property
    def _cold_keys(self):
        """The cold key blocks as ``CompressedPerChannelKV`` containers (``core.py:1011-1038``
        keeps them in a list of this name)."""
        return _ColdView(self, "keys")

    @property
    def _cold_values(self):
        return _ColdView(self, "values")

    @property
    def _cold_lengths(self):
        return _ColdView(self, "lengths")

    # ------------------------------------------------------------------ properties --
    @property
    def length(self) -> int:
        """Total number of tokens (cold + hot)."""
        return self._ctx.lengths(0, 0)[0]

    @property
    def cold_length(self) -> int:
        return self._ctx.lengths(0, 0)[1]

    @property
    def hot_length(self) -> int:
        return self._ctx.lengths(0, 0)[2]

    @property
    def context(self) -> KVContext:
        """The underlying device context."""
        return self._ctx

    # --------------------------------------------------------------------- append ----
    def _to_device(self, x, what):
        import torch

        if isinstance(x, torch.Tensor):
            t = x
        else:
            t = torch.from_numpy(np.ascontiguousarray(x))
        if t.dim() == 4:  # (1, H, T, D) -> (T, H, D)
            if t.shape[0] != 1:
                raise ValueError(f"{what}: batch dimension must be 1")
            t = t[0].permute(1, 0, 2)
        elif t.dim() == 2:  # (H, D)
            t = t[None]
        elif t.dim() != 3:
            raise ValueError(f"{what}: expected (1,H,1,D), (H,D) or (T,H,D), got {tuple(x.shape)}")
        if t.shape[1] != self.n_heads or t.shape[2] != self.head_dim:
            raise ValueError(f"{what}: expected {self.n_heads} heads of dim {self.head_dim}")
        return t.to(device=self._ctx.device, dtype=self._ctx.kv_dtype)[None].contiguous()

    def append(self, key, value) -> None:
        """Add the K/V of one token: ``(1, n_heads, 1, head_dim)`` or ``(n_heads,
        head_dim)`` (numpy or torch).  Flushes the oldest half of an over-full hot window
        into one compressed block, as ``core.py:986-1038`` does."""
        self._ctx.append(0, self._to_device(key, "key"), self._to_device(value, "value"))

    def append_many(self, keys, values) -> None:
        """Bulk form of :meth:`append`: ``(T, n_heads, head_dim)`` or ``(1, n_heads, T,
        head_dim)``.  Produces exactly the blocks T single appends would."""
        self._ctx.append(0, self._to_device(keys, "keys"), self._to_device(values, "values"))

    # -------------------------------------------------------------------- getters ----
    def _range(self, start, end, keys):
        n = self.length
        start, end = max(0, start), min(end, n)
        if end <= start:
            return np.zeros((1, self.n_heads, 0, self.head_dim), dtype=np.float32)
        k, v = self._ctx.dequant(0, 0, start, end, keys=keys, values=not keys)
        return (k if keys else v).cpu().numpy()[None]

    def get_keys(self, start: int, end: int) -> np.ndarray:
        """Dequantised keys of ``[start, end)``: ``(1, n_heads, n, head_dim)`` float32."""
        return self._range(start, end, True)

    def get_values(self, start: int, end: int) -> np.ndarray:
        return self._range(start, end, False)

    # --------------------------------------------------------------------- decode ----
    def fused_decode(self, query, method: str = "warp"):
        """One decode-step attention output over the whole cache, computed on the codes.

        ``query``: ``(n_q_heads, head_dim)`` or ``(1, n_q_heads, 1, head_dim)``; returns
        ``(n_q_heads, head_dim)`` float32 — a numpy array for numpy input, a CUDA tensor
        for tensor input.  Unlike the reference (``core.py:1193``) it does not require
        ``key_bits == value_bits``.
        """
        import torch

        if self.length == 0:
            raise RuntimeError("cache is empty")
        is_np = not isinstance(query, torch.Tensor)
        q = torch.from_numpy(np.ascontiguousarray(query, dtype=np.float32)) if is_np else query
        hq = self._ctx.n_q_heads
        q = q.reshape(1, hq, self.head_dim).to(self._ctx.device)
        if q.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            q = q.float()
        out = self._ctx.decode(0, q)[0]
        return out.cpu().numpy() if is_np else out

    # ---------------------------------------------------------------------- stats ----
    def memory_stats(self) -> dict[str, float]:
        """``cold_bytes``, ``hot_bytes``, ``total_bytes``, ``uncompressed_equivalent_bytes``
        (float32 K+V, as the reference counts it) and ``effective_ratio``
        (``core.py:1267-1296``)."""
        cold, hot = self._ctx.memory_stats(0, 0)
        total = cold + hot
        unc = float(self.length * self.n_heads * self.head_dim * 4 * 2)
        return {
            "cold_bytes": float(cold),
            "hot_bytes": float(hot),
            "total_bytes": float(total),
            "uncompressed_equivalent_bytes": unc,
            "effective_ratio": unc / max(total, 1),
        }

    def clear(self) -> None:
        """Reset the cache to empty."""
        self._ctx.clear(0, 0)
        self._blocks.clear()

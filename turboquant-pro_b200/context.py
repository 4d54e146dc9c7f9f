"""KVContext — a GPU-resident group of compressed two-tier KV caches.

One context holds ``n_layers x n_seqs`` caches that share geometry, rotation and
codebooks; each of them behaves exactly like one reference ``TurboQuantKVCache``
(``turboquant_pro/core.py:818-1307``).  Batch, layers and GQA do not exist in the
reference's cache API — they are what a serving engine adds around it — so this class is
the extension point the benchmark configurations use, and the single-cache façade in
:mod:`cache` is a thin view of a 1 x 1 context.

PyTorch is used for device memory and streams only; all computation happens in the
hand-written kernels behind the C ABI (``include/tqb200.h``).
"""

from __future__ import annotations

import ctypes as C
import math

import numpy as np

from . import _lib
from ._lib import REGIONS, TqBuffers, TqGeom, TqSizes, check

# Lloyd-Max centroids of N(0, 1) for 3 and 4 bits — the direction codebook of the value
# quantiser (turboquant_pro/core.py:70-93).
_LLOYD_MAX = {
    3: (-1.748, -1.050, -0.500, -0.069, 0.069, 0.500, 1.050, 1.748),
    4: (-2.401, -1.844, -1.437, -1.099, -0.800, -0.524, -0.262, -0.066,
        0.066, 0.262, 0.524, 0.800, 1.099, 1.437, 1.844, 2.401),
}


def value_codebook(head_dim: int, bits: int):
    """Centroids (scaled by 1/sqrt(d), rounded to float32) and the float32 mid-point
    boundaries, as ``TurboQuantKV.__init__`` builds them (core.py:229-241)."""
    if bits not in _LLOYD_MAX:
        raise NotImplementedError(f"value_bits={bits}: the CUDA path implements 3 and 4")
    c = (np.asarray(_LLOYD_MAX[bits], dtype=np.float64) * (1.0 / math.sqrt(head_dim))).astype(
        np.float32)
    bnd = ((c[:-1] + c[1:]) / np.float32(2.0)).astype(np.float32)
    return c, bnd


def rotation_matrix(head_dim: int, seed):
    """Seeded random orthogonal matrix and its transpose (core.py:246-260): QR of a
    float32 standard-normal matrix drawn from ``np.random.default_rng(seed)``."""
    rng = np.random.default_rng(seed)
    g = rng.standard_normal((head_dim, head_dim)).astype(np.float32)
    q, _ = np.linalg.qr(g)
    return np.ascontiguousarray(q), np.ascontiguousarray(q.T)


def _torch():
    import torch

    return torch


def _dtype_code(torch_dtype) -> int:
    torch = _torch()
    return {torch.float32: _lib.TQ_F32, torch.float16: _lib.TQ_F16,
            torch.bfloat16: _lib.TQ_BF16}[torch_dtype]


def _torch_dtype(name):
    torch = _torch()
    if isinstance(name, torch.dtype):
        return name
    key = np.dtype(name).name if not isinstance(name, str) else name
    return {"float32": torch.float32, "float16": torch.float16,
            "bfloat16": torch.bfloat16}[key]


KEY_MODES = ("nf4_asym", "nf4", "uniform", "polar")  # TQ_KEYS_* of the C ABI, in order


class KVContext:
    """``n_layers x n_seqs`` compressed KV caches on one GPU.

    Args:
        n_layers, n_seqs, n_kv_heads, n_q_heads: cache-group geometry; query head ``i``
            attends KV head ``i // (n_q_heads // n_kv_heads)``.
        head_dim: 128.
        key_bits: 4.  value_bits: 3 or 4 (PolarQuant values).
        key_mode: per-channel key grid, ``"nf4_asym"`` (default), ``"nf4"`` (symmetric) or
            ``"uniform"`` (``per_channel_kv.py:285-401``); or ``"polar"``, the legacy format in
            which keys go through the value quantiser (``core.py:1022-1033``;
            ``key_bits == value_bits``, no outliers; served by the general decode kernel).
        key_mean_mask: ``(head_dim,)`` booleans, asymmetric NF4 only: the channels that keep
            their mean as zero-point (the reference's ``zero_point="sparse"``); default all.
        hot_window: tokens kept uncompressed (2..512); a flush moves the oldest
            ``(hot_window + 1) // 2`` tokens into one cold block.
        outlier_frac: per-channel fraction of fp16 outliers kept beside the key codes.
        max_tokens_per_seq: capacity each sequence is sized for.
        kv_dtype: element type of appended tokens and of the hot window.
        seed: seed of the rotation matrix; ``pi`` overrides it with an explicit matrix.
        device: CUDA device ordinal.
    """

    def __init__(self, n_layers=1, n_seqs=1, n_kv_heads=8, n_q_heads=None, head_dim=128,
                 key_bits=4, value_bits=3, hot_window=512, outlier_frac=0.02,
                 max_tokens_per_seq=8192, kv_dtype="float32", seed=None, pi=None, device=0,
                 key_mode="nf4_asym", key_mean_mask=None):
        torch = _torch()
        if not torch.cuda.is_available():
            raise RuntimeError("KVContext needs a CUDA device: this package has no CPU fallback")
        self._lib = _lib.load()
        self.device = torch.device("cuda", device)
        self.kv_dtype = _torch_dtype(kv_dtype)
        g = TqGeom()
        g.n_layers, g.n_seqs, g.n_kv_heads = n_layers, n_seqs, n_kv_heads
        g.n_q_heads = n_q_heads if n_q_heads is not None else n_kv_heads
        g.head_dim, g.key_bits, g.value_bits = head_dim, key_bits, value_bits
        if key_mode not in KEY_MODES:
            raise ValueError(f"key_mode must be one of {KEY_MODES}, got {key_mode!r}")
        self.key_mode = key_mode
        g.key_mode = KEY_MODES.index(key_mode)
        g.hot_window = hot_window
        g.kv_dtype = _dtype_code(self.kv_dtype)
        g.max_tokens_per_seq = max_tokens_per_seq
        g.outlier_frac = float(outlier_frac)
        check(self._lib.tq_geom_finish(C.byref(g)))
        self.geom = g
        sizes = TqSizes()
        check(self._lib.tq_ctx_sizes(C.byref(g), C.byref(sizes)))
        self.sizes = {n: int(getattr(sizes, n)) for n in REGIONS}
        # device memory comes from torch's allocator; the library allocates nothing
        self._regions = {n: torch.zeros(self.sizes[n], dtype=torch.uint8, device=self.device)
                         for n in REGIONS}
        bufs = TqBuffers()
        for n in REGIONS:
            setattr(bufs, n, self._regions[n].data_ptr())
        if pi is None:
            pi, pi_t = rotation_matrix(head_dim, seed)
        else:
            pi = np.ascontiguousarray(pi, dtype=np.float32)
            pi_t = np.ascontiguousarray(pi.T)
        self.pi, self.pi_t = pi, pi_t
        self.centroids, self.boundaries = value_codebook(head_dim, value_bits)
        handle = C.c_void_p()
        with torch.cuda.device(self.device):
            check(self._lib.tq_ctx_create(
                C.byref(g), C.byref(bufs), device, pi.ctypes.data, pi_t.ctypes.data,
                self.centroids.ctypes.data, self.boundaries.ctypes.data,
                self._stream(), C.byref(handle)))
        self._h = handle
        self.key_mean_mask = None
        if key_mean_mask is not None:
            self.set_key_mean_mask(key_mean_mask)

    # -- plumbing --------------------------------------------------------------------
    def _stream(self):
        return C.c_void_p(_torch().cuda.current_stream(self.device).cuda_stream)

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self._lib.tq_ctx_destroy(h)
            self._h = None

    @property
    def n_layers(self):
        return self.geom.n_layers

    @property
    def n_seqs(self):
        return self.geom.n_seqs

    @property
    def n_kv_heads(self):
        return self.geom.n_kv_heads

    @property
    def n_q_heads(self):
        return self.geom.n_q_heads

    @property
    def block_tokens(self):
        return self.geom.block_tokens

    def device_bytes(self) -> int:
        """Bytes of device memory held by this context."""
        return sum(self.sizes.values())

    # -- append ----------------------------------------------------------------------
    def append(self, layer: int, k, v, seq_begin: int = 0) -> None:
        """Append tokens to ``k.shape[0]`` consecutive sequences of ``layer``.

        ``k``/``v``: CUDA tensors ``[n_seqs', T, n_kv_heads, D]`` (any strides with a
        contiguous last dimension) of ``kv_dtype``.  Performs every flush the reference
        would perform for token-by-token appends, with the same block boundaries.
        """
        torch = _torch()
        if k.dim() != 4 or k.shape != v.shape:
            raise ValueError(f"expected k, v of shape [n_seqs, T, H, D], got {tuple(k.shape)} "
                             f"and {tuple(v.shape)}")
        if k.shape[2] != self.n_kv_heads or k.shape[3] != self.geom.head_dim:
            raise ValueError("head count / head_dim do not match the context")
        if k.dtype != self.kv_dtype or v.dtype != self.kv_dtype:
            k = k.to(self.kv_dtype)
            v = v.to(self.kv_dtype)
        if k.device != self.device:
            k = k.to(self.device)
            v = v.to(self.device)
        if k.stride(3) != 1:
            k = k.contiguous()
        if v.stride() != k.stride():
            v = v.contiguous()
            k = k.contiguous()
        with torch.cuda.device(self.device):
            check(self._lib.tq_append(self._h, layer, seq_begin, k.shape[0], k.data_ptr(),
                                      v.data_ptr(), k.shape[1], k.stride(0), k.stride(1),
                                      k.stride(2), self._stream()))

    # -- decode ----------------------------------------------------------------------
    def _check_q(self, q):
        g = self.geom
        if tuple(q.shape) != (g.n_seqs, g.n_q_heads, g.head_dim):
            raise ValueError(f"expected q of shape {(g.n_seqs, g.n_q_heads, g.head_dim)}, "
                             f"got {tuple(q.shape)}")
        if q.device != self.device:
            raise ValueError(f"q lives on {q.device}, the context on {self.device}")
        return q.contiguous()

    def _check_result(self, t, shape, name):
        torch = _torch()
        if t is None:
            return torch.empty(shape, dtype=torch.float32, device=self.device)
        if tuple(t.shape) != tuple(shape) or t.dtype != torch.float32 or t.device != self.device \
                or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous float32 tensor of shape {tuple(shape)} "
                             f"on {self.device}")
        return t

    def decode(self, layer: int, q, out=None, check_status: bool = False):
        """One decode step of attention on the codes for every sequence of ``layer``.

        ``q``: CUDA tensor ``[n_seqs, n_q_heads, D]`` (float32 / float16 / bfloat16).
        Returns float32 ``[n_seqs, n_q_heads, D]``.  With ``check_status`` the call
        synchronises and raises :class:`TqError` if the kernel reported a wait that ran out
        (status bit 1: the output is then undefined).
        """
        torch = _torch()
        g = self.geom
        q = self._check_q(q)
        out = self._check_result(out, (g.n_seqs, g.n_q_heads, g.head_dim), "out")
        with torch.cuda.device(self.device):
            check(self._lib.tq_decode(self._h, layer, q.data_ptr(), _dtype_code(q.dtype),
                                      out.data_ptr(), self._stream()))
        if check_status:
            self.raise_on_timeout()
        return out

    def raise_on_timeout(self) -> int:
        """Reads the status word (synchronises); raises if a bounded wait of a decode kernel ran
        out since the last read, else returns the other flags."""
        flags = self.status()
        if flags & 2:
            raise _lib.TqError(-3, "a bounded wait inside the decode kernel ran out; the "
                                   "output of that call is undefined")
        return flags

    def decode_static_scratch(self, layer: int, q, out=None):
        """:meth:`decode` for callers that may not allocate or lend working memory: the
        split-K partials live in a fixed array inside the library (at most 1024
        (sequence, query head) pairs; calls must not overlap on the device).  ``out`` should
        be passed by such callers; it is created here only as a convenience."""
        torch = _torch()
        g = self.geom
        q = self._check_q(q)
        out = self._check_result(out, (g.n_seqs, g.n_q_heads, g.head_dim), "out")
        with torch.cuda.device(self.device):
            check(self._lib.tq_decode_static_scratch(self._h, layer, q.data_ptr(),
                                                     _dtype_code(q.dtype), out.data_ptr(),
                                                     self._stream()))
        return out

    def decode_partial(self, layer: int, q, block_begin: int, block_end: int, with_hot: bool,
                       mlo=None):
        """Un-normalised ``(m, l, o)`` states over cold blocks ``[block_begin, block_end)``
        (+ the hot window): float32 ``[n_seqs, n_q_heads, 2 + D]``."""
        torch = _torch()
        g = self.geom
        q = self._check_q(q)
        mlo = self._check_result(mlo, (g.n_seqs, g.n_q_heads, 2 + g.head_dim), "mlo")
        with torch.cuda.device(self.device):
            check(self._lib.tq_decode_partial(self._h, layer, q.data_ptr(), _dtype_code(q.dtype),
                                              block_begin, block_end, int(bool(with_hot)),
                                              mlo.data_ptr(), self._stream()))
        return mlo

    def decode_exchange(self, layer: int, q, block_begin: int, block_end: int, with_hot: bool,
                        exchange, out=None, phases: int = 3):
        """``decode_partial`` over this rank's blocks and the exchange + merge of the states
        with the other ranks (``exchange``: a :class:`~turboquant_pro_b200.parallel.PeerExchange`
        or its raw handle) in one call: the kernel that merges the rank's own partials hands its
        rows to the other ranks and merges theirs.  Returns the final ``[n_seqs, n_q_heads, D]``
        output.  Raises ``NotImplementedError`` where the layer has no such fused form; the
        two-call form (``decode_partial`` then ``PeerExchange.gather_merge``) works everywhere
        and gives the same bits."""
        torch = _torch()
        g = self.geom
        q = self._check_q(q)
        out = self._check_result(out, (g.n_seqs, g.n_q_heads, g.head_dim), "out")
        h = getattr(exchange, "_h", exchange)
        with torch.cuda.device(self.device):
            check(self._lib.tq_decode_exchange(self._h, layer, q.data_ptr(), _dtype_code(q.dtype),
                                               block_begin, block_end, int(bool(with_hot)), h,
                                               out.data_ptr(), phases, self._stream()))
        return out

    def lse_combine(self, mlo, out=None):
        """Merge gathered states ``[n_parts, n_rows, 2 + D]`` into ``[n_rows, D]``."""
        torch = _torch()
        if mlo.dim() != 3 or mlo.shape[2] != 2 + self.geom.head_dim or mlo.dtype != torch.float32 \
                or mlo.device != self.device:
            raise ValueError(f"expected float32 states [n_parts, n_rows, {2 + self.geom.head_dim}] "
                             f"on {self.device}, got {tuple(mlo.shape)} {mlo.dtype} on {mlo.device}")
        mlo = mlo.contiguous()
        n_parts, n_rows, w = mlo.shape
        out = self._check_result(out, (n_rows, w - 2), "out")
        with torch.cuda.device(self.device):
            check(self._lib.tq_lse_combine(mlo.data_ptr(), n_parts, n_rows, w - 2,
                                           out.data_ptr(), self._stream()))
        return out

    # -- read-back -------------------------------------------------------------------
    def dequant(self, layer: int, seq: int, start: int, end: int, keys=True, values=True):
        """Dequantised keys / values of tokens ``[start, end)``: float32 CUDA tensors
        ``[n_kv_heads, end - start, D]`` (``None`` for the one not requested)."""
        torch = _torch()
        g = self.geom
        n = max(end - start, 0)
        k = torch.empty((g.n_kv_heads, n, g.head_dim), dtype=torch.float32,
                        device=self.device) if keys else None
        v = torch.empty((g.n_kv_heads, n, g.head_dim), dtype=torch.float32,
                        device=self.device) if values else None
        with torch.cuda.device(self.device):
            check(self._lib.tq_dequant_range(self._h, layer, seq, start, end,
                                             k.data_ptr() if keys else None,
                                             v.data_ptr() if values else None, self._stream()))
        return k, v

    def export_block(self, layer: int, seq: int, block: int) -> dict:
        """Cold block ``block`` in the reference's container layout (host numpy arrays):
        the fields of ``CompressedPerChannelKV`` and ``CompressedKV``."""
        g = self.geom
        h, s, d = g.n_kv_heads, g.block_tokens, g.head_dim
        polar = self.key_mode == "polar"
        key_idx = np.empty(h * s * d * g.key_bits // 8 if polar else h * s * d // 2, np.uint8)
        scale = np.empty((1, h, s) if polar else (1, h, d), np.float32)  # polar: the key norms
        mean = np.empty((1, h, d), np.float32)
        cap = h * s * d
        oidx = np.empty(cap, np.int32)
        oval = np.empty(cap, np.uint16)
        n_out = C.c_int32(0)
        val_idx = np.empty(h * s * d * g.value_bits // 8, np.uint8)
        norms = np.empty((1, h, s), np.float32)
        with _torch().cuda.device(self.device):
            check(self._lib.tq_export_block(
                self._h, layer, seq, block, key_idx.ctypes.data, scale.ctypes.data,
                mean.ctypes.data, oidx.ctypes.data, oval.ctypes.data, cap, C.byref(n_out),
                val_idx.ctypes.data, norms.ctypes.data, self._stream()))
        n = n_out.value
        has = g.outlier_k > 0
        if polar:
            return {"key_indices": key_idx, "key_norms": scale, "nf4_scale": None,
                    "nf4_mean": None, "outlier_idx": None, "outlier_val": None,
                    "value_indices": val_idx, "value_norms": norms, "shape": (1, h, s, d),
                    "key_bits": g.key_bits, "value_bits": g.value_bits}
        return {
            "key_indices": key_idx, "nf4_scale": scale, "nf4_mean": mean,
            "outlier_idx": oidx[:n].copy() if has else None,
            "outlier_val": oval[:n].copy().view(np.float16) if has else None,
            "value_indices": val_idx, "value_norms": norms,
            "shape": (1, h, s, d), "key_bits": g.key_bits, "value_bits": g.value_bits,
        }

    def export_blob(self, layer: int, seq: int, block: int, rope_theta: float | None = None,
                    zero_point: str = "calibrated") -> bytes:
        """Cold block ``block`` as one ``tqp-kv-npz/1`` byte string, the layout of the
        reference's vLLM connector (``connectors/vllm_v1.py:113-137``); see
        :mod:`turboquant_pro_b200.kv_blob`.  ``zero_point`` / ``rope_theta`` name the key
        zero-point mode the context was set up with (``"sparse"`` after
        :meth:`set_key_mean_mask`, ``"bias"`` after :meth:`set_key_bias_means`)."""
        from .kv_blob import block_to_blob

        dt = {0: "float32", 1: "float16", 2: "bfloat16"}[self.geom.kv_dtype]
        return block_to_blob(self.export_block(layer, seq, block), key_mode=self.key_mode,
                             zero_point=zero_point, mean_mask=self.key_mean_mask,
                             rope_theta=rope_theta,
                             position_start=block * self.geom.block_tokens, dtype=dt)

    def import_block(self, layer: int, seq: int, block: int, blk: dict) -> None:
        """The inverse of :meth:`export_block`: writes cold block ``block`` of a cleared cache
        from the container arrays (``nf4_mean`` is the full ``(1, H, D)`` zero-point).
        :meth:`restore_hot` then sets the length."""
        g = self.geom
        h, s, d = g.n_kv_heads, g.block_tokens, g.head_dim
        key_idx = np.ascontiguousarray(blk["key_indices"], dtype=np.uint8).reshape(-1)
        scale = np.ascontiguousarray(blk["nf4_scale"], dtype=np.float32).reshape(-1)
        mean = np.ascontiguousarray(blk["nf4_mean"], dtype=np.float32).reshape(-1)
        val_idx = np.ascontiguousarray(blk["value_indices"], dtype=np.uint8).reshape(-1)
        norms = np.ascontiguousarray(blk["value_norms"], dtype=np.float32).reshape(-1)
        if key_idx.size != h * s * d // 2 or scale.size != h * d or mean.size != h * d \
                or val_idx.size != h * s * d * g.value_bits // 8 or norms.size != h * s:
            raise ValueError("container arrays do not match this context's block shape "
                             f"(H={h}, S={s}, D={d}, value_bits={g.value_bits})")
        oidx = blk.get("outlier_idx")
        n_out = 0
        if oidx is not None and len(oidx):
            oidx = np.ascontiguousarray(oidx, dtype=np.int32)
            oval = np.ascontiguousarray(blk["outlier_val"]).view(np.uint16).reshape(-1)
            if oval.size != oidx.size:
                raise ValueError("outlier_idx and outlier_val differ in length")
            n_out = int(oidx.size)
        with _torch().cuda.device(self.device):
            check(self._lib.tq_import_block(
                self._h, layer, seq, block, key_idx.ctypes.data, scale.ctypes.data,
                mean.ctypes.data, oidx.ctypes.data if n_out else None,
                oval.ctypes.data if n_out else None, n_out, val_idx.ctypes.data,
                norms.ctypes.data, self._stream()))

    def restore_hot(self, layer: int, seq: int, n_tokens: int, hot_k, hot_v) -> None:
        """Completes a restore: the cache holds ``n_tokens`` tokens, its cold blocks were
        imported, and ``hot_k`` / ``hot_v`` (tensors ``[tokens, n_kv_heads, D]``) are the tokens after the last cold block."""
        torch = _torch()
        g = self.geom
        n_hot = n_tokens - self.cold_blocks(n_tokens) * g.block_tokens
        for t in (hot_k, hot_v):
            if tuple(t.shape) != (n_hot, g.n_kv_heads, g.head_dim):
                raise ValueError(f"expected hot tensors of shape "
                                 f"{(n_hot, g.n_kv_heads, g.head_dim)}, got {tuple(t.shape)}")
        k = hot_k.to(device=self.device, dtype=self.kv_dtype).contiguous()
        v = hot_v.to(device=self.device, dtype=self.kv_dtype).contiguous()
        with torch.cuda.device(self.device):
            check(self._lib.tq_restore_hot(self._h, layer, seq, n_tokens, k.data_ptr(),
                                           v.data_ptr(), k.stride(0), k.stride(1),
                                           self._stream()))

    def cold_blocks(self, n_tokens: int) -> int:
        """Cold blocks of a cache that holds ``n_tokens`` tokens (the reference's flush rule:
        the oldest half of an over-full hot window becomes a block)."""
        g = self.geom
        return 0 if n_tokens <= g.hot_window else 1 + (n_tokens - g.hot_window - 1) // g.block_tokens

    def import_blob(self, layer: int, seq: int, block: int, blob: bytes,
                    bias_means=None) -> None:
        """Writes cold block ``block`` from a ``tqp-kv-npz/1`` byte string (see
        :mod:`turboquant_pro_b200.kv_blob`).  A blob with the ``sparse`` zero-point needs this
        context's channel mask (:meth:`set_key_mean_mask`); one with the ``bias`` zero-point
        stores no means, so ``bias_means`` ``(n_kv_heads, D)`` of this block must be given."""
        from .kv_blob import blob_to_block, block_from_parsed

        parsed = blob_to_block(blob)
        self.import_block(layer, seq, block, block_from_parsed(
            parsed, key_mode=self.key_mode, mean_mask=self.key_mean_mask, bias_means=bias_means,
            geom=(self.geom.n_kv_heads, self.geom.block_tokens, self.geom.head_dim,
                  self.geom.value_bits)))

    def export_state(self, layer: int, seq: int, rope_theta: float | None = None,
                     zero_point: str = "calibrated") -> dict:
        """Everything one cache holds, for offload: its cold blocks as ``tqp-kv-npz/1`` byte
        strings and the uncompressed hot window as raw 16/32-bit words.  :meth:`import_state`
        of a context with the same geometry, seed and key format restores it exactly."""
        total, cold, _hot = self.lengths(layer, seq)
        nb = cold // self.geom.block_tokens
        blocks = [self.export_blob(layer, seq, b, rope_theta=rope_theta, zero_point=zero_point)
                  for b in range(nb)]
        torch = _torch()
        if total > cold:  # the window's values are stored exactly
            hk, hv = self.dequant(layer, seq, cold, total)
        else:
            hk = hv = torch.empty((self.geom.n_kv_heads, 0, self.geom.head_dim), device=self.device)
        raw = []
        for t in (hk, hv):
            t = t.permute(1, 0, 2).to(self.kv_dtype).contiguous().cpu()
            word = _torch().int32 if t.element_size() == 4 else _torch().int16
            raw.append(t.view(word).numpy().copy())
        return {"n_tokens": total, "blocks": blocks, "hot_k": raw[0], "hot_v": raw[1],
                "kv_dtype": str(self.kv_dtype).replace("torch.", ""),
                "geom": (self.geom.n_kv_heads, self.geom.block_tokens, self.geom.head_dim,
                         self.geom.value_bits), "key_mode": self.key_mode}

    def import_state(self, layer: int, seq: int, state: dict, bias_means=None) -> None:
        """Replaces the cache of ``(layer, seq)`` by an exported one (see :meth:`export_state`).
        ``bias_means`` ``[n_blocks, n_kv_heads, D]`` is needed for blocks written with the
        ``bias`` zero-point."""
        torch = _torch()
        g = self.geom
        mine = (g.n_kv_heads, g.block_tokens, g.head_dim, g.value_bits)
        if tuple(state["geom"]) != mine or state["key_mode"] != self.key_mode \
                or state["kv_dtype"] != str(self.kv_dtype).replace("torch.", ""):
            raise ValueError("the exported cache has another geometry, key format or dtype")
        n = int(state["n_tokens"])
        if len(state["blocks"]) != self.cold_blocks(n):
            raise ValueError("block count does not match the token count")
        self.clear(layer, seq)
        for b, blob in enumerate(state["blocks"]):
            self.import_blob(layer, seq, b, blob,
                             bias_means=None if bias_means is None else bias_means[b])
        if n:
            hot = [torch.from_numpy(np.ascontiguousarray(state[name])).view(self.kv_dtype)
                   for name in ("hot_k", "hot_v")]
            self.restore_hot(layer, seq, n, hot[0], hot[1])

    # -- bookkeeping -----------------------------------------------------------------
    def lengths(self, layer: int, seq: int):
        """(total, cold, hot) token counts of one cache."""
        t, c, h = C.c_int32(), C.c_int32(), C.c_int32()
        check(self._lib.tq_seq_lengths(self._h, layer, seq, C.byref(t), C.byref(c), C.byref(h)))
        return t.value, c.value, h.value

    def memory_stats(self, layer: int, seq: int):
        """(cold_bytes, hot_bytes) counted like the reference's containers."""
        cold, hot = C.c_double(), C.c_double()
        with _torch().cuda.device(self.device):
            check(self._lib.tq_memory_stats(self._h, layer, seq, C.byref(cold), C.byref(hot),
                                            self._stream()))
        return cold.value, hot.value

    def clear(self, layer: int, seq: int = -1) -> None:
        with _torch().cuda.device(self.device):
            check(self._lib.tq_clear(self._h, layer, seq, self._stream()))

    def status(self) -> int:
        """Device status flags (bit 0: an outlier pool overflowed; bit 1: a bounded wait of the
        tensor-core decode kernel ran out and that call's output is undefined); clears them."""
        f = C.c_int32()
        with _torch().cuda.device(self.device):
            check(self._lib.tq_status(self._h, C.byref(f), self._stream()))
        return f.value

    def decode_bytes(self, layer: int) -> float:
        """Algorithmic bytes one :meth:`decode` of ``layer`` reads."""
        b = C.c_double()
        check(self._lib.tq_decode_bytes(self._h, layer, C.byref(b)))
        return b.value

    def last_launches(self) -> int:
        return int(self._lib.tq_last_launches(self._h))

    def set_key_mean_mask(self, mask) -> None:
        """Channels whose mean is kept as the key zero-point (``None``: all).  Applies to the
        blocks encoded from now on."""
        m = None
        if mask is not None:
            m = np.ascontiguousarray(np.asarray(mask).astype(bool).astype(np.uint8))
            if m.shape != (self.geom.head_dim,):
                raise ValueError(f"expected a mask of {self.geom.head_dim} channels")
        with _torch().cuda.device(self.device):
            check(self._lib.tq_set_key_mean_mask(self._h, m.ctypes.data if m is not None else None,
                                                 self._stream()))
        self.key_mean_mask = None if m is None else m.astype(bool)

    def set_key_bias_means(self, means) -> None:
        """Given key zero-points, one ``(n_kv_heads, head_dim)`` row per cold block index
        (``[max_blocks, n_kv_heads, head_dim]`` float32; ``None`` goes back to measured
        means): the reference's ``zero_point="bias"``.  Applies to blocks encoded from now
        on."""
        g = self.geom
        m = None
        if means is not None:
            m = np.ascontiguousarray(means, dtype=np.float32)
            if m.shape != (g.max_blocks, g.n_kv_heads, g.head_dim):
                raise ValueError(f"expected means of shape "
                                 f"{(g.max_blocks, g.n_kv_heads, g.head_dim)}, got {m.shape}")
        with _torch().cuda.device(self.device):
            check(self._lib.tq_set_key_bias_means(
                self._h, m.ctypes.data if m is not None else None, self._stream()))

    def set_kernel(self, which: str = "auto") -> None:
        """``"auto"``: tensor-core kernel where the geometry allows; ``"general"``: always the
        general-shape float32 kernel."""
        check(self._lib.tq_set_kernel(self._h, {"auto": 0, "general": 1}[which]))

    def last_kernel(self) -> str:
        """Which kernel served the most recent decode: ``"tensor-core"``, ``"general"`` or
        ``"none"``."""
        return {0: "none", 1: "tensor-core", 2: "general"}[int(self._lib.tq_last_kernel(self._h))]

    def debug_wait(self, wait_limit: int = 0, withhold_tile: int = -1) -> None:
        """Test hook of the decode kernel's bounded waits: a shorter probe limit and a tile of
        the first CTA whose copy is never started (see ``tq_debug_wait``)."""
        check(self._lib.tq_debug_wait(self._h, int(wait_limit), int(withhold_tile)))

    def trace(self, on: bool, read: bool = False):
        """Switch the decode kernel's pipeline stamping on/off; with ``read`` return the
        stamps of the last traced decode as a (64, 8) uint64 array of SM clocks."""
        buf = np.zeros((64, 8), np.uint64) if read else None
        with _torch().cuda.device(self.device):
            check(self._lib.tq_debug_trace(self._h, int(bool(on)),
                                           buf.ctypes.data if read else None, self._stream()))
        return buf

    def profile(self, on: bool) -> None:
        """Bracket the attention and combine kernels of every decode with CUDA events."""
        check(self._lib.tq_profile_enable(self._h, int(bool(on))))

    def profile_read(self):
        """(attention-kernel ms, combine-kernel ms, calls) summed since the last read."""
        a, c, n = C.c_double(), C.c_double(), C.c_int32()
        with _torch().cuda.device(self.device):
            check(self._lib.tq_profile_read(self._h, C.byref(a), C.byref(c), C.byref(n)))
        return a.value, c.value, n.value

"""CPU oracle for the compressed-KV hot path (TEST INFRASTRUCTURE, not product code).

A numpy restatement of the reference's append/encode + dequantise-then-attend path.
Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may
import this module; the product package never does.

Every arithmetic step whose *order* decides the emitted bits is written out
explicitly (sequential sums, the 8-accumulator norm, multiply-then-add rotation) so
the result does not depend on which SIMD/FMA loop a given numpy build dispatches to.
Parity is pinned: ``tests/golden/*.npz`` were produced by importing the reference
itself (``tests/golden/make_golden.py``) and ``tests/test_oracle_golden.py`` checks
every function here against them bit for bit.

Reference locations restated here (paths inside the reference project):

* key encoder ............ ``turboquant_pro/per_channel_kv.py:269-401``
* key packing ............ ``turboquant_pro/per_channel_kv.py:87-100``
* key decoder ............ ``turboquant_pro/per_channel_kv.py:497-539``
* value codebooks ........ ``turboquant_pro/core.py:70-93, 229-241``
* rotation matrix ........ ``turboquant_pro/core.py:246-260``
* value encoder .......... ``turboquant_pro/core.py:542-617``
* value packing .......... ``turboquant_pro/core.py:350-441``
* value decoder .......... ``turboquant_pro/core.py:619-654``
* two-tier cache ......... ``turboquant_pro/core.py:986-1117``
* partial merge .......... ``turboquant_pro/kv_fused.py:101-153``
* fused key score ........ ``turboquant_pro/kv_fused_pck.py:54-127, 196-236``
"""

from __future__ import annotations

import math

import numpy as np

F32 = np.float32

# NormalFloat-4 levels (QLoRA, Dettmers et al. 2023); per_channel_kv.py:64-84.
NF4 = np.array(
    [
        -1.0,
        -0.6961928009986877,
        -0.5250730514526367,
        -0.39491748809814453,
        -0.28444138169288635,
        -0.18477343022823334,
        -0.09105003625154495,
        0.0,
        0.07958029955625534,
        0.16093020141124725,
        0.24611230194568634,
        0.33791524171829224,
        0.44070982933044434,
        0.5626170039176941,
        0.7229568362236023,
        1.0,
    ],
    dtype=F32,
)

# Lloyd-Max centroids of N(0,1) for 2/3/4 bits; core.py:70-93.
LLOYD_MAX = {
    2: np.array([-1.510, -0.453, 0.453, 1.510]),
    3: np.array([-1.748, -1.050, -0.500, -0.069, 0.069, 0.500, 1.050, 1.748]),
    4: np.array(
        [-2.401, -1.844, -1.437, -1.099, -0.800, -0.524, -0.262, -0.066,
         0.066, 0.262, 0.524, 0.800, 1.099, 1.437, 1.844, 2.401]
    ),
}


# --------------------------------------------------------------------------- #
# constants                                                                    #
# --------------------------------------------------------------------------- #

def value_tables(head_dim: int, bits: int):
    """Centroids and bin boundaries of the PolarQuant direction codebook.

    core.py:229-241 — the raw table is scaled in float64 by ``1/sqrt(d)``, rounded to
    float32, and the boundaries are float32 mid-points of adjacent centroids.
    """
    scale = 1.0 / math.sqrt(head_dim)
    c = (LLOYD_MAX[bits] * scale).astype(F32)
    bnd = ((c[:-1] + c[1:]) / F32(2.0)).astype(F32)
    return c, bnd


def rotation(head_dim: int, seed):
    """Random orthogonal matrix ``Pi`` and its transposed copy (core.py:246-260)."""
    rng = np.random.default_rng(seed)
    g = rng.standard_normal((head_dim, head_dim)).astype(F32)
    q, _ = np.linalg.qr(g)
    return np.ascontiguousarray(q), np.ascontiguousarray(q.T)


def block_tokens(hot_window: int) -> int:
    """Tokens per cold block: half of an over-full hot window (core.py:1013)."""
    return (hot_window + 1) // 2


def n_cold_blocks(n_tokens: int, hot_window: int) -> int:
    """Cold blocks after ``n_tokens`` single-token appends (core.py:1008-1014)."""
    if n_tokens <= hot_window:
        return 0
    return 1 + (n_tokens - hot_window - 1) // block_tokens(hot_window)


# --------------------------------------------------------------------------- #
# arithmetic helpers with pinned evaluation order                              #
# --------------------------------------------------------------------------- #

def _seq_sum_axis(x: np.ndarray, axis: int) -> np.ndarray:
    """Left-to-right float32 sum along ``axis``: ((x0+x1)+x2)+..."""
    x = np.moveaxis(x, axis, 0)
    acc = x[0].astype(F32, copy=True)
    for i in range(1, x.shape[0]):
        acc = (acc + x[i]).astype(F32)
    return acc


def _pairwise_sum_last(a: np.ndarray) -> np.ndarray:
    """numpy's pairwise float32 summation along the last axis, written out.

    n < 8: plain loop.  n <= 128: eight strided accumulators combined as
    ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7)), then the tail.  n > 128: split at
    ``n//2`` rounded down to a multiple of 8 and recurse.
    """
    n = a.shape[-1]
    if n < 8:
        acc = np.zeros(a.shape[:-1], dtype=F32)
        # numpy starts from the first element, which equals 0 + a0 for finite data
        acc = a[..., 0].astype(F32, copy=True) if n else acc
        for i in range(1, n):
            acc = (acc + a[..., i]).astype(F32)
        return acc
    if n <= 128:
        r = [a[..., j].astype(F32, copy=True) for j in range(8)]
        full = n - (n % 8)
        for i in range(8, full, 8):
            for j in range(8):
                r[j] = (r[j] + a[..., i + j]).astype(F32)
        res = ((r[0] + r[1]) + (r[2] + r[3])) + ((r[4] + r[5]) + (r[6] + r[7]))
        res = res.astype(F32)
        for i in range(full, n):
            res = (res + a[..., i]).astype(F32)
        return res
    n2 = n // 2
    n2 -= n2 % 8
    return (_pairwise_sum_last(a[..., :n2]) + _pairwise_sum_last(a[..., n2:])).astype(F32)


def _rotate(x: np.ndarray, mat: np.ndarray) -> np.ndarray:
    """``y[..., e] = sum_d x[..., d] * mat[d, e]`` accumulated left to right over d,
    each product rounded to float32 before the (rounded) add — no fused multiply-add."""
    acc = (x[..., 0:1] * mat[0]).astype(F32)
    for d in range(1, x.shape[-1]):
        acc = (acc + (x[..., d:d + 1] * mat[d]).astype(F32)).astype(F32)
    return acc


# --------------------------------------------------------------------------- #
# keys: per-channel asymmetric NF4 + fp16 outlier side-list                    #
# --------------------------------------------------------------------------- #

def outlier_count(n_tokens: int, frac: float) -> int:
    """Entries kept per channel: max(1, round(S*frac)), Python banker's rounding."""
    return max(1, int(round(n_tokens * frac)))


def key_outliers(x: np.ndarray, frac: float):
    """Per-channel top-magnitude entries (per_channel_kv.py:269-283).

    ``x`` is (H, S, D).  Returns ascending flat int32 indices into (H, S, D) and the
    float16 values there; every element tied with the k-th largest magnitude is kept.
    """
    if frac <= 0.0:
        return None, None
    h, s, d = x.shape
    k = outlier_count(s, frac)
    if k >= s:
        mask = np.ones(x.shape, dtype=bool)
    else:
        absx = np.abs(x)
        kth = np.sort(absx, axis=1)[:, s - k:s - k + 1, :]
        mask = absx >= kth
    idx = np.flatnonzero(mask).astype(np.int32)
    val = x.reshape(-1)[idx].astype(np.float16)
    return idx, val


KEY_MODES = ("nf4_asym", "nf4", "uniform")  # the per-channel key grids with a fused form


def key_grid(mode: str) -> np.ndarray:
    """The 16-level grid of a key mode: dequant = mean + scale * grid[code]
    (kv_fused_pck.py:54-94)."""
    return np.arange(16, dtype=F32) if mode == "uniform" else NF4


def dc_channel_mask(rope_theta: float, head_dim: int, window: int) -> np.ndarray:
    """Channels whose rotary wavelength exceeds ``window`` tokens (per_channel_kv.py:233-241):
    pair i of the rotate-half layout turns with angular frequency theta^(-2i/D), so its
    wavelength is 2*pi*theta^(2i/D); channels i and i + D/2 share it."""
    half = head_dim // 2
    inv_freq = rope_theta ** (-2.0 * np.arange(half) / head_dim)
    wavelength = 2.0 * np.pi / inv_freq
    return np.tile(wavelength, 2)[:head_dim] > float(window)


def rope_averaged_bias(k_bias, rope_theta: float, head_dim: int, start: int, n: int):
    """The "bias" zero-point (per_channel_kv.py:243-267): the key-projection bias ``(H, D)``
    rotated by RoPE and averaged over positions ``[start, start + n)``.  The means of cos and
    sin are taken in float64 and rounded to float32; the rotation itself
    (b*cos + rotate_half(b)*sin) is float32."""
    half = head_dim // 2
    inv_freq = rope_theta ** (-2.0 * np.arange(half, dtype=np.float64) / head_dim)
    angle = np.arange(start, start + n, dtype=np.float64)[:, None] * inv_freq[None, :]
    mean_cos = np.cos(angle).mean(axis=0)
    mean_sin = np.sin(angle).mean(axis=0)
    cos_full = np.concatenate([mean_cos, mean_cos]).astype(F32)
    sin_full = np.concatenate([mean_sin, mean_sin]).astype(F32)
    b = np.asarray(k_bias, dtype=F32).reshape(-1, head_dim)
    rotated_half = np.concatenate([-b[:, half:], b[:, :half]], axis=1)
    return b * cos_full[None, :] + rotated_half * sin_full[None, :]


def encode_keys(x: np.ndarray, outlier_frac: float = 0.0, mode: str = "nf4_asym",
                dc_mask: np.ndarray | None = None, given_mean: np.ndarray | None = None):
    """Per-channel 4-bit key block encoder (per_channel_kv.py:285-401).

    ``x`` (H, S, D) any float dtype.  Returns a dict with unpacked ``codes`` (H,S,D)
    uint8, per-channel ``scale`` and ``mean`` (H,D) such that the dense value is
    ``mean + scale * grid[code]``, and the outlier side-list (``out_idx``, ``out_val``) or
    ``None``s.  Modes:

    * ``"nf4_asym"`` (:324-353, :377-401): mean over tokens, scale = max|x-mean| floored at
      1e-8, level = fl(mean + fl(scale*NF4[l])), nearest level, first minimum wins;
    * ``"nf4"`` (:354-357): mean = 0, scale = max|x| floored, level = fl(scale*NF4[l]);
    * ``"uniform"`` (:303-318): mean = min, scale = fl(max(max-min, 1e-8) / 15),
      code = clip(round_half_even(fl(fl(x-min)/scale)), 0, 15).

    ``dc_mask`` (D,) bool, asymmetric NF4 only: the "sparse" zero-point (:337-342) keeps the
    mean on the masked channels and uses 0 elsewhere.  ``given_mean`` (H, D), asymmetric NF4
    only: the "bias" zero-point (:327-336) uses it instead of the measured mean.
    """
    if mode not in KEY_MODES:
        raise ValueError(f"unknown key mode {mode!r}")
    x = np.asarray(x, dtype=F32)
    h, s, d = x.shape
    out_idx, out_val = key_outliers(x, outlier_frac)
    if mode == "uniform":
        mn = x.min(axis=1)
        mx = x.max(axis=1)
        scale = (np.maximum((mx - mn).astype(F32), F32(1e-8)) / F32(15)).astype(F32)
        q = ((x - mn[:, None, :]).astype(F32) / scale[:, None, :]).astype(F32)
        codes = np.clip(np.round(q), 0, 15).astype(np.uint8)
        return {"codes": codes, "scale": scale, "mean": mn.astype(F32), "out_idx": out_idx,
                "out_val": out_val, "mode": mode}
    if mode == "nf4_asym":
        mean = (_seq_sum_axis(x, 1) / F32(s)).astype(F32)
        if given_mean is not None:
            mean = np.asarray(given_mean, dtype=F32)
        if dc_mask is not None:
            mean = (mean * np.asarray(dc_mask, dtype=bool)[None, :]).astype(F32)
        xc = (x - mean[:, None, :]).astype(F32)
        amax = np.maximum(np.abs(xc).max(axis=1), F32(1e-8)).astype(F32)
        # level l of channel (h, d): fl(mean + fl(amax * NF4[l]))
        levels = (mean[..., None] + (amax[..., None] * NF4).astype(F32)).astype(F32)  # (H,D,16)
    else:
        mean = np.zeros((h, d), dtype=F32)
        amax = np.maximum(np.abs(x).max(axis=1), F32(1e-8)).astype(F32)
        levels = (amax[..., None] * NF4).astype(F32)
    # nearest level, first minimum wins
    dist = np.abs((x[:, :, :, None] - levels[:, None, :, :]).astype(F32))  # (H,S,D,16)
    codes = dist.argmin(axis=-1).astype(np.uint8)
    return {
        "codes": codes,
        "scale": amax,
        "mean": mean,
        "out_idx": out_idx,
        "out_val": out_val,
        "mode": mode,
    }


def _rev4(c: np.ndarray) -> np.ndarray:
    c = c.astype(np.uint8)
    return ((c & 1) << 3) | ((c & 2) << 1) | ((c & 4) >> 1) | ((c & 8) >> 3)


def pack_key_codes(codes: np.ndarray) -> np.ndarray:
    """4-bit key packing (per_channel_kv.py:87-93): each code's bits are emitted
    LSB-first into an MSB-first byte stream, i.e. byte = rev4(even) << 4 | rev4(odd)."""
    flat = codes.reshape(-1)
    assert flat.size % 2 == 0
    return ((_rev4(flat[0::2]) << 4) | _rev4(flat[1::2])).astype(np.uint8)


def unpack_key_codes(packed: np.ndarray, n_values: int) -> np.ndarray:
    packed = packed.reshape(-1)
    out = np.empty(packed.size * 2, dtype=np.uint8)
    out[0::2] = _rev4(packed >> 4)
    out[1::2] = _rev4(packed & 0xF)
    return out[:n_values]


def dequant_keys(codes, scale, mean, out_idx=None, out_val=None, mode="nf4_asym") -> np.ndarray:
    """Key block decoder (per_channel_kv.py:497-539): level = fl(fl(scale*grid)+mean)
    (symmetric NF4 adds no mean; uniform is fl(fl(code*scale)+zero), the same expression),
    then outlier positions are overwritten with their float16 values."""
    levels = (scale[..., None] * key_grid(mode)).astype(F32)  # (H,D,16)
    if mode != "nf4":
        levels = (levels + mean[..., None]).astype(F32)
    h, s, d = codes.shape
    out = np.take_along_axis(
        levels[:, None, :, :], codes[..., None].astype(np.int64), axis=-1
    )[..., 0].astype(F32)
    out = np.ascontiguousarray(out)
    if out_idx is not None:
        out.reshape(-1)[out_idx] = out_val.astype(F32)
    return out


# --------------------------------------------------------------------------- #
# values: PolarQuant (norm + rotated Lloyd-Max direction codes)                #
# --------------------------------------------------------------------------- #

def encode_values(x: np.ndarray, pi_t: np.ndarray, boundaries: np.ndarray):
    """PolarQuant value encoder (core.py:562-593).

    ``x`` (H, S, D).  norm = sqrt(pairwise sum of squares); unit = x / max(norm, 1e-30);
    y = unit @ Pi_T (sequential, unfused); code = number of boundaries strictly below y.
    """
    x = np.asarray(x, dtype=F32)
    sq = (x * x).astype(F32)
    norms = np.sqrt(_pairwise_sum_last(sq)).astype(F32)
    unit = (x / np.maximum(norms, F32(1e-30))[..., None]).astype(F32)
    y = _rotate(unit, pi_t)
    codes = np.searchsorted(boundaries, y, side="left").astype(np.uint8)
    return {"codes": codes, "norms": norms}


def pack_value_codes(codes: np.ndarray, bits: int) -> np.ndarray:
    """LSB-first packing of direction codes (core.py:350-398)."""
    flat = codes.reshape(-1).astype(np.uint32)
    if bits == 4:
        assert flat.size % 2 == 0
        return (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)
    if bits == 3:
        assert flat.size % 8 == 0
        g = flat.reshape(-1, 8)
        w = np.zeros(g.shape[0], dtype=np.uint32)
        for i in range(8):
            w |= g[:, i] << (3 * i)
        out = np.empty((g.shape[0], 3), dtype=np.uint8)
        out[:, 0] = w & 0xFF
        out[:, 1] = (w >> 8) & 0xFF
        out[:, 2] = (w >> 16) & 0xFF
        return out.reshape(-1)
    if bits == 2:
        assert flat.size % 4 == 0
        g = flat.reshape(-1, 4)
        return (g[:, 0] | (g[:, 1] << 2) | (g[:, 2] << 4) | (g[:, 3] << 6)).astype(np.uint8)
    raise ValueError(f"unsupported value bits {bits}")


def unpack_value_codes(packed: np.ndarray, n_values: int, bits: int) -> np.ndarray:
    p = packed.reshape(-1).astype(np.uint32)
    if bits == 4:
        out = np.empty(p.size * 2, dtype=np.uint8)
        out[0::2] = p & 0xF
        out[1::2] = p >> 4
        return out[:n_values]
    if bits == 3:
        t = p.reshape(-1, 3)
        w = t[:, 0] | (t[:, 1] << 8) | (t[:, 2] << 16)
        out = np.stack([(w >> (3 * i)) & 7 for i in range(8)], axis=1).astype(np.uint8)
        return out.reshape(-1)[:n_values]
    if bits == 2:
        out = np.stack([(p >> (2 * i)) & 3 for i in range(4)], axis=1).astype(np.uint8)
        return out.reshape(-1)[:n_values]
    raise ValueError(f"unsupported value bits {bits}")


def dequant_values(codes, norms, centroids, pi) -> np.ndarray:
    """Value block decoder (core.py:645-652): centroid lookup, inverse rotation
    (sequential, unfused), scale by the stored norm."""
    y = centroids[codes.astype(np.int64)].astype(F32)
    x = _rotate(y, pi)
    return (x * norms[..., None]).astype(F32)


# --------------------------------------------------------------------------- #
# attention                                                                    #
# --------------------------------------------------------------------------- #

def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray) -> np.ndarray:
    """fp32 ``softmax(q K^T / sqrt(D)) V`` for one decode step.

    ``q`` (Hq, D), ``k``/``v`` (Hkv, S, D); query head i reads KV head
    ``i // (Hq // Hkv)``.  Returns (Hq, D) float32.
    """
    q = np.asarray(q, dtype=F32)
    hq, d = q.shape
    hkv = k.shape[0]
    g = hq // hkv
    kk = np.repeat(np.asarray(k, dtype=F32), g, axis=0)
    vv = np.repeat(np.asarray(v, dtype=F32), g, axis=0)
    sc = np.einsum("hd,hsd->hs", q, kk) / F32(math.sqrt(d))
    sc = sc - sc.max(axis=-1, keepdims=True)
    e = np.exp(sc)
    p = e / e.sum(axis=-1, keepdims=True)
    return np.einsum("hs,hsd->hd", p, vv).astype(F32)


def partials(q, k, v, scale):
    """Unnormalised online-softmax state (m, l, acc) of a token range
    (kv_fused.py:101-117); GQA as in :func:`attention`."""
    q = np.asarray(q, dtype=F32)
    g = q.shape[0] // k.shape[0]
    kk = np.repeat(np.asarray(k, dtype=F32), g, axis=0)
    vv = np.repeat(np.asarray(v, dtype=F32), g, axis=0)
    sc = np.einsum("hd,hsd->hs", q, kk) * F32(scale)
    m = sc.max(axis=1)
    e = np.exp(sc - m[:, None])
    return m, e.sum(axis=1), np.einsum("hs,hsd->hd", e, vv)


def merge_partials(parts):
    """LSE merge of (m, l, acc) states (kv_fused.py:139-153)."""
    big = parts[0][0]
    for m, _, _ in parts[1:]:
        big = np.maximum(big, m)
    num = np.zeros_like(parts[0][2])
    den = np.zeros_like(parts[0][1])
    for m, l, acc in parts:
        w = np.exp(m - big)
        num = num + acc * w[:, None]
        den = den + l * w
    return num / den[:, None]


def outlier_deltas(block):
    """Token-major list of score corrections for one key block
    (kv_fused_pck.py:97-127): delta = fp16 value - dense dequantised value.

    Returns (h, s, d, delta) arrays sorted by (h, s, d)."""
    if block["out_idx"] is None:
        z = np.zeros(0, dtype=np.int64)
        return z, z, z, np.zeros(0, dtype=F32)
    codes = block["codes"]
    hh, s, d = codes.shape
    flat = block["out_idx"].astype(np.int64)
    h_i = flat // (s * d)
    s_i = (flat // d) % s
    d_i = flat % d
    grid = key_grid(block.get("mode", "nf4_asym"))
    dense = (block["mean"][h_i, d_i]
             + block["scale"][h_i, d_i] * grid[codes[h_i, s_i, d_i]]).astype(F32)
    delta = (block["out_val"].astype(F32) - dense).astype(F32)
    return h_i, s_i, d_i, delta


def fused_key_scores(q, block):
    """Score of every token of a key block computed on the codes
    (kv_fused_pck.py:196-209): q.mean + sum_d (q_d scale_d) NF4[code] + outlier deltas.
    ``q`` (H, D) — one query head per KV head."""
    q = np.asarray(q, dtype=F32)
    w = q * block["scale"]
    bias = (q * block["mean"]).sum(axis=1)
    grid = key_grid(block.get("mode", "nf4_asym"))
    sc = np.einsum("hd,hsd->hs", w, grid[block["codes"].astype(np.int64)]) + bias[:, None]
    h_i, s_i, d_i, delta = outlier_deltas(block)
    if h_i.size:
        corr = np.zeros(sc.shape, dtype=np.float64)
        np.add.at(corr, (h_i, s_i), q.astype(np.float64)[h_i, d_i] * delta.astype(np.float64))
        sc = sc + corr.astype(F32)
    return sc


# --------------------------------------------------------------------------- #
# two-tier cache                                                               #
# --------------------------------------------------------------------------- #

class OracleCache:
    """Two-tier KV cache of one layer and one sequence (core.py:818-1307).

    Tokens are appended one at a time into a hot list; when it exceeds ``hot_window``
    the oldest half is encoded into one cold block.  Keys use asymmetric NF4 with an
    optional outlier list, values use PolarQuant with ``value_bits``.
    """

    def __init__(self, head_dim=128, n_heads=32, key_bits=4, value_bits=4, hot_window=512,
                 outlier_frac=0.02, seed=None, key_mode="nf4_asym", rope_theta=None,
                 k_bias=None):
        if key_mode == "polar":
            # the legacy format (core.py:1022-1033): keys through the value quantiser
            if key_bits != value_bits:
                raise ValueError("PolarQuant keys are restated for key_bits == value_bits")
            outlier_frac = 0.0
        elif key_bits != 4:
            raise ValueError("the per-channel key formats restated here are 4-bit")
        self.key_mode = key_mode
        # rope_theta alone selects the "sparse" zero-point (means only on long-wavelength
        # channels); with k_bias it selects the "bias" zero-point (no measured mean at all)
        self.rope_theta = rope_theta
        self.k_bias = None if k_bias is None else np.asarray(k_bias, F32).reshape(n_heads, head_dim)
        self.head_dim, self.n_heads = head_dim, n_heads
        self.key_bits, self.value_bits = key_bits, value_bits
        self.hot_window, self.outlier_frac = hot_window, outlier_frac
        self.pi, self.pi_t = rotation(head_dim, seed)
        self.centroids, self.boundaries = value_tables(head_dim, value_bits)
        self.hot_k: list[np.ndarray] = []
        self.hot_v: list[np.ndarray] = []
        self.cold_k: list[dict] = []
        self.cold_v: list[dict] = []
        self.cold_lengths: list[int] = []
        self.length = 0

    def _dc_mask(self, n_tokens: int):
        """The sparse zero-point's channel mask for a block of ``n_tokens`` (the window the
        wavelengths are compared with is the block itself), or None."""
        if self.rope_theta is None or self.k_bias is not None:
            return None
        return dc_channel_mask(self.rope_theta, self.head_dim, n_tokens)

    @property
    def cold_length(self):
        return sum(self.cold_lengths)

    @property
    def hot_length(self):
        return len(self.hot_k)

    def append(self, key, value):
        """One token; ``key``/``value`` are (H, D)."""
        self.hot_k.append(np.asarray(key))
        self.hot_v.append(np.asarray(value))
        self.length += 1
        if len(self.hot_k) > self.hot_window:
            self._flush()

    def _flush(self):
        n = len(self.hot_k) // 2
        if n == 0:
            return
        kb = np.stack(self.hot_k[:n], axis=1)  # (H, n, D)
        vb = np.stack(self.hot_v[:n], axis=1)
        given = None
        if self.k_bias is not None:
            given = rope_averaged_bias(self.k_bias, self.rope_theta, self.head_dim,
                                       sum(self.cold_lengths), n)
        if self.key_mode == "polar":
            self.cold_k.append(encode_values(kb, self.pi_t, self.boundaries))
        else:
            self.cold_k.append(encode_keys(kb, self.outlier_frac, self.key_mode,
                                           self._dc_mask(n), given))
        self.cold_v.append(encode_values(vb, self.pi_t, self.boundaries))
        self.cold_lengths.append(n)
        del self.hot_k[:n]
        del self.hot_v[:n]

    def keys(self) -> np.ndarray:
        """All keys (H, N, D) float32: dequantised cold blocks then the hot tokens."""
        if self.key_mode == "polar":
            parts = [dequant_values(b["codes"], b["norms"], self.centroids, self.pi)
                     for b in self.cold_k]
        else:
            parts = [dequant_keys(b["codes"], b["scale"], b["mean"], b["out_idx"], b["out_val"],
                                  self.key_mode)
                     for b in self.cold_k]
        if self.hot_k:
            parts.append(np.stack(self.hot_k, axis=1).astype(F32))
        if not parts:
            return np.zeros((self.n_heads, 0, self.head_dim), dtype=F32)
        return np.concatenate(parts, axis=1)

    def values(self) -> np.ndarray:
        parts = [dequant_values(b["codes"], b["norms"], self.centroids, self.pi)
                 for b in self.cold_v]
        if self.hot_v:
            parts.append(np.stack(self.hot_v, axis=1).astype(F32))
        if not parts:
            return np.zeros((self.n_heads, 0, self.head_dim), dtype=F32)
        return np.concatenate(parts, axis=1)

    def attend(self, q) -> np.ndarray:
        """Dequantise-then-attend output (Hq, D): the parity oracle for decode."""
        return attention(q, self.keys(), self.values())

    def memory_stats(self):
        """Byte accounting of core.py:1267-1296 (reference container sizes)."""
        h, d = self.n_heads, self.head_dim
        cold = 0
        for kb, vb, n in zip(self.cold_k, self.cold_v, self.cold_lengths):
            if self.key_mode == "polar":  # two CompressedKV containers
                cold += 2 * ((h * n * d * self.value_bits + 7) // 8 + 4 * h * n)
                continue
            # per-channel float32 scalars: scale + mean (symmetric NF4 stores no mean)
            n_mean = (0 if self.k_bias is not None else
                      d if self.rope_theta is None else int(self._dc_mask(n).sum()))
            cold += (h * n * d * self.key_bits // 8 + 4 * h * d
                     + (0 if self.key_mode == "nf4" else 4 * h * n_mean))
            if kb["out_idx"] is not None:
                cold += kb["out_idx"].size * 6
            cold += (h * n * d * self.value_bits + 7) // 8 + 4 * h * n
        hot = sum(k.nbytes + v.nbytes for k, v in zip(self.hot_k, self.hot_v))
        total = cold + hot
        unc = self.length * h * d * 4 * 2
        return {
            "cold_bytes": float(cold),
            "hot_bytes": float(hot),
            "total_bytes": float(total),
            "uncompressed_equivalent_bytes": float(unc),
            "effective_ratio": float(unc) / max(total, 1),
        }

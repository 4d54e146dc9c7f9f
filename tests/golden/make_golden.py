"""Generate the golden fixtures in this directory by running the REFERENCE itself.

Usage (only where the reference is available)::

    TQ_REF_PATH=/path/to/turboquant-pro python tests/golden/make_golden.py

Without ``TQ_REF_PATH`` the copy that ``make -C oracle ref`` puts under ``oracle/_ref`` is used.

The reference is imported, never copied: this script feeds it seeded inputs through
its public API (``PerChannelKV.compress``, ``TurboQuantKV.compress``,
``TurboQuantKVCache.append/get_keys/get_values/fused_decode``) and stores inputs and
outputs as ``.npz`` files.  The tests compare the CPU oracle and the CUDA library with
these files, so they run on machines that do not have the reference.
"""

from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("TQ_REF_PATH") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "oracle", "_ref")
sys.path.insert(0, REF)

from turboquant_pro.core import TurboQuantKV, TurboQuantKVCache  # noqa: E402
from turboquant_pro.per_channel_kv import PerChannelKV  # noqa: E402

D = 128


def _scaled(rng, shape_hd, n_tokens, gain_channels=3):
    h, d = shape_hd
    sk = np.exp(rng.normal(0.0, 0.5, size=(h, d)))
    sv = np.exp(rng.normal(0.0, 0.5, size=(h, d)))
    for i in range(h):
        sk[i, rng.choice(d, size=gain_channels, replace=False)] *= 20.0
    k = rng.standard_normal((n_tokens, h, d)) * sk
    v = rng.standard_normal((n_tokens, h, d)) * sv
    return k.astype(np.float32), v.astype(np.float32)


def _attend(q, k, v):
    """fp32 softmax(qK^T/sqrt(D))V with query head i reading KV head i // G."""
    g = q.shape[0] // k.shape[0]
    kk = np.repeat(k, g, axis=0)
    vv = np.repeat(v, g, axis=0)
    sc = np.einsum("hd,hsd->hs", q, kk) / np.float32(np.sqrt(q.shape[1]))
    sc = sc - sc.max(axis=-1, keepdims=True)
    e = np.exp(sc)
    p = e / e.sum(axis=-1, keepdims=True)
    return np.einsum("hs,hsd->hd", p, vv).astype(np.float32)


def block_case(name, seed, h, s, value_bits, round_to=None, dtype=np.float32):
    """One (1, H, S, D) block through both stateless encoders."""
    rng = np.random.default_rng(seed)
    k, v = _scaled(rng, (h, D), s)
    if round_to is not None:  # coarse grid -> many magnitude ties and exact mid-points
        k = (np.round(k / round_to) * round_to).astype(np.float32)
        v = (np.round(v / round_to) * round_to).astype(np.float32)
    k = k.astype(dtype)
    v = v.astype(dtype)
    kb = np.ascontiguousarray(np.moveaxis(k, 0, 1))[None]  # (1,H,S,D)
    vb = np.ascontiguousarray(np.moveaxis(v, 0, 1))[None]
    kq = PerChannelKV(head_dim=D, n_heads=h, bits=4, nf4_asym=True, outlier_frac=0.02)
    tq = TurboQuantKV(head_dim=D, n_heads=h, bits=value_bits, key_bits=4,
                      value_bits=value_bits, use_gpu=False, seed=seed)
    ck = kq.compress(kb, packed=True)
    cv = tq.compress(vb, packed=True, kind="value")
    np.savez_compressed(
        os.path.join(HERE, name),
        k=k, v=v, seed=seed, value_bits=value_bits,
        key_indices=ck.indices, nf4_scale=ck.nf4_scale, nf4_mean=ck.nf4_mean,
        outlier_idx=ck.outlier_idx, outlier_val=ck.outlier_val,
        value_indices=cv.indices, value_norms=cv.norms,
        pi=tq._Pi, pi_t=tq._Pi_T,
        centroids=tq._codebooks[value_bits][0], boundaries=tq._codebooks[value_bits][1],
        key_dequant=kq.decompress(ck)[0], value_dequant=tq.decompress(cv)[0],
    )


_KEY_MODE_FLAGS = {"nf4_asym": {"key_nf4_asym": True}, "nf4": {"key_nf4": True}, "uniform": {}}


def _key_fields(ck):
    """(scale, mean) of a key container as (1, H, D) arrays whatever its mode: the NF4
    family keeps them in nf4_scale / nf4_mean (no mean when symmetric), the uniform grid in
    scale / zero."""
    if ck.nf4_scale is not None:
        mean = ck.nf4_mean if ck.nf4_mean is not None else np.zeros_like(ck.nf4_scale)
        return ck.nf4_scale, mean
    return ck.scale[:, :, 0, :], ck.zero[:, :, 0, :]


def key_block_case(name, seed, h, s, mode, frac, round_to=None, dtype=np.float32):
    """One (1, H, S, D) key block through the per-channel encoder in another grid mode."""
    rng = np.random.default_rng(seed)
    k, _ = _scaled(rng, (h, D), s)
    k = k + rng.standard_normal((1, h, D)).astype(np.float32)  # per-channel offsets
    if round_to is not None:
        k = (np.round(k / round_to) * round_to).astype(np.float32)
    k = k.astype(dtype)
    kb = np.ascontiguousarray(np.moveaxis(k, 0, 1))[None]
    flags = {"nf4_asym": {"nf4_asym": True}, "nf4": {"nf4": True}, "uniform": {}}[mode]
    kq = PerChannelKV(head_dim=D, n_heads=h, bits=4, outlier_frac=frac, **flags)
    ck = kq.compress(kb, packed=True)
    scale, mean = _key_fields(ck)
    out = dict(k=k, seed=seed, mode=mode, frac=frac, key_indices=ck.indices, key_scale=scale,
               key_mean=mean, key_dequant=kq.decompress(ck)[0])
    if ck.outlier_idx is not None:
        out["outlier_idx"] = ck.outlier_idx
        out["outlier_val"] = ck.outlier_val
    np.savez_compressed(os.path.join(HERE, name), **out)


def cache_case(name, seed, h, n_tokens, hot_window, value_bits, n_q_heads, dtype=np.float32,
               with_fused=False, key_mode="nf4_asym", sparse_theta=None, bias_theta=None):
    """A cache filled token by token; stores every cold container and the
    dequantise-then-attend output (plus ``fused_decode`` where the reference has it)."""
    rng = np.random.default_rng(seed)
    k, v = _scaled(rng, (h, D), n_tokens)
    k = k.astype(dtype)
    v = v.astype(dtype)
    q = rng.standard_normal((n_q_heads, D)).astype(np.float32)
    k_bias = None
    if bias_theta is not None:  # a key-projection bias, and keys that carry it
        k_bias = (3.0 * rng.standard_normal((h, D))).astype(np.float32)
        k = (k.astype(np.float32) + k_bias[None]).astype(dtype)
    cache = TurboQuantKVCache(
        head_dim=D, n_heads=h, bits=value_bits, key_bits=4, value_bits=value_bits,
        hot_window=hot_window, use_gpu=False, seed=seed, key_outlier_frac=0.02,
        key_zero_point="bias" if bias_theta else ("sparse" if sparse_theta else "calibrated"),
        key_rope_theta=bias_theta or sparse_theta, key_k_bias=k_bias,
        **_KEY_MODE_FLAGS[key_mode],
    )
    for t in range(n_tokens):
        cache.append(k[t], v[t])
    keys = cache.get_keys(0, cache.length)[0]
    vals = cache.get_values(0, cache.length)[0]
    out = {
        "k": k, "v": v, "q": q, "seed": seed, "hot_window": hot_window,
        "value_bits": value_bits, "n_blocks": len(cache._cold_keys),
        "cold_lengths": np.asarray(cache._cold_lengths, dtype=np.int32),
        "length": cache.length, "hot_length": cache.hot_length,
        "attn": _attend(q, keys, vals),
        "keys_head0": keys[0], "values_head0": vals[0],
        "pi": cache._tq._Pi,
    }
    st = cache.memory_stats()
    out["memory_stats"] = np.array([st["cold_bytes"], st["hot_bytes"], st["total_bytes"],
                                    st["uncompressed_equivalent_bytes"]], dtype=np.float64)
    for i, (ck, cv) in enumerate(zip(cache._cold_keys, cache._cold_values)):
        out[f"b{i}_key_indices"] = ck.indices
        if bias_theta is not None:  # nothing stored: the zero-point is recomputed from k_bias
            out[f"b{i}_nf4_scale"] = ck.nf4_scale
            out[f"b{i}_nf4_mean"] = cache._kq.rope_averaged_bias(
                k_bias, bias_theta, D, ck.position_start, cache._cold_lengths[i])[None]
            out["k_bias"] = k_bias
        else:
            out[f"b{i}_nf4_scale"], out[f"b{i}_nf4_mean"] = _key_fields(ck)
        if sparse_theta is not None:  # compact (1, H, n_dc) means -> full width, zeros elsewhere
            dc = PerChannelKV.dc_channel_mask(sparse_theta, D, cache._cold_lengths[i])
            full = np.zeros_like(ck.nf4_scale)
            full[:, :, dc] = ck.nf4_mean
            out[f"b{i}_nf4_mean"] = full
            out["dc_mask"] = dc
        out[f"b{i}_outlier_idx"] = ck.outlier_idx
        out[f"b{i}_outlier_val"] = ck.outlier_val
        out[f"b{i}_value_indices"] = cv.indices
        out[f"b{i}_value_norms"] = cv.norms
    if with_fused:
        assert n_q_heads == h
        out["fused"] = np.asarray(cache.fused_decode(q), dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, name), **out)


def polar_keys_case(name, seed, h, n_tokens, hot_window, bits, dtype=np.float32):
    """The legacy key format (``per_channel_keys=False``): keys through the value quantiser.
    Stores every cold container (both are ``CompressedKV``), the dequantised tensors, the
    dequantise-then-attend output and ``fused_decode``."""
    rng = np.random.default_rng(seed)
    k, v = _scaled(rng, (h, D), n_tokens)
    k = k.astype(dtype)
    v = v.astype(dtype)
    q = rng.standard_normal((h, D)).astype(np.float32)
    cache = TurboQuantKVCache(head_dim=D, n_heads=h, bits=bits, hot_window=hot_window,
                              use_gpu=False, seed=seed, per_channel_keys=False)
    for t in range(n_tokens):
        cache.append(k[t], v[t])
    keys = cache.get_keys(0, cache.length)[0]
    vals = cache.get_values(0, cache.length)[0]
    st = cache.memory_stats()
    out = {
        "k": k, "v": v, "q": q, "seed": seed, "hot_window": hot_window, "bits": bits,
        "n_blocks": len(cache._cold_keys),
        "cold_lengths": np.asarray(cache._cold_lengths, dtype=np.int32),
        "length": cache.length, "hot_length": cache.hot_length,
        "attn": _attend(q, keys, vals), "keys_head0": keys[0], "values_head0": vals[0],
        "pi": cache._tq._Pi,
        "fused": np.asarray(cache.fused_decode(q), dtype=np.float32),
        "memory_stats": np.array([st["cold_bytes"], st["hot_bytes"], st["total_bytes"],
                                  st["uncompressed_equivalent_bytes"]], dtype=np.float64),
    }
    for i, (ck, cv) in enumerate(zip(cache._cold_keys, cache._cold_values)):
        out[f"b{i}_key_indices"] = ck.indices
        out[f"b{i}_key_norms"] = ck.norms
        out[f"b{i}_value_indices"] = cv.indices
        out[f"b{i}_value_norms"] = cv.norms
    np.savez_compressed(os.path.join(HERE, name), **out)


def pack_known_answer():
    """The reference's own known-answer 3-bit packing vector (tests/test_core.py:228-258)
    and the same codes through the other widths and through the key packer."""
    from turboquant_pro.per_channel_kv import _pack_indices

    tq = TurboQuantKV(head_dim=64, bits=3, use_gpu=False, seed=0)
    codes8 = np.arange(8, dtype=np.uint8)
    codes16 = np.arange(16, dtype=np.uint8)
    np.savez_compressed(
        os.path.join(HERE, "pack_known.npz"),
        codes8=codes8, codes16=codes16,
        v3=tq._pack_bits(codes8, bits=3),
        v4=tq._pack_bits(codes16, bits=4),
        v2=tq._pack_bits(codes8 & 3, bits=2),
        k4=_pack_indices(codes16, 4),
    )


def main():
    block_case("block_k4v3.npz", seed=11, h=2, s=256, value_bits=3)
    block_case("block_k4v4_f16.npz", seed=12, h=2, s=256, value_bits=4, dtype=np.float16)
    block_case("block_ties.npz", seed=13, h=2, s=256, value_bits=3, round_to=0.25)
    block_case("block_short.npz", seed=14, h=3, s=8, value_bits=4)
    cache_case("cache_w16.npz", seed=21, h=2, n_tokens=83, hot_window=16, value_bits=4,
               n_q_heads=2, with_fused=True)
    cache_case("cache_w512_gqa.npz", seed=22, h=2, n_tokens=800, hot_window=512, value_bits=3,
               n_q_heads=8, dtype=np.float16)
    cache_case("cache_w7.npz", seed=23, h=1, n_tokens=30, hot_window=7, value_bits=3,
               n_q_heads=4)
    pack_known_answer()
    other_key_grids()
    blob_case()
    polar_keys_case("cache_polar_keys_v3.npz", seed=41, h=2, n_tokens=900, hot_window=512, bits=3,
                    dtype=np.float16)
    polar_keys_case("cache_polar_keys_v4_w16.npz", seed=42, h=2, n_tokens=70, hot_window=16,
                    bits=4)
    print("golden fixtures written to", HERE)


def blob_case():
    """A cold block of a small cache written by the reference's own blob writer
    (connectors/vllm_v1.py:113-137), with the tokens that produced it."""
    from turboquant_pro.connectors import vllm_v1 as conn

    rng = np.random.default_rng(41)
    k, v = _scaled(rng, (2, D), 20)
    cache = TurboQuantKVCache(head_dim=D, n_heads=2, bits=3, key_bits=4, value_bits=3,
                              hot_window=16, use_gpu=False, seed=41, key_nf4_asym=True,
                              key_outlier_frac=0.02)
    for t in range(20):
        cache.append(k[t], v[t])
    ck, cv = cache._cold_keys[0], cache._cold_values[0]
    rec = conn._BlockRecord(key_payload=ck, value_payload=cv, shape=tuple(ck.shape),
                            dtype="float32", num_tokens=ck.shape[2], head_dim=D, n_heads=2)
    blob = conn._rec_to_blob(rec)
    np.savez_compressed(os.path.join(HERE, "blob_ref.npz"), k=k, v=v, pi=cache._tq._Pi,
                        blob=np.frombuffer(blob, dtype=np.uint8), hot_window=16, seed=41)


def other_key_grids():
    """Blocks and caches in the other per-channel key grids that have a fused form."""
    key_block_case("keys_uniform.npz", seed=31, h=2, s=256, mode="uniform", frac=0.02)
    key_block_case("keys_uniform_ties.npz", seed=32, h=2, s=256, mode="uniform", frac=0.0,
                   round_to=0.25, dtype=np.float16)
    key_block_case("keys_nf4.npz", seed=33, h=2, s=256, mode="nf4", frac=0.02)
    cache_case("cache_uniform.npz", seed=34, h=2, n_tokens=700, hot_window=512, value_bits=4,
               n_q_heads=2, key_mode="uniform")
    cache_case("cache_nf4_gqa.npz", seed=35, h=2, n_tokens=700, hot_window=512, value_bits=3,
               n_q_heads=8, dtype=np.float16, key_mode="nf4")
    cache_case("cache_sparse_zp.npz", seed=36, h=2, n_tokens=700, hot_window=512, value_bits=3,
               n_q_heads=4, dtype=np.float16, sparse_theta=10000.0)
    cache_case("cache_bias_zp.npz", seed=37, h=2, n_tokens=1100, hot_window=512, value_bits=3,
               n_q_heads=4, dtype=np.float16, bias_theta=10000.0)


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] in ("other_key_grids", "blob_case"):
        globals()[sys.argv[1]]()
    else:
        main()

"""One compressed KV block as a self-describing byte string (codec ``tqp-kv-npz/1``).

The reference's vLLM connector stores a (request, layer) block as one ``.npz`` archive: the
arrays of the key and value containers under ``k.*`` / ``v.*`` plus a JSON header with the
scalars (``connectors/vllm_v1.py:67``, ``:113-196``).  This module writes and reads that
layout for blocks exported from the GPU context (``KVContext.export_block``), so blocks
produced here can be consumed by the reference and the other way round.  No pickle is
involved in either direction; the reader refuses what it does not know instead of guessing
(codec string, size limits, dtype whitelist), as the reference's reader does.

``block_from_parsed`` turns a parsed blob back into the arrays ``KVContext.import_block``
takes, so a stored block goes into device pages without passing through dense tensors.
"""

from __future__ import annotations

import io
import json

import numpy as np

CODEC = "tqp-kv-npz/1"
_OK_DTYPES = {"uint8", "int8", "int16", "int32", "int64", "float16", "float32", "float64", "bool"}

__all__ = ["CODEC", "block_to_blob", "blob_to_block", "block_from_parsed"]


def _tuple(v):
    return {"__tuple__": [int(x) for x in v]}


def _dtype(name):
    return {"__dtype__": str(np.dtype(name))}


def block_to_blob(block: dict, *, key_mode: str = "nf4_asym", zero_point: str = "calibrated",
                  mean_mask=None, rope_theta: float | None = None, position_start: int = 0,
                  dtype: str = "float32") -> bytes:
    """Serialise one exported cold block.

    ``block`` is the dict of ``KVContext.export_block`` (reference container layout:
    bit-reversed packed key nibbles, LSB-first packed value codes, ``(1, H, D)`` key scale
    and mean, flat int32 outlier indices with float16 values, ``(1, H, S)`` value norms).
    ``key_mode`` / ``zero_point`` say how the key scalars are to be named and which of them
    the format stores: uniform keys as ``scale`` / ``zero`` ``(1, H, 1, D)``; symmetric NF4
    without a mean; the ``sparse`` zero-point with the means of the ``mean_mask`` channels
    only; the ``bias`` zero-point with none (``rope_theta`` and ``position_start`` let the
    reader recompute it).  ``dtype`` is the element type the tokens had.
    """
    shape = tuple(int(x) for x in block["shape"])
    k_arr: dict[str, np.ndarray] = {"indices": np.ascontiguousarray(block["key_indices"])}
    k_sc = {"scale": None, "zero": None, "bits": int(block["key_bits"]), "shape": _tuple(shape),
            "packed": True, "levels": None, "original_dtype": _dtype("float32"),
            "zp_mode": "calibrated", "rope_theta": None, "position_start": int(position_start)}
    scale, mean = np.asarray(block["nf4_scale"]), np.asarray(block["nf4_mean"])
    if key_mode == "uniform":
        del k_sc["scale"], k_sc["zero"]
        k_arr["scale"] = np.ascontiguousarray(scale[:, :, None, :])
        k_arr["zero"] = np.ascontiguousarray(mean[:, :, None, :])
        k_sc["nf4_scale"] = k_sc["nf4_mean"] = None
    else:
        k_arr["nf4_scale"] = np.ascontiguousarray(scale)
        if key_mode == "nf4":
            k_sc["nf4_mean"] = None
        elif zero_point == "sparse":
            if mean_mask is None or rope_theta is None:
                raise ValueError("the sparse zero-point needs mean_mask and rope_theta")
            k_arr["nf4_mean"] = np.ascontiguousarray(mean[:, :, np.asarray(mean_mask, bool)])
            k_sc["zp_mode"], k_sc["rope_theta"] = "sparse", float(rope_theta)
        elif zero_point == "bias":
            if rope_theta is None:
                raise ValueError("the bias zero-point needs rope_theta")
            k_sc["nf4_mean"] = None
            k_sc["zp_mode"], k_sc["rope_theta"] = "bias", float(rope_theta)
        else:
            k_arr["nf4_mean"] = np.ascontiguousarray(mean)
    if block.get("outlier_idx") is not None:
        k_arr["outlier_idx"] = np.ascontiguousarray(block["outlier_idx"], dtype=np.int32)
        k_arr["outlier_val"] = np.ascontiguousarray(block["outlier_val"]).view(np.float16)
    else:
        k_sc["outlier_idx"] = k_sc["outlier_val"] = None
    v_arr = {"indices": np.ascontiguousarray(block["value_indices"]),
             "norms": np.ascontiguousarray(block["value_norms"], dtype=np.float32)}
    v_sc = {"bits": int(block["value_bits"]), "original_dtype": _dtype("float32"),
            "packed": True, "n_values": int(np.prod(shape)), "shape": _tuple(shape)}
    header = {"codec": CODEC, "shape": list(shape), "dtype": str(dtype),
              "num_tokens": shape[2], "head_dim": shape[3], "n_heads": shape[1],
              "key_scalars": k_sc, "value_scalars": v_sc}
    buf = io.BytesIO()
    np.savez(buf, __header__=np.frombuffer(json.dumps(header).encode(), dtype=np.uint8),
             **{f"k.{n}": a for n, a in k_arr.items()}, **{f"v.{n}": a for n, a in v_arr.items()})
    return buf.getvalue()


def _scalars(d: dict) -> dict:
    out = {}
    for name, v in d.items():
        if isinstance(v, dict) and "__dtype__" in v:
            out[name] = np.dtype(v["__dtype__"])
        elif isinstance(v, dict) and "__tuple__" in v:
            out[name] = tuple(v["__tuple__"])
        else:
            out[name] = v
    return out


def blob_to_block(blob: bytes, max_bytes: int = 1 << 30) -> dict:
    """Parse one blob: ``{"header": {...}, "key": {field: array or scalar}, "value": {...}}``.

    Raises ``ValueError`` for a blob or a decompressed payload above ``max_bytes``, for a
    codec string other than ``tqp-kv-npz/1`` and for array dtypes outside the numeric
    whitelist (object arrays cannot be loaded at all: ``allow_pickle=False``).
    """
    if len(blob) > max_bytes:
        raise ValueError(f"blob exceeds max_bytes ({len(blob)} > {max_bytes})")
    with np.load(io.BytesIO(blob), allow_pickle=False) as z:
        if "__header__" not in z.files:
            raise ValueError("not a KV block blob: no header")
        header = json.loads(bytes(z["__header__"]).decode())
        if header.get("codec") != CODEC:
            raise ValueError(f"unknown record codec {header.get('codec')!r}; this reader "
                             f"handles {CODEC!r} only")
        total = 0
        key, value = {}, {}
        for name in z.files:
            if name == "__header__":
                continue
            a = z[name]
            if str(a.dtype) not in _OK_DTYPES:
                raise ValueError(f"dtype {a.dtype} of {name} is not allowed")
            total += a.nbytes
            if total > max_bytes:
                raise ValueError("decompressed size exceeds max_bytes")
            if name.startswith("k."):
                key[name[2:]] = a
            elif name.startswith("v."):
                value[name[2:]] = a
            else:
                raise ValueError(f"unexpected member {name!r}")
    key.update(_scalars(header["key_scalars"]))
    value.update(_scalars(header["value_scalars"]))
    meta = {k: header[k] for k in ("codec", "shape", "dtype", "num_tokens", "head_dim", "n_heads")}
    meta["shape"] = tuple(meta["shape"])
    return {"header": meta, "key": key, "value": value}


def block_from_parsed(parsed: dict, *, key_mode: str = "nf4_asym", mean_mask=None,
                      bias_means=None, geom=None) -> dict:
    """The arrays of ``KVContext.import_block`` from the result of :func:`blob_to_block`.

    The key scalars are brought back to one full ``(1, H, D)`` scale and zero-point: the
    uniform grid's ``scale`` / ``zero``; symmetric NF4 with zeros; the ``sparse`` zero-point
    scattered to the ``mean_mask`` channels; the ``bias`` zero-point from ``bias_means``
    ``(H, D)`` (the blob stores none: the reader recomputes it from the model's k-bias, the
    block's first position and ``rope_theta``).  ``geom`` ``(H, S, D, value_bits)``, when given,
    is checked against the blob's header.
    """
    key, value, meta = parsed["key"], parsed["value"], parsed["header"]
    _, h, s, d = meta["shape"]
    if geom is not None and (h, s, d, int(value["bits"])) != tuple(geom):
        raise ValueError(f"blob holds a block of (H, S, D, value_bits) = "
                         f"{(h, s, d, int(value['bits']))}, the context expects {tuple(geom)}")
    if int(key["bits"]) != 4 or not key.get("packed", True) or not value.get("packed", True):
        raise ValueError("only packed blocks with 4-bit keys can be imported")
    uniform = "scale" in key and key.get("nf4_scale") is None
    if uniform != (key_mode == "uniform"):
        raise ValueError("the blob's key grid differs from the context's key_mode")
    if uniform:
        scale = np.asarray(key["scale"], np.float32).reshape(1, h, d)
        mean = np.asarray(key["zero"], np.float32).reshape(1, h, d)
    else:
        scale = np.asarray(key["nf4_scale"], np.float32).reshape(1, h, d)
        zp = key.get("zp_mode", "calibrated")
        stored = key.get("nf4_mean")
        if key_mode == "nf4":
            if stored is not None:
                raise ValueError("the blob holds key means, the context is symmetric NF4")
            mean = np.zeros((1, h, d), np.float32)
        elif zp == "sparse":
            if mean_mask is None:
                raise ValueError("a sparse zero-point needs the context's channel mask")
            mask = np.asarray(mean_mask, bool)
            stored = np.asarray(stored, np.float32)
            if stored.shape[-1] != int(mask.sum()):
                raise ValueError("the blob's sparse means do not match the channel mask")
            mean = np.zeros((1, h, d), np.float32)
            mean[:, :, mask] = stored.reshape(1, h, -1)
        elif zp == "bias":
            if bias_means is None:
                raise ValueError("a bias zero-point stores no means: pass bias_means")
            mean = np.asarray(bias_means, np.float32).reshape(1, h, d)
        else:
            if stored is None:
                raise ValueError("the blob holds no key means, the context expects them")
            mean = np.asarray(stored, np.float32).reshape(1, h, d)
    oidx = key.get("outlier_idx")
    return {
        "key_indices": np.asarray(key["indices"], np.uint8), "nf4_scale": scale, "nf4_mean": mean,
        "outlier_idx": None if oidx is None else np.asarray(oidx, np.int32),
        "outlier_val": None if oidx is None else np.asarray(key["outlier_val"]),
        "value_indices": np.asarray(value["indices"], np.uint8),
        "value_norms": np.asarray(value["norms"], np.float32),
        "shape": (1, h, s, d), "key_bits": 4, "value_bits": int(value["bits"]),
    }

"""The KV block wire format (codec tqp-kv-npz/1): the reader parses a blob written by the
reference's own writer, the writer reproduces it from the same containers, and the reader's
refusals (codec, size, member names) hold.  CPU only; the GPU leg is in test_gpu_parity.py."""

from __future__ import annotations

import io
import json

import numpy as np
import pytest

from conftest import load_golden
from oracle import tq_oracle as orc
from turboquant_pro_b200.kv_blob import CODEC, blob_to_block, block_to_blob


def _oracle_block(g):
    """The first cold block of the fixture's cache, as an export_block-style dict."""
    k, v = g["k"], g["v"]
    c = orc.OracleCache(128, 2, 4, 3, int(g["hot_window"]), 0.02, int(g["seed"]))
    c.pi, c.pi_t = g["pi"], np.ascontiguousarray(g["pi"].T)
    for t in range(k.shape[0]):
        c.append(k[t], v[t])
    kb, vb = c.cold_k[0], c.cold_v[0]
    s = c.cold_lengths[0]
    return {
        "key_indices": orc.pack_key_codes(kb["codes"]), "nf4_scale": kb["scale"][None],
        "nf4_mean": kb["mean"][None], "outlier_idx": kb["out_idx"], "outlier_val": kb["out_val"],
        "value_indices": orc.pack_value_codes(vb["codes"], 3), "value_norms": vb["norms"][None],
        "shape": (1, 2, s, 128), "key_bits": 4, "value_bits": 3,
    }


def test_reads_reference_blob_and_writes_the_same_members():
    g = load_golden("blob_ref.npz")
    ref = blob_to_block(g["blob"].tobytes())
    assert ref["header"]["codec"] == CODEC and ref["header"]["shape"] == (1, 2, 8, 128)
    assert ref["key"]["zp_mode"] == "calibrated" and ref["key"]["bits"] == 4
    assert ref["value"]["bits"] == 3 and ref["value"]["n_values"] == 2 * 8 * 128
    mine = blob_to_block(block_to_blob(_oracle_block(g)))
    assert mine["header"] == ref["header"]
    for part in ("key", "value"):
        assert sorted(mine[part]) == sorted(ref[part])
        for name, want in ref[part].items():
            got = mine[part][name]
            if isinstance(want, np.ndarray):
                assert got.dtype == want.dtype and np.array_equal(got, want), name
            else:
                assert got == want, name


@pytest.mark.parametrize("mode,zp", [("uniform", "calibrated"), ("nf4", "calibrated"),
                                     ("nf4_asym", "sparse"), ("nf4_asym", "bias")])
def test_other_key_formats_name_their_scalars_like_the_reference(mode, zp):
    g = load_golden("blob_ref.npz")
    blk = _oracle_block(g)
    mask = np.arange(128) % 2 == 0
    out = blob_to_block(block_to_blob(blk, key_mode=mode, zero_point=zp, mean_mask=mask,
                                      rope_theta=1e4, position_start=24))
    key = out["key"]
    if mode == "uniform":
        assert key["scale"].shape == (1, 2, 1, 128) and key["zero"].shape == (1, 2, 1, 128)
        assert key["nf4_scale"] is None
    elif mode == "nf4":
        assert key["nf4_mean"] is None and key["nf4_scale"].shape == (1, 2, 128)
    elif zp == "sparse":
        assert key["nf4_mean"].shape == (1, 2, 64) and key["zp_mode"] == "sparse"
        assert key["rope_theta"] == 1e4
    else:
        assert key["nf4_mean"] is None and key["zp_mode"] == "bias"
        assert key["position_start"] == 24


def test_reader_refusals():
    g = load_golden("blob_ref.npz")
    blob = g["blob"].tobytes()
    with pytest.raises(ValueError, match="max_bytes"):
        blob_to_block(blob, max_bytes=100)
    z = np.load(io.BytesIO(blob), allow_pickle=False)
    members = {n: z[n] for n in z.files}
    bomb = dict(members)
    bomb["k.indices"] = np.zeros(4 << 20, np.uint8)  # 4 MB that deflate to a few KB
    buf = io.BytesIO()
    np.savez_compressed(buf, **bomb)
    assert len(buf.getvalue()) < 100_000
    with pytest.raises(ValueError, match="decompressed size"):
        blob_to_block(buf.getvalue(), max_bytes=100_000)
    hdr = json.loads(bytes(members["__header__"]).decode())
    hdr["codec"] = "tqp-kv-npz/2"
    members["__header__"] = np.frombuffer(json.dumps(hdr).encode(), dtype=np.uint8)
    buf = io.BytesIO()
    np.savez(buf, **members)
    with pytest.raises(ValueError, match="unknown record codec"):
        blob_to_block(buf.getvalue())
    hdr["codec"] = CODEC
    members["__header__"] = np.frombuffer(json.dumps(hdr).encode(), dtype=np.uint8)
    members["x.extra"] = np.zeros(3, np.uint8)
    buf = io.BytesIO()
    np.savez(buf, **members)
    with pytest.raises(ValueError, match="unexpected member"):
        blob_to_block(buf.getvalue())


def test_parsed_blob_gives_back_the_container_arrays():
    """blob -> arrays for KVContext.import_block: the reference's blob yields exactly the
    oracle's containers; the other zero-point forms are brought back to full scale / mean."""
    from turboquant_pro_b200.kv_blob import block_from_parsed

    g = load_golden("blob_ref.npz")
    want = _oracle_block(g)
    got = block_from_parsed(blob_to_block(g["blob"].tobytes()), geom=(2, 8, 128, 3))
    for name in ("key_indices", "nf4_scale", "nf4_mean", "outlier_idx", "value_indices",
                 "value_norms"):
        assert np.array_equal(np.asarray(got[name]).reshape(-1),
                              np.asarray(want[name]).reshape(-1)), name
    assert np.array_equal(np.asarray(got["outlier_val"]).view(np.uint16),
                          np.asarray(want["outlier_val"]).view(np.uint16))
    with pytest.raises(ValueError):
        block_from_parsed(blob_to_block(g["blob"].tobytes()), geom=(2, 8, 128, 4))
    with pytest.raises(ValueError):  # an NF4 blob into a context with the uniform grid
        block_from_parsed(blob_to_block(g["blob"].tobytes()), key_mode="uniform")
    mask = np.arange(128) % 2 == 0
    sparse = blob_to_block(block_to_blob(want, zero_point="sparse", mean_mask=mask, rope_theta=1e4))
    back = block_from_parsed(sparse, mean_mask=mask)
    assert np.array_equal(back["nf4_mean"][..., mask], want["nf4_mean"][..., mask])
    assert not back["nf4_mean"][..., ~mask].any()
    with pytest.raises(ValueError):
        block_from_parsed(sparse)
    bias = blob_to_block(block_to_blob(want, zero_point="bias", rope_theta=1e4))
    with pytest.raises(ValueError):
        block_from_parsed(bias)
    given = np.full((2, 128), 0.25, np.float32)
    assert np.array_equal(block_from_parsed(bias, bias_means=given)["nf4_mean"][0], given)
    uni = blob_to_block(block_to_blob(want, key_mode="uniform"))
    back = block_from_parsed(uni, key_mode="uniform")
    assert np.array_equal(back["nf4_scale"], want["nf4_scale"])
    assert np.array_equal(back["nf4_mean"], want["nf4_mean"])
    sym = blob_to_block(block_to_blob(want, key_mode="nf4"))
    assert not block_from_parsed(sym, key_mode="nf4")["nf4_mean"].any()

"""Pins the C restatement (oracle/tq_oracle.c) against the reference fixtures."""

from __future__ import annotations

import numpy as np
import pytest

from oracle import c_oracle as co
from oracle import tq_oracle as orc

from conftest import load_golden

BLOCKS = ["block_k4v3.npz", "block_k4v4_f16.npz", "block_ties.npz", "block_short.npz"]


def _hsd(x):
    return np.ascontiguousarray(np.moveaxis(np.asarray(x, dtype=np.float32), 0, 1))


@pytest.mark.parametrize("name", BLOCKS)
def test_c_key_encoder(name):
    g = load_golden(name)
    x = _hsd(g["k"])
    enc = co.encode_keys(x, orc.outlier_count(x.shape[1], 0.02))
    assert np.array_equal(orc.pack_key_codes(enc["codes"]), g["key_indices"])
    assert np.array_equal(enc["scale"], g["nf4_scale"][0])
    assert np.array_equal(enc["mean"], g["nf4_mean"][0])
    assert np.array_equal(enc["out_idx"], g["outlier_idx"])
    assert np.array_equal(enc["out_val"].view(np.uint16), g["outlier_val"].view(np.uint16))
    deq = co.dequant_keys(enc["codes"], enc["scale"], enc["mean"], enc["out_idx"], enc["out_val"])
    assert np.array_equal(deq, g["key_dequant"])


@pytest.mark.parametrize("name", BLOCKS)
def test_c_value_encoder(name):
    g = load_golden(name)
    bits = int(g["value_bits"])
    enc = co.encode_values(_hsd(g["v"]), g["pi_t"], g["boundaries"])
    assert np.array_equal(enc["norms"], g["value_norms"][0])
    assert np.array_equal(orc.pack_value_codes(enc["codes"], bits), g["value_indices"])
    deq = co.dequant_values(enc["codes"], enc["norms"], g["centroids"], g["pi"])
    assert np.array_equal(deq, g["value_dequant"])


def test_c_attention_matches_numpy():
    rng = np.random.default_rng(3)
    q = rng.standard_normal((8, 128)).astype(np.float32)
    k = rng.standard_normal((2, 300, 128)).astype(np.float32)
    v = rng.standard_normal((2, 300, 128)).astype(np.float32)
    assert np.allclose(co.attention(q, k, v), orc.attention(q, k, v), rtol=1e-5, atol=1e-6)
    assert co.num_threads() >= 1

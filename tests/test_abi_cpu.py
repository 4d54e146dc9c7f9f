"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header
declares, and its host-only entry points (geometry, sizes) behave.  No kernel runs here."""

from __future__ import annotations

import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge

    ge._load_build_module().build()
    from turboquant_pro_b200 import _lib

    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tqb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tq_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    from turboquant_pro_b200 import _lib

    names = _declared_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/tqb200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert lib.tq_version() == 100


def _geom(**kw):
    from turboquant_pro_b200._lib import TqGeom

    g = TqGeom()
    vals = dict(n_layers=1, n_seqs=1, n_kv_heads=8, n_q_heads=32, head_dim=128, key_bits=4,
                value_bits=3, hot_window=512, kv_dtype=1, max_tokens_per_seq=8192,
                outlier_frac=0.02)
    vals.update(kw)
    for k, v in vals.items():
        setattr(g, k, v)
    return g


def test_geometry_matches_reference_block_rule(lib):
    from oracle import tq_oracle as orc

    for w in (2, 7, 16, 64, 511, 512):
        g = _geom(hot_window=w, max_tokens_per_seq=5000)
        assert lib.tq_geom_finish(C.byref(g)) == 0
        assert g.block_tokens == orc.block_tokens(w)
        assert g.max_blocks == max(1, orc.n_cold_blocks(5000, w))
        assert g.hot_cap % g.block_tokens == 0 and g.hot_cap > w
        assert g.outlier_k == orc.outlier_count(g.block_tokens, 0.02)
        assert g.page_bytes % 128 == 0 and g.block_tokens_pad % 16 == 0
    g = _geom()
    assert lib.tq_geom_finish(C.byref(g)) == 0
    # one page = 16 KB key codes + 12 KB 3-bit value codes + norms + scale + mean, then the
    # header, second copy of the widest channels' codes, and the page's by-token outlier copy
    assert (g.k_bytes, g.v_bytes, g.hdr_off, g.ent_off) == (16384, 12288, 30720, 30720 + 576)
    assert g.page_bytes == 30720 + 4096
    # within 1 % of the reference's container bytes for the same block
    assert g.page_bytes <= 1.01 * (16384 + 12288 + 1024 + 1024 + 6 * 5 * 128)
    assert g.group == 4 and g.outlier_k == 5


@pytest.mark.parametrize("kw,code", [
    (dict(head_dim=64), -2), (dict(key_bits=3), -2), (dict(value_bits=2), -2),
    (dict(hot_window=1024), -2), (dict(n_q_heads=12), -1), (dict(outlier_frac=1.5), -1),
    (dict(kv_dtype=7), -1), (dict(n_seqs=0), -1),
])
def test_geometry_rejects(lib, kw, code):
    g = _geom(**kw)
    assert lib.tq_geom_finish(C.byref(g)) == code
    assert lib.tq_last_error() != b""


def test_sizes_and_null_handling(lib):
    from turboquant_pro_b200._lib import TqSizes

    g = _geom(n_layers=32, n_seqs=32)
    assert lib.tq_geom_finish(C.byref(g)) == 0
    s = TqSizes()
    assert lib.tq_ctx_sizes(C.byref(g), C.byref(s)) == 0
    assert s.pages == 32 * 32 * 8 * g.max_blocks * g.page_bytes
    assert s.hot_k == 32 * 32 * 8 * g.hot_cap * 128 * 2
    assert lib.tq_ctx_sizes(None, C.byref(s)) == -1
    assert lib.tq_seq_lengths(None, 0, 0, None, None, None) == -1
    assert lib.tq_decode(None, 0, None, 0, None, None) == -1


def test_value_encoder_switch_checks_its_argument(lib):
    """tq_set_value_encoder: 0 (mma.sync), 1 (tcgen05), -1 (the default); nothing else.  The
    switch is host state, so this needs no GPU."""
    try:
        for kind in (0, 1, -1):
            assert lib.tq_set_value_encoder(kind) == 0
        for kind in (2, -2, 7):
            assert lib.tq_set_value_encoder(kind) == -1
            assert b"value encoder" in lib.tq_last_error()
    finally:
        assert lib.tq_set_value_encoder(-1) == 0


def test_facade_refuses_cpu():
    import torch

    from turboquant_pro_b200 import TurboQuantKVCache

    with pytest.raises(RuntimeError):
        TurboQuantKVCache.robust(use_gpu=False)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            TurboQuantKVCache.robust(n_heads=2)

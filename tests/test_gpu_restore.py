"""Restoring a cache from exported blocks (tq_import_block + tq_restore_hot): the restored
context holds the same containers bit for bit, answers a decode step like the original and
goes on appending like it; also through the tqp-kv-npz/1 wire format."""

from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CONTAINER_FIELDS = ("key_indices", "nf4_scale", "nf4_mean", "outlier_idx", "value_indices",
                    "value_norms")


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    return torch


def _same_block(a, b):
    for name in CONTAINER_FIELDS:
        if a[name] is None:
            assert b[name] is None, name
        else:
            assert np.array_equal(a[name], b[name]), name
    if a["outlier_val"] is not None:
        assert np.array_equal(a["outlier_val"].view(np.uint16), b["outlier_val"].view(np.uint16))


def _restore(torch, src, dst, layer, seq, via_blob=False, **blob_kw):
    total, cold, _hot = src.lengths(layer, seq)
    nb = cold // src.geom.block_tokens
    dst.clear(layer, seq)
    for b in reversed(range(nb)):  # any order
        if via_blob:
            dst.import_blob(layer, seq, b, src.export_blob(layer, seq, b, **blob_kw))
        else:
            dst.import_block(layer, seq, b, src.export_block(layer, seq, b))
    hk, hv = src.dequant(layer, seq, cold, total)  # the hot window is stored exactly
    dst.restore_hot(layer, seq, total, hk.permute(1, 0, 2), hv.permute(1, 0, 2))
    return nb


@pytest.mark.parametrize("mode,frac,vb,dt,w,n", [
    ("nf4_asym", 0.02, 3, "float16", 512, 1500),
    ("nf4_asym", 0.02, 4, "bfloat16", 512, 1290),
    ("uniform", 0.0, 3, "float32", 512, 800),
    ("nf4", 0.05, 3, "float16", 64, 200),       # general-shape kernel, 32-token blocks
])
def test_restored_cache_equals_the_original(torch_cuda, mode, frac, vb, dt, w, n):
    torch = torch_cuda
    from turboquant_pro_b200 import KVContext
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp = 2, 4
    kw = dict(n_layers=2, n_seqs=2, n_kv_heads=h, n_q_heads=h * grp, value_bits=vb, hot_window=w,
              outlier_frac=frac, max_tokens_per_seq=n + 600, kv_dtype=dt, seed=11, key_mode=mode)
    src, dst = KVContext(**kw), KVContext(**kw)
    k, v = make_kv(5, h, n + 300, dtype=np.float32)
    kt, vt = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    layer, seq = 1, 1
    src.append(layer, kt[None, :n].expand(2, -1, -1, -1).contiguous(),
               vt[None, :n].expand(2, -1, -1, -1).contiguous())
    dst.append(layer, kt[None, :40].expand(2, -1, -1, -1).contiguous(),
               vt[None, :40].expand(2, -1, -1, -1).contiguous())  # stale content to replace
    with pytest.raises(ValueError):  # not cleared
        dst.import_block(layer, seq, 0, src.export_block(layer, seq, 0))
    nb = _restore(torch, src, dst, layer, seq)
    assert nb >= 2 and dst.lengths(layer, seq) == src.lengths(layer, seq)
    assert dst.lengths(layer, 0)[0] == 40  # the other sequence is untouched
    for b in range(nb):
        _same_block(src.export_block(layer, seq, b), dst.export_block(layer, seq, b))
    assert dst.memory_stats(layer, seq) == src.memory_stats(layer, seq)
    ks, vs = src.dequant(layer, seq, 0, n)
    kd, vd = dst.dequant(layer, seq, 0, n)
    assert torch.equal(ks, kd) and torch.equal(vs, vd)
    q = torch.from_numpy(np.stack([make_q(3, h * grp), make_q(4, h * grp)])).cuda()
    # a token's outliers are stored in channel order by the encoder and by the importer alike,
    # so equal containers mean equal page images and the decode agrees bit for bit
    a, b = src.decode(layer, q)[seq], dst.decode(layer, q)[seq]
    assert torch.equal(a, b)
    # both go on: the next cold blocks (pool cursors, ring positions) come out the same
    src.clear(layer, 0)
    dst.clear(layer, 0)
    for c in (src, dst):
        c.append(layer, kt[None, n:n + 300].contiguous(), vt[None, n:n + 300].contiguous(),
                 seq_begin=seq)
    assert dst.lengths(layer, seq) == src.lengths(layer, seq)
    nb2 = src.lengths(layer, seq)[1] // src.geom.block_tokens
    assert nb2 > nb
    for blk in range(nb2):
        _same_block(src.export_block(layer, seq, blk), dst.export_block(layer, seq, blk))
    # a token's outliers are stored in channel order by the encoder and by the importer alike,
    # so equal containers mean equal page images and the decode agrees bit for bit
    a, b = src.decode(layer, q)[seq], dst.decode(layer, q)[seq]
    assert torch.equal(a, b)
    assert src.status() == 0 and dst.status() == 0


def test_restore_with_heavy_tokens_and_through_the_wire_format(torch_cuda):
    """Overflow lists and a spilled page survive the restore; the same through blobs, with the
    sparse zero-point (means of the masked channels only travel)."""
    torch = torch_cuda
    from turboquant_pro_b200 import KVContext
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp, n, w = 2, 4, 1100, 512
    k, v = make_kv(33, h, n, dtype=np.float16)
    k = k.astype(np.float32)
    for tok, head, chans in ((5, 0, slice(None)), (300, 0, slice(0, 20)), (301, 0, slice(10, 30)),
                             (100, 1, slice(0, 128, 3))):
        b0 = tok // 256 * 256
        k[tok, head, chans] = 1.5 * np.abs(k[b0:b0 + 256, head, chans]).max(axis=0)
    k = k.astype(np.float16)
    mask = np.arange(128) >= 32
    kw = dict(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=h * grp, value_bits=3, hot_window=w,
              max_tokens_per_seq=n, kv_dtype="float16", seed=33, key_mean_mask=mask)
    src, dst, dst2 = KVContext(**kw), KVContext(**kw), KVContext(**kw)
    src.append(0, torch.from_numpy(k)[None].cuda(), torch.from_numpy(v)[None].cuda())
    q = torch.from_numpy(make_q(33, h * grp))[None].cuda()
    want = src.decode(0, q)
    nb = _restore(torch, src, dst, 0, 0)
    nb2 = _restore(torch, src, dst2, 0, 0, via_blob=True, zero_point="sparse", rope_theta=1e4)
    assert nb == nb2 == 3
    for c in (dst, dst2):
        for b in range(nb):
            _same_block(src.export_block(0, 0, b), c.export_block(0, 0, b))
        assert torch.equal(c.decode(0, q), want)
        c.set_kernel("general")
        assert torch.allclose(c.decode(0, q), want, rtol=2e-2, atol=2e-3)
        assert c.status() == 0
    # wrong block shape, and a block index the context cannot hold
    blk = src.export_block(0, 0, 0)
    dst.clear(0, 0)
    with pytest.raises(ValueError):
        dst.import_block(0, 0, 0, dict(blk, key_indices=blk["key_indices"][:-1]))
    with pytest.raises(RuntimeError):
        dst.import_block(0, 0, dst.geom.max_blocks, blk)
    bad = dict(blk, outlier_idx=blk["outlier_idx"][::-1].copy())
    with pytest.raises(ValueError):
        dst.import_block(0, 0, 0, bad)


@pytest.mark.parametrize("dt", ["float16", "bfloat16", "float32"])
def test_export_state_import_state_round_trip(torch_cuda, dt):
    """The offload pair: one call takes everything a cache holds, one call puts it back into
    another context (here: another sequence slot of another context)."""
    torch = torch_cuda
    from turboquant_pro_b200 import KVContext
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp, n = 2, 2, 1000
    kw = dict(n_layers=1, n_seqs=2, n_kv_heads=h, n_q_heads=h * grp, value_bits=3,
              hot_window=512, max_tokens_per_seq=n + 8, kv_dtype=dt, seed=2)
    src, dst = KVContext(**kw), KVContext(**kw)
    k, v = make_kv(9, h, n, dtype=np.float32)
    kt, vt = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    src.append(0, kt[None], vt[None])
    state = src.export_state(0, 0)
    assert state["n_tokens"] == n and len(state["blocks"]) == 2
    assert all(isinstance(b, bytes) for b in state["blocks"])
    dst.import_state(0, 1, state)
    assert dst.lengths(0, 1) == src.lengths(0, 0) and dst.lengths(0, 0)[0] == 0
    ks, vs = src.dequant(0, 0, 0, n)
    kd, vd = dst.dequant(0, 1, 0, n)
    assert torch.equal(ks, kd) and torch.equal(vs, vd)
    q = torch.from_numpy(np.stack([make_q(1, h * grp)] * 2)).cuda()
    dst.append(0, kt[None, :3], vt[None, :3])  # the untouched slot gets a few tokens of its own
    src.append(0, kt[None, :3], vt[None, :3], seq_begin=1)
    assert torch.allclose(dst.decode(0, q)[1], src.decode(0, q)[0], rtol=1e-5, atol=1e-6)
    empty = KVContext(**kw).export_state(0, 0)
    dst.import_state(0, 1, empty)
    assert dst.lengths(0, 1) == (0, 0, 0)
    with pytest.raises(ValueError):
        KVContext(**dict(kw, value_bits=4)).import_state(0, 0, state)

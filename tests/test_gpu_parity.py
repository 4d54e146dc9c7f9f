"""GPU parity tests: every call goes through the C ABI (via the ctypes binding) and is
compared with the reference fixtures and with the CPU oracle on the same seeded inputs.

Bars: emitted codes, scales, means, outlier lists, norms and the dequantised getters are
bit-exact; attention outputs are within rtol 2e-2 / atol 2e-3 of dequantise-then-attend.
"""

from __future__ import annotations

import numpy as np
import pytest

from conftest import load_golden

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 2e-3


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    return torch


def _ctx(**kw):
    from turboquant_pro_b200 import KVContext

    return KVContext(**kw)


def _np_dtype_name(a):
    return "float16" if a.dtype == np.float16 else "float32"


def _dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _oracle(h, vb, w, pi, k, v, frac=0.02):
    from oracle import tq_oracle as orc

    c = orc.OracleCache(128, h, 4, vb, w, frac, 0)
    c.pi, c.pi_t = pi, np.ascontiguousarray(pi.T)
    for t in range(k.shape[0]):
        c.append(k[t], v[t])
    return c


def _check_block(blk, kb, vb_blk, vb):
    from oracle import tq_oracle as orc

    assert np.array_equal(blk["key_indices"], orc.pack_key_codes(kb["codes"]))
    assert np.array_equal(blk["nf4_scale"][0], kb["scale"])
    assert np.array_equal(blk["nf4_mean"][0], kb["mean"])
    assert np.array_equal(blk["outlier_idx"], kb["out_idx"])
    assert np.array_equal(blk["outlier_val"].view(np.uint16), kb["out_val"].view(np.uint16))
    assert np.array_equal(blk["value_indices"], orc.pack_value_codes(vb_blk["codes"], vb))
    assert np.array_equal(blk["value_norms"][0], vb_blk["norms"])


# ------------------------------------------------------------------------------------ #
# encoders against the reference fixtures                                               #
# ------------------------------------------------------------------------------------ #

@pytest.mark.parametrize("name", ["block_k4v3.npz", "block_k4v4_f16.npz", "block_ties.npz",
                                  "block_short.npz"])
def test_block_encoders_bit_exact_vs_reference(torch_cuda, name):
    """One cold block flushed by the CUDA encoders == the reference's containers."""
    torch = torch_cuda
    g = load_golden(name)
    k, v = g["k"], g["v"]                       # (S, H, D)
    s, h, _ = k.shape
    w = 2 * s                                   # block size (w+1)//2 == s
    vb = int(g["value_bits"])
    ctx = _ctx(n_layers=1, n_seqs=1, n_kv_heads=h, value_bits=vb, hot_window=w,
               max_tokens_per_seq=4 * w, kv_dtype=_np_dtype_name(k), pi=g["pi"])
    fill = np.zeros((w + 1 - s, h, 128), dtype=k.dtype)
    kk = np.concatenate([k, fill + 1]) [None]
    vv = np.concatenate([v, fill + 1])[None]
    ctx.append(0, _dev(torch, kk), _dev(torch, vv))
    assert ctx.lengths(0, 0) == (w + 1, s, w + 1 - s)
    blk = ctx.export_block(0, 0, 0)
    assert np.array_equal(blk["key_indices"], g["key_indices"])
    assert np.array_equal(blk["nf4_scale"], g["nf4_scale"])
    assert np.array_equal(blk["nf4_mean"], g["nf4_mean"])
    assert np.array_equal(blk["outlier_idx"], g["outlier_idx"])
    assert np.array_equal(blk["outlier_val"].view(np.uint16), g["outlier_val"].view(np.uint16))
    assert np.array_equal(blk["value_norms"], g["value_norms"])
    assert np.array_equal(blk["value_indices"], g["value_indices"])
    kd, vd = ctx.dequant(0, 0, 0, s)
    assert np.array_equal(kd.cpu().numpy(), g["key_dequant"])
    assert np.array_equal(vd.cpu().numpy(), g["value_dequant"])
    assert ctx.status() == 0


@pytest.mark.parametrize("name,vb,bulk", [
    ("cache_w16.npz", 4, False), ("cache_w16.npz", 4, True),
    ("cache_w512_gqa.npz", 3, True), ("cache_w512_gqa.npz", 3, False),
    ("cache_w7.npz", 3, False), ("cache_w7.npz", 3, True),
])
def test_cache_matches_reference(torch_cuda, name, vb, bulk):
    """A cache filled token by token (or in one bulk call) reproduces the reference's cold
    blocks, getters, statistics and dequantise-then-attend output."""
    torch = torch_cuda
    g = load_golden(name)
    k, v, q = g["k"], g["v"], g["q"]
    n, h, _ = k.shape
    w = int(g["hot_window"])
    ctx = _ctx(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=q.shape[0], value_bits=vb,
               hot_window=w, max_tokens_per_seq=n + 8, kv_dtype=_np_dtype_name(k), pi=g["pi"])
    kd, vd = _dev(torch, k[None]), _dev(torch, v[None])
    if bulk:
        cut = n // 3  # two calls: exercises blocks that straddle ring and new tokens
        ctx.append(0, kd[:, :cut], vd[:, :cut])
        ctx.append(0, kd[:, cut:], vd[:, cut:])
    else:
        for t in range(n):
            ctx.append(0, kd[:, t:t + 1], vd[:, t:t + 1])
    total, cold, hot = ctx.lengths(0, 0)
    assert (total, hot) == (int(g["length"]), int(g["hot_length"]))
    nb = int(g["n_blocks"])
    assert cold == int(g["cold_lengths"].sum())
    for i in range(nb):
        blk = ctx.export_block(0, 0, i)
        assert np.array_equal(blk["key_indices"], g[f"b{i}_key_indices"])
        assert np.array_equal(blk["nf4_scale"], g[f"b{i}_nf4_scale"])
        assert np.array_equal(blk["nf4_mean"], g[f"b{i}_nf4_mean"])
        assert np.array_equal(blk["outlier_idx"], g[f"b{i}_outlier_idx"])
        assert np.array_equal(blk["outlier_val"].view(np.uint16),
                              g[f"b{i}_outlier_val"].view(np.uint16))
        assert np.array_equal(blk["value_indices"], g[f"b{i}_value_indices"])
        assert np.array_equal(blk["value_norms"], g[f"b{i}_value_norms"])
    keys, vals = ctx.dequant(0, 0, 0, total)
    assert np.array_equal(keys[0].cpu().numpy(), g["keys_head0"])
    assert np.array_equal(vals[0].cpu().numpy(), g["values_head0"])
    cold_b, hot_b = ctx.memory_stats(0, 0)
    assert [cold_b, hot_b] == g["memory_stats"][:2].tolist()
    out = ctx.decode(0, _dev(torch, q[None]))[0].cpu().numpy()
    err = np.abs(out - g["attn"]).max()
    assert np.allclose(out, g["attn"], rtol=RTOL, atol=ATOL), f"max abs err {err}"
    if "fused" in g.files:
        assert np.allclose(out, g["fused"], rtol=RTOL, atol=ATOL)
    assert ctx.status() == 0


@pytest.mark.parametrize("name,bulk", [("cache_polar_keys_v3.npz", False),
                                       ("cache_polar_keys_v3.npz", True),
                                       ("cache_polar_keys_v4_w16.npz", False)])
def test_polar_keys_cache_matches_reference(torch_cuda, name, bulk):
    """``TurboQuantKVCache(per_channel_keys=False)``, the legacy key format in which keys go
    through the value quantiser (core.py:1022-1033) and decode is ``_cold_partials``
    (kv_fused.py:84-98): cold containers, getters and statistics of the reference bit for bit,
    ``fused_decode`` within the attention tolerance."""
    torch = torch_cuda
    from turboquant_pro_b200 import TurboQuantKVCache

    g = load_golden(name)
    k, v, q = g["k"], g["v"], g["q"]
    n, h, _ = k.shape
    bits = int(g["bits"])
    cache = TurboQuantKVCache(head_dim=128, n_heads=h, bits=bits, hot_window=int(g["hot_window"]),
                              seed=int(g["seed"]), per_channel_keys=False, max_tokens=n + 8,
                              dtype=_np_dtype_name(k))
    assert np.array_equal(cache._tq._Pi, g["pi"])
    if bulk:
        cache._ctx.append(0, _dev(torch, k[None]), _dev(torch, v[None]))
    else:
        for t in range(n):
            cache.append(k[t], v[t])
    assert (cache.length, cache.hot_length) == (int(g["length"]), int(g["hot_length"]))
    assert list(cache._cold_lengths) == g["cold_lengths"].tolist()
    assert len(cache._cold_keys) == int(g["n_blocks"])
    for i in range(int(g["n_blocks"])):
        ck, cv = cache._cold_keys[i], cache._cold_values[i]
        assert ck.bits == bits and ck.packed
        assert np.array_equal(ck.indices, g[f"b{i}_key_indices"])
        assert np.array_equal(ck.norms, g[f"b{i}_key_norms"])
        assert np.array_equal(cv.indices, g[f"b{i}_value_indices"])
        assert np.array_equal(cv.norms, g[f"b{i}_value_norms"])
    keys = np.asarray(cache.get_keys(0, cache.length))
    vals = np.asarray(cache.get_values(0, cache.length))
    assert keys.shape == (1, h, n, 128)
    assert np.array_equal(keys[0, 0], g["keys_head0"])
    assert np.array_equal(vals[0, 0], g["values_head0"])
    st = cache.memory_stats()
    assert [st["cold_bytes"], st["hot_bytes"], st["total_bytes"],
            st["uncompressed_equivalent_bytes"]] == g["memory_stats"].tolist()
    out = np.asarray(cache.fused_decode(q))
    assert np.allclose(out, g["attn"], rtol=RTOL, atol=ATOL), np.abs(out - g["attn"]).max()
    assert np.allclose(out, g["fused"], rtol=RTOL, atol=ATOL)
    assert cache._ctx.last_kernel() == "general" and cache._ctx.status() == 0
    # the sequence-split partials of this format merge to the same output
    ctx = cache._ctx
    qd = _dev(torch, q[None])
    nb = int(g["n_blocks"])
    parts = torch.stack([ctx.decode_partial(0, qd, 0, nb // 2, False),
                         ctx.decode_partial(0, qd, nb // 2, 1 << 20, True)])
    merged = ctx.lse_combine(parts.reshape(2, h, 130)).cpu().numpy()
    assert np.allclose(merged, out, rtol=1e-3, atol=1e-4)
    # formats this key mode does not take
    with pytest.raises(NotImplementedError):
        TurboQuantKVCache(head_dim=128, n_heads=h, bits=3, key_bits=4, value_bits=3,
                          per_channel_keys=False)


# ------------------------------------------------------------------------------------ #
# decode against the oracle on seeded synthetic tensors                                 #
# ------------------------------------------------------------------------------------ #

@pytest.mark.parametrize("h,grp,n,w,vb,dt", [
    (2, 1, 1500, 512, 4, "float32"),     # MHA, K4/V4, float32 hot window (config-0 shape)
    (2, 4, 1500, 512, 3, "float16"),     # GQA 4, K4/V3 (Llama-3-8B shape)
    (1, 8, 1100, 512, 4, "float16"),     # GQA 8 (Llama-3-70B shape)
    (2, 4, 300, 512, 3, "bfloat16"),     # hot only
    (2, 4, 1300, 512, 4, "bfloat16"),    # bfloat16 tokens through both encoders (3 cold blocks)
    (2, 2, 770, 512, 3, "float16"),      # exactly at a flush boundary + 1
    (1, 7, 200, 64, 3, "float32"),       # odd group (Qwen2.5-7B shape), small window
    (1, 16, 150, 32, 4, "float16"),      # group 16
])
def test_decode_vs_oracle(torch_cuda, h, grp, n, w, vb, dt):
    torch = torch_cuda
    from turboquant_pro_b200.synth import make_kv, make_q

    seed = 100 + n
    k, v = make_kv(seed, h, n, dtype=np.float16)
    if dt == "bfloat16":
        kt = torch.from_numpy(k.astype(np.float32)).to(torch.bfloat16)
        vt = torch.from_numpy(v.astype(np.float32)).to(torch.bfloat16)
        k, v = kt.float().numpy(), vt.float().numpy()
    else:
        kt, vt = torch.from_numpy(k.astype(dt)), torch.from_numpy(v.astype(dt))
        k, v = k.astype(np.float32), v.astype(np.float32)
    q = make_q(seed, h * grp)
    ctx = _ctx(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=h * grp, value_bits=vb,
               hot_window=w, max_tokens_per_seq=n + 8, kv_dtype=dt, seed=seed)
    ctx.append(0, kt[None].cuda(), vt[None].cuda())
    ref = _oracle(h, vb, w, ctx.pi, k, v)
    for i in range(len(ref.cold_k)):
        _check_block(ctx.export_block(0, 0, i), ref.cold_k[i], ref.cold_v[i], vb)
    want = ref.attend(q)
    for qdt in (torch.float32, torch.bfloat16):
        qq = torch.from_numpy(q).to(qdt)
        got = ctx.decode(0, qq[None].cuda())[0].cpu().numpy()
        want_q = ref.attend(qq.float().numpy())
        err = np.abs(got - want_q).max()
        assert np.allclose(got, want_q, rtol=RTOL, atol=ATOL), f"{qdt}: max abs err {err}"
    assert want.shape == (h * grp, 128)


@pytest.mark.parametrize("dt", ["float16", "float32"])
def test_rows_off_the_16_byte_grid_encode_the_same(torch_cuda, dt):
    """Tokens handed over as a view whose rows start one element past a 16-byte boundary (the
    encoders then load element by element) give the same pages, bit for bit, as the same tokens
    in a contiguous tensor."""
    torch = torch_cuda
    from turboquant_pro_b200.synth import make_kv

    h, n, w, vb = 2, 1100, 512, 3
    k, v = make_kv(77, h, n, dtype=np.float16)
    tdt = getattr(torch, dt)
    kt, vt = torch.from_numpy(k).to(tdt).cuda(), torch.from_numpy(v).to(tdt).cuda()
    wide_k = torch.zeros((1, n, h, 129), dtype=tdt, device="cuda")
    wide_v = torch.zeros((1, n, h, 129), dtype=tdt, device="cuda")
    wide_k[0, :, :, 1:] = kt
    wide_v[0, :, :, 1:] = vt
    blocks = []
    for src_k, src_v in ((kt[None], vt[None]), (wide_k[..., 1:], wide_v[..., 1:])):
        ctx = _ctx(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=h, value_bits=vb, hot_window=w,
                   max_tokens_per_seq=n + 8, kv_dtype=dt, seed=5)
        assert src_k.stride(3) == 1
        ctx.append(0, src_k, src_v)
        assert ctx.status() == 0
        nb = ctx.lengths(0, 0)[1] // 256
        assert nb >= 2
        blocks.append([ctx.export_block(0, 0, i) for i in range(nb)])
    assert len(blocks[0]) == len(blocks[1])
    for a, b in zip(*blocks):
        assert a.keys() == b.keys()
        for name in a:
            if a[name] is None:
                assert b[name] is None
            else:
                assert np.array_equal(np.asarray(a[name]), np.asarray(b[name])), name


@pytest.mark.parametrize("dt,vb,key_mode", [("float16", 3, "nf4_asym"), ("bfloat16", 4, "nf4_asym"),
                                            ("float32", 3, "nf4_asym"), ("float16", 4, "polar"),
                                            ("float16", 3, "polar")])
@pytest.mark.parametrize("aligned", [True, False])
def test_value_encoder_on_tcgen05_writes_the_same_pages(torch_cuda, dt, vb, key_mode, aligned):
    """The value encoder whose rotation runs on tcgen05.mma (accumulators in tensor memory)
    (the default; checked against the oracle and the golden fixtures by every other test of
    this file) and the one on mma.sync write the same pages, bit for bit, for every element
    type, code width and row alignment, and for keys in PolarQuant form; the tokens include
    all-zero rows, whose products sit on a code boundary in every channel."""
    torch = torch_cuda
    from turboquant_pro_b200._lib import load
    from turboquant_pro_b200.synth import make_kv

    lib = load()
    h, n, w = 2, 1100, 512
    k, v = make_kv(78, h, n, dtype=np.float16)
    # all-zero tokens rotate onto a code boundary in every channel: three in one group, a whole
    # group, and one that goes through the hot ring first (more boundary cases at once than
    # the encoder's list of deferred recomputations holds)
    for lo, hi in ((5, 8), (32, 48), (300, 301), (720, 722)):
        v[lo:hi] = 0
        k[lo:hi] = 0
    tdt = getattr(torch, dt)
    kt, vt = torch.from_numpy(k).to(tdt).cuda(), torch.from_numpy(v).to(tdt).cuda()
    if aligned:
        src_k, src_v = kt[None], vt[None]
    else:
        wide_k = torch.zeros((1, n, h, 129), dtype=tdt, device="cuda")
        wide_v = torch.zeros((1, n, h, 129), dtype=tdt, device="cuda")
        wide_k[0, :, :, 1:] = kt
        wide_v[0, :, :, 1:] = vt
        src_k, src_v = wide_k[..., 1:], wide_v[..., 1:]
    extra = dict(key_mode="polar", key_bits=vb, outlier_frac=0.0) if key_mode == "polar" else {}
    blocks = []
    try:
        for kind in (0, 1):
            assert lib.tq_set_value_encoder(kind) == 0
            ctx = _ctx(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=h, value_bits=vb,
                       hot_window=w, max_tokens_per_seq=n + 8, kv_dtype=dt, seed=5, **extra)
            # in two calls, so that the second one also reads rows from the hot ring
            ctx.append(0, src_k[:, :700], src_v[:, :700])
            ctx.append(0, src_k[:, 700:], src_v[:, 700:])
            assert ctx.status() == 0
            nb = ctx.lengths(0, 0)[1] // 256
            assert nb >= 2
            blocks.append([ctx.export_block(0, 0, i) for i in range(nb)])
    finally:
        assert lib.tq_set_value_encoder(-1) == 0
    assert lib.tq_set_value_encoder(2) != 0
    assert len(blocks[0]) == len(blocks[1])
    if key_mode != "polar" and aligned:
        kf, vf = kt.float().cpu().numpy(), vt.float().cpu().numpy()
        ref = _oracle(h, vb, w, ctx.pi, kf, vf)
        assert len(ref.cold_k) == len(blocks[1])
        for i, blk in enumerate(blocks[1]):
            _check_block(blk, ref.cold_k[i], ref.cold_v[i], vb)
    for a, b in zip(*blocks):
        assert a.keys() == b.keys()
        for name in a:
            if a[name] is None:
                assert b[name] is None
            else:
                assert np.array_equal(np.asarray(a[name]), np.asarray(b[name])), name


@pytest.mark.parametrize("vb,aligned", [(3, True), (4, True), (3, False)])
def test_value_encoders_agree_on_many_groups_per_cta(torch_cuda, vb, aligned):
    """Flushes of more than three thousand groups of 16 tokens (more than three per 128-thread
    part of the tcgen05 encoder, so that its pipeline of three groups in flight runs full and
    drains) give the pages of the mma.sync encoder bit for bit, in every block of every
    sequence and head; the second call also takes rows from the hot ring, and one variant
    hands the tokens over off the 16-byte grid."""
    torch = torch_cuda
    from turboquant_pro_b200._lib import load

    lib = load()
    b, h, n = 2, 8, 4200
    gen = torch.Generator(device="cuda")
    gen.manual_seed(11)
    k = torch.randn((b, n, h, 128), generator=gen, device="cuda").half()
    v = torch.randn((b, n, h, 128), generator=gen, device="cuda").half()
    if not aligned:
        wide_k = torch.zeros((b, n, h, 129), dtype=torch.float16, device="cuda")
        wide_v = torch.zeros((b, n, h, 129), dtype=torch.float16, device="cuda")
        wide_k[..., 1:] = k
        wide_v[..., 1:] = v
        k, v = wide_k[..., 1:], wide_v[..., 1:]
    blocks = []
    try:
        for kind in (0, 1):
            assert lib.tq_set_value_encoder(kind) == 0
            ctx = _ctx(n_layers=1, n_seqs=b, n_kv_heads=h, n_q_heads=h, value_bits=vb,
                       hot_window=512, max_tokens_per_seq=n + 8, kv_dtype="float16", seed=6)
            ctx.append(0, k[:, :900], v[:, :900])
            ctx.append(0, k[:, 900:], v[:, 900:])
            assert ctx.status() == 0
            nb = ctx.lengths(0, 0)[1] // 256
            assert nb >= 14
            blocks.append([ctx.export_block(0, s, i) for s in range(b) for i in range(nb)])
    finally:
        assert lib.tq_set_value_encoder(-1) == 0
    for x, y in zip(*blocks):
        for name in ("value_indices", "value_norms", "key_indices"):
            assert np.array_equal(np.asarray(x[name]), np.asarray(y[name])), name


def test_batched_layers_ragged(torch_cuda):
    """Several layers and sequences with different lengths in one context; each cache is
    independent and matches its own oracle."""
    torch = torch_cuda
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp, w, vb = 2, 4, 64, 3
    lens = [0, 45, 200, 129]
    ctx = _ctx(n_layers=2, n_seqs=len(lens), n_kv_heads=h, n_q_heads=h * grp, value_bits=vb,
               hot_window=w, max_tokens_per_seq=256, kv_dtype="float16", seed=3)
    refs = {}
    for layer in range(2):
        for s, n in enumerate(lens):
            if n == 0:
                continue
            k, v = make_kv(1000 + 10 * layer + s, h, n, dtype=np.float16)
            ctx.append(layer, _dev(torch, k[None]), _dev(torch, v[None]), seq_begin=s)
            refs[(layer, s)] = _oracle(h, vb, w, ctx.pi, k.astype(np.float32),
                                       v.astype(np.float32))
    for layer in range(2):
        q = np.stack([make_q(7 + s + 100 * layer, h * grp) for s in range(len(lens))])
        out = ctx.decode(layer, _dev(torch, q)).cpu().numpy()
        assert np.all(out[0] == 0.0)  # empty sequence -> zeros
        for s, n in enumerate(lens):
            if n == 0:
                continue
            want = refs[(layer, s)].attend(q[s])
            assert np.allclose(out[s], want, rtol=RTOL, atol=ATOL), (layer, s)
    # clearing one sequence leaves the others intact
    ctx.clear(0, 2)
    assert ctx.lengths(0, 2) == (0, 0, 0) and ctx.lengths(0, 3)[0] == 129
    k, v = make_kv(55, h, 100, dtype=np.float16)
    ctx.append(0, _dev(torch, k[None]), _dev(torch, v[None]), seq_begin=2)
    ref = _oracle(h, vb, w, ctx.pi, k.astype(np.float32), v.astype(np.float32))
    q = np.stack([make_q(70 + s, h * grp) for s in range(len(lens))])
    out = ctx.decode(0, _dev(torch, q)).cpu().numpy()
    assert np.allclose(out[2], ref.attend(q[2]), rtol=RTOL, atol=ATOL)
    assert np.allclose(out[3], refs[(0, 3)].attend(q[3]), rtol=RTOL, atol=ATOL)


def test_sequence_split_partials_merge(torch_cuda):
    """Partial (m, l, o) states over disjoint block ranges + the hot window merge to the
    full decode (the multi-device sequence split, emulated on one device)."""
    torch = torch_cuda
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp, n, w, vb = 2, 4, 1400, 128, 3
    k, v = make_kv(9, h, n, dtype=np.float16)
    q = _dev(torch, make_q(9, h * grp)[None])
    ctx = _ctx(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=h * grp, value_bits=vb,
               hot_window=w, max_tokens_per_seq=n, kv_dtype="float16", seed=9)
    ctx.append(0, _dev(torch, k[None]), _dev(torch, v[None]))
    full = ctx.decode(0, q).cpu().numpy()
    nb = ctx.lengths(0, 0)[1] // ctx.block_tokens
    world = 4
    parts = []
    for r in range(world):
        lo, hi = nb * r // world, nb * (r + 1) // world
        parts.append(ctx.decode_partial(0, q, lo, hi, with_hot=(r == world - 1)).clone())
    mlo = torch.stack(parts).reshape(world, h * grp, 130)
    merged = ctx.lse_combine(mlo).cpu().numpy()
    assert np.allclose(merged, full[0], rtol=1e-4, atol=1e-5)
    ref = _oracle(h, vb, w, ctx.pi, k.astype(np.float32), v.astype(np.float32))
    assert np.allclose(merged, ref.attend(make_q(9, h * grp)), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("grp,vb,dt", [(4, 3, "float16"), (8, 4, "float16"), (1, 4, "float32"),
                                        (2, 3, "bfloat16"), (4, 4, "bfloat16")])
def test_tensor_core_and_general_kernels_agree(torch_cuda, grp, vb, dt):
    """Ragged batch at the production geometry (256-token blocks): the tensor-core kernel
    and the general-shape kernel compute the same attention, and both match the oracle."""
    torch = torch_cuda
    from turboquant_pro_b200.synth import make_kv, make_q

    h, w = 2, 512
    lens = [0, 300, 513, 1300, 2200, 769]
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}[dt]
    ctx = _ctx(n_layers=1, n_seqs=len(lens), n_kv_heads=h, n_q_heads=h * grp, value_bits=vb,
               hot_window=w, max_tokens_per_seq=2304, kv_dtype=dt, seed=17)
    refs = {}
    for s, n in enumerate(lens):
        if n == 0:
            continue
        k, v = make_kv(300 + s, h, n, dtype=np.float16)
        kt = torch.from_numpy(k.astype(np.float32)).to(tdt)
        vt = torch.from_numpy(v.astype(np.float32)).to(tdt)
        ctx.append(0, kt[None].cuda(), vt[None].cuda(), seq_begin=s)
        refs[s] = _oracle(h, vb, w, ctx.pi, kt.float().numpy(), vt.float().numpy())
    q = np.stack([make_q(40 + s, h * grp) for s in range(len(lens))])
    qd = _dev(torch, q).to(torch.bfloat16)
    qf = qd.float().cpu().numpy()
    fast = ctx.decode(0, qd).cpu().numpy()
    ctx.set_kernel("general")
    slow = ctx.decode(0, qd).cpu().numpy()
    ctx.set_kernel("auto")
    assert ctx.status() == 0
    assert np.all(fast[0] == 0.0)
    for s, n in enumerate(lens):
        if n == 0:
            continue
        want = refs[s].attend(qf[s])
        assert np.allclose(slow[s], want, rtol=RTOL, atol=ATOL), f"general kernel, seq {s}"
        err = np.abs(fast[s] - want).max()
        assert np.allclose(fast[s], want, rtol=RTOL, atol=ATOL), f"seq {s}: max abs err {err}"
        assert np.allclose(fast[s], slow[s], rtol=RTOL, atol=ATOL)


def test_long_sequence_many_ctas_per_unit(torch_cuda):
    """One long sequence of one KV head: its pages spread over every CTA of the persistent
    kernel (one tile each), so the combine merges many partials; also the sequence-split
    partial path of the same kernel."""
    torch = torch_cuda
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp, n, w, vb = 1, 4, 30000, 512, 3
    k, v = make_kv(77, h, n, dtype=np.float16)
    ctx = _ctx(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=grp, value_bits=vb, hot_window=w,
               max_tokens_per_seq=n, kv_dtype="float16", seed=77)
    ctx.append(0, _dev(torch, k[None]), _dev(torch, v[None]))
    q = make_q(77, grp)
    qd = _dev(torch, q[None])
    fast = ctx.decode(0, qd)[0].cpu().numpy()
    ctx.set_kernel("general")
    slow = ctx.decode(0, qd)[0].cpu().numpy()
    ctx.set_kernel("auto")
    assert np.allclose(fast, slow, rtol=RTOL, atol=ATOL), np.abs(fast - slow).max()
    nb = ctx.lengths(0, 0)[1] // ctx.block_tokens
    world = 3
    parts = [ctx.decode_partial(0, qd, nb * r // world, nb * (r + 1) // world,
                                with_hot=(r == world - 1)).clone() for r in range(world)]
    merged = ctx.lse_combine(torch.stack(parts).reshape(world, grp, 130)).cpu().numpy()
    assert np.allclose(merged, fast, rtol=1e-3, atol=1e-4), np.abs(merged - fast).max()
    assert ctx.status() == 0
    # dequantise-then-attend on the device getters, in float64 on the host
    kd, vd = ctx.dequant(0, 0, 0, n)
    kd, vd = kd.cpu().numpy().astype(np.float64), vd.cpu().numpy().astype(np.float64)
    sc = np.einsum("gd,sd->gs", q.astype(np.float64), kd[0]) / np.sqrt(128.0)
    p = np.exp(sc - sc.max(axis=1, keepdims=True))
    want = (p / p.sum(axis=1, keepdims=True)) @ vd[0]
    assert np.allclose(fast, want, rtol=RTOL, atol=ATOL), np.abs(fast - want).max()


def test_facade_matches_reference_api(torch_cuda):
    """TurboQuantKVCache: the reference's constructor, append, getters, fused_decode,
    memory_stats and clear, checked on the reference's own cache fixture."""
    from turboquant_pro_b200 import AutoConfig, TurboQuantKVCache

    g = load_golden("cache_w16.npz")
    k, v, q = g["k"], g["v"], g["q"]
    cache = TurboQuantKVCache.robust(head_dim=128, n_heads=2, key_bits=4, value_bits=4,
                                     hot_window=16, seed=int(g["seed"]), max_tokens=256)
    with pytest.raises(RuntimeError, match="cache is empty"):
        cache.fused_decode(q)
    for t in range(k.shape[0]):
        if t % 2:
            cache.append(k[t], v[t])                              # (H, D)
        else:
            cache.append(k[t][None, :, None, :], v[t][None, :, None, :])  # (1, H, 1, D)
    assert cache.length == int(g["length"]) and cache.hot_length == int(g["hot_length"])
    assert cache.cold_length == int(g["cold_lengths"].sum())
    keys = cache.get_keys(0, cache.length)
    assert keys.shape == (1, 2, cache.length, 128) and keys.dtype == np.float32
    # the rotation comes from this host's LAPACK; keys do not depend on it
    assert np.array_equal(keys[0, 0], g["keys_head0"])
    assert cache.get_keys(5, 5).shape == (1, 2, 0, 128)
    out = cache.fused_decode(q)
    assert out.shape == (2, 128)
    assert np.allclose(out, g["attn"], rtol=RTOL, atol=ATOL)
    st = cache.memory_stats()
    assert st["cold_bytes"] == g["memory_stats"][0] and st["hot_bytes"] == g["memory_stats"][1]
    assert st["uncompressed_equivalent_bytes"] == g["memory_stats"][3]
    cache.clear()
    assert cache.length == 0
    cfg = AutoConfig.from_pretrained("llama-3-8b")
    c2 = cfg.build_cache(hot_window=32, use_gpu=True, seed=1, max_tokens=128)
    assert (c2.key_bits, c2.value_bits, c2.n_heads, c2.hot_window) == (4, 3, 8, 32)
    with pytest.raises(NotImplementedError):
        TurboQuantKVCache(head_dim=128, n_heads=2, bits=3)  # 3-bit uniform keys
    with pytest.raises(NotImplementedError):
        TurboQuantKVCache(head_dim=128, n_heads=2, bits=4, key_nuq=True)
    with pytest.raises(ValueError):
        TurboQuantKVCache(head_dim=128, n_heads=2, bits=4, key_nf4_asym=True,
                          key_zero_point="bias", key_rope_theta=1e4)  # no k_bias
    TurboQuantKVCache(head_dim=128, n_heads=2, bits=4, key_nf4_asym=True, max_tokens=64,
                      key_zero_point="bias", key_rope_theta=1e4, key_k_bias=np.ones(256))
    sp = TurboQuantKVCache(head_dim=128, n_heads=2, bits=4, key_nf4_asym=True, max_tokens=64,
                           key_zero_point="sparse", key_rope_theta=1e4)
    assert int(sp.context.key_mean_mask.sum()) == 76  # wavelengths beyond a 256-token block


def test_abi_error_codes(torch_cuda):
    """Invalid calls come back as status codes / the reference's exception types, and never
    reach a kernel launch."""
    torch = torch_cuda
    ctx = _ctx(n_layers=1, n_seqs=2, n_kv_heads=2, value_bits=3, hot_window=16,
               max_tokens_per_seq=32, kv_dtype="float16", seed=0)
    k = torch.zeros((1, 40, 2, 128), dtype=torch.float16, device="cuda")
    from turboquant_pro_b200._lib import TqError

    with pytest.raises(TqError, match="CAPACITY"):
        ctx.append(0, k, k)
    with pytest.raises(ValueError):
        ctx.append(3, k[:, :4], k[:, :4])          # bad layer
    with pytest.raises(ValueError):
        ctx.append(0, k[:, :4], k[:, :4], seq_begin=2)  # bad sequence
    with pytest.raises(ValueError):
        ctx.dequant(0, 0, 0, 5)                    # range beyond the stored tokens
    with pytest.raises(ValueError):
        ctx.decode(0, torch.zeros((2, 3, 128), device="cuda"))
    assert ctx.lengths(0, 0) == (0, 0, 0)
    with pytest.raises(NotImplementedError):
        _ctx(n_kv_heads=2, head_dim=64)
    with pytest.raises(NotImplementedError):
        _ctx(n_kv_heads=2, value_bits=2)


def test_degenerate_blocks(torch_cuda):
    """All-equal and all-zero blocks: every entry ties with the k-th magnitude, so the whole
    block lands in the outlier list, as in the reference; the pool absorbs it."""
    torch = torch_cuda
    h, w = 1, 16
    k = np.zeros((20, h, 128), np.float32)
    k[:8] = 0.5
    v = np.ones((20, h, 128), np.float32)
    v[3] = 0.0  # zero-norm value token
    ctx = _ctx(n_layers=1, n_seqs=1, n_kv_heads=h, value_bits=3, hot_window=w,
               max_tokens_per_seq=64, kv_dtype="float32", seed=2)
    ctx.append(0, _dev(torch, k[None]), _dev(torch, v[None]))
    ref = _oracle(h, 3, w, ctx.pi, k, v)
    blk = ctx.export_block(0, 0, 0)
    _check_block(blk, ref.cold_k[0], ref.cold_v[0], 3)
    assert blk["outlier_idx"].size == 8 * 128
    q = np.ones((1, 128), np.float32)
    out = ctx.decode(0, _dev(torch, q[None]))[0].cpu().numpy()
    assert np.allclose(out, ref.attend(q), rtol=RTOL, atol=ATOL)
    assert ctx.status() == 0


# ------------------------------------------------------------------------------------ #
# the other per-channel key grids (uniform, symmetric NF4)                              #
# ------------------------------------------------------------------------------------ #

@pytest.mark.parametrize("name,mode,frac", [("keys_uniform.npz", "uniform", 0.02),
                                            ("keys_uniform_ties.npz", "uniform", 0.0),
                                            ("keys_nf4.npz", "nf4", 0.02)])
def test_other_key_grids_encoder_bit_exact(torch_cuda, name, mode, frac):
    """One 256-token block flushed through the CUDA key encoder in each mode: packed codes,
    scale, mean / zero, outliers and the getter's dequantised keys equal the reference's."""
    torch = torch_cuda
    g = load_golden(name)
    k = g["k"]  # (S, H, D)
    s, h = k.shape[0], k.shape[1]
    dt = _np_dtype_name(k)
    # hot_window 511 -> blocks of 256 tokens; 512 + 1 tokens force exactly one flush... the
    # fixture is a single block, so fill the window with copies and flush once
    pad = np.zeros((257, h, 128), dtype=k.dtype)
    ctx = _ctx(n_layers=1, n_seqs=1, n_kv_heads=h, value_bits=4, hot_window=512,
               max_tokens_per_seq=1024, kv_dtype=dt, outlier_frac=frac, key_mode=mode, seed=0)
    both = np.concatenate([k, pad], axis=0)
    ctx.append(0, _dev(torch, both)[None], _dev(torch, both)[None])
    assert ctx.lengths(0, 0) == (513, 256, 257)
    blk = ctx.export_block(0, 0, 0)
    assert np.array_equal(blk["key_indices"], g["key_indices"])
    assert np.array_equal(blk["nf4_scale"], g["key_scale"])
    assert np.array_equal(blk["nf4_mean"], g["key_mean"])
    if frac > 0:
        assert np.array_equal(blk["outlier_idx"], g["outlier_idx"])
        assert np.array_equal(blk["outlier_val"].view(np.uint16), g["outlier_val"].view(np.uint16))
    keys, _ = ctx.dequant(0, 0, 0, 256, values=False)
    assert np.array_equal(keys.cpu().numpy(), g["key_dequant"])


@pytest.mark.parametrize("name,mode,vb", [("cache_uniform.npz", "uniform", 4),
                                          ("cache_nf4_gqa.npz", "nf4", 3),
                                          ("cache_sparse_zp.npz", "nf4_asym", 3),
                                          ("cache_bias_zp.npz", "nf4_asym", 3)])
def test_other_key_grids_cache_and_decode(torch_cuda, name, mode, vb):
    """Caches in the other key grids: every cold container equals the reference's and the
    decode on codes (both kernels) matches its dequantise-then-attend output."""
    torch = torch_cuda
    g = load_golden(name)
    k, v, q = g["k"], g["v"], g["q"]
    h, hq = k.shape[1], q.shape[0]
    ctx = _ctx(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=hq, value_bits=vb,
               hot_window=int(g["hot_window"]), max_tokens_per_seq=1280,
               kv_dtype=_np_dtype_name(k), key_mode=mode, seed=int(g["seed"]), pi=g["pi"],
               key_mean_mask=g["dc_mask"] if "dc_mask" in g else None)
    if "k_bias" in g:  # the "bias" zero-point: one given mean per block index
        from turboquant_pro_b200.autoconfig import rope_averaged_bias

        f = ctx.block_tokens
        ctx.set_key_bias_means(np.stack([rope_averaged_bias(g["k_bias"], 10000.0, 128, b * f, f)
                                         for b in range(ctx.geom.max_blocks)]))
    ctx.append(0, _dev(torch, k)[None], _dev(torch, v)[None])
    assert ctx.lengths(0, 0)[0] == int(g["length"])
    for i in range(int(g["n_blocks"])):
        blk = ctx.export_block(0, 0, i)
        assert np.array_equal(blk["key_indices"], g[f"b{i}_key_indices"])
        assert np.array_equal(blk["nf4_scale"], g[f"b{i}_nf4_scale"])
        assert np.array_equal(blk["nf4_mean"], g[f"b{i}_nf4_mean"])
        assert np.array_equal(blk["outlier_idx"], g[f"b{i}_outlier_idx"])
        assert np.array_equal(blk["value_indices"], g[f"b{i}_value_indices"])
    keys, vals = ctx.dequant(0, 0, 0, int(g["length"]))
    assert np.array_equal(keys.cpu().numpy()[0], g["keys_head0"])
    qq = _dev(torch, q)[None]
    got = ctx.decode(0, qq)[0].cpu().numpy()
    assert np.allclose(got, g["attn"], rtol=RTOL, atol=ATOL), np.abs(got - g["attn"]).max()
    ctx.set_kernel("general")
    gen = ctx.decode(0, qq)[0].cpu().numpy()
    assert np.allclose(gen, g["attn"], rtol=RTOL, atol=ATOL), np.abs(gen - g["attn"]).max()
    cold, hot = ctx.memory_stats(0, 0)
    assert cold == g["memory_stats"][0] and hot == g["memory_stats"][1]


def test_facade_key_grid_flags(torch_cuda):
    """The reference's constructor flags select the grid: neither flag = uniform,
    key_nf4 = symmetric NF4, key_nf4_asym = asymmetric NF4."""
    from turboquant_pro_b200 import AutoConfig, TurboQuantKVCache

    assert TurboQuantKVCache(head_dim=128, n_heads=2, bits=4, max_tokens=64).key_mode == "uniform"
    assert TurboQuantKVCache(head_dim=128, n_heads=2, bits=4, key_nf4=True,
                             max_tokens=64).key_mode == "nf4"
    assert TurboQuantKVCache.robust(128, 2, max_tokens=64).key_mode == "nf4_asym"
    c = AutoConfig.from_pretrained("llama-3-8b").build_cache(robust=False, hot_window=32,
                                                             max_tokens=64)
    assert c.key_mode == "uniform" and c.key_outlier_frac == 0.0


def test_export_blob_equals_reference_blob(torch_cuda):
    """A block exported from the device in the wire format of the reference's vLLM connector
    carries the same arrays and scalars as the blob the reference wrote for the same tokens."""
    torch = torch_cuda
    from turboquant_pro_b200.kv_blob import blob_to_block

    g = load_golden("blob_ref.npz")
    k, v = g["k"], g["v"]
    ctx = _ctx(n_layers=1, n_seqs=1, n_kv_heads=2, value_bits=3, hot_window=int(g["hot_window"]),
               max_tokens_per_seq=64, kv_dtype="float32", seed=int(g["seed"]), pi=g["pi"])
    ctx.append(0, _dev(torch, k)[None], _dev(torch, v)[None])
    ref = blob_to_block(g["blob"].tobytes())
    got = blob_to_block(ctx.export_blob(0, 0, 0))
    assert got["header"] == ref["header"]
    for part in ("key", "value"):
        assert sorted(got[part]) == sorted(ref[part])
        for name, want in ref[part].items():
            if isinstance(want, np.ndarray):
                assert got[part][name].dtype == want.dtype, name
                assert np.array_equal(got[part][name], want), name
            else:
                assert got[part][name] == want, name

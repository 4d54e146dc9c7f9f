"""Parity at the shapes of the benchmark configurations (through the C ABI).

Config 0 runs at full size against the CPU oracle.  The larger configurations are checked
at reduced batch / layer counts with the same per-sequence geometry, bit-exactly for the
encoders on sampled blocks and, where the oracle would take too long, through
size-independent properties: the tensor-core kernel against the general-shape kernel,
sequence-split partials against the full decode, bulk appends against token-by-token appends.
"""

from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 2e-3


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    return torch


def _c_oracle_cache(k, v, h, vb, w, pi):
    """Cold blocks + hot tokens of one sequence through the C restatement (fast)."""
    from oracle import c_oracle as co
    from oracle import tq_oracle as orc

    f = orc.block_tokens(w)
    n = k.shape[0]
    nb = orc.n_cold_blocks(n, w)
    cent, bnd = orc.value_tables(128, vb)
    pi_t = np.ascontiguousarray(pi.T)
    kout = orc.outlier_count(f, 0.02)
    kb, vbk = [], []
    for b in range(nb):
        xs = np.ascontiguousarray(np.moveaxis(k[b * f:(b + 1) * f], 0, 1), dtype=np.float32)
        vs = np.ascontiguousarray(np.moveaxis(v[b * f:(b + 1) * f], 0, 1), dtype=np.float32)
        kb.append(co.encode_keys(xs, kout))
        vbk.append(co.encode_values(vs, pi_t, bnd))
    keys = [co.dequant_keys(b["codes"], b["scale"], b["mean"], b["out_idx"], b["out_val"])
            for b in kb]
    vals = [co.dequant_values(b["codes"], b["norms"], cent, pi) for b in vbk]
    keys.append(np.moveaxis(k[nb * f:], 0, 1).astype(np.float32))
    vals.append(np.moveaxis(v[nb * f:], 0, 1).astype(np.float32))
    return kb, vbk, np.concatenate(keys, axis=1), np.concatenate(vals, axis=1)


def _check_export(blk, kb, vb_blk, vb):
    from oracle import tq_oracle as orc

    assert np.array_equal(blk["key_indices"], orc.pack_key_codes(kb["codes"]))
    assert np.array_equal(blk["nf4_scale"][0], kb["scale"])
    assert np.array_equal(blk["nf4_mean"][0], kb["mean"])
    assert np.array_equal(blk["outlier_idx"], kb["out_idx"])
    assert np.array_equal(blk["outlier_val"].view(np.uint16), kb["out_val"].view(np.uint16))
    assert np.array_equal(blk["value_indices"], orc.pack_value_codes(vb_blk["codes"], vb))
    assert np.array_equal(blk["value_norms"][0], vb_blk["norms"])


def test_config0_full_size(torch_cuda):
    """MHA 32 heads x 128, batch 1, context 4096, robust() K4/V4, hot window 512, fp32 K/V:
    every cold block bit-exact, decode within tolerance of dequantise-then-attend."""
    torch = torch_cuda
    from oracle import c_oracle as co
    from turboquant_pro_b200 import TurboQuantKVCache
    from turboquant_pro_b200.synth import make_kv, make_q

    h, n, w, vb, seed = 32, 4096, 512, 4, 0
    k, v = make_kv(seed, h, n)
    q = make_q(seed, h)
    cache = TurboQuantKVCache.robust(head_dim=128, n_heads=h, hot_window=w, seed=seed,
                                     max_tokens=n + 8)
    cache.append_many(k, v)
    assert (cache.length, cache.cold_length, cache.hot_length) == (4096, 3584, 512)
    ctx = cache.context
    kb, vbk, keys, vals = _c_oracle_cache(k, v, h, vb, w, ctx.pi)
    assert len(kb) == 14
    for i in range(14):
        _check_export(ctx.export_block(0, 0, i), kb[i], vbk[i], vb)
    want = co.attention(q, keys, vals)
    got = cache.fused_decode(q)
    err = np.abs(got - want).max()
    assert np.allclose(got, want, rtol=RTOL, atol=ATOL), f"max abs err {err}"
    # the getters return the same dequantised tensors as the oracle, bit for bit
    assert np.array_equal(cache.get_keys(0, n)[0], keys)
    assert np.array_equal(cache.get_values(0, n)[0], vals)
    st = cache.memory_stats()
    assert st["hot_bytes"] == 2 * 512 * h * 128 * 4
    assert 3.5 < st["effective_ratio"] < 4.5


def test_config1_shape_reduced_batch(torch_cuda):
    """Llama-3-8B shape (32 q / 8 KV heads, K4/V3, fp16 K/V, bf16 q, context 8192) with 2
    layers and 3 sequences: encoders bit-exact on sampled blocks, decode within tolerance."""
    torch = torch_cuda
    from oracle import c_oracle as co
    from turboquant_pro_b200 import AutoConfig
    from turboquant_pro_b200.synth import make_kv, make_q

    cfg = AutoConfig.from_pretrained("llama-3-8b")
    L, B, n = 2, 3, 8192
    ctx = cfg.build_context(n_seqs=B, max_tokens_per_seq=n, n_layers=L, seed=4)
    data = {}
    for layer in range(L):
        ks, vs = [], []
        for s in range(B):
            k, v = make_kv(100 * layer + s, 8, n, dtype=np.float16)
            data[(layer, s)] = (k, v)
            ks.append(k)
            vs.append(v)
        ctx.append(layer, torch.from_numpy(np.stack(ks)).cuda(), torch.from_numpy(np.stack(vs)).cuda())
    assert ctx.lengths(1, 2) == (8192, 7680, 512)
    for layer, s in ((0, 0), (1, 2)):
        k, v = data[(layer, s)]
        kb, vbk, keys, vals = _c_oracle_cache(k.astype(np.float32), v.astype(np.float32), 8, 3,
                                              512, ctx.pi)
        for i in (0, 13, 29):
            _check_export(ctx.export_block(layer, s, i), kb[i], vbk[i], 3)
        q = np.stack([make_q(9 + j, 32) for j in range(B)])
        qd = torch.from_numpy(q).cuda().to(torch.bfloat16)
        out = ctx.decode(layer, qd).cpu().numpy()
        want = co.attention(qd[s].float().cpu().numpy(), keys, vals)
        err = np.abs(out[s] - want).max()
        assert np.allclose(out[s], want, rtol=RTOL, atol=ATOL), f"max abs err {err}"
    assert ctx.status() == 0


def test_config2_long_context_split(torch_cuda):
    """One sequence of 131072 tokens (510 blocks + 512 hot), Llama-3-8B shape: the decode
    equals the general-shape kernel, and 1/2/4/8-way sequence splits merged by the LSE
    combine equal the unsplit result."""
    torch = torch_cuda
    from turboquant_pro_b200 import AutoConfig

    cfg = AutoConfig.from_pretrained("llama-3-8b")
    n = 131072
    ctx = cfg.build_context(n_seqs=1, max_tokens_per_seq=n, n_layers=1, seed=2)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2)
    scale = torch.exp(0.5 * torch.randn((8, 128), generator=gen, device="cuda"))
    for t0 in range(0, n, 16384):
        k = (torch.randn((1, 16384, 8, 128), generator=gen, device="cuda") * scale).half()
        v = torch.randn((1, 16384, 8, 128), generator=gen, device="cuda").half()
        ctx.append(0, k, v)
    assert ctx.lengths(0, 0) == (n, 510 * 256, 512)
    q = torch.randn((1, 32, 128), generator=gen, device="cuda").to(torch.bfloat16)
    full = ctx.decode(0, q).cpu().numpy()
    ctx.set_kernel("general")
    slow = ctx.decode(0, q).cpu().numpy()
    ctx.set_kernel("auto")
    assert np.allclose(full, slow, rtol=RTOL, atol=ATOL), np.abs(full - slow).max()
    # the longest softmax of the configurations against the CPU oracle (dequantise-then-attend
    # in the C restatement) on two of the KV heads: their 8 query heads
    from oracle import c_oracle as co

    for head in (0, 5):
        kd, vd = ctx.dequant(0, 0, 0, n)
        keys = kd[head:head + 1].cpu().numpy()
        vals = vd[head:head + 1].cpu().numpy()
        del kd, vd
        qh = q[0, 4 * head:4 * head + 4].float().cpu().numpy()
        want = co.attention(qh, keys, vals)
        got = full[0, 4 * head:4 * head + 4]
        assert np.allclose(got, want, rtol=RTOL, atol=ATOL), (head, np.abs(got - want).max())
    for world in (2, 4, 8):
        parts = [ctx.decode_partial(0, q, 510 * r // world, 510 * (r + 1) // world,
                                    with_hot=(r == world - 1)).clone() for r in range(world)]
        merged = ctx.lse_combine(torch.stack(parts).reshape(world, 32, 130)).cpu().numpy()
        assert np.allclose(merged, full[0], rtol=1e-3, atol=1e-4), (world,
                                                                     np.abs(merged - full[0]).max())
    assert ctx.status() == 0


def test_config3_shape_ragged_group8(torch_cuda):
    """Llama-3-70B shape sharded to one KV head per rank (8 q heads on 1 KV head, K4/V4),
    ragged contexts in [1024, 32768]: tensor-core kernel == general kernel == oracle."""
    torch = torch_cuda
    from oracle import c_oracle as co
    from turboquant_pro_b200 import AutoConfig
    from turboquant_pro_b200.synth import make_kv, make_q

    cfg = AutoConfig.from_pretrained("llama-3-70b", target="quality")
    assert (cfg.key_bits, cfg.value_bits, cfg.n_q_heads, cfg.n_kv_heads) == (4, 4, 64, 8)
    rng = np.random.default_rng(3)
    lens = [1024, 32768] + rng.integers(1024, 32769, size=4).tolist()
    ctx = cfg.build_context(n_seqs=len(lens), max_tokens_per_seq=32768, n_layers=1, seed=6,
                            n_kv_heads=1)  # this rank's shard: 1 KV head, its 8 q heads
    assert ctx.n_q_heads == 8
    data = []
    for s, n in enumerate(lens):
        k, v = make_kv(700 + s, 1, n, dtype=np.float16)
        data.append((k, v))
        ctx.append(0, torch.from_numpy(k)[None].cuda(), torch.from_numpy(v)[None].cuda(),
                   seq_begin=s)
    q = np.stack([make_q(80 + s, 8) for s in range(len(lens))])
    qd = torch.from_numpy(q).cuda().to(torch.bfloat16)
    fast = ctx.decode(0, qd).cpu().numpy()
    ctx.set_kernel("general")
    slow = ctx.decode(0, qd).cpu().numpy()
    ctx.set_kernel("auto")
    assert np.allclose(fast, slow, rtol=RTOL, atol=ATOL), np.abs(fast - slow).max()
    for s in (0, 2):
        k, v = data[s]
        kb, vbk, keys, vals = _c_oracle_cache(k.astype(np.float32), v.astype(np.float32), 1, 4,
                                              512, ctx.pi)
        _check_export(ctx.export_block(0, s, len(kb) - 1), kb[-1], vbk[-1], 4)
        want = co.attention(qd[s].float().cpu().numpy(), keys, vals)
        assert np.allclose(fast[s], want, rtol=RTOL, atol=ATOL), np.abs(fast[s] - want).max()
    assert ctx.status() == 0


def test_config4_prefill_then_decode_appends(torch_cuda):
    """Prefill-append of 16384 tokens followed by 256 single-token appends (one flush happens
    on the way): identical blocks to a token-by-token oracle, bit for bit."""
    torch = torch_cuda
    from turboquant_pro_b200 import AutoConfig
    from turboquant_pro_b200.synth import make_kv

    cfg = AutoConfig.from_pretrained("llama-3-8b")
    B, n0, steps = 2, 16384, 256
    ctx = cfg.build_context(n_seqs=B, max_tokens_per_seq=n0 + steps, n_layers=1, seed=8)
    ks, vs = zip(*[make_kv(900 + s, 8, n0 + steps, dtype=np.float16) for s in range(B)])
    k_all, v_all = torch.from_numpy(np.stack(ks)).cuda(), torch.from_numpy(np.stack(vs)).cuda()
    ctx.append(0, k_all[:, :n0], v_all[:, :n0])
    assert ctx.lengths(0, 0) == (n0, 62 * 256, 512)
    for t in range(n0, n0 + steps):
        ctx.append(0, k_all[:, t:t + 1], v_all[:, t:t + 1])
    assert ctx.lengths(0, 1) == (n0 + steps, 63 * 256, 512)
    kb, vbk, _, _ = _c_oracle_cache(ks[1].astype(np.float32), vs[1].astype(np.float32), 8, 3, 512,
                                    ctx.pi)
    assert len(kb) == 63
    for i in (0, 31, 61, 62):  # 62 is the block flushed during the single-token appends
        _check_export(ctx.export_block(0, 1, i), kb[i], vbk[i], 3)
    assert ctx.status() == 0


def test_page_wide_channel_side_codes(torch_cuda):
    """The page header names the four channels with the largest scale (ties to the lower
    channel) and repeats their codes token by token; both must agree with the oracle's
    scales and codes, since the tensor-core kernel corrects its scores from them."""
    torch = torch_cuda
    from oracle import tq_oracle as orc
    from turboquant_pro_b200 import KVContext
    from turboquant_pro_b200.synth import make_kv

    h, n, w = 2, 1100, 512
    k, v = make_kv(21, h, n, dtype=np.float16)
    k[:600, 0, 7] = k[:600, 0, 3]  # equal scales on two channels of the first block
    ctx = KVContext(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=h, value_bits=3,
                    hot_window=w, max_tokens_per_seq=n, kv_dtype="float16", seed=21)
    ctx.append(0, torch.from_numpy(k)[None].cuda(), torch.from_numpy(v)[None].cuda())
    torch.cuda.synchronize()
    g = ctx.geom
    f = g.block_tokens
    nb = orc.n_cold_blocks(n, w)
    assert nb >= 2
    pages = ctx._regions["pages"].cpu().numpy()
    for head in range(h):
        for b in range(nb):
            enc = orc.encode_keys(np.moveaxis(k[b * f:(b + 1) * f, head:head + 1], 0, 1), 0.02)
            scale, codes = enc["scale"][0], enc["codes"][0]
            order = np.lexsort((np.arange(128), -scale.astype(np.float64)))[:4]
            off = (head * g.max_blocks + b) * g.page_bytes + g.hdr_off
            assert pages[off + 8:off + 12].tolist() == order.tolist()
            side = pages[off + 64:off + 64 + 2 * f].view(np.uint16)
            want = sum(codes[:, order[i]].astype(np.uint16) << (4 * i) for i in range(4))
            assert np.array_equal(side, want)


def test_heavy_tokens_overflow_and_spill(torch_cuda):
    """Tokens that are outliers on many channels at once: more entries than a token's fixed
    slots in the page (overflow list) and more than the page's overflow list holds (the kernel
    then reads the pool's list).  Tensor-core kernel == general kernel == oracle, and two
    calls give identical bits."""
    torch = torch_cuda
    from oracle import tq_oracle as orc
    from turboquant_pro_b200 import KVContext
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp, n, w, vb = 2, 4, 1100, 512, 3
    k, v = make_kv(33, h, n, dtype=np.float16)
    k = k.astype(np.float32)

    def boost(tok, head, chans):
        # the largest magnitude of its block on every given channel: certainly an outlier
        b0 = tok // 256 * 256
        k[tok, head, chans] = 1.5 * np.abs(k[b0:b0 + 256, head, chans]).max(axis=0)

    boost(5, 0, slice(None))          # block 0, head 0: one token on all 128 channels -> spill
    boost(300, 0, slice(0, 20))       # block 1, head 0: two tokens of one strip, 20 channels each
    boost(301, 0, slice(10, 30))
    boost(256 + 200, 0, slice(90, 102))  # and one token of the last strip
    boost(100, 1, slice(0, 128, 3))   # head 1, block 0: 43 channels on one token
    k = k.astype(np.float16)
    q = make_q(33, h * grp)
    ctx = KVContext(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=h * grp, value_bits=vb,
                    hot_window=w, max_tokens_per_seq=n, kv_dtype="float16", seed=33)
    ctx.append(0, torch.from_numpy(k)[None].cuda(), torch.from_numpy(v)[None].cuda())
    torch.cuda.synchronize()
    g = ctx.geom
    pages = ctx._regions["pages"].cpu().numpy()
    flags = {}
    for head in range(h):
        for b in range(2):
            off = (head * g.max_blocks + b) * g.page_bytes + g.hdr_off
            hdr = pages[off:off + 64]
            flags[(head, b)] = (int(hdr[12:14].view(np.uint16)[0]), int(hdr[14:16].view(np.uint16)[0]))
    assert flags[(0, 0)][1] == 1                      # spilled
    assert flags[(0, 1)][1] == 0 and flags[(0, 1)][0] >= 40   # overflow list in use
    assert flags[(1, 0)][1] == 0 and flags[(1, 0)][0] >= 30
    kb, vbk, kk, vv = _c_oracle_cache(k, v, h, vb, w, ctx.pi)
    want = orc.attention(q, kk, vv)
    qq = torch.from_numpy(q)[None].cuda()
    got = ctx.decode(0, qq)[0].cpu().numpy()
    again = ctx.decode(0, qq)[0].cpu().numpy()
    assert ctx.last_launches() == 2
    assert np.array_equal(got, again)
    ctx.set_kernel("general")
    gen = ctx.decode(0, qq)[0].cpu().numpy()
    ctx.set_kernel("auto")
    assert np.allclose(got, want, rtol=RTOL, atol=ATOL), np.abs(got - want).max()
    assert np.allclose(got, gen, rtol=RTOL, atol=ATOL), np.abs(got - gen).max()
    assert ctx.status() == 0


@pytest.mark.parametrize("seed", range(10))
def test_random_geometries_kernels_agree(torch_cuda, seed):
    """Randomised geometry (sequences, heads, GQA group, value bits, element type, ragged
    lengths incl. empty and hot-only sequences, appended in random chunks): the tensor-core
    kernel, the general kernel and sequence-split partials give the same attention."""
    torch = torch_cuda
    from turboquant_pro_b200 import KVContext
    from turboquant_pro_b200.synth import make_kv, make_q

    rng = np.random.default_rng(1000 + seed)
    n_seqs, h = int(rng.integers(1, 5)), int(rng.integers(1, 4))
    grp = int(rng.choice([1, 2, 4, 8]))
    vb = int(rng.choice([3, 4]))
    dt = str(rng.choice(["float16", "bfloat16", "float32"]))
    mode = str(rng.choice(["nf4_asym", "nf4", "uniform"]))
    lens = [int(rng.choice([0, int(rng.integers(1, 513)), int(rng.integers(513, 2600))]))
            for _ in range(n_seqs)]
    if max(lens) == 0:
        lens[0] = 700
    ctx = KVContext(n_layers=1, n_seqs=n_seqs, n_kv_heads=h, n_q_heads=h * grp, value_bits=vb,
                    hot_window=512, max_tokens_per_seq=2600, kv_dtype=dt, key_mode=mode,
                    seed=seed)
    tdt = getattr(torch, dt)
    for s, n in enumerate(lens):
        if n == 0:
            continue
        k, v = make_kv(2000 + 10 * seed + s, h, n, dtype=np.float32)
        pos = 0
        while pos < n:  # random chunks, some of them single tokens
            step = int(rng.choice([1, int(rng.integers(1, 700))]))
            kt = torch.from_numpy(k[pos:pos + step]).to(tdt)[None].cuda()
            vt = torch.from_numpy(v[pos:pos + step]).to(tdt)[None].cuda()
            ctx.append(0, kt, vt, seq_begin=s)
            pos += step
    assert [ctx.lengths(0, s)[0] for s in range(n_seqs)] == lens
    q = torch.from_numpy(np.stack([make_q(3000 + seed + s, h * grp) for s in range(n_seqs)])).cuda()
    fast = ctx.decode(0, q).cpu().numpy()
    ctx.set_kernel("general")
    slow = ctx.decode(0, q).cpu().numpy()
    ctx.set_kernel("auto")
    assert ctx.status() == 0
    assert np.allclose(fast, slow, rtol=RTOL, atol=ATOL), np.abs(fast - slow).max()
    for s, n in enumerate(lens):
        if n == 0:
            assert not fast[s].any()
    # two ranges of cold blocks + the hot window, merged, equal the full decode
    nb = max(ctx.lengths(0, s)[1] for s in range(n_seqs)) // 256
    cut = nb // 2
    parts = torch.stack([ctx.decode_partial(0, q, 0, cut, False),
                         ctx.decode_partial(0, q, cut, 1 << 20, True)])
    merged = ctx.lse_combine(parts.reshape(2, n_seqs * h * grp, 130)).cpu().numpy()
    live = np.repeat(np.asarray(lens) > 0, h * grp)
    assert np.allclose(merged[live], fast.reshape(-1, 128)[live], rtol=1e-3, atol=1e-4)


def test_many_units_take_the_tensor_core_kernel(torch_cuda):
    """More (sequence, KV head) units than one launch's plan holds (65 sequences x 8 KV heads =
    520): the layer is served by several launches of the tensor-core kernel, not by the
    general-shape one, and both kernels agree."""
    torch = torch_cuda
    from turboquant_pro_b200 import KVContext

    B, h, grp = 65, 8, 4
    ctx = KVContext(n_layers=1, n_seqs=B, n_kv_heads=h, n_q_heads=h * grp, value_bits=3,
                    hot_window=512, max_tokens_per_seq=1400, kv_dtype="float16", seed=6)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(6)
    lens = [int(x) for x in torch.randint(1, 1400, (B,), generator=gen, device="cuda").cpu()]
    lens[3], lens[64] = 1400, 1337  # a long one in each launch
    for s0 in range(B):
        k = torch.randn((1, lens[s0], h, 128), generator=gen, device="cuda").half()
        v = torch.randn((1, lens[s0], h, 128), generator=gen, device="cuda").half()
        ctx.append(0, k, v, seq_begin=s0)
    q = torch.randn((B, h * grp, 128), generator=gen, device="cuda").to(torch.bfloat16)
    fast = ctx.decode(0, q).cpu().numpy()
    assert ctx.last_kernel() == "tensor-core"
    assert ctx.last_launches() == 4  # two attention launches, two combines
    ctx.set_kernel("general")
    slow = ctx.decode(0, q).cpu().numpy()
    assert ctx.last_kernel() == "general"
    assert np.allclose(fast, slow, rtol=RTOL, atol=ATOL), np.abs(fast - slow).max()
    assert ctx.status() == 0


def test_decode_bits_depend_on_the_tokens_only(torch_cuda):
    """Two encodes of the same tokens (separate contexts, different append chunking) give the
    same page images, so the decode outputs are equal bit for bit."""
    torch = torch_cuda
    from turboquant_pro_b200 import KVContext
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp, n = 2, 4, 2100
    k, v = make_kv(77, h, n, dtype=np.float16)
    kt, vt = torch.from_numpy(k)[None].cuda(), torch.from_numpy(v)[None].cuda()
    kw = dict(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=h * grp, value_bits=3, hot_window=512,
              max_tokens_per_seq=n, kv_dtype="float16", seed=77)
    a, b = KVContext(**kw), KVContext(**kw)
    a.append(0, kt, vt)
    for t0 in range(0, n, 333):
        b.append(0, kt[:, t0:t0 + 333], vt[:, t0:t0 + 333])
    q = torch.from_numpy(make_q(77, h * grp))[None].cuda()
    assert torch.equal(a.decode(0, q), b.decode(0, q))
    a.set_kernel("general")
    b.set_kernel("general")
    assert torch.equal(a.decode(0, q), b.decode(0, q))


def test_wait_that_runs_out_is_reported_and_leaves_the_context_usable(torch_cuda):
    """The bounded waits of the tensor-core kernel: the test hook withholds the copy of one
    tile (nothing else is disturbed) and shortens the probe limit; the kernel returns, the
    status word carries bit 1, ``check_status`` raises, and the next decode is correct."""
    torch = torch_cuda
    from turboquant_pro_b200 import KVContext
    from turboquant_pro_b200._lib import TqError
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp, n = 2, 4, 3000
    k, v = make_kv(8, h, n, dtype=np.float16)
    ctx = KVContext(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=h * grp, value_bits=3,
                    hot_window=512, max_tokens_per_seq=n, kv_dtype="float16", seed=8)
    ctx.append(0, torch.from_numpy(k)[None].cuda(), torch.from_numpy(v)[None].cuda())
    q = torch.from_numpy(make_q(8, h * grp))[None].cuda()
    good = ctx.decode(0, q).clone()
    assert ctx.last_kernel() == "tensor-core" and ctx.status() == 0
    ctx.debug_wait(wait_limit=64, withhold_tile=0)
    with pytest.raises(TqError, match="wait"):
        ctx.decode(0, q, check_status=True)
    assert ctx.status() == 0  # reading the flags cleared them
    ctx.decode(0, q)
    torch.cuda.synchronize()
    assert ctx.status() & 2
    ctx.debug_wait()  # defaults: nothing withheld
    again = ctx.decode(0, q, check_status=True)
    assert torch.equal(again, good)

"""Multi-rank logic of the sequence split on CPU ranks (gloo, world size 2): the block
partition, the all-gather of (m, l, o) states in rank order and the LSE merge reproduce
single-rank attention.  The states come from the CPU oracle; the merge is restated in
torch so that no GPU is needed."""

from __future__ import annotations

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import tq_oracle as orc
        from turboquant_pro_b200.parallel import gather_states, split_blocks
        from turboquant_pro_b200.synth import make_kv, make_q

        h, grp, n, w = 2, 2, 150, 16
        k, v = make_kv(4, h, n)
        q = make_q(4, h * grp)
        cache = orc.OracleCache(128, h, 4, 3, w, 0.02, seed=4)
        for t in range(n):
            cache.append(k[t], v[t])
        keys, vals = cache.keys(), cache.values()
        f = orc.block_tokens(w)
        nb = len(cache.cold_k)
        lo, hi, with_hot = split_blocks(nb, rank, world)
        assert with_hot == (rank == world - 1)
        t0, t1 = lo * f, (hi * f if not with_hot else n)
        scale = 1.0 / np.sqrt(128.0)
        if t1 > t0:
            m, l, acc = orc.partials(q, keys[:, t0:t1], vals[:, t0:t1], scale)
        else:
            m = np.full(h * grp, -np.inf, np.float32)
            l = np.zeros(h * grp, np.float32)
            acc = np.zeros((h * grp, 128), np.float32)
        mlo = torch.from_numpy(np.concatenate([m[:, None], l[:, None], acc], axis=1).astype(np.float32))
        g = gather_states(mlo)
        assert g.shape == (world, h * grp, 130)
        assert torch.equal(g[rank], mlo)
        big = g[:, :, 0].max(dim=0).values
        wgt = torch.exp(g[:, :, 0] - big)
        out = (g[:, :, 2:] * wgt[:, :, None]).sum(0) / (g[:, :, 1] * wgt).sum(0)[:, None]
        want = cache.attend(q)
        ok = np.allclose(out.numpy(), want, rtol=1e-4, atol=1e-5)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sequence_split_two_ranks():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_shard_ranges_cover_everything():
    from turboquant_pro_b200.parallel import shard_range, split_blocks

    for n in (0, 1, 7, 30, 510):
        for world in (1, 2, 4, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert [split_blocks(n, r, world)[2] for r in range(world)] == \
                [False] * (world - 1) + [True]
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_sequence_shard_gives_each_rank_exactly_its_blocks():
    """Sharded storage of the sequence split: the tokens a rank feeds to its own cache make
    that cache flush exactly the rank's range of the sequence's cold blocks (the reference's
    flush rule applied to the rank's tokens), the ranges tile the sequence's blocks, token
    ranges start on block boundaries, and only the last rank holds the hot window."""
    from turboquant_pro_b200.parallel import n_cold_blocks, sequence_shard, shard_range

    for w in (512, 16, 7, 5):
        f = (w + 1) // 2
        for n in (0, 3, w, w + 1, w + 2, 3000, 8192, 131072, 131071):
            nb = n_cold_blocks(n, w)
            for world in (1, 2, 3, 4, 8):
                total = 0
                for r in range(world):
                    lo, hi, k, with_hot = sequence_shard(n, w, r, world)
                    b_lo, b_hi = shard_range(nb, r, world)
                    assert k == b_hi - b_lo and lo == b_lo * f and hi <= n
                    assert n_cold_blocks(hi - lo, w) == k  # what the rank's cache will flush
                    assert with_hot == (r == world - 1)
                    if with_hot:
                        assert hi == n  # the last rank stores through the end of the sequence
                    total += k
                assert total == nb

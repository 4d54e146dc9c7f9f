"""Multi-GPU layer: one process per GPU, ``torch.distributed`` for the plumbing.

The decode path shards in three ways, two of which need no communication at all:

* **batch shard** — sequences are split over ranks; every rank holds all layers and heads
  of its sequences.  No collective on the attention path.
* **KV-head shard** — rank r owns a contiguous range of KV heads (and their query
  heads) for every sequence.  No collective inside attention (the output stays
  head-sharded for the projection that follows).
* **sequence split** — one long sequence; rank r attends a contiguous range of cold
  blocks, the last rank also attends the hot window.  Each rank produces the
  un-normalised state ``(m, l, o[D])`` per query head, one ``all_gather`` moves the
  states into every rank's local memory, and the LSE-combine kernel merges them in rank
  order (``merge_partials``, ``turboquant_pro/kv_fused.py:139-153``, is associative up
  to rounding; a fixed order makes the result reproducible).  No kernel reads another
  GPU's memory.

The reference has no multi-GPU path; this module is new design around its partial-merge
algebra.
"""

from __future__ import annotations


def shard_range(n_items: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced ``[lo, hi)`` share of ``n_items`` for ``rank``."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank / world size")
    return n_items * rank // world, n_items * (rank + 1) // world


def split_blocks(n_blocks: int, rank: int, world: int) -> tuple[int, int, bool]:
    """Sequence-split share of ``rank``: cold blocks ``[lo, hi)`` and whether this rank
    also attends the hot window (the last rank does — it is where new tokens arrive)."""
    lo, hi = shard_range(n_blocks, rank, world)
    return lo, hi, rank == world - 1


def gather_states(mlo, group=None):
    """All-gather per-rank states ``[rows, 2 + D]`` into ``[world, rows, 2 + D]`` in rank
    order.  Works on any backend (NCCL on GPUs, gloo on CPU)."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    flat = mlo.contiguous().reshape(-1)
    out = torch.empty(world * flat.numel(), dtype=mlo.dtype, device=mlo.device)
    dist.all_gather_into_tensor(out, flat, group=group)
    return out.reshape((world,) + tuple(mlo.shape))


class SequenceSplitDecoder:
    """Decode step of one long sequence whose cold blocks are split over the ranks of a
    process group.

    Every rank holds a :class:`KVContext` with the same geometry and the same appended
    tokens' bookkeeping; rank r reads only its block range during decode, so the HBM
    traffic per rank is ``1 / world`` of the sequence.
    """

    def __init__(self, ctx, group=None):
        import torch.distributed as dist

        self.ctx = ctx
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def decode(self, layer: int, q):
        """``q``: ``[n_seqs, n_q_heads, D]`` replicated on every rank.  Returns the full
        attention output ``[n_seqs, n_q_heads, D]`` on every rank."""
        ctx = self.ctx
        n_blocks = max(ctx.lengths(layer, s)[1] for s in range(ctx.n_seqs)) // ctx.block_tokens
        lo, hi, with_hot = split_blocks(n_blocks, self.rank, self.world)
        mlo = ctx.decode_partial(layer, q, lo, hi, with_hot)
        rows = mlo.shape[0] * mlo.shape[1]
        gathered = gather_states(mlo.reshape(rows, mlo.shape[2]), self.group)
        out = ctx.lse_combine(gathered)
        return out.reshape(mlo.shape[0], mlo.shape[1], -1)

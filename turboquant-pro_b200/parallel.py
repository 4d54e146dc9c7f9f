"""Multi-GPU layer: one process per GPU, ``torch.distributed`` for the plumbing.

The decode path shards in three ways, two of which need no communication at all:

* **batch shard** — sequences are split over ranks; every rank holds all layers and heads
  of its sequences.  No collective on the attention path.
* **KV-head shard** — rank r owns a contiguous range of KV heads (and their query
  heads) for every sequence.  No collective inside attention (the output stays
  head-sharded for the projection that follows).
* **sequence split** — one long sequence; rank r attends a contiguous range of cold
  blocks, the last rank also attends the hot window.  Each rank produces the
  un-normalised state ``(m, l, o[D])`` per query head; the states reach every rank's
  local memory and are merged there in rank order (``merge_partials``,
  ``turboquant_pro/kv_fused.py:139-153``, is associative up to rounding; a fixed order makes
  the result reproducible).  Two transports: :class:`PeerExchange` — one kernel per step
  that stores the rows into every rank's memory with peer stores over NVLink, signals,
  waits (bounded) and merges — or, where peer mappings are not to be had, one NCCL
  ``all_gather`` followed by the LSE-combine kernel.  Both give the same bits.  No kernel
  reads another GPU's memory; the exchange kernel writes to it.

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


class PeerExchange:
    """The (m, l, o) states of a sequence split, exchanged and merged by one kernel per call.

    One object per rank of ``group`` (one process per GPU): the constructor allocates the
    rank's region through the library, trades CUDA IPC handles with the other ranks
    (an ``all_gather`` of 64 bytes), maps their regions and ends with a barrier.
    ``gather_merge(mlo)`` then equals ``lse_combine(gather_states(mlo))`` bit for bit, with no
    collective call: rows travel as peer stores over NVLink and a rank waits only for the rows
    it merges.  Every rank must make the same sequence of calls.  A wait that runs out (a rank
    that never arrives) raises ``RuntimeError`` at the next :meth:`check`.
    """

    def __init__(self, rows: int, head_dim: int = 128, device=None, group=None):
        import ctypes as C

        import torch
        import torch.distributed as dist

        from ._lib import check, load

        self._lib = load()
        self._check = check
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.rows = int(rows)
        self.head_dim = int(head_dim)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        # Every rank takes part in every collective call below whether or not its own set-up
        # succeeded, and all ranks then raise together or none does.
        self._h = None
        ok, mine = 1, (C.c_uint8 * 64)()
        try:
            h = C.c_void_p()
            check(self._lib.tq_xchg_create(self.device.index, self.rank, self.world, self.rows,
                                           self.head_dim, C.byref(h)))
            self._h = h
            check(self._lib.tq_xchg_ipc_handle(self._h, mine))
        except Exception as e:  # noqa: BLE001
            ok, self._error = 0, repr(e)
        t = torch.tensor([ok] + list(bytes(mine)), dtype=torch.uint8, device=self.device)
        allh = torch.empty(self.world * 65, dtype=torch.uint8, device=self.device)
        dist.all_gather_into_tensor(allh, t, group=group)
        allh = allh.cpu().numpy().tobytes()
        ok = int(all(allh[65 * p] == 1 for p in range(self.world)))
        if ok:
            try:
                for p in range(self.world):
                    if p != self.rank:
                        buf = (C.c_uint8 * 64).from_buffer_copy(allh[65 * p + 1:65 * p + 65])
                        check(self._lib.tq_xchg_open_peer(self._h, p, buf))
            except Exception as e:  # noqa: BLE001
                ok, self._error = 0, repr(e)
        flag = torch.tensor([ok], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)  # also the barrier: every
        # region is zeroed and mapped before the first exchange
        if int(flag.item()) != 1:
            if self._h is not None:
                self._lib.tq_xchg_destroy(self._h)
                self._h = None
            raise RuntimeError("peer-memory exchange could not be set up on every rank: "
                               + getattr(self, "_error", "another rank failed"))

    def gather_merge(self, mlo, out=None, stream=None):
        """``mlo``: this rank's states ``[rows, 2 + D]`` float32 (CUDA, contiguous).  Returns
        the merged attention output ``[rows, D]``."""
        import torch

        if tuple(mlo.shape) != (self.rows, 2 + self.head_dim) or mlo.dtype != torch.float32 \
                or mlo.device != self.device or not mlo.is_contiguous():
            raise ValueError(f"expected contiguous float32 states [{self.rows}, "
                             f"{2 + self.head_dim}] on {self.device}")
        if out is None:
            out = torch.empty((self.rows, self.head_dim), dtype=torch.float32, device=self.device)
        elif tuple(out.shape) != (self.rows, self.head_dim) or out.dtype != torch.float32 \
                or out.device != self.device or not out.is_contiguous():
            raise ValueError("bad out tensor")
        st = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        with torch.cuda.device(self.device):
            self._check(self._lib.tq_xchg_gather_merge(self._h, mlo.data_ptr(), out.data_ptr(), 3,
                                                       st))
        return out

    def set_wait_limit(self, probes: int) -> None:
        self._check(self._lib.tq_xchg_set_wait_limit(self._h, int(probes)))

    def status(self) -> int:
        import ctypes as C

        import torch

        v = C.c_int32(0)
        with torch.cuda.device(self.device):
            self._check(self._lib.tq_xchg_status(
                self._h, C.byref(v), torch.cuda.current_stream(self.device).cuda_stream))
        return v.value

    def check(self) -> None:
        """Raises if a wait of an earlier exchange ran out (synchronises the stream)."""
        if self.status() & 1:
            raise RuntimeError("a rank's attention states did not arrive within the wait limit")

    def close(self) -> None:
        """Unmaps the peers and frees the region; a collective call (ends with a barrier before
        the memory goes away)."""
        import torch
        import torch.distributed as dist

        if getattr(self, "_h", None) is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
            self._lib.tq_xchg_destroy(self._h)
            self._h = None


def n_cold_blocks(n_tokens: int, hot_window: int) -> int:
    """Cold blocks of a cache holding ``n_tokens`` tokens (the reference's flush rule,
    ``turboquant_pro/core.py:1008-1014``: once the window overflows, its oldest half becomes
    a block)."""
    f = (hot_window + 1) // 2
    return 0 if n_tokens <= hot_window else 1 + (n_tokens - hot_window - 1) // f


def sequence_shard(n_tokens: int, hot_window: int, rank: int, world: int):
    """What rank ``rank`` of ``world`` stores of one sequence of ``n_tokens`` tokens under the
    sequence split: ``(tok_lo, tok_hi, n_blocks, with_hot)``.

    The sequence's cold blocks are divided into contiguous, balanced ranges.  A rank feeds
    tokens ``[tok_lo, tok_hi)`` to a cache of its own; that cache then holds exactly
    ``n_blocks`` cold blocks, and they are the global blocks of the rank's range bit for bit
    (a block is encoded from its own tokens only, and ``tok_lo`` is a block boundary).  To
    make the cache flush its last block, a rank other than the last feeds
    ``hot_window + 1 - block`` tokens beyond its range; they stay in that cache's window and
    are never attended (``with_hot`` is False).  The last rank stores everything from its
    first block to the end of the sequence: its window is the sequence's window, and new
    tokens are appended there."""
    f = (hot_window + 1) // 2
    nb = n_cold_blocks(n_tokens, hot_window)
    lo, hi = shard_range(nb, rank, world)
    if rank == world - 1:
        return lo * f, n_tokens, hi - lo, True
    if hi == lo:
        return lo * f, lo * f, 0, False
    return lo * f, hi * f + (hot_window + 1 - f), hi - lo, False


class ShardedSequenceCache:
    """Sequence split with sharded storage: every rank of the process group keeps only its own
    contiguous range of each sequence's cold blocks (plus, on the last rank, the hot window),
    in a :class:`KVContext` of its own.  Storage, encode work and decode traffic per rank are
    ``1 / world`` of the sequence; a decode step is one partial decode per rank, one
    ``all_gather`` of the ``(m, l, o)`` states and the LSE merge in rank order.

    The sequences of one cache must have the same length (a decode step attends them together).
    Tokens appended after the prefill go to the last rank, which also keeps the blocks they
    later flush into: the split is balanced at prefill time.
    """

    def __init__(self, ctx, group=None):
        import torch.distributed as dist

        self.ctx = ctx
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.n_tokens = [0] * ctx.n_layers      # global length per layer
        self.prefilled = [False] * ctx.n_layers
        self.exchange = None                    # PeerExchange, see use_peer_exchange()
        self.fused = False                      # let the merge kernel run the exchange
        self._fused = None                      # whether decode_exchange serves this geometry

    @staticmethod
    def local_capacity(n_tokens: int, hot_window: int, rank: int, world: int, extra: int = 0):
        """``max_tokens_per_seq`` a rank's context needs for a sequence of ``n_tokens`` tokens
        plus ``extra`` tokens appended later."""
        lo, hi, _nb, last = sequence_shard(n_tokens, hot_window, rank, world)
        return max(hi - lo + (extra if last else 0), hot_window + 1)

    def shard(self, n_tokens: int):
        return sequence_shard(n_tokens, self.ctx.geom.hot_window, self.rank, self.world)

    def prefill(self, layer: int, n_tokens: int, make_tokens, chunk: int = 16384) -> None:
        """Fills ``layer`` of an empty cache with a sequence of ``n_tokens`` tokens.
        ``make_tokens(t0, t1)`` returns the ``(k, v)`` CUDA tensors ``[n_seqs, t1 - t0, H, D]``
        of tokens ``[t0, t1)``; it is asked only for this rank's share."""
        if self.prefilled[layer] or self.n_tokens[layer]:
            raise RuntimeError("prefill needs an empty layer")
        lo, hi, _nb, _last = self.shard(n_tokens)
        for t0 in range(lo, hi, chunk):
            k, v = make_tokens(t0, min(hi, t0 + chunk))
            self.ctx.append(layer, k, v)
        self.n_tokens[layer] = n_tokens
        self.prefilled[layer] = True

    def append(self, layer: int, k, v) -> None:
        """Appends new tokens (``[n_seqs, T, H, D]``, the same on every rank): only the last
        rank, the owner of the hot window, stores them."""
        if self.rank == self.world - 1:
            self.ctx.append(layer, k, v)
        self.n_tokens[layer] += k.shape[1]

    def local_blocks(self, layer: int) -> int:
        """Cold blocks this rank holds, all of which it attends, in ``layer``."""
        _total, cold, _hot = self.ctx.lengths(layer, 0)
        return cold // self.ctx.geom.block_tokens

    def decode_partial(self, layer: int, q, mlo=None):
        """This rank's un-normalised state over its own blocks (+ the window on the last
        rank): ``[n_seqs, n_q_heads, 2 + D]``."""
        last = self.rank == self.world - 1
        return self.ctx.decode_partial(layer, q, 0, self.local_blocks(layer), last, mlo=mlo)

    def decode(self, layer: int, q, out=None):
        """One decode step for every sequence: ``[n_seqs, n_q_heads, D]`` on every rank."""
        if self.exchange is not None and self.fused and self._fused is not False:
            # one call: the merge kernel of the partial decode runs the exchange itself
            try:
                res = self.ctx.decode_exchange(layer, q, 0, self.local_blocks(layer),
                                               self.rank == self.world - 1, self.exchange, out=out)
                self._fused = True
                return res
            except NotImplementedError:
                if self._fused:  # it worked before: a real error
                    raise
                self._fused = False  # this geometry: two calls (the same on every rank)
        mlo = self.decode_partial(layer, q)
        rows = mlo.shape[0] * mlo.shape[1]
        out2 = None if out is None else out.reshape(rows, -1)
        if self.exchange is not None:
            res = self.exchange.gather_merge(mlo.reshape(rows, mlo.shape[2]), out=out2)
            return res.reshape(mlo.shape[0], mlo.shape[1], -1)
        if self.world == 1:
            gathered = mlo.reshape(1, rows, mlo.shape[2])
        else:
            gathered = gather_states(mlo.reshape(rows, mlo.shape[2]), self.group)
        res = self.ctx.lse_combine(gathered, out=out2)
        return res.reshape(mlo.shape[0], mlo.shape[1], -1)

    def use_peer_exchange(self, on: bool = True, fused: bool = False):
        """Switches the decode step's transport to :class:`PeerExchange` (a collective call:
        every rank of the group makes it) or back to the NCCL all-gather.  Returns whether the
        peer transport is in use afterwards; where peer mappings cannot be set up on some
        rank, every rank stays on the all-gather.  ``fused`` lets the merge kernel of the
        partial decode run the exchange itself (``KVContext.decode_exchange``) instead of a
        kernel of its own after it: one launch less, measured a little faster on two GPUs and
        a little slower on eight."""
        self.fused = bool(fused)
        import torch
        import torch.distributed as dist

        if self.exchange is not None:
            self.exchange.close()
            self.exchange = None
        if not on or self.world == 1:
            return False
        g = self.ctx.geom
        ok, ex = 1, None
        try:
            ex = PeerExchange(g.n_seqs * g.n_q_heads, g.head_dim, self.ctx.device, self.group)
        except Exception:  # noqa: BLE001  (no peer access between these GPUs / processes)
            ok = 0
        flag = torch.tensor([ok], dtype=torch.int32, device=self.ctx.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 1:
            self.exchange = ex
            return True
        if ex is not None:
            ex.close()
        return False


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

"""The peer-memory exchange of sequence-split attention states (`tq_xchg_*`), on one GPU.

Two ranks are emulated by two exchange objects of one process whose regions point at each
other.  Kernels that wait for one another must not run as separate launches on one GPU, so
the test uses the split form of the call: both ranks publish first (phase 1), then both wait
and merge (phase 2) — every flag is already set when a wait looks at it.  The result must be
the bits of `tq_lse_combine` on the gathered states.  The error path is driven by a rank that
never publishes: the bounded wait runs out, the status bit is set, nothing hangs.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

D = 128


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    return torch


def _make(lib, rank, world, rows):
    from turboquant_pro_b200._lib import check

    h = C.c_void_p()
    check(lib.tq_xchg_create(0, rank, world, rows, D, C.byref(h)))
    return h


def _states(torch, seed, rows):
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    mlo = torch.randn((rows, 2 + D), generator=gen, device="cuda")
    mlo[:, 0] = mlo[:, 0] * 5.0                      # maxima (natural-log domain)
    mlo[:, 1] = mlo[:, 1].abs() + 0.1                # sums
    mlo[rows // 3, 0] = float("-inf")                # a rank that attended nothing for a row
    mlo[rows // 3, 1] = 0.0
    mlo[rows // 3, 2:] = 0.0
    return mlo.contiguous()


@pytest.mark.parametrize("rows", [5, 37, 96])
def test_two_ranks_on_one_gpu_give_the_bits_of_lse_combine(torch_cuda, rows):
    torch = torch_cuda
    from turboquant_pro_b200._lib import check, load

    lib = load()
    st = torch.cuda.current_stream().cuda_stream
    xs = [_make(lib, r, 2, rows) for r in range(2)]
    try:
        check(lib.tq_xchg_set_peer(xs[0], 1, lib.tq_xchg_base(xs[1])))
        check(lib.tq_xchg_set_peer(xs[1], 0, lib.tq_xchg_base(xs[0])))
        for it in range(5):  # both slots, several epochs
            mlo = [_states(torch, 10 * it + r, rows) for r in range(2)]
            if it == 3:      # a row nobody attended: zeros out
                for m in mlo:
                    m[0, 0], m[0, 1] = float("-inf"), 0.0
            out = [torch.full((rows, D), 7.0, device="cuda") for _ in range(2)]
            for r in range(2):
                check(lib.tq_xchg_gather_merge(xs[r], mlo[r].data_ptr(), None, 1, st))
            for r in range(2):
                check(lib.tq_xchg_gather_merge(xs[r], mlo[r].data_ptr(), out[r].data_ptr(), 2, st))
            want = torch.empty((rows, D), device="cuda")
            both = torch.stack(mlo).contiguous()
            check(lib.tq_lse_combine(both.data_ptr(), 2, rows, D, want.data_ptr(), st))
            torch.cuda.synchronize()
            for r in range(2):
                assert torch.equal(out[r], want), (it, r, (out[r] - want).abs().max().item())
                v = C.c_int32(-1)
                check(lib.tq_xchg_status(xs[r], C.byref(v), st))
                assert v.value == 0
    finally:
        torch.cuda.synchronize()
        for x in xs:
            lib.tq_xchg_destroy(x)


def test_one_rank_is_a_plain_normalisation(torch_cuda):
    torch = torch_cuda
    from turboquant_pro_b200._lib import check, load

    lib = load()
    st = torch.cuda.current_stream().cuda_stream
    rows = 12
    x = _make(lib, 0, 1, rows)
    try:
        for it in range(3):
            mlo = _states(torch, 50 + it, rows)
            out = torch.empty((rows, D), device="cuda")
            want = torch.empty((rows, D), device="cuda")
            check(lib.tq_xchg_gather_merge(x, mlo.data_ptr(), out.data_ptr(), 3, st))
            check(lib.tq_lse_combine(mlo.data_ptr(), 1, rows, D, want.data_ptr(), st))
            torch.cuda.synchronize()
            assert torch.equal(out, want)
    finally:
        lib.tq_xchg_destroy(x)


def test_a_rank_that_never_arrives_is_reported_not_waited_for(torch_cuda):
    torch = torch_cuda
    from turboquant_pro_b200._lib import check, load

    lib = load()
    st = torch.cuda.current_stream().cuda_stream
    rows = 8
    xs = [_make(lib, r, 2, rows) for r in range(2)]
    try:
        check(lib.tq_xchg_set_peer(xs[0], 1, lib.tq_xchg_base(xs[1])))
        check(lib.tq_xchg_set_peer(xs[1], 0, lib.tq_xchg_base(xs[0])))
        check(lib.tq_xchg_set_wait_limit(xs[0], 2000))   # about 0.2 ms of probes
        mlo = _states(torch, 3, rows)
        out = torch.full((rows, D), 7.0, device="cuda")
        check(lib.tq_xchg_gather_merge(xs[0], mlo.data_ptr(), out.data_ptr(), 3, st))
        torch.cuda.synchronize()                         # returns: the wait is bounded
        v = C.c_int32(0)
        check(lib.tq_xchg_status(xs[0], C.byref(v), st))
        assert v.value & 1
        assert not out.any()                             # rows it could not merge are zero
        # the context is still usable
        t = torch.ones(4, device="cuda") * 2
        assert float(t.sum()) == 8.0
    finally:
        torch.cuda.synchronize()
        for x in xs:
            lib.tq_xchg_destroy(x)


def test_bad_arguments_are_refused(torch_cuda):
    from turboquant_pro_b200._lib import load

    lib = load()
    h = C.c_void_p()
    assert lib.tq_xchg_create(0, 2, 2, 8, D, C.byref(h)) == -1     # rank outside the world
    assert lib.tq_xchg_create(0, 0, 17, 8, D, C.byref(h)) == -1    # more than 16 ranks
    assert lib.tq_xchg_create(0, 0, 2, 8, 64, C.byref(h)) == -2    # head_dim
    x = _make(lib, 0, 2, 8)
    try:
        assert lib.tq_xchg_gather_merge(x, None, None, 3, None) == -1
        assert lib.tq_xchg_set_peer(x, 0, lib.tq_xchg_base(x)) == -1  # own rank
        assert lib.tq_xchg_region_bytes(x) >= 2 * 2 * 8 * 130 * 4
    finally:
        lib.tq_xchg_destroy(x)


def test_merge_kernel_that_runs_the_exchange_itself(torch_cuda):
    """Two ranks of a sequence split emulated on one GPU: the same 3 000-token sequence in two
    contexts, each attending its half of the cold blocks (the second also the hot window).
    Both publish through the merge kernel of their partial decode (phase 1), then both wait and
    merge (phase 2).  The result equals the two-call form bit for bit and the whole decode
    within the merge's rounding."""
    torch = torch_cuda
    from turboquant_pro_b200 import KVContext
    from turboquant_pro_b200._lib import check, load
    from turboquant_pro_b200.parallel import split_blocks
    from turboquant_pro_b200.synth import make_kv, make_q

    lib = load()
    st = torch.cuda.current_stream().cuda_stream
    h, grp, n = 2, 4, 3000
    rows = h * grp
    k, v = make_kv(9, h, n, dtype=np.float16)
    q = torch.from_numpy(make_q(9, rows))[None].cuda().to(torch.bfloat16)
    ctxs = []
    for _ in range(2):
        c = KVContext(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=rows, value_bits=3,
                      hot_window=512, max_tokens_per_seq=n, kv_dtype="float16", seed=9)
        c.append(0, torch.from_numpy(k)[None].cuda(), torch.from_numpy(v)[None].cuda())
        ctxs.append(c)
    whole = ctxs[0].decode(0, q)
    nb = ctxs[0].lengths(0, 0)[1] // 256
    xs = [_make(lib, r, 2, rows) for r in range(2)]
    try:
        check(lib.tq_xchg_set_peer(xs[0], 1, lib.tq_xchg_base(xs[1])))
        check(lib.tq_xchg_set_peer(xs[1], 0, lib.tq_xchg_base(xs[0])))
        for it in range(3):
            shares = [split_blocks(nb, r, 2) for r in range(2)]
            mlo = [ctxs[r].decode_partial(0, q, *shares[r]).reshape(rows, 2 + D).contiguous()
                   for r in range(2)]
            want = torch.empty((rows, D), device="cuda")
            both = torch.stack(mlo).contiguous()
            check(lib.tq_lse_combine(both.data_ptr(), 2, rows, D, want.data_ptr(), st))
            out = [torch.full((rows, D), 7.0, device="cuda") for _ in range(2)]
            for r in range(2):
                ctxs[r].decode_exchange(0, q, *shares[r], xs[r], phases=1)
            for r in range(2):
                check(lib.tq_xchg_gather_merge(xs[r], mlo[r].data_ptr(), out[r].data_ptr(), 2, st))
            torch.cuda.synchronize()
            for r in range(2):
                assert torch.equal(out[r], want), (it, r)
                assert ctxs[r].last_kernel() == "tensor-core" and ctxs[r].status() == 0
            assert torch.allclose(want.reshape(whole.shape), whole, rtol=1e-3, atol=1e-4)
    finally:
        torch.cuda.synchronize()
        for x in xs:
            lib.tq_xchg_destroy(x)


def test_one_rank_fused_exchange_equals_decode(torch_cuda):
    """World size 1: the fused call is a plain decode through the exchange path."""
    torch = torch_cuda
    from turboquant_pro_b200 import KVContext
    from turboquant_pro_b200._lib import load
    from turboquant_pro_b200.synth import make_kv, make_q

    lib = load()
    h, grp, n = 2, 8, 1500
    rows = h * grp
    k, v = make_kv(4, h, n, dtype=np.float16)
    q = torch.from_numpy(make_q(4, rows))[None].cuda()
    c = KVContext(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=rows, value_bits=4,
                  hot_window=512, max_tokens_per_seq=n, kv_dtype="float16", seed=4)
    c.append(0, torch.from_numpy(k)[None].cuda(), torch.from_numpy(v)[None].cuda())
    whole = c.decode(0, q)
    x = _make(lib, 0, 1, rows)
    try:
        for _ in range(3):
            got = c.decode_exchange(0, q, 0, 1 << 20, True, x)
            torch.cuda.synchronize()
            assert torch.allclose(got, whole, rtol=1e-5, atol=1e-6)
    finally:
        lib.tq_xchg_destroy(x)

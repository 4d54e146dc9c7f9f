"""The decode entry point that needs no working memory from its caller.

Some users of this library sit inside a host engine that hands them nothing but the query
and the output tensor, or run in a phase where the process must not allocate device memory
any more.  ``tq_decode_static_scratch`` serves them: its split-K partials live in a fixed
array that is part of the library image.  This test drives it through the C ABI and checks
it against the regular ``tq_decode`` on two consecutive calls (the array is reused and keeps
the previous call's contents, which must not leak into the next result).

The file name makes pytest collect it last, so a run that stops at the first failure has
already run every other test.
"""

from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 2e-3


def test_static_scratch_decode_matches_regular_decode():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    from turboquant_pro_b200 import KVContext
    from turboquant_pro_b200._lib import TqError
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp, w = 2, 4, 512
    lens = [700, 1300, 40]
    ctx = KVContext(n_layers=1, n_seqs=len(lens), n_kv_heads=h, n_q_heads=h * grp, value_bits=3,
                    hot_window=w, max_tokens_per_seq=1536, kv_dtype="float16", seed=31)
    for s, n in enumerate(lens):
        k, v = make_kv(500 + s, h, n, dtype=np.float16)
        ctx.append(0, torch.from_numpy(k)[None].cuda(), torch.from_numpy(v)[None].cuda(),
                   seq_begin=s)
    out = torch.empty((len(lens), h * grp, 128), dtype=torch.float32, device="cuda")
    # first call on this device: the library looks up the array's address and the driver loads
    # the kernels' code; neither is an allocation by the library, but both can move the
    # driver's free-memory figure, so the measured calls below come after it
    ctx.decode_static_scratch(0, torch.zeros((len(lens), h * grp, 128), device="cuda"), out=out)
    for call in range(2):  # second call: different queries over the array the first one used
        q = np.stack([make_q(60 + 10 * call + s, h * grp) for s in range(len(lens))])
        qd = torch.from_numpy(q).cuda()
        want = ctx.decode(0, qd).cpu().numpy()
        # the property the entry point exists for: with `out` supplied the call takes no device
        # memory, neither from torch's allocator nor from the driver
        torch.cuda.synchronize()
        held, (free0, _) = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()
        ctx.decode_static_scratch(0, qd, out=out)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == held
        assert torch.cuda.mem_get_info()[0] == free0
        got = out.cpu().numpy()
        err = np.abs(got - want).max()
        assert np.allclose(got, want, rtol=RTOL, atol=ATOL), f"call {call}: max abs err {err}"
        ctx.set_kernel("general")  # same kernel family: agreement far below the tolerance
        same = ctx.decode(0, qd).cpu().numpy()
        ctx.set_kernel("auto")
        assert np.allclose(got, same, rtol=1e-4, atol=1e-5)
    assert ctx.status() == 0
    # contexts beyond the fixed array's capacity are refused, not truncated
    big = KVContext(n_layers=1, n_seqs=40, n_kv_heads=8, n_q_heads=32, value_bits=3,
                    hot_window=16, max_tokens_per_seq=32, kv_dtype="float16", seed=1)
    qb = torch.zeros((40, 32, 128), device="cuda")
    with pytest.raises(TqError, match="CAPACITY"):
        big.decode_static_scratch(0, qb)

"""TurboQuantKVManager (the reference's multi-layer manager, vllm_plugin.py:64-260) on one GPU
context: per-layer store / load / attend / statistics against the CPU oracle."""

from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 2e-3


def test_manager_layers_are_independent_caches():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    from oracle import tq_oracle as orc
    from turboquant_pro_b200.manager import TurboQuantKVManager
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp, w = 2, 2, 64
    lens = [150, 97, 0]
    mgr = TurboQuantKVManager(n_layers=3, n_kv_heads=h, head_dim=128, bits=3, hot_window=w,
                              n_q_heads=h * grp, max_tokens=256, dtype="float32", seed=4)
    refs = []
    for layer, n in enumerate(lens):
        ref = orc.OracleCache(128, h, 4, 3, w, 0.02, 4)
        ref.pi, ref.pi_t = mgr.context.pi, mgr.context.pi_t
        if n:
            k, v = make_kv(40 + layer, h, n, dtype=np.float32)
            mgr.store(layer, k[:n - 1], v[:n - 1])     # bulk (T, H, D)
            mgr.store(layer, k[n - 1], v[n - 1])       # then one token (H, D)
            for t in range(n):
                ref.append(k[t], v[t])
        refs.append(ref)
    assert mgr.n_layers == 3 and [mgr.length(i) for i in range(3)] == lens
    for layer, (n, ref) in enumerate(zip(lens, refs)):
        keys, vals = mgr.load(layer)
        assert keys.shape == (1, h, n, 128)
        if n == 0:
            with pytest.raises(RuntimeError):
                mgr.attend(layer, np.zeros((h * grp, 128), np.float32))
            continue
        assert np.array_equal(keys[0], ref.keys()) and np.array_equal(vals[0], ref.values())
        part_k, _ = mgr.load(layer, 60, 80)
        assert np.array_equal(part_k[0], ref.keys()[:, 60:80])
        q = make_q(7 + layer, h * grp)
        got = mgr.attend(layer, q)
        assert np.allclose(got, ref.attend(q), rtol=RTOL, atol=ATOL)
        st, want = mgr.layer_stats(layer), ref.memory_stats()
        assert (st.length, st.cold_length, st.hot_length) == (n, ref.cold_length, ref.hot_length)
        assert st.cold_bytes == want["cold_bytes"] and st.hot_bytes == want["hot_bytes"]
        assert st.uncompressed_bytes == want["uncompressed_equivalent_bytes"]
    agg = mgr.memory_stats()
    assert agg["n_layers"] == 3 and agg["total_tokens"] == 150
    assert agg["total_bytes"] == sum(mgr.layer_stats(i).total_bytes for i in range(3))
    assert mgr.estimate_capacity(1.0) > w
    with pytest.raises(NotImplementedError):
        TurboQuantKVManager(n_layers=1, n_kv_heads=2, bits=3, robust=False)
    mgr.clear()
    assert [mgr.length(i) for i in range(3)] == [0, 0, 0]

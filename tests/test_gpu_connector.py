"""The vLLM-style connector on the device store: paged save through a block table, restore into
pages, attention on the stored codes, eviction, hand-off between stores.  The stored blocks are
checked against the CPU oracle (containers bit for bit, dequantised tokens exactly)."""

from __future__ import annotations

from types import SimpleNamespace

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    return torch


def _paged(torch, k, v, block_size, table, n_blocks):
    """An engine-style paged layer tensor [2, n_blocks, block_size, H, D] holding the tokens of
    one request in the blocks of `table` (other blocks hold junk)."""
    n, h, d = k.shape
    kv = torch.full((2, n_blocks, block_size, h, d), 7.0, dtype=torch.float16, device="cuda")
    pos = torch.arange(n, device="cuda")
    ids = torch.as_tensor(table, device="cuda")
    kv[0][ids[pos // block_size], pos % block_size] = k
    kv[1][ids[pos // block_size], pos % block_size] = v
    return kv


def test_paged_save_load_attend_evict(torch_cuda):
    torch = torch_cuda
    from oracle import tq_oracle as orc
    from turboquant_pro_b200.connector import DeviceBlockStore, TurboQuantKVConnector
    from turboquant_pro_b200.synth import make_kv, make_q

    h, grp, n, bs = 2, 4, 900, 16
    store = DeviceBlockStore(n_layers=3, n_kv_heads=h, n_q_heads=h * grp, max_requests=2,
                             max_tokens=1024, value_bits=4, seed=9)
    conn = TurboQuantKVConnector(store=store)
    k, v = make_kv(21, h, n, dtype=np.float16)
    kt, vt = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    table = [5, 2, 62, 63] + list(range(8, 8 + 53))  # 57 distinct blocks of 16 tokens, out of order
    kv_layer = _paged(torch, kt, vt, bs, table, 64)
    meta = SimpleNamespace(request_id="req-a", block_table=table, num_tokens=n)
    conn.save_kv_layer("model.layers.1.self_attn.attn", kv_layer, meta)
    conn.wait_for_save()
    assert store.matched_tokens("req-a") == n
    assert conn.get_num_new_matched_tokens(SimpleNamespace(request_id="req-a"), 100) == (800, False)
    assert store.layer_index("model.layers.1.self_attn.attn") == 1

    # what the device holds equals the CPU oracle fed the same tokens
    ref = orc.OracleCache(128, h, 4, 4, 512, 0.02, 9)
    ref.pi, ref.pi_t = store.ctx.pi, store.ctx.pi_t
    for t in range(n):
        ref.append(k[t], v[t])
    blk = store.ctx.export_block(1, store._slot["req-a"], 0)
    assert np.array_equal(blk["key_indices"], orc.pack_key_codes(ref.cold_k[0]["codes"]))
    assert np.array_equal(blk["value_indices"], orc.pack_value_codes(ref.cold_v[0]["codes"], 4))
    kd, vd = store.load("req-a", "model.layers.1.self_attn.attn")
    assert np.array_equal(kd.cpu().numpy(), ref.keys()) and np.array_equal(vd.cpu().numpy(), ref.values())
    assert store.load("req-a", "model.layers.2.self_attn.attn") is None  # nothing saved there
    assert store.load("nobody", 1) is None

    # decode step on the stored codes
    q = make_q(21, h * grp)
    out = store.attend(1, {"req-a": torch.from_numpy(q).cuda(), "nobody": torch.zeros(8, 128)})
    assert set(out) == {"req-a"}
    assert np.allclose(out["req-a"].cpu().numpy(), ref.attend(q), rtol=2e-2, atol=2e-3)

    # restore into fresh pages through another block table (scheduler -> worker hand-over)
    table2 = list(range(63, 63 - 57, -1))
    conn.update_state_after_alloc(SimpleNamespace(request_id="req-a"), table2)
    cmeta = conn.build_connector_meta()
    fresh = torch.zeros_like(kv_layer)
    restored = conn.start_load_kv(kv_caches={"model.layers.1.self_attn.attn": fresh},
                                  connector_meta=cmeta)
    assert restored == 1
    pos = torch.arange(n, device="cuda")
    ids = torch.as_tensor(table2, device="cuda")
    got_k = fresh[0][ids[pos // bs], pos % bs].float().cpu().numpy()
    assert np.array_equal(got_k, np.moveaxis(ref.keys(), 0, 1).astype(np.float16).astype(np.float32))

    # a second request fits, a third is refused (two slots), eviction frees a slot
    assert store.save("req-b", 0, kt[:40], vt[:40])
    assert not store.save("req-c", 0, kt[:40], vt[:40])
    assert store.stats()["rejected"] == 1
    conn.get_finished({"req-a"})
    assert store.matched_tokens("req-a") == 0 and store.load("req-a", 1) is None
    assert store.save("req-c", 0, kt[:40], vt[:40])
    assert store.ctx.status() == 0


def test_hand_off_between_stores(torch_cuda):
    torch = torch_cuda
    from turboquant_pro_b200.connector import DeviceBlockStore
    from turboquant_pro_b200.synth import make_kv, make_q

    h, n = 2, 700
    kw = dict(n_layers=2, n_kv_heads=h, n_q_heads=h, max_requests=2, max_tokens=1024,
              value_bits=3, seed=4)
    a, b = DeviceBlockStore(**kw), DeviceBlockStore(**kw)
    k, v = make_kv(3, h, n, dtype=np.float16)
    kt, vt = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    for layer in range(2):
        assert a.save("r", layer, kt, vt)
    state = a.export_request("r")
    assert set(state["layers"]) == {0, 1}
    b.save("other", 0, kt[:10], vt[:10])  # the receiving store is not empty
    assert b.import_request(state) and b.matched_tokens("r") == n
    for layer in range(2):
        ka, va = a.load("r", layer)
        kb, vb = b.load("r", layer)
        assert torch.equal(ka, kb) and torch.equal(va, vb)
    q = torch.from_numpy(make_q(3, h)).cuda()
    assert torch.allclose(a.attend(1, {"r": q})["r"], b.attend(1, {"r": q})["r"], rtol=1e-5, atol=1e-6)
    assert a.export_request("unknown") is None

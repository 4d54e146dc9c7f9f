"""The transformers cache adapter: a tiny random Llama generates with its K/V held in the
compressed GPU context.  Decode steps attended on the codes must agree with the model run on
dense K/V that the CPU oracle dequantised from the same tokens (stock SDPA attention, nothing
of the GPU library on that side), with the adapter's own dense mode, and stay close to the
exact DynamicCache."""

from __future__ import annotations

import pytest

pytestmark = pytest.mark.gpu


def _tiny_llama(torch, dtype):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=97, hidden_size=256, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                      max_position_embeddings=2048, rms_norm_eps=1e-5, tie_word_embeddings=False)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).to(device="cuda", dtype=dtype).eval()


def _oracle_cache(torch, model, seed, hot_window, value_bits):
    """A cache whose layers keep every sequence in the CPU oracle's two-tier cache and hand the
    model the dense dequantised history (the reference adapter's behaviour, with the oracle
    as the compressor); a prompt into an empty cache is attended on its own K/V."""
    import numpy as np
    from transformers.cache_utils import Cache, CacheLayerMixin

    from oracle import tq_oracle as orc

    class OracleLayer(CacheLayerMixin):
        is_compileable = False
        is_sliding = False

        def __init__(self):
            super().__init__()
            self.caches = None
            self.n = 0
            self.is_initialized = False

        def lazy_initialization(self, key_states, value_states):
            b, h, _t, d = key_states.shape
            self.caches = [orc.OracleCache(d, h, 4, value_bits, hot_window, 0.02, seed)
                           for _ in range(b)]
            self.is_initialized = True

        def update(self, key_states, value_states, *args, **kwargs):
            if not self.is_initialized:
                self.lazy_initialization(key_states, value_states)
            k = key_states.float().cpu().numpy()
            v = value_states.float().cpu().numpy()
            for s, c in enumerate(self.caches):
                for t in range(k.shape[2]):
                    c.append(k[s, :, t], v[s, :, t])
            prev, self.n = self.n, self.n + k.shape[2]
            if prev == 0:
                return key_states, value_states
            ks = np.stack([c.keys() for c in self.caches])
            vs = np.stack([c.values() for c in self.caches])
            return (torch.from_numpy(ks).to(key_states), torch.from_numpy(vs).to(value_states))

        def get_seq_length(self):
            return self.n

        def get_mask_sizes(self, query_length):
            return self.n + query_length, 0

        def get_max_cache_shape(self):
            return -1

    return Cache(layers=[OracleLayer() for _ in range(model.config.num_hidden_layers)])


def _run(torch, model, cache, ids, steps):
    """Prompt, then one forced token per step (the same for every cache, so the runs see
    identical inputs); returns the logits of every decode step."""
    logits = []
    with torch.no_grad():
        model(input_ids=ids, past_key_values=cache, use_cache=True)
        for i in range(steps.shape[1]):
            out = model(input_ids=steps[:, i:i + 1], past_key_values=cache, use_cache=True)
            logits.append(out.logits[:, -1].float())
    return torch.stack(logits)


@pytest.mark.parametrize("dtype_name", ["float16", "bfloat16"])
def test_generate_on_codes_matches_dense_history(dtype_name):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    from transformers import DynamicCache

    from turboquant_pro_b200.hf_cache import TurboQuantCache, enable_turboquant_cache

    dtype = getattr(torch, dtype_name)
    model = _tiny_llama(torch, dtype)
    gen = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 97, (2, 600), generator=gen).cuda()
    steps = torch.randint(0, 97, (2, 5), generator=gen).cuda()
    exact = _run(torch, model, DynamicCache(config=model.config), ids, steps)

    fused_cache = enable_turboquant_cache(model, hot_window=512, value_bits=4, max_tokens=1024)
    fused = _run(torch, model, fused_cache, ids, steps)
    ctx = fused_cache.context
    assert ctx.lengths(0, 0) == (605, 256, 349) and ctx.lengths(1, 1) == (605, 256, 349)
    assert ctx.last_launches() == 2 and ctx.status() == 0  # the decode kernels ran

    dense_cache = TurboQuantCache(model.config, hot_window=512, value_bits=4, max_tokens=1024,
                                  dense=True)
    dense = _run(torch, model, dense_cache, ids, steps)

    # same stored codes, two ways of attending them
    assert torch.allclose(fused, dense, rtol=2e-2, atol=2e-2), (fused - dense).abs().max()
    # the independent side: tokens compressed and dequantised by the CPU oracle, attended by
    # the stock SDPA implementation
    model.config._attn_implementation = "sdpa"
    want = _run(torch, model, _oracle_cache(torch, model, 0, 512, 4), ids, steps)
    model.config._attn_implementation = "turboquant"
    assert torch.allclose(fused, want, rtol=2e-2, atol=2e-2), (fused - want).abs().max()
    # and the compression itself keeps the logits near the uncompressed cache
    cos = torch.nn.functional.cosine_similarity(fused.flatten(1), exact.flatten(1), dim=1)
    assert bool((cos > 0.98).all()), cos
    assert fused_cache.get_seq_length() == 605
    fused_cache.crop(300)
    assert fused_cache.get_seq_length() == 300 and ctx.lengths(0, 0)[0] == 300


def test_two_caches_and_uncached_calls_do_not_cross():
    """The attention function reaches a cache only through the key tensor that cache's update
    returned: a second cache of the same model, and a forward without any cache, see their own
    tokens (not the history the first cache stored for the same layer index)."""
    import torch

    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    from turboquant_pro_b200.hf_cache import TurboQuantCache, enable_turboquant_cache

    model = _tiny_llama(torch, torch.float16)
    gen = torch.Generator().manual_seed(3)
    ids_a = torch.randint(0, 97, (1, 40), generator=gen).cuda()
    ids_b = torch.randint(0, 97, (1, 25), generator=gen).cuda()
    tok = torch.randint(0, 97, (1, 1), generator=gen).cuda()
    a = enable_turboquant_cache(model, hot_window=512, value_bits=4, max_tokens=128)
    b = TurboQuantCache(model.config, hot_window=512, value_bits=4, max_tokens=128)
    with torch.no_grad():
        model(input_ids=ids_a, past_key_values=a, use_cache=True)
        model(input_ids=ids_b, past_key_values=b, use_cache=True)
        alone = model(input_ids=tok, use_cache=False).logits  # no history at all
        model.config._attn_implementation = "sdpa"
        alone_ref = model(input_ids=tok, use_cache=False).logits
        model.config._attn_implementation = "turboquant"
        step_a = model(input_ids=tok, past_key_values=a, use_cache=True).logits[:, -1].float()
        step_b = model(input_ids=tok, past_key_values=b, use_cache=True).logits[:, -1].float()
        # the same two steps with each cache alone in its own run
        a2 = TurboQuantCache(model.config, hot_window=512, value_bits=4, max_tokens=128)
        model(input_ids=ids_a, past_key_values=a2, use_cache=True)
        want_a = model(input_ids=tok, past_key_values=a2, use_cache=True).logits[:, -1].float()
        b2 = TurboQuantCache(model.config, hot_window=512, value_bits=4, max_tokens=128)
        model(input_ids=ids_b, past_key_values=b2, use_cache=True)
        want_b = model(input_ids=tok, past_key_values=b2, use_cache=True).logits[:, -1].float()
    assert torch.allclose(alone, alone_ref, rtol=1e-3, atol=1e-3)
    assert torch.equal(step_a, want_a) and torch.equal(step_b, want_b)
    assert not torch.allclose(step_a, step_b, atol=1e-3)

"""The transformers cache adapter: a tiny random Llama generates with its K/V held in the
compressed GPU context.  Decode steps attended on the codes must agree with the same cache
handing the model dense (dequantised) K/V — the reference adapter's behaviour — and stay close
to the exact DynamicCache."""

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
    # and the compression itself keeps the logits near the uncompressed cache
    cos = torch.nn.functional.cosine_similarity(fused.flatten(1), exact.flatten(1), dim=1)
    assert bool((cos > 0.98).all()), cos
    assert fused_cache.get_seq_length() == 605
    fused_cache.crop(300)
    assert fused_cache.get_seq_length() == 300 and ctx.lengths(0, 0)[0] == 300

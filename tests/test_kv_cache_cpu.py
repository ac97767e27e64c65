"""The preallocated KV cache on CPU: block-cyclic ownership of appended tokens, the HF `Cache`
contract the stock (in-window) attention uses, and capacity checks."""
import json
import os

import pytest
import torch

from conftest import PKG


def _cfg(**over):
    from transformers.models.qwen3.configuration_qwen3 import Qwen3Config
    with open(os.path.join(PKG, "model_configs", "Qwen3-1.7B-Base-jetlong_fused", "config.json")) as f:
        d = json.load(f)
    d.pop("auto_map"); d.pop("architectures")
    d.update(dict(num_hidden_layers=2, vocab_size=160, hidden_size=128, intermediate_size=256,
                  num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_window_layers=2))
    d.update(over)
    cfg = Qwen3Config(**d)
    cfg._attn_implementation = "sdpa"
    return cfg


def test_every_token_is_stored_once_at_its_block_cyclic_row():
    from jetlm.kernels.kv_cache import BifocalKVCache
    from jetlm.kernels.sequence_parallel import SequenceShard
    cfg = _cfg()
    world, block = 3, 4
    pieces = [24, 1, 1, 1, 12, 1, 1, 1, 1, 1, 1, 1, 1]          # chunks of whole stripes, then single tokens
    total = sum(pieces)
    caches = [BifocalKVCache(cfg, total, batch=1, device="cpu", dtype=torch.float32,
                             shard=SequenceShard(r, world, block=block)) for r in range(world)]
    pos = 0
    for n in pieces:
        stored = 0
        for r, cache in enumerate(caches):
            layer = cache.layers[1]
            k_dst, v_dst = layer.reserve(n)
            own = [p for p in range(pos, pos + n) if (p // block) % world == r]
            assert k_dst.shape[1] == len(own)
            for i, p in enumerate(own):
                k_dst[:, i] = float(p)
                v_dst[:, i] = float(-p)
            layer.commit(n)
            stored += len(own)
        assert stored == n
        pos += n
    for r, cache in enumerate(caches):
        layer, sh = cache.layers[1], cache.shard
        want = sh.owned_rows(total).float()
        assert layer.get_seq_length() == total and layer.rows == sh.n_owned(total)
        assert torch.equal(layer.key_rows()[0, :, 0, 0], want)
        assert torch.equal(layer.value_rows()[0, :, 1, 5], -want)
        assert cache.get_seq_length() == 0                      # layer 0 was never written
        assert cache.group_scratch(layer.rows).stride() == layer.key_rows().stride()


def test_capacity_is_enforced_and_reset_reuses_the_buffers():
    from jetlm.kernels.kv_cache import BifocalKVCache
    cache = BifocalKVCache(_cfg(), 200, device="cpu", dtype=torch.float32)
    layer = cache.layers[0]
    assert cache.max_tokens == 256                               # rounded up to whole 128-row blocks
    layer.reserve(256); layer.commit(256)
    with pytest.raises(RuntimeError, match="capacity"):
        layer.reserve(1)
    ptr = layer.keys.data_ptr()
    cache.reset()
    assert cache.get_seq_length() == 0 and layer.keys.data_ptr() == ptr
    k, _ = layer.reserve(3)
    assert k.shape[1] == 3


@torch.inference_mode()
def test_stock_attention_runs_on_the_static_cache():
    """Inside the pretrained window the model uses HF attention through Cache.update: chunked prefill and
    decode steps on the static cache give the logits of the same calls on a DynamicCache."""
    from transformers import DynamicCache
    from jetlm.kernels.kv_cache import BifocalKVCache
    from jetlm.modeling.jetlong_fused import Qwen3JetLongFusedForCausalLM
    cfg = _cfg()
    cfg.jetlong["w"], cfg.jetlong["w_0"] = 4096, 16
    torch.manual_seed(3)
    model = Qwen3JetLongFusedForCausalLM(cfg).eval()
    ids = torch.randint(0, 160, (2, 40))
    outs = []
    for cache in (DynamicCache(config=cfg), BifocalKVCache(cfg, 64, batch=2, device="cpu", dtype=torch.float32)):
        logits = [model(input_ids=ids[:, :17], past_key_values=cache, use_cache=True).logits,
                  model(input_ids=ids[:, 17:36], past_key_values=cache, use_cache=True).logits]
        for t in range(36, 40):
            logits.append(model(input_ids=ids[:, t: t + 1], past_key_values=cache, use_cache=True).logits)
        outs.append(torch.cat(logits, dim=1))
        assert cache.get_seq_length() == 40
    assert torch.allclose(outs[0], outs[1], atol=1e-5, rtol=1e-5)


@torch.inference_mode()
def test_hf_generate_accepts_the_static_cache():
    """HF `generate` (chunked prefill, greedy) with the preallocated cache passed as past_key_values returns the
    tokens it returns with its own DynamicCache."""
    from transformers import GenerationConfig
    from jetlm.kernels.kv_cache import BifocalKVCache
    from jetlm.modeling.jetlong_fused import Qwen3JetLongFusedForCausalLM
    cfg = _cfg()
    cfg.jetlong["w"], cfg.jetlong["w_0"] = 4096, 16
    torch.manual_seed(3)
    model = Qwen3JetLongFusedForCausalLM(cfg).eval()
    ids = torch.randint(0, 160, (1, 40))
    gen = GenerationConfig(max_new_tokens=5, do_sample=False, pad_token_id=0, eos_token_id=None,
                           prefill_chunk_size=16, disable_compile=True)
    want = model.generate(ids, generation_config=gen)
    cache = BifocalKVCache(cfg, 64, batch=1, device="cpu", dtype=torch.float32)
    got = model.generate(ids, generation_config=gen, past_key_values=cache)
    assert got.tolist() == want.tolist()
    assert cache.get_seq_length() == 44

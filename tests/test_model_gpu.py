"""The `jetlong_fused` model surface on the B200 kernels against the unmodified reference modeling
file (fixture model_tiny.npz: same weights, same token ids; the reference ran on CPU with its torch
oracle as attention backend, in fp32 and in bf16)."""
import json
import os

import pytest
import torch

import jetlong_oracle as orc
from conftest import ROOT

pytestmark = pytest.mark.gpu


def _tiny_model(g, dtype=torch.bfloat16):
    from transformers.models.qwen3.configuration_qwen3 import Qwen3Config
    from jetlm.modeling.jetlong_fused import Qwen3JetLongFusedForCausalLM
    with open(os.path.join(ROOT, "jet-long_b200", "model_configs", "Qwen3-1.7B-Base-jetlong_fused", "config.json")) as f:
        d = json.load(f)
    assert d["architectures"] == ["Qwen3JetLongFusedForCausalLM"]
    assert d["auto_map"]["AutoModelForCausalLM"] == "modeling_qwen3_jetlong_fused.Qwen3JetLongFusedForCausalLM"
    d.pop("auto_map"); d.pop("architectures")
    d.update(dict(num_hidden_layers=2, vocab_size=128, hidden_size=128, intermediate_size=256,
                  num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_window_layers=2))
    cfg = Qwen3Config(**d)
    cfg.jetlong["w"] = g.meta["w"]
    cfg.jetlong["w_0"] = g.meta["w0"]
    cfg._attn_implementation = "sdpa"
    model = Qwen3JetLongFusedForCausalLM(cfg).eval()
    sd = {k[3:]: g[k].float() for k in g.keys() if k.startswith("w::")}
    model.load_state_dict(sd, strict=True)            # stock Qwen3 parameter names, zero mismatches
    inv = model.model.rotary_emb.inv_freq.clone()
    model = model.to("cuda", dtype)
    model.model.rotary_emb.inv_freq = inv.cuda()       # a checkpoint load keeps fp32 RoPE frequencies
    return model


@torch.inference_mode()
def test_prefill_then_decode_logits_match_reference(golden):
    g = golden("model_tiny.npz")
    model = _tiny_model(g)
    ids = g["input_ids"].cuda()
    S, n_dec = g.meta["S_prefill"], g.meta["n_decode"]
    out = model(input_ids=ids[:, :S], use_cache=True)
    logits = [out.logits[:, -1].float()]
    cache = out.past_key_values
    for t in range(n_dec):
        out = model(input_ids=ids[:, S + t:S + t + 1], past_key_values=cache, use_cache=True)
        logits.append(out.logits[:, -1].float())
    got = torch.stack(logits, 1).cpu()
    ref32, ref16 = g["fp32::logits"], g["bf16::logits"]
    d, cos = orc.compare(got, ref32)
    d_ref, cos_ref = orc.compare(ref16, ref32)
    # the reference's own bf16 run is the yardstick for what bf16 weights/activations cost
    assert cos >= 0.999 and d <= max(2.0 * d_ref, 0.1), (d, cos, d_ref, cos_ref)


@torch.inference_mode()
def test_chunked_prefill_matches_fresh_prefill_rows(golden):
    """With ONE layer, a 120 + 80 chunked prefill reproduces rows 120.. of the fresh 200-token prefill
    (the second chunk uses the same G for all keys), exercising seqstart_q > 0 and the regroup of
    previously cached keys.  (With more layers the results differ by design: the first chunk's hidden
    states were formed with that chunk's smaller G.)"""
    g = golden("model_tiny.npz")
    model = _tiny_model(g)
    model.model.layers = model.model.layers[:1]
    model.config.num_hidden_layers = 1
    ids = g["input_ids"].cuda()[:, :200]
    fresh = model(input_ids=ids, use_cache=True).logits.float()
    out1 = model(input_ids=ids[:, :120], use_cache=True)
    out2 = model(input_ids=ids[:, 120:], past_key_values=out1.past_key_values, use_cache=True)
    d, cos = orc.compare(out2.logits.float().cpu(), fresh[:, 120:].cpu())
    assert cos >= 0.9995 and d <= 0.1, (d, cos)


@torch.inference_mode()
def test_short_context_uses_stock_attention_and_decode_guard(golden):
    g = golden("model_tiny.npz")
    model = _tiny_model(g)
    ids = g["input_ids"].cuda()
    out = model(input_ids=ids[:, :40], use_cache=True)            # 40 <= w = 64: stock path
    assert out.logits.shape == (1, 40, 128)
    model.train()
    with pytest.raises(RuntimeError, match="inference-only"):
        model(input_ids=ids[:, :100])


@torch.inference_mode()
def test_hf_generate_with_chunked_prefill(golden):
    """HF `generate` drives the model the way the reference's evaluation wrapper does (chunked prefill,
    then one forward per token): in-window chunk -> extended chunks with a growing cache -> decode
    steps off the cache.  Greedy tokens must equal a hand-rolled loop over the same model."""
    from transformers import GenerationConfig
    g = golden("model_tiny.npz")
    model = _tiny_model(g)
    ids = g["input_ids"].cuda()[:, :150]
    gen_cfg = GenerationConfig(max_new_tokens=4, do_sample=False, prefill_chunk_size=50, disable_compile=True,
                               pad_token_id=0, eos_token_id=None)
    out = model.generate(ids, generation_config=gen_cfg)
    assert out.shape == (1, 154)
    cache = None
    for lo in range(0, 150, 50):
        res = model(input_ids=ids[:, lo:lo + 50], past_key_values=cache, use_cache=True)
        cache = res.past_key_values
    toks = []
    nxt = res.logits[:, -1].argmax(-1, keepdim=True)
    for _ in range(4):
        toks.append(int(nxt))
        res = model(input_ids=nxt, past_key_values=cache, use_cache=True)
        nxt = res.logits[:, -1].argmax(-1, keepdim=True)
    assert out[0, 150:].tolist() == toks


def _drive(model, ids, cache, chunks, n_dec):
    """Chunked prefill then teacher-forced one-token steps; returns the logits of every call, concatenated."""
    logits, lo = [], 0
    for n in chunks:
        logits.append(model(input_ids=ids[:, lo: lo + n], past_key_values=cache, use_cache=True).logits.float())
        lo += n
    for t in range(lo, lo + n_dec):
        logits.append(model(input_ids=ids[:, t: t + 1], past_key_values=cache, use_cache=True).logits.float())
    return torch.cat(logits, dim=1)


@torch.inference_mode()
def test_static_cache_reproduces_dynamic_cache_logits(golden):
    """Keys written straight into the preallocated cache by the fused norm -> RoPE pass, regrouped keys in
    the shared scratch, decode off the in-place rows: the same kernels see the same operands as with
    DynamicCache, so the logits agree to the last bit.  Chunks: in-window (40), extended (60 + 50)."""
    from transformers import DynamicCache
    from jetlm.kernels.kv_cache import BifocalKVCache
    g = golden("model_tiny.npz")
    model = _tiny_model(g)
    ids = g["input_ids"].cuda()
    want = _drive(model, ids, DynamicCache(config=model.config), (40, 60, 50), 5)
    cache = BifocalKVCache(model.config, 160, device="cuda", dtype=torch.bfloat16)
    got = _drive(model, ids, cache, (40, 60, 50), 5)
    assert cache.get_seq_length() == 155
    assert torch.equal(got, want)
    cache.reset()                                     # fresh extended prefill (keys regrouped by the fused pass)
    assert torch.equal(_drive(model, ids, cache, (150,), 3), _drive(model, ids, DynamicCache(config=model.config), (150,), 3))


@torch.inference_mode()
def test_kernels_within_window_match_stock_attention(golden):
    """With `kernels_within_window` the bifocal kernels also serve L <= w (G = 1: one effective class).
    Logits must agree with the stock attention path to bf16 accuracy, through prefill, the crossing of
    the window and decode."""
    from jetlm.kernels.kv_cache import BifocalKVCache
    g = golden("model_tiny.npz")
    model = _tiny_model(g)
    ids = g["input_ids"].cuda()
    want = _drive(model, ids, BifocalKVCache(model.config, 128, device="cuda", dtype=torch.bfloat16), (30, 20), 20)
    model.model.kernels_within_window = True
    got = _drive(model, ids, BifocalKVCache(model.config, 128, device="cuda", dtype=torch.bfloat16), (30, 20), 20)
    d, cos = orc.compare(got.cpu(), want.cpu())
    assert cos >= 0.9995 and d <= 0.1, (d, cos)


@torch.inference_mode()
def test_generate_long_equals_a_hand_rolled_greedy_loop(golden):
    from transformers import DynamicCache
    g = golden("model_tiny.npz")
    model = _tiny_model(g)
    ids = g["input_ids"].cuda()[:, :150]
    out = model.generate_long(ids, max_new_tokens=5, chunk_tokens=64)
    cache = DynamicCache(config=model.config)
    for lo in range(0, 150, 64):
        res = model(input_ids=ids[:, lo: lo + 64], past_key_values=cache, use_cache=True)
    toks, nxt = [], res.logits[:, -1].argmax(-1, keepdim=True)
    for _ in range(5):
        toks.append(int(nxt))
        nxt = model(input_ids=nxt, past_key_values=cache, use_cache=True).logits[:, -1].argmax(-1, keepdim=True)
    assert out.tolist() == [toks]


@torch.inference_mode()
@pytest.mark.parametrize("static_cache", [False, True])
def test_left_padded_batch_matches_unpadded_samples(golden, static_cache):
    """A left-padded batch of two prompts (150 and 130 tokens; same G in every call) through chunked prefill
    (100 + 50 rows) and two decode steps gives, on the real rows, the logits of each prompt run alone."""
    from transformers import DynamicCache
    from jetlm.kernels.kv_cache import BifocalKVCache
    g = golden("model_tiny.npz")
    model = _tiny_model(g)
    ids = g["input_ids"].cuda()
    a, b, pad = ids[:, :152], ids[:, 30:162], 20
    batch = torch.cat([a, torch.cat([torch.zeros(1, pad, dtype=ids.dtype, device="cuda"), b], 1)], 0)      # (2, 152)
    mask = torch.ones_like(batch)
    mask[1, :pad] = 0
    pos = (mask.cumsum(-1) - 1).clamp(min=0)
    new = lambda n: (BifocalKVCache(model.config, 256, batch=n, device="cuda", dtype=torch.bfloat16) if static_cache
                     else DynamicCache(config=model.config))

    def run(tokens, cuts, mask=None, pos=None):
        cache, outs, lo = new(tokens.shape[0]), [], 0
        for hi in cuts:
            kw = {} if mask is None else dict(attention_mask=mask[:, :hi], position_ids=pos[:, lo:hi])
            outs.append(model(input_ids=tokens[:, lo:hi], past_key_values=cache, use_cache=True, **kw).logits.float())
            lo = hi
        return torch.cat(outs, 1)

    got = run(batch, (100, 150, 151, 152), mask, pos)
    want_a = run(a, (100, 150, 151, 152))
    want_b = run(b, (80, 130, 131, 132))
    for name, x, y in (("a", got[0], want_a[0]), ("b", got[1, pad:], want_b[0])):
        d, cos = orc.compare(x.cpu(), y.cpu())
        assert cos >= 0.9995 and d <= 0.1, (name, d, cos)
    assert torch.isfinite(got).all()

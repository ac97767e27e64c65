"""The `jetlong_fused` method surface, checked on CPU: a model directory made of the shipped
config.json + the modeling file loads through AutoModelForCausalLM with trust_remote_code (the way
the reference's loaders do it), keeps stock Qwen3 parameter names, and runs the in-window path."""
import json
import os
import shutil

import pytest
import torch

from conftest import PKG


def _make_model_dir(tmp_path):
    src_cfg = os.path.join(PKG, "model_configs", "Qwen3-1.7B-Base-jetlong_fused", "config.json")
    with open(src_cfg) as f:
        cfg = json.load(f)
    cfg.update(dict(num_hidden_layers=2, vocab_size=160, hidden_size=128, intermediate_size=256,
                    num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_window_layers=2))
    cfg["jetlong"]["w"], cfg["jetlong"]["w_0"] = 64, 16
    d = tmp_path / "Qwen3-tiny-jetlong_fused"
    d.mkdir()
    with open(d / "config.json", "w") as f:
        json.dump(cfg, f)
    shutil.copy(os.path.join(PKG, "jetlm", "modeling", "jetlong_fused", "modeling_qwen3_jetlong_fused.py"), d)
    return d


def test_auto_model_loads_the_variant_directory(tmp_path):
    from transformers import AutoConfig, AutoModelForCausalLM
    d = _make_model_dir(tmp_path)
    config = AutoConfig.from_pretrained(str(d), trust_remote_code=True)
    assert config.jetlong == {"w": 64, "w_0": 16, "yarn_alpha": 1, "yarn_beta": 32}
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(config, trust_remote_code=True).eval()
    assert type(model).__name__ == "Qwen3JetLongFusedForCausalLM"
    names = set(model.state_dict().keys())
    assert "model.layers.1.self_attn.q_norm.weight" in names and "model.layers.0.self_attn.o_proj.weight" in names
    assert not any("rotary" in n or "jetlong" in n for n in names)        # no extra parameters or buffers to load
    model.save_pretrained(str(d), safe_serialization=True)
    again = AutoModelForCausalLM.from_pretrained(str(d), trust_remote_code=True, attn_implementation="sdpa").eval()
    ids = torch.arange(40).view(1, 40) % 160
    with torch.inference_mode():
        a = model(input_ids=ids).logits
        b = again(input_ids=ids).logits
    assert torch.allclose(a, b, atol=1e-5)


def test_in_window_path_equals_stock_qwen3(tmp_path):
    """L <= w: the model is stock Qwen3 (reference modeling :299-320)."""
    from transformers import AutoConfig, AutoModelForCausalLM
    from transformers.models.qwen3.modeling_qwen3 import Qwen3ForCausalLM
    d = _make_model_dir(tmp_path)
    config = AutoConfig.from_pretrained(str(d), trust_remote_code=True)
    config._attn_implementation = "eager"
    torch.manual_seed(1)
    ours = AutoModelForCausalLM.from_config(config, trust_remote_code=True).float().eval()
    stock = Qwen3ForCausalLM(config).float().eval()
    stock.load_state_dict(ours.state_dict(), strict=True)
    ids = torch.randint(0, 160, (2, 50))
    with torch.inference_mode():
        a = ours(input_ids=ids, use_cache=True)
        b = stock(input_ids=ids, use_cache=True)
        assert torch.allclose(a.logits, b.logits, atol=1e-5)
        nxt = torch.randint(0, 160, (2, 1))
        a2 = ours(input_ids=nxt, past_key_values=a.past_key_values, use_cache=True).logits
        b2 = stock(input_ids=nxt, past_key_values=b.past_key_values, use_cache=True).logits
        assert torch.allclose(a2, b2, atol=1e-5)


def test_extended_path_has_no_cpu_fallback(tmp_path):
    from transformers import AutoConfig, AutoModelForCausalLM
    d = _make_model_dir(tmp_path)
    config = AutoConfig.from_pretrained(str(d), trust_remote_code=True)
    model = AutoModelForCausalLM.from_config(config, trust_remote_code=True).eval()
    with torch.inference_mode(), pytest.raises((ValueError, RuntimeError)):
        model(input_ids=torch.zeros(1, 100, dtype=torch.long))     # L > w on CPU tensors: the kernels refuse, nothing falls back

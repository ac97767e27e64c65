"""Golden fixtures for the self-extend and DCA position maps, produced by the REFERENCE's own
unmodified modeling files (imported, never copied) running their eager paths on CPU in fp32.

Called from make_golden.py.  For each method a 1-layer random-init attention module is driven
directly; the fixture stores the un-rotated post-norm q/k, v, and the attention output taken
before the output projection (o_proj is swapped for an identity), for a fresh prefill and for
one decode step on top of it.
"""
from __future__ import annotations

import importlib.util
import json
import os
import sys

import numpy as np
import torch
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _tiny_config(root, variant, extra_key, extra):
    from transformers.models.qwen3.configuration_qwen3 import Qwen3Config
    with open(os.path.join(root, "model_configs", variant, "config.json")) as f:
        d = json.load(f)
    d.pop("auto_map", None)
    d.pop("architectures", None)
    d.update(dict(num_hidden_layers=1, vocab_size=128, hidden_size=256, intermediate_size=512,
                  num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_window_layers=1))
    d[extra_key] = extra
    cfg = Qwen3Config(**d)
    cfg._attn_implementation = "eager"
    return cfg


def _raw_qkv(attn, hidden):
    shp = (*hidden.shape[:-1], -1, attn.head_dim)
    q = attn.q_norm(attn.q_proj(hidden).view(shp))
    k = attn.k_norm(attn.k_proj(hidden).view(shp))
    v = attn.v_proj(hidden).view(shp)
    return q, k, v            # (B, S, H, D)


def _causal_additive(S, Skv):
    qi = torch.arange(Skv - S, Skv).view(S, 1)
    ki = torch.arange(Skv).view(1, Skv)
    m = torch.zeros(S, Skv)
    m.masked_fill_(ki > qi, float("-inf"))
    return m.view(1, 1, S, Skv)


def _eager_fa(q, k, v, causal):
    """Stand-in for the FA2 wrapper the DCA file calls: (B,H,T,D) in, ((B,H,T,D), (B,H,T)) out."""
    H, Hk = q.shape[1], k.shape[1]
    k = k.repeat_interleave(H // Hk, dim=1)
    v = v.repeat_interleave(H // Hk, dim=1)
    s = torch.einsum("bhqd,bhkd->bhqk", q.float(), k.float()) * (q.shape[-1] ** -0.5)
    if causal:
        T, Tk = q.shape[2], k.shape[2]
        qi = torch.arange(Tk - T, Tk).view(T, 1)
        ki = torch.arange(Tk).view(1, Tk)
        s = s.masked_fill(ki > qi, float("-inf"))
    lse = torch.logsumexp(s, -1)
    out = torch.einsum("bhqk,bhkd->bhqd", torch.softmax(s, -1), v.float()).to(q.dtype)
    return out, lse


def gen_selfext(root, name, *, seed=21, S=200, Gs=4, W=32):
    from transformers.cache_utils import DynamicCache
    mod = _load(os.path.join(root, "jetlm/modeling/selfext/modeling_qwen3_selfext.py"), "modeling_qwen3_selfext")
    cfg = _tiny_config(root, "Qwen3-1.7B-Base-selfext", "selfext",
                       dict(group_size=Gs, window_size=W, scale_base=-1, use_flash_attn=False))
    torch.manual_seed(seed)
    model = mod.Qwen3SelfExtendModel(cfg).eval().float()
    attn = model.layers[0].self_attn
    attn.o_proj = nn.Identity()
    hidden = torch.randn(1, S + 1, cfg.hidden_size)
    with torch.inference_mode():
        q, k, v = _raw_qkv(attn, hidden)
        cache = DynamicCache(config=cfg)
        pos = torch.arange(S).view(1, S)
        out_p, _ = attn(hidden[:, :S], None, _causal_additive(S, S), position_ids=pos,
                        past_key_values=cache, cache_position=torch.arange(S))
        out_d, _ = attn(hidden[:, S:], None, _causal_additive(1, S + 1), position_ids=torch.tensor([[S]]),
                        past_key_values=cache, cache_position=torch.tensor([S]))
    H, D = cfg.num_attention_heads, cfg.head_dim
    np.savez(os.path.join(HERE, name), q_raw=q.numpy(), k_raw=k.numpy(), v=v.numpy(),
             out_prefill=out_p.view(1, S, H, D).numpy(), out_decode=out_d.view(1, 1, H, D).numpy(),
             inv_freq=model.rotary_emb.inv_freq.float().numpy(),
             meta=json.dumps(dict(seed=seed, S=S, group_size=Gs, window_size=W)))


def gen_dca(root, name, *, seed=22, S=200, s=64, w=16):
    from transformers.cache_utils import DynamicCache
    mod = _load(os.path.join(root, "jetlm/modeling/dca/modeling_qwen3_dca.py"), "modeling_qwen3_dca")
    mod._do_fa = _eager_fa
    cfg = _tiny_config(root, "Qwen3-1.7B-Base-dca", "dca", dict(chunk_size=s, local_window=w))
    torch.manual_seed(seed)
    model = mod.Qwen3DcaModel(cfg).eval().float()
    attn = model.layers[0].self_attn
    attn.o_proj = nn.Identity()
    hidden = torch.randn(1, S + 1, cfg.hidden_size)
    with torch.inference_mode():
        q, k, v = _raw_qkv(attn, hidden)
        cache = DynamicCache(config=cfg)
        pos = torch.arange(S).view(1, S)
        out_p, _ = attn(hidden[:, :S], None, None, position_ids=pos, past_key_values=cache,
                        cache_position=torch.arange(S))
        out_d, _ = attn(hidden[:, S:], None, None, position_ids=torch.tensor([[S]]), past_key_values=cache,
                        cache_position=torch.tensor([S]))
    H, D = cfg.num_attention_heads, cfg.head_dim
    np.savez(os.path.join(HERE, name), q_raw=q.numpy(), k_raw=k.numpy(), v=v.numpy(),
             out_prefill=out_p.view(1, S, H, D).numpy(), out_decode=out_d.view(1, 1, H, D).numpy(),
             inv_freq=model.rotary_emb.inv_freq.float().numpy(),
             meta=json.dumps(dict(seed=seed, S=S, chunk_size=s, local_window=w)))


def _eager_flash_attn_forward(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size_left=-1,
                              window_size_right=-1, softcap=0.0, alibi_slopes=None, return_softmax=False):
    """Stand-in for flash_attn's `_flash_attn_forward` (the jetlong_freq file imports it inside forward):
    (B,S,H,D) in, (out (B,S,H,D), lse (B,H,S), None, None) out; causal aligned to the bottom right, keys
    further than window_size_left behind the query masked."""
    H, Hk = q.shape[2], k.shape[2]
    kk = k.repeat_interleave(H // Hk, dim=2).float()
    vv = v.repeat_interleave(H // Hk, dim=2).float()
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kk) * softmax_scale
    T, Tk = q.shape[1], k.shape[1]
    qi = torch.arange(Tk - T, Tk).view(T, 1)
    ki = torch.arange(Tk).view(1, Tk)
    if causal:
        s = s.masked_fill(ki > qi, float("-inf"))
    if window_size_left >= 0:
        s = s.masked_fill(qi - ki > window_size_left, float("-inf"))
    lse = torch.logsumexp(s, -1)
    out = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vv).to(q.dtype)
    return out, lse, None, None


def gen_jetlong_freq(root, name, *, seed=23, S=200, w=64, w_0=16):
    """jetlong_freq (per-frequency far-class rotation + softmax temperature): prefill of S tokens and one
    decode step through the reference's attention module, its flash-attn calls served by the eager stand-in."""
    import types
    from transformers.cache_utils import DynamicCache
    mod = _load(os.path.join(root, "jetlm/modeling/jetlong_freq/modeling_qwen3_jetlong_freq.py"),
                "modeling_qwen3_jetlong_freq")          # imports transformers first: it probes the real flash_attn
    fa = types.ModuleType("flash_attn")
    fai = types.ModuleType("flash_attn.flash_attn_interface")
    fai._flash_attn_forward = _eager_flash_attn_forward
    fa.flash_attn_interface = fai
    saved = {k: sys.modules.get(k) for k in ("flash_attn", "flash_attn.flash_attn_interface")}
    sys.modules["flash_attn"], sys.modules["flash_attn.flash_attn_interface"] = fa, fai
    try:
        cfg = _tiny_config(root, "Qwen3-1.7B-Base-jetlong_freq", "jetlong_freq",
                           dict(w=w, w_0=w_0, yarn_alpha=1, yarn_beta=32))
        torch.manual_seed(seed)
        model = mod.Qwen3JetLongFreqModel(cfg).eval().float()
        attn = model.layers[0].self_attn
        attn.o_proj = nn.Identity()
        hidden = torch.randn(1, S + 1, cfg.hidden_size)
        with torch.inference_mode():
            q, k, v = _raw_qkv(attn, hidden)
            cache = DynamicCache(config=cfg)
            pe_p = model.rotary_emb(hidden[:, :S], torch.arange(S).view(1, S))
            out_p, _ = attn(hidden[:, :S], pe_p, None, past_key_values=cache, cache_position=torch.arange(S))
            pe_d = model.rotary_emb(hidden[:, S:], torch.tensor([[S]]))
            out_d, _ = attn(hidden[:, S:], pe_d, None, past_key_values=cache, cache_position=torch.tensor([S]))
    finally:
        for key, val in saved.items():
            if val is None:
                sys.modules.pop(key, None)
            else:
                sys.modules[key] = val
    assert len(pe_p) == 4 and len(pe_d) == 4
    H, D = cfg.num_attention_heads, cfg.head_dim
    np.savez(os.path.join(HERE, name), q_raw=q.numpy(), k_raw=k.numpy(), v=v.numpy(),
             out_prefill=out_p.view(1, S, H, D).numpy(), out_decode=out_d.view(1, 1, H, D).numpy(),
             inv_freq=model.rotary_emb.inv_freq.float().numpy(),
             delta_inv_freq_prefill=pe_p[2].float().numpy(), delta_inv_freq_decode=pe_d[2].float().numpy(),
             ntk_ramp=model.rotary_emb.ntk_ramp.float().numpy(),
             meta=json.dumps(dict(seed=seed, S=S, w=w, w_0=w_0, attn_scale_prefill=float(pe_p[3]),
                                  attn_scale_decode=float(pe_d[3]))))

"""Generate the golden fixtures in this directory by running the REFERENCE's own code.

Run once, in an environment where the Jet-Long checkout is importable:

    python tests/golden/make_golden.py --reference /path/to/Jet-Long

It imports (never copies) the reference's torch oracle functions, its decode backend, its
N-way split merge and its unmodified `jetlong_fused` modeling file, feeds them seeded inputs
and stores inputs + outputs as small .npz files.  The tests then check both the CPU oracle
(oracle/jetlong_oracle.py) and the CUDA kernels against these files, so neither needs the
reference checkout at test time.  bf16 tensors are stored as their uint16 bit patterns.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit pattern array."""
    assert t.dtype == torch.bfloat16
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float32).contiguous().numpy()


def load_module(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def gen_prefill(ref_tests, name, *, seed, B, S, Skv, H, Hk, D, w0):
    """Mirrors the reference's kernel-level prefill test: independent random base/group operands."""
    torch.manual_seed(seed)
    seqstart = Skv - S
    qb = torch.randn(B, S, H, D).bfloat16()
    qg = torch.randn(B, S, H, D).bfloat16()
    kb = torch.randn(B, Skv, Hk, D).bfloat16()
    kg = torch.randn(B, Skv, Hk, D).bfloat16()
    v = torch.randn(B, Skv, Hk, D).bfloat16()
    qi = torch.arange(S).view(1, S, 1)
    ki = torch.arange(Skv).view(1, 1, Skv)
    local = ((ki <= qi + seqstart) & (ki >= qi + seqstart - w0)).expand(B, -1, -1)
    distant = (ki < qi + seqstart - w0).expand(B, -1, -1)
    lo, ll = ref_tests._attention_ref(qb.float(), kb.float(), v.float(), local)
    do, dl = ref_tests._attention_ref(qg.float(), kg.float(), v.float(), distant)
    out = ref_tests._merge_ref(lo, ll, do, dl)
    lse = torch.logaddexp(ll, dl)
    np.savez(os.path.join(HERE, name), q_base=bits(qb), q_group=bits(qg), k_base=bits(kb),
             k_group=bits(kg), v=bits(v), out=f32(out), lse=f32(lse),
             meta=json.dumps(dict(seed=seed, B=B, S=S, Skv=Skv, H=H, Hk=Hk, D=D, w0=w0, seqstart=seqstart)))


def gen_decode(ref_tests, ref_backend, name, *, seed, B, ctx, H, Hk, D, w, w0):
    """Mirrors the reference's kernel-level decode test (real regrouping of q and the far keys)
    and runs the reference backend's own torch decode on the same tensors."""
    torch.manual_seed(seed)
    G = math.ceil(ctx / w)
    boundary = ctx - 1 - w0
    qb = torch.randn(B, 1, H, D).bfloat16()
    kbase = torch.randn(B, ctx, Hk, D).bfloat16()
    v = torch.randn(B, ctx, Hk, D).bfloat16()
    inv_freq = torch.rand(D // 2, dtype=torch.float32)
    pos = torch.full((B, 1), ctx - 1, dtype=torch.long)
    dq = torch.floor(pos.float() / G) - pos.float()
    qg = ref_tests._correction_rotate_ref(qb.transpose(1, 2), dq, inv_freq).transpose(1, 2).contiguous()
    idx = torch.arange(boundary, dtype=torch.float32)
    dk = (torch.floor(idx / G) - idx).unsqueeze(0).expand(B, -1)
    kfar = kbase[:, :boundary].contiguous()
    kfar_g = ref_tests._correction_rotate_ref(kfar.transpose(1, 2), dk, inv_freq).transpose(1, 2).contiguous()
    knear = kbase[:, boundary:].contiguous()
    no, nl = ref_tests._attention_ref(qb.float(), knear.float(), v[:, boundary:].float())
    do, dl = ref_tests._attention_ref(qg.float(), kfar_g.float(), v[:, :boundary].float())
    out = ref_tests._merge_ref(no, nl, do, dl)
    lse = torch.logaddexp(nl, dl)
    out_backend = ref_backend._reference_jetlong_decode(
        qb.float(), qg.float(), knear.float(), v[:, boundary:].float(), kfar_g.float(), v[:, :boundary].float())
    np.savez(os.path.join(HERE, name), q_base=bits(qb), q_group=bits(qg), k_cache_base=bits(kbase),
             k_far_group=bits(kfar_g), v_cache=bits(v), inv_freq=inv_freq.numpy(),
             out=f32(out), lse=f32(lse), out_backend=f32(out_backend),
             meta=json.dumps(dict(seed=seed, B=B, ctx=ctx, H=H, Hk=Hk, D=D, w=w, w0=w0, G=G, boundary=boundary)))


def gen_decode_near_heavy(ref_tests, name, *, seed, B, near, far, H, Hk, D):
    """Mirrors the regression test where the near keys are aligned with the query so that the
    near region carries real weight although the far region is larger."""
    torch.manual_seed(seed)
    qb = torch.randn(B, 1, H, D).bfloat16()
    qg = torch.randn(B, 1, H, D).bfloat16()
    qkv = qb.view(B, 1, Hk, H // Hk, D).mean(3)
    kn = (qkv.expand(B, near, Hk, D) + 0.1 * torch.randn(B, near, Hk, D).bfloat16()).contiguous()
    vn = torch.randn(B, near, Hk, D).bfloat16()
    kf = (0.3 * torch.randn(B, far, Hk, D).bfloat16()).contiguous()
    vf = torch.randn(B, far, Hk, D).bfloat16()
    no, nl = ref_tests._attention_ref(qb.float(), kn.float(), vn.float())
    do, dl = ref_tests._attention_ref(qg.float(), kf.float(), vf.float())
    out = ref_tests._merge_ref(no, nl, do, dl)
    near_frac = float((nl - torch.logaddexp(nl, dl)).exp().mean())
    assert near_frac > 0.3, near_frac
    np.savez(os.path.join(HERE, name), q_base=bits(qb), q_group=bits(qg), k_near=bits(kn), v_near=bits(vn),
             k_far=bits(kf), v_far=bits(vf), out=f32(out), lse=f32(torch.logaddexp(nl, dl)),
             meta=json.dumps(dict(seed=seed, B=B, near=near, far=far, H=H, Hk=Hk, D=D, near_frac=near_frac)))


def gen_rotate(ref_tests, ref_model, name, *, seed, B, S, H, D):
    """Base RoPE and correction rotation, both from the tests' fp32-angle helper and from the
    modeling file's bf16 helpers."""
    torch.manual_seed(seed)
    x = torch.randn(B, H, S, D).bfloat16()
    inv_freq = 1.0 / (1.0e6 ** (torch.arange(0, D, 2, dtype=torch.int64).float() / D))
    pos = (torch.arange(S) + 100000).view(1, S).expand(B, -1)
    G = 4
    delta = torch.floor(pos.float() / G) - pos.float()
    r_tests = ref_tests._correction_rotate_ref(x, delta, inv_freq)
    r_model = ref_model.correction_rotate_per_sample(x, delta, inv_freq, torch.bfloat16)
    ang = pos.float().unsqueeze(-1) * inv_freq.view(1, 1, -1)
    emb = torch.cat((ang, ang), -1)
    cos, sin = emb.cos().bfloat16(), emb.sin().bfloat16()
    xb, _ = ref_model.apply_rotary_pos_emb(x, x, cos, sin)
    r_fp32 = ref_tests._correction_rotate_ref(x.float(), delta, inv_freq)
    np.savez(os.path.join(HERE, name), x=bits(x), inv_freq=inv_freq.numpy(), pos=pos.numpy(), delta=delta.numpy(),
             rot_tests=bits(r_tests), rot_model=bits(r_model), base_model=bits(xb), rot_fp32=f32(r_fp32),
             meta=json.dumps(dict(seed=seed, B=B, S=S, H=H, D=D, G=G)))


def gen_merge(ref_decode, ref_tests, name, *, seed, N, B, S, H, D):
    torch.manual_seed(seed)
    o = torch.randn(N, B, S, H, D).bfloat16()
    lse = torch.randn(N, B, H, S) * 3.0
    lse[0, :, 0, 0] = -float("inf")          # one empty partial
    # the reference's N-way merge is written for S == 1 partials laid out (N*B, 1, H, D) / (N*B, H, 1)
    outs, lses = [], []
    for s in range(S):
        op = o[:, :, s:s + 1].reshape(N * B, 1, H, D).float()
        lp = lse[:, :, :, s:s + 1].reshape(N * B, H, 1)
        om, lm = ref_decode._merge_splitk_partials_ref(op, lp, batch=B, num_splits=N, return_lse=True)
        outs.append(om)
        lses.append(lm)
    out = torch.cat(outs, dim=1)
    lse_m = torch.cat(lses, dim=2)
    two = ref_tests._merge_ref(o[0].float(), lse[0], o[1].float(), lse[1])
    np.savez(os.path.join(HERE, name), o_parts=bits(o), lse_parts=f32(lse), out=f32(out), lse=f32(lse_m),
             out_two=f32(two), meta=json.dumps(dict(seed=seed, N=N, B=B, S=S, H=H, D=D)))


def tiny_config(reference_root, variant, **over):
    from transformers.models.qwen3.configuration_qwen3 import Qwen3Config
    with open(os.path.join(reference_root, "model_configs", variant, "config.json")) as f:
        d = json.load(f)
    d.pop("auto_map", None)
    d.pop("architectures", None)
    d.update(dict(num_hidden_layers=2, vocab_size=128, hidden_size=128, intermediate_size=256,
                  num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_window_layers=2))
    d.update(over)
    cfg = Qwen3Config(**d)
    return cfg


def gen_model(reference_root, ref_tests, name, *, seed, S_prefill, n_decode, w, w0):
    """Drive the UNMODIFIED reference modeling file on CPU in fp32 and in bf16, with the fused
    backend entry points replaced by the reference tests' torch oracle; record what crosses the
    backend boundary and the logits."""
    sys.path.insert(0, reference_root)
    mod = load_module(os.path.join(reference_root, "jetlm/modeling/jetlong_fused/modeling_qwen3_jetlong_fused.py"),
                      "modeling_qwen3_jetlong_fused")
    import jetlm.kernels.cute_jetlong_backend as backend

    calls = []

    def oracle_prefill(query_base, query_group, key_base, key_group, value, *, seqstart_q, window_size_left,
                       softmax_scale, has_any_pad, training):
        qb, qg, kb, kg, v = (t.transpose(1, 2).contiguous() for t in (query_base, query_group, key_base, key_group, value))
        S, Skv = qb.shape[1], kb.shape[1]
        qi = torch.arange(S).view(1, S, 1)
        ki = torch.arange(Skv).view(1, 1, Skv)
        local = ((ki <= qi + seqstart_q) & (ki >= qi + seqstart_q - window_size_left)).expand(qb.shape[0], -1, -1)
        distant = (ki < qi + seqstart_q - window_size_left).expand(qb.shape[0], -1, -1)
        lo, ll = ref_tests._attention_ref(qb, kb, v, local)
        do, dl = ref_tests._attention_ref(qg, kg, v, distant)
        out = ref_tests._merge_ref(lo, ll, do, dl)
        calls.append(dict(kind="prefill", q_base=qb, q_group=qg, k_base=kb, k_group=kg, v=v, seqstart=int(seqstart_q),
                          w0=int(window_size_left), out=out))
        return out

    real_decode = backend.fused_jetlong_decode

    def recording_decode(query_base, query_group, key_near, value_near, key_distant_group, value_distant, **kw):
        out = real_decode(query_base, query_group, key_near, value_near, key_distant_group, value_distant, **kw)
        calls.append(dict(kind="decode", q_base=query_base, q_group=query_group, k_near=key_near, v_near=value_near,
                          k_far=key_distant_group, v_far=value_distant, G=int(kw["group_size"]), out=out))
        return out

    backend.fused_jetlong_prefill = oracle_prefill
    backend.fused_jetlong_decode = recording_decode
    os.environ["JETLM_JETLONG_FUSED_DECODE"] = "ref"

    cfg = tiny_config(reference_root, "Qwen3-1.7B-Base-jetlong_fused")
    cfg.jetlong["w"] = w
    cfg.jetlong["w_0"] = w0
    cfg._attn_implementation = "eager"
    torch.manual_seed(seed)
    model = mod.Qwen3JetLongFusedForCausalLM(cfg).eval()
    for prm in model.parameters():                       # weights exactly representable in bf16
        prm.data = prm.data.bfloat16().float()
    inv_freq32 = model.model.rotary_emb.inv_freq.clone()
    for i, layer in enumerate(model.model.layers):
        layer.attention_type = cfg.layer_types[i]        # transformers >= 5.5 no longer sets it
    ids = torch.randint(0, cfg.vocab_size, (1, S_prefill + n_decode))
    save = {"input_ids": ids.numpy(), "meta": json.dumps(dict(seed=seed, S_prefill=S_prefill, n_decode=n_decode, w=w, w0=w0))}
    sd = {k: v for k, v in model.state_dict().items()}
    for k, v in sd.items():
        save["w::" + k] = bits(v.bfloat16())
    for tag, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        calls.clear()
        m = model.to(dtype)
        # a loaded checkpoint keeps the fp32 RoPE frequencies; a blanket dtype cast would round them
        m.model.rotary_emb.inv_freq = inv_freq32.clone()
        m.model.rotary_emb.original_inv_freq = inv_freq32.clone()
        with torch.inference_mode():
            out = m(input_ids=ids[:, :S_prefill], use_cache=True)
            logits = [out.logits[:, -1].float()]
            cache = out.past_key_values
            for t in range(n_decode):
                out = m(input_ids=ids[:, S_prefill + t:S_prefill + t + 1], past_key_values=cache, use_cache=True)
                logits.append(out.logits[:, -1].float())
        save[f"{tag}::logits"] = f32(torch.stack(logits, 1))
        # layer-0 boundary tensors of the prefill call and of the first decode call
        pre = next(c for c in calls if c["kind"] == "prefill")
        dec = next(c for c in calls if c["kind"] == "decode")
        for key in ("q_base", "q_group", "k_base", "k_group", "v", "out"):
            t = pre[key]
            save[f"{tag}::prefill::{key}"] = bits(t) if t.dtype == torch.bfloat16 else f32(t)
        save[f"{tag}::prefill::seqstart"] = np.int64(pre["seqstart"])
        for key in ("q_base", "q_group", "k_near", "v_near", "k_far", "v_far", "out"):
            t = dec[key].contiguous()
            save[f"{tag}::decode::{key}"] = bits(t) if t.dtype == torch.bfloat16 else f32(t)
        save[f"{tag}::decode::G"] = np.int64(dec["G"])
        save[f"{tag}::n_prefill_calls"] = np.int64(sum(c["kind"] == "prefill" for c in calls))
        save[f"{tag}::n_decode_calls"] = np.int64(sum(c["kind"] == "decode" for c in calls))
    np.savez(os.path.join(HERE, name), **save)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a Jet-Long checkout (its code is imported, never copied)")
    args = ap.parse_args()
    root = os.path.abspath(args.reference)
    sys.path.insert(0, root)
    ref_tests = load_module(os.path.join(root, "tests/test_fa4_cute_kernels.py"), "ref_test_fa4_cute_kernels")
    import jetlm.kernels.cute_decode_sm90 as ref_decode
    import jetlm.kernels.cute_jetlong_backend as ref_backend
    ref_model = load_module(os.path.join(root, "jetlm/modeling/jetlong_fused/modeling_qwen3_jetlong_fused.py"),
                            "modeling_qwen3_jetlong_fused")
    torch.set_num_threads(8)
    gen_prefill(ref_tests, "prefill_fresh.npz", seed=3, B=1, S=192, Skv=192, H=4, Hk=2, D=128, w0=64)
    gen_prefill(ref_tests, "prefill_chunked.npz", seed=11, B=2, S=80, Skv=208, H=4, Hk=2, D=128, w0=37)
    gen_decode(ref_tests, ref_backend, "decode_regrouped.npz", seed=2, B=1, ctx=1153, H=4, Hk=2, D=128, w=512, w0=128)
    gen_decode_near_heavy(ref_tests, "decode_near_heavy.npz", seed=7, B=1, near=128, far=640, H=4, Hk=2, D=128)
    gen_rotate(ref_tests, ref_model, "rotate.npz", seed=5, B=1, S=96, H=2, D=128)
    gen_merge(ref_decode, ref_tests, "merge_nway.npz", seed=13, N=5, B=2, S=3, H=4, D=128)
    gen_model(root, ref_tests, "model_tiny.npz", seed=123, S_prefill=200, n_decode=3, w=64, w0=16)
    from make_golden_posmaps import gen_selfext, gen_dca, gen_jetlong_freq  # noqa: E402  (sibling script)
    gen_selfext(root, "selfext_tiny.npz")
    gen_dca(root, "dca_tiny.npz")
    gen_jetlong_freq(root, "jetlong_freq_tiny.npz")
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    sys.path.insert(0, HERE)
    main()

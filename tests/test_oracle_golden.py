"""The CPU oracle against outputs of the reference's own code (fixtures in tests/golden/).

These pin the oracle: every function the GPU parity tests rely on reproduces what the
reference's torch composition, decode backend, N-way merge, RoPE helpers and unmodified
modeling files produced for the same inputs.
"""
import torch

import jetlong_oracle as orc

TOL = 2e-5


def _close(a, b, tol=TOL):
    d, cos = orc.compare(a, b)
    assert d <= tol and cos > 0.99999, (d, cos)


def test_prefill_two_branch_and_single_pass(golden):
    for name in ("prefill_fresh.npz", "prefill_chunked.npz"):
        g = golden(name)
        kw = dict(seqstart=g.meta["seqstart"], w0=g.meta["w0"])
        args = [g[k] for k in ("q_base", "q_group", "k_base", "k_group", "v")]
        out, lse = orc.jetlong_prefill(*args, **kw)
        _close(out, g["out"]); _close(lse, g["lse"])
        out1, lse1 = orc.jetlong_prefill_single_pass(*args, **kw)
        _close(out1, g["out"]); _close(lse1, g["lse"])


def test_decode_composition(golden):
    g = golden("decode_regrouped.npz")
    b = g.meta["boundary"]
    kc, vc = g["k_cache_base"], g["v_cache"]
    out, lse = orc.jetlong_decode(g["q_base"], g["q_group"], kc[:, b:], vc[:, b:], g["k_far_group"], vc[:, :b])
    _close(out, g["out"]); _close(lse, g["lse"]); _close(out, g["out_backend"])
    g = golden("decode_near_heavy.npz")
    out, lse = orc.jetlong_decode(g["q_base"], g["q_group"], g["k_near"], g["v_near"], g["k_far"], g["v_far"])
    _close(out, g["out"]); _close(lse, g["lse"])


def test_decode_regroup_from_base_cache(golden):
    """Far keys regrouped by the oracle from the base-rotated cache equal the reference's."""
    g = golden("decode_regrouped.npz")
    b, G = g.meta["boundary"], g.meta["G"]
    pos = torch.arange(b).view(1, b)
    kfar = orc.rotate_bshd(g["k_cache_base"][:, :b], orc.regroup_delta(pos, G), g["inv_freq"], torch.bfloat16)
    assert torch.equal(kfar, g["k_far_group"])
    qpos = torch.full((1, 1), g.meta["ctx"] - 1)
    qg = orc.rotate_bshd(g["q_base"], orc.regroup_delta(qpos, G), g["inv_freq"], torch.bfloat16)
    assert torch.equal(qg, g["q_group"])


def test_rotation_helpers(golden):
    g = golden("rotate.npz")
    x = g["x"].transpose(1, 2)                      # (B,S,H,D)
    delta = g["delta"]
    r = orc.rotate_bshd(x, delta, g["inv_freq"], torch.bfloat16).transpose(1, 2)
    assert torch.equal(r, g["rot_tests"]) and torch.equal(r, g["rot_model"])
    rb = orc.rotate_bshd(x, g["pos"], g["inv_freq"], torch.bfloat16).transpose(1, 2)
    assert torch.equal(rb, g["base_model"])
    # fp32 operand, bf16-rounded tables: what the reference helper does when handed fp32 data
    r32 = orc.rotate_bshd(x.float(), delta, g["inv_freq"], torch.float32).transpose(1, 2)
    _close(r32, g["rot_fp32"], 1e-6)
    assert torch.allclose(orc.default_inv_freq(128, 1.0e6), g["inv_freq"], rtol=0, atol=0)


def test_merge_nway_and_two_way(golden):
    g = golden("merge_nway.npz")
    out, lse = orc.merge_partials(g["o_parts"], g["lse_parts"])
    _close(out, g["out"]); _close(lse, g["lse"])
    o2, _ = orc.merge2(g["o_parts"][0], g["lse_parts"][0], g["o_parts"][1], g["lse_parts"][1])
    _close(o2, g["out_two"])


def test_merge_rounded_matches_fp32_within_storage_rounding(golden):
    g = golden("merge_nway.npz")
    o, l = g["o_parts"], g["lse_parts"]
    l = torch.where(torch.isfinite(l), l, torch.full_like(l, -30.0))
    r = orc.merge2_rounded(o[0], l[0], o[1], l[1])
    e, _ = orc.merge2(o[0], l[0], o[1], l[1])
    d, cos = orc.compare(r, e)
    assert d < 5e-2 and cos > 0.9999


def test_model_boundary_operands(golden):
    """q/k operands built by the oracle from positions equal what the unmodified reference
    modeling file handed to its backend (fp32 run: tolerance; bf16 run: via attention output)."""
    g = golden("model_tiny.npz")
    w, w0, S = g.meta["w"], g.meta["w0"], g.meta["S_prefill"]
    for tag in ("fp32", "bf16"):
        p = {k: g[f"{tag}::prefill::{k}"] for k in ("q_base", "q_group", "k_base", "k_group", "v", "out")}
        out, _ = orc.jetlong_prefill(p["q_base"], p["q_group"], p["k_base"], p["k_group"], p["v"],
                                     seqstart=int(g[f"{tag}::prefill::seqstart"]), w0=w0)
        _close(out, p["out"], 2e-5 if tag == "fp32" else 1e-2)
        d = {k: g[f"{tag}::decode::{k}"] for k in ("q_base", "q_group", "k_near", "v_near", "k_far", "v_far", "out")}
        assert d["k_near"].shape[1] == w0 + 1 and d["k_far"].shape[1] == S - w0
        assert int(g[f"{tag}::decode::G"]) == orc.group_size_for(S, w)
        out, _ = orc.jetlong_decode(d["q_base"], d["q_group"], d["k_near"], d["v_near"], d["k_far"], d["v_far"])
        _close(out, d["out"], 2e-5 if tag == "fp32" else 1e-2)
    # regrouping identity on the fp32 run: q_group = rotate(q_base, floor(p/G)-p)
    G = orc.group_size_for(S - 1, w)
    pos = torch.arange(S).view(1, S)
    qb, qg = g["fp32::prefill::q_base"], g["fp32::prefill::q_group"]
    _close(orc.rotate_bshd(qb, orc.regroup_delta(pos, G), orc.default_inv_freq()), qg, 1e-5)


def _posmap_case(g, kind, params):
    S = g.meta["S"]
    q, k, v = g["q_raw"], g["k_raw"], g["v"]
    pos = torch.arange(S + 1)
    out, _ = orc.posmap_attention(kind, q[:, :S], k[:, :S], v[:, :S], q_positions=pos[:S], k_positions=pos[:S],
                                  params=params, inv_freq=g["inv_freq"])
    _close(out, g["out_prefill"], 1e-5)
    out, _ = orc.posmap_attention(kind, q[:, S:], k, v, q_positions=pos[S:], k_positions=pos,
                                  params=params, inv_freq=g["inv_freq"])
    _close(out, g["out_decode"], 1e-5)


def test_posmap_selfext(golden):
    g = golden("selfext_tiny.npz")
    _posmap_case(g, "selfext", dict(window_size=g.meta["window_size"], group_size=g.meta["group_size"]))


def test_posmap_dca(golden):
    g = golden("dca_tiny.npz")
    _posmap_case(g, "dca", dict(chunk_size=g.meta["chunk_size"], local_window=g.meta["local_window"]))


def test_jetlong_freq_against_the_reference_module(golden):
    """Fixture: the reference's jetlong_freq attention module (fp32, eager stand-in for its flash-attn calls)."""
    g = golden("jetlong_freq_tiny.npz")
    S, w, w0 = g.meta["S"], g.meta["w"], g.meta["w_0"]
    inv = g["inv_freq"]
    ramp = orc.yarn_ramp(128, w, 1.0e6)
    _close(ramp, g["ntk_ramp"], 1e-7)
    q, k, v = g["q_raw"], g["k_raw"], g["v"]
    pos = torch.arange(S + 1).view(1, -1)
    for tag, l_curr, qs, ks, want in (("prefill", S, slice(0, S), slice(0, S), g["out_prefill"]),
                                      ("decode", S + 1, slice(S, S + 1), slice(0, S + 1), g["out_decode"])):
        delta, scale = orc.jetlong_freq_params(l_curr, w, w0, inv, ramp)
        _close(delta, g[f"delta_inv_freq_{tag}"], 1e-9)
        assert abs(scale - g.meta[f"attn_scale_{tag}"]) < 1e-7
        out, _ = orc.jetlong_freq_attention(q[:, qs], k[:, ks], v[:, ks], q_positions=pos[:, qs], k_positions=pos[:, ks],
                                            w_0=w0, inv_freq=inv, delta_inv_freq=delta, scale=scale)
        _close(out, want, 2e-5)


def test_posmap_jetlong_equals_two_branch(golden):
    g = golden("model_tiny.npz")
    S, w, w0 = g.meta["S_prefill"], g.meta["w"], g.meta["w0"]
    G = orc.group_size_for(S - 1, w)
    torch.manual_seed(0)
    q = torch.randn(1, 96, 4, 128); k = torch.randn(1, 96, 2, 128); v = torch.randn(1, 96, 2, 128)
    pos = torch.arange(96) + 1000
    out, lse = orc.posmap_attention("jetlong", q, k, v, q_positions=pos, k_positions=pos,
                                    params=dict(w_0=w0, G=G), inv_freq=orc.default_inv_freq())
    # the two-step rotation (base, then correction) differs from the direct rotation only by fp32 angle rounding
    qb, qg, kb, kg = orc.jetlong_operands(q, k, q_positions=pos.view(1, -1), k_positions=pos.view(1, -1),
                                          group_size=G, inv_freq=orc.default_inv_freq())
    out2, lse2 = orc.jetlong_prefill(qb, qg, kb, kg, v, seqstart=0, w0=w0)
    _close(out, out2, 1e-4); _close(lse, lse2, 1e-4)

"""GPU parity: the CUDA kernels, called through the C ABI, against the golden fixtures produced by
the reference's own code and against the CPU oracle on seeded inputs.

Tolerances (bf16 kernels vs an fp32 oracle fed the same bf16 inputs): output max-abs <= 2e-2 and
cosine >= 0.9999; LSE max-abs <= 1e-3.
"""
import math

import pytest
import torch

import jetlong_oracle as orc

pytestmark = pytest.mark.gpu

OUT_TOL, COS_TOL, LSE_TOL = 2e-2, 0.9999, 1e-3


def _ops():
    from jetlm.kernels import jetlong_ops
    return jetlong_ops


def _check(out, lse, exp_out, exp_lse, what=""):
    d, cos = orc.compare(out.float().cpu(), exp_out)
    assert d <= OUT_TOL and cos >= COS_TOL, f"{what}: out max-abs {d:.3e} cos {cos:.6f}"
    if lse is not None:
        dl, _ = orc.compare(lse.float().cpu(), exp_lse)
        assert dl <= LSE_TOL, f"{what}: lse max-abs {dl:.3e}"


def _dev(*ts):
    return [t.cuda() for t in ts]


# ------------------------------------------------------------------------------------------------
# merge
# ------------------------------------------------------------------------------------------------

def test_merge_nway_golden(golden):
    g = golden("merge_nway.npz")
    o, l = g["o_parts"].cuda(), g["lse_parts"].cuda()
    out, lse = _ops().merge_partials(o, l)
    torch.cuda.synchronize()
    _check(out, lse, g["out"], g["lse"], "merge n-way")
    out2 = _ops().merge_partials([o[0], o[1]], [l[0], l[1]], return_lse=False)
    _check(out2, None, g["out_two"], None, "merge 2-way")


def test_merge2_bshd_reference_rounding(golden):
    from jetlm.kernels.merge_fused import merge2_bshd
    torch.manual_seed(4)
    a = torch.randn(2, 37, 8, 128).bfloat16()
    b = torch.randn(2, 37, 8, 128).bfloat16()
    la, lb = torch.randn(2, 8, 37) * 2, torch.randn(2, 8, 37) * 2
    exp = orc.merge2_rounded(a, la, b, lb)
    got = merge2_bshd(a.cuda(), la.cuda(), b.cuda(), lb.cuda()).cpu()
    # identical op sequence; the device exp/divide may differ in the last bit before the bf16 rounding
    diff = (got.float() - exp.float()).abs()
    assert float(diff.max()) <= 2 ** -6 and float((diff > 0).float().mean()) < 0.02
    out = torch.empty_like(a).cuda()
    assert merge2_bshd(a.cuda(), la.cuda(), b.cuda(), lb.cuda(), out=out).data_ptr() == out.data_ptr()


@pytest.mark.parametrize("n", [1, 3, 8, 16])
def test_merge_random(n):
    torch.manual_seed(n)
    o = torch.randn(n, 1, 130, 4, 128).bfloat16()
    l = torch.randn(n, 1, 4, 130) * 4
    l[0, 0, 1, 5] = -float("inf")
    eo, el = orc.merge_partials(o, l)
    out, lse = _ops().merge_partials(o.cuda(), l.cuda())
    _check(out, lse, eo, el, f"merge n={n}")


def test_merge_all_empty_row():
    o = torch.randn(2, 1, 2, 2, 128).bfloat16()
    l = torch.full((2, 1, 2, 2), -float("inf"))
    out, lse = _ops().merge_partials(o.cuda(), l.cuda())
    assert torch.all(out == 0) and torch.all(torch.isinf(lse) & (lse < 0))


# ------------------------------------------------------------------------------------------------
# rotate
# ------------------------------------------------------------------------------------------------

def test_rotate_golden_and_large_positions(golden):
    ops = _ops()
    g = golden("rotate.npz")
    x = g["x"].transpose(1, 2).contiguous()            # (B,S,H,D) bf16
    inv = g["inv_freq"]
    pos0 = int(g["pos"][0, 0])
    G = g.meta["G"]
    got = ops.rope_regroup(x.cuda(), inv.cuda(), group_size=G, pos0=pos0).cpu()
    exp = g["rot_fp32"].transpose(1, 2)
    d, cos = orc.compare(got.float(), exp)
    assert d <= 2 ** -6 and cos > 0.99999, (d, cos)    # one bf16 rounding of an fp32-exact rotation
    S = x.shape[1]
    for p0 in (0, 131072 - S, 1048576 - S):
        pos = (torch.arange(S) + p0).view(1, S)
        exp = orc.rotate_bshd(x.float(), pos, inv)
        got = ops.rope_base(x.cuda(), inv.cuda(), pos0=p0).cpu()
        d, cos = orc.compare(got.float(), exp)
        assert d <= 2 ** -5 and cos > 0.99999, (p0, d, cos)


def test_rotate_strided_into_cache():
    ops = _ops()
    torch.manual_seed(1)
    inv = orc.default_inv_freq()
    x = torch.randn(2, 50, 2, 128).bfloat16()
    cache = torch.zeros(2, 2, 96, 128, dtype=torch.bfloat16, device="cuda")      # (B,Hk,S,D)
    ops.rope_base(x.cuda(), inv.cuda(), pos0=7, out=cache.transpose(1, 2)[:, 7:57])
    exp = orc.rotate_bshd(x.float(), (torch.arange(50) + 7).view(1, -1).expand(2, -1), inv)
    d, _ = orc.compare(cache.transpose(1, 2)[:, 7:57].float().cpu(), exp)
    assert d <= 2 ** -5
    assert torch.all(cache[:, :, :7] == 0) and torch.all(cache[:, :, 57:] == 0)


@pytest.mark.parametrize("hidden", [2048, 2560, 4096])
def test_rmsnorm_fused_pass(hidden):
    """One-pass RMSNorm (+ residual add) reproduces Qwen3RMSNorm's bf16 results."""
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RMSNorm
    ops = _ops()
    torch.manual_seed(hidden)
    x = (torch.randn(3, 37, hidden) * 2).bfloat16()
    res = torch.randn(3, 37, hidden).bfloat16()
    norm = Qwen3RMSNorm(hidden, eps=1e-6).bfloat16()
    norm.weight.data = (1 + 0.3 * torch.randn(hidden)).bfloat16()
    exp = norm(x)
    got = ops.rmsnorm(x.cuda(), norm.weight.data.cuda(), eps=1e-6).cpu()
    diff = (got.float() - exp.float()).abs()
    assert float((diff > 0).float().mean()) < 0.01 and float(diff.max()) <= 2 ** -5      # rsqrt last-bit differences only
    s_exp = res + x
    summed, got2 = ops.rmsnorm(x.cuda(), norm.weight.data.cuda(), eps=1e-6, residual=res.cuda())
    assert torch.equal(summed.cpu(), s_exp)
    diff = (got2.cpu().float() - norm(s_exp).float()).abs()
    assert float((diff > 0).float().mean()) < 0.01 and float(diff.max()) <= 2 ** -5


def test_silu_mul_fused_pass():
    """silu(gate) * up in one pass against torch's two bf16 ops: at most one bf16 step apart, and only rarely."""
    ops = _ops()
    torch.manual_seed(8)
    g = (torch.randn(3, 1000, 1536, device="cuda") * 3).bfloat16()
    u = torch.randn(3, 1000, 1536, device="cuda").bfloat16()
    got = ops.silu_mul(g, u).float()
    want = (torch.nn.functional.silu(g) * u).float()
    diff = (got - want).abs()
    assert float((diff > 0).float().mean()) < 0.01 and float((diff / want.abs().clamp_min(1e-6)).max()) <= 2 ** -7
    with pytest.raises(ValueError):
        ops.silu_mul(g, u[:, :, :8])


def test_norm_rope_fused_pass():
    """RMSNorm + base RoPE + regroup in one kernel == Qwen3RMSNorm (its bf16 roundings) followed by the
    oracle's fp32 rotations; strided output straight into a (B,Hk,S,D) cache, block-cyclic positions."""
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RMSNorm
    ops = _ops()
    torch.manual_seed(17)
    B, S, H, D, G, p0 = 2, 300, 6, 128, 4, 100000
    inv = orc.default_inv_freq()
    x = (torch.randn(B, S, H, D) * 3).bfloat16()
    norm = Qwen3RMSNorm(D, eps=1e-6)
    norm.weight.data = (1 + 0.2 * torch.randn(D)).bfloat16().float()
    y = norm.bfloat16()(x)                                      # HF arithmetic on CPU, bf16 in / bf16 out
    pos = (torch.arange(S) + p0).view(1, S).expand(B, -1)
    eb = orc.rotate_bshd(y.float(), pos, inv)
    eg = orc.rotate_bshd(eb, orc.regroup_delta(pos, G), inv)
    base, grp = ops.norm_rope(x.cuda(), norm.weight.data.bfloat16().cuda(), inv.cuda(), eps=1e-6, pos0=p0, group_size=G)
    for got, exp in ((base, eb), (grp, eg)):
        d, cos = orc.compare(got.float().cpu(), exp)
        assert d <= 2 ** -4 and cos > 0.99998, (d, cos)          # |y| up to ~8: one bf16 ulp there is 2^-5
    cache = torch.zeros(B, H, S + 9, D, dtype=torch.bfloat16, device="cuda")
    ops.norm_rope(x.cuda(), norm.weight.data.bfloat16().cuda(), inv.cuda(), eps=1e-6, pos0=p0,
                  out_base=cache.transpose(1, 2)[:, 4:4 + S])
    assert torch.equal(cache.transpose(1, 2)[:, 4:4 + S], base) and torch.all(cache[:, :, :4] == 0)
    # block-cyclic stripe positions: rows of rank 1 of 2 with block 128
    Sb = 256
    rows = torch.cat([torch.arange(128, 256), torch.arange(384, 512)])
    xs = x[:, :Sb]
    ys = y[:, :Sb]
    posb = (rows + p0).view(1, -1).expand(B, -1)
    exp = orc.rotate_bshd(ys.float(), posb, inv)
    got = ops.norm_rope(xs.cuda().contiguous(), norm.weight.data.bfloat16().cuda(), inv.cuda(), eps=1e-6, pos0=p0 + 128,
                        pos_block=128, pos_block_stride=256)
    d, cos = orc.compare(got.float().cpu(), exp)
    assert d <= 2 ** -4 and cos > 0.99998, (d, cos)


# ------------------------------------------------------------------------------------------------
# prefill
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("impl", [0, 1, 2])
@pytest.mark.parametrize("name", ["prefill_fresh.npz", "prefill_chunked.npz"])
def test_prefill_golden(golden, name, impl):
    g = golden(name)
    qb, qg, kb, kg, v = _dev(*(g[k] for k in ("q_base", "q_group", "k_base", "k_group", "v")))
    B = qb.shape[0]
    ss = g.meta["seqstart"]
    out, lse = _ops().jetlong_prefill(qb, qg, kb, kg, v, seqstart_q=torch.full((B,), ss, dtype=torch.int32, device="cuda"),
                                      seqstart_q_scalar=ss, window_size_left=g.meta["w0"], impl=impl)
    _check(out, lse, g["out"], g["lse"], f"{name} impl={impl}")


def _prefill_case(seed, B, S, Skv, H, Hk, w0, impl, strided=False, q_scale=1.0, k_ramp=0.0):
    torch.manual_seed(seed)
    D = 128
    qb, qg = torch.randn(B, S, H, D).bfloat16(), torch.randn(B, S, H, D).bfloat16()
    kb, kg, v = (torch.randn(B, Skv, Hk, D).bfloat16() for _ in range(3))
    qb, qg = (qb.float() * q_scale).bfloat16(), (qg.float() * q_scale).bfloat16()
    if q_scale != 1.0:   # near one-hot rows return single values of V: keep them below 1 so that a bf16 step stays under the tolerance
        v = (v.float() * 0.25).bfloat16()
    if k_ramp:      # key norms grow with the position: the row maximum keeps rising from tile to tile
        r = (1.0 + k_ramp * torch.arange(Skv).float() / Skv).view(1, Skv, 1, 1)
        kb, kg = (kb.float() * r).bfloat16(), (kg.float() * r).bfloat16()
    eo, el = orc.jetlong_prefill(qb, qg, kb, kg, v, seqstart=Skv - S, w0=w0)
    dq, dqg, dkb, dkg, dv = _dev(qb, qg, kb, kg, v)
    if strided:   # (B,H,S,D) storage viewed as (B,S,H,D), the layout the modeling file hands over
        dq, dqg, dkb, dkg, dv = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (dq, dqg, dkb, dkg, dv))
    out, lse = _ops().posmap_prefill([dq, dqg], [dkb, dkg], dv, pmap=_ops().PositionMap.jetlong(w0),
                                     q_pos0=Skv - S, impl=impl)
    _check(out, lse, eo, el, f"prefill seed={seed} S={S} Skv={Skv} w0={w0} impl={impl}")


@pytest.mark.parametrize("impl", [0, 1, 2])
@pytest.mark.parametrize("S,Skv,w0", [(1, 1, 0), (5, 5, 0), (64, 64, 1), (127, 127, 63), (128, 128, 64), (129, 129, 65),
                                      (300, 300, 0), (300, 300, 1000), (257, 257, 128), (96, 480, 100), (2, 700, 31),
                                      (384, 384, 127), (384, 384, 128), (384, 384, 129)])
def test_prefill_shapes(S, Skv, w0, impl):
    _prefill_case(S * 7 + w0, 1, S, Skv, 4, 2, w0, impl)


@pytest.mark.parametrize("impl", [0, 2])
@pytest.mark.parametrize("q_scale,k_ramp,w0", [(6.0, 0.0, 300), (30.0, 0.0, 300), (4.0, 20.0, 3000), (20.0, 8.0, 100)])
def test_prefill_row_maximum_jumps(q_scale, k_ramp, w0, impl):
    """Scores whose row maximum jumps by far more than 2^8 between key tiles, again and again: the running
    reference of the online softmax is raised and the output accumulator rescaled many times per row (in the
    CTA-pair kernel by either of the two threads that share a row)."""
    _prefill_case(11, 1, 1024, 2048, 4, 2, w0, impl, q_scale=q_scale, k_ramp=k_ramp)
    _prefill_case(12, 1, 1500, 2300, 8, 4, w0, impl, q_scale=q_scale, k_ramp=k_ramp)


@pytest.mark.parametrize("impl", [0, 1, 2])
def test_prefill_batch_heads_strided(impl):
    _prefill_case(5, 2, 200, 328, 8, 2, 50, impl, strided=True)
    _prefill_case(6, 1, 260, 260, 6, 6, 77, impl)


@pytest.mark.parametrize("impl", [0, 1, 2])
def test_prefill_config1_geometry(impl):
    """16 query heads, 8 kv heads, head_dim 128, S = 4096, w_0 = 1024, real regrouped operands (G = 2)."""
    torch.manual_seed(0)
    B, S, H, Hk, D, w0, G = 1, 4096, 16, 8, 128, 1024, 2
    q, k, v = torch.randn(B, S, H, D), torch.randn(B, S, Hk, D), torch.randn(B, S, Hk, D)
    pos = torch.arange(S).view(1, S)
    qb, qg, kb, kg = orc.jetlong_operands(q, k, q_positions=pos, k_positions=pos, group_size=G,
                                          inv_freq=orc.default_inv_freq())
    qb, qg, kb, kg, v = (t.bfloat16() for t in (qb, qg, kb, kg, v))
    eo, el = orc.jetlong_prefill(qb, qg, kb, kg, v, seqstart=0, w0=w0)
    out, lse = _ops().posmap_prefill(_dev(qb, qg), _dev(kb, kg), v.cuda(), pmap=_ops().PositionMap.jetlong(w0),
                                     q_pos0=0, impl=impl)
    _check(out, lse, eo, el, f"config-1 impl={impl}")


def test_prefill_impls_agree_large():
    """At a size the CPU oracle cannot reach, the three GPU kernels must agree with each other."""
    torch.manual_seed(9)
    B, S, H, Hk, D, w0 = 1, 8192 + 37, 4, 2, 128, 2048
    ts = [torch.randn(B, S, h, D, device="cuda").bfloat16() for h in (H, H, Hk, Hk, Hk)]
    pm = _ops().PositionMap.jetlong(w0)
    o0, l0 = _ops().posmap_prefill(ts[:2], ts[2:4], ts[4], pmap=pm, q_pos0=0, impl=0)
    o1, l1 = _ops().posmap_prefill(ts[:2], ts[2:4], ts[4], pmap=pm, q_pos0=0, impl=1)
    o2, l2 = _ops().posmap_prefill(ts[:2], ts[2:4], ts[4], pmap=pm, q_pos0=0, impl=2)
    _check(o0, l0, o1.float().cpu(), l1.cpu(), "impl 0 vs impl 1")
    _check(o2, l2, o1.float().cpu(), l1.cpu(), "impl 2 vs impl 1")


@pytest.mark.parametrize("S,H,Hk,w0,impl", [(65536, 16, 8, 32768, 0), (131072, 32, 8, 32768, 0), (65536, 16, 8, 32768, 2)])
def test_prefill_full_size_spot_rows(S, H, Hk, w0, impl):
    """The benchmark geometries (Qwen3-1.7B at 65536 tokens, Qwen3-4B/8B at 131072 tokens, w_0 = 32768) in one
    launch; sampled (row, head) pairs — first rows, both sides of the class boundary, tile edges, the last
    row — are recomputed by the fp32 oracle from the same bf16 operands."""
    ops = _ops()
    torch.manual_seed(S // 1024 + H)
    D = 128
    mk = lambda h: torch.randn(1, S, h, D, device="cuda").bfloat16()
    qb, qg, kb, kg, v = mk(H), mk(H), mk(Hk), mk(Hk), mk(Hk)
    out, lse = ops.posmap_prefill([qb, qg], [kb, kg], v, pmap=ops.PositionMap.jetlong(w0), q_pos0=0, impl=impl)
    assert _native_status_clean()
    rows = [0, 1, 127, 128, 255, 256, w0 - 1, w0, w0 + 1, w0 + 129, S // 2 + 77, S - w0 - 1, S - 257, S - 1]
    rep = H // Hk
    for i, r in enumerate(rows):
        h = (7 * i + 3) % H
        kvh = h // rep
        sl = lambda t, hh: t[:, : r + 1, hh: hh + 1].float().cpu()
        eo, el = orc.jetlong_prefill(qb[:, r: r + 1, h: h + 1].float().cpu(), qg[:, r: r + 1, h: h + 1].float().cpu(),
                                     sl(kb, kvh), sl(kg, kvh), sl(v, kvh), seqstart=r, w0=w0)
        _check(out[:, r: r + 1, h: h + 1], lse[:, h: h + 1, r: r + 1], eo, el, f"S={S} row {r} head {h}")


def _native_status_clean():
    from jetlm.kernels import _native
    torch.cuda.synchronize()
    return _native.lib().jl_prefill_status() == 0


@pytest.mark.parametrize("impl", [0, 2])
def test_prefill_stripe_batching_matches_per_stripe_launches(impl):
    """Stripe batching (the sequence-parallel Q exchange): the block-cyclic query stripes of four ranks against one
    key tensor in two launches (stripes 1,2 and 3,0 - the second wraps) == one launch per stripe, bit for bit; the
    per-stripe form is the one the block-cyclic tests check against the oracle."""
    ops = _ops()
    torch.manual_seed(21)
    W, blk, S_loc, H, Hk, D, w0 = 4, 256, 512, 4, 2, 128, 300
    Skv = W * S_loc
    q, qg = (torch.randn(W, S_loc, H, D, device="cuda").bfloat16() for _ in range(2))
    k, kg, v = (torch.randn(1, Skv, Hk, D, device="cuda").bfloat16() for _ in range(3))
    pm = ops.PositionMap.jetlong(w0)
    geo = dict(q_block=blk, q_block_stride=W * blk)
    ref_o, ref_l = [], []
    for r in range(W):
        o, l = ops.posmap_prefill([q[r:r + 1], qg[r:r + 1]], [k, kg], v, pmap=pm, q_pos0=r * blk, impl=impl, **geo)
        ref_o.append(o)
        ref_l.append(l)
    out = torch.full((W, S_loc, H, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    lse = torch.full((W, H, S_loc), float("nan"), device="cuda")
    ops.posmap_prefill([q, qg], [k, kg], v, pmap=pm, q_pos0=0, impl=impl, out=out, lse=lse, stripes=(1, 2, blk), **geo)
    assert torch.isnan(out[0].float()).all() and torch.isnan(out[3].float()).all()          # untouched stripes
    ops.posmap_prefill([q, qg], [k, kg], v, pmap=pm, q_pos0=0, impl=impl, out=out, lse=lse, stripes=(3, 2, blk), **geo)
    assert torch.equal(out, torch.cat(ref_o)) and torch.equal(lse, torch.cat(ref_l))
    assert _native_status_clean()


@pytest.mark.parametrize("impl", [0, 2])
def test_prefill_block_cyclic_keys(impl):
    """A rank's block-cyclic stripe of the keys + merge of the stripes == attention over all keys."""
    ops = _ops()
    torch.manual_seed(12)
    B, S, H, Hk, D, w0, blk, R = 1, 512, 4, 2, 128, 100, 128, 2
    qb, qg = torch.randn(B, S, H, D).bfloat16(), torch.randn(B, S, H, D).bfloat16()
    kb, kg, v = (torch.randn(B, S, Hk, D).bfloat16() for _ in range(3))
    eo, el = orc.jetlong_prefill(qb, qg, kb, kg, v, seqstart=0, w0=w0)
    outs, lses = [], []
    for r in range(R):
        idx = torch.cat([torch.arange(b0, b0 + blk) for b0 in range(r * blk, S, R * blk)])
        o, l = ops.posmap_prefill(_dev(qb, qg), _dev(kb[:, idx].contiguous(), kg[:, idx].contiguous()),
                                  v[:, idx].contiguous().cuda(), pmap=ops.PositionMap.jetlong(w0), q_pos0=0,
                                  k_pos0=r * blk, k_block=blk, k_block_stride=R * blk, impl=impl)
        outs.append(o)
        lses.append(l)
    out, lse = ops.merge_partials(outs, lses)
    _check(out, lse, eo, el, "block-cyclic stripes")


# ------------------------------------------------------------------------------------------------
# decode
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("splits", [0, 1, 4, 7])
def test_decode_golden_pregrouped(golden, splits):
    g = golden("decode_regrouped.npz")
    b = g.meta["boundary"]
    kc, vc, kfg, qb, qg = _dev(g["k_cache_base"], g["v_cache"], g["k_far_group"], g["q_base"], g["q_group"])
    B, H = qb.shape[0], qb.shape[2]
    lse = torch.empty(B, H, 1, device="cuda")
    out, lse = _ops().jetlong_decode(qb, qg, kc[:, b:], vc[:, b:], kfg, vc[:, :b],
                                     seqused_near=torch.full((B,), kc.shape[1] - b, dtype=torch.int32, device="cuda"),
                                     seqused_distant=torch.full((B,), b, dtype=torch.int32, device="cuda"),
                                     inv_freq=g["inv_freq"].cuda(), group_size=g.meta["G"], lse=lse,
                                     num_splits=splits, distant_k_grouped=True)
    _check(out, lse.squeeze(-1).unsqueeze(-1), g["out"], g["lse"], f"decode golden splits={splits}")


def test_decode_golden_in_kernel_regroup(golden):
    """Far keys regrouped inside the kernel from the base-rotated cache, read in place."""
    g = golden("decode_regrouped.npz")
    b = g.meta["boundary"]
    kc, vc, qb, qg = _dev(g["k_cache_base"], g["v_cache"], g["q_base"], g["q_group"])
    B, H = qb.shape[0], qb.shape[2]
    ops = _ops()
    segs = [ops.KvSegment(kc[:, :b], vc[:, :b], q_class=1, rotate=True, pos0=0), ops.KvSegment(kc[:, b:], vc[:, b:], q_class=0)]
    out, lse = ops.decode_segments([qb, qg], segs, inv_freq=g["inv_freq"].cuda(), group_size=g.meta["G"])
    # oracle: exact fp32 regrouping of the bf16 cache (the fixture's far keys carry the reference's bf16 table rounding)
    pos = torch.arange(b).view(1, b)
    kfar = orc.rotate_bshd(g["k_cache_base"][:, :b].float(), orc.regroup_delta(pos, g.meta["G"]), g["inv_freq"])
    eo, el = orc.jetlong_decode(g["q_base"], g["q_group"], g["k_cache_base"][:, b:], g["v_cache"][:, b:], kfar, g["v_cache"][:, :b])
    _check(out, lse, eo, el, "decode in-kernel regroup")
    _check(out, None, g["out"], None, "decode in-kernel regroup vs reference fixture")


def test_decode_near_heavy_golden(golden):
    g = golden("decode_near_heavy.npz")
    qb, qg, kn, vn, kf, vf = _dev(*(g[k] for k in ("q_base", "q_group", "k_near", "v_near", "k_far", "v_far")))
    ops = _ops()
    out, lse = ops.decode_segments([qb, qg], [ops.KvSegment(kf, vf, 1), ops.KvSegment(kn, vn, 0)], num_splits=4)
    _check(out, lse, g["out"], g["lse"], "decode near-heavy")


@pytest.mark.parametrize("B,H,Hk,near,far", [(1, 8, 4, 1, 1), (2, 16, 8, 33, 224), (3, 32, 8, 513, 1500), (1, 16, 16, 64, 64),
                                            (1, 32, 8, 4097, 12000)])
def test_decode_shapes_strided_cache(B, H, Hk, near, far):
    """(B,Hk,S,D) cache read in place through strides; per-sequence valid lengths on the far segment."""
    ops = _ops()
    torch.manual_seed(B * 100 + near)
    D = 128
    ctx = near + far
    qb, qg = torch.randn(B, 1, H, D).bfloat16(), torch.randn(B, 1, H, D).bfloat16()
    kc = torch.randn(B, Hk, ctx + 5, D).bfloat16()
    vc = torch.randn(B, Hk, ctx + 5, D).bfloat16()
    kv, vv = kc.transpose(1, 2), vc.transpose(1, 2)
    eo, el = orc.jetlong_decode(qb, qg, kv[:, far:ctx], vv[:, far:ctx], kv[:, :far], vv[:, :far])
    dk, dv = kc.cuda().transpose(1, 2), vc.cuda().transpose(1, 2)
    segs = [ops.KvSegment(dk[:, :far], dv[:, :far], 1), ops.KvSegment(dk[:, far:ctx], dv[:, far:ctx], 0)]
    out, lse = ops.decode_segments(_dev(qb, qg), segs)
    _check(out, lse, eo, el, f"decode B={B} H={H} near={near} far={far}")
    # per-sequence lengths: sequence 0 only sees the first far//2 far keys
    lens = torch.full((B,), far, dtype=torch.int32)
    lens[0] = far // 2
    segs[0].len_dev = lens.cuda()
    out, lse = ops.decode_segments(_dev(qb, qg), segs)
    eo0, el0 = orc.jetlong_decode(qb[:1], qg[:1], kv[:1, far:ctx], vv[:1, far:ctx], kv[:1, :far // 2], vv[:1, :far // 2])
    _check(out[:1], lse[:1], eo0, el0, "decode with device lengths")


def test_decode_kv_shards_merge():
    """Splitting the keys into per-rank shards, decoding each and merging == decoding everything."""
    ops = _ops()
    torch.manual_seed(21)
    B, H, Hk, D, ctx, w0, G, R = 1, 8, 2, 128, 2000, 300, 3, 4
    inv = orc.default_inv_freq()
    qb, qg = torch.randn(B, 1, H, D).bfloat16(), torch.randn(B, 1, H, D).bfloat16()
    kc, vc = torch.randn(B, ctx, Hk, D).bfloat16(), torch.randn(B, ctx, Hk, D).bfloat16()
    boundary = ctx - 1 - w0
    pos = torch.arange(boundary).view(1, -1)
    kfar = orc.rotate_bshd(kc[:, :boundary].float(), orc.regroup_delta(pos, G), inv)
    eo, el = orc.jetlong_decode(qb, qg, kc[:, boundary:], vc[:, boundary:], kfar, vc[:, :boundary])
    dk, dv, dqb, dqg = _dev(kc, vc, qb, qg)
    outs, lses = [], []
    per = ctx // R
    for r in range(R):
        lo, hi = r * per, (r + 1) * per if r < R - 1 else ctx
        segs = []
        if lo < boundary:
            segs.append(ops.KvSegment(dk[:, lo:min(hi, boundary)], dv[:, lo:min(hi, boundary)], 1, rotate=True, pos0=lo))
        if hi > boundary:
            segs.append(ops.KvSegment(dk[:, max(lo, boundary):hi], dv[:, max(lo, boundary):hi], 0))
        o, l = ops.decode_segments([dqb, dqg], segs, inv_freq=inv.cuda(), group_size=G)
        outs.append(o)
        lses.append(l)
    out, lse = ops.merge_partials(outs, lses)
    _check(out, lse, eo, el, "sharded decode + merge")


@pytest.mark.parametrize("B,H,Hk,near,far,splits,blk", [(1, 32, 8, 300, 1000, 0, 0), (2, 16, 8, 17, 513, 5, 0), (1, 64, 16, 129, 2050, 0, 0),
                                                       (3, 8, 8, 1, 95, 1, 0), (1, 32, 8, 700, 4096, 0, 256)])
def test_decode_in_kernel_regroup_shared_angle_kernel(B, H, Hk, near, far, splits, blk):
    """kv_heads a multiple of 8 and a rotating segment: the call runs on the kernel that forms every rotation angle
    once for eight kv heads (one CTA per key range, one warp per kv head).  Ragged lengths, several split counts,
    per-sequence lengths on the far segment, and a block-cyclic stripe (positions p0 + (row // blk) * 4 * blk + row % blk)."""
    ops = _ops()
    torch.manual_seed(B * 1000 + far)
    D, G = 128, 5
    inv = orc.default_inv_freq()
    qb, qg = torch.randn(B, 1, H, D).bfloat16(), torch.randn(B, 1, H, D).bfloat16()
    ctx = near + far
    kc = torch.randn(B, Hk, ctx, D).bfloat16().transpose(1, 2)          # (B,S,Hk,D) view of a (B,Hk,S,D) cache
    vc = torch.randn(B, Hk, ctx, D).bfloat16().transpose(1, 2)
    rows = torch.arange(far)
    pos = (1000 + (rows // blk) * 4 * blk + rows % blk) if blk else 1000 + rows
    geo = dict(pos0=1000, pos_block=blk, pos_block_stride=4 * blk) if blk else dict(pos0=1000)
    # the kernel rounds the regrouped keys to bf16 before the tensor cores read them, as the reference's own path
    # does (correction_rotate_per_sample returns bf16); with as few as 32 keys that rounding is visible in the LSE
    kfar = orc.rotate_bshd(kc[:, :far].float(), orc.regroup_delta(pos.view(1, -1).expand(B, -1), G), inv).bfloat16().float()
    eo, el = orc.jetlong_decode(qb, qg, kc[:, far:], vc[:, far:], kfar, vc[:, :far])
    dk, dv = kc.cuda(), vc.cuda()
    segs = [ops.KvSegment(dk[:, :far], dv[:, :far], 1, rotate=True, **geo), ops.KvSegment(dk[:, far:], dv[:, far:], 0)]
    out, lse = ops.decode_segments(_dev(qb, qg), segs, inv_freq=inv.cuda(), group_size=G, num_splits=splits)
    _check(out, lse, eo, el, f"shared-angle decode B={B} H={H}/{Hk} near={near} far={far} splits={splits} blk={blk}")
    if B > 1:          # per-sequence lengths: sequence 0 only sees the first far // 3 far keys
        lens = torch.full((B,), far, dtype=torch.int32)
        lens[0] = far // 3
        segs[0].len_dev = lens.cuda()
        out, lse = ops.decode_segments(_dev(qb, qg), segs, inv_freq=inv.cuda(), group_size=G, num_splits=splits)
        n0 = far // 3
        eo0, el0 = orc.jetlong_decode(qb[:1], qg[:1], kc[:1, far:], vc[:1, far:], kfar[:1, :n0], vc[:1, :n0])
        _check(out[:1], lse[:1], eo0, el0, "shared-angle decode with device lengths")


# ------------------------------------------------------------------------------------------------
# backend entry points on the tensors the unmodified reference modeling file produced
# ------------------------------------------------------------------------------------------------

def test_backend_entry_points_on_model_boundary(golden):
    from jetlm.kernels import cute_jetlong_backend as be
    g = golden("model_tiny.npz")
    w0 = g.meta["w0"]
    p = {k: g[f"bf16::prefill::{k}"] for k in ("q_base", "q_group", "k_base", "k_group", "v", "out")}
    bhsd = lambda t: t.cuda().transpose(1, 2)          # the modeling file hands over (B,H,S,D) views
    out = be.fused_jetlong_prefill(bhsd(p["q_base"]), bhsd(p["q_group"]), bhsd(p["k_base"]), bhsd(p["k_group"]), bhsd(p["v"]),
                                   seqstart_q=int(g["bf16::prefill::seqstart"]), window_size_left=w0,
                                   softmax_scale=128 ** -0.5, has_any_pad=False, training=False)
    assert out.shape == p["out"].shape
    eo, _ = orc.jetlong_prefill(p["q_base"], p["q_group"], p["k_base"], p["k_group"], p["v"],
                                seqstart=int(g["bf16::prefill::seqstart"]), w0=w0)
    _check(out, None, eo, None, "backend prefill")
    d = {k: g[f"bf16::decode::{k}"] for k in ("q_base", "q_group", "k_near", "v_near", "k_far", "v_far", "out")}
    out = be.fused_jetlong_decode(*(d[k].cuda() for k in ("q_base", "q_group", "k_near", "v_near", "k_far", "v_far")),
                                  inv_freq=orc.default_inv_freq().cuda(), group_size=int(g["bf16::decode::G"]),
                                  has_any_pad=False, training=False)
    eo, _ = orc.jetlong_decode(*(d[k] for k in ("q_base", "q_group", "k_near", "v_near", "k_far", "v_far")))
    _check(out, None, eo, None, "backend decode")
    _check(out, None, d["out"].float(), None, "backend decode vs reference bf16 output")


# ------------------------------------------------------------------------------------------------
# other position maps through the same kernels
# ------------------------------------------------------------------------------------------------

def _posmap_gpu(g, kind, impl=0):
    """Rotation kernels vs the fp32 oracle rotation; the attention kernel vs the oracle attention on
    the very operands the kernel consumed; and end to end vs the reference's own output."""
    ops = _ops()
    S = g.meta["S"]
    inv = g["inv_freq"]
    q, k, v = (g[n].bfloat16() for n in ("q_raw", "k_raw", "v"))
    dq, dk, dv, dinv = q.cuda(), k.cuda(), v.cuda(), inv.cuda()
    if kind == "selfext":
        W, Gs = g.meta["window_size"], g.meta["group_size"]
        params = dict(window_size=W, group_size=Gs)
        pm = ops.PositionMap.selfext(W)
        q_ops = lambda x, p0: [ops.rope_base(x, dinv, pos0=p0), ops.rope_rotate(x, dinv, pos0=p0, div=Gs, add=W - W // Gs)]
        k_ops = lambda x: [ops.rope_base(x, dinv), ops.rope_rotate(x, dinv, div=Gs)]
    else:
        s, w = g.meta["chunk_size"], g.meta["local_window"]
        params = dict(chunk_size=s, local_window=w)
        pm = ops.PositionMap.dca(s)
        q_ops = lambda x, p0: [ops.rope_rotate(x, dinv, pos0=p0, div_mul=0, mod=s, mod_mul=1),
                               ops.rope_rotate(x, dinv, pos0=p0, div_mul=0, mod=s, mod_mul=1, add=s, t_max=s + w),
                               ops.rope_rotate(x, dinv, pos0=p0, div_mul=0, add=s + w)]
        def k_ops(x):
            kr = ops.rope_rotate(x, dinv, div_mul=0, mod=s, mod_mul=1)
            return [kr, kr, kr]
    pos = torch.arange(S + 1)
    # (1) rotation kernels: one bf16 rounding away from the fp32 rotation at the class positions
    _, qpos, kpos = orc.posmap_classes(kind, pos[:S], pos[:S], params)
    qo, ko = q_ops(dq[:, :S], 0), k_ops(dk[:, :S])
    for got, x, pp in list(zip(qo, [q] * 3, qpos)) + list(zip(ko, [k] * 3, kpos)):
        exp = orc.rotate_bshd(x[:, :S].float(), pp.view(1, -1), inv)
        d, cos = orc.compare(got.float().cpu(), exp)
        assert d <= 2 ** -5 and cos > 0.99999, (kind, d, cos)
    # (2) attention kernel on those operands
    eo, el = orc.posmap_attention_from_operands(kind, [t.cpu() for t in qo], [t.cpu() for t in ko], v[:, :S],
                                                q_positions=pos[:S], k_positions=pos[:S], params=params)
    out, lse = ops.posmap_prefill(qo, ko, dv[:, :S], pmap=pm, q_pos0=0, impl=impl)
    _check(out, lse, eo, el, f"{kind} prefill")
    # (3) end to end against the reference's fp32 eager output (it never rounds inputs or operands to bf16)
    d, cos = orc.compare(out.float().cpu(), g["out_prefill"])
    assert d < 3e-2 and cos > 0.999, (kind, d, cos)
    # one decode step (query at position S over S + 1 keys) through the prefill kernel's Sq = 1 case
    qo, ko = q_ops(dq[:, S:], S), k_ops(dk)
    eo, el = orc.posmap_attention_from_operands(kind, [t.cpu() for t in qo], [t.cpu() for t in ko], v,
                                                q_positions=pos[S:], k_positions=pos, params=params)
    out, lse = ops.posmap_prefill(qo, ko, dv, pmap=pm, q_pos0=S, impl=impl)
    _check(out, lse, eo, el, f"{kind} decode-as-prefill")
    d, cos = orc.compare(out.float().cpu(), g["out_decode"])
    assert d < 3e-2 and cos > 0.999, (kind, d, cos)
    return qo, ko, dv, (eo, el)


def test_posmap_selfext(golden):
    g = golden("selfext_tiny.npz")
    ops = _ops()
    qo, ko, dv, (eo, el) = _posmap_gpu(g, "selfext")
    S, W = g.meta["S"], g.meta["window_size"]
    b = S + 1 - W                                            # keys [b, S] are the W neighbours
    segs = [ops.KvSegment(ko[1][:, :b], dv[:, :b], 1), ops.KvSegment(ko[0][:, b:], dv[:, b:], 0)]
    out, lse = ops.decode_segments(qo, segs)
    _check(out, lse, eo, el, "selfext decode kernel")


@pytest.mark.parametrize("kind", ["selfext", "dca"])
def test_posmap_maps_on_the_cta_pair_kernel(golden, kind):
    """The band map of self-extend and the three-class chunk map of DCA through the CTA-pair kernel."""
    _posmap_gpu(golden(kind + "_tiny.npz"), kind, impl=2)


def test_posmap_dca(golden):
    g = golden("dca_tiny.npz")
    ops = _ops()
    qo, ko, dv, (eo, el) = _posmap_gpu(g, "dca")
    S, s = g.meta["S"], g.meta["chunk_size"]
    n = S // s                                               # complete chunks before the query's chunk
    segs = [ops.KvSegment(ko[0][:, :s * (n - 1)], dv[:, :s * (n - 1)], 2),
            ops.KvSegment(ko[0][:, s * (n - 1):s * n], dv[:, s * (n - 1):s * n], 1),
            ops.KvSegment(ko[0][:, s * n:], dv[:, s * n:], 0)]
    out, lse = ops.decode_segments(qo, segs)
    _check(out, lse, eo, el, "dca decode kernel")


def test_jetlong_freq_prefill_and_decode(golden):
    """jetlong_freq through the band map: operands from jl_rotate with delta_inv_freq, one kernel pass with
    the temperature scale; decode corrects the far keys in-kernel.  Checked against the oracle on the very
    bf16 operands and, end to end, against the reference module's fp32 output."""
    from jetlm.kernels import cute_jetlong_backend as be
    g = golden("jetlong_freq_tiny.npz")
    ops = _ops()
    S, w, w0 = g.meta["S"], g.meta["w"], g.meta["w_0"]
    inv = g["inv_freq"]
    ramp = orc.yarn_ramp(128, w, 1.0e6)
    pos = torch.arange(S + 1).view(1, -1)
    q, k, v = g["q_raw"].bfloat16(), g["k_raw"].bfloat16(), g["v"].bfloat16()
    dq, dk, dv = _dev(q, k, v)
    qb = ops.rope_base(dq, inv.cuda())                      # (B,S+1,H,D) base-rotated, as the model caches them
    kb = ops.rope_base(dk, inv.cuda())
    bhsd = lambda x: x.transpose(1, 2)
    # prefill of S tokens
    delta, scale = orc.jetlong_freq_params(S, w, w0, inv, ramp)
    out = be.fused_jetlong_freq_prefill(bhsd(qb[:, :S]), bhsd(kb[:, :S]), bhsd(dv[:, :S]), delta_inv_freq=delta.cuda(),
                                        attn_scale=scale, seqstart_q=0, window_size_left=w0)
    qd = orc.rotate_bshd(qb[:, :S].float().cpu(), (pos[:, :S] - w0), delta)
    ky = orc.rotate_bshd(kb[:, :S].float().cpu(), pos[:, :S], delta)
    eo, _ = orc.posmap_attention_from_operands("jetlong", [qb[:, :S].cpu(), qd.bfloat16()], [kb[:, :S].cpu(), ky.bfloat16()],
                                               v[:, :S].bfloat16(), q_positions=pos[0, :S], k_positions=pos[0, :S],
                                               params=dict(w_0=w0, G=1), scale=scale)
    _check(out, None, eo, None, "jetlong_freq prefill")
    d, cos = orc.compare(out.float().cpu(), g["out_prefill"])
    assert d < 3e-2 and cos > 0.999, (d, cos)
    # decode of token S over S + 1 cached keys
    delta, scale = orc.jetlong_freq_params(S + 1, w, w0, inv, ramp)
    out, lse = be.fused_jetlong_freq_decode(qb[:, S:], bhsd(kb), bhsd(dv), delta_inv_freq=delta.cuda(), attn_scale=scale,
                                            max_q_pos=S, window_size_left=w0, return_lse=True)
    b = S - w0
    qd = orc.rotate_bshd(qb[:, S:].float().cpu(), torch.tensor([[b]]), delta).bfloat16()
    ky = orc.rotate_bshd(kb[:, :b].float().cpu(), pos[:, :b], delta)
    eo, el = orc.jetlong_decode(qb[:, S:].cpu(), qd, kb[:, b:].cpu(), v[:, b:].bfloat16(), ky, v[:, :b].bfloat16(), scale=scale)
    _check(out, lse, eo, el, "jetlong_freq decode")
    d, cos = orc.compare(out.float().cpu(), g["out_decode"])
    assert d < 3e-2 and cos > 0.999, (d, cos)


# ------------------------------------------------------------------------------------------------
# size-independent properties at full benchmark sizes
# ------------------------------------------------------------------------------------------------

def test_decode_full_context_properties():
    """ctx = 131072, 32/8 heads: (1) v == const => out == const, (2) split count does not change the
    result, (3) lse >= max score bound.  No CPU oracle is needed at this size."""
    ops = _ops()
    torch.manual_seed(3)
    B, H, Hk, D, ctx, w0 = 1, 32, 8, 128, 131072, 32768
    q = torch.randn(B, 1, H, D, device="cuda").bfloat16()
    qg = torch.randn(B, 1, H, D, device="cuda").bfloat16()
    k = torch.randn(B, ctx, Hk, D, device="cuda").bfloat16()
    v = torch.randn(B, ctx, Hk, D, device="cuda").bfloat16()
    b = ctx - 1 - w0
    segs = [ops.KvSegment(k[:, :b], v[:, :b], 1), ops.KvSegment(k[:, b:], v[:, b:], 0)]
    o_auto, l_auto = ops.decode_segments([q, qg], segs)
    o_8, l_8 = ops.decode_segments([q, qg], segs, num_splits=8)
    assert float((o_auto.float() - o_8.float()).abs().max()) <= 4e-3
    assert float((l_auto - l_8).abs().max()) <= 1e-4
    ones = torch.full_like(v, 0.5)
    segs1 = [ops.KvSegment(k[:, :b], ones[:, :b], 1), ops.KvSegment(k[:, b:], ones[:, b:], 0)]
    o_c, _ = ops.decode_segments([q, qg], segs1)
    assert float((o_c.float() - 0.5).abs().max()) <= 4e-3
    # spot rows against the oracle: one kv head, all its query heads
    eo, el = orc.jetlong_decode(q[:, :, :4].cpu(), qg[:, :, :4].cpu(), k[:, b:, :1].cpu(), v[:, b:, :1].cpu(),
                                k[:, :b, :1].cpu(), v[:, :b, :1].cpu())
    _check(o_auto[:, :, :4], l_auto[:, :4], eo, el, "decode 128K spot heads")


@pytest.mark.parametrize("kind", ["jetlong", "selfext", "dca"])
def test_position_maps_at_long_positions(kind):
    """The three position maps through the same rotate + prefill kernels at positions just below 131072
    (large RoPE angles), 8 query / 2 kv heads, a key count that is not a tile multiple.  The rotation
    kernels are checked against the fp32 rotation, the attention kernel against the oracle on the very
    operands it consumed."""
    ops = _ops()
    torch.manual_seed(40)
    B, S, H, Hk, D = 1, 2304 + 77, 8, 2, 128
    P0 = 131072 - S
    inv = orc.default_inv_freq()
    dinv = inv.cuda()
    q, k, v = torch.randn(B, S, H, D).bfloat16(), torch.randn(B, S, Hk, D).bfloat16(), torch.randn(B, S, Hk, D).bfloat16()
    dq, dk, dv = q.cuda(), k.cuda(), v.cuda()
    pos = torch.arange(S) + P0
    if kind == "jetlong":
        G, w0 = 4, 700
        params, pm = dict(w_0=w0, G=G), ops.PositionMap.jetlong(w0)
        qb, kb = ops.rope_base(dq, dinv, pos0=P0), ops.rope_base(dk, dinv, pos0=P0)
        qo = [qb, ops.rope_regroup(qb, dinv, group_size=G, pos0=P0)]
        ko = [kb, ops.rope_regroup(kb, dinv, group_size=G, pos0=P0)]
    elif kind == "selfext":
        Gs, W = 8, 512
        params, pm = dict(window_size=W, group_size=Gs), ops.PositionMap.selfext(W)
        qo = [ops.rope_base(dq, dinv, pos0=P0), ops.rope_rotate(dq, dinv, pos0=P0, div=Gs, add=W - W // Gs)]
        ko = [ops.rope_base(dk, dinv, pos0=P0), ops.rope_rotate(dk, dinv, pos0=P0, div=Gs)]
    else:
        s, w = 1024, 128
        params, pm = dict(chunk_size=s, local_window=w), ops.PositionMap.dca(s)
        qo = [ops.rope_rotate(dq, dinv, pos0=P0, div_mul=0, mod=s, mod_mul=1),
              ops.rope_rotate(dq, dinv, pos0=P0, div_mul=0, mod=s, mod_mul=1, add=s, t_max=s + w),
              ops.rope_rotate(dq, dinv, pos0=P0, div_mul=0, add=s + w)]
        kr = ops.rope_rotate(dk, dinv, pos0=P0, div_mul=0, mod=s, mod_mul=1)
        ko = [kr, kr, kr]
    _, qpos, kpos = orc.posmap_classes(kind, pos, pos, params)
    if kind == "jetlong":      # operands follow the reference's two-step composition: base, then correction by floor(p/G) - p
        exp_q = [orc.rotate_bshd(q.float(), pos.view(1, -1), inv)]
        exp_q.append(orc.rotate_bshd(qo[0].float().cpu(), orc.regroup_delta(pos.view(1, -1), params["G"]), inv))
        for got, exp in zip(qo, exp_q):
            d, cos = orc.compare(got.float().cpu(), exp)
            assert d <= 2 ** -5 and cos > 0.99999, (kind, d, cos)
    else:
        for got, pp in zip(qo, qpos):
            d, cos = orc.compare(got.float().cpu(), orc.rotate_bshd(q.float(), pp.view(1, -1), inv))
            assert d <= 2 ** -5 and cos > 0.99999, (kind, d, cos)
    eo, el = orc.posmap_attention_from_operands(kind, [t.cpu() for t in qo], [t.cpu() for t in ko], v,
                                                q_positions=pos, k_positions=pos, params=params)
    for impl in (0, 1, 2):
        out, lse = ops.posmap_prefill(qo, ko, dv, pmap=pm, q_pos0=P0, k_pos0=P0, impl=impl)
        _check(out, lse, eo, el, f"{kind} at positions ~131072, impl={impl}")


def test_prefill_status_word_is_clean():
    """No bounded wait inside the tcgen05 kernel gave up during the tests above."""
    from jetlm.kernels import _native
    torch.cuda.synchronize()
    assert _native.lib().jl_prefill_status() == 0

"""Parity at the sizes the benchmark configurations are quoted on, for the kernel configurations that
only small cases covered before: the CHUNK map (dual chunk attention) and self-extend's band at 131072
tokens, the block-cyclic query / key geometry every multi-GPU launch uses, and the decode kernel's
in-kernel regroup at a 131072-key context.  One launch at full size; sampled (row, head) pairs are
recomputed by the fp32 CPU oracle from the very bf16 operands the kernel consumed.

Reference semantics: jetlm/modeling/dca/modeling_qwen3_dca.py:363-423 (intra / successive / inter chunk
positions), jetlm/modeling/selfext/modeling_qwen3_selfext.py:353-387 (neighbour window + grouped positions),
jetlm/modeling/jetlong_fused/modeling_qwen3_jetlong_fused.py:375-379 (regrouped far operands).

Tolerances: output max-abs <= 2e-2 and cosine >= 0.9999, LSE max-abs <= 1e-3.
"""
import pytest
import torch

import jetlong_oracle as orc

pytestmark = pytest.mark.gpu

OUT_TOL, COS_TOL, LSE_TOL = 2e-2, 0.9999, 1e-3


def _ops():
    from jetlm.kernels import jetlong_ops
    return jetlong_ops


def _check(out, lse, exp_out, exp_lse, what):
    d, cos = orc.compare(out.float().cpu(), exp_out)
    assert d <= OUT_TOL and cos >= COS_TOL, f"{what}: out max-abs {d:.3e} cos {cos:.6f}"
    dl, _ = orc.compare(lse.float().cpu(), exp_lse)
    assert dl <= LSE_TOL, f"{what}: lse max-abs {dl:.3e}"


def _status_clean():
    from jetlm.kernels import _native
    torch.cuda.synchronize()
    return _native.lib().jl_prefill_status() == 0


def _spot_rows(kind, params, qo, ko, v, out, lse, rows, H, Hk, q_positions, k_positions):
    """Oracle rows: query row r of head h against every key row whose position is <= the query's."""
    rep = H // Hk
    for i, r in enumerate(rows):
        h = (7 * i + 3) % H
        kvh = h // rep
        pq = q_positions[r: r + 1]
        n_k = int((k_positions <= int(pq)).sum())          # key rows are in ascending position order
        qs = [t[:, r: r + 1, h: h + 1].float().cpu() for t in qo]
        ks = [t[:, :n_k, kvh: kvh + 1].float().cpu() for t in ko]
        vs = v[:, :n_k, kvh: kvh + 1].float().cpu()
        if n_k == 0:
            assert torch.all(out[:, r, h] == 0) and torch.isinf(lse[:, h, r]).all(), f"{kind} row {r}: expected an empty row"
            continue
        eo, el = orc.posmap_attention_from_operands(kind, qs, ks, vs, q_positions=pq, k_positions=k_positions[:n_k], params=params)
        _check(out[:, r: r + 1, h: h + 1], lse[:, h: h + 1, r: r + 1], eo, el, f"{kind} row {r} (position {int(pq)}) head {h}")


@pytest.mark.parametrize("kind", ["dca", "selfext"])
def test_position_maps_full_size_spot_rows(kind):
    """BASELINE config 3 geometry: 32 query / 8 kv heads, 131072 tokens; DCA with chunk 32768 (local window 4096)
    and self-extend with group 8 / neighbour window 2048, operands produced by the rotate kernel."""
    ops = _ops()
    torch.manual_seed(31 if kind == "dca" else 32)
    S, H, Hk, D = 131072, 32, 8, 128
    dinv = orc.default_inv_freq().cuda()
    q = torch.randn(1, S, H, D, device="cuda").bfloat16()
    k = torch.randn(1, S, Hk, D, device="cuda").bfloat16()
    v = torch.randn(1, S, Hk, D, device="cuda").bfloat16()
    if kind == "dca":
        s, w = 32768, 4096
        params, pm = dict(chunk_size=s, local_window=w), ops.PositionMap.dca(s)
        qo = [ops.rope_rotate(q, dinv, div_mul=0, mod=s, mod_mul=1),
              ops.rope_rotate(q, dinv, div_mul=0, mod=s, mod_mul=1, add=s, t_max=s + w),
              ops.rope_rotate(q, dinv, div_mul=0, add=s + w)]
        kr = ops.rope_rotate(k, dinv, div_mul=0, mod=s, mod_mul=1)
        ko = [kr, kr, kr]
        rows = [0, 1, 255, 256, s - 1, s, s + 1, s + 127, 2 * s - 1, 2 * s, 2 * s + 1, 3 * s - 129, 3 * s + 300, S - 257, S - 1]
    else:
        W, Gs = 2048, 8
        params, pm = dict(window_size=W, group_size=Gs), ops.PositionMap.selfext(W)
        qo = [ops.rope_base(q, dinv), ops.rope_rotate(q, dinv, div=Gs, add=W - W // Gs)]
        ko = [ops.rope_base(k, dinv), ops.rope_rotate(k, dinv, div=Gs)]
        rows = [0, 1, 127, 128, W - 2, W - 1, W, W + 1, W + 129, 2 * W + 255, S // 2 + 77, S - W - 1, S - 257, S - 1]
    del q, k
    out, lse = ops.posmap_prefill(qo, ko, v, pmap=pm, q_pos0=0)
    assert _status_clean()
    pos = torch.arange(S)
    _spot_rows(kind, params, qo, ko, v, out, lse, rows, H, Hk, pos, pos)


def test_block_cyclic_stripes_full_size_spot_rows():
    """The geometry of every multi-GPU prefill launch: 131072 positions in blocks of 1024 dealt to 8 ranks; the
    query stripe of rank 5 (16384 rows) against the key stripe of rank 3, both block-cyclic, jetlong map with
    w_0 = 32768.  The oracle sees the same stripe with its true positions."""
    ops = _ops()
    torch.manual_seed(33)
    S, H, Hk, D, w0, blk, world, rq, rk = 131072, 32, 8, 128, 32768, 1024, 8, 5, 3
    n_loc = S // world
    mk = lambda h: torch.randn(1, n_loc, h, D, device="cuda").bfloat16()
    qb, qg, kb, kg, v = mk(H), mk(H), mk(Hk), mk(Hk), mk(Hk)
    out, lse = ops.posmap_prefill([qb, qg], [kb, kg], v, pmap=ops.PositionMap.jetlong(w0),
                                  q_pos0=rq * blk, q_block=blk, q_block_stride=world * blk,
                                  k_pos0=rk * blk, k_block=blk, k_block_stride=world * blk)
    assert _status_clean()
    i = torch.arange(n_loc)
    q_positions = rq * blk + (i // blk) * world * blk + i % blk
    k_positions = rk * blk + (i // blk) * world * blk + i % blk
    # first block (no key of rank 3 yet at its first rows? positions 5120.. see keys 3072..4095), block edges,
    # rows whose near window ends inside / at the edge of a key block, the last rows
    rows = [0, 1, 255, 256, 1023, 1024, 1025, 4 * blk - 1, 4 * blk, 4 * blk + 129, 5 * blk + 511, n_loc // 2 + 77,
            n_loc - 1025, n_loc - 257, n_loc - 1]
    _spot_rows("jetlong", dict(w_0=w0, G=4), [qb, qg], [kb, kg], v, out, lse, rows, H, Hk, q_positions, k_positions)


@pytest.mark.parametrize("impl", [0, 2])
def test_block_cyclic_query_stripe_against_all_keys_spot_rows(impl):
    """The other multi-GPU form: one rank's block-cyclic query stripe (blocks of 256, rank 6 of 8) against ALL
    131072 keys in position order (gathered K / V)."""
    ops = _ops()
    torch.manual_seed(34)
    S, H, Hk, D, w0, blk, world, rq = 131072, 32, 8, 128, 32768, 256, 8, 6
    n_loc = S // world
    qb, qg = (torch.randn(1, n_loc, H, D, device="cuda").bfloat16() for _ in range(2))
    kb, kg, v = (torch.randn(1, S, Hk, D, device="cuda").bfloat16() for _ in range(3))
    out, lse = ops.posmap_prefill([qb, qg], [kb, kg], v, pmap=ops.PositionMap.jetlong(w0),
                                  q_pos0=rq * blk, q_block=blk, q_block_stride=world * blk, impl=impl)
    assert _status_clean()
    i = torch.arange(n_loc)
    q_positions = rq * blk + (i // blk) * world * blk + i % blk
    rows = [0, 1, 255, 256, 257, 16 * blk - 1, 16 * blk, 16 * blk + 3, 17 * blk + 130, n_loc // 2 + 77, n_loc - 257, n_loc - 1]
    _spot_rows("jetlong", dict(w_0=w0, G=4), [qb, qg], [kb, kg], v, out, lse, rows, H, Hk, q_positions, torch.arange(S))


@pytest.mark.parametrize("B", [1, 2])
def test_decode_in_kernel_regroup_full_context_spot_heads(B):
    """ctx = 131072, 32 / 8 heads, G = 4, w_0 = 32768: the far keys are regrouped inside the kernel from the
    base-rotated cache.  All query heads of two kv heads against the oracle, whose far keys are the exact fp32
    regrouping of the same bf16 cache; and the pre-grouped path fed that regrouping rounded to bf16."""
    ops = _ops()
    torch.manual_seed(35 + B)
    H, Hk, D, ctx, w0, G = 32, 8, 128, 131072, 32768, 4
    inv = orc.default_inv_freq()
    q = torch.randn(B, 1, H, D, device="cuda").bfloat16()
    qg = torch.randn(B, 1, H, D, device="cuda").bfloat16()
    k = torch.randn(B, ctx, Hk, D, device="cuda").bfloat16()
    v = torch.randn(B, ctx, Hk, D, device="cuda").bfloat16()
    b = ctx - 1 - w0
    segs = [ops.KvSegment(k[:, :b], v[:, :b], 1, rotate=True, pos0=0), ops.KvSegment(k[:, b:], v[:, b:], 0)]
    out, lse = ops.decode_segments([q, qg], segs, inv_freq=inv.cuda(), group_size=G)
    out8, lse8 = ops.decode_segments([q, qg], segs, inv_freq=inv.cuda(), group_size=G, num_splits=8)
    assert float((out.float() - out8.float()).abs().max()) <= 4e-3 and float((lse - lse8).abs().max()) <= 1e-4
    pos = torch.arange(b).view(1, b).expand(B, b)
    rep = H // Hk
    for kvh in (0, 5):
        hs = slice(kvh * rep, (kvh + 1) * rep)
        kfar = orc.rotate_bshd(k[:, :b, kvh: kvh + 1].float().cpu(), orc.regroup_delta(pos, G), inv)
        eo, el = orc.jetlong_decode(q[:, :, hs].cpu(), qg[:, :, hs].cpu(), k[:, b:, kvh: kvh + 1].cpu(), v[:, b:, kvh: kvh + 1].cpu(),
                                    kfar, v[:, :b, kvh: kvh + 1].cpu())
        _check(out[:, :, hs], lse[:, hs], eo, el, f"decode in-kernel regroup, ctx 131072, B={B}, kv head {kvh}")


def test_million_token_context_g32_decode_and_prefill_rows():
    """BASELINE config 5 geometry on one GPU at the operator level: positions up to 1,048,576 with G = 32
    (w = w_0 = 32768), where the fp32 RoPE angles are largest.  (1) decode of the token at position 2^20 - 1 over
    the whole base-rotated cache with the far keys regrouped in-kernel; (2) a 512-row prefill chunk that ends at
    2^20 against all keys (operands from jl_rotate), and the same chunk with the far class remapped inside the
    kernel.  All query heads of one kv head / sampled rows against the fp32 oracle."""
    ops = _ops()
    torch.manual_seed(77)
    H, Hk, D, ctx, w0, G = 8, 2, 128, 1 << 20, 32768, 32
    inv = orc.default_inv_freq()
    dinv = inv.cuda()
    k_raw = torch.randn(1, ctx, Hk, D, device="cuda").bfloat16()
    v = torch.randn(1, ctx, Hk, D, device="cuda").bfloat16()
    kb = ops.rope_base(k_raw, dinv)
    del k_raw
    rep = H // Hk
    # ---- (1) decode ----
    q_raw = torch.randn(1, 1, H, D, device="cuda").bfloat16()
    qb = ops.rope_base(q_raw, dinv, pos0=ctx - 1)
    qg = ops.rope_regroup(qb, dinv, group_size=G, pos0=ctx - 1)
    b = ctx - 1 - w0
    segs = [ops.KvSegment(kb[:, :b], v[:, :b], 1, rotate=True, pos0=0), ops.KvSegment(kb[:, b:], v[:, b:], 0)]
    out, lse = ops.decode_segments([qb, qg], segs, inv_freq=dinv, group_size=G)
    kvh = 1
    hs = slice(kvh * rep, (kvh + 1) * rep)
    pos = torch.arange(b).view(1, b)
    kfar = orc.rotate_bshd(kb[:, :b, kvh: kvh + 1].float().cpu(), orc.regroup_delta(pos, G), inv)
    eo, el = orc.jetlong_decode(qb[:, :, hs].cpu(), qg[:, :, hs].cpu(), kb[:, b:, kvh: kvh + 1].cpu(), v[:, b:, kvh: kvh + 1].cpu(),
                                kfar, v[:, :b, kvh: kvh + 1].cpu())
    _check(out[:, :, hs], lse[:, hs], eo, el, "decode at 2^20 keys, G = 32, in-kernel regroup")
    # ---- (2) the last 512-row chunk of a chunked prefill ----
    Sq = 512
    q_raw = torch.randn(1, Sq, H, D, device="cuda").bfloat16()
    qb = ops.rope_base(q_raw, dinv, pos0=ctx - Sq)
    qg = ops.rope_regroup(qb, dinv, group_size=G, pos0=ctx - Sq)
    kg = ops.rope_regroup(kb, dinv, group_size=G)
    pm = ops.PositionMap.jetlong(w0)
    out, lse = ops.posmap_prefill([qb, qg], [kb, kg], v, pmap=pm, q_pos0=ctx - Sq)
    out_r, lse_r = ops.posmap_prefill([qb], [kb], v, pmap=pm, q_pos0=ctx - Sq, remap_far=(dinv, G))
    assert _status_clean()
    d, cos = orc.compare(out_r.float().cpu(), out.float().cpu())
    dl, _ = orc.compare(lse_r.cpu(), lse.cpu())
    assert d <= OUT_TOL and cos >= COS_TOL and dl <= LSE_TOL, ("in-kernel remap vs pre-rotated operands", d, cos, dl)
    for i, r in enumerate((0, 255, 256, Sq - 1)):
        h = (3 * i + 1) % H
        kvh = h // rep
        n_k = ctx - Sq + r + 1
        # oracle operands: the fp32 regrouping of the bf16 base-rotated tensors, rounded to bf16 as both kernel paths
        # round the far-class operands before the tensor cores read them
        kpos = torch.arange(n_k).view(1, n_k)
        kg_ref = orc.rotate_bshd(kb[:, :n_k, kvh: kvh + 1].float().cpu(), orc.regroup_delta(kpos, G), inv).bfloat16().float()
        qg_ref = orc.rotate_bshd(qb[:, r: r + 1, h: h + 1].float().cpu(), orc.regroup_delta(torch.tensor([[ctx - Sq + r]]), G), inv).bfloat16().float()
        eo, el = orc.jetlong_prefill(qb[:, r: r + 1, h: h + 1].float().cpu(), qg_ref, kb[:, :n_k, kvh: kvh + 1].float().cpu(), kg_ref,
                                     v[:, :n_k, kvh: kvh + 1].float().cpu(), seqstart=ctx - Sq + r, w0=w0)
        _check(out[:, r: r + 1, h: h + 1], lse[:, h: h + 1, r: r + 1], eo, el, f"prefill row at position {ctx - Sq + r}, pre-rotated operands")
        _check(out_r[:, r: r + 1, h: h + 1], lse_r[:, h: h + 1, r: r + 1], eo, el, f"prefill row at position {ctx - Sq + r}, in-kernel remap")


@pytest.mark.parametrize("S,Skv,w0,G", [(300, 300, 100, 3), (700, 1500, 200, 4), (1, 900, 64, 7), (513, 513, 0, 2)])
def test_in_kernel_far_remap_matches_the_oracle(S, Skv, w0, G):
    """jl_prefill with remap_far_in_kernel: only base-rotated q / k go in; the far class is rotated per tile in
    shared memory and rounded to bf16 there, as the pre-rotated operands are.  Against the oracle's two-branch
    composition on the fp32 regrouping of the same tensors rounded to bf16, at positions near 131072 so that the
    angles are large."""
    ops = _ops()
    torch.manual_seed(S + G)
    B, H, Hk, D = 1, 4, 2, 128
    P0 = 131072 - Skv
    inv = orc.default_inv_freq()
    q_raw, k_raw = torch.randn(B, S, H, D).bfloat16(), torch.randn(B, Skv, Hk, D).bfloat16()
    v = torch.randn(B, Skv, Hk, D).bfloat16()
    qb = ops.rope_base(q_raw.cuda(), inv.cuda(), pos0=P0 + Skv - S)
    kb = ops.rope_base(k_raw.cuda(), inv.cuda(), pos0=P0)
    out, lse = ops.posmap_prefill([qb], [kb], v.cuda(), pmap=ops.PositionMap.jetlong(w0), q_pos0=P0 + Skv - S, k_pos0=P0,
                                  remap_far=(inv.cuda(), G))
    assert _status_clean()
    qpos = (torch.arange(S) + P0 + Skv - S).view(1, S)
    kpos = (torch.arange(Skv) + P0).view(1, Skv)
    qg = orc.rotate_bshd(qb.float().cpu(), orc.regroup_delta(qpos, G), inv).bfloat16().float()
    kg = orc.rotate_bshd(kb.float().cpu(), orc.regroup_delta(kpos, G), inv).bfloat16().float()
    eo, el = orc.jetlong_prefill(qb.float().cpu(), qg, kb.float().cpu(), kg, v.float(), seqstart=Skv - S, w0=w0)
    _check(out, lse, eo, el, f"in-kernel remap S={S} Skv={Skv} w0={w0} G={G}")

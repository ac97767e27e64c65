"""Device-resident decode-step state: jl_step_advance, jl_decode_append, device-side segment
geometry in jl_decode, and the CUDA-graph decode driver built on them."""
import pytest
import torch

import jetlong_oracle as orc
from test_model_gpu import _tiny_model

pytestmark = pytest.mark.gpu


def _ops():
    from jetlm.kernels import jetlong_ops
    return jetlong_ops


@pytest.mark.parametrize("world,block,w_0", [(1, 1, 37), (3, 8, 37), (4, 16, 0), (2, 8, 500)])
def test_step_advance_follows_the_block_cyclic_geometry(world, block, w_0):
    from jetlm.kernels.sequence_parallel import SequenceShard
    ops = _ops()
    for rank in range(world):
        sh = SequenceShard(rank, world, block=block) if world > 1 else None
        st = ops.StepState(2, "cuda", w_0, sh)
        st.set_next_position(90)
        rows = []
        for pos in range(90, 140):
            st.advance()
            got, steps = st.state.tolist()[:5], int(st.steps)
            assert steps == pos - 89                      # advances made on this state, never rewound
            n_owned = (lambda n: sh.n_owned(n)) if sh is not None else (lambda n: n)
            own = 1 if sh is None else int((pos // block) % world == rank)
            n_far = n_owned(max(pos - w_0, 0))
            want = [pos, n_owned(pos), own, n_far, n_owned(pos) + own - n_far]
            assert got == want, (rank, pos, got, want)
            assert st.lens.tolist() == [[want[3]] * 2, [want[4]] * 2]
            rows.append(got)


def test_decode_append_equals_norm_rope_and_writes_the_owned_row():
    ops = _ops()
    torch.manual_seed(4)
    B, H, Hk, D, cap, G = 2, 8, 2, 128, 64, 3
    inv = orc.default_inv_freq().cuda()
    mk = lambda *s: torch.randn(*s, device="cuda").bfloat16()
    qkv = mk(B, 1, (H + 2 * Hk) * D)                      # one fused projection output: strided q / k / v views
    q = qkv[..., : H * D].view(B, 1, H, D)
    k = qkv[..., H * D: (H + Hk) * D].view(B, 1, Hk, D)
    v = qkv[..., (H + Hk) * D:].view(B, 1, Hk, D)
    qw, kw = mk(D), mk(D)
    kc, vc = torch.zeros(B, cap, Hk, D, device="cuda").bfloat16(), torch.zeros(B, cap, Hk, D, device="cuda").bfloat16()
    st = ops.StepState(B, "cuda", 10)
    st.set_next_position(41)
    st.advance()
    qb, qg = ops.decode_append(q, k, v, qw, kw, inv, kc, vc, st, q_eps=1e-6, k_eps=1e-5, group_size=G)
    qb_ref, qg_ref = ops.norm_rope(q, qw, inv, eps=1e-6, pos0=41, group_size=G)
    kb_ref = ops.norm_rope(k, kw, inv, eps=1e-5, pos0=41)
    assert torch.equal(qb, qb_ref) and torch.equal(qg, qg_ref)
    assert torch.equal(kc[:, 41:42], kb_ref) and torch.equal(vc[:, 41:42], v)
    assert not kc[:, :41].any() and not kc[:, 42:].any() and not vc[:, 42:].any()
    # a rank that does not own the position writes nothing; group_size 1 returns one query operand
    from jetlm.kernels.sequence_parallel import SequenceShard
    st2 = ops.StepState(B, "cuda", 10, SequenceShard(1, 2, block=8))
    st2.set_next_position(41)                             # block 5 -> rank 1 owns it; position 48 -> rank 0
    st2.advance()
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    a, b = ops.decode_append(q, k, v, qw, kw, inv, kc2, vc2, st2, q_eps=1e-6, k_eps=1e-5, group_size=1)
    assert a is b and torch.equal(a, qb_ref)
    row = st2.state[1].item()
    assert row == 17 and torch.equal(kc2[:, row: row + 1], kb_ref) and kc2.float().abs().sum() == kb_ref.float().abs().sum()
    st2.set_next_position(48)
    st2.advance()
    kc2.zero_(); vc2.zero_()
    ops.decode_append(q, k, v, qw, kw, inv, kc2, vc2, st2, q_eps=1e-6, k_eps=1e-5, group_size=1)
    assert st2.state[2].item() == 0 and not kc2.any() and not vc2.any()


@pytest.mark.parametrize("n_far,n_near", [(0, 70), (130, 1), (333, 267), (1000, 24)])
def test_device_side_segment_geometry_equals_sliced_segments(n_far, n_near):
    """Whole cache + (len_dev, row0_dev) from the step state == explicit slices, with the same split count."""
    ops = _ops()
    torch.manual_seed(n_far + n_near)
    B, H, Hk, D, cap, G = 2, 8, 2, 128, 1100, 4
    inv = orc.default_inv_freq().cuda()
    mk = lambda *s: torch.randn(*s, device="cuda").bfloat16()
    qb, qg, kc, vc = mk(B, 1, H, D), mk(B, 1, H, D), mk(B, cap, Hk, D), mk(B, cap, Hk, D)
    st = ops.StepState(B, "cuda", 0)
    st.state[:5].copy_(torch.tensor([0, 0, 1, n_far, n_near]))
    st.lens[0] = n_far
    st.lens[1] = n_near
    kw = dict(inv_freq=inv, group_size=G, num_splits=2)
    segs = [ops.KvSegment(kc, vc, 1, rotate=True, len_dev=st.far_lens),
            ops.KvSegment(kc, vc, 0, len_dev=st.near_lens, row0_dev=st.n_far)]
    out, lse = ops.decode_segments([qb, qg], segs, **kw)
    ref = [ops.KvSegment(kc[:, :n_far], vc[:, :n_far], 1, rotate=True)] if n_far else []
    ref.append(ops.KvSegment(kc[:, n_far: n_far + n_near], vc[:, n_far: n_far + n_near], 0))
    out_ref, lse_ref = ops.decode_segments([qb, qg], ref, **kw)
    assert torch.equal(out, out_ref) and torch.equal(lse, lse_ref)
    # a shift past the described rows reads nothing instead of running off the buffer
    st.state[3] = cap + 50
    out2, lse2 = ops.decode_segments([qb, qg], segs[1:], **kw)
    assert torch.isinf(lse2).all() and not out2.any()


@torch.inference_mode()
def test_graphed_decode_equals_eager_decode(golden):
    """Greedy tokens from the replayed CUDA graph == tokens from the Python-launched steps, across a
    change of the group size (prompt 186, w = 64: G goes 3 -> 4 at L = 193) and with an in-window start."""
    g = golden("model_tiny.npz")
    model = _tiny_model(g)
    ids = g["input_ids"].cuda()
    for prompt, chunk, new in ((186, 64, 12), (150, 150, 6)):
        eager = model.generate_long(ids[:, :prompt], max_new_tokens=new, chunk_tokens=chunk)
        graphed = model.generate_long(ids[:, :prompt], max_new_tokens=new, chunk_tokens=chunk, cuda_graph=True)
        assert graphed.tolist() == eager.tolist(), (prompt, graphed.tolist(), eager.tolist())
    model.model.kernels_within_window = True            # G = 1 graph first, then G = 2 after crossing w
    eager = model.generate_long(ids[:, :60], max_new_tokens=10, chunk_tokens=60)
    graphed = model.generate_long(ids[:, :60], max_new_tokens=10, chunk_tokens=60, cuda_graph=True)
    assert graphed.tolist() == eager.tolist()


@torch.inference_mode()
def test_graphed_step_hidden_state_equals_eager_forward(golden):
    from jetlm.kernels.decode_graph import GraphedDecodeStep
    from jetlm.kernels.kv_cache import BifocalKVCache
    g = golden("model_tiny.npz")
    model = _tiny_model(g)
    ids = g["input_ids"].cuda()
    caches = [BifocalKVCache(model.config, 256, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    for c in caches:
        model(input_ids=ids[:, :150], past_key_values=c, use_cache=True)
    want = model(input_ids=ids[:, 150:151], past_key_values=caches[0], use_cache=True).logits.float()
    step = GraphedDecodeStep(model, caches[1])
    step.step.set_next_position(150)
    step.step.advance()
    hidden = model.model.decode_step(ids[:, 150:151], caches[1], step.step, group=3)
    got = model.lm_head(hidden).float()
    d, cos = orc.compare(got.cpu(), want.cpu())
    assert cos >= 0.99999 and d <= 2e-2, (d, cos)
    assert torch.equal(caches[1].layers[0].keys[:, 150], caches[0].layers[0].keys[:, 150])


@torch.inference_mode()
def test_graphed_decode_with_regrouped_far_key_cache(golden):
    """The far rows are kept regrouped in a second key buffer (bulk pass at capture, one row per step): same
    greedy tokens as the eager steps, and the buffer equals a fresh regroup of the base keys, bit for bit,
    also after G changed (prompt 186 -> G 3, 4)."""
    from jetlm.kernels.kv_cache import BifocalKVCache
    g = golden("model_tiny.npz")
    model = _tiny_model(g)
    ids = g["input_ids"].cuda()
    ops = _ops()
    w, w0 = g.meta["w"], g.meta["w0"]
    for prompt, new in ((186, 12), (150, 6)):
        eager = model.generate_long(ids[:, :prompt], max_new_tokens=new, chunk_tokens=64)
        cache = BifocalKVCache(model.config, 256, device="cuda", dtype=torch.bfloat16, regrouped_far_keys=True)
        graphed = model.generate_long(ids[:, :prompt], max_new_tokens=new, chunk_tokens=64, past_key_values=cache,
                                      cuda_graph=True)
        assert graphed.tolist() == eager.tolist()
        last = cache.get_seq_length() - 1                     # position of the last decoded-from token
        G, n_far = -(-(last + 1) // w), last - w0
        inv = model.model.rotary_emb.inv_freq
        for layer in cache.layers:
            want = ops.rope_regroup(layer.keys[:, :n_far], inv, group_size=G)
            assert torch.equal(layer.group_keys[:, :n_far], want)

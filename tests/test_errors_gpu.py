"""Error conventions at the Python boundary that need CUDA tensors to be reached — they mirror the
three rejection tests of the reference's kernel test file (tests/test_fa4_cute_kernels.py:328-385, :430-451)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(head_dim=64):
    B, ctx, H, Hk = 1, 16, 4, 2
    q = torch.randn(B, 1, H, head_dim, device="cuda", dtype=torch.bfloat16)
    kn = torch.randn(B, 4, Hk, head_dim, device="cuda", dtype=torch.bfloat16)
    kd = torch.randn(B, ctx - 4, Hk, head_dim, device="cuda", dtype=torch.bfloat16)
    meta = dict(seqused_near=torch.full((B,), 4, device="cuda", dtype=torch.int32),
                seqused_distant=torch.full((B,), ctx - 4, device="cuda", dtype=torch.int32),
                inv_freq=torch.rand(head_dim // 2, device="cuda"), group_size=4)
    return q, kn, kd, meta


def test_decode_rejects_noncontiguous_output():
    from jetlm.kernels.jetlong_ops import fa4_cute_decode_sm90_jetlong_fused as decode
    q, kn, kd, meta = _inputs()
    out = torch.empty(1, 1, 4, 128, device="cuda", dtype=torch.bfloat16)[..., ::2]
    assert not out.is_contiguous()
    with pytest.raises(ValueError, match="out must be contiguous"):
        decode(q, torch.randn_like(q), kn, torch.randn_like(kn), kd, torch.randn_like(kd), out=out, **meta)


def test_decode_rejects_bad_metadata():
    from jetlm.kernels.jetlong_ops import fa4_cute_decode_sm90_jetlong_fused as decode
    q, kn, kd, meta = _inputs()
    with pytest.raises(ValueError, match="active_splits must have dtype torch.int32"):
        decode(q, torch.randn_like(q), kn, torch.randn_like(kn), kd, torch.randn_like(kd),
               active_splits=torch.ones(1, device="cuda", dtype=torch.int64), **meta)


def test_prefill_rejects_unsupported_metadata():
    from jetlm.kernels.jetlong_ops import fa4_cute_prefill_sm90_jetlong_fused as prefill
    q = torch.randn(1, 16, 4, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 16, 2, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="unsupported metadata arguments.*seqused_q"):
        prefill(q, q, k, k, k, seqstart_q=torch.zeros(1, device="cuda", dtype=torch.int32), window_size_left=4,
                seqused_q=torch.full((1,), 16, device="cuda", dtype=torch.int32))


def test_unsupported_head_dim_is_a_clear_error():
    from jetlm.kernels import jetlong_ops as ops
    from jetlm.kernels._native import NativeError
    q = torch.randn(1, 16, 4, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 16, 2, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(NativeError, match="head_dim must be 128"):
        ops.posmap_prefill([q, q], [k, k], k, pmap=ops.PositionMap.jetlong(4), q_pos0=0)


def test_prefill_refuses_shapes_the_tcgen05_kernel_does_not_cover():
    """impl 0 never changes kernel silently: a key block that is not a multiple of the 128-key tile is refused
    (the reference's prefill raises on what it does not support, cute_prefill_sm90.py:114-178); the mma.sync
    cross-check kernel still takes the same call when it is asked for by name (impl = 1)."""
    from jetlm.kernels import jetlong_ops as ops
    from jetlm.kernels._native import JL_ERR_UNSUPPORTED, NativeError
    q = torch.randn(1, 256, 4, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 256, 2, 128, device="cuda", dtype=torch.bfloat16)
    kw = dict(pmap=ops.PositionMap.jetlong(40), q_pos0=0, k_pos0=64, k_block=64, k_block_stride=128)
    with pytest.raises(NativeError, match="k_block must be a multiple of 128") as err:
        ops.posmap_prefill([q, q], [k, k], k, **kw)
    assert err.value.status == JL_ERR_UNSUPPORTED
    out, _ = ops.posmap_prefill([q, q], [k, k], k, impl=1, **kw)
    assert torch.isfinite(out.float()).all()
    with pytest.raises(NativeError, match="q_block must be a multiple of 256"):
        ops.posmap_prefill([q, q], [k, k], k, pmap=ops.PositionMap.jetlong(40), q_pos0=0, q_block=128, q_block_stride=256)


def test_prefill_cta_pair_kernel_refuses_what_it_does_not_cover():
    """impl 2 (the CTA-pair kernel) has no in-kernel remap of the far class; an unknown impl is a bad argument."""
    from jetlm.kernels import jetlong_ops as ops
    from jetlm.kernels._native import JL_ERR_BAD_ARG, JL_ERR_UNSUPPORTED, NativeError
    q = torch.randn(1, 256, 4, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 256, 2, 128, device="cuda", dtype=torch.bfloat16)
    inv = torch.ones(64, device="cuda")
    with pytest.raises(NativeError, match="in-kernel remap") as err:
        ops.posmap_prefill([q], [k], k, pmap=ops.PositionMap.jetlong(40), q_pos0=0, remap_far=(inv, 4), impl=2)
    assert err.value.status == JL_ERR_UNSUPPORTED
    with pytest.raises(NativeError, match="impl must be 0, 1 or 2") as err:
        ops.posmap_prefill([q, q], [k, k], k, pmap=ops.PositionMap.jetlong(40), q_pos0=0, impl=3)
    assert err.value.status == JL_ERR_BAD_ARG
    with pytest.raises(NativeError, match="stripe batching needs impl 0 or 2") as err:
        ops.posmap_prefill([q, q], [k, k], k, pmap=ops.PositionMap.jetlong(40), q_pos0=0, impl=1, stripes=(0, 1, 256))
    assert err.value.status == JL_ERR_UNSUPPORTED
    with pytest.raises(ValueError, match="stripes"):
        ops.posmap_prefill([q, q], [k, k], k, pmap=ops.PositionMap.jetlong(40), q_pos0=0, stripes=(1, 1, 256))


@pytest.mark.parametrize("impl", [0, 2])
def test_prefill_without_keys_returns_empty_rows(impl):
    from jetlm.kernels import jetlong_ops as ops
    q = torch.randn(1, 300, 4, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.empty(1, 0, 2, 128, device="cuda", dtype=torch.bfloat16)
    out, lse = ops.posmap_prefill([q, q], [k, k], k, pmap=ops.PositionMap.jetlong(40), q_pos0=0, impl=impl)
    assert torch.all(out == 0) and torch.all(torch.isinf(lse) & (lse < 0))


def test_peer_merge_wait_runs_out_and_reports_it():
    """The bounded wait of jl_peer_merge, made to run out on ONE GPU: the kernel is told it is rank 0 of 2, both
    exchange buffers are local memory, and nobody plays rank 1, so its flag never arrives.  The kernel must
    return after the limit (20 ms here), raise the status word, and leave the context usable; ops.check_status()
    turns the word into an exception.  With world = 1 the same call completes and the status stays clear."""
    import time
    from types import SimpleNamespace
    from jetlm.kernels import _native as n, jetlong_ops as ops
    B, H, D = 2, 8, 128
    torch.manual_seed(0)
    po = torch.randn(B, 1, H, D, device="cuda").bfloat16()
    pl = torch.randn(B, H, 1, device="cuda")

    class FakeExchange:
        def __init__(self, world):
            self.nbytes = int(n.lib().jl_peer_merge_buffer_bytes(world, B, H, D))
            self.bufs = [torch.zeros(self.nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
            self.ptrs = [t.data_ptr() for t in self.bufs]
            self.shard = SimpleNamespace(rank=0, world=world)
            self.batch, self.heads, self.head_dim = B, H, D
            self.status = torch.zeros(1, dtype=torch.int32, device="cuda")

    solo = FakeExchange(1)
    ops.register_peer_exchange(solo)
    out, lse = ops.peer_merge(po, pl, solo, epoch_base=None, epoch_stride=1, epoch_offset=1, return_lse=True)
    torch.cuda.synchronize()
    assert int(solo.status) == 0 and torch.equal(out, po) and torch.allclose(lse, pl)
    ops.check_status()

    alone = FakeExchange(2)
    ops.register_peer_exchange(alone)
    t0 = time.perf_counter()
    ops.peer_merge(po, pl, alone, epoch_base=None, epoch_stride=1, epoch_offset=1, wait_limit_ms=20)
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert int(alone.status) == 1, "the wait should have given up"
    assert 0.015 <= waited < 0.5, waited
    with pytest.raises(RuntimeError, match="bounded wait"):
        ops.check_status()
    alone.status.zero_()
    # the context is intact: the next kernel runs and is correct
    out, _ = ops.peer_merge(po, pl, solo, epoch_base=None, epoch_stride=1, epoch_offset=2, return_lse=True)
    torch.cuda.synchronize()
    assert torch.equal(out, po)
    ops.check_status()

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

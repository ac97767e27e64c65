"""Backend entry points the `jetlong_fused` modeling file imports — same names, arguments, return
layouts and error behaviour as the reference's jetlm/kernels/cute_jetlong_backend.py (:42-75
fused_jetlong_prefill, :109-166 fused_jetlong_decode), running on the B200 kernels.

Differences that are invisible to the caller: the (B,H,S,D) inputs are read in place through their
strides (no transpose/contiguous copies, no 2S packing, no padding of the distant region to a
compile bucket), the split count is sized to fill the GPU, and one kernel pass covers both regions.
"""
from __future__ import annotations

import torch

from . import jetlong_ops as ops


def fused_jetlong_prefill(query_base, query_group, key_base, key_group, value, *, seqstart_q: int,
                          window_size_left: int, softmax_scale: float, has_any_pad: bool, training: bool):
    """(B,H,S,D) / (B,Hk,Skv,D) views in, attention output (B,S,H,D) out."""
    if training:
        raise RuntimeError("JetLong backend 'fused' is inference-only")
    if has_any_pad:
        raise RuntimeError("JetLong backend 'fused' does not support left-padded prefill batches")
    t = lambda x: x.transpose(1, 2)
    out = ops.posmap_prefill([t(query_base), t(query_group)], [t(key_base), t(key_group)], t(value),
                             pmap=ops.PositionMap.jetlong(int(window_size_left)), q_pos0=int(seqstart_q),
                             softmax_scale=softmax_scale, return_lse=False)
    return out


def fused_jetlong_decode(query_base, query_group, key_near, value_near, key_distant_group, value_distant, *,
                         inv_freq, group_size: int, has_any_pad: bool, training: bool):
    """(B,1,H,D) queries and (B,N,Hk,D) key/value views (slices of the cache, read in place) in,
    (B,1,H,D) out.  key_distant_group is already regrouped by the caller, as in the reference."""
    if training:
        raise RuntimeError("JetLong backend 'fused' is inference-only")
    if has_any_pad:
        raise RuntimeError("JetLong backend 'fused' does not support left-padded decode batches")
    if key_distant_group.shape[1] == 0:
        raise RuntimeError("JetLong backend 'fused' requires a non-empty distant decode region")
    segs = [ops.KvSegment(key_distant_group, value_distant, q_class=1),
            ops.KvSegment(key_near, value_near, q_class=0)]
    return ops.decode_segments([query_base, query_group], segs, return_lse=False)

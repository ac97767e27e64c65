"""2-way (O, LSE) merge with the reference's `merge2_bshd` contract (jetlm/kernels/merge_fused.py:76-93
and csrc/merge_fused.cu:135-168 in the Jet-Long repository), served by the N-way B200 merge kernel.

`merge2_bshd` keeps the reference's arithmetic, including the rounding to the storage dtype after
every step; `merge_partials` (jetlong_ops) is the fp32, N-way, LSE-emitting form the fused paths use.
"""
from __future__ import annotations

import torch

from .jetlong_ops import merge_partials


def _ensure_bshd_contiguous(out: torch.Tensor, lse: torch.Tensor):
    if out.dim() != 4 or lse.dim() != 3:
        raise ValueError("expected out=(B,S,H,D) and lse=(B,H,S)")
    if not out.is_cuda or not lse.is_cuda:
        raise ValueError("fused merge requires CUDA tensors")
    return out.contiguous(), lse.float().contiguous()


def merge2_bshd(out_a, lse_a, out_b, lse_b, out=None, *, round_like_reference: bool = True):
    """Merge two attention branches: out_* (B,S,H,D), lse_* (B,H,S) -> (B,S,H,D)."""
    out_a, lse_a = _ensure_bshd_contiguous(out_a, lse_a)
    out_b, lse_b = _ensure_bshd_contiguous(out_b, lse_b)
    return merge_partials([out_a, out_b], [lse_a, lse_b], out=out, return_lse=False,
                          round_like_reference=round_like_reference)

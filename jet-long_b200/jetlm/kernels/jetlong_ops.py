"""Kernel-level Python operators over the C ABI (tensor contracts of the reference's level-2 API).

Reference counterparts (paths inside the Jet-Long repository):
  jetlong_prefill   jetlm/kernels/cute_prefill_sm90.py:114-230   fa4_cute_prefill_sm90_jetlong_fused
  jetlong_decode    jetlm/kernels/cute_decode_sm90.py:2748-2799  fa4_cute_decode_sm90_jetlong_fused
  merge_partials    jetlm/kernels/cute_decode_sm90.py:199-240 and jetlm/kernels/merge_fused.py:76-93
  rope_rotate       jetlm/modeling/jetlong_fused/modeling_qwen3_jetlong_fused.py:171-176, :209-226

All tensors are (B, S, H, D) *views*: any strides are accepted as long as head_dim is contiguous and
every stride is a multiple of 8 elements, so (B, H, S, D) cache tensors are passed as
`.transpose(1, 2)` without a copy.  Kernels run on the current torch CUDA stream.  Nothing here
computes attention in PyTorch: a missing extension or a failing call raises.
"""
from __future__ import annotations

import ctypes as C
import math
import weakref
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _native as N

_SUPPORTED_DTYPES = (torch.bfloat16,)


# ----------------------------------------------------------------------------------------------
# plumbing
# ----------------------------------------------------------------------------------------------

def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_arch(op: str, device: torch.device) -> None:
    major, _ = torch.cuda.get_device_capability(device)
    if major != 10:
        raise RuntimeError(f"{op} requires sm_100 (B200)")


def _require_contiguous(op: str, name: str, t: torch.Tensor) -> None:
    if not t.is_contiguous():
        raise ValueError(f"{op}: {name} must be contiguous; call {name}.contiguous() before invoking the kernel")


def _check_view(op: str, name: str, t: torch.Tensor) -> None:
    if t.dim() != 4:
        raise ValueError(f"{op} expects rank-4 BSHD tensors")
    if t.shape[-1] > 1 and t.stride(-1) != 1:
        raise ValueError(f"{op}: {name} must have a contiguous head_dim; call {name}.contiguous()")
    # size-1 dims may carry arbitrary strides; they are never multiplied by a non-zero index
    if any(t.shape[i] > 1 and t.stride(i) % 8 for i in range(3)):
        raise ValueError(f"{op}: {name} strides must be multiples of 8 elements")
    if t.data_ptr() % 16:
        raise ValueError(f"{op}: {name} must be 16-byte aligned")


def _st(t: torch.Tensor, i: int) -> int:
    return t.stride(i) if t.shape[i] > 1 else 0


def _call(name: str, fn) -> None:
    """Run one C-ABI call and raise on a non-zero status."""
    N.check(name, fn())


# ----------------------------------------------------------------------------------------------
# status words of the bounded waits
# ----------------------------------------------------------------------------------------------

_PEER_EXCHANGES: "weakref.WeakSet" = weakref.WeakSet()      # every live sequence_parallel.PeerExchange


def register_peer_exchange(exchange) -> None:
    _PEER_EXCHANGES.add(exchange)


def kernel_status() -> dict:
    """What the kernels' bounded waits reported since the last call (synchronises the current device; reading a
    raised prefill status clears it): {"prefill_wait_timeouts": 0 / 1, "peer_exchange_failed": bool}."""
    failed = any(bool(ex.status.item()) for ex in list(_PEER_EXCHANGES))
    return dict(prefill_wait_timeouts=int(N.lib().jl_prefill_status()), peer_exchange_failed=failed)


def clear_peer_status() -> None:
    """Put the status words of every live peer exchange back to zero (after a reported timeout has been handled)."""
    for ex in list(_PEER_EXCHANGES):
        ex.status.zero_()


def check_status() -> None:
    """Raise if a bounded wait inside jl_prefill or jl_peer_merge gave up: the results produced since the
    last check are then invalid.  Call at a point that synchronises anyway (end of a step, before logits leave)."""
    st = kernel_status()
    if st["prefill_wait_timeouts"] or st["peer_exchange_failed"]:
        raise RuntimeError(f"a bounded wait inside the attention kernels gave up ({st}); results since the last "
                           f"check are invalid")


_WORKSPACES: dict[tuple, torch.Tensor] = {}
_SPARE_WORKSPACES: dict[int, list] = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Split-KV scratch, cached per (device, stream) so concurrent streams never share it.  Zeroed once:
    the arrival counters at its head must start at zero, and every launch leaves them zero.

    A CUDA-graph capture runs on a stream of its own and so asks for a workspace of its own; zeroing one there
    would put a memset node into the graph.  Every eager call therefore leaves one zeroed spare per device
    behind, and a capturing call takes it."""
    key = (device.index, _stream())
    ws = _WORKSPACES.get(key)
    capturing = torch.cuda.is_current_stream_capturing()
    if ws is None or ws.numel() < nbytes:
        spares = _SPARE_WORKSPACES.setdefault(device.index, [])
        fit = next((t for t in spares if t.numel() >= nbytes), None) if capturing else None
        if fit is not None:
            spares.remove(fit)
            ws = fit
        else:
            ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    if not capturing:
        spares = _SPARE_WORKSPACES.setdefault(device.index, [])
        if not any(t.numel() >= nbytes for t in spares):
            spares[:] = [torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)]
    return ws


@dataclass(frozen=True)
class PositionMap:
    """Which (q operand, k operand) pair scores a (query, key) position pair (see jl_posmap)."""
    kind: int
    n_classes: int
    near_span: int = 0
    chunk: int = 1

    @staticmethod
    def jetlong(w_0: int) -> "PositionMap":
        return PositionMap(N.JL_MAP_BAND, 2, near_span=int(w_0))

    @staticmethod
    def selfext(window_size: int) -> "PositionMap":
        return PositionMap(N.JL_MAP_BAND, 2, near_span=int(window_size) - 1)

    @staticmethod
    def dca(chunk_size: int) -> "PositionMap":
        return PositionMap(N.JL_MAP_CHUNK, 3, chunk=int(chunk_size))

    def c_struct(self) -> N.PosMap:
        return N.PosMap(self.kind, self.n_classes, self.near_span, self.chunk)


# ----------------------------------------------------------------------------------------------
# rotate
# ----------------------------------------------------------------------------------------------

_BIG = (1 << 62)


def rope_rotate(x: torch.Tensor, inv_freq: torch.Tensor, *, pos0: int = 0, div: int = 1, div_mul: int = 1,
                mod: int = _BIG, mod_mul: int = 0, add: int = 0, t_max: int = _BIG,
                pos_block: int = 0, pos_block_stride: int = 0,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = rotate-half RoPE of x (B,S,H,D view) at t(p) = min((p//div)*div_mul + (p%mod)*mod_mul + add, t_max),
    p = pos0 + row (or the block-cyclic pos0 + (row // pos_block) * pos_block_stride + row % pos_block).
    fp32 math on the angles fp32(t)*inv_freq, one rounding to bf16."""
    op = "rope_rotate"
    _check_view(op, "x", x)
    if x.dtype not in _SUPPORTED_DTYPES:
        raise ValueError(f"{op}: x must be torch.bfloat16, got {x.dtype}")
    _require_arch(op, x.device)
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    _check_view(op, "out", out)
    if out.shape != x.shape:
        raise ValueError(f"{op}: out must have shape {tuple(x.shape)}")
    inv_freq = inv_freq.to(device=x.device, dtype=torch.float32).contiguous()
    if inv_freq.numel() < x.shape[-1] // 2:
        raise ValueError(f"{op}: inv_freq must have shape ({x.shape[-1] // 2},) or larger")
    B, S, H, D = x.shape
    a = N.RotateArgs(x.data_ptr(), out.data_ptr(), _st(x, 0), _st(x, 1), _st(x, 2), _st(out, 0), _st(out, 1), _st(out, 2),
                     B, S, H, D, int(pos0), int(div), int(div_mul), int(mod), int(mod_mul), int(add), int(t_max),
                     inv_freq.data_ptr(), int(pos_block), int(pos_block_stride))
    with torch.cuda.device(x.device):
        _call("jl_rotate", lambda: N.lib().jl_rotate(C.byref(a), _stream()))
    return out


def rope_base(x, inv_freq, *, pos0=0, pos_block=0, pos_block_stride=0, out=None):
    """Base RoPE: t = p."""
    return rope_rotate(x, inv_freq, pos0=pos0, pos_block=pos_block, pos_block_stride=pos_block_stride, out=out)


def rope_regroup(x_base, inv_freq, *, group_size: int, pos0=0, pos_block=0, pos_block_stride=0, out=None):
    """jetlong far-class operand from a base-rotated tensor: extra rotation by floor(p/G) - p."""
    return rope_rotate(x_base, inv_freq, pos0=pos0, div=int(group_size), div_mul=1, mod=_BIG, mod_mul=-1,
                       pos_block=pos_block, pos_block_stride=pos_block_stride, out=out)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, *, eps: float, residual: Optional[torch.Tensor] = None):
    """Qwen3RMSNorm over the last dimension in one pass.  With `residual`, returns (x + residual, norm(x + residual));
    otherwise norm(x).  x / residual: contiguous bf16 (..., hidden)."""
    op = "rmsnorm"
    if x.dtype not in _SUPPORTED_DTYPES or weight.dtype != x.dtype or not x.is_cuda:
        raise ValueError(f"{op}: x and weight must be CUDA torch.bfloat16 tensors")
    _require_contiguous(op, "x", x)
    _require_arch(op, x.device)
    hidden = x.shape[-1]
    out = torch.empty_like(x)
    a = N.RmsNormArgs(x.data_ptr(), None, weight.data_ptr(), None, out.data_ptr(), x.numel() // hidden, hidden, float(eps))
    summed = None
    if residual is not None:
        if residual.shape != x.shape or residual.dtype != x.dtype:
            raise ValueError(f"{op}: residual must match x")
        _require_contiguous(op, "residual", residual)
        summed = torch.empty_like(x)
        a.residual, a.sum_out = residual.data_ptr(), summed.data_ptr()
    with torch.cuda.device(x.device):
        _call("jl_rmsnorm", lambda: N.lib().jl_rmsnorm(C.byref(a), _stream()))
    return (summed, out) if residual is not None else out


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up in one pass (contiguous bf16 tensors of one shape, numel a multiple of 8)."""
    op = "silu_mul"
    if gate.dtype not in _SUPPORTED_DTYPES or up.dtype != gate.dtype or not gate.is_cuda or gate.shape != up.shape:
        raise ValueError(f"{op}: gate and up must be CUDA torch.bfloat16 tensors of one shape")
    _require_contiguous(op, "gate", gate)
    _require_contiguous(op, "up", up)
    _require_arch(op, gate.device)
    out = torch.empty_like(gate)
    a = N.SiluMulArgs(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel())
    with torch.cuda.device(gate.device):
        _call("jl_silu_mul", lambda: N.lib().jl_silu_mul(C.byref(a), _stream()))
    return out


def norm_rope(x: torch.Tensor, weight: torch.Tensor, inv_freq: torch.Tensor, *, eps: float, pos0: int = 0,
              group_size: Optional[int] = None, pos_block: int = 0, pos_block_stride: int = 0,
              out_base: Optional[torch.Tensor] = None, out_group: Optional[torch.Tensor] = None):
    """Per-head RMSNorm (Qwen3RMSNorm roundings) + base RoPE of a (B,S,H,D) projection output in one
    pass; with group_size also the jetlong-regrouped operand.  Returns out_base or (out_base, out_group)."""
    op = "norm_rope"
    _check_view(op, "x", x)
    if x.dtype not in _SUPPORTED_DTYPES or weight.dtype != x.dtype:
        raise ValueError(f"{op}: x and weight must be torch.bfloat16")
    _require_arch(op, x.device)
    B, S, H, D = x.shape
    if weight.numel() != D or not weight.is_contiguous():
        raise ValueError(f"{op}: weight must be a contiguous ({D},) tensor")
    if out_base is None:
        out_base = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    want_group = group_size is not None
    if want_group and out_group is None:
        out_group = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    for name, t in (("out_base", out_base),) + ((("out_group", out_group),) if want_group else ()):
        _check_view(op, name, t)
        if t.shape != x.shape:
            raise ValueError(f"{op}: {name} must have shape {tuple(x.shape)}")
    inv_freq = inv_freq.to(device=x.device, dtype=torch.float32).contiguous()
    a = N.NormRopeArgs(x.data_ptr(), weight.data_ptr(), out_base.data_ptr(), out_group.data_ptr() if want_group else None,
                       _st(x, 0), _st(x, 1), _st(x, 2), _st(out_base, 0), _st(out_base, 1), _st(out_base, 2),
                       *((_st(out_group, 0), _st(out_group, 1), _st(out_group, 2)) if want_group else (0, 0, 0)),
                       B, S, H, D, float(eps), int(group_size) if want_group else 1,
                       int(pos0), int(pos_block), int(pos_block_stride), inv_freq.data_ptr())
    with torch.cuda.device(x.device):
        _call("jl_norm_rope", lambda: N.lib().jl_norm_rope(C.byref(a), _stream()))
    return (out_base, out_group) if want_group else out_base


# ----------------------------------------------------------------------------------------------
# merge
# ----------------------------------------------------------------------------------------------

def merge_partials(o_parts: Sequence[torch.Tensor], lse_parts: Sequence[torch.Tensor], *,
                   out: Optional[torch.Tensor] = None, lse_out: Optional[torch.Tensor] = None,
                   return_lse: bool = True, round_like_reference: bool = False):
    """N-way (O, LSE) merge.  o_parts[i]: (B,S,H,D) contiguous bf16; lse_parts[i]: (B,H,S) fp32 contiguous.
    A stacked (N,B,S,H,D) / (N,B,H,S) pair is accepted too.  Returns out or (out, lse)."""
    op = "merge_partials"
    if isinstance(o_parts, torch.Tensor):
        o_parts = list(o_parts.unbind(0))
    if isinstance(lse_parts, torch.Tensor):
        lse_parts = list(lse_parts.unbind(0))
    n = len(o_parts)
    if n < 1 or n > N.JL_MAX_PARTS or len(lse_parts) != n:
        raise ValueError(f"{op}: need between 1 and {N.JL_MAX_PARTS} (out, lse) pairs")
    o0 = o_parts[0]
    if o0.dim() != 4 or lse_parts[0].dim() != 3:
        raise ValueError("expected out=(B,S,H,D) and lse=(B,H,S)")
    if not o0.is_cuda:
        raise ValueError("fused merge requires CUDA tensors")
    if o0.dtype not in _SUPPORTED_DTYPES:
        raise ValueError(f"{op}: partial outputs must be torch.bfloat16, got {o0.dtype}")
    _require_arch(op, o0.device)
    B, S, H, D = o0.shape
    for i, (o, l) in enumerate(zip(o_parts, lse_parts)):
        if o.shape != o0.shape or o.dtype != o0.dtype or o.device != o0.device:
            raise ValueError(f"{op}: part {i} shape/dtype/device mismatch")
        if tuple(l.shape) != (B, H, S) or l.dtype != torch.float32 or l.device != o0.device:
            raise ValueError(f"{op}: lse of part {i} must be float32 with shape {(B, H, S)}")
        _require_contiguous(op, f"o_parts[{i}]", o)
        _require_contiguous(op, f"lse_parts[{i}]", l)
    if out is None:
        out = torch.empty_like(o0)
    else:
        if out.shape != o0.shape or out.dtype != o0.dtype or out.device != o0.device:
            raise ValueError(f"{op}: out shape/dtype/device mismatch")
        _require_contiguous(op, "out", out)
    if lse_out is None and return_lse:
        lse_out = torch.empty(B, H, S, dtype=torch.float32, device=o0.device)
    if lse_out is not None:
        if tuple(lse_out.shape) != (B, H, S) or lse_out.dtype != torch.float32:
            raise ValueError(f"{op}: lse_out must be float32 with shape {(B, H, S)}")
        _require_contiguous(op, "lse_out", lse_out)
    a = N.MergeArgs()
    for i in range(n):
        a.o[i] = o_parts[i].data_ptr()
        a.lse[i] = lse_parts[i].data_ptr()
    a.n_parts, a.batch, a.seqlen, a.heads, a.head_dim = n, B, S, H, D
    a.round_like_reference = int(bool(round_like_reference))
    a.out = out.data_ptr()
    a.lse_out = lse_out.data_ptr() if lse_out is not None else None
    with torch.cuda.device(o0.device):
        _call("jl_merge", lambda: N.lib().jl_merge(C.byref(a), _stream()))
    return (out, lse_out) if return_lse else out


# ----------------------------------------------------------------------------------------------
# prefill
# ----------------------------------------------------------------------------------------------

def posmap_prefill(q_ops: Sequence[torch.Tensor], k_ops: Sequence[torch.Tensor], v: torch.Tensor, *,
                   pmap: PositionMap, q_pos0: int, k_pos0: int = 0, softmax_scale: Optional[float] = None,
                   k_block: int = 0, k_block_stride: int = 0, q_block: int = 0, q_block_stride: int = 0,
                   out: Optional[torch.Tensor] = None,
                   lse: Optional[torch.Tensor] = None, return_lse: bool = True, impl: int = 0,
                   remap_far: Optional[tuple] = None, stripes: Optional[tuple] = None):
    """Single-pass position-mapped causal attention (see jl_prefill).  q_ops[c]: (B,Sq,H,D) views sharing
    strides; k_ops[c], v: (B,Skv,Hk,D) views (all k_ops share strides).  Returns (out, lse) or out.
    remap_far = (inv_freq, group_size): jetlong band map with the far class formed INSIDE the kernel from the
    base-rotated operands; pass only [q_base] and [k_base].
    stripes = (first, count, pos_step): stripe batching.  q_ops / out / lse then hold W query stripes along dim 0
    (stripe e at positions q_pos0 + e * pos_step, plus the q_block rule), k_ops / v hold ONE batch element, and this
    launch processes stripes (first + i) % W for i < count, all against the same keys."""
    op = "posmap_prefill"
    keep = []
    if remap_far is not None:
        if len(q_ops) != 1 or len(k_ops) != 1 or pmap.kind != N.JL_MAP_BAND:
            raise ValueError(f"{op}: remap_far takes the band map and one base-rotated q and k operand")
        q_ops, k_ops = [q_ops[0], q_ops[0]], [k_ops[0], k_ops[0]]
    if len(q_ops) != pmap.n_classes or len(k_ops) != pmap.n_classes:
        raise ValueError(f"{op}: the position map has {pmap.n_classes} classes; got {len(q_ops)} q and {len(k_ops)} k operands")
    q0, k0 = q_ops[0], k_ops[0]
    tensors = [(f"q[{i}]", t) for i, t in enumerate(q_ops)] + [(f"k[{i}]", t) for i, t in enumerate(k_ops)] + [("v", v)]
    if not all(t.is_cuda for _, t in tensors):
        raise ValueError(f"{op} requires CUDA tensors")
    for name, t in tensors:
        _check_view(op, name, t)
    if q0.dtype not in _SUPPORTED_DTYPES:
        raise ValueError(f"{op}: q must have dtype torch.bfloat16, got {q0.dtype}")
    if not all(t.dtype == q0.dtype for _, t in tensors):
        raise ValueError(f"{op}: Q/K/V tensors must share dtype")
    if not all(t.device == q0.device for _, t in tensors):
        raise ValueError(f"{op}: all tensors must be on the same CUDA device")
    for t in q_ops[1:]:
        if t.shape != q0.shape or [_st(t, i) for i in range(3)] != [_st(q0, i) for i in range(3)]:
            raise ValueError(f"{op}: query operands must share shape and strides")
    for t in k_ops[1:]:
        if t.shape != k0.shape or [_st(t, i) for i in range(3)] != [_st(k0, i) for i in range(3)]:
            raise ValueError(f"{op}: key operands must share shape and strides")
    if k0.shape != v.shape:
        raise ValueError(f"{op}: keys and value must share shape")
    if stripes is not None:
        if k0.shape[0] != 1 or not (0 <= int(stripes[0]) < q0.shape[0]) or not (1 <= int(stripes[1]) <= q0.shape[0]):
            raise ValueError(f"{op}: stripes = (first, count, pos_step) needs one key batch element, "
                             f"0 <= first < {q0.shape[0]} and 1 <= count <= {q0.shape[0]}")
    elif q0.shape[0] != k0.shape[0]:
        raise ValueError(f"{op}: Q/K batch must match")
    if q0.shape[3] != k0.shape[3]:
        raise ValueError(f"{op}: Q/K head-dim must match")
    if q0.shape[2] % k0.shape[2] != 0:
        raise ValueError(f"{op}: q heads must be divisible by kv heads")
    _require_arch(op, q0.device)
    B, Sq, H, D = q0.shape
    Skv, Hk = k0.shape[1], k0.shape[2]
    if out is None:
        out = torch.empty(B, Sq, H, D, dtype=q0.dtype, device=q0.device)
    else:
        if tuple(out.shape) != (B, Sq, H, D) or out.dtype != q0.dtype or out.device != q0.device:
            raise ValueError(f"{op}: out must be {q0.dtype} with shape {(B, Sq, H, D)}")
        _check_view(op, "out", out)
    if lse is None and return_lse:
        lse = torch.empty(B, H, Sq, dtype=torch.float32, device=q0.device)
    if lse is not None:
        if tuple(lse.shape) != (B, H, Sq) or lse.dtype != torch.float32:
            raise ValueError(f"{op}: lse must be float32 with shape {(B, H, Sq)}")
        _require_contiguous(op, "lse", lse)
    a = N.PrefillArgs()
    for c in range(pmap.n_classes):
        a.q[c] = q_ops[c].data_ptr()
        a.k[c] = k_ops[c].data_ptr()
    a.v, a.out = v.data_ptr(), out.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.q_stride_b, a.q_stride_s, a.q_stride_h = _st(q0, 0), _st(q0, 1), _st(q0, 2)
    a.k_stride_b, a.k_stride_s, a.k_stride_h = _st(k0, 0), _st(k0, 1), _st(k0, 2)
    a.v_stride_b, a.v_stride_s, a.v_stride_h = _st(v, 0), _st(v, 1), _st(v, 2)
    a.o_stride_b, a.o_stride_s, a.o_stride_h = _st(out, 0), _st(out, 1), _st(out, 2)
    a.batch, a.seqlen_q, a.seqlen_k, a.heads, a.kv_heads, a.head_dim = B, Sq, Skv, H, Hk, D
    a.q_pos0, a.k_pos0, a.k_block, a.k_block_stride = int(q_pos0), int(k_pos0), int(k_block), int(k_block_stride)
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    a.map = pmap.c_struct()
    a.impl = int(impl)
    a.q_block, a.q_block_stride = int(q_block), int(q_block_stride)
    if stripes is not None:
        a.batch = int(stripes[1])
        a.q_batch_first, a.q_batch_wrap, a.q_pos0_batch_step = int(stripes[0]), B, int(stripes[2])
    if remap_far is not None:
        inv_freq = remap_far[0].to(device=q0.device, dtype=torch.float32).contiguous()
        keep.append(inv_freq)
        a.remap_far_in_kernel, a.group_size, a.inv_freq = 1, int(remap_far[1]), inv_freq.data_ptr()
    with torch.cuda.device(q0.device):
        _call("jl_prefill", lambda: N.lib().jl_prefill(C.byref(a), _stream()))
    return (out, lse) if return_lse else out


def jetlong_prefill(q_base, q_group, k_base, k_group, value, *, seqstart_q: torch.Tensor,
                    seqstart_q_scalar: Optional[int] = None, window_size_left: int,
                    softmax_scale: Optional[float] = None, tile_m: int = 128, tile_n: int = 128,
                    seqused_q=None, seqused_k=None, inv_freq=None, group_size=None, num_stages=None,
                    deterministic: bool = False, out=None, impl: int = 0):
    """Fused bifocal prefill with the tensor contract of the reference's level-2 entry point:
    (B,S,H,D) base/group operands, int32 seqstart_q (B,), returns (out (B,S,H,D), lse (B,H,S))."""
    op = "jetlong_prefill"
    unsupported = {"seqused_q": seqused_q, "seqused_k": seqused_k, "inv_freq": inv_freq,
                   "group_size": group_size, "num_stages": num_stages}
    used = [n for n, val in unsupported.items() if val is not None]
    if used:
        raise ValueError(f"{op}: unsupported metadata arguments for the fused prefill: {', '.join(used)}")
    if not all(t.is_cuda for t in (q_base, q_group, k_base, k_group, value, seqstart_q)):
        raise ValueError(f"{op} requires CUDA tensors")
    if not all(t.dim() == 4 for t in (q_base, q_group, k_base, k_group, value)):
        raise ValueError(f"{op} expects rank-4 BSHD tensors")
    if q_base.shape != q_group.shape:
        raise ValueError(f"{op}: q_base and q_group must share shape")
    if k_base.shape != k_group.shape or k_base.shape != value.shape:
        raise ValueError(f"{op}: k_base, k_group, and value must share shape")
    if seqstart_q.dtype != torch.int32 or seqstart_q.dim() != 1 or seqstart_q.shape[0] != q_base.shape[0]:
        raise ValueError(f"{op}: seqstart_q must be int32 with shape (batch,)")
    if tile_m <= 0 or tile_n <= 0:
        raise ValueError(f"{op}: tile_m and tile_n must be positive")
    if seqstart_q_scalar is None:
        vals = set(int(x) for x in seqstart_q.detach().cpu().tolist())
        if len(vals) != 1:
            raise ValueError("prefill fastpath requires uniform seqstart_q across batch")
        seqstart_q_scalar = vals.pop()
    return posmap_prefill([q_base, q_group], [k_base, k_group], value, pmap=PositionMap.jetlong(window_size_left),
                          q_pos0=int(seqstart_q_scalar), k_pos0=0, softmax_scale=softmax_scale, out=out, impl=impl)


# ----------------------------------------------------------------------------------------------
# decode
# ----------------------------------------------------------------------------------------------

@dataclass
class KvSegment:
    """One key/value range read in place by the decode kernel (see jl_kv_segment)."""
    k: torch.Tensor            # (B, len, Hk, D) view
    v: torch.Tensor
    q_class: int               # index into the query operand list
    rotate: bool = False       # regroup the keys in-kernel by (floor(p/G) - p) * inv_freq
    pos0: int = 0              # absolute position of row 0 (used when rotate)
    len_dev: Optional[torch.Tensor] = None   # optional int32 (B,) valid lengths
    pos_block: int = 0         # > 0: rows are a block-cyclic stripe, position = pos0 + (row // pos_block) * stride + row % pos_block
    pos_block_stride: int = 0
    row0_dev: Optional[torch.Tensor] = None  # optional int64 device scalar: the segment starts at that row of k / v


def decode_segments(q_ops: Sequence[Optional[torch.Tensor]], segments: Sequence[KvSegment], *,
                    softmax_scale: Optional[float] = None, inv_freq: Optional[torch.Tensor] = None,
                    group_size: int = 1, num_splits: int = 0, out: Optional[torch.Tensor] = None,
                    lse: Optional[torch.Tensor] = None, return_lse: bool = True,
                    workspace: Optional[torch.Tensor] = None):
    """Split-KV decode of one query token per sequence over in-place key segments (see jl_decode).
    q_ops[c]: (B,1,H,D) views sharing strides (None for unused classes).  Returns (out (B,1,H,D), lse (B,H,1)).
    A caller-provided `workspace` must have had its first 16 KB zeroed once (torch.zeros) before its first use."""
    op = "decode_segments"
    q0 = next(t for t in q_ops if t is not None)
    if q0.dim() != 4:
        raise ValueError(f"{op} expects rank-4 BSHD tensors")
    if q0.shape[1] != 1:
        raise ValueError(f"{op} requires seqlen_q == 1")
    if q0.dtype not in _SUPPORTED_DTYPES:
        raise ValueError(f"{op}: query must have dtype torch.bfloat16, got {q0.dtype}")
    if not q0.is_cuda:
        raise ValueError(f"{op} requires CUDA Q/K/V tensors")
    if not 1 <= len(segments) <= N.JL_MAX_SEGMENTS:
        raise ValueError(f"{op}: between 1 and {N.JL_MAX_SEGMENTS} segments")
    _require_arch(op, q0.device)
    B, _, H, D = q0.shape
    a = N.DecodeArgs()
    for c, t in enumerate(q_ops):
        if t is None:
            continue
        if t.shape != q0.shape or t.dtype != q0.dtype or t.device != q0.device:
            raise ValueError(f"{op}: query operands must share shape, dtype and device")
        _check_view(op, f"q[{c}]", t)
        if (_st(t, 0), _st(t, 2)) != (_st(q0, 0), _st(q0, 2)):
            raise ValueError(f"{op}: query operands must share strides")
        a.q[c] = t.data_ptr()
    a.q_stride_b, a.q_stride_h = _st(q0, 0), _st(q0, 2)
    Hk = segments[0].k.shape[2]
    total = 0
    keep = []
    for i, s in enumerate(segments):
        if s.k.dim() != 4 or s.v.dim() != 4:
            raise ValueError(f"{op} expects rank-4 BSHD tensors")
        if s.k.shape[:3] != s.v.shape[:3]:
            raise ValueError(f"{op}: each K/V branch must share batch, sequence, and head dimensions")
        if s.k.shape[0] != B:
            raise ValueError(f"{op}: Q/K/V batch sizes must match")
        if s.k.shape[2] != Hk:
            raise ValueError(f"{op}: near and distant KV head counts must match")
        if s.k.shape[-1] != D or s.v.shape[-1] != D:
            raise ValueError(f"{op}: query and key head_dim must match")
        if s.k.dtype != q0.dtype or s.v.dtype != q0.dtype:
            raise ValueError(f"{op}: Q/K/V tensors must share dtype")
        if s.k.device != q0.device or s.v.device != q0.device:
            raise ValueError(f"{op}: Q/K/V tensors must be on the same CUDA device")
        _check_view(op, f"segment[{i}].k", s.k)
        _check_view(op, f"segment[{i}].v", s.v)
        g = a.seg[i]
        g.k, g.v = s.k.data_ptr(), s.v.data_ptr()
        g.k_stride_b, g.k_stride_s, g.k_stride_h = _st(s.k, 0), _st(s.k, 1), _st(s.k, 2)
        g.v_stride_b, g.v_stride_s, g.v_stride_h = _st(s.v, 0), _st(s.v, 1), _st(s.v, 2)
        if s.len_dev is not None:
            if tuple(s.len_dev.shape) != (B,) or s.len_dev.dtype != torch.int32 or s.len_dev.device != q0.device:
                raise ValueError(f"{op}: segment lengths must be int32 with shape ({B},) on {q0.device}")
            keep.append(s.len_dev.contiguous())
            g.len_dev = keep[-1].data_ptr()
        g.pos0, g.len, g.q_class, g.rotate = int(s.pos0), int(s.k.shape[1]), int(s.q_class), int(bool(s.rotate))
        g.pos_block, g.pos_block_stride = int(s.pos_block), int(s.pos_block_stride)
        if s.row0_dev is not None:
            if s.row0_dev.numel() != 1 or s.row0_dev.dtype != torch.int64 or s.row0_dev.device != q0.device:
                raise ValueError(f"{op}: segment row offset must be one int64 on {q0.device}")
            g.row0_dev = s.row0_dev.data_ptr()
        total += int(s.k.shape[1])
    if H % Hk != 0:
        raise ValueError(f"{op}: query heads must be divisible by kv heads")
    a.n_segments, a.batch, a.heads, a.kv_heads, a.head_dim = len(segments), B, H, Hk, D
    a.num_splits = int(num_splits)
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    if inv_freq is not None:
        inv_freq = inv_freq.to(device=q0.device, dtype=torch.float32).contiguous()
        keep.append(inv_freq)
        a.inv_freq = inv_freq.data_ptr()
    a.group_size = int(group_size)
    if out is None:
        out = torch.empty(B, 1, H, D, dtype=q0.dtype, device=q0.device)
    if lse is None and return_lse:
        lse = torch.empty(B, H, 1, dtype=torch.float32, device=q0.device)
    a.out = out.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.o_stride_b, a.o_stride_h = _st(out, 0), _st(out, 2)
    lib = N.lib()
    # the library picks the split count (and the kernel) itself: size the scratch for its upper bound unless told
    need = lib.jl_decode_workspace_bytes(B, H, D, int(num_splits) if num_splits > 0 else 0)
    ws = workspace if workspace is not None else _workspace(q0.device, need)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel() * ws.element_size()
    with torch.cuda.device(q0.device):
        _call("jl_decode", lambda: lib.jl_decode(C.byref(a), _stream()))
    return (out, lse) if return_lse else out


class StepState:
    """Decode-step facts kept on the device (see jl_step_advance): `state` int64 (5,) =
    [pos, row, own, n_far, n_near] and `lens` int32 (2, B) = [n_far] * B, [n_near] * B.  Kernels whose host
    arguments never change read them, so one captured CUDA graph serves every new token."""

    def __init__(self, batch: int, device, w_0: int, shard=None):
        self.batch, self.w_0, self.shard = int(batch), int(w_0), shard
        self.state = torch.zeros(N.JL_STEP_STATE_WORDS, dtype=torch.int64, device=device)
        self.lens = torch.zeros(2, batch, dtype=torch.int32, device=device)

    @property
    def steps(self) -> torch.Tensor:
        """Number of advances made so far (device scalar, never rewound)."""
        return self.state[5:6]

    def peer_exchange(self, batch: int, heads: int, head_dim: int):
        """The peer-memory exchange of this (sharded) state, created on first use; None when the ranks could
        not all set it up (then the caller exchanges with NCCL)."""
        if getattr(self, "_peer", None) is None:
            from .sequence_parallel import make_peer_exchange
            self._peer = make_peer_exchange(self.shard, batch, heads, head_dim, self.state.device) or False
        return self._peer or None

    def set_next_position(self, pos: int) -> None:
        """The next advance() will describe the token at absolute position `pos`."""
        self.state[0] = int(pos) - 1

    def advance(self) -> None:
        sh = self.shard
        a = N.StepAdvanceArgs(self.state.data_ptr(), self.lens.data_ptr(), self.batch,
                              sh.rank if sh is not None else 0, sh.world if sh is not None else 1, 0,
                              sh.block if sh is not None else 1, self.w_0)
        with torch.cuda.device(self.state.device):
            _call("jl_step_advance", lambda: N.lib().jl_step_advance(C.byref(a), _stream()))

    # views the kernels take
    @property
    def position(self) -> torch.Tensor:
        return self.state[0:1]

    @property
    def n_far(self) -> torch.Tensor:
        return self.state[3:4]

    @property
    def far_lens(self) -> torch.Tensor:
        return self.lens[0]

    @property
    def near_lens(self) -> torch.Tensor:
        return self.lens[1]


def decode_append(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor,
                  inv_freq: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step: StepState, *,
                  q_eps: float, k_eps: float, group_size: int = 1, k_group_cache: Optional[torch.Tensor] = None):
    """One launch between the projections and the attention of a decode step: per-head RMSNorm + RoPE of
    q (B,1,H,D) and k (B,1,Hk,D) at the device-side position, the regrouped query when group_size > 1, and
    the write of the new key / value into row step.state[1] of k_cache / v_cache (B,rows,Hk,D) on the rank
    that owns the position.  k_group_cache (same shape and strides as k_cache), if given, keeps regrouped
    copies of the far rows: the call rewrites the newest far row (row n_far - 1) from k_cache.
    Returns (q_base, q_group), each (B,1,H,D); q_group is q_base when group_size == 1."""
    op = "decode_append"
    for name, t in (("q", q), ("k", k), ("v", v), ("k_cache", k_cache), ("v_cache", v_cache)):
        _check_view(op, name, t)
        if t.dtype not in _SUPPORTED_DTYPES:
            raise ValueError(f"{op}: {name} must be torch.bfloat16")
    _require_arch(op, q.device)
    B, one, H, D = q.shape
    Hk = k.shape[2]
    if one != 1 or k.shape != (B, 1, Hk, D) or v.shape != (B, 1, Hk, D):
        raise ValueError(f"{op}: expects q (B,1,H,D) and k, v (B,1,Hk,D)")
    if k_cache.shape[0] != B or k_cache.shape[2:] != (Hk, D) or v_cache.shape != k_cache.shape:
        raise ValueError(f"{op}: caches must be (B, rows, Hk, D)")
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w.numel() != D or not w.is_contiguous() or w.dtype != q.dtype:
            raise ValueError(f"{op}: {name} must be a contiguous ({D},) tensor of the query dtype")
    if k_group_cache is not None and (k_group_cache.shape != k_cache.shape or k_group_cache.stride() != k_cache.stride()
                                      or k_group_cache.dtype != k_cache.dtype):
        raise ValueError(f"{op}: k_group_cache must match k_cache in shape, strides and dtype")
    sh = step.shard if step.shard is not None and step.shard.world > 1 else None
    inv_freq = inv_freq.to(device=q.device, dtype=torch.float32).contiguous()
    q_base = torch.empty(B, 1, H, D, dtype=q.dtype, device=q.device)
    q_group = torch.empty(B, 1, H, D, dtype=q.dtype, device=q.device) if group_size > 1 else None
    a = N.DecodeAppendArgs(q.data_ptr(), k.data_ptr(), v.data_ptr(),
                           _st(q, 0), _st(q, 2), _st(k, 0), _st(k, 2), _st(v, 0), _st(v, 2),
                           q_weight.data_ptr(), k_weight.data_ptr(), float(q_eps), float(k_eps),
                           q_base.data_ptr(), q_group.data_ptr() if q_group is not None else None,
                           k_cache.data_ptr(), v_cache.data_ptr(),
                           _st(k_cache, 0), _st(k_cache, 1), _st(k_cache, 2), _st(v_cache, 0), _st(v_cache, 1), _st(v_cache, 2),
                           B, H, Hk, D, int(group_size), 0, int(k_cache.shape[1]), inv_freq.data_ptr(), step.state.data_ptr(),
                           k_group_cache.data_ptr() if k_group_cache is not None else None,
                           sh.rank * sh.block if sh is not None else 0, sh.block if sh is not None else 0,
                           sh.world * sh.block if sh is not None else 0)
    with torch.cuda.device(q.device):
        _call("jl_decode_append", lambda: N.lib().jl_decode_append(C.byref(a), _stream()))
    return q_base, (q_group if q_group is not None else q_base)


def peer_merge(part_o: torch.Tensor, part_lse: torch.Tensor, exchange, *, epoch_base: Optional[torch.Tensor],
               epoch_stride: int, epoch_offset: int, return_lse: bool = False, wait_limit_ms: int = 0):
    """Push this rank's decode partial (part_o (B,1,H,D) bf16, part_lse (B,H,1) fp32, both contiguous) to all
    ranks of `exchange` (sequence_parallel.PeerExchange) through peer-mapped memory, wait for theirs (at most
    wait_limit_ms, default 1 s; then exchange.status is raised and the result is invalid: check_status()) and merge
    (see jl_peer_merge).  The epoch (*epoch_base) * epoch_stride + epoch_offset must be >= 1, equal on all ranks
    and grow by exactly 1 from one call on this exchange to the next.  Returns out (B,1,H,D) or (out, lse)."""
    op = "peer_merge"
    B, one, H, D = part_o.shape
    if one != 1 or part_o.dtype not in _SUPPORTED_DTYPES or part_lse.dtype != torch.float32 or part_lse.numel() != B * H:
        raise ValueError(f"{op}: expects part_o (B,1,H,D) bf16 and part_lse (B,H,1) fp32")
    _require_contiguous(op, "part_o", part_o)
    _require_contiguous(op, "part_lse", part_lse)
    if (B, H, D) != (exchange.batch, exchange.heads, exchange.head_dim):
        raise ValueError(f"{op}: the exchange was built for (batch, heads, head_dim) = "
                         f"{(exchange.batch, exchange.heads, exchange.head_dim)}, got {(B, H, D)}")
    _require_arch(op, part_o.device)
    out = torch.empty_like(part_o)
    lse = torch.empty(B, H, 1, dtype=torch.float32, device=part_o.device) if return_lse else None
    a = N.PeerMergeArgs()
    a.part_o, a.part_lse = part_o.data_ptr(), part_lse.data_ptr()
    for r, ptr in enumerate(exchange.ptrs):
        a.peer_buf[r] = ptr
    a.buffer_bytes = exchange.nbytes
    a.rank, a.world = exchange.shard.rank, exchange.shard.world
    a.batch, a.heads, a.head_dim = B, H, D
    if epoch_base is not None:
        if epoch_base.numel() != 1 or epoch_base.dtype != torch.int64 or epoch_base.device != part_o.device:
            raise ValueError(f"{op}: epoch_base must be one int64 on {part_o.device}")
        a.epoch_base_dev = epoch_base.data_ptr()
    a.epoch_stride, a.epoch_offset = int(epoch_stride), int(epoch_offset)
    a.out = out.data_ptr()
    a.lse_out = lse.data_ptr() if lse is not None else None
    a.status = exchange.status.data_ptr()
    a.wait_limit_ms = int(wait_limit_ms)
    with torch.cuda.device(part_o.device):
        _call("jl_peer_merge", lambda: N.lib().jl_peer_merge(C.byref(a), _stream()))
    return (out, lse) if return_lse else out


def _require_output(op, name, t, shape, dtype, device):
    if t is None:
        return
    if tuple(t.shape) != shape:
        raise ValueError(f"{op}: {name} must have shape {shape}, got {tuple(t.shape)}")
    if t.dtype != dtype:
        raise ValueError(f"{op}: {name} must have dtype {dtype}, got {t.dtype}")
    if t.device != device:
        raise ValueError(f"{op}: {name} must be on device {device}, got {t.device}")
    _require_contiguous(op, name, t)


def _require_metadata(op, name, t, shape, device):
    if tuple(t.shape) != shape:
        raise ValueError(f"{op}: {name} must have shape {shape}, got {tuple(t.shape)}")
    if t.dtype != torch.int32:
        raise ValueError(f"{op}: {name} must have dtype torch.int32, got {t.dtype}")
    if t.device != device:
        raise ValueError(f"{op}: {name} must be on device {device}, got {t.device}")


def jetlong_decode(query_base, query_group, key_near, value_near, key_distant, value_distant, *,
                   seqused_near: torch.Tensor, seqused_distant: torch.Tensor, jetlong_meta=None,
                   inv_freq: torch.Tensor, group_size: int, out=None, lse=None, tile_m: int = 64,
                   tile_n: int = 128, num_stages: int = 3, pack_gqa=None, k_mode: str = "consumer",
                   num_splits: int = 0, active_splits=None, distant_k_grouped: bool = False,
                   distant_pos0: int = 0):
    """Fused bifocal decode with the tensor contract of the reference's level-2 entry point.

    Near keys are scored with query_base, distant keys with query_group.  With
    distant_k_grouped=False the distant keys are base-rotated and are regrouped in-kernel
    (positions distant_pos0 + row).  Returns out, or (out, lse) when an lse tensor is passed."""
    op = "jetlong_decode"
    named = (("query_base", query_base), ("query_group", query_group), ("key_near", key_near),
             ("value_near", value_near), ("key_distant", key_distant), ("value_distant", value_distant))
    if not all(t.dim() == 4 for _, t in named):
        raise ValueError(f"{op} expects rank-4 BSHD tensors")
    if query_base.shape != query_group.shape:
        raise ValueError(f"{op}: query_base and query_group must share shape")
    if query_base.shape[1] != 1:
        raise ValueError(f"{op} requires seqlen_q == 1")
    if not all(t.is_cuda for _, t in named):
        raise ValueError(f"{op} requires CUDA Q/K/V tensors")
    if num_splits < 0:
        raise ValueError(f"{op}: num_splits must be >= 0")
    if inv_freq.device != query_base.device:
        raise ValueError(f"{op}: inv_freq must be on device {query_base.device}, got {inv_freq.device}")
    if inv_freq.dim() != 1 or inv_freq.numel() < query_base.shape[-1] // 2:
        raise ValueError(f"{op}: inv_freq must have shape ({query_base.shape[-1] // 2},) or larger")
    if not torch.is_floating_point(inv_freq):
        raise ValueError(f"{op}: inv_freq must be a floating-point tensor, got {inv_freq.dtype}")
    B, _, H, D = query_base.shape
    dev = query_base.device
    _require_metadata(op, "seqused_near", seqused_near, (B,), dev)
    _require_metadata(op, "seqused_distant", seqused_distant, (B,), dev)
    _require_output(op, "out", out, (B, 1, H, value_near.shape[-1]), query_base.dtype, dev)
    _require_output(op, "lse", lse, (B, H, 1), torch.float32, dev)
    if jetlong_meta is not None:
        if jetlong_meta.dtype != torch.int32 or jetlong_meta.dim() != 2 or jetlong_meta.shape[1] < 3:
            raise ValueError("jetlong_meta must be int32 with shape (B, >=3): [total_kv_len, boundary, group_size]")
    if active_splits is not None:
        _require_metadata(op, "active_splits", active_splits, (B,), dev)
    return_lse = lse is not None
    segs = [KvSegment(key_distant, value_distant, q_class=1, rotate=not distant_k_grouped, pos0=distant_pos0,
                      len_dev=seqused_distant),
            KvSegment(key_near, value_near, q_class=0, len_dev=seqused_near)]
    res = decode_segments([query_base, query_group], segs, inv_freq=inv_freq, group_size=group_size,
                          num_splits=num_splits, out=out, lse=lse, return_lse=return_lse)
    return res


# Names the reference's tests and benches import; same tensor contracts, B200 kernels underneath.
fa4_cute_prefill_sm90_jetlong_fused = jetlong_prefill
fa4_cute_decode_sm90_jetlong_fused = jetlong_decode

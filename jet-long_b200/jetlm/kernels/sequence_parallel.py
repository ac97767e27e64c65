"""KV-sequence sharding of the bifocal attention across the GPUs of one node.

Softmax attention over a key set is associative under the (O, LSE) merge, so the key positions are
split across ranks, every rank attends all its queries to its own keys, the partial (O, LSE) pairs
are exchanged with ONE all-gather (NCCL over NVLink; remote data always lands in local HBM before
the merge kernel reads it) and merged N-way on every rank.  There is no counterpart in the
reference, which only replicates whole models across GPUs.

Prefill uses a block-cyclic placement (block b belongs to rank b % world) so that causal work and
cache memory are balanced; decode uses contiguous ranges.  The geometry helpers are pure Python and
are exercised on CPU ranks (gloo) by the tests; the attention and merge callables are injected, so
the same driver runs the CUDA kernels on GPUs and the oracle in those CPU tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist


@dataclass
class SequenceShard:
    rank: int
    world: int
    block: int = 1024                 # keys per placement block (multiple of the kernels' 128-key tile)
    group: Optional[object] = None    # torch.distributed process group (None = default)

    # ---- block-cyclic placement (prefill) ----
    def owned_rows(self, n_keys: int) -> torch.Tensor:
        """Global key rows owned by this rank, ascending."""
        starts = range(self.rank * self.block, n_keys, self.world * self.block)
        if len(starts) == 0:
            return torch.empty(0, dtype=torch.long)
        return torch.cat([torch.arange(s, min(s + self.block, n_keys)) for s in starts])

    def n_owned(self, n_keys: int) -> int:
        full, rem = divmod(n_keys, self.world * self.block)
        extra = min(max(rem - self.rank * self.block, 0), self.block)
        return full * self.block + extra

    def geometry(self) -> tuple[int, int, int]:
        """(k_pos0, k_block, k_block_stride) of the owned rows for jl_prefill's key-position map."""
        return self.rank * self.block, self.block, self.world * self.block

    def take_stripe(self, x: torch.Tensor, dim: int = 1) -> torch.Tensor:
        """The owned blocks of x along `dim`, packed contiguously (what this rank's cache holds)."""
        n = x.shape[dim]
        idx = self.owned_rows(n).to(x.device)
        return x.index_select(dim, idx)

    # ---- contiguous placement (decode) ----
    def contiguous_range(self, n_keys: int) -> tuple[int, int]:
        per = -(-n_keys // self.world)
        lo = min(self.rank * per, n_keys)
        return lo, min(lo + per, n_keys)


class PartialBuffer:
    """One allocation that is both where this rank's kernel writes its partial (O, LSE) and the
    receive buffer of the all-gather: slot r holds rank r's O (bf16/fp32) followed by its LSE (fp32).
    The local kernel writes straight into slot `rank`, the collective runs in place, and the merge
    kernel reads the slots where they land — no packing or unpacking copies."""

    def __init__(self, shard: SequenceShard, out_shape, lse_shape, out_dtype, device):
        self.shard = shard
        self.out_shape, self.lse_shape, self.out_dtype = tuple(out_shape), tuple(lse_shape), out_dtype
        esz = torch.empty(0, dtype=out_dtype).element_size()
        n_out = 1
        for d in out_shape:
            n_out *= d
        n_lse = 1
        for d in lse_shape:
            n_lse *= d
        self.o_bytes = (n_out * esz + 255) // 256 * 256            # keep the LSE block 256-byte aligned
        self.slot_bytes = (self.o_bytes + n_lse * 4 + 255) // 256 * 256
        self._n_out, self._n_lse, self._esz = n_out, n_lse, esz
        self.buf = torch.empty(shard.world, self.slot_bytes, dtype=torch.uint8, device=device)

    def out_view(self, r: int) -> torch.Tensor:
        return self.buf[r, : self._n_out * self._esz].view(self.out_dtype).view(self.out_shape)

    def lse_view(self, r: int) -> torch.Tensor:
        return self.buf[r, self.o_bytes: self.o_bytes + self._n_lse * 4].view(torch.float32).view(self.lse_shape)

    def gather(self):
        """In-place all-gather of the slots; returns ([out_r], [lse_r]) views for r in range(world)."""
        sh = self.shard
        dist.all_gather_into_tensor(self.buf.view(-1), self.buf[sh.rank].view(-1), group=sh.group)
        return [self.out_view(r) for r in range(sh.world)], [self.lse_view(r) for r in range(sh.world)]


PEER_EXCHANGE_VALIDATED_WORLDS = (2, 4, 8)      # rank counts on which jl_peer_merge has been run against the NCCL path


class PeerExchange:
    """Exchange buffers for `jl_peer_merge`: one symmetric allocation per rank, mapped into every rank of the
    group (torch symmetric memory: CUDA virtual-memory handles exchanged once at set-up), zeroed, plus the
    device status word the kernel raises if a bounded wait gives up.  The buffers serve one monotonically
    growing epoch sequence; create a new object for a new sequence."""

    def __init__(self, shard: SequenceShard, batch: int, heads: int, head_dim: int, device):
        import torch.distributed._symmetric_memory as symm_mem
        from . import _native as N
        self.shard, self.batch, self.heads, self.head_dim = shard, int(batch), int(heads), int(head_dim)
        self.nbytes = int(N.lib().jl_peer_merge_buffer_bytes(shard.world, batch, heads, head_dim))
        if self.nbytes == 0:
            raise ValueError("unsupported shape for the peer exchange")
        group = shard.group if shard.group is not None else dist.group.WORLD
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.ptrs) != shard.world or self.ptrs[shard.rank] != self.buf.data_ptr():
            raise RuntimeError("symmetric memory rendezvous returned an unexpected mapping")
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        from . import jetlong_ops
        jetlong_ops.register_peer_exchange(self)       # so that jetlong_ops.check_status() sees this status word
        self.epoch = torch.zeros(1, dtype=torch.int64, device=device)     # for callers without an epoch source of their own
        torch.cuda.synchronize(device)
        dist.barrier(group=group)             # every rank's zeroes are in place before anyone pushes

    def failed(self) -> bool:
        """True if a wait inside jl_peer_merge ever gave up (synchronises)."""
        return bool(self.status.item())


def make_peer_exchange(shard: SequenceShard, batch: int, heads: int, head_dim: int, device) -> Optional[PeerExchange]:
    """A PeerExchange if EVERY rank of the shard could set one up (the ranks agree through an all-reduce, so they
    all take the same path), else None.  JETLONG_PEER_EXCHANGE=0 disables it, =1 enables it for any rank count;
    unset, it is used for the rank counts it has been validated on (PEER_EXCHANGE_VALIDATED_WORLDS)."""
    import os
    import warnings
    ok, ex = 1, None
    mode = os.environ.get("JETLONG_PEER_EXCHANGE", "")
    if mode == "0" or (mode != "1" and shard.world not in PEER_EXCHANGE_VALIDATED_WORLDS):
        ok = 0
    else:
        try:
            ex = PeerExchange(shard, batch, heads, head_dim, device)
        except Exception as err:                # no symmetric-memory support on this system
            warnings.warn(f"peer-memory exchange unavailable ({err}); using NCCL")
            ok = 0
    agree = torch.tensor([ok], dtype=torch.int32, device=device)
    dist.all_reduce(agree, op=dist.ReduceOp.MIN, group=shard.group)
    return ex if int(agree) == 1 else None


class StripeExchange:
    """Receive buffers of the sequence-parallel Q exchange in symmetric memory.  A rank writes the partial (O, LSE) it
    computed for the query stripe of rank d straight into rank d's buffer with peer-to-peer copies on a side stream:
    the copy engines move them, no SM is needed, so they run under the next attention launch (an NCCL send / receive
    kernel does not get an SM while the attention grid has blocks to place: its CTAs hold every register of theirs).
    One small all-reduce per call, issued after this rank's side stream has drained, tells every rank that all
    partials addressed to it have landed.  Two buffers alternate from call to call, so a fast rank that is already
    writing the next call's partials never touches what a slow rank is still merging (it cannot be two calls ahead:
    the all-reduce in between needs the slow rank, whose stream reaches it only after that merge)."""

    def __init__(self, shard: SequenceShard, batch: int, rows: int, heads: int, head_dim: int, dtype, device):
        import torch.distributed._symmetric_memory as symm_mem
        N = shard.world
        self.shard = shard
        self.o_shape, self.l_shape = (N, batch, rows, heads, head_dim), (N, batch, heads, rows)
        esz = torch.empty(0, dtype=dtype).element_size()
        o_bytes = (N * batch * rows * heads * head_dim * esz + 255) // 256 * 256
        slot = o_bytes + (N * batch * heads * rows * 4 + 255) // 256 * 256
        group = shard.group if shard.group is not None else dist.group.WORLD
        self.buf = symm_mem.empty(2 * slot, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        view = lambda r, p: (self.handle.get_buffer(r, self.o_shape, dtype, (p * slot) // esz),
                             self.handle.get_buffer(r, self.l_shape, torch.float32, (p * slot + o_bytes) // 4))
        self.views = [[view(r, p) for r in range(N)] for p in range(2)]          # [buffer][rank] -> (O, LSE) of that rank
        self.side = torch.cuda.Stream(device=device)
        self.token = torch.zeros(1, dtype=torch.int32, device=device)
        self.parity = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def begin(self):
        """Start a call: returns this rank's receive views (O (N,B,rows,H,D), LSE (N,B,H,rows)) of the call's buffer."""
        self.parity ^= 1
        return self.views[self.parity][self.shard.rank]

    def push(self, dests, send_o, send_l):
        """Copy send_o[d] / send_l[d] (the partial of rank d's stripe, computed by kernels already enqueued on the
        current stream) into rank d's slot for this rank, on the side stream."""
        me = self.shard.rank
        self.side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.side):
            for d in dests:
                o, l = self.views[self.parity][d]
                o[me].copy_(send_o[d], non_blocking=True)
                l[me].copy_(send_l[d], non_blocking=True)

    def finish(self):
        """All pushes of all ranks are complete when this returns (on the current stream)."""
        torch.cuda.current_stream().wait_stream(self.side)
        dist.all_reduce(self.token, group=self.shard.group)


def make_stripe_exchange(shard: SequenceShard, batch: int, rows: int, heads: int, head_dim: int, dtype, device):
    """A StripeExchange if EVERY rank could set one up (agreed through an all-reduce), else None (the NCCL all-to-all
    is used).  JETLONG_PREFILL_PEER_COPY=0 disables it."""
    import os
    import warnings
    ok, ex = 1, None
    if os.environ.get("JETLONG_PREFILL_PEER_COPY", "") == "0":
        ok = 0
    else:
        try:
            ex = StripeExchange(shard, batch, rows, heads, head_dim, dtype, device)
        except Exception as err:                # no symmetric-memory support on this system
            warnings.warn(f"peer-copy exchange unavailable ({err}); using the NCCL all-to-all")
            ok = 0
    agree = torch.tensor([ok], dtype=torch.int32, device=device)
    dist.all_reduce(agree, op=dist.ReduceOp.MIN, group=shard.group)
    return ex if int(agree) == 1 else None


def interleave_stripes(stage: torch.Tensor, block: int, out: torch.Tensor) -> torch.Tensor:
    """Block-cyclic stripes, rank-major as an all-gather delivers them, into position order.
    stage (N, C, B, R, ...): rank r's R rows are positions r*block + (i // block) * N*block + i % block;
    out (C, B, R * N, ...): row p is position p.  One strided copy."""
    N, C, B, R = stage.shape[:4]
    tail = tuple(stage.shape[4:])
    if R % block != 0:
        raise ValueError(f"stripes must hold whole blocks: {R} rows, block {block}")
    nb = R // block
    if tuple(out.shape) != (C, B, R * N) + tail:
        raise ValueError(f"out must have shape {(C, B, R * N) + tail}, got {tuple(out.shape)}")
    src = stage.view(N, C, B, nb, block, *tail).permute(1, 2, 3, 0, 4, *range(5, 5 + len(tail)))
    out.view(C, B, nb, N, block, *tail).copy_(src)
    return out


def gather_partials(out: torch.Tensor, lse: torch.Tensor, shard: SequenceShard):
    """All-gather one (O, LSE) pair per rank.  out (B,S,H,D), lse (B,H,S) fp32 ->
    (outs (world,B,S,H,D), lses (world,B,H,S)), identical on every rank."""
    outs = torch.empty((shard.world, *out.shape), dtype=out.dtype, device=out.device)
    lses = torch.empty((shard.world, *lse.shape), dtype=lse.dtype, device=lse.device)
    dist.all_gather_into_tensor(outs.view(-1), out.contiguous().view(-1), group=shard.group)
    dist.all_gather_into_tensor(lses.view(-1), lse.contiguous().view(-1), group=shard.group)
    return outs, lses


def sharded_attention(local_attention: Callable[..., tuple[torch.Tensor, torch.Tensor]],
                      merge: Callable[[Sequence[torch.Tensor], Sequence[torch.Tensor]], tuple[torch.Tensor, torch.Tensor]],
                      shard: SequenceShard, buffer: Optional[PartialBuffer] = None):
    """partial (O, LSE) over this rank's keys -> all-gather -> N-way merge.  Returns (out, lse).

    Without `buffer`, local_attention() returns its (out, lse) and they are gathered into fresh tensors.
    With `buffer`, local_attention(out=..., lse=...) must write into the given views (slot `rank` of the
    buffer) and the gather runs in place."""
    if buffer is not None:
        local_attention(out=buffer.out_view(shard.rank), lse=buffer.lse_view(shard.rank))
        if shard.world == 1:
            return buffer.out_view(0), buffer.lse_view(0)
        outs, lses = buffer.gather()
        return merge(outs, lses)
    out, lse = local_attention()
    if shard.world == 1:
        return out, lse
    outs, lses = gather_partials(out, lse, shard)
    return merge(list(outs.unbind(0)), list(lses.unbind(0)))

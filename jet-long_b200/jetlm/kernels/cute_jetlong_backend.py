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
from .sequence_parallel import (PartialBuffer, SequenceShard, interleave_stripes, make_peer_exchange,
                                sharded_attention)

_SHARD: SequenceShard | None = None
_BUFFERS: dict[tuple, PartialBuffer] = {}


def _partial_buffer(shard, out_shape, lse_shape, dtype, device) -> PartialBuffer:
    """Gather buffers are cached per shape: the same (O, LSE) exchange repeats every layer and step."""
    key = (shard.rank, shard.world, tuple(out_shape), tuple(lse_shape), dtype, device)
    buf = _BUFFERS.get(key)
    if buf is None:
        buf = _BUFFERS[key] = PartialBuffer(shard, out_shape, lse_shape, dtype, device)
    return buf


_PEERS: dict[tuple, object] = {}


def _sharded_decode(part, sh, query_base, return_lse: bool, exchange):
    """Exchange and merge the ranks' decode partials.  part(out, lse) runs this rank's kernel (into the given
    tensors, or fresh ones when they are None).  exchange: "peer" = jl_peer_merge over peer-mapped memory,
    "nccl" = all-gather + jl_merge, None = peer when the ranks can set it up, else NCCL."""
    B, _, H, D = query_base.shape
    ex = None
    if exchange != "nccl":
        key = (sh.rank, sh.world, B, H, D, query_base.device)
        if key not in _PEERS:
            _PEERS[key] = make_peer_exchange(sh, B, H, D, query_base.device)
        ex = _PEERS[key]
        if ex is None and exchange == "peer":
            raise RuntimeError("the peer-memory exchange could not be set up on every rank")
    if ex is not None:
        part_o, part_lse = part(None, None)
        ex.epoch.add_(1)                    # in-stream, so a captured graph advances it on every replay
        return ops.peer_merge(part_o, part_lse, ex, epoch_base=ex.epoch, epoch_stride=1, epoch_offset=0,
                              return_lse=return_lse)
    buf = _partial_buffer(sh, (B, 1, H, D), (B, H, 1), query_base.dtype, query_base.device)
    out, lse = sharded_attention(part, ops.merge_partials, sh, buf)
    return (out, lse) if return_lse else out


def configure_sequence_sharding(shard: SequenceShard | None) -> None:
    """Split the key sequence of every following call across the ranks of `shard` (None = off).
    Prefill takes a block-cyclic stripe of the keys, decode a contiguous range; partial (O, LSE)
    pairs are all-gathered and merged, so every rank still returns the full result."""
    global _SHARD
    _SHARD = shard if shard is not None and shard.world > 1 else None


def sequence_shard() -> SequenceShard | None:
    return _SHARD


def token_sharded_prefill_mode(world: int, n_keys_total: int, n_queries_total: int, heads: int, kv_heads: int) -> str:
    """Which exchange the token-sharded prefill uses.  "kv_gather": all-gather K_base and V, every rank attends
    its own query stripe to ALL keys in one launch (no return trip, no merge); per rank it receives
    (N-1)/N * n_keys_total * kv_heads * D * 2 * 2 bytes.  "q_exchange": all-gather Q, every rank attends all
    query stripes to its OWN key stripe, partial (O, LSE) go back by all-to-all and are merged; it receives
    about (N-1)/N * n_queries_total * heads * D * 2 * 2 bytes, however long the cache already is.  The smaller
    volume wins: a fresh prompt under grouped-query attention gathers K / V (4x fewer bytes at 32 / 8 heads),
    a late chunk of a long chunked prefill keeps its keys at home.  JETLONG_SP_PREFILL=kv|q overrides."""
    import os
    forced = os.environ.get("JETLONG_SP_PREFILL", "")
    if forced in ("kv", "q"):
        return "kv_gather" if forced == "kv" else "q_exchange"
    return "kv_gather" if n_keys_total * kv_heads <= n_queries_total * heads else "q_exchange"


class KvGather:
    """An all-gather of this rank's K_base / V stripes that is already in flight (token_sharded_kv_gather_begin):
    the model starts it as soon as the keys and values of a layer exist, so that it runs behind the query projection."""

    def __init__(self, bufs, work, rows):
        self.bufs, self.work, self.rows = bufs, work, rows


def token_sharded_kv_gather_begin(key_base, value) -> KvGather:
    """Start the K/V gather of the "kv_gather" exchange: key_base / value (B, R, Hk, D) views of this rank's cache
    stripe.  Returns the handle fused_jetlong_prefill_token_sharded(..., gather=handle) finishes."""
    import torch.distributed as dist
    sh = _SHARD
    if sh is None:
        raise RuntimeError("token-sharded prefill needs configure_sequence_sharding(...) first")
    N, blk, me = sh.world, sh.block, sh.rank
    B, R, Hk, D = key_base.shape
    if R % blk != 0:
        raise ValueError(f"token-sharded prefill needs whole blocks per rank: {R} cache rows, block {blk}")
    dev, dt = key_base.device, key_base.dtype
    key = ("kvg", me, N, B, R, Hk, D, dt, dev)
    bufs = _BUFFERS.get(key)
    if bufs is None:
        for old in [k for k in _BUFFERS if k[0] == "kvg"]:      # a chunked prefill changes R every call: keep one set
            del _BUFFERS[old]
        bufs = _BUFFERS[key] = dict(
            stage=torch.empty(N, 2, B, R, Hk, D, dtype=dt, device=dev),        # [rank][K / V] stripes as they arrive
            full=torch.empty(2, B, R * N, Hk, D, dtype=dt, device=dev),        # K_base / V in position order
            k_grp=torch.empty(B, R * N, Hk, D, dtype=dt, device=dev))
    stage = bufs["stage"]
    stage[me, 0].copy_(key_base)
    stage[me, 1].copy_(value)
    work = dist.all_gather_into_tensor(stage.view(-1), stage[me].view(-1), group=sh.group, async_op=True)
    return KvGather(bufs, work, R)


def _prefill_kv_gather(query_base, key_base, value, *, q_start, inv_freq, group_size, window_size_left, softmax_scale,
                       gather=None):
    """Token-sharded prefill by gathering the keys: see token_sharded_prefill_mode.  The ranks' stripes arrive
    rank-major; one strided copy puts them into position order, the far-class keys are regrouped locally from the
    gathered base keys (one jl_rotate pass), and ONE jl_prefill launch attends this rank's block-cyclic query
    stripe to the whole key range."""
    sh = _SHARD
    N, blk, me = sh.world, sh.block, sh.rank
    B, S_loc, H, D = query_base.shape
    if gather is None:
        gather = token_sharded_kv_gather_begin(key_base, value)
    elif gather.rows != key_base.shape[1]:
        raise ValueError("the K/V gather handle was started for a different cache length")
    stage, full, k_grp = gather.bufs["stage"], gather.bufs["full"], gather.bufs["k_grp"]
    stride = N * blk
    regroup = int(group_size) > 1
    q_grp = query_base
    if regroup:     # the regrouped queries need no remote data: formed while the gather is in flight
        q_grp = ops.rope_regroup(query_base, inv_freq, group_size=int(group_size), pos0=int(q_start) + me * blk, pos_block=blk,
                                 pos_block_stride=stride)
    gather.work.wait()
    interleave_stripes(stage, blk, full)
    if regroup:
        ops.rope_regroup(full[0], inv_freq, group_size=int(group_size), pos0=0, out=k_grp)
    return ops.posmap_prefill([query_base, q_grp], [full[0], k_grp if regroup else full[0]], full[1],
                              pmap=ops.PositionMap.jetlong(int(window_size_left)), q_pos0=int(q_start) + me * blk,
                              q_block=blk, q_block_stride=stride, k_pos0=0, softmax_scale=softmax_scale, return_lse=False)


LAST_TOKEN_SHARDED_MODE = None      # "kv_gather" / "q_exchange": what the most recent token-sharded prefill call used


def fused_jetlong_prefill_token_sharded(query_base, key_base, key_group, value, *, q_start: int, inv_freq,
                                        group_size: int, window_size_left: int, softmax_scale: float, mode=None,
                                        gather=None):
    """Bifocal prefill when the TOKENS are sharded block-cyclically over the ranks (every rank ran the
    projections only for its own stripe of the prompt and keeps only its stripe of the KV cache).

    query_base (B, S_loc, H, D): this rank's base-rotated queries, row i at position
    q_start + rank*blk + (i // blk) * world*blk + i % blk.  key_base / key_group / value
    (B, Skv_loc, Hk, D) views: this rank's cache stripe (same geometry from position 0); key_group may be
    None (it is only read by the "q_exchange" form, which regroups on demand).
    mode None picks the cheaper exchange (token_sharded_prefill_mode); gather: a K/V gather the caller has already
    started with token_sharded_kv_gather_begin (kv_gather mode only).  The "q_exchange" form:
    all-gather the base-rotated queries (the regrouped ones are re-derived locally), attend
    every rank's query stripe to the local key stripe, send each partial (O, LSE) to the rank that
    owns those query rows (all-to-all), merge the N partials of the local rows.  Returns (B, S_loc, H, D).
    There K and V never cross NVLink; per layer a rank receives one copy of Q and one copy of O."""
    global LAST_TOKEN_SHARDED_MODE
    if _SHARD is None:
        raise RuntimeError("token-sharded prefill needs configure_sequence_sharding(...) first")
    if mode is None:
        mode = token_sharded_prefill_mode(_SHARD.world, key_base.shape[1] * _SHARD.world, query_base.shape[1] * _SHARD.world,
                                          query_base.shape[2], key_base.shape[2])
    LAST_TOKEN_SHARDED_MODE = mode
    if mode == "kv_gather":
        return _prefill_kv_gather(query_base, key_base, value, q_start=q_start, inv_freq=inv_freq, group_size=group_size,
                                  window_size_left=window_size_left, softmax_scale=softmax_scale, gather=gather)
    if key_group is None:
        key_group = key_base
        if int(group_size) > 1:
            key_group = torch.empty_strided(key_base.shape, key_base.stride(), dtype=key_base.dtype, device=key_base.device)
            ops.rope_regroup(key_base, inv_freq, group_size=int(group_size), pos0=_SHARD.rank * _SHARD.block,
                             pos_block=_SHARD.block, pos_block_stride=_SHARD.world * _SHARD.block, out=key_group)
    import torch.distributed as dist
    sh = _SHARD
    if sh is None:
        raise RuntimeError("token-sharded prefill needs configure_sequence_sharding(...) first")
    N, blk = sh.world, sh.block
    B, S_loc, H, D = query_base.shape
    if S_loc % blk != 0:
        raise ValueError(f"token-sharded prefill needs whole blocks per rank: {S_loc} local rows, block {blk}")
    dev, dt = query_base.device, query_base.dtype
    key = ("tok", sh.rank, N, B, S_loc, H, D, dt, dev)
    bufs = _BUFFERS.get(key)
    if bufs is None:
        bufs = _BUFFERS[key] = dict(
            q_all=torch.empty(N, B, S_loc, H, D, dtype=dt, device=dev),
            q_grp=torch.empty(N, B, S_loc, H, D, dtype=dt, device=dev),
            send_o=torch.empty(N, B, S_loc, H, D, dtype=dt, device=dev),
            send_l=torch.empty(N, B, H, S_loc, dtype=torch.float32, device=dev))
    if "peer" not in bufs:
        from .sequence_parallel import make_stripe_exchange
        bufs["peer"] = make_stripe_exchange(sh, B, S_loc, H, D, dt, dev)       # None: the NCCL all-to-all below
    peer = bufs["peer"]
    q_all, q_grp = bufs["q_all"], bufs["q_grp"]
    send_o, send_l = bufs["send_o"], bufs["send_l"]
    if peer is not None:
        recv_o, recv_l = peer.begin()              # this call's receive buffer in symmetric memory
    else:
        if "recv_o" not in bufs:                   # receive buffers of the all-to-all
            bufs["recv_o"] = torch.empty(N, B, S_loc, H, D, dtype=dt, device=dev)
            bufs["recv_l"] = torch.empty(N, B, H, S_loc, dtype=torch.float32, device=dev)
        recv_o, recv_l = bufs["recv_o"], bufs["recv_l"]
    pmap = ops.PositionMap.jetlong(int(window_size_left))
    stride = N * blk
    me = sh.rank

    def regroup(qb, r):
        ops.rope_regroup(qb, inv_freq, group_size=int(group_size), pos0=int(q_start) + r * blk, pos_block=blk,
                         pos_block_stride=stride, out=q_grp[r])

    def attend(qb, r, out, lse):
        """Queries of rank r's stripe (base-rotated, (B,S_loc,H,D)) against the local key stripe."""
        regroup(qb, r)
        ops.posmap_prefill([qb, q_grp[r]], [key_base, key_group], value, pmap=pmap,
                           q_pos0=int(q_start) + r * blk, q_block=blk, q_block_stride=stride,
                           k_pos0=me * blk, k_block=blk, k_block_stride=stride, softmax_scale=softmax_scale,
                           out=out, lse=lse)

    def attend_stripes(ranks):
        """The query stripes of consecutive ranks (mod N) against the local key stripe, partials into the send
        buffers.  With one sequence per batch the stripes are the batch of ONE launch (the kernel takes the stripe
        index modulo N and offsets the positions by a block per stripe), so the launch has enough CTAs to fill
        every SM for many rounds; N launches of one stripe each leave the last round of each partly empty."""
        if not ranks:
            return
        if B != 1:
            for r in ranks:
                attend(q_all[r], r, send_o[r], send_l[r])
            return
        for r in ranks:
            regroup(q_all[r], r)
        ops.posmap_prefill([q_all[:, 0], q_grp[:, 0]], [key_base, key_group], value, pmap=pmap,
                           q_pos0=int(q_start), q_block=blk, q_block_stride=stride,
                           k_pos0=me * blk, k_block=blk, k_block_stride=stride, softmax_scale=softmax_scale,
                           out=send_o[:, 0], lse=send_l[:, 0], stripes=(ranks[0], len(ranks), blk))

    def exchange(dests, async_op):
        """Send the partials of the query stripes owned by `dests`; receive my rows' partials from the
        ranks for which I am in the same phase (dest = source + k  <=>  source = dest - k)."""
        ks = [(d - me) % N for d in dests]
        srcs = {(me - k) % N for k in ks}
        e_o, e_l = send_o.new_empty(0), send_l.new_empty(0)
        works = []
        works.append(dist.all_to_all([recv_o[s].view(-1) if s in srcs else e_o for s in range(N)],
                                     [send_o[d].view(-1) if d in dests else e_o for d in range(N)],
                                     group=sh.group, async_op=async_op))
        works.append(dist.all_to_all([recv_l[s].view(-1) if s in srcs else e_l for s in range(N)],
                                     [send_l[d].view(-1) if d in dests else e_l for d in range(N)],
                                     group=sh.group, async_op=async_op))
        return works

    # 1. the query all-gather; the other ranks' stripes follow in two phases, the first phase's partials travel while
    #    the second is computed
    gather = dist.all_gather_into_tensor(q_all.view(-1), query_base.contiguous().view(-1), group=sh.group, async_op=True)
    order = [(me + k) % N for k in range(1, N)]
    first, second = order[: (N - 1 + 1) // 2], order[(N - 1 + 1) // 2:]
    if B == 1:
        # my own stripe rides in the first batched launch (a launch of one stripe leaves the SMs' last round half
        # empty; the gather it could hide is a hundredth of a late chunk's attention); its partial stays where it lands
        gather.wait()
        attend_stripes([me] + first)
        own_o, own_l = send_o[me], send_l[me]
    else:
        attend(query_base, me, recv_o[me], recv_l[me])       # needs no remote data: runs under the gather
        gather.wait()
        attend_stripes(first)
        own_o, own_l = recv_o[me], recv_l[me]
    if peer is not None:
        peer.push(first, send_o, send_l)          # peer-to-peer copies on a side stream, under the second launch
        attend_stripes(second)
        peer.push(second, send_o, send_l)
        peer.finish()
    else:
        pending = exchange(set(first), async_op=bool(second))
        attend_stripes(second)
        if second:
            for w in pending:
                w.wait()
            exchange(set(second), async_op=False)
    outs = [own_o if r == me else recv_o[r] for r in range(N)]
    lses = [own_l if r == me else recv_l[r] for r in range(N)]
    return ops.merge_partials(outs, lses, return_lse=False)


def fused_jetlong_prefill(query_base, query_group, key_base, key_group, value, *, seqstart_q: int,
                          window_size_left: int, softmax_scale: float, has_any_pad: bool, training: bool):
    """(B,H,S,D) / (B,Hk,Skv,D) views in, attention output (B,S,H,D) out."""
    if training:
        raise RuntimeError("JetLong backend 'fused' is inference-only")
    if has_any_pad:
        raise RuntimeError("JetLong backend 'fused' does not support left-padded prefill batches")
    t = lambda x: x.transpose(1, 2)
    if _SHARD is not None:
        sh = _SHARD
        pos0, blk, stride = sh.geometry()
        kb, kg, vv = (sh.take_stripe(x, dim=2) for x in (key_base, key_group, value))     # this rank's cache stripe
        B, H, S, D = query_base.shape
        local = lambda out, lse: ops.posmap_prefill([t(query_base), t(query_group)], [t(kb), t(kg)], t(vv),
                                                    pmap=ops.PositionMap.jetlong(int(window_size_left)),
                                                    q_pos0=int(seqstart_q), k_pos0=pos0, k_block=blk, k_block_stride=stride,
                                                    softmax_scale=softmax_scale, out=out, lse=lse)
        buf = _partial_buffer(sh, (B, S, H, D), (B, H, S), query_base.dtype, query_base.device)
        out, _ = sharded_attention(local, ops.merge_partials, sh, buf)
        return out
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


def fused_jetlong_decode_cache(query_base, query_group, key_cache, value_cache, *, boundary: int, inv_freq,
                               group_size: int, softmax_scale=None, has_any_pad: bool, training: bool,
                               cache_pos0: int = 0, return_lse: bool = False, key_cache_group=None, exchange=None):
    """Decode straight off a base-rotated (B,Hk,S,D) cache: keys [0, boundary) are the far class and are
    regrouped inside the kernel while they stream, keys [boundary, S) are the near class.  Replaces the
    reference's per-token host-side regroup of the whole distant cache plus its slice / pad copies
    (modeling :428-440, backend :143-155).  cache_pos0 is the absolute position of cache row 0 (non-zero
    for a sequence shard).  key_cache_group, if given, is a (B,Hk,S,D) cache of already regrouped keys: the far
    class then reads it as stored (the reference's contract) instead of regrouping key_cache in-kernel."""
    if training:
        raise RuntimeError("JetLong backend 'fused' is inference-only")
    if has_any_pad:
        raise RuntimeError("JetLong backend 'fused' does not support left-padded decode batches")
    kc, vc = key_cache.transpose(1, 2), value_cache.transpose(1, 2)        # (B,S,Hk,D) views
    kg = key_cache_group.transpose(1, 2) if key_cache_group is not None else None
    if _SHARD is not None and cache_pos0 == 0:
        sh = _SHARD
        lo, hi = sh.contiguous_range(kc.shape[1])
        B, _, H, D = query_base.shape
        part = lambda out, lse: _decode_range(query_base, query_group, kc[:, lo:hi], vc[:, lo:hi], int(boundary) - lo, lo,
                                              inv_freq, group_size, softmax_scale, True, out=out, lse=lse,
                                              kg=kg[:, lo:hi] if kg is not None else None, allow_empty=True)
        return _sharded_decode(part, sh, query_base, return_lse, exchange)
    return _decode_range(query_base, query_group, kc, vc, int(boundary) - int(cache_pos0), int(cache_pos0),
                         inv_freq, group_size, softmax_scale, return_lse, kg=kg)


def fused_jetlong_decode_cache_stripe(query_base, query_group, key_stripe, value_stripe, *, boundary: int, inv_freq,
                                      group_size: int, softmax_scale=None, return_lse: bool = False, exchange=None):
    """Decode when every rank holds only its block-cyclic stripe of the base-rotated cache, as the
    token-sharded prefill leaves it: key_stripe / value_stripe (B,Hk,S_loc,D), local row i at position
    rank*blk + (i // blk) * world*blk + i % blk.  Local rows below `boundary` are the far class
    (regrouped in-kernel at their true positions), the rest the near class; partial (O, LSE) pairs
    are all-gathered and merged, so every rank returns the full (B,1,H,D) result."""
    sh = _SHARD
    if sh is None:
        raise RuntimeError("fused_jetlong_decode_cache_stripe needs configure_sequence_sharding(...) first")
    kc, vc = key_stripe.transpose(1, 2), value_stripe.transpose(1, 2)
    n_far = min(sh.n_owned(int(boundary)), kc.shape[1])
    B, _, H, D = query_base.shape

    def part(out, lse):
        segs = []
        if n_far > 0:
            segs.append(ops.KvSegment(kc[:, :n_far], vc[:, :n_far], q_class=1, rotate=True, pos0=sh.rank * sh.block,
                                      pos_block=sh.block, pos_block_stride=sh.world * sh.block))
        if n_far < kc.shape[1]:
            segs.append(ops.KvSegment(kc[:, n_far:], vc[:, n_far:], q_class=0))
        if not segs:                       # this rank owns no key yet: an empty partial
            out = torch.zeros_like(query_base) if out is None else out.zero_()
            lse = (torch.full((B, H, 1), float("-inf"), device=query_base.device) if lse is None
                   else lse.fill_(float("-inf")))
            return out, lse
        return ops.decode_segments([query_base, query_group], segs, inv_freq=inv_freq, group_size=int(group_size),
                                   softmax_scale=softmax_scale, out=out, lse=lse)

    return _sharded_decode(part, sh, query_base, return_lse, exchange)


def fused_jetlong_decode_step(query_base, query_group, key_rows, value_rows, *, step, inv_freq, group_size: int,
                              softmax_scale=None, key_group_rows=None, exchange_slot=None):
    """Decode whose token-dependent facts come from device memory (ops.StepState), so the launch can sit in
    a CUDA graph that is replayed for every new token.  key_rows / value_rows: this rank's WHOLE
    (B, capacity, Hk, D) cache buffers; the far class is rows [0, n_far) (regrouped in-kernel when
    group_size > 1, or read as stored from key_group_rows when that regrouped copy is given), the near class
    rows [n_far, n_far + n_near), both read from `step`.  With a sharded
    step the partial (O, LSE) pairs are all-gathered and merged as in fused_jetlong_decode_cache_stripe."""
    sh = step.shard if step.shard is not None and step.shard.world > 1 else None
    geo = dict(pos0=sh.rank * sh.block, pos_block=sh.block, pos_block_stride=sh.world * sh.block) if sh is not None else {}
    if key_group_rows is not None and int(group_size) > 1:
        far = ops.KvSegment(key_group_rows, value_rows, q_class=1, len_dev=step.far_lens)
    else:
        far = ops.KvSegment(key_rows, value_rows, q_class=1, rotate=int(group_size) > 1, len_dev=step.far_lens, **geo)
    segs = [far, ops.KvSegment(key_rows, value_rows, q_class=0, len_dev=step.near_lens, row0_dev=step.n_far)]
    B, _, H, D = query_base.shape
    run = lambda out, lse: ops.decode_segments([query_base, query_group], segs, inv_freq=inv_freq,
                                               group_size=int(group_size), softmax_scale=softmax_scale, out=out, lse=lse)
    if sh is None:
        return run(None, None)[0]
    ex = step.peer_exchange(B, H, D) if exchange_slot is not None else None
    if ex is not None:
        part_o, part_lse = run(None, None)
        return ops.peer_merge(part_o, part_lse, ex, epoch_base=step.steps, epoch_stride=int(exchange_slot[1]),
                              epoch_offset=int(exchange_slot[0]) + 1)
    buf = _partial_buffer(sh, (B, 1, H, D), (B, H, 1), query_base.dtype, query_base.device)
    out, _ = sharded_attention(run, ops.merge_partials, sh, buf)
    return out


# ---------------------------------------------------------------------------------------------------
# jetlong_freq: same band map, far class rotated per frequency by delta_inv_freq, softmax with a temperature
# ---------------------------------------------------------------------------------------------------

_NO_GROUPING = 1 << 30      # floor(p / G) = 0 for every position: the in-kernel regroup angle becomes -p * inv_freq


def fused_jetlong_freq_prefill(query_base, key_base, value, *, delta_inv_freq, attn_scale: float, seqstart_q: int,
                               window_size_left: int):
    """PATH 2 of the reference's jetlong_freq attention (modeling_qwen3_jetlong_freq.py:380-443) in one
    kernel pass instead of three flash-attn calls and a subtractive merge: base scores where
    0 <= pq - pk <= w_0, corrected scores elsewhere, one softmax with scale attn_scale.
    query_base (B,H,S,D) / key_base, value (B,Hk,Skv,D): base-rotated views, keys from position 0.
    Returns (B,S,H,D).  (Queries at positions <= w_0 have no far keys, so their corrected operand is never
    read; it is formed at pq - w_0 without the reference's clamp at 0.)"""
    t = lambda x: x.transpose(1, 2)
    w_0 = int(window_size_left)
    like = lambda x: torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device)   # operands share strides
    q_dist = ops.rope_rotate(t(query_base), delta_inv_freq, pos0=int(seqstart_q), add=-w_0, out=like(t(query_base)))
    k_yarn = ops.rope_rotate(t(key_base), delta_inv_freq, pos0=0, out=like(t(key_base)))
    return ops.posmap_prefill([t(query_base), q_dist], [t(key_base), k_yarn], t(value), pmap=ops.PositionMap.jetlong(w_0),
                              q_pos0=int(seqstart_q), softmax_scale=float(attn_scale), return_lse=False)


def fused_jetlong_freq_decode(query_base, key_cache, value_cache, *, delta_inv_freq, attn_scale: float, max_q_pos: int,
                              window_size_left: int, return_lse: bool = False):
    """PATH 3 (modeling_qwen3_jetlong_freq.py:445-503) straight off the base-rotated (B,Hk,S,D) cache:
    keys [0, boundary) are corrected inside the kernel while they stream (angle p * delta_inv_freq),
    keys [boundary, S) are scored as stored; boundary = max(max_q_pos - w_0, 0).  query_base (B,1,H,D)."""
    boundary = max(int(max_q_pos) - int(window_size_left), 0)
    kc, vc = key_cache.transpose(1, 2), value_cache.transpose(1, 2)
    q_dist = ops.rope_rotate(query_base, delta_inv_freq, pos0=boundary) if boundary > 0 else query_base
    segs = []
    if boundary > 0:
        segs.append(ops.KvSegment(kc[:, :boundary], vc[:, :boundary], q_class=1, rotate=True, pos0=0))
    if boundary < kc.shape[1]:
        segs.append(ops.KvSegment(kc[:, boundary:], vc[:, boundary:], q_class=0))
    neg = -delta_inv_freq.to(device=query_base.device, dtype=torch.float32)
    return ops.decode_segments([query_base, q_dist], segs, inv_freq=neg, group_size=_NO_GROUPING,
                               softmax_scale=float(attn_scale), return_lse=return_lse)


def _decode_range(query_base, query_group, kc, vc, b, pos0, inv_freq, group_size, softmax_scale, return_lse,
                  out=None, lse=None, kg=None, allow_empty=False):
    """Decode over rows of a (B,S,Hk,D) cache view whose row 0 has absolute position pos0; rows < b are far."""
    b = max(0, min(b, kc.shape[1]))
    segs = []
    if b > 0 and kg is not None:
        segs.append(ops.KvSegment(kg[:, :b], vc[:, :b], q_class=1))
    elif b > 0:
        segs.append(ops.KvSegment(kc[:, :b], vc[:, :b], q_class=1, rotate=True, pos0=int(pos0)))
    if b < kc.shape[1]:
        segs.append(ops.KvSegment(kc[:, b:], vc[:, b:], q_class=0))
    if not segs:
        if not allow_empty:
            raise RuntimeError("JetLong backend 'fused' got an empty key range")
        # a rank of a sharded call that owns no key still has to reach the exchange: an empty partial (0, -inf)
        B, _, H, _ = query_base.shape
        out = torch.zeros_like(query_base) if out is None else out.zero_()
        lse = (torch.full((B, H, 1), float("-inf"), device=query_base.device) if lse is None else lse.fill_(float("-inf")))
        return (out, lse) if return_lse else out
    return ops.decode_segments([query_base, query_group], segs, inv_freq=inv_freq, group_size=int(group_size),
                               softmax_scale=softmax_scale, return_lse=return_lse, out=out, lse=lse)

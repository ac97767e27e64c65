"""One CUDA graph per decoded token.

The reference's decode step cannot be captured: every layer reads positions back to the host
(modeling_qwen3_jetlong_fused.py:145, :342, :406) and HF's DynamicCache reallocates.  Here the cache is
preallocated (kv_cache.BifocalKVCache), the position / cache row / class lengths of the token live in
device memory (jetlong_ops.StepState, advanced by the graph's first node) and every kernel launch has
token-independent host arguments, so the whole step — embedding, 36 layers, lm_head, greedy argmax, and
with a sharded cache the NCCL all-gathers and the token broadcast — is captured once per group size G
and replayed.  G = ceil(L / w) changes only every w tokens; a new graph is captured when it does.
"""
from __future__ import annotations

import math

import torch

from . import jetlong_ops as ops
from .kv_cache import BifocalKVCache


class GraphedDecodeStep:
    def __init__(self, lm, cache: BifocalKVCache):
        if not isinstance(cache, BifocalKVCache):
            raise TypeError("GraphedDecodeStep needs a BifocalKVCache")
        rot = lm.model.rotary_emb
        self.lm, self.cache = lm, cache
        self.w, self.w_0 = int(rot.jetlong_w), int(rot.jetlong_w_0)
        first = cache.layers[0]
        self.batch = first.keys.shape[0]
        self.device = first.keys.device
        shard = cache.shard if cache.shard is not None and cache.shard.world > 1 else None
        self.shard = shard
        self.step = ops.StepState(self.batch, self.device, self.w_0, shard)
        self.token = torch.zeros(self.batch, 1, dtype=torch.long, device=self.device)
        self._graph, self._graph_group = None, None
        self._device_pos = None            # position the device-side state will describe after its next advance
        # the peer exchange's status word is mirrored into pinned host memory by the graph's last node, so a
        # wait that gave up is noticed at the next call without a synchronisation
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()

    def _body(self, group: int) -> None:
        self.step.advance()
        hidden = self.lm.model.decode_step(self.token, self.cache, self.step, group)
        nxt = self.lm.lm_head(hidden[:, -1:, :]).argmax(-1)
        if self.shard is not None:        # ranks compute the same logits; one source keeps them in lock-step regardless
            import torch.distributed as dist
            src = dist.get_global_rank(self.shard.group, 0) if self.shard.group is not None else 0
            dist.broadcast(nxt, src=src, group=self.shard.group)
        self.token.copy_(nxt)
        peer = getattr(self.step, "_peer", None)
        if peer:
            self._status_host.copy_(peer.status, non_blocking=True)

    def check(self) -> None:
        """Raise if a bounded wait of the peer exchange gave up in a replay that has completed (no synchronisation:
        reads the pinned mirror; `ops.check_status()` is the synchronising form)."""
        if int(self._status_host[0]) != 0:
            raise RuntimeError("jl_peer_merge gave up waiting for another rank during a decode step; the tokens "
                               "produced since are invalid")

    def _refresh_group_keys(self, group: int, pos: int) -> None:
        """With a regrouped far-key cache: regroup every row that is far for the token at `pos` with this G
        (one pass per layer; afterwards every step adds the one row that may have crossed the boundary)."""
        if group <= 1 or self.cache.layers[0].group_keys is None:
            return
        sh = self.shard
        boundary = max(pos - self.w_0, 0)
        n_far = sh.n_owned(boundary) if sh is not None else boundary
        if n_far <= 0:
            return
        geo = dict(pos0=sh.rank * sh.block, pos_block=sh.block, pos_block_stride=sh.world * sh.block) if sh is not None else {}
        inv_freq = self.lm.model.rotary_emb.inv_freq
        for layer in self.cache.layers:
            ops.rope_regroup(layer.keys[:, :n_far], inv_freq, group_size=group, out=layer.group_keys[:, :n_far], **geo)

    def _capture(self, group: int, pos: int) -> None:
        self._refresh_group_keys(group, pos)
        keep = self.token.clone()
        cur = torch.cuda.current_stream(self.device)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):     # one real run first: library handles, workspaces and NCCL set-up
            self.step.set_next_position(pos)
            self._body(group)
        cur.wait_stream(side)
        self.token.copy_(keep)
        self.step.set_next_position(pos)
        torch.cuda.synchronize(self.device)
        self._graph = None                 # release the previous graph's memory before capturing the next
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._body(group)
        self._graph, self._graph_group, self._device_pos = graph, group, pos
        if self.shard is not None:
            # capture takes a different time on every rank; line the ranks up again so that the first replay's
            # bounded waits only have to cover kernel-time skew
            import torch.distributed as dist
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.shard.group)

    @torch.no_grad()
    def __call__(self, token=None) -> torch.Tensor:
        """Feed `token` (B,1) — by default the token this object produced last — and return the next greedy
        token.  The result is the object's static buffer: clone it to keep it past the next call."""
        self.check()
        pos = self.cache.get_seq_length()
        group = max(1, math.ceil((pos + 1) / self.w))
        if token is not None:
            self.token.copy_(token)
        if self._graph is None or self._graph_group != group:
            self._capture(group, pos)
        elif self._device_pos != pos:      # the cache moved without us (eager steps, reset): re-seed the device state
            self.step.set_next_position(pos)
            self._refresh_group_keys(group, pos)
        self._graph.replay()
        for layer in self.cache.layers:
            layer.commit(1)
        self._device_pos = pos + 1
        return self.token

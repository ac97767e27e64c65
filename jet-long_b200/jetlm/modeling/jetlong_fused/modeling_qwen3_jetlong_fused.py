"""Qwen3 with JetLong bifocal attention on the B200 kernels — the `jetlong_fused` method surface.

Same class names, config keys (`config.jetlong = {"w", "w_0", ...}`), parameter names and
`auto_map` target as the reference's jetlm/modeling/jetlong_fused/modeling_qwen3_jetlong_fused.py,
so a `*-jetlong_fused` model directory loads unchanged.  What differs is below the surface:

  * within the pretrained window (L <= w) attention is stock Qwen3 (reference :299-320);
  * beyond it, the extended prefill / decode paths (reference :322-461) keep the reference's
    position semantics — exact RoPE for 0 <= q-k <= w_0, positions floor(p/G) beyond, with
    G = ceil(L/w) recomputed per forward call — but RoPE, regrouping and attention run in the
    sm_100a kernels: fused fp32 rotation passes instead of ~10 elementwise torch kernels, one
    single-pass bifocal attention kernel instead of packed-2S FA4 + merge, and a decode kernel that
    regroups the far keys while it streams the cache instead of re-rotating the whole distant
    cache on the host side every token;
  * no per-layer host synchronisation: positions come from the cache length on the host.

Runs under transformers >= 5.5 (layer types read from config, no reliance on cache_position).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
from torch import nn

from transformers.cache_utils import Cache, DynamicCache
from transformers.generation import GenerationMixin
from transformers.masking_utils import create_causal_mask, create_sliding_window_causal_mask
from transformers.modeling_outputs import BaseModelOutputWithPast, CausalLMOutputWithPast
from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
from transformers.models.qwen3.configuration_qwen3 import Qwen3Config
from transformers.models.qwen3.modeling_qwen3 import (
    Qwen3DecoderLayer,
    Qwen3PreTrainedModel,
    Qwen3RMSNorm,
    Qwen3RotaryEmbedding,
    apply_rotary_pos_emb,
    eager_attention_forward,
)
from transformers.utils import can_return_tuple
from transformers.utils.generic import merge_with_config_defaults
from transformers.utils.output_capturing import capture_outputs


def _jetlong_cfg(config) -> Optional[dict]:
    cfg = getattr(config, "jetlong", None)
    if cfg is None and hasattr(config, "to_dict"):
        cfg = config.to_dict().get("jetlong", None)
    return cfg


@dataclass
class BifocalPlan:
    """Host-side facts about one extended forward call, shared by all layers."""
    group_size: int          # G = ceil(L_curr / w)
    q_pos0: int              # absolute position of the first query token
    max_q_pos: int           # absolute position of the last query token
    has_any_pad: bool        # a left-padded batch
    token_shard: object = None   # SequenceShard when this rank holds a block-cyclic stripe of the KV cache
    replicated: bool = False     # sharded cache, but every rank runs all tokens of this call (decode)
    step: object = None          # ops.StepState: positions and cache rows come from device memory (graph replay)
    pads: Optional[list] = None  # left-padded batch: number of leading pad rows of every sample's cache


class Qwen3JetLongFusedRotaryEmbedding(Qwen3RotaryEmbedding):
    """Base RoPE tables plus, past the pretrained window, the dynamic group size.

    Returns (cos, sin) while L_curr = max position + 1 <= w, else
    (cos, sin, G, inv_freq, position_ids, plan) — the first five entries are the reference's
    extended tuple (:148-158); `plan` carries the same facts as host integers."""

    def __init__(self, config: Qwen3Config, device=None):
        super().__init__(config, device)
        cfg = _jetlong_cfg(config)
        self.jetlong_enabled = cfg is not None
        if self.jetlong_enabled:
            self.jetlong_w = int(cfg["w"])
            self.jetlong_w_0 = int(cfg["w_0"])

    @torch.no_grad()
    def forward(self, x, position_ids, max_position: Optional[int] = None, kv_len: Optional[int] = None,
                first_position: Optional[int] = None, token_shard=None, replicated: bool = False,
                kernels_within_window: bool = False):
        """kernels_within_window: return the extended tuple (with G = 1) inside the pretrained window too, so
        that the attention runs on the bifocal kernels there as well (both classes then score alike)."""
        cos, sin = super().forward(x, position_ids)
        if not self.jetlong_enabled:
            return cos, sin
        if max_position is None:
            max_position = int(position_ids.max().item())      # caller-supplied positions: read them back
        l_curr = max_position + 1
        if l_curr <= self.jetlong_w and not kernels_within_window:
            return cos, sin
        group = max(1, math.ceil(l_curr / self.jetlong_w))
        seq = position_ids.shape[-1]
        has_pad, pads = False, None
        if position_ids.shape[0] > 1 and kv_len is not None:
            pads = (kv_len - 1 - position_ids[:, -1]).tolist()       # the last token of sample b sits at kv_len-1-pad_b
            has_pad = any(n > 0 for n in pads)
        first = first_position if first_position is not None else max_position - seq + 1
        plan = BifocalPlan(group, first, max_position, has_pad, token_shard, replicated, None, pads if has_pad else None)
        return cos, sin, group, self.inv_freq.to(device=x.device, dtype=torch.float32), position_ids, plan


class Qwen3JetLongFusedAttention(nn.Module):
    """Qwen3 attention whose long-context branch is the bifocal kernel family."""

    def __init__(self, config: Qwen3Config, layer_idx: int):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.layer_type = config.layer_types[layer_idx] if hasattr(config, "layer_types") else None
        self.head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_kv_heads
        self.scaling = self.head_dim ** -0.5
        self.attention_dropout = config.attention_dropout
        self.is_causal = True
        bias = config.attention_bias
        self.q_proj = nn.Linear(config.hidden_size, self.num_heads * self.head_dim, bias=bias)
        self.k_proj = nn.Linear(config.hidden_size, self.num_kv_heads * self.head_dim, bias=bias)
        self.v_proj = nn.Linear(config.hidden_size, self.num_kv_heads * self.head_dim, bias=bias)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, config.hidden_size, bias=bias)
        self.q_norm = Qwen3RMSNorm(self.head_dim, eps=config.rms_norm_eps)
        self.k_norm = Qwen3RMSNorm(self.head_dim, eps=config.rms_norm_eps)
        self.sliding_window = config.sliding_window if self.layer_type == "sliding_attention" else None
        cfg = _jetlong_cfg(config)
        self.jetlong_enabled = cfg is not None
        if self.jetlong_enabled:
            self.jetlong_w = int(cfg["w"])
            self.jetlong_w_0 = int(cfg["w_0"])

    # -- stock Qwen3 attention (inside the pretrained window) --------------------------------------
    def _within_window(self, q, k, v, position_embeddings, attention_mask, past_key_values, out_shape, **kwargs):
        cos, sin = position_embeddings[:2]
        q, k, v = (t.transpose(1, 2) for t in (q, k, v))
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        if past_key_values is not None:
            k, v = past_key_values.update(k, v, self.layer_idx, {"sin": sin, "cos": cos})
        interface = ALL_ATTENTION_FUNCTIONS.get_interface(self.config._attn_implementation, eager_attention_forward)
        out, weights = interface(self, q, k, v, attention_mask,
                                 dropout=0.0 if not self.training else self.attention_dropout,
                                 scaling=self.scaling, sliding_window=self.sliding_window, **kwargs)
        return self.o_proj(out.reshape(*out_shape, -1).contiguous()), weights

    def forward(self, hidden_states, position_embeddings, attention_mask=None, past_key_values: Cache | None = None,
                cache_position=None, **kwargs):
        bsz, seq = hidden_states.shape[:2]
        out_shape = (bsz, seq)
        H, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        k = self.k_proj(hidden_states).view(bsz, seq, Hk, D)         # per-head RMSNorm is applied below
        v = self.v_proj(hidden_states).view(bsz, seq, Hk, D)
        plan0 = position_embeddings[5] if len(position_embeddings) > 5 else None
        if plan0 is not None and plan0.step is None and plan0.token_shard is not None and not plan0.replicated:
            # sequence-parallel prefill: the keys and values go first, so that their exchange between the ranks can
            # already run behind the query projection
            from jetlm.kernels import cute_jetlong_backend as backend
            from jetlm.kernels import jetlong_ops as ops
            make_q = lambda: self.q_proj(hidden_states).view(bsz, seq, H, D)
            return self._token_sharded(make_q, k, v, plan0, position_embeddings[2], position_embeddings[3], past_key_values,
                                       out_shape, backend, ops)
        q = self.q_proj(hidden_states).view(bsz, seq, H, D)

        if len(position_embeddings) < 4:
            return self._within_window(self.q_norm(q), self.k_norm(k), v, position_embeddings, attention_mask,
                                       past_key_values, out_shape, **kwargs)

        # ---- extended (bifocal) paths -------------------------------------------------------------
        from jetlm.kernels import cute_jetlong_backend as backend      # resolved per call: the plugin seam
        from jetlm.kernels import jetlong_ops as ops

        group, inv_freq = position_embeddings[2], position_embeddings[3]
        plan: BifocalPlan | None = position_embeddings[5] if len(position_embeddings) > 5 else None
        if plan is None:      # driven with the reference's 5-tuple: recover the host facts from the tensors
            pos = position_embeddings[4]
            mx = int(pos.max().item())
            plan = BifocalPlan(int(group), mx - seq + 1, mx, False)
        if self.training:
            raise RuntimeError("JetLong backend 'fused' is inference-only")
        w_0 = self.jetlong_w_0
        q_eps, k_eps = self.q_norm.variance_epsilon, self.k_norm.variance_epsilon

        if plan.step is not None:
            # decode step whose position, cache row and class lengths live on the device: two launches
            # (norm -> RoPE -> cache write, attention) with token-independent host arguments
            slot = past_key_values.layers[self.layer_idx]
            kg = slot.group_keys if group > 1 else None      # regrouped copies of the far rows, when the cache keeps them
            q_base, q_group = ops.decode_append(q, k, v, self.q_norm.weight, self.k_norm.weight, inv_freq,
                                                slot.keys, slot.values, plan.step, q_eps=q_eps, k_eps=k_eps,
                                                group_size=group, k_group_cache=kg)
            attn = backend.fused_jetlong_decode_step(q_base, q_group, slot.keys, slot.values, step=plan.step,
                                                     inv_freq=inv_freq, group_size=group, softmax_scale=self.scaling,
                                                     key_group_rows=kg,
                                                     exchange_slot=(self.layer_idx, self.config.num_hidden_layers))
            return self.o_proj(attn.reshape(*out_shape, -1)), None

        if plan.token_shard is not None:
            return self._token_sharded(q, k, v, plan, group, inv_freq, past_key_values, out_shape, backend, ops)

        from jetlm.kernels.kv_cache import BifocalKVCache
        slot = past_key_values.layers[self.layer_idx] if isinstance(past_key_values, BifocalKVCache) else None
        if slot is not None:
            seen = slot.get_seq_length()
        else:
            seen = past_key_values.get_seq_length(self.layer_idx) if past_key_values is not None else 0
        if plan.pads is not None and getattr(self.config, "jetlong_allow_left_padding", True):
            return self._extended_left_padded(q, k, v, plan, group, inv_freq, past_key_values, slot, seen, out_shape,
                                              backend, ops)
        regroup = group > 1          # G = 1 (inside the pretrained window): both classes score alike
        # q/k RMSNorm + base RoPE (+ regroup) in one fused pass each; K lands straight in its cache rows
        if regroup:
            q_base, q_group = ops.norm_rope(q, self.q_norm.weight, inv_freq, eps=q_eps, pos0=plan.q_pos0, group_size=group)
        else:
            q_base = q_group = ops.norm_rope(q, self.q_norm.weight, inv_freq, eps=q_eps, pos0=plan.q_pos0)
        if slot is not None:
            k_new, v_dst = slot.reserve(seq)                           # (B, seq, Hk, D) rows of the static cache
        else:
            k_new = torch.empty(bsz, Hk, seq, D, dtype=k.dtype, device=k.device).transpose(1, 2)
        k_group = None
        if seen == 0 and seq > 1 and regroup:      # no older keys: the regrouped keys of this call are all there is
            k_group = (past_key_values.group_scratch(seq) if slot is not None
                       else torch.empty(bsz, Hk, seq, D, dtype=k.dtype, device=k.device).transpose(1, 2))
            ops.norm_rope(k, self.k_norm.weight, inv_freq, eps=k_eps, pos0=plan.q_pos0, group_size=group,
                          out_base=k_new, out_group=k_group)
        else:
            ops.norm_rope(k, self.k_norm.weight, inv_freq, eps=k_eps, pos0=plan.q_pos0, out_base=k_new)
        if slot is not None:
            v_dst.copy_(v)
            slot.commit(seq)
            k_all, v_all = slot.key_rows(), slot.value_rows()         # (B, len, Hk, D) views
        elif past_key_values is not None:
            k_all, v_all = past_key_values.update(k_new.transpose(1, 2), v.transpose(1, 2), self.layer_idx, {})
            k_all, v_all = k_all.transpose(1, 2), v_all.transpose(1, 2)
        else:
            k_all, v_all = k_new, v
        kv_len = k_all.shape[1]

        if seq > 1:
            # prefill / chunked prefill: regroup every cached key once for this call's G, then one kernel
            if not regroup:
                k_group = k_all
            elif k_group is None:
                k_group = (past_key_values.group_scratch(kv_len) if slot is not None
                           else torch.empty(bsz, Hk, kv_len, D, dtype=k_all.dtype, device=k_all.device).transpose(1, 2))
                ops.rope_regroup(k_all, inv_freq, group_size=group, pos0=0, out=k_group)
            if k_all.stride() != k_group.stride():           # a cache that hands out non-dense views
                k_all = k_all.contiguous()
            attn = backend.fused_jetlong_prefill(
                q_base.transpose(1, 2), q_group.transpose(1, 2), k_all.transpose(1, 2), k_group.transpose(1, 2),
                v_all.transpose(1, 2), seqstart_q=kv_len - seq, window_size_left=w_0, softmax_scale=self.scaling,
                has_any_pad=plan.has_any_pad, training=self.training)
        else:
            boundary = max(plan.max_q_pos - w_0, 0)
            if boundary == 0 and regroup:
                raise RuntimeError(
                    f"jetlong_fused requires a non-empty distant decode region (decode context must exceed "
                    f"w_0={w_0}); use the 'jetlong' method for short contexts.")
            attn = backend.fused_jetlong_decode_cache(
                q_base, q_group, k_all.transpose(1, 2), v_all.transpose(1, 2), boundary=boundary, inv_freq=inv_freq,
                group_size=group, softmax_scale=self.scaling, has_any_pad=plan.has_any_pad, training=self.training)
        return self.o_proj(attn.reshape(*out_shape, -1)), None

    def _extended_left_padded(self, q, k, v, plan, group, inv_freq, past_key_values, slot, seen, out_shape, backend, ops):
        """Left-padded batch (the reference's fused backend rejects it, cute_jetlong_backend.py:57-58, :124-125;
        its non-fused method serves it through varlen attention, modeling_qwen3_jetlong.py:403-460).
        Sample b carries plan.pads[b] leading pad rows in the cache; its real tokens are positions 0, 1, ... .
        Every sample is attended on the row slices that skip its pads — views, no copies — with its own
        position origin, so the kernels see B unpadded sequences.  Pad rows produce zeros."""
        bsz, seq = out_shape
        H, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        w_0 = self.jetlong_w_0
        q_eps, k_eps = self.q_norm.variance_epsilon, self.k_norm.variance_epsilon
        regroup = group > 1
        pads = [int(n) for n in plan.pads]
        first = [min(max(n - seen, 0), seq) for n in pads]          # first real query row of this call, per sample
        q_base = torch.zeros(bsz, seq, H, D, dtype=q.dtype, device=q.device)
        q_group = torch.zeros_like(q_base) if regroup else q_base
        if slot is not None:
            k_new, v_dst = slot.reserve(seq)
        else:
            k_new = torch.zeros(bsz, Hk, seq, D, dtype=k.dtype, device=k.device).transpose(1, 2)
        for b, r0 in enumerate(first):
            if r0 >= seq:
                continue
            pos0 = seen + r0 - pads[b]
            kw = dict(group_size=group, out_group=q_group[b: b + 1, r0:]) if regroup else {}
            ops.norm_rope(q[b: b + 1, r0:], self.q_norm.weight, inv_freq, eps=q_eps, pos0=pos0,
                          out_base=q_base[b: b + 1, r0:], **kw)
            ops.norm_rope(k[b: b + 1, r0:], self.k_norm.weight, inv_freq, eps=k_eps, pos0=pos0,
                          out_base=k_new[b: b + 1, r0:])
        if slot is not None:
            v_dst.copy_(v)
            slot.commit(seq)
            k_all, v_all = slot.key_rows(), slot.value_rows()
        elif past_key_values is not None:
            k_all, v_all = past_key_values.update(k_new.transpose(1, 2), v.transpose(1, 2), self.layer_idx, {})
            k_all, v_all = k_all.transpose(1, 2), v_all.transpose(1, 2)
        else:
            k_all, v_all = k_new, v
        kv_len = k_all.shape[1]
        attn = torch.zeros(bsz, seq, H, D, dtype=q.dtype, device=q.device)
        pmap = ops.PositionMap.jetlong(w_0)
        for b, r0 in enumerate(first):
            if r0 >= seq:
                continue
            kb, vb = k_all[b: b + 1, pads[b]:], v_all[b: b + 1, pads[b]:]
            qb, qg = q_base[b: b + 1, r0:], q_group[b: b + 1, r0:]
            if seq > 1:
                kg = kb
                if regroup:
                    kg = torch.empty_strided(kb.shape, kb.stride(), dtype=kb.dtype, device=kb.device)
                    ops.rope_regroup(kb, inv_freq, group_size=group, pos0=0, out=kg)
                out_b = ops.posmap_prefill([qb, qg], [kb, kg], vb, pmap=pmap, q_pos0=seen + r0 - pads[b],
                                           softmax_scale=self.scaling, return_lse=False)
            else:
                boundary = max(kv_len - 1 - pads[b] - w_0, 0)
                out_b = backend.fused_jetlong_decode_cache(
                    qb, qg, kb.transpose(1, 2), vb.transpose(1, 2), boundary=boundary, inv_freq=inv_freq,
                    group_size=group, softmax_scale=self.scaling, has_any_pad=False, training=self.training)
            attn[b: b + 1, r0:] = out_b
        return self.o_proj(attn.reshape(bsz, seq, -1)), None

    def _token_sharded(self, q, k, v, plan, group, inv_freq, past_key_values, out_shape, backend, ops):
        """Sequence-parallel attention over a cache of which this rank keeps a block-cyclic stripe.
        Prefill chunk (plan.replicated False): this rank ran the projections for its stripe of the chunk
        only; the attention exchanges Q and partial (O, LSE) between ranks.  Decode (plan.replicated True):
        every rank ran the one new token; its key and value are stored by the rank that owns the position,
        every rank attends the query to its stripe and the partials are all-gathered and merged."""
        from jetlm.kernels.kv_cache import BifocalKVCache
        sh = plan.token_shard
        bsz, seq = out_shape
        Hk, D = self.num_kv_heads, self.head_dim
        slot = past_key_values.layers[self.layer_idx] if isinstance(past_key_values, BifocalKVCache) else None
        q_eps, k_eps = self.q_norm.variance_epsilon, self.k_norm.variance_epsilon

        if plan.replicated:
            if slot is None:
                raise RuntimeError("token-sharded decode needs a BifocalKVCache built with the same SequenceShard")
            if seq != 1:
                raise ValueError("token-sharded decode takes one token per call")
            if group > 1:
                q_base, q_group = ops.norm_rope(q, self.q_norm.weight, inv_freq, eps=q_eps, pos0=plan.q_pos0, group_size=group)
            else:
                q_base = q_group = ops.norm_rope(q, self.q_norm.weight, inv_freq, eps=q_eps, pos0=plan.q_pos0)
            k_dst, v_dst = slot.reserve(1)
            if k_dst.shape[1] == 1:                                   # this rank owns the new position
                ops.norm_rope(k, self.k_norm.weight, inv_freq, eps=k_eps, pos0=plan.q_pos0, out_base=k_dst)
                v_dst.copy_(v)
            slot.commit(1)
            attn = backend.fused_jetlong_decode_cache_stripe(
                q_base, q_group, slot.key_rows().transpose(1, 2), slot.value_rows().transpose(1, 2),
                boundary=max(plan.max_q_pos - self.jetlong_w_0, 0), inv_freq=inv_freq, group_size=group,
                softmax_scale=self.scaling)
            return self.o_proj(attn.reshape(bsz, seq, -1)), None

        geo = dict(pos_block=sh.block, pos_block_stride=sh.world * sh.block)
        pos0 = plan.q_pos0 + sh.rank * sh.block
        if slot is not None:
            k_new, v_dst = slot.reserve(seq * sh.world)
            if k_new.shape[1] != seq:
                raise RuntimeError("token-sharded prefill chunks must start on a multiple of world * block tokens")
        else:
            k_new = torch.empty(bsz, Hk, seq, D, dtype=k.dtype, device=k.device).transpose(1, 2)
        ops.norm_rope(k, self.k_norm.weight, inv_freq, eps=k_eps, pos0=pos0, out_base=k_new, **geo)
        if slot is not None:
            v_dst.copy_(v)
            slot.commit(seq * sh.world)
            k_all, v_all = slot.key_rows(), slot.value_rows()
        elif past_key_values is not None:
            k_all, v_all = past_key_values.update(k_new.transpose(1, 2), v.transpose(1, 2), self.layer_idx, {})
            k_all, v_all = k_all.transpose(1, 2), v_all.transpose(1, 2)
        else:
            k_all, v_all = k_new, v
        mode = backend.token_sharded_prefill_mode(sh.world, k_all.shape[1] * sh.world, seq * sh.world, self.num_heads, Hk)
        gather = backend.token_sharded_kv_gather_begin(k_all, v_all) if mode == "kv_gather" else None
        if callable(q):                  # prefill: the query projection runs while the K/V gather is in flight
            q = q()
        q_base = ops.norm_rope(q, self.q_norm.weight, inv_freq, eps=q_eps, pos0=pos0, **geo)
        k_group = None                   # the K/V-gather form regroups the gathered keys itself
        if mode == "q_exchange":
            if group > 1:
                k_group = (past_key_values.group_scratch(k_all.shape[1]) if slot is not None
                           else torch.empty(bsz, Hk, k_all.shape[1], D, dtype=k_all.dtype, device=k_all.device).transpose(1, 2))
                ops.rope_regroup(k_all, inv_freq, group_size=group, pos0=sh.rank * sh.block, out=k_group, **geo)
            else:
                k_group = k_all
        attn = backend.fused_jetlong_prefill_token_sharded(
            q_base, k_all, k_group, v_all, q_start=plan.q_pos0,
            inv_freq=inv_freq, group_size=group, window_size_left=self.jetlong_w_0, softmax_scale=self.scaling, mode=mode,
            gather=gather)
        return self.o_proj(attn.reshape(bsz, seq, -1)), None


class Qwen3JetLongFusedDecoderLayer(Qwen3DecoderLayer):
    def __init__(self, config: Qwen3Config, layer_idx: int):
        super().__init__(config, layer_idx)
        self.self_attn = Qwen3JetLongFusedAttention(config=config, layer_idx=layer_idx)
        self.attention_type = config.layer_types[layer_idx]

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_values: Cache | None = None,
                use_cache=False, position_embeddings=None, **kwargs):
        """Same dataflow as the stock layer; on a B200 in bf16 inference the two RMSNorms run as single fused
        passes (the second one folded with the residual add), with Qwen3RMSNorm's own roundings."""
        fused = (hidden_states.is_cuda and hidden_states.dtype == torch.bfloat16 and not self.training
                 and hidden_states.shape[-1] % 8 == 0 and hidden_states.shape[-1] <= 8192
                 and len(position_embeddings) >= 4)
        if not fused:
            return super().forward(hidden_states, attention_mask=attention_mask, position_ids=position_ids,
                                   past_key_values=past_key_values, use_cache=use_cache,
                                   position_embeddings=position_embeddings, **kwargs)
        from jetlm.kernels import jetlong_ops as ops
        residual = hidden_states.contiguous()
        h = ops.rmsnorm(residual, self.input_layernorm.weight, eps=self.input_layernorm.variance_epsilon)
        h, _ = self.self_attn(hidden_states=h, attention_mask=attention_mask, position_ids=position_ids,
                              past_key_values=past_key_values, use_cache=use_cache,
                              position_embeddings=position_embeddings, **kwargs)
        residual, h = ops.rmsnorm(h.contiguous(), self.post_attention_layernorm.weight,
                                  eps=self.post_attention_layernorm.variance_epsilon, residual=residual)
        mlp = self.mlp
        if self.self_attn.config.hidden_act == "silu" and mlp.intermediate_size % 8 == 0:
            h = mlp.down_proj(ops.silu_mul(mlp.gate_proj(h), mlp.up_proj(h)))       # one elementwise pass, not two
        else:
            h = mlp(h)
        return residual + h


class Qwen3JetLongFusedModel(Qwen3PreTrainedModel):
    def __init__(self, config: Qwen3Config):
        super().__init__(config)
        self.padding_idx = config.pad_token_id
        self.vocab_size = config.vocab_size
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, self.padding_idx)
        self.layers = nn.ModuleList(
            Qwen3JetLongFusedDecoderLayer(config, i) for i in range(config.num_hidden_layers))
        self.norm = Qwen3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.rotary_emb = Qwen3JetLongFusedRotaryEmbedding(config=config)
        self.gradient_checkpointing = False
        self.has_sliding_layers = "sliding_attention" in self.config.layer_types
        self.post_init()

    @merge_with_config_defaults
    @capture_outputs
    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values: Cache | None = None,
                inputs_embeds=None, use_cache=None, cache_position=None, **kwargs) -> BaseModelOutputWithPast:
        if (input_ids is None) ^ (inputs_embeds is not None):
            raise ValueError("You must specify exactly one of input_ids or inputs_embeds")
        from jetlm.kernels import cute_jetlong_backend as backend
        shard = backend.sequence_shard() if getattr(self, "token_sharded", False) else None
        if shard is not None:
            return self._forward_token_sharded(input_ids, past_key_values, use_cache, shard, **kwargs)
        if inputs_embeds is None:
            inputs_embeds = self.embed_tokens(input_ids)
        if use_cache and past_key_values is None:
            past_key_values = DynamicCache(config=self.config)
        seen = past_key_values.get_seq_length() if past_key_values is not None else 0
        seq = inputs_embeds.shape[1]
        host_max = None
        if position_ids is None:
            if cache_position is not None:
                position_ids = cache_position.unsqueeze(0)
            else:
                position_ids = (torch.arange(seq, device=inputs_embeds.device) + seen).unsqueeze(0)
                host_max = seen + seq - 1                     # known without touching the device
        hidden = inputs_embeds
        kww = bool(getattr(self, "kernels_within_window", False)) and hidden.is_cuda and not self.training
        position_embeddings = self.rotary_emb(hidden, position_ids, max_position=host_max, kv_len=seen + seq,
                                              kernels_within_window=kww)
        extended = len(position_embeddings) >= 4

        mask_map = attention_mask if isinstance(attention_mask, dict) else None
        if mask_map is None and not extended:                  # the bifocal kernels mask by position
            mk = dict(config=self.config, inputs_embeds=inputs_embeds, attention_mask=attention_mask,
                      past_key_values=past_key_values, position_ids=position_ids)
            mask_map = {"full_attention": create_causal_mask(**mk)}
            if self.has_sliding_layers:
                mask_map["sliding_attention"] = create_sliding_window_causal_mask(**mk)

        for i, layer in enumerate(self.layers[: self.config.num_hidden_layers]):
            hidden = layer(hidden,
                           attention_mask=None if extended else mask_map[self.config.layer_types[i]],
                           position_embeddings=position_embeddings, position_ids=position_ids,
                           past_key_values=past_key_values, use_cache=use_cache, **kwargs)
        hidden = self.norm(hidden)
        self._check_kernel_status(extended)
        return BaseModelOutputWithPast(last_hidden_state=hidden,
                                       past_key_values=past_key_values if use_cache else None)

    def _check_kernel_status(self, extended: bool) -> None:
        """With `model.check_kernel_status = True` (or JETLONG_CHECK_STATUS=1) every extended forward ends by
        reading the status words of the kernels' bounded waits and raises if one gave up.  Off by default: the
        read synchronises the device."""
        import os
        if extended and (getattr(self, "check_kernel_status", False) or os.environ.get("JETLONG_CHECK_STATUS") == "1"):
            from jetlm.kernels import jetlong_ops as ops
            ops.check_status()

    def decode_step(self, token, cache, step, group: int):
        """One-token forward with no host-side dependence on the position: `step` (ops.StepState) was advanced
        on the device for this token, `cache` is the BifocalKVCache the step was built for and `group` the
        group size G of this call.  Safe to capture in a CUDA graph.  Returns the final hidden state (B,1,hidden);
        the caller commits the token to the cache's host-side counters."""
        inv_freq = self.rotary_emb.inv_freq.to(device=token.device, dtype=torch.float32)
        plan = BifocalPlan(int(group), -1, -1, False, step.shard, True, step)
        position_embeddings = (None, None, int(group), inv_freq, None, plan)
        hidden = self.embed_tokens(token)
        for layer in self.layers[: self.config.num_hidden_layers]:
            hidden = layer(hidden, attention_mask=None, position_embeddings=position_embeddings,
                           position_ids=None, past_key_values=cache, use_cache=True)
        return self.norm(hidden)

    def _forward_token_sharded(self, input_ids, past_key_values, use_cache, shard, **kwargs) -> BaseModelOutputWithPast:
        """Sequence-parallel forward; `input_ids` is the whole (B, S) call on every rank.
        S a multiple of world * block (a prefill chunk): this rank embeds, projects and stores only its
        block-cyclic stripe of the tokens and returns the hidden states of that stripe, in stripe order.
        S = 1 (decode, needs a BifocalKVCache): every rank runs the token; the rank that owns its position
        stores its key and value; every rank returns the same hidden state."""
        from jetlm.kernels.kv_cache import BifocalKVCache
        if input_ids is None:
            raise ValueError("token-sharded forward takes input_ids")
        seq = input_ids.shape[1]
        replicated = seq == 1
        if not replicated and seq % (shard.world * shard.block) != 0:
            raise ValueError(f"token-sharded prefill needs a multiple of {shard.world * shard.block} tokens, got {seq}")
        if use_cache and past_key_values is None:
            past_key_values = DynamicCache(config=self.config)
        if isinstance(past_key_values, BifocalKVCache):
            seen = past_key_values.get_seq_length()
        else:       # a cache that only knows this rank's rows (whole stripes so far)
            seen = (past_key_values.get_seq_length() if past_key_values is not None else 0) * shard.world
        if replicated:
            hidden = self.embed_tokens(input_ids)
            position_ids = torch.full((1, 1), seen, dtype=torch.long, device=input_ids.device)
        else:
            rows = shard.owned_rows(seq).to(input_ids.device)
            hidden = self.embed_tokens(input_ids[:, rows])
            position_ids = (rows + seen).unsqueeze(0)
        position_embeddings = self.rotary_emb(hidden, position_ids, max_position=seen + seq - 1, kv_len=None,
                                              first_position=seen, token_shard=shard, replicated=replicated,
                                              kernels_within_window=True)
        for layer in self.layers[: self.config.num_hidden_layers]:
            hidden = layer(hidden, attention_mask=None, position_embeddings=position_embeddings,
                           position_ids=position_ids, past_key_values=past_key_values, use_cache=use_cache, **kwargs)
        hidden = self.norm(hidden)
        self._check_kernel_status(True)
        return BaseModelOutputWithPast(last_hidden_state=hidden, past_key_values=past_key_values if use_cache else None)


class Qwen3JetLongFusedForCausalLM(Qwen3PreTrainedModel, GenerationMixin):
    _tied_weights_keys = {"lm_head.weight": "model.embed_tokens.weight"}
    _tp_plan = {"lm_head": "colwise_gather_output"}
    _pp_plan = {"lm_head": (["hidden_states"], ["logits"])}

    def __init__(self, config):
        super().__init__(config)
        self.model = Qwen3JetLongFusedModel(config)
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def set_input_embeddings(self, value):
        self.model.embed_tokens = value

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, new_embeddings):
        self.lm_head = new_embeddings

    def set_decoder(self, decoder):
        self.model = decoder

    def get_decoder(self):
        return self.model

    @can_return_tuple
    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values: Cache | None = None,
                inputs_embeds=None, labels=None, use_cache=None, cache_position=None, logits_to_keep=0,
                **kwargs) -> CausalLMOutputWithPast:
        outputs: BaseModelOutputWithPast = self.model(
            input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
            past_key_values=past_key_values, inputs_embeds=inputs_embeds, use_cache=use_cache,
            cache_position=cache_position, **kwargs)
        hidden = outputs.last_hidden_state
        keep = slice(-logits_to_keep, None) if isinstance(logits_to_keep, int) else logits_to_keep
        logits = self.lm_head(hidden[:, keep, :])
        loss = None
        if labels is not None:
            loss = self.loss_function(logits=logits, labels=labels, vocab_size=self.config.vocab_size, **kwargs)
        return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=outputs.past_key_values,
                                      hidden_states=outputs.hidden_states, attentions=outputs.attentions)


    @torch.no_grad()
    def generate_long(self, input_ids, max_new_tokens: int, chunk_tokens: int = 32768, past_key_values=None,
                      cuda_graph: bool = False):
        """Greedy continuation of a long prompt: chunked prefill into a preallocated BifocalKVCache, then
        one-token steps on the same cache.  G is recomputed per call from the length reached so far, as in
        the reference (:145-158), so the result depends on the chunk schedule exactly as the reference's does.

        With `model.token_sharded = True` and sequence sharding configured, every rank calls this with the
        same arguments: each keeps a block-cyclic stripe of the cache (the prompt length and chunk_tokens
        must then be multiples of world * block) and all ranks return the same tokens.
        cuda_graph: replay one captured graph per decoded token (jetlm.kernels.decode_graph) instead of
        launching the step from Python.  Returns (B, max_new_tokens) token ids."""
        import torch.distributed as dist
        from jetlm.kernels import cute_jetlong_backend as backend
        from jetlm.kernels.kv_cache import BifocalKVCache
        shard = backend.sequence_shard() if getattr(self.model, "token_sharded", False) else None
        bsz, n_prompt = input_ids.shape
        if past_key_values is None:
            past_key_values = BifocalKVCache(self.config, n_prompt + max_new_tokens, batch=bsz, device=input_ids.device,
                                             dtype=self.lm_head.weight.dtype, shard=shard)

        def rank_of(r):
            return dist.get_global_rank(shard.group, r) if shard.group is not None else r

        hidden = None
        for lo in range(0, n_prompt, chunk_tokens):
            hidden = self.model(input_ids=input_ids[:, lo: lo + chunk_tokens], past_key_values=past_key_values,
                                use_cache=True).last_hidden_state
        token = self.lm_head(hidden[:, -1:, :]).argmax(-1)               # (B, 1)
        if shard is not None:        # the prompt's last block lives on the last rank
            dist.broadcast(token, src=rank_of(shard.world - 1), group=shard.group)
        out = [token]
        if cuda_graph and max_new_tokens > 1:
            from jetlm.kernels.decode_graph import GraphedDecodeStep
            step = GraphedDecodeStep(self, past_key_values)
            for i in range(max_new_tokens - 1):
                out.append(step(token if i == 0 else None).clone())
            return torch.cat(out, dim=1)
        for _ in range(max_new_tokens - 1):
            hidden = self.model(input_ids=token, past_key_values=past_key_values, use_cache=True).last_hidden_state
            token = self.lm_head(hidden[:, -1:, :]).argmax(-1)
            if shard is not None:    # ranks compute the same logits; one source keeps them in lock-step regardless
                dist.broadcast(token, src=rank_of(0), group=shard.group)
            out.append(token)
        return torch.cat(out, dim=1)


__all__ = ["Qwen3JetLongFusedForCausalLM", "Qwen3JetLongFusedModel", "Qwen3JetLongFusedRotaryEmbedding"]

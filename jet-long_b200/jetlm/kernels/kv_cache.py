"""Preallocated, shard-aware KV cache for the bifocal attention kernels.

The reference keeps its keys and values in HF's `DynamicCache`, which concatenates on every update
(modeling_qwen3_jetlong_fused.py:292-294, :335-340): at a 128K context every decoded token copies the
whole cache of every layer.  Here each layer owns one (B, capacity, Hk, D) buffer per operand, laid
out token-major so that
  * the fused norm -> RoPE pass (`jl_norm_rope`) writes new keys straight into their rows,
  * the kernels read the rows in place through strided (B, S, Hk, D) views,
  * appending never moves old rows.
With a `SequenceShard` the buffer holds only the rows of this rank's block-cyclic stripe: local row i
is the token at position rank*block + (i // block) * world*block + i % block, which is the geometry
`jl_prefill` (k_pos0 / k_block / k_block_stride) and `jl_decode` segments (pos_block / pos_block_stride)
understand.  A token is stored by exactly one rank.

The class is a `transformers.Cache`, so HF code paths (mask sizes, `get_seq_length`, `update` from the
stock attention inside the pretrained window) keep working on it.
"""
from __future__ import annotations

from typing import Optional

import torch
from transformers.cache_utils import Cache, CacheLayerMixin

from .sequence_parallel import SequenceShard


class BifocalStaticLayer(CacheLayerMixin):
    is_sliding = False
    is_compileable = False

    def __init__(self, batch: int, capacity: int, kv_heads: int, head_dim: int, dtype, device,
                 shard: Optional[SequenceShard] = None, regrouped_far_keys: bool = False):
        super().__init__()
        self.shard = shard
        self.capacity = int(capacity)                 # rows this rank can hold
        self.keys = torch.empty(batch, self.capacity, kv_heads, head_dim, dtype=dtype, device=device)
        self.values = torch.empty_like(self.keys)
        # optional second key buffer: regrouped copies of the far rows, maintained by the graph decode driver
        self.group_keys = torch.empty_like(self.keys) if regrouped_far_keys else None
        self.dtype, self.device = dtype, self.keys.device
        self.is_initialized = True
        self.tokens = 0                                # tokens seen by this layer (all ranks)
        self.rows = 0                                  # rows held by this rank

    # ---- geometry ----
    def _owned_below(self, n_tokens: int) -> int:
        return n_tokens if self.shard is None else self.shard.n_owned(n_tokens)

    def reserve(self, n_tokens: int):
        """Views (B, n_own, Hk, D) of the rows this rank stores for the next n_tokens tokens (n_own may be 0).
        The caller fills them and then calls commit(n_tokens)."""
        n_own = self._owned_below(self.tokens + n_tokens) - self.rows
        if self.rows + n_own > self.capacity:
            raise RuntimeError(f"KV cache capacity exceeded: {self.rows + n_own} rows > {self.capacity}")
        return self.keys[:, self.rows: self.rows + n_own], self.values[:, self.rows: self.rows + n_own]

    def commit(self, n_tokens: int) -> None:
        self.tokens += n_tokens
        self.rows = self._owned_below(self.tokens)

    def key_rows(self) -> torch.Tensor:
        return self.keys[:, : self.rows]

    def value_rows(self) -> torch.Tensor:
        return self.values[:, : self.rows]

    # ---- transformers.CacheLayerMixin ----
    def lazy_initialization(self, key_states, value_states) -> None:
        return None

    def update(self, key_states, value_states, *args, **kwargs):
        """HF contract: (B, Hk, S, D) in, the (B, Hk, len, D) views of everything cached out."""
        if self.shard is not None and self.shard.world > 1:
            raise RuntimeError("a sharded BifocalKVCache is filled through reserve()/commit() by the bifocal attention")
        n = key_states.shape[2]
        k_dst, v_dst = self.reserve(n)
        k_dst.copy_(key_states.transpose(1, 2))
        v_dst.copy_(value_states.transpose(1, 2))
        self.commit(n)
        return self.key_rows().transpose(1, 2), self.value_rows().transpose(1, 2)

    def get_seq_length(self) -> int:
        return self.tokens

    def get_mask_sizes(self, query_length: int):
        return self.tokens + query_length, 0

    def get_max_cache_shape(self) -> int:
        return self.capacity * (self.shard.world if self.shard is not None else 1)

    def reset(self) -> None:
        self.tokens = 0
        self.rows = 0


class BifocalKVCache(Cache):
    """One BifocalStaticLayer per decoder layer plus one shared scratch buffer of a layer's size, which
    holds the regrouped keys of the layer being attended during a (chunked) prefill call.
    regrouped_far_keys=True adds a second key buffer per layer (+50 % cache memory): the CUDA-graph decode
    driver keeps regrouped copies of the far rows there, so a decode step streams the far keys as stored
    instead of rotating them for every token (the reference regroups the whole distant cache per token,
    modeling_qwen3_jetlong_fused.py:428-440)."""

    def __init__(self, config, max_tokens: int, batch: int = 1, device=None, dtype=torch.bfloat16,
                 shard: Optional[SequenceShard] = None, regrouped_far_keys: bool = False):
        head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        world = shard.world if shard is not None else 1
        block = shard.block if shard is not None else 128
        per_rank = -(-int(max_tokens) // (world * block)) * block        # whole blocks, so every stripe fits
        layers = [BifocalStaticLayer(batch, per_rank, config.num_key_value_heads, head_dim, dtype, device, shard,
                                     regrouped_far_keys)
                  for _ in range(config.num_hidden_layers)]
        super().__init__(layers=layers)
        self.shard = shard
        self.max_tokens = per_rank * world
        self._scratch = torch.empty_like(layers[0].keys)

    def group_scratch(self, rows: int) -> torch.Tensor:
        """(B, rows, Hk, D) view with the strides of a layer's key rows."""
        return self._scratch[:, :rows]

    def reset(self) -> None:
        for layer in self.layers:
            layer.reset()

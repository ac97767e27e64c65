/*
 * jetlong_b200 — C ABI of the B200 (sm_100a) bifocal-RoPE attention kernels.
 *
 * This is the native boundary a Jet-Long maintainer binds instead of the reference's
 * JIT-compiled pybind module and CuTe-DSL launchers.  Plain pointers, sizes and strides only;
 * no torch types.  Every tensor is caller-owned device memory; the library never allocates.
 * All work is enqueued on the stream passed in; no call synchronises or reads device memory
 * on the host, so calls are CUDA-graph capturable.
 *
 * Element type of q/k/v/out is bf16 (JL_BF16) unless noted; lse is fp32.  Strides are in ELEMENTS.
 * The innermost (head_dim) dimension is always contiguous and head_dim must be 128.
 *
 * Reference interfaces replaced (paths inside the Jet-Long repository):
 *   jl_merge          jetlm/kernels/csrc/merge_fused.cpp:32-54  (merge2_bshd / merge2_bshd_out),
 *                     jetlm/kernels/csrc/merge_fused.cu:135-168, and the torch N-way merge
 *                     jetlm/kernels/cute_decode_sm90.py:199-240
 *   jl_prefill        jetlm/kernels/cute_prefill_sm90.py:114-230 (fa4_cute_prefill_sm90_jetlong_fused:
 *                     pack to 2S + block-sparse FA4 call + merge2_bshd + logaddexp)
 *   jl_decode         jetlm/kernels/cute_decode_sm90.py:2748-2799 (fa4_cute_decode_sm90_jetlong_fused)
 *                     and its launcher :2454-2745
 *   jl_decode_workspace_bytes   the module-level split-K workspace cache, cute_decode_sm90.py:165-196
 *   jl_rotate         the torch elementwise RoPE / regroup passes,
 *                     jetlm/modeling/jetlong_fused/modeling_qwen3_jetlong_fused.py:171-176, :209-226
 */
#ifndef JETLONG_B200_H_
#define JETLONG_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define JL_MAX_CLASSES 3
#define JL_MAX_SEGMENTS 4
#define JL_MAX_PARTS 16

/* Status codes returned by every entry point. */
enum {
  JL_OK = 0,
  JL_ERR_BAD_ARG = 1,        /* null pointer, negative size, misaligned pointer or stride        */
  JL_ERR_UNSUPPORTED = 2,    /* valid request outside what the kernels implement (e.g. head_dim) */
  JL_ERR_LAUNCH = 3,         /* the CUDA runtime refused the launch                              */
  JL_ERR_ARCH = 4,           /* current device is not sm_100                                     */
  JL_ERR_WORKSPACE = 5       /* workspace missing or smaller than jl_*_workspace_bytes           */
};

/* Library version (major*10000 + minor*100 + patch). */
int jl_version(void);
/* Static description of a status code. */
const char* jl_status_string(int status);
/* Detail message of the last failing call on this host thread ("" if none). */
const char* jl_last_error(void);

/* ---------------------------------------------------------------------------------------------
 * Position map: which (query operand, key operand) pair scores a (query, key) position pair.
 *
 * JL_MAP_BAND  (jetlong, self-extend): class 0 iff 0 <= pq - pk <= near_span, class 1 iff
 *              pq - pk > near_span.  jetlong: near_span = w_0 (w_0 + 1 near keys);
 *              self-extend: near_span = window_size - 1.
 * JL_MAP_CHUNK (dual chunk attention): class = min(pq / chunk - pk / chunk, 2)
 *              (0 intra, 1 successive, 2 inter).
 * Pairs with pk > pq are masked (causal).  Class c is scored as q[c] . k[c]; operands of
 * different classes may alias (DCA uses one key tensor for all three classes).
 * ------------------------------------------------------------------------------------------- */
enum { JL_MAP_BAND = 0, JL_MAP_CHUNK = 1 };

typedef struct {
  int32_t kind;        /* JL_MAP_BAND or JL_MAP_CHUNK */
  int32_t n_classes;   /* 2 for BAND, 3 for CHUNK     */
  int64_t near_span;   /* BAND                        */
  int64_t chunk;       /* CHUNK                       */
} jl_posmap;

/* ---------------------------------------------------------------------------------------------
 * jl_prefill — single-pass position-mapped causal attention for a block of Sq query tokens
 * against Skv keys.  One online softmax spans all classes; no packed 2S tensors, no separate
 * merge.  Key row j has absolute position k_pos0 + (j / k_block) * k_block_stride + (j % k_block):
 * a contiguous cache uses k_block <= 0; a block-cyclic shard of a sequence-parallel cache uses its
 * stripe geometry.  Query rows follow the same rule with q_pos0 / q_block / q_block_stride (a
 * contiguous block of queries uses q_block <= 0, i.e. row i is at q_pos0 + i; q_block must be a
 * multiple of 256 otherwise).
 *
 * q[c]: (B, Sq, H, D)   k[c], v: (B, Skv, Hk, D)   out: (B, Sq, H, D)   lse: (B, H, Sq) fp32.
 * lse may be NULL.  Rows that see no key produce a zero output row and lse = -inf.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  const void* q[JL_MAX_CLASSES];
  const void* k[JL_MAX_CLASSES];
  const void* v;
  void* out;
  float* lse;
  int64_t q_stride_b, q_stride_s, q_stride_h;
  int64_t k_stride_b, k_stride_s, k_stride_h;
  int64_t v_stride_b, v_stride_s, v_stride_h;
  int64_t o_stride_b, o_stride_s, o_stride_h;
  int32_t batch, seqlen_q, seqlen_k, heads, kv_heads, head_dim;
  int64_t q_pos0;
  int64_t k_pos0;
  int64_t k_block;          /* <= 0 means contiguous */
  int64_t k_block_stride;
  float softmax_scale;
  jl_posmap map;
  int32_t impl;             /* 0 = the tcgen05 kernel (one CTA per 256 query rows); 1 = the mma.sync kernel kept as an on-GPU
                               cross-check; 2 = the tcgen05 CTA-pair kernel (a cluster of two CTAs per 256 query rows,
                               cta_group::2 MMAs, every K / V tile split between the two), same results as impl 0.
                               impl 0 and 2 refuse (JL_ERR_UNSUPPORTED, never a silent change of kernel) a k_block that is
                               not a multiple of 128, a q_block that is not a multiple of 256, and more than two distinct
                               key tensors; impl 2 also refuses remap_far_in_kernel */
  int64_t q_block;          /* <= 0 means contiguous */
  int64_t q_block_stride;
  /* Far-field positions remapped INSIDE the kernel (band map, impl 0 only): with remap_far_in_kernel != 0 the far
   * class is formed from the class-0 operands, which must be base-rotated (position p): every query tile and
   * every key tile of the far phase is rotated in shared memory by (floor(p / group_size) - p) * inv_freq before
   * the tensor cores read it, so q[1] / k[1] are ignored (may be NULL) and no regrouped copy of Q or K exists in
   * HBM.  Replaces correction_rotate_per_sample on q and on the whole key cache,
   * modeling_qwen3_jetlong_fused.py:375-379; the reference's own in-kernel form of the idea is
   * apply_jetlong_k_transform_smem, cute_decode_sm90.py:931-966.  Slower than the pre-rotated operands (the
   * rotation is repeated by every CTA that visits a key tile), so the Python layer leaves it off by default. */
  int32_t remap_far_in_kernel;
  int32_t group_size;
  const float* inv_freq;    /* (head_dim/2,) fp32 device array; needed only with remap_far_in_kernel */
  /* Stripe batching (impl 0 and 2; no reference counterpart — the reference has no sequence parallelism): with
   * q_batch_wrap > 0, q[], out and lse hold q_batch_wrap batch elements (their batch strides apply), this launch
   * processes `batch` of them, element (q_batch_first + i) % q_batch_wrap for i = 0 .. batch - 1, the rows of element
   * e sit at positions q_pos0 + e * q_pos0_batch_step (+ the q_block rule), and ALL of them attend batch element 0 of
   * k[] and v.  One launch then covers the query stripes of several ranks against this rank's key stripe. */
  int32_t q_batch_first;
  int32_t q_batch_wrap;
  int64_t q_pos0_batch_step;
} jl_prefill_args;

int jl_prefill(const jl_prefill_args* args, void* cuda_stream);
/* Diagnostic (synchronises the device): 0 if no bounded wait inside the prefill kernel has given up on
 * the current device since the last call, non-zero otherwise (reading a raised status clears it).
 * A kernel whose wait gives up (1 s) drains and returns instead of hanging; its output, and that of
 * every prefill launched before the status is read, is invalid.  No reference counterpart. */
int jl_prefill_status(void);

/* ---------------------------------------------------------------------------------------------
 * jl_decode — split-KV attention of ONE query token per sequence over up to JL_MAX_SEGMENTS key
 * segments read in place (no slicing, padding or regrouping copies).  Segment s is scored with
 * query operand q[seg[s].q_class].  If seg[s].rotate != 0 the keys of that segment are rotated
 * in-kernel by (floor(p / group_size) - p) * inv_freq, p = seg[s].pos0 + row (or, for a block-cyclic
 * cache stripe, seg[s].pos0 + (row / pos_block) * pos_block_stride + row % pos_block), i.e. the far
 * class of the jetlong map is formed on the fly from a base-rotated cache.
 *
 * q[c]: (B, 1, H, D)   seg[s].k / .v: (B, len, Hk, D)   out: (B, 1, H, D)   lse: (B, H) fp32.
 * seg[s].len_dev, if not NULL, is an int32 device array (B,) of per-sequence valid lengths
 * (<= len).  With len_dev and row0_dev a launch whose host arguments never change (a CUDA-graph node)
 * follows a growing cache: see jl_step_advance.  workspace holds 16 KB of arrival counters followed by the
 * fp32 split partials; size it with jl_decode_workspace_bytes.  The splits of a (batch, kv head) are merged
 * by the last of their CTAs to finish (reference idea: the in-kernel split combine,
 * cute_decode_sm90.py:1769-1785), which it learns from those counters: the first 16 KB of a workspace must be
 * ZERO the first time it is used (cudaMemset once after allocating it); every launch leaves them zero, so
 * the same workspace can serve any later call, of any shape, on the same stream.  batch * kv_heads <= 4096.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  const void* k;
  const void* v;
  int64_t k_stride_b, k_stride_s, k_stride_h;
  int64_t v_stride_b, v_stride_s, v_stride_h;
  const int32_t* len_dev;
  int64_t pos0;
  int32_t len;
  int32_t q_class;
  int32_t rotate;
  int32_t reserved;
  int64_t pos_block;        /* <= 0 means contiguous positions; else a multiple of 8 */
  int64_t pos_block_stride;
  const int64_t* row0_dev;  /* optional device scalar: the segment starts at row *row0_dev of k / v (len and
                               len_dev count from there; positions are those of the shifted rows) */
} jl_kv_segment;

typedef struct {
  const void* q[JL_MAX_CLASSES];
  int64_t q_stride_b, q_stride_h;
  jl_kv_segment seg[JL_MAX_SEGMENTS];
  int32_t n_segments;
  int32_t batch, heads, kv_heads, head_dim;
  int32_t num_splits;       /* <= 0: chosen by the library to fill the GPU */
  float softmax_scale;
  const float* inv_freq;    /* (head_dim/2,) fp32 device array; needed only when a segment rotates */
  int32_t group_size;
  int32_t reserved;
  void* out;
  float* lse;               /* may be NULL */
  int64_t o_stride_b, o_stride_h;
  void* workspace;
  size_t workspace_bytes;
} jl_decode_args;

/* Bytes of workspace jl_decode needs for (batch, heads, head_dim) with at most max_splits splits
 * (max_splits <= 0: the library's own upper bound for automatic splitting). */
size_t jl_decode_workspace_bytes(int32_t batch, int32_t heads, int32_t head_dim, int32_t max_splits);
/* Number of splits jl_decode would pick for num_splits <= 0 when no segment rotates.  A call that regroups far keys
 * in-kernel (a segment with rotate != 0) with kv_heads a multiple of 8 and at most 8 query heads per kv head runs on a
 * differently gridded kernel (one CTA per key range over eight kv heads, which forms every rotation angle once instead
 * of once per kv head) and picks up to 148 / (batch * kv_heads / 8) splits: size a workspace that must serve both with
 * jl_decode_workspace_bytes(..., max_splits <= 0). */
int32_t jl_decode_auto_splits(int32_t batch, int32_t kv_heads, int64_t total_keys);
int jl_decode(const jl_decode_args* args, void* cuda_stream);

/* jl_decode_static — jl_decode for callers that cannot allocate device memory.  (No counterpart in
 * the reference, whose Python layer always allocates its split-K workspace with torch.)
 *
 * Who needs it: a server that gives its whole device-memory budget to one arena when it starts and
 * treats any later cudaMalloc as a bug (it may fail, and it can stall every stream on the device
 * while it runs), or a plug-in that is handed nothing but input and output pointers and has no
 * allocator of its own.  Such a caller has nowhere to get the split-KV workspace from, so this
 * variant keeps the partials in a fixed array that is part of the library image.
 *
 * Same arguments and results as jl_decode; args->workspace and args->workspace_bytes are ignored.
 * The library makes no allocation on this path.
 *   - Limit: 16 KB of counters plus the partials, batch * heads * splits * (head_dim + 1) * 4 bytes, must fit in
 *     jl_decode_static_scratch_bytes() (4 MiB; batch * heads * splits <= 8096).  Larger requests are
 *     refused with JL_ERR_WORKSPACE and a message naming both sizes; nothing is launched.
 *   - Cost: every GPU on which the library is loaded carries those 4 MiB until the process exits.
 *   - The first call on each device looks up the array's device address (one cheap runtime query, made
 *     with that device current).  Make that first call during start-up, before any stream capture
 *     begins.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left in it.
 *     The counters at its head start at zero (the array is zero when the library is loaded) and every
 *     launch puts them back; each launch writes every partial slot it later reads.  Two calls
 *     whose kernels may overlap on the GPU (different streams, no dependency between them) race on
 *     it; order them on one stream or with events, or give the overlapping ones jl_decode with
 *     workspaces of their own. */
int jl_decode_static(const jl_decode_args* args, void* cuda_stream);
size_t jl_decode_static_scratch_bytes(void);

/* ---------------------------------------------------------------------------------------------
 * jl_merge — N-way (O, LSE) merge of partial attention results over disjoint key sets:
 *   out = sum_p O_p e^{lse_p - m} / sum_p e^{lse_p - m},  lse = m + log sum_p e^{lse_p - m}.
 * o[p]: (B, S, H, D) contiguous, lse[p]: (B, H, S) fp32 contiguous.  lse_out may be NULL.
 * round_like_reference != 0 (n_parts == 2 only) reproduces the storage-dtype rounding after every
 * arithmetic step of the reference kernel (merge_fused.cu:100-111), including its 1e-7 clamp.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  const void* o[JL_MAX_PARTS];
  const float* lse[JL_MAX_PARTS];
  int32_t n_parts;
  int32_t batch, seqlen, heads, head_dim;
  int32_t round_like_reference;
  void* out;
  float* lse_out;
} jl_merge_args;

int jl_merge(const jl_merge_args* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------------
 * jl_rotate — rotate-half RoPE of x by an integer position function, fp32 math, one rounding:
 *   t(p)  = min((p / div) * div_mul + (p % mod) * mod_mul + add, t_max),
 *   p     = pos0 + row, or pos0 + (row / pos_block) * pos_block_stride + row % pos_block for a block-cyclic stripe
 *   theta = fp32(t) * inv_freq[d]            (one fp32 rounding, as the reference forms it)
 *   out[d], out[d+D/2] = x[d] cos - x[d+D/2] sin, x[d+D/2] cos + x[d] sin
 * Covers base RoPE (t = p), the jetlong regroup of base-rotated tensors (t = p/G - p),
 * self-extend's grouped positions (t = p/Gs + shift) and DCA's mod / clamped / constant positions.
 * x, out: (B, S, Hx, D) with element strides; out may alias x or point into a KV cache.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  const void* x;
  void* out;
  int64_t x_stride_b, x_stride_s, x_stride_h;
  int64_t o_stride_b, o_stride_s, o_stride_h;
  int32_t batch, seqlen, heads, head_dim;
  int64_t pos0;
  int64_t div, div_mul, mod, mod_mul, add, t_max;
  const float* inv_freq;    /* (head_dim/2,) fp32 device array */
  int64_t pos_block;        /* <= 0 means contiguous */
  int64_t pos_block_stride;
} jl_rotate_args;

int jl_rotate(const jl_rotate_args* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------------
 * jl_norm_rope — per-head RMSNorm, base RoPE and (optionally) the jetlong regroup of a projection
 * output in ONE pass: replaces q_norm / k_norm (Qwen3RMSNorm: fp32 statistics, normalised value
 * rounded to bf16, then multiplied by the bf16 weight), apply_rotary_pos_emb and
 * correction_rotate_per_sample (modeling_qwen3_jetlong_fused.py:292-294, :171-176, :209-226).
 *   y          = weight * bf16(x * rsqrt(mean(x^2) + eps))            (Qwen3RMSNorm's roundings)
 *   out_base   = R(p) y                                               p from pos0 / pos_block / pos_block_stride
 *   out_group  = R(floor(p / group_size) - p) R(p) y                  (fp32 composition, one rounding; may be NULL)
 * x, out_base, out_group: (B, S, Hx, D) with element strides; out_base may point into a KV cache.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  const void* x;
  const void* weight;       /* (head_dim,) bf16 */
  void* out_base;
  void* out_group;          /* may be NULL */
  int64_t x_stride_b, x_stride_s, x_stride_h;
  int64_t b_stride_b, b_stride_s, b_stride_h;
  int64_t g_stride_b, g_stride_s, g_stride_h;
  int32_t batch, seqlen, heads, head_dim;
  float eps;
  int32_t group_size;
  int64_t pos0, pos_block, pos_block_stride;
  const float* inv_freq;    /* (head_dim/2,) fp32 device array */
} jl_norm_rope_args;

int jl_norm_rope(const jl_norm_rope_args* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------------
 * jl_rmsnorm — Qwen3RMSNorm over the hidden dimension in one pass, optionally fused with the residual
 * add that precedes it in the decoder layer (transformers' Qwen3DecoderLayer, which the reference's
 * modeling file inherits at modeling_qwen3_jetlong_fused.py:468-471):
 *   h   = x (+ residual)                       (bf16; written to sum_out when residual != NULL)
 *   out = weight * bf16(h * rsqrt(mean(h^2) + eps))
 * x, residual, sum_out, out: (rows, hidden) contiguous bf16; hidden a multiple of 8 and <= 8192.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  const void* x;
  const void* residual;     /* may be NULL */
  const void* weight;       /* (hidden,) bf16 */
  void* sum_out;            /* required when residual != NULL; may alias residual or x */
  void* out;
  int64_t rows;
  int32_t hidden;
  float eps;
} jl_rmsnorm_args;

int jl_rmsnorm(const jl_rmsnorm_args* args, void* cuda_stream);

/* jl_silu_mul — out = silu(gate) * up over `count` contiguous bf16 values (a multiple of 8), the elementwise
 * part of the Qwen3 MLP the decoder layer runs between its projections (transformers' Qwen3MLP, inherited at
 * modeling_qwen3_jetlong_fused.py:468-471), in one pass; roundings as torch's two bf16 ops.  out may alias gate or up. */
typedef struct {
  const void* gate;
  const void* up;
  void* out;
  int64_t count;
} jl_silu_mul_args;

int jl_silu_mul(const jl_silu_mul_args* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------------
 * Decode-step state on the device, so that one captured CUDA graph can be replayed for every new
 * token.  The reference's decode step reads positions back to the host in every layer
 * (modeling_qwen3_jetlong_fused.py:145, :342, :406) and cannot be captured; here the per-token facts
 * live in device memory and kernels whose host arguments are fixed read them.  No reference counterpart.
 *
 * state: int64[JL_STEP_STATE_WORDS] = { pos, row, own, n_far, n_near, steps }
 *   pos    absolute position of the token being decoded
 *   row    cache row (of this rank's stripe) the token's key / value go to
 *   own    1 if this rank stores the token (always 1 without sharding)
 *   n_far  rows of this rank's cache in the far class: positions < pos - w_0
 *   n_near rows in the near class, the new token included when owned
 *   steps  number of advances made on this state (never rewound; an epoch source for jl_peer_merge)
 * jl_step_advance: pos <- pos + 1, steps <- steps + 1, the other words recomputed for a cache sharded block-cyclically
 * (block `block`, this rank `rank` of `world`; world = 1: contiguous).  lens, if not NULL, is an
 * int32[2 * batch] device array that receives n_far (first batch entries) and n_near (next batch
 * entries) for jl_kv_segment.len_dev.  Initialise state[0] to (next position - 1) from the host.
 * ------------------------------------------------------------------------------------------- */
#define JL_STEP_STATE_WORDS 6
typedef struct {
  int64_t* state;
  int32_t* lens;            /* may be NULL */
  int32_t batch;
  int32_t rank, world;
  int32_t reserved;
  int64_t block;
  int64_t w_0;
} jl_step_advance_args;

int jl_step_advance(const jl_step_advance_args* args, void* cuda_stream);

/* jl_decode_append — everything between the q/k/v projections and the attention of one decode step, in
 * one launch: per-head RMSNorm of q and k, base RoPE at state->pos, the regrouped query, and the
 * write of the new key (base-rotated) and value into row state->row of the cache when state->own
 * (replaces q_norm / k_norm, apply_rotary_pos_emb, correction_rotate_per_sample on q and the
 * DynamicCache update, modeling_qwen3_jetlong_fused.py:292-294, :329-340, :375-376).  Same roundings as
 * jl_norm_rope.  q: (B, H, D), k / v: (B, Hk, D) rows with strides; q_base / q_group: (B, H, D)
 * contiguous; k_cache / v_cache: (B, rows, Hk, D) with strides.
 * k_group_cache (optional, same shape and strides as k_cache) holds REGROUPED copies of the far rows, so
 * that the attention reads them as stored instead of rotating them for every token: each call rewrites
 * row n_far - 1 (the row that may just have crossed into the far class) as
 * R(floor(p / group_size) - p) k_cache[row], p = pos0 + row or the block-cyclic
 * pos0 + (row / pos_block) * pos_block_stride + row % pos_block, with jl_rotate's arithmetic. */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  int64_t q_stride_b, q_stride_h, k_stride_b, k_stride_h, v_stride_b, v_stride_h;
  const void* q_weight;     /* (head_dim,) bf16 */
  const void* k_weight;
  float q_eps, k_eps;
  void* q_base;
  void* q_group;
  void* k_cache;
  void* v_cache;
  int64_t kc_stride_b, kc_stride_s, kc_stride_h, vc_stride_b, vc_stride_s, vc_stride_h;
  int32_t batch, heads, kv_heads, head_dim;
  int32_t group_size;
  int32_t reserved;
  int64_t cache_rows;       /* capacity: a row index at or past it is never written */
  const float* inv_freq;    /* (head_dim/2,) fp32 device array */
  const int64_t* state;     /* device, JL_STEP_STATE_WORDS words */
  void* k_group_cache;      /* may be NULL */
  int64_t pos0;
  int64_t pos_block;        /* <= 0 means contiguous */
  int64_t pos_block_stride;
} jl_decode_append_args;

int jl_decode_append(const jl_decode_append_args* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------------
 * jl_peer_merge — the exchange step of the KV-sharded decode fused with the N-way merge, over
 * peer-mapped memory instead of a collective library call: every rank pushes its partial (O, LSE) into
 * every rank's exchange buffer with plain peer stores (NVLink), publishes a per-source flag, waits (at
 * most wait_limit_ms, 1 s by default; then *status = 1 and the result is invalid — the kernel never hangs)
 * for the other ranks' flags and merges the `world` partials that have landed in its own memory.  A caller
 * must read *status at its next synchronisation point and discard the step (or redo the exchange with a
 * collective) when it is set; ranks must not drift apart by more than the limit between calls.  No reference counterpart
 * (the reference is single-GPU; its split-K merge is cute_decode_sm90.py:199-215).
 *
 * part_o (batch, heads, 128) bf16 contiguous, part_lse (batch, heads) fp32: this rank's partial.
 * peer_buf[r]: rank r's exchange buffer as mapped into THIS process (peer_buf[rank] is the local one);
 * every buffer has jl_peer_merge_buffer_bytes(world, batch, heads, head_dim) bytes, the same size on all
 * ranks, and starts zeroed.  All ranks call with the same shapes and the same epoch
 *   e = (*epoch_base_dev) * epoch_stride + epoch_offset >= 1,
 * which must grow by exactly 1 from one use of the buffers to the next (two parities alternate on it).
 * out (batch, heads, 128) bf16, lse_out (batch, heads) fp32 or NULL.  One launch per rank, every rank on
 * its own GPU.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  const void* part_o;
  const float* part_lse;
  void* peer_buf[JL_MAX_PARTS];
  size_t buffer_bytes;
  int32_t rank, world;
  int32_t batch, heads, head_dim;
  int32_t wait_limit_ms;           /* longest wait for the other ranks' flags; <= 0: 1000 */
  const int64_t* epoch_base_dev;   /* NULL: base 0 */
  int64_t epoch_stride, epoch_offset;
  void* out;
  float* lse_out;
  int32_t* status;                 /* device word, raised to 1 when a wait gave up */
} jl_peer_merge_args;

size_t jl_peer_merge_buffer_bytes(int32_t world, int32_t batch, int32_t heads, int32_t head_dim);
int jl_peer_merge(const jl_peer_merge_args* args, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* JETLONG_B200_H_ */

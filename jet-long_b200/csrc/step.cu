// Device-resident decode-step state and the fused "q/k norm -> RoPE -> cache write" kernel that reads it,
// so that a whole decode step can be one replayed CUDA graph: no kernel argument on the host changes
// from token to token.
#include "jl_common.cuh"

namespace jl {

namespace {

// rows of a block-cyclic stripe (rank r of `world`, block `block`) among the first n tokens
__device__ __forceinline__ int64_t rows_owned(int64_t n, int64_t rank, int64_t world, int64_t block) {
  if (world <= 1) return n;
  const int64_t span = world * block, full = n / span, rem = n % span;
  int64_t extra = rem - rank * block;
  extra = extra < 0 ? 0 : (extra > block ? block : extra);
  return full * block + extra;
}

__global__ void step_advance_kernel(int64_t* state, int32_t* lens, int batch, int64_t rank, int64_t world,
                                    int64_t block, int64_t w_0) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int64_t pos = state[0] + 1;
  const int64_t row = rows_owned(pos, rank, world, block);
  const int64_t own = world <= 1 ? 1 : ((pos / block) % world == rank ? 1 : 0);
  const int64_t boundary = pos - w_0 > 0 ? pos - w_0 : 0;
  const int64_t n_far = rows_owned(boundary, rank, world, block);
  const int64_t n_near = row + own - n_far;
  state[0] = pos; state[1] = row; state[2] = own; state[3] = n_far; state[4] = n_near; state[5] += 1;
  if (lens != nullptr)
    for (int b = 0; b < batch; ++b) {
      lens[b] = static_cast<int32_t>(n_far);
      lens[batch + b] = static_cast<int32_t>(n_near);
    }
}

struct AppendParams {
  const __nv_bfloat16 *q, *k, *v, *qw, *kw;
  int64_t qs_b, qs_h, ks_b, ks_h, vs_b, vs_h;
  float q_eps, k_eps;
  __nv_bfloat16 *q_base, *q_group, *kc, *vc;
  int64_t kcs_b, kcs_s, kcs_h, vcs_b, vcs_s, vcs_h;
  int batch, heads, kv_heads, group_size;
  int64_t cache_rows;
  const float* inv_freq;
  const int64_t* state;
  __nv_bfloat16* kg;           // optional regrouped copy of the far rows (strides of kc)
  int64_t pos0, pos_block, pos_block_stride;
};

// One warp per (batch, head) row of 128 values: query heads, then key heads, then value heads, then (with a
// regrouped far-key cache) the key heads of the newest far row.
__global__ void __launch_bounds__(128) decode_append_kernel(const AppendParams p) {
  const int lane = threadIdx.x & 31;
  const int per_b = p.heads + 2 * p.kv_heads + (p.kg != nullptr ? p.kv_heads : 0);
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= p.batch * per_b) return;
  const int b = item / per_b, h = item % per_b;
  const int64_t pos = p.state[0], row = p.state[1];
  const bool own = p.state[2] != 0 && row >= 0 && row < p.cache_rows;

  if (h >= p.heads + 2 * p.kv_heads) {                  // regroup the last far row: R(floor(p/G) - p) k_cache[row]
    const int64_t far_row = p.state[3] - 1;
    if (far_row < 0 || far_row >= p.cache_rows) return;
    const int hk = h - p.heads - 2 * p.kv_heads;
    const int64_t kp = key_position(far_row, p.pos0, p.pos_block, p.pos_block_stride);
    const float tf = static_cast<float>(kp / p.group_size - kp);
    float s0, c0, s1, c1;
    sincosf(__fmul_rn(tf, p.inv_freq[2 * lane]), &s0, &c0);
    sincosf(__fmul_rn(tf, p.inv_freq[2 * lane + 1]), &s1, &c1);
    const int64_t off = b * p.kcs_b + far_row * p.kcs_s + hk * p.kcs_h;
    const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p.kc + off + 2 * lane));
    const float2 bb = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p.kc + off + 64 + 2 * lane));
    *reinterpret_cast<uint32_t*>(p.kg + off + 2 * lane) = pack_bf16x2(a.x * c0 - bb.x * s0, a.y * c1 - bb.y * s1);
    *reinterpret_cast<uint32_t*>(p.kg + off + 64 + 2 * lane) = pack_bf16x2(bb.x * c0 + a.x * s0, bb.y * c1 + a.y * s1);
    return;
  }

  if (h >= p.heads + p.kv_heads) {                      // value head: plain copy into the cache row
    if (!own) return;
    const int hv = h - p.heads - p.kv_heads;
    const uint2 val = *reinterpret_cast<const uint2*>(p.v + b * p.vs_b + hv * p.vs_h + 4 * lane);
    *reinterpret_cast<uint2*>(p.vc + b * p.vcs_b + row * p.vcs_s + hv * p.vcs_h + 4 * lane) = val;
    return;
  }
  const bool is_q = h < p.heads;
  if (!is_q && !own) return;
  const int hh = is_q ? h : h - p.heads;
  const __nv_bfloat16* x = is_q ? p.q + b * p.qs_b + hh * p.qs_h : p.k + b * p.ks_b + hh * p.ks_h;
  const __nv_bfloat16* w = is_q ? p.qw : p.kw;
  const float f0 = p.inv_freq[2 * lane], f1 = p.inv_freq[2 * lane + 1];
  const float2 w_lo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + 2 * lane));
  const float2 w_hi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + 64 + 2 * lane));
  const float tb = static_cast<float>(pos);
  float sb0, cb0, sb1, cb1;
  sincosf(__fmul_rn(tb, f0), &sb0, &cb0);
  sincosf(__fmul_rn(tb, f1), &sb1, &cb1);
  const float2 lo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + 2 * lane));
  const float2 hi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + 64 + 2 * lane));
  float bl0, bl1, bh0, bh1;
  norm_rope_head(lo, hi, w_lo, w_hi, is_q ? p.q_eps : p.k_eps, sb0, cb0, sb1, cb1, bl0, bl1, bh0, bh1);
  if (!is_q) {
    __nv_bfloat16* dst = p.kc + b * p.kcs_b + row * p.kcs_s + hh * p.kcs_h;
    *reinterpret_cast<uint32_t*>(dst + 2 * lane) = pack_bf16x2(bl0, bl1);
    *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = pack_bf16x2(bh0, bh1);
    return;
  }
  __nv_bfloat16* qb = p.q_base + (static_cast<int64_t>(b) * p.heads + hh) * kHeadDim;
  *reinterpret_cast<uint32_t*>(qb + 2 * lane) = pack_bf16x2(bl0, bl1);
  *reinterpret_cast<uint32_t*>(qb + 64 + 2 * lane) = pack_bf16x2(bh0, bh1);
  if (p.q_group != nullptr) {
    const float td = static_cast<float>(pos / p.group_size - pos);
    float sd0, cd0, sd1, cd1;
    sincosf(__fmul_rn(td, f0), &sd0, &cd0);
    sincosf(__fmul_rn(td, f1), &sd1, &cd1);
    __nv_bfloat16* qg = p.q_group + (static_cast<int64_t>(b) * p.heads + hh) * kHeadDim;
    *reinterpret_cast<uint32_t*>(qg + 2 * lane) = pack_bf16x2(bl0 * cd0 - bh0 * sd0, bl1 * cd1 - bh1 * sd1);
    *reinterpret_cast<uint32_t*>(qg + 64 + 2 * lane) = pack_bf16x2(bh0 * cd0 + bl0 * sd0, bh1 * cd1 + bl1 * sd1);
  }
}

}  // namespace

int launch_step_advance(const jl_step_advance_args* a, cudaStream_t stream) {
  if (a->state == nullptr) return fail(JL_ERR_BAD_ARG, "jl_step_advance: state is NULL");
  if (a->batch < 0 || a->world < 1 || a->rank < 0 || a->rank >= a->world)
    return fail(JL_ERR_BAD_ARG, "jl_step_advance: need batch >= 0 and 0 <= rank < world");
  if (a->world > 1 && a->block < 1) return fail(JL_ERR_BAD_ARG, "jl_step_advance: block must be >= 1 when world > 1");
  if (a->w_0 < 0) return fail(JL_ERR_BAD_ARG, "jl_step_advance: w_0 must be >= 0");
  step_advance_kernel<<<1, 32, 0, stream>>>(a->state, a->lens, a->batch, a->rank, a->world, a->block, a->w_0);
  return check_launch("jl_step_advance");
}

int launch_decode_append(const jl_decode_append_args* a, cudaStream_t stream) {
  if (a->head_dim != kHeadDim) return fail(JL_ERR_UNSUPPORTED, "jl_decode_append: head_dim must be 128, got %d", a->head_dim);
  if (a->q == nullptr || a->k == nullptr || a->v == nullptr || a->q_weight == nullptr || a->k_weight == nullptr ||
      a->q_base == nullptr || a->k_cache == nullptr || a->v_cache == nullptr || a->inv_freq == nullptr || a->state == nullptr)
    return fail(JL_ERR_BAD_ARG, "jl_decode_append: NULL pointer");
  if (a->batch < 0 || a->heads < 1 || a->kv_heads < 1 || a->cache_rows < 0)
    return fail(JL_ERR_BAD_ARG, "jl_decode_append: sizes out of range");
  if (a->q_group != nullptr && a->group_size < 1) return fail(JL_ERR_BAD_ARG, "jl_decode_append: group_size must be >= 1");
  const int64_t st[] = {a->q_stride_b, a->q_stride_h, a->k_stride_b, a->k_stride_h, a->v_stride_b, a->v_stride_h,
                        a->kc_stride_b, a->kc_stride_s, a->kc_stride_h, a->vc_stride_b, a->vc_stride_s, a->vc_stride_h};
  for (int64_t v : st)
    if (v % 4 != 0) return fail(JL_ERR_BAD_ARG, "jl_decode_append: strides must be multiples of 4 elements");
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
                         reinterpret_cast<uintptr_t>(a->q_base) | reinterpret_cast<uintptr_t>(a->q_group) |
                         reinterpret_cast<uintptr_t>(a->k_cache) | reinterpret_cast<uintptr_t>(a->v_cache) |
                         reinterpret_cast<uintptr_t>(a->q_weight) | reinterpret_cast<uintptr_t>(a->k_weight);
  if (ptrs & 7) return fail(JL_ERR_BAD_ARG, "jl_decode_append: pointers must be 8-byte aligned");
  if (a->batch == 0) return JL_OK;
  AppendParams p{};
  p.q = static_cast<const __nv_bfloat16*>(a->q); p.k = static_cast<const __nv_bfloat16*>(a->k);
  p.v = static_cast<const __nv_bfloat16*>(a->v);
  p.qw = static_cast<const __nv_bfloat16*>(a->q_weight); p.kw = static_cast<const __nv_bfloat16*>(a->k_weight);
  p.qs_b = a->q_stride_b; p.qs_h = a->q_stride_h; p.ks_b = a->k_stride_b; p.ks_h = a->k_stride_h;
  p.vs_b = a->v_stride_b; p.vs_h = a->v_stride_h;
  p.q_eps = a->q_eps; p.k_eps = a->k_eps;
  p.q_base = static_cast<__nv_bfloat16*>(a->q_base); p.q_group = static_cast<__nv_bfloat16*>(a->q_group);
  p.kc = static_cast<__nv_bfloat16*>(a->k_cache); p.vc = static_cast<__nv_bfloat16*>(a->v_cache);
  p.kcs_b = a->kc_stride_b; p.kcs_s = a->kc_stride_s; p.kcs_h = a->kc_stride_h;
  p.vcs_b = a->vc_stride_b; p.vcs_s = a->vc_stride_s; p.vcs_h = a->vc_stride_h;
  p.batch = a->batch; p.heads = a->heads; p.kv_heads = a->kv_heads;
  p.group_size = a->group_size > 0 ? a->group_size : 1;
  p.cache_rows = a->cache_rows;
  p.inv_freq = a->inv_freq; p.state = a->state;
  p.kg = static_cast<__nv_bfloat16*>(a->k_group_cache);
  p.pos0 = a->pos0;
  p.pos_block = a->pos_block > 0 ? a->pos_block : 0;
  p.pos_block_stride = a->pos_block_stride;
  if (reinterpret_cast<uintptr_t>(a->k_group_cache) & 7) return fail(JL_ERR_BAD_ARG, "jl_decode_append: pointers must be 8-byte aligned");
  const int items = a->batch * (a->heads + 2 * a->kv_heads + (p.kg != nullptr ? a->kv_heads : 0));
  decode_append_kernel<<<(items + 3) / 4, 128, 0, stream>>>(p);
  return check_launch("jl_decode_append");
}

}  // namespace jl

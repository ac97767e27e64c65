// Rotate-half RoPE by an integer position function (base RoPE, jetlong regroup, self-extend and
// DCA class positions) — one fused elementwise pass, fp32 math, a single rounding to bf16.
//
// One thread owns a (row, d) / (row, d + 64) pair group: 8 consecutive d (one 16-byte vector) from
// each half, so loads and stores stay 128-bit.  8 threads cover a 128-wide head row.
#include "jl_common.cuh"

namespace jl {

struct RotateParams {
  const __nv_bfloat16* x;
  __nv_bfloat16* out;
  int64_t xs_b, xs_s, xs_h, os_b, os_s, os_h;
  int batch, seqlen, heads;
  int64_t pos0, div, div_mul, mod, mod_mul, add, t_max, pos_block, pos_block_stride;
  const float* inv_freq;
};

__global__ void __launch_bounds__(256) rotate_kernel(const RotateParams p) {
  __shared__ float s_freq[kHeadDim / 2];
  if (threadIdx.x < kHeadDim / 2) s_freq[threadIdx.x] = p.inv_freq[threadIdx.x];
  __syncthreads();
  const int64_t total = static_cast<int64_t>(p.batch) * p.seqlen * p.heads * 8;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx & 7);          // which 8-wide d group of the first half
    int64_t r = idx >> 3;
    const int h = static_cast<int>(r % p.heads);
    r /= p.heads;
    const int64_t s = r % p.seqlen;
    const int64_t b = r / p.seqlen;
    const int64_t pos = key_position(s, p.pos0, p.pos_block, p.pos_block_stride);
    int64_t t = (pos / p.div) * p.div_mul + (pos % p.mod) * p.mod_mul + p.add;
    t = t < p.t_max ? t : p.t_max;
    const float tf = static_cast<float>(t);
    const __nv_bfloat16* xr = p.x + b * p.xs_b + s * p.xs_s + h * p.xs_h;
    __nv_bfloat16* orow = p.out + b * p.os_b + s * p.os_s + h * p.os_h;
    const uint4 lo = *reinterpret_cast<const uint4*>(xr + c * 8);
    const uint4 hi = *reinterpret_cast<const uint4*>(xr + 64 + c * 8);
    const uint32_t* ul = reinterpret_cast<const uint32_t*>(&lo);
    const uint32_t* uh = reinterpret_cast<const uint32_t*>(&hi);
    uint4 rl, rh;
    uint32_t* pl = reinterpret_cast<uint32_t*>(&rl);
    uint32_t* ph = reinterpret_cast<uint32_t*>(&rh);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(ul[j]);
      const float2 bb = unpack_bf16x2(uh[j]);
      float s0, c0, s1, c1;
      sincosf(__fmul_rn(tf, s_freq[c * 8 + 2 * j]), &s0, &c0);
      sincosf(__fmul_rn(tf, s_freq[c * 8 + 2 * j + 1]), &s1, &c1);
      pl[j] = pack_bf16x2(a.x * c0 - bb.x * s0, a.y * c1 - bb.y * s1);
      ph[j] = pack_bf16x2(bb.x * c0 + a.x * s0, bb.y * c1 + a.y * s1);
    }
    *reinterpret_cast<uint4*>(orow + c * 8) = rl;
    *reinterpret_cast<uint4*>(orow + 64 + c * 8) = rh;
  }
}

int launch_rotate(const jl_rotate_args* a, cudaStream_t stream) {
  if (a->head_dim != kHeadDim) return fail(JL_ERR_UNSUPPORTED, "jl_rotate: head_dim must be 128, got %d", a->head_dim);
  if (a->x == nullptr || a->out == nullptr || a->inv_freq == nullptr) return fail(JL_ERR_BAD_ARG, "jl_rotate: NULL pointer");
  if (a->batch < 0 || a->seqlen < 0 || a->heads < 0) return fail(JL_ERR_BAD_ARG, "jl_rotate: negative size");
  if (a->div < 1 || a->mod < 1) return fail(JL_ERR_BAD_ARG, "jl_rotate: div and mod must be >= 1");
  const int64_t strides[] = {a->x_stride_b, a->x_stride_s, a->x_stride_h, a->o_stride_b, a->o_stride_s, a->o_stride_h};
  for (int64_t st : strides)
    if (st % 8 != 0) return fail(JL_ERR_BAD_ARG, "jl_rotate: strides must be multiples of 8 elements (16 bytes)");
  if ((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->out)) & 15)
    return fail(JL_ERR_BAD_ARG, "jl_rotate: pointers must be 16-byte aligned");
  RotateParams p{};
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.xs_b = a->x_stride_b; p.xs_s = a->x_stride_s; p.xs_h = a->x_stride_h;
  p.os_b = a->o_stride_b; p.os_s = a->o_stride_s; p.os_h = a->o_stride_h;
  p.batch = a->batch; p.seqlen = a->seqlen; p.heads = a->heads;
  p.pos0 = a->pos0; p.div = a->div; p.div_mul = a->div_mul; p.mod = a->mod; p.mod_mul = a->mod_mul;
  p.add = a->add; p.t_max = a->t_max;
  p.pos_block = (a->pos_block > 0 && a->pos_block < a->seqlen) ? a->pos_block : 0;
  p.pos_block_stride = a->pos_block_stride;
  p.inv_freq = a->inv_freq;
  const int64_t total = static_cast<int64_t>(a->batch) * a->seqlen * a->heads * 8;
  if (total == 0) return JL_OK;
  const int64_t blocks = (total + 255) / 256;
  const int grid = static_cast<int>(blocks < 148 * 8 ? blocks : 148 * 8);
  rotate_kernel<<<grid, 256, 0, stream>>>(p);
  return check_launch("jl_rotate");
}

// ---------------------------------------------------------------------------------------------
// RMSNorm + base RoPE (+ regroup) of a projection output, one pass.  One warp per token row, looping
// over the heads: lane l owns dims 2l, 2l+1 and their rotation partners 64+2l, 64+2l+1, so the four
// sincos of the row (base angle and regroup angle for two frequencies) are computed once and reused
// by every head, each half-row load is one coalesced 128-byte request, and the RMS statistic is a
// five-step warp reduction.
// ---------------------------------------------------------------------------------------------
struct NormRopeParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* w;
  __nv_bfloat16* ob;
  __nv_bfloat16* og;
  int64_t xs_b, xs_s, xs_h, bs_b, bs_s, bs_h, gs_b, gs_s, gs_h;
  int batch, seqlen, heads, group_size;
  float eps;
  int64_t pos0, pos_block, pos_block_stride;
  const float* inv_freq;
};

__global__ void __launch_bounds__(256) norm_rope_kernel(const NormRopeParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t rows = static_cast<int64_t>(p.batch) * p.seqlen;
  const float f0 = p.inv_freq[2 * lane], f1 = p.inv_freq[2 * lane + 1];
  const float2 w_lo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p.w + 2 * lane));
  const float2 w_hi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p.w + 64 + 2 * lane));
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5)) {
    const int64_t s = row % p.seqlen, b = row / p.seqlen;
    const int64_t pos = key_position(s, p.pos0, p.pos_block, p.pos_block_stride);
    const float tb = static_cast<float>(pos), td = static_cast<float>(pos / p.group_size - pos);
    float sb0, cb0, sb1, cb1, sd0 = 0.f, cd0 = 1.f, sd1 = 0.f, cd1 = 1.f;
    sincosf(__fmul_rn(tb, f0), &sb0, &cb0);
    sincosf(__fmul_rn(tb, f1), &sb1, &cb1);
    if (p.og != nullptr) {
      sincosf(__fmul_rn(td, f0), &sd0, &cd0);
      sincosf(__fmul_rn(td, f1), &sd1, &cd1);
    }
    const __nv_bfloat16* xr = p.x + b * p.xs_b + s * p.xs_s;
    __nv_bfloat16* br = p.ob + b * p.bs_b + s * p.bs_s;
    __nv_bfloat16* gr = p.og != nullptr ? p.og + b * p.gs_b + s * p.gs_s : nullptr;
    for (int h = 0; h < p.heads; ++h) {
      const float2 lo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(xr + h * p.xs_h + 2 * lane));
      const float2 hi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(xr + h * p.xs_h + 64 + 2 * lane));
      float bl0, bl1, bh0, bh1;
      norm_rope_head(lo, hi, w_lo, w_hi, p.eps, sb0, cb0, sb1, cb1, bl0, bl1, bh0, bh1);
      *reinterpret_cast<uint32_t*>(br + h * p.bs_h + 2 * lane) = pack_bf16x2(bl0, bl1);
      *reinterpret_cast<uint32_t*>(br + h * p.bs_h + 64 + 2 * lane) = pack_bf16x2(bh0, bh1);
      if (gr != nullptr) {
        *reinterpret_cast<uint32_t*>(gr + h * p.gs_h + 2 * lane) = pack_bf16x2(bl0 * cd0 - bh0 * sd0, bl1 * cd1 - bh1 * sd1);
        *reinterpret_cast<uint32_t*>(gr + h * p.gs_h + 64 + 2 * lane) = pack_bf16x2(bh0 * cd0 + bl0 * sd0, bh1 * cd1 + bl1 * sd1);
      }
    }
  }
}

int launch_norm_rope(const jl_norm_rope_args* a, cudaStream_t stream) {
  if (a->head_dim != kHeadDim) return fail(JL_ERR_UNSUPPORTED, "jl_norm_rope: head_dim must be 128, got %d", a->head_dim);
  if (a->x == nullptr || a->weight == nullptr || a->out_base == nullptr || a->inv_freq == nullptr)
    return fail(JL_ERR_BAD_ARG, "jl_norm_rope: NULL pointer");
  if (a->batch < 0 || a->seqlen < 0 || a->heads < 0) return fail(JL_ERR_BAD_ARG, "jl_norm_rope: negative size");
  if (a->out_group != nullptr && a->group_size < 1) return fail(JL_ERR_BAD_ARG, "jl_norm_rope: group_size must be >= 1");
  const int64_t st[] = {a->x_stride_b, a->x_stride_s, a->x_stride_h, a->b_stride_b, a->b_stride_s, a->b_stride_h,
                        a->g_stride_b, a->g_stride_s, a->g_stride_h};
  for (int64_t v : st)
    if (v % 2 != 0) return fail(JL_ERR_BAD_ARG, "jl_norm_rope: strides must be even (4-byte aligned rows)");
  if ((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->weight) | reinterpret_cast<uintptr_t>(a->out_base) |
       reinterpret_cast<uintptr_t>(a->out_group)) & 3)
    return fail(JL_ERR_BAD_ARG, "jl_norm_rope: pointers must be 4-byte aligned");
  NormRopeParams p{};
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.w = static_cast<const __nv_bfloat16*>(a->weight);
  p.ob = static_cast<__nv_bfloat16*>(a->out_base);
  p.og = static_cast<__nv_bfloat16*>(a->out_group);
  p.xs_b = a->x_stride_b; p.xs_s = a->x_stride_s; p.xs_h = a->x_stride_h;
  p.bs_b = a->b_stride_b; p.bs_s = a->b_stride_s; p.bs_h = a->b_stride_h;
  p.gs_b = a->g_stride_b; p.gs_s = a->g_stride_s; p.gs_h = a->g_stride_h;
  p.batch = a->batch; p.seqlen = a->seqlen; p.heads = a->heads;
  p.group_size = a->group_size > 0 ? a->group_size : 1;
  p.eps = a->eps;
  p.pos0 = a->pos0;
  p.pos_block = (a->pos_block > 0 && a->pos_block < a->seqlen) ? a->pos_block : 0;
  p.pos_block_stride = a->pos_block_stride;
  p.inv_freq = a->inv_freq;
  const int64_t rows = static_cast<int64_t>(a->batch) * a->seqlen;
  if (rows == 0 || a->heads == 0) return JL_OK;
  const int64_t blocks = (rows + 7) / 8;
  const int grid = static_cast<int>(blocks < 148 * 8 ? blocks : 148 * 8);
  norm_rope_kernel<<<grid, 256, 0, stream>>>(p);
  return check_launch("jl_norm_rope");
}

// ---------------------------------------------------------------------------------------------
// RMSNorm over the hidden dimension (+ fused residual add): one CTA of 256 threads per row at a time,
// the row lives in registers (up to four 16-byte vectors per thread), one block reduction.
// ---------------------------------------------------------------------------------------------
struct RmsParams {
  const uint4* x;
  const uint4* res;
  const uint4* w;
  uint4* sum_out;
  uint4* out;
  int64_t rows;
  int n_vec;        // hidden / 8
  float inv_hidden, eps;
};

__global__ void __launch_bounds__(256) rmsnorm_kernel(const RmsParams p) {
  __shared__ float s_part[8];
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  uint4 wv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (t + i * 256 < p.n_vec) wv[i] = p.w[t + i * 256];
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    uint4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = t + i * 256;
      if (c < p.n_vec) {
        v[i] = p.x[row * p.n_vec + c];
        uint32_t* u = reinterpret_cast<uint32_t*>(&v[i]);
        if (p.res != nullptr) {
          const uint4 r = p.res[row * p.n_vec + c];
          const uint32_t* ur = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 a = unpack_bf16x2(u[j]), b = unpack_bf16x2(ur[j]);
            u[j] = pack_bf16x2(a.x + b.x, a.y + b.y);
          }
          p.sum_out[row * p.n_vec + c] = v[i];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = unpack_bf16x2(u[j]);
          ss = fmaf(a.x, a.x, fmaf(a.y, a.y, ss));
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (lane == 0) s_part[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += s_part[i];
    __syncthreads();
    const float r = rsqrtf(tot * p.inv_hidden + p.eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = t + i * 256;
      if (c < p.n_vec) {
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&v[i]);
        const uint32_t* uw = reinterpret_cast<const uint32_t*>(&wv[i]);
        uint4 o;
        uint32_t* uo = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = unpack_bf16x2(u[j]), w2 = unpack_bf16x2(uw[j]);
          const float2 n = unpack_bf16x2(pack_bf16x2(a.x * r, a.y * r));      // normalised value rounded to bf16 first
          uo[j] = pack_bf16x2(w2.x * n.x, w2.y * n.y);
        }
        p.out[row * p.n_vec + c] = o;
      }
    }
  }
}

int launch_rmsnorm(const jl_rmsnorm_args* a, cudaStream_t stream) {
  if (a->x == nullptr || a->weight == nullptr || a->out == nullptr) return fail(JL_ERR_BAD_ARG, "jl_rmsnorm: NULL pointer");
  if (a->residual != nullptr && a->sum_out == nullptr) return fail(JL_ERR_BAD_ARG, "jl_rmsnorm: sum_out is required with a residual");
  if (a->hidden <= 0 || a->hidden % 8 != 0 || a->hidden > 8192)
    return fail(JL_ERR_UNSUPPORTED, "jl_rmsnorm: hidden must be a multiple of 8 and <= 8192, got %d", a->hidden);
  if (a->rows < 0) return fail(JL_ERR_BAD_ARG, "jl_rmsnorm: negative row count");
  if ((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->residual) | reinterpret_cast<uintptr_t>(a->weight) |
       reinterpret_cast<uintptr_t>(a->sum_out) | reinterpret_cast<uintptr_t>(a->out)) & 15)
    return fail(JL_ERR_BAD_ARG, "jl_rmsnorm: pointers must be 16-byte aligned");
  if (a->rows == 0) return JL_OK;
  RmsParams p{};
  p.x = static_cast<const uint4*>(a->x);
  p.res = static_cast<const uint4*>(a->residual);
  p.w = static_cast<const uint4*>(a->weight);
  p.sum_out = static_cast<uint4*>(a->sum_out);
  p.out = static_cast<uint4*>(a->out);
  p.rows = a->rows;
  p.n_vec = a->hidden / 8;
  p.inv_hidden = 1.f / static_cast<float>(a->hidden);
  p.eps = a->eps;
  const int grid = static_cast<int>(a->rows < 148 * 8 ? a->rows : 148 * 8);
  rmsnorm_kernel<<<grid, 256, 0, stream>>>(p);
  return check_launch("jl_rmsnorm");
}

// ---------------------------------------------------------------------------------------------
// SiLU(gate) * up of the Qwen3 MLP in one pass (torch runs two: the activation, then the product).
// Roundings as torch's bf16 ops: silu evaluated in fp32 and rounded to bf16, product rounded again.
__global__ void __launch_bounds__(256) silu_mul_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                                       uint4* __restrict__ out, int64_t n_vec) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 g = gate[i], u = up[i];
    const uint32_t* gw = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* uw = reinterpret_cast<const uint32_t*>(&u);
    uint4 r;
    uint32_t* rw = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(gw[j]), b = unpack_bf16x2(uw[j]);
      auto rb = [](float v) { return __bfloat162float(__float2bfloat16(v)); };
      const float s0 = rb(a.x / (1.f + expf(-a.x))), s1 = rb(a.y / (1.f + expf(-a.y)));
      rw[j] = pack_bf16x2(s0 * b.x, s1 * b.y);
    }
    out[i] = r;
  }
}

int launch_silu_mul(const jl_silu_mul_args* a, cudaStream_t stream) {
  if (a->gate == nullptr || a->up == nullptr || a->out == nullptr) return fail(JL_ERR_BAD_ARG, "jl_silu_mul: NULL pointer");
  if (a->count < 0 || a->count % 8 != 0) return fail(JL_ERR_BAD_ARG, "jl_silu_mul: count must be a non-negative multiple of 8");
  if ((reinterpret_cast<uintptr_t>(a->gate) | reinterpret_cast<uintptr_t>(a->up) | reinterpret_cast<uintptr_t>(a->out)) & 15)
    return fail(JL_ERR_BAD_ARG, "jl_silu_mul: pointers must be 16-byte aligned");
  if (a->count == 0) return JL_OK;
  const int64_t n_vec = a->count / 8;
  const int64_t blocks = (n_vec + 255) / 256;
  const int grid = static_cast<int>(blocks < 148 * 16 ? blocks : 148 * 16);
  silu_mul_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint4*>(a->gate), static_cast<const uint4*>(a->up),
                                            static_cast<uint4*>(a->out), n_vec);
  return check_launch("jl_silu_mul");
}

}  // namespace jl

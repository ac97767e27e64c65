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

}  // namespace jl

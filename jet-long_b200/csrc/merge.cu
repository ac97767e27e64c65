// N-way (O, LSE) merge of partial attention results — HBM-bound streaming kernel.
//
// Work layout: one output row (b, s, h) of head_dim = 128 bf16 is 256 bytes; 16 threads own a row
// and each moves one 16-byte vector per part, so a warp reads two fully coalesced 256-byte rows per
// part.  The per-row softmax weights are computed once per row (every thread of the row reads the
// same N fp32 LSE values, which the L1 broadcasts), not once per element.
#include "jl_common.cuh"

namespace jl {

struct MergeParams {
  const uint4* o[JL_MAX_PARTS];
  const float* lse[JL_MAX_PARTS];
  uint4* out;
  float* lse_out;
  int n_parts;
  int64_t rows;       // B * S * H
  int seqlen, heads;
  int round_like_reference;
};

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16(x)); }

// One row, NPARTS > 0: the part count is a compile-time constant so that every part's 16-byte load and
// LSE load is issued before the first is consumed (NPARTS * 16 B in flight per thread); NPARTS == 0:
// run-time count, loads issued part by part.
template <int NPARTS>
__device__ __forceinline__ void merge_row(const MergeParams& p, int64_t row, int lane16, int64_t lidx) {
  constexpr int kMax = NPARTS > 0 ? NPARTS : 1;
  const int n = NPARTS > 0 ? NPARTS : p.n_parts;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  float m = -INFINITY, wsum = 0.f;
  if (NPARTS > 0) {
    uint4 x[kMax];
    float l[kMax];
#pragma unroll
    for (int i = 0; i < kMax; ++i) {
      x[i] = p.o[i][row * 16 + lane16];
      l[i] = p.lse[i][lidx];
    }
#pragma unroll
    for (int i = 0; i < kMax; ++i) m = fmaxf(m, l[i]);
    const float m_safe = (m == -INFINITY) ? 0.f : m;
#pragma unroll
    for (int i = 0; i < kMax; ++i) {
      const float w = exp2f((l[i] - m_safe) * kLog2e);
      wsum += w;
      const uint32_t* u = reinterpret_cast<const uint32_t*>(&x[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(u[j]);
        acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
        acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
      }
    }
    m = m_safe;
  } else {
    for (int i = 0; i < n; ++i) m = fmaxf(m, p.lse[i][lidx]);
    const float m_safe = (m == -INFINITY) ? 0.f : m;
    for (int i = 0; i < n; ++i) {
      const float w = exp2f((p.lse[i][lidx] - m_safe) * kLog2e);
      wsum += w;
      const uint4 x = p.o[i][row * 16 + lane16];
      const uint32_t* u = reinterpret_cast<const uint32_t*>(&x);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(u[j]);
        acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
        acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
      }
    }
    m = m_safe;
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  uint4 r;
  uint32_t* ur = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) ur[j] = pack_bf16x2(acc[2 * j] * inv, acc[2 * j + 1] * inv);
  p.out[row * 16 + lane16] = r;
  if (p.lse_out != nullptr && lane16 == 0) p.lse_out[lidx] = wsum > 0.f ? m + logf(wsum) : -INFINITY;
}

template <int NPARTS>
__global__ void __launch_bounds__(256) merge_kernel(const MergeParams p) {
  const int lane16 = threadIdx.x & 15;
  const int64_t row_stride = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 4);
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 4) + (threadIdx.x >> 4); row < p.rows;
       row += row_stride) {
    const int64_t h = row % p.heads;
    const int64_t bs = row / p.heads;
    const int64_t s = bs % p.seqlen;
    const int64_t b = bs / p.seqlen;
    const int64_t lidx = (b * p.heads + h) * p.seqlen + s;

    if (p.round_like_reference) {
      // Two parts; every intermediate is rounded to bf16 like the torch op sequence it replaces.
      const float la = p.lse[0][lidx], lb = p.lse[1][lidx];
      const float m = fmaxf(la, lb);
      const float wa = __expf(la - m), wb = __expf(lb - m);
      const float den = fmaxf(wa + wb, 1.0e-7f);
      const float wan = round_bf16(wa / den), wbn = round_bf16(wb / den);
      const uint4 xa = p.o[0][row * 16 + lane16], xb = p.o[1][row * 16 + lane16];
      const uint32_t* ua = reinterpret_cast<const uint32_t*>(&xa);
      const uint32_t* ub = reinterpret_cast<const uint32_t*>(&xb);
      uint4 r;
      uint32_t* ur = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = unpack_bf16x2(ua[i]), bb = unpack_bf16x2(ub[i]);
        const float lo = round_bf16(wan * a.x) + round_bf16(wbn * bb.x);
        const float hi = round_bf16(wan * a.y) + round_bf16(wbn * bb.y);
        ur[i] = pack_bf16x2(lo, hi);
      }
      p.out[row * 16 + lane16] = r;
      if (p.lse_out != nullptr && lane16 == 0) p.lse_out[lidx] = m + __logf(wa + wb);
      continue;
    }

    merge_row<NPARTS>(p, row, lane16, lidx);
  }
}

int launch_merge(const jl_merge_args* a, cudaStream_t stream) {
  if (a->n_parts < 1 || a->n_parts > JL_MAX_PARTS) return fail(JL_ERR_BAD_ARG, "jl_merge: n_parts must be in [1, %d]", JL_MAX_PARTS);
  if (a->head_dim != kHeadDim) return fail(JL_ERR_UNSUPPORTED, "jl_merge: head_dim must be 128, got %d", a->head_dim);
  if (a->batch < 0 || a->seqlen < 0 || a->heads <= 0) return fail(JL_ERR_BAD_ARG, "jl_merge: negative size");
  if (a->round_like_reference && a->n_parts != 2) return fail(JL_ERR_BAD_ARG, "jl_merge: round_like_reference needs exactly 2 parts");
  if (a->out == nullptr) return fail(JL_ERR_BAD_ARG, "jl_merge: out is NULL");
  MergeParams p{};
  for (int i = 0; i < a->n_parts; ++i) {
    if (a->o[i] == nullptr || a->lse[i] == nullptr) return fail(JL_ERR_BAD_ARG, "jl_merge: part %d has a NULL pointer", i);
    if (reinterpret_cast<uintptr_t>(a->o[i]) & 15) return fail(JL_ERR_BAD_ARG, "jl_merge: part %d is not 16-byte aligned", i);
    p.o[i] = static_cast<const uint4*>(a->o[i]);
    p.lse[i] = a->lse[i];
  }
  if (reinterpret_cast<uintptr_t>(a->out) & 15) return fail(JL_ERR_BAD_ARG, "jl_merge: out is not 16-byte aligned");
  p.out = static_cast<uint4*>(a->out);
  p.lse_out = a->lse_out;
  p.n_parts = a->n_parts;
  p.rows = static_cast<int64_t>(a->batch) * a->seqlen * a->heads;
  p.seqlen = a->seqlen;
  p.heads = a->heads;
  p.round_like_reference = a->round_like_reference;
  if (p.rows == 0) return JL_OK;
  const int64_t blocks_needed = (p.rows + 15) / 16;
  const int grid = static_cast<int>(blocks_needed < 148 * 32 ? blocks_needed : 148 * 32);
  switch (a->round_like_reference ? 0 : a->n_parts) {
    case 2: merge_kernel<2><<<grid, 256, 0, stream>>>(p); break;
    case 4: merge_kernel<4><<<grid, 256, 0, stream>>>(p); break;
    case 8: merge_kernel<8><<<grid, 256, 0, stream>>>(p); break;
    default: merge_kernel<0><<<grid, 256, 0, stream>>>(p); break;
  }
  return check_launch("jl_merge");
}

}  // namespace jl

// Shared device/host helpers for the jetlong_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/jetlong_b200.h"

namespace jl {

constexpr int kHeadDim = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Host-side error reporting (thread-local detail string behind jl_last_error()).
void set_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);
int check_launch(const char* what);
int check_device_arch();

// ---------------------------------------------------------------------------------------------
// Small device helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  // bf16 -> fp32 is a 16-bit left shift
  float2 r;
  r.x = __uint_as_float(u << 16);
  r.y = __uint_as_float(u & 0xffff0000u);
  return r;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 16-byte async copy global -> shared; src_bytes == 0 zero-fills (used for rows past the end).
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` in a [rows][128 bf16] tile whose rows
// are 256 bytes; the chunk index is XOR-swizzled with the row so that 8 consecutive rows of one
// logical chunk land in 8 different bank groups (conflict-free ldmatrix).
__device__ __forceinline__ uint32_t swz256(int row, int chunk) {
  return static_cast<uint32_t>(row * 256 + ((chunk ^ (row & 7)) << 4));
}

// Absolute position of key row j of a (possibly block-cyclic) key tensor.
__device__ __host__ __forceinline__ int64_t key_position(int64_t j, int64_t pos0, int64_t block, int64_t block_stride) {
  if (block <= 0) return pos0 + j;
  return pos0 + (j / block) * block_stride + (j % block);
}

// sin/cos of an fp32 angle of any magnitude reached by RoPE positions (|theta| up to ~1e6 rad):
// two-constant Cody-Waite reduction by 2*pi.  The first FMA subtracts k * fl32(2*pi) with the product
// kept exact inside the FMA, so the cancellation costs nothing; the second adds back k times the
// representation error of fl32(2*pi).  The SFU approximations are then used on [-pi, pi] only.
__device__ __forceinline__ void sincos_reduced(float theta, float* s, float* c) {
  const float k = rintf(theta * 0.15915494309189535f);
  float r = fmaf(-k, 6.2831854820251465f, theta);
  r = fmaf(k, 1.7484555314695172e-7f, r);
  *s = __sinf(r);
  *c = __cosf(r);
}

// One head row of "per-head Qwen3RMSNorm -> base RoPE", for the lane that holds dims (2l, 2l+1) in lo and
// (64+2l, 64+2l+1) in hi.  Qwen3RMSNorm rounds the normalised value to bf16 before the (bf16) weight
// multiply; the rotation is fp32 and the caller rounds once when it stores.  Shared by the prefill-side
// pass and the decode-step kernel so that both produce the same bits.
__device__ __forceinline__ void norm_rope_head(float2 lo, float2 hi, float2 w_lo, float2 w_hi, float eps,
                                               float sb0, float cb0, float sb1, float cb1,
                                               float& bl0, float& bl1, float& bh0, float& bh1) {
  float ss = lo.x * lo.x + lo.y * lo.y + hi.x * hi.x + hi.y * hi.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  const float r = rsqrtf(ss * (1.f / 128.f) + eps);
  auto rb = [](float v) { return __bfloat162float(__float2bfloat16(v)); };
  const float y0 = rb(w_lo.x * rb(lo.x * r)), y1 = rb(w_lo.y * rb(lo.y * r));
  const float z0 = rb(w_hi.x * rb(hi.x * r)), z1 = rb(w_hi.y * rb(hi.y * r));
  bl0 = y0 * cb0 - z0 * sb0; bl1 = y1 * cb1 - z1 * sb1;
  bh0 = z0 * cb0 + y0 * sb0; bh1 = z1 * cb1 + y1 * sb1;
}

}  // namespace jl

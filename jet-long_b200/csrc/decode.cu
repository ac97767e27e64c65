// Split-KV single-token decode attention with GQA head packing — an HBM-streaming kernel.
//
// Grid (split, kv_head, batch); 4 warps per CTA.  The keys of all segments form one virtual
// sequence that is cut into `num_splits` contiguous ranges.  Each warp streams its own 16-row
// slices of 64-key K/V tiles through a private 3-stage cp.async pipeline (128-bit loads, rows read
// in place through the caller's strides, XOR-swizzled in shared memory), so warps never wait on
// one another.  The H/Hk query heads that share a kv head are packed into the M dimension of
// m16n8k16 tensor-core MMAs (rows past H/Hk are zero), scores go through a base-2 online softmax,
// and P.V accumulates in registers.  Far-class keys of a base-rotated cache can be regrouped on the
// fly (rotation by (floor(p/G) - p) * inv_freq in registers) so the cache is read exactly once.
// Each CTA writes one normalised fp32 partial (O, LSE) per query head.  The splits of a (batch, kv head)
// are merged by whichever of its CTAs finishes last: every CTA bumps an arrival counter after its
// partials are visible, and the one that sees splits - 1 merges (the partials are still in L2) and
// puts the counter back to zero.  Nothing spins, and there is no second launch.
#include "jl_common.cuh"

namespace jl {

constexpr int kDecWarps = 4;
constexpr int kDecTile = 64;                 // keys per tile (16 per warp)
constexpr int kDecStages = 3;
constexpr int kDecMaxSplits = 296;           // 2 resident CTAs on each of 148 SMs
constexpr int kStageBytes = kDecTile * 256;  // one K or V tile
constexpr int kDecMaxCounters = 4096;        // arrival counters at the head of the workspace: batch * kv_heads <= 4096
constexpr size_t kDecCounterBytes = kDecMaxCounters * sizeof(int);

struct DecSeg {
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  int64_t ks_b, ks_s, ks_h, vs_b, vs_s, vs_h;
  const int32_t* len_dev;
  const int64_t* row0_dev;
  int64_t pos0, pos_block, pos_block_stride;
  int len, q_class, rotate;
};

struct DecParams {
  const __nv_bfloat16* q[JL_MAX_CLASSES];
  int64_t qs_b, qs_h;
  DecSeg seg[JL_MAX_SEGMENTS];
  int n_seg, batch, heads, kv_heads, num_splits, group_size;
  float scale_log2;
  const float* inv_freq;
  float* part_o;     // (B, H, splits, 128)
  float* part_lse;   // (B, H, splits)
  int* arrivals;     // (B, Hk) arrival counters, zero between launches
  __nv_bfloat16* out;
  int64_t os_b, os_h;
  float* lse_out;    // (B, H) or NULL
};

struct DecSmem {
  uint8_t kv[kDecStages][2][kStageBytes];          // [stage][K/V][64 rows x 256 B]; reused for the warp merge
  uint8_t q[JL_MAX_CLASSES][16 * 256];
  float inv_freq[64];
};

// Merge the split partials of one (batch, head) with ONE WARP: every lane owns 4 of the 128 output dims
// (one 16-byte load per partial), lanes share the split weights by shuffle.  The partials were written by
// other SMs, so they are read through L2 (ld.cg), never from this SM's L1.
__device__ __forceinline__ void combine_head_warp(const float* part_o, const float* part_lse, int64_t base, int num_splits,
                                                  int lane, __nv_bfloat16* out_row, float* lse_out) {
  constexpr int kBatch = 16;               // independent 16-byte loads in flight per lane (the accumulators of the main loop are dead here)
  const float4* po = reinterpret_cast<const float4*>(part_o) + base * 32 + lane;       // 32 float4 per partial row
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  // the first batch of partial rows needs no weight yet: it travels together with the LSE values
  float4 x[kBatch];
#pragma unroll
  for (int k = 0; k < kBatch; ++k) x[k] = k < num_splits ? __ldcg(po + static_cast<int64_t>(k) * 32) : zero4;
  float m = -INFINITY;
  for (int s = lane; s < num_splits; s += 32) m = fmaxf(m, __ldcg(part_lse + base + s));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  const float ms = m == -INFINITY ? 0.f : m;
  float wsum = 0.f;
  float4 acc = zero4;
  for (int s0 = 0; s0 < num_splits; s0 += 32) {
    const int n = min(32, num_splits - s0);
    if (s0 > 0) {
#pragma unroll
      for (int k = 0; k < kBatch; ++k) x[k] = k < n ? __ldcg(po + static_cast<int64_t>(s0 + k) * 32) : zero4;
    }
    // weights of splits s0 .. s0 + 31: lane i holds the weight of split s0 + i (these LSE values were just read: L2 hits)
    const float w_mine = s0 + lane < num_splits ? exp2f((__ldcg(part_lse + base + s0 + lane) - ms) * kLog2e) : 0.f;
    for (int k0 = 0; k0 < n; k0 += kBatch) {
      float4 nx[kBatch];
#pragma unroll
      for (int k = 0; k < kBatch; ++k)     // next batch in flight while this one is folded in
        nx[k] = k0 + kBatch + k < n ? __ldcg(po + static_cast<int64_t>(s0 + k0 + kBatch + k) * 32) : zero4;
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        const float w = __shfl_sync(0xffffffffu, w_mine, (k0 + k) & 31);
        const float wk = k0 + k < n ? w : 0.f;
        wsum += wk;
        acc.x = fmaf(wk, x[k].x, acc.x); acc.y = fmaf(wk, x[k].y, acc.y);
        acc.z = fmaf(wk, x[k].z, acc.z); acc.w = fmaf(wk, x[k].w, acc.w);
      }
#pragma unroll
      for (int k = 0; k < kBatch; ++k) x[k] = nx[k];
    }
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  uint2 packed;
  packed.x = pack_bf16x2(acc.x * inv, acc.y * inv);
  packed.y = pack_bf16x2(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(out_row + lane * 4) = packed;
  if (lse_out != nullptr && lane == 0) *lse_out = wsum > 0.f ? ms + logf(wsum) : -INFINITY;
}

__global__ void __launch_bounds__(kDecWarps * 32, 2) decode_kernel(const DecParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  DecSmem& sm = *reinterpret_cast<DecSmem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int rep = p.heads / p.kv_heads;            // query heads per kv head (<= 16)

  // ---- this CTA's key range in the virtual concatenation of the segments ----
  int seg_len[JL_MAX_SEGMENTS];
  int64_t seg_row0[JL_MAX_SEGMENTS];      // first row of the segment inside its k / v tensors (device-side shift)
  int64_t total = 0;
#pragma unroll
  for (int s = 0; s < JL_MAX_SEGMENTS; ++s) {
    int len = 0;
    int64_t r0 = 0;
    if (s < p.n_seg) {
      len = p.seg[s].len;
      if (p.seg[s].len_dev != nullptr) len = min(len, max(p.seg[s].len_dev[b], 0));
      if (p.seg[s].row0_dev != nullptr) {        // never read past the rows the host described
        r0 = min(max(*p.seg[s].row0_dev, static_cast<int64_t>(0)), static_cast<int64_t>(p.seg[s].len));
        len = min(len, static_cast<int>(p.seg[s].len - r0));
      }
    }
    seg_len[s] = len;
    seg_row0[s] = r0;
    total += len;
  }
  int64_t per = (total + p.num_splits - 1) / p.num_splits;
  per = (per + kDecTile - 1) / kDecTile * kDecTile;
  const int64_t range_lo = min(static_cast<int64_t>(split) * per, total);
  const int64_t range_hi = min(range_lo + per, total);

  int seg_lo[JL_MAX_SEGMENTS], seg_tiles[JL_MAX_SEGMENTS], seg_hi[JL_MAX_SEGMENTS];
  int n_tiles = 0;
  {
    int64_t base = 0;
#pragma unroll
    for (int s = 0; s < JL_MAX_SEGMENTS; ++s) {
      const int64_t lo = max(range_lo, base) - base, hi = min(range_hi, base + seg_len[s]) - base;
      seg_lo[s] = static_cast<int>(lo);
      seg_hi[s] = static_cast<int>(hi);
      seg_tiles[s] = hi > lo ? static_cast<int>((hi - lo + kDecTile - 1) / kDecTile) : 0;
      n_tiles += seg_tiles[s];
      base += seg_len[s];
    }
  }

  auto locate = [&](int t, int& s_out, int& row0, int& valid) {
    int s = 0;
#pragma unroll
    for (int i = 0; i < JL_MAX_SEGMENTS - 1; ++i)
      if (s == i && t >= seg_tiles[i]) { t -= seg_tiles[i]; s = i + 1; }
    s_out = s;
    row0 = seg_lo[s] + t * kDecTile;
    valid = min(kDecTile, seg_hi[s] - row0);
  };
  auto shift_of = [&](int s) {
    int64_t r0 = seg_row0[0];
#pragma unroll
    for (int i = 1; i < JL_MAX_SEGMENTS; ++i) r0 = s == i ? seg_row0[i] : r0;
    return r0;
  };

  // Each warp copies rows [16*warp, 16*warp+16) of a tile: lane -> (row = lane/16 + 2*j, chunk = lane%16).
  auto issue = [&](int t) {
    if (t < n_tiles) {
      int s, row0, valid;
      locate(t, s, row0, valid);
      const DecSeg& sg = p.seg[s];
      const int64_t shift = shift_of(s);
      const int stage = t % kDecStages;
      const __nv_bfloat16* kb = sg.k + b * sg.ks_b + kvh * sg.ks_h;
      const __nv_bfloat16* vb = sg.v + b * sg.vs_b + kvh * sg.vs_h;
      const uint32_t ks = smem_u32(sm.kv[stage][0]), vs = smem_u32(sm.kv[stage][1]);
      const int chunk = lane & 15;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int r = warp * 16 + (lane >> 4) + 2 * j;
        const bool ok = r < valid;
        const int64_t grow = shift + (ok ? row0 + r : row0);      // keep the address in range when zero-filling
        cp_async_16(ks + swz256(r, chunk), kb + grow * sg.ks_s + chunk * 8, ok);
        cp_async_16(vs + swz256(r, chunk), vb + grow * sg.vs_s + chunk * 8, ok);
      }
    }
    cp_async_commit();
  };

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  // start streaming K/V before anything else: the first tiles' latency overlaps the query staging
#pragma unroll
  for (int t = 0; t < kDecStages - 1; ++t) issue(t);

  // ---- stage the packed query rows of every class (rows >= rep are zero) ----
  for (int i = threadIdx.x; i < JL_MAX_CLASSES * 16 * 16; i += blockDim.x) {
    const int c = i / 256, row = (i / 16) % 16, chunk = i % 16;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (p.q[c] != nullptr && row < rep)
      val = *reinterpret_cast<const uint4*>(p.q[c] + b * p.qs_b + (kvh * rep + row) * p.qs_h + chunk * 8);
    *reinterpret_cast<uint4*>(&sm.q[c][swz256(row, chunk)]) = val;
  }
  if (threadIdx.x < 64) sm.inv_freq[threadIdx.x] = p.inv_freq != nullptr ? p.inv_freq[threadIdx.x] : 0.f;

  __syncthreads();

  for (int t = 0; t < n_tiles; ++t) {
    cp_async_wait<kDecStages - 2>();
    __syncwarp();
    issue(t + kDecStages - 1);     // refills the stage consumed in the previous iteration (warp-private rows)

    int s, row0, valid;
    locate(t, s, row0, valid);
    const DecSeg& sg = p.seg[s];
    const int stage = t % kDecStages;
    const uint32_t ks = smem_u32(sm.kv[stage][0]), vs = smem_u32(sm.kv[stage][1]);
    const uint32_t qs = smem_u32(sm.q[sg.q_class]);
    const int wvalid = valid - warp * 16;           // valid keys among this warp's 16
    if (wvalid <= 0) continue;                      // warp-uniform

    // ---- K fragments for the warp's 16 keys: kf[kk] = {nblk0 k-lo, nblk0 k-hi, nblk1 k-lo, nblk1 k-hi} ----
    uint32_t kf[8][4];
    {
      const int r = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) ldmatrix_x4(kf[kk], ks + swz256(r, 2 * kk + ((lane >> 3) & 1)));
    }
    if (sg.rotate) {
      // element (key n, dim d) of kf[kk][i]: n = 8*(i/2) + lane/4, d = 16*kk + 8*(i%2) + 2*(lane%4) + {0,1};
      // its rotation partner d + 64 sits in kf[kk + 4][i].
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int64_t pos = key_position(shift_of(s) + row0 + warp * 16 + half * 8 + (lane >> 2), sg.pos0, sg.pos_block,
                                         sg.pos_block_stride);
        const float tf = static_cast<float>(pos / p.group_size - pos);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int i = half * 2 + e;
            const int d = 16 * kk + 8 * e + 2 * (lane & 3);
            float s0, c0, s1, c1;
            sincos_reduced(__fmul_rn(tf, sm.inv_freq[d]), &s0, &c0);
            sincos_reduced(__fmul_rn(tf, sm.inv_freq[d + 1]), &s1, &c1);
            const float2 lo = unpack_bf16x2(kf[kk][i]), hi = unpack_bf16x2(kf[kk + 4][i]);
            kf[kk][i] = pack_bf16x2(lo.x * c0 - hi.x * s0, lo.y * c1 - hi.y * s1);
            kf[kk + 4][i] = pack_bf16x2(hi.x * c0 + lo.x * s0, hi.y * c1 + lo.y * s1);
          }
        }
      }
    }

    // ---- S = Q K^T for 16 (packed head) rows x 16 keys ----
    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, qs + swz256(lane & 15, 2 * kk + (lane >> 4)));
      mma_bf16_16816(sc[0], a, kf[kk][0], kf[kk][1]);
      mma_bf16_16816(sc[1], a, kf[kk][2], kf[kk][3]);
    }

    // ---- online softmax (base 2); thread holds rows g = lane/4 (regs 0,1) and g + 8 (regs 2,3) ----
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = nb * 8 + 2 * (lane & 3) + (e & 1);
        const float v = key < wvalid ? sc[nb][e] * p.scale_log2 : -INFINITY;
        sc[nb][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;
      alpha[h] = fast_exp2(m_run[h] - m_use[h]);
      m_run[h] = m_new;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = fast_exp2(sc[nb][e] - m_use[e >> 1]);
        sc[nb][e] = pv;
        rs[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
      l_run[h] = l_run[h] * alpha[h] + rs[h];
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }

    // ---- O += P V ----
    uint32_t pa[4];
    pa[0] = pack_bf16x2(sc[0][0], sc[0][1]);
    pa[1] = pack_bf16x2(sc[0][2], sc[0][3]);
    pa[2] = pack_bf16x2(sc[1][0], sc[1][1]);
    pa[3] = pack_bf16x2(sc[1][2], sc[1][3]);
    {
      const int r = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, vs + swz256(r, 2 * j + (lane >> 4)));
        mma_bf16_16816(o[2 * j], pa, vf[0], vf[1]);
        mma_bf16_16816(o[2 * j + 1], pa, vf[2], vf[3]);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the 4 warps' states through shared memory (reusing the K/V stages) ----
  float* mo = reinterpret_cast<float*>(&sm.kv[0][0][0]);        // [warp][16 rows][128]
  float* mm = mo + kDecWarps * 16 * 128;                        // [warp][16]
  float* ml = mm + kDecWarps * 16;                              // [warp][16]
  {
    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float* dst = mo + (warp * 16 + g) * 128 + i * 8 + 2 * tq;
      dst[0] = o[i][0]; dst[1] = o[i][1];
      dst[8 * 128] = o[i][2]; dst[8 * 128 + 1] = o[i][3];
    }
    if (tq == 0) {
      mm[warp * 16 + g] = m_run[0]; mm[warp * 16 + g + 8] = m_run[1];
      ml[warp * 16 + g] = l_run[0]; ml[warp * 16 + g + 8] = l_run[1];
    }
  }
  __syncthreads();
  for (int row = 0; row < rep; ++row) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, mm[w * 16 + row]);
    const float Ms = M == -INFINITY ? 0.f : M;
    float L = 0.f, acc = 0.f;
    const int d = threadIdx.x;                                   // 128 threads == 128 dims
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float f = fast_exp2(mm[w * 16 + row] - Ms);
      L += ml[w * 16 + row] * f;
      acc += mo[(w * 16 + row) * 128 + d] * f;
    }
    const int head = kvh * rep + row;
    const int64_t pidx = (static_cast<int64_t>(b) * p.heads + head) * p.num_splits + split;
    p.part_o[pidx * 128 + d] = L > 0.f ? acc / L : 0.f;
    if (d == 0) p.part_lse[pidx] = L > 0.f ? (Ms + log2f(L)) * kLn2 : -INFINITY;
  }

  // ---- the last CTA of this (batch, kv head) to get here merges the splits ----
  __shared__ int s_last;
  __syncthreads();                       // every thread's partial writes are ordered before thread 0's fence
  if (threadIdx.x == 0) {
    __threadfence();                     // ... which makes them visible device-wide before the arrival is counted
    int* counter = p.arrivals + b * p.kv_heads + kvh;
    const int seen = atomicAdd(counter, 1);
    s_last = seen == p.num_splits - 1;
    if (s_last) {
      *counter = 0;                      // nobody else touches it until the next launch
      __threadfence();                   // the other CTAs' partials are visible to the reads below
    }
  }
  __syncthreads();
  if (!s_last) return;
  for (int row = warp; row < rep; row += kDecWarps) {       // one warp per query head
    const int head = kvh * rep + row;
    const int64_t bh = static_cast<int64_t>(b) * p.heads + head;
    combine_head_warp(p.part_o, p.part_lse, bh * p.num_splits, p.num_splits, lane, p.out + b * p.os_b + head * p.os_h,
                      p.lse_out != nullptr ? p.lse_out + bh : nullptr);
  }
}

// ---------------------------------------------------------------------------------------------
// The same decode for calls that regroup far keys inside the kernel, re-gridded so that the rotation
// angles are formed once per key instead of once per key and kv head.
//
// The angle (floor(p / G) - p) * inv_freq[d] of a far key depends on its position and the frequency, not on
// the head.  Here one CTA owns a key range for EIGHT kv heads of a batch row: grid (split, kv_heads / 8,
// batch), 8 warps, warp w streams the keys of kv head 8 * blockIdx.y + w through its own 3-stage cp.async
// pipeline, 16 keys per step, all warps on the same 16 keys.  The 256 threads form the (sin, cos) of the NEXT
// step's 16 keys x 64 frequencies together (4 per thread instead of 32) into a double-buffered table in
// shared memory; one CTA barrier per step orders the table hand-over.  Every warp owns its head's whole key
// range, so there is no cross-warp merge; the splits are merged by decode_combine_kernel.
// ---------------------------------------------------------------------------------------------
constexpr int kWideWarps = 8;                // kv heads per CTA
constexpr int kWideTile = 16;                // keys per step
constexpr int kWideMaxSplits = 148;          // one CTA per SM
constexpr int kWideScRow = 72;               // float2 per table row: 64 used, padded so that 8 lanes x 16 B never share a bank

struct WideSmem {
  uint8_t kv[kWideWarps][kDecStages][2][kWideTile * 256];      // [warp][stage][K/V][16 rows x 256 B]
  uint8_t q[kWideWarps][8 * 256];                              // the (<= 8) query rows of the class in use, per kv head
  float2 sc[2][kWideTile][kWideScRow];                         // (sin, cos) per key and frequency of the current / next step
  float inv_freq[64];
};

__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}

__global__ void __launch_bounds__(kWideWarps * 32, 1) decode_wide_kernel(const DecParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  WideSmem& sm = *reinterpret_cast<WideSmem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kvh = blockIdx.y * kWideWarps + warp, b = blockIdx.z;
  const int rep = p.heads / p.kv_heads;            // query heads per kv head (<= 8 here)

  // ---- this CTA's key range in the virtual concatenation of the segments (as in decode_kernel, 16-key steps) ----
  int seg_len[JL_MAX_SEGMENTS];
  int64_t seg_row0[JL_MAX_SEGMENTS];
  int64_t total = 0;
#pragma unroll
  for (int s = 0; s < JL_MAX_SEGMENTS; ++s) {
    int len = 0;
    int64_t r0 = 0;
    if (s < p.n_seg) {
      len = p.seg[s].len;
      if (p.seg[s].len_dev != nullptr) len = min(len, max(p.seg[s].len_dev[b], 0));
      if (p.seg[s].row0_dev != nullptr) {
        r0 = min(max(*p.seg[s].row0_dev, static_cast<int64_t>(0)), static_cast<int64_t>(p.seg[s].len));
        len = min(len, static_cast<int>(p.seg[s].len - r0));
      }
    }
    seg_len[s] = len;
    seg_row0[s] = r0;
    total += len;
  }
  int64_t per = (total + p.num_splits - 1) / p.num_splits;
  per = (per + kWideTile - 1) / kWideTile * kWideTile;
  const int64_t range_lo = min(static_cast<int64_t>(split) * per, total);
  const int64_t range_hi = min(range_lo + per, total);
  int seg_lo[JL_MAX_SEGMENTS], seg_tiles[JL_MAX_SEGMENTS], seg_hi[JL_MAX_SEGMENTS];
  int n_tiles = 0;
  {
    int64_t base = 0;
#pragma unroll
    for (int s = 0; s < JL_MAX_SEGMENTS; ++s) {
      const int64_t lo = max(range_lo, base) - base, hi = min(range_hi, base + seg_len[s]) - base;
      seg_lo[s] = static_cast<int>(lo);
      seg_hi[s] = static_cast<int>(hi);
      seg_tiles[s] = hi > lo ? static_cast<int>((hi - lo + kWideTile - 1) / kWideTile) : 0;
      n_tiles += seg_tiles[s];
      base += seg_len[s];
    }
  }
  auto locate = [&](int t, int& s_out, int& row0, int& valid) {
    int s = 0;
#pragma unroll
    for (int i = 0; i < JL_MAX_SEGMENTS - 1; ++i)
      if (s == i && t >= seg_tiles[i]) { t -= seg_tiles[i]; s = i + 1; }
    s_out = s;
    row0 = seg_lo[s] + t * kWideTile;
    valid = min(kWideTile, seg_hi[s] - row0);
  };
  auto shift_of = [&](int s) {
    int64_t r0 = seg_row0[0];
#pragma unroll
    for (int i = 1; i < JL_MAX_SEGMENTS; ++i) r0 = s == i ? seg_row0[i] : r0;
    return r0;
  };

  // the warp copies the 16 rows of a step for ITS kv head: lane -> (row = lane/16 + 2*j, chunk = lane%16)
  auto issue = [&](int t) {
    if (t < n_tiles) {
      int s, row0, valid;
      locate(t, s, row0, valid);
      const DecSeg& sg = p.seg[s];
      const int64_t shift = shift_of(s);
      const int stage = t % kDecStages;
      const __nv_bfloat16* kb = sg.k + b * sg.ks_b + kvh * sg.ks_h;
      const __nv_bfloat16* vb = sg.v + b * sg.vs_b + kvh * sg.vs_h;
      const uint32_t ks = smem_u32(sm.kv[warp][stage][0]), vs = smem_u32(sm.kv[warp][stage][1]);
      const int chunk = lane & 15;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int r = (lane >> 4) + 2 * j;
        const bool ok = r < valid;
        const int64_t grow = shift + (ok ? row0 + r : row0);      // keep the address in range when zero-filling
        cp_async_16(ks + swz256(r, chunk), kb + grow * sg.ks_s + chunk * 8, ok);
        cp_async_16(vs + swz256(r, chunk), vb + grow * sg.vs_s + chunk * 8, ok);
      }
    }
    cp_async_commit();
  };
  // All 256 threads: (sin, cos) of step t's 16 keys x 64 frequencies (only for a rotating segment).  Thread -> one key
  // and four consecutive frequencies, so one position and one division by G per thread.  The values are formed in
  // registers BEFORE the step's barrier (the wait for the slowest warp hides their latency) and stored after it.
  const int tab_key = threadIdx.x >> 4, tab_d0 = (threadIdx.x & 15) * 4;
  auto table_values = [&](int t, float4& a, float4& b2) -> bool {
    if (t >= n_tiles) return false;
    int s, row0, valid;
    locate(t, s, row0, valid);
    const DecSeg& sg = p.seg[s];
    if (!sg.rotate) return false;
    const int64_t pos = key_position(shift_of(s) + row0 + tab_key, sg.pos0, sg.pos_block, sg.pos_block_stride);
    const int64_t grouped = (pos >= 0 && pos < (int64_t(1) << 31))
                                ? static_cast<int64_t>(static_cast<uint32_t>(pos) / static_cast<uint32_t>(p.group_size))
                                : pos / p.group_size;
    const float tf = static_cast<float>(grouped - pos);
    sincos_reduced(__fmul_rn(tf, sm.inv_freq[tab_d0 + 0]), &a.x, &a.y);
    sincos_reduced(__fmul_rn(tf, sm.inv_freq[tab_d0 + 1]), &a.z, &a.w);
    sincos_reduced(__fmul_rn(tf, sm.inv_freq[tab_d0 + 2]), &b2.x, &b2.y);
    sincos_reduced(__fmul_rn(tf, sm.inv_freq[tab_d0 + 3]), &b2.z, &b2.w);
    return true;
  };
  auto table_store = [&](int t, const float4& a, const float4& b2) {
    float4* dst = reinterpret_cast<float4*>(&sm.sc[t & 1][tab_key][tab_d0]);
    dst[0] = a;
    dst[1] = b2;
  };

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run = -INFINITY, l_run = 0.f;             // rows 0..7 of the packed query heads (rows 8..15 are padding)

#pragma unroll
  for (int t = 0; t < kDecStages - 1; ++t) issue(t);
  if (threadIdx.x < 64) sm.inv_freq[threadIdx.x] = p.inv_freq != nullptr ? p.inv_freq[threadIdx.x] : 0.f;
  __syncthreads();
  {
    float4 a, b2;
    if (table_values(0, a, b2)) table_store(0, a, b2);
  }
  int q_loaded = -1;

  for (int t = 0; t < n_tiles; ++t) {
    float4 tab_a, tab_b;
    const bool tab_next = table_values(t + 1, tab_a, tab_b);
    __syncthreads();               // table t is complete; nobody still reads the buffer table t + 1 goes to
    if (tab_next) table_store(t + 1, tab_a, tab_b);
    cp_async_wait<kDecStages - 2>();
    __syncwarp();
    issue(t + kDecStages - 1);     // refills the stage consumed in the previous iteration (warp-private)

    int s, row0, valid;
    locate(t, s, row0, valid);
    const DecSeg& sg = p.seg[s];
    if (sg.q_class != q_loaded) {  // the query rows of this segment's class, for this warp's kv head (warp-private tile)
      __syncwarp();
      for (int i = lane; i < 8 * 16; i += 32) {
        const int row = i >> 4, chunk = i & 15;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (row < rep) val = *reinterpret_cast<const uint4*>(p.q[sg.q_class] + b * p.qs_b + (kvh * rep + row) * p.qs_h + chunk * 8);
        *reinterpret_cast<uint4*>(&sm.q[warp][swz256(row, chunk)]) = val;
      }
      q_loaded = sg.q_class;
      __syncwarp();
    }
    const int stage = t % kDecStages;
    const uint32_t ks = smem_u32(sm.kv[warp][stage][0]), vs = smem_u32(sm.kv[warp][stage][1]);
    const uint32_t qs = smem_u32(sm.q[warp]);

    // ---- K fragments of the 16 keys: kf[kk] = {nblk0 k-lo, nblk0 k-hi, nblk1 k-lo, nblk1 k-hi} ----
    uint32_t kf[8][4];
    {
      const int r = (lane & 7) + ((lane >> 4) << 3);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) ldmatrix_x4(kf[kk], ks + swz256(r, 2 * kk + ((lane >> 3) & 1)));
    }
    if (sg.rotate) {
      // element (key n, dim d) of kf[kk][i]: n = 8*(i/2) + lane/4, d = 16*kk + 8*(i%2) + 2*(lane%4) + {0,1};
      // its rotation partner d + 64 sits in kf[kk + 4][i].  (sin, cos) of (n, d) and (n, d + 1): one 16-byte read.
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const float2* row = sm.sc[t & 1][half * 8 + (lane >> 2)];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int i = half * 2 + e;
            const int d = 16 * kk + 8 * e + 2 * (lane & 3);
            const float4 t4 = *reinterpret_cast<const float4*>(row + d);      // sin d, cos d, sin d+1, cos d+1
            const float2 lo = unpack_bf16x2(kf[kk][i]), hi = unpack_bf16x2(kf[kk + 4][i]);
            kf[kk][i] = pack_bf16x2(lo.x * t4.y - hi.x * t4.x, lo.y * t4.w - hi.y * t4.z);
            kf[kk + 4][i] = pack_bf16x2(hi.x * t4.y + lo.x * t4.x, hi.y * t4.w + lo.y * t4.z);
          }
        }
      }
    }

    // ---- S = Q K^T for 8 (packed head) rows x 16 keys; rows 8..15 of the A fragment are zero ----
    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      uint32_t a[4] = {0u, 0u, 0u, 0u};
      ldmatrix_x2(a[0], a[2], qs + swz256(lane & 7, 2 * kk + ((lane >> 3) & 1)));
      mma_bf16_16816(sc[0], a, kf[kk][0], kf[kk][1]);
      mma_bf16_16816(sc[1], a, kf[kk][2], kf[kk][3]);
    }

    // ---- online softmax (base 2); the thread holds row lane/4 in regs 0,1 of each n-block ----
    float mx = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = nb * 8 + 2 * (lane & 3) + e;
        const float v = key < valid ? sc[nb][e] * p.scale_log2 : -INFINITY;
        sc[nb][e] = v;
        mx = fmaxf(mx, v);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    const float alpha = fast_exp2(m_run - m_use);
    m_run = m_new;
    float rs = 0.f;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float pv = fast_exp2(sc[nb][e] - m_use);
        sc[nb][e] = pv;
        rs += pv;
      }
    }
    rs += __shfl_xor_sync(0xffffffffu, rs, 1);
    rs += __shfl_xor_sync(0xffffffffu, rs, 2);
    l_run = l_run * alpha + rs;
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i][0] *= alpha; o[i][1] *= alpha; }

    // ---- O += P V (rows 8..15 of P are zero) ----
    uint32_t pa[4];
    pa[0] = pack_bf16x2(sc[0][0], sc[0][1]);
    pa[1] = 0u;
    pa[2] = pack_bf16x2(sc[1][0], sc[1][1]);
    pa[3] = 0u;
    {
      const int r = (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, vs + swz256(r, 2 * j + (lane >> 4)));
        mma_bf16_16816(o[2 * j], pa, vf[0], vf[1]);
        mma_bf16_16816(o[2 * j + 1], pa, vf[2], vf[3]);
      }
    }
  }
  cp_async_wait<0>();

  // ---- one normalised fp32 partial (O, LSE) per query head of this warp's kv head ----
  const int g = lane >> 2, tq = lane & 3;
  if (g < rep) {
    const int head = kvh * rep + g;
    const int64_t pidx = (static_cast<int64_t>(b) * p.heads + head) * p.num_splits + split;
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i)
      *reinterpret_cast<float2*>(p.part_o + pidx * 128 + i * 8 + 2 * tq) = make_float2(o[i][0] * inv, o[i][1] * inv);
    if (tq == 0) p.part_lse[pidx] = l_run > 0.f ? ((m_run == -INFINITY ? 0.f : m_run) + log2f(l_run)) * kLn2 : -INFINITY;
  }
}

// Merges the splits of the wide kernel: one warp per (batch, head).
__global__ void __launch_bounds__(128) decode_combine_kernel(const DecParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x * 4 + warp, b = blockIdx.y;
  if (head >= p.heads) return;
  const int64_t bh = static_cast<int64_t>(b) * p.heads + head;
  combine_head_warp(p.part_o, p.part_lse, bh * p.num_splits, p.num_splits, lane, p.out + b * p.os_b + head * p.os_h,
                    p.lse_out != nullptr ? p.lse_out + bh : nullptr);
}

int32_t decode_auto_splits(int32_t batch, int32_t kv_heads, int64_t total_keys) {
  const int64_t ctas = static_cast<int64_t>(batch > 0 ? batch : 1) * (kv_heads > 0 ? kv_heads : 1);
  int64_t s = kDecMaxSplits / ctas;
  const int64_t tiles = (total_keys + kDecTile - 1) / kDecTile;
  if (s > tiles) s = tiles;
  if (s < 1) s = 1;
  return static_cast<int32_t>(s);
}

size_t decode_workspace_bytes(int32_t batch, int32_t heads, int32_t head_dim, int32_t max_splits) {
  if (batch <= 0 || heads <= 0 || head_dim <= 0) return 0;
  const size_t splits = max_splits > 0 ? static_cast<size_t>(max_splits) : static_cast<size_t>(kDecMaxSplits);
  return kDecCounterBytes + static_cast<size_t>(batch) * heads * splits * (static_cast<size_t>(head_dim) + 1) * sizeof(float);
}

// Calls that regroup far keys in-kernel go to the kernel that forms each rotation angle once for eight kv heads.
static bool decode_uses_wide_kernel(const jl_decode_args* a) {
  if (a->kv_heads <= 0 || a->kv_heads % kWideWarps != 0 || a->heads % a->kv_heads != 0 || a->heads / a->kv_heads > 8) return false;
  for (int s = 0; s < a->n_segments && s < JL_MAX_SEGMENTS; ++s)
    if (a->seg[s].rotate != 0 && a->seg[s].len > 0) return true;
  return false;
}

// The split count of a call (the caller's, or enough CTAs to fill the GPU), never more than there are key tiles.
static int decode_plan_splits(const jl_decode_args* a, int64_t total, bool wide) {
  int64_t splits, tiles;
  if (wide) {
    const int64_t ctas = static_cast<int64_t>(a->batch) * (a->kv_heads / kWideWarps);
    splits = a->num_splits > 0 ? a->num_splits : kWideMaxSplits / (ctas > 0 ? ctas : 1);
    tiles = (total + kWideTile - 1) / kWideTile;
  } else {
    splits = a->num_splits > 0 ? a->num_splits : decode_auto_splits(a->batch, a->kv_heads, total);
    tiles = (total + kDecTile - 1) / kDecTile;
  }
  if (splits > tiles) splits = tiles;
  if (splits > kDecMaxSplits) splits = kDecMaxSplits;
  return static_cast<int>(splits > 0 ? splits : 1);
}

int launch_decode(const jl_decode_args* a, cudaStream_t stream) {
  if (a->head_dim != kHeadDim) return fail(JL_ERR_UNSUPPORTED, "jl_decode: head_dim must be 128, got %d", a->head_dim);
  if (a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0) return fail(JL_ERR_BAD_ARG, "jl_decode: batch/heads/kv_heads must be positive");
  if (a->heads % a->kv_heads != 0) return fail(JL_ERR_BAD_ARG, "jl_decode: heads must be divisible by kv_heads");
  if (a->heads / a->kv_heads > 16) return fail(JL_ERR_UNSUPPORTED, "jl_decode: at most 16 query heads per kv head");
  if (static_cast<int64_t>(a->batch) * a->kv_heads > kDecMaxCounters)
    return fail(JL_ERR_UNSUPPORTED, "jl_decode: batch * kv_heads must be at most %d", kDecMaxCounters);
  if (a->n_segments < 1 || a->n_segments > JL_MAX_SEGMENTS) return fail(JL_ERR_BAD_ARG, "jl_decode: n_segments must be in [1, %d]", JL_MAX_SEGMENTS);
  if (a->out == nullptr) return fail(JL_ERR_BAD_ARG, "jl_decode: out is NULL");
  if (a->q_stride_b % 8 || a->q_stride_h % 8) return fail(JL_ERR_BAD_ARG, "jl_decode: q strides must be multiples of 8 elements");
  if ((reinterpret_cast<uintptr_t>(a->out) & 7) || a->o_stride_b % 4 || a->o_stride_h % 4)
    return fail(JL_ERR_BAD_ARG, "jl_decode: out must be 8-byte aligned with strides that are multiples of 4 elements");
  DecParams p{};
  int64_t total = 0;
  bool any_rotate = false;
  for (int c = 0; c < JL_MAX_CLASSES; ++c) {
    if (reinterpret_cast<uintptr_t>(a->q[c]) & 15) return fail(JL_ERR_BAD_ARG, "jl_decode: q[%d] is not 16-byte aligned", c);
    p.q[c] = static_cast<const __nv_bfloat16*>(a->q[c]);
  }
  for (int s = 0; s < a->n_segments; ++s) {
    const jl_kv_segment& g = a->seg[s];
    if (g.len < 0) return fail(JL_ERR_BAD_ARG, "jl_decode: segment %d has negative length", s);
    if (g.q_class < 0 || g.q_class >= JL_MAX_CLASSES || a->q[g.q_class] == nullptr)
      return fail(JL_ERR_BAD_ARG, "jl_decode: segment %d names a missing query operand", s);
    if (g.len > 0 && (g.k == nullptr || g.v == nullptr)) return fail(JL_ERR_BAD_ARG, "jl_decode: segment %d has NULL k/v", s);
    if ((reinterpret_cast<uintptr_t>(g.k) | reinterpret_cast<uintptr_t>(g.v)) & 15)
      return fail(JL_ERR_BAD_ARG, "jl_decode: segment %d k/v not 16-byte aligned", s);
    const int64_t st[] = {g.k_stride_b, g.k_stride_s, g.k_stride_h, g.v_stride_b, g.v_stride_s, g.v_stride_h};
    for (int64_t x : st)
      if (x % 8 != 0) return fail(JL_ERR_BAD_ARG, "jl_decode: segment %d strides must be multiples of 8 elements", s);
    DecSeg& d = p.seg[s];
    d.k = static_cast<const __nv_bfloat16*>(g.k);
    d.v = static_cast<const __nv_bfloat16*>(g.v);
    d.ks_b = g.k_stride_b; d.ks_s = g.k_stride_s; d.ks_h = g.k_stride_h;
    d.vs_b = g.v_stride_b; d.vs_s = g.v_stride_s; d.vs_h = g.v_stride_h;
    d.len_dev = g.len_dev;
    d.row0_dev = g.row0_dev;
    d.pos0 = g.pos0;
    d.pos_block = g.pos_block > 0 ? g.pos_block : 0;
    d.pos_block_stride = g.pos_block_stride;
    if (d.pos_block % 8 != 0) return fail(JL_ERR_BAD_ARG, "jl_decode: segment %d pos_block must be a multiple of 8", s);
    d.len = g.len;
    d.q_class = g.q_class;
    d.rotate = g.rotate != 0;
    any_rotate |= g.rotate != 0;
    total += g.len;
  }
  if (any_rotate && (a->inv_freq == nullptr || a->group_size < 1))
    return fail(JL_ERR_BAD_ARG, "jl_decode: rotating segments need inv_freq and group_size >= 1");
  const bool wide = decode_uses_wide_kernel(a);
  const int splits = decode_plan_splits(a, total, wide);
  const size_t need = decode_workspace_bytes(a->batch, a->heads, a->head_dim, splits);
  if (a->workspace == nullptr || a->workspace_bytes < need)
    return fail(JL_ERR_WORKSPACE, "jl_decode: workspace of %zu bytes needed, %zu given", need, a->workspace_bytes);
  if (reinterpret_cast<uintptr_t>(a->workspace) & 15) return fail(JL_ERR_BAD_ARG, "jl_decode: workspace not 16-byte aligned");
  p.qs_b = a->q_stride_b; p.qs_h = a->q_stride_h;
  p.n_seg = a->n_segments; p.batch = a->batch; p.heads = a->heads; p.kv_heads = a->kv_heads;
  p.num_splits = splits;
  p.group_size = a->group_size > 0 ? a->group_size : 1;
  p.scale_log2 = a->softmax_scale * kLog2e;
  p.inv_freq = a->inv_freq;
  p.arrivals = static_cast<int*>(a->workspace);
  p.part_o = reinterpret_cast<float*>(static_cast<uint8_t*>(a->workspace) + kDecCounterBytes);
  p.part_lse = p.part_o + static_cast<size_t>(a->batch) * a->heads * splits * kHeadDim;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.os_b = a->o_stride_b; p.os_h = a->o_stride_h;
  p.lse_out = a->lse;

  // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute
  static bool attr_set[64] = {false};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(JL_ERR_LAUNCH, "jl_decode: no current CUDA device");
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(DecSmem))) != cudaSuccess ||
        cudaFuncSetAttribute(decode_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(WideSmem))) != cudaSuccess)
      return check_launch("jl_decode (shared memory opt-in)");
    attr_set[dev] = true;
  }
  if (wide) {
    dim3 grid(splits, a->kv_heads / kWideWarps, a->batch);
    decode_wide_kernel<<<grid, kWideWarps * 32, sizeof(WideSmem), stream>>>(p);
    const int rc = check_launch("jl_decode (shared-angle kernel)");
    if (rc != JL_OK) return rc;
    dim3 cgrid((a->heads + 3) / 4, a->batch);
    decode_combine_kernel<<<cgrid, 128, 0, stream>>>(p);
    return check_launch("jl_decode (combine)");
  }
  dim3 grid(splits, a->kv_heads, a->batch);
  decode_kernel<<<grid, kDecWarps * 32, sizeof(DecSmem), stream>>>(p);
  return check_launch("jl_decode");
}

// ---------------------------------------------------------------------------------------------
// Decode with built-in scratch: for callers that are not allowed to allocate device memory.
//
// The split-KV partials normally live in a workspace the caller allocates.  Some callers cannot do
// that: a serving process that hands all of its device memory to one arena at start-up and forbids
// any later cudaMalloc (an allocation there can fail, fragment the arena's neighbour, or stall every
// stream of the device while the driver services it), or a plug-in that only receives raw input and
// output pointers from its host and owns no allocator at all.  For them the scratch is this fixed
// array inside the library image (zero when the image is loaded, which is what the arrival counters at
// its head need; the kernel puts them back to zero).  It costs kStaticScratchBytes on every GPU that loads the library,
// for the life of the process, whether or not this entry point is ever used.
// ---------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = size_t(4) << 20;      // 4 MiB: 16 KB of arrival counters + partials for B * H * splits <= 8096 at head_dim 128
static __device__ __align__(256) float g_decode_scratch[kStaticScratchBytes / sizeof(float)];

int launch_decode_static(const jl_decode_args* a, cudaStream_t stream) {
  // In host code `g_decode_scratch` is only a handle for the runtime, not a device pointer, so the
  // device address is looked up once per device (with that device current) and cached.
  static float* device_addr[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(JL_ERR_LAUNCH, "jl_decode_static: no current CUDA device");
  if (device_addr[dev] == nullptr) {
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_decode_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(JL_ERR_LAUNCH, "jl_decode_static: cannot resolve the built-in scratch array: %s", cudaGetErrorString(e));
    device_addr[dev] = ptr;
  }
  if (a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->n_segments < 1 || a->n_segments > JL_MAX_SEGMENTS)
    return fail(JL_ERR_BAD_ARG, "jl_decode_static: batch/heads/kv_heads/n_segments out of range");
  int64_t total = 0;
  for (int s = 0; s < a->n_segments; ++s) total += a->seg[s].len > 0 ? a->seg[s].len : 0;
  const int splits = decode_plan_splits(a, total, decode_uses_wide_kernel(a));
  const size_t need = decode_workspace_bytes(a->batch, a->heads, a->head_dim, splits);
  if (need > kStaticScratchBytes)
    return fail(JL_ERR_WORKSPACE,
                "jl_decode_static: batch %d x heads %d x %d splits needs %zu bytes of scratch but the built-in array holds %zu; "
                "lower num_splits or the batch, or use jl_decode with a caller-provided workspace",
                a->batch, a->heads, splits, need, kStaticScratchBytes);
  jl_decode_args with_scratch = *a;
  with_scratch.num_splits = splits;
  with_scratch.workspace = device_addr[dev];
  with_scratch.workspace_bytes = kStaticScratchBytes;
  return launch_decode(&with_scratch, stream);
}

size_t decode_static_scratch_bytes() { return kStaticScratchBytes; }

}  // namespace jl

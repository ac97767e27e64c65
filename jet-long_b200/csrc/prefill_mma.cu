// Position-mapped causal prefill attention on the legacy warp-level tensor path (mma.sync).
//
// This is the first-generation kernel: correct for every position map, tile shape and stride the
// API accepts, and kept as the on-GPU cross-check for the tcgen05 kernel (impl = 1 in
// jl_prefill_args).  One CTA = 128 query rows of one head (8 warps x 16 rows); K/V stream in
// 64-key tiles through a double-buffered cp.async pipeline.  Per (q-tile, k-tile) the classes
// present are derived arithmetically from the tile's position bounds; a tile crossed by a class
// boundary computes one QK^T per class present and selects per element before the shared online
// softmax, so one pass covers near and far fields with no second kernel and no packed 2S tensors.
#include "jl_common.cuh"

namespace jl {

constexpr int kPfM = 128, kPfN = 64, kPfWarps = 8;
constexpr int kQTileBytes = kPfM * 256, kKTileBytes = kPfN * 256;

struct PfParams {
  const __nv_bfloat16* q[JL_MAX_CLASSES];
  const __nv_bfloat16* k[JL_MAX_CLASSES];
  const __nv_bfloat16* v;
  __nv_bfloat16* out;
  float* lse;
  int64_t qs_b, qs_s, qs_h, ks_b, ks_s, ks_h, vs_b, vs_s, vs_h, os_b, os_s, os_h;
  int batch, sq, sk, heads, kv_heads;
  int64_t q_pos0, k_pos0, k_block, k_block_stride, q_block, q_block_stride;
  float scale_log2;
  int map_kind, n_classes;
  int64_t near_span, chunk;
  int k_slot[JL_MAX_CLASSES];     // which of the (at most two) distinct key tensors class c reads
  int n_k_slots;
};

__device__ __forceinline__ int class_of(int kind, int64_t pq, int64_t pk, int64_t near_span, int64_t chunk) {
  if (pk > pq) return -1;
  if (kind == JL_MAP_BAND) return (pq - pk <= near_span) ? 0 : 1;
  const int64_t cd = pq / chunk - pk / chunk;
  return cd < 2 ? static_cast<int>(cd) : 2;
}

__global__ void __launch_bounds__(kPfWarps * 32, 1) prefill_mma_kernel(const PfParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  // layout: Q[n_classes][32 KB] | stage0: K[n_k_slots][16 KB], V[16 KB] | stage1: ...
  uint8_t* sq = smem;
  const int stage_bytes = (p.n_k_slots + 1) * kKTileBytes;
  uint8_t* sstage = smem + p.n_classes * kQTileBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;              // heaviest (latest) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.heads / p.kv_heads);
  const int q0 = qt * kPfM;
  const int q_valid = min(kPfM, p.sq - q0);
  // a 128-row query tile never straddles a position block (q_block is a multiple of 256)
  const int64_t pq_first = key_position(q0, p.q_pos0, p.q_block, p.q_block_stride), pq_last = pq_first + q_valid - 1;

  // ---- Q tiles of every class (zero-filled past the end) ----
  for (int c = 0; c < p.n_classes; ++c) {
    const __nv_bfloat16* qb = p.q[c] + b * p.qs_b + h * p.qs_h;
    const uint32_t dst = smem_u32(sq + c * kQTileBytes);
    for (int i = threadIdx.x; i < kPfM * 16; i += blockDim.x) {
      const int row = i >> 4, chunk = i & 15;
      const bool ok = row < q_valid;
      cp_async_16(dst + swz256(row, chunk), qb + static_cast<int64_t>(ok ? q0 + row : q0) * p.qs_s + chunk * 8, ok);
    }
  }
  cp_async_commit();

  // ---- key tiles this CTA visits: those whose first position is <= the last query position ----
  const int n_ktiles_all = (p.sk + kPfN - 1) / kPfN;
  int n_ktiles = 0;
  for (int j = 0; j < n_ktiles_all; ++j) {     // positions are monotone in j; short scalar loop
    if (key_position(static_cast<int64_t>(j) * kPfN, p.k_pos0, p.k_block, p.k_block_stride) > pq_last) break;
    n_ktiles = j + 1;
  }

  // classes present in tile j (bit c), and whether any element needs per-element treatment
  auto classify = [&](int j, uint32_t& present, bool& uniform) {
    const int kv_valid = min(kPfN, p.sk - j * kPfN);
    const int64_t kp_first = key_position(static_cast<int64_t>(j) * kPfN, p.k_pos0, p.k_block, p.k_block_stride);
    const int64_t kp_last = kp_first + kv_valid - 1;
    present = 0;
    if (p.map_kind == JL_MAP_BAND) {
      const int64_t dmin = pq_first - kp_last, dmax = pq_last - kp_first;
      if (dmax >= 0 && dmin <= p.near_span) present |= 1u;
      if (dmax > p.near_span) present |= 2u;
    } else {
      const int64_t lo = pq_first / p.chunk - kp_last / p.chunk, hi = pq_last / p.chunk - kp_first / p.chunk;
      for (int64_t cd = (lo < 0 ? 0 : lo); cd <= hi && cd <= 2; ++cd) present |= 1u << cd;
      if (hi >= 2) present |= 4u;
    }
    const bool one_class = (present & (present - 1)) == 0;
    uniform = one_class && kp_last <= pq_first && kv_valid == kPfN;
  };

  auto load_tile = [&](int j, int stage) {
    if (j < n_ktiles) {
      uint32_t present; bool uniform;
      classify(j, present, uniform);
      const int kv_valid = min(kPfN, p.sk - j * kPfN);
      uint8_t* st = sstage + stage * stage_bytes;
      bool slot_done[2] = {false, false};
      for (int c = 0; c < p.n_classes; ++c) {
        if (!(present >> c & 1u)) continue;
        const int slot = p.k_slot[c];
        if (slot_done[slot]) continue;
        slot_done[slot] = true;
        const __nv_bfloat16* kb = p.k[c] + b * p.ks_b + kvh * p.ks_h;
        const uint32_t dst = smem_u32(st + slot * kKTileBytes);
        for (int i = threadIdx.x; i < kPfN * 16; i += blockDim.x) {
          const int row = i >> 4, chunk = i & 15;
          const bool ok = row < kv_valid;
          cp_async_16(dst + swz256(row, chunk), kb + static_cast<int64_t>(j * kPfN + (ok ? row : 0)) * p.ks_s + chunk * 8, ok);
        }
      }
      const __nv_bfloat16* vb = p.v + b * p.vs_b + kvh * p.vs_h;
      const uint32_t dst = smem_u32(st + p.n_k_slots * kKTileBytes);
      for (int i = threadIdx.x; i < kPfN * 16; i += blockDim.x) {
        const int row = i >> 4, chunk = i & 15;
        const bool ok = row < kv_valid;
        cp_async_16(dst + swz256(row, chunk), vb + static_cast<int64_t>(j * kPfN + (ok ? row : 0)) * p.vs_s + chunk * 8, ok);
      }
    }
    cp_async_commit();
  };

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int g = lane >> 2, tq = lane & 3;
  const int64_t pq_row[2] = {pq_first + warp * 16 + g, pq_first + warp * 16 + g + 8};

  load_tile(0, 0);
  for (int j = 0; j < n_ktiles; ++j) {
    const int stage = j & 1;
    load_tile(j + 1, stage ^ 1);     // the other stage was released by the barrier ending iteration j-1
    cp_async_wait<1>();
    __syncthreads();

    uint32_t present; bool uniform;
    classify(j, present, uniform);
    const int kv_valid = min(kPfN, p.sk - j * kPfN);
    const int64_t kp_first = key_position(static_cast<int64_t>(j) * kPfN, p.k_pos0, p.k_block, p.k_block_stride);
    uint8_t* st = sstage + stage * stage_bytes;

    float sel[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) { sel[nb][0] = sel[nb][1] = sel[nb][2] = sel[nb][3] = -INFINITY; }

    for (int c = 0; c < p.n_classes; ++c) {
      if (!(present >> c & 1u)) continue;
      float tmp[8][4];
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) { tmp[nb][0] = tmp[nb][1] = tmp[nb][2] = tmp[nb][3] = 0.f; }
      const uint32_t qs = smem_u32(sq + c * kQTileBytes);
      const uint32_t ks = smem_u32(st + p.k_slot[c] * kKTileBytes);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, qs + swz256(warp * 16 + (lane & 15), 2 * kk + (lane >> 4)));
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t kf[4];
          ldmatrix_x4(kf, ks + swz256(16 * np + (lane & 7) + ((lane >> 4) << 3), 2 * kk + ((lane >> 3) & 1)));
          mma_bf16_16816(tmp[2 * np], a, kf[0], kf[1]);
          mma_bf16_16816(tmp[2 * np + 1], a, kf[2], kf[3]);
        }
      }
      if (uniform) {
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
          for (int e = 0; e < 4; ++e) sel[nb][e] = tmp[nb][e] * p.scale_log2;
        }
      } else {
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = nb * 8 + 2 * tq + (e & 1);
            const int cls = col < kv_valid ? class_of(p.map_kind, pq_row[e >> 1], kp_first + col, p.near_span, p.chunk) : -1;
            if (cls == c) sel[nb][e] = tmp[nb][e] * p.scale_log2;
          }
        }
      }
    }

    // ---- online softmax over the 64 keys of this tile ----
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], sel[nb][e]);
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;
      alpha[r] = fast_exp2(m_run[r] - m_use[r]);
      m_run[r] = m_new;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = fast_exp2(sel[nb][e] - m_use[e >> 1]);
        sel[nb][e] = pv;
        rs[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
      l_run[r] = l_run[r] * alpha[r] + rs[r];
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }

    // ---- O += P V ----
    const uint32_t vs = smem_u32(st + p.n_k_slots * kKTileBytes);
#pragma unroll
    for (int ks16 = 0; ks16 < 4; ++ks16) {
      uint32_t pa[4];
      pa[0] = pack_bf16x2(sel[2 * ks16][0], sel[2 * ks16][1]);
      pa[1] = pack_bf16x2(sel[2 * ks16][2], sel[2 * ks16][3]);
      pa[2] = pack_bf16x2(sel[2 * ks16 + 1][0], sel[2 * ks16 + 1][1]);
      pa[3] = pack_bf16x2(sel[2 * ks16 + 1][2], sel[2 * ks16 + 1][3]);
      const int r = 16 * ks16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
      for (int jd = 0; jd < 8; ++jd) {
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, vs + swz256(r, 2 * jd + (lane >> 4)));
        mma_bf16_16816(o[2 * jd], pa, vf[0], vf[1]);
        mma_bf16_16816(o[2 * jd + 1], pa, vf[2], vf[3]);
      }
    }
    __syncthreads();                 // everyone is done with this stage before it is refilled
  }
  cp_async_wait<0>();

  // ---- epilogue ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + 8 * r;
    if (row >= q_valid) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    __nv_bfloat16* orow = p.out + b * p.os_b + static_cast<int64_t>(q0 + row) * p.os_s + h * p.os_h;
#pragma unroll
    for (int i = 0; i < 16; ++i)
      *reinterpret_cast<uint32_t*>(orow + i * 8 + 2 * tq) = pack_bf16x2(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    if (p.lse != nullptr && tq == 0)
      p.lse[(static_cast<int64_t>(b) * p.heads + h) * p.sq + q0 + row] =
          l_run[r] > 0.f ? (m_run[r] + log2f(l_run[r])) * kLn2 : -INFINITY;
  }
}

int launch_prefill_mma(const jl_prefill_args* a, cudaStream_t stream) {
  PfParams p{};
  int n_slots = 0;
  const void* slot_ptr[2] = {nullptr, nullptr};
  for (int c = 0; c < a->map.n_classes; ++c) {
    p.q[c] = static_cast<const __nv_bfloat16*>(a->q[c]);
    p.k[c] = static_cast<const __nv_bfloat16*>(a->k[c]);
    int slot = -1;
    for (int s = 0; s < n_slots; ++s)
      if (slot_ptr[s] == a->k[c]) slot = s;
    if (slot < 0) {
      if (n_slots == 2) return fail(JL_ERR_UNSUPPORTED, "jl_prefill: at most two distinct key operands");
      slot_ptr[n_slots] = a->k[c];
      slot = n_slots++;
    }
    p.k_slot[c] = slot;
  }
  p.n_k_slots = n_slots;
  p.v = static_cast<const __nv_bfloat16*>(a->v);
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.qs_b = a->q_stride_b; p.qs_s = a->q_stride_s; p.qs_h = a->q_stride_h;
  p.ks_b = a->k_stride_b; p.ks_s = a->k_stride_s; p.ks_h = a->k_stride_h;
  p.vs_b = a->v_stride_b; p.vs_s = a->v_stride_s; p.vs_h = a->v_stride_h;
  p.os_b = a->o_stride_b; p.os_s = a->o_stride_s; p.os_h = a->o_stride_h;
  p.batch = a->batch; p.sq = a->seqlen_q; p.sk = a->seqlen_k; p.heads = a->heads; p.kv_heads = a->kv_heads;
  p.q_pos0 = a->q_pos0; p.k_pos0 = a->k_pos0;
  p.k_block = (a->k_block > 0 && a->k_block < a->seqlen_k) ? a->k_block : 0;
  p.k_block_stride = a->k_block_stride;
  p.q_block = (a->q_block > 0 && a->q_block < a->seqlen_q) ? a->q_block : 0;
  p.q_block_stride = a->q_block_stride;
  if (p.q_block % 256 != 0) return fail(JL_ERR_UNSUPPORTED, "jl_prefill: q_block must be a multiple of 256");
  if (p.k_block > 0 && p.k_block % kPfN != 0)
    return fail(JL_ERR_UNSUPPORTED, "jl_prefill: k_block must be a multiple of %d", kPfN);
  p.scale_log2 = a->softmax_scale * kLog2e;
  p.map_kind = a->map.kind; p.n_classes = a->map.n_classes;
  p.near_span = a->map.near_span; p.chunk = a->map.chunk > 0 ? a->map.chunk : 1;
  const int smem = p.n_classes * kQTileBytes + 2 * (n_slots + 1) * kKTileBytes;
  if (cudaFuncSetAttribute(prefill_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * kQTileBytes + 6 * kKTileBytes) != cudaSuccess)
    return check_launch("jl_prefill (shared memory opt-in)");
  dim3 grid((a->seqlen_q + kPfM - 1) / kPfM, a->heads, a->batch);
  prefill_mma_kernel<<<grid, kPfWarps * 32, smem, stream>>>(p);
  return check_launch("jl_prefill (mma.sync)");
}

}  // namespace jl

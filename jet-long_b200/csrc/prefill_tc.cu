// Single-pass position-mapped causal prefill attention on the Blackwell tensor path:
// TMA-staged tiles -> tcgen05.mma (QK^T from shared memory, PV with P in tensor memory) -> TMEM
// accumulators, one online softmax carried across every position class.
//
// CTA = 256 query rows of one head = two 128-row query tiles that ping-pong on the tensor pipe.
//   warp 0      TMA producer (Q tiles of the current class, K ring of 3, V ring of 2; 128B swizzle)
//   warp 1      MMA issuer (one elected thread): S_t = Q_t K_j^T (SS), O_t += P_t V_j (TS)
//   warp 2      TMEM allocator (all 512 columns: S0 | S1 | O0 | O1; P_t overlays the first 64 columns of S_t)
//   warps 4-7   softmax of query tile 0: one thread per row (= TMEM lane), 128 scores in registers
//   warps 8-11  softmax of query tile 1
// Position map: the classes are processed as PHASES.  In phase c the CTA holds the class-c query
// operand in shared memory and visits only the key tiles in which class c occurs for some of its
// rows; per row, the keys of class c inside a tile form one column interval, so the mask is two
// integer compares and tiles strictly inside a class need none.  A key tile crossed by a class
// boundary is simply visited in both phases with complementary masks; the running (max, sum, O)
// state is shared, so there is no second QK^T accumulator, no select, and no merge pass.
// Rescaling of O is lazy: it happens only when a row maximum grows by more than 2^8.
// Every wait is bounded; a wait that gives up sets a status word and lets the kernel drain.
#include <cuda.h>
#include <cstdio>

#include "jl_common.cuh"


namespace jl {

namespace tc {

constexpr int kTileM = 128, kTileN = 128, kRowsPerCta = 256;
constexpr int kKStages = 3, kVStages = 2;
constexpr int kTileBytes = 128 * 256;           // 128 rows x 128 bf16
constexpr int kHalfBytes = 128 * 128;           // one 64-column half (a TMA box)
constexpr int kThreads = 384;
constexpr int kRegsLow = 72, kRegsHigh = 216;   // per-role register budgets; 128 x 72 + 256 x 216 = the launch total 384 x 168
// Build-time diagnostics for timing experiments only (results are wrong): 1 = exponentials replaced by the identity,
// 2 = the softmax warps only hand the barriers on, 4 = scores are loaded and their maximum taken, nothing else,
// 5 = per-role clock counters of CTA 0 printed, 6 = as 2 and the K / V rings are filled only once, 7 = as 2 without Q K^T.
#ifndef JL_DIAG
#define JL_DIAG 0
#endif
#ifndef JL_POLY_MASK
#define JL_POLY_MASK 0x11
#endif
// Which of every 8 consecutive score pairs take the FMA-pipe exp2 (bit i = pair i); the rest use the SFU.
// The set is spread evenly so that SFU instructions are separated by FMA-pipe work in program order.
constexpr unsigned kPolyMask = JL_POLY_MASK;
constexpr int64_t kNegInfPos = -(int64_t(1) << 60);

struct Params {
  int sq, sk, heads, kv_heads, batch;
  int64_t q_pos0, k_pos0, k_block, k_block_stride, q_block, q_block_stride;
  float scale_log2;
  int map_kind, n_classes;
  int64_t near_span, chunk;
  int k_map[JL_MAX_CLASSES];      // index into the distinct key tensor maps
  __nv_bfloat16* out;
  float* lse;
  int64_t os_b, os_s, os_h;
  int* status;                    // device status word (0 = ok)
  // In-kernel remap of the far class (BAND map): class 1 reads the class-0 tensors and warps 2-3 rotate every
  // landed tile in shared memory by (floor(p / group_size) - p) * inv_freq before the tensor pipe reads it.
  int remap, group_size;
  int head_group;                 // query heads whose CTAs are interleaved along grid x (heaviest rows first across all of them)
  // Stripe batching: with batch_wrap > 0 grid z = i addresses batch element (batch_first + i) % batch_wrap of q, out and
  // lse, whose rows start at position q_pos0 + element * q_pos0_batch_step; every element reads batch element 0 of k / v.
  int batch_first, batch_wrap;
  int64_t q_pos0_batch_step;
  const float* inv_freq;
};

struct Maps {
  CUtensorMap q[JL_MAX_CLASSES];
  CUtensorMap k[2];
  CUtensorMap v;
};

struct Smem {
  alignas(1024) uint8_t q[2][kTileBytes];
  alignas(1024) uint8_t k[kKStages][kTileBytes];
  alignas(1024) uint8_t v[kVStages][kTileBytes];
  uint64_t q_full, q_free, k_full[kKStages], k_empty[kKStages], v_full[kVStages], v_empty[kVStages];
  uint64_t s_full[2], p_half[2][2], all_done;     // p_half[t][h]: probabilities of keys 64h..64h+63 of tile t are in TMEM
  uint64_t q_ready, k_ready[kKStages];            // in-kernel remap only: the tile has been rotated (or needs no rotation)
  uint32_t tmem_base;
  int failed;
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  A wait that has not been satisfied after kWaitLimitNs (1 s) gives up and raises the CTA's
// `failed` flag; from then on every wait of the CTA returns at once, so the kernel drains instead of
// hanging (its output is then invalid and the status word tells the host).  CTAs that start after
// the device status word has been raised skip their waits from the beginning.
constexpr uint64_t kWaitLimitNs = 1000ull * 1000 * 1000;      // 1 s: far beyond any legitimate wait, even on a time-sliced GPU
template <class SmemT>
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, SmemT& sm) {
  if (mbar_try_wait(bar, parity)) return;
  volatile int* failed = reinterpret_cast<volatile int*>(&sm.failed);
  if (*failed) return;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return;
    if (*failed) return;
    if (globaltimer_ns() - t0 > kWaitLimitNs) { *failed = 1; return; }
  }
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  // start address | leading byte offset | stride byte offset | version 1 (sm_100) | 128-byte swizzle
  return static_cast<uint64_t>((saddr >> 4) & 0x3FFF) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// kind::f16 instruction descriptor: fp32 accumulate, bf16 A and B, M x N tile
__device__ __host__ constexpr uint32_t instr_desc(int m, int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

#define JL_R32(r, o) "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7]), \
  "=r"(r[o + 8]), "=r"(r[o + 9]), "=r"(r[o + 10]), "=r"(r[o + 11]), "=r"(r[o + 12]), "=r"(r[o + 13]), "=r"(r[o + 14]), "=r"(r[o + 15]), \
  "=r"(r[o + 16]), "=r"(r[o + 17]), "=r"(r[o + 18]), "=r"(r[o + 19]), "=r"(r[o + 20]), "=r"(r[o + 21]), "=r"(r[o + 22]), "=r"(r[o + 23]), \
  "=r"(r[o + 24]), "=r"(r[o + 25]), "=r"(r[o + 26]), "=r"(r[o + 27]), "=r"(r[o + 28]), "=r"(r[o + 29]), "=r"(r[o + 30]), "=r"(r[o + 31])
#define JL_W32(r, o) "r"(r[o + 0]), "r"(r[o + 1]), "r"(r[o + 2]), "r"(r[o + 3]), "r"(r[o + 4]), "r"(r[o + 5]), "r"(r[o + 6]), "r"(r[o + 7]), \
  "r"(r[o + 8]), "r"(r[o + 9]), "r"(r[o + 10]), "r"(r[o + 11]), "r"(r[o + 12]), "r"(r[o + 13]), "r"(r[o + 14]), "r"(r[o + 15]), \
  "r"(r[o + 16]), "r"(r[o + 17]), "r"(r[o + 18]), "r"(r[o + 19]), "r"(r[o + 20]), "r"(r[o + 21]), "r"(r[o + 22]), "r"(r[o + 23]), \
  "r"(r[o + 24]), "r"(r[o + 25]), "r"(r[o + 26]), "r"(r[o + 27]), "r"(r[o + 28]), "r"(r[o + 29]), "r"(r[o + 30]), "r"(r[o + 31])
#define JL_TMEM_LD32(taddr, r, o)                                                                                          \
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18," \
               "%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"                                               \
               : JL_R32(r, o) : "r"(taddr))
#define JL_TMEM_ST32(taddr, r, o)                                                                                          \
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17," \
               "%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"                                              \
               ::"r"(taddr), JL_W32(r, o) : "memory")
#define JL_TMEM_ST16(taddr, r, o)                                                                                          \
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"     \
               ::"r"(taddr), "r"(r[o + 0]), "r"(r[o + 1]), "r"(r[o + 2]), "r"(r[o + 3]), "r"(r[o + 4]), "r"(r[o + 5]),       \
                 "r"(r[o + 6]), "r"(r[o + 7]), "r"(r[o + 8]), "r"(r[o + 9]), "r"(r[o + 10]), "r"(r[o + 11]), "r"(r[o + 12]), \
                 "r"(r[o + 13]), "r"(r[o + 14]), "r"(r[o + 15]) : "memory")
// ---- packed fp32 pairs (one instruction per two lanes of work) and the FMA-pipe exp2 ----
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add2_round_down(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rm.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 2^x for a pair, on the FMA and integer pipes only (the SFU is the co-bottleneck of attention at
// head_dim 128).  x = n + f with n = floor(x) taken from a round-down add of 1.5 * 2^23 (n then
// sits in the low mantissa bits), f in [0, 1); 2^f by a cubic with equi-ripple relative error
// 7.5e-5 (fitted for this file; the result feeds a bf16 rounding of relative step 3.9e-3);
// 2^n is applied by adding n to the exponent field.  x is clamped at -126 so the exponent cannot wrap.
__device__ __forceinline__ uint64_t exp2_pair_fma(uint64_t x) {
  float x0, x1;
  unpack2(x, x0, x1);
  x = pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const uint64_t magic = pack2(12582912.f, 12582912.f);
  const uint64_t t = add2_round_down(x, magic);
  const uint64_t f = sub2(x, sub2(t, magic));
  uint64_t q = fma2(pack2(0.07802429050207138f, 0.07802429050207138f), f, pack2(0.22606779634952545f, 0.22606779634952545f));
  q = fma2(q, f, pack2(0.695833146572113f, 0.695833146572113f));
  q = fma2(q, f, pack2(0.9999252557754517f, 0.9999252557754517f));
  float t0, t1, q0, q1;
  unpack2(t, t0, t1);
  unpack2(q, q0, q1);
  return pack2(__uint_as_float(__float_as_uint(t0) * 8388608u + __float_as_uint(q0)),      // (n << 23) + bits: one IMAD
               __uint_as_float(__float_as_uint(t1) * 8388608u + __float_as_uint(q1)));
}
__device__ __forceinline__ uint64_t exp2_pair_sfu(uint64_t x) {
  float x0, x1;
  unpack2(x, x0, x1);
  return pack2(fast_exp2(x0), fast_exp2(x1));
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// Position-map arithmetic shared by all roles
// ---------------------------------------------------------------------------------------------
// Inclusive range of key POSITIONS that belong to class c for a query at position pq.
__device__ __forceinline__ void class_interval(const Params& p, int c, int64_t pq, int64_t& lo, int64_t& hi) {
  if (p.map_kind == JL_MAP_BAND) {
    if (c == 0) { lo = pq - p.near_span; hi = pq; }
    else        { lo = kNegInfPos;       hi = pq - p.near_span - 1; }
  } else {
    const int64_t cs = pq / p.chunk * p.chunk;
    if (c == 0)      { lo = cs;           hi = pq; }
    else if (c == 1) { lo = cs - p.chunk; hi = cs - 1; }
    else             { lo = kNegInfPos;   hi = cs - p.chunk - 1; }
  }
}
// First local key row whose position is >= pos, and last local row whose position is <= pos
// (rows are laid out in blocks of k_block positions every k_block_stride positions; k_block == 0: contiguous).
__device__ __forceinline__ int64_t row_at_or_after(const Params& p, int64_t pos) {
  const int64_t rel = pos - p.k_pos0;
  if (rel <= 0) return 0;
  if (p.k_block <= 0) return rel;
  const int64_t b = rel / p.k_block_stride, off = rel - b * p.k_block_stride;
  return off < p.k_block ? b * p.k_block + off : (b + 1) * p.k_block;
}
__device__ __forceinline__ int64_t row_at_or_before(const Params& p, int64_t pos) {
  const int64_t rel = pos - p.k_pos0;
  if (rel < 0) return -1;
  if (p.k_block <= 0) return rel;
  const int64_t b = rel / p.k_block_stride, off = rel - b * p.k_block_stride;
  return off < p.k_block ? b * p.k_block + off : b * p.k_block + p.k_block - 1;
}

struct Schedule {
  int n_phases;
  int cls[JL_MAX_CLASSES], j_lo[JL_MAX_CLASSES], n_tiles[JL_MAX_CLASSES];
  int total;
};

__device__ __forceinline__ Schedule make_schedule(const Params& p, int q_row0, int64_t q_pos0) {
  Schedule s;
  s.n_phases = 0;
  s.total = 0;
  const int rows = min(kRowsPerCta, p.sq - q_row0);
  // the CTA's 256 rows never straddle a position block (q_block is a multiple of 256)
  const int64_t pq_first = key_position(q_row0, q_pos0, p.q_block, p.q_block_stride), pq_last = pq_first + rows - 1;
  for (int c = p.n_classes - 1; c >= 0; --c) {       // far classes first, the diagonal last
    int64_t lo, hi, dummy;
    class_interval(p, c, pq_first, lo, dummy);
    class_interval(p, c, pq_last, dummy, hi);
    if (hi < lo) continue;
    int64_t r_lo = row_at_or_after(p, lo), r_hi = row_at_or_before(p, hi);
    if (r_hi > p.sk - 1) r_hi = p.sk - 1;
    if (r_lo > r_hi) continue;
    const int i = s.n_phases++;
    s.cls[i] = c;
    s.j_lo[i] = static_cast<int>(r_lo / kTileN);
    s.n_tiles[i] = static_cast<int>(r_hi / kTileN) - s.j_lo[i] + 1;
    s.total += s.n_tiles[i];
  }
  return s;
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1) prefill_tc_kernel(const __grid_constant__ Maps maps, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid x = (query tile pair, head within the group), the latest (heaviest) rows first over the whole group of heads
  const int q_tile_pair = static_cast<int>(gridDim.x / p.head_group) - 1 - static_cast<int>(blockIdx.x / p.head_group);
  const int head = blockIdx.y * p.head_group + static_cast<int>(blockIdx.x % p.head_group);
  const int b = p.batch_wrap > 0 ? (p.batch_first + static_cast<int>(blockIdx.z)) % p.batch_wrap : static_cast<int>(blockIdx.z);
  const int b_kv = p.batch_wrap > 0 ? 0 : b;
  const int64_t q_pos0 = p.q_pos0 + b * p.q_pos0_batch_step;
  const int kvh = head / (p.heads / p.kv_heads);
  const int q_row0 = q_tile_pair * kRowsPerCta;
  const Schedule sched = make_schedule(p, q_row0, q_pos0);

  if (threadIdx.x == 0) {
    sm.failed = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    mbar_init(&sm.q_full, 1);
    mbar_init(&sm.q_free, 1);
    for (int i = 0; i < kKStages; ++i) { mbar_init(&sm.k_full[i], 1); mbar_init(&sm.k_empty[i], 1); }
    for (int i = 0; i < kVStages; ++i) { mbar_init(&sm.v_full[i], 1); mbar_init(&sm.v_empty[i], 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(&sm.s_full[t], 1); mbar_init(&sm.p_half[t][0], 128); mbar_init(&sm.p_half[t][1], 128); }
    mbar_init(&sm.all_done, 1);
    mbar_init(&sm.q_ready, 64);
    for (int i = 0; i < kKStages; ++i) mbar_init(&sm.k_ready[i], 64);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  // Register budget per role: the data-movement warpgroup gives registers back, the two softmax
  // warpgroups (one thread per row, 128 scores live) take them.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLow));
  if (warp == 0) {
    // ===================================== TMA producer =====================================
    if (lane == 0) {
      int g = 0;
      for (int ph = 0; ph < sched.n_phases; ++ph) {
        const int c = sched.cls[ph];
        // the query tiles of this class replace the previous class's once its QK^T MMAs have retired
        mbar_wait(&sm.q_free, (ph & 1) ^ 1, sm);
        mbar_expect_tx(&sm.q_full, 2 * kTileBytes);
        for (int t = 0; t < 2; ++t)
          for (int h = 0; h < 2; ++h)
            tma_load_4d(sm.q[t] + h * kHalfBytes, &maps.q[c], &sm.q_full, h * 64, head, q_row0 + t * kTileM, b);
        const CUtensorMap* km = &maps.k[p.k_map[c]];
        for (int jj = 0; jj < sched.n_tiles[ph]; ++jj, ++g) {
          const int row = (sched.j_lo[ph] + jj) * kTileN;
          const int ks = g % kKStages, vs = g % kVStages;
          mbar_wait(&sm.k_empty[ks], ((g / kKStages) & 1) ^ 1, sm);
#if JL_DIAG == 6
          if (g >= kKStages) mbar_arrive(&sm.k_full[ks]); else {      // timing experiment: the ring is filled once, never again
#endif
          mbar_expect_tx(&sm.k_full[ks], kTileBytes);
          for (int h = 0; h < 2; ++h) tma_load_4d(sm.k[ks] + h * kHalfBytes, km, &sm.k_full[ks], h * 64, kvh, row, b_kv);
#if JL_DIAG == 6
          }
#endif
          mbar_wait(&sm.v_empty[vs], ((g / kVStages) & 1) ^ 1, sm);
#if JL_DIAG == 6
          if (g >= kVStages) mbar_arrive(&sm.v_full[vs]); else {
#endif
          mbar_expect_tx(&sm.v_full[vs], kTileBytes);
          for (int h = 0; h < 2; ++h) tma_load_4d(sm.v[vs] + h * kHalfBytes, &maps.v, &sm.v_full[vs], h * 64, kvh, row, b_kv);
#if JL_DIAG == 6
          }
#endif
        }
      }
    }
  } else if (warp == 1) {
    // ====================================== MMA issuer ======================================
    // The whole warp walks the schedule so that barrier parities, ring indices and descriptors are
    // warp-uniform values; one elected lane issues the tcgen05 instructions and their commits.
    if (sched.total > 0) {
      uint32_t leader;
      asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(leader));
      const uint32_t idesc_qk = instr_desc(kTileM, kTileN, 0);
      const uint32_t idesc_pv = instr_desc(kTileM, kHeadDim, 1);
      const uint64_t q_desc0 = smem_desc(smem_u32(sm.q[0]), 16, 1024);
      const uint64_t k_desc0 = smem_desc(smem_u32(sm.k[0]), 16, 1024);
      const uint64_t v_desc0 = smem_desc(smem_u32(sm.v[0]), kHalfBytes, 1024);
      auto issue_qk = [&](int t, int g) {
        const int ks = g % kKStages;
        const uint64_t qd = q_desc0 + static_cast<uint64_t>((t * kTileBytes) >> 4);
        const uint64_t kd = k_desc0 + static_cast<uint64_t>((ks * kTileBytes) >> 4);
        if (leader) {
#if JL_DIAG != 7
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t off = static_cast<uint64_t>(((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4);
            mma_ss(tmem + t * 128, qd + off, kd + off, idesc_qk, kk > 0);
          }
#endif
          mma_commit(&sm.s_full[t]);
        }
      };
#if JL_DIAG == 5
      long long w_p[2][2] = {{0, 0}, {0, 0}}, w_k = 0, w_v = 0;
      const long long t_begin = clock64();
#define JL_TIMED(acc, stmt) { const long long t0_ = clock64(); stmt; acc += clock64() - t0_; }
#else
#define JL_TIMED(acc, stmt) { stmt; }
#endif
      int g = 0;           // global tile counter (K/V ring index, barrier parities)
      for (int ph = 0; ph < sched.n_phases; ++ph) {
        uint64_t* const q_bar = p.remap ? &sm.q_ready : &sm.q_full;           // with the in-kernel remap the tiles pass
        uint64_t* const k_bar = p.remap ? sm.k_ready : sm.k_full;             // through warps 2-3 first
        mbar_wait(q_bar, ph & 1, sm);
        const int n = sched.n_tiles[ph];
        mbar_wait(&k_bar[g % kKStages], (g / kKStages) & 1, sm);
        tc_fence_after();
        issue_qk(0, g);
        issue_qk(1, g);
        if (leader) {
          if (n == 1) mma_commit(&sm.q_free);
          mma_commit(&sm.k_empty[g % kKStages]);
        }
        for (int jj = 0; jj < n; ++jj, ++g) {
          const int vs = g % kVStages;
          const bool more = jj + 1 < n;
          const uint64_t vd = v_desc0 + static_cast<uint64_t>((vs * kTileBytes) >> 4);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            // the softmax warps publish P in two halves so that the first four k-steps of P V overlap
            // the exponentials of the second half
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              JL_TIMED(w_p[t][h], mbar_wait(&sm.p_half[t][h], g & 1, sm));
              if (t == 0 && h == 0) JL_TIMED(w_v, mbar_wait(&sm.v_full[vs], (g / kVStages) & 1, sm));
              tc_fence_after();
              if (leader) {
#pragma unroll
                for (int kk = 4 * h; kk < 4 * h + 4; ++kk)
                  mma_ts(tmem + 256 + t * 128, tmem + t * 128 + kk * 8, vd + static_cast<uint64_t>((kk * 2048) >> 4), idesc_pv,
                         (g > 0 || kk > 0) ? 1u : 0u);
                if (t == 1 && h == 1) mma_commit(&sm.v_empty[vs]);
              }
            }
            if (more) {
              const int gn = g + 1;
              if (t == 0) { JL_TIMED(w_k, mbar_wait(&k_bar[gn % kKStages], (gn / kKStages) & 1, sm)); tc_fence_after(); }
              issue_qk(t, gn);
              if (t == 1 && leader) {
                if (jj + 2 == n) mma_commit(&sm.q_free);       // last QK^T of this phase issued
                mma_commit(&sm.k_empty[gn % kKStages]);
              }
            }
          }
        }
      }
      if (leader) mma_commit(&sm.all_done);
      __syncwarp();
#if JL_DIAG == 5
      if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && g > 0)
        printf("mma warp: %d tiles, %lld clk/tile; waits per tile: P00 %lld P01 %lld P10 %lld P11 %lld K %lld V %lld\n", g,
               (clock64() - t_begin) / g, w_p[0][0] / g, w_p[0][1] / g, w_p[1][0] / g, w_p[1][1] / g, w_k / g, w_v / g);
#endif
    }
  } else if (p.remap) {
    // =========================== in-kernel remap of the far class ===========================
    // Warps 2-3 (64 threads).  Far phase: the query tiles and every key tile arrive base-rotated (the class-0
    // tensors) and are rotated here, in shared memory, to the remapped position floor(p / G): each thread takes
    // a 16-byte chunk (8 dims) of a row in the low half and the matching chunk of the high half (rotate-half
    // pairs d <-> d + 64), with the angle fp32(floor(p / G) - p) * inv_freq[d] formed exactly as jl_rotate does.
    // Other phases: the tiles are passed on untouched.  Generic-proxy writes are fenced for the tensor pipe.
    const int tid = threadIdx.x - 64;
    auto rotate_tile = [&](uint8_t* tile, int64_t row_pos0, int64_t block, int64_t block_stride, int64_t row0, int rows) {
      for (int idx = tid; idx < 128 * 8; idx += 64) {
        const int r = idx >> 3, ch = idx & 7;
        if (r >= rows) continue;
        const int64_t pos = key_position(row0 + r, row_pos0, block, block_stride);
        const float tf = static_cast<float>(pos / p.group_size - pos);
        uint8_t* lo_ptr = tile + r * 128 + ((ch ^ (r & 7)) << 4);
        uint4 lo = *reinterpret_cast<uint4*>(lo_ptr), hi = *reinterpret_cast<uint4*>(lo_ptr + kHalfBytes);
        uint32_t* lw = reinterpret_cast<uint32_t*>(&lo);
        uint32_t* hw = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int d = ch * 8 + 2 * j;
          float s0, c0, s1, c1;
          sincos_reduced(__fmul_rn(tf, __ldg(p.inv_freq + d)), &s0, &c0);
          sincos_reduced(__fmul_rn(tf, __ldg(p.inv_freq + d + 1)), &s1, &c1);
          const float2 l = unpack_bf16x2(lw[j]), h = unpack_bf16x2(hw[j]);
          lw[j] = pack_bf16x2(l.x * c0 - h.x * s0, l.y * c1 - h.y * s1);
          hw[j] = pack_bf16x2(h.x * c0 + l.x * s0, h.y * c1 + l.y * s1);
        }
        *reinterpret_cast<uint4*>(lo_ptr) = lo;
        *reinterpret_cast<uint4*>(lo_ptr + kHalfBytes) = hi;
      }
    };
    if (warp >= 2) {
      int g = 0;
      for (int ph = 0; ph < sched.n_phases; ++ph) {
        const bool far = sched.cls[ph] == 1;
        mbar_wait(&sm.q_full, ph & 1, sm);
        if (far) {
          for (int t = 0; t < 2; ++t)
            rotate_tile(sm.q[t], q_pos0, p.q_block, p.q_block_stride, q_row0 + t * kTileM, min(kTileM, max(p.sq - (q_row0 + t * kTileM), 0)));
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        mbar_arrive(&sm.q_ready);
        for (int jj = 0; jj < sched.n_tiles[ph]; ++jj, ++g) {
          const int ks = g % kKStages;
          mbar_wait(&sm.k_full[ks], (g / kKStages) & 1, sm);
          if (far) {
            const int64_t row0 = static_cast<int64_t>(sched.j_lo[ph] + jj) * kTileN;
            rotate_tile(sm.k[ks], p.k_pos0, p.k_block, p.k_block_stride, row0, static_cast<int>(min(static_cast<int64_t>(kTileN), p.sk - row0)));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          }
          mbar_arrive(&sm.k_ready[ks]);
        }
      }
    }
  }
  } else {
    // ================================ softmax + epilogue ================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsHigh));
    const int t = (warp - 4) >> 2;                          // query tile 0 / 1
    const int quad = warp & 3;                              // TMEM lane quadrant this warp may access
    const int row_in_tile = quad * 32 + lane;
    const int q_row = q_row0 + t * kTileM + row_in_tile;
    const bool row_valid = q_row < p.sq;
    const int64_t pq_cta0 = key_position(q_row0, q_pos0, p.q_block, p.q_block_stride);     // position of the CTA's first row
    const int64_t pq = pq_cta0 + (row_valid ? q_row : p.sq - 1) - q_row0;
    // bounds of this tile's valid rows, for the uniform-tile test
    const int tile_rows = min(kTileM, p.sq - (q_row0 + t * kTileM));
    const int64_t pq_t0 = pq_cta0 + t * kTileM;
    const int64_t pq_t1 = pq_t0 + (tile_rows > 0 ? tile_rows - 1 : 0);
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem + lane_base + t * 128;        // my row of scores; the bf16 P overlays its first 64 columns
    const uint32_t t_o = tmem + lane_base + 256 + t * 128;  // my row of the output accumulator
    const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2);

    float m_ref = -INFINITY, l_sum = 0.f;
    int g = 0;
#if JL_DIAG == 5
    long long d_wait = 0, d_h0 = 0, d_h1 = 0;
#endif
    // 32 scores s[e0 .. e0 + 31] -> 16 packed bf16 probability pairs at columns col .. col + 15 of the P region,
    // their sum added to acc2, and (kMax) their maxima folded into m4
    auto exp_block = [&](const uint32_t (&s)[128], int e0, uint64_t negm2, uint32_t col, uint64_t (&acc2)[4]) {
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int e = e0 + 2 * i;
        const uint64_t x = fma2(pack2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), scale2, negm2);
#if JL_DIAG == 1
        const uint64_t pp = x;
#else
        const uint64_t pp = ((kPolyMask >> (i & 7)) & 1u) ? exp2_pair_fma(x) : exp2_pair_sfu(x);
#endif
        acc2[i & 3] = add2(acc2[i & 3], pp);
        float p0, p1;
        unpack2(pp, p0, p1);
        pk[i] = pack_bf16x2(p0, p1);
      }
      JL_TMEM_ST16(t_s + col, pk, 0);
    };
    auto max_block = [&](const uint32_t (&s)[128], int e0, float (&m4)[4]) {
#pragma unroll
      for (int i = 0; i < 16; ++i) m4[i & 3] = max3(m4[i & 3], __uint_as_float(s[e0 + 2 * i]), __uint_as_float(s[e0 + 2 * i + 1]));
    };
    auto publish = [&](int half) {
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.p_half[t][half]);
    };
    // the row maximum grew by more than 2^8 for some row of the warp: new reference, O and the row sum follow
    auto raise_reference = [&](float mx, bool rescale_o) {
      const float m_new = fmaxf(m_ref, mx);
      const float alpha = m_new == -INFINITY ? 1.f : fast_exp2(m_ref - m_new);
      l_sum *= alpha;
      if (rescale_o) {
        // O_t is quiescent here: S_t(g) ready implies P_t V(g-1) retired, and P_t V(g) waits for our P
#pragma unroll
        for (int cchunk = 0; cchunk < 4; ++cchunk) {
          uint32_t o[32];
          JL_TMEM_LD32(t_o + cchunk * 32, o, 0);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          JL_TMEM_ST32(t_o + cchunk * 32, o, 0);
        }
      }
      m_ref = m_new;
    };

    for (int ph = 0; ph < sched.n_phases; ++ph) {
      const int c = sched.cls[ph];
      int64_t row_lo, row_hi, tile_lo_max, tile_hi_min, dummy;
      class_interval(p, c, pq, row_lo, row_hi);
      class_interval(p, c, pq_t1, tile_lo_max, dummy);      // largest lower bound over the tile's rows
      class_interval(p, c, pq_t0, dummy, tile_hi_min);      // smallest upper bound over the tile's rows
      for (int jj = 0; jj < sched.n_tiles[ph]; ++jj, ++g) {
        const int j = sched.j_lo[ph] + jj;
        const int64_t tp0 = key_position(static_cast<int64_t>(j) * kTileN, p.k_pos0, p.k_block, p.k_block_stride);
        const int valid = min(kTileN, p.sk - j * kTileN);
        const bool uniform = valid == kTileN && tile_lo_max <= tp0 && tile_hi_min >= tp0 + kTileN - 1;

#if JL_DIAG == 5
        const long long c0 = clock64();
#endif
        mbar_wait(&sm.s_full[t], g & 1, sm);
        tc_fence_after();
#if JL_DIAG == 5
        const long long c1 = clock64();
        d_wait += c1 - c0;
#endif
#if JL_DIAG == 2 || JL_DIAG == 6 || JL_DIAG == 7
        tc_fence_before();
        mbar_arrive(&sm.p_half[t][0]);
        mbar_arrive(&sm.p_half[t][1]);
        continue;
#endif
        uint32_t s[128];
        uint64_t acc2[4] = {0ull, 0ull, 0ull, 0ull};
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        {
          // scores -> registers and row maximum (4 independent chains of 3-input max)
          if (uniform) {
            // the 32-column loads are software-pipelined against the reduction: chunk c+1 is in flight while chunk c is reduced
            JL_TMEM_LD32(t_s + 0, s, 0);
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              tmem_wait_ld();
              if (ch + 1 < 4) JL_TMEM_LD32(t_s + (ch + 1) * 32, s, (ch + 1) * 32);
              max_block(s, ch * 32, m4);
            }
          } else {
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) JL_TMEM_LD32(t_s + ch * 32, s, ch * 32);
            tmem_wait_ld();
            const int64_t lo64 = row_lo - tp0, hi64 = row_hi - tp0 + 1;
            const int c_lo = lo64 < 0 ? 0 : (lo64 > 128 ? 128 : static_cast<int>(lo64));
            const int c_hi = hi64 < 0 ? 0 : (hi64 > valid ? valid : static_cast<int>(hi64));
#pragma unroll
            for (int i = 0; i < 128; ++i)
              if (!(i >= c_lo && i < c_hi)) s[i] = 0xff800000u;        // -inf
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) max_block(s, ch * 32, m4);
          }
          const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
#if JL_DIAG == 4
          l_sum += mx;
          tc_fence_before();
          mbar_arrive(&sm.p_half[t][0]);
          mbar_arrive(&sm.p_half[t][1]);
          continue;
#endif
          // lazy rescale: only when some row of the warp outgrew its reference maximum by 2^8
          if (__any_sync(0xffffffffu, mx > m_ref + 8.f)) raise_reference(mx, g > 0);
          const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
          const uint64_t negm2 = pack2(-m_use, -m_use);
          // p = 2^(s * scale - m): packed FMA, then the exponentials split between the FMA pipe and the SFU (kPolyMask).
          // The probabilities of keys 0..63 are published first, with their own barrier, so that the first four
          // k-steps of P V never wait for the last exponentials.
          exp_block(s, 0, negm2, 0, acc2);
          exp_block(s, 32, negm2, 16, acc2);
          publish(0);
#if JL_DIAG == 5
          const long long c2 = clock64();
          d_h0 += c2 - c1;
#endif
          exp_block(s, 64, negm2, 32, acc2);
          exp_block(s, 96, negm2, 48, acc2);
          publish(1);
#if JL_DIAG == 5
          d_h1 += clock64() - c2;
#endif
        }
        {
          float a0, a1;
          unpack2(add2(add2(acc2[0], acc2[1]), add2(acc2[2], acc2[3])), a0, a1);
          l_sum += a0 + a1;
        }
      }
    }

#if JL_DIAG == 5
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (warp & 3) == 0 && g > 0)
      printf("softmax tile %d: %d tiles; per tile: wait S %lld, S ready -> first half published %lld, -> second half published %lld\n",
             t, g, d_wait / g, d_h0 / g, d_h1 / g);
#endif
    // ---- epilogue: O / l -> bf16, LSE ----
    if (sched.total > 0) {
      mbar_wait(&sm.all_done, 0, sm);
      tc_fence_after();
    }
    const bool seen = m_ref != -INFINITY;                 // masked scores add ~1e-38 each to l_sum, never to m_ref
    const float inv = seen ? 1.f / l_sum : 0.f;
    __nv_bfloat16* orow = p.out + b * p.os_b + static_cast<int64_t>(q_row) * p.os_s + head * p.os_h;
#pragma unroll
    for (int cchunk = 0; cchunk < 4; ++cchunk) {
      uint32_t o[32];
      if (sched.total > 0) {
        JL_TMEM_LD32(t_o + cchunk * 32, o, 0);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0u;
      }
      if (row_valid) {
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[v4 * 8 + 0]) * inv, __uint_as_float(o[v4 * 8 + 1]) * inv);
          w.y = pack_bf16x2(__uint_as_float(o[v4 * 8 + 2]) * inv, __uint_as_float(o[v4 * 8 + 3]) * inv);
          w.z = pack_bf16x2(__uint_as_float(o[v4 * 8 + 4]) * inv, __uint_as_float(o[v4 * 8 + 5]) * inv);
          w.w = pack_bf16x2(__uint_as_float(o[v4 * 8 + 6]) * inv, __uint_as_float(o[v4 * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + cchunk * 32 + v4 * 8) = w;
        }
      }
    }
    if (row_valid && p.lse != nullptr)
      p.lse[(static_cast<int64_t>(b) * p.heads + head) * p.sq + q_row] = seen ? (m_ref + log2f(l_sum)) * kLn2 : -INFINITY;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
  }
  if (threadIdx.x == 0 && sm.failed && p.status != nullptr) atomicExch(p.status, 1);
}

// ---------------------------------------------------------------------------------------------
// The paired kernel: a cluster of two CTAs works on 256 query rows (128 each) with cta_group::2 MMAs
// ---------------------------------------------------------------------------------------------
// Every key / value tile is split between the two CTAs (each loads 64 of the 128 keys of K and 64 of the 128
// columns of V; the tensor cores of the pair read both halves), so a CTA holds only its own 128 query rows and
// half of every streamed tile.  Its tensor memory then has room for two score buffers and two probability
// buffers beside ONE output accumulator:
//     S_a | S_b | O | P_a | P_b   =  128 + 128 + 128 + 64 + 64 = 512 columns
// The two softmax warpgroups take alternate key tiles of the same 128 rows (warps 4-7: even tiles, buffers a;
// warps 8-11: odd tiles, buffers b), one thread per row as in the single-CTA kernel.  A score buffer is handed
// back as soon as its scores are in registers, and Q K^T and P V are issued by two different warps (1 and 2 of
// the even CTA): Q K^T of tile g + 2 starts when the scores of tile g have been read, whatever P V is waiting
// for, so neither the softmax threads nor the tensor pipe wait for each other's full round trip.
// Both threads of a row add into the same O, so they share the row's reference maximum: it lives in shared
// memory, is decided in tile order (the thread of tile g waits until the decision of tile g-1 is posted, which
// happens a tile earlier in time) and the thread that raises it rescales O once P V of the previous tile has
// retired and before its own P lets the next P V start.
// Only the even CTA of the pair issues MMAs; its barriers collect the arrivals of both CTAs, its commits go
// to the barriers of both.  All query classes stay resident in shared memory, so the look-ahead crosses phases.
namespace pair {

constexpr int kRows = 128;                       // query rows per CTA
constexpr int kKStages = 4, kVStages = 3;
constexpr int kQBytes = 128 * 256;               // 128 rows x 128 bf16 (two 64-column halves of 16 KB)
constexpr int kQHalf = 128 * 128;
constexpr int kKBytes = 64 * 256;                // this CTA's 64 keys x 128 bf16 (two 64-column halves of 8 KB)
constexpr int kKHalf = 64 * 128;
constexpr int kVBytes = 128 * 128;               // 128 keys x this CTA's 64 columns

struct Maps {
  CUtensorMap q[JL_MAX_CLASSES];     // box 64 x 1 x 128 x 1
  CUtensorMap k[2];                  // box 64 x 1 x 64 x 1
  CUtensorMap v;                     // box 64 x 1 x 128 x 1
};

struct Smem {
  alignas(1024) uint8_t q[JL_MAX_CLASSES][kQBytes];
  alignas(1024) uint8_t k[kKStages][kKBytes];
  alignas(1024) uint8_t v[kVStages][kVBytes];
  float ref_val[kRows];                          // the row's reference maximum (log2 domain) after the last decided tile
  int ref_seq[4];                                // per 32 rows: number of tiles whose reference has been decided
  float row_sum[2][kRows];
  // leader-only barriers (both CTAs arrive on the even CTA's copy): q_full, k_full, v_full, s_free, p_full
  uint64_t q_full[JL_MAX_CLASSES], k_full[kKStages], v_full[kVStages], s_free[2], p_full[2][2];
  // per-CTA barriers, signalled by the commits of the leader's MMA warps
  uint64_t k_empty[kKStages], v_empty[kVStages], s_full[2], pv_done[2], all_done;
  uint32_t tmem_base;
  int failed;
};

__device__ __forceinline__ uint32_t leader_addr(const void* local) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(r) : "r"(smem_u32(local)));
  return r;
}
__device__ __forceinline__ void arrive_leader(uint32_t leader_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(leader_bar) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load of this CTA's part of a tile; the bytes are counted on the leader's barrier
__device__ __forceinline__ void tma_load_pair(void* dst, const CUtensorMap* map, uint32_t leader_bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void mma2_ss(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma2_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// commit of the pair's MMAs, delivered to the barrier at the same offset in both CTAs (one plain commit per CTA:
// the second names the other CTA's barrier by its cluster address)
__device__ __forceinline__ void commit_both(uint64_t* bar) {
  const uint32_t own = smem_u32(bar);
  uint32_t other;
  asm volatile("mapa.shared::cluster.u32 %0, %1, 1;" : "=r"(other) : "r"(own));
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(own) : "memory");
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(other) : "memory");
}
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// Bounded wait until the reference of `need` tiles has been decided for the 32 rows of a quadrant
__device__ __forceinline__ int load_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void store_release(int* p, int v) {
  asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void wait_ref_seq(const int* seq, int need, Smem& sm) {
  if (load_acquire(seq) >= need) return;
  volatile int* failed = reinterpret_cast<volatile int*>(&sm.failed);
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (load_acquire(seq) >= need) return;
    if (*failed) return;
    if (globaltimer_ns() - t0 > kWaitLimitNs) { *failed = 1; return; }
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
prefill_pair_kernel(const __grid_constant__ Maps maps, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // the same offset in both CTAs: the dynamic shared memory of the two CTAs starts at the same window address
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(blockIdx.x & 1);                       // rank in the pair; 0 issues the MMAs
  // grid x = (pair of query tiles, head within the group, rank), the latest (heaviest) rows first over the group of heads
  const int slot = static_cast<int>(blockIdx.x >> 1);
  const int pair_idx = static_cast<int>((gridDim.x >> 1) / p.head_group) - 1 - slot / p.head_group;
  const int head = blockIdx.y * p.head_group + slot % p.head_group;
  const int b = p.batch_wrap > 0 ? (p.batch_first + static_cast<int>(blockIdx.z)) % p.batch_wrap : static_cast<int>(blockIdx.z);
  const int b_kv = p.batch_wrap > 0 ? 0 : b;
  const int64_t q_pos0 = p.q_pos0 + b * p.q_pos0_batch_step;
  const int kvh = head / (p.heads / p.kv_heads);
  const int q_row0_pair = pair_idx * kRowsPerCta;
  const int q_row0 = q_row0_pair + rank * kRows;
  const Schedule sched = make_schedule(p, q_row0_pair, q_pos0);            // both CTAs walk the same tiles

  if (threadIdx.x == 0) {
    sm.failed = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    for (int c = 0; c < JL_MAX_CLASSES; ++c) mbar_init(&sm.q_full[c], 1);
    for (int i = 0; i < kKStages; ++i) { mbar_init(&sm.k_full[i], 1); mbar_init(&sm.k_empty[i], 1); }
    for (int i = 0; i < kVStages; ++i) { mbar_init(&sm.v_full[i], 1); mbar_init(&sm.v_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.s_full[i], 1);
      mbar_init(&sm.s_free[i], 8);                // one arrival per warp of the buffer's warpgroup, either CTA
      mbar_init(&sm.p_full[i][0], 8);
      mbar_init(&sm.p_full[i][1], 8);
      mbar_init(&sm.pv_done[i], 1);
    }
    mbar_init(&sm.all_done, 1);
    for (int i = 0; i < 4; ++i) sm.ref_seq[i] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < kRows) sm.ref_val[threadIdx.x] = -INFINITY;
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  // tile g of the schedule -> (class, key tile)
  auto tile_of = [&](int g, int& c, int& j, bool& first_of_phase) {
    int ph = 0, base = 0;
    while (ph + 1 < sched.n_phases && g >= base + sched.n_tiles[ph]) { base += sched.n_tiles[ph]; ++ph; }
    c = sched.cls[ph];
    j = sched.j_lo[ph] + (g - base);
    first_of_phase = g == base;
  };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLow));
    if (warp == 0) {
      // ============================ TMA producer of Q and K (both CTAs) ============================
      if (lane == 0 && sched.total > 0) {
        for (int ph = 0; ph < sched.n_phases; ++ph) {
          const int c = sched.cls[ph];
          if (rank == 0) mbar_expect_tx(&sm.q_full[c], 2 * kQBytes);
          const uint32_t bar = leader_addr(&sm.q_full[c]);
          for (int h = 0; h < 2; ++h) tma_load_pair(sm.q[c] + h * kQHalf, &maps.q[c], bar, h * 64, head, q_row0, b);
        }
        for (int g = 0; g < sched.total; ++g) {
          int c, j;
          bool first;
          tile_of(g, c, j, first);
          const CUtensorMap* km = &maps.k[p.k_map[c]];
          const int ks = g % kKStages;
          mbar_wait(&sm.k_empty[ks], ((g / kKStages) & 1) ^ 1, sm);
          if (rank == 0) mbar_expect_tx(&sm.k_full[ks], 2 * kKBytes);
          const uint32_t kbar = leader_addr(&sm.k_full[ks]);
          for (int h = 0; h < 2; ++h) tma_load_pair(sm.k[ks] + h * kKHalf, km, kbar, h * 64, kvh, j * kTileN + rank * 64, b_kv);
        }
      }
    } else if (warp == 3) {
      // ================================ TMA producer of V (both CTAs) ================================
      if (lane == 0) {
        for (int g = 0; g < sched.total; ++g) {
          int c, j;
          bool first;
          tile_of(g, c, j, first);
          const int vs = g % kVStages;
          mbar_wait(&sm.v_empty[vs], ((g / kVStages) & 1) ^ 1, sm);
          if (rank == 0) mbar_expect_tx(&sm.v_full[vs], 2 * kVBytes);
          tma_load_pair(sm.v[vs], &maps.v, leader_addr(&sm.v_full[vs]), rank * 64, kvh, j * kTileN, b_kv);
        }
      }
    } else if (warp == 1 && rank == 0) {
      // ============================== Q K^T issuer (leader CTA) ==============================
      // Two issuing warps, so that a late P never holds back a Q K^T whose score buffer is already free
      // (and the other way round): this warp is gated by K tiles and freed score buffers only.
      if (sched.total > 0) {
        uint32_t leader;
        asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(leader));
        const uint32_t idesc_qk = instr_desc(256, kTileN, 0);
        const uint64_t q_desc0 = smem_desc(smem_u32(sm.q[0]), 16, 1024);
        const uint64_t k_desc0 = smem_desc(smem_u32(sm.k[0]), 16, 1024);
#if JL_DIAG == 5
        long long w_k = 0, w_sf = 0;
        const long long t_begin = clock64();
#endif
        for (int g = 0; g < sched.total; ++g) {
          int c, j;
          bool first;
          tile_of(g, c, j, first);
          if (first) mbar_wait(&sm.q_full[c], 0, sm);
          const int ks = g % kKStages;
          JL_TIMED(w_k, mbar_wait(&sm.k_full[ks], (g / kKStages) & 1, sm));
          if (g >= 2) JL_TIMED(w_sf, mbar_wait(&sm.s_free[g & 1], ((g >> 1) - 1) & 1, sm));      // the scores of tile g-2 are in registers
          tc_fence_after();
          const uint64_t qd = q_desc0 + static_cast<uint64_t>((c * kQBytes) >> 4);
          const uint64_t kd = k_desc0 + static_cast<uint64_t>((ks * kKBytes) >> 4);
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint64_t off_a = static_cast<uint64_t>(((kk >> 2) * kQHalf + (kk & 3) * 32) >> 4);
              const uint64_t off_b = static_cast<uint64_t>(((kk >> 2) * kKHalf + (kk & 3) * 32) >> 4);
              mma2_ss(tmem + (g & 1) * 128, qd + off_a, kd + off_b, idesc_qk, kk > 0);
            }
            commit_both(&sm.s_full[g & 1]);
            commit_both(&sm.k_empty[ks]);
          }
          __syncwarp();
        }
#if JL_DIAG == 5
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0)
          printf("pair QK warp: %d tiles, %lld clk/tile; waits per tile: K %lld S-free %lld\n", sched.total,
                 (clock64() - t_begin) / sched.total, w_k / sched.total, w_sf / sched.total);
#endif
      }
    } else if (warp == 2 && rank == 0) {
      // =============================== P V issuer (leader CTA) ===============================
      if (sched.total > 0) {
        uint32_t leader;
        asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(leader));
        const uint32_t idesc_pv = instr_desc(256, kHeadDim, 1);
        const uint64_t v_desc0 = smem_desc(smem_u32(sm.v[0]), kVBytes, 1024);
#if JL_DIAG == 5
        long long w_v = 0, w_p0 = 0, w_p1 = 0;
        const long long t_begin = clock64();
#endif
        for (int g = 0; g < sched.total; ++g) {
          const int vs = g % kVStages, pb = g & 1;
          const uint64_t vd = v_desc0 + static_cast<uint64_t>((vs * kVBytes) >> 4);
          JL_TIMED(w_v, mbar_wait(&sm.v_full[vs], (g / kVStages) & 1, sm));
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (h == 0) { JL_TIMED(w_p0, mbar_wait(&sm.p_full[pb][h], (g >> 1) & 1, sm)); }
            else { JL_TIMED(w_p1, mbar_wait(&sm.p_full[pb][h], (g >> 1) & 1, sm)); }
            tc_fence_after();
            if (leader) {
#pragma unroll
              for (int kk = 4 * h; kk < 4 * h + 4; ++kk)
                mma2_ts(tmem + 256, tmem + 384 + pb * 64 + kk * 8, vd + static_cast<uint64_t>((kk * 2048) >> 4), idesc_pv,
                        (g > 0 || kk > 0) ? 1u : 0u);
              if (h == 1) {
                commit_both(&sm.pv_done[pb]);
                commit_both(&sm.v_empty[vs]);
              }
            }
            __syncwarp();
          }
        }
        if (leader) commit_both(&sm.all_done);
        __syncwarp();
#if JL_DIAG == 5
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0)
          printf("pair PV warp: %d tiles, %lld clk/tile; waits per tile: V %lld P0 %lld P1 %lld\n", sched.total,
                 (clock64() - t_begin) / sched.total, w_v / sched.total, w_p0 / sched.total, w_p1 / sched.total);
#endif
      }
    }
  } else {
    // ===================== softmax + epilogue (one thread per row, alternate key tiles) =====================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsHigh));
    const int wg = (warp - 4) >> 2;                        // takes the tiles g with (g & 1) == wg; epilogue: output columns 64 wg ..
    const int quad = warp & 3;
    const int r_in_tile = quad * 32 + lane;
    const int q_row = q_row0 + r_in_tile;
    const bool row_valid = q_row < p.sq;
    const int64_t pq = key_position(q_row, q_pos0, p.q_block, p.q_block_stride);
    const int tile_rows = min(kRows, p.sq - q_row0);
    const int64_t pq_t0 = key_position(q_row0, q_pos0, p.q_block, p.q_block_stride);
    const int64_t pq_t1 = pq_t0 + (tile_rows > 0 ? tile_rows - 1 : 0);
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem + lane_base + wg * 128;             // my row of my score buffer
    const uint32_t t_p = tmem + lane_base + 384 + wg * 64;        // my row of my probability buffer
    const uint32_t t_o = tmem + lane_base + 256;                  // the row's output accumulator (shared with the other warpgroup)
    const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2);
    const uint32_t s_free_bar = leader_addr(&sm.s_free[wg]);
    const uint32_t p_full_bar[2] = {leader_addr(&sm.p_full[wg][0]), leader_addr(&sm.p_full[wg][1])};
    volatile float* ref_val = sm.ref_val;

    float my_ref = -INFINITY, l_sum = 0.f;                 // l_sum is expressed relative to my_ref
#if JL_DIAG == 5
    long long d_ws = 0, d_ld = 0, d_ref = 0, d_pv = 0, d_exp = 0;
    int d_n = 0;
#endif
    auto exp_block = [&](const uint32_t (&s)[128], int e0, uint64_t negm2, uint32_t col, uint64_t (&acc2)[4]) {
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int e = e0 + 2 * i;
        const uint64_t x = fma2(pack2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), scale2, negm2);
        const uint64_t pp = ((kPolyMask >> (i & 7)) & 1u) ? exp2_pair_fma(x) : exp2_pair_sfu(x);
        acc2[i & 3] = add2(acc2[i & 3], pp);
        float p0, p1;
        unpack2(pp, p0, p1);
        pk[i] = pack_bf16x2(p0, p1);
      }
      JL_TMEM_ST16(t_p + col, pk, 0);
    };
    auto max_block = [&](const uint32_t (&s)[128], int e0, float (&m4)[4]) {
#pragma unroll
      for (int i = 0; i < 16; ++i) m4[i & 3] = max3(m4[i & 3], __uint_as_float(s[e0 + 2 * i]), __uint_as_float(s[e0 + 2 * i + 1]));
    };
    auto publish = [&](int half) {
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) arrive_leader(p_full_bar[half]);
    };

    int g = 0;
    for (int ph = 0; ph < sched.n_phases; ++ph) {
      const int c = sched.cls[ph];
      int64_t row_lo, row_hi, tile_lo_max, tile_hi_min, dummy;
      class_interval(p, c, pq, row_lo, row_hi);
      class_interval(p, c, pq_t1, tile_lo_max, dummy);
      class_interval(p, c, pq_t0, dummy, tile_hi_min);
      for (int jj = 0; jj < sched.n_tiles[ph]; ++jj, ++g) {
        if ((g & 1) != wg) continue;
        const int n = g >> 1;                              // my n-th tile
        const int j = sched.j_lo[ph] + jj;
        const int64_t tp0 = key_position(static_cast<int64_t>(j) * kTileN, p.k_pos0, p.k_block, p.k_block_stride);
        const int valid = min(kTileN, p.sk - j * kTileN);
        const bool uniform = valid == kTileN && tile_lo_max <= tp0 && tile_hi_min >= tp0 + kTileN - 1;

#if JL_DIAG == 5
        const long long c0 = clock64();
#endif
        mbar_wait(&sm.s_full[wg], n & 1, sm);
        tc_fence_after();
#if JL_DIAG == 5
        const long long c1 = clock64();
#endif
#if JL_DIAG == 2
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_leader(s_free_bar);
        if (n >= 1) mbar_wait(&sm.pv_done[wg], (n - 1) & 1, sm);
        if (lane == 0) { arrive_leader(p_full_bar[0]); arrive_leader(p_full_bar[1]); }
        continue;
#endif
        uint32_t s[128];
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        // scores -> registers and row maximum; the score buffer goes back to the tensor pipe as soon as it has been read
        JL_TMEM_LD32(t_s + 0, s, 0);
        // under the latency of the first load: P V of my previous tile has read the probability buffer (it has
        // long retired; P V of tile g-3 then has too, which the parity wait of a rescale below relies on), and
        // the reference tile g-1 left, if it is already posted
        if (n >= 1) {
          mbar_wait(&sm.pv_done[wg], (n - 1) & 1, sm);
          tc_fence_after();
        }
        const bool ref_early = load_acquire(&sm.ref_seq[quad]) >= g;
        float ref_prev = ref_val[r_in_tile];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          tmem_wait_ld();
          if (ch + 1 < 4) {
            JL_TMEM_LD32(t_s + (ch + 1) * 32, s, (ch + 1) * 32);
          } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_leader(s_free_bar);
          }
          if (uniform) max_block(s, ch * 32, m4);
        }
        if (!uniform) {
          const int64_t lo64 = row_lo - tp0, hi64 = row_hi - tp0 + 1;
          const int c_lo = lo64 < 0 ? 0 : (lo64 > 128 ? 128 : static_cast<int>(lo64));
          const int c_hi = hi64 < 0 ? 0 : (hi64 > valid ? valid : static_cast<int>(hi64));
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (!(i >= c_lo && i < c_hi)) s[i] = 0xff800000u;        // -inf
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) max_block(s, ch * 32, m4);
        }
        const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
#if JL_DIAG == 5
        const long long c2 = clock64();
#endif
        // the reference of this tile: the one tile g-1 left, raised if some row of the warp outgrew it by 2^8
        if (!ref_early) {
          wait_ref_seq(&sm.ref_seq[quad], g, sm);
          ref_prev = ref_val[r_in_tile];
        }
        const bool raise = __any_sync(0xffffffffu, mx > ref_prev + 8.f);
        const float ref_new = raise ? fmaxf(ref_prev, mx) : ref_prev;
        if (raise) ref_val[r_in_tile] = ref_new;
        __syncwarp();                                      // orders the lanes' writes before lane 0's release
        if (lane == 0) store_release(&sm.ref_seq[quad], g + 1);
        if (raise && g > 0) {
          // O follows the reference: P V of tile g-1 has to retire first, P V of tile g waits for this thread's P
          const float alpha = ref_new == -INFINITY ? 1.f : fast_exp2(ref_prev - ref_new);
          mbar_wait(&sm.pv_done[(g - 1) & 1], ((g - 1) >> 1) & 1, sm);
          tc_fence_after();
#pragma unroll
          for (int cchunk = 0; cchunk < 4; ++cchunk) {
            uint32_t o[32];
            JL_TMEM_LD32(t_o + cchunk * 32, o, 0);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            JL_TMEM_ST32(t_o + cchunk * 32, o, 0);
          }
        }
        if (ref_new != my_ref) {
          l_sum *= ref_new == -INFINITY ? 1.f : fast_exp2(my_ref - ref_new);
          my_ref = ref_new;
        }
#if JL_DIAG == 5
        const long long c3 = clock64();
        const long long c4 = c3;
#endif
        const float m_use = my_ref == -INFINITY ? 0.f : my_ref;
        const uint64_t negm2 = pack2(-m_use, -m_use);
        uint64_t acc2[4] = {0ull, 0ull, 0ull, 0ull};
        exp_block(s, 0, negm2, 0, acc2);
        exp_block(s, 32, negm2, 16, acc2);
        publish(0);
        exp_block(s, 64, negm2, 32, acc2);
        exp_block(s, 96, negm2, 48, acc2);
        publish(1);
        float a0, a1;
        unpack2(add2(add2(acc2[0], acc2[1]), add2(acc2[2], acc2[3])), a0, a1);
        l_sum += a0 + a1;
#if JL_DIAG == 5
        d_ws += c1 - c0; d_ld += c2 - c1; d_ref += c3 - c2; d_pv += c4 - c3; d_exp += clock64() - c4; ++d_n;
#endif
      }
    }
#if JL_DIAG == 5
    if (blockIdx.x < 2 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && quad == 0 && d_n > 0)
      printf("pair softmax rank %d wg %d: %d tiles; per tile: wait S %lld, load+max %lld, reference %lld, wait P buffer %lld, exps+publish %lld\n",
             rank, wg, d_n, d_ws / d_n, d_ld / d_n, d_ref / d_n, d_pv / d_n, d_exp / d_n);
#endif

    // ---- epilogue: O / l -> bf16, LSE ----
    if (sched.total > 0) {
      mbar_wait(&sm.all_done, 0, sm);
      tc_fence_after();
#if JL_DIAG != 2
      wait_ref_seq(&sm.ref_seq[quad], sched.total, sm);
#endif
    }
    const float ref_fin = ref_val[r_in_tile];
    const bool seen = ref_fin != -INFINITY;
    sm.row_sum[wg][r_in_tile] = (seen && my_ref != -INFINITY) ? l_sum * fast_exp2(my_ref - ref_fin) : 0.f;
    softmax_bar();
    const float l_row = sm.row_sum[0][r_in_tile] + sm.row_sum[1][r_in_tile];
    const float inv = seen ? 1.f / l_row : 0.f;
    __nv_bfloat16* orow = p.out + b * p.os_b + static_cast<int64_t>(q_row) * p.os_s + head * p.os_h + wg * 64;
#pragma unroll
    for (int cchunk = 0; cchunk < 2; ++cchunk) {
      uint32_t o[32];
      if (sched.total > 0) {
        JL_TMEM_LD32(t_o + wg * 64 + cchunk * 32, o, 0);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0u;
      }
      if (row_valid) {
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[v4 * 8 + 0]) * inv, __uint_as_float(o[v4 * 8 + 1]) * inv);
          w.y = pack_bf16x2(__uint_as_float(o[v4 * 8 + 2]) * inv, __uint_as_float(o[v4 * 8 + 3]) * inv);
          w.z = pack_bf16x2(__uint_as_float(o[v4 * 8 + 4]) * inv, __uint_as_float(o[v4 * 8 + 5]) * inv);
          w.w = pack_bf16x2(__uint_as_float(o[v4 * 8 + 6]) * inv, __uint_as_float(o[v4 * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + cchunk * 32 + v4 * 8) = w;
        }
      }
    }
    if (wg == 0 && row_valid && p.lse != nullptr)
      p.lse[(static_cast<int64_t>(b) * p.heads + head) * p.sq + q_row] = seen ? (ref_fin + log2f(l_row)) * kLn2 : -INFINITY;
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();               // neither CTA leaves (or frees tensor memory) while the other may still signal it
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
  }
  if (threadIdx.x == 0 && sm.failed && p.status != nullptr) atomicExch(p.status, 1);
}

}  // namespace pair

}  // namespace tc

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    cudaDriverEntryPointQueryResult q;
    void* ptr = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess) fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// (B, S, Hx, 128) bf16 view -> 4-D map (d, h, s, b), box 64 x 1 x box_rows x 1, 128-byte swizzle, zero fill past the end.
static int make_map(CUtensorMap* m, const void* base, int batch, int seq, int heads, int64_t sb, int64_t ss, int64_t sh, int box_rows = 128) {
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return fail(JL_ERR_LAUNCH, "jl_prefill: cuTensorMapEncodeTiled is not available from the driver");
  // size-1 dimensions may arrive with stride 0; the encoder wants positive multiples of 16 bytes
  const int64_t dflt = 256;
  const cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(seq), static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>((heads > 1 && sh > 0 ? sh : dflt / 2) * 2),
                                 static_cast<cuuint64_t>((seq > 1 && ss > 0 ? ss : dflt / 2) * 2),
                                 static_cast<cuuint64_t>((batch > 1 && sb > 0 ? sb : dflt / 2) * 2)};
  const cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(box_rows), 1};
  const cuuint32_t es[4] = {1, 1, 1, 1};
  const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(JL_ERR_BAD_ARG, "jl_prefill: tensor map encoding failed (CUresult %d)", static_cast<int>(r));
  return JL_OK;
}

// NULL if the tcgen05 kernel covers the request, else the reason it does not.
const char* prefill_tc_unsupported_reason(const jl_prefill_args* a) {
  if (a->k_block > 0 && a->k_block < a->seqlen_k && (a->k_block % tc::kTileN != 0))
    return "k_block must be a multiple of 128 (the key tile)";
  if (a->q_block > 0 && a->q_block < a->seqlen_q && (a->q_block % tc::kRowsPerCta != 0))
    return "q_block must be a multiple of 256 (the query rows of one CTA)";
  if (a->remap_far_in_kernel) {
    if (a->map.kind != JL_MAP_BAND) return "remap_far_in_kernel needs the band map";
    if (a->inv_freq == nullptr || a->group_size < 1) return "remap_far_in_kernel needs inv_freq and group_size >= 1";
    return nullptr;
  }
  int distinct = 0;
  const void* seen[2] = {nullptr, nullptr};
  for (int c = 0; c < a->map.n_classes; ++c) {
    bool found = false;
    for (int i = 0; i < distinct; ++i) found |= seen[i] == a->k[c];
    if (!found) {
      if (distinct == 2) return "at most two distinct key tensors";
      seen[distinct++] = a->k[c];
    }
  }
  return nullptr;
}

// Status word of the bounded waits: a file-scope device variable (no allocation), one per device image.
__device__ int g_prefill_status = 0;

static int* status_word() {
  static int* words[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (words[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_prefill_status) != cudaSuccess) return nullptr;
    words[dev] = static_cast<int*>(ptr);
  }
  return words[dev];
}

int prefill_tc_status() {
  int* w = status_word();
  int v = 0;
  if (w != nullptr) {
    if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v != 0) cudaMemset(w, 0, sizeof(int));      // reading a raised status clears it, so later launches run again
  }
  return v;
}

// Tensor maps and kernel parameters of a request (shared by the two tcgen05 kernels; k_box_rows = key rows per TMA box).
static int prepare(const jl_prefill_args* a, CUtensorMap* qmaps, CUtensorMap* kmaps, CUtensorMap* vmap, tc::Params& p, int k_box_rows) {
  int n_k = 0;
  const void* kptr[2] = {nullptr, nullptr};
  const bool no_keys = a->seqlen_k == 0;      // nothing is loaded then: the key / value maps only have to be well formed
  const bool remap = a->remap_far_in_kernel != 0;      // the far class then reads the class-0 tensors
  const bool striped = a->q_batch_wrap > 0;            // stripe batching: q / out hold q_batch_wrap elements, k / v one
  const int q_batches = striped ? a->q_batch_wrap : a->batch, kv_batches = striped ? 1 : a->batch;
  for (int c = 0; c < a->map.n_classes; ++c) {
    const void* qc = remap ? a->q[0] : a->q[c];
    const void* kc = remap ? a->k[0] : a->k[c];
    int rc = make_map(&qmaps[c], qc, q_batches, a->seqlen_q, a->heads, a->q_stride_b, a->q_stride_s, a->q_stride_h);
    if (rc != JL_OK) return rc;
    int slot = -1;
    for (int i = 0; i < n_k; ++i)
      if (kptr[i] == kc) slot = i;
    if (slot < 0) {
      slot = n_k++;
      kptr[slot] = kc;
      rc = no_keys ? make_map(&kmaps[slot], a->q[0], 1, 1, 1, 0, 0, 0, k_box_rows)
                   : make_map(&kmaps[slot], kc, kv_batches, a->seqlen_k, a->kv_heads, a->k_stride_b, a->k_stride_s, a->k_stride_h, k_box_rows);
      if (rc != JL_OK) return rc;
    }
    p.k_map[c] = slot;
  }
  for (int c = a->map.n_classes; c < JL_MAX_CLASSES; ++c) qmaps[c] = qmaps[0];
  if (n_k == 1) kmaps[1] = kmaps[0];
  int rc = no_keys ? make_map(vmap, a->q[0], 1, 1, 1, 0, 0, 0)
                   : make_map(vmap, a->v, kv_batches, a->seqlen_k, a->kv_heads, a->v_stride_b, a->v_stride_s, a->v_stride_h);
  if (rc != JL_OK) return rc;
  p.sq = a->seqlen_q; p.sk = a->seqlen_k; p.heads = a->heads; p.kv_heads = a->kv_heads; p.batch = a->batch;
  p.q_pos0 = a->q_pos0; p.k_pos0 = a->k_pos0;
  p.k_block = (a->k_block > 0 && a->k_block < a->seqlen_k) ? a->k_block : 0;
  p.k_block_stride = a->k_block_stride;
  p.q_block = (a->q_block > 0 && a->q_block < a->seqlen_q) ? a->q_block : 0;
  p.q_block_stride = a->q_block_stride;
  p.scale_log2 = a->softmax_scale * kLog2e;
  p.map_kind = a->map.kind; p.n_classes = a->map.n_classes;
  p.near_span = a->map.near_span; p.chunk = a->map.chunk > 0 ? a->map.chunk : 1;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.os_b = a->o_stride_b; p.os_s = a->o_stride_s; p.os_h = a->o_stride_h;
  p.status = status_word();
  p.remap = a->remap_far_in_kernel != 0;
  p.group_size = a->group_size > 0 ? a->group_size : 1;
  p.inv_freq = a->inv_freq;
  p.batch_first = striped ? a->q_batch_first : 0;
  p.batch_wrap = striped ? a->q_batch_wrap : 0;
  p.q_pos0_batch_step = striped ? a->q_pos0_batch_step : 0;
  return JL_OK;
}

// Query heads interleaved along grid x: those of two kv heads where the head count allows, else of one, else one head.
static int head_group_of(const jl_prefill_args* a) {
  const int rep = a->heads / a->kv_heads;
  if (a->heads % (2 * rep) == 0) return 2 * rep;
  return a->heads % rep == 0 ? rep : 1;
}

int launch_prefill_tc(const jl_prefill_args* a, cudaStream_t stream) {
  tc::Maps maps;
  tc::Params p{};
  const int rc = prepare(a, maps.q, maps.k, &maps.v, p, 128);
  if (rc != JL_OK) return rc;
  const int smem = static_cast<int>(sizeof(tc::Smem)) + 1024;
  // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute
  static bool attr_done[64] = {false};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(JL_ERR_LAUNCH, "jl_prefill: no current CUDA device");
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(tc::prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return check_launch("jl_prefill (shared memory opt-in)");
    attr_done[dev] = true;
  }
  // The query heads of two kv heads share a run of the grid, so that the longest CTAs of all of them start first (a
  // head at a time leaves the last head's longest CTA as a tail; all heads at once stream every kv head's K / V through
  // L2 together and lose its reuse: 32768 / 131072 / 16384 tokens, 32 / 8 heads: 1296 / 1204 / 942 TFLOP/s a head at a
  // time, 1310 / 1209 / 966 with 8 heads per run, 1279 / 1148 / 898 with all 32).
  p.head_group = head_group_of(a);
  const int hg = p.head_group;
  dim3 grid(((a->seqlen_q + tc::kRowsPerCta - 1) / tc::kRowsPerCta) * hg, a->heads / hg, a->batch);
  tc::prefill_tc_kernel<<<grid, tc::kThreads, smem, stream>>>(maps, p);
  return check_launch("jl_prefill (tcgen05)");
}

// NULL if the paired (two-CTA) kernel covers the request, else the reason it does not.
const char* prefill_pair_unsupported_reason(const jl_prefill_args* a) {
  if (a->remap_far_in_kernel) return "the in-kernel remap runs on the single-CTA kernel";
  return prefill_tc_unsupported_reason(a);
}

int launch_prefill_pair(const jl_prefill_args* a, cudaStream_t stream) {
  tc::pair::Maps maps;
  tc::Params p{};
  const int rc = prepare(a, maps.q, maps.k, &maps.v, p, 64);
  if (rc != JL_OK) return rc;
  const int smem = static_cast<int>(sizeof(tc::pair::Smem)) + 1024;
  static bool attr_done[64] = {false};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(JL_ERR_LAUNCH, "jl_prefill: no current CUDA device");
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(tc::pair::prefill_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return check_launch("jl_prefill (shared memory opt-in)");
    attr_done[dev] = true;
  }
  // one cluster of two CTAs per 256 query rows (the cluster shape is a compile-time attribute of the kernel)
  const int hg = head_group_of(a);           // as in launch_prefill_tc
  p.head_group = hg;
  dim3 grid(2 * ((a->seqlen_q + tc::kRowsPerCta - 1) / tc::kRowsPerCta) * hg, a->heads / hg, a->batch);
  tc::pair::prefill_pair_kernel<<<grid, tc::kThreads, smem, stream>>>(maps, p);
  return check_launch("jl_prefill (tcgen05, CTA pairs)");
}

}  // namespace jl

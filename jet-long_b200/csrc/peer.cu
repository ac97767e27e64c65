// Exchange of decode partials between the GPUs of a node through peer-mapped memory, fused with the
// N-way (O, LSE) merge: one kernel per rank pushes this rank's partial into every rank's exchange buffer
// with plain peer stores over NVLink, publishes a flag, waits for the other ranks' flags and merges what
// has landed in its own memory.  Only stores cross NVLink: no loads from peer memory, remote data is always read
// from local HBM.  Every wait is bounded in time: a wait that gives up raises a status word and the
// kernel returns (its output is then invalid), it never hangs or traps.
//
// Exchange buffer of one rank (identical layout on every rank):
//   O    [2 parities][world slots][rows][128] bf16
//   LSE  [2 parities][world slots][rows]      fp32
//   flag [world sources][ctas]                int64   (last epoch whose data from that source has landed)
// Two parities: a rank may already push exchange e + 1 while a slower rank still merges exchange e.
#include "jl_common.cuh"

namespace jl {

namespace {

constexpr int kPeerRowsPerCta = 32;
constexpr int kPeerThreads = 128;

__host__ __device__ inline int64_t peer_align(int64_t x) { return (x + 255) / 256 * 256; }

struct PeerLayout {
  int64_t o_bytes, lse_off, lse_bytes, flag_off, total;
  int ctas;
};

__host__ __device__ inline PeerLayout peer_layout(int world, int64_t rows) {
  PeerLayout l;
  l.ctas = static_cast<int>((rows + kPeerRowsPerCta - 1) / kPeerRowsPerCta);
  l.o_bytes = peer_align(2 * static_cast<int64_t>(world) * rows * kHeadDim * 2);
  l.lse_off = l.o_bytes;
  l.lse_bytes = peer_align(2 * static_cast<int64_t>(world) * rows * 4);
  l.flag_off = l.lse_off + l.lse_bytes;
  l.total = l.flag_off + peer_align(static_cast<int64_t>(world) * l.ctas * 8);
  return l;
}

struct PeerParams {
  const uint4* part_o;       // (rows, 128) bf16
  const float* part_lse;     // (rows,)
  uint8_t* buf[JL_MAX_PARTS];
  int rank, world;
  int64_t rows;
  const int64_t* epoch_base;
  int64_t epoch_stride, epoch_offset;
  uint4* out;
  float* lse_out;
  int* status;
  uint64_t wait_limit_ns;
};

__device__ __forceinline__ uint64_t peer_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(kPeerThreads) peer_merge_kernel(const PeerParams p) {
  const PeerLayout lay = peer_layout(p.world, p.rows);
  const int64_t epoch = (p.epoch_base != nullptr ? *p.epoch_base : 0) * p.epoch_stride + p.epoch_offset;
  const int par = static_cast<int>(epoch & 1);
  const int cta = blockIdx.x, tid = threadIdx.x;
  const int64_t row0 = static_cast<int64_t>(cta) * kPeerRowsPerCta;
  const int nrows = static_cast<int>(min(static_cast<int64_t>(kPeerRowsPerCta), p.rows - row0));
  // element offsets inside a buffer
  const int64_t slot_rows = (static_cast<int64_t>(par) * p.world + p.rank) * p.rows + row0;     // my slot, my rows

  // ---- push my rows into every rank's buffer (my own included) ----
  for (int dst = 0; dst < p.world; ++dst) {
    uint4* o_dst = reinterpret_cast<uint4*>(p.buf[dst]) + slot_rows * 16;
    for (int i = tid; i < nrows * 16; i += kPeerThreads) o_dst[i] = p.part_o[row0 * 16 + i];
    float* l_dst = reinterpret_cast<float*>(p.buf[dst] + lay.lse_off) + slot_rows;
    if (tid < nrows) l_dst[tid] = p.part_lse[row0 + tid];
  }
  __threadfence_system();
  __syncthreads();
  if (tid < p.world) {
    volatile int64_t* flag = reinterpret_cast<volatile int64_t*>(p.buf[tid] + lay.flag_off) + static_cast<int64_t>(p.rank) * lay.ctas + cta;
    *flag = epoch;
  }

  // ---- wait until every rank's rows of this exchange have landed here ----
  __shared__ int s_failed;
  if (tid == 0) s_failed = 0;
  __syncthreads();
  if (tid < p.world) {
    volatile int64_t* flag = reinterpret_cast<volatile int64_t*>(p.buf[p.rank] + lay.flag_off) + static_cast<int64_t>(tid) * lay.ctas + cta;
    if (*flag < epoch) {
      const uint64_t t0 = peer_timer_ns();
      while (*flag < epoch) {
        if (peer_timer_ns() - t0 > p.wait_limit_ns) { s_failed = 1; break; }
      }
    }
    __threadfence_system();
  }
  __syncthreads();
  if (s_failed) {
    if (tid == 0 && p.status != nullptr) atomicExch(p.status, 1);
    return;
  }

  // ---- merge the world partials of my rows from local memory: 4 threads per row, 32 dims each ----
  const int r = tid >> 2, part = tid & 3;
  if (r < nrows) {
    const uint8_t* mine = p.buf[p.rank];
    const float* lse_base = reinterpret_cast<const float*>(mine + lay.lse_off);
    float m = -INFINITY;
    for (int s = 0; s < p.world; ++s) m = fmaxf(m, lse_base[(static_cast<int64_t>(par) * p.world + s) * p.rows + row0 + r]);
    const float m_safe = m == -INFINITY ? 0.f : m;
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
    float wsum = 0.f;
    for (int s = 0; s < p.world; ++s) {
      const int64_t srow = (static_cast<int64_t>(par) * p.world + s) * p.rows + row0 + r;
      const float w = exp2f((lse_base[srow] - m_safe) * kLog2e);
      wsum += w;
      const uint4* src = reinterpret_cast<const uint4*>(mine) + srow * 16 + part * 4;
#pragma unroll
      for (int v4 = 0; v4 < 4; ++v4) {
        const uint4 x = src[v4];
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&x);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          acc[v4 * 8 + 2 * j] = fmaf(w, f.x, acc[v4 * 8 + 2 * j]);
          acc[v4 * 8 + 2 * j + 1] = fmaf(w, f.y, acc[v4 * 8 + 2 * j + 1]);
        }
      }
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    uint4* dst = p.out + (row0 + r) * 16 + part * 4;
#pragma unroll
    for (int v4 = 0; v4 < 4; ++v4) {
      uint4 y;
      uint32_t* uy = reinterpret_cast<uint32_t*>(&y);
#pragma unroll
      for (int j = 0; j < 4; ++j) uy[j] = pack_bf16x2(acc[v4 * 8 + 2 * j] * inv, acc[v4 * 8 + 2 * j + 1] * inv);
      dst[v4] = y;
    }
    if (p.lse_out != nullptr && part == 0) p.lse_out[row0 + r] = wsum > 0.f ? m_safe + logf(wsum) : -INFINITY;
  }
}

}  // namespace

size_t peer_merge_buffer_bytes(int32_t world, int32_t batch, int32_t heads) {
  if (world < 1 || batch < 1 || heads < 1) return 0;
  return static_cast<size_t>(peer_layout(world, static_cast<int64_t>(batch) * heads).total);
}

int launch_peer_merge(const jl_peer_merge_args* a, cudaStream_t stream) {
  if (a->head_dim != kHeadDim) return fail(JL_ERR_UNSUPPORTED, "jl_peer_merge: head_dim must be 128, got %d", a->head_dim);
  if (a->world < 1 || a->world > JL_MAX_PARTS || a->rank < 0 || a->rank >= a->world)
    return fail(JL_ERR_BAD_ARG, "jl_peer_merge: need 1 <= world <= %d and 0 <= rank < world", JL_MAX_PARTS);
  if (a->batch < 1 || a->heads < 1) return fail(JL_ERR_BAD_ARG, "jl_peer_merge: batch and heads must be positive");
  if (a->part_o == nullptr || a->part_lse == nullptr || a->out == nullptr || a->status == nullptr)
    return fail(JL_ERR_BAD_ARG, "jl_peer_merge: NULL pointer");
  if ((reinterpret_cast<uintptr_t>(a->part_o) | reinterpret_cast<uintptr_t>(a->out)) & 15)
    return fail(JL_ERR_BAD_ARG, "jl_peer_merge: part_o and out must be 16-byte aligned");
  const size_t need = peer_merge_buffer_bytes(a->world, a->batch, a->heads);
  if (a->buffer_bytes < need)
    return fail(JL_ERR_WORKSPACE, "jl_peer_merge: exchange buffers of %zu bytes needed, %zu given", need, a->buffer_bytes);
  PeerParams p{};
  for (int r = 0; r < a->world; ++r) {
    if (a->peer_buf[r] == nullptr || (reinterpret_cast<uintptr_t>(a->peer_buf[r]) & 255))
      return fail(JL_ERR_BAD_ARG, "jl_peer_merge: peer_buf[%d] must be a non-NULL 256-byte aligned mapping", r);
    p.buf[r] = static_cast<uint8_t*>(a->peer_buf[r]);
  }
  p.part_o = static_cast<const uint4*>(a->part_o);
  p.part_lse = a->part_lse;
  p.rank = a->rank; p.world = a->world;
  p.rows = static_cast<int64_t>(a->batch) * a->heads;
  p.epoch_base = a->epoch_base_dev;
  p.epoch_stride = a->epoch_stride; p.epoch_offset = a->epoch_offset;
  p.out = static_cast<uint4*>(a->out);
  p.lse_out = a->lse_out;
  p.status = a->status;
  p.wait_limit_ns = static_cast<uint64_t>(a->wait_limit_ms > 0 ? a->wait_limit_ms : 1000) * 1000000ull;
  const int ctas = static_cast<int>((p.rows + kPeerRowsPerCta - 1) / kPeerRowsPerCta);
  if (ctas > 148) return fail(JL_ERR_UNSUPPORTED, "jl_peer_merge: batch * heads must be at most %d", 148 * kPeerRowsPerCta);
  peer_merge_kernel<<<ctas, kPeerThreads, 0, stream>>>(p);
  return check_launch("jl_peer_merge");
}

}  // namespace jl

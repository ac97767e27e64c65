// extern "C" entry points of libjetlong_b200: argument validation, error reporting, dispatch.
#include <cstdarg>
#include <cstdio>

#include "jl_common.cuh"

namespace jl {

int launch_merge(const jl_merge_args* a, cudaStream_t stream);
int launch_rotate(const jl_rotate_args* a, cudaStream_t stream);
int launch_norm_rope(const jl_norm_rope_args* a, cudaStream_t stream);
int launch_rmsnorm(const jl_rmsnorm_args* a, cudaStream_t stream);
int launch_silu_mul(const jl_silu_mul_args* a, cudaStream_t stream);
int launch_peer_merge(const jl_peer_merge_args* a, cudaStream_t stream);
size_t peer_merge_buffer_bytes(int32_t world, int32_t batch, int32_t heads);
int launch_step_advance(const jl_step_advance_args* a, cudaStream_t stream);
int launch_decode_append(const jl_decode_append_args* a, cudaStream_t stream);
int launch_decode(const jl_decode_args* a, cudaStream_t stream);
int launch_decode_static(const jl_decode_args* a, cudaStream_t stream);
size_t decode_static_scratch_bytes();
int launch_prefill_mma(const jl_prefill_args* a, cudaStream_t stream);
int launch_prefill_tc(const jl_prefill_args* a, cudaStream_t stream);
const char* prefill_tc_unsupported_reason(const jl_prefill_args* a);
int launch_prefill_pair(const jl_prefill_args* a, cudaStream_t stream);
const char* prefill_pair_unsupported_reason(const jl_prefill_args* a);
int prefill_tc_status();
int32_t decode_auto_splits(int32_t batch, int32_t kv_heads, int64_t total_keys);
size_t decode_workspace_bytes(int32_t batch, int32_t heads, int32_t head_dim, int32_t max_splits);

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return JL_OK;
  return fail(JL_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

int check_device_arch() {
  static thread_local int cached_dev = -1;
  static thread_local int cached_ok = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(JL_ERR_LAUNCH, "no current CUDA device");
  if (dev != cached_dev) {
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cached_dev = dev;
    cached_ok = (major == 10);
  }
  if (!cached_ok) return fail(JL_ERR_ARCH, "jetlong_b200 kernels require an sm_100 (B200) device");
  return JL_OK;
}

static int validate_prefill(const jl_prefill_args* a) {
  if (a == nullptr) return fail(JL_ERR_BAD_ARG, "jl_prefill: args is NULL");
  if (a->head_dim != kHeadDim) return fail(JL_ERR_UNSUPPORTED, "jl_prefill: head_dim must be 128, got %d", a->head_dim);
  if (a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->seqlen_q < 0 || a->seqlen_k < 0)
    return fail(JL_ERR_BAD_ARG, "jl_prefill: sizes must be positive");
  if (a->heads % a->kv_heads) return fail(JL_ERR_BAD_ARG, "jl_prefill: heads must be divisible by kv_heads");
  if (a->map.kind != JL_MAP_BAND && a->map.kind != JL_MAP_CHUNK) return fail(JL_ERR_BAD_ARG, "jl_prefill: unknown position map kind %d", a->map.kind);
  const int want = a->map.kind == JL_MAP_BAND ? 2 : 3;
  if (a->map.n_classes != want) return fail(JL_ERR_BAD_ARG, "jl_prefill: map kind %d needs n_classes == %d", a->map.kind, want);
  if (a->map.kind == JL_MAP_BAND && a->map.near_span < 0) return fail(JL_ERR_BAD_ARG, "jl_prefill: near_span must be >= 0");
  if (a->map.kind == JL_MAP_CHUNK && a->map.chunk < 1) return fail(JL_ERR_BAD_ARG, "jl_prefill: chunk must be >= 1");
  if (a->q_batch_wrap < 0 || (a->q_batch_wrap > 0 && (a->q_batch_first < 0 || a->q_batch_first >= a->q_batch_wrap || a->batch > a->q_batch_wrap)))
    return fail(JL_ERR_BAD_ARG, "jl_prefill: stripe batching needs 0 <= q_batch_first < q_batch_wrap and batch <= q_batch_wrap");
  if (a->q_batch_wrap > 0 && a->impl == 1) return fail(JL_ERR_UNSUPPORTED, "jl_prefill: stripe batching needs impl 0 or 2");
  const bool keys = a->seqlen_k > 0;          // an empty key range may come with NULL key / value pointers
  if ((keys && a->v == nullptr) || a->out == nullptr) return fail(JL_ERR_BAD_ARG, "jl_prefill: v/out is NULL");
  uintptr_t bits = reinterpret_cast<uintptr_t>(a->v) | reinterpret_cast<uintptr_t>(a->out);
  for (int c = 0; c < a->map.n_classes; ++c) {
    if (c > 0 && a->remap_far_in_kernel && a->impl != 1) continue;      // formed in-kernel from class 0
    if (a->q[c] == nullptr || (keys && a->k[c] == nullptr)) return fail(JL_ERR_BAD_ARG, "jl_prefill: operand of class %d is NULL", c);
    bits |= reinterpret_cast<uintptr_t>(a->q[c]) | reinterpret_cast<uintptr_t>(a->k[c]);
  }
  if (bits & 15) return fail(JL_ERR_BAD_ARG, "jl_prefill: pointers must be 16-byte aligned");
  const int64_t st[] = {a->q_stride_b, a->q_stride_s, a->q_stride_h, a->k_stride_b, a->k_stride_s, a->k_stride_h,
                        a->v_stride_b, a->v_stride_s, a->v_stride_h, a->o_stride_b, a->o_stride_s, a->o_stride_h};
  for (int64_t x : st)
    if (x % 8 != 0) return fail(JL_ERR_BAD_ARG, "jl_prefill: strides must be multiples of 8 elements (16 bytes)");
  return JL_OK;
}

}  // namespace jl

extern "C" {

int jl_version(void) { return 100; }

const char* jl_status_string(int status) {
  switch (status) {
    case JL_OK: return "ok";
    case JL_ERR_BAD_ARG: return "bad argument";
    case JL_ERR_UNSUPPORTED: return "unsupported configuration";
    case JL_ERR_LAUNCH: return "CUDA launch failure";
    case JL_ERR_ARCH: return "device is not sm_100";
    case JL_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
  }
}

const char* jl_last_error(void) { return jl::g_err; }

int jl_merge(const jl_merge_args* args, void* cuda_stream) {
  if (args == nullptr) return jl::fail(JL_ERR_BAD_ARG, "jl_merge: args is NULL");
  int rc = jl::check_device_arch();
  if (rc != JL_OK) return rc;
  return jl::launch_merge(args, static_cast<cudaStream_t>(cuda_stream));
}

int jl_rotate(const jl_rotate_args* args, void* cuda_stream) {
  if (args == nullptr) return jl::fail(JL_ERR_BAD_ARG, "jl_rotate: args is NULL");
  int rc = jl::check_device_arch();
  if (rc != JL_OK) return rc;
  return jl::launch_rotate(args, static_cast<cudaStream_t>(cuda_stream));
}

int jl_rmsnorm(const jl_rmsnorm_args* args, void* cuda_stream) {
  if (args == nullptr) return jl::fail(JL_ERR_BAD_ARG, "jl_rmsnorm: args is NULL");
  int rc = jl::check_device_arch();
  if (rc != JL_OK) return rc;
  return jl::launch_rmsnorm(args, static_cast<cudaStream_t>(cuda_stream));
}

int jl_norm_rope(const jl_norm_rope_args* args, void* cuda_stream) {
  if (args == nullptr) return jl::fail(JL_ERR_BAD_ARG, "jl_norm_rope: args is NULL");
  int rc = jl::check_device_arch();
  if (rc != JL_OK) return rc;
  return jl::launch_norm_rope(args, static_cast<cudaStream_t>(cuda_stream));
}

size_t jl_peer_merge_buffer_bytes(int32_t world, int32_t batch, int32_t heads, int32_t head_dim) {
  return head_dim == 128 ? jl::peer_merge_buffer_bytes(world, batch, heads) : 0;
}

int jl_peer_merge(const jl_peer_merge_args* args, void* cuda_stream) {
  if (args == nullptr) return jl::fail(JL_ERR_BAD_ARG, "jl_peer_merge: args is NULL");
  int rc = jl::check_device_arch();
  if (rc != JL_OK) return rc;
  return jl::launch_peer_merge(args, static_cast<cudaStream_t>(cuda_stream));
}

int jl_silu_mul(const jl_silu_mul_args* args, void* cuda_stream) {
  if (args == nullptr) return jl::fail(JL_ERR_BAD_ARG, "jl_silu_mul: args is NULL");
  int rc = jl::check_device_arch();
  if (rc != JL_OK) return rc;
  return jl::launch_silu_mul(args, static_cast<cudaStream_t>(cuda_stream));
}

int jl_step_advance(const jl_step_advance_args* args, void* cuda_stream) {
  if (args == nullptr) return jl::fail(JL_ERR_BAD_ARG, "jl_step_advance: args is NULL");
  int rc = jl::check_device_arch();
  if (rc != JL_OK) return rc;
  return jl::launch_step_advance(args, static_cast<cudaStream_t>(cuda_stream));
}

int jl_decode_append(const jl_decode_append_args* args, void* cuda_stream) {
  if (args == nullptr) return jl::fail(JL_ERR_BAD_ARG, "jl_decode_append: args is NULL");
  int rc = jl::check_device_arch();
  if (rc != JL_OK) return rc;
  return jl::launch_decode_append(args, static_cast<cudaStream_t>(cuda_stream));
}

size_t jl_decode_workspace_bytes(int32_t batch, int32_t heads, int32_t head_dim, int32_t max_splits) {
  return jl::decode_workspace_bytes(batch, heads, head_dim, max_splits);
}

int32_t jl_decode_auto_splits(int32_t batch, int32_t kv_heads, int64_t total_keys) {
  return jl::decode_auto_splits(batch, kv_heads, total_keys);
}

int jl_decode(const jl_decode_args* args, void* cuda_stream) {
  if (args == nullptr) return jl::fail(JL_ERR_BAD_ARG, "jl_decode: args is NULL");
  int rc = jl::check_device_arch();
  if (rc != JL_OK) return rc;
  return jl::launch_decode(args, static_cast<cudaStream_t>(cuda_stream));
}

int jl_decode_static(const jl_decode_args* args, void* cuda_stream) {
  if (args == nullptr) return jl::fail(JL_ERR_BAD_ARG, "jl_decode_static: args is NULL");
  int rc = jl::check_device_arch();
  if (rc != JL_OK) return rc;
  return jl::launch_decode_static(args, static_cast<cudaStream_t>(cuda_stream));
}

size_t jl_decode_static_scratch_bytes(void) { return jl::decode_static_scratch_bytes(); }

int jl_prefill_status(void) { return jl::prefill_tc_status(); }

int jl_prefill(const jl_prefill_args* args, void* cuda_stream) {
  int rc = jl::validate_prefill(args);
  if (rc != JL_OK) return rc;
  rc = jl::check_device_arch();
  if (rc != JL_OK) return rc;
  if (args->seqlen_q == 0) return JL_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (args->impl == 1) {                                                  // explicit cross-check kernel only
    if (args->remap_far_in_kernel) return jl::fail(JL_ERR_UNSUPPORTED, "jl_prefill: remap_far_in_kernel needs impl 0");
    return jl::launch_prefill_mma(args, stream);
  }
  if (args->impl == 2) {                                                  // the CTA-pair kernel, asked for by name
    if (const char* why = jl::prefill_pair_unsupported_reason(args))
      return jl::fail(JL_ERR_UNSUPPORTED, "jl_prefill: %s", why);
    return jl::launch_prefill_pair(args, stream);
  }
  if (args->impl != 0) return jl::fail(JL_ERR_BAD_ARG, "jl_prefill: impl must be 0, 1 or 2, got %d", args->impl);
  if (const char* why = jl::prefill_tc_unsupported_reason(args))
    return jl::fail(JL_ERR_UNSUPPORTED, "jl_prefill: %s", why);
  return jl::launch_prefill_tc(args, stream);
}

}  // extern "C"

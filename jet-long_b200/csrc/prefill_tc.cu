// placeholder until the tcgen05 kernel lands: everything routes to the mma.sync kernel
#include "jl_common.cuh"
namespace jl {
bool prefill_tc_supports(const jl_prefill_args*) { return false; }
int launch_prefill_tc(const jl_prefill_args*, cudaStream_t) { return fail(JL_ERR_UNSUPPORTED, "tcgen05 prefill not built"); }
}  // namespace jl

// Placeholder translation unit: the tensor-core prefill kernel is built in its own step.
#include "common.cuh"
namespace bitnet {
bool prefill_supports(size_t, size_t, size_t) { return false; }
size_t prefill_workspace_bytes(size_t, size_t, size_t) { return 0; }
bitnet_status_t launch_prefill(const ForwardArgs &, void *, size_t, cudaStream_t)
{
    return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "prefill kernel not built");
}
}  // namespace bitnet

// C-ABI entry point of the backward pass (placeholder until the kernels land).
#include "b2a_host.cuh"

extern "C" {

size_t b2a_bwd_workspace_bytes(int32_t, int32_t, int32_t, int32_t, int32_t, int32_t) { return 256; }

int b2a_bwd(const b2a_bwd_args*, void*) {
    return b2a::fail(B2A_ERR_INVALID_ARGUMENT, "b2a_bwd is not implemented yet");
}

}  // extern "C"

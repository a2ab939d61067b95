#include "tc_kernels.cuh"

namespace fbla {

bool tc_supported(const KParams&, int) { return false; }
int64_t tc_workspace_bytes(const KParams&) { return 0; }
cudaError_t tc_fwd_state(const KParams&, int, const void*, const void*, const void*, float*, void*,
                         cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t tc_fwd_out(const KParams&, int, const void*, const void*, const float*, void*, cudaStream_t) {
    return cudaErrorNotSupported;
}
cudaError_t tc_bwd_state(const KParams&, int, const void*, const void*, const void*, const float*, void*,
                         void*, float*, void*, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t tc_bwd_in(const KParams&, int, const void*, const void*, const float*, void*, void*, void*,
                      cudaStream_t) { return cudaErrorNotSupported; }

}  // namespace fbla

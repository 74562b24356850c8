#include "lq4_gemm.cuh"

namespace lq4 {

bool gemm_supported(uint32_t, uint32_t, uint32_t, uint32_t) { return false; }
size_t gemm_workspace_bytes(uint32_t, uint32_t, uint32_t, uint32_t) { return 0; }
cudaError_t launch_gemm_tc(const void*, int, const uint8_t*, float*, uint64_t, uint32_t, uint32_t, uint32_t,
                           const float*, const float*, uint32_t, float, void*, size_t, int32_t*, int, cudaStream_t,
                           int*, std::string* err) {
    if (err) *err = "not built";
    return cudaErrorNotSupported;
}

}  // namespace lq4

// Prefill path (m > 16): tcgen05 tensor-core kernel; see lq4_gemm.cu.
#pragma once

#include <string>

#include "lq4_common.cuh"

namespace lq4 {

bool gemm_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t rank);
size_t gemm_workspace_bytes(uint32_t m, uint32_t n, uint32_t k, uint32_t rank);
// x is [m, k] f32 or bf16 (already rotated if a rotation applies); y is overwritten.
cudaError_t launch_gemm_tc(const void* x, int x_dtype, const uint8_t* w, float* y, uint64_t ldy, uint32_t m,
                           uint32_t n, uint32_t k, const float* la, const float* lb, uint32_t rank, float lscale,
                           void* workspace, size_t workspace_bytes, int32_t* status, int sm_count, cudaStream_t s,
                           int* launches, std::string* err, const int64_t* peer_off = nullptr, uint32_t n_peers = 0);
// peer_off[0 .. n_peers): byte offsets from an element of y to the same element of each peer's output buffer; the
// epilogue then stores every result there as well (fused all-gather of an N-sharded product).

}  // namespace lq4

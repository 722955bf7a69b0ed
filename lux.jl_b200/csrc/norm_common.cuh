// Helpers shared by the row-normalisation kernels (layernorm.cu, groupnorm.cu).
#pragma once
#include "common.cuh"

namespace lb2 {

template <int RT> __device__ __forceinline__ float row_sum(float v, float* smem) {
  if constexpr (RT == 32) return warp_sum(v);
  else return block_sum(v, smem);
}

inline int32_t check_norm_common(const void* y, const void* x, const void* gamma, const void* beta,
                                 const float* sm, const float* si, int32_t dtype, int32_t act) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(valid_act(act), LB2_BAD_ARG, "unknown activation %d", (int)act);
  LB2_REQUIRE(y && x && sm && si, LB2_BAD_ARG, "null tensor pointer");
  LB2_REQUIRE((gamma == nullptr) == (beta == nullptr), LB2_BAD_ARG, "scale and bias must both be given or both be null");
  const size_t es = dtype_size(dtype);
  LB2_REQUIRE(aligned_to(y, es) && aligned_to(x, es) && aligned_to(gamma, es) && aligned_to(beta, es) &&
                  aligned_to(sm, 4) && aligned_to(si, 4),
              LB2_BAD_ALIGN, "pointer not aligned to the element size");
  return LB2_OK;
}

}  // namespace lb2

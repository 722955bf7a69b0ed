// Internal interface of eltwise.cu, shared with the dense and conv pullbacks.
#pragma once
#include "common.cuh"

namespace lb2 {

// dx = dy .* act'(out | pre) on the (S, C, B) view (S == 1: C x B matrices with leading
// dimensions ld_*), and, when db != nullptr, db[c] (+)= sum_{s,b} dx through the fp32 partials
// in `ws` (act_bwd_workspace_bytes). dx may be nullptr when only the sum is wanted.
int32_t launch_act_bwd(void* dx, void* db, const void* dy, const void* out, const void* pre, int64_t S,
                       int64_t C, int64_t B, int64_t ld_dx, int64_t ld_dy, int64_t ld_ref, int32_t dtype,
                       int32_t act, int accumulate_db, float* ws, cudaStream_t st);
size_t act_bwd_workspace_bytes(int64_t S, int64_t C, int64_t B);
int32_t check_act_bwd_args(const void* dy, const void* out, const void* pre, int32_t dtype, int32_t act);

}  // namespace lb2

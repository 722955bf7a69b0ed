// Internal GEMM interface shared by the dense, matmul and convolution entry points.
//
// Every contraction is expressed as  D[Mm x Nn] = A[Mm x Kc] * B[Nn x Kc]^T  with D stored
// column-major (Mm contiguous, leading dimension ldd). An operand is "MN-major" when its
// non-contracted index is the contiguous one (element (i,k) at i + k*ld) and "K-major" when the
// contracted index is contiguous (element (i,k) at k + i*ld). Julia's W*x is A = W (MN-major),
// B = x (K-major); W'*g is both K-major; g*x' is both MN-major.
#pragma once
#include "common.cuh"

namespace lb2 {

struct GemmOperand {
  const void* ptr;
  int64_t ld;
  bool mn_major;
};

struct GemmEpilogue {
  const void* bias = nullptr;  // length Mm (broadcast along Nn), storage dtype; may be null
  int32_t act = LB2_ACT_IDENTITY;
  void* preact = nullptr;      // optional store of (acc + bias) before the activation; ld = ldd
  int32_t accumulate = 0;      // D += result (activation must be identity)
};

// CUDA-core tiled GEMM: any shape, any leading dimension, exact fp32 accumulation.
int32_t gemm_simt_launch(void* D, int64_t ldd, GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc,
                         int32_t dtype, const GemmEpilogue& epi, cudaStream_t st, int batch = 1, int64_t bs_a = 0, int64_t bs_b = 0,
                         int64_t bs_d = 0);

// tcgen05 / TMEM / TMA GEMM. `tc_supported` tells whether the pointers and leading dimensions
// satisfy the TMA rules (16-byte aligned bases, strides multiple of 16 bytes).
bool gemm_tc_supported(const void* D, int64_t ldd, GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc,
                       int32_t dtype, int split3);
// fp32 storage: split3 != 0 runs the error-compensated 3xTF32 scheme and needs
// gemm_tc_split_workspace_bytes(...) bytes of scratch for the hi/lo operand copies.
size_t gemm_tc_split_workspace_bytes(GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc);
int32_t gemm_tc_launch(void* D, int64_t ldd, GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc,
                       int32_t dtype, int split3, uint32_t flags, const GemmEpilogue& epi, void* split_ws,
                       cudaStream_t st);

// Picks the tensor-core kernel when it applies, the CUDA-core kernel otherwise.
size_t gemm_workspace_bytes(GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc, int32_t dtype,
                            uint32_t flags);
int32_t gemm_dispatch(void* D, int64_t ldd, GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc,
                      int32_t dtype, uint32_t flags, const GemmEpilogue& epi, void* ws, size_t ws_bytes,
                      cudaStream_t st);

extern thread_local int32_t g_last_gemm_plan[8];   // see gemm_tc.cu

}  // namespace lb2

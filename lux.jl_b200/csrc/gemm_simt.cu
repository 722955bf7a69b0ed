// CUDA-core GEMM used for shapes the tensor-core kernel cannot take (leading dimensions that
// break the 16-byte TMA stride rule, tiny problems) and as the exact-fp32 route.
// D[Mm x Nn] = A[Mm x Kc] * B[Nn x Kc]^T, fp32 accumulation in a fixed k order (deterministic),
// 64x64 tile per CTA, 4x4 micro-tile per thread, bias + activation fused in the epilogue.
#include "gemm.cuh"

namespace lb2 {

template <typename T, int ACT>
__global__ void __launch_bounds__(256) gemm_simt_kernel(T* __restrict__ D, int64_t ldd, const T* __restrict__ A,
                                                        int64_t sa_m, int64_t sa_k, const T* __restrict__ B,
                                                        int64_t sb_n, int64_t sb_k, int64_t Mm, int64_t Nn, int64_t Kc,
                                                        const T* __restrict__ bias, T* __restrict__ preact,
                                                        int accumulate, int64_t bs_a, int64_t bs_b, int64_t bs_d) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int TM = 64, TN = 64, TK = 16;
  // blockIdx.z = batch element (strides in elements; 0 repeats an operand)
  A += (int64_t)blockIdx.z * bs_a;
  B += (int64_t)blockIdx.z * bs_b;
  D += (int64_t)blockIdx.z * bs_d;
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;  // tx -> m micro-tile, ty -> n micro-tile
  const int64_t m0 = (int64_t)blockIdx.x * TM, n0 = (int64_t)blockIdx.y * TN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int64_t k0 = 0; k0 < Kc; k0 += TK) {
    // 64 x 16 elements per operand, 4 per thread. Index so that the contiguous global
    // dimension is walked by consecutive threads whichever way the operand is stored.
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int idx = tid + r * 256;
      int mi, ki;
      if (sa_m == 1) { mi = idx % TM; ki = idx / TM; } else { ki = idx % TK; mi = idx / TK; }
      const int64_t m = m0 + mi, k = k0 + ki;
      As[ki][mi] = (m < Mm && k < Kc) ? to_f32(A[m * sa_m + k * sa_k]) : 0.f;
      int ni, kj;
      if (sb_n == 1) { ni = idx % TN; kj = idx / TN; } else { kj = idx % TK; ni = idx / TK; }
      const int64_t n = n0 + ni, kk = k0 + kj;
      Bs[kj][ni] = (n < Nn && kk < Kc) ? to_f32(B[n * sb_n + kk * sb_k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][tx * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][ty * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int64_t n = n0 + ty * 4 + j;
    if (n >= Nn) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t m = m0 + tx * 4 + i;
      if (m >= Mm) continue;
      float v = acc[i][j];
      if (bias) v += to_f32(bias[m]);
      if (preact) preact[n * ldd + m] = from_f32<T>(v);
      v = act_apply<ACT, FAST>(v);
      if (accumulate) v += to_f32(D[n * ldd + m]);
      D[n * ldd + m] = from_f32<T>(v);
    }
  }
}

int32_t gemm_simt_launch(void* D, int64_t ldd, GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc,
                         int32_t dtype, const GemmEpilogue& epi, cudaStream_t st, int batch, int64_t bs_a, int64_t bs_b,
                         int64_t bs_d) {
  if (Mm == 0 || Nn == 0 || batch <= 0) return LB2_OK;
  LB2_REQUIRE(batch <= 65535, LB2_BAD_SHAPE, "CUDA-core GEMM: more than 65535 batch elements in one launch");
  dim3 grid((unsigned)((Mm + 63) / 64), (unsigned)((Nn + 63) / 64), (unsigned)batch);
  LB2_REQUIRE(grid.y <= 65535, LB2_BAD_SHAPE, "CUDA-core GEMM: N extent too large (%lld)", (long long)Nn);
  const int64_t sa_m = A.mn_major ? 1 : A.ld, sa_k = A.mn_major ? A.ld : 1;
  const int64_t sb_n = B.mn_major ? 1 : B.ld, sb_k = B.mn_major ? B.ld : 1;
  LB2_DISPATCH_DTYPE(dtype, {
    LB2_DISPATCH_ACT(epi.act, {
      gemm_simt_kernel<T, ACT><<<grid, 256, 0, st>>>((T*)D, ldd, (const T*)A.ptr, sa_m, sa_k, (const T*)B.ptr, sb_n,
                                                     sb_k, Mm, Nn, Kc, (const T*)epi.bias, (T*)epi.preact,
                                                     epi.accumulate, bs_a, bs_b, bs_d);
    });
  });
  LB2_CHECK_LAUNCH("gemm_simt");
  return LB2_OK;
}

}  // namespace lb2

// Batched matrix product and the softmax of scaled-dot-product attention: the pieces LuxLib composes in
// lib/LuxLib/src/impl/attention.jl:76-118 (batched_matmul(k, q .* scale) -> mask / bias -> softmax(dims = 1) ->
// batched_matmul(v, weights)) and lib/LuxLib/src/impl/batched_mul.jl:1-60.
//
// lb2_batched_matmul: C[:, :, i] = op(A[:, :, i]) * op(B[:, :, i]) for i < batch, each operand with its own leading
// dimension and batch stride (a stride of 0 repeats the matrix: the "size-1 batch dimension" case of the reference and
// the shared key / value heads of grouped-query attention). Small products (the usual attention tiles) run as ONE launch
// of the CUDA-core GEMM with the batch index on the grid's z axis; large ones go to the tensor-core GEMM per element.
//
// Attention softmax over the key index s of logits[s, l, hb]: y = softmax_s(mask ? scale * logits + bias : -inf), one
// warp per (l, hb) column, three passes over a column that stays in L1. Backward: dlogits = scale * y .* (dy - sum_s y dy),
// optionally dbias = y .* (dy - sum_s y dy).
#include "common.cuh"
#include "gemm.cuh"

namespace lb2 {

template <typename T>
__global__ void __launch_bounds__(256) attn_softmax_fwd_kernel(T* __restrict__ y, const T* __restrict__ logits, const T* __restrict__ bias,
                                                               int64_t bias_bs, const uint8_t* __restrict__ mask, int64_t mask_bs,
                                                               int causal, float scale, int64_t S, int64_t L, int64_t cols) {
  const int lane = threadIdx.x & 31;
  const int64_t col = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (col >= cols) return;
  const int64_t l = col % L, hb = col / L;
  const T* z = logits + col * S;
  const T* bz = bias != nullptr ? bias + hb * bias_bs + l * S : nullptr;
  const uint8_t* mz = mask != nullptr ? mask + hb * mask_bs + l * S : nullptr;
  T* out = y + col * S;
  auto value = [&](int64_t s) {
    float v = to_f32(z[s]) * scale;
    if (bz != nullptr) v += to_f32(bz[s]);
    const bool keep = (mz == nullptr || mz[s] != 0) && (!causal || s <= l);   // causal mask = triu(trues(S, L)): key s <= query l
    return keep ? v : -INFINITY;
  };
  float m = -INFINITY;
  for (int64_t s = lane; s < S; s += 32) m = fmaxf(m, value(s));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float se = 0.f;
  for (int64_t s = lane; s < S; s += 32) se += expf(value(s) - m);
  se = warp_sum(se);
  const float inv = 1.f / se;
  for (int64_t s = lane; s < S; s += 32) out[s] = from_f32<T>(expf(value(s) - m) * inv);
}

template <typename T>
__global__ void __launch_bounds__(256) attn_softmax_bwd_kernel(T* __restrict__ dlogits, T* __restrict__ dbias, const T* __restrict__ dy,
                                                               const T* __restrict__ y, float scale, int64_t S, int64_t cols) {
  const int lane = threadIdx.x & 31;
  const int64_t col = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (col >= cols) return;
  const T* yy = y + col * S;
  const T* gg = dy + col * S;
  float dot = 0.f;
  for (int64_t s = lane; s < S; s += 32) dot = fmaf(to_f32(yy[s]), to_f32(gg[s]), dot);
  dot = warp_sum(dot);
  for (int64_t s = lane; s < S; s += 32) {
    const float d = to_f32(yy[s]) * (to_f32(gg[s]) - dot);
    if (dlogits != nullptr) dlogits[col * S + s] = from_f32<T>(d * scale);
    if (dbias != nullptr) dbias[col * S + s] = from_f32<T>(d);
  }
}

}  // namespace lb2

using namespace lb2;

extern "C" {

size_t lb2_batched_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t dtype, uint32_t flags) {
  return lb2_matmul_workspace_bytes(M, N, K, dtype, flags);
}

int32_t lb2_batched_matmul(void* C, const void* A, const void* B, int64_t M, int64_t N, int64_t K, int64_t batch, int64_t lda,
                           int64_t ldb, int64_t ldc, int64_t stride_a, int64_t stride_b, int64_t stride_c, int32_t transA,
                           int32_t transB, int32_t dtype, int32_t accumulate, uint32_t flags, void* workspace,
                           size_t workspace_bytes, void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(M >= 0 && N >= 0 && K >= 0 && batch >= 0, LB2_BAD_SHAPE, "negative extent");
  LB2_REQUIRE(stride_a >= 0 && stride_b >= 0 && stride_c >= 0, LB2_BAD_SHAPE, "negative batch stride");
  if (M == 0 || N == 0 || batch == 0) return LB2_OK;
  LB2_REQUIRE(batch == 1 || stride_c >= 1, LB2_BAD_SHAPE, "the results of different batch elements must not overlap (stride_c = 0)");
  const int64_t a_rows = transA ? K : M, b_rows = transB ? N : K;
  LB2_REQUIRE(lda >= (a_rows > 1 ? a_rows : 1) && ldb >= (b_rows > 1 ? b_rows : 1) && ldc >= M, LB2_BAD_SHAPE,
              "leading dimension smaller than the number of rows");
  LB2_REQUIRE(C != nullptr && (K == 0 || (A != nullptr && B != nullptr)), LB2_BAD_ARG, "null tensor pointer");
  const size_t es = dtype_size(dtype);
  LB2_REQUIRE(aligned_to(C, es) && aligned_to(A, es) && aligned_to(B, es), LB2_BAD_ALIGN, "pointer not aligned to the element size");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool small = (double)M * (double)N * (double)K < 256.0 * 256.0 * 256.0 || (flags & LB2_FLAG_FORCE_SIMT);
  if (K > 0 && small) {
    GemmEpilogue epi;
    epi.accumulate = accumulate;
    for (int64_t b0 = 0; b0 < batch; b0 += 65535) {
      const int nb = (int)(batch - b0 < 65535 ? batch - b0 : 65535);
      GemmOperand a{static_cast<const uint8_t*>(A) + (size_t)(b0 * stride_a) * es, lda, transA == 0};
      GemmOperand b{static_cast<const uint8_t*>(B) + (size_t)(b0 * stride_b) * es, ldb, transB != 0};
      int32_t rc = gemm_simt_launch(static_cast<uint8_t*>(C) + (size_t)(b0 * stride_c) * es, ldc, a, b, M, N, K, dtype, epi, st, nb,
                                    stride_a, stride_b, stride_c);
      if (rc != LB2_OK) return rc;
    }
    return LB2_OK;
  }
  for (int64_t i = 0; i < batch; ++i) {
    int32_t rc = lb2_matmul(static_cast<uint8_t*>(C) + (size_t)(i * stride_c) * es, static_cast<const uint8_t*>(A) + (size_t)(i * stride_a) * es,
                            static_cast<const uint8_t*>(B) + (size_t)(i * stride_b) * es, M, N, K, lda, ldb, ldc, transA, transB, dtype,
                            accumulate, flags, workspace, workspace_bytes, stream);
    if (rc != LB2_OK) return rc;
  }
  return LB2_OK;
}

int32_t lb2_attention_softmax_fwd(void* y, const void* logits, const void* bias, int64_t bias_batch_stride, const uint8_t* mask,
                                  int64_t mask_batch_stride, int32_t causal, double scale, int64_t S, int64_t L, int64_t HB,
                                  int32_t dtype, void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(S >= 0 && L >= 0 && HB >= 0, LB2_BAD_SHAPE, "negative extent");
  LB2_REQUIRE(bias_batch_stride == 0 || bias_batch_stride == S * L, LB2_BAD_SHAPE, "bias batch stride must be 0 or S*L");
  LB2_REQUIRE(mask_batch_stride == 0 || mask_batch_stride == S * L, LB2_BAD_SHAPE, "mask batch stride must be 0 or S*L");
  if (S == 0 || L == 0 || HB == 0) return LB2_OK;
  LB2_REQUIRE(y != nullptr && logits != nullptr, LB2_BAD_ARG, "null tensor pointer");
  const size_t es = dtype_size(dtype);
  LB2_REQUIRE(aligned_to(y, es) && aligned_to(logits, es) && aligned_to(bias, es), LB2_BAD_ALIGN, "pointer not aligned to the element size");
  const int64_t cols = L * HB;
  LB2_REQUIRE((cols + 7) / 8 <= 0x7FFFFFFF, LB2_BAD_SHAPE, "too many columns");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LB2_DISPATCH_DTYPE(dtype, {
    attn_softmax_fwd_kernel<T><<<(unsigned)((cols + 7) / 8), 256, 0, st>>>((T*)y, (const T*)logits, (const T*)bias, bias_batch_stride, mask,
                                                                           mask_batch_stride, causal, (float)scale, S, L, cols);
  });
  LB2_CHECK_LAUNCH("attention softmax");
  return LB2_OK;
}

int32_t lb2_attention_softmax_bwd(void* dlogits, void* dbias, const void* dy, const void* y, double scale, int64_t S, int64_t L,
                                  int64_t HB, int32_t dtype, void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(S >= 0 && L >= 0 && HB >= 0, LB2_BAD_SHAPE, "negative extent");
  if (S == 0 || L == 0 || HB == 0) return LB2_OK;
  LB2_REQUIRE((dlogits != nullptr || dbias != nullptr) && dy != nullptr && y != nullptr, LB2_BAD_ARG, "null tensor pointer");
  const size_t es = dtype_size(dtype);
  LB2_REQUIRE(aligned_to(dlogits, es) && aligned_to(dbias, es) && aligned_to(dy, es) && aligned_to(y, es), LB2_BAD_ALIGN,
              "pointer not aligned to the element size");
  const int64_t cols = L * HB;
  LB2_REQUIRE((cols + 7) / 8 <= 0x7FFFFFFF, LB2_BAD_SHAPE, "too many columns");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LB2_DISPATCH_DTYPE(dtype, {
    attn_softmax_bwd_kernel<T><<<(unsigned)((cols + 7) / 8), 256, 0, st>>>((T*)dlogits, (T*)dbias, (const T*)dy, (const T*)y, (float)scale, S, cols);
  });
  LB2_CHECK_LAUNCH("attention softmax backward");
  return LB2_OK;
}

}  // extern "C"

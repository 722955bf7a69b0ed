// Mean-squared-error loss and its gradient in one pass: MSELoss() of src/helpers/losses.jl:659 =
// GenericLossFunction(l2_distance_loss; agg = mean) with derivative 2*(x - y) (src/helpers/losses.jl:121-125), the
// loss the reference's own ResNet harness differentiates. loss = mean((yhat - y)^2), dyhat = 2*(yhat - y)/n.
// Bandwidth-bound (2 reads, 1 write per element); the sum is formed per CTA and then in a fixed order by one CTA
// (deterministic, no atomics).
#include "common.cuh"

namespace lb2 {

constexpr int kLossBlocks = 256;

template <typename T>
__global__ void __launch_bounds__(256) mse_partial_kernel(T* __restrict__ dyhat, float* __restrict__ partial,
                                                          const T* __restrict__ yhat, const T* __restrict__ y, int64_t n) {
  __shared__ float red[32];
  const float scale = 2.f / (float)n;
  float acc = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float d = to_f32(yhat[i]) - to_f32(y[i]);
    acc = fmaf(d, d, acc);
    if (dyhat != nullptr) dyhat[i] = from_f32<T>(d * scale);
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

__global__ void __launch_bounds__(256) mse_finish_kernel(float* __restrict__ loss, const float* __restrict__ partial, int blocks,
                                                         int64_t n) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < blocks; i += blockDim.x) acc += partial[i];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) *loss = acc / (float)n;
}

// CrossEntropyLoss(; dims = 1, agg = mean) of src/helpers/losses.jl:383-416 on a (K classes, B columns) column-major
// pair of arrays, one warp per column. logits = Val(true) (:408-412): loss = mean_b( -sum_k yt[k,b] * logsoftmax(yhat)[k,b] )
// with gradient (softmax(yhat) * sum_k yt - yt) / B; logits = Val(false) (:414-416): loss = mean_b( -sum_k xlogy(yt, yhat + eps) )
// with gradient -yt / (yhat + eps) / B. yt = label smoothing of y (src/helpers/losses.jl:172-177):
// (1 - alpha) * y + alpha / K. The per-column terms go to a workspace and are summed in a fixed order by one CTA.
template <typename T, bool LOGITS>
__global__ void __launch_bounds__(256) xent_columns_kernel(T* __restrict__ dyhat, float* __restrict__ terms, const T* __restrict__ yhat,
                                                           const T* __restrict__ y, int64_t K, int64_t B, float alpha, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t col = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (col >= B) return;
  const T* zh = yhat + col * K;
  const T* yy = y + col * K;
  T* dz = dyhat != nullptr ? dyhat + col * K : nullptr;
  const float smooth = alpha / (float)K, keep = 1.f - alpha, invB = 1.f / (float)B;
  if constexpr (LOGITS) {
    float m = -INFINITY;
    for (int64_t k = lane; k < K; k += 32) m = fmaxf(m, to_f32(zh[k]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float se = 0.f, sy = 0.f, syz = 0.f;
    for (int64_t k = lane; k < K; k += 32) {
      const float z = to_f32(zh[k]) - m, t = fmaf(keep, to_f32(yy[k]), smooth);
      se += expf(z);
      sy += t;
      syz = fmaf(t, z, syz);
    }
    se = warp_sum(se); sy = warp_sum(sy); syz = warp_sum(syz);
    const float lse = logf(se);
    if (lane == 0) terms[col] = fmaf(sy, lse, -syz);            // -sum t * (z - lse)
    if (dz != nullptr) {
      const float scale = sy * invB / se;
      for (int64_t k = lane; k < K; k += 32) {
        const float z = to_f32(zh[k]) - m, t = fmaf(keep, to_f32(yy[k]), smooth);
        dz[k] = from_f32<T>(fmaf(expf(z), scale, -t * invB));
      }
    }
  } else {
    float acc = 0.f;
    for (int64_t k = lane; k < K; k += 32) {
      const float p = to_f32(zh[k]) + eps, t = fmaf(keep, to_f32(yy[k]), smooth);
      acc -= t == 0.f ? 0.f : t * logf(p);                        // xlogy: zero where the target is zero
      if (dz != nullptr) dz[k] = from_f32<T>(-t / p * invB);
    }
    acc = warp_sum(acc);
    if (lane == 0) terms[col] = acc;
  }
}

__global__ void __launch_bounds__(256) xent_finish_kernel(float* __restrict__ loss, const float* __restrict__ terms, int64_t B) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int64_t i = threadIdx.x; i < B; i += blockDim.x) acc += terms[i];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) *loss = acc / (float)B;
}

}  // namespace lb2

using namespace lb2;

extern "C" {

size_t lb2_mse_loss_workspace_bytes(int64_t n) { return n > 0 ? (size_t)kLossBlocks * sizeof(float) : 0; }

int32_t lb2_mse_loss(float* loss, void* dyhat, const void* yhat, const void* y, int64_t n, int32_t dtype, void* workspace,
                     size_t workspace_bytes, void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(n >= 0, LB2_BAD_SHAPE, "negative length");
  LB2_REQUIRE(loss != nullptr, LB2_BAD_ARG, "loss is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n == 0) {   // mean over nothing: NaN in the reference (0/0); reported as such
    const float nanv = __builtin_nanf("");
    cudaMemcpyAsync(loss, &nanv, sizeof(float), cudaMemcpyHostToDevice, st);
    return LB2_OK;
  }
  LB2_REQUIRE(yhat && y, LB2_BAD_ARG, "null tensor pointer");
  const size_t es = dtype_size(dtype);
  LB2_REQUIRE(aligned_to(dyhat, es) && aligned_to(yhat, es) && aligned_to(y, es) && aligned_to(loss, 4), LB2_BAD_ALIGN,
              "pointer not aligned to the element size");
  LB2_REQUIRE(workspace && workspace_bytes >= lb2_mse_loss_workspace_bytes(n), LB2_WORKSPACE_TOO_SMALL, "workspace of %zu bytes needed",
              lb2_mse_loss_workspace_bytes(n));
  LB2_REQUIRE(aligned_to(workspace, 4), LB2_BAD_ALIGN, "workspace must be 4-byte aligned");
  float* partial = static_cast<float*>(workspace);
  int64_t want = (n + 255) / 256;
  const int blocks = (int)(want < kLossBlocks ? want : kLossBlocks);
  LB2_DISPATCH_DTYPE(dtype, { mse_partial_kernel<T><<<blocks, 256, 0, st>>>((T*)dyhat, partial, (const T*)yhat, (const T*)y, n); });
  LB2_CHECK_LAUNCH("mse_loss");
  mse_finish_kernel<<<1, 256, 0, st>>>(loss, partial, blocks, n);
  LB2_CHECK_LAUNCH("mse_loss finish");
  return LB2_OK;
}

size_t lb2_cross_entropy_workspace_bytes(int64_t K, int64_t B) { return (K > 0 && B > 0) ? align_up((size_t)B * sizeof(float), 256) : 0; }

int32_t lb2_cross_entropy(float* loss, void* dyhat, const void* yhat, const void* y, int64_t K, int64_t B, int32_t from_logits,
                          double label_smoothing, double epsilon, int32_t dtype, void* workspace, size_t workspace_bytes,
                          void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(K >= 0 && B >= 0, LB2_BAD_SHAPE, "negative extent");
  LB2_REQUIRE(label_smoothing >= 0.0 && label_smoothing <= 1.0, LB2_BAD_ARG, "label_smoothing must lie in [0, 1]");
  LB2_REQUIRE(loss != nullptr, LB2_BAD_ARG, "loss is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (K == 0 || B == 0) {   // mean over nothing: NaN in the reference (0/0)
    const float nanv = __builtin_nanf("");
    cudaMemcpyAsync(loss, &nanv, sizeof(float), cudaMemcpyHostToDevice, st);
    return LB2_OK;
  }
  LB2_REQUIRE(yhat && y, LB2_BAD_ARG, "null tensor pointer");
  const size_t es = dtype_size(dtype);
  LB2_REQUIRE(aligned_to(dyhat, es) && aligned_to(yhat, es) && aligned_to(y, es) && aligned_to(loss, 4), LB2_BAD_ALIGN,
              "pointer not aligned to the element size");
  LB2_REQUIRE(workspace && workspace_bytes >= lb2_cross_entropy_workspace_bytes(K, B), LB2_WORKSPACE_TOO_SMALL,
              "workspace of %zu bytes needed", lb2_cross_entropy_workspace_bytes(K, B));
  LB2_REQUIRE(aligned_to(workspace, 4), LB2_BAD_ALIGN, "workspace must be 4-byte aligned");
  float* terms = static_cast<float*>(workspace);
  const unsigned grid = (unsigned)((B + 7) / 8);
  LB2_DISPATCH_DTYPE(dtype, {
    if (from_logits) xent_columns_kernel<T, true><<<grid, 256, 0, st>>>((T*)dyhat, terms, (const T*)yhat, (const T*)y, K, B, (float)label_smoothing, (float)epsilon);
    else xent_columns_kernel<T, false><<<grid, 256, 0, st>>>((T*)dyhat, terms, (const T*)yhat, (const T*)y, K, B, (float)label_smoothing, (float)epsilon);
  });
  LB2_CHECK_LAUNCH("cross_entropy");
  xent_finish_kernel<<<1, 256, 0, st>>>(loss, terms, B);
  LB2_CHECK_LAUNCH("cross_entropy finish");
  return LB2_OK;
}

}  // extern "C"

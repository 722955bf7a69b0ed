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

}  // extern "C"

// Optimiser step for a whole bucket of parameter leaves in one launch, meant to run right after the
// bucket's gradient all-reduce (the leaf loop of Optimisers.update! driven by
// DistributedOptimizer, src/distributed/public_api.jl:270-278, src/helpers/training.jl:241-245).
// The 1/world averaging of the all-reduce is folded in as `grad_scale`, so the collective can be a
// plain sum. Rules follow Optimisers.jl 0.4.6 (a dependency of the reference, not vendored):
//   Descent:   x -= eta * g
//   Momentum:  v = rho * v + eta * g;                      x -= v
//   Adam:      m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;
//              x -= eta * (m / (1 - b1^t)) / (sqrt(v / (1 - b2^t)) + eps)
// State arrays have the parameter's element type, as in Optimisers.jl; an optional fp32 master copy
// of a bf16 parameter is updated instead of the rounded value and the parameter is re-rounded from it.
// Bandwidth-bound: algorithmic bytes per element = (2 + 2*states) * sizeof(T) + grad read.
#include "common.cuh"

namespace lb2 {

constexpr int kOptMaxLeaves = 48;
constexpr int kOptChunk = 256 * 16;   // elements per CTA step

struct OptBucket {
  void* param[kOptMaxLeaves];
  const void* grad[kOptMaxLeaves];
  void* s1[kOptMaxLeaves];
  void* s2[kOptMaxLeaves];
  float* master[kOptMaxLeaves];
  int64_t n[kOptMaxLeaves];
  int32_t first_block[kOptMaxLeaves + 1];   // prefix sum of ceil(n / kOptChunk)
  int32_t n_leaves;
  int32_t rule;
  float eta, rho, beta1, beta2, eps, bc1, bc2, grad_scale;
};

template <typename T>
__global__ void __launch_bounds__(256) opt_step_kernel(const __grid_constant__ OptBucket bk) {
  // which leaf does this block work on: binary search over the prefix table
  int lo = 0, hi = bk.n_leaves;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if ((int)blockIdx.x >= bk.first_block[mid]) lo = mid; else hi = mid;
  }
  const int leaf = lo;
  const int64_t n = bk.n[leaf];
  const int64_t begin = (int64_t)(blockIdx.x - bk.first_block[leaf]) * kOptChunk;
  const int64_t end = begin + kOptChunk < n ? begin + kOptChunk : n;
  T* p = static_cast<T*>(bk.param[leaf]);
  const T* g = static_cast<const T*>(bk.grad[leaf]);
  T* s1 = static_cast<T*>(bk.s1[leaf]);
  T* s2 = static_cast<T*>(bk.s2[leaf]);
  float* master = bk.master[leaf];
  for (int64_t i = begin + threadIdx.x; i < end; i += 256) {
    const float gi = to_f32(g[i]) * bk.grad_scale;
    float x = master != nullptr ? master[i] : to_f32(p[i]);
    if (bk.rule == LB2_OPT_DESCENT) {
      x -= bk.eta * gi;
    } else if (bk.rule == LB2_OPT_MOMENTUM) {
      const float v = bk.rho * to_f32(s1[i]) + bk.eta * gi;
      s1[i] = from_f32<T>(v);
      x -= to_f32(s1[i]);   // the stored (rounded) velocity is what Optimisers.jl subtracts
    } else {
      const float m = bk.beta1 * to_f32(s1[i]) + (1.f - bk.beta1) * gi;
      const float v = bk.beta2 * to_f32(s2[i]) + (1.f - bk.beta2) * gi * gi;
      s1[i] = from_f32<T>(m);
      s2[i] = from_f32<T>(v);
      const float mr = to_f32(s1[i]), vr = to_f32(s2[i]);
      x -= mr / bk.bc1 / (sqrtf(vr / bk.bc2) + bk.eps) * bk.eta;
    }
    if (master != nullptr) master[i] = x;
    p[i] = from_f32<T>(x);
  }
}

}  // namespace lb2

using namespace lb2;

extern "C" {

int32_t lb2_optimizer_step(const lb2_opt_leaf* leaves, int32_t n_leaves, int32_t rule, double eta, double rho_or_beta1,
                           double beta2, double eps, int64_t step, double grad_scale, int32_t dtype, void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(rule == LB2_OPT_DESCENT || rule == LB2_OPT_MOMENTUM || rule == LB2_OPT_ADAM, LB2_BAD_ARG, "unknown optimiser rule %d", (int)rule);
  LB2_REQUIRE(n_leaves >= 0 && (n_leaves == 0 || leaves != nullptr), LB2_BAD_ARG, "bad leaf list");
  LB2_REQUIRE(step >= 1, LB2_BAD_ARG, "step counts from 1");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t es = dtype_size(dtype);
  // Adam: 1 - beta^t, with beta^t built up as a running float product the way Optimisers.jl carries it in its
  // state. Computed once per call; the loop stops as soon as both products have underflowed to zero (about 1e5
  // steps for beta = 0.999), so its cost does not grow with the step count.
  float bc1 = 1.f, bc2 = 1.f;
  if (rule == LB2_OPT_ADAM) {
    float b1t = 1.f, b2t = 1.f;
    for (int64_t k = 0; k < step && (b1t != 0.f || b2t != 0.f); ++k) { b1t *= (float)rho_or_beta1; b2t *= (float)beta2; }
    bc1 = 1.f - b1t; bc2 = 1.f - b2t;
  }
  int32_t done = 0;
  while (done < n_leaves) {
    OptBucket bk{};
    bk.rule = rule;
    bk.eta = (float)eta; bk.rho = (float)rho_or_beta1; bk.beta1 = (float)rho_or_beta1; bk.beta2 = (float)beta2; bk.eps = (float)eps;
    bk.bc1 = bc1; bk.bc2 = bc2;
    bk.grad_scale = (float)grad_scale;
    int32_t blocks = 0, k = 0;
    for (; k < kOptMaxLeaves && done + k < n_leaves; ++k) {
      const lb2_opt_leaf& lf = leaves[done + k];
      LB2_REQUIRE(lf.n >= 0, LB2_BAD_SHAPE, "negative leaf length");
      LB2_REQUIRE(lf.n == 0 || (lf.param && lf.grad), LB2_BAD_ARG, "leaf %d: null parameter or gradient", (int)(done + k));
      LB2_REQUIRE(lf.n == 0 || rule == LB2_OPT_DESCENT || lf.state1, LB2_BAD_ARG, "leaf %d: optimiser state missing", (int)(done + k));
      LB2_REQUIRE(lf.n == 0 || rule != LB2_OPT_ADAM || lf.state2, LB2_BAD_ARG, "leaf %d: second Adam moment missing", (int)(done + k));
      LB2_REQUIRE(aligned_to(lf.param, es) && aligned_to(lf.grad, es) && aligned_to(lf.state1, es) && aligned_to(lf.state2, es) &&
                      aligned_to(lf.master, 4),
                  LB2_BAD_ALIGN, "leaf %d: pointer not aligned to its element size", (int)(done + k));
      const int64_t nb = (lf.n + kOptChunk - 1) / kOptChunk;
      LB2_REQUIRE(nb < (1 << 30) - blocks, LB2_BAD_SHAPE, "bucket too large for one launch");
      bk.param[k] = lf.param; bk.grad[k] = lf.grad; bk.s1[k] = lf.state1; bk.s2[k] = lf.state2; bk.master[k] = lf.master;
      bk.n[k] = lf.n;
      bk.first_block[k] = blocks;
      blocks += (int32_t)nb;
    }
    bk.first_block[k] = blocks;
    bk.n_leaves = k;
    if (blocks > 0) {
      LB2_DISPATCH_DTYPE(dtype, { opt_step_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(bk); });
      LB2_CHECK_LAUNCH("optimizer_step");
    }
    done += k;
  }
  return LB2_OK;
}

}  // extern "C"

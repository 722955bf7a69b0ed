// The Scale layer's computation (src/layers/basic.jl:452-461): y = act.(x .* weight .+ bias), weight and bias of the
// layer's `dims`, x of shape (dims..., batch...), broadcast over the trailing batch dimensions. Seen here as a
// (D, B) column-major matrix with D = prod(dims) contiguous and a weight / bias vector of length D.
// Reverse (broadcast AD): g = dy .* act'(x .* w .+ b); dx = g .* w; dw = sum over the batch of g .* x; db = sum over
// the batch of g. The pre-activation is rebuilt from x, so nothing but x is needed from the forward pass.
// Bandwidth-bound: forward 2 element passes, backward 3. The batch sums are formed per CTA slice in registers, then in
// a fixed order by a second kernel (deterministic, no atomics).
#include "common.cuh"

namespace lb2 {

constexpr int kScaleSlices = 64;   // batch slices of the backward (rows of the partial-sum workspace)

template <typename T, int ACT, bool VEC>
__global__ void __launch_bounds__(256) scale_fwd_kernel(T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ w,
                                                        const T* __restrict__ b, int64_t D, int64_t B, int act_rt) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = VEC ? Vec16<T>::N : 1;
  const int64_t dv = D / V;                  // feature vectors per column
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < dv; v += (int64_t)gridDim.x * blockDim.x) {
    if constexpr (VEC) {
      const Vec16<T> wv = load16(w + v * V);
      Vec16<T> bv;
      if (b != nullptr) bv = load16(b + v * V);
      for (int64_t n = blockIdx.y; n < B; n += gridDim.y) {
        const Vec16<T> xv = load16_stream(x + n * D + v * V);
        store16_stream(y + n * D + v * V, vec_from<T>([&](int j) {
          return act_apply_any<ACT, FAST>(act_rt, fmaf(xv.get(j), wv.get(j), b != nullptr ? bv.get(j) : 0.f));
        }));
      }
    } else {
      const float wf = to_f32(w[v]), bf = b != nullptr ? to_f32(b[v]) : 0.f;
      for (int64_t n = blockIdx.y; n < B; n += gridDim.y)
        y[n * D + v] = from_f32<T>(act_apply_any<ACT, FAST>(act_rt, fmaf(to_f32(x[n * D + v]), wf, bf)));
    }
  }
}

// partial: [gridDim.y][2][D] fp32 (dw then db); slice blockIdx.y adds its batch columns in ascending order
template <typename T, int ACT, bool VEC>
__global__ void __launch_bounds__(256) scale_bwd_kernel(T* __restrict__ dx, float* __restrict__ partial, const T* __restrict__ dy,
                                                        const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                                        int64_t D, int64_t B, int act_rt) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = VEC ? Vec16<T>::N : 1;
  const int64_t dv = D / V;
  float* pw = partial + (int64_t)blockIdx.y * 2 * D;
  float* pb = pw + D;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < dv; v += (int64_t)gridDim.x * blockDim.x) {
    float aw[V], ab[V];
#pragma unroll
    for (int j = 0; j < V; ++j) { aw[j] = 0.f; ab[j] = 0.f; }
    if constexpr (VEC) {
      const Vec16<T> wv = load16(w + v * V);
      Vec16<T> bv;
      if (b != nullptr) bv = load16(b + v * V);
      for (int64_t n = blockIdx.y; n < B; n += gridDim.y) {
        const Vec16<T> xv = load16_stream(x + n * D + v * V), gv = load16_stream(dy + n * D + v * V);
        store16_stream(dx + n * D + v * V, vec_from<T>([&](int j) {
          const float xf = xv.get(j), wf = wv.get(j);
          float g = gv.get(j);
          if constexpr (ACT != LB2_ACT_IDENTITY) g *= act_grad_pre_any<ACT, FAST>(act_rt, fmaf(xf, wf, b != nullptr ? bv.get(j) : 0.f));
          aw[j] = fmaf(g, xf, aw[j]);
          ab[j] += g;
          return g * wf;
        }));
      }
    } else {
      const float wf = to_f32(w[v]), bf = b != nullptr ? to_f32(b[v]) : 0.f;
      for (int64_t n = blockIdx.y; n < B; n += gridDim.y) {
        const float xf = to_f32(x[n * D + v]);
        float g = to_f32(dy[n * D + v]);
        if constexpr (ACT != LB2_ACT_IDENTITY) g *= act_grad_pre_any<ACT, FAST>(act_rt, fmaf(xf, wf, bf));
        aw[0] = fmaf(g, xf, aw[0]);
        ab[0] += g;
        dx[n * D + v] = from_f32<T>(g * wf);
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) { pw[v * V + j] = aw[j]; pb[v * V + j] = ab[j]; }
  }
}

// dw[i] = sum_k partial[k][0][i], db[i] = sum_k partial[k][1][i]: block (32 features, 32 slices), slice y adds parts
// y, y + 32, ... in ascending order, then the slice sums are added in slice order (a fixed order).
template <typename T>
__global__ void __launch_bounds__(1024) scale_finish_kernel(T* __restrict__ dw, T* __restrict__ db, const float* __restrict__ partial,
                                                            int64_t D, int parts) {
  __shared__ float sw[32][33], sb[32][33];
  const int64_t i = (int64_t)blockIdx.x * 32 + threadIdx.x;
  float a = 0.f, c = 0.f;
  if (i < D) {
    for (int k = threadIdx.y; k < parts; k += 32) {
      a += partial[((int64_t)k * 2) * D + i];
      c += partial[((int64_t)k * 2 + 1) * D + i];
    }
  }
  sw[threadIdx.y][threadIdx.x] = a;
  sb[threadIdx.y][threadIdx.x] = c;
  __syncthreads();
  if (threadIdx.y == 0 && i < D) {
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int r = 0; r < 32; ++r) { tw += sw[r][threadIdx.x]; tb += sb[r][threadIdx.x]; }
    dw[i] = from_f32<T>(tw);
    if (db != nullptr) db[i] = from_f32<T>(tb);
  }
}

static int scale_slices(int64_t B) { return (int)(B < kScaleSlices ? (B < 1 ? 1 : B) : kScaleSlices); }

static dim3 scale_grid(int64_t dv, int slices) {
  int64_t gx = (dv + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8 / slices + 1;
  if (gx > cap) gx = cap;
  if (gx < 1) gx = 1;
  return dim3((unsigned)gx, (unsigned)slices, 1);
}

}  // namespace lb2

using namespace lb2;

extern "C" {

int32_t lb2_scale_fwd(void* y, const void* x, const void* w, const void* b, int64_t D, int64_t B, int32_t dtype, int32_t act,
                      void* stream) {
  LB2_REQUIRE(D >= 0 && B >= 0, LB2_BAD_SHAPE, "bad extent");
  LB2_REQUIRE(dtype == LB2_F32 || dtype == LB2_BF16, LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(act >= LB2_ACT_IDENTITY && act <= LB2_ACT_SWISH, LB2_BAD_ARG, "unknown activation %d", (int)act);
  if (D == 0 || B == 0) return LB2_OK;
  LB2_REQUIRE(y != nullptr && x != nullptr && w != nullptr, LB2_BAD_ARG, "y, x and weight must not be null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t es = dtype_size(dtype);
  const bool vec = aligned_to(y, 16) && aligned_to(x, 16) && aligned_to(w, 16) && (!b || aligned_to(b, 16)) && (D * es) % 16 == 0;
  const int slices = scale_slices(B);
  LB2_DISPATCH_DTYPE(dtype, {
    LB2_DISPATCH_ACT3(act, {
      if (vec) scale_fwd_kernel<T, ACT, true><<<scale_grid(D / Vec16<T>::N, slices), 256, 0, st>>>((T*)y, (const T*)x, (const T*)w, (const T*)b, D, B, act);
      else scale_fwd_kernel<T, ACT, false><<<scale_grid(D, slices), 256, 0, st>>>((T*)y, (const T*)x, (const T*)w, (const T*)b, D, B, act);
    });
  });
  LB2_CHECK_LAUNCH("scale_fwd");
  return LB2_OK;
}

size_t lb2_scale_bwd_workspace_bytes(int64_t D, int64_t B) {
  if (D <= 0 || B <= 0) return 0;
  return align_up((size_t)scale_slices(B) * 2 * (size_t)D * sizeof(float), 256);
}

int32_t lb2_scale_bwd(void* dx, void* dw, void* db, const void* dy, const void* x, const void* w, const void* b, int64_t D,
                      int64_t B, int32_t dtype, int32_t act, void* workspace, size_t workspace_bytes, void* stream) {
  LB2_REQUIRE(D >= 0 && B >= 0, LB2_BAD_SHAPE, "bad extent");
  LB2_REQUIRE(dtype == LB2_F32 || dtype == LB2_BF16, LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(act >= LB2_ACT_IDENTITY && act <= LB2_ACT_SWISH, LB2_BAD_ARG, "unknown activation %d", (int)act);
  if (D == 0) return LB2_OK;
  LB2_REQUIRE(dw != nullptr && w != nullptr, LB2_BAD_ARG, "dw and weight must not be null");
  LB2_REQUIRE((db == nullptr) == (b == nullptr), LB2_BAD_ARG, "db is wanted exactly when the layer has a bias");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t es = dtype_size(dtype);
  if (B == 0) {   // sums over an empty batch
    cudaError_t e = cudaMemsetAsync(dw, 0, (size_t)D * es, st);
    if (e == cudaSuccess && db != nullptr) e = cudaMemsetAsync(db, 0, (size_t)D * es, st);
    LB2_REQUIRE(e == cudaSuccess, LB2_LAUNCH_FAIL, "scale_bwd: %s", cudaGetErrorString(e));
    return LB2_OK;
  }
  LB2_REQUIRE(dx != nullptr && dy != nullptr && x != nullptr, LB2_BAD_ARG, "dx, dy and x must not be null");
  LB2_REQUIRE(workspace != nullptr && workspace_bytes >= lb2_scale_bwd_workspace_bytes(D, B), LB2_WORKSPACE_TOO_SMALL,
              "scale_bwd needs %zu bytes of workspace", lb2_scale_bwd_workspace_bytes(D, B));
  LB2_REQUIRE(aligned_to(workspace, 16), LB2_BAD_ALIGN, "workspace must be 16-byte aligned");
  const bool vec = aligned_to(dx, 16) && aligned_to(dy, 16) && aligned_to(x, 16) && aligned_to(w, 16) && (!b || aligned_to(b, 16)) &&
                   (D * es) % 16 == 0;
  const int slices = scale_slices(B);
  float* ws = static_cast<float*>(workspace);
  LB2_DISPATCH_DTYPE(dtype, {
    LB2_DISPATCH_ACT3(act, {
      if (vec) scale_bwd_kernel<T, ACT, true><<<scale_grid(D / Vec16<T>::N, slices), 256, 0, st>>>((T*)dx, ws, (const T*)dy, (const T*)x, (const T*)w, (const T*)b, D, B, act);
      else scale_bwd_kernel<T, ACT, false><<<scale_grid(D, slices), 256, 0, st>>>((T*)dx, ws, (const T*)dy, (const T*)x, (const T*)w, (const T*)b, D, B, act);
    });
    LB2_CHECK_LAUNCH("scale_bwd");
    scale_finish_kernel<T><<<(unsigned)((D + 31) / 32), dim3(32, 32), 0, st>>>((T*)dw, (T*)db, ws, D, slices);
  });
  LB2_CHECK_LAUNCH("scale_bwd_finish");
  return LB2_OK;
}

}  // extern "C"

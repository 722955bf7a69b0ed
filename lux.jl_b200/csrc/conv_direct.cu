// Direct (CUDA-core) convolution: the catch-all for every ConvDims the implicit-GEMM tensor-core
// path does not take (1-D / 3-D, dilation, groups, odd strides, unaligned widths). Forward, data
// gradient and filter gradient, each with fp32 accumulation in a fixed order (deterministic).
// Layout: x (in..., Cin, N), w (k..., Cin/groups, Cout), y (out..., Cout, N), column-major;
// true convolution (kernel flipped) unless flipkernel is set — NNlib semantics as used by
// lib/LuxLib/src/impl/conv.jl:29-60.
#include "conv.cuh"

namespace lb2 {

// tap position of kernel index kk along dim d
__device__ __forceinline__ int tap_of(const ConvGeom& g, int d, int kk) {
  return (g.flip ? kk : (g.k[d] - 1 - kk)) * g.dil[d];
}

template <typename T, int ACT>
__global__ void __launch_bounds__(256) conv_fwd_direct_kernel(T* __restrict__ y, T* __restrict__ preact,
                                                              const T* __restrict__ x, const T* __restrict__ w,
                                                              const T* __restrict__ bias, const ConvGeom g) {
  constexpr bool FAST = sizeof(T) == 2;
  const int64_t total = (int64_t)g.out[0] * g.out[1] * g.out[2] * g.cout * g.batch;
  const int cin_g = g.cin / g.groups, cout_g = g.cout / g.groups;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i;
    const int o0 = (int)(r % g.out[0]); r /= g.out[0];
    const int o1 = (int)(r % g.out[1]); r /= g.out[1];
    const int o2 = (int)(r % g.out[2]); r /= g.out[2];
    const int co = (int)(r % g.cout);
    const int n = (int)(r / g.cout);
    const int grp = co / cout_g;
    float acc = 0.f;
    for (int ci = 0; ci < cin_g; ++ci) {
      const int cx = grp * cin_g + ci;
      for (int k2 = 0; k2 < g.k[2]; ++k2) {
        const int p2 = o2 * g.stride[2] - g.pad_lo[2] + tap_of(g, 2, k2);
        if (p2 < 0 || p2 >= g.in[2]) continue;
        for (int k1 = 0; k1 < g.k[1]; ++k1) {
          const int p1 = o1 * g.stride[1] - g.pad_lo[1] + tap_of(g, 1, k1);
          if (p1 < 0 || p1 >= g.in[1]) continue;
          for (int k0 = 0; k0 < g.k[0]; ++k0) {
            const int p0 = o0 * g.stride[0] - g.pad_lo[0] + tap_of(g, 0, k0);
            if (p0 < 0 || p0 >= g.in[0]) continue;
            const int64_t xi = ((((int64_t)n * g.cin + cx) * g.in[2] + p2) * g.in[1] + p1) * g.in[0] + p0;
            const int64_t wi = ((((int64_t)co * cin_g + ci) * g.k[2] + k2) * g.k[1] + k1) * g.k[0] + k0;
            acc = fmaf(to_f32(x[xi]), to_f32(w[wi]), acc);
          }
        }
      }
    }
    if (bias) acc += to_f32(bias[co]);
    if (preact) preact[i] = from_f32<T>(acc);
    y[i] = from_f32<T>(act_apply<ACT, FAST>(acc));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) conv_dgrad_direct_kernel(T* __restrict__ dx, const T* __restrict__ dy,
                                                                const T* __restrict__ w, const ConvGeom g) {
  const int64_t total = (int64_t)g.in[0] * g.in[1] * g.in[2] * g.cin * g.batch;
  const int cin_g = g.cin / g.groups, cout_g = g.cout / g.groups;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i;
    const int p0 = (int)(r % g.in[0]); r /= g.in[0];
    const int p1 = (int)(r % g.in[1]); r /= g.in[1];
    const int p2 = (int)(r % g.in[2]); r /= g.in[2];
    const int cx = (int)(r % g.cin);
    const int n = (int)(r / g.cin);
    const int grp = cx / cin_g, ci = cx % cin_g;
    float acc = 0.f;
    for (int k2 = 0; k2 < g.k[2]; ++k2) {
      const int q2 = p2 + g.pad_lo[2] - tap_of(g, 2, k2);
      if (q2 < 0 || q2 % g.stride[2] != 0) continue;
      const int o2 = q2 / g.stride[2];
      if (o2 >= g.out[2]) continue;
      for (int k1 = 0; k1 < g.k[1]; ++k1) {
        const int q1 = p1 + g.pad_lo[1] - tap_of(g, 1, k1);
        if (q1 < 0 || q1 % g.stride[1] != 0) continue;
        const int o1 = q1 / g.stride[1];
        if (o1 >= g.out[1]) continue;
        for (int k0 = 0; k0 < g.k[0]; ++k0) {
          const int q0 = p0 + g.pad_lo[0] - tap_of(g, 0, k0);
          if (q0 < 0 || q0 % g.stride[0] != 0) continue;
          const int o0 = q0 / g.stride[0];
          if (o0 >= g.out[0]) continue;
          for (int cj = 0; cj < cout_g; ++cj) {
            const int co = grp * cout_g + cj;
            const int64_t yi = ((((int64_t)n * g.cout + co) * g.out[2] + o2) * g.out[1] + o1) * g.out[0] + o0;
            const int64_t wi = ((((int64_t)co * cin_g + ci) * g.k[2] + k2) * g.k[1] + k1) * g.k[0] + k0;
            acc = fmaf(to_f32(dy[yi]), to_f32(w[wi]), acc);
          }
        }
      }
    }
    dx[i] = from_f32<T>(acc);
  }
}

// one CTA per weight element; threads stride over (out..., batch)
template <typename T>
__global__ void __launch_bounds__(256) conv_wgrad_direct_kernel(T* __restrict__ dw, const T* __restrict__ x,
                                                                const T* __restrict__ dy, const ConvGeom g) {
  __shared__ float red[32];
  const int cin_g = g.cin / g.groups, cout_g = g.cout / g.groups;
  int64_t r = blockIdx.x;
  const int k0 = (int)(r % g.k[0]); r /= g.k[0];
  const int k1 = (int)(r % g.k[1]); r /= g.k[1];
  const int k2 = (int)(r % g.k[2]); r /= g.k[2];
  const int ci = (int)(r % cin_g);
  const int co = (int)(r / cin_g);
  const int cx = (co / cout_g) * cin_g + ci;
  const int t0 = tap_of(g, 0, k0) - g.pad_lo[0], t1 = tap_of(g, 1, k1) - g.pad_lo[1], t2 = tap_of(g, 2, k2) - g.pad_lo[2];
  const int64_t per_img = (int64_t)g.out[0] * g.out[1] * g.out[2];
  const int64_t total = per_img * g.batch;
  float acc = 0.f;
  for (int64_t i = threadIdx.x; i < total; i += blockDim.x) {
    int64_t q = i;
    const int o0 = (int)(q % g.out[0]); q /= g.out[0];
    const int o1 = (int)(q % g.out[1]); q /= g.out[1];
    const int o2 = (int)(q % g.out[2]);
    const int n = (int)(q / g.out[2]);
    const int p0 = o0 * g.stride[0] + t0, p1 = o1 * g.stride[1] + t1, p2 = o2 * g.stride[2] + t2;
    if (p0 < 0 || p0 >= g.in[0] || p1 < 0 || p1 >= g.in[1] || p2 < 0 || p2 >= g.in[2]) continue;
    const int64_t xi = ((((int64_t)n * g.cin + cx) * g.in[2] + p2) * g.in[1] + p1) * g.in[0] + p0;
    const int64_t yi = ((((int64_t)n * g.cout + co) * g.out[2] + o2) * g.out[1] + o1) * g.out[0] + o0;
    acc = fmaf(to_f32(x[xi]), to_f32(dy[yi]), acc);
  }
  const float s = block_sum(acc, red);
  if (threadIdx.x == 0) dw[blockIdx.x] = from_f32<T>(s);
}

static unsigned flat_grid(int64_t total) {
  int64_t g = (total + 255) / 256, cap = (int64_t)sm_count() * 32;
  return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
}

int32_t conv_fwd_direct(void* y, void* preact, const void* x, const void* w, const void* bias, const ConvGeom& g,
                        int32_t dtype, int32_t act, cudaStream_t st) {
  const int64_t total = (int64_t)g.out[0] * g.out[1] * g.out[2] * g.cout * g.batch;
  LB2_DISPATCH_DTYPE(dtype, {
    LB2_DISPATCH_ACT(act, {
      conv_fwd_direct_kernel<T, ACT><<<flat_grid(total), 256, 0, st>>>((T*)y, (T*)preact, (const T*)x, (const T*)w, (const T*)bias, g);
    });
  });
  LB2_CHECK_LAUNCH("conv_fwd_direct");
  return LB2_OK;
}

int32_t conv_dgrad_direct(void* dx, const void* dy, const void* w, const ConvGeom& g, int32_t dtype, cudaStream_t st) {
  const int64_t total = (int64_t)g.in[0] * g.in[1] * g.in[2] * g.cin * g.batch;
  LB2_DISPATCH_DTYPE(dtype, { conv_dgrad_direct_kernel<T><<<flat_grid(total), 256, 0, st>>>((T*)dx, (const T*)dy, (const T*)w, g); });
  LB2_CHECK_LAUNCH("conv_dgrad_direct");
  return LB2_OK;
}

int32_t conv_wgrad_direct(void* dw, const void* x, const void* dy, const ConvGeom& g, int32_t dtype, cudaStream_t st) {
  const int64_t nw = (int64_t)g.k[0] * g.k[1] * g.k[2] * (g.cin / g.groups) * g.cout;
  LB2_REQUIRE(nw <= 0x7FFFFFFF, LB2_BAD_SHAPE, "too many filter elements");
  LB2_DISPATCH_DTYPE(dtype, { conv_wgrad_direct_kernel<T><<<(unsigned)nw, 256, 0, st>>>((T*)dw, (const T*)x, (const T*)dy, g); });
  LB2_CHECK_LAUNCH("conv_wgrad_direct");
  return LB2_OK;
}

}  // namespace lb2

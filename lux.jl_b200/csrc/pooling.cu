// Max / mean pooling, forward and backward, on the WHCN (column-major) layout — the glue between the
// conv blocks of a conv net (src/layers/pooling.jl:42-54 -> NNlib.maxpool / NNlib.meanpool, and the
// global pools of :47-48,56-57 as the window == input case).
//
// Semantics follow NNlib's direct CPU kernels (NNlib 0.9, a dependency of the reference, not
// vendored): windows are clipped to the input (padding never wins a max), the mean always divides
// by the full window size, and the max-pool gradient goes to the FIRST element of the window that
// equals the maximum, scanning kw fastest, then kh, then kd.
// Bandwidth-bound: a CTA walks whole (channel, sample) planes, one thread per output (forward) / per input (backward,
// a gather over the windows that cover it, so the sums are formed in a fixed order: deterministic, no atomics).
#include "common.cuh"

namespace lb2 {

struct PoolGeom {
  int in[3], k[3], stride[3], pad[3], dil[3], out[3];
  int64_t planes;   // channels * batch
};

// One CTA walks whole (channel, sample) planes, so all index arithmetic inside a plane is 32-bit and the plane's
// rows stay in L1 / L2 while the windows that share them are evaluated.
template <typename T, bool MAX>
__global__ void __launch_bounds__(256) pool_fwd_kernel(T* __restrict__ y, const T* __restrict__ x, const PoolGeom g) {
  const int out_sp = g.out[0] * g.out[1] * g.out[2];
  const int in_sp = g.in[0] * g.in[1] * g.in[2];
  const float inv_win = 1.f / (float)(g.k[0] * g.k[1] * g.k[2]);
  for (int64_t plane = blockIdx.x; plane < g.planes; plane += gridDim.x) {
    const T* xp = x + plane * in_sp;
    T* yp = y + plane * out_sp;
    for (int i = threadIdx.x; i < out_sp; i += blockDim.x) {
      int r = i;
      const int ow = r % g.out[0]; r /= g.out[0];
      const int oh = r % g.out[1];
      const int od = r / g.out[1];
      float acc = MAX ? -INFINITY : 0.f;
      for (int kd = 0; kd < g.k[2]; ++kd) {
        const int d = od * g.stride[2] - g.pad[2] + kd * g.dil[2];
        if (d < 0 || d >= g.in[2]) continue;
        for (int kh = 0; kh < g.k[1]; ++kh) {
          const int h = oh * g.stride[1] - g.pad[1] + kh * g.dil[1];
          if (h < 0 || h >= g.in[1]) continue;
          const T* row = xp + (d * g.in[1] + h) * g.in[0];
          for (int kw = 0; kw < g.k[0]; ++kw) {
            const int w = ow * g.stride[0] - g.pad[0] + kw * g.dil[0];
            if (w < 0 || w >= g.in[0]) continue;
            const float v = to_f32(row[w]);
            if (MAX) acc = fmaxf(acc, v); else acc += v;
          }
        }
      }
      yp[i] = from_f32<T>(MAX ? acc : acc * inv_win);
    }
  }
}

// Global pooling (window == whole unpadded input): one warp per (channel, sample) plane, lanes stride through
// the plane's contiguous elements, then a butterfly - a fixed order, so deterministic.
template <typename T, bool MAX>
__global__ void __launch_bounds__(256) pool_global_fwd_kernel(T* __restrict__ y, const T* __restrict__ x, int64_t S, int64_t planes) {
  const int lane = threadIdx.x & 31;
  const int64_t wstride = (int64_t)gridDim.x * 8;
  for (int64_t plane = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); plane < planes; plane += wstride) {
    const T* xp = x + plane * S;
    float acc = MAX ? -INFINITY : 0.f;
    for (int64_t i = lane; i < S; i += 32) {
      const float v = to_f32(xp[i]);
      if (MAX) acc = fmaxf(acc, v); else acc += v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, acc, o);
      if (MAX) acc = fmaxf(acc, other); else acc += other;
    }
    if (lane == 0) y[plane] = from_f32<T>(MAX ? acc : acc / (float)S);
  }
}

// Global pooling backward: the mean spreads dy / S over the plane; the max gives dy to the first maximal element.
template <typename T, bool MAX>
__global__ void __launch_bounds__(256) pool_global_bwd_kernel(T* __restrict__ dx, const T* __restrict__ dy, const T* __restrict__ y,
                                                              const T* __restrict__ x, int64_t S, int64_t planes) {
  const int lane = threadIdx.x & 31;
  const int64_t wstride = (int64_t)gridDim.x * 8;
  for (int64_t plane = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); plane < planes; plane += wstride) {
    const float g = to_f32(dy[plane]);
    T* dxp = dx + plane * S;
    if (MAX) {
      const T* xp = x + plane * S;
      const float ymax = to_f32(y[plane]);
      long long first = S;
      for (int64_t i = lane; i < S && first == S; i += 32)
        if (to_f32(xp[i]) == ymax) first = i;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const long long other = __shfl_xor_sync(0xffffffffu, first, o);
        first = other < first ? other : first;
      }
      for (int64_t i = lane; i < S; i += 32) dxp[i] = from_f32<T>(i == first ? g : 0.f);
    } else {
      const T v = from_f32<T>(g / (float)S);
      for (int64_t i = lane; i < S; i += 32) dxp[i] = v;
    }
  }
}

// Does the window of output (ow, oh, od) give its max-pool gradient to input (w, h, d)? True when that
// input is the first element, in (kw fastest, kh, kd) order, equal to the window maximum ymax.
template <typename T>
__device__ __forceinline__ bool first_max_is(const T* xp, const PoolGeom& g, int ow, int oh, int od, float ymax, int w, int h,
                                             int d) {
  for (int kd = 0; kd < g.k[2]; ++kd) {
    const int dd = od * g.stride[2] - g.pad[2] + kd * g.dil[2];
    if (dd < 0 || dd >= g.in[2]) continue;
    for (int kh = 0; kh < g.k[1]; ++kh) {
      const int hh = oh * g.stride[1] - g.pad[1] + kh * g.dil[1];
      if (hh < 0 || hh >= g.in[1]) continue;
      for (int kw = 0; kw < g.k[0]; ++kw) {
        const int ww = ow * g.stride[0] - g.pad[0] + kw * g.dil[0];
        if (ww < 0 || ww >= g.in[0]) continue;
        if (to_f32(xp[((int64_t)dd * g.in[1] + hh) * g.in[0] + ww]) == ymax) return ww == w && hh == h && dd == d;
      }
    }
  }
  return false;
}

template <typename T, bool MAX>
__global__ void __launch_bounds__(256) pool_bwd_kernel(T* __restrict__ dx, const T* __restrict__ dy, const T* __restrict__ y,
                                                       const T* __restrict__ x, const PoolGeom g) {
  const int out_sp = g.out[0] * g.out[1] * g.out[2];
  const int in_sp = g.in[0] * g.in[1] * g.in[2];
  const float inv_win = 1.f / (float)(g.k[0] * g.k[1] * g.k[2]);
  for (int64_t plane = blockIdx.x; plane < g.planes; plane += gridDim.x) {
    const T* xp = MAX ? x + plane * in_sp : nullptr;
    const T* yp = MAX ? y + plane * out_sp : nullptr;
    const T* dyp = dy + plane * out_sp;
    T* dxp = dx + plane * in_sp;
    for (int i = threadIdx.x; i < in_sp; i += blockDim.x) {
      int r = i;
      const int w = r % g.in[0]; r /= g.in[0];
      const int h = r % g.in[1];
      const int d = r / g.in[1];
      const float xv = MAX ? to_f32(xp[i]) : 0.f;
      float acc = 0.f;
      // outputs whose window holds this input: o*stride - pad + kk*dil == coordinate with kk in [0, k), i.e.
      // o in [ceil((coordinate + pad - (k-1)*dil) / stride), floor((coordinate + pad) / stride)], dil | remainder
      int lo[3], hi[3];
      const int coord[3] = {w, h, d};
#pragma unroll
      for (int a = 0; a < 3; ++a) {
        const int top = coord[a] + g.pad[a];
        const int bot = top - (g.k[a] - 1) * g.dil[a];
        lo[a] = bot <= 0 ? 0 : (bot + g.stride[a] - 1) / g.stride[a];
        hi[a] = min(g.out[a] - 1, top / g.stride[a]);
      }
      for (int od = lo[2]; od <= hi[2]; ++od) {
        if ((d + g.pad[2] - od * g.stride[2]) % g.dil[2] != 0) continue;
        for (int oh = lo[1]; oh <= hi[1]; ++oh) {
          if ((h + g.pad[1] - oh * g.stride[1]) % g.dil[1] != 0) continue;
          for (int ow = lo[0]; ow <= hi[0]; ++ow) {
            if ((w + g.pad[0] - ow * g.stride[0]) % g.dil[0] != 0) continue;
            const int o = (od * g.out[1] + oh) * g.out[0] + ow;
            if (MAX) {
              // only an element equal to the window's maximum can receive its gradient; the scan for an earlier
              // equal element (the tie rule) runs for those alone
              const float ym = to_f32(yp[o]);
              if (xv == ym && first_max_is(xp, g, ow, oh, od, ym, w, h, d)) acc += to_f32(dyp[o]);
            } else {
              acc += to_f32(dyp[o]) * inv_win;
            }
          }
        }
      }
      dxp[i] = from_f32<T>(acc);
    }
  }
}

// ---- 2-D windows without dilation (the pooling layers of a conv net): no runtime divisions per element ----------
// Threads are laid out as 128 columns x 2 rows over a plane; STRIDE is a compile-time constant for the common
// strides (0 = read it from the geometry), so the window ranges are shifts and compares.
template <int STRIDE> __device__ __forceinline__ int div_stride(int v, int s) {   // floor(v / stride), v >= 0
  if constexpr (STRIDE == 1) return v;
  else if constexpr (STRIDE == 2) return v >> 1;
  else return v / s;
}

template <typename T, bool MAX, int STRIDE>
__global__ void __launch_bounds__(256) pool2d_fwd_kernel(T* __restrict__ y, const T* __restrict__ x, const PoolGeom g) {
  const int W = g.in[0], H = g.in[1], OW = g.out[0], OH = g.out[1];
  const int sw = STRIDE ? STRIDE : g.stride[0], sh = STRIDE ? STRIDE : g.stride[1];
  const int tx = threadIdx.x & 127, ty = threadIdx.x >> 7;
  const float inv_win = 1.f / (float)(g.k[0] * g.k[1]);
  for (int64_t plane = blockIdx.x; plane < g.planes; plane += gridDim.x) {
    const T* xp = x + plane * (int64_t)(W * H);
    T* yp = y + plane * (int64_t)(OW * OH);
    for (int oh = ty; oh < OH; oh += 2) {
      const int h0 = oh * sh - g.pad[1];
      const int kh_lo = h0 < 0 ? -h0 : 0, kh_hi = min(g.k[1], H - h0);
      for (int ow = tx; ow < OW; ow += 128) {
        const int w0 = ow * sw - g.pad[0];
        const int kw_lo = w0 < 0 ? -w0 : 0, kw_hi = min(g.k[0], W - w0);
        float acc = MAX ? -INFINITY : 0.f;
        for (int kh = kh_lo; kh < kh_hi; ++kh) {
          const T* row = xp + (h0 + kh) * W + w0;
          for (int kw = kw_lo; kw < kw_hi; ++kw) {
            const float v = to_f32(row[kw]);
            if (MAX) acc = fmaxf(acc, v); else acc += v;
          }
        }
        yp[oh * OW + ow] = from_f32<T>(MAX ? acc : acc * inv_win);
      }
    }
  }
}

template <typename T, bool MAX, int STRIDE>
__global__ void __launch_bounds__(256) pool2d_bwd_kernel(T* __restrict__ dx, const T* __restrict__ dy, const T* __restrict__ y,
                                                         const T* __restrict__ x, const PoolGeom g) {
  const int W = g.in[0], H = g.in[1], OW = g.out[0], OH = g.out[1], kW = g.k[0], kH = g.k[1];
  const int sw = STRIDE ? STRIDE : g.stride[0], sh = STRIDE ? STRIDE : g.stride[1];
  const int tx = threadIdx.x & 127, ty = threadIdx.x >> 7;
  const float inv_win = 1.f / (float)(kW * kH);
  for (int64_t plane = blockIdx.x; plane < g.planes; plane += gridDim.x) {
    const T* xp = MAX ? x + plane * (int64_t)(W * H) : nullptr;
    const T* yp = MAX ? y + plane * (int64_t)(OW * OH) : nullptr;
    const T* dyp = dy + plane * (int64_t)(OW * OH);
    T* dxp = dx + plane * (int64_t)(W * H);
    for (int h = ty; h < H; h += 2) {
      // outputs whose window holds row h: oh*sh - pad <= h <= oh*sh - pad + kH - 1
      const int top = h + g.pad[1], bot = top - (kH - 1);
      const int oh_lo = bot <= 0 ? 0 : div_stride<STRIDE>(bot + sh - 1, sh);
      const int oh_hi = min(OH - 1, div_stride<STRIDE>(top, sh));
      for (int w = tx; w < W; w += 128) {
        const int topw = w + g.pad[0], botw = topw - (kW - 1);
        const int ow_lo = botw <= 0 ? 0 : div_stride<STRIDE>(botw + sw - 1, sw);
        const int ow_hi = min(OW - 1, div_stride<STRIDE>(topw, sw));
        const float xv = MAX ? to_f32(xp[h * W + w]) : 0.f;
        float acc = 0.f;
        for (int oh = oh_lo; oh <= oh_hi; ++oh) {
          for (int ow = ow_lo; ow <= ow_hi; ++ow) {
            const int o = oh * OW + ow;
            if (MAX) {
              const float ym = to_f32(yp[o]);
              if (xv == ym) {
                // the gradient goes to the FIRST element of the window equal to its maximum (kw fastest, then kh)
                const int h0 = oh * sh - g.pad[1], w0 = ow * sw - g.pad[0];
                bool first = true;
                for (int kh = max(0, -h0); first && h0 + kh <= h; ++kh) {
                  const int kw_end = (h0 + kh == h) ? (w - w0) : min(kW, W - w0);
                  for (int kw = max(0, -w0); kw < kw_end; ++kw)
                    if (to_f32(xp[(h0 + kh) * W + w0 + kw]) == ym) { first = false; break; }
                }
                if (first) acc += to_f32(dyp[o]);
              }
            } else {
              acc += to_f32(dyp[o]) * inv_win;
            }
          }
        }
        dxp[h * W + w] = from_f32<T>(acc);
      }
    }
  }
}

// ---- 2-D windows, planes staged in shared memory ------------------------------------------------------------------
// The direct kernels above issue chains of dependent 2-byte global loads per element (x, then the y of each window,
// then possibly a scan of the window) and are latency-bound. When a plane of x together with its y and dy planes fits
// in shared memory, a CTA stages them with 16-byte loads, evaluates every window from shared memory and writes the
// result rows coalesced. Threads form (256 / Wp) rows of Wp columns, Wp = the row length rounded up to a power of two.
// Stages n elements into shared memory. With `vec` (16-byte aligned source, n*sizeof(T) a multiple of 16) the copies
// are asynchronous 16-byte global->shared copies, all in flight at once; pool_stage_wait() must precede the barrier
// that publishes them.
template <typename T>
__device__ __forceinline__ void pool_stage(T* dst, const T* src, int n, bool vec) {
  if (vec) {
    const int nv = (int)((size_t)n * sizeof(T) / 16);
    const uint32_t d0 = (uint32_t)__cvta_generic_to_shared(dst);
    for (int i = threadIdx.x; i < nv; i += blockDim.x)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d0 + 16u * (uint32_t)i), "l"(reinterpret_cast<const uint4*>(src) + i) : "memory");
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
  }
}
__device__ __forceinline__ void pool_stage_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Window scans with the window extent K known at compile time (K x K taps, fully unrolled). Taps that fall into the
// padding are ALIASED onto the window's first valid row / column instead of being skipped: a padded row above the
// plane reads the first valid row (the same elements, met again later at their true place, where a strict comparison
// cannot replace them), a padded row below reads it after every true tap (and cannot win either); columns likewise.
// The recorded position is computed from the aliased coordinates and is therefore always the true position of the
// element read. The scan is then free of predicates and of loop overhead. Needs a window with at least one valid row
// and column (pool_fixed_window() checks that on the host). cofs[kw] = the aliased column of tap kw.
template <int K>
__device__ __forceinline__ void pool_alias_columns(int (&cofs)[K], int w0, int W) {
  const int wfirst = max(w0, 0);
#pragma unroll
  for (int kw = 0; kw < K; ++kw) cofs[kw] = (unsigned)(w0 + kw) < (unsigned)W ? w0 + kw : wfirst;
}
template <typename T, int K>
__device__ __forceinline__ void pool_window_argmax(const T* __restrict__ sx, int W, int H, int h0, const int (&cofs)[K], float& best, int& where) {
  const int hfirst = max(h0, 0);
#pragma unroll
  for (int kh = 0; kh < K; ++kh) {
    const int rb = ((unsigned)(h0 + kh) < (unsigned)H ? h0 + kh : hfirst) * W;
#pragma unroll
    for (int kw = 0; kw < K; ++kw) {
      const int i = rb + cofs[kw];
      const float v = to_f32(sx[i]);
      if (kh == 0 && kw == 0) { best = v; where = i; }        // the first valid element is taken unconditionally
      else { const bool take = v > best; best = take ? v : best; where = take ? i : where; }
    }
  }
}
template <typename T, int K>
__device__ __forceinline__ float pool_window_max(const T* __restrict__ sx, int W, int H, int h0, const int (&cofs)[K]) {
  const int hfirst = max(h0, 0);
  float best = -INFINITY;
#pragma unroll
  for (int kh = 0; kh < K; ++kh) {
    const int rb = ((unsigned)(h0 + kh) < (unsigned)H ? h0 + kh : hfirst) * W;
#pragma unroll
    for (int kw = 0; kw < K; ++kw) best = fmaxf(best, to_f32(sx[rb + cofs[kw]]));
  }
  return best;
}

template <typename T, bool MAX, int STRIDE, int K>
__global__ void __launch_bounds__(256) pool2d_fwd_smem_kernel(T* __restrict__ y, const T* __restrict__ x, const PoolGeom g, int lw,
                                                              int vec) {
  static_assert(K == 0 || MAX, "the unrolled scan is the max scan");
  extern __shared__ __align__(16) uint8_t pool_smem[];
  T* sx = reinterpret_cast<T*>(pool_smem);
  const int W = g.in[0], H = g.in[1], OW = g.out[0], OH = g.out[1];
  const int sw = STRIDE ? STRIDE : g.stride[0], sh = STRIDE ? STRIDE : g.stride[1];
  const int tx = threadIdx.x & ((1 << lw) - 1), ty = threadIdx.x >> lw, rows = 256 >> lw;
  const float inv_win = 1.f / (float)(g.k[0] * g.k[1]);
  for (int64_t plane = blockIdx.x; plane < g.planes; plane += gridDim.x) {
    __syncthreads();
    pool_stage(sx, x + plane * (int64_t)(W * H), W * H, vec != 0);
    pool_stage_wait();
    __syncthreads();
    T* yp = y + plane * (int64_t)(OW * OH);
    if (tx < OW) {
      const int w0 = tx * sw - g.pad[0];
      if constexpr (K > 0) {
        int cofs[K];
        pool_alias_columns<K>(cofs, w0, W);
        for (int oh = ty; oh < OH; oh += rows) yp[oh * OW + tx] = from_f32<T>(pool_window_max<T, K>(sx, W, H, oh * sh - g.pad[1], cofs));
      } else {
        const int kw_lo = w0 < 0 ? -w0 : 0, kw_hi = min(g.k[0], W - w0);
        for (int oh = ty; oh < OH; oh += rows) {
          const int h0 = oh * sh - g.pad[1];
          const int kh_lo = h0 < 0 ? -h0 : 0, kh_hi = min(g.k[1], H - h0);
          float acc = MAX ? -INFINITY : 0.f;
          for (int kh = kh_lo; kh < kh_hi; ++kh) {
            const T* row = sx + (h0 + kh) * W + w0;
            for (int kw = kw_lo; kw < kw_hi; ++kw) {
              const float v = to_f32(row[kw]);
              if (MAX) acc = fmaxf(acc, v); else acc += v;
            }
          }
          yp[oh * OW + tx] = from_f32<T>(MAX ? acc : acc * inv_win);
        }
      }
    }
  }
}

// Backward of mean pooling: one thread per INPUT element adds dy of the covering windows.
template <typename T, int STRIDE>
__global__ void __launch_bounds__(256) pool2d_meanbwd_smem_kernel(T* __restrict__ dx, const T* __restrict__ dy, const PoolGeom g, int lw,
                                                                  int vec_out) {
  extern __shared__ __align__(16) uint8_t pool_smem[];
  T* sdy = reinterpret_cast<T*>(pool_smem);
  const int W = g.in[0], H = g.in[1], OW = g.out[0], OH = g.out[1], kW = g.k[0], kH = g.k[1];
  const int sw = STRIDE ? STRIDE : g.stride[0], sh = STRIDE ? STRIDE : g.stride[1];
  const int tx = threadIdx.x & ((1 << lw) - 1), ty = threadIdx.x >> lw, rows = 256 >> lw;
  const float inv_win = 1.f / (float)(kW * kH);
  for (int64_t plane = blockIdx.x; plane < g.planes; plane += gridDim.x) {
    __syncthreads();
    pool_stage(sdy, dy + plane * (int64_t)(OW * OH), OW * OH, vec_out != 0);
    pool_stage_wait();
    __syncthreads();
    T* dxp = dx + plane * (int64_t)(W * H);
    if (tx < W) {
      const int w = tx;
      const int topw = w + g.pad[0], botw = topw - (kW - 1);
      const int ow_lo = botw <= 0 ? 0 : div_stride<STRIDE>(botw + sw - 1, sw);
      const int ow_hi = min(OW - 1, div_stride<STRIDE>(topw, sw));
      for (int h = ty; h < H; h += rows) {
        const int top = h + g.pad[1], bot = top - (kH - 1);
        const int oh_lo = bot <= 0 ? 0 : div_stride<STRIDE>(bot + sh - 1, sh);
        const int oh_hi = min(OH - 1, div_stride<STRIDE>(top, sh));
        float acc = 0.f;
        for (int oh = oh_lo; oh <= oh_hi; ++oh)
          for (int ow = ow_lo; ow <= ow_hi; ++ow) acc += to_f32(sdy[oh * OW + ow]);
        dxp[h * W + w] = from_f32<T>(acc * inv_win);
      }
    }
  }
}

// Backward of max pooling, window-centric: a thread owns a window, finds its first maximal element (scan in
// kw-fastest order with a strict comparison, NNlib's tie rule) and adds the window's dy to that element's fp32
// accumulator in shared memory. Windows are visited in ceil(kW/sw) x ceil(kH/sh) classes of equal (ow mod cw,
// oh mod ch): two windows of one class do not overlap, so the additions within a class touch distinct accumulators
// and need no atomics, and the order of additions into one accumulator is fixed (class order): the result is
// deterministic. The plane of accumulators is then rounded and written with 16-byte stores. The per-element work of
// the input-centric form (bounds of the covering windows for each of W*H elements) is gone; what is left is one scan
// per window. The forward result y is not needed.
template <typename T, int STRIDE, int K>
__global__ void __launch_bounds__(1024, 2) pool2d_maxbwd_smem_kernel(T* __restrict__ dx, const T* __restrict__ dy, const T* __restrict__ x,
                                                                 const PoolGeom g, int lw, int vec_in, int vec_out, int off_acc, int off_dy,
                                                                 int cw, int ch) {
  extern __shared__ __align__(16) uint8_t pool_smem[];
  T* sx = reinterpret_cast<T*>(pool_smem);
  float* sacc = reinterpret_cast<float*>(pool_smem + off_acc);
  T* sdy = reinterpret_cast<T*>(pool_smem + off_dy);
  const int W = g.in[0], H = g.in[1], OW = g.out[0], OH = g.out[1], kW = g.k[0], kH = g.k[1];
  const int sw = STRIDE ? STRIDE : g.stride[0], sh = STRIDE ? STRIDE : g.stride[1];
  const int tx = threadIdx.x & ((1 << lw) - 1), ty = threadIdx.x >> lw, rows = (int)blockDim.x >> lw;
  const int n = W * H, n4 = (n + 3) >> 2;
  for (int64_t plane = blockIdx.x; plane < g.planes; plane += gridDim.x) {
    __syncthreads();
    pool_stage(sx, x + plane * (int64_t)n, n, vec_in != 0);
    pool_stage(sdy, dy + plane * (int64_t)(OW * OH), OW * OH, vec_out != 0);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) reinterpret_cast<float4*>(sacc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    pool_stage_wait();
    __syncthreads();
    for (int ci = 0; ci < ch; ++ci)
      for (int cj = 0; cj < cw; ++cj) {
        const int ow = cj + tx * cw;
        if (ow < OW) {
          const int w0 = ow * sw - g.pad[0];
          if constexpr (K > 0) {
            int cofs[K];
            pool_alias_columns<K>(cofs, w0, W);
            for (int oh = ci + ty * ch; oh < OH; oh += rows * ch) {
              float best;
              int where;
              pool_window_argmax<T, K>(sx, W, H, oh * sh - g.pad[1], cofs, best, where);
              sacc[where] += to_f32(sdy[oh * OW + ow]);
            }
          } else {
            const int kw_lo = w0 < 0 ? -w0 : 0, kw_hi = min(kW, W - w0);
            for (int oh = ci + ty * ch; oh < OH; oh += rows * ch) {
              const int h0 = oh * sh - g.pad[1];
              const int kh_lo = h0 < 0 ? -h0 : 0, kh_hi = min(kH, H - h0);
              float best = -INFINITY;
              int where = -1;
              for (int kh = kh_lo; kh < kh_hi; ++kh) {
                const int r = (h0 + kh) * W + w0;
                for (int kw = kw_lo; kw < kw_hi; ++kw) {
                  const float v = to_f32(sx[r + kw]);
                  const bool take = v > best || where < 0;
                  best = take ? v : best;
                  where = take ? r + kw : where;
                }
              }
              if (where >= 0) sacc[where] += to_f32(sdy[oh * OW + ow]);
            }
          }
        }
        __syncthreads();
      }
    T* dxp = dx + plane * (int64_t)n;
    if (vec_in) {      // n * sizeof(T) is a multiple of 16 and the plane starts on 16 bytes
      constexpr int PER = 16 / (int)sizeof(T);
      for (int i = threadIdx.x; i < n / PER; i += blockDim.x) {
        alignas(16) T out[PER];
#pragma unroll
        for (int j = 0; j < PER; j += 4) {
          const float4 a = reinterpret_cast<const float4*>(sacc)[(i * PER + j) >> 2];
          out[j] = from_f32<T>(a.x); out[j + 1] = from_f32<T>(a.y); out[j + 2] = from_f32<T>(a.z); out[j + 3] = from_f32<T>(a.w);
        }
        reinterpret_cast<uint4*>(dxp)[i] = *reinterpret_cast<const uint4*>(out);
      }
    } else {
      for (int i = threadIdx.x; i < n; i += blockDim.x) dxp[i] = from_f32<T>(sacc[i]);
    }
  }
}

// pointer types of a staged kernel's output / input parameters (so one generic launcher serves both storage types)
template <typename T, typename... R> T* pool_arg_y(void (*)(T*, const T*, R...));
template <typename T, typename... R> const T* pool_arg_x(void (*)(T*, const T*, R...));

// shared-memory layout of the staged kernels. Forward: the x plane. Mean backward: the dy plane. Max backward:
// x plane | fp32 accumulators of dx (a multiple of four) | dy plane, each starting on 16 bytes; two CTAs of 256
// threads per SM while that is at most 112 KB, one up to 200 KB.
struct PoolSmem { int off_acc, off_dy, bytes, lw_in, lw_out, lw_cls, cw, ch; bool ok; };
static PoolSmem pool_smem_plan(const PoolGeom& g, size_t es, int what /*0 fwd, 1 mean bwd, 2 max bwd*/) {
  PoolSmem p{};
  const size_t n = (size_t)g.in[0] * g.in[1], no = (size_t)g.out[0] * g.out[1];
  const size_t xb = align_up(n * es, 16), yb = align_up(no * es, 16), ab = align_up(n * sizeof(float), 16);
  p.off_acc = (int)xb; p.off_dy = (int)(xb + ab);
  p.bytes = (int)(what == 0 ? xb : what == 1 ? yb : xb + ab + yb);
  auto lg = [](int v) { int l = 5; while ((1 << l) < v) ++l; return l; };
  p.cw = (g.k[0] + g.stride[0] - 1) / g.stride[0];
  p.ch = (g.k[1] + g.stride[1] - 1) / g.stride[1];
  p.lw_in = lg(g.in[0]); p.lw_out = lg(g.out[0]); p.lw_cls = lg((g.out[0] + p.cw - 1) / p.cw);
  p.ok = (size_t)p.bytes <= (what == 2 ? 200u : 96u) * 1024 && xb + ab + yb < ((size_t)1 << 30) && p.lw_in <= 8 && p.lw_out <= 8 &&
         g.out[0] >= 1 && g.out[1] >= 1 && p.cw * p.ch <= 64;
  return p;
}

// 2 or 3 when the window is K x K and every window holds at least one valid row and column (the condition of the
// unrolled scans with aliased padding taps), else 0.
static int pool_fixed_window(const PoolGeom& g) {
  if (g.k[0] != g.k[1] || (g.k[0] != 2 && g.k[0] != 3)) return 0;
  for (int i = 0; i < 2; ++i) {
    if (g.out[i] < 1 || g.in[i] < 1) return 0;
    const int last0 = (g.out[i] - 1) * g.stride[i] - g.pad[i];     // first tap of the last window
    if (g.pad[i] >= g.k[i] || last0 >= g.in[i]) return 0;
  }
  return g.k[0];
}

static bool pool_is_2d_plain(const PoolGeom& g) {
  return g.in[2] == 1 && g.k[2] == 1 && g.out[2] == 1 && g.dil[0] == 1 && g.dil[1] == 1 && g.pad[2] == 0 &&
         (int64_t)g.in[0] * g.in[1] < ((int64_t)1 << 30);
}

static int32_t make_pool_geom(const lb2_pool_desc* d, PoolGeom* g) {
  LB2_REQUIRE(d != nullptr, LB2_BAD_ARG, "pool descriptor is null");
  LB2_REQUIRE(d->ndim >= 1 && d->ndim <= 3, LB2_BAD_SHAPE, "spatial rank %d not in 1..3", (int)d->ndim);
  LB2_REQUIRE(d->channels >= 0 && d->batch >= 0, LB2_BAD_SHAPE, "bad channel / batch extents");
  for (int i = 0; i < 3; ++i) {
    const bool live = i < d->ndim;
    g->in[i] = live ? d->in[i] : 1;
    g->k[i] = live ? d->k[i] : 1;
    g->stride[i] = live ? d->stride[i] : 1;
    g->pad[i] = live ? d->pad_lo[i] : 0;
    g->dil[i] = live ? d->dilation[i] : 1;
    const int pad_hi = live ? d->pad_hi[i] : 0;
    LB2_REQUIRE(g->in[i] >= 0 && g->k[i] >= 1 && g->stride[i] >= 1 && g->dil[i] >= 1 && g->pad[i] >= 0 && pad_hi >= 0, LB2_BAD_SHAPE,
                "bad extent / window / stride / dilation / padding in dim %d", i);
    const int span = g->in[i] + g->pad[i] + pad_hi - g->dil[i] * (g->k[i] - 1) - 1;
    g->out[i] = span < 0 ? 0 : span / g->stride[i] + 1;
  }
  g->planes = (int64_t)d->channels * d->batch;
  LB2_REQUIRE((int64_t)g->in[0] * g->in[1] * g->in[2] < ((int64_t)1 << 31), LB2_BAD_SHAPE, "a (channel, sample) plane must hold fewer than 2^31 elements");
  return LB2_OK;
}

static unsigned plane_grid(int64_t planes) {
  const int64_t cap = (int64_t)sm_count() * 16;
  return (unsigned)(planes < 1 ? 1 : (planes > cap ? cap : planes));
}

static unsigned pool_grid(int64_t total) {
  int64_t gsz = (total + 255) / 256, cap = (int64_t)sm_count() * 16;
  return (unsigned)(gsz < 1 ? 1 : (gsz > cap ? cap : gsz));
}

}  // namespace lb2

using namespace lb2;

extern "C" {

int32_t lb2_pool_output_size(const lb2_pool_desc* d, int32_t* out) {
  PoolGeom g;
  int32_t rc = make_pool_geom(d, &g);
  if (rc != LB2_OK) return rc;
  LB2_REQUIRE(out != nullptr, LB2_BAD_ARG, "out is null");
  for (int i = 0; i < d->ndim; ++i) out[i] = g.out[i];
  return LB2_OK;
}

int32_t lb2_pool_fwd(void* y, const void* x, const lb2_pool_desc* d, int32_t kind, int32_t dtype, void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(kind == LB2_POOL_MAX || kind == LB2_POOL_MEAN, LB2_BAD_ARG, "unknown pooling kind %d", (int)kind);
  PoolGeom g;
  int32_t rc = make_pool_geom(d, &g);
  if (rc != LB2_OK) return rc;
  const int64_t total = (int64_t)g.out[0] * g.out[1] * g.out[2] * g.planes;
  if (total == 0) return LB2_OK;
  LB2_REQUIRE(y && x, LB2_BAD_ARG, "null tensor pointer");
  LB2_REQUIRE(aligned_to(y, dtype_size(dtype)) && aligned_to(x, dtype_size(dtype)), LB2_BAD_ALIGN, "pointer not aligned to the element size");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  bool global = true;
  for (int i = 0; i < 3; ++i) global = global && g.out[i] == 1 && g.pad[i] == 0 && g.dil[i] == 1 && g.k[i] == g.in[i];
  if (global) {
    const int64_t S = (int64_t)g.in[0] * g.in[1] * g.in[2];
    LB2_DISPATCH_DTYPE(dtype, {
      if (kind == LB2_POOL_MAX) pool_global_fwd_kernel<T, true><<<pool_grid(g.planes * 32), 256, 0, st>>>((T*)y, (const T*)x, S, g.planes);
      else pool_global_fwd_kernel<T, false><<<pool_grid(g.planes * 32), 256, 0, st>>>((T*)y, (const T*)x, S, g.planes);
    });
    LB2_CHECK_LAUNCH("pool_global_fwd");
    return LB2_OK;
  }
  if (pool_is_2d_plain(g)) {
    const bool same = g.stride[0] == g.stride[1];
    const PoolSmem sp = pool_smem_plan(g, dtype_size(dtype), 0);
    if (sp.ok) {
      const int vec = (aligned_to(x, 16) && ((size_t)g.in[0] * g.in[1] * dtype_size(dtype)) % 16 == 0) ? 1 : 0;
      const int st2 = same && g.stride[0] <= 2 ? g.stride[0] : 0;
      auto launch = [&](auto kernel) -> int32_t {
        if (sp.bytes > 48 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.bytes);
          if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "pool2d_fwd: cannot reserve %d bytes of shared memory: %s", sp.bytes, cudaGetErrorString(e));
        }
        kernel<<<plane_grid(g.planes), 256, sp.bytes, st>>>((decltype(pool_arg_y(kernel)))y, (decltype(pool_arg_x(kernel)))x, g, sp.lw_out, vec);
        LB2_CHECK_LAUNCH("pool2d_fwd (staged)");
        return LB2_OK;
      };
      const int kfix = kind == LB2_POOL_MAX ? pool_fixed_window(g) : 0;
      LB2_DISPATCH_DTYPE(dtype, {
        if (kind == LB2_POOL_MAX) {
          if (kfix == 3) return st2 == 1 ? launch(pool2d_fwd_smem_kernel<T, true, 1, 3>) : st2 == 2 ? launch(pool2d_fwd_smem_kernel<T, true, 2, 3>) : launch(pool2d_fwd_smem_kernel<T, true, 0, 3>);
          if (kfix == 2) return st2 == 1 ? launch(pool2d_fwd_smem_kernel<T, true, 1, 2>) : st2 == 2 ? launch(pool2d_fwd_smem_kernel<T, true, 2, 2>) : launch(pool2d_fwd_smem_kernel<T, true, 0, 2>);
          return st2 == 1 ? launch(pool2d_fwd_smem_kernel<T, true, 1, 0>) : st2 == 2 ? launch(pool2d_fwd_smem_kernel<T, true, 2, 0>) : launch(pool2d_fwd_smem_kernel<T, true, 0, 0>);
        }
        return st2 == 1 ? launch(pool2d_fwd_smem_kernel<T, false, 1, 0>) : st2 == 2 ? launch(pool2d_fwd_smem_kernel<T, false, 2, 0>) : launch(pool2d_fwd_smem_kernel<T, false, 0, 0>);
      });
    }
    LB2_DISPATCH_DTYPE(dtype, {
      if (kind == LB2_POOL_MAX) {
        if (same && g.stride[0] == 1) pool2d_fwd_kernel<T, true, 1><<<plane_grid(g.planes), 256, 0, st>>>((T*)y, (const T*)x, g);
        else if (same && g.stride[0] == 2) pool2d_fwd_kernel<T, true, 2><<<plane_grid(g.planes), 256, 0, st>>>((T*)y, (const T*)x, g);
        else pool2d_fwd_kernel<T, true, 0><<<plane_grid(g.planes), 256, 0, st>>>((T*)y, (const T*)x, g);
      } else {
        if (same && g.stride[0] == 1) pool2d_fwd_kernel<T, false, 1><<<plane_grid(g.planes), 256, 0, st>>>((T*)y, (const T*)x, g);
        else if (same && g.stride[0] == 2) pool2d_fwd_kernel<T, false, 2><<<plane_grid(g.planes), 256, 0, st>>>((T*)y, (const T*)x, g);
        else pool2d_fwd_kernel<T, false, 0><<<plane_grid(g.planes), 256, 0, st>>>((T*)y, (const T*)x, g);
      }
    });
    LB2_CHECK_LAUNCH("pool2d_fwd");
    return LB2_OK;
  }
  LB2_DISPATCH_DTYPE(dtype, {
    if (kind == LB2_POOL_MAX) pool_fwd_kernel<T, true><<<plane_grid(g.planes), 256, 0, st>>>((T*)y, (const T*)x, g);
    else pool_fwd_kernel<T, false><<<plane_grid(g.planes), 256, 0, st>>>((T*)y, (const T*)x, g);
  });
  LB2_CHECK_LAUNCH("pool_fwd");
  return LB2_OK;
}

int32_t lb2_pool_bwd(void* dx, const void* dy, const void* y, const void* x, const lb2_pool_desc* d, int32_t kind,
                     int32_t dtype, void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(kind == LB2_POOL_MAX || kind == LB2_POOL_MEAN, LB2_BAD_ARG, "unknown pooling kind %d", (int)kind);
  PoolGeom g;
  int32_t rc = make_pool_geom(d, &g);
  if (rc != LB2_OK) return rc;
  const int64_t total = (int64_t)g.in[0] * g.in[1] * g.in[2] * g.planes;
  if (total == 0) return LB2_OK;
  LB2_REQUIRE(dx != nullptr, LB2_BAD_ARG, "dx is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t out_total = (int64_t)g.out[0] * g.out[1] * g.out[2] * g.planes;
  if (out_total == 0) {
    cudaMemsetAsync(dx, 0, (size_t)total * dtype_size(dtype), st);
    return LB2_OK;
  }
  LB2_REQUIRE(dy != nullptr, LB2_BAD_ARG, "dy is null");
  LB2_REQUIRE(kind == LB2_POOL_MEAN || (y && x), LB2_BAD_ARG, "max pooling needs y and x for its gradient");
  const size_t es = dtype_size(dtype);
  LB2_REQUIRE(aligned_to(dx, es) && aligned_to(dy, es) && aligned_to(y, es) && aligned_to(x, es), LB2_BAD_ALIGN,
              "pointer not aligned to the element size");
  bool global = true;
  for (int i = 0; i < 3; ++i) global = global && g.out[i] == 1 && g.pad[i] == 0 && g.dil[i] == 1 && g.k[i] == g.in[i];
  if (global) {
    const int64_t S = (int64_t)g.in[0] * g.in[1] * g.in[2];
    LB2_DISPATCH_DTYPE(dtype, {
      if (kind == LB2_POOL_MAX) pool_global_bwd_kernel<T, true><<<pool_grid(g.planes * 32), 256, 0, st>>>((T*)dx, (const T*)dy, (const T*)y, (const T*)x, S, g.planes);
      else pool_global_bwd_kernel<T, false><<<pool_grid(g.planes * 32), 256, 0, st>>>((T*)dx, (const T*)dy, nullptr, nullptr, S, g.planes);
    });
    LB2_CHECK_LAUNCH("pool_global_bwd");
    return LB2_OK;
  }
  if (pool_is_2d_plain(g)) {
    const bool same = g.stride[0] == g.stride[1];
    const PoolSmem sp = pool_smem_plan(g, es, kind == LB2_POOL_MAX ? 2 : 1);
    if (sp.ok) {
      const int vec_in = (aligned_to(x, 16) && aligned_to(dx, 16) && ((size_t)g.in[0] * g.in[1] * es) % 16 == 0) ? 1 : 0;
      const int vec_out = (aligned_to(dy, 16) && ((size_t)g.out[0] * g.out[1] * es) % 16 == 0) ? 1 : 0;
      const int st2 = same && g.stride[0] <= 2 ? g.stride[0] : 0;
      auto reserve = [&](auto kernel) -> int32_t {
        if (sp.bytes > 48 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.bytes);
          if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "pool2d_bwd: cannot reserve %d bytes of shared memory: %s", sp.bytes, cudaGetErrorString(e));
        }
        return LB2_OK;
      };
      auto launch_max = [&](auto kernel) -> int32_t {
        if (int32_t rc = reserve(kernel)) return rc;
        // a class of windows is one pass of 1024 threads for planes up to about 64 x 64 outputs; small planes take fewer
        const int per_class = ((g.out[1] + sp.ch - 1) / sp.ch) << sp.lw_cls;
        const int threads = per_class > 512 ? 1024 : per_class > 256 ? 512 : 256;
        kernel<<<plane_grid(g.planes), threads, sp.bytes, st>>>((decltype(pool_arg_y(kernel)))dx, (decltype(pool_arg_x(kernel)))dy,
                                                            (decltype(pool_arg_x(kernel)))x, g, sp.lw_cls, vec_in, vec_out, sp.off_acc, sp.off_dy, sp.cw, sp.ch);
        LB2_CHECK_LAUNCH("pool2d_bwd (max, staged)");
        return LB2_OK;
      };
      auto launch_mean = [&](auto kernel) -> int32_t {
        if (int32_t rc = reserve(kernel)) return rc;
        kernel<<<plane_grid(g.planes), 256, sp.bytes, st>>>((decltype(pool_arg_y(kernel)))dx, (decltype(pool_arg_x(kernel)))dy, g, sp.lw_in, vec_out);
        LB2_CHECK_LAUNCH("pool2d_bwd (mean, staged)");
        return LB2_OK;
      };
      LB2_DISPATCH_DTYPE(dtype, {
        if (kind == LB2_POOL_MAX) {
          const int kfix = pool_fixed_window(g);
          if (kfix == 3) return st2 == 1 ? launch_max(pool2d_maxbwd_smem_kernel<T, 1, 3>) : st2 == 2 ? launch_max(pool2d_maxbwd_smem_kernel<T, 2, 3>) : launch_max(pool2d_maxbwd_smem_kernel<T, 0, 3>);
          if (kfix == 2) return st2 == 1 ? launch_max(pool2d_maxbwd_smem_kernel<T, 1, 2>) : st2 == 2 ? launch_max(pool2d_maxbwd_smem_kernel<T, 2, 2>) : launch_max(pool2d_maxbwd_smem_kernel<T, 0, 2>);
          return st2 == 1 ? launch_max(pool2d_maxbwd_smem_kernel<T, 1, 0>) : st2 == 2 ? launch_max(pool2d_maxbwd_smem_kernel<T, 2, 0>) : launch_max(pool2d_maxbwd_smem_kernel<T, 0, 0>);
        }
        return st2 == 1 ? launch_mean(pool2d_meanbwd_smem_kernel<T, 1>) : st2 == 2 ? launch_mean(pool2d_meanbwd_smem_kernel<T, 2>) : launch_mean(pool2d_meanbwd_smem_kernel<T, 0>);
      });
    }
    LB2_DISPATCH_DTYPE(dtype, {
      if (kind == LB2_POOL_MAX) {
        if (same && g.stride[0] == 1) pool2d_bwd_kernel<T, true, 1><<<plane_grid(g.planes), 256, 0, st>>>((T*)dx, (const T*)dy, (const T*)y, (const T*)x, g);
        else if (same && g.stride[0] == 2) pool2d_bwd_kernel<T, true, 2><<<plane_grid(g.planes), 256, 0, st>>>((T*)dx, (const T*)dy, (const T*)y, (const T*)x, g);
        else pool2d_bwd_kernel<T, true, 0><<<plane_grid(g.planes), 256, 0, st>>>((T*)dx, (const T*)dy, (const T*)y, (const T*)x, g);
      } else {
        if (same && g.stride[0] == 1) pool2d_bwd_kernel<T, false, 1><<<plane_grid(g.planes), 256, 0, st>>>((T*)dx, (const T*)dy, nullptr, nullptr, g);
        else if (same && g.stride[0] == 2) pool2d_bwd_kernel<T, false, 2><<<plane_grid(g.planes), 256, 0, st>>>((T*)dx, (const T*)dy, nullptr, nullptr, g);
        else pool2d_bwd_kernel<T, false, 0><<<plane_grid(g.planes), 256, 0, st>>>((T*)dx, (const T*)dy, nullptr, nullptr, g);
      }
    });
    LB2_CHECK_LAUNCH("pool2d_bwd");
    return LB2_OK;
  }
  LB2_DISPATCH_DTYPE(dtype, {
    if (kind == LB2_POOL_MAX) pool_bwd_kernel<T, true><<<plane_grid(g.planes), 256, 0, st>>>((T*)dx, (const T*)dy, (const T*)y, (const T*)x, g);
    else pool_bwd_kernel<T, false><<<plane_grid(g.planes), 256, 0, st>>>((T*)dx, (const T*)dy, nullptr, nullptr, g);
  });
  LB2_CHECK_LAUNCH("pool_bwd");
  return LB2_OK;
}

}  // extern "C"

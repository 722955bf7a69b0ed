// Bandwidth-bound element-wise kernels: activation, bias+activation and their pullbacks
// (activation derivative fused with the bias-gradient reduction in one pass over the data).
//
// Data layout: the (S, C, B) column-major view of lib/LuxLib/src/impl/bias_activation.jl:229-235;
// S contiguous. Every thread moves 16-byte vectors; reductions are two-stage with a fixed
// order (per-CTA partials in the caller's workspace, then one finishing kernel), so results are
// run-to-run deterministic — no float atomics.
#include "common.cuh"
#include "eltwise.cuh"

namespace lb2 {

// ------------------------------------------------------------------------------------------
// forward: y = act(x + bias[c])
// ------------------------------------------------------------------------------------------
template <typename T, int ACT, bool VEC, bool HAS_BIAS>
__global__ void __launch_bounds__(256) bias_act_fwd_kernel(T* __restrict__ y, const T* __restrict__ x,
                                                           const T* __restrict__ bias, int64_t n, int64_t S,
                                                           int64_t C) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = VEC ? Vec16<T>::N : 1;
  const int64_t nvec = n / V;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const int64_t e = i * V;
    if constexpr (VEC) {
      // VEC is only selected when S % V == 0 (one channel per vector) or there is no bias
      float b = 0.f;
      if constexpr (HAS_BIAS) b = to_f32(bias[(e / S) % C]);
      const Vec16<T> v = load16_stream(x + e);
      store16_stream(y + e, vec_from<T>([&](int j) { return act_apply<ACT, FAST>(v.get(j) + b); }));
    } else {
      float b = 0.f;
      if constexpr (HAS_BIAS) b = to_f32(bias[(e / S) % C]);
      y[e] = from_f32<T>(act_apply<ACT, FAST>(to_f32(x[e]) + b));
    }
  }
  if constexpr (VEC && !HAS_BIAS) {  // ragged tail of a flat array
    const int64_t e = nvec * V + threadIdx.x;
    if (blockIdx.x == 0 && e < n) y[e] = from_f32<T>(act_apply<ACT, FAST>(to_f32(x[e])));
  }
}

// Dense-shaped forward (S == 1): bias varies along the contiguous dimension.
template <typename T, int ACT, bool VEC>
__global__ void __launch_bounds__(256) bias_act_fwd_s1_kernel(T* __restrict__ y, const T* __restrict__ x,
                                                              const T* __restrict__ bias, int64_t n, int64_t C) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = VEC ? Vec16<T>::N : 1;
  const int64_t nvec = n / V;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const int64_t e = i * V;
    const int64_t c = e % C;  // C % V == 0 on the vector path
    if constexpr (VEC) {
      const Vec16<T> v = load16_stream(x + e);
      const Vec16<T> bv = load16(bias + c);
      store16_stream(y + e, vec_from<T>([&](int j) { return act_apply<ACT, FAST>(v.get(j) + bv.get(j)); }));
    } else {
      y[e] = from_f32<T>(act_apply<ACT, FAST>(to_f32(x[e]) + to_f32(bias[c])));
    }
  }
}

template <typename T, int ACT>
static int32_t launch_bias_act_fwd(T* y, const T* x, const T* bias, int64_t S, int64_t C, int64_t B,
                                   cudaStream_t st) {
  const int64_t n = S * C * B;
  constexpr int V = Vec16<T>::N;
  const bool ptr_ok = aligned_to(y, 16) && aligned_to(x, 16);
  const int threads = 256;
  auto grid_for = [&](int64_t items) {
    int64_t g = (items + threads - 1) / threads;
    int64_t cap = (int64_t)sm_count() * 16;
    return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
  };
  if (bias && S == 1) {
    const bool vec = ptr_ok && aligned_to(bias, 16) && (C % V == 0);
    if (vec) bias_act_fwd_s1_kernel<T, ACT, true><<<grid_for(n / V), threads, 0, st>>>(y, x, bias, n, C);
    else bias_act_fwd_s1_kernel<T, ACT, false><<<grid_for(n), threads, 0, st>>>(y, x, bias, n, C);
  } else if (bias) {
    const bool vec = ptr_ok && (S % V == 0);
    if (vec) bias_act_fwd_kernel<T, ACT, true, true><<<grid_for(n / V), threads, 0, st>>>(y, x, bias, n, S, C);
    else bias_act_fwd_kernel<T, ACT, false, true><<<grid_for(n), threads, 0, st>>>(y, x, bias, n, S, C);
  } else {
    const bool vec = ptr_ok && n >= V;
    if (vec) bias_act_fwd_kernel<T, ACT, true, false><<<grid_for(n / V), threads, 0, st>>>(y, x, nullptr, n, S, C);
    else bias_act_fwd_kernel<T, ACT, false, false><<<grid_for(n), threads, 0, st>>>(y, x, nullptr, n, S, C);
  }
  LB2_CHECK_LAUNCH("bias_act_fwd");
  return LB2_OK;
}

// ------------------------------------------------------------------------------------------
// backward: dx = dy * act'(out|pre); optional per-channel partial sums of dx
// ------------------------------------------------------------------------------------------
template <int ACT, bool FAST, bool FROM_PRE> __device__ __forceinline__ float dact_sel(float v) {
  if constexpr (FROM_PRE) return act_grad_pre<ACT, FAST>(v);
  else return act_grad_out<ACT>(v);
}

// Matrix-shaped (S == 1): C x B with leading dimension ld; reduce over B.
// block (32, 8): x -> vector of V channels, y -> row slot; grid (strips, chunks).
template <typename T, int ACT, bool VEC, bool FROM_PRE, bool WANT_SUM>
__global__ void __launch_bounds__(256) act_bwd_s1_kernel(T* __restrict__ dx, float* __restrict__ partial,
                                                         const T* __restrict__ dy, const T* __restrict__ ref,
                                                         int64_t C, int64_t B, int64_t ld_dx, int64_t ld_dy,
                                                         int64_t ld_ref, int64_t rows_per_chunk) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = VEC ? Vec16<T>::N : 1;
  __shared__ float red[8][32 * V + 1];
  const int64_t c0 = ((int64_t)blockIdx.x * 32 + threadIdx.x) * V;
  const int64_t b_begin = (int64_t)blockIdx.y * rows_per_chunk;
  const int64_t b_end = min(B, b_begin + rows_per_chunk);
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.f;
  if (c0 < C) {
    for (int64_t b = b_begin + threadIdx.y; b < b_end; b += 8) {
      if constexpr (VEC) {
        Vec16<T> g = load16_stream(dy + b * ld_dy + c0);
        if constexpr (ACT != LB2_ACT_IDENTITY) {
          Vec16<T> r = load16_stream(ref + b * ld_ref + c0);
          const Vec16<T> g0 = g;
          g = vec_from<T>([&](int j) { return g0.get(j) * dact_sel<ACT, FAST, FROM_PRE>(r.get(j)); });
        }
        if (dx) store16(dx + b * ld_dx + c0, g);
        if constexpr (WANT_SUM) {
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] += g.get(j);  // sums the stored (rounded) values
        }
      } else {
        float g = to_f32(dy[b * ld_dy + c0]);
        if constexpr (ACT != LB2_ACT_IDENTITY) g *= dact_sel<ACT, FAST, FROM_PRE>(to_f32(ref[b * ld_ref + c0]));
        T gs = from_f32<T>(g);
        if (dx) dx[b * ld_dx + c0] = gs;
        if constexpr (WANT_SUM) acc[0] += to_f32(gs);
      }
    }
  }
  if constexpr (WANT_SUM) {
#pragma unroll
    for (int j = 0; j < V; ++j) red[threadIdx.y][threadIdx.x * V + j] = acc[j];
    __syncthreads();
    const int tid = threadIdx.y * 32 + threadIdx.x;
    for (int col = tid; col < 32 * V; col += 256) {
      float s = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) s += red[r][col];
      int64_t c = (int64_t)blockIdx.x * 32 * V + col;
      if (c < C) partial[(int64_t)blockIdx.y * C + c] = s;
    }
  }
}

// General (S > 1): grid (C, chunks); the CTA walks rows (c, b) of S contiguous elements.
template <typename T, int ACT, bool VEC, bool FROM_PRE, bool WANT_SUM>
__global__ void __launch_bounds__(256) act_bwd_kernel(T* __restrict__ dx, float* __restrict__ partial,
                                                      const T* __restrict__ dy, const T* __restrict__ ref,
                                                      int64_t S, int64_t C, int64_t B, int64_t rows_per_chunk) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = VEC ? Vec16<T>::N : 1;
  __shared__ float red[32];
  const int64_t c = blockIdx.x;
  const int64_t b_begin = (int64_t)blockIdx.y * rows_per_chunk;
  const int64_t b_end = min(B, b_begin + rows_per_chunk);
  const int64_t sv = S / V;  // VEC only when S % V == 0
  float acc = 0.f;
  if constexpr (VEC) {
    // A warp takes units of 128 vectors (4 per lane, all loads issued before any is used) of one (channel,
    // sample) row; the unit -> (sample, segment) division happens once per unit.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t upr = (uint32_t)((sv + 127) / 128);
    const int64_t units = (b_end - b_begin) * (int64_t)upr;
    for (int64_t u = warp; u < units; u += 8) {
      const int64_t b = b_begin + u / upr;
      const int64_t v0 = (int64_t)(u % upr) * 128 + lane;
      const int64_t base = (b * C + c) * S;
      Vec16<T> g[4], r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t v = v0 + k * 32;
        if (v < sv) {
          g[k] = load16_stream(dy + base + v * V);
          if constexpr (ACT != LB2_ACT_IDENTITY) r[k] = load16_stream(ref + base + v * V);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t v = v0 + k * 32;
        if (v < sv) {
          if constexpr (ACT != LB2_ACT_IDENTITY) {
            const Vec16<T> g0 = g[k];
            g[k] = vec_from<T>([&](int j) { return g0.get(j) * dact_sel<ACT, FAST, FROM_PRE>(r[k].get(j)); });
          }
          if (dx) store16(dx + base + v * V, g[k]);
          if constexpr (WANT_SUM) {
#pragma unroll
            for (int j = 0; j < V; ++j) acc += g[k].get(j);
          }
        }
      }
    }
  } else {
    const int64_t items = (b_end - b_begin) * sv;
    for (int64_t it = threadIdx.x; it < items; it += blockDim.x) {
      const int64_t b = b_begin + it / sv;
      const int64_t e = (b * C + c) * S + (it % sv) * V;
      float g = to_f32(dy[e]);
      if constexpr (ACT != LB2_ACT_IDENTITY) g *= dact_sel<ACT, FAST, FROM_PRE>(to_f32(ref[e]));
      T gs = from_f32<T>(g);
      if (dx) dx[e] = gs;
      if constexpr (WANT_SUM) acc += to_f32(gs);
    }
  }
  if constexpr (WANT_SUM) {
    float s = block_sum(acc, red);
    if (threadIdx.x == 0) partial[(int64_t)blockIdx.y * C + c] = s;
  }
}

// Flat pullback without a reduction: dx = dy * act'(ref) over n contiguous elements.
template <typename T, int ACT, bool VEC, bool FROM_PRE>
__global__ void __launch_bounds__(256) act_bwd_flat_kernel(T* __restrict__ dx, const T* __restrict__ dy,
                                                           const T* __restrict__ ref, int64_t n) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = VEC ? Vec16<T>::N : 1;
  const int64_t nvec = n / V;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const int64_t e = i * V;
    if constexpr (VEC) {
      Vec16<T> g = load16_stream(dy + e);
      Vec16<T> r = load16_stream(ref + e);
      store16_stream(dx + e, vec_from<T>([&](int j) { return g.get(j) * dact_sel<ACT, FAST, FROM_PRE>(r.get(j)); }));
    } else {
      dx[e] = from_f32<T>(to_f32(dy[e]) * dact_sel<ACT, FAST, FROM_PRE>(to_f32(ref[e])));
    }
  }
  if constexpr (VEC) {
    const int64_t e = nvec * V + threadIdx.x;
    if (blockIdx.x == 0 && e < n) dx[e] = from_f32<T>(to_f32(dy[e]) * dact_sel<ACT, FAST, FROM_PRE>(to_f32(ref[e])));
  }
}

template <typename T, int ACT, bool FROM_PRE>
static int32_t launch_act_bwd_flat_t(T* dx, const T* dy, const T* ref, int64_t n, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  if constexpr (ACT == LB2_ACT_IDENTITY) {
    if (dx != dy) cudaMemcpyAsync(dx, dy, (size_t)n * sizeof(T), cudaMemcpyDeviceToDevice, st);
    LB2_CHECK_LAUNCH("act_bwd_flat(copy)");
    return LB2_OK;
  }
  const bool vec = aligned_to(dx, 16) && aligned_to(dy, 16) && aligned_to(ref, 16) && n >= V;
  const int64_t items = vec ? n / V : n;
  int64_t g = (items + 255) / 256, cap = (int64_t)sm_count() * 16;
  unsigned grid = (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
  if (vec) act_bwd_flat_kernel<T, ACT, true, FROM_PRE><<<grid, 256, 0, st>>>(dx, dy, ref, n);
  else act_bwd_flat_kernel<T, ACT, false, FROM_PRE><<<grid, 256, 0, st>>>(dx, dy, ref, n);
  LB2_CHECK_LAUNCH("act_bwd_flat");
  return LB2_OK;
}

static int32_t launch_act_bwd_flat(void* dx, const void* dy, const void* out, const void* pre, int64_t n,
                                   int32_t dtype, int32_t act, cudaStream_t st) {
  const bool from_pre = (pre != nullptr);
  const void* ref = from_pre ? pre : out;
  LB2_DISPATCH_DTYPE(dtype, {
    LB2_DISPATCH_ACT(act, {
      if (from_pre)
        return launch_act_bwd_flat_t<T, ACT, true>((T*)dx, (const T*)dy, (const T*)ref, n, st);
      else if constexpr (ACT == LB2_ACT_IDENTITY || ACT == LB2_ACT_RELU || ACT == LB2_ACT_TANH || ACT == LB2_ACT_SIGMOID)
        return launch_act_bwd_flat_t<T, ACT, false>((T*)dx, (const T*)dy, (const T*)ref, n, st);
      else
        return fail(LB2_BAD_ARG, "activation %d needs the pre-activation for its derivative", (int)act);
    });
  });
  return LB2_OK;
}

// db[c] (+)= sum over chunks of partial[chunk][c], in chunk order.
template <typename T>
__global__ void finish_colsum_kernel(T* __restrict__ out, const float* __restrict__ partial, int64_t C,
                                     int chunks, int accumulate) {
  int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int k = 0; k < chunks; ++k) s += partial[(int64_t)k * C + c];
  if (accumulate) s += to_f32(out[c]);
  out[c] = from_f32<T>(s);
}

int act_bwd_chunks(int64_t S, int64_t C, int64_t B) {
  // enough CTAs to fill the machine a few times over, never more chunks than rows
  const int64_t target = (int64_t)sm_count() * 4;
  int64_t ctas_per_chunk = (S == 1) ? (C + 255) / 256 : C;
  if (ctas_per_chunk < 1) ctas_per_chunk = 1;
  int64_t chunks = (target + ctas_per_chunk - 1) / ctas_per_chunk;
  if (S == 1) {
    int64_t maxc = (B + 63) / 64;  // at least 64 rows per chunk
    if (chunks > maxc) chunks = maxc;
  } else if (chunks > B) {
    chunks = B;
  }
  if (chunks < 1) chunks = 1;
  if (chunks > 1024) chunks = 1024;
  return (int)chunks;
}

size_t act_bwd_workspace_bytes(int64_t S, int64_t C, int64_t B) {
  return align_up((size_t)act_bwd_chunks(S, C, B) * (size_t)C * sizeof(float), 256);
}

template <typename T, int ACT, bool FROM_PRE>
static int32_t launch_act_bwd_t(T* dx, T* db, const T* dy, const T* ref, int64_t S, int64_t C, int64_t B,
                                int64_t ld_dx, int64_t ld_dy, int64_t ld_ref, int accumulate_db, float* ws,
                                cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  const int chunks = act_bwd_chunks(S, C, B);
  const int64_t rows_per_chunk = (B + chunks - 1) / chunks;
  const bool ptr_ok = aligned_to(dy, 16) && (!dx || aligned_to(dx, 16)) && (!ref || aligned_to(ref, 16));
  if (S == 1) {
    const bool vec = ptr_ok && C % V == 0 && ld_dx % V == 0 && ld_dy % V == 0 && ld_ref % V == 0;
    dim3 block(32, 8);
    if (vec) {
      dim3 grid((unsigned)((C + 32 * V - 1) / (32 * V)), chunks);
      if (db) act_bwd_s1_kernel<T, ACT, true, FROM_PRE, true><<<grid, block, 0, st>>>(dx, ws, dy, ref, C, B, ld_dx, ld_dy, ld_ref, rows_per_chunk);
      else act_bwd_s1_kernel<T, ACT, true, FROM_PRE, false><<<grid, block, 0, st>>>(dx, ws, dy, ref, C, B, ld_dx, ld_dy, ld_ref, rows_per_chunk);
    } else {
      dim3 grid((unsigned)((C + 31) / 32), chunks);
      if (db) act_bwd_s1_kernel<T, ACT, false, FROM_PRE, true><<<grid, block, 0, st>>>(dx, ws, dy, ref, C, B, ld_dx, ld_dy, ld_ref, rows_per_chunk);
      else act_bwd_s1_kernel<T, ACT, false, FROM_PRE, false><<<grid, block, 0, st>>>(dx, ws, dy, ref, C, B, ld_dx, ld_dy, ld_ref, rows_per_chunk);
    }
  } else {
    const bool vec = ptr_ok && S % V == 0;
    dim3 grid((unsigned)C, chunks);
    if (vec) {
      if (db) act_bwd_kernel<T, ACT, true, FROM_PRE, true><<<grid, 256, 0, st>>>(dx, ws, dy, ref, S, C, B, rows_per_chunk);
      else act_bwd_kernel<T, ACT, true, FROM_PRE, false><<<grid, 256, 0, st>>>(dx, ws, dy, ref, S, C, B, rows_per_chunk);
    } else {
      if (db) act_bwd_kernel<T, ACT, false, FROM_PRE, true><<<grid, 256, 0, st>>>(dx, ws, dy, ref, S, C, B, rows_per_chunk);
      else act_bwd_kernel<T, ACT, false, FROM_PRE, false><<<grid, 256, 0, st>>>(dx, ws, dy, ref, S, C, B, rows_per_chunk);
    }
  }
  LB2_CHECK_LAUNCH("act_bwd");
  if (db) {
    finish_colsum_kernel<T><<<(unsigned)((C + 255) / 256), 256, 0, st>>>(db, ws, C, chunks, accumulate_db);
    LB2_CHECK_LAUNCH("finish_colsum");
  }
  return LB2_OK;
}

// Shared by lb2_act_bwd, lb2_bias_act_bwd, lb2_dense_bwd and lb2_conv_bwd.
int32_t launch_act_bwd(void* dx, void* db, const void* dy, const void* out, const void* pre, int64_t S,
                       int64_t C, int64_t B, int64_t ld_dx, int64_t ld_dy, int64_t ld_ref, int32_t dtype,
                       int32_t act, int accumulate_db, float* ws, cudaStream_t st) {
  const bool from_pre = (pre != nullptr);
  const void* ref = from_pre ? pre : out;
  LB2_DISPATCH_DTYPE(dtype, {
    LB2_DISPATCH_ACT(act, {
      if (from_pre)
        return launch_act_bwd_t<T, ACT, true>((T*)dx, (T*)db, (const T*)dy, (const T*)ref, S, C, B, ld_dx, ld_dy, ld_ref, accumulate_db, ws, st);
      else if constexpr (ACT == LB2_ACT_IDENTITY || ACT == LB2_ACT_RELU || ACT == LB2_ACT_TANH || ACT == LB2_ACT_SIGMOID)
        return launch_act_bwd_t<T, ACT, false>((T*)dx, (T*)db, (const T*)dy, (const T*)ref, S, C, B, ld_dx, ld_dy, ld_ref, accumulate_db, ws, st);
      else
        return fail(LB2_BAD_ARG, "activation %d needs the pre-activation for its derivative", (int)act);
    });
  });
  return LB2_OK;
}

int32_t check_act_bwd_args(const void* dy, const void* out, const void* pre, int32_t dtype, int32_t act) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(valid_act(act), LB2_BAD_ARG, "unknown activation %d", (int)act);
  LB2_REQUIRE(dy != nullptr, LB2_BAD_ARG, "dy is null");
  if (act != LB2_ACT_IDENTITY) {
    LB2_REQUIRE(out != nullptr || pre != nullptr, LB2_BAD_ARG, "need `out` or `pre` for the activation derivative");
    LB2_REQUIRE(pre != nullptr || act_grad_from_output(act), LB2_BAD_ARG,
                "activation %d needs the pre-activation for its derivative", (int)act);
  }
  return LB2_OK;
}

}  // namespace lb2

using namespace lb2;

extern "C" {

int32_t lb2_bias_act_fwd(void* y, const void* x, const void* bias, int64_t S, int64_t C, int64_t B,
                         int32_t dtype, int32_t act, void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(valid_act(act), LB2_BAD_ARG, "unknown activation %d", (int)act);
  LB2_REQUIRE(S >= 0 && C >= 0 && B >= 0, LB2_BAD_SHAPE, "negative extent");
  if (S == 0 || C == 0 || B == 0) return LB2_OK;
  LB2_REQUIRE(y && x, LB2_BAD_ARG, "null tensor pointer");
  const size_t es = dtype_size(dtype);
  LB2_REQUIRE(aligned_to(y, es) && aligned_to(x, es) && (!bias || aligned_to(bias, es)), LB2_BAD_ALIGN,
              "pointer not aligned to the element size");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LB2_DISPATCH_DTYPE(dtype, {
    LB2_DISPATCH_ACT(act, { return launch_bias_act_fwd<T, ACT>((T*)y, (const T*)x, (const T*)bias, S, C, B, st); });
  });
  return LB2_OK;
}

int32_t lb2_act_fwd(void* y, const void* x, int64_t n, int32_t dtype, int32_t act, void* stream) {
  LB2_REQUIRE(n >= 0, LB2_BAD_SHAPE, "negative length");
  return lb2_bias_act_fwd(y, x, nullptr, n, 1, 1, dtype, act, stream);
}

size_t lb2_bias_act_bwd_workspace_bytes(int64_t S, int64_t C, int64_t B) {
  if (S <= 0 || C <= 0 || B <= 0) return 0;
  return act_bwd_workspace_bytes(S, C, B);
}

int32_t lb2_bias_act_bwd(void* dx, void* dbias, const void* dy, const void* out, const void* pre, int64_t S,
                         int64_t C, int64_t B, int32_t dtype, int32_t act, void* workspace,
                         size_t workspace_bytes, void* stream) {
  LB2_REQUIRE(S >= 0 && C >= 0 && B >= 0, LB2_BAD_SHAPE, "negative extent");
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(valid_act(act), LB2_BAD_ARG, "unknown activation %d", (int)act);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (S == 0 || C == 0 || B == 0) {
    if (dbias && C > 0) cudaMemsetAsync(dbias, 0, (size_t)C * dtype_size(dtype), st);
    return LB2_OK;
  }
  int32_t rc = check_act_bwd_args(dy, out, pre, dtype, act);
  if (rc != LB2_OK) return rc;
  LB2_REQUIRE(dx || dbias, LB2_BAD_ARG, "nothing to compute: dx and dbias are both null");
  if (dbias) {
    LB2_REQUIRE(workspace != nullptr && workspace_bytes >= act_bwd_workspace_bytes(S, C, B), LB2_WORKSPACE_TOO_SMALL,
                "workspace of %zu bytes needed", act_bwd_workspace_bytes(S, C, B));
    LB2_REQUIRE(aligned_to(workspace, 16), LB2_BAD_ALIGN, "workspace must be 16-byte aligned");
  }
  return launch_act_bwd(dx, dbias, dy, out, pre, S, C, B, C, C, C, dtype, act, 0, (float*)workspace, st);
}

int32_t lb2_act_bwd(void* dx, const void* dy, const void* out, const void* pre, int64_t n, int32_t dtype,
                    int32_t act, void* stream) {
  LB2_REQUIRE(n >= 0, LB2_BAD_SHAPE, "negative length");
  if (n == 0) return LB2_OK;
  LB2_REQUIRE(dx != nullptr, LB2_BAD_ARG, "dx is null");
  int32_t rc = check_act_bwd_args(dy, out, pre, dtype, act);
  if (rc != LB2_OK) return rc;
  return launch_act_bwd_flat(dx, dy, out, pre, n, dtype, act, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

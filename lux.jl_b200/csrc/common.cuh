// Shared device/host helpers for libluxlib_b200: status handling, dtype traits,
// vector loads and the scalar activation set with its derivatives.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/luxlib_b200.h"

namespace lb2 {

// ---- host-side error plumbing ---------------------------------------------------------------
void set_error(const char* fmt, ...);  // thread-local message, defined in api.cu
int32_t fail(int32_t status, const char* fmt, ...);
int sm_count();                        // cached per device
unsigned int* device_status_word();    // per-device status word written by bounded waits

#define LB2_REQUIRE(cond, status, ...)                      \
  do {                                                      \
    if (!(cond)) return ::lb2::fail((status), __VA_ARGS__); \
  } while (0)

#define LB2_CHECK_LAUNCH(what)                                                         \
  do {                                                                                 \
    cudaError_t e__ = cudaGetLastError();                                              \
    if (e__ != cudaSuccess)                                                            \
      return ::lb2::fail(LB2_LAUNCH_FAIL, "%s: %s", (what), cudaGetErrorString(e__)); \
  } while (0)

inline bool valid_dtype(int32_t d) { return d == LB2_F32 || d == LB2_BF16; }
inline bool valid_act(int32_t a) { return a >= LB2_ACT_IDENTITY && a <= LB2_ACT_SWISH; }
inline size_t dtype_size(int32_t d) { return d == LB2_BF16 ? 2 : 4; }
inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
__device__ __forceinline__ bool aligned_to_dev(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
// sigma' computable from the output alone (lib/LuxLib/src/traits.jl:59-65)
inline bool act_grad_from_output(int32_t a) {
  return a == LB2_ACT_IDENTITY || a == LB2_ACT_RELU || a == LB2_ACT_TANH || a == LB2_ACT_SIGMOID;
}
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- element access ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 16-byte vector of T: 4 floats or 8 bf16.
template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  union {
    uint4 raw;
    uint32_t w[4];
  };
  __device__ __forceinline__ Vec16() {}
  __device__ __forceinline__ float get(int i) const {
    if constexpr (sizeof(T) == 4) {
      return __uint_as_float(w[i]);
    } else {
      const uint32_t u = w[i >> 1];
      return __uint_as_float((i & 1) ? (u & 0xFFFF0000u) : (u << 16));
    }
  }
  __device__ __forceinline__ void set(int i, float v) {
    if constexpr (sizeof(T) == 4) {
      w[i] = __float_as_uint(v);
    } else {
      const uint32_t h = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
      uint32_t& u = w[i >> 1];
      u = (i & 1) ? ((u & 0x0000FFFFu) | (h << 16)) : ((u & 0xFFFF0000u) | h);
    }
  }
  // elements i (even) and i+1 at once: one packed conversion for bf16
  __device__ __forceinline__ void set2(int i, float a, float b) {
    if constexpr (sizeof(T) == 4) {
      w[i] = __float_as_uint(a);
      w[i + 1] = __float_as_uint(b);
    } else {
      uint32_t u;
      asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(u) : "f"(b), "f"(a));
      w[i >> 1] = u;
    }
  }
};
// builds a vector from f(j), j = 0..N-1, converting two elements per instruction for bf16
template <typename T, typename F> __device__ __forceinline__ Vec16<T> vec_from(F&& f) {
  Vec16<T> o;
#pragma unroll
  for (int j = 0; j < Vec16<T>::N; j += 2) o.set2(j, f(j), f(j + 1));
  return o;
}
template <typename T> __device__ __forceinline__ Vec16<T> load16(const T* p) {
  Vec16<T> v;
  v.raw = *reinterpret_cast<const uint4*>(p);
  return v;
}
// streaming variants: data touched once
template <typename T> __device__ __forceinline__ Vec16<T> load16_stream(const T* p) {
  Vec16<T> v;
  v.raw = __ldcs(reinterpret_cast<const uint4*>(p));
  return v;
}
template <typename T> __device__ __forceinline__ void store16(T* p, const Vec16<T>& v) {
  *reinterpret_cast<uint4*>(p) = v.raw;
}
template <typename T> __device__ __forceinline__ void store16_stream(T* p, const Vec16<T>& v) {
  __stcs(reinterpret_cast<uint4*>(p), v.raw);
}

// ---- activations ------------------------------------------------------------------------------
// FAST = true selects hardware approximations (tanh.approx / __expf); used only where the
// storage type is bf16, whose rounding error dwarfs theirs.
template <bool FAST> __device__ __forceinline__ float tanh_sel(float x) {
  if constexpr (FAST) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  } else {
    return tanhf(x);
  }
}
template <bool FAST> __device__ __forceinline__ float sigmoid_sel(float x) {
  if constexpr (FAST) {
    return 0.5f * tanh_sel<true>(0.5f * x) + 0.5f;
  } else {
    return x >= 0.f ? 1.f / (1.f + expf(-x)) : (expf(x) / (1.f + expf(x)));
  }
}

constexpr float kGeluA = 0.044715f;
constexpr float kGeluL = 0.7978845608028654f;  // sqrt(2/pi)

template <int ACT, bool FAST> __device__ __forceinline__ float act_apply(float x) {
  if constexpr (ACT == LB2_ACT_IDENTITY) return x;
  if constexpr (ACT == LB2_ACT_RELU) return fmaxf(x, 0.f);
  if constexpr (ACT == LB2_ACT_GELU_TANH) {
    float inner = kGeluL * (x + kGeluA * x * x * x);
    return 0.5f * x * (1.f + tanh_sel<FAST>(inner));
  }
  if constexpr (ACT == LB2_ACT_GELU_ERF) return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
  if constexpr (ACT == LB2_ACT_TANH) return tanh_sel<FAST>(x);
  if constexpr (ACT == LB2_ACT_SIGMOID) return sigmoid_sel<FAST>(x);
  if constexpr (ACT == LB2_ACT_SWISH) return x * sigmoid_sel<FAST>(x);
  return x;
}

// derivative from the pre-activation x
template <int ACT, bool FAST> __device__ __forceinline__ float act_grad_pre(float x) {
  if constexpr (ACT == LB2_ACT_IDENTITY) return 1.f;
  if constexpr (ACT == LB2_ACT_RELU) return x > 0.f ? 1.f : 0.f;
  if constexpr (ACT == LB2_ACT_GELU_TANH) {
    float inner = kGeluL * (x + kGeluA * x * x * x);
    float t = tanh_sel<FAST>(inner);
    float dinner = kGeluL * (1.f + 3.f * kGeluA * x * x);
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * dinner;
  }
  if constexpr (ACT == LB2_ACT_GELU_ERF) {
    float cdf = 0.5f * (1.f + erff(x * 0.7071067811865476f));
    float pdf = expf(-0.5f * x * x) * 0.3989422804014327f;
    return cdf + x * pdf;
  }
  if constexpr (ACT == LB2_ACT_TANH) {
    float t = tanh_sel<FAST>(x);
    return 1.f - t * t;
  }
  if constexpr (ACT == LB2_ACT_SIGMOID) {
    float s = sigmoid_sel<FAST>(x);
    return s * (1.f - s);
  }
  if constexpr (ACT == LB2_ACT_SWISH) {
    float s = sigmoid_sel<FAST>(x);
    return s + x * s * (1.f - s);
  }
  return 1.f;
}

// derivative from the output (identity / relu / tanh / sigmoid only)
template <int ACT> __device__ __forceinline__ float act_grad_out(float o) {
  if constexpr (ACT == LB2_ACT_RELU) return o > 0.f ? 1.f : 0.f;
  if constexpr (ACT == LB2_ACT_TANH) return 1.f - o * o;
  if constexpr (ACT == LB2_ACT_SIGMOID) return o * (1.f - o);
  return 1.f;
}

// ACT >= 0: compile-time activation; ACT == -1: chosen at run time from `act_rt` (used by the
// normalisation kernels, where only identity and relu are worth a dedicated instantiation).
template <int ACT, bool FAST> __device__ __forceinline__ float act_apply_any(int act_rt, float x) {
  if constexpr (ACT >= 0) {
    return act_apply<ACT, FAST>(x);
  } else {
    switch (act_rt) {
      case LB2_ACT_RELU: return act_apply<LB2_ACT_RELU, FAST>(x);
      case LB2_ACT_GELU_TANH: return act_apply<LB2_ACT_GELU_TANH, FAST>(x);
      case LB2_ACT_GELU_ERF: return act_apply<LB2_ACT_GELU_ERF, FAST>(x);
      case LB2_ACT_TANH: return act_apply<LB2_ACT_TANH, FAST>(x);
      case LB2_ACT_SIGMOID: return act_apply<LB2_ACT_SIGMOID, FAST>(x);
      case LB2_ACT_SWISH: return act_apply<LB2_ACT_SWISH, FAST>(x);
      default: return x;
    }
  }
}
template <int ACT, bool FAST> __device__ __forceinline__ float act_grad_pre_any(int act_rt, float x) {
  if constexpr (ACT >= 0) {
    return act_grad_pre<ACT, FAST>(x);
  } else {
    switch (act_rt) {
      case LB2_ACT_RELU: return act_grad_pre<LB2_ACT_RELU, FAST>(x);
      case LB2_ACT_GELU_TANH: return act_grad_pre<LB2_ACT_GELU_TANH, FAST>(x);
      case LB2_ACT_GELU_ERF: return act_grad_pre<LB2_ACT_GELU_ERF, FAST>(x);
      case LB2_ACT_TANH: return act_grad_pre<LB2_ACT_TANH, FAST>(x);
      case LB2_ACT_SIGMOID: return act_grad_pre<LB2_ACT_SIGMOID, FAST>(x);
      case LB2_ACT_SWISH: return act_grad_pre<LB2_ACT_SWISH, FAST>(x);
      default: return 1.f;
    }
  }
}

#define LB2_DISPATCH_ACT3(act, ...)                                                      \
  switch (act) {                                                                         \
    case LB2_ACT_IDENTITY: { constexpr int ACT = LB2_ACT_IDENTITY; __VA_ARGS__; } break;  \
    case LB2_ACT_RELU: { constexpr int ACT = LB2_ACT_RELU; __VA_ARGS__; } break;          \
    default: { constexpr int ACT = -1; __VA_ARGS__; } break;                              \
  }

// Dispatch a runtime activation enum to a compile-time one.
#define LB2_DISPATCH_ACT(act, ...)                                                        \
  switch (act) {                                                                          \
    case LB2_ACT_IDENTITY: { constexpr int ACT = LB2_ACT_IDENTITY; __VA_ARGS__; } break;   \
    case LB2_ACT_RELU: { constexpr int ACT = LB2_ACT_RELU; __VA_ARGS__; } break;           \
    case LB2_ACT_GELU_TANH: { constexpr int ACT = LB2_ACT_GELU_TANH; __VA_ARGS__; } break; \
    case LB2_ACT_GELU_ERF: { constexpr int ACT = LB2_ACT_GELU_ERF; __VA_ARGS__; } break;   \
    case LB2_ACT_TANH: { constexpr int ACT = LB2_ACT_TANH; __VA_ARGS__; } break;           \
    case LB2_ACT_SIGMOID: { constexpr int ACT = LB2_ACT_SIGMOID; __VA_ARGS__; } break;     \
    default: { constexpr int ACT = LB2_ACT_SWISH; __VA_ARGS__; } break;                    \
  }

#define LB2_DISPATCH_DTYPE(dtype, ...)                               \
  if ((dtype) == LB2_F32) { using T = float; __VA_ARGS__; }          \
  else { using T = __nv_bfloat16; __VA_ARGS__; }

// ---- reductions ---------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide sum of `v`; result valid in every thread. `smem` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float* smem) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // protect smem reuse across consecutive calls
  if (lane == 0) smem[w] = v;
  __syncthreads();
  float t = (lane < nw) ? smem[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

}  // namespace lb2

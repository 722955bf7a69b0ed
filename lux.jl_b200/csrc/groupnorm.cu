// GroupNorm (and, with one channel per group, InstanceNorm), forward and backward: bandwidth-bound
// kernels that normalise contiguous rows = one (group, sample) block of S*C/G elements of the
// column-major (S, C/G, G, B) view.
//
// Forward: the row is read ONCE with 128-bit loads into registers (NV vectors per thread),
// two-pass variance over registers, 128-bit stores. Backward: a chunk-streaming kernel for rows of
// any length (producer warp + shared-memory ring; the second pass over a row is served by L2), with
// register-cached and scalar generic kernels for short or unaligned rows. The backward forms
// per-channel sums first (they are also the affine-gradient contributions of the sample) and
// derives the two group reductions from them; everything is reduced in a fixed order:
// deterministic. HBM traffic is the algorithmic figure: read x, write y; read x, dy, write dx.
//
// Algorithmic bytes per element: forward 2*sizeof(T), backward 3*sizeof(T).
#include <stdlib.h>

#include "norm_common.cuh"
#include "tc_ptx.cuh"

namespace lb2 {

// =============================================================================================
// GroupNorm: row = one (group, sample) block of L = S * Cg contiguous elements; channel of
// element i is g*Cg + i / S.
// =============================================================================================
template <typename T, int ACT, bool AFFINE, int NV, int BT>
__global__ void __launch_bounds__(BT) gn_fwd_cached_kernel(T* __restrict__ y, float* __restrict__ mean_out,
                                                           float* __restrict__ inv_out, const T* __restrict__ x,
                                                           const T* __restrict__ gamma, const T* __restrict__ beta,
                                                           int64_t S, int64_t Cg, int64_t G, int64_t rows, float eps, int act_rt) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = Vec16<T>::N;
  __shared__ float red[32];
  const int64_t L = S * Cg;
  const float invL = 1.f / (float)L;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int64_t g = row % G;
    const T* xr = x + row * L;
    Vec16<T> xv[NV];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * BT + threadIdx.x) * V;
      if (i < L) {
        xv[k] = load16_stream(xr + i);
#pragma unroll
        for (int j = 0; j < V; ++j) s += xv[k].get(j);
      }
    }
    const float mean = block_sum(s, red) * invL;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * BT + threadIdx.x) * V;
      if (i < L) {
#pragma unroll
        for (int j = 0; j < V; ++j) { float d = xv[k].get(j) - mean; q += d * d; }
      }
    }
    const float var = block_sum(q, red) * invL;
    const float inv = 1.f / sqrtf(var + eps);
    if (threadIdx.x == 0) { mean_out[row] = mean; inv_out[row] = inv; }
    T* yr = y + row * L;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * BT + threadIdx.x) * V;
      if (i < L) {
        float gp = inv, bp = -mean * inv;
        if constexpr (AFFINE) {  // S % V == 0: one channel per vector
          const int64_t c = g * Cg + i / S;
          gp = to_f32(gamma[c]) * inv;
          bp = to_f32(beta[c]) - mean * gp;
        }
        store16_stream(yr + i, vec_from<T>([&](int j) { return act_apply_any<ACT, FAST>(act_rt, fmaf(xv[k].get(j), gp, bp)); }));
      }
    }
  }
}

template <typename T, int ACT, bool AFFINE>
__global__ void __launch_bounds__(512) gn_fwd_generic_kernel(T* __restrict__ y, float* __restrict__ mean_out,
                                                             float* __restrict__ inv_out, const T* __restrict__ x,
                                                             const T* __restrict__ gamma, const T* __restrict__ beta,
                                                             int64_t S, int64_t Cg, int64_t G, int64_t rows, float eps, int act_rt) {
  constexpr bool FAST = sizeof(T) == 2;
  __shared__ float red[32];
  const int64_t L = S * Cg;
  const float invL = 1.f / (float)L;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int64_t g = row % G;
    const T* xr = x + row * L;
    float s = 0.f;
    for (int64_t i = threadIdx.x; i < L; i += blockDim.x) s += to_f32(xr[i]);
    const float mean = block_sum(s, red) * invL;
    float q = 0.f;
    for (int64_t i = threadIdx.x; i < L; i += blockDim.x) { float d = to_f32(xr[i]) - mean; q += d * d; }
    const float var = block_sum(q, red) * invL;
    const float inv = 1.f / sqrtf(var + eps);
    if (threadIdx.x == 0) { mean_out[row] = mean; inv_out[row] = inv; }
    T* yr = y + row * L;
    for (int64_t i = threadIdx.x; i < L; i += blockDim.x) {
      float gp = inv, bp = -mean * inv;
      if constexpr (AFFINE) {
        const int64_t c = g * Cg + i / S;
        gp = to_f32(gamma[c]) * inv;
        bp = to_f32(beta[c]) - mean * gp;
      }
      yr[i] = from_f32<T>(act_apply_any<ACT, FAST>(act_rt, fmaf(to_f32(xr[i]), gp, bp)));
    }
  }
}

// Backward. Per-channel sums ds[j] = sum_s d*xhat, db[j] = sum_s d (d = dy*act') are formed first
// (they are also the affine-gradient contributions of this sample), the two group reductions
// follow from them: sum g = sum_j gamma_j db[j], sum g*xhat = sum_j gamma_j ds[j].
// chan_out: [B][C][2] fp32 per-sample channel sums for the finishing kernel.
// Fast path needs S % (32*V) == 0 so that every warp-wide vector row lies in one channel.
template <typename T, int ACT, bool AFFINE, int NV, int BT>
__global__ void __launch_bounds__(BT) gn_bwd_cached_kernel(T* __restrict__ dx, float* __restrict__ chan_out,
                                                           const T* __restrict__ dy, const T* __restrict__ x,
                                                           const T* __restrict__ gamma, const T* __restrict__ beta,
                                                           const float* __restrict__ mean_in,
                                                           const float* __restrict__ inv_in, int64_t S, int64_t Cg,
                                                           int64_t G, int64_t rows, int act_rt) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = Vec16<T>::N;
  constexpr int NW = BT / 32;
  extern __shared__ float dyn[];            // ds[Cg], db[Cg]
  __shared__ float slots[2][NV][NW];
  __shared__ float red[32];
  float* ds = dyn;
  float* dbs = dyn + Cg;
  const int64_t L = S * Cg;
  const float invL = 1.f / (float)L;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t slots_per_chan = S / (32 * V);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int64_t g = row % G, n = row / G;
    const T* xr = x + row * L;
    const T* dyr = dy + row * L;
    const float mean = mean_in[row], inv = inv_in[row];
    Vec16<T> xv[NV];
    float dv[NV][V];
    __syncthreads();  // previous row's readers of ds/dbs/slots are done
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * BT + threadIdx.x) * V;
      float a = 0.f, b = 0.f;
      if (i < L) {
        xv[k] = load16_stream(xr + i);
        Vec16<T> gy = load16_stream(dyr + i);
        float gp = inv, bp = -mean * inv;
        if constexpr (AFFINE && ACT != LB2_ACT_IDENTITY) {
          const int64_t c = g * Cg + i / S;
          gp = to_f32(gamma[c]) * inv;
          bp = to_f32(beta[c]) - mean * gp;
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float d = gy.get(j);
          if constexpr (ACT != LB2_ACT_IDENTITY) d *= act_grad_pre_any<ACT, FAST>(act_rt, fmaf(xv[k].get(j), gp, bp));
          dv[k][j] = d;
          a += d * ((xv[k].get(j) - mean) * inv);
          b += d;
        }
      }
      a = warp_sum(a);
      b = warp_sum(b);
      if (lane == 0) { slots[0][k][warp] = a; slots[1][k][warp] = b; }
    }
    __syncthreads();
    // channel j owns slots_per_chan consecutive (k, warp) slots in element order
    for (int64_t j = threadIdx.x; j < Cg; j += BT) {
      float a = 0.f, b = 0.f;
      const int64_t first = j * slots_per_chan;
      for (int64_t q = 0; q < slots_per_chan; ++q) {
        const int64_t sl = first + q;  // global warp-row index = k*NW + warp
        a += slots[0][sl / NW][sl % NW];
        b += slots[1][sl / NW][sl % NW];
      }
      ds[j] = a;
      dbs[j] = b;
      if constexpr (AFFINE) {
        float* co = chan_out + ((n * (G * Cg)) + g * Cg + j) * 2;
        co[0] = a;
        co[1] = b;
      }
    }
    __syncthreads();
    float s1 = 0.f, s2 = 0.f;
    for (int64_t j = threadIdx.x; j < Cg; j += BT) {
      float gm = 1.f;
      if constexpr (AFFINE) gm = to_f32(gamma[g * Cg + j]);
      s1 += gm * dbs[j];
      s2 += gm * ds[j];
    }
    const float m1 = block_sum(s1, red) * invL;
    const float m2 = block_sum(s2, red) * invL;
    T* dxr = dx + row * L;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * BT + threadIdx.x) * V;
      if (i < L) {
        float gm = 1.f;
        if constexpr (AFFINE) gm = to_f32(gamma[g * Cg + i / S]);
        store16_stream(dxr + i, vec_from<T>([&](int j) {
          const float xh = (xv[k].get(j) - mean) * inv;
          return inv * (dv[k][j] * gm - m1 - xh * m2);
        }));
      }
    }
  }
}

// Generic backward: one warp per channel for the per-channel sums, scalar accesses.
template <typename T, int ACT, bool AFFINE>
__global__ void __launch_bounds__(512) gn_bwd_generic_kernel(T* __restrict__ dx, float* __restrict__ chan_out,
                                                             const T* __restrict__ dy, const T* __restrict__ x,
                                                             const T* __restrict__ gamma, const T* __restrict__ beta,
                                                             const float* __restrict__ mean_in,
                                                             const float* __restrict__ inv_in, int64_t S, int64_t Cg,
                                                             int64_t G, int64_t rows, int act_rt) {
  constexpr bool FAST = sizeof(T) == 2;
  extern __shared__ float dyn[];
  __shared__ float red[32];
  float* ds = dyn;
  float* dbs = dyn + Cg;
  const int64_t L = S * Cg;
  const float invL = 1.f / (float)L;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int64_t g = row % G, n = row / G;
    const T* xr = x + row * L;
    const T* dyr = dy + row * L;
    const float mean = mean_in[row], inv = inv_in[row];
    auto d_of = [&](int64_t i, int64_t c, float& xh) {
      const float xv = to_f32(xr[i]);
      xh = (xv - mean) * inv;
      float d = to_f32(dyr[i]);
      if constexpr (ACT != LB2_ACT_IDENTITY) {
        float gp = inv, bp = -mean * inv;
        if constexpr (AFFINE) { gp = to_f32(gamma[c]) * inv; bp = to_f32(beta[c]) - mean * gp; }
        d *= act_grad_pre_any<ACT, FAST>(act_rt, fmaf(xv, gp, bp));
      }
      return d;
    };
    __syncthreads();
    for (int64_t j = warp; j < Cg; j += nw) {
      float a = 0.f, b = 0.f;
      for (int64_t s = lane; s < S; s += 32) {
        float xh;
        const float d = d_of(j * S + s, g * Cg + j, xh);
        a += d * xh;
        b += d;
      }
      a = warp_sum(a);
      b = warp_sum(b);
      if (lane == 0) {
        ds[j] = a;
        dbs[j] = b;
        if constexpr (AFFINE) {
          float* co = chan_out + ((n * (G * Cg)) + g * Cg + j) * 2;
          co[0] = a;
          co[1] = b;
        }
      }
    }
    __syncthreads();
    float s1 = 0.f, s2 = 0.f;
    for (int64_t j = threadIdx.x; j < Cg; j += blockDim.x) {
      float gm = 1.f;
      if constexpr (AFFINE) gm = to_f32(gamma[g * Cg + j]);
      s1 += gm * dbs[j];
      s2 += gm * ds[j];
    }
    const float m1 = block_sum(s1, red) * invL;
    const float m2 = block_sum(s2, red) * invL;
    T* dxr = dx + row * L;
    for (int64_t i = threadIdx.x; i < L; i += blockDim.x) {
      const int64_t c = g * Cg + i / S;
      float xh;
      const float d = d_of(i, c, xh);
      float gm = 1.f;
      if constexpr (AFFINE) gm = to_f32(gamma[c]);
      dxr[i] = from_f32<T>(inv * (d * gm - m1 - xh * m2));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Streaming variants for rows of any length. A producer warp feeds fixed-size chunks of the row
// through a shared-memory ring with 1-D bulk copies, several chunks (and rows) ahead of the 256
// compute threads, once per pass over the row: the first pass comes from HBM, the repeats hit L2
// (a CTA's row is at most a few hundred KB old). The copies never stop while the compute threads
// sit in a reduction, and nothing is cached in registers, so two CTAs share an SM.
// Forward: three passes (sum, centred squares, apply) - the same two-pass variance as the cached
// kernel. Backward: two passes (per-channel sums, dx). Waits are time-bounded; a thread whose wait
// expired stops touching the ring and all threads leave together after the next reduction.
// ---------------------------------------------------------------------------------------------
constexpr int kGnCompute = 256;
constexpr int kGnThreads = kGnCompute + 32;
constexpr int kGnVecsPerChunk = 2;                              // 16-byte vectors per thread per chunk
constexpr uint32_t kGnChunkBytes = kGnCompute * 16 * kGnVecsPerChunk;  // 8 KB per tensor
constexpr int kGnHeaderBytes = 1024;

template <typename T, int ACT, bool AFFINE>
__global__ void __launch_bounds__(kGnThreads, 2)
gn_fwd_stream_kernel(T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ inv_out,
                     const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, uint32_t S,
                     uint32_t Cg, uint32_t G, int64_t rows, float eps, int act_rt, int stages, unsigned int* status) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = Vec16<T>::N;
  constexpr uint32_t CE = kGnChunkBytes / sizeof(T);  // elements per chunk
  extern __shared__ __align__(1024) uint8_t gn_smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(gn_smem);
  uint64_t* empty = full + stages;
  float* red = reinterpret_cast<float*>(gn_smem + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gn_smem + 768);
  uint8_t* data = gn_smem + kGnHeaderBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const uint32_t L = S * Cg;
  const uint32_t nchunks = (L + CE - 1) / CE;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kGnCompute / 32); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int64_t nrows = blockIdx.x < rows ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if (warp == kGnCompute / 32) {
    if (lane == 0) {
      uint32_t st = 0, ph = 0;
      for (int64_t r = 0; r < nrows; ++r) {
        const T* xr = x + (blockIdx.x + r * gridDim.x) * (int64_t)L;
        for (int pass = 0; pass < 3; ++pass) {
          for (uint32_t c = 0; c < nchunks; ++c) {
            if (!mbar_wait(&empty[st], ph ^ 1u, status, 0x2000000u)) return;
            const uint32_t left = (L - c * CE) * (uint32_t)sizeof(T);
            const uint32_t bytes = left < kGnChunkBytes ? left : kGnChunkBytes;
            mbar_expect_tx(&full[st], bytes);
            bulk_load_1d(smem_u32(data + (size_t)st * kGnChunkBytes), xr + (size_t)c * CE, bytes, &full[st]);
            if (++st == (uint32_t)stages) { st = 0; ph ^= 1u; }
          }
        }
      }
    }
    return;
  }
  const float invL = 1.f / (float)L;
  uint32_t st = 0, ph = 0;
  bool dead = false;
  // one pass over the row's chunks; body(vector, element offset in row)
  auto sweep = [&](auto&& body) {
    for (uint32_t c = 0; c < nchunks; ++c) {
      if (!dead && !mbar_wait_warp(&full[st], ph, status, 0x4000000u)) { dead = true; *abort_flag = 1; }
      if (!dead) {
        const T* sx = reinterpret_cast<const T*>(data + (size_t)st * kGnChunkBytes);
#pragma unroll
        for (int k = 0; k < kGnVecsPerChunk; ++k) {
          const uint32_t off = (uint32_t)(k * kGnCompute + t) * V;
          const uint32_t i = c * CE + off;
          if (i < L) body(load16(sx + off), i);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
      }
      if (++st == (uint32_t)stages) { st = 0; ph ^= 1u; }
    }
  };
  for (int64_t r = 0; r < nrows; ++r) {
    const int64_t row = blockIdx.x + r * gridDim.x;
    const uint32_t g = (uint32_t)(row % G);
    float s = 0.f;
    sweep([&](const Vec16<T>& v, uint32_t) {
#pragma unroll
      for (int j = 0; j < V; ++j) s += v.get(j);
    });
    const float mean = group_sum(s, red, kGnCompute) * invL;
    if (*abort_flag) { drain_after_abort(); break; }
    float q = 0.f;
    sweep([&](const Vec16<T>& v, uint32_t) {
#pragma unroll
      for (int j = 0; j < V; ++j) { const float d = v.get(j) - mean; q = fmaf(d, d, q); }
    });
    const float var = group_sum(q, red, kGnCompute) * invL;
    if (*abort_flag) { drain_after_abort(); break; }
    const float inv = 1.f / sqrtf(var + eps);
    if (t == 0) { mean_out[row] = mean; inv_out[row] = inv; }
    T* yr = y + row * (int64_t)L;
    sweep([&](const Vec16<T>& v, uint32_t i) {
      float gp = inv, bp = -mean * inv;
      if constexpr (AFFINE) {  // S % V == 0: one channel per vector
        const uint32_t c = g * Cg + i / S;
        gp = to_f32(gamma[c]) * inv;
        bp = to_f32(beta[c]) - mean * gp;
      }
      store16_stream(yr + i, vec_from<T>([&](int j) { return act_apply_any<ACT, FAST>(act_rt, fmaf(v.get(j), gp, bp)); }));
    });
  }
}

// Backward; shared memory after the header: ds[Cg], db[Cg], slots[nslots][8] pairs (every warp-wide
// vector row of the group, in element order, leaves eight quarter-warp partial sums: two shuffle steps
// per row instead of ten), then the ring (x chunk + dy chunk per stage).
template <typename T, int ACT, bool AFFINE>
__global__ void __launch_bounds__(kGnThreads, 2)
gn_bwd_stream_kernel(T* __restrict__ dx, float* __restrict__ chan_out, const T* __restrict__ dy,
                     const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                     const float* __restrict__ mean_in, const float* __restrict__ inv_in, uint32_t S, uint32_t Cg,
                     uint32_t G, int64_t rows, int act_rt, int stages, uint32_t aux_bytes, unsigned int* status, int resident) {
  // resident: the ring has exactly one stage per chunk of a row (stages == nchunks), so the row stays in shared memory
  // from the first pass to the second: it is fetched once, the second pass waits for nothing, and a stage is released
  // (to the next row's copy) only after its second use.
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = Vec16<T>::N;
  constexpr uint32_t CE = kGnChunkBytes / sizeof(T);
  constexpr uint32_t kSlotsPerChunk = kGnVecsPerChunk * (kGnCompute / 32);
  extern __shared__ __align__(1024) uint8_t gn_smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(gn_smem);
  uint64_t* empty = full + stages;
  float* red = reinterpret_cast<float*>(gn_smem + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gn_smem + 768);
  const uint32_t L = S * Cg;
  const uint32_t nslots = L / (32 * V);
  float* ds = reinterpret_cast<float*>(gn_smem + kGnHeaderBytes);
  float* dbs = ds + Cg;
  float2* slots = reinterpret_cast<float2*>(dbs + Cg);   // ds + 2*Cg floats: 8-byte aligned
  uint8_t* data = gn_smem + kGnHeaderBytes + aux_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const uint32_t nchunks = (L + CE - 1) / CE;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kGnCompute / 32); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int64_t nrows = blockIdx.x < rows ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if (warp == kGnCompute / 32) {
    if (lane == 0) {
      uint32_t st = 0, ph = 0;
      for (int64_t r = 0; r < nrows; ++r) {
        const int64_t base = (blockIdx.x + r * gridDim.x) * (int64_t)L;
        for (int pass = 0; pass < (resident ? 1 : 2); ++pass) {
          for (uint32_t c = 0; c < nchunks; ++c) {
            if (!mbar_wait(&empty[st], ph ^ 1u, status, 0x8000000u)) return;
            const uint32_t left = (L - c * CE) * (uint32_t)sizeof(T);
            const uint32_t bytes = left < kGnChunkBytes ? left : kGnChunkBytes;
            uint8_t* dst = data + (size_t)st * 2 * kGnChunkBytes;
            mbar_expect_tx(&full[st], 2 * bytes);
            bulk_load_1d(smem_u32(dst), x + base + (size_t)c * CE, bytes, &full[st]);
            bulk_load_1d(smem_u32(dst + kGnChunkBytes), dy + base + (size_t)c * CE, bytes, &full[st]);
            if (++st == (uint32_t)stages) { st = 0; ph ^= 1u; }
          }
        }
      }
    }
    return;
  }
  const float invL = 1.f / (float)L;
  const uint32_t slots_per_chan = S / (32 * V);
  uint32_t st = 0, ph = 0;
  bool dead = false;
  for (int64_t r = 0; r < nrows; ++r) {
    const int64_t row = blockIdx.x + r * gridDim.x;
    const uint32_t g = (uint32_t)(row % G);
    const int64_t n = row / G;
    const float mean = mean_in[row], inv = inv_in[row];
    // d = dy * act'(pre) for one vector; xh = normalised input
    auto d_of = [&](const Vec16<T>& xv, const Vec16<T>& gy, uint32_t i, int j) {
      float d = gy.get(j);
      if constexpr (ACT != LB2_ACT_IDENTITY) {
        float gp = inv, bp = -mean * inv;
        if constexpr (AFFINE) {
          const uint32_t c = g * Cg + i / S;
          gp = to_f32(gamma[c]) * inv;
          bp = to_f32(beta[c]) - mean * gp;
        }
        d *= act_grad_pre_any<ACT, FAST>(act_rt, fmaf(xv.get(j), gp, bp));
      }
      return d;
    };
    // pass 1: one (sum d*xh, sum d) pair per warp-wide vector row
    for (uint32_t c = 0; c < nchunks; ++c) {
      if (!dead && !mbar_wait_warp(&full[st], ph, status, 0x10000000u)) { dead = true; *abort_flag = 1; }
      const T* sx = reinterpret_cast<const T*>(data + (size_t)st * 2 * kGnChunkBytes);
      const T* sdy = reinterpret_cast<const T*>(data + (size_t)st * 2 * kGnChunkBytes + kGnChunkBytes);
#pragma unroll
      for (int k = 0; k < kGnVecsPerChunk; ++k) {
        const uint32_t off = (uint32_t)(k * kGnCompute + t) * V;
        const uint32_t i = c * CE + off;
        float a = 0.f, b = 0.f;
        if (!dead && i < L) {
          const Vec16<T> xv = load16(sx + off), gy = load16(sdy + off);
#pragma unroll
          for (int j = 0; j < V; ++j) {
            const float d = d_of(xv, gy, i, j);
            a = fmaf(d, (xv.get(j) - mean) * inv, a);
            b += d;
          }
        }
        a += __shfl_xor_sync(0xffffffffu, a, 16);
        b += __shfl_xor_sync(0xffffffffu, b, 16);
        a += __shfl_xor_sync(0xffffffffu, a, 8);
        b += __shfl_xor_sync(0xffffffffu, b, 8);
        const uint32_t sl = c * kSlotsPerChunk + (uint32_t)(k * (kGnCompute / 32) + warp);
        if (lane < 8 && sl < nslots) slots[sl * 8 + lane] = make_float2(a, b);
      }
      if (!dead && !resident) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
      }
      if (++st == (uint32_t)stages) { st = 0; ph ^= 1u; }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kGnCompute) : "memory");
    // channel j owns slots_per_chan consecutive rows = a contiguous run of 8 * slots_per_chan pairs;
    // one warp per channel, lanes stride through the run, then a butterfly (fixed order: deterministic)
    for (uint32_t j = warp; j < Cg; j += kGnCompute / 32) {
      float a = 0.f, b = 0.f;
      const float2* run = slots + (size_t)j * slots_per_chan * 8;
      for (uint32_t q = lane; q < slots_per_chan * 8; q += 32) { a += run[q].x; b += run[q].y; }
      a = warp_sum(a);
      b = warp_sum(b);
      if (lane == 0) {
        ds[j] = a;
        dbs[j] = b;
        if constexpr (AFFINE) {
          float* co = chan_out + ((n * ((int64_t)G * Cg)) + (int64_t)g * Cg + j) * 2;
          co[0] = a;
          co[1] = b;
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kGnCompute) : "memory");
    float s1 = 0.f, s2 = 0.f;
    for (uint32_t j = t; j < Cg; j += kGnCompute) {
      float gm = 1.f;
      if constexpr (AFFINE) gm = to_f32(gamma[g * Cg + j]);
      s1 = fmaf(gm, dbs[j], s1);
      s2 = fmaf(gm, ds[j], s2);
    }
    const float2 m12 = group_sum2(s1, s2, red, kGnCompute);
    if (*abort_flag) { drain_after_abort(); break; }
    const float m1 = m12.x * invL, m2 = m12.y * invL;
    T* dxr = dx + row * (int64_t)L;
    // pass 2: dx = inv * (d*gamma - m1 - xh*m2)
    for (uint32_t c = 0; c < nchunks; ++c) {
      const uint32_t sc = resident ? c : st;      // resident: chunk c sits in stage c since the first pass
      if (!resident && !dead && !mbar_wait_warp(&full[st], ph, status, 0x20000000u)) { dead = true; *abort_flag = 1; }
      if (!dead) {
        const T* sx = reinterpret_cast<const T*>(data + (size_t)sc * 2 * kGnChunkBytes);
        const T* sdy = reinterpret_cast<const T*>(data + (size_t)sc * 2 * kGnChunkBytes + kGnChunkBytes);
#pragma unroll
        for (int k = 0; k < kGnVecsPerChunk; ++k) {
          const uint32_t off = (uint32_t)(k * kGnCompute + t) * V;
          const uint32_t i = c * CE + off;
          if (i < L) {
            const Vec16<T> xv = load16(sx + off), gy = load16(sdy + off);
            float gm = 1.f;
            if constexpr (AFFINE) gm = to_f32(gamma[g * Cg + i / S]);
            store16_stream(dxr + i, vec_from<T>([&](int j) {
              const float xh = (xv.get(j) - mean) * inv;
              return inv * (d_of(xv, gy, i, j) * gm - m1 - xh * m2);
            }));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[sc]);
      }
      if (!resident && ++st == (uint32_t)stages) { st = 0; ph ^= 1u; }
    }
  }
}

// Which directions may take the chunk-streaming kernels: bit 0 = forward, bit 1 = backward. The cached forward is
// faster wherever it applies, so only the backward streams.
static constexpr int gn_stream_mask() { return 2; }

// dgamma[c] = sum_n chan[n][c][0], dbeta[c] = sum_n chan[n][c][1]. block (32 channels, 32 slices): slice y adds
// samples y, y+32, ... in ascending order, then the slice sums are added in slice order: a fixed order, deterministic,
// and a chain of B/32 loads per thread instead of B.
constexpr int kGnFinishSlices = 32;
template <typename T>
__global__ void __launch_bounds__(32 * kGnFinishSlices) gn_finish_kernel(T* __restrict__ dgamma, T* __restrict__ dbeta,
                                                                        const float* __restrict__ chan, int64_t C, int64_t B) {
  __shared__ float sg[kGnFinishSlices][33], sb[kGnFinishSlices][33];
  const int64_t c = (int64_t)blockIdx.x * 32 + threadIdx.x;
  float ag = 0.f, ab = 0.f;
  if (c < C) {
#pragma unroll 4
    for (int64_t n = threadIdx.y; n < B; n += kGnFinishSlices) {
      const float2 v = __ldcs(reinterpret_cast<const float2*>(chan) + n * C + c);
      ag += v.x;
      ab += v.y;
    }
  }
  sg[threadIdx.y][threadIdx.x] = ag;
  sb[threadIdx.y][threadIdx.x] = ab;
  __syncthreads();
  if (threadIdx.y == 0 && c < C) {
    float tg = 0.f, tb = 0.f;
#pragma unroll
    for (int r = 0; r < kGnFinishSlices; ++r) { tg += sg[r][threadIdx.x]; tb += sb[r][threadIdx.x]; }
    dgamma[c] = from_f32<T>(tg);
    dbeta[c] = from_f32<T>(tb);
  }
}

template <typename T, int ACT, bool AFFINE>
static int32_t gn_fwd_launch(T* y, float* sm, float* si, const T* x, const T* g, const T* b, int64_t S, int64_t C,
                             int64_t G, int64_t B, float eps, int32_t act, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  const int64_t Cg = C / G, L = S * Cg, rows = G * B;
  const bool al = aligned_to(y, 16) && aligned_to(x, 16) && (S % V == 0);
  const int sms = sm_count();
  const int64_t vecs = L / V;
  int grid = (int)(rows < (int64_t)sms * 4 ? rows : (int64_t)sms * 4);
  const bool fits32 = L < (int64_t)1 << 31 && G < (int64_t)1 << 31;
  if ((gn_stream_mask() & 1) && al && fits32 && L * (int64_t)sizeof(T) >= 2 * (int64_t)kGnChunkBytes) {
    unsigned int* status = device_status_word();
    LB2_REQUIRE(status != nullptr, LB2_LAUNCH_FAIL, "groupnorm: device status word unavailable");
    const int stages = 12;
    const int smem = kGnHeaderBytes + stages * (int)kGnChunkBytes;
    cudaError_t e = cudaFuncSetAttribute(gn_fwd_stream_kernel<T, ACT, AFFINE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    LB2_REQUIRE(e == cudaSuccess, LB2_LAUNCH_FAIL, "groupnorm: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    grid = (int)(rows < (int64_t)sms * 2 ? rows : (int64_t)sms * 2);
    gn_fwd_stream_kernel<T, ACT, AFFINE><<<grid, kGnThreads, smem, st>>>(y, sm, si, x, g, b, (uint32_t)S, (uint32_t)Cg, (uint32_t)G, rows, eps, act, stages, status);
  } else if (al && vecs <= 256 * 8) {
    const int nv = vecs <= 256 ? 1 : (vecs <= 512 ? 2 : (vecs <= 1024 ? 4 : 8));
    if (nv == 1) gn_fwd_cached_kernel<T, ACT, AFFINE, 1, 256><<<grid, 256, 0, st>>>(y, sm, si, x, g, b, S, Cg, G, rows, eps, act);
    else if (nv == 2) gn_fwd_cached_kernel<T, ACT, AFFINE, 2, 256><<<grid, 256, 0, st>>>(y, sm, si, x, g, b, S, Cg, G, rows, eps, act);
    else if (nv == 4) gn_fwd_cached_kernel<T, ACT, AFFINE, 4, 256><<<grid, 256, 0, st>>>(y, sm, si, x, g, b, S, Cg, G, rows, eps, act);
    else gn_fwd_cached_kernel<T, ACT, AFFINE, 8, 256><<<grid, 256, 0, st>>>(y, sm, si, x, g, b, S, Cg, G, rows, eps, act);
  } else if (al && vecs <= 512 * 8) {
    grid = (int)(rows < (int64_t)sms * 2 ? rows : (int64_t)sms * 2);
    gn_fwd_cached_kernel<T, ACT, AFFINE, 8, 512><<<grid, 512, 0, st>>>(y, sm, si, x, g, b, S, Cg, G, rows, eps, act);
  } else if (al && vecs <= 1024 * 8) {
    grid = (int)(rows < (int64_t)sms ? rows : (int64_t)sms);
    gn_fwd_cached_kernel<T, ACT, AFFINE, 8, 1024><<<grid, 1024, 0, st>>>(y, sm, si, x, g, b, S, Cg, G, rows, eps, act);
  } else {
    gn_fwd_generic_kernel<T, ACT, AFFINE><<<grid, 512, 0, st>>>(y, sm, si, x, g, b, S, Cg, G, rows, eps, act);
  }
  LB2_CHECK_LAUNCH("groupnorm_fwd");
  return LB2_OK;
}

template <typename T, int ACT, bool AFFINE>
static int32_t gn_bwd_launch(T* dx, T* dg, T* db, const T* dy, const T* x, const T* g, const T* b, const float* sm,
                             const float* si, int64_t S, int64_t C, int64_t G, int64_t B, float* ws, int32_t act, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  const int64_t Cg = C / G, L = S * Cg, rows = G * B;
  const size_t dyn = (size_t)Cg * 2 * sizeof(float);
  LB2_REQUIRE(dyn <= 40 * 1024, LB2_BAD_SHAPE, "groupnorm backward supports at most 5120 channels per group");
  const bool al = aligned_to(dx, 16) && aligned_to(dy, 16) && aligned_to(x, 16) && (S % (32 * V) == 0);
  const int sms = sm_count();
  const int64_t vecs = L / V;
  int grid = (int)(rows < (int64_t)sms * 2 ? rows : (int64_t)sms * 2);
  const bool fits32 = L < (int64_t)1 << 31 && G < (int64_t)1 << 31;
  const size_t aux = align_up((size_t)(2 * Cg + 2 + 16 * (L / (32 * V))) * sizeof(float), 128);
  if ((gn_stream_mask() & 2) && al && fits32 && aux <= 64 * 1024 && L * (int64_t)sizeof(T) >= 2 * (int64_t)kGnChunkBytes) {
    unsigned int* status = device_status_word();
    LB2_REQUIRE(status != nullptr, LB2_LAUNCH_FAIL, "groupnorm: device status word unavailable");
    // rows of at most four chunks per operand (64 KB of x and dy together) stay resident between the passes
    const int64_t nchunks = (L * (int64_t)sizeof(T) + kGnChunkBytes - 1) / kGnChunkBytes;
    const int resident = nchunks <= 4 ? 1 : 0;
    const int stages = resident ? (int)nchunks : 6;
    const int smem = kGnHeaderBytes + (int)aux + stages * 2 * (int)kGnChunkBytes;
    cudaError_t e = cudaFuncSetAttribute(gn_bwd_stream_kernel<T, ACT, AFFINE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    LB2_REQUIRE(e == cudaSuccess, LB2_LAUNCH_FAIL, "groupnorm: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    const int per_sm = smem <= 112 * 1024 ? 2 : 1;
    grid = (int)(rows < (int64_t)sms * per_sm ? rows : (int64_t)sms * per_sm);
    gn_bwd_stream_kernel<T, ACT, AFFINE><<<grid, kGnThreads, smem, st>>>(dx, ws, dy, x, g, b, sm, si, (uint32_t)S, (uint32_t)Cg, (uint32_t)G, rows, act, stages, (uint32_t)aux, status, resident);
  } else if (al && vecs <= 512 * 4) {
    const int nv = vecs <= 512 ? 1 : (vecs <= 1024 ? 2 : 4);
    if (nv == 1) gn_bwd_cached_kernel<T, ACT, AFFINE, 1, 512><<<grid, 512, dyn, st>>>(dx, ws, dy, x, g, b, sm, si, S, Cg, G, rows, act);
    else if (nv == 2) gn_bwd_cached_kernel<T, ACT, AFFINE, 2, 512><<<grid, 512, dyn, st>>>(dx, ws, dy, x, g, b, sm, si, S, Cg, G, rows, act);
    else gn_bwd_cached_kernel<T, ACT, AFFINE, 4, 512><<<grid, 512, dyn, st>>>(dx, ws, dy, x, g, b, sm, si, S, Cg, G, rows, act);
  } else if (al && vecs <= 1024 * 4) {
    grid = (int)(rows < (int64_t)sms ? rows : (int64_t)sms);
    gn_bwd_cached_kernel<T, ACT, AFFINE, 4, 1024><<<grid, 1024, dyn, st>>>(dx, ws, dy, x, g, b, sm, si, S, Cg, G, rows, act);
  } else {
    gn_bwd_generic_kernel<T, ACT, AFFINE><<<grid, 512, dyn, st>>>(dx, ws, dy, x, g, b, sm, si, S, Cg, G, rows, act);
  }
  LB2_CHECK_LAUNCH("groupnorm_bwd");
  if constexpr (AFFINE) {
    gn_finish_kernel<T><<<(unsigned)((C + 31) / 32), dim3(32, kGnFinishSlices), 0, st>>>(dg, db, ws, C, B);
    LB2_CHECK_LAUNCH("groupnorm_bwd_finish");
  }
  return LB2_OK;
}

// InstanceNorm running statistics: one thread per channel walks the batch in order (deterministic).
template <typename T>
__global__ void in_update_stats_kernel(T* __restrict__ new_rmean, T* __restrict__ new_rvar, const T* __restrict__ rmean,
                                       const T* __restrict__ rvar, const float* __restrict__ save_mean,
                                       const float* __restrict__ save_inv, int64_t S, int64_t C, int64_t B,
                                       float momentum, float eps) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float sm = 0.f, sv = 0.f;
  for (int64_t b = 0; b < B; ++b) {
    const float inv = save_inv[b * C + c];
    sm += save_mean[b * C + c];
    sv += 1.f / (inv * inv) - eps;
  }
  const float mu = sm / (float)B, var = sv / (float)B;
  const float m = (float)S;
  const float m1 = momentum, m2 = momentum * m / (m - 1.f), m3 = 1.f - m1;
  new_rmean[c] = from_f32<T>(m3 * to_f32(rmean[c]) + m1 * mu);
  new_rvar[c] = from_f32<T>(m3 * to_f32(rvar[c]) + m2 * var);
}

}  // namespace lb2

using namespace lb2;

extern "C" {

int32_t lb2_groupnorm_fwd(void* y, float* save_mean, float* save_invstd, const void* x, const void* gamma,
                          const void* beta, int64_t S, int64_t C, int64_t G, int64_t B, double eps, int32_t dtype,
                          int32_t act, void* stream) {
  LB2_REQUIRE(S >= 0 && C >= 0 && B >= 0 && G >= 1, LB2_BAD_SHAPE, "bad extent");
  LB2_REQUIRE(C % G == 0, LB2_BAD_SHAPE, "number of channels (%lld) must be divisible by groups (%lld)", (long long)C, (long long)G);
  if (S == 0 || C == 0 || B == 0) return LB2_OK;
  int32_t rc = check_norm_common(y, x, gamma, beta, save_mean, save_invstd, dtype, act);
  if (rc != LB2_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LB2_DISPATCH_DTYPE(dtype, {
    LB2_DISPATCH_ACT3(act, {
      if (gamma) return gn_fwd_launch<T, ACT, true>((T*)y, save_mean, save_invstd, (const T*)x, (const T*)gamma, (const T*)beta, S, C, G, B, (float)eps, act, st);
      else return gn_fwd_launch<T, ACT, false>((T*)y, save_mean, save_invstd, (const T*)x, nullptr, nullptr, S, C, G, B, (float)eps, act, st);
    });
  });
  return LB2_OK;
}

int32_t lb2_instancenorm_update_stats(void* new_rmean, void* new_rvar, const void* rmean, const void* rvar,
                                      const float* save_mean, const float* save_invstd, int64_t S, int64_t C, int64_t B,
                                      double momentum, double eps, int32_t dtype, void* stream) {
  LB2_REQUIRE(S >= 0 && C >= 0 && B >= 0, LB2_BAD_SHAPE, "bad extent");
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  if (C == 0) return LB2_OK;
  LB2_REQUIRE(new_rmean && new_rvar && rmean && rvar, LB2_BAD_ARG, "null running-statistics pointer");
  LB2_REQUIRE(B > 0 && S > 0, LB2_BAD_SHAPE, "running statistics need a non-empty batch");
  LB2_REQUIRE(save_mean && save_invstd, LB2_BAD_ARG, "saved statistics are null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LB2_DISPATCH_DTYPE(dtype, {
    in_update_stats_kernel<T><<<(unsigned)((C + 127) / 128), 128, 0, st>>>((T*)new_rmean, (T*)new_rvar, (const T*)rmean,
                                                                          (const T*)rvar, save_mean, save_invstd, S, C, B,
                                                                          (float)momentum, (float)eps);
  });
  LB2_CHECK_LAUNCH("instancenorm_update_stats");
  return LB2_OK;
}

size_t lb2_groupnorm_bwd_workspace_bytes(int64_t S, int64_t C, int64_t G, int64_t B) {
  (void)S; (void)G;
  if (C <= 0 || B <= 0) return 0;
  return align_up((size_t)C * (size_t)B * 2 * sizeof(float), 256);
}

int32_t lb2_groupnorm_bwd(void* dx, void* dgamma, void* dbeta, const void* dy, const void* x, const void* gamma,
                          const void* beta, const float* save_mean, const float* save_invstd, int64_t S, int64_t C,
                          int64_t G, int64_t B, int32_t dtype, int32_t act, void* workspace, size_t workspace_bytes,
                          void* stream) {
  LB2_REQUIRE(S >= 0 && C >= 0 && B >= 0 && G >= 1, LB2_BAD_SHAPE, "bad extent");
  LB2_REQUIRE(C % G == 0, LB2_BAD_SHAPE, "number of channels (%lld) must be divisible by groups (%lld)", (long long)C, (long long)G);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (S == 0 || C == 0 || B == 0) {
    if (C > 0 && dgamma && valid_dtype(dtype)) {
      cudaMemsetAsync(dgamma, 0, (size_t)C * dtype_size(dtype), st);
      cudaMemsetAsync(dbeta, 0, (size_t)C * dtype_size(dtype), st);
    }
    return LB2_OK;
  }
  int32_t rc = check_norm_common(dx, x, gamma, beta, save_mean, save_invstd, dtype, act);
  if (rc != LB2_OK) return rc;
  LB2_REQUIRE(dy != nullptr, LB2_BAD_ARG, "dy is null");
  LB2_REQUIRE(!gamma || (dgamma && dbeta), LB2_BAD_ARG, "dgamma/dbeta required when scale is given");
  if (gamma) {
    LB2_REQUIRE(workspace && workspace_bytes >= lb2_groupnorm_bwd_workspace_bytes(S, C, G, B), LB2_WORKSPACE_TOO_SMALL,
                "workspace of %zu bytes needed", lb2_groupnorm_bwd_workspace_bytes(S, C, G, B));
    LB2_REQUIRE(aligned_to(workspace, 16), LB2_BAD_ALIGN, "workspace must be 16-byte aligned");
  }
  LB2_DISPATCH_DTYPE(dtype, {
    LB2_DISPATCH_ACT3(act, {
      if (gamma) return gn_bwd_launch<T, ACT, true>((T*)dx, (T*)dgamma, (T*)dbeta, (const T*)dy, (const T*)x, (const T*)gamma, (const T*)beta, save_mean, save_invstd, S, C, G, B, (float*)workspace, act, st);
      else return gn_bwd_launch<T, ACT, false>((T*)dx, nullptr, nullptr, (const T*)dy, (const T*)x, nullptr, nullptr, save_mean, save_invstd, S, C, G, B, (float*)workspace, act, st);
    });
  });
  return LB2_OK;
}

}  // extern "C"

// LayerNorm, forward and backward: bandwidth-bound kernels that normalise contiguous rows of D
// features (Julia column-major, so the normalised extent is contiguous).
//
// Three tiers. Ring kernels (the common case, rows of a few KB to ~100 KB): a producer warp streams
// whole rows into a shared-memory ring with 1-D bulk copies several rows ahead of 256 compute
// threads; the forward takes a two-pass (mean, then centred sum of squares) variance over
// registers, the backward keeps the row in its ring stage through both of its passes. Cached
// kernels (short rows): the row is read ONCE with 128-bit loads into registers. Generic kernels:
// scalar, multi-pass (second and third reads served by L2) for shapes the others cannot take.
// The backward fuses both of its reductions (sum g, sum g*xhat) in one pass and accumulates the
// affine gradients per thread across rows; all cross-CTA reductions are two-stage in a fixed
// order: deterministic. HBM traffic is the algorithmic figure: read x, write y; read x, dy, write dx.
//
// Algorithmic bytes per element: forward 2*sizeof(T), backward 3*sizeof(T).
#include "norm_common.cuh"
#include "tc_ptx.cuh"

namespace lb2 {

// =============================================================================================
// LayerNorm
// =============================================================================================
// RT = threads per row (32: one warp per row, 8 rows per CTA; 256/512: one CTA per row).
template <typename T, int ACT, bool AFFINE, int RT, int NV, int BT>
__global__ void __launch_bounds__(BT) ln_fwd_cached_kernel(T* __restrict__ y, float* __restrict__ mean_out,
                                                           float* __restrict__ inv_out, const T* __restrict__ x,
                                                           const T* __restrict__ gamma, const T* __restrict__ beta,
                                                           int64_t D, int64_t R, float eps, int act_rt) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = Vec16<T>::N;
  constexpr int ROWS = BT / RT;
  __shared__ float red[32];
  const int t = threadIdx.x % RT, slot = threadIdx.x / RT;
  Vec16<T> gv[NV], bv[NV];
  if constexpr (AFFINE) {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * RT + t) * V;
      if (i < D) { gv[k] = load16(gamma + i); bv[k] = load16(beta + i); }
    }
  }
  const float invD = 1.f / (float)D;
  for (int64_t row = (int64_t)blockIdx.x * ROWS + slot; row < R; row += (int64_t)gridDim.x * ROWS) {
    const T* xr = x + row * D;
    Vec16<T> xv[NV];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * RT + t) * V;
      if (i < D) {
        xv[k] = load16_stream(xr + i);
#pragma unroll
        for (int j = 0; j < V; ++j) s += xv[k].get(j);
      }
    }
    const float mean = row_sum<RT>(s, red) * invD;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * RT + t) * V;
      if (i < D) {
#pragma unroll
        for (int j = 0; j < V; ++j) { float d = xv[k].get(j) - mean; q += d * d; }
      }
    }
    const float var = row_sum<RT>(q, red) * invD;
    const float inv = 1.f / sqrtf(var + eps);
    if (t == 0) { mean_out[row] = mean; inv_out[row] = inv; }
    T* yr = y + row * D;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * RT + t) * V;
      if (i < D) {
        store16_stream(yr + i, vec_from<T>([&](int j) {
          float gp = inv, bp = -mean * inv;
          if constexpr (AFFINE) { gp = gv[k].get(j) * inv; bp = bv[k].get(j) - mean * gp; }
          return act_apply_any<ACT, FAST>(act_rt, fmaf(xv[k].get(j), gp, bp));
        }));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Warp-per-row forward for 2-byte elements: a lane keeps NV 16-byte vectors of the row PACKED in registers (a row of
// 4096 bf16 is 16 vectors = 64 registers per lane), so both passes read registers, the only reduction is a warp
// butterfly (no block barrier, no shared-memory ring, no spin on an mbarrier) and the warps of an SM are in different
// phases of their rows at any time, which is what keeps loads in flight. Scale and shift are staged in shared memory
// once per CTA and read per use. Statistics in one pass over d = x - K, K = the row's first element.
// ---------------------------------------------------------------------------------------------
template <typename T, int ACT, bool AFFINE, int NV>
__global__ void __launch_bounds__(256, 2) ln_fwd_warp_kernel(T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ inv_out,
                                                             const T* __restrict__ x, const T* __restrict__ gamma,
                                                             const T* __restrict__ beta, int64_t D, int64_t R, float eps, int act_rt) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = Vec16<T>::N;
  extern __shared__ __align__(16) uint8_t ln_warp_smem[];
  T* sg = reinterpret_cast<T*>(ln_warp_smem);
  T* sb = sg + D;
  if constexpr (AFFINE) {
    for (int64_t i = (int64_t)threadIdx.x * V; i < D; i += (int64_t)blockDim.x * V) {
      store16(sg + i, load16(gamma + i));
      store16(sb + i, load16(beta + i));
    }
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const float invD = 1.f / (float)D;
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < R; row += warps) {
    const T* xr = x + row * D;
    Vec16<T> xv[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * 32 + lane) * V;
      if (i < D) xv[k] = load16_stream(xr + i);
    }
    const float K0 = __shfl_sync(0xffffffffu, xv[0].get(0), 0);
    float s = 0.f, q = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      if (((int64_t)k * 32 + lane) * V < D) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float d = xv[k].get(j) - K0;
          s += d;
          q = fmaf(d, d, q);
        }
      }
    }
    s = warp_sum(s);
    q = warp_sum(q);
    const float dm = s * invD;                                   // mean - K
    const float var = fmaxf(fmaf(-dm, dm, q * invD), 0.f);
    const float inv = 1.f / sqrtf(var + eps);
    const float nmi = -dm * inv;
    if (lane == 0) { mean_out[row] = K0 + dm; inv_out[row] = inv; }
    T* yr = y + row * D;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * 32 + lane) * V;
      if (i < D) {
        Vec16<T> gv, bv;
        if constexpr (AFFINE) { gv = load16(sg + i); bv = load16(sb + i); }
        store16_stream(yr + i, vec_from<T>([&](int j) {
          float v = fmaf(xv[k].get(j) - K0, inv, nmi);             // (x - mean) * inv
          if constexpr (AFFINE) v = fmaf(v, gv.get(j), bv.get(j));
          return act_apply_any<ACT, FAST>(act_rt, v);
        }));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Ring-buffered variants (one CTA per row, 256 compute threads + one copy-producer warp).
// The phases of a row (load, two reductions, store) leave the memory system idle while a CTA
// reduces, and with rows held in registers only a couple of CTAs fit per SM. Here a producer
// warp streams whole rows into a shared-memory ring with 1-D bulk copies (cp.async.bulk +
// mbarrier transaction counts), several rows ahead of the compute warps, so loads stay in
// flight through every phase. Compute warps copy their vectors from the ring into registers and
// release the stage at once. Waits are time-bounded; an expired wait raises an abort flag that
// all compute threads observe at the same point (after a barrier), so nobody is left behind.
// ---------------------------------------------------------------------------------------------
constexpr int kRingCompute = 256;
constexpr int kRingThreads = kRingCompute + 32;

template <typename T, int ACT, bool AFFINE, int NV>
__global__ void __launch_bounds__(kRingThreads)
ln_fwd_ring_kernel(T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ inv_out, const T* __restrict__ x,
                   const T* __restrict__ gamma, const T* __restrict__ beta, int64_t D, int64_t R, float eps, int act_rt,
                   int stages, unsigned int* status) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = Vec16<T>::N;
  extern __shared__ __align__(1024) uint8_t ring_smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(ring_smem);
  uint64_t* empty = full + stages;
  float* red = reinterpret_cast<float*>(ring_smem + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ring_smem + 768);
  uint8_t* data = ring_smem + 1024;
  const uint32_t row_bytes = (uint32_t)(D * sizeof(T));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kRingCompute / 32); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int64_t nrows = blockIdx.x < R ? (R - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if (warp == kRingCompute / 32) {
    if (lane == 0) {
      for (int64_t i = 0; i < nrows; ++i) {
        const int st = (int)(i % stages);
        const uint32_t ph = (uint32_t)((i / stages) & 1);
        if (!mbar_wait(&empty[st], ph ^ 1u, status, 0x200000u)) break;
        const int64_t row = blockIdx.x + i * gridDim.x;
        mbar_expect_tx(&full[st], row_bytes);
        bulk_load_1d(smem_u32(data + (size_t)st * row_bytes), x + row * D, row_bytes, &full[st]);
      }
    }
    return;
  }
  // scale and shift of this thread's features, unpacked once (the per-row work is then free of conversions)
  float gf[NV][V], bf[NV][V];
  if constexpr (AFFINE) {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * kRingCompute + t) * V;
      if (i < D) {
        const Vec16<T> gv = load16(gamma + i), bv = load16(beta + i);
#pragma unroll
        for (int j = 0; j < V; ++j) { gf[k][j] = gv.get(j); bf[k][j] = bv.get(j); }
      }
    }
  }
  const float invD = 1.f / (float)D;
  // Two rows per round: a round costs a fixed chain (wait, pass, block reduction with two barriers, pass) that does not
  // depend on the row length, so short rows (2-byte elements) are bound by rounds per second, not by bytes; two rows
  // share one reduction (four sums) and halve the number of rounds.
  constexpr int kRowsPerRound = sizeof(T) == 2 ? 2 : 1;   // 4-byte rows are long enough to be bandwidth-bound one at a time
  for (int64_t it = 0; it < nrows; it += kRowsPerRound) {
    const bool two = kRowsPerRound == 2 && it + 1 < nrows;
    const int st0 = (int)(it % stages), st1 = (int)((it + 1) % stages);
    const uint32_t ph0 = (uint32_t)((it / stages) & 1), ph1 = (uint32_t)(((it + 1) / stages) & 1);
    const int64_t row0 = blockIdx.x + it * gridDim.x, row1 = row0 + gridDim.x;
    if (!mbar_wait_warp(&full[st0], ph0, status, 0x400000u)) *abort_flag = 1;
    if (two && !mbar_wait_warp(&full[st1], ph1, status, 0x400000u)) *abort_flag = 1;
    const T* sx0 = reinterpret_cast<const T*>(data + (size_t)st0 * row_bytes);
    const T* sx1 = reinterpret_cast<const T*>(data + (size_t)st1 * row_bytes);
    // One pass over a row: sums of d = x - K and of d^2 with K = the row's first element (a sample of the row, so
    // |mean - K| is of the order of the deviation and var = E[d^2] - E[d]^2 does not cancel), reduced together.
    const float K0 = to_f32(sx0[0]), K1 = two ? to_f32(sx1[0]) : 0.f;
    float df0[NV][V], df1[NV][V];
    float s0 = 0.f, q0 = 0.f, s1 = 0.f, q1 = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * kRingCompute + t) * V;
      if (i < D) {
        const Vec16<T> xv = load16(sx0 + i);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float d = xv.get(j) - K0;
          df0[k][j] = d;
          s0 += d;
          q0 = fmaf(d, d, q0);
        }
        if (two) {
          const Vec16<T> xw = load16(sx1 + i);
#pragma unroll
          for (int j = 0; j < V; ++j) {
            const float d = xw.get(j) - K1;
            df1[k][j] = d;
            s1 += d;
            q1 = fmaf(d, d, q1);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) { mbar_arrive(&empty[st0]); if (two) mbar_arrive(&empty[st1]); }
    const float4 sq = group_sum4(s0, q0, s1, q1, red, kRingCompute);
    if (*abort_flag) { drain_after_abort(); break; }
    auto finish = [&](float su, float sq2, float K, int64_t row, float (&df)[NV][V]) {
      const float dm = su * invD;                                  // mean - K
      const float var = fmaxf(fmaf(-dm, dm, sq2 * invD), 0.f);
      const float inv = 1.f / sqrtf(var + eps);
      const float nmi = -dm * inv;
      if (t == 0) { mean_out[row] = K + dm; inv_out[row] = inv; }
      T* yr = y + row * D;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int64_t i = ((int64_t)k * kRingCompute + t) * V;
        if (i < D) {
          store16_stream(yr + i, vec_from<T>([&](int j) {
            float v = fmaf(df[k][j], inv, nmi);                      // (x - mean) * inv
            if constexpr (AFFINE) v = fmaf(v, gf[k][j], bf[k][j]);
            return act_apply_any<ACT, FAST>(act_rt, v);
          }));
        }
      }
    };
    finish(sq.x, sq.y, K0, row0, df0);
    if (two) finish(sq.z, sq.w, K1, row1, df1);
  }
}

template <typename T, int ACT, bool AFFINE, int NV>
__global__ void __launch_bounds__(kRingThreads, (NV * Vec16<T>::N <= 16) ? 2 : 1)
ln_bwd_ring_kernel(T* __restrict__ dx, float* __restrict__ partial, const T* __restrict__ dy, const T* __restrict__ x,
                   const T* __restrict__ gamma, const T* __restrict__ beta, const float* __restrict__ mean_in,
                   const float* __restrict__ inv_in, int64_t D, int64_t R, int act_rt, int stages, unsigned int* status) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = Vec16<T>::N;
  extern __shared__ __align__(1024) uint8_t ring_smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(ring_smem);
  uint64_t* empty = full + stages;
  float* red = reinterpret_cast<float*>(ring_smem + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ring_smem + 768);
  uint8_t* data = ring_smem + 1024;
  const uint32_t row_bytes = (uint32_t)(D * sizeof(T));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kRingCompute / 32); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int64_t nrows = blockIdx.x < R ? (R - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if (warp == kRingCompute / 32) {
    if (lane == 0) {
      for (int64_t i = 0; i < nrows; ++i) {
        const int st = (int)(i % stages);
        const uint32_t ph = (uint32_t)((i / stages) & 1);
        if (!mbar_wait(&empty[st], ph ^ 1u, status, 0x800000u)) break;
        const int64_t row = blockIdx.x + i * gridDim.x;
        mbar_expect_tx(&full[st], 2 * row_bytes);
        bulk_load_1d(smem_u32(data + (size_t)st * 2 * row_bytes), x + row * D, row_bytes, &full[st]);
        bulk_load_1d(smem_u32(data + (size_t)st * 2 * row_bytes + row_bytes), dy + row * D, row_bytes, &full[st]);
      }
    }
    return;
  }
  // the scale of this thread's features unpacked once; the shift is needed only to rebuild a pre-activation
  float gf[NV][V];
  Vec16<T> bv[NV];
  float adg[NV][V], adb[NV][V];
  if constexpr (AFFINE) {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * kRingCompute + t) * V;
      if (i < D) {
        const Vec16<T> gv = load16(gamma + i);
#pragma unroll
        for (int j = 0; j < V; ++j) gf[k][j] = gv.get(j);
        if constexpr (ACT != LB2_ACT_IDENTITY) bv[k] = load16(beta + i);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) { adg[k][j] = 0.f; adb[k][j] = 0.f; }
    }
  }
  const float invD = 1.f / (float)D;
  // Two rows per round (see the forward kernel): the rows stay in their ring stages through both passes, the
  // dgamma / dbeta accumulators are per feature and therefore shared by the two rows (row order kept), and one
  // reduction of four sums serves both.
  constexpr int kRowsPerRound = sizeof(T) == 2 ? 2 : 1;   // 4-byte rows are long enough to be bandwidth-bound one at a time
  for (int64_t it = 0; it < nrows; it += kRowsPerRound) {
    const bool two = kRowsPerRound == 2 && it + 1 < nrows;
    const int st0 = (int)(it % stages), st1 = (int)((it + 1) % stages);
    const uint32_t ph0 = (uint32_t)((it / stages) & 1), ph1 = (uint32_t)(((it + 1) / stages) & 1);
    const int64_t row0 = blockIdx.x + it * gridDim.x, row1 = row0 + gridDim.x;
    const float mean0 = mean_in[row0], inv0 = inv_in[row0];
    const float mean1 = two ? mean_in[row1] : 0.f, inv1 = two ? inv_in[row1] : 0.f;
    if (!mbar_wait_warp(&full[st0], ph0, status, 0x1000000u)) *abort_flag = 1;
    if (two && !mbar_wait_warp(&full[st1], ph1, status, 0x1000000u)) *abort_flag = 1;
    // d = dy * act'(pre-activation), the pre-activation rebuilt as ((x - mean) * inv) * gamma + beta
    auto act_scaled = [&](float d, float xh, int k, int j) {
      if constexpr (ACT != LB2_ACT_IDENTITY) {
        float pre = xh;
        if constexpr (AFFINE) pre = fmaf(xh, gf[k][j], bv[k].get(j));
        d *= act_grad_pre_any<ACT, FAST>(act_rt, pre);
      }
      return d;
    };
    auto pass1 = [&](int st, float mean, float inv, float& s1, float& s2) {
      const T* sx = reinterpret_cast<const T*>(data + (size_t)st * 2 * row_bytes);
      const T* sdy = reinterpret_cast<const T*>(data + (size_t)st * 2 * row_bytes + row_bytes);
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int64_t i = ((int64_t)k * kRingCompute + t) * V;
        if (i < D) {
          const Vec16<T> xv = load16(sx + i), gy = load16(sdy + i);
#pragma unroll
          for (int j = 0; j < V; ++j) {
            const float xh = (xv.get(j) - mean) * inv;
            const float d = act_scaled(gy.get(j), xh, k, j);
            float g = d;
            if constexpr (AFFINE) {
              adg[k][j] = fmaf(d, xh, adg[k][j]);
              adb[k][j] += d;
              g = d * gf[k][j];
            }
            s1 += g;
            s2 = fmaf(g, xh, s2);
          }
        }
      }
    };
    float s1a = 0.f, s2a = 0.f, s1b = 0.f, s2b = 0.f;
    pass1(st0, mean0, inv0, s1a, s2a);
    if (two) pass1(st1, mean1, inv1, s1b, s2b);
    const float4 m = group_sum4(s1a, s2a, s1b, s2b, red, kRingCompute);
    if (*abort_flag) { drain_after_abort(); break; }
    // dx = inv * (g - m1 - xh * m2) = g * inv + (x * c1i + c0m): the xh term folded into one multiply-add on x
    auto pass2 = [&](int st, int64_t row, float mean, float inv, float sum1, float sum2) {
      const T* sx = reinterpret_cast<const T*>(data + (size_t)st * 2 * row_bytes);
      const T* sdy = reinterpret_cast<const T*>(data + (size_t)st * 2 * row_bytes + row_bytes);
      const float m1 = sum1 * invD, m2 = sum2 * invD;
      const float c1i = -inv * m2 * inv;
      const float c0m = fmaf(-mean, c1i, -inv * m1);
      T* dxr = dx + row * D;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int64_t i = ((int64_t)k * kRingCompute + t) * V;
        if (i < D) {
          const Vec16<T> xv = load16(sx + i), gy = load16(sdy + i);
          store16_stream(dxr + i, vec_from<T>([&](int j) {
            const float xf = xv.get(j);
            float d = gy.get(j);
            if constexpr (ACT != LB2_ACT_IDENTITY) d = act_scaled(d, (xf - mean) * inv, k, j);
            if constexpr (AFFINE) d *= gf[k][j];
            return fmaf(d, inv, fmaf(xf, c1i, c0m));
          }));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
    };
    pass2(st0, row0, mean0, inv0, m.x, m.y);
    if (two) pass2(st1, row1, mean1, inv1, m.z, m.w);
  }
  if constexpr (AFFINE) {
    float* pg = partial + (int64_t)blockIdx.x * 2 * D;
    float* pb = pg + D;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * kRingCompute + t) * V;
      if (i < D) {
#pragma unroll
        for (int j = 0; j < V; ++j) { pg[i + j] = adg[k][j]; pb[i + j] = adb[k][j]; }
      }
    }
  }
}

// Generic: one CTA per row, scalar accesses, three passes (passes 2 and 3 hit L1/L2).
template <typename T, int ACT, bool AFFINE>
__global__ void __launch_bounds__(256) ln_fwd_generic_kernel(T* __restrict__ y, float* __restrict__ mean_out,
                                                             float* __restrict__ inv_out, const T* __restrict__ x,
                                                             const T* __restrict__ gamma, const T* __restrict__ beta,
                                                             int64_t D, int64_t R, float eps, int act_rt) {
  constexpr bool FAST = sizeof(T) == 2;
  __shared__ float red[32];
  const float invD = 1.f / (float)D;
  for (int64_t row = blockIdx.x; row < R; row += gridDim.x) {
    const T* xr = x + row * D;
    float s = 0.f;
    for (int64_t i = threadIdx.x; i < D; i += blockDim.x) s += to_f32(xr[i]);
    const float mean = block_sum(s, red) * invD;
    float q = 0.f;
    for (int64_t i = threadIdx.x; i < D; i += blockDim.x) { float d = to_f32(xr[i]) - mean; q += d * d; }
    const float var = block_sum(q, red) * invD;
    const float inv = 1.f / sqrtf(var + eps);
    if (threadIdx.x == 0) { mean_out[row] = mean; inv_out[row] = inv; }
    T* yr = y + row * D;
    for (int64_t i = threadIdx.x; i < D; i += blockDim.x) {
      float gp = inv, bp = -mean * inv;
      if constexpr (AFFINE) { gp = to_f32(gamma[i]) * inv; bp = to_f32(beta[i]) - mean * gp; }
      yr[i] = from_f32<T>(act_apply_any<ACT, FAST>(act_rt, fmaf(to_f32(xr[i]), gp, bp)));
    }
  }
}

// Backward, cached. partial: [gridDim.x][2][D] fp32 (dgamma then dbeta) when AFFINE.
template <typename T, int ACT, bool AFFINE, int RT, int NV, int BT>
__global__ void __launch_bounds__(BT) ln_bwd_cached_kernel(T* __restrict__ dx, float* __restrict__ partial,
                                                           const T* __restrict__ dy, const T* __restrict__ x,
                                                           const T* __restrict__ gamma, const T* __restrict__ beta,
                                                           const float* __restrict__ mean_in,
                                                           const float* __restrict__ inv_in, int64_t D, int64_t R, int act_rt) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int V = Vec16<T>::N;
  constexpr int ROWS = BT / RT;
  __shared__ float red[32];
  const int t = threadIdx.x % RT, slot = threadIdx.x / RT;
  Vec16<T> gv[NV], bv[NV];
  float adg[NV][V], adb[NV][V];
  if constexpr (AFFINE) {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * RT + t) * V;
      if (i < D) { gv[k] = load16(gamma + i); bv[k] = load16(beta + i); }
#pragma unroll
      for (int j = 0; j < V; ++j) { adg[k][j] = 0.f; adb[k][j] = 0.f; }
    }
  }
  const float invD = 1.f / (float)D;
  for (int64_t row = (int64_t)blockIdx.x * ROWS + slot; row < R; row += (int64_t)gridDim.x * ROWS) {
    const T* xr = x + row * D;
    const T* dyr = dy + row * D;
    const float mean = mean_in[row], inv = inv_in[row];
    Vec16<T> xv[NV], gy[NV];  // gy is overwritten in place with g = dy*act'*gamma (kept in fp32 bits for f32)
    float gf[NV][V];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * RT + t) * V;
      if (i < D) {
        xv[k] = load16_stream(xr + i);
        gy[k] = load16_stream(dyr + i);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = (xv[k].get(j) - mean) * inv;
          float d = gy[k].get(j);
          if constexpr (ACT != LB2_ACT_IDENTITY) {
            float gp = inv, bp = -mean * inv;
            if constexpr (AFFINE) { gp = gv[k].get(j) * inv; bp = bv[k].get(j) - mean * gp; }
            d *= act_grad_pre_any<ACT, FAST>(act_rt, fmaf(xv[k].get(j), gp, bp));
          }
          float g = d;
          if constexpr (AFFINE) {
            adg[k][j] += d * xh;
            adb[k][j] += d;
            g = d * gv[k].get(j);
          }
          gf[k][j] = g;
          s1 += g;
          s2 += g * xh;
        }
      }
    }
    // both reductions of the backward in one pass over registers
    const float m1 = row_sum<RT>(s1, red) * invD;
    const float m2 = row_sum<RT>(s2, red) * invD;
    T* dxr = dx + row * D;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = ((int64_t)k * RT + t) * V;
      if (i < D) {
        store16_stream(dxr + i, vec_from<T>([&](int j) {
          const float xh = (xv[k].get(j) - mean) * inv;
          return inv * (gf[k][j] - m1 - xh * m2);
        }));
      }
    }
  }
  if constexpr (AFFINE) {
    float* pg = partial + (int64_t)blockIdx.x * 2 * D;
    float* pb = pg + D;
    if constexpr (ROWS == 1) {
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int64_t i = ((int64_t)k * RT + t) * V;
        if (i < D) {
#pragma unroll
          for (int j = 0; j < V; ++j) { pg[i + j] = adg[k][j]; pb[i + j] = adb[k][j]; }
        }
      }
    } else {
      // warp-per-row: fold the CTA's row slots through shared memory in slot order
      __shared__ float fold[ROWS][32 * V + 1];
      for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          __syncthreads();
#pragma unroll
          for (int j = 0; j < V; ++j) fold[slot][t * V + j] = pass == 0 ? adg[k][j] : adb[k][j];
          __syncthreads();
          for (int col = threadIdx.x; col < 32 * V; col += BT) {
            float s = 0.f;
#pragma unroll
            for (int r = 0; r < ROWS; ++r) s += fold[r][col];
            const int64_t i = (int64_t)k * RT * V + col;
            if (i < D) (pass == 0 ? pg : pb)[i] = s;
          }
        }
      }
    }
  }
}

// Backward, generic: one CTA per row; affine-gradient partials accumulate in the workspace rows
// owned by this CTA (each feature is always touched by the same thread: no race).
template <typename T, int ACT, bool AFFINE>
__global__ void __launch_bounds__(256) ln_bwd_generic_kernel(T* __restrict__ dx, float* __restrict__ partial,
                                                             const T* __restrict__ dy, const T* __restrict__ x,
                                                             const T* __restrict__ gamma, const T* __restrict__ beta,
                                                             const float* __restrict__ mean_in,
                                                             const float* __restrict__ inv_in, int64_t D, int64_t R, int act_rt) {
  constexpr bool FAST = sizeof(T) == 2;
  __shared__ float red[32];
  float* pg = partial + (int64_t)blockIdx.x * 2 * D;
  float* pb = pg + D;
  if constexpr (AFFINE) {
    for (int64_t i = threadIdx.x; i < D; i += blockDim.x) { pg[i] = 0.f; pb[i] = 0.f; }
  }
  const float invD = 1.f / (float)D;
  for (int64_t row = blockIdx.x; row < R; row += gridDim.x) {
    const T* xr = x + row * D;
    const T* dyr = dy + row * D;
    const float mean = mean_in[row], inv = inv_in[row];
    auto g_of = [&](int64_t i, float& xh, float& d) {
      const float xv = to_f32(xr[i]);
      xh = (xv - mean) * inv;
      d = to_f32(dyr[i]);
      if constexpr (ACT != LB2_ACT_IDENTITY) {
        float gp = inv, bp = -mean * inv;
        if constexpr (AFFINE) { gp = to_f32(gamma[i]) * inv; bp = to_f32(beta[i]) - mean * gp; }
        d *= act_grad_pre_any<ACT, FAST>(act_rt, fmaf(xv, gp, bp));
      }
      float g = d;
      if constexpr (AFFINE) g = d * to_f32(gamma[i]);
      return g;
    };
    float s1 = 0.f, s2 = 0.f;
    for (int64_t i = threadIdx.x; i < D; i += blockDim.x) {
      float xh, d;
      const float g = g_of(i, xh, d);
      s1 += g;
      s2 += g * xh;
      if constexpr (AFFINE) { pg[i] += d * xh; pb[i] += d; }
    }
    const float m1 = block_sum(s1, red) * invD;
    const float m2 = block_sum(s2, red) * invD;
    T* dxr = dx + row * D;
    for (int64_t i = threadIdx.x; i < D; i += blockDim.x) {
      float xh, d;
      const float g = g_of(i, xh, d);
      dxr[i] = from_f32<T>(inv * (g - m1 - xh * m2));
    }
  }
}

// out[i] = sum_k partial[k][which][i]. block (32 features, 32 slices): slice y adds parts y, y+32, ... in
// ascending order (a short chain of independent loads: the kernel is latency-bound, not bandwidth-bound), then the
// slice sums are added in slice order: a fixed order, deterministic.
constexpr int kLnFinishSlices = 32;
template <typename T>
__global__ void __launch_bounds__(32 * kLnFinishSlices) ln_finish_kernel(T* __restrict__ dgamma, T* __restrict__ dbeta,
                                                                        const float* __restrict__ partial, int64_t D, int parts) {
  __shared__ float sg[kLnFinishSlices][33], sb[kLnFinishSlices][33];
  const int64_t i = (int64_t)blockIdx.x * 32 + threadIdx.x;
  float ag = 0.f, ab = 0.f;
  if (i < D) {
#pragma unroll 4
    for (int k = threadIdx.y; k < parts; k += kLnFinishSlices) {
      ag += __ldcs(partial + ((int64_t)k * 2) * D + i);
      ab += __ldcs(partial + ((int64_t)k * 2 + 1) * D + i);
    }
  }
  sg[threadIdx.y][threadIdx.x] = ag;
  sb[threadIdx.y][threadIdx.x] = ab;
  __syncthreads();
  if (threadIdx.y == 0 && i < D) {
    float tg = 0.f, tb = 0.f;
#pragma unroll
    for (int r = 0; r < kLnFinishSlices; ++r) { tg += sg[r][threadIdx.x]; tb += sb[r][threadIdx.x]; }
    dgamma[i] = from_f32<T>(tg);
    dbeta[i] = from_f32<T>(tb);
  }
}

struct LnPlan {
  bool cached;
  int rt, nv, bt, grid;
  bool ring;        // rows streamed through a shared-memory ring by a producer warp
  int stages, smem;
};

template <typename T> static LnPlan ln_plan(int64_t D, int64_t R, bool aligned, bool bwd) {
  constexpr int V = Vec16<T>::N;
  LnPlan p{};
  const int sms = sm_count();
  p.cached = aligned && (D % V == 0);
  const int64_t vecs = D / V;
  const int max_nv = bwd ? 4 : 8;
  if (p.cached && vecs <= 32 * 4) {  // small rows: one warp per row
    p.rt = 32; p.bt = 256;
    p.nv = vecs <= 32 ? 1 : (vecs <= 64 ? 2 : 4);
    int64_t ctas = (R + 7) / 8;
    p.grid = (int)(ctas < (int64_t)sms * 8 ? ctas : (int64_t)sms * 8);
  } else if (p.cached && vecs <= 256 * max_nv) {
    p.rt = 256; p.bt = 256;
    p.nv = vecs <= 256 ? 1 : (vecs <= 512 ? 2 : (vecs <= 1024 ? 4 : 8));
    p.grid = (int)(R < (int64_t)sms * 4 ? R : (int64_t)sms * 4);
  } else if (p.cached && vecs <= 512 * max_nv) {
    p.rt = 512; p.bt = 512;
    p.nv = vecs <= 512 * 4 ? 4 : 8;
    p.grid = (int)(R < (int64_t)sms * 2 ? R : (int64_t)sms * 2);
  } else {
    p.cached = false;
    p.rt = 256; p.bt = 256; p.nv = 0;
    p.grid = (int)(R < (int64_t)sms * 4 ? R : (int64_t)sms * 4);
  }
  if (p.cached && p.rt == 256) {
    // ring variant: stage = one row of x (forward) or of x and dy (backward)
    const int64_t stage_bytes = D * (int64_t)sizeof(T) * (bwd ? 2 : 1);
    int stages = (int)((96 * 1024) / stage_bytes);
    if (stages > 6) stages = 6;
    if (stages < 2 && 2 * stage_bytes <= 200 * 1024) stages = 2;
    if (stages >= 2) {
      p.ring = true;
      p.stages = stages;
      p.smem = 1024 + (int)(stages * stage_bytes);
      int per_sm = (220 * 1024) / p.smem;
      if (per_sm > 4) per_sm = 4;
      if (per_sm < 1) per_sm = 1;
      p.grid = (int)(R < (int64_t)sms * per_sm ? R : (int64_t)sms * per_sm);
    }
  }
  if (p.grid < 1) p.grid = 1;
  return p;
}

template <typename K>
static int32_t ring_smem_attr(K kernel, int smem) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "layernorm: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
  return LB2_OK;
}

#define LN_RING_CASE(KERNEL, NV_, ...)                                                        \
  {                                                                                           \
    int32_t rc__ = ring_smem_attr(KERNEL<T, ACT, AFFINE, NV_>, p.smem);                       \
    if (rc__ != LB2_OK) return rc__;                                                          \
    KERNEL<T, ACT, AFFINE, NV_><<<p.grid, kRingThreads, p.smem, st>>>(__VA_ARGS__);           \
  }
#define LN_RING_SWITCH(KERNEL, ...)                                  \
  if (p.nv == 1) LN_RING_CASE(KERNEL, 1, __VA_ARGS__)                \
  else if (p.nv == 2) LN_RING_CASE(KERNEL, 2, __VA_ARGS__)           \
  else if (p.nv == 4) LN_RING_CASE(KERNEL, 4, __VA_ARGS__)           \
  else LN_RING_CASE(KERNEL, 8, __VA_ARGS__)
#define LN_RING_SWITCH_BWD(KERNEL, ...)                              \
  if (p.nv == 1) LN_RING_CASE(KERNEL, 1, __VA_ARGS__)                \
  else if (p.nv == 2) LN_RING_CASE(KERNEL, 2, __VA_ARGS__)           \
  else LN_RING_CASE(KERNEL, 4, __VA_ARGS__)

#define LN_LAUNCH_CACHED(KERNEL, RT_, NV_, BT_, ...)                                   \
  KERNEL<T, ACT, AFFINE, RT_, NV_, BT_><<<p.grid, BT_, 0, st>>>(__VA_ARGS__, act)

#define LN_SWITCH(KERNEL, ...)                                                          \
  if (p.rt == 32) {                                                                     \
    if (p.nv == 1) LN_LAUNCH_CACHED(KERNEL, 32, 1, 256, __VA_ARGS__);                   \
    else if (p.nv == 2) LN_LAUNCH_CACHED(KERNEL, 32, 2, 256, __VA_ARGS__);              \
    else LN_LAUNCH_CACHED(KERNEL, 32, 4, 256, __VA_ARGS__);                             \
  } else if (p.rt == 256) {                                                             \
    if (p.nv == 1) LN_LAUNCH_CACHED(KERNEL, 256, 1, 256, __VA_ARGS__);                  \
    else if (p.nv == 2) LN_LAUNCH_CACHED(KERNEL, 256, 2, 256, __VA_ARGS__);             \
    else if (p.nv == 4) LN_LAUNCH_CACHED(KERNEL, 256, 4, 256, __VA_ARGS__);             \
    else LN_LAUNCH_CACHED(KERNEL, 256, 8, 256, __VA_ARGS__);                            \
  } else {                                                                              \
    if (p.nv == 4) LN_LAUNCH_CACHED(KERNEL, 512, 4, 512, __VA_ARGS__);                  \
    else LN_LAUNCH_CACHED(KERNEL, 512, 8, 512, __VA_ARGS__);                            \
  }

// the backward never caches more than 4 vectors per thread (see ln_plan)
#define LN_SWITCH_BWD(KERNEL, ...)                                                      \
  if (p.rt == 32) {                                                                     \
    if (p.nv == 1) LN_LAUNCH_CACHED(KERNEL, 32, 1, 256, __VA_ARGS__);                   \
    else if (p.nv == 2) LN_LAUNCH_CACHED(KERNEL, 32, 2, 256, __VA_ARGS__);              \
    else LN_LAUNCH_CACHED(KERNEL, 32, 4, 256, __VA_ARGS__);                             \
  } else if (p.rt == 256) {                                                             \
    if (p.nv == 1) LN_LAUNCH_CACHED(KERNEL, 256, 1, 256, __VA_ARGS__);                  \
    else if (p.nv == 2) LN_LAUNCH_CACHED(KERNEL, 256, 2, 256, __VA_ARGS__);             \
    else LN_LAUNCH_CACHED(KERNEL, 256, 4, 256, __VA_ARGS__);                            \
  } else {                                                                              \
    LN_LAUNCH_CACHED(KERNEL, 512, 4, 512, __VA_ARGS__);                                 \
  }

template <typename T, int ACT, bool AFFINE>
static int32_t ln_fwd_launch(T* y, float* sm, float* si, const T* x, const T* g, const T* b, int64_t D, int64_t R,
                             float eps, int32_t act, cudaStream_t st) {
  const bool al = aligned_to(y, 16) && aligned_to(x, 16) && (!g || (aligned_to(g, 16) && aligned_to(b, 16)));
  const LnPlan p = ln_plan<T>(D, R, al, false);
  constexpr int V = Vec16<T>::N;
  if (sizeof(T) == 2 && p.cached && D % V == 0 && D / V > 32 * 4 && D / V <= 32 * 16 && R >= (int64_t)sm_count() * 16) {
    // rows of 1025 to 4096 two-byte elements, enough of them to give every resident warp several rows
    const int smem = AFFINE ? (int)(2 * D * sizeof(T)) : 0;
    const int grid = sm_count() * 2;
    const int64_t vecs = D / V;
    if (vecs <= 32 * 8) ln_fwd_warp_kernel<T, ACT, AFFINE, 8><<<grid, 256, smem, st>>>(y, sm, si, x, g, b, D, R, eps, act);
    else ln_fwd_warp_kernel<T, ACT, AFFINE, 16><<<grid, 256, smem, st>>>(y, sm, si, x, g, b, D, R, eps, act);
  } else if (p.ring) {
    unsigned int* status = device_status_word();
    LB2_REQUIRE(status != nullptr, LB2_LAUNCH_FAIL, "layernorm: device status word unavailable");
    LN_RING_SWITCH(ln_fwd_ring_kernel, y, sm, si, x, g, b, D, R, eps, act, p.stages, status)
  } else if (p.cached) {
    LN_SWITCH(ln_fwd_cached_kernel, y, sm, si, x, g, b, D, R, eps);
  } else {
    ln_fwd_generic_kernel<T, ACT, AFFINE><<<p.grid, 256, 0, st>>>(y, sm, si, x, g, b, D, R, eps, act);
  }
  LB2_CHECK_LAUNCH("layernorm_fwd");
  return LB2_OK;
}

template <typename T, int ACT, bool AFFINE>
static int32_t ln_bwd_launch(T* dx, T* dg, T* db, const T* dy, const T* x, const T* g, const T* b, const float* sm,
                             const float* si, int64_t D, int64_t R, float* ws, int32_t act, cudaStream_t st) {
  const bool al = aligned_to(dx, 16) && aligned_to(dy, 16) && aligned_to(x, 16) &&
                  (!g || (aligned_to(g, 16) && aligned_to(b, 16)));
  const LnPlan p = ln_plan<T>(D, R, al, true);
  if (p.ring) {
    unsigned int* status = device_status_word();
    LB2_REQUIRE(status != nullptr, LB2_LAUNCH_FAIL, "layernorm: device status word unavailable");
    LN_RING_SWITCH_BWD(ln_bwd_ring_kernel, dx, ws, dy, x, g, b, sm, si, D, R, act, p.stages, status)
  } else if (p.cached) {
    LN_SWITCH_BWD(ln_bwd_cached_kernel, dx, ws, dy, x, g, b, sm, si, D, R);
  } else {
    ln_bwd_generic_kernel<T, ACT, AFFINE><<<p.grid, 256, 0, st>>>(dx, ws, dy, x, g, b, sm, si, D, R, act);
  }
  LB2_CHECK_LAUNCH("layernorm_bwd");
  if constexpr (AFFINE) {
    ln_finish_kernel<T><<<(unsigned)((D + 31) / 32), dim3(32, kLnFinishSlices), 0, st>>>(dg, db, ws, D, p.grid);
    LB2_CHECK_LAUNCH("layernorm_bwd_finish");
  }
  return LB2_OK;
}

static size_t ln_bwd_ws_bytes(int64_t D, int64_t R) {
  // upper bound over both dtypes / alignments: grid <= 8 * SMs
  int64_t g = (int64_t)sm_count() * 8;
  if (R < g) g = R;
  if (g < 1) g = 1;
  return align_up((size_t)g * 2 * (size_t)D * sizeof(float), 256);
}

}  // namespace lb2

using namespace lb2;

extern "C" {

int32_t lb2_layernorm_fwd(void* y, float* save_mean, float* save_invstd, const void* x, const void* gamma,
                          const void* beta, int64_t D, int64_t R, double eps, int32_t dtype, int32_t act,
                          void* stream) {
  LB2_REQUIRE(D >= 0 && R >= 0, LB2_BAD_SHAPE, "negative extent");
  if (D == 0 || R == 0) return LB2_OK;
  int32_t rc = check_norm_common(y, x, gamma, beta, save_mean, save_invstd, dtype, act);
  if (rc != LB2_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LB2_DISPATCH_DTYPE(dtype, {
    LB2_DISPATCH_ACT3(act, {
      if (gamma) return ln_fwd_launch<T, ACT, true>((T*)y, save_mean, save_invstd, (const T*)x, (const T*)gamma, (const T*)beta, D, R, (float)eps, act, st);
      else return ln_fwd_launch<T, ACT, false>((T*)y, save_mean, save_invstd, (const T*)x, nullptr, nullptr, D, R, (float)eps, act, st);
    });
  });
  return LB2_OK;
}

size_t lb2_layernorm_bwd_workspace_bytes(int64_t D, int64_t R) {
  if (D <= 0 || R <= 0) return 0;
  return ln_bwd_ws_bytes(D, R);
}

int32_t lb2_layernorm_bwd(void* dx, void* dgamma, void* dbeta, const void* dy, const void* x, const void* gamma,
                          const void* beta, const float* save_mean, const float* save_invstd, int64_t D, int64_t R,
                          int32_t dtype, int32_t act, void* workspace, size_t workspace_bytes, void* stream) {
  LB2_REQUIRE(D >= 0 && R >= 0, LB2_BAD_SHAPE, "negative extent");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (D == 0 || R == 0) {
    if (D > 0 && dgamma && valid_dtype(dtype)) {
      cudaMemsetAsync(dgamma, 0, (size_t)D * dtype_size(dtype), st);
      cudaMemsetAsync(dbeta, 0, (size_t)D * dtype_size(dtype), st);
    }
    return LB2_OK;
  }
  int32_t rc = check_norm_common(dx, x, gamma, beta, save_mean, save_invstd, dtype, act);
  if (rc != LB2_OK) return rc;
  LB2_REQUIRE(dy != nullptr, LB2_BAD_ARG, "dy is null");
  LB2_REQUIRE(!gamma || (dgamma && dbeta), LB2_BAD_ARG, "dgamma/dbeta required when scale is given");
  if (gamma) {
    LB2_REQUIRE(workspace && workspace_bytes >= ln_bwd_ws_bytes(D, R), LB2_WORKSPACE_TOO_SMALL,
                "workspace of %zu bytes needed", ln_bwd_ws_bytes(D, R));
    LB2_REQUIRE(aligned_to(workspace, 16), LB2_BAD_ALIGN, "workspace must be 16-byte aligned");
  }
  LB2_DISPATCH_DTYPE(dtype, {
    LB2_DISPATCH_ACT3(act, {
      if (gamma) return ln_bwd_launch<T, ACT, true>((T*)dx, (T*)dgamma, (T*)dbeta, (const T*)dy, (const T*)x, (const T*)gamma, (const T*)beta, save_mean, save_invstd, D, R, (float*)workspace, act, st);
      else return ln_bwd_launch<T, ACT, false>((T*)dx, nullptr, nullptr, (const T*)dy, (const T*)x, nullptr, nullptr, save_mean, save_invstd, D, R, (float*)workspace, act, st);
    });
  });
  return LB2_OK;
}

}  // extern "C"

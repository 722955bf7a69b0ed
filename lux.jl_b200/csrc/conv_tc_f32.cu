// Tensor-core convolution for Float32 storage on sm_100a: the implicit GEMM of conv_tc.cu with
// kind::tf32 MMAs made fp32-accurate.
//
// Accuracy. A tf32 product keeps 11 bits of each factor, so every operand is split on the way in,
// hi = tf32(x), lo = x - hi, and each k-block forms three products (hi*hi, hi*lo, lo*hi). The
// tensor core also TRUNCATES when it adds into its TMEM accumulator, an error that grows with the
// number of accumulating MMAs (about 1e-7 relative each), so TMEM only ever holds one k-block's
// MMAs (hi*hi in one accumulator, the two small products in another): the eight accumulating warps
// pull those partials out of TMEM (a ring of chunk buffers, so the following k-blocks' MMAs overlap) and add it round-to-nearest into fp32 registers. The filter gradient,
// whose contraction runs over every output position of every image, stays within 1e-5 this way.
//
// Shapes taken: as the bf16 path (2-D, stride 1, dilation 1, groups 1, output width == input
// width) with W a multiple of 4 elements (16-byte TMA start coordinates).
//
// Forward / data gradient: out[s, co] = sum over k-blocks (tap, 32 channels) of A[s, ci] * Wp[co, k];
// A is MN-major (s contiguous) straight from kW copies of the input shifted along W (the H shift is
// a TMA start coordinate, out-of-range rows are zero-filled = the padding), in the 32-byte-atom
// 128-byte swizzle the tensor core needs to transpose 32-bit elements; the packed filter is K-major.
// Filter gradient: sum_s x[s + shift(tap)] * g[s] = sum_s' x[s'] * g[s' - shift(tap)], so it reuses the W-shifted
// copies of g that the data gradient makes anyway: rows = (tap, co) from those copies, columns = ci from a flat
// hi/lo split of x, contraction over (image, 32-position blocks), both operands K-major, split over CTAs along
// the contraction, fp32 partials reduced in a fixed order.
//
// Roofline: tensor pipe (tf32 rate, three products per useful one); algorithmic FLOPs =
// 2*Wo*Ho*N*Cout*Cin*kW*kH per pass.
#include <stdlib.h>

#include "conv.cuh"
#include "tc_ptx.cuh"

namespace lb2 {

constexpr int kF32Threads = 384;   // warps 0-2: TMA / MMA / TMEM, warps 4-11: accumulate + epilogue
constexpr int kF32BM = 128;
constexpr int kF32MaxKb = 160;     // k-blocks (tap, 32-channel chunk) of the forward kernel
constexpr int kF32MaxRg = 128;     // row groups (tap, 64-channel chunk) of the filter gradient

__device__ __forceinline__ void split_tf32(float v, float& hi, float& lo) {
  uint32_t h;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
  hi = __uint_as_float(h);
  lo = v - hi;
}

// ----------------------------------------------------------------------------------------------
// layout passes
// ----------------------------------------------------------------------------------------------
// hi/lo[t][row][w] = split(in[row][w + t - pad_w])  (0 outside the row), t = 0..kW-1; W % 4 == 0
__global__ void __launch_bounds__(256) conv_shift_split_kernel(float* __restrict__ hi, float* __restrict__ lo,
                                                               const float* __restrict__ in, int W, int64_t rows, int kW,
                                                               int pad_w) {
  const int groups = W / 4;
  const int64_t total = rows * groups;
  const int64_t copy_stride = rows * W;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / groups;
    const int w0 = (int)(i % groups) * 4;
    const float* src = in + row * W;
    float wh[12], wl[12];   // window of 4 + kW - 1 inputs starting at w0 - pad_w, already split
#pragma unroll
    for (int j = 0; j < 11; ++j) {
      const int w = w0 - pad_w + j;
      const float v = (j < 4 + kW - 1 && w >= 0 && w < W) ? __ldg(src + w) : 0.f;
      split_tf32(v, wh[j], wl[j]);
    }
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      if (t < kW) {
        const int64_t o = (int64_t)t * copy_stride + row * W + w0;
        __stcs(reinterpret_cast<float4*>(hi + o), make_float4(wh[t], wh[t + 1], wh[t + 2], wh[t + 3]));
        __stcs(reinterpret_cast<float4*>(lo + o), make_float4(wl[t], wl[t + 1], wl[t + 2], wl[t + 3]));
      }
    }
  }
}

// hi/lo split of a flat array (n % 4 == 0 handled by the scalar tail)
__global__ void __launch_bounds__(256) conv_split_flat_kernel(float* __restrict__ hi, float* __restrict__ lo,
                                                              const float* __restrict__ x, int64_t n) {
  const int64_t n4 = n / 4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 v = __ldcs(reinterpret_cast<const float4*>(x) + i);
    float4 h, l;
    split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
    reinterpret_cast<float4*>(hi)[i] = h;
    reinterpret_cast<float4*>(lo)[i] = l;
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - n4 * 4)) {
    const int64_t i = n4 * 4 + threadIdx.x;
    split_tf32(x[i], hi[i], lo[i]);
  }
}

// Packed, split filter for the forward / data-gradient GEMM: Wp[nrow][kb*32 + j], nrow = GEMM output
// channel, k-block kb = (tap, 32-channel chunk). `transpose` selects the data-gradient packing
// (GEMM output channel = conv input channel, taps reversed).
struct PackGeomF32 {
  int kW, kH, cin, cout, flip, transpose, chunks, n_rows, k_total;
};

__global__ void __launch_bounds__(256) conv_pack_split_filter_kernel(float* __restrict__ wh, float* __restrict__ wl,
                                                                     const float* __restrict__ w, const PackGeomF32 g) {
  const int64_t total = (int64_t)g.n_rows * g.k_total;
  const int kc = g.transpose ? g.cout : g.cin;   // contracted channels
  const int nc = g.transpose ? g.cin : g.cout;   // GEMM output channels
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int row = (int)(i / g.k_total);
    const int col = (int)(i % g.k_total);
    const int kb = col / 32, j = col % 32;
    const int tap = kb / g.chunks, c = (kb % g.chunks) * 32 + j;
    const int tw = tap % g.kW, th = tap / g.kW;   // tap position: input offset (tw - pad_w, th - pad_h)
    float v = 0.f;
    if (row < nc && c < kc) {
      // forward: tap position t pairs with filter index k, t = flip ? k : K-1-k; the data gradient
      // visits position K-1-t of the forward tap
      const int tw_f = g.transpose ? g.kW - 1 - tw : tw, th_f = g.transpose ? g.kH - 1 - th : th;
      const int kw = g.flip ? tw_f : g.kW - 1 - tw_f, kh = g.flip ? th_f : g.kH - 1 - th_f;
      const int ci = g.transpose ? row : c, co = g.transpose ? c : row;
      v = w[((int64_t)(co * g.cin + ci) * g.kH + kh) * g.kW + kw];
    }
    split_tf32(v, wh[i], wl[i]);
  }
}

// ----------------------------------------------------------------------------------------------
// forward / data-gradient kernel
// ----------------------------------------------------------------------------------------------
struct ConvF32Params {
  int32_t S_out, n_img, n_out;
  int32_t tiles_m, tiles_n, num_kb;
  uint32_t idesc, idesc_wide;   // MMA width BN (A_lo * B_hi) and 2*BN (A_hi * [B_hi ; B_lo])
  uint32_t a_desc_hi, a_desc_lbo, a_k_advance;
  uint32_t b_desc_hi, b_desc_lbo, b_k_advance;
  float* y;
  float* preact;
  const float* bias;      // per GEMM output channel, or null
  int32_t act;
  unsigned int* status;
  int16_t a_shift[kF32MaxKb];   // start-coordinate offset along s (multiple of 4 elements)
  int16_t a_chan[kF32MaxKb];    // first contracted channel of the k-block
  int8_t a_copy[kF32MaxKb];     // which W-shifted copy
};

template <int BN> struct ConvF32Cfg {
  static constexpr int A_BYTES = kF32BM * 128;            // 128 positions x 32 channels (fp32), one of hi / lo
  static constexpr int B_BYTES = BN * 128;                // BN rows x 32 contracted elements
  static constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);   // stage = [A_hi | A_lo | B_hi | B_lo]
  static constexpr int CHUNK_COLS = 2 * BN;               // TMEM columns per k-block: [hi*hi | hi*lo + lo*hi]
  static constexpr int CHUNKS = 512 / CHUNK_COLS < 4 ? 512 / CHUNK_COLS : 4;
  static constexpr int STAGES = (200 * 1024) / STAGE_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

// One k-block = 8 MMAs. B_hi and B_lo sit back to back in the stage, so per k-step ONE MMA of width 2*BN
// forms A_hi * [B_hi ; B_lo] (columns [0, BN) = hi*hi, [BN, 2*BN) = hi*lo) and a second of width BN adds
// A_lo * B_hi onto the small-term columns. The large and the small products thus have accumulators
// of their own and meet in fp32 registers.
__device__ __forceinline__ void issue_split_kblock(uint32_t d_tmem, uint32_t bn, uint32_t sA_hi, uint32_t sA_lo, uint32_t sB,
                                                   uint32_t a_hi, uint32_t a_lbo, uint32_t a_adv, uint32_t b_hi,
                                                   uint32_t b_lbo, uint32_t b_adv, uint32_t idesc_wide, uint32_t idesc) {
  const uint32_t ah32 = ((sA_hi >> 4) & 0x3FFFu) | a_lbo;
  const uint32_t al32 = ((sA_lo >> 4) & 0x3FFFu) | a_lbo;
  const uint32_t b32 = ((sB >> 4) & 0x3FFFu) | b_lbo;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    const uint64_t adh = ((uint64_t)a_hi << 32) | (uint64_t)(ah32 + ks * a_adv);
    const uint64_t adl = ((uint64_t)a_hi << 32) | (uint64_t)(al32 + ks * a_adv);
    const uint64_t bd = ((uint64_t)b_hi << 32) | (uint64_t)(b32 + ks * b_adv);
    umma<true>(d_tmem, adh, bd, idesc_wide, ks != 0 ? 1u : 0u);
    umma<true>(d_tmem + bn, adl, bd, idesc, 1u);
  }
}

template <int BN, int ACT>
__global__ void __launch_bounds__(kF32Threads, 1)
conv_tc_f32_fwd_kernel(const __grid_constant__ CUtensorMap tmXh, const __grid_constant__ CUtensorMap tmXl,
                       const __grid_constant__ CUtensorMap tmWh, const __grid_constant__ CUtensorMap tmWl,
                       const __grid_constant__ ConvF32Params p) {
  using Cfg = ConvF32Cfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* chunk_full = bars + 2 * STAGES;   // [CHUNKS] MMA -> accumulating warps
  uint64_t* chunk_empty = chunk_full + Cfg::CHUNKS;     // [CHUNKS] accumulating warps -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(chunk_empty + Cfg::CHUNKS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_per_n = p.tiles_m * p.n_img;
  const int num_tiles = tiles_per_n * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < Cfg::CHUNKS; ++a) { mbar_init(&chunk_full[a], 1); mbar_init(&chunk_empty[a], 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, Cfg::CHUNKS * Cfg::CHUNK_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (m tile fastest, image, n tile)
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmXh); tma_prefetch_desc(&tmXl); tma_prefetch_desc(&tmWh); tma_prefetch_desc(&tmWl);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int t = tile % tiles_per_n, n0 = (tile / tiles_per_n) * BN;
        const int m0 = (t % p.tiles_m) * kF32BM, img = t / p.tiles_m;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, p.status, 0x1000u)) { ok = false; break; }
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES, sB = sA + 2 * Cfg::A_BYTES;
          const int c0 = m0 + p.a_shift[kb];
#pragma unroll
          for (int bx = 0; bx < 4; ++bx) {   // four boxes of 32 positions x 32 channels
            tma_load_4d(sA + bx * 4096, &tmXh, c0 + bx * 32, p.a_chan[kb], img, p.a_copy[kb], &full[stage]);
            tma_load_4d(sA + Cfg::A_BYTES + bx * 4096, &tmXl, c0 + bx * 32, p.a_chan[kb], img, p.a_copy[kb], &full[stage]);
          }
          tma_load_2d(sB, &tmWh, kb * 32, n0, &full[stage]);
          tma_load_2d(sB + Cfg::B_BYTES, &tmWl, kb * 32, n0, &full[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, ch = 0, ch_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&chunk_empty[ch], ch_phase ^ 1u, p.status, 0x2000u)) { ok = false; break; }
          if (!mbar_wait(&full[stage], phase, p.status, 0x4000u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES, sB = sA + 2 * Cfg::A_BYTES;
          issue_split_kblock(tmem_base + ch * Cfg::CHUNK_COLS, BN, sA, sA + Cfg::A_BYTES, sB, p.a_desc_hi, p.a_desc_lbo,
                             p.a_k_advance, p.b_desc_hi, p.b_desc_lbo, p.b_k_advance, p.idesc_wide, p.idesc);
          umma_commit(&empty[stage]);
          umma_commit(&chunk_full[ch]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          if (++ch == Cfg::CHUNKS) { ch = 0; ch_phase ^= 1u; }
        }
      }
    }
  } else if (warp >= 4) {
    // Two warps share each TMEM lane quarter and split the tile's columns. A thread owns one output
    // position s; consecutive lanes write consecutive s of one channel plane (128-byte runs).
    const int q = warp & 3, half = (warp - 4) >> 2;
    constexpr int COLS = BN / 2;
    uint32_t ch = 0, ch_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int t = tile % tiles_per_n, n0 = (tile / tiles_per_n) * BN;
      const int m0 = (t % p.tiles_m) * kF32BM, img = t / p.tiles_m;
      float sum[COLS];
#pragma unroll
      for (int j = 0; j < COLS; ++j) sum[j] = 0.f;
      for (int kb = 0; kb < p.num_kb; ++kb) {
        if (!mbar_wait_warp(&chunk_full[ch], ch_phase, p.status, 0x8000u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + ch * Cfg::CHUNK_COLS + half * COLS;
        uint32_t r[COLS], rs[COLS];   // hi*hi and the two small products
#pragma unroll
        for (int c = 0; c < COLS / 32; ++c) {
          tmem_ld32(t0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
          tmem_ld32(t0 + BN + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&rs[c * 32]));
        }
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&chunk_empty[ch]);
#pragma unroll
        for (int j = 0; j < COLS; ++j) sum[j] += __uint_as_float(rs[j]) + __uint_as_float(r[j]);
        if (++ch == Cfg::CHUNKS) { ch = 0; ch_phase ^= 1u; }
      }
      if (!ok) break;
      const int s = m0 + q * 32 + lane;
      if (s < p.S_out) {
        const int col0 = n0 + half * COLS;
        const int64_t cs = p.S_out;
        const int64_t base = (int64_t)s + cs * ((int64_t)p.n_out * img + col0);
        float* yp = p.y + base;
        float* pp = p.preact != nullptr ? p.preact + base : nullptr;
#pragma unroll
        for (int j = 0; j < COLS; ++j) {
          if (col0 + j < p.n_out) {
            const float v = sum[j] + (p.bias != nullptr ? __ldg(p.bias + col0 + j) : 0.f);
            if (pp != nullptr) pp[j * cs] = v;
            yp[j * cs] = act_apply_any<ACT, false>(p.act, v);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (*reinterpret_cast<volatile unsigned int*>(p.status) != 0) {
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::CHUNKS * Cfg::CHUNK_COLS);
  }
}

// ----------------------------------------------------------------------------------------------
// filter-gradient kernel
// ----------------------------------------------------------------------------------------------
// Row groups of 64 rows: rg = tap * chunks + chunk (64 input channels). An M tile stacks row groups
// 2j and 2j+1. A work item is (m tile, n tile, K split); a k-block is 32 output positions of one image.
struct ConvF32WgParams {
  int32_t S_out, n_img, n_out;
  int32_t s_blocks;                  // 32-position blocks per image
  int32_t m_tiles, tiles_n, splits;
  int32_t kb_total, kb_per_split;
  int32_t n_rg;
  uint32_t idesc, idesc_wide;
  uint32_t desc_hi, desc_lbo, k_advance;   // both operands K-major SW128
  float* partial;                    // [splits][m_tiles*128][n_pad]
  int32_t n_pad;
  unsigned int* status;
  int16_t rg_shift[kF32MaxRg];
  int16_t rg_chan[kF32MaxRg];
  int8_t rg_copy[kF32MaxRg];
};

template <int BN>
__global__ void __launch_bounds__(kF32Threads, 1)
conv_tc_f32_wgrad_kernel(const __grid_constant__ CUtensorMap tmXh, const __grid_constant__ CUtensorMap tmXl,
                         const __grid_constant__ CUtensorMap tmGh, const __grid_constant__ CUtensorMap tmGl,
                         const __grid_constant__ ConvF32WgParams p) {
  using Cfg = ConvF32Cfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* chunk_full = bars + 2 * STAGES;
  uint64_t* chunk_empty = chunk_full + Cfg::CHUNKS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(chunk_empty + Cfg::CHUNKS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_items = p.m_tiles * p.tiles_n * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < Cfg::CHUNKS; ++a) { mbar_init(&chunk_full[a], 1); mbar_init(&chunk_empty[a], 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, Cfg::CHUNKS * Cfg::CHUNK_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // item -> (m tile fastest, n tile, split)
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmXh); tma_prefetch_desc(&tmXl); tma_prefetch_desc(&tmGh); tma_prefetch_desc(&tmGl);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int mt = item % p.m_tiles, nt = (item / p.m_tiles) % p.tiles_n, z = item / (p.m_tiles * p.tiles_n);
        const int kb_lo = z * p.kb_per_split, kb_hi = min(p.kb_total, kb_lo + p.kb_per_split);
        const int rg0 = 2 * mt, rg1 = 2 * mt + 1;
        const bool two = rg1 < p.n_rg;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, p.status, 0x20000u)) { ok = false; break; }
          const int img = kb / p.s_blocks, s0 = (kb % p.s_blocks) * 32;
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES, sB = sA + 2 * Cfg::A_BYTES;
          mbar_expect_tx(&full[stage], (uint32_t)(2 * (Cfg::B_BYTES + (two ? Cfg::A_BYTES : Cfg::A_BYTES / 2))));
          tma_load_4d(sA, &tmXh, s0 + p.rg_shift[rg0], p.rg_chan[rg0], img, p.rg_copy[rg0], &full[stage]);
          tma_load_4d(sA + Cfg::A_BYTES, &tmXl, s0 + p.rg_shift[rg0], p.rg_chan[rg0], img, p.rg_copy[rg0], &full[stage]);
          if (two) {
            tma_load_4d(sA + Cfg::A_BYTES / 2, &tmXh, s0 + p.rg_shift[rg1], p.rg_chan[rg1], img, p.rg_copy[rg1], &full[stage]);
            tma_load_4d(sA + Cfg::A_BYTES + Cfg::A_BYTES / 2, &tmXl, s0 + p.rg_shift[rg1], p.rg_chan[rg1], img, p.rg_copy[rg1], &full[stage]);
          }
          tma_load_4d(sB, &tmGh, s0, nt * BN, img, 0, &full[stage]);
          tma_load_4d(sB + Cfg::B_BYTES, &tmGl, s0, nt * BN, img, 0, &full[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, ch = 0, ch_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int z = item / (p.m_tiles * p.tiles_n);
        const int kb_lo = z * p.kb_per_split, kb_hi = min(p.kb_total, kb_lo + p.kb_per_split);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&chunk_empty[ch], ch_phase ^ 1u, p.status, 0x40000u)) { ok = false; break; }
          if (!mbar_wait(&full[stage], phase, p.status, 0x80000u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES, sB = sA + 2 * Cfg::A_BYTES;
          issue_split_kblock(tmem_base + ch * Cfg::CHUNK_COLS, BN, sA, sA + Cfg::A_BYTES, sB, p.desc_hi, p.desc_lbo, p.k_advance,
                             p.desc_hi, p.desc_lbo, p.k_advance, p.idesc_wide, p.idesc);
          umma_commit(&empty[stage]);
          umma_commit(&chunk_full[ch]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          if (++ch == Cfg::CHUNKS) { ch = 0; ch_phase ^= 1u; }
        }
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3, half = (warp - 4) >> 2;
    constexpr int COLS = BN / 2;
    uint32_t ch = 0, ch_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const int mt = item % p.m_tiles, nt = (item / p.m_tiles) % p.tiles_n, z = item / (p.m_tiles * p.tiles_n);
      const int kb_lo = z * p.kb_per_split, kb_hi = min(p.kb_total, kb_lo + p.kb_per_split);
      float sum[COLS];
#pragma unroll
      for (int j = 0; j < COLS; ++j) sum[j] = 0.f;
      for (int kb = kb_lo; kb < kb_hi; ++kb) {
        if (!mbar_wait_warp(&chunk_full[ch], ch_phase, p.status, 0x100000u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + ch * Cfg::CHUNK_COLS + half * COLS;
        uint32_t r[COLS], rs[COLS];   // hi*hi and the two small products
#pragma unroll
        for (int c = 0; c < COLS / 32; ++c) {
          tmem_ld32(t0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
          tmem_ld32(t0 + BN + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&rs[c * 32]));
        }
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&chunk_empty[ch]);
#pragma unroll
        for (int j = 0; j < COLS; ++j) sum[j] += __uint_as_float(rs[j]) + __uint_as_float(r[j]);
        if (++ch == Cfg::CHUNKS) { ch = 0; ch_phase ^= 1u; }
      }
      if (!ok) break;
      const int row = mt * 128 + q * 32 + lane;
      float* dst = p.partial + ((int64_t)z * p.m_tiles * 128 + row) * p.n_pad + nt * BN + half * COLS;
      // A row group that was not loaded (odd tail) leaves stale shared memory under the MMA: its rows
      // are never read by the reduction, but they are written as zeros to keep the buffer defined.
      const bool live = (row / 64) < p.n_rg;
#pragma unroll
      for (int j = 0; j < COLS; ++j) dst[j] = live ? sum[j] : 0.f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (*reinterpret_cast<volatile unsigned int*>(p.status) != 0) {
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::CHUNKS * Cfg::CHUNK_COLS);
  }
}

// dw[kw,kh,ci,co] = sum over splits (ascending) of partial[z][row][ci]. The filter gradient is formed with the
// roles swapped (rows = taps of the DATA-gradient geometry x output channels, columns = input channels):
// row = ((K-1-th)*kW + (K-1-tw)) * chunks * 64 + co, with (tw, th) the forward tap of filter index (kw, kh).
__global__ void __launch_bounds__(256) conv_f32_wgrad_reduce_swapped_kernel(float* __restrict__ dw, const float* __restrict__ partial,
                                                                            int kW, int kH, int cin, int cout, int flip,
                                                                            int chunks, int rows_pad, int n_pad, int splits) {
  const int64_t total = (int64_t)kW * kH * cin * cout;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i;
    const int kw = (int)(r % kW); r /= kW;
    const int kh = (int)(r % kH); r /= kH;
    const int ci = (int)(r % cin);
    const int co = (int)(r / cin);
    const int tw = flip ? kw : kW - 1 - kw, th = flip ? kh : kH - 1 - kh;
    const int twp = kW - 1 - tw, thp = kH - 1 - th;
    const int rg = (thp * kW + twp) * chunks + co / 64;
    const int64_t row = (int64_t)rg * 64 + co % 64;
    float s = 0.f;
    for (int z = 0; z < splits; ++z) s += partial[((int64_t)z * rows_pad + row) * n_pad + ci];
    dw[i] = s;
  }
}

// ----------------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------------
namespace {

// One implicit-GEMM problem: out (W, Ho, Cn, N) = taps over in (W, Hi, Ck, N)
struct ConvGemmF32 {
  int W, Hi, Ho, Ck, Cn, N, kW, kH, pad_w, pad_h;
};

bool f32_map_4d(CUtensorMap* map, const void* ptr, int64_t d0, int64_t d1, int64_t d2, int64_t d3, int box0, int box1,
                bool atom32) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc) return false;
  cuuint64_t dims[4] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)d2, (cuuint64_t)d3};
  cuuint64_t strides[3] = {(cuuint64_t)d0 * 4, (cuuint64_t)d0 * d1 * 4, (cuuint64_t)d0 * d1 * d2 * 4};
  cuuint32_t box[4] = {(cuuint32_t)box0, (cuuint32_t)box1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool f32_map_2d(CUtensorMap* map, const void* ptr, int64_t d0, int64_t d1, int box0, int box1) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)d0, (cuuint64_t)d1};
  cuuint64_t strides[1] = {(cuuint64_t)d0 * 4};
  cuuint32_t box[2] = {(cuuint32_t)box0, (cuuint32_t)box1};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int f32_bn(int cn) { return cn <= 64 ? 64 : 128; }
int f32_chunks32(int ck) { return (ck + 31) / 32; }
int f32_chunks64(int ck) { return (ck + 63) / 64; }

bool f32_gemm_ok(const ConvGemmF32& c) {
  if (c.W % 4 != 0 || c.kW < 1 || c.kW > 8 || c.kH < 1) return false;
  if (c.kW * c.kH * f32_chunks32(c.Ck) > kF32MaxKb) return false;
  if ((int64_t)(c.kH + c.pad_h) * c.W > 32000) return false;
  if ((int64_t)c.W * c.Hi >= (1 << 30) || (int64_t)c.W * c.Ho >= (1 << 30)) return false;
  return tensor_map_encoder() != nullptr;
}

ConvGemmF32 f32_fwd_gemm(const ConvGeom& g) {
  return ConvGemmF32{g.in[0], g.in[1], g.out[1], g.cin, g.cout, g.batch, g.k[0], g.k[1], g.pad_lo[0], g.pad_lo[1]};
}
ConvGemmF32 f32_dgrad_gemm(const ConvGeom& g) {
  return ConvGemmF32{g.in[0], g.out[1], g.in[1], g.cout, g.cin, g.batch, g.k[0], g.k[1], g.k[0] - 1 - g.pad_lo[0], g.k[1] - 1 - g.pad_lo[1]};
}
PackGeomF32 f32_pack_geom(const ConvGeom& g, const ConvGemmF32& c, int transpose) {
  PackGeomF32 pg{};
  pg.kW = g.k[0]; pg.kH = g.k[1]; pg.cin = g.cin; pg.cout = g.cout; pg.flip = g.flip; pg.transpose = transpose;
  pg.chunks = f32_chunks32(c.Ck);
  const int bn = f32_bn(c.Cn);
  pg.n_rows = ((c.Cn + bn - 1) / bn) * bn;
  pg.k_total = c.kW * c.kH * pg.chunks * 32;
  return pg;
}

size_t f32_copy_bytes(const ConvGemmF32& c) { return align_up((size_t)c.kW * c.W * c.Hi * c.Ck * c.N * 4, 1024); }
size_t f32_packed_bytes(const ConvGemmF32& c) {
  const int bn = f32_bn(c.Cn);
  const size_t rows = (size_t)((c.Cn + bn - 1) / bn) * bn;
  return align_up(rows * (size_t)(c.kW * c.kH * f32_chunks32(c.Ck) * 32) * 4, 1024);
}
size_t f32_gemm_bytes(const ConvGemmF32& c) { return 2 * f32_copy_bytes(c) + 2 * f32_packed_bytes(c); }

unsigned f32_flat_grid(int64_t total) {
  int64_t gsz = (total + 255) / 256, cap = (int64_t)sm_count() * 16;
  return (unsigned)(gsz < 1 ? 1 : (gsz > cap ? cap : gsz));
}

// out = act(implicit GEMM + bias); workspace = copies hi | copies lo | filter hi | filter lo
void f32_make_copies(float* ch, float* cl, const float* in, const ConvGemmF32& c, cudaStream_t st) {
  const int64_t rows = (int64_t)c.Hi * c.Ck * c.N;
  conv_shift_split_kernel<<<f32_flat_grid(rows * (c.W / 4)), 256, 0, st>>>(ch, cl, in, c.W, rows, c.kW, c.pad_w);
}

int32_t run_f32_gemm(float* out, float* preact, const float* bias, int32_t act, const float* in, const float* w,
                     const ConvGemmF32& c, const PackGeomF32& pg, uint8_t* ws, cudaStream_t st, bool copies_ready = false) {
  float* ch = reinterpret_cast<float*>(ws);
  float* cl = reinterpret_cast<float*>(ws + f32_copy_bytes(c));
  float* wh = reinterpret_cast<float*>(ws + 2 * f32_copy_bytes(c));
  float* wl = reinterpret_cast<float*>(ws + 2 * f32_copy_bytes(c) + f32_packed_bytes(c));
  if (!copies_ready) f32_make_copies(ch, cl, in, c, st);
  conv_pack_split_filter_kernel<<<f32_flat_grid((int64_t)pg.n_rows * pg.k_total), 256, 0, st>>>(wh, wl, w, pg);
  LB2_CHECK_LAUNCH("conv_tc_f32 layout passes");

  const int bn = f32_bn(c.Cn);
  ConvF32Params p{};
  p.S_out = c.W * c.Ho;
  p.n_img = c.N;
  p.n_out = c.Cn;
  p.tiles_m = (p.S_out + kF32BM - 1) / kF32BM;
  p.tiles_n = (c.Cn + bn - 1) / bn;
  const int chunks = pg.chunks;
  p.num_kb = c.kW * c.kH * chunks;
  for (int kb = 0; kb < p.num_kb; ++kb) {
    const int tap = kb / chunks, tw = tap % c.kW, th = tap / c.kW;
    p.a_shift[kb] = (int16_t)((th - c.pad_h) * c.W);
    p.a_chan[kb] = (int16_t)((kb % chunks) * 32);
    p.a_copy[kb] = (int8_t)tw;
  }
  // A: tf32, MN-major, four boxes of (32 positions x 32 channels) in the 32-byte-atom 128-byte swizzle:
  // LBO = 4096 (next box), SBO = 512 (4 channel rows), 8 channels (1024 B) per MMA
  p.a_desc_hi = (uint32_t)((512u >> 4) & 0x3FFFu) | (1u << 14) | (1u << 29);
  p.a_desc_lbo = ((4096u >> 4) & 0x3FFFu) << 16;
  p.a_k_advance = 1024u >> 4;
  // B: tf32, K-major rows of 128 bytes: SBO = 1024, 32 bytes per MMA
  p.b_desc_hi = (uint32_t)((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
  p.b_desc_lbo = 1u << 16;
  p.b_k_advance = 32u >> 4;
  p.idesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (0u << 16) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(kF32BM >> 4) << 24);
  p.idesc_wide = (p.idesc & ~(0x3Fu << 17)) | ((uint32_t)((2 * bn) >> 3) << 17);
  p.y = out; p.preact = preact; p.bias = bias; p.act = act;
  p.status = device_status_word();
  LB2_REQUIRE(p.status != nullptr, LB2_LAUNCH_FAIL, "conv_tc_f32: device status word unavailable");
  CUtensorMap mXh, mXl, mWh, mWl;
  if (!f32_map_4d(&mXh, ch, (int64_t)c.W * c.Hi, c.Ck, c.N, c.kW, 32, 32, true) ||
      !f32_map_4d(&mXl, cl, (int64_t)c.W * c.Hi, c.Ck, c.N, c.kW, 32, 32, true) ||
      !f32_map_2d(&mWh, wh, pg.k_total, pg.n_rows, 32, bn) || !f32_map_2d(&mWl, wl, pg.k_total, pg.n_rows, 32, bn))
    return fail(LB2_LAUNCH_FAIL, "conv_tc_f32: cuTensorMapEncodeTiled failed");
  const int num_tiles = p.tiles_m * p.n_img * p.tiles_n;
  const int grid = num_tiles < sm_count() ? num_tiles : sm_count();
  auto launch = [&](auto kernel, int smem) -> int32_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "conv_tc_f32: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    kernel<<<grid, kF32Threads, smem, st>>>(mXh, mXl, mWh, mWl, p);
    LB2_CHECK_LAUNCH("conv_tc_f32_fwd");
    return LB2_OK;
  };
  if (bn == 64) {
    switch (act) {
      case LB2_ACT_IDENTITY: return launch(conv_tc_f32_fwd_kernel<64, LB2_ACT_IDENTITY>, ConvF32Cfg<64>::SMEM_BYTES);
      case LB2_ACT_RELU: return launch(conv_tc_f32_fwd_kernel<64, LB2_ACT_RELU>, ConvF32Cfg<64>::SMEM_BYTES);
      default: return launch(conv_tc_f32_fwd_kernel<64, -1>, ConvF32Cfg<64>::SMEM_BYTES);
    }
  }
  switch (act) {
    case LB2_ACT_IDENTITY: return launch(conv_tc_f32_fwd_kernel<128, LB2_ACT_IDENTITY>, ConvF32Cfg<128>::SMEM_BYTES);
    case LB2_ACT_RELU: return launch(conv_tc_f32_fwd_kernel<128, LB2_ACT_RELU>, ConvF32Cfg<128>::SMEM_BYTES);
    default: return launch(conv_tc_f32_fwd_kernel<128, -1>, ConvF32Cfg<128>::SMEM_BYTES);
  }
}

struct WgPlanF32 {
  int bn, chunks, n_rg, m_tiles, tiles_n, s_blocks, kb_total, splits, kb_per_split, n_pad;
};
size_t f32_wg_partial_bytes(const WgPlanF32& w) {
  return align_up((size_t)w.splits * w.m_tiles * 128 * w.n_pad * sizeof(float), 1024);
}
size_t f32_y_bytes(const ConvGeom& g) { return align_up((size_t)g.out[0] * g.out[1] * g.cout * g.batch * 4, 1024); }
size_t f32_x_bytes(const ConvGeom& g) { return align_up((size_t)g.in[0] * g.in[1] * g.cin * g.batch * 4, 1024); }

// Filter gradient with the roles swapped: rows = (tap of the data-gradient geometry, output channel) from the
// W-shifted copies of g that the data gradient needs anyway, columns = input channels from a flat split of x.
WgPlanF32 f32_wg_plan_swapped(const ConvGeom& g) {
  WgPlanF32 w{};
  w.bn = f32_bn(g.cin);
  w.chunks = f32_chunks64(g.cout);
  w.n_rg = g.k[0] * g.k[1] * w.chunks;
  w.m_tiles = (w.n_rg + 1) / 2;
  w.tiles_n = (g.cin + w.bn - 1) / w.bn;
  w.n_pad = w.tiles_n * w.bn;
  const int S_in = g.in[0] * g.in[1];
  w.s_blocks = (S_in + 31) / 32;
  w.kb_total = g.batch * w.s_blocks;
  int splits = sm_count() / (w.m_tiles * w.tiles_n);
  if (splits < 1) splits = 1;
  if (splits > w.kb_total) splits = w.kb_total;
  w.kb_per_split = (w.kb_total + splits - 1) / splits;
  w.splits = (w.kb_total + w.kb_per_split - 1) / w.kb_per_split;
  return w;
}

}  // namespace

bool conv_tc_f32_supported(const ConvGeom& g) {
  if (g.ndim != 2 || g.groups != 1) return false;
  if (g.stride[0] != 1 || g.stride[1] != 1 || g.dil[0] != 1 || g.dil[1] != 1) return false;
  if (g.out[0] != g.in[0] || g.out[0] <= 0 || g.out[1] <= 0 || g.batch <= 0 || g.cin <= 0 || g.cout <= 0) return false;
  if (g.pad_lo[0] > g.k[0] - 1 || g.pad_lo[1] > g.k[1] - 1) return false;  // data gradient needs K-1-pad >= 0
  if (!f32_gemm_ok(f32_fwd_gemm(g)) || !f32_gemm_ok(f32_dgrad_gemm(g))) return false;
  if (g.k[0] * g.k[1] * f32_chunks64(g.cin) > kF32MaxRg || g.k[0] * g.k[1] * f32_chunks64(g.cout) > kF32MaxRg) return false;
  return true;
}

size_t conv_tc_f32_fwd_workspace_bytes(const ConvGeom& g) { return f32_gemm_bytes(f32_fwd_gemm(g)); }

// backward workspace: g copies hi | lo | packed filter hi | lo (the data-gradient GEMM's layout) | x hi | x lo | partials
size_t conv_tc_f32_bwd_workspace_bytes(const ConvGeom& g) {
  return f32_gemm_bytes(f32_dgrad_gemm(g)) + 2 * f32_x_bytes(g) + f32_wg_partial_bytes(f32_wg_plan_swapped(g));
}

int32_t conv_tc_f32_fwd(void* y, void* preact, const void* x, const void* w, const void* bias, const ConvGeom& g,
                        int32_t act, void* ws, cudaStream_t st) {
  const ConvGemmF32 c = f32_fwd_gemm(g);
  return run_f32_gemm((float*)y, (float*)preact, (const float*)bias, act, (const float*)x, (const float*)w, c,
                      f32_pack_geom(g, c, 0), static_cast<uint8_t*>(ws), st);
}

// Both gradients from ONE set of W-shifted hi/lo copies of g: the data gradient reads them as its A operand;
// the filter gradient sum_s x[s + shift(tap)] * g[s] is rewritten as sum_s' x[s'] * g[s' - shift(tap)], which is
// the same copies at the data-gradient tap (K-1-tw, K-1-th), stacked along M, against a flat split of x.
int32_t conv_tc_f32_bwd(void* dw, void* dx, const void* x, const void* gy, const void* w, const ConvGeom& g, void* ws_,
                        cudaStream_t st) {
  uint8_t* ws = static_cast<uint8_t*>(ws_);
  const ConvGemmF32 d = f32_dgrad_gemm(g);
  float* ch = reinterpret_cast<float*>(ws);
  float* cl = reinterpret_cast<float*>(ws + f32_copy_bytes(d));
  f32_make_copies(ch, cl, (const float*)gy, d, st);
  LB2_CHECK_LAUNCH("conv_tc_f32 shifted copies");
  if (dx != nullptr) {
    int32_t rc = run_f32_gemm((float*)dx, nullptr, nullptr, LB2_ACT_IDENTITY, (const float*)gy, (const float*)w, d,
                              f32_pack_geom(g, d, 1), ws, st, true);
    if (rc != LB2_OK) return rc;
  }
  if (dw == nullptr) return LB2_OK;
  const WgPlanF32 w_ = f32_wg_plan_swapped(g);
  float* xh = reinterpret_cast<float*>(ws + f32_gemm_bytes(d));
  float* xl = reinterpret_cast<float*>(ws + f32_gemm_bytes(d) + f32_x_bytes(g));
  float* partial = reinterpret_cast<float*>(ws + f32_gemm_bytes(d) + 2 * f32_x_bytes(g));
  const int64_t nx = (int64_t)g.in[0] * g.in[1] * g.cin * g.batch;
  conv_split_flat_kernel<<<f32_flat_grid(nx / 4 + 1), 256, 0, st>>>(xh, xl, (const float*)x, nx);
  LB2_CHECK_LAUNCH("conv_tc_f32 split of x");
  ConvF32WgParams p{};
  p.S_out = g.in[0] * g.in[1];          // contraction extent: input positions
  p.n_img = g.batch; p.n_out = g.cin;
  p.s_blocks = w_.s_blocks; p.m_tiles = w_.m_tiles; p.tiles_n = w_.tiles_n; p.splits = w_.splits;
  p.kb_total = w_.kb_total; p.kb_per_split = w_.kb_per_split; p.n_rg = w_.n_rg;
  p.idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(w_.bn >> 3) << 17) | ((uint32_t)(kF32BM >> 4) << 24);
  p.idesc_wide = (p.idesc & ~(0x3Fu << 17)) | ((uint32_t)((2 * w_.bn) >> 3) << 17);
  p.desc_hi = (uint32_t)((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
  p.desc_lbo = 1u << 16;
  p.k_advance = 32u >> 4;
  p.partial = partial; p.n_pad = w_.n_pad;
  p.status = device_status_word();
  LB2_REQUIRE(p.status != nullptr, LB2_LAUNCH_FAIL, "conv_tc_f32: device status word unavailable");
  for (int rg = 0; rg < w_.n_rg; ++rg) {
    const int tap = rg / w_.chunks, twp = tap % d.kW, thp = tap / d.kW;   // tap of the data-gradient geometry
    p.rg_shift[rg] = (int16_t)((thp - d.pad_h) * d.W);
    p.rg_chan[rg] = (int16_t)((rg % w_.chunks) * 64);
    p.rg_copy[rg] = (int8_t)twp;
  }
  CUtensorMap mGh, mGl, mXh, mXl;
  if (!f32_map_4d(&mGh, ch, (int64_t)d.W * d.Hi, d.Ck, d.N, d.kW, 32, 64, false) ||
      !f32_map_4d(&mGl, cl, (int64_t)d.W * d.Hi, d.Ck, d.N, d.kW, 32, 64, false) ||
      !f32_map_4d(&mXh, xh, (int64_t)p.S_out, g.cin, g.batch, 1, 32, w_.bn, false) ||
      !f32_map_4d(&mXl, xl, (int64_t)p.S_out, g.cin, g.batch, 1, 32, w_.bn, false))
    return fail(LB2_LAUNCH_FAIL, "conv_tc_f32: cuTensorMapEncodeTiled failed");
  const int items = w_.m_tiles * w_.tiles_n * w_.splits;
  const int grid = items < sm_count() ? items : sm_count();
  auto launch = [&](auto kernel, int smem) -> int32_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "conv_tc_f32: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    kernel<<<grid, kF32Threads, smem, st>>>(mGh, mGl, mXh, mXl, p);
    LB2_CHECK_LAUNCH("conv_tc_f32_wgrad");
    return LB2_OK;
  };
  int32_t rc = w_.bn == 64 ? launch(conv_tc_f32_wgrad_kernel<64>, ConvF32Cfg<64>::SMEM_BYTES)
                           : launch(conv_tc_f32_wgrad_kernel<128>, ConvF32Cfg<128>::SMEM_BYTES);
  if (rc != LB2_OK) return rc;
  const int64_t nw = (int64_t)g.k[0] * g.k[1] * g.cin * g.cout;
  conv_f32_wgrad_reduce_swapped_kernel<<<f32_flat_grid(nw), 256, 0, st>>>((float*)dw, partial, g.k[0], g.k[1], g.cin, g.cout, g.flip,
                                                                          w_.chunks, w_.m_tiles * 128, w_.n_pad, w_.splits);
  LB2_CHECK_LAUNCH("conv_f32_wgrad_reduce");
  return LB2_OK;
}

}  // namespace lb2

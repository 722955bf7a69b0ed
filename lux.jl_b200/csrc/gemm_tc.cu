// Tensor-core GEMM for sm_100a: TMA -> 128B-swizzled shared-memory ring -> tcgen05.mma with the
// accumulator in TMEM -> tcgen05.ld epilogue with bias + activation fused.
//
//   D[Mm x Nn] = A[Mm x Kc] * B[Nn x Kc]^T      (D column-major, Mm contiguous)
//
// One persistent CTA per SM, 384 threads, warp-specialised:
//   warp 0      TMA producer (one elected lane): fills a ring of STAGES {A,B} k-blocks
//   warp 1      MMA issuer  (one elected lane): 4 tcgen05.mma (K=16 bf16 / K=8 tf32) per k-block,
//               tcgen05.commit releases the smem stage / publishes the accumulator
//   warp 2      TMEM allocator (512 columns = two 128 x BN fp32 accumulators, so the epilogue of
//               tile i overlaps the main loop of tile i+1)
//   warps 4-11  epilogue, two warps per TMEM lane quarter, each taking half of the tile's columns:
//               tcgen05.ld 32 lanes x 32 columns -> +bias -> activation -> global
//               (lane = output row = contiguous index of D, so every warp store is a 64/128-byte run)
// Operands may be K-major or MN-major in global memory; both are fetched with tiled TMA boxes
// of 128-byte rows (SWIZZLE_128B) and described to the MMA through the matching shared-memory
// matrix descriptor, so no transposition pass ever runs. fp32 storage uses kind::tf32, by default
// as an error-compensated 3-product split (hi*hi + lo*hi + hi*lo) with per-k-block accumulation in
// registers (gemm_tc_f32acc_kernel) that restores fp32 accuracy. Large bf16 / single-pass tf32 problems
// run on the CTA-pair kernel (gemm_tc_pair_kernel: cta_group::2, one 256 x 256 tile per pair of SMs).
// No TMA load uses multicast. Every mbarrier wait is bounded; on expiry the kernel sets
// a status word, drains and returns, and the host reports LB2_TIMEOUT from lb2_poll_device_status.
//
// Roofline: tensor-pipe bound; algorithmic FLOPs = 2*Mm*Nn*Kc per launch.
#include <cuda.h>

#include <mutex>

#include "gemm.cuh"
#include "tc_ptx.cuh"

namespace lb2 {

// ----------------------------------------------------------------------------------------------
// kernel
// ----------------------------------------------------------------------------------------------
// How one operand tile is fetched and described (filled in on the host).
struct OperandPlan {
  int32_t boxes;        // TMA boxes per k-block
  int32_t box_bytes;    // bytes each box lands in shared memory
  int32_t mn_step;      // MN-major: elements of the MN extent covered by one box; K-major: unused
  int32_t mn_major;     // 1: coordinates are {mn, k}; 0: {k, mn}
  uint32_t desc_hi;     // upper 32 bits of the UMMA smem descriptor (SBO, version, swizzle)
  uint32_t desc_lbo;    // LBO field already shifted into bits [16,30) of the lower word
  uint32_t k_advance;   // descriptor start-address increment (bytes >> 4) per MMA k-step
};

struct TcParams {
  OperandPlan a, b;
  int64_t Mm, Nn, Kc;
  int32_t bk;           // elements of K per k-block (64 bf16 / 32 tf32)
  int32_t tiles_m, tiles_n, num_kb;
  uint32_t idesc;
  void* D;
  int64_t ldd;
  const void* bias;
  void* preact;
  int32_t act, accumulate;
  unsigned int* status;
  int32_t raster_h;     // tiles are walked in bands of this many tile rows (see tile_coords)
  // CTA-pair kernel only: work slots [0, full_slots) are whole 256 x 256 tiles; slots [full_slots, total_slots) are the
  // two 128-column halves of the tiles that would otherwise form a partly filled last wave (see pair_slot)
  int32_t full_slots, total_slots;
  uint32_t idesc_half;  // instruction descriptor of a half tile (N = 128)
};

// Tile order. Walking all tile rows of one tile column before the next makes the CTAs that run at the same time
// share one B panel but touch every A panel; for long contractions that working set falls out of L2 between
// waves. Tiles are walked in bands of `raster_h` tile rows instead (row index fastest inside a band), so the
// tiles in flight cover a roughly square block of the output and consecutive waves reuse the band's A panels.
__device__ __forceinline__ void tile_coords(const TcParams& p, int tile, int* tm, int* tn) {
  const int band_tiles = p.raster_h * p.tiles_n;
  const int band = tile / band_tiles;
  const int in_band = tile - band * band_tiles;
  const int rows_left = p.tiles_m - band * p.raster_h;
  const int h = rows_left < p.raster_h ? rows_left : p.raster_h;
  *tm = band * p.raster_h + in_band % h;
  *tn = in_band / h;
}

// Work slot of the CTA-pair kernel -> (tile, half). A persistent grid of C pairs walks T tiles in ceil(T / C) waves,
// and the last wave is as long as the others however few tiles it holds (256 tiles on 74 pairs: 3.46 waves of work in
// the time of 4). When the T mod C leftover tiles are at most C / 2, each of them is issued as two 128-column halves to
// two different pairs instead: the last wave then takes half the time. A half tile loads all of A and half of the B
// boxes (which is why this needs an MN-major B, whose tile arrives as several 64-wide boxes) and issues MMAs of N = 128.
__device__ __forceinline__ void pair_slot(const TcParams& p, int slot, int* tile, int* halved, int* which) {
  if (slot < p.full_slots) { *tile = slot; *halved = 0; *which = 0; return; }
  const int h = slot - p.full_slots;
  *tile = p.full_slots + (h >> 1);
  *halved = 1;
  *which = h & 1;
}

constexpr int kBM = 128;
constexpr int kKSteps = 4;  // MMA k-steps per k-block (128 bytes of K per row / 32 bytes per step)

template <int BN, bool TF32, bool SPLIT3> struct TcCfg {
  static constexpr int A_BYTES = kBM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = (A_BYTES + B_BYTES) * (SPLIT3 ? 2 : 1);
  static constexpr int STAGES = (200 * 1024) / STAGE_BYTES < 8 ? (200 * 1024) / STAGE_BYTES : 8;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

constexpr int kThreadsSingle = 384;  // warps 0-2: TMA / MMA / TMEM, warps 4-11: epilogue (two per TMEM lane quarter)

template <int BN, bool TF32, bool SPLIT3, int ACT, typename OutT>
__global__ void __launch_bounds__(kThreadsSingle, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmA_lo, const __grid_constant__ CUtensorMap tmB_lo,
               const __grid_constant__ TcParams p) {
  using Cfg = TcCfg<BN, TF32, SPLIT3>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr bool FAST = sizeof(OutT) == 2;
  extern __shared__ uint8_t smem_raw[];
  // SWIZZLE_128B tiles must start on 1024-byte boundaries
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;                    // [STAGES]  TMA -> MMA
  uint64_t* empty = bars + STAGES;          // [STAGES]  MMA -> TMA
  uint64_t* acc_full = bars + 2 * STAGES;   // [2]       MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;       // [2]       epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if constexpr (SPLIT3) { tma_prefetch_desc(&tmA_lo); tma_prefetch_desc(&tmB_lo); }
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(p, tile, &tm, &tn);
        const int m0 = tm * kBM, n0 = tn * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, p.status, 0x1u)) { ok = false; break; }
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          const int k0 = kb * p.bk;
          for (int bx = 0; bx < p.a.boxes; ++bx) {
            const int32_t c0 = p.a.mn_major ? m0 + bx * p.a.mn_step : k0;
            const int32_t c1 = p.a.mn_major ? k0 : m0;
            tma_load_2d(sA + bx * p.a.box_bytes, &tmA, c0, c1, &full[stage]);
            if constexpr (SPLIT3) tma_load_2d(sA + Cfg::A_BYTES + Cfg::B_BYTES + bx * p.a.box_bytes, &tmA_lo, c0, c1, &full[stage]);
          }
          for (int bx = 0; bx < p.b.boxes; ++bx) {
            const int32_t c0 = p.b.mn_major ? n0 + bx * p.b.mn_step : k0;
            const int32_t c1 = p.b.mn_major ? k0 : n0;
            tma_load_2d(sB + bx * p.b.box_bytes, &tmB, c0, c1, &full[stage]);
            if constexpr (SPLIT3) tma_load_2d(sB + Cfg::A_BYTES + Cfg::B_BYTES + bx * p.b.box_bytes, &tmB_lo, c0, c1, &full[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, p.status, 0x2u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, p.status, 0x4u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          const uint32_t a_lo32 = ((sA >> 4) & 0x3FFFu) | p.a.desc_lbo;
          const uint32_t b_lo32 = ((sB >> 4) & 0x3FFFu) | p.b.desc_lbo;
          constexpr uint32_t LO_OFF = (Cfg::A_BYTES + Cfg::B_BYTES) >> 4;
#pragma unroll
          for (int ks = 0; ks < kKSteps; ++ks) {
            const uint64_t ad = ((uint64_t)p.a.desc_hi << 32) | (uint64_t)(a_lo32 + ks * p.a.k_advance);
            const uint64_t bd = ((uint64_t)p.b.desc_hi << 32) | (uint64_t)(b_lo32 + ks * p.b.k_advance);
            umma<TF32>(d_tmem, ad, bd, p.idesc, (kb | ks) != 0 ? 1u : 0u);
            if constexpr (SPLIT3) {
              umma<TF32>(d_tmem, ad + LO_OFF, bd, p.idesc, 1u);  // lo(A) * hi(B)
              umma<TF32>(d_tmem, ad, bd + LO_OFF, p.idesc, 1u);  // hi(A) * lo(B)
            }
          }
          umma_commit(&empty[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp >= 4) {
    // ---------------- epilogue ----------------
    // Two warps share each TMEM lane quarter and split the tile's columns. A thread owns output row m
    // (the contiguous index of D) and walks its columns with a pointer stride of ldd.
    const int q = warp & 3, half = (warp - 4) >> 2;
    constexpr int COLS = BN / 2;
    uint32_t acc = 0, acc_phase = 0;
    OutT* D = reinterpret_cast<OutT*>(p.D);
    OutT* P = reinterpret_cast<OutT*>(p.preact);
    const OutT* bias = reinterpret_cast<const OutT*>(p.bias);
    const int64_t ldd = p.ldd;
    const bool accumulate = p.accumulate != 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(p, tile, &tm, &tn);
      const int m0 = tm * kBM, n0 = tn * BN + half * COLS;
      if (!mbar_wait_warp(&acc_full[acc], acc_phase, p.status, 0x8u)) { ok = false; break; }
      tc_fence_after();
      const int64_t m = (int64_t)m0 + q * 32 + lane;
      const bool m_ok = m < p.Mm;
      float bv = 0.f;
      if (bias != nullptr && m_ok) bv = to_f32(bias[m]);
      const int64_t rem = p.Nn - n0;
      const int lim = rem < COLS ? (int)rem : COLS;   // live columns (may be <= 0)
      OutT* dp = D + (int64_t)n0 * ldd + m;
      OutT* pp = P != nullptr ? P + (int64_t)n0 * ldd + m : nullptr;
#pragma unroll 1
      for (int c = 0; c < COLS / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + half * COLS + c * 32, r);
        tmem_ld_wait();
        if (m_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c * 32 + j < lim) {
              float v = __uint_as_float(r[j]) + bv;
              if (pp != nullptr) pp[j * ldd] = from_f32<OutT>(v);
              v = act_apply_any<ACT, FAST>(p.act, v);
              if (accumulate) v += to_f32(dp[j * ldd]);
              dp[j * ldd] = from_f32<OutT>(v);
            }
          }
        }
        dp += 32 * ldd;
        if (pp != nullptr) pp += 32 * ldd;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    // After an expired wait, copies may still be landing: give them a bounded moment first.
    if (*reinterpret_cast<volatile unsigned int*>(p.status) != 0) {
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ----------------------------------------------------------------------------------------------
// fp32-accurate kernel (3xTF32 with register accumulation).
// The tensor core adds into its TMEM accumulator with truncation, and that error grows linearly
// with the number of accumulating MMAs (measured: ~1e-7 relative per MMA, 1.9e-5 at K = 512 when a
// whole K loop accumulates in TMEM). Here TMEM only ever holds ONE k-block's worth of products
// (12 MMAs: hi*hi, lo*hi, hi*lo over 4 k-steps): after every k-block the eight epilogue warps pull
// the 128 x 128 partial out of TMEM (two chunk buffers, so the next k-block's MMAs overlap) and add
// it, round-to-nearest, into fp32 registers (64 per thread). Bias, activation and the store happen
// once per tile from those registers. 128 x 128 tiles, 3 stages of {A_hi, B_hi, A_lo, B_lo}.
// ----------------------------------------------------------------------------------------------
constexpr int kAccThreads = 384;  // warps 0-2 as in the other kernels, warps 4-11 accumulate + epilogue
constexpr int kAccBN = 128;

template <int ACT>
__global__ void __launch_bounds__(kAccThreads, 1)
gemm_tc_f32acc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmA_lo, const __grid_constant__ CUtensorMap tmB_lo,
                      const __grid_constant__ TcParams p) {
  using Cfg = TcCfg<kAccBN, true, true>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int BN = kAccBN;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* chunk_full = bars + 2 * STAGES;   // [2] MMA -> accumulating warps (one k-block of products is in TMEM)
  uint64_t* chunk_empty = chunk_full + 2;     // [2] accumulating warps -> MMA (chunk buffer may be overwritten)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(chunk_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&chunk_full[a], 1); mbar_init(&chunk_empty[a], 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmA_lo); tma_prefetch_desc(&tmB_lo);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(p, tile, &tm, &tn);
        const int m0 = tm * kBM, n0 = tn * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, p.status, 0x100u)) { ok = false; break; }
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          constexpr uint32_t LO = Cfg::A_BYTES + Cfg::B_BYTES;
          const int k0 = kb * p.bk;
          for (int bx = 0; bx < p.a.boxes; ++bx) {
            const int32_t c0 = p.a.mn_major ? m0 + bx * p.a.mn_step : k0;
            const int32_t c1 = p.a.mn_major ? k0 : m0;
            tma_load_2d(sA + bx * p.a.box_bytes, &tmA, c0, c1, &full[stage]);
            tma_load_2d(sA + LO + bx * p.a.box_bytes, &tmA_lo, c0, c1, &full[stage]);
          }
          for (int bx = 0; bx < p.b.boxes; ++bx) {
            const int32_t c0 = p.b.mn_major ? n0 + bx * p.b.mn_step : k0;
            const int32_t c1 = p.b.mn_major ? k0 : n0;
            tma_load_2d(sB + bx * p.b.box_bytes, &tmB, c0, c1, &full[stage]);
            tma_load_2d(sB + LO + bx * p.b.box_bytes, &tmB_lo, c0, c1, &full[stage]);
          }
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
          if (!mbar_wait(&chunk_empty[ch], ch_phase ^ 1u, p.status, 0x200u)) { ok = false; break; }
          if (!mbar_wait(&full[stage], phase, p.status, 0x400u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + ch * BN;
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          const uint32_t a_lo32 = ((sA >> 4) & 0x3FFFu) | p.a.desc_lbo;
          const uint32_t b_lo32 = ((sB >> 4) & 0x3FFFu) | p.b.desc_lbo;
          constexpr uint32_t LO_OFF = (Cfg::A_BYTES + Cfg::B_BYTES) >> 4;
          // small terms first, so the large hi*hi products are added last
#pragma unroll
          for (int ks = 0; ks < kKSteps; ++ks) {
            const uint64_t ad = ((uint64_t)p.a.desc_hi << 32) | (uint64_t)(a_lo32 + ks * p.a.k_advance);
            const uint64_t bd = ((uint64_t)p.b.desc_hi << 32) | (uint64_t)(b_lo32 + ks * p.b.k_advance);
            umma<true>(d_tmem, ad + LO_OFF, bd, p.idesc, ks != 0 ? 1u : 0u);
            umma<true>(d_tmem, ad, bd + LO_OFF, p.idesc, 1u);
          }
#pragma unroll
          for (int ks = 0; ks < kKSteps; ++ks) {
            const uint64_t ad = ((uint64_t)p.a.desc_hi << 32) | (uint64_t)(a_lo32 + ks * p.a.k_advance);
            const uint64_t bd = ((uint64_t)p.b.desc_hi << 32) | (uint64_t)(b_lo32 + ks * p.b.k_advance);
            umma<true>(d_tmem, ad, bd, p.idesc, 1u);
          }
          umma_commit(&empty[stage]);
          umma_commit(&chunk_full[ch]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          if (++ch == 2) { ch = 0; ch_phase ^= 1u; }
        }
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3;             // TMEM lane quarter
    const int half = (warp - 4) >> 2;   // which 64 of the tile's 128 columns
    uint32_t ch = 0, ch_phase = 0;
    float* D = reinterpret_cast<float*>(p.D);
    float* P = reinterpret_cast<float*>(p.preact);
    const float* bias = reinterpret_cast<const float*>(p.bias);
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(p, tile, &tm, &tn);
      const int m0 = tm * kBM, n0 = tn * BN;
      float sum[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) sum[j] = 0.f;
      for (int kb = 0; kb < p.num_kb; ++kb) {
        if (!mbar_wait_warp(&chunk_full[ch], ch_phase, p.status, 0x800u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + ch * BN + half * 64;
        uint32_t r0[32], r1[32];
        tmem_ld32(t0, r0);
        tmem_ld32(t0 + 32, r1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&chunk_empty[ch]);
#pragma unroll
        for (int j = 0; j < 32; ++j) { sum[j] += __uint_as_float(r0[j]); sum[32 + j] += __uint_as_float(r1[j]); }
        if (++ch == 2) { ch = 0; ch_phase ^= 1u; }
      }
      if (!ok) break;
      const int64_t m = (int64_t)m0 + q * 32 + lane;
      if (m < p.Mm) {
        const float bv = bias != nullptr ? bias[m] : 0.f;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const int64_t n = (int64_t)n0 + half * 64 + j;
          if (n < p.Nn) {
            float v = sum[j] + bv;
            const int64_t off = n * p.ldd + m;
            if (P != nullptr) P[off] = v;
            v = act_apply_any<ACT, false>(p.act, v);
            if (p.accumulate) v += D[off];
            D[off] = v;
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
    tmem_dealloc(tmem_base, 256);
  }
}

// ----------------------------------------------------------------------------------------------
// CTA-pair kernel: the two CTAs of a cluster (two SMs of one TPC) work on one 256 x 256 tile with
// tcgen05.mma.cta_group::2. Per 64-deep k-block each CTA loads its own 128 rows of A and its own 128 of the
// tile's 256 B rows: 32 KB for 512 tensor-pipe cycles of work, where a lone CTA on a 128 x 256 tile needs
// 48 KB, and the tensor core of each SM reads only half of B from its own shared memory. Operand fill plus
// operand reads then fit the shared-memory bandwidth of an SM, which is what bounds the single-CTA kernel.
// Each CTA keeps its 128 x 256 half of the accumulator in its own TMEM (two buffers, so the epilogue of
// tile i runs under the main loop of tile i+1) and runs its own eight-warp epilogue.
// The leader CTA (cluster rank 0) issues every MMA. Synchronisation per stage:
//   full[s]   (the leader's)  one arrive.expect_tx by the leader's producer for BOTH CTAs' bytes; the
//             partner's TMA loads carry cta_group::2 and complete their bytes on the leader's barrier
//   empty[s]  (one per CTA)   ONE tcgen05.commit with a cluster-multicast mask arrives on both CTAs' barriers
//             once the MMAs that read the stage have finished
//   acc_full  (one per CTA)   the same multicast commit after a tile's last MMA
//   acc_empty (the leader's)  one arrival per CTA, sent by one thread after that CTA's epilogue warps have
//             met at a named barrier (the partner's arrival is a remote mbarrier arrive)
// The multicast here is an mbarrier arrival, not a load. All waits are time-bounded.
// ----------------------------------------------------------------------------------------------
constexpr int kPairBN = 256;
constexpr int kPairThreads = 384;   // warps 0-2: TMA / MMA / TMEM; warps 4-11: epilogue

struct PairCfg {
  static constexpr int A_BYTES = kBM * 128;       // this CTA's 128 rows of A
  static constexpr int B_BYTES = kBM * 128;       // this CTA's 128 of the tile's 256 B rows
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 7;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <bool TF32, int ACT, typename OutT>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ TcParams p) {
  using Cfg = PairCfg;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int BN = kPairBN;
  constexpr bool FAST = sizeof(OutT) == 2;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;                    // [STAGES]  both CTAs' TMA -> leader's MMA (the leader's copy is used)
  uint64_t* empty = bars + STAGES;          // [STAGES]  MMA -> this CTA's TMA producer
  uint64_t* acc_full = bars + 2 * STAGES;   // [2]       MMA -> this CTA's epilogue
  uint64_t* acc_empty = acc_full + 2;       // [2]       both CTAs' epilogues -> leader's MMA (the leader's copy)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();        // 0 = leader
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 2); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();   // barriers of both CTAs are initialised before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA) ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int slot = cluster_id; slot < p.total_slots && ok; slot += num_clusters) {
        int tile, halved, which, tm, tn;
        pair_slot(p, slot, &tile, &halved, &which);
        tile_coords(p, tile, &tm, &tn);
        const int bn_eff = halved ? BN / 2 : BN;                 // columns of this work item
        const int b_boxes = halved ? p.b.boxes / 2 : p.b.boxes;  // B boxes this CTA loads per k-block
        const int m0 = tm * (2 * kBM) + (int)rank * kBM;
        const int n0 = tn * BN + which * (BN / 2) + (int)rank * (bn_eff / 2);
        const uint32_t stage_tx = 2u * (uint32_t)(Cfg::A_BYTES + b_boxes * p.b.box_bytes);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, p.status, 0x10u)) { ok = false; break; }
          const uint32_t leader_full = map_to_cta(smem_u32(&full[stage]), 0);
          // The partner's bytes may be counted before this arrive (the transaction count then goes negative for
          // a moment); the phase cannot complete before it, because it is the barrier's only pending arrival.
          if (rank == 0) mbar_expect_tx(&full[stage], stage_tx);
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          const int k0 = kb * p.bk;
          for (int bx = 0; bx < p.a.boxes; ++bx) {
            const int32_t c0 = p.a.mn_major ? m0 + bx * p.a.mn_step : k0;
            const int32_t c1 = p.a.mn_major ? k0 : m0;
            tma_load_2d_pair(sA + bx * p.a.box_bytes, &tmA, c0, c1, leader_full);
          }
          for (int bx = 0; bx < b_boxes; ++bx) {
            const int32_t c0 = p.b.mn_major ? n0 + bx * p.b.mn_step : k0;
            const int32_t c1 = p.b.mn_major ? k0 : n0;
            tma_load_2d_pair(sB + bx * p.b.box_bytes, &tmB, c0, c1, leader_full);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int slot = cluster_id; slot < p.total_slots && ok; slot += num_clusters) {
        const uint32_t idesc = slot < p.full_slots ? p.idesc : p.idesc_half;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, p.status, 0x20u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, p.status, 0x40u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          const uint32_t a_lo32 = ((sA >> 4) & 0x3FFFu) | p.a.desc_lbo;
          const uint32_t b_lo32 = ((sB >> 4) & 0x3FFFu) | p.b.desc_lbo;
#pragma unroll
          for (int ks = 0; ks < kKSteps; ++ks) {
            const uint64_t ad = ((uint64_t)p.a.desc_hi << 32) | (uint64_t)(a_lo32 + ks * p.a.k_advance);
            const uint64_t bd = ((uint64_t)p.b.desc_hi << 32) | (uint64_t)(b_lo32 + ks * p.b.k_advance);
            umma_pair<TF32>(d_tmem, ad, bd, idesc, (kb | ks) != 0 ? 1u : 0u);
          }
          umma_commit_pair_both(smem_u32(&empty[stage]));   // frees this stage in both CTAs
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair_both(smem_u32(&acc_full[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp >= 4) {
    // ---------------- epilogue (both CTAs, each on its own 128 rows) ----------------
    const int q = warp & 3, half = (warp - 4) >> 2;
    uint32_t acc = 0, acc_phase = 0;
    OutT* D = reinterpret_cast<OutT*>(p.D);
    OutT* P = reinterpret_cast<OutT*>(p.preact);
    const OutT* bias = reinterpret_cast<const OutT*>(p.bias);
    const int64_t ldd = p.ldd;
    const bool accumulate = p.accumulate != 0;
    const uint32_t leader_acc_empty0 = map_to_cta(smem_u32(&acc_empty[0]), 0);
    bool ok = true;
    for (int slot = cluster_id; slot < p.total_slots && ok; slot += num_clusters) {
      int tile, halved, which, tm, tn;
      pair_slot(p, slot, &tile, &halved, &which);
      tile_coords(p, tile, &tm, &tn);
      const int COLS = halved ? BN / 4 : BN / 2;      // columns per epilogue warp group
      const int m0 = tm * (2 * kBM) + (int)rank * kBM;
      const int n0 = tn * BN + which * (BN / 2) + half * COLS;
      if (!mbar_wait_warp(&acc_full[acc], acc_phase, p.status, 0x80u)) { ok = false; break; }
      tc_fence_after();
      const int64_t m = (int64_t)m0 + q * 32 + lane;
      const bool m_ok = m < p.Mm;
      float bv = 0.f;
      if (bias != nullptr && m_ok) bv = to_f32(bias[m]);
      const int64_t rem = p.Nn - n0;
      const int lim = rem < COLS ? (int)rem : COLS;   // live columns (may be <= 0)
      OutT* dp = D + (int64_t)n0 * ldd + m;
      OutT* pp = P != nullptr ? P + (int64_t)n0 * ldd + m : nullptr;
#pragma unroll 1
      for (int c = 0; c < COLS / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + half * COLS + c * 32, r);
        tmem_ld_wait();
        if (m_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c * 32 + j < lim) {
              float v = __uint_as_float(r[j]) + bv;
              if (pp != nullptr) pp[j * ldd] = from_f32<OutT>(v);
              v = act_apply_any<ACT, FAST>(p.act, v);
              if (accumulate) v += to_f32(dp[j * ldd]);
              dp[j * ldd] = from_f32<OutT>(v);
            }
          }
        }
        dp += 32 * ldd;
        if (pp != nullptr) pp += 32 * ldd;
      }
      // this CTA's eight epilogue warps have all read their part of the accumulator: one arrival for the CTA
      tc_fence_before();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (warp == 4 && lane == 0) {
        if (rank == 0) mbar_arrive(&acc_empty[acc]);
        else mbar_arrive_cluster(leader_acc_empty0 + acc * 8u);
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  cluster_sync_all();   // neither CTA leaves (or frees TMEM) while its partner may still touch it
  if (warp == 2) {
    if (*reinterpret_cast<volatile unsigned int*>(p.status) != 0) {
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// ----------------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------------
// What the calling thread's last tensor-core GEMM launch looked like (read by lb2_last_gemm_plan; tests use it to
// assert which kernel and which tile schedule a shape takes): kernel (1 single-CTA, 2 CTA pair), tile_m, tile_n,
// tiles, workers (CTAs or CTA pairs), full_slots, total_slots.
thread_local int32_t g_last_gemm_plan[8] = {0, 0, 0, 0, 0, 0, 0, 0};
void record_gemm_plan(int kernel, int tile_m, int tile_n, int tiles, int workers, int full_slots, int total_slots) {
  int32_t* r = g_last_gemm_plan;
  r[0] = kernel; r[1] = tile_m; r[2] = tile_n; r[3] = tiles; r[4] = workers; r[5] = full_slots; r[6] = total_slots; r[7] = 0;
}
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 2-D map over an operand. K-major: dims {K, MN}; MN-major: dims {MN, K}. Box = 128-byte rows.
static bool make_operand_map(CUtensorMap* map, const GemmOperand& op, int64_t mn, int64_t kc, int elem_bytes,
                             int tile_mn, int bk, OperandPlan* plan, bool tf32) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  const int row_elems = 128 / elem_bytes;  // elements in a 128-byte row
  cuuint64_t dims[2];
  cuuint32_t box[2];
  if (op.mn_major) {
    dims[0] = (cuuint64_t)mn; dims[1] = (cuuint64_t)kc;
    box[0] = (cuuint32_t)row_elems; box[1] = (cuuint32_t)bk;
    plan->boxes = tile_mn / row_elems;
    plan->box_bytes = bk * 128;
    plan->mn_step = row_elems;
    plan->mn_major = 1;
    // canonical MN-major SW128 layout: 8 k-rows of 128 bytes form an atom (SBO = 1024 between
    // atoms along K); the next 128 bytes of MN live in the next box (LBO = box_bytes).
    plan->desc_lbo = ((uint32_t)(plan->box_bytes >> 4) & 0x3FFFu) << 16;
    plan->k_advance = (uint32_t)(((tf32 ? 8 : 16) * 128) >> 4);
  } else {
    dims[0] = (cuuint64_t)kc; dims[1] = (cuuint64_t)mn;
    box[0] = (cuuint32_t)row_elems; box[1] = (cuuint32_t)tile_mn;
    plan->boxes = 1;
    plan->box_bytes = tile_mn * 128;
    plan->mn_step = 0;
    plan->mn_major = 0;
    plan->desc_lbo = (1u & 0x3FFFu) << 16;  // ignored for swizzled K-major layouts
    plan->k_advance = 32 >> 4;              // 32 bytes of K per MMA step inside the 128-byte row
  }
  // Descriptor upper word: SBO (bits 32-45), version 1 (bits 46-47), layout type (bits 61-63).
  // 16-bit and K-major operands: SWIZZLE_128B (type 2), atoms of 8 rows x 128 bytes -> SBO = 1024.
  // MN-major tf32 operands: the tensor core transposes 32-bit elements only from the "128-byte
  // swizzle with 32-byte atoms" layout (type 1): atoms of 4 k-rows x 128 bytes -> SBO = 512, and
  // the TMA box is written with the matching CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B mode.
  const bool base32 = tf32 && op.mn_major;
  const uint32_t sbo = base32 ? 512u : 1024u;
  plan->desc_hi = (uint32_t)((sbo >> 4) & 0x3FFFu) | (1u << 14) | ((base32 ? 1u : 2u) << 29);
  cuuint64_t strides[1] = {(cuuint64_t)op.ld * (cuuint64_t)elem_bytes};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                   const_cast<void*>(op.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   base32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool gemm_tc_supported(const void* D, int64_t ldd, GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc,
                       int32_t dtype, int split3) {
  (void)ldd;
  if (Mm <= 0 || Nn <= 0 || Kc <= 0) return false;
  if (Mm > 0x7FFFFFFF || Nn > 0x7FFFFFFF || Kc > 0x7FFFFFFF) return false;
  const size_t es = dtype_size(dtype);
  if (!aligned_to(D, es)) return false;
  if (!(dtype == LB2_F32 && split3)) {  // the 3xTF32 route reads packed, aligned copies of its operands instead
    if (!aligned_to(A.ptr, 16) || !aligned_to(B.ptr, 16)) return false;
    if ((A.ld * (int64_t)es) % 16 != 0 || (B.ld * (int64_t)es) % 16 != 0) return false;
  }
  if (!encode_fn()) return false;
  return true;
}

// hi = round-to-nearest tf32 of x, lo = x - hi (exact in fp32). The copies are packed: leading
// dimension = rows rounded up to 4 elements (the 16-byte TMA stride rule).
__global__ void __launch_bounds__(256) split_tf32_kernel(float* __restrict__ hi, float* __restrict__ lo,
                                                         const float* __restrict__ x, int64_t rows, int64_t cols,
                                                         int64_t ld_in, int64_t ld_out) {
  const int64_t n = rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c = i / rows, r = i % rows;
    const float v = x[c * ld_in + r];
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
    const float hf = __uint_as_float(h);
    hi[c * ld_out + r] = hf;
    lo[c * ld_out + r] = v - hf;
  }
}

static int64_t packed_ld(int64_t rows) { return (rows + 3) / 4 * 4; }
static int64_t operand_rows(const GemmOperand& op, int64_t mn, int64_t kc) { return op.mn_major ? mn : kc; }
static int64_t operand_cols(const GemmOperand& op, int64_t mn, int64_t kc) { return op.mn_major ? kc : mn; }
static size_t operand_bytes(const GemmOperand& op, int64_t mn, int64_t kc) {
  return align_up((size_t)packed_ld(operand_rows(op, mn, kc)) * (size_t)operand_cols(op, mn, kc) * sizeof(float), 256);
}

size_t gemm_tc_split_workspace_bytes(GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc) {
  return 2 * operand_bytes(A, Mm, Kc) + 2 * operand_bytes(B, Nn, Kc);
}

static int reserved_sms(uint32_t flags) { return (int)((flags >> 16) & 0x7Fu); }

template <int BN, bool TF32, bool SPLIT3, typename OutT>
static int32_t tc_launch_cfg(const CUtensorMap& mA, const CUtensorMap& mB, const CUtensorMap& mAl, const CUtensorMap& mBl,
                             const TcParams& p, int max_ctas, cudaStream_t st) {
  using Cfg = TcCfg<BN, TF32, SPLIT3>;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < max_ctas ? tiles : max_ctas;
  auto launch = [&](auto kernel) -> int32_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "gemm_tc: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
    record_gemm_plan(1, kBM, BN, tiles, grid, tiles, tiles);
    kernel<<<grid, kThreadsSingle, Cfg::SMEM_BYTES, st>>>(mA, mB, mAl, mBl, p);
    LB2_CHECK_LAUNCH("gemm_tc");
    return LB2_OK;
  };
  switch (p.act) {
    case LB2_ACT_IDENTITY: return launch(gemm_tc_kernel<BN, TF32, SPLIT3, LB2_ACT_IDENTITY, OutT>);
    case LB2_ACT_RELU: return launch(gemm_tc_kernel<BN, TF32, SPLIT3, LB2_ACT_RELU, OutT>);
    case LB2_ACT_GELU_TANH: return launch(gemm_tc_kernel<BN, TF32, SPLIT3, LB2_ACT_GELU_TANH, OutT>);
    default: return launch(gemm_tc_kernel<BN, TF32, SPLIT3, -1, OutT>);
  }
}

static int32_t tc_launch_f32acc(const CUtensorMap& mA, const CUtensorMap& mB, const CUtensorMap& mAl, const CUtensorMap& mBl,
                                const TcParams& p, int max_ctas, cudaStream_t st) {
  using Cfg = TcCfg<kAccBN, true, true>;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < max_ctas ? tiles : max_ctas;
  auto launch = [&](auto kernel) -> int32_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "gemm_tc_f32acc: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
    kernel<<<grid, kAccThreads, Cfg::SMEM_BYTES, st>>>(mA, mB, mAl, mBl, p);
    LB2_CHECK_LAUNCH("gemm_tc_f32acc");
    return LB2_OK;
  };
  switch (p.act) {
    case LB2_ACT_IDENTITY: return launch(gemm_tc_f32acc_kernel<LB2_ACT_IDENTITY>);
    case LB2_ACT_RELU: return launch(gemm_tc_f32acc_kernel<LB2_ACT_RELU>);
    default: return launch(gemm_tc_f32acc_kernel<-1>);
  }
}

// CTA pairs the device can hold at once (GPC boundaries can leave a few SMs unpaired). Tiles are dealt
// round-robin to the clusters, so every cluster of a launch must be resident from the start. Cached per device.
template <typename Kernel>
static int resident_pairs(Kernel kernel, cudaLaunchConfig_t* cfg) {
  static std::mutex mu;
  static int resident[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return sm_count() / 2;
  std::lock_guard<std::mutex> lk(mu);
  if (resident[dev] == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    resident[dev] = n;
  }
  return resident[dev];
}

template <bool TF32, typename OutT>
static int32_t tc_launch_pair(const CUtensorMap& mA, const CUtensorMap& mB, const TcParams& p, int reserve, cudaStream_t st) {
  using Cfg = PairCfg;
  const int tiles = p.tiles_m * p.tiles_n;
  auto launch = [&](auto kernel) -> int32_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "gemm_tc_pair: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() & ~1, 1, 1);
    cfg.blockDim = dim3(kPairThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = resident_pairs(kernel, &cfg) - (reserve + 1) / 2;
    if (clusters < 1) clusters = 1;
    if (tiles < clusters) clusters = tiles;
    cfg.gridDim = dim3(2 * clusters, 1, 1);
    TcParams q = p;
    q.full_slots = q.total_slots = tiles;
    const int rem = tiles % clusters;
    if (rem > 0 && 2 * rem <= clusters && q.b.mn_major && q.b.boxes % 2 == 0) {   // halve the tiles of a thin last wave
      q.full_slots = tiles - rem;
      q.total_slots = tiles + rem;
    }
    record_gemm_plan(2, 2 * kBM, kPairBN, tiles, clusters, q.full_slots, q.total_slots);
    e = cudaLaunchKernelEx(&cfg, kernel, mA, mB, q);
    if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "gemm_tc_pair: %s", cudaGetErrorString(e));
    return LB2_OK;
  };
  switch (p.act) {
    case LB2_ACT_IDENTITY: return launch(gemm_tc_pair_kernel<TF32, LB2_ACT_IDENTITY, OutT>);
    case LB2_ACT_RELU: return launch(gemm_tc_pair_kernel<TF32, LB2_ACT_RELU, OutT>);
    case LB2_ACT_GELU_TANH: return launch(gemm_tc_pair_kernel<TF32, LB2_ACT_GELU_TANH, OutT>);
    default: return launch(gemm_tc_pair_kernel<TF32, -1, OutT>);
  }
}

int32_t gemm_tc_launch(void* D, int64_t ldd, GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc,
                       int32_t dtype, int split3, uint32_t flags, const GemmEpilogue& epi, void* split_ws,
                       cudaStream_t st) {
  const bool tf32 = dtype == LB2_F32;
  const int es = tf32 ? 4 : 2;
  const int bk = 128 / es;
  const bool split = tf32 && split3;
  // Kernel choice. Under the board's power limit the single-CTA kernel with 128 x 256 tiles is as fast as the
  // CTA-pair kernel for K-major operands (forward and dX of a dense layer: 1131 / 1151 against 1100 / 1136 TFLOP/s
  // on 4096 x 8192 x 4096), while the pair kernel wins when both operands are MN-major (dW: 981 against 933), whose
  // tiles arrive as several 64-wide boxes per k-block. So the pair kernel is the default for that layout when the
  // problem has enough 256 x 256 tiles to occupy most SM pairs; LB2_FLAG_CTA_PAIR asks for it for any layout (from an
  // eighth of the pairs on), LB2_FLAG_NO_CTA_PAIR rules it out. 128 x 128 tiles when that is what it takes to fill
  // the machine or to fit the doubled 3xTF32 stages.
  const int64_t pair_tiles = ((Mm + 2 * kBM - 1) / (2 * kBM)) * ((Nn + kPairBN - 1) / kPairBN);
  const bool want_pair = (flags & LB2_FLAG_CTA_PAIR) ? pair_tiles >= sm_count() / 8
                                                     : (A.mn_major && B.mn_major && pair_tiles >= sm_count() / 2 - 16);
  const bool pair = !split && !(flags & LB2_FLAG_NO_CTA_PAIR) && want_pair;
  int bn = 256;
  if (pair) bn = kPairBN / 2;  // rows of B each CTA of a pair loads
  else if (split) bn = 128;
  else if (((Mm + kBM - 1) / kBM) * ((Nn + 255) / 256) < sm_count()) bn = 128;

  TcParams p{};
  CUtensorMap mA, mB, mAl, mBl;
  if (!split) {
    if (!make_operand_map(&mA, A, Mm, Kc, es, kBM, bk, &p.a, tf32) || !make_operand_map(&mB, B, Nn, Kc, es, bn, bk, &p.b, tf32))
      return fail(LB2_LAUNCH_FAIL, "gemm_tc: cuTensorMapEncodeTiled failed");
    mAl = mA; mBl = mB;
  } else {
    LB2_REQUIRE(split_ws != nullptr && aligned_to(split_ws, 256), LB2_WORKSPACE_TOO_SMALL, "3xTF32 GEMM needs its split workspace");
    uint8_t* w = static_cast<uint8_t*>(split_ws);
    float* a_hi = reinterpret_cast<float*>(w); w += operand_bytes(A, Mm, Kc);
    float* a_lo = reinterpret_cast<float*>(w); w += operand_bytes(A, Mm, Kc);
    float* b_hi = reinterpret_cast<float*>(w); w += operand_bytes(B, Nn, Kc);
    float* b_lo = reinterpret_cast<float*>(w);
    const int64_t a_rows = operand_rows(A, Mm, Kc), a_cols = operand_cols(A, Mm, Kc);
    const int64_t b_rows = operand_rows(B, Nn, Kc), b_cols = operand_cols(B, Nn, Kc);
    const int g = sm_count() * 8;
    split_tf32_kernel<<<g, 256, 0, st>>>(a_hi, a_lo, (const float*)A.ptr, a_rows, a_cols, A.ld, packed_ld(a_rows));
    split_tf32_kernel<<<g, 256, 0, st>>>(b_hi, b_lo, (const float*)B.ptr, b_rows, b_cols, B.ld, packed_ld(b_rows));
    LB2_CHECK_LAUNCH("split_tf32");
    GemmOperand Ah = A, Al = A, Bh = B, Bl = B;
    Ah.ptr = a_hi; Al.ptr = a_lo; Bh.ptr = b_hi; Bl.ptr = b_lo;
    Ah.ld = Al.ld = packed_ld(a_rows);
    Bh.ld = Bl.ld = packed_ld(b_rows);
    OperandPlan dummy;
    if (!make_operand_map(&mA, Ah, Mm, Kc, es, kBM, bk, &p.a, tf32) || !make_operand_map(&mAl, Al, Mm, Kc, es, kBM, bk, &dummy, tf32) ||
        !make_operand_map(&mB, Bh, Nn, Kc, es, bn, bk, &p.b, tf32) || !make_operand_map(&mBl, Bl, Nn, Kc, es, bn, bk, &dummy, tf32))
      return fail(LB2_LAUNCH_FAIL, "gemm_tc: cuTensorMapEncodeTiled failed (split operands)");
  }
  p.Mm = Mm; p.Nn = Nn; p.Kc = Kc;
  p.bk = bk;
  const int tile_m = pair ? 2 * kBM : kBM, tile_n = pair ? kPairBN : bn;
  p.tiles_m = (int)((Mm + tile_m - 1) / tile_m);
  p.tiles_n = (int)((Nn + tile_n - 1) / tile_n);
  p.num_kb = (int)((Kc + bk - 1) / bk);
  // Band height of the tile order. If the A panels of all tile rows fit a third of L2 together, walk all of them per
  // tile column (A stays resident, B streams through once). Otherwise take as many tile rows as fit that budget, but
  // not fewer than what makes the tiles in flight (one per CTA or CTA pair) cover a roughly square block of the
  // output, i.e. about sqrt(workers * tile_n / tile_m) tile rows.
  {
    const int workers = pair ? sm_count() / 2 : sm_count();
    int h_sq = 1;
    while ((h_sq + 1) * (h_sq + 1) * tile_m <= workers * tile_n) ++h_sq;
    const double panel_bytes = (double)tile_m * (double)Kc * es;
    int h = (int)(48.0 * 1024 * 1024 / panel_bytes);
    if (h < h_sq) h = h_sq;
    p.raster_h = h < p.tiles_m ? h : p.tiles_m;
    if (p.raster_h < 1) p.raster_h = 1;
  }
  // instruction descriptor: D = f32 (bit 4), A/B format (bits 7-9 / 10-12: 1 = bf16, 2 = tf32),
  // A/B major (bits 15 / 16: 1 = MN-major), N >> 3 (bits 17-22), M >> 4 (bits 24-28)
  const uint32_t fmt = tf32 ? 2u : 1u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((A.mn_major ? 1u : 0u) << 15) | ((B.mn_major ? 1u : 0u) << 16) |
            ((uint32_t)(tile_n >> 3) << 17) | ((uint32_t)(tile_m >> 4) << 24);
  p.idesc_half = (p.idesc & ~(0x3Fu << 17)) | ((uint32_t)((tile_n / 2) >> 3) << 17);
  p.D = D; p.ldd = ldd;
  p.bias = epi.bias; p.preact = epi.preact; p.act = epi.act; p.accumulate = epi.accumulate;
  p.status = device_status_word();
  LB2_REQUIRE(p.status != nullptr, LB2_LAUNCH_FAIL, "gemm_tc: device status word unavailable");
  const int reserve = reserved_sms(flags);
  int max_ctas = sm_count() - reserve;
  if (max_ctas < 1) max_ctas = 1;
  if (pair) {
    if (tf32) return tc_launch_pair<true, float>(mA, mB, p, reserve, st);
    return tc_launch_pair<false, __nv_bfloat16>(mA, mB, p, reserve, st);
  }
  if (tf32) {
    if (split) return tc_launch_f32acc(mA, mB, mAl, mBl, p, max_ctas, st);
    if (bn == 256) return tc_launch_cfg<256, true, false, float>(mA, mB, mAl, mBl, p, max_ctas, st);
    return tc_launch_cfg<128, true, false, float>(mA, mB, mAl, mBl, p, max_ctas, st);
  }
  if (bn == 256) return tc_launch_cfg<256, false, false, __nv_bfloat16>(mA, mB, mAl, mBl, p, max_ctas, st);
  return tc_launch_cfg<128, false, false, __nv_bfloat16>(mA, mB, mAl, mBl, p, max_ctas, st);
}

// ----------------------------------------------------------------------------------------------
// dispatch between the tensor-core and CUDA-core kernels
// ----------------------------------------------------------------------------------------------
static bool use_tc(const void* D, int64_t ldd, GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc,
                   int32_t dtype, uint32_t flags) {
  if (flags & LB2_FLAG_FORCE_SIMT) return false;
  if (Mm * Nn * Kc < (int64_t)64 * 64 * 64) return false;  // latency-bound either way; skip descriptor encoding
  return gemm_tc_supported(D, ldd, A, B, Mm, Nn, Kc, dtype, (flags & LB2_FLAG_TF32_1X) ? 0 : 1);
}

size_t gemm_workspace_bytes(GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc, int32_t dtype,
                            uint32_t flags) {
  if (dtype != LB2_F32 || (flags & (LB2_FLAG_TF32_1X | LB2_FLAG_FORCE_SIMT))) return 0;
  if (Mm <= 0 || Nn <= 0 || Kc <= 0) return 0;
  return gemm_tc_split_workspace_bytes(A, B, Mm, Nn, Kc);
}

int32_t gemm_dispatch(void* D, int64_t ldd, GemmOperand A, GemmOperand B, int64_t Mm, int64_t Nn, int64_t Kc,
                      int32_t dtype, uint32_t flags, const GemmEpilogue& epi, void* ws, size_t ws_bytes,
                      cudaStream_t st) {
  if (Mm == 0 || Nn == 0) return LB2_OK;
  if (Kc > 0 && use_tc(D, ldd, A, B, Mm, Nn, Kc, dtype, flags)) {
    const int split3 = (dtype == LB2_F32 && !(flags & LB2_FLAG_TF32_1X)) ? 1 : 0;
    if (split3) {
      const size_t need = gemm_tc_split_workspace_bytes(A, B, Mm, Nn, Kc);
      LB2_REQUIRE(ws != nullptr && ws_bytes >= need, LB2_WORKSPACE_TOO_SMALL, "fp32 GEMM needs %zu bytes of workspace", need);
    }
    return gemm_tc_launch(D, ldd, A, B, Mm, Nn, Kc, dtype, split3, flags, epi, ws, st);
  }
  return gemm_simt_launch(D, ldd, A, B, Mm, Nn, Kc, dtype, epi, st);
}

}  // namespace lb2

// Tensor-core convolution for sm_100a (bf16 storage, fp32 accumulation in TMEM), fast case: implicit GEMM on the
// WHCN (column-major) bytes themselves, no copy of the input for the forward and the data gradient.
//
// Shapes taken: 2-D, stride 1, dilation 1, groups 1, output width == input width ("same" along W), W a multiple of 8,
// kernel width <= 4 and a filter small enough to stay RESIDENT in shared memory next to the operand ring (the
// 64-channel 3x3 stage of a ResNet). Every other bf16 geometry is served by the general path of conv_cw.cu.
//
// Formulation. With s = w + W*h the flattened spatial index of one image, a kernel tap (tw, th) reads x at
// s + (tw - pad_w) + (th - pad_h)*W. The H part of that shift is a multiple of 16 bytes and is applied as a TMA start
// coordinate on a tensor map (s, channel, image) whose out-of-range rows are zero-filled — the top/bottom padding.
// The W part is a single-element shift, which a TMA tile cannot start on; it is applied in the EPILOGUE instead
// (conv_tc_fwd2_kernel): per k-step ONE MMA of width kW*64 multiplies the A tile (128 positions x 64 channels,
// MN-major) with the kW taps of a kernel row side by side, giving kW accumulators that the epilogue adds shifted by one
// row each (warp shuffles plus a few rows exchanged through shared memory), masked at the image-row ends.
// The data gradient is the same kernel on dy with the filter packed flipped and transposed.
// The filter gradient (conv_tc_wgrad2_kernel) contracts over (s, image): M = 128 output channels (rows of dy),
// N = kW*64 = the kW taps of a kernel row x 64 input channels, read from kW-1 W-shifted copies of x made by one
// bandwidth pass (the unshifted tap comes from x itself); fp32 partials per K-split in the workspace and a
// fixed-order reduction — deterministic. With at most 64 output channels (conv_tc_wgrad_rows_kernel) the kernel-row shift
// moves onto dy, two kernel rows share one 128-row MMA, and the tap tiles are cut out of the unshifted x tile in shared
// memory, so no copies of x are made and x and dy are read once; the bias gradient of an identity-activation layer is
// summed from the same dy tiles.
//
// Roofline: tensor pipe; algorithmic FLOPs = 2*Wo*Ho*N*Cout*Cin*kW*kH per pass.
#include "conv.cuh"
#include "tc_ptx.cuh"

namespace lb2 {

constexpr int kConvThreads = 384;   // warps 0-2: TMA / MMA / TMEM, warps 4-11: epilogue (two per TMEM lane quarter)
constexpr int kConvBM = 128;

// ----------------------------------------------------------------------------------------------
// layout passes
// ----------------------------------------------------------------------------------------------
// out[t][n][c][h][w] = in[n][c][h][w + t - pad_w]  (0 outside the row), t = 0..kW-1
template <typename T>
__global__ void __launch_bounds__(256) conv_shift_copies_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                                int W, int64_t rows, int kW, int pad_w, int skip) {
  // one thread per 8-element group of a row; rows = H*C*N
  const int groups = (W + 7) / 8;
  const int64_t total = rows * groups;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / groups;
    const int w0 = (int)(i % groups) * 8;
    const T* src = in + row * W;
    // the 8 outputs of every copy need inputs w0 - pad_w + t .. +7: fetch the covering window once
    T win[8 + 8];
    const int lo = w0 - pad_w;  // window start (copy 0)
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int w = lo + j;
      win[j] = (j < 8 + kW - 1 && w >= 0 && w < W) ? src[w] : from_f32<T>(0.f);
    }
    for (int t = 0; t < kW; ++t) {
      if (t == skip) continue;   // the caller reads this copy (shift 0) from the input itself
      T* dst = out + ((int64_t)t * rows + row) * W + w0;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (w0 + j < W) dst[j] = win[j + t];
    }
  }
}

// 2-byte elements, compile-time kernel width and padding: every thread moves 16-byte vectors. The 8
// outputs of copy t start D = t - PAD elements away from the thread's aligned group, so they are
// cut out of the three aligned vectors around it with static funnel shifts.
template <int KW, int PAD>
__global__ void __launch_bounds__(256) conv_shift_copies_vec_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ in,
                                                                    int W, int64_t rows, int skip) {
  const int groups = W / 8;
  const int64_t total = rows * groups;
  const int64_t copy_stride = rows * W;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / groups;
    const int gq = (int)(i % groups);
    const uint4* src = reinterpret_cast<const uint4*>(in + row * W);
    const uint4 z = make_uint4(0, 0, 0, 0);
    const uint4 vm = gq > 0 ? __ldg(src + gq - 1) : z;
    const uint4 v0 = __ldg(src + gq);
    const uint4 vp = gq + 1 < groups ? __ldg(src + gq + 1) : z;
    const uint32_t win[12] = {vm.x, vm.y, vm.z, vm.w, v0.x, v0.y, v0.z, v0.w, vp.x, vp.y, vp.z, vp.w};  // 24 elements, ours at 8..15
#pragma unroll
    for (int t = 0; t < KW; ++t) {
      if (t == skip) continue;              // the caller reads this copy (shift 0) from the input itself
      constexpr int BASE = 8 - PAD;         // element index of output 0 of copy 0 inside the window
      const int e = BASE + t;               // compile-time after unrolling
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int q = (e >> 1) + k;
        o[k] = (e & 1) ? __funnelshift_r(win[q], win[q + 1], 16) : win[q];
      }
      __stcs(reinterpret_cast<uint4*>(out + (int64_t)t * copy_stride + row * W) + gq, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
}

static bool launch_shift_copies_vec(void* out, const void* in, int W, int64_t rows, int kW, int pad_w, unsigned grid,
                                    cudaStream_t st, int skip = -1) {
  uint16_t* o = static_cast<uint16_t*>(out);
  const uint16_t* i = static_cast<const uint16_t*>(in);
#define LB2_SHIFT_CASE(KW_, PAD_)                                                         \
  if (kW == KW_ && pad_w == PAD_) {                                                       \
    conv_shift_copies_vec_kernel<KW_, PAD_><<<grid, 256, 0, st>>>(o, i, W, rows, skip);   \
    return true;                                                                          \
  }
  LB2_SHIFT_CASE(1, 0)
  LB2_SHIFT_CASE(3, 1)
  LB2_SHIFT_CASE(3, 0)
  LB2_SHIFT_CASE(3, 2)
  LB2_SHIFT_CASE(5, 2)
  LB2_SHIFT_CASE(7, 3)
#undef LB2_SHIFT_CASE
  return false;
}

// Packed filter for the forward / data-gradient GEMM: Wp[nrow][kb*64 + j], nrow = GEMM output channel,
// k-block kb = (tap, 64-channel chunk). `transpose` selects the data-gradient packing (output channel
// of the GEMM = conv input channel, taps reversed).
struct PackGeom {
  int kW, kH, cin, cout;   // of the convolution's filter w (kW, kH, cin, cout)
  int flip;                // ConvDims flipkernel
  int transpose;           // 0: forward, 1: data gradient
  int chunks;              // 64-channel chunks of the contracted channel count
  int n_rows, k_total;     // rows (padded to the N tile) and columns of Wp
};

template <typename T>
__global__ void __launch_bounds__(256) conv_pack_filter_kernel(T* __restrict__ wp, const T* __restrict__ w,
                                                               const PackGeom g) {
  const int64_t total = (int64_t)g.n_rows * g.k_total;
  const int kc = g.transpose ? g.cout : g.cin;   // contracted channels
  const int nc = g.transpose ? g.cin : g.cout;   // GEMM output channels
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int row = (int)(i / g.k_total);
    const int col = (int)(i % g.k_total);
    const int kb = col / 64, j = col % 64;
    const int tap = kb / g.chunks, c = (kb % g.chunks) * 64 + j;
    const int tw = tap % g.kW, th = tap / g.kW;   // tap position: x offset (tw - pad_w, th - pad_h)
    float v = 0.f;
    if (row < nc && c < kc) {
      // forward: tap position t corresponds to filter index k with t = flip ? k : K-1-k
      // data gradient: position t' = K-1-t of the forward tap
      int tw_f = g.transpose ? g.kW - 1 - tw : tw, th_f = g.transpose ? g.kH - 1 - th : th;
      const int kw = g.flip ? tw_f : g.kW - 1 - tw_f, kh = g.flip ? th_f : g.kH - 1 - th_f;
      const int ci = g.transpose ? row : c, co = g.transpose ? c : row;
      v = to_f32(w[((int64_t)(co * g.cin + ci) * g.kH + kh) * g.kW + kw]);
    }
    wp[i] = from_f32<T>(v);
  }
}

// ----------------------------------------------------------------------------------------------
// forward / data-gradient kernel, shift-in-epilogue variant (kernel width <= 4, 64-channel N tiles)
// ----------------------------------------------------------------------------------------------
// Reads x directly (no shifted copies). For every kernel row th the A tile (128 positions x 64
// channels) is loaded ONCE and multiplied with the kW filter taps of that row into kW separate TMEM
// accumulators D_tw. The taps' single-element shifts along W are applied when the accumulators
// are combined: y[s] = sum_tw D_tw[s + tw - pad_w] (masked where w + tw - pad_w leaves the image
// row). Accumulator rows are TMEM lanes, so the shift is a warp shuffle, with the few rows that
// cross a warp boundary exchanged through shared memory. A tile covers MMA rows s0-8 .. s0+119 and
// produces the 112 outputs s0 .. s0+111 (the 8-row halo keeps the TMA start coordinate 16-byte
// aligned). Besides a third of the operand traffic this gives the tensor core kW independent
// accumulation chains to interleave (back-to-back MMAs into ONE accumulator are latency-bound at
// this N) and 4*kW MMAs per pipeline hand-over instead of 4.
struct ConvTc2Params {
  int32_t W, S_out, n_img, n_out;
  int32_t tiles_m, tiles_n, kW, kH, chunks, pad_w;
  int32_t stages;
  int32_t edge_rows;          // accumulator rows a neighbouring lane quarter needs per tap: max(pad_w, kW - 1 - pad_w)
  int32_t out_stage_stride;   // bytes of output staging per epilogue group (one tile, or two with a pre-activation)
  uint32_t idesc;
  uint32_t a_desc_hi, a_desc_lbo, a_k_advance;
  uint32_t b_desc_hi, b_desc_lbo, b_k_advance;
  void* y;
  void* preact;
  const void* bias;
  int32_t act;
  unsigned int* status;
  int16_t row_shift[16];   // per kernel row th: (th - pad_h) * W
};

constexpr int kHalo = 8;
// warps 0-2: TMA / MMA / TMEM; warps 4-11 and 12-19: two epilogue groups of eight warps. Group g owns TMEM
// accumulator g and every second tile, with its own edge rows, staging buffers and named barrier, so one
// group's TMEM reads, shuffles and store run under the other's (the epilogue of a tile takes longer than its MMAs).
constexpr int kConv2Threads = 640;
constexpr int kTileOut = kConvBM - 2 * kHalo;   // 112 outputs per tile

template <int KW, int ACT>
__global__ void __launch_bounds__(kConv2Threads, 1)
conv_tc_fwd2_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                    const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmP,
                    const __grid_constant__ ConvTc2Params p) {
  constexpr int BN = 64;
  constexpr int A_BYTES = kConvBM * 128;
  constexpr int B_BYTES = BN * 128;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int num_b = KW * p.kH * p.chunks;       // resident filter tiles, index (th*kW + tw)*chunks + chunk
  const int num_kb = p.kH * p.chunks;             // A stages per tile
  const uint32_t sB0 = smem_base;
  const uint32_t sA0 = smem_base + num_b * B_BYTES;
  uint8_t* after = smem_gen + num_b * B_BYTES + p.stages * A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(after);
  uint64_t* full = bars;
  uint64_t* empty = bars + p.stages;
  uint64_t* acc_full = bars + 2 * p.stages;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* b_full = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(b_full + 1);
  // accumulator rows that cross a warp boundary: edge[group][half][quarter][tw][edge_rows][32 cols]
  float* edge = reinterpret_cast<float*>(after + 512);
  // one flag per epilogue group, written and read only by that group's warps around the group's own barrier (the
  // other group learns of a failure through its own bounded waits)
  volatile int* abort_flag = reinterpret_cast<volatile int*>(after + 448);
  const int ER = p.edge_rows;
  const int EDGE_Q = KW * ER * 32;   // floats per (group, half, quarter)
  // output staging for the TMA store: per group [64 channels][112 positions] bf16, one tile for y and one for the
  // pre-activation. Rows of a tile start 16 bytes off a 32-byte sector in global memory, so direct
  // 2-byte stores from registers would leave half-written sectors; the tiled store writes whole runs.
  constexpr int STAGE_OUT = BN * kTileOut * 2;
  uint8_t* out_stage = after + 512 + 2 * 2 * 4 * EDGE_Q * 4;
  __shared__ float sbias[BN];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int tiles_per_n = p.tiles_m * p.n_img;
  const int nt = blockIdx.x % p.tiles_n;
  const int first = blockIdx.x / p.tiles_n, step = gridDim.x / p.tiles_n;
  const int n0 = nt * BN;
  constexpr uint32_t tmem_cols = (2 * KW * BN) > 256 ? 512u : 256u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }
    mbar_init(b_full, 1);
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  {
    const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(p.bias);
    for (int c = threadIdx.x; c < BN; c += blockDim.x)
      sbias[c] = (bias != nullptr && n0 + c < p.n_out) ? __bfloat162float(bias[n0 + c]) : 0.f;
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      tma_prefetch_desc(&tmW);
      mbar_expect_tx(b_full, (uint32_t)(num_b * B_BYTES));
      // packed filter column block (th*KW + tw)*chunks + chunk  ->  resident slot (th*chunks + chunk)*KW + tw,
      // so that the KW taps of one (kernel row, channel chunk) form ONE K-major operand of KW*64 rows
      for (int th = 0; th < p.kH; ++th)
        for (int tw = 0; tw < KW; ++tw)
          for (int ch = 0; ch < p.chunks; ++ch)
            tma_load_2d(sB0 + ((th * p.chunks + ch) * KW + tw) * B_BYTES, &tmW, ((th * KW + tw) * p.chunks + ch) * 64, n0, b_full);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = first; t < tiles_per_n && ok; t += step) {
        const int s0 = (t % p.tiles_m) * kTileOut - kHalo, img = t / p.tiles_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, p.status, 0x1000u)) { ok = false; break; }
          mbar_expect_tx(&full[stage], A_BYTES);
          const uint32_t sA = sA0 + stage * A_BYTES;
          const int th = kb / p.chunks, chunk = kb % p.chunks;
          const int c0 = s0 + p.row_shift[th];
          tma_load_4d(sA, &tmX, c0, chunk * 64, img, 0, &full[stage]);
          tma_load_4d(sA + A_BYTES / 2, &tmX, c0 + 64, chunk * 64, img, 0, &full[stage]);
          if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = mbar_wait(b_full, 0, p.status, 0x2000u);
      for (int t = first; t < tiles_per_n && ok; t += step) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, p.status, 0x4000u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * (KW * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, p.status, 0x8000u)) { ok = false; break; }
          tc_fence_after();
          const int th = kb / p.chunks, chunk = kb % p.chunks;
          const uint32_t sA = sA0 + stage * A_BYTES;
          const uint32_t a_lo32 = ((sA >> 4) & 0x3FFFu) | p.a_desc_lbo;
          // one MMA of N = KW*64 per k-step: its column blocks are the per-tap accumulators D_tw
          const uint32_t sB = sB0 + (uint32_t)((th * p.chunks + chunk) * KW * B_BYTES);
          const uint32_t b_lo32 = ((sB >> 4) & 0x3FFFu) | p.b_desc_lbo;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t ad = ((uint64_t)p.a_desc_hi << 32) | (uint64_t)(a_lo32 + ks * p.a_k_advance);
            const uint64_t bd = ((uint64_t)p.b_desc_hi << 32) | (uint64_t)(b_lo32 + ks * p.b_k_advance);
            umma<false>(d0, ad, bd, p.idesc, (kb | ks) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp >= 4) {
    const int grp = (warp - 4) >> 3;                  // epilogue group = TMEM accumulator it drains
    const int q = warp & 3, half = ((warp - 4) >> 2) & 1;   // lane quarter; which 32 of the 64 channels
    const int r = q * 32 + lane;                      // MMA row of this thread
    const uint32_t acc = (uint32_t)grp;
    uint32_t acc_phase = 0;
    uint8_t* my_stage = out_stage + grp * p.out_stage_stride;
    const bool leader = (warp == 4 + 8 * grp) && lane == 0;
    const __nv_bfloat16* P = reinterpret_cast<const __nv_bfloat16*>(p.preact);   // only tested for null here
    const float* sb = sbias + half * 32;
    const uint32_t parity = (uint32_t)grp;           // edge-row buffer of this group
    for (int t = first + grp * step; t < tiles_per_n; t += 2 * step) {
      const int s0 = (t % p.tiles_m) * kTileOut - kHalo, img = t / p.tiles_m;
      if (!mbar_wait_warp(&acc_full[acc], acc_phase, p.status, 0x10000u)) abort_flag[grp] = 1;
      tc_fence_after();
      const int s = s0 + r;
      const int w = ((s % p.W) + p.W) % p.W;   // column inside the image row (s is negative in the first halo)
      const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + acc * (KW * BN) + half * 32;
      float* eb = edge + (size_t)((parity * 2 + half) * 4 + q) * EDGE_Q;
      // pass 1: publish the rows a neighbouring quarter needs (last -d rows for d < 0, first d rows for d > 0)
#pragma unroll
      for (int tw = 0; tw < KW; ++tw) {
        const int d = tw - p.pad_w;
        if (d != 0) {
          uint32_t rt[32];
          tmem_ld32(t_acc + tw * BN, rt);
          tmem_ld_wait();
          int idx = -1;
          if (d < 0 && lane >= 32 + d) idx = lane - (32 + d);
          if (d > 0 && lane < d) idx = lane;
          if (idx >= 0) {
            float* e = eb + (tw * ER + idx) * 32;
#pragma unroll
            for (int j = 0; j < 32; ++j) e[j] = __uint_as_float(rt[j]);
          }
        }
      }
      // one barrier over the group's eight warps: edge rows are published, the group's previous store has
      // finished reading its staging buffers, and an expired wait is seen by everyone at the same point
      if (leader) tma_store_wait_read<0>();
      if (grp == 0) asm volatile("bar.sync 4, 256;" ::: "memory"); else asm volatile("bar.sync 5, 256;" ::: "memory");
      if (abort_flag[grp]) break;
      // pass 2: combine the taps
      float out[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) out[j] = sb[j];
#pragma unroll
      for (int tw = 0; tw < KW; ++tw) {
        const int d = tw - p.pad_w;
        uint32_t rt[32];
        tmem_ld32(t_acc + tw * BN, rt);
        tmem_ld_wait();
        if (d == 0) {
#pragma unroll
          for (int j = 0; j < 32; ++j) out[j] += __uint_as_float(rt[j]);
        } else {
          const bool in_row = (w + d >= 0) && (w + d < p.W);
          const int src = lane + d;
          const bool local = src >= 0 && src < 32;
          const int qn = src < 0 ? q - 1 : q + 1;
          const float* en = nullptr;
          if (!local && qn >= 0 && qn < 4) {
            const float* nb = edge + (size_t)((parity * 2 + half) * 4 + qn) * EDGE_Q;
            en = nb + (tw * ER + (src < 0 ? lane : src - 32)) * 32;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float v = __shfl_sync(0xffffffffu, __uint_as_float(rt[j]), src & 31);
            if (!local) v = en != nullptr ? en[j] : 0.f;
            if (in_row) out[j] += v;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      // stage the tile in shared memory ([channel][position]) and let one thread issue the tiled store
      const bool valid = r >= kHalo && r < kConvBM - kHalo;
      if (valid) {
        __nv_bfloat16* so = reinterpret_cast<__nv_bfloat16*>(my_stage) + (half * 32) * kTileOut + (r - kHalo);
        __nv_bfloat16* sp = so + BN * kTileOut;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (P != nullptr) sp[j * kTileOut] = __float2bfloat16_rn(out[j]);
          so[j * kTileOut] = __float2bfloat16_rn(act_apply_any<ACT, true>(p.act, out[j]));
        }
      }
      fence_proxy_async_smem();
      if (grp == 0) asm volatile("bar.sync 4, 256;" ::: "memory"); else asm volatile("bar.sync 5, 256;" ::: "memory");
      if (leader) {
        const int so0 = (t % p.tiles_m) * kTileOut;
        tma_store_3d(&tmY, smem_u32(my_stage), so0, n0, img);
        if (P != nullptr) tma_store_3d(&tmP, smem_u32(my_stage + STAGE_OUT), so0, n0, img);
        tma_store_commit();
      }
      acc_phase ^= 1u;
    }
    if (leader) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (*reinterpret_cast<volatile unsigned int*>(p.status) != 0) {
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ----------------------------------------------------------------------------------------------
// filter-gradient kernel, wide-N variant (kernel width <= 4)
// ----------------------------------------------------------------------------------------------
// The cost of a tcgen05.mma here depends little on its width, so the narrow (N = 64) MMAs of the kernel above are
// bound by their count. This variant turns the problem around: M = 128 output channels (rows of g), N = kW * 64 =
// the kW taps of one kernel row x 64 input channels (the kW shifted copies of x side by side), so one MMA covers
// what kW of the narrow ones did. A work item is (kernel row, 64-channel chunk, 128-channel output tile, K split);
// partial[z][group][co_local][tw*64 + ci_local] in fp32, reduced in a fixed order afterwards.
struct ConvWg2Params {
  int32_t n_img;
  int32_t s_blocks;                 // 64-position blocks per image
  int32_t kW, kH, chunks, co_tiles; // groups = kH * chunks * co_tiles
  int32_t splits, kb_total, kb_per_split;
  uint32_t idesc;
  uint32_t desc_hi, desc_lbo, k_advance;   // both operands K-major SW128
  float* partial;
  unsigned int* status;
  int32_t center_tw;                // tap whose shift along W is zero: read from x itself (-1: none)
  int16_t row_shift[16];            // per kernel row th: (th - pad_h) * W
};

template <int KW>
__global__ void __launch_bounds__(kConvThreads, 1)
conv_tc_wgrad2_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmX0,
                      const __grid_constant__ CUtensorMap tmG, const __grid_constant__ ConvWg2Params p) {
  constexpr int BN = KW * 64;
  constexpr int A_BYTES = kConvBM * 128;      // 128 output channels x 64 positions
  constexpr int B_BYTES = BN * 128;           // kW taps x 64 input channels x 64 positions
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int STAGES = (200 * 1024) / STAGE_BYTES > 8 ? 8 : (200 * 1024) / STAGE_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN > 256 ? 512u : (2 * BN > 128 ? 256u : 128u);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = p.kH * p.chunks * p.co_tiles;
  const int num_items = groups * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // item -> (group fastest, split); group -> (co tile fastest, chunk, kernel row)
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      tma_prefetch_desc(&tmX0);
      tma_prefetch_desc(&tmG);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int grp = item % groups, z = item / groups;
        const int kb_lo = z * p.kb_per_split, kb_hi = min(p.kb_total, kb_lo + p.kb_per_split);
        const int ct = grp % p.co_tiles, chunk = (grp / p.co_tiles) % p.chunks, th = grp / (p.co_tiles * p.chunks);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, p.status, 0x20000u)) { ok = false; break; }
          const int img = kb / p.s_blocks, s0 = (kb % p.s_blocks) * 64;
          const uint32_t sA = smem_base + stage * STAGE_BYTES, sB = sA + A_BYTES;
          mbar_expect_tx(&full[stage], (uint32_t)STAGE_BYTES);
          tma_load_4d(sA, &tmG, s0, ct * 128, img, 0, &full[stage]);
          tma_load_4d(sA + A_BYTES / 2, &tmG, s0, ct * 128 + 64, img, 0, &full[stage]);   // rows past the last channel are zero-filled
#pragma unroll
          for (int tw = 0; tw < KW; ++tw) {
            if (tw == p.center_tw) tma_load_4d(sB + tw * (64 * 128), &tmX0, s0 + p.row_shift[th], chunk * 64, img, 0, &full[stage]);
            else tma_load_4d(sB + tw * (64 * 128), &tmX, s0 + p.row_shift[th], chunk * 64, img, tw, &full[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int z = item / groups;
        const int kb_lo = z * p.kb_per_split, kb_hi = min(p.kb_total, kb_lo + p.kb_per_split);
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, p.status, 0x40000u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full[stage], phase, p.status, 0x80000u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * STAGE_BYTES, sB = sA + A_BYTES;
          const uint32_t a_lo32 = ((sA >> 4) & 0x3FFFu) | p.desc_lbo;
          const uint32_t b_lo32 = ((sB >> 4) & 0x3FFFu) | p.desc_lbo;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t ad = ((uint64_t)p.desc_hi << 32) | (uint64_t)(a_lo32 + ks * p.k_advance);
            const uint64_t bd = ((uint64_t)p.desc_hi << 32) | (uint64_t)(b_lo32 + ks * p.k_advance);
            umma<false>(d_tmem, ad, bd, p.idesc, (kb > kb_lo || ks != 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3, half = (warp - 4) >> 2;   // lane quarter; which half of the BN columns
    constexpr int COLS = BN / 2;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const int grp = item % groups, z = item / groups;
      if (!mbar_wait_warp(&acc_full[acc], acc_phase, p.status, 0x100000u)) { ok = false; break; }
      tc_fence_after();
      const int row = q * 32 + lane;
      float* dst = p.partial + (((int64_t)z * groups + grp) * 128 + row) * BN + half * COLS;
#pragma unroll 1
      for (int c = 0; c < COLS / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + half * COLS + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[c * 32 + j] = __uint_as_float(r[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (*reinterpret_cast<volatile unsigned int*>(p.status) != 0) {
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// dw[kw,kh,ci,co] = sum over splits (ascending) of partial[z][(th, chunk, co tile)][co % 128][tw*64 + ci % 64]
template <typename T>
__global__ void __launch_bounds__(256) conv_wgrad2_reduce_kernel(T* __restrict__ dw, const float* __restrict__ partial,
                                                                 int kW, int kH, int cin, int cout, int flip, int chunks,
                                                                 int co_tiles, int splits) {
  const int64_t total = (int64_t)kW * kH * cin * cout;
  const int groups = kH * chunks * co_tiles, bn = kW * 64;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i;
    const int kw = (int)(r % kW); r /= kW;
    const int kh = (int)(r % kH); r /= kH;
    const int ci = (int)(r % cin);
    const int co = (int)(r / cin);
    const int tw = flip ? kw : kW - 1 - kw, th = flip ? kh : kH - 1 - kh;
    const int grp = (th * chunks + ci / 64) * co_tiles + co / 128;
    const int64_t off = ((int64_t)grp * 128 + co % 128) * bn + tw * 64 + ci % 64;
    float s = 0.f;
    for (int z = 0; z < splits; ++z) s += partial[(int64_t)z * groups * 128 * bn + off];
    dw[i] = from_f32<T>(s);
  }
}


// ----------------------------------------------------------------------------------------------
// filter-gradient kernel for at most 64 output channels: kernel rows stacked along M, tap shifts made in shared memory
// ----------------------------------------------------------------------------------------------
// With 64 output channels the 128 accumulator rows of the kernel above are half empty and every kernel row loads the
// wide x operand again. Substituting s' = s + (th - pad_h)*W in
//   dw[tw, th, ci, co] = sum_s dy[co, s] * x_tw[ci, s + (th - pad_h)*W]
// moves the kernel-row shift onto dy: dw = sum_s' dy[co, s' - (th - pad_h)*W] * x_tw[ci, s']. One stage then holds the kW
// tap tiles of x at the positions s' ONCE and kH tiles of dy (64 rows each), each fetched at its own start coordinate
// (out-of-image positions zero-filled by the tensor map); two kernel rows form one A operand of 128 rows, so a 64-position
// block takes ceil(kH/2) * 4 MMAs for all kernel rows.
//
// The tap tiles x_tw[ci, s'] = x[ci, s' + tw - pad_w] (0 where the shift leaves the image row) are not read from shifted
// copies in global memory: the producer loads the unshifted tile (the tap tw = pad_w, in its final swizzled layout) and
// the 8 positions either side of it, and the eight epilogue warps, idle during the main loop, cut the other taps out of
// it: per 16-byte chunk a funnel shift over the chunk and its two neighbours, masked at the image-row ends (W is a
// multiple of 8 and blocks start on a multiple of 64, so a row end can only fall on a chunk boundary), stored at the
// chunk's swizzled place in the tap's tile. Operand traffic per block: (kH + 1) * 8 KB + 2 KB.
//
// A work item is (64-channel chunk, K split z) with one contiguous range of position blocks per split (interleaved
// blocks measured the same kernel time; consecutive blocks of a CTA share the shifted dy rows and 256-byte L2 sectors).
// partial[z][chunk][pair][(th & 1)*64 + co][tw*64 + ci] in fp32, reduced in a fixed order afterwards. For an odd kH the
// upper half of the last pair multiplies whatever follows the dy tiles in the stage (the first x tile); those accumulator
// rows are never read. With a bias gradient requested the same warps also add up the unshifted dy tile of every stage
// (db = sum of dy over positions and images; partial sums per split, reduced with the filter gradient).
struct ConvWg3Params {
  int32_t n_img;
  int32_t W;
  int32_t s_blocks;                 // 64-position blocks per image (input positions)
  int32_t kH, chunks, pairs;
  int32_t splits, kb_total, kb_per_split;
  uint32_t idesc;
  uint32_t desc_hi, desc_lbo, k_advance;   // both operands K-major SW128
  float* partial;
  float* db_partial;                // [split][64] sums of dy over the split's positions, or null
  int32_t db_th;                    // the kernel row whose dy tile is unshifted (th = pad_h)
  unsigned int* status;
  int16_t row_shift[16];            // per kernel row th: (th - pad_h) * W
};

// 16-byte chunk of tap shift D cut out of the window [chunk c-1 | chunk c | chunk c+1] (12 words, 24 elements)
template <int D>
__device__ __forceinline__ uint4 conv_shifted_chunk(const uint32_t (&win)[12], bool row_start, bool row_end) {
  constexpr int e = 8 + D;
  uint32_t o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    constexpr int q0 = e >> 1;
    o[k] = (e & 1) ? __funnelshift_r(win[q0 + k], win[q0 + k + 1], 16) : win[q0 + k];
  }
  if (D < 0 && row_start) {
#pragma unroll
    for (int k = 0; k < -D; ++k) o[k >> 1] &= (k & 1) ? 0x0000FFFFu : 0xFFFF0000u;
  }
  if (D > 0 && row_end) {
#pragma unroll
    for (int k = 8 - D; k < 8; ++k) o[k >> 1] &= (k & 1) ? 0x0000FFFFu : 0xFFFF0000u;
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

template <int KW, int PAD>
__global__ void __launch_bounds__(kConvThreads, 1)
conv_tc_wgrad_rows_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmXh,
                          const __grid_constant__ CUtensorMap tmG, const __grid_constant__ ConvWg3Params p, int stages,
                          int stage_bytes, uint32_t tmem_cols) {
  constexpr int BN = KW * 64;
  constexpr int TILE = 64 * 128;              // 64 rows x 64 positions
  constexpr int HALO = 64 * 16;               // 64 rows x 8 positions
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + stages * stage_bytes);
  uint64_t* raw_full = bars;                  // TMA has landed: dy tiles, the unshifted x tile, the two halos
  uint64_t* full = bars + stages;             // the shifted tap tiles are written (eight warps arrive)
  uint64_t* empty = bars + 2 * stages;
  uint64_t* acc_full = bars + 3 * stages;
  uint64_t* acc_empty = acc_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_items = p.chunks * p.splits;
  const int a_bytes = p.kH * TILE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&full[s], 8); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 8);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // item -> (chunk fastest, split)
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      tma_prefetch_desc(&tmXh);
      tma_prefetch_desc(&tmG);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int chunk = item % p.chunks, z = item / p.chunks;
        const int kb_lo = z * p.kb_per_split, kb_hi = min(p.kb_total, kb_lo + p.kb_per_split);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, p.status, 0x20000u)) { ok = false; break; }
          const int img = kb / p.s_blocks, s0 = (kb % p.s_blocks) * 64;
          const uint32_t sA = smem_base + stage * stage_bytes, sB = sA + a_bytes, sH = sB + KW * TILE;
          mbar_expect_tx(&raw_full[stage], (uint32_t)((p.kH + 1) * TILE + 2 * HALO));
          for (int th = 0; th < p.kH; ++th) tma_load_4d(sA + th * TILE, &tmG, s0 - p.row_shift[th], 0, img, 0, &raw_full[stage]);
          tma_load_4d(sB + PAD * TILE, &tmX, s0, chunk * 64, img, 0, &raw_full[stage]);
          tma_load_4d(sH, &tmXh, s0 - 8, chunk * 64, img, 0, &raw_full[stage]);
          tma_load_4d(sH + HALO, &tmXh, s0 + 64, chunk * 64, img, 0, &raw_full[stage]);
          if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int z = item / p.chunks;
        const int kb_lo = z * p.kb_per_split, kb_hi = min(p.kb_total, kb_lo + p.kb_per_split);
        if (!mbar_wait(acc_empty, acc_phase ^ 1u, p.status, 0x40000u)) { ok = false; break; }
        tc_fence_after();
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&raw_full[stage], phase, p.status, 0x80000u) || !mbar_wait(&full[stage], phase, p.status, 0x80000u)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * stage_bytes, sB = sA + a_bytes;
          const uint32_t b_lo32 = ((sB >> 4) & 0x3FFFu) | p.desc_lbo;
          for (int pi = 0; pi < p.pairs; ++pi) {
            const uint32_t a_lo32 = (((sA + pi * 2 * TILE) >> 4) & 0x3FFFu) | p.desc_lbo;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const uint64_t ad = ((uint64_t)p.desc_hi << 32) | (uint64_t)(a_lo32 + ks * p.k_advance);
              const uint64_t bd = ((uint64_t)p.desc_hi << 32) | (uint64_t)(b_lo32 + ks * p.k_advance);
              umma<false>(tmem_base + pi * BN, ad, bd, p.idesc, (kb > kb_lo || ks != 0) ? 1u : 0u);
            }
          }
          umma_commit(&empty[stage]);
          if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(acc_full);
        acc_phase ^= 1u;
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3, half = (warp - 4) >> 2;   // lane quarter; which half of the BN columns
    const int tid = threadIdx.x - 128;                // 0..255 over the eight warps
    constexpr int COLS = BN / 2;
    uint32_t stage = 0, phase = 0, acc_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const int z = item / p.chunks;
      const int kb_lo = z * p.kb_per_split, kb_hi = min(p.kb_total, kb_lo + p.kb_per_split);
      // bias gradient on the side: the unshifted dy tile of every stage is the split's share of dy, each element once
      const bool with_db = p.db_partial != nullptr && item % p.chunks == 0;
      float db_acc[2] = {0.f, 0.f};
      // main loop: the tap tiles of every stage
      for (int kb = kb_lo; kb < kb_hi; ++kb) {
        if (!mbar_wait_warp(&raw_full[stage], phase, p.status, 0x200000u)) { ok = false; break; }
        if (with_db) {
          const uint8_t* gt = smem_gen + stage * stage_bytes + p.db_th * TILE;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int task = tid + i * 256;
            const int r = task >> 3, c = task & 7;
            const uint4 v = *reinterpret_cast<const uint4*>(gt + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
            const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
            float sum = 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k) sum += __uint_as_float(wds[k] << 16) + __uint_as_float(wds[k] & 0xFFFF0000u);
            db_acc[i] += sum;
          }
        }
        if (KW > 1) {
          uint8_t* sB = smem_gen + stage * stage_bytes + a_bytes;
          const uint8_t* centre = sB + PAD * TILE;
          const uint8_t* halo = sB + KW * TILE;
          const int base_w = ((kb % p.s_blocks) * 64) % p.W;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int task = tid + i * 256;
            const int r = task >> 3, c = task & 7;
            const int w0 = (base_w + 8 * c) % p.W;
            const int row_off = (r >> 3) * 1024 + (r & 7) * 128;
            const int sw = r & 7;
            const uint4 v0 = *reinterpret_cast<const uint4*>(centre + row_off + ((c ^ sw) << 4));
            const uint4 vm = c > 0 ? *reinterpret_cast<const uint4*>(centre + row_off + (((c - 1) ^ sw) << 4))
                                   : *reinterpret_cast<const uint4*>(halo + r * 16);
            const uint4 vp = c < 7 ? *reinterpret_cast<const uint4*>(centre + row_off + (((c + 1) ^ sw) << 4))
                                   : *reinterpret_cast<const uint4*>(halo + HALO + r * 16);
            const uint32_t win[12] = {vm.x, vm.y, vm.z, vm.w, v0.x, v0.y, v0.z, v0.w, vp.x, vp.y, vp.z, vp.w};
            const bool row_start = w0 == 0, row_end = w0 == p.W - 8;
            const int dst_off = row_off + ((c ^ sw) << 4);
#pragma unroll
            for (int tw = 0; tw < KW; ++tw) {
              if (tw == PAD) continue;
              uint4 o;
              // tw - PAD is a compile-time constant after unrolling; spelled out so that the template argument is one
              switch (tw - PAD) {
                case -3: o = conv_shifted_chunk<-3>(win, row_start, row_end); break;
                case -2: o = conv_shifted_chunk<-2>(win, row_start, row_end); break;
                case -1: o = conv_shifted_chunk<-1>(win, row_start, row_end); break;
                case 1: o = conv_shifted_chunk<1>(win, row_start, row_end); break;
                case 2: o = conv_shifted_chunk<2>(win, row_start, row_end); break;
                default: o = conv_shifted_chunk<3>(win, row_start, row_end); break;
              }
              *reinterpret_cast<uint4*>(sB + tw * TILE + dst_off) = o;
            }
          }
          fence_proxy_async_smem();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[stage]);
        if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (with_db) {   // the eight lanes of a row (chunks 0-7) are neighbours in the warp
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          float v = db_acc[i];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          if ((tid & 7) == 0) p.db_partial[z * 64 + (tid >> 3) + 32 * i] = v;
        }
      }
      // epilogue: the accumulators of this item
      if (!mbar_wait_warp(acc_full, acc_phase, p.status, 0x100000u)) { ok = false; break; }
      tc_fence_after();
      const int row = q * 32 + lane;
      for (int pi = 0; pi < p.pairs; ++pi) {
        if (2 * pi + (q >> 1) >= p.kH) continue;   // upper half of an odd last pair: nothing to keep
        float* dst = p.partial + (((int64_t)item * p.pairs + pi) * 128 + row) * BN + half * COLS;
#pragma unroll 1
        for (int c = 0; c < COLS / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + pi * BN + half * COLS + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) dst[c * 32 + j] = __uint_as_float(r[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
      acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (*reinterpret_cast<volatile unsigned int*>(p.status) != 0) {
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// dw[kw,kh,ci,co] = sum over splits of partial[z][chunk][th / 2][(th & 1)*64 + co][tw*64 + ci % 64]. A block takes 64
// consecutive columns of the partial layout (coalesced reads) in four slices of the split index; every slice adds its
// splits in ascending order and the four slice sums are combined in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256) conv_wgrad_rows_reduce_kernel(T* __restrict__ dw, const float* __restrict__ partial,
                                                                     int kW, int kH, int cin, int cout, int flip, int chunks,
                                                                     int pairs, int splits, T* __restrict__ db,
                                                                     const float* __restrict__ db_partial) {
  __shared__ float part[4][64];
  if (db != nullptr && blockIdx.x == 0 && threadIdx.x < 64 && (int)threadIdx.x < cout) {   // db[co] = sum over splits, ascending
    float s = 0.f;
    for (int z = 0; z < splits; ++z) s += db_partial[z * 64 + threadIdx.x];
    db[threadIdx.x] = from_f32<T>(s);
  }
  const int bn = kW * 64;
  const int64_t per_split = (int64_t)chunks * pairs * 128 * bn;
  const int col = threadIdx.x & 63, zs = threadIdx.x >> 6;
  for (int64_t base = (int64_t)blockIdx.x * 64; base < per_split; base += (int64_t)gridDim.x * 64) {
    const int64_t off = base + col;
    float s = 0.f;
#pragma unroll 4
    for (int z = zs; z < splits; z += 4) s += __ldcs(partial + (int64_t)z * per_split + off);
    part[zs][col] = s;
    __syncthreads();
    if (zs == 0) {
      const float total = ((part[0][col] + part[1][col]) + part[2][col]) + part[3][col];
      const int c = (int)(off % bn);
      int64_t r = off / bn;
      const int row = (int)(r % 128); r /= 128;
      const int pi = (int)(r % pairs);
      const int chunk = (int)(r / pairs);
      const int th = 2 * pi + (row >> 6), co = row & 63, tw = c >> 6, ci = chunk * 64 + (c & 63);
      if (th < kH && co < cout && ci < cin) {
        const int kw = flip ? tw : kW - 1 - tw, kh = flip ? th : kH - 1 - th;
        dw[kw + (int64_t)kW * (kh + (int64_t)kH * (ci + (int64_t)cin * co))] = from_f32<T>(total);
      }
    }
    __syncthreads();
  }
}

// ----------------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------------
// One implicit-GEMM problem: out (W, Ho, Cn, N) = taps over in (W, Hi, Ck, N)
struct ConvGemm {
  int W, Hi, Ho, Ck, Cn, N, kW, kH, pad_w, pad_h;
};

static bool bf16_map_4d(CUtensorMap* map, const void* ptr, int64_t d0, int64_t d1, int64_t d2, int64_t d3,
                        int box0, int box1, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc) return false;
  cuuint64_t dims[4] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)d2, (cuuint64_t)d3};
  cuuint64_t strides[3] = {(cuuint64_t)d0 * 2, (cuuint64_t)d0 * d1 * 2, (cuuint64_t)d0 * d1 * d2 * 2};
  cuuint32_t box[4] = {(cuuint32_t)box0, (cuuint32_t)box1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
static bool bf16_map_2d(CUtensorMap* map, const void* ptr, int64_t d0, int64_t d1, int box0, int box1) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)d0, (cuuint64_t)d1};
  cuuint64_t strides[1] = {(cuuint64_t)d0 * 2};
  cuuint32_t box[2] = {(cuuint32_t)box0, (cuuint32_t)box1};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// output tensor (S_out, channels, images) for the tiled store: box = 112 positions x 64 channels, no swizzle
static bool bf16_map_out(CUtensorMap* map, const void* ptr, int64_t s_out, int64_t ch, int64_t n) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc) return false;
  cuuint64_t dims[3] = {(cuuint64_t)s_out, (cuuint64_t)ch, (cuuint64_t)n};
  cuuint64_t strides[2] = {(cuuint64_t)s_out * 2, (cuuint64_t)s_out * ch * 2};
  cuuint32_t box[3] = {(cuuint32_t)(kConvBM - 16), 64, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int conv_chunks(int ck) { return (ck + 63) / 64; }

// shift-in-epilogue kernel: kernel width <= 4, filter resident next to at least 3 A stages and the edge buffers
// A-ring depth; `with_preact` = the launch also stages a pre-activation tile per epilogue group
static int conv_edge_rows(const ConvGemm& c) { return c.pad_w > c.kW - 1 - c.pad_w ? c.pad_w : c.kW - 1 - c.pad_w; }
static int conv_edge_bytes(const ConvGemm& c) { return 2 * 2 * 4 * c.kW * conv_edge_rows(c) * 32 * 4; }
static int conv_fwd2_stages(const ConvGemm& c, bool with_preact = true) {
  if (c.kW > 4 || c.kH > 16) return 0;
  const int resident = c.kW * c.kH * conv_chunks(c.Ck) * 64 * 128;
  const int edges = conv_edge_bytes(c) + 2 * (with_preact ? 2 : 1) * 64 * (kConvBM - 16) * 2;   // edge rows + output staging of both epilogue groups
  int st = (224 * 1024 - resident - edges) / (kConvBM * 128);
  return st > 8 ? 8 : st;
}
static bool conv_use_fwd2(const ConvGemm& c) { return conv_fwd2_stages(c) >= 3; }

static bool conv_gemm_ok(const ConvGemm& c) {
  if (c.W % 8 == 0 && c.kW >= 1 && c.kH >= 1 && conv_use_fwd2(c) && (int64_t)(c.kH + c.pad_h) * c.W <= 32000 &&
      (int64_t)c.W * c.Hi < (1 << 30) && (int64_t)c.W * c.Ho < (1 << 30))
    return tensor_map_encoder() != nullptr;
  return false;
}

bool conv_tc_supported(const ConvGeom& g, int32_t dtype) {
  if (dtype == LB2_F32) return conv_tc_f32_supported(g);
  if (dtype != LB2_BF16 || g.ndim != 2 || g.groups != 1) return false;
  if (g.stride[0] != 1 || g.stride[1] != 1 || g.dil[0] != 1 || g.dil[1] != 1) return false;
  if (g.out[0] != g.in[0] || g.out[0] <= 0 || g.out[1] <= 0 || g.batch <= 0 || g.cin <= 0 || g.cout <= 0) return false;
  if (g.pad_lo[0] > g.k[0] - 1 || g.pad_lo[1] > g.k[1] - 1) return false;  // data gradient needs K-1-pad >= 0
  const ConvGemm f{g.in[0], g.in[1], g.out[1], g.cin, g.cout, g.batch, g.k[0], g.k[1], g.pad_lo[0], g.pad_lo[1]};
  const ConvGemm d{g.in[0], g.out[1], g.in[1], g.cout, g.cin, g.batch, g.k[0], g.k[1], g.k[0] - 1 - g.pad_lo[0], g.k[1] - 1 - g.pad_lo[1]};
  // only the fast case stays here (filter resident in shared memory, shift-in-epilogue kernels in both directions);
  // every other bf16 geometry is served by the general path of conv_cw.cu
  if (!conv_gemm_ok(f) || !conv_gemm_ok(d) || !conv_use_fwd2(f) || !conv_use_fwd2(d)) return false;
  return true;
}

static size_t copies_bytes(const ConvGemm& c) { return align_up((size_t)c.kW * c.W * c.Hi * c.Ck * c.N * 2, 1024); }
static size_t packed_bytes(const ConvGemm& c) {
  const int bn = 64;
  const size_t rows = (size_t)((c.Cn + bn - 1) / bn) * bn;
  return align_up(rows * (size_t)(c.kW * c.kH * conv_chunks(c.Ck) * 64) * 2, 1024);
}

static unsigned flat_grid_tc(int64_t total) {
  int64_t gsz = (total + 255) / 256, cap = (int64_t)sm_count() * 16;
  return (unsigned)(gsz < 1 ? 1 : (gsz > cap ? cap : gsz));
}

// out = act(implicit GEMM + bias); workspace = shifted copies | packed filter
static int32_t run_conv_gemm(void* out, void* preact, const void* bias, int32_t act, const void* in, const void* w,
                             const ConvGemm& c, const PackGeom& pg, uint8_t* ws, cudaStream_t st) {
  using T = __nv_bfloat16;
  if (conv_use_fwd2(c)) {
    T* wp2 = reinterpret_cast<T*>(ws);
    conv_pack_filter_kernel<T><<<flat_grid_tc((int64_t)pg.n_rows * pg.k_total), 256, 0, st>>>(wp2, (const T*)w, pg);
    LB2_CHECK_LAUNCH("conv_tc filter packing");
    ConvTc2Params q{};
    q.W = c.W; q.S_out = c.W * c.Ho; q.n_img = c.N; q.n_out = c.Cn;
    q.tiles_m = (q.S_out + kTileOut - 1) / kTileOut;
    q.tiles_n = (c.Cn + 63) / 64;
    q.kW = c.kW; q.kH = c.kH; q.chunks = conv_chunks(c.Ck); q.pad_w = c.pad_w;
    q.stages = conv_fwd2_stages(c, preact != nullptr);
    q.edge_rows = conv_edge_rows(c);
    q.out_stage_stride = (preact != nullptr ? 2 : 1) * 64 * kTileOut * 2;
    for (int th = 0; th < c.kH; ++th) q.row_shift[th] = (int16_t)((th - c.pad_h) * c.W);
    q.a_desc_hi = (uint32_t)((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
    q.a_desc_lbo = ((8192u >> 4) & 0x3FFFu) << 16;
    q.a_k_advance = 2048u >> 4;
    q.b_desc_hi = q.a_desc_hi;
    q.b_desc_lbo = 1u << 16;
    q.b_k_advance = 32u >> 4;
    q.idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)((c.kW * 64) >> 3) << 17) | ((uint32_t)(kConvBM >> 4) << 24);
    q.y = out; q.preact = preact; q.bias = bias; q.act = act;
    q.status = device_status_word();
    LB2_REQUIRE(q.status != nullptr, LB2_LAUNCH_FAIL, "conv_tc: device status word unavailable");
    CUtensorMap mX2, mW2, mY2, mP2;
    if (!bf16_map_4d(&mX2, in, (int64_t)c.W * c.Hi, c.Ck, c.N, 1, 64, 64) || !bf16_map_2d(&mW2, wp2, pg.k_total, pg.n_rows, 64, 64) ||
        !bf16_map_out(&mY2, out, q.S_out, c.Cn, c.N) || !bf16_map_out(&mP2, preact != nullptr ? preact : out, q.S_out, c.Cn, c.N))
      return fail(LB2_LAUNCH_FAIL, "conv_tc: cuTensorMapEncodeTiled failed");
    const int num_b = c.kW * c.kH * q.chunks;
    const int smem2 = num_b * 64 * 128 + q.stages * kConvBM * 128 + 512 + conv_edge_bytes(c) + 2 * q.out_stage_stride + 1024 + 256;
    const int tiles_per_n2 = q.tiles_m * q.n_img;
    int per_n2 = sm_count() / q.tiles_n;
    if (per_n2 > tiles_per_n2) per_n2 = tiles_per_n2;
    if (per_n2 < 1) per_n2 = 1;
    const int grid2 = per_n2 * q.tiles_n;
    auto launch2 = [&](auto kernel) -> int32_t {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
      if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "conv_tc: cannot reserve %d bytes of shared memory: %s", smem2, cudaGetErrorString(e));
      kernel<<<grid2, kConv2Threads, smem2, st>>>(mX2, mW2, mY2, mP2, q);
      LB2_CHECK_LAUNCH("conv_tc_fwd2");
      return LB2_OK;
    };
#define LB2_FWD2_ACT(KW_)                                                                    \
    switch (act) {                                                                           \
      case LB2_ACT_IDENTITY: return launch2(conv_tc_fwd2_kernel<KW_, LB2_ACT_IDENTITY>);     \
      case LB2_ACT_RELU: return launch2(conv_tc_fwd2_kernel<KW_, LB2_ACT_RELU>);             \
      default: return launch2(conv_tc_fwd2_kernel<KW_, -1>);                                 \
    }
    switch (c.kW) {
      case 1: LB2_FWD2_ACT(1)
      case 2: LB2_FWD2_ACT(2)
      case 3: LB2_FWD2_ACT(3)
      default: LB2_FWD2_ACT(4)
    }
#undef LB2_FWD2_ACT
  }
  return fail(LB2_BAD_SHAPE, "conv_tc: geometry outside the resident-filter fast case");
}

static ConvGemm fwd_gemm(const ConvGeom& g) {
  return ConvGemm{g.in[0], g.in[1], g.out[1], g.cin, g.cout, g.batch, g.k[0], g.k[1], g.pad_lo[0], g.pad_lo[1]};
}
static ConvGemm dgrad_gemm(const ConvGeom& g) {
  return ConvGemm{g.in[0], g.out[1], g.in[1], g.cout, g.cin, g.batch, g.k[0], g.k[1], g.k[0] - 1 - g.pad_lo[0], g.k[1] - 1 - g.pad_lo[1]};
}
static PackGeom pack_geom(const ConvGeom& g, const ConvGemm& c, int transpose) {
  PackGeom pg{};
  pg.kW = g.k[0]; pg.kH = g.k[1]; pg.cin = g.cin; pg.cout = g.cout; pg.flip = g.flip; pg.transpose = transpose;
  pg.chunks = conv_chunks(c.Ck);
  const int bn = 64;
  pg.n_rows = ((c.Cn + bn - 1) / bn) * bn;
  pg.k_total = c.kW * c.kH * pg.chunks * 64;
  return pg;
}

size_t conv_tc_fwd_workspace_bytes(const ConvGeom& g, int32_t dtype) {
  if (dtype == LB2_F32) return conv_tc_f32_fwd_workspace_bytes(g);
  const ConvGemm c = fwd_gemm(g);
  return packed_bytes(c);
}

int32_t conv_tc_fwd(void* y, void* preact, const void* x, const void* w, const void* bias, const ConvGeom& g,
                    int32_t dtype, int32_t act, void* ws, cudaStream_t st) {
  if (dtype == LB2_F32) return conv_tc_f32_fwd(y, preact, x, w, bias, g, act, ws, st);
  const ConvGemm c = fwd_gemm(g);
  return run_conv_gemm(y, preact, bias, act, x, w, c, pack_geom(g, c, 0), static_cast<uint8_t*>(ws), st);
}

// ---- filter gradient plan
// wide-N variant: kernel width <= 4 (N = kW * 64 <= 256), kH <= 16
struct Wg2Plan {
  bool ok;
  int chunks, co_tiles, groups, s_blocks, kb_total, splits, kb_per_split;
};
static Wg2Plan wg2_plan(const ConvGeom& g) {
  Wg2Plan w{};
  if (g.k[0] > 4 || g.k[1] > 16) return w;
  w.ok = true;
  w.chunks = conv_chunks(g.cin);
  w.co_tiles = (g.cout + 127) / 128;
  w.groups = g.k[1] * w.chunks * w.co_tiles;
  const int S_out = g.out[0] * g.out[1];
  w.s_blocks = (S_out + 63) / 64;
  w.kb_total = g.batch * w.s_blocks;
  int splits = sm_count() / w.groups;
  if (splits < 1) splits = 1;
  if (splits > w.kb_total) splits = w.kb_total;
  w.kb_per_split = (w.kb_total + splits - 1) / splits;
  w.splits = (w.kb_total + w.kb_per_split - 1) / w.kb_per_split;
  return w;
}
static size_t wg2_partial_bytes(const ConvGeom& g, const Wg2Plan& w) {
  return align_up((size_t)w.splits * w.groups * 128 * (g.k[0] * 64) * sizeof(float), 1024);
}
// kernel rows stacked along M: at most 64 output channels, all accumulators (one per pair of kernel rows) in TMEM at once
struct Wg3Plan {
  bool ok;
  int chunks, pairs, s_blocks, kb_total, splits, kb_per_split, stages, stage_bytes;
  uint32_t tmem_cols;
};
static Wg3Plan wg3_plan(const ConvGeom& g) {
  Wg3Plan w{};
  if (g.k[0] > 4 || g.k[1] > 16 || g.cout > 64 || g.pad_lo[0] < 0 || g.pad_lo[0] >= g.k[0] || g.in[0] % 8 != 0) return w;
  w.pairs = (g.k[1] + 1) / 2;
  const int cols = w.pairs * g.k[0] * 64;
  if (cols > 512) return w;
  w.tmem_cols = 32;
  while ((int)w.tmem_cols < cols) w.tmem_cols *= 2;
  w.stage_bytes = (g.k[1] + g.k[0]) * 64 * 128 + 2 * 64 * 16;   // dy tiles, tap tiles, the two 8-position halos of x
  w.stages = (200 * 1024) / w.stage_bytes;
  if (w.stages > 8) w.stages = 8;
  if (w.stages < 2) return w;
  w.ok = true;
  w.chunks = conv_chunks(g.cin);
  w.s_blocks = (g.in[0] * g.in[1] + 63) / 64;
  w.kb_total = g.batch * w.s_blocks;
  int splits = sm_count() / w.chunks;
  if (splits < 1) splits = 1;
  if (splits > w.kb_total) splits = w.kb_total;
  w.kb_per_split = (w.kb_total + splits - 1) / splits;
  w.splits = (w.kb_total + w.kb_per_split - 1) / w.kb_per_split;
  return w;
}
static size_t wg3_partial_bytes(const ConvGeom& g, const Wg3Plan& w) {
  return align_up((size_t)w.splits * w.chunks * w.pairs * 128 * (g.k[0] * 64) * sizeof(float), 1024);
}
static size_t wg3_db_partial_bytes(const Wg3Plan& w) { return align_up((size_t)w.splits * 64 * sizeof(float), 1024); }
static size_t wg_any_partial_bytes(const ConvGeom& g) {
  const Wg3Plan w3 = wg3_plan(g);
  return w3.ok ? wg3_partial_bytes(g, w3) + wg3_db_partial_bytes(w3) : wg2_partial_bytes(g, wg2_plan(g));
}

bool conv_tc_wgrad_makes_db(const ConvGeom& g, int32_t dtype) {
  // the unshifted dy tile must exist (0 <= pad_h < kH) and the input position blocks must cover every output position
  return dtype == LB2_BF16 && wg3_plan(g).ok && g.pad_lo[1] >= 0 && g.pad_lo[1] < g.k[1] && g.out[1] <= g.in[1];
}

size_t conv_tc_bwd_workspace_bytes(const ConvGeom& g, int32_t dtype) {
  if (dtype == LB2_F32) return conv_tc_f32_bwd_workspace_bytes(g);
  const ConvGemm d = dgrad_gemm(g), f = fwd_gemm(g);
  const size_t dgrad = packed_bytes(d);
  const size_t wgrad = copies_bytes(f) + wg_any_partial_bytes(g);
  return dgrad > wgrad ? dgrad : wgrad;   // the two gradients run one after the other in the same region
}

int32_t conv_tc_dgrad(void* dx, const void* gy, const void* w, const ConvGeom& g, int32_t dtype, void* ws, cudaStream_t st) {
  if (dtype == LB2_F32) return fail(LB2_BAD_ARG, "Float32 gradients are computed by conv_tc_f32_bwd");
  const ConvGemm c = dgrad_gemm(g);
  return run_conv_gemm(dx, nullptr, nullptr, LB2_ACT_IDENTITY, gy, w, c, pack_geom(g, c, 1), static_cast<uint8_t*>(ws), st);
}

int32_t conv_tc_wgrad(void* dw, const void* x, const void* gy, const ConvGeom& g, int32_t dtype, void* ws_, cudaStream_t st, void* db) {
  if (dtype == LB2_F32) return fail(LB2_BAD_ARG, "Float32 gradients are computed by conv_tc_f32_bwd");
  using T = __nv_bfloat16;
  uint8_t* ws = static_cast<uint8_t*>(ws_);
  const ConvGemm f = fwd_gemm(g);
  T* copies = reinterpret_cast<T*>(ws);
  float* partial = reinterpret_cast<float*>(ws + copies_bytes(f));
  const int64_t rows = (int64_t)f.Hi * f.Ck * f.N;
  const Wg3Plan w3 = wg3_plan(g);
  if (w3.ok) {   // no copies of x: the taps are cut out of the unshifted tile in shared memory
    ConvWg3Params q{};
    q.n_img = g.batch; q.W = f.W; q.s_blocks = w3.s_blocks;
    q.kH = f.kH; q.chunks = w3.chunks; q.pairs = w3.pairs;
    q.splits = w3.splits; q.kb_total = w3.kb_total; q.kb_per_split = w3.kb_per_split;
    q.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((f.kW * 64) >> 3) << 17) | ((uint32_t)(kConvBM >> 4) << 24);
    q.desc_hi = (uint32_t)((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
    q.desc_lbo = 1u << 16;
    q.k_advance = 32u >> 4;
    q.partial = partial;
    float* db_partial = reinterpret_cast<float*>(ws + copies_bytes(f) + wg3_partial_bytes(g, w3));
    const bool with_db = db != nullptr && conv_tc_wgrad_makes_db(g, dtype);
    q.db_partial = with_db ? db_partial : nullptr;
    q.db_th = f.pad_h;
    q.status = device_status_word();
    LB2_REQUIRE(q.status != nullptr, LB2_LAUNCH_FAIL, "conv_tc: device status word unavailable");
    for (int th = 0; th < f.kH; ++th) q.row_shift[th] = (int16_t)((th - f.pad_h) * f.W);
    CUtensorMap mX3, mXh3, mG3;
    if (!bf16_map_4d(&mX3, x, (int64_t)f.W * f.Hi, f.Ck, f.N, 1, 64, 64) ||
        !bf16_map_4d(&mXh3, x, (int64_t)f.W * f.Hi, f.Ck, f.N, 1, 8, 64, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !bf16_map_4d(&mG3, gy, (int64_t)g.out[0] * g.out[1], g.cout, g.batch, 1, 64, 64))
      return fail(LB2_LAUNCH_FAIL, "conv_tc: cuTensorMapEncodeTiled failed");
    const int smem3 = w3.stages * w3.stage_bytes + 1024 + 256 + 64 * 8;
    const int items3 = w3.chunks * w3.splits;
    const int grid3 = items3 < sm_count() ? items3 : sm_count();
    auto launch3 = [&](auto kernel) -> int32_t {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem3);
      if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "conv_tc: cannot reserve %d bytes of shared memory: %s", smem3, cudaGetErrorString(e));
      kernel<<<grid3, kConvThreads, smem3, st>>>(mX3, mXh3, mG3, q, w3.stages, w3.stage_bytes, w3.tmem_cols);
      LB2_CHECK_LAUNCH("conv_tc_wgrad_rows");
      return LB2_OK;
    };
    int32_t rc3 = LB2_OK;
    switch (f.kW * 4 + f.pad_w) {
      case 1 * 4 + 0: rc3 = launch3(conv_tc_wgrad_rows_kernel<1, 0>); break;
      case 2 * 4 + 0: rc3 = launch3(conv_tc_wgrad_rows_kernel<2, 0>); break;
      case 2 * 4 + 1: rc3 = launch3(conv_tc_wgrad_rows_kernel<2, 1>); break;
      case 3 * 4 + 0: rc3 = launch3(conv_tc_wgrad_rows_kernel<3, 0>); break;
      case 3 * 4 + 1: rc3 = launch3(conv_tc_wgrad_rows_kernel<3, 1>); break;
      case 3 * 4 + 2: rc3 = launch3(conv_tc_wgrad_rows_kernel<3, 2>); break;
      case 4 * 4 + 0: rc3 = launch3(conv_tc_wgrad_rows_kernel<4, 0>); break;
      case 4 * 4 + 1: rc3 = launch3(conv_tc_wgrad_rows_kernel<4, 1>); break;
      case 4 * 4 + 2: rc3 = launch3(conv_tc_wgrad_rows_kernel<4, 2>); break;
      default: rc3 = launch3(conv_tc_wgrad_rows_kernel<4, 3>); break;
    }
    if (rc3 != LB2_OK) return rc3;
    const int64_t per_split3 = (int64_t)w3.chunks * w3.pairs * 128 * (f.kW * 64);
    conv_wgrad_rows_reduce_kernel<T><<<(unsigned)(per_split3 / 64), 256, 0, st>>>((T*)dw, partial, g.k[0], g.k[1], g.cin, g.cout, g.flip,
                                                                               w3.chunks, w3.pairs, w3.splits, with_db ? (T*)db : nullptr, db_partial);
    LB2_CHECK_LAUNCH("conv_wgrad_rows_reduce");
    return LB2_OK;
  }
  const Wg2Plan w2 = wg2_plan(g);
  // the wide-N kernel reads the unshifted tap straight from x, so that copy is not made
  const int skip = (w2.ok && f.pad_w >= 0 && f.pad_w < f.kW) ? f.pad_w : -1;
  if (!launch_shift_copies_vec(copies, x, f.W, rows, f.kW, f.pad_w, flat_grid_tc(rows * (f.W / 8)), st, skip))
    conv_shift_copies_kernel<T><<<flat_grid_tc(rows * ((f.W + 7) / 8)), 256, 0, st>>>(copies, (const T*)x, f.W, rows, f.kW, f.pad_w, skip);
  LB2_CHECK_LAUNCH("conv_tc shifted copies");
  if (w2.ok) {
    ConvWg2Params q{};
    q.n_img = g.batch; q.s_blocks = w2.s_blocks;
    q.kW = f.kW; q.kH = f.kH; q.chunks = w2.chunks; q.co_tiles = w2.co_tiles;
    q.splits = w2.splits; q.kb_total = w2.kb_total; q.kb_per_split = w2.kb_per_split;
    q.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((f.kW * 64) >> 3) << 17) | ((uint32_t)(kConvBM >> 4) << 24);
    q.desc_hi = (uint32_t)((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
    q.desc_lbo = 1u << 16;
    q.k_advance = 32u >> 4;
    q.partial = partial;
    q.status = device_status_word();
    LB2_REQUIRE(q.status != nullptr, LB2_LAUNCH_FAIL, "conv_tc: device status word unavailable");
    for (int th = 0; th < f.kH; ++th) q.row_shift[th] = (int16_t)((th - f.pad_h) * f.W);
    q.center_tw = skip;
    CUtensorMap mX2, mX0, mG2;
    if (!bf16_map_4d(&mX2, copies, (int64_t)f.W * f.Hi, f.Ck, f.N, f.kW, 64, 64) ||
        !bf16_map_4d(&mX0, x, (int64_t)f.W * f.Hi, f.Ck, f.N, 1, 64, 64) ||
        !bf16_map_4d(&mG2, gy, (int64_t)g.out[0] * g.out[1], g.cout, g.batch, 1, 64, 64))
      return fail(LB2_LAUNCH_FAIL, "conv_tc: cuTensorMapEncodeTiled failed");
    const int stage_bytes = kConvBM * 128 + f.kW * 64 * 128;
    int nst = (200 * 1024) / stage_bytes;
    if (nst > 8) nst = 8;
    const int smem2 = nst * stage_bytes + 1024 + 256 + 64 * 8;
    const int items2 = w2.groups * w2.splits;
    const int grid2 = items2 < sm_count() ? items2 : sm_count();
    auto launch2 = [&](auto kernel) -> int32_t {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
      if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "conv_tc: cannot reserve %d bytes of shared memory: %s", smem2, cudaGetErrorString(e));
      kernel<<<grid2, kConvThreads, smem2, st>>>(mX2, mX0, mG2, q);
      LB2_CHECK_LAUNCH("conv_tc_wgrad2");
      return LB2_OK;
    };
    int32_t rc2 = f.kW == 1 ? launch2(conv_tc_wgrad2_kernel<1>) : f.kW == 2 ? launch2(conv_tc_wgrad2_kernel<2>)
                : f.kW == 3 ? launch2(conv_tc_wgrad2_kernel<3>) : launch2(conv_tc_wgrad2_kernel<4>);
    if (rc2 != LB2_OK) return rc2;
    const int64_t nw2 = (int64_t)g.k[0] * g.k[1] * g.cin * g.cout;
    conv_wgrad2_reduce_kernel<T><<<flat_grid_tc(nw2), 256, 0, st>>>((T*)dw, partial, g.k[0], g.k[1], g.cin, g.cout, g.flip, w2.chunks,
                                                                 w2.co_tiles, w2.splits);
    LB2_CHECK_LAUNCH("conv_wgrad2_reduce");
    return LB2_OK;
  }
  return fail(LB2_BAD_SHAPE, "conv_tc: geometry outside the resident-filter fast case");
}

}  // namespace lb2

// General tensor-core convolution for sm_100a (bf16 storage, fp32 accumulation in TMEM): implicit GEMM for any
// 2-D ConvDims with groups == 1 — any stride, padding, dilation, kernel size and channel counts — which is what
// the layers of a ResNet need beyond the stride-1 64-channel case served by conv_tc.cu (strided 3x3 and 1x1
// convolutions, the 7x7 stem, 128/256/512-channel stages whose filters do not fit in shared memory).
//
// Layout. The arrays at the boundary are WHCN (width contiguous). A kernel tap shifts the input by single elements
// along W, which a TMA tile cannot start on (16-byte rule) while W is the contiguous index. So every operand that
// is read through shifted windows is first rewritten channel-innermost ("CWHN": c contiguous, then w, h, n; the
// channel count padded to a multiple of 8) by one bandwidth pass into the caller's workspace. On that copy a tap
// shift, the padding (out-of-range rows are zero-filled by TMA) and the stride (TMA traversal stride) are all
// start coordinates / box parameters of a 4-D tensor map, and a tile of 64 channels x up to 128 positions lands in
// shared memory as a K-major, 128-byte-swizzled MMA operand. Outputs are written straight in WHCN.
//
//   forward        y[pos, co]  = sum over (tap, 64-channel chunk) of  Xc[pos + tap, ci] * Wp[co, (tap, ci)]
//                  M = 128 output positions (a w x h x image box), N = 64 / 128 / 256 output channels
//   data gradient  the same kernel on the channel-innermost copy of dy with the filter transposed; for stride s the
//                  input positions split into s*s classes by (w mod s, h mod s), each class being a stride-1
//                  problem over the taps that reach it, written to its strided subset of dx
//   filter grad.   dw[co, (tap, ci)] = sum over positions of  dYc[pos, co] * Xc[pos + tap, ci]: M = 128 output
//                  channels, N = up to four (tap, 64-channel chunk) column groups side by side (each loaded by its
//                  own TMA box), contraction over 64-position blocks split over CTAs; fp32 partials per split and a
//                  fixed-order reduction (deterministic)
// A small-channel input whose kW taps fit one 64-channel chunk together (the 3-channel stem) is copied with the kW
// taps folded into the channel index, so a kernel row costs one k-block instead of kW; when the stride along H is
// s >= 2 and s kernel rows fit the chunk as well, s rows are folded too (row s*q - pad + d of the input becomes
// channel group d of row q of the copy), which turns the kH taps into ceil(kH / s) stride-1 taps along q.
//
// All kernels are persistent, warp-specialised (TMA producer, MMA issuer, TMEM allocator, eight epilogue warps) with
// bounded mbarrier waits, like the GEMM kernels. Roofline: tensor pipe; algorithmic FLOPs = 2*Wo*Ho*N*Cout*Cin*kW*kH
// per pass.
#include "conv.cuh"
#include "tc_ptx.cuh"

namespace lb2 {

namespace {

constexpr int kCwThreads = 384;
constexpr int kCwBM = 128;
constexpr int kCwMaxKb = 160;     // k-blocks (tap x 64-channel chunk) per launch

inline int round_up(int v, int a) { return (v + a - 1) / a * a; }

// ----------------------------------------------------------------------------------------------
// layout passes
// ----------------------------------------------------------------------------------------------
// out[n][s][c] (c contiguous, Cp channels, zero beyond C)  <-  in[n][c][s] (s = w + W*h contiguous): per image a
// C x S matrix is transposed in 64 x 64 tiles through shared memory. VW = elements per global load (8: 16-byte
// loads when the planes are 16-byte aligned, i.e. S % 8 == 0; 4 for S % 4 == 0; 1 otherwise); stores are always
// 16 bytes wide along c (Cp is a multiple of 8).
template <int VW>
__global__ void __launch_bounds__(256) cw_transpose_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ in,
                                                           int S, int C, int Cp, int N) {
  constexpr int PITCH = 66;                         // elements per tile row: 33 words, odd, spreads the banks
  __shared__ uint16_t tile[64 * PITCH];
  const int st = (S + 63) / 64, ct = (Cp + 63) / 64;
  const int64_t blocks = (int64_t)N * st * ct;
  for (int64_t b = blockIdx.x; b < blocks; b += gridDim.x) {
    int64_t r = b;
    const int ci = (int)(r % ct); r /= ct;
    const int si = (int)(r % st);
    const int n = (int)(r / st);
    const int s0 = si * 64, c0 = ci * 64;
    __syncthreads();
    // load: rows of the tile = channels, VW consecutive s per thread
    constexpr int VPR = 64 / VW;                    // vectors per row
    for (int v = threadIdx.x; v < 64 * VPR; v += 256) {
      const int j = v / VPR, q = (v % VPR) * VW;
      const int c = c0 + j, sx = s0 + q;
      uint16_t e[VW];
      if (c < C && sx + VW <= S) {
        const uint16_t* src = in + ((int64_t)n * C + c) * S + sx;
        if constexpr (VW == 8) {
          const uint4 u = __ldg(reinterpret_cast<const uint4*>(src));
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) { e[2 * k] = (uint16_t)(w[k] & 0xFFFFu); e[2 * k + 1] = (uint16_t)(w[k] >> 16); }
        } else if constexpr (VW == 4) {
          const uint2 u = __ldg(reinterpret_cast<const uint2*>(src));
          e[0] = (uint16_t)(u.x & 0xFFFFu); e[1] = (uint16_t)(u.x >> 16); e[2] = (uint16_t)(u.y & 0xFFFFu); e[3] = (uint16_t)(u.y >> 16);
        } else {
          e[0] = src[0];
        }
      } else {
#pragma unroll
        for (int k = 0; k < VW; ++k) e[k] = (c < C && sx + k < S) ? in[((int64_t)n * C + c) * S + sx + k] : (uint16_t)0;
      }
#pragma unroll
      for (int k = 0; k < VW; ++k) tile[j * PITCH + q + k] = e[k];
    }
    __syncthreads();
    // store: rows = positions, 8 consecutive channels (16 bytes) per thread
    for (int v = threadIdx.x; v < 64 * 8; v += 256) {
      const int j = v / 8, q = (v % 8) * 8;
      const int sx = s0 + j, c = c0 + q;
      if (sx < S && c < Cp) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
          w[k] = (uint32_t)tile[(q + 2 * k) * PITCH + j] | ((uint32_t)tile[(q + 2 * k + 1) * PITCH + j] << 16);
        *reinterpret_cast<uint4*>(out + ((int64_t)n * S + sx) * Cp + c) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
}

// Folded copy for small channel counts: out[n][q][ow][(d*kW + tw)*C + c] = in[n][c][hq][ow*s + tw*dil - pad] (0 outside),
// hq = q when only the kW taps are folded (FR = 1, d = 0), hq = sh*q - pad_h + d when FR = sh kernel rows are folded
// too. Channels padded with zeros to Cp. One thread per group of 8 output channels (one 16-byte store).
__global__ void __launch_bounds__(256) cw_transpose_fold_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ in,
                                                                int W, int H, int C, int Cp, int N, int OW, int HQ, int kW,
                                                                int s, int dil, int pad, int FR, int sh, int pad_h) {
  const int groups = Cp / 8;
  const int64_t total = (int64_t)N * HQ * OW * groups;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i;
    const int qg = (int)(r % groups); r /= groups;
    const int ow = (int)(r % OW); r /= OW;
    const int q = (int)(r % HQ);
    const int n = (int)(r / HQ);
    uint16_t e[8];
    // (d, tw, c) of the group's first channel by division, of the following seven by carrying
    int d = (qg * 8) / (kW * C), rem = (qg * 8) % (kW * C);
    int tw = rem / C, c = rem % C;
    const uint16_t* plane0 = in + (int64_t)n * C * H * W;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      uint16_t v = 0;
      if (d < FR) {
        const int w = ow * s + tw * dil - pad;
        const int h = FR >= 2 ? sh * q - pad_h + d : q;
        if (w >= 0 && w < W && h >= 0 && h < H) v = __ldg(plane0 + ((int64_t)c * H + h) * W + w);
      }
      e[k] = v;
      if (++c == C) { c = 0; if (++tw == kW) { tw = 0; ++d; } }
    }
    *reinterpret_cast<uint4*>(out + i * 8) = make_uint4((uint32_t)e[0] | ((uint32_t)e[1] << 16), (uint32_t)e[2] | ((uint32_t)e[3] << 16),
                                                      (uint32_t)e[4] | ((uint32_t)e[5] << 16), (uint32_t)e[6] | ((uint32_t)e[7] << 16));
  }
}

// Packed filter Wp[row][tap][chunk][64]. Forward: row = co, contracted channel = ci. Data gradient (transpose): row =
// ci, contracted channel = co. tap = th*kW + tw in tap positions (filter index = flip ? t : K-1-t per dim).
// fold >= 1: the contracted index of a tap is (d, tw, ci) in ONE chunk, d < fold kernel rows per tap (fold = 1: taps
// run over th; fold = s >= 2: tap p covers kernel rows s*p .. s*p + s - 1).
struct CwPack {
  int kW, kH, cin, cout, flip, transpose, fold, chunks, n_rows, k_total;
};
__global__ void __launch_bounds__(256) cw_pack_filter_kernel(__nv_bfloat16* __restrict__ wp, const __nv_bfloat16* __restrict__ w,
                                                             const CwPack g) {
  const int64_t total = (int64_t)g.n_rows * g.k_total;
  const int kc = g.transpose ? g.cout : g.cin;
  const int nc = g.transpose ? g.cin : g.cout;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int row = (int)(i / g.k_total);
    const int col = (int)(i % g.k_total);
    const int kb = col / 64, j = col % 64;
    float v = 0.f;
    if (row < nc) {
      int tw, th, c;
      bool live;
      if (g.fold) {
        const int d = j / (g.kW * g.cin), rem = j % (g.kW * g.cin);
        th = g.fold >= 2 ? g.fold * kb + d : kb;
        tw = rem / g.cin; c = rem % g.cin;
        live = d < g.fold && th < g.kH;
      } else {
        const int tap = kb / g.chunks;
        tw = tap % g.kW; th = tap / g.kW;
        c = (kb % g.chunks) * 64 + j;
        live = c < kc;
      }
      if (live) {
        const int kw = g.flip ? tw : g.kW - 1 - tw, kh = g.flip ? th : g.kH - 1 - th;
        const int ci = g.transpose ? row : c, co = g.transpose ? c : row;
        v = __bfloat162float(w[((int64_t)(co * g.cin + ci) * g.kH + kh) * g.kW + kw]);
      }
    }
    wp[i] = __float2bfloat16_rn(v);
  }
}

// The same packing for unfolded filters, one block per (packed row, 64-channel chunk): the block's kW*kH x 64 filter
// elements are read in the filter's own order (one contiguous run for the forward packing, 64 runs of kW*kH elements for
// the data-gradient packing), turned in shared memory and written as kW*kH runs of 128 bytes. The flat kernel above reads
// 2-byte elements kW*kH (forward) or kW*kH*cin (data gradient) apart.
__global__ void __launch_bounds__(256) cw_pack_filter_rows_kernel(__nv_bfloat16* __restrict__ wp, const __nv_bfloat16* __restrict__ w,
                                                                  const CwPack g) {
  extern __shared__ __nv_bfloat16 cw_pack_tile[];   // [64 contracted channels][taps], the filter's (kh, kw) order
  const int taps = g.kW * g.kH;
  const int kc = g.transpose ? g.cout : g.cin;
  const int nc = g.transpose ? g.cin : g.cout;
  const int chunk = blockIdx.x % g.chunks, row = blockIdx.x / g.chunks;
  const int n_c = row < nc ? min(64, kc - chunk * 64) : 0;
  for (int e = threadIdx.x; e < 64 * taps; e += 256) {
    const int c = e / taps, t = e - c * taps;
    __nv_bfloat16 v = __float2bfloat16_rn(0.f);
    if (c < n_c) {
      const int64_t src = g.transpose ? ((int64_t)(chunk * 64 + c) * g.cin + row) * taps + t
                                      : ((int64_t)row * g.cin + chunk * 64) * taps + e;
      v = w[src];
    }
    cw_pack_tile[e] = v;
  }
  __syncthreads();
  __nv_bfloat16* dst = wp + (int64_t)row * g.k_total + chunk * 64;
  for (int e = threadIdx.x; e < 64 * taps; e += 256) {
    const int tap = e >> 6, j = e & 63;
    const int tw = tap % g.kW, th = tap / g.kW;
    const int kw = g.flip ? tw : g.kW - 1 - tw, kh = g.flip ? th : g.kH - 1 - th;
    dst[(int64_t)tap * g.chunks * 64 + j] = cw_pack_tile[j * taps + kh * g.kW + kw];
  }
}

unsigned flat_grid(int64_t total);

// filter packing of either kind
static void cw_pack_filter(__nv_bfloat16* wp, const __nv_bfloat16* w, const CwPack& pk, cudaStream_t st) {
  const size_t tile = (size_t)pk.kW * pk.kH * 64 * sizeof(__nv_bfloat16);
  if (pk.fold == 0 && tile <= 48 * 1024)
    cw_pack_filter_rows_kernel<<<(unsigned)((int64_t)pk.n_rows * pk.chunks), 256, tile, st>>>(wp, w, pk);
  else
    cw_pack_filter_kernel<<<flat_grid((int64_t)pk.n_rows * pk.k_total), 256, 0, st>>>(wp, w, pk);
}

// ----------------------------------------------------------------------------------------------
// forward / data-gradient kernel
// ----------------------------------------------------------------------------------------------
struct CwFwdParams {
  // grid of output positions of this (sub)problem and its tiling: a tile is a BW x BH x BI box of positions
  int32_t OW, OH, NI;
  int32_t BW, BH, BI;
  int32_t tiles_w, tiles_h, tiles_i, tiles_n;
  int32_t sw, sh;              // input coordinate step per output position (the TMA traversal stride)
  int32_t n_out;               // output channels of the GEMM
  int32_t num_kb;
  // where position (a, b) of the grid lands in the output array (full extents FW x FH, channel planes of FW*FH)
  int32_t FW, FH, ow_step, ow_off, oh_step, oh_off;
  uint32_t idesc;
  void* y;
  void* preact;
  const void* bias;
  int32_t act;
  unsigned int* status;
  float* sums_partial;         // SUMS kernels: [gridDim.x][BN][2] per-CTA sums of y and y^2 per channel of the CTA's column tile
  int16_t kb_dw[kCwMaxKb], kb_dh[kCwMaxKb];   // input start coordinate offsets of the k-block's tap
  int16_t kb_c0[kCwMaxKb];                    // first contracted channel
  int32_t kb_k0[kCwMaxKb];                    // column of the packed filter
};

constexpr uint32_t kDescHiSw128 = (uint32_t)((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);

// Sum over the 32 lanes of a warp of v[j], for each j: lane j ends up with the sum of everybody's v[j] (a butterfly
// that halves the values a lane carries at every step: 31 shuffles for 32 sums instead of 160; fixed order).
__device__ __forceinline__ float warp_transpose_sum(float (&v)[32], int lane) {
#pragma unroll
  for (int k = 16; k >= 1; k >>= 1) {
    const bool up = (lane & k) != 0;
#pragma unroll
    for (int i = 0; i < k; ++i) {
      const float send = up ? v[i] : v[i + k];
      const float keep = up ? v[i + k] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, k);
    }
  }
  return v[0];
}

// SUMS: the epilogue also forms, per output channel, the sums of the STORED values y and of y^2 over every position
// this CTA writes (what a BatchNorm statistics pass over y would read back from memory). The grid is a multiple of
// tiles_n, so a CTA always works on the same column tile and a lane can keep "its" channel's running sums in
// registers (lane j of an epilogue warp owns channel j of each 32-column chunk of the warp's half); at the end the
// four warps that share the channels (the TMEM lane quarters) are added in order and the CTA writes one partial row.
template <int BN, int ACT, bool SUMS = false>
__global__ void __launch_bounds__(kCwThreads, 1)
conv_cw_fwd_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const __grid_constant__ CwFwdParams p) {
  constexpr int A_BYTES = kCwBM * 128;
  constexpr int B_BYTES = BN * 128;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int STAGES = (200 * 1024) / STAGE_BYTES > 8 ? 8 : (200 * 1024) / STAGE_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32u : (uint32_t)(2 * BN);
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
  const int num_tiles = p.tiles_w * p.tiles_h * p.tiles_i * p.tiles_n;
  const uint32_t a_bytes = (uint32_t)(p.BW * p.BH * p.BI * 128);   // bytes one A box writes (64 channels x positions)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Rows of an A stage beyond the box (positions past BW*BH*BI) are never written by TMA. They only feed
  // accumulator rows that are never stored; the ring is zeroed once so that nothing undefined enters the MMAs.
  for (int i = threadIdx.x * 16; i < STAGES * STAGE_BYTES; i += blockDim.x * 16)
    *reinterpret_cast<uint4*>(smem_gen + i) = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  if (warp == 2) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (co tile fastest, w tile, h tile, image tile)
  auto tile_coords = [&](int tile, int* tn, int* tw, int* th, int* ti) {
    *tn = tile % p.tiles_n; tile /= p.tiles_n;
    *tw = tile % p.tiles_w; tile /= p.tiles_w;
    *th = tile % p.tiles_h;
    *ti = tile / p.tiles_h;
  };

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      tma_prefetch_desc(&tmW);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tn, tw, th, ti;
        tile_coords(tile, &tn, &tw, &th, &ti);
        const int w0 = tw * p.BW * p.sw, h0 = th * p.BH * p.sh, i0 = ti * p.BI, n0 = tn * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, p.status, 0x1000u)) { ok = false; break; }
          mbar_expect_tx(&full[stage], a_bytes + (uint32_t)B_BYTES);
          const uint32_t sA = smem_base + stage * STAGE_BYTES, sB = sA + A_BYTES;
          tma_load_4d(sA, &tmX, p.kb_c0[kb], w0 + p.kb_dw[kb], h0 + p.kb_dh[kb], i0, &full[stage]);
          tma_load_2d(sB, &tmW, p.kb_k0[kb], n0, &full[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, p.status, 0x2000u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, p.status, 0x4000u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * STAGE_BYTES, sB = sA + A_BYTES;
          const uint32_t a_lo32 = ((sA >> 4) & 0x3FFFu) | (1u << 16);
          const uint32_t b_lo32 = ((sB >> 4) & 0x3FFFu) | (1u << 16);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t ad = ((uint64_t)kDescHiSw128 << 32) | (uint64_t)(a_lo32 + ks * 2);
            const uint64_t bd = ((uint64_t)kDescHiSw128 << 32) | (uint64_t)(b_lo32 + ks * 2);
            umma<false>(d_tmem, ad, bd, p.idesc, (kb | ks) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp >= 4) {
    // Two warps share each TMEM lane quarter and split the tile's channels. A thread owns one output position and
    // walks its channels with a pointer stride of one channel plane.
    const int q = warp & 3, half = (warp - 4) >> 2;
    constexpr int COLS = BN / 2;
    uint32_t acc = 0, acc_phase = 0;
    __nv_bfloat16* Y = reinterpret_cast<__nv_bfloat16*>(p.y);
    __nv_bfloat16* P = reinterpret_cast<__nv_bfloat16*>(p.preact);
    const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(p.bias);
    const int64_t plane = (int64_t)p.FW * p.FH;
    const int pos = q * 32 + lane;
    const int iw = pos % p.BW, ih = (pos / p.BW) % p.BH, ii = pos / (p.BW * p.BH);
    bool ok = true;
    float run_s[COLS / 32], run_q[COLS / 32];          // SUMS: this lane's channel of every chunk
#pragma unroll
    for (int c = 0; c < COLS / 32; ++c) { run_s[c] = 0.f; run_q[c] = 0.f; }
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tn, tw, th, ti;
      tile_coords(tile, &tn, &tw, &th, &ti);
      if (!mbar_wait_warp(&acc_full[acc], acc_phase, p.status, 0x8000u)) { ok = false; break; }
      tc_fence_after();
      const int a = tw * p.BW + iw, b = th * p.BH + ih, img = ti * p.BI + ii;
      const bool live = ii < p.BI && a < p.OW && b < p.OH && img < p.NI;
      const int col0 = tn * BN + half * COLS;
      const int lim = min(COLS, p.n_out - col0);
      const int64_t base = (int64_t)(a * p.ow_step + p.ow_off) + (int64_t)p.FW * (b * p.oh_step + p.oh_off) +
                           plane * ((int64_t)p.n_out * img + col0);
      __nv_bfloat16* yp = Y + base;
      __nv_bfloat16* pp = P != nullptr ? P + base : nullptr;
      if constexpr (SUMS) {
#pragma unroll
        for (int c = 0; c < COLS / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + half * COLS + c * 32, r);
          tmem_ld_wait();
          float sv[32], sq[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float stored = 0.f;
            if (live && c * 32 + j < lim) {
              float v = __uint_as_float(r[j]);
              if (bias != nullptr) v += __bfloat162float(bias[col0 + c * 32 + j]);
              const __nv_bfloat16 o = __float2bfloat16_rn(act_apply_any<ACT, true>(p.act, v));
              yp[j * plane] = o;
              stored = __bfloat162float(o);
            }
            sv[j] = stored;
            sq[j] = stored * stored;
          }
          run_s[c] += warp_transpose_sum(sv, lane);
          run_q[c] += warp_transpose_sum(sq, lane);
          yp += 32 * plane;
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < COLS / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + half * COLS + c * 32, r);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (c * 32 + j < lim) {
                float v = __uint_as_float(r[j]);
                if (bias != nullptr) v += __bfloat162float(bias[col0 + c * 32 + j]);
                if (pp != nullptr) pp[j * plane] = __float2bfloat16_rn(v);
                yp[j * plane] = __float2bfloat16_rn(act_apply_any<ACT, true>(p.act, v));
              }
            }
          }
          yp += 32 * plane;
          if (pp != nullptr) pp += 32 * plane;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if constexpr (SUMS) {
      // every tile of this CTA is finished (its loads consumed, its accumulators read), so the operand ring is free:
      // the eight warps park their sums there, [q][half][chunk][lane] pairs
      float2* park = reinterpret_cast<float2*>(smem_gen);
#pragma unroll
      for (int c = 0; c < COLS / 32; ++c) park[((q * 2 + half) * (COLS / 32) + c) * 32 + lane] = make_float2(run_s[c], run_q[c]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if constexpr (SUMS) {
    constexpr int COLS = BN / 2;
    if (warp >= 4 && (warp & 3) == 0) {          // one warp per half adds the four lane quarters in order
      const int half = (warp - 4) >> 2;
      const float2* park = reinterpret_cast<const float2*>(smem_gen);
      float* out = p.sums_partial + (int64_t)blockIdx.x * BN * 2;
#pragma unroll
      for (int c = 0; c < COLS / 32; ++c) {
        float sum = 0.f, sqs = 0.f;
#pragma unroll
        for (int qi = 0; qi < 4; ++qi) {
          const float2 v = park[((qi * 2 + half) * (COLS / 32) + c) * 32 + lane];
          sum += v.x;
          sqs += v.y;
        }
        const int ch = half * COLS + c * 32 + lane;
        out[ch * 2] = sum;
        out[ch * 2 + 1] = sqs;
      }
    }
  }
  if (warp == 2) {
    if (*reinterpret_cast<volatile unsigned int*>(p.status) != 0) drain_after_abort();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------------------------
// filter-gradient kernel
// ----------------------------------------------------------------------------------------------
struct CwWgParams {
  int32_t OW, OH, NI;                 // output (dy) grid
  int32_t KW_, KH_, KI_;              // a k-block is a KW_ x KH_ x KI_ box of output positions (64 in all)
  int32_t kbw, kbh, kbi;              // k-blocks along each of them
  int32_t sw, sh;                     // input step per output position
  int32_t co_tiles, groups, pairs_per_group, n_pairs;
  int32_t splits, kb_total, kb_per_split;
  uint32_t idesc;
  float* partial;                     // [splits][co_tiles][groups][128][pairs_per_group*64]
  unsigned int* status;
  int16_t pr_dw[kCwMaxKb], pr_dh[kCwMaxKb], pr_c0[kCwMaxKb];   // per (tap, chunk) pair: input offsets, first channel
};

template <int NP>   // column groups per MMA: N = NP * 64
__global__ void __launch_bounds__(kCwThreads, 1)
conv_cw_wgrad_kernel(const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmX,
                     const __grid_constant__ CwWgParams p) {
  constexpr int BN = NP * 64;
  constexpr int A_BYTES = kCwBM * 128;       // 128 output channels (two 64-wide boxes) x 64 positions
  constexpr int B_BYTES = BN * 128;          // NP column groups x 64 positions
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int STAGES = (200 * 1024) / STAGE_BYTES > 8 ? 8 : (200 * 1024) / STAGE_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN <= 128 ? 128u : (2 * BN <= 256 ? 256u : 512u);
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
  const int per_split = p.co_tiles * p.groups;
  const int num_items = per_split * p.splits;

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

  // item -> (co tile fastest, group, split)
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmG);
      tma_prefetch_desc(&tmX);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int ct = item % p.co_tiles, grp = (item / p.co_tiles) % p.groups, z = item / per_split;
        const int kb_lo = z * p.kb_per_split, kb_hi = min(p.kb_total, kb_lo + p.kb_per_split);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, p.status, 0x20000u)) { ok = false; break; }
          const int bw = kb % p.kbw, bh = (kb / p.kbw) % p.kbh, bi = kb / (p.kbw * p.kbh);
          const int a0 = bw * p.KW_, b0 = bh * p.KH_, i0 = bi * p.KI_;
          const uint32_t sA = smem_base + stage * STAGE_BYTES, sB = sA + A_BYTES;
          mbar_expect_tx(&full[stage], (uint32_t)STAGE_BYTES);
          tma_load_4d(sA, &tmG, ct * 128, a0, b0, i0, &full[stage]);
          tma_load_4d(sA + A_BYTES / 2, &tmG, ct * 128 + 64, a0, b0, i0, &full[stage]);   // channels past the last are zero-filled
#pragma unroll
          for (int j = 0; j < NP; ++j) {
            int pr = grp * p.pairs_per_group + j;
            if (pr >= p.n_pairs) pr = grp * p.pairs_per_group;   // filler column group (its results are never read)
            tma_load_4d(sB + j * (64 * 128), &tmX, p.pr_c0[pr], a0 * p.sw + p.pr_dw[pr], b0 * p.sh + p.pr_dh[pr], i0, &full[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      // both operands MN-major: 64-wide groups of the non-contracted index are 8192 bytes apart (LBO), eight
      // positions form a 1024-byte swizzle atom (SBO), one MMA step covers 16 positions = 2048 bytes
      constexpr uint32_t LBO = ((8192u >> 4) & 0x3FFFu) << 16;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int z = item / per_split;
        const int kb_lo = z * p.kb_per_split, kb_hi = min(p.kb_total, kb_lo + p.kb_per_split);
        if (kb_lo >= kb_hi) continue;   // an empty split contributes nothing (the epilogue writes zeros)
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, p.status, 0x40000u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full[stage], phase, p.status, 0x80000u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * STAGE_BYTES, sB = sA + A_BYTES;
          const uint32_t a_lo32 = ((sA >> 4) & 0x3FFFu) | LBO;
          const uint32_t b_lo32 = ((sB >> 4) & 0x3FFFu) | LBO;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t ad = ((uint64_t)kDescHiSw128 << 32) | (uint64_t)(a_lo32 + ks * (2048u >> 4));
            const uint64_t bd = ((uint64_t)kDescHiSw128 << 32) | (uint64_t)(b_lo32 + ks * (2048u >> 4));
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
    const int q = warp & 3, half = (warp - 4) >> 2;
    constexpr int COLS = BN / 2;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const int z = item / per_split;
      const bool empty_range = z * p.kb_per_split >= p.kb_total;
      if (!empty_range) {
        if (!mbar_wait_warp(&acc_full[acc], acc_phase, p.status, 0x100000u)) { ok = false; break; }
        tc_fence_after();
      }
      const int row = q * 32 + lane;
      float* dst = p.partial + ((int64_t)item * 128 + row) * BN + half * COLS;
#pragma unroll 1
      for (int c = 0; c < COLS / 32; ++c) {
        uint32_t r[32];
        if (!empty_range) {
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + half * COLS + c * 32, r);
          tmem_ld_wait();
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[c * 32 + j] = empty_range ? 0.f : __uint_as_float(r[j]);
      }
      if (!empty_range) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (*reinterpret_cast<volatile unsigned int*>(p.status) != 0) drain_after_abort();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// dw[kw,kh,ci,co] = sum over splits (ascending) of partial[z][co tile][group][co % 128][slot*64 + column]
struct CwReduce {
  int kW, kH, cin, cout, flip, fold, chunks, co_tiles, groups, pairs_per_group, splits;
};
// Sums the split-K partials and scatters them into dw. A block takes one 64-column slot of one partial row, i.e. one
// (output channel, (tap, chunk) pair): thread x reads consecutive floats (coalesced, where the old per-output indexing
// read 4 scattered bytes per split), the four y slices add splits y, y + 4, ... in ascending order and are then added
// in slice order (a fixed order); the destination index is rebuilt from (pair, column).
constexpr int kCwReduceSlices = 4;
template <typename T>
__global__ void __launch_bounds__(64 * kCwReduceSlices) conv_cw_wgrad_reduce_kernel(T* __restrict__ dw, const float* __restrict__ partial,
                                                                                    const CwReduce g) {
  __shared__ float part[kCwReduceSlices][64];
  const int bn = g.pairs_per_group * 64;
  const int64_t split_stride = (int64_t)g.co_tiles * g.groups * 128 * bn;
  // blockIdx.x -> (slot, row, co tile, group), slot fastest
  int64_t r = blockIdx.x;
  const int slot = (int)(r % g.pairs_per_group); r /= g.pairs_per_group;
  const int row = (int)(r % 128); r /= 128;
  const int ct = (int)(r % g.co_tiles);
  const int grp = (int)(r / g.co_tiles);
  const int co = ct * 128 + row;
  const int pair = grp * g.pairs_per_group + slot;
  const int n_taps = g.fold >= 2 ? (g.kH + g.fold - 1) / g.fold : (g.fold ? g.kH : g.kW * g.kH);
  if (co >= g.cout || pair >= n_taps * g.chunks) return;
  const int col = threadIdx.x;
  const int64_t off = (((int64_t)(grp * g.co_tiles + ct)) * 128 + row) * bn + slot * 64 + col;
  float s = 0.f;
  for (int z = threadIdx.y; z < g.splits; z += kCwReduceSlices) s += partial[z * split_stride + off];
  part[threadIdx.y][col] = s;
  __syncthreads();
  if (threadIdx.y != 0) return;
#pragma unroll
  for (int y = 1; y < kCwReduceSlices; ++y) s += part[y][col];
  int tw, th, ci;
  if (g.fold >= 2) {
    const int q = col / g.cin;
    ci = col % g.cin;
    tw = q % g.kW;
    const int thm = q / g.kW;
    th = pair * g.fold + thm;
    if (thm >= g.fold || th >= g.kH) return;
  } else if (g.fold) {
    tw = col / g.cin;
    ci = col % g.cin;
    th = pair;
    if (tw >= g.kW) return;
  } else {
    const int tap = pair / g.chunks;
    ci = (pair % g.chunks) * 64 + col;
    if (ci >= g.cin) return;
    th = tap / g.kW;
    tw = tap % g.kW;
  }
  const int kw = g.flip ? tw : g.kW - 1 - tw, kh = g.flip ? th : g.kH - 1 - th;
  dw[kw + (int64_t)g.kW * (kh + (int64_t)g.kH * (ci + (int64_t)g.cin * co))] = from_f32<T>(s);
}

// The same sum for unfolded filters (every layer but a small-channel stem), one block per (output channel, 64-channel
// chunk of the input): the four y slices take taps y, y + 4, ..., each thread adds the splits of its (tap, input channel)
// in ascending order from consecutive floats of the partial rows, the block collects the kW*kH x 64 values in shared
// memory in dw's own order and writes them as ONE contiguous run of dw (the per-slot kernel above writes 2-byte elements
// kW*kH apart and needs a block per 64 outputs: 36864 blocks of one load each for a 3x3 512->512 filter).
template <typename T>
__global__ void __launch_bounds__(256) conv_cw_wgrad_reduce_rows_kernel(T* __restrict__ dw, const float* __restrict__ partial,
                                                                        const CwReduce g) {
  extern __shared__ float cw_reduce_tile[];   // [64 input channels][taps], dw's order
  const int taps = g.kW * g.kH;
  const int chunk = blockIdx.x % g.chunks, co = blockIdx.x / g.chunks;
  const int ct = co / 128, row = co % 128;
  const int bn = g.pairs_per_group * 64;
  const int64_t split_stride = (int64_t)g.co_tiles * g.groups * 128 * bn;
  const int col = threadIdx.x & 63, y = threadIdx.x >> 6;
  for (int tap = y; tap < taps; tap += 4) {
    const int pair = tap * g.chunks + chunk;
    const int grp = pair / g.pairs_per_group, slot = pair % g.pairs_per_group;
    const float* src = partial + (((int64_t)(grp * g.co_tiles + ct)) * 128 + row) * bn + slot * 64 + col;
    float s = 0.f;
#pragma unroll 4
    for (int z = 0; z < g.splits; ++z) s += __ldcs(src + z * split_stride);
    const int th = tap / g.kW, tw = tap % g.kW;
    const int kw = g.flip ? tw : g.kW - 1 - tw, kh = g.flip ? th : g.kH - 1 - th;
    cw_reduce_tile[col * taps + kw + g.kW * kh] = s;
  }
  __syncthreads();
  const int n_ci = min(64, g.cin - chunk * 64);
  T* dst = dw + ((int64_t)co * g.cin + chunk * 64) * taps;
  for (int e = threadIdx.x; e < n_ci * taps; e += 256) dst[e] = from_f32<T>(cw_reduce_tile[e]);
}

// ----------------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------------
// 4-D map over a channel-innermost array (Cp, W, H, N): box = 64 channels x bw x bh x bi positions, traversal
// strides (sw, sh) along w and h. 128-byte swizzle (a box row is 64 channels = 128 bytes).
bool cw_map(CUtensorMap* map, const void* ptr, int Cp, int W, int H, int N, int bw, int bh, int bi, int sw, int sh) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc) return false;
  cuuint64_t dims[4] = {(cuuint64_t)Cp, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)Cp * 2, (cuuint64_t)Cp * W * 2, (cuuint64_t)Cp * W * H * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)(bw * sw), (cuuint32_t)(bh * sh), (cuuint32_t)bi};
  cuuint32_t estr[4] = {1, (cuuint32_t)sw, (cuuint32_t)sh, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool cw_map_2d(CUtensorMap* map, const void* ptr, int64_t d0, int64_t d1, int box0, int box1) {
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

unsigned flat_grid(int64_t total) {
  int64_t gsz = (total + 255) / 256, cap = (int64_t)sm_count() * 16;
  return (unsigned)(gsz < 1 ? 1 : (gsz > cap ? cap : gsz));
}

int cw_bn(int n_out) { return n_out <= 64 ? 64 : (n_out <= 128 ? 128 : 256); }

// Kernel rows folded into the channel index of the input copy together with the kW taps (forward and filter gradient
// of small-channel inputs): 0 = no folding, 1 = the kW taps only, s >= 2 = the s rows a stride-s step spans as well.
int cw_fold(const ConvGeom& g) {
  if (g.k[0] <= 1 || g.k[0] * g.cin > 64) return 0;
  const int sh = g.stride[1];
  if (sh >= 2 && g.dil[1] == 1 && g.k[1] > 1 && sh * g.k[0] * g.cin <= 64) return sh;
  return 1;
}
// taps (k-blocks per output tile) of a folded problem
int cw_fold_taps(const ConvGeom& g, int fold) { return fold >= 2 ? (g.k[1] + fold - 1) / fold : g.k[1]; }

struct CwCopy {      // channel-innermost copy of an activation array
  int Cp, W, H;      // padded channels, spatial extents of the copy (W = output width when folded)
  size_t bytes;
};
CwCopy cw_copy_of_x(const ConvGeom& g) {
  CwCopy c{};
  const int fold = cw_fold(g);
  if (fold) { c.Cp = round_up(fold * g.k[0] * g.cin, 8); c.W = g.out[0]; }
  else { c.Cp = round_up(g.cin, 8); c.W = g.in[0]; }
  c.H = fold >= 2 ? g.out[1] + cw_fold_taps(g, fold) - 1 : g.in[1];
  c.bytes = align_up((size_t)c.Cp * c.W * c.H * g.batch * 2, 1024);
  return c;
}
CwCopy cw_copy_of_y(const ConvGeom& g) {
  CwCopy c{};
  c.Cp = round_up(g.cout, 8); c.W = g.out[0]; c.H = g.out[1];
  c.bytes = align_up((size_t)c.Cp * c.W * c.H * g.batch * 2, 1024);
  return c;
}
size_t cw_packed_bytes(int n_rows_real, int taps, int chunks) {
  const int bn = cw_bn(n_rows_real);
  return align_up((size_t)round_up(n_rows_real, bn) * taps * chunks * 64 * 2, 1024);
}

// position box of a forward tile: whole rows when they fit, several rows / images per tile when rows are short
void cw_tile_box(int OW, int OH, int NI, int* BW, int* BH, int* BI) {
  *BW = OW < kCwBM ? OW : kCwBM;
  *BH = kCwBM / *BW; if (*BH > OH) *BH = OH; if (*BH < 1) *BH = 1;
  *BI = (*BH == OH) ? kCwBM / (*BW * *BH) : 1;
  if (*BI > NI) *BI = NI; if (*BI < 1) *BI = 1;
}

int32_t cw_transpose(void* out, const void* in, int W, int H, int C, int Cp, int N, cudaStream_t st) {
  const int S = W * H;
  const int64_t blocks = (int64_t)N * ((S + 63) / 64) * ((Cp + 63) / 64);
  const int64_t cap = (int64_t)sm_count() * 8;
  const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
  uint16_t* o = (uint16_t*)out;
  const uint16_t* i = (const uint16_t*)in;
  if (S % 8 == 0 && aligned_to(in, 16)) cw_transpose_kernel<8><<<grid, 256, 0, st>>>(o, i, S, C, Cp, N);
  else if (S % 4 == 0 && aligned_to(in, 8)) cw_transpose_kernel<4><<<grid, 256, 0, st>>>(o, i, S, C, Cp, N);
  else cw_transpose_kernel<1><<<grid, 256, 0, st>>>(o, i, S, C, Cp, N);
  LB2_CHECK_LAUNCH("conv_cw transpose");
  return LB2_OK;
}

int32_t cw_copy_x(void* xc, const void* x, const ConvGeom& g, const CwCopy& c, cudaStream_t st) {
  const int fold = cw_fold(g);
  if (fold) {
    cw_transpose_fold_kernel<<<flat_grid((int64_t)(c.Cp / 8) * c.W * c.H * g.batch), 256, 0, st>>>(
        (uint16_t*)xc, (const uint16_t*)x, g.in[0], g.in[1], g.cin, c.Cp, g.batch, g.out[0], c.H, g.k[0], g.stride[0], g.dil[0], g.pad_lo[0],
        fold, g.stride[1], g.pad_lo[1]);
    LB2_CHECK_LAUNCH("conv_cw folded copy");
    return LB2_OK;
  }
  return cw_transpose(xc, x, g.in[0], g.in[1], g.cin, c.Cp, g.batch, st);
}

template <int BN>
int32_t cw_launch_fwd(const CUtensorMap& mX, const CUtensorMap& mW, const CwFwdParams& p, int32_t act, cudaStream_t st, int* grid_out) {
  constexpr int STAGE_BYTES = kCwBM * 128 + BN * 128;
  constexpr int STAGES = (200 * 1024) / STAGE_BYTES > 8 ? 8 : (200 * 1024) / STAGE_BYTES;
  constexpr int smem = STAGES * STAGE_BYTES + 1024 + 256;
  const int tiles = p.tiles_w * p.tiles_h * p.tiles_i * p.tiles_n;
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (p.sums_partial != nullptr) {
    // a multiple of tiles_n (tiles is one): blockIdx.x % tiles_n is then the column tile of every tile of the CTA
    grid = grid / p.tiles_n * p.tiles_n;
    if (grid < p.tiles_n) grid = p.tiles_n;
  }
  if (grid_out != nullptr) *grid_out = grid;
  auto launch = [&](auto kernel) -> int32_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "conv_cw: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    kernel<<<grid, kCwThreads, smem, st>>>(mX, mW, p);
    LB2_CHECK_LAUNCH("conv_cw_fwd");
    return LB2_OK;
  };
  if (p.sums_partial != nullptr) {
    if (act == LB2_ACT_IDENTITY) return launch(conv_cw_fwd_kernel<BN, LB2_ACT_IDENTITY, true>);
    return launch(conv_cw_fwd_kernel<BN, -1, true>);
  }
  switch (act) {
    case LB2_ACT_IDENTITY: return launch(conv_cw_fwd_kernel<BN, LB2_ACT_IDENTITY>);
    case LB2_ACT_RELU: return launch(conv_cw_fwd_kernel<BN, LB2_ACT_RELU>);
    default: return launch(conv_cw_fwd_kernel<BN, -1>);
  }
}

// sums[ch][0..1] = sum over the CTAs of column tile ch / bn (ascending block index) of their partial rows
__global__ void __launch_bounds__(256) cw_sums_finish_kernel(float* __restrict__ sums, const float* __restrict__ partial, int grid, int tiles_n,
                                                             int bn, int cout) {
  // one warp per channel: lane l adds the CTA rows tn + (l, l + 32, ...) * tiles_n in ascending order, the lanes are
  // combined by a butterfly (a fixed order)
  const int ch = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (ch >= cout) return;
  const int tn = ch / bn, j = ch % bn;
  double a = 0.0, q = 0.0;
  for (int k = tn + lane * tiles_n; k < grid; k += 32 * tiles_n) {
    const float2 v = *reinterpret_cast<const float2*>(partial + ((int64_t)k * bn + j) * 2);
    a += (double)v.x;
    q += (double)v.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    q += __shfl_xor_sync(0xffffffffu, q, o);
  }
  if (lane == 0) {
    sums[ch * 2] = (float)a;
    sums[ch * 2 + 1] = (float)q;
  }
}

// One implicit-GEMM launch: grid of OW x OH x NI positions, n_out channels, the given taps of the packed filter.
struct CwTap { int dw, dh, tap_index; };
int32_t cw_run_gemm(void* out, void* preact, const void* bias, int32_t act, const void* src_c, int Cp_src, int Wsrc, int Hsrc,
                    int NI, int k_chunks, const void* wp, int wp_rows, int wp_cols, const CwTap* taps, int n_taps,
                    int OW, int OH, int sw, int sh, int n_out, int FW, int FH, int ow_step, int ow_off, int oh_step, int oh_off,
                    cudaStream_t st, float* sums = nullptr, float* sums_partial = nullptr) {
  CwFwdParams p{};
  p.OW = OW; p.OH = OH; p.NI = NI;
  cw_tile_box(OW, OH, NI, &p.BW, &p.BH, &p.BI);
  const int bn = cw_bn(n_out);
  p.tiles_w = (OW + p.BW - 1) / p.BW; p.tiles_h = (OH + p.BH - 1) / p.BH; p.tiles_i = (NI + p.BI - 1) / p.BI;
  p.tiles_n = (n_out + bn - 1) / bn;
  p.sw = sw; p.sh = sh; p.n_out = n_out;
  p.num_kb = n_taps * k_chunks;
  LB2_REQUIRE(p.num_kb >= 1 && p.num_kb <= kCwMaxKb, LB2_BAD_SHAPE, "conv_cw: %d k-blocks exceed the launch table", p.num_kb);
  for (int t = 0; t < n_taps; ++t)
    for (int ch = 0; ch < k_chunks; ++ch) {
      const int kb = t * k_chunks + ch;
      p.kb_dw[kb] = (int16_t)taps[t].dw; p.kb_dh[kb] = (int16_t)taps[t].dh;
      p.kb_c0[kb] = (int16_t)(ch * 64);
      p.kb_k0[kb] = (taps[t].tap_index * k_chunks + ch) * 64;
    }
  p.FW = FW; p.FH = FH; p.ow_step = ow_step; p.ow_off = ow_off; p.oh_step = oh_step; p.oh_off = oh_off;
  p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(kCwBM >> 4) << 24);
  p.y = out; p.preact = preact; p.bias = bias; p.act = act;
  p.sums_partial = sums != nullptr ? sums_partial : nullptr;
  p.status = device_status_word();
  LB2_REQUIRE(p.status != nullptr, LB2_LAUNCH_FAIL, "conv_cw: device status word unavailable");
  CUtensorMap mX, mW;
  if (!cw_map(&mX, src_c, Cp_src, Wsrc, Hsrc, NI, p.BW, p.BH, p.BI, sw, sh) || !cw_map_2d(&mW, wp, wp_cols, wp_rows, 64, bn))
    return fail(LB2_LAUNCH_FAIL, "conv_cw: cuTensorMapEncodeTiled failed");
  int grid = 0;
  const int32_t rc = bn == 64 ? cw_launch_fwd<64>(mX, mW, p, act, st, &grid)
                   : bn == 128 ? cw_launch_fwd<128>(mX, mW, p, act, st, &grid) : cw_launch_fwd<256>(mX, mW, p, act, st, &grid);
  if (rc != LB2_OK || sums == nullptr) return rc;
  cw_sums_finish_kernel<<<(unsigned)((n_out + 7) / 8), 256, 0, st>>>(sums, sums_partial, grid, p.tiles_n, bn, n_out);
  LB2_CHECK_LAUNCH("conv_cw channel sums");
  return LB2_OK;
}

}  // namespace

// ---- public (library-internal) interface ------------------------------------------------------------
// k-blocks (64-wide contraction steps) one output tile of the forward kernel takes: taps x channel chunks, or the
// folded tap count of a small-channel stem
int conv_cw_fwd_kblocks(const ConvGeom& g) {
  const int fold = cw_fold(g);
  return fold ? cw_fold_taps(g, fold) : g.k[0] * g.k[1] * ((g.cin + 63) / 64);
}

bool conv_cw_supported(const ConvGeom& g, int32_t dtype) {
  if (dtype != LB2_BF16 || g.ndim != 2 || g.groups != 1) return false;
  if (g.out[0] <= 0 || g.out[1] <= 0 || g.batch <= 0 || g.cin <= 0 || g.cout <= 0) return false;
  if (g.stride[0] > 4 || g.stride[1] > 4) return false;               // box extent = positions x stride must stay <= 256
  const int fold0 = cw_fold(g);
  const int chunks = fold0 ? 1 : (g.cin + 63) / 64, taps = fold0 ? cw_fold_taps(g, fold0) : g.k[0] * g.k[1];
  if (taps * chunks > kCwMaxKb) return false;
  if (g.k[0] * g.k[1] * ((g.cout + 63) / 64) > kCwMaxKb) return false;   // data gradient contracts over output channels
  if (g.k[0] * g.dil[0] > 120 || g.k[1] * g.dil[1] > 120) return false;
  int BW, BH, BI;
  cw_tile_box(g.out[0], g.out[1], g.batch, &BW, &BH, &BI);
  if (BW * g.stride[0] > 256 || BH * g.stride[1] > 256) return false;  // TMA box extents
  if ((int64_t)g.in[0] * g.in[1] * g.cin * g.batch >= ((int64_t)1 << 40)) return false;
  return tensor_map_encoder() != nullptr;
}

// per-CTA rows of the channel-sum partials: at most one CTA per SM, 256 channels, two floats
static size_t cw_sums_partial_bytes() { return align_up((size_t)sm_count() * 256 * 2 * sizeof(float), 1024); }

size_t conv_cw_fwd_workspace_bytes(const ConvGeom& g) {
  const int fold = cw_fold(g);
  return align_up(cw_copy_of_x(g).bytes + cw_packed_bytes(g.cout, fold ? cw_fold_taps(g, fold) : g.k[0] * g.k[1], fold ? 1 : (g.cin + 63) / 64), 1024) +
         cw_sums_partial_bytes();
}

// `sums` (fp32 [cout][2], may be null): per output channel the sums of the stored y and of y^2, formed in the epilogue
int32_t conv_cw_fwd(void* y, void* preact, const void* x, const void* w, const void* bias, const ConvGeom& g, int32_t act,
                    void* ws_, cudaStream_t st, float* sums) {
  uint8_t* ws = static_cast<uint8_t*>(ws_);
  const int fold = cw_fold(g);
  const CwCopy xc = cw_copy_of_x(g);
  int32_t rc = cw_copy_x(ws, x, g, xc, st);
  if (rc != LB2_OK) return rc;
  __nv_bfloat16* wp = reinterpret_cast<__nv_bfloat16*>(ws + xc.bytes);
  CwPack pk{};
  pk.kW = g.k[0]; pk.kH = g.k[1]; pk.cin = g.cin; pk.cout = g.cout; pk.flip = g.flip; pk.transpose = 0; pk.fold = fold;
  pk.chunks = fold ? 1 : (g.cin + 63) / 64;
  const int n_taps = fold ? cw_fold_taps(g, fold) : g.k[0] * g.k[1];
  pk.n_rows = round_up(g.cout, cw_bn(g.cout));
  pk.k_total = n_taps * pk.chunks * 64;
  cw_pack_filter(wp, (const __nv_bfloat16*)w, pk, st);
  LB2_CHECK_LAUNCH("conv_cw filter packing");
  CwTap taps[kCwMaxKb];
  for (int t = 0; t < n_taps; ++t) {
    if (fold >= 2) taps[t] = CwTap{0, t, t};                                        // rows of the copy: q = oh + t
    else if (fold) taps[t] = CwTap{0, t * g.dil[1] - g.pad_lo[1], t};
    else taps[t] = CwTap{(t % g.k[0]) * g.dil[0] - g.pad_lo[0], (t / g.k[0]) * g.dil[1] - g.pad_lo[1], t};
  }
  float* sums_partial = reinterpret_cast<float*>(ws + align_up(xc.bytes + cw_packed_bytes(g.cout, n_taps, pk.chunks), 1024));
  return cw_run_gemm(y, preact, bias, act, ws, xc.Cp, xc.W, xc.H, g.batch, pk.chunks, wp, pk.n_rows, pk.k_total, taps, n_taps,
                     g.out[0], g.out[1], fold ? 1 : g.stride[0], fold >= 2 ? 1 : g.stride[1], g.cout, g.out[0], g.out[1], 1, 0, 1, 0, st,
                     sums, sums_partial);
}

// ---- backward ---------------------------------------------------------------------------------------
namespace {

struct CwWgPlan {
  int chunks, n_pairs, ppg, groups, co_tiles;
  int KW_, KH_, KI_, kbw, kbh, kbi, kb_total, splits, kb_per_split;
  size_t partial_bytes;
};
CwWgPlan cw_wg_plan(const ConvGeom& g) {
  CwWgPlan w{};
  const int fold = cw_fold(g);
  w.chunks = fold ? 1 : (g.cin + 63) / 64;
  w.n_pairs = (fold ? cw_fold_taps(g, fold) : g.k[0] * g.k[1]) * w.chunks;
  // column groups per MMA: the largest of 4, 3, 2 that divides the pair count, else 4 with filler groups
  w.ppg = w.n_pairs >= 4 ? 4 : w.n_pairs;
  for (int c = 4; c >= 2; --c)
    if (w.n_pairs % c == 0) { w.ppg = c; break; }
  w.groups = (w.n_pairs + w.ppg - 1) / w.ppg;
  w.co_tiles = (g.cout + 127) / 128;
  // 64 positions per k-block: whole (or 64-wide pieces of) rows, several rows / images when rows are short
  const int OW = g.out[0], OH = g.out[1];
  int kw = 64;
  while (kw / 2 >= OW) kw /= 2;        // smallest power of two >= OW, at most 64
  w.KW_ = kw; w.KH_ = 64 / kw;
  if (w.KH_ > OH) { int kh = 1; while (kh < OH) kh *= 2; w.KH_ = kh; }
  w.KI_ = 64 / (w.KW_ * w.KH_);
  w.kbw = (OW + w.KW_ - 1) / w.KW_; w.kbh = (OH + w.KH_ - 1) / w.KH_; w.kbi = (g.batch + w.KI_ - 1) / w.KI_;
  w.kb_total = w.kbw * w.kbh * w.kbi;
  const int items = w.co_tiles * w.groups;
  int splits = (2 * sm_count()) / items;   // about two items per CTA so that tails even out
  if (splits < 1) splits = 1;
  if (splits > w.kb_total) splits = w.kb_total;
  w.kb_per_split = (w.kb_total + splits - 1) / splits;
  w.splits = (w.kb_total + w.kb_per_split - 1) / w.kb_per_split;
  w.partial_bytes = align_up((size_t)w.splits * items * 128 * (w.ppg * 64) * sizeof(float), 1024);
  return w;
}

}  // namespace

size_t conv_cw_bwd_workspace_bytes(const ConvGeom& g) {
  const size_t gy = cw_copy_of_y(g).bytes;
  const size_t dgrad = cw_packed_bytes(g.cin, g.k[0] * g.k[1], (g.cout + 63) / 64);
  const size_t wgrad = cw_copy_of_x(g).bytes + cw_wg_plan(g).partial_bytes;
  return gy + (dgrad > wgrad ? dgrad : wgrad);
}

// both gradients (either output may be null) from one channel-innermost copy of gy. With `x_is_copy`, x points at the
// channel-innermost copy that conv_cw_fwd left at the start of its workspace (same geometry, same x).
int32_t conv_cw_bwd(void* dw, void* dx, const void* x, const void* gy, const void* w, const ConvGeom& g, void* ws_, cudaStream_t st,
                    bool x_is_copy) {
  uint8_t* ws = static_cast<uint8_t*>(ws_);
  const CwCopy yc = cw_copy_of_y(g);
  int32_t rc = cw_transpose(ws, gy, g.out[0], g.out[1], g.cout, yc.Cp, g.batch, st);
  if (rc != LB2_OK) return rc;
  uint8_t* rest = ws + yc.bytes;

  if (dw != nullptr) {
    const int fold = cw_fold(g);
    const CwCopy xc = cw_copy_of_x(g);
    uint8_t* xcopy = rest;
    if (x_is_copy) {
      xcopy = static_cast<uint8_t*>(const_cast<void*>(x));
    } else {
      rc = cw_copy_x(rest, x, g, xc, st);
      if (rc != LB2_OK) return rc;
    }
    const CwWgPlan pl = cw_wg_plan(g);
    CwWgParams q{};
    q.OW = g.out[0]; q.OH = g.out[1]; q.NI = g.batch;
    q.KW_ = pl.KW_; q.KH_ = pl.KH_; q.KI_ = pl.KI_; q.kbw = pl.kbw; q.kbh = pl.kbh; q.kbi = pl.kbi;
    q.sw = fold ? 1 : g.stride[0]; q.sh = fold >= 2 ? 1 : g.stride[1];
    q.co_tiles = pl.co_tiles; q.groups = pl.groups; q.pairs_per_group = pl.ppg; q.n_pairs = pl.n_pairs;
    q.splits = pl.splits; q.kb_total = pl.kb_total; q.kb_per_split = pl.kb_per_split;
    // A (gy copy) and B (x copy) both MN-major: bits 15 and 16
    q.idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)((pl.ppg * 64) >> 3) << 17) | ((uint32_t)(kCwBM >> 4) << 24);
    q.partial = reinterpret_cast<float*>(rest + (x_is_copy ? 0 : xc.bytes));
    q.status = device_status_word();
    LB2_REQUIRE(q.status != nullptr, LB2_LAUNCH_FAIL, "conv_cw: device status word unavailable");
    const int n_taps = fold ? cw_fold_taps(g, fold) : g.k[0] * g.k[1];
    for (int t = 0; t < n_taps; ++t)
      for (int ch = 0; ch < pl.chunks; ++ch) {
        const int pr = t * pl.chunks + ch;
        q.pr_dw[pr] = (int16_t)(fold ? 0 : (t % g.k[0]) * g.dil[0] - g.pad_lo[0]);
        q.pr_dh[pr] = (int16_t)(fold >= 2 ? t : (fold ? t : t / g.k[0]) * g.dil[1] - g.pad_lo[1]);
        q.pr_c0[pr] = (int16_t)(ch * 64);
      }
    CUtensorMap mG, mX;
    if (!cw_map(&mG, ws, yc.Cp, yc.W, yc.H, g.batch, pl.KW_, pl.KH_, pl.KI_, 1, 1) ||
        !cw_map(&mX, xcopy, xc.Cp, xc.W, xc.H, g.batch, pl.KW_, pl.KH_, pl.KI_, q.sw, q.sh))
      return fail(LB2_LAUNCH_FAIL, "conv_cw: cuTensorMapEncodeTiled failed");
    const int items = pl.co_tiles * pl.groups * pl.splits;
    const int grid = items < sm_count() ? items : sm_count();
    auto launch = [&](auto kernel, int np) -> int32_t {
      const int stage_bytes = kCwBM * 128 + np * 64 * 128;
      int nst = (200 * 1024) / stage_bytes;
      if (nst > 8) nst = 8;
      const int smem = nst * stage_bytes + 1024 + 256;
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "conv_cw: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
      kernel<<<grid, kCwThreads, smem, st>>>(mG, mX, q);
      LB2_CHECK_LAUNCH("conv_cw_wgrad");
      return LB2_OK;
    };
    rc = pl.ppg == 1 ? launch(conv_cw_wgrad_kernel<1>, 1) : pl.ppg == 2 ? launch(conv_cw_wgrad_kernel<2>, 2)
       : pl.ppg == 3 ? launch(conv_cw_wgrad_kernel<3>, 3) : launch(conv_cw_wgrad_kernel<4>, 4);
    if (rc != LB2_OK) return rc;
    CwReduce rd{g.k[0], g.k[1], g.cin, g.cout, g.flip, fold, pl.chunks, pl.co_tiles, pl.groups, pl.ppg, pl.splits};
    // few splits = a large filter: per-(channel, chunk) blocks with contiguous writes; many splits = a small filter
    // with little else to parallelise over: the per-slot kernel, whose y slices share the splits
    if (fold == 0 && pl.splits <= 16 && g.k[0] * g.k[1] * 64 * sizeof(float) <= 48 * 1024)
      conv_cw_wgrad_reduce_rows_kernel<__nv_bfloat16><<<(unsigned)((int64_t)g.cout * pl.chunks), 256, g.k[0] * g.k[1] * 64 * sizeof(float), st>>>(
          (__nv_bfloat16*)dw, q.partial, rd);
    else
      conv_cw_wgrad_reduce_kernel<__nv_bfloat16><<<(unsigned)((int64_t)pl.groups * pl.co_tiles * 128 * pl.ppg), dim3(64, kCwReduceSlices), 0, st>>>(
          (__nv_bfloat16*)dw, q.partial, rd);
    LB2_CHECK_LAUNCH("conv_cw_wgrad_reduce");
  }

  if (dx != nullptr) {
    // dx[i] = sum over taps t with (i + pad - t*dil) divisible by the stride of gy[(i + pad - t*dil) / stride] * Wf[t]:
    // per residue class of i (mod stride) a stride-1 problem over gy's copy, written to that class's subset of dx.
    __nv_bfloat16* wp = reinterpret_cast<__nv_bfloat16*>(rest);
    CwPack pk{};
    pk.kW = g.k[0]; pk.kH = g.k[1]; pk.cin = g.cin; pk.cout = g.cout; pk.flip = g.flip; pk.transpose = 1; pk.fold = 0;
    pk.chunks = (g.cout + 63) / 64;
    pk.n_rows = round_up(g.cin, cw_bn(g.cin));
    pk.k_total = g.k[0] * g.k[1] * pk.chunks * 64;
    cw_pack_filter(wp, (const __nv_bfloat16*)w, pk, st);
    LB2_CHECK_LAUNCH("conv_cw filter packing (data gradient)");
    const int sw = g.stride[0], sh = g.stride[1];
    auto class_taps = [&](int pw, int ph, CwTap* taps) {
      int n = 0;
      for (int th = 0; th < g.k[1]; ++th) {
        const int nh = ph + g.pad_lo[1] - th * g.dil[1];
        if (((nh % sh) + sh) % sh != 0) continue;
        for (int tw = 0; tw < g.k[0]; ++tw) {
          const int nw = pw + g.pad_lo[0] - tw * g.dil[0];
          if (((nw % sw) + sw) % sw != 0) continue;
          taps[n++] = CwTap{nw / sw, nh / sh, th * g.k[0] + tw};   // exact: nw, nh are multiples of the stride
        }
      }
      return n;
    };
    bool any_empty = false;
    {
      CwTap taps[kCwMaxKb];
      for (int ph = 0; ph < sh && ph < g.in[1]; ++ph)
        for (int pw = 0; pw < sw && pw < g.in[0]; ++pw)
          if (class_taps(pw, ph, taps) == 0) any_empty = true;
    }
    if (any_empty) {   // classes no tap reaches stay zero
      cudaError_t e = cudaMemsetAsync(dx, 0, (size_t)g.in[0] * g.in[1] * g.cin * g.batch * 2, st);
      if (e != cudaSuccess) return fail(LB2_LAUNCH_FAIL, "conv_cw: clearing dx failed: %s", cudaGetErrorString(e));
    }
    for (int ph = 0; ph < sh && ph < g.in[1]; ++ph)
      for (int pw = 0; pw < sw && pw < g.in[0]; ++pw) {
        CwTap taps[kCwMaxKb];
        const int n = class_taps(pw, ph, taps);
        if (n == 0) continue;
        const int OWc = (g.in[0] - pw + sw - 1) / sw, OHc = (g.in[1] - ph + sh - 1) / sh;
        rc = cw_run_gemm(dx, nullptr, nullptr, LB2_ACT_IDENTITY, ws, yc.Cp, yc.W, yc.H, g.batch, pk.chunks, wp, pk.n_rows, pk.k_total,
                         taps, n, OWc, OHc, 1, 1, g.cin, g.in[0], g.in[1], sw, pw, sh, ph, st);
        if (rc != LB2_OK) return rc;
      }
  }
  return LB2_OK;
}

}  // namespace lb2

// Convolution entry points: y = act(conv(x, w) + b) and the pullback ∇fused_conv
// (lib/LuxLib/src/impl/conv.jl:261-275): g = dy .* act', dw = ∇conv_filter(x, g),
// dx = ∇conv_data(g, w), db = sum over (spatial, batch) of g.
#include "conv.cuh"
#include "eltwise.cuh"

using namespace lb2;

namespace {

int32_t make_geom(const lb2_conv_desc* d, ConvGeom* g) {
  LB2_REQUIRE(d != nullptr, LB2_BAD_ARG, "conv descriptor is null");
  LB2_REQUIRE(d->ndim >= 1 && d->ndim <= 3, LB2_BAD_SHAPE, "spatial rank %d not in 1..3", (int)d->ndim);
  LB2_REQUIRE(d->groups >= 1 && d->cin >= 0 && d->cout >= 0 && d->batch >= 0, LB2_BAD_SHAPE, "bad channel / batch extents");
  LB2_REQUIRE(d->cin % d->groups == 0 && d->cout % d->groups == 0, LB2_BAD_SHAPE,
              "channels (%d -> %d) must be divisible by groups (%d)", (int)d->cin, (int)d->cout, (int)d->groups);
  for (int i = 0; i < 3; ++i) {
    const bool live = i < d->ndim;
    g->in[i] = live ? d->in[i] : 1;
    g->k[i] = live ? d->k[i] : 1;
    g->stride[i] = live ? d->stride[i] : 1;
    g->pad_lo[i] = live ? d->pad_lo[i] : 0;
    g->pad_hi[i] = live ? d->pad_hi[i] : 0;
    g->dil[i] = live ? d->dilation[i] : 1;
    LB2_REQUIRE(g->in[i] >= 0 && g->k[i] >= 1 && g->stride[i] >= 1 && g->dil[i] >= 1 && g->pad_lo[i] >= 0 && g->pad_hi[i] >= 0,
                LB2_BAD_SHAPE, "bad extent / stride / dilation / padding in dim %d", i);
    const int span = g->in[i] + g->pad_lo[i] + g->pad_hi[i] - g->dil[i] * (g->k[i] - 1) - 1;
    g->out[i] = span < 0 ? 0 : span / g->stride[i] + 1;
  }
  g->groups = d->groups;
  g->flip = d->flipkernel ? 1 : 0;
  g->cin = d->cin;
  g->cout = d->cout;
  g->batch = d->batch;
  g->ndim = d->ndim;
  return LB2_OK;
}

// Which kernels serve a geometry: 1 = tensor-core path on the WHCN bytes (conv_tc*.cu), 2 = general bf16 tensor-core
// path on channel-innermost copies (conv_cw.cu), 0 = CUDA-core direct kernels.
int conv_route(const ConvGeom& g, int32_t dtype) {
  if (conv_tc_supported(g, dtype)) return 1;
  if (conv_cw_supported(g, dtype)) return 2;
  return 0;
}

int64_t y_numel(const ConvGeom& g) { return (int64_t)g.out[0] * g.out[1] * g.out[2] * g.cout * g.batch; }
int64_t y_spatial(const ConvGeom& g) { return (int64_t)g.out[0] * g.out[1] * g.out[2]; }

struct ConvBwdLayout {
  size_t g_bytes, red_bytes, tc_bytes;
  size_t total() const { return g_bytes + red_bytes + tc_bytes; }
};
ConvBwdLayout conv_bwd_layout(const ConvGeom& g, int32_t dtype, int32_t act) {
  ConvBwdLayout l{};
  const int64_t n = y_numel(g);
  if (n <= 0) return l;
  l.g_bytes = act == LB2_ACT_IDENTITY ? 0 : align_up((size_t)n * dtype_size(dtype), 1024);
  l.red_bytes = align_up(act_bwd_workspace_bytes(y_spatial(g), g.cout, g.batch), 1024);
  const int route = conv_route(g, dtype);
  l.tc_bytes = route == 1 ? conv_tc_bwd_workspace_bytes(g, dtype) : (route == 2 ? conv_cw_bwd_workspace_bytes(g) : 0);
  return l;
}

}  // namespace

extern "C" {

int32_t lb2_conv_output_size(const lb2_conv_desc* d, int32_t* out) {
  ConvGeom g;
  int32_t rc = make_geom(d, &g);
  if (rc != LB2_OK) return rc;
  LB2_REQUIRE(out != nullptr, LB2_BAD_ARG, "out is null");
  for (int i = 0; i < d->ndim; ++i) out[i] = g.out[i];
  return LB2_OK;
}

size_t lb2_conv_fwd_workspace_bytes(const lb2_conv_desc* d, int32_t dtype) {
  ConvGeom g;
  if (!valid_dtype(dtype) || make_geom(d, &g) != LB2_OK || y_numel(g) == 0) return 0;
  const int route = conv_route(g, dtype);
  return route == 1 ? conv_tc_fwd_workspace_bytes(g, dtype) : (route == 2 ? conv_cw_fwd_workspace_bytes(g) : 0);
}

int32_t lb2_conv_fwd(void* y, void* preact, const void* x, const void* w, const void* b, const lb2_conv_desc* d,
                     int32_t dtype, int32_t act, uint32_t flags, void* workspace, size_t workspace_bytes,
                     void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(valid_act(act), LB2_BAD_ARG, "unknown activation %d", (int)act);
  ConvGeom g;
  int32_t rc = make_geom(d, &g);
  if (rc != LB2_OK) return rc;
  if (y_numel(g) == 0) return LB2_OK;
  LB2_REQUIRE(y && x && w, LB2_BAD_ARG, "null tensor pointer");
  const size_t es = dtype_size(dtype);
  LB2_REQUIRE(aligned_to(y, es) && aligned_to(preact, es) && aligned_to(x, es) && aligned_to(w, es) && aligned_to(b, es),
              LB2_BAD_ALIGN, "pointer not aligned to the element size");
  // The tensor-core kernels on the WHCN bytes move x, y and the pre-activation with TMA (16-byte aligned bases); an
  // offset view of a larger array that breaks that rule goes to the general path (which copies its input) or to the
  // direct kernels instead of being rejected.
  int route = (flags & LB2_FLAG_FORCE_SIMT) ? 0 : conv_route(g, dtype);
  if (route == 1 && !(aligned_to(x, 16) && aligned_to(y, 16) && aligned_to(preact, 16)))
    route = (conv_cw_supported(g, dtype) && conv_cw_fwd_workspace_bytes(g) <= workspace_bytes) ? 2 : 0;
  if (route != 0) {
    const size_t need = route == 1 ? conv_tc_fwd_workspace_bytes(g, dtype) : conv_cw_fwd_workspace_bytes(g);
    LB2_REQUIRE(workspace != nullptr && workspace_bytes >= need, LB2_WORKSPACE_TOO_SMALL, "workspace of %zu bytes needed", need);
    LB2_REQUIRE(aligned_to(workspace, 256), LB2_BAD_ALIGN, "workspace must be 256-byte aligned");
    if (route == 1) return conv_tc_fwd(y, preact, x, w, b, g, dtype, act, workspace, static_cast<cudaStream_t>(stream));
    return conv_cw_fwd(y, preact, x, w, b, g, act, workspace, static_cast<cudaStream_t>(stream));
  }
  return conv_fwd_direct(y, preact, x, w, b, g, dtype, act, static_cast<cudaStream_t>(stream));
}

int32_t lb2_conv_fwd_leaves_x_copy(const lb2_conv_desc* d, int32_t dtype) {
  ConvGeom g;
  if (!valid_dtype(dtype) || make_geom(d, &g) != LB2_OK || y_numel(g) == 0) return 0;
  return conv_route(g, dtype) == 2 ? 1 : 0;
}

// The epilogue sums cost about a thousand instructions per warp and tile; they disappear behind the tile's MMAs only
// when the contraction is long enough (16 k-blocks of 64: a 3x3 filter over 128 input channels and up). Shorter
// contractions (1x1 projections, the folded stem) are faster with BatchNorm's own statistics pass.
int32_t lb2_conv_fwd_sums_is_fused(const lb2_conv_desc* d, int32_t dtype) {
  ConvGeom g;
  if (!valid_dtype(dtype) || make_geom(d, &g) != LB2_OK || y_numel(g) == 0) return 0;
  if (conv_route(g, dtype) != 2) return 0;
  return conv_cw_fwd_kblocks(g) >= 16 ? 1 : 0;   // counted as the kernel runs it: a folded 7x7 stem has 4, not 49
}

size_t lb2_conv_fwd_sums_workspace_bytes(const lb2_conv_desc* d, int32_t dtype) {
  ConvGeom g;
  if (!valid_dtype(dtype) || make_geom(d, &g) != LB2_OK) return 0;
  const size_t conv = align_up(lb2_conv_fwd_workspace_bytes(d, dtype), 1024);
  if (conv_route(g, dtype) == 2) return conv;
  return conv + lb2_channel_sums_workspace_bytes(y_spatial(g), g.cout, g.batch);
}

int32_t lb2_conv_fwd_sums(void* y, float* sums, const void* x, const void* w, const lb2_conv_desc* d, int32_t dtype, uint32_t flags,
                          void* workspace, size_t workspace_bytes, void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(sums != nullptr, LB2_BAD_ARG, "sums is null");
  ConvGeom g;
  int32_t rc = make_geom(d, &g);
  if (rc != LB2_OK) return rc;
  if (g.cout == 0) return LB2_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (y_numel(g) == 0) {
    cudaMemsetAsync(sums, 0, (size_t)g.cout * 2 * sizeof(float), st);
    return LB2_OK;
  }
  LB2_REQUIRE(workspace_bytes >= lb2_conv_fwd_sums_workspace_bytes(d, dtype), LB2_WORKSPACE_TOO_SMALL, "workspace of %zu bytes needed",
              lb2_conv_fwd_sums_workspace_bytes(d, dtype));
  const bool fused = !(flags & LB2_FLAG_FORCE_SIMT) && conv_route(g, dtype) == 2;
  if (fused) {
    LB2_REQUIRE(y && x && w, LB2_BAD_ARG, "null tensor pointer");
    LB2_REQUIRE(workspace != nullptr && aligned_to(workspace, 256), LB2_BAD_ALIGN, "workspace must be 256-byte aligned");
    LB2_REQUIRE(aligned_to(y, 2) && aligned_to(x, 2) && aligned_to(w, 2), LB2_BAD_ALIGN, "pointer not aligned to the element size");
    return conv_cw_fwd(y, nullptr, x, w, nullptr, g, LB2_ACT_IDENTITY, workspace, st, sums);
  }
  const size_t conv = align_up(lb2_conv_fwd_workspace_bytes(d, dtype), 1024);
  rc = lb2_conv_fwd(y, nullptr, x, w, nullptr, d, dtype, LB2_ACT_IDENTITY, flags, workspace, conv, stream);
  if (rc != LB2_OK) return rc;
  uint8_t* rest = static_cast<uint8_t*>(workspace) + conv;
  return lb2_channel_sums(sums, y, y_spatial(g), g.cout, g.batch, dtype, rest, workspace_bytes - conv, stream);
}

size_t lb2_conv_bwd_workspace_bytes(const lb2_conv_desc* d, int32_t dtype, int32_t act) {
  ConvGeom g;
  if (!valid_dtype(dtype) || make_geom(d, &g) != LB2_OK) return 0;
  return conv_bwd_layout(g, dtype, act).total();
}

int32_t lb2_conv_bwd(void* dw, void* dx, void* db, const void* dy, const void* out, const void* preact,
                     const void* x, const void* w, const lb2_conv_desc* d, int32_t dtype, int32_t act, uint32_t flags,
                     void* workspace, size_t workspace_bytes, void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(valid_act(act), LB2_BAD_ARG, "unknown activation %d", (int)act);
  ConvGeom g;
  int32_t rc = make_geom(d, &g);
  if (rc != LB2_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t es = dtype_size(dtype);
  const int64_t nw = (int64_t)g.k[0] * g.k[1] * g.k[2] * (g.cin / g.groups) * g.cout;
  const int64_t nx = (int64_t)g.in[0] * g.in[1] * g.in[2] * g.cin * g.batch;
  if (y_numel(g) == 0) {  // nothing flows back: zero gradients
    if (dw && nw > 0) cudaMemsetAsync(dw, 0, (size_t)nw * es, st);
    if (dx && nx > 0) cudaMemsetAsync(dx, 0, (size_t)nx * es, st);
    if (db && g.cout > 0) cudaMemsetAsync(db, 0, (size_t)g.cout * es, st);
    return LB2_OK;
  }
  rc = check_act_bwd_args(dy, out, preact, dtype, act);
  if (rc != LB2_OK) return rc;
  LB2_REQUIRE((!dw || x) && (!dx || w), LB2_BAD_ARG, "x / w needed for the requested gradients are null");
  LB2_REQUIRE(aligned_to(dw, es) && aligned_to(dx, es) && aligned_to(db, es) && aligned_to(dy, es) && aligned_to(out, es) &&
                  aligned_to(preact, es) && aligned_to(x, es) && aligned_to(w, es),
              LB2_BAD_ALIGN, "pointer not aligned to the element size");
  const ConvBwdLayout lay = conv_bwd_layout(g, dtype, act);
  LB2_REQUIRE(workspace != nullptr && workspace_bytes >= lay.total(), LB2_WORKSPACE_TOO_SMALL, "workspace of %zu bytes needed", lay.total());
  LB2_REQUIRE(aligned_to(workspace, 256), LB2_BAD_ALIGN, "workspace must be 256-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* red = reinterpret_cast<float*>(ws + lay.g_bytes);
  const int64_t S = y_spatial(g);
  const void* gptr = dy;
  const int route = (flags & LB2_FLAG_FORCE_SIMT) ? 0 : (lay.tc_bytes > 0 ? conv_route(g, dtype) : 0);
  // identity activation on the bf16 fast case: the filter-gradient kernel adds up dy on the side, no pass of its own
  const bool db_by_wgrad = act == LB2_ACT_IDENTITY && db && dw && route == 1 && dtype == LB2_BF16 && aligned_to(dy, 16) &&
                           aligned_to(x, 16) && aligned_to(dx, 16) && conv_tc_wgrad_makes_db(g, dtype);
  if (act != LB2_ACT_IDENTITY) {
    rc = launch_act_bwd(ws, db, dy, out, preact, S, g.cout, g.batch, g.cout, g.cout, g.cout, dtype, act, 0, red, st);
    if (rc != LB2_OK) return rc;
    gptr = ws;
  } else if (db && !db_by_wgrad) {
    rc = launch_act_bwd(nullptr, db, dy, nullptr, nullptr, S, g.cout, g.batch, g.cout, g.cout, g.cout, dtype, act, 0, red, st);
    if (rc != LB2_OK) return rc;
  }
  const bool x_is_copy = (flags & LB2_FLAG_X_COPY_GIVEN) != 0;
  LB2_REQUIRE(!x_is_copy || (route == 2 && aligned_to(x, 256)), LB2_BAD_ARG,
              "LB2_FLAG_X_COPY_GIVEN: this geometry does not run on the path that leaves a copy of x (or the pointer is not a workspace start)");
  void* tc_ws = ws + lay.g_bytes + lay.red_bytes;
  if (route == 2) return conv_cw_bwd(dw, (dx && nx > 0) ? dx : nullptr, x, gptr, w, g, tc_ws, st, x_is_copy);
  // TMA needs 16-byte aligned bases for everything it loads (g, x) or stores (dx); other views go to the direct kernels
  const bool tc = route == 1 && aligned_to(gptr, 16) && aligned_to(x, 16) && aligned_to(dx, 16);
  if (tc && dtype == LB2_F32) {   // both gradients share one set of shifted copies of g
    return conv_tc_f32_bwd(dw, (dx && nx > 0) ? dx : nullptr, x, gptr, w, g, tc_ws, st);
  }
  if (dw) {
    rc = tc ? conv_tc_wgrad(dw, x, gptr, g, dtype, tc_ws, st, db_by_wgrad ? db : nullptr) : conv_wgrad_direct(dw, x, gptr, g, dtype, st);
    if (rc != LB2_OK) return rc;
  }
  if (dx && nx > 0) {
    rc = tc ? conv_tc_dgrad(dx, gptr, w, g, dtype, tc_ws, st) : conv_dgrad_direct(dx, gptr, w, g, dtype, st);
    if (rc != LB2_OK) return rc;
  }
  return LB2_OK;
}

}  // extern "C"

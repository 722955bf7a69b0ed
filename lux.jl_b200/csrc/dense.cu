// Dense layer entry points: y = act(W*x + b) and its pullback, plus the plain matmul used by the
// matmul / matmuladd rules. Forward is ONE tensor-core GEMM with bias + activation (and the
// optional pre-activation store) in its epilogue. The pullback runs one bandwidth-bound pass
// g = dy .* act'(.) that also yields db = sum over columns of g, then the two tensor-core GEMMs
// dW = g * x' (both operands MN-major) and dx = W' * g (both K-major) straight from the
// column-major arrays — no transposed copies.
#include "eltwise.cuh"
#include "gemm.cuh"

using namespace lb2;

namespace {

int32_t check_dense_common(int64_t M, int64_t N, int64_t K, int64_t ldw, int64_t ldx, int64_t ldy, int32_t dtype,
                           int32_t act) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(valid_act(act), LB2_BAD_ARG, "unknown activation %d", (int)act);
  LB2_REQUIRE(M >= 0 && N >= 0 && K >= 0, LB2_BAD_SHAPE, "negative extent");
  LB2_REQUIRE(ldw >= (M > 1 ? M : 1) && ldx >= (K > 1 ? K : 1) && ldy >= (M > 1 ? M : 1), LB2_BAD_SHAPE,
              "leading dimension smaller than the number of rows (ldw=%lld ldx=%lld ldy=%lld)", (long long)ldw,
              (long long)ldx, (long long)ldy);
  return LB2_OK;
}

struct BwdLayout {
  size_t g_bytes, red_bytes, gemm_bytes;
  size_t total() const { return g_bytes + red_bytes + gemm_bytes; }
};

BwdLayout bwd_layout(int64_t M, int64_t N, int64_t K, int32_t dtype, int32_t act, uint32_t flags) {
  BwdLayout l{};
  if (M <= 0 || N <= 0) return l;
  l.g_bytes = act == LB2_ACT_IDENTITY ? 0 : align_up((size_t)M * (size_t)N * dtype_size(dtype), 256);
  l.red_bytes = act_bwd_workspace_bytes(1, M, N);
  GemmOperand g{nullptr, M, true}, x{nullptr, K, true}, w{nullptr, M, false}, gk{nullptr, M, false};
  const size_t a = gemm_workspace_bytes(g, x, M, K, N, dtype, flags);   // dW
  const size_t b = gemm_workspace_bytes(w, gk, K, N, M, dtype, flags);  // dx
  l.gemm_bytes = a > b ? a : b;
  return l;
}

}  // namespace

extern "C" {

size_t lb2_dense_fwd_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t dtype, uint32_t flags) {
  GemmOperand w{nullptr, M, true}, x{nullptr, K, false};
  return gemm_workspace_bytes(w, x, M, N, K, dtype, flags);
}

int32_t lb2_dense_fwd(void* y, void* preact, const void* W, const void* x, const void* b, int64_t M, int64_t N,
                      int64_t K, int64_t ldw, int64_t ldx, int64_t ldy, int32_t dtype, int32_t act, uint32_t flags,
                      void* workspace, size_t workspace_bytes, void* stream) {
  int32_t rc = check_dense_common(M, N, K, ldw, ldx, ldy, dtype, act);
  if (rc != LB2_OK) return rc;
  if (M == 0 || N == 0) return LB2_OK;
  LB2_REQUIRE(y != nullptr && (K == 0 || (W != nullptr && x != nullptr)), LB2_BAD_ARG, "null tensor pointer");
  const size_t es = dtype_size(dtype);
  LB2_REQUIRE(aligned_to(y, es) && aligned_to(W, es) && aligned_to(x, es) && aligned_to(b, es) && aligned_to(preact, es),
              LB2_BAD_ALIGN, "pointer not aligned to the element size");
  LB2_REQUIRE(workspace == nullptr || aligned_to(workspace, 256), LB2_BAD_ALIGN, "workspace must be 256-byte aligned");
  GemmOperand A{W, ldw, true};   // W (M x K): output-feature index contiguous
  GemmOperand B{x, ldx, false};  // x (K x N): contraction index contiguous
  GemmEpilogue epi;
  epi.bias = b;
  epi.act = act;
  epi.preact = preact;
  return gemm_dispatch(y, ldy, A, B, M, N, K, dtype, flags, epi, workspace, workspace_bytes,
                       static_cast<cudaStream_t>(stream));
}

size_t lb2_dense_bwd_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t dtype, int32_t act, uint32_t flags) {
  if (!valid_dtype(dtype)) return 0;
  return bwd_layout(M, N, K, dtype, act, flags).total();
}

int32_t lb2_dense_bwd(void* dW, void* dx, void* db, const void* dy, const void* out, const void* preact,
                      const void* W, const void* x, int64_t M, int64_t N, int64_t K, int64_t ldw, int64_t ldx,
                      int64_t ldy, int32_t dtype, int32_t act, int32_t accumulate, uint32_t flags, void* workspace,
                      size_t workspace_bytes, void* stream) {
  int32_t rc = check_dense_common(M, N, K, ldw, ldx, ldy, dtype, act);
  if (rc != LB2_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t es = dtype_size(dtype);
  if (M == 0 || N == 0 || K == 0) {
    // empty contraction: gradients are zero (unless accumulating into existing values)
    if (!accumulate) {
      if (dW && M > 0 && K > 0) cudaMemset2DAsync(dW, (size_t)ldw * es, 0, (size_t)M * es, (size_t)K, st);
      if (dx && K > 0 && N > 0) cudaMemset2DAsync(dx, (size_t)ldx * es, 0, (size_t)K * es, (size_t)N, st);
      if (db && M > 0 && N == 0) cudaMemsetAsync(db, 0, (size_t)M * es, st);
    }
    if (!(M > 0 && N > 0 && db)) return LB2_OK;
  }
  rc = check_act_bwd_args(dy, out, preact, dtype, act);
  if (rc != LB2_OK) return rc;
  LB2_REQUIRE((!dW || x) && (!dx || W), LB2_BAD_ARG, "W / x needed for the requested gradients are null");
  LB2_REQUIRE(aligned_to(dW, es) && aligned_to(dx, es) && aligned_to(db, es) && aligned_to(dy, es) && aligned_to(out, es) &&
                  aligned_to(preact, es) && aligned_to(W, es) && aligned_to(x, es),
              LB2_BAD_ALIGN, "pointer not aligned to the element size");
  const BwdLayout lay = bwd_layout(M, N, K, dtype, act, flags);
  LB2_REQUIRE(lay.total() == 0 || (workspace != nullptr && workspace_bytes >= lay.total()), LB2_WORKSPACE_TOO_SMALL,
              "workspace of %zu bytes needed", lay.total());
  LB2_REQUIRE(workspace == nullptr || aligned_to(workspace, 256), LB2_BAD_ALIGN, "workspace must be 256-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  void* gbuf = ws;
  float* red = reinterpret_cast<float*>(ws + lay.g_bytes);
  void* gemm_ws = ws + lay.g_bytes + lay.red_bytes;

  // g = dy .* act'  (+ db = column sums of g) in one pass
  const void* g = dy;
  int64_t ldg = ldy;
  if (act != LB2_ACT_IDENTITY) {
    rc = launch_act_bwd(gbuf, db, dy, out, preact, 1, M, N, M, ldy, ldy, dtype, act, accumulate, red, st);
    if (rc != LB2_OK) return rc;
    g = gbuf;
    ldg = M;
  } else if (db) {
    rc = launch_act_bwd(nullptr, db, dy, nullptr, nullptr, 1, M, N, M, ldy, ldy, dtype, act, accumulate, red, st);
    if (rc != LB2_OK) return rc;
  }
  if (K == 0) return LB2_OK;
  GemmEpilogue epi;
  epi.accumulate = accumulate;
  if (dW) {  // dW (M x K) = g (M x N) * x' : contraction over the batch; both operands MN-major
    GemmOperand A{g, ldg, true}, B{x, ldx, true};
    rc = gemm_dispatch(dW, ldw, A, B, M, K, N, dtype, flags, epi, gemm_ws, lay.gemm_bytes, st);
    if (rc != LB2_OK) return rc;
  }
  if (dx) {  // dx (K x N) = W' * g : contraction over output features; both operands K-major
    GemmOperand A{W, ldw, false}, B{g, ldg, false};
    rc = gemm_dispatch(dx, ldx, A, B, K, N, M, dtype, flags, epi, gemm_ws, lay.gemm_bytes, st);
    if (rc != LB2_OK) return rc;
  }
  return LB2_OK;
}

size_t lb2_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t dtype, uint32_t flags) {
  // the split copies are packed, so their size depends on the extents only, not on how op(A), op(B) are stored
  GemmOperand a{nullptr, M, true}, b{nullptr, K, false};
  GemmOperand at{nullptr, K, false}, bt{nullptr, N, true};
  const size_t s0 = gemm_workspace_bytes(a, b, M, N, K, dtype, flags);
  const size_t s1 = gemm_workspace_bytes(at, bt, M, N, K, dtype, flags);
  const size_t s2 = gemm_workspace_bytes(a, bt, M, N, K, dtype, flags);
  const size_t s3 = gemm_workspace_bytes(at, b, M, N, K, dtype, flags);
  size_t m = s0 > s1 ? s0 : s1;
  m = m > s2 ? m : s2;
  return m > s3 ? m : s3;
}

int32_t lb2_matmul(void* C, const void* A, const void* B, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                   int64_t ldc, int32_t transA, int32_t transB, int32_t dtype, int32_t accumulate, uint32_t flags,
                   void* workspace, size_t workspace_bytes, void* stream) {
  LB2_REQUIRE(valid_dtype(dtype), LB2_UNSUPPORTED_DTYPE, "dtype %d not supported", (int)dtype);
  LB2_REQUIRE(M >= 0 && N >= 0 && K >= 0, LB2_BAD_SHAPE, "negative extent");
  if (M == 0 || N == 0) return LB2_OK;
  const int64_t a_rows = transA ? K : M, b_rows = transB ? N : K;
  LB2_REQUIRE(lda >= (a_rows > 1 ? a_rows : 1) && ldb >= (b_rows > 1 ? b_rows : 1) && ldc >= M, LB2_BAD_SHAPE,
              "leading dimension smaller than the number of rows");
  LB2_REQUIRE(C != nullptr && (K == 0 || (A != nullptr && B != nullptr)), LB2_BAD_ARG, "null tensor pointer");
  const size_t es = dtype_size(dtype);
  LB2_REQUIRE(aligned_to(C, es) && aligned_to(A, es) && aligned_to(B, es), LB2_BAD_ALIGN, "pointer not aligned to the element size");
  LB2_REQUIRE(workspace == nullptr || aligned_to(workspace, 256), LB2_BAD_ALIGN, "workspace must be 256-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (K == 0) {
    if (!accumulate) cudaMemset2DAsync(C, (size_t)ldc * es, 0, (size_t)M * es, (size_t)N, st);
    return LB2_OK;
  }
  // op(A) is M x K: stored M x K (row index contiguous -> MN-major) or K x M (K contiguous -> K-major)
  GemmOperand a{A, lda, transA == 0};
  // op(B) is K x N: stored K x N (K contiguous -> K-major) or N x K (N contiguous -> MN-major)
  GemmOperand b{B, ldb, transB != 0};
  GemmEpilogue epi;
  epi.accumulate = accumulate;
  return gemm_dispatch(C, ldc, a, b, M, N, K, dtype, flags, epi, workspace, workspace_bytes, st);
}

}  // extern "C"

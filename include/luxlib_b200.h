/*
 * luxlib_b200.h — C ABI of libluxlib_b200.so: hand-written sm_100a kernels for LuxLib's
 * fused layer hot path (dense / conv / batch-, group-, layer-norm, bias+activation) and
 * their reverse-mode rules.
 *
 * Conventions (all entry points):
 *   - Every array is a raw DEVICE pointer to Julia column-major storage. "ld*" arguments are
 *     leading dimensions in elements.
 *   - `dtype` selects the storage type of every tensor argument of the call (LB2_F32 or
 *     LB2_BF16); accumulation is always fp32. Per-channel statistics (save_mean, save_invstd)
 *     and workspaces are always fp32.
 *   - Work is enqueued asynchronously on `stream` (a cudaStream_t passed as void*); the library
 *     never synchronises the device, never allocates device memory, never falls back to a
 *     vendor library or to the CPU. Scratch memory is supplied by the caller (`workspace`,
 *     `workspace_bytes`; sizes from the lb2_*_workspace_bytes queries, which are upper bounds
 *     that depend only on the listed extents). A workspace must be 256-byte aligned.
 *   - Return value: 0 (LB2_OK) or a negative lb2_status. Nothing is launched when an error is
 *     returned. Zero-sized problems return LB2_OK without launching
 *     (lib/LuxLib/test/common_ops/bias_act_tests.jl:119-131).
 *   - Re-entrant; the current CUDA device of the calling thread is used.
 *
 * Each declaration cites the reference interface (path inside LuxDL/Lux.jl) it replaces.
 */
#ifndef LUXLIB_B200_H
#define LUXLIB_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define LB2_API __attribute__((visibility("default")))
#else
#define LB2_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  LB2_OK = 0,
  LB2_BAD_ARG = -1,           /* null pointer, unknown enum, inconsistent optional arguments */
  LB2_BAD_SHAPE = -2,         /* DimensionMismatch in the reference */
  LB2_BAD_ALIGN = -3,         /* pointer not aligned to the element size / vector width */
  LB2_UNSUPPORTED_DTYPE = -4, /* e.g. Float64: caller keeps those on its old path */
  LB2_LAUNCH_FAIL = -5,       /* CUDA reported an error at launch */
  LB2_TIMEOUT = -6,           /* a bounded device-side wait expired (reported by lb2_poll_device_status) */
  LB2_WORKSPACE_TOO_SMALL = -7
} lb2_status;

typedef enum { LB2_F32 = 0, LB2_BF16 = 1 } lb2_dtype;

/* Activations named by the north-star path (NNlib scalar functions). tanh_fast / sigmoid_fast,
 * which NNlib.fast_act substitutes at src/layers/basic.jl:368, map to TANH / SIGMOID. */
typedef enum {
  LB2_ACT_IDENTITY = 0,
  LB2_ACT_RELU = 1,
  LB2_ACT_GELU_TANH = 2, /* 0.5x(1+tanh(sqrt(2/pi)(x+0.044715x^3))) */
  LB2_ACT_GELU_ERF = 3,  /* 0.5x(1+erf(x/sqrt2)) */
  LB2_ACT_TANH = 4,
  LB2_ACT_SIGMOID = 5,
  LB2_ACT_SWISH = 6
} lb2_act;

/* flags */
#define LB2_FLAG_TF32_1X 1u /* fp32 GEMM/conv: single-pass TF32 (rel err ~1e-3) instead of the
                               default error-compensated 3xTF32 split (rel err ~1e-6) */
#define LB2_FLAG_FORCE_SIMT 2u /* route a contraction through the CUDA-core kernel (debug / odd shapes) */
#define LB2_FLAG_CTA_PAIR 4u /* tensor-core GEMM: take the CTA-pair kernel (cta_group::2, 256x256 tiles) for any operand layout
                                once the problem occupies an eighth of the SM pairs (default: only for two MN-major operands) */
#define LB2_FLAG_NO_CTA_PAIR 8u /* tensor-core GEMM: never take the CTA-pair kernel */
/* lb2_conv_bwd only: the `x` argument is not x but the start of the workspace that lb2_conv_fwd was given for the same
 * descriptor and x (and that the caller has kept untouched since): the general tensor-core path leaves its
 * channel-innermost copy of x there and the filter gradient then reads that copy instead of making it again. Valid
 * only where lb2_conv_fwd_leaves_x_copy() returns 1; refused (LB2_BAD_ARG) elsewhere. */
#define LB2_FLAG_X_COPY_GIVEN 16u
/* Per call: the persistent tensor-core GEMM of this call leaves n SMs (0..127) unoccupied, for a kernel the caller
 * runs beside it on another stream — e.g. the NCCL all-reduce of parameter gradients that Lux's DistributedOptimizer
 * issues (src/distributed/public_api.jl:275-278) under the remaining backward GEMM. */
#define LB2_FLAG_RESERVE_SMS(n) (((uint32_t)(n) & 0x7Fu) << 16)

/* ---- library ------------------------------------------------------------------------- */
LB2_API int32_t lb2_version(void);
LB2_API const char* lb2_status_string(int32_t status);
/* Thread-local description of the last non-OK status returned on this thread. Mirrors the
 * 0 / -1 + warning convention of cublaslt_matmul_fused!
 * (lib/LuxLib/ext/CUDAExt/cublaslt.jl:184-185,292), without its fallback (:386-402). */
LB2_API const char* lb2_last_error_string(void);
/* Reads (and clears) the device-side status word that kernels with bounded waits write when a
 * wait expires. Synchronises `stream`. Returns LB2_OK or LB2_TIMEOUT. */
LB2_API int32_t lb2_poll_device_status(void* stream);

/* Self-test of the bounded device-side waits (no counterpart in the reference): launches one thread that waits, with
 * the given limit (1 us .. 100 ms), on a barrier nothing arrives at — the wait routine of the tensor-core kernels. The
 * wait expires, the kernel records it and returns; lb2_poll_device_status then reports LB2_TIMEOUT once and the
 * device stays usable. */
/* Diagnostics: the calling thread's last tensor-core GEMM launch (dense, matmul): out[0] kernel (1 single-CTA,
 * 2 CTA pair; 0 none yet), out[1], out[2] tile rows and columns, out[3] tiles, out[4] CTAs or CTA pairs launched,
 * out[5], out[6] whole-tile and total work slots (they differ when the tiles of a thin last wave are halved). */
LB2_API int32_t lb2_last_gemm_plan(int32_t* out, int32_t n);
LB2_API int32_t lb2_selftest_bounded_wait(uint64_t limit_ns, void* stream);

/* ---- activation / bias-activation ------------------------------------------------------ */
/* y = act.(x) over n elements.  Replaces activation!  (lib/LuxLib/src/impl/activation.jl:103-133). */
LB2_API int32_t lb2_act_fwd(void* y, const void* x, int64_t n, int32_t dtype, int32_t act, void* stream);
/* dx = dy .* act'(out, pre).  `pre` may be NULL for identity/relu/tanh/sigmoid (derivative from the
 * output only, lib/LuxLib/src/traits.jl:59-65); `out` may be NULL when `pre` is given.
 * Replaces ∇activation (lib/LuxLib/src/impl/activation.jl:135-154). */
LB2_API int32_t lb2_act_bwd(void* dx, const void* dy, const void* out, const void* pre, int64_t n,
                    int32_t dtype, int32_t act, void* stream);
/* y[s,c,b] = act(x[s,c,b] + bias[c]) on the (S, C, B) view of x
 * (lib/LuxLib/src/impl/bias_activation.jl:222-270; view at :229-235). bias may be NULL. */
LB2_API int32_t lb2_bias_act_fwd(void* y, const void* x, const void* bias, int64_t S, int64_t C, int64_t B,
                         int32_t dtype, int32_t act, void* stream);
/* dx = dy .* act'; dbias[c] = sum_{s,b} dx   (rrule lib/LuxLib/src/impl/bias_activation.jl:55-141,
 * ∇bias_add lib/LuxLib/src/impl/common_ops.jl:25-38). dbias may be NULL. dx may alias dy. */
LB2_API size_t lb2_bias_act_bwd_workspace_bytes(int64_t S, int64_t C, int64_t B);
LB2_API int32_t lb2_bias_act_bwd(void* dx, void* dbias, const void* dy, const void* out, const void* pre,
                         int64_t S, int64_t C, int64_t B, int32_t dtype, int32_t act,
                         void* workspace, size_t workspace_bytes, void* stream);

/* ---- dense ----------------------------------------------------------------------------- */
/* y (M x N) = act.(W (M x K) * x (K x N) .+ b (M)); optionally also stores the pre-activation
 * (needed by the gelu / swish pullback). Replaces fused_dense! / cublasLt_fused_dense!
 * (lib/LuxLib/src/impl/dense.jl:46-69, lib/LuxLib/ext/CUDAExt/cublaslt.jl:351-403) and
 * matmuladd! (lib/LuxLib/src/impl/matmul.jl:73-94) when act = identity. b, preact may be NULL. */
LB2_API size_t lb2_dense_fwd_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t dtype, uint32_t flags);
LB2_API int32_t lb2_dense_fwd(void* y, void* preact, const void* W, const void* x, const void* b,
                      int64_t M, int64_t N, int64_t K, int64_t ldw, int64_t ldx, int64_t ldy,
                      int32_t dtype, int32_t act, uint32_t flags, void* workspace,
                      size_t workspace_bytes, void* stream);
/* Pullback of the above (lib/LuxLib/src/impl/dense.jl:71-113,290-291):
 *   g  = dy .* act'(out, preact)          (out and/or preact as for lb2_act_bwd; ld = ldy)
 *   dW = g * x'   dx = W' * g   db = sum over columns of g
 * Any of dW, dx, db may be NULL (not computed). accumulate != 0 adds into dW, dx, db instead of
 * overwriting them — the Enzyme shadow contract (lib/LuxLib/src/impl/dense.jl:253-283:
 *   mul!(dW, g, x', true, true); mul!(dx, W', g, true, true); db .+= sum(g)). The last step of that rule,
 * zeroing the output shadow dy (impl/dense.jl:281), is left to the caller: dy is read-only here. */
LB2_API size_t lb2_dense_bwd_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t dtype, int32_t act,
                                     uint32_t flags);
LB2_API int32_t lb2_dense_bwd(void* dW, void* dx, void* db, const void* dy, const void* out,
                      const void* preact, const void* W, const void* x, int64_t M, int64_t N,
                      int64_t K, int64_t ldw, int64_t ldx, int64_t ldy, int32_t dtype, int32_t act,
                      int32_t accumulate, uint32_t flags, void* workspace, size_t workspace_bytes,
                      void* stream);
/* C (M x N) = op(A) * op(B) (+ C when accumulate), op = transpose when trans* != 0; A is stored
 * (M x K) or (K x M), B (K x N) or (N x K). Replaces matmul! on CuArrays
 * (lib/LuxLib/src/impl/matmul.jl:96-125) and the two GEMMs of its rrule (:228-249). */
LB2_API size_t lb2_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t dtype, uint32_t flags);
LB2_API int32_t lb2_matmul(void* C, const void* A, const void* B, int64_t M, int64_t N, int64_t K,
                   int64_t lda, int64_t ldb, int64_t ldc, int32_t transA, int32_t transB,
                   int32_t dtype, int32_t accumulate, uint32_t flags, void* workspace,
                   size_t workspace_bytes, void* stream);

/* ---- convolution ------------------------------------------------------------------------ */
/* The fields NNlib.DenseConvDims is built from at src/layers/conv.jl:253-256. Arrays are
 * x (in[0..nd) , Cin, N), w (k[0..nd), Cin/groups, Cout), y (out[0..nd), Cout, N), column-major. */
typedef struct {
  int32_t ndim;      /* spatial rank 1..3 */
  int32_t in[3];     /* input spatial extents */
  int32_t k[3];      /* kernel extents */
  int32_t stride[3];
  int32_t pad_lo[3];
  int32_t pad_hi[3];
  int32_t dilation[3];
  int32_t groups;
  int32_t flipkernel; /* 0 = true convolution (kernel flipped, the Lux default); 1 = cross-correlation */
  int32_t cin, cout, batch;
} lb2_conv_desc;
/* Fills out[0..ndim) with (in + pad_lo + pad_hi - dil*(k-1) - 1) / stride + 1 (src/layers/conv.jl:175-177). */
LB2_API int32_t lb2_conv_output_size(const lb2_conv_desc* d, int32_t* out);
/* y = act.(conv(x, w) .+ b); optional pre-activation store. Replaces conv_bias_act / conv!
 * for CUDADevice (lib/LuxLib/src/impl/conv.jl:42-60,157-166). */
LB2_API size_t lb2_conv_fwd_workspace_bytes(const lb2_conv_desc* d, int32_t dtype);
LB2_API int32_t lb2_conv_fwd(void* y, void* preact, const void* x, const void* w, const void* b,
                     const lb2_conv_desc* d, int32_t dtype, int32_t act, uint32_t flags,
                     void* workspace, size_t workspace_bytes, void* stream);
/* 1 when lb2_conv_fwd (without LB2_FLAG_FORCE_SIMT, on 16-byte aligned arrays) leaves a reusable copy of x at the
 * start of its workspace for this geometry (see LB2_FLAG_X_COPY_GIVEN), else 0. The reference keeps x itself for
 * ∇conv_filter (lib/LuxLib/src/impl/conv.jl:261-275); no counterpart in the reference for the copy. */
LB2_API int32_t lb2_conv_fwd_leaves_x_copy(const lb2_conv_desc* d, int32_t dtype);
/* conv -> BatchNorm(act) pairs (perf/resnet/resnet.jl:17-22: Conv without bias, src/layers/conv.jl:251-260, then
 * BatchNorm carrying the activation, src/layers/normalize.jl:149-190): the convolution (identity activation, no bias) that also returns per output channel the sums of the
 * stored y and of y^2 (fp32 [cout][2]) — BatchNorm's statistics pass without reading y back. On the general bf16
 * tensor-core path the sums are formed in the convolution's epilogue; elsewhere a separate pass over y forms them.
 * lb2_conv_fwd_sums_is_fused() == 1 says that the epilogue form applies AND pays (a contraction of at least 16
 * k-blocks of 64 hides it); callers should keep the plain conv + BatchNorm pair otherwise. The workspace keeps lb2_conv_fwd's layout (LB2_FLAG_X_COPY_GIVEN applies). */
LB2_API int32_t lb2_conv_fwd_sums_is_fused(const lb2_conv_desc* d, int32_t dtype);
LB2_API size_t lb2_conv_fwd_sums_workspace_bytes(const lb2_conv_desc* d, int32_t dtype);
LB2_API int32_t lb2_conv_fwd_sums(void* y, float* sums, const void* x, const void* w, const lb2_conv_desc* d, int32_t dtype,
                                  uint32_t flags, void* workspace, size_t workspace_bytes, void* stream);
/* Pullback ∇fused_conv (lib/LuxLib/src/impl/conv.jl:261-275): g = dy .* act'(out, preact);
 * dw = ∇conv_filter(x, g); dx = ∇conv_data(g, w); db = sum_{spatial,N} g. Outputs may be NULL. */
LB2_API size_t lb2_conv_bwd_workspace_bytes(const lb2_conv_desc* d, int32_t dtype, int32_t act);
LB2_API int32_t lb2_conv_bwd(void* dw, void* dx, void* db, const void* dy, const void* out,
                     const void* preact, const void* x, const void* w, const lb2_conv_desc* d,
                     int32_t dtype, int32_t act, uint32_t flags, void* workspace,
                     size_t workspace_bytes, void* stream);

/* ---- batchnorm --------------------------------------------------------------------------- */
/* x viewed as (S = prod(spatial), C, B) exactly as lib/LuxLib/src/impl/batchnorm.jl:90.
 * Training forward: batch statistics (biased variance), y = act(x*g' + b'), g' = gamma/sqrt(var+eps),
 * b' = beta - mean*g' (impl/batchnorm.jl:149-176); save_mean / save_invstd (fp32, C) are kept for
 * the backward; when rmean/rvar are given the updated running statistics
 * new = (1-m)*old + m*{mean, var*n/(n-1)} (lib/LuxLib/src/impl/normalization.jl:95-110) are written
 * to new_rmean/new_rvar (dtype `dtype`; may alias rmean/rvar). gamma/beta both NULL or both given.
 * Replaces Impl.batchnorm for CuArrays (lib/LuxLib/ext/cuDNNExt/cuDNNExt.jl:26-40) and
 * batchnorm_affine_normalize_internal! (lib/LuxLib/src/impl/batchnorm.jl:302-331). */
LB2_API size_t lb2_batchnorm_workspace_bytes(int64_t S, int64_t C, int64_t B);
LB2_API int32_t lb2_batchnorm_fwd_train(void* y, float* save_mean, float* save_invstd, void* new_rmean,
                                void* new_rvar, const void* x, const void* gamma, const void* beta,
                                const void* rmean, const void* rvar, int64_t S, int64_t C, int64_t B,
                                double momentum, double eps, int32_t dtype, int32_t act,
                                void* workspace, size_t workspace_bytes, void* stream);
/* Same operation as lb2_batchnorm_fwd_train for callers that cannot hand over a workspace because
 * they have no way to allocate one: code that runs where the host's GPU allocator must not be
 * entered (a Julia finalizer or another GC-time callback, where CUDA.jl's memory pool is off
 * limits) or a host whose device memory was carved up front by its owner, which gives this library
 * tensors but no allocator. It has no counterpart in the reference. The scratch is a fixed array
 * inside the library (LB2_BATCHNORM_STATIC_SCRATCH_BYTES per GPU, held from library load until
 * process exit); the call allocates nothing and calls no allocating routine. Problems whose scratch
 * need (lb2_batchnorm_workspace_bytes) exceeds that size are rejected with
 * LB2_WORKSPACE_TOO_SMALL (argument errors and empty problems are answered before the device is
 * touched). The first call on each device looks up the array's device address, and the first call
 * of each kernel variant (storage type x activation x small-tensor / single-launch path) makes the
 * CUDA runtime load that kernel's code, which may allocate and synchronise inside the driver: make
 * one call of every variant you will use before any stream capture and before entering a context
 * where that is not allowed. All calls on a device share the one array, which keeps the previous
 * call's contents (the call clears the words that must start at zero): two calls whose kernels may
 * overlap on the GPU (different streams) race on it — serialise them. */
#define LB2_BATCHNORM_STATIC_SCRATCH_BYTES (4u << 20)
LB2_API int32_t lb2_batchnorm_fwd_train_static(void* y, float* save_mean, float* save_invstd,
                                               void* new_rmean, void* new_rvar, const void* x,
                                               const void* gamma, const void* beta, const void* rmean,
                                               const void* rvar, int64_t S, int64_t C, int64_t B,
                                               double momentum, double eps, int32_t dtype, int32_t act,
                                               void* stream);
/* Inference forward with given statistics (lib/LuxLib/src/impl/normalization.jl:136-143). */
/* Per-channel sums of x and x^2 over the (S, C, B) view (fp32 [C][2]), and the training forward that starts from
 * such sums instead of its own statistics pass: mean = s1/n, var = s2/n - mean^2 (biased), then exactly
 * lb2_batchnorm_fwd_train's normalisation, saved statistics and running-statistics update. Workspace as for
 * lb2_batchnorm_fwd_train. */
LB2_API size_t lb2_channel_sums_workspace_bytes(int64_t S, int64_t C, int64_t B);
LB2_API int32_t lb2_channel_sums(float* sums, const void* x, int64_t S, int64_t C, int64_t B, int32_t dtype,
                                 void* workspace, size_t workspace_bytes, void* stream);
LB2_API int32_t lb2_batchnorm_fwd_train_sums(void* y, float* save_mean, float* save_invstd, void* new_rmean,
                                             void* new_rvar, const void* x, const void* gamma, const void* beta,
                                             const void* rmean, const void* rvar, const float* sums, int64_t S,
                                             int64_t C, int64_t B, double momentum, double eps, int32_t dtype,
                                             int32_t act, void* workspace, size_t workspace_bytes, void* stream);
LB2_API int32_t lb2_batchnorm_fwd_infer(void* y, const void* x, const void* gamma, const void* beta,
                                const void* rmean, const void* rvar, int64_t S, int64_t C, int64_t B,
                                double eps, int32_t dtype, int32_t act, void* stream);
/* Backward of the training forward: ∇batchnorm_affine_normalize (impl/batchnorm.jl:517-663)
 * chained through the mean_var rrule (lib/LuxLib/src/impl/common_ops.jl:45-61); the activation
 * derivative is applied inside from the recomputed pre-activation. dgamma/dbeta NULL when
 * gamma is NULL. */
LB2_API int32_t lb2_batchnorm_bwd(void* dx, void* dgamma, void* dbeta, const void* dy, const void* x,
                          const void* gamma, const void* beta, const float* save_mean,
                          const float* save_invstd, int64_t S, int64_t C, int64_t B, int32_t dtype,
                          int32_t act, void* workspace, size_t workspace_bytes, void* stream);

/* Backward of the forward with GIVEN statistics (inference mode, "frozen" BatchNorm): the rrule of
 * batchnorm_affine_normalize_internal (lib/LuxLib/src/impl/batchnorm.jl:405-443) differentiates for whatever mean
 * and variance it is handed; statistics that did not come from the batch carry no gradient, so
 *   dx = dy*act' * gamma/sqrt(rvar+eps),  dgamma = sum(dy*act' * (x-rmean)/sqrt(rvar+eps)),  dbeta = sum(dy*act').
 * Workspace: lb2_batchnorm_workspace_bytes(S, C, B). */
LB2_API int32_t lb2_batchnorm_bwd_infer(void* dx, void* dgamma, void* dbeta, const void* dy, const void* x,
                                const void* gamma, const void* beta, const void* rmean, const void* rvar,
                                int64_t S, int64_t C, int64_t B, double eps, int32_t dtype, int32_t act,
                                void* workspace, size_t workspace_bytes, void* stream);

/* ---- pooling ------------------------------------------------------------------------------- */
/* Max / mean pooling on WHCN arrays: x (in..., channels, batch) -> y (out..., channels, batch). Backs the
 * pooling layers of src/layers/pooling.jl:42-57 (NNlib.maxpool / NNlib.meanpool with a PoolDims; the global
 * pools are the window == input case). NNlib CPU semantics: windows are clipped to the input, the mean divides
 * by the full window size, the max-pool gradient goes to the first window element equal to the maximum
 * (kw fastest). lb2_pool_bwd: dx from dy (and y, x for max pooling; both may be NULL for mean pooling). */
enum { LB2_POOL_MAX = 0, LB2_POOL_MEAN = 1 };
typedef struct lb2_pool_desc {
  int32_t ndim;          /* spatial dims, 1..3 */
  int32_t in[3];
  int32_t k[3];
  int32_t stride[3];
  int32_t pad_lo[3];
  int32_t pad_hi[3];
  int32_t dilation[3];
  int32_t channels;
  int32_t batch;
} lb2_pool_desc;
LB2_API int32_t lb2_pool_output_size(const lb2_pool_desc* desc, int32_t* out);
LB2_API int32_t lb2_pool_fwd(void* y, const void* x, const lb2_pool_desc* desc, int32_t kind, int32_t dtype, void* stream);
LB2_API int32_t lb2_pool_bwd(void* dx, const void* dy, const void* y, const void* x, const lb2_pool_desc* desc,
                          int32_t kind, int32_t dtype, void* stream);

/* ---- batched matrix product, attention softmax ----------------------------------------------------- */
/* batched_matmul (lib/LuxLib/src/api/batched_mul.jl:56-70, impl/batched_mul.jl:1-60 after its reshape to 3-D):
 * C[:, :, i] = op(A[:, :, i]) * op(B[:, :, i]), i < batch, column-major with leading dimensions and batch strides in
 * elements; a stride of 0 repeats an operand (batch dimension of size 1). accumulate = 1: C += ... */
LB2_API size_t lb2_batched_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t dtype, uint32_t flags);
LB2_API int32_t lb2_batched_matmul(void* C, const void* A, const void* B, int64_t M, int64_t N, int64_t K, int64_t batch,
                                   int64_t lda, int64_t ldb, int64_t ldc, int64_t stride_a, int64_t stride_b,
                                   int64_t stride_c, int32_t transA, int32_t transB, int32_t dtype, int32_t accumulate,
                                   uint32_t flags, void* workspace, size_t workspace_bytes, void* stream);
/* The softmax step of scaled_dot_product_attention (lib/LuxLib/src/impl/attention.jl:76-131) on logits[S, L, HB]
 * (key index first): y = softmax over s of (keep ? scale * logits + bias : -inf), keep = mask (bytes, nonzero = keep;
 * NULL = all) and, with causal = 1, s <= l (make_causal_mask = triu(trues(S, L)), :131-137). bias / mask have the shape
 * [S, L] (batch stride 0) or [S, L, HB] (batch stride S*L). Backward: dlogits = scale * y .* (dy - sum_s y .* dy) and /
 * or dbias = y .* (dy - sum_s y .* dy) (either may be NULL). */
LB2_API int32_t lb2_attention_softmax_fwd(void* y, const void* logits, const void* bias, int64_t bias_batch_stride,
                                          const uint8_t* mask, int64_t mask_batch_stride, int32_t causal, double scale,
                                          int64_t S, int64_t L, int64_t HB, int32_t dtype, void* stream);
LB2_API int32_t lb2_attention_softmax_bwd(void* dlogits, void* dbias, const void* dy, const void* y, double scale,
                                          int64_t S, int64_t L, int64_t HB, int32_t dtype, void* stream);

/* ---- Scale layer ------------------------------------------------------------------------------- */
/* y = act.(x .* weight .+ bias) (src/layers/basic.jl:452-461; the {False} method has no bias: bias = NULL) with
 * weight / bias of the layer's dims and x of shape (dims..., batch...): a (D, B) column-major view, D = prod(dims).
 * Backward: g = dy .* act'(x .* weight .+ bias) (the pre-activation is rebuilt from x), dx = g .* weight,
 * dweight = sum over the batch of g .* x, dbias = sum over the batch of g (fixed summation order).
 * dbias is NULL exactly when bias is NULL. */
LB2_API int32_t lb2_scale_fwd(void* y, const void* x, const void* weight, const void* bias, int64_t D, int64_t B,
                              int32_t dtype, int32_t act, void* stream);
LB2_API size_t lb2_scale_bwd_workspace_bytes(int64_t D, int64_t B);
LB2_API int32_t lb2_scale_bwd(void* dx, void* dweight, void* dbias, const void* dy, const void* x, const void* weight,
                              const void* bias, int64_t D, int64_t B, int32_t dtype, int32_t act, void* workspace,
                              size_t workspace_bytes, void* stream);

/* ---- loss ---------------------------------------------------------------------------------------- */
/* MSELoss() (src/helpers/losses.jl:659: GenericLossFunction(l2_distance_loss; agg = mean), derivative 2(x - y) at
 * :121-125) and its gradient in one pass over n elements: *loss = mean((yhat - y)^2) (fp32, device scalar),
 * dyhat = 2 (yhat - y) / n (may be NULL, may alias yhat). */
LB2_API size_t lb2_mse_loss_workspace_bytes(int64_t n);
LB2_API int32_t lb2_mse_loss(float* loss, void* dyhat, const void* yhat, const void* y, int64_t n, int32_t dtype,
                             void* workspace, size_t workspace_bytes, void* stream);

/* CrossEntropyLoss(; dims = 1, agg = mean, logits, label_smoothing, epsilon) (src/helpers/losses.jl:383-416) on
 * (K classes, B columns) column-major arrays: *loss (fp32 device scalar) and, unless NULL, its gradient dyhat.
 * from_logits = 1: -sum(yt .* logsoftmax(yhat; dims = 1)) per column (:408-412); from_logits = 0:
 * -sum(xlogy.(yt, yhat .+ epsilon)) (:414-416), epsilon = eps(T) in the reference when not given.
 * yt = (1 - label_smoothing) * y + label_smoothing / K (:172-177). Workspace: one float per column. */
LB2_API size_t lb2_cross_entropy_workspace_bytes(int64_t K, int64_t B);
LB2_API int32_t lb2_cross_entropy(float* loss, void* dyhat, const void* yhat, const void* y, int64_t K, int64_t B,
                                  int32_t from_logits, double label_smoothing, double epsilon, int32_t dtype,
                                  void* workspace, size_t workspace_bytes, void* stream);

/* ---- optimiser step for a bucket of leaves ------------------------------------------------ */
/* The leaf loop that Optimisers.update! runs under DistributedOptimizer
 * (src/distributed/public_api.jl:270-278: allreduce!(backend, grad, avg) then apply! of the wrapped rule;
 * src/helpers/training.jl:241-245) as ONE launch per bucket of leaves, issued right after the bucket's
 * all-reduce. grad_scale multiplies every gradient first (1/world turns a sum all-reduce into the average).
 * Rules as in Optimisers.jl 0.4.6 (Descent, Momentum, Adam); state arrays have the parameter's dtype;
 * `master` (optional, fp32, same length) is updated in full precision and the parameter re-rounded from it.
 * `step` counts from 1 (Adam bias correction 1 - beta^step). `leaves` is a HOST array of device pointers. */
enum { LB2_OPT_DESCENT = 0, LB2_OPT_MOMENTUM = 1, LB2_OPT_ADAM = 2 };
typedef struct lb2_opt_leaf {
  void* param;
  const void* grad;
  void* state1;   /* Momentum: velocity; Adam: first moment; Descent: NULL */
  void* state2;   /* Adam: second moment; otherwise NULL */
  float* master;  /* optional fp32 master copy, or NULL */
  int64_t n;
} lb2_opt_leaf;
LB2_API int32_t lb2_optimizer_step(const lb2_opt_leaf* leaves, int32_t n_leaves, int32_t rule, double eta,
                          double rho_or_beta1, double beta2, double eps, int64_t step, double grad_scale,
                          int32_t dtype, void* stream);

/* ---- instancenorm --------------------------------------------------------------------------- */
/* LuxLib.instancenorm (lib/LuxLib/src/api/instancenorm.jl:32-77; generic normalization path,
 * lib/LuxLib/src/impl/normalization.jl:148-208 with reduce_dims = 1..N-2) is served by the existing
 * kernels: per-instance statistics = lb2_groupnorm_fwd / lb2_groupnorm_bwd with G = C, running
 * statistics in test mode = lb2_batchnorm_fwd_infer. This entry point is the one missing piece, the
 * running-statistics update of training mode (update_normalization_statistics,
 * impl/normalization.jl:95-110): the per-(channel, sample) statistics saved by lb2_groupnorm_fwd
 * (row b*C + c; variance recovered as 1/invstd^2 - eps) are averaged over the batch, then
 *   new_rmean = (1-m) rmean + m mean_b(mu),  new_rvar = (1-m) rvar + m S/(S-1) mean_b(var). */
LB2_API int32_t lb2_instancenorm_update_stats(void* new_rmean, void* new_rvar, const void* rmean, const void* rvar,
                          const float* save_mean, const float* save_invstd, int64_t S, int64_t C,
                          int64_t B, double momentum, double eps, int32_t dtype, void* stream);

/* ---- groupnorm ----------------------------------------------------------------------------- */
/* x viewed as (S, C/G, G, B) (lib/LuxLib/src/impl/groupnorm.jl:5-22,76-78); statistics per
 * (group, sample); save_mean / save_invstd are fp32 of length G*B. Replaces
 * groupnorm_affine_normalize_internal! (impl/groupnorm.jl:286-313). */
LB2_API int32_t lb2_groupnorm_fwd(void* y, float* save_mean, float* save_invstd, const void* x,
                          const void* gamma, const void* beta, int64_t S, int64_t C, int64_t G,
                          int64_t B, double eps, int32_t dtype, int32_t act, void* stream);
/* ∇groupnorm_affine_normalize! (impl/groupnorm.jl:477-564) chained through mean_var. */
LB2_API size_t lb2_groupnorm_bwd_workspace_bytes(int64_t S, int64_t C, int64_t G, int64_t B);
LB2_API int32_t lb2_groupnorm_bwd(void* dx, void* dgamma, void* dbeta, const void* dy, const void* x,
                          const void* gamma, const void* beta, const float* save_mean,
                          const float* save_invstd, int64_t S, int64_t C, int64_t G, int64_t B,
                          int32_t dtype, int32_t act, void* workspace, size_t workspace_bytes,
                          void* stream);

/* ---- layernorm ------------------------------------------------------------------------------ */
/* Row case of Impl.layernorm (lib/LuxLib/src/impl/layernorm.jl:3-14): x viewed as (D, R) with the
 * normalised dims leading; gamma/beta of length D or both NULL. */
LB2_API int32_t lb2_layernorm_fwd(void* y, float* save_mean, float* save_invstd, const void* x,
                          const void* gamma, const void* beta, int64_t D, int64_t R, double eps,
                          int32_t dtype, int32_t act, void* stream);
LB2_API size_t lb2_layernorm_bwd_workspace_bytes(int64_t D, int64_t R);
LB2_API int32_t lb2_layernorm_bwd(void* dx, void* dgamma, void* dbeta, const void* dy, const void* x,
                          const void* gamma, const void* beta, const float* save_mean,
                          const float* save_invstd, int64_t D, int64_t R, int32_t dtype, int32_t act,
                          void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LUXLIB_B200_H */

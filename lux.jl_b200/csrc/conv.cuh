// Internal convolution interface.
#pragma once
#include "common.cuh"

namespace lb2 {

// lb2_conv_desc normalised to three spatial dims (missing dims have extent 1).
struct ConvGeom {
  int in[3], k[3], stride[3], pad_lo[3], pad_hi[3], dil[3], out[3];
  int groups, flip, cin, cout, batch, ndim;
};

int32_t conv_fwd_direct(void* y, void* preact, const void* x, const void* w, const void* bias, const ConvGeom& g,
                        int32_t dtype, int32_t act, cudaStream_t st);
int32_t conv_dgrad_direct(void* dx, const void* dy, const void* w, const ConvGeom& g, int32_t dtype, cudaStream_t st);
int32_t conv_wgrad_direct(void* dw, const void* x, const void* dy, const ConvGeom& g, int32_t dtype, cudaStream_t st);

// Tensor-core implicit-GEMM path on the WHCN bytes themselves (2-D, stride 1, dilation 1, groups 1, output width ==
// input width, filter small enough to stay resident in shared memory); bf16 in conv_tc.cu, Float32 (split tf32 with
// register accumulation) in conv_tc_f32.cu.
bool conv_tc_supported(const ConvGeom& g, int32_t dtype);
size_t conv_tc_fwd_workspace_bytes(const ConvGeom& g, int32_t dtype);
size_t conv_tc_bwd_workspace_bytes(const ConvGeom& g, int32_t dtype);
int32_t conv_tc_fwd(void* y, void* preact, const void* x, const void* w, const void* bias, const ConvGeom& g,
                    int32_t dtype, int32_t act, void* ws, cudaStream_t st);
int32_t conv_tc_dgrad(void* dx, const void* gy, const void* w, const ConvGeom& g, int32_t dtype, void* ws, cudaStream_t st);
// `db` (optional): also the bias gradient sum_{positions, images} gy, where conv_tc_wgrad_makes_db says the kernel can
int32_t conv_tc_wgrad(void* dw, const void* x, const void* gy, const ConvGeom& g, int32_t dtype, void* ws, cudaStream_t st,
                      void* db = nullptr);
bool conv_tc_wgrad_makes_db(const ConvGeom& g, int32_t dtype);

// General bf16 tensor-core path on channel-innermost copies (conv_cw.cu): any 2-D stride / padding / dilation /
// kernel size / channel counts with groups == 1.
bool conv_cw_supported(const ConvGeom& g, int32_t dtype);
int conv_cw_fwd_kblocks(const ConvGeom& g);
size_t conv_cw_fwd_workspace_bytes(const ConvGeom& g);
size_t conv_cw_bwd_workspace_bytes(const ConvGeom& g);
int32_t conv_cw_fwd(void* y, void* preact, const void* x, const void* w, const void* bias, const ConvGeom& g, int32_t act,
                    void* ws, cudaStream_t st, float* sums = nullptr);
// both gradients (either of dw, dx may be null) from one channel-innermost copy of gy
int32_t conv_cw_bwd(void* dw, void* dx, const void* x, const void* gy, const void* w, const ConvGeom& g, void* ws,
                    cudaStream_t st, bool x_is_copy = false);

bool conv_tc_f32_supported(const ConvGeom& g);
size_t conv_tc_f32_fwd_workspace_bytes(const ConvGeom& g);
size_t conv_tc_f32_bwd_workspace_bytes(const ConvGeom& g);
int32_t conv_tc_f32_fwd(void* y, void* preact, const void* x, const void* w, const void* bias, const ConvGeom& g,
                        int32_t act, void* ws, cudaStream_t st);
// both gradients (either of dw, dx may be null) from one set of shifted copies of gy
int32_t conv_tc_f32_bwd(void* dw, void* dx, const void* x, const void* gy, const void* w, const ConvGeom& g, void* ws,
                        cudaStream_t st);

}  // namespace lb2

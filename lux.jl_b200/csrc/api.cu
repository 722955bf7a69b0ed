// Library-level entry points: version, status strings, thread-local error text and the
// per-device status word that kernels with bounded waits report through.
#include <stdarg.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "gemm.cuh"
#include "tc_ptx.cuh"

namespace lb2 {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int32_t fail(int32_t status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

// Per-device caches, created lazily under a mutex — the analogue of the cuBLASLt handle cache
// at lib/LuxLib/ext/CUDAExt/cublaslt.jl:66-82.
static std::mutex g_mu;
static int g_sm_count[64] = {0};

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

// One status word per device, living in the module's own global memory (no allocation).
__device__ unsigned int g_device_status = 0;

unsigned int* device_status_word() {
  unsigned int* p = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_device_status) != cudaSuccess) return nullptr;
  return p;
}

// One thread waits, with the given limit, on an mbarrier that nothing ever arrives at: the same wait routine the
// tensor-core kernels use, so its expiry path (status word set, kernel returns, context intact) can be exercised
// without any kernel having to hang.
__global__ void selftest_bounded_wait_kernel(unsigned int* status, uint64_t limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait_limit(&bar, 0, status, 0x40000000u, limit_ns);
  }
}

}  // namespace lb2

extern "C" {

int32_t lb2_version(void) { return 102; }

int32_t lb2_last_gemm_plan(int32_t* out, int32_t n) {
  LB2_REQUIRE(out != nullptr && n >= 0, LB2_BAD_ARG, "out is null");
  for (int i = 0; i < n && i < 8; ++i) out[i] = lb2::g_last_gemm_plan[i];
  return LB2_OK;
}

int32_t lb2_selftest_bounded_wait(uint64_t limit_ns, void* stream) {
  LB2_REQUIRE(limit_ns >= 1000 && limit_ns <= 100000000ull, LB2_BAD_ARG, "limit must be between 1 microsecond and 100 milliseconds");
  unsigned int* st = lb2::device_status_word();
  LB2_REQUIRE(st != nullptr, LB2_LAUNCH_FAIL, "status word unavailable");
  lb2::selftest_bounded_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(st, limit_ns);
  LB2_CHECK_LAUNCH("selftest_bounded_wait");
  return LB2_OK;
}

const char* lb2_status_string(int32_t s) {
  switch (s) {
    case LB2_OK: return "ok";
    case LB2_BAD_ARG: return "bad argument";
    case LB2_BAD_SHAPE: return "dimension mismatch";
    case LB2_BAD_ALIGN: return "misaligned pointer or leading dimension";
    case LB2_UNSUPPORTED_DTYPE: return "unsupported dtype";
    case LB2_LAUNCH_FAIL: return "kernel launch failed";
    case LB2_TIMEOUT: return "device-side wait timed out";
    case LB2_WORKSPACE_TOO_SMALL: return "workspace too small";
    default: return "unknown status";
  }
}

const char* lb2_last_error_string(void) { return lb2::g_err; }

int32_t lb2_poll_device_status(void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned int* p = lb2::device_status_word();
  if (!p) return lb2::fail(LB2_LAUNCH_FAIL, "status word unavailable");
  unsigned int h = 0;
  if (cudaMemcpyAsync(&h, p, sizeof(h), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess)
    return lb2::fail(LB2_LAUNCH_FAIL, "status read failed: %s", cudaGetErrorString(cudaGetLastError()));
  if (h != 0) {
    cudaMemsetAsync(p, 0, sizeof(h), st);
    cudaStreamSynchronize(st);
    return lb2::fail(LB2_TIMEOUT, "a bounded device-side wait expired (code 0x%x)", h);
  }
  return LB2_OK;
}

}  // extern "C"

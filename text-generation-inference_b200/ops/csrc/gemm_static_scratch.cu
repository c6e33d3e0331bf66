// Allocation-free front end of the bf16 stream-K GEMM: the scratch memory the kernel needs (status
// word, per-tile arrival counters, partial-tile workspace) is a file-scope device array of this
// library instead of caller-provided buffers.  See gemm_static_scratch.h for the contract.
#include "gemm_static_scratch.h"

#include <cuda_runtime.h>

#include <mutex>

extern "C" {
// existing entry points of gemm_sm100.cu
int tgi_gemm_bf16(const void* X, const void* W, void* C, const void* bias, int M, int N, int K, int max_ctas,
                  float* ws, int* counters, int* status, cudaStream_t stream);
int tgi_gemm_num_tiles(int M, int N);
long long tgi_gemm_workspace_floats(int M, int ctas);
}

namespace {

constexpr size_t kStatusBytes = 256;
constexpr size_t kCounterBytes = static_cast<size_t>(TGI_STATIC_GEMM_MAX_TILES) * sizeof(int);
constexpr size_t kScratchBytes = TGI_STATIC_GEMM_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// layout: [0, 256) status word (first int used) | counters | fp32 workspace
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

std::mutex g_mutex;
unsigned char* g_base[kMaxDevices] = {nullptr};

// Device address of g_scratch on the current device, resolved once per device.
int scratch_base(unsigned char** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return TGI_STATIC_GEMM_ERR_SETUP;
  if (dev < 0 || dev >= kMaxDevices) return TGI_STATIC_GEMM_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_base[dev] == nullptr) {
    unsigned char* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scratch);
    if (e != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();  // leave no sticky-looking error behind for the caller
      return TGI_STATIC_GEMM_ERR_SETUP;
    }
    g_base[dev] = p;
  }
  *out = g_base[dev];
  return 0;
}

}  // namespace

extern "C" {

int tgi_gemm_static_setup(void) {
  unsigned char* base = nullptr;
  return scratch_base(&base);
}

int tgi_gemm_bf16_static(const void* X, const void* W, void* C, const void* bias, int M, int N, int K,
                         cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (tgi_gemm_num_tiles(M, N) > TGI_STATIC_GEMM_MAX_TILES) return TGI_STATIC_GEMM_ERR_TOO_LARGE;
  static_assert(kStatusBytes + kCounterBytes + 2ull * TGI_STATIC_GEMM_MAX_CTAS * 32768 * sizeof(float) == kScratchBytes,
                "scratch layout and size macro disagree");
  if (tgi_gemm_workspace_floats(M, TGI_STATIC_GEMM_MAX_CTAS) * static_cast<long long>(sizeof(float)) >
      static_cast<long long>(kScratchBytes - kStatusBytes - kCounterBytes))
    return TGI_STATIC_GEMM_ERR_TOO_LARGE;
  unsigned char* base = nullptr;
  const int rc = scratch_base(&base);
  if (rc != 0) return rc;
  int* status = reinterpret_cast<int*>(base);
  int* counters = reinterpret_cast<int*>(base + kStatusBytes);
  float* ws = reinterpret_cast<float*>(base + kStatusBytes + kCounterBytes);
  // status word and counters start every call at zero
  if (cudaMemsetAsync(base, 0, kStatusBytes + kCounterBytes, stream) != cudaSuccess) return TGI_STATIC_GEMM_ERR_CLEAR;
  return tgi_gemm_bf16(X, W, C, bias, M, N, K, TGI_STATIC_GEMM_MAX_CTAS, ws, counters, status, stream);
}

int tgi_gemm_static_status(int* host_status, cudaStream_t stream) {
  unsigned char* base = nullptr;
  const int rc = scratch_base(&base);
  if (rc != 0) return rc;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return -3;
  if (cudaMemcpy(host_status, base, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -3;
  return 0;
}

const char* tgi_gemm_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case TGI_STATIC_GEMM_ERR_SETUP: return "static scratch: could not resolve the device address of the scratch array";
    case TGI_STATIC_GEMM_ERR_TOO_LARGE:
      return "static scratch: problem has more output tiles than the static counters hold (limit 4096 tiles)";
    case TGI_STATIC_GEMM_ERR_DEVICE: return "static scratch: device ordinal beyond the per-device table (limit 64)";
    case TGI_STATIC_GEMM_ERR_CLEAR: return "static scratch: clearing counters and status on the stream failed";
    case -10: return "gemm: K must be a multiple of 8";
    case -2: return "gemm: could not raise the dynamic shared memory limit";
    case -3: return "gemm: CUDA runtime error at launch";
    default: return "gemm: tensor-map encoding or another launch error";
  }
}

}  // extern "C"

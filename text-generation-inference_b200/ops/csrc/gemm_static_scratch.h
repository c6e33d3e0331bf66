// bf16 stream-K GEMM entry point that allocates no memory.
//
// This entry point has no counterpart in the reference server: it exists for hosts of this kernel
// library that cannot bring a device allocator with them.  Two kinds of caller are meant.  A plain C
// or C++ host that uses the library through its C ABI (a probe, a harness, an embedding server
// without PyTorch) has no caching allocator to carve the stream-K workspace from.  And a serving
// loop that must stay free of device-wide stalls cannot call
// cudaMalloc / cudaFree between steps, because both synchronise the whole device and every decode
// stream would wait behind them.  For these callers the workspace, the per-tile arrival counters and
// the kernel status word live in one file-scope `static __device__` array inside the library.
//
// Limits (all stated here are checked; a call beyond them fails with a negative code and launches
// nothing):
//   * the launch uses at most TGI_STATIC_GEMM_MAX_CTAS CTAs, so the partial-tile workspace is
//     2 * 32 * 128 KiB = 8 MiB;
//   * the problem may have at most TGI_STATIC_GEMM_MAX_TILES output tiles (one counter each);
//   * K must be a multiple of 8 (16-byte row pitch for TMA), as for tgi_gemm_bf16.
//
// Set-up: the first call on a device (or an explicit tgi_gemm_static_setup) resolves the device
// address of the array with cudaGetSymbolAddress while that device is current and remembers it per
// device.  Make that first call before any stream capture starts in the process, since it is a
// synchronous runtime query.  Later calls only enqueue work on `stream`.
//
// Sharing: every call on a device uses the same array.  Each call first clears the counters and the
// status word on `stream` (they must start at zero; the workspace itself needs no clearing because a
// slot is always written before it is read).  Two calls that can overlap in time (different streams,
// or different host threads on different streams) race on the array and give wrong results: order
// them on one stream or with events.
#pragma once
#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TGI_STATIC_GEMM_MAX_CTAS 32
#define TGI_STATIC_GEMM_MAX_TILES 4096
// bytes of the static scratch array: status block + counters + workspace
#define TGI_STATIC_GEMM_SCRATCH_BYTES (256 + TGI_STATIC_GEMM_MAX_TILES * 4 + 2 * TGI_STATIC_GEMM_MAX_CTAS * 32768 * 4)

// error codes of the functions below (besides the codes tgi_gemm_bf16 itself may return)
#define TGI_STATIC_GEMM_ERR_SETUP (-200)     // cudaGetDevice / cudaGetSymbolAddress failed
#define TGI_STATIC_GEMM_ERR_TOO_LARGE (-201) // more output tiles than TGI_STATIC_GEMM_MAX_TILES
#define TGI_STATIC_GEMM_ERR_DEVICE (-202)    // device ordinal outside the per-device table
#define TGI_STATIC_GEMM_ERR_CLEAR (-203)     // enqueueing the clear of counters/status failed

// Resolves the scratch address for the current device.  Idempotent; returns 0 on success.
int tgi_gemm_static_setup(void);

// C[M,N] = X[M,K] @ W[N,K]^T (+ bias[N]), bf16 in and out, fp32 accumulation; same operand layout as
// tgi_gemm_bf16.  Returns 0 when the work was enqueued on `stream`.
int tgi_gemm_bf16_static(const void* X, const void* W, void* C, const void* bias, int M, int N, int K,
                         cudaStream_t stream);

// Copies the kernel status word of the current device to *host_status after synchronising `stream`
// (0 = no bounded wait ran out).  Returns 0 on success.  Read it before the next tgi_gemm_bf16_static
// call on the device: that call clears the word, so an error that was never polled is lost.
int tgi_gemm_static_status(int* host_status, cudaStream_t stream);

// Human-readable text for a code returned by the functions above.
const char* tgi_gemm_static_strerror(int code);

#ifdef __cplusplus
}
#endif

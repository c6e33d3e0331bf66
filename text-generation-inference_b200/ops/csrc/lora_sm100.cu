// Multi-adapter LoRA for ragged batches: every token row carries the index of its adapter (0 = none) and
// the two kernels apply  out[t, col0 + n] += scale[a] * B_a[n, :] . (A_a[:, :] . x[t, :])  for all rows in
// two launches per target projection, whatever the mix of adapters in the batch.
//
// Replaces, in the reference, the punica SGMV / BGMV kernels behind `layers/lora.py:35-232`
// (`lora_a_sgmv_cutlass`, `lora_b_sgmv_cutlass`, `add_lora_a_bgmv`, `add_lora_b_bgmv`) and their per-batch
// segment / pointer-array metadata (`adapters/lora.py:287-487`).
//
// Both steps are bandwidth-bound on adapter weights that stay in L2 (rank <= 128, so A and B of one
// projection are at most a few MB per adapter), far from tensor-core territory at decode sizes:
//   shrink   one CTA per token row; each warp takes rows of A and reduces a 16-byte-vectorised dot
//            product with shuffles; result v[t, 0..r) in fp32 (all-reduced by the caller for
//            row-parallel targets).
//   expand   one thread per output column: B_a[n, 0..r) is contiguous (r bf16 values), v[t, :] sits in
//            shared memory; the sum is added to the bf16 output in place.
// The pointer tables (one entry per adapter, entry 0 unused) live in device memory and are built once
// per (layer, projection) when adapters are attached, so a step passes no host pointers and the launches
// can be captured in a CUDA graph.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.cuh"

namespace {

constexpr int kMaxRank = 128;

__global__ void __launch_bounds__(128)
lora_shrink_kernel(const __nv_bfloat16* __restrict__ x, const long long* __restrict__ a_ptrs,
                   const int* __restrict__ ranks, const int* __restrict__ token_adapter, float* __restrict__ v, int H,
                   int rmax) {
  tgi::pdl_wait();
  tgi::pdl_trigger();
  const int t = blockIdx.x;
  const int a = token_adapter[t];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* vrow = v + static_cast<size_t>(t) * rmax;
  const __nv_bfloat16* A = a > 0 ? reinterpret_cast<const __nv_bfloat16*>(a_ptrs[a]) : nullptr;
  const int r = A != nullptr ? ranks[a] : 0;
  for (int i = r + threadIdx.x; i < rmax; i += blockDim.x) vrow[i] = 0.f;   // columns past this adapter's rank
  if (r == 0) return;
  const __nv_bfloat16* xr = x + static_cast<size_t>(t) * H;
  for (int row = warp; row < r; row += 4) {
    const __nv_bfloat16* ar = A + static_cast<size_t>(row) * H;
    float acc = 0.f;
    for (int c = lane * 8; c < H; c += 32 * 8) {      // H is a multiple of 8 (checked by the launcher)
      const uint4 xa = *reinterpret_cast<const uint4*>(xr + c);
      const uint4 aa = *reinterpret_cast<const uint4*>(ar + c);
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xa);
      const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&aa);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = __bfloat1622float2(xp[j]), af = __bfloat1622float2(ap[j]);
        acc = fmaf(xf.x, af.x, acc);
        acc = fmaf(xf.y, af.y, acc);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) vrow[row] = acc;
  }
}

__global__ void __launch_bounds__(256)
lora_expand_kernel(const float* __restrict__ v, const long long* __restrict__ b_ptrs, const int* __restrict__ ranks,
                   const float* __restrict__ scales, const int* __restrict__ token_adapter,
                   __nv_bfloat16* __restrict__ out, long long out_stride, int col0, int N, int rmax) {
  tgi::pdl_wait();
  tgi::pdl_trigger();
  __shared__ float sv[kMaxRank];
  const int t = blockIdx.x;
  const int a = token_adapter[t];
  if (a <= 0) return;
  const __nv_bfloat16* B = reinterpret_cast<const __nv_bfloat16*>(b_ptrs[a]);
  const int r = ranks[a];
  if (B == nullptr || r == 0) return;
  for (int i = threadIdx.x; i < r; i += blockDim.x) sv[i] = v[static_cast<size_t>(t) * rmax + i];
  __syncthreads();
  const int n = blockIdx.y * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const __nv_bfloat16* br = B + static_cast<size_t>(n) * r;
  float acc = 0.f;
  if ((r & 7) == 0) {
    for (int c = 0; c < r; c += 8) {
      const uint4 bb = *reinterpret_cast<const uint4*>(br + c);
      const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&bb);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 bf = __bfloat1622float2(bp[j]);
        acc = fmaf(bf.x, sv[c + 2 * j], acc);
        acc = fmaf(bf.y, sv[c + 2 * j + 1], acc);
      }
    }
  } else {
    for (int c = 0; c < r; ++c) acc = fmaf(__bfloat162float(br[c]), sv[c], acc);
  }
  __nv_bfloat16* o = out + static_cast<size_t>(t) * out_stride + col0 + n;
  *o = __float2bfloat16(__bfloat162float(*o) + scales[a] * acc);
}

}  // namespace

extern "C" {

// v[T, rmax] = A_{adapter(t)} x[t]; rows without an adapter and columns past an adapter's rank are zeroed.
int tgi_lora_shrink(const void* x, const long long* a_ptrs, const int* ranks, const int* token_adapter, float* v, int T,
                    int H, int rmax, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || rmax <= 0 || rmax > kMaxRank) return -10;
  tgi::launch(lora_shrink_kernel, dim3(T), dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(x), a_ptrs, ranks,
              token_adapter, v, H, rmax);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// out[t, col0 + n] += scale_a * B_a[n, :] . v[t, :]   for n < N
int tgi_lora_expand(const float* v, const long long* b_ptrs, const int* ranks, const float* scales,
                    const int* token_adapter, void* out, long long out_stride, int col0, int T, int N, int rmax,
                    cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (rmax <= 0 || rmax > kMaxRank) return -10;
  dim3 grid(T, (N + 255) / 256);
  tgi::launch(lora_expand_kernel, dim3(grid), dim3(256), 0, stream, v, b_ptrs, ranks, scales, token_adapter,
              static_cast<__nv_bfloat16*>(out), out_stride, col0, N, rmax);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"

// Sparse mixture-of-experts on sm_100a without a host round trip:
//
//   tgi_moe_topk_softmax   softmax over the router logits + top-k (+ renormalisation), one warp per token
//   tgi_moe_sort           groups the (token, slot) pairs of the LOCAL experts by expert: per-expert counts
//                          and offsets, position of every pair in the grouped order, and the inverse list
//   tgi_moe_gather         copies the token rows into the grouped activation matrix
//   tgi_moe_grouped_gemm   one launch over all local experts: tcgen05 / TMEM / TMA GEMM whose tile list is
//                          derived on the device from the per-expert counts.  Two epilogues: gate_up with
//                          act(gate) * up fused (writes [rows, I]), down with the routing weight applied
//                          (writes [rows, H])
//   tgi_moe_combine        sums the top-k rows of every token in slot order (fixed order: bit-reproducible)
//
// Replaces, in the reference, `fused_topk` / `grouped_topk` + `moe_align_block_size` + the Triton
// `fused_experts` pair of grouped GEMMs + the weighted sum (layers/moe/unquantized.py:166-270,
// layers/moe/__init__.py:197-284).  Nothing here depends on the routing result on the host, so a decode
// step with routed experts is captured in a CUDA graph and a step only touches the rows that were routed.
//
// Grouped GEMM.  Rows of the grouped matrix belong to expert e for offsets[e] <= row < offsets[e + 1].
// A tile is 128 rows x 256 weight rows of one expert; tiles of an expert are numbered weight-tile major
// so that CTAs working side by side share the weight tile in L2.  A tile that starts inside an expert's
// range may run past its end: the extra rows belong to the next expert (or are padding) and are computed
// but not stored.  Roles inside a CTA as in gemm_sm100.cu (TMA producer warp, one MMA-issuing thread,
// eight epilogue warps), two TMEM accumulator buffers of 256 columns so that the epilogue of a tile
// overlaps the main loop of the next; all waits bounded.
#include <cuda_bf16.h>

#include <atomic>

#include "launch.cuh"
#include "sm100.cuh"
#include "tensor_map.cuh"

using namespace sm100;

namespace {

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 8;

__device__ __forceinline__ void report(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// ------------------------------------------------------------------------------------------------
// routing: softmax + top-k
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
moe_topk_softmax_kernel(const T* __restrict__ logits, int tokens, int E, int k, int renorm, float* __restrict__ out_w,
                        int* __restrict__ out_ids) {
  tgi::pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  float v[kMaxExperts / 32];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxExperts / 32; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? static_cast<float>(logits[static_cast<size_t>(t) * E + e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxExperts / 32; ++i) {
    v[i] = (i * 32 + lane) < E ? __expf(v[i] - mx) : -1.f;   // -1: not a candidate (probabilities are >= 0)
    sum += fmaxf(v[i], 0.f);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  float picked_sum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    // arg-max over the remaining candidates; ties go to the lower expert index
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > best) {
        best = v[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) v[best_e >> 5] = -1.f;
    picked_sum += best * inv;
    if (lane == j) {
      my_w = best * inv;
      my_id = best_e;
    }
  }
  if (lane < k) {
    out_w[static_cast<size_t>(t) * k + lane] = renorm ? my_w / picked_sum : my_w;
    out_ids[static_cast<size_t>(t) * k + lane] = my_id;
  }
}

// ------------------------------------------------------------------------------------------------
// grouping of the (token, slot) pairs by local expert.  One CTA; shared-memory counters.
//   pos[entry]        position of the pair in the grouped order, -1 when its expert is not local
//   order[position]   entry (token * k + slot) found at that position
//   offsets[e]        first position of local expert e; offsets[E_local] = number of grouped rows
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int entries, int first, int e_local, int* __restrict__ pos,
                int* __restrict__ order, int* __restrict__ offsets) {
  tgi::pdl_wait();
  __shared__ int cnt[kMaxExperts];
  __shared__ int off[kMaxExperts + 1];
  for (int e = threadIdx.x; e < e_local; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = ids[i] - first;
    if (e >= 0 && e < e_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < e_local; ++e) {
      off[e] = run;
      run += cnt[e];
    }
    off[e_local] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= e_local; e += blockDim.x) offsets[e] = off[e];
  for (int e = threadIdx.x; e < e_local; e += blockDim.x) cnt[e] = 0;   // reused as cursors
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = ids[i] - first;
    if (e >= 0 && e < e_local) {
      const int p = off[e] + atomicAdd(&cnt[e], 1);
      pos[i] = p;
      order[p] = i;
    } else {
      pos[i] = -1;
    }
  }
}

// grouped[p, :] = x[order[p] / k, :] for p < offsets[e_local]; 16-byte accesses (H % 8 == 0)
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ order, const int* __restrict__ offsets,
                  int e_local, int k, int H, __nv_bfloat16* __restrict__ grouped) {
  tgi::pdl_wait();
  const int rows = offsets[e_local];
  const int vec = H >> 3;
  for (int p = blockIdx.x; p < rows; p += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(order[p] / k) * H);
    uint4* dst = reinterpret_cast<uint4*>(grouped + static_cast<size_t>(p) * H);
    for (int i = threadIdx.x; i < vec; i += blockDim.x) dst[i] = src[i];
  }
}

// out[t, :] = sum over slots of y[pos[t, slot], :] (slots whose expert is not local contribute nothing)
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos, int tokens, int k, int H,
                   __nv_bfloat16* __restrict__ out) {
  tgi::pdl_wait();
  const int vec = H >> 3;
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    int p[kMaxTopK];
#pragma unroll
    for (int j = 0; j < kMaxTopK; ++j) p[j] = j < k ? pos[static_cast<size_t>(t) * k + j] : -1;
    for (int i = threadIdx.x; i < vec; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < kMaxTopK; ++j) {
        if (p[j] < 0) continue;
        const uint4 raw = reinterpret_cast<const uint4*>(y + static_cast<size_t>(p[j]) * H)[i];
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h2[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
      __nv_bfloat162 o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H)[i] = *reinterpret_cast<uint4*>(o);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// grouped GEMM
// ------------------------------------------------------------------------------------------------
constexpr int kThreads = 384;
constexpr int kEpiWarps = 8;
constexpr int kStages = 4;
constexpr int kStageBytes = 16384 + 32768;   // 128 rows of A + 256 weight rows, 128 bytes (64 bf16) of K each
constexpr int kBufCols = 256;

__device__ __forceinline__ float act_fn(float x, int act) {
  switch (act) {
    case 0: return x / (1.f + __expf(-x));                                              // silu
    case 1: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));                   // gelu (erf)
    case 2: {                                                                           // gelu (tanh)
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    default: return x / (1.f + __expf(-1.702f * x));                                    // quick gelu
  }
}

struct TileWalk {
  // tile -> (expert, first row, rows of the expert left from there, weight tile)
  const int* prefix;   // [e_local + 1] tiles before expert e (shared memory)
  const int* offsets;  // [e_local + 1] rows before expert e (shared memory)
  int e_local, n_tiles;
  __device__ __forceinline__ void locate(int tile, int& e, int& row0, int& rows_left, int& nt) const {
    int lo = 0;
    while (lo + 1 < e_local && prefix[lo + 1] <= tile) ++lo;   // e_local <= 256: a short linear walk
    e = lo;
    const int local = tile - prefix[e];
    const int cnt = offsets[e + 1] - offsets[e];
    const int mt_e = (cnt + 127) >> 7;
    nt = local / mt_e;
    const int mt = local - nt * mt_e;
    row0 = offsets[e] + mt * 128;
    rows_left = cnt - mt * 128;
  }
};

// MODE 0: gate_up.  Weights [e_local, 2 * I, K]: gate rows then up rows; a tile takes 128 gate rows and the
//         matching 128 up rows, the epilogue writes act(gate) * up to out[row, nt * 128 + j], out [rows, I].
// MODE 1: down.  Weights [e_local, Nw, K]; the epilogue writes scale[row] * acc to out[row, nt * 256 + j].
template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                        const int* __restrict__ g_offsets, int e_local, int Nw, int K, int act,
                        const float* __restrict__ topk_w, const int* __restrict__ order,
                        __nv_bfloat16* __restrict__ out, int out_cols, int* __restrict__ status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty = full + kStages;
  uint64_t* tmem_full = empty + kStages;     // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  int* s_offsets = reinterpret_cast<int*>(tmem_holder + 2);   // [e_local + 1]
  int* s_prefix = s_offsets + kMaxExperts + 1;                  // [e_local + 1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // weight tiles per expert: gate_up pairs 128 gate rows with 128 up rows (Nw = 2 * I), down takes 256 rows
  const int n_tiles = MODE == 0 ? (Nw / 2 + 127) / 128 : (Nw + 255) / 256;
  const int KB = (K + 63) / 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], kEpiWarps);
    }
    fence_barrier_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 2 * kBufCols);
    tmem_relinquish();
  }
  tgi::pdl_wait();      // the counts come from the sort kernel before this one
  tgi::pdl_trigger();
  if (threadIdx.x == 32) {
    int run = 0;
    for (int e = 0; e < e_local; ++e) {
      s_offsets[e] = g_offsets[e];
      s_prefix[e] = run;
      run += ((g_offsets[e + 1] - g_offsets[e] + 127) >> 7) * n_tiles;
    }
    s_offsets[e_local] = g_offsets[e_local];
    s_prefix[e_local] = run;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int total_tiles = s_prefix[e_local];
  TileWalk walk{s_prefix, s_offsets, e_local, n_tiles};

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_a = policy_evict_last();
      int it = 0, issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int e, row0, rows_left, nt;
        walk.locate(tile, e, row0, rows_left, nt);
        const int w_row0 = MODE == 0 ? e * Nw + nt * 128 : e * Nw + nt * 256;
        const int w_row1 = MODE == 0 ? e * Nw + Nw / 2 + nt * 128 : w_row0 + 128;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kStages;
          if (it >= kStages) ok = mbar_wait(&empty[s], ((it / kStages) - 1) & 1);
          if (!ok) { report(status, kErrProducerWait); break; }
          uint8_t* st = smem + s * kStageBytes;
          mbar_arrive_expect_tx(&full[s], kStageBytes);
          tma_load_2d_hint(st, &tmA, &full[s], kb * 64, row0, pol_a);
          tma_load_2d_hint(st + 16384, &tmW, &full[s], kb * 64, w_row0, pol_w);
          tma_load_2d_hint(st + 32768, &tmW, &full[s], kb * 64, w_row1, pol_w);
          issued = it + 1;
        }
      }
      if (!ok) {
        for (int j = max(0, issued - kStages); j < issued; ++j)
          mbar_wait(&full[j % kStages], (j / kStages) & 1, 1u << 12);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(128, 256, 1, 1);
      int it = 0, use = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++use) {
        const int b = use & 1;
        if (use >= 2 && !mbar_wait(&tmem_empty[b], ((use >> 1) - 1) & 1)) {
          report(status, kErrMmaWaitAccum);
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&full[s], (it / kStages) & 1)) {
            report(status, kErrMmaWaitFull);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
          const uint64_t da = make_desc_sw128(a_addr);
          const uint64_t dw = make_desc_sw128(a_addr + 16384);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_f16(tmem_base + b * kBufCols, da + (k * 32 >> 4), dw + (k * 32 >> 4), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(&empty[s]);
        }
        if (ok) tc_commit(&tmem_full[b]);
      }
    }
  } else if (warp >= 4) {
    // ---------------- epilogue ----------------
    const int ew = warp - 4;
    const int quarter = warp & 3;          // TMEM lane quarter this warp may read
    const int g = ew >> 2;                 // column group
    const int r_local = quarter * 32 + lane;
    int use = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++use) {
      int e, row0, rows_left, nt;
      walk.locate(tile, e, row0, rows_left, nt);
      const int b = use & 1;
      if (!mbar_wait(&tmem_full[b], (use >> 1) & 1)) {
        report(status, kErrEpilogueWait);
        break;
      }
      tc_fence_after();
      const bool row_ok = r_local < rows_left;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + b * kBufCols;
      const size_t row = static_cast<size_t>(row0 + r_local);
      if (MODE == 0) {
        // gate columns [g * 64, g * 64 + 64) and the matching up columns 128 further
        const int col0 = nt * 128 + g * 64;
#pragma unroll
        for (int c = 0; c < 64; c += 32) {
          uint32_t gv[32], uv[32];
          tmem_ld_32x32b_x32(lane_addr + g * 64 + c, gv);
          tmem_ld_32x32b_x32(lane_addr + 128 + g * 64 + c, uv);
          tmem_ld_wait();
          if (row_ok) {
            __nv_bfloat16* dst = out + row * out_cols + col0 + c;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + c + j >= out_cols) break;
              __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float a0 = act_fn(__uint_as_float(gv[j + 2 * q]), act) * __uint_as_float(uv[j + 2 * q]);
                const float a1 = act_fn(__uint_as_float(gv[j + 2 * q + 1]), act) * __uint_as_float(uv[j + 2 * q + 1]);
                o[q] = __floats2bfloat162_rn(a0, a1);
              }
              *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<uint4*>(o);
            }
          }
        }
      } else {
        const int col0 = nt * 256 + g * 128;
        const float sc = row_ok ? topk_w[order[row]] : 0.f;   // routing weight of this (token, slot) pair
#pragma unroll
        for (int c = 0; c < 128; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(lane_addr + g * 128 + c, v);
          tmem_ld_wait();
          if (row_ok) {
            __nv_bfloat16* dst = out + row * out_cols + col0 + c;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + c + j >= out_cols) break;
              __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q)
                o[q] = __floats2bfloat162_rn(__uint_as_float(v[j + 2 * q]) * sc, __uint_as_float(v[j + 2 * q + 1]) * sc);
              *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<uint4*>(o);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[b]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * kBufCols);
}

template <int MODE>
int launch_grouped(const void* A, int rows_cap, const void* W, int e_local, int Nw, int K, const int* offsets, int act,
                   const float* topk_w, const int* order, void* out, int out_cols, int ctas, int* status,
                   cudaStream_t stream) {
  CUtensorMap tmA, tmW;
  int rc = tgi::make_map_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, A, rows_cap, K, static_cast<uint64_t>(K) * 2, 128, 64,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = tgi::make_map_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, W, static_cast<uint64_t>(e_local) * Nw, K,
                        static_cast<uint64_t>(K) * 2, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  const size_t smem = kStages * kStageBytes + 1024 + 256 + 2 * (kMaxExperts + 1) * 4;
  auto kern = moe_grouped_gemm_kernel<MODE>;
  static std::atomic<unsigned long long> attr_set{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -2;
  const unsigned long long bit = 1ull << (dev & 63);
  if (!(attr_set.load(std::memory_order_acquire) & bit)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return -2;
    attr_set.fetch_or(bit, std::memory_order_release);
  }
  const cudaError_t err = tgi::launch(kern, dim3(ctas), dim3(kThreads), smem, stream, tmA, tmW, offsets, e_local, Nw, K, act,
                                      topk_w, order, static_cast<__nv_bfloat16*>(out), out_cols, status);
  return err == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace

extern "C" {

// logits [tokens, E] (fp32 when is_f32, else bf16) -> weights fp32 [tokens, k], ids int32 [tokens, k]
int tgi_moe_topk_softmax(const void* logits, int is_f32, int tokens, int E, int k, int renorm, float* out_w, int* out_ids,
                         cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (E < 1 || E > kMaxExperts || k < 1 || k > kMaxTopK || k > E) return -30;
  const dim3 grid((tokens + 3) / 4), block(128);
  cudaError_t err;
  if (is_f32)
    err = tgi::launch(moe_topk_softmax_kernel<float>, grid, block, 0, stream, static_cast<const float*>(logits), tokens, E,
                      k, renorm, out_w, out_ids);
  else
    err = tgi::launch(moe_topk_softmax_kernel<__nv_bfloat16>, grid, block, 0, stream,
                      static_cast<const __nv_bfloat16*>(logits), tokens, E, k, renorm, out_w, out_ids);
  return err == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ids int32 [entries] (entries = tokens * k); local experts are first .. first + e_local - 1
int tgi_moe_sort(const int* ids, int entries, int first, int e_local, int* pos, int* order, int* offsets,
                 cudaStream_t stream) {
  if (e_local < 1 || e_local > kMaxExperts) return -30;
  const cudaError_t err =
      tgi::launch(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, ids, entries, first, e_local, pos, order, offsets);
  return err == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int tgi_moe_gather(const void* x, const int* order, const int* offsets, int e_local, int k, int H, int max_rows,
                   void* grouped, cudaStream_t stream) {
  if (H % 8 != 0) return -31;
  if (max_rows <= 0) return 0;
  const int grid = max_rows < 2048 ? max_rows : 2048;
  const cudaError_t err = tgi::launch(moe_gather_kernel, dim3(grid), dim3(256), 0, stream,
                                      static_cast<const __nv_bfloat16*>(x), order, offsets, e_local, k, H,
                                      static_cast<__nv_bfloat16*>(grouped));
  return err == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// mode 0: out[rows_cap, Nw / 2] = act(A Wg^T) * (A Wu^T); mode 1: out[rows_cap, Nw] = w[row] * (A W^T).
// A [rows_cap, K] bf16 grouped by expert, W [e_local, Nw, K] bf16, offsets [e_local + 1] on the device.
int tgi_moe_grouped_gemm(int mode, const void* A, int rows_cap, const void* W, int e_local, int Nw, int K,
                         const int* offsets, int act, const float* topk_w, const int* order, void* out, int ctas,
                         int* status, cudaStream_t stream) {
  if (rows_cap <= 0) return 0;
  if (e_local < 1 || e_local > kMaxExperts || K % 8 != 0 || ctas < 1) return -30;
  if (mode == 0) {
    if (Nw % 2 != 0 || (Nw / 2) % 8 != 0) return -31;
    return launch_grouped<0>(A, rows_cap, W, e_local, Nw, K, offsets, act, topk_w, order, out, Nw / 2, ctas, status, stream);
  }
  if (Nw % 8 != 0) return -31;
  return launch_grouped<1>(A, rows_cap, W, e_local, Nw, K, offsets, act, topk_w, order, out, Nw, ctas, status, stream);
}

int tgi_moe_combine(const void* y, const int* pos, int tokens, int k, int H, void* out, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H % 8 != 0 || k > kMaxTopK) return -31;
  const int grid = tokens < 4096 ? tokens : 4096;
  const cudaError_t err = tgi::launch(moe_combine_kernel, dim3(grid), dim3(256), 0, stream,
                                      static_cast<const __nv_bfloat16*>(y), pos, tokens, k, H,
                                      static_cast<__nv_bfloat16*>(out));
  return err == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"

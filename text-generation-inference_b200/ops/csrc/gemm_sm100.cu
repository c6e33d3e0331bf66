// tcgen05 / TMEM / TMA GEMMs for sm_100a:   C[M, N] = X[M, K] * W[N, K]^T (+ bias)
//
//   gemm_bf16       X, W bf16, fp32 accumulation in TMEM, bf16 output
//   gemm_fp8_block  X, W e4m3 with block scales (X: 1x128 per token, W: 128x128), the scheme of
//                   DeepSeek-style fp8 checkpoints: every 128-deep K block is multiplied on the
//                   tensor cores into a fresh TMEM accumulator and promoted into fp32 registers
//                   with the product of the two block scales.
//
// Replaces, in the reference, cuBLAS `F.linear` (layers/linear.py:44) and the fp8 paths
// `w8a8_block_fp8_matmul` / `cutlass_scaled_mm` / `torch._scaled_mm` (layers/fp8.py:507-579).
//
// Orientation ("swap AB"): the 128 TMEM lanes (the MMA M dimension) run over weight rows n, the
// MMA N dimension (BN = 32..256) runs over tokens m.  A decode step has few tokens and huge weight
// matrices, so every CTA streams one 128-row weight slab exactly once from HBM while the token
// tile stays L2 resident; prefill simply uses more token tiles.  Work that has few 128-row slabs
// (narrow N, e.g. tensor-parallel shards) is split along K; partial tiles go through an fp32
// workspace and the last CTA of a tile reduces them in a fixed order (deterministic).
//
// Roles inside a CTA: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, the remaining
// warps = epilogue.  All waits are bounded (sm100.cuh): on expiry the kernel records an error code in
// `status`, drains its outstanding TMA loads, frees TMEM and returns.
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int kTileN = 128;          // weight rows per CTA (MMA M)
constexpr int kRowBytes = 128;       // K bytes per smem row (one 128B swizzle atom)

template <int BN>
struct TileCfg {
  static constexpr int kWBytes = kTileN * kRowBytes;  // 16 KB
  static constexpr int kXBytes = BN * kRowBytes;
  static constexpr int kStageBytes = kWBytes + kXBytes;
};

__device__ __forceinline__ void report(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// Split-K tail shared by both kernels: every CTA has written its fp32 partial tile to
// ws[(tile * splits + split) * BN * 128 + col * 128 + lane]; the last arriver sums them.
template <int BN>
__device__ __forceinline__ bool splitk_is_last(int* counters, int tile, int splits, int* smem_flag) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int old = atomicAdd(&counters[tile], 1);
    int last = (old == splits - 1);
    if (last) counters[tile] = 0;  // self-cleaning: ready for the next launch / graph replay
    *smem_flag = last;
  }
  __syncthreads();
  bool last = *smem_flag != 0;
  if (last) __threadfence();
  return last;
}

// ------------------------------------------------------------------------------------------------
// bf16
// ------------------------------------------------------------------------------------------------
template <int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                 __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                 int splits, float* __restrict__ ws, int* __restrict__ counters, int* __restrict__ status) {
  using Cfg = TileCfg<BN>;
  constexpr int BK = 64;  // bf16 elements per 128-byte row
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::kStageBytes);
  uint64_t* empty = full + STAGES;
  uint64_t* accum_full = empty + STAGES;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_full + 1);
  int* flag = reinterpret_cast<int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kTileN;
  const int m0 = blockIdx.y * BN;
  const int split = blockIdx.z;
  const int kb_total = (K + BK - 1) / BK;
  const int kb_per = (kb_total + splits - 1) / splits;
  const int kb_begin = split * kb_per;
  const int kb_end = min(kb_total, kb_begin + kb_per);
  const int nkb = max(0, kb_end - kb_begin);
  constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum_full, 1);
    fence_barrier_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      const uint64_t pol_w = policy_evict_first();   // weights are streamed once
      const uint64_t pol_x = policy_evict_last();    // the token tile is re-read by every slab
      int issued = 0;
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        if (i >= STAGES) ok = mbar_wait(&empty[s], ((i / STAGES) - 1) & 1);
        if (!ok) { report(status, kErrProducerWait); break; }
        uint8_t* st = smem + s * Cfg::kStageBytes;
        mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
        tma_load_2d_hint(st, &tmW, &full[s], (kb_begin + i) * BK, n0, pol_w);
        tma_load_2d_hint(st + Cfg::kWBytes, &tmX, &full[s], (kb_begin + i) * BK, m0, pol_x);
        issued = i + 1;
      }
      if (!ok) {
        // drain: wait (bounded) for the loads already issued so none lands after the CTA exits
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(&full[i % STAGES], (i / STAGES) & 1, 1u << 16);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(kTileN, BN, 1, 1);
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(&full[s], (i / STAGES) & 1);
        if (!ok) { report(status, kErrMmaWaitFull); break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * Cfg::kStageBytes);
        const uint64_t da = make_desc_sw128(a_addr);
        const uint64_t db = make_desc_sw128(a_addr + Cfg::kWBytes);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          mma_f16(tmem_base, da + (k * 32 >> 4), db + (k * 32 >> 4), idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&empty[s]);
      }
      if (ok) tc_commit(accum_full);
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;
    const int n = n0 + quarter * 32 + lane;
    bool ok = nkb == 0 ? true : mbar_wait(accum_full, 0);
    if (!ok) report(status, kErrEpilogueWait);
    tc_fence_after();
    if (ok) {
      const float b = (bias != nullptr && n < N) ? __bfloat162float(bias[n]) : 0.f;
      const int tile = blockIdx.y * gridDim.x + blockIdx.x;
      float* wsp = ws + (static_cast<size_t>(tile) * splits + split) * (BN * kTileN) + quarter * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        if (nkb > 0) {
          tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0;
        }
        if (splits == 1) {
          if (n < N) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int m = m0 + c + j;
              if (m < M) C[static_cast<size_t>(m) * N + n] = __float2bfloat16(__uint_as_float(v[j]) + b);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) wsp[(c + j) * kTileN] = __uint_as_float(v[j]);
        }
      }
    }
  }

  if (splits > 1) {
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    if (splitk_is_last<BN>(counters, tile, splits, flag)) {
      const float* base = ws + static_cast<size_t>(tile) * splits * (BN * kTileN);
      for (int idx = threadIdx.x; idx < BN * kTileN; idx += blockDim.x) {
        const int col = idx / kTileN, ln = idx % kTileN;
        const int m = m0 + col, n = n0 + ln;
        if (m < M && n < N) {
          float acc = bias != nullptr ? __bfloat162float(bias[n]) : 0.f;
          for (int s = 0; s < splits; ++s) acc += base[static_cast<size_t>(s) * (BN * kTileN) + idx];
          C[static_cast<size_t>(m) * N + n] = __float2bfloat16(acc);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------------------------------
// block-scaled e4m3
// ------------------------------------------------------------------------------------------------
// xs_t: activation scales, K-block major: xs_t[kb * xs_pitch + m]   (fp32, pitch multiple of 4)
// wscale: weight scales [ceil(N/128), K/128] row-major
template <int BN, int STAGES>
__global__ void __launch_bounds__(BN >= 64 ? 320 : 192, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                      const __grid_constant__ CUtensorMap tmS, const float* __restrict__ wscale,
                      __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                      int splits, float* __restrict__ ws, int* __restrict__ counters, int* __restrict__ status) {
  using Cfg = TileCfg<BN>;
  constexpr int BK = 128;                       // e4m3 elements per 128-byte row
  constexpr int EPI_WARPS = BN >= 64 ? 8 : 4;
  constexpr int COLS = BN / (EPI_WARPS / 4);    // token columns per epilogue warp
  constexpr int SC_STAGES = STAGES + 2;
  constexpr int kMaxKB = 256;                   // K <= 32768
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sc_ring = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes);   // [SC_STAGES][BN]
  float* ws_s = sc_ring + SC_STAGES * BN;                                       // [kMaxKB]
  uint64_t* full = reinterpret_cast<uint64_t*>(ws_s + kMaxKB);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;      // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  int* flag = reinterpret_cast<int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kTileN;
  const int m0 = blockIdx.y * BN;
  const int split = blockIdx.z;
  const int kb_total = K / BK;
  const int kb_per = (kb_total + splits - 1) / splits;
  const int kb_begin = split * kb_per;
  const int kb_end = min(kb_total, kb_begin + kb_per);
  const int nkb = max(0, kb_end - kb_begin);
  constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], EPI_WARPS);
    }
    fence_barrier_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmX);
    prefetch_tensormap(&tmS);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  // weight-scale row of this slab for the K range of this split
  for (int i = threadIdx.x; i < nkb; i += blockDim.x) ws_s[i] = wscale[static_cast<size_t>(blockIdx.x) * kb_total + kb_begin + i];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  float acc[COLS];
#pragma unroll
  for (int j = 0; j < COLS; ++j) acc[j] = 0.f;

  if (warp == 0) {
    if (elect_one()) {
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      int issued = 0;
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        if (i >= STAGES) ok = mbar_wait(&empty[s], ((i / STAGES) - 1) & 1);
        if (!ok) { report(status, kErrProducerWait); break; }
        uint8_t* st = smem + s * Cfg::kStageBytes;
        mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes + BN * 4);
        tma_load_2d_hint(st, &tmW, &full[s], (kb_begin + i) * BK, n0, pol_w);
        tma_load_2d_hint(st + Cfg::kWBytes, &tmX, &full[s], (kb_begin + i) * BK, m0, pol_x);
        tma_load_2d(sc_ring + (i % SC_STAGES) * BN, &tmS, &full[s], m0, kb_begin + i);
        issued = i + 1;
      }
      if (!ok) {
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(&full[i % STAGES], (i / STAGES) & 1, 1u << 16);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(kTileN, BN, 0, 0);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        const int b = i & 1;
        if (i >= 2 && !mbar_wait(&tmem_empty[b], ((i >> 1) - 1) & 1)) { report(status, kErrMmaWaitAccum); break; }
        if (!mbar_wait(&full[s], (i / STAGES) & 1)) { report(status, kErrMmaWaitFull); break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * Cfg::kStageBytes);
        const uint64_t da = make_desc_sw128(a_addr);
        const uint64_t db = make_desc_sw128(a_addr + Cfg::kWBytes);
#pragma unroll
        for (int k = 0; k < BK / 32; ++k) {
          mma_f8f6f4(tmem_base + b * BN, da + (k * 32 >> 4), db + (k * 32 >> 4), idesc, k > 0 ? 1u : 0u);
        }
        tc_commit(&empty[s]);
        tc_commit(&tmem_full[b]);
      }
    }
  } else {
    // ---------------- promotion + epilogue ----------------
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int col0 = (ew / 4) * COLS;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    bool ok = true;
    for (int i = 0; i < nkb; ++i) {
      const int b = i & 1;
      ok = mbar_wait(&tmem_full[b], (i >> 1) & 1);
      if (!ok) { report(status, kErrEpilogueWait); break; }
      tc_fence_after();
      const float wsc = ws_s[i];
      const float4* sc = reinterpret_cast<const float4*>(sc_ring + (i % SC_STAGES) * BN + col0);
#pragma unroll
      for (int c = 0; c < COLS; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(lane_addr + b * BN + col0 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 s4 = sc[(c + j) >> 2];
          acc[c + j + 0] = fmaf(__uint_as_float(v[j + 0]), s4.x * wsc, acc[c + j + 0]);
          acc[c + j + 1] = fmaf(__uint_as_float(v[j + 1]), s4.y * wsc, acc[c + j + 1]);
          acc[c + j + 2] = fmaf(__uint_as_float(v[j + 2]), s4.z * wsc, acc[c + j + 2]);
          acc[c + j + 3] = fmaf(__uint_as_float(v[j + 3]), s4.w * wsc, acc[c + j + 3]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[b]);
    }
    if (ok) {
      const int n = n0 + quarter * 32 + lane;
      if (splits == 1) {
        if (n < N) {
          const float bv = bias != nullptr ? __bfloat162float(bias[n]) : 0.f;
#pragma unroll
          for (int j = 0; j < COLS; ++j) {
            const int m = m0 + col0 + j;
            if (m < M) C[static_cast<size_t>(m) * N + n] = __float2bfloat16(acc[j] + bv);
          }
        }
      } else {
        const int tile = blockIdx.y * gridDim.x + blockIdx.x;
        float* wsp = ws + (static_cast<size_t>(tile) * splits + split) * (BN * kTileN) + quarter * 32 + lane;
#pragma unroll
        for (int j = 0; j < COLS; ++j) wsp[(col0 + j) * kTileN] = acc[j];
      }
    }
  }

  if (splits > 1) {
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    if (splitk_is_last<BN>(counters, tile, splits, flag)) {
      const float* base = ws + static_cast<size_t>(tile) * splits * (BN * kTileN);
      for (int idx = threadIdx.x; idx < BN * kTileN; idx += blockDim.x) {
        const int col = idx / kTileN, ln = idx % kTileN;
        const int m = m0 + col, n = n0 + ln;
        if (m < M && n < N) {
          float a = bias != nullptr ? __bfloat162float(bias[n]) : 0.f;
          for (int s = 0; s < splits; ++s) a += base[static_cast<size_t>(s) * (BN * kTileN) + idx];
          C[static_cast<size_t>(m) * N + n] = __float2bfloat16(a);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elem` bytes; box = [box_rows, box_cols]
int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem, const void* ptr, uint64_t rows, uint64_t cols,
                uint64_t row_pitch_bytes, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle sw) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -100;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
}

template <int BN, int STAGES>
int launch_bf16(const void* X, const void* W, void* C, const void* bias, int M, int N, int K, int splits, float* ws,
                int* counters, int* status, cudaStream_t stream) {
  using Cfg = TileCfg<BN>;
  CUtensorMap tmW, tmX;
  int rc = make_map_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, N, K, static_cast<uint64_t>(K) * 2, kTileN, 64,
                       CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, M, K, static_cast<uint64_t>(K) * 2, BN, 64,
                   CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  const size_t smem = STAGES * Cfg::kStageBytes + 1024 + 256;
  auto kern = gemm_bf16_kernel<BN, STAGES>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return -2;
    attr_set = true;
  }
  dim3 grid((N + kTileN - 1) / kTileN, (M + BN - 1) / BN, splits);
  kern<<<grid, 192, smem, stream>>>(tmW, tmX, static_cast<__nv_bfloat16*>(C), static_cast<const __nv_bfloat16*>(bias),
                                    M, N, K, splits, ws, counters, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

template <int BN, int STAGES>
int launch_fp8(const void* X, const float* xs_t, int xs_pitch, const void* W, const float* wscale, void* C,
               const void* bias, int M, int N, int K, int splits, float* ws, int* counters, int* status,
               cudaStream_t stream) {
  using Cfg = TileCfg<BN>;
  CUtensorMap tmW, tmX, tmS;
  int rc = make_map_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, N, K, static_cast<uint64_t>(K), kTileN, 128,
                       CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, X, M, K, static_cast<uint64_t>(K), BN, 128,
                   CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_map_2d(&tmS, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, xs_t, K / 128, M, static_cast<uint64_t>(xs_pitch) * 4, 1,
                   BN, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  const size_t smem = STAGES * Cfg::kStageBytes + (STAGES + 2) * BN * 4 + 256 * 4 + 1024 + 256;
  auto kern = gemm_fp8_block_kernel<BN, STAGES>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return -2;
    attr_set = true;
  }
  dim3 grid((N + kTileN - 1) / kTileN, (M + BN - 1) / BN, splits);
  kern<<<grid, BN >= 64 ? 320 : 192, smem, stream>>>(tmW, tmX, tmS, wscale, static_cast<__nv_bfloat16*>(C),
                                                     static_cast<const __nv_bfloat16*>(bias), M, N, K, splits, ws,
                                                     counters, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int pick_bn(int M) {
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

}  // namespace

extern "C" {

// Number of K splits for a problem: enough CTAs to fill the 148 SMs when there are few weight slabs,
// never more than the K blocks allow, and bounded by the workspace.
int tgi_gemm_pick_splits(int M, int N, int K, int bk, int sm_count) {
  const int bn = pick_bn(M);
  const int tiles = ((N + kTileN - 1) / kTileN) * ((M + bn - 1) / bn);
  const int kb = (K + bk - 1) / bk;
  if (tiles >= sm_count) return 1;
  int splits = (sm_count + tiles - 1) / tiles;
  const int max_by_k = kb / 4 > 0 ? kb / 4 : 1;   // keep at least 4 K blocks per CTA
  if (splits > max_by_k) splits = max_by_k;
  if (splits > 16) splits = 16;
  return splits < 1 ? 1 : splits;
}

// Floats of split-K workspace needed by a launch.
long long tgi_gemm_workspace_floats(int M, int N, int splits) {
  if (splits <= 1) return 0;
  const int bn = pick_bn(M);
  const long long tiles = static_cast<long long>((N + kTileN - 1) / kTileN) * ((M + bn - 1) / bn);
  return tiles * splits * bn * kTileN;
}

int tgi_gemm_bf16(const void* X, const void* W, void* C, const void* bias, int M, int N, int K, int splits, float* ws,
                  int* counters, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0) return -10;  // TMA row pitch must be a multiple of 16 bytes
  switch (pick_bn(M)) {
    case 32: return launch_bf16<32, 8>(X, W, C, bias, M, N, K, splits, ws, counters, status, stream);
    case 64: return launch_bf16<64, 6>(X, W, C, bias, M, N, K, splits, ws, counters, status, stream);
    case 128: return launch_bf16<128, 5>(X, W, C, bias, M, N, K, splits, ws, counters, status, stream);
    default: return launch_bf16<256, 4>(X, W, C, bias, M, N, K, splits, ws, counters, status, stream);
  }
}

int tgi_gemm_fp8_block(const void* X, const float* xs_t, int xs_pitch, const void* W, const float* wscale, void* C,
                       const void* bias, int M, int N, int K, int splits, float* ws, int* counters, int* status,
                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 128 != 0 || K > 32768 || xs_pitch % 4 != 0) return -10;
  switch (pick_bn(M)) {
    case 32: return launch_fp8<32, 8>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, splits, ws, counters, status, stream);
    case 64: return launch_fp8<64, 6>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, splits, ws, counters, status, stream);
    case 128: return launch_fp8<128, 5>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, splits, ws, counters, status, stream);
    default: return launch_fp8<256, 4>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, splits, ws, counters, status, stream);
  }
}

}  // extern "C"

// Weight-only quantised GEMM for sm_100a:   C[M, N] = X[M, K] (bf16) * dequant(Wq)[N, K]^T (+ bias)
//
//   4-bit:  Wq uint8 [N, K / 2], element k of a row in byte k / 2 (even k: low nibble), values 0..15;
//           w = (q - zp[g, n]) * scale[g, n]  with g = k / group  (zp: the zero point as a bf16 number, 8 when
//           absent; GPTQ, AWQ and symmetric formats are all served after a one-time repack at load,
//           utils/quantization.py)
//   8-bit:  Wq int8 [N, K], w = q * scale[g, n]  (EETQ, LLM.int8 weights, compressed-tensors W8A16)
//
// Replaces, in the reference, the Marlin / exllama / AWQ / EETQ weight-only GEMMs (layers/marlin/gptq.py:371-440,
// server/exllamav2_kernels/.../q_gemm.cu, layers/awq/quantize/cuda.py:19-49, layers/eetq.py:27-47): the packed
// weights stay packed in device memory (a 4-bit 70B model is 35 GB, not 140 GB) and a decode step streams a
// quarter of the bytes of the bf16 GEMM.
//
// The tensor cores take bf16 operands from shared memory, so the weight tile is dequantised on its way there:
//   warp 0      TMA producer: token tile [128 x 64 bf16] with the 128-byte swizzle, and the RAW weight tile
//               [128 rows x 32 or 64 bytes]
//   warps 4-11  converters, half a weight row per thread: unpack, (q - zp) * scale in fp32, round to bf16 once (the
//               same number the whole-matrix dequantisation gives) and store the 64 bytes into the operand tile in
//               the swizzled layout the MMA descriptor expects (16-byte chunk c of row r goes to chunk c ^ (r & 7)),
//               then `fence.proxy.async` and an arrival on the stage's `wready` barrier
//   warp 1      one thread issues tcgen05.mma (kind::f16, M 128 x N 128, accumulators in TMEM, two buffers)
//   warps 12-15 epilogue: TMEM -> registers -> bf16 rows of C (or fp32 partials when K is split)
// Work units are (output tile, K split); with more than one split the partial tiles go to an fp32 workspace and a
// second kernel adds them in split order (deterministic).  All waits are bounded (sm100.cuh).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

#include "launch.cuh"
#include "sm100.cuh"
#include "tensor_map.cuh"

using namespace sm100;

namespace {

constexpr int kThreads = 512;
// Two rings.  The packed weights are what comes from HBM.  A K block of 64 is only 32 bytes of a 4-bit weight row,
// and fetching 32-byte slivers of 128 rows that lie 4 KB apart ran the DRAM at a tenth of its bandwidth (measured:
// 0.6 TB/s), so the weights are fetched in slabs of 128 bytes per row (4 K blocks of 4-bit, 2 of 8-bit weights:
// whole DRAM bursts) into a ring of kRaw slabs of 16 KB, which also keeps 64 KB per SM in flight.  The token tile
// (from L2) and the converted weight tile, 16 KB each, use a ring of kStages slots of their own.
constexpr int kStages = 3;
constexpr int kRaw = 4;
constexpr int kTileM = 128, kTileN = 128, kBK = 64;

__device__ __forceinline__ void report(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

template <int BITS>
struct WqCfg {
  static constexpr int kRawRowBytes = kBK * BITS / 8;              // 32 (4-bit) or 64 (8-bit)
  static constexpr int kSlab = 128 / kRawRowBytes;                    // K blocks per slab: 4 or 2
  static constexpr int kSlabBytes = kTileN * 128;                     // 16 KB
  static constexpr int kXBytes = kTileM * 128;
  static constexpr int kWBytes = kTileN * 128;
  static constexpr int kStageBytes = kXBytes + kWBytes;               // token tile + converted weight tile
  static constexpr int kRawOff = kStages * kStageBytes;               // raw slots follow the stages
  static constexpr int kBarOff = kRawOff + kRaw * kSlabBytes;
};

template <int BITS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_wq_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmQ,
               const __half* __restrict__ scale, const __half* __restrict__ zp, int group,
               __nv_bfloat16* __restrict__ C, float* __restrict__ partial, const __nv_bfloat16* __restrict__ bias, int M,
               int N, int K, int splits, int* __restrict__ status) {
  using Cfg = WqCfg<BITS>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOff);     // token tile landed
  uint64_t* empty = full + kStages;          // MMAs done with the stage (token tile and converted weights)
  uint64_t* wready = empty + kStages;        // converted weight tile written
  uint64_t* raw_full = wready + kStages;     // [kRaw] packed weights landed
  uint64_t* raw_empty = raw_full + kRaw;     // [kRaw] converters have read them
  uint64_t* tmem_full = raw_empty + kRaw;    // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (N + kTileN - 1) / kTileN, m_tiles = (M + kTileM - 1) / kTileM;
  const int KB = (K + kBK - 1) / kBK;
  const int kb_per = (KB + splits - 1) / splits;
  const int units = n_tiles * m_tiles * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&wready[s], 8);
    }
    for (int s = 0; s < kRaw; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 8);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);
    }
    fence_barrier_init();
    prefetch_tensormap(&tmX);
    prefetch_tensormap(&tmQ);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  tgi::pdl_wait();
  tgi::pdl_trigger();

  // unit -> (tile coordinates, K-block range); the weight tile is the slow index so that the CTAs working at
  // the same time stream different weight rows and share the token tiles in L2
  auto decode = [&](int unit, int& tm, int& tn, int& kb0, int& kb1) {
    const int sp = unit % splits;
    const int tile = unit / splits;
    tm = tile % m_tiles;
    tn = tile / m_tiles;
    kb0 = sp * kb_per;
    kb1 = min(KB, kb0 + kb_per);
  };

  if (warp == 0) {
    // ---------------- TMA producer of the token tiles ----------------
    if (elect_one()) {
      const uint64_t pol_x = policy_evict_last();
      int it = 0, issued = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        int tm, tn, kb0, kb1;
        decode(unit, tm, tn, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          if (it >= kStages) ok = mbar_wait(&empty[s], ((it / kStages) - 1) & 1);
          if (!ok) { report(status, kErrProducerWait); break; }
          mbar_arrive_expect_tx(&full[s], Cfg::kXBytes);
          tma_load_2d_hint(smem + s * Cfg::kStageBytes, &tmX, &full[s], kb * kBK, tm * kTileM, pol_x);
          issued = it + 1;
        }
      }
      if (!ok)
        for (int j = max(0, issued - kStages); j < issued; ++j) mbar_wait(&full[j % kStages], (j / kStages) & 1, 1u << 12);
    }
  } else if (warp == 2) {
    // ---------------- TMA producer of the packed weights (runs kRaw slabs ahead) ----------------
    if (elect_one()) {
      const uint64_t pol_w = policy_evict_first();
      int it = 0, issued = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        int tm, tn, kb0, kb1;
        decode(unit, tm, tn, kb0, kb1);
        // a unit whose K range starts or ends inside a slab fetches the whole slab; bytes past the end of a row
        // are filled with zeros by the copy and meet zero token columns
        for (int sl = kb0 / Cfg::kSlab; sl <= (kb1 - 1) / Cfg::kSlab; ++sl, ++it) {
          const int s = it % kRaw;
          if (it >= kRaw) ok = mbar_wait(&raw_empty[s], ((it / kRaw) - 1) & 1);
          if (!ok) { report(status, kErrProducerWait); break; }
          mbar_arrive_expect_tx(&raw_full[s], Cfg::kSlabBytes);
          tma_load_2d_hint(smem + Cfg::kRawOff + s * Cfg::kSlabBytes, &tmQ, &raw_full[s], sl * 128, tn * kTileN, pol_w);
          issued = it + 1;
        }
      }
      if (!ok)
        for (int j = max(0, issued - kRaw); j < issued; ++j) mbar_wait(&raw_full[j % kRaw], (j / kRaw) & 1, 1u << 12);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(kTileM, kTileN, 0, 0);     // fp16 x fp16 (tokens are cast once per call)
      int it = 0, use = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++use) {
        int tm, tn, kb0, kb1;
        decode(unit, tm, tn, kb0, kb1);
        const int b = use & 1;
        if (use >= 2 && !mbar_wait(&tmem_empty[b], ((use >> 1) - 1) & 1)) {
          report(status, kErrMmaWaitAccum);
          break;
        }
        tc_fence_after();
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          // token tile landed (TMA), weight tile converted
          if (!mbar_wait(&full[s], (it / kStages) & 1) || !mbar_wait(&wready[s], (it / kStages) & 1)) {
            report(status, kErrMmaWaitFull);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t x_addr = smem_u32(smem + s * Cfg::kStageBytes);
          const uint64_t dx = make_desc_sw128(x_addr);
          const uint64_t dw = make_desc_sw128(x_addr + Cfg::kXBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_f16(tmem_base + b * 128, dx + (k * 32 >> 4), dw + (k * 32 >> 4), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          tc_commit(&empty[s]);
        }
        if (ok) tc_commit(&tmem_full[b]);
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ---------------- converters: half a weight row per thread ----------------
    const int t = (warp - 4) * 32 + lane;       // 0..255
    const int r = t >> 1, half = t & 1;         // row of the tile, which 32 elements of its 64
    int it = 0, rit = -1;
    bool ok = true;
    for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
      int tm, tn, kb0, kb1;
      decode(unit, tm, tn, kb0, kb1);
      int cur_slab = -1;
      const int n = min(tn * kTileN + r, N - 1);          // rows past N are loaded as zeros and never stored
      // scale and zero point of a group come from global memory: the next group's pair is requested one K block
      // early so that its latency passes under the wait and the conversion of the current block
      int g_cur = -1, g_next = -1;
      __half sc = __float2half(0.f), zq = __float2half(8.f), sc_next = sc, zq_next = zq;
      auto fetch = [&](int g, __half& s_out, __half& z_out) {
        s_out = scale[static_cast<size_t>(g) * N + n];
        z_out = (BITS == 4 && zp != nullptr) ? zp[static_cast<size_t>(g) * N + n] : __float2half(8.f);
      };
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % kStages;
        const int g = (kb * kBK) / group;
        if (g != g_cur) {
          if (g == g_next) {
            sc = sc_next;
            zq = zq_next;
          } else {
            fetch(g, sc, zq);
          }
          g_cur = g;
        }
        const int g_after = ((kb + 1) * kBK) / group;
        if (kb + 1 < kb1 && g_after != g_cur && g_after != g_next) {
          fetch(g_after, sc_next, zq_next);
          g_next = g_after;
        }
        // the slab with this K block's packed weights landed; the converted tile of the stage is free once the MMAs
        // that read its previous contents are done
        if (kb / Cfg::kSlab != cur_slab) {
          cur_slab = kb / Cfg::kSlab;
          ++rit;
          if (!mbar_wait(&raw_full[rit % kRaw], (rit / kRaw) & 1)) {
            report(status, kErrMmaWaitFull);
            ok = false;
            break;
          }
        }
        const int rs = rit % kRaw;
        if (it >= kStages && !mbar_wait(&empty[s], ((it / kStages) - 1) & 1)) {
          report(status, kErrMmaWaitFull);
          ok = false;
          break;
        }
        uint8_t* st = smem + s * Cfg::kStageBytes;
        const uint8_t* raw = smem + Cfg::kRawOff + rs * Cfg::kSlabBytes + r * 128 + (kb % Cfg::kSlab) * Cfg::kRawRowBytes +
                             half * (Cfg::kRawRowBytes / 2);
        uint8_t* dst = st + Cfg::kXBytes + r * 128;
        if (BITS == 4) {
          // Eight nibbles of a word become four fp16 pairs with one LOP3 each: (w & 0x000f000f) | 0x64006400 is the
          // pair (1024 + n0, 1024 + n4), the mask 0x00f000f0 gives (1024 + 16 n1, 1024 + 16 n5).  Subtracting
          // 1024 + zp (or multiplying by 1/16 and adding -(64 + zp)) is exact in fp16 for integer zero points, one
          // multiplication by the group's scale follows: about two instructions per weight instead of six.  The
          // converted tile is fp16 (11 significant bits) and the MMA runs fp16 x fp16 on an fp16 copy of the tokens
          // (mixing bf16 tokens with fp16 weights in one kind::f16 instruction is not done: both operands use
          // the same format here).
          const __half2 s2 = __half2half2(sc);
          const __half2 z_lo = __half2half2(__hadd(__float2half(1024.f), zq));           // 1024 + zp
          const __half2 z_hi = __half2half2(__hneg(__hadd(__float2half(64.f), zq)));     // -(64 + zp)
          const __half2 sixteenth = __float2half2_rn(0.0625f);
          const uint4 q = *reinterpret_cast<const uint4*>(raw);
          const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {         // chunk 4 * half + cc: the eight elements of word cc
            uint32_t w = words[cc];
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              uint32_t lo, hi;
              asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xEA;" : "=r"(lo) : "r"(w));
              asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xEA;" : "=r"(hi) : "r"(w));
              const __half2 a = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&lo), z_lo), s2);
              const __half2 b2 = __hmul2(__hfma2(*reinterpret_cast<const __half2*>(&hi), sixteenth, z_hi), s2);
              p[2 * j] = *reinterpret_cast<const uint32_t*>(&a);        // elements (2j, 2j + 4)
              p[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&b2);   // elements (2j + 1, 2j + 5)
              w >>= 8;
            }
            uint32_t o[4];
            asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(o[0]) : "r"(p[0]), "r"(p[1]));     // e0, e1
            asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(o[1]) : "r"(p[2]), "r"(p[3]));     // e2, e3
            asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(o[2]) : "r"(p[0]), "r"(p[1]));     // e4, e5
            asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(o[3]) : "r"(p[2]), "r"(p[3]));     // e6, e7
            const int c = half * 4 + cc;
            *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
          const float scf = __half2float(sc);
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {         // chunk 4 * half + cc: bytes 8 cc .. 8 cc + 7 of this half
            const uint2 q = *reinterpret_cast<const uint2*>(raw + cc * 8);
            const uint32_t w2[2] = {q.x, q.y};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int a = static_cast<int8_t>((w2[j >> 1] >> (16 * (j & 1))) & 0xFF);
              const int b = static_cast<int8_t>((w2[j >> 1] >> (16 * (j & 1) + 8)) & 0xFF);
              const __half2 v = __floats2half2_rn(static_cast<float>(a) * scf, static_cast<float>(b) * scf);
              o[j] = *reinterpret_cast<const uint32_t*>(&v);
            }
            const int c = half * 4 + cc;
            *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        fence_proxy_async();        // the generic-proxy stores above become visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&wready[s]);
          if (kb % Cfg::kSlab == Cfg::kSlab - 1 || kb == kb1 - 1) mbar_arrive(&raw_empty[rs]);     // done with the slab
        }
      }
    }
  } else if (warp >= 12) {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;
    const int r_local = quarter * 32 + lane;
    int use = 0;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x, ++use) {
      int tm, tn, kb0, kb1;
      decode(unit, tm, tn, kb0, kb1);
      const int b = use & 1;
      if (!mbar_wait(&tmem_full[b], (use >> 1) & 1)) {
        report(status, kErrEpilogueWait);
        break;
      }
      tc_fence_after();
      const int m = tm * kTileM + r_local;
      const int n0 = tn * kTileN;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + b * 128;
      const int sp = unit % splits;
#pragma unroll
      for (int c = 0; c < kTileN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(lane_addr + c, v);
        tmem_ld_wait();
        if (m < M) {
          if (splits == 1) {
            __nv_bfloat16* dst = C + static_cast<size_t>(m) * N + n0 + c;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (n0 + c + j >= N) break;
              __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                float f0 = __uint_as_float(v[j + 2 * q]), f1 = __uint_as_float(v[j + 2 * q + 1]);
                if (bias != nullptr) {
                  f0 += __bfloat162float(bias[n0 + c + j + 2 * q]);
                  f1 += __bfloat162float(bias[n0 + c + j + 2 * q + 1]);
                }
                o[q] = __floats2bfloat162_rn(f0, f1);
              }
              *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<uint4*>(o);
            }
          } else {
            float* dst = partial + (static_cast<size_t>(sp) * M + m) * N + n0 + c;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (n0 + c + j >= N) break;
              *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
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
  if (warp == 1) tmem_dealloc(tmem_base, 256);
}

// tokens bf16 -> fp16, clamped to the fp16 range (weight-only kernels of the reference run in fp16 too:
// layers/marlin/gptq.py, layers/gptq/exllamav2.py), 8 values per thread
__global__ void __launch_bounds__(256)
wq_cast_kernel(const __nv_bfloat16* __restrict__ x, __half* __restrict__ y, long long vecs) {
  tgi::pdl_wait();
  tgi::pdl_trigger();
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[v];
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(b[i]);
      f.x = fminf(fmaxf(f.x, -65504.f), 65504.f);
      f.y = fminf(fmaxf(f.y, -65504.f), 65504.f);
      const __half2 h = __floats2half2_rn(f.x, f.y);
      o[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(y)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// C = sum over splits (in split order) of the fp32 partials (+ bias), 8 outputs per thread
__global__ void __launch_bounds__(256)
wq_reduce_kernel(const float* __restrict__ partial, const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ C,
                 int M, int N, int splits) {
  tgi::pdl_wait();
  const size_t total = static_cast<size_t>(M) * N / 8;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < splits; ++s) {
      const float4* p = reinterpret_cast<const float4*>(partial + static_cast<size_t>(s) * M * N + i * 8);
      const float4 a = p[0], b = p[1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    const int col = static_cast<int>((i * 8) % N);
    __nv_bfloat162 o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float f0 = acc[2 * q], f1 = acc[2 * q + 1];
      if (bias != nullptr) {
        f0 += __bfloat162float(bias[col + 2 * q]);
        f1 += __bfloat162float(bias[col + 2 * q + 1]);
      }
      o[q] = __floats2bfloat162_rn(f0, f1);
    }
    reinterpret_cast<uint4*>(C)[i] = *reinterpret_cast<uint4*>(o);
  }
}

// Whole-matrix dequantisation to bf16 [N, K] (prefill-sized steps run the bf16 GEMM on it)
template <int BITS>
__global__ void __launch_bounds__(256)
wq_dequant_kernel(const uint8_t* __restrict__ wq, const __half* __restrict__ scale, const __half* __restrict__ zp,
                  int group, __nv_bfloat16* __restrict__ out, int N, int K) {
  const size_t total = static_cast<size_t>(N) * K / 8;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t e = i * 8;
    const int n = static_cast<int>(e / K), k = static_cast<int>(e % K);
    const int g = k / group;
    const float sc = __half2float(scale[static_cast<size_t>(g) * N + n]);
    float f[8];
    if (BITS == 4) {
      const float z = zp != nullptr ? __half2float(zp[static_cast<size_t>(g) * N + n]) : 8.f;
      const float off = -(128.f + z) * sc;      // same arithmetic as the GEMM's converters
      const uint32_t w = *reinterpret_cast<const uint32_t*>(wq + e / 2);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = fmaf(128.f + static_cast<float>((w >> (4 * j)) & 0xF), sc, off);
    } else {
      const uint2 w = *reinterpret_cast<const uint2*>(wq + e);
      const uint32_t ww[2] = {w.x, w.y};
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = static_cast<float>(static_cast<int8_t>((ww[j >> 2] >> (8 * (j & 3))) & 0xFF)) * sc;
    }
    __nv_bfloat162 o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) o[q] = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]);
    reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<uint4*>(o);
  }
}

template <int BITS>
int launch_wq(const void* X, void* Xh, const void* Wq, const void* scale, const void* zp, int group, void* C, float* partial,
              long long partial_floats, const void* bias, int M, int N, int K, int ctas, int* status, cudaStream_t stream) {
  using Cfg = WqCfg<BITS>;
  CUtensorMap tmX, tmQ;
  {
    const long long vecs = static_cast<long long>(M) * K / 8;
    const int cgrid = static_cast<int>(vecs / 256 + 1 < 1184 ? vecs / 256 + 1 : 1184);
    if (tgi::launch(wq_cast_kernel, dim3(cgrid), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(X),
                    static_cast<__half*>(Xh), vecs) != cudaSuccess)
      return -3;
  }
  int rc = tgi::make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, Xh, M, K, static_cast<uint64_t>(K) * 2, 128, kBK,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  const uint64_t row_bytes = static_cast<uint64_t>(K) * BITS / 8;
  rc = tgi::make_map_2d(&tmQ, CU_TENSOR_MAP_DATA_TYPE_UINT8, Wq, N, row_bytes, row_bytes, kTileN, 128,
                        CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  const size_t smem = Cfg::kBarOff + 1024 + 512;
  auto kern = gemm_wq_kernel<BITS>;
  static std::atomic<unsigned long long> attr_set{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -2;
  const unsigned long long bit = 1ull << (dev & 63);
  if (!(attr_set.load(std::memory_order_acquire) & bit)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return -2;
    attr_set.fetch_or(bit, std::memory_order_release);
  }
  int per_sm = 1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
  ctas *= per_sm > 2 ? 2 : per_sm;
  // K splits: enough units to occupy the GPU, at least 8 K blocks per unit, bounded by the workspace
  const int tiles = ((N + kTileN - 1) / kTileN) * ((M + kTileM - 1) / kTileM);
  const int KB = (K + kBK - 1) / kBK;
  // K splits: the kernel's time is (rounds of units per CTA) x (K blocks per unit); 448 tiles on 148 CTAs are 4
  // rounds of whole tiles but 13 rounds of quarter tiles (416 instead of 512 K blocks on the busiest CTA).  Each split
  // adds a partial tile and work for the reduce kernel, charged here as 8 K blocks per split.
  int splits = 1;
  if (partial != nullptr) {
    long long best = -1;
    for (int sp = 1; sp <= 16; sp *= 2) {
      if (KB % sp != 0 || KB / sp < 8 || static_cast<long long>(sp) * M * N > partial_floats) break;
      const long long rounds = (static_cast<long long>(tiles) * sp + ctas - 1) / ctas;
      const long long cost = rounds * (KB / sp) + (sp > 1 ? 8LL * sp : 0);
      if (best < 0 || cost < best) {
        best = cost;
        splits = sp;
      }
    }
  }
  if (N % 8 != 0) splits = 1;
  int grid = tiles * splits < ctas ? tiles * splits : ctas;
  if (grid < 1) grid = 1;
  cudaError_t err = tgi::launch(kern, dim3(grid), dim3(kThreads), smem, stream, tmX, tmQ,
                                static_cast<const __half*>(scale), static_cast<const __half*>(zp), group,
                                static_cast<__nv_bfloat16*>(C), partial, static_cast<const __nv_bfloat16*>(bias), M, N, K,
                                splits, status);
  if (err != cudaSuccess || cudaGetLastError() != cudaSuccess) return -3;
  if (splits > 1) {
    const long long vecs = static_cast<long long>(M) * N / 8;
    const int rgrid = static_cast<int>(vecs / 256 + 1 < 2048 ? vecs / 256 + 1 : 2048);
    err = tgi::launch(wq_reduce_kernel, dim3(rgrid), dim3(256), 0, stream, static_cast<const float*>(partial),
                      static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(C), M, N, splits);
    if (err != cudaSuccess || cudaGetLastError() != cudaSuccess) return -3;
  }
  return 0;
}

}  // namespace

extern "C" {

// bits: 4 (Wq uint8 [N, K / 2]) or 8 (Wq int8 [N, K]); scale / zp fp16 [K / group, N] (zp may be null: the 4-bit
// zero point is then 8, the 8-bit format has none); partial: fp32 workspace of `partial_floats` floats or null.
int tgi_gemm_wq(int bits, const void* X, void* Xh, const void* Wq, const void* scale, const void* zp, int group, void* C,
                float* partial, long long partial_floats, const void* bias, int M, int N, int K, int ctas, int* status,
                cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % kBK != 0 || group < kBK || group % kBK != 0 || N % 8 != 0 || ctas < 1) return -10;
  if (bits == 4) return launch_wq<4>(X, Xh, Wq, scale, zp, group, C, partial, partial_floats, bias, M, N, K, ctas, status, stream);
  if (bits == 8) return launch_wq<8>(X, Xh, Wq, scale, nullptr, group, C, partial, partial_floats, bias, M, N, K, ctas, status, stream);
  return -11;
}

// out bf16 [N, K] = dequantised weight (same formats as tgi_gemm_wq)
int tgi_wq_dequant(int bits, const void* Wq, const void* scale, const void* zp, int group, void* out, int N, int K,
                   cudaStream_t stream) {
  if (N <= 0 || K <= 0) return 0;
  if (K % 8 != 0 || group % 8 != 0) return -10;
  const long long vecs = static_cast<long long>(N) * K / 8;
  const int grid = static_cast<int>(vecs / 256 + 1 < 8192 ? vecs / 256 + 1 : 8192);
  if (bits == 4)
    tgi::launch(wq_dequant_kernel<4>, dim3(grid), dim3(256), 0, stream, static_cast<const uint8_t*>(Wq),
                static_cast<const __half*>(scale), static_cast<const __half*>(zp), group,
                static_cast<__nv_bfloat16*>(out), N, K);
  else if (bits == 8)
    tgi::launch(wq_dequant_kernel<8>, dim3(grid), dim3(256), 0, stream, static_cast<const uint8_t*>(Wq),
                static_cast<const __half*>(scale), static_cast<const __half*>(nullptr), group,
                static_cast<__nv_bfloat16*>(out), N, K);
  else
    return -11;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"

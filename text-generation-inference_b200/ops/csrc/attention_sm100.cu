// Paged causal attention for ragged batches (sm_100a build): prefill / chunked prefill with a cached
// prefix, and split-KV decode.  KV pages are [num_blocks, block_size, Hkv, D] in bf16 or e4m3 (per
// KV-head scale folded into the softmax scale and the output).
//
// Replaces, in the reference, flashinfer `BatchPrefillWithPagedKVCache` / FA2 `varlen_fwd`
// (layers/attention/cuda.py:244-296) and flashinfer `BatchDecodeWithPagedKVCache` /
// `paged_attention_v1/v2` (layers/attention/cuda.py:73-185).
//
// Structure: flash-attention style online softmax on mma.sync m16n8k16 fragments.
//
//   prefill_kernel      a CTA of 4 warps owns 64 query rows of one head; K/V tiles of 64 tokens are gathered
//                       page by page with cp.async into a double-buffered, XOR-swizzled shared-memory tile
//                       (e4m3 pages are widened to fp16 in shared memory, which is exact).
//   decode_kernel_v2    GQA-packed: the query heads that share one KV head form the 16 MMA rows of a warp, so
//                       each KV byte is read once.  Every warp runs its own 2-stage cp.async ring over chunks
//                       of 16 or 32 tokens of its slice of the KV range (no CTA-wide barrier in the loop).
//                       e4m3 K is fed to the MMA directly: the Q fragments are loaded with a k-permutation that
//                       matches the byte order of a 32-bit K word, and `cvt.rn.f16x2.e4m3x2` widens in
//                       registers; V is widened to fp16 in shared memory for ldmatrix.trans.
//   decode_merge_kernel combines the (max, sum, output) partials of the KV splits.
//
// The tensor-core path here is the legacy mma.sync one: a tcgen05 / TMEM formulation of both kernels is
// the open performance item of this file (decode is issue-bound at 0.39 of the HBM roofline, prefill reaches
// about 100 TFLOP/s).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "launch.cuh"
#include "sm100.cuh"
#include "tensor_map.cuh"

namespace {

constexpr int kTile = 64;        // KV tokens per tile
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // src-size 0 => the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[4], const void* p) {   // fills r[0], r[1]
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
template <bool F16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (F16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}
template <bool F16>
__device__ __forceinline__ uint32_t pack2(float x, float y) {
  if (F16) {
    __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  return *reinterpret_cast<uint32_t*>(&h);
}

// 16-bit tile [rows][D], 16-byte chunks XOR-swizzled by the row index
template <int D>
__device__ __forceinline__ int swz(int row, int chunk) {
  return row * D + ((chunk ^ (row & 7)) << 3);   // element offset
}

struct Params {
  const __nv_bfloat16* q;       // [T, Hq, D]
  const void* k_cache;          // [blocks, bs, Hkv, D]
  const void* v_cache;
  const int* block_tables;      // [B, max_blocks]
  const int* cu_seqlens_q;      // [B+1]
  const int* kv_lens;           // [B]
  const float* k_scale;         // [Hkv] or null
  const float* v_scale;
  __nv_bfloat16* out;           // [T, Hq, D]
  float* part_o;                // decode partials [B, Hq, nsplit, D]
  float* part_ml;               // [B, Hq, nsplit, 2]
  const int* horizon;           // optional [T]: last KV position query row t may see (>= its own position);
                                // rows of an image block that attend to each other in both directions (prefill only)
  int max_blocks, block_size, bs_shift, Hq, Hkv, num_blocks;   // block_size == 1 << bs_shift
  float scale, softcap;
  int window;
  int nsplit;
};

// Gather one 64-token K or V tile (tokens t0..t0+63 of sequence b, KV head kvh) into shared memory.
// bf16 pages land directly in the swizzled compute tile; e4m3 pages land in a raw staging tile.
template <int D, bool FP8>
__device__ __forceinline__ void load_tile(const Params& p, const void* cache, int b, int kvh, int t0, int L,
                                          void* dst) {
  constexpr int EB = FP8 ? 1 : 2;
  constexpr int CPR = D * EB / 16;                 // 16-byte chunks per token row
  constexpr int TOTAL = kTile * CPR;
  const char* base = static_cast<const char*>(cache);
  for (int c = threadIdx.x; c < TOTAL; c += blockDim.x) {
    const int row = c / CPR, cc = c % CPR;
    const int t = t0 + row;
    bool valid = t < L;
    const char* src = base;
    if (valid) {
      const int blk = p.block_tables[static_cast<size_t>(b) * p.max_blocks + (t >> p.bs_shift)];
      valid = blk >= 0 && blk < p.num_blocks;     // self-check on the block table
      const size_t slot = (static_cast<size_t>(blk) << p.bs_shift) + (t & (p.block_size - 1));
      if (valid) src = base + ((slot * p.Hkv + kvh) * D) * EB + cc * 16;
    }
    char* d;
    if (FP8) d = static_cast<char*>(dst) + row * D + cc * 16;                       // raw, unswizzled
    else d = reinterpret_cast<char*>(static_cast<uint16_t*>(dst) + swz<D>(row, cc));
    cp_async16(d, src, valid);
  }
}

// two e4m3 values -> packed fp16x2 (exact), one instruction
__device__ __forceinline__ uint32_t cvt_e4m3x2_f16x2(uint16_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}

// widen a raw e4m3 tile [64][D] to the swizzled fp16 compute tile
template <int D>
__device__ __forceinline__ void widen_tile(const uint8_t* raw, __half* dst) {
  constexpr int CPR = D / 16;
  for (int c = threadIdx.x; c < kTile * CPR; c += blockDim.x) {
    const int row = c / CPR, cc = c % CPR;
    const uint4 v = *reinterpret_cast<const uint4*>(raw + row * D + cc * 16);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = cvt_e4m3x2_f16x2(static_cast<uint16_t>(w[i] & 0xFFFF));
      o[2 * i + 1] = cvt_e4m3x2_f16x2(static_cast<uint16_t>(w[i] >> 16));
    }
    *reinterpret_cast<uint4*>(dst + swz<D>(row, 2 * cc)) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(dst + swz<D>(row, 2 * cc + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// One warp: S[16 x NT*8] = Q[16 x D] * K[tokens x D]^T for token n-tiles nt0 .. nt0+NT-1 (NT even).
template <int D, int NT, bool F16>
__device__ __forceinline__ void qk_warp(const uint32_t (&qf)[D / 16][4], const uint16_t* sK, int nt0,
                                        float (&s)[NT][4]) {
  const int lane = threadIdx.x & 31;
  const int mi = lane >> 3;
#pragma unroll
  for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      const int tok = (nt0 + 2 * np) * 8 + (lane & 7) + (mi >> 1) * 8;
      uint32_t b[4];
      ldsm_x4(b, sK + swz<D>(tok, ks * 2 + (mi & 1)));
      mma16816<F16>(s[2 * np], qf[ks], b[0], b[1]);
      mma16816<F16>(s[2 * np + 1], qf[ks], b[2], b[3]);
    }
  }
}

// One warp: O[16 x D] += P[16 x NT*8] * V[tokens x D]
template <int D, int NT, bool F16>
__device__ __forceinline__ void pv_warp(const float (&s)[NT][4], const uint16_t* sV, int nt0, float (&o)[D / 8][4]) {
  const int lane = threadIdx.x & 31;
  const int mi = lane >> 3;
#pragma unroll
  for (int kt = 0; kt < NT / 2; ++kt) {
    uint32_t a[4];
    a[0] = pack2<F16>(s[2 * kt][0], s[2 * kt][1]);
    a[1] = pack2<F16>(s[2 * kt][2], s[2 * kt][3]);
    a[2] = pack2<F16>(s[2 * kt + 1][0], s[2 * kt + 1][1]);
    a[3] = pack2<F16>(s[2 * kt + 1][2], s[2 * kt + 1][3]);
    const int tok = (nt0 + 2 * kt) * 8 + (lane & 7) + (mi & 1) * 8;
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t b[4];
      ldsm_x4_t(b, sV + swz<D>(tok, dp * 2 + (mi >> 1)));
      mma16816<F16>(o[2 * dp], a, b[0], b[1]);
      mma16816<F16>(o[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// Online-softmax update of one warp's 16 rows over NT n-tiles.  pos0/pos1: absolute positions of the
// thread's two rows (lane/4 and lane/4+8); tbase: first token of n-tile 0.
__device__ __forceinline__ float fast_exp2(float x) {   // ex2.approx: 2 ulp, -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int NT>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&alpha)[2],
                                               int tbase, int pos0, int pos1, int L, int window, float scale_log2,
                                               float softcap, float raw_scale, int hz0 = -1, int hz1 = -1) {
  // hz0 / hz1: last visible KV position of the two rows (defaults: their own positions, i.e. causal)
  if (hz0 < 0) hz0 = pos0;
  if (hz1 < 0) hz1 = pos1;
  const int lane = threadIdx.x & 31;
  float mx[2] = {-INFINITY, -INFINITY};
  // a tile that lies entirely below the diagonal of all 16 rows of the warp, inside the window and inside the
  // sequence needs no per-element mask (warp-uniform test: the warp's first row is pos0 - lane / 4)
  const int row_lo = hz0 - (lane >> 2), row_hi = pos0 - (lane >> 2) + 15, t_last = tbase + NT * 8 - 1;
  const bool plain = softcap <= 0.f && t_last <= row_lo && t_last < L && (window <= 0 || tbase > row_hi - window);
  if (plain) {
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      mx[0] = fmaxf(mx[0], fmaxf(s[i][0], s[i][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[i][2], s[i][3]));
    }
    mx[0] *= scale_log2;   // scale_log2 > 0
    mx[1] *= scale_log2;
  } else {
#pragma unroll
    for (int i = 0; i < NT; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = tbase + i * 8 + (lane & 3) * 2 + (e & 1);
        const int pos = (e < 2) ? pos0 : pos1;
        const int hz = (e < 2) ? hz0 : hz1;
        float v = s[i][e];
        if (softcap > 0.f) v = softcap * tanhf(v * raw_scale / softcap) * kLog2e;
        else v = v * scale_log2;
        const bool ok = t <= hz && t < L && (window <= 0 || t > pos - window);
        v = ok ? v : -INFINITY;
        s[i][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float mn = fmaxf(m[r], mx[r]);
    alpha[r] = (mn == -INFINITY) ? 0.f : fast_exp2(m[r] - mn);
    m[r] = mn;
  }
  float rs[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < NT; ++i) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float mm = m[e >> 1];
      float pv;
      if (plain) pv = fast_exp2(fmaf(s[i][e], scale_log2, -mm));
      else pv = (mm == -INFINITY) ? 0.f : fast_exp2(s[i][e] - mm);
      s[i][e] = pv;
      rs[e >> 1] += pv;
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
    rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
    l[r] = l[r] * alpha[r] + rs[r];
  }
}

template <int D, bool FP8>
struct Smem {
  static constexpr int kTileElems = kTile * D;                      // 16-bit elements per compute tile
  static constexpr int kQBytes = kTile * D * 2;
  // bf16 pages: 2 stages of compute tiles.  e4m3 pages: 2 stages raw + 1 compute tile.
  static constexpr int kKVBytes = FP8 ? (2 * kTile * D + kTile * D * 2) : (2 * kTile * D * 2);
  static constexpr int kBytes = kQBytes + 2 * kKVBytes;
};

// ------------------------------------------------------------------------------------------------
// prefill: grid (q tiles, Hq, B), block 128
// ------------------------------------------------------------------------------------------------
template <int D, bool FP8>
__global__ void __launch_bounds__(128)
prefill_kernel(Params p) {
  tgi::pdl_wait();      // inputs come from earlier kernels of the stream
  tgi::pdl_trigger();   // let the next kernel be placed while this one runs
  extern __shared__ __align__(128) uint8_t smem[];
  using S = Smem<D, FP8>;
  uint16_t* sQ = reinterpret_cast<uint16_t*>(smem);
  uint8_t* kv = smem + S::kQBytes;
  // layout after Q: [K region][V region]; each region = stages (raw for FP8) + compute tile (FP8)
  uint8_t* kreg = kv;
  uint8_t* vreg = kv + S::kKVBytes;

  const int b = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  const int q_begin = p.cu_seqlens_q[b], n = p.cu_seqlens_q[b + 1] - q_begin;
  if (qt * kTile >= n) return;
  const int L = p.kv_lens[b];
  const int kvh = h / (p.Hq / p.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_base = qt * kTile;                         // first query row of this CTA inside the chunk
  const int pos_first = L - n + row_base;
  const int pos_last = min(L - 1, pos_first + kTile - 1);
  int t_lo = 0;
  if (p.window > 0) t_lo = max(0, pos_first - p.window + 1) / kTile * kTile;
  const int t_hi = p.horizon != nullptr ? L : pos_last + 1;   // exclusive; with horizons a row may see up to L - 1
  const int ntiles = (t_hi - t_lo + kTile - 1) / kTile;

  // ---- Q tile -> shared (bf16, or fp16 for e4m3 pages) ----
  for (int c = threadIdx.x; c < kTile * (D / 8); c += blockDim.x) {
    const int row = c / (D / 8), cc = c % (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row_base + row < n)
      v = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(q_begin + row_base + row) * p.Hq + h) * D + cc * 8);
    if (FP8) {
      const __nv_bfloat162* bv = reinterpret_cast<const __nv_bfloat162*>(&v);
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(bv[i]);
        o[i] = pack2<true>(f.x, f.y);
      }
      v = make_uint4(o[0], o[1], o[2], o[3]);
    }
    *reinterpret_cast<uint4*>(sQ + swz<D>(row, cc)) = v;
  }
  auto stage_ptr = [&](uint8_t* region, int stg) -> void* {
    return FP8 ? static_cast<void*>(region + stg * kTile * D) : static_cast<void*>(region + stg * kTile * D * 2);
  };
  // first tile
  load_tile<D, FP8>(p, p.k_cache, b, kvh, t_lo, L, stage_ptr(kreg, 0));
  load_tile<D, FP8>(p, p.v_cache, b, kvh, t_lo, L, stage_ptr(vreg, 0));
  cp_async_commit();
  __syncthreads();

  uint32_t qf[D / 16][4];
  {
    const int mi = lane >> 3;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldsm_x4(qf[ks], sQ + swz<D>(warp * 16 + (lane & 7) + (mi & 1) * 8, ks * 2 + (mi >> 1)));
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const float ks = p.k_scale ? p.k_scale[kvh] : 1.f;
  const float vs = p.v_scale ? p.v_scale[kvh] : 1.f;
  const float raw_scale = p.scale * (FP8 ? ks : 1.f);
  const float scale_log2 = raw_scale * kLog2e;
  const int pos0 = pos_first + warp * 16 + (lane >> 2);
  const int pos1 = pos0 + 8;
  int hz0 = pos0, hz1 = pos1;
  if (p.horizon != nullptr) {
    const int r0 = row_base + warp * 16 + (lane >> 2), r1 = r0 + 8;
    if (r0 < n) hz0 = max(pos0, min(p.horizon[q_begin + r0], L - 1));
    if (r1 < n) hz1 = max(pos1, min(p.horizon[q_begin + r1], L - 1));
  }

  for (int j = 0; j < ntiles; ++j) {
    const int stg = j & 1;
    if (j + 1 < ntiles) {
      load_tile<D, FP8>(p, p.k_cache, b, kvh, t_lo + (j + 1) * kTile, L, stage_ptr(kreg, stg ^ 1));
      load_tile<D, FP8>(p, p.v_cache, b, kvh, t_lo + (j + 1) * kTile, L, stage_ptr(vreg, stg ^ 1));
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint16_t* cK;
    const uint16_t* cV;
    if (FP8) {
      __half* ck = reinterpret_cast<__half*>(kreg + 2 * kTile * D);
      __half* cv = reinterpret_cast<__half*>(vreg + 2 * kTile * D);
      widen_tile<D>(kreg + stg * kTile * D, ck);
      widen_tile<D>(vreg + stg * kTile * D, cv);
      __syncthreads();
      cK = reinterpret_cast<const uint16_t*>(ck);
      cV = reinterpret_cast<const uint16_t*>(cv);
    } else {
      cK = reinterpret_cast<const uint16_t*>(kreg + stg * kTile * D * 2);
      cV = reinterpret_cast<const uint16_t*>(vreg + stg * kTile * D * 2);
    }
    float s[8][4];
    qk_warp<D, 8, FP8>(qf, cK, 0, s);
    float alpha[2];
    softmax_update<8>(s, m, l, alpha, t_lo + j * kTile, pos0, pos1, L, p.window, scale_log2, p.softcap, raw_scale,
                      hz0, hz1);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
    pv_warp<D, 8, FP8>(s, cV, 0, o);
    __syncthreads();
  }
  cp_async_wait<0>();

  const float inv0 = l[0] > 0.f ? (FP8 ? vs : 1.f) / l[0] : 0.f;
  const float inv1 = l[1] > 0.f ? (FP8 ? vs : 1.f) / l[1] : 0.f;
  const int r0 = row_base + warp * 16 + (lane >> 2), r1 = r0 + 8;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    const int col = i * 8 + (lane & 3) * 2;
    if (r0 < n)
      *reinterpret_cast<__nv_bfloat162*>(p.out + (static_cast<size_t>(q_begin + r0) * p.Hq + h) * D + col) =
          __floats2bfloat162_rn(o[i][0] * inv0, o[i][1] * inv0);
    if (r1 < n)
      *reinterpret_cast<__nv_bfloat162*>(p.out + (static_cast<size_t>(q_begin + r1) * p.Hq + h) * D + col) =
          __floats2bfloat162_rn(o[i][2] * inv1, o[i][3] * inv1);
  }
}

// ------------------------------------------------------------------------------------------------
// decode, warp-independent pipelines.  grid (B, Hkv * gchunks, nsplit), block 128.
// The KV range of the split is cut in chunks of CT tokens; warp w takes chunks w, w+4, ...  Every
// warp runs its own 3-deep cp.async ring and never synchronises with the other warps until the
// final merge, so the CTA keeps (4 warps x 2 chunks) of KV loads in flight and a warp that waits
// for memory does not stall the others.
// ------------------------------------------------------------------------------------------------
template <int D, bool FP8>
struct DecodeSmem {
  static constexpr int CT = (FP8 && D <= 128) ? 32 : 16;        // tokens per warp chunk
  static constexpr int EB = FP8 ? 1 : 2;
  static constexpr int kStages = 2;
  static constexpr int kQBytes = 16 * D * 2;
  static constexpr int kChunkBytes = CT * D * EB;               // one K or V chunk as stored in the cache
  static constexpr int kRingBytes = kStages * 2 * kChunkBytes;  // per warp: stages x (K, V)
  static constexpr int kCompBytes = FP8 ? CT * D * 2 : 0;       // per warp: widened V (e4m3 pages only)
  static constexpr int kWarpBytes = kRingBytes + kCompBytes;
  static constexpr int kMergeBytes = 4 * 16 * D * 4 + 4 * 16 * 2 * 4;
  static constexpr int kBytes = kQBytes + (4 * kWarpBytes > kMergeBytes ? 4 * kWarpBytes : kMergeBytes);
};

// one warp gathers CT tokens of K or V (sequence b, KV head kvh, tokens t0..) into `dst`
// RAW_SWZ: e4m3 rows are stored with their 16-byte chunks XOR-ed by the row index, the layout the
// direct K-fragment loads below read without bank conflicts.
template <int D, bool FP8, int CT, bool RAW_SWZ>
__device__ __forceinline__ void warp_load_chunk(const Params& p, const void* cache, int b, int kvh, int t0, int t_end,
                                                void* dst, int lane) {
  constexpr int EB = FP8 ? 1 : 2;
  constexpr int CPR = D * EB / 16;
  const char* base = static_cast<const char*>(cache);
#pragma unroll
  for (int c = lane; c < CT * CPR; c += 32) {
    const int row = c / CPR, cc = c % CPR;
    const int t = t0 + row;
    bool valid = t < t_end;
    const char* src = base;
    if (valid) {
      const int blk = p.block_tables[static_cast<size_t>(b) * p.max_blocks + (t >> p.bs_shift)];
      valid = blk >= 0 && blk < p.num_blocks;     // self-check on the block table
      const size_t slot = (static_cast<size_t>(blk) << p.bs_shift) + (t & (p.block_size - 1));
      if (valid) src = base + ((slot * p.Hkv + kvh) * D) * EB + cc * 16;
    }
    char* d;
    if (FP8) d = static_cast<char*>(dst) + row * D + ((RAW_SWZ ? (cc ^ (row & (CPR < 8 ? CPR - 1 : 7))) : cc) << 4);
    else d = reinterpret_cast<char*>(static_cast<uint16_t*>(dst) + swz<D>(row, cc));
    cp_async16(d, src, valid);
  }
}

// S[16 x NT*8] = Q * K^T with K read straight from the raw e4m3 chunk: lane (g = lane/4, j = lane%4)
// loads the 4 consecutive bytes d = 16*ks + 4j .. +3 of token row g and widens them to the two B
// fragments of the k-step.  The MMA's k index is therefore a permutation of d inside each group of
// 16; the Q fragments (`load_q_frags_permuted`) use the same permutation, so the dot products are
// unchanged.
template <int D, int NT>
__device__ __forceinline__ void qk_warp_e4m3(const uint32_t (&qf)[D / 16][4], const uint8_t* rawK, float (&s)[NT][4]) {
  constexpr int CPR = D / 16;
  constexpr int SW = CPR < 8 ? CPR - 1 : 7;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, j = lane & 3;
#pragma unroll
  for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int tok = nt * 8 + g;
      const uint32_t w = *reinterpret_cast<const uint32_t*>(rawK + tok * D + ((ks ^ (tok & SW)) << 4) + j * 4);
      mma16816<true>(s[nt], qf[ks], cvt_e4m3x2_f16x2(static_cast<uint16_t>(w & 0xFFFF)),
                     cvt_e4m3x2_f16x2(static_cast<uint16_t>(w >> 16)));
    }
  }
}

// A fragments of the fp16 Q tile [16][D] (plain row-major) under the k permutation of qk_warp_e4m3
template <int D>
__device__ __forceinline__ void load_q_frags_permuted(const uint16_t* sQ, uint32_t (&qf)[D / 16][4]) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, j = lane & 3;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const uint2 lo = *reinterpret_cast<const uint2*>(sQ + g * D + ks * 16 + 4 * j);         // d = 4j .. 4j+3
    const uint2 hi = *reinterpret_cast<const uint2*>(sQ + (g + 8) * D + ks * 16 + 4 * j);
    qf[ks][0] = lo.x;   // row g,   k = 2j, 2j+1   <- d = 4j, 4j+1
    qf[ks][1] = hi.x;   // row g+8
    qf[ks][2] = lo.y;   // row g,   k = 2j+8, 2j+9 <- d = 4j+2, 4j+3
    qf[ks][3] = hi.y;
  }
}

template <int D, int CT>
__device__ __forceinline__ void warp_widen_chunk(const uint8_t* raw, __half* dst, int lane) {
  constexpr int CPR = D / 16;
#pragma unroll
  for (int c = lane; c < CT * CPR; c += 32) {
    const int row = c / CPR, cc = c % CPR;
    const uint4 v = *reinterpret_cast<const uint4*>(raw + row * D + cc * 16);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = cvt_e4m3x2_f16x2(static_cast<uint16_t>(w[i] & 0xFFFF));
      o[2 * i + 1] = cvt_e4m3x2_f16x2(static_cast<uint16_t>(w[i] >> 16));
    }
    *reinterpret_cast<uint4*>(dst + swz<D>(row, 2 * cc)) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(dst + swz<D>(row, 2 * cc + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

template <int D, bool FP8>
__global__ void __launch_bounds__(128)
decode_kernel_v2(Params p) {
  tgi::pdl_wait();      // inputs come from earlier kernels of the stream
  tgi::pdl_trigger();   // let the next kernel be placed while this one runs
  extern __shared__ __align__(128) uint8_t smem[];
  using S = DecodeSmem<D, FP8>;
  constexpr int CT = S::CT;
  constexpr int NT = CT / 8;
  uint16_t* sQ = reinterpret_cast<uint16_t*>(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* wbase = smem + S::kQBytes + warp * S::kWarpBytes;

  const int G = p.Hq / p.Hkv;
  const int gchunks = (G + 15) / 16;
  // KV heads are the fastest grid dimension: the CTAs that read the neighbouring slices of a token row run
  // at about the same time, which keeps the DRAM pages open
  const int b = blockIdx.y;
  const int kvh = blockIdx.x / gchunks, gc = blockIdx.x % gchunks;
  const int split = blockIdx.z;
  const int h0 = kvh * G + gc * 16;
  const int rows = min(16, G - gc * 16);
  const int L = p.kv_lens[b];
  const int q_row = p.cu_seqlens_q[b];
  if (p.cu_seqlens_q[b + 1] == q_row) return;   // sequence contributes no query this step
  const int pos = L - 1;
  int t_lo = 0;
  if (p.window > 0) t_lo = max(0, pos - p.window + 1) / CT * CT;
  const int chunks_total = (L - t_lo + CT - 1) / CT;
  const int chunks_per = (chunks_total + p.nsplit - 1) / p.nsplit;
  const int c0 = split * chunks_per;
  const int c1 = min(chunks_total, c0 + chunks_per);
  // chunks of this warp: c0 + warp + 4*i
  const int my_n = (c1 - c0 - warp + 3) / 4 > 0 ? (c1 - c0 - warp + 3) / 4 : 0;

  for (int c = threadIdx.x; c < 16 * (D / 8); c += blockDim.x) {
    const int row = c / (D / 8), cc = c % (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows) v = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(q_row) * p.Hq + h0 + row) * D + cc * 8);
    if (FP8) {
      const __nv_bfloat162* bv = reinterpret_cast<const __nv_bfloat162*>(&v);
      uint32_t o4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(bv[i]);
        o4[i] = pack2<true>(f.x, f.y);
      }
      v = make_uint4(o4[0], o4[1], o4[2], o4[3]);
    }
    // e4m3 pages: plain row-major fp16 Q (read by load_q_frags_permuted); bf16 pages: swizzled for ldmatrix
    if (FP8) *reinterpret_cast<uint4*>(sQ + row * D + cc * 8) = v;
    else *reinterpret_cast<uint4*>(sQ + swz<D>(row, cc)) = v;
  }
  auto kstage = [&](int stg) -> void* { return wbase + stg * 2 * S::kChunkBytes; };
  auto vstage = [&](int stg) -> void* { return wbase + stg * 2 * S::kChunkBytes + S::kChunkBytes; };
  auto issue = [&](int i) {
    if (i < my_n) {
      const int t0 = t_lo + (c0 + warp + 4 * i) * CT;
      warp_load_chunk<D, FP8, CT, true>(p, p.k_cache, b, kvh, t0, L, kstage(i % S::kStages), lane);
      warp_load_chunk<D, FP8, CT, false>(p, p.v_cache, b, kvh, t0, L, vstage(i % S::kStages), lane);
    }
    cp_async_commit();
  };
  issue(0);
  __syncthreads();   // Q tile visible to every warp

  uint32_t qf[D / 16][4];
  if (FP8) {
    load_q_frags_permuted<D>(sQ, qf);
  } else {
    const int mi = lane >> 3;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) ldsm_x4(qf[ks], sQ + swz<D>((lane & 7) + (mi & 1) * 8, ks * 2 + (mi >> 1)));
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const float ksc = p.k_scale ? p.k_scale[kvh] : 1.f;
  const float vsc = p.v_scale ? p.v_scale[kvh] : 1.f;
  const float raw_scale = p.scale * (FP8 ? ksc : 1.f);
  const float scale_log2 = raw_scale * kLog2e;

  for (int i = 0; i < my_n; ++i) {
    // the stage that chunk i+1 goes to was last read in iteration i-1 (program order + the
    // __syncwarp at the end of that iteration make those reads complete before this write)
    issue(i + 1);
    cp_async_wait<1>();
    __syncwarp();
    const uint16_t* cV;
    float s[NT][4];
    if (FP8) {
      __half* cv = reinterpret_cast<__half*>(wbase + S::kRingBytes);
      qk_warp_e4m3<D, NT>(qf, static_cast<const uint8_t*>(kstage(i % S::kStages)), s);
      warp_widen_chunk<D, CT>(static_cast<const uint8_t*>(vstage(i % S::kStages)), cv, lane);
      __syncwarp();
      cV = reinterpret_cast<const uint16_t*>(cv);
    } else {
      qk_warp<D, NT, false>(qf, static_cast<const uint16_t*>(kstage(i % S::kStages)), 0, s);
      cV = static_cast<const uint16_t*>(vstage(i % S::kStages));
    }
    float alpha[2];
    softmax_update<NT>(s, m, l, alpha, t_lo + (c0 + warp + 4 * i) * CT, pos, pos, L, p.window, scale_log2, p.softcap,
                       raw_scale);
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o[j][0] *= alpha[0]; o[j][1] *= alpha[0];
      o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
    }
    pv_warp<D, NT, FP8>(s, cV, 0, o);
    __syncwarp();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the four warps through shared memory (the rings are no longer needed) ----
  float* mO = reinterpret_cast<float*>(smem + S::kQBytes);   // [4][16][D]
  float* mML = mO + 4 * 16 * D;                              // [4][16][2]
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int col = i * 8 + (lane & 3) * 2;
      mO[(warp * 16 + r0) * D + col] = o[i][0];
      mO[(warp * 16 + r0) * D + col + 1] = o[i][1];
      mO[(warp * 16 + r1) * D + col] = o[i][2];
      mO[(warp * 16 + r1) * D + col + 1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      mML[(warp * 16 + r0) * 2] = m[0];
      mML[(warp * 16 + r0) * 2 + 1] = l[0];
      mML[(warp * 16 + r1) * 2] = m[1];
      mML[(warp * 16 + r1) * 2 + 1] = l[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows * D; idx += blockDim.x) {
    const int row = idx / D, col = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, mML[(w * 16 + row) * 2]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mML[(w * 16 + row) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
      acc += mO[(w * 16 + row) * D + col] * f;
      ll += mML[(w * 16 + row) * 2 + 1] * f;
    }
    const int h = h0 + row;
    if (p.nsplit == 1) {
      const float inv = ll > 0.f ? (FP8 ? vsc : 1.f) / ll : 0.f;
      p.out[(static_cast<size_t>(q_row) * p.Hq + h) * D + col] = __float2bfloat16(acc * inv);
    } else {
      const size_t pi = (static_cast<size_t>(b) * p.Hq + h) * p.nsplit + split;
      p.part_o[pi * D + col] = ll > 0.f ? acc * ((FP8 ? vsc : 1.f) / ll) : 0.f;
      if (col == 0) {
        p.part_ml[pi * 2] = mm;
        p.part_ml[pi * 2 + 1] = ll;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// decode over e4m3 pages with D = 128 and at most 8 query heads per KV head: decode_kernel_v3.
// grid (B, Hkv, nsplit), block 128.  As in v2 every warp walks its own chunks of the KV range, but
//   * the pages arrive by TMA: one `cp.async.bulk.tensor.2d` per 16 tokens of K or V (box 16 x 128
//     bytes, 128-byte swizzle) on a per-warp mbarrier ring, so a chunk costs four copy instructions
//     instead of a block-table lookup and a cp.async per 16 bytes and lane;
//   * the MMAs are transposed: S^T[tokens x heads] = K Q^T and O^T[d x heads] = V^T P^T, so the 8 query
//     heads are the N = 8 of m16n8k16 (nothing is padded to 16 rows) and K and V are A operands read
//     with 16-byte shared-memory loads straight from the raw e4m3 tiles.  Inside an MMA the order of
//     the contracted index and of the rows is free, so every lane takes the bytes as they lie in its
//     loads: for Q K^T lane (g, j) owns 16 consecutive head dimensions of token rho(g) and rho(g)+8
//     (rho = 3-bit reversal, which makes the two rows of a quarter-warp hit different banks under the
//     TMA swizzle); for P V it owns dimensions 16g..16g+15 of four tokens and pairs the bytes of two
//     tokens with `prmt` before `cvt.rn.f16x2.e4m3x2`.  No widened copy of V exists in shared memory;
//   * P goes through a 640-byte per-warp tile (heads x tokens, fp16) to change from accumulator to
//     B-operand layout; row sums stay per lane until the end.
// Every mbarrier wait is bounded; a wait that runs out sets `g_attn_status` and the warp stops
// consuming, waits (bounded) for the copies it still has in flight and takes part in the merge.
// ------------------------------------------------------------------------------------------------
__device__ int g_attn_status = 0;

template <int CT_, int STAGES_, bool FP8_ = true>
struct DecodeV3 {
  static constexpr int D = 128;
  static constexpr bool FP8 = FP8_;                     // e4m3 pages (1 byte per element) or bf16 pages
  static constexpr int EB = FP8_ ? 1 : 2;
  static constexpr int CT = CT_;                        // tokens per warp chunk (16 or 32)
  static constexpr int kStages = STAGES_;
  static constexpr int kStageBytes = 2 * CT * D * EB;   // K then V; a 16-token group is EB boxes of 16 x 128 bytes
  static constexpr int kWarpRing = kStages * kStageBytes;
  static constexpr int kRingBytes = 4 * kWarpRing;
  static constexpr int kQBytes = 8 * D * 2;
  static constexpr int kPPitch = CT + 8;                // halves per head row of the P tile
  static constexpr int kPBytes = 8 * kPPitch * 2;
  static constexpr int kOffQ = kRingBytes;
  static constexpr int kOffP = kOffQ + kQBytes;
  static constexpr int kOffBar = kOffP + 4 * kPBytes;
  static constexpr int kBytes = kOffBar + 4 * kStages * 8;
  static constexpr int kMergeBytes = 4 * 8 * D * 4 + 4 * 8 * 2 * 4;
  static constexpr int kFit = (227 * 1024) / (kBytes + 1024);
  static constexpr int kCap = (CT == 16 && FP8_) ? 4 : 3;  // 32-token chunks need about 146 registers per thread
  static constexpr int kMinBlocks = kFit > kCap ? kCap : kFit;
  static_assert(kMergeBytes <= kRingBytes, "merge scratch must fit in the rings");
  static_assert(CT == 16 || CT == 32, "chunks are one or two 16-token boxes");
};

__device__ __forceinline__ int bitrev3(int x) { return ((x & 1) << 2) | (x & 2) | ((x >> 2) & 1); }

// the two e4m3 pairs of a 32-bit word as fp16x2 (low pair, high pair)
__device__ __forceinline__ void cvt_e4m3x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 l, h;\n\t"
      "mov.b32 {l, h}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, l;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
      : "=r"(lo), "=r"(hi)
      : "r"(w));
}

template <class S>
__global__ void __launch_bounds__(128, S::kMinBlocks)
decode_kernel_v3(Params p, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
  tgi::pdl_wait();
  tgi::pdl_trigger();
  constexpr int D = S::D, CT = S::CT, MT = CT / 16, EB = S::EB;
  constexpr bool FP8 = S::FP8;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, j = lane & 3;
  uint8_t* ring = smem + warp * S::kWarpRing;
  uint16_t* sQ = reinterpret_cast<uint16_t*>(smem + S::kOffQ);
  uint16_t* sP = reinterpret_cast<uint16_t*>(smem + S::kOffP + warp * S::kPBytes);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::kOffBar) + warp * S::kStages;

  const int G = p.Hq / p.Hkv;           // <= 8 (checked by the launcher)
  // the KV heads of a sequence are neighbouring CTAs: their 128-byte slices of a token row are then fetched
  // at about the same time, which keeps the DRAM pages open
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int h0 = kvh * G;
  const int L = p.kv_lens[b];
  const int q_row = p.cu_seqlens_q[b];
  if (p.cu_seqlens_q[b + 1] == q_row) return;   // sequence contributes no query this step
  const int pos = L - 1;
  int t_lo = 0;
  if (p.window > 0) t_lo = max(0, pos - p.window + 1) / CT * CT;
  const int chunks_total = (L - t_lo + CT - 1) / CT;
  const int chunks_per = (chunks_total + p.nsplit - 1) / p.nsplit;
  const int c0 = split * chunks_per;
  const int c1 = min(chunks_total, c0 + chunks_per);
  const int my_n = (c1 - c0 - warp + 3) / 4 > 0 ? (c1 - c0 - warp + 3) / 4 : 0;   // chunks c0 + warp + 4 i

  if (lane == 0) {
    sm100::prefetch_tensormap(&tmK);
    sm100::prefetch_tensormap(&tmV);
#pragma unroll
    for (int s = 0; s < S::kStages; ++s) sm100::mbar_init(&full[s], 1);
    sm100::fence_barrier_init();
  }
  __syncwarp();

  // lanes 0..2*MT*EB-1 each fetch one box of 16 tokens x 128 bytes: lane = 2 * box + (0: K, 1: V); with bf16
  // pages a token row is two boxes (head dimensions 0-63 and 64-127).  The block-table entry of chunk i+1 is
  // read when chunk i is issued, so that no copy waits for a global load.
  const int isv = lane & 1, box = lane >> 1;
  auto first_token = [&](int i) {
    int t = t_lo + (c0 + warp + 4 * i) * CT + (box / EB) * 16;
    if (t >= L) t = (L - 1) & ~15;   // past the end: fetch the last group again (masked below)
    return t;
  };
  auto table_entry = [&](int i) {
    if (i >= my_n || lane >= 2 * MT * EB) return 0;
    return p.block_tables[static_cast<size_t>(b) * p.max_blocks + (first_token(i) >> p.bs_shift)];
  };
  int blk_next = table_entry(0);
  auto issue = [&](int i) {
    if (i >= my_n) return;
    const int stg = i % S::kStages;
    if (lane == 0) {
      sm100::fence_proxy_async();   // the stage's earlier reads (generic proxy) precede the refill
      sm100::mbar_arrive_expect_tx(&full[stg], S::kStageBytes);
    }
    __syncwarp();
    if (lane < 2 * MT * EB) {
      const int row = (blk_next << p.bs_shift) + (first_token(i) & (p.block_size - 1));
      sm100::tma_load_2d(ring + stg * S::kStageBytes + isv * (CT * D * EB) + box * 2048, isv ? &tmV : &tmK, &full[stg],
                         kvh * D * EB + (box % EB) * 128, row);
    }
    blk_next = table_entry(i + 1);
  };
  static_assert(2 * MT * EB <= 32 && 2 * MT * EB * 2048 == S::kStageBytes, "a stage is MT*EB boxes of K and of V");
#pragma unroll
  for (int s = 0; s < S::kStages - 1; ++s) issue(s);

  // Q rows of this KV head as fp16, [8][D] row-major (rows past G are zero)
  for (int c = threadIdx.x; c < 8 * (D / 8); c += blockDim.x) {
    const int row = c / (D / 8), cc = c % (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < G) {
      v = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(q_row) * p.Hq + h0 + row) * D + cc * 8);
      if (FP8) {                                   // e4m3 K widens exactly to fp16: Q follows
        const __nv_bfloat162* bv = reinterpret_cast<const __nv_bfloat162*>(&v);
        uint32_t o4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(bv[i]);
          o4[i] = pack2<true>(f.x, f.y);
        }
        v = make_uint4(o4[0], o4[1], o4[2], o4[3]);
      }
    }
    *reinterpret_cast<uint4*>(sQ + row * D + cc * 8) = v;
  }
  __syncthreads();

  // B fragments of Q^T.  e4m3 pages: for k-step (q, i) lane (head g, j) holds Q[g][64 q + 16 j + 4 i .. + 3].
  // bf16 pages: a 16-byte load of K is 8 dimensions = 2 k-steps, unit 4 q + j of the row: Q[g][8 (4 q + j) + 4 i .. + 3].
  constexpr int NQ = FP8 ? 2 : 4, NI = FP8 ? 4 : 2;
  uint32_t qb[NQ][NI][2];
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    if (FP8) {
      const uint4 lo = *reinterpret_cast<const uint4*>(sQ + g * D + 64 * q + 16 * j);
      const uint4 hi = *reinterpret_cast<const uint4*>(sQ + g * D + 64 * q + 16 * j + 8);
      qb[q][0][0] = lo.x; qb[q][0][1] = lo.y; qb[q][1][0] = lo.z; qb[q][1][1] = lo.w;
      qb[q][NI - 2][0] = hi.x; qb[q][NI - 2][1] = hi.y; qb[q][NI - 1][0] = hi.z; qb[q][NI - 1][1] = hi.w;
    } else {
      const uint4 lo = *reinterpret_cast<const uint4*>(sQ + g * D + 8 * (4 * q + j));
      qb[q][0][0] = lo.x; qb[q][0][1] = lo.y; qb[q][1][0] = lo.z; qb[q][1][1] = lo.w;
    }
  }

  // o[i]: dimensions 16 g + 2 i (elements 0, 1) and 16 g + 2 i + 1 (elements 2, 3) of heads 2j (0, 2) and 2j+1 (1, 3)
  float o[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};   // heads 2j, 2j+1; l is this lane's share
  const float ksc = p.k_scale ? p.k_scale[kvh] : 1.f;
  const float vsc = p.v_scale ? p.v_scale[kvh] : 1.f;
  const float raw_scale = p.scale * (FP8 ? ksc : 1.f);
  const float scale_log2 = raw_scale * kLog2e;
  const int rg = bitrev3(g);                      // token row (mod 8) of this lane's S^T rows
  const int rj0 = bitrev3(j), rj1 = bitrev3(j + 4);   // token rows (mod 8) of this lane's V loads
  bool failed = false;
  int done = 0;

  for (int i = 0; i < my_n; ++i) {
    issue(i + S::kStages - 1);
    if (!__all_sync(0xffffffffu, sm100::mbar_wait(&full[i % S::kStages], (i / S::kStages) & 1))) {
      failed = true;   // warp-uniform
      break;
    }
    done = i + 1;
    const uint8_t* sK = ring + (i % S::kStages) * S::kStageBytes;
    const uint8_t* sV = sK + CT * D * EB;
    const int tbase = t_lo + (c0 + warp + 4 * i) * CT;

    // ---- S^T = K Q^T (two accumulators per 16 tokens keep the dependent MMA chains short) ----
    float s[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float s2[2][4];
#pragma unroll
      for (int e = 0; e < 4; ++e) s2[0][e] = s2[1][e] = 0.f;
      if (FP8) {
        const uint8_t* ra = sK + (mt * 16 + rg) * D;
        const uint8_t* rb = ra + 8 * D;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int off = ((4 * q + j) ^ rg) << 4;
          const uint4 wa = *reinterpret_cast<const uint4*>(ra + off);
          const uint4 wb = *reinterpret_cast<const uint4*>(rb + off);
          const uint32_t a4[4] = {wa.x, wa.y, wa.z, wa.w}, b4[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint32_t a[4];
            cvt_e4m3x4(a4[k], a[0], a[2]);
            cvt_e4m3x4(b4[k], a[1], a[3]);
            mma16816<true>(s2[q], a, qb[q % NQ][k % NI][0], qb[q % NQ][k % NI][1]);
          }
        }
      } else {
        // bf16 rows are two boxes of 128 bytes; unit 4 q + j of the row is unit (4 q + j) % 8 of box q / 2
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint8_t* ra = sK + ((mt * 2 + (q >> 1)) * 16 + rg) * 128;
          const int off = ((4 * (q & 1) + j) ^ rg) << 4;
          const uint4 wa = *reinterpret_cast<const uint4*>(ra + off);
          const uint4 wb = *reinterpret_cast<const uint4*>(ra + 8 * 128 + off);
          const uint32_t a0[4] = {wa.x, wb.x, wa.y, wb.y}, a1[4] = {wa.z, wb.z, wa.w, wb.w};
          mma16816<false>(s2[q & 1], a0, qb[q % NQ][0][0], qb[q % NQ][0][1]);
          mma16816<false>(s2[q & 1], a1, qb[q % NQ][1][0], qb[q % NQ][1][1]);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) s[mt][e] = s2[0][e] + s2[1][e];
    }

    // ---- online softmax over the tokens of the chunk, per head ----
    // m[] is kept in the scaled log2 domain; a chunk that needs no masking takes the short path
    const bool plain = p.softcap <= 0.f && tbase + CT <= L && (p.window <= 0 || tbase > pos - p.window);
    float mx[2] = {-INFINITY, -INFINITY};
    if (plain) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mx[0] = fmaxf(mx[0], fmaxf(s[mt][0], s[mt][2]));
        mx[1] = fmaxf(mx[1], fmaxf(s[mt][1], s[mt][3]));
      }
      mx[0] *= scale_log2;   // scale_log2 > 0
      mx[1] *= scale_log2;
    } else {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int t = tbase + mt * 16 + rg + (e >> 1) * 8;
          float v = s[mt][e];
          if (p.softcap > 0.f) v = p.softcap * tanhf(v * raw_scale / p.softcap) * kLog2e;
          else v = v * scale_log2;
          const bool ok = t < L && (p.window <= 0 || t > pos - p.window);
          v = ok ? v : -INFINITY;
          s[mt][e] = v;
          mx[e & 1] = fmaxf(mx[e & 1], v);
        }
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 4));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 8));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 16));
      const float mn = fmaxf(m[r], mx[r]);
      alpha[r] = (mn == -INFINITY) ? 0.f : fast_exp2(m[r] - mn);
      m[r] = mn;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mm = m[e & 1];
        float pv;
        if (plain) pv = fast_exp2(fmaf(s[mt][e], scale_log2, -mm));
        else pv = (mm == -INFINITY) ? 0.f : fast_exp2(s[mt][e] - mm);
        s[mt][e] = pv;
        rs[e & 1] += pv;
      }
      // contraction index of P V inside the 16 tokens: 2 g (token rho(g)) and 2 g + 1 (token rho(g) + 8)
      *reinterpret_cast<uint32_t*>(sP + (2 * j) * S::kPPitch + mt * 16 + 2 * g) = pack2<FP8>(s[mt][0], s[mt][2]);
      *reinterpret_cast<uint32_t*>(sP + (2 * j + 1) * S::kPPitch + mt * 16 + 2 * g) = pack2<FP8>(s[mt][1], s[mt][3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l[r] = l[r] * alpha[r] + rs[r];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      o[k][0] *= alpha[0]; o[k][2] *= alpha[0];
      o[k][1] *= alpha[1]; o[k][3] *= alpha[1];
    }
    __syncwarp();
    uint32_t pb[4];   // B fragments of P^T: (b0, b1) of k-step 0, then of k-step 1
    if (MT == 2) ldsm_x4(pb, sP + (lane & 7) * S::kPPitch + (lane >> 3) * 8);
    else ldsm_x2(pb, sP + (lane & 7) * S::kPPitch + ((lane >> 3) & 1) * 8);

    // ---- O^T += V^T P^T ----
#pragma unroll
    for (int ks = 0; ks < MT; ++ks) {
      if (FP8) {
        const uint8_t* base = sV + ks * 16 * D;
        const uint4 wa = *reinterpret_cast<const uint4*>(base + rj0 * D + ((g ^ rj0) << 4));         // k = 2j
        const uint4 wb = *reinterpret_cast<const uint4*>(base + (rj0 + 8) * D + ((g ^ rj0) << 4));   // k = 2j + 1
        const uint4 wc = *reinterpret_cast<const uint4*>(base + rj1 * D + ((g ^ rj1) << 4));         // k = 2j + 8
        const uint4 wd = *reinterpret_cast<const uint4*>(base + (rj1 + 8) * D + ((g ^ rj1) << 4));   // k = 2j + 9
        const uint32_t a4[4] = {wa.x, wa.y, wa.z, wa.w}, b4[4] = {wb.x, wb.y, wb.z, wb.w};
        const uint32_t c4[4] = {wc.x, wc.y, wc.z, wc.w}, d4[4] = {wd.x, wd.y, wd.z, wd.w};
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          // bytes 4x .. 4x+3 of the lane's 16 dimensions: (0, 1) feed o[2x], (2, 3) feed o[2x+1]
          uint32_t a[4], a2[4];
          cvt_e4m3x4(__byte_perm(a4[x], b4[x], 0x5140), a[0], a[1]);
          cvt_e4m3x4(__byte_perm(c4[x], d4[x], 0x5140), a[2], a[3]);
          cvt_e4m3x4(__byte_perm(a4[x], b4[x], 0x7362), a2[0], a2[1]);
          cvt_e4m3x4(__byte_perm(c4[x], d4[x], 0x7362), a2[2], a2[3]);
          mma16816<true>(o[2 * x], a, pb[2 * ks], pb[2 * ks + 1]);
          mma16816<true>(o[2 * x + 1], a2, pb[2 * ks], pb[2 * ks + 1]);
        }
      } else {
        // bf16: the lane owns dimensions 8 g .. 8 g + 7 of each half of the head (unit g of both boxes);
        // o[4 hf + x] collects dimensions 64 hf + 8 g + 2 x (elements 0, 1) and + 2 x + 1 (elements 2, 3)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const uint8_t* base = sV + (ks * 2 + hf) * 2048;
          const uint4 wa = *reinterpret_cast<const uint4*>(base + rj0 * 128 + ((g ^ rj0) << 4));
          const uint4 wb = *reinterpret_cast<const uint4*>(base + (rj0 + 8) * 128 + ((g ^ rj0) << 4));
          const uint4 wc = *reinterpret_cast<const uint4*>(base + rj1 * 128 + ((g ^ rj1) << 4));
          const uint4 wd = *reinterpret_cast<const uint4*>(base + (rj1 + 8) * 128 + ((g ^ rj1) << 4));
          const uint32_t a4[4] = {wa.x, wa.y, wa.z, wa.w}, b4[4] = {wb.x, wb.y, wb.z, wb.w};
          const uint32_t c4[4] = {wc.x, wc.y, wc.z, wc.w}, d4[4] = {wd.x, wd.y, wd.z, wd.w};
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const uint32_t a[4] = {__byte_perm(a4[x], b4[x], 0x5410), __byte_perm(a4[x], b4[x], 0x7632),
                                   __byte_perm(c4[x], d4[x], 0x5410), __byte_perm(c4[x], d4[x], 0x7632)};
            mma16816<false>(o[4 * hf + x], a, pb[2 * ks], pb[2 * ks + 1]);
          }
        }
      }
    }
    __syncwarp();   // the stage and the P tile are free for the next iteration
  }
  if (failed) {
    if (lane == 0) atomicOr(&g_attn_status, 1);
    // copies issued but not consumed: chunks done .. min(my_n, done + kStages - 1) - 1 (the refill of
    // iteration `done` was issued before its wait ran out)
    for (int i = done; i < my_n && i < done + S::kStages; ++i) sm100::mbar_wait(&full[i % S::kStages], (i / S::kStages) & 1);
  }
  __syncthreads();

  // ---- merge the four warps through shared memory (the rings are no longer needed) ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 4);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 8);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 16);
  }
  float* mO = reinterpret_cast<float*>(smem);   // [4][8][D]
  float* mML = mO + 4 * 8 * D;                  // [4][8][2]
  {
    // e4m3: the lane holds dimensions 16 g .. 16 g + 15; bf16: 8 g .. 8 g + 7 of each half of the head
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      float* r0 = mO + (warp * 8 + 2 * j) * D + (FP8 ? 16 * g + 4 * x : 64 * (x >> 1) + 8 * g + 4 * (x & 1));
      float* r1 = r0 + D;
      *reinterpret_cast<float4*>(r0) = make_float4(o[2 * x][0], o[2 * x][2], o[2 * x + 1][0], o[2 * x + 1][2]);
      *reinterpret_cast<float4*>(r1) = make_float4(o[2 * x][1], o[2 * x][3], o[2 * x + 1][1], o[2 * x + 1][3]);
    }
    if (g == 0) {
      mML[(warp * 8 + 2 * j) * 2] = m[0];
      mML[(warp * 8 + 2 * j) * 2 + 1] = l[0];
      mML[(warp * 8 + 2 * j + 1) * 2] = m[1];
      mML[(warp * 8 + 2 * j + 1) * 2 + 1] = l[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int row = idx / D, col = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, mML[(w * 8 + row) * 2]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mML[(w * 8 + row) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
      acc += mO[(w * 8 + row) * D + col] * f;
      ll += mML[(w * 8 + row) * 2 + 1] * f;
    }
    const int h = h0 + row;
    if (p.nsplit == 1) {
      const float inv = ll > 0.f ? (FP8 ? vsc : 1.f) / ll : 0.f;
      p.out[(static_cast<size_t>(q_row) * p.Hq + h) * D + col] = __float2bfloat16(acc * inv);
    } else {
      const size_t pi = (static_cast<size_t>(b) * p.Hq + h) * p.nsplit + split;
      p.part_o[pi * D + col] = ll > 0.f ? acc * ((FP8 ? vsc : 1.f) / ll) : 0.f;
      if (col == 0) {
        p.part_ml[pi * 2] = mm;
        p.part_ml[pi * 2 + 1] = ll;
      }
    }
  }
}

// merge split partials: grid (B, Hq), block D
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ cu_seqlens_q, __nv_bfloat16* __restrict__ out, int Hq,
                                    int D, int nsplit) {
  tgi::pdl_wait();
  tgi::pdl_trigger();
  const int b = blockIdx.x, h = blockIdx.y;
  if (cu_seqlens_q[b + 1] == cu_seqlens_q[b]) return;
  const size_t base = (static_cast<size_t>(b) * Hq + h) * nsplit;
  float mm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) {
    const float l = part_ml[(base + s) * 2 + 1];
    if (l > 0.f) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  }
  for (int col = threadIdx.x; col < D; col += blockDim.x) {
    float acc = 0.f, wsum = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float l = part_ml[(base + s) * 2 + 1];
      if (l > 0.f) {
        const float w = l * exp2f(part_ml[(base + s) * 2] - mm);
        acc += part_o[(base + s) * D + col] * w;
        wsum += w;
      }
    }
    out[(static_cast<size_t>(cu_seqlens_q[b]) * Hq + h) * D + col] = __float2bfloat16(wsum > 0.f ? acc / wsum : 0.f);
  }
}

// `TGI_B200_ATTN_V3=0` keeps e4m3 decode on decode_kernel_v2
bool decode_v3_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("TGI_B200_ATTN_V3");
    return v == nullptr || std::strcmp(v, "0") != 0;
  }();
  return on;
}

// Tensor map of one e4m3 K or V page pool viewed as [slots, Hkv * 128] bytes, box 16 slots x 128 bytes.
// Pools live as long as the model, so the maps are cached by (device, pointer, geometry).
const CUtensorMap* page_map(const void* cache, const Params& p, int eb) {
  struct Key {
    int dev;
    const void* ptr;
    int blocks, bs, hkv, eb;
    bool operator==(const Key& o) const {
      return dev == o.dev && ptr == o.ptr && blocks == o.blocks && bs == o.bs && hkv == o.hkv && eb == o.eb;
    }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      return std::hash<const void*>()(k.ptr) ^ (static_cast<size_t>(k.blocks) * 1000003u) ^
             (static_cast<size_t>(k.bs) << 20) ^ (static_cast<size_t>(k.hkv) << 28) ^ static_cast<size_t>(k.dev);
    }
  };
  static std::mutex mu;
  static std::unordered_map<Key, CUtensorMap*, Hash> maps;
  Key key{0, cache, p.num_blocks, p.block_size, p.Hkv, eb};
  if (cudaGetDevice(&key.dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  auto it = maps.find(key);
  if (it != maps.end()) return it->second;
  void* raw = nullptr;
  if (posix_memalign(&raw, 64, sizeof(CUtensorMap)) != 0) return nullptr;
  CUtensorMap* m = static_cast<CUtensorMap*>(raw);
  const uint64_t pitch = static_cast<uint64_t>(p.Hkv) * 128 * eb;   // bytes per slot: Hkv heads of 128 elements
  const uint64_t slots = static_cast<uint64_t>(p.num_blocks) * p.block_size;
  if (tgi::make_map_2d(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, cache, slots, pitch, pitch, 16, 128,
                       CU_TENSOR_MAP_SWIZZLE_128B) != 0) {
    free(raw);
    return nullptr;
  }
  maps.emplace(key, m);
  return m;
}

template <class S>
int launch_v3_cfg(const Params& p, int B, cudaStream_t stream) {
  auto k = decode_kernel_v3<S>;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes) != cudaSuccess) return -2;
    set = true;
  }
  const CUtensorMap* tk = page_map(p.k_cache, p, S::EB);
  const CUtensorMap* tv = page_map(p.v_cache, p, S::EB);
  if (tk == nullptr || tv == nullptr) return -14;
  dim3 grid(p.Hkv, B, p.nsplit);
  tgi::launch(k, dim3(grid), dim3(128), S::kBytes, stream, p, *tk, *tv);
  if (p.nsplit > 1) {
    dim3 g2(B, p.Hq);
    tgi::launch(decode_merge_kernel, dim3(g2), dim3(128), 0, stream, p.part_o, p.part_ml, p.cu_seqlens_q, p.out, p.Hq,
                128, p.nsplit);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// chunk size and ring depth of decode_kernel_v3; `TGI_B200_ATTN_V3_CFG` = "<tokens>x<stages>" picks another
// of the compiled shapes
template <bool FP8>
int launch_v3(const Params& p, int B, cudaStream_t stream) {
  static const int cfg = [] {
    const char* v = std::getenv("TGI_B200_ATTN_V3_CFG");
    if (v == nullptr) return 0;
    if (std::strcmp(v, "32x2") == 0) return 322;
    if (std::strcmp(v, "32x3") == 0) return 323;
    if (std::strcmp(v, "16x4") == 0) return 164;
    if (std::strcmp(v, "16x2") == 0) return 162;
    return 163;
  }();
  if (!FP8) {
    // bf16 pages: a 16-token chunk is 8 KB, so two stages leave room for 3 CTAs (12 warps) per SM
    if (cfg == 163) return launch_v3_cfg<DecodeV3<16, 3, false>>(p, B, stream);
    return launch_v3_cfg<DecodeV3<16, 2, false>>(p, B, stream);
  }
  if (cfg == 0) {
    // measured: 32-token chunks are 1-3 % faster on grids of many waves (256 sequences x 8 KV heads), 16-token
    // chunks with 16 warps per SM clearly faster on small grids (256 x 1 KV head: 29 us against 36 us)
    if (static_cast<long long>(B) * p.Hkv * p.nsplit >= 1536) return launch_v3_cfg<DecodeV3<32, 2>>(p, B, stream);
    return launch_v3_cfg<DecodeV3<16, 3>>(p, B, stream);
  }
  switch (cfg) {
    case 322: return launch_v3_cfg<DecodeV3<32, 2>>(p, B, stream);
    case 323: return launch_v3_cfg<DecodeV3<32, 3>>(p, B, stream);
    case 164: return launch_v3_cfg<DecodeV3<16, 4>>(p, B, stream);
    default: return launch_v3_cfg<DecodeV3<16, 3>>(p, B, stream);   // 4 CTAs (16 warps) per SM
  }
}

// tcgen05 / TMEM prefill kernel (attention_prefill_sm100.cu): head size 128, pages of 16 tokens
extern "C" int tgi_prefill_attention_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                                        const int* cu_seqlens_q, const int* kv_lens, const float* k_scale,
                                        const float* v_scale, void* out, int B, int max_q, int max_blocks, int num_blocks,
                                        int Hq, int Hkv, float scale, float softcap, int window, int fp8_kv,
                                        const int* horizon, int* status, cudaStream_t stream);

bool prefill_tc_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("TGI_B200_PREFILL_TC");
    return v == nullptr || std::strcmp(v, "0") != 0;
  }();
  return on;
}

template <int D, bool FP8>
int launch(const Params& p, int B, int max_q, cudaStream_t stream) {
  using S = Smem<D, FP8>;
  const int smem = S::kBytes;
  if (max_q > 1 && D == 128 && p.block_size == 16 && B <= 65535 && prefill_tc_enabled()) {
    int* status = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_attn_status) != cudaSuccess) return -2;
    return tgi_prefill_attention_tc(p.q, p.k_cache, p.v_cache, p.block_tables, p.cu_seqlens_q, p.kv_lens, p.k_scale,
                                    p.v_scale, p.out, B, max_q, p.max_blocks, p.num_blocks, p.Hq, p.Hkv, p.scale, p.softcap,
                                    p.window, FP8 ? 1 : 0, p.horizon, status, stream);
  }
  if (max_q > 1) {
    auto k = prefill_kernel<D, FP8>;
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
      set = true;
    }
    dim3 grid((max_q + kTile - 1) / kTile, p.Hq, B);
    tgi::launch(k, dim3(grid), dim3(128), smem, stream, p);
  } else if (B > 65535) {
    return -15;   // the batch index is grid dimension y
  } else if (D == 128 && p.Hq / p.Hkv <= 8 && p.block_size >= 16 && decode_v3_enabled()) {
    return launch_v3<FP8>(p, B, stream);
  } else {
    auto k = decode_kernel_v2<D, FP8>;
    constexpr int dsmem = DecodeSmem<D, FP8>::kBytes;
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, dsmem) != cudaSuccess) return -2;
      set = true;
    }
    const int G = p.Hq / p.Hkv;
    dim3 grid(p.Hkv * ((G + 15) / 16), B, p.nsplit);
    tgi::launch(k, dim3(grid), dim3(128), dsmem, stream, p);
    if (p.nsplit > 1) {
      dim3 g2(B, p.Hq);
      tgi::launch(decode_merge_kernel, dim3(g2), dim3(D < 128 ? D : 128), 0, stream, p.part_o, p.part_ml, p.cu_seqlens_q, p.out, p.Hq, D,
                                                                p.nsplit);
    }
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace

extern "C" {

// Split count for a decode launch.  A grid that already has one CTA per SM is not split: measured on B200,
// the partial results and the merge kernel cost more than the better balance gains (256 sequences x 1 KV
// head, 1280 tokens: 25 us unsplit, 29 us in two splits, 34 us in four).  Smaller grids are split into
// enough CTAs for two waves, bounded by the tiles a sequence of max_kv tokens has.
int tgi_attn_decode_splits(int B, int Hkv, int G, int max_kv, int sm_count) {
  const int ctas = B * Hkv * ((G + 15) / 16);
  if (ctas >= sm_count) {
    // long sequences on a grid of fewer than four CTAs per SM: split down to 2048 tokens per CTA
    if (ctas >= 4 * sm_count || max_kv < 4096) return 1;
    int want = (4 * sm_count + ctas - 1) / ctas;
    if (want > max_kv / 2048) want = max_kv / 2048;
    return want < 1 ? 1 : want;
  }
  int want = (2 * sm_count + ctas - 1) / ctas;
  const int tiles = (max_kv + kTile - 1) / kTile;
  if (want > tiles) want = tiles;
  if (want > 64) want = 64;
  return want < 1 ? 1 : want;
}

// Error word of the decode kernels (bit 0: a page copy did not arrive within the wait bound); `reset`
// clears it after reading.  Synchronises with the device.
int tgi_attn_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int));
  }
  return v;
}

// `horizon` (optional, prefill only): per query row the last KV position it may attend to; null = causal
int tgi_paged_attention_ex(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                           const int* cu_seqlens_q, const int* kv_lens, const float* k_scale, const float* v_scale,
                           void* out, float* part_o, float* part_ml, int B, int max_q, int max_blocks, int block_size,
                           int num_blocks, int Hq, int Hkv, int D, float scale, float softcap, int window, int nsplit,
                           int fp8_kv, const int* horizon, cudaStream_t stream);

int tgi_paged_attention(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                        const int* cu_seqlens_q, const int* kv_lens, const float* k_scale, const float* v_scale,
                        void* out, float* part_o, float* part_ml, int B, int max_q, int max_blocks, int block_size,
                        int num_blocks, int Hq, int Hkv, int D, float scale, float softcap, int window, int nsplit,
                        int fp8_kv, cudaStream_t stream) {
  return tgi_paged_attention_ex(q, k_cache, v_cache, block_tables, cu_seqlens_q, kv_lens, k_scale, v_scale, out, part_o,
                                part_ml, B, max_q, max_blocks, block_size, num_blocks, Hq, Hkv, D, scale, softcap, window,
                                nsplit, fp8_kv, nullptr, stream);
}

int tgi_paged_attention_ex(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                           const int* cu_seqlens_q, const int* kv_lens, const float* k_scale, const float* v_scale,
                           void* out, float* part_o, float* part_ml, int B, int max_q, int max_blocks, int block_size,
                           int num_blocks, int Hq, int Hkv, int D, float scale, float softcap, int window, int nsplit,
                           int fp8_kv, const int* horizon, cudaStream_t stream) {
  if (B <= 0 || max_q <= 0) return 0;
  if (Hq % Hkv != 0) return -10;
  Params p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.block_tables = block_tables;
  p.cu_seqlens_q = cu_seqlens_q;
  p.kv_lens = kv_lens;
  p.k_scale = k_scale;
  p.v_scale = v_scale;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.horizon = max_q > 1 ? horizon : nullptr;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  if (block_size <= 0 || (block_size & (block_size - 1)) != 0) return -13;   // pages hold a power-of-two token count
  p.bs_shift = 0;
  while ((1 << p.bs_shift) < block_size) ++p.bs_shift;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.num_blocks = num_blocks;
  p.scale = scale;
  p.softcap = softcap;
  p.window = window;
  p.nsplit = (max_q > 1 || nsplit < 1) ? 1 : nsplit;
  if (p.nsplit > 1 && (part_o == nullptr || part_ml == nullptr)) return -11;
  switch (D) {
    case 64: return fp8_kv ? launch<64, true>(p, B, max_q, stream) : launch<64, false>(p, B, max_q, stream);
    case 128: return fp8_kv ? launch<128, true>(p, B, max_q, stream) : launch<128, false>(p, B, max_q, stream);
    case 256: return fp8_kv ? launch<256, true>(p, B, max_q, stream) : launch<256, false>(p, B, max_q, stream);
    default: return -12;
  }
}

}  // extern "C"

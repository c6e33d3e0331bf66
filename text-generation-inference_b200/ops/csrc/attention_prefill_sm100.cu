// Paged causal prefill attention on the 5th-generation tensor cores (sm_100a): head size 128, pages of 16
// tokens, bf16 or e4m3 KV pages, ragged batches with a cached prefix (chunked prefill), GQA, sliding
// window, soft-capping and per-row horizons.
//
// Replaces, in the reference, flashinfer `BatchPrefillWithPagedKVCache` / FA2 `varlen_fwd`
// (layers/attention/cuda.py:244-296, layers/attention/flashinfer.py:58-128).
//
// A CTA owns 128 query rows of one head and walks the KV range in tiles of 128 tokens:
//   S  = Q K^T     tcgen05.mma, M 128 (rows) x N 128 (keys) x K 128 (head dim), accumulator in TMEM
//   P  = softmax   eight warps, two threads per row (64 keys each; they exchange the row maximum through shared
//                  memory and keep separate partial sums): TMEM -> registers, online max / sum, P as 16-bit values
//                  into a shared-memory tile in the swizzled operand layout.  Tiles that a row sees completely
//                  (below the diagonal, inside the window and the sequence) take a path without per-element masks
//   PV = P V       tcgen05.mma, M 128 x N 128 (head dim) x K 128 (keys); V is taken as the MN-major operand, i.e.
//                  exactly as the page boxes land in shared memory (rows = tokens, 128 bytes = 64 head elements)
//   O  = O a + PV  eight warps keep the running output in registers (64 columns per thread), rescale it by the
//                  row's a = exp2(m_old - m_new) and add the tile's product read back from TMEM
// K and V pages are fetched with TMA boxes of one page (16 tokens x 128 bytes) straight from the page pool, no
// per-lane address arithmetic.  e4m3 pages are widened to fp16 (exact) on their way into the operand tiles by the
// eight output warps, which are idle most of a tile (64 bytes per thread), and the MMAs then run in fp16 (Q is
// converted once); bf16 pages feed bf16 MMAs directly.
// The S accumulator and the PV accumulator are double-buffered in TMEM (4 x 128 columns), so the tensor core
// computes S of the next tile while the softmax warps work on the current one.
// Every wait is bounded; a wait that runs out sets the status word, the CTA drains and frees its TMEM.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "launch.cuh"
#include "sm100.cuh"
#include "tensor_map.cuh"

using namespace sm100;

namespace {

constexpr int kD = 128;            // head size
constexpr int kRows = 128;         // query rows per CTA
constexpr int kKeys = 128;         // KV tokens per tile
constexpr int kPage = 16;          // tokens per page
constexpr int kThreads = 640;            // 20 warps: K producer, MMA, V producer, spare, 8 softmax, 8 output
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kSlab = kRows * 128;             // bytes of one [128 rows x 128 bytes] swizzled slab
constexpr int kTileBytes = 2 * kSlab;          // a 128 x 128 tile of 16-bit values: two slabs (32 KB)

struct PrefillParams {
  const __nv_bfloat16* q;       // [T, Hq, 128]
  const int* block_tables;      // [B, max_blocks]
  const int* cu_seqlens_q;      // [B + 1]
  const int* kv_lens;           // [B]
  const float* k_scale;         // [Hkv] or null (e4m3 pages)
  const float* v_scale;
  __nv_bfloat16* out;           // [T, Hq, 128]
  const int* horizon;           // optional [T]
  int max_blocks, Hq, Hkv, num_blocks;
  float scale, softcap;
  int window;
  int* status;
};

__device__ __forceinline__ void report(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// MN-major operand with the 128-byte swizzle (rows = K index, 128 bytes = 64 MN elements per row; groups of 8
// rows 1024 bytes apart; the next 64 MN elements `lbo` bytes further): the layout TMA leaves a [tokens x head]
// tile in.  Canonical form: cute/atom/mma_traits_sm100.hpp, make_umma_desc<Major::MN>.
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// instruction descriptor: D fp32, A K-major, B K-major or MN-major, fmt 0 = f16, 1 = bf16
__device__ __forceinline__ constexpr uint32_t idesc16(uint32_t fmt, bool b_mn) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (0u << 15) | ((b_mn ? 1u : 0u) << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ uint32_t swz_chunk(int row, int chunk) { return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4)); }
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
  tmem_ld_32x32b_x32(addr, r);
  tmem_ld_wait(r);
}

// 2^x on the FMA pipe, for x <= 0: the special-function unit does 16 ex2 per cycle and SM and is the busiest
// unit of a tile (16 K exponentials), so every kPolyEvery-th probability is computed this way instead.  Round x to
// the nearest integer with the 1.5 * 2^23 trick, evaluate a cubic for 2^f on [-0.5, 0.5] (relative error 1.4e-4,
// well under the 16-bit rounding of P) and add the integer to the exponent field.
constexpr int kPolyEvery = 4;
__device__ __forceinline__ float poly_exp2(float x) {
  x = fmaxf(x, -125.f);
  const float t = x + 12582912.f;
  const float f = x - (t - 12582912.f);
  float r = fmaf(0.05502927f, f, 0.24225698f);
  r = fmaf(r, f, 0.69325305f);
  r = fmaf(r, f, 0.99995134f);
  return __int_as_float(__float_as_int(r) + (__float_as_int(t) << 23));
}
__device__ __forceinline__ float fast_tanh(float y) {      // 1 - 2 / (1 + e^(2y)); saturates cleanly at +-1
  return 1.f - __fdividef(2.f, 1.f + fast_exp2(y * (2.f * kLog2e)));
}
// How a softmax thread reads its scores.  Key i of a 32-key group is visible when i - lo lies in [0, range]
// (one unsigned compare); with soft-capping a raw score x becomes cap_out * tanh(x * cap_in), already in log2 units,
// otherwise it is scaled by scale_log2 (> 0) — after the maximum in the first pass, inside the FMA in the second.
struct ScoreArgs {
  float scale_log2, cap_in, cap_out;
  int lo;
  unsigned range;
};
template <bool MASK, bool CAP>
__device__ __forceinline__ float group_max(const uint32_t (&v)[32], float mx, const ScoreArgs& a) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float x = __uint_as_float(v[i]);
    if (CAP) x = a.cap_out * fast_tanh(x * a.cap_in);
    if (MASK) x = static_cast<unsigned>(i - a.lo) <= a.range ? x : -INFINITY;
    mx = fmaxf(mx, x);
  }
  return mx;
}
// Probabilities of a 32-key group as sixteen packed 16-bit pairs (fp16 next to fp16 V tiles, bf16 otherwise);
// returns their sum.  m is the row maximum in log2 units.
template <bool MASK, bool CAP, bool F16>
__device__ __forceinline__ float group_prob(const uint32_t (&v)[32], uint32_t (&packed)[16], float m, const ScoreArgs& a) {
  float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float pr[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float x = __uint_as_float(v[i + e]);
      if (CAP) pr[e] = fast_exp2(a.cap_out * fast_tanh(x * a.cap_in) - m);
      else if (kPolyEvery > 0 && (i + e) % kPolyEvery == 1) pr[e] = poly_exp2(fmaf(x, a.scale_log2, -m));
      else pr[e] = fast_exp2(fmaf(x, a.scale_log2, -m));
      if (MASK) pr[e] = static_cast<unsigned>(i + e - a.lo) <= a.range ? pr[e] : 0.f;
    }
    rs0 += pr[0];
    rs1 += pr[1];
    if (F16) {
      const __half2 hh = __floats2half2_rn(pr[0], pr[1]);
      packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&hh);
    } else {
      const __nv_bfloat162 bb = __floats2bfloat162_rn(pr[0], pr[1]);
      packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&bb);
    }
  }
  return rs0 + rs1;
}

// Shared memory (bytes):  Q 32 K | K: bf16 2 x 32 K, e4m3 raw 2 x 16 K + converted 32 K | V: same | P 32 K | barriers
template <bool FP8>
struct Layout {
  static constexpr int kQ = 0;
  static constexpr int kK = kTileBytes;
  static constexpr int kKBytes = 2 * kTileBytes;                  // 64 KB in both modes
  static constexpr int kV = kK + kKBytes;
  static constexpr int kP = kV + kKBytes;
  // two P tiles: the softmax of tile j + 1 writes one while the PV product of tile j still reads the other.  The
  // final partial row sums (float [2][128]) are written into the P tile that the last product does not read.
  static constexpr int kBars = kP + 2 * kTileBytes;               // 224 KB
  static constexpr int kAlpha = kBars + 256;                      // float [2][128]
  static constexpr int kRowMax = kAlpha + 2 * 128 * 4;            // float [2][128]: row maxima of the two halves
  static constexpr int kAbort = kRowMax + 2 * 128 * 4;            // int [4][2]: a softmax thread of the lane quarter gave up
  // no slack for aligning the base: the kernel checks that the dynamic shared memory starts on a 1024-byte
  // boundary (it does when the kernel has no static shared memory) and reports an error otherwise
  static constexpr int kTotal = kAbort + 64;
  static_assert(kTotal <= 227 * 1024, "shared memory of a CTA");
  // e4m3: raw stage s at kK + s * 16 K, converted tile at kK + 32 K
  static constexpr int kRawStage = kKeys * 128;
};

template <bool FP8>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const PrefillParams p) {
  using L = Layout<FP8>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0u) {       // uniform over the CTA, before anything is allocated
    if (threadIdx.x == 0) report(p.status, kErrProducerWait);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* k_full = bars;            // [2] TMA landed (bf16: operand tile, e4m3: raw tile)
  uint64_t* k_free = bars + 2;        // [2] bf16: MMA done with the stage; e4m3: converters done with the raw stage
  uint64_t* v_full = bars + 4;        // [2]
  uint64_t* v_free = bars + 6;        // [2]
  uint64_t* kc_ready = bars + 8;      // e4m3: converted K tile written      (1 buffer)
  uint64_t* kc_free = bars + 9;       // e4m3: MMA done with the converted K tile
  uint64_t* vc_ready = bars + 10;
  uint64_t* vc_free = bars + 11;
  uint64_t* s_full = bars + 12;       // [2] S accumulator written
  uint64_t* s_free = bars + 14;       // [2] softmax warps have read it
  uint64_t* p_ready = bars + 24;      // [2] P tile written
  uint64_t* p_free = bars + 26;       // [2] PV MMA done with the P tile
  uint64_t* pv_full = bars + 18;      // [2] PV accumulator written
  uint64_t* pv_free = bars + 20;      // [2] O warps have read it
  uint64_t* l_ready = bars + 22;      // final row sums written
  uint64_t* q_ready = bars + 23;      // Q tile staged (18 warps)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 28);
  float* s_alpha = reinterpret_cast<float*>(smem + L::kAlpha);
  float* s_rowmax = reinterpret_cast<float*>(smem + L::kRowMax);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + L::kAbort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int qt = gridDim.x - 1 - blockIdx.x;       // long tiles (late rows) first: the grid drains on short ones
  const int q_begin = p.cu_seqlens_q[b], n = p.cu_seqlens_q[b + 1] - q_begin;
  if (qt * kRows >= n) return;                       // uniform over the CTA, before anything is allocated
  const int Lkv = p.kv_lens[b];
  const int kvh = h / (p.Hq / p.Hkv);
  const int row_base = qt * kRows;
  const int pos_first = Lkv - n + row_base;
  const int pos_last = min(Lkv - 1, pos_first + kRows - 1);
  int t_lo = 0;
  if (p.window > 0) t_lo = max(0, pos_first - p.window + 1) / kKeys * kKeys;
  const int t_hi = p.horizon != nullptr ? Lkv : pos_last + 1;
  const int ntiles = (t_hi - t_lo + kKeys - 1) / kKeys;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_free[i], FP8 ? 8 : 1);      // e4m3: the eight converting warps
      mbar_init(&v_free[i], FP8 ? 8 : 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 8);
      mbar_init(&pv_full[i], 1);
      mbar_init(&pv_free[i], 8);
    }
    mbar_init(kc_ready, 8);
    mbar_init(kc_free, 1);
    mbar_init(vc_ready, 8);
    mbar_init(vc_free, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&p_ready[i], 8);
      mbar_init(&p_free[i], 1);
    }
    mbar_init(l_ready, 8);
    mbar_init(q_ready, 18);
    for (int i = 0; i < 8; ++i) s_abort[i] = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tgi::pdl_wait();
  tgi::pdl_trigger();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tS = tmem_base, tPV = tmem_base + 256;

  // ---------------- TMA producers: one box per page and 64-element half of the head ----------------
  // A thread's TMA copies issue one after the other (about 400 cycles each, measured), so a tile's boxes are
  // spread over lanes: lane l copies page l % 8, half (l / 8) % 2.  Lanes 0..7 read the tile's block ids with one
  // coalesced load; lane 0 does the waits and posts the expected byte count.  Warp 0 brings K and warp 2 brings
  // V, each on its own ring of two stages.
  auto produce = [&](bool do_k, bool do_v) {
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      const int s = j & 1;
      const int t0 = t_lo + j * kKeys;
      int blk = 0;
      if (lane < kKeys / kPage) {
        const int blk_i = (t0 >> 4) + lane;
        if (blk_i < p.max_blocks) blk = p.block_tables[static_cast<size_t>(b) * p.max_blocks + blk_i];
        blk = min(max(blk, 0), p.num_blocks - 1);        // pages past the sequence are masked later
      }
      blk = __shfl_sync(0xffffffffu, blk, lane & 7);
      if (lane == 0) {
        if (do_k) {
          if (j >= 2) ok = mbar_wait(&k_free[s], ((j >> 1) - 1) & 1);
          if (ok) mbar_arrive_expect_tx(&k_full[s], FP8 ? L::kRawStage : kTileBytes);
        }
        if (do_v && ok) {
          if (j >= 2) ok = mbar_wait(&v_free[s], ((j >> 1) - 1) & 1);
          if (ok) mbar_arrive_expect_tx(&v_full[s], FP8 ? L::kRawStage : kTileBytes);
        }
        if (!ok) report(p.status, kErrProducerWait);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      const int pg = lane & 7;
      if (FP8) {
        // one 128-byte-wide box covers the whole head
        if (lane < 8) {
          if (do_k) tma_load_2d(smem + L::kK + s * L::kRawStage + pg * (kPage * 128), &tmK, &k_full[s], kvh * kD, blk * kPage);
          if (do_v) tma_load_2d(smem + L::kV + s * L::kRawStage + pg * (kPage * 128), &tmV, &v_full[s], kvh * kD, blk * kPage);
        }
      } else if (lane < 16) {
        const int hf = lane >> 3;
        if (do_k)
          tma_load_2d(smem + L::kK + s * kTileBytes + hf * kSlab + pg * (kPage * 128), &tmK, &k_full[s], kvh * kD + hf * 64, blk * kPage);
        if (do_v)
          tma_load_2d(smem + L::kV + s * kTileBytes + hf * kSlab + pg * (kPage * 128), &tmV, &v_full[s], kvh * kD + hf * 64, blk * kPage);
      }
      __syncwarp();
    }
  };
  if (warp != 0 && warp != 2) {
    // ---- Q tile -> shared, swizzled operand layout (two slabs of 64 head elements); fp16 for e4m3 pages.  The
    // two producer warps are already fetching K and V meanwhile; the MMA issuer waits for q_ready. ----
    const int st = (warp == 1 ? 0 : warp - 2) * 32 + lane;       // 0..575
    for (int c = st; c < kRows * 16; c += 18 * 32) {
      const int row = c >> 4, ch = c & 15;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row_base + row < n)
        v = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(q_begin + row_base + row) * p.Hq + h) * kD + ch * 8);
      if (FP8) {
        const __nv_bfloat162* bv = reinterpret_cast<const __nv_bfloat162*>(&v);
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(bv[i]);
          const __half2 hh = __floats2half2_rn(f.x, f.y);
          o[i] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        v = make_uint4(o[0], o[1], o[2], o[3]);
      }
      *reinterpret_cast<uint4*>(smem + L::kQ + (ch >> 3) * kSlab + swz_chunk(row, ch & 7)) = v;
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) mbar_arrive(q_ready);
  }
  if (warp == 0) {
    produce(true, false);
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t id_qk = idesc16(FP8 ? 0u : 1u, false);
      constexpr uint32_t id_pv = idesc16(FP8 ? 0u : 1u, true);
      const uint32_t q_addr = smem_u32(smem + L::kQ);
      const uint32_t p_base = smem_u32(smem + L::kP);
      bool ok = true;
      auto issue_qk = [&](int j) {
        const int s = j & 1;
        if (j >= 2 && !mbar_wait(&s_free[s], ((j >> 1) - 1) & 1)) { report(p.status, kErrMmaWaitAccum); return false; }
        uint32_t k_addr;
        if (FP8) {
          if (!mbar_wait(kc_ready, j & 1)) { report(p.status, kErrMmaWaitFull); return false; }
          k_addr = smem_u32(smem + L::kK + 2 * L::kRawStage);
        } else {
          if (!mbar_wait(&k_full[s], (j >> 1) & 1)) { report(p.status, kErrMmaWaitFull); return false; }
          k_addr = smem_u32(smem + L::kK + s * kTileBytes);
        }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {      // 16 head elements (32 bytes) per MMA; 4 per slab
          const uint64_t da = make_desc_sw128(q_addr + (k >> 2) * kSlab) + ((k & 3) * 32 >> 4);
          const uint64_t db = make_desc_sw128(k_addr + (k >> 2) * kSlab) + ((k & 3) * 32 >> 4);
          mma_f16(tS + s * 128, da, db, id_qk, k > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[s]);
        tc_commit(FP8 ? kc_free : &k_free[s]);
        return true;
      };
      auto issue_pv = [&](int j) {
        const int s = j & 1;
        if (j >= 2 && !mbar_wait(&pv_free[s], ((j >> 1) - 1) & 1)) { report(p.status, kErrMmaWaitAccum); return false; }
        uint32_t v_addr;
        if (FP8) {
          if (!mbar_wait(vc_ready, j & 1)) { report(p.status, kErrMmaWaitFull); return false; }
          v_addr = smem_u32(smem + L::kV + 2 * L::kRawStage);
        } else {
          if (!mbar_wait(&v_full[s], (j >> 1) & 1)) { report(p.status, kErrMmaWaitFull); return false; }
          v_addr = smem_u32(smem + L::kV + s * kTileBytes);
        }
        if (!mbar_wait(&p_ready[s], (j >> 1) & 1)) { report(p.status, kErrMmaWaitFull); return false; }
        const uint32_t p_addr = p_base + s * kTileBytes;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {      // 16 keys per MMA: 32 bytes along a P row, two 8-row groups of V
          const uint64_t da = make_desc_sw128(p_addr + (k >> 2) * kSlab) + ((k & 3) * 32 >> 4);
          const uint64_t db = make_desc_mn_sw128(v_addr + k * 2048, kSlab);
          mma_f16(tPV + s * 128, da, db, id_pv, k > 0 ? 1u : 0u);
        }
        tc_commit(&pv_full[s]);
        tc_commit(&p_free[s]);
        tc_commit(FP8 ? vc_free : &v_free[s]);
        return true;
      };
      ok = mbar_wait(q_ready, 0);
      if (!ok) report(p.status, kErrMmaWaitFull);
      ok = ok && issue_qk(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) ok = issue_qk(j + 1);      // S of the next tile overlaps the softmax of this one
        if (ok) ok = issue_pv(j);
      }
    }
  } else if (warp == 2) {
    produce(false, true);
  } else if (warp == 3) {
    // spare
  } else if (warp < 12) {
    // ---------------- softmax: two threads per query row, 64 keys each ----------------
    const int quarter = warp & 3;
    const int hf = (warp - 4) >> 2;              // which 64 keys of the tile
    const int r = quarter * 32 + lane;
    const int pos = pos_first + r;
    int hz = pos;
    if (p.horizon != nullptr && row_base + r < n) hz = max(pos, min(p.horizon[q_begin + row_base + r], Lkv - 1));
    const float ks = (FP8 && p.k_scale != nullptr) ? p.k_scale[kvh] : 1.f;
    const float raw_scale = p.scale * ks;
    const float scale_log2 = raw_scale * kLog2e;
    const uint32_t lane_addr = tS + (static_cast<uint32_t>(quarter * 32) << 16) + hf * 64;
    const bool cap = p.softcap > 0.f;
    ScoreArgs sa;
    sa.scale_log2 = scale_log2;
    sa.cap_in = cap ? raw_scale / p.softcap : 0.f;
    sa.cap_out = p.softcap * kLog2e;
    // visible keys of this row: [t_min, t_max]
    const int t_max = min(hz, Lkv - 1);
    const int t_min = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    float m = -INFINITY, l = 0.f;
    // The two threads of a row meet at a named barrier once per tile, so they must leave the loop together: a
    // thread whose wait ran out raises the quarter's flag of the NEXT barrier's parity and keeps walking to that
    // barrier; everyone reads the flag right after the barrier, where all 64 threads see the same value.
    bool fail = false;
    for (int j = 0; j < ntiles; ++j) {
      const int s = j & 1;
      const int t0 = t_lo + j * kKeys + hf * 64;    // first key of this thread's half
      if (!fail && !mbar_wait(&s_full[s], (j >> 1) & 1)) { report(p.status, kErrEpilogueWait); fail = true; }
      if (fail) s_abort[quarter * 2 + s] = 1;
      tc_fence_after();
      // a warp whose rows all see their whole half of the tile (below the diagonal / horizon, inside the window and
      // the sequence) takes the code without masks; the choice is per warp so that no path diverges
      const bool plain = __all_sync(0xffffffffu, !cap && t0 >= t_min && t0 + 63 <= t_max);
      sa.range = t_max >= t_min ? static_cast<unsigned>(t_max - t_min) : 0u;
      // pass 1: maximum of the (masked) scores of this half
      float mx = -INFINITY;
      uint32_t v[32];            // after pass 1 it still holds the second 32-key group: pass 2 starts with that one
      if (!fail) {
#pragma unroll 1
        for (int c = 0; c < 64; c += 32) {
          tmem_ld32(lane_addr + s * 128 + c, v);
          sa.lo = t_max >= t_min ? t_min - (t0 + c) : (1 << 30);
          if (plain) mx = group_max<false, false>(v, mx, sa);
          else if (!cap) mx = group_max<true, false>(v, mx, sa);
          else mx = group_max<true, true>(v, mx, sa);
        }
      }
      if (!cap) mx *= scale_log2;     // scale_log2 > 0
      // the two halves of a row agree on the maximum through shared memory (one named barrier per lane quarter)
      s_rowmax[hf * 128 + r] = mx;
      asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
      if (s_abort[quarter * 2 + s] != 0) break;
      const float m_new = fmaxf(m, fmaxf(mx, s_rowmax[(hf ^ 1) * 128 + r]));
      const float alpha = m_new == -INFINITY ? 0.f : fast_exp2(m - m_new);
      // the P tile and this parity's alpha slot are free once the PV product two tiles back was consumed
      if (j >= 2 && !mbar_wait(&p_free[s], ((j >> 1) - 1) & 1)) { report(p.status, kErrEpilogueWait); fail = true; }
      if (!fail && j >= 2 && !mbar_wait(&pv_free[s], ((j >> 1) - 1) & 1)) { report(p.status, kErrEpilogueWait); fail = true; }
      if (fail) continue;
      // pass 2: probabilities as 16-bit values into the P operand tile, partial row sum.  A row without a visible
      // key so far has m_new = -inf: every key of it is masked, so the value never reaches P.
      float rs = 0.f;
#pragma unroll 1
      for (int c = 32; c >= 0; c -= 32) {
        if (c == 0) tmem_ld32(lane_addr + s * 128, v);
        uint32_t packed[16];
        sa.lo = t_max >= t_min ? t_min - (t0 + c) : (1 << 30);
        if (plain) rs += group_prob<false, false, FP8>(v, packed, m_new, sa);
        else if (!cap) rs += group_prob<true, false, FP8>(v, packed, m_new, sa);
        else rs += group_prob<true, true, FP8>(v, packed, m_new, sa);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {      // four 16-byte chunks (8 keys each) of this 32-key group
          const int ch = hf * 8 + (c >> 3) + q4;   // chunk index among the row's 16
          *reinterpret_cast<uint4*>(smem + L::kP + s * kTileBytes + (ch >> 3) * kSlab + swz_chunk(r, ch & 7)) =
              make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
        }
      }
      l = l * alpha + rs;
      m = m_new;
      if (hf == 0) s_alpha[s * 128 + r] = alpha;
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_free[s]);
        mbar_arrive(&p_ready[s]);
      }
    }
    // partial row sums into the P tile the last product does not read; that tile was last read by the product of
    // the tile before the last one
    if (!fail && ntiles >= 2 && !mbar_wait(&p_free[ntiles & 1], ((ntiles - 2) >> 1) & 1)) {
      report(p.status, kErrEpilogueWait);
      fail = true;
    }
    if (!fail) {
      reinterpret_cast<float*>(smem + L::kP + (ntiles & 1) * kTileBytes)[hf * 128 + r] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(l_ready);
    }
  } else {
    // ---------------- running output: 64 columns per thread ----------------
    const int quarter = warp & 3;
    const int half = (warp - 12) >> 2;           // columns [64 * half, 64 * half + 64)
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = tPV + (static_cast<uint32_t>(quarter * 32) << 16) + half * 64;
    float o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.f;
    bool ok = true;
    // e4m3 pages: raw [128 tokens x 128 bytes] stage -> fp16 operand tile (one buffer per K and V), 64 bytes per
    // thread.  Tile i's K may be written once the S product of tile i - 1 has left the buffer, its V once the PV
    // product of tile i - 1 has.
    const int ot = (warp - 12) * 32 + lane;      // 0..255: token row ot / 2, bytes [64 * (ot % 2), +64)
    auto convert = [&](int kv, int i) {
      const int st = i & 1;
      uint64_t* full = kv == 0 ? &k_full[st] : &v_full[st];
      uint64_t* raw_free = kv == 0 ? &k_free[st] : &v_free[st];
      if (!mbar_wait(full, (i >> 1) & 1)) { report(p.status, kErrMmaWaitFull); return false; }
      if (i >= 1 && !mbar_wait(kv == 0 ? kc_free : vc_free, (i - 1) & 1)) { report(p.status, kErrMmaWaitAccum); return false; }
      const int row = ot >> 1, hb = ot & 1;
      const uint8_t* raw = smem + (kv == 0 ? L::kK : L::kV) + st * L::kRawStage + row * 128 + hb * 64;
      uint8_t* dst = smem + (kv == 0 ? L::kK : L::kV) + 2 * L::kRawStage + hb * kSlab;   // 64 bytes -> one 128-byte slab row
#pragma unroll
      for (int c16 = 0; c16 < 4; ++c16) {          // 16 e4m3 bytes -> two 16-byte chunks of fp16
        const uint4 q = *reinterpret_cast<const uint4*>(raw + c16 * 16);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t cv[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(cv[2 * e]) : "h"(static_cast<unsigned short>(w[e] & 0xFFFFu)));
          asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(cv[2 * e + 1]) : "h"(static_cast<unsigned short>(w[e] >> 16)));
        }
        *reinterpret_cast<uint4*>(dst + swz_chunk(row, 2 * c16)) = make_uint4(cv[0], cv[1], cv[2], cv[3]);
        *reinterpret_cast<uint4*>(dst + swz_chunk(row, 2 * c16 + 1)) = make_uint4(cv[4], cv[5], cv[6], cv[7]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(kv == 0 ? kc_ready : vc_ready);
        mbar_arrive(raw_free);
      }
      return true;
    };
    if (FP8) {
      ok = convert(0, 0);
      if (ok && ntiles > 1) ok = convert(0, 1);
      if (ok) ok = convert(1, 0);
    }
    for (int j = 0; j < ntiles && ok; ++j) {
      const int s = j & 1;
      if (FP8 && j + 2 < ntiles && !convert(0, j + 2)) { ok = false; break; }
      if (!mbar_wait(&pv_full[s], (j >> 1) & 1)) { report(p.status, kErrEpilogueWait); ok = false; break; }
      tc_fence_after();
      const float alpha = s_alpha[s * 128 + r];
#pragma unroll
      for (int c = 0; c < 64; c += 16) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(lane_addr + s * 128 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) o[c + i] = fmaf(o[c + i], alpha, __uint_as_float(v[i]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pv_free[s]);
      if (FP8 && j + 1 < ntiles && !convert(1, j + 1)) { ok = false; break; }
    }
    if (ok && mbar_wait(l_ready, 0)) {
      const float vs = (FP8 && p.v_scale != nullptr) ? p.v_scale[kvh] : 1.f;
      const float* s_rowsum = reinterpret_cast<const float*>(smem + L::kP + (ntiles & 1) * kTileBytes);
      const float l = s_rowsum[r] + s_rowsum[128 + r];
      const float inv = l > 0.f ? vs / l : 0.f;
      if (row_base + r < n) {
        __nv_bfloat16* dst = p.out + (static_cast<size_t>(q_begin + row_base + r) * p.Hq + h) * kD + half * 64;
#pragma unroll
        for (int c = 0; c < 64; c += 8) {
          __nv_bfloat162 w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) w[e] = __floats2bfloat162_rn(o[c + 2 * e] * inv, o[c + 2 * e + 1] * inv);
          *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<uint4*>(w);
        }
      }
    } else if (ok) {
      report(p.status, kErrEpilogueWait);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

template <bool FP8>
int launch_prefill(const PrefillParams& p, const void* k_cache, const void* v_cache, int B, int max_q, cudaStream_t stream) {
  using L = Layout<FP8>;
  CUtensorMap tmK, tmV;
  const uint64_t rows = static_cast<uint64_t>(p.num_blocks) * kPage;
  const uint64_t cols = static_cast<uint64_t>(p.Hkv) * kD;
  int rc;
  if (FP8) {
    rc = tgi::make_map_2d(&tmK, CU_TENSOR_MAP_DATA_TYPE_UINT8, k_cache, rows, cols, cols, kPage, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = tgi::make_map_2d(&tmV, CU_TENSOR_MAP_DATA_TYPE_UINT8, v_cache, rows, cols, cols, kPage, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
  } else {
    rc = tgi::make_map_2d(&tmK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, k_cache, rows, cols, cols * 2, kPage, 64,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = tgi::make_map_2d(&tmV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, v_cache, rows, cols, cols * 2, kPage, 64,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc) return rc;
  auto kern = prefill_tc_kernel<FP8>;
  static std::atomic<unsigned long long> attr_set{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -2;
  const unsigned long long bit = 1ull << (dev & 63);
  if (!(attr_set.load(std::memory_order_acquire) & bit)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return -2;
    attr_set.fetch_or(bit, std::memory_order_release);
  }
  const dim3 grid((max_q + kRows - 1) / kRows, p.Hq, B);
  const cudaError_t err = tgi::launch(kern, grid, dim3(kThreads), static_cast<size_t>(L::kTotal), stream, tmK, tmV, p);
  return err == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace

extern "C" {

// Prefill attention for head size 128 and pages of 16 tokens.  q / out [T, Hq, 128] bf16; caches
// [num_blocks, 16, Hkv, 128] bf16 or e4m3 (fp8_kv); the other arguments as in tgi_paged_attention_ex.
int tgi_prefill_attention_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                             const int* cu_seqlens_q, const int* kv_lens, const float* k_scale, const float* v_scale,
                             void* out, int B, int max_q, int max_blocks, int num_blocks, int Hq, int Hkv, float scale,
                             float softcap, int window, int fp8_kv, const int* horizon, int* status, cudaStream_t stream) {
  if (B <= 0 || max_q <= 0) return 0;
  if (Hq % Hkv != 0 || B > 65535 || Hq > 65535) return -10;
  PrefillParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.block_tables = block_tables;
  p.cu_seqlens_q = cu_seqlens_q;
  p.kv_lens = kv_lens;
  p.k_scale = k_scale;
  p.v_scale = v_scale;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.horizon = horizon;
  p.max_blocks = max_blocks;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.num_blocks = num_blocks;
  p.scale = scale;
  p.softcap = softcap;
  p.window = window;
  p.status = status;
  return fp8_kv ? launch_prefill<true>(p, k_cache, v_cache, B, max_q, stream)
                : launch_prefill<false>(p, k_cache, v_cache, B, max_q, stream);
}

}  // extern "C"

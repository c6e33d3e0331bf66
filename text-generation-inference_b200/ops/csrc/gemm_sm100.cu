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
// Tile: 256 tokens x 128 weight rows (two 128-lane MMAs sharing the weight tile) when M > 128,
// 128 tokens x 256 weight rows otherwise.  TMEM lanes run over TOKENS and columns over weight
// rows.  That orientation is what makes the fp8 promotion cheap: the combined block scale
// a_scale[m, kb] * w_scale[slab, kb] is one scalar per thread and K block, kept in a register,
// instead of a vector that every lane would have to fetch from shared memory (measured: broadcast
// loads of a per-column scale vector cost 2x the FMAs they feed, because shared memory delivers
// 128 B/clk per SM however many lanes read the same word).  It also gives every thread one
// contiguous 256-byte row of C to store.
//
// Scheduling: persistent stream-K.  The work is the flattened list of (output tile, K block)
// units; the grid has one CTA per SM and CTA c owns the contiguous unit range
// [c*U/G, (c+1)*U/G), so every SM streams the same number of weight bytes whatever the shape (a
// tensor-parallel shard with 10 weight slabs keeps all 148 SMs busy).  A tile whose K range is
// shared by several CTAs is finished through an fp32 workspace: every contributor stores its
// partial tile, the last one to arrive (atomic counter per tile) sums them in CTA order, so the
// result does not depend on arrival order.
//
// Roles inside a CTA (384 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner
// (warps 2, 3 idle; the four give their registers away with setmaxnreg), warps 4..11 = promotion /
// epilogue.  All waits are bounded (sm100.cuh): on expiry the kernel records an error code in
// `status`, drains its outstanding TMA loads, frees TMEM and returns.
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int kThreads = 384;
constexpr int kEpiWarps = 8;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kCols = 128;                 // accumulator columns per epilogue thread
constexpr int kTileElems = 256 * 128;      // outputs per tile in both configurations
constexpr int kBufCols = 256;              // TMEM columns per accumulator buffer (two buffers)

template <int MH, int TN>
struct TileCfg {
  static_assert(MH * TN == 256, "an accumulator buffer is 256 TMEM columns");
  static constexpr int TM = MH * 128;                  // tokens per tile
  static constexpr int kXBytes = TM * 128;             // one 128-byte K row per token
  static constexpr int kWBytes = TN * 128;
  static constexpr int kStageBytes = kXBytes + kWBytes;   // 48 KB
};

__device__ __forceinline__ void report(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

template <int REGS>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}
template <int REGS>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}
__device__ __forceinline__ void epi_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
}

// fp32 accumulators of one epilogue thread.  Plain scalar FMAs with the scale in a register:
// measured on B200, this form overlaps completely with the TMEM loads (about 400 clk per K block
// for 8 warps x 128 columns), while packed fma.rn.f32x2 through inline asm was 3x slower because of
// the register-pair moves it needs around every instruction.
struct AccPairs {
  float v[kCols];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int j = 0; j < kCols; ++j) v[j] = 0.f;
  }
  __device__ __forceinline__ float get(int j) const { return v[j]; }
  __device__ __forceinline__ void set_pair(int j2, float lo, float hi) {
    v[2 * j2] = lo;
    v[2 * j2 + 1] = hi;
  }
  // v[2*j2], v[2*j2+1] += x * s
  __device__ __forceinline__ void fma_pair(int j2, uint32_t x0, uint32_t x1, float s) {
    v[2 * j2] = fmaf(__uint_as_float(x0), s, v[2 * j2]);
    v[2 * j2 + 1] = fmaf(__uint_as_float(x1), s, v[2 * j2 + 1]);
  }
};

struct Sched {
  int n_tiles, m_tiles, KB, grid;
  long long units;
  __device__ __forceinline__ long long begin(int c) const { return units * c / grid; }
  __device__ __forceinline__ int owner(long long u) const {   // CTA whose range contains unit u
    int c = static_cast<int>(u * grid / units);
    while (c + 1 < grid && begin(c + 1) <= u) ++c;
    while (c > 0 && begin(c) > u) --c;
    return c;
  }
};

// Walks the (tile, K block) units of a CTA without a division per step (a 64-bit divide per K
// block in each role cost more than the K block's tensor-core time).
struct UnitIter {
  int tn, tm, kb;
  __device__ __forceinline__ UnitIter(long long u, const Sched& s) {
    const int tile = static_cast<int>(u / s.KB);
    kb = static_cast<int>(u - static_cast<long long>(tile) * s.KB);
    tn = tile / s.m_tiles;
    tm = tile - tn * s.m_tiles;
  }
  __device__ __forceinline__ void next(const Sched& s) {
    if (++kb == s.KB) {
      kb = 0;
      if (++tm == s.m_tiles) {
        tm = 0;
        ++tn;
      }
    }
  }
};

// ------------------------------------------------------------------------------------------------
// xs_t: activation scales, K-block major: xs_t[kb * xs_pitch + m]   (fp32, pitch multiple of 4)
// wscale: weight scales [ceil(N/128), K/128] row-major
// ws: 2 partial-tile slots per CTA; counters: one int per output tile (self-resetting)
// ------------------------------------------------------------------------------------------------
template <int MH, int TN, int STAGES, bool FP8>
__global__ void __launch_bounds__(kThreads, 1)
gemm_streamk_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    const __grid_constant__ CUtensorMap tmS, const float* __restrict__ wscale,
                    __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                    float* __restrict__ ws, int* __restrict__ counters, int* __restrict__ status) {
  using Cfg = TileCfg<MH, TN>;
  constexpr int TM = Cfg::TM;
  constexpr int BK = FP8 ? 128 : 64;            // elements per 128-byte row
  constexpr int SC_STAGES = STAGES + 2;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sc_ring = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes);   // [SC_STAGES][TM] (fp8 only)
  uint64_t* full = reinterpret_cast<uint64_t*>(sc_ring + (FP8 ? SC_STAGES * TM : 0));
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;      // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  int* flag = reinterpret_cast<int*>(tmem_holder + 1);
  {
    // self-check: the carve-up above must fit in the dynamic shared memory of the launch
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if (reinterpret_cast<uint8_t*>(flag + 1) - smem_raw > static_cast<ptrdiff_t>(dyn_bytes)) {
      report(status, kErrSmemLayout);
      return;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Sched sch;
  sch.n_tiles = (N + TN - 1) / TN;
  sch.m_tiles = (M + TM - 1) / TM;
  sch.KB = (K + BK - 1) / BK;
  sch.grid = gridDim.x;
  sch.units = static_cast<long long>(sch.n_tiles) * sch.m_tiles * sch.KB;
  const long long u0 = sch.begin(blockIdx.x), u1 = sch.begin(blockIdx.x + 1);
  const int nunits = static_cast<int>(u1 - u0);
  constexpr uint32_t kTmemCols = 2 * kBufCols;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], kEpiWarps);
    }
    fence_barrier_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmX);
    if (FP8) prefetch_tensormap(&tmS);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp < 4) {
    reg_dec<40>();
    if (warp == 0) {
      // ---------------- TMA producer ----------------
      if (elect_one()) {
        const uint64_t pol_w = policy_evict_first();   // weights are streamed once
        const uint64_t pol_x = policy_evict_last();    // token tiles are re-read by every weight slab
        int issued = 0;
        bool ok = true;
        UnitIter ui(u0, sch);
        for (int it = 0; it < nunits && ok; ++it, ui.next(sch)) {
          const int kb = ui.kb;
          const int n0 = ui.tn * TN, m0 = ui.tm * TM;
          const int s = it % STAGES;
          if (it >= STAGES) ok = mbar_wait(&empty[s], ((it / STAGES) - 1) & 1);
          if (!ok) { report(status, kErrProducerWait); break; }
          uint8_t* st = smem + s * Cfg::kStageBytes;
          mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes + (FP8 ? TM * 4 : 0));
#pragma unroll
          for (int h = 0; h < MH; ++h) tma_load_2d_hint(st + h * 16384, &tmX, &full[s], kb * BK, m0 + h * 128, pol_x);
#pragma unroll
          for (int h = 0; h < TN / 128; ++h)
            tma_load_2d_hint(st + Cfg::kXBytes + h * 16384, &tmW, &full[s], kb * BK, n0 + h * 128, pol_w);
          if (FP8) tma_load_2d(sc_ring + (it % SC_STAGES) * TM, &tmS, &full[s], m0, kb);
          issued = it + 1;
        }
        if (!ok) {
          // drain: wait (bounded) for the loads already issued so none lands after the CTA exits
          for (int it = max(0, issued - STAGES); it < issued; ++it)
            mbar_wait(&full[it % STAGES], (it / STAGES) & 1, 1u << 12);
        }
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer ----------------
      if (elect_one()) {
        constexpr uint32_t idesc = FP8 ? make_idesc(128, TN, 0, 0) : make_idesc(128, TN, 1, 1);
        int seg = 0;        // accumulator uses so far (fp8: one per K block, bf16: one per tile segment)
        UnitIter ui(u0, sch);
        for (int it = 0; it < nunits; ++it, ui.next(sch)) {
          const int kb = ui.kb;
          const bool seg_start = (it == 0) || kb == 0;
          const bool seg_end = (it == nunits - 1) || kb == sch.KB - 1;
          const int use = FP8 ? it : seg;
          const int b = use & 1;
          if ((FP8 || seg_start) && use >= 2 && !mbar_wait(&tmem_empty[b], ((use >> 1) - 1) & 1)) {
            report(status, kErrMmaWaitAccum);
            break;
          }
          const int s = it % STAGES;
          if (!mbar_wait(&full[s], (it / STAGES) & 1)) { report(status, kErrMmaWaitFull); break; }
          tc_fence_after();
          const uint32_t x_addr = smem_u32(smem + s * Cfg::kStageBytes);
          const uint64_t dw = make_desc_sw128(x_addr + Cfg::kXBytes);
#pragma unroll
          for (int h = 0; h < MH; ++h) {
            const uint64_t dx = make_desc_sw128(x_addr + h * 16384);
#pragma unroll
            for (int k = 0; k < 4; ++k) {   // 4 MMAs of 32 bytes of K each per 128-byte row
              const uint32_t accumulate = FP8 ? (k > 0) : (!seg_start || k > 0);
              const uint32_t d = tmem_base + b * kBufCols + h * TN;
              if (FP8) mma_f8f6f4(d, dx + (k * 32 >> 4), dw + (k * 32 >> 4), idesc, accumulate);
              else mma_f16(d, dx + (k * 32 >> 4), dw + (k * 32 >> 4), idesc, accumulate);
            }
          }
          tc_commit(&empty[s]);
          if (FP8 || seg_end) tc_commit(&tmem_full[b]);
          if (seg_end) ++seg;
        }
      }
    }
  } else {
    // ---------------- promotion + epilogue ----------------
    reg_inc<232>();
    const int ew = warp - 4;
    const int quarter = warp & 3;
    const int g = ew >> 2;                                   // token half (MH == 2) or column half (MH == 1)
    const int col_base = g * kCols;                          // first TMEM column of this thread inside a buffer
    const int m_local = (MH == 2 ? g * 128 : 0) + quarter * 32 + lane;
    const int n_off = (MH == 2 ? 0 : g * kCols);
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + col_base;
    const int et = threadIdx.x - 128;                        // index among the epilogue threads
    AccPairs acc;
    int seg = 0;
    int seg_kb0 = 0;
    bool ok = true;
    UnitIter ui(u0, sch);
    for (int it = 0; it < nunits && ok; ++it, ui.next(sch)) {
      const int kb = ui.kb;
      const int tile = ui.tn * sch.m_tiles + ui.tm;
      const int n0 = ui.tn * TN, m0 = ui.tm * TM;
      const bool seg_start = (it == 0) || kb == 0;
      const bool seg_end = (it == nunits - 1) || kb == sch.KB - 1;
      // a warp whose 32 token rows are all padding has nothing to promote (warp-uniform)
      const bool warp_active = (m0 + m_local - lane) < M && (n0 + n_off) < N;
      if (seg_start) {
        seg_kb0 = kb;
        acc.zero();
      }
      if (FP8) {
        const int b = it & 1;
        ok = mbar_wait(&tmem_full[b], (it >> 1) & 1);
        if (!ok) { report(status, kErrEpilogueWait); break; }
        tc_fence_after();
        if (warp_active) {
          const float s = sc_ring[(it % SC_STAGES) * TM + m_local] *
                          __ldg(&wscale[static_cast<size_t>((n0 + n_off) >> 7) * sch.KB + kb]);
          uint32_t v[2][32];
          tmem_ld_32x32b_x32(lane_addr + b * kBufCols, v[0]);
#pragma unroll
          for (int c = 0; c < kCols; c += 32) {
            uint32_t(&cur)[32] = v[(c >> 5) & 1];
            tmem_ld_wait(cur);
            if (c + 32 < kCols) tmem_ld_32x32b_x32(lane_addr + b * kBufCols + c + 32, v[((c >> 5) + 1) & 1]);
#pragma unroll
            for (int j = 0; j < 32; j += 2) acc.fma_pair((c + j) >> 1, cur[j], cur[j + 1], s);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[b]);
      } else if (seg_end) {
        const int b = seg & 1;
        ok = mbar_wait(&tmem_full[b], (seg >> 1) & 1);
        if (!ok) { report(status, kErrEpilogueWait); break; }
        tc_fence_after();
        if (warp_active) {
#pragma unroll
          for (int c = 0; c < kCols; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(lane_addr + b * kBufCols + c, v);
            tmem_ld_wait(v);
#pragma unroll
            for (int j = 0; j < 32; j += 2)
              acc.set_pair((c + j) >> 1, __uint_as_float(v[j]), __uint_as_float(v[j + 1]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[b]);
      }
      if (!seg_end) continue;
      ++seg;
      // ---- finish the segment [seg_kb0, kb] of `tile` ----
      const int m = m0 + m_local;
      const int nb = n0 + n_off;                              // first output column of this thread
      const bool whole = seg_kb0 == 0 && kb == sch.KB - 1;
      bool store = whole;
      if (!whole) {
        // partial tile: store to this CTA's slot (head slot if the tile is the CTA's first, else tail slot)
        const int first_tile = static_cast<int>(u0 / sch.KB);
        const int slot = blockIdx.x * 2 + (tile == first_tile ? 0 : 1);
        float4* wsp = reinterpret_cast<float4*>(ws + static_cast<size_t>(slot) * kTileElems) + et;
#pragma unroll
        for (int j = 0; j < kCols; j += 4)
          wsp[(j >> 2) * kEpiThreads] = make_float4(acc.get(j), acc.get(j + 1), acc.get(j + 2), acc.get(j + 3));
        __threadfence();
        epi_barrier();
        const long long t_lo = static_cast<long long>(tile) * sch.KB, t_hi = t_lo + sch.KB - 1;
        const int c_lo = sch.owner(t_lo), c_hi = sch.owner(t_hi);
        if (et == 0) {
          const int old = atomicAdd(&counters[tile], 1);
          const int last = (old == c_hi - c_lo);
          if (last) counters[tile] = 0;   // self-cleaning: ready for the next launch / graph replay
          *flag = last;
        }
        epi_barrier();
        const bool last = *flag != 0;
        epi_barrier();                    // everyone has read the flag before it can be rewritten
        if (last) {
          __threadfence();
          acc.zero();
          for (int c = c_lo; c <= c_hi; ++c) {
            const int c_first_tile = static_cast<int>(sch.begin(c) / sch.KB);
            const int cslot = c * 2 + (tile == c_first_tile ? 0 : 1);
            const float4* src = reinterpret_cast<const float4*>(ws + static_cast<size_t>(cslot) * kTileElems) + et;
#pragma unroll
            for (int j = 0; j < kCols; j += 4) {
              const float4 t = __ldcg(src + (j >> 2) * kEpiThreads);
              acc.set_pair(j >> 1, acc.get(j) + t.x, acc.get(j + 1) + t.y);
              acc.set_pair((j >> 1) + 1, acc.get(j + 2) + t.z, acc.get(j + 3) + t.w);
            }
          }
          store = true;
        }
      }
      if (store && m < M && nb < N) {
        __nv_bfloat16* crow = C + static_cast<size_t>(m) * N + nb;
        const bool vec_ok = (N % 8 == 0);
#pragma unroll
        for (int j = 0; j < kCols; j += 8) {
          if (nb + j >= N) break;
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            f[e] = acc.get(j + e);
            if (bias != nullptr && nb + j + e < N) f[e] += __bfloat162float(bias[nb + j + e]);
          }
          if (vec_ok && nb + j + 8 <= N) {
            __nv_bfloat162 o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
            *reinterpret_cast<uint4*>(crow + j) = *reinterpret_cast<uint4*>(o);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (nb + j + e < N) crow[j + e] = __float2bfloat16(f[e]);
          }
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

// 2-D row-major tensor [rows, cols]; box = [box_rows, box_cols]
int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* ptr, uint64_t rows, uint64_t cols,
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

template <int MH, int TN, int STAGES, bool FP8>
int launch(const void* X, const float* xs_t, int xs_pitch, const void* W, const float* wscale, void* C,
           const void* bias, int M, int N, int K, int max_ctas, float* ws, int* counters, int* status,
           cudaStream_t stream) {
  using Cfg = TileCfg<MH, TN>;
  constexpr int BK = FP8 ? 128 : 64;
  CUtensorMap tmW, tmX, tmS;
  const CUtensorMapDataType dt = FP8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint64_t pitch = static_cast<uint64_t>(K) * (FP8 ? 1 : 2);
  // both operands are fetched in boxes of 128 rows x 128 bytes (one swizzle atom wide)
  int rc = make_map_2d(&tmW, dt, W, N, K, pitch, 128, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_map_2d(&tmX, dt, X, M, K, pitch, 128, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  if (FP8) {
    rc = make_map_2d(&tmS, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, xs_t, K / 128, M, static_cast<uint64_t>(xs_pitch) * 4, 1,
                     Cfg::TM, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  } else {
    tmS = tmX;
  }
  // stages + (fp8) activation-scale ring [STAGES+2][TM] + alignment slack + barriers
  const size_t smem = STAGES * Cfg::kStageBytes + (FP8 ? (STAGES + 2) * Cfg::TM * 4 : 0) + 1024 + 256;
  auto kern = gemm_streamk_kernel<MH, TN, STAGES, FP8>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return -2;
    attr_set = true;
  }
  const long long units =
      static_cast<long long>((N + TN - 1) / TN) * ((M + Cfg::TM - 1) / Cfg::TM) * ((K + BK - 1) / BK);
  int grid = max_ctas;
  if (grid > units) grid = static_cast<int>(units);
  if (grid < 1) grid = 1;
  kern<<<grid, kThreads, smem, stream>>>(tmW, tmX, tmS, wscale, static_cast<__nv_bfloat16*>(C),
                                         static_cast<const __nv_bfloat16*>(bias), M, N, K, ws, counters, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace

extern "C" {

// Floats of stream-K workspace a launch with `ctas` CTAs may touch (two partial-tile slots per CTA).
long long tgi_gemm_workspace_floats(int M, int ctas) {
  (void)M;
  return 2LL * ctas * kTileElems;
}

// Output tiles of a problem (the counters array needs one int per tile).
int tgi_gemm_num_tiles(int M, int N) {
  if (M > 128) return ((N + 127) / 128) * ((M + 255) / 256);
  return ((N + 255) / 256) * ((M + 127) / 128);
}

int tgi_gemm_bf16(const void* X, const void* W, void* C, const void* bias, int M, int N, int K, int max_ctas,
                  float* ws, int* counters, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0) return -10;  // TMA row pitch must be a multiple of 16 bytes
  if (M > 128)
    return launch<2, 128, 4, false>(X, nullptr, 0, W, nullptr, C, bias, M, N, K, max_ctas, ws, counters, status, stream);
  return launch<1, 256, 4, false>(X, nullptr, 0, W, nullptr, C, bias, M, N, K, max_ctas, ws, counters, status, stream);
}

int tgi_gemm_fp8_block(const void* X, const float* xs_t, int xs_pitch, const void* W, const float* wscale, void* C,
                       const void* bias, int M, int N, int K, int max_ctas, float* ws, int* counters, int* status,
                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 128 != 0 || xs_pitch % 4 != 0) return -10;
  if (M > 128)
    return launch<2, 128, 4, true>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, max_ctas, ws, counters, status, stream);
  return launch<1, 256, 4, true>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, max_ctas, ws, counters, status, stream);
}

}  // extern "C"

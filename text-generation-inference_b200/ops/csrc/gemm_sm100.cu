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
// Tile: 128 tokens x 256 weight rows per CTA for M <= 128.  For M > 128 two CTAs of a cluster work
// as a pair (`cta_group::2`) on 256 tokens x 256 weight rows: each CTA loads its own 128 tokens and
// one half of the 256 weight rows, the even CTA issues MMAs of 256 x 256 that read the weight
// halves from both CTAs' shared memory, and each CTA finds the accumulator rows of its tokens in
// its own TMEM.  Per K block a CTA then moves 32 KB through L2 -> shared memory for 128 x 256
// outputs where a single CTA needs 48 KB (the activation tile is not fetched once per 128 weight
// rows any more).  Measured on B200 against the 256 x 128 single-CTA tile, which is kept for
// launches that cannot form pairs: bf16 4096 x 8192 x 8192 1050 against 874 TFLOP/s; block-scaled
// fp8 256 x 57344 x 8192 180 against 187 us (there the hand-over of every K block's products to
// the promotion warps, not operand traffic, sets the pace).
//
// TMEM lanes run over TOKENS and columns over weight rows.  That orientation is what makes the
// fp8 promotion cheap: the combined block scale a_scale[m, kb] * w_scale[slab, kb] is one scalar per thread and K block, kept in a register,
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
// partial tile and counts its arrival; after its own main loop each contributor waits (bounded)
// for the others and reduces its own slice of the tile's columns, summing the partials in CTA
// order, so the work of the fix-up is spread over the contributors and the result does not depend
// on arrival order.  Problems with fewer tiles than SMs use whole tiles or a few aligned K splits
// instead when that is cheaper (see launch()).
//
// Roles inside a CTA (384 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner
// (warps 2, 3 idle; the four give their registers away with setmaxnreg), warps 4..11 = promotion /
// epilogue.  All waits are bounded (sm100.cuh): on expiry the kernel records an error code in
// `status`, drains its outstanding TMA loads, frees TMEM and returns.
//
// Barriers of a pair: `full[s]` lives in the even CTA and counts the bytes of both CTAs' loads
// (every load names it through its cluster address; only the even CTA's producer posts the
// expected byte count); `empty[s]` and `tmem_full[b]` exist in both CTAs and are signalled in both
// by one multicast `tcgen05.commit`; `tmem_empty[b]` lives in the even CTA and collects the
// arrivals of both CTAs' epilogue warps.  Both CTAs meet at a cluster barrier after barrier
// initialisation and before TMEM is freed, on every path, error paths included.
#include <atomic>

#include "launch.cuh"
#include "tensor_map.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int kThreads = 384;
constexpr int kEpiWarps = 8;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kCols = 128;                 // accumulator columns per epilogue thread
constexpr int kTileElems = 256 * 128;      // outputs per tile in both configurations
constexpr int kBufCols = 256;              // TMEM columns per accumulator buffer (two buffers)

template <int MH, int TN, bool PAIR, bool FP8 = false, bool MX = false>
struct TileCfg {
  static_assert(MH * TN == 256, "an accumulator buffer is 256 TMEM columns");
  static_assert(!PAIR || MH == 1, "a pair runs the 128 x 256 per-CTA configuration");
  static constexpr int CM = MH * 128;                  // tokens per CTA
  static constexpr int TM = PAIR ? 256 : CM;           // tokens per tile (a pair's tile spans both CTAs)
  static constexpr int WROWS = PAIR ? TN / 2 : TN;     // weight rows this CTA loads
  static constexpr int kXBytes = CM * 128;             // one 128-byte K row per token
  static constexpr int kWBytes = WROWS * 128;
  static constexpr int kStageBytes = kXBytes + kWBytes;   // 48 KB, 32 KB in a pair
  // Block-scaled fp8 hands every K block's products to the epilogue.  With two token halves (MH == 2) each
  // half of an accumulator buffer is signalled on its own full / drained barrier pair, so the promotion of
  // half 0 starts while the MMAs of half 1 still run.  (Splitting the 256 columns of the MH == 1 buffers
  // into 2 or 4 separately signalled column groups was measured slower: 180 -> 195 -> 222 us on
  // 256 x 57344 x 8192, the extra commits and waits of the single issuing thread cost more than they hide.)
  static constexpr int SUB = (FP8 && !MX && MH == 2) ? 2 : 1;
};

// Optional destination of the output rows in peer memory (tensor-parallel row-parallel GEMMs): row m
// of the partial product belongs to rank m / rows_per and is stored, as bf16, straight into that
// rank's heap at slot [this rank][m % rows_per], so the reduce-scatter transport happens in the
// epilogue while other tiles are still being computed.  When the whole grid has stored everything,
// the last CTA raises this rank's flag in every owner's heap (value: a call counter kept in device
// memory, so CUDA-graph replays work).  world == 0 means "store to C as usual".
struct PushArgs {
  unsigned char* heap[8];
  long long off_slots;      // byte offset of the slots [world][rows_per][N] bf16 in every heap
  long long off_flags;      // byte offset of uint32 flags [8] in every heap, indexed by source rank
  int rank, world, rows_per;
  int* done_ctas;           // local counter of CTAs that finished their stores (self-resetting)
  unsigned int* epoch;      // local call counter
};

constexpr int kMaxGrid = 160;              // upper bound of the grid size (one CTA per SM)
int g_last_grid = 0;                       // CTAs of the most recent launch (diagnostics)
constexpr int kSplitPolls = 1 << 20;       // polls of a split-tile counter before giving up (about 0.1 s)

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

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
// MX: block-scaled fp8 on `tcgen05.mma.kind::mxf8f6f4.block_scale`.  Operands, scales and scheduling are those of the
// fp8 mode, but the two block scales of a K block (powers of two, a precondition of this mode) are handed to the
// tensor core as E8M0 scale factors in TMEM, so a tile accumulates over all of its K blocks in TMEM like a bf16
// tile and the per-K-block promotion disappears.  TMEM: one accumulator buffer (columns 0..255) and a ring of
// scale-factor columns (16 per stage, from column 256): A's rows use 4 columns per 128 tokens, B's 4 per 128
// weight rows.  Four epilogue warps (one per lane quarter) write a stage's scale factors when its copy has landed.
template <int MH, int TN, int STAGES, bool FP8, bool PAIR, bool MX = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_streamk_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    const __grid_constant__ CUtensorMap tmS, const float* __restrict__ wscale,
                    __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                    float* __restrict__ ws, int* __restrict__ counters, int* __restrict__ status,
                    const __grid_constant__ PushArgs push) {
  using Cfg = TileCfg<MH, TN, PAIR, FP8, MX>;
  static_assert(!MX || FP8, "the block-scaled mode is built for fp8 operands");
  constexpr bool PROMOTE = FP8 && !MX;          // per-K-block promotion in the epilogue warps
  // first element of output row m: in C, or in the owner's peer-memory slot of this rank
  auto out_row = [&](int m) -> __nv_bfloat16* {
    if (push.world == 0) return C + static_cast<size_t>(m) * N;
    const int owner = m / push.rows_per;
    const int lr = m - owner * push.rows_per;
    return reinterpret_cast<__nv_bfloat16*>(push.heap[owner] + push.off_slots) +
           (static_cast<size_t>(push.rank) * push.rows_per + lr) * N;
  };
  constexpr int TM = Cfg::TM;
  constexpr int CM = Cfg::CM;
  constexpr int BK = FP8 ? 128 : 64;            // elements per 128-byte row
  // position in the pair: the even CTA leads (issues the MMAs, owns `full` and `tmem_empty`)
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  constexpr int SC_STAGES = STAGES + 2;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sc_ring = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes);   // [SC_STAGES][CM] (fp8 only)
  uint64_t* full = reinterpret_cast<uint64_t*>(sc_ring + (FP8 ? SC_STAGES * CM : 0));
  uint64_t* empty = full + STAGES;
  constexpr int SUB = Cfg::SUB;              // separately signalled parts of an accumulator buffer
  uint64_t* tmem_full = empty + STAGES;      // [2 * SUB]
  uint64_t* tmem_empty = tmem_full + 8;      // [2 * SUB]
  uint64_t* sf_ready = tmem_empty + 8;       // [2 * STAGES] scale factors of a K block written to TMEM (MX)
  uint64_t* sc_full = sf_ready + 16;         // [SC_STAGES] activation scales of a K block landed (MX)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(sc_full + 8);
  int* flag = reinterpret_cast<int*>(tmem_holder + 1);
  int* cslots = flag + 1;                    // [kMaxGrid] workspace slot of every contributor of a split tile
  {
    // self-check: the carve-up above must fit in the dynamic shared memory of the launch
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if (reinterpret_cast<uint8_t*>(cslots + kMaxGrid) - smem_raw > static_cast<ptrdiff_t>(dyn_bytes)) {
      report(status, kErrSmemLayout);
      if (PAIR) {   // uniform over the cluster (same launch parameters): meet the peer at both cluster barriers
        cluster_sync();
        cluster_sync();
      }
      return;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // every barrier of a pair is signalled at least in part from the other CTA: short re-evaluation interval
  auto wait = [](uint64_t* bar, uint32_t parity) { return PAIR ? mbar_wait_fast(bar, parity) : mbar_wait(bar, parity); };
  Sched sch;
  sch.n_tiles = (N + TN - 1) / TN;
  sch.m_tiles = (M + TM - 1) / TM;
  sch.KB = (K + BK - 1) / BK;
  sch.grid = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  sch.units = static_cast<long long>(sch.n_tiles) * sch.m_tiles * sch.KB;
  const long long u0 = sch.begin(worker), u1 = sch.begin(worker + 1);
  const int nunits = static_cast<int>(u1 - u0);
  constexpr uint32_t kTmemCols = 2 * kBufCols;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      if (MX) {
        mbar_init(&sf_ready[s], PAIR ? 8 : 4);            // four writer warps per CTA
        mbar_init(&sf_ready[STAGES + s], PAIR ? 8 : 4);
      }
    }
    if (MX)
      for (int s = 0; s < SC_STAGES; ++s) mbar_init(&sc_full[s], 1);
    for (int b = 0; b < 2 * SUB; ++b) {
      mbar_init(&tmem_full[b], 1);
      // a part is drained by the four warps (one per lane quarter) of one epilogue group, the whole buffer by all eight
      mbar_init(&tmem_empty[b], (PAIR ? 2 : 1) * (SUB > 1 ? kEpiWarps / 2 : kEpiWarps));
    }
    fence_barrier_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmX);
    if (FP8) prefetch_tensormap(&tmS);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_holder, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_holder, kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync();   // the peer's barriers are initialised before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // cluster addresses of the barriers that live in the leading CTA
  const uint32_t full0_remote = PAIR ? map_to_cta(smem_u32(&full[0]), 0) : 0u;
  const uint32_t tmem_empty0_remote = PAIR ? map_to_cta(smem_u32(&tmem_empty[0]), 0) : 0u;
  const uint32_t sf_ready0_remote = (PAIR && MX) ? map_to_cta(smem_u32(&sf_ready[0]), 0) : 0u;
  // Barrier set-up, TMEM allocation and descriptor prefetch above touch no tensor data, so they overlap
  // with the tail of the previous kernel; from here on the operands (and the workspace) are used.
  tgi::pdl_wait();
  tgi::pdl_trigger();

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
          if (it >= STAGES) ok = wait(&empty[s], ((it / STAGES) - 1) & 1);
          if (!ok) { report(status, kErrProducerWait); break; }
          uint8_t* st = smem + s * Cfg::kStageBytes;
          // MX: with a stage go the activation scales of the K block AFTER its own (with the first stage also its
          // own), on barriers of their own, so that a K block's scale factors are in TMEM before its operands land
          const bool sc_next = MX && it + 1 < nunits;
          constexpr uint32_t kCtaBytes = Cfg::kStageBytes + (PROMOTE ? CM * 4 : 0);
          if (PAIR) {
            // both CTAs' bytes are counted on the leader's barrier; only the leader posts the expectation
            const uint32_t bar = full0_remote + s * 8;
            if (crank == 0) mbar_arrive_expect_tx(&full[s], 2 * kCtaBytes);
            tma_load_2d_pair_hint(st, &tmX, bar, kb * BK, m0 + static_cast<int>(crank) * CM, pol_x);
            tma_load_2d_pair_hint(st + Cfg::kXBytes, &tmW, bar, kb * BK, n0 + static_cast<int>(crank) * Cfg::WROWS, pol_w);
            if (PROMOTE) tma_load_2d_pair(sc_ring + (it % SC_STAGES) * CM, &tmS, bar, m0 + static_cast<int>(crank) * CM, kb);
            if (MX) {      // every CTA fetches the scales of its own token rows, on its own barriers
              if (it == 0) {
                mbar_arrive_expect_tx(&sc_full[0], CM * 4);
                tma_load_2d(sc_ring, &tmS, &sc_full[0], m0 + static_cast<int>(crank) * CM, kb);
              }
              if (sc_next) {
                UnitIter nxt = ui;
                nxt.next(sch);
                const int slot = (it + 1) % SC_STAGES;
                mbar_arrive_expect_tx(&sc_full[slot], CM * 4);
                tma_load_2d(sc_ring + slot * CM, &tmS, &sc_full[slot], nxt.tm * TM + static_cast<int>(crank) * CM, nxt.kb);
              }
            }
          } else {
            mbar_arrive_expect_tx(&full[s], kCtaBytes);
#pragma unroll
            for (int h = 0; h < MH; ++h) tma_load_2d_hint(st + h * 16384, &tmX, &full[s], kb * BK, m0 + h * 128, pol_x);
#pragma unroll
            for (int h = 0; h < TN / 128; ++h)
              tma_load_2d_hint(st + Cfg::kXBytes + h * 16384, &tmW, &full[s], kb * BK, n0 + h * 128, pol_w);
            if (PROMOTE) tma_load_2d(sc_ring + (it % SC_STAGES) * TM, &tmS, &full[s], m0, kb);
            if (MX) {
              if (it == 0) {
                mbar_arrive_expect_tx(&sc_full[0], CM * 4);
                tma_load_2d(sc_ring, &tmS, &sc_full[0], m0, kb);
              }
              if (sc_next) {
                // the slot's previous scales (K block it - STAGES - 1) were turned into scale factors before the MMAs
                // of K block it - STAGES could run, and those are complete (this stage was free)
                UnitIter nxt = ui;
                nxt.next(sch);
                const int slot = (it + 1) % SC_STAGES;
                mbar_arrive_expect_tx(&sc_full[slot], CM * 4);
                tma_load_2d(sc_ring + slot * TM, &tmS, &sc_full[slot], nxt.tm * TM, nxt.kb);
              }
            }
          }
          issued = it + 1;
        }
        if (!ok && (!PAIR || crank == 0)) {
          // drain: wait (bounded) for the loads already issued so none lands after the CTA exits (in a pair
          // the cluster barrier at the end additionally keeps both CTAs alive until both producers are done)
          for (int it = max(0, issued - STAGES); it < issued; ++it)
            mbar_wait(&full[it % STAGES], (it / STAGES) & 1, 1u << 12);
          if (MX)      // the scale copies that went out with the last stages
            for (int j = max(0, issued - 1); j <= issued; ++j) mbar_wait(&sc_full[j % SC_STAGES], (j / SC_STAGES) & 1, 1u << 12);
        }
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer (in a pair: the leading CTA only) ----------------
      if (crank == 0 && elect_one()) {
        constexpr int MMA_M = PAIR ? 256 : 128;
        constexpr uint32_t idesc = FP8 ? make_idesc(MMA_M, TN, 0, 0) : make_idesc(MMA_M, TN, 1, 1);
        constexpr uint32_t kSfCol0 = kBufCols;       // first scale-factor column (MX)
        int seg = 0;        // accumulator uses so far (fp8: one per K block, bf16: one per tile segment)
        UnitIter ui(u0, sch);
        for (int it = 0; it < nunits; ++it, ui.next(sch)) {
          const int kb = ui.kb;
          const bool seg_start = (it == 0) || kb == 0;
          const bool seg_end = (it == nunits - 1) || kb == sch.KB - 1;
          const int use = PROMOTE ? it : seg;
          const int b = MX ? 0 : use & 1;            // MX: a single accumulator buffer
          if (!PROMOTE && seg_start &&
              (MX ? (use >= 1 && !wait(&tmem_empty[0], (use - 1) & 1))
                  : (use >= 2 && !wait(&tmem_empty[b], ((use >> 1) - 1) & 1)))) {
            report(status, kErrMmaWaitAccum);
            break;
          }
          const int s = it % STAGES;
          if (!wait(&full[s], (it / STAGES) & 1)) { report(status, kErrMmaWaitFull); break; }
          const int sfs = it % (2 * STAGES);      // scale-factor slot: a ring twice as long as the stages
          if (MX && !wait(&sf_ready[sfs], (it / (2 * STAGES)) & 1)) { report(status, kErrMmaWaitFull); break; }
          tc_fence_after();
          const uint32_t x_addr = smem_u32(smem + s * Cfg::kStageBytes);
          bool acc_ok = true;
          const uint64_t dw = make_desc_sw128(x_addr + Cfg::kXBytes);
#pragma unroll
          for (int h = 0; h < MH; ++h) {   // token halves
            if (PROMOTE) {
              const int p = SUB == 2 ? h : 0;
              if (use >= 2 && !wait(&tmem_empty[b * SUB + p], ((use >> 1) - 1) & 1)) { acc_ok = false; break; }
              tc_fence_after();
            }
            const uint64_t dx = make_desc_sw128(x_addr + h * 16384);
            const uint32_t d = tmem_base + b * kBufCols + h * TN;
#pragma unroll
            for (int k = 0; k < 4; ++k) {   // 4 MMAs of 32 bytes of K each per 128-byte row
              const uint32_t accumulate = PROMOTE ? (k > 0) : (!seg_start || k > 0);
              if (MX) {
                // scale-factor byte k of the stage's columns: the k-th 32-deep slice of the K block
                const uint32_t tsf = tmem_base + kSfCol0 + sfs * 16;
                if (PAIR)
                  mma_mxf8f6f4_pair(d, dx + (k * 32 >> 4), dw + (k * 32 >> 4), make_idesc_mx(MMA_M, TN, k, k), tsf + h * 4,
                                    tsf + 8, accumulate);
                else
                  mma_mxf8f6f4(d, dx + (k * 32 >> 4), dw + (k * 32 >> 4), make_idesc_mx(MMA_M, TN, k, k), tsf + h * 4, tsf + 8,
                               accumulate);
              } else if (PAIR) {
                if (FP8) mma_f8f6f4_pair(d, dx + (k * 32 >> 4), dw + (k * 32 >> 4), idesc, accumulate);
                else mma_f16_pair(d, dx + (k * 32 >> 4), dw + (k * 32 >> 4), idesc, accumulate);
              } else {
                if (FP8) mma_f8f6f4(d, dx + (k * 32 >> 4), dw + (k * 32 >> 4), idesc, accumulate);
                else mma_f16(d, dx + (k * 32 >> 4), dw + (k * 32 >> 4), idesc, accumulate);
              }
            }
            if (PROMOTE) {   // hand this part to the epilogue (of both CTAs in a pair)
              const int p = SUB == 2 ? h : 0;
              if (PAIR) tc_commit_pair(&tmem_full[b * SUB + p], 3);
              else tc_commit(&tmem_full[b * SUB + p]);
            }
          }
          if (!acc_ok) { report(status, kErrMmaWaitAccum); break; }
          if (PAIR) {
            tc_commit_pair(&empty[s], 3);                                  // frees the stage in both CTAs
            if (!PROMOTE && seg_end) tc_commit_pair(&tmem_full[b], 3);
          } else {
            tc_commit(&empty[s]);
            if (!PROMOTE && seg_end) tc_commit(&tmem_full[b]);
          }
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
    const int m_cta = (MH == 2 ? g * 128 : 0) + quarter * 32 + lane;      // token row inside this CTA's part
    const int m_local = m_cta + static_cast<int>(crank) * CM;              // ... inside the tile
    const int n_off = (MH == 2 ? 0 : g * kCols);
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + col_base;
    const int et = threadIdx.x - 128;                        // index among the epilogue threads
    AccPairs acc;
    int seg = 0;
    int seg_kb0 = 0;
    bool ok = true;
    // arrival on the accumulator-drained barrier: local, or in the leading CTA of a pair
    auto release_accum = [&](int hb) {
      if (PAIR) mbar_arrive_remote(tmem_empty0_remote + hb * 8);
      else mbar_arrive(&tmem_empty[hb]);
    };
    // split tiles are finished per CTA: in a pair every CTA owns the token half it accumulated
    auto counter_of = [&](int tile) { return PAIR ? tile * 2 + static_cast<int>(crank) : tile; };
    int pend_tile[2];      // tiles this CTA holds only a part of (at most its first and its last)
    int npend = 0;
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
      if (MX && ew < 4) {
        // scale factors of this K block into the stage's TMEM columns: rows 32 * blk + lane of an operand go to
        // column blk of this warp's lane quarter, the block scale's exponent in all four bytes
        // The scales of K block `it` were requested together with the copies of K block `it - 1` (the first with its
        // own), so this write is done before the block's operands land.  The scale-factor ring is 2 * STAGES long:
        // the scales of block `it` are requested when the MMAs of block `it - 1 - STAGES` are complete, which
        // covers the slot's previous user `it - 2 * STAGES`.
        ok = wait(&sc_full[it % SC_STAGES], (it / SC_STAGES) & 1);
        if (!ok) { report(status, kErrEpilogueWait); break; }
        const int sfs = it % (2 * STAGES);
        const uint32_t tsf = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kBufCols + sfs * 16;
        const float* sc = sc_ring + (it % SC_STAGES) * CM;
#pragma unroll
        for (int h = 0; h < MH; ++h) {
          uint32_t w[4];
#pragma unroll
          for (int blk = 0; blk < 4; ++blk)
            w[blk] = ((__float_as_uint(sc[h * 128 + blk * 32 + lane]) >> 23) & 0xFFu) * 0x01010101u;
          tmem_st_32x32b_x4(tsf + h * 4, w);
        }
#pragma unroll
        for (int j = 0; j < TN / 128; ++j) {
          // a tile that hangs over the last weight rows reads the last block's scale for the rows that do not exist
          const int wb = min((n0 >> 7) + j, (N - 1) >> 7);
          const float sw = __ldg(&wscale[static_cast<size_t>(wb) * sch.KB + kb]);
          const uint32_t e = ((__float_as_uint(sw) >> 23) & 0xFFu) * 0x01010101u;
          const uint32_t w[4] = {e, e, e, e};
          tmem_st_32x32b_x4(tsf + 8 + j * 4, w);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_remote(sf_ready0_remote + sfs * 8);      // the leading CTA issues the MMAs
          else mbar_arrive(&sf_ready[sfs]);
        }
      }
      if (PROMOTE) {
        const int b = it & 1;
        const int hb = b * SUB + (SUB == 2 ? g : 0);   // g: token half of this warp when MH == 2
        ok = wait(&tmem_full[hb], (it >> 1) & 1);
        if (!ok) { report(status, kErrEpilogueWait); break; }
        tc_fence_after();
        if (warp_active) {
          const float s = sc_ring[(it % SC_STAGES) * CM + m_cta] *
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
        if (lane == 0) release_accum(hb);
      } else if (seg_end) {
        const int b = MX ? 0 : seg & 1;
        ok = mbar_wait_relaxed(&tmem_full[b], MX ? (seg & 1) : ((seg >> 1) & 1));
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
        if (lane == 0) release_accum(b);
      }
      if (!seg_end) continue;
      ++seg;
      // ---- finish the segment [seg_kb0, kb] of `tile` ----
      const int m = m0 + m_local;
      const int nb = n0 + n_off;                              // first output column of this thread
      const bool whole = seg_kb0 == 0 && kb == sch.KB - 1;
      if (!whole) {
        // Partial tile: publish the fp32 partial sums in this CTA's slot (head slot if the tile is the
        // CTA's first, else tail slot) and count the arrival.  The tile is finished after the main
        // loop, when every contributor reduces its own slice of the columns (see below).
        const int first_tile = static_cast<int>(u0 / sch.KB);
        const int slot = blockIdx.x * 2 + (tile == first_tile ? 0 : 1);
        float4* wsp = reinterpret_cast<float4*>(ws + static_cast<size_t>(slot) * kTileElems) + et;
#pragma unroll
        for (int j = 0; j < kCols; j += 4)
          wsp[(j >> 2) * kEpiThreads] = make_float4(acc.get(j), acc.get(j + 1), acc.get(j + 2), acc.get(j + 3));
        __threadfence();
        epi_barrier();
        if (et == 0) atomicAdd(&counters[counter_of(tile)], 1);
        pend_tile[npend++] = tile;
        continue;
      }
      if (m < M && nb < N) {
        __nv_bfloat16* crow = out_row(m) + nb;
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

    // ---- finish the tiles this CTA shares with other CTAs ----
    // Every contributor of a split tile has published its partial sums by now or will soon: all
    // CTAs of the grid are resident (one per SM) and none waits before it has published everything.
    // Contributor i of n reduces float4 columns [32 i / n, 32 (i+1) / n) of all rows, summing the
    // partials in CTA order (so the result does not depend on timing), and stores them.  The tile
    // counter counts n arrivals, then n departures; the last departure resets it for the next launch.
    for (int p = 0; p < npend && ok; ++p) {
      const int tile = pend_tile[p];
      const int tn = tile / sch.m_tiles, tm = tile - tn * sch.m_tiles;
      const int n0 = tn * TN, m0 = tm * TM;
      const long long t_lo = static_cast<long long>(tile) * sch.KB, t_hi = t_lo + sch.KB - 1;
      const int c_lo = sch.owner(t_lo), c_hi = sch.owner(t_hi);
      const int n = c_hi - c_lo + 1;
      const int mine = worker - c_lo;
      // contributor c is a CTA, or in a pair the CTA of worker c that holds the same token half as this one
      for (int c = c_lo + et; c <= c_hi; c += kEpiThreads)
        cslots[c - c_lo] = (PAIR ? c * 2 + static_cast<int>(crank) : c) * 2 +
                           (tile == static_cast<int>(sch.begin(c) / sch.KB) ? 0 : 1);
      if (et == 0) {
        int polls = 0;
        int seen;
        while ((seen = ld_acquire_gpu(&counters[counter_of(tile)])) < n && ++polls < kSplitPolls) __nanosleep(64);
        *flag = seen >= n;
      }
      epi_barrier();
      ok = *flag != 0;
      if (!ok) {
        report(status, kErrSplitKWait);
        break;
      }
      const int jc0 = mine * (kCols / 4) / n, jc1 = (mine + 1) * (kCols / 4) / n;
      const int m = m0 + m_local;
      const int nb = n0 + n_off;
      const float4* wsb = reinterpret_cast<const float4*>(ws) + et;
      for (int jc = jc0; jc < jc1; ++jc) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i = 0; i < n; ++i) {
          const float4 t = __ldcg(wsb + static_cast<size_t>(cslots[i]) * (kTileElems / 4) + jc * kEpiThreads);
          sum.x += t.x;
          sum.y += t.y;
          sum.z += t.z;
          sum.w += t.w;
        }
        const int col = nb + jc * 4;
        if (m < M && col < N) {
          float f[4] = {sum.x, sum.y, sum.z, sum.w};
          if (bias != nullptr) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (col + e < N) f[e] += __bfloat162float(bias[col + e]);
          }
          __nv_bfloat16* cp = out_row(m) + col;
          if ((N & 3) == 0) {
            __nv_bfloat162 o[2] = {__floats2bfloat162_rn(f[0], f[1]), __floats2bfloat162_rn(f[2], f[3])};
            *reinterpret_cast<uint2*>(cp) = *reinterpret_cast<uint2*>(o);
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (col + e < N) cp[e] = __float2bfloat16(f[e]);
          }
        }
      }
      epi_barrier();   // all reads of the partials and of cslots are done
      if (et == 0) {
        const int old = atomicAdd(&counters[counter_of(tile)], 1);
        if (old == 2 * n - 1) counters[counter_of(tile)] = 0;
      }
    }

    // ---- peer-memory output: tell the row owners that this rank's partial sums have landed ----
    if (push.world > 0) {
      epi_barrier();                       // every store of this CTA was issued
      if (et == 0) {
        __threadfence_system();            // ... and is ordered before the count below, at system scope
        const int old = atomicAdd(push.done_ctas, 1);
        if (old == static_cast<int>(gridDim.x) - 1) {
          *push.done_ctas = 0;
          const unsigned int e = *push.epoch + 1u;
          *push.epoch = e;
          __threadfence_system();          // the other CTAs' stores (observed through the counter) before the flags
          for (int r = 0; r < push.world; ++r) {
            unsigned int* f = reinterpret_cast<unsigned int*>(push.heap[r] + push.off_flags) + push.rank;
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(f), "r"(e) : "memory");
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync();   // neither CTA frees TMEM or leaves while the other may still use its memory
  if (warp == 1) {
    if (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
using tgi::make_map_2d;

int g_streamk_small = 0;   // 1: problems with fewer tiles than workers may also be spread by stream-K

template <int MH, int TN, int STAGES, bool FP8, bool PAIR, bool MX = false>
int launch(const void* X, const float* xs_t, int xs_pitch, const void* W, const float* wscale, void* C,
           const void* bias, int M, int N, int K, int max_ctas, float* ws, int* counters, int* status,
           cudaStream_t stream, const PushArgs* push_args = nullptr) {
  using Cfg = TileCfg<MH, TN, PAIR, FP8, MX>;
  PushArgs push;
  if (push_args != nullptr) {
    push = *push_args;
  } else {
    memset(&push, 0, sizeof(push));
  }
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
                     Cfg::CM, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  } else {
    tmS = tmX;
  }
  // stages + (fp8) activation-scale ring [STAGES+2][CM] + alignment slack + barriers
  const size_t smem = STAGES * Cfg::kStageBytes + (FP8 ? (STAGES + 2) * Cfg::CM * 4 : 0) + 1024 + 512 + kMaxGrid * 4;
  auto kern = gemm_streamk_kernel<MH, TN, STAGES, FP8, PAIR, MX>;
  // The shared-memory opt-in is a per-device attribute of the function; the number of CTA pairs that can
  // be resident at once (a GPC with an odd number of usable SMs cannot pair its last one) is a property of
  // the device too.  Both are looked up once per device ordinal.
  static std::atomic<unsigned long long> attr_set{0};
  static std::atomic<int> max_pairs[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -2;
  const unsigned long long dev_bit = 1ull << (dev & 63);
  if (!(attr_set.load(std::memory_order_acquire) & dev_bit)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return -2;
    if (PAIR) {
      cudaLaunchConfig_t q{};
      q.gridDim = dim3(2 * kMaxGrid);
      q.blockDim = dim3(kThreads);
      q.dynamicSmemBytes = smem;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2;
      qa[0].val.clusterDim.y = 1;
      qa[0].val.clusterDim.z = 1;
      q.attrs = qa;
      q.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, kern, &q) != cudaSuccess || clusters < 1) {
        cudaGetLastError();
        return -4;
      }
      max_pairs[dev & 63].store(clusters, std::memory_order_relaxed);
    }
    attr_set.fetch_or(dev_bit, std::memory_order_release);
  }
  // workers: CTAs, or CTA pairs
  int max_workers = PAIR ? max_ctas / 2 : max_ctas;
  if (PAIR && max_workers > max_pairs[dev & 63].load(std::memory_order_relaxed))
    max_workers = max_pairs[dev & 63].load(std::memory_order_relaxed);
  if (max_workers > (PAIR ? kMaxGrid / 2 : kMaxGrid)) max_workers = PAIR ? kMaxGrid / 2 : kMaxGrid;
  if (max_workers < 1) return -4;
  const long long units =
      static_cast<long long>((N + TN - 1) / TN) * ((M + Cfg::TM - 1) / Cfg::TM) * ((K + BK - 1) / BK);
  // Number of workers.  Splitting a tile between workers costs a 128 KB fp32 partial per contributing CTA (as
  // much traffic as 8 K blocks of weights), so small problems prefer whole tiles or a few aligned splits:
  //   stream-K over all workers:  ceil(units / workers) K blocks each, plus the fix-up (~2 blocks)
  //   tiles x s aligned splits:   ceil(KB / s) K blocks each, s = 1 needs no fix-up at all
  const int KBn = (K + BK - 1) / BK;
  const int tiles = static_cast<int>(units / KBn);
  int grid = max_workers;
  if (grid > units) grid = static_cast<int>(units);
  if (grid < 1) grid = 1;
  if (tiles <= max_workers) {
    // Rough costs in microseconds, from timelines measured on B200: a K block takes about 0.4 us per
    // CTA; every partial tile costs 128 KB written and read through L2 by all CTAs at once (about
    // 0.05 us each at ~5 TB/s) and a split adds ~3 us of publish / wait / reduce latency.
    const double kUnit = 0.4, kPartial = 0.05, kSync = 3.0;
    const double partials_sk = static_cast<double>(grid + tiles < 2 * grid ? grid + tiles : 2 * grid);
    double best = static_cast<double>((units + grid - 1) / grid) * kUnit + partials_sk * kPartial + kSync;
    // Measured on B200, aligned splits win wherever both apply: 256 x 10240 x 8192 bf16 51.1 us against 64.4 with
    // stream-K, 256 x 8192 x 8192 46.5 against 54.4, 32 x 8192 x 28672 fp8 53.0 against 63.9, fp8 pairs 256 x 10240 x
    // 8192 36.1 against 54.3.  So stream-K is left to problems with more tiles than workers unless it is asked for.
    if (!g_streamk_small) best = 1e30;
    for (int s = 1; s <= max_workers / tiles && s <= KBn; ++s) {
      const double c = static_cast<double>((KBn + s - 1) / s) * kUnit + (s > 1 ? tiles * s * kPartial + kSync : 0.0);
      if (c < best) {
        best = c;
        grid = tiles * s;
      }
    }
  }
  g_last_grid = PAIR ? 2 * grid : grid;
  const cudaError_t err =
      tgi::launch_cluster(kern, dim3(PAIR ? 2 * grid : grid), dim3(kThreads), smem, stream, PAIR ? 2 : 1, tmW, tmX, tmS,
                          wscale, static_cast<__nv_bfloat16*>(C), static_cast<const __nv_bfloat16*>(bias), M, N, K, ws,
                          counters, status, push);
  return err == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int fill_push(PushArgs& p, void* const* heaps, int rank, int world, int rows_per, long long off_slots,
              long long off_flags, int* done_ctas, unsigned int* epoch, int M) {
  if (world < 2 || world > 8 || rank < 0 || rank >= world || rows_per < 1) return -20;
  if (static_cast<long long>(rows_per) * world < M) return -21;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < world; ++i) p.heap[i] = static_cast<unsigned char*>(heaps[i]);
  p.off_slots = off_slots;
  p.off_flags = off_flags;
  p.rank = rank;
  p.world = world;
  p.rows_per = rows_per;
  p.done_ctas = done_ctas;
  p.epoch = epoch;
  return 0;
}

}  // namespace

static int g_wide_m = 128;
static int g_pairs = 1;
static int g_pair_min_tiles = 32;
static int g_fp8_mx = 0;          // block-scaled MMA for fp8 (scales must be powers of two)
static int g_mx_pairs = 1;        // CTA pairs in the block-scaled mode

namespace {
template <bool FP8>
int dispatch(const void* X, const float* xs_t, int xs_pitch, const void* W, const float* wscale, void* C, const void* bias,
             int M, int N, int K, int max_ctas, float* ws, int* counters, int* status, cudaStream_t stream,
             const PushArgs* push) {
  if (FP8 && g_fp8_mx) {
    if (M <= g_wide_m)
      return launch<1, 256, 4, FP8, false, FP8>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, max_ctas, ws, counters,
                                                 status, stream, push);
    const long long mx_pair_tiles = static_cast<long long>((N + 255) / 256) * ((M + 255) / 256);
    // pairs need enough work to repay their fixed cost: 256 x 8192 x 4096 (32 tiles of 32 K blocks) takes 30.7 us in
    // pairs and 25.6 us on single CTAs, 256 x 8192 x 8192 37.1 against 38.3, 256 x 8192 x 14336 47.5 against 51.2
    // (a caller that lowers the tile threshold, as the tests do to reach pairs with small problems, lifts this one too)
    const long long mx_pair_units = mx_pair_tiles * ((K + 127) / 128);
    if (g_pairs && g_mx_pairs && max_ctas >= 2 && mx_pair_tiles >= g_pair_min_tiles &&
        (mx_pair_units >= 2048 || g_pair_min_tiles < 32)) {
      const int rc = launch<1, 256, 6, FP8, FP8, FP8>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, max_ctas, ws, counters,
                                                       status, stream, push);
      if (rc != -4) return rc;
    }
    return launch<2, 128, 4, FP8, false, FP8>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, max_ctas, ws, counters, status,
                                               stream, push);
  }
  if (M <= g_wide_m)
    return launch<1, 256, 4, FP8, false>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, max_ctas, ws, counters, status,
                                         stream, push);
  // Pairs pay off when there are enough 256 x 256 tiles to go round: with few tiles (tensor-parallel shards, narrow
  // projections) the 74 pairs split K deeper than 148 single CTAs on 256 x 128 tiles do, and the fix-up of split
  // tiles costs more than the saved operand traffic (measured: 256 x 7168 x 8192 51 us in pairs, 48 us without).
  const long long pair_tiles = static_cast<long long>((N + 255) / 256) * ((M + 255) / 256);
  if (g_pairs && max_ctas >= 2 && pair_tiles >= g_pair_min_tiles) {
    const int rc = launch<1, 256, 6, FP8, true>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, max_ctas, ws, counters,
                                                status, stream, push);
    if (rc != -4) return rc;   // -4: this device cannot place a pair; fall back to single CTAs
  }
  return launch<2, 128, 4, FP8, false>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, max_ctas, ws, counters, status,
                                       stream, push);
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
  const int a = ((N + 127) / 128) * ((M + 255) / 256);
  const int b = ((N + 255) / 256) * ((M + 127) / 128);
  const int c = 2 * ((N + 255) / 256) * ((M + 255) / 256);   // a pair keeps one counter per CTA and tile
  return a > b ? (a > c ? a : c) : (b > c ? b : c);   // upper bound over all tile shapes
}

// Token counts up to this limit use one CTA per 128 x 256 tile (weights-wide); larger ones CTA pairs on
// 256 x 256 tiles, or single CTAs on 256 x 128 tiles when pairs are switched off.
void tgi_gemm_set_wide_m(int m) { g_wide_m = m < 128 ? 128 : m; }
void tgi_gemm_set_pairs(int on) { g_pairs = on != 0; }
// fp8 GEMMs on the block-scaled MMA: every activation and weight scale handed to tgi_gemm_fp8_block must then be a
// power of two (their exponents become the E8M0 scale factors; mantissa bits are ignored)
void tgi_gemm_set_fp8_mx(int on) { g_fp8_mx = on != 0; }
void tgi_gemm_set_mx_pairs(int on) { g_mx_pairs = on != 0; }
void tgi_gemm_set_streamk_small(int on) { g_streamk_small = on != 0; }
void tgi_gemm_set_pair_min_tiles(int n) { g_pair_min_tiles = n < 1 ? 1 : n; }
// CTAs of the most recent GEMM launch of this process (diagnostics and benchmarks).
int tgi_gemm_last_grid(void) { return g_last_grid; }

int tgi_gemm_bf16(const void* X, const void* W, void* C, const void* bias, int M, int N, int K, int max_ctas,
                  float* ws, int* counters, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0) return -10;  // TMA row pitch must be a multiple of 16 bytes
  return dispatch<false>(X, nullptr, 0, W, nullptr, C, bias, M, N, K, max_ctas, ws, counters, status, stream, nullptr);
}

int tgi_gemm_fp8_block(const void* X, const float* xs_t, int xs_pitch, const void* W, const float* wscale, void* C,
                       const void* bias, int M, int N, int K, int max_ctas, float* ws, int* counters, int* status,
                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 128 != 0 || xs_pitch % 4 != 0) return -10;
  return dispatch<true>(X, xs_t, xs_pitch, W, wscale, C, bias, M, N, K, max_ctas, ws, counters, status, stream, nullptr);
}

// Row-parallel GEMMs of a tensor-parallel group: same products, but every output row is stored into the
// peer-memory slot of the rank that owns the row (see PushArgs) and the owners are flagged at the end.
// `fp8` selects the block-scaled path (xs_t / wscale as in tgi_gemm_fp8_block, ignored otherwise).
int tgi_gemm_push(int fp8, const void* X, const float* xs_t, int xs_pitch, const void* W, const float* wscale,
                  const void* bias, int M, int N, int K, int max_ctas, float* ws, int* counters, int* status,
                  void* const* heaps, int rank, int world, int rows_per, long long off_slots, long long off_flags,
                  int* done_ctas, unsigned int* epoch, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (N % 8 != 0) return -22;   // 16-byte row segments in the slots
  PushArgs p;
  const int rc = fill_push(p, heaps, rank, world, rows_per, off_slots, off_flags, done_ctas, epoch, M);
  if (rc) return rc;
  if (fp8) {
    if (K % 128 != 0 || xs_pitch % 4 != 0) return -10;
    return dispatch<true>(X, xs_t, xs_pitch, W, wscale, nullptr, bias, M, N, K, max_ctas, ws, counters, status, stream, &p);
  }
  if (K % 8 != 0) return -10;
  return dispatch<false>(X, nullptr, 0, W, nullptr, nullptr, bias, M, N, K, max_ctas, ws, counters, status, stream, &p);
}

}  // extern "C"

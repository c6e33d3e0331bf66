// Tensor-parallel collectives over NVLink peer memory (one process per GPU, sm_100a).
//
// Every rank owns a "heap" allocated with cudaMalloc and mapped into all other ranks with CUDA IPC;
// the same byte offset means the same logical buffer on every rank.  The kernels below replace the
// NCCL all-reduce that follows every row-parallel linear in the reference
// (layers/tensor_parallel.py:202-209) and the separate residual-add + RMSNorm (+ fp8 quantisation)
// that follows it (layers/layernorm.py:161-187, layers/fp8.py:149-159):
//
//   peer_reduce_kernel: rows of the [T, H] partial sums are split across ranks.  The owner of a row
//   pulls the eight partial rows with peer loads, adds them in fp32 in rank order, optionally adds
//   the residual row it keeps locally, applies RMSNorm (+ 1x128 e4m3 quantisation), and pushes the
//   finished row into the gather buffer of every rank with peer stores.  Norm work is divided by
//   the number of ranks and every element crosses NVLink once in and once out.
//
// Synchronisation is block to block: block b of rank r only depends on block b of the other ranks,
// through flags in the destination's heap that carry a per-block call counter kept in device
// memory (so a captured CUDA graph replays correctly).  Every wait is bounded by wall-clock time;
// a wait that runs out sets the status word and the block returns.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.cuh"
#include "sampling.cuh"
#include "sm100.cuh"

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxBlocks = 256;           // flag slots per phase
constexpr float kFp8Max = 448.f;
// Scale of a 128-wide activation block.  With g_quant_pow2 set (the block-scaled MMA takes power-of-two scale
// factors) it is rounded up to the next power of two: the quantised values then use at least half of the e4m3
// range, which costs no relative precision.
__device__ int g_quant_pow2 = 0;
__device__ __forceinline__ float block_scale(float amax) {
  float s = fmaxf(amax, 1e-12f) / kFp8Max;
  if (g_quant_pow2) s = __uint_as_float((__float_as_uint(s) + 0x007FFFFFu) & 0xFF800000u);
  return s;
}
// Default limit of a wait on a flag that another rank writes.  The limit travels as a kernel argument so
// that a test can make it short (tgi_peer_set_wait_ns) and watch a wait run out: a flag that nothing sets
// ends the kernel with status kErrPeerWait after that time, the context stays usable.
unsigned long long g_peer_wait_ns = 2000000000ull;   // 2 s

struct PeerArgs {
  unsigned char* heap[kMaxRanks];   // heap base of every rank as mapped in this process
  int rank, world;
  int T, H;                         // rows and row length (elements) of the reduced matrix
  long long off_partial;            // [T, H] bf16 partial sums, written by the local producer
  long long off_gather;             // gathered result: [T, H] bf16, or [T, H] e4m3 when quantising
  long long off_gscale;             // gathered activation scales, fp32 [H/128][pitch]
  int gscale_pitch;
  long long off_flags;              // uint32 [2][kMaxBlocks][kMaxRanks]
  unsigned int* epoch;              // local, uint32 [kMaxBlocks]: calls made so far by each block
  const __nv_bfloat16* residual_in; // local [rows_per_rank, H] or nullptr
  __nv_bfloat16* residual_out;      // local [rows_per_rank, H] or nullptr
  const __nv_bfloat16* weight;      // norm weight [H]
  float eps, w_offset;
  int* status;
  unsigned long long wait_ns;       // limit of every wait on a peer's flag
  int pushed;                       // 1: the partial rows were pushed into this rank's slots by the producers
  long long off_push_flags;         // uint32 [8] in every heap: call counter of each source's last finished push
  const unsigned int* push_epoch;   // local: call counter of this rank's own producer (all ranks agree on it)
};

struct __align__(16) bf16x8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16(x)); }

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_relaxed_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// 16-byte load that bypasses L1 (the data was written by another GPU or is read by one)
__device__ __forceinline__ uint4 ld_cg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

// Block-level flag exchange with the same block of every other rank.
struct BlockSync {
  const PeerArgs& a;
  unsigned int e;          // value of this call
  int* failed;             // shared-memory flag
  __device__ BlockSync(const PeerArgs& args, int* failed_smem) : a(args), failed(failed_smem) {
    e = a.epoch[blockIdx.x] + 1u;
  }
  __device__ unsigned int* flag(int owner, int phase, int src) const {
    return reinterpret_cast<unsigned int*>(a.heap[owner] + a.off_flags) +
           (static_cast<size_t>(phase) * kMaxBlocks + blockIdx.x) * kMaxRanks + src;
  }
  // all writes of this block made before the call become visible to the peers that see the flag
  // `fence`: order this block's earlier writes before the flag.  Phase 0 announces data that the
  // previous kernel of the stream wrote into this GPU's own memory; the kernel boundary already made
  // it visible at the L2 that serves the peers' loads, so no fence is needed there (it costs ~3 us).
  __device__ void signal(int phase, bool fence) const {
    __syncthreads();
    if (threadIdx.x < a.world) {
      if (fence) __threadfence_system();
      st_relaxed_sys(flag(threadIdx.x, phase, a.rank), e);
    }
  }
  // returns false (for the whole block) when a peer did not signal in time
  __device__ bool wait(int phase) const {
    if (threadIdx.x < a.world) {
      const unsigned int* f = flag(a.rank, phase, threadIdx.x);
      const unsigned long long t0 = global_ns();
      unsigned int polls = 0;
      while (static_cast<int>(ld_relaxed_sys(f) - e) < 0) {
        if ((++polls & 63u) == 0 && global_ns() - t0 > a.wait_ns) {
          atomicExch(a.status, sm100::kErrPeerWait);
          *failed = 1;
          break;
        }
      }
      (void)ld_acquire_sys(f);   // one acquire after the flag was seen: later reads observe the peer's data
    }
    __syncthreads();
    return *failed == 0;
  }
  __device__ void finish() const {
    __syncthreads();
    if (threadIdx.x == 0) a.epoch[blockIdx.x] = e;
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x + 31) / 32) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}
__device__ __forceinline__ uint2 quant8(const float (&f)[8], float scale) {
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float q = fminf(fmaxf(f[4 * h + i] / scale, -kFp8Max), kFp8Max);
      acc |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
    }
    w[h] = acc;
  }
  return make_uint2(w[0], w[1]);
}
__device__ __forceinline__ float group16_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum of the `world` partial vectors (8 bf16 each) at element offset `elem` of the partial buffers,
// in rank order, rounded to bf16 like the all-reduced bf16 tensor it stands for.
// Pull mode: source s holds row `row` of its own [T, H] partial buffer.  Pushed mode: the producers
// already stored their rows into this rank's slots [source][rows_per][H] (GEMM epilogue, PushArgs of
// gemm_sm100.cu), so all loads are local.
__device__ __forceinline__ void pull_sum8(const PeerArgs& a, int row, int lr, int rows_per, int col,
                                          float (&acc)[8]) {
  uint4 raw[kMaxRanks];
#pragma unroll
  for (int s = 0; s < kMaxRanks; ++s)
    if (s < a.world) {
      const size_t elem = a.pushed ? (static_cast<size_t>(s) * rows_per + lr) * a.H + col
                                   : static_cast<size_t>(row) * a.H + col;
      raw[s] = ld_cg16(a.heap[a.pushed ? a.rank : s] + a.off_partial + elem * 2);
    }
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
  for (int s = 0; s < kMaxRanks; ++s)
    if (s < a.world) {
      float f[8];
      unpack8(raw[s], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = round_bf16(acc[j]);
}

// NORM = false: plain all-reduce (bf16 result in every rank's gather buffer).
// NORM = true : + residual add, RMSNorm, and with QUANT 1x128 e4m3 quantisation of the result.
template <bool NORM, bool QUANT, int VPT>
__global__ void __launch_bounds__(1024)
peer_reduce_kernel(const PeerArgs a) {
  __shared__ float red[32];
  __shared__ int failed;
  tgi::pdl_wait();
  tgi::pdl_trigger();
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  BlockSync sync(a, &failed);
  const int rows_per = (a.T + a.world - 1) / a.world;
  const int row0 = a.rank * rows_per;
  const int my_rows = max(0, min(a.T, row0 + rows_per) - row0);
  const int nvec = a.H / 8;

  bool ok;
  if (a.pushed) {
    // the producers flagged their pushes themselves: wait until every source's counter reached this call
    if (threadIdx.x < a.world) {
      const unsigned int want = *a.push_epoch;
      const unsigned int* f = reinterpret_cast<const unsigned int*>(a.heap[a.rank] + a.off_push_flags) + threadIdx.x;
      const unsigned long long t0 = global_ns();
      unsigned int polls = 0;
      while (static_cast<int>(ld_relaxed_sys(f) - want) < 0) {
        if ((++polls & 63u) == 0 && global_ns() - t0 > a.wait_ns) {
          atomicExch(a.status, sm100::kErrPeerWait);
          failed = 1;
          break;
        }
      }
      (void)ld_acquire_sys(f);
    }
    __syncthreads();
    ok = failed == 0;
  } else {
    sync.signal(0, false);                     // my producer kernel has finished: its partial rows may be read
    ok = sync.wait(0);
  }
  if (ok) {
    for (int lr = blockIdx.x; lr < my_rows; lr += gridDim.x) {
      const int row = row0 + lr;
      const size_t rbase = static_cast<size_t>(row) * a.H;
      if (!NORM) {
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
          float acc[8];
          pull_sum8(a, row, lr, rows_per, v * 8, acc);
          const uint4 packed = pack8(acc);
#pragma unroll
          for (int d = 0; d < kMaxRanks; ++d)
            if (d < a.world) *reinterpret_cast<uint4*>(a.heap[d] + a.off_gather + (rbase + v * 8) * 2) = packed;
        }
      } else {
        float s[VPT][8];
        float sumsq = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = threadIdx.x + i * blockDim.x;
          if (v < nvec) {
            const size_t lbase = static_cast<size_t>(lr) * a.H + v * 8;
            uint4 res_raw = make_uint4(0, 0, 0, 0);   // issued before the peer loads so the latencies overlap
            if (a.residual_in != nullptr) res_raw = *reinterpret_cast<const uint4*>(a.residual_in + lbase);
            pull_sum8(a, row, lr, rows_per, v * 8, s[i]);
            if (a.residual_in != nullptr) {
              float r[8];
              unpack8(res_raw, r);
#pragma unroll
              for (int j = 0; j < 8; ++j) s[i][j] = round_bf16(s[i][j] + r[j]);
            }
            if (a.residual_out != nullptr) *reinterpret_cast<uint4*>(a.residual_out + lbase) = pack8(s[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) sumsq += s[i][j] * s[i][j];
          }
        }
        const float rstd = rsqrtf(block_sum(sumsq, red) / a.H + a.eps);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = threadIdx.x + i * blockDim.x;
          const bool active = v < nvec;
          float y[8];
          if (active) {
            float w[8];
            unpack8(*reinterpret_cast<const uint4*>(a.weight + v * 8), w);
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = round_bf16(s[i][j] * rstd * (w[j] + a.w_offset));
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = 0.f;
          }
          if (QUANT) {
            float amax = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(y[j]));
            amax = group16_max(amax);
            const float scale = block_scale(amax);
            if (active) {
              const uint2 q = quant8(y, scale);
#pragma unroll
              for (int d = 0; d < kMaxRanks; ++d)
                if (d < a.world) {
                  *reinterpret_cast<uint2*>(a.heap[d] + a.off_gather + rbase + v * 8) = q;
                  if ((v & 15) == 0)
                    reinterpret_cast<float*>(a.heap[d] + a.off_gscale)[static_cast<size_t>(v >> 4) * a.gscale_pitch + row] =
                        scale;
                }
            }
          } else if (active) {
            const uint4 packed = pack8(y);
#pragma unroll
            for (int d = 0; d < kMaxRanks; ++d)
              if (d < a.world) *reinterpret_cast<uint4*>(a.heap[d] + a.off_gather + (rbase + v * 8) * 2) = packed;
          }
        }
      }
    }
    sync.signal(1, true);                     // my rows are in everybody's gather buffer
    ok = sync.wait(1);                  // and everybody's rows are in mine
  }
  sync.finish();
}

// ------------------------------------------------------------------------------------------------
// Vocabulary-parallel greedy sampling.  The reference all-gathers the [B, V] logits of the sharded
// lm_head (layers/tensor_parallel.py:75-104) and runs log_softmax + argmax on the full matrix.  Here
// every rank reduces its own [B, V / world] slice to one candidate per row,
//     (m, i, s) = (max logit, global index of the max, sum of exp(x - m) over the slice),
// pushes the 16-byte candidate into every rank's heap and merges the `world` candidates of a row:
//     M = max m_r,  token = i of the rank holding M (lowest rank on ties),
//     logprob = M - (M + log sum_r s_r exp(m_r - M)).
// 16 bytes per row and rank cross NVLink instead of V / world logits.
// ------------------------------------------------------------------------------------------------
struct __align__(16) Candidate {
  float m;
  int idx;
  float s;
  int pad;
};

__global__ void __launch_bounds__(1024)
peer_argmax_kernel(const PeerArgs a, const __nv_bfloat16* __restrict__ logits, long long row_stride, int vocab_start,
                   float logit_scale, long long off_cand, long long* __restrict__ ids, float* __restrict__ logprob) {
  __shared__ float sm_m[32], sm_s[32];
  __shared__ int sm_i[32];
  __shared__ int failed;
  tgi::pdl_wait();
  tgi::pdl_trigger();
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  BlockSync sync(a, &failed);
  const int B = a.T, Vl = a.H;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int row = blockIdx.x; row < B; row += gridDim.x) {
    const __nv_bfloat16* x = logits + static_cast<size_t>(row) * row_stride;
    float m = -INFINITY, s = 0.f;
    int idx = 0x7fffffff;
    for (int v = threadIdx.x; v < Vl; v += blockDim.x) {
      const float val = __bfloat162float(x[v]) * logit_scale;
      if (val > m) {
        s = s * __expf(m - val) + 1.f;
        m = val;
        idx = v;
      } else if (val != -INFINITY) {
        s += __expf(val - m);
      }
    }
    // merge (m, idx, s) across the warp, then across warps; ties keep the smaller index
    auto merge = [](float& m1, int& i1, float& s1, float m2, int i2, float s2) {
      if (m2 == -INFINITY) return;      // the other side saw no finite logit
      if (m2 > m1 || (m2 == m1 && i2 < i1)) {
        s1 = s1 * __expf(m1 - m2) + s2;
        m1 = m2;
        i1 = i2;
      } else if (m2 != -INFINITY) {
        s1 += s2 * __expf(m2 - m1);
      }
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      merge(m, idx, s, m2, i2, s2);
    }
    __syncthreads();
    if (lane == 0) {
      sm_m[warp] = m;
      sm_i[warp] = idx;
      sm_s[warp] = s;
    }
    __syncthreads();
    if (warp == 0) {
      const int nw = blockDim.x >> 5;
      m = lane < nw ? sm_m[lane] : -INFINITY;
      idx = lane < nw ? sm_i[lane] : 0x7fffffff;
      s = lane < nw ? sm_s[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
        const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        merge(m, idx, s, m2, i2, s2);
      }
      if (lane < a.world) {
        Candidate c;
        c.m = m;
        c.idx = idx + vocab_start;
        c.s = s;
        c.pad = 0;
        Candidate* dst = reinterpret_cast<Candidate*>(a.heap[lane] + off_cand) + static_cast<size_t>(row) * kMaxRanks + a.rank;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&c);
      }
    }
  }
  sync.signal(1, true);
  const bool ok = sync.wait(1);
  if (ok) {
    for (int row = blockIdx.x; row < B; row += gridDim.x) {
      if (threadIdx.x == 0) {
        const Candidate* mine = reinterpret_cast<const Candidate*>(a.heap[a.rank] + off_cand) + static_cast<size_t>(row) * kMaxRanks;
        float M = -INFINITY;
        int best = 0;
        Candidate c[kMaxRanks];
        for (int r = 0; r < a.world; ++r) {
          const uint4 raw = ld_cg16(mine + r);
          c[r] = *reinterpret_cast<const Candidate*>(&raw);
          if (c[r].m > M) {
            M = c[r].m;
            best = r;
          }
        }
        float sum = 0.f;
        for (int r = 0; r < a.world; ++r) sum += c[r].s * __expf(c[r].m - M);
        ids[row] = c[best].idx;
        logprob[row] = -__logf(sum);
      }
    }
  }
  sync.finish();
}

// ------------------------------------------------------------------------------------------------
// Vocabulary-parallel sampling.  The reference gathers the [B, V] logits of the sharded lm_head on every rank
// and runs its warper chain on the full matrix (layers/tensor_parallel.py:75-104, utils/tokens.py:233-503).
// Here every rank keeps its [B, V / world] slice and the ranks agree on the result through a few scalars per
// row: the fused single-GPU sampler (fused_ops.cu `sample_kernel`) only ever needs block-wide reductions of the
// row (max, counts and probability mass above a threshold, the arg-max of the Gumbel-perturbed scores), so each
// of them becomes a block reduction over the slice followed by an exchange of one 8-byte word per rank.
//
//   x_j = score_j / T;   top-k / top-p thresholds by a 4-way search on the order-preserving integer image of
//   the float (16 exchange rounds for 32 bits);   sample = argmax_j x_j + g_j with g_j keyed by the GLOBAL
//   index j, so the draw equals the single-GPU draw for the same seed;   logprob = x_c - logsumexp(kept set).
//
// Exchange: a word is (value bits, sequence number) written with one 64-bit store into the slot
// [block][round parity][word][source rank] of every rank's heap; the reader polls its own slot until the
// sequence number is the expected one.  No separate flag or fence is needed because value and sequence number
// travel in the same 8 aligned bytes.  A rank can run at most one round ahead of another (it needs everybody's
// word of round n before it writes round n + 1), so two parities suffice.  The sequence counter of every block
// lives in device memory and keeps counting across launches and CUDA-graph replays.  Waits are bounded.
// ------------------------------------------------------------------------------------------------
constexpr int kXWords = 4;   // words per exchange round

struct SampleArgs {
  const float* temperature;          // [B] or null
  const int* top_k;                  // [B] or null
  const float* top_p;                // [B] or null
  const unsigned char* do_sample;    // [B] or null
  const long long* seeds;            // [B] or null
  const int* steps;                  // [B] or null
  long long off_xchg;                // heap offset of uint64 [kMaxBlocks][2][kXWords][kMaxRanks]
  unsigned int* xseq;                // local uint32 [kMaxBlocks]: exchange rounds made so far by each block
  int vocab_total;
};

struct Exchange {
  const PeerArgs& a;
  long long off;
  unsigned int seq;          // rounds done so far by this block (same value on every rank)
  int* failed;
  float (*recv)[kMaxRanks];  // shared memory [kXWords][kMaxRanks]
  __device__ unsigned long long* slot(int owner, unsigned int parity, int word, int src) const {
    return reinterpret_cast<unsigned long long*>(a.heap[owner] + off) +
           ((static_cast<size_t>(blockIdx.x) * 2 + parity) * kXWords + word) * kMaxRanks + src;
  }
  // Every thread calls with the same (block-uniform) values; afterwards recv[w][r] holds rank r's word w.
  // Returns false for the whole block when a peer's word did not arrive in time.
  template <int NW>
  __device__ bool all_gather(const float (&v)[NW]) {
    const unsigned int want = seq + 1u;
    const unsigned int parity = want & 1u;
    const int t = threadIdx.x;
    if (t < a.world * NW) {
      const int peer = t / NW, w = t - peer * NW;
      const unsigned long long word = (static_cast<unsigned long long>(want) << 32) | __float_as_uint(v[w]);
      asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(slot(peer, parity, w, a.rank)), "l"(word) : "memory");
    }
    if (t < a.world * NW) {
      const int src = t / NW, w = t - src * NW;
      const unsigned long long* p = slot(a.rank, parity, w, src);
      const unsigned long long t0 = global_ns();
      unsigned int polls = 0;
      unsigned long long word;
      while (true) {
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(p) : "memory");
        if (static_cast<unsigned int>(word >> 32) == want) break;
        if ((++polls & 63u) == 0 && global_ns() - t0 > a.wait_ns) {
          atomicExch(a.status, sm100::kErrPeerWait);
          *failed = 1;
          break;
        }
      }
      recv[w][src] = __uint_as_float(static_cast<unsigned int>(word));
    }
    __syncthreads();
    seq = want;
    return *failed == 0;
  }
};

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = red[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
  __syncthreads();
  return m;
}

// three block sums at once (the quartile points of one search round)
__device__ __forceinline__ void block_sum3(float (&v)[3], float (*red3)[32]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 3; ++i) v[i] = warp_sum(v[i]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < 3; ++i) red3[i][warp] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red3[i][w];   // fixed order: same result in every thread
    v[i] = t;
  }
  __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(1024)
peer_sample_kernel(const PeerArgs a, const SampleArgs sa, const T* __restrict__ scores, long long row_stride,
                   int vocab_start, float logit_scale, long long* __restrict__ ids, float* __restrict__ logprob) {
  using tgi_sampling::gumbel_noise;
  using tgi_sampling::order_bits;
  __shared__ float red[32];
  __shared__ float red3[3][32];
  __shared__ float recv[kXWords][kMaxRanks];
  __shared__ float s_key[32], s_x[32];
  __shared__ int s_idx[32];
  __shared__ int failed;
  tgi::pdl_wait();
  tgi::pdl_trigger();
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  Exchange xc{a, sa.off_xchg, sa.xseq[blockIdx.x], &failed, recv};
  const int B = a.T, Vl = a.H;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  bool ok = true;

  for (int row = blockIdx.x; row < B && ok; row += gridDim.x) {
    const T* x_row = scores + static_cast<size_t>(row) * row_stride;
    const float temp = sa.temperature != nullptr ? sa.temperature[row] : 1.f;
    const float inv_t = logit_scale / (temp > 0.f ? temp : 1.f);
    auto val = [&](int i) { return static_cast<float>(x_row[i]) * inv_t; };
    auto sum_ranks = [&](int w) {
      float t = 0.f;
      for (int r = 0; r < a.world; ++r) t += recv[w][r];
      return t;
    };
    // ---- max over the whole vocabulary ----
    float m = -INFINITY;
    for (int i = threadIdx.x; i < Vl; i += blockDim.x) m = fmaxf(m, val(i));
    m = block_max(m, red);
    {
      const float v1[1] = {m};
      ok = xc.all_gather<1>(v1);
      if (!ok) break;
      for (int r = 0; r < a.world; ++r) m = fmaxf(m, recv[0][r]);
      __syncthreads();
    }
    // ---- thresholds: smallest t with  sum_{bits(x) > t, bits(x) >= floor} w(x) < limit  (w = 1 or exp(x - m)) ----
    uint32_t keep_from = 0u;
    auto search = [&](bool mass, float limit, uint32_t floor_bits) -> uint32_t {
      uint32_t lo = floor_bits, hi = order_bits(m);
      while (lo < hi && ok) {
        const uint32_t w = hi - lo;
        const uint32_t c[3] = {lo + (w >> 2), lo + (w >> 1), lo + (w >> 1) + (w >> 2)};   // lo <= c0 <= c1 <= c2 < hi
        float acc[3] = {0.f, 0.f, 0.f};
        for (int i = threadIdx.x; i < Vl; i += blockDim.x) {
          const float x = val(i);
          const uint32_t b = order_bits(x);
          if (b < floor_bits) continue;
          const float wgt = mass ? __expf(x - m) : 1.f;
#pragma unroll
          for (int q = 0; q < 3; ++q)
            if (b > c[q]) acc[q] += wgt;
        }
        block_sum3(acc, red3);
        ok = xc.all_gather<3>(acc);
        if (!ok) break;
        const float t0 = sum_ranks(0), t1 = sum_ranks(1), t2 = sum_ranks(2);
        __syncthreads();
        if (t0 < limit) hi = c[0];
        else if (t1 < limit) { lo = c[0] + 1; hi = c[1]; }
        else if (t2 < limit) { lo = c[1] + 1; hi = c[2]; }
        else lo = c[2] + 1;
      }
      return lo;
    };
    const int k = sa.top_k != nullptr ? sa.top_k[row] : 0;
    if (k > 0 && k < sa.vocab_total) keep_from = search(false, static_cast<float>(k), 0u);
    if (!ok) break;
    const float p = sa.top_p != nullptr ? sa.top_p[row] : 1.f;
    if (p < 1.f) {
      float z[1] = {0.f};
      for (int i = threadIdx.x; i < Vl; i += blockDim.x) {
        const float x = val(i);
        if (order_bits(x) >= keep_from) z[0] += __expf(x - m);
      }
      z[0] = block_sum(z[0], red);
      ok = xc.all_gather<1>(z);
      if (!ok) break;
      const float ztot = sum_ranks(0);
      __syncthreads();
      const uint32_t t = search(true, p * ztot, keep_from);
      if (!ok) break;
      keep_from = max(keep_from, t);
    }
    // ---- sample over the kept set ----
    const bool sample = sa.do_sample != nullptr && sa.do_sample[row] != 0;
    const uint64_t seed = sa.seeds != nullptr ? static_cast<uint64_t>(sa.seeds[row]) : 0ull;
    const uint32_t step = sa.steps != nullptr ? static_cast<uint32_t>(sa.steps[row]) : 0u;
    float z = 0.f, best = -INFINITY, best_x = 0.f;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < Vl; i += blockDim.x) {
      const float x = val(i);
      if (order_bits(x) < keep_from || x == -INFINITY) continue;
      z += __expf(x - m);
      const int gi = i + vocab_start;
      const float key = sample ? x + gumbel_noise(static_cast<uint32_t>(gi), step, seed) : x;
      if (key > best || (key == best && gi < best_i)) {
        best = key;
        best_i = gi;
        best_x = x;
      }
    }
    z = block_sum(z, red);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float k2 = __shfl_xor_sync(0xffffffffu, best, o);
      const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
      const float x2 = __shfl_xor_sync(0xffffffffu, best_x, o);
      if (k2 > best || (k2 == best && i2 < best_i)) {
        best = k2;
        best_i = i2;
        best_x = x2;
      }
    }
    __syncthreads();
    if (lane == 0) {
      s_key[warp] = best;
      s_idx[warp] = best_i;
      s_x[warp] = best_x;
    }
    __syncthreads();
    for (int w = 0; w < (blockDim.x >> 5); ++w)   // every thread folds the warps in the same order
      if (s_key[w] > best || (s_key[w] == best && s_idx[w] < best_i)) {
        best = s_key[w];
        best_i = s_idx[w];
        best_x = s_x[w];
      }
    __syncthreads();
    {
      const float v4[4] = {z, best, __int_as_float(best_i), best_x};
      ok = xc.all_gather<4>(v4);
      if (!ok) break;
      if (threadIdx.x == 0) {
        float zt = 0.f, bk = -INFINITY, bx = 0.f;
        int bi = 0x7fffffff;
        for (int r = 0; r < a.world; ++r) {
          zt += recv[0][r];
          const float kr = recv[1][r];
          const int ir = __float_as_int(recv[2][r]);
          if (kr > bk || (kr == bk && ir < bi)) {
            bk = kr;
            bi = ir;
            bx = recv[3][r];
          }
        }
        ids[row] = bi == 0x7fffffff ? 0 : bi;
        logprob[row] = bx - m - __logf(zt);
      }
      __syncthreads();
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) sa.xseq[blockIdx.x] = xc.seq;
}

template <bool NORM, bool QUANT>
int launch_reduce(const PeerArgs& a, int blocks, cudaStream_t stream) {
  const int nvec = a.H / 8;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  if (NORM && nvec > 1024)
    tgi::launch(peer_reduce_kernel<NORM, QUANT, 2>, dim3(blocks), dim3(threads), 0, stream, a);
  else
    tgi::launch(peer_reduce_kernel<NORM, QUANT, 1>, dim3(blocks), dim3(threads), 0, stream, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace

extern "C" {

// ---- heap management (set-up time only) ----------------------------------------------------
int tgi_peer_alloc(long long bytes, void** ptr) {
  if (cudaMalloc(ptr, static_cast<size_t>(bytes)) != cudaSuccess) return -1;
  if (cudaMemset(*ptr, 0, static_cast<size_t>(bytes)) != cudaSuccess) return -2;
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : -3;
}
int tgi_peer_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }
int tgi_peer_export(void* ptr, unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return -1;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
int tgi_peer_import(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  const cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
int tgi_peer_unmap(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }
int tgi_peer_max_blocks() { return kMaxBlocks; }
// Limit (nanoseconds) of the waits on peer flags for kernels launched from now on; returns the previous one.
unsigned long long tgi_peer_set_wait_ns(unsigned long long ns) {
  const unsigned long long old = g_peer_wait_ns;
  if (ns > 0) g_peer_wait_ns = ns;
  return old;
}

// ---- the collective --------------------------------------------------------------------------
// mode 0: all-reduce; 1: + residual + RMSNorm -> bf16; 2: + residual + RMSNorm + e4m3 quantisation.
int tgi_peer_reduce(void* const* heaps, int rank, int world, int T, int H, long long off_partial, long long off_gather,
                    long long off_gscale, int gscale_pitch, long long off_flags, unsigned int* epoch,
                    const void* residual_in, void* residual_out, const void* weight, float eps, float w_offset,
                    int mode, int blocks, int* status, int pushed, long long off_push_flags,
                    const unsigned int* push_epoch, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return -10;
  if (H % 8 != 0 || blocks < 1 || blocks > kMaxBlocks) return -11;
  if (mode != 0 && H > 16384) return -12;
  if (mode == 2 && H % 128 != 0) return -13;
  PeerArgs a;
  for (int i = 0; i < kMaxRanks; ++i) a.heap[i] = i < world ? static_cast<unsigned char*>(heaps[i]) : nullptr;
  a.rank = rank;
  a.world = world;
  a.T = T;
  a.H = H;
  a.off_partial = off_partial;
  a.off_gather = off_gather;
  a.off_gscale = off_gscale;
  a.gscale_pitch = gscale_pitch;
  a.off_flags = off_flags;
  a.epoch = epoch;
  a.residual_in = static_cast<const __nv_bfloat16*>(residual_in);
  a.residual_out = static_cast<__nv_bfloat16*>(residual_out);
  a.weight = static_cast<const __nv_bfloat16*>(weight);
  a.eps = eps;
  a.w_offset = w_offset;
  a.status = status;
  a.wait_ns = g_peer_wait_ns;
  a.pushed = pushed;
  a.off_push_flags = off_push_flags;
  a.push_epoch = push_epoch;
  if (pushed && push_epoch == nullptr) return -15;
  switch (mode) {
    case 0: return launch_reduce<false, false>(a, blocks, stream);
    case 1: return launch_reduce<true, false>(a, blocks, stream);
    case 2: return launch_reduce<true, true>(a, blocks, stream);
    default: return -14;
  }
}

// Greedy token and its log-probability from vocabulary-sharded logits: see peer_argmax_kernel.
int tgi_peer_argmax(void* const* heaps, int rank, int world, const void* logits, int B, int Vl, long long row_stride,
                    int vocab_start, float logit_scale, long long off_cand, long long off_flags, unsigned int* epoch,
                    long long* ids, float* logprob, int blocks, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return -10;
  if (blocks < 1 || blocks > kMaxBlocks) return -11;
  PeerArgs a;
  for (int i = 0; i < kMaxRanks; ++i) a.heap[i] = i < world ? static_cast<unsigned char*>(heaps[i]) : nullptr;
  a.rank = rank;
  a.world = world;
  a.T = B;
  a.H = Vl;
  a.off_partial = a.off_gather = a.off_gscale = 0;
  a.gscale_pitch = 0;
  a.off_flags = off_flags;
  a.epoch = epoch;
  a.residual_in = nullptr;
  a.residual_out = nullptr;
  a.weight = nullptr;
  a.eps = a.w_offset = 0.f;
  a.status = status;
  a.wait_ns = g_peer_wait_ns;
  a.pushed = 0;
  a.off_push_flags = 0;
  a.push_epoch = nullptr;
  tgi::launch(peer_argmax_kernel, dim3(blocks), dim3(1024), 0, stream, a, static_cast<const __nv_bfloat16*>(logits),
              row_stride, vocab_start, logit_scale, off_cand, ids, logprob);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Vocabulary-parallel sampling (temperature, top-k, top-p, seeded Gumbel-max or arg-max, log-probability) on the
// rank's slice `scores` [B, Vl] (bf16 logits, or fp32 scores that already carry the penalties); see
// peer_sample_kernel.  Per-row parameter arrays may be null (stage off).  Every rank gets the same ids.
int tgi_peer_sample(void* const* heaps, int rank, int world, const void* scores, int is_fp32, int B, int Vl,
                    long long row_stride, int vocab_start, int vocab_total, float logit_scale, const float* temperature,
                    const int* top_k, const float* top_p, const unsigned char* do_sample, const long long* seeds,
                    const int* steps, long long off_xchg, unsigned int* xseq, long long* ids, float* logprob, int blocks,
                    int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return -10;
  if (blocks < 1 || blocks > kMaxBlocks) return -11;
  PeerArgs a;
  for (int i = 0; i < kMaxRanks; ++i) a.heap[i] = i < world ? static_cast<unsigned char*>(heaps[i]) : nullptr;
  a.rank = rank;
  a.world = world;
  a.T = B;
  a.H = Vl;
  a.off_partial = a.off_gather = a.off_gscale = 0;
  a.gscale_pitch = 0;
  a.off_flags = 0;
  a.epoch = nullptr;
  a.residual_in = nullptr;
  a.residual_out = nullptr;
  a.weight = nullptr;
  a.eps = a.w_offset = 0.f;
  a.status = status;
  a.wait_ns = g_peer_wait_ns;
  a.pushed = 0;
  a.off_push_flags = 0;
  a.push_epoch = nullptr;
  SampleArgs sa;
  sa.temperature = temperature;
  sa.top_k = top_k;
  sa.top_p = top_p;
  sa.do_sample = do_sample;
  sa.seeds = seeds;
  sa.steps = steps;
  sa.off_xchg = off_xchg;
  sa.xseq = xseq;
  sa.vocab_total = vocab_total;
  if (is_fp32)
    tgi::launch(peer_sample_kernel<float>, dim3(blocks), dim3(1024), 0, stream, a, sa, static_cast<const float*>(scores),
                row_stride, vocab_start, logit_scale, ids, logprob);
  else
    tgi::launch(peer_sample_kernel<__nv_bfloat16>, dim3(blocks), dim3(1024), 0, stream, a, sa,
                static_cast<const __nv_bfloat16*>(scores), row_stride, vocab_start, logit_scale, ids, logprob);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// bytes of the exchange region that tgi_peer_sample needs in every heap
long long tgi_peer_sample_xchg_bytes() { return static_cast<long long>(kMaxBlocks) * 2 * kXWords * kMaxRanks * 8; }

}  // extern "C"

extern "C" int tgi_peer_set_quant_pow2(int on) {
  const int v = on != 0;
  return cudaMemcpyToSymbol(g_quant_pow2, &v, sizeof(v)) == cudaSuccess ? 0 : -3;
}

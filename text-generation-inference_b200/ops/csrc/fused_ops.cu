// Bandwidth-bound fused kernels of the decoder layer (sm_100a):
//   rms_norm / layer_norm with residual add, optional 1x128 e4m3 quantisation of the output
//   RoPE + paged KV-cache store (bf16 or e4m3 with per-head scale)
//   act(gate) * up, optional quantisation
//   dynamic 1x128 e4m3 activation quantisation
//   embedding gather, greedy argmax + log-probability
//
// They replace, in the reference: `dropout_layer_norm.dropout_add_ln_fwd` (layers/layernorm.py:161-187),
// `rotary.apply_rotary` x2 + `KVCache.store` (layers/rotary.py:54-64, layers/attention/kv_cache.py:184-240),
// the separate SiLU and multiply torch ops (flash_llama_modeling.py:400-404), `scaled_fp8_quant` /
// `per_token_group_quant_fp8` (layers/fp8.py:149-159, 508-526), `F.embedding`, and the
// log_softmax + argmax pair of the greedy sampler (utils/tokens.py).
//
// Activation scales are written K-block major, `scale_t[kb * pitch + token]`, the layout the
// block-scaled GEMM fetches with one TMA box per K block.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sampling.cuh"
#include "launch.cuh"

namespace {

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

struct __align__(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16(x)); }

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

// 8 fp32 -> 8 e4m3 (two 32-bit words)
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

// amax over the 16 lanes that share one 128-element group (8 elements per lane)
__device__ __forceinline__ float group16_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ------------------------------------------------------------------------------------------------
// residual add + RMSNorm / LayerNorm (+ quant).  One CTA per token; VPT 16-byte vectors per thread.
// ------------------------------------------------------------------------------------------------
template <int VPT, bool LAYER, bool QUANT>
__global__ void __launch_bounds__(1024)
norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
            const __nv_bfloat16* __restrict__ weight, const __nv_bfloat16* __restrict__ bias,
            __nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ res_out, uint8_t* __restrict__ q_out,
            float* __restrict__ scale_t, int scale_pitch, int H, float eps, float w_offset) {
  tgi::pdl_wait();      // inputs come from earlier kernels of the stream
  tgi::pdl_trigger();   // let the next kernel be placed while this one runs
  __shared__ float red[32];
  const int row = blockIdx.x;
  const size_t base = static_cast<size_t>(row) * H;
  const int nvec = H / 8;
  float s[VPT][8];
  float sum = 0.f, sumsq = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float a[8];
      unpack8(*reinterpret_cast<const bf16x8*>(x + base + v * 8), a);
      if (residual != nullptr) {
        float r[8];
        unpack8(*reinterpret_cast<const bf16x8*>(residual + base + v * 8), r);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = round_bf16(a[j] + r[j]);
      }
      if (res_out != nullptr) *reinterpret_cast<bf16x8*>(res_out + base + v * 8) = pack8(a);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[i][j] = a[j];
        sum += a[j];
        sumsq += a[j] * a[j];
      }
    }
  }
  float mean = 0.f;
  float var;
  if (LAYER) {
    mean = block_sum(sum, red) / H;
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) d += (s[i][j] - mean) * (s[i][j] - mean);
      }
    }
    var = block_sum(d, red) / H;
  } else {
    var = block_sum(sumsq, red) / H;
  }
  const float rstd = rsqrtf(var + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    const bool active = v < nvec;
    float y[8];
    if (active) {
      float w[8];
      unpack8(*reinterpret_cast<const bf16x8*>(weight + v * 8), w);
      float b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (LAYER && bias != nullptr) unpack8(*reinterpret_cast<const bf16x8*>(bias + v * 8), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = round_bf16((s[i][j] - mean) * rstd * (w[j] + w_offset) + b[j]);
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
        *reinterpret_cast<uint2*>(q_out + base + v * 8) = quant8(y, scale);
        if ((v & 15) == 0) scale_t[static_cast<size_t>(v >> 4) * scale_pitch + row] = scale;
      }
    } else if (active) {
      *reinterpret_cast<bf16x8*>(out + base + v * 8) = pack8(y);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// act(gate) * up (+ quant): in [T, 2I] -> out [T, I]
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float act_fn(float x, int act) {
  switch (act) {
    case 0: return __fdividef(x, 1.f + __expf(-x));                                     // silu (fast division)
    case 1: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));                   // gelu (erf)
    case 2: {                                                                           // gelu (tanh)
      const float k = 0.7978845608028654f;
      return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
    }
    case 3: return fmaxf(x, 0.f);                                                       // relu
    default: return x / (1.f + __expf(-1.702f * x));                                    // quick gelu
  }
}

// NV 16-byte vectors (8 elements each) of gate and of up per thread; a 128-element quantisation group is spread
// over 16 / NV lanes.  NV = 2 halves the per-element index / shuffle overhead (the kernel is instruction bound).
template <bool QUANT, int NV>
__global__ void __launch_bounds__(256)
act_mul_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, uint8_t* __restrict__ q_out,
               float* __restrict__ scale_t, int scale_pitch, int I, int act) {
  tgi::pdl_wait();      // inputs come from earlier kernels of the stream
  tgi::pdl_trigger();   // let the next kernel be placed while this one runs
  constexpr int E = 8 * NV;            // elements per thread
  constexpr int LANES = 128 / E;       // lanes per quantisation group
  const int row = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = v < I / E;
  float y[NV][8];
  if (active) {
    const __nv_bfloat16* p = in + static_cast<size_t>(row) * 2 * I + static_cast<size_t>(v) * E;
    bf16x8 gv[NV], uv[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      gv[k] = *reinterpret_cast<const bf16x8*>(p + k * 8);
      uv[k] = *reinterpret_cast<const bf16x8*>(p + I + k * 8);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float g[8], u[8];
      unpack8(gv[k], g);
      unpack8(uv[k], u);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[k][j] = round_bf16(act_fn(g[j], act) * u[j]);
    }
  } else {
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) y[k][j] = 0.f;
  }
  if (QUANT) {
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(y[k][j]));
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = block_scale(amax);
    if (active) {
      uint8_t* q = q_out + static_cast<size_t>(row) * I + static_cast<size_t>(v) * E;
      if (NV == 2) {
        const uint2 lo = quant8(y[0], scale), hi = quant8(y[NV - 1], scale);
        *reinterpret_cast<uint4*>(q) = make_uint4(lo.x, lo.y, hi.x, hi.y);
      } else {
        *reinterpret_cast<uint2*>(q) = quant8(y[0], scale);
      }
      if ((v & (LANES - 1)) == 0) scale_t[static_cast<size_t>(v / LANES) * scale_pitch + row] = scale;
    }
  } else if (active) {
    __nv_bfloat16* o = out + static_cast<size_t>(row) * I + static_cast<size_t>(v) * E;
#pragma unroll
    for (int k = 0; k < NV; ++k) *reinterpret_cast<bf16x8*>(o + k * 8) = pack8(y[k]);
  }
}

// dynamic 1x128 quantisation of x[T, K]
__global__ void __launch_bounds__(256)
quant_act_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q_out, float* __restrict__ scale_t,
                 int scale_pitch, int K) {
  tgi::pdl_wait();      // inputs come from earlier kernels of the stream
  tgi::pdl_trigger();   // let the next kernel be placed while this one runs
  const int row = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = v < K / 8;
  float y[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (active) unpack8(*reinterpret_cast<const bf16x8*>(x + static_cast<size_t>(row) * K + v * 8), y);
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(y[j]));
  amax = group16_max(amax);
  const float scale = block_scale(amax);
  if (active) {
    *reinterpret_cast<uint2*>(q_out + static_cast<size_t>(row) * K + v * 8) = quant8(y, scale);
    if ((v & 15) == 0) scale_t[static_cast<size_t>(v >> 4) * scale_pitch + row] = scale;
  }
}

// ------------------------------------------------------------------------------------------------
// RoPE + KV store.  grid = tokens, block = 256 threads looping over (head, pair) work items.
// qkv[T, (Hq + 2 Hkv) * D] -> q_out[T, Hq, D] (rotated), k/v written at `slots` of the paged cache.
// ------------------------------------------------------------------------------------------------
template <bool FP8_CACHE>
__global__ void __launch_bounds__(256)
rope_cache_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                  const float* __restrict__ cos_sin, const int* __restrict__ slots, __nv_bfloat16* __restrict__ q_out,
                  void* __restrict__ k_cache, void* __restrict__ v_cache, const float* __restrict__ k_scale,
                  const float* __restrict__ v_scale, int Hq, int Hkv, int D, int rot, int neox, long long num_slots,
                  int max_pos) {
  tgi::pdl_wait();      // inputs come from earlier kernels of the stream
  tgi::pdl_trigger();   // let the next kernel be placed while this one runs
  const int t = blockIdx.x;
  // a position beyond the rotary table (operator asked for more tokens than the model supports) reads
  // the table's last row instead of running off its end
  const int pos = min(max(positions[t], 0), max_pos - 1);
  const long long slot = slots[t];
  const __nv_bfloat16* src = qkv + static_cast<size_t>(t) * (Hq + 2 * Hkv) * D;
  const float* cs = cos_sin + static_cast<size_t>(pos) * rot;
  const int half = D / 2;         // work items per head: D/2 element pairs
  const int rh = rot / 2;
  const int total = (Hq + 2 * Hkv) * half;
  const bool slot_ok = slot >= 0 && slot < num_slots;   // self-check: never write outside the cache
  for (int w = threadIdx.x; w < total; w += blockDim.x) {
    const int h = w / half, p = w % half;
    // element indices of the pair handled by this work item
    int i0, i1;
    bool rotate;
    if (neox) {
      // pairs (p, p + rot/2) for p < rot/2; the un-rotated tail is handled as plain copies
      if (p < rh) { i0 = p; i1 = p + rh; rotate = true; }
      else { i0 = rot + 2 * (p - rh); i1 = i0 + 1; rotate = false; }
    } else {
      i0 = 2 * p; i1 = 2 * p + 1; rotate = (i1 < rot);
    }
    float x0 = __bfloat162float(src[h * D + i0]);
    float x1 = __bfloat162float(src[h * D + i1]);
    if (h < Hq + Hkv && rotate) {
      const int f = p;   // frequency index
      const float c = cs[f], s = cs[rh + f];
      const float r0 = x0 * c - x1 * s;
      const float r1 = x1 * c + x0 * s;
      x0 = r0;
      x1 = r1;
    }
    if (h < Hq) {
      __nv_bfloat16* q = q_out + (static_cast<size_t>(t) * Hq + h) * D;
      q[i0] = __float2bfloat16(x0);
      q[i1] = __float2bfloat16(x1);
    } else if (slot_ok) {
      const bool is_k = h < Hq + Hkv;
      const int kvh = is_k ? h - Hq : h - Hq - Hkv;
      const size_t off = (static_cast<size_t>(slot) * Hkv + kvh) * D;
      if (FP8_CACHE) {
        const float* sc = is_k ? k_scale : v_scale;
        const float scv = sc != nullptr ? sc[kvh] : 1.f;
        // rotate in bf16 precision first (what a bf16 cache would hold), then quantise
        x0 = round_bf16(x0);
        x1 = round_bf16(x1);
        uint8_t* dst = static_cast<uint8_t*>(is_k ? k_cache : v_cache) + off;
        dst[i0] = static_cast<uint8_t>(
            __nv_cvt_float_to_fp8(fminf(fmaxf(x0 / scv, -kFp8Max), kFp8Max), __NV_SATFINITE, __NV_E4M3));
        dst[i1] = static_cast<uint8_t>(
            __nv_cvt_float_to_fp8(fminf(fmaxf(x1 / scv, -kFp8Max), kFp8Max), __NV_SATFINITE, __NV_E4M3));
      } else {
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(is_k ? k_cache : v_cache) + off;
        dst[i0] = __float2bfloat16(x0);
        dst[i1] = __float2bfloat16(x1);
      }
    }
  }
}

// Vector form for the common layout (NeoX halves, rotary over the whole head, D a multiple of 16): a work
// item is 8 consecutive elements of the first half of a head together with their partners in the
// second half, so every access is 16 bytes (8 bytes into an e4m3 cache) and the table rows are read
// as float4.  Same arithmetic, element by element, as the scalar kernel above.
template <bool FP8_CACHE>
__global__ void __launch_bounds__(128)
rope_cache_vec_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                      const float* __restrict__ cos_sin, const int* __restrict__ slots,
                      __nv_bfloat16* __restrict__ q_out, void* __restrict__ k_cache, void* __restrict__ v_cache,
                      const float* __restrict__ k_scale, const float* __restrict__ v_scale, int Hq, int Hkv, int D,
                      long long num_slots, int max_pos) {
  tgi::pdl_wait();
  tgi::pdl_trigger();
  const int t = blockIdx.x;
  const int pos = min(max(positions[t], 0), max_pos - 1);
  const long long slot = slots[t];
  const bool slot_ok = slot >= 0 && slot < num_slots;   // self-check: never write outside the cache
  const __nv_bfloat16* src = qkv + static_cast<size_t>(t) * (Hq + 2 * Hkv) * D;
  const float* cs = cos_sin + static_cast<size_t>(pos) * D;
  const int half = D / 2;
  const int per_head = D / 16;
  const int total = (Hq + 2 * Hkv) * per_head;
  for (int w = threadIdx.x; w < total; w += blockDim.x) {
    const int h = w / per_head, c = w - h * per_head;
    float a[8], b[8];
    unpack8(*reinterpret_cast<const bf16x8*>(src + h * D + 8 * c), a);
    unpack8(*reinterpret_cast<const bf16x8*>(src + h * D + half + 8 * c), b);
    if (h < Hq + Hkv) {
      const float4 c0 = *reinterpret_cast<const float4*>(cs + 8 * c), c1 = *reinterpret_cast<const float4*>(cs + 8 * c + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(cs + half + 8 * c);
      const float4 s1 = *reinterpret_cast<const float4*>(cs + half + 8 * c + 4);
      const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float r0 = a[j] * cc[j] - b[j] * ss[j];
        const float r1 = b[j] * cc[j] + a[j] * ss[j];
        a[j] = r0;
        b[j] = r1;
      }
    }
    if (h < Hq) {
      __nv_bfloat16* q = q_out + (static_cast<size_t>(t) * Hq + h) * D;
      *reinterpret_cast<bf16x8*>(q + 8 * c) = pack8(a);
      *reinterpret_cast<bf16x8*>(q + half + 8 * c) = pack8(b);
    } else if (slot_ok) {
      const bool is_k = h < Hq + Hkv;
      const int kvh = is_k ? h - Hq : h - Hq - Hkv;
      const size_t off = (static_cast<size_t>(slot) * Hkv + kvh) * D;
      if (FP8_CACHE) {
        const float* sc = is_k ? k_scale : v_scale;
        const float scv = sc != nullptr ? sc[kvh] : 1.f;
        __align__(8) uint8_t qa[8];
        __align__(8) uint8_t qb[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // rotate in bf16 precision first (what a bf16 cache would hold), then quantise
          qa[j] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(
              fminf(fmaxf(round_bf16(a[j]) / scv, -kFp8Max), kFp8Max), __NV_SATFINITE, __NV_E4M3));
          qb[j] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(
              fminf(fmaxf(round_bf16(b[j]) / scv, -kFp8Max), kFp8Max), __NV_SATFINITE, __NV_E4M3));
        }
        uint8_t* dst = static_cast<uint8_t*>(is_k ? k_cache : v_cache) + off;
        *reinterpret_cast<uint2*>(dst + 8 * c) = *reinterpret_cast<const uint2*>(qa);
        *reinterpret_cast<uint2*>(dst + half + 8 * c) = *reinterpret_cast<const uint2*>(qb);
      } else {
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(is_k ? k_cache : v_cache) + off;
        *reinterpret_cast<bf16x8*>(dst + 8 * c) = pack8(a);
        *reinterpret_cast<bf16x8*>(dst + half + 8 * c) = pack8(b);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, __nv_bfloat16* __restrict__ out,
                 int H, int rows) {
  tgi::pdl_wait();      // inputs come from earlier kernels of the stream
  tgi::pdl_trigger();   // let the next kernel be placed while this one runs
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= rows) id = rows - 1;  // self-check: clamp instead of reading out of bounds
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) dst[v] = src[v];
}

// greedy: ids[b] = argmax(logits[b]), logprob[b] = log_softmax(logits[b])[ids[b]]
template <typename T>
__global__ void __launch_bounds__(1024)
argmax_logprob_kernel(const T* __restrict__ logits, long long* __restrict__ ids, float* __restrict__ logprob, int V,
                      long long row_stride) {
  tgi::pdl_wait();      // inputs come from earlier kernels of the stream
  tgi::pdl_trigger();   // let the next kernel be placed while this one runs
  __shared__ float s_m[32], s_s[32];
  __shared__ int s_i[32];
  const T* row = logits + static_cast<size_t>(blockIdx.x) * row_stride;
  float m = -INFINITY, s = 0.f;
  int best = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float x = static_cast<float>(row[i]);
    if (x > m) {
      s = s * __expf(m - x) + 1.f;
      m = x;
      best = i;
    } else {
      s += __expf(x - m);
    }
  }
  // merge (m, s, best) across the block; ties resolve to the smallest index like torch.argmax
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const int b2 = __shfl_xor_sync(0xffffffffu, best, o);
    const float mm = fmaxf(m, m2);
    const float ns = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
    if (m2 > m || (m2 == m && b2 < best)) best = b2;
    m = mm;
    s = ns;
  }
  if (lane == 0) { s_m[warp] = m; s_s[warp] = s; s_i[warp] = best; }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) / 32;
    m = lane < nw ? s_m[lane] : -INFINITY;
    s = lane < nw ? s_s[lane] : 0.f;
    best = lane < nw ? s_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      const int b2 = __shfl_xor_sync(0xffffffffu, best, o);
      const float mm = fmaxf(m, m2);
      const float ns = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
      if (m2 > m || (m2 == m && b2 < best)) best = b2;
      m = mm;
      s = ns;
    }
    if (lane == 0) {
      ids[blockIdx.x] = best;
      logprob[blockIdx.x] = -logf(s);
    }
  }
}


// ------------------------------------------------------------------------------------------------
// Fused sampler: temperature, top-k, top-p, Gumbel-max sampling (or argmax) and the log-probability of
// the chosen token, one CTA per row.  Replaces the reference's chain of logits warpers and its
// `probs / Exp(1)` multinomial with a CPU generator per request (utils/tokens.py:346-399,
// utils/logits_process.py:25-358): no sort, no [B, V] probability matrix, no host round trip.
//
//   x_j = logit_j / T
//   top-k: keep x_j >= (k-th largest x);  top-p: keep x_j unless the mass of strictly larger entries
//   already reaches p (same sets as the sort-based torch filters).  Both thresholds are found by
//   bisection on the order-preserving integer image of the float, which is exact and needs no sort.
//   sample: argmax_j (x_j + g_j) over the kept set, g_j = -log(-log u_j), u_j from Philox4x32-10
//   keyed by the request's seed with counter (j, step): reproducible for a given seed.
//   logprob = x_c - logsumexp over the kept set.
// ------------------------------------------------------------------------------------------------
using tgi_sampling::gumbel_noise;
using tgi_sampling::order_bits;

// Calls f(index, score / T) for every entry of a row, the CTA's threads striding over it; 16-byte loads where the
// row allows it (8 bf16 or 4 fp32 per thread and step).
template <typename T, typename F>
__device__ __forceinline__ void scan_row(const T* __restrict__ row, int V, float inv_t, F&& f) {
  constexpr int VEC = 16 / sizeof(T);
  const int nvec = (reinterpret_cast<uintptr_t>(row) & 15) == 0 ? V / VEC : 0;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(row)[v];
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < VEC; ++j) f(v * VEC + j, static_cast<float>(e[j]) * inv_t);
  }
  for (int i = nvec * VEC + threadIdx.x; i < V; i += blockDim.x) f(i, static_cast<float>(row[i]) * inv_t);
}

// smallest order_bits threshold t such that  sum_{x : bits(x) > t} w(x) < limit   (w = 1 or exp(x - m)),
// not below floor_bits and not above the bits of the row maximum.
// Radix select over the four bytes of the ordered bits, most significant first: one pass over the row per byte
// builds a 256-bin histogram of the weights of the entries that match the bytes found so far, and a walk down
// the bins finds the byte of t (the lowest bin whose entries can still be left out).  Five passes replace the
// 32 of a bisection.  Weights are accumulated as 2^-40 fixed point in 64-bit integers, so the sums do not depend
// on the order in which the lanes' atomics land: the same row always yields the same threshold.
constexpr int kHistCopies = 16;          // one histogram per pair of warps (1024 threads)
constexpr float kFixedOne = 1099511627776.f;   // 2^40

template <typename T, bool MASS>
__device__ uint32_t find_threshold(const T* __restrict__ row, int V, float inv_t, float m, float limit, uint32_t floor_bits,
                                   unsigned long long* hist, unsigned long long* tot) {
  const unsigned long long lim = MASS ? static_cast<unsigned long long>(fmaxf(limit, 0.f) * kFixedOne)
                                      : static_cast<unsigned long long>(fmaxf(limit, 0.f));
  const int copy = (threadIdx.x >> 5) % kHistCopies;
  uint32_t prefix = 0u;
  unsigned long long above = 0ull;         // weight of the entries whose leading bytes exceed the prefix
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < kHistCopies * 256; i += blockDim.x) hist[i] = 0ull;
    __syncthreads();
    const uint32_t hi_mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    unsigned int* hist32 = reinterpret_cast<unsigned int*>(hist);      // counts fit 32 bits: the cheaper atomic
    scan_row(row, V, inv_t, [&](int, float x) {
      const uint32_t b = order_bits(x);
      if (b >= floor_bits && (b & hi_mask) == prefix) {
        if (MASS) atomicAdd(&hist[copy * 256 + ((b >> shift) & 255u)], static_cast<unsigned long long>(__expf(x - m) * kFixedOne));
        else atomicAdd(&hist32[copy * 256 + ((b >> shift) & 255u)], 1u);
      }
    });
    __syncthreads();
    if (threadIdx.x < 256) {
      unsigned long long t = 0ull;
#pragma unroll
      for (int c = 0; c < kHistCopies; ++c)
        t += MASS ? hist[c * 256 + threadIdx.x] : static_cast<unsigned long long>(reinterpret_cast<unsigned int*>(hist)[c * 256 + threadIdx.x]);
      tot[threadIdx.x] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      // S(v) = above + sum of the bins over v is the weight left out when t ends in bin v; S(255) < lim holds on
      // entry, and going one bin down adds that bin: stop before the sum would reach lim
      unsigned long long run = above;
      int v = 255;
      while (v > 0 && run + tot[v] < lim) {
        run += tot[v];
        --v;
      }
      tot[256] = run;
      tot[257] = static_cast<unsigned long long>(v);
    }
    __syncthreads();
    above = tot[256];
    prefix |= static_cast<uint32_t>(tot[257]) << shift;
    __syncthreads();
  }
  return max(min(prefix, order_bits(m)), floor_bits);
}

// Typical-p (utils/logits_process.py:389-448): over the entries the earlier filters kept, with p_j their
// renormalised probabilities and H their entropy, keep the entries with the smallest |-log p_j - H| whose mass
// reaches `mass`.  Returns the largest kept deviation as float bits (deviations are >= 0, so their bit patterns
// order like the values); found by bisection, no sort.
template <typename T>
__device__ uint32_t typical_threshold(const T* __restrict__ row, int V, float inv_t, float m, uint32_t keep_from, float mass,
                                      float* red, float* log_z_out, float* entropy_out) {
  float z = 0.f;
  scan_row(row, V, inv_t, [&](int, float x) {
    if (order_bits(x) >= keep_from && x != -INFINITY) z += __expf(x - m);
  });
  const float log_z = __logf(block_sum(z, red));
  float h = 0.f;
  scan_row(row, V, inv_t, [&](int, float x) {
    if (order_bits(x) >= keep_from && x != -INFINITY) {
      const float lp = x - m - log_z;
      h -= __expf(lp) * lp;
    }
  });
  const float H = block_sum(h, red);
  *log_z_out = log_z;
  *entropy_out = H;
  uint32_t lo = 0u, hi = 0x7f800000u;       // predicate "mass of deviations <= t reaches `mass`": true at +inf
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    float acc = 0.f;
    scan_row(row, V, inv_t, [&](int, float x) {
      if (order_bits(x) >= keep_from && x != -INFINITY) {
        const float lp = x - m - log_z;
        if (__float_as_uint(fabsf(-lp - H)) <= mid) acc += __expf(lp);
      }
    });
    if (block_sum(acc, red) >= mass) hi = mid;
    else lo = mid + 1;
  }
  return lo;
}

template <typename T>
__global__ void __launch_bounds__(1024)
sample_kernel(const T* __restrict__ scores, long long row_stride, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ typical_p,
              const unsigned char* __restrict__ do_sample,
              const long long* __restrict__ seeds, const int* __restrict__ steps, long long* __restrict__ ids,
              float* __restrict__ logprob, int V) {
  tgi::pdl_wait();      // inputs come from earlier kernels of the stream
  tgi::pdl_trigger();   // let the next kernel be placed while this one runs
  __shared__ float red[32];
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ unsigned long long s_hist[kHistCopies * 256];
  __shared__ unsigned long long s_tot[258];
  const int b = blockIdx.x;
  const T* row = scores + static_cast<size_t>(b) * row_stride;
  const float temp = temperature != nullptr ? temperature[b] : 1.f;
  const float inv_t = 1.f / (temp > 0.f ? temp : 1.f);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // ---- max ----
  float m = -INFINITY;
  scan_row(row, V, inv_t, [&](int, float x) { m = fmaxf(m, x); });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __syncthreads();
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = red[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
  __syncthreads();
  // ---- thresholds ----
  uint32_t keep_from = 0u;                      // keep entries whose order_bits >= keep_from
  const int k = top_k != nullptr ? top_k[b] : 0;
  if (k > 0 && k < V) keep_from = find_threshold<T, false>(row, V, inv_t, m, static_cast<float>(k), 0u, s_hist, s_tot);
  const float p = top_p != nullptr ? top_p[b] : 1.f;
  if (p < 1.f) {
    float z = 0.f;
    scan_row(row, V, inv_t, [&](int, float x) {
      if (order_bits(x) >= keep_from) z += __expf(x - m);
    });
    z = block_sum(z, red);
    const uint32_t t = find_threshold<T, true>(row, V, inv_t, m, p * z, keep_from, s_hist, s_tot);
    keep_from = max(keep_from, t);
  }
  const float typ = typical_p != nullptr ? typical_p[b] : 1.f;
  uint32_t typ_bits = 0xffffffffu;
  float typ_log_z = 0.f, typ_h = 0.f;
  if (typ < 1.f) typ_bits = typical_threshold<T>(row, V, inv_t, m, keep_from, typ, red, &typ_log_z, &typ_h);
  // ---- sample over the kept set ----
  const bool sample = do_sample != nullptr && do_sample[b] != 0;
  const uint64_t seed = seeds != nullptr ? static_cast<uint64_t>(seeds[b]) : 0ull;
  const uint32_t step = steps != nullptr ? static_cast<uint32_t>(steps[b]) : 0u;
  float z = 0.f, best = -INFINITY, best_x = 0.f;
  int best_i = 0x7fffffff;
  scan_row(row, V, inv_t, [&](int i, float x) {
    if (order_bits(x) < keep_from || x == -INFINITY) return;
    if (typ < 1.f && __float_as_uint(fabsf(-(x - m - typ_log_z) - typ_h)) > typ_bits) return;
    z += __expf(x - m);
    const float key = sample ? x + gumbel_noise(static_cast<uint32_t>(i), step, seed) : x;
    if (key > best || (key == best && i < best_i)) {
      best = key;
      best_i = i;
      best_x = x;
    }
  });
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
    red[warp] = best;
    s_idx[warp] = best_i;
    s_val[warp] = best_x;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w)
      if (red[w] > best || (red[w] == best && s_idx[w] < best_i)) {
        best = red[w];
        best_i = s_idx[w];
        best_x = s_val[w];
      }
    ids[b] = best_i == 0x7fffffff ? 0 : best_i;
    logprob[b] = best_x - m - __logf(z);
  }
}

// ------------------------------------------------------------------------------------------------
// Repetition and frequency penalties on fp32 scores, in place, one CTA per row, from the row's token history
// (reference: utils/logits_process.py:151-218).  `scores` may be a vocabulary slice [vocab_start,
// vocab_start + V): ids outside the slice are skipped.  Repetition: every token of the history gets
// score * p when negative, else score / p, once however often it occurs (the value is computed from the
// untouched `logits`, so duplicates write the same number).  Frequency: score -= p * occurrences.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(1024)
penalties_kernel(const T* __restrict__ logits, long long in_stride, float* __restrict__ scores, long long out_stride,
                 const long long* __restrict__ history, int L, const float* __restrict__ rep, const float* __restrict__ freq,
                 int vocab_start, int V, float logit_scale) {
  tgi::pdl_wait();
  const int b = blockIdx.x;
  const T* in = logits + static_cast<size_t>(b) * in_stride;
  float* out = scores + static_cast<size_t>(b) * out_stride;
  {
    // the copy is the bulk of the kernel: 16-byte loads, 16-byte stores where both rows allow it
    constexpr int VEC = 16 / sizeof(T);
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const int nvec = aligned ? V / VEC : 0;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 raw = reinterpret_cast<const uint4*>(in)[v];
      const T* e = reinterpret_cast<const T*>(&raw);
      float f[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) f[j] = static_cast<float>(e[j]) * logit_scale;
#pragma unroll
      for (int j = 0; j < VEC; j += 4)
        reinterpret_cast<float4*>(out + static_cast<size_t>(v) * VEC)[j >> 2] = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
    }
    for (int i = nvec * VEC + threadIdx.x; i < V; i += blockDim.x) out[i] = static_cast<float>(in[i]) * logit_scale;
  }
  __syncthreads();
  const long long* h = history + static_cast<size_t>(b) * L;
  const float rp = rep != nullptr ? rep[b] : 1.f;
  if (rp != 1.f) {
    for (int l = threadIdx.x; l < L; l += blockDim.x) {
      const long long t = h[l] - vocab_start;
      if (t < 0 || t >= V) continue;
      const float x = static_cast<float>(in[t]) * logit_scale;
      out[t] = x < 0.f ? x * rp : x / rp;
    }
    __syncthreads();
  }
  const float fp = freq != nullptr ? freq[b] : 0.f;
  if (fp != 0.f) {
    for (int l = threadIdx.x; l < L; l += blockDim.x) {
      const long long t = h[l] - vocab_start;
      if (t < 0 || t >= V) continue;
      atomicAdd(&out[t], -fp);
    }
  }
}


// Per-head normalisation of the q and k heads of a fused qkv row, in place (Qwen3, Gemma-3, OLMoE-style RMSNorm
// over head_dim; Cohere-style LayerNorm without bias).  One warp per (token, head); the weight is [D] shared by all
// heads (head_stride 0) or [heads, D].  Replaces, in the reference, the q_norm / k_norm modules applied to the
// reshaped projections (custom_modeling/flash_qwen3_modeling.py, flash_gemma3_modeling.py, flash_cohere_modeling.py).
__global__ void __launch_bounds__(256) qk_norm_kernel(__nv_bfloat16* qkv, long long row_stride, int T, int nh, int nkv, int D,
                                                      const __nv_bfloat16* qw, const __nv_bfloat16* kw, int q_head_stride,
                                                      int k_head_stride, float eps, float w_offset, int layer) {
  tgi::pdl_wait();
  tgi::pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long unit = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int heads = nh + nkv;
  if (unit >= static_cast<long long>(T) * heads) return;
  const int t = static_cast<int>(unit / heads), hd = static_cast<int>(unit % heads);
  const bool is_q = hd < nh;
  __nv_bfloat162* row = reinterpret_cast<__nv_bfloat162*>(qkv + t * row_stride + static_cast<long long>(hd) * D);
  const __nv_bfloat16* w = is_q ? qw + static_cast<long long>(hd) * q_head_stride : kw + static_cast<long long>(hd - nh) * k_head_stride;
  const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(w);
  const int pairs = D >> 1;
  float2 v[4];                      // D <= 256
  float sum = 0.f, sq = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int p = lane + i * 32;
    v[i] = p < pairs ? __bfloat1622float2(row[p]) : make_float2(0.f, 0.f);
    sum += v[i].x + v[i].y;
    sq += v[i].x * v[i].x + v[i].y * v[i].y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
  }
  const float mean = layer ? sum / D : 0.f;
  const float var = layer ? fmaxf(sq / D - mean * mean, 0.f) : sq / D;
  const float inv = rsqrtf(var + eps);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int p = lane + i * 32;
    if (p < pairs) {
      const float2 g = __bfloat1622float2(w2[p]);
      row[p] = __floats2bfloat162_rn((v[i].x - mean) * inv * (g.x + w_offset), (v[i].y - mean) * inv * (g.y + w_offset));
    }
  }
}

}  // namespace

extern "C" {

// qkv bf16 [T, row_stride]: heads 0..nh-1 are q, nh..nh+nkv-1 are k, each D wide; weights bf16
int tgi_qk_norm(void* qkv, long long row_stride, int T, int nh, int nkv, int D, const void* qw, const void* kw,
                int q_head_stride, int k_head_stride, float eps, float w_offset, int layer, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D % 2 != 0 || D > 256 || row_stride % 2 != 0) return -10;
  const long long units = static_cast<long long>(T) * (nh + nkv);
  tgi::launch(qk_norm_kernel, dim3(static_cast<unsigned>((units + 7) / 8)), dim3(256), 0, stream,
              static_cast<__nv_bfloat16*>(qkv), row_stride, T, nh, nkv, D, static_cast<const __nv_bfloat16*>(qw),
              static_cast<const __nv_bfloat16*>(kw), q_head_stride, k_head_stride, eps, w_offset, layer);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// scores[B, V] (fp32) = penalised(logits[B, V] * logit_scale); history int64 [B, L]; rep / freq fp32 [B] or null
int tgi_penalties(const void* logits, int is_fp32, long long in_stride, float* scores, long long out_stride,
                  const long long* history, int L, const float* rep, const float* freq, int vocab_start, int B, int V,
                  float logit_scale, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (is_fp32)
    tgi::launch(penalties_kernel<float>, dim3(B), dim3(1024), 0, stream, static_cast<const float*>(logits), in_stride, scores,
                out_stride, history, L, rep, freq, vocab_start, V, logit_scale);
  else
    tgi::launch(penalties_kernel<__nv_bfloat16>, dim3(B), dim3(1024), 0, stream, static_cast<const __nv_bfloat16*>(logits),
                in_stride, scores, out_stride, history, L, rep, freq, vocab_start, V, logit_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int tgi_norm(const void* x, const void* residual, const void* weight, const void* bias, void* out, void* res_out,
             void* q_out, float* scale_t, int scale_pitch, int T, int H, float eps, float w_offset, int layer,
             cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || H > 16384) return -10;
  const bool quant = q_out != nullptr;
  if (quant && H % 128 != 0) return -11;
  const int nvec = H / 8;
  int threads = ((nvec + 31) / 32) * 32;
  int vpt = 1;
  if (threads > 1024) { vpt = 2; threads = (((nvec + 1) / 2 + 31) / 32) * 32; }
  auto x_ = static_cast<const __nv_bfloat16*>(x);
  auto r_ = static_cast<const __nv_bfloat16*>(residual);
  auto w_ = static_cast<const __nv_bfloat16*>(weight);
  auto b_ = static_cast<const __nv_bfloat16*>(bias);
  auto o_ = static_cast<__nv_bfloat16*>(out);
  auto ro_ = static_cast<__nv_bfloat16*>(res_out);
  auto q_ = static_cast<uint8_t*>(q_out);
#define LAUNCH(VPT, LAYER, QUANT) \
  tgi::launch(norm_kernel<VPT, LAYER, QUANT>, dim3(T), dim3(threads), 0, stream, x_, r_, w_, b_, o_, ro_, q_, scale_t, scale_pitch, H, eps, w_offset)
  if (vpt == 1) {
    if (layer) { if (quant) LAUNCH(1, true, true); else LAUNCH(1, true, false); }
    else { if (quant) LAUNCH(1, false, true); else LAUNCH(1, false, false); }
  } else {
    if (layer) { if (quant) LAUNCH(2, true, true); else LAUNCH(2, true, false); }
    else { if (quant) LAUNCH(2, false, true); else LAUNCH(2, false, false); }
  }
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int tgi_act_mul(const void* in, void* out, void* q_out, float* scale_t, int scale_pitch, int T, int I, int act,
                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I % 8 != 0) return -10;
  const bool quant = q_out != nullptr;
  if (quant && I % 128 != 0) return -11;
  if (quant) {   // I % 128 == 0: 16 elements per thread
    dim3 grid((I / 16 + 255) / 256, T);
    tgi::launch(act_mul_kernel<true, 2>, dim3(grid), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(in), nullptr,
                static_cast<uint8_t*>(q_out), scale_t, scale_pitch, I, act);
  } else if (I % 16 == 0) {
    dim3 grid((I / 16 + 255) / 256, T);
    tgi::launch(act_mul_kernel<false, 2>, dim3(grid), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(in),
                static_cast<__nv_bfloat16*>(out), nullptr, nullptr, 0, I, act);
  } else {
    dim3 grid((I / 8 + 255) / 256, T);
    tgi::launch(act_mul_kernel<false, 1>, dim3(grid), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(in),
                static_cast<__nv_bfloat16*>(out), nullptr, nullptr, 0, I, act);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int tgi_quant_act(const void* x, void* q_out, float* scale_t, int scale_pitch, int T, int K, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (K % 128 != 0) return -10;
  dim3 grid((K / 8 + 255) / 256, T);
  tgi::launch(quant_act_kernel, dim3(grid), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q_out),
                                             scale_t, scale_pitch, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int tgi_rope_cache(const void* qkv, const int* positions, const float* cos_sin, const int* slots, void* q_out,
                   void* k_cache, void* v_cache, const float* k_scale, const float* v_scale, int T, int Hq, int Hkv,
                   int D, int rot, int neox, long long num_slots, int fp8_cache, int max_pos, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D % 2 != 0 || rot % 2 != 0 || rot > D || max_pos < 1) return -10;
  const bool aligned = (reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                        reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
                        reinterpret_cast<uintptr_t>(cos_sin)) % 16 == 0;
  if (neox && rot == D && D % 16 == 0 && aligned) {
    const int items = (Hq + 2 * Hkv) * (D / 16);
    const int threads = items >= 128 ? 128 : (items >= 64 ? 64 : 32);
    if (fp8_cache)
      tgi::launch(rope_cache_vec_kernel<true>, dim3(T), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(qkv),
                  positions, cos_sin, slots, static_cast<__nv_bfloat16*>(q_out), k_cache, v_cache, k_scale, v_scale, Hq,
                  Hkv, D, num_slots, max_pos);
    else
      tgi::launch(rope_cache_vec_kernel<false>, dim3(T), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(qkv),
                  positions, cos_sin, slots, static_cast<__nv_bfloat16*>(q_out), k_cache, v_cache, k_scale, v_scale, Hq,
                  Hkv, D, num_slots, max_pos);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  }
  if (fp8_cache)
    tgi::launch(rope_cache_kernel<true>, dim3(T), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(qkv), positions, cos_sin, slots,
                                                   static_cast<__nv_bfloat16*>(q_out), k_cache, v_cache, k_scale,
                                                   v_scale, Hq, Hkv, D, rot, neox, num_slots, max_pos);
  else
    tgi::launch(rope_cache_kernel<false>, dim3(T), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(qkv), positions, cos_sin, slots,
                                                    static_cast<__nv_bfloat16*>(q_out), k_cache, v_cache, k_scale,
                                                    v_scale, Hq, Hkv, D, rot, neox, num_slots, max_pos);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int tgi_embedding(const int* ids, const void* table, void* out, int T, int H, int rows, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -10;
  tgi::launch(embedding_kernel, dim3(T), dim3(256), 0, stream, ids, static_cast<const __nv_bfloat16*>(table),
                                          static_cast<__nv_bfloat16*>(out), H, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int tgi_argmax_logprob(const void* logits, long long* ids, float* logprob, int B, int V, long long row_stride,
                       int is_fp32, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (is_fp32)
    tgi::launch(argmax_logprob_kernel<float>, dim3(B), dim3(1024), 0, stream, static_cast<const float*>(logits), ids, logprob, V, row_stride);
  else
    tgi::launch(argmax_logprob_kernel<__nv_bfloat16>, dim3(B), dim3(1024), 0, stream, static_cast<const __nv_bfloat16*>(logits), ids,
                                                                 logprob, V, row_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Fused temperature / top-k / top-p / sampling; any of temperature, top_k, top_p, do_sample, seeds, steps may be
// null (stage off).  `is_fp32` selects the element type of `scores`.
int tgi_sample(const void* scores, long long row_stride, int is_fp32, const float* temperature, const int* top_k,
               const float* top_p, const float* typical_p, const unsigned char* do_sample, const long long* seeds,
               const int* steps, long long* ids, float* logprob, int B, int V, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (V <= 0) return -10;
  if (is_fp32)
    tgi::launch(sample_kernel<float>, dim3(B), dim3(1024), 0, stream, static_cast<const float*>(scores), row_stride, temperature, top_k, top_p,
                                                 typical_p, do_sample, seeds, steps, ids, logprob, V);
  else
    tgi::launch(sample_kernel<__nv_bfloat16>, dim3(B), dim3(1024), 0, stream, static_cast<const __nv_bfloat16*>(scores), row_stride, temperature,
                                                         top_k, top_p, typical_p, do_sample, seeds, steps, ids, logprob, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"

extern "C" int tgi_quant_set_pow2(int on) {
  const int v = on != 0;
  return cudaMemcpyToSymbol(g_quant_pow2, &v, sizeof(v)) == cudaSuccess ? 0 : -3;
}

// Quantisation pre-pass of the 8-bit attention variant (per-block INT8 Q/K, per-channel FP8 V),
// following the published SageAttention recipe:
//   K is centred per (batch, head, channel) over the tokens (softmax is invariant to it),
//   Q (pre-multiplied by softmax_scale * log2 e) gets one scale per 128-token block,
//   K one scale per 64-token block, V one scale per (batch, head, channel) so that max |v| -> 448.
// All tensors are [B, S, H, 128]; the 8-bit outputs are contiguous in that layout.
//
// Both kernels are HBM-bound streams.  A CTA of 256 threads covers 16 token rows at a time: 16
// consecutive threads read one 256-byte head row as 16-byte vectors, so every warp request is two
// full rows.  Algorithmic bytes: colstat reads K and V once (4 * S * H * 128 bytes); quant reads Q, K,
// V once and writes one byte per element (6 + 3 = 9 bytes per (token, head, channel) triple).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "elementwise.cuh"

namespace chitu {

constexpr int kQ8BlockQ = 128;  // tokens per Q scale
constexpr int kQ8BlockK = 64;   // tokens per K scale
constexpr int kQ8QuantThreads = 256;

// eight consecutive 16-bit values: raw load, and conversion to floats
__device__ __forceinline__ uint4 q8_load_raw(const void* base, size_t elem) {
  return __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + elem));
}
__device__ __forceinline__ void q8_unpack8(const uint4 raw, int dtype, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (dtype == 0) {  // bf16 (dtype code 0): the value is the high half of an fp32 pattern
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const float2 h = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = h.x;
      f[2 * i + 1] = h.y;
    }
  }
}

// Column statistics of K and V over 128 tokens per CTA, accumulated with atomics into
// k_sum [B,H,128] (plain sums) and v_amax [B,H,128] (bit pattern of a non-negative float).
// Both must be zero before the launch.  grid = (H, ceil(S / 128), B): heads vary fastest, so CTAs
// that run together read neighbouring 256-byte pieces of the same token rows.
__global__ void __launch_bounds__(kQ8QuantThreads)
q8_colstat_kernel(const void* __restrict__ k, const void* __restrict__ v, int dtype, long long ks_b, long long ks_s,
                  long long ks_h, long long vs_b, long long vs_s, long long vs_h, int S, int H,
                  float* __restrict__ k_sum, unsigned* __restrict__ v_amax) {
  __shared__ float sh_sum[8][128];
  __shared__ float sh_max[8][128];
  const int h = blockIdx.x, b = blockIdx.z;
  const int sub = threadIdx.x >> 4;        // row within a pass of 16
  const int c0 = (threadIdx.x & 15) * 8;   // first channel of this thread
  float sum[8], amax[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) sum[e] = amax[e] = 0.f;
#pragma unroll 4
  for (int pass = 0; pass < 8; ++pass) {
    const int s = blockIdx.y * 128 + pass * 16 + sub;
    if (s < S) {
      float fk[8], fv[8];
      const uint4 rk = q8_load_raw(k, static_cast<size_t>(b * ks_b + s * ks_s + h * ks_h + c0));
      const uint4 rv = q8_load_raw(v, static_cast<size_t>(b * vs_b + s * vs_s + h * vs_h + c0));
      q8_unpack8(rk, dtype, fk);
      q8_unpack8(rv, dtype, fv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        sum[e] += fk[e];
        amax[e] = fmaxf(amax[e], fabsf(fv[e]));
      }
    }
  }
  // lanes l and l + 16 of a warp hold the same channels
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    sum[e] += __shfl_xor_sync(0xffffffffu, sum[e], 16);
    amax[e] = fmaxf(amax[e], __shfl_xor_sync(0xffffffffu, amax[e], 16));
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane < 16) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      sh_sum[warp][c0 + e] = sum[e];
      sh_max[warp][c0 + e] = amax[e];
    }
  }
  __syncthreads();
  if (threadIdx.x < 128) {
    float s_all = 0.f, m_all = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      s_all += sh_sum[w][threadIdx.x];
      m_all = fmaxf(m_all, sh_max[w][threadIdx.x]);
    }
    const size_t idx = (static_cast<size_t>(b) * H + h) * 128 + threadIdx.x;
    atomicAdd(k_sum + idx, s_all);
    atomicMax(v_amax + idx, __float_as_uint(m_all));
  }
}

struct Q8QuantParams {
  const void* x[3];          // q, k, v
  long long xs_b[3], xs_s[3], xs_h[3];
  uint8_t* out[3];           // 8-bit copies, [B, S, H, 128] contiguous
  int S[3];                  // tokens of q, k, v
  int first_block[4];        // block index ranges along grid.y: q | k | v
  int dtype, H;
  float pre_scale;           // softmax_scale * log2 e, applied to q
  const float* k_sum;        // [B, H, 128] column sums of k
  const unsigned* v_amax;    // [B, H, 128] column max |v| (float bit patterns)
  float* q_scale;            // [B, H, ceil(Sq / 128)]
  float* k_scale;            // [B, H, ceil(Sk / 64)]
  float* q_corr;             // [B, H, Sq]: q' . mean(k), what the centring removed from every score of the row
};

// One CTA per (head, token block, batch) of q (128 tokens), k (64 tokens) or v (128 tokens); heads vary
// fastest across the grid for the same locality as in q8_colstat_kernel:
//   q -> int8 of x * pre_scale, one scale per block, plus q_corr
//   k -> int8 of x - mean_k, one scale per block
//   v -> e4m3 of x * 448 / amax per channel
// The scale arrays receive the dequantisation factor max|x| / 127.
__global__ void __launch_bounds__(kQ8QuantThreads, 4)
q8_quant_kernel(const __grid_constant__ Q8QuantParams p) {
  __shared__ float red[8];
  const int which = (blockIdx.y >= p.first_block[2]) ? 2 : (blockIdx.y >= p.first_block[1]) ? 1 : 0;
  const int blk = blockIdx.y - p.first_block[which];
  const int block_tokens = (which == 1) ? kQ8BlockK : kQ8BlockQ;
  const int n_pass = block_tokens / 16;
  const int h = blockIdx.x, b = blockIdx.z;
  const int S = p.S[which];
  const int sub = threadIdx.x >> 4;
  const int c0 = (threadIdx.x & 15) * 8;
  const size_t stat = (static_cast<size_t>(b) * p.H + h) * 128 + c0;

  float chan[8];  // q, k: mean of k per channel; v: 448 / amax per channel
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    if (which == 2)
      chan[e] = 448.0f / fmaxf(__uint_as_float(p.v_amax[stat + e]), 1e-8f);
    else
      chan[e] = p.k_sum[stat + e] / static_cast<float>(p.S[1]);
  }

  // all loads of the block first (up to eight 16-byte requests in flight per thread), then the math
  uint4 raw[8];
#pragma unroll
  for (int pass = 0; pass < 8; ++pass) {
    const int s = blk * block_tokens + pass * 16 + sub;
    raw[pass] = make_uint4(0u, 0u, 0u, 0u);
    if (pass < n_pass && s < S)
      raw[pass] = q8_load_raw(p.x[which],
                              static_cast<size_t>(b * p.xs_b[which] + s * p.xs_s[which] + h * p.xs_h[which] + c0));
  }
  // first sweep over the registers: block maximum (and q_corr); second sweep: quantise.  The transformed
  // values are recomputed rather than kept, which halves the register count and doubles the CTAs per SM.
  auto transformed = [&](int pass, float (&f)[8]) {
    q8_unpack8(raw[pass], p.dtype, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (which == 0) f[e] *= p.pre_scale;
      else if (which == 1) f[e] -= chan[e];
      else f[e] *= chan[e];
    }
  };
  float amax = 0.f;
  if (which != 2) {
#pragma unroll
    for (int pass = 0; pass < 8; ++pass) {
      const int s = blk * block_tokens + pass * 16 + sub;
      const bool valid = pass < n_pass && s < S;
      float f[8];
      transformed(pass, f);  // rows that were not loaded hold zeros: harmless for the maximum
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (which == 0) dot = fmaf(f[e], chan[e], dot);
        if (valid) amax = fmaxf(amax, fabsf(f[e]));
      }
      if (which == 0 && pass < n_pass) {  // whole-warp shuffles: the two rows of a warp may differ in validity
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (valid && (threadIdx.x & 15) == 0) p.q_corr[(static_cast<size_t>(b) * p.H + h) * S + s] = dot;
      }
    }
  }

  float inv = 1.f;
  if (which != 2) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    float bmax = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) bmax = fmaxf(bmax, red[w]);
    const float scale = fmaxf(bmax, 1e-8f) / 127.0f;
    inv = 1.0f / scale;
    if (threadIdx.x == 0) {
      const int n_blocks = (S + block_tokens - 1) / block_tokens;
      float* scales = (which == 0) ? p.q_scale : p.k_scale;
      scales[(static_cast<size_t>(b) * p.H + h) * n_blocks + blk] = scale;
    }
  }

#pragma unroll
  for (int pass = 0; pass < 8; ++pass) {
    const int s = blk * block_tokens + pass * 16 + sub;
    if (pass < n_pass && s < S) {
      float f[8];
      transformed(pass, f);
      uint32_t w[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t word = 0;
        if (which == 2) {
          uint16_t lo, hi;  // two E4M3 bytes per conversion (first source operand -> high byte)
          asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(f[q * 4 + 1]), "f"(f[q * 4]));
          asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(f[q * 4 + 3]), "f"(f[q * 4 + 2]));
          word = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = max(-127, min(127, __float2int_rn(f[q * 4 + e] * inv)));
            word |= (static_cast<uint32_t>(r) & 0xffu) << (8 * e);
          }
        }
        w[q] = word;
      }
      *reinterpret_cast<uint2*>(p.out[which] + ((static_cast<size_t>(b) * S + s) * p.H + h) * 128 + c0) =
          make_uint2(w[0], w[1]);
    }
  }
}

}  // namespace chitu

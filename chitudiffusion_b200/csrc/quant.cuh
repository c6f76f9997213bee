// Quantisation pre-pass of the 8-bit attention variant (per-block INT8 Q/K, per-channel FP8 V),
// following the published SageAttention recipe:
//   K is centred per (batch, head, channel) over the tokens (softmax is invariant to it),
//   Q (pre-multiplied by softmax_scale * log2 e) gets one scale per 128-token block,
//   K one scale per 64-token block, V one scale per (batch, head, channel) so that max |v| -> 448.
// All tensors are [B, S, H, 128]; the 8-bit outputs are contiguous in that layout.
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

// Column statistics of K and V over a chunk of tokens, accumulated with atomics into
// k_sum [B,H,128] (plain sums) and v_amax [B,H,128] (bit pattern of a non-negative float).
// Both must be zero before the launch.  grid = (chunks, H, B), 128 threads = one channel each.
__global__ void __launch_bounds__(128)
q8_colstat_kernel(const void* __restrict__ k, const void* __restrict__ v, int dtype, long long ks_b, long long ks_s,
                  long long ks_h, long long vs_b, long long vs_s, long long vs_h, int S, int H,
                  int tokens_per_chunk, float* __restrict__ k_sum, unsigned* __restrict__ v_amax) {
  const int d = threadIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int s0 = blockIdx.x * tokens_per_chunk;
  const int s1 = min(S, s0 + tokens_per_chunk);
  float sum = 0.f, amax = 0.f;
  for (int s = s0; s < s1; ++s) {
    sum += ld_as_float(k, dtype, static_cast<size_t>(b * ks_b + s * ks_s + h * ks_h + d));
    amax = fmaxf(amax, fabsf(ld_as_float(v, dtype, static_cast<size_t>(b * vs_b + s * vs_s + h * vs_h + d))));
  }
  const size_t idx = (static_cast<size_t>(b) * H + h) * 128 + d;
  atomicAdd(k_sum + idx, sum);
  atomicMax(v_amax + idx, __float_as_uint(amax));
}

// One CTA per (token block, head, batch); thread = one token row of 128 channels.
//   mode 0: Q  -> int8, x * pre_scale, one scale per block of kQ8BlockQ tokens; q_corr[b,h,s] = q' . mean(k)
//   mode 1: K  -> int8, x - k_sum / S, one scale per block of kQ8BlockK tokens
//   mode 2: V  -> e4m3, x / (v_amax / 448) per channel (no block scale)
// scales [B, H, n_blocks] receive the dequantisation factor (max|x| / 127).
__global__ void __launch_bounds__(128)
q8_quant_kernel(const void* __restrict__ x, int dtype, long long xs_b, long long xs_s, long long xs_h, int S, int H,
                int mode, float pre_scale, const float* __restrict__ k_sum, const unsigned* __restrict__ v_amax,
                uint8_t* __restrict__ out, float* __restrict__ scales, int block_tokens,
                float* __restrict__ q_corr, int k_tokens) {
  __shared__ float red[4];
  __shared__ float chan[128];
  const int h = blockIdx.y, b = blockIdx.z;
  const int n_blocks = gridDim.x;
  const int s = blockIdx.x * block_tokens + threadIdx.x;
  const bool valid = threadIdx.x < block_tokens && s < S;
  const size_t stat = (static_cast<size_t>(b) * H + h) * 128;
  if (mode == 1 || mode == 0) chan[threadIdx.x] = k_sum[stat + threadIdx.x] / static_cast<float>(k_tokens);
  if (mode == 2) chan[threadIdx.x] = 448.0f / fmaxf(__uint_as_float(v_amax[stat + threadIdx.x]), 1e-8f);
  __syncthreads();

  float vals[128];
  float amax = 0.f;
  if (valid) {
    const size_t base = static_cast<size_t>(b * xs_b + s * xs_s + h * xs_h);
#pragma unroll
    for (int d = 0; d < 128; d += 4) {
      const float4 f = ld4(x, dtype, base + d);
      vals[d] = f.x; vals[d + 1] = f.y; vals[d + 2] = f.z; vals[d + 3] = f.w;
    }
#pragma unroll
    for (int d = 0; d < 128; ++d) {
      if (mode == 0) vals[d] *= pre_scale;
      if (mode == 1) vals[d] -= chan[d];
      if (mode == 2) vals[d] *= chan[d];
      amax = fmaxf(amax, fabsf(vals[d]));
    }
  } else {
#pragma unroll
    for (int d = 0; d < 128; ++d) vals[d] = 0.f;
  }
  if (mode == 0 && valid && q_corr != nullptr) {
    // q' . mean(k): what the centring of K removed from every score of this row (base-2 domain)
    float dot = 0.f;
#pragma unroll
    for (int d = 0; d < 128; ++d) dot = fmaf(vals[d], chan[d], dot);
    q_corr[(static_cast<size_t>(b) * H + h) * S + s] = dot;
  }
  float inv = 1.f;
  if (mode != 2) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    const float bmax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const float scale = fmaxf(bmax, 1e-8f) / 127.0f;
    inv = 1.0f / scale;
    if (threadIdx.x == 0) scales[(static_cast<size_t>(b) * H + h) * n_blocks + blockIdx.x] = scale;
  }
  if (!valid) return;
  uint4* dst = reinterpret_cast<uint4*>(out + ((static_cast<size_t>(b) * S + s) * H + h) * 128);
#pragma unroll
  for (int d = 0; d < 128; d += 16) {
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float f = vals[d + q * 4 + e];
        uint32_t byte;
        if (mode == 2) {
          byte = static_cast<uint32_t>(__nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3));
        } else {
          const int r = max(-127, min(127, __float2int_rn(f * inv)));
          byte = static_cast<uint32_t>(r) & 0xffu;
        }
        word |= byte << (8 * e);
      }
      w[q] = word;
    }
    dst[d >> 4] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace chitu

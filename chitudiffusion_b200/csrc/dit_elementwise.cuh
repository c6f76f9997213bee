// Elementwise tails of a DiT block either side of the attention path (HBM-bound streams):
//
//   layernorm_affine_kernel   out = LayerNorm(x) * mul + add   -> 16 bit
//       the modulated input of the self-attention and of the FFN, LayerNorm(x) * (1 + scale) + shift,
//       and the affine LayerNorm in front of the cross-attention: one pass over the residual
//       stream instead of the reference's LayerNorm + float() + multiply + add kernels
//   gate_residual_kernel      x += y * gate                    (residual stream in place, 16-bit branch output)
//
// The residual stream is fp32 (Wan) or 16-bit (Flux).  Algorithmic bytes per element with an fp32
// stream: LayerNorm 4 read + 2 written; gated residual 4 + 2 read, 4 written.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace chitu {

constexpr int kLnThreads = 256;
constexpr int kLnMaxVec = 8;  // float4 per thread: rows of up to 8192 channels

struct LayerNormParams {
  const void* x;         // [rows, C] residual stream: fp32, or 16-bit (x_dtype 0 bf16, 1 fp16, 2 fp32)
  int x_dtype;
  void* out;             // [rows, C] bf16 / fp16
  const float* mul;      // [B or 1, C] fp32, or nullptr (= 1)
  const float* add;      // [B or 1, C] fp32, or nullptr (= 0)
  long long mul_batch_stride, add_batch_stride;  // elements between batches (0: one vector for all)
  long long rows, rows_per_batch;
  int C;
  int add_one;           // multiply by (1 + mul) instead of mul
  int out_fp16;
  float eps;
};

// four consecutive stream elements as floats / back (dtype 0 bf16, 1 fp16, 2 fp32)
__device__ __forceinline__ float4 stream_ld4(const void* p, int dtype, size_t vec) {
  if (dtype == 2) return __ldcs(reinterpret_cast<const float4*>(p) + vec);
  const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(p) + vec);
  float2 a, b;
  if (dtype == 0) {
    a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  } else {
    a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
  }
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void stream_st4(void* p, int dtype, size_t vec, float4 v) {
  if (dtype == 2) {
    reinterpret_cast<float4*>(p)[vec] = v;
    return;
  }
  uint2 o;
  if (dtype == 0) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    o.x = *reinterpret_cast<const uint32_t*>(&lo);
    o.y = *reinterpret_cast<const uint32_t*>(&hi);
  } else {
    const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    o.x = *reinterpret_cast<const uint32_t*>(&lo);
    o.y = *reinterpret_cast<const uint32_t*>(&hi);
  }
  reinterpret_cast<uint2*>(p)[vec] = o;
}

__device__ __forceinline__ float ln_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5;
  __syncthreads();  // red[] may still be read from the previous reduction
  if ((threadIdx.x & 31) == 0) red[warp] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < kLnThreads / 32; ++w) s += red[w];
  return s;
}

// One CTA per row at a time (grid-stride over rows); the row lives in registers between the two
// reductions (mean, then the centred sum of squares).
__global__ void __launch_bounds__(kLnThreads)
layernorm_affine_kernel(const LayerNormParams p) {
  __shared__ float red[kLnThreads / 32];
  const int n_vec = p.C >> 2;
  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const size_t row_vec0 = static_cast<size_t>(row) * n_vec;
    float4 v[kLnMaxVec];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kLnMaxVec; ++i) {
      const int idx = threadIdx.x + i * kLnThreads;
      if (idx < n_vec) {
        v[i] = stream_ld4(p.x, p.x_dtype, row_vec0 + idx);  // streamed once
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    }
    const float mean = ln_block_sum(sum, red) / static_cast<float>(p.C);
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < kLnMaxVec; ++i) {
      const int idx = threadIdx.x + i * kLnThreads;
      if (idx < n_vec) {
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
        sq += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
      }
    }
    const float rstd = rsqrtf(ln_block_sum(sq, red) / static_cast<float>(p.C) + p.eps);
    const long long b = row / p.rows_per_batch;
    const float4* mul = p.mul ? reinterpret_cast<const float4*>(p.mul + b * p.mul_batch_stride) : nullptr;
    const float4* add = p.add ? reinterpret_cast<const float4*>(p.add + b * p.add_batch_stride) : nullptr;
    uint2* dst = reinterpret_cast<uint2*>(static_cast<uint16_t*>(p.out) + row * p.C);
    const float one = p.add_one ? 1.f : 0.f;
#pragma unroll
    for (int i = 0; i < kLnMaxVec; ++i) {
      const int idx = threadIdx.x + i * kLnThreads;
      if (idx < n_vec) {
        float4 m = mul ? __ldg(mul + idx) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 a = add ? __ldg(add + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (mul) { m.x += one; m.y += one; m.z += one; m.w += one; }
        const float r0 = fmaf(v[i].x * rstd, m.x, a.x), r1 = fmaf(v[i].y * rstd, m.y, a.y);
        const float r2 = fmaf(v[i].z * rstd, m.z, a.z), r3 = fmaf(v[i].w * rstd, m.w, a.w);
        uint2 o;
        if (p.out_fp16) {
          const __half2 lo = __floats2half2_rn(r0, r1), hi = __floats2half2_rn(r2, r3);
          o.x = *reinterpret_cast<const uint32_t*>(&lo);
          o.y = *reinterpret_cast<const uint32_t*>(&hi);
        } else {
          const __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
          o.x = *reinterpret_cast<const uint32_t*>(&lo);
          o.y = *reinterpret_cast<const uint32_t*>(&hi);
        }
        dst[idx] = o;
      }
    }
  }
}

// Warp-per-row form for rows of at most 8 KiB (Flux: 3072 bf16 channels, Wan-1.3B: 1536 fp32): the row
// sits in registers as raw 16-byte vectors (up to 16 per lane, all loads in flight at once), the two
// reductions are warp shuffles, and nothing waits at a block barrier.  Lane l owns vectors l, l + 32, ...
constexpr int kLnWarpMaxVec = 16;

template <int kXDtype>
__device__ __forceinline__ void ln_unpack(const uint4 raw, float (&f)[8]) {
  // 16 bytes of the stream: 8 values when 16-bit, 4 when fp32 (f[4..7] unused)
  if constexpr (kXDtype == 2) {
    f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y);
    f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
    f[4] = f[5] = f[6] = f[7] = 0.f;
  } else {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (kXDtype == 0) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      } else {
        const float2 h = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        f[2 * i] = h.x;
        f[2 * i + 1] = h.y;
      }
    }
  }
}

template <int kXDtype>
__global__ void __launch_bounds__(256) layernorm_affine_warp_kernel(const LayerNormParams p) {
  constexpr int kPer = kXDtype == 2 ? 4 : 8;  // channels per 16-byte vector
  const int lane = threadIdx.x & 31;
  const int n_vec = p.C / kPer;               // vectors per row (a multiple of 32: checked by the host)
  const int per_lane = n_vec >> 5;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const float inv_c = 1.0f / static_cast<float>(p.C);
  const float one = p.add_one ? 1.f : 0.f;
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < p.rows;
       row += warps) {
    const uint4* src = reinterpret_cast<const uint4*>(p.x) + static_cast<size_t>(row) * n_vec;
    uint4 raw[kLnWarpMaxVec];
#pragma unroll
    for (int i = 0; i < kLnWarpMaxVec; ++i)
      if (i < per_lane) raw[i] = __ldcs(src + lane + i * 32);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kLnWarpMaxVec; ++i)
      if (i < per_lane) {
        float f[8];
        ln_unpack<kXDtype>(raw[i], f);
#pragma unroll
        for (int e = 0; e < kPer; ++e) sum += f[e];
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum * inv_c;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < kLnWarpMaxVec; ++i)
      if (i < per_lane) {
        float f[8];
        ln_unpack<kXDtype>(raw[i], f);
#pragma unroll
        for (int e = 0; e < kPer; ++e) sq = fmaf(f[e] - mean, f[e] - mean, sq);
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq * inv_c + p.eps);
    const long long b = row / p.rows_per_batch;
    const float* mul = p.mul ? p.mul + b * p.mul_batch_stride : nullptr;
    const float* add = p.add ? p.add + b * p.add_batch_stride : nullptr;
    uint16_t* dst = static_cast<uint16_t*>(p.out) + static_cast<size_t>(row) * p.C;
#pragma unroll
    for (int i = 0; i < kLnWarpMaxVec; ++i)
      if (i < per_lane) {
        const int c0 = (lane + i * 32) * kPer;
        float f[8], r[8];
        ln_unpack<kXDtype>(raw[i], f);
#pragma unroll
        for (int q = 0; q < kPer; q += 4) {
          float4 m = mul ? __ldg(reinterpret_cast<const float4*>(mul + c0 + q)) : make_float4(1.f, 1.f, 1.f, 1.f);
          const float4 a = add ? __ldg(reinterpret_cast<const float4*>(add + c0 + q)) : make_float4(0.f, 0.f, 0.f, 0.f);
          if (mul) { m.x += one; m.y += one; m.z += one; m.w += one; }
          r[q] = fmaf((f[q] - mean) * rstd, m.x, a.x);
          r[q + 1] = fmaf((f[q + 1] - mean) * rstd, m.y, a.y);
          r[q + 2] = fmaf((f[q + 2] - mean) * rstd, m.z, a.z);
          r[q + 3] = fmaf((f[q + 3] - mean) * rstd, m.w, a.w);
        }
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < kPer / 2; ++q) {
          if (p.out_fp16) {
            const __half2 h = __floats2half2_rn(r[2 * q], r[2 * q + 1]);
            o[q] = *reinterpret_cast<const uint32_t*>(&h);
          } else {
            const __nv_bfloat162 h = __floats2bfloat162_rn(r[2 * q], r[2 * q + 1]);
            o[q] = *reinterpret_cast<const uint32_t*>(&h);
          }
        }
        if constexpr (kPer == 8)
          *reinterpret_cast<uint4*>(dst + c0) = make_uint4(o[0], o[1], o[2], o[3]);
        else
          *reinterpret_cast<uint2*>(dst + c0) = make_uint2(o[0], o[1]);
      }
  }
}

struct GateResidualParams {
  void* x;               // [rows, C] residual stream (x_dtype 0 bf16, 1 fp16, 2 fp32), updated in place
  int x_dtype;
  const void* y;         // [rows, C] bf16 / fp16 branch output
  const float* gate;     // [B or 1, C] fp32, or nullptr (= 1)
  long long gate_batch_stride;
  long long rows, rows_per_batch;
  int C;
  int y_fp16;
};

__global__ void __launch_bounds__(256)
gate_residual_kernel(const GateResidualParams p) {
  const int n_vec = p.C >> 2;
  const long long total = p.rows * n_vec;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long row = i / n_vec;
    const int idx = static_cast<int>(i - row * n_vec);
    float4 xv = stream_ld4(p.x, p.x_dtype, static_cast<size_t>(i));
    const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(p.y) + i);
    float2 y0, y1;
    if (p.y_fp16) {
      y0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
      y1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    } else {
      y0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      y1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    }
    float4 g = make_float4(1.f, 1.f, 1.f, 1.f);
    if (p.gate) g = __ldg(reinterpret_cast<const float4*>(p.gate + (row / p.rows_per_batch) * p.gate_batch_stride) + idx);
    xv.x = fmaf(y0.x, g.x, xv.x);
    xv.y = fmaf(y0.y, g.y, xv.y);
    xv.z = fmaf(y1.x, g.z, xv.z);
    xv.w = fmaf(y1.y, g.w, xv.w);
    stream_st4(p.x, p.x_dtype, static_cast<size_t>(i), xv);
  }
}

// ----------------------------------------------------------------------------
// Classifier-free guidance: out = uncond + scale * (cond - uncond), optionally rescaled row by row to
// the norm of the conditional prediction (out *= ||cond|| / ||out|| over the last dim).  One warp per
// row, three passes over registers-sized chunks are avoided by keeping the row sums in two
// accumulators and re-reading the (L1 / L2 resident) row for the rescaled store.
// ----------------------------------------------------------------------------
struct CfgCombineParams {
  const void* cond;
  const void* uncond;
  void* out;
  long long rows;
  int C;
  int dtype;       // kBF16 / kFP16 / kFP32 of all three tensors
  int rescale;
  float scale;
};

__device__ __forceinline__ float cfg_ld(const void* p, int dtype, size_t i) {
  if (dtype == 2) return static_cast<const float*>(p)[i];
  if (dtype == 0) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void cfg_st(void* p, int dtype, size_t i, float v) {
  if (dtype == 2) static_cast<float*>(p)[i] = v;
  else if (dtype == 0) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else static_cast<__half*>(p)[i] = __float2half_rn(v);
}

__global__ void __launch_bounds__(256) cfg_combine_kernel(const CfgCombineParams p) {
  const int lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < p.rows;
       row += warps) {
    const size_t base = static_cast<size_t>(row) * p.C;
    float factor = 1.f;
    if (p.rescale) {
      float nc = 0.f, no = 0.f;
      for (int c = lane; c < p.C; c += 32) {
        const float a = cfg_ld(p.cond, p.dtype, base + c), b = cfg_ld(p.uncond, p.dtype, base + c);
        // the reference forms `combined` in the tensors' dtype before taking its norm
        float o = b + p.scale * (a - b);
        if (p.dtype == 0) o = __bfloat162float(__float2bfloat16_rn(o));
        else if (p.dtype == 1) o = __half2float(__float2half_rn(o));
        nc = fmaf(a, a, nc);
        no = fmaf(o, o, no);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        nc += __shfl_xor_sync(0xffffffffu, nc, o);
        no += __shfl_xor_sync(0xffffffffu, no, o);
      }
      factor = sqrtf(nc) / sqrtf(no);
    }
    for (int c = lane; c < p.C; c += 32) {
      const float a = cfg_ld(p.cond, p.dtype, base + c), b = cfg_ld(p.uncond, p.dtype, base + c);
      cfg_st(p.out, p.dtype, base + c, (b + p.scale * (a - b)) * factor);
    }
  }
}

}  // namespace chitu

// HBM-bound kernels around the attention core: LSE combine of partial results,
// the pre-attention RMSNorm + rotary transform, and the 16-byte strided copy
// used for all-to-all send/receive layouts.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "peer_sync.cuh"

namespace chitu {

enum : int { kBF16 = 0, kFP16 = 1, kFP32 = 2 };

__device__ __forceinline__ float ld_as_float(const void* p, int dtype, size_t i) {
  if (dtype == kFP32) return static_cast<const float*>(p)[i];
  if (dtype == kBF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ float round_to(float x, int dtype) {
  if (dtype == kBF16) return __bfloat162float(__float2bfloat16_rn(x));
  if (dtype == kFP16) return __half2float(__float2half_rn(x));
  return x;
}
__device__ __forceinline__ uint32_t pack16(float lo, float hi, int dtype) {
  if (dtype == kBF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Load 4 consecutive elements starting at element index i (i % 4 == 0).
__device__ __forceinline__ float4 ld4(const void* p, int dtype, size_t i) {
  if (dtype == kFP32) return *reinterpret_cast<const float4*>(static_cast<const float*>(p) + i);
  const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p) + i);
  float4 r;
  if (dtype == kBF16) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    r = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  } else {
    const __half2 a = *reinterpret_cast<const __half2*>(&raw.x);
    const __half2 b = *reinterpret_cast<const __half2*>(&raw.y);
    r = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  return r;
}
__device__ __forceinline__ void st4(void* p, int dtype, size_t i, float4 v) {
  if (dtype == kFP32) {
    *reinterpret_cast<float4*>(static_cast<float*>(p) + i) = v;
  } else {
    uint2 raw;
    raw.x = pack16(v.x, v.y, dtype);
    raw.y = pack16(v.z, v.w, dtype);
    *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p) + i) = raw;
  }
}

// ----------------------------------------------------------------------------
// LSE combine: one warp per (b, s, h) row of D values.
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
lse_combine_kernel(float* __restrict__ acc_out, float* __restrict__ acc_lse, const void* __restrict__ blk_out,
                   const float* __restrict__ blk_lse, int B, int S, int H, int D, int blk_dtype, int first,
                   void* __restrict__ final_out, int final_dtype) {
  const int lane = threadIdx.x & 31;
  const long long warps_total = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long rows = static_cast<long long>(B) * S * H;
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += warps_total) {
    const int h = static_cast<int>(row % H);
    const long long bs = row / H;
    const int s = static_cast<int>(bs % S);
    const int b = static_cast<int>(bs / S);
    const float lb = blk_lse[(static_cast<size_t>(b) * H + h) * S + s];
    float w = 0.f, new_lse = lb;
    if (!first) {
      const float la = acc_lse[row];
      const float x = lb - la;  // weight of the block = sigmoid(lse_b - lse)
      w = 1.0f / (1.0f + expf(-x));
      // lse - logsigmoid(lse - lse_b), logsigmoid(y) = min(y, 0) - log1p(exp(-|y|))
      const float y = -x;
      new_lse = la - (fminf(y, 0.f) - log1pf(expf(-fabsf(y))));
    }
    const size_t base = static_cast<size_t>(row) * D;
    for (int d = lane * 4; d < D; d += 128) {
      const float4 ob = ld4(blk_out, blk_dtype, base + d);
      float4 r = ob;
      if (!first) {
        const float4 oa = *reinterpret_cast<const float4*>(acc_out + base + d);
        r.x = oa.x - w * (oa.x - ob.x);
        r.y = oa.y - w * (oa.y - ob.y);
        r.z = oa.z - w * (oa.z - ob.z);
        r.w = oa.w - w * (oa.w - ob.w);
      }
      *reinterpret_cast<float4*>(acc_out + base + d) = r;
      if (final_out != nullptr) st4(final_out, final_dtype, base + d, r);
    }
    if (lane == 0) acc_lse[row] = new_lse;
  }
}

// ----------------------------------------------------------------------------
// RMSNorm + rotary + cast: one CTA per token, 8-element vectors in registers.
// ----------------------------------------------------------------------------
struct NormRopeParams {
  const void* x;
  int in_dtype;
  long long x_row_stride;
  const void* weight;
  int w_dtype;
  float eps;
  int norm_mode;  // 0 full channel dim, 1 per head, 2 none
  int rope_mode;  // 0 none, 1 three-axis grid, 2 per-token table
  const float2* table;
  int table_rows;
  int gf, gh, gw, n_t, n_h;
  long long pos_offset;
  void* out;
  int out_dtype;
  long long os_b, os_s, os_g, os_h;
  int heads_per_group;
  int B, S, H, D;
  int round_mid;
  // Scattered output (head-to-sequence exchange fused into the store): when n_out_ptrs > 0,
  // head group g = h / heads_per_group is written to out_ptrs[g] (its own or a peer GPU's
  // buffer) instead of out + g * os_g.
  void* out_ptrs[8];
  int n_out_ptrs;
  // Statistics-only job (norm_mode 0): when rstd_out is set the job writes rstd_out[b * S + s] =
  // rsqrt(mean_C(x^2) + eps) - the factor the attention kernel needs to normalise q in place - and
  // stores nothing else.
  float* rstd_out;
};

constexpr int kNormMaxThreads = 1024;  // one 8-channel vector per thread: up to 8192 channels per token

// 8 consecutive input elements of a token row, as loaded (one 16-byte request for 16-bit inputs,
// two for fp32) and converted to floats
template <int kInDtype>
struct RawVec8 {
  uint4 a;
};
template <>
struct RawVec8<kFP32> {
  uint4 a, b;
};
template <int kInDtype>
__device__ __forceinline__ RawVec8<kInDtype> ld_raw8(const void* p, size_t i) {
  RawVec8<kInDtype> r;
  if constexpr (kInDtype == kFP32) {
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const float*>(p) + i);
    r.a = __ldcs(src);
    r.b = __ldcs(src + 1);
  } else {
    r.a = __ldcs(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p) + i));
  }
  return r;
}
template <int kInDtype>
__device__ __forceinline__ void unpack8(const RawVec8<kInDtype>& r, float (&v)[8]) {
  if constexpr (kInDtype == kFP32) {
    v[0] = __uint_as_float(r.a.x); v[1] = __uint_as_float(r.a.y); v[2] = __uint_as_float(r.a.z);
    v[3] = __uint_as_float(r.a.w); v[4] = __uint_as_float(r.b.x); v[5] = __uint_as_float(r.b.y);
    v[6] = __uint_as_float(r.b.z); v[7] = __uint_as_float(r.b.w);
  } else {
    const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (kInDtype == kBF16) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
      }
    }
  }
}

// Persistent kernel: thread i of the CTA owns channels [8i, 8i+8) of every token the CTA
// visits, so the norm weights live in registers.  A CTA works on kTok consecutive tokens per
// iteration and has the raw vectors of the next kTok tokens in flight meanwhile (up to 128 bytes of
// loads per thread: the pass is latency-bound, and bytes in flight are what buys bandwidth).
// Full-width statistics need one block reduction per iteration, per-head statistics only warp
// shuffles.
// Up to three tensors (q, k, v) of one layer share a launch: blockIdx.y picks the job.  Jobs 0 and
// 1 use the template's norm / rotary modes; a job whose own modes are (2, 0) is a plain cast /
// scatter (the v tensor).
struct NormRopeBatch {
  NormRopeParams job[3];
  // when signal is set, the last CTA of the launch tells every peer that this rank's rows have landed
  PeerSync sync;
  int signal;
};

// tokens per iteration: 4 for 16-bit inputs, 2 for fp32 (the same bytes in flight)
template <int kInDtype>
struct NormRopeTokens {
  static constexpr int value = kInDtype == kFP32 ? 2 : 4;
};

// One job of a launch.  Everything that does not change inside a launch is a template argument, so
// the token loop carries no run-time mode tests: kNormMode / kRopeMode as documented at
// NormRopeParams, kRound 0 (no intermediate rounding), 1 (round the normalised value to the input
// type, as `type_as(x)` does) or 2 (also round after the weight multiply), kOutBf16 the store type.
template <int kInDtype, int kNormMode, int kRopeMode, int kRound, bool kOutBf16>
__device__ __forceinline__ void qk_norm_rope_job(const NormRopeParams& p, float (*red)[NormRopeTokens<kInDtype>::value][kNormMaxThreads / 32]) {
  constexpr int kTok = NormRopeTokens<kInDtype>::value;
  constexpr int kOutDtype = kOutBf16 ? kBF16 : kFP16;
  const int C = p.H * p.D;
  const int c0 = threadIdx.x * 8;
  const bool active = c0 < C;
  const int h = active ? c0 / p.D : 0;
  const int d0 = c0 - h * p.D;
  const int half_d = p.D >> 1;
  const int vec_per_head = p.D >> 3;
  const int n_warps = blockDim.x >> 5;
  const int tokens = p.B * p.S;  // the host refuses problems whose token count or positions pass 2^31
  const float inv_n = 1.0f / static_cast<float>(kNormMode == 0 ? C : p.D);

  float wgt[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) wgt[e] = 1.f;
  if (kNormMode != 2 && p.weight != nullptr && active) {
    const int w0 = (kNormMode == 0) ? c0 : d0;
#pragma unroll
    for (int e = 0; e < 8; ++e) wgt[e] = ld_as_float(p.weight, p.w_dtype, w0 + e);
  }
  const int grp = h / p.heads_per_group;
  const long long out_h = (p.n_out_ptrs > 0 ? 0 : grp * p.os_g) + (h % p.heads_per_group) * p.os_h + d0;
  // a null entry in out_ptrs drops that head group (replicated rows of which a rank keeps only its own heads)
  const bool keep = p.n_out_ptrs == 0 || p.out_ptrs[active ? grp : 0] != nullptr;
  uint16_t* const out_base = static_cast<uint16_t*>(p.n_out_ptrs > 0 ? p.out_ptrs[grp] : p.out) + out_h;
  const int grid_tokens = p.gf * p.gh * p.gw;
  const int pos0 = static_cast<int>(p.pos_offset);

  // 32-bit index arithmetic throughout: a 64-bit division costs more than the rest of a token's math
  int base = static_cast<int>(blockIdx.x) * kTok;
  const int step = static_cast<int>(gridDim.x) * kTok;
  RawVec8<kInDtype> cur[kTok], nxt[kTok];
#pragma unroll
  for (int i = 0; i < kTok; ++i) {
    cur[i].a = make_uint4(0u, 0u, 0u, 0u);
    if constexpr (kInDtype == kFP32) cur[i].b = make_uint4(0u, 0u, 0u, 0u);
    nxt[i] = cur[i];
    if (active && base + i < tokens)
      cur[i] = ld_raw8<kInDtype>(p.x, static_cast<size_t>(base + i) * p.x_row_stride + c0);
  }
  int phase = 0;
  for (; base < tokens; base += step, phase ^= 1) {
#pragma unroll
    for (int i = 0; i < kTok; ++i)
      if (active && base + step + i < tokens)
        nxt[i] = ld_raw8<kInDtype>(p.x, static_cast<size_t>(base + step + i) * p.x_row_stride + c0);

    float rstd_full[kTok];
    if constexpr (kNormMode == 0) {
      // full-width statistics of the kTok tokens with one barrier
#pragma unroll
      for (int i = 0; i < kTok; ++i) {
        float v[8];
        unpack8<kInDtype>(cur[i], v);
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((threadIdx.x & 31) == 0) red[phase][i][threadIdx.x >> 5] = ss;
      }
      __syncthreads();  // red[phase] is rewritten two iterations later, after the next barrier
      // every warp sums the per-warp partials itself: one shared-memory read per lane, then shuffles
#pragma unroll
      for (int i = 0; i < kTok; ++i) {
        const int lane = threadIdx.x & 31;
        float tot = lane < n_warps ? red[phase][i][lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
        rstd_full[i] = rsqrtf(tot * inv_n + p.eps);
      }
    }

    // batch and position of the first token of the iteration; the others follow by increments
    int b = base / p.S;
    int s = base - b * p.S;
    int pf = 0, ph = 0, pw = 0;  // (frame, row, column) of the token on the three-axis grid
    if constexpr (kRopeMode == 1) {
      const int n = pos0 + s;
      const int row = n / p.gw;
      pw = n - row * p.gw;
      pf = row / p.gh;
      ph = row - pf * p.gh;
    }
    if constexpr (kNormMode == 0) {
      if (p.rstd_out != nullptr) {
        if (threadIdx.x == 0) {
#pragma unroll
          for (int i = 0; i < kTok; ++i)
            if (base + i < tokens) p.rstd_out[base + i] = rstd_full[i];
        }
#pragma unroll
        for (int i = 0; i < kTok; ++i) cur[i] = nxt[i];
        continue;
      }
    }
#pragma unroll
    for (int i = 0; i < kTok; ++i) {
      if (base + i >= tokens) break;  // uniform over the CTA
      float v[8];
      unpack8<kInDtype>(cur[i], v);
      // rotary factors first: their (L1 / L2) loads overlap the statistics below
      float rc[4], rs[4];
      bool rotate = false;
      if (kRopeMode != 0 && active) {
        const int n = pos0 + s;
        if constexpr (kRopeMode == 2) {
          if (n < p.table_rows) {
            rotate = true;
            // per-token table: the four (cos, sin) pairs of this vector are 32 contiguous bytes
            const float4* trow =
                reinterpret_cast<const float4*>(p.table + static_cast<long long>(n) * half_d + (d0 >> 1));
            const float4 c0v = __ldg(trow), c1v = __ldg(trow + 1);
            rc[0] = c0v.x; rs[0] = c0v.y; rc[1] = c0v.z; rs[1] = c0v.w;
            rc[2] = c1v.x; rs[2] = c1v.y; rc[3] = c1v.z; rs[3] = c1v.w;
          }
        } else if (n < grid_tokens) {  // padding tokens past the grid pass through
          rotate = true;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int j = (d0 >> 1) + q;
            const int trow = (j < p.n_t) ? pf : ((j < p.n_t + p.n_h) ? ph : pw);
            const float2 cs = __ldg(&p.table[trow * half_d + j]);
            rc[q] = cs.x;
            rs[q] = cs.y;
          }
        }
      }

      float rstd = 1.f;
      if constexpr (kNormMode == 0) {
        rstd = rstd_full[i];
      } else if constexpr (kNormMode == 1) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
        if (vec_per_head == 16) {  // head_dim 128: the sixteen lanes of a head
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        } else {
          for (int o = vec_per_head >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        }
        rstd = rsqrtf(ss * inv_n + p.eps);
      }
      if (active && keep) {
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float t = v[e];
          if constexpr (kNormMode != 2) {
            t *= rstd;
            if constexpr (kRound >= 1) t = round_to(t, kInDtype);
            t *= wgt[e];
            if constexpr (kRound == 2) t = round_to(t, p.w_dtype);
          }
          y[e] = t;
        }
        if (rotate) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float re = y[2 * q] * rc[q] - y[2 * q + 1] * rs[q];
            const float im = y[2 * q] * rs[q] + y[2 * q + 1] * rc[q];
            y[2 * q] = re;
            y[2 * q + 1] = im;
          }
        }
        uint4 o;
        o.x = pack16(y[0], y[1], kOutDtype);
        o.y = pack16(y[2], y[3], kOutDtype);
        o.z = pack16(y[4], y[5], kOutDtype);
        o.w = pack16(y[6], y[7], kOutDtype);
        *reinterpret_cast<uint4*>(out_base + b * p.os_b + s * p.os_s) = o;
      }
      if (++s == p.S) {  // next batch: positions restart at the offset
        s = 0;
        ++b;
        if constexpr (kRopeMode == 1) {
          const int row = pos0 / p.gw;
          pw = pos0 - row * p.gw;
          pf = row / p.gh;
          ph = row - pf * p.gh;
        }
      } else if constexpr (kRopeMode == 1) {
        if (++pw == p.gw) {
          pw = 0;
          if (++ph == p.gh) {
            ph = 0;
            ++pf;
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kTok; ++i) cur[i] = nxt[i];
  }
}

// Picks the instance of the job blockIdx.y points at: a job whose own modes are (2, 0) is a plain
// cast / scatter whatever the launch's template modes are.
template <int kInDtype, int kNormModeT, int kRopeModeT>
__device__ __forceinline__ void qk_norm_rope_dispatch(const NormRopeBatch& batch,
                                                      float (*red)[NormRopeTokens<kInDtype>::value][kNormMaxThreads / 32]) {
  const NormRopeParams& p = batch.job[blockIdx.y];
  const bool out_bf16 = p.out_dtype == kBF16;
  if (p.norm_mode == 2 && p.rope_mode == 0) {
    if (out_bf16) qk_norm_rope_job<kInDtype, 2, 0, 0, true>(p, red);
    else qk_norm_rope_job<kInDtype, 2, 0, 0, false>(p, red);
    return;
  }
  // rounding of the weight product only where the reference's dtypes make it round (16-bit weight
  // and input); a missing weight multiplies by one, exactly
  const bool round_mid = p.round_mid && kNormModeT != 2;
  const bool round_w = round_mid && p.weight != nullptr && p.w_dtype != kFP32 && kInDtype != kFP32;
  const int round = round_w ? 2 : (round_mid ? 1 : 0);
  if (out_bf16) {
    if (round == 0) qk_norm_rope_job<kInDtype, kNormModeT, kRopeModeT, 0, true>(p, red);
    else if (round == 1) qk_norm_rope_job<kInDtype, kNormModeT, kRopeModeT, 1, true>(p, red);
    else qk_norm_rope_job<kInDtype, kNormModeT, kRopeModeT, 2, true>(p, red);
  } else {
    if (round == 0) qk_norm_rope_job<kInDtype, kNormModeT, kRopeModeT, 0, false>(p, red);
    else if (round == 1) qk_norm_rope_job<kInDtype, kNormModeT, kRopeModeT, 1, false>(p, red);
    else qk_norm_rope_job<kInDtype, kNormModeT, kRopeModeT, 2, false>(p, red);
  }
}

// Picks the instance of the job blockIdx.y points at: a job whose own modes are (2, 0) is a plain
// cast / scatter whatever the launch's template modes are.  A launch that feeds the fused exchange
// ends by publishing "my rows have landed" to every peer (last-block pattern).
template <int kInDtype, int kNormModeT, int kRopeModeT>
__device__ __forceinline__ void qk_norm_rope_body(const NormRopeBatch& batch) {
  __shared__ float red[2][NormRopeTokens<kInDtype>::value][kNormMaxThreads / 32];
  qk_norm_rope_dispatch<kInDtype, kNormModeT, kRopeModeT>(batch, red);
  if (batch.signal) {
    __syncthreads();
    if (threadIdx.x == 0) {
      if (batch.signal == 2)  // push mode: query rows went straight to the peers and are announced here; key and
                              // value rows were staged locally, the attention launch's copy CTAs announce those
        publish_when_last(batch.sync, kSyncScatterDone, kSyncInEpoch, kSyncQFlag, gridDim.x * gridDim.y);
      else
        publish_when_last(batch.sync, kSyncScatterDone, kSyncInEpoch, kSyncInFlag, gridDim.x * gridDim.y);
    }
  }
}

// Two entry points that differ only in their register budget: rows of up to 4096 channels (at most
// 512 threads) get 80 registers per thread - two iterations of raw vectors without spilling, two
// CTAs of 384 threads per SM; wider rows run with the 64 registers that 1024 threads leave.
template <int kInDtype, int kNormModeT, int kRopeModeT>
__global__ void __maxnreg__(80) qk_norm_rope_kernel(const __grid_constant__ NormRopeBatch batch) {
  qk_norm_rope_body<kInDtype, kNormModeT, kRopeModeT>(batch);
}
template <int kInDtype, int kNormModeT, int kRopeModeT>
__global__ void __launch_bounds__(kNormMaxThreads)
qk_norm_rope_wide_kernel(const __grid_constant__ NormRopeBatch batch) {
  qk_norm_rope_body<kInDtype, kNormModeT, kRopeModeT>(batch);
}

// ----------------------------------------------------------------------------
// strided copy of 16-byte vectors: dst contiguous [n0, n1, n2, n3, row_vecs]
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
strided_copy_kernel(const uint8_t* __restrict__ src, uint4* __restrict__ dst, long long n1, long long n2, long long n3,
                    long long row_vecs, long long st0, long long st1, long long st2, long long st3, long long total) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long r = i / row_vecs;
    const long long vec = i - r * row_vecs;
    const long long i3 = r % n3; r /= n3;
    const long long i2 = r % n2; r /= n2;
    const long long i1 = r % n1;
    const long long i0 = r / n1;
    const uint4* sp = reinterpret_cast<const uint4*>(src + i0 * st0 + i1 * st1 + i2 * st2 + i3 * st3) + vec;
    dst[i] = *sp;
  }
}

// ----------------------------------------------------------------------------
// Row scatter of 16-byte vectors: src is contiguous [B, n_dest * rows, row_vecs]; row
// (b, i * rows + j) goes to dst[i] + b * dst_batch + j * dst_row (+ the offset already folded into
// dst[i]).  The destinations may be peer-mapped buffers of other GPUs (plain stores).
// ----------------------------------------------------------------------------
struct ScatterRowsParams {
  uint8_t* dst[8];
  int n_dest;
  long long B, rows, row_vecs;
  long long dst_batch_bytes, dst_row_bytes;
};

__global__ void __launch_bounds__(256)
scatter_rows_kernel(const uint4* __restrict__ src, const ScatterRowsParams p) {
  const long long total = p.B * p.n_dest * p.rows * p.row_vecs;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long r = i / p.row_vecs;
    const long long vec = i - r * p.row_vecs;
    const long long j = r % p.rows; r /= p.rows;
    const long long d = r % p.n_dest;
    const long long b = r / p.n_dest;
    reinterpret_cast<uint4*>(p.dst[d] + b * p.dst_batch_bytes + j * p.dst_row_bytes)[vec] = src[i];
  }
}

// ----------------------------------------------------------------------------
// Barrier among the GPUs of one exchange group over peer-mapped flag arrays.
// Thread i tells peer i "rank `rank` has reached `epoch`" (release store, system scope) and
// then waits until peer i has said the same to us.  The wait is bounded; on timeout the
// status word is set and the kernel returns.
// ----------------------------------------------------------------------------
struct PeerBarrierParams {
  int* flags[8];  // flags[i]: base of rank i's flag array (world + 1 ints), mapped into this process
  int rank, world;
  int* status;
  long long timeout_cycles;
};

// The epoch lives on the device (slot `world` of the local flag array) and advances by one per
// barrier on every rank, so the kernel takes no per-call argument and can be replayed from a
// CUDA graph.
__global__ void peer_barrier_kernel(const PeerBarrierParams p) {
  const int i = threadIdx.x;
  int* counter = p.flags[p.rank] + p.world;
  const int epoch = *counter + 1;
  __syncwarp();
  if (i < p.world) {
    __threadfence_system();  // order this stream's earlier peer stores before the flag
    int* remote = p.flags[i] + p.rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const int* mine = p.flags[p.rank] + i;
    const long long t0 = clock64();
    int seen;
    unsigned spins = 0;
    while (true) {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (seen - epoch >= 0) break;  // epochs only grow (wrap-safe comparison)
      if ((++spins & 0xff) == 0 && clock64() - t0 > p.timeout_cycles) {
        if (p.status) atomicCAS(p.status, 0, 5);
        break;
      }
    }
  }
  __syncwarp();
  if (i == 0) *counter = epoch;
}

}  // namespace chitu

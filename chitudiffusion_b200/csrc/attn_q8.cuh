// 8-bit variant of the attention forward for head_dim 128 on sm_100a:
//   S = Q8 K8^T   tcgen05.mma kind::i8     (INT8 operands, INT32 accumulators in TMEM)
//   O += P8 V8    tcgen05.mma kind::f8f6f4 (E4M3 operands, FP32 accumulators in TMEM)
// with per-block Q/K scales and a per-channel V scale from the quantisation pre-pass (quant.cuh).
// Same CTA shape and protocol as attn_fwd_kernel: two 128-row query tiles per CTA, warps 0-3 / 4-7
// softmax for tile 0 / 1 (one thread = one score row), warp 8 MMA issuer, warp 9 TMA producer,
// TMEM columns S0 | S1 | O0 | O1; P overlays the first 32 columns of its S tile (four E4M3 values
// per column).  Tiles are 128 rows x 128 bytes = 16 KiB, one 128-byte-swizzle panel.
//
// Q is quantised after multiplication by softmax_scale * log2(e), so score = s_int * sq * sk is
// already in the base-2 domain.  Probabilities are kept as 2^(score - m + 4) with the lazy-rescale
// threshold at 4, i.e. in (0, 256], inside E4M3's range (max 448) with four extra binades of head
// room at the small end; the common factor cancels in O / l.
#pragma once

#include <type_traits>

#include "attn_fwd.cuh"
#include "ptx.cuh"

namespace chitu {

constexpr int kQ8TileBytes = 128 * 128;  // 16 KiB
constexpr int kQ8Stages = 8;             // K/V ring slots
constexpr int kQ8Threads = 384;
constexpr int kQ8SmemBytes = (2 + kQ8Stages) * kQ8TileBytes + 256 + 1024;
constexpr float kQ8Shift = 4.0f;      // exponent offset of the stored probabilities
constexpr float kQ8Threshold = 4.0f;  // lazy-rescale threshold (log2 units)
#ifndef CHITU_Q8_POLY_PAIRS
#define CHITU_Q8_POLY_PAIRS 4
#endif
constexpr int kQ8PolyPairs = CHITU_Q8_POLY_PAIRS;  // of every 8 score pairs, how many take the polynomial 2^x

struct AttnQ8Params {
  void* out;              // [B, Sq, H, 128] contiguous, bf16 / fp16
  float* lse;             // [B, H, Sq] fp32 natural-log, or nullptr
  int* status;
  int B, H, Sq, Sk;
  int is_fp16;
  const float* q_scale;   // [B, H, ceil(Sq / 128)]
  const float* k_scale;   // [B, H, ceil(Sk / 64)]
  const unsigned* v_amax; // [B, H, 128] bit patterns of max |v| per channel (dequantisation = amax / 448)
  const float* q_corr;    // [B, H, Sq] q' . mean(k) in the base-2 domain (undoes the K centring in the LSE)
#ifdef CHITU_ATTN_TIMING
  long long* dbg;
#endif
};

// 2^x for a pair of values on the FMA pipe, quadratic form of exp2_poly2 (max relative error 1.7e-3:
// enough for probabilities that are rounded to three mantissa bits)
__device__ __forceinline__ float2 exp2_quad2(float2 x) {
  const float kMagic = 12582912.f;
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 t = __fadd2_rd(x, make_float2(kMagic, kMagic));
  const float2 nf = __fadd2_rn(t, make_float2(-kMagic, -kMagic));
  const float2 f = __fadd2_rn(x, make_float2(-nf.x, -nf.y));
  float2 r = __ffma2_rn(make_float2(0.33718944f, 0.33718944f), f, make_float2(0.6576363f, 0.6576363f));
  r = __ffma2_rn(r, f, make_float2(1.0017247f, 1.0017247f));
  r.x = __uint_as_float(__float_as_uint(r.x) + (__float_as_uint(t.x) << 23));
  r.y = __uint_as_float(__float_as_uint(r.y) + (__float_as_uint(t.y) << 23));
  return r;
}

// two floats -> two E4M3 bytes (first argument in the low byte)
__device__ __forceinline__ uint32_t pack_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

template <bool kFp16>
__global__ void __launch_bounds__(kQ8Threads, 1)
attn_q8_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const AttnQ8Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_smem = smem_base;
  const uint32_t kv_smem = smem_base + 2 * kQ8TileBytes;
  const uint32_t bar_base = kv_smem + kQ8Stages * kQ8TileBytes;
  const uint32_t bar_q_full = bar_base;                       // [2]
  const uint32_t bar_kv_full = bar_base + 16;                 // [kQ8Stages]
  const uint32_t bar_kv_empty = bar_kv_full + 8 * kQ8Stages;  // [kQ8Stages]
  const uint32_t bar_s_full = bar_kv_empty + 8 * kQ8Stages;   // [2]
  const uint32_t bar_p_full = bar_s_full + 16;                // [2 tiles][2 halves]
  const uint32_t bar_o_final = bar_p_full + 32;               // [2]
  uint8_t* tail = smem_gen + (2 + kQ8Stages) * kQ8TileBytes + (16 + 16 * kQ8Stages + 64);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * 256;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int n_kv = (p.Sk + 127) / 128;
  const int n_qt = (q0 + 128 < p.Sq) ? 2 : 1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_full + 8, 1);
    for (int s = 0; s < kQ8Stages; ++s) {
      mbar_init(bar_kv_full + 8 * s, 1);
      mbar_init(bar_kv_empty + 8 * s, 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_s_full + 8 * t, 1);
      mbar_init(bar_p_full + 16 * t, 128);
      mbar_init(bar_p_full + 16 * t + 8, 128);
      mbar_init(bar_o_final + 8 * t, 1);
    }
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  if (warp == 9 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 9) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        for (int t = 0; t < n_qt; ++t) {
          mbar_arrive_expect_tx(bar_q_full + 8 * t, kQ8TileBytes);
          tma_load_4d(q_smem + t * kQ8TileBytes, &tm_q, bar_q_full + 8 * t, 0, head, q0 + t * 128, batch);
        }
      }
      const int n_items = 2 * n_kv;  // K_0, V_0, K_1, V_1, ...
      for (int i = 0; i < n_items; ++i) {
        const int slot = i % kQ8Stages;
        const int round = i / kQ8Stages;
        if (round > 0) mbar_wait(bar_kv_empty + 8 * slot, (round - 1) & 1, abort_flag, p.status, kDevTimeoutLoad);
        if (lane == 0) {
          const uint32_t bar = bar_kv_full + 8 * slot;
          mbar_arrive_expect_tx(bar, kQ8TileBytes);
          tma_load_4d(kv_smem + slot * kQ8TileBytes, (i & 1) ? &tm_v : &tm_k, bar, 0, head, (i >> 1) * 128, batch);
        }
        __syncwarp();
      }
      if (*abort_flag && lane == 0) {
        for (int i = max(0, n_items - kQ8Stages); i < n_items; ++i)
          for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar_kv_full + 8 * (i % kQ8Stages), (i / kQ8Stages) & 1);
               ++spin) {
          }
      }
    } else if (warp == 8) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t kIdescQK = umma_idesc(2, 1, 1, 0, 128, 128);  // s32 += s8 * s8, K-major / K-major
      constexpr uint32_t kIdescPV = umma_idesc(1, 0, 0, 1, 128, 128);  // f32 += e4m3 * e4m3, B MN-major
      const bool leader = elect_one();
      const uint64_t q_desc0 = umma_smem_desc_sw128(q_smem, 16, 1024);
      const uint64_t kv_desc0 = umma_smem_desc_sw128(kv_smem, 16, 1024);
      auto issue_qk = [&](int t, int slot) {
        // 4 steps of 32 bytes along head_dim inside the single 128-byte panel
        const uint64_t a0 = q_desc0 + static_cast<uint64_t>((t * kQ8TileBytes) >> 4);
        const uint64_t b0 = kv_desc0 + static_cast<uint64_t>((slot * kQ8TileBytes) >> 4);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_ss_i8(tmem_base + t * 128, a0 + 2 * k, b0 + 2 * k, kIdescQK, k > 0);
      };
      auto issue_pv_half = [&](int t, int slot, int h, bool accumulate) {
        // keys [64h, 64h+64) in 2 steps of 32: A = P (four E4M3 per TMEM column), B = V rows as loaded (MN-major)
        const uint64_t b0 = kv_desc0 + static_cast<uint64_t>((slot * kQ8TileBytes + h * 8192) >> 4);
        const uint32_t acc0 = accumulate ? 1u : 0u;
#pragma unroll
        for (int k = 0; k < 2; ++k)
          umma_ts_f8(tmem_base + 256 + t * 128, tmem_base + t * 128 + h * 16 + k * 8,
                     b0 + static_cast<uint64_t>((k * 4096) >> 4), kIdescPV, k > 0 ? 1u : acc0);
      };
      auto wait_item = [&](int i) {
        mbar_wait(bar_kv_full + 8 * (i % kQ8Stages), (i / kQ8Stages) & 1, abort_flag, p.status, kDevTimeoutMma);
      };
      mbar_wait(bar_q_full, 0, abort_flag, p.status, kDevTimeoutMma);
      wait_item(0);
      tc_fence_after_sync();
      if (leader) {
        issue_qk(0, 0);
        umma_commit(bar_s_full);
      }
      __syncwarp();
      if (n_qt > 1) {
        mbar_wait(bar_q_full + 8, 0, abort_flag, p.status, kDevTimeoutMma);
        tc_fence_after_sync();
        if (leader) {
          issue_qk(1, 0);
          umma_commit(bar_s_full + 8);
        }
        __syncwarp();
      }
      if (leader) umma_commit(bar_kv_empty);
      __syncwarp();
      for (int j = 0; j < n_kv; ++j) {
        const bool more = (j + 1 < n_kv);
        const int iv = 2 * j + 1, ik = 2 * j + 2;
        if (more) wait_item(ik);
        wait_item(iv);
        for (int t = 0; t < n_qt; ++t) {
          mbar_wait(bar_p_full + 16 * t, j & 1, abort_flag, p.status, kDevTimeoutMma);
          tc_fence_after_sync();
          if (leader) issue_pv_half(t, iv % kQ8Stages, 0, j > 0);
          __syncwarp();
          mbar_wait(bar_p_full + 16 * t + 8, j & 1, abort_flag, p.status, kDevTimeoutMma);
          tc_fence_after_sync();
          if (leader) {
            issue_pv_half(t, iv % kQ8Stages, 1, true);
            if (more) {
              issue_qk(t, ik % kQ8Stages);
              umma_commit(bar_s_full + 8 * t);
            } else {
              umma_commit(bar_o_final + 8 * t);
            }
          }
          __syncwarp();
        }
        if (leader && more) {
          umma_commit(bar_kv_empty + 8 * (iv % kQ8Stages));
          umma_commit(bar_kv_empty + 8 * (ik % kQ8Stages));
        }
        __syncwarp();
      }
    }
  } else {
#include "attn_q8_softmax.inc"
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace chitu

// Dense non-causal attention forward for head_dim 128 on sm_100a.
//
// One CTA owns one (batch, head, 256-query-row block): two 128-row query tiles
// that ping-pong on the tensor core.  Roles (384 threads):
//   warps 0-3  softmax for query tile 0   (thread = one score row, no shuffles)
//   warps 4-7  softmax for query tile 1
//   warp  8    MMA issuer (one thread issues tcgen05.mma, accumulators in TMEM)
//   warp  9    TMA producer (Q once, then K_j / V_j through a 5-slot ring)
//   warps 10-11 idle (they complete the third warpgroup so that registers can be
//              re-assigned per warpgroup: 48 for warps 8-11, 224 for the softmax warps)
//
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each.  The
// probabilities P are written back as packed 16-bit pairs over the first 64
// columns of their S buffer and feed the PV MMA straight from tensor memory.
//
// Softmax is the online form in base 2 with lazy rescaling: the running maximum
// used for the exponent only moves when the true maximum has grown by more than
// 2^8, so O is rescaled rarely.  Because the tensor pipe executes MMAs in issue
// order and S_{j+1} is committed after PV_j, seeing S_{j+1} implies PV_j is
// complete and O may be touched.
#pragma once

#include "elementwise.cuh"
#include "peer_sync.cuh"
#include "ptx.cuh"

namespace chitu {

constexpr int kHeadDim = 128;
constexpr int kTileM = 128;   // query rows per tile (UMMA M)
constexpr int kTileN = 128;   // keys per tile (UMMA N of QK^T, K extent of PV)
constexpr int kQTiles = 2;    // query tiles per CTA
constexpr int kStages = 5;    // K/V ring slots
constexpr int kTileBytes = kTileN * kHeadDim * 2;  // 32 KiB
constexpr int kHalfTileBytes = kTileBytes / 2;     // one 64-column swizzle panel
constexpr int kAttnThreads = 384;  // 8 softmax warps + MMA warp + TMA warp + 2 idle warps completing the warpgroup
constexpr int kSmemBarrierBytes = 256;
constexpr int kAttnSmemBytes = (kQTiles + kStages) * kTileBytes + kSmemBarrierBytes + 1024;  // +1024: manual alignment
constexpr float kRescaleThreshold = 8.0f;  // log2 units
#ifndef CHITU_POLY_PAIRS
#define CHITU_POLY_PAIRS 3
#endif
constexpr int kPolyPairs = CHITU_POLY_PAIRS;  // of every 8 score pairs, how many take the polynomial 2^x

struct AttnParams {
  void* out;        // [B, Sq, H, 128] contiguous, 16-bit
  float* lse;       // [B, H, Sq] fp32 natural-log, or nullptr
  int* status;      // device status word, or nullptr
  int B, H, Sq, Sk;
  float scale_log2; // softmax_scale * log2(e)
  int is_fp16;      // 0 = bf16, 1 = fp16
  // Scattered output (sequence-to-head exchange fused into the epilogue): when n_dest > 0, query
  // row r goes to destination r / rows_per_dest (its own or a peer GPU's buffer) at local row
  // r % rows_per_dest, byte address
  //   out_ptrs[dest] + batch * dest_batch_bytes + local_row * dest_row_bytes + dest_head_bytes + head * 256
  void* out_ptrs[8];
  int n_dest;
  int rows_per_dest;
  long long dest_batch_bytes, dest_row_bytes, dest_head_bytes;
  // Split over keys (under-filled grids): blockIdx.z = batch * n_splits + split; split s takes
  // key tiles [s * tiles_per_split, (s+1) * tiles_per_split).  With n_splits > 1 each CTA parks the
  // normalised fp32 rows of its key range and their log-sum-exps in scratch memory and bumps the
  // counter of its (batch, head, query block); the CTA that completes the count - the last of the
  // n_splits to finish - merges all ranges and writes the result, so no second launch is needed:
  //   split_count [batch][head][query block] int32, zero between calls (the merging CTA resets it)
  //   part_o   [n_splits][tile][32 chunks][128 rows] float4  (tile = ((batch * H + head) * query blocks
  //            + block) * 2 + t; chunk-major so that a warp's 32 rows are 512 contiguous bytes)
  //   part_lse [n_splits][tile][128 rows] fp32 (natural log)
  int n_splits, tiles_per_split;
  // cluster_merge (two key ranges only): the two CTAs of a query block are launched as a thread-block cluster;
  // the CTA of the second range writes its rows into the first one's shared memory (the K/V ring, idle by
  // then) and the first merges them with its own - no scratch memory, no counter.
  int cluster_merge;
  int split_strided;  // split s takes key tiles s, s + n_splits, ... instead of a contiguous range
  int* split_count;
  float* part_o;
  float* part_lse;
  // Fused exchange (in_flags != nullptr): the rows of q / k / v were stored into this GPU's buffers by
  // n_src ranks, rows_per_src consecutive rows each, and rank s announces them in in_flags[s] (see
  // peer_sync.cuh).  The TMA producer waits - bounded - for a rank's flag to reach *in_epoch before
  // the first copy that touches its rows, and visits the key tiles that are wholly local_src's first,
  // so the tensor pipe starts on rows that are already here.  With signal_out the last CTA tells
  // every peer that this rank's output rows have landed (only when the keys are not split: a split
  // call leaves that to the merge kernel).
  const int* in_flags;
  const int* in_epoch;
  int rows_per_src, local_src;
  long long flag_timeout;
  PeerSync sync;
  int signal_out;
  // Push mode (push_ctas > 0): key and value rows this rank owes its peers are staged in local memory, and
  // the launch is one-dimensional: its first push_ctas CTAs do no attention, they copy the staged rows
  // into the peers' buffers while the attention CTAs of the same launch already work - in push_order, the
  // order in which the receivers walk their keys: the first push_first peers, then the others (announced
  // in in_flags).  The attention CTAs follow, (query block, batch x split, head) in that order of
  // significance, grid_q x grid_z x grid_h of them.  Query rows are normally delivered and announced
  // (q_flags) by the staging launch itself; push_src[0] != nullptr makes the copy CTAs send them too,
  // first.  The rank's own rows are already in place and have no flag.  Copy CTAs never wait for anything
  // and are the first CTAs of the grid, so they are on the machine before an attention CTA can wait for
  // a peer's: the GPUs cannot starve one another of copy CTAs.
  int push_ctas, grid_q, grid_h, grid_z, push_rounds, push_first, rot_other;
  int push_order[8];
  const uint4* push_src[3];  // staged q, k, v: block d (push_vecs 16-byte vectors) holds the rows for rank d
  uint4* push_dst[3][8];     // where this rank's block starts in rank d's gathered q, k, v
  long long push_vecs;
  const int* q_flags;
  // Replicated prefix (the text tokens of the Qwen-Image layout): rows [0, prefix_rows) of q, k and v
  // are this rank's own copies (no arrival flag to wait for; the exchanged rows start at prefix_rows),
  // and the output rows of the prefix are stored to EVERY rank's prefix_ptrs buffer - each rank computes
  // them for its own heads only and all ranks need all heads.
  int prefix_rows;
  void* prefix_ptrs[8];
  long long prefix_batch_bytes, prefix_row_bytes, prefix_head_bytes;
  // Pre-attention transform of Q inside the kernel (q_norm_mode != 2 or q_rope_mode != 0): q is the RAW
  // projection output.  Once a query tile has landed in shared memory, the softmax warps - idle until
  // the first scores arrive - apply RMSNorm, weight, rotary embedding and the 16-bit rounding to it in
  // place, with exactly the arithmetic (and summation order) of qk_norm_rope_kernel, and only then is
  // the MMA warp released.  Modes as in NormRopeParams, except norm mode 0: the full-width statistic
  // cannot be formed from one head, so the caller passes rstd[b * Sq + s] computed elsewhere.
  int q_norm_mode, q_rope_mode, q_round_mid, q_w_dtype;
  const void* q_weight;   // [128] (mode 1) or [H * 128] (mode 0), or nullptr
  const float* q_rstd;    // [B, Sq] fp32 (mode 0)
  float q_eps;
  const float2* q_table;  // (cos, sin) pairs, [rows][64]
  int q_table_rows, q_gf, q_gh, q_gw, q_n_t, q_n_h;
  long long q_pos_offset;
#ifdef CHITU_ATTN_TIMING
  long long* dbg;   // per-phase clock totals of CTA 0 (development builds only)
#endif
};

template <bool kFp16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  if constexpr (kFp16) {
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x for a pair of values on the FMA pipe (no MUFU): split x = n + f with a round-down magic
// add, evaluate a cubic minimax polynomial for 2^f on [0, 1) (max relative error 7.5e-5, far
// below the 16-bit rounding of the probabilities) and add n to the exponent field.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  const float kMagic = 12582912.f;  // 1.5 * 2^23: x + kMagic rounded down holds floor(x) in its low mantissa bits
  x.x = fmaxf(x.x, -126.f);  // keeps the exponent field non-negative (the polynomial can dip just below 1)
  x.y = fmaxf(x.y, -126.f);
  const float2 t = __fadd2_rd(x, make_float2(kMagic, kMagic));
  const float2 nf = __fadd2_rn(t, make_float2(-kMagic, -kMagic));
  const float2 f = __fadd2_rn(x, make_float2(-nf.x, -nf.y));
  float2 r = __ffma2_rn(make_float2(0.07802403f, 0.07802403f), f, make_float2(0.22606707f, 0.22606707f));
  r = __ffma2_rn(r, f, make_float2(0.69583399f, 0.69583399f));
  r = __ffma2_rn(r, f, make_float2(0.99992513f, 0.99992513f));
  r.x = __uint_as_float(__float_as_uint(r.x) + (__float_as_uint(t.x) << 23));
  r.y = __uint_as_float(__float_as_uint(r.y) + (__float_as_uint(t.y) << 23));
  return r;
}

// The four softmax warps of a query tile rewrite it in shared memory.  As in the pre-pass kernel a
// thread owns one 8-value vector (16 threads per row, so a warp works on two rows at a time and the
// tile takes 16 rounds); the sum of squares is the same 16-lane butterfly, so the numbers match the
// pre-pass bit for bit.  Rotary factors and weights do not depend on the tile's data: they are
// fetched (coalesced) BEFORE waiting for the tile, so their latency hides behind the tile copy.
template <bool kFp16, typename WaitFn>
__device__ __forceinline__ void transform_q_tile(uint8_t* tile, int warp_in_tile, int lane, int head, int batch,
                                                 int row0, const AttnParams& p, WaitFn wait_for_tile) {
  constexpr int kIn = kFp16 ? kFP16 : kBF16;
  constexpr int kRounds = kTileM / 8;  // 4 warps x 2 rows per round
  const int sub = lane >> 4;   // which of the warp's two rows
  const int l16 = lane & 15;   // vector inside the row: channels [8 l16, 8 l16 + 8)
  const int panel = l16 >> 3, chunk = l16 & 7;
  const bool normed = p.q_norm_mode != 2;
  const int round = !normed || !p.q_round_mid ? 0 : ((p.q_weight != nullptr && p.q_w_dtype != kFP32) ? 2 : 1);
  float wgt[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) wgt[e] = 1.f;
  if (normed && p.q_weight != nullptr) {
    const int w0 = (p.q_norm_mode == 0 ? head * kHeadDim : 0) + l16 * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) wgt[e] = ld_as_float(p.q_weight, p.q_w_dtype, w0 + e);
  }
  // rotary factors (4 pairs per vector) and full-width factors of this thread's 16 rows
  float4 cs[kRounds][2];
  float rstd_row[kRounds];
  unsigned rotate_mask = 0;
  const long long grid_tokens = static_cast<long long>(p.q_gf) * p.q_gh * p.q_gw;
#pragma unroll
  for (int it = 0; it < kRounds; ++it) {
    const int r = it * 8 + warp_in_tile * 2 + sub;
    const int row = row0 + r;
    const long long n = p.q_pos_offset + row;
    rstd_row[it] = 1.f;
    if (p.q_norm_mode == 0) rstd_row[it] = __ldg(&p.q_rstd[static_cast<size_t>(batch) * p.Sq + min(row, p.Sq - 1)]);
    cs[it][0] = cs[it][1] = make_float4(1.f, 0.f, 1.f, 0.f);
    if (p.q_rope_mode == 2) {
      if (n < p.q_table_rows) {
        rotate_mask |= 1u << it;
        const float4* trow = reinterpret_cast<const float4*>(p.q_table + n * (kHeadDim / 2) + l16 * 4);
        cs[it][0] = __ldg(trow);
        cs[it][1] = __ldg(trow + 1);
      }
    } else if (p.q_rope_mode == 1) {
      if (n < grid_tokens) {
        rotate_mask |= 1u << it;
        const int ni = static_cast<int>(n);
        const int r2 = ni / p.q_gw;
        const int pw = ni - r2 * p.q_gw;
        const int pf = r2 / p.q_gh;
        const int ph = r2 - pf * p.q_gh;
        float2 f[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j = l16 * 4 + q;
          const int trow = (j < p.q_n_t) ? pf : ((j < p.q_n_t + p.q_n_h) ? ph : pw);
          f[q] = __ldg(&p.q_table[trow * (kHeadDim / 2) + j]);
        }
        cs[it][0] = make_float4(f[0].x, f[0].y, f[1].x, f[1].y);
        cs[it][1] = make_float4(f[2].x, f[2].y, f[3].x, f[3].y);
      }
    }
  }
  wait_for_tile();
#pragma unroll
  for (int it = 0; it < kRounds; ++it) {
    const int r = it * 8 + warp_in_tile * 2 + sub;
    uint8_t* addr = tile + panel * kHalfTileBytes + r * 128 + ((chunk ^ (r & 7)) << 4);
    RawVec8<kIn> raw;
    raw.a = *reinterpret_cast<const uint4*>(addr);
    float v[8];
    unpack8<kIn>(raw, v);
    float rstd = rstd_row[it];
    if (p.q_norm_mode == 1) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      rstd = rsqrtf(ss * (1.0f / kHeadDim) + p.q_eps);
    }
    float y[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float t = v[e];
      if (normed) {
        t *= rstd;
        if (round >= 1) t = round_to(t, kIn);
        t *= wgt[e];
        if (round == 2) t = round_to(t, p.q_w_dtype);
      }
      y[e] = t;
    }
    if ((rotate_mask >> it) & 1u) {
      const float rc[4] = {cs[it][0].x, cs[it][0].z, cs[it][1].x, cs[it][1].z};
      const float rs[4] = {cs[it][0].y, cs[it][0].w, cs[it][1].y, cs[it][1].w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float re = y[2 * q] * rc[q] - y[2 * q + 1] * rs[q];
        const float im = y[2 * q] * rs[q] + y[2 * q + 1] * rc[q];
        y[2 * q] = re;
        y[2 * q + 1] = im;
      }
    }
    uint4 o;
    o.x = pack16(y[0], y[1], kIn);
    o.y = pack16(y[2], y[3], kIn);
    o.z = pack16(y[4], y[5], kIn);
    o.w = pack16(y[6], y[7], kIn);
    *reinterpret_cast<uint4*>(addr) = o;
  }
}

// The copy CTAs of push mode (see AttnParams): `id` of `n` CTAs, blockDim.x threads each.
// One stage is a list of equally long segments (a tensor's block for one peer each); the threads walk the
// concatenation with a fixed stride and keep eight 16-byte loads in flight each - the copy is latency
// bound, and a segment alone (two vectors per thread on eight GPUs) would leave the pipeline empty.
template <typename SegFn>
__device__ __forceinline__ void push_segments(int n_seg, long long vecs, long long first, long long stride,
                                              SegFn seg_fn) {
  int seg = 0;
  long long i = first;
  while (i >= vecs) {
    i -= vecs;
    ++seg;
  }
  while (seg < n_seg) {
    uint4 t[8];
    uint4* d[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      d[u] = nullptr;
      if (seg < n_seg) {
        const uint4* src;
        uint4* dst;
        seg_fn(seg, src, dst);
        t[u] = __ldg(src + i);
        d[u] = dst + i;
        i += stride;
        while (i >= vecs) {
          i -= vecs;
          ++seg;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (d[u] != nullptr) *d[u] = t[u];
  }
}

__device__ __forceinline__ void push_rows(const AttnParams& p, int id, int n) {
  const int epoch = *reinterpret_cast<const volatile int*>(p.in_epoch);
  const long long stride = static_cast<long long>(n) * blockDim.x;
  const long long first = static_cast<long long>(id) * blockDim.x + threadIdx.x;
  if (p.push_src[0] != nullptr) {  // query rows too (a staging launch that left them to this one)
    push_segments(p.push_rounds, p.push_vecs, first, stride, [&](int seg, const uint4*& src, uint4*& dst) {
      const int dest = p.push_order[seg];
      src = p.push_src[0] + dest * p.push_vecs;
      dst = p.push_dst[0][dest];
    });
    // (the CTA holds its next stores back until the fence of this stage has completed: a fence that has to
    // outwait stores still being issued around it delayed the announcement by a whole stage)
    __syncthreads();
    if (threadIdx.x == 0) push_phase_done(p.sync, 0, n, kSyncQFlag, 0xffu, epoch);
    __syncthreads();
  }
  // key and value rows in two stages (the peers that need them first, then the rest): a stage ends with
  // one fence, and a fence costs a round trip to the peers, so there are few of them
  int r = 0;
  for (int stage = 0; stage < 2; ++stage) {
    const int r_end = stage == 0 ? p.push_first : p.push_rounds;
    if (r_end <= r) continue;
    push_segments(2 * (r_end - r), p.push_vecs, first, stride, [&](int seg, const uint4*& src, uint4*& dst) {
      const int dest = p.push_order[r + (seg >> 1)];
      const int t = 1 + (seg & 1);
      src = p.push_src[t] + dest * p.push_vecs;
      dst = p.push_dst[t][dest];
    });
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned dests = 0;
      for (int i = r; i < r_end; ++i) dests |= 1u << p.push_order[i];
      push_phase_done(p.sync, 1 + stage, n, kSyncInFlag, dests, epoch);
    }
    __syncthreads();
    r = r_end;
  }
}

#ifdef CHITU_ATTN_TIMING
#define CHITU_TRACE(i)                                                                                       \
  do {                                                                                                       \
    if (p.dbg != nullptr) {                                                                                  \
      unsigned long long t_;                                                                                 \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                                 \
      p.dbg[64 + 8 * (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)) + (i)] = (long long)t_; \
    }                                                                                                        \
  } while (0)
#else
#define CHITU_TRACE(i)
#endif

// Thread-block cluster helpers (cluster_merge).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void st_cluster_f1(uint32_t addr, float a) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
}

// (query block, head, batch x split) of an attention CTA.  The grid is (query blocks, batch x splits, heads):
// CTAs that follow one another in launch order share a head - all the key ranges of a query block included -
// so the CTAs resident at one time stream few heads' keys and values through L2.  Read afresh from the special registers each time
// (the asm is volatile), so that the epilogue can ask again instead of keeping four values in registers
// through the whole key loop.
__device__ __forceinline__ void attn_cta_coords(const AttnParams& p, int& qblock, int& head, int& bz) {
  unsigned x, y, z;
  asm volatile("mov.u32 %0, %%ctaid.x;" : "=r"(x));
  asm volatile("mov.u32 %0, %%ctaid.y;" : "=r"(y));
  asm volatile("mov.u32 %0, %%ctaid.z;" : "=r"(z));
  qblock = static_cast<int>(x);
  bz = static_cast<int>(y);
  head = static_cast<int>(z);
  if (p.push_ctas > 0) {
    int lin = qblock - p.push_ctas;
    int low = 0;
    if (p.cluster_merge) {  // the two key ranges of a query block are neighbours: they form the cluster
      low = lin & 1;
      lin >>= 1;
    }
    const int rest = lin / p.grid_q;
    qblock = lin - rest * p.grid_q;
    const int gz = p.cluster_merge ? p.grid_z >> 1 : p.grid_z;
    head = rest / gz;
    bz = rest - head * gz;
    if (p.cluster_merge) bz = bz * 2 + low;
  }
}

template <bool kFp16>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  if (threadIdx.x == 0) CHITU_TRACE(0);
  if (p.push_ctas > 0 && static_cast<int>(blockIdx.x) < p.push_ctas) {  // a copy CTA: no tensor memory, no barriers
    push_rows(p, blockIdx.x, p.push_ctas);
    if (threadIdx.x == 0) CHITU_TRACE(6);
    return;
  }
  int bx, by, bz;
  attn_cta_coords(p, bx, by, bz);

  const uint32_t q_smem = smem_base;                          // 2 tiles
  const uint32_t kv_smem = smem_base + kQTiles * kTileBytes;  // kStages tiles
  const uint32_t bar_base = kv_smem + kStages * kTileBytes;
  // barrier map (8 bytes each)
  const uint32_t bar_q_full = bar_base;                     // [2]
  const uint32_t bar_kv_full = bar_base + 16;               // [kStages]
  const uint32_t bar_kv_empty = bar_kv_full + 8 * kStages;  // [kStages]
  const uint32_t bar_s_full = bar_kv_empty + 8 * kStages;   // [2]
  const uint32_t bar_p_full = bar_s_full + 16;              // [2][2]  (tile, key half): P half stored
  const uint32_t bar_o_final = bar_p_full + 32;             // [2]
  uint8_t* tail = smem_gen + (kQTiles + kStages) * kTileBytes + (16 + 16 * kStages + 64);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8);
  const uint32_t bar_drain = smem_u32(tail + 16);  // only used when a wait has run out (see the MMA warp's exit)
  volatile int* merge_flag = reinterpret_cast<volatile int*>(tail + 40);  // this CTA merges the key ranges
  const uint32_t bar_q_ready = smem_u32(tail + 24);  // [2] a query tile has been transformed in place (128 arrivals)
  const bool q_fuse = p.q_norm_mode != 2 || p.q_rope_mode != 0;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qblock = bx;
  const int q0 = qblock * (kQTiles * kTileM);
  const int head = by;
  const int batch = bz / p.n_splits;
  const int split = bz - batch * p.n_splits;
  const int n_kv_total = (p.Sk + kTileN - 1) / kTileN;
  // This CTA's key tiles: kv0 + kv_step * u for u in [0, n_kv).  A contiguous range (kv_step 1), or - with
  // the fused exchange - every n_splits-th tile (split_strided): then each CTA of a query block holds some of
  // this rank's own rows and can start at once, instead of one of them idling until a peer's rows land.
  const int kv_step = p.split_strided ? p.n_splits : 1;
  const int kv0 = p.split_strided ? split : split * p.tiles_per_split;
  const int n_kv = p.split_strided ? (n_kv_total - split + p.n_splits - 1) / p.n_splits
                                   : min(p.tiles_per_split, n_kv_total - kv0);  // >= 1 (the host sizes the splits)
  const int n_qt = (q0 + kTileM < p.Sq) ? 2 : 1;
  // step j of this CTA works on its tile u = (j + rot) % n_kv: with the fused exchange the walk starts at the
  // first of its tiles made only of this rank's own rows
  int rot = 0;
  if (p.in_flags != nullptr) {
    const int own_lo = p.prefix_rows + p.local_src * p.rows_per_src;
    const int first_local = (own_lo + kTileN - 1) / kTileN;
    const int u0 = first_local <= kv0 ? 0 : (first_local - kv0 + kv_step - 1) / kv_step;
    const int tile0 = kv0 + kv_step * u0;
    if (u0 < n_kv && tile0 * kTileN >= own_lo && (tile0 + 1) * kTileN <= own_lo + p.rows_per_src)
      rot = u0;
    else if (p.rot_other < n_kv)
      rot = p.rot_other;
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_full + 8, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_kv_full + 8 * s, 1);
      mbar_init(bar_kv_empty + 8 * s, 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_s_full + 8 * t, 1);
      mbar_init(bar_p_full + 16 * t, kTileM);
      mbar_init(bar_p_full + 16 * t + 8, kTileM);
      mbar_init(bar_o_final + 8 * t, 1);
    }
    mbar_init(bar_drain, 1);
    mbar_init(bar_q_ready, kTileM);
    mbar_init(bar_q_ready + 8, kTileM);
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

  // Registers move from the warpgroup holding the two single-thread roles to the softmax warps.
  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 9) {
    // ------------------------------------------------------------------ TMA producer
    // arrival flags of the fused exchange: lane 0 remembers which source ranks it has already seen
    // (push mode: the rank's own rows were put in place by the staging launch and have no flag; query rows
    // and key / value rows are announced separately)
    uint32_t src_ready = p.push_ctas > 0 ? 1u << p.local_src : 0u;
    uint32_t q_ready = src_ready;
    const int flag_epoch = (p.in_flags != nullptr && lane == 0) ? *reinterpret_cast<const volatile int*>(p.in_epoch) : 0;
    auto wait_rows = [&](const int* flags, uint32_t& ready, int row_lo, int row_hi, int rows_total) {
      // rows [row_lo, row_hi) of a gathered tensor
      if (flags == nullptr) return;
      const int last = min(row_hi, rows_total) - 1 - p.prefix_rows;  // rows of the prefix are local
      if (last < 0) return;
      for (int src = max(row_lo - p.prefix_rows, 0) / p.rows_per_src; src <= last / p.rows_per_src; ++src) {
        if ((ready >> src) & 1u) continue;
        if (!wait_flag(flags + src, flag_epoch, p.flag_timeout, p.status)) *abort_flag = 1;
        ready |= 1u << src;
        CHITU_TRACE(1);
        // the rows were written by a peer's ordinary stores and are about to be read by the copy engine
        asm volatile("fence.proxy.async.global;" ::: "memory");
      }
    };
    if (lane == 0) {
      wait_rows(p.push_ctas > 0 ? p.q_flags : p.in_flags, q_ready, q0, q0 + n_qt * kTileM, p.Sq);
      CHITU_TRACE(7);
      for (int t = 0; t < n_qt; ++t) {
        mbar_arrive_expect_tx(bar_q_full + 8 * t, kTileBytes);
        tma_load_4d(q_smem + t * kTileBytes, &tm_q, bar_q_full + 8 * t, 0, head, q0 + t * kTileM, batch);
        tma_load_4d(q_smem + t * kTileBytes + kHalfTileBytes, &tm_q, bar_q_full + 8 * t, 64, head, q0 + t * kTileM,
                    batch);
      }
    }
    const int n_items = 2 * n_kv;  // K_0, V_0, K_1, V_1, ...
    for (int i = 0; i < n_items; ++i) {
      const int slot = i % kStages;
      const int round = i / kStages;
      if (round > 0) mbar_wait(bar_kv_empty + 8 * slot, (round - 1) & 1, abort_flag, p.status, kDevTimeoutLoad);
      if (lane == 0) {
        const CUtensorMap* tm = (i & 1) ? &tm_v : &tm_k;
        const int rel = (i >> 1) + rot;  // this item's tile among the CTA's own, wrapped without a division
        const int row = (kv0 + kv_step * (rel >= n_kv ? rel - n_kv : rel)) * kTileN;
        wait_rows(p.in_flags, src_ready, row, row + kTileN, p.Sk);
        const uint32_t dst = kv_smem + slot * kTileBytes;
        const uint32_t bar = bar_kv_full + 8 * slot;
        mbar_arrive_expect_tx(bar, kTileBytes);
        tma_load_4d(dst, tm, bar, 0, head, row, batch);
        tma_load_4d(dst + kHalfTileBytes, tm, bar, 64, head, row, batch);
      }
      __syncwarp();
    }
    if (lane == 0) CHITU_TRACE(2);
    if (*abort_flag && lane == 0) {
      // A role gave up: make sure no bulk copy of ours is still landing in this
      // CTA's shared memory before the CTA retires (bounded polls): the Q tiles, then the last
      // copy into every K/V slot.
      for (int t = 0; t < n_qt; ++t)
        for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar_q_full + 8 * t, 0); ++spin) {
        }
      for (int i = max(0, n_items - kStages); i < n_items; ++i) {
        const uint32_t bar = bar_kv_full + 8 * (i % kStages);
        const uint32_t par = (i / kStages) & 1;
        for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar, par); ++spin) {
        }
      }
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t kIdescQK = umma_idesc(1, kFp16 ? 0 : 1, kFp16 ? 0 : 1, 0, kTileM, kTileN);
    constexpr uint32_t kIdescPV = umma_idesc(1, kFp16 ? 0 : 1, kFp16 ? 0 : 1, 1, kTileM, kHeadDim);
    // One elected thread issues every MMA and every commit.  Operand descriptors are built
    // once; inside the loops only their start-address field moves.
    const bool leader = elect_one();
    const uint64_t q_desc0 = umma_smem_desc_sw128(q_smem, 16, 1024);
    const uint64_t k_desc0 = umma_smem_desc_sw128(kv_smem, 16, 1024);
    const uint64_t v_desc0 = umma_smem_desc_sw128(kv_smem, kHalfTileBytes, 1024);
    auto issue_qk = [&](int t, int slot) {
      // S_t = Q_t K^T : both operands K-major, 8 steps of 16 along head_dim
      const uint64_t a0 = q_desc0 + static_cast<uint64_t>((t * kTileBytes) >> 4);
      const uint64_t b0 = k_desc0 + static_cast<uint64_t>((slot * kTileBytes) >> 4);
      const uint32_t d = tmem_base + t * kTileN;
#pragma unroll
      for (int k = 0; k < kHeadDim / 16; ++k) {
        const uint64_t off = static_cast<uint64_t>(((k >> 2) * kHalfTileBytes + (k & 3) * 32) >> 4);
        umma_ss_f16(d, a0 + off, b0 + off, kIdescQK, k > 0);
      }
    };
    auto issue_pv_half = [&](int t, int slot, int h, bool accumulate) {
      // O_t += P_t[:, 64h .. 64h+64) V[64h .. 64h+64) : A = P from tensor memory (two 16-bit values
      // per column), B = V tile as loaded ([key][d], d contiguous => MN-major), 4 steps of 16 keys
      const uint64_t b0 = v_desc0 + static_cast<uint64_t>((slot * kTileBytes + h * 8192) >> 4);
      const uint32_t d = tmem_base + 2 * kTileN + t * kHeadDim;
      const uint32_t a = tmem_base + t * kTileN + h * 32;
      const uint32_t acc0 = accumulate ? 1u : 0u;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        umma_ts_f16(d, a + k * 8, b0 + static_cast<uint64_t>((k * 2048) >> 4), kIdescPV, k > 0 ? 1u : acc0);
      }
    };
    auto wait_item = [&](int i) {
      mbar_wait(bar_kv_full + 8 * (i % kStages), (i / kStages) & 1, abort_flag, p.status, kDevTimeoutMma);
    };

    mbar_wait(q_fuse ? bar_q_ready : bar_q_full, 0, abort_flag, p.status, kDevTimeoutMma);
    wait_item(0);
    tc_fence_after_sync();
    if (leader) {
      issue_qk(0, 0);
      umma_commit(bar_s_full);
    }
    __syncwarp();
    if (n_qt > 1) {
      mbar_wait((q_fuse ? bar_q_ready : bar_q_full) + 8, 0, abort_flag, p.status, kDevTimeoutMma);
      tc_fence_after_sync();
      if (leader) {
        issue_qk(1, 0);
        umma_commit(bar_s_full + 8);
      }
      __syncwarp();
    }
    if (leader) umma_commit(bar_kv_empty);  // K_0 free once both QK^T have run
    __syncwarp();

    for (int j = 0; j < n_kv; ++j) {
      const bool more = (j + 1 < n_kv);
      const int iv = 2 * j + 1;  // V_j
      const int ik = 2 * j + 2;  // K_{j+1}
      if (more) wait_item(ik);
      wait_item(iv);
      for (int t = 0; t < n_qt; ++t) {
        // the PV MMAs of the first 64 keys start while the softmax warps still work on the rest
        mbar_wait(bar_p_full + 16 * t, j & 1, abort_flag, p.status, kDevTimeoutMma);
        tc_fence_after_sync();
        if (leader) issue_pv_half(t, iv % kStages, 0, j > 0);
        __syncwarp();
        mbar_wait(bar_p_full + 16 * t + 8, j & 1, abort_flag, p.status, kDevTimeoutMma);
        tc_fence_after_sync();
        if (leader) {
          issue_pv_half(t, iv % kStages, 1, true);
          if (more) {
            issue_qk(t, ik % kStages);
            umma_commit(bar_s_full + 8 * t);
          } else {
            umma_commit(bar_o_final + 8 * t);
          }
        }
        __syncwarp();
      }
      // the last step releases nothing: its o_final commits stay the CTA's final barrier arrivals
      if (leader && more) {
        umma_commit(bar_kv_empty + 8 * (iv % kStages));
        umma_commit(bar_kv_empty + 8 * (ik % kStages));
      }
      __syncwarp();
    }
    if (*abort_flag) {
      // A wait ran out somewhere: MMAs already issued may still be running.  One more commit and a
      // bounded poll on it, so that nothing writes tensor memory after it has been freed below.
      if (leader) umma_commit(bar_drain);
      __syncwarp();
      for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar_drain, 0); ++spin) {
      }
    }
  }
  if (p.cluster_merge) {  // the two cluster barriers of the epilogue (every thread of both CTAs takes part)
    cluster_sync_all();
    cluster_sync_all();
  }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int t = warp >> 2;
    if (t >= n_qt && p.cluster_merge) {
      cluster_sync_all();
      cluster_sync_all();
    }
    if (t < n_qt) {
      const int quad = warp & 3;
      const int row_in_tile = quad * 32 + lane;
      const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
      const uint32_t t_s = tmem_base + lane_base + t * kTileN;
      const uint32_t t_o = tmem_base + lane_base + 2 * kTileN + t * kHeadDim;
      if (q_fuse) {
        // this tile's four warps: fetch rotary factors, wait for the tile, rewrite it, hand it to the MMA warp
#ifdef CHITU_ATTN_TIMING
        long long qt0 = clock64(), qt1 = 0;
#endif
        transform_q_tile<kFp16>(smem_gen + t * kTileBytes, quad, lane, head, batch, q0 + t * kTileM, p, [&] {
#ifdef CHITU_ATTN_TIMING
          qt1 = clock64();
#endif
          mbar_wait(bar_q_full + 8 * t, 0, abort_flag, p.status, kDevTimeoutSoftmax);
#ifdef CHITU_ATTN_TIMING
          if (p.dbg != nullptr && bx == 0 && by == 0 && bz == 0 && threadIdx.x == 0) {
            p.dbg[24] = qt1 - qt0;
            p.dbg[25] = clock64() - qt1;
            qt1 = clock64();
          }
#endif
        });
        fence_proxy_async_smem();  // the rewritten tile is read by the tensor core through the async proxy
        mbar_arrive(bar_q_ready + 8 * t);
#ifdef CHITU_ATTN_TIMING
        if (p.dbg != nullptr && bx == 0 && by == 0 && bz == 0 && threadIdx.x == 0)
          p.dbg[26] = clock64() - qt1;
#endif
      }
      const float sl2 = p.scale_log2;
      const int tail_valid = p.Sk - (n_kv_total - 1) * kTileN;  // 1..128 valid keys in the last tile of K
      float m_used = -INFINITY;
      float l_sum = 0.f;

#ifdef CHITU_ATTN_TIMING
      long long tw = 0, tl = 0, tm = 0, ts = 0, c0, c1;
#define TICK(acc) c1 = clock64(); acc += c1 - c0; c0 = c1;
#else
#define TICK(acc)
#endif
      int jt = rot;  // the CTA's tile of step j (advanced without a division)
      // the tile whose tail may need masking, if it is one of this CTA's
      const int last_rel = (n_kv_total - 1 - kv0) % kv_step == 0 ? (n_kv_total - 1 - kv0) / kv_step : -1;
      for (int j = 0; j < n_kv; ++j) {
#ifdef CHITU_ATTN_TIMING
        c0 = clock64();
#endif
        mbar_wait(bar_s_full + 8 * t, j & 1, abort_flag, p.status, kDevTimeoutSoftmax);
        tc_fence_after_sync();
        TICK(tw)
        // Row of 128 scores into registers, 32 columns per load; the load of chunk
        // c+1 is in flight while the running maximum of chunk c is taken.
        uint32_t s[4][32];
        const bool last_tile = (jt == last_rel && tail_valid < kTileN);
        if (++jt == n_kv) jt = 0;
        float mx0 = -INFINITY, mx1 = -INFINITY;
        tmem_ld32(t_s, s[0]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_wait_ld();
          if (c < 3) tmem_ld32(t_s + (c + 1) * 32, s[c + 1]);
          if (last_tile) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i >= tail_valid) s[c][i] = 0xff800000u;  // -inf
          }
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            mx0 = max3(mx0, __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
            mx1 = max3(mx1, __uint_as_float(s[c][i + 2]), __uint_as_float(s[c][i + 3]));
          }
        }
        TICK(tl)
        const float mx = fmaxf(mx0, mx1);

        if (j == 0) {
          m_used = mx;
        } else {
          const bool need = (mx - m_used) * sl2 > kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            const float f = need ? fast_exp2((m_used - mx) * sl2) : 1.0f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
              tmem_ld32(t_o + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
              tmem_st32(t_o + c * 32, o);
            }
            l_sum *= f;
            if (need) m_used = mx;
          }
        }

        // p = 2^(s*scale - m*scale): packed two-wide FMA / add, one MUFU per element
        const float2 sl2_2 = make_float2(sl2, sl2);
        const float neg_m = -m_used * sl2;
        const float2 neg_m2 = make_float2(neg_m, neg_m);
        uint32_t pk[2][32];
        float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float2 x0 = __ffma2_rn(make_float2(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1])), sl2_2, neg_m2);
            float2 x1 =
                __ffma2_rn(make_float2(__uint_as_float(s[c][i + 2]), __uint_as_float(s[c][i + 3])), sl2_2, neg_m2);
            // kPolyPairs of every 8 pairs take the FMA-pipe polynomial, the rest the MUFU unit, so
            // that both pipes stay busy (this iteration handles pairs 2g and 2g+1, g = i / 4)
            constexpr int kPolyOdd = kPolyPairs < 4 ? kPolyPairs : 4;
            constexpr int kPolyEven = kPolyPairs > 4 ? kPolyPairs - 4 : 0;
            if (((i >> 2) & 3) < kPolyEven) {
              x0 = exp2_poly2(x0);
            } else {
              x0.x = fast_exp2(x0.x);
              x0.y = fast_exp2(x0.y);
            }
            if (((i >> 2) & 3) < kPolyOdd) {
              x1 = exp2_poly2(x1);
            } else {
              x1.x = fast_exp2(x1.x);
              x1.y = fast_exp2(x1.y);
            }
            la = __fadd2_rn(la, x0);
            lb = __fadd2_rn(lb, x1);
            pk[c >> 1][(c & 1) * 16 + (i >> 1)] = pack2<kFp16>(x0.x, x0.y);
            pk[c >> 1][(c & 1) * 16 + (i >> 1) + 1] = pack2<kFp16>(x1.x, x1.y);
            if ((c & 1) == 1 && i == 28) {
              // 64 probabilities done: hand this half to the MMA warp
              TICK(tm)
              tmem_st32(t_s + (c >> 1) * 32, pk[c >> 1]);
              tmem_wait_st();
              tc_fence_before_sync();
              mbar_arrive(bar_p_full + 16 * t + 8 * (c >> 1));
              TICK(ts)
            }
          }
        l_sum += (la.x + la.y) + (lb.x + lb.y);
      }
#ifdef CHITU_ATTN_TIMING
      if (p.dbg != nullptr && bx == 0 && by == 0 && bz == 0 && lane == 0 && (warp & 3) == 0) {
        p.dbg[t * 4 + 0] = tw; p.dbg[t * 4 + 1] = tl; p.dbg[t * 4 + 2] = tm; p.dbg[t * 4 + 3] = ts;
      }
#endif

      // epilogue: O / l -> 16-bit, row-contiguous 256-byte stores; LSE in natural log
      if (t == 0 && row_in_tile == 0) CHITU_TRACE(3);
      mbar_wait(bar_o_final + 8 * t, 0, abort_flag, p.status, kDevTimeoutEpilogue);
      tc_fence_after_sync();
      int qblock, head, ez;
      attn_cta_coords(p, qblock, head, ez);
      const int batch = ez / p.n_splits;
      const int split = ez - batch * p.n_splits;
      const int row = qblock * (kQTiles * kTileM) + t * kTileM + row_in_tile;
      const float inv_l = 1.0f / l_sum;
      uint4* dst;
      const bool in_prefix = p.n_dest != 0 && row < p.prefix_rows;
      if (p.n_dest == 0) {
        dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) +
                                       ((static_cast<size_t>(batch) * p.Sq + row) * p.H + head) * (kHeadDim * 2));
      } else if (in_prefix) {
        dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.prefix_ptrs[0]) + batch * p.prefix_batch_bytes +
                                       row * p.prefix_row_bytes + p.prefix_head_bytes + head * (kHeadDim * 2));
      } else {
        const int si = row - p.prefix_rows;
        const int dest = min(si / p.rows_per_dest, p.n_dest - 1);
        const long long local_row = si - static_cast<long long>(dest) * p.rows_per_dest;
        dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out_ptrs[dest]) + batch * p.dest_batch_bytes +
                                       local_row * p.dest_row_bytes + p.dest_head_bytes + head * (kHeadDim * 2));
      }
      uint8_t* stage = smem_gen + t * kTileBytes;
      // a 32-column piece of the final row, packed and parked in this query tile's shared memory
      auto park = [&](int c, const float (&f)[32]) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 v;
          v.x = pack2<kFp16>(f[i], f[i + 1]);
          v.y = pack2<kFp16>(f[i + 2], f[i + 3]);
          v.z = pack2<kFp16>(f[i + 4], f[i + 5]);
          v.w = pack2<kFp16>(f[i + 6], f[i + 7]);
          const int chunk = c * 4 + (i >> 3);
          *reinterpret_cast<uint4*>(stage + row_in_tile * 256 + ((chunk ^ (row_in_tile & 7)) << 4)) = v;
        }
      };
      float lse_row = (m_used * sl2 + log2f(l_sum)) * 0.6931471805599453f;
      bool write_out = true;
      if (p.n_splits == 1) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(t_o + c * 32, o);
          tmem_wait_ld();
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(o[i]) * inv_l;
          park(c, f);
        }
      } else if (p.cluster_merge) {
        // Two key ranges, two CTAs of one cluster.  After the first barrier both K/V rings are idle; the CTA of
        // the second range writes its normalised rows (chunk-major: a warp's 32 rows are 512 contiguous bytes)
        // and log-sum-exps into the first CTA's ring; after the second barrier the first CTA merges them with
        // the rows it still holds in tensor memory.
        constexpr uint32_t kPartTile = 32 * kTileM * 16;  // one query tile of fp32 rows: 64 KiB
        const uint32_t slot = kv_smem + t * kPartTile + row_in_tile * 16;
        const uint32_t lse_slot = kv_smem + 2 * kPartTile + (t * kTileM + row_in_tile) * 4;
        cluster_sync_all();
        if (split == 1) {
          const uint32_t remote = mapa_shared(slot, 0);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32(t_o + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              st_cluster_f4(remote + (c * 8 + (i >> 2)) * (kTileM * 16), __uint_as_float(o[i]) * inv_l,
                            __uint_as_float(o[i + 1]) * inv_l, __uint_as_float(o[i + 2]) * inv_l,
                            __uint_as_float(o[i + 3]) * inv_l);
          }
          st_cluster_f1(mapa_shared(lse_slot, 0), lse_row);
          write_out = false;
        }
        cluster_sync_all();
        if (split == 0) {
          float other_lse;
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(other_lse) : "r"(lse_slot));
          const float mx = fmaxf(lse_row, other_lse);
          float w_self = expf(lse_row - mx), w_other = expf(other_lse - mx);
          const float wsum = w_self + w_other;
          lse_row = mx + logf(wsum);
          w_self *= inv_l / wsum;
          w_other /= wsum;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32(t_o + c * 32, o);
            tmem_wait_ld();
            float f[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 v;
              asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                           : "r"(slot + (c * 8 + j) * (kTileM * 16)));
              f[4 * j] = fmaf(w_other, v.x, __uint_as_float(o[4 * j]) * w_self);
              f[4 * j + 1] = fmaf(w_other, v.y, __uint_as_float(o[4 * j + 1]) * w_self);
              f[4 * j + 2] = fmaf(w_other, v.z, __uint_as_float(o[4 * j + 2]) * w_self);
              f[4 * j + 3] = fmaf(w_other, v.w, __uint_as_float(o[4 * j + 3]) * w_self);
            }
            park(c, f);
          }
        }
      } else {
        // (1) this key range's normalised rows and log-sum-exp go to scratch
        const int n_qblocks = p.push_ctas > 0 ? p.grid_q : static_cast<int>(gridDim.x);
        const size_t tiles_total = static_cast<size_t>(p.B) * p.H * n_qblocks * 2;
        const size_t tile_id = ((static_cast<size_t>(batch) * p.H + head) * n_qblocks + qblock) * 2 + t;
        float4* mine = reinterpret_cast<float4*>(p.part_o) + (split * tiles_total + tile_id) * (32 * kTileM) + row_in_tile;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(t_o + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            mine[(c * 8 + (i >> 2)) * kTileM] =
                make_float4(__uint_as_float(o[i]) * inv_l, __uint_as_float(o[i + 1]) * inv_l,
                            __uint_as_float(o[i + 2]) * inv_l, __uint_as_float(o[i + 3]) * inv_l);
        }
        p.part_lse[(split * tiles_total + tile_id) * kTileM + row_in_tile] = lse_row;
        // (2) the CTA's softmax threads meet; one of them counts the CTA in and learns whether it is the
        //     last of the n_splits that share this query block
        asm volatile("bar.sync 1, %0;" ::"r"(n_qt * kTileM) : "memory");
        if (threadIdx.x == 0) {
          __threadfence();
          int* counter = p.split_count + (static_cast<size_t>(batch) * p.H + head) * n_qblocks + qblock;
          const int prev = atomicAdd(counter, 1);
          const int last = prev + 1 == p.n_splits;
          if (last) *counter = 0;
          __threadfence();
          *merge_flag = last;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(n_qt * kTileM) : "memory");
        write_out = *merge_flag != 0;
        if (write_out) {
          // (3) merge: out = sum_i exp(lse_i - lse) * part_i, lse = log sum_i exp(lse_i)
          const float* lses = p.part_lse + tile_id * kTileM + row_in_tile;
          const size_t lse_stride = tiles_total * kTileM;
          float mx = -INFINITY;
          for (int i = 0; i < p.n_splits; ++i) mx = fmaxf(mx, __ldcg(lses + i * lse_stride));
          float wsum = 0.f;
          for (int i = 0; i < p.n_splits; ++i) wsum += expf(__ldcg(lses + i * lse_stride) - mx);
          const float inv_w = 1.0f / wsum;
          lse_row = mx + logf(wsum);
          const float4* parts = reinterpret_cast<const float4*>(p.part_o) + tile_id * (32 * kTileM) + row_in_tile;
          const size_t part_stride = tiles_total * (32 * kTileM);
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = 0.f;
            for (int s_i = 0; s_i < p.n_splits; ++s_i) {
              const float w = expf(__ldcg(lses + s_i * lse_stride) - mx) * inv_w;
              const float4* src = parts + s_i * part_stride + (c * 8) * kTileM;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 v = __ldcg(src + j * kTileM);
                f[4 * j] = fmaf(w, v.x, f[4 * j]);
                f[4 * j + 1] = fmaf(w, v.y, f[4 * j + 1]);
                f[4 * j + 2] = fmaf(w, v.z, f[4 * j + 2]);
                f[4 * j + 3] = fmaf(w, v.w, f[4 * j + 3]);
              }
            }
            park(c, f);
          }
        }
      }
      if (write_out) {
        // Rows go out through this query tile's shared memory (its last reader, the final QK^T, has completed):
        // each thread has parked its 256-byte row there, now the warp stores its own 32 rows two at a time, 512
        // contiguous bytes per instruction.  A row per thread straight to global memory would leave the SM as
        // 16-byte pieces, which peer stores over NVLink carry at a fraction of the link rate.
        __syncwarp();
        const unsigned long long my_dst = row < p.Sq ? reinterpret_cast<unsigned long long>(dst) : 0ull;
        const int chunk = lane & 15;
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
          const int owner = 2 * i + (lane >> 4);  // the lane whose row this half-warp stores
          const unsigned long long base = __shfl_sync(0xffffffffu, my_dst, owner);
          const int to_all = __shfl_sync(0xffffffffu, static_cast<int>(in_prefix), owner);
          const int r = quad * 32 + owner;
          const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 256 + ((chunk ^ (r & 7)) << 4));
          if (base != 0ull) {
            reinterpret_cast<uint4*>(base)[chunk] = v;
            if (to_all) {  // a replicated row: the same bytes for the other ranks
              const long long off = static_cast<long long>(base - reinterpret_cast<unsigned long long>(p.prefix_ptrs[0]));
              for (int d = 1; d < p.n_dest; ++d)
                reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.prefix_ptrs[d]) + off)[chunk] = v;
            }
          }
        }
      }
      if (t == 0 && row_in_tile == 0) CHITU_TRACE(4);
      if (write_out && p.lse != nullptr && row < p.Sq)
        p.lse[(static_cast<size_t>(batch) * p.H + head) * p.Sq + row] = lse_row;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) CHITU_TRACE(5);
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (p.signal_out && threadIdx.x == 0)
    publish_when_last(p.sync, kSyncAttnDone, kSyncOutEpoch, kSyncOutFlag, p.push_ctas > 0 ? p.grid_q * p.grid_h * p.grid_z : gridDim.x * gridDim.y * gridDim.z);
  if (threadIdx.x == 0) CHITU_TRACE(6);
}

}  // namespace chitu

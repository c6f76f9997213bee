// extern "C" boundary of libchitu_b200.so: argument checks, tensor-map
// construction and kernel launches.  Nothing here allocates device memory,
// synchronises the device or throws.
#include "../../include/chitu_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "attn_fwd.cuh"
#include "elementwise.cuh"
#include "dit_elementwise.cuh"
#include "quant.cuh"
#include "attn_q8.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(CHITU_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }
  });
  return fn;
}

// Tensor map over a [B, S, H, 128] 16-bit tensor with element strides {b, s, h, 1}:
// dims (innermost first) d, h, s, b; box = 64 x 1 x 128 x 1 with 128-byte swizzle,
// i.e. one 128-row x 128-byte panel per copy; rows past S read as zero.
int make_qkv_map(CUtensorMap* map, const void* base, int B, int S, int H, const int64_t* st, const char* name,
                 int box_rows = 128) {
  auto encode = get_encode_fn();
  if (!encode) return fail(CHITU_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
  if (reinterpret_cast<uintptr_t>(base) & 15) return fail(CHITU_E_INVALID, "%s: base must be 16-byte aligned", name);
  if (st[3] != 1) return fail(CHITU_E_INVALID, "%s: head_dim stride must be 1 (got %lld)", name, (long long)st[3]);
  for (int i = 0; i < 3; ++i) {
    const bool degenerate = (i == 0 && B == 1) || (i == 1 && S == 1) || (i == 2 && H == 1);
    if (!degenerate && (st[i] <= 0 || (st[i] & 7)))
      return fail(CHITU_E_INVALID, "%s: stride[%d] = %lld must be a positive multiple of 8 elements", name, i,
                  (long long)st[i]);
  }
  auto stride_bytes = [&](int i, int extent) -> cuuint64_t {
    // a dimension of extent 1 never advances; give it any legal stride
    return (extent == 1 || st[i] <= 0 || (st[i] & 7)) ? 256 : static_cast<cuuint64_t>(st[i]) * 2;
  };
  cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(B)};
  cuuint64_t strides[3] = {stride_bytes(2, H), stride_bytes(1, S), stride_bytes(0, B)};
  cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CHITU_E_CUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", name, (int)r);
  return CHITU_OK;
}

int grid_for(long long work_items, int per_block, int max_blocks) {
  long long g = (work_items + per_block - 1) / per_block;
  if (g < 1) g = 1;
  if (g > max_blocks) g = max_blocks;
  return static_cast<int>(g);
}

int elem_size(int dtype) { return dtype == CHITU_DTYPE_FP32 ? 4 : 2; }

// The opt-in to more than 48 KB of dynamic shared memory belongs to the function IN THE CURRENT
// DEVICE'S CONTEXT, so a process that drives several GPUs has to make it once per device.
constexpr int kMaxDevices = 64;
template <typename Kernel>
cudaError_t ensure_dynamic_smem(Kernel kernel, int bytes, bool (&done)[kMaxDevices], std::mutex& mu) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  std::lock_guard<std::mutex> lock(mu);
  if (!done[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    done[dev] = true;
  }
  return cudaSuccess;
}

// How the key tiles of one attention call are cut into ranges: the requested count is clamped to
// the number of tiles and then shrunk until no range is empty.
struct SplitPlan {
  int n_splits, tiles_per_split;
};
SplitPlan plan_key_splits(int Sk, int requested) {
  const int tiles = (Sk + chitu::kTileN - 1) / chitu::kTileN;
  int n = requested < tiles ? requested : tiles;
  if (n < 1) n = 1;
  const int per = (tiles + n - 1) / n;
  return SplitPlan{(tiles + per - 1) / per, per};
}

// Clock budget of the flag waits (peer barrier, arrival flags); about a second by default.
long long g_flag_wait_cycles = 1ll << 31;

// Two key ranges merge through a thread-block cluster's shared memory instead of scratch memory.
int g_cluster_merge = 1;

}  // namespace

#ifdef CHITU_ATTN_TIMING
static long long* g_dbg = nullptr;
extern "C" void chitu_b200_set_dbg(long long* ptr) { g_dbg = ptr; }
#endif

extern "C" {

int chitu_b200_version(void) { return 100; }

unsigned chitu_b200_caps(void) {
  return CHITU_CAP_ATTN_BF16 | CHITU_CAP_ATTN_FP16 | CHITU_CAP_NORM_ROPE | CHITU_CAP_LSE_COMBINE | CHITU_CAP_A2A_LAYOUT |
         CHITU_CAP_PEER_EXCHANGE | CHITU_CAP_ATTN_Q8;
}

const char* chitu_b200_last_error(void) { return g_err; }

}  // extern "C"

namespace {

struct OutScatter {
  void* const* ptrs = nullptr;
  int n_dest = 0;
  int rows_per_dest = 0;
  int64_t batch_stride = 0, row_stride = 0, head_offset = 0;  // elements
};

struct KeySplit {
  int n_splits = 1;
  void* workspace = nullptr;
  int64_t workspace_bytes = 0;
};

// Fused-exchange synchronisation of one call: wait for the arrival flags of the ranks whose rows are
// read (rows_per_src rows each) and, at the end, announce this rank's output rows.
struct Exchange {
  const chitu_b200_peer_sync* sync = nullptr;
  int rows_per_src = 0;
  // replicated prefix rows (local copies; their outputs go to every rank)
  int prefix_rows = 0;
  void* const* prefix_ptrs = nullptr;
  int64_t prefix_batch_stride = 0, prefix_row_stride = 0, prefix_head_offset = 0;  // elements
  const chitu_b200_push* push = nullptr;  // copy CTAs inside the attention launch
};

// Copy CTAs of push mode: 40, or - where the attention CTAs alone leave SMs idle - what fits beside them
// (8 to 48), so that the whole grid is resident at once.  They are the first CTAs of a one-dimensional
// grid and never wait for anything.
int plan_push_ctas(int B, int Sq, int H, int n_splits) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return 0;
  const long long qblocks = (Sq + chitu::kQTiles * chitu::kTileM - 1) / (chitu::kQTiles * chitu::kTileM);
  const long long free_sms = sms - qblocks * H * B * n_splits;
  if (free_sms >= 8) return static_cast<int>(free_sms < 48 ? free_sms : 48);
  return sms >= 80 ? 40 : 0;
}

int fill_peer_sync(chitu::PeerSync* ps, const chitu_b200_peer_sync* sync, const char* what) {
  if (!sync || !sync->blocks || sync->world < 1 || sync->world > 8 || sync->rank < 0 || sync->rank >= sync->world)
    return fail(CHITU_E_INVALID, "%s: need a sync descriptor with 1..8 ranks and a rank inside the group", what);
  for (int i = 0; i < 8; ++i) ps->blocks[i] = i < sync->world ? sync->blocks[i] : nullptr;
  for (int i = 0; i < sync->world; ++i)
    if (!ps->blocks[i] || (reinterpret_cast<uintptr_t>(ps->blocks[i]) & 3))
      return fail(CHITU_E_INVALID, "%s: sync block of rank %d null or misaligned", what, i);
  ps->rank = sync->rank;
  ps->world = sync->world;
  ps->timeout_cycles = g_flag_wait_cycles;
  return CHITU_OK;
}

// Key-split scratch: a fixed header of per-query-block counters (zero between calls), then the partial
// rows and their log-sum-exps, whole 128-row tiles (see AttnParams).
constexpr int64_t kSplitHeaderBytes = CHITU_SPLITKV_HEADER_BYTES;
int64_t splitkv_workspace_bytes(int B, int Sq, int H, int D, int n_splits) {
  if (n_splits <= 1) return 0;
  const int64_t qblocks = (Sq + chitu::kQTiles * chitu::kTileM - 1) / (chitu::kQTiles * chitu::kTileM);
  const int64_t rows = static_cast<int64_t>(B) * H * qblocks * chitu::kQTiles * chitu::kTileM;
  return kSplitHeaderBytes + static_cast<int64_t>(n_splits) * rows * (static_cast<int64_t>(D) + 1) * 4;
}

int attn_fwd_impl(const void* q, const void* k, const void* v, void* out, const OutScatter& sc, float* lse, int B,
                  int Sq, int Sk, int H, int D, const int64_t* q_strides, const int64_t* k_strides,
                  const int64_t* v_strides, float softmax_scale, int dtype, int* status, void* stream,
                  const KeySplit& ks = KeySplit{}, const Exchange& ex = Exchange{},
                  const chitu_b200_q_pre* qpre = nullptr) {
  if (!q || !k || !v || (!out && sc.n_dest == 0) || !q_strides || !k_strides || !v_strides)
    return fail(CHITU_E_INVALID, "attn_fwd: null pointer argument");
  if (sc.n_dest != 0) {
    if (sc.n_dest < 0 || sc.n_dest > 8 || !sc.ptrs) return fail(CHITU_E_INVALID, "attn_fwd: 1..8 destinations");
    if (sc.rows_per_dest <= 0 || static_cast<int64_t>(sc.rows_per_dest) * sc.n_dest + ex.prefix_rows < Sq)
      return fail(CHITU_E_INVALID, "attn_fwd: destinations do not cover the query rows");
    if ((sc.batch_stride | sc.row_stride | sc.head_offset) & 7)
      return fail(CHITU_E_INVALID, "attn_fwd: destination strides must be multiples of 8 elements");
    for (int i = 0; i < sc.n_dest; ++i)
      if (!sc.ptrs[i] || (reinterpret_cast<uintptr_t>(sc.ptrs[i]) & 15))
        return fail(CHITU_E_INVALID, "attn_fwd: destination %d null or not 16-byte aligned", i);
  }
  if (B <= 0 || H <= 0 || Sq <= 0 || Sk <= 0)
    return fail(CHITU_E_INVALID, "attn_fwd: B, H, Sq, Sk must be positive (got %d, %d, %d, %d)", B, H, Sq, Sk);
  if (D != chitu::kHeadDim) return fail(CHITU_E_UNSUPPORTED, "attn_fwd: head_dim %d not supported (only 128)", D);
  if (dtype != CHITU_DTYPE_BF16 && dtype != CHITU_DTYPE_FP16)
    return fail(CHITU_E_UNSUPPORTED, "attn_fwd: dtype must be bf16 or fp16");
  if (!(softmax_scale > 0.f)) return fail(CHITU_E_UNSUPPORTED, "attn_fwd: softmax_scale must be positive");
  if (sc.n_dest == 0 && (reinterpret_cast<uintptr_t>(out) & 15))
    return fail(CHITU_E_INVALID, "attn_fwd: out must be 16-byte aligned");
  if (H > 65535 || B > 65535) return fail(CHITU_E_UNSUPPORTED, "attn_fwd: H and B must be below 65536");

  if (ks.n_splits < 1 || ks.n_splits > 64) return fail(CHITU_E_INVALID, "attn_fwd: n_splits must be in 1..64");
  const SplitPlan plan = plan_key_splits(Sk, ks.n_splits);
  const int n_splits = plan.n_splits, tiles_per_split = plan.tiles_per_split;
  if (n_splits > 1) {
    if (!ks.workspace || (reinterpret_cast<uintptr_t>(ks.workspace) & 15))
      return fail(CHITU_E_INVALID, "attn_fwd: split over keys needs a 16-byte aligned workspace");
    if (ks.workspace_bytes < splitkv_workspace_bytes(B, Sq, H, D, n_splits))
      return fail(CHITU_E_INVALID, "attn_fwd: workspace too small (%lld bytes needed)",
                  (long long)splitkv_workspace_bytes(B, Sq, H, D, n_splits));
    if (static_cast<int64_t>(B) * n_splits > 65535) return fail(CHITU_E_UNSUPPORTED, "attn_fwd: B * n_splits too large");
    const int64_t qblocks = (Sq + chitu::kQTiles * chitu::kTileM - 1) / (chitu::kQTiles * chitu::kTileM);
    if (static_cast<int64_t>(B) * H * qblocks * 4 > kSplitHeaderBytes)
      return fail(CHITU_E_UNSUPPORTED, "attn_fwd: a split over keys serves at most %lld query blocks x heads x batch",
                  (long long)(kSplitHeaderBytes / 4));
  }

  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_qkv_map(&tq, q, B, Sq, H, q_strides, "q")) != CHITU_OK) return rc;
  if ((rc = make_qkv_map(&tk, k, B, Sk, H, k_strides, "k")) != CHITU_OK) return rc;
  if ((rc = make_qkv_map(&tv, v, B, Sk, H, v_strides, "v")) != CHITU_OK) return rc;

  chitu::AttnParams p;
  p.out = out;
  p.lse = lse;
  p.status = status;
  p.B = B;
  p.H = H;
  p.Sq = Sq;
  p.Sk = Sk;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.is_fp16 = dtype == CHITU_DTYPE_FP16;
  p.n_dest = sc.n_dest;
  p.rows_per_dest = sc.rows_per_dest;
  p.dest_batch_bytes = sc.batch_stride * 2;
  p.dest_row_bytes = sc.row_stride * 2;
  p.dest_head_bytes = sc.head_offset * 2;
  for (int i = 0; i < 8; ++i) p.out_ptrs[i] = i < sc.n_dest ? sc.ptrs[i] : nullptr;
  p.n_splits = n_splits;
  p.tiles_per_split = tiles_per_split;
  p.split_count = static_cast<int*>(ks.workspace);
  p.part_o = p.part_lse = nullptr;
  if (n_splits > 1) {
    const int64_t qblocks = (Sq + chitu::kQTiles * chitu::kTileM - 1) / (chitu::kQTiles * chitu::kTileM);
    const size_t rows = static_cast<size_t>(B) * H * qblocks * chitu::kQTiles * chitu::kTileM;
    p.part_o = reinterpret_cast<float*>(static_cast<uint8_t*>(ks.workspace) + kSplitHeaderBytes);
    p.part_lse = p.part_o + static_cast<size_t>(n_splits) * rows * D;
  }
  p.q_norm_mode = 2;
  p.q_rope_mode = 0;
  p.q_round_mid = 0;
  p.q_w_dtype = CHITU_DTYPE_FP32;
  p.q_weight = nullptr;
  p.q_rstd = nullptr;
  p.q_eps = 0.f;
  p.q_table = nullptr;
  p.q_table_rows = p.q_gf = p.q_gh = p.q_gw = p.q_n_t = p.q_n_h = 0;
  p.q_pos_offset = 0;
  if (qpre != nullptr) {
    if (qpre->norm_mode < 0 || qpre->norm_mode > 2 || qpre->rope_mode < 0 || qpre->rope_mode > 2)
      return fail(CHITU_E_INVALID, "attn_fwd_qpre: bad mode");
    if (qpre->norm_mode == 0 && !qpre->rstd)
      return fail(CHITU_E_INVALID, "attn_fwd_qpre: full-width norm needs the per-token rstd vector");
    if (qpre->w_dtype < 0 || qpre->w_dtype > 2) return fail(CHITU_E_INVALID, "attn_fwd_qpre: bad weight dtype");
    if (qpre->rope_mode != 0) {
      if (!qpre->rope_table || qpre->table_rows <= 0) return fail(CHITU_E_INVALID, "attn_fwd_qpre: rope table missing");
      if (qpre->pos_offset < 0 || qpre->pos_offset + Sq >= (1LL << 31))
        return fail(CHITU_E_UNSUPPORTED, "attn_fwd_qpre: positions must stay below 2^31");
      if (qpre->rope_mode == 1) {
        if (qpre->gf <= 0 || qpre->gh <= 0 || qpre->gw <= 0 || qpre->n_t < 0 || qpre->n_h < 0 ||
            qpre->n_t + qpre->n_h > D / 2)
          return fail(CHITU_E_INVALID, "attn_fwd_qpre: grid / axis split out of range");
        if (qpre->gf > qpre->table_rows || qpre->gh > qpre->table_rows || qpre->gw > qpre->table_rows)
          return fail(CHITU_E_INVALID, "attn_fwd_qpre: rope table has fewer rows than the grid extent");
      }
    }
    p.q_norm_mode = qpre->norm_mode;
    p.q_rope_mode = qpre->rope_mode;
    p.q_round_mid = qpre->round_mid;
    p.q_w_dtype = qpre->w_dtype;
    p.q_weight = qpre->weight;
    p.q_rstd = qpre->rstd;
    p.q_eps = qpre->eps;
    p.q_table = reinterpret_cast<const float2*>(qpre->rope_table);
    p.q_table_rows = qpre->table_rows;
    p.q_gf = qpre->gf;
    p.q_gh = qpre->gh;
    p.q_gw = qpre->gw;
    p.q_n_t = qpre->n_t;
    p.q_n_h = qpre->n_h;
    p.q_pos_offset = qpre->pos_offset;
  }
  p.prefix_rows = 0;
  for (int i = 0; i < 8; ++i) p.prefix_ptrs[i] = nullptr;
  p.prefix_batch_bytes = p.prefix_row_bytes = p.prefix_head_bytes = 0;
  p.in_flags = nullptr;
  p.in_epoch = nullptr;
  p.rows_per_src = p.local_src = 0;
  p.flag_timeout = g_flag_wait_cycles;
  p.signal_out = 0;
  for (int i = 0; i < 8; ++i) p.sync.blocks[i] = nullptr;
  p.sync.rank = p.sync.world = 0;
  p.sync.timeout_cycles = g_flag_wait_cycles;
  if (ex.sync != nullptr) {
    if ((rc = fill_peer_sync(&p.sync, ex.sync, "attn_fwd_exchange")) != CHITU_OK) return rc;
    if (ex.rows_per_src <= 0 ||
        static_cast<int64_t>(ex.rows_per_src) * p.sync.world + ex.prefix_rows < (Sq > Sk ? Sq : Sk))
      return fail(CHITU_E_INVALID, "attn_fwd_exchange: prefix_rows + rows_per_src * world must cover the sequence");
    if (ex.prefix_rows < 0 || (ex.prefix_rows > 0 && (!ex.prefix_ptrs || sc.n_dest <= 0)))
      return fail(CHITU_E_INVALID, "attn_fwd_exchange: a replicated prefix needs its destination buffers");
    if ((ex.prefix_batch_stride | ex.prefix_row_stride | ex.prefix_head_offset) & 7)
      return fail(CHITU_E_INVALID, "attn_fwd_exchange: prefix strides must be multiples of 8 elements");
    for (int i = 0; i < sc.n_dest && ex.prefix_rows > 0; ++i)
      if (!ex.prefix_ptrs[i] || (reinterpret_cast<uintptr_t>(ex.prefix_ptrs[i]) & 15))
        return fail(CHITU_E_INVALID, "attn_fwd_exchange: prefix destination %d null or not 16-byte aligned", i);
    p.prefix_rows = ex.prefix_rows;
    for (int i = 0; i < sc.n_dest && ex.prefix_rows > 0; ++i) p.prefix_ptrs[i] = ex.prefix_ptrs[i];
    p.prefix_batch_bytes = ex.prefix_batch_stride * 2;
    p.prefix_row_bytes = ex.prefix_row_stride * 2;
    p.prefix_head_bytes = ex.prefix_head_offset * 2;
    p.in_flags = p.sync.blocks[p.sync.rank] + chitu::kSyncInFlag;
    p.in_epoch = p.sync.blocks[p.sync.rank] + chitu::kSyncInEpoch;
    p.rows_per_src = ex.rows_per_src;
    p.local_src = p.sync.rank;
    p.signal_out = 1;
  }
  p.cluster_merge = (n_splits == 2 && g_cluster_merge) ? 1 : 0;
  // with the fused exchange the key ranges interleave, so that every CTA of a query block holds own rows
  p.split_strided = (ex.sync != nullptr && n_splits > 1) ? 1 : 0;
  p.push_ctas = p.grid_q = p.grid_h = p.grid_z = p.push_rounds = p.push_first = p.rot_other = 0;
  p.push_vecs = 0;
  p.q_flags = nullptr;
  for (int t = 0; t < 3; ++t) {
    p.push_src[t] = nullptr;
    for (int i = 0; i < 8; ++i) p.push_dst[t][i] = nullptr;
  }
  for (int i = 0; i < 8; ++i) p.push_order[i] = 0;
  if (ex.push != nullptr) {
    const int world = p.sync.world, me = p.sync.rank;
    if (ex.sync == nullptr || world < 2) return fail(CHITU_E_INVALID, "attn_fwd_exchange_push: needs a sync descriptor");
    if (ex.prefix_rows != 0 || qpre != nullptr)
      return fail(CHITU_E_UNSUPPORTED, "attn_fwd_exchange_push: no replicated prefix, no in-kernel q transform");
    if (ex.push->block_bytes <= 0 || (ex.push->block_bytes & 15))
      return fail(CHITU_E_INVALID, "attn_fwd_exchange_push: block_bytes must be a positive multiple of 16");
    p.push_ctas = plan_push_ctas(B, Sq, H, n_splits);
    if (p.push_ctas == 0) return fail(CHITU_E_UNSUPPORTED, "attn_fwd_exchange_push: this device has too few SMs");
    p.grid_q = (Sq + chitu::kQTiles * chitu::kTileM - 1) / (chitu::kQTiles * chitu::kTileM);
    p.grid_h = H;
    p.grid_z = B * n_splits;
    if (static_cast<int64_t>(p.grid_q) * H * B * n_splits + p.push_ctas >= (1LL << 31))
      return fail(CHITU_E_UNSUPPORTED, "attn_fwd_exchange_push: grid too large");
    for (int t = 0; t < 3; ++t) {
      if (t == 0 && !ex.push->stage[0]) continue;  // query rows were delivered by the staging launch
      if (!ex.push->stage[t] || (reinterpret_cast<uintptr_t>(ex.push->stage[t]) & 15) || !ex.push->dest[t])
        return fail(CHITU_E_INVALID, "attn_fwd_exchange_push: staging area %d null or misaligned", t);
      p.push_src[t] = static_cast<const uint4*>(ex.push->stage[t]);
      for (int i = 0; i < world; ++i) {
        if (i == me) continue;
        if (!ex.push->dest[t][i] || (reinterpret_cast<uintptr_t>(ex.push->dest[t][i]) & 15))
          return fail(CHITU_E_INVALID, "attn_fwd_exchange_push: destination %d of tensor %d null or misaligned", i, t);
        p.push_dst[t][i] = static_cast<uint4*>(ex.push->dest[t][i]);
      }
    }
    p.push_vecs = ex.push->block_bytes / 16;
    p.q_flags = p.sync.blocks[me] + chitu::kSyncQFlag;
    // Serve the peers in the order in which they will ask for this rank's rows: receiver d walks the source
    // ranks of a key range upwards, starting at itself where the range holds it, at the range's first
    // source otherwise.
    const int ranges = (!p.split_strided && world % n_splits == 0) ? n_splits : 1;
    const int len = world / ranges;
    int pos[8], n = 0;
    for (int d = 0; d < world; ++d) {
      if (d == me) continue;
      const int lo = me / len * len;
      pos[d] = (d / len == me / len) ? (me - d + len) % len : (me - lo - d % len + len) % len;
      p.push_order[n++] = d;
    }
    for (int i = 1; i < n; ++i)  // insertion sort by (position in the receiver's walk, distance)
      for (int j = i; j > 0; --j) {
        const int a = p.push_order[j - 1], b = p.push_order[j];
        const int da = (me - a + world) % world, db = (me - b + world) % world;
        if (pos[a] < pos[b] || (pos[a] == pos[b] && da <= db)) break;
        p.push_order[j - 1] = b;
        p.push_order[j] = a;
      }
    p.push_rounds = n;
    p.push_first = (n + 1) / 2;
    // a CTA whose key range holds none of this rank's own rows starts its walk at a source that depends on
    // the rank, so that the receivers do not all ask the same source first
    p.rot_other = static_cast<int>((static_cast<long long>(me % len) * ex.rows_per_src) / chitu::kTileN);
  }
#ifdef CHITU_ATTN_TIMING
  p.dbg = g_dbg;
#endif

  static bool attr_done[2][kMaxDevices] = {};
  static std::mutex attr_mu;
  const cudaError_t attr_err =
      p.is_fp16 ? ensure_dynamic_smem(chitu::attn_fwd_kernel<true>, chitu::kAttnSmemBytes, attr_done[1], attr_mu)
                : ensure_dynamic_smem(chitu::attn_fwd_kernel<false>, chitu::kAttnSmemBytes, attr_done[0], attr_mu);
  if (attr_err != cudaSuccess) return cuda_fail(attr_err, "attn_fwd: cudaFuncSetAttribute");

  const unsigned qblocks_x = (Sq + chitu::kQTiles * chitu::kTileM - 1) / (chitu::kQTiles * chitu::kTileM);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(chitu::kAttnThreads);
  cfg.dynamicSmemBytes = chitu::kAttnSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute cluster_attr[1];
  auto set_grid = [&]() {
    cfg.gridDim = dim3(qblocks_x, B * n_splits, H);
    if (p.push_ctas > 0) cfg.gridDim = dim3(p.push_ctas + p.grid_q * p.grid_h * p.grid_z, 1, 1);
    cfg.numAttrs = 0;
    cfg.attrs = nullptr;
    if (p.cluster_merge) {  // the two key ranges of a query block: neighbours along y, or along x in the 1-d grid
      cluster_attr[0].id = cudaLaunchAttributeClusterDimension;
      cluster_attr[0].val.clusterDim.x = p.push_ctas > 0 ? 2 : 1;
      cluster_attr[0].val.clusterDim.y = p.push_ctas > 0 ? 1 : 2;
      cluster_attr[0].val.clusterDim.z = 1;
      cfg.attrs = cluster_attr;
      cfg.numAttrs = 1;
    }
  };
  if (p.cluster_merge && p.push_ctas > 0) {
    // Copy CTAs pair up like everything else in a clustered grid, and the grid should stay resident at once
    // where it was going to be: ask how many clusters fit and give the copy CTAs what the attention leaves.
    p.push_ctas &= ~1;
    set_grid();
    int max_clusters = 0;
    const cudaError_t oe = p.is_fp16
        ? cudaOccupancyMaxActiveClusters(&max_clusters, chitu::attn_fwd_kernel<true>, &cfg)
        : cudaOccupancyMaxActiveClusters(&max_clusters, chitu::attn_fwd_kernel<false>, &cfg);
    const long long attn_ctas = static_cast<long long>(p.grid_q) * p.grid_h * p.grid_z;
    if (oe != cudaSuccess || max_clusters <= 0) {
      (void)cudaGetLastError();
      p.cluster_merge = 0;
    } else if (attn_ctas + p.push_ctas > 2LL * max_clusters && attn_ctas < 2LL * max_clusters) {
      const long long room = 2LL * max_clusters - attn_ctas;
      if (room >= 8) p.push_ctas = static_cast<int>(room < 48 ? room : 48) & ~1;
      else p.cluster_merge = 0;
    }
  }
  set_grid();
  {
    const cudaError_t le = p.is_fp16 ? cudaLaunchKernelEx(&cfg, chitu::attn_fwd_kernel<true>, tq, tk, tv, p)
                                     : cudaLaunchKernelEx(&cfg, chitu::attn_fwd_kernel<false>, tq, tk, tv, p);
    if (le != cudaSuccess) return cuda_fail(le, "attn_fwd: launch");
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "attn_fwd: launch");
  return CHITU_OK;
}

}  // namespace

extern "C" {

int chitu_b200_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int Sq, int Sk,
                        int H, int D, const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                        float softmax_scale, int dtype, int* status, void* stream) {
  return attn_fwd_impl(q, k, v, out, OutScatter{}, lse, B, Sq, Sk, H, D, q_strides, k_strides, v_strides,
                       softmax_scale, dtype, status, stream);
}

int64_t chitu_b200_attn_splitkv_workspace_bytes(int B, int Sq, int H, int D, int n_splits) {
  return splitkv_workspace_bytes(B, Sq, H, D, n_splits);
}

int chitu_b200_attn_fwd_splitkv(const void* q, const void* k, const void* v, void* out, float* lse, int B, int Sq,
                                int Sk, int H, int D, const int64_t* q_strides, const int64_t* k_strides,
                                const int64_t* v_strides, float softmax_scale, int dtype, int n_splits,
                                void* workspace, int64_t workspace_bytes, int* status, void* stream) {
  KeySplit ks;
  ks.n_splits = n_splits;
  ks.workspace = workspace;
  ks.workspace_bytes = workspace_bytes;
  return attn_fwd_impl(q, k, v, out, OutScatter{}, lse, B, Sq, Sk, H, D, q_strides, k_strides, v_strides,
                       softmax_scale, dtype, status, stream, ks);
}

int chitu_b200_attn_fwd_scatter(const void* q, const void* k, const void* v, void* const* out_ptrs, int n_dest,
                                int rows_per_dest, int64_t dest_batch_stride, int64_t dest_row_stride,
                                int64_t dest_head_offset, float* lse, int B, int Sq, int Sk, int H, int D,
                                const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                float softmax_scale, int dtype, int n_splits, void* workspace,
                                int64_t workspace_bytes, int* status, void* stream) {
  KeySplit ks;
  ks.n_splits = n_splits;
  ks.workspace = workspace;
  ks.workspace_bytes = workspace_bytes;
  OutScatter sc;
  sc.ptrs = out_ptrs;
  sc.n_dest = n_dest;
  sc.rows_per_dest = rows_per_dest;
  sc.batch_stride = dest_batch_stride;
  sc.row_stride = dest_row_stride;
  sc.head_offset = dest_head_offset;
  if (n_dest <= 0) return fail(CHITU_E_INVALID, "attn_fwd_scatter: n_dest must be positive");
  return attn_fwd_impl(q, k, v, nullptr, sc, lse, B, Sq, Sk, H, D, q_strides, k_strides, v_strides, softmax_scale,
                       dtype, status, stream, ks);
}

int chitu_b200_attn_fwd_exchange(const void* q, const void* k, const void* v, void* const* out_ptrs, int n_dest,
                                 int rows_per_dest, int64_t dest_batch_stride, int64_t dest_row_stride,
                                 int64_t dest_head_offset, int B, int Sq, int Sk, int H, int D,
                                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                 float softmax_scale, int dtype, int n_splits, void* workspace,
                                 int64_t workspace_bytes, int rows_per_src, int prefix_rows,
                                 void* const* prefix_ptrs, int64_t prefix_batch_stride, int64_t prefix_row_stride,
                                 int64_t prefix_head_offset, const chitu_b200_peer_sync* sync, int* status,
                                 void* stream) {
  KeySplit ks;
  ks.n_splits = n_splits;
  ks.workspace = workspace;
  ks.workspace_bytes = workspace_bytes;
  OutScatter sc;
  sc.ptrs = out_ptrs;
  sc.n_dest = n_dest;
  sc.rows_per_dest = rows_per_dest;
  sc.batch_stride = dest_batch_stride;
  sc.row_stride = dest_row_stride;
  sc.head_offset = dest_head_offset;
  if (n_dest <= 0) return fail(CHITU_E_INVALID, "attn_fwd_exchange: n_dest must be positive");
  if (!sync) return fail(CHITU_E_INVALID, "attn_fwd_exchange: sync descriptor missing");
  Exchange ex;
  ex.sync = sync;
  ex.rows_per_src = rows_per_src;
  ex.prefix_rows = prefix_rows;
  ex.prefix_ptrs = prefix_ptrs;
  ex.prefix_batch_stride = prefix_batch_stride;
  ex.prefix_row_stride = prefix_row_stride;
  ex.prefix_head_offset = prefix_head_offset;
  return attn_fwd_impl(q, k, v, nullptr, sc, nullptr, B, Sq, Sk, H, D, q_strides, k_strides, v_strides, softmax_scale,
                       dtype, status, stream, ks, ex);
}

int chitu_b200_push_ctas(int B, int Sq, int H, int n_splits) {
  if (B <= 0 || Sq <= 0 || H <= 0 || n_splits < 1) return 0;
  return plan_push_ctas(B, Sq, H, n_splits);
}

int chitu_b200_attn_fwd_exchange_push(const void* q, const void* k, const void* v, void* const* out_ptrs, int n_dest,
                                      int rows_per_dest, int64_t dest_batch_stride, int64_t dest_row_stride,
                                      int64_t dest_head_offset, int B, int Sq, int Sk, int H, int D,
                                      const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                      float softmax_scale, int dtype, int n_splits, void* workspace,
                                      int64_t workspace_bytes, int rows_per_src, const chitu_b200_push* push,
                                      const chitu_b200_peer_sync* sync, int* status, void* stream) {
  KeySplit ks;
  ks.n_splits = n_splits;
  ks.workspace = workspace;
  ks.workspace_bytes = workspace_bytes;
  OutScatter sc;
  sc.ptrs = out_ptrs;
  sc.n_dest = n_dest;
  sc.rows_per_dest = rows_per_dest;
  sc.batch_stride = dest_batch_stride;
  sc.row_stride = dest_row_stride;
  sc.head_offset = dest_head_offset;
  if (n_dest <= 0) return fail(CHITU_E_INVALID, "attn_fwd_exchange_push: n_dest must be positive");
  if (!sync || !push) return fail(CHITU_E_INVALID, "attn_fwd_exchange_push: sync or push descriptor missing");
  Exchange ex;
  ex.sync = sync;
  ex.rows_per_src = rows_per_src;
  ex.push = push;
  return attn_fwd_impl(q, k, v, nullptr, sc, nullptr, B, Sq, Sk, H, D, q_strides, k_strides, v_strides, softmax_scale,
                       dtype, status, stream, ks, ex);
}

int chitu_b200_attn_fwd_qpre(const void* q_raw, const void* k, const void* v, void* out, float* lse, int B, int Sq, int Sk,
                             int H, int D, const int64_t* q_strides, const int64_t* k_strides,
                             const int64_t* v_strides, float softmax_scale, int dtype, const chitu_b200_q_pre* q_pre,
                             int n_splits, void* workspace, int64_t workspace_bytes, int* status, void* stream) {
  if (!q_pre) return fail(CHITU_E_INVALID, "attn_fwd_qpre: transform descriptor missing");
  KeySplit ks;
  ks.n_splits = n_splits;
  ks.workspace = workspace;
  ks.workspace_bytes = workspace_bytes;
  return attn_fwd_impl(q_raw, k, v, out, OutScatter{}, lse, B, Sq, Sk, H, D, q_strides, k_strides, v_strides,
                       softmax_scale, dtype, status, stream, ks, Exchange{}, q_pre);
}

int chitu_b200_peer_wait_outputs(const chitu_b200_peer_sync* sync, int* status, void* stream) {
  chitu::PeerSync ps;
  int rc = fill_peer_sync(&ps, sync, "peer_wait_outputs");
  if (rc != CHITU_OK) return rc;
  chitu::peer_wait_outputs_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ps, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "peer_wait_outputs: launch");
  return CHITU_OK;
}

int chitu_b200_lse_combine(float* acc_out, float* acc_lse, const void* block_out, const float* block_lse, int B, int S,
                           int H, int D, int block_dtype, int first, void* final_out, int final_dtype, void* stream) {
  if (!acc_out || !acc_lse || !block_out || !block_lse) return fail(CHITU_E_INVALID, "lse_combine: null pointer");
  if (B <= 0 || S <= 0 || H <= 0 || D <= 0 || (D & 3))
    return fail(CHITU_E_INVALID, "lse_combine: bad shape (D must be a multiple of 4)");
  if (block_dtype < 0 || block_dtype > 2 || (final_out && (final_dtype < 0 || final_dtype > 2)))
    return fail(CHITU_E_INVALID, "lse_combine: bad dtype");
  if ((reinterpret_cast<uintptr_t>(acc_out) | reinterpret_cast<uintptr_t>(block_out) |
       reinterpret_cast<uintptr_t>(final_out)) & 15)
    return fail(CHITU_E_INVALID, "lse_combine: buffers must be 16-byte aligned");
  const long long rows = static_cast<long long>(B) * S * H;
  const int grid = grid_for(rows, 8, 148 * 16);
  chitu::lse_combine_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      acc_out, acc_lse, block_out, block_lse, B, S, H, D, block_dtype, first, final_out, final_dtype);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "lse_combine: launch");
  return CHITU_OK;
}

}  // extern "C"

namespace {

struct NormRopeShared {
  int in_dtype, w_dtype;
  float eps;
  const float* rope_table;
  int table_rows, gf, gh, gw;
  const int* axis_split;
  int64_t pos_offset;
  int out_dtype;
  const int64_t* out_strides;
  int heads_per_group, B, S, H, D, round_mid;
};

int qk_norm_rope_batch_impl(const chitu_b200_norm_rope_job* jobs, int n_jobs, const NormRopeShared& sh, void* stream,
                            const chitu_b200_peer_sync* sync = nullptr, bool stage_only = false) {
  if (!jobs || n_jobs < 1 || n_jobs > 3) return fail(CHITU_E_INVALID, "qk_norm_rope: 1..3 jobs per launch");
  if (!sh.out_strides) return fail(CHITU_E_INVALID, "qk_norm_rope: null pointer");
  const int B = sh.B, S = sh.S, H = sh.H, D = sh.D;
  if (B <= 0 || S <= 0 || H <= 0 || D <= 0) return fail(CHITU_E_INVALID, "qk_norm_rope: bad shape");
  if (static_cast<long long>(B) * S + 4096LL * 8 >= (1LL << 31) || sh.pos_offset < 0 ||
      sh.pos_offset + S >= (1LL << 31))
    return fail(CHITU_E_UNSUPPORTED, "qk_norm_rope: token count and positions must stay below 2^31");
  if (D & 7) return fail(CHITU_E_INVALID, "qk_norm_rope: head_dim must be a multiple of 8");
  const long long C = static_cast<long long>(H) * D;
  if (C > chitu::kNormMaxThreads * 8)
    return fail(CHITU_E_UNSUPPORTED, "qk_norm_rope: at most %d channels per token", chitu::kNormMaxThreads * 8);
  if (sh.in_dtype < 0 || sh.in_dtype > 2 || (sh.out_dtype != CHITU_DTYPE_BF16 && sh.out_dtype != CHITU_DTYPE_FP16))
    return fail(CHITU_E_INVALID, "qk_norm_rope: bad dtype");
  if (sh.w_dtype < 0 || sh.w_dtype > 2) return fail(CHITU_E_INVALID, "qk_norm_rope: bad weight dtype");
  if (sh.heads_per_group <= 0 || H % sh.heads_per_group)
    return fail(CHITU_E_INVALID, "qk_norm_rope: heads_per_group must divide H");
  for (int i = 0; i < 4; ++i)
    if (sh.out_strides[i] & 7) return fail(CHITU_E_INVALID, "qk_norm_rope: out_strides must be multiples of 8 elements");
  const long long tokens = static_cast<long long>(B) * S;
  if (tokens > 2147483647LL) return fail(CHITU_E_UNSUPPORTED, "qk_norm_rope: too many tokens");

  chitu::NormRopeBatch batch;
  batch.signal = 0;
  for (int i = 0; i < 8; ++i) batch.sync.blocks[i] = nullptr;
  batch.sync.rank = batch.sync.world = 0;
  batch.sync.timeout_cycles = g_flag_wait_cycles;
  if (sync != nullptr) {
    const int rc = fill_peer_sync(&batch.sync, sync, "qk_norm_rope_batch_signal");
    if (rc != CHITU_OK) return rc;
    batch.signal = stage_only ? 2 : 1;
  }
  for (int j = 0; j < n_jobs; ++j) {
    const chitu_b200_norm_rope_job& jb = jobs[j];
    chitu::NormRopeParams& p = batch.job[j];
    if (!jb.x || (!jb.out && jb.n_out_ptrs == 0 && !jb.rstd_out))
      return fail(CHITU_E_INVALID, "qk_norm_rope: null pointer");
    if (jb.rstd_out && jb.norm_mode != 0)
      return fail(CHITU_E_INVALID, "qk_norm_rope: a statistics-only job needs norm_mode 0");
    if (jb.n_out_ptrs != 0) {
      if (jb.n_out_ptrs < 0 || jb.n_out_ptrs > 8 || !jb.out_ptrs || jb.n_out_ptrs * sh.heads_per_group != H)
        return fail(CHITU_E_INVALID, "qk_norm_rope: need one destination per head group (at most 8)");
      bool any = false;
      for (int i = 0; i < jb.n_out_ptrs; ++i) {
        if (reinterpret_cast<uintptr_t>(jb.out_ptrs[i]) & 15)
          return fail(CHITU_E_INVALID, "qk_norm_rope: destination %d not 16-byte aligned", i);
        any = any || jb.out_ptrs[i] != nullptr;  // a null entry drops that head group
      }
      if (!any) return fail(CHITU_E_INVALID, "qk_norm_rope: every destination is null");
    }
    if (jb.norm_mode < 0 || jb.norm_mode > 2 || jb.rope_mode < 0 || jb.rope_mode > 2)
      return fail(CHITU_E_INVALID, "qk_norm_rope: bad mode");
    if (jb.norm_mode == 1) {
      const int vph = D >> 3;
      if (vph > 32 || (vph & (vph - 1)))
        return fail(CHITU_E_UNSUPPORTED, "qk_norm_rope: per-head norm needs D in {8..256} power of two");
    }
    if (jb.x_row_stride < C || (jb.x_row_stride * elem_size(sh.in_dtype)) % 16)
      return fail(CHITU_E_INVALID, "qk_norm_rope: x_row_stride must cover H*D and keep rows 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(jb.x) | reinterpret_cast<uintptr_t>(jb.out)) & 15)
      return fail(CHITU_E_INVALID, "qk_norm_rope: x and out must be 16-byte aligned");
    p.n_t = p.n_h = 0;
    if (jb.rope_mode != 0) {
      if (!sh.rope_table || sh.table_rows <= 0) return fail(CHITU_E_INVALID, "qk_norm_rope: rope table missing");
      if (jb.rope_mode == 1) {
        if (!sh.axis_split || sh.gf <= 0 || sh.gh <= 0 || sh.gw <= 0)
          return fail(CHITU_E_INVALID, "qk_norm_rope: grid / axis_split missing");
        if (sh.axis_split[0] < 0 || sh.axis_split[1] < 0 || sh.axis_split[0] + sh.axis_split[1] > D / 2)
          return fail(CHITU_E_INVALID, "qk_norm_rope: axis_split out of range");
        if (sh.gf > sh.table_rows || sh.gh > sh.table_rows || sh.gw > sh.table_rows)
          return fail(CHITU_E_INVALID, "qk_norm_rope: rope table has fewer rows than the grid extent");
        p.n_t = sh.axis_split[0];
        p.n_h = sh.axis_split[1];
      }
    }
    p.x = jb.x;
    p.in_dtype = sh.in_dtype;
    p.x_row_stride = jb.x_row_stride;
    p.weight = jb.weight;
    p.w_dtype = sh.w_dtype;
    p.eps = sh.eps;
    p.norm_mode = jb.norm_mode;
    p.rope_mode = jb.rope_mode;
    p.table = reinterpret_cast<const float2*>(sh.rope_table);
    p.table_rows = sh.table_rows;
    p.gf = sh.gf;
    p.gh = sh.gh;
    p.gw = sh.gw;
    p.pos_offset = sh.pos_offset;
    p.out = jb.out;
    p.out_dtype = sh.out_dtype;
    p.os_b = sh.out_strides[0];
    p.os_s = sh.out_strides[1];
    p.os_g = sh.out_strides[2];
    p.os_h = sh.out_strides[3];
    p.heads_per_group = sh.heads_per_group;
    p.B = B;
    p.S = S;
    p.H = H;
    p.D = D;
    p.round_mid = sh.round_mid;
    p.n_out_ptrs = jb.n_out_ptrs;
    for (int i = 0; i < 8; ++i) p.out_ptrs[i] = i < jb.n_out_ptrs ? jb.out_ptrs[i] : nullptr;
    p.rstd_out = jb.rstd_out;
  }
  // one 8-channel vector per thread, whole warps; the grid fills the 148 SMs a few CTAs deep
  const int threads = static_cast<int>(((C / 8) + 31) / 32 * 32);
  // CTAs that can be resident per SM: 80 registers per thread up to 512 threads, 64 above
  const int per_sm = std::max(1, std::min(2048 / threads, 65536 / (threads * (threads <= 512 ? 80 : 64))));
  const int per_job = (per_sm + n_jobs - 1) / n_jobs;
  const long long tok_per_iter = sh.in_dtype == CHITU_DTYPE_FP32 ? 2 : 4;  // NormRopeTokens
  const long long iters = (tokens + tok_per_iter - 1) / tok_per_iter;
  const unsigned gx = static_cast<unsigned>(iters < 148LL * per_job ? iters : 148LL * per_job);
  const dim3 grid(gx, n_jobs);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the kernel is specialised on the modes of job 0; other jobs either share them or are plain
  const int nm = jobs[0].norm_mode, rm = jobs[0].rope_mode;
  for (int j = 1; j < n_jobs; ++j) {
    const bool same = jobs[j].norm_mode == nm && jobs[j].rope_mode == rm;
    const bool plain = jobs[j].norm_mode == 2 && jobs[j].rope_mode == 0;
    if (!same && !plain) return fail(CHITU_E_UNSUPPORTED, "qk_norm_rope: jobs of one launch share modes or are plain copies");
  }
#define CHITU_NR_LAUNCH(IN, NM, RM)                                                    \
  if (threads <= 512)                                                                  \
    chitu::qk_norm_rope_kernel<IN, NM, RM><<<grid, threads, 0, st>>>(batch);           \
  else                                                                                 \
    chitu::qk_norm_rope_wide_kernel<IN, NM, RM><<<grid, threads, 0, st>>>(batch)
#define CHITU_NR_ROPE(IN, NM)                     \
  switch (rm) {                                   \
    case 0: CHITU_NR_LAUNCH(IN, NM, 0); break;    \
    case 1: CHITU_NR_LAUNCH(IN, NM, 1); break;    \
    default: CHITU_NR_LAUNCH(IN, NM, 2); break;   \
  }
#define CHITU_NR_NORM(IN)                         \
  switch (nm) {                                   \
    case 0: CHITU_NR_ROPE(IN, 0); break;          \
    case 1: CHITU_NR_ROPE(IN, 1); break;          \
    default: CHITU_NR_ROPE(IN, 2); break;         \
  }
  switch (sh.in_dtype) {
    case CHITU_DTYPE_BF16: CHITU_NR_NORM(0); break;
    case CHITU_DTYPE_FP16: CHITU_NR_NORM(1); break;
    default: CHITU_NR_NORM(2); break;
  }
#undef CHITU_NR_NORM
#undef CHITU_NR_ROPE
#undef CHITU_NR_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "qk_norm_rope: launch");
  return CHITU_OK;
}

int qk_norm_rope_impl(const void* x, int in_dtype, int64_t x_row_stride, const void* weight, int w_dtype, float eps,
                      int norm_mode, int rope_mode, const float* rope_table, int table_rows, int gf, int gh, int gw,
                      const int* axis_split, int64_t pos_offset, void* out, void* const* out_ptrs, int n_out_ptrs,
                      int out_dtype, const int64_t* out_strides, int heads_per_group, int B, int S, int H, int D,
                      int round_mid, void* stream) {
  chitu_b200_norm_rope_job job;
  job.x = x;
  job.x_row_stride = x_row_stride;
  job.weight = weight;
  job.norm_mode = norm_mode;
  job.rope_mode = rope_mode;
  job.out = out;
  job.out_ptrs = out_ptrs;
  job.n_out_ptrs = n_out_ptrs;
  job.rstd_out = nullptr;
  NormRopeShared sh{in_dtype, w_dtype,  eps,         rope_table,      table_rows, gf, gh, gw, axis_split, pos_offset,
                    out_dtype, out_strides, heads_per_group, B, S, H, D, round_mid};
  return qk_norm_rope_batch_impl(&job, 1, sh, stream);
}

}  // namespace

extern "C" {

int chitu_b200_qk_norm_rope(const void* x, int in_dtype, int64_t x_row_stride, const void* weight, int w_dtype,
                            float eps, int norm_mode, int rope_mode, const float* rope_table, int table_rows, int gf,
                            int gh, int gw, const int* axis_split, int64_t pos_offset, void* out, int out_dtype,
                            const int64_t* out_strides, int heads_per_group, int B, int S, int H, int D, int round_mid,
                            void* stream) {
  return qk_norm_rope_impl(x, in_dtype, x_row_stride, weight, w_dtype, eps, norm_mode, rope_mode, rope_table,
                           table_rows, gf, gh, gw, axis_split, pos_offset, out, nullptr, 0, out_dtype, out_strides,
                           heads_per_group, B, S, H, D, round_mid, stream);
}

int chitu_b200_qk_norm_rope_scatter(const void* x, int in_dtype, int64_t x_row_stride, const void* weight,
                                    int w_dtype, float eps, int norm_mode, int rope_mode, const float* rope_table,
                                    int table_rows, int gf, int gh, int gw, const int* axis_split, int64_t pos_offset,
                                    void* const* out_ptrs, int n_out_ptrs, int out_dtype, const int64_t* out_strides,
                                    int heads_per_group, int B, int S, int H, int D, int round_mid, void* stream) {
  if (n_out_ptrs <= 0) return fail(CHITU_E_INVALID, "qk_norm_rope_scatter: n_out_ptrs must be positive");
  return qk_norm_rope_impl(x, in_dtype, x_row_stride, weight, w_dtype, eps, norm_mode, rope_mode, rope_table,
                           table_rows, gf, gh, gw, axis_split, pos_offset, nullptr, out_ptrs, n_out_ptrs, out_dtype,
                           out_strides, heads_per_group, B, S, H, D, round_mid, stream);
}

int chitu_b200_qk_norm_rope_batch(const chitu_b200_norm_rope_job* jobs, int n_jobs, int in_dtype, int w_dtype,
                                  float eps, const float* rope_table, int table_rows, int gf, int gh, int gw,
                                  const int* axis_split, int64_t pos_offset, int out_dtype,
                                  const int64_t* out_strides, int heads_per_group, int B, int S, int H, int D,
                                  int round_mid, void* stream) {
  NormRopeShared sh{in_dtype, w_dtype,  eps,         rope_table,      table_rows, gf, gh, gw, axis_split, pos_offset,
                    out_dtype, out_strides, heads_per_group, B, S, H, D, round_mid};
  return qk_norm_rope_batch_impl(jobs, n_jobs, sh, stream);
}

int chitu_b200_qk_norm_rope_batch_signal(const chitu_b200_norm_rope_job* jobs, int n_jobs, int in_dtype, int w_dtype,
                                         float eps, const float* rope_table, int table_rows, int gf, int gh, int gw,
                                         const int* axis_split, int64_t pos_offset, int out_dtype,
                                         const int64_t* out_strides, int heads_per_group, int B, int S, int H, int D,
                                         int round_mid, const chitu_b200_peer_sync* sync, void* stream) {
  if (!sync) return fail(CHITU_E_INVALID, "qk_norm_rope_batch_signal: sync descriptor missing");
  NormRopeShared sh{in_dtype, w_dtype,  eps,         rope_table,      table_rows, gf, gh, gw, axis_split, pos_offset,
                    out_dtype, out_strides, heads_per_group, B, S, H, D, round_mid};
  return qk_norm_rope_batch_impl(jobs, n_jobs, sh, stream, sync);
}

int chitu_b200_qk_norm_rope_batch_stage(const chitu_b200_norm_rope_job* jobs, int n_jobs, int in_dtype, int w_dtype,
                                        float eps, const float* rope_table, int table_rows, int gf, int gh, int gw,
                                        const int* axis_split, int64_t pos_offset, int out_dtype,
                                        const int64_t* out_strides, int heads_per_group, int B, int S, int H, int D,
                                        int round_mid, const chitu_b200_peer_sync* sync, void* stream) {
  if (!sync) return fail(CHITU_E_INVALID, "qk_norm_rope_batch_stage: sync descriptor missing");
  NormRopeShared sh{in_dtype, w_dtype,  eps,         rope_table,      table_rows, gf, gh, gw, axis_split, pos_offset,
                    out_dtype, out_strides, heads_per_group, B, S, H, D, round_mid};
  return qk_norm_rope_batch_impl(jobs, n_jobs, sh, stream, sync, /*stage_only=*/true);
}

int chitu_b200_peer_barrier(int* const* flag_ptrs, int rank, int world, int* status, void* stream) {
  if (!flag_ptrs || world < 1 || world > 8 || rank < 0 || rank >= world)
    return fail(CHITU_E_INVALID, "peer_barrier: need 1..8 ranks and a rank inside the group");
  chitu::PeerBarrierParams p;
  for (int i = 0; i < 8; ++i) p.flags[i] = i < world ? flag_ptrs[i] : nullptr;
  for (int i = 0; i < world; ++i)
    if (!p.flags[i]) return fail(CHITU_E_INVALID, "peer_barrier: null flag array for rank %d", i);
  p.rank = rank;
  p.world = world;
  p.status = status;
  p.timeout_cycles = g_flag_wait_cycles;
  chitu::peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "peer_barrier: launch");
  return CHITU_OK;
}

int chitu_b200_stamp(unsigned long long* slot, void* stream) {
  if (!slot || (reinterpret_cast<uintptr_t>(slot) & 7)) return fail(CHITU_E_INVALID, "stamp: slot null or misaligned");
  chitu::stamp_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(slot);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "stamp: launch");
  return CHITU_OK;
}

int chitu_b200_set_cluster_merge(int enable) {
  const int old = g_cluster_merge;
  if (enable >= 0) g_cluster_merge = enable ? 1 : 0;
  return old;
}

long long chitu_b200_set_flag_wait_cycles(long long cycles) {
  const long long old = g_flag_wait_cycles;
  if (cycles > 0) g_flag_wait_cycles = cycles;
  return old;
}

int chitu_b200_strided_copy(const void* src, void* dst, int64_t n0, int64_t n1, int64_t n2, int64_t n3,
                            int64_t row_bytes, const int64_t* src_strides_bytes, void* stream) {
  if (!src || !dst || !src_strides_bytes) return fail(CHITU_E_INVALID, "strided_copy: null pointer");
  if (n0 <= 0 || n1 <= 0 || n2 <= 0 || n3 <= 0 || row_bytes <= 0 || (row_bytes & 15))
    return fail(CHITU_E_INVALID, "strided_copy: extents must be positive and row_bytes a multiple of 16");
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)
    return fail(CHITU_E_INVALID, "strided_copy: src and dst must be 16-byte aligned");
  for (int i = 0; i < 4; ++i)
    if (src_strides_bytes[i] & 15) return fail(CHITU_E_INVALID, "strided_copy: strides must be multiples of 16 bytes");
  const long long row_vecs = row_bytes / 16;
  const long long total = n0 * n1 * n2 * n3 * row_vecs;
  const int grid = grid_for(total, 256 * 4, 148 * 8);
  chitu::strided_copy_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), static_cast<uint4*>(dst), n1, n2, n3, row_vecs, src_strides_bytes[0],
      src_strides_bytes[1], src_strides_bytes[2], src_strides_bytes[3], total);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "strided_copy: launch");
  return CHITU_OK;
}

int chitu_b200_layernorm_modulate(const void* x, int x_dtype, void* out, int out_dtype, int64_t rows, int64_t rows_per_batch, int C,
                                  const float* mul, int64_t mul_batch_stride, const float* add,
                                  int64_t add_batch_stride, int add_one, float eps, void* stream) {
  if (!x || !out) return fail(CHITU_E_INVALID, "layernorm_modulate: null pointer");
  if (rows <= 0 || rows_per_batch <= 0 || C <= 0 || (C & 3) || C > chitu::kLnThreads * chitu::kLnMaxVec * 4)
    return fail(CHITU_E_UNSUPPORTED, "layernorm_modulate: C must be a multiple of 4 up to %d",
                chitu::kLnThreads * chitu::kLnMaxVec * 4);
  if (out_dtype != CHITU_DTYPE_BF16 && out_dtype != CHITU_DTYPE_FP16)
    return fail(CHITU_E_UNSUPPORTED, "layernorm_modulate: out_dtype must be bf16 or fp16");
  if (x_dtype < 0 || x_dtype > 2) return fail(CHITU_E_UNSUPPORTED, "layernorm_modulate: x_dtype must be bf16, fp16 or fp32");
  if ((mul_batch_stride & 3) || (add_batch_stride & 3) ||
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(mul) | reinterpret_cast<uintptr_t>(add)) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 7))
    return fail(CHITU_E_INVALID, "layernorm_modulate: x, mul, add must be 16-byte aligned, out 8-byte aligned");
  chitu::LayerNormParams p;
  p.x = x;
  p.x_dtype = x_dtype;
  p.out = out;
  p.mul = mul;
  p.add = add;
  p.mul_batch_stride = mul_batch_stride;
  p.add_batch_stride = add_batch_stride;
  p.rows = rows;
  p.rows_per_batch = rows_per_batch;
  p.C = C;
  p.add_one = add_one;
  p.out_fp16 = out_dtype == CHITU_DTYPE_FP16;
  p.eps = eps;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int per_vec = x_dtype == CHITU_DTYPE_FP32 ? 4 : 8;
  if (C % (32 * per_vec) == 0 && C / per_vec / 32 <= chitu::kLnWarpMaxVec &&
      !(reinterpret_cast<uintptr_t>(out) & 15)) {
    // rows of at most 8 KiB: one warp per row, eight rows per CTA
    const int grid = static_cast<int>(std::min<int64_t>((rows + 7) / 8, 148 * 8));
    if (x_dtype == CHITU_DTYPE_BF16)
      chitu::layernorm_affine_warp_kernel<0><<<grid, 256, 0, st>>>(p);
    else if (x_dtype == CHITU_DTYPE_FP16)
      chitu::layernorm_affine_warp_kernel<1><<<grid, 256, 0, st>>>(p);
    else
      chitu::layernorm_affine_warp_kernel<2><<<grid, 256, 0, st>>>(p);
  } else {
    const int grid = static_cast<int>(std::min<int64_t>(rows, 148 * 8));
    chitu::layernorm_affine_kernel<<<grid, chitu::kLnThreads, 0, st>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "layernorm_modulate: launch");
  return CHITU_OK;
}

int chitu_b200_gate_residual(void* x, int x_dtype, const void* y, int y_dtype, int64_t rows, int64_t rows_per_batch, int C,
                             const float* gate, int64_t gate_batch_stride, void* stream) {
  if (!x || !y) return fail(CHITU_E_INVALID, "gate_residual: null pointer");
  if (rows <= 0 || rows_per_batch <= 0 || C <= 0 || (C & 3))
    return fail(CHITU_E_INVALID, "gate_residual: rows must be positive and C a multiple of 4");
  if (y_dtype != CHITU_DTYPE_BF16 && y_dtype != CHITU_DTYPE_FP16)
    return fail(CHITU_E_UNSUPPORTED, "gate_residual: y must be bf16 or fp16");
  if (x_dtype < 0 || x_dtype > 2) return fail(CHITU_E_UNSUPPORTED, "gate_residual: x_dtype must be bf16, fp16 or fp32");
  if ((gate_batch_stride & 3) || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gate)) & 15) ||
      (reinterpret_cast<uintptr_t>(y) & 7))
    return fail(CHITU_E_INVALID, "gate_residual: x and gate must be 16-byte aligned, y 8-byte aligned");
  chitu::GateResidualParams p;
  p.x = x;
  p.x_dtype = x_dtype;
  p.y = y;
  p.gate = gate;
  p.gate_batch_stride = gate_batch_stride;
  p.rows = rows;
  p.rows_per_batch = rows_per_batch;
  p.C = C;
  p.y_fp16 = y_dtype == CHITU_DTYPE_FP16;
  const long long total = rows * (C >> 2);
  const int grid = grid_for(total, 256 * 4, 148 * 8);
  chitu::gate_residual_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "gate_residual: launch");
  return CHITU_OK;
}

int chitu_b200_cfg_combine(const void* cond, const void* uncond, void* out, int dtype, int64_t rows, int C, float scale,
                           int rescale, void* stream) {
  if (!cond || !uncond || !out) return fail(CHITU_E_INVALID, "cfg_combine: null pointer");
  if (rows <= 0 || C <= 0) return fail(CHITU_E_INVALID, "cfg_combine: rows and C must be positive");
  if (dtype < 0 || dtype > 2) return fail(CHITU_E_UNSUPPORTED, "cfg_combine: dtype must be bf16, fp16 or fp32");
  chitu::CfgCombineParams p;
  p.cond = cond;
  p.uncond = uncond;
  p.out = out;
  p.rows = rows;
  p.C = C;
  p.dtype = dtype;
  p.rescale = rescale;
  p.scale = scale;
  const int grid = grid_for(rows, 8, 148 * 8);
  chitu::cfg_combine_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "cfg_combine: launch");
  return CHITU_OK;
}

int chitu_b200_scatter_rows(const void* src, void* const* dst_ptrs, int n_dest, int64_t B, int64_t rows,
                            int64_t row_bytes, int64_t dst_batch_stride_bytes, int64_t dst_row_stride_bytes,
                            void* stream) {
  if (!src || !dst_ptrs) return fail(CHITU_E_INVALID, "scatter_rows: null pointer");
  if (n_dest < 1 || n_dest > 8) return fail(CHITU_E_INVALID, "scatter_rows: n_dest must be 1..8");
  if (B <= 0 || rows <= 0 || row_bytes <= 0 || (row_bytes & 15) || (dst_batch_stride_bytes & 15) ||
      (dst_row_stride_bytes & 15))
    return fail(CHITU_E_INVALID, "scatter_rows: extents must be positive, byte counts multiples of 16");
  chitu::ScatterRowsParams p;
  for (int i = 0; i < 8; ++i) p.dst[i] = nullptr;
  for (int i = 0; i < n_dest; ++i) {
    if (!dst_ptrs[i] || (reinterpret_cast<uintptr_t>(dst_ptrs[i]) & 15))
      return fail(CHITU_E_INVALID, "scatter_rows: destinations must be non-null and 16-byte aligned");
    p.dst[i] = static_cast<uint8_t*>(dst_ptrs[i]);
  }
  if (reinterpret_cast<uintptr_t>(src) & 15) return fail(CHITU_E_INVALID, "scatter_rows: src must be 16-byte aligned");
  p.n_dest = n_dest;
  p.B = B;
  p.rows = rows;
  p.row_vecs = row_bytes / 16;
  p.dst_batch_bytes = dst_batch_stride_bytes;
  p.dst_row_bytes = dst_row_stride_bytes;
  const long long total = B * n_dest * rows * p.row_vecs;
  const int grid = grid_for(total, 256 * 4, 148 * 8);
  chitu::scatter_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(src), p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "scatter_rows: launch");
  return CHITU_OK;
}

int chitu_b200_peer_copy_2d(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes,
                            int64_t width_bytes, int64_t rows, void* stream) {
  if (!dst || !src) return fail(CHITU_E_INVALID, "peer_copy_2d: null pointer");
  if (width_bytes <= 0 || rows <= 0 || dst_pitch_bytes < width_bytes || src_pitch_bytes < width_bytes)
    return fail(CHITU_E_INVALID, "peer_copy_2d: width and rows must be positive, pitches at least the width");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (rows == 1 || (dst_pitch_bytes == width_bytes && src_pitch_bytes == width_bytes))
    e = cudaMemcpyAsync(dst, src, static_cast<size_t>(width_bytes * rows), cudaMemcpyDeviceToDevice, st);
  else
    e = cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_pitch_bytes), src, static_cast<size_t>(src_pitch_bytes),
                          static_cast<size_t>(width_bytes), static_cast<size_t>(rows), cudaMemcpyDeviceToDevice, st);
  if (e != cudaSuccess) return cuda_fail(e, "peer_copy_2d");
  return CHITU_OK;
}

}  // extern "C"

// ----------------------------------------------------------------------------
// Key-split attention for callers that may not allocate.
//
// Some hosts of this library cannot hand over a scratch buffer: an inference server that gave
// every free byte of device memory to its own pool at start-up has nothing left to allocate from,
// and a plugin called from inside somebody else's step function has no business calling
// cudaMalloc there (it may fail, and it stalls every stream of the device while it runs).  For
// them the scratch of the key-split path lives in a fixed array inside the library image.
//
// The array below is a DEVICE symbol.  In host code its name is only a handle: the usable device
// address comes from cudaGetSymbolAddress, looked up once per device with that device current.
// ----------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = 32u << 20;  // 32 MiB, resident on every GPU that loads the library
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

void* g_static_scratch_ptr[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;

// Device address of the scratch array on the CURRENT device (looked up on first use).
int static_scratch_for_current_device(void** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "attn_fwd_splitkv_static: cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return fail(CHITU_E_UNSUPPORTED, "attn_fwd_splitkv_static: device index %d", dev);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "attn_fwd_splitkv_static: cudaGetSymbolAddress");
    g_static_scratch_ptr[dev] = p;
  }
  *ptr = g_static_scratch_ptr[dev];
  return CHITU_OK;
}

}  // namespace

extern "C" int chitu_b200_attn_fwd_splitkv_static(const void* q, const void* k, const void* v, void* out, float* lse,
                                                  int B, int Sq, int Sk, int H, int D, const int64_t* q_strides,
                                                  const int64_t* k_strides, const int64_t* v_strides,
                                                  float softmax_scale, int dtype, int n_splits, int* status,
                                                  void* stream) {
  if (n_splits < 1 || n_splits > 64) return fail(CHITU_E_INVALID, "attn_fwd_splitkv_static: n_splits must be in 1..64");
  if (B <= 0 || Sq <= 0 || Sk <= 0 || H <= 0 || D <= 0)
    return fail(CHITU_E_INVALID, "attn_fwd_splitkv_static: B, Sq, Sk, H, D must be positive");
  // the same clamping the general path applies, so the size check below is the real requirement
  const int n = plan_key_splits(Sk, n_splits).n_splits;
  const int64_t need = splitkv_workspace_bytes(B, Sq, H, D, n);
  if (need > static_cast<int64_t>(kStaticScratchBytes))
    return fail(CHITU_E_INVALID,
                "attn_fwd_splitkv_static: %d key ranges of [%d x %d x %d x %d] need %lld bytes of scratch, the built-in "
                "array holds %lld; use fewer ranges or chitu_b200_attn_fwd_splitkv with your own workspace",
                n, B, Sq, H, D, (long long)need, (long long)kStaticScratchBytes);
  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc != CHITU_OK) return rc;
  KeySplit ks;
  ks.n_splits = n_splits;
  ks.workspace = scratch;
  ks.workspace_bytes = static_cast<int64_t>(kStaticScratchBytes);
  return attn_fwd_impl(q, k, v, out, OutScatter{}, lse, B, Sq, Sk, H, D, q_strides, k_strides, v_strides,
                       softmax_scale, dtype, status, stream, ks);
}

// ----------------------------------------------------------------------------
// 8-bit attention: quantisation pre-pass + INT8 / FP8 tensor-core kernel
// ----------------------------------------------------------------------------
namespace {

struct Q8Layout {
  int64_t q8, k8, v8, q_scale, k_scale, k_sum, v_amax, q_corr, total;
};

int64_t align256(int64_t n) { return (n + 255) / 256 * 256; }

Q8Layout q8_layout(int B, int Sq, int Sk, int H) {
  Q8Layout L;
  int64_t off = 0;
  auto take = [&](int64_t bytes) {
    const int64_t at = off;
    off += align256(bytes);
    return at;
  };
  L.q8 = take(static_cast<int64_t>(B) * Sq * H * 128);
  L.k8 = take(static_cast<int64_t>(B) * Sk * H * 128);
  L.v8 = take(static_cast<int64_t>(B) * Sk * H * 128);
  L.q_scale = take(static_cast<int64_t>(B) * H * ((Sq + 127) / 128) * 4);
  L.k_scale = take(static_cast<int64_t>(B) * H * ((Sk + 63) / 64) * 4);
  L.k_sum = take(static_cast<int64_t>(B) * H * 128 * 4);
  L.v_amax = take(static_cast<int64_t>(B) * H * 128 * 4);  // directly after k_sum: one memset clears both
  L.q_corr = take(static_cast<int64_t>(B) * H * Sq * 4);
  L.total = off;
  return L;
}

// Tensor map over a contiguous [B, S, H, 128] byte tensor: one 128-row x 128-byte panel per copy.
int make_u8_map(CUtensorMap* map, const void* base, int B, int S, int H, const char* name) {
  auto encode = get_encode_fn();
  if (!encode) return fail(CHITU_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(B)};
  cuuint64_t strides[3] = {128, static_cast<cuuint64_t>(H) * 128, static_cast<cuuint64_t>(S) * H * 128};
  cuuint32_t box[4] = {128, 1, 128, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CHITU_E_CUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", name, (int)r);
  return CHITU_OK;
}

}  // namespace

extern "C" int64_t chitu_b200_attn_q8_workspace_bytes(int B, int Sq, int Sk, int H) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || H <= 0) return 0;
  return q8_layout(B, Sq, Sk, H).total;
}

extern "C" int chitu_b200_attn_fwd_q8(const void* q, const void* k, const void* v, void* out, float* lse, int B, int Sq,
                                      int Sk, int H, int D, const int64_t* q_strides, const int64_t* k_strides,
                                      const int64_t* v_strides, float softmax_scale, int dtype, void* workspace,
                                      int64_t workspace_bytes, int* status, void* stream) {
  if (!q || !k || !v || !out || !q_strides || !k_strides || !v_strides || !workspace)
    return fail(CHITU_E_INVALID, "attn_fwd_q8: null pointer argument");
  if (B <= 0 || H <= 0 || Sq <= 0 || Sk <= 0) return fail(CHITU_E_INVALID, "attn_fwd_q8: B, H, Sq, Sk must be positive");
  if (D != 128) return fail(CHITU_E_UNSUPPORTED, "attn_fwd_q8: head_dim %d not supported (only 128)", D);
  if (dtype != CHITU_DTYPE_BF16 && dtype != CHITU_DTYPE_FP16)
    return fail(CHITU_E_UNSUPPORTED, "attn_fwd_q8: dtype must be bf16 or fp16");
  if (!(softmax_scale > 0.f)) return fail(CHITU_E_UNSUPPORTED, "attn_fwd_q8: softmax_scale must be positive");
  if (H > 65535 || B > 65535) return fail(CHITU_E_UNSUPPORTED, "attn_fwd_q8: H and B must be below 65536");
  if ((Sq + 127) / 128 + (Sk + 63) / 64 + (Sk + 127) / 128 > 65535)
    return fail(CHITU_E_UNSUPPORTED, "attn_fwd_q8: sequences too long for the quantisation grid");
  for (const int64_t* st : {q_strides, k_strides, v_strides})
    if (st[3] != 1 || (st[0] & 3) || (st[1] & 3) || (st[2] & 3))
      return fail(CHITU_E_INVALID, "attn_fwd_q8: head_dim stride must be 1, the others multiples of 4 elements");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(CHITU_E_INVALID, "attn_fwd_q8: q, k, v, out must be 16-byte aligned");
  const Q8Layout L = q8_layout(B, Sq, Sk, H);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) || workspace_bytes < L.total)
    return fail(CHITU_E_INVALID, "attn_fwd_q8: workspace must be 256-byte aligned and hold %lld bytes", (long long)L.total);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* q8 = ws + L.q8;
  uint8_t* k8 = ws + L.k8;
  uint8_t* v8 = ws + L.v8;
  float* q_scale = reinterpret_cast<float*>(ws + L.q_scale);
  float* k_scale = reinterpret_cast<float*>(ws + L.k_scale);
  float* k_sum = reinterpret_cast<float*>(ws + L.k_sum);
  unsigned* v_amax = reinterpret_cast<unsigned*>(ws + L.v_amax);
  float* q_corr = reinterpret_cast<float*>(ws + L.q_corr);
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  cudaError_t e = cudaMemsetAsync(k_sum, 0, static_cast<size_t>(L.q_corr - L.k_sum), st);  // k_sum and v_amax
  if (e != cudaSuccess) return cuda_fail(e, "attn_fwd_q8: memset");
  chitu::q8_colstat_kernel<<<dim3(H, (Sk + 127) / 128, B), chitu::kQ8QuantThreads, 0, st>>>(
      k, v, dtype, k_strides[0], k_strides[1], k_strides[2], v_strides[0], v_strides[1], v_strides[2], Sk, H, k_sum,
      v_amax);
  chitu::Q8QuantParams qp;
  const void* xs[3] = {q, k, v};
  const int64_t* strides[3] = {q_strides, k_strides, v_strides};
  uint8_t* outs[3] = {q8, k8, v8};
  const int tokens[3] = {Sq, Sk, Sk};
  const int blocks[3] = {(Sq + 127) / 128, (Sk + 63) / 64, (Sk + 127) / 128};
  qp.first_block[0] = 0;
  for (int i = 0; i < 3; ++i) {
    qp.x[i] = xs[i];
    qp.xs_b[i] = strides[i][0];
    qp.xs_s[i] = strides[i][1];
    qp.xs_h[i] = strides[i][2];
    qp.out[i] = outs[i];
    qp.S[i] = tokens[i];
    qp.first_block[i + 1] = qp.first_block[i] + blocks[i];
  }
  qp.dtype = dtype;
  qp.H = H;
  qp.pre_scale = softmax_scale * 1.4426950408889634f;
  qp.k_sum = k_sum;
  qp.v_amax = v_amax;
  qp.q_scale = q_scale;
  qp.k_scale = k_scale;
  qp.q_corr = q_corr;
  chitu::q8_quant_kernel<<<dim3(H, qp.first_block[3], B), chitu::kQ8QuantThreads, 0, st>>>(qp);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "attn_fwd_q8: quantisation launch");

  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_u8_map(&tq, q8, B, Sq, H, "q8")) != CHITU_OK) return rc;
  if ((rc = make_u8_map(&tk, k8, B, Sk, H, "k8")) != CHITU_OK) return rc;
  if ((rc = make_u8_map(&tv, v8, B, Sk, H, "v8")) != CHITU_OK) return rc;
  chitu::AttnQ8Params p;
  p.out = out;
  p.lse = lse;
  p.status = status;
  p.B = B;
  p.H = H;
  p.Sq = Sq;
  p.Sk = Sk;
  p.is_fp16 = dtype == CHITU_DTYPE_FP16;
  p.q_scale = q_scale;
  p.k_scale = k_scale;
  p.v_amax = v_amax;
  p.q_corr = q_corr;
#ifdef CHITU_ATTN_TIMING
  p.dbg = g_dbg;
#endif
  static bool attr_done[2][kMaxDevices] = {};
  static std::mutex attr_mu;
  const cudaError_t attr_err =
      p.is_fp16 ? ensure_dynamic_smem(chitu::attn_q8_kernel<true>, chitu::kQ8SmemBytes, attr_done[1], attr_mu)
                : ensure_dynamic_smem(chitu::attn_q8_kernel<false>, chitu::kQ8SmemBytes, attr_done[0], attr_mu);
  if (attr_err != cudaSuccess) return cuda_fail(attr_err, "attn_fwd_q8: cudaFuncSetAttribute");
  dim3 grid((Sq + 255) / 256, H, B);
  if (p.is_fp16)
    chitu::attn_q8_kernel<true><<<grid, chitu::kQ8Threads, chitu::kQ8SmemBytes, st>>>(tq, tk, tv, p);
  else
    chitu::attn_q8_kernel<false><<<grid, chitu::kQ8Threads, chitu::kQ8SmemBytes, st>>>(tq, tk, tv, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "attn_fwd_q8: launch");
  return CHITU_OK;
}


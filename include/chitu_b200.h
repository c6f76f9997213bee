/*
 * chitu_b200.h - C ABI of the B200-native attention hot path.
 *
 * A shared library (libchitu_b200.so) with plain-C entry points: raw device
 * pointers, integer shapes and element strides, a CUDA stream handle passed as
 * void*.  No entry point allocates device memory, synchronises the device or
 * throws; each returns 0 on success or a negative CHITU_E_* code, and
 * chitu_b200_last_error() gives the message for the calling thread.  Kernels
 * that can wait on another agent take an optional device status word
 * (int32, zero-initialised by the caller) which they set to a positive code if
 * a bounded wait ran out; the launch itself still returns 0.
 *
 * Tensors follow the reference's layouts: q/k/v/out are [B, S, H, D]
 * (D = 128 contiguous), the block log-sum-exp is [B, H, S] fp32 (natural log,
 * softmax scale included).
 *
 * Each declaration names the reference interface it stands in for
 * (file:line inside the ChituDiffusion tree).
 */
#ifndef CHITU_B200_H_
#define CHITU_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CHITU_OK 0
#define CHITU_E_INVALID (-1)     /* bad argument (shape, stride, alignment, null) */
#define CHITU_E_UNSUPPORTED (-2) /* valid request this library does not implement */
#define CHITU_E_CUDA (-3)        /* a CUDA runtime / driver call failed */

#define CHITU_DTYPE_BF16 0
#define CHITU_DTYPE_FP16 1
#define CHITU_DTYPE_FP32 2

/* Library version (major*10000 + minor*100 + patch) and capability bits. */
int chitu_b200_version(void);
#define CHITU_CAP_ATTN_BF16 1u
#define CHITU_CAP_ATTN_FP16 2u
#define CHITU_CAP_NORM_ROPE 4u
#define CHITU_CAP_LSE_COMBINE 8u
#define CHITU_CAP_A2A_LAYOUT 16u
#define CHITU_CAP_PEER_EXCHANGE 32u
#define CHITU_CAP_ATTN_Q8 64u
unsigned chitu_b200_caps(void);
const char* chitu_b200_last_error(void);

/*
 * Dense non-causal attention forward, softmax(scale * q k^T) v.
 * Replaces the per-rank kernel call behind DiffusionAttnBackend.__call__
 * (chitu_diffusion/modules/attention/diffusion_attn_backend.py:131-207, the
 * torch-SDPA form at :270-315 and the flash form at :404-447).
 *
 *   q            [B, Sq, H, 128], element strides q_strides[4] = {b, s, h, d}; d stride must be 1,
 *                the others multiples of 8 elements; base 16-byte aligned.  Same for k, v ([B, Sk, H, 128]).
 *   out          [B, Sq, H, 128] contiguous, same dtype as q.
 *   lse          [B, H, Sq] fp32 or NULL.
 *   dtype        CHITU_DTYPE_BF16 or CHITU_DTYPE_FP16.
 *   status       optional device int32, see above.
 */
int chitu_b200_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int Sq, int Sk,
                        int H, int D, const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                        float softmax_scale, int dtype, int* status, void* stream);

/*
 * The same attention with the keys split into n_splits ranges that run as separate CTAs (for grids
 * that would leave most of the 148 SMs idle: few query rows or few heads per GPU).  Each CTA parks its
 * partial rows in the workspace; the last of the n_splits CTAs of a query block to finish merges them
 * and writes the result - one launch.  Same reference call sites as chitu_b200_attn_fwd.  The split count
 * is clamped to the number of 128-key tiles; with one split no workspace is touched.
 *
 *   workspace        device scratch of at least chitu_b200_attn_splitkv_workspace_bytes(...) bytes,
 *                    16-byte aligned.  Its first CHITU_SPLITKV_HEADER_BYTES hold one counter per
 *                    (batch, head, 256-row query block) - at most CHITU_SPLITKV_HEADER_BYTES / 4 of them,
 *                    more is CHITU_E_UNSUPPORTED - and must be ZERO before the first call; every call
 *                    that completes leaves them zero again (a call that ended with a non-zero status
 *                    word may not: clear the header before reusing the workspace).  The rest - fp32
 *                    partial rows and their log-sum-exps, in whole 128-row tiles - needs no initialisation.
 */
#define CHITU_SPLITKV_HEADER_BYTES 65536
int64_t chitu_b200_attn_splitkv_workspace_bytes(int B, int Sq, int H, int D, int n_splits);
int chitu_b200_attn_fwd_splitkv(const void* q, const void* k, const void* v, void* out, float* lse, int B, int Sq,
                                int Sk, int H, int D, const int64_t* q_strides, const int64_t* k_strides,
                                const int64_t* v_strides, float softmax_scale, int dtype, int n_splits,
                                void* workspace, int64_t workspace_bytes, int* status, void* stream);

/*
 * chitu_b200_attn_fwd_splitkv for callers that cannot allocate device memory.  (No counterpart in the
 * reference: ChituDiffusion always runs inside torch's allocator.)
 *
 * Meant for hosts that have no scratch buffer to give: a server that committed all free device
 * memory to its own pool at start-up, or a plugin invoked in the middle of another runtime's step,
 * where calling cudaMalloc is off the table (it can fail, and it stalls the whole device while it
 * runs).  The partial results live in a 32 MiB array built into the library image, present on every
 * GPU that loads the library for as long as the process lives.  This call, and everything it
 * reaches, calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 *   - Limit: the key-split scratch, chitu_b200_attn_splitkv_workspace_bytes(B, Sq, H, D, n) bytes for the
 *     effective split count n, must fit in 32 MiB; larger requests return CHITU_E_INVALID with the sizes
 *     in chitu_b200_last_error().  Arguments and results are those of chitu_b200_attn_fwd_splitkv.
 *   - First call on a device: looks up the array's device address (cudaGetSymbolAddress, with the
 *     caller's current device current) and caches it.  Make that first call before starting any
 *     stream capture on that device.  With CUDA's default lazy module loading this first call is also
 *     the moment the library's device image - the 32 MiB array included - becomes resident on that
 *     GPU, so a host that hands all free memory to its own pool must make the first call (or load the
 *     process with CUDA_MODULE_LOADING=EAGER and touch the library once) BEFORE it commits that pool;
 *     afterwards nothing more is taken.  cudaDeviceReset() destroys the array and invalidates the
 *     cached address: a process that resets a device must not call this entry point on it again.
 *   - One array per GPU, shared by every call: it keeps the previous call's partial results and nothing
 *     in it needs clearing, because each call overwrites every row it later reads and returns the counters
 *     at its head (zero when the library is loaded) to zero.  Two calls that run
 *     at the same time on one GPU (different streams, or different threads) race on it; serialise them.
 */
int chitu_b200_attn_fwd_splitkv_static(const void* q, const void* k, const void* v, void* out, float* lse, int B,
                                       int Sq, int Sk, int H, int D, const int64_t* q_strides,
                                       const int64_t* k_strides, const int64_t* v_strides, float softmax_scale,
                                       int dtype, int n_splits, int* status, void* stream);

/*
 * Attention whose QUERY pre-attention transform runs inside the kernel: q_raw is the projection output
 * ([B, Sq, H, 128], strides as for chitu_b200_attn_fwd); once a query tile has landed in shared memory the
 * kernel applies RMSNorm, weight, rotary embedding and the 16-bit rounding to it in place - the arithmetic
 * and summation order of chitu_b200_qk_norm_rope, so the result equals transforming q with that call first
 * - and only then starts the tensor-core work.  The q half of the pre-pass (one read and one write of q)
 * disappears; k still goes through chitu_b200_qk_norm_rope, because every query block of a head re-reads
 * every key tile and would repeat its transform.  Replaces the q chain of WanSelfAttention.forward
 * (chitu_diffusion/models/model_wan.py:152-153,194-195,198) and of the Flux / Qwen processors
 * (chitu_diffusion/modules/attention/flux_attention.py:139-151) together with the attention call.
 *
 *   norm_mode   1 = per-head RMSNorm over the 128 channels (weight: [128] or NULL);
 *               0 = full-width RMSNorm whose per-token factor the caller supplies: rstd[b * Sq + s] fp32
 *                   (one head cannot form a statistic over all heads; weight: [H * 128] or NULL);
 *               2 = none
 *   rope_mode, rope_table, table_rows, gf, gh, gw, n_t, n_h, pos_offset, round_mid, eps, w_dtype:
 *               as in chitu_b200_qk_norm_rope (n_t, n_h = its axis_split)
 *   n_splits, workspace: as in chitu_b200_attn_fwd_splitkv (1 and NULL for no key split)
 */
typedef struct {
  int norm_mode, rope_mode, round_mid, w_dtype;
  const void* weight;
  const float* rstd;
  float eps;
  const float* rope_table;
  int table_rows, gf, gh, gw, n_t, n_h;
  int64_t pos_offset;
} chitu_b200_q_pre;
int chitu_b200_attn_fwd_qpre(const void* q_raw, const void* k, const void* v, void* out, float* lse, int B, int Sq, int Sk,
                             int H, int D, const int64_t* q_strides, const int64_t* k_strides,
                             const int64_t* v_strides, float softmax_scale, int dtype, const chitu_b200_q_pre* q_pre,
                             int n_splits, void* workspace, int64_t workspace_bytes, int* status, void* stream);

/*
 * Quantised attention: per-block INT8 Q K^T, E4M3 P V, fp32 accumulation, 16-bit output.
 * Stands in for the SageAttention backend call sageattn(q, k, v, tensor_layout="NHD", ...)
 * (chitu_diffusion/modules/attention/diffusion_attn_backend.py:242-268).  The call runs the
 * quantisation pre-pass (K centred over the tokens; Q scaled by softmax_scale*log2 e and quantised per
 * 128-token block, K per 64-token block, V to E4M3 per channel) and then the 8-bit kernel.
 * Arguments as chitu_b200_attn_fwd; `workspace` (256-byte aligned, at least
 * chitu_b200_attn_q8_workspace_bytes(B, Sq, Sk, H) bytes) receives the 8-bit copies and scales and
 * needs no initialisation.  Unlike the reference call, softmax_scale is honoured.
 */
int64_t chitu_b200_attn_q8_workspace_bytes(int B, int Sq, int Sk, int H);
int chitu_b200_attn_fwd_q8(const void* q, const void* k, const void* v, void* out, float* lse, int B, int Sq, int Sk,
                           int H, int D, const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                           float softmax_scale, int dtype, void* workspace, int64_t workspace_bytes, int* status,
                           void* stream);

/*
 * Fold one partial attention result into the running (out, lse) pair:
 *   out <- out - sigmoid(lse_b - lse) * (out - out_b),  lse <- lse - logsigmoid(lse - lse_b)
 * or, when `first` is non-zero, initialise them from the block.
 * Replaces update_out_and_lse (chitu_diffusion/runtime/parallel_utils.py:59-97).
 *
 *   acc_out      [B, S, H, D] fp32 contiguous (read-modify-write)
 *   acc_lse      [B, S, H] fp32 contiguous (the reference's [B, S, H, 1])
 *   block_out    [B, S, H, D] contiguous, block_dtype in {BF16, FP16, FP32}
 *   block_lse    [B, H, S] fp32 contiguous
 *   final_out    optional [B, S, H, D] contiguous of final_dtype: also written with the merged result
 */
int chitu_b200_lse_combine(float* acc_out, float* acc_lse, const void* block_out, const float* block_lse, int B, int S,
                           int H, int D, int block_dtype, int first, void* final_out, int final_dtype, void* stream);

/*
 * Pre-attention transform for one of q / k: RMSNorm, rotary embedding on
 * interleaved pairs, cast to 16 bit, written with arbitrary output placement
 * (so the result can land directly in an all-to-all send buffer).
 * Replaces WanRMSNorm.forward + rope_apply / rope_apply_with_cp + half()
 * (chitu_diffusion/models/model_wan.py:49-65,83-110,80-81;
 *  chitu_diffusion/modules/utils/wan/__init__.py:31-67) and, with
 * norm_mode = 1, the per-head RMSNorm + rotary embedding of the Flux / Qwen
 * processors (chitu_diffusion/modules/attention/flux_attention.py:96-171).
 *
 *   x            [B, S, H*D] rows, element row stride x_row_stride (batch stride = S * x_row_stride)
 *   in_dtype     BF16 / FP16 / FP32
 *   weight       [H*D] (norm_mode 0) or [D] (norm_mode 1) or NULL (unit weight); w_dtype BF16 / FP32
 *   norm_mode    0 = statistics over all H*D channels of a token, 1 = per head over D, 2 = no norm
 *   rope_mode    0 = none,
 *                1 = three-axis grid: token n (global index pos_offset + local index) sits at
 *                    (frame, row, column) = (n / (gh*gw), (n / gw) % gh, n % gw); pair j takes its angle from
 *                    the frame position for j < n_t, from the row position for n_t <= j < n_t + n_h, from the
 *                    column position otherwise (n_t, n_h: axis_split); rope_table is [max_pos, D/2] float2
 *                    (cos, sin), row = position along the pair's axis; tokens with n >= gf*gh*gw pass through
 *                    unrotated; token count and positions must stay below 2^31,
 *                2 = per-token table: rope_table is [S_table, D/2] float2 indexed by pos_offset + local index.
 *   axis_split   {n_t, n_h} pairs for rope_mode 1 (n_w = D/2 - n_t - n_h)
 *   out          16-bit; element (b, s, h, d) is written at
 *                out + b*out_strides[0] + s*out_strides[1] + (h / heads_per_group)*out_strides[2]
 *                    + (h % heads_per_group)*out_strides[3] + d
 *   round_mid    non-zero: round the normalised value to in_dtype before the weight multiply and round the
 *                product to w_dtype when that is 16-bit (the reference's type_as / promotion order)
 */
int chitu_b200_qk_norm_rope(const void* x, int in_dtype, int64_t x_row_stride, const void* weight, int w_dtype,
                            float eps, int norm_mode, int rope_mode, const float* rope_table, int table_rows,
                            int gf, int gh, int gw, const int* axis_split, int64_t pos_offset, void* out,
                            int out_dtype, const int64_t* out_strides, int heads_per_group, int B, int S, int H, int D,
                            int round_mid, void* stream);

/*
 * q, k (and v) of one layer in ONE launch: up to three jobs that share shape, dtypes, rotary table
 * and output placement, each with its own input, weight and modes (v is usually norm_mode 2,
 * rope_mode 0: a plain cast / scatter).  Same reference lines as chitu_b200_qk_norm_rope - it replaces
 * the q and k chains of WanSelfAttention.forward (chitu_diffusion/models/model_wan.py:152-156,194-200)
 * at once.  A job writes to `out`, or, when n_out_ptrs > 0, head group g goes to out_ptrs[g] as in
 * chitu_b200_qk_norm_rope_scatter.
 */
typedef struct {
  const void* x;
  int64_t x_row_stride;
  const void* weight; /* NULL = unit weight */
  int norm_mode, rope_mode;
  void* out;
  void* const* out_ptrs;
  int n_out_ptrs;
  float* rstd_out; /* NULL, or (norm_mode 0): write only rstd_out[b * S + s] = rsqrt(mean_C(x^2) + eps), the factor
                      chitu_b200_attn_fwd_qpre takes for q; nothing else is stored by this job */
} chitu_b200_norm_rope_job;
int chitu_b200_qk_norm_rope_batch(const chitu_b200_norm_rope_job* jobs, int n_jobs, int in_dtype, int w_dtype,
                                  float eps, const float* rope_table, int table_rows, int gf, int gh, int gw,
                                  const int* axis_split, int64_t pos_offset, int out_dtype,
                                  const int64_t* out_strides, int heads_per_group, int B, int S, int H, int D,
                                  int round_mid, void* stream);

/*
 * Layout shuffles either side of the Ulysses all-to-all (packed single-buffer form).
 * Replace the permute + contiguous() pairs in CommGroup._all_to_all_single
 * (chitu_diffusion/core/distributed/comm_group.py:350-384).
 *
 *   pack_heads:    x [B, s, U*hc, D] (strided)      -> send [U, B, s, hc, D]
 *   unpack_seq:    recv [U, B, s, hc, D]            -> y [B, U*s, hc, D]
 *   pack_seq:      x [B, U*sc, h, D] (strided)      -> send [U, B, sc, h, D]
 *   unpack_heads:  recv [U, B, sc, h, D]            -> y [B, sc, U*h, D]
 * All are one generic 5-d strided copy of 16-byte vectors: dst is contiguous
 * [n0, n1, n2, n3, row_bytes]; src strides are given in bytes per index.
 */
int chitu_b200_strided_copy(const void* src, void* dst, int64_t n0, int64_t n1, int64_t n2, int64_t n3,
                            int64_t row_bytes, const int64_t* src_strides_bytes, void* stream);

/*
 * Elementwise tails of the DiT block around the attention path (WanAttentionBlock.forward,
 * chitu_diffusion/models/model_wan.py:321-366).
 *
 * chitu_b200_layernorm_modulate: out[r, :] = LayerNorm(x[r, :]) * m + a in one pass over the residual
 *   stream x [rows, C] (x_dtype: fp32 as in the Wan block, or 16-bit as in the Flux blocks,
 *   chitu_diffusion/models/model_flux1.py:90-236), statistics in fp32, 16-bit out; m = mul[b] (or 1 + mul[b] when add_one) and a = add[b] with
 *   b = r / rows_per_batch; a batch stride of 0 shares one vector among batches; null mul / add mean 1 / 0.
 *   With add_one it is `norm1(x).float() * (1 + e[1]) + e[0]` (:344-345, :353) including the cast the
 *   following Linear applies; without, the affine WanLayerNorm norm3 (:68-78, :303-305, :352).
 * chitu_b200_gate_residual: x[r, :] += y[r, :] * gate[b] in place (x of x_dtype, y 16-bit; null gate = 1):
 *   `x = x + y * e[2]` (:347-348, :354-355) and the ungated cross-attention residual (:352).
 */
int chitu_b200_layernorm_modulate(const void* x, int x_dtype, void* out, int out_dtype, int64_t rows, int64_t rows_per_batch, int C,
                                  const float* mul, int64_t mul_batch_stride, const float* add,
                                  int64_t add_batch_stride, int add_one, float eps, void* stream);
int chitu_b200_gate_residual(void* x, int x_dtype, const void* y, int y_dtype, int64_t rows, int64_t rows_per_batch, int C,
                             const float* gate, int64_t gate_batch_stride, void* stream);

/*
 * Classifier-free-guidance combine of the two branch predictions after the CFG-parallel all-gather
 * (CfgDispatcher.all_gather_cfg_noise_preds, chitu_diffusion/runtime/generator.py:134-149):
 *   out = uncond + scale * (cond - uncond)                        (runtime/adapter/wan.py:224-228)
 * and, with rescale != 0, the norm-preserving form of the Qwen-Image adapter
 *   out *= ||cond|| / ||out|| over the last dim                   (runtime/adapter/qwen_image.py:678-681).
 * cond, uncond, out are contiguous [rows, C] of one dtype (out may alias either input).
 */
int chitu_b200_cfg_combine(const void* cond, const void* uncond, void* out, int dtype, int64_t rows, int C, float scale,
                           int rescale, void* stream);

/*
 * Ring and all-gather-KV exchange over peer-mapped memory: every rank publishes its K/V block in a
 * buffer mapped into its peers, and a reader pulls the block it needs for the next ring step into
 * local memory with the copy engines while the attention kernel works on the current block.  Replaces
 * the send/recv rotation of DiffusionAttention_with_CP._cp_forward
 * (chitu_diffusion/modules/attention/diffusion_attn_backend.py:783-835, built on
 * CommGroup.p2p_isend/p2p_irecv/p2p_commit/p2p_wait, chitu_diffusion/core/distributed/comm_group.py:305-327)
 * and the all_gather + cat of the AGCP branch (diffusion_attn_backend.py:581-597,739-742).
 *
 * chitu_b200_peer_copy_2d: `rows` pieces of width_bytes from src (pitch src_pitch_bytes) to dst (pitch
 *   dst_pitch_bytes); either side may be peer-mapped.  A device-to-device cudaMemcpy(2D)Async on
 *   `stream`: no SM is used.
 * chitu_b200_scatter_rows: src is contiguous [B, n_dest*rows, row_bytes]; row (b, i*rows + j) is stored
 *   to dst_ptrs[i] + b*dst_batch_stride_bytes + j*dst_row_stride_bytes.  Used to hand the merged fp32
 *   result of a Ulysses x ring call back to the sequence owners (the all-to-all at :825-828).
 */
int chitu_b200_peer_copy_2d(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes,
                            int64_t width_bytes, int64_t rows, void* stream);
int chitu_b200_scatter_rows(const void* src, void* const* dst_ptrs, int n_dest, int64_t B, int64_t rows,
                            int64_t row_bytes, int64_t dst_batch_stride_bytes, int64_t dst_row_stride_bytes,
                            void* stream);

/*
 * Ulysses exchange fused into the kernels either side of it, over peer-mapped memory of the GPUs
 * of one node (NVLink).  Together they replace the three all-to-all calls before and the one after
 * the attention kernel in DiffusionAttention_with_CP._cp_forward
 * (chitu_diffusion/modules/attention/diffusion_attn_backend.py:778-781,825-828) and the pack /
 * unpack copies of CommGroup._all_to_all_single (chitu_diffusion/core/distributed/comm_group.py:350-384).
 *
 * chitu_b200_qk_norm_rope_scatter: as chitu_b200_qk_norm_rope, but head group g = h / heads_per_group
 *   is written to out_ptrs[g] (rank g's buffer, mapped into this process) at
 *   b*out_strides[0] + s*out_strides[1] + (h % heads_per_group)*out_strides[3] + d; out_strides[2] is ignored.
 *   With norm_mode 2 and rope_mode 0 it is the plain scatter used for v.
 * chitu_b200_attn_fwd_scatter: as chitu_b200_attn_fwd, but query row r is written to
 *   out_ptrs[r / rows_per_dest] at element offset
 *   batch*dest_batch_stride + (r % rows_per_dest)*dest_row_stride + dest_head_offset + head*128 + d;
 *   n_splits / workspace as in chitu_b200_attn_fwd_splitkv (the CTA that merges the ranges does the scattered store).
 * chitu_b200_peer_barrier: every rank enqueues it the same number of times; flag_ptrs[i] is rank i's
 *   array of `world + 1` int32 (zero-initialised: one flag per peer, then the local epoch counter)
 *   mapped into this process.  The epoch is kept on the device, so the call can be replayed from a
 *   CUDA graph.  The wait is bounded (about a second); on timeout *status is set to 5 and the kernel
 *   returns.
 */
int chitu_b200_qk_norm_rope_scatter(const void* x, int in_dtype, int64_t x_row_stride, const void* weight,
                                    int w_dtype, float eps, int norm_mode, int rope_mode, const float* rope_table,
                                    int table_rows, int gf, int gh, int gw, const int* axis_split, int64_t pos_offset,
                                    void* const* out_ptrs, int n_out_ptrs, int out_dtype, const int64_t* out_strides,
                                    int heads_per_group, int B, int S, int H, int D, int round_mid, void* stream);
int chitu_b200_attn_fwd_scatter(const void* q, const void* k, const void* v, void* const* out_ptrs, int n_dest,
                                int rows_per_dest, int64_t dest_batch_stride, int64_t dest_row_stride,
                                int64_t dest_head_offset, float* lse, int B, int Sq, int Sk, int H, int D,
                                const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                float softmax_scale, int dtype, int n_splits, void* workspace,
                                int64_t workspace_bytes, int* status, void* stream);
int chitu_b200_peer_barrier(int* const* flag_ptrs, int rank, int world, int* status, void* stream);

/*
 * The same exchange without barrier launches: arrival flags.  (Same reference lines as above; what they
 * replace in addition is the stream-order wait the reference gets from NCCL between its all-to-all and the
 * attention kernel.)
 *
 * Every rank owns a "sync block" of CHITU_SYNC_INTS int32 in peer-mapped memory, zero before first use;
 * sync->blocks[i] is rank i's block as mapped into this process.  All counters in it are per-layer epochs
 * kept on the device, so the three calls below take no per-layer argument and replay from a CUDA graph;
 * every rank must issue the same sequence of them.
 *
 * chitu_b200_qk_norm_rope_batch_signal: chitu_b200_qk_norm_rope_batch whose last CTA, once all of the
 *   launch's stores are ordered, writes the new epoch into every peer's "rows of rank r have landed" flag.
 *   One signalling launch per layer (put q, k and v in it).
 * chitu_b200_attn_fwd_exchange: chitu_b200_attn_fwd_scatter over buffers filled that way.  Rows
 *   [s*rows_per_src, (s+1)*rows_per_src) of q, k and v came from rank s: the kernel's copy warp waits
 *   (bounded, status 5 on timeout) for rank s's flag before its first copy that touches them, and walks
 *   the key tiles starting with this rank's own rows.  When the last output row has been stored it writes
 *   the new epoch into every peer's "outputs of rank r have landed" flag.
 *   Replicated prefix (the text tokens of the Qwen-Image layout, cp_attn_with_full_txt,
 *   diffusion_attn_backend.py:839-984): rows [0, prefix_rows) of q, k and v are this rank's own copies - no
 *   flag is waited for, the exchanged rows start at prefix_rows - and the output rows of the prefix, which
 *   each rank computes for its own heads only, are stored to EVERY rank's prefix_ptrs[i] buffer at
 *   batch*prefix_batch_stride + row*prefix_row_stride + prefix_head_offset + head*128 + d (the all-gather
 *   of the text output over heads, :968-984).  prefix_rows = 0: none.  A null entry in the out_ptrs of
 *   chitu_b200_qk_norm_rope_scatter / _batch drops that head group (a rank keeps only its own heads of the
 *   replicated rows).
 * chitu_b200_peer_wait_outputs: one warp that waits (bounded) until every rank's output flag has reached
 *   the next epoch: after it, this rank's output buffer is complete, and - because a rank signals only
 *   when its whole attention grid has finished - its q / k / v buffers may be overwritten by the next layer.
 */
#define CHITU_SYNC_INTS 64
typedef struct {
  int* const* blocks;
  int rank, world;
} chitu_b200_peer_sync;
int chitu_b200_qk_norm_rope_batch_signal(const chitu_b200_norm_rope_job* jobs, int n_jobs, int in_dtype, int w_dtype,
                                         float eps, const float* rope_table, int table_rows, int gf, int gh, int gw,
                                         const int* axis_split, int64_t pos_offset, int out_dtype,
                                         const int64_t* out_strides, int heads_per_group, int B, int S, int H, int D,
                                         int round_mid, const chitu_b200_peer_sync* sync, void* stream);
int chitu_b200_attn_fwd_exchange(const void* q, const void* k, const void* v, void* const* out_ptrs, int n_dest,
                                 int rows_per_dest, int64_t dest_batch_stride, int64_t dest_row_stride,
                                 int64_t dest_head_offset, int B, int Sq, int Sk, int H, int D,
                                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                 float softmax_scale, int dtype, int n_splits, void* workspace,
                                 int64_t workspace_bytes, int rows_per_src, int prefix_rows,
                                 void* const* prefix_ptrs, int64_t prefix_batch_stride, int64_t prefix_row_stride,
                                 int64_t prefix_head_offset, const chitu_b200_peer_sync* sync, int* status,
                                 void* stream);
int chitu_b200_peer_wait_outputs(const chitu_b200_peer_sync* sync, int* status, void* stream);

/*
 * Push mode: the same exchange with the key / value transfer overlapped with the attention itself, for small
 * grids, where the exchange is a large share of a layer (Flux on 2 to 8 GPUs).  (Same reference lines; what it
 * replaces in addition is the overlap the reference gets from its side-stream all-to-all in
 * attention_fused, diffusion_attn_backend.py:638-737.)
 *
 * chitu_b200_qk_norm_rope_batch_stage: chitu_b200_qk_norm_rope_batch_signal that announces QUERY rows only
 *   (a flag of their own): point the q job's out_ptrs at the peers' gathered buffers as before, and the k and
 *   v jobs' at LOCAL memory - this rank's own head group in its own gathered buffers, the other groups in a
 *   staging area, block d (block_bytes) holding the rows for rank d in the layout they will have there.
 * chitu_b200_attn_fwd_exchange_push: chitu_b200_attn_fwd_exchange whose grid is extended by copy CTAs
 *   that move the staged blocks into the peers' buffers while the attention CTAs already run: key and
 *   value rows in the order in which the receivers walk their keys, in two stages announced by flags
 *   (stage[0] non-null: the query rows as well, first, for a staging launch that kept them local).  The
 *   attention CTAs wait per source rank for the query rows of their block and for each key / value block
 *   as they reach it; this rank's own rows are already in place.  With a key split under this exchange,
 *   range s takes key tiles s, s + n_splits, ...: every CTA of a query block holds own rows to start on.  The copy CTAs are the first CTAs of the (one-dimensional) grid and never wait, so
 *   they are on the machine before any attention CTA can wait for a peer's; chitu_b200_push_ctas says
 *   how many a shape gets on the current device (40, or what fits beside the attention CTAs where those
 *   leave 8 or more SMs idle).  dest[t][d] is where this rank's block starts in rank d's gathered
 *   q (t = 0), k (1), v (2); entry `rank` is ignored.
 */
typedef struct {
  const void* stage[3];
  void* const* dest[3];
  int64_t block_bytes; /* multiple of 16 */
} chitu_b200_push;
int chitu_b200_push_ctas(int B, int Sq, int H, int n_splits);
int chitu_b200_qk_norm_rope_batch_stage(const chitu_b200_norm_rope_job* jobs, int n_jobs, int in_dtype, int w_dtype,
                                        float eps, const float* rope_table, int table_rows, int gf, int gh, int gw,
                                        const int* axis_split, int64_t pos_offset, int out_dtype,
                                        const int64_t* out_strides, int heads_per_group, int B, int S, int H, int D,
                                        int round_mid, const chitu_b200_peer_sync* sync, void* stream);
int chitu_b200_attn_fwd_exchange_push(const void* q, const void* k, const void* v, void* const* out_ptrs, int n_dest,
                                      int rows_per_dest, int64_t dest_batch_stride, int64_t dest_row_stride,
                                      int64_t dest_head_offset, int B, int Sq, int Sk, int H, int D,
                                      const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                      float softmax_scale, int dtype, int n_splits, void* workspace,
                                      int64_t workspace_bytes, int rows_per_src, const chitu_b200_push* push,
                                      const chitu_b200_peer_sync* sync, int* status, void* stream);

/*
 * Clock budget (GPU cycles) of the flag waits in chitu_b200_peer_barrier and in the arrival-flag
 * polls of the fused exchange; applies to launches made after the call, process-wide.  Returns the
 * previous budget; a non-positive argument only queries.  The default, 2^31 cycles, is about a second -
 * the order of the process-group timeouts the reference relies on to notice a lost rank
 * (chitu_diffusion/core/distributed/comm_group.py:149); tests shorten it so that a wait nobody answers
 * gives up within milliseconds and reports status 5.
 */
long long chitu_b200_set_flag_wait_cycles(long long cycles);

/*
 * How two key ranges (n_splits = 2) are merged, process-wide, for launches made after the call: 1 (default) -
 * the two CTAs of a query block form a thread-block cluster and the second hands its rows to the first
 * through distributed shared memory; 0 - through the workspace, like every other split count.  Returns the
 * previous setting; a negative argument only queries.  No reference counterpart.
 */
int chitu_b200_set_cluster_merge(int enable);

/*
 * Measurement aid, no reference counterpart: a one-thread kernel that writes the GPU's nanosecond timer
 * (%globaltimer) into *slot.  Enqueued between the launches of a layer - also inside a captured graph,
 * where events cannot be read back - it gives the per-launch timeline that bench.py reports.
 */
int chitu_b200_stamp(unsigned long long* slot, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CHITU_B200_H_ */

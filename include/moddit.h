/*
 * moddit.h — C ABI of the B200 (sm_100a) implementation of the MOD-DiT sparse-attention hot path.
 *
 * Conventions for every entry point
 *   - plain pointers and sizes only; all tensor pointers are DEVICE pointers owned by the caller;
 *   - nothing is allocated or freed, and the host is never synchronised with the device: all work
 *     is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream);
 *   - the return value is 0 on success or a negative MODDIT_E_* code; a message for the last
 *     failure on the calling thread is available from moddit_last_error_string();
 *   - q/k/v/out tensors are contiguous (BH, N, D) — "HND" with batch folded into heads — of
 *     `dtype` MODDIT_BF16 or MODDIT_FP16, 16-byte aligned;
 *   - "map" tensors are the reference's block sparsity maps: (H, n, n) float16, 1 = nothing there.
 *
 * Each declaration cites the reference interface it replaces (paths inside the MOD-DiT project).
 */
#ifndef MODDIT_H_
#define MODDIT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MODDIT_BF16 0
#define MODDIT_FP16 1

#define MODDIT_OK 0
#define MODDIT_E_ARG (-1)         /* null pointer, negative size, inconsistent arguments */
#define MODDIT_E_UNSUPPORTED (-2) /* head_dim / block_size / size outside what the kernels cover */
#define MODDIT_E_ALIGN (-3)       /* pointer not 16-byte aligned */
#define MODDIT_E_WORKSPACE (-4)   /* workspace pointer null or too small */
#define MODDIT_E_CUDA (-5)        /* a CUDA runtime/driver call failed (message has the detail) */
#define MODDIT_E_DEVICE (-6)      /* device is not compute capability 10.x */

/* layout codes for masks (token order of the sequence) — MoD/mod/triton_flash_sparsity.py:101-120 */
#define MODDIT_LAYOUT_WAN 0       /* video only */
#define MODDIT_LAYOUT_HUNYUAN 1   /* video first, then text */
#define MODDIT_LAYOUT_COGVIDEOX 2 /* text first, then video */

/* per-head mode codes — MoD/mod/attn_mask.py:408-410,484-486 */
#define MODDIT_MODE_SPARSE 0
#define MODDIT_MODE_BLOCK_DIAGONAL 1
#define MODDIT_MODE_FULL 2

/* Version of this ABI (bumped on any signature change). */
int moddit_abi_version(void);
/* Message describing the last failure on the calling thread ("" if none). */
const char* moddit_last_error_string(void);

/* ---------------------------------------------------------------------------------------------
 * Block mean-pooling of Q and K (no reference function; the specification's first stage.  Nearest
 * reference call site: MoD/mod/attn_mask.py:611-614).
 *   x    : (BH, N, D) bf16/fp16            out : (BH, ceil(N/block_size), D) float32
 * The last block may be short; its mean is over the tokens present.
 */
int moddit_pool_blocks(const void* x, int dtype, int BH, int N, int D, int block_size,
                       float* out, void* stream);

/* The same pooling for a sequence-parallel caller, before the sequence->head exchange (no reference
 * counterpart; the reference pools nothing and re-shards through its host framework).  A rank holds
 * `rows_local` consecutive rows of every head; the first block may start in the previous rank's rows, which
 * arrive in `halo` ((heads, halo_capacity, D), `halo_rows` of them valid, < block_size).  Block i of the
 * rows halo ++ x is block `block_base + i` of the sequence; its mean is stored to the rank owning the head:
 * peer_out[h / heads_per_peer] is that rank's (heads_per_peer, total_blocks, D) float32 buffer (peer-mapped
 * memory is fine: plain stores).  Results equal moddit_pool_blocks on the gathered head bit for bit.
 */
int moddit_pool_blocks_shard(const void* x, const void* halo, int dtype, int heads, int rows_local,
                             int halo_rows, int halo_capacity, int D, int block_size, int n_blocks,
                             float* const* peer_out, int n_peers, int heads_per_peer, int total_blocks,
                             int block_base, void* stream);

/* Pooled stand-in for the sparsity map: with l_ij = qbar[h,qo+i,:].kbar[h,ko+j,:]*scale over the n video
 * blocks, map[h,i,j] = 1 - exp(l_ij - max_j l_ij), written as float16 (no reference function; consumed
 * exactly like the reference map of MoD/mod/triton_flash_sparsity.py:275-341: 1 = nothing there).
 *   qbar,kbar : (BH, nb, D) float32      map : (BH, n, n) float16
 */
int moddit_pooled_map(const float* qbar, const float* kbar, int BH, int nb, int D,
                      int q_block_offset, int k_block_offset, int n, float scale,
                      void* map_f16, void* stream);

/* The same map, bit for bit, in three small launches through a caller-owned workspace of
 * moddit_pooled_map_workspace_bytes(BH, n, D) bytes (16-byte aligned; 4 * BH * n * n for float32 logits plus
 * 8 * BH * n * D for the means split into bfloat16 head / remainder rows): the logits become a batched matrix
 * product with one CTA per 64 x 128 tile, and a last kernel takes the row maxima.  Several times faster than the
 * one-launch form at 24 heads x 900 blocks, and it keeps its speed when a rank holds few heads; no limit on n from
 * shared memory.
 */
size_t moddit_pooled_map_workspace_bytes(int BH, int n, int D);
int moddit_pooled_map_ws(const float* qbar, const float* kbar, int BH, int nb, int D,
                         int q_block_offset, int k_block_offset, int n, float scale,
                         void* map_f16, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Exact sparsity-map replay.  Replaces the pybind function `sparsity_map(q,k,lse,scale,log_thr,
 * q_off,k_off,video_blocks,block_size)` of MoD/mod/cuda_flash_sparsity_kernel.cu:289-334 (kernel
 * :41-169) and the Triton twin MoD/mod/triton_flash_sparsity.py:28-98,181-225.
 *   q,k : (BH, N, D); lse : (BH, N) float32 natural log; map : (BH, n, n) float16
 *   map = count(S[r,c] < lse[r] + log_threshold) / block_size^2 with S = round_dtype(q*scale) k^T.
 */
int moddit_replay_map(const void* q, const void* k, const float* lse, int dtype, int BH, int N, int D,
                      int block_size, float softmax_scale, float log_threshold, int q_video_offset,
                      int k_video_offset, int video_blocks, void* map_f16, void* stream);

/* The same map through a second, independently written kernel (warp-level mma.sync products from register
 * fragments; no TMA, no tensor memory, no waits, hence no status words).  Same arguments and result definition as
 * moddit_replay_map; the two differ only by the order of float32 additions inside a dot product, i.e. in a few
 * comparisons within rounding of the threshold.  It stands where the reference has a second kernel for the same
 * job, the Triton `_sparsity_kernel` behind `_triton_sparsity_map` (MoD/mod/triton_flash_sparsity.py:28-98,181-225),
 * so that the reference test which checks one replay kernel against the other (tests/test_flash_sparsity.py:61-104)
 * still compares two code paths. */
int moddit_replay_map_mma(const void* q, const void* k, const float* lse, int dtype, int BH, int N, int D,
                          int block_size, float softmax_scale, float log_threshold, int q_video_offset,
                          int k_video_offset, int video_blocks, void* map_f16, void* stream);

/* Reads and clears the status words of the replay kernel on the current device (code, block, role,
 * position; all zero unless a bounded wait inside the kernel expired, in which case the maps written
 * since the last call are invalid).  Synchronises `stream`.  No reference counterpart: the reference
 * kernel has no waits. */
int moddit_replay_status(int32_t* host_status4, void* stream);

/* ---------------------------------------------------------------------------------------------
 * M^T S: diagonal sums (offsets -(n-1)..n-1), column sums and the per-frame block-diagonal sum of
 * every head's map, in one pass.  Replaces `compute_mts(S_T, blocks_per_frame)` of
 * MoD/mod/cuda_lstsq_kernel.cu:421-482 (kernels :17-162) and `compute_mts_pytorch`
 * (MoD/mod/cuda_lstsq.py:91-139).  Optionally first merges history as MoD/mod/attn_mask.py:671-675
 * does: merged = keep_mask ? cur : prev, written to `merged_out` (may alias `prev`).
 *   map        : (H, n, n) float16 (current map)
 *   prev       : NULL or (H, n, n) float16       keep_mask : NULL or bool bytes; element (h,i,j) at
 *                keep_mask[h*mask_head_stride + (i+mask_off)*mask_row_stride + (j+mask_off)]
 *   mts        : (H, 3n) float32 = [2n-1 diagonals | n columns | 1 block]
 *   workspace  : moddit_mts_workspace_bytes(H, n) bytes of scratch (contents irrelevant on entry)
 */
size_t moddit_mts_workspace_bytes(int H, int n);
int moddit_mts(const void* map_f16, const void* prev_f16, const uint8_t* keep_mask,
               int64_t mask_head_stride, int64_t mask_row_stride, int mask_off, void* merged_out_f16,
               int H, int n, int blocks_per_frame, float* mts, void* workspace, size_t workspace_bytes,
               void* stream);

/* moddit_mts for callers that cannot hand over a workspace and cannot allocate one.  (No counterpart in
 * the reference.)  Such callers exist: a plug-in run by a host that gives it nothing but input and output
 * buffers and forbids device allocation inside the call, or a process whose framework has already
 * reserved all device memory for its own pool, so that a cudaMalloc from a library would fail.
 * The scratch for the per-tile partial sums is an 8 MiB array built into the library's device image
 * (moddit_mts_noalloc_max_bytes()); every GPU that loads the library holds it until the process exits.
 *   - no history merge: map (H, n, n) float16 in, mts (H, 3n) float32 out, same values as moddit_mts;
 *   - sizes whose scratch need, moddit_mts_workspace_bytes(H, n), exceeds the array are refused with
 *     MODDIT_E_UNSUPPORTED (HunyuanVideo's H=24, n=900 needs 5.1 MB and fits);
 *   - the call allocates and frees nothing.  The first call on each device looks up the array's device
 *     address (cudaGetSymbolAddress); make that first call outside any stream capture.  With the CUDA
 *     runtime's default lazy module loading, that first call is also when the driver loads this part of the
 *     library onto the device and sets the 8 MiB aside: in a process whose framework takes all remaining
 *     device memory, make one warm-up call at start-up, before the framework does (or run with
 *     CUDA_MODULE_LOADING=EAGER, which moves the reservation to library load);
 *   - all calls on a device share the one array and it keeps the last call's contents.  Nothing in it
 *     has to start at zero (each call overwrites what it later reads), but two calls whose kernels can
 *     overlap on the GPU (different streams without an ordering between them) race on it.
 */
size_t moddit_mts_noalloc_max_bytes(void);
int moddit_mts_noalloc(const void* map_f16, int H, int n, int blocks_per_frame, float* mts, void* stream);

/* Structural Gram matrix M^T M + reg*I, (3n x 3n) float32.  Replaces `compute_mtm(S_T, bpf, reg)` of
 * MoD/mod/cuda_lstsq_kernel.cu:319-418 and `compute_mtm_pytorch` (MoD/mod/cuda_lstsq.py:42-89). */
int moddit_mtm(int n, int blocks_per_frame, float regularization, float* mtm, void* stream);

/* The map described by fitted line intensities: out[h,i,j] = d[h, j-i+n-1] + 2*c[h,j] + b_d[h] where rows i and
 * columns j lie in the same frame (blocks of blocks_per_frame, whole frames only).  Replaces
 * `reconstruct_attention_map` (MoD/mod/cuda_lstsq.py:271-360, Python loops over every element there); c is the
 * halved vertical intensity that `solve_lstsq` returns.  d (H, 2n-1), c (H, n), b_d (H) float32; out (H, n, n) float32. */
int moddit_reconstruct_map(const float* d, const float* c, const float* b_d, int H, int n, int blocks_per_frame,
                           float* out, void* stream);

/* One-time set-up of the solve for a geometry (n, blocks_per_frame, regularization): eliminates the
 * 2n-1 diagonal unknowns analytically and inverts the remaining (n+1)x(n+1) system in float64.
 * Replaces the cached `torch.linalg.cholesky(MTM)` of MoD/mod/cuda_lstsq.py:153-186.
 *   factor    : moddit_solve_factor_bytes(n) bytes, filled here, read by moddit_solve
 *   workspace : moddit_solve_prepare_workspace_bytes(n) bytes of scratch
 */
size_t moddit_solve_factor_bytes(int n);
size_t moddit_solve_prepare_workspace_bytes(int n);
int moddit_solve_prepare(int n, int blocks_per_frame, double regularization, void* factor,
                         void* workspace, size_t workspace_bytes, void* stream);

/* X = (M^T M + reg I)^-1 M^T S for all heads.  Replaces `_solve_all_heads` /
 * `torch.cholesky_solve` of MoD/mod/cuda_lstsq.py:189-208,245-261.
 *   mts : (H, 3n) float32        X : (H, 3n) float32, same unknown order
 *   workspace : moddit_solve_workspace_bytes(H, n) bytes of scratch
 */
size_t moddit_solve_workspace_bytes(int H, int n);
int moddit_solve(const float* mts, const void* factor, int H, int n, int blocks_per_frame,
                 double regularization, float* X, void* workspace, size_t workspace_bytes, void* stream);

/* The same solve for small systems in the form the specification words it: the normal equations M^T M + reg*I
 * (3n x 3n, float32, closed form) are built in one CTA's shared memory and Cholesky-factored there
 * (moddit_solve_small_prepare, once per (n, blocks_per_frame, reg): the reference caches its factor the same way,
 * MoD/mod/cuda_lstsq.py:153-186); per call the factor is brought into shared memory and one warp per head runs the
 * forward and back substitution for that head's right-hand side (moddit_solve_small).  Float32 arithmetic like the
 * reference's torch.linalg.cholesky + torch.cholesky_solve on the same system (:177,203); no workspace.
 * Limited to n <= moddit_solve_small_max_n() (3n = 224 unknowns fit shared memory; the first configuration of the
 * specification has n = 64); larger n return MODDIT_E_UNSUPPORTED - use moddit_solve_prepare + moddit_solve, whose
 * structured elimination has no such limit.
 *   factor : moddit_solve_small_factor_bytes(n) bytes (the lower-triangular factor, (3n)^2 float32)
 *   mts    : (H, 3n) float32      X : (H, 3n) float32, same unknown order as moddit_solve */
int moddit_solve_small_max_n(void);
size_t moddit_solve_small_factor_bytes(int n);
int moddit_solve_small_prepare(int n, int blocks_per_frame, float regularization, float* factor, void* stream);
int moddit_solve_small(const float* mts, const float* factor, int H, int n, float* X, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Line selection.  Replaces `choose_topk_lines` (MoD/mod/attn_mask.py:351-370): extrapolate
 * cur + (cur-last)/predict_T for verticals c (H,n) and diagonals d (H,2n-1), concatenate [c | d],
 * pick the k = min(top_k, 3n-1) smallest per head.  Output (H,k) int64 indices in ascending
 * (value, index) order; equal values are taken lowest index first, NaN sorts last.
 */
int moddit_select_lines(const float* cur_c, const float* cur_d, const float* last_c, const float* last_d,
                        int H, int n, int top_k, float predict_T, int64_t* selected, void* stream);

/* Per-head mode from the last block-diagonal coefficient: b_d <= threshold -> BLOCK_DIAGONAL else
 * SPARSE.  Replaces `check_bd_values` (MoD/mod/attn_mask.py:336-349) as called at :408-410. */
int moddit_head_modes(const float* b_d, int H, float threshold, int32_t* modes, void* stream);

/* Bool block mask from selected lines.  Replaces `generate_mask_from_lines`
 * (MoD/mod/attn_mask.py:440-559).  mask: (H, nbt, nbt) bool bytes where nbt = n for WAN and the total
 * number of blocks otherwise; text rows/columns are all true; the video region is the union of the
 * selected columns/diagonals, plus row/bpf == col/bpf for BLOCK_DIAGONAL heads; FULL heads are all true.
 */
int moddit_mask_from_lines(const int64_t* selected, int k, const int32_t* modes, int H, int n,
                           int blocks_per_frame, int layout, int text_blocks, int nbt, uint8_t* mask,
                           void* stream);

/* Static block mask of the radial comparison mode (`--sparse_type radial`).  Replaces `get_radial_mask`
 * (MoD/mod/get_radial_mask.py:157-164; construction :84-130, :47-82, :18-31) for one head - the reference
 * repeats the same mask for every head.  layout: MODDIT_LAYOUT_HUNYUAN or MODDIT_LAYOUT_WAN (the reference
 * raises for anything else).  mask: (seq_len/block_size)^2 bool bytes, text rows and columns all true.
 * The reference always calls it with block_size 128 and decay_factor 0.2. */
int moddit_radial_mask(int layout, int video_tokens, int num_frames, int seq_len, int block_size,
                       float decay_factor, uint8_t* mask, void* stream);

/* Cumulative-mass selection on a darkness map (no reference function).  keep: (H,n,n) bool bytes. */
int moddit_select_mass(const void* map_f16, int H, int n, float tau, uint8_t* keep, void* stream);

/* The two stages of the `--sparse_type spargeattn` comparison mode that the reference delegates to the
 * third-party call `spas_sage2_attn_meansim_topk_cuda(q, k, v, topk=0.5, is_causal=False)`
 * (MoD/mod/attn_mask.py:611-614; the package is an unpinned git submodule whose sources are not in the
 * reference tree, so this follows the method's published description: blocks are represented by their mean,
 * each query block keeps the `topk` share of key blocks with the largest pooled score, and blocks whose rows
 * are not similar to one another are not trusted to their mean).
 * moddit_block_similarity: sim[bh, i] = mean cosine similarity over all pairs of rows of block i of x (BH, N, D),
 *   after subtracting center[bh, :] (float32, may be null) from every row; out (BH, ceil(N/block_size)) float32.
 * moddit_select_topk_blocks: per (head, query block) the `count` key blocks with the smallest map value
 *   (map as moddit_pooled_map writes it: 0 = brightest; ties to the lowest index); row_full (H, n) bool bytes
 *   keeps whole rows, col_keep (H, n) keeps columns in every row (either may be null).  keep: (H, n, n) bool bytes.
 */
int moddit_block_similarity(const void* x, int dtype, int BH, int N, int D, int block_size, const float* center,
                            float* out, void* stream);
int moddit_select_topk_blocks(const void* map_f16, int H, int n, int count, const uint8_t* row_full,
                              const uint8_t* col_keep, uint8_t* keep, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Work lists for the sparse forward: for each (mask head, pair of 128-row query tiles) the key tiles
 * that either tile needs, ascending, each as (key_tile << 8) | (flagsB << 4) | flagsA where flag bit
 * (2*row_half + col_half) marks a kept 64x64 quarter (block_size 128: 0 or 0xF).
 *   mask    : (Hm, nbq, nbk) bool bytes, blocks of `block_size` tokens on the grid that starts at token 0
 *   counts  : (Hm, npairs) int32      entries : (Hm, npairs, ntiles) int32,
 *   order   : NULL or Hm*npairs int32: start order of the (head, pair) work items, order[pos] = head*npairs+pair:
 *             the two longest pairs of every head first, then head after head with the longer lists first
 *             (ties by index); the sparse forward starts its blocks in this order
 *   npairs = ceil(ceil(N/128)/2), ntiles = ceil(N/128); key blocks >= kv_block_limit are dropped.
 * Re-encodes the mask that MoD/mod/attn_mask.py:297-317 hands to the third-party sparse kernel.
 */
int moddit_tile_lists(const uint8_t* mask, int Hm, int nbq, int nbk, int block_size, int N,
                      int kv_block_limit, int32_t* counts, int32_t* entries, int32_t* order, void* stream);
/* The start order alone, for launches over groups of heads: heads [g*heads_per_group, (g+1)*heads_per_group) form
 * group g, whose part of `order` starts at g*heads_per_group*npairs, is laid out like the order of a launch with
 * that many heads and holds indices relative to the group's first head.  heads_per_group = Hm gives the order
 * moddit_tile_lists writes.  (Several GPUs: the sparse forward of a group of heads starts as soon as that group's
 * rows have arrived from the peers.)
 */
int moddit_order_pairs(const int32_t* counts, int Hm, int npairs, int heads_per_group, int32_t* order, void* stream);

/* Block-sparse flash-attention forward.  Replaces `AttentionSparseEngine` (MoD/mod/attn_mask.py:266-331:
 * block_sparse_sage2_attn_cuda for video rows, flashinfer prefill for text rows, sageattn for all-true
 * masks) and, with all-true lists and `lse` non-null, the dense pass of
 * MoD/mod/triton_flash_sparsity.py:314-324.
 *   q,k,v,out : (BH, N, D); head bh uses lists of mask head bh % Hm
 *   order     : NULL (work items in index order) or the Hm*npairs start order from moddit_tile_lists
 *   rows < q_split attend keys < kv_len_lo, other rows keys < kv_len_hi
 *   lse       : NULL or (BH, N) float32 natural-log row log-sum-exp
 *   status    : device int32[4], zeroed by the caller; non-zero afterwards means a bounded wait
 *               expired inside the kernel (status[0]=code, [1]=block, [2]=role) and `out` is invalid
 */
int moddit_sparse_attn_fwd(const void* q, const void* k, const void* v, int dtype, int BH, int N, int D,
                           const int32_t* counts, const int32_t* entries, const int32_t* order, int Hm,
                           float softmax_scale, int q_split, int kv_len_lo, int kv_len_hi, void* out,
                           float* lse, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Strided row copy: `rows` rows of `width_bytes` bytes from src (pitch src_pitch) to dst (pitch dst_pitch).
 * `dst` may be a peer GPU's memory mapped into this process; the kernel uses plain loads and stores.  It is
 * the building block of the sequence<->head re-shard (the reference has only dead hooks for that exchange,
 * MoD/models/cogvideox/attention_processor.py:138-155,220-229).  All of pointers, pitches and width must be
 * multiples of 16 bytes.
 */
int moddit_copy_rows(const void* src, void* dst, int64_t src_pitch, int64_t dst_pitch, int64_t width_bytes,
                     int rows, void* stream);
/* The same copy for n_jobs (at most 24) source/destination pairs in one launch; `src` and `dst` are HOST
 * arrays of device pointers. */
int moddit_copy_rows_multi(const void* const* src, void* const* dst, int n_jobs, int64_t src_pitch,
                           int64_t dst_pitch, int64_t width_bytes, int rows, void* stream);
/* The same jobs on at most `max_ctas` CTAs that walk 64 KB segments round-robin: an exchange that runs beside other
 * kernels leaves them the rest of the GPU (moddit_copy_rows_multi fills it). */
int moddit_copy_rows_narrow(const void* const* src, void* const* dst, int n_jobs, int64_t src_pitch,
                            int64_t dst_pitch, int64_t width_bytes, int rows, int max_ctas, void* stream);

/* The same copy on the GPU's copy engines (one asynchronous 2-D copy, no kernel): for the bulk pieces of the
 * re-shard, which then neither occupy SMs nor compete with the step's kernels; no alignment requirement. */
int moddit_copy_rows_dma(const void* src, void* dst, int64_t src_pitch, int64_t dst_pitch, int64_t width_bytes,
                         int rows, void* stream);

/* moddit_sparse_attn_fwd with the output re-shard fused into the epilogue: rows of sequence shard r
 * ([r*N/n_peers, (r+1)*N/n_peers)) of local head bh are stored into peer_out[r], a (total_heads, N/n_peers, D)
 * buffer of rank r mapped into this process, at head `head_base + bh` (plain peer stores).  `peer_out` is a
 * HOST array of n_peers (at most 8) device pointers.  The caller separates these stores from the readers
 * with its own cross-rank barrier.  No reference counterpart beyond the dead hooks cited above. */
int moddit_sparse_attn_fwd_scatter(const void* q, const void* k, const void* v, int dtype, int BH, int N, int D,
                                   const int32_t* counts, const int32_t* entries, const int32_t* order, int Hm,
                                   float softmax_scale, int q_split, int kv_len_lo, int kv_len_hi,
                                   void* const* peer_out, int n_peers, int head_base, float* lse,
                                   int32_t* status, void* stream);

/* Attention prologue: the steps of the reference's attention processors between the q/k/v projections and the
 * attention call, in one pass (MoD/models/hunyuan/attention_processor.py:57-106: unflatten + transpose,
 * norm_q / norm_k, rotary embedding of the latent tokens, concatenation with the text stream;
 * MoD/models/wan/attention_processor.py:70-93,123-125; MoD/models/cogvideox/attention_processor.py:113-135).
 * The normalisation modules and the Hunyuan/CogVideoX rotary function come from the `diffusers` package, which
 * the reference leaves unpinned and which is not part of its tree; their arithmetic is restated here:
 *   MODDIT_NORM_RMS_HEAD      y = T(T(x * rsqrt(mean_D(x^2) + eps)) * w)         (RMSNorm over head_dim)
 *   MODDIT_NORM_RMS_ALL_HEADS the same with the mean over all H*D values of the token, w of H*D values (Wan)
 *   MODDIT_NORM_LAYER         y = T((x - mean) * rsqrt(var + eps) * w + b)       (LayerNorm over head_dim)
 * (float32 arithmetic, T(.) = rounding to the tensors' 16-bit type; null weight/bias = 1/0), then for tokens
 * s in [rope_lo, rope_hi), with c = rope_cos[s - rope_lo], n = rope_sin[s - rope_lo] (float32 rows of D):
 *   MODDIT_ROPE_ELEMENTWISE        out[2i] = y[2i]*c[2i] - y[2i+1]*n[2i],   out[2i+1] = y[2i]*n[2i+1] + y[2i+1]*c[2i+1]
 *   MODDIT_ROPE_EVEN_COS_ODD_SIN   out[2i] = y[2i]*c[2i] - y[2i+1]*n[2i+1], out[2i+1] = y[2i]*n[2i+1] + y[2i+1]*c[2i]
 *   MODDIT_ROPE_PAIR               tables of D/2 values per token, one (c[i], n[i]) per pair:
 *                                  out[2i] = y[2i]*c[i] - y[2i+1]*n[i],     out[2i+1] = y[2i]*n[i] + y[2i+1]*c[i]
 * (the second is the function defined at MoD/models/wan/attention_processor.py:78-90; the third equals both
 * others on the tables the models use, whose entries repeat over each pair, at half the table traffic),
 * products rounded separately in float32, the sum rounded once to T.  v is only moved.
 *   q_in,k_in,v_in : (B, S, >= H*D) token-major, `token_stride` elements between tokens (a slice of a fused
 *                    projection is fine); any of them may be null and is then skipped
 *   q_out,k_out,v_out : (B, H, N_out, D) head-major; token s is stored at row dst_row0 + s, so a text stream
 *                    projected separately is appended by a second call
 *   q_pool,k_pool  : optional (B*H, ceil(N_out/block_size), D) float32 block means of the stored q / k rows
 *                    (what moddit_pool_blocks returns for the finished tensor, bit for bit); needs dst_row0
 *                    on a block boundary and S a multiple of block_size unless the call ends the sequence
 *   workspace      : moddit_qkv_prologue_workspace_bytes(...) bytes, only for MODDIT_NORM_RMS_ALL_HEADS
 */
#define MODDIT_NORM_NONE 0
#define MODDIT_NORM_RMS_HEAD 1
#define MODDIT_NORM_RMS_ALL_HEADS 2
#define MODDIT_NORM_LAYER 3
#define MODDIT_ROPE_ELEMENTWISE 0
#define MODDIT_ROPE_EVEN_COS_ODD_SIN 1
#define MODDIT_ROPE_PAIR 2
size_t moddit_qkv_prologue_workspace_bytes(int B, int S, int norm_kind);
int moddit_qkv_prologue(const void* q_in, const void* k_in, const void* v_in, int dtype, int B, int S, int H,
                        int D, int64_t token_stride, int norm_kind, const void* q_weight, const void* q_bias,
                        const void* k_weight, const void* k_bias, float eps, const float* rope_cos,
                        const float* rope_sin, int rope_form, int rope_lo, int rope_hi, void* q_out, void* k_out,
                        void* v_out, int N_out, int dst_row0, float* q_pool, float* k_pool, int block_size,
                        void* workspace, size_t ws_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MODDIT_H_ */

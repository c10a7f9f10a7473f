/*
 * logo_b200 -- C ABI of the B200 (sm_100a) kernels behind the LoGo attention hot path.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its comment says "host".
 *   - The device that owns the pointers and the stream must be the calling thread's current
 *     device (cudaSetDevice) when an entry point is called: launches, the per-device caches
 *     (SM count, kernel attributes) and the static scratch of logo_select_rows_static all go
 *     by the current device.
 *   - The caller owns all memory (inputs, outputs, workspaces); the library never
 *     allocates, frees or keeps device memory across calls, and never synchronises
 *     the host with the device. All work is enqueued on `stream`.
 *   - Token tensors are packed varlen: rows are tokens of all sequences back to back,
 *     `cu_seqlens[n_seq + 1]` (int32) holds the sequence boundaries.
 *   - Functions return LOGO_OK (0) or an error code; logo_last_error() gives the text.
 *     Device-side problems (a bounded wait that expired, an index out of range) are
 *     reported asynchronously through the caller-provided `status` word (int32,
 *     device memory, zero-initialised by the caller); 0 = ok.
 *   - Only head_dim 128 and bf16 activations are supported.
 *
 * Each entry point cites the reference interface (Pan-Yuqi/Logo, path:line) it replaces.
 */
#ifndef LOGO_B200_H_
#define LOGO_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* logo_stream_t; /* == cudaStream_t */

enum {
  LOGO_OK = 0,
  LOGO_ERR_INVALID = 1,     /* bad shape, dtype, alignment or argument            */
  LOGO_ERR_CUDA = 2,        /* a CUDA runtime / driver call failed                */
  LOGO_ERR_UNSUPPORTED = 3, /* valid request outside what the kernels implement   */
  LOGO_ERR_WORKSPACE = 4    /* workspace too small                                */
};

enum {
  LOGO_DTYPE_BF16 = 0,
  LOGO_DTYPE_F32 = 1,
  LOGO_DTYPE_F16 = 2,
  LOGO_DTYPE_BOOL = 3 /* one byte per element, non-zero = true */
};

/* Values a kernel may leave in the device status word. */
enum {
  LOGO_DEV_OK = 0,
  LOGO_DEV_WAIT_TIMEOUT = 1, /* a bounded barrier wait expired; results are invalid */
  LOGO_DEV_BAD_INDEX = 2,    /* an index derived from q_idx / cu_seqlens was out of range */
  LOGO_DEV_SCAN_TIMEOUT = 3  /* the prefix-scan look-back gave up                     */
};

/* Query-tile height of the attention kernels (compacted rows per tile). */
#define LOGO_TILE 128

/* Size of the `meta` buffer and the slots the attention kernels use in it. */
#define LOGO_META_INTS 16
#define LOGO_META_COUNTER_SQ_FWD 8
#define LOGO_META_COUNTER_SWA_FWD 9
#define LOGO_META_COUNTER_SQ_DKV 10
#define LOGO_META_COUNTER_SQ_DQ 11
#define LOGO_META_COUNTER_SWA_DKV 12
#define LOGO_META_COUNTER_SWA_DQ 13

/* Library version: major * 10000 + minor * 100 + patch. */
int logo_version(void);

/* Copies the calling thread's last error text into buf (host, NUL-terminated); returns its length. */
int logo_last_error(char* buf, int n);

/* ------------------------------------------------------------------------------------------
 * Row selection and compaction.
 * Replaces logo/ops/common.py:71-107 (build_selection), :110-124 (prepare_chunk_indices) and
 * the threshold test of logo/layers/logo.py:190, plus the counters of logo/layers/logo.py:251-255.
 *
 *   gate        [n_tokens] of gate_dtype (BF16 / F16 / F32: row i is selected iff
 *               float(gate[i]) >= float(*thres); BOOL: row i is selected iff gate[i] != 0,
 *               thres is ignored and may be NULL)
 *   thres       device scalar of thres_dtype (BF16 / F16 / F32)
 *   cu_seqlens  [n_seq + 1] int32, non-decreasing, cu_seqlens[0] == 0, cu_seqlens[n_seq] == n_tokens
 * Outputs
 *   q_idx        [n_tokens] int64; the first Sq entries are the selected token indices, ascending
 *   pos_ids      [n_tokens] int32; position of each selected token inside its sequence
 *   cu_seqlens_q [n_seq + 1] int32; prefix sum of selected rows per sequence
 *   tile_off     [4][n_seq + 1] int32 work-tile prefix sums consumed by the attention kernels:
 *                row 0: ceil(selected rows of the sequence / 256)  (query-tile pairs, global branch)
 *                row 1: ceil(sequence length / 128)                (key tiles, backward)
 *                row 2: ceil(sequence length / 256)                (query-tile pairs, local branch)
 *                row 3: ceil(selected rows of the sequence / 128)  (query tiles, backward)
 *   meta         [LOGO_META_INTS] int32: [0] Sq, [1..4] totals of rows 0..3, [5..7] 0; entries 8..15 are
 *                scratch of the attention kernels (their work-claim counters, reset at every launch):
 *                two launches of the same attention entry point that share one meta buffer must not
 *                overlap on the GPU
 *   gate_sum     [1] fp32, sum of float(gate) over all rows (0 for BOOL); may be NULL
 *   workspace    logo_select_workspace_bytes(n_tokens) bytes, 16-byte aligned
 * Nothing is copied to the host: Sq stays on the device, so q_idx / pos_ids are sized for n_tokens.
 * ------------------------------------------------------------------------------------------ */
size_t logo_select_workspace_bytes(int n_tokens);

int logo_select_rows(const void* gate, int gate_dtype, const void* thres, int thres_dtype,
                     const int32_t* cu_seqlens, int n_seq, int n_tokens, int64_t* q_idx, int32_t* pos_ids,
                     int32_t* cu_seqlens_q, int32_t* tile_off, int32_t* meta, float* gate_sum, void* workspace,
                     size_t workspace_bytes, int32_t* status, logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * logo_select_rows without a caller workspace. It has no counterpart in the reference.
 *
 * For hosts that may not allocate device memory themselves -- a plugin inside a serving
 * process whose memory budget is fixed at start-up, or a step on a latency-critical path where
 * cudaMalloc / cudaFree are off limits because they serialise the device -- the scan scratch
 * lives in a static device array inside the library (about 6 KB; every GPU that loads the
 * library holds it until the process exits). Inputs and outputs are still the caller's and
 * mean exactly what they mean for logo_select_rows; results are identical.
 *
 *   - n_tokens must not exceed LOGO_SELECT_STATIC_MAX_TOKENS; larger inputs are refused with
 *     LOGO_ERR_UNSUPPORTED and an explanatory logo_last_error() text.
 *   - The call performs no cudaMalloc / cudaFree and calls no allocating library routine.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and caches it; make that first call
 *     before any stream capture begins.
 *   - All calls on a device share the one array, and it still holds what the previous call
 *     wrote: the function clears the part it needs on `stream` first. Two calls that can overlap
 *     on the GPU (different streams, or different host threads) race on it -- serialise them.
 *   - The cached address does not survive cudaDeviceReset: do not call this entry point on a
 *     device after resetting it.
 * ------------------------------------------------------------------------------------------ */
#define LOGO_SELECT_STATIC_MAX_TOKENS (1 << 20)

int logo_select_rows_static(const void* gate, int gate_dtype, const void* thres, int thres_dtype,
                            const int32_t* cu_seqlens, int n_seq, int n_tokens, int64_t* q_idx, int32_t* pos_ids,
                            int32_t* cu_seqlens_q, int32_t* tile_off, int32_t* meta, float* gate_sum,
                            int32_t* status, logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Query-sparse causal attention, forward (global branch).
 * Replaces logo/ops/selected_full_attn.py:33-121 (sq_full_attn_fwd_kernel), :340-362 (_fwd) and the
 * gather / scatter of :461,469-470 (SQFullAttentionFunction.forward).
 *
 *   q [n_tokens, hq, 128], k, v [n_tokens, h, 128] bf16, contiguous; hq % h == 0
 *   q_idx, pos_ids, cu_seqlens_q, tile_off, meta: outputs of logo_select_rows
 *   o   [n_tokens, hq, 128] bf16: rows listed in q_idx are written; with zero_fill != 0 every other
 *       row is set to 0 by the same kernel (the reference returns zeros for unselected rows, :469-471)
 *   lse [n_tokens, hq] fp32 or NULL: base-2 log-sum-exp of scale * log2(e) * q.k for selected rows
 *       (the reference keeps it compacted, :118-121; here it is indexed by token)
 *   scale: softmax scale, > 0 (the reference default is 128 ** -0.5, :523-524)
 * ------------------------------------------------------------------------------------------ */
int logo_sq_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int64_t* q_idx,
                     const int32_t* pos_ids, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                     const int32_t* tile_off, int32_t* meta, int n_seq, int n_tokens, int hq, int h, int d,
                     float scale, int zero_fill, int32_t* status, logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Sliding-window causal attention, forward (local branch): row i attends keys [i - window, i] of
 * its own sequence. Replaces the flash-attn call of logo/layers/logo.py:166-179 (through
 * logo/layers/utils.py:157-178 with window_size=(window, window), causal).
 *   tile_off, meta: outputs of logo_select_rows for the same cu_seqlens (rows 2 / entry 3 are used)
 * ------------------------------------------------------------------------------------------ */
int logo_swa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int32_t* cu_seqlens,
                 const int32_t* tile_off, int32_t* meta, int n_seq, int n_tokens, int hq, int h, int d,
                 int window, float scale, int32_t* status, logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Backward of both attention branches.
 * logo_sq_attn_bwd replaces logo/ops/selected_full_attn.py:124-138 (delta), :141-228 (dQ),
 * :231-337 (dK/dV), :374-402 (_compute_q_start_blk), :405-446 (_bwd incl. the GQA reduction of
 * :444-445) and the gather / scatter / casts of :483-491 (SQFullAttentionFunction.backward).
 * logo_swa_bwd is the backward of the flash-attn call of logo/layers/logo.py:166-179.
 *
 *   q, k, v, o, lse: as given to / produced by the matching forward call
 *   d_o [n_tokens, hq, 128] bf16: gradient of o (rows of unselected tokens are ignored)
 *   dq  [n_tokens, hq, 128] bf16: fully written (zeros on unselected rows, :487-488)
 *   dk, dv [n_tokens, h, 128] bf16: fully written
 *   workspace: logo_attn_bwd_workspace_bytes(n_tokens, hq, gathered) bytes, 256-byte aligned;
 *              gathered = 1 for logo_sq_attn_bwd (packed copies of the selected Q / dO rows,
 *              head-major lse and delta, fp32 dQ accumulator, the per-row lse / delta terms the single
 *              pass feeds to the tensor core), 0 for logo_swa_bwd (the same without the packed copies)
 *
 * Two implementations exist per branch (0 = global / logo_sq_attn_bwd, 1 = local / logo_swa_bwd),
 * chosen process-wide with logo_set_backward_mode(branch, mode):
 *   mode 0  single pass: S and dP are formed once per (query tile, key tile) pair and give dK, dV
 *           and dQ (five tile products; the reference's two kernels, :141-337, execute seven). dQ is
 *           summed over key tiles with fp32 reductions in global memory whose order is not fixed,
 *           so dq may differ between two runs in the last bit of the sum; dk and dv are
 *           reproducible. Default for branch 0.
 *   mode 1  two kernels (dK/dV, then dQ), every output accumulated in a fixed order: bit-identical
 *           results from run to run. Default for branch 1.
 * ------------------------------------------------------------------------------------------ */
size_t logo_attn_bwd_workspace_bytes(int n_tokens, int hq, int gathered);

int logo_set_backward_mode(int branch, int mode);
int logo_get_backward_mode(int branch); /* current mode of the branch, -1 for an unknown branch */

int logo_sq_attn_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                     void* dq, void* dk, void* dv, const int64_t* q_idx, const int32_t* pos_ids,
                     const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* tile_off,
                     int32_t* meta, void* workspace, size_t workspace_bytes, int n_seq, int n_tokens, int hq,
                     int h, int d, float scale, int32_t* status, logo_stream_t stream);

int logo_swa_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                 void* dq, void* dk, void* dv, const int32_t* cu_seqlens, const int32_t* tile_off,
                 int32_t* meta, void* workspace, size_t workspace_bytes, int n_seq, int n_tokens, int hq, int h,
                 int d, int window, float scale, int32_t* status, logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Per-branch RMSNorm + gate mask + blend.
 * Replaces logo/modules/layernorm.py:17-22 as used at logo/layers/logo.py:180-182 and :225-227,
 * and the masked blend of logo/layers/logo.py:256-258:
 *     g = gate >= thres ? gate : 0;   out = (1 - g) * norm_l(local) + g * norm_g(glob)
 *   local, glob [n_tokens, h, 128] bf16 (glob rows of unselected tokens are never read)
 *   gate [n_tokens] bf16; thres: device scalar (bf16 / fp16 / fp32)
 *   w_local, w_global [128] of w_dtype (bf16 / fp32); ignored when use_norm == 0
 *   out [n_tokens, h * 128] bf16
 * The backward writes d_local, d_glob [n_tokens, h, 128] bf16 (d_glob = 0 on unselected tokens),
 * d_gate [n_tokens] bf16 (0 where the gate was masked) and the two [128] weight gradients
 * (w_dtype; may be NULL). workspace: logo_fuse_bwd_workspace_bytes(n_tokens) bytes.
 * ------------------------------------------------------------------------------------------ */
int logo_fuse_fwd(const void* local, const void* glob, const void* gate, int gate_dtype, const void* thres,
                  int thres_dtype, const void* w_local, const void* w_global, int w_dtype, void* out, int n_tokens,
                  int h, int d, float eps, int use_norm, logo_stream_t stream);

size_t logo_fuse_bwd_workspace_bytes(int n_tokens);

int logo_fuse_bwd(const void* d_out, const void* local, const void* glob, const void* gate, int gate_dtype,
                  const void* thres, int thres_dtype, const void* w_local, const void* w_global, int w_dtype,
                  void* d_local, void* d_glob, void* d_gate, void* d_w_local, void* d_w_global, int n_tokens, int h,
                  int d, float eps, int use_norm, void* workspace, size_t workspace_bytes, logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * RMSNorm forward over rows of any width (logo/modules/layernorm.py:9-26, the module the model
 * also uses for its decoder-stack norms):
 *     out = weight * bf16(x * rsqrt(mean(x^2) + eps))
 *   x, out [rows, dim] bf16 contiguous, weight [dim] bf16, dim a multiple of 8.
 * Inference path only (no gradient kernel): the Python module falls back to the eager expression
 * whenever autograd needs the graph.
 * ------------------------------------------------------------------------------------------ */
int logo_rmsnorm_fwd(const void* x, const void* weight, void* out, long long rows, int dim, float eps,
                     logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Gated activation of the model's MLP (logo/modules/mlp.py:25, hidden_act "silu"):
 *     out = silu(gate) * up      (silu in fp32, rounded to bf16, then one bf16 multiplication)
 *   gate, up: bf16 rows of `dim` elements at element strides gate_stride / up_stride (multiples of 8:
 *   the two halves of a fused gate-up projection can be passed as views); out [rows, dim] packed.
 * Inference path only (no gradient kernel).
 * ------------------------------------------------------------------------------------------ */
int logo_silu_mul(const void* gate, long long gate_stride, const void* up, long long up_stride, void* out,
                  long long rows, int dim, logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Rotary position embedding. Replaces apply_rotary_pos_emb (logo/modules/rotary.py:81-106, rotate_half :81-85) as
 * called at logo/layers/logo.py:136-139 for both branches:
 *     out = (x * cos) + (rotate_half(x) * sin)
 * with the three bf16 roundings of that eager expression, in one pass.
 *   x: bf16 rows of 128, row (token t, head h) at x + t * x_stride_tok + h * x_stride_head (element
 *      strides, multiples of 8); out [n_tokens, heads, 128] bf16 packed (may alias a packed x);
 *   cos, sin [n_tokens, 128] bf16
 *   inverse != 0 applies the transposed rotation: the gradient with respect to x of the
 *   expression above, given the output gradient in `x`.
 * ------------------------------------------------------------------------------------------ */
int logo_rope(const void* x, long long x_stride_tok, long long x_stride_head, void* out, const void* cos,
              const void* sin, int n_tokens, int heads, int d, int inverse, logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Per-head re-parameterisation of the global branch fused with the rotary embedding. Replaces the
 * einsum of logo/layers/logo.py:86-94 ('b l h d, h d e -> b l h e'), apply_rotary_pos_emb at
 * logo/layers/logo.py:137-139 and the transpose / contiguous copies of :156-158 for one tensor:
 *     out[t, h, :] = rope( bf16( x[t, h, :] @ w[h] ) )
 *   x    bf16 rows of heads * 128 at x_stride elements (a multiple of 8) per token
 *   w    bf16 [heads, 128, 128] ([head][in][out], the layout of q/k/v_global_proj)
 *   rows NULL: every token. Otherwise the ascending token indices to compute (q_idx of
 *        logo_select_rows) with their count in the device scalar n_rows: only those rows of `out`
 *        are written -- the global QUERY projection is needed for selected rows only.
 *   cos_t, sin_t [n_tokens, 128] bf16, or both NULL for no rotation (the value projection)
 *   out  bf16 [n_tokens, heads * 128], token-major
 * The product is rounded to bf16 before the rotation, and the rotation keeps the three bf16 roundings
 * of the eager expression (as logo_rope does).
 * ------------------------------------------------------------------------------------------ */
int logo_proj_rope(const void* x, long long x_stride, const void* w, const int64_t* rows, const int32_t* n_rows,
                   const void* cos_t, const void* sin_t, void* out, int n_tokens, int heads, int d, int32_t* status,
                   logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * KV cache (bf16, head-major):
 *   global branch: k_cache, v_cache [batch, h, t_max, 128]; token p of a sequence sits at row p
 *   local branch : k_ring,  v_ring  [batch, h, ring, 128];  token p sits at row p % ring
 *                  (ring = window + 1 keeps exactly the keys a decode step may see)
 *
 * logo_cache_append replaces the torch.cat updates of logo/cache.py:79-118 and the per-step
 * transpose().contiguous() copies of logo/layers/logo.py:153-158: it writes t_new new tokens per
 * sequence in place. Inputs are [batch, t_new, h, 128] views with element strides
 * (stride_b, stride_t, stride_h), multiples of 8. Token t of sequence b lands at position
 * (start_lens ? start_lens[b] : start) + t. Either pair (ring / cache) may be NULL.
 *
 * logo_decode_attn replaces the q_len == 1 path of logo/layers/logo.py:166-179 (local, 129 keys)
 * and :228-249 (global): one query per sequence against the cache. Sequences whose
 * gate[b] < *thres skip the global branch entirely and get o_global = 0 (the reference runs
 * dense attention for every sequence whenever any gate passes and masks afterwards, :229-256).
 *   q_local, q_global, o_local, o_global [batch, hq, 128] bf16
 *   ctx_lens [batch] int32: cached tokens of each sequence INCLUDING the token just appended
 *   max_ctx: upper bound of ctx_lens known to the host (sizes the grid); hq / h in {1, 2, 4}
 *   workspace: logo_decode_workspace_bytes(batch, hq, max_ctx) bytes
 * ------------------------------------------------------------------------------------------ */
int logo_cache_append(const void* k_local, const void* v_local, const void* k_global, const void* v_global,
                      long long stride_b, long long stride_t, long long stride_h, void* k_ring, void* v_ring,
                      int ring, void* k_cache, void* v_cache, int t_max, const int32_t* start_lens, int start,
                      int batch, int t_new, int h, int d, int32_t* status, logo_stream_t stream);

size_t logo_decode_workspace_bytes(int batch, int hq, int max_ctx);

int logo_decode_attn(const void* q_local, const void* q_global, const void* k_ring, const void* v_ring, int ring,
                     const void* k_cache, const void* v_cache, int t_max, const int32_t* ctx_lens, const void* gate,
                     int gate_dtype, const void* thres, int thres_dtype, void* o_local, void* o_global, int batch,
                     int hq, int h, int d, int max_ctx, float scale, void* workspace, size_t workspace_bytes,
                     int32_t* status, logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Language-model loss over lm_head logits. Replaces the label shift, the packed-boundary masking and
 * the CrossEntropyLoss of logo/modeling_logo.py:380-407.
 *
 * logo_shift_labels: targets[i] = labels[i + 1] for every token that has a successor INSIDE its packed
 *   sequence, ignore_index otherwise (the reference shifts logits / labels by one and sets
 *   shift_labels[cu_seqlens[1:-1] - 1] = -100, :392-394); n_valid [1] int32 receives the number of
 *   targets that are not ignore_index (the denominator of the mean).
 * logo_ce_rows: for each of `rows` rows of bf16 logits (row r at logits + r * row_stride elements;
 *   vocab and row_stride multiples of 8): row_loss[r] = logsumexp(row) - row[target] in fp32 (0 for an
 *   ignored row). With write_grad != 0 the row is then overwritten in place by the gradient of
 *   upstream * mean loss, (softmax(row) - onehot(target)) * upstream / *n_valid, as bf16 (zeros for an
 *   ignored row): the caller multiplies it with the lm_head weight / the hidden states and never holds
 *   fp32 logits (the reference upcasts the whole [tokens, vocab] tensor, :385).
 * ------------------------------------------------------------------------------------------ */
int logo_shift_labels(const int64_t* labels, const int32_t* cu_seqlens, int n_seq, int n_tokens,
                      long long ignore_index, int64_t* targets, int32_t* n_valid, logo_stream_t stream);

int logo_ce_rows(void* logits, long long row_stride, const int64_t* targets, long long ignore_index, float* row_loss,
                 const int32_t* n_valid, float upstream, int rows, int vocab, int write_grad, int32_t* status,
                 logo_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Per-kernel timing for benchmarks (no counterpart in the reference). While enabled on the
 * calling host thread, every launch of the kernels below is bracketed by CUDA events on its
 * stream. logo_profile_read waits for those events, returns per kernel kind the summed device
 * time in ms and the number of launches since the last read, and releases the events.
 *   kind 0 select + finalize, 1 attention forward, 2 backward preprocess,
 *        3 backward dK/dV, 4 backward dQ (the two-kernel backward),
 *        5 single-pass backward, 6 its dQ convert / scatter kernel
 * ------------------------------------------------------------------------------------------ */
int logo_profile_enable(int on);
/* Creates the events for `n_launches` timed kernel launches ahead of time (at most 4096), so that a
 * timed loop creates none: the driver can stall a stream for milliseconds when its event pool grows. */
int logo_profile_reserve(int n_launches);
int logo_profile_read(double* total_ms, int* launches, int n);

/* ------------------------------------------------------------------------------------------
 * Diagnostics: single-tile tcgen05 matrix multiply used by the GPU test-suite to pin the
 * shared-memory / tensor-memory operand encodings the attention kernels rely on.
 * No counterpart in the reference.
 *   mode 0: C = A * B^T   (A, B both K-major in shared memory)
 *   mode 1: C = A * B     (B row-major [k][n], i.e. MN-major operand)
 *   mode 2: C = A * B     (A staged in tensor memory, B MN-major)
 *   mode 3: C = A^T * B   (both operands MN-major: rows of a and b are the reduction index)
 *   mode 4: C = A * B^T + A[:, 0:16] * B[:, 0:16]^T   (mode 0 plus a ninth k-step whose [128][16]
 *           operand tiles use the 32-byte swizzle)
 *   mode 5: C = A * B^T + 1 x (a[0, 0:16] . B[:, 0:16]^T)   (the ninth k-step's A operand is a 256-byte
 *           tile of identical rows without swizzle; kstep_bytes / sbo_bytes are its distances between
 *           K chunks / 8-row groups: 128 / 0)
 *   a, b: bf16 [128][128] row-major; c: fp32 [128][128]
 *   flags bit 0 / bit 2: stage A / B through thread-written swizzled shared memory instead of TMA.
 *   flags bit 3: nothing ever arms the barrier the kernel waits on, so the wait runs out: the kernel
 *     must return with LOGO_DEV_WAIT_TIMEOUT in `status` and leave c untouched (the test of the
 *     bounded waits every kernel of this library shares).
 *   flags bits 8-23: limit of every wait of this launch in microseconds (0: the default, 1 s).
 * ------------------------------------------------------------------------------------------ */
int logo_umma_selftest(int mode, int flags, const void* a, const void* b, float* c, uint32_t lbo_bytes,
                       uint32_t sbo_bytes, uint32_t kstep_bytes, int32_t* status, logo_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LOGO_B200_H_ */

/* C ABI of libflagtree_b200.so: hand-written sm_100a kernels behind plain pointers and sizes.
 *
 * Conventions
 *  - Every entry point returns an int status (FTB_OK = 0).  Nothing aborts or exits.
 *  - Pointers are device pointers unless a comment says "host".  `stream` is a cudaStream_t
 *    passed as void* (NULL = the legacy default stream).  No entry point synchronises the
 *    host unless documented.
 *  - Strides are in ELEMENTS of the tensor's dtype; the innermost dimension is contiguous.
 *  - Inputs are never written.
 *
 * Each declaration cites the reference interface (file:line inside the FlagTree checkout)
 * whose role it takes over.
 */
#ifndef FLAGTREE_B200_H_
#define FLAGTREE_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define FTB_API __attribute__((visibility("default")))
#else
#define FTB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
  FTB_OK = 0,
  FTB_ERR_INVALID = 1,     /* bad argument: shape, stride, alignment, null pointer           */
  FTB_ERR_CUDA = 2,        /* a CUDA runtime call failed (see ftb_last_error_string)          */
  FTB_ERR_TIMEOUT = 3,     /* a bounded device-side wait ran out                              */
  FTB_ERR_BAD_INDEX = 4,   /* an index other than the -1 padding that names no row (never read) */
  FTB_ERR_UNSUPPORTED = 5
};

/* Library/ABI version and last error text (host string, valid until the next failing call). */
FTB_API int ftb_abi_version(void);
FTB_API const char* ftb_last_error_string(void);

/* ------------------------------------------------------------------------------------------
 * Top-k sparse MLA forward.
 *
 * Replaces the two launches of the reference's gather-by-index MLA decode attention:
 *   third_party/mthreads/python/test/wmma/test_accuracy_musa_vllm_mla.py:206-337
 *     (_fwd_grouped_kernel_stage1: gather, q.k over 512+64 dims, online softmax, p.v)
 *   same file :426-477 (_fwd_kernel_stage2: merge of the kv splits)
 *   and their host wrappers :340-423, :480-510, :571-620 (decode_attention_fwd).
 * The reference's Req_to_tokens table with PAGE_SIZE=1 is `indices`; B_Seqlen is implied by
 * the -1 padding.  Splitting over the kv axis is internal.
 * ------------------------------------------------------------------------------------------ */
typedef struct ftb_sparse_mla_args {
  const void* q;            /* bf16 [s_q, h, 576]                                           */
  const void* kv;           /* bf16 [s_kv, 576]  (dense form)  -- or --
                               e4m3 [num_pages*page_size, 576] (paged FP8 form)               */
  const int32_t* indices;   /* int32 [s_q, topk]; -1 = padding.  Paged form: LOGICAL positions */
  void* out;                /* bf16 [s_q, h, 512]                                           */
  float* lse;               /* fp32 [s_q, h]; natural log unless lse_base2                   */
  int32_t s_q, h, s_kv, topk;
  int64_t q_stride_token, q_stride_head;
  int64_t kv_stride_row;
  int64_t idx_stride_token;
  int64_t out_stride_token, out_stride_head;
  int64_t lse_stride_token;
  float sm_scale;
  int32_t lse_base2;        /* 0: lse = log sum exp(s);  1: log2 sum 2^(s*log2 e)            */
  int32_t algo_id;          /* 0 = default = 5; 1 = one CTA per (token, output half); 2 = few heads
                               (h <= 32, bf16 form without splits): one CTA per token, scores
                               transposed; 5 = persistent role-split CTA pairs that walk through the
                               tokens (scores in one CTA, values in the other); 6 = paged FP8 form
                               only: dequantise the selected rows, then the persistent kernel    */
  int32_t* status;          /* optional device int32: kernels OR-in a non-zero FTB_ERR_* code */
  /* Paged FP8 form (kv_is_fp8 != 0): physical row = block_table[seq, p / page] * page + p % page,
   * the rule of test_accuracy_musa_vllm_mla.py:278-283.  Query token t belongs to sequence
   * t / q_per_seq.  A logical index >= context_lens[seq] is treated as padding.            */
  int32_t kv_is_fp8;
  const float* kv_scale;        /* fp32 [num_pages]: value = fp8 * scale                     */
  const int32_t* block_table;   /* int32 [n_seq, block_table_stride]                          */
  const int32_t* context_lens;  /* int32 [n_seq]                                              */
  int32_t page_size, q_per_seq;
  int64_t block_table_stride;
  /* Diagnostic tap of the library's own tests, not part of the stable interface: fp32
   * [s_q, 128, topk_padded_to_64] raw (unscaled) scores of the one-CTA kernel.  Pass NULL. */
  float* dbg_scores;
  /* Split of the top-k axis (for few query tokens, e.g. decode): n_splits > 1 makes every split write a
   * partial result to `workspace` (ftb_sparse_mla_workspace_bytes() bytes of device memory, contents
   * need not be initialised) and a merge kernel combine them, the role of _fwd_kernel_stage2
   * (test_accuracy_musa_vllm_mla.py:426-477).  0 or 1 = no split, no workspace. */
  int32_t n_splits;
  void* workspace;
  int64_t workspace_bytes;
} ftb_sparse_mla_args;

FTB_API int ftb_sparse_mla_fwd(const ftb_sparse_mla_args* args, void* stream);
FTB_API int64_t ftb_sparse_mla_workspace_bytes(int32_t s_q, int32_t h, int32_t n_splits);
/* Paged FP8 form, two passes: when `workspace` holds at least this many bytes (16-byte aligned) and
 * n_splits <= 1, the selected rows are first converted to a compact bf16 table (row = token * topk + j,
 * the role of the dequantising loads of decode_attention_int4kv.py:345-450, done once per row instead of
 * inside the attention loop) and the persistent bf16 kernel runs on that table.  algo_id 6 demands this
 * path, algo_id 0 takes it when the workspace allows. */
FTB_API int64_t ftb_sparse_mla_dequant_workspace_bytes(int32_t s_q, int32_t topk);
/* Same operation for callers that cannot allocate device memory (an engine that owns the whole device
 * through its own pool, a sandboxed plugin, a latency path that must stay clear of the allocator).  It has
 * no counterpart in the reference, whose wrappers always receive `attn_logits` from the caller.
 * The split scratch is a fixed array of ftb_sparse_mla_static_scratch_bytes() (32 MiB) inside the library
 * image, resident on every GPU that loads the library until the process exits; `workspace` in `args` is
 * ignored.  A problem whose ftb_sparse_mla_workspace_bytes(s_q, h, n_splits) exceeds that size is
 * rejected with FTB_ERR_INVALID.  No cudaMalloc / cudaFree or other allocating call is made.  The first
 * call on each device looks up the array's device address (cudaGetSymbolAddress): make that call before
 * starting any stream capture.  All calls on a device share the array: two calls that overlap on the GPU
 * (different streams) race on it, and nothing in it needs to be, or is, cleared between calls. */
FTB_API int ftb_sparse_mla_fwd_static_scratch(const ftb_sparse_mla_args* args, void* stream);
FTB_API int64_t ftb_sparse_mla_static_scratch_bytes(void);
/* sizeof(ftb_sparse_mla_args) as compiled into the library (for bindings to check their mirror). */
FTB_API int ftb_sizeof_sparse_mla_args(void);

/* Merge of partial sparse-MLA results over disjoint sets of key/value rows: the reference's second launch,
 *   third_party/mthreads/python/test/wmma/test_accuracy_musa_vllm_mla.py:426-477 (_fwd_kernel_stage2) with its
 *   launcher :480-510, as an operation of its own.  The parts are outputs of ftb_sparse_mla_fwd (bf16, each
 *   normalised by its own sum) or fp32 partials, with their log-sum-exps; typical callers shard a long context
 *   over GPUs (each rank runs the forward on its rows, the parts are gathered, this merges them) or split the
 *   top-k list themselves.  out = sum_k w_k part_k / sum_k w_k with w_k = exp(lse_k - max lse); the merged
 *   log-sum-exp, which the reference does not store, is written too.  A part with lse = -inf (no valid row)
 *   has weight 0; if every part is empty the result is out = 0, lse = -inf. */
typedef struct ftb_sparse_mla_merge_args {
  const void* part_out;      /* bf16 or fp32: part k, token t, head a at k*part_stride_part + t*part_stride_token
                                + a*part_stride_head (elements), 512 contiguous values                        */
  const float* part_lse;     /* fp32: k*lse_stride_part + t*lse_stride_part_token + a                          */
  void* out;                 /* bf16 [s_q, h, 512]                                                             */
  float* lse;                /* fp32 [s_q, h]                                                                  */
  int32_t s_q, h, n_parts;
  int32_t part_is_fp32;      /* 0: part_out is bf16, 1: fp32                                                   */
  int32_t lse_base2;         /* 0: part_lse and lse are natural logs, 1: base 2 (as ftb_sparse_mla_args)       */
  int64_t part_stride_part, part_stride_token, part_stride_head;
  int64_t lse_stride_part, lse_stride_part_token;
  int64_t out_stride_token, out_stride_head, lse_stride_token;
} ftb_sparse_mla_merge_args;
FTB_API int ftb_sparse_mla_merge(const ftb_sparse_mla_merge_args* args, void* stream);
FTB_API int ftb_sizeof_sparse_mla_merge_args(void);

/* ------------------------------------------------------------------------------------------
 * Top-k index producer, the step in front of the sparse MLA forward: for every query token the positions of the
 * `topk` largest scores among its first lengths[t] key positions (all s_kv when lengths is NULL), in ascending
 * position order, padded with -1: the `indices` argument of ftb_sparse_mla_fwd.  Exact and deterministic: floats
 * are ordered by value (-0 below +0, NaN patterns above +inf), ties go to the lower position.  The reference has no
 * such kernel; its nearest relatives are the look-up-table builders of the block-sparse ops,
 *   python/triton/ops/blocksparse/matmul.py:117-127, which also turn a selection into index lists on the device.
 * ------------------------------------------------------------------------------------------ */
typedef struct ftb_topk_args {
  const float* scores;        /* fp32 [s_q, s_kv], scores_stride_token elements between tokens */
  const int32_t* lengths;     /* int32 [s_q] or NULL                                            */
  int32_t* out;               /* int32 [s_q, topk], out_stride_token elements between tokens   */
  int32_t s_q, s_kv, topk;
  int64_t scores_stride_token, out_stride_token;
} ftb_topk_args;
FTB_API int ftb_topk_indices(const ftb_topk_args* args, void* stream);
FTB_API int ftb_sizeof_topk_args(void);

/* ------------------------------------------------------------------------------------------
 * Write path of the paged FP8 latent cache (the producer of the format the paged forward reads):
 * new latent rows are quantised to e4m3 with one fp32 scale per page and scattered into their slots.
 * Analogue of the reference's quantising cache writer
 *   third_party/hcu/python/test/unit/sglang/decode_attention_int4kv.py:934
 *   (destindex_copy_quantize_int4kv_init; its reader is the dequantiser at :821), with e4m3 values and a
 *   per-page scale in place of int4 values and per-group scale / zero point.
 * slot = page * page_size + position in the page; -1 skips the row; slots of one call must be distinct.
 * kv_scale[page] == 0 marks an empty page.  A call raises the scale of each page it touches to
 * max(old, max|new rows| / 448) (at least 1e-12 / 448); where that raises the scale of a page that already
 * held rows, the page's bytes are requantised, e4m3(decode(byte) * old / new), before the new rows are
 * written.  `workspace`: ftb_kv_cache_write_workspace_bytes(num_pages) bytes, contents arbitrary.
 * ------------------------------------------------------------------------------------------ */
typedef struct ftb_kv_cache_write_args {
  const void* rows;              /* bf16 [n_rows, 576], row_stride elements between rows              */
  const int32_t* slot_mapping;   /* int32 [n_rows]                                                    */
  void* kv_cache;                /* e4m3 [num_pages * page_size, 576], contiguous                      */
  float* kv_scale;               /* fp32 [num_pages]                                                  */
  int32_t n_rows, num_pages, page_size;
  int64_t row_stride;
  void* workspace;
  int64_t workspace_bytes;
  int32_t* status;               /* optional: FTB_ERR_BAD_INDEX for a slot past the last page          */
} ftb_kv_cache_write_args;
FTB_API int ftb_kv_cache_write_fp8(const ftb_kv_cache_write_args* args, void* stream);
FTB_API int64_t ftb_kv_cache_write_workspace_bytes(int32_t num_pages);
FTB_API int ftb_sizeof_kv_cache_write_args(void);

/* ------------------------------------------------------------------------------------------
 * Dense GEMM  C[M,N] = A[M,K] . B[K,N]  (bf16 in, fp32 accumulate, bf16 out; row-major).
 *
 * Takes the place of the Triton kernel behind the reference's matmul op,
 *   python/triton/ops/matmul.py:92-151 (_kernel) launched from :218-227, at the `spec("matmul_kernel",
 *   grid, a, b, c, M, N, K, ...)` backend hook of :218: it writes into the caller-allocated `c`.
 * fp32 accumulation for bf16 inputs follows matmul.py:184-190.
 * ------------------------------------------------------------------------------------------ */
typedef struct ftb_gemm_args {
  const void* a;   /* bf16 [m, k], lda */
  const void* b;   /* bf16 [k, n], ldb */
  void* c;         /* bf16 [m, n], ldc */
  int32_t m, n, k;
  int64_t lda, ldb, ldc;
  int32_t* status; /* optional device status word */
} ftb_gemm_args;

FTB_API int ftb_gemm_bf16(const ftb_gemm_args* args, void* stream);
FTB_API int ftb_sizeof_gemm_args(void);

/* ------------------------------------------------------------------------------------------
 * Block-scaled FP8 GEMM: A [m,k] e4m3 with one fp32 scale per 1x128 block (a_scale [m, k/128]),
 * B [k,n] e4m3 with one fp32 scale per 128x128 block (b_scale [k/128, n/128]), bf16 output,
 *   C = sum_kb (A[:,kb] . B[kb,:]) * a_scale[:,kb] (x) b_scale[kb, :/128],  fp32 accumulation per K block.
 * GEMM core: python/triton/ops/matmul.py:92-151 with fp8 operands (:135-136, :204-213) and the fp8
 * descriptor GEMM of third_party/mthreads/python/test/sqmma/base_cases/test_batch_fp8.py:8-25; the
 * block scales have no counterpart in the reference op.  k and n must be multiples of 128.
 * ------------------------------------------------------------------------------------------ */
typedef struct ftb_gemm_fp8_args {
  const void* a;          /* e4m3 [m, k], lda (bytes = elements) */
  const void* b;          /* e4m3 [k, n] row-major with ldb, or, when b_kmajor is set, its transpose [n, k] row-major with
                             ldb (the layout a linear layer keeps its weight in; same speed, same bits) */
  void* c;                /* bf16 [m, n], ldc */
  const float* a_scale;   /* fp32 [m, k/128], row stride a_scale_ld */
  const float* b_scale;   /* fp32 [k/128, n/128], row stride b_scale_ld */
  int32_t m, n, k;
  int64_t lda, ldb, ldc, a_scale_ld, b_scale_ld;
  int32_t* status;
  int32_t b_kmajor;       /* 0: b is [k, n] row-major; 1: b points at the transpose [n, k] row-major */
} ftb_gemm_fp8_args;

FTB_API int ftb_gemm_fp8_blockscaled(const ftb_gemm_fp8_args* args, void* stream);
FTB_API int ftb_sizeof_gemm_fp8_args(void);

/* ------------------------------------------------------------------------------------------
 * Row-parallel GEMM fused with reduce-scatter (tensor parallel size tp, one rank per GPU).
 *
 * Rank r holds A_r [M, K/tp] and B_r [K/tp, N]; C = sum_r A_r.B_r; rank r receives rows
 * [r*M/tp, (r+1)*M/tp) of C as bf16.  The reference has no collective of any kind (no call site of
 * a reduce-scatter exists in it); the GEMM core replaces python/triton/ops/matmul.py:92-151 and the
 * persistent tile loop of python/test/unit/hopper/test_persistent_warp_specialized_gemm.py:38-125,
 * and the cross-rank sum follows the definition "sum over ranks in rank order, fp32, scatter along M".
 *
 * Workspace: every rank provides a receive buffer (recv_bytes) and a flag buffer (flag_bytes), both
 * zero-initialised and mapped into every peer (CUDA IPC, cuMem export, or a symmetric-memory
 * allocator); `recv_ptrs[i]` / `flag_ptrs[i]` are THIS process's device pointers to rank i's buffers
 * (host arrays of tp pointers).  One call may be in flight per context; calls must be issued in the
 * same order on every rank.  Device-side waits are bounded (FTB_ERR_TIMEOUT in the status word).
 * ------------------------------------------------------------------------------------------ */
typedef struct ftb_gemm_rs_ctx ftb_gemm_rs_ctx;
FTB_API int ftb_gemm_rs_workspace_bytes(int m, int n, int tp, int64_t* recv_bytes, int64_t* flag_bytes);
FTB_API int ftb_gemm_rs_ctx_create(ftb_gemm_rs_ctx** ctx, int rank, int tp, int m, int n,
                                   void* const* recv_ptrs, void* const* flag_ptrs);
/* Optional: `mc_recv_ptr` is an NVSwitch multicast mapping of all ranks' receive buffers (same size and
 * layout on every rank).  When set (before the first call, on every rank) the reduce-scatter is done
 * by pull: partial tiles stay in the producing rank's buffer and each owner fetches the cross-rank sum
 * with in-switch reduction (multimem.ld_reduce, fp32 accumulate).  NULL keeps the push protocol. */
FTB_API int ftb_gemm_rs_ctx_set_multicast(ftb_gemm_rs_ctx* ctx, void* mc_recv_ptr);
/* Staged protocol for the bf16 calls of a context (before its first call): the GEMM runs once per group of
 * row shards in rotated order (own group last), the owners learn after each group that this rank's partial
 * of their rows is complete, and one reduce kernel (in-switch reduction or peer loads) finishes the rank's
 * shard.  0 = the fused kernel (default).  The FP8 form always works this way. */
FTB_API int ftb_gemm_rs_ctx_set_staged(ftb_gemm_rs_ctx* ctx, int staged);
/* Copy-engine exchange for the bf16 calls of a context (before its first call; allocates a local partial of
 * 2 * m * n bytes and a second stream): one GEMM launch stores the other ranks' row shards into the local partial
 * in rotated order, the own shard last; as pieces of a shard complete, a second stream copies them into the owner's
 * receive slot with device-to-device copies (carried out by the copy engines, no SM involved) and raises the
 * owner's flags; the epilogue of the own rows waits (bounded) for the peers' flags and adds their partials in fp32,
 * so the result is rounded once and there is no reduce pass.  The call returns on `stream` as usual; the second
 * stream is joined to it.  A context of this protocol serves bf16 calls only. */
FTB_API int ftb_gemm_rs_ctx_set_copy_engine(ftb_gemm_rs_ctx* ctx, int on);
/* Longest time, in SM clock cycles, that a kernel of this context waits for another rank before it gives up,
 * sets FTB_ERR_TIMEOUT in the status word and returns (default about one second).  After a timeout the
 * context is dead: later calls return at once with the status word unchanged; destroy it and create a new one
 * on every rank. */
FTB_API int ftb_gemm_rs_ctx_set_wait_limit(ftb_gemm_rs_ctx* ctx, int64_t cycles);
FTB_API int ftb_gemm_rs_ctx_destroy(ftb_gemm_rs_ctx* ctx);
/* a [m, k_local] bf16, b [k_local, n] bf16, out [m/tp, n] bf16 (this rank's shard). */
FTB_API int ftb_gemm_rs(ftb_gemm_rs_ctx* ctx, const void* a, const void* b, void* out, int k_local,
                        int64_t lda, int64_t ldb, int64_t ldo, int32_t* status, void* stream);

/* CUDA IPC helpers for callers without a symmetric-memory allocator: allocate a zeroed device buffer
 * and export a 64-byte handle; open a peer's handle (enables peer access lazily); close; free. */
/* Block-scaled FP8 form of the same collective: rank r passes A_r [m, k_local] e4m3 with fp32 scales per
 * 1 x 128 block ([m, k_local / 128]) and B_r [k_local, n] e4m3 with fp32 scales per 128 x 128 block, and
 * gets rows [r * m / tp, (r + 1) * m / tp) of sum_r dequant(A_r) . dequant(B_r) as bf16.  The reference has
 * no counterpart (its fp8 matmul, python/triton/ops/matmul.py:162-228, is single-device and unscaled).  A
 * context serves either ftb_gemm_rs or ftb_gemm_rs_fp8 calls, not both; n and k_local are multiples of 128. */
FTB_API int ftb_gemm_rs_fp8(ftb_gemm_rs_ctx* ctx, const void* a, const void* b, const float* a_scale,
                            const float* b_scale, void* out, int k_local, int64_t lda, int64_t ldb,
                            int64_t a_scale_ld, int64_t b_scale_ld, int64_t ldo, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * All-gather + GEMM, the column-parallel sibling that feeds ftb_gemm_rs in a tensor-parallel block: rank r
 * holds the row shard A_r [m / tp, k] bf16 and its weight columns B_r [k, n_local]; every rank gets
 * C_r [m, n_local] = A . B_r with A the shards of all ranks stacked in rank order.  The reference has no
 * collective; the GEMM core replaces python/triton/ops/matmul.py:92-151 as above.  The shards travel on the copy
 * engines while the GEMM already multiplies the rows that have arrived (own rows first).
 * Workspace: every rank provides a gather buffer (ag_bytes) and a flag buffer (flag_bytes), zero-initialised and
 * mapped into every peer; `ag_ptrs[i]` / `flag_ptrs[i]` are this process's pointers to rank i's.  One call in
 * flight per context, same order on every rank; device-side waits are bounded (FTB_ERR_TIMEOUT), the stream
 * waits of the second stream are not.
 * ------------------------------------------------------------------------------------------ */
typedef struct ftb_ag_gemm_ctx ftb_ag_gemm_ctx;
FTB_API int ftb_ag_gemm_workspace_bytes(int m, int k, int tp, int64_t* ag_bytes, int64_t* flag_bytes);
FTB_API int ftb_ag_gemm_ctx_create(ftb_ag_gemm_ctx** ctx, int rank, int tp, int m, int k, void* const* ag_ptrs,
                                   void* const* flag_ptrs);
FTB_API int ftb_ag_gemm_ctx_set_wait_limit(ftb_ag_gemm_ctx* ctx, int64_t cycles);
FTB_API int ftb_ag_gemm_ctx_destroy(ftb_ag_gemm_ctx* ctx);
/* a_shard [m / tp, k] bf16 (lda), b [k, n_local] bf16 (ldb), out [m, n_local] bf16 (ldc). */
FTB_API int ftb_ag_gemm(ftb_ag_gemm_ctx* ctx, const void* a_shard, const void* b, void* out, int n_local, int64_t lda,
                        int64_t ldb, int64_t ldc, int32_t* status, void* stream);

FTB_API int ftb_ipc_alloc(int64_t bytes, void** ptr, uint8_t handle[64]);
FTB_API int ftb_ipc_open(const uint8_t handle[64], void** ptr);
FTB_API int ftb_ipc_close(void* ptr);
FTB_API int ftb_ipc_free(void* ptr);

#ifdef __cplusplus
}
#endif
#endif /* FLAGTREE_B200_H_ */

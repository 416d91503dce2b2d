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
  FTB_ERR_BAD_INDEX = 4,   /* an index outside [0,S_kv) other than the -1 padding was seen    */
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
  int32_t algo_id;          /* 0 = library default                                            */
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
  /* Optional debug tap: fp32 [s_q, 128, topk_padded_to_64] raw (unscaled) scores. NULL = off. */
  float* dbg_scores;
} ftb_sparse_mla_args;

FTB_API int ftb_sparse_mla_fwd(const ftb_sparse_mla_args* args, void* stream);
/* sizeof(ftb_sparse_mla_args) as compiled into the library (for bindings to check their mirror). */
FTB_API int ftb_sizeof_sparse_mla_args(void);

#ifdef __cplusplus
}
#endif
#endif /* FLAGTREE_B200_H_ */

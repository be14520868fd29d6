/*
 * dsv32_b200 -- C ABI of the B200 (sm_100a) implementation of the DeepSeek-V3.2
 * quantized sparse-attention decode path.
 *
 * Every entry point takes a struct of plain device pointers and sizes plus a CUDA
 * stream (cudaStream_t passed as void*).  Calls only enqueue work on that stream and
 * return immediately: 0 = enqueued, negative = rejected on the host (nothing was
 * launched; dsv32_last_error() holds the reason for the calling thread).
 * The caller owns every buffer, including the workspace.  All tensors are contiguous
 * and row-major.  Paths cited below are relative to the reference project root.
 */
#ifndef DSV32_B200_H_
#define DSV32_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSV32_ABI_VERSION 2

/* host-side return codes */
#define DSV32_OK 0
#define DSV32_ERR_INVALID_ARG (-1)
#define DSV32_ERR_WORKSPACE (-2)
#define DSV32_ERR_CUDA (-3)
#define DSV32_ERR_UNSUPPORTED (-4)

/* device status word 0 (args.status, 4 x uint32, caller-zeroed; optional, may be NULL) */
#define DSV32_STATUS_OK 0u
#define DSV32_STATUS_BAD_PAGE 1u    /* a page-table entry on the valid range was < 0 or >= number of blocks */
#define DSV32_STATUS_BAD_INDEX 2u   /* a top-k index pointed outside the request's page table              */
#define DSV32_STATUS_TIMEOUT 3u     /* a bounded device-side wait gave up (word 1 = location id)            */
#define DSV32_STATUS_INTERNAL 4u    /* a kernel found its own launch state inconsistent (word 1 = location id) */

/* ---------------------------------------------------------------------------------------
 * Sparse flash attention over the int8 paged latent cache.
 * Replaces sparse_flash_attention_quant_d / _p / _d_950
 * (models/deepseek_v32_exp/sparse_flash_attention_quant_impl.py:655-674, 734, 572; compute
 * body :45-286).  For token t = b_idx*s1 + i only the first
 * K = min(max(act_seq[b_idx] - s1 + 1 + i, 0), topk) entries of topk_indices[t] are used.
 * The workspace (always required; size from dsv32_sfa_workspace_bytes) holds the resolved cache
 * row of every selected key and, when the keys of a token are split over several CTAs, the
 * fp32 partial outputs.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const void* query_nope;        /* bf16 [b*s1*n_q, 512]                  */
  const void* query_rope;        /* bf16 [b*s1*n_q, 64]                   */
  const void* key_nope;          /* int8 [rows, 512]                      */
  const void* key_rope;          /* bf16 [rows, 64]                       */
  const float* k_nope_scales;    /* fp32 [rows, 4] (one per 128-dim group) */
  const int32_t* topk_indices;   /* int32 [b*s1, topk]                    */
  const int32_t* block_table;    /* int32 [b, max_blocks]                 */
  const int32_t* kv_act_seqs;    /* int32 [b]                             */
  void* attention_out;           /* bf16 [b, s1, n_q, 512]                */
  void* workspace;               /* >= dsv32_sfa_workspace_bytes(...)     */
  size_t workspace_bytes;
  uint32_t* status;              /* device uint32[4] or NULL              */
  int64_t rows;                  /* block_num * block_size                */
  int32_t b, s1, n_q, topk, block_size, max_blocks;
  int32_t kv_splits;             /* 0 = choose automatically              */
  float softmax_scale;
} Dsv32SfaArgs;

size_t dsv32_sfa_workspace_bytes(int32_t b, int32_t s1, int32_t n_q, int32_t topk, int32_t kv_splits);
int dsv32_sfa_quant(const Dsv32SfaArgs* args, void* cuda_stream);
/* The branch of the same operator for a latent cache that is not quantised
 * (sparse_flash_attention_quant_impl.py:216-259): key_nope is bf16 [rows, 512], k_nope_scales is
 * ignored and may be NULL.  n_q must be 128. */
int dsv32_sfa_bf16_cache(const Dsv32SfaArgs* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * The same attention over the fused cache layout ("store 8, compute 16"): one 656-byte row per
 * token = 512 int8 latent dims | 64 bf16 rope dims | 4 fp32 scales (one per 128-dim group).
 * Replaces sparse_attention_antiquant_d / _p / _d_950
 * (models/deepseek_v32_exp/sparse_attention_antiquant_impl.py:287-356, 358-420, 739-768;
 * row layout: deepseekv32_sparse_attention_antiquant.py:262-272).  Workspace and status as for
 * dsv32_sfa_quant (dsv32_sfa_workspace_bytes).
 * ------------------------------------------------------------------------------------- */
#define DSV32_ANTIQUANT_ROW_BYTES 656
typedef struct {
  const void* query_nope;        /* bf16 [b*s1*n_q, 512]                  */
  const void* query_rope;        /* bf16 [b*s1*n_q, 64]                   */
  const void* nope_cache;        /* int8 [rows, 656]                      */
  const int32_t* topk_indices;   /* int32 [b*s1, topk]                    */
  const int32_t* block_table;    /* int32 [b, max_blocks]                 */
  const int32_t* kv_act_seqs;    /* int32 [b]                             */
  void* attention_out;           /* bf16 [b, s1, n_q, 512]                */
  void* workspace;               /* >= dsv32_sfa_workspace_bytes(...)     */
  size_t workspace_bytes;
  uint32_t* status;              /* device uint32[4] or NULL              */
  int64_t rows;                  /* block_num * block_size                */
  int32_t b, s1, n_q, topk, block_size, max_blocks;
  int32_t kv_splits;             /* 0 = choose automatically              */
  float softmax_scale;
} Dsv32SaAntiquantArgs;

int dsv32_sparse_attention_antiquant(const Dsv32SaAntiquantArgs* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * DeepSeek-V4 sparse compress attention: every query token attends to the last win_size
 * positions of its request in the un-compressed bf16 cache (the window) and to the rows
 * of the compressed bf16 cache that cmp_sparse_indices selects; a cache row of 512 dims is
 * key and value at once, and one attention sink per head joins the softmax denominator.
 * Replaces sparse_compress_flash_attention_kernel / npu_sparse_compress_flash_attention
 * (models/deepseek_v4/sparse_compress_flash_attention_impl.py:172-213 / 240-299; compute
 * :47-168).  Token i of a request with s1 = actual_seq_q[r+1] - actual_seq_q[r] tokens:
 *   cur_len  = max(seqused_kv[r] - s1 + 1 + i, 0), window = positions [cur_len - min(cur_len,
 *   win_size), cur_len);  selected = first min(max(seqused_kv[r] / cmp_ratio - s1 + 1 + i, 0),
 *   topk) entries of cmp_sparse_indices[token] (negative entries are skipped).
 * cmp_mode DSV32_SCFA_ALL_COMPRESSED instead takes every compressed position
 *   [0, min(cur_len / cmp_ratio, topk)) and ignores cmp_sparse_indices (may be NULL): the
 *   compress_flash_attention operator (models/deepseek_v4/compress_flash_attention_impl.py:
 *   60-112 cfa_attention, :119-219 c128_decode_impl).  topk == 0 leaves the window alone: the
 *   sliding-window attention operator (models/deepseek_v4/win_attention_impl.py:78-260,263-289);
 *   cmp_kv / cmp_block_table may then be NULL.
 * workspace: dsv32_scfa_workspace_bytes(t, topk, win_size) bytes, 256-byte aligned.
 * ------------------------------------------------------------------------------------- */
#define DSV32_SCFA_SELECTED 0
#define DSV32_SCFA_ALL_COMPRESSED 1
typedef struct {
  const void* query;                  /* bf16 [t*n_q, 512]                         */
  const int32_t* actual_seq_q;        /* int32 [b+1], first token of each request; [b] = t */
  const void* ori_kv;                 /* bf16 [ori_rows, 512]                      */
  const void* cmp_kv;                 /* bf16 [cmp_rows, 512]                      */
  const int32_t* ori_block_table;     /* int32 [b, ori_max_blocks]                 */
  const int32_t* cmp_block_table;     /* int32 [b, cmp_max_blocks]                 */
  const float* atten_sink;            /* fp32 [n_q]                                */
  const int32_t* seqused_kv;          /* int32 [b], un-compressed sequence lengths */
  const int32_t* cmp_sparse_indices;  /* int32 [t, topk]                           */
  void* attention_out;                /* bf16 [t*n_q, 512]                         */
  void* workspace;
  size_t workspace_bytes;
  uint32_t* status;                   /* device uint32[4] or NULL                  */
  int64_t ori_rows, cmp_rows;
  int32_t t, b, n_q, topk, block_size, win_size, cmp_ratio, ori_max_blocks, cmp_max_blocks;
  int32_t cmp_mode;                   /* DSV32_SCFA_SELECTED or DSV32_SCFA_ALL_COMPRESSED */
  float softmax_scale;
} Dsv32ScfaArgs;

int dsv32_sparse_compress_attention(const Dsv32ScfaArgs* args, void* cuda_stream);
size_t dsv32_scfa_workspace_bytes(int32_t t, int32_t topk, int32_t win_size);

/* ---------------------------------------------------------------------------------------
 * Lightning indexer: int8 q.k scores (+ReLU, 2^-11, fp16 round, per-head weighted sum,
 * key scale) and top-k selection.
 * Replaces lightning_indexer_decode
 * (models/deepseek_v32_exp/lightning_indexer_quant_impl.py:226-275; score part :114-177,
 * top-k part :179-216).  topk_res rows hold indices by descending score, equal scores by
 * ascending index, then -1 pads.
 * key_begin/key_end (logical key positions) restrict the scan to a shard of the key
 * range; pass 0 / INT32_MAX for the whole context.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const int8_t* idx_query;        /* int8 [b*s1, 64, 128]                 */
  const void* idx_query_scale;    /* fp16 [b*s1, 64]                      */
  const int8_t* idx_key_cache;    /* int8 [num_blocks, block_size, 1, 128] */
  const void* idx_key_scale;      /* fp16 [num_blocks, block_size, 1]     */
  const void* idx_weight;         /* fp16 [b*s1, 64]                      */
  const int32_t* act_seq_key;     /* int32 [b]                            */
  const int32_t* block_table;     /* int32 [b, max_blocks]                */
  int32_t* topk_res;              /* int32 [b*s1, 1, selected_count] or NULL (scores only) */
  float* topk_scores;             /* fp32 [b*s1, selected_count] or NULL: scores of topk_res (-inf pads) */
  float* scores_out;              /* fp32 [b*s1, score_ld] or NULL: use workspace           */
  int32_t* dots_out;              /* int32 [b*s1, 64, score_ld] or NULL (verification only) */
  void* workspace;
  size_t workspace_bytes;
  uint32_t* status;
  int64_t num_blocks;
  int32_t b, s1, block_size, max_blocks, selected_count;
  int32_t score_ld;               /* row stride of scores_out/dots_out in elements (>= max_blocks*block_size); 0 = that value */
  int32_t key_begin, key_end;
} Dsv32IndexerArgs;

size_t dsv32_indexer_workspace_bytes(int32_t b, int32_t s1, int32_t max_blocks, int32_t block_size);
int dsv32_indexer_topk(const Dsv32IndexerArgs* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * The same operator as one stage of a key-range-sharded indexer over several GPUs of a node
 * (no counterpart in the reference, whose indexer is single-device:
 * lightning_indexer_quant_impl.py:31-32).  One request (b = 1) whose s1 query tokens are
 * owned by ranks in consecutive slices of tokens_per_rank tokens: every rank scores all
 * tokens against its own key range (key_begin / key_end) and the top-k kernel stores a
 * token's row -- indices and scores -- straight into the buffers of the rank that owns the
 * token: idx_ptrs[owner] int32 / score_ptrs[owner] fp32, each
 * [tokens_per_rank, world, selected_count], at [token - owner * tokens_per_rank][rank].
 * The pointers of the other ranks are peer-mapped device addresses (symmetric memory or
 * CUDA IPC); the stores are plain st.global, carried by NVLink.  Nothing is exchanged
 * afterwards: once every rank's call has completed (a barrier across the ranks, stream-
 * ordered after this call), each rank holds world * selected_count candidates per own token
 * and re-selects with dsv32_topk_select (explicit ids).  args.topk_res / topk_scores are
 * ignored.  At most 8 ranks.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int32_t world, rank, tokens_per_rank;
  int32_t reserved;
  void* idx_ptrs[8];     /* int32 [tokens_per_rank, world, selected_count] on rank r */
  void* score_ptrs[8];   /* fp32  [tokens_per_rank, world, selected_count] on rank r */
} Dsv32TopkScatter;

int dsv32_indexer_topk_scatter(const Dsv32IndexerArgs* args, const Dsv32TopkScatter* scatter, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * The same operator for callers that must not allocate device memory (no counterpart in the
 * reference, whose launcher always allocates its workspace through a callback).  The fp32
 * score rows -- the operator's only scratch -- are kept in a fixed array inside the library
 * image, so neither the caller nor the library calls cudaMalloc / cudaFree or any allocating
 * routine; inputs and outputs are still the caller's.  args.workspace and args.scores_out are
 * ignored.
 *   - Limit: b * s1 * max_blocks * block_size <= DSV32_NOALLOC_INDEXER_MAX_SCORES (8 MiB of
 *     scores); larger problems are rejected with DSV32_ERR_WORKSPACE and a message.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call before any
 *     stream capture begins.
 *   - All calls on a device share the one array, which keeps the previous call's contents
 *     (nothing in it needs clearing: every score that is read is written first).  Two calls
 *     that overlap on the GPU (different streams) race on it -- serialise them.
 * ------------------------------------------------------------------------------------- */
#define DSV32_NOALLOC_INDEXER_MAX_SCORES 2097152ull
int dsv32_indexer_topk_noalloc(const Dsv32IndexerArgs* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * Row-wise top-k over fp32 scores (the selection stage alone).
 * Semantics of pypto.topk as used at lightning_indexer_quant_impl.py:179-216; tie rule of
 * framework/src/interface/interpreter/calculator/calc_torch.cpp:2481-2495.
 * ids == NULL: entry j of a row has id j + id_base.  With ids (candidate merge), ties are
 * broken by ascending id and entries with id < 0 are ignored.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const float* scores;            /* fp32 [rows, ld]                      */
  const int32_t* ids;             /* int32 [rows, ld] or NULL             */
  const int32_t* counts;          /* int32 [rows]: valid entries per row  */
  int32_t* out_idx;               /* int32 [rows, k]                      */
  float* out_scores;              /* fp32 [rows, k] or NULL               */
  int32_t rows, ld, k, id_base;
} Dsv32TopkArgs;

int dsv32_topk_select(const Dsv32TopkArgs* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * Indexer prolog (quant): W8A8 q projection, k projection + LayerNorm, RoPE, 128x128
 * "Hadamard" matmul, per-row int8 quantisation, cache scatter, head weights.
 * Replaces lightning_indexer_prolog_quant
 * (models/deepseek_v32_exp/lightning_indexer_prolog_quant_impl.py:325-543).
 * Weights are plain row-major [K, N] (the reference passes an NZ-formatted view of the
 * same logical matrices).  k_cache / k_scale_cache are updated in place at rows
 * k_cache_index[t]; no other row is touched.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const void* x;                  /* bf16 [t, 7168]                       */
  const int8_t* q_norm;           /* int8 [t, 1536]                       */
  const float* q_norm_scale;      /* fp32 [t, 1]                          */
  const int8_t* w_qb;             /* int8 [1536, 8192]                    */
  const float* w_qb_scale;        /* fp32 [8192, 1]                       */
  const void* wk;                 /* bf16 [7168, 128]                     */
  const void* w_proj;             /* bf16 [7168, 64]                      */
  const void* ln_gamma_k;         /* bf16 [128]                           */
  const void* ln_beta_k;          /* bf16 [128]                           */
  const void* cos_idx_rope;       /* bf16 [t, 64]                         */
  const void* sin_idx_rope;       /* bf16 [t, 64]                         */
  const void* hadamard_q;         /* bf16 [128, 128]                      */
  const void* hadamard_k;         /* bf16 [128, 128]                      */
  const int64_t* k_cache_index;   /* int64 [t]                            */
  int8_t* q_int8;                 /* out int8 [t, 64, 128]                */
  void* q_scale;                  /* out fp16 [t, 64, 1]                  */
  int8_t* k_cache;                /* in/out int8 [cache_rows, 128]        */
  void* k_scale_cache;            /* in/out fp16 [cache_rows]             */
  void* weights;                  /* out fp16 [t, 64]                     */
  void* workspace;
  size_t workspace_bytes;
  uint32_t* status;
  int64_t cache_rows;
  int32_t t;
  float ln_eps;
} Dsv32PrologArgs;

size_t dsv32_prolog_workspace_bytes(int32_t t);
int dsv32_indexer_prolog(const Dsv32PrologArgs* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * DeepSeek-V4 indexer prolog (quant): query path and head weights, no key path.
 * Replaces quant_lightning_indexer_prolog_kernel / npu_quant_lightning_indexer_prolog
 * (models/deepseek_v4/lightning_indexer_prolog_quant_v4_impl.py:118-266 / 78-115):
 *   q = int8 quant per (token, head) of  bf16( [nope | irope(rope)] . hadamard ),
 *       [nope | rope] = bf16( int32(qr . idx_wq_b) * qr_scale * idx_wq_b_scale ) per head (64 + 64 dims),
 *       irope = interleaved inverse rotary embedding on the last 64 dims;
 *   weights = fp16( float(bf16(x . weights_proj)) * 64^-0.5 * 128^-0.5 ).
 * Fixed sizes: q_lora_rank 1024, 64 heads of 128 dims, rope 64; h (hidden size) is free.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const int8_t* qr;               /* int8 [t, 1024]                       */
  const int8_t* idx_wq_b;         /* int8 [1024, 8192], row-major         */
  const void* x;                  /* bf16 [t, h]                          */
  const void* weights_proj;       /* bf16 [h, 64], row-major              */
  const void* cos;                /* bf16 [t, 64]                         */
  const void* sin;                /* bf16 [t, 64]                         */
  const void* hadamard;           /* bf16 [128, 128]                      */
  const float* qr_scale;          /* fp32 [t, 1]                          */
  const float* idx_wq_b_scale;    /* fp32 [8192, 1]                       */
  int8_t* q;                      /* out int8 [t, 64, 128]                */
  void* weights;                  /* out fp16 [t, 64]                     */
  void* q_scale;                  /* out fp16 [t, 64]                     */
  void* workspace;                /* >= dsv32_prolog_v4_workspace_bytes(t, h), 16-byte aligned */
  size_t workspace_bytes;
  uint32_t* status;
  int32_t t, h;
} Dsv32PrologV4Args;

int dsv32_indexer_prolog_v4(const Dsv32PrologV4Args* args, void* cuda_stream);
size_t dsv32_prolog_v4_workspace_bytes(int32_t t, int32_t h);

/* ---------------------------------------------------------------------------------------
 * Page-grouped lightning-indexer prolog with 8-bit float formats.  Replaces
 * lightning_indexer_prolog_quant of python/tests/st/operator/pg/lightning_indexer_prolog_quant_mxfp8_impl.py:230-401
 * (format DSV32_PG_FORMAT_MXFP8: float8 E4M3 codes, one E8M0 scale per 32 reduction elements of q_norm and of
 * w_qb) and of lightning_indexer_prolog_quant_hif8_impl.py:230-406 (format DSV32_PG_FORMAT_HIF8: HiF8 codes, one
 * fp32 scale per token and per output column):
 *   q       = quant( bf16( rope_first64( bf16(q_norm . w_qb, scales applied) ) . hadamard_q ) ) per (token, head)
 *   k       = quant( bf16( rope_first64( bf16( rmsnorm( bf16(x . wk) ) * gamma_k ) ) . hadamard_k ) ) per token,
 *             scattered with its scale into the caches at rows k_cache_index / k_scale_cache_index
 *   weights = bf16( bf16( bf16(x . w_proj) * heads^-0.5 ) * 128^-0.5 )
 *   quant(v) = 8-bit codes of v / scale with scale = amax(|v|) * fl(1 / max_code), max_code 448 (E4M3,
 *   saturating) or 32768 (HiF8: nearest value, ties away from zero, saturating)
 * The caches are page-grouped: row r lives in page r / block_size at slot r % block_size, pages
 * k_block_stride (bytes) apart -- a strided view into a buffer that other caches share.  head_dim is 128,
 * the rotary part the first 64 dims; q_lora is a multiple of 256, h of 512, heads <= 128.
 * ------------------------------------------------------------------------------------- */
#define DSV32_PG_FORMAT_MXFP8 0
#define DSV32_PG_FORMAT_HIF8 1
typedef struct {
  const void* x;                    /* bf16 [t, h]                                                  */
  const uint8_t* q_norm;            /* codes [t, q_lora]                                            */
  const void* q_norm_scale;         /* MXFP8: E8M0 [t, q_lora / 32]; HiF8: fp32 [t]                 */
  const uint8_t* w_qb;              /* codes [q_lora, heads * 128]                                  */
  const void* w_qb_scale;           /* MXFP8: E8M0 [q_lora / 64, heads * 128, 2]; HiF8: fp32 [heads * 128] */
  const void* wk;                   /* bf16 [h, 128]                                                */
  const void* w_proj;               /* bf16 [h, heads]                                              */
  const void* gamma_k;              /* bf16 [128]                                                   */
  const void* cos_idx_rope;         /* bf16 [t, 64]                                                 */
  const void* sin_idx_rope;         /* bf16 [t, 64]                                                 */
  const void* hadamard_q;           /* bf16 [128, 128]                                              */
  const void* hadamard_k;           /* bf16 [128, 128]                                              */
  const int64_t* k_cache_index;     /* int64 [t]                                                    */
  const int64_t* k_scale_cache_index; /* int64 [t]                                                  */
  uint8_t* q_quant;                 /* out codes [t, heads, 128]                                    */
  float* q_scale;                   /* out fp32 [t, heads]                                          */
  uint8_t* k_cache;                 /* in/out codes, page-grouped (see above)                       */
  float* k_scale_cache;             /* in/out fp32, page-grouped                                    */
  void* weights;                    /* out bf16 [t, heads]                                          */
  void* workspace;                  /* >= dsv32_pg_indexer_prolog_workspace_bytes(...), 256-byte aligned */
  size_t workspace_bytes;
  uint32_t* status;
  int64_t cache_rows;               /* pages * block_size                                           */
  int64_t k_block_stride;           /* bytes between pages of k_cache (>= block_size * 128)         */
  int64_t k_scale_block_stride;     /* bytes between pages of k_scale_cache (>= block_size * 4)     */
  int32_t t, h, q_lora, heads, block_size, format;
  float eps;                        /* RMSNorm epsilon (the operator uses 1e-6)                     */
} Dsv32PgPrologArgs;

int dsv32_pg_indexer_prolog(const Dsv32PgPrologArgs* args, void* cuda_stream);
size_t dsv32_pg_indexer_prolog_workspace_bytes(int32_t t, int32_t h, int32_t q_lora, int32_t heads);

/* ---------------------------------------------------------------------------------------
 * Matrix products on this library's tcgen05 kernel, for the projections of the DeepSeek-V4 operators
 * whose host code lives in Python (models/deepseek_v4/mla_prolog_quant_v4_impl.py:438-520, mla_prolog_v4_impl.py,
 * compressor_impl.py:421-923: their `pypto.matmul` calls).
 *   dsv32_gemm_bf16: C[t, n] = A[t, k] x B, bf16 operands, fp32 accumulation; B is [k, n] row-major
 *     (b_layout 0) or [n, k] row-major (b_layout 1: a weight held one row per output column); C is fp32
 *     (c_dtype 0) or bf16 (c_dtype 1, one rounding of the fp32 sum).  k a multiple of 64, n of 8.
 *   dsv32_gemm_i8: int32 C[t, n] = int8 A[t, k] x int8 B[k, n]; k a multiple of 128, n of 256.
 * All pointers 16-byte aligned.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const void* a;                    /* bf16 [t, k]                                  */
  const void* b;                    /* bf16 [k, n] or [n, k] (b_layout)             */
  void* c;                          /* out fp32 or bf16 [t, n] (c_dtype)            */
  void* workspace;                  /* >= dsv32_gemm_bf16_workspace_bytes(t, k, n), 256-byte aligned */
  size_t workspace_bytes;
  uint32_t* status;
  int32_t t, k, n, b_layout, c_dtype;
} Dsv32GemmBf16Args;
int dsv32_gemm_bf16(const Dsv32GemmBf16Args* args, void* cuda_stream);
size_t dsv32_gemm_bf16_workspace_bytes(int32_t t, int32_t k, int32_t n);

typedef struct {
  const int8_t* a;                  /* int8 [t, k]                                  */
  const int8_t* b;                  /* int8 [k, n]                                  */
  int32_t* c;                       /* out int32 [t, n]                             */
  uint32_t* status;
  int32_t t, k, n;
} Dsv32GemmI8Args;
int dsv32_gemm_i8(const Dsv32GemmI8Args* args, void* cuda_stream);

/* Array conversions of the HiF8 format (device pointers; n elements):
 * direction 0: fp32 -> codes (nearest value, ties away from zero, saturating at 2^15), 1: codes -> fp32. */
int dsv32_hif8_convert(int32_t direction, const void* in, void* out, int64_t n, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * MLA prolog (quant).  Replaces mla_prolog_quant_d / _p
 * (models/deepseek_v32_exp/mla_prolog_quant_impl.py:848-875 / 751-778) and is the MLA half of
 * the fused entry below:
 *   q_a  = bf16(x . w_dq) -> RMSNorm(gamma_cq) -> bf16 -> per-token int8 -> q_norm, q_norm_scale
 *   q_b  = bf16(int32(q_norm . w_uq_qr) * q_norm_scale * w_qb_scale), per head 128 nope + 64 rope dims
 *   query_nope = bf16(q_b nope . w_uk[head]);  query_rope = de-interleave + rotate-half RoPE of q_b rope
 *   kv_a = bf16(x . w_dkv_kr): first 512 -> RMSNorm(gamma_ckv) -> four 128-dim int8 groups + fp32
 *          scales -> kv_cache / k_scale_cache at rows cache_index; last 64 -> RoPE -> kr_cache
 * All four projections run in this library's tensor-core kernels; weights are plain row-major
 * [K, N] (the reference passes NZ-formatted views of the same logical matrices).  Caches are
 * updated in place; no other row is touched.  One call enqueues everything on cuda_stream.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const void* x;                  /* bf16 [t, 7168]                                   */
  const void* w_dq;               /* bf16 [7168, 1536]                                */
  const int8_t* w_uq_qr;          /* int8 [1536, 24576]                               */
  const float* w_qb_scale;        /* fp32 [24576]                                     */
  const void* w_uk;               /* bf16 [128, 128, 512]                             */
  const void* w_dkv_kr;           /* bf16 [7168, 576]                                 */
  const void* gamma_cq;           /* bf16 [1536]                                      */
  const void* gamma_ckv;          /* bf16 [512]                                       */
  const void* cos;                /* bf16 [t, 64]                                     */
  const void* sin;                /* bf16 [t, 64]                                     */
  const int64_t* cache_index;     /* int64 [t]                                        */
  int8_t* kv_cache;               /* in/out int8 [cache_rows, 512]                    */
  void* kr_cache;                 /* in/out bf16 [cache_rows, 64]                     */
  float* k_scale_cache;           /* in/out fp32 [cache_rows, 4]                      */
  int8_t* q_norm;                 /* out int8 [t, 1536]                               */
  float* q_norm_scale;            /* out fp32 [t]                                     */
  void* query_nope;               /* out bf16 [t, 128, 512]                           */
  void* query_rope;               /* out bf16 [t, 128, 64]                            */
  void* workspace;                /* >= dsv32_mla_prolog_workspace_bytes(t), 256-byte aligned */
  size_t workspace_bytes;
  uint32_t* status;
  int64_t cache_rows;
  int32_t t;
  float eps_cq, eps_ckv;
} Dsv32MlaPrologArgs;

int dsv32_mla_prolog(const Dsv32MlaPrologArgs* args, void* cuda_stream);
size_t dsv32_mla_prolog_workspace_bytes(int32_t t);

/* ---------------------------------------------------------------------------------------
 * Fused MLA prolog + indexer prolog (quant).  Replaces mla_indexer_prolog_quant_d / _p
 * (models/deepseek_v32_exp/mla_indexer_prolog_quant_impl.py:486-528 / 327-369): the MLA half
 * above, whose int8 q_norm / q_norm_scale feed the indexer half (dsv32_indexer_prolog) on the
 * device, as in the reference (:112-211, 213-317).  `indexer.x`, `indexer.q_norm` and
 * `indexer.q_norm_scale` must be the pointers of the MLA half.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  Dsv32MlaPrologArgs mla;
  Dsv32PrologArgs indexer;
} Dsv32FusedPrologArgs;

int dsv32_mla_indexer_prolog(const Dsv32FusedPrologArgs* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * Diagnostic with no counterpart in the reference: launches one tiny CTA that waits, for at
 * most budget_cycles SM clock cycles, on a barrier nothing ever arrives at (no copy or tensor-
 * core operation is in flight), so that the give-up path of the kernels' bounded waits can be
 * observed -- status[0] = DSV32_STATUS_TIMEOUT, status[1] = 99 -- without stalling a real
 * kernel.  The kernels themselves wait for about a second (2e9 cycles) before giving up.
 * ------------------------------------------------------------------------------------- */
int dsv32_wait_selftest(uint32_t* status, int64_t budget_cycles, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * Next decode step of a batch, on the device: act_seq[b] += grow, then the cache rows of the
 * step's s1 tokens by the reference's rule for its test data
 * (models/deepseek_v32_exp/deepseekv32_mla_indexer_prolog_quant.py:184-194):
 *   pos = act_seq[b] - s1 + j,  cache_index[b, j] = block_table[b, pos / block_size] * block_size + pos % block_size.
 * A position beyond the page table or on an unassigned page (-1) sets the status word and
 * yields cache_index -1, which the prologs report and skip.  The reference computes this on the
 * host for every call; a captured multi-step decode loop needs it on the stream.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int32_t* act_seq;               /* in/out int32 [b]: length including the current step's tokens */
  const int32_t* block_table;     /* int32 [b, max_blocks]                                        */
  int64_t* cache_index;           /* out int64 [b, s1]                                            */
  uint32_t* status;
  int32_t b, s1;
  int32_t grow;                   /* tokens every request appends in the step being prepared (usually s1) */
  int32_t block_size, max_blocks;
} Dsv32AdvanceArgs;

int dsv32_decode_advance(const Dsv32AdvanceArgs* args, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * Fused element-wise stages of the DeepSeek-V4 MLA prolog (quant), between its three
 * projections (dsv32_gemm_bf16 / dsv32_gemm_i8).  Replaces the vector work of mla_prolog_v4 / mla_prolog_v4_in
 * (models/deepseek_v4/mla_prolog_quant_v4_impl.py:406-517 / 567-629):
 *   stage 0: q_a = x.wq_a (fp32) -> RMSNorm * gamma_cq -> per-token int8 quant -> qr, qr_scale
 *   stage 1: q_b = qr.wq_b (int32) -> * qr_scale * wq_b_scale -> per-head RMSNorm (no weight)
 *            -> bf16 -> interleaved rotary embedding on the last 64 of 512 dims -> q
 *   stage 2: kv_a = x.wkv (fp32) -> RMSNorm * gamma_ckv -> bf16 -> rotary on the last 64 -> kv
 * Fixed sizes: q_lora_rank 1024, head_dim 512, rope 64; the head count is free.
 * quant == 0 selects the operator without quantisation (models/deepseek_v4/mla_prolog_v4_impl.py:
 * 310-390, 415-455): the GEMM results q_a / q_b / kv_a are bf16, qr is written as bf16 and
 * qr_scale / wq_b_scale are not used.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const void* q_a;                /* stage 0: fp32 (quant == 0: bf16) [t, 1024]      */
  const void* gamma_cq;           /* bf16 [1024]                                     */
  void* qr;                       /* stage 0 out: int8 (bf16) [t, 1024]              */
  float* qr_scale;                /* stage 0 out / stage 1 in: fp32 [t]              */
  const void* q_b;                /* stage 1: int32 (bf16) [t, q_b_ld], first heads*512 columns */
  const float* wq_b_scale;        /* fp32 [heads*512]                                */
  void* q_out;                    /* stage 1 out: bf16 [t, heads, 512]               */
  const void* kv_a;               /* stage 2: fp32 (bf16) [t, 512]                   */
  const void* gamma_ckv;          /* bf16 [512]                                      */
  void* kv_out;                   /* stage 2 out: bf16 [t, 512]                      */
  const void* cos;                /* bf16 [t, 64]                                    */
  const void* sin;                /* bf16 [t, 64]                                    */
  int32_t t, heads, q_b_ld;
  int32_t quant;                  /* 1: quantised operator, 0: bf16 operator         */
  float eps;
} Dsv32MlaV4StageArgs;

int dsv32_mla_prolog_v4_stage(const Dsv32MlaV4StageArgs* args, int32_t stage, void* cuda_stream);

/* ---------------------------------------------------------------------------------------
 * DeepSeek-V4 hyper-connection pre-mix.  Replaces hc_pre_kernel / hc_pre_kernel_prefill /
 * npu_hc_pre (models/deepseek_v4/hc_pre_impl.py:100-206 / 216-309 / 371-392):
 *   mix = (x as [t, 16384]) . hc_fn^T / sqrt(mean(x^2) + norm_eps)                  [t, 24]
 *   pre = sigmoid(mix[0:4] * hc_scale[0] + hc_base[0:4]) + hc_eps
 *   post = 2 * sigmoid(mix[4:8] * hc_scale[1] + hc_base[4:8])
 *   comb = Sinkhorn(mix[8:24] * hc_scale[2] + hc_base[8:24], iters, hc_eps)        [t, 4, 4]
 *   y = bf16(sum_h pre[h] * x[:, h, :])                                            [t, 4096]
 * Fixed sizes: 4 streams of 4096.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const void* x;                  /* bf16 [t, 4, 4096]                    */
  const float* hc_fn;             /* fp32 [24, 16384]                     */
  const float* hc_scale;          /* fp32 [3]                             */
  const float* hc_base;           /* fp32 [24]                            */
  void* y;                        /* out bf16 [t, 4096]                   */
  float* post;                    /* out fp32 [t, 4]                      */
  float* comb;                    /* out fp32 [t, 4, 4]                   */
  void* workspace;                /* >= dsv32_hc_pre_workspace_bytes(t), 16-byte aligned */
  size_t workspace_bytes;
  int32_t t, hc_mult, d, iters;   /* hc_mult must be 4, d 4096, iters >= 1 */
  float norm_eps, hc_eps;
} Dsv32HcPreArgs;

int dsv32_hc_pre(const Dsv32HcPreArgs* args, void* cuda_stream);
size_t dsv32_hc_pre_workspace_bytes(int32_t t);

/* ---------------------------------------------------------------------------------------
 * DeepSeek-V4 KV compressor: state update + compression, between the operator's GEMMs.
 * Replaces the vector work of compressor_ratio_4_kernel / compressor_ratio_4_rotate_kernel /
 * compressor_ratio_128_kernel (models/deepseek_v4/compressor_impl.py:421-923; entry
 * npu_compressor :139-226).  For token i of request r at position pos = start_pos[r] + i:
 * the rows kv_total / score_total (+ ape[pos % ratio]) are stored into the paged states at
 * pos; when (pos + 1) % ratio == 0 the window ending at pos is compressed (softmax over its
 * score rows per column, weighted sum of its kv rows; ratio 4 uses the first halves of the
 * previous window and the second halves of this one), RMS-normalised with `weight`, rotated
 * (interleaved rotary on the last 64 dims, row r of sin / cos) and written to out[r].
 * Rows of `out` of requests that did not compress are left untouched.
 * coff = 2 with ratio 4 (overlapping windows), 1 with ratio 128; d <= 512.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const float* kv_total;          /* fp32 [b*s1, coff*d]                  */
  const float* score_total;       /* fp32 [b*s1, coff*d]                  */
  const float* ape;               /* fp32 [ratio, coff*d]                 */
  const float* weight;            /* fp32 [d]                             */
  float* kv_state;                /* in/out fp32 [kv_blocks, 128, coff*d] */
  float* score_state;             /* in/out fp32 [score_blocks, 128, coff*d] */
  const int32_t* kv_block_table;  /* int32 [b, kv_cols]                   */
  const int32_t* score_block_table; /* int32 [b, score_cols]              */
  const void* sin;                /* bf16 [>= b, 64]                      */
  const void* cos;                /* bf16 [>= b, 64]                      */
  const int32_t* start_pos;       /* int32 [b]                            */
  void* out;                      /* out bf16 [>= b, d]                   */
  uint32_t* status;
  int64_t kv_blocks, score_blocks;
  int32_t b, s1, d, ratio, kv_cols, score_cols;
  float eps;
} Dsv32CompressorArgs;

int dsv32_compressor_update(const Dsv32CompressorArgs* args, void* cuda_stream);

/* library-wide */
int dsv32_abi_version(void);
const char* dsv32_last_error(void);
/* Number of kernel launches enqueued by this library in this process (for launch accounting). */
uint64_t dsv32_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* DSV32_B200_H_ */

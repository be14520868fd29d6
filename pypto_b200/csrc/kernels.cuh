// Kernel-side parameter blocks and launchers shared by api.cu and the kernel translation units.
#pragma once
#include "common.cuh"

namespace dsv32 {

struct TopkParams {
  const float* scores;
  const int32_t* ids;
  const int32_t* counts;
  const int32_t* act_seq;
  int32_t* out_idx;
  float* out_scores;
  int s1, key_begin, key_end;
  int ld, k, id_base;
  // Key-range-sharded indexer of one long request (scatter_world > 0): row = query token; the row's results do not go
  // to out_idx / out_scores but into the buffers of the rank that owns the token (tokens_per_rank consecutive tokens
  // each), at [token - first token of the owner][this rank][k] -- plain stores, over NVLink for the other ranks.
  int scatter_world, scatter_rank, scatter_per;
  int32_t* scatter_idx[8];
  float* scatter_sc[8];
};
int launch_topk(const TopkParams& p, int rows, cudaStream_t stream);

struct IndexerParams {
  const int8_t* q;
  const __half* q_scale;
  const __half* weight;
  const int8_t* keys;
  const __half* key_scale;
  const int32_t* act_seq;
  const int32_t* block_table;
  float* scores;
  int32_t* dots;
  uint32_t* status;
  long long num_blocks;
  int b, s1, block_size, max_blocks, ld;
  int key_begin, key_end;
  int blocks_per_cta;  // key blocks one CTA of the tcgen05 kernel walks (chosen by its launcher)
};
int launch_indexer_scores_tc(const IndexerParams& p, cudaStream_t stream);

struct SfaParams {
  const __nv_bfloat16* q_nope;
  const __nv_bfloat16* q_rope;
  const int8_t* k_nope;
  const __nv_bfloat16* k_rope;
  const float* k_scales;
  const int32_t* topk_idx;
  const int32_t* block_table;
  const int32_t* act_seq;
  __nv_bfloat16* out;
  float* part_o;
  float* part_lse;
  int32_t* row_ids;  // [t, topk] cache row + 1 of every selected key, 0 = none (scratch, tcgen05 kernel only)
  uint32_t* status;
  long long rows;
  int b, s1, nq, topk, block_size, max_blocks, splits;
  int bs_shift;  // log2(block_size) when it is a power of two, else -1
  // byte distance between consecutive cache rows in each of the three arrays: 512 / 128 / 16 for separate
  // arrays, 656 / 656 / 656 when the three parts of a row sit side by side in one array
  int nope_stride, rope_stride, scale_stride;
  int kn_bf16;  // 1: the latent cache is bf16 [rows, 512] and there are no scales (tcgen05 kernel only)
  float scale;
  // DeepSeek-V4 sparse compress attention only (compress != 0; tcgen05 kernel, bf16 rows of 512 dims that serve
  // as key and value, no rope part).  A token's key list is its window rows of k_nope (paged by block_table)
  // followed by the rows of k_nope2 that sel_idx selects (paged by block_table2); `topk` is then the length of
  // that list (win_size + sel_topk) and act_seq holds the un-compressed sequence lengths.
  int compress;
  const __nv_bfloat16* k_nope2;
  const int32_t* block_table2;
  const int32_t* seq_q;     // [b + 1] first token of every request, seq_q[b] = number of tokens
  const float* sinks;       // [nq] attention sinks
  int32_t* key_counts;      // [t] scratch: keys in each token's list
  long long rows2;
  int max_blocks2, win_size, sel_topk, cmp_ratio, t_total;
  int pair;       // tokens 2k, 2k+1 of a request share a CTA (<= 64 heads): 1 = key lists without an index tensor,
                  // 2 = selected compressed keys (the union of both selections is built by scfa_pair_ids_kernel)
  int cmp_dense;  // 1: every compressed position [0, cur_len / cmp_ratio) instead of the rows topk_idx selects
};
int launch_sfa_tc(const SfaParams& p, cudaStream_t stream);
int launch_sfa_combine(const SfaParams& p, cudaStream_t stream);

struct PrologParams {
  const __nv_bfloat16* x;
  const int8_t* q_norm;
  const float* q_norm_scale;
  const int8_t* w_qb;
  const float* w_qb_scale;
  const __nv_bfloat16* wk;
  const __nv_bfloat16* w_proj;
  const __nv_bfloat16* ln_gamma;
  const __nv_bfloat16* ln_beta;
  const __nv_bfloat16* cos;
  const __nv_bfloat16* sin;
  const __nv_bfloat16* had_q;
  const __nv_bfloat16* had_k;
  const long long* cache_index;
  int8_t* q_int8;
  __half* q_scale;
  int8_t* k_cache;
  __half* k_scale_cache;
  __half* weights;
  float* partial;
  uint32_t* status;
  long long cache_rows;
  int t;
  float eps;
};
constexpr int kPrologKSplits = 16;  // CTAs that share the 7168-long reduction of x . [wk | w_proj]
int launch_prolog_tc(const PrologParams& p, cudaStream_t stream);
int launch_prolog_v4(const PrologParams& p, int h, float w_scale, cudaStream_t stream);
size_t prolog_v4_workspace_bytes(int t, int h);
size_t prolog_workspace_bytes(int t);


// MLA prolog (quant): x . [w_dq | w_dkv_kr] has 1536 + 576 = 2112 output columns and its reduction over the hidden
// size (112 chunks of 64) is split over kMlaXSplits CTAs, whose fp32 partial sums the two finish kernels add in a fixed order.
constexpr int kMlaXSplits = 8;
constexpr int kMlaXCols = 2176;   // 2112 rounded up to whole column tiles of 128 (the last 64 are padding)

struct MlaStageParams {
  const float* partial;        // [kMlaXSplits][t][kMlaXCols] partial sums of x . [w_dq | w_dkv_kr]
  const __nv_bfloat16* gamma_cq;
  int8_t* q_norm;
  float* q_norm_scale;
  const __nv_bfloat16* gamma_ckv;
  const __nv_bfloat16* cos;
  const __nv_bfloat16* sin;
  const long long* cache_index;
  int8_t* kv_cache;
  __nv_bfloat16* kr_cache;
  float* k_scale_cache;
  uint32_t* status;
  long long cache_rows;
  int t;
  float eps_cq, eps_ckv;
};
int launch_mla_finish(const MlaStageParams& p, cudaStream_t stream);

struct MlaParams {
  const __nv_bfloat16* x;          // [t, 7168]
  const __nv_bfloat16* w_dq;       // [7168, 1536]
  const int8_t* w_uq_qr;           // [1536, 128 * 192]
  const float* w_qb_scale;         // [128 * 192]
  const __nv_bfloat16* w_uk;       // [128, 128, 512]
  const __nv_bfloat16* w_dkv_kr;   // [7168, 576]
  const __nv_bfloat16* gamma_cq;
  const __nv_bfloat16* gamma_ckv;
  const __nv_bfloat16* cos;        // [t, 64]
  const __nv_bfloat16* sin;
  const long long* cache_index;    // [t]
  int8_t* kv_cache;                // [cache_rows, 512]
  __nv_bfloat16* kr_cache;         // [cache_rows, 64]
  float* k_scale_cache;            // [cache_rows, 4]
  int8_t* q_norm;                  // out [t, 1536]
  float* q_norm_scale;             // out [t]
  __nv_bfloat16* q_nope;           // out [t, 128, 512]
  __nv_bfloat16* q_rope;           // out [t, 128, 64]
  void* workspace;                 // mla_prolog_workspace_bytes(t), 256-byte aligned
  uint32_t* status;
  long long cache_rows;
  int t;
  float eps_cq, eps_ckv;
};
int launch_mla_prolog(const MlaParams& p, cudaStream_t stream);
// bf16 tcgen05 GEMM as a building block (mla_prolog_tc.cu): fp32 partial sums, one [t, ldc] slab per reduction split
int launch_bf16_gemm_partial(const __nv_bfloat16* a, int t, int k, const __nv_bfloat16* b, int b_cols, int n_tiles,
                             int splits, float* partial, int ldc, uint32_t* status, cudaStream_t stream,
                             bool b_kmajor = false);
// C[t, n] (fp32 or bf16) = A[t, k] x B (bf16; B as [k, n], or with b_kmajor as [n, k]) through partial sums in `workspace`
int launch_bf16_gemm(const __nv_bfloat16* a, int t, int k, const __nv_bfloat16* b, int n, bool b_kmajor, void* out,
                     bool out_bf16, void* workspace, uint32_t* status, cudaStream_t stream);
size_t bf16_gemm_workspace_bytes(int t, int k, int n);
int launch_i8_gemm(const int8_t* a, int t, int k, const int8_t* b, int n, int32_t* c, uint32_t* status, cudaStream_t stream);
size_t mla_prolog_workspace_bytes(int t);

// Page-grouped indexer prolog with 8-bit float formats (pg_prolog.cu)
struct PgPrologParams {
  const __nv_bfloat16* x;              // [t, h]
  const uint8_t* q_norm;               // [t, q_lora] codes
  const uint8_t* q_norm_scale_e8;      // MXFP8: E8M0 [t, q_lora / 32]
  const float* q_norm_scale_f32;       // HiF8: [t]
  const uint8_t* w_qb;                 // [q_lora, n] codes
  const uint8_t* w_qb_scale_e8;        // MXFP8: E8M0 [q_lora / 64, n, 2]
  const float* w_qb_scale_f32;         // HiF8: [n]
  const __nv_bfloat16* wk;             // [h, 128]
  const __nv_bfloat16* w_proj;         // [h, heads]
  const __nv_bfloat16* gamma_k;        // [128]
  const __nv_bfloat16* cos;            // [t, 64]
  const __nv_bfloat16* sin;
  const __nv_bfloat16* hadamard_q;     // [128, 128]
  const __nv_bfloat16* hadamard_k;
  const long long* k_cache_index;      // [t]
  const long long* k_scale_cache_index;
  uint8_t* q_out;                      // [t, heads, 128] codes
  float* q_scale_out;                  // [t, heads]
  uint8_t* k_cache;                    // page p, slot s, dim d at p * k_block_stride + s * 128 + d
  float* k_scale_cache;                // page p, slot s at byte p * k_scale_block_stride + 4 s
  __nv_bfloat16* weights_out;          // [t, heads]
  uint32_t* status;
  long long cache_rows, k_block_stride, k_scale_block_stride;
  int t, h, q_lora, heads, n, block_size, format;
  float eps, heads_rsqrt;
};
int launch_pg_prolog(const PgPrologParams& p, void* workspace, cudaStream_t stream);
size_t pg_prolog_workspace_bytes(int t, int h, int q_lora, int heads);
int launch_hif8_convert(int direction, const void* in, void* out, long long n, cudaStream_t stream);

struct MlaV4StageParams {
  // quant != 0: the quantised operator (fp32 / int32 GEMM results, int8 qr); 0: the bf16 operator (bf16 throughout)
  const void* q_a;                // stage 0: fp32 (bf16) [t, 1024]
  const __nv_bfloat16* gamma_cq;  // bf16 [1024]
  void* qr;                       // stage 0 out: int8 (bf16) [t, 1024]
  float* qr_scale;                // stage 0 out / stage 1 in: fp32 [t] (quantised operator only)
  const void* q_b;                // stage 1: int32 (bf16) [t, q_b_ld], first heads*512 columns
  const float* wq_b_scale;        // fp32 [heads*512]
  __nv_bfloat16* q_out;           // stage 1 out: bf16 [t, heads, 512]
  const void* kv_a;               // stage 2: fp32 (bf16) [t, 512]
  const __nv_bfloat16* gamma_ckv; // bf16 [512]
  __nv_bfloat16* kv_out;          // stage 2 out: bf16 [t, 512]
  const __nv_bfloat16* cos;       // bf16 [t, 64]
  const __nv_bfloat16* sin;
  int t, heads, q_b_ld, quant;
  float eps;
};
int launch_mla_v4_stage(const MlaV4StageParams& p, int stage, cudaStream_t stream);

struct AdvanceParams {
  int32_t* act_seq;              // in/out [b]
  const int32_t* block_table;    // [b, max_blocks]
  long long* cache_index;        // out [b, s1]
  uint32_t* status;
  int b, s1, grow, block_size, max_blocks;
};
int launch_decode_advance(const AdvanceParams& p, cudaStream_t stream);

struct CompressorParams {
  const float* kv_total;       // [b*s1, coff*d]  x . wkv^T
  const float* score_total;    // [b*s1, coff*d]  x . wgate^T
  const float* ape;            // [ratio, coff*d]
  const float* weight;         // [d]
  float* kv_state;             // [kv_blocks, 128, coff*d]
  float* score_state;          // [score_blocks, 128, coff*d]
  const int32_t* kv_table;     // [b, kv_cols]
  const int32_t* score_table;  // [b, score_cols]
  const __nv_bfloat16* sin;    // [>= b, 64]
  const __nv_bfloat16* cos;
  const int32_t* start_pos;    // [b]
  __nv_bfloat16* out;          // [>= b, d]
  uint32_t* status;
  long long kv_blocks, score_blocks;
  int b, s1, d, coff, ratio, kv_cols, score_cols;
  float eps;
};
int launch_compressor(const CompressorParams& p, cudaStream_t stream);

struct HcPreParams {
  const __nv_bfloat16* x;   // [t, 4, 4096]
  const float* hc_fn;       // [24, 16384]
  const float* hc_scale;    // [3]
  const float* hc_base;     // [24]
  __nv_bfloat16* y;         // [t, 4096]
  float* post;              // [t, 4]
  float* comb;              // [t, 4, 4]
  float* partial;           // workspace: [groups, t, 24] partial dot products
  int t, iters;
  float norm_eps, hc_eps;
};
int launch_hc_pre(const HcPreParams& p, cudaStream_t stream);
size_t hc_pre_workspace_bytes(int t);

}  // namespace dsv32

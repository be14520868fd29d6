// C ABI of libdsv32_b200.so: argument validation, workspace carving and kernel launches.
// Declarations and the reference interfaces they replace: include/dsv32_b200.h.
#include <atomic>
#include <climits>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace dsv32 {

// ---- bookkeeping -----------------------------------------------------------------------------------
static thread_local char g_err[512] = "";
static std::atomic<uint64_t> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }
int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
    return DSV32_ERR_CUDA;
  }
  return DSV32_OK;
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Key splits of the attention kernel.  Its CTAs (one per token, half of the value dims and split) run one per SM
// in waves; a CTA costs its key tiles plus about 3.5 tile times of set-up and epilogue, and a split run pays a
// combine pass over the partial results.  The split count that minimises waves x (tiles per CTA + fixed cost) is taken; sequence lengths
// live on the device, so every token is assumed to select `topk` keys.
static int pick_sfa_splits(int t, int nq, int topk, int requested) {
  (void)nq;
  const int max_splits = topk / 128 > 0 ? (topk / 128 < 16 ? topk / 128 : 16) : 1;
  if (requested > 0) return requested < max_splits ? requested : max_splits;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = (topk + 63) / 64;
  int best = 1;
  double best_cost = 0.0;
  for (int s = 1; s <= max_splits; ++s) {
    const long long ctas = 2ll * t * s;
    const long long waves = (ctas + sms - 1) / sms;
    const int per = (((topk + s - 1) / s) + 63) / 64;  // tiles of one CTA
    if (s > 1 && per * (s - 1) >= tiles) continue;     // a split that would be empty
    // combine pass: every split writes and re-reads a 128 x 512 fp32 partial (0.5 MB: 0.034 tile times at copy speed)
    const double cost = static_cast<double>(waves) * (per + 3.5) + (s > 1 ? 0.5 + 0.034 * t * s : 0.0);
    if (s == 1 || cost < best_cost) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

}  // namespace dsv32

using namespace dsv32;

#define REQUIRE(cond, ...)           \
  do {                               \
    if (!(cond)) {                   \
      set_error(__VA_ARGS__);        \
      return DSV32_ERR_INVALID_ARG;  \
    }                                \
  } while (0)

extern "C" {

int dsv32_abi_version(void) { return DSV32_ABI_VERSION; }
const char* dsv32_last_error(void) { return g_err; }
uint64_t dsv32_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

// ---- sparse flash attention ---------------------------------------------------------------------------
size_t dsv32_sfa_workspace_bytes(int32_t b, int32_t s1, int32_t n_q, int32_t topk, int32_t kv_splits) {
  if (b <= 0 || s1 <= 0 || n_q <= 0 || topk <= 0) return 0;
  const size_t t = static_cast<size_t>(b) * s1;
  size_t bytes = align_up(t * topk * sizeof(int32_t), 256);  // cache row of every selected key
  const int splits = pick_sfa_splits(b * s1, n_q, topk, kv_splits);
  if (splits > 1)
    bytes += align_up(t * splits * n_q * kKvLora * sizeof(float), 256) + align_up(t * splits * n_q * sizeof(float), 256);
  return bytes;
}

static int sfa_run(const Dsv32SfaArgs* a, void* cuda_stream, int nope_stride, int rope_stride, int scale_stride,
                   bool bf16_cache = false) {
  REQUIRE(a != nullptr, "sfa: args is NULL");
  REQUIRE(a->b >= 0 && a->s1 >= 1, "sfa: bad b=%d s1=%d", a->b, a->s1);
  if (a->b == 0) return DSV32_OK;
  REQUIRE(a->n_q >= 1 && a->n_q <= 128, "sfa: n_q=%d must be in [1, 128]", a->n_q);
  REQUIRE(a->topk >= 1, "sfa: topk=%d must be >= 1", a->topk);
  REQUIRE(a->block_size >= 1 && a->max_blocks >= 1, "sfa: bad block_size=%d max_blocks=%d", a->block_size,
          a->max_blocks);
  REQUIRE(a->rows >= 0, "sfa: rows=%lld must be >= 0", static_cast<long long>(a->rows));
  REQUIRE(a->query_nope && a->query_rope && a->key_nope && a->key_rope && (a->k_nope_scales || bf16_cache) &&
              a->topk_indices && a->block_table && a->kv_act_seqs && a->attention_out,
          "sfa: NULL tensor pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(a->key_nope) % 16 == 0 && reinterpret_cast<uintptr_t>(a->key_rope) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->k_nope_scales) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->query_nope) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->query_rope) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->attention_out) % 16 == 0,
          "sfa: tensors must be 16-byte aligned");
  const int t = a->b * a->s1;
  const int splits = pick_sfa_splits(t, a->n_q, a->topk, a->kv_splits);
  SfaParams p{};
  p.q_nope = static_cast<const __nv_bfloat16*>(a->query_nope);
  p.q_rope = static_cast<const __nv_bfloat16*>(a->query_rope);
  p.k_nope = static_cast<const int8_t*>(a->key_nope);
  p.k_rope = static_cast<const __nv_bfloat16*>(a->key_rope);
  p.k_scales = a->k_nope_scales;
  p.topk_idx = a->topk_indices;
  p.block_table = a->block_table;
  p.act_seq = a->kv_act_seqs;
  p.out = static_cast<__nv_bfloat16*>(a->attention_out);
  p.status = a->status;
  p.rows = a->rows;
  p.b = a->b; p.s1 = a->s1; p.nq = a->n_q; p.topk = a->topk; p.block_size = a->block_size;
  p.bs_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1 << sh) == a->block_size) p.bs_shift = sh;
  p.max_blocks = a->max_blocks; p.splits = splits; p.scale = a->softmax_scale;
  p.nope_stride = nope_stride; p.rope_stride = rope_stride; p.scale_stride = scale_stride;
  p.kn_bf16 = bf16_cache ? 1 : 0;
  {
    const size_t need = dsv32_sfa_workspace_bytes(a->b, a->s1, a->n_q, a->topk, splits);
    if (a->workspace == nullptr || a->workspace_bytes < need ||
        reinterpret_cast<uintptr_t>(a->workspace) % 256 != 0) {
      set_error("sfa: workspace of %zu bytes (256-byte aligned) required, got %zu", need, a->workspace_bytes);
      return DSV32_ERR_WORKSPACE;
    }
    char* ws = static_cast<char*>(a->workspace);
    p.row_ids = reinterpret_cast<int32_t*>(ws);
    ws += align_up(static_cast<size_t>(t) * a->topk * sizeof(int32_t), 256);
    if (splits > 1) {
      const size_t o_bytes = align_up(static_cast<size_t>(t) * splits * a->n_q * kKvLora * sizeof(float), 256);
      p.part_o = reinterpret_cast<float*>(ws);
      p.part_lse = reinterpret_cast<float*>(ws + o_bytes);
    }
  }
  return launch_sfa_tc(p, static_cast<cudaStream_t>(cuda_stream));
}

int dsv32_sfa_quant(const Dsv32SfaArgs* a, void* cuda_stream) { return sfa_run(a, cuda_stream, kKvLora, kRopeDim * 2, 16); }

int dsv32_sfa_bf16_cache(const Dsv32SfaArgs* a, void* cuda_stream) {
  return sfa_run(a, cuda_stream, kKvLora * 2, kRopeDim * 2, 0, true);
}

int dsv32_sparse_attention_antiquant(const Dsv32SaAntiquantArgs* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "sa_antiquant: args is NULL");
  REQUIRE(a->b <= 0 || a->nope_cache != nullptr, "sa_antiquant: NULL cache pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(a->nope_cache) % 16 == 0, "sa_antiquant: the cache must be 16-byte aligned");
  // one row = 512 int8 latent dims | 64 bf16 rope dims | 4 fp32 group scales
  const char* cache = static_cast<const char*>(a->nope_cache);
  Dsv32SfaArgs s{};
  s.query_nope = a->query_nope;
  s.query_rope = a->query_rope;
  s.key_nope = cache;
  s.key_rope = cache + kKvLora;
  s.k_nope_scales = reinterpret_cast<const float*>(cache + kKvLora + kRopeDim * 2);
  s.topk_indices = a->topk_indices;
  s.block_table = a->block_table;
  s.kv_act_seqs = a->kv_act_seqs;
  s.attention_out = a->attention_out;
  s.workspace = a->workspace;
  s.workspace_bytes = a->workspace_bytes;
  s.status = a->status;
  s.rows = a->rows;
  s.b = a->b; s.s1 = a->s1; s.n_q = a->n_q; s.topk = a->topk; s.block_size = a->block_size;
  s.max_blocks = a->max_blocks; s.kv_splits = a->kv_splits; s.softmax_scale = a->softmax_scale;
  return sfa_run(&s, cuda_stream, DSV32_ANTIQUANT_ROW_BYTES, DSV32_ANTIQUANT_ROW_BYTES, DSV32_ANTIQUANT_ROW_BYTES);
}

// ---- DeepSeek-V4 sparse compress attention ------------------------------------------------------------------
size_t dsv32_scfa_workspace_bytes(int32_t t, int32_t topk, int32_t win_size) {
  if (t <= 0 || topk < 0 || win_size < 0) return 0;
  // cache row of every listed key (one more slot: the union window of two paired tokens) + the length of every list
  return align_up(static_cast<size_t>(t) * (2 * static_cast<size_t>(topk) + win_size + 1) * sizeof(int32_t), 256) +
         align_up(static_cast<size_t>(t) * sizeof(int32_t), 256);
}

int dsv32_sparse_compress_attention(const Dsv32ScfaArgs* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "scfa: args is NULL");
  REQUIRE(a->t >= 0 && a->b >= 0, "scfa: bad t=%d b=%d", a->t, a->b);
  if (a->t == 0 || a->b == 0) return DSV32_OK;
  REQUIRE(a->n_q >= 1 && a->n_q <= 128, "scfa: n_q=%d must be in [1, 128]", a->n_q);
  REQUIRE(a->topk >= 0 && a->win_size >= 0 && a->topk + a->win_size >= 1, "scfa: bad topk=%d win_size=%d", a->topk,
          a->win_size);
  REQUIRE(a->cmp_ratio >= 1, "scfa: cmp_ratio=%d must be >= 1", a->cmp_ratio);
  REQUIRE(a->block_size >= 1 && a->ori_max_blocks >= 1 && (a->cmp_max_blocks >= 1 || a->topk == 0),
          "scfa: bad block_size=%d ori_max_blocks=%d cmp_max_blocks=%d", a->block_size, a->ori_max_blocks,
          a->cmp_max_blocks);
  REQUIRE(a->ori_rows >= 0 && a->cmp_rows >= 0, "scfa: bad ori_rows=%lld cmp_rows=%lld",
          static_cast<long long>(a->ori_rows), static_cast<long long>(a->cmp_rows));
  REQUIRE(a->cmp_mode == DSV32_SCFA_SELECTED || a->cmp_mode == DSV32_SCFA_ALL_COMPRESSED, "scfa: bad cmp_mode=%d",
          a->cmp_mode);
  REQUIRE(a->query && a->actual_seq_q && a->ori_kv && a->ori_block_table && a->atten_sink && a->seqused_kv &&
              a->attention_out,
          "scfa: NULL tensor pointer");
  REQUIRE(a->topk == 0 || (a->cmp_kv && a->cmp_block_table &&
                           (a->cmp_sparse_indices || a->cmp_mode == DSV32_SCFA_ALL_COMPRESSED)),
          "scfa: NULL compressed-cache pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(a->query) % 16 == 0 && reinterpret_cast<uintptr_t>(a->ori_kv) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->cmp_kv) % 16 == 0 && reinterpret_cast<uintptr_t>(a->attention_out) % 16 == 0,
          "scfa: tensors must be 16-byte aligned");
  SfaParams p{};
  p.compress = 1;
  p.kn_bf16 = 1;
  p.q_nope = static_cast<const __nv_bfloat16*>(a->query);
  p.k_nope = static_cast<const int8_t*>(a->ori_kv);
  p.k_nope2 = static_cast<const __nv_bfloat16*>(a->cmp_kv);
  p.topk_idx = a->cmp_sparse_indices;
  p.block_table = a->ori_block_table;
  p.block_table2 = a->cmp_block_table;
  p.act_seq = a->seqused_kv;
  p.seq_q = a->actual_seq_q;
  p.sinks = a->atten_sink;
  p.out = static_cast<__nv_bfloat16*>(a->attention_out);
  p.status = a->status;
  p.rows = a->ori_rows;
  p.rows2 = a->cmp_rows;
  p.b = a->b; p.s1 = 1; p.t_total = a->t; p.nq = a->n_q;
  // Tokens 2k, 2k+1 of a request share a CTA when the heads of both fit the 128-row tile: their window differs in one
  // position; the compressed keys are the same but one (all-compressed) or the union of both selections (selected,
  // as long as a request's compressed positions fit the pre-pass' bitmaps).
  p.pair = 0;
  if (a->n_q <= 64) {
    if (a->cmp_mode == DSV32_SCFA_ALL_COMPRESSED || a->topk == 0) p.pair = 1;
    else if (static_cast<long long>(a->cmp_max_blocks) * a->block_size <= 131072 && a->t >= 2) p.pair = 2;
  }
  // slots of a key list: the union window of two paired tokens is one longer, the union of two selections up to twice
  p.topk = a->win_size + 1 + (p.pair == 2 ? 2 * a->topk : a->topk);
  p.sel_topk = a->topk; p.win_size = a->win_size; p.cmp_ratio = a->cmp_ratio;
  p.cmp_dense = a->cmp_mode == DSV32_SCFA_ALL_COMPRESSED ? 1 : 0;
  p.block_size = a->block_size;
  p.bs_shift = -1;
  p.max_blocks = a->ori_max_blocks; p.max_blocks2 = a->cmp_max_blocks;
  p.splits = 1;
  p.scale = a->softmax_scale;
  p.nope_stride = kKvLora * 2; p.rope_stride = 0; p.scale_stride = 0;
  const size_t need = dsv32_scfa_workspace_bytes(a->t, a->topk, a->win_size);
  if (a->workspace == nullptr || a->workspace_bytes < need || reinterpret_cast<uintptr_t>(a->workspace) % 256 != 0) {
    set_error("scfa: workspace of %zu bytes (256-byte aligned) required, got %zu", need, a->workspace_bytes);
    return DSV32_ERR_WORKSPACE;
  }
  char* ws = static_cast<char*>(a->workspace);
  p.row_ids = reinterpret_cast<int32_t*>(ws);
  p.key_counts = reinterpret_cast<int32_t*>(
      ws + align_up(static_cast<size_t>(a->t) * (2 * static_cast<size_t>(a->topk) + a->win_size + 1) * sizeof(int32_t), 256));
  return launch_sfa_tc(p, static_cast<cudaStream_t>(cuda_stream));
}

// ---- lightning indexer --------------------------------------------------------------------------------
size_t dsv32_indexer_workspace_bytes(int32_t b, int32_t s1, int32_t max_blocks, int32_t block_size) {
  if (b <= 0 || s1 <= 0 || max_blocks <= 0 || block_size <= 0) return 0;
  return align_up(static_cast<size_t>(b) * s1 * max_blocks * block_size * sizeof(float), 256);
}

static int indexer_topk_run(const Dsv32IndexerArgs* a, const Dsv32TopkScatter* sc, void* cuda_stream);

int dsv32_indexer_topk(const Dsv32IndexerArgs* a, void* cuda_stream) { return indexer_topk_run(a, nullptr, cuda_stream); }

int dsv32_indexer_topk_scatter(const Dsv32IndexerArgs* a, const Dsv32TopkScatter* sc, void* cuda_stream) {
  REQUIRE(a != nullptr && sc != nullptr, "indexer scatter: args is NULL");
  REQUIRE(a->b == 1, "indexer scatter: one request (b=%d)", a->b);
  REQUIRE(sc->world >= 1 && sc->world <= 8 && sc->rank >= 0 && sc->rank < sc->world,
          "indexer scatter: bad world=%d rank=%d (at most 8 ranks)", sc->world, sc->rank);
  REQUIRE(sc->tokens_per_rank >= 1 && static_cast<long long>(sc->tokens_per_rank) * sc->world >= a->s1,
          "indexer scatter: tokens_per_rank=%d x world=%d does not cover s1=%d", sc->tokens_per_rank, sc->world, a->s1);
  REQUIRE(a->selected_count >= 1 && a->selected_count <= 2048, "indexer scatter: selected_count=%d must be in [1, 2048]",
          a->selected_count);
  for (int r = 0; r < sc->world; ++r)
    REQUIRE(sc->idx_ptrs[r] != nullptr && sc->score_ptrs[r] != nullptr &&
                reinterpret_cast<uintptr_t>(sc->idx_ptrs[r]) % 16 == 0 && reinterpret_cast<uintptr_t>(sc->score_ptrs[r]) % 16 == 0,
            "indexer scatter: NULL or unaligned buffer of rank %d", r);
  return indexer_topk_run(a, sc, cuda_stream);
}

static int indexer_topk_run(const Dsv32IndexerArgs* a, const Dsv32TopkScatter* sc, void* cuda_stream) {
  REQUIRE(a != nullptr, "indexer: args is NULL");
  REQUIRE(a->b >= 0 && a->s1 >= 1, "indexer: bad b=%d s1=%d", a->b, a->s1);
  if (a->b == 0) return DSV32_OK;
  REQUIRE(a->block_size == 128, "indexer: block_size=%d (only 128 is supported)", a->block_size);
  REQUIRE(a->max_blocks >= 1 && a->num_blocks >= 0, "indexer: bad max_blocks=%d num_blocks=%lld", a->max_blocks,
          static_cast<long long>(a->num_blocks));
  REQUIRE(a->idx_query && a->idx_query_scale && a->idx_key_cache && a->idx_key_scale && a->idx_weight &&
              a->act_seq_key && a->block_table,
          "indexer: NULL tensor pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(a->idx_query) % 16 == 0 && reinterpret_cast<uintptr_t>(a->idx_key_cache) % 16 == 0,
          "indexer: idx_query / idx_key_cache must be 16-byte aligned");
  REQUIRE(a->topk_res == nullptr || (a->selected_count >= 1 && a->selected_count <= 2048),
          "indexer: selected_count=%d must be in [1, 2048]", a->selected_count);
  REQUIRE(a->key_begin >= 0 && a->key_end > a->key_begin, "indexer: bad key range [%d, %d)", a->key_begin, a->key_end);
  const int full_ld = a->max_blocks * a->block_size;
  const int ld = a->score_ld > 0 ? a->score_ld : full_ld;
  REQUIRE(ld >= full_ld, "indexer: score_ld=%d smaller than max_blocks*block_size=%d", ld, full_ld);
  REQUIRE(a->dots_out == nullptr || a->scores_out != nullptr || ld == full_ld, "indexer: bad dots_out stride");
  float* scores = a->scores_out;
  if (scores == nullptr) {
    const size_t need = dsv32_indexer_workspace_bytes(a->b, a->s1, a->max_blocks, a->block_size);
    if (a->workspace == nullptr || a->workspace_bytes < need || ld != full_ld) {
      set_error("indexer: workspace of %zu bytes required, got %zu", need, a->workspace_bytes);
      return DSV32_ERR_WORKSPACE;
    }
    scores = static_cast<float*>(a->workspace);
  }
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  IndexerParams p{};
  p.q = a->idx_query;
  p.q_scale = static_cast<const __half*>(a->idx_query_scale);
  p.weight = static_cast<const __half*>(a->idx_weight);
  p.keys = a->idx_key_cache;
  p.key_scale = static_cast<const __half*>(a->idx_key_scale);
  p.act_seq = a->act_seq_key;
  p.block_table = a->block_table;
  p.scores = scores;
  p.dots = a->dots_out;
  p.status = a->status;
  p.num_blocks = a->num_blocks;
  p.b = a->b; p.s1 = a->s1; p.block_size = a->block_size; p.max_blocks = a->max_blocks; p.ld = ld;
  p.key_begin = a->key_begin;
  p.key_end = a->key_end;
  int rc = launch_indexer_scores_tc(p, st);
  if (rc != DSV32_OK || (a->topk_res == nullptr && sc == nullptr)) return rc;
  TopkParams tp{};
  if (sc != nullptr) {
    tp.scatter_world = sc->world;
    tp.scatter_rank = sc->rank;
    tp.scatter_per = sc->tokens_per_rank;
    for (int r = 0; r < sc->world; ++r) {
      tp.scatter_idx[r] = static_cast<int32_t*>(sc->idx_ptrs[r]);
      tp.scatter_sc[r] = static_cast<float*>(sc->score_ptrs[r]);
    }
  }
  tp.scores = scores;
  tp.ids = nullptr;
  tp.counts = nullptr;
  tp.act_seq = a->act_seq_key;
  tp.out_idx = a->topk_res;
  tp.out_scores = a->topk_scores;
  tp.s1 = a->s1;
  tp.key_begin = a->key_begin;
  tp.key_end = a->key_end < full_ld ? a->key_end : full_ld;  // scores exist up to the page table's capacity
  tp.ld = ld;
  tp.k = a->selected_count;
  tp.id_base = 0;
  return launch_topk(tp, a->b * a->s1, st);
}

int dsv32_topk_select(const Dsv32TopkArgs* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "topk: args is NULL");
  REQUIRE(a->rows >= 0 && a->ld >= 1, "topk: bad rows=%d ld=%d", a->rows, a->ld);
  if (a->rows == 0) return DSV32_OK;
  REQUIRE(a->k >= 1 && a->k <= 2048, "topk: k=%d must be in [1, 2048]", a->k);
  REQUIRE(a->scores && a->counts && a->out_idx, "topk: NULL tensor pointer");
  TopkParams tp{};
  tp.scores = a->scores;
  tp.ids = a->ids;
  tp.counts = a->counts;
  tp.act_seq = nullptr;
  tp.out_idx = a->out_idx;
  tp.out_scores = a->out_scores;
  tp.s1 = 1;
  tp.key_begin = 0;
  tp.key_end = INT_MAX;
  tp.ld = a->ld;
  tp.k = a->k;
  tp.id_base = a->id_base;
  return launch_topk(tp, a->rows, static_cast<cudaStream_t>(cuda_stream));
}

// ---- indexer prolog -----------------------------------------------------------------------------------
size_t dsv32_prolog_v4_workspace_bytes(int32_t t, int32_t h) { return align_up(prolog_v4_workspace_bytes(t, h), 256); }

int dsv32_indexer_prolog_v4(const Dsv32PrologV4Args* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "prolog v4: args is NULL");
  REQUIRE(a->t >= 0, "prolog v4: bad t=%d", a->t);
  if (a->t == 0) return DSV32_OK;
  REQUIRE(a->h >= 1, "prolog v4: bad h=%d", a->h);
  REQUIRE(a->qr && a->idx_wq_b && a->x && a->weights_proj && a->cos && a->sin && a->hadamard && a->qr_scale &&
              a->idx_wq_b_scale && a->q && a->weights && a->q_scale,
          "prolog v4: NULL tensor pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(a->qr) % 16 == 0 && reinterpret_cast<uintptr_t>(a->idx_wq_b) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->hadamard) % 16 == 0 && reinterpret_cast<uintptr_t>(a->q) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->cos) % 4 == 0 && reinterpret_cast<uintptr_t>(a->sin) % 4 == 0,
          "prolog v4: qr / idx_wq_b / hadamard / q must be 16-byte aligned, cos / sin 4-byte aligned");
  const size_t need_v4 = prolog_v4_workspace_bytes(a->t, a->h);
  if (a->workspace == nullptr || a->workspace_bytes < need_v4 || reinterpret_cast<uintptr_t>(a->workspace) % 16 != 0) {
    set_error("prolog v4: workspace of %zu bytes (16-byte aligned) required, got %zu", need_v4, a->workspace_bytes);
    return DSV32_ERR_WORKSPACE;
  }
  PrologParams p{};
  p.partial = static_cast<float*>(a->workspace);
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.q_norm = a->qr;
  p.q_norm_scale = a->qr_scale;
  p.w_qb = a->idx_wq_b;
  p.w_qb_scale = a->idx_wq_b_scale;
  p.w_proj = static_cast<const __nv_bfloat16*>(a->weights_proj);
  p.cos = static_cast<const __nv_bfloat16*>(a->cos);
  p.sin = static_cast<const __nv_bfloat16*>(a->sin);
  p.had_q = static_cast<const __nv_bfloat16*>(a->hadamard);
  p.q_int8 = a->q;
  p.q_scale = static_cast<__half*>(a->q_scale);
  p.weights = static_cast<__half*>(a->weights);
  p.status = a->status;
  p.t = a->t;
  // 64^-0.5 * 128^-0.5 as the reference multiplies it in: (w * 0.125) * 128^-0.5, the first factor being exact
  const float w_scale = 0.125f * static_cast<float>(1.0 / sqrt(128.0));
  return launch_prolog_v4(p, a->h, w_scale, static_cast<cudaStream_t>(cuda_stream));
}

size_t dsv32_pg_indexer_prolog_workspace_bytes(int32_t t, int32_t h, int32_t q_lora, int32_t heads) {
  return pg_prolog_workspace_bytes(t, h, q_lora, heads);
}

int dsv32_pg_indexer_prolog(const Dsv32PgPrologArgs* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "pg prolog: args is NULL");
  REQUIRE(a->t >= 0 && a->t <= (1 << 22), "pg prolog: t=%d must be in [0, 2^22]", a->t);
  if (a->t == 0) return DSV32_OK;
  REQUIRE(a->format == DSV32_PG_FORMAT_MXFP8 || a->format == DSV32_PG_FORMAT_HIF8, "pg prolog: unknown format %d", a->format);
  REQUIRE(a->h >= 512 && a->h % 512 == 0, "pg prolog: h=%d must be a positive multiple of 512", a->h);
  REQUIRE(a->q_lora >= 256 && a->q_lora % 256 == 0, "pg prolog: q_lora=%d must be a positive multiple of 256", a->q_lora);
  REQUIRE(a->heads >= 1 && a->heads <= 128, "pg prolog: heads=%d must be in [1, 128]", a->heads);
  REQUIRE(a->block_size >= 1 && a->cache_rows >= 0 && a->cache_rows % a->block_size == 0,
          "pg prolog: cache_rows=%lld must be a whole number of pages of %d rows", static_cast<long long>(a->cache_rows),
          a->block_size);
  REQUIRE(a->k_block_stride >= static_cast<int64_t>(a->block_size) * 128 &&
              a->k_scale_block_stride >= static_cast<int64_t>(a->block_size) * 4 && a->k_scale_block_stride % 4 == 0,
          "pg prolog: page strides %lld / %lld are smaller than a page (or the scale stride is not a multiple of 4)",
          static_cast<long long>(a->k_block_stride), static_cast<long long>(a->k_scale_block_stride));
  REQUIRE(a->x && a->q_norm && a->q_norm_scale && a->w_qb && a->w_qb_scale && a->wk && a->w_proj && a->gamma_k &&
              a->cos_idx_rope && a->sin_idx_rope && a->hadamard_q && a->hadamard_k && a->k_cache_index &&
              a->k_scale_cache_index && a->q_quant && a->q_scale && a->k_cache && a->k_scale_cache && a->weights,
          "pg prolog: NULL tensor pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(a->x) % 16 == 0 && reinterpret_cast<uintptr_t>(a->q_norm) % 8 == 0 &&
              reinterpret_cast<uintptr_t>(a->w_qb) % 8 == 0 && reinterpret_cast<uintptr_t>(a->k_scale_cache) % 4 == 0,
          "pg prolog: x must be 16-byte aligned, q_norm / w_qb 8-byte aligned, k_scale_cache 4-byte aligned");
  const size_t need = pg_prolog_workspace_bytes(a->t, a->h, a->q_lora, a->heads);
  if (a->workspace == nullptr || a->workspace_bytes < need || reinterpret_cast<uintptr_t>(a->workspace) % 256 != 0) {
    set_error("pg prolog: workspace of %zu bytes (256-byte aligned) required, got %zu", need, a->workspace_bytes);
    return DSV32_ERR_WORKSPACE;
  }
  PgPrologParams p{};
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.q_norm = a->q_norm;
  p.w_qb = a->w_qb;
  if (a->format == DSV32_PG_FORMAT_MXFP8) {
    p.q_norm_scale_e8 = static_cast<const uint8_t*>(a->q_norm_scale);
    p.w_qb_scale_e8 = static_cast<const uint8_t*>(a->w_qb_scale);
  } else {
    p.q_norm_scale_f32 = static_cast<const float*>(a->q_norm_scale);
    p.w_qb_scale_f32 = static_cast<const float*>(a->w_qb_scale);
  }
  p.wk = static_cast<const __nv_bfloat16*>(a->wk);
  p.w_proj = static_cast<const __nv_bfloat16*>(a->w_proj);
  p.gamma_k = static_cast<const __nv_bfloat16*>(a->gamma_k);
  p.cos = static_cast<const __nv_bfloat16*>(a->cos_idx_rope);
  p.sin = static_cast<const __nv_bfloat16*>(a->sin_idx_rope);
  p.hadamard_q = static_cast<const __nv_bfloat16*>(a->hadamard_q);
  p.hadamard_k = static_cast<const __nv_bfloat16*>(a->hadamard_k);
  p.k_cache_index = reinterpret_cast<const long long*>(a->k_cache_index);
  p.k_scale_cache_index = reinterpret_cast<const long long*>(a->k_scale_cache_index);
  p.q_out = a->q_quant;
  p.q_scale_out = a->q_scale;
  p.k_cache = a->k_cache;
  p.k_scale_cache = a->k_scale_cache;
  p.weights_out = static_cast<__nv_bfloat16*>(a->weights);
  p.status = a->status;
  p.cache_rows = a->cache_rows;
  p.k_block_stride = a->k_block_stride;
  p.k_scale_block_stride = a->k_scale_block_stride;
  p.t = a->t; p.h = a->h; p.q_lora = a->q_lora; p.heads = a->heads; p.n = a->heads * 128;
  p.block_size = a->block_size; p.format = a->format;
  p.eps = a->eps;
  p.heads_rsqrt = static_cast<float>(1.0 / sqrt(static_cast<double>(a->heads)));
  return launch_pg_prolog(p, a->workspace, static_cast<cudaStream_t>(cuda_stream));
}

size_t dsv32_gemm_bf16_workspace_bytes(int32_t t, int32_t k, int32_t n) { return bf16_gemm_workspace_bytes(t, k, n); }

int dsv32_gemm_bf16(const Dsv32GemmBf16Args* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "gemm bf16: args is NULL");
  REQUIRE(a->t >= 0, "gemm bf16: bad t=%d", a->t);
  if (a->t == 0) return DSV32_OK;
  REQUIRE(a->k >= 64 && a->k % 64 == 0, "gemm bf16: k=%d must be a positive multiple of 64", a->k);
  REQUIRE(a->n >= 8 && a->n % 8 == 0, "gemm bf16: n=%d must be a positive multiple of 8", a->n);
  REQUIRE((a->b_layout == 0 || a->b_layout == 1) && (a->c_dtype == 0 || a->c_dtype == 1),
          "gemm bf16: b_layout=%d / c_dtype=%d must be 0 or 1", a->b_layout, a->c_dtype);
  REQUIRE(a->a && a->b && a->c, "gemm bf16: NULL tensor pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(a->a) % 16 == 0 && reinterpret_cast<uintptr_t>(a->b) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->c) % 16 == 0,
          "gemm bf16: a / b / c must be 16-byte aligned");
  const size_t need = bf16_gemm_workspace_bytes(a->t, a->k, a->n);
  if (a->workspace == nullptr || a->workspace_bytes < need || reinterpret_cast<uintptr_t>(a->workspace) % 256 != 0) {
    set_error("gemm bf16: workspace of %zu bytes (256-byte aligned) required, got %zu", need, a->workspace_bytes);
    return DSV32_ERR_WORKSPACE;
  }
  return launch_bf16_gemm(static_cast<const __nv_bfloat16*>(a->a), a->t, a->k, static_cast<const __nv_bfloat16*>(a->b), a->n,
                          a->b_layout == 1, a->c, a->c_dtype == 1, a->workspace, a->status,
                          static_cast<cudaStream_t>(cuda_stream));
}

int dsv32_gemm_i8(const Dsv32GemmI8Args* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "gemm int8: args is NULL");
  REQUIRE(a->t >= 0, "gemm int8: bad t=%d", a->t);
  if (a->t == 0) return DSV32_OK;
  REQUIRE(a->a && a->b && a->c, "gemm int8: NULL tensor pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(a->a) % 16 == 0 && reinterpret_cast<uintptr_t>(a->b) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->c) % 16 == 0,
          "gemm int8: a / b / c must be 16-byte aligned");
  return launch_i8_gemm(a->a, a->t, a->k, a->b, a->n, a->c, a->status, static_cast<cudaStream_t>(cuda_stream));
}

int dsv32_hif8_convert(int32_t direction, const void* in, void* out, int64_t n, void* cuda_stream) {
  REQUIRE(direction == 0 || direction == 1, "hif8 convert: direction %d is neither 0 (encode) nor 1 (decode)", direction);
  REQUIRE(n >= 0, "hif8 convert: bad n=%lld", static_cast<long long>(n));
  if (n == 0) return DSV32_OK;
  REQUIRE(in != nullptr && out != nullptr, "hif8 convert: NULL pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(direction == 0 ? in : out) % 4 == 0, "hif8 convert: the fp32 array must be 4-byte aligned");
  return launch_hif8_convert(direction, in, out, n, static_cast<cudaStream_t>(cuda_stream));
}

size_t dsv32_prolog_workspace_bytes(int32_t t) { return t > 0 ? align_up(prolog_workspace_bytes(t), 256) : 0; }

int dsv32_indexer_prolog(const Dsv32PrologArgs* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "prolog: args is NULL");
  REQUIRE(a->t >= 0, "prolog: bad t=%d", a->t);
  if (a->t == 0) return DSV32_OK;
  REQUIRE(a->x && a->q_norm && a->q_norm_scale && a->w_qb && a->w_qb_scale && a->wk && a->w_proj && a->ln_gamma_k &&
              a->ln_beta_k && a->cos_idx_rope && a->sin_idx_rope && a->hadamard_q && a->hadamard_k &&
              a->k_cache_index && a->q_int8 && a->q_scale && a->k_cache && a->k_scale_cache && a->weights,
          "prolog: NULL tensor pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(a->q_norm) % 16 == 0 && reinterpret_cast<uintptr_t>(a->w_qb) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->hadamard_q) % 16 == 0 && reinterpret_cast<uintptr_t>(a->hadamard_k) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->x) % 16 == 0 && reinterpret_cast<uintptr_t>(a->wk) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->w_proj) % 16 == 0,
          "prolog: x / q_norm / weights / hadamard matrices must be 16-byte aligned");
  REQUIRE(a->cache_rows >= 1, "prolog: cache_rows=%lld must be >= 1", static_cast<long long>(a->cache_rows));
  const size_t need = dsv32_prolog_workspace_bytes(a->t);
  if (a->workspace == nullptr || a->workspace_bytes < need) {
    set_error("prolog: workspace of %zu bytes required, got %zu", need, a->workspace_bytes);
    return DSV32_ERR_WORKSPACE;
  }
  PrologParams p{};
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.q_norm = a->q_norm;
  p.q_norm_scale = a->q_norm_scale;
  p.w_qb = a->w_qb;
  p.w_qb_scale = a->w_qb_scale;
  p.wk = static_cast<const __nv_bfloat16*>(a->wk);
  p.w_proj = static_cast<const __nv_bfloat16*>(a->w_proj);
  p.ln_gamma = static_cast<const __nv_bfloat16*>(a->ln_gamma_k);
  p.ln_beta = static_cast<const __nv_bfloat16*>(a->ln_beta_k);
  p.cos = static_cast<const __nv_bfloat16*>(a->cos_idx_rope);
  p.sin = static_cast<const __nv_bfloat16*>(a->sin_idx_rope);
  p.had_q = static_cast<const __nv_bfloat16*>(a->hadamard_q);
  p.had_k = static_cast<const __nv_bfloat16*>(a->hadamard_k);
  p.cache_index = reinterpret_cast<const long long*>(a->k_cache_index);
  p.q_int8 = a->q_int8;
  p.q_scale = static_cast<__half*>(a->q_scale);
  p.k_cache = a->k_cache;
  p.k_scale_cache = static_cast<__half*>(a->k_scale_cache);
  p.weights = static_cast<__half*>(a->weights);
  p.partial = static_cast<float*>(a->workspace);
  p.status = a->status;
  p.cache_rows = a->cache_rows;
  p.t = a->t;
  p.eps = a->ln_eps;
  return launch_prolog_tc(p, static_cast<cudaStream_t>(cuda_stream));
}

// ---- MLA prolog and the fused MLA + indexer prolog ---------------------------------------------------------------
size_t dsv32_mla_prolog_workspace_bytes(int32_t t) { return mla_prolog_workspace_bytes(t); }

static int mla_fill(const Dsv32MlaPrologArgs* a, MlaParams& p) {
  REQUIRE(a->x && a->w_dq && a->w_uq_qr && a->w_qb_scale && a->w_uk && a->w_dkv_kr && a->gamma_cq && a->gamma_ckv &&
              a->cos && a->sin && a->cache_index && a->kv_cache && a->kr_cache && a->k_scale_cache && a->q_norm &&
              a->q_norm_scale && a->query_nope && a->query_rope,
          "mla prolog: NULL tensor pointer");
  REQUIRE(a->cache_rows >= 1, "mla prolog: cache_rows=%lld must be >= 1", static_cast<long long>(a->cache_rows));
  REQUIRE(reinterpret_cast<uintptr_t>(a->x) % 16 == 0 && reinterpret_cast<uintptr_t>(a->w_dq) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->w_uq_qr) % 16 == 0 && reinterpret_cast<uintptr_t>(a->w_uk) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->w_dkv_kr) % 16 == 0 && reinterpret_cast<uintptr_t>(a->q_norm) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->query_nope) % 16 == 0 && reinterpret_cast<uintptr_t>(a->query_rope) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->cos) % 4 == 0 && reinterpret_cast<uintptr_t>(a->sin) % 4 == 0,
          "mla prolog: x / weights / q_norm / query outputs must be 16-byte aligned, cos / sin 4-byte aligned");
  const size_t need = mla_prolog_workspace_bytes(a->t);
  if (a->workspace == nullptr || a->workspace_bytes < need || reinterpret_cast<uintptr_t>(a->workspace) % 256 != 0) {
    set_error("mla prolog: workspace of %zu bytes (256-byte aligned) required, got %zu", need, a->workspace_bytes);
    return DSV32_ERR_WORKSPACE;
  }
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.w_dq = static_cast<const __nv_bfloat16*>(a->w_dq);
  p.w_uq_qr = a->w_uq_qr;
  p.w_qb_scale = a->w_qb_scale;
  p.w_uk = static_cast<const __nv_bfloat16*>(a->w_uk);
  p.w_dkv_kr = static_cast<const __nv_bfloat16*>(a->w_dkv_kr);
  p.gamma_cq = static_cast<const __nv_bfloat16*>(a->gamma_cq);
  p.gamma_ckv = static_cast<const __nv_bfloat16*>(a->gamma_ckv);
  p.cos = static_cast<const __nv_bfloat16*>(a->cos);
  p.sin = static_cast<const __nv_bfloat16*>(a->sin);
  p.cache_index = reinterpret_cast<const long long*>(a->cache_index);
  p.kv_cache = a->kv_cache;
  p.kr_cache = static_cast<__nv_bfloat16*>(a->kr_cache);
  p.k_scale_cache = a->k_scale_cache;
  p.q_norm = a->q_norm;
  p.q_norm_scale = a->q_norm_scale;
  p.q_nope = static_cast<__nv_bfloat16*>(a->query_nope);
  p.q_rope = static_cast<__nv_bfloat16*>(a->query_rope);
  p.workspace = a->workspace;
  p.status = a->status;
  p.cache_rows = a->cache_rows;
  p.t = a->t;
  p.eps_cq = a->eps_cq;
  p.eps_ckv = a->eps_ckv;
  return DSV32_OK;
}

int dsv32_mla_prolog(const Dsv32MlaPrologArgs* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "mla prolog: args is NULL");
  REQUIRE(a->t >= 0, "mla prolog: bad t=%d", a->t);
  if (a->t == 0) return DSV32_OK;
  MlaParams p{};
  const int rc = mla_fill(a, p);
  if (rc != DSV32_OK) return rc;
  return launch_mla_prolog(p, static_cast<cudaStream_t>(cuda_stream));
}

int dsv32_mla_indexer_prolog(const Dsv32FusedPrologArgs* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "mla indexer prolog: args is NULL");
  REQUIRE(a->mla.t == a->indexer.t, "mla indexer prolog: token counts differ (%d / %d)", a->mla.t, a->indexer.t);
  // the indexer half reads the int8 q_norm / q_norm_scale the MLA half writes, and the same x
  REQUIRE(a->indexer.q_norm == a->mla.q_norm && a->indexer.q_norm_scale == a->mla.q_norm_scale &&
              a->indexer.x == a->mla.x,
          "mla indexer prolog: the indexer half must take x, q_norm and q_norm_scale of the MLA half");
  int rc = dsv32_mla_prolog(&a->mla, cuda_stream);
  if (rc != DSV32_OK) return rc;
  return dsv32_indexer_prolog(&a->indexer, cuda_stream);
}

// ---- diagnostic: a bounded device-side wait that runs out ---------------------------------------------------------
int dsv32_wait_selftest(uint32_t* status, int64_t budget_cycles, void* cuda_stream) {
  REQUIRE(status != nullptr, "wait selftest: status is NULL");
  REQUIRE(budget_cycles >= 0 && budget_cycles <= 2000000000ll, "wait selftest: budget of %lld cycles is out of range",
          static_cast<long long>(budget_cycles));
  return launch_wait_selftest(status, budget_cycles, static_cast<cudaStream_t>(cuda_stream));
}

// ---- multi-step decode: next step's sequence lengths and cache rows ----------------------------------------------
int dsv32_decode_advance(const Dsv32AdvanceArgs* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "decode advance: args is NULL");
  REQUIRE(a->b >= 0 && a->s1 >= 1, "decode advance: bad b=%d s1=%d", a->b, a->s1);
  if (a->b == 0) return DSV32_OK;
  REQUIRE(a->grow >= 0, "decode advance: grow=%d must be >= 0", a->grow);
  REQUIRE(a->block_size >= 1 && a->max_blocks >= 1, "decode advance: bad block_size=%d max_blocks=%d", a->block_size,
          a->max_blocks);
  REQUIRE(a->act_seq && a->block_table && a->cache_index, "decode advance: NULL tensor pointer");
  AdvanceParams p{};
  p.act_seq = a->act_seq;
  p.block_table = a->block_table;
  p.cache_index = reinterpret_cast<long long*>(a->cache_index);
  p.status = a->status;
  p.b = a->b; p.s1 = a->s1; p.grow = a->grow; p.block_size = a->block_size; p.max_blocks = a->max_blocks;
  return launch_decode_advance(p, static_cast<cudaStream_t>(cuda_stream));
}

int dsv32_mla_prolog_v4_stage(const Dsv32MlaV4StageArgs* a, int32_t stage, void* cuda_stream) {
  REQUIRE(a != nullptr, "mla v4: args is NULL");
  REQUIRE(stage >= 0 && stage <= 2, "mla v4: stage=%d must be 0, 1 or 2", stage);
  REQUIRE(a->t >= 0, "mla v4: bad t=%d", a->t);
  if (a->t == 0) return DSV32_OK;
  REQUIRE(a->quant == 0 || a->quant == 1, "mla v4: quant=%d must be 0 or 1", a->quant);
  if (stage == 0)
    REQUIRE(a->q_a && a->gamma_cq && a->qr && (a->qr_scale || !a->quant), "mla v4 stage 0: NULL tensor pointer");
  if (stage == 1)
    REQUIRE(a->q_b && ((a->qr_scale && a->wq_b_scale) || !a->quant) && a->q_out && a->cos && a->sin && a->heads >= 1 &&
                a->heads <= 65535 && a->q_b_ld >= a->heads * 512,
            "mla v4 stage 1: NULL tensor pointer, bad heads=%d or q_b_ld=%d too small", a->heads, a->q_b_ld);
  if (stage == 2) REQUIRE(a->kv_a && a->gamma_ckv && a->kv_out && a->cos && a->sin, "mla v4 stage 2: NULL tensor pointer");
  MlaV4StageParams p{};
  p.q_a = a->q_a;
  p.gamma_cq = static_cast<const __nv_bfloat16*>(a->gamma_cq);
  p.qr = a->qr;
  p.qr_scale = a->qr_scale;
  p.q_b = a->q_b;
  p.wq_b_scale = a->wq_b_scale;
  p.q_out = static_cast<__nv_bfloat16*>(a->q_out);
  p.kv_a = a->kv_a;
  p.gamma_ckv = static_cast<const __nv_bfloat16*>(a->gamma_ckv);
  p.kv_out = static_cast<__nv_bfloat16*>(a->kv_out);
  p.cos = static_cast<const __nv_bfloat16*>(a->cos);
  p.sin = static_cast<const __nv_bfloat16*>(a->sin);
  p.t = a->t; p.heads = a->heads; p.q_b_ld = a->q_b_ld; p.quant = a->quant;
  p.eps = a->eps;
  return launch_mla_v4_stage(p, stage, static_cast<cudaStream_t>(cuda_stream));
}

size_t dsv32_hc_pre_workspace_bytes(int32_t t) { return align_up(hc_pre_workspace_bytes(t), 256); }

int dsv32_hc_pre(const Dsv32HcPreArgs* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "hc_pre: args is NULL");
  REQUIRE(a->t >= 0, "hc_pre: bad t=%d", a->t);
  if (a->t == 0) return DSV32_OK;
  REQUIRE(a->hc_mult == 4 && a->d == 4096, "hc_pre: only 4 streams of 4096 are supported (got %d x %d)", a->hc_mult, a->d);
  REQUIRE(a->iters >= 1, "hc_pre: iters=%d must be >= 1", a->iters);
  REQUIRE(a->x && a->hc_fn && a->hc_scale && a->hc_base && a->y && a->post && a->comb, "hc_pre: NULL tensor pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(a->x) % 16 == 0 && reinterpret_cast<uintptr_t>(a->y) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(a->hc_fn) % 16 == 0,
          "hc_pre: x, y and hc_fn must be 16-byte aligned");
  const size_t need = hc_pre_workspace_bytes(a->t);
  if (a->workspace == nullptr || a->workspace_bytes < need || reinterpret_cast<uintptr_t>(a->workspace) % 16 != 0) {
    set_error("hc_pre: workspace of %zu bytes (16-byte aligned) required, got %zu", need, a->workspace_bytes);
    return DSV32_ERR_WORKSPACE;
  }
  HcPreParams p{};
  p.partial = static_cast<float*>(a->workspace);
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.hc_fn = a->hc_fn;
  p.hc_scale = a->hc_scale;
  p.hc_base = a->hc_base;
  p.y = static_cast<__nv_bfloat16*>(a->y);
  p.post = a->post;
  p.comb = a->comb;
  p.t = a->t;
  p.iters = a->iters;
  p.norm_eps = a->norm_eps;
  p.hc_eps = a->hc_eps;
  return launch_hc_pre(p, static_cast<cudaStream_t>(cuda_stream));
}

int dsv32_compressor_update(const Dsv32CompressorArgs* a, void* cuda_stream) {
  REQUIRE(a != nullptr, "compressor: args is NULL");
  REQUIRE(a->b >= 0 && a->s1 >= 0, "compressor: bad b=%d s1=%d", a->b, a->s1);
  if (a->b == 0 || a->s1 == 0) return DSV32_OK;
  REQUIRE(a->ratio == 4 || a->ratio == 128, "compressor: ratio=%d must be 4 or 128", a->ratio);
  REQUIRE(a->d >= 64 && a->d <= 512 && a->d % 2 == 0, "compressor: d=%d must be even and in [64, 512]", a->d);
  REQUIRE(a->kv_cols >= 1 && a->score_cols >= 1 && a->kv_blocks >= 1 && a->score_blocks >= 1,
          "compressor: empty block table or state");
  REQUIRE(a->kv_total && a->score_total && a->ape && a->weight && a->kv_state && a->score_state &&
              a->kv_block_table && a->score_block_table && a->sin && a->cos && a->start_pos && a->out,
          "compressor: NULL tensor pointer");
  REQUIRE(reinterpret_cast<uintptr_t>(a->kv_state) % 16 == 0 && reinterpret_cast<uintptr_t>(a->score_state) % 16 == 0,
          "compressor: the states must be 16-byte aligned");
  CompressorParams p{};
  p.kv_total = a->kv_total;
  p.score_total = a->score_total;
  p.ape = a->ape;
  p.weight = a->weight;
  p.kv_state = a->kv_state;
  p.score_state = a->score_state;
  p.kv_table = a->kv_block_table;
  p.score_table = a->score_block_table;
  p.sin = static_cast<const __nv_bfloat16*>(a->sin);
  p.cos = static_cast<const __nv_bfloat16*>(a->cos);
  p.start_pos = a->start_pos;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.status = a->status;
  p.kv_blocks = a->kv_blocks;
  p.score_blocks = a->score_blocks;
  p.b = a->b; p.s1 = a->s1; p.d = a->d; p.ratio = a->ratio;
  p.coff = a->ratio == 4 ? 2 : 1;
  p.kv_cols = a->kv_cols; p.score_cols = a->score_cols;
  p.eps = a->eps;
  return launch_compressor(p, static_cast<cudaStream_t>(cuda_stream));
}

}  // extern "C"

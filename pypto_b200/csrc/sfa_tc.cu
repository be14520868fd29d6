// Sparse flash attention over the int8 paged latent KV cache on tcgen05 tensor cores (sm_100a).
// Follows models/deepseek_v32_exp/sparse_flash_attention_quant_impl.py:121-286 (golden:
// deepseekv32_sparse_flash_attention_quant.py:174-259).
//
// One CTA = (token, half of the 512 value dims, key split); M = all 128 query heads.
// Tensor memory (512 columns x 128 lanes, lane = head):
//   [  0,256)  O accumulator for this CTA's 256 value dims (fp32)
//   [256,320)  S buffer 0   (64 keys, fp32) -- after the softmax its first 32 columns hold P (bf16 pairs)
//   [320,384)  S buffer 1
//   [384,512)  Q dims 0..255 as bf16 pairs (A operand read straight from tensor memory)
// Shared memory: Q dims 256..575 (five 128x64 bf16 chunks, 128-byte swizzle, loaded by TMA) and two K
// stages of 64 gathered keys x 576 dims (nine 64x64 bf16 chunks, 128-byte swizzle).  A stage is read
// K-major by S = Q K^T and MN-major (as V) by O += P V, so the dequantised rows are written once.
// Warps: 0 = issuer of the S MMAs / tensor-memory owner, 1..4 = softmax + O rescale + epilogue (one head per
// thread, so row max / row sum need no shuffles; lane 0 of warp 1 also issues the PV MMAs), 5..20 = gather +
// dequantise producers (raw rows held in registers two tiles ahead of their use).  A stage is refilled in two steps: the chunks only S reads (the other half's value
// dims, the rope dims) as soon as S of the tile two back has completed, this CTA's own value chunks once its
// PV has.  The cache row of every selected key comes from a pre-pass (sfa_row_ids_kernel).
// The running maximum is only raised when a tile exceeds it by more than 2^8 (warp-uniform decision), so
// the read-modify-write of O in tensor memory is rare; P stays below 2^8 in between.
//
// The same kernel, as mode 2, is the DeepSeek-V4 sparse compress attention
// (models/deepseek_v4/sparse_compress_flash_attention_impl.py:47-168): bf16 rows of 512 dims that are key and
// value at once (no rope part: 32 instead of 36 MMAs per S tile), a key list made of the token's window rows of
// one cache followed by selected rows of a second (compressed) cache, up to 128 query heads (heads past n_q
// are idle lanes of the M = 128 tile), and one attention sink per head added to the softmax denominator.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace dsv32 {

constexpr int kStProducerWarps = 16;
constexpr int kStThreads = (5 + kStProducerWarps) * 32;   // 21 warps: MMA issuer, 4 softmax, 16 gather + dequantise
constexpr int kStTile = 64;              // keys per tile
constexpr int kStChunkBytes = kStTile * 128;       // one 64-dim chunk of a K stage (8 KB)
constexpr int kStStageBytes = 9 * kStChunkBytes;   // 73,728
constexpr int kStQChunkBytes = 128 * 128;          // one 64-dim chunk of Q (16 KB)
constexpr int kStQsBytes = 5 * kStQChunkBytes;     // dims 256..575
constexpr int kStOffQ = 2 * kStStageBytes;
constexpr int kStOffValid = kStOffQ + kStQsBytes;  // int[2][64]
constexpr int kStRingTiles = 8;            // tiles of row ids in flight per producer warp
constexpr int kStOffRing = kStOffValid + 2 * kStTile * 4;   // int[16 producer warps][8 tiles][4 rows]
constexpr int kStOffBars = kStOffRing + kStProducerWarps * kStRingTiles * 4 * 4;
constexpr int kStNumBars = 2 + 2 + 2 + 2 + 1;      // full[2], s_full[2], p_ready[2], pv_done[2], q_ready
constexpr int kStOffTmem = kStOffBars + kStNumBars * 8;
constexpr size_t kStSmemBytes = kStOffTmem + 16;   // no alignment slack: the kernel checks that its window is 1024-byte aligned
static_assert(kStSmemBytes <= 232448, "shared memory of one CTA (227 KB)");

constexpr uint32_t kColO = 0, kColS = 256, kColQ = 384;

constexpr float kRescaleThreshold = 8.0f;  // log2 units

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Raw cache data of one row as held by one producer thread.  kBf16: the latent cache is already bf16 (no scales;
// twice the bytes), otherwise int8 with one fp32 scale per 128-dim group.
constexpr int kModeInt8 = 0, kModeBf16 = 1, kModeCompress = 2;

template <bool kBf16>
struct StPrefetchT {
  int4 nope[kBf16 ? 8 : 4];
  int4 rope;
  float4 sc;
  bool valid;
};

// 16 int8 -> 16 bf16 = bf16_rn( float(int8) * scale ), bit for bit as the golden: float(int8) is built without
// the conversion pipe -- (2^23 + (x ^ 0x80)) read as a float, minus (2^23 + 128), is exactly x -- and the product
// is one fp32 rounding followed by the bf16 rounding.
__device__ __forceinline__ void st_dequant16(const int4& raw, float sc, uint4& lo, uint4& hi) {
  const int w[4] = {raw.x, raw.y, raw.z, raw.w};
  const uint64_t bias = f2_pack(0xCB000080u, 0xCB000080u);  // -(2^23 + 128) twice
  const uint64_t sc2 = f2_pack(__float_as_uint(sc), __float_as_uint(sc));
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t u = static_cast<uint32_t>(w[i]) ^ 0x80808080u;
    const uint64_t a = f2_pack(__byte_perm(u, 0x4B000000u, 0x7540), __byte_perm(u, 0x4B000000u, 0x7541));
    const uint64_t b = f2_pack(__byte_perm(u, 0x4B000000u, 0x7542), __byte_perm(u, 0x4B000000u, 0x7543));
    o[2 * i] = f2_to_bf16x2(f2_mul(f2_add(a, bias), sc2));
    o[2 * i + 1] = f2_to_bf16x2(f2_mul(f2_add(b, bias), sc2));
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// Cache row of every selected key (row + 1; 0 = no key: a -1 entry, a position past the token's valid count,
// or an entry that failed validation, which is also reported through the status word).  Paged-gather
// semantics of python/pypto/experimental/gather.py:18-87: row = block_table[b, idx / block] * block + idx % block.
__global__ void __launch_bounds__(256) sfa_row_ids_kernel(SfaParams p) {
  const int tok = blockIdx.y;
  const int j = blockIdx.x * 256 + threadIdx.x;
  if (j >= p.topk) return;
  const int bi = tok / p.s1, si = tok % p.s1;
  const int cnt = min(max(p.act_seq[bi] - p.s1 + 1 + si, 0), p.topk);
  int out = 0;
  if (j < cnt) {
    const int idx = __ldg(p.topk_idx + static_cast<size_t>(tok) * p.topk + j);
    if (idx >= 0) {
      const int lb = idx / p.block_size;
      if (lb >= p.max_blocks) {
        report_status(p.status, DSV32_STATUS_BAD_INDEX, tok, idx);
      } else {
        const int pb = __ldg(p.block_table + static_cast<size_t>(bi) * p.max_blocks + lb);
        const long long row = static_cast<long long>(pb) * p.block_size + idx % p.block_size;
        if (pb < 0 || row >= p.rows) report_status(p.status, DSV32_STATUS_BAD_PAGE, tok, idx);
        else out = static_cast<int>(row) + 1;
      }
    }
  }
  p.row_ids[static_cast<size_t>(tok) * p.topk + j] = out;
}

// Key list of every token for the sparse compress attention: first the window rows (the last
// min(cur_len, win_size) positions before cur_len = max(seq - s1 + 1 + i, 0), paged by block_table), then the
// rows of the compressed cache named by the first min(max(seq / cmp_ratio - s1 + 1 + i, 0), sel_topk) entries of
// the token's index row (paged by block_table2)  (sparse_compress_flash_attention_impl.py:83-131) -- or, with
// cmp_dense, every compressed position below cur_len / cmp_ratio (compress_flash_attention_impl.py:160-186).
// An entry is row + 1 in bits 0..28, bit 29 = "a key of this token", bit 31 = row of the compressed cache;
// 0 = no key.
// With p.pair (at most 64 heads, key lists that do not depend on an index tensor) the tokens 2k and 2k+1 of a
// request share one CTA: lanes 0..63 of the M = 128 tile are the heads of the first, lanes 64..127 those of the
// second.  The list is then the union of both lists -- they differ in one window position and at most one
// compressed position -- with bit 29 / bit 30 = member of the first / second token's list; it is stored in the
// first token's slot, and the second token's count is -1 ("done by the partner").
__global__ void __launch_bounds__(256) scfa_row_ids_kernel(SfaParams p) {
  const int tok = blockIdx.y;
  const int j = blockIdx.x * 256 + threadIdx.x;
  if (j >= p.topk) return;
  // request of this token: the last bi with seq_q[bi] <= tok
  int lo = 0, hi = p.b;  // invariant: seq_q[lo] <= tok < seq_q[hi] for well-formed input
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(p.seq_q + mid) <= tok) lo = mid; else hi = mid;
  }
  const int bi = lo;
  const int q0 = __ldg(p.seq_q + bi), q1 = __ldg(p.seq_q + bi + 1);
  uint32_t out = 0;
  int count = 0;
  if (tok < q0 || tok >= q1) {
    if (j == 0) report_status(p.status, DSV32_STATUS_BAD_INDEX, tok, bi);
  } else if (p.pair && ((tok - q0) & 1)) {
    count = -1;  // second token of a pair
  } else {
    const int s1 = q1 - q0, si = tok - q0;
    const int seq = __ldg(p.act_seq + bi);
    const bool has_b = p.pair && si + 1 < s1;
    // first token (a), second token (b = a + 1 position) of the pair; without pairing only a
    const int len_a = max(seq - s1 + 1 + si, 0), len_b = has_b ? max(seq - s1 + 2 + si, 0) : len_a;
    const int win_a = min(len_a, p.win_size), win_b = min(len_b, p.win_size);
    const int sel_a = p.cmp_dense ? min(len_a / p.cmp_ratio, p.sel_topk)
                                  : min(max(seq / p.cmp_ratio - s1 + 1 + si, 0), p.sel_topk);
    const int sel_b = has_b ? min(len_b / p.cmp_ratio, p.sel_topk) : sel_a;   // pairs only exist with cmp_dense / no index
    const int w_start = len_a - win_a;              // first window position of the union (b's window starts later or equal)
    const int w_len = len_b - w_start;              // union window: [w_start, len_b)
    const int sel_u = max(sel_a, sel_b);
    count = w_len + sel_u;
    if (j < w_len) {
      const int pos = w_start + j;
      const uint32_t mem = (pos < len_a ? 1u : 0u) | ((has_b && pos >= len_b - win_b) ? 2u : 0u);
      const int lb = pos / p.block_size;
      if (lb >= p.max_blocks) {
        report_status(p.status, DSV32_STATUS_BAD_INDEX, tok, pos);
      } else {
        const int pb = __ldg(p.block_table + static_cast<size_t>(bi) * p.max_blocks + lb);
        const long long row = static_cast<long long>(pb) * p.block_size + pos % p.block_size;
        if (pb < 0 || row >= p.rows) report_status(p.status, DSV32_STATUS_BAD_PAGE, tok, pos);
        else out = (static_cast<uint32_t>(row) + 1u) | (mem << 29);
      }
    } else if (j < count) {
      const int e = j - w_len;
      const int idx = (p.cmp_dense || p.topk_idx == nullptr) ? e : __ldg(p.topk_idx + static_cast<size_t>(tok) * p.sel_topk + e);
      const uint32_t mem = (e < sel_a ? 1u : 0u) | ((has_b && e < sel_b) ? 2u : 0u);
      if (idx >= 0) {
        const int lb = idx / p.block_size;
        if (lb >= p.max_blocks2) {
          report_status(p.status, DSV32_STATUS_BAD_INDEX, tok, idx);
        } else {
          const int pb = __ldg(p.block_table2 + static_cast<size_t>(bi) * p.max_blocks2 + lb);
          const long long row = static_cast<long long>(pb) * p.block_size + idx % p.block_size;
          if (pb < 0 || row >= p.rows2) report_status(p.status, DSV32_STATUS_BAD_PAGE, tok, idx);
          else out = (static_cast<uint32_t>(row) + 1u) | (mem << 29) | 0x80000000u;
        }
      }
    }
  }
  p.row_ids[static_cast<size_t>(tok) * p.topk + j] = static_cast<int>(out);
  if (j == 0) p.key_counts[tok] = count;
}

// The same for the operator whose compressed keys come from an index tensor (p.pair == 2): one CTA per token.
// The CTA of the first token of a pair builds the union of both tokens' selections: two bitmaps over the compressed
// positions (shared memory) say which token selected what; the list is the union window, then the first token's
// entries (bit 30 set as well where the second token selected the same position), then the second token's
// entries that the first did not select, compacted in their original order by a block-wide scan (deterministic).
constexpr int kPairBitmapWords = 4096;   // 131,072 compressed positions per request at most

__global__ void __launch_bounds__(256) scfa_pair_ids_kernel(SfaParams p) {
  __shared__ uint32_t bm_a[kPairBitmapWords], bm_b[kPairBitmapWords];
  __shared__ int warp_cnt[8];
  const int tok = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int lo = 0, hi = p.b;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(p.seq_q + mid) <= tok) lo = mid; else hi = mid;
  }
  const int bi = lo;
  const int q0 = __ldg(p.seq_q + bi), q1 = __ldg(p.seq_q + bi + 1);
  int32_t* list = p.row_ids + static_cast<size_t>(tok) * p.topk;
  if (tok < q0 || tok >= q1) {
    if (tid == 0) {
      report_status(p.status, DSV32_STATUS_BAD_INDEX, tok, bi);
      p.key_counts[tok] = 0;
    }
    return;
  }
  const int s1 = q1 - q0, si = tok - q0;
  if (si & 1) {
    if (tid == 0) p.key_counts[tok] = -1;  // second token of a pair
    return;
  }
  const int seq = __ldg(p.act_seq + bi);
  const bool has_b = si + 1 < s1;
  const int len_a = max(seq - s1 + 1 + si, 0), len_b = has_b ? max(seq - s1 + 2 + si, 0) : len_a;
  const int win_a = min(len_a, p.win_size), win_b = min(len_b, p.win_size);
  const int sel_a = min(max(seq / p.cmp_ratio - s1 + 1 + si, 0), p.sel_topk);
  const int sel_b = has_b ? min(max(seq / p.cmp_ratio - s1 + 2 + si, 0), p.sel_topk) : 0;
  const int w_start = len_a - win_a, w_len = len_b - w_start;
  const int cap = p.max_blocks2 * p.block_size;   // compressed positions of a request (<= 32 * kPairBitmapWords)
  auto resolve = [&](int idx, uint32_t mem) -> uint32_t {   // entry of compressed position idx, 0 if it cannot be used
    if (idx < 0) return 0u;
    if (idx >= cap) {
      report_status(p.status, DSV32_STATUS_BAD_INDEX, tok, idx);
      return 0u;
    }
    const int pb = __ldg(p.block_table2 + static_cast<size_t>(bi) * p.max_blocks2 + idx / p.block_size);
    const long long row = static_cast<long long>(pb) * p.block_size + idx % p.block_size;
    if (pb < 0 || row >= p.rows2) {
      report_status(p.status, DSV32_STATUS_BAD_PAGE, tok, idx);
      return 0u;
    }
    return (static_cast<uint32_t>(row) + 1u) | (mem << 29) | 0x80000000u;
  };
  // window
  for (int j = tid; j < w_len; j += 256) {
    const int pos = w_start + j;
    const uint32_t mem = (pos < len_a ? 1u : 0u) | ((has_b && pos >= len_b - win_b) ? 2u : 0u);
    uint32_t out = 0;
    const int lb = pos / p.block_size;
    if (lb >= p.max_blocks) {
      report_status(p.status, DSV32_STATUS_BAD_INDEX, tok, pos);
    } else {
      const int pb = __ldg(p.block_table + static_cast<size_t>(bi) * p.max_blocks + lb);
      const long long row = static_cast<long long>(pb) * p.block_size + pos % p.block_size;
      if (pb < 0 || row >= p.rows) report_status(p.status, DSV32_STATUS_BAD_PAGE, tok, pos);
      else out = (static_cast<uint32_t>(row) + 1u) | (mem << 29);
    }
    list[j] = static_cast<int>(out);
  }
  // bitmaps of both selections
  const int words = (cap + 31) / 32;
  for (int i = tid; i < words; i += 256) { bm_a[i] = 0u; bm_b[i] = 0u; }
  __syncthreads();
  const int32_t* ia = p.topk_idx + static_cast<size_t>(tok) * p.sel_topk;
  const int32_t* ib = ia + p.sel_topk;   // the next token's index row
  for (int e = tid; e < sel_a; e += 256) {
    const int idx = __ldg(ia + e);
    if (idx >= 0 && idx < cap) atomicOr(&bm_a[idx >> 5], 1u << (idx & 31));
  }
  for (int e = tid; e < sel_b; e += 256) {
    const int idx = __ldg(ib + e);
    if (idx >= 0 && idx < cap) atomicOr(&bm_b[idx >> 5], 1u << (idx & 31));
  }
  __syncthreads();
  // the first token's entries, in place
  for (int e = tid; e < sel_a; e += 256) {
    const int idx = __ldg(ia + e);
    const bool in_b = idx >= 0 && idx < cap && ((bm_b[idx >> 5] >> (idx & 31)) & 1u);
    list[w_len + e] = static_cast<int>(resolve(idx, in_b ? 3u : 1u));
  }
  // the second token's entries that the first did not select, compacted in order
  int base = w_len + sel_a;
  for (int e0 = 0; e0 < sel_b; e0 += 256) {
    const int e = e0 + tid;
    int idx = -1;
    if (e < sel_b) idx = __ldg(ib + e);
    const bool take = idx >= 0 && !(idx < cap && ((bm_a[idx >> 5] >> (idx & 31)) & 1u));
    const uint32_t ballot = __ballot_sync(0xffffffffu, take);
    if (lane == 0) warp_cnt[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if (w < warp) before += warp_cnt[w];
      total += warp_cnt[w];
    }
    if (take) list[base + before + __popc(ballot & ((1u << lane) - 1u))] = static_cast<int>(resolve(idx, 2u));
    base += total;
    __syncthreads();
  }
  if (tid == 0) p.key_counts[tok] = base;
}

template <int kMode>
__global__ void __launch_bounds__(kStThreads, 1) sfa_tc_kernel(const __grid_constant__ CUtensorMap qn_map,
                                                               const __grid_constant__ CUtensorMap qr_map,
                                                               SfaParams p) {
  // The swizzled tiles need a 1024-byte aligned base.  The kernel has no static shared memory, so its dynamic
  // window starts on such a boundary; should that ever not hold, the CTA reports it and leaves before any barrier.
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0) report_status(p.status, DSV32_STATUS_INTERNAL, 40, smem_u32(smem));
    return;
  }
  unsigned char* k_s = smem;
  unsigned char* q_s = smem + kStOffQ;
  int* valid_s = reinterpret_cast<int*>(smem + kStOffValid);
  int* ring_s = reinterpret_cast<int*>(smem + kStOffRing);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStOffBars);
  uint64_t* full_bar = bars;         // [2] producers -> MMA            (one arrival per producer warp)
  uint64_t* sfull_bar = bars + 2;    // [2] S complete -> softmax       (tcgen05.commit)
  uint64_t* pready_bar = bars + 4;   // [2] P stored -> MMA             (128 thread arrivals)
  uint64_t* pvdone_bar = bars + 6;   // [2] PV complete -> producers / MMA / softmax (tcgen05.commit)
  uint64_t* q_bar = bars + 8;        //     Q in place -> MMA           (TMA tx + 128 thread arrivals)
  uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(smem + kStOffTmem);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int half = blockIdx.x;  // which 256 value dims
  const int tok = blockIdx.y;
  const int split = blockIdx.z;
  constexpr bool kBf16 = kMode != kModeInt8;
  constexpr bool kCompress = kMode == kModeCompress;
  constexpr int kSteps = kCompress ? 32 : 36;  // 16-dim MMA steps of one S tile (no rope dims in mode 2)
  int cnt;
  int live_rows = p.nq;   // lanes (query rows) of the M = 128 tile that belong to this CTA's token(s)
  if constexpr (kCompress) {
    const int raw = p.key_counts[tok];
    if (raw < 0) return;  // second token of a pair: its heads are lanes 64.. of the partner's CTA
    cnt = min(raw, p.topk);
    if (p.pair && tok + 1 < p.t_total && p.key_counts[tok + 1] < 0) live_rows = 2 * p.nq;
  } else {
    const int bi = tok / p.s1, si = tok % p.s1;
    cnt = min(max(p.act_seq[bi] - p.s1 + 1 + si, 0), p.topk);
  }
  const int per = (((cnt + p.splits - 1) / p.splits) + kStTile - 1) / kStTile * kStTile;
  const int k_lo = split * per;
  const int k_hi = min(cnt, k_lo + per);
  const int ntiles = (k_hi > k_lo) ? (k_hi - k_lo + kStTile - 1) / kStTile : 0;

  if (ntiles == 0) {  // nothing to attend to: zero row block (uniform for the CTA)
    for (int i = tid; i < 128 * 64; i += kStThreads) {
      const int h = i >> 6, c = i & 63;  // 64 chunks of 4 dims
      if (h >= live_rows) continue;
      if (p.splits == 1) {
        *reinterpret_cast<uint2*>(p.out + (static_cast<size_t>(tok) * p.nq + h) * kKvLora + half * 256 + c * 4) =
            make_uint2(0u, 0u);
      } else {
        const size_t prow = (static_cast<size_t>(tok) * p.splits + split) * p.nq + h;
        *reinterpret_cast<float4*>(p.part_o + prow * kKvLora + half * 256 + c * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
        if (half == 0 && c == 0) p.part_lse[prow] = -INFINITY;
      }
    }
    return;
  }

  // ---- setup -------------------------------------------------------------------------------------------
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&qn_map);
      tma_prefetch_desc(&qr_map);
      mbar_init(&full_bar[0], kStProducerWarps);
      mbar_init(&full_bar[1], kStProducerWarps);
      mbar_init(&sfull_bar[0], 1);
      mbar_init(&sfull_bar[1], 1);
      mbar_init(&pready_bar[0], 128);
      mbar_init(&pready_bar[1], 128);
      mbar_init(&pvdone_bar[0], 1);
      mbar_init(&pvdone_bar[1], 1);
      mbar_init(q_bar, 129);
      mbar_fence_init();
    }
    __syncwarp();
    tmem_alloc(tmem_ptr_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_s;

  if (warp == 0) {
    // ================================ MMA issuer ==========================================================
    // The whole warp runs the loop (uniform operands, no divergent region); lane 0 issues.
    const bool leader = lane == 0;
    if (leader) {
      // Q dims 256..575 -> shared memory (TMA, 128-byte swizzle): nope chunks 4..7 and the rope chunk
      mbar_arrive_expect_tx(q_bar, kCompress ? 4 * kStQChunkBytes : kStQsBytes);
      for (int c = 0; c < 4; ++c)
        tma_load_2d(q_s + c * kStQChunkBytes, &qn_map, (4 + c) * 128, tok * p.nq, q_bar);
      if constexpr (!kCompress) tma_load_2d(q_s + 4 * kStQChunkBytes, &qr_map, 0, tok * p.nq, q_bar);
    }
    __syncwarp();
    constexpr uint32_t idesc_s = umma_idesc_bf16(128, kStTile, false, false);
    bool ok = __all_sync(0xffffffffu, mbar_wait(q_bar, 0, p.status, 10));
    const uint32_t tbase = __shfl_sync(0xffffffffu, tmem_base, 0);

    // Descriptors are assembled from precomputed 32-bit halves: per MMA only the start-address field moves.
    constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, 128-byte swizzle
    auto desc = [](uint32_t lo) -> uint64_t {
      uint64_t d;
      asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(kDescHi));
      return d;
    };
    const uint32_t q_lo = ((smem_u32(q_s) >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t stage0_lo = ((smem_u32(k_s) >> 4) & 0x3FFFu) | (1u << 16);   // K-major (S)

    // This warp issues S = Q K^T of every tile; PV is issued by a warp of the softmax group as soon as
    // P is stored, so that it never waits behind the issue of the next S (the issuer blocks while the
    // tensor-core queue is full).  MMAs of both issuers execute in the order they enter the queue; S(i+2),
    // which overwrites the buffer PV(i) reads P from, is only issued after the producers have seen PV(i)
    // complete (they refill its K stage before signalling `full`).
    for (int i = 0; ok && i < ntiles; ++i) {
      const int s = i & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], (i >> 1) & 1, p.status, 11));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d = tbase + kColS + s * kStTile;
      const uint32_t klo = stage0_lo + s * (kStStageBytes >> 4);
#pragma unroll
      for (int ks = 0; ks < 16; ++ks)  // Q dims 0..255 from tensor memory
        umma_f16_ts_if(leader, d, tbase + kColQ + ks * 8, desc(klo + (((ks >> 2) * kStChunkBytes + (ks & 3) * 32) >> 4)),
                       idesc_s, ks > 0 ? 1u : 0u);
#pragma unroll
      for (int ks = 16; ks < kSteps; ++ks)  // Q dims 256..575 (256..511 in mode 2) from shared memory
        umma_f16_ss_if(leader, d, desc(q_lo + ((((ks >> 2) - 4) * kStQChunkBytes + (ks & 3) * 32) >> 4)),
                       desc(klo + (((ks >> 2) * kStChunkBytes + (ks & 3) * 32) >> 4)), idesc_s, 1u);
      umma_commit_if(leader, &sfull_bar[s]);
    }
  } else if (warp <= 4) {
    // ================================ softmax / epilogue ==================================================
    const int quarter = warp & 3;
    const int head = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    // Q dims 0..255 of this head -> tensor memory as bf16 pairs
    {
      const uint4* qrow = reinterpret_cast<const uint4*>(p.q_nope + (static_cast<size_t>(tok) * p.nq + head) * kKvLora);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 v = make_uint4(0u, 0u, 0u, 0u);
          if (head < live_rows) v = __ldg(qrow + c * 8 + j);
          r[4 * j] = v.x; r[4 * j + 1] = v.y; r[4 * j + 2] = v.z; r[4 * j + 3] = v.w;
        }
        tmem_st_32x32b_x32(tmem_base + lane_addr + kColQ + c * 32, r);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(q_bar);
    }
    const float sc2 = p.scale * 1.4426950408889634f;  // softmax scale in log2 units
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int i = 0; ok && i < ntiles; ++i) {
      const int s = i & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&sfull_bar[s], (i >> 1) & 1, p.status, 20))) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + lane_addr + kColS + s * kStTile;
      // Masking is only needed when the tile holds an invalid key (tail of the list, or a -1 entry).
      // A flag holds membership bits: bit 0 = a key of the token in lanes 0..63 (the only token unless two share
      // the CTA), bit 1 = a key of the token in lanes 64..127.
      const int* vm = valid_s + s * kStTile;
      const int hb = !kCompress ? 1 : (head < p.nq ? 1 : (head < live_rows ? 2 : 3));   // idle lanes take every key
      // The shortcut must hold for every lane of the warp: with fewer than 32 heads per token a warp holds heads
      // of both tokens (and idle lanes), so the flags are tested against the bits of all of them.
      const uint32_t need_bits = __reduce_or_sync(0xffffffffu, static_cast<uint32_t>(hb == 3 ? 0 : hb));
      const bool all_valid = __all_sync(0xffffffffu, (static_cast<uint32_t>(vm[lane]) & need_bits) == need_bits &&
                                                         (static_cast<uint32_t>(vm[32 + lane]) & need_bits) == need_bits);
      // The 64 scores of a row are read from tensor memory twice, 32 at a time -- once for the row maximum, once
      // for the exponentials -- instead of being held in 64 registers: tensor-memory loads are cheap, and the
      // register file is what limits the number of gather warps.
      uint32_t r[32];
      float m_raw = -INFINITY;  // row maximum of the raw scores (the softmax scale is positive)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        tmem_ld_32x32b_x32(s_addr + 32 * h, r);
        tmem_ld_wait();
        if (!all_valid) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (!(vm[32 * h + j] & hb)) r[j] = 0xff800000u;       // -inf
        }
#pragma unroll
        for (int j = 0; j < 32; j += 2) m_raw = fmaxf(m_raw, fmaxf(__uint_as_float(r[j]), __uint_as_float(r[j + 1])));
      }
      const float m_tile = m_raw * sc2;
      const bool need = m_tile > m_run + kRescaleThreshold;  // also true on the first non-empty tile (m_run = -inf)
      if (__any_sync(0xffffffffu, need)) {
        const float m_new = need ? m_tile : m_run;
        const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_run - m_new);  // m_run = -inf -> 0
        l_run *= alpha;
        m_run = m_new;
        if (i > 0) {  // O holds data: scale this head's row (the previous PV must have finished)
          if (!__all_sync(0xffffffffu, mbar_wait(&pvdone_bar[(i - 1) & 1], ((i - 1) >> 1) & 1, p.status, 21))) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(tmem_base + lane_addr + kColO + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st_32x32b_x32(tmem_base + lane_addr + kColO + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
      // p = 2^(s*scale*log2e - m): packed fp32 arithmetic (two keys per FMA and per addition), one ex2 per key
      const uint64_t sc22 = f2_pack(__float_as_uint(sc2), __float_as_uint(sc2));
      const uint64_t negm2 = f2_pack(__float_as_uint(neg_m), __float_as_uint(neg_m));
      uint64_t lsum_a = 0ull, lsum_b = 0ull;   // two pairs of partial row sums
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        tmem_ld_32x32b_x32(s_addr + 32 * h, r);
        tmem_ld_wait();
        if (!all_valid) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (!(vm[32 * h + j] & hb)) r[j] = 0xff800000u;
        }
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float p0, p1, p2, p3;
          f2_unpack(f2_fma(f2_pack(r[j], r[j + 1]), sc22, negm2), p0, p1);
          f2_unpack(f2_fma(f2_pack(r[j + 2], r[j + 3]), sc22, negm2), p2, p3);
          p0 = fast_exp2(p0);
          p1 = fast_exp2(p1);
          p2 = fast_exp2(p2);
          p3 = fast_exp2(p3);
          lsum_a = f2_add(lsum_a, f2_pack(__float_as_uint(p0), __float_as_uint(p1)));
          lsum_b = f2_add(lsum_b, f2_pack(__float_as_uint(p2), __float_as_uint(p3)));
          pk[j >> 1] = pack_bf16x2(p0, p1);
          pk[(j >> 1) + 1] = pack_bf16x2(p2, p3);
        }
        // P (32 keys as 16 bf16 pairs) over the first half of the S buffer: columns 16h .. 16h+15 held scores
        // that have been consumed (h = 1) or are this pass's own (h = 0); columns 32.. are still intact for h = 1
        tmem_st_32x32b_x16(s_addr + 16 * h, pk);
      }
      {
        float a0, a1, b0, b1;
        f2_unpack(lsum_a, a0, a1);
        f2_unpack(lsum_b, b0, b1);
        l_run += (a0 + a1) + (b0 + b1);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&pready_bar[s]);
      if (warp == 1) {  // second MMA issuer: PV of this tile, as soon as all four softmax warps have stored P
        // (the whole warp waits and computes the uniform operands; lane 0 issues)
        if (!__all_sync(0xffffffffu, mbar_wait(&pready_bar[s], (i >> 1) & 1, p.status, 13))) { ok = false; break; }
        constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 256, false, true);
        constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, 128-byte swizzle
        const uint32_t tbase = __shfl_sync(0xffffffffu, tmem_base, 0);
        const uint32_t a = smem_u32(k_s) + s * kStStageBytes;
        const uint32_t vlo = (((a + 4 * half * kStChunkBytes) >> 4) & 0x3FFFu) | ((kStChunkBytes >> 4) << 16);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {  // 16 keys per instruction; V = this CTA's four 64-dim chunks, MN-major
          uint64_t d;
          asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(vlo + ((kk * 2048) >> 4)), "r"(kDescHi));
          umma_f16_ts_if(lane == 0, tbase + kColO, tbase + kColS + s * kStTile + kk * 8, d, idesc_pv,
                         (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit_if(lane == 0, &pvdone_bar[s]);
      }
    }
    // ---- epilogue: O / l -> bf16 (or fp32 partial + log-sum-exp for a key split) -----------------------------
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&pvdone_bar[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1, p.status, 22));
    if (ok) {
      tc_fence_after();
      if constexpr (kCompress) {  // the sink joins the denominator only: + exp(sink - max), in the units of m_run
        if (head < live_rows && m_run != -INFINITY)
          l_run += exp2f(fmaf(__ldg(p.sinks + (head >= p.nq ? head - p.nq : head)), 1.4426950408889634f, -m_run));
      }
      const float inv = (l_run > 0.f) ? 1.f / l_run : 0.f;
      // tcgen05.ld is a warp-wide instruction: a warp whose lanes are partly idle (a head count that is not a
      // multiple of 32) runs the loops below as a whole and only the stores are per lane.
      const bool live = head < live_rows;
      if (quarter * 32 >= live_rows) {
        // idle warp of the M = 128 tile: nothing to store
      } else if (p.splits == 1) {
        __nv_bfloat16* orow = p.out + (static_cast<size_t>(tok) * p.nq + head) * kKvLora + half * 256;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + kColO + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
            if (live) *reinterpret_cast<uint4*>(orow + c * 32 + j) = v;
          }
        }
      } else {
        const size_t prow = (static_cast<size_t>(tok) * p.splits + split) * p.nq + head;
        float* orow = p.part_o + prow * kKvLora + half * 256;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + kColO + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            if (live)
              *reinterpret_cast<float4*>(orow + c * 32 + j) =
                  make_float4(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv,
                              __uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
        }
        if (half == 0 && live)
          p.part_lse[prow] = (l_run > 0.f) ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      }
    }
  } else {
    // ================================ gather + dequantise producers ========================================
    // 512 threads: thread (gkey, gpart) owns the 16-byte column gpart of every 128-byte group of key row gkey of
    // each tile.  Raw rows travel global -> registers TWO tiles ahead of their use (two register sets that
    // alternate by tile parity; one set for the bf16 caches, whose rows are twice as wide), are dequantised and
    // stored into the swizzled K stage once the MMAs of the tile two back have released it.
    const int ptid = tid - 160;            // 0..511
    const int gkey = ptid >> 3, gpart = ptid & 7;
    const int pw = warp - 5;               // this warp's rows of a tile: 4*pw .. 4*pw + 3
#ifndef DSV32_SFA_DEPTH
#define DSV32_SFA_DEPTH 1
#endif
    constexpr int kDepth = kBf16 ? 1 : DSV32_SFA_DEPTH;  // register sets = tiles of raw rows in flight
    // The cache row of every selected key was resolved by the pre-pass (row + 1, 0 = none).  Row ids travel
    // global -> shared memory with 4-byte cp.async six tiles ahead (ring of eight tiles per warp), so that the
    // L2 prefetch (four tiles ahead) and the loads (kDepth tiles ahead) find them in place.
    int* ring = ring_s + pw * (kStRingTiles * 4);
    const int32_t* ids_row = p.row_ids + static_cast<size_t>(tok) * p.topk;
    auto fetch_ids = [&](int tile) {
      if (lane < 4) {
        const int j = k_lo + tile * kStTile + 4 * pw + lane;
        const bool in = tile < ntiles && j < k_hi;
        const uint32_t dst = smem_u32(ring + (tile & (kStRingTiles - 1)) * 4 + lane);
        const int32_t* src = ids_row + (in ? j : 0);
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(in ? 4 : 0) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // Mode 2 keeps the pre-pass entry as it is (bit 31 = row of the second cache, low bits = row + 1, 0 = none);
    // the other modes turn it into the row, -1 = none.
    auto row_of = [&](int tile) -> long long {
      const int v = ring[(tile & (kStRingTiles - 1)) * 4 + (lane >> 3)];
      if constexpr (kCompress) return static_cast<long long>(v);
      else return static_cast<long long>(v) - 1;
    };
    const unsigned char* nope_b = reinterpret_cast<const unsigned char*>(p.k_nope);
    const unsigned char* rope_b = reinterpret_cast<const unsigned char*>(p.k_rope);
    const unsigned char* scale_b = reinterpret_cast<const unsigned char*>(p.k_scales);
    const bool fused_rows = p.nope_stride == p.rope_stride;  // one 656-byte row holds all three parts
    auto l2_prefetch = [&](long long row) {  // the 128-byte lines of a row, one per thread column
      if constexpr (kCompress) {
        const int v = static_cast<int>(row);
        if (v != 0) {
          const unsigned char* base = v < 0 ? reinterpret_cast<const unsigned char*>(p.k_nope2) : nope_b;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(base + static_cast<long long>((v & 0x1fffffff) - 1) * 1024 + gpart * 128));
        }
        return;
      }
      if (row < 0) return;
      const void* a = nullptr;
      if (fused_rows) {
        if (gpart < 6) a = nope_b + row * p.nope_stride + gpart * 128;  // 656 bytes touch at most six lines
      } else if constexpr (kBf16) {
        a = nope_b + row * p.nope_stride + gpart * 128;                 // eight lines of bf16 latent dims
        if (gpart == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(rope_b + row * p.rope_stride));
      } else if (gpart < 4) {
        a = nope_b + row * p.nope_stride + gpart * 128;
      } else if (gpart == 4) {
        a = rope_b + row * p.rope_stride;
      } else if (gpart == 5) {
        a = scale_b + row * p.scale_stride;
      }
      if (a != nullptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
    };
    // Register layout of a row: nope[0..1] / sc.x,.y = this CTA's own value dims (128-dim groups 2*half, 2*half+1),
    // nope[2..3] / sc.z,.w = the other half's.  The runtime half only enters the addresses.
    const int q_own = 2 * half, q_oth = 2 * (half ^ 1);
    using StPrefetch = StPrefetchT<kBf16>;
    auto issue_loads = [&](long long row, StPrefetch& pf) {
      const int4* src;
      if constexpr (kCompress) {
        const int v = static_cast<int>(row);
        pf.valid = v != 0;
        const unsigned char* base = v < 0 ? reinterpret_cast<const unsigned char*>(p.k_nope2) : nope_b;
        src = reinterpret_cast<const int4*>(base + static_cast<long long>((v & 0x1fffffff) - 1) * 1024);
      } else {
        pf.valid = row >= 0;
        src = reinterpret_cast<const int4*>(nope_b + row * p.nope_stride);
      }
      if (pf.valid) {
        if constexpr (kBf16) {  // this thread's 16 dims of a 128-dim group are two consecutive 16-byte units
          pf.nope[0] = __ldg(src + 2 * gpart + 16 * q_own);
          pf.nope[1] = __ldg(src + 2 * gpart + 16 * q_own + 1);
          pf.nope[2] = __ldg(src + 2 * gpart + 16 * (q_own + 1));
          pf.nope[3] = __ldg(src + 2 * gpart + 16 * (q_own + 1) + 1);
          pf.nope[4] = __ldg(src + 2 * gpart + 16 * q_oth);
          pf.nope[5] = __ldg(src + 2 * gpart + 16 * q_oth + 1);
          pf.nope[6] = __ldg(src + 2 * gpart + 16 * (q_oth + 1));
          pf.nope[7] = __ldg(src + 2 * gpart + 16 * (q_oth + 1) + 1);
          if constexpr (!kCompress) pf.rope = __ldg(reinterpret_cast<const int4*>(rope_b + row * p.rope_stride) + gpart);
        } else {
          pf.nope[0] = __ldg(src + gpart + 8 * q_own);
          pf.nope[1] = __ldg(src + gpart + 8 * (q_own + 1));
          pf.nope[2] = __ldg(src + gpart + 8 * q_oth);
          pf.nope[3] = __ldg(src + gpart + 8 * (q_oth + 1));
          pf.rope = __ldg(reinterpret_cast<const int4*>(rope_b + row * p.rope_stride) + gpart);
          const float* sc_row = reinterpret_cast<const float*>(scale_b + row * p.scale_stride);
          const float2 so = __ldg(reinterpret_cast<const float2*>(sc_row + q_own));
          const float2 sx = __ldg(reinterpret_cast<const float2*>(sc_row + q_oth));
          pf.sc = make_float4(so.x, so.y, sx.x, sx.y);
        }
      }
    };
    // This thread's two 16-byte units of a 128-byte line of its key row, 128-byte swizzle; the row is the same
    // in every tile, so the offsets inside a stage are fixed.
    const int u0 = (gpart & 3) * 2;
    const uint32_t off_lo = static_cast<uint32_t>(gkey * 128 + ((u0 ^ (gkey & 7)) << 4));
    const uint32_t off_hi = static_cast<uint32_t>(gkey * 128 + (((u0 + 1) ^ (gkey & 7)) << 4));
    const uint32_t off_rope = static_cast<uint32_t>(8 * kStChunkBytes + gkey * 128 + ((gpart ^ (gkey & 7)) << 4));
    // group k of the row held in pf (k = 0, 1 -> this CTA's own value dims, 2, 3 -> the other half's) as bf16
    auto make_group = [&](int k, const StPrefetch& pf, uint4& lo, uint4& hi) {
      lo = make_uint4(0, 0, 0, 0);
      hi = lo;
      if constexpr (kBf16) {
        if (pf.valid) {
          const int4 a = pf.nope[2 * k], b = pf.nope[2 * k + 1];
          lo = make_uint4(a.x, a.y, a.z, a.w);
          hi = make_uint4(b.x, b.y, b.z, b.w);
        }
      } else {
        const float sc = k == 0 ? pf.sc.x : k == 1 ? pf.sc.y : k == 2 ? pf.sc.z : pf.sc.w;
        if (pf.valid) st_dequant16(pf.nope[k], sc, lo, hi);
      }
    };
    // ... into the two 16-byte units this thread owns of 128-dim group q
    auto store_group = [&](unsigned char* stage, int q, const uint4& lo, const uint4& hi) {
      unsigned char* chunk = stage + (2 * q + (gpart >> 2)) * kStChunkBytes;  // 64-dim chunk 0..7
      *reinterpret_cast<uint4*>(chunk + off_lo) = lo;
      *reinterpret_cast<uint4*>(chunk + off_hi) = hi;
    };
    // The chunks that only S reads (the other half's value dims and the rope dims)
    auto commit_other = [&](int tile, const StPrefetch& pf) {
      unsigned char* stage = k_s + (tile & 1) * kStStageBytes;
      uint4 lo, hi;
      make_group(2, pf, lo, hi);
      store_group(stage, q_oth, lo, hi);
      make_group(3, pf, lo, hi);
      store_group(stage, q_oth + 1, lo, hi);
      if constexpr (!kCompress) {
        const int4 v = pf.valid ? pf.rope : make_int4(0, 0, 0, 0);
        *reinterpret_cast<int4*>(stage + off_rope) = v;
      }
    };
    // One tile: refill its stage from `pf`, then start the loads of the tile kDepth ahead into the same registers.
    auto do_tile = [&](int i, StPrefetch& pf) -> bool {
      const int s = i & 1;
      // Once S of tile i-2 has completed, every chunk of the stage except this CTA's own value chunks is free
      // (both waits pass at once for i < 2): that part of the refill runs under the softmax and PV of tile i-2.
      const uint32_t prev = ((i >> 1) & 1) ^ 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&sfull_bar[s], prev, p.status, 30))) return false;
      commit_other(i, pf);
      // The chunks that PV reads as V (this CTA's own value dims) are free once PV of tile i-2 has completed.  That
      // wait is on the critical path (PV(i-2) -> refill -> S(i)), so the rows are dequantised before it and only
      // the stores (and the validity flags the softmax reads) come after it.
      uint4 own_lo[2], own_hi[2];
      make_group(0, pf, own_lo[0], own_hi[0]);
      make_group(1, pf, own_lo[1], own_hi[1]);
      if (!__all_sync(0xffffffffu, mbar_wait(&pvdone_bar[s], prev, p.status, 31))) return false;
      {
        unsigned char* stage = k_s + s * kStStageBytes;
        store_group(stage, q_own, own_lo[0], own_hi[0]);
        store_group(stage, q_own + 1, own_lo[1], own_hi[1]);
        if (gpart == 0) {  // membership bits for the softmax; the tile's ids are still in the ring (mode 2 keeps them raw)
          if constexpr (kCompress) valid_s[s * kStTile + gkey] = (static_cast<int>(row_of(i)) >> 29) & 3;
          else valid_s[s * kStTile + gkey] = pf.valid ? 1 : 0;
        }
      }
      fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor-core (async) proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_bar[s]);
      // The loads of the tile kDepth ahead go out after the hand-over: issued before the wait above they hold the
      // warp at the load/store unit (its miss queue is the scarce resource) and the hand-over comes later (measured).
      fetch_ids(i + 6);
      asm volatile("cp.async.wait_group 2;" ::: "memory");   // ids up to tile i + 4 have landed
      __syncwarp();
      if (i + kDepth < ntiles) issue_loads(row_of(i + kDepth), pf);
      if (i + 4 < ntiles) l2_prefetch(row_of(i + 4));
      return true;
    };

    StPrefetch pfA, pfB;
    for (int tl = 0; tl < 6; ++tl) fetch_ids(tl);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    issue_loads(row_of(0), pfA);
    if constexpr (kDepth == 2) {
      if (1 < ntiles) issue_loads(row_of(1), pfB);
      else pfB.valid = false;
    }
    for (int tl = kDepth; tl < 4; ++tl)
      if (tl < ntiles) l2_prefetch(row_of(tl));
    for (int i = 0; i < ntiles; i += 2) {
      if (!do_tile(i, pfA)) break;
      if (i + 1 < ntiles && !do_tile(i + 1, kDepth == 2 ? pfB : pfA)) break;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");   // no row-id copy may still be in flight at exit
  }

  // ---- teardown ------------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int launch_sfa_tc(const SfaParams& p, cudaStream_t stream) {
  const int t = p.compress ? p.t_total : p.b * p.s1;
  if (t <= 0) return DSV32_OK;
  if (p.nq < 1 || p.nq > 128) {
    set_error("sfa: n_q=%d must be in [1, 128] (the heads of a token are the rows of one M = 128 tile)", p.nq);
    return DSV32_ERR_UNSUPPORTED;
  }
  if (p.compress && p.splits != 1) {
    set_error("sfa: the compress variant runs without a key split");
    return DSV32_ERR_UNSUPPORTED;
  }
  CUtensorMap qn_map, qr_map;
  int rc = make_tensor_map_2d_u8(&qn_map, p.q_nope, static_cast<uint64_t>(t) * p.nq, kKvLora * 2, 128, 128);
  if (rc != DSV32_OK) return rc;
  if (p.compress) {
    qr_map = qn_map;  // no rope part: the second map is never used
  } else {
    rc = make_tensor_map_2d_u8(&qr_map, p.q_rope, static_cast<uint64_t>(t) * p.nq, kRopeDim * 2, 128, 128);
    if (rc != DSV32_OK) return rc;
  }
  cudaFuncSetAttribute(sfa_tc_kernel<kModeInt8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStSmemBytes);
  cudaFuncSetAttribute(sfa_tc_kernel<kModeBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStSmemBytes);
  cudaFuncSetAttribute(sfa_tc_kernel<kModeCompress>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStSmemBytes);
  if (p.compress && (p.rows > 0x1ffffffeLL || p.rows2 > 0x1ffffffeLL)) {
    set_error("sfa: the compress variant addresses at most 2^29-2 rows per cache (got %lld / %lld)",
              static_cast<long long>(p.rows), static_cast<long long>(p.rows2));
    return DSV32_ERR_UNSUPPORTED;
  }
  if (p.pair && p.nq > 64) {
    set_error("sfa: two tokens per CTA need n_q <= 64 (got %d)", p.nq);
    return DSV32_ERR_UNSUPPORTED;
  }
  if (p.rows > 0x7ffffffeLL || (p.compress && p.rows2 > 0x7ffffffeLL)) {
    set_error("sfa: the tcgen05 kernel addresses at most 2^31-2 cache rows (got %lld)", static_cast<long long>(p.rows));
    return DSV32_ERR_UNSUPPORTED;
  }
  if (p.compress && p.pair == 2) {
    scfa_pair_ids_kernel<<<t, 256, 0, stream>>>(p);
    count_launch();
    rc = check_launch("scfa_pair_ids_kernel");
  } else if (p.compress) {
    scfa_row_ids_kernel<<<dim3((p.topk + 255) / 256, t), 256, 0, stream>>>(p);
    count_launch();
    rc = check_launch("scfa_row_ids_kernel");
  } else {
    sfa_row_ids_kernel<<<dim3((p.topk + 255) / 256, t), 256, 0, stream>>>(p);
    count_launch();
    rc = check_launch("sfa_row_ids_kernel");
  }
  if (rc != DSV32_OK) return rc;
  dim3 grid(2, t, p.splits);
  if (p.compress) sfa_tc_kernel<kModeCompress><<<grid, kStThreads, kStSmemBytes, stream>>>(qn_map, qr_map, p);
  else if (p.kn_bf16) sfa_tc_kernel<kModeBf16><<<grid, kStThreads, kStSmemBytes, stream>>>(qn_map, qr_map, p);
  else sfa_tc_kernel<kModeInt8><<<grid, kStThreads, kStSmemBytes, stream>>>(qn_map, qr_map, p);
  count_launch();
  rc = check_launch("sfa_tc_kernel");
  if (rc == DSV32_OK && p.splits > 1) rc = launch_sfa_combine(p, stream);
  return rc;
}

}  // namespace dsv32

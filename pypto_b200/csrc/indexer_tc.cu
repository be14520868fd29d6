// Lightning-indexer scores on the 5th-generation tensor cores (tcgen05, int8 -> int32 in tensor memory).
//
//   D[key, (token, head)] = K_block[128 keys x 128] . Q[(token, head) x 128]^T          (kind::i8, exact)
//   score[token, key]     = ( sum_h ws[token,h] * fp16( relu(D) * 2^-11 ) ) * k_scale[key]
//
// Keys are the M dimension: a 128-key cache block is one 16 KB TMA tile (128-byte swizzle) and one
// M=128 MMA tile, and every epilogue thread owns one key with all its (token, head) columns, so the head
// reduction is an fp32 sum in registers (four interleaved partial sums, fixed order), with no shuffles.
// Follows models/deepseek_v32_exp/lightning_indexer_quant_impl.py:114-177 (golden:
// deepseekv32_lightning_indexer_quant.py:209-242).
//
// Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer + tensor-memory owner, then the epilogue warps
// (one TMEM lane quarter each; with two or more tokens per CTA there are eight of them and the two warps of
// a quarter split the tokens, which doubles the warps available to hide latency).  Key blocks go through a 4-stage shared-memory ring;
// the accumulator is double-buffered in tensor memory so the epilogue of block i overlaps the MMA of i+1.
#include <mutex>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace dsv32 {

constexpr int kTcBlocksPerCta = 64;  // upper bound; the launcher picks the actual count per call
constexpr int kKeyTileBytes = 128 * 128;

// Shared memory of one CTA (offsets from the 1024-byte aligned base).  The ring of key blocks is what keeps
// bytes in flight: with up to two tokens the query tile is 16 KB and five stages fit twice per SM.
template <int TOK>
struct TcSmemLayout {
  static constexpr int stages = TOK <= 2 ? 5 : 4;
  static constexpr int keys = 0;                               // stages x 16 KB
  static constexpr int q = stages * kKeyTileBytes;             // 64 * TOK rows x 128 B
  static constexpr int ws = q + 64 * TOK * 128;                // 64 * TOK fp16 weights (1 KB reserved)
  static constexpr int phys = ws + 256 * 4;                    // kTcBlocksPerCta ints
  static constexpr int bars = phys + ((kTcBlocksPerCta * 4 + 7) / 8) * 8;  // 8-byte aligned
  static constexpr int nbars = 2 * stages + 4 + 1;
  static constexpr int tmem_ptr = bars + nbars * 8;
  static constexpr int total = tmem_ptr + 16;
  static constexpr size_t bytes = total + 1024;                // slack for manual 1024-byte alignment
  static_assert(bars % 8 == 0 && q % 1024 == 0, "shared-memory layout alignment");
};

template <int TOK>
struct TcShape {
  static constexpr int kEpilogueWarps = TOK >= 2 ? 8 : 4;
  static constexpr int kThreads = 64 + 32 * kEpilogueWarps;
  static constexpr int kTokPerWarp = TOK / (kEpilogueWarps / 4);  // tokens handled by one epilogue warp
};

template <int TOK>
__global__ void __launch_bounds__(TcShape<TOK>::kThreads, 2) indexer_scores_tc_kernel(const __grid_constant__ CUtensorMap key_map,
                                                                      const __grid_constant__ CUtensorMap q_map,
                                                                      IndexerParams p) {
  constexpr int N = 64 * TOK;
  constexpr int kEpThreads = 32 * TcShape<TOK>::kEpilogueWarps;
  constexpr int TPW = TcShape<TOK>::kTokPerWarp;
  constexpr uint32_t kTmemCols = 2 * N < 32 ? 32 : 2 * N;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using Lay = TcSmemLayout<TOK>;
  constexpr int kTcStages = Lay::stages;
  unsigned char* k_s = smem + Lay::keys;
  unsigned char* q_s = smem + Lay::q;
  uint32_t* ws_s = reinterpret_cast<uint32_t*>(smem + Lay::ws);  // fp16 pairs
  int* phys_s = reinterpret_cast<int*>(smem + Lay::phys);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Lay::bars);
  uint64_t* full_bar = bars;                       // [kTcStages]
  uint64_t* empty_bar = bars + kTcStages;          // [kTcStages]
  uint64_t* tfull_bar = bars + 2 * kTcStages;      // [2]
  uint64_t* tempty_bar = bars + 2 * kTcStages + 2; // [2]
  uint64_t* q_bar = bars + 2 * kTcStages + 4;
  uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(smem + Lay::tmem_ptr);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = blockIdx.y;
  const int tok0 = blockIdx.z * TOK;
  const int ntok = min(TOK, p.s1 - tok0);
  const int bs = 128;
  // A sequence length beyond what the request's page-table row can describe is reported and clamped: nothing is
  // read past the row of the page table or written past the row of the score buffer.
  int L = p.act_seq[b];
  if (L > p.max_blocks * bs) {
    if (threadIdx.x == 0 && blockIdx.x == 0) report_status(p.status, DSV32_STATUS_BAD_INDEX, b, static_cast<uint32_t>(L));
    L = p.max_blocks * bs;
  }
  const int hi = min(L, p.key_end);
  const int blk_begin = p.key_begin / bs + blockIdx.x * p.blocks_per_cta;
  const int blk_end = min(blk_begin + p.blocks_per_cta, (hi + bs - 1) / bs);
  if (blk_begin >= blk_end || hi <= p.key_begin) return;  // uniform for the CTA
  const int nblk = blk_end - blk_begin;
  const size_t row0 = static_cast<size_t>(b) * p.s1 + tok0;

  // ---- setup ----------------------------------------------------------------------------------------
  if (warp == 0) {
    for (int j = lane; j < kTcBlocksPerCta; j += 32) {
      int phys = 0;
      if (j < nblk) {
        phys = p.block_table[static_cast<size_t>(b) * p.max_blocks + blk_begin + j];
        if (phys < 0 || phys >= p.num_blocks) {
          report_status(p.status, DSV32_STATUS_BAD_PAGE, b, blk_begin + j);
          phys = 0;
        }
      }
      phys_s[j] = phys;
    }
    if (lane == 0) {
      tma_prefetch_desc(&key_map);
      tma_prefetch_desc(&q_map);
      for (int i = 0; i < kTcStages; ++i) {
        mbar_init(&full_bar[i], 1);
        mbar_init(&empty_bar[i], 1);
      }
      mbar_init(&tfull_bar[0], 1);
      mbar_init(&tfull_bar[1], 1);
      mbar_init(&tempty_bar[0], kEpThreads);
      mbar_init(&tempty_bar[1], kEpThreads);
      mbar_init(q_bar, 1);
      mbar_fence_init();
    }
  } else if (warp == 1) {
    tmem_alloc(tmem_ptr_s, kTmemCols);
    tmem_relinquish();
  } else {
    __half* ws_h = reinterpret_cast<__half*>(ws_s);  // ws = fp16(q_scale * weight), one per (token, head)
    for (int i = tid - 64; i < N; i += kEpThreads)
      ws_h[i] = (i < ntok * 64) ? __hmul(p.q_scale[row0 * 64 + i], p.weight[row0 * 64 + i]) : __float2half(0.f);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_s;

  if (warp == 0) {
    // ---- TMA producer ----------------------------------------------------------------------------------
    if (lane == 0) {
      // the key cache is read once per call and is far larger than L2: mark it evict-first so that the score rows
      // written below stay in L2 for the top-k that follows
      const uint64_t evict_first = l2_policy_evict_first();
      mbar_arrive_expect_tx(q_bar, N * 128);
      tma_load_2d(q_s, &q_map, 0, static_cast<int>(row0 * 64), q_bar);
      for (int i = 0; i < nblk; ++i) {
        const int s = i % kTcStages;
        if (!mbar_wait(&empty_bar[s], ((i / kTcStages) & 1) ^ 1, p.status, 1)) break;
        mbar_arrive_expect_tx(&full_bar[s], kKeyTileBytes);
        tma_load_2d_hint(k_s + s * kKeyTileBytes, &key_map, 0, phys_s[i] * 128, &full_bar[s], evict_first);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer --------------------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_i8(128, N);
      const uint64_t b_desc0 = umma_smem_desc_sw128(smem_u32(q_s), 16, 1024);
      bool ok = mbar_wait(q_bar, 0, p.status, 2);
      for (int i = 0; ok && i < nblk; ++i) {
        const int s = i % kTcStages, a = i & 1;
        if (!mbar_wait(&full_bar[s], (i / kTcStages) & 1, p.status, 3)) break;
        if (!mbar_wait(&tempty_bar[a], ((i >> 1) & 1) ^ 1, p.status, 4)) break;
        tc_fence_after();
        const uint64_t a_desc0 = umma_smem_desc_sw128(smem_u32(k_s + s * kKeyTileBytes), 16, 1024);
        const uint32_t d_tmem = tmem_base + a * N;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)  // K = 32 int8 per instruction: advance 32 B inside the swizzle atom
          umma_i8_ss(d_tmem, a_desc0 + 2 * ks, b_desc0 + 2 * ks, idesc, ks > 0 ? 1u : 0u);
        umma_commit(&empty_bar[s]);   // the stage may be refilled once these MMAs have read it
        umma_commit(&tfull_bar[a]);   // the accumulator is complete
      }
    }
  } else {
    // ---- epilogue: TMEM lane quarter = warp % 4; warp group (warp - 2) / 4 owns tokens [tg*TPW, tg*TPW + TPW) ----
    const int quarter = warp & 3;
    const int tg = (warp - 2) >> 2;
    const int key_in_blk = quarter * 32 + lane;
    // the key scale of a block is fetched one block ahead so that its latency is not exposed
    __half ks_next = p.key_scale[static_cast<size_t>(phys_s[0]) * bs + key_in_blk];
    for (int i = 0; i < nblk; ++i) {
      const int a = i & 1;
      const float ks = __half2float(ks_next);
      if (i + 1 < nblk) ks_next = p.key_scale[static_cast<size_t>(phys_s[i + 1]) * bs + key_in_blk];
      if (!__all_sync(0xffffffffu, mbar_wait(&tfull_bar[a], (i >> 1) & 1, p.status, 5))) break;
      tc_fence_after();
      const int pos = (blk_begin + i) * bs + key_in_blk;
      const bool in_range = pos < hi && pos >= p.key_begin;
      // four partial sums per token break the dependent-FMA chain; they are added in a fixed order
      float acc[TPW][4];
#pragma unroll
      for (int t = 0; t < TPW; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * N + tg * TPW * 64;
#pragma unroll
      for (int c = 0; c < TPW * 2; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int tl = c >> 1;               // token within this warp's group
        const int t = tg * TPW + tl;         // token within the CTA
        const int h0 = (c & 1) * 32;
        if (p.dots != nullptr && in_range && t < ntok) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            p.dots[((row0 + t) * 64 + h0 + j) * static_cast<size_t>(p.ld) + pos] = static_cast<int32_t>(r[j]);
        }
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          // dot * 2^-11 exactly: (2^23 + 2^22 + dot) as a float, then one FMA
          const float f0 = fmaf(__int_as_float(static_cast<int>(r[j]) + 0x4B400000), 1.f / 2048.f, -6144.f);
          const float f1 = fmaf(__int_as_float(static_cast<int>(r[j + 1]) + 0x4B400000), 1.f / 2048.f, -6144.f);
          const float f2 = fmaf(__int_as_float(static_cast<int>(r[j + 2]) + 0x4B400000), 1.f / 2048.f, -6144.f);
          const float f3 = fmaf(__int_as_float(static_cast<int>(r[j + 3]) + 0x4B400000), 1.f / 2048.f, -6144.f);
          uint32_t pk0, pk1;  // fp16 round-to-nearest-even with ReLU, two at a time
          asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(pk0) : "f"(f1), "f"(f0));
          asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(pk1) : "f"(f3), "f"(f2));
          const uint2 w = *reinterpret_cast<const uint2*>(&ws_s[(t * 64 + h0 + j) >> 1]);  // four fp16 weights
          // acc(fp32) += r(fp16) * ws(fp16): the product of two fp16 values is exact in fp32
          asm("{\n\t.reg .b16 rl, rh, wl, wh;\n\t"
              "mov.b32 {rl, rh}, %2;\n\tmov.b32 {wl, wh}, %3;\n\t"
              "fma.rn.f32.f16 %0, rl, wl, %0;\n\tfma.rn.f32.f16 %1, rh, wh, %1;\n\t}"
              : "+f"(acc[tl][0]), "+f"(acc[tl][1]) : "r"(pk0), "r"(w.x));
          asm("{\n\t.reg .b16 rl, rh, wl, wh;\n\t"
              "mov.b32 {rl, rh}, %2;\n\tmov.b32 {wl, wh}, %3;\n\t"
              "fma.rn.f32.f16 %0, rl, wl, %0;\n\tfma.rn.f32.f16 %1, rh, wh, %1;\n\t}"
              : "+f"(acc[tl][2]), "+f"(acc[tl][3]) : "r"(pk1), "r"(w.y));
        }
      }
      // all tcgen05.ld of this accumulator are complete: hand it back to the MMA warp
      tc_fence_before();
      mbar_arrive(&tempty_bar[a]);
      if (in_range) {
#pragma unroll
        for (int tl = 0; tl < TPW; ++tl)
          if (tg * TPW + tl < ntok)
            p.scores[(row0 + tg * TPW + tl) * static_cast<size_t>(p.ld) + pos] =
                ((acc[tl][0] + acc[tl][1]) + (acc[tl][2] + acc[tl][3])) * ks;
      }
    }
  }

  // ---- teardown -----------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

int make_tensor_map_2d_u8(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                          uint32_t box_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return DSV32_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_bytes, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (base %p rows %llu row_bytes %llu)", static_cast<int>(r), base,
              static_cast<unsigned long long>(rows), static_cast<unsigned long long>(row_bytes));
    return DSV32_ERR_CUDA;
  }
  return DSV32_OK;
}

__global__ void __launch_bounds__(32) wait_selftest_kernel(uint32_t* status, long long budget) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  // nobody arrives: the wait gives up after `budget` cycles, records DSV32_STATUS_TIMEOUT (location 99), returns false
  if (threadIdx.x == 0) (void)mbar_wait(&bar, 0, status, 99, budget);
}

int launch_wait_selftest(uint32_t* status, long long budget_cycles, cudaStream_t stream) {
  wait_selftest_kernel<<<1, 32, 0, stream>>>(status, budget_cycles);
  count_launch();
  return check_launch("wait_selftest_kernel");
}

template <int TOK>
static int launch_tc(const IndexerParams& p, const CUtensorMap& key_map, dim3 grid, cudaStream_t stream) {
  CUtensorMap q_map;
  const uint64_t q_rows = static_cast<uint64_t>(p.b) * p.s1 * 64;
  int rc = make_tensor_map_2d_u8(&q_map, p.q, q_rows, 128, 64 * TOK, 128);
  if (rc != DSV32_OK) return rc;
  cudaFuncSetAttribute(indexer_scores_tc_kernel<TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcSmemLayout<TOK>::bytes);
  indexer_scores_tc_kernel<TOK><<<grid, TcShape<TOK>::kThreads, TcSmemLayout<TOK>::bytes, stream>>>(key_map, q_map, p);
  count_launch();
  return check_launch("indexer_scores_tc_kernel");
}

int launch_indexer_scores_tc(const IndexerParams& p, cudaStream_t stream) {
  const int nblk = p.max_blocks - p.key_begin / p.block_size;
  if (nblk <= 0 || p.b <= 0) return DSV32_OK;
  if (p.num_blocks <= 0) {
    set_error("indexer: empty key cache");
    return DSV32_ERR_INVALID_ARG;
  }
  CUtensorMap key_map;
  int rc = make_tensor_map_2d_u8(&key_map, p.keys, static_cast<uint64_t>(p.num_blocks) * 128, 128, 128, 128);
  if (rc != DSV32_OK) return rc;
  // Key blocks per CTA.  The CTAs run in rounds of (resident CTAs per SM) x (SMs), and a CTA spends about two
  // block times filling its pipeline; pick the count that minimises rounds x (count + 2), so that the last
  // round is not mostly empty (measured: 57 instead of 32 blocks per CTA at 64 requests x 512 blocks, -5 %).
  // Context lengths live on the device, so the longest request stands for all of them.
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tok_groups = p.s1 <= 2 ? 1 : (p.s1 + 3) / 4;
  const long long slots = static_cast<long long>(sms) * (p.s1 <= 2 ? 2 : 1);  // tensor memory: 512 columns per SM
  int best_chunk = 32;
  long long best_cost = -1;
  for (int chunk = 8; chunk <= kTcBlocksPerCta; ++chunk) {
    const long long ctas = static_cast<long long>((nblk + chunk - 1) / chunk) * p.b * tok_groups;
    const long long rounds = (ctas + slots - 1) / slots;
    const long long cost = rounds * (chunk + 2);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best_chunk = chunk;
    }
  }
  IndexerParams q = p;
  q.blocks_per_cta = best_chunk;
  dim3 grid((nblk + best_chunk - 1) / best_chunk, p.b, 1);
  if (p.s1 == 1) return launch_tc<1>(q, key_map, grid, stream);
  if (p.s1 == 2) return launch_tc<2>(q, key_map, grid, stream);
  grid.z = (p.s1 + 3) / 4;
  return launch_tc<4>(q, key_map, grid, stream);
}

}  // namespace dsv32

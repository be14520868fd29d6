// Lightning-indexer scores: per request, stream the paged int8 index-key cache once and produce
//   score[token, key] = ( sum_h  ws[token,h] * fp16( relu(q[token,h] . k[key]) * 2^-11 ) ) * k_scale[key]
// with ws = fp16(q_scale * weight).  Follows the score part of
// models/deepseek_v32_exp/lightning_indexer_quant_impl.py:114-177 (golden:
// deepseekv32_lightning_indexer_quant.py:209-242).
//
// This file holds the warp-MMA (mma.sync m16n8k32 s8) implementation: keys are the M dimension so that
// one thread ends up with many heads of the same key and the head reduction stays mostly in registers.
#include "kernels.cuh"

namespace dsv32 {


constexpr int kIdxThreads = 128;
constexpr int kIdxBlocksPerCta = 8;
constexpr int kRowPad = 144;  // 128 B payload + 16 B pad: conflict-free ldmatrix rows

template <int TOK>
__global__ void __launch_bounds__(kIdxThreads) indexer_scores_mma_kernel(IndexerParams p) {
  constexpr int NT = TOK * 8;  // n-tiles of 8 heads
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* q_s = smem;                                   // [TOK*64][144]
  unsigned char* k_s = q_s + TOK * 64 * kRowPad;               // [2][128][144]
  float* ws_s = reinterpret_cast<float*>(k_s + 2 * 128 * kRowPad);  // [TOK*64]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tig = lane & 3;
  const int b = blockIdx.y;
  const int tok0 = blockIdx.z * TOK;  // first token (within the request) of this CTA
  const int ntok = min(TOK, p.s1 - tok0);
  const int L = p.act_seq[b];
  const int hi = min(L, p.key_end);
  const int bs = p.block_size;  // 128
  const int blk_begin = p.key_begin / bs + blockIdx.x * kIdxBlocksPerCta;
  const int blk_end = min(blk_begin + kIdxBlocksPerCta, (hi + bs - 1) / bs);
  if (blk_begin >= blk_end || hi <= p.key_begin) return;
  const int32_t* bt = p.block_table + static_cast<size_t>(b) * p.max_blocks;
  const size_t row0 = static_cast<size_t>(b) * p.s1 + tok0;

  // ---- stage q (int8) and ws = fp16(q_scale*weight) as fp32 -----------------------------------
  for (int c = tid; c < TOK * 64 * 8; c += kIdxThreads) {
    const int r = c >> 3, ch = c & 7;
    int4 v = make_int4(0, 0, 0, 0);
    if (r < ntok * 64) v = *reinterpret_cast<const int4*>(p.q + (row0 * 64 + r) * 128 + ch * 16);
    *reinterpret_cast<int4*>(q_s + r * kRowPad + ch * 16) = v;
  }
  for (int r = tid; r < TOK * 64; r += kIdxThreads) {
    float w = 0.f;
    if (r < ntok * 64) w = __half2float(__hmul(p.q_scale[row0 * 64 + r], p.weight[row0 * 64 + r]));
    ws_s[r] = w;
  }

  auto load_block = [&](int blk, int stage) {
    int phys = bt[blk];
    if (phys < 0 || phys >= p.num_blocks) {
      if (tid == 0) report_status(p.status, DSV32_STATUS_BAD_PAGE, b, blk);
      phys = 0;
    }
    const int8_t* src = p.keys + static_cast<size_t>(phys) * bs * 128;
    unsigned char* dst = k_s + stage * 128 * kRowPad;
    for (int c = tid; c < 128 * 8; c += kIdxThreads) {
      const int r = c >> 3, ch = c & 7;
      cp_async16(dst + r * kRowPad + ch * 16, src + r * 128 + ch * 16);
    }
    cp_async_commit();
    return phys;
  };

  int phys_cur = load_block(blk_begin, 0);
  for (int blk = blk_begin; blk < blk_end; ++blk) {
    const int stage = (blk - blk_begin) & 1;
    int phys_next = 0;
    if (blk + 1 < blk_end) {
      phys_next = load_block(blk + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const unsigned char* kb = k_s + stage * 128 * kRowPad;

#pragma unroll 1
    for (int mt = 0; mt < 2; ++mt) {
      const int key0 = warp * 32 + mt * 16;  // first key (in block) of this 16-key tile
      int acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t a0, a1, a2, a3;
        {
          const int r = key0 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int cb = ks * 32 + (lane >> 4) * 16;
          ldmatrix_x4(a0, a1, a2, a3, smem_u32(kb + r * kRowPad + cb));
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint32_t b0, b1;
          const int r = nt * 8 + (lane & 7);
          const int cb = ks * 32 + ((lane >> 3) & 1) * 16;
          ldmatrix_x2(b0, b1, smem_u32(q_s + r * kRowPad + cb));
          mma_s8_16832(acc[nt], a0, a1, a2, a3, b0, b1);
        }
      }
      // ---- epilogue: relu, 2^-11, fp16 round, weighted head sum --------------------------------
      const int pos_lo = blk * bs + key0 + g;  // logical key of rows g / g+8
      const int pos_hi = pos_lo + 8;
      if (p.dots != nullptr) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int t = nt >> 3, h = (nt & 7) * 8 + 2 * tig;
          if (t < ntok) {
            int32_t* d = p.dots + ((row0 + t) * 64 + h) * static_cast<size_t>(p.ld);
            if (pos_lo < hi) { d[pos_lo] = acc[nt][0]; d[p.ld + pos_lo] = acc[nt][1]; }
            if (pos_hi < hi) { d[pos_hi] = acc[nt][2]; d[p.ld + pos_hi] = acc[nt][3]; }
          }
        }
      }
      float s_lo[TOK], s_hi[TOK];
#pragma unroll
      for (int t = 0; t < TOK; ++t) s_lo[t] = s_hi[t] = 0.f;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int t = nt >> 3, h = (nt & 7) * 8 + 2 * tig;
        const float w0 = ws_s[t * 64 + h], w1 = ws_s[t * 64 + h + 1];
        const float r0 = __half2float(__float2half_rn(fmaxf(static_cast<float>(acc[nt][0]), 0.f) * (1.f / 2048.f)));
        const float r1 = __half2float(__float2half_rn(fmaxf(static_cast<float>(acc[nt][1]), 0.f) * (1.f / 2048.f)));
        const float r2 = __half2float(__float2half_rn(fmaxf(static_cast<float>(acc[nt][2]), 0.f) * (1.f / 2048.f)));
        const float r3 = __half2float(__float2half_rn(fmaxf(static_cast<float>(acc[nt][3]), 0.f) * (1.f / 2048.f)));
        s_lo[t] = fmaf(w0, r0, s_lo[t]);
        s_lo[t] = fmaf(w1, r1, s_lo[t]);
        s_hi[t] = fmaf(w0, r2, s_hi[t]);
        s_hi[t] = fmaf(w1, r3, s_hi[t]);
      }
#pragma unroll
      for (int t = 0; t < TOK; ++t) {
        s_lo[t] += __shfl_xor_sync(0xffffffffu, s_lo[t], 1);
        s_lo[t] += __shfl_xor_sync(0xffffffffu, s_lo[t], 2);
        s_hi[t] += __shfl_xor_sync(0xffffffffu, s_hi[t], 1);
        s_hi[t] += __shfl_xor_sync(0xffffffffu, s_hi[t], 2);
      }
      if (tig == 0) {
        const __half* ksc = p.key_scale + static_cast<size_t>(phys_cur) * bs + key0 + g;
        const float kl = __half2float(ksc[0]), kh = __half2float(ksc[8]);
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
          if (t < ntok) {
            float* srow = p.scores + (row0 + t) * static_cast<size_t>(p.ld);
            if (pos_lo < hi && pos_lo >= p.key_begin) srow[pos_lo] = s_lo[t] * kl;
            if (pos_hi < hi && pos_hi >= p.key_begin) srow[pos_hi] = s_hi[t] * kh;
          }
        }
      }
    }
    __syncthreads();
    phys_cur = phys_next;
  }
}

int launch_indexer_scores_mma(const IndexerParams& p, cudaStream_t stream) {
  const int nblk = p.max_blocks - p.key_begin / p.block_size;
  if (nblk <= 0 || p.b <= 0) return DSV32_OK;
  dim3 grid((nblk + kIdxBlocksPerCta - 1) / kIdxBlocksPerCta, p.b, 1);
  if (p.s1 == 1) {
    const size_t sm = 1 * 64 * kRowPad + 2 * 128 * kRowPad + 1 * 64 * sizeof(float);
    cudaFuncSetAttribute(indexer_scores_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    indexer_scores_mma_kernel<1><<<grid, kIdxThreads, sm, stream>>>(p);
  } else {
    grid.z = (p.s1 + 1) / 2;
    const size_t sm = 2 * 64 * kRowPad + 2 * 128 * kRowPad + 2 * 64 * sizeof(float);
    cudaFuncSetAttribute(indexer_scores_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    indexer_scores_mma_kernel<2><<<grid, kIdxThreads, sm, stream>>>(p);
  }
  count_launch();
  return check_launch("indexer_scores_mma_kernel");
}

}  // namespace dsv32

// DeepSeek-V4 KV compressor: state update and compression step between its library GEMMs.
// Follows models/deepseek_v4/compressor_impl.py:421-923 (golden golden_compress,
// models/deepseek_v4/test_compressor.py:76-187).  For request b and its token i at position pos = start_pos[b] + i:
//   kv    = x . wkv^T,  score = x . wgate^T + ape[pos % ratio]          (the two GEMMs come from the host layer, fp32)
//   kv_state[page(pos), pos % 128] = kv;  score_state[...] = score        (paged fp32 state, 128 positions per page)
//   if (pos + 1) % ratio == 0, the ratio positions that end at pos are compressed into one row:
//     ratio 128: softmax over the 128 score rows of the page, per column; kv = sum_r kv_r * softmax_r
//     ratio 4 (overlapping windows, state rows are [first half | second half] of 2 d columns): the rows are the
//       FIRST halves of the previous window's 4 positions and the SECOND halves of this window's 4 positions; a
//       request whose start position is below the ratio has no previous window (weight 0)
//     then bf16 -> RMSNorm * weight -> bf16 -> interleaved rotary embedding on the last 64 dims -> out[b]
// One CTA per request; its tokens are handled in order because a later token's compression reads the rows an
// earlier one wrote.  With ratio 4 a thread owns a column and walks its 8 rows; with ratio 128 the threads are
// (four columns) x (a group of the 128 rows), each keeps a running maximum / sum / weighted sum with 16-byte loads
// and the row groups are merged through shared memory, as are the RMSNorm sum and the rotary partner.
#include "kernels.cuh"

namespace dsv32 {

namespace {
constexpr int kCompThreads = 256, kCompPage = 128, kCompMaxD = 512, kCompRope = 64;

__device__ __forceinline__ float comp_bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
}  // namespace

__global__ void __launch_bounds__(kCompThreads) compressor_update_kernel(CompressorParams p) {
  __shared__ float val_s[kCompMaxD];
  __shared__ float red_s[kCompThreads / 32];
  __shared__ float merge_s[kCompThreads * 4 * 3];   // (maximum, sum, weighted sum) of the row groups 1.. per column
  const int b = blockIdx.x, tid = threadIdx.x;
  const int d = p.d, cd = p.coff * p.d, ratio = p.ratio;
  const int start = p.start_pos[b];
  for (int i = 0; i < p.s1; ++i) {
    const int pos = start + i;
    const int lb = pos / kCompPage, cur = pos % kCompPage;
    if (start < 0 || lb >= p.kv_cols || lb >= p.score_cols) {
      if (tid == 0) report_status(p.status, DSV32_STATUS_BAD_INDEX, b, pos);
      return;
    }
    const long long kb = p.kv_table[static_cast<size_t>(b) * p.kv_cols + lb];
    const long long sb = p.score_table[static_cast<size_t>(b) * p.score_cols + lb];
    if (kb < 0 || kb >= p.kv_blocks || sb < 0 || sb >= p.score_blocks) {
      if (tid == 0) report_status(p.status, DSV32_STATUS_BAD_PAGE, b, pos);
      return;
    }
    float* kv_row = p.kv_state + (kb * kCompPage + cur) * cd;
    float* sc_row = p.score_state + (sb * kCompPage + cur) * cd;
    const size_t trow = (static_cast<size_t>(b) * p.s1 + i) * cd;
    const float* ape = p.ape + static_cast<size_t>(pos % ratio) * cd;
    for (int c = tid; c < cd; c += kCompThreads) {
      kv_row[c] = p.kv_total[trow + c];
      sc_row[c] = p.score_total[trow + c] + ape[c];
    }
    __syncthreads();  // the rows just written are read below by other threads of this CTA
    if ((pos + 1) % ratio != 0) continue;

    // ---- the rows that are compressed -------------------------------------------------------------------
    const bool overlap = p.coff == 2;
    int nrows, pre_rows = 0;
    const float *kv0 = nullptr, *sc0 = nullptr;   // first group of rows (previous window, first halves)
    const float *kv1, *sc1;                       // second group (this window; second halves when overlapping)
    if (overlap) {
      const int cur_start = (pos - ratio + 1) % kCompPage;
      kv1 = p.kv_state + (kb * kCompPage + cur_start) * cd + d;
      sc1 = p.score_state + (sb * kCompPage + cur_start) * cd + d;
      nrows = ratio;
      if (start >= ratio) {
        const int p0 = pos - 2 * ratio + 1;       // >= 0 here
        const int lbp = p0 / kCompPage;
        const long long pkb = p.kv_table[static_cast<size_t>(b) * p.kv_cols + lbp];
        const long long psb = p.score_table[static_cast<size_t>(b) * p.score_cols + lbp];
        if (pkb < 0 || pkb >= p.kv_blocks || psb < 0 || psb >= p.score_blocks) {
          if (tid == 0) report_status(p.status, DSV32_STATUS_BAD_PAGE, b, p0);
          return;
        }
        kv0 = p.kv_state + (pkb * kCompPage + p0 % kCompPage) * cd;
        sc0 = p.score_state + (psb * kCompPage + p0 % kCompPage) * cd;
        pre_rows = ratio;
      }
    } else {
      kv1 = p.kv_state + kb * kCompPage * cd;     // the whole page: positions pos - 127 .. pos
      sc1 = p.score_state + sb * kCompPage * cd;
      nrows = kCompPage;
    }
    // ---- per column: softmax over the rows, weighted sum ------------------------------------------------------
    float sq = 0.f;
    if (!overlap && (d & 3) == 0 && (kCompThreads % (d / 4)) == 0) {
      // 128 rows: threads = (group of four columns) x (group of rows); each walks its rows once with 16-byte
      // loads, keeping a running maximum, sum and weighted sum per column; the row groups are then merged.
      const int ncg = d / 4, nrg = kCompThreads / ncg;
      const int cg = tid % ncg, rg = tid / ncg;
      const int rows_per = (kCompPage + nrg - 1) / nrg;
      const int r0 = rg * rows_per, r1 = min(kCompPage, r0 + rows_per);
      float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, sm[4] = {0.f, 0.f, 0.f, 0.f}, ac[4] = {0.f, 0.f, 0.f, 0.f};
      for (int r = r0; r < r1; ++r) {
        const float4 s4 = *reinterpret_cast<const float4*>(sc1 + static_cast<size_t>(r) * cd + 4 * cg);
        const float4 k4 = *reinterpret_cast<const float4*>(kv1 + static_cast<size_t>(r) * cd + 4 * cg);
        const float sv[4] = {s4.x, s4.y, s4.z, s4.w}, kv[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float mn = fmaxf(m[j], sv[j]);
          const float f = expf(m[j] - mn), e = expf(sv[j] - mn);   // exp(-inf) = 0 on the first row
          sm[j] = sm[j] * f + e;
          ac[j] = ac[j] * f + kv[j] * e;
          m[j] = mn;
        }
      }
      if (rg > 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          merge_s[((rg - 1) * d + 4 * cg + j) * 3 + 0] = m[j];
          merge_s[((rg - 1) * d + 4 * cg + j) * 3 + 1] = sm[j];
          merge_s[((rg - 1) * d + 4 * cg + j) * 3 + 2] = ac[j];
        }
      }
      __syncthreads();
      if (rg == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float mm = m[j];
          for (int g = 1; g < nrg; ++g) mm = fmaxf(mm, merge_s[((g - 1) * d + 4 * cg + j) * 3]);
          float f = expf(m[j] - mm);
          float st = sm[j] * f, at = ac[j] * f;
          for (int g = 1; g < nrg; ++g) {
            const float* q = &merge_s[((g - 1) * d + 4 * cg + j) * 3];
            f = expf(q[0] - mm);
            st += q[1] * f;
            at += q[2] * f;
          }
          const float v = comp_bf16r(__fdiv_rn(at, st));
          val_s[4 * cg + j] = v;
          sq += v * v;
        }
      }
    } else {
      for (int c = tid; c < d; c += kCompThreads) {
        float m = -INFINITY;
        for (int r = 0; r < pre_rows; ++r) m = fmaxf(m, sc0[static_cast<size_t>(r) * cd + c]);
        for (int r = 0; r < nrows; ++r) m = fmaxf(m, sc1[static_cast<size_t>(r) * cd + c]);
        float sum = 0.f;
        for (int r = 0; r < pre_rows; ++r) sum += expf(sc0[static_cast<size_t>(r) * cd + c] - m);
        for (int r = 0; r < nrows; ++r) sum += expf(sc1[static_cast<size_t>(r) * cd + c] - m);
        float acc = 0.f;
        for (int r = 0; r < pre_rows; ++r)
          acc += kv0[static_cast<size_t>(r) * cd + c] * __fdiv_rn(expf(sc0[static_cast<size_t>(r) * cd + c] - m), sum);
        for (int r = 0; r < nrows; ++r)
          acc += kv1[static_cast<size_t>(r) * cd + c] * __fdiv_rn(expf(sc1[static_cast<size_t>(r) * cd + c] - m), sum);
        const float v = comp_bf16r(acc);
        val_s[c] = v;
        sq += v * v;
      }
    }
    // ---- RMSNorm * weight -> bf16 ---------------------------------------------------------------------------
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if ((tid & 31) == 0) red_s[tid >> 5] = sq;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kCompThreads / 32; ++w) total += red_s[w];
    const float rinv = __fdiv_rn(1.0f, sqrtf(total / static_cast<float>(d) + p.eps));
    for (int c = tid; c < d; c += kCompThreads) val_s[c] = comp_bf16r(p.weight[c] * (val_s[c] * rinv));
    __syncthreads();
    // ---- rotary embedding on the last 64 dims (pairs 2i, 2i+1), write the row ---------------------------------
    const __nv_bfloat16* cosr = p.cos + static_cast<size_t>(b) * kCompRope;
    const __nv_bfloat16* sinr = p.sin + static_cast<size_t>(b) * kCompRope;
    __nv_bfloat16* orow = p.out + static_cast<size_t>(b) * d;
    for (int c = tid; c < d; c += kCompThreads) {
      float v = val_s[c];
      const int j = c - (d - kCompRope);
      if (j >= 0) {
        const float partner = (j & 1) ? val_s[c - 1] : -val_s[c + 1];
        v = __fadd_rn(__fmul_rn(v, __bfloat162float(cosr[j])), __fmul_rn(partner, __bfloat162float(sinr[j])));
      }
      orow[c] = __float2bfloat16_rn(v);
    }
    __syncthreads();  // val_s / red_s are reused by the next token
  }
}

int launch_compressor(const CompressorParams& p, cudaStream_t stream) {
  if (p.b <= 0 || p.s1 <= 0) return DSV32_OK;
  compressor_update_kernel<<<p.b, kCompThreads, 0, stream>>>(p);
  count_launch();
  return check_launch("compressor_update_kernel");
}

}  // namespace dsv32

// Row-wise top-k by block-wide radix select (one CTA per row), followed by a bitonic sort of the
// selected entries so that rows come out by descending score, equal scores by ascending id.
//
// Selection key: 64-bit composite  (sortable(score) << 32) | (0xFFFFFFFF - id).  Digits of 12/12/8 bits
// are resolved from the top; a pass only histograms entries that match the prefix found so far, and the
// loop stops as soon as the bucket holding the k-th entry is wholly selected (for distinct scores that is
// after the three score digits).  Semantics: pypto.topk as used at
// models/deepseek_v32_exp/lightning_indexer_quant_impl.py:179-216 with the tie rule of
// framework/src/interface/interpreter/calculator/calc_torch.cpp:2481-2495.
#include "kernels.cuh"

namespace dsv32 {

constexpr int kTopkThreads = 1024;
constexpr int kTopkMaxK = 2048;
constexpr int kHistBins = 4096;


__device__ __forceinline__ int row_count(const TopkParams& p, int row, int& col0) {
  if (p.counts != nullptr) {
    col0 = 0;
    return max(min(p.counts[row], p.ld), 0);
  }
  const int b = row / p.s1, i = row % p.s1;
  const int eff = p.act_seq[b] - (p.s1 - 1 - i);
  const int hi = min(min(eff, p.key_end), p.ld);
  col0 = p.key_begin;
  return max(hi - p.key_begin, 0);
}

__device__ __forceinline__ uint64_t composite_key(float s, uint32_t id) {
  return (static_cast<uint64_t>(float_to_key(s)) << 32) | static_cast<uint64_t>(0xFFFFFFFFu - id);
}

// Exclusive prefix (in thread order) of one value per thread, 1024 threads.
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* warp_tot /*[32]*/, uint32_t& total) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_tot[wid] = inc;
  __syncthreads();
  uint32_t wv = warp_tot[lane];
  uint32_t winc = wv;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xffffffffu, winc, o);
    if (lane >= o) winc += t;
  }
  total = __shfl_sync(0xffffffffu, winc, 31);
  const uint32_t wex = __shfl_sync(0xffffffffu, winc - wv, wid);
  __syncthreads();
  return wex + inc - v;
}

__global__ void __launch_bounds__(kTopkThreads) topk_select_kernel(TopkParams p) {
  __shared__ uint32_t hist[kHistBins];
  __shared__ uint64_t sel[kTopkMaxK];
  __shared__ uint32_t warp_tot[32];
  __shared__ uint32_t s_bin, s_above, s_bucket, s_nsel;

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  int col0;
  const int n = row_count(p, row, col0);
  const float* srow = p.scores + static_cast<size_t>(row) * p.ld + col0;
  const int32_t* irow = p.ids ? p.ids + static_cast<size_t>(row) * p.ld + col0 : nullptr;
  const uint32_t idb = static_cast<uint32_t>(col0 + p.id_base);
  int32_t* orow = p.out_idx + static_cast<size_t>(row) * p.k;
  float* osrow = p.out_scores ? p.out_scores + static_cast<size_t>(row) * p.k : nullptr;

  uint64_t prefix = 0, mask = 0;
  uint32_t k_rem = static_cast<uint32_t>(min(p.k, n));

  if (n > 0) {
    const int shifts[6] = {52, 40, 32, 20, 8, 0};
    const int nbits[6] = {12, 12, 8, 12, 12, 8};
    for (int pass = 0; pass < 6; ++pass) {
      for (int i = tid; i < kHistBins; i += kTopkThreads) hist[i] = 0;
      __syncthreads();
      const int shift = shifts[pass];
      const uint32_t dmask = (1u << nbits[pass]) - 1u;
#pragma unroll 4
      for (int j = tid; j < n; j += kTopkThreads) {
        const float s = srow[j];
        uint32_t id = idb + j;
        if (irow) {
          const int32_t v = irow[j];
          if (v < 0) continue;
          id = static_cast<uint32_t>(v);
        }
        const uint64_t c = composite_key(s, id);
        if ((c & mask) == prefix) atomicAdd(&hist[static_cast<uint32_t>(c >> shift) & dmask], 1u);
      }
      __syncthreads();
      // bins are visited from the top: thread t owns descending-order slots [4t, 4t+4)
      uint32_t h[4], tsum = 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        h[q] = hist[kHistBins - 1 - (4 * tid + q)];
        tsum += h[q];
      }
      uint32_t total;
      uint32_t above = block_exclusive_scan(tsum, warp_tot, total);
      if (pass == 0 && total <= k_rem) {
        // fewer valid entries than k: everything valid is selected (mask stays 0)
        k_rem = total;
        break;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (above < k_rem && above + h[q] >= k_rem) {
          s_bin = static_cast<uint32_t>(kHistBins - 1 - (4 * tid + q));
          s_above = above;
          s_bucket = h[q];
        }
        above += h[q];
      }
      __syncthreads();
      // note: bins above the digit range are empty, so s_bin always lies inside it
      prefix |= static_cast<uint64_t>(s_bin) << shift;
      mask |= static_cast<uint64_t>(dmask) << shift;
      const uint32_t need = k_rem - s_above;  // entries still to take from the selected bucket
      const bool done = (s_bucket == need);
      __syncthreads();
      if (done) break;
      // entries strictly above the bucket are already decided; keep counting inside the bucket only
      // (the final emission re-derives membership from prefix/mask, so k_rem is not needed after this)
      k_rem = need + 0u;
      // k_rem now counts within the bucket; "above" for later passes is relative to the bucket because
      // only bucket members are histogrammed.
    }
  }

  // ---- emission: every valid entry whose masked key is >= prefix ------------------------------
  if (tid == 0) s_nsel = 0;
  __syncthreads();
  if (n > 0) {
#pragma unroll 4
    for (int j = tid; j < n; j += kTopkThreads) {
      const float s = srow[j];
      uint32_t id = idb + j;
      if (irow) {
        const int32_t v = irow[j];
        if (v < 0) continue;
        id = static_cast<uint32_t>(v);
      }
      const uint64_t c = composite_key(s, id);
      if ((c & mask) >= prefix) {
        const uint32_t slot = atomicAdd(&s_nsel, 1u);
        if (slot < kTopkMaxK) sel[slot] = c;
      }
    }
  }
  __syncthreads();
  const int nsel = min(static_cast<int>(s_nsel), min(p.k, kTopkMaxK));
  int npad = 2;
  while (npad < nsel) npad <<= 1;
  for (int i = tid; i < npad; i += kTopkThreads)
    if (i >= nsel) sel[i] = 0ull;
  // ---- bitonic sort, descending --------------------------------------------------------------
  for (int size = 2; size <= npad; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      for (int t = tid; t < (npad >> 1); t += kTopkThreads) {
        const int i = 2 * t - (t & (stride - 1));
        const int j = i + stride;
        const bool up = ((i & size) == 0);
        const uint64_t a = sel[i], b = sel[j];
        if ((a < b) == up) {
          sel[i] = b;
          sel[j] = a;
        }
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < p.k; i += kTopkThreads) {
    if (i < nsel) {
      const uint64_t c = sel[i];
      orow[i] = static_cast<int32_t>(0xFFFFFFFFu - static_cast<uint32_t>(c));
      if (osrow) osrow[i] = key_to_float(static_cast<uint32_t>(c >> 32));
    } else {
      orow[i] = -1;
      if (osrow) osrow[i] = -INFINITY;
    }
  }
}

int launch_topk(const TopkParams& p, int rows, cudaStream_t stream) {
  if (rows <= 0) return DSV32_OK;
  topk_select_kernel<<<rows, kTopkThreads, 0, stream>>>(p);
  count_launch();
  return check_launch("topk_select_kernel");
}

}  // namespace dsv32

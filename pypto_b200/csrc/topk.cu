// Row-wise top-k by block-wide radix select (one CTA per row), followed by an ordering of the selected entries
// so that rows come out by descending score, equal scores by ascending id: a counting sort on the top eleven bits
// of the span the selected scores actually cover, then each entry's rank inside its (small) bucket -- or, when
// the scores crowd into few buckets (plateaus of equal scores), a bitonic sort.
//
// Selection key: 64-bit composite  (sortable(score) << 32) | (0xFFFFFFFF - id).
// Fast path (position ids): two scans of the row.  Scan 1 histograms the top 12 key bits; scan 2 sends
// every entry above the bucket that holds the k-th entry straight to the output list and collects the
// bucket itself into a shared-memory candidate list, on which the remaining digits (12/8 score bits, then
// 12/12/8 id bits, early exit) are resolved without touching global memory again.
// General path (explicit ids, or a candidate list that does not fit): the same digit loop over the row
// in global memory.  Semantics: pypto.topk as used at
// models/deepseek_v32_exp/lightning_indexer_quant_impl.py:179-216 with the tie rule of
// framework/src/interface/interpreter/calculator/calc_torch.cpp:2481-2495.
//
// Rows are few in decode (batch x query positions), so a row may be split over the CTAs of a thread-block cluster:
// every CTA scans its slice of the row (both scans).  After scan 1 each CTA adds the occupied bins of its slice
// histogram into a merged histogram in every CTA's shared memory, so that all of them find the threshold bucket
// without a further exchange; after scan 2 each CTA appends its slice lists to those of the cluster's first CTA,
// which finishes the row alone.  Two cluster barriers lie on the path (a third, at the start, is waited for only
// after scan 1).
#include <cooperative_groups.h>

#include "kernels.cuh"

namespace dsv32 {

namespace cg = cooperative_groups;

constexpr int kTopkThreads = 1024;
constexpr int kTopkMaxK = 2048;
constexpr int kHistBins = 4096;
constexpr int kCandCap = 4096;
constexpr int kSplitMinFloat4 = 12288;  // shortest row (in float4) that is split over a cluster
constexpr int kSortBuckets = 2048;    // buckets of the counting sort over the span of the selected scores
constexpr int kSortGroupCap = 96;     // largest bucket that is ordered by ranking; beyond it the bitonic sort takes over
constexpr size_t kTopkSmemBytes = kHistBins * 4 + kTopkMaxK * 8 + kCandCap * 8;   // histogram, output list, candidate list
// A cluster launch adds the merged histogram, and asks for more than half of an SM's shared memory, so that every
// CTA has an SM to itself: two CTAs that share one run their scans at half the speed each, and the split gains
// nothing.  The plain launch keeps the small request: what it leaves is L1, where scan 2 finds part of the row.
constexpr size_t kTopkClusterSmemBytes = 120 * 1024;
static_assert(kTopkClusterSmemBytes >= kTopkSmemBytes + kHistBins * 4, "room for the merged histogram");
static_assert(2 * kSortBuckets * 4 <= kHistBins * 4 && 2 * kTopkMaxK <= kCandCap, "the counting sort reuses these areas");

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

struct SelectState {
  uint64_t prefix, mask;  // an entry is selected iff (key & mask) >= prefix
  uint32_t k_rem;         // entries still to be taken from the bucket (key & mask) == prefix
  bool done;
};

// After a histogram of the current digit has been built over the entries with (key & mask) == prefix:
// find the bin that holds the k_rem-th entry from the top and narrow the state.  `total` = histogram sum.
__device__ __forceinline__ void narrow(SelectState& st, const uint32_t* hist, uint32_t* warp_tot, uint32_t* s_tmp,
                                       int shift, uint32_t dmask, uint32_t& total) {
  const int tid = threadIdx.x;
  uint32_t h[4], tsum = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {  // bins are visited from the top: thread t owns descending slots [4t, 4t+4)
    h[q] = hist[kHistBins - 1 - (4 * tid + q)];
    tsum += h[q];
  }
  uint32_t above = block_exclusive_scan(tsum, warp_tot, total);
  if (total <= st.k_rem && st.mask == 0) {  // fewer valid entries than k: everything valid is selected
    st.k_rem = total;
    st.done = true;
    return;
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    if (above < st.k_rem && above + h[q] >= st.k_rem) {
      s_tmp[0] = static_cast<uint32_t>(kHistBins - 1 - (4 * tid + q));
      s_tmp[1] = above;
      s_tmp[2] = h[q];
    }
    above += h[q];
  }
  __syncthreads();
  st.prefix |= static_cast<uint64_t>(s_tmp[0]) << shift;
  st.mask |= static_cast<uint64_t>(dmask) << shift;
  const uint32_t need = st.k_rem - s_tmp[1];
  st.done = (s_tmp[2] == need);  // the whole bucket is selected
  st.k_rem = need;
  __syncthreads();
}

__constant__ int kShifts[6] = {52, 40, 32, 20, 8, 0};
__constant__ int kDigitBits[6] = {12, 12, 8, 12, 12, 8};

// Digit loop over an arbitrary entry source: get(j, key) returns false for entries to skip.
template <class Get>
__device__ __forceinline__ void radix_passes(SelectState& st, int first_pass, int n, Get get, uint32_t* hist,
                                             uint32_t* warp_tot, uint32_t* s_tmp) {
  const int tid = threadIdx.x;
  for (int pass = first_pass; pass < 6 && !st.done; ++pass) {
    for (int i = tid; i < kHistBins; i += kTopkThreads) hist[i] = 0;
    __syncthreads();
    const int shift = kShifts[pass];
    const uint32_t dmask = (1u << kDigitBits[pass]) - 1u;
    for (int j = tid; j < n; j += kTopkThreads) {
      uint64_t c;
      if (!get(j, c)) continue;
      if ((c & st.mask) == st.prefix) atomicAdd(&hist[static_cast<uint32_t>(c >> shift) & dmask], 1u);
    }
    __syncthreads();
    uint32_t total;
    narrow(st, hist, warp_tot, s_tmp, shift, dmask, total);
  }
}

// Scan 2 over the float4 range [j, hi4) of a row, U float4 per thread and step, for the warps that lie inside the
// range as a whole; returns the first index this thread has not covered.  An entry is kept when its key is not
// below `bin_lo`: with flip = 0x80000000 for a threshold among the non-negative scores and 0xFFFFFFFF otherwise
// that is (bits ^ flip) >= bin_lo, two instructions, and most entries end there.  The kept ones (a few per cent)
// are then taken one per lane and round: the warp counts winners and threshold-bucket entries by ballot, reserves
// their slots with one atomic per list and stores them.
template <int U>
__device__ __forceinline__ int scan2_chunks(int j, int hi4, const float4* srow4, const float* srow, uint32_t flip,
                                            uint32_t bin_lo, uint32_t win_lo, bool top_bin, uint32_t idb,
                                            uint64_t* sel, uint64_t* cand, uint32_t* n_sel, uint32_t* n_cand) {
  constexpr uint32_t kFull = 0xFFFFFFFFu;
  const int lane = threadIdx.x & 31;
  const uint32_t lanes_below = (1u << lane) - 1u;
  for (; j - lane + 31 + (U - 1) * kTopkThreads < hi4; j += U * kTopkThreads) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = *reinterpret_cast<const uint4*>(srow4 + j + u * kTopkThreads);
    uint32_t km = 0;   // bit 4u+c: component c of float4 u is kept
#pragma unroll
    for (int u = 0; u < U; ++u) {
      km |= ((v[u].x ^ flip) >= bin_lo ? 1u : 0u) << (4 * u);
      km |= ((v[u].y ^ flip) >= bin_lo ? 1u : 0u) << (4 * u + 1);
      km |= ((v[u].z ^ flip) >= bin_lo ? 1u : 0u) << (4 * u + 2);
      km |= ((v[u].w ^ flip) >= bin_lo ? 1u : 0u) << (4 * u + 3);
    }
    while (__any_sync(kFull, km != 0)) {
      const bool act = km != 0;
      bool win = false;
      uint64_t c = 0;
      if (act) {
        const int e = __ffs(km) - 1;
        km &= km - 1u;
        const int col = 4 * (j + (e >> 2) * kTopkThreads) + (e & 3);
        const uint32_t k32 = float_to_key(srow[col]);   // read again (cache hit) rather than indexed out of registers
        c = (static_cast<uint64_t>(k32) << 32) | static_cast<uint64_t>(0xFFFFFFFFu - (idb + col));
        win = !top_bin && k32 >= win_lo;
      }
      const uint32_t bw = __ballot_sync(kFull, act && win), bt = __ballot_sync(kFull, act && !win);
      uint32_t base_w = 0, base_t = 0;
      if (lane == 0) {
        if (bw) base_w = atomicAdd(n_sel, static_cast<uint32_t>(__popc(bw)));
        if (bt) base_t = atomicAdd(n_cand, static_cast<uint32_t>(__popc(bt)));
      }
      base_w = __shfl_sync(kFull, base_w, 0);
      base_t = __shfl_sync(kFull, base_t, 0);
      if (act) {
        if (win) sel[base_w + __popc(bw & lanes_below)] = c;
        else cand[base_t + __popc(bt & lanes_below)] = c;
      }
    }
  }
  return j;
}

__global__ void __launch_bounds__(kTopkThreads) topk_select_kernel(TopkParams p, int csize) {
  extern __shared__ __align__(16) unsigned char topk_smem[];
  uint32_t* hist = reinterpret_cast<uint32_t*>(topk_smem);
  uint64_t* sel = reinterpret_cast<uint64_t*>(topk_smem + kHistBins * 4);
  uint64_t* cand = sel + kTopkMaxK;
  uint32_t* merged = reinterpret_cast<uint32_t*>(cand + kCandCap);   // the row's histogram when the row is split
  __shared__ uint32_t warp_tot[32];
  __shared__ uint32_t s_tmp[4];
  __shared__ uint32_t s_nsel, s_ncand, s_kmin, s_kmax, s_maxgroup;
  __shared__ uint32_t s_base[2];    // where this CTA's slice lists go in the first CTA's lists

  // csize CTAs (one cluster; 1 = no cluster, and then no cluster call is made) share a row
  cg::cluster_group cluster = cg::this_cluster();
  const int crank = csize > 1 ? static_cast<int>(cluster.block_rank()) : 0;
  const int row = blockIdx.x / csize;
  const int tid = threadIdx.x;
  int col0;
  const int n = row_count(p, row, col0);
  const float* srow = p.scores + static_cast<size_t>(row) * p.ld + col0;
  const int32_t* irow = p.ids ? p.ids + static_cast<size_t>(row) * p.ld + col0 : nullptr;
  const uint32_t idb = static_cast<uint32_t>(col0 + p.id_base);
  int32_t* orow = p.out_idx + static_cast<size_t>(row) * p.k;
  float* osrow = p.out_scores ? p.out_scores + static_cast<size_t>(row) * p.k : nullptr;
  if (p.scatter_world > 0) {   // the row goes to the rank that owns this token
    const int owner = row / p.scatter_per;
    const size_t at = (static_cast<size_t>(row - owner * p.scatter_per) * p.scatter_world + p.scatter_rank) * p.k;
    orow = p.scatter_idx[owner] + at;
    osrow = p.scatter_sc[owner] + at;
  }

  if (tid == 0) {
    s_nsel = 0;
    s_ncand = 0;
    s_kmin = 0xFFFFFFFFu;
    s_kmax = 0u;
    s_maxgroup = 0u;
  }
  SelectState st{0, 0, static_cast<uint32_t>(min(p.k, n)), false};
  auto from_global = [&](int j, uint64_t& c) -> bool {
    uint32_t id = idb + j;
    if (irow) {
      const int32_t v = irow[j];
      if (v < 0) return false;
      id = static_cast<uint32_t>(v);
    }
    c = composite_key(srow[j], id);
    return true;
  };

  bool emitted = false;
  const bool vec = (reinterpret_cast<uintptr_t>(srow) & 15) == 0;
  const int n4 = vec ? (n >> 2) : 0;
  // a short row is left to the first CTA (the barriers would cost more than the scans); all CTAs of the cluster decide alike
  const bool split = csize > 1 && irow == nullptr && n4 >= kSplitMinFloat4;
  if (!split && crank != 0) return;
  if (n > 0 && irow == nullptr) {
    // ---- fast path: scan 1 = histogram of the top 12 key bits (vectorised when the row is 16-byte aligned) ----
    for (int i = tid; i < kHistBins; i += kTopkThreads) hist[i] = 0;
    if (split)
      for (int i = tid; i < kHistBins; i += kTopkThreads) merged[i] = 0;
    __syncthreads();
    if (split) cluster.barrier_arrive();   // "my merged histogram is cleared"; waited for after scan 1
    const float4* srow4 = reinterpret_cast<const float4*>(srow);
    int lo4 = 0, hi4 = n4;   // this CTA's slice, in float4
    if (split) {
      lo4 = static_cast<int>(static_cast<long long>(n4) * crank / csize);
      hi4 = static_cast<int>(static_cast<long long>(n4) * (crank + 1) / csize);
    }
    {
      int j = lo4 + tid;
      for (; j + 3 * kTopkThreads < hi4; j += 4 * kTopkThreads) {  // four independent loads in flight per thread
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = srow4[j + u * kTopkThreads];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          atomicAdd(&hist[float_to_key(v[u].x) >> 20], 1u);
          atomicAdd(&hist[float_to_key(v[u].y) >> 20], 1u);
          atomicAdd(&hist[float_to_key(v[u].z) >> 20], 1u);
          atomicAdd(&hist[float_to_key(v[u].w) >> 20], 1u);
        }
      }
      for (; j < hi4; j += kTopkThreads) {
        const float4 v = srow4[j];
        atomicAdd(&hist[float_to_key(v.x) >> 20], 1u);
        atomicAdd(&hist[float_to_key(v.y) >> 20], 1u);
        atomicAdd(&hist[float_to_key(v.z) >> 20], 1u);
        atomicAdd(&hist[float_to_key(v.w) >> 20], 1u);
      }
    }
    if (crank == 0)
      for (int j = n4 * 4 + tid; j < n; j += kTopkThreads) atomicAdd(&hist[float_to_key(srow[j]) >> 20], 1u);
    __syncthreads();
    const uint32_t* row_hist = hist;
    if (split) {
      cluster.barrier_wait();   // every CTA's merged histogram is cleared
      const uint4 mine = reinterpret_cast<const uint4*>(hist)[tid];   // 1024 threads x 4 bins
      const uint32_t cnt[4] = {mine.x, mine.y, mine.z, mine.w};
#pragma unroll
      for (int b = 0; b < 4; ++b)
        if (cnt[b] != 0)
          for (int q = 0; q < csize; ++q) atomicAdd(cluster.map_shared_rank(merged, q) + 4 * tid + b, cnt[b]);
      cluster.sync();           // all slices are in every merged histogram
      row_hist = merged;
    }
    // mode 0: the first digit settles the row (emission below); 1: scan 2; 2: the threshold bucket does not fit the
    // candidate list (digit loop over global memory).  The CTAs of a split row all work this out, from equal data.
    uint32_t total;
    narrow(st, row_hist, warp_tot, s_tmp, 52, 0xFFFu, total);
    const uint32_t mode = st.done ? 0u : (s_tmp[2] <= static_cast<uint32_t>(kCandCap) ? 1u : 2u);
    const uint32_t bin = static_cast<uint32_t>(st.prefix >> 52);
    if (mode != 1u && crank != 0) return;   // the first CTA finishes such a row alone; no cluster call follows
    if (mode == 1u) {
      // ---- scan 2: winners go to the output list, the threshold bucket to the candidate list ---------------
      const uint32_t bin_lo = bin << 20, win_lo = (bin + 1u) << 20;   // smallest keys of the threshold bucket / of the next
      const bool top_bin = bin == 0xFFFu;                              // no bucket above the topmost one
      const uint32_t flip = (bin_lo & 0x80000000u) ? 0x80000000u : 0xFFFFFFFFu;
      auto place = [&](float s, int j) {
        const uint32_t k32 = float_to_key(s);
        const uint32_t b = k32 >> 20;
        if (b < bin) return;
        const uint64_t c = (static_cast<uint64_t>(k32) << 32) | static_cast<uint64_t>(0xFFFFFFFFu - (idb + j));
        if (b > bin) sel[atomicAdd(&s_nsel, 1u)] = c;
        else cand[atomicAdd(&s_ncand, 1u)] = c;
      };
      {
        int j = lo4 + tid;
        j = scan2_chunks<4>(j, hi4, srow4, srow, flip, bin_lo, win_lo, top_bin, idb, sel, cand, &s_nsel, &s_ncand);
        j = scan2_chunks<1>(j, hi4, srow4, srow, flip, bin_lo, win_lo, top_bin, idb, sel, cand, &s_nsel, &s_ncand);
        for (; j < hi4; j += kTopkThreads) {   // the warp that straddles the end of the slice
          const float4 v = srow4[j];
          place(v.x, 4 * j);
          place(v.y, 4 * j + 1);
          place(v.z, 4 * j + 2);
          place(v.w, 4 * j + 3);
        }
      }
      if (crank == 0)
        for (int j = n4 * 4 + tid; j < n; j += kTopkThreads) place(srow[j], j);
      __syncthreads();
      if (split) {
        if (crank != 0) {   // append this slice's lists to the first CTA's
          const uint32_t nw = s_nsel, nt = s_ncand;
          if (tid == 0) {
            s_base[0] = nw ? atomicAdd(cluster.map_shared_rank(&s_nsel, 0), nw) : 0u;
            s_base[1] = nt ? atomicAdd(cluster.map_shared_rank(&s_ncand, 0), nt) : 0u;
          }
          __syncthreads();
          uint64_t* sel0 = cluster.map_shared_rank(sel, 0) + s_base[0];
          uint64_t* cand0 = cluster.map_shared_rank(cand, 0) + s_base[1];
          for (uint32_t i = tid; i < nw; i += kTopkThreads) sel0[i] = sel[i];
          for (uint32_t i = tid; i < nt; i += kTopkThreads) cand0[i] = cand[i];
        }
        cluster.sync();   // the first CTA holds all lists; the others are done
        if (crank != 0) return;
      }
      const int ncand = static_cast<int>(s_ncand);
      auto from_cand = [&](int j, uint64_t& c) -> bool {
        c = cand[j];
        return true;
      };
      radix_passes(st, 1, ncand, from_cand, hist, warp_tot, s_tmp);
      for (int j = tid; j < ncand; j += kTopkThreads) {
        const uint64_t c = cand[j];
        if ((c & st.mask) >= st.prefix) sel[atomicAdd(&s_nsel, 1u)] = c;
      }
      emitted = true;
    } else if (mode == 2u) {
      radix_passes(st, 1, n, from_global, hist, warp_tot, s_tmp);  // bucket too large for the candidate list
    }
  } else if (n > 0) {
    radix_passes(st, 0, n, from_global, hist, warp_tot, s_tmp);
  }
  __syncthreads();
  if (n > 0 && !emitted) {
    // ---- emission: every valid entry whose masked key is >= prefix ---------------------------------------------
    for (int j = tid; j < n; j += kTopkThreads) {
      uint64_t c;
      if (!from_global(j, c)) continue;
      if ((c & st.mask) >= st.prefix) {
        const uint32_t slot = atomicAdd(&s_nsel, 1u);
        if (slot < kTopkMaxK) sel[slot] = c;
      }
    }
  }
  __syncthreads();
  const int nsel = min(static_cast<int>(s_nsel), min(p.k, kTopkMaxK));
  // ---- counting sort on the span of the selected scores, then the rank inside each bucket -----------------------
  // bucket = (largest key - key) >> shift with the shift that maps the span onto kSortBuckets buckets: bucket 0
  // holds the largest scores.  Entries land bucket by bucket in arrival order (`grp`), then every entry counts the
  // larger keys of its bucket (keys are distinct: they carry the id) and takes that slot (`ordered`).
  uint32_t* bcount = hist;                  // entries per bucket, consumed as fill counters
  uint32_t* bstart = hist + kSortBuckets;   // first slot of every bucket
  uint64_t* grp = cand;                     // the candidate list is done with
  uint64_t* ordered_s = cand + kTopkMaxK;
  const uint64_t* ordered = sel;
  bool ranked = false;
  if (nsel >= 64) {
    uint32_t kmin = 0xFFFFFFFFu, kmax = 0u;
    for (int i = tid; i < nsel; i += kTopkThreads) {
      const uint32_t k32 = static_cast<uint32_t>(sel[i] >> 32);
      kmin = min(kmin, k32);
      kmax = max(kmax, k32);
    }
    kmin = __reduce_min_sync(0xffffffffu, kmin);
    kmax = __reduce_max_sync(0xffffffffu, kmax);
    if ((tid & 31) == 0 && kmin <= kmax) {
      atomicMin(&s_kmin, kmin);
      atomicMax(&s_kmax, kmax);
    }
    for (int i = tid; i < 2 * kSortBuckets; i += kTopkThreads) hist[i] = 0;
    __syncthreads();
    kmin = s_kmin;
    kmax = s_kmax;
    const uint32_t span = kmax - kmin;
    const int shift = span < static_cast<uint32_t>(kSortBuckets) ? 0 : (32 - __clz(span)) - 11;   // span >> shift < 2048
    for (int i = tid; i < nsel; i += kTopkThreads)
      atomicAdd(&bcount[(kmax - static_cast<uint32_t>(sel[i] >> 32)) >> shift], 1u);
    __syncthreads();
    {  // exclusive scan over the buckets, two per thread; the largest bucket decides whether ranking is cheap
      const uint32_t c0 = bcount[2 * tid], c1 = bcount[2 * tid + 1];
      uint32_t total;
      const uint32_t ex = block_exclusive_scan(c0 + c1, warp_tot, total);
      bstart[2 * tid] = ex;
      bstart[2 * tid + 1] = ex + c0;
      const uint32_t mx = __reduce_max_sync(0xffffffffu, max(c0, c1));
      if ((tid & 31) == 0) atomicMax(&s_maxgroup, mx);
    }
    __syncthreads();
    ranked = s_maxgroup <= static_cast<uint32_t>(kSortGroupCap);
    if (ranked) {
      for (int i = tid; i < nsel; i += kTopkThreads) {
        const uint64_t c = sel[i];
        const uint32_t b = (kmax - static_cast<uint32_t>(c >> 32)) >> shift;
        grp[bstart[b] + (atomicSub(&bcount[b], 1u) - 1u)] = c;
      }
      __syncthreads();
      for (int i = tid; i < nsel; i += kTopkThreads) {
        const uint64_t c = grp[i];
        const uint32_t b = (kmax - static_cast<uint32_t>(c >> 32)) >> shift;
        const uint32_t start = bstart[b];
        const uint32_t end = b + 1 < static_cast<uint32_t>(kSortBuckets) ? bstart[b + 1] : static_cast<uint32_t>(nsel);
        uint32_t rank = 0;
        for (uint32_t j = start; j < end; ++j) rank += grp[j] > c ? 1u : 0u;
        ordered_s[start + rank] = c;
      }
      ordered = ordered_s;
    }
  }
  int npad = 2;
  while (npad < nsel) npad <<= 1;
  if (!ranked) {
  for (int i = tid; i < npad; i += kTopkThreads)
    if (i >= nsel) sel[i] = 0ull;
  // ---- bitonic sort, descending ------------------------------------------------------------------------------
  // Thread t owns elements 2t and 2t+1.  Compare-exchange steps with a stride of 32 or less stay inside a
  // warp (stride 1 inside the thread, the others by shuffle), so only the steps with a stride of 64 or more
  // go through shared memory and a block barrier: 15 of the 66 steps of a 2048-element sort.
  if (npad >= 64) {
    const bool active = tid < (npad >> 1);  // whole warps: npad/2 is a multiple of 32
    const int e0 = 2 * tid;
    auto warp_steps = [&](uint64_t& a, uint64_t& b, int size, int first_stride) {
      const bool up = ((e0 & size) == 0);
      for (int stride = first_stride; stride >= 2; stride >>= 1) {
        const uint64_t pa = __shfl_xor_sync(0xffffffffu, a, stride >> 1);
        const uint64_t pb = __shfl_xor_sync(0xffffffffu, b, stride >> 1);
        const bool keep_max = (((e0 & stride) == 0) == up);
        a = keep_max ? (a > pa ? a : pa) : (a < pa ? a : pa);
        b = keep_max ? (b > pb ? b : pb) : (b < pb ? b : pb);
      }
      if ((a < b) == up) {  // stride 1
        const uint64_t t = a;
        a = b;
        b = t;
      }
    };
    __syncthreads();
    if (active) {
      uint64_t a = sel[e0], b = sel[e0 + 1];
      for (int size = 2; size <= 64; size <<= 1) warp_steps(a, b, size, size >> 1);
      sel[e0] = a;
      sel[e0 + 1] = b;
    }
    for (int size = 128; size <= npad; size <<= 1) {
      for (int stride = size >> 1; stride >= 64; stride >>= 1) {
        __syncthreads();
        if (active) {
          const int i = 2 * tid - (tid & (stride - 1));
          const int j = i + stride;
          const bool up = ((i & size) == 0);
          const uint64_t a = sel[i], b = sel[j];
          if ((a < b) == up) {
            sel[i] = b;
            sel[j] = a;
          }
        }
      }
      __syncthreads();
      if (active) {
        uint64_t a = sel[e0], b = sel[e0 + 1];
        warp_steps(a, b, size, 32);
        sel[e0] = a;
        sel[e0 + 1] = b;
      }
    }
  } else {
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
  }
  }  // !ranked
  __syncthreads();
  for (int i = tid; i < p.k; i += kTopkThreads) {
    if (i < nsel) {
      const uint64_t c = ordered[i];
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
  cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTopkClusterSmemBytes);
  // A cluster per row while rows are few: the largest of 8/4/2 CTAs for which the device can hold all rows'
  // clusters at once (a CTA fills an SM, and a cluster has to find its SMs within one GPC).  Rows with explicit
  // ids, and short rows, are not split.
  static int room[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};   // room[c]: clusters of c CTAs the device holds at once; 0 = not asked yet
  int csize = 1;
  const int longest = p.counts != nullptr ? p.ld : min(p.ld, p.key_end) - p.key_begin;   // no row has more entries
  if (p.ids == nullptr && longest / 4 >= kSplitMinFloat4)
    for (int c = 8; c > 1; c >>= 1) {
      if (room[c] == 0) {
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3(c);
        probe.blockDim = dim3(kTopkThreads);
        probe.dynamicSmemBytes = kTopkClusterSmemBytes;
        cudaLaunchAttribute pattr;
        pattr.id = cudaLaunchAttributeClusterDimension;
        pattr.val.clusterDim.x = c;
        pattr.val.clusterDim.y = 1;
        pattr.val.clusterDim.z = 1;
        probe.attrs = &pattr;
        probe.numAttrs = 1;
        int clusters = 0;
        const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, topk_select_kernel, &probe);
        if (e != cudaSuccess) cudaGetLastError();
        room[c] = (e == cudaSuccess && clusters > 0) ? clusters : -1;
      }
      if (rows <= room[c]) {
        csize = c;
        break;
      }
    }
  if (csize == 1) {
    topk_select_kernel<<<rows, kTopkThreads, kTopkSmemBytes, stream>>>(p, 1);
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * csize);
    cfg.blockDim = dim3(kTopkThreads);
    cfg.dynamicSmemBytes = kTopkClusterSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = csize;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, topk_select_kernel, p, csize);
  }
  count_launch();
  return check_launch("topk_select_kernel");
}

}  // namespace dsv32

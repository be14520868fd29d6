// Indexer prolog (quant) on tcgen05 tensor cores.  Follows
// models/deepseek_v32_exp/lightning_indexer_prolog_quant_impl.py:423-543 (golden:
// deepseekv32_lightning_indexer_prolog_quant.py:220-288).
//
// Q kernel, one CTA per (index head, tile of 128 tokens):
//   D1[token, 128 dims] = q_norm[token, 1536] (int8, K-major)  x  w_qb[1536, head*128 ..] (int8, MN-major)
//        -> epilogue 1 (thread = token): * q_norm_scale * w_qb_scale -> bf16 -> RoPE(dims 0..63) -> bf16,
//           written back to tensor memory as bf16 pairs
//   D2[token, 128]      = R (bf16, from tensor memory)  x  hadamard_q[128, 128] (bf16, MN-major)
//        -> epilogue 2: bf16 round -> per-row amax -> int8 quantisation -> q_int8 / q_scale
// K/W kernel, one CTA per (slice of the 7168-long reduction, tile of 128 tokens):
//   D[token, 192] = x[token, slice] (bf16) x [wk | w_proj][slice, 192] (bf16, MN-major) -> fp32 partial sums;
//   the per-token finish kernel (prolog.cu) reduces them in a fixed order and completes the K and W paths.
// Weights stream through a 4-stage TMA ring exactly once per CTA; no multicast.
//
// The Q kernel has a second instantiation for the DeepSeek-V4 indexer prolog
// (models/deepseek_v4/lightning_indexer_prolog_quant_v4_impl.py:118-266): reduction length 1024 instead of 1536
// and, in epilogue 1, the rotary embedding on dims 64..127 in its interleaved, inverse form
// (out[2i] = x[2i] cos[2i] + x[2i+1] sin[2i], out[2i+1] = x[2i+1] cos[2i+1] - x[2i] sin[2i+1]).  That operator has
// no K path; its head weights come from prolog_v4_weights_partial_kernel / _finish_kernel.
#include <mutex>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace dsv32 {

constexpr int kPqThreads = 192;
constexpr int kPqStages = 4;
constexpr int kPqChunk = 16384;                 // 128 rows x 128 B
constexpr int kPqStageBytes = 2 * kPqChunk;     // A chunk + B chunk
constexpr int kPqOffH = kPqStages * kPqStageBytes;        // hadamard: 2 x [128 k rows][128 B]
constexpr int kPqOffWs = kPqOffH + 2 * kPqChunk;          // 128 floats (w_qb_scale of this head)
constexpr int kPqOffBars = kPqOffWs + 512;
constexpr int kPqNumBars = 2 * kPqStages + 4;             // full, empty, h_bar, d1_full, r_ready, d2_full
constexpr int kPqOffTmem = kPqOffBars + kPqNumBars * 8;
constexpr size_t kPqSmemBytes = kPqOffTmem + 16 + 1024;
constexpr int kVariantV32 = 0, kVariantV4 = 1;

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <int kVariant>
__global__ void __launch_bounds__(kPqThreads, 1) prolog_q_tc_kernel(const __grid_constant__ CUtensorMap qn_map,
                                                                    const __grid_constant__ CUtensorMap w_map,
                                                                    const __grid_constant__ CUtensorMap h_map,
                                                                    PrologParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* ring = smem;
  unsigned char* h_s = smem + kPqOffH;
  float* ws_s = reinterpret_cast<float*>(smem + kPqOffWs);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPqOffBars);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kPqStages;
  uint64_t* h_bar = bars + 2 * kPqStages;
  uint64_t* d1_bar = h_bar + 1;
  uint64_t* r_bar = h_bar + 2;
  uint64_t* d2_bar = h_bar + 3;
  uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(smem + kPqOffTmem);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int head = blockIdx.x;
  const int t0 = blockIdx.y * 128;
  constexpr int kQr = kVariant == kVariantV4 ? 1024 : 1536;
  constexpr int kChunks = kQr / 128;  // 12 (8) reduction chunks of 128

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&qn_map);
      tma_prefetch_desc(&w_map);
      tma_prefetch_desc(&h_map);
      for (int i = 0; i < kPqStages; ++i) {
        mbar_init(&full_bar[i], 1);
        mbar_init(&empty_bar[i], 1);
      }
      mbar_init(h_bar, 1);
      mbar_init(d1_bar, 1);
      mbar_init(r_bar, 128);
      mbar_init(d2_bar, 1);
      mbar_fence_init();
    }
  } else if (warp == 1) {
    tmem_alloc(tmem_ptr_s, 512);
    tmem_relinquish();
  } else {
    const int i = tid - 64;
    ws_s[i] = p.w_qb_scale[head * 128 + i];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_s;
  constexpr uint32_t kColD1 = 0, kColR = 128, kColD2 = 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(h_bar, 2 * kPqChunk);
      tma_load_2d(h_s, &h_map, 0, 0, h_bar);
      tma_load_2d(h_s + kPqChunk, &h_map, 128, 0, h_bar);
      for (int c = 0; c < kChunks; ++c) {
        const int s = c % kPqStages;
        if (!mbar_wait(&empty_bar[s], ((c / kPqStages) & 1) ^ 1, p.status, 40)) break;
        mbar_arrive_expect_tx(&full_bar[s], kPqStageBytes);
        tma_load_2d(ring + s * kPqStageBytes, &qn_map, c * 128, t0, &full_bar[s]);                 // A: tokens x 128 k
        tma_load_2d(ring + s * kPqStageBytes + kPqChunk, &w_map, head * 128, c * 128, &full_bar[s]);  // B: 128 k x 128 n
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc1 = umma_idesc_i8(128, 128, true);
      constexpr uint32_t idesc2 = umma_idesc_bf16(128, 128, false, true);
      bool ok = true;
      for (int c = 0; ok && c < kChunks; ++c) {
        const int s = c % kPqStages;
        if (!mbar_wait(&full_bar[s], (c / kPqStages) & 1, p.status, 41)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_s = smem_u32(ring + s * kPqStageBytes), b_s = a_s + kPqChunk;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)  // 32 k per instruction: A advances 32 B in its row, B advances 32 k rows
          umma_i8_ss(tmem_base + kColD1, umma_smem_desc_sw128(a_s + ks * 32, 16, 1024),
                     umma_smem_desc_sw128(b_s + ks * 4096, kPqChunk, 1024), idesc1, (c > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      if (ok) {
        umma_commit(d1_bar);
        ok = mbar_wait(h_bar, 0, p.status, 42) && mbar_wait(r_bar, 0, p.status, 43);
      }
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)  // 16 dims per instruction; hadamard rows = k, two 64-column chunks
          umma_f16_ts(tmem_base + kColD2, tmem_base + kColR + ks * 8,
                      umma_smem_desc_sw128(smem_u32(h_s) + ks * 2048, kPqChunk, 1024), idesc2, ks > 0 ? 1u : 0u);
        umma_commit(d2_bar);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int tok = t0 + quarter * 32 + lane;
    const bool live = tok < p.t;
    const int tk = live ? tok : 0;  // clamp for loads
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = __all_sync(0xffffffffu, mbar_wait(d1_bar, 0, p.status, 44));
    if (ok) {
      tc_fence_after();
      const float qs = p.q_norm_scale[tk];
      if constexpr (kVariant == kVariantV32) {
      // ---- dims 0..63: dequantise, round to bf16, RoPE (rotate-half over pairs d, d+32), round to bf16 -------
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(tmem_base + lane_addr + kColD1, r0);
      tmem_ld_32x32b_x32(tmem_base + lane_addr + kColD1 + 32, r1);
      tmem_ld_wait();
      const __nv_bfloat16* cosr = p.cos + static_cast<size_t>(tk) * 64;
      const __nv_bfloat16* sinr = p.sin + static_cast<size_t>(tk) * 64;
      uint32_t lo[16], hi[16];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint4 c_lo = *reinterpret_cast<const uint4*>(cosr + g * 8), c_hi = *reinterpret_cast<const uint4*>(cosr + 32 + g * 8);
        const uint4 s_lo = *reinterpret_cast<const uint4*>(sinr + g * 8), s_hi = *reinterpret_cast<const uint4*>(sinr + 32 + g * 8);
        const uint32_t cl[4] = {c_lo.x, c_lo.y, c_lo.z, c_lo.w}, ch[4] = {c_hi.x, c_hi.y, c_hi.z, c_hi.w};
        const uint32_t sl[4] = {s_lo.x, s_lo.y, s_lo.z, s_lo.w}, sh[4] = {s_hi.x, s_hi.y, s_hi.z, s_hi.w};
        float o_lo[8], o_hi[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int d = g * 8 + e;
          const float x1 = bf16_round(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r0[d])), qs), ws_s[d]));
          const float x2 = bf16_round(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r1[d])), qs), ws_s[32 + d]));
          const uint32_t cw_l = cl[e >> 1], cw_h = ch[e >> 1], sw_l = sl[e >> 1], sw_h = sh[e >> 1];
          const float c1 = __uint_as_float((e & 1) ? (cw_l & 0xffff0000u) : (cw_l << 16));
          const float c2 = __uint_as_float((e & 1) ? (cw_h & 0xffff0000u) : (cw_h << 16));
          const float s1 = __uint_as_float((e & 1) ? (sw_l & 0xffff0000u) : (sw_l << 16));
          const float s2 = __uint_as_float((e & 1) ? (sw_h & 0xffff0000u) : (sw_h << 16));
          o_lo[e] = __fadd_rn(__fmul_rn(x1, c1), __fmul_rn(-x2, s1));
          o_hi[e] = __fadd_rn(__fmul_rn(x2, c2), __fmul_rn(x1, s2));
        }
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          lo[g * 4 + (e >> 1)] = pack_bf16x2(o_lo[e], o_lo[e + 1]);
          hi[g * 4 + (e >> 1)] = pack_bf16x2(o_hi[e], o_hi[e + 1]);
        }
      }
      uint32_t pk[32];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        pk[j] = lo[j];
        pk[16 + j] = hi[j];
      }
      tmem_st_32x32b_x32(tmem_base + lane_addr + kColR, pk);
      // ---- dims 64..127: dequantise and round to bf16 only ---------------------------------------------------
      tmem_ld_32x32b_x32(tmem_base + lane_addr + kColD1 + 64, r0);
      tmem_ld_32x32b_x32(tmem_base + lane_addr + kColD1 + 96, r1);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        pk[j >> 1] = pack_bf16x2(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r0[j])), qs), ws_s[64 + j]),
                                 __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r0[j + 1])), qs), ws_s[65 + j]));
        pk[16 + (j >> 1)] = pack_bf16x2(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r1[j])), qs), ws_s[96 + j]),
                                        __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r1[j + 1])), qs), ws_s[97 + j]));
      }
      tmem_st_32x32b_x32(tmem_base + lane_addr + kColR + 32, pk);
      } else {
        // ---- dims 0..63: dequantise and round to bf16 only ---------------------------------------------------
        uint32_t r0[32], r1[32], pk[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColD1, r0);
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColD1 + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          pk[j >> 1] = pack_bf16x2(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r0[j])), qs), ws_s[j]),
                                   __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r0[j + 1])), qs), ws_s[j + 1]));
          pk[16 + (j >> 1)] = pack_bf16x2(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r1[j])), qs), ws_s[32 + j]),
                                          __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r1[j + 1])), qs), ws_s[33 + j]));
        }
        tmem_st_32x32b_x32(tmem_base + lane_addr + kColR, pk);
        // ---- dims 64..127: dequantise, round to bf16, interleaved inverse rotary embedding, round to bf16 ------
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColD1 + 64, r0);
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColD1 + 96, r1);
        tmem_ld_wait();
        const uint32_t* cosw = reinterpret_cast<const uint32_t*>(p.cos + static_cast<size_t>(tk) * 64);
        const uint32_t* sinw = reinterpret_cast<const uint32_t*>(p.sin + static_cast<size_t>(tk) * 64);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const uint32_t* r = half == 0 ? r0 : r1;
#pragma unroll
          for (int j = 0; j < 32; j += 2) {  // rope dims 32*half + j, + j + 1 (head dims 64 + those)
            const int d = 32 * half + j;
            const float xe = bf16_round(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r[j])), qs), ws_s[64 + d]));
            const float xo = bf16_round(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r[j + 1])), qs), ws_s[65 + d]));
            const uint32_t cw = __ldg(cosw + (d >> 1)), sw = __ldg(sinw + (d >> 1));
            const float ce = __uint_as_float(cw << 16), co = __uint_as_float(cw & 0xffff0000u);
            const float se = __uint_as_float(sw << 16), so = __uint_as_float(sw & 0xffff0000u);
            const float oe = __fadd_rn(__fmul_rn(xe, ce), __fmul_rn(xo, se));
            const float oo = __fadd_rn(__fmul_rn(xo, co), __fmul_rn(-xe, so));
            pk[16 * half + (j >> 1)] = pack_bf16x2(oe, oo);
          }
        }
        tmem_st_32x32b_x32(tmem_base + lane_addr + kColR + 32, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(r_bar);
      ok = __all_sync(0xffffffffu, mbar_wait(d2_bar, 0, p.status, 45));
    }
    if (ok) {
      tc_fence_after();
      // ---- pass 1: row amax of the bf16-rounded hadamard output -------------------------------------------
      float amax = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColD2 + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(bf16_round(__uint_as_float(r[j]))));
      }
      const float sq = __fdiv_rn(127.0f, amax);
      int8_t* qrow = p.q_int8 + (static_cast<size_t>(tk) * 64 + head) * 128;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColD2 + c * 32, r);
        tmem_ld_wait();
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const int q0 = static_cast<int>(rintf(__fmul_rn(bf16_round(__uint_as_float(r[j])), sq)));
          const int q1 = static_cast<int>(rintf(__fmul_rn(bf16_round(__uint_as_float(r[j + 1])), sq)));
          const int q2 = static_cast<int>(rintf(__fmul_rn(bf16_round(__uint_as_float(r[j + 2])), sq)));
          const int q3 = static_cast<int>(rintf(__fmul_rn(bf16_round(__uint_as_float(r[j + 3])), sq)));
          w[j >> 2] = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) | (static_cast<uint32_t>(q3 & 0xff) << 24);
        }
        if (live) {
          *reinterpret_cast<uint4*>(qrow + c * 32) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(qrow + c * 32 + 16) = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
      if (live) p.q_scale[static_cast<size_t>(tok) * 64 + head] = __float2half_rn(__fdiv_rn(1.0f, sq));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------------------
// K/W partial sums:  D[token, 0..127 | 128..191] = x[token, slice] x [wk | w_proj][slice, :]
// ---------------------------------------------------------------------------------------------------------
constexpr int kKwStages = 4;
constexpr int kKwABytes = 16384;                 // 128 tokens x 64 k (bf16)
constexpr int kKwBChunk = 8192;                  // 64 k rows x 128 B (64 n)
constexpr int kKwStageBytes = kKwABytes + 3 * kKwBChunk;   // 40 KB
constexpr int kKwOffBars = kKwStages * kKwStageBytes;
constexpr int kKwNumBars = 2 * kKwStages + 1;
constexpr int kKwOffTmem = kKwOffBars + kKwNumBars * 8;
constexpr size_t kKwSmemBytes = kKwOffTmem + 16 + 1024;
constexpr int kKwChunksTotal = 7168 / 64;        // 112 reduction chunks of 64

__global__ void __launch_bounds__(kPqThreads, 1) prolog_kw_tc_kernel(const __grid_constant__ CUtensorMap x_map,
                                                                     const __grid_constant__ CUtensorMap wk_map,
                                                                     const __grid_constant__ CUtensorMap wp_map,
                                                                     PrologParams p, int chunks_per_cta) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kKwOffBars);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kKwStages;
  uint64_t* d_bar = bars + 2 * kKwStages;
  uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(smem + kKwOffTmem);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x;
  const int t0 = blockIdx.y * 128;
  const int c_begin = split * chunks_per_cta;
  const int nchunks = min(chunks_per_cta, kKwChunksTotal - c_begin);  // >= 1 by construction of the grid

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&x_map);
      tma_prefetch_desc(&wk_map);
      tma_prefetch_desc(&wp_map);
      for (int i = 0; i < kKwStages; ++i) {
        mbar_init(&full_bar[i], 1);
        mbar_init(&empty_bar[i], 1);
      }
      mbar_init(d_bar, 1);
      mbar_fence_init();
    }
  } else if (warp == 1) {
    tmem_alloc(tmem_ptr_s, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_s;

  if (warp == 0) {
    if (lane == 0) {
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % kKwStages;
        const int k0 = (c_begin + c) * 64;
        if (!mbar_wait(&empty_bar[s], ((c / kKwStages) & 1) ^ 1, p.status, 50)) break;
        unsigned char* st = smem + s * kKwStageBytes;
        mbar_arrive_expect_tx(&full_bar[s], kKwStageBytes);
        tma_load_2d(st, &x_map, k0 * 2, t0, &full_bar[s]);                       // tokens x 64 k
        tma_load_2d(st + kKwABytes, &wk_map, 0, k0, &full_bar[s]);               // 64 k x wk cols 0..63
        tma_load_2d(st + kKwABytes + kKwBChunk, &wk_map, 128, k0, &full_bar[s]); // 64 k x wk cols 64..127
        tma_load_2d(st + kKwABytes + 2 * kKwBChunk, &wp_map, 0, k0, &full_bar[s]);  // 64 k x w_proj cols 0..63
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 192, false, true);
      bool ok = true;
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % kKwStages;
        if (!mbar_wait(&full_bar[s], (c / kKwStages) & 1, p.status, 51)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_s = smem_u32(smem + s * kKwStageBytes), b_s = a_s + kKwABytes;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)  // 16 k per instruction
          umma_f16_ss(tmem_base, umma_smem_desc_sw128(a_s + ks * 32, 16, 1024),
                      umma_smem_desc_sw128(b_s + ks * 2048, kKwBChunk, 1024), idesc, (c > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(d_bar);
    }
  } else {
    const int quarter = warp & 3;
    const int tok = t0 + quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    if (__all_sync(0xffffffffu, mbar_wait(d_bar, 0, p.status, 52))) {
      tc_fence_after();
      float* prow = p.partial + (static_cast<size_t>(split) * p.t + (tok < p.t ? tok : 0)) * 192;
#pragma unroll 1
      for (int c = 0; c < 6; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + c * 32, r);
        tmem_ld_wait();
        if (tok < p.t) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(prow + c * 32 + j) =
                make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                            __uint_as_float(r[j + 3]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// ---- host ---------------------------------------------------------------------------------------------------
int launch_prolog_finish(const PrologParams& p, int splits, cudaStream_t stream);  // prolog.cu

constexpr int prolog_tc_splits() { return kPrologKSplits; }  // 7 reduction chunks of 64 per CTA

// The Q path and the K/W path of the prolog are independent (64 and 16 CTAs per 128 tokens, both latency-
// bound), so the Q kernel runs on a side stream of the library, forked from and joined back into the caller's
// stream with events; the pattern is legal under stream capture.  One side stream and event pair per device,
// created on the first call for that device (make that call outside a capture: creating a stream is not a
// capturable operation).
struct PrologFork {
  cudaStream_t side = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};
static PrologFork* prolog_fork_for_device() {
  static PrologFork forks[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  PrologFork& f = forks[dev];
  if (f.side == nullptr) {
    if (cudaStreamCreateWithFlags(&f.side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&f.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&f.join, cudaEventDisableTiming) != cudaSuccess) {
      (void)cudaGetLastError();
      f = PrologFork{};
      return nullptr;  // fall back to one stream
    }
  }
  return &f;
}

int launch_prolog_tc(const PrologParams& p, cudaStream_t stream) {
  if (p.t <= 0) return DSV32_OK;
  const int tiles = (p.t + 127) / 128;
  CUtensorMap qn_map, w_map, h_map, x_map, wk_map, wp_map;
  int rc = make_tensor_map_2d_u8(&qn_map, p.q_norm, p.t, 1536, 128, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&w_map, p.w_qb, 1536, 8192, 128, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&h_map, p.had_q, 128, 256, 128, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&x_map, p.x, p.t, 7168 * 2, 128, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&wk_map, p.wk, 7168, 256, 64, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&wp_map, p.w_proj, 7168, 128, 64, 128);
  if (rc != DSV32_OK) return rc;
  PrologFork* fk = prolog_fork_for_device();
  cudaStream_t q_stream = stream;
  if (fk != nullptr) {
    if (cudaEventRecord(fk->fork, stream) == cudaSuccess && cudaStreamWaitEvent(fk->side, fk->fork, 0) == cudaSuccess) {
      q_stream = fk->side;
    } else {
      (void)cudaGetLastError();
      fk = nullptr;
    }
  }
  cudaFuncSetAttribute(prolog_q_tc_kernel<kVariantV32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPqSmemBytes);
  prolog_q_tc_kernel<kVariantV32><<<dim3(64, tiles), kPqThreads, kPqSmemBytes, q_stream>>>(qn_map, w_map, h_map, p);
  count_launch();
  rc = check_launch("prolog_q_tc_kernel");
  if (fk != nullptr && cudaEventRecord(fk->join, fk->side) != cudaSuccess) rc = check_launch("prolog side stream");
  if (rc == DSV32_OK) {
    const int splits = prolog_tc_splits();
    const int per = (kKwChunksTotal + splits - 1) / splits;
    cudaFuncSetAttribute(prolog_kw_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kKwSmemBytes);
    prolog_kw_tc_kernel<<<dim3(splits, tiles), kPqThreads, kKwSmemBytes, stream>>>(x_map, wk_map, wp_map, p, per);
    count_launch();
    rc = check_launch("prolog_kw_tc_kernel");
    if (rc == DSV32_OK) rc = launch_prolog_finish(p, splits, stream);
  }
  // always join, also after an error above: the caller's stream must not run ahead of the side stream
  if (fk != nullptr && cudaStreamWaitEvent(stream, fk->join, 0) != cudaSuccess && rc == DSV32_OK)
    rc = check_launch("prolog side stream join");
  return rc;
}

// ---------------------------------------------------------------------------------------------------------
// DeepSeek-V4 indexer prolog: head weights = fp16( float(bf16(x . w_proj)) * scale )
// (lightning_indexer_prolog_quant_v4_impl.py:253-266).  The reduction over the hidden size is split into slices of
// 512 and the tokens into tiles of 16: a CTA stages its 16 x 512 piece of x in shared memory (as floats) and
// thread (k group, head) walks a quarter of the slice, reading one weight (coalesced over the 64 heads) for 16
// fused multiply-adds with broadcast x values.  Partial sums [slice][token][head] are added in a fixed order by
// the finish kernel, which rounds to bf16, scales and writes fp16.
// ---------------------------------------------------------------------------------------------------------
constexpr int kW4Tok = 16, kW4Slice = 512, kW4Threads = 256;

__global__ void __launch_bounds__(kW4Threads) prolog_v4_weights_partial_kernel(const __nv_bfloat16* __restrict__ x,
                                                                               const __nv_bfloat16* __restrict__ w_proj,
                                                                               float* __restrict__ partial, int t, int h) {
  __shared__ __align__(16) float x_s[kW4Tok * kW4Slice];   // 32 KB
  __shared__ float red_s[3 * kW4Tok * 64];                 // 12 KB
  const int tid = threadIdx.x;
  const int t0 = blockIdx.x * kW4Tok, k0 = blockIdx.y * kW4Slice;
  const int klen = min(kW4Slice, h - k0);
  for (int i = tid; i < kW4Tok * kW4Slice; i += kW4Threads) {
    const int tok = i / kW4Slice, k = i % kW4Slice;
    x_s[i] = (t0 + tok < t && k < klen) ? __bfloat162float(x[static_cast<size_t>(t0 + tok) * h + k0 + k]) : 0.f;
  }
  __syncthreads();
  const int n = tid & 63, kg = tid >> 6;
  float acc[kW4Tok];
#pragma unroll
  for (int i = 0; i < kW4Tok; ++i) acc[i] = 0.f;
  const int kb = kg * (kW4Slice / 4), ke = min(kb + kW4Slice / 4, klen);
  const __nv_bfloat16* wp = w_proj + static_cast<size_t>(k0) * 64 + n;
  int k = kb;
  for (; k + 4 <= ke; k += 4) {
    const float w0 = __bfloat162float(wp[static_cast<size_t>(k) * 64]), w1 = __bfloat162float(wp[static_cast<size_t>(k + 1) * 64]);
    const float w2 = __bfloat162float(wp[static_cast<size_t>(k + 2) * 64]), w3 = __bfloat162float(wp[static_cast<size_t>(k + 3) * 64]);
#pragma unroll
    for (int i = 0; i < kW4Tok; ++i) {
      const float4 xv = *reinterpret_cast<const float4*>(&x_s[i * kW4Slice + k]);   // broadcast
      acc[i] = fmaf(xv.x, w0, acc[i]);
      acc[i] = fmaf(xv.y, w1, acc[i]);
      acc[i] = fmaf(xv.z, w2, acc[i]);
      acc[i] = fmaf(xv.w, w3, acc[i]);
    }
  }
  for (; k < ke; ++k) {
    const float w0 = __bfloat162float(wp[static_cast<size_t>(k) * 64]);
#pragma unroll
    for (int i = 0; i < kW4Tok; ++i) acc[i] = fmaf(x_s[i * kW4Slice + k], w0, acc[i]);
  }
  if (kg > 0) {
#pragma unroll
    for (int i = 0; i < kW4Tok; ++i) red_s[((kg - 1) * kW4Tok + i) * 64 + n] = acc[i];
  }
  __syncthreads();
  if (kg == 0) {
#pragma unroll
    for (int i = 0; i < kW4Tok; ++i) {
      if (t0 + i < t) {
        const float s = ((acc[i] + red_s[i * 64 + n]) + red_s[(kW4Tok + i) * 64 + n]) + red_s[(2 * kW4Tok + i) * 64 + n];
        partial[(static_cast<size_t>(blockIdx.y) * t + t0 + i) * 64 + n] = s;
      }
    }
  }
}

__global__ void __launch_bounds__(64) prolog_v4_weights_finish_kernel(const float* __restrict__ partial,
                                                                      __half* __restrict__ weights, int t, int slices,
                                                                      float scale) {
  const int tok = blockIdx.x, n = threadIdx.x;
  float s = 0.f;
  for (int g = 0; g < slices; ++g) s += partial[(static_cast<size_t>(g) * t + tok) * 64 + n];
  weights[static_cast<size_t>(tok) * 64 + n] = __float2half_rn(__fmul_rn(bf16_round(s), scale));
}

size_t prolog_v4_workspace_bytes(int t, int h) {
  if (t <= 0 || h <= 0) return 0;
  return static_cast<size_t>((h + kW4Slice - 1) / kW4Slice) * t * 64 * sizeof(float);
}

int launch_prolog_v4(const PrologParams& p, int h, float w_scale, cudaStream_t stream) {
  if (p.t <= 0) return DSV32_OK;
  const int tiles = (p.t + 127) / 128;
  CUtensorMap qn_map, w_map, h_map;
  int rc = make_tensor_map_2d_u8(&qn_map, p.q_norm, p.t, 1024, 128, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&w_map, p.w_qb, 1024, 8192, 128, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&h_map, p.had_q, 128, 256, 128, 128);
  if (rc != DSV32_OK) return rc;
  // the Q path and the weights path are independent: fork the weights kernel onto the side stream
  PrologFork* fk = prolog_fork_for_device();
  cudaStream_t w_stream = stream;
  if (fk != nullptr) {
    if (cudaEventRecord(fk->fork, stream) == cudaSuccess && cudaStreamWaitEvent(fk->side, fk->fork, 0) == cudaSuccess) {
      w_stream = fk->side;
    } else {
      (void)cudaGetLastError();
      fk = nullptr;
    }
  }
  const int slices = (h + kW4Slice - 1) / kW4Slice;
  prolog_v4_weights_partial_kernel<<<dim3((p.t + kW4Tok - 1) / kW4Tok, slices), kW4Threads, 0, w_stream>>>(
      p.x, p.w_proj, p.partial, p.t, h);
  count_launch();
  rc = check_launch("prolog_v4_weights_partial_kernel");
  if (rc == DSV32_OK) {
    prolog_v4_weights_finish_kernel<<<p.t, 64, 0, w_stream>>>(p.partial, p.weights, p.t, slices, w_scale);
    count_launch();
    rc = check_launch("prolog_v4_weights_finish_kernel");
  }
  if (fk != nullptr && cudaEventRecord(fk->join, fk->side) != cudaSuccess) rc = check_launch("prolog side stream");
  if (rc == DSV32_OK) {
    cudaFuncSetAttribute(prolog_q_tc_kernel<kVariantV4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPqSmemBytes);
    prolog_q_tc_kernel<kVariantV4><<<dim3(64, tiles), kPqThreads, kPqSmemBytes, stream>>>(qn_map, w_map, h_map, p);
    count_launch();
    rc = check_launch("prolog_q_tc_kernel (v4)");
  }
  if (fk != nullptr && cudaStreamWaitEvent(stream, fk->join, 0) != cudaSuccess && rc == DSV32_OK)
    rc = check_launch("prolog side stream join");
  return rc;
}

}  // namespace dsv32

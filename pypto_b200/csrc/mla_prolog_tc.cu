// The four projections of the MLA prolog (quant) on tcgen05 tensor cores -- the MLA half of
// mla_indexer_prolog_quant (models/deepseek_v32_exp/mla_indexer_prolog_quant_impl.py:112-211; projections
// mla_prolog_quant_impl.py:452-459 x.w_dq, :480 q_norm.w_uq_qr, :499-509 x.w_dkv_kr, :667 q_nope.w_uk; golden
// deepseekv32_mla_indexer_prolog_quant.py:395-539).
//
// One kernel template, three instantiations.  A CTA computes D[128 tokens x N] = A[tokens, k range] x B[k range, N]
// with the activations K-major (row-major [tokens, K]) and the weights MN-major (row-major [K, N], as the caller
// holds them), both streamed by TMA (128-byte swizzle, never multicast) through a ring of shared-memory stages;
// the accumulator lives in tensor memory and every epilogue thread owns one token row.
//   kXproj  bf16  x[t,7168] x [w_dq | w_dkv_kr] (2112 columns in 17 tiles of 128), the reduction split over eight CTAs;
//                 fp32 partial sums go to the workspace (finished by mla_finish_kernel)
//   kQb     int8  q_norm[t,1536] x w_uq_qr[1536, 128 heads x 192], 256 columns per CTA; the epilogue dequantises
//                 (x q_norm_scale x w_qb_scale -> bf16), sends the 128 "nope" dims of a head to a compact
//                 [t,128,128] buffer and the 64 "rope" dims through the de-interleaving rotary embedding to q_rope
//   kUk     bf16  per head: nope[t,128] x w_uk[head][128,512] (one CTA per head) -> q_nope[t,128,512] bf16
// The weights (85 MB) are read once; the projections are bound by that stream, not by arithmetic.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace dsv32 {

constexpr int kGemmThreads = 192;   // warp 0: TMA producer, warp 1: MMA issuer + tensor-memory owner, 2..5: epilogue
constexpr int kMlaH = 7168, kMlaQLora = 1536, kMlaHeads = 128, kMlaNope = 128, kMlaRope = 64, kMlaLora = 512;

enum { kXproj = 0, kQb = 1, kUk = 2, kI8 = 3 };

struct MlaGemmParams {
  float* partial;                  // kXproj out: [kMlaXSplits][t][kMlaXCols]
  const float* q_norm_scale;       // kQb: [t]
  const float* w_qb_scale;         // kQb: [24576]
  const __nv_bfloat16* cos;        // kQb: [t, 64]
  const __nv_bfloat16* sin;
  __nv_bfloat16* q_nope_in;        // kQb out / kUk in: [t, 128, 128]
  __nv_bfloat16* q_rope;           // kQb out: [t, 128, 64]
  __nv_bfloat16* q_nope;           // kUk out: [t, 128, 512]
  uint32_t* status;
  int t;
  // kXproj: reduction chunks (of 64) per CTA, row stride of a partial slab in floats, and the first column tile
  // that reads the second weight matrix
  int k_chunks, ldc, tile_switch;
  int b_kmajor;                    // kXproj: the weights are held as [n, k] (each row one output column) instead of [k, n]
  int32_t* c_i32;                  // kI8 out: [t, ldc] int32 (ldc = n, a multiple of 256); k_chunks = k / 128
};

template <int kKind>
struct GemmShape {
  static constexpr bool kInt8 = kKind == kQb || kKind == kI8;
  // 128-byte column chunks of B per stage: 128 / 256 / 512 columns per CTA.  Few, wide CTAs with deep rings: what
  // bounds these kernels is the bytes of weights one SM keeps in flight, not the number of CTAs.
  static constexpr int kNChunks = kKind == kUk ? 8 : 2;
  static constexpr int kN = kNChunks * (kInt8 ? 128 : 64);
  static constexpr int kMmaN = kN > 256 ? 256 : kN;                   // columns per MMA instruction
  static constexpr int kKRows = kInt8 ? 128 : 64;                     // reduction elements per stage (128 B of A)
  static constexpr int kABytes = 128 * 128;
  static constexpr int kBChunk = kKRows * 128;
  static constexpr int kStageBytes = kABytes + kNChunks * kBChunk;    // 32 / 48 / 80 KB
  static constexpr int kStages = kKind == kXproj ? 6 : (kInt8 ? 4 : 2);
  static constexpr int kChunksTotal = kKind == kXproj ? kMlaH / 64 : (kKind == kQb ? kMlaQLora / 128 : kMlaNope / 64);
  static constexpr int kOffWs = kStages * kStageBytes;                // kQb: 256 column scales
  static constexpr int kOffBars = kOffWs + 1024;
  static constexpr int kOffTmem = kOffBars + (2 * kStages + 1) * 8;
  static constexpr size_t kSmemBytes = kOffTmem + 16 + 1024;          // slack for manual 1024-byte alignment
  static constexpr uint32_t kTmemCols = kN < 32 ? 32 : kN;
};
constexpr int kMlaXTilesQ = kMlaQLora / 128;                          // 12 column tiles of w_dq, then 5 of w_dkv_kr
constexpr int kMlaXTiles = kMlaXCols / 128;                           // (the last one half past the matrix: zero-filled)

__device__ __forceinline__ float mla_bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <int kKind>
__global__ void __launch_bounds__(kGemmThreads, 1)
mla_gemm_tc_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map0,
                   const __grid_constant__ CUtensorMap b_map1, MlaGemmParams p) {
  using Sh = GemmShape<kKind>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* ws_s = reinterpret_cast<float*>(smem + Sh::kOffWs);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Sh::kOffBars);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Sh::kStages;
  uint64_t* d_bar = bars + 2 * Sh::kStages;
  uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(smem + Sh::kOffTmem);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = blockIdx.x;          // kXproj: column tile of 128; kQb: column tile of 256 (two of 128); kUk: head
  const int split = blockIdx.y;         // kXproj only
  const int t0 = blockIdx.z * 128;
  // reduction chunks of this CTA
  int c_begin = 0, nchunks = Sh::kChunksTotal;
  if constexpr (kKind == kXproj) {
    c_begin = split * p.k_chunks;
    nchunks = p.k_chunks;
  } else if constexpr (kKind == kI8) {
    nchunks = p.k_chunks;
  }

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&a_map);
      tma_prefetch_desc(&b_map0);
      if constexpr (kKind == kXproj) tma_prefetch_desc(&b_map1);
      for (int i = 0; i < Sh::kStages; ++i) {
        mbar_init(&full_bar[i], 1);
        mbar_init(&empty_bar[i], 1);
      }
      mbar_init(d_bar, 1);
      mbar_fence_init();
    }
  } else if (warp == 1) {
    tmem_alloc(tmem_ptr_s, Sh::kTmemCols);
    tmem_relinquish();
  } else if constexpr (kKind == kQb) {
    ws_s[tid - 64] = p.w_qb_scale[tile * 256 + (tid - 64)];
    ws_s[tid + 64] = p.w_qb_scale[tile * 256 + 128 + (tid - 64)];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_s;

  if (warp == 0) {
    // ---- TMA producer -------------------------------------------------------------------------------------
    if (lane == 0) {
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % Sh::kStages;
        if (!mbar_wait(&empty_bar[s], ((c / Sh::kStages) & 1) ^ 1, p.status, 60)) break;
        unsigned char* st = smem + s * Sh::kStageBytes;
        mbar_arrive_expect_tx(&full_bar[s], Sh::kStageBytes);
        const int k0 = (c_begin + c) * Sh::kKRows;   // first reduction element of the chunk
        if constexpr (kKind == kXproj) {
          tma_load_2d(st, &a_map, k0 * 2, t0, &full_bar[s]);
          if (p.b_kmajor) {   // 128 weight rows (output columns) x 64 reduction elements: one 16 KB box, laid out like A
            tma_load_2d(st + Sh::kABytes, &b_map0, k0 * 2, tile * 128, &full_bar[s]);
            continue;
          }
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            if (tile < p.tile_switch) tma_load_2d(st + Sh::kABytes + j * Sh::kBChunk, &b_map0, tile * 256 + j * 128, k0, &full_bar[s]);
            else tma_load_2d(st + Sh::kABytes + j * Sh::kBChunk, &b_map1, (tile - p.tile_switch) * 256 + j * 128, k0, &full_bar[s]);
          }
        } else if constexpr (Sh::kInt8) {
          tma_load_2d(st, &a_map, k0, t0, &full_bar[s]);
#pragma unroll
          for (int j = 0; j < 2; ++j)
            tma_load_2d(st + Sh::kABytes + j * Sh::kBChunk, &b_map0, tile * 256 + j * 128, k0, &full_bar[s]);
        } else {
          tma_load_2d(st, &a_map, tile * 256 + k0 * 2, t0, &full_bar[s]);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            tma_load_2d(st + Sh::kABytes + j * Sh::kBChunk, &b_map0, j * 128, tile * kMlaNope + k0, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the whole warp runs the loop (uniform operands), lane 0 issues ---------------------------
    const bool leader = lane == 0;
    constexpr uint32_t idesc_mn = Sh::kInt8 ? umma_idesc_i8(128, Sh::kMmaN, true) : umma_idesc_bf16(128, Sh::kMmaN, false, true);
    constexpr uint32_t idesc_k = umma_idesc_bf16(128, Sh::kMmaN, false, false);
    const bool b_kmajor = kKind == kXproj && p.b_kmajor != 0;
    const uint32_t idesc = b_kmajor ? idesc_k : idesc_mn;
    const uint32_t tbase = __shfl_sync(0xffffffffu, tmem_base, 0);
    bool ok = true;
    for (int c = 0; c < nchunks; ++c) {
      const int s = c % Sh::kStages;
      ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], (c / Sh::kStages) & 1, p.status, 61));
      if (!ok) break;
      tc_fence_after();
      const uint32_t a_s = smem_u32(smem + s * Sh::kStageBytes), b_s = a_s + Sh::kABytes;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {  // 32 bytes of A's row per instruction: 32 int8 / 16 bf16 reduction elements
        const uint64_t ad = umma_smem_desc_sw128(a_s + ks * 32, 16, 1024);
        const uint32_t acc = (c > 0 || ks > 0) ? 1u : 0u;
#pragma unroll
        for (int h = 0; h < Sh::kN / Sh::kMmaN; ++h) {  // 512 columns: two instructions of 256
          const uint64_t bd = b_kmajor ? umma_smem_desc_sw128(b_s + ks * 32, 16, 1024)
                                       : umma_smem_desc_sw128(b_s + h * (Sh::kMmaN / (Sh::kInt8 ? 128 : 64)) * Sh::kBChunk +
                                                                  ks * (Sh::kInt8 ? 4096 : 2048), Sh::kBChunk, 1024);
          if constexpr (Sh::kInt8) {
            asm volatile(
                "{\n\t.reg .pred pa, pl;\n\tsetp.ne.b32 pa, %4, 0;\n\tsetp.ne.b32 pl, %5, 0;\n\t"
                "@pl tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, pa;\n\t}" ::"r"(tbase + h * Sh::kMmaN),
                "l"(ad), "l"(bd), "r"(idesc), "r"(acc), "r"(static_cast<uint32_t>(leader))
                : "memory");
          } else {
            umma_f16_ss_if(leader, tbase + h * Sh::kMmaN, ad, bd, idesc, acc);
          }
        }
      }
      umma_commit_if(leader, &empty_bar[s]);
    }
    if (ok) umma_commit_if(leader, d_bar);
  } else {
    // ---- epilogue: thread = token row (tensor-memory lane quarter = warp % 4) ------------------------------------
    const int quarter = warp & 3;
    const int tok = t0 + quarter * 32 + lane;
    const bool live = tok < p.t;
    const int tk = live ? tok : 0;  // clamp for loads
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    if (__all_sync(0xffffffffu, mbar_wait(d_bar, 0, p.status, 62))) {
      tc_fence_after();
      if constexpr (kKind == kXproj) {
        float* prow = p.partial + (static_cast<size_t>(split) * p.t + tk) * p.ldc + tile * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + c * 32, r);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(prow + c * 32 + j) =
                  make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                              __uint_as_float(r[j + 3]));
          }
        }
      } else if constexpr (kKind == kI8) {
        int32_t* crow = p.c_i32 + static_cast<size_t>(tk) * p.ldc + tile * 256;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + c * 32, r);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<uint4*>(crow + c * 32 + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
          }
        }
      } else if constexpr (kKind == kQb) {
        // 384 columns = two heads: column tile 3j is the nope part of head 2j, tile 3j+1 its rope part followed by
        // nope dims 0..63 of head 2j+1, tile 3j+2 nope dims 64..127 of head 2j+1 followed by its rope part.
        const float qs = p.q_norm_scale[tk];
#pragma unroll 1
        for (int sub = 0; sub < 2; ++sub) {   // the CTA's 256 columns are two tiles of 128
        const int tile128 = tile * 2 + sub;
        const int m = tile128 % 3, pair = tile128 / 3;
        auto dequant32 = [&](int g, float (&v)[32]) {  // columns 32g .. 32g+31 of the tile -> bf16-rounded floats
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + sub * 128 + g * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = mla_bf16r(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(r[j])), qs), ws_s[sub * 128 + g * 32 + j]));
        };
        auto store_nope32 = [&](int head, int d0, const float (&v)[32]) {  // nope dims d0 .. d0+31 of `head`
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 32; j += 2) w[j >> 1] = pack_bf16x2(v[j], v[j + 1]);
          if (live) {
            uint4* dst = reinterpret_cast<uint4*>(p.q_nope_in + (static_cast<size_t>(tk) * kMlaHeads + head) * kMlaNope + d0);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          }
        };
        // De-interleave (even dims, then odd dims) and rotate-half rotary embedding: out[j] = x[2j] cos[j] - x[2j+1] sin[j]
        // for j < 32, out[j] = x[2(j-32)+1] cos[j] + x[2(j-32)] sin[j] for j >= 32; products and sum rounded separately.
        auto rope_store = [&](int head, const float (&xa)[32], const float (&xb)[32]) {  // xa = x[0..31], xb = x[32..63]
          const uint32_t* cw = reinterpret_cast<const uint32_t*>(p.cos + static_cast<size_t>(tk) * kMlaRope);
          const uint32_t* sw = reinterpret_cast<const uint32_t*>(p.sin + static_cast<size_t>(tk) * kMlaRope);
          uint32_t w[32];
#pragma unroll
          for (int jp = 0; jp < 16; ++jp) {  // output pairs (2jp, 2jp+1) of the first half and (32+2jp, 33+2jp) of the second
            const uint32_t c_lo = __ldg(cw + jp), s_lo = __ldg(sw + jp), c_hi = __ldg(cw + 16 + jp), s_hi = __ldg(sw + 16 + jp);
            float o_lo[2], o_hi[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int j = 2 * jp + e;                  // j < 32; inputs x[2j], x[2j+1]
              const float xe = (2 * j < 32) ? xa[(2 * j) & 31] : xb[(2 * j) & 31];
              const float xo = (2 * j + 1 < 32) ? xa[(2 * j + 1) & 31] : xb[(2 * j + 1) & 31];
              const float cl = __uint_as_float(e ? (c_lo & 0xffff0000u) : (c_lo << 16));
              const float sl = __uint_as_float(e ? (s_lo & 0xffff0000u) : (s_lo << 16));
              const float ch = __uint_as_float(e ? (c_hi & 0xffff0000u) : (c_hi << 16));
              const float sh = __uint_as_float(e ? (s_hi & 0xffff0000u) : (s_hi << 16));
              o_lo[e] = __fadd_rn(__fmul_rn(xe, cl), __fmul_rn(-xo, sl));
              o_hi[e] = __fadd_rn(__fmul_rn(xo, ch), __fmul_rn(xe, sh));
            }
            w[jp] = pack_bf16x2(o_lo[0], o_lo[1]);
            w[16 + jp] = pack_bf16x2(o_hi[0], o_hi[1]);
          }
          if (live) {
            uint4* dst = reinterpret_cast<uint4*>(p.q_rope + (static_cast<size_t>(tk) * kMlaHeads + head) * kMlaRope);
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          }
        };
        float va[32], vb[32];
        if (m == 0) {
#pragma unroll 1
          for (int g = 0; g < 4; ++g) {
            dequant32(g, va);
            store_nope32(2 * pair, g * 32, va);
          }
        } else if (m == 1) {
          dequant32(0, va);
          dequant32(1, vb);
          rope_store(2 * pair, va, vb);
          dequant32(2, va);
          store_nope32(2 * pair + 1, 0, va);
          dequant32(3, va);
          store_nope32(2 * pair + 1, 32, va);
        } else {
          dequant32(0, va);
          store_nope32(2 * pair + 1, 64, va);
          dequant32(1, va);
          store_nope32(2 * pair + 1, 96, va);
          dequant32(2, va);
          dequant32(3, vb);
          rope_store(2 * pair + 1, va, vb);
        }
        }
      } else {
        __nv_bfloat16* orow = p.q_nope + (static_cast<size_t>(tk) * kMlaHeads + tile) * kMlaLora;
#pragma unroll 1
        for (int c = 0; c < 16; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + c * 32, r);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
              *reinterpret_cast<uint4*>(orow + c * 32 + j) = v;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, Sh::kTmemCols);
  }
}

template <int kKind>
static int launch_gemm(const CUtensorMap& a_map, const CUtensorMap& b0, const CUtensorMap& b1, const MlaGemmParams& gp,
                       dim3 grid, cudaStream_t stream, const char* what) {
  using Sh = GemmShape<kKind>;
  cudaFuncSetAttribute(mla_gemm_tc_kernel<kKind>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Sh::kSmemBytes);
  mla_gemm_tc_kernel<kKind><<<grid, kGemmThreads, Sh::kSmemBytes, stream>>>(a_map, b0, b1, gp);
  count_launch();
  return check_launch(what);
}

size_t mla_prolog_workspace_bytes(int t) {
  if (t <= 0) return 0;
  const size_t partial = static_cast<size_t>(kMlaXSplits) * t * kMlaXCols * sizeof(float);
  const size_t nope_in = static_cast<size_t>(t) * kMlaHeads * kMlaNope * sizeof(__nv_bfloat16);
  return (partial + 255) / 256 * 256 + (nope_in + 255) / 256 * 256;
}

// The MLA prolog on one stream: x projections -> (RMSNorm + int8 quantisation -> q_b projection with dequantisation
// and rotary embedding -> w_uk projection) and (RMSNorm + cache quantisation + rotary embedding + cache scatter).
int launch_mla_prolog(const MlaParams& p, cudaStream_t stream) {
  if (p.t <= 0) return DSV32_OK;
  const int tiles = (p.t + 127) / 128;
  char* ws = static_cast<char*>(p.workspace);
  float* partial = reinterpret_cast<float*>(ws);
  const size_t partial_bytes = (static_cast<size_t>(kMlaXSplits) * p.t * kMlaXCols * sizeof(float) + 255) / 256 * 256;
  __nv_bfloat16* nope_in = reinterpret_cast<__nv_bfloat16*>(ws + partial_bytes);

  CUtensorMap x_map, wdq_map, wkv_map, qn_map, wqb_map, ni_map, wuk_map;
  int rc = make_tensor_map_2d_u8(&x_map, p.x, p.t, kMlaH * 2, 128, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&wdq_map, p.w_dq, kMlaH, kMlaQLora * 2, 64, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&wkv_map, p.w_dkv_kr, kMlaH, (kMlaLora + kMlaRope) * 2, 64, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&qn_map, p.q_norm, p.t, kMlaQLora, 128, 128);
  if (rc == DSV32_OK)
    rc = make_tensor_map_2d_u8(&wqb_map, p.w_uq_qr, kMlaQLora, kMlaHeads * (kMlaNope + kMlaRope), 128, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&ni_map, nope_in, p.t, kMlaHeads * kMlaNope * 2, 128, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&wuk_map, p.w_uk, kMlaHeads * kMlaNope, kMlaLora * 2, 64, 128);
  static_assert(kMlaXTiles * 128 == kMlaXCols && kMlaXTilesQ * 128 == kMlaQLora, "column tiles of the x projections");
  if (rc != DSV32_OK) return rc;

  MlaGemmParams gp{};
  gp.partial = partial;
  gp.q_norm_scale = p.q_norm_scale;
  gp.w_qb_scale = p.w_qb_scale;
  gp.cos = p.cos;
  gp.sin = p.sin;
  gp.q_nope_in = nope_in;
  gp.q_rope = p.q_rope;
  gp.q_nope = p.q_nope;
  gp.status = p.status;
  gp.t = p.t;
  gp.k_chunks = GemmShape<kXproj>::kChunksTotal / kMlaXSplits;
  gp.ldc = kMlaXCols;
  gp.tile_switch = kMlaXTilesQ;

  rc = launch_gemm<kXproj>(x_map, wdq_map, wkv_map, gp, dim3(kMlaXTiles, kMlaXSplits, tiles), stream,
                           "mla_gemm_tc_kernel (x projections)");
  if (rc != DSV32_OK) return rc;
  MlaStageParams sp{};
  sp.partial = partial;
  sp.gamma_cq = p.gamma_cq;
  sp.q_norm = p.q_norm;
  sp.q_norm_scale = p.q_norm_scale;
  sp.gamma_ckv = p.gamma_ckv;
  sp.cos = p.cos;
  sp.sin = p.sin;
  sp.cache_index = p.cache_index;
  sp.kv_cache = p.kv_cache;
  sp.kr_cache = p.kr_cache;
  sp.k_scale_cache = p.k_scale_cache;
  sp.status = p.status;
  sp.cache_rows = p.cache_rows;
  sp.t = p.t;
  sp.eps_cq = p.eps_cq;
  sp.eps_ckv = p.eps_ckv;
  rc = launch_mla_finish(sp, stream);
  if (rc != DSV32_OK) return rc;
  rc = launch_gemm<kQb>(qn_map, wqb_map, wqb_map, gp, dim3(kMlaHeads * (kMlaNope + kMlaRope) / 256, 1, tiles), stream,
                        "mla_gemm_tc_kernel (q_norm . w_uq_qr)");
  if (rc != DSV32_OK) return rc;
  return launch_gemm<kUk>(ni_map, wuk_map, wuk_map, gp, dim3(kMlaHeads, 1, tiles), stream,
                          "mla_gemm_tc_kernel (q_nope . w_uk)");
}

// The same bf16 kernel as a building block: fp32 partial sums, one [t, ldc] slab per reduction split, of
// A[t, k] (row-major) x B for column tiles 0 .. n_tiles-1 of 128, where B is [k, b_cols] row-major, or with
// b_kmajor [b_cols, k] row-major (one row per output column; rows past b_cols read as zero).  k must be a multiple
// of 64 * splits; both matrices 16-byte aligned with rows that are multiples of 16 bytes.
int launch_bf16_gemm_partial(const __nv_bfloat16* a, int t, int k, const __nv_bfloat16* b, int b_cols, int n_tiles,
                             int splits, float* partial, int ldc, uint32_t* status, cudaStream_t stream, bool b_kmajor) {
  if (t <= 0) return DSV32_OK;
  if (k <= 0 || splits <= 0 || k % (64 * splits) != 0 || ldc < n_tiles * 128) {
    set_error("bf16 gemm: k=%d must be a multiple of 64 x %d splits and ldc=%d must hold %d column tiles", k, splits, ldc, n_tiles);
    return DSV32_ERR_INVALID_ARG;
  }
  CUtensorMap a_map, b_map;
  int rc = make_tensor_map_2d_u8(&a_map, a, t, static_cast<uint64_t>(k) * 2, 128, 128);
  if (rc == DSV32_OK) {
    if (b_kmajor) rc = make_tensor_map_2d_u8(&b_map, b, b_cols, static_cast<uint64_t>(k) * 2, 128, 128);
    else rc = make_tensor_map_2d_u8(&b_map, b, k, static_cast<uint64_t>(b_cols) * 2, 64, 128);
  }
  if (rc != DSV32_OK) return rc;
  MlaGemmParams gp{};
  gp.partial = partial;
  gp.status = status;
  gp.t = t;
  gp.k_chunks = k / 64 / splits;
  gp.ldc = ldc;
  gp.tile_switch = n_tiles;   // every tile reads the one weight matrix
  gp.b_kmajor = b_kmajor ? 1 : 0;
  return launch_gemm<kXproj>(a_map, b_map, b_map, gp, dim3(n_tiles, splits, (t + 127) / 128), stream,
                             "mla_gemm_tc_kernel (bf16 partial sums)");
}

// int32 C[t, n] = int8 A[t, k] (row-major) x int8 B[k, n] (row-major): k a multiple of 128, n of 256.
int launch_i8_gemm(const int8_t* a, int t, int k, const int8_t* b, int n, int32_t* c, uint32_t* status, cudaStream_t stream) {
  if (t <= 0) return DSV32_OK;
  if (k <= 0 || k % 128 != 0 || n <= 0 || n % 256 != 0) {
    set_error("int8 gemm: k=%d must be a positive multiple of 128 and n=%d of 256", k, n);
    return DSV32_ERR_INVALID_ARG;
  }
  CUtensorMap a_map, b_map;
  int rc = make_tensor_map_2d_u8(&a_map, a, t, k, 128, 128);
  if (rc == DSV32_OK) rc = make_tensor_map_2d_u8(&b_map, b, k, n, 128, 128);
  if (rc != DSV32_OK) return rc;
  MlaGemmParams gp{};
  gp.status = status;
  gp.t = t;
  gp.k_chunks = k / 128;
  gp.ldc = n;
  gp.c_i32 = c;
  return launch_gemm<kI8>(a_map, b_map, b_map, gp, dim3(n / 256, 1, (t + 127) / 128), stream, "mla_gemm_tc_kernel (int8)");
}

// out[t, n] (fp32, or bf16 with one rounding) = sum over the reduction splits, in order, of the fp32 slabs [t, ldp]
__global__ void __launch_bounds__(256) gemm_reduce_kernel(const float* partial, int splits, int t, int ldp, int n, void* out,
                                                          int out_bf16) {
  const long long total = static_cast<long long>(t) * n;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * 256) {
    const long long row = i / n, col = i % n;
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[(static_cast<size_t>(s) * t + row) * ldp + col];
    if (out_bf16) static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(acc);
    else static_cast<float*>(out)[i] = acc;
  }
}

static int gemm_splits(int t, int k, int n) {
  const int chunks = k / 64, ctas = ((n + 127) / 128) * ((t + 127) / 128);
  int best = 1;
  for (int s = 1; s <= 16; ++s)
    if (chunks % s == 0 && ctas * s <= 296) best = s;   // at most two CTAs' worth of work per SM
  return best;
}

size_t bf16_gemm_workspace_bytes(int t, int k, int n) {
  if (t <= 0 || k <= 0 || n <= 0 || k % 64 != 0) return 0;
  const size_t ldp = static_cast<size_t>((n + 127) / 128) * 128;
  return (static_cast<size_t>(gemm_splits(t, k, n)) * t * ldp * sizeof(float) + 255) / 256 * 256;
}

int launch_bf16_gemm(const __nv_bfloat16* a, int t, int k, const __nv_bfloat16* b, int n, bool b_kmajor, void* out,
                     bool out_bf16, void* workspace, uint32_t* status, cudaStream_t stream) {
  if (t <= 0) return DSV32_OK;
  const int splits = gemm_splits(t, k, n), n_tiles = (n + 127) / 128, ldp = n_tiles * 128;
  float* partial = static_cast<float*>(workspace);
  int rc = launch_bf16_gemm_partial(a, t, k, b, n, n_tiles, splits, partial, ldp, status, stream, b_kmajor);
  if (rc != DSV32_OK) return rc;
  const long long total = static_cast<long long>(t) * n;
  const long long blocks = (total + 255) / 256;
  gemm_reduce_kernel<<<static_cast<int>(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, stream>>>(partial, splits, t, ldp, n, out,
                                                                                                out_bf16 ? 1 : 0);
  count_launch();
  return check_launch("gemm_reduce_kernel");
}

}  // namespace dsv32

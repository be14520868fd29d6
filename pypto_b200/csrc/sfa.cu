// Sparse flash attention over the int8 paged latent KV cache (absorbed MLA: 576-d QK^T, 512-d PV).
// Follows models/deepseek_v32_exp/sparse_flash_attention_quant_impl.py:121-286 (golden:
// deepseekv32_sparse_flash_attention_quant.py:174-259).
//
// Warp-MMA implementation (mma.sync m16n8k16 bf16).  One CTA = (token, 64 query heads, key split):
//   gather 32 selected rows -> dequantise to bf16 in shared memory (per 128-dim group scale, rounded to
//   bf16 exactly as the golden does) -> S = Q K^T -> online softmax -> O += P V.
// 8 warps: warp = (head group of 16) x (half).  For S a half is 16 of the tile's 32 keys, for PV it is 256
// of the 512 value dims, so no MMA is computed twice; P and the per-half row maxima are exchanged
// through shared memory.
#include "kernels.cuh"

namespace dsv32 {


constexpr int kSfaThreads = 256;
constexpr int kSfaHeads = 64;      // heads per CTA
constexpr int kSfaTile = 32;       // keys per tile
constexpr int kQkStride = kQkDim * 2 + 16;  // bytes per smem row of Q / K (1168)
constexpr int kPStride = kSfaTile * 2 + 16; // bytes per smem row of P (80)

constexpr size_t kSfaSmemQ = (size_t)kSfaHeads * kQkStride;
constexpr size_t kSfaSmemK = (size_t)kSfaTile * kQkStride;
constexpr size_t kSfaSmemP = (size_t)kSfaHeads * kPStride;
constexpr size_t kSfaSmemBytes = kSfaSmemQ + 2 * kSfaSmemK + kSfaSmemP + (2 * 64 + 2 * 64) * sizeof(float) +
                                 2 * kSfaTile * sizeof(int);

struct TilePrefetch {
  int4 nope[4];
  int4 rope;
  float4 sc;
  bool valid;
};

__device__ __forceinline__ void dequant16(const int4& raw, float sc, uint4& lo, uint4& hi) {
  // 16 int8 -> 16 bf16 = bf16_rn( float(int8) * scale )
  const int w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float f0 = static_cast<float>(static_cast<int8_t>(w[i] & 0xff)) * sc;
    const float f1 = static_cast<float>(static_cast<int8_t>((w[i] >> 8) & 0xff)) * sc;
    const float f2 = static_cast<float>(static_cast<int8_t>((w[i] >> 16) & 0xff)) * sc;
    const float f3 = static_cast<float>(static_cast<int8_t>((w[i] >> 24) & 0xff)) * sc;
    o[2 * i] = pack_bf16x2(f0, f1);
    o[2 * i + 1] = pack_bf16x2(f2, f3);
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

__global__ void __launch_bounds__(kSfaThreads, 1) sfa_mma_kernel(SfaParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* q_s = smem;
  unsigned char* k_s = q_s + kSfaSmemQ;
  unsigned char* p_s = k_s + 2 * kSfaSmemK;
  float* mx_s = reinterpret_cast<float*>(p_s + kSfaSmemP);  // [2][64]
  float* l_s = mx_s + 128;                                  // [2][64]
  int* valid_s = reinterpret_cast<int*>(l_s + 128);         // [2][32]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tig = lane & 3;
  const int hg = warp & 3, half = warp >> 2;
  const int head0 = blockIdx.x * kSfaHeads;
  const int tok = blockIdx.y;
  const int split = blockIdx.z;
  const int bi = tok / p.s1, si = tok % p.s1;
  const int cnt = min(max(p.act_seq[bi] - p.s1 + 1 + si, 0), p.topk);
  const int per = (((cnt + p.splits - 1) / p.splits) + kSfaTile - 1) / kSfaTile * kSfaTile;
  const int k_lo = split * per;
  const int k_hi = min(cnt, k_lo + per);
  const int ntiles = (k_hi > k_lo) ? (k_hi - k_lo + kSfaTile - 1) / kSfaTile : 0;
  const int32_t* idx_row = p.topk_idx + static_cast<size_t>(tok) * p.topk;
  const int32_t* bt = p.block_table + static_cast<size_t>(bi) * p.max_blocks;

  // ---- stage Q ---------------------------------------------------------------------------------
  {
    const __nv_bfloat16* qn = p.q_nope + (static_cast<size_t>(tok) * p.nq + head0) * kKvLora;
    const __nv_bfloat16* qr = p.q_rope + (static_cast<size_t>(tok) * p.nq + head0) * kRopeDim;
    for (int c = tid; c < kSfaHeads * 72; c += kSfaThreads) {
      const int r = c / 72, ch = c % 72;
      const void* src = (ch < 64) ? static_cast<const void*>(qn + r * kKvLora + ch * 8)
                                  : static_cast<const void*>(qr + r * kRopeDim + (ch - 64) * 8);
      cp_async16(q_s + r * kQkStride + ch * 16, src);
    }
    cp_async_commit();
  }

  // gather mapping: thread -> (key = tid/8, part = tid%8); 16-byte chunks part + 8*j, j = 0..3
  const int gkey = tid >> 3, gpart = tid & 7;

  auto prefetch = [&](int tile, TilePrefetch& pf) {
    const int j = k_lo + tile * kSfaTile + gkey;
    pf.valid = false;
    if (j < k_hi) {
      const int idx = idx_row[j];
      if (idx >= 0) {
        const int lb = idx / p.block_size;
        long long row = -1;
        if (lb < p.max_blocks) {
          const int pb = bt[lb];
          row = static_cast<long long>(pb) * p.block_size + idx % p.block_size;
          if (pb < 0 || row >= p.rows) {
            report_status(p.status, DSV32_STATUS_BAD_PAGE, bi, lb);
            row = -1;
          }
        } else {
          report_status(p.status, DSV32_STATUS_BAD_INDEX, tok, j);
        }
        if (row >= 0) {
          pf.valid = true;
          const int4* src = reinterpret_cast<const int4*>(reinterpret_cast<const unsigned char*>(p.k_nope) + row * p.nope_stride);
#pragma unroll
          for (int q = 0; q < 4; ++q) pf.nope[q] = __ldg(src + gpart + 8 * q);
          pf.rope = __ldg(reinterpret_cast<const int4*>(reinterpret_cast<const unsigned char*>(p.k_rope) + row * p.rope_stride) + gpart);
          pf.sc = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const unsigned char*>(p.k_scales) + row * p.scale_stride));
        }
      }
    }
  };
  auto commit = [&](int tile, const TilePrefetch& pf) {
    unsigned char* dst = k_s + (tile & 1) * kSfaSmemK + gkey * kQkStride;
    if (pf.valid) {
      const float sc[4] = {pf.sc.x, pf.sc.y, pf.sc.z, pf.sc.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 lo, hi;
        dequant16(pf.nope[q], sc[q], lo, hi);
        const int chunk = gpart + 8 * q;  // 16 dims each
        *reinterpret_cast<uint4*>(dst + chunk * 32) = lo;
        *reinterpret_cast<uint4*>(dst + chunk * 32 + 16) = hi;
      }
      *reinterpret_cast<int4*>(dst + 1024 + gpart * 16) = pf.rope;
    } else {
      const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int chunk = gpart + 8 * q;
        *reinterpret_cast<uint4*>(dst + chunk * 32) = z;
        *reinterpret_cast<uint4*>(dst + chunk * 32 + 16) = z;
      }
      *reinterpret_cast<uint4*>(dst + 1024 + gpart * 16) = z;
    }
    if (gpart == 0) valid_s[(tile & 1) * kSfaTile + gkey] = pf.valid ? 1 : 0;
  };

  float o[32][4];
#pragma unroll
  for (int i = 0; i < 32; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};  // rows g, g+8 of this head group
  float l_run[2] = {0.f, 0.f};              // over this warp's S keys only

  TilePrefetch pf;
  if (ntiles > 0) {
    prefetch(0, pf);
    commit(0, pf);
  }
  cp_async_wait<0>();
  __syncthreads();

  const int qrow_base = hg * 16;
  for (int tile = 0; tile < ntiles; ++tile) {
    const unsigned char* kb = k_s + (tile & 1) * kSfaSmemK;
    const bool has_next = (tile + 1 < ntiles);
    if (has_next) prefetch(tile + 1, pf);

    // ---- S = Q K^T for 16 heads x 16 keys (keys half*16 ..) ------------------------------------
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    {
      const uint32_t a_addr =
          smem_u32(q_s + (qrow_base + (lane & 7) + ((lane >> 3) & 1) * 8) * kQkStride + (lane >> 4) * 16);
      const uint32_t b_addr =
          smem_u32(kb + (half * 16 + (lane >> 4) * 8 + (lane & 7)) * kQkStride + ((lane >> 3) & 1) * 16);
#pragma unroll 4
      for (int ks = 0; ks < kQkDim / 16; ++ks) {
        uint32_t a[4], b0, b1, b2, b3;
        ldmatrix_x4(a[0], a[1], a[2], a[3], a_addr + ks * 32);
        ldmatrix_x4(b0, b1, b2, b3, b_addr + ks * 32);
        mma_bf16_16816(s[0], a, b0, b1);
        mma_bf16_16816(s[1], a, b2, b3);
      }
    }
    // scale + mask, tile-local row max over this warp's 16 keys
    const int* vmask = valid_s + (tile & 1) * kSfaTile;
    float mloc[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int kc = half * 16 + nt * 8 + 2 * tig;
      const bool v0 = vmask[kc] != 0, v1 = vmask[kc + 1] != 0;
      s[nt][0] = v0 ? s[nt][0] * p.scale : -INFINITY;
      s[nt][1] = v1 ? s[nt][1] * p.scale : -INFINITY;
      s[nt][2] = v0 ? s[nt][2] * p.scale : -INFINITY;
      s[nt][3] = v1 ? s[nt][3] * p.scale : -INFINITY;
      mloc[0] = fmaxf(mloc[0], fmaxf(s[nt][0], s[nt][1]));
      mloc[1] = fmaxf(mloc[1], fmaxf(s[nt][2], s[nt][3]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mloc[r] = fmaxf(mloc[r], __shfl_xor_sync(0xffffffffu, mloc[r], 1));
      mloc[r] = fmaxf(mloc[r], __shfl_xor_sync(0xffffffffu, mloc[r], 2));
    }
    if (tig == 0) {
      mx_s[half * 64 + qrow_base + g] = mloc[0];
      mx_s[half * 64 + qrow_base + g + 8] = mloc[1];
    }
    __syncthreads();
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = qrow_base + g + r * 8;
      const float m_new = fmaxf(m_run[r], fmaxf(mx_s[row], mx_s[64 + row]));
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[r] = __expf(m_run[r] - m_use[r]);  // m_run = -inf -> 0
      m_run[r] = m_new;
    }
    float lsum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float p0 = __expf(s[nt][0] - m_use[0]);
      const float p1 = __expf(s[nt][1] - m_use[0]);
      const float p2 = __expf(s[nt][2] - m_use[1]);
      const float p3 = __expf(s[nt][3] - m_use[1]);
      lsum[0] += p0 + p1;
      lsum[1] += p2 + p3;
      const int kc = half * 16 + nt * 8 + 2 * tig;
      *reinterpret_cast<uint32_t*>(p_s + (qrow_base + g) * kPStride + kc * 2) = pack_bf16x2(p0, p1);
      *reinterpret_cast<uint32_t*>(p_s + (qrow_base + g + 8) * kPStride + kc * 2) = pack_bf16x2(p2, p3);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      lsum[r] += __shfl_xor_sync(0xffffffffu, lsum[r], 1);
      lsum[r] += __shfl_xor_sync(0xffffffffu, lsum[r], 2);
      l_run[r] = l_run[r] * alpha[r] + lsum[r];
    }
    __syncthreads();

    // ---- O = O*alpha + P V   (16 heads x 256 value dims: dims half*256 ..) ----------------------
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a[0], a[1], a[2], a[3],
                  smem_u32(p_s + (qrow_base + (lane & 7) + ((lane >> 3) & 1) * 8) * kPStride + ks * 32 +
                           (lane >> 4) * 16));
      const uint32_t v_addr = smem_u32(kb + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kQkStride +
                                       (half * 256 + (lane >> 4) * 8) * 2);
#pragma unroll
      for (int np = 0; np < 16; ++np) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, v_addr + np * 32);
        mma_bf16_16816(o[2 * np], a, b0, b1);
        mma_bf16_16816(o[2 * np + 1], a, b2, b3);
      }
    }
    if (has_next) commit(tile + 1, pf);
    __syncthreads();
  }

  // ---- finalize ----------------------------------------------------------------------------------
  if (tig == 0) {
    l_s[half * 64 + qrow_base + g] = l_run[0];
    l_s[half * 64 + qrow_base + g + 8] = l_run[1];
  }
  __syncthreads();
  float inv[2], lse[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = qrow_base + g + r * 8;
    const float l = l_s[row] + l_s[64 + row];
    inv[r] = (l > 0.f) ? 1.f / l : 0.f;
    lse[r] = (l > 0.f) ? m_run[r] + __logf(l) : -INFINITY;
  }
  if (p.splits == 1) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      __nv_bfloat16* orow =
          p.out + (static_cast<size_t>(tok) * p.nq + head0 + qrow_base + g + r * 8) * kKvLora + half * 256;
#pragma unroll
      for (int nt = 0; nt < 32; ++nt) {
        *reinterpret_cast<uint32_t*>(orow + nt * 8 + 2 * tig) =
            pack_bf16x2(o[nt][2 * r] * inv[r], o[nt][2 * r + 1] * inv[r]);
      }
    }
  } else {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const size_t prow = (static_cast<size_t>(tok) * p.splits + split) * p.nq + head0 + qrow_base + g + r * 8;
      float* orow = p.part_o + prow * kKvLora + half * 256;
#pragma unroll
      for (int nt = 0; nt < 32; ++nt) {
        *reinterpret_cast<float2*>(orow + nt * 8 + 2 * tig) =
            make_float2(o[nt][2 * r] * inv[r], o[nt][2 * r + 1] * inv[r]);
      }
      if (half == 0 && tig == 0) p.part_lse[prow] = lse[r];
    }
  }
}

// Split-KV combine: out = sum_s w_s * O_s with w_s = exp(lse_s - max) / sum exp(lse - max).
__global__ void __launch_bounds__(128) sfa_combine_kernel(const float* part_o, const float* part_lse,
                                                          __nv_bfloat16* out, int splits, int nq) {
  const size_t row = blockIdx.x;  // token*nq + head
  const size_t tok = row / nq, head = row % nq;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_lse[(tok * splits + s) * nq + head]);
  float wsum = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float l = part_lse[(tok * splits + s) * nq + head];
    wsum += (l == -INFINITY) ? 0.f : __expf(l - mx);
  }
  const float inv = (wsum > 0.f) ? 1.f / wsum : 0.f;
  const int d = threadIdx.x * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < splits; ++s) {
    const float l = part_lse[(tok * splits + s) * nq + head];
    if (l == -INFINITY) continue;
    const float w = __expf(l - mx) * inv;
    const float4 v = *reinterpret_cast<const float4*>(part_o + ((tok * splits + s) * nq + head) * kKvLora + d);
    acc.x += w * v.x;
    acc.y += w * v.y;
    acc.z += w * v.z;
    acc.w += w * v.w;
  }
  uint2 pk = make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
  *reinterpret_cast<uint2*>(out + row * kKvLora + d) = pk;
}

int launch_sfa_mma(const SfaParams& p, cudaStream_t stream) {
  const int t = p.b * p.s1;
  if (t <= 0) return DSV32_OK;
  cudaFuncSetAttribute(sfa_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSfaSmemBytes);
  dim3 grid(p.nq / kSfaHeads, t, p.splits);
  sfa_mma_kernel<<<grid, kSfaThreads, kSfaSmemBytes, stream>>>(p);
  count_launch();
  int rc = check_launch("sfa_mma_kernel");
  if (rc != DSV32_OK) return rc;
  if (p.splits > 1) rc = launch_sfa_combine(p, stream);
  return rc;
}

int launch_sfa_combine(const SfaParams& p, cudaStream_t stream) {
  const int t = p.b * p.s1;
  sfa_combine_kernel<<<t * p.nq, 128, 0, stream>>>(p.part_o, p.part_lse, p.out, p.splits, p.nq);
  count_launch();
  return check_launch("sfa_combine_kernel");
}

}  // namespace dsv32

// Element-wise stages of the MLA prolog (quant) -- the MLA half of mla_indexer_prolog_quant
// (models/deepseek_v32_exp/mla_indexer_prolog_quant_impl.py:112-211; helpers mla_prolog_quant_impl.py:96-361;
// golden deepseekv32_mla_indexer_prolog_quant.py:395-539) -- that follow the split-reduction projection
// x . [w_dq | w_dkv_kr] of mla_prolog_tc.cu (one launch, blockIdx.y selects the stage): both first add its fp32 partial sums in a fixed order and round
// to bf16 (the reference's q_a / kv_a).
//   stage 0: q_a (columns 0..1535) -> RMSNorm(gamma_cq) -> bf16 -> per-token int8 quant -> q_norm, q_norm_scale
//   stage 2: kv_a (columns 1536..2111) -> RMSNorm(gamma_ckv) of the first 512 -> four 128-dim int8 groups + fp32
//            scales scattered into the latent cache; last 64 -> de-interleave + RoPE -> rope cache
// (the dequantisation and rotary embedding of the q_b projection are the epilogue of that projection's kernel)
#include "kernels.cuh"

namespace dsv32 {

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// q_a / kv_a element: the projection's partial sums added in split order, rounded to bf16
__device__ __forceinline__ float partial_sum_bf16(const MlaStageParams& p, int tok, int col) {
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < kMlaXSplits; ++k) s += p.partial[(static_cast<size_t>(k) * p.t + tok) * kMlaXCols + col];
  return bf16r(s);
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) s += red[w];
  __syncthreads();
  return s;
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) s = fmaxf(s, red[w]);
  __syncthreads();
  return s;
}

// rotate-half RoPE on a de-interleaved 64-vector held in shared memory (fp32 values of bf16 numbers):
// x' = [x0, x2, .., x62, x1, x3, .., x63];  out[j] = x'[j]*cos[j] + rot(x')[j]*sin[j]
__device__ __forceinline__ float rope_deinterleaved(const float* x, int j, const __nv_bfloat16* cos,
                                                    const __nv_bfloat16* sin) {
  const float xj = (j < 32) ? x[2 * j] : x[2 * (j - 32) + 1];
  const float xr = (j < 32) ? -x[2 * j + 1] : x[2 * (j - 32)];  // rotate_half: (-x'[j+32], x'[j-32])
  return __fadd_rn(__fmul_rn(xj, __bfloat162float(cos[j])), __fmul_rn(xr, __bfloat162float(sin[j])));
}

// ---- stage 0: one CTA per token, 512 threads (three of the 1536 dims each) ------------------------------------------
__device__ __forceinline__ void mla_rmsnorm_quant(const MlaStageParams& p, int tok, float* red) {
  const int tid = threadIdx.x;
  float x[3], ss = 0.f;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    x[i] = partial_sum_bf16(p, tok, tid + i * 512);
    ss += __fmul_rn(__fmul_rn(x[i], x[i]), 1.0f / 1536.0f);
  }
  const float rms = sqrtf(block_sum<512>(ss, red) + p.eps_cq);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    x[i] = bf16r(__fmul_rn(__fdiv_rn(x[i], rms), __bfloat162float(p.gamma_cq[tid + i * 512])));
    amax = fmaxf(amax, fabsf(x[i]));
  }
  amax = block_max<512>(amax, red);
  const float sq = __fdiv_rn(127.0f, amax);
#pragma unroll
  for (int i = 0; i < 3; ++i)
    p.q_norm[static_cast<size_t>(tok) * 1536 + tid + i * 512] = static_cast<int8_t>(static_cast<int>(rintf(__fmul_rn(x[i], sq))));
  if (tid == 0) p.q_norm_scale[tok] = __fdiv_rn(1.0f, sq);
}

// ---- stage 2: one CTA per token, 512 threads -------------------------------------------------------------------
__global__ void __launch_bounds__(512) mla_finish_kernel(MlaStageParams p) {
  __shared__ float red[16];
  __shared__ float gmax[4];
  __shared__ float rope_s[64];
  const int tok = blockIdx.x, tid = threadIdx.x;
  if (blockIdx.y == 0) {   // both stages in one launch: blockIdx.y selects (uniform for the CTA)
    mla_rmsnorm_quant(p, tok, red);
    return;
  }
  const float x = partial_sum_bf16(p, tok, 1536 + tid);
  if (tid < 64) rope_s[tid] = partial_sum_bf16(p, tok, 1536 + 512 + tid);
  const float rms = sqrtf(block_sum<512>(__fmul_rn(__fmul_rn(x, x), 1.0f / 512.0f), red) + p.eps_ckv);
  const float y = bf16r(__fmul_rn(__fdiv_rn(x, rms), __bfloat162float(p.gamma_ckv[tid])));
  // per 128-dim group (4 warps) maximum
  float a = fabsf(y);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
  if ((tid & 31) == 0) red[tid >> 5] = a;
  __syncthreads();
  if (tid < 4) gmax[tid] = fmaxf(fmaxf(red[4 * tid], red[4 * tid + 1]), fmaxf(red[4 * tid + 2], red[4 * tid + 3]));
  __syncthreads();
  const long long crow = p.cache_index[tok];
  if (crow < 0 || crow >= p.cache_rows) {
    if (tid == 0) report_status(p.status, DSV32_STATUS_BAD_INDEX, tok, 1);
    return;
  }
  const float sq = __fdiv_rn(127.0f, gmax[tid >> 7]);
  p.kv_cache[crow * 512 + tid] = static_cast<int8_t>(static_cast<int>(rintf(__fmul_rn(y, sq))));
  if ((tid & 127) == 0) p.k_scale_cache[crow * 4 + (tid >> 7)] = __fdiv_rn(1.0f, sq);
  if (tid < 64)
    p.kr_cache[crow * 64 + tid] = __float2bfloat16_rn(
        rope_deinterleaved(rope_s, tid, p.cos + static_cast<size_t>(tok) * 64, p.sin + static_cast<size_t>(tok) * 64));
}

int launch_mla_finish(const MlaStageParams& p, cudaStream_t stream) {
  if (p.t <= 0) return DSV32_OK;
  mla_finish_kernel<<<dim3(p.t, 2), 512, 0, stream>>>(p);
  count_launch();
  return check_launch("mla_finish_kernel");
}

}  // namespace dsv32

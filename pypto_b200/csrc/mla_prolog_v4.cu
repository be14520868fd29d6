// Fused element-wise stages of the DeepSeek-V4 MLA prolog (quant)
// (models/deepseek_v4/mla_prolog_quant_v4_impl.py:406-517; golden mla_prolog_compute,
// models/deepseek_v4/test_mla_prolog_quant_v4.py:138-189).  The three plain projections between the stages
// (x.wq_a and x.wkv with fp32 results, int8 qr.wq_b) are library GEMMs issued by the host layer.
//   stage 0: q_a (fp32 [t, 1024]) -> RMSNorm * gamma_cq (fp32) -> per-token int8 quant -> qr, qr_scale
//   stage 1: q_b (int32 [t, heads*512]) -> * qr_scale * wq_b_scale -> per-head RMSNorm without weight -> bf16;
//            last 64 dims of a head: interleaved rotary embedding -> q [t, heads, 512]
//   stage 2: kv_a (fp32 [t, 512]) -> RMSNorm * gamma_ckv -> bf16; last 64 dims: interleaved rotary -> kv [t, 512]
// The operator without quantisation (models/deepseek_v4/mla_prolog_v4_impl.py:310-390; golden
// models/deepseek_v4/test_mla_prolog_v4.py:117-158) is the kQuant = false instantiation of the same kernels: its
// three GEMMs return bf16, stage 0 writes qr as bf16 without quantising and stage 1 has nothing to dequantise.
// Rotary form (apply_rotary_pos_emb_v2, test_mla_prolog_quant_v4.py:84-106): pairs (2i, 2i+1),
//   out[2i] = x[2i] cos[2i] - x[2i+1] sin[2i],  out[2i+1] = x[2i+1] cos[2i+1] + x[2i] sin[2i+1]   (fp32, then bf16).
#include "kernels.cuh"

namespace dsv32 {

namespace {

__device__ __forceinline__ float v4_bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <int THREADS>
__device__ __forceinline__ float v4_block_sum(float v, float* red) {
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
__device__ __forceinline__ float v4_block_max(float v, float* red) {
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

// interleaved rotary embedding of element j (0..63) of a 64-vector of bf16 values held as floats
__device__ __forceinline__ float v4_rope(const float* x, int j, const __nv_bfloat16* cos, const __nv_bfloat16* sin) {
  const float partner = (j & 1) ? x[j - 1] : -x[j + 1];
  return __fadd_rn(__fmul_rn(x[j], __bfloat162float(cos[j])), __fmul_rn(partner, __bfloat162float(sin[j])));
}

}  // namespace

// ---- stage 0: one CTA per token, 256 threads, 4 elements each ---------------------------------------------
template <bool kQuant>
__global__ void __launch_bounds__(256) mla_v4_rmsnorm_quant_kernel(MlaV4StageParams p) {
  __shared__ float red[8];
  const int tok = blockIdx.x, tid = threadIdx.x;
  float x[4], ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const size_t at = static_cast<size_t>(tok) * 1024 + tid + i * 256;
    x[i] = kQuant ? static_cast<const float*>(p.q_a)[at] : __bfloat162float(static_cast<const __nv_bfloat16*>(p.q_a)[at]);
    ss += __fmul_rn(__fmul_rn(x[i], x[i]), 1.0f / 1024.0f);
  }
  const float rms = sqrtf(v4_block_sum<256>(ss, red) + p.eps);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[i] = __fmul_rn(__fdiv_rn(x[i], rms), __bfloat162float(p.gamma_cq[tid + i * 256]));
    amax = fmaxf(amax, fabsf(x[i]));
  }
  if constexpr (!kQuant) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      static_cast<__nv_bfloat16*>(p.qr)[static_cast<size_t>(tok) * 1024 + tid + i * 256] = __float2bfloat16_rn(x[i]);
    return;
  }
  amax = v4_block_max<256>(amax, red);
  const float sq = __fdiv_rn(127.0f, amax);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    static_cast<int8_t*>(p.qr)[static_cast<size_t>(tok) * 1024 + tid + i * 256] =
        static_cast<int8_t>(static_cast<int>(rintf(__fmul_rn(x[i], sq))));
  if (tid == 0) p.qr_scale[tok] = __fdiv_rn(1.0f, sq);
}

// ---- stage 1: one CTA per (token, head), 256 threads, 2 elements each ---------------------------------------
template <bool kQuant>
__global__ void __launch_bounds__(256) mla_v4_q_finish_kernel(MlaV4StageParams p) {
  __shared__ float red[8];
  __shared__ float rope_s[64];
  const int tok = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
  const size_t col0 = static_cast<size_t>(head) * 512;
  const size_t row0 = static_cast<size_t>(tok) * p.q_b_ld + col0;
  float qs = 0.f;
  if constexpr (kQuant) qs = p.qr_scale[tok];
  float x[2], ss = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int d = tid + i * 256;
    if constexpr (kQuant)
      x[i] = __fmul_rn(__fmul_rn(__int2float_rn(static_cast<const int32_t*>(p.q_b)[row0 + d]), qs), p.wq_b_scale[col0 + d]);
    else
      x[i] = __bfloat162float(static_cast<const __nv_bfloat16*>(p.q_b)[row0 + d]);
    ss += __fmul_rn(__fmul_rn(x[i], x[i]), 1.0f / 512.0f);
  }
  const float rms = sqrtf(v4_block_sum<256>(ss, red) + p.eps);
  __nv_bfloat16* out = p.q_out + (static_cast<size_t>(tok) * p.heads + head) * 512;
  const float y0 = v4_bf16r(__fdiv_rn(x[0], rms));  // dims 0..255: never rope
  out[tid] = __float2bfloat16_rn(y0);
  const float y1 = v4_bf16r(__fdiv_rn(x[1], rms));  // dims 256..511: rope for dims >= 448
  const int d1 = tid + 256;
  if (d1 < 448) out[d1] = __float2bfloat16_rn(y1);
  else rope_s[d1 - 448] = y1;
  __syncthreads();
  if (d1 >= 448) {
    const int j = d1 - 448;
    out[d1] = __float2bfloat16_rn(v4_rope(rope_s, j, p.cos + static_cast<size_t>(tok) * 64, p.sin + static_cast<size_t>(tok) * 64));
  }
}

// ---- stage 2: one CTA per token, 512 threads ------------------------------------------------------------------
template <bool kQuant>
__global__ void __launch_bounds__(512) mla_v4_kv_finish_kernel(MlaV4StageParams p) {
  __shared__ float red[16];
  __shared__ float rope_s[64];
  const int tok = blockIdx.x, tid = threadIdx.x;
  const size_t at = static_cast<size_t>(tok) * 512 + tid;
  const float x = kQuant ? static_cast<const float*>(p.kv_a)[at] : __bfloat162float(static_cast<const __nv_bfloat16*>(p.kv_a)[at]);
  const float rms = sqrtf(v4_block_sum<512>(__fmul_rn(__fmul_rn(x, x), 1.0f / 512.0f), red) + p.eps);
  const float y = v4_bf16r(__fmul_rn(__fdiv_rn(x, rms), __bfloat162float(p.gamma_ckv[tid])));
  __nv_bfloat16* out = p.kv_out + static_cast<size_t>(tok) * 512;
  if (tid < 448) out[tid] = __float2bfloat16_rn(y);
  else rope_s[tid - 448] = y;
  __syncthreads();
  if (tid >= 448)
    out[tid] = __float2bfloat16_rn(
        v4_rope(rope_s, tid - 448, p.cos + static_cast<size_t>(tok) * 64, p.sin + static_cast<size_t>(tok) * 64));
}

int launch_mla_v4_stage(const MlaV4StageParams& p, int stage, cudaStream_t stream) {
  if (p.t <= 0) return DSV32_OK;
  if (stage == 0) {
    if (p.quant) mla_v4_rmsnorm_quant_kernel<true><<<p.t, 256, 0, stream>>>(p);
    else mla_v4_rmsnorm_quant_kernel<false><<<p.t, 256, 0, stream>>>(p);
  } else if (stage == 1) {
    if (p.quant) mla_v4_q_finish_kernel<true><<<dim3(p.t, p.heads), 256, 0, stream>>>(p);
    else mla_v4_q_finish_kernel<false><<<dim3(p.t, p.heads), 256, 0, stream>>>(p);
  } else {
    if (p.quant) mla_v4_kv_finish_kernel<true><<<p.t, 512, 0, stream>>>(p);
    else mla_v4_kv_finish_kernel<false><<<p.t, 512, 0, stream>>>(p);
  }
  count_launch();
  return check_launch("mla v4 prolog stage kernel");
}

}  // namespace dsv32

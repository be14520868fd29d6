// Indexer prolog (quant).  Follows models/deepseek_v32_exp/lightning_indexer_prolog_quant_impl.py:423-543
// (golden: deepseekv32_lightning_indexer_prolog_quant.py:220-288):
//   Q: int8 q_norm x int8 w_qb -> int32 -> *q_norm_scale -> *w_qb_scale -> bf16 -> RoPE(first 64 dims)
//      -> x hadamard_q (128x128) -> bf16 -> per-(token,head) int8 quant, fp16 scale
//   K: x x wk (fp32) -> LayerNorm -> bf16 -> RoPE -> x hadamard_k -> bf16 -> int8 quant -> cache scatter
//   W: bf16(x x w_proj) * 64^-0.5 * 128^-0.5 -> fp16
// The Q path and the split-K product x . [wk | w_proj] run on the tensor cores (prolog_tc.cu); the kernel here
// (one CTA per token) adds the fp32 partial sums of that product in a fixed order and finishes the K and W
// paths.
#include "kernels.cuh"

namespace dsv32 {


constexpr int kKwCols = 192;          // 128 (wk) + 64 (w_proj)

// rotate-half RoPE on dims [0,64) of a 128-vector held in shared memory as bf16-rounded floats.
// out = bf16( x*cos + rot(x)*sin ), each product and the sum rounded separately in fp32 as torch does.
__device__ __forceinline__ float rope_elem(const float* v, int d, const __nv_bfloat16* cos, const __nv_bfloat16* sin) {
  const float c = __bfloat162float(cos[d]), s = __bfloat162float(sin[d]);
  const float r = (d < 32) ? -v[d + 32] : v[d - 32];
  return __bfloat162float(__float2bfloat16_rn(__fadd_rn(__fmul_rn(v[d], c), __fmul_rn(r, s))));
}

// ---------------------------------------------------------------------------------------------------
// Finish of the K and W paths.  grid = t tokens; 192 threads (128 for K, 64 for W)
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kKwCols) prolog_kw_finish_kernel(PrologParams p, int nsplits) {
  __shared__ float v_s[128], r_s[128];
  __shared__ float red_s[4], red2_s[4];
  __shared__ __align__(16) __nv_bfloat16 had_s[128][128];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tok = blockIdx.x;
  // the hadamard matrix (32 KB) travels to shared memory asynchronously, under the reduction / LayerNorm / RoPE below
  for (int c = tid; c < 128 * 16; c += kKwCols) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(&had_s[c / 16][(c % 16) * 8]));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(p.had_k + c * 8) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  float sum = 0.f;
  for (int kc = 0; kc < nsplits; ++kc) sum += p.partial[(static_cast<size_t>(kc) * p.t + tok) * kKwCols + tid];

  if (tid >= 128) {  // W path (no barriers below are skipped: the K path barriers are executed by all threads)
    const float w = __bfloat162float(__float2bfloat16_rn(sum));
    p.weights[static_cast<size_t>(tok) * 64 + (tid - 128)] =
        __float2half_rn(__fmul_rn(__fmul_rn(w, 0.125f), 0.08838834764831845f));
  }
  // LayerNorm over the 128 K values (threads 0..127 = warps 0..3)
  float s1 = (tid < 128) ? sum : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s1 += __shfl_xor_sync(0xffffffffu, s1, o);
  if (tid < 128 && lane == 0) red_s[warp] = s1;
  __syncthreads();
  const float mean = (red_s[0] + red_s[1] + red_s[2] + red_s[3]) * (1.0f / 128.0f);
  const float dlt = sum - mean;
  float s2 = (tid < 128) ? dlt * dlt : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  if (tid < 128 && lane == 0) red2_s[warp] = s2;
  __syncthreads();
  const float var = (red2_s[0] + red2_s[1] + red2_s[2] + red2_s[3]) * (1.0f / 128.0f);
  if (tid < 128) {
    float y = __fdiv_rn(dlt, sqrtf(var + p.eps));
    y = __fadd_rn(__fmul_rn(y, __bfloat162float(p.ln_gamma[tid])), __bfloat162float(p.ln_beta[tid]));
    v_s[tid] = __bfloat162float(__float2bfloat16_rn(y));
  }
  __syncthreads();
  if (tid < 128)
    r_s[tid] = (tid < 64) ? rope_elem(v_s, tid, p.cos + static_cast<size_t>(tok) * 64, p.sin + static_cast<size_t>(tok) * 64)
                          : v_s[tid];
  asm volatile("cp.async.wait_group 0;" ::: "memory");   // this thread's pieces of the hadamard matrix have landed
  __syncthreads();
  float hv = 0.f;
  if (tid < 128) {
#pragma unroll 8
    for (int k = 0; k < 128; ++k) hv = fmaf(r_s[k], __bfloat162float(had_s[k][tid]), hv);
    hv = __bfloat162float(__float2bfloat16_rn(hv));
  }
  float mine = (tid < 128) ? fabsf(hv) : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mine = fmaxf(mine, __shfl_xor_sync(0xffffffffu, mine, o));
  __syncthreads();
  if (tid < 128 && lane == 0) red_s[warp] = mine;
  __syncthreads();
  const float a = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
  if (tid < 128) {
    const long long row = p.cache_index[tok];
    if (row < 0 || row >= p.cache_rows) {
      if (tid == 0) report_status(p.status, DSV32_STATUS_BAD_INDEX, tok, 0);
    } else {
      const float sq = __fdiv_rn(127.0f, a);
      const float qf = rintf(__fmul_rn(hv, sq));
      p.k_cache[row * 128 + tid] = static_cast<int8_t>(static_cast<int>(qf));
      if (tid == 0) p.k_scale_cache[row] = __float2half_rn(__fdiv_rn(1.0f, sq));
    }
  }
}

int launch_prolog_finish(const PrologParams& p, int splits, cudaStream_t stream) {
  prolog_kw_finish_kernel<<<p.t, kKwCols, 0, stream>>>(p, splits);
  count_launch();
  return check_launch("prolog_kw_finish_kernel");
}

size_t prolog_workspace_bytes(int t) { return static_cast<size_t>(kPrologKSplits) * t * kKwCols * sizeof(float); }

}  // namespace dsv32

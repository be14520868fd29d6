// Indexer prolog (quant).  Follows models/deepseek_v32_exp/lightning_indexer_prolog_quant_impl.py:423-543
// (golden: deepseekv32_lightning_indexer_prolog_quant.py:220-288):
//   Q: int8 q_norm x int8 w_qb -> int32 -> *q_norm_scale -> *w_qb_scale -> bf16 -> RoPE(first 64 dims)
//      -> x hadamard_q (128x128) -> bf16 -> per-(token,head) int8 quant, fp16 scale
//   K: x x wk (fp32) -> LayerNorm -> bf16 -> RoPE -> x hadamard_k -> bf16 -> int8 quant -> cache scatter
//   W: bf16(x x w_proj) * 64^-0.5 * 128^-0.5 -> fp16
// Kernel 1 (one CTA per index head and 16-token chunk) streams w_qb once and finishes the whole Q path in
// shared memory.  Kernel 2 streams wk|w_proj with a split over the 7168-long reduction and leaves fp32
// partial sums in the workspace; kernel 3 (one CTA per token) reduces them in a fixed order and finishes
// the K and W paths.
#include "kernels.cuh"

namespace dsv32 {


constexpr int kH = 7168, kQr = 1536, kTokChunk = 16;
constexpr int kKSplits = 56;          // 7168 / 128
constexpr int kKwCols = 192;          // 128 (wk) + 64 (w_proj)

// rotate-half RoPE on dims [0,64) of a 128-vector held in shared memory as bf16-rounded floats.
// out = bf16( x*cos + rot(x)*sin ), each product and the sum rounded separately in fp32 as torch does.
__device__ __forceinline__ float rope_elem(const float* v, int d, const __nv_bfloat16* cos, const __nv_bfloat16* sin) {
  const float c = __bfloat162float(cos[d]), s = __bfloat162float(sin[d]);
  const float r = (d < 32) ? -v[d + 32] : v[d - 32];
  return __bfloat162float(__float2bfloat16_rn(__fadd_rn(__fmul_rn(v[d], c), __fmul_rn(r, s))));
}

// ---------------------------------------------------------------------------------------------------
// Kernel 1: Q path.  grid = (64 heads, ceil(t/16)); 256 threads = 8 warps, warp w owns k in [192w, 192w+192)
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prolog_q_kernel(PrologParams p) {
  __shared__ __align__(16) int8_t qn_s[kTokChunk][kQr];   // 24 KB
  __shared__ int acc_s[kTokChunk][128];                   // 8 KB
  __shared__ float v_s[128], r_s[128];
  __shared__ float red_s[4];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int head = blockIdx.x;
  const int t0 = blockIdx.y * kTokChunk;
  const int nt = min(kTokChunk, p.t - t0);

  for (int c = tid; c < kTokChunk * (kQr / 16); c += 256) {
    const int r = c / (kQr / 16), ch = c % (kQr / 16);
    int4 v = make_int4(0, 0, 0, 0);
    if (r < nt) v = *reinterpret_cast<const int4*>(p.q_norm + static_cast<size_t>(t0 + r) * kQr + ch * 16);
    *reinterpret_cast<int4*>(&qn_s[r][ch * 16]) = v;
  }
  for (int c = tid; c < kTokChunk * 128; c += 256) acc_s[c / 128][c % 128] = 0;
  __syncthreads();

  // int8 GEMM: lane owns 4 consecutive output columns of this head
  int acc[kTokChunk][4];
#pragma unroll
  for (int i = 0; i < kTokChunk; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0;
  const int8_t* wbase = p.w_qb + head * 128 + lane * 4;
  const int kbeg = warp * (kQr / 8);
#pragma unroll 2
  for (int k = kbeg; k < kbeg + kQr / 8; k += 4) {
    uint32_t w0 = *reinterpret_cast<const uint32_t*>(wbase + static_cast<size_t>(k) * 8192);
    uint32_t w1 = *reinterpret_cast<const uint32_t*>(wbase + static_cast<size_t>(k + 1) * 8192);
    uint32_t w2 = *reinterpret_cast<const uint32_t*>(wbase + static_cast<size_t>(k + 2) * 8192);
    uint32_t w3 = *reinterpret_cast<const uint32_t*>(wbase + static_cast<size_t>(k + 3) * 8192);
    // 4x4 byte transpose: c_j = (w0.b_j, w1.b_j, w2.b_j, w3.b_j)
    const uint32_t t01l = __byte_perm(w0, w1, 0x5140), t01h = __byte_perm(w0, w1, 0x7362);
    const uint32_t t23l = __byte_perm(w2, w3, 0x5140), t23h = __byte_perm(w2, w3, 0x7362);
    const uint32_t c0 = __byte_perm(t01l, t23l, 0x5410), c1 = __byte_perm(t01l, t23l, 0x7632);
    const uint32_t c2 = __byte_perm(t01h, t23h, 0x5410), c3 = __byte_perm(t01h, t23h, 0x7632);
#pragma unroll
    for (int i = 0; i < kTokChunk; ++i) {
      const int qv = *reinterpret_cast<const int*>(&qn_s[i][k]);
      acc[i][0] = __dp4a(qv, static_cast<int>(c0), acc[i][0]);
      acc[i][1] = __dp4a(qv, static_cast<int>(c1), acc[i][1]);
      acc[i][2] = __dp4a(qv, static_cast<int>(c2), acc[i][2]);
      acc[i][3] = __dp4a(qv, static_cast<int>(c3), acc[i][3]);
    }
  }
#pragma unroll
  for (int i = 0; i < kTokChunk; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) atomicAdd(&acc_s[i][lane * 4 + j], acc[i][j]);
  }
  __syncthreads();

  // per token: dequant -> bf16 -> RoPE -> Hadamard -> bf16 -> quant.  Threads 0..127 own one dim each.
  for (int i = 0; i < nt; ++i) {
    const int tok = t0 + i;
    if (tid < 128) {
      float f = static_cast<float>(acc_s[i][tid]);
      f = __fmul_rn(f, p.q_norm_scale[tok]);
      f = __fmul_rn(f, p.w_qb_scale[head * 128 + tid]);
      v_s[tid] = __bfloat162float(__float2bfloat16_rn(f));
    }
    __syncthreads();
    if (tid < 128)
      r_s[tid] = (tid < 64) ? rope_elem(v_s, tid, p.cos + static_cast<size_t>(tok) * 64, p.sin + static_cast<size_t>(tok) * 64)
                            : v_s[tid];
    __syncthreads();
    float hv = 0.f;
    if (tid < 128) {
#pragma unroll 8
      for (int k = 0; k < 128; ++k) hv = fmaf(r_s[k], __bfloat162float(p.had_q[k * 128 + tid]), hv);
      hv = __bfloat162float(__float2bfloat16_rn(hv));
    }
    // all 256 threads take part in the barriers inside block128_amax; upper half contributes 0
    float a;
    {
      float mine = (tid < 128) ? fabsf(hv) : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mine = fmaxf(mine, __shfl_xor_sync(0xffffffffu, mine, o));
      if (tid < 128 && lane == 0) red_s[warp] = mine;
      __syncthreads();
      a = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
      __syncthreads();
    }
    if (tid < 128) {
      const float sq = __fdiv_rn(127.0f, a);
      const float qf = rintf(__fmul_rn(hv, sq));
      p.q_int8[(static_cast<size_t>(tok) * 64 + head) * 128 + tid] = static_cast<int8_t>(static_cast<int>(qf));
      if (tid == 0) p.q_scale[static_cast<size_t>(tok) * 64 + head] = __float2half_rn(__fdiv_rn(1.0f, sq));
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Kernel 2: partial sums of x x [wk | w_proj].  grid = (56 k-chunks of 128, ceil(t/16)); 192 threads
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kKwCols) prolog_kw_partial_kernel(PrologParams p) {
  __shared__ float x_s[kTokChunk][128];
  const int tid = threadIdx.x;
  const int kc = blockIdx.x;
  const int t0 = blockIdx.y * kTokChunk;
  const int nt = min(kTokChunk, p.t - t0);
  for (int c = tid; c < kTokChunk * 128; c += kKwCols) {
    const int r = c / 128, k = c % 128;
    x_s[r][k] = (r < nt) ? __bfloat162float(p.x[static_cast<size_t>(t0 + r) * kH + kc * 128 + k]) : 0.f;
  }
  __syncthreads();
  float acc[kTokChunk];
#pragma unroll
  for (int i = 0; i < kTokChunk; ++i) acc[i] = 0.f;
  const bool is_k = tid < 128;
  const __nv_bfloat16* w = is_k ? p.wk + static_cast<size_t>(kc) * 128 * 128 + tid
                                : p.w_proj + static_cast<size_t>(kc) * 128 * 64 + (tid - 128);
  const int ldw = is_k ? 128 : 64;
#pragma unroll 4
  for (int k = 0; k < 128; ++k) {
    const float wv = __bfloat162float(w[static_cast<size_t>(k) * ldw]);
#pragma unroll
    for (int i = 0; i < kTokChunk; ++i) acc[i] = fmaf(x_s[i][k], wv, acc[i]);
  }
  for (int i = 0; i < nt; ++i)
    p.partial[(static_cast<size_t>(kc) * p.t + t0 + i) * kKwCols + tid] = acc[i];
}

// ---------------------------------------------------------------------------------------------------
// Kernel 3: finish K and W paths.  grid = t tokens; 192 threads (128 for K, 64 for W)
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

int launch_prolog(const PrologParams& p, cudaStream_t stream) {
  if (p.t <= 0) return DSV32_OK;
  const int chunks = (p.t + kTokChunk - 1) / kTokChunk;
  prolog_q_kernel<<<dim3(64, chunks), 256, 0, stream>>>(p);
  count_launch();
  int rc = check_launch("prolog_q_kernel");
  if (rc != DSV32_OK) return rc;
  prolog_kw_partial_kernel<<<dim3(kKSplits, chunks), kKwCols, 0, stream>>>(p);
  count_launch();
  rc = check_launch("prolog_kw_partial_kernel");
  if (rc != DSV32_OK) return rc;
  return launch_prolog_finish(p, kKSplits, stream);
}

size_t prolog_workspace_bytes(int t) { return static_cast<size_t>(kKSplits) * t * kKwCols * sizeof(float); }

}  // namespace dsv32

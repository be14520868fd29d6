// Page-grouped lightning-indexer prolog with 8-bit float formats (MXFP8 E4M3 with E8M0 block scales, and HiF8).
// Follows python/tests/st/operator/pg/lightning_indexer_prolog_quant_mxfp8_impl.py:230-401 and
// lightning_indexer_prolog_quant_hif8_impl.py:230-406 (golden: test_pg_lightning_indexer_prolog_quant_mxfp8.py:272-345).
//
//   pg_unpack_kernel   the 8-bit operands of q_norm . w_qb widened to bf16 -- exactly: an E4M3 or HiF8 value has at
//                      most four significant bits and an E8M0 scale is a power of two -- and [wk | w_proj] packed
//                      into one [h, 256] matrix, so that both products run on the bf16 tcgen05 GEMM
//                      (launch_bf16_gemm_partial, fp32 accumulation: the sum the golden forms in fp32)
//   pg_q_finish_kernel one (token, head) per CTA: partial sums added in a fixed order, (HiF8: x token scale x column
//                      scale,) bf16; rotate-half rotary embedding of dims 0..63; x hadamard_q; per-row dynamic
//                      quantisation to the 8-bit format with an fp32 scale
//   pg_k_finish_kernel one token per CTA: bf16, RMSNorm, rotary embedding, x hadamard_k, quantisation, scatter of the
//                      code row and of its scale into the page-grouped caches; and the head weights
// Every bf16 rounding sits where the operator puts it; products and sums of the rotary embedding are rounded
// separately (no fused multiply-add), as the operator's separate vector instructions do.
#include <cuda_fp8.h>

#include "kernels.cuh"

namespace dsv32 {

constexpr int kPgDim = 128, kPgRope = 64, kPgXwCols = 256;

__device__ __forceinline__ float pg_bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// ---- HiF8 (bit layout: framework/src/interface/machine/device/tilefwk/aicore_print_base.h:361-484) -----------------
// sign | prefix-coded exponent width | sign-magnitude exponent with an implied leading one | mantissa:
//   0000mmm 2^(m-23) (m = 0: zero, or NaN with the sign bit)   0001mmm e = 0   001emmm e = +-1   01semmm e = +-(2+e)
//   10seemm e = +-(4+ee)   11seeem e = +-(8+eee), e = +15 with mantissa 1 is infinity
__device__ __forceinline__ float pg_pow2(int e) { return __int_as_float((e + 127) << 23); }  // -126 <= e <= 127

__device__ __forceinline__ float hif8_to_float(uint32_t code) {
  const uint32_t low = code & 0x7Fu;
  const float sign = (code & 0x80u) ? -1.f : 1.f;
  if ((low >> 3) == 0u) {
    const int m = static_cast<int>(low & 7u);
    if (m == 0) return (code & 0x80u) ? __int_as_float(0x7fc00000) : 0.f;
    return sign * pg_pow2(m - 23);
  }
  int ev, mant, bits;
  if ((low >> 3) == 1u) {
    ev = 0; mant = low & 7; bits = 3;
  } else if ((low >> 4) == 1u) {
    ev = ((low >> 3) & 1u) ? -1 : 1; mant = low & 7; bits = 3;
  } else if ((low >> 5) == 1u) {
    const int eb = (low >> 3) & 3;
    ev = (2 + (eb & 1)) * ((eb >> 1) ? -1 : 1); mant = low & 7; bits = 3;
  } else if ((low >> 5) == 2u) {
    const int eb = (low >> 2) & 7;
    ev = (4 + (eb & 3)) * ((eb >> 2) ? -1 : 1); mant = low & 3; bits = 2;
  } else {
    const int eb = (low >> 1) & 15;
    ev = (8 + (eb & 7)) * ((eb >> 3) ? -1 : 1); mant = low & 1; bits = 1;
    if (ev == 15 && mant == 1) return sign * __int_as_float(0x7f800000);
  }
  return sign * pg_pow2(ev) * (1.f + static_cast<float>(mant) * pg_pow2(-bits));
}
__device__ __forceinline__ int hif8_mantissa_bits(int e) {
  const int ae = e < 0 ? -e : e;
  return ae <= 3 ? 3 : (ae <= 7 ? 2 : 1);
}
// Nearest representable value, a tie to the larger magnitude, magnitudes above 2^15 to 2^15; NaN to the NaN code.
__device__ __forceinline__ uint32_t float_to_hif8(float x) {
  if (x != x) return 0x80u;
  const uint32_t sign = (__float_as_uint(x) >> 24) & 0x80u;
  const float mag = fminf(fabsf(x), 32768.f);
  if (mag < pg_pow2(-23)) return 0u;                             // nearer to zero, which has no sign
  int e = static_cast<int>((__float_as_uint(mag) >> 23) & 0xffu) - 127;   // floor(log2(mag)); mag is a normal fp32
  uint32_t mant = 0u;
  if (e < -15) {
    // only powers of two down here: 2^-22 .. 2^-16, then 2^-15 above and zero below; the midpoint goes up
    if (e == -23 || mag >= 1.5f * pg_pow2(e)) ++e;
    if (e <= -16) return sign | static_cast<uint32_t>(e + 23);
  } else {
    const int bits = hif8_mantissa_bits(e);
    const float q = mag * pg_pow2(bits - e);                     // in [2^bits, 2^(bits+1)), exact
    int qi = static_cast<int>(q);                                // floor
    if (q - static_cast<float>(qi) >= 0.5f) ++qi;                // half away from zero (q - floor(q) is exact)
    if (qi == (2 << bits)) ++e;                                  // carried into the next exponent, mantissa 0
    else mant = (static_cast<uint32_t>(qi) & ((1u << bits) - 1u));
  }
  const int ae = e < 0 ? -e : e;
  const uint32_t es = e < 0 ? 1u : 0u;
  if (ae == 0) return sign | 0x08u | mant;
  if (ae == 1) return sign | 0x10u | (es << 3) | mant;
  if (ae <= 3) return sign | 0x20u | (es << 4) | (static_cast<uint32_t>(ae - 2) << 3) | mant;
  if (ae <= 7) return sign | 0x40u | (es << 4) | (static_cast<uint32_t>(ae - 4) << 2) | mant;
  return sign | 0x60u | (es << 4) | (static_cast<uint32_t>(ae - 8) << 1) | mant;
}

__device__ __forceinline__ float e4m3_to_float(uint32_t code) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(code), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
__device__ __forceinline__ float e8m0_to_float(uint32_t code) {  // 2^(code - 127); code 255 is NaN
  if (code == 255u) return __int_as_float(0x7fc00000);
  return code == 0u ? __int_as_float(0x00400000) : __int_as_float(static_cast<int>(code << 23));
}

// ---- operands to bf16 ----------------------------------------------------------------------------------------------
// grid-stride over three regions, eight elements per thread
__global__ void __launch_bounds__(256) pg_unpack_kernel(PgPrologParams p, __nv_bfloat16* q_bf, __nv_bfloat16* w_bf,
                                                        __nv_bfloat16* xw_bf) {
  const long long nq = static_cast<long long>(p.t) * p.q_lora / 8;
  const long long nw = static_cast<long long>(p.q_lora) * p.n / 8;
  const long long nx = static_cast<long long>(p.h) * kPgXwCols / 8;
  const bool mx = p.format == DSV32_PG_FORMAT_MXFP8;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < nq + nw + nx; i += static_cast<long long>(gridDim.x) * 256) {
    uint32_t w[4];
    if (i < nq + nw) {
      const bool is_q = i < nq;
      const long long e0 = (is_q ? i : i - nq) * 8;                // first of eight consecutive elements of a row
      const uint8_t* src = (is_q ? p.q_norm : p.w_qb) + e0;
      const uint2 raw = *reinterpret_cast<const uint2*>(src);
      float scale[8];
      if (!mx) {
#pragma unroll
        for (int j = 0; j < 8; ++j) scale[j] = 1.f;
      } else if (is_q) {                                           // one scale per 32 reduction elements of the row
        const long long row = e0 / p.q_lora, k = e0 % p.q_lora;
        const float s = e8m0_to_float(p.q_norm_scale_e8[row * (p.q_lora / 32) + k / 32]);
#pragma unroll
        for (int j = 0; j < 8; ++j) scale[j] = s;
      } else {                                                     // block kb of column c: [kb / 2][c][kb % 2]
        const long long k = e0 / p.n, c0 = e0 % p.n;
        const long long kb = k / 32;
#pragma unroll
        for (int j = 0; j < 8; ++j) scale[j] = e8m0_to_float(p.w_qb_scale_e8[((kb >> 1) * p.n + c0 + j) * 2 + (kb & 1)]);
      }
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t code = ((j < 4 ? raw.x : raw.y) >> (8 * (j & 3))) & 0xffu;
        v[j] = (mx ? e4m3_to_float(code) : hif8_to_float(code)) * scale[j];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
      *reinterpret_cast<uint4*>((is_q ? q_bf : w_bf) + e0) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      const long long e0 = (i - nq - nw) * 8;
      const long long k = e0 / kPgXwCols;
      const int c0 = static_cast<int>(e0 % kPgXwCols);
      __nv_bfloat16 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = c0 + j;
        v[j] = c < kPgDim ? p.wk[k * kPgDim + c]
                          : (c < kPgDim + p.heads ? p.w_proj[k * p.heads + (c - kPgDim)] : __float2bfloat16_rn(0.f));
      }
      *reinterpret_cast<uint4*>(xw_bf + e0) = *reinterpret_cast<const uint4*>(v);
    }
  }
}

// ---- shared tail of both finish kernels: rotary embedding, Hadamard product, quantisation ---------------------------
// `v` is this thread's element (dim = threadIdx.x) of a 128-dim row as a bf16-valued float; returns the 8-bit code and
// leaves the row's scale in *scale_out (the same value in every thread).
__device__ __forceinline__ uint32_t pg_rope_hadamard_quant(float v, const __nv_bfloat16* cos_row, const __nv_bfloat16* sin_row,
                                                           const __nv_bfloat16* hadamard, int format, float* row_s,
                                                           float* red_s, float* scale_out) {
  const int j = threadIdx.x;
  row_s[j] = v;
  __syncthreads();
  if (j < kPgRope) {   // [-x2, x1] rotation inside the first 64 dims
    const float c = __bfloat162float(cos_row[j]), s = __bfloat162float(sin_row[j]);
    const float other = j < 32 ? -row_s[j + 32] : row_s[j - 32];
    v = pg_bf16r(__fadd_rn(__fmul_rn(v, c), __fmul_rn(other, s)));
  }
  __syncthreads();
  row_s[j] = v;
  __syncthreads();
  float acc = 0.f;
#pragma unroll 8
  for (int i = 0; i < kPgDim; ++i) acc = fmaf(row_s[i], __bfloat162float(hadamard[i * kPgDim + j]), acc);
  const float hv = pg_bf16r(acc);
  // row maximum of |hv|
  float m = fabsf(hv);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((j & 31) == 0) red_s[j >> 5] = m;
  __syncthreads();
  m = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
  const bool mx = format == DSV32_PG_FORMAT_MXFP8;
  const float scale = __fmul_rn(m, mx ? (1.0f / 448.0f) : (1.0f / 32768.0f));
  *scale_out = scale;
  const float y = __fdiv_rn(hv, scale);
  if (mx) return static_cast<uint32_t>(__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3));
  return float_to_hif8(y);
}

__global__ void __launch_bounds__(kPgDim) pg_q_finish_kernel(PgPrologParams p, const float* partial, int splits) {
  __shared__ float row_s[kPgDim];
  __shared__ float red_s[4];
  const int head = blockIdx.x % p.heads, tok = blockIdx.x / p.heads, j = threadIdx.x;   // t * heads CTAs in x: no 65,535 limit
  const int col = head * kPgDim + j;
  float acc = 0.f;
  for (int s = 0; s < splits; ++s) acc += partial[(static_cast<size_t>(s) * p.t + tok) * p.n + col];
  if (p.format == DSV32_PG_FORMAT_HIF8) acc = __fmul_rn(__fmul_rn(acc, p.q_norm_scale_f32[tok]), p.w_qb_scale_f32[col]);
  float scale;
  const uint32_t code = pg_rope_hadamard_quant(pg_bf16r(acc), p.cos + static_cast<size_t>(tok) * kPgRope,
                                               p.sin + static_cast<size_t>(tok) * kPgRope, p.hadamard_q, p.format, row_s,
                                               red_s, &scale);
  p.q_out[(static_cast<size_t>(tok) * p.heads + head) * kPgDim + j] = static_cast<uint8_t>(code);
  if (j == 0) p.q_scale_out[static_cast<size_t>(tok) * p.heads + head] = scale;
}

__global__ void __launch_bounds__(kPgDim) pg_k_finish_kernel(PgPrologParams p, const float* partial, int splits) {
  __shared__ float row_s[kPgDim];
  __shared__ float red_s[4];
  __shared__ float ms_s[4];
  const int tok = blockIdx.x, j = threadIdx.x;
  float acc = 0.f, wacc = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* prow = partial + (static_cast<size_t>(s) * p.t + tok) * kPgXwCols;
    acc += prow[j];
    if (j < p.heads) wacc += prow[kPgDim + j];
  }
  // head weights: bf16, x heads^-0.5 -> bf16, x 128^-0.5 -> bf16
  if (j < p.heads) {
    float w = pg_bf16r(wacc);
    w = pg_bf16r(__fmul_rn(w, p.heads_rsqrt));
    p.weights_out[static_cast<size_t>(tok) * p.heads + j] = __float2bfloat16_rn(__fmul_rn(w, 0.08838834764831845f));
  }
  // RMSNorm: x / sqrt(sum(x^2 / 128) + eps) * gamma
  const float k = pg_bf16r(acc);
  float sq = __fmul_rn(__fmul_rn(k, k), 1.0f / 128.0f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if ((j & 31) == 0) ms_s[j >> 5] = sq;
  __syncthreads();
  const float ms = (ms_s[0] + ms_s[1]) + (ms_s[2] + ms_s[3]);
  const float kn = pg_bf16r(__fmul_rn(__fdiv_rn(k, __fsqrt_rn(ms + p.eps)), __bfloat162float(p.gamma_k[j])));
  float scale;
  const uint32_t code = pg_rope_hadamard_quant(kn, p.cos + static_cast<size_t>(tok) * kPgRope,
                                               p.sin + static_cast<size_t>(tok) * kPgRope, p.hadamard_k, p.format, row_s,
                                               red_s, &scale);
  // scatter into the page-grouped caches: row r lives in page r / block_size at slot r % block_size
  const long long r = p.k_cache_index[tok], rs = p.k_scale_cache_index[tok];
  if (r < 0 || r >= p.cache_rows || rs < 0 || rs >= p.cache_rows) {
    if (j == 0) report_status(p.status, DSV32_STATUS_BAD_INDEX, tok, static_cast<uint32_t>(r < 0 || r >= p.cache_rows ? r : rs));
    return;
  }
  p.k_cache[(r / p.block_size) * p.k_block_stride + (r % p.block_size) * kPgDim + j] = static_cast<uint8_t>(code);
  if (j == 0)
    *reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(p.k_scale_cache) + (rs / p.block_size) * p.k_scale_block_stride +
                              (rs % p.block_size) * sizeof(float)) = scale;
}

__global__ void __launch_bounds__(256) hif8_convert_kernel(int direction, const void* in, void* out, long long n) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * 256) {
    if (direction == 0) static_cast<uint8_t*>(out)[i] = static_cast<uint8_t>(float_to_hif8(static_cast<const float*>(in)[i]));
    else static_cast<float*>(out)[i] = hif8_to_float(static_cast<const uint8_t*>(in)[i]);
  }
}

int launch_hif8_convert(int direction, const void* in, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return DSV32_OK;
  const long long blocks = (n + 255) / 256;
  hif8_convert_kernel<<<static_cast<int>(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, stream>>>(direction, in, out, n);
  count_launch();
  return check_launch("hif8_convert_kernel");
}

static int pg_q_splits(int t) { return t <= 256 ? 4 : (t <= 512 ? 2 : 1); }
static int pg_x_splits(int t) { return t <= 1024 ? 8 : 2; }
static size_t pg_align(size_t b) { return (b + 255) / 256 * 256; }

size_t pg_prolog_workspace_bytes(int t, int h, int q_lora, int heads) {
  if (t <= 0 || h <= 0 || q_lora <= 0 || heads <= 0) return 0;
  const size_t n = static_cast<size_t>(heads) * kPgDim;
  return pg_align(static_cast<size_t>(t) * q_lora * 2) + pg_align(static_cast<size_t>(q_lora) * n * 2) +
         pg_align(static_cast<size_t>(h) * kPgXwCols * 2) + pg_align(static_cast<size_t>(pg_q_splits(t)) * t * n * 4) +
         pg_align(static_cast<size_t>(pg_x_splits(t)) * t * kPgXwCols * 4);
}

int launch_pg_prolog(const PgPrologParams& p, void* workspace, cudaStream_t stream) {
  if (p.t <= 0) return DSV32_OK;
  char* ws = static_cast<char*>(workspace);
  __nv_bfloat16* q_bf = reinterpret_cast<__nv_bfloat16*>(ws);
  ws += pg_align(static_cast<size_t>(p.t) * p.q_lora * 2);
  __nv_bfloat16* w_bf = reinterpret_cast<__nv_bfloat16*>(ws);
  ws += pg_align(static_cast<size_t>(p.q_lora) * p.n * 2);
  __nv_bfloat16* xw_bf = reinterpret_cast<__nv_bfloat16*>(ws);
  ws += pg_align(static_cast<size_t>(p.h) * kPgXwCols * 2);
  float* part_q = reinterpret_cast<float*>(ws);
  const int qs = pg_q_splits(p.t), xs = pg_x_splits(p.t);
  ws += pg_align(static_cast<size_t>(qs) * p.t * p.n * 4);
  float* part_x = reinterpret_cast<float*>(ws);

  const long long items = (static_cast<long long>(p.t) * p.q_lora + static_cast<long long>(p.q_lora) * p.n +
                           static_cast<long long>(p.h) * kPgXwCols) / 8;
  const int blocks = static_cast<int>(items / 256 + 1 < 148 * 8 ? items / 256 + 1 : 148 * 8);
  pg_unpack_kernel<<<blocks, 256, 0, stream>>>(p, q_bf, w_bf, xw_bf);
  count_launch();
  int rc = check_launch("pg_unpack_kernel");
  if (rc != DSV32_OK) return rc;
  rc = launch_bf16_gemm_partial(q_bf, p.t, p.q_lora, w_bf, p.n, p.n / 128, qs, part_q, p.n, p.status, stream);
  if (rc != DSV32_OK) return rc;
  rc = launch_bf16_gemm_partial(p.x, p.t, p.h, xw_bf, kPgXwCols, kPgXwCols / 128, xs, part_x, kPgXwCols, p.status, stream);
  if (rc != DSV32_OK) return rc;
  pg_q_finish_kernel<<<p.heads * p.t, kPgDim, 0, stream>>>(p, part_q, qs);
  count_launch();
  rc = check_launch("pg_q_finish_kernel");
  if (rc != DSV32_OK) return rc;
  pg_k_finish_kernel<<<p.t, kPgDim, 0, stream>>>(p, part_x, xs);
  count_launch();
  return check_launch("pg_k_finish_kernel");
}

}  // namespace dsv32

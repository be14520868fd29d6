// DeepSeek-V4 hyper-connection pre-mix ("hc_pre").
// Follows models/deepseek_v4/hc_pre_impl.py:23-206 (golden gen_hc_pre, models/deepseek_v4/test_hc_pre.py:26-118).
// Per token, with x [4 streams, 4096] bf16 read as one 16384-vector:
//   mix[24]  = (x . hc_fn[m, :]) / sqrt(mean(x^2) + norm_eps)                       (fp32)
//   pre[4]   = sigmoid(mix[0:4]  * scale[0] + base[0:4])  + hc_eps
//   post[4]  = 2 * sigmoid(mix[4:8] * scale[1] + base[4:8])
//   comb[4,4]= Sinkhorn(mix[8:24] * scale[2] + base[8:24]): row softmax + hc_eps, column normalisation, then
//              (iters - 1) x (row normalisation, column normalisation), every divisor with + hc_eps
//   y[4096]  = bf16( sum_h pre[h] * x[h, :] )
// Two kernels.  hc_pre_dots_kernel splits the 16384-long reduction into 128 slices of 128 columns: a CTA holds
// the 24 x 128 slice of hc_fn in shared memory and applies it to a tile of up to 128 tokens, so hc_fn (1.5 MB) is
// read once per token tile instead of once per token; a lane owns 6 outputs x 2 tokens, so every lane works and
// there are no shuffles in the loop.  Partial sums go to a workspace [group][token][24]; with
// many tokens a CTA walks several slices and adds them up in registers first.
// hc_pre_finish_kernel (one CTA per token) reads the token's x with 16-byte loads, takes its sum of squares, adds
// the partials in a fixed order, runs the 4x4 Sinkhorn on 16 lanes of a warp (row / column sums by shuffles)
// and writes y from the x values it holds.  DRAM traffic: x twice at most
// (the second read hits L2 for decode-sized batches), y once.
#include "kernels.cuh"

namespace dsv32 {

namespace {
constexpr int kHc = 4, kHcD = 4096, kHcK = kHc * kHcD, kHcMix = (2 + kHc) * kHc, kHcOut = kHcMix + 1;
constexpr int kHcSlice = 128, kHcSlices = kHcK / kHcSlice;   // 128 slices of 128 columns
constexpr int kHcTokTile = 128, kHcDotThreads = 256, kHcFinThreads = 512;
constexpr int kHcPad = kHcSlice + 4;                          // padded row stride of the shared-memory tiles
constexpr size_t kHcDotSmem = static_cast<size_t>(kHcMix + kHcTokTile) * kHcPad * sizeof(float);   // 80,256 bytes

__device__ __forceinline__ float hc_sigmoid(float v) { return __fdiv_rn(1.0f, 1.0f + expf(-v)); }
}  // namespace

// grid (groups, token tiles); a group = slices_per_cta consecutive slices.  Dynamic shared memory:
// w_s[24][132] (a slice of hc_fn, row stride padded so that the four output groups of a warp hit different banks)
// and x_s[128][132] (the token tile's slice of x as floats, padded so that the eight token groups do).
// Lane = (output group og = lane / 8: outputs 6 og .. 6 og + 5) x (token group tg = lane % 8: tokens tg, tg + 8 of
// the warp's 16): per four columns 6 + 2 sixteen-byte shared-memory loads (broadcast within a group) feed 48 FMAs.
__global__ void __launch_bounds__(kHcDotThreads) hc_pre_dots_kernel(HcPreParams p, int slices_per_cta) {
  extern __shared__ __align__(16) float hc_smem[];
  float* w_s = hc_smem;                               // [kHcMix][kHcPad]
  float* x_s = hc_smem + kHcMix * kHcPad;             // [kHcTokTile][kHcPad]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = blockIdx.x, t0 = blockIdx.y * kHcTokTile;
  const int ntok = min(kHcTokTile, p.t - t0);
  const int og = lane >> 3, tg = lane & 7;
  const int tok_a = warp * 16 + tg, tok_b = tok_a + 8;
  float acc_a[6], acc_b[6];
#pragma unroll
  for (int i = 0; i < 6; ++i) acc_a[i] = acc_b[i] = 0.f;
  for (int s = 0; s < slices_per_cta; ++s) {
    const int k0 = (group * slices_per_cta + s) * kHcSlice;
    __syncthreads();  // the previous slice has been consumed
    for (int i = tid; i < kHcMix * (kHcSlice / 4); i += kHcDotThreads) {
      const int m = i / (kHcSlice / 4), c4 = i % (kHcSlice / 4);
      *reinterpret_cast<float4*>(&w_s[m * kHcPad + 4 * c4]) =
          __ldg(reinterpret_cast<const float4*>(p.hc_fn + static_cast<size_t>(m) * kHcK + k0 + 4 * c4));
    }
    for (int i = tid; i < kHcTokTile * (kHcSlice / 4); i += kHcDotThreads) {
      const int tok = i / (kHcSlice / 4), c4 = i % (kHcSlice / 4);
      float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tok < ntok) {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(p.x + static_cast<size_t>(t0 + tok) * kHcK + k0 + 4 * c4));
        f = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                        __uint_as_float(v.y & 0xffff0000u));
      }
      *reinterpret_cast<float4*>(&x_s[tok * kHcPad + 4 * c4]) = f;
    }
    __syncthreads();
    if (warp * 16 < ntok) {
      const float* wl = w_s + og * 6 * kHcPad;
      const float* xa = x_s + tok_a * kHcPad;
      const float* xb = x_s + tok_b * kHcPad;
#pragma unroll 2
      for (int col = 0; col < kHcSlice; col += 4) {
        const float4 va = *reinterpret_cast<const float4*>(xa + col);
        const float4 vb = *reinterpret_cast<const float4*>(xb + col);
#pragma unroll
        for (int i = 0; i < 6; ++i) {
          const float4 w = *reinterpret_cast<const float4*>(wl + i * kHcPad + col);
          acc_a[i] = fmaf(va.x, w.x, acc_a[i]);
          acc_a[i] = fmaf(va.y, w.y, acc_a[i]);
          acc_a[i] = fmaf(va.z, w.z, acc_a[i]);
          acc_a[i] = fmaf(va.w, w.w, acc_a[i]);
          acc_b[i] = fmaf(vb.x, w.x, acc_b[i]);
          acc_b[i] = fmaf(vb.y, w.y, acc_b[i]);
          acc_b[i] = fmaf(vb.z, w.z, acc_b[i]);
          acc_b[i] = fmaf(vb.w, w.w, acc_b[i]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 6; ++i) {
    if (tok_a < ntok) p.partial[(static_cast<size_t>(group) * p.t + t0 + tok_a) * kHcMix + og * 6 + i] = acc_a[i];
    if (tok_b < ntok) p.partial[(static_cast<size_t>(group) * p.t + t0 + tok_b) * kHcMix + og * 6 + i] = acc_b[i];
  }
}

__global__ void __launch_bounds__(kHcFinThreads) hc_pre_finish_kernel(HcPreParams p, int groups) {
  __shared__ float red_s[kHcFinThreads / 32][32];
  __shared__ float mix_s[kHcOut];
  __shared__ float pre_s[kHc];
  const int tok = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // this thread's 32 values of x: columns 8 tid .. 8 tid + 7 of the four streams, one 16-byte load per stream
  const __nv_bfloat16* xrow = p.x + static_cast<size_t>(tok) * kHcK;
  float x[kHc][8];
  float sq = 0.f;
#pragma unroll
  for (int h = 0; h < kHc; ++h) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(xrow + h * kHcD + 8 * tid));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      x[h][2 * j] = __uint_as_float(w[j] << 16);
      x[h][2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      sq = fmaf(x[h][2 * j], x[h][2 * j], sq);
      sq = fmaf(x[h][2 * j + 1], x[h][2 * j + 1], sq);
    }
  }
  // partial dot products: lane = output m, warp w adds the groups w, w + 16, ...; then the 16 warps in order
  float part = 0.f;
  if (lane < kHcMix)
    for (int g = warp; g < groups; g += kHcFinThreads / 32) part += p.partial[(static_cast<size_t>(g) * p.t + tok) * kHcMix + lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  red_s[warp][lane] = (lane == kHcMix) ? sq : part;   // column 24 carries the sum of squares
  __syncthreads();
  if (tid < kHcOut) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kHcFinThreads / 32; ++w) s += red_s[w][tid];
    mix_s[tid] = s;
  }
  __syncthreads();
  if (warp == 0) {
    const float denom = sqrtf(__fdiv_rn(mix_s[kHcMix], static_cast<float>(kHcK)) + p.norm_eps);
    if (lane < kHc) {
      const float v = __fdiv_rn(mix_s[lane], denom);
      pre_s[lane] = hc_sigmoid(fmaf(v, p.hc_scale[0], p.hc_base[lane])) + p.hc_eps;
    } else if (lane < 2 * kHc) {
      const float v = __fdiv_rn(mix_s[lane], denom);
      p.post[static_cast<size_t>(tok) * kHc + (lane - kHc)] = 2.0f * hc_sigmoid(fmaf(v, p.hc_scale[1], p.hc_base[lane]));
    }
    // Sinkhorn on lanes 0..15: lane = 4 * row + col; sums over a row = lanes differing in bits 0..1, over a
    // column = lanes differing in bits 2..3.  Lanes 16..31 run the same code on copies and store nothing.
    const int e = lane & 15;
    float c = fmaf(__fdiv_rn(mix_s[2 * kHc + e], denom), p.hc_scale[2], p.hc_base[2 * kHc + e]);
    float rmax = fmaxf(c, __shfl_xor_sync(0xffffffffu, c, 1));
    rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
    c = expf(c - rmax);
    auto row_sum = [](float v) {
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      return v + __shfl_xor_sync(0xffffffffu, v, 2);
    };
    auto col_sum = [](float v) {
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      return v + __shfl_xor_sync(0xffffffffu, v, 8);
    };
    c = __fdiv_rn(c, row_sum(c)) + p.hc_eps;
    c = __fdiv_rn(c, col_sum(c) + p.hc_eps);
    for (int it = 1; it < p.iters; ++it) {
      c = __fdiv_rn(c, row_sum(c) + p.hc_eps);
      c = __fdiv_rn(c, col_sum(c) + p.hc_eps);
    }
    if (lane < kHc * kHc) p.comb[static_cast<size_t>(tok) * (kHc * kHc) + lane] = c;
  }
  __syncthreads();
  const float p0 = pre_s[0], p1 = pre_s[1], p2 = pre_s[2], p3 = pre_s[3];
  uint32_t out[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float s0 = __fmul_rn(p0, x[0][2 * j]), s1 = __fmul_rn(p0, x[0][2 * j + 1]);
    s0 = __fadd_rn(s0, __fmul_rn(p1, x[1][2 * j]));
    s1 = __fadd_rn(s1, __fmul_rn(p1, x[1][2 * j + 1]));
    s0 = __fadd_rn(s0, __fmul_rn(p2, x[2][2 * j]));
    s1 = __fadd_rn(s1, __fmul_rn(p2, x[2][2 * j + 1]));
    s0 = __fadd_rn(s0, __fmul_rn(p3, x[3][2 * j]));
    s1 = __fadd_rn(s1, __fmul_rn(p3, x[3][2 * j + 1]));
    const __nv_bfloat162 b = __floats2bfloat162_rn(s0, s1);
    out[j] = *reinterpret_cast<const uint32_t*>(&b);
  }
  *reinterpret_cast<uint4*>(p.y + static_cast<size_t>(tok) * kHcD + 8 * tid) = make_uint4(out[0], out[1], out[2], out[3]);
}

// Slices per CTA: 1 while that leaves the GPU short of CTAs, more (a power of two up to 32) with many token tiles.
static int hc_pre_slices_per_cta(int t) {
  const int tiles = (t + kHcTokTile - 1) / kHcTokTile;
  int spc = 1;
  while (spc < 32 && (kHcSlices / (spc * 2)) * tiles >= 592) spc *= 2;
  return spc;
}

size_t hc_pre_workspace_bytes(int t) {
  if (t <= 0) return 0;
  return static_cast<size_t>(kHcSlices / hc_pre_slices_per_cta(t)) * t * kHcMix * sizeof(float);
}

int launch_hc_pre(const HcPreParams& p, cudaStream_t stream) {
  if (p.t <= 0) return DSV32_OK;
  const int spc = hc_pre_slices_per_cta(p.t);
  const int groups = kHcSlices / spc;
  const int tiles = (p.t + kHcTokTile - 1) / kHcTokTile;
  cudaFuncSetAttribute(hc_pre_dots_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kHcDotSmem));
  hc_pre_dots_kernel<<<dim3(groups, tiles), kHcDotThreads, kHcDotSmem, stream>>>(p, spc);
  count_launch();
  int rc = check_launch("hc_pre_dots_kernel");
  if (rc != DSV32_OK) return rc;
  hc_pre_finish_kernel<<<p.t, kHcFinThreads, 0, stream>>>(p, groups);
  count_launch();
  return check_launch("hc_pre_finish_kernel");
}

}  // namespace dsv32

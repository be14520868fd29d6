// Split-KV combine of the sparse flash attention: every key split leaves a normalised fp32 partial output and
// the log-sum-exp of its scores; the result is out = sum_s w_s * O_s with w_s = exp(lse_s - max) / sum exp(lse - max)
// (the flash-decoding merge; the operator itself is models/deepseek_v32_exp/sparse_flash_attention_quant_impl.py:121-286).
#include "kernels.cuh"

namespace dsv32 {

// One CTA per (token, head) row of 512 value dims, four dims per thread.
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

int launch_sfa_combine(const SfaParams& p, cudaStream_t stream) {
  const int t = p.b * p.s1;
  sfa_combine_kernel<<<t * p.nq, 128, 0, stream>>>(p.part_o, p.part_lse, p.out, p.splits, p.nq);
  count_launch();
  return check_launch("sfa_combine_kernel");
}

}  // namespace dsv32

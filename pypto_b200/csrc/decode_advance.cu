// Moves a decode batch to its next step on the device: every request's sequence length grows by the tokens the
// next step appends, and the cache rows those tokens will be written to follow from the page table by the
// reference's rule (models/deepseek_v32_exp/deepseekv32_mla_indexer_prolog_quant.py:184-194):
//   pos = act_seq - s1 + j,   cache_index[b, j] = block_table[b, pos / block_size] * block_size + pos % block_size.
// A launch of one small kernel, so that a multi-step decode loop (prologs -> indexer -> attention -> advance) can be
// captured in a CUDA graph without a host round trip between steps.
#include "kernels.cuh"

namespace dsv32 {

__global__ void __launch_bounds__(128) decode_advance_kernel(AdvanceParams p) {
  const int bi = blockIdx.x * 128 + threadIdx.x;  // one thread per request: it alone reads and writes the request's length
  if (bi >= p.b) return;
  const int seq = p.act_seq[bi] + p.grow;         // length including the tokens of the step being prepared
  for (int j = 0; j < p.s1; ++j) {
    const int pos = seq - p.s1 + j;
    long long row = -1;                           // -1: the prologs report the token and skip its cache rows
    if (pos >= 0) {
      const int lb = pos / p.block_size;
      if (lb >= p.max_blocks) {
        report_status(p.status, DSV32_STATUS_BAD_INDEX, bi, static_cast<uint32_t>(pos));
      } else {
        const int pb = p.block_table[static_cast<size_t>(bi) * p.max_blocks + lb];
        if (pb < 0) report_status(p.status, DSV32_STATUS_BAD_PAGE, bi, static_cast<uint32_t>(pos));
        else row = static_cast<long long>(pb) * p.block_size + pos % p.block_size;
      }
    }
    p.cache_index[static_cast<size_t>(bi) * p.s1 + j] = row;
  }
  p.act_seq[bi] = seq;
}

int launch_decode_advance(const AdvanceParams& p, cudaStream_t stream) {
  if (p.b <= 0 || p.s1 <= 0) return DSV32_OK;
  decode_advance_kernel<<<(p.b + 127) / 128, 128, 0, stream>>>(p);
  count_launch();
  return check_launch("decode_advance_kernel");
}

}  // namespace dsv32

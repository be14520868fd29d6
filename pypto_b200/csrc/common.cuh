// Shared device/host helpers for the dsv32_b200 kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dsv32_b200.h"

namespace dsv32 {

// ---- host-side bookkeeping (api.cu) -------------------------------------------------
void set_error(const char* fmt, ...);
void count_launch(int n = 1);
int check_launch(const char* what);  // cudaGetLastError -> DSV32_ERR_CUDA + message

constexpr int kIdxHeads = 64;
constexpr int kIdxDim = 128;
constexpr int kKvLora = 512;
constexpr int kRopeDim = 64;
constexpr int kQkDim = kKvLora + kRopeDim;  // 576

// ---- device helpers -----------------------------------------------------------------
__device__ __forceinline__ void report_status(uint32_t* status, uint32_t code, uint32_t a, uint32_t b) {
  if (status != nullptr && atomicCAS(status, 0u, code) == 0u) {
    status[1] = a;
    status[2] = b;
  }
}

// order-preserving map fp32 -> uint32 (larger float -> larger key); NaN sorts above +inf
__device__ __forceinline__ uint32_t float_to_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace dsv32

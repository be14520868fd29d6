// Allocation-free variant of the lightning indexer + top-k entry point.
//
// Some callers cannot allocate device memory at the time they need this operator: a serving loop that
// has handed the whole device to its own memory pool and runs with allocation disabled, a plugin host
// that forbids cudaMalloc inside operator calls, or code running where an allocation would
// synchronise the device.  For them the fp32 score rows (the only scratch memory of this operator) live
// in a fixed array inside the library image instead of a caller- or library-allocated workspace.
#include <mutex>

#include "kernels.cuh"

namespace dsv32 {

// 8 MiB of scores: b * s1 * max_blocks * block_size <= 2,097,152 (for example 16 query tokens at a
// 128K-token context, or 32 at 64K).  Every GPU that loads the library holds this array until exit.
constexpr size_t kNoAllocScratchBytes = DSV32_NOALLOC_INDEXER_MAX_SCORES * sizeof(float);
static __device__ __align__(256) unsigned char g_indexer_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices];  // device address of g_indexer_scratch, per device
static std::mutex g_scratch_mutex;

// In host code `g_indexer_scratch` is only a handle for the runtime, not a device address; the address
// that kernels may use is looked up once per device, with that device current.  "That device" is the CURRENT
// device of the calling thread, which must be the device `cuda_stream` belongs to.
static int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("indexer (no-alloc): cannot identify the current device: %s", cudaGetErrorString(e));
    return DSV32_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] != nullptr) {
    // A device reset (or a destroyed and re-created primary context) makes the remembered address stale: it is
    // kept only while the runtime still knows it as device memory of this device.
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, g_scratch_addr[dev]) != cudaSuccess || attr.type != cudaMemoryTypeDevice ||
        attr.device != dev) {
      (void)cudaGetLastError();
      g_scratch_addr[dev] = nullptr;
    }
  }
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_indexer_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      set_error("indexer (no-alloc): cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return DSV32_ERR_CUDA;
    }
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return DSV32_OK;
}

}  // namespace dsv32

extern "C" int dsv32_indexer_topk_noalloc(const Dsv32IndexerArgs* a, void* cuda_stream) {
  using namespace dsv32;
  if (a == nullptr) {
    set_error("indexer (no-alloc): args is NULL");
    return DSV32_ERR_INVALID_ARG;
  }
  if (a->b < 0 || a->s1 < 1 || a->max_blocks < 1 || a->block_size != 128) {
    set_error("indexer (no-alloc): bad b=%d s1=%d max_blocks=%d block_size=%d", a->b, a->s1, a->max_blocks,
              a->block_size);
    return DSV32_ERR_INVALID_ARG;
  }
  const unsigned long long need =
      static_cast<unsigned long long>(a->b) * a->s1 * a->max_blocks * a->block_size;
  if (need > DSV32_NOALLOC_INDEXER_MAX_SCORES) {
    set_error("indexer (no-alloc): b*s1*max_blocks*block_size = %llu scores exceed the built-in scratch of %llu; "
              "use dsv32_indexer_topk with a caller workspace",
              need, static_cast<unsigned long long>(DSV32_NOALLOC_INDEXER_MAX_SCORES));
    return DSV32_ERR_WORKSPACE;
  }
  if (a->score_ld != 0 && a->score_ld != a->max_blocks * a->block_size) {
    set_error("indexer (no-alloc): score_ld must be 0 or max_blocks*block_size");
    return DSV32_ERR_INVALID_ARG;
  }
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != DSV32_OK) return rc;
  Dsv32IndexerArgs args = *a;
  args.scores_out = static_cast<float*>(scratch);  // score rows go to the built-in array
  args.workspace = nullptr;
  args.workspace_bytes = 0;
  args.score_ld = 0;
  return dsv32_indexer_topk(&args, cuda_stream);
}

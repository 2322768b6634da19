// dz_sbmm_static: the SBMM entry point for callers that cannot allocate device
// memory.  Some hosts of this library run it from contexts where cudaMalloc is
// off limits -- a serving loop that has handed all device memory to its own
// pool, a plugin loaded into a process whose allocator it must not touch, code
// that runs while a CUDA graph is being captured on another stream of the
// device.  dz_sbmm asks such a caller for a workspace it has no way to get.
// This variant keeps the kernel's scratch (status word, per-tile counters,
// split-K partial tiles) in a fixed array that is part of the library image, so
// the call allocates nothing: no cudaMalloc / cudaFree, no allocating library
// routine, and the caller passes inputs and outputs only.
//
// The price is a fixed maximum size and one shared buffer:
//   * at most kStaticMaxTokens tokens per call, and the caller must pass the
//     tokens sorted by slot (tokens_sorted = 1), because the unsorted path
//     needs a gather buffer proportional to M * K;
//   * every GPU that loads the library holds kStaticBytes of device memory from
//     load until process exit;
//   * all calls on a device use the same array, which keeps whatever the last
//     call left in it.  The status word and the tile counters are cleared at the
//     start of every call (a memset on the caller's stream); the partial tiles
//     are always written before they are read.  Two calls that overlap on the GPU
//     (different streams, no ordering between them) race on the array and give
//     undefined results -- order them.
#include <mutex>

#include "dz_common.cuh"

namespace dz {
namespace {

constexpr int kStaticMaxTokens = 64;
// status + counters (16640 B) and 160 CTAs x 2 partial tiles x 64 columns x 128 rows x 4 B
constexpr size_t kStaticBytes = 16640 + (size_t)160 * 2 * kStaticMaxTokens * 128 * 4;
constexpr size_t kStaticClearBytes = 16640;

// Device-resident scratch.  In host code this name is only a handle for the
// runtime's symbol table, never a device address: the address the kernel gets
// is looked up with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

std::mutex g_setup_mutex;
void* g_scratch_ptr[64] = {nullptr};

// Once per device, with that device current: resolve the array's device address.
int static_scratch_for_current_device(void** out) {
  int dev = 0;
  DZ_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return DZ_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    DZ_CUDA_OK(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (!ptr) return DZ_ERR_CUDA;
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return DZ_OK;
}

}  // namespace
}  // namespace dz

using namespace dz;

extern "C" int dz_sbmm_static_max_tokens(void) { return kStaticMaxTokens; }

extern "C" int dz_sbmm_static(const dz_sbmm_args* args, void* stream) {
  if (!args) return DZ_ERR_INVALID_ARG;
  if (args->M < 0) return DZ_ERR_INVALID_ARG;
  if (args->M == 0) return DZ_OK;
  if (args->M > kStaticMaxTokens) return DZ_ERR_TOO_LARGE;   // scratch is sized for 64 tokens
  if (!args->tokens_sorted) return DZ_ERR_TOO_LARGE;         // the gather buffer does not fit
  if (!args->x || !args->w_base || !args->y || !args->qweight || !args->meta || !args->scales ||
      !args->segments)
    return DZ_ERR_INVALID_ARG;
  if (args->N <= 0 || args->K <= 0) return DZ_ERR_INVALID_ARG;
  if (args->N % kTileN != 0 || args->K % kBlockK != 0 || (args->bits != 2 && args->bits != 4))
    return DZ_ERR_SHAPE;
  if (args->dtype != DZ_DTYPE_F16 && args->dtype != DZ_DTYPE_BF16) return DZ_ERR_INVALID_ARG;
  if (args->num_slots <= 0 || args->num_slots > kMaxSlots) return DZ_ERR_INVALID_ARG;
  if (!aligned16(args->x) || !aligned16(args->w_base) || !aligned16(args->y) ||
      !aligned16(args->qweight) || !aligned16(args->meta) || (args->qweight_stride & 15) ||
      (args->meta_stride & 15) || (args->scales_stride & 1))
    return DZ_ERR_ALIGNMENT;
  if (sbmm_workspace_bytes(args->M, args->N, args->K, 1) > kStaticBytes) return DZ_ERR_TOO_LARGE;

  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);   // first call on a device: set-up
  if (rc) return rc;

  cudaStream_t st = (cudaStream_t)stream;
  // the status word and the tile counters must start at zero
  DZ_CUDA_OK(cudaMemsetAsync(scratch, 0, kStaticClearBytes, st));
  dz_sbmm_args a = *args;
  a.workspace = scratch;
  a.workspace_bytes = kStaticBytes;
  return launch_sbmm(a, false, st);
}

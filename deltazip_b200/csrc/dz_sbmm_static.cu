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
//     call left in it.  The tile counters are cleared at the start of every call
//     (a memset on the caller's stream); the partial tiles are always written
//     before they are read.  The status word is NOT cleared per call: what a
//     kernel reports there (a rejected batch, a wait that ran out) stays until
//     dz_sbmm_static_status reads and clears it.  Two calls that overlap on the
//     GPU (different streams, no ordering between them) race on the array and
//     give undefined results -- order them.
#include <mutex>

#include "dz_common.cuh"

namespace dz {
namespace {

constexpr int kStaticMaxTokens = 64;
// status word + tile counters, then the parked partial tiles of a 64-token call
constexpr size_t kStaticBytes = kWsPartials + (size_t)kMaxCtas * 2 * kStaticMaxTokens * 128 * 4;
static_assert(kWsStatus + sizeof(int) <= kWsCounters, "status word precedes the counters");
static_assert(kStaticMaxTokens % 16 == 0 && kStaticMaxTokens <= kTokenBlock,
              "the partial area below is that of one token block of kStaticMaxTokens columns");

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
  if (args->M > kStaticMaxTokens) return DZ_ERR_TOO_LARGE;   // scratch is sized for 64 tokens
  if (args->M > 0 && !args->tokens_sorted) return DZ_ERR_TOO_LARGE;   // no room for a gather buffer
  int rc = check_sbmm_args(args, false, /*check_workspace=*/false);   // same rules as dz_sbmm
  if (rc || args->M == 0) return rc;
  if (sbmm_workspace_bytes(args->M, args->N, args->K, 1) > kStaticBytes) return DZ_ERR_TOO_LARGE;

  void* scratch = nullptr;
  rc = static_scratch_for_current_device(&scratch);   // first call on a device: set-up
  if (rc) return rc;

  cudaStream_t st = (cudaStream_t)stream;
  // the tile counters must start at zero; the status word before them is left alone
  DZ_CUDA_OK(cudaMemsetAsync(static_cast<unsigned char*>(scratch) + kWsCounters, 0,
                             kWsCountersBytes, st));
  dz_sbmm_args a = *args;
  a.workspace = scratch;
  a.workspace_bytes = kStaticBytes;
  return launch_sbmm(a, false, st);
}

// Reads and clears the status word of the built-in scratch on the current device.  Works on
// the cached device address and a stack variable of the caller: no allocation.
extern "C" int dz_sbmm_static_status(void* stream, int* host_out) {
  if (!host_out) return DZ_ERR_INVALID_ARG;
  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  int* word = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch) + kWsStatus);
  DZ_CUDA_OK(cudaMemcpyAsync(host_out, word, sizeof(int), cudaMemcpyDeviceToHost, st));
  DZ_CUDA_OK(cudaMemsetAsync(word, 0, sizeof(int), st));
  DZ_CUDA_OK(cudaStreamSynchronize(st));
  return DZ_OK;
}

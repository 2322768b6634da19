// One-shot all-reduce (sum) over peer memory for the small [tokens, hidden] partial outputs of
// the row-parallel delta layers.  Role of the reference's CustomAllreduce
// (serving/vllm/model_executor/parallel_utils/custom_all_reduce.py:187-262, kernels in
// serving/csrc/custom_all_reduce.cuh); the design here is different:
//
//   * every rank owns one "region" (cudaMalloc'ed by this library, exported through CUDA IPC):
//     a flag table and two staging buffers used alternately;
//   * a call is ONE kernel per rank.  Block b of every rank handles slice b of the message: it
//     (1) copies its slice of the input into the rank's staging buffer (skipped when the caller
//     wrote its data there directly), (2) stores the call's epoch into flag[rank][b] of every
//     peer with a system-scope release, (3) waits, bounded, until flag[peer][b] of its own table
//     holds the epoch for every peer, (4) sums slice b of all ranks' staging buffers in rank
//     order in fp32 (plain peer loads over NVLink) and writes the result.  No grid-wide
//     synchronisation is needed because slice b is produced and consumed by block b everywhere.
//   * staging buffers alternate between calls: a rank can only be one call ahead of a peer
//     (step 3 of call n+1 needs the peer's flag of call n+1), so a buffer is never overwritten
//     while a peer may still read it.
//   * all ranks add in the same order, so every rank gets bit-identical results.
//
// A wait that does not complete within the time limit records DZ_ERR_TIMEOUT in the region's
// status word and the kernel returns without reducing; nothing spins forever.
// No multicast objects are used, only ordinary peer loads and stores.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <string.h>

#include <new>

#include "dz_common.cuh"

struct dz_allreduce_ctx {
  int rank = 0, world = 0, device = 0;
  size_t max_bytes = 0, region_bytes = 0;
  uint8_t* region = nullptr;               // own region
  uint8_t* peers[8] = {nullptr};           // regions of all ranks (own included), rank order
  bool imported[8] = {false};
  unsigned epoch = 0;                      // calls so far
  bool connected = false;
};

namespace dz {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxBlocks = 64;
constexpr int kArThreads = 512;
constexpr size_t kStatusOff = 0;                        // int status
constexpr size_t kFlagsOff = 4096;                      // uint32 flag[kMaxWorld][kMaxBlocks]
constexpr size_t kStagingOff = 8192;
constexpr unsigned long long kArTimeoutNs = 1000ull * 1000 * 1000;

struct ArParams {
  uint8_t* peers[kMaxWorld];
  const void* in;
  void* out;
  long long count;          // elements
  int rank, world, parity, copy_in;
  unsigned epoch;
  size_t staging_bytes;     // bytes of one staging buffer
};

__device__ __forceinline__ unsigned long long ar_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint4 ld_peer(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

template <typename T> struct Vec;   // 16-byte vector of T <-> fp32
template <> struct Vec<__half> {
  static constexpr int kN = 8;
  static __device__ __forceinline__ void add(float* acc, const uint4& v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* acc) {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
    return v;
  }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int kN = 8;
  static __device__ __forceinline__ void add(float* acc, const uint4& v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* acc) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    return v;
  }
};
template <> struct Vec<float> {
  static constexpr int kN = 4;
  static __device__ __forceinline__ void add(float* acc, const uint4& v) {
    acc[0] += __uint_as_float(v.x);
    acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z);
    acc[3] += __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* acc) {
    return make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]),
                      __float_as_uint(acc[3]));
  }
};

template <typename T, int WORLD>
__global__ void __launch_bounds__(kArThreads)
allreduce_oneshot_kernel(const ArParams p) {
  __shared__ int s_abort;
  const int b = blockIdx.x, nb = gridDim.x;
  const long long nvec = p.count / Vec<T>::kN;            // 16-byte vectors in the message
  const long long per = (nvec + nb - 1) / nb;
  const long long v0 = min(nvec, (long long)b * per), v1 = min(nvec, v0 + per);
  uint8_t* const mine = p.peers[p.rank];
  uint4* const my_stage =
      reinterpret_cast<uint4*>(mine + kStagingOff + (size_t)p.parity * p.staging_bytes);
  if (threadIdx.x == 0) s_abort = 0;

  // Launched with programmatic stream serialization: everything above overlaps the tail of
  // the kernel that produced the input; its writes are visible after this wait.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // (1) this block's slice of the input into the staging buffer
  if (p.copy_in) {
    const uint4* src = reinterpret_cast<const uint4*>(p.in);
    for (long long i = v0 + threadIdx.x; i < v1; i += kArThreads) my_stage[i] = src[i];
  }
  __syncthreads();

  // (2) + (3): one thread per peer publishes this slice and waits for the peer's
  if (threadIdx.x < WORLD && threadIdx.x != p.rank) {
    const int peer = threadIdx.x;
    unsigned* remote =
        reinterpret_cast<unsigned*>(p.peers[peer] + kFlagsOff) + p.rank * kMaxBlocks + b;
    // this block's copy (or, when the producer wrote the staging buffer directly, the earlier
    // kernel's stores, ordered before this point by the dependency wait) must be visible to the
    // peer before the flag: a system-scope release in both cases
    if (p.copy_in) __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(p.epoch) : "memory");
    const unsigned* local =
        reinterpret_cast<const unsigned*>(mine + kFlagsOff) + peer * kMaxBlocks + b;
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
      unsigned seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(local) : "memory");
      if ((int)(seen - p.epoch) >= 0) break;
      if ((it & 255u) == 255u) {
        const unsigned long long now = ar_globaltimer();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > kArTimeoutNs) {
          s_abort = 1;
          atomicCAS(reinterpret_cast<int*>(mine + kStatusOff), 0, (int)DZ_ERR_TIMEOUT);
          break;
        }
      }
    }
  }
  __syncthreads();
  if (s_abort) return;

  // (4) sum of slice b over the ranks, in rank order; two vectors per rank in flight per thread
  const uint4* stage[WORLD];
#pragma unroll
  for (int r = 0; r < WORLD; ++r)
    stage[r] = reinterpret_cast<const uint4*>(p.peers[r] + kStagingOff +
                                              (size_t)p.parity * p.staging_bytes);
  uint4* dst = reinterpret_cast<uint4*>(p.out);
  for (long long i = v0 + threadIdx.x; i < v1; i += 2 * kArThreads) {
    const long long i2 = i + kArThreads;
    const bool two = i2 < v1;
    uint4 va[WORLD], vb[WORLD];
#pragma unroll
    for (int r = 0; r < WORLD; ++r) {
      va[r] = ld_peer(stage[r] + i);
      if (two) vb[r] = ld_peer(stage[r] + i2);
    }
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int r = 0; r < WORLD; ++r) Vec<T>::add(acc, va[r]);
    dst[i] = Vec<T>::pack(acc);
    if (two) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int r = 0; r < WORLD; ++r) Vec<T>::add(acc, vb[r]);
      dst[i2] = Vec<T>::pack(acc);
    }
  }
}

template <typename T>
cudaError_t launch_allreduce(const ArParams& p, int blocks, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kArThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  switch (p.world) {
    case 1: return cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<T, 1>, p);
    case 2: return cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<T, 2>, p);
    case 3: return cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<T, 3>, p);
    case 4: return cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<T, 4>, p);
    case 5: return cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<T, 5>, p);
    case 6: return cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<T, 6>, p);
    case 7: return cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<T, 7>, p);
    default: return cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<T, 8>, p);
  }
}

}  // namespace
}  // namespace dz

using namespace dz;

extern "C" {

size_t dz_allreduce_region_bytes(size_t max_bytes) {
  return kStagingOff + 2 * ((max_bytes + 255) & ~(size_t)255);
}

int dz_allreduce_create(dz_allreduce_ctx** out, int rank, int world, size_t max_bytes) {
  if (!out || world < 1 || world > kMaxWorld || rank < 0 || rank >= world || max_bytes == 0)
    return DZ_ERR_INVALID_ARG;
  dz_allreduce_ctx* c = new (std::nothrow) dz_allreduce_ctx();
  if (!c) return DZ_ERR_CUDA;
  c->rank = rank;
  c->world = world;
  c->max_bytes = (max_bytes + 255) & ~(size_t)255;
  c->region_bytes = dz_allreduce_region_bytes(max_bytes);
  if (cudaGetDevice(&c->device) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&c->region), c->region_bytes) != cudaSuccess ||
      cudaMemset(c->region, 0, kStagingOff) != cudaSuccess) {
    if (c->region) cudaFree(c->region);
    delete c;
    return DZ_ERR_CUDA;
  }
  c->peers[rank] = c->region;
  c->connected = (world == 1);
  *out = c;
  return DZ_OK;
}

int dz_allreduce_export(dz_allreduce_ctx* c, unsigned char* handle) {
  if (!c || !handle) return DZ_ERR_INVALID_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  DZ_CUDA_OK(cudaIpcGetMemHandle(&h, c->region));
  memcpy(handle, &h, sizeof(h));
  return DZ_OK;
}

int dz_allreduce_connect(dz_allreduce_ctx* c, const unsigned char* handles) {
  if (!c || !handles) return DZ_ERR_INVALID_ARG;
  if (c->connected) return DZ_OK;
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)r * 64, sizeof(h));
    void* ptr = nullptr;
    DZ_CUDA_OK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    c->peers[r] = reinterpret_cast<uint8_t*>(ptr);
    c->imported[r] = true;
  }
  c->connected = true;
  return DZ_OK;
}

int dz_allreduce_staging(dz_allreduce_ctx* c, void** ptr, size_t* bytes) {
  if (!c || !ptr) return DZ_ERR_INVALID_ARG;
  *ptr = c->region + kStagingOff + (size_t)(c->epoch & 1u) * c->max_bytes;
  if (bytes) *bytes = c->max_bytes;
  return DZ_OK;
}

int dz_allreduce_run(dz_allreduce_ctx* c, const void* in, void* out, int64_t count, int dtype,
                     void* stream) {
  if (!c || !in || !out || count < 0) return DZ_ERR_INVALID_ARG;
  if (!c->connected) return DZ_ERR_INVALID_ARG;
  const size_t esz = dtype == DZ_DTYPE_F32 ? 4 : 2;
  if (dtype != DZ_DTYPE_F16 && dtype != DZ_DTYPE_BF16 && dtype != DZ_DTYPE_F32)
    return DZ_ERR_UNSUPPORTED;
  const size_t bytes = (size_t)count * esz;
  if (bytes > c->max_bytes) return DZ_ERR_TOO_LARGE;
  if (bytes % 16 || ((uintptr_t)in & 15) || ((uintptr_t)out & 15)) return DZ_ERR_ALIGNMENT;
  if (count == 0) return DZ_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  ArParams p;
  for (int r = 0; r < kMaxWorld; ++r) p.peers[r] = c->peers[r < c->world ? r : 0];
  p.parity = (int)(c->epoch & 1u);
  const void* staging = c->region + kStagingOff + (size_t)p.parity * c->max_bytes;
  p.in = in;
  p.out = out;
  p.count = count;
  p.rank = c->rank;
  p.world = c->world;
  p.copy_in = (in != staging) ? 1 : 0;
  p.epoch = ++c->epoch;
  p.staging_bytes = c->max_bytes;
  // one block per 8 KB (one vector per thread and rank), at most kMaxBlocks; every rank
  // computes the same number
  int blocks = (int)((bytes + 8191) / 8192);
  blocks = blocks < 1 ? 1 : (blocks > kMaxBlocks ? kMaxBlocks : blocks);
  if (dtype == DZ_DTYPE_F16) DZ_CUDA_OK(launch_allreduce<__half>(p, blocks, st));
  else if (dtype == DZ_DTYPE_BF16) DZ_CUDA_OK(launch_allreduce<__nv_bfloat16>(p, blocks, st));
  else DZ_CUDA_OK(launch_allreduce<float>(p, blocks, st));
  return DZ_OK;
}

int dz_allreduce_status(dz_allreduce_ctx* c, int* status) {
  if (!c || !status) return DZ_ERR_INVALID_ARG;
  DZ_CUDA_OK(cudaMemcpy(status, c->region + kStatusOff, sizeof(int), cudaMemcpyDeviceToHost));
  return DZ_OK;
}

int dz_allreduce_destroy(dz_allreduce_ctx* c) {
  if (!c) return DZ_OK;
  for (int r = 0; r < c->world; ++r)
    if (c->imported[r]) cudaIpcCloseMemHandle(c->peers[r]);
  if (c->region) cudaFree(c->region);
  delete c;
  return DZ_OK;
}

}  // extern "C"

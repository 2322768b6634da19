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
// Larger messages on more ranks use a second, two-stage kernel with the same flag protocol
// (the reference switches the same way, serving/csrc/custom_all_reduce.cuh:443-456, kernels
// :181-250): the message is cut into `world` parts; (A) rank r sums part r of all ranks' staging
// buffers and puts the sum back into part r of its own staging buffer (nobody else reads that
// part in stage A), (B) publishes it with a second flag and every rank collects the reduced
// parts of all peers.  Each rank then pulls 2 (world-1)/world of the message over NVLink
// instead of (world-1) times the message.
//
// Third form, fused with the producer: the row-parallel SBMM does not write its partial output
// to local memory at all -- its epilogue stores every finished output tile straight into a
// receive slot (one per source rank) inside EVERY rank's region and then raises a per-tile flag
// there (dz_allreduce_push_target hands the kernel the addresses).  The transfer rides under the
// SBMM's own tail; the reduction (dz_allreduce_run_pushed) only waits for flags that are usually
// set already and sums slots in local memory, in rank order.
//
// Fourth form, for regions the caller allocated as symmetric memory with a multicast mapping
// (dz_allreduce_create_external): after the same flag exchange, every rank reads its result with
// multimem.ld_reduce -- the NVSwitch adds the ranks' copies in flight (fp32 accumulation) and one
// load returns the sum, so a rank pulls the message once instead of (world - 1) times.
//
// A wait that does not complete within the time limit records DZ_ERR_TIMEOUT in the region's
// status word and the kernel returns without reducing; nothing spins forever.
// The first three forms use ordinary peer loads and stores only.
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
  int force_variant = 0;                   // 0: by size, 1: one-shot, 2: two-stage, 3: in-switch (tests / tuning)
  bool owned = true;                       // region allocated (and IPC-exported) by this library
  uint8_t* multicast = nullptr;            // multicast address of the regions (NVSwitch), or null
  bool nvls_default = false;               // use the in-switch kernel when no variant is forced
};

namespace dz {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxBlocks = 64;
constexpr int kArThreads = 512;
constexpr size_t kStatusOff = 0;                        // int status
constexpr size_t kFlagsOff = 4096;                      // uint32 flag[kMaxWorld][kMaxBlocks]
constexpr size_t kFlags2Off = 4096 + 2048;              // second table (two-stage kernel, stage B)
constexpr size_t kPushFlagsOff = 8192;                  // uint32 flag[kMaxWorld][DZ_PUSH_MAX_FLAGS]
constexpr size_t kStagingOff = 16384;
constexpr size_t kPushSlotBytes = (size_t)2 << 20;      // receive slot per source rank and parity
static_assert(kMaxWorld * DZ_PUSH_MAX_FLAGS * 4 <= kStagingOff - kPushFlagsOff, "push flag table");
static_assert(kMaxWorld * kMaxBlocks * 4 <= 2048, "flag tables are 2 KB each");
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

// Publishes `epoch` in table `flags_off`, entry [rank][b], of every peer and waits (bounded) until
// every peer's entry [peer][b] of the own table holds it.  Called by the first WORLD threads.
template <int WORLD>
__device__ __forceinline__ void publish_and_wait(const ArParams& p, size_t flags_off, int b,
                                                 bool fence_first, int* s_abort) {
  if (threadIdx.x < WORLD && (int)threadIdx.x != p.rank) {
    const int peer = threadIdx.x;
    uint8_t* const mine = p.peers[p.rank];
    unsigned* remote = reinterpret_cast<unsigned*>(p.peers[peer] + flags_off) + p.rank * kMaxBlocks + b;
    // the block's stores were ordered before this thread by the preceding __syncthreads(); the
    // system-scope release makes them visible to the peer before the flag
    (void)fence_first;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(p.epoch) : "memory");
    const unsigned* local = reinterpret_cast<const unsigned*>(mine + flags_off) + peer * kMaxBlocks + b;
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
          *s_abort = 1;
          atomicCAS(reinterpret_cast<int*>(mine + kStatusOff), 0, (int)DZ_ERR_TIMEOUT);
          break;
        }
      }
    }
  }
}

// Two-stage form.  Vectors [0, nvec) are cut into WORLD parts of P = ceil(nvec / WORLD) vectors
// and every part into gridDim.x sub-slices; block b works on sub-slice b of every part.
template <typename T, int WORLD>
__global__ void __launch_bounds__(kArThreads)
allreduce_twostage_kernel(const ArParams p) {
  __shared__ int s_abort;
  const int b = blockIdx.x, nb = gridDim.x;
  const long long nvec = p.count / Vec<T>::kN;
  const long long P = (nvec + WORLD - 1) / WORLD;
  const long long S = (P + nb - 1) / nb;
  uint8_t* const mine = p.peers[p.rank];
  uint4* const my_stage =
      reinterpret_cast<uint4*>(mine + kStagingOff + (size_t)p.parity * p.staging_bytes);
  if (threadIdx.x == 0) s_abort = 0;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // sub-slice b of part r: [lo(r), hi(r))
  auto lo = [&](int r) { return min(nvec, min((long long)r * P + (long long)b * S, (long long)(r + 1) * P)); };
  auto hi = [&](int r) { return min(nvec, min((long long)r * P + (long long)(b + 1) * S, (long long)(r + 1) * P)); };

  // copy-in: this block stages its sub-slice of every part
  if (p.copy_in) {
    const uint4* src = reinterpret_cast<const uint4*>(p.in);
#pragma unroll
    for (int r = 0; r < WORLD; ++r)
      for (long long i = lo(r) + threadIdx.x; i < hi(r); i += kArThreads) my_stage[i] = src[i];
  }
  __syncthreads();
  publish_and_wait<WORLD>(p, kFlagsOff, b, p.copy_in != 0, &s_abort);
  __syncthreads();
  if (s_abort) return;

  // stage A: sum of sub-slice b of part `rank` over the ranks, in rank order, into the own buffer
  const uint4* stage[WORLD];
#pragma unroll
  for (int r = 0; r < WORLD; ++r)
    stage[r] = reinterpret_cast<const uint4*>(p.peers[r] + kStagingOff +
                                              (size_t)p.parity * p.staging_bytes);
  uint4* dst = reinterpret_cast<uint4*>(p.out);
  for (long long i = lo(p.rank) + threadIdx.x; i < hi(p.rank); i += kArThreads) {
    uint4 v[WORLD];
#pragma unroll
    for (int r = 0; r < WORLD; ++r) v[r] = ld_peer(stage[r] + i);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int r = 0; r < WORLD; ++r) Vec<T>::add(acc, v[r]);
    const uint4 sum = Vec<T>::pack(acc);
    my_stage[i] = sum;       // only this rank reads part `rank` of its own buffer in stage A
    dst[i] = sum;
  }
  __syncthreads();
  // stage B: the reduced sub-slice is visible to the peers before the second flag
  publish_and_wait<WORLD>(p, kFlags2Off, b, true, &s_abort);
  __syncthreads();
  if (s_abort) return;
#pragma unroll
  for (int r = 0; r < WORLD; ++r) {
    if (r == p.rank) continue;
    for (long long i = lo(r) + threadIdx.x; i < hi(r); i += kArThreads) dst[i] = ld_peer(stage[r] + i);
  }
}

// In-switch reduction: 16 bytes of the sum over all ranks from one multimem load.
template <typename T> struct McLoad;
template <> struct McLoad<__half> {
  static __device__ __forceinline__ uint4 sum(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct McLoad<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 sum(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct McLoad<float> {
  static __device__ __forceinline__ uint4 sum(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};

// Same slicing and flag exchange as the one-shot kernel; the sum comes from the switch.
template <typename T, int WORLD>
__global__ void __launch_bounds__(kArThreads)
allreduce_nvls_kernel(const ArParams p, const uint8_t* __restrict__ mc_region) {
  __shared__ int s_abort;
  const int b = blockIdx.x, nb = gridDim.x;
  const long long nvec = p.count / Vec<T>::kN;
  const long long per = (nvec + nb - 1) / nb;
  const long long v0 = min(nvec, (long long)b * per), v1 = min(nvec, v0 + per);
  uint8_t* const mine = p.peers[p.rank];
  uint4* const my_stage =
      reinterpret_cast<uint4*>(mine + kStagingOff + (size_t)p.parity * p.staging_bytes);
  if (threadIdx.x == 0) s_abort = 0;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (p.copy_in) {
    const uint4* src = reinterpret_cast<const uint4*>(p.in);
    for (long long i = v0 + threadIdx.x; i < v1; i += kArThreads) my_stage[i] = src[i];
  }
  __syncthreads();
  publish_and_wait<WORLD>(p, kFlagsOff, b, p.copy_in != 0, &s_abort);
  __syncthreads();
  if (s_abort) return;
  asm volatile("fence.acq_rel.sys;" ::: "memory");
  const uint4* mc_stage =
      reinterpret_cast<const uint4*>(mc_region + kStagingOff + (size_t)p.parity * p.staging_bytes);
  uint4* dst = reinterpret_cast<uint4*>(p.out);
  for (long long i = v0 + threadIdx.x; i < v1; i += kArThreads) dst[i] = McLoad<T>::sum(mc_stage + i);
}

// Reduction of tiles the producers pushed.  Block b handles output tile b (128 columns of every
// row): it waits (bounded) until every source rank has raised the tile's flag for every token
// block, then sums the `world` receive slots of the own region in rank order.
struct PushedParams {
  uint8_t* region;          // own region
  void* out;
  int M, N, world, parity, token_blocks, num_tiles;
  unsigned epoch;
  size_t push_off;          // byte offset of the receive slots inside the region
};

template <typename T, int WORLD>
__global__ void __launch_bounds__(256)
allreduce_pushed_kernel(const PushedParams p) {
  __shared__ int s_abort;
  const int tile = blockIdx.x;
  if (threadIdx.x == 0) s_abort = 0;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __syncthreads();
  // one waiting thread per (source rank, token block)
  for (int w = threadIdx.x; w < WORLD * p.token_blocks; w += 256) {
    const int src = w / p.token_blocks, tb = w % p.token_blocks;
    const unsigned* flag = reinterpret_cast<const unsigned*>(p.region + kPushFlagsOff) +
                           src * DZ_PUSH_MAX_FLAGS + tb * p.num_tiles + tile;
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
      unsigned seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
      if ((int)(seen - p.epoch) >= 0) break;
      if ((it & 255u) == 255u) {
        const unsigned long long now = ar_globaltimer();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > kArTimeoutNs) {
          s_abort = 1;
          atomicCAS(reinterpret_cast<int*>(p.region + kStatusOff), 0, (int)DZ_ERR_TIMEOUT);
          break;
        }
      }
    }
  }
  __syncthreads();
  if (s_abort) return;
  const uint8_t* slots = p.region + p.push_off + (size_t)p.parity * WORLD * kPushSlotBytes;
  constexpr int kVecPerTileRow = 128 / Vec<T>::kN;         // 16-byte vectors of one row of a tile
  const int row_vec = p.N / Vec<T>::kN;
  uint4* dst = reinterpret_cast<uint4*>(p.out);
  for (int i = threadIdx.x; i < p.M * kVecPerTileRow; i += 256) {
    const int row = i / kVecPerTileRow, v = i % kVecPerTileRow;
    const size_t idx = (size_t)row * row_vec + (size_t)tile * kVecPerTileRow + v;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int r = 0; r < WORLD; ++r) {
      const uint4 x = __ldcg(reinterpret_cast<const uint4*>(slots + (size_t)r * kPushSlotBytes) + idx);
      Vec<T>::add(acc, x);
    }
    dst[idx] = Vec<T>::pack(acc);
  }
}

template <typename T>
cudaError_t launch_pushed(const PushedParams& p, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.num_tiles);
  cfg.blockDim = dim3(256);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  switch (p.world) {
    case 2: return cudaLaunchKernelEx(&cfg, allreduce_pushed_kernel<T, 2>, p);
    case 3: return cudaLaunchKernelEx(&cfg, allreduce_pushed_kernel<T, 3>, p);
    case 4: return cudaLaunchKernelEx(&cfg, allreduce_pushed_kernel<T, 4>, p);
    case 5: return cudaLaunchKernelEx(&cfg, allreduce_pushed_kernel<T, 5>, p);
    case 6: return cudaLaunchKernelEx(&cfg, allreduce_pushed_kernel<T, 6>, p);
    case 7: return cudaLaunchKernelEx(&cfg, allreduce_pushed_kernel<T, 7>, p);
    default: return cudaLaunchKernelEx(&cfg, allreduce_pushed_kernel<T, 8>, p);
  }
}

template <typename T>
cudaError_t launch_nvls(const ArParams& p, const uint8_t* mc, int blocks, cudaStream_t st) {
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
    case 2: return cudaLaunchKernelEx(&cfg, allreduce_nvls_kernel<T, 2>, p, mc);
    case 3: return cudaLaunchKernelEx(&cfg, allreduce_nvls_kernel<T, 3>, p, mc);
    case 4: return cudaLaunchKernelEx(&cfg, allreduce_nvls_kernel<T, 4>, p, mc);
    case 5: return cudaLaunchKernelEx(&cfg, allreduce_nvls_kernel<T, 5>, p, mc);
    case 6: return cudaLaunchKernelEx(&cfg, allreduce_nvls_kernel<T, 6>, p, mc);
    case 7: return cudaLaunchKernelEx(&cfg, allreduce_nvls_kernel<T, 7>, p, mc);
    default: return cudaLaunchKernelEx(&cfg, allreduce_nvls_kernel<T, 8>, p, mc);
  }
}

template <typename T>
cudaError_t launch_allreduce(const ArParams& p, int blocks, bool two_stage, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kArThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (two_stage) {
    switch (p.world) {
      case 3: return cudaLaunchKernelEx(&cfg, allreduce_twostage_kernel<T, 3>, p);
      case 4: return cudaLaunchKernelEx(&cfg, allreduce_twostage_kernel<T, 4>, p);
      case 5: return cudaLaunchKernelEx(&cfg, allreduce_twostage_kernel<T, 5>, p);
      case 6: return cudaLaunchKernelEx(&cfg, allreduce_twostage_kernel<T, 6>, p);
      case 7: return cudaLaunchKernelEx(&cfg, allreduce_twostage_kernel<T, 7>, p);
      default: return cudaLaunchKernelEx(&cfg, allreduce_twostage_kernel<T, 8>, p);
    }
  }
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
  // header and flag tables, two staging buffers, then 2 (parity) x 8 receive slots
  return kStagingOff + 2 * ((max_bytes + 255) & ~(size_t)255) + 2 * kMaxWorld * kPushSlotBytes;
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
      cudaMemset(c->region, 0, kStagingOff) != cudaSuccess) {   // status word and all flag tables
    if (c->region) cudaFree(c->region);
    delete c;
    return DZ_ERR_CUDA;
  }
  c->peers[rank] = c->region;
  c->connected = (world == 1);
  *out = c;
  return DZ_OK;
}

int dz_allreduce_create_external(dz_allreduce_ctx** out, int rank, int world, size_t max_bytes,
                                 void* const* regions, void* multicast_region) {
  if (!out || !regions || world < 1 || world > kMaxWorld || rank < 0 || rank >= world || max_bytes == 0)
    return DZ_ERR_INVALID_ARG;
  for (int r = 0; r < world; ++r)
    if (!regions[r] || ((uintptr_t)regions[r] & 255)) return DZ_ERR_ALIGNMENT;
  dz_allreduce_ctx* c = new (std::nothrow) dz_allreduce_ctx();
  if (!c) return DZ_ERR_CUDA;
  c->rank = rank;
  c->world = world;
  c->max_bytes = (max_bytes + 255) & ~(size_t)255;
  c->region_bytes = dz_allreduce_region_bytes(max_bytes);
  if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; return DZ_ERR_CUDA; }
  c->owned = false;
  for (int r = 0; r < world; ++r) c->peers[r] = reinterpret_cast<uint8_t*>(regions[r]);
  c->region = c->peers[rank];
  c->multicast = reinterpret_cast<uint8_t*>(multicast_region);
  c->connected = true;
  *out = c;
  return DZ_OK;
}

int dz_allreduce_export(dz_allreduce_ctx* c, unsigned char* handle) {
  if (!c || !handle || !c->owned) return DZ_ERR_INVALID_ARG;
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
  // One-shot for the sizes the row-parallel layers produce at decode (0.5 - 2.6 MB at 64 - 256
  // tokens), two-stage above.  The reference switches at 512 KB (up to 4 ranks) / 256 KB (up to
  // 8); measured on B200 / NVLink 5 the two extra latency-bound phases of the two-stage form
  // cost more than the traffic they save until the message reaches several MB (4 ranks,
  // 512 KB: 13 us one-shot against 33 us two-stage).  Every rank computes the same choice and
  // the same block count.
  bool two_stage = c->world > 2 && bytes >= (size_t)4 * 1024 * 1024;
  if (c->force_variant == 1) two_stage = false;
  if (c->force_variant == 2 && c->world > 2) two_stage = true;
  // in-switch reduction where the regions have a multicast mapping: forced, or by default from
  // 64 KB up on more than two ranks (below that the plain one-shot kernel is as fast)
  const bool nvls = c->multicast != nullptr && c->world > 1 &&
                    (c->force_variant == 3 ||
                     (c->force_variant == 0 && c->nvls_default && c->world > 2 && bytes >= 64 * 1024));
  if (nvls) {
    int nblocks = (int)((bytes + 8191) / 8192);
    nblocks = nblocks < 1 ? 1 : (nblocks > kMaxBlocks ? kMaxBlocks : nblocks);
    if (dtype == DZ_DTYPE_F16) DZ_CUDA_OK(launch_nvls<__half>(p, c->multicast, nblocks, st));
    else if (dtype == DZ_DTYPE_BF16) DZ_CUDA_OK(launch_nvls<__nv_bfloat16>(p, c->multicast, nblocks, st));
    else DZ_CUDA_OK(launch_nvls<float>(p, c->multicast, nblocks, st));
    return DZ_OK;
  }
  int blocks;
  if (two_stage) {
    // every block handles one sub-slice (~4 KB) of each of the `world` parts
    blocks = (int)((bytes / c->world + 4095) / 4096);
  } else {
    // one block per 8 KB (one vector per thread and rank)
    blocks = (int)((bytes + 8191) / 8192);
  }
  blocks = blocks < 1 ? 1 : (blocks > kMaxBlocks ? kMaxBlocks : blocks);
  if (dtype == DZ_DTYPE_F16) DZ_CUDA_OK(launch_allreduce<__half>(p, blocks, two_stage, st));
  else if (dtype == DZ_DTYPE_BF16) DZ_CUDA_OK(launch_allreduce<__nv_bfloat16>(p, blocks, two_stage, st));
  else DZ_CUDA_OK(launch_allreduce<float>(p, blocks, two_stage, st));
  return DZ_OK;
}

int dz_allreduce_push_target(dz_allreduce_ctx* c, int M, int N, int dtype, dz_push_target* t) {
  if (!c || !t || !c->connected) return DZ_ERR_INVALID_ARG;
  if (dtype != DZ_DTYPE_F16 && dtype != DZ_DTYPE_BF16) return DZ_ERR_UNSUPPORTED;
  if (M <= 0 || N <= 0 || N % 128) return DZ_ERR_SHAPE;
  const int tbs = (M + 127) / 128;
  if ((size_t)M * N * 2 > kPushSlotBytes || tbs * (N / 128) > DZ_PUSH_MAX_FLAGS) return DZ_ERR_TOO_LARGE;
  const size_t push_off = kStagingOff + 2 * c->max_bytes;
  const unsigned parity = c->epoch & 1u;
  memset(t, 0, sizeof(*t));
  t->world = c->world;
  t->rank = c->rank;
  t->epoch = c->epoch + 1;
  for (int r = 0; r < c->world; ++r) {
    // this rank's receive slot and flag row inside rank r's region
    t->data[r] = c->peers[r] + push_off + ((size_t)parity * c->world + c->rank) * kPushSlotBytes;
    t->flags[r] = c->peers[r] + kPushFlagsOff + (size_t)c->rank * DZ_PUSH_MAX_FLAGS * 4;
  }
  return DZ_OK;
}

int dz_allreduce_run_pushed(dz_allreduce_ctx* c, void* out, int M, int N, int dtype, void* stream) {
  if (!c || !out || !c->connected) return DZ_ERR_INVALID_ARG;
  if (dtype != DZ_DTYPE_F16 && dtype != DZ_DTYPE_BF16) return DZ_ERR_UNSUPPORTED;
  if (M <= 0 || N <= 0 || N % 128) return DZ_ERR_SHAPE;
  const int tbs = (M + 127) / 128;
  if ((size_t)M * N * 2 > kPushSlotBytes || tbs * (N / 128) > DZ_PUSH_MAX_FLAGS) return DZ_ERR_TOO_LARGE;
  if ((uintptr_t)out & 15) return DZ_ERR_ALIGNMENT;
  PushedParams p;
  p.region = c->region;
  p.out = out;
  p.M = M; p.N = N; p.world = c->world;
  p.parity = (int)(c->epoch & 1u);
  p.token_blocks = tbs;
  p.num_tiles = N / 128;
  p.epoch = ++c->epoch;
  p.push_off = kStagingOff + 2 * c->max_bytes;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == DZ_DTYPE_F16) DZ_CUDA_OK(launch_pushed<__half>(p, st));
  else DZ_CUDA_OK(launch_pushed<__nv_bfloat16>(p, st));
  return DZ_OK;
}

int dz_allreduce_set_variant(dz_allreduce_ctx* c, int variant) {
  if (!c || variant < 0 || variant > 4) return DZ_ERR_INVALID_ARG;
  if (variant == 3 && !c->multicast) return DZ_ERR_UNSUPPORTED;
  if (variant == 4) {                      // "by size, in-switch kernel allowed"
    if (!c->multicast) return DZ_ERR_UNSUPPORTED;
    c->force_variant = 0;
    c->nvls_default = true;
    return DZ_OK;
  }
  c->force_variant = variant;
  if (variant == 0) c->nvls_default = false;
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
  if (c->region && c->owned) cudaFree(c->region);
  delete c;
  return DZ_OK;
}

}  // extern "C"

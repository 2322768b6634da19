// Building blocks shared by the tcgen05 kernels of this library: mbarrier / TMA / tcgen05 PTX
// wrappers with bounded waits, shared-memory matrix descriptors, and the host-side tensor-map
// cache.  Everything here is inline; including files place their kernels in namespace dz.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>

#include "dz_common.cuh"

namespace dz {

constexpr unsigned long long kTimeoutNs = 400ull * 1000 * 1000;   // limit of every device-side wait

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait (slow path).  Returns at once when the CTA is aborting.
static __device__ __noinline__ void mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                            int* status) {
  if (*abort_flag) return;
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return;
    __nanosleep(32);   // keep polling warps out of the issue slots of working ones
    if ((it & 63u) == 63u) {
      if (*abort_flag) return;
      const unsigned long long now = globaltimer();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > kTimeoutNs) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, (int)DZ_ERR_TIMEOUT);
        return;
      }
    }
  }
}
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status) {
  if (mbar_try_wait(bar, parity)) return;
  mbar_wait_slow(bar, parity, abort_flag, status);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Instruction descriptor, kind::f16: fp16 A/B (K-major), fp32 accumulate, M = 128.
// DT: 0 = fp16, 1 = bf16 operands.
template <int DT>
__device__ __forceinline__ uint32_t make_idesc(int n, bool sparse) {
  return (sparse ? (1u << 2) : 0u) | (1u << 4) | ((uint32_t)DT << 7) | ((uint32_t)DT << 10) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
template <int DT>
__device__ __forceinline__ void store_out(void* y, size_t idx, float v, int accumulate) {
  if (DT == 0) {
    __half* o = reinterpret_cast<__half*>(y) + idx;
    if (accumulate) v += __half2float(*o);
    *o = __float2half_rn(v);
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(y) + idx;
    if (accumulate) v += __bfloat162float(*o);
    *o = __float2bfloat16_rn(v);
  }
}
// Shared-memory matrix descriptors (K-major tile, 128-byte swizzle, rows 128 B
// apart, 8-row groups 1024 B apart) are handled as (lo, hi) 32-bit halves: hi
// is the same for every such tile, lo carries the start address.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr) {
  return ((saddr >> 4) & 0x3FFFu) | (1u << 16);
}
// four dense MMAs over one 64-wide k half-tile (k advances 32 B = 2 descriptor units)
__device__ __forceinline__ void umma_ss_x4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .b64 da, db;\n\t"
      ".reg .b32 al, bl;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.eq.b32 q, %5, %5;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
      "add.u32 al, %1, 2;\n\t"
      "add.u32 bl, %2, 2;\n\t"
      "mov.b64 da, {al, %3};\n\t"
      "mov.b64 db, {bl, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, q;\n\t"
      "add.u32 al, %1, 4;\n\t"
      "add.u32 bl, %2, 4;\n\t"
      "mov.b64 da, {al, %3};\n\t"
      "mov.b64 db, {bl, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, q;\n\t"
      "add.u32 al, %1, 6;\n\t"
      "add.u32 bl, %2, 6;\n\t"
      "mov.b64 da, {al, %3};\n\t"
      "mov.b64 db, {bl, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, q;\n\t"
      "}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// two 2:4-sparse MMAs over one 64-wide k half of a window: compressed A
// (8 TMEM columns each) and metadata (one column each, addressed as the even
// column of the pair + sparsity selector) in tensor memory, B in shared memory
// (k advances 64 B = 4 descriptor units)
__device__ __forceinline__ void umma_ts_sp_x2(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                              uint32_t e_tmem, uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      ".reg .b64 db;\n\t"
      ".reg .b32 bl, a1, i1;\n\t"
      "setp.eq.b32 q, %1, %1;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.sp.cta_group::1.kind::f16 [%0], [%1], db, [%3], %4, q;\n\t"
      "add.u32 bl, %2, 4;\n\t"
      "add.u32 a1, %1, 8;\n\t"
      "or.b32 i1, %4, 1;\n\t"
      "mov.b64 db, {bl, %5};\n\t"
      "tcgen05.mma.sp.cta_group::1.kind::f16 [%0], [a1], db, [%3], i1, q;\n\t"
      "}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(e_tmem), "r"(idesc), "r"(kDescHi)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st16_zero(uint32_t taddr) {
  const uint32_t z = 0;
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr),
      "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c,
                                         uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr),
               "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// shared-memory accesses by 32-bit shared address (volatile: they keep their order relative to
// the barrier waits, which are volatile too)
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v));
}
__device__ __forceinline__ void sts128(uint32_t a, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w));
}
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}


// position and wait parity inside a ring of `size` mbarrier-guarded slots
struct Ring {
  int idx, par, size;
  __device__ __forceinline__ Ring(int size_, int par0) : idx(0), par(par0), size(size_) {}
  __device__ __forceinline__ void advance() {
    if (++idx == size) { idx = 0; par ^= 1; }
  }
};

// ---------------------------------------------------------------------------
// Host side: tensor maps
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// fp16 row-major [rows, K] matrix, box = 64 (k) x box_rows, 128-byte swizzle
inline int encode_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows, int dt) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return DZ_ERR_CUDA;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DZ_OK : DZ_ERR_CUDA;
}

// Tensor maps depend only on (pointer, rows, K, box): a small per-thread cache
// keeps the driver's encode call off the per-layer launch path.
struct MapKey {
  const void* ptr;
  int rows, K, box, dt;
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
};
inline int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows, int dt) {
  constexpr int kEntries = 1024;
  static thread_local MapEntry* cache = nullptr;
  if (!cache) cache = new MapEntry[kEntries]();
  const uintptr_t h = (reinterpret_cast<uintptr_t>(ptr) >> 8) * 0x9E3779B97F4A7C15ull;
  MapEntry& e = cache[((h >> 40) ^ (uintptr_t)box_rows) % kEntries];
  if (e.key.ptr == ptr && e.key.rows == rows && e.key.K == K && e.key.box == box_rows &&
      e.key.dt == dt) {
    *map = e.map;
    return DZ_OK;
  }
  int rc = encode_map(map, ptr, rows, K, box_rows, dt);
  if (rc == DZ_OK) {
    e.key = MapKey{ptr, rows, K, box_rows, dt};
    e.map = *map;
  }
  return rc;
}


}  // namespace dz

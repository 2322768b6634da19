// Grouped dense GEMM for layers with a full replacement matrix per delta (the output / lm_head
// matrix):  y[i] = x[i] T_{g(i)}^T, where T_g is the base matrix for tokens of slot -1 and the
// delta's own matrix for tokens of slot g.  One launch per token block serves every group that is
// present in the batch and streams each present matrix from HBM exactly once; matrices of slots
// without tokens are never touched.  Takes over apply_delta_uncompressed
// (serving/vllm/delta/deltazip_marlin.py:21-53), which loops over the distinct ids on the host.
//
// Shape of the work: "virtual tiles" (present group, 128 rows of the vocabulary) are dealt
// round-robin to one persistent CTA per SM.  The 128 rows are the MMA's M dimension, the (sorted)
// tokens of the token block its N dimension, exactly as in the SBMM kernel; the epilogue stores
// only the columns whose token belongs to the tile's group.  Three roles: a TMA producer thread
// (W tile + x half-tile per 64-wide k step into a 4-stage ring), an MMA-issuing thread (dense
// tcgen05.mma into one of two TMEM accumulators), and four epilogue warps (tcgen05.ld, mask,
// store) that drain one accumulator while the next tile fills the other.  The list of present
// groups is derived by every CTA from the batch's segment table, so no host knowledge of the
// batch is needed.  All waits are bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include "dz_common.cuh"
#include "dz_tc.cuh"

namespace dz {
namespace {

constexpr int kGStages = 4;
constexpr int kGThreads = 192;          // warp 0 producer, warp 1 MMA + TMEM owner, warps 2..5 epilogue
constexpr int kGTmemCols = 256;         // two accumulators of up to 128 columns
constexpr int kGWTile = 128 * 128;      // bytes of one W tile [128 rows x 64 k] fp16

struct GParams {
  int M, K, V, num_slots;               // V: rows of every matrix (multiple of 128)
  int row0, cols;                       // this launch: sorted rows [row0, row0 + cols)
  int xb_bytes;
  long long ldy;
  const uint8_t* seg;
  void* y;
  int* status;
};

template <int DT>
__global__ void __launch_bounds__(kGThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_base,
                    const __grid_constant__ CUtensorMap map_stack,
                    const __grid_constant__ CUtensorMap map_x, const GParams p) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t s_full[kGStages], s_empty[kGStages], s_acc_full[2], s_acc_empty[2];
  __shared__ int s_slot[kTokenBlock];
  __shared__ int s_present[kTokenBlock + 1];
  __shared__ int s_npresent, s_abort;
  __shared__ uint32_t s_tmem_base;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t sbase = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t s_w = sbase;
  const uint32_t s_x = sbase + kGStages * kGWTile;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kGStages; ++i) {
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&s_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&s_acc_full[i]), 1);
      mbar_init(smem_u32(&s_acc_empty[i]), 128);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_base) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_stack) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "n"(kGTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // everything below reads the predecessor's output (x, possibly the table)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const SegHeader* hdr = reinterpret_cast<const SegHeader*>(p.seg);
  const SegLayout lay = seg_layout(p.M, p.num_slots);
  const int* perm = reinterpret_cast<const int*>(p.seg + lay.perm);
  const int* slot_of = reinterpret_cast<const int*>(p.seg + lay.slot_of);
  const bool bad = hdr->capacity_M != p.M || hdr->num_slots != p.num_slots;
  for (int i = threadIdx.x; i < kTokenBlock; i += kGThreads) {
    const int prow = p.row0 + i;
    s_slot[i] = (!bad && prow < p.M) ? slot_of[prow] : -2;     // -2: padding column, no group
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) {
    // distinct slots of the block in sorted order (-1 first)
    int n = 0, last = -3;
    for (int i = 0; i < p.cols; ++i) {
      const int s = s_slot[i];
      if (s != -2 && s != last) { s_present[n++] = s; last = s; }
    }
    s_npresent = n;
    if (bad && blockIdx.x == 0) atomicCAS(p.status, 0, (int)DZ_ERR_INVALID_ARG);
  }
  __syncthreads();
  const int npresent = s_npresent;
  const int tiles_v = p.V / kTileN;
  const int total = npresent * tiles_v;
  const int ksteps = p.K / kBlockK;
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    if (lane == 0) {
      Ring r(kGStages, 1);
      for (int vt = blockIdx.x; vt < total; vt += gridDim.x) {
        const int g = s_present[vt / tiles_v];
        const int t = vt % tiles_v;
        const CUtensorMap* mw = g < 0 ? &map_base : &map_stack;
        const int n0 = (g < 0 ? 0 : g * p.V) + t * kTileN;
        for (int ks = 0; ks < ksteps; ++ks) {
          mbar_wait(smem_u32(&s_empty[r.idx]), r.par, abort_flag, p.status);
          const uint32_t full = smem_u32(&s_full[r.idx]);
          mbar_expect_tx(full, kGWTile + p.xb_bytes);
          tma_load_2d(s_w + r.idx * kGWTile, mw, ks * kBlockK, n0, full);
          tma_load_2d(s_x + r.idx * p.xb_bytes, &map_x, ks * kBlockK, p.row0, full);
          r.advance();
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      Ring r(kGStages, 0);
      const uint32_t idesc = make_idesc<DT>(p.cols, false);
      int it = 0;
      for (int vt = blockIdx.x; vt < total; vt += gridDim.x, ++it) {
        const int a = it & 1;
        mbar_wait(smem_u32(&s_acc_empty[a]), ((it >> 1) & 1) ^ 1, abort_flag, p.status);
        tc_fence_after();
        for (int ks = 0; ks < ksteps; ++ks) {
          mbar_wait(smem_u32(&s_full[r.idx]), r.par, abort_flag, p.status);
          tc_fence_after();
          umma_ss_x4(tmem_base + a * 128, desc_lo(s_w + r.idx * kGWTile),
                     desc_lo(s_x + r.idx * p.xb_bytes), idesc, ks > 0 ? 1u : 0u);
          umma_commit(smem_u32(&s_empty[r.idx]));
          r.advance();
        }
        umma_commit(smem_u32(&s_acc_full[a]));
      }
    }
  } else {
    const int q = warp & 3;
    const int rrow = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    int it = 0;
    for (int vt = blockIdx.x; vt < total; vt += gridDim.x, ++it) {
      const int a = it & 1;
      const int g = s_present[vt / tiles_v];
      const int t = vt % tiles_v;
      mbar_wait(smem_u32(&s_acc_full[a]), (it >> 1) & 1, abort_flag, p.status);
      tc_fence_after();
      for (int c8 = 0; c8 < p.cols; c8 += 8) {
        bool any = false;
#pragma unroll
        for (int i = 0; i < 8; ++i) any |= (s_slot[c8 + i] == g);
        if (!any) continue;                       // uniform over the warp: s_slot is shared
        uint32_t v[8];
        tmem_ld8(lane_addr + a * 128 + c8, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (s_slot[c8 + i] == g) {
            const int tok = perm[p.row0 + c8 + i];
            store_out<DT>(p.y, (size_t)tok * (size_t)p.ldy + t * kTileN + rrow, __uint_as_float(v[i]), 0);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&s_acc_empty[a]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    const unsigned long long t0 = globaltimer();
    while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "n"(kGTmemCols)
                 : "memory");
  }
}

__global__ void gather_rows_kernel2(const uint4* __restrict__ x, const uint8_t* __restrict__ seg,
                                    uint4* __restrict__ xs, int M, int row_vec) {
  const SegHeader* hdr = reinterpret_cast<const SegHeader*>(seg);
  const SegLayout lay = seg_layout(hdr->capacity_M, hdr->num_slots);
  const int* perm = reinterpret_cast<const int*>(seg + lay.perm);
  const int prow = blockIdx.x;
  if (prow >= M) return;
  const uint4* src = x + (size_t)perm[prow] * row_vec;
  uint4* dst = xs + (size_t)prow * row_vec;
  for (int i = threadIdx.x; i < row_vec; i += blockDim.x) dst[i] = src[i];
}

}  // namespace
}  // namespace dz

using namespace dz;

extern "C" {

size_t dz_grouped_gemm_workspace_bytes(int M, int K, int tokens_sorted) {
  if (M <= 0 || K <= 0) return 0;
  return 256 + (tokens_sorted ? 0 : (size_t)round_up(M, 16) * K * 2);
}

int dz_grouped_gemm(const void* x, const void* base_matrix, const void* delta_matrices,
                    int64_t matrix_stride_bytes, const void* segments, void* y, int M, int V, int K,
                    int num_slots, int dtype, int tokens_sorted, int64_t y_stride, void* workspace,
                    size_t workspace_bytes, void* stream) {
  if (M < 0) return DZ_ERR_INVALID_ARG;
  if (M == 0) return DZ_OK;
  if (!x || !base_matrix || !segments || !y || !workspace) return DZ_ERR_INVALID_ARG;
  if (V <= 0 || K <= 0 || num_slots < 0 || num_slots > kMaxSlots) return DZ_ERR_INVALID_ARG;
  if (V % kTileN || K % kBlockK) return DZ_ERR_SHAPE;
  if (num_slots > 0 && (!delta_matrices || matrix_stride_bytes != (int64_t)V * K * 2))
    return DZ_ERR_INVALID_ARG;               // the stack must be dense [slots, V, K]
  if (dtype != DZ_DTYPE_F16 && dtype != DZ_DTYPE_BF16) return DZ_ERR_INVALID_ARG;
  if (!aligned16(x) || !aligned16(base_matrix) || !aligned16(delta_matrices) || !aligned16(y) ||
      !aligned16(workspace))
    return DZ_ERR_ALIGNMENT;
  if (y_stride != 0 && (y_stride < V || (y_stride & 7))) return DZ_ERR_INVALID_ARG;
  if (workspace_bytes < dz_grouped_gemm_workspace_bytes(M, K, tokens_sorted)) return DZ_ERR_WORKSPACE;
  if ((long long)num_slots * V >= (1ll << 31)) return DZ_ERR_TOO_LARGE;

  cudaStream_t st = (cudaStream_t)stream;
  int dev = 0, sms = 0;
  DZ_CUDA_OK(cudaGetDevice(&dev));
  DZ_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  const void* xsrc = x;
  if (!tokens_sorted) {
    uint8_t* xs = ws + 256;
    gather_rows_kernel2<<<M, 128, 0, st>>>((const uint4*)x, (const uint8_t*)segments, (uint4*)xs, M, K / 8);
    DZ_CUDA_OK(cudaGetLastError());
    xsrc = xs;
  }
  const int dt = dtype == DZ_DTYPE_BF16 ? 1 : 0;
  CUtensorMap map_base, map_stack, map_x;
  int rc = make_map(&map_base, base_matrix, V, K, 128, dt);
  if (rc) return rc;
  if (num_slots > 0) rc = make_map(&map_stack, delta_matrices, num_slots * V, K, 128, dt);
  else map_stack = map_base;
  if (rc) return rc;

  GParams p;
  p.M = M; p.K = K; p.V = V; p.num_slots = num_slots;
  p.ldy = y_stride ? y_stride : V;
  p.seg = (const uint8_t*)segments;
  p.y = y;
  p.status = reinterpret_cast<int*>(ws);
  static bool attr_set[64][2] = {};
  const int num_tb = (M + kTokenBlock - 1) / kTokenBlock;
  for (int tb = 0; tb < num_tb; ++tb) {
    p.row0 = tb * kTokenBlock;
    p.cols = min(kTokenBlock, round_up(M - p.row0, 16));
    p.xb_bytes = p.cols * 128;
    rc = make_map(&map_x, xsrc, M, K, p.cols, dt);
    if (rc) return rc;
    const size_t smem = (size_t)kGStages * (kGWTile + p.xb_bytes) + 1024;
    auto kern = dt ? grouped_gemm_kernel<1> : grouped_gemm_kernel<0>;
    if (!attr_set[dev & 63][dt]) {
      DZ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 140 * 1024));
      attr_set[dev & 63][dt] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms);
    cfg.blockDim = dim3(kGThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DZ_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, map_base, map_stack, map_x, p));
  }
  return DZ_OK;
}

}  // extern "C"

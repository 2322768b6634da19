// The SBMM hot path for sm_100a:  y = x W^T + x dequant(delta_slot)^T, fused in one
// tensor-memory accumulator.
//
// Operand roles.  The 128 output features of a tile are the MMA's M dimension
// (TMEM lanes), the tokens of a token block (<= 256, sorted by slot) are its N
// dimension (TMEM columns), so a decode batch never pads M up to 128 and every
// weight byte is streamed from HBM exactly once.
//   base  : A = W tile [128 x 64] fp16 (TMA, 128B swizzle), B = x tile
//           [cols x 64] (TMA), dense tcgen05.mma, N = cols.
//   delta : the packed codes and 2:4 metadata of (slot, tile, k-unit) arrive by
//           bulk copy; four warps expand the codes to the *compressed* fp16 A
//           operand in swizzled shared memory (one row per thread, one logic op
//           + one subtract + one multiply per fp16 pair), copy the metadata
//           into tensor memory, and zero the rows of the slot's token window
//           that belong to other slots; tcgen05.mma.sp then accumulates into
//           the window's columns of the SAME accumulator the base product used.
//
// Work split.  (tile, k-unit of 128) pairs are divided evenly over one CTA per
// SM ("stream-K"): a CTA walks a contiguous unit range, which may cover the
// tail of one tile, whole tiles and the head of another.  A fragment that does
// not cover a whole tile parks its fp32 partial in the workspace; the last
// fragment of a tile to finish (a per-tile counter) adds the partials in fixed
// order, so results do not depend on timing.
//
// Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, then four
// warpgroups of 128 threads that expand codes (delta stage s goes to warpgroup
// s mod 4, so several stages are expanded at once and each scheduler has four
// warps to hide latency with) and share the epilogue by column chunks.
// Every mbarrier wait is bounded: on a timeout the CTA records DZ_ERR_TIMEOUT,
// raises an abort flag that turns every later wait into a no-op, runs its
// (bounded) loops to the end and frees its tensor memory.
#include <cuda.h>

#include <stdlib.h>

#include <mutex>
#include <unordered_map>

#include "dz_common.cuh"

namespace dz {

namespace {

constexpr int kNumWG = 4;                      // code-expansion warpgroups (128 threads each)
constexpr int kThreads = 64 + 128 * kNumWG;
constexpr int kUnitK = 128;                    // dense k per work unit
constexpr int kATile = 128 * 128;              // bytes: 128 rows x 128 B
constexpr int kNumABuf = kNumWG;               // expanded-A buffers, one per warpgroup
constexpr int kDeltaStages = 6;                // upper bound; Params::delta_stages are used
constexpr int kRawBytes = 4096;                // codes of one unit (4-bit)
constexpr int kMetaBytes = 2048;               // metadata of one unit
constexpr int kWinBytes = 2 * kMaxWindowCols * 128;
constexpr int kDeltaStageBytes = kRawBytes + kMetaBytes + kWinBytes;
constexpr int kBaseRingBytes = 72 * 1024;
constexpr int kMaxWin = 256;                   // windows of one token block
constexpr int kTmemCols = 512;
constexpr int kMetaCol = 256;                  // first TMEM column of the metadata buffers
constexpr unsigned long long kTimeoutNs = 400ull * 1000 * 1000;
constexpr int kMaxCtas = 160;

static_assert(kDeltaStageBytes % 1024 == 0, "stage regions stay 1024-byte aligned");

struct Params {
  int M, N, K, bits;
  int num_kunits, num_tiles, num_kblocks;
  int token_block, row0, cols;     // this launch: sorted rows [row0, row0 + cols)
  int base_only, tokens_sorted;
  int debug;   // experiment switches (bit 0: skip code expansion, bit 1: skip window zeroing)
  int grid, total_units;
  int base_stages, delta_stages, xb_bytes;
  const uint8_t* qweight;
  const uint8_t* meta;
  const uint8_t* scales;
  long long qstride, mstride, sstride;
  const uint8_t* seg;
  __half* y;
  float* partials;
  int* counters;
  int* status;
};

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
// Bounded wait.  Returns at once when the CTA is aborting.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status) {
  if (*abort_flag) return;
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return;
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
// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128 B
// apart, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)1 << 16;             // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset
  d |= (uint64_t)1 << 46;             // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;             // SWIZZLE_128B
  return d;
}
// Instruction descriptor, kind::f16: fp16 A/B (K-major), fp32 accumulate, M = 128.
__device__ __forceinline__ uint32_t make_idesc(int n, bool sparse) {
  return (sparse ? (1u << 2) : 0u) | (1u << 4) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ss_sp(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                           uint32_t e_tmem, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.sp.cta_group::1.kind::f16 [%0], %1, %2, [%3], %4, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c,
                                         uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr),
               "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// (v >> shift) & mask | 0x64006400, i.e. the fp16 pair (1024 + code_lo, 1024 + code_hi)
template <uint32_t MASK>
__device__ __forceinline__ uint32_t extract_pair(uint32_t w, int shift) {
  uint32_t r;
  const uint32_t s = w >> shift;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(s), "n"(MASK), "n"(0x64006400));
  return r;
}

struct Fragment {
  int tile, ku0, ku1;
};

// CTA that owns unit u when `total` units are split evenly over `grid` CTAs
// (CTA c owns [c*total/grid, (c+1)*total/grid)).
__device__ __forceinline__ int cta_of_unit(long long u, int grid, int total) {
  return (int)(((u + 1) * grid - 1) / total);
}

struct WinS {
  int slot, col0, ncols, lohi;  // col0 relative to the token block; lohi = lo | hi << 16 (relative)
};

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
template <int BITS>
__global__ void __launch_bounds__(kThreads, 1)
sbmm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const __grid_constant__ CUtensorMap map_x32,
               const __grid_constant__ CUtensorMap map_xc, const Params p) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t s_bars[4 + 4 + 2 * kDeltaStages + 2 * kNumABuf + 2];
  __shared__ WinS s_win[kMaxWin];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort, s_last;

  // ---- early uniform exits (before any barrier or TMEM state exists) ----
  int nwin = 0, win_begin = 0;
  const int* perm = nullptr;
  const Window* gwin = nullptr;
  if (p.seg) {
    const SegHeader* hdr = reinterpret_cast<const SegHeader*>(p.seg);
    if (p.tokens_sorted && !hdr->sorted) {
      if (threadIdx.x == 0 && blockIdx.x == 0) atomicCAS(p.status, 0, (int)DZ_ERR_INVALID_ARG);
      return;
    }
    const SegLayout lay = seg_layout(hdr->capacity_M, hdr->num_slots);
    perm = reinterpret_cast<const int*>(p.seg + lay.perm);
    if (!p.base_only) {
      const int* bb = reinterpret_cast<const int*>(p.seg + lay.block_begin);
      win_begin = bb[p.token_block];
      nwin = min(bb[p.token_block + 1] - win_begin, kMaxWin);
      gwin = reinterpret_cast<const Window*>(p.seg + lay.windows) + win_begin;
    }
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- shared memory carve-up (1024-byte aligned regions) ----
  const uint32_t dyn0 = smem_u32(smem_dyn);
  const uint32_t sbase = (dyn0 + 1023u) & ~1023u;
  uint8_t* const sgen = smem_dyn + (sbase - dyn0);
  const int base_stage_bytes = kATile + p.xb_bytes;
  const uint32_t s_base_ring = sbase;
  const uint32_t s_delta_ring = s_base_ring + p.base_stages * base_stage_bytes;
  const uint32_t s_abuf = s_delta_ring + p.delta_stages * kDeltaStageBytes;
  uint8_t* const g_delta_ring = sgen + p.base_stages * base_stage_bytes;
  uint8_t* const g_abuf = g_delta_ring + p.delta_stages * kDeltaStageBytes;

  uint64_t* bar_base_full = s_bars;
  uint64_t* bar_base_empty = s_bars + 4;
  uint64_t* bar_d_full = s_bars + 8;
  uint64_t* bar_d_empty = bar_d_full + kDeltaStages;
  uint64_t* bar_a_ready = bar_d_empty + kDeltaStages;
  uint64_t* bar_a_free = bar_a_ready + kNumABuf;
  uint64_t* bar_acc_full = bar_a_free + kNumABuf;
  uint64_t* bar_acc_empty = bar_acc_full + 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&bar_base_full[i]), 1);
      mbar_init(smem_u32(&bar_base_empty[i]), 1);
    }
    for (int i = 0; i < kDeltaStages; ++i) {
      mbar_init(smem_u32(&bar_d_full[i]), 1);
      mbar_init(smem_u32(&bar_d_empty[i]), 1);
    }
    for (int i = 0; i < kNumABuf; ++i) {
      mbar_init(smem_u32(&bar_a_ready[i]), 128);
      mbar_init(smem_u32(&bar_a_free[i]), 1);
    }
    mbar_init(smem_u32(bar_acc_full), 1);
    mbar_init(smem_u32(bar_acc_empty), 128 * kNumWG);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x32) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_xc) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "n"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  for (int i = threadIdx.x; i < nwin; i += kThreads) {
    const Window w = gwin[i];
    WinS ws;
    ws.slot = w.slot;
    ws.col0 = w.col0 - p.row0;
    ws.ncols = w.ncols;
    ws.lohi = (w.lo - w.col0) | ((w.hi - w.col0) << 16);
    s_win[i] = ws;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  // ---- this CTA's unit range ----
  const int cta = blockIdx.x;
  const long long U = p.total_units;
  const int u_begin = (int)((long long)cta * U / p.grid);
  const int u_end = (int)((long long)(cta + 1) * U / p.grid);
  const int KU = p.num_kunits;

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      int sb = 0, pb = 1, sd = 0, pd = 1;
      for (int u = u_begin; u < u_end;) {
        const int tile = u / KU, ku0 = u % KU;
        const int ku1 = min(KU, ku0 + (u_end - u));
        const int n0 = tile * kTileN;
        for (int ku = ku0; ku < ku1; ++ku) {
          const int k0 = ku * kUnitK;
          const int nhalf = min(2, (p.K - k0) / kBlockK);
          for (int h = 0; h < nhalf; ++h) {
            mbar_wait(smem_u32(&bar_base_empty[sb]), pb, abort_flag, p.status);
            const uint32_t full = smem_u32(&bar_base_full[sb]);
            mbar_expect_tx(full, kATile + p.xb_bytes);
            const uint32_t dstA = s_base_ring + sb * base_stage_bytes;
            tma_load_2d(dstA, &map_w, k0 + h * kBlockK, n0, full);
            tma_load_2d(dstA + kATile, &map_xc, k0 + h * kBlockK, p.row0, full);
            if (++sb == p.base_stages) { sb = 0; pb ^= 1; }
          }
          for (int w = 0; w < nwin; ++w) {
            const WinS ws = s_win[w];
            mbar_wait(smem_u32(&bar_d_empty[sd]), pd, abort_flag, p.status);
            const uint32_t full = smem_u32(&bar_d_full[sd]);
            const uint32_t code_bytes = nhalf * codes_block_bytes(BITS);
            const uint32_t meta_bytes = nhalf * kMetaBlockBytes;
            const uint32_t win_bytes = nhalf * ws.ncols * 128;
            mbar_expect_tx(full, code_bytes + meta_bytes + win_bytes);
            const size_t blk = (size_t)tile * p.num_kblocks + (size_t)ku * 2;
            const uint32_t dst = s_delta_ring + sd * kDeltaStageBytes;
            bulk_load(dst, p.qweight + (size_t)ws.slot * p.qstride + blk * codes_block_bytes(BITS),
                      code_bytes, full);
            bulk_load(dst + kRawBytes, p.meta + (size_t)ws.slot * p.mstride + blk * kMetaBlockBytes,
                      meta_bytes, full);
            for (int h = 0; h < nhalf; ++h)
              tma_load_2d(dst + kRawBytes + kMetaBytes + h * ws.ncols * 128,
                          ws.ncols == 16 ? &map_x : &map_x32, k0 + h * kBlockK,
                          p.row0 + ws.col0, full);
            if (++sd == p.delta_stages) { sd = 0; pd ^= 1; }
          }
        }
        u += ku1 - ku0;
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      int sb = 0, pb = 0, sd = 0, pdm = 0, ab = 0, pa = 0, pacc = 1;
      const uint32_t idesc_base = make_idesc(p.cols, false);
      for (int u = u_begin; u < u_end;) {
        const int ku0 = u % KU;
        const int ku1 = min(KU, ku0 + (u_end - u));
        mbar_wait(smem_u32(bar_acc_empty), pacc, abort_flag, p.status);
        pacc ^= 1;
        tc_fence_after();
        uint32_t acc = 0;
        for (int ku = ku0; ku < ku1; ++ku) {
          const int k0 = ku * kUnitK;
          const int nhalf = min(2, (p.K - k0) / kBlockK);
          for (int h = 0; h < nhalf; ++h) {
            mbar_wait(smem_u32(&bar_base_full[sb]), pb, abort_flag, p.status);
            tc_fence_after();
            const uint32_t a0 = s_base_ring + sb * base_stage_bytes;
            const uint64_t adesc = make_desc(a0);
            const uint64_t bdesc = make_desc(a0 + kATile);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              umma_ss(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc_base, acc);
              acc = 1;
            }
            umma_commit(smem_u32(&bar_base_empty[sb]));
            if (++sb == p.base_stages) { sb = 0; pb ^= 1; }
          }
          for (int w = 0; w < nwin; ++w) {
            const WinS ws = s_win[w];
            mbar_wait(smem_u32(&bar_d_full[sd]), pdm, abort_flag, p.status);
            mbar_wait(smem_u32(&bar_a_ready[ab]), pa, abort_flag, p.status);
            tc_fence_after();
            const uint64_t adesc = make_desc(s_abuf + ab * kATile);
            const uint32_t winb = s_delta_ring + sd * kDeltaStageBytes + kRawBytes + kMetaBytes;
            const uint32_t idesc = make_idesc(ws.ncols, true);
            const uint32_t dcol = tmem_base + ws.col0;
            const uint32_t ecol = tmem_base + kMetaCol + ab * 4;
            for (int j = 0; j < nhalf * 2; ++j) {
              const uint64_t bdesc = make_desc(winb + (j >> 1) * ws.ncols * 128) + 4 * (j & 1);
              // metadata of MMA j sits in column j of the buffer; the instruction
              // takes the even column of the pair and selects inside it with the
              // descriptor's sparsity-selector bits
              umma_ss_sp(dcol, adesc + 2 * j, bdesc, ecol + (j & ~1), idesc | (uint32_t)(j & 1), 1u);
            }
            umma_commit(smem_u32(&bar_a_free[ab]));
            umma_commit(smem_u32(&bar_d_empty[sd]));
            if (++ab == kNumABuf) { ab = 0; pa ^= 1; }
            if (++sd == p.delta_stages) { sd = 0; pdm ^= 1; }
          }
        }
        umma_commit(smem_u32(bar_acc_full));
        u += ku1 - ku0;
      }
    }
  } else {
    // ================= code expansion + epilogue (warps 2..) =================
    const int q = warp & 3;              // TMEM lane quarter this warp may touch
    const int r = q * 32 + lane;         // tile row == TMEM lane
    const int wg = (warp - 2) >> 2;      // warpgroup index
    const int wg_tid = (threadIdx.x - 64) & 127;
    const int ep_tid = threadIdx.x - 64;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const int ab = wg;                   // this warpgroup's expanded-A buffer
    int sd = 0, pd = 0, pa = 1, pacc = 0, seq = 0;
    bool cta_first_fragment = true;
    const __half2 kBias = __half2half2(__ushort_as_half((unsigned short)(BITS == 4 ? 0x6408 : 0x6402)));

    for (int u = u_begin; u < u_end;) {
      const int tile = u / KU, ku0 = u % KU;
      const int ku1 = min(KU, ku0 + (u_end - u));
      const int n0 = tile * kTileN;
      for (int ku = ku0; ku < ku1; ++ku) {
        const int k0 = ku * kUnitK;
        const int nhalf = min(2, (p.K - k0) / kBlockK);
        for (int w = 0; w < nwin; ++w) {
          if ((seq++ % kNumWG) != wg) {  // another warpgroup's stage
            // Still observe its "full" phase: a parity wait can only tell the
            // current phase from the previous one, so every consumer has to see
            // every phase of a ring slot in order.
            mbar_wait(smem_u32(&bar_d_full[sd]), pd, abort_flag, p.status);
            if (++sd == p.delta_stages) { sd = 0; pd ^= 1; }
            continue;
          }
          const WinS ws = s_win[w];
          const __half sc = *reinterpret_cast<const __half*>(p.scales + (size_t)ws.slot * p.sstride +
                                                             (size_t)(n0 + r) * 2);
          const __half2 sc2 = __half2half2(sc);
          mbar_wait(smem_u32(&bar_d_full[sd]), pd, abort_flag, p.status);
          mbar_wait(smem_u32(&bar_a_free[ab]), pa, abort_flag, p.status);
          const uint8_t* raw = g_delta_ring + sd * kDeltaStageBytes;
          uint8_t* arow = g_abuf + ab * kATile + r * 128;
          uint32_t mw[4] = {0, 0, 0, 0};
          for (int h = 0; h < ((p.debug & 1) ? 0 : nhalf); ++h) {
            if (BITS == 4) {
              const uint4 cw = *reinterpret_cast<const uint4*>(raw + h * 2048 + r * 16);
              const uint32_t wv[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
              for (int wi = 0; wi < 4; ++wi) {
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint32_t t = extract_pair<0x000f000fu>(wv[wi], 4 * j);
                  __half2 hv = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t), kBias), sc2);
                  o[j] = *reinterpret_cast<uint32_t*>(&hv);
                }
                const int c = h * 4 + wi;
                *reinterpret_cast<uint4*>(arow + ((c ^ (r & 7)) << 4)) =
                    make_uint4(o[0], o[1], o[2], o[3]);
              }
            } else {
              const uint2 cw = *reinterpret_cast<const uint2*>(raw + h * 1024 + r * 8);
              const uint32_t wv[2] = {cw.x, cw.y};
#pragma unroll
              for (int wi = 0; wi < 2; ++wi) {
#pragma unroll
                for (int half8 = 0; half8 < 2; ++half8) {
                  uint32_t o[4];
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    uint32_t t = extract_pair<0x00030003u>(wv[wi], 2 * (half8 * 4 + j));
                    __half2 hv = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t), kBias), sc2);
                    o[j] = *reinterpret_cast<uint32_t*>(&hv);
                  }
                  const int c = h * 4 + wi * 2 + half8;
                  *reinterpret_cast<uint4*>(arow + ((c ^ (r & 7)) << 4)) =
                      make_uint4(o[0], o[1], o[2], o[3]);
                }
              }
            }
            const uint2 m2 = *reinterpret_cast<const uint2*>(raw + kRawBytes + h * 1024 + r * 8);
            mw[h * 2] = m2.x;
            mw[h * 2 + 1] = m2.y;
          }
          tmem_st4(lane_addr + kMetaCol + ab * 4, mw[0], mw[1], mw[2], mw[3]);
          // zero the window rows that belong to other slots
          {
            const int lo = ws.lohi & 0xFFFF, hi = ws.lohi >> 16;
            uint8_t* winb = const_cast<uint8_t*>(raw) + kRawBytes + kMetaBytes;
            const int total = (p.debug & 2) ? 0 : nhalf * ws.ncols * 8;
            for (int idx = wg_tid; idx < total; idx += 128) {
              const int row = (idx >> 3) % ws.ncols;
              if (row < lo || row >= hi)
                *reinterpret_cast<uint4*>(winb + (size_t)idx * 16) = make_uint4(0, 0, 0, 0);
            }
          }
          fence_proxy_async();
          tc_fence_before();
          mbar_arrive(smem_u32(&bar_a_ready[ab]));
          pa ^= 1;
          if (++sd == p.delta_stages) { sd = 0; pd ^= 1; }
        }
      }

      // ---------------- epilogue of this fragment ----------------
      mbar_wait(smem_u32(bar_acc_full), pacc, abort_flag, p.status);
      pacc ^= 1;
      tc_fence_after();
      const bool full_tile = (ku0 == 0 && ku1 == KU);
      float* my_partial = p.partials +
                          ((size_t)cta * 2 + (cta_first_fragment ? 0 : 1)) * ((size_t)p.cols * 128);
      for (int c = wg; c < p.cols / 16; c += kNumWG) {
        uint32_t v[16];
        tmem_ld16(lane_addr + c * 16, v);
        if (full_tile) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int prow = p.row0 + c * 16 + i;
            if (prow < p.M) {
              const int tok = perm ? perm[prow] : prow;
              p.y[(size_t)tok * p.N + n0 + r] = __float2half_rn(__uint_as_float(v[i]));
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            __stcg(my_partial + (size_t)(c * 16 + i) * 128 + r, __uint_as_float(v[i]));
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(bar_acc_empty));

      if (!full_tile) {
        // fragments of this tile, in CTA order
        const int c_first = cta_of_unit((long long)tile * KU, p.grid, p.total_units);
        const int c_last = cta_of_unit((long long)(tile + 1) * KU - 1, p.grid, p.total_units);
        const int nfrag = c_last - c_first + 1;
        __threadfence();
        named_bar_sync(1, 128 * kNumWG);
        if (ep_tid == 0) {
          const int old = atomicAdd(&p.counters[tile], 1);
          s_last = (old == nfrag - 1) ? 1 : 0;
        }
        named_bar_sync(1, 128 * kNumWG);
        if (s_last) {
          __threadfence();
          // 8 columns per pass so that eight independent L2 loads are in flight
          // per fragment (a column-at-a-time loop is a chain of L2 latencies)
          for (int cb = wg * 8; cb < p.cols; cb += kNumWG * 8) {
            float sum[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) sum[i] = 0.f;
            for (int f = 0; f < nfrag; ++f) {
              const int cc = c_first + f;
              const int cu0 = (int)((long long)cc * U / p.grid);
              const int slot = cc * 2 + ((cu0 / KU) == tile ? 0 : 1);
              const float* src = p.partials + (size_t)slot * ((size_t)p.cols * 128) + (size_t)cb * 128 + r;
#pragma unroll
              for (int i = 0; i < 8; ++i) sum[i] += __ldcg(src + i * 128);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int prow = p.row0 + cb + i;
              if (prow < p.M) {
                const int tok = perm ? perm[prow] : prow;
                p.y[(size_t)tok * p.N + n0 + r] = __float2half_rn(sum[i]);
              }
            }
          }
          if (ep_tid == 0) p.counters[tile] = 0;
        }
        named_bar_sync(1, 128 * kNumWG);
      }
      cta_first_fragment = false;
      u += ku1 - ku0;
    }
  }

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    // give copies still in flight a bounded time to land before the CTA's
    // shared memory is released
    const unsigned long long t0 = globaltimer();
    while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "n"(kTmemCols)
                 : "memory");
  }
}

// gathers x rows into sorted order: xs[p] = x[perm[p]]
__global__ void gather_rows_kernel(const uint4* __restrict__ x, const uint8_t* __restrict__ seg,
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

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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
int encode_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return DZ_ERR_CUDA;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DZ_OK : DZ_ERR_CUDA;
}

// Tensor maps depend only on (pointer, rows, K, box): a small per-thread cache
// keeps the driver's encode call off the per-layer launch path.
struct MapKey {
  const void* ptr;
  int rows, K, box;
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
};
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
  constexpr int kEntries = 1024;
  static thread_local MapEntry* cache = nullptr;
  if (!cache) cache = new MapEntry[kEntries]();
  const uintptr_t h = (reinterpret_cast<uintptr_t>(ptr) >> 8) * 0x9E3779B97F4A7C15ull;
  MapEntry& e = cache[(h >> 40) % kEntries ^ (box_rows & 7)];
  if (e.key.ptr == ptr && e.key.rows == rows && e.key.K == K && e.key.box == box_rows) {
    *map = e.map;
    return DZ_OK;
  }
  int rc = encode_map(map, ptr, rows, K, box_rows);
  if (rc == DZ_OK) {
    e.key = MapKey{ptr, rows, K, box_rows};
    e.map = *map;
  }
  return rc;
}

struct DeviceInfo {
  int sms = 0;
  bool attr_set[2] = {false, false};
};
DeviceInfo& device_info(int dev) {
  static DeviceInfo info[64];
  return info[dev & 63];
}

constexpr size_t kWsStatus = 0;
constexpr size_t kWsCounters = 256;
constexpr size_t kWsCountersBytes = 16384;
constexpr size_t kWsPartials = kWsCounters + kWsCountersBytes;

inline size_t partial_bytes(int M) {
  const int cols = min(kTokenBlock, round_up(M, 16));
  return (size_t)kMaxCtas * 2 * cols * 128 * sizeof(float);
}

}  // namespace

size_t sbmm_workspace_bytes(int M, int N, int K, int tokens_sorted) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  size_t b = kWsPartials + partial_bytes(M);
  if (!tokens_sorted) b += (size_t)round_up(M, 16) * K * 2 + 1024;
  return b;
}

int launch_sbmm(const dz_sbmm_args& a, bool base_only, cudaStream_t st) {
  int dev = 0;
  DZ_CUDA_OK(cudaGetDevice(&dev));
  DeviceInfo& di = device_info(dev);
  if (di.sms == 0) DZ_CUDA_OK(cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev));
  if (a.N / kTileN > (int)(kWsCountersBytes / 4)) return DZ_ERR_TOO_LARGE;

  uint8_t* ws = reinterpret_cast<uint8_t*>(a.workspace);
  const bool sorted = base_only || a.tokens_sorted != 0;
  const void* xsrc = a.x;
  if (!sorted) {
    uint8_t* xs = ws + ((kWsPartials + partial_bytes(a.M) + 1023) & ~(size_t)1023);
    gather_rows_kernel<<<a.M, 128, 0, st>>>((const uint4*)a.x, (const uint8_t*)a.segments,
                                             (uint4*)xs, a.M, a.K / 8);
    DZ_CUDA_OK(cudaGetLastError());
    xsrc = xs;
  }

  CUtensorMap map_w, map_x, map_x32, map_xc;
  int rc = make_map(&map_w, a.w_base, a.N, a.K, 128);
  if (rc) return rc;
  rc = make_map(&map_x, xsrc, a.M, a.K, 16);
  if (rc) return rc;
  rc = make_map(&map_x32, xsrc, a.M, a.K, 32);
  if (rc) return rc;

  Params p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.bits = a.bits;
  p.num_kblocks = a.K / kBlockK;
  p.num_kunits = (a.K + kUnitK - 1) / kUnitK;
  p.num_tiles = a.N / kTileN;
  p.base_only = base_only ? 1 : 0;
  { const char* e = getenv("DZ_DEBUG"); p.debug = e ? atoi(e) : 0; }
  p.tokens_sorted = sorted ? 1 : 0;
  p.total_units = p.num_tiles * p.num_kunits;
  p.grid = min(min(di.sms, kMaxCtas), p.total_units);
  p.qweight = (const uint8_t*)a.qweight;
  p.meta = (const uint8_t*)a.meta;
  p.scales = (const uint8_t*)a.scales;
  p.qstride = a.qweight_stride; p.mstride = a.meta_stride; p.sstride = a.scales_stride;
  p.seg = base_only ? nullptr : (const uint8_t*)a.segments;
  p.y = (__half*)a.y;
  p.status = reinterpret_cast<int*>(ws + kWsStatus);
  p.counters = reinterpret_cast<int*>(ws + kWsCounters);
  p.partials = reinterpret_cast<float*>(ws + kWsPartials);

  const int bits_idx = (a.bits == 2) ? 0 : 1;
  const int num_tb = (a.M + kTokenBlock - 1) / kTokenBlock;
  for (int tb = 0; tb < num_tb; ++tb) {
    p.token_block = tb;
    p.row0 = tb * kTokenBlock;
    p.cols = min(kTokenBlock, round_up(a.M - p.row0, 16));
    p.xb_bytes = p.cols * 128;
    p.base_stages = max(2, min(4, kBaseRingBytes / (kATile + p.xb_bytes)));
    p.delta_stages = p.cols <= 64 ? 5 : (p.cols <= 128 ? 4 : 3);
    rc = make_map(&map_xc, xsrc, a.M, a.K, p.cols);
    if (rc) return rc;
    const size_t smem = (size_t)p.base_stages * (kATile + p.xb_bytes) +
                        (size_t)p.delta_stages * kDeltaStageBytes + (size_t)kNumABuf * kATile + 1024;
    auto kern = (a.bits == 2) ? sbmm_tc_kernel<2> : sbmm_tc_kernel<4>;
    if (!di.attr_set[bits_idx]) {
      DZ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 222 * 1024));
      di.attr_set[bits_idx] = true;
    }
    kern<<<p.grid, kThreads, smem, st>>>(map_w, map_x, map_x32, map_xc, p);
    DZ_CUDA_OK(cudaGetLastError());
  }
  return DZ_OK;
}

}  // namespace dz

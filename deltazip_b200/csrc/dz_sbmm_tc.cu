// The SBMM hot path for sm_100a:  y = x W^T + x dequant(delta_slot)^T, base and
// delta products accumulated side by side in tensor memory and added in the
// epilogue -- no dense delta and no separate add kernel ever exist.
//
// Operand roles.  The 128 output features of a tile are the MMA's M dimension
// (TMEM lanes), the tokens of a token block (<= 128, sorted by slot) are its N
// dimension (TMEM columns), so a decode batch never pads M up to 128 and every
// weight byte is streamed from HBM exactly once.
//   base  : A = W tile [128 x 64] fp16 (TMA, 128B swizzle), B = x half-tile
//           [cols x 64] (TMA), dense tcgen05.mma (SS), N = cols, into D_base.
//   delta : the packed codes and 2:4 metadata of (slot, tile, k-unit) arrive by
//           bulk copy; a warpgroup expands the codes to the *compressed* fp16 A
//           operand directly into tensor memory (one row per thread, one logic
//           op + one subtract per fp16 pair, tcgen05.st; the per-channel scale
//           is applied to the accumulated sums in the epilogue), stores
//           the metadata next to it, and copies the slot's token window out of
//           the resident x tile with the rows of other slots zeroed;
//           tcgen05.mma.sp (A and metadata in TMEM, B in shared memory) then
//           accumulates into the window's columns of D_delta.
//
// Issue parallelism.  One thread can issue a tcgen05.mma only every ~150-200
// cycles whatever its size, and a decode batch makes many small MMAs (N = 16 or
// 32 tokens per slot).  The windows of a token block are therefore dealt to C
// "classes" (window w -> class w mod C), each with its own expansion
// warpgroup, its own MMA-issuing thread, two expanded-A buffers and its own
// sub-ring of packed stages; a further thread issues the base MMAs.  A column
// of D_delta receives non-zero products from one window only (the rows of all
// other windows over that column are zero), and that window always belongs to
// the same class, so the summation order of every output is fixed no matter how
// the issuers interleave.
//
// Work split.  (tile, k-unit of 128) pairs are divided over one CTA per SM
// ("stream-K", with a tile's epilogue counted as two more units): a CTA walks a
// contiguous unit range, which may cover the tail of one tile, whole tiles and
// the head of another.  The fragments of a split tile settle it through two
// per-tile counters: each claims a ticket; all but the holder of the last
// ticket park their fp32 partial in the workspace; the last holder adds the
// parked partials and its own accumulators in CTA order, so results do not
// depend on timing.
//
// Every mbarrier wait is bounded: on a timeout the CTA records DZ_ERR_TIMEOUT,
// raises an abort flag that turns every later wait into a no-op, runs its
// (bounded) loops to the end and frees its tensor memory.  Each barrier has a
// single, in-order waiter per phase sequence (a parity wait cannot tell phase n
// from phase n + 2).
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdlib.h>

#include <mutex>

#include "dz_common.cuh"
#include "dz_tc.cuh"

namespace dz {

namespace {

constexpr int kNumWG = 4;                      // warpgroups (128 threads each)
constexpr int kWarpWX = 0;                     // TMA producer: W tiles, x half-tiles
constexpr int kWarpBase = 1;                   // base MMA issuer, TMEM owner
constexpr int kWarpR = 2;                      // bulk-copy producer: packed delta stages
// Role layout (overridable at compile time for experiments):
//   DZ_ISSUER_WARPS  delta MMA issuer warps (one issuing thread each) starting at warp 3; with
//                    2 * classes <= DZ_ISSUER_WARPS every class has two issuers
//   DZ_FIRST_WG_WARP first of the 16 expansion / epilogue warps
//   DZ_SVC_REGS / DZ_EXP_REGS  when non-zero the service warps (below DZ_FIRST_WG_WARP, which must
//                    then be a multiple of 4) shrink to DZ_SVC_REGS registers per thread and the
//                    expansion warps grow to DZ_EXP_REGS (setmaxnreg)
#ifndef DZ_ISSUER_WARPS
#define DZ_ISSUER_WARPS 4
#endif
#ifndef DZ_FIRST_WG_WARP
#define DZ_FIRST_WG_WARP (3 + DZ_ISSUER_WARPS)
#endif
#ifndef DZ_SVC_REGS
#define DZ_SVC_REGS 0
#define DZ_EXP_REGS 0
#endif
constexpr int kWarpIssuer0 = 3;
constexpr int kIssuerWarps = DZ_ISSUER_WARPS;
constexpr int kFirstWGWarp = DZ_FIRST_WG_WARP;   // any 4 consecutive warps cover the 4 TMEM lane quarters
constexpr int kServiceRegs = DZ_SVC_REGS, kExpandRegs = DZ_EXP_REGS;
static_assert(kWarpIssuer0 + kIssuerWarps <= kFirstWGWarp, "role layout");
static_assert(kServiceRegs == 0 || kFirstWGWarp % 4 == 0, "setmaxnreg works on whole warpgroups");
static_assert((kFirstWGWarp * kServiceRegs + 4 * kNumWG * kExpandRegs) * 32 <= 65536, "register file");
constexpr int kThreads = 32 * kFirstWGWarp + 128 * kNumWG;
constexpr int kUnitK = 128;                    // dense k per work unit
constexpr int kWTile = 128 * 128;              // bytes: 128 rows x 128 B
constexpr int kMetaBytes = 2048;               // metadata of one unit
// codes of one unit: 128 rows x 64 kept values x bits; a packed stage = codes, then metadata
__host__ __device__ constexpr int raw_bytes(int bits) { return 128 * 64 * bits / 8; }
__host__ __device__ constexpr int rstage_bytes(int bits) { return raw_bytes(bits) + kMetaBytes; }
#ifndef DZ_MAX_R_PER_CLASS
#define DZ_MAX_R_PER_CLASS 6
#endif
// Ring depths for token blocks wider than 64 columns, in half-tiles.  The x ring must hold two
// whole k-units: with three half-tiles the second half of the next unit could only be requested
// once every class had finished the current one, and its latency showed in every unit (measured:
// 4 + 2 is 9-13 % faster than 3 + 3 on 128-token batches; a W stage is free again as soon as the
// base MMA has read it, so two suffice).
#ifndef DZ_W_STAGES_WIDE
#define DZ_W_STAGES_WIDE 2
#endif
#ifndef DZ_X_STAGES_WIDE
#define DZ_X_STAGES_WIDE 4
#endif
constexpr int kWinBytes = 2 * kMaxWindowCols * 128;   // window buffer (B operand of one stage)
constexpr int kMaxW = 4, kMaxX = 4, kMaxR = 24, kMaxBuf = 8;
constexpr int kMaxWin = 128;                   // windows of one token block
constexpr int kTmemCols = 512;
constexpr int kSmemBudget = 216 * 1024;
constexpr int kEpilogueUnits = 2;               // cost of a tile's epilogue in k-units (work split)
constexpr int kPrefetchTiles = 8;               // W half-tiles prefetched to L2 in the prologue
// Per-CTA wall-clock marks (8 x u64 per CTA in the upper part of the counter region) are
// compiled in only with -DDZ_INSTRUMENT; the shipped kernel carries none.
#ifdef DZ_INSTRUMENT
constexpr bool kInstr = true;
#else
constexpr bool kInstr = false;
#endif

// TMEM columns: D_base [0, dcols), D_delta [dcols, 2 dcols), then 32 columns of
// expanded A per buffer, then 4 columns of metadata per buffer.
//   dcols = 64  : 4 classes, 8 buffers -> 128 + 256 + 32 = 416 columns
//   dcols = 128 : 3 classes, 6 buffers -> 256 + 192 + 24 = 472 columns

struct Params {
  int M, N, K, bits, num_slots;
  int num_kunits, num_tiles, num_kblocks;
  int token_block, row0, cols;     // this launch: sorted rows [row0, row0 + cols)
  int base_only, delta_only, tokens_sorted;   // delta_only: no base product (w_base absent)
  int accumulate;                             // y += result
  int stable;                                 // weights, slots and table are not the predecessor's output
  long long ldy;                              // elements between rows of y
  int grid, total_units, epi_units;   // total_units counts virtual units
  int w_stages, x_stages, r_per_class, xb_bytes;
  int nclass, dcols;
  const uint8_t* qweight;
  const uint8_t* meta;
  const uint8_t* scales;
  long long qstride, mstride, sstride;
  const uint8_t* seg;
  void* y;          // fp16 or bf16, like x and W
  float* partials;
  int* counters;
  int* status;
  // fused all-reduce: finished tiles go to every rank's receive slot, then a flag per tile
  int push_world;
  unsigned push_epoch;
  void* push_data[8];
  unsigned* push_flags[8];
};

// The pair (code_lo - zero, code_hi - zero) as fp16 (DT = 0) or bf16 (DT = 1) from the
// BITS-wide fields at bit P of both half-words of w, without shifting: OR-ing the field
// into the mantissa of 2^(m-P) (m = 10 / 7 mantissa bits) gives 2^(m-P) + code (the field
// has weight 2^-P there), and one subtraction of 2^(m-P) + zero leaves the exact small
// integer.  Needs P + BITS <= m.
template <int BITS, int P, int DT>
__device__ __forceinline__ uint32_t code_pair(uint32_t w) {
  constexpr uint32_t kMant = DT == 0 ? 10u : 7u;
  constexpr uint32_t kExpBias = DT == 0 ? 15u : 127u;
  static_assert(P + BITS <= (DT == 0 ? 10 : 7), "field must sit inside the mantissa");
  constexpr uint32_t kMask = ((((1u << BITS) - 1u) << P)) * 0x00010001u;
  constexpr uint32_t kMagic = ((kExpBias + kMant - P) << kMant) * 0x00010001u;
  constexpr uint32_t kBiasBits =
      (((kExpBias + kMant - P) << kMant) | ((1u << (BITS - 1)) << P)) * 0x00010001u;
  uint32_t t;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t) : "r"(w), "n"(kMask), "n"(kMagic));
  uint32_t b = kBiasBits;
  if (DT == 0) {
    __half2 hv = __hsub2(*reinterpret_cast<__half2*>(&t), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&hv);
  } else {
    __nv_bfloat162 hv =
        __hsub2(*reinterpret_cast<__nv_bfloat162*>(&t), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&hv);
  }
}
// the 8 (4-bit) or 16 (2-bit) kept values of one packed word -> 4 / 8 pairs
template <int DT>
__device__ __forceinline__ void expand_word4(uint32_t w, uint32_t* o) {
  if (DT == 0) {
    const uint32_t s = w >> 8;
    o[0] = code_pair<4, 0, 0>(w);
    o[1] = code_pair<4, 4, 0>(w);
    o[2] = code_pair<4, 0, 0>(s);
    o[3] = code_pair<4, 4, 0>(s);
  } else {   // 7 mantissa bits hold one nibble at a time
    o[0] = code_pair<4, 0, 1>(w);
    o[1] = code_pair<4, 0, 1>(w >> 4);
    o[2] = code_pair<4, 0, 1>(w >> 8);
    o[3] = code_pair<4, 0, 1>(w >> 12);
  }
}
template <int DT>
__device__ __forceinline__ void expand_word2(uint32_t w, uint32_t* o) {
  if (DT == 0) {
    const uint32_t s = w >> 10;
    o[0] = code_pair<2, 0, 0>(w);
    o[1] = code_pair<2, 2, 0>(w);
    o[2] = code_pair<2, 4, 0>(w);
    o[3] = code_pair<2, 6, 0>(w);
    o[4] = code_pair<2, 8, 0>(w);
    o[5] = code_pair<2, 0, 0>(s);
    o[6] = code_pair<2, 2, 0>(s);
    o[7] = code_pair<2, 4, 0>(s);
  } else {
    const uint32_t s = w >> 6, u = w >> 12;
    o[0] = code_pair<2, 0, 1>(w);
    o[1] = code_pair<2, 2, 1>(w);
    o[2] = code_pair<2, 4, 1>(w);
    o[3] = code_pair<2, 0, 1>(s);
    o[4] = code_pair<2, 2, 1>(s);
    o[5] = code_pair<2, 4, 1>(s);
    o[6] = code_pair<2, 0, 1>(u);
    o[7] = code_pair<2, 2, 1>(u);
  }
}

// Work split.  Every tile is given KU + E "virtual" units: its KU k-units followed by E units
// that stand for the cost of the tile's epilogue, and the virtual units are divided evenly
// over the CTAs (CTA c owns [c*V/grid, (c+1)*V/grid)).  A CTA that finishes a tile in the middle
// of its range is thereby given fewer k-units than one that does not.
// First real unit (tile * KU + ku) of CTA c:
// (32-bit arithmetic: the host refuses shapes with V * grid >= 2^31)
__device__ __forceinline__ int split_begin(int c, int grid, int KU, int E, int V) {
  const int v = (int)((unsigned)c * (unsigned)V / (unsigned)grid);
  const int tile = v / (KU + E);
  const int off = v - tile * (KU + E);
  return tile * KU + min(off, KU);
}
// CTA that owns k-unit ku of `tile`
__device__ __forceinline__ int split_owner(int tile, int ku, int grid, int KU, int E, int V) {
  const unsigned v = (unsigned)(tile * (KU + E) + ku);
  return (int)(((v + 1u) * (unsigned)grid - 1u) / (unsigned)V);
}

struct WinS {
  int slot, col0, ncols, lohi;  // col0 relative to the token block; lohi = lo | hi << 16 (relative)
};


// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
// Per-mode constants.  WIDE = token block of more than 64 columns: three classes and a 128-column
// accumulator pair; otherwise four classes and 64 columns.  The packed-stage ring depth follows
// from the shared-memory budget at the mode's widest block.
__host__ __device__ constexpr int mode_classes(bool wide) { return wide ? 3 : 4; }
__host__ __device__ constexpr int mode_dcols(bool wide) { return wide ? 128 : 64; }
__host__ __device__ constexpr int mode_w_stages(bool wide) { return wide ? DZ_W_STAGES_WIDE : 3; }
__host__ __device__ constexpr int mode_x_stages(bool wide) { return wide ? DZ_X_STAGES_WIDE : 4; }
__host__ __device__ constexpr int mode_r_per_class(int bits, bool wide) {
  const int fixed = mode_x_stages(wide) * mode_dcols(wide) * 128 + mode_w_stages(wide) * kWTile +
                    2 * kNumWG * kWinBytes;
  const int r = (kSmemBudget - fixed) / (mode_classes(wide) * rstage_bytes(bits));
  return r < DZ_MAX_R_PER_CLASS ? r : DZ_MAX_R_PER_CLASS;
}
static_assert(mode_r_per_class(4, false) >= 2 && mode_r_per_class(4, true) >= 2, "ring too shallow");
static_assert(mode_classes(false) * mode_r_per_class(2, false) <= kMaxR, "ring barriers");

// FULLK: K is a multiple of the 128-wide k-unit, so every unit has both half-tiles (the common
// case; the tests on one half-tile in the loops fold away).
template <int BITS, int DT, bool FULLK, bool WIDE>
__global__ void __launch_bounds__(kThreads, 1)
sbmm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_xc,
               const Params p) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t s_bars[2 * kMaxW + 2 * kMaxX + 2 * kMaxR + 2 * kMaxBuf + 2 + kNumWG];
  __shared__ WinS s_win[kMaxWin];
  __shared__ int s_slot[kTokenBlock];   // slot of each column of the token block (-1: base only)
  __shared__ int s_tok[kTokenBlock];    // output row of each column (the table's permutation)
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort, s_last, s_npre;
  __shared__ uint32_t s_fixpar[kNumWG];

  constexpr bool INSTR = kInstr;
  unsigned long long* const tl =
      reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(p.counters) + 4096) +
      (size_t)blockIdx.x * 8;
  if (INSTR && threadIdx.x == 0) tl[0] = globaltimer();
  // INSTR: cycles spent by expansion warpgroup 0 (thread 0) and by the class-0 issuer in each
  // part of their loops, 16 x u64 per CTA behind the parking slots of the last grid CTA
  unsigned long long* const acct =
      reinterpret_cast<unsigned long long*>(p.partials + (size_t)kMaxCtas * 2 * p.cols * 128 - 160 * 16 * 2) +
      (size_t)blockIdx.x * 16;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int C = mode_classes(WIDE);
  constexpr int kDcols = mode_dcols(WIDE);
  constexpr int kWStages = mode_w_stages(WIDE), kXStages = mode_x_stages(WIDE);
  constexpr int kRPer = mode_r_per_class(BITS, WIDE);
  const int nbuf = 2 * C;

  // ---- shared memory carve-up (1024-byte aligned regions) ----
  const uint32_t dyn0 = smem_u32(smem_dyn);
  const uint32_t sbase = (dyn0 + 1023u) & ~1023u;
  const uint32_t s_wring = sbase;
  const uint32_t off_x = kWStages * kWTile;
  const uint32_t off_win = off_x + kXStages * p.xb_bytes;
  const uint32_t off_r = off_win + 2 * kNumWG * kWinBytes;   // every warpgroup owns two
  const uint32_t s_xring = sbase + off_x;
  const uint32_t s_winbuf = sbase + off_win;
  const uint32_t s_rring = sbase + off_r;

  uint64_t* bar_w_full = s_bars;
  uint64_t* bar_w_empty = bar_w_full + kMaxW;
  uint64_t* bar_x_full = bar_w_empty + kMaxW;
  uint64_t* bar_x_empty = bar_x_full + kMaxX;
  uint64_t* bar_r_full = bar_x_empty + kMaxX;
  uint64_t* bar_r_empty = bar_r_full + kMaxR;
  uint64_t* bar_a_ready = bar_r_empty + kMaxR;
  uint64_t* bar_a_free = bar_a_ready + kMaxBuf;
  uint64_t* bar_acc_full = bar_a_free + kMaxBuf;
  uint64_t* bar_acc_empty = bar_acc_full + 1;
  uint64_t* bar_fix = bar_acc_empty + 1;   // per warpgroup: parked partials landed in its scratch

  // ---- this CTA's unit range ----
  const int cta = blockIdx.x;
  const int U = p.total_units;   // virtual units
  const int u_begin = split_begin(cta, p.grid, p.num_kunits, p.epi_units, U);
  const int u_end = split_begin(cta + 1, p.grid, p.num_kunits, p.epi_units, U);
  const int KU = p.num_kunits;

  // ---- part of the prologue that reads nothing an earlier kernel may still be writing ----
  // (barriers whose arrival counts do not depend on the batch, tensor memory, L2 prefetches of
  // the first W tiles).  Under programmatic dependent launch this runs while the predecessor's
  // last CTAs are still draining.
  // Thread 0 needs only the W ring's "full" barriers to request the first W tiles, so it sets
  // those up itself and, in the early-start form, issues the copies at once; the other barriers
  // are initialised by one thread each meanwhile.
  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxW; ++i) mbar_init(smem_u32(&bar_w_full[i]), 1);
    s_abort = 0;
    s_npre = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_xc) : "memory");
    if (p.stable && !p.delta_only) {
      int issued = 0;
      const int npre = min(kWStages, kXStages);
      for (int u = u_begin; u < u_end && issued < npre; ++u) {
        const int n0 = (u / KU) * kTileN, k0 = (u % KU) * kUnitK;
        const int nhalf = FULLK ? 2 : min(2, (p.K - k0) / kBlockK);
        for (int h = 0; h < nhalf && issued < npre; ++h, ++issued) {
          const uint32_t wfull = smem_u32(&bar_w_full[issued]);
          mbar_expect_tx(wfull, kWTile);
          tma_load_2d(s_wring + issued * kWTile, &map_w, k0 + h * kBlockK, n0, wfull);
        }
      }
      s_npre = issued;
    }
    // pull the first W tiles of this CTA's range towards L2 (a prefetch consumes no data, so it
    // is safe whatever the predecessor writes)
    int issued = 0;
    for (int u = u_begin; u < u_end && issued < kPrefetchTiles && !p.delta_only; ++u) {
      const int n0 = (u / KU) * kTileN, k0 = (u % KU) * kUnitK;
      const int nhalf = FULLK ? 2 : min(2, (p.K - k0) / kBlockK);
      for (int h = 0; h < nhalf; ++h, ++issued)
        asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(&map_w),
                     "r"(k0 + h * kBlockK), "r"(n0)
                     : "memory");
    }
  }
  {
    // every other barrier whose arrival count does not depend on the batch: thread 32 + i takes
    // barrier i of the array (x_empty and acc_full follow once the table has been read)
    const int i = (int)threadIdx.x - 32;
    constexpr int kBars = 2 * kMaxW + 2 * kMaxX + 2 * kMaxR + 2 * kMaxBuf + 2 + kNumWG;
    if (i >= kMaxW && i < kBars) {
      uint64_t* b = s_bars + i;
      const bool later = (b >= bar_x_empty && b < bar_x_empty + kMaxX) || b == bar_acc_full;
      uint32_t count = 1;
      if ((b >= bar_r_empty && b < bar_r_empty + kMaxR) || (b >= bar_a_ready && b < bar_a_ready + kMaxBuf))
        count = 128;
      else if (b == bar_acc_empty)
        count = 128 * kNumWG;
      if (!later) {
        mbar_init(smem_u32(b), count);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
      }
    }
    if (i >= 0 && i < kNumWG) s_fixpar[i] = 0;
  }
  // ---- the batch: windows and per-column slots of this token block ----
  // The table's array offsets follow from (M, num_slots), which the call states; the header
  // must agree.  All loads are independent of each other (one L2 round trip) and go to
  // registers first: in the early-start form they are issued here, in front of the tensor
  // memory allocation and the first barrier, so that their latency is hidden; the default form
  // issues them behind the wait for the predecessor (the table may be its output).
  const int* perm = nullptr;
  const int* slot_of = nullptr;
  const Window* wins = nullptr;
  int t_hdr_m = 0, t_hdr_slots = 0, t_hdr_sorted = 0, t_win_end = 0, t_win_begin = 0;
  int t_slot = -1, t_tok = p.row0 + (int)threadIdx.x;
  int t_wslot = 0, t_wcol0 = 0, t_wncols = 0, t_wlo = 0, t_whi = 0;
  auto load_table = [&]() {
    if (!p.seg) return;
    const SegHeader* hdr = reinterpret_cast<const SegHeader*>(p.seg);
    const SegLayout lay = seg_layout(p.M, p.num_slots);
    perm = reinterpret_cast<const int*>(p.seg + lay.perm);
    slot_of = reinterpret_cast<const int*>(p.seg + lay.slot_of);
    const int* bb = reinterpret_cast<const int*>(p.seg + lay.block_begin);
    wins = reinterpret_cast<const Window*>(p.seg + lay.windows);
    t_hdr_m = hdr->capacity_M; t_hdr_slots = hdr->num_slots; t_hdr_sorted = hdr->sorted;
    t_win_end = p.base_only ? 0 : bb[p.token_block + 1];
    if (p.token_block == 0) {
      // the windows of token block 0 start at entry 0; entries beyond the block's count are
      // read (inside the table) but never used
      const int cap = min(kMaxWin, seg_max_windows(p.M, p.num_slots));
      if (!p.base_only && (int)threadIdx.x < cap) {
        const Window* w = wins + threadIdx.x;
        t_wslot = w->slot; t_wcol0 = w->col0; t_wncols = w->ncols; t_wlo = w->lo; t_whi = w->hi;
      }
    } else if (!p.base_only) {
      t_win_begin = bb[p.token_block];
    }
    if ((int)threadIdx.x < kTokenBlock) {
      const int prow = p.row0 + (int)threadIdx.x;
      if (prow < p.M) {
        if (!p.base_only) t_slot = slot_of[prow];
        t_tok = perm[prow];
      }
    }
  };
  if (p.stable) load_table();
  if (warp == kWarpBase) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "n"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  // Programmatic dependent launch: this grid may be scheduled while its predecessor in the
  // stream is still draining.  Nothing the predecessor may write is touched before the wait,
  // which returns once the predecessor has completed and its writes are visible; then the next
  // kernel in the stream is allowed to be scheduled early in turn.
  //   default: the predecessor may have written anything (x, the segment table, weights), so
  //            every thread waits here;
  //   stable : the caller states that the base weight, the slot stacks and the segment table are
  //            not the predecessor's output.  Only x (and the shared workspace, y) still depend
  //            on it, and they are first touched by copies the TMA producer thread issues, so
  //            that thread alone waits (at the start of its role) and everything else -- the
  //            table, the first W tiles, the packed stages, the expansion of the first windows
  //            -- proceeds under the predecessor's tail.
  if (!p.stable) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    load_table();
  }
  if (INSTR && threadIdx.x == 0) tl[1] = globaltimer();

  // Default form: the first W and x tiles are requested here, right behind the wait; the
  // producer warp skips them later.  (The early-start form requested its W tiles above and
  // leaves x to the producer thread.)
  if (threadIdx.x == 0 && !p.stable) {
    int issued = 0;
    const int npre = min(kWStages, kXStages);
    for (int u = u_begin; u < u_end && issued < npre; ++u) {
      const int n0 = (u / KU) * kTileN, k0 = (u % KU) * kUnitK;
      const int nhalf = FULLK ? 2 : min(2, (p.K - k0) / kBlockK);
      for (int h = 0; h < nhalf && issued < npre; ++h, ++issued) {
        const uint32_t xfull = smem_u32(&bar_x_full[issued]);
        mbar_expect_tx(xfull, p.xb_bytes);
        tma_load_2d(s_xring + issued * p.xb_bytes, &map_xc, k0 + h * kBlockK, p.row0, xfull);
        if (!p.delta_only) {
          const uint32_t wfull = smem_u32(&bar_w_full[issued]);
          mbar_expect_tx(wfull, kWTile);
          tma_load_2d(s_wring + issued * kWTile, &map_w, k0 + h * kBlockK, n0, wfull);
        }
      }
    }
    s_npre = issued;
  }

  // ---- the table's entries go to shared memory ----
  int nwin = 0;
  bool bad = false;
  if (p.seg) {
    bad = (t_hdr_m != p.M) || (t_hdr_slots != p.num_slots) || (p.tokens_sorted && !t_hdr_sorted);
    if (!p.base_only && !bad) nwin = min(t_win_end - t_win_begin, kMaxWin);
    if (p.token_block == 0) {
      const int cap = min(kMaxWin, seg_max_windows(p.M, p.num_slots));
      if (!p.base_only && (int)threadIdx.x < cap) {
        WinS ws;
        ws.slot = t_wslot;
        ws.col0 = t_wcol0 - p.row0;
        ws.ncols = t_wncols;
        ws.lohi = (t_wlo - t_wcol0) | ((t_whi - t_wcol0) << 16);
        s_win[threadIdx.x] = ws;
      }
    } else {
      for (int i = threadIdx.x; i < nwin; i += kThreads) {
        const Window w = wins[t_win_begin + i];
        WinS ws;
        ws.slot = w.slot;
        ws.col0 = w.col0 - p.row0;
        ws.ncols = w.ncols;
        ws.lohi = (w.lo - w.col0) | ((w.hi - w.col0) << 16);
        s_win[i] = ws;
      }
    }
  }
  if ((int)threadIdx.x < kTokenBlock) {
    s_slot[threadIdx.x] = t_slot;
    s_tok[threadIdx.x] = t_tok;
  }
  if (threadIdx.x == 0) {
    // freed by the base issuer's commit and, when there are windows, by every thread of every
    // active expansion warpgroup
    for (int i = 0; i < kMaxX; ++i)
      mbar_init(smem_u32(&bar_x_empty[i]), 1 + (nwin > 0 ? 128 * C : 0));
    mbar_init(smem_u32(bar_acc_full), 1 + (nwin > 0 ? (2 * C <= kIssuerWarps ? 2 * C : C) : 0));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (bad && blockIdx.x == 0) atomicCAS(p.status, 0, (int)DZ_ERR_INVALID_ARG);
  }
  // D_delta starts at zero (the delta MMAs always accumulate)
  if (warp >= kFirstWGWarp && nwin > 0) {
    const int wg = (warp - kFirstWGWarp) >> 2;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    for (int c = wg; c < p.cols / 16; c += kNumWG) tmem_st16_zero(lane_addr + kDcols + c * 16);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (INSTR && threadIdx.x == 0) tl[2] = globaltimer();
  // register hand-over between the role groups (whole warpgroups execute the same form)
  if (kServiceRegs != 0) {
    if (warp < kFirstWGWarp) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kServiceRegs));
    else asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kExpandRegs));
  }
  const int npre_w = s_npre;                     // W half-tiles requested in the prologue
  const int npre_x = p.stable ? 0 : s_npre;      // x half-tiles requested in the prologue
  const uint32_t a_col0 = 2 * kDcols;          // TMEM column of expanded-A buffer 0
  const uint32_t e_col0 = a_col0 + nbuf * 32;   // TMEM column of metadata buffer 0

  if (bad) {
    // rejected batch: nothing runs, but the tiles requested in the prologue must land before
    // this CTA's shared memory is released
    if (threadIdx.x == 0) {
      for (int i = 0; i < npre_x; ++i) mbar_wait(smem_u32(&bar_x_full[i]), 0, abort_flag, nullptr);
      if (!p.delta_only)
        for (int i = 0; i < npre_w; ++i) mbar_wait(smem_u32(&bar_w_full[i]), 0, abort_flag, nullptr);
    }
  } else if (warp == kWarpWX) {
    // ====================== TMA producer: W tiles and x half-tiles ======================
    if (lane == 0) {
      if (p.stable) {
        // the only thread whose copies read the predecessor's output
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
      }
      Ring rw(kWStages, 1), rx(kXStages, 1);
      int cnt = 0;   // half-tiles so far; the first ones were requested in the prologue
      for (int u = u_begin; u < u_end;) {
        const int tile = u / KU, ku0 = u % KU;
        const int ku1 = min(KU, ku0 + (u_end - u));
        const int n0 = tile * kTileN;
        for (int ku = ku0; ku < ku1; ++ku) {
          const int k0 = ku * kUnitK;
          const int nhalf = FULLK ? 2 : min(2, (p.K - k0) / kBlockK);
          for (int h = 0; h < nhalf; ++h) {
            if (cnt >= npre_x) {
              mbar_wait(smem_u32(&bar_x_empty[rx.idx]), rx.par, abort_flag, p.status);
              const uint32_t xfull = smem_u32(&bar_x_full[rx.idx]);
              mbar_expect_tx(xfull, p.xb_bytes);
              tma_load_2d(s_xring + rx.idx * p.xb_bytes, &map_xc, k0 + h * kBlockK, p.row0, xfull);
            }
            if (!p.delta_only && cnt >= npre_w) {
              mbar_wait(smem_u32(&bar_w_empty[rw.idx]), rw.par, abort_flag, p.status);
              const uint32_t wfull = smem_u32(&bar_w_full[rw.idx]);
              mbar_expect_tx(wfull, kWTile);
              tma_load_2d(s_wring + rw.idx * kWTile, &map_w, k0 + h * kBlockK, n0, wfull);
            }
            ++cnt;
            rx.advance();
            rw.advance();
          }
        }
        u += ku1 - ku0;
      }
    }
  } else if (warp == kWarpR) {
    // ====================== bulk-copy producer: packed delta stages ======================
    // class t = w mod C owns sub-ring t (r_per_class slots); its n-th stage uses
    // slot n mod r_per_class
    // lane t handles class t: the lanes run the same loop in lock step, so one
    // warp instruction issues the copies of up to C stages
    if (lane < C && nwin > 0) {
      const int t = lane;
      const int cnt_t = (nwin - t + C - 1) / C;
      const int cnt_max = (nwin + C - 1) / C;
      int rs = 0;
      uint32_t par = 1;
      for (int u = u_begin; u < u_end;) {
        const int tile = u / KU, ku0 = u % KU;
        const int ku1 = min(KU, ku0 + (u_end - u));
        for (int ku = ku0; ku < ku1; ++ku) {
          const int nhalf = FULLK ? 2 : min(2, (p.K - ku * kUnitK) / kBlockK);
          const uint32_t code_bytes = nhalf * codes_block_bytes(BITS);
          const uint32_t meta_bytes = nhalf * kMetaBlockBytes;
          const size_t blk = (size_t)tile * p.num_kblocks + (size_t)ku * 2;
          for (int j = 0; j < cnt_max; ++j) {
            if (j < cnt_t) {
              const int slot_idx = t * kRPer + rs;
              const int slot = s_win[t + j * C].slot;
              mbar_wait(smem_u32(&bar_r_empty[slot_idx]), par, abort_flag, p.status);
              const uint32_t full = smem_u32(&bar_r_full[slot_idx]);
              mbar_expect_tx(full, code_bytes + meta_bytes);
              const uint32_t dst = s_rring + slot_idx * rstage_bytes(BITS);
              bulk_load(dst, p.qweight + (size_t)slot * p.qstride + blk * codes_block_bytes(BITS),
                        code_bytes, full);
              bulk_load(dst + raw_bytes(BITS),
                        p.meta + (size_t)slot * p.mstride + blk * kMetaBlockBytes, meta_bytes, full);
              if (++rs == kRPer) { rs = 0; par ^= 1; }
            }
          }
        }
        u += ku1 - ku0;
      }
    }
  } else if (warp == kWarpBase) {
    // =========================== base MMA issuer ===========================
    if (lane == 0) {
      Ring rw(kWStages, 0), rx(kXStages, 0);
      int pacc = 1;
      const uint32_t idesc_base = make_idesc<DT>(p.cols, false);
      for (int u = u_begin; u < u_end;) {
        const int ku0 = u % KU;
        const int ku1 = min(KU, ku0 + (u_end - u));
        mbar_wait(smem_u32(bar_acc_empty), pacc, abort_flag, p.status);
        pacc ^= 1;
        tc_fence_after();
        uint32_t acc = 0;
        for (int ku = ku0; ku < ku1; ++ku) {
          const int nhalf = FULLK ? 2 : min(2, (p.K - ku * kUnitK) / kBlockK);
          for (int h = 0; h < nhalf; ++h) {
            mbar_wait(smem_u32(&bar_x_full[rx.idx]), rx.par, abort_flag, p.status);
            if (!p.delta_only) {
              mbar_wait(smem_u32(&bar_w_full[rw.idx]), rw.par, abort_flag, p.status);
              tc_fence_after();
              if (INSTR && u == u_begin && ku == ku0 && h == 0) tl[3] = globaltimer();
              umma_ss_x4(tmem_base, desc_lo(s_wring + rw.idx * kWTile),
                         desc_lo(s_xring + rx.idx * p.xb_bytes), idesc_base, acc);
              acc = 1;
              umma_commit(smem_u32(&bar_w_empty[rw.idx]));
            }
            umma_commit(smem_u32(&bar_x_empty[rx.idx]));
            rw.advance();
            rx.advance();
          }
        }
        umma_commit(smem_u32(bar_acc_full));
        u += ku1 - ku0;
      }
      if (INSTR) tl[4] = globaltimer();
    }
  } else if (warp >= kWarpIssuer0 && warp < kWarpIssuer0 + kIssuerWarps) {
    // =========================== delta MMA issuers of class t ===========================
    // A thread's MMAs cost ~200 cycles each to issue whatever their width, and a window needs
    // four.  Where the warps allow it (2 * classes <= kIssuerWarps) a class has two issuing
    // threads: one takes the class's even windows (expanded-A buffer 0), the other the odd ones
    // (buffer 1).  Different windows of a class put their non-zero products into different
    // accumulator columns, so the order in which the two threads' MMAs run changes no sum.
    const int iw = warp - kWarpIssuer0;
    const bool paired = 2 * C <= kIssuerWarps;
    const int t = iw % C;
    const int par = paired ? iw / C : -1;      // -1: this thread takes every window of its class
    if (lane == 0 && iw < (paired ? 2 * C : C) && nwin > 0) {
      const int cnt_t = (nwin - t + C - 1) / C;
      int pacc = 1, n = 0;
      long long i_wait = 0, i_issue = 0, i_acc = 0, tq = 0;
      for (int u = u_begin; u < u_end;) {
        const int ku0 = u % KU;
        const int ku1 = min(KU, ku0 + (u_end - u));
        if (INSTR) tq = clock64();
        mbar_wait(smem_u32(bar_acc_empty), pacc, abort_flag, p.status);
        if (INSTR) i_acc += clock64() - tq;
        pacc ^= 1;
        tc_fence_after();
        for (int ku = ku0; ku < ku1; ++ku) {
          const int nhalf = FULLK ? 2 : min(2, (p.K - ku * kUnitK) / kBlockK);
          for (int j = 0; j < cnt_t; ++j, ++n) {
            if (par >= 0 && (n & 1) != par) continue;
            const WinS ws = s_win[t + j * C];
            const int buf = t + C * (n & 1);
            if (INSTR) tq = clock64();
            mbar_wait(smem_u32(&bar_a_ready[buf]), (n >> 1) & 1, abort_flag, p.status);
            if (INSTR) { const long long t2 = clock64(); i_wait += t2 - tq; tq = t2; }
            tc_fence_after();
            const uint32_t win_lo = desc_lo(s_winbuf + buf * kWinBytes);
            const uint32_t idesc = make_idesc<DT>(ws.ncols, true);
            const uint32_t dcol = tmem_base + kDcols + ws.col0;
            const uint32_t acol = tmem_base + a_col0 + buf * 32;
            const uint32_t ecol = tmem_base + e_col0 + buf * 4;
            umma_ts_sp_x2(dcol, acol, win_lo, ecol, idesc);
            if (nhalf == 2) umma_ts_sp_x2(dcol, acol + 16, win_lo + ws.ncols * 8, ecol + 2, idesc);
            umma_commit(smem_u32(&bar_a_free[buf]));
            if (INSTR) i_issue += clock64() - tq;
          }
        }
        umma_commit(smem_u32(bar_acc_full));
        u += ku1 - ku0;
      }
      if (INSTR && iw == 0) { acct[8] = i_wait; acct[9] = i_issue; acct[10] = i_acc; acct[11] = n; }
    }
  } else if (warp >= kFirstWGWarp) {
    // ================= code expansion (class = warpgroup) + epilogue =================
    const int q = warp & 3;              // TMEM lane quarter this warp may touch
    const int r = q * 32 + lane;         // tile row == TMEM lane
    const int wg = (warp - kFirstWGWarp) >> 2;
    const int wg_tid = (threadIdx.x - 32 * kFirstWGWarp) & 127;
    const int ep_tid = threadIdx.x - 32 * kFirstWGWarp;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const bool active = (wg < C) && nwin > 0;
    const int cnt_t = active ? (nwin - wg + C - 1) / C : 0;
    Ring rx(kXStages, 0);
    int pacc = 0, n = 0, rs = 0;
    uint32_t rpar = 0;
    bool cta_first_fragment = true;
    long long a_x = 0, a_r = 0, a_free = 0, a_exp = 0, a_win = 0, a_fin = 0, a_epi = 0, tq = 0;
    const bool acc_on = INSTR && ep_tid == 0;

    for (int u = u_begin; u < u_end;) {
      const int tile = u / KU, ku0 = u % KU;
      const int ku1 = min(KU, ku0 + (u_end - u));
      const int n0 = tile * kTileN;
      for (int ku = ku0; ku < ku1 && active; ++ku) {
        const int k0 = ku * kUnitK;
        const int nhalf = FULLK ? 2 : min(2, (p.K - k0) / kBlockK);
        // the unit's x half-tiles
        uint32_t xsrc0 = 0, xsrc1 = 0;
        int xslot0 = 0, xslot1 = 0;
        if (acc_on) tq = clock64();
        for (int h = 0; h < nhalf; ++h) {
          mbar_wait(smem_u32(&bar_x_full[rx.idx]), rx.par, abort_flag, p.status);
          if (h == 0) { xsrc0 = s_xring + rx.idx * p.xb_bytes; xslot0 = rx.idx; }
          else { xsrc1 = s_xring + rx.idx * p.xb_bytes; xslot1 = rx.idx; }
          rx.advance();
        }
        for (int j = 0; j < cnt_t; ++j, ++n) {
          const WinS ws = s_win[wg + j * C];
          const int buf = wg + C * (n & 1);
          const int rslot = wg * kRPer + rs;
          if (acc_on) { const long long t2 = clock64(); if (j == 0) a_x += t2 - tq; tq = t2; }
          mbar_wait(smem_u32(&bar_r_full[rslot]), rpar, abort_flag, p.status);
          if (acc_on) { const long long t2 = clock64(); a_r += t2 - tq; tq = t2; }
          if (++rs == kRPer) { rs = 0; rpar ^= 1; }
          mbar_wait(smem_u32(&bar_a_free[buf]), ((n >> 1) & 1) ^ 1, abort_flag, p.status);
          if (acc_on) { const long long t2 = clock64(); a_free += t2 - tq; tq = t2; }
          tc_fence_after();
          const uint32_t raw = s_rring + rslot * rstage_bytes(BITS);
          const uint32_t my_win = s_winbuf + buf * kWinBytes;
          uint32_t mw[4] = {0, 0, 0, 0};
          auto expand_half = [&](const int h) {
            uint32_t o[16];
            if (BITS == 4) {
              const uint4 cw = lds128(raw + h * 2048 + r * 16);
              const uint32_t wv[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
              for (int wi = 0; wi < 4; ++wi) expand_word4<DT>(wv[wi], o + wi * 4);
            } else {
              const uint2 cw = lds64(raw + h * 1024 + r * 8);
              const uint32_t wv[2] = {cw.x, cw.y};
#pragma unroll
              for (int wi = 0; wi < 2; ++wi) expand_word2<DT>(wv[wi], o + wi * 8);
            }
            // compressed A of this half: 32 fp16 = 16 columns of the row's lane
            tmem_st16(lane_addr + a_col0 + buf * 32 + h * 16, o);
            const uint2 m2 = lds64(raw + raw_bytes(BITS) + h * 1024 + r * 8);
            mw[h * 2] = m2.x;
            mw[h * 2 + 1] = m2.y;
          };
          expand_half(0);
          if (nhalf == 2) expand_half(1);
          tmem_st4(lane_addr + e_col0 + buf * 4, mw[0], mw[1], mw[2], mw[3]);
          // the packed stage has been consumed
          mbar_arrive(smem_u32(&bar_r_empty[rslot]));
          if (acc_on) { const long long t2 = clock64(); a_exp += t2 - tq; tq = t2; }
          // the slot's token window: rows of the resident x half-tiles, other slots' rows zeroed
          // (16-byte chunk c of a half = row c >> 3; both halves' chunks are requested together)
          {
            const int lo = ws.lohi & 0xFFFF, hi = ws.lohi >> 16;
            const uint32_t x0 = xsrc0 + ws.col0 * 128;
            const uint32_t x1 = xsrc1 + ws.col0 * 128;
            const uint32_t half_bytes = ws.ncols * 128;
            const uint4 zero4 = make_uint4(0, 0, 0, 0);
            for (int c = wg_tid; c < ws.ncols * 8; c += 128) {
              const int row = c >> 3;
              const bool in = row >= lo && row < hi;
              uint4 v0 = zero4, v1 = zero4;
              if (in) {
                v0 = lds128(x0 + c * 16);
                if (nhalf == 2) v1 = lds128(x1 + c * 16);
              }
              sts128(my_win + c * 16, v0);
              if (nhalf == 2) sts128(my_win + half_bytes + c * 16, v1);
            }
          }
          if (acc_on) { const long long t2 = clock64(); a_win += t2 - tq; tq = t2; }
          fence_proxy_async();
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(smem_u32(&bar_a_ready[buf]));
          if (acc_on) { const long long t2 = clock64(); a_fin += t2 - tq; tq = t2; }
        }
        // this warpgroup no longer reads the unit's x half-tiles
        mbar_arrive(smem_u32(&bar_x_empty[xslot0]));
        if (nhalf == 2) mbar_arrive(smem_u32(&bar_x_empty[xslot1]));
      }

      // ---------------- epilogue of this fragment ----------------
      // A fragment that does not cover its whole tile settles the tile with the other
      // fragments through two counters: `ticket` (claimed while this fragment's last MMAs
      // drain) and `parked`.  The holder of the last ticket never parks anything: it waits
      // until the others have parked (they hold earlier tickets, so they are already in their
      // epilogues and depend on nothing), then adds their partials to its own accumulators in
      // fragment order, straight from registers.  Every other fragment parks its partial and
      // leaves with a single fire-and-forget release increment.
      if (acc_on) tq = clock64();
      const bool full_tile = (ku0 == 0 && ku1 == KU);
      int c_first = 0, nfrag = 1, ticket = 0;
      uint32_t slot_first = 0;   // parking slot (0/1) of the tile's first fragment
      if (!full_tile) {
        c_first = split_owner(tile, 0, p.grid, KU, p.epi_units, U);
        nfrag = split_owner(tile, KU - 1, p.grid, KU, p.epi_units, U) - c_first + 1;
        slot_first = (split_begin(c_first, p.grid, KU, p.epi_units, U) / KU == tile) ? 0u : 1u;
        if (ep_tid == 0) ticket = atomicAdd(&p.counters[2 * tile], 1);
      }
      // D_delta holds sums of (code - zero) * x; the per-channel scale of each
      // column's slot is applied here.  The scales are requested before the wait for the
      // fragment's last MMAs, so they arrive while those drain.
      uint32_t csc[8];   // fp16 bit patterns of column chunk `wg`, two columns per word
#pragma unroll
      for (int i = 0; i < 8; ++i) csc[i] = 0;
      if (nwin > 0 && wg < p.cols / 16) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int slot = s_slot[wg * 16 + i];
          uint32_t v = 0;
          if (slot >= 0)
            v = *reinterpret_cast<const unsigned short*>(p.scales + (size_t)slot * p.sstride +
                                                         (size_t)(n0 + r) * 2);
          csc[i >> 1] |= v << (16 * (i & 1));
        }
      }
      mbar_wait(smem_u32(bar_acc_full), pacc, abort_flag, p.status);
      pacc ^= 1;
      tc_fence_after();
      if (INSTR && ep_tid == 0 && ku1 - ku0 == u_end - u) tl[5] = globaltimer();
      bool last = false;
      if (!full_tile) {
        if (ep_tid == 0) {
          const int is_last = (ticket == nfrag - 1) ? 1 : 0;
          if (is_last) {
            // bounded wait for the earlier ticket holders' partials
            unsigned long long t0 = 0;
            for (uint32_t it = 0;; ++it) {
              int parked;
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];"
                           : "=r"(parked)
                           : "l"(p.counters + 2 * tile + 1)
                           : "memory");
              if (parked >= nfrag - 1 || *abort_flag) break;
              __nanosleep(64);
              if ((it & 63u) == 63u) {
                const unsigned long long now = globaltimer();
                if (t0 == 0) {
                  t0 = now;
                } else if (now - t0 > kTimeoutNs) {
                  *abort_flag = 1;
                  atomicCAS(p.status, 0, (int)DZ_ERR_TIMEOUT);
                  break;
                }
              }
            }
            // the tile is settled once this fragment has written it: counters back to zero
            // (not after a timeout: late fragments may still add to them, and the caller
            // has to clear the workspace after DZ_ERR_TIMEOUT anyway)
            if (!*abort_flag) {
              p.counters[2 * tile] = 0;
              p.counters[2 * tile + 1] = 0;
            }
          }
          s_last = is_last;
        }
        named_bar_sync(1, 128 * kNumWG);
        last = s_last != 0;
      }
      // this fragment's parking slot, as a float index into the partials
      const uint32_t my_park = (uint32_t)(cta * 2 + (cta_first_fragment ? 0 : 1)) * (uint32_t)(p.cols * 128);
      // phase of the warpgroup's fix-up barrier (kept in shared memory between fragments)
      uint32_t fixpar = last ? s_fixpar[wg] : 0;
      for (int c = wg; c < p.cols / 16; c += kNumWG) {
        if (nwin > 0 && c != wg) {   // second chunk of a wide token block: its scales are fetched here
#pragma unroll
          for (int i = 0; i < 8; ++i) csc[i] = 0;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int slot = s_slot[c * 16 + i];
            uint32_t sv = 0;
            if (slot >= 0)
              sv = *reinterpret_cast<const unsigned short*>(p.scales + (size_t)slot * p.sstride +
                                                            (size_t)(n0 + r) * 2);
            csc[i >> 1] |= sv << (16 * (i & 1));
          }
        }
        // eight columns at a time keep the epilogue's register needs below the main loop's
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          const int col = c * 16 + hb * 8;
          uint32_t v[8], d[8];
          if (p.delta_only) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0;
          } else {
            tmem_ld8(lane_addr + col, v);
          }
          if (nwin > 0) tmem_ld8(lane_addr + kDcols + col, d);
          tmem_wait_ld();
          if (nwin > 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t pair = csc[hb * 4 + (i >> 1)];
              const float sc = __half2float(__ushort_as_half((unsigned short)(pair >> (16 * (i & 1)))));
              v[i] = __float_as_uint(fmaf(sc, __uint_as_float(d[i]), __uint_as_float(v[i])));
            }
          }
          if (last) {
            // Sum over the tile's fragments in CTA order, this fragment's accumulators taking
            // their own place in that order.  Everything is summed out of shared memory: the
            // thread's own 8 values go to slot 3 of the scratch, the other fragments' parked
            // columns arrive three fragments at a time by bulk copies (one L2 round trip for
            // 3 x 8 columns).  The scratch is the warpgroup's own two window buffers, idle
            // until its next expansion.
            const int my_f = cta - c_first;
            const uint32_t scr0 = s_winbuf + (wg < C ? wg : 2 * C + 2 * (wg - C)) * kWinBytes + r * 4;
            const uint32_t scr1 = scr0 + (wg < C ? C : 1) * kWinBytes;
            const uint32_t fixbar = smem_u32(&bar_fix[wg]);
            named_bar_sync(2 + wg, 128);   // nobody still reads the scratch (previous columns)
#pragma unroll
            for (int i = 0; i < 8; ++i) sts32(scr1 + 4096 + i * 512, v[i]);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0;   // from here on v is the running sum
            for (int j = 0; j < nfrag - 1; j += 3) {
              const int cnt = min(3, nfrag - 1 - j);
              if (j > 0) named_bar_sync(2 + wg, 128);
              if (wg_tid == 0) {
                // the scratch was written by generic stores (shared), the parked partials by
                // other CTAs' generic stores (global): both must be ordered before the bulk
                // copies, which go through the async proxy
                fence_proxy_async();
                asm volatile("fence.proxy.async.global;" ::: "memory");
                mbar_expect_tx(fixbar, cnt * 4096);
#pragma unroll
                for (int ff = 0; ff < 3; ++ff) {
                  if (ff >= cnt) break;
                  const int o = j + ff;   // o-th other fragment = fragment o, or o + 1 past this one
                  const int f = o + (o >= my_f ? 1 : 0);
                  // only the tile's first fragment can be its CTA's second parking slot
                  const uint32_t slot = (uint32_t)(c_first + f) * 2 + (f == 0 ? slot_first : 0);
                  const uint32_t off = (slot * (uint32_t)p.cols + (uint32_t)col) * 512u;
                  bulk_load((ff < 2 ? scr0 : scr1) - r * 4 + (ff & 1) * 4096,
                            reinterpret_cast<const uint8_t*>(p.partials) + off, 4096, fixbar);
                }
              }
              mbar_wait(fixbar, fixpar, abort_flag, p.status);
              fixpar ^= 1;
#pragma unroll
              for (int ff = 0; ff < 3; ++ff) {
                if (ff >= cnt) break;
                if (j + ff == my_f) {   // this fragment comes right before its successor
#pragma unroll
                  for (int i = 0; i < 8; ++i)
                    v[i] = __float_as_uint(__uint_as_float(v[i]) +
                                           __uint_as_float(lds32(scr1 + 4096 + i * 512)));
                }
                const uint32_t src = (ff < 2 ? scr0 : scr1) + (ff & 1) * 4096;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(lds32(src + i * 512)));
              }
            }
            if (my_f == nfrag - 1) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                v[i] = __float_as_uint(__uint_as_float(v[i]) +
                                       __uint_as_float(lds32(scr1 + 4096 + i * 512)));
            }
          }
          if (full_tile || last) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int prow = p.row0 + col + i;
              if (prow < p.M) {
                const int tok = s_tok[col + i];   // read in the prologue: no L2 round trip here
                const size_t at = (size_t)tok * (size_t)p.ldy + n0 + r;
                if (p.push_world == 0) {
                  store_out<DT>(p.y, at, __uint_as_float(v[i]), p.accumulate);
                } else {
                  for (int pr = 0; pr < p.push_world; ++pr)
                    store_out<DT>(p.push_data[pr], at, __uint_as_float(v[i]), 0);
                }
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              __stcg(p.partials + (my_park + (uint32_t)((col + i) * 128 + r)), __uint_as_float(v[i]));
          }
        }
        if (nwin > 0) tmem_st16_zero(lane_addr + kDcols + c * 16);   // D_delta restarts from zero
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(smem_u32(bar_acc_empty));
      // (every thread read s_fixpar before the first barrier of its fix-up rounds)
      if (last && wg_tid == 0) s_fixpar[wg] = fixpar;

      if (!full_tile && !last) {
        // release pattern: every thread's partial stores happen before the barrier; one
        // thread then publishes with a device-scope release
        named_bar_sync(1, 128 * kNumWG);
        if (ep_tid == 0)
          asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.counters + 2 * tile + 1)
                       : "memory");
      } else if (p.push_world != 0) {
        // the tile is complete in every rank's receive slot once all epilogue threads' stores
        // are ordered before the flags (same pattern, system scope: the readers are other GPUs)
        named_bar_sync(1, 128 * kNumWG);
        if (ep_tid == 0) {
          __threadfence_system();
          for (int pr = 0; pr < p.push_world; ++pr)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(
                             p.push_flags[pr] + p.token_block * p.num_tiles + tile),
                         "r"(p.push_epoch)
                         : "memory");
        }
      }
      cta_first_fragment = false;
      u += ku1 - ku0;
      if (acc_on) a_epi += clock64() - tq;
    }
    if (INSTR && ep_tid == 0) tl[6] = globaltimer();
    if (acc_on) {
      acct[0] = a_x; acct[1] = a_r; acct[2] = a_free; acct[3] = a_exp; acct[4] = a_win;
      acct[5] = a_fin; acct[6] = a_epi; acct[7] = n;
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
  if (warp == kWarpBase) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "n"(kTmemCols)
                 : "memory");
  }
  if (INSTR && threadIdx.x == 0) tl[7] = globaltimer();
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
struct DeviceInfo {
  int sms = 0;
  bool attr_set[16] = {};
};
DeviceInfo& device_info(int dev) {
  static DeviceInfo info[64];
  return info[dev & 63];
}

}  // namespace

size_t sbmm_workspace_bytes(int M, int N, int K, int tokens_sorted) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  size_t b = kWsPartials + sbmm_partial_bytes(M);
  if (!tokens_sorted) b += (size_t)round_up(M, 16) * K * 2 + 1024;
  return b;
}

int launch_sbmm(const dz_sbmm_args& a, bool base_only, cudaStream_t st) {
  int dev = 0;
  DZ_CUDA_OK(cudaGetDevice(&dev));
  DeviceInfo& di = device_info(dev);
  if (di.sms == 0) DZ_CUDA_OK(cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev));
  if (a.N / kTileN > (int)(kWsCountersBytes / 8)) return DZ_ERR_TOO_LARGE;

  uint8_t* ws = reinterpret_cast<uint8_t*>(a.workspace);
  const bool sorted = base_only || a.tokens_sorted != 0;
  const void* xsrc = a.x;
  if (!sorted) {
    uint8_t* xs = ws + ((kWsPartials + sbmm_partial_bytes(a.M) + 1023) & ~(size_t)1023);
    gather_rows_kernel<<<a.M, 128, 0, st>>>((const uint4*)a.x, (const uint8_t*)a.segments,
                                             (uint4*)xs, a.M, a.K / 8);
    DZ_CUDA_OK(cudaGetLastError());
    xsrc = xs;
  }

  CUtensorMap map_w, map_xc;
  const int dt = (a.dtype == DZ_DTYPE_BF16) ? 1 : 0;
  int rc = DZ_OK;
  if (a.w_base) {
    rc = make_map(&map_w, a.w_base, a.N, a.K, 128, dt);
    if (rc) return rc;
  } else if (base_only) {
    return DZ_ERR_INVALID_ARG;
  } else {
    memset(&map_w, 0, sizeof(map_w));   // never used: the kernel issues no W loads
  }

  Params p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.bits = a.bits; p.num_slots = a.num_slots;
  p.num_kblocks = a.K / kBlockK;
  p.num_kunits = (a.K + kUnitK - 1) / kUnitK;
  p.num_tiles = a.N / kTileN;
  p.base_only = base_only ? 1 : 0;
  p.delta_only = (!base_only && a.w_base == nullptr) ? 1 : 0;
  p.push_world = 0;
  p.push_epoch = 0;
  if (a.push) {
    p.push_world = a.push->world;
    p.push_epoch = a.push->epoch;
    for (int r = 0; r < 8; ++r) {
      p.push_data[r] = a.push->data[r];
      p.push_flags[r] = reinterpret_cast<unsigned*>(a.push->flags[r]);
    }
  }
  p.accumulate = (a.flags & DZ_SBMM_ACCUMULATE) ? 1 : 0;
  p.stable = (a.flags & DZ_SBMM_INPUTS_STABLE) ? 1 : 0;
  p.ldy = (a.y_stride && !a.push) ? a.y_stride : a.N;
  p.tokens_sorted = sorted ? 1 : 0;
  p.epi_units = kEpilogueUnits;
  p.total_units = p.num_tiles * (p.num_kunits + p.epi_units);
  p.grid = min(min(di.sms, kMaxCtas), p.num_tiles * p.num_kunits);
#ifdef DZ_TUNE_ENV
  {
    static const int min_units = getenv("DZ_MIN_UNITS") ? atoi(getenv("DZ_MIN_UNITS")) : 0;
    if (min_units > 0)
      p.grid = max(min(p.grid, p.num_tiles), min(p.grid, p.num_tiles * (p.num_kunits + p.epi_units) / min_units));
  }
#endif
  if ((long long)(p.total_units + 1) * p.grid >= (1ll << 31)) return DZ_ERR_TOO_LARGE;
  p.qweight = (const uint8_t*)a.qweight;
  p.meta = (const uint8_t*)a.meta;
  p.scales = (const uint8_t*)a.scales;
  p.qstride = a.qweight_stride; p.mstride = a.meta_stride; p.sstride = a.scales_stride;
  p.seg = base_only ? nullptr : (const uint8_t*)a.segments;
  p.y = a.y;
  p.status = reinterpret_cast<int*>(ws + kWsStatus);
  p.counters = reinterpret_cast<int*>(ws + kWsCounters);
  p.partials = reinterpret_cast<float*>(ws + kWsPartials);

  const int num_tb = (a.M + kTokenBlock - 1) / kTokenBlock;
  for (int tb = 0; tb < num_tb; ++tb) {
    p.token_block = tb;
    p.row0 = tb * kTokenBlock;
    p.cols = min(kTokenBlock, round_up(a.M - p.row0, 16));
    p.xb_bytes = p.cols * 128;
    p.dcols = p.cols <= 64 ? 64 : 128;
    p.nclass = p.cols <= 64 ? 4 : 3;
    p.x_stages = p.cols <= 64 ? 4 : DZ_X_STAGES_WIDE;
    p.w_stages = p.cols <= 64 ? 3 : DZ_W_STAGES_WIDE;
    const int fixed = p.x_stages * p.xb_bytes + p.w_stages * kWTile + 2 * kNumWG * kWinBytes;
    const int rstage = rstage_bytes(a.bits);
    const bool wide = p.cols > 64;
    p.r_per_class = mode_r_per_class(a.bits, wide);
    rc = make_map(&map_xc, xsrc, a.M, a.K, p.cols, dt);
    if (rc) return rc;
    const size_t smem = (size_t)fixed + (size_t)p.nclass * p.r_per_class * rstage + 1024;
    const bool fullk = (a.K % kUnitK) == 0;
    using Kern = void (*)(const CUtensorMap, const CUtensorMap, const Params);
    static const Kern kerns[16] = {
        sbmm_tc_kernel<2, 0, false, false>, sbmm_tc_kernel<4, 0, false, false>,
        sbmm_tc_kernel<2, 1, false, false>, sbmm_tc_kernel<4, 1, false, false>,
        sbmm_tc_kernel<2, 0, true, false>,  sbmm_tc_kernel<4, 0, true, false>,
        sbmm_tc_kernel<2, 1, true, false>,  sbmm_tc_kernel<4, 1, true, false>,
        sbmm_tc_kernel<2, 0, false, true>,  sbmm_tc_kernel<4, 0, false, true>,
        sbmm_tc_kernel<2, 1, false, true>,  sbmm_tc_kernel<4, 1, false, true>,
        sbmm_tc_kernel<2, 0, true, true>,   sbmm_tc_kernel<4, 0, true, true>,
        sbmm_tc_kernel<2, 1, true, true>,   sbmm_tc_kernel<4, 1, true, true>};
    const int kidx = ((a.bits == 2) ? 0 : 1) + (dt ? 2 : 0) + (fullk ? 4 : 0) + (wide ? 8 : 0);
    Kern kern = kerns[kidx];
    if (!di.attr_set[kidx]) {
      DZ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
      di.attr_set[kidx] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DZ_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, map_w, map_xc, p));
  }
  return DZ_OK;
}

}  // namespace dz

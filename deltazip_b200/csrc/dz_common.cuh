// Shared definitions of the deltazip_b200 CUDA sources: status codes, the slot
// layout (where a code / a 2:4 position of element (n, k) lives) and the batch
// segment table.  Host and device code use the same index functions.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/deltazip_b200.h"

namespace dz {

// ---------------------------------------------------------------------------
// Slot layout.
//
// Rows (output features) are grouped in tiles of 128, the reduction dimension
// in blocks of 64 dense k (= 16 groups of four = 32 kept values per row).
// Block (t, kb) of the code array holds, for each of the 128 rows of tile t,
// `4*bits` contiguous bytes (16 B at 4-bit, 8 B at 2-bit); blocks of one tile
// are contiguous over kb, so a CTA that owns (tile, k-range) streams one
// contiguous byte range.  Inside a row's bytes the kept values e = 0..31 (in
// ascending k order: e = 2*group + which) sit in 32-bit words of 32/bits
// codes; within a word, local element e' lives at bit
//     (e' & 1) * 16 + bits * (e' >> 1)
// so that (word >> (bits*j)) & 0x000f000f (or 0x00030003) yields elements
// (2j, 2j+1) in the low / high half-word: one logic op per fp16 pair.
//
// Block (t, kb) of the meta array is 128 "lanes" x 2 words of 32 bit.  Word c
// (c = 0, 1) covers dense k [32c, 32c+32) of the block and is laid out the way
// the 2:4-sparse tensor-core MMA reads its metadata from tensor memory for
// 16-bit operands: lane L = (r & 7) + 8*kh + 16*(r >> 4) carries, in its low
// (r & 8 == 0) or high (r & 8 != 0) half-word, the four 4-bit entries of row r
// for the k-half kh (16 dense k = 4 groups); an entry is i0 | i1 << 2 with
// i0 < i1 the positions (0..3) of the two kept values inside the group.
// ---------------------------------------------------------------------------
constexpr int kTileN = 128;
constexpr int kBlockK = 64;
constexpr int kKeptPerBlock = 32;

__host__ __device__ inline int codes_row_bytes(int bits) { return 4 * bits; }
__host__ __device__ inline int codes_block_bytes(int bits) { return kTileN * 4 * bits; }
__host__ __device__ inline size_t codes_offset(int n, int kb, int num_kb, int bits) {
  return ((size_t)(n >> 7) * num_kb + kb) * codes_block_bytes(bits) +
         (size_t)(n & 127) * codes_row_bytes(bits);
}
// word index (within the row's bytes) and bit shift of kept value e (0..31)
__host__ __device__ inline int code_word(int e, int bits) { return e / (32 / bits); }
__host__ __device__ inline int code_shift(int e, int bits) {
  int el = e % (32 / bits);
  return (el & 1) * 16 + bits * (el >> 1);
}

constexpr int kMetaBlockBytes = kTileN * 8;
// byte offset of the 16-bit metadata entry of row n, block kb, word c, k-half kh
__host__ __device__ inline size_t meta_offset(int n, int kb, int num_kb, int c, int kh) {
  int r = n & 127;
  int lane = (r & 7) + 8 * kh + 16 * (r >> 4);
  int half = (r >> 3) & 1;
  return (((size_t)(n >> 7) * num_kb + kb) * kTileN + lane) * 8 + c * 4 + half * 2;
}

// ---------------------------------------------------------------------------
// Segment table (device memory, written by build_segments_kernel).
//
// Tokens are put in "sorted order": ascending slot id, -1 (base only) first.
// perm[p] is the original row of sorted position p; slot_of[p] its slot.
// Sorted positions are cut into token blocks of kTokenBlock columns (one
// accumulator pass each).  A "window" is a 16-aligned span of sorted positions
// inside one token block that covers (part of) one slot's segment: the delta
// MMA for that slot runs over the window's columns with rows outside
// [lo, hi) zeroed.
// ---------------------------------------------------------------------------
constexpr int kTokenBlock = 128;
constexpr int kMaxWindowCols = 32;
constexpr int kMaxSlots = 4096;

struct SegHeader {
  int32_t M;
  int32_t num_slots;
  int32_t num_token_blocks;
  int32_t sorted;        // 1: input order already sorted, perm is the identity
  int32_t status;        // dz_status found while building (slot range)
  int32_t num_windows;
  int32_t num_active;    // distinct slots >= 0 present in the batch
  int32_t capacity_M;    // M the table was sized for
  int32_t pad[8];
};
static_assert(sizeof(SegHeader) == 64, "header is one 64-byte line");

struct Window {
  int32_t slot;
  int32_t col0;   // first sorted position, multiple of 16
  int32_t ncols;  // 16 or 32
  int32_t lo;     // valid sorted positions [lo, hi)
  int32_t hi;
  int32_t pad[3];
};
static_assert(sizeof(Window) == 32, "window entry is 32 bytes");

__host__ __device__ inline int round_up(int a, int b) { return (a + b - 1) / b * b; }
__host__ __device__ inline int seg_max_windows(int M, int num_slots) {
  int nb = (M + kTokenBlock - 1) / kTokenBlock;
  return M / 16 + 2 * num_slots + 2 * nb + 8;
}
// byte offsets of the arrays behind the header
struct SegLayout {
  size_t perm, slot_of, block_begin, windows, total;
};
__host__ __device__ inline SegLayout seg_layout(int M, int num_slots) {
  SegLayout l;
  int mr = round_up(M > 0 ? M : 1, 64);
  int nb = (M + kTokenBlock - 1) / kTokenBlock;
  size_t o = sizeof(SegHeader);
  l.perm = o;            o += (size_t)mr * 4;
  l.slot_of = o;         o += (size_t)mr * 4;
  l.block_begin = o;     o += (size_t)round_up(nb + 2, 16) * 4;
  l.windows = o;         o += (size_t)seg_max_windows(M, num_slots) * sizeof(Window);
  l.total = o;
  return l;
}

// ---------------------------------------------------------------------------
// Host-side helpers
// ---------------------------------------------------------------------------
void set_last_cuda_error(cudaError_t e, const char* where);
#define DZ_CUDA_OK(expr)                                   \
  do {                                                     \
    cudaError_t e__ = (expr);                              \
    if (e__ != cudaSuccess) {                              \
      ::dz::set_last_cuda_error(e__, #expr);               \
      return DZ_ERR_CUDA;                                  \
    }                                                      \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// kernel launchers implemented in the other translation units
int launch_convert_from_gptq(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                             int N, int K, int bits, void* sq, void* sm, uint16_t* ss,
                             int* status_word, cudaStream_t st);
int launch_unpack(const void* sq, const void* sm, const uint16_t* ss, int N, int K, int bits,
                  uint16_t* out, cudaStream_t st);
int launch_build_segments(const void* indices, int index_dtype, int M, int num_slots,
                          void* segments, cudaStream_t st);

// ---------------------------------------------------------------------------
// SBMM workspace: [status word | per-tile counters | parked split-K partials | gather buffer].
// Shared by the launcher, the argument checks and the entry point with built-in scratch.
// ---------------------------------------------------------------------------
constexpr size_t kWsStatus = 0;            // int: first error a kernel met (sticky until read)
constexpr size_t kWsCounters = 256;        // int[2 * tiles]: ticket / parked per tile
constexpr size_t kWsCountersBytes = 16384;
constexpr size_t kWsPartials = kWsCounters + kWsCountersBytes;
constexpr int kMaxCtas = 160;              // upper bound of the SBMM grid (one CTA per SM)
__host__ __device__ inline size_t sbmm_partial_bytes(int M) {
  const int cols = M < 128 ? round_up(M, 16) : 128;
  return (size_t)kMaxCtas * 2 * cols * 128 * sizeof(float);
}
size_t sbmm_workspace_bytes(int M, int N, int K, int tokens_sorted);
// Argument checks of dz_sbmm / dz_base_gemm; `check_workspace` = false for callers that
// supply the scratch themselves.
int check_sbmm_args(const dz_sbmm_args* a, bool base_only, bool check_workspace);
int launch_sbmm(const dz_sbmm_args& a, bool base_only, cudaStream_t st);

}  // namespace dz

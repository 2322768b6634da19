// Batch metadata: per-token slot ids -> segment table (sorted order, permutation,
// 16-aligned windows per slot and token block).  One CTA; the work is a few
// thousand integers per scheduling step and is shared by every layer's SBMM.
#include "dz_common.cuh"

namespace dz {

namespace {

__device__ __forceinline__ int load_index(const void* indices, int dtype, int i) {
  long long v = (dtype == DZ_INDEX_I64) ? reinterpret_cast<const long long*>(indices)[i]
                                        : (long long)reinterpret_cast<const int*>(indices)[i];
  return (int)v;
}

__global__ void __launch_bounds__(1024)
build_segments_kernel(const void* __restrict__ indices, int dtype, int M, int num_slots,
                      uint8_t* __restrict__ table) {
  extern __shared__ int smem[];
  int* counts = smem;                    // [num_slots + 1], bucket b = slot + 1
  int* cursor = smem + num_slots + 1;    // [num_slots + 1]
  __shared__ int s_unsorted, s_status;

  SegHeader* hdr = reinterpret_cast<SegHeader*>(table);
  const SegLayout lay = seg_layout(M, num_slots);
  int* perm = reinterpret_cast<int*>(table + lay.perm);
  int* slot_of = reinterpret_cast<int*>(table + lay.slot_of);
  int* block_begin = reinterpret_cast<int*>(table + lay.block_begin);
  Window* windows = reinterpret_cast<Window*>(table + lay.windows);

  const int tid = threadIdx.x;
  for (int i = tid; i <= num_slots; i += blockDim.x) counts[i] = 0;
  if (tid == 0) { s_unsorted = 0; s_status = 0; }
  __syncthreads();

  for (int i = tid; i < M; i += blockDim.x) {
    int s = load_index(indices, dtype, i);
    if (s >= num_slots) { s_status = DZ_ERR_SLOT_RANGE; s = -1; }
    if (s < -1) s = -1;
    if (i > 0) {
      int p = load_index(indices, dtype, i - 1);
      if (p >= num_slots || p < -1) p = -1;
      if (p > s) s_unsorted = 1;
    }
    atomicAdd(&counts[s + 1], 1);
  }
  __syncthreads();

  if (tid == 0) {
    int run = 0, active = 0;
    for (int b = 0; b <= num_slots; ++b) {
      int c = counts[b];
      cursor[b] = run;
      if (b > 0 && c > 0) ++active;
      run += c;
    }
    hdr->M = M;
    hdr->capacity_M = M;
    hdr->num_slots = num_slots;
    hdr->num_token_blocks = (M + kTokenBlock - 1) / kTokenBlock;
    hdr->sorted = s_unsorted ? 0 : 1;
    hdr->status = s_status;
    hdr->num_active = active;

    // windows, in ascending sorted position (hence grouped by token block)
    const int nb = hdr->num_token_blocks;
    int nw = 0, next_block = 0;
    for (int b = 1; b <= num_slots; ++b) {
      int s0 = cursor[b], e0 = s0 + counts[b];
      while (s0 < e0) {
        const int tb = s0 / kTokenBlock;
        const int pe = min(e0, (tb + 1) * kTokenBlock);  // piece [s0, pe) inside block tb
        while (next_block <= tb) block_begin[next_block++] = nw;
        int c0 = s0 & ~15;
        const int c1 = (pe + 15) & ~15;
        while (c0 < c1) {
          const int nc = min(kMaxWindowCols, c1 - c0);
          Window w;
          w.slot = b - 1;
          w.col0 = c0;
          w.ncols = nc;
          w.lo = max(s0, c0);
          w.hi = min(pe, c0 + nc);
          w.pad[0] = w.pad[1] = w.pad[2] = 0;
          windows[nw++] = w;
          c0 += nc;
        }
        s0 = pe;
      }
    }
    while (next_block <= nb) block_begin[next_block++] = nw;
    hdr->num_windows = nw;
  }
  __syncthreads();

  const bool sorted = (s_unsorted == 0);
  for (int i = tid; i < M; i += blockDim.x) {
    int s = load_index(indices, dtype, i);
    if (s >= num_slots || s < -1) s = -1;
    int pos = sorted ? i : atomicAdd(&cursor[s + 1], 1);
    perm[pos] = i;
    slot_of[pos] = s;
  }
}

}  // namespace

int launch_build_segments(const void* indices, int index_dtype, int M, int num_slots,
                          void* segments, cudaStream_t st) {
  // The table's array offsets depend on M; the header records it (capacity_M)
  // so that readers and the builder agree.
  size_t smem = (size_t)(num_slots + 1) * 2 * sizeof(int);
  build_segments_kernel<<<1, 1024, smem, st>>>(indices, index_dtype, M, num_slots,
                                               (uint8_t*)segments);
  DZ_CUDA_OK(cudaGetLastError());
  return DZ_OK;
}

}  // namespace dz

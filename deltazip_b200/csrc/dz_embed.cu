// Per-delta embedding lookup: y[i] = table_{slot(i)}[token(i)], where slot -1 selects the
// base table.  The reference replaces (not adds) the embedding per delta in a Python loop
// over the distinct ids (serving/vllm/delta/deltazip_marlin.py:56-86); here it is one gather
// kernel, 16 bytes per thread, bound by HBM/L2 on a few hundred KB.
#include "dz_common.cuh"

namespace dz {
namespace {

__global__ void delta_embedding_kernel(const long long* __restrict__ tokens,
                                       const void* __restrict__ indices, int index_dtype, int M,
                                       int row_vec, const uint4* __restrict__ base_table,
                                       const uint8_t* __restrict__ delta_tables,
                                       long long table_stride, int num_slots, long long vocab,
                                       uint4* __restrict__ y, int* status) {
  const int i = blockIdx.x;
  if (i >= M) return;
  long long slot = (index_dtype == DZ_INDEX_I64) ? reinterpret_cast<const long long*>(indices)[i]
                                                 : (long long)reinterpret_cast<const int*>(indices)[i];
  if (slot >= num_slots) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, (int)DZ_ERR_SLOT_RANGE);
    slot = -1;
  }
  long long tok = tokens[i];
  if (tok < 0 || tok >= vocab) {   // out-of-vocabulary id: zero row, flagged
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, (int)DZ_ERR_INVALID_ARG);
    for (int c = threadIdx.x; c < row_vec; c += blockDim.x) y[(size_t)i * row_vec + c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* table = slot < 0 ? base_table
                                : reinterpret_cast<const uint4*>(delta_tables + slot * table_stride);
  const uint4* src = table + (size_t)tok * row_vec;
  for (int c = threadIdx.x; c < row_vec; c += blockDim.x) y[(size_t)i * row_vec + c] = src[c];
}

}  // namespace
}  // namespace dz

using namespace dz;

extern "C" int dz_delta_embedding(const int64_t* token_ids, const void* indices, int index_dtype,
                                  int M, int hidden, const void* base_table,
                                  const void* delta_tables, int64_t table_stride_bytes,
                                  int num_slots, int64_t vocab, void* y, int* status_word,
                                  void* stream) {
  if (M < 0 || hidden <= 0 || vocab <= 0 || num_slots < 0) return DZ_ERR_INVALID_ARG;
  if (M == 0) return DZ_OK;
  if (!token_ids || !indices || !base_table || !y || (num_slots > 0 && !delta_tables))
    return DZ_ERR_INVALID_ARG;
  if (index_dtype != DZ_INDEX_I32 && index_dtype != DZ_INDEX_I64) return DZ_ERR_INVALID_ARG;
  if (hidden % 8 != 0) return DZ_ERR_SHAPE;   // rows are moved 16 bytes at a time (2-byte elements)
  if (!aligned16(base_table) || !aligned16(y) || (delta_tables && !aligned16(delta_tables)) ||
      (table_stride_bytes & 15))
    return DZ_ERR_ALIGNMENT;
  delta_embedding_kernel<<<M, 128, 0, (cudaStream_t)stream>>>(
      (const long long*)token_ids, indices, index_dtype, M, hidden / 8, (const uint4*)base_table,
      (const uint8_t*)delta_tables, table_stride_bytes, num_slots, vocab, (uint4*)y, status_word);
  DZ_CUDA_OK(cudaGetLastError());
  return DZ_OK;
}

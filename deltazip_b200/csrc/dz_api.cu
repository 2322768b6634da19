// The C ABI: argument validation and dispatch to the kernel launchers.
#include <stdio.h>
#include <string.h>

#include "dz_common.cuh"

namespace dz {

static thread_local char g_cuda_error[256] = "";

void set_last_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", where, cudaGetErrorString(e));
}

int launch_sbmm_simt(const dz_sbmm_args& a, bool base_only, cudaStream_t st);

// An empty kernel launched the ordinary way: it starts only after everything before it in the
// stream has completed with its writes visible, so a later kernel that begins early under
// programmatic dependent launch overlaps at most this kernel, never the writers before it.
__global__ void stream_fence_kernel() {}
int launch_stream_fence(cudaStream_t st) {
  stream_fence_kernel<<<1, 32, 0, st>>>();
  DZ_CUDA_OK(cudaGetLastError());
  return DZ_OK;
}

static int check_shape(int N, int K, int bits) {
  if (N <= 0 || K <= 0) return DZ_ERR_INVALID_ARG;
  if (N % kTileN != 0 || K % kBlockK != 0) return DZ_ERR_SHAPE;
  if (bits != 2 && bits != 4) return DZ_ERR_SHAPE;
  return DZ_OK;
}

int check_sbmm_args(const dz_sbmm_args* a, bool base_only, bool check_workspace) {
  if (!a) return DZ_ERR_INVALID_ARG;
  if (a->M < 0) return DZ_ERR_INVALID_ARG;
  if (a->M == 0) return DZ_OK;  // nothing to do; pointers may be null
  // w_base may be absent for dz_sbmm: only the delta products are then computed
  if (!a->x || (!a->y && !a->push) || (base_only && !a->w_base)) return DZ_ERR_INVALID_ARG;
  if (a->push) {
    if (a->push->world < 2 || a->push->world > 8 || (a->flags & DZ_SBMM_ACCUMULATE))
      return DZ_ERR_INVALID_ARG;
    if ((size_t)((a->M + 127) / 128) * (size_t)(a->N / 128) > DZ_PUSH_MAX_FLAGS) return DZ_ERR_TOO_LARGE;
    for (int r = 0; r < a->push->world; ++r)
      if (!a->push->data[r] || !a->push->flags[r]) return DZ_ERR_INVALID_ARG;
  }
  int rc = check_shape(a->N, a->K, base_only ? 4 : a->bits);
  if (rc) return rc;
  if (a->dtype != DZ_DTYPE_F16 && a->dtype != DZ_DTYPE_BF16) return DZ_ERR_INVALID_ARG;
  if (!aligned16(a->x) || !aligned16(a->w_base) || (!a->push && !aligned16(a->y))) return DZ_ERR_ALIGNMENT;
  if (!base_only) {
    if (!a->qweight || !a->meta || !a->scales || !a->segments) return DZ_ERR_INVALID_ARG;
    if (a->num_slots <= 0 || a->num_slots > kMaxSlots) return DZ_ERR_INVALID_ARG;
    if (!aligned16(a->qweight) || !aligned16(a->meta) || (a->qweight_stride & 15) ||
        (a->meta_stride & 15) || (a->scales_stride & 1))
      return DZ_ERR_ALIGNMENT;
  }
  if (a->flags & ~(int32_t)(DZ_SBMM_ACCUMULATE | DZ_SBMM_INPUTS_STABLE)) return DZ_ERR_INVALID_ARG;
  if (a->y_stride != 0 && (a->y_stride < a->N || (a->y_stride & 7))) return DZ_ERR_INVALID_ARG;
  if (!check_workspace) return DZ_OK;
  if (a->workspace_bytes <
      sbmm_workspace_bytes(a->M, a->N, a->K, base_only ? 1 : a->tokens_sorted))
    return DZ_ERR_WORKSPACE;
  if (a->workspace_bytes && (!a->workspace || !aligned16(a->workspace))) return DZ_ERR_ALIGNMENT;
  return DZ_OK;
}

}  // namespace dz

using namespace dz;

extern "C" {

int dz_version(void) { return 100; }

const char* dz_status_string(int s) {
  switch (s) {
    case DZ_OK: return "ok";
    case DZ_ERR_INVALID_ARG: return "invalid argument";
    case DZ_ERR_SHAPE: return "unsupported shape (need N % 128 == 0, K % 64 == 0, bits in {2,4})";
    case DZ_ERR_ALIGNMENT: return "pointer or stride not 16-byte aligned";
    case DZ_ERR_WORKSPACE: return "workspace too small";
    case DZ_ERR_SLOT_RANGE: return "delta index out of range";
    case DZ_ERR_NOT_2_4: return "weights are not 2:4 sparse";
    case DZ_ERR_NOT_SYMMETRIC: return "zero-point is not the symmetric one";
    case DZ_ERR_CUDA: return "CUDA call failed";
    case DZ_ERR_TIMEOUT: return "device-side wait timed out";
    case DZ_ERR_UNSUPPORTED: return "not implemented in this build";
    case DZ_ERR_TOO_LARGE: return "size beyond the entry point's fixed maximum";
    default: return "unknown status";
  }
}

const char* dz_last_cuda_error(void) { return g_cuda_error; }

size_t dz_slot_qweight_bytes(int N, int K, int bits) {
  if (check_shape(N, K, bits)) return 0;
  return (size_t)N * K * bits / 16;  // K/2 kept values per row, bits each
}
size_t dz_slot_meta_bytes(int N, int K) {
  if (check_shape(N, K, 4)) return 0;
  return (size_t)N * K / 8;  // 4 bits per group of four
}
size_t dz_slot_scales_bytes(int N) { return N > 0 ? (size_t)N * 2 : 0; }

int dz_convert_from_gptq(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                         int N, int K, int bits, void* slot_qweight, void* slot_meta,
                         uint16_t* slot_scales, int* status_word, void* stream) {
  if (!qweight || !qzeros || !scales || !slot_qweight || !slot_meta || !slot_scales)
    return DZ_ERR_INVALID_ARG;
  int rc = check_shape(N, K, bits);
  if (rc) return rc;
  if (!aligned16(slot_qweight) || !aligned16(slot_meta)) return DZ_ERR_ALIGNMENT;
  rc = launch_convert_from_gptq(qweight, qzeros, scales, N, K, bits, slot_qweight, slot_meta,
                                slot_scales, status_word, (cudaStream_t)stream);
  return rc ? rc : launch_stream_fence((cudaStream_t)stream);
}

int dz_unpack(const void* slot_qweight, const void* slot_meta, const uint16_t* slot_scales, int N,
              int K, int bits, uint16_t* delta_out, void* stream) {
  if (!slot_qweight || !slot_meta || !slot_scales || !delta_out) return DZ_ERR_INVALID_ARG;
  int rc = check_shape(N, K, bits);
  if (rc) return rc;
  if (!aligned16(slot_qweight) || !aligned16(slot_meta) || !aligned16(delta_out))
    return DZ_ERR_ALIGNMENT;
  return launch_unpack(slot_qweight, slot_meta, slot_scales, N, K, bits, delta_out,
                       (cudaStream_t)stream);
}

size_t dz_segments_bytes(int M, int num_slots) {
  if (M < 0 || num_slots < 0) return 0;
  return seg_layout(M, num_slots).total;
}

int dz_build_segments(const void* indices, int index_dtype, int M, int num_slots, void* segments,
                      void* stream) {
  if (!segments || (M > 0 && !indices)) return DZ_ERR_INVALID_ARG;
  if (M < 0 || num_slots < 0 || num_slots > kMaxSlots) return DZ_ERR_INVALID_ARG;
  if (index_dtype != DZ_INDEX_I32 && index_dtype != DZ_INDEX_I64) return DZ_ERR_INVALID_ARG;
  if (!aligned16(segments)) return DZ_ERR_ALIGNMENT;
  int rc = launch_build_segments(indices, index_dtype, M, num_slots, segments, (cudaStream_t)stream);
  return rc ? rc : launch_stream_fence((cudaStream_t)stream);
}

size_t dz_sbmm_workspace_bytes(int M, int N, int K, int tokens_sorted) {
  return sbmm_workspace_bytes(M, N, K, tokens_sorted);
}

int dz_sbmm(const dz_sbmm_args* args, void* stream) {
  int rc = check_sbmm_args(args, false, true);
  if (rc || args->M == 0) return rc;
  return launch_sbmm(*args, false, (cudaStream_t)stream);
}

int dz_base_gemm(const dz_sbmm_args* args, void* stream) {
  int rc = check_sbmm_args(args, true, true);
  if (rc || args->M == 0) return rc;
  return launch_sbmm(*args, true, (cudaStream_t)stream);
}

// Validation twin of dz_sbmm on CUDA cores (same arguments, no workspace use).
int dz_sbmm_simt(const dz_sbmm_args* args, void* stream) {
  int rc = check_sbmm_args(args, false, true);
  if (rc || args->M == 0) return rc;
  if (args->dtype != DZ_DTYPE_F16) return DZ_ERR_UNSUPPORTED;   // the twin is fp16 only
  if (args->push || (args->flags & DZ_SBMM_ACCUMULATE) || (args->y_stride && args->y_stride != args->N) || !args->w_base)
    return DZ_ERR_UNSUPPORTED;                                   // plain y = base + delta only
  return launch_sbmm_simt(*args, false, (cudaStream_t)stream);
}

int dz_slot_upload(void* dst_device, const void* src_pinned_host, size_t bytes, int zero_first,
                   void* copy_stream) {
  if (!dst_device || (!src_pinned_host && bytes)) return DZ_ERR_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)copy_stream;
  if (bytes == 0) return DZ_OK;
  if (zero_first) DZ_CUDA_OK(cudaMemsetAsync(dst_device, 0, bytes, st));
  DZ_CUDA_OK(cudaMemcpyAsync(dst_device, src_pinned_host, bytes, cudaMemcpyHostToDevice, st));
  return DZ_OK;
}

int dz_slot_reset(void* dst_device, size_t bytes, void* stream) {
  if (!dst_device) return DZ_ERR_INVALID_ARG;
  if (bytes) {
    DZ_CUDA_OK(cudaMemsetAsync(dst_device, 0, bytes, (cudaStream_t)stream));
    return launch_stream_fence((cudaStream_t)stream);
  }
  return DZ_OK;
}

int dz_stream_fence(void* stream) { return launch_stream_fence((cudaStream_t)stream); }

int dz_read_status(int* status_word, void* stream, int* host_out) {
  if (!status_word || !host_out) return DZ_ERR_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  DZ_CUDA_OK(cudaMemcpyAsync(host_out, status_word, sizeof(int), cudaMemcpyDeviceToHost, st));
  DZ_CUDA_OK(cudaMemsetAsync(status_word, 0, sizeof(int), st));
  DZ_CUDA_OK(cudaStreamSynchronize(st));
  return DZ_OK;
}

}  // extern "C"

/*
 * deltazip_b200 -- C ABI of the B200-native selective batched matmul (SBMM) path.
 *
 * Plain C: pointers and sizes only.  All data pointers are CUDA device pointers
 * unless a parameter says "host".  `stream` is a cudaStream_t passed as void*
 * (NULL = the legacy default stream).  Every entry point returns a dz_status
 * (0 = ok) and never exits, traps or synchronises the device unless it says so.
 * Nothing here allocates device memory on the hot path: the caller supplies a
 * workspace of dz_sbmm_workspace_bytes().
 *
 * Each declaration cites the piece of the reference (eth-easl/deltazip, paths
 * relative to its checkout) whose role it takes over.
 */
#ifndef DELTAZIP_B200_H_
#define DELTAZIP_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  DZ_OK = 0,
  DZ_ERR_INVALID_ARG = 1,   /* null pointer, negative size, bad enum            */
  DZ_ERR_SHAPE = 2,         /* N % 128 != 0, K % 64 != 0, unsupported bits      */
  DZ_ERR_ALIGNMENT = 3,     /* pointer / stride not 16-byte aligned             */
  DZ_ERR_WORKSPACE = 4,     /* workspace too small                              */
  DZ_ERR_SLOT_RANGE = 5,    /* a delta index >= num_slots                       */
  DZ_ERR_NOT_2_4 = 6,       /* converter: a group of 4 holds more than 2 codes
                               different from the zero-point                    */
  DZ_ERR_NOT_SYMMETRIC = 7, /* converter: a stored zero-point != 2^(bits-1) - 1 */
  DZ_ERR_CUDA = 8,          /* a CUDA runtime / driver call failed              */
  DZ_ERR_TIMEOUT = 9,       /* a bounded device-side wait ran out               */
  DZ_ERR_UNSUPPORTED = 10,  /* valid request this build does not implement      */
  DZ_ERR_TOO_LARGE = 11     /* size beyond a fixed maximum of the entry point   */
} dz_status;

enum { DZ_DTYPE_F16 = 0, DZ_DTYPE_BF16 = 1, DZ_DTYPE_F32 = 2 /* all-reduce only */ };
enum { DZ_INDEX_I32 = 0, DZ_INDEX_I64 = 1 };

/* Library version (major*10000 + minor*100 + patch). */
int dz_version(void);
/* Static, human readable text for a dz_status. */
const char* dz_status_string(int status);
/* Text of the last CUDA error this thread's calls into the library met ("" if none). */
const char* dz_last_cuda_error(void);

/* ------------------------------------------------------------------------
 * Slot format.  One delta of one linear layer [N out, K in] occupies three
 * device arrays whose names, dtypes and outer shapes are those the reference's
 * delta layers allocate (serving/vllm/delta/layers_marlin.py:311-333,407-429,
 * 510-534):
 *   qweight int32 [K*bits/128, 2N]   codes of the K/2 kept values of every row
 *   meta    int16 [N, K/16]          2:4 positions (two 2-bit indices / group)
 *   scales  fp16  [1, N]             per-output-channel scale
 * The element order inside qweight / meta is this library's own (tile-major,
 * see dz_convert_from_gptq); the reference's order is that of an external
 * package whose source it does not ship.
 * ------------------------------------------------------------------------ */
size_t dz_slot_qweight_bytes(int N, int K, int bits);
size_t dz_slot_meta_bytes(int N, int K);
size_t dz_slot_scales_bytes(int N);

/*
 * GPTQ layout -> slot layout, on the device.
 * Takes the tensors deltazip/nn_modules/qlinear.py:83-183 (QuantLinear.pack)
 * writes: qweight int32 [K*bits/32, N], qzeros int32 [1, N*bits/32], scales
 * fp16 [1, N]; fills the role of deltazip/utils/converter.py:12-101, which hands
 * the same tensors to an external packer.  bits in {2, 4}.
 * `status_word` (device int, may be NULL) receives the first DZ_ERR_NOT_2_4 /
 * DZ_ERR_NOT_SYMMETRIC found; the call itself is asynchronous.
 */
int dz_convert_from_gptq(const int32_t* qweight, const int32_t* qzeros,
                         const uint16_t* scales, int N, int K, int bits,
                         void* slot_qweight, void* slot_meta, uint16_t* slot_scales,
                         int* status_word, void* stream);

/*
 * Slot layout -> dense delta, fp16 [N, K] row-major; bit-identical to
 * QuantLinear.unpack (deltazip/nn_modules/qlinear.py:185-264) of the GPTQ
 * tensors the slot was converted from.
 */
int dz_unpack(const void* slot_qweight, const void* slot_meta, const uint16_t* slot_scales,
              int N, int K, int bits, uint16_t* delta_out, void* stream);

/*
 * Batch metadata.  Turns the per-token slot ids (`indices`, the `base_indices`
 * tensor of serving/vllm/delta/models.py:69-145, -1 = base model only) into the
 * segment table the SBMM kernel walks.  Build once per scheduling step and share
 * across all layers, as the reference shares its index buffers
 * (serving/vllm/delta/models.py:407-430).  `segments` must hold
 * dz_segments_bytes(M_max, num_slots) bytes.  Indices >= num_slots set
 * DZ_ERR_SLOT_RANGE in the table's status field and are treated as -1.
 */
size_t dz_segments_bytes(int M, int num_slots);
int dz_build_segments(const void* indices, int index_dtype, int M, int num_slots,
                      void* segments, void* stream);

/*
 * The hot path:  y[i] = x[i] W^T + x[i] dequant(delta_{indices[i]})^T.
 * Replaces apply_delta (serving/vllm/delta/deltazip_marlin.py:10-19), i.e. the
 * external sbmm_4bit_2_4_native(qweight_stacked, x, meta_stacked, scales_stacked,
 * indices, base_weight), and the separate base GEMM
 * (serving/vllm/model_executor/layers/linear.py:85-96).
 */
/* Where a row-parallel SBMM sends its partial output when it is fused with the all-reduce
 * that follows (filled by dz_allreduce_push_target, see there). */
#define DZ_PUSH_MAX_FLAGS 256
typedef struct {
  int32_t world, rank;
  uint32_t epoch;           /* value the per-tile flags are raised to                  */
  uint32_t reserved;
  void* data[8];            /* rank r's receive slot for this rank's [M, N] partial     */
  void* flags[8];           /* rank r's flag row for this rank (uint32 per tile)        */
} dz_push_target;

typedef struct {
  const void* x;            /* [M, K] row-major, 16-byte aligned                 */
  const void* w_base;       /* [N, K] row-major, 16-byte aligned; NULL for dz_sbmm:
                               y = x dequant(delta)^T only (rows of slot -1 get 0),
                               the product the reference's GPTQ-layout ops add to a
                               separately computed base output
                               (serving/vllm/delta/deltazip.py:14-153)             */
  const void* qweight;      /* slot 0 of the qweight stack                       */
  const void* meta;         /* slot 0 of the meta stack                          */
  const void* scales;       /* slot 0 of the scales stack                        */
  int64_t qweight_stride;   /* bytes between consecutive slots                   */
  int64_t meta_stride;
  int64_t scales_stride;
  const void* segments;     /* table from dz_build_segments for this batch       */
  void* y;                  /* [M, N] row-major                                  */
  int32_t M, N, K;
  int32_t num_slots;
  int32_t bits;             /* 2 or 4 (all slots of a stack share it)            */
  int32_t dtype;            /* DZ_DTYPE_* of x, w_base and y                     */
  int32_t tokens_sorted;    /* 1: caller guarantees `indices` were non-decreasing
                               (the reference's scheduler sorts each batch by
                               delta id, serving/vllm/core/scheduler.py:101-104);
                               x is then read in place.  0: no promise -- x is
                               first gathered into sorted order inside the
                               workspace (a plain copy when the batch happens to
                               be sorted); no host synchronisation either way.
                               A wrong promise is detected (DZ_ERR_INVALID_ARG in
                               the workspace status word) and nothing is computed. */
  int32_t flags;            /* DZ_SBMM_* bits, 0 = none                          */
  void* workspace;          /* >= dz_sbmm_workspace_bytes(M, N, K, tokens_sorted);
                               zero-filled once by the caller before first use;
                               its first int is a status word (dz_read_status)  */
  size_t workspace_bytes;
  int64_t y_stride;         /* elements between consecutive rows of y; 0 = N.
                               With a stride > N the call writes the columns
                               [0, N) of a wider output, i.e. one slice of a
                               merged layer (add_delta_slice,
                               serving/vllm/delta/deltazip.py:41-78)             */
  const dz_push_target* push; /* host pointer or NULL.  Non-NULL (row-parallel layer under
                               tensor parallelism): instead of writing y, the epilogue
                               stores every finished output tile into the receive slot
                               of every rank and raises the tile's flag there;
                               dz_allreduce_run_pushed then produces the reduced
                               [M, N].  y and y_stride are ignored, DZ_SBMM_ACCUMULATE
                               is not allowed                                      */
} dz_sbmm_args;

/* flags of dz_sbmm_args */
enum {
  DZ_SBMM_ACCUMULATE = 1,   /* y += result instead of y = result: the in-place form
                               of the reference's GPTQ-layout ops (add_delta,
                               serving/vllm/delta/deltazip.py:14-38); the sum is
                               formed in fp32 and rounded once                    */
  DZ_SBMM_INPUTS_STABLE = 2 /* the caller states that w_base, the slot stacks and the
                               segment table were NOT written by the operation that
                               immediately precedes this call in the stream (true for
                               every layer call of a decode step: weights are static
                               and the table is built once per step).  The kernel then
                               loads them while its predecessor is still finishing and
                               waits for the predecessor only before it touches x.
                               Tables built by dz_build_segments and slots written by
                               dz_convert_from_gptq / dz_slot_reset always qualify
                               (those calls end with a stream fence); after other
                               writers (e.g. a framework's copy kernel) call
                               dz_stream_fence first or leave the flag off            */
};

size_t dz_sbmm_workspace_bytes(int M, int N, int K, int tokens_sorted);
int dz_sbmm(const dz_sbmm_args* args, void* stream);

/*
 * dz_sbmm for callers that cannot allocate device memory (no counterpart in the
 * reference, which allocates freely through PyTorch).  Same arguments and
 * results as dz_sbmm (w_base may be NULL, flags and y_stride are honoured), but
 * `workspace` / `workspace_bytes` are ignored: the scratch lives in a fixed
 * array inside the library, so the call makes no cudaMalloc / cudaFree and
 * calls no allocating routine.  Limits: M <= dz_sbmm_static_max_tokens() (64)
 * and tokens_sorted must be 1, otherwise DZ_ERR_TOO_LARGE.  Each GPU that loads
 * the library holds about 10.5 MB for this array until the process exits.  The
 * first call on a device looks up the array's device address (make it before
 * any stream capture).  All calls on a device share the array: calls that
 * overlap on the GPU race -- order them.
 *
 * Device-side findings (DZ_ERR_INVALID_ARG: a wrong tokens_sorted promise or a
 * segment table built for another M / num_slots, in which case the kernel
 * computes nothing and y is left as it was; DZ_ERR_TIMEOUT: a bounded wait ran
 * out) land in a status word inside the array.  It stays set until
 * dz_sbmm_static_status reads and clears it (synchronises `stream`; allocates
 * nothing either).
 */
int dz_sbmm_static(const dz_sbmm_args* args, void* stream);
int dz_sbmm_static_max_tokens(void);
int dz_sbmm_static_status(void* stream, int* host_out);

/* Base GEMM alone, y = x W^T (all tokens -1); same argument block, the slot
 * pointers and `segments` may be NULL.
 * serving/vllm/model_executor/layers/linear.py:85-96 */
int dz_base_gemm(const dz_sbmm_args* args, void* stream);

/*
 * Per-delta embedding: y[i] = table_{indices[i]}[token_ids[i]] (2-byte elements, `hidden`
 * per row), indices[i] == -1 selects `base_table`; the delta tables are full replacement
 * tables stacked `table_stride_bytes` apart.  Replaces apply_delta_embed
 * (serving/vllm/delta/deltazip_marlin.py:56-86).  Token ids outside [0, vocab) give a
 * zero row and DZ_ERR_INVALID_ARG in `status_word` (device int, may be NULL).
 */
int dz_delta_embedding(const int64_t* token_ids, const void* indices, int index_dtype, int M,
                       int hidden, const void* base_table, const void* delta_tables,
                       int64_t table_stride_bytes, int num_slots, int64_t vocab, void* y,
                       int* status_word, void* stream);

/*
 * Layers with a full replacement matrix per delta (the output matrix / lm_head):
 *   y[i] = x[i] T^T with T = base_matrix [V, K] for tokens of slot -1 and delta_matrices[slot]
 *   (a dense stack [num_slots, V, K], matrix_stride_bytes = V*K*2) otherwise.
 * One launch per 128 tokens serves all groups present in the batch; every present matrix is
 * streamed once, matrices of slots without tokens are not read, nothing synchronises with the
 * host.  `segments` is the batch's table (dz_build_segments over the per-row slot ids),
 * tokens_sorted as for dz_sbmm, y [M, V] (rows y_stride elements apart, 0 = V).  V % 128 == 0,
 * K % 64 == 0.  `workspace` >= dz_grouped_gemm_workspace_bytes(), zero-filled once; its first
 * int is a status word (dz_read_status).  Replaces apply_delta_uncompressed
 * (serving/vllm/delta/deltazip_marlin.py:21-53), which loops over the distinct ids on the host.
 */
size_t dz_grouped_gemm_workspace_bytes(int M, int K, int tokens_sorted);
int dz_grouped_gemm(const void* x, const void* base_matrix, const void* delta_matrices,
                    int64_t matrix_stride_bytes, const void* segments, void* y, int M, int V, int K,
                    int num_slots, int dtype, int tokens_sorted, int64_t y_stride, void* workspace,
                    size_t workspace_bytes, void* stream);

/*
 * The steps between the SBMM calls of a decoder layer at decode time, so that a decode step is a
 * chain of this library's launches.  2-byte elements of `dtype`; 16-byte aligned pointers; all
 * enqueue one kernel on `stream` and return.
 *
 * dz_rms_norm: residual == NULL: out = rmsnorm(x) * weight.  residual != NULL: residual = x +
 *   residual, out = rmsnorm(residual) * weight (out may alias x).  x, out, residual [M, hidden],
 *   hidden % 8 == 0, hidden <= 16384.  serving/csrc/ops.h:37-47 (rms_norm, fused_add_rms_norm),
 *   semantics of serving/vllm/model_executor/layers/layernorm.py:27-66.
 * dz_silu_and_mul: out[m, i] = silu(x[m, i]) * x[m, inter + i]; x [M, 2*inter], out [M, inter].
 *   serving/csrc/ops.h:67.
 * dz_rotary_and_cache: rotary position embedding (neox pairing, base `rope_theta`) in place on
 *   the q and k heads of the fused rows qkv [M, (q_heads + 2*kv_heads) * 128], then k (rotated)
 *   and v written to the paged cache at slot_mapping[token] = block * block_size + offset
 *   (negative or slot_mapping == NULL: not cached).  Cache layout: [slots, kv_heads, 128] for K
 *   and for V.  head_dim must be 128.  serving/csrc/ops.h:49 + serving/csrc/cache.h:18.
 * dz_paged_attention_decode: one query token per sequence against its cached keys/values:
 *   out [num_seqs, q_heads * 128]; q is read from the fused rows (q_row_stride elements apart, a
 *   multiple of 8); q_heads / kv_heads must be 1, 2, 4 or 8;
 *   block_tables int32 [num_seqs, max_blocks]; seq_lens int32 [num_seqs] (cached tokens,
 *   the current one included).  splits > 1 divides every sequence's keys over that many CTAs
 *   (for few long sequences) and needs `workspace` of dz_paged_attention_workspace_bytes(),
 *   zero-filled once.  serving/csrc/ops.h:6 (paged_attention_v1).
 */
int dz_rms_norm(const void* x, void* residual, const void* weight, void* out, int M, int hidden,
                float eps, int dtype, void* stream);
int dz_silu_and_mul(const void* x, void* out, int M, int inter, int dtype, void* stream);
int dz_rotary_and_cache(void* qkv, const int64_t* positions, const int64_t* slot_mapping,
                        void* k_cache, void* v_cache, int M, int q_heads, int kv_heads,
                        int head_dim, float rope_theta, int dtype, void* stream);
size_t dz_paged_attention_workspace_bytes(int num_seqs, int q_heads, int kv_heads, int splits);
int dz_paged_attention_decode(const void* qkv, int q_row_stride, void* out, const void* k_cache,
                              const void* v_cache, const int32_t* block_tables, int max_blocks,
                              const int32_t* seq_lens, int num_seqs, int q_heads, int kv_heads,
                              int head_dim, int block_size, float scale, int splits,
                              void* workspace, size_t workspace_bytes, int dtype, void* stream);

/*
 * Compression on the device (float32 in, the reference's arithmetic operation by operation).
 *
 * dz_quant_find_params: per-row symmetric grid of W [N, K]: scale[n], zero[n] = 2^(bits-1)
 *   (Quantizer.find_params, deltazip/core/quant.py:48-86, per channel, symmetric).
 * dz_sparsegpt_block: one block of <= 128 columns of SparseGPT.fasterprune with 2:4 pruning
 *   (deltazip/core/sparsegpt.py:98-146): W_block points at column i1 of the current W (row
 *   stride ldw), hinv_block at element (i1, i1) of the upper Cholesky factor of H^-1 (row stride
 *   ldh).  Writes Q [N, count] (pruned + quantised block) and Err [N, count] ((w - q) / Hinv_ii)
 *   and adds every row's loss to loss[n] (may be NULL).  The caller copies Q into W and applies
 *   W[:, i2:] -= Err @ Hinv[i1:i2, i2:] before the next block.  count % 4 == 0.
 * dz_pack_gptq: QuantLinear.pack (deltazip/nn_modules/qlinear.py:83-183, one group) of the
 *   quantised W [N, K]: qweight int32 [K*bits/32, N], qzeros int32 [1, N*bits/32], scales fp16
 *   [1, N] -- the tensors the reference stores and dz_convert_from_gptq reads.
 */
int dz_quant_find_params(const float* W, int N, int K, int bits, float* scale, float* zero, void* stream);
int dz_sparsegpt_block(const float* W_block, int64_t ldw, const float* hinv_block, int64_t ldh,
                       const float* scale, const float* zero, int bits, int N, int count, float* Q,
                       float* Err, float* loss, void* stream);
int dz_pack_gptq(const float* Wq, const float* scale, const float* zero, int N, int K, int bits,
                 int32_t* qweight, int32_t* qzeros, uint16_t* scales, void* stream);

/*
 * Delta swap-in: one asynchronous host->device copy of a delta's slot bytes
 * from PINNED host memory on `copy_stream`, preceded by a zero fill of the
 * destination when `zero_first` != 0 (the reference resets a slot before it
 * overwrites it, serving/vllm/delta/layers_marlin.py:342-360).  Returns without
 * waiting; record / wait on an event in `copy_stream` to publish the slot.
 */
int dz_slot_upload(void* dst_device, const void* src_pinned_host, size_t bytes,
                   int zero_first, void* copy_stream);
int dz_slot_reset(void* dst_device, size_t bytes, void* stream);

/*
 * All-reduce (sum) of the row-parallel layers' partial outputs over peer memory,
 * one process per GPU on one node.  Replaces the reference's CustomAllreduce
 * (serving/vllm/model_executor/parallel_utils/custom_all_reduce.py:187-262,
 * serving/csrc/custom_all_reduce.cuh; called from communication_op.py:17-40
 * after serving/vllm/delta/layers_marlin.py:583-584).
 *
 *   create   allocates this rank's region (flags + two staging buffers) with
 *            cudaMalloc -- set-up time, never on the hot path;
 *   export   writes the region's 64-byte CUDA IPC handle; the caller exchanges
 *            the handles of all ranks by any means (torch.distributed here);
 *   connect  takes world * 64 bytes of handles in rank order and maps the peers;
 *   staging  returns where the NEXT run's input may be produced in place (the
 *            row-parallel SBMM writes y there, which saves the copy-in);
 *   run      enqueues one kernel on `stream`: out = sum over ranks of in, fp32
 *            accumulation in rank order (bit-identical on every rank); count
 *            elements of DZ_DTYPE_*, count * size <= max_bytes and a multiple
 *            of 16, pointers 16-byte aligned; `out` may be any device buffer.
 *            Every rank must issue the same sequence of runs.  Not capturable
 *            into a CUDA graph (the call's epoch is a kernel argument).
 *   status   reads the region's status word: DZ_ERR_TIMEOUT when a peer's data
 *            did not arrive within one second (the kernel then returns without
 *            reducing instead of waiting forever).
 */
typedef struct dz_allreduce_ctx dz_allreduce_ctx;
size_t dz_allreduce_region_bytes(size_t max_bytes);
int dz_allreduce_create(dz_allreduce_ctx** ctx, int rank, int world, size_t max_bytes);
/* Same context over regions the CALLER allocated, one per rank, each dz_allreduce_region_bytes()
 * large, 256-byte aligned, peer-accessible from this rank (regions[r] = this process's address of
 * rank r's region), with their first 16 KB zero-filled on every rank before any run -- e.g.
 * symmetric memory.  `multicast_region` (may be NULL) is the address under which one access
 * reaches all ranks' regions through the NVSwitch; with it, variant 3 / 4 of
 * dz_allreduce_set_variant reads sums with multimem.ld_reduce (in-switch reduction).  No export /
 * connect step; destroy leaves the regions alone. */
int dz_allreduce_create_external(dz_allreduce_ctx** ctx, int rank, int world, size_t max_bytes,
                                 void* const* regions, void* multicast_region);
int dz_allreduce_export(dz_allreduce_ctx* ctx, unsigned char* handle64);
int dz_allreduce_connect(dz_allreduce_ctx* ctx, const unsigned char* handles);
int dz_allreduce_staging(dz_allreduce_ctx* ctx, void** ptr, size_t* bytes);
int dz_allreduce_run(dz_allreduce_ctx* ctx, const void* in, void* out, int64_t count,
                     int dtype, void* stream);
int dz_allreduce_status(dz_allreduce_ctx* ctx, int* status);
/*
 * Fused form (producer pushes, consumer sums locally).  For the NEXT reduction of an [M, N]
 * tensor of `dtype` (N % 128 == 0, M*N*2 <= 2 MB): push_target fills the addresses a dz_sbmm
 * call takes in args->push; after that call (the calls of all its token blocks are one call),
 * run_pushed enqueues the kernel that waits for every rank's tiles and writes the sum to `out`
 * (fp32 accumulation in rank order, bit-identical on all ranks).  push_target -> dz_sbmm ->
 * run_pushed must follow each other on one stream, and every rank must issue the same sequence
 * of reductions of either kind.  The role the reference gives to an all-reduce call after the
 * row-parallel layer (serving/vllm/delta/layers_marlin.py:583-584).
 */
int dz_allreduce_push_target(dz_allreduce_ctx* ctx, int M, int N, int dtype, dz_push_target* target);
int dz_allreduce_run_pushed(dz_allreduce_ctx* ctx, void* out, int M, int N, int dtype, void* stream);
/* Kernel choice of later runs: 0 = by message size and rank count (one kernel that sums whole
 * slices for decode-size messages, a reduce-scatter + all-gather kernel for large ones; the
 * reference switches the same way, serving/csrc/custom_all_reduce.cuh:443-456), 1 = always the
 * former, 2 = the latter whenever there are more than two ranks, 3 = always the in-switch kernel
 * (needs a multicast region), 4 = like 0 but with the in-switch kernel for messages of 64 KB and
 * more on more than two ranks.  Every rank must make the same choice. */
int dz_allreduce_set_variant(dz_allreduce_ctx* ctx, int variant);
int dz_allreduce_destroy(dz_allreduce_ctx* ctx);

/* Enqueues an empty kernel: whatever was enqueued before it has completed, with its writes
 * visible, before any later kernel's early (pre-dependency) part can start.  See
 * DZ_SBMM_INPUTS_STABLE. */
int dz_stream_fence(void* stream);

/* Reads and clears a device status word (synchronises `stream`). */
int dz_read_status(int* status_word, void* stream, int* host_out);

#ifdef __cplusplus
}
#endif
#endif /* DELTAZIP_B200_H_ */

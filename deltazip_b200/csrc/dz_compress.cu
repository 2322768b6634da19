// Compressor kernels: the steps of the reference's offline compression that are not plain
// dense linear algebra, for one linear layer's delta W [N, K] (float32):
//
//   sparsegpt_block_kernel   one 128-column block of SparseGPT.fasterprune with prunen:prunem =
//                            2:4 (deltazip/core/sparsegpt.py:98-146): per group of four columns
//                            the two entries with the smallest w^2 / Hinv_ii^2 are pruned, every
//                            entry goes through the symmetric per-row quantiser
//                            (deltazip/core/quant.py:9-18), and the quantisation / pruning error
//                            of column i is fed forward into the block's later columns through
//                            row i of the upper Cholesky factor of H^-1 (:139-141).  Rows of W are
//                            independent, so one warp owns one row: lane l holds columns l, l+32,
//                            l+64, l+96 of the block; the block of Hinv sits in shared memory.
//                            Outputs Q (quantised block) and Err ((w - q) / Hinv_ii per column),
//                            from which the caller forms the update of the columns behind the
//                            block, W[:, i2:] -= Err @ Hinv[i1:i2, i2:] (:146), a plain GEMM.
//   pack_gptq_kernel         QuantLinear.pack (deltazip/nn_modules/qlinear.py:83-183) for one
//                            quantisation group: codes round((W + zero*scale) / fp16(scale))
//                            packed along K into int32 words, zero points (minus one) packed
//                            along N, scales as fp16 -- the GPTQ-layout tensors the reference
//                            stores, bit for bit.
//
// Arithmetic follows the reference's float32 operations one by one (IEEE division, products and
// differences rounded separately, round-half-even), so that results can be compared bit for bit
// with the reference run on the same inputs wherever no long accumulation is involved.
#include "dz_common.cuh"

namespace dz {
namespace {

constexpr int kCBlock = 128;

__device__ __forceinline__ float quantize_sym(float w, float scale, float zero, float maxq) {
  // quant.py:9-18: q = clamp(round(w / scale) + zero, 0, maxq); return scale * (q - zero)
  float q = rintf(__fdiv_rn(w, scale)) + zero;
  q = fminf(fmaxf(q, 0.f), maxq);
  return __fmul_rn(scale, q - zero);
}

// grid: ceil(N / 8) blocks of 8 warps; W1: [N, ldw] block start (column i1), count <= 128 columns
__global__ void __launch_bounds__(256)
sparsegpt_block_kernel(const float* __restrict__ W, long long ldw, const float* __restrict__ hinv,
                       long long ldh, const float* __restrict__ scale, const float* __restrict__ zero,
                       float maxq, int N, int count, float* __restrict__ Q, float* __restrict__ Err,
                       float* __restrict__ loss) {
  extern __shared__ float s_h_raw[];                       // [128][128] floats
  float (*s_h)[kCBlock] = reinterpret_cast<float (*)[kCBlock]>(s_h_raw);
  for (int i = threadIdx.x; i < count * count; i += 256) {
    const int r = i / count, c = i % count;
    s_h[r][c] = c >= r ? hinv[(size_t)r * ldh + c] : 0.f;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= N) return;
  const float sc = scale[row], zp = zero[row];
  float w[4], q[4], e[4];
  bool pruned[4] = {false, false, false, false};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = lane + 32 * j;
    w[j] = c < count ? W[(size_t)row * ldw + c] : 0.f;
    q[j] = e[j] = 0.f;
  }
  float row_loss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    for (int l = 0; l < 32; ++l) {
      const int i = 32 * j + l;
      if (i >= count) break;
      if ((i & 3) == 0) {
        // the group's four columns live in lanes l .. l+3 (same j): rank by w^2 / d^2, prune
        // the two smallest (ties: the lower column first, as a stable selection does)
        const float d = (lane >= l && lane < l + 4 && 32 * j + lane < count) ? s_h[32 * j + lane][32 * j + lane] : 1.f;
        const float mine = __fdiv_rn(__fmul_rn(w[j], w[j]), __fmul_rn(d, d));
        float v[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) v[t] = __shfl_sync(0xffffffffu, mine, (l + t) & 31);
        if (lane >= l && lane < l + 4) {
          const int me = lane - l;
          int smaller = 0;
#pragma unroll
          for (int t = 0; t < 4; ++t)
            smaller += (v[t] < v[me] || (v[t] == v[me] && t < me)) ? 1 : 0;
          pruned[j] = smaller < 2;
        }
      }
      // column i: its owner lane quantises, everybody behind it receives the error
      float err = 0.f;
      if (lane == l) {
        const float d = s_h[i][i];
        const float wi = w[j];
        const float qi = quantize_sym(pruned[j] ? 0.f : wi, sc, zp, maxq);
        q[j] = qi;
        const float diff = wi - qi;
        err = __fdiv_rn(diff, d);
        e[j] = err;
        row_loss += __fdiv_rn(__fmul_rn(diff, diff), __fmul_rn(d, d));
      }
      err = __shfl_sync(0xffffffffu, err, l);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int c = lane + 32 * jj;
        // W1[:, i:] -= err * Hinv1[i, i:]  (column i itself included, as in the reference)
        if (c >= i && c < count) w[jj] = __fsub_rn(w[jj], __fmul_rn(err, s_h[i][c]));
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = lane + 32 * j;
    if (c < count) {
      Q[(size_t)row * count + c] = q[j];
      Err[(size_t)row * count + c] = e[j];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) row_loss += __shfl_xor_sync(0xffffffffu, row_loss, o);
  if (lane == 0 && loss) loss[row] += row_loss * 0.5f;
}

// one thread per packed word: grid covers [K*bits/32, N]
__global__ void pack_gptq_kernel(const float* __restrict__ Wq, const float* __restrict__ scale,
                                 const float* __restrict__ zero, int N, int K, int bits,
                                 int32_t* __restrict__ qweight, int32_t* __restrict__ qzeros,
                                 __half* __restrict__ scales) {
  const int per = 32 / bits;
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int kw = blockIdx.y;
  if (n >= N) return;
  const float sc = scale[n], zp = zero[n];
  const __half sh = __float2half_rn(sc);
  const float scf = __half2float(sh);
  const float sz = __fmul_rn(zp, sc);
  uint32_t word = 0;
  for (int j = 0; j < per; ++j) {
    const float v = Wq[(size_t)n * K + (size_t)kw * per + j];
    const int code = (int)rintf(__fdiv_rn(v + sz, scf));
    word |= ((uint32_t)code) << (bits * j);
  }
  qweight[(size_t)kw * N + n] = (int32_t)word;
  if (kw == 0) {
    scales[n] = sh;
    if (n % per == 0) {
      uint32_t z = 0;
      for (int j = 0; j < per && n + j < N; ++j)
        z |= ((uint32_t)(zero[n + j] - 1.f)) << (bits * j);
      qzeros[n / per] = (int32_t)z;
    }
  }
}

// per-row symmetric grid (quant.py:48-86 with perchannel, sym, no mse): one warp per row
__global__ void find_params_kernel(const float* __restrict__ W, int N, int K, float maxq,
                                   float* __restrict__ scale, float* __restrict__ zero) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= N) return;
  float mn = 0.f, mx = 0.f;
  for (int c = lane; c < K; c += 32) {
    const float v = W[(size_t)row * K + c];
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (lane == 0) {
    mx = fmaxf(fabsf(mn), mx);
    if (mn < 0.f) mn = -mx;
    if (mn == 0.f && mx == 0.f) { mn = -1.f; mx = 1.f; }
    scale[row] = __fdiv_rn(mx - mn, maxq);
    zero[row] = (maxq + 1.f) * 0.5f;
  }
}

}  // namespace
}  // namespace dz

using namespace dz;

extern "C" {

int dz_quant_find_params(const float* W, int N, int K, int bits, float* scale, float* zero, void* stream) {
  if (!W || !scale || !zero || N <= 0 || K <= 0) return DZ_ERR_INVALID_ARG;
  if (bits != 2 && bits != 4 && bits != 8) return DZ_ERR_SHAPE;
  find_params_kernel<<<(N + 7) / 8, 256, 0, (cudaStream_t)stream>>>(W, N, K, (float)((1 << bits) - 1), scale, zero);
  DZ_CUDA_OK(cudaGetLastError());
  return DZ_OK;
}

int dz_sparsegpt_block(const float* W_block, int64_t ldw, const float* hinv_block, int64_t ldh,
                       const float* scale, const float* zero, int bits, int N, int count, float* Q,
                       float* Err, float* loss, void* stream) {
  if (!W_block || !hinv_block || !scale || !zero || !Q || !Err) return DZ_ERR_INVALID_ARG;
  if (N <= 0 || count <= 0 || count > kCBlock || (count & 3)) return DZ_ERR_SHAPE;
  if (bits != 2 && bits != 4 && bits != 8) return DZ_ERR_SHAPE;
  constexpr int kSmem = kCBlock * kCBlock * sizeof(float);
  static bool attr_set[64] = {};
  int dev = 0;
  DZ_CUDA_OK(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    DZ_CUDA_OK(cudaFuncSetAttribute(sparsegpt_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    attr_set[dev & 63] = true;
  }
  sparsegpt_block_kernel<<<(N + 7) / 8, 256, kSmem, (cudaStream_t)stream>>>(
      W_block, ldw, hinv_block, ldh, scale, zero, (float)((1 << bits) - 1), N, count, Q, Err, loss);
  DZ_CUDA_OK(cudaGetLastError());
  return DZ_OK;
}

int dz_pack_gptq(const float* Wq, const float* scale, const float* zero, int N, int K, int bits,
                 int32_t* qweight, int32_t* qzeros, uint16_t* scales, void* stream) {
  if (!Wq || !scale || !zero || !qweight || !qzeros || !scales) return DZ_ERR_INVALID_ARG;
  if (bits != 2 && bits != 4 && bits != 8) return DZ_ERR_SHAPE;
  const int per = 32 / bits;
  if (N <= 0 || K <= 0 || K % per || N % per) return DZ_ERR_SHAPE;
  const dim3 grid((N + 255) / 256, K / per);
  pack_gptq_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(Wq, scale, zero, N, K, bits, qweight, qzeros,
                                                           reinterpret_cast<__half*>(scales));
  DZ_CUDA_OK(cudaGetLastError());
  return DZ_OK;
}

}  // extern "C"

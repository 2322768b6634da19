// Format kernels: GPTQ layout -> slot layout (convert) and slot layout -> dense
// fp16 delta (unpack).  Both are byte/integer work bound by HBM; one thread owns
// one (output row, 64-wide k block) so that reads of the GPTQ words are
// coalesced across rows and each thread writes whole 16/8-byte units.
#include "dz_common.cuh"

namespace dz {

namespace {

// Kept pair of a group of four, from the mask of positions whose code differs
// from the zero-point.  Rule: the non-zero positions in ascending order; when
// fewer than two, the lowest-index remaining positions fill up and the pair is
// re-sorted.  More than two set bits is not 2:4 (the two lowest are taken and
// the caller flags the error).
__device__ __forceinline__ void kept_pair(unsigned nzmask, int& i0, int& i1) {
  int cnt = __popc(nzmask);
  if (cnt >= 2) {
    i0 = __ffs(nzmask) - 1;
    i1 = __ffs(nzmask & (nzmask - 1)) - 1;
  } else if (cnt == 1) {
    int p = __ffs(nzmask) - 1;
    int q = (p == 0) ? 1 : 0;
    i0 = min(p, q);
    i1 = max(p, q);
  } else {
    i0 = 0;
    i1 = 1;
  }
}

template <int BITS>
__global__ void __launch_bounds__(128)
convert_from_gptq_kernel(const uint32_t* __restrict__ qweight, const uint32_t* __restrict__ qzeros,
                         const uint16_t* __restrict__ scales, int N, int K,
                         uint8_t* __restrict__ sq, uint8_t* __restrict__ sm,
                         uint16_t* __restrict__ ss, int* status_word) {
  constexpr int PER = 32 / BITS;          // codes per GPTQ word
  constexpr unsigned MAXQ = (1u << BITS) - 1;
  constexpr int WORDS_IN = kBlockK / PER; // GPTQ words per block per row
  const int n = blockIdx.x * 128 + threadIdx.x;
  const int kb = blockIdx.y;
  const int num_kb = K / kBlockK;
  if (n >= N) return;

  const unsigned zstored = (qzeros[n / PER] >> (BITS * (n % PER))) & MAXQ;
  const unsigned z = zstored + 1;
  if (z != (1u << (BITS - 1)) && status_word) atomicCAS(status_word, 0, (int)DZ_ERR_NOT_SYMMETRIC);

  uint32_t win[WORDS_IN];
#pragma unroll
  for (int i = 0; i < WORDS_IN; ++i) win[i] = qweight[(size_t)(kb * WORDS_IN + i) * N + n];

  uint32_t wout[BITS];
#pragma unroll
  for (int i = 0; i < BITS; ++i) wout[i] = 0;
  uint32_t mh[2][2] = {{0, 0}, {0, 0}};
  bool bad = false;

#pragma unroll
  for (int g = 0; g < 16; ++g) {
    unsigned c[4];
    unsigned nz = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int k = g * 4 + j;
      c[j] = (win[k / PER] >> (BITS * (k % PER))) & MAXQ;
      nz |= (c[j] != z ? 1u : 0u) << j;
    }
    if (__popc(nz) > 2) bad = true;
    int i0, i1;
    kept_pair(nz, i0, i1);
    unsigned c0 = (i0 == 0) ? c[0] : (i0 == 1) ? c[1] : c[2];
    unsigned c1 = (i1 == 1) ? c[1] : (i1 == 2) ? c[2] : c[3];
    const int e0 = 2 * g, e1 = 2 * g + 1;
    wout[code_word(e0, BITS)] |= c0 << code_shift(e0, BITS);
    wout[code_word(e1, BITS)] |= c1 << code_shift(e1, BITS);
    mh[g >> 3][(g >> 2) & 1] |= (unsigned)(i0 | (i1 << 2)) << (4 * (g & 3));
  }
  if (bad && status_word) atomicCAS(status_word, 0, (int)DZ_ERR_NOT_2_4);

  uint8_t* dst = sq + codes_offset(n, kb, num_kb, BITS);
  if (BITS == 4) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(wout[0], wout[1], wout[2], wout[BITS - 1]);
  } else {
    *reinterpret_cast<uint2*>(dst) = make_uint2(wout[0], wout[1]);
  }
#pragma unroll
  for (int c2 = 0; c2 < 2; ++c2)
#pragma unroll
    for (int kh = 0; kh < 2; ++kh)
      *reinterpret_cast<uint16_t*>(sm + meta_offset(n, kb, num_kb, c2, kh)) = (uint16_t)mh[c2][kh];
  if (kb == 0) ss[n] = scales[n];
}

template <int BITS>
__global__ void __launch_bounds__(128)
unpack_kernel(const uint8_t* __restrict__ sq, const uint8_t* __restrict__ sm,
              const uint16_t* __restrict__ ss, int N, int K, uint16_t* __restrict__ out) {
  constexpr unsigned MAXQ = (1u << BITS) - 1;
  constexpr int Z = 1 << (BITS - 1);
  const int n = blockIdx.x * 128 + threadIdx.x;
  const int kb = blockIdx.y;
  const int num_kb = K / kBlockK;
  if (n >= N) return;

  uint32_t w[BITS];
  const uint8_t* src = sq + codes_offset(n, kb, num_kb, BITS);
  if (BITS == 4) {
    uint4 v = *reinterpret_cast<const uint4*>(src);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[BITS - 1] = v.w;
  } else {
    uint2 v = *reinterpret_cast<const uint2*>(src);
    w[0] = v.x; w[1] = v.y;
  }
  const __half scale = __ushort_as_half(ss[n]);

  __align__(16) __half d[kBlockK];
#pragma unroll
  for (int i = 0; i < kBlockK; ++i) d[i] = __ushort_as_half((unsigned short)0);

#pragma unroll
  for (int c = 0; c < 2; ++c)
#pragma unroll
    for (int kh = 0; kh < 2; ++kh) {
      const unsigned m16 = *reinterpret_cast<const uint16_t*>(sm + meta_offset(n, kb, num_kb, c, kh));
#pragma unroll
      for (int gg = 0; gg < 4; ++gg) {
        const int g = c * 8 + kh * 4 + gg;
        const unsigned nib = (m16 >> (4 * gg)) & 0xF;
        const int i0 = nib & 3, i1 = (nib >> 2) & 3;
        const int e0 = 2 * g, e1 = 2 * g + 1;
        const int q0 = (int)((w[code_word(e0, BITS)] >> code_shift(e0, BITS)) & MAXQ);
        const int q1 = (int)((w[code_word(e1, BITS)] >> code_shift(e1, BITS)) & MAXQ);
        // one fp16 product of the fp16 scale and an exact small integer
        const __half v0 = __hmul(scale, __int2half_rn(q0 - Z));
        const __half v1 = __hmul(scale, __int2half_rn(q1 - Z));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j == i0) d[g * 4 + j] = v0;
          if (j == i1 && i1 != i0) d[g * 4 + j] = v1;
        }
      }
    }
  uint4* o = reinterpret_cast<uint4*>(out + (size_t)n * K + (size_t)kb * kBlockK);
  const uint4* dv = reinterpret_cast<const uint4*>(d);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = dv[i];
}

}  // namespace

int launch_convert_from_gptq(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                             int N, int K, int bits, void* sq, void* sm, uint16_t* ss,
                             int* status_word, cudaStream_t st) {
  dim3 grid(N / 128, K / kBlockK), block(128);
  if (bits == 4)
    convert_from_gptq_kernel<4><<<grid, block, 0, st>>>(
        (const uint32_t*)qweight, (const uint32_t*)qzeros, scales, N, K, (uint8_t*)sq, (uint8_t*)sm,
        ss, status_word);
  else
    convert_from_gptq_kernel<2><<<grid, block, 0, st>>>(
        (const uint32_t*)qweight, (const uint32_t*)qzeros, scales, N, K, (uint8_t*)sq, (uint8_t*)sm,
        ss, status_word);
  DZ_CUDA_OK(cudaGetLastError());
  return DZ_OK;
}

int launch_unpack(const void* sq, const void* sm, const uint16_t* ss, int N, int K, int bits,
                  uint16_t* out, cudaStream_t st) {
  dim3 grid(N / 128, K / kBlockK), block(128);
  if (bits == 4)
    unpack_kernel<4><<<grid, block, 0, st>>>((const uint8_t*)sq, (const uint8_t*)sm, ss, N, K, out);
  else
    unpack_kernel<2><<<grid, block, 0, st>>>((const uint8_t*)sq, (const uint8_t*)sm, ss, N, K, out);
  DZ_CUDA_OK(cudaGetLastError());
  return DZ_OK;
}

}  // namespace dz

// Correctness-first SBMM on CUDA cores: one thread per output row of a 128-row
// tile, eight tokens per CTA, fp32 accumulation.  It reads the same slot layout
// and segment table as the tensor-core kernel and exists to validate those
// (and the host plumbing) independently of the tcgen05 code path.
#include "dz_common.cuh"

namespace dz {

namespace {

constexpr int kTok = 8;

template <int BITS>
__global__ void __launch_bounds__(128)
sbmm_simt_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                 const uint8_t* __restrict__ qweight, const uint8_t* __restrict__ meta,
                 const uint8_t* __restrict__ scales, long long qstride, long long mstride,
                 long long sstride, const uint8_t* __restrict__ seg, __half* __restrict__ y,
                 int M, int N, int K, int base_only) {
  constexpr unsigned MAXQ = (1u << BITS) - 1;
  constexpr int Z = 1 << (BITS - 1);
  __shared__ __half xs[kTok][kBlockK];
  __shared__ int s_perm[kTok], s_slot[kTok];

  const int r = threadIdx.x;
  const int n = blockIdx.x * 128 + r;
  const int p0 = blockIdx.y * kTok;
  const int num_kb = K / kBlockK;

  if (r < kTok) {
    int p = p0 + r;
    int tok = -1, slot = -1;
    if (p < M) {
      if (seg) {
        const SegHeader* hdr = reinterpret_cast<const SegHeader*>(seg);
        const SegLayout lay = seg_layout(hdr->capacity_M, hdr->num_slots);
        tok = reinterpret_cast<const int*>(seg + lay.perm)[p];
        slot = base_only ? -1 : reinterpret_cast<const int*>(seg + lay.slot_of)[p];
      } else {
        tok = p;
      }
    }
    s_perm[r] = tok;
    s_slot[r] = slot;
  }
  __syncthreads();

  float acc[kTok];
#pragma unroll
  for (int j = 0; j < kTok; ++j) acc[j] = 0.f;

  for (int kb = 0; kb < num_kb; ++kb) {
    {  // x tile: 8 tokens x 64 k, 4 halves per thread
      const int j = r >> 4, k4 = (r & 15) * 4;
      uint2 v = make_uint2(0, 0);
      if (s_perm[j] >= 0)
        v = *reinterpret_cast<const uint2*>(x + (size_t)s_perm[j] * K + kb * kBlockK + k4);
      *reinterpret_cast<uint2*>(&xs[j][k4]) = v;
    }
    __syncthreads();

    // base row
    const uint4* wrow = reinterpret_cast<const uint4*>(w + (size_t)n * K + kb * kBlockK);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4 v = wrow[c];
      const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float wf = __half2float(h[i]);
#pragma unroll
        for (int j = 0; j < kTok; ++j) acc[j] += wf * __half2float(xs[j][c * 8 + i]);
      }
    }

    // deltas: runs of equal slot among the CTA's tokens
    int j = 0;
    while (j < kTok) {
      const int slot = s_slot[j];
      int j1 = j + 1;
      while (j1 < kTok && s_slot[j1] == slot) ++j1;
      if (slot >= 0) {
        const uint8_t* qsrc = qweight + (size_t)slot * qstride + codes_offset(n, kb, num_kb, BITS);
        uint32_t cw[BITS];
        if (BITS == 4) {
          uint4 v = *reinterpret_cast<const uint4*>(qsrc);
          cw[0] = v.x; cw[1] = v.y; cw[2] = v.z; cw[BITS - 1] = v.w;
        } else {
          uint2 v = *reinterpret_cast<const uint2*>(qsrc);
          cw[0] = v.x; cw[1] = v.y;
        }
        const __half scale =
            *reinterpret_cast<const __half*>(scales + (size_t)slot * sstride + (size_t)n * 2);
        const uint8_t* msrc = meta + (size_t)slot * mstride;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int kh = 0; kh < 2; ++kh) {
            const unsigned m16 =
                *reinterpret_cast<const uint16_t*>(msrc + meta_offset(n, kb, num_kb, c, kh));
#pragma unroll
            for (int gg = 0; gg < 4; ++gg) {
              const int g = c * 8 + kh * 4 + gg;
              const unsigned nib = (m16 >> (4 * gg)) & 0xF;
              const int k0 = g * 4 + (nib & 3), k1 = g * 4 + ((nib >> 2) & 3);
              const int e0 = 2 * g, e1 = 2 * g + 1;
              const int q0 = (int)((cw[code_word(e0, BITS)] >> code_shift(e0, BITS)) & MAXQ);
              const int q1 = (int)((cw[code_word(e1, BITS)] >> code_shift(e1, BITS)) & MAXQ);
              const float v0 = __half2float(__hmul(scale, __int2half_rn(q0 - Z)));
              const float v1 = __half2float(__hmul(scale, __int2half_rn(q1 - Z)));
              for (int t = j; t < j1; ++t) {
                acc[t] += v0 * __half2float(xs[t][k0]);
                acc[t] += v1 * __half2float(xs[t][k1]);
              }
            }
          }
      }
      j = j1;
    }
    __syncthreads();
  }

#pragma unroll
  for (int j = 0; j < kTok; ++j)
    if (s_perm[j] >= 0) y[(size_t)s_perm[j] * N + n] = __float2half_rn(acc[j]);
}

}  // namespace

int launch_sbmm_simt(const dz_sbmm_args& a, bool base_only, cudaStream_t st) {
  dim3 grid(a.N / 128, (a.M + kTok - 1) / kTok), block(128);
  if (a.M == 0) return DZ_OK;
  if (a.bits == 4)
    sbmm_simt_kernel<4><<<grid, block, 0, st>>>(
        (const __half*)a.x, (const __half*)a.w_base, (const uint8_t*)a.qweight,
        (const uint8_t*)a.meta, (const uint8_t*)a.scales, a.qweight_stride, a.meta_stride,
        a.scales_stride, (const uint8_t*)a.segments, (__half*)a.y, a.M, a.N, a.K, base_only);
  else
    sbmm_simt_kernel<2><<<grid, block, 0, st>>>(
        (const __half*)a.x, (const __half*)a.w_base, (const uint8_t*)a.qweight,
        (const uint8_t*)a.meta, (const uint8_t*)a.scales, a.qweight_stride, a.meta_stride,
        a.scales_stride, (const uint8_t*)a.segments, (__half*)a.y, a.M, a.N, a.K, base_only);
  DZ_CUDA_OK(cudaGetLastError());
  return DZ_OK;
}

}  // namespace dz

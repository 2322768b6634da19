// The element-wise and attention steps that sit between the SBMM calls of a decoder layer at
// decode time.  All of them are HBM-bound passes over [tokens, hidden]-sized activations or over
// the paged KV cache; they exist so that a decode step is a chain of this library's launches
// with no host work in between.  Roles in the reference (serving/csrc/ops.h, cache.h):
//   rms_norm / fused_add_rms_norm   ops.h:37-47   (layernorm_kernels.cu)
//   silu_and_mul                    ops.h:67      (activation_kernels.cu)
//   rotary_embedding (neox)         ops.h:49      (pos_encoding_kernels.cu)
//   reshape_and_cache               cache.h:18    (cache_kernels.cu)
//   paged_attention_v1              ops.h:6       (attention/attention_kernels.cu)
// Layouts are this library's own: the KV cache is [num_blocks, block_size, kv_heads, 128] for K
// and for V (one 256-byte row per token and head), head size 128 only (every Llama-2 size).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "dz_common.cuh"

namespace dz {
namespace {

constexpr int kHeadDim = 128;

template <typename T> struct Cvt;
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float2 up(uint32_t v) {
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
  }
  static __device__ __forceinline__ uint32_t down(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float round(float a) { return __half2float(__float2half_rn(a)); }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float2 up(uint32_t v) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
  }
  static __device__ __forceinline__ uint32_t down(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float round(float a) {
    return __bfloat162float(__float2bfloat16_rn(a));
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------
// RMSNorm, optionally preceded by the residual add.  One CTA per token row; the row is read
// once into registers (hidden <= 8 * 8 * 256 = 16384).
//   residual == nullptr:  out = norm(x) * w
//   residual != nullptr:  residual = x + residual (rounded to T);  out = norm(residual) * w
// The normalised value is rounded to T before the multiplication by the weight, as the
// reference's kernel and its PyTorch twin do (layernorm.py:27-45).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
rms_norm_kernel(const uint4* __restrict__ x, uint4* __restrict__ residual,
                const uint4* __restrict__ w, uint4* __restrict__ out, int hidden, float eps) {
  constexpr int kMaxVec = 8;                      // 16-byte vectors per thread
  __shared__ float s_part[8];
  const int nvec = hidden / 8;
  const size_t row = (size_t)blockIdx.x * nvec;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  float v[kMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < nvec) {
      const uint4 a = x[row + i];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
      if (residual) {
        const uint4 r = residual[row + i];
        const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 fa = Cvt<T>::up(aw[q]), fr = Cvt<T>::up(rw[q]);
          o[q] = Cvt<T>::down(fa.x + fr.x, fa.y + fr.y);
          const float2 s = Cvt<T>::up(o[q]);
          v[j][2 * q] = s.x;
          v[j][2 * q + 1] = s.y;
        }
        residual[row + i] = make_uint4(o[0], o[1], o[2], o[3]);
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 fa = Cvt<T>::up(aw[q]);
          v[j][2 * q] = fa.x;
          v[j][2 * q + 1] = fa.y;
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) ss += v[j][q] * v[j][q];
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += s_part[i];
  const float inv = rsqrtf(tot / (float)hidden + eps);
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < nvec) {
      const uint4 ww = w[i];
      const uint32_t wv[4] = {ww.x, ww.y, ww.z, ww.w};
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fw = Cvt<T>::up(wv[q]);
        o[q] = Cvt<T>::down(Cvt<T>::round(v[j][2 * q] * inv) * fw.x,
                            Cvt<T>::round(v[j][2 * q + 1] * inv) * fw.y);
      }
      out[row + i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// out[m, i] = silu(x[m, i]) * x[m, inter + i]
template <typename T>
__global__ void __launch_bounds__(256)
silu_and_mul_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, int inter) {
  const int nvec = inter / 8;
  const size_t in_row = (size_t)blockIdx.y * 2 * nvec, out_row = (size_t)blockIdx.y * nvec;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (int i = blockIdx.x * 256 + threadIdx.x; i < nvec; i += gridDim.x * 256) {
    const uint4 g = x[in_row + i], u = x[in_row + nvec + i];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 fg = Cvt<T>::up(gw[q]), fu = Cvt<T>::up(uw[q]);
      // silu in float, rounded to T, then the product (the order of the reference's kernel)
      const float s0 = Cvt<T>::round(fg.x / (1.f + __expf(-fg.x)));
      const float s1 = Cvt<T>::round(fg.y / (1.f + __expf(-fg.y)));
      o[q] = Cvt<T>::down(s0 * fu.x, s1 * fu.y);
    }
    out[out_row + i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---------------------------------------------------------------------------
// Rotary position embedding (neox style: dims d and d + 64 form a pair) applied in place to the
// q and k parts of a fused qkv row, followed by the write of the rotated k and of v into the
// paged cache at `slot_mapping[token]` (block * block_size + offset; < 0 = not cached).
// Grid (tokens, heads / 4): one warp per (token, head), so every warp makes one round trip to
// memory instead of walking the heads of its token one after another; a lane owns dims
// [2l, 2l+2) and [64+2l, 64+2l+2).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
rotary_cache_kernel(T* __restrict__ qkv, const int64_t* __restrict__ positions,
                    const int64_t* __restrict__ slot_mapping, T* __restrict__ k_cache,
                    T* __restrict__ v_cache, int q_heads, int kv_heads, float log2_theta) {
  const int tok = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const float pos = (float)positions[tok];
  const int64_t slot = slot_mapping ? slot_mapping[tok] : -1;
  T* row = qkv + (size_t)tok * (q_heads + 2 * kv_heads) * kHeadDim;
  // angles of this lane's two pair indices i = 2l, 2l+1:  pos * theta^(-2i/128)
  float cs[2], sn[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float inv_freq = exp2f(-log2_theta * (float)(2 * (2 * lane + j)) / (float)kHeadDim);
    sincosf(pos * inv_freq, &sn[j], &cs[j]);
  }
  const int h = blockIdx.y * 4 + warp;
  if (h < q_heads + 2 * kv_heads) {
    uint32_t* p = reinterpret_cast<uint32_t*>(row + (size_t)h * kHeadDim);
    uint32_t lo = p[lane], hi = p[32 + lane];
    if (h < q_heads + kv_heads) {
      const float2 a = Cvt<T>::up(lo), b = Cvt<T>::up(hi);
      lo = Cvt<T>::down(a.x * cs[0] - b.x * sn[0], a.y * cs[1] - b.y * sn[1]);
      hi = Cvt<T>::down(b.x * cs[0] + a.x * sn[0], b.y * cs[1] + a.y * sn[1]);
      p[lane] = lo;
      p[32 + lane] = hi;
    }
    if (h >= q_heads && slot >= 0) {
      const bool is_k = h < q_heads + kv_heads;
      const int kh = is_k ? h - q_heads : h - q_heads - kv_heads;
      uint32_t* c = reinterpret_cast<uint32_t*>((is_k ? k_cache : v_cache) +
                                                ((size_t)slot * kv_heads + kh) * kHeadDim);
      c[lane] = lo;
      c[32 + lane] = hi;
    }
  }
}

// ---------------------------------------------------------------------------
// Decode attention over the paged cache: one query token per sequence.
// Grid (kv_heads, sequences, splits); a CTA handles the G = q_heads / kv_heads query heads that
// share one kv head, over the key range of its split, so K and V are read once.  The warps take
// the rows of the range in turn (how the lanes share a row depends on G, see the two forms
// below), scores are reduced with shuffles, softmax is computed online and the warps' partial
// (max, sum, acc) are merged through shared memory.
// With splits > 1 the CTA writes its partial triple to `partial` and the last CTA of a
// (sequence, kv head) to arrive -- counted with an atomic ticket -- merges the splits; nothing
// waits on anything.
// ---------------------------------------------------------------------------
template <typename T, int G>
__global__ void __launch_bounds__(256)
paged_decode_attention_kernel(const T* __restrict__ qkv, int q_row_stride, T* __restrict__ out,
                              const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                              const int* __restrict__ block_tables, int max_blocks,
                              const int* __restrict__ seq_lens, int block_size, int kv_heads,
                              float scale, int splits, float* __restrict__ partial,
                              int* __restrict__ tickets) {
  constexpr int kWarps = 8;
  __shared__ float s_m[kWarps][G], s_l[kWarps][G];
  __shared__ float s_acc[kWarps][G][kHeadDim];
  __shared__ int s_last;
  const int kh = blockIdx.x, seq = blockIdx.y, split = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int len = seq_lens[seq];
  const int per = (len + splits - 1) / splits;
  const int t0 = split * per, t1 = min(len, t0 + per);
  const int q_heads = kv_heads * G;

  const int* table = block_tables + (size_t)seq * max_blocks;
  if constexpr (G <= 2) {
    // Few query heads per key/value head: the kernel is a pure stream of K and V rows, so what
    // counts is bytes in flight.  A half-warp owns a row (16 lanes x 16 bytes), a warp two rows
    // per load instruction, and two such pairs are requested per iteration: 64 bytes in flight
    // per lane.  Each half-warp keeps its own running (max, sum, accumulator); the halves are
    // merged by shuffles at the end, the warps through shared memory as in the general form.
    const int half = lane >> 4, hl = lane & 15;
    float q[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const uint4 v = *reinterpret_cast<const uint4*>(qkv + (size_t)seq * q_row_stride +
                                                      (size_t)(kh * G + g) * kHeadDim + hl * 8);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Cvt<T>::up(w[j]);
        q[g][2 * j] = f.x * scale;
        q[g][2 * j + 1] = f.y * scale;
      }
    }
    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
    }
    for (int base = t0 + 2 * warp; base < t1; base += 4 * kWarps) {
      const int ta = base + half, tb = ta + 2 * kWarps;
      const bool va_ok = ta < t1, vb_ok = tb < t1;
      const int tac = min(ta, t1 - 1), tbc = min(tb, t1 - 1);     // rows read for absent tokens
      const size_t ra = ((size_t)table[tac / block_size] * block_size + tac % block_size) * kv_heads + kh;
      const size_t rb = ((size_t)table[tbc / block_size] * block_size + tbc % block_size) * kv_heads + kh;
      const uint4 ka = *reinterpret_cast<const uint4*>(k_cache + ra * kHeadDim + hl * 8);
      const uint4 kb = *reinterpret_cast<const uint4*>(k_cache + rb * kHeadDim + hl * 8);
      const uint4 va = *reinterpret_cast<const uint4*>(v_cache + ra * kHeadDim + hl * 8);
      const uint4 vb = *reinterpret_cast<const uint4*>(v_cache + rb * kHeadDim + hl * 8);
      float fka[8], fkb[8], fva[8], fvb[8];
      {
        const uint32_t wa[4] = {ka.x, ka.y, ka.z, ka.w}, wb[4] = {kb.x, kb.y, kb.z, kb.w};
        const uint32_t xa[4] = {va.x, va.y, va.z, va.w}, xb[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = Cvt<T>::up(wa[j]); fka[2 * j] = f.x; fka[2 * j + 1] = f.y;
          f = Cvt<T>::up(wb[j]); fkb[2 * j] = f.x; fkb[2 * j + 1] = f.y;
          f = Cvt<T>::up(xa[j]); fva[2 * j] = f.x; fva[2 * j + 1] = f.y;
          f = Cvt<T>::up(xb[j]); fvb[2 * j] = f.x; fvb[2 * j + 1] = f.y;
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { sa += q[g][j] * fka[j]; sb += q[g][j] * fkb[j]; }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {            // within the half-warp
          sa += __shfl_xor_sync(0xffffffffu, sa, o);
          sb += __shfl_xor_sync(0xffffffffu, sb, o);
        }
        if (va_ok) {                                  // vb_ok implies va_ok
          if (!vb_ok) sb = -INFINITY;
          const float mn = fmaxf(m[g], fmaxf(sa, sb));
          const float c = __expf(m[g] - mn), pa = __expf(sa - mn), pb = __expf(sb - mn);
          l[g] = l[g] * c + pa + pb;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[g][j] = acc[g][j] * c + pa * fva[j] + pb * fvb[j];
          m[g] = mn;
        }
      }
    }
    // merge the two half-warps, then hand the warp's state to shared memory
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], 16);
      const float lo = __shfl_xor_sync(0xffffffffu, l[g], 16);
      const float mm = fmaxf(m[g], mo);
      const float c0 = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mm);
      const float c1 = (mo == -INFINITY) ? 0.f : __expf(mo - mm);
      const float ll = l[g] * c0 + lo * c1;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][j], 16);
        acc[g][j] = acc[g][j] * c0 + ao * c1;
      }
      if (lane == 0) { s_m[warp][g] = mm; s_l[warp][g] = ll; }
      if (half == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) s_acc[warp][g][hl * 8 + j] = acc[g][j];
      }
    }
  } else {
    // Grouped queries (4 or 8 query heads per kv head): lane -> (head g, part of the row), LPH =
    // 32 / G lanes per head, each with 128 / LPH = 4 G dims of q and of the accumulator.  A warp
    // takes one key/value row per step; the lanes of all heads read the same bytes of it (the
    // loads coalesce into one row), a score needs log2(LPH) shuffles instead of five per head,
    // and the K and V loads of a step are in flight together.
    constexpr int LPH = 32 / G, DPL = 4 * G, NV = DPL / 8;     // NV 16-byte loads per row part
    const int g = lane / LPH, part = lane % LPH;
    float q[DPL], acc[DPL];
    {
      const T* qp = qkv + (size_t)seq * q_row_stride + (size_t)(kh * G + g) * kHeadDim + part * DPL;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const uint4 u = *reinterpret_cast<const uint4*>(qp + v * 8);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Cvt<T>::up(w[j]);
          q[v * 8 + 2 * j] = f.x * scale;
          q[v * 8 + 2 * j + 1] = f.y * scale;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[j] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int t = t0 + warp; t < t1; t += kWarps) {
      const size_t r = ((size_t)table[t / block_size] * block_size + t % block_size) * kv_heads + kh;
      uint4 kk[NV], vv[NV];
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        kk[v] = *reinterpret_cast<const uint4*>(k_cache + r * kHeadDim + part * DPL + v * 8);
        vv[v] = *reinterpret_cast<const uint4*>(v_cache + r * kHeadDim + part * DPL + v * 8);
      }
      float sc = 0.f;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const uint32_t w[4] = {kk[v].x, kk[v].y, kk[v].z, kk[v].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Cvt<T>::up(w[j]);
          sc += q[v * 8 + 2 * j] * f.x + q[v * 8 + 2 * j + 1] * f.y;
        }
      }
#pragma unroll
      for (int o = LPH / 2; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
      const float mn = fmaxf(m, sc);
      const float c = __expf(m - mn), pw = __expf(sc - mn);
      l = l * c + pw;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const uint32_t w[4] = {vv[v].x, vv[v].y, vv[v].z, vv[v].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Cvt<T>::up(w[j]);
          acc[v * 8 + 2 * j] = acc[v * 8 + 2 * j] * c + pw * f.x;
          acc[v * 8 + 2 * j + 1] = acc[v * 8 + 2 * j + 1] * c + pw * f.y;
        }
      }
      m = mn;
    }
    if (part == 0) { s_m[warp][g] = m; s_l[warp][g] = l; }
#pragma unroll
    for (int j = 0; j < DPL; ++j) s_acc[warp][g][part * DPL + j] = acc[j];
  }
  __syncthreads();
  // thread (g, d) pairs: G * 128 values, 256 threads
  for (int i = threadIdx.x; i < G * kHeadDim; i += 256) {
    const int g = i / kHeadDim, d = i % kHeadDim;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, s_m[w][g]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float c = (s_m[w][g] == -INFINITY) ? 0.f : __expf(s_m[w][g] - mm);
      ll += s_l[w][g] * c;
      a += s_acc[w][g][d] * c;
    }
    const int head = kh * G + g;
    if (splits == 1) {
      out[((size_t)seq * q_heads + head) * kHeadDim + d] =
          (T)(ll > 0.f ? a / ll : 0.f);
    } else {
      float* pp = partial + (((size_t)seq * q_heads + head) * splits + split) * (kHeadDim + 2);
      pp[d] = a;
      if (d == 0) { pp[kHeadDim] = mm; pp[kHeadDim + 1] = ll; }
    }
  }
  if (splits == 1) return;
  // the last split of this (sequence, kv head) to finish merges all of them
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(&tickets[seq * kv_heads + kh], 1);
    s_last = (done == splits - 1);
    if (s_last) tickets[seq * kv_heads + kh] = 0;      // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < G * kHeadDim; i += 256) {
    const int g = i / kHeadDim, d = i % kHeadDim;
    const int head = kh * G + g;
    const float* pp = partial + ((size_t)seq * q_heads + head) * splits * (kHeadDim + 2);
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, __ldcg(pp + s * (kHeadDim + 2) + kHeadDim));
    float ll = 0.f, a = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = __ldcg(pp + s * (kHeadDim + 2) + kHeadDim);
      const float c = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
      ll += __ldcg(pp + s * (kHeadDim + 2) + kHeadDim + 1) * c;
      a += __ldcg(pp + s * (kHeadDim + 2) + d) * c;
    }
    out[((size_t)seq * q_heads + head) * kHeadDim + d] = (T)(ll > 0.f ? a / ll : 0.f);
  }
}

template <typename K, typename... Args>
cudaError_t launch_pdl(K kern, dim3 grid, dim3 block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <typename T>
int attention_dispatch(int group, dim3 grid, cudaStream_t st, const T* qkv, int q_row_stride, T* out,
                       const T* kc, const T* vc, const int* bt, int max_blocks, const int* sl,
                       int block_size, int kv_heads, float scale, int splits, float* partial,
                       int* tickets) {
  switch (group) {
    case 1: DZ_CUDA_OK(launch_pdl(paged_decode_attention_kernel<T, 1>, grid, dim3(256), st, qkv, q_row_stride, out, kc, vc, bt, max_blocks, sl, block_size, kv_heads, scale, splits, partial, tickets)); break;
    case 2: DZ_CUDA_OK(launch_pdl(paged_decode_attention_kernel<T, 2>, grid, dim3(256), st, qkv, q_row_stride, out, kc, vc, bt, max_blocks, sl, block_size, kv_heads, scale, splits, partial, tickets)); break;
    case 4: DZ_CUDA_OK(launch_pdl(paged_decode_attention_kernel<T, 4>, grid, dim3(256), st, qkv, q_row_stride, out, kc, vc, bt, max_blocks, sl, block_size, kv_heads, scale, splits, partial, tickets)); break;
    case 8: DZ_CUDA_OK(launch_pdl(paged_decode_attention_kernel<T, 8>, grid, dim3(256), st, qkv, q_row_stride, out, kc, vc, bt, max_blocks, sl, block_size, kv_heads, scale, splits, partial, tickets)); break;
    default: return DZ_ERR_UNSUPPORTED;
  }
  return DZ_OK;
}

}  // namespace
}  // namespace dz

using namespace dz;

extern "C" {

int dz_rms_norm(const void* x, void* residual, const void* weight, void* out, int M, int hidden,
                float eps, int dtype, void* stream) {
  if (!x || !weight || !out || M < 0 || hidden <= 0) return DZ_ERR_INVALID_ARG;
  if (hidden % 8 || hidden > 8 * 8 * 256) return DZ_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(weight) || !aligned16(out) || (residual && !aligned16(residual)))
    return DZ_ERR_ALIGNMENT;
  if (dtype != DZ_DTYPE_F16 && dtype != DZ_DTYPE_BF16) return DZ_ERR_INVALID_ARG;
  if (M == 0) return DZ_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == DZ_DTYPE_F16)
    DZ_CUDA_OK(launch_pdl(rms_norm_kernel<__half>, dim3(M), dim3(256), st, (const uint4*)x,
                          (uint4*)residual, (const uint4*)weight, (uint4*)out, hidden, eps));
  else
    DZ_CUDA_OK(launch_pdl(rms_norm_kernel<__nv_bfloat16>, dim3(M), dim3(256), st, (const uint4*)x,
                          (uint4*)residual, (const uint4*)weight, (uint4*)out, hidden, eps));
  return DZ_OK;
}

int dz_silu_and_mul(const void* x, void* out, int M, int inter, int dtype, void* stream) {
  if (!x || !out || M < 0 || inter <= 0) return DZ_ERR_INVALID_ARG;
  if (inter % 8) return DZ_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(out)) return DZ_ERR_ALIGNMENT;
  if (dtype != DZ_DTYPE_F16 && dtype != DZ_DTYPE_BF16) return DZ_ERR_INVALID_ARG;
  if (M == 0) return DZ_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid((inter / 8 + 255) / 256, M);
  if (dtype == DZ_DTYPE_F16)
    DZ_CUDA_OK(launch_pdl(silu_and_mul_kernel<__half>, grid, dim3(256), st, (const uint4*)x,
                          (uint4*)out, inter));
  else
    DZ_CUDA_OK(launch_pdl(silu_and_mul_kernel<__nv_bfloat16>, grid, dim3(256), st,
                          (const uint4*)x, (uint4*)out, inter));
  return DZ_OK;
}

int dz_rotary_and_cache(void* qkv, const int64_t* positions, const int64_t* slot_mapping,
                        void* k_cache, void* v_cache, int M, int q_heads, int kv_heads, int head_dim,
                        float rope_theta, int dtype, void* stream) {
  if (!qkv || !positions || M < 0 || q_heads <= 0 || kv_heads <= 0) return DZ_ERR_INVALID_ARG;
  if (head_dim != kHeadDim) return DZ_ERR_SHAPE;
  if (slot_mapping && (!k_cache || !v_cache)) return DZ_ERR_INVALID_ARG;
  if (!aligned16(qkv) || !aligned16(k_cache) || !aligned16(v_cache)) return DZ_ERR_ALIGNMENT;
  if (dtype != DZ_DTYPE_F16 && dtype != DZ_DTYPE_BF16) return DZ_ERR_INVALID_ARG;
  if (M == 0) return DZ_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const float l2t = log2f(rope_theta);
  const dim3 grid(M, (q_heads + 2 * kv_heads + 3) / 4);
  if (dtype == DZ_DTYPE_F16)
    DZ_CUDA_OK(launch_pdl(rotary_cache_kernel<__half>, grid, dim3(128), st, (__half*)qkv, positions,
                          slot_mapping, (__half*)k_cache, (__half*)v_cache, q_heads, kv_heads, l2t));
  else
    DZ_CUDA_OK(launch_pdl(rotary_cache_kernel<__nv_bfloat16>, grid, dim3(128), st,
                          (__nv_bfloat16*)qkv, positions, slot_mapping, (__nv_bfloat16*)k_cache,
                          (__nv_bfloat16*)v_cache, q_heads, kv_heads, l2t));
  return DZ_OK;
}

size_t dz_paged_attention_workspace_bytes(int num_seqs, int q_heads, int kv_heads, int splits) {
  if (num_seqs <= 0 || q_heads <= 0 || kv_heads <= 0 || splits <= 0) return 0;
  // tickets (rounded to 256 bytes) + partial triples
  const size_t tickets = (((size_t)num_seqs * kv_heads * 4) + 255) & ~(size_t)255;
  return tickets + (splits > 1 ? (size_t)num_seqs * q_heads * splits * (kHeadDim + 2) * 4 : 0);
}

int dz_paged_attention_decode(const void* qkv, int q_row_stride, void* out, const void* k_cache,
                              const void* v_cache, const int32_t* block_tables, int max_blocks,
                              const int32_t* seq_lens, int num_seqs, int q_heads, int kv_heads,
                              int head_dim, int block_size, float scale, int splits,
                              void* workspace, size_t workspace_bytes, int dtype, void* stream) {
  if (!qkv || !out || !k_cache || !v_cache || !block_tables || !seq_lens) return DZ_ERR_INVALID_ARG;
  if (num_seqs < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || block_size <= 0 ||
      max_blocks <= 0 || splits < 1 || splits > 64)
    return DZ_ERR_INVALID_ARG;
  if (head_dim != kHeadDim) return DZ_ERR_SHAPE;
  if ((q_row_stride & 7) || !aligned16(qkv) || !aligned16(out) || !aligned16(k_cache) ||
      !aligned16(v_cache))
    return DZ_ERR_ALIGNMENT;
  if (dtype != DZ_DTYPE_F16 && dtype != DZ_DTYPE_BF16) return DZ_ERR_INVALID_ARG;
  if (num_seqs == 0) return DZ_OK;
  float* partial = nullptr;
  int* tickets = nullptr;
  if (splits > 1) {
    if (!workspace || workspace_bytes < dz_paged_attention_workspace_bytes(num_seqs, q_heads, kv_heads, splits))
      return DZ_ERR_WORKSPACE;
    tickets = reinterpret_cast<int*>(workspace);
    partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) +
                                       ((((size_t)num_seqs * kv_heads * 4) + 255) & ~(size_t)255));
  }
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid(kv_heads, num_seqs, splits);
  const int group = q_heads / kv_heads;
  if (dtype == DZ_DTYPE_F16)
    return attention_dispatch<__half>(group, grid, st, (const __half*)qkv, q_row_stride, (__half*)out,
                                      (const __half*)k_cache, (const __half*)v_cache, block_tables,
                                      max_blocks, seq_lens, block_size, kv_heads, scale, splits,
                                      partial, tickets);
  return attention_dispatch<__nv_bfloat16>(group, grid, st, (const __nv_bfloat16*)qkv, q_row_stride,
                                           (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache,
                                           (const __nv_bfloat16*)v_cache, block_tables, max_blocks,
                                           seq_lens, block_size, kv_heads, scale, splits, partial,
                                           tickets);
}

}  // extern "C"

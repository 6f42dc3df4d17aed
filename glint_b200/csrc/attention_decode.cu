// Attention of single tokens over the paged cache, bfloat16 storage, split over the keys.
//
// Memory-bound work: every key and value row of the request is read once per kv head and shared
// by all query heads of its group.  grid = (tokens, kv heads, splits); a block of 128 threads is
// 16 groups of 8 lanes; a group takes one key at a time (one row of a 16-token page per group
// and round), its 8 lanes covering the head in 16-byte pieces.  Each group keeps a running
// (max, sum, weighted values) per query head in 32-bit (src/tensor/flash.rs:65-123); groups are
// merged in shared memory, splits by a second small kernel, both in a fixed order.
// Score = (q.k) * multiplier, then cap * tanh(score / cap) (src/tensor/flash.rs:76-87); keys from
// max(0, pos - window + 1) to pos (src/transformer/forward.rs:574-582).
#include "common.cuh"

namespace glint {

constexpr int DEC_THREADS = 128;
constexpr int DEC_GROUPS = 16;    // 8-lane groups per block

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// CH: 16-byte pieces per lane (head_dim <= 64 * CH).  GH: query heads handled per pass.
template <int CH, int GH>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ positions,
                        const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_pages,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ partial, int nh, int nkv, int hd,
                        int page_size, int num_pages, float multiplier, float cap, int window, int splits,
                        int* __restrict__ status) {
  extern __shared__ float smem[];   // [DEC_GROUPS][GH][hd + 2]
  const int t = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = nh / nkv;
  const int lane8 = threadIdx.x & 7, group = threadIdx.x >> 3;
  // groups of one warp run different numbers of rounds: shuffles name only the group's own lanes
  const unsigned gmask = 0xFFu << (threadIdx.x & 24);
  const int pieces = hd >> 3;                    // 16-byte pieces per row
  const int pos = positions[t];
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n_keys = pos + 1 - first;
  // splits take whole multiples of 16 keys, fixed by the key count alone
  const int per_split = (((n_keys + splits - 1) / splits) + 15) & ~15;
  const int begin = first + split * per_split;
  const int end = min(pos + 1, begin + per_split);
  const int* table = block_table + (size_t)token_seq[t] * max_pages;
  const size_t row_stride = (size_t)hd;
  const int stride_f = hd + 2;

  for (int pass = 0; pass * GH < G; ++pass) {
    float qf[GH][CH * 8], acc[GH][CH * 8], m[GH], l[GH];
#pragma unroll
    for (int j = 0; j < GH; ++j) {
      const int hg = pass * GH + j;
      const __nv_bfloat16* qrow = q + ((size_t)t * nh + kvh * G + (hg < G ? hg : 0)) * hd;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int piece = lane8 + 8 * c;
        if (piece < pieces && hg < G) {
          unpack8(*reinterpret_cast<const uint4*>(qrow + piece * 8), &qf[j][c * 8]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) qf[j][c * 8 + i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[j][c * 8 + i] = 0.f;
      }
      m[j] = -INFINITY;
      l[j] = 0.f;
    }
    for (int key = begin + group; key < end; key += DEC_GROUPS) {
      const int page = table[key / page_size];
      if (page < 0 || page >= num_pages) {
        if (lane8 == 0) atomicExch(status, 3);
        continue;
      }
      const size_t base = (((size_t)page * nkv + kvh) * page_size + (key % page_size)) * row_stride;
      uint4 kraw[CH], vraw[CH];
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int piece = lane8 + 8 * c;
        if (piece < pieces) {
          kraw[c] = __ldg(reinterpret_cast<const uint4*>(k_pool + base + piece * 8));
          vraw[c] = __ldg(reinterpret_cast<const uint4*>(v_pool + base + piece * 8));
        } else {
          kraw[c] = make_uint4(0, 0, 0, 0);
          vraw[c] = make_uint4(0, 0, 0, 0);
        }
      }
      float dot[GH];
#pragma unroll
      for (int j = 0; j < GH; ++j) dot[j] = 0.f;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        float kf[8];
        unpack8(kraw[c], kf);
#pragma unroll
        for (int j = 0; j < GH; ++j)
#pragma unroll
          for (int i = 0; i < 8; ++i) dot[j] = fmaf(qf[j][c * 8 + i], kf[i], dot[j]);
      }
      float e[GH];
#pragma unroll
      for (int j = 0; j < GH; ++j) {
        float d = dot[j];
        d += __shfl_xor_sync(gmask, d, 1);
        d += __shfl_xor_sync(gmask, d, 2);
        d += __shfl_xor_sync(gmask, d, 4);
        const float s = softcap(d * multiplier, cap);
        const float m_new = fmaxf(m[j], s);
        const float corr = __expf(m[j] - m_new);
        e[j] = __expf(s - m_new);
        l[j] = l[j] * corr + e[j];
        m[j] = m_new;
#pragma unroll
        for (int i = 0; i < CH * 8; ++i) acc[j][i] *= corr;
      }
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        float vf[8];
        unpack8(vraw[c], vf);
#pragma unroll
        for (int j = 0; j < GH; ++j)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[j][c * 8 + i] = fmaf(e[j], vf[i], acc[j][c * 8 + i]);
      }
    }
    // ---- merge the 16 groups of the block, in group order -------------------------------------------
    __syncthreads();   // the previous pass may still be reading smem
#pragma unroll
    for (int j = 0; j < GH; ++j) {
      float* dst = smem + ((size_t)group * GH + j) * stride_f;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int piece = lane8 + 8 * c;
        if (piece < pieces)
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[piece * 8 + i] = acc[j][c * 8 + i];
      }
      if (lane8 == 0) {
        dst[hd] = m[j];
        dst[hd + 1] = l[j];
      }
    }
    __syncthreads();
    for (int j = 0; j < GH; ++j) {
      const int hg = pass * GH + j;
      if (hg >= G) break;
      const int head = kvh * G + hg;
      float M = -INFINITY;
      for (int g = 0; g < DEC_GROUPS; ++g) M = fmaxf(M, smem[((size_t)g * GH + j) * stride_f + hd]);
      float L = 0.f;
      float w[DEC_GROUPS];
#pragma unroll
      for (int g = 0; g < DEC_GROUPS; ++g) {
        const float mg = smem[((size_t)g * GH + j) * stride_f + hd];
        w[g] = mg == -INFINITY ? 0.f : __expf(mg - M);
        L += smem[((size_t)g * GH + j) * stride_f + hd + 1] * w[g];
      }
      for (int d = threadIdx.x; d < hd; d += DEC_THREADS) {
        float o = 0.f;
#pragma unroll
        for (int g = 0; g < DEC_GROUPS; ++g) o += smem[((size_t)g * GH + j) * stride_f + d] * w[g];
        if (splits == 1) {
          out[((size_t)t * nh + head) * hd + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
        } else {
          partial[(((size_t)t * nh + head) * splits + split) * (hd + 2) + d] = o;
        }
      }
      if (splits > 1 && threadIdx.x == 0) {
        float* pp = partial + (((size_t)t * nh + head) * splits + split) * (hd + 2);
        pp[hd] = M;
        pp[hd + 1] = L;
      }
    }
  }
}

// out[t, head, :] = sum over splits of partial values, rescaled to the common maximum.  One warp
// reads every split's (max, sum) at once; the weighted values are added in split order.
__global__ void __launch_bounds__(128)
attention_combine_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int hd, int splits) {
  __shared__ float w[64];
  __shared__ float inv_l;
  const size_t row = blockIdx.x;     // t * nh + head
  const float* p = partial + row * splits * (hd + 2);
  if (threadIdx.x < 32) {
    float ms[2], ls[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int s = threadIdx.x + 32 * u;
      ms[u] = s < splits ? p[(size_t)s * (hd + 2) + hd] : -INFINITY;
      ls[u] = s < splits ? p[(size_t)s * (hd + 2) + hd + 1] : 0.f;
    }
    const float M = warp_max(fmaxf(ms[0], ms[1]));
    float L = 0.f;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int s = threadIdx.x + 32 * u;
      const float ws = ms[u] == -INFINITY ? 0.f : __expf(ms[u] - M);
      if (s < 64) w[s] = ws;
      L += ls[u] * ws;
    }
    L = warp_sum(L);
    if (threadIdx.x == 0) inv_l = L > 0.f ? 1.0f / L : 0.f;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < splits; ++s) o += p[(size_t)s * (hd + 2) + d] * w[s];
    out[row * hd + d] = __float2bfloat16_rn(o * inv_l);
  }
}

}  // namespace glint

using namespace glint;

GLINT_API long long glint_attention_decode_partial_floats(int T, int nh, int hd, int splits) {
  return (long long)T * nh * splits * (hd + 2);
}

// head_dim a multiple of 8 up to 512.  `partial` is needed when splits > 1 and must hold
// glint_attention_decode_partial_floats(...) floats.
GLINT_API int glint_attention_decode(const void* q, const void* k_pool, const void* v_pool, const int* positions,
                                     const int* token_seq, const int* block_table, int max_pages, void* out,
                                     float* partial, int T, int nh, int nkv, int hd, int page_size, int num_pages,
                                     float multiplier, float cap, int window, int splits, int* status,
                                     cudaStream_t stream) {
  if (T <= 0) return GLINT_OK;
  if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || splits < 1) return GLINT_ERR_BAD_ARG;
  if (hd % 8 || hd <= 0 || hd > 512) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (splits > 1 && !partial) return GLINT_ERR_BAD_ARG;
  if (nkv > 65535 || splits > 64) return GLINT_ERR_UNSUPPORTED_SIZE;
  dim3 grid(T, nkv, splits);
  const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)k_pool,
                      *vv = (const __nv_bfloat16*)v_pool;
  __nv_bfloat16* oo = (__nv_bfloat16*)out;
#define LAUNCH(CH, GH)                                                                                         \
  {                                                                                                            \
    const size_t smem = (size_t)DEC_GROUPS * GH * (hd + 2) * sizeof(float);                                    \
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<CH, GH>,                                      \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
    if (e != cudaSuccess) return (int)e;                                                                       \
    attention_decode_kernel<CH, GH><<<grid, DEC_THREADS, smem, stream>>>(                                      \
        qq, kk, vv, positions, token_seq, block_table, max_pages, oo, partial, nh, nkv, hd, page_size, num_pages, \
        multiplier, cap, window, splits, status);                                                              \
  }
  if (hd <= 64) LAUNCH(1, 4)
  else if (hd <= 128) LAUNCH(2, 4)
  else if (hd <= 256) LAUNCH(4, 2)
  else LAUNCH(8, 1)
#undef LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (splits > 1) {
    attention_combine_kernel<<<T * nh, 128, 0, stream>>>(partial, oo, hd, splits);
    e = cudaGetLastError();
  }
  return (int)e;
}

// Attention of single tokens over the paged cache, bfloat16 storage, split over the keys.
//
// Memory-bound work: every key and value row of the request is read once per kv head and shared
// by all query heads of its group.  grid = (tokens, kv heads, splits).  One thread of the block
// streams the request's pages (a page of one kv head is contiguous) into a ring of shared-memory
// stages with bulk asynchronous copies that complete on an mbarrier, so the memory system stays
// busy while the other threads compute.  The block's 128 threads are 16 groups of 8 lanes; a
// group takes one key row of the page at a time, its 8 lanes covering the head in 16-byte
// pieces.  Each group keeps a running (max, sum, weighted values) per query head in 32-bit
// (src/tensor/flash.rs:65-123); groups are merged in shared memory in group order.  With more
// than one split, partial results go to a workspace and the block that arrives last at the
// (token, kv head) counter merges the splits in split order and resets the counter: no
// spinning, no second launch, a fixed order of addition.
// Score = (q.k) * multiplier, then cap * tanh(score / cap) (src/tensor/flash.rs:76-87); keys from
// max(0, pos - window + 1) to pos (src/transformer/forward.rs:574-582).
#include "common.cuh"
#include "tcgen05.cuh"

namespace glint {

constexpr int DEC_THREADS = 128;   // consumer threads: 16 groups of 8 lanes
constexpr int DEC_GROUPS = 16;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int DEC_BLOCK = DEC_THREADS + 32;   // plus one producer warp
constexpr int DEC_MAX_STAGES = 8;
constexpr int DEC_MAX_SPLITS = 64;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// Contiguous global -> shared copy that reports its bytes to an mbarrier.
__device__ __forceinline__ void bulk_copy(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   tc::smem_u32(smem_dst)),
               "l"(src), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct DecodeShared {
  uint64_t full[DEC_MAX_STAGES];
  uint64_t empty[DEC_MAX_STAGES];
  int abort_flag;
  int is_last;
  float w[DEC_MAX_SPLITS];
  float inv_l;
};

// CH: 16-byte pieces per lane (head_dim <= 64 * CH).  GH: query heads handled per pass.
template <int CH, int GH>
__global__ void __launch_bounds__(DEC_BLOCK, 2)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ positions,
                        const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_pages,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ partial, int* __restrict__ counters,
                        int nh, int nkv, int hd, int page_size, int num_pages, float multiplier, float cap,
                        int window, int splits, int stages, int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t dec_smem[];
  const int t = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = nh / nkv;
  const int lane8 = threadIdx.x & 7, group = threadIdx.x >> 3;
  // groups of one warp may see different key ranges: shuffles name only the group's own lanes
  const unsigned gmask = 0xFFu << (threadIdx.x & 24);
  const int pieces = hd >> 3;                    // 16-byte pieces per row
  const int pos = positions[t];
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  // the split takes whole pages, counted from the page that holds the first key
  const int page_lo = first / page_size, page_hi = pos / page_size;
  const int pages_per_split = (page_hi - page_lo + splits) / splits;
  const int my_lo = page_lo + split * pages_per_split;
  const int my_hi = min(page_hi + 1, my_lo + pages_per_split);     // exclusive
  const int n_pages = max(0, my_hi - my_lo);
  const int* table = block_table + (size_t)token_seq[t] * max_pages;
  const uint32_t page_bytes = (uint32_t)page_size * hd * 2;
  const int stride_f = hd + 2;

  // shared memory: stages of [K page | V page], then the merge area, then barriers
  uint8_t* ring = dec_smem;
  float* merge = reinterpret_cast<float*>(ring + (size_t)stages * 2 * page_bytes);
  DecodeShared* sh = reinterpret_cast<DecodeShared*>(merge + (size_t)DEC_WARPS * GH * stride_f);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      tc::mbar_init(&sh->full[s], 1);
      tc::mbar_init(&sh->empty[s], DEC_WARPS);
    }
    sh->abort_flag = 0;
    sh->is_last = 0;
    tc::fence_barrier_init();
  }
  __syncthreads();
  volatile int* abort_flag = &sh->abort_flag;

  const int n_pass = (G + GH - 1) / GH;
  const int n_iter = n_pages * n_pass;       // every pass streams the split's pages again

  if (threadIdx.x >= DEC_THREADS) {
    // ---- producer warp: looks up 32 pages at a time, one lane starts the copies ----------------------
    const int lane = threadIdx.x & 31;
    for (int base = 0; base < n_iter; base += 32) {
      const int mine = base + lane;
      int page = 0;
      if (mine < n_iter) {
        page = table[my_lo + mine % n_pages];
        if (page < 0 || page >= num_pages) {     // never read outside the pool; report it
          atomicExch(status, 3);
          page = 0;
        }
      }
      for (int j = 0; j < 32 && base + j < n_iter; ++j) {
        const int it = base + j;
        const int pg = __shfl_sync(0xffffffffu, page, j);
        if (lane == 0) {
          const int s = it % stages;
          bool ok = true;
          if (it >= stages) ok = tc::mbar_wait(&sh->empty[s], ((it / stages) - 1) & 1, abort_flag);
          if (ok) {
            const size_t off = ((size_t)pg * nkv + kvh) * page_size * hd;
            tc::mbar_expect_tx(&sh->full[s], 2 * page_bytes);
            bulk_copy(ring + (size_t)s * 2 * page_bytes, k_pool + off, page_bytes, &sh->full[s]);
            bulk_copy(ring + (size_t)s * 2 * page_bytes + page_bytes, v_pool + off, page_bytes, &sh->full[s]);
          }
        }
      }
    }
    return;
  }

  const float score_scale = cap > 0.f ? multiplier / cap : multiplier;
  int it = 0;
  for (int pass = 0; pass < n_pass; ++pass) {
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
    for (int pi = 0; pi < n_pages; ++pi, ++it) {
      const int s = it % stages;
      const bool ok = tc::mbar_wait(&sh->full[s], (it / stages) & 1, abort_flag);
      const uint8_t* kpage = ring + (size_t)s * 2 * page_bytes;
      const uint8_t* vpage = kpage + page_bytes;
      const int key0 = (my_lo + pi) * page_size;
      for (int r = group; r < page_size && ok; r += DEC_GROUPS) {
        const int key = key0 + r;
        if (key < first || key > pos) continue;        // uniform within the group
        float dot[GH];
#pragma unroll
        for (int j = 0; j < GH; ++j) dot[j] = 0.f;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const int piece = lane8 + 8 * c;
          if (piece < pieces) {
            float kf[8];
            unpack8(*reinterpret_cast<const uint4*>(kpage + ((size_t)r * hd + piece * 8) * 2), kf);
#pragma unroll
            for (int j = 0; j < GH; ++j)
#pragma unroll
              for (int i = 0; i < 8; ++i) dot[j] = fmaf(qf[j][c * 8 + i], kf[i], dot[j]);
          }
        }
        float e[GH];
#pragma unroll
        for (int j = 0; j < GH; ++j) {
          float d = dot[j];
          d += __shfl_xor_sync(gmask, d, 1);
          d += __shfl_xor_sync(gmask, d, 2);
          d += __shfl_xor_sync(gmask, d, 4);
          const float sc = cap > 0.f ? cap * tanhf(d * score_scale) : d * score_scale;
          const float m_new = fmaxf(m[j], sc);
          const float corr = __expf(m[j] - m_new);
          e[j] = __expf(sc - m_new);
          l[j] = l[j] * corr + e[j];
          m[j] = m_new;
#pragma unroll
          for (int i = 0; i < CH * 8; ++i) acc[j][i] *= corr;
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const int piece = lane8 + 8 * c;
          if (piece < pieces) {
            float vf[8];
            unpack8(*reinterpret_cast<const uint4*>(vpage + ((size_t)r * hd + piece * 8) * 2), vf);
#pragma unroll
            for (int j = 0; j < GH; ++j)
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[j][c * 8 + i] = fmaf(e[j], vf[i], acc[j][c * 8 + i]);
          }
        }
      }
      __syncwarp();
      if ((threadIdx.x & 31) == 0) tc::mbar_arrive(&sh->empty[s]);   // this warp is done with stage s
    }
    // ---- merge: first the 4 groups of each warp by shuffles, then the 4 warps in shared memory -----
#pragma unroll
    for (int j = 0; j < GH; ++j) {
#pragma unroll
      for (int x = 8; x <= 16; x <<= 1) {
        const float m_o = __shfl_xor_sync(0xffffffffu, m[j], x);
        const float l_o = __shfl_xor_sync(0xffffffffu, l[j], x);
        const float M = fmaxf(m[j], m_o);
        const float wa = m[j] == -INFINITY ? 0.f : __expf(m[j] - M);
        const float wb = m_o == -INFINITY ? 0.f : __expf(m_o - M);
        l[j] = l[j] * wa + l_o * wb;
        m[j] = M;
#pragma unroll
        for (int i = 0; i < CH * 8; ++i) {
          const float a_o = __shfl_xor_sync(0xffffffffu, acc[j][i], x);
          acc[j][i] = acc[j][i] * wa + a_o * wb;
        }
      }
    }
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) < 8) {
#pragma unroll
      for (int j = 0; j < GH; ++j) {
        float* dst = merge + ((size_t)warp * GH + j) * stride_f;
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
    }
    consumer_sync();
    for (int j = 0; j < GH; ++j) {
      const int hg = pass * GH + j;
      if (hg >= G) break;
      const int head = kvh * G + hg;
      float M = -INFINITY;
#pragma unroll
      for (int g = 0; g < DEC_WARPS; ++g) M = fmaxf(M, merge[((size_t)g * GH + j) * stride_f + hd]);
      float L = 0.f;
      float w[DEC_WARPS];
#pragma unroll
      for (int g = 0; g < DEC_WARPS; ++g) {
        const float mg = merge[((size_t)g * GH + j) * stride_f + hd];
        w[g] = mg == -INFINITY ? 0.f : __expf(mg - M);
        L += merge[((size_t)g * GH + j) * stride_f + hd + 1] * w[g];
      }
      for (int d = threadIdx.x; d < hd; d += DEC_THREADS) {
        float o = 0.f;
#pragma unroll
        for (int g = 0; g < DEC_WARPS; ++g) o += merge[((size_t)g * GH + j) * stride_f + d] * w[g];
        if (splits == 1) {
          out[((size_t)t * nh + head) * hd + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
        } else {
          partial[(((size_t)t * nh + head) * splits + split) * stride_f + d] = o;
        }
      }
      if (splits > 1 && threadIdx.x == 0) {
        float* pp = partial + (((size_t)t * nh + head) * splits + split) * stride_f;
        pp[hd] = M;
        pp[hd + 1] = L;
      }
    }
    consumer_sync();   // the merge area is reused by the next pass
  }

  // ---- the last block of this (token, kv head) merges the splits, in split order ---------------------
  if (splits > 1) {
    __threadfence();
    consumer_sync();
    if (threadIdx.x == 0) {
      const int prev = atomicAdd(&counters[t * nkv + kvh], 1);
      sh->is_last = (prev == splits - 1);
    }
    consumer_sync();
    if (sh->is_last) {
      __threadfence();
      for (int hg = 0; hg < G; ++hg) {
        const size_t row = (size_t)t * nh + kvh * G + hg;
        const float* p = partial + row * splits * stride_f;
        if (threadIdx.x < 32) {
          float ms[2], ls[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int s = threadIdx.x + 32 * u;
            ms[u] = s < splits ? __ldcg(p + (size_t)s * stride_f + hd) : -INFINITY;
            ls[u] = s < splits ? __ldcg(p + (size_t)s * stride_f + hd + 1) : 0.f;
          }
          const float M = warp_max(fmaxf(ms[0], ms[1]));
          float L = 0.f;
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const float ws = ms[u] == -INFINITY ? 0.f : __expf(ms[u] - M);
            sh->w[threadIdx.x + 32 * u] = ws;
            L += ls[u] * ws;
          }
          L = warp_sum(L);
          if (threadIdx.x == 0) sh->inv_l = L > 0.f ? 1.0f / L : 0.f;
        }
        consumer_sync();
        // warp w adds splits w, w+4, ... (all their loads in flight), then the 4 warps are added in order
        {
          const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
          for (int d0 = 0; d0 < hd; d0 += 32 * 4) {
            const int d = d0 + lane * 4;
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            if (d < hd) {
#pragma unroll 4
              for (int sidx = warp; sidx < splits; sidx += DEC_WARPS) {
                const float2 lo = __ldcg(reinterpret_cast<const float2*>(p + (size_t)sidx * stride_f + d));
                const float2 hi = __ldcg(reinterpret_cast<const float2*>(p + (size_t)sidx * stride_f + d + 2));
                const float ws = sh->w[sidx];
                o.x += lo.x * ws; o.y += lo.y * ws; o.z += hi.x * ws; o.w += hi.y * ws;
              }
              float* dst = merge + (size_t)warp * stride_f + d;
              dst[0] = o.x; dst[1] = o.y; dst[2] = o.z; dst[3] = o.w;
            }
          }
        }
        consumer_sync();
        for (int d = threadIdx.x; d < hd; d += DEC_THREADS) {
          float o = 0.f;
#pragma unroll
          for (int wv = 0; wv < DEC_WARPS; ++wv) o += merge[(size_t)wv * stride_f + d];
          out[row * hd + d] = __float2bfloat16_rn(o * sh->inv_l);
        }
        consumer_sync();
      }
      if (threadIdx.x == 0) counters[t * nkv + kvh] = 0;   // ready for the next launch on this stream
    }
  }
  if (threadIdx.x == 0 && sh->abort_flag) atomicExch(status, 4);
}

}  // namespace glint

using namespace glint;

GLINT_API long long glint_attention_decode_partial_floats(int T, int nh, int hd, int splits) {
  return (long long)T * nh * splits * (hd + 2);
}

// head_dim a multiple of 8 up to 512, splits up to 64.  When splits > 1, `partial` must hold
// glint_attention_decode_partial_floats(...) floats and `counters` T * nkv zeroed ints (the
// kernel leaves them zero).
GLINT_API int glint_attention_decode(const void* q, const void* k_pool, const void* v_pool, const int* positions,
                                     const int* token_seq, const int* block_table, int max_pages, void* out,
                                     float* partial, int* counters, int T, int nh, int nkv, int hd, int page_size,
                                     int num_pages, float multiplier, float cap, int window, int splits,
                                     int* status, cudaStream_t stream) {
  if (T <= 0) return GLINT_OK;
  if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || splits < 1) return GLINT_ERR_BAD_ARG;
  if (hd % 8 || hd <= 0 || hd > 512) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (splits > 1 && (!partial || !counters)) return GLINT_ERR_BAD_ARG;
  if (nkv > 65535 || splits > DEC_MAX_SPLITS) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)q) & 15) return GLINT_ERR_UNSUPPORTED_SIZE;
  const long long page_bytes = (long long)page_size * hd * 2;
  dim3 grid(T, nkv, splits);
  const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)k_pool,
                      *vv = (const __nv_bfloat16*)v_pool;
  __nv_bfloat16* oo = (__nv_bfloat16*)out;
#define LAUNCH(CH, GH)                                                                                         \
  {                                                                                                            \
    const long long fixed = (long long)DEC_WARPS * GH * (hd + 2) * 4 + sizeof(DecodeShared) + 128;            \
    int stages = (int)((110 * 1024 - fixed) / (2 * page_bytes));                                                \
    if (stages > DEC_MAX_STAGES) stages = DEC_MAX_STAGES;                                                      \
    if (stages < 2) stages = 2;                                                                                \
    const long long smem = stages * 2 * page_bytes + fixed;                                                    \
    if (smem > 227 * 1024) return GLINT_ERR_UNSUPPORTED_SIZE;                                                  \
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<CH, GH>,                                      \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
    if (e != cudaSuccess) return (int)e;                                                                       \
    attention_decode_kernel<CH, GH><<<grid, DEC_BLOCK, smem, stream>>>(                                      \
        qq, kk, vv, positions, token_seq, block_table, max_pages, oo, partial, counters, nh, nkv, hd, page_size, \
        num_pages, multiplier, cap, window, splits, stages, status);                                           \
  }
  if (hd <= 64) LAUNCH(1, 4)
  else if (hd <= 128) LAUNCH(2, 4)
  else if (hd <= 256) LAUNCH(4, 2)
  else LAUNCH(8, 1)
#undef LAUNCH
  return (int)cudaGetLastError();
}

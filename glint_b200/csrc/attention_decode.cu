// Attention of single tokens over the paged cache, bfloat16 storage, split over the keys.
//
// Memory-bound work: every key and value row of the request is read once per kv head and shared
// by all query heads of its group.  grid = (tokens, kv heads, splits).  A producer warp streams
// the request's pages into a ring of shared-memory stages with TMA tile loads (128-byte swizzle,
// completion on an mbarrier); four consumer warps take the pages in turn.  A consumer computes,
// per 16 keys, scores^T = K q^T and out^T += V^T p^T with mma.sync tiles in which the N
// dimension (8) holds the query heads of the group, so that keys and values are the large
// operands read straight from shared memory and nothing is padded to a 128-row tile.  Scores,
// soft cap, running max/sum and the output accumulator are 32-bit (src/tensor/flash.rs:65-123);
// probabilities are rounded to bfloat16 for the second product.  The four warps are merged in
// shared memory in warp order.  With more than one split, the splits of a (token, kv head) are
// the blocks of one thread-block cluster: every block leaves its partial result in its own shared
// memory, and after a cluster barrier each block adds up, in split order, its share of the output
// elements from the shared memory of all of them (distributed shared memory): no workspace in
// global memory, no counter, no second launch, a fixed order of addition.
// Score = (q.k) * multiplier, then cap * tanh(score / cap) (src/tensor/flash.rs:76-87); keys from
// max(0, pos - window + 1) to pos (src/transformer/forward.rs:574-582).
#include "common.cuh"
#include "tcgen05.cuh"

namespace glint {

constexpr int DEC_WARPS = 4;                      // consumer warps
constexpr int DEC_THREADS = DEC_WARPS * 32;
constexpr int DEC_BLOCK = DEC_THREADS + 32;       // plus the producer warp
constexpr int DEC_MAX_STAGES = 12;
constexpr int DEC_MAX_SPLITS = 16;                // blocks of a cluster
constexpr int DEC_HEADS = 8;                      // query heads per pass (the MMA's N)
constexpr int SUB_BYTES_PER_ROW = 128;            // one swizzle row: 64 bf16

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Byte offset of (row, 16-byte chunk) inside a tile of rows x 128 bytes stored with the 128-byte
// swizzle: chunk c of row r sits at chunk (c ^ (r & 7)).
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return (uint32_t)(row * SUB_BYTES_PER_ROW + ((chunk ^ (row & 7)) << 4));
}

struct DecodeShared {
  uint64_t full[DEC_MAX_STAGES];
  uint64_t empty[DEC_MAX_STAGES];
  int abort_flag;
};

// HD: register capacity (head_dim <= HD; head_dim and page_size are multiples of 16).
template <int HD>
__global__ void __launch_bounds__(DEC_BLOCK, 2)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const __nv_bfloat16* __restrict__ q, const int* __restrict__ positions,
                        const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_pages,
                        __nv_bfloat16* __restrict__ out, int nh, int nkv, int hd, int page_size, int num_pages, float multiplier, float cap,
                        int window, int splits, int stages, int whole_page, int* __restrict__ status) {
  extern __shared__ uint8_t dec_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dec_raw) + 1023) & ~(uintptr_t)1023);
  const int t = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = nh / nkv;
  const int HP = G < DEC_HEADS ? G : DEC_HEADS;          // heads per pass
  const int n_pass = (G + DEC_HEADS - 1) / DEC_HEADS;
  const int hd16 = hd >> 4;
  const int nsub = (hd + 63) >> 6;                        // 64-wide column tiles of a page
  const uint32_t sub_bytes = (uint32_t)page_size * SUB_BYTES_PER_ROW;
  const uint32_t page_bytes = nsub * sub_bytes;
  const int pos = positions[t];
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  // the split takes whole pages, counted from the page that holds the first key
  const int page_lo = first / page_size, page_hi = pos / page_size;
  const int pages_per_split = (page_hi - page_lo + splits) / splits;
  const int my_lo = page_lo + split * pages_per_split;
  const int my_hi = min(page_hi + 1, my_lo + pages_per_split);     // exclusive
  const int n_pages = max(0, my_hi - my_lo);
  const int n_iter = n_pages * n_pass;                    // every pass streams the split's pages again
  const int* table = block_table + (size_t)token_seq[t] * max_pages;
  const int stride_f = hd + 2;

  float* merge = reinterpret_cast<float*>(ring + (size_t)stages * 2 * page_bytes);
  float* xchg = merge + (size_t)DEC_WARPS * HP * stride_f;      // [G][hd + 2]: what the other splits read
  DecodeShared* sh = reinterpret_cast<DecodeShared*>(xchg + (splits > 1 ? (size_t)G * stride_f : 0));

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      tc::mbar_init(&sh->full[s], 1);
      tc::mbar_init(&sh->empty[s], 1);
    }
    sh->abort_flag = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(&map_k);
    tc::tma_prefetch_desc(&map_v);
  }
  __syncthreads();
  pdl_wait_release();                           // the keys of this step and q come from earlier kernels
  volatile int* abort_flag = &sh->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (warp == DEC_WARPS) {
    // ---- producer warp: looks up 32 pages at a time, one lane starts the tile loads ------------------
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
        if (tc::elect_one()) {                   // elect.sync: operands of the copies stay in uniform registers
          const int s = it % stages;
          bool ok = true;
          if (it >= stages) ok = tc::mbar_wait(&sh->empty[s], ((it / stages) - 1) & 1, abort_flag);
          if (ok) {
            uint8_t* kdst = ring + (size_t)s * 2 * page_bytes;
            const int row = (pg * nkv + kvh) * page_size;
            tc::mbar_expect_tx(&sh->full[s], 2 * page_bytes);
            if (whole_page) {      // one box per page: the copy unit spends about 65 cycles on every box
              tc::tma_load_3d(kdst, &map_k, &sh->full[s], 0, row, 0);
              tc::tma_load_3d(kdst + page_bytes, &map_v, &sh->full[s], 0, row, 0);
            } else {
              for (int sub = 0; sub < nsub; ++sub) {
                tc::tma_load_2d(kdst + sub * sub_bytes, &map_k, &sh->full[s], sub * 64, row);
                tc::tma_load_2d(kdst + page_bytes + sub * sub_bytes, &map_v, &sh->full[s], sub * 64, row);
              }
            }
          }
        }
      }
    }
  } else {
  // ---- consumer warps ----------------------------------------------------------------------------------
  const int g = lane >> 2, tq = lane & 3;
  const float score_scale = cap > 0.f ? multiplier / cap : multiplier;
  const uint32_t ring_addr = tc::smem_u32(ring);
  for (int pass = 0; pass < n_pass; ++pass) {
    // q^T as the B operand: this thread holds dims (16 ks + 2 tq, +1) and (+8, +9) of head g
    uint32_t qb[HD / 16][2];
    {
      const int hg = pass * DEC_HEADS + g;
      const __nv_bfloat16* qrow = q + ((size_t)t * nh + kvh * G + (hg < G ? hg : 0)) * hd;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const bool in = ks < hd16 && hg < G;
        qb[ks][0] = in ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + tq * 2) : 0u;
        qb[ks][1] = in ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + tq * 2) : 0u;
      }
    }
    float o[HD / 16][4];
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    // Iteration `it` (over all passes) belongs to warp it % 4 and stage it % stages; the stage count
    // is a multiple of 4, so a stage is always read by the same warp and that warp sees every
    // phase of the stage's barrier (a waiter that skipped a phase would match the wrong parity).
    const int it_lo = pass * n_pages, it_hi = it_lo + n_pages;
    for (int it = it_lo + ((warp - it_lo) % DEC_WARPS + DEC_WARPS) % DEC_WARPS; it < it_hi; it += DEC_WARPS) {
      const int pi = it - it_lo;
      const int s = it % stages;
      const bool ok = tc::mbar_wait(&sh->full[s], (it / stages) & 1, abort_flag);
      const uint32_t kbase = ring_addr + (uint32_t)s * 2 * page_bytes;
      const uint32_t vbase = kbase + page_bytes;
      for (int tile = 0; tile * 16 < page_size && ok; ++tile) {
        const int key0 = (my_lo + pi) * page_size + tile * 16;
        if (key0 > pos || key0 + 15 < first) continue;            // the whole tile is masked
        float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          if (ks < hd16) {
            uint32_t a[4];
            const int row = tile * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            ldsm_x4(a, kbase + (ks >> 2) * sub_bytes + swz(row, (ks & 3) * 2 + (lane >> 4)));
            mma16816(sc, a, qb[ks][0], qb[ks][1]);
          }
        }
        // sc[0], sc[1]: key g, heads 2tq, 2tq+1;  sc[2], sc[3]: key g + 8, same heads
        const bool va = key0 + g >= first && key0 + g <= pos;
        const bool vb = key0 + g + 8 >= first && key0 + g + 8 <= pos;
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float xa = sc[h] * score_scale, xb = sc[2 + h] * score_scale;
          if (cap > 0.f) {
            xa = cap * tanhf(xa);
            xb = cap * tanhf(xb);
          }
          xa = va ? xa : -INFINITY;
          xb = vb ? xb : -INFINITY;
          float mx = fmaxf(xa, xb);
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
          const float m_new = fmaxf(m[h], mx);
          const float base = m_new == -INFINITY ? 0.f : m_new;
          corr[h] = __expf(m[h] - base);
          const float pa = __expf(xa - base), pb = __expf(xb - base);
          l[h] = l[h] * corr[h] + pa + pb;       // this thread's keys only; lanes are added at the end
          m[h] = m_new;
          sc[h] = pa;
          sc[2 + h] = pb;
        }
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
          for (int i = 0; i < HD / 16; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[1];
            o[i][2] *= corr[0];
            o[i][3] *= corr[1];
          }
        }
        // value rows of masked keys may hold anything (a page's unwritten tail): zero them, since
        // 0 * NaN would poison the product.  Only the first and last tile of a range get here.
        if (key0 < first || key0 + 15 > pos) {
          for (int r = 0; r < 16; ++r) {
            const int key = key0 + r;
            if (key >= first && key <= pos) continue;
            for (int c = lane; c < nsub * 8; c += 32)
              *reinterpret_cast<uint4*>(ring + (size_t)s * 2 * page_bytes + page_bytes + (c >> 3) * sub_bytes +
                                        (tile * 16 + r) * SUB_BYTES_PER_ROW + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          __syncwarp();
        }
        // p^T as the B operand: keys (2tq, 2tq+1) and (+8) of head g, by an 8x8 transpose in the warp
        const uint32_t b0 = movmatrix_trans(pack2(sc[0], sc[1]));
        const uint32_t b1 = movmatrix_trans(pack2(sc[2], sc[3]));
#pragma unroll
        for (int blk = 0; blk < HD / 16; ++blk) {
          if (blk < hd16) {
            uint32_t a[4];
            const int i = lane >> 3;
            const int key = tile * 16 + (lane & 7) + (i >> 1) * 8;
            ldsm_x4_trans(a, vbase + (blk >> 2) * sub_bytes + swz(key, (blk & 3) * 2 + (i & 1)));
            mma16816(o[blk], a, b0, b1);
          }
        }
      }
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->empty[s]);     // this warp is done with stage s
    }
    // ---- this warp's totals, then the four warps are merged in shared memory, in warp order ----------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 4);
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 8);
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 16);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int head = 2 * tq + h;
      if (head < HP && pass * DEC_HEADS + head < G) {
        float* dst = merge + ((size_t)warp * HP + head) * stride_f;
#pragma unroll
        for (int blk = 0; blk < HD / 16; ++blk) {
          if (blk < hd16) {
            dst[blk * 16 + g] = o[blk][h];
            dst[blk * 16 + g + 8] = o[blk][2 + h];
          }
        }
        if (g == 0) {
          dst[hd] = m[h];
          dst[hd + 1] = l[h];
        }
      }
    }
    consumer_sync();
    for (int j = 0; j < HP; ++j) {
      const int hg = pass * DEC_HEADS + j;
      if (hg >= G) break;
      const int head = kvh * G + hg;
      float M = -INFINITY;
#pragma unroll
      for (int wv = 0; wv < DEC_WARPS; ++wv) M = fmaxf(M, merge[((size_t)wv * HP + j) * stride_f + hd]);
      float L = 0.f;
      float w[DEC_WARPS];
#pragma unroll
      for (int wv = 0; wv < DEC_WARPS; ++wv) {
        const float mg = merge[((size_t)wv * HP + j) * stride_f + hd];
        w[wv] = mg == -INFINITY ? 0.f : __expf(mg - M);
        L += merge[((size_t)wv * HP + j) * stride_f + hd + 1] * w[wv];
      }
      for (int d = threadIdx.x; d < hd; d += DEC_THREADS) {
        float ov = 0.f;
#pragma unroll
        for (int wv = 0; wv < DEC_WARPS; ++wv) ov += merge[((size_t)wv * HP + j) * stride_f + d] * w[wv];
        if (splits == 1) {
          out[((size_t)t * nh + head) * hd + d] = __float2bfloat16_rn(L > 0.f ? ov / L : 0.f);
        } else {
          xchg[(size_t)hg * stride_f + d] = ov;
        }
      }
      if (splits > 1 && threadIdx.x == 0) {
        xchg[(size_t)hg * stride_f + hd] = M;
        xchg[(size_t)hg * stride_f + hd + 1] = L;
      }
    }
    consumer_sync();   // the merge area is reused by the next pass
  }

  }  // consumer warps

  // ---- the splits of this (token, kv head) are merged across the cluster, in split order ------------
  if (splits > 1) {
    cluster_sync();                                  // every block's xchg is written and visible
    if (warp < DEC_WARPS) {
      const int total = G * hd;
      const int per = (total + splits - 1) / splits; // this block's share of the output elements
      const uint32_t xchg_addr = tc::smem_u32(xchg);
      for (int e = split * per + (int)threadIdx.x; e < min(total, (split + 1) * per); e += DEC_THREADS) {
        const int hg = e / hd, d = e - hg * hd;
        const uint32_t row_addr = xchg_addr + (uint32_t)(hg * stride_f) * 4;
        float ms[DEC_MAX_SPLITS], ls[DEC_MAX_SPLITS], os[DEC_MAX_SPLITS];
        float M = -INFINITY;
#pragma unroll
        for (int sidx = 0; sidx < DEC_MAX_SPLITS; ++sidx) {
          if (sidx < splits) {
            const uint32_t peer = cluster_map(row_addr, sidx);
            ms[sidx] = cluster_load(peer + hd * 4);
            ls[sidx] = cluster_load(peer + (hd + 1) * 4);
            os[sidx] = cluster_load(peer + d * 4);
            M = fmaxf(M, ms[sidx]);
          }
        }
        float L = 0.f, ov = 0.f;
#pragma unroll
        for (int sidx = 0; sidx < DEC_MAX_SPLITS; ++sidx) {
          if (sidx < splits) {
            const float ws = ms[sidx] == -INFINITY ? 0.f : __expf(ms[sidx] - M);
            L += ls[sidx] * ws;
            ov += os[sidx] * ws;
          }
        }
        out[((size_t)t * nh + kvh * G + hg) * hd + d] = __float2bfloat16_rn(L > 0.f ? ov / L : 0.f);
      }
    }
    cluster_sync();                                  // nobody leaves while its shared memory is being read
  }
  if (threadIdx.x == 0 && sh->abort_flag) atomicExch(status, 4);
}

// ---- host side ---------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn decode_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// A pool [pages][kv heads][page_size][head_dim] viewed as rows of head_dim, in boxes of
// page_size rows x 64 columns with the 128-byte swizzle.  When head_dim is a multiple of 64 the
// 64-column slices become a third dimension, and one box brings a whole page as
// [slice][row][64 columns], which is the layout the separate boxes give.
static int pool_map(CUtensorMap* map, const void* pool, long long rows, int hd, int page_size, bool whole_page) {
  EncodeTiledFn fn = decode_encode_fn();
  if (!fn) return GLINT_ERR_BAD_ARG;
  if (whole_page) {
    cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(hd / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)hd * 2, 128};
    cuuint32_t box[3] = {64, (cuuint32_t)page_size, (cuuint32_t)(hd / 64)};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(pool), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? GLINT_OK : GLINT_ERR_BAD_ARG;
  }
  cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)page_size};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? GLINT_OK : GLINT_ERR_BAD_ARG;
}

}  // namespace glint

using namespace glint;

// Largest number of splits (blocks of one cluster) this device takes: 8 everywhere, 16 where the
// driver schedules clusters of that size for this kernel's launch shape.
GLINT_API int glint_attention_decode_max_splits() { return DEC_MAX_SPLITS; }

GLINT_API int glint_attention_decode_supported(int nh, int nkv, int hd, int page_size) {
  return (nkv > 0 && nh % nkv == 0 && hd % 16 == 0 && hd >= 16 && hd <= 256 && page_size % 16 == 0 &&
          page_size >= 16 && page_size <= 256) ? 1 : 0;
}

// head_dim a multiple of 16 up to 256, page_size a multiple of 16 up to 256, splits up to 16 (more
// than 8 need a device that schedules such clusters; the launch fails with an error otherwise).
GLINT_API int glint_attention_decode(const void* q, const void* k_pool, const void* v_pool, const int* positions,
                                     const int* token_seq, const int* block_table, int max_pages, void* out,
                                     int T, int nh, int nkv, int hd, int page_size,
                                     int num_pages, float multiplier, float cap, int window, int splits,
                                     int* status, cudaStream_t stream) {
  if (T <= 0) return GLINT_OK;
  if (page_size <= 0 || splits < 1 || nkv <= 0) return GLINT_ERR_BAD_ARG;
  if (!glint_attention_decode_supported(nh, nkv, hd, page_size)) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (nkv > 65535 || splits > DEC_MAX_SPLITS) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)k_pool | (uintptr_t)v_pool) & 15 || ((uintptr_t)q & 3)) return GLINT_ERR_UNSUPPORTED_SIZE;
  CUtensorMap map_k, map_v;
  const long long rows = (long long)num_pages * nkv * page_size;
  const int whole_page = (hd % 64 == 0 && page_size <= 256) ? 1 : 0;
  int rc = pool_map(&map_k, k_pool, rows, hd, page_size, whole_page);
  if (rc != GLINT_OK) return rc;
  rc = pool_map(&map_v, v_pool, rows, hd, page_size, whole_page);
  if (rc != GLINT_OK) return rc;
  const int G = nh / nkv;
  const int HP = G < DEC_HEADS ? G : DEC_HEADS;
  const long long page_bytes = (long long)((hd + 63) / 64) * page_size * SUB_BYTES_PER_ROW;
  const long long fixed = (long long)DEC_WARPS * HP * (hd + 2) * 4 + (splits > 1 ? (long long)G * (hd + 2) * 4 : 0) +
                          sizeof(DecodeShared) + 1024 + 64;
  // a multiple of the consumer warps (see the kernel), as many as let two blocks share an SM
  int stages = (int)((110 * 1024 - fixed) / (2 * page_bytes)) / DEC_WARPS * DEC_WARPS;
  if (stages > DEC_MAX_STAGES) stages = DEC_MAX_STAGES;
  if (stages < DEC_WARPS) stages = DEC_WARPS;
  const long long smem = stages * 2 * page_bytes + fixed;
  if (smem > 227 * 1024) return GLINT_ERR_UNSUPPORTED_SIZE;
  dim3 grid(T, nkv, splits);
  const __nv_bfloat16* qq = (const __nv_bfloat16*)q;
  __nv_bfloat16* oo = (__nv_bfloat16*)out;
#define LAUNCH(HD)                                                                                              \
  {                                                                                                             \
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem);                                                            \
    if (e != cudaSuccess) return (int)e;                                                                        \
    if (splits > 8) {                                                                                           \
      e = cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);   \
      if (e != cudaSuccess) return (int)e;                                                                      \
    }                                                                                                           \
    e = launch_kernel_cluster(attention_decode_kernel<HD>, grid, dim3(DEC_BLOCK), (size_t)smem, stream, splits,  \
                              map_k, map_v, qq, positions, token_seq, block_table, max_pages, oo, nh, nkv, hd,    \
                              page_size, num_pages, multiplier, cap, window, splits, stages, whole_page, status); \
    if (e != cudaSuccess) return (int)e;                                                                        \
  }
  if (hd <= 64) LAUNCH(64)
  else if (hd <= 128) LAUNCH(128)
  else LAUNCH(256)
#undef LAUNCH
  return (int)cudaGetLastError();
}

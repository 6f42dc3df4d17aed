// Attention of single tokens over the paged cache, bfloat16 storage, split over the keys.
//
// Memory-bound work: every key and value row of the request is read once per kv head and shared
// by all query heads of its group.  grid = (tokens, kv heads, splits).  A producer warp streams
// the request's pages into a ring of shared-memory stages with TMA tile loads (128-byte swizzle,
// completion on an mbarrier); three or four consumer warps take the pages in turn.  A consumer computes,
// per 16 keys, scores^T = K q^T and out^T += V^T p^T with mma.sync tiles in which the N
// dimension (8) holds the query heads of the group, so that keys and values are the large
// operands read straight from shared memory and nothing is padded to a 128-row tile.  Scores,
// soft cap, running max/sum and the output accumulator are 32-bit (src/tensor/flash.rs:65-123);
// probabilities are rounded to bfloat16 for the second product.  The warps are merged in
// shared memory in warp order.  With more than one split, the splits of a (token, kv head) are
// the blocks of one thread-block cluster: every block leaves its partial result in its own shared
// memory, and after a cluster barrier each block adds up, in split order, its share of the output
// elements from the shared memory of all of them (distributed shared memory): no workspace in
// global memory, no counter, no second launch, a fixed order of addition.
// A second kernel (attention_decode_stream_kernel, further down) cuts the pages of ALL (token, kv head)
// pairs of a launch into equal shares for two blocks per SM instead, for launches whose contexts are of
// uneven length or whose clusters would not fill the SMs; the runtime chooses between the two.
// Score = (q.k) * multiplier, then cap * tanh(score / cap) (src/tensor/flash.rs:76-87); keys from
// max(0, pos - window + 1) to pos (src/transformer/forward.rs:574-582).
#include "common.cuh"
#include "tcgen05.cuh"

namespace glint {

// Consumer warps: a template parameter of both kernels, chosen by the host.  The ring holds a multiple of this
// many stages (see the kernels), and two blocks of an SM have room for six stages of a page of head size 256 each
// but not for eight, so three warps keep 96 KB in flight per block where four keep 64 KB; the products are a
// tenth of a block's time either way.  64 requests x 4 kv heads at 2176 keys: 99.9 -> 89.6 us with three (0.97
// of the measured HBM bandwidth); 56 requests of uneven length in the page-sharing kernel: 105.8 -> 101.0 us.
// Launches of a few tokens keep four: their blocks hold 75 KB of shared memory instead of 107, and whole decode
// steps of the 9B shape at 1 to 8 requests are 4 to 7 % faster with them (4.16 against 4.40 ms at one request:
// the products on either side of the attention kernel lose their overlap with it), while from 16 requests on
// three are faster (6.08 against 6.27 ms; 2B shape at 64: 4.03 against 4.29 ms).
static inline int decode_consumer_warps(int tokens) { return tokens <= 8 ? 4 : 3; }
constexpr int DEC_MAX_STAGES = 12;
constexpr int DEC_MAX_SPLITS = 16;                // blocks of a cluster
constexpr int DEC_HEADS = 8;                      // query heads per pass (the MMA's N)
constexpr int SUB_BYTES_PER_ROW = 128;            // one swizzle row: 64 bf16

template <int W>
__device__ __forceinline__ void consumer_sync_w() { asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory"); }

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

// One page of keys and values in a stage of the ring, for one warp: scores^T = K q^T per 16 keys, soft cap,
// running maximum and sum, out^T += V^T p^T.  `page_key0` is the index of the page's first key in its
// request; keys outside [first, pos] are masked.  m, l: this thread's heads 2 tq and 2 tq + 1 (l over this
// thread's keys only).
template <int HD>
__device__ __forceinline__ void decode_page(float (&o)[HD / 16][4], float (&m)[2], float (&l)[2],
                                            const uint32_t (&qb)[HD / 16][2], uint32_t kbase, uint32_t vbase,
                                            uint8_t* vstage, int page_key0, int pos, int first, int page_size,
                                            int hd16, int nsub, uint32_t sub_bytes, float cap, float score_scale,
                                            int lane) {
  const int g = lane >> 2;
  for (int tile = 0; tile * 16 < page_size; ++tile) {
    const int key0 = page_key0 + tile * 16;
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
          *reinterpret_cast<uint4*>(vstage + (c >> 3) * sub_bytes +
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
}

// HD: register capacity (head_dim <= HD; head_dim and page_size are multiples of 16).
template <int HD, int CW>
__global__ void __launch_bounds__(CW * 32 + 32, 2)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const __nv_bfloat16* __restrict__ q, const int* __restrict__ positions,
                        const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_pages,
                        __nv_bfloat16* __restrict__ out, int nh, int nkv, int hd, int page_size, int num_pages, float multiplier, float cap,
                        int window, int splits, int stages, int whole_page, int* __restrict__ status) {
  constexpr int DEC_WARPS = CW, DEC_THREADS = CW * 32;          // consumer warps; one more warp is the producer
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

    // Iteration `it` (over all passes) belongs to warp it % warps and stage it % stages; the stage count
    // is a multiple of the warps, so a stage is always read by the same warp and that warp sees every
    // phase of the stage's barrier (a waiter that skipped a phase would match the wrong parity).
    const int it_lo = pass * n_pages, it_hi = it_lo + n_pages;
    for (int it = it_lo + ((warp - it_lo) % DEC_WARPS + DEC_WARPS) % DEC_WARPS; it < it_hi; it += DEC_WARPS) {
      const int pi = it - it_lo;
      const int s = it % stages;
      const bool ok = tc::mbar_wait(&sh->full[s], (it / stages) & 1, abort_flag);
      const uint32_t kbase = ring_addr + (uint32_t)s * 2 * page_bytes;
      const uint32_t vbase = kbase + page_bytes;
      if (ok)
        decode_page<HD>(o, m, l, qb, kbase, vbase, ring + (size_t)s * 2 * page_bytes + page_bytes,
                        (my_lo + pi) * page_size, pos, first, page_size, hd16, nsub, sub_bytes, cap, score_scale, lane);
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->empty[s]);     // this warp is done with stage s
    }
    // ---- this warp's totals, then the warps are merged in shared memory, in warp order ---------------
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
    consumer_sync_w<DEC_WARPS>();
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
    consumer_sync_w<DEC_WARPS>();   // the merge area is reused by the next pass
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

// ---- the same attention with the keys of the whole launch shared evenly among the blocks -----------------
//
// The pages of all (token, kv head) pairs of a launch, in order, are one sequence; block b takes units
// [b W, (b + 1) W) of it, whatever pairs they belong to, and streams them through its ring without a break.
// A unit is a page, and every pair is preceded by `pair_cost` empty units that stand for what a pair costs a
// block beside its pages (the query, the merge of the warps, the result): without them a block whose share
// is forty requests of one page each would take forty times that while the others wait.
// A pair whose pages lie inside one block is finished there; a pair that several blocks share gets a
// partial result from each in a workspace, and the block that leaves its part last adds them up, in block
// order.  So a launch lasts as long as its bytes take and not as long as its longest context (56 requests of
// 200 to 4,600 keys: a block per pair streams the longest alone at about 32 GB/s while the SMs of the short
// ones stand idle), every SM streams from the first page to the last, and without clusters the launch may
// start under its predecessor's tail.  One block (decode_stream_plan_kernel) finds W and where each
// block begins, once per step for all layers with the same window.
struct StreamPlan {
  const int4* starts;     // [blocks][2]: (token, kv head, unit within the pair, units this block takes),
                          //              (W, the token's position, its row of the block table, pair_cost)
  float* partials;        // [blocks][2][G][head_dim + 4]: a block's first pair (begun by another block) and its
                          // last (finished by another block)
  int* arrive;            // [tokens][kv heads]: blocks that have left their part; back at 0 after the launch
};

struct StreamShared {
  uint64_t full[DEC_MAX_STAGES];
  uint64_t empty[DEC_MAX_STAGES];
  int abort_flag;
  int last_one;
};

// One pair's range within a block: computed alike by the producer and the consumers.
struct StreamSegment {
  int pos, first, page_lo, pages;   // of the pair's token: last key, first key, first page, pages
};
__device__ __forceinline__ StreamSegment stream_segment(int pos, int window, int page_size) {
  StreamSegment s;
  s.pos = pos;
  s.first = (window > 0 && s.pos - window + 1 > 0) ? s.pos - window + 1 : 0;
  s.page_lo = s.first / page_size;
  s.pages = s.pos / page_size - s.page_lo + 1;
  return s;
}

template <int HD, int CW>
__global__ void __launch_bounds__(CW * 32 + 32, 2)
attention_decode_stream_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                               const __nv_bfloat16* __restrict__ q, const int* __restrict__ positions,
                               const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_pages,
                               __nv_bfloat16* __restrict__ out, int T, int nh, int nkv, int hd, int page_size,
                               int num_pages, float multiplier, float cap, int window, int stages, int whole_page,
                               int early, const StreamPlan plan, int* __restrict__ status) {
  constexpr int DEC_WARPS = CW, DEC_THREADS = CW * 32;          // consumer warps; one more warp is the producer
  extern __shared__ uint8_t dec_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dec_raw) + 1023) & ~(uintptr_t)1023);
  const int G = nh / nkv;                                  // at most DEC_HEADS (the host checks)
  const int hd16 = hd >> 4;
  const int nsub = (hd + 63) >> 6;
  const uint32_t sub_bytes = (uint32_t)page_size * SUB_BYTES_PER_ROW;
  const uint32_t page_bytes = nsub * sub_bytes;
  const int stride_f = hd + 2;
  const int pstride = hd + 4;                              // rows of the workspace: 16-byte aligned
  float* merge = reinterpret_cast<float*>(ring + (size_t)stages * 2 * page_bytes);   // [warps][G][hd + 2]
  StreamShared* sh = reinterpret_cast<StreamShared*>(merge + (size_t)DEC_WARPS * G * stride_f);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      tc::mbar_init(&sh->full[s], 1);
      tc::mbar_init(&sh->empty[s], 1);
    }
    sh->abort_flag = 0;
    sh->last_one = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(&map_k);
    tc::tma_prefetch_desc(&map_v);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // q and the newest key and value of every token come from the kernel before this one.  With `early` the
  // caller promises that nothing else does: the tokens belong to different requests, so that only the last
  // page of a token's range is being written, and the plan was made by a kernel further back.  The producer
  // warp then starts the block's first pages on their way before it waits for that kernel, as many as the ring
  // holds, and they arrive while that kernel finishes.
  bool waited = !(early && warp == DEC_WARPS);
  if (waited) pdl_wait_release();
  const int4 start = plan.starts[2 * blockIdx.x], start2 = plan.starts[2 * blockIdx.x + 1];
  if (start.w <= 0) return;                     // fewer pages than blocks
  const int W = start2.x;
  volatile int* abort_flag = &sh->abort_flag;

  // The first pair's position and table row come with the plan: two loads fewer between the wait and the
  // first page on its way.
  const int pair_cost = start2.w;
  int t = start.x, kvh = start.y, voff = start.z, remaining = start.w, it0 = 0;   // voff, remaining: in units
  int pos_t = start2.y, row_t = start2.z;
  if (warp == DEC_WARPS) {
    // ---- producer warp: pair after pair, 32 page lookups at a time, one lane starts the tile loads --------
    while (remaining > 0 && t < T) {
      const StreamSegment sg = stream_segment(pos_t, window, page_size);
      const int units = min(remaining, pair_cost + sg.pages - voff);      // of this pair in this block
      const int off = max(voff, pair_cost) - pair_cost;                   // first page
      const int n = max(0, voff + units - pair_cost - off);               // pages
      const int* table = block_table + (size_t)row_t * max_pages + sg.page_lo + off;
      for (int base = 0; base < n; base += 32) {
        int page = 0;
        if (base + lane < n) {
          page = table[base + lane];
          if (page < 0 || page >= num_pages) {     // never read outside the pool; report it
            atomicExch(status, 3);
            page = 0;
          }
        }
        for (int j = 0; j < 32 && base + j < n; ++j) {
          const int it = it0 + base + j;
          const int pg = __shfl_sync(0xffffffffu, page, j);
          // the ring is full, or this is the page that the kernel before is writing: time to wait for it
          if (!waited && (it >= stages || off + base + j == sg.pages - 1)) {
            pdl_wait_release();
            waited = true;
          }
          if (tc::elect_one()) {
            const int s = it % stages;
            bool ok = true;
            if (it >= stages) ok = tc::mbar_wait(&sh->empty[s], ((it / stages) - 1) & 1, abort_flag);
            if (ok) {
              uint8_t* kdst = ring + (size_t)s * 2 * page_bytes;
              const int row = (pg * nkv + kvh) * page_size;
              tc::mbar_expect_tx(&sh->full[s], 2 * page_bytes);
              if (whole_page) {
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
      remaining -= units;
      it0 += n;
      voff = 0;
      if (++kvh == nkv) {
        kvh = 0;
        if (++t < T && remaining > 0) {
          pos_t = positions[t];
          row_t = token_seq[t];
        }
      }
    }
    if (!waited) pdl_wait_release();
    return;
  }

  // ---- consumer warps ------------------------------------------------------------------------------------
  const int g = lane >> 2, tq = lane & 3;
  const float score_scale = cap > 0.f ? multiplier / cap : multiplier;
  const uint32_t ring_addr = tc::smem_u32(ring);
  long long cursor = (long long)blockIdx.x * W;                 // where this block stands in the launch's sequence
  while (remaining > 0 && t < T) {
    const StreamSegment sg = stream_segment(pos_t, window, page_size);
    const int units = min(remaining, pair_cost + sg.pages - voff);
    const int off = max(voff, pair_cost) - pair_cost;
    const int n = max(0, voff + units - pair_cost - off);
    const long long pair_begin = cursor - voff + pair_cost;     // the pair's first page in the launch's sequence
    cursor += units;
    remaining -= units;
    voff = 0;
    if (n == 0) {                                               // only the empty units before the pair's pages
      if (++kvh == nkv) {
        kvh = 0;
        if (++t < T && remaining > 0) pos_t = positions[t];
      }
      continue;
    }
    const bool begins = off == 0, ends = off + n == sg.pages;   // does this block hold the pair's first / last page
    // q^T as the B operand: this thread holds dims (16 ks + 2 tq, +1) and (+8, +9) of head g
    uint32_t qb[HD / 16][2];
    {
      const __nv_bfloat16* qrow = q + ((size_t)t * nh + kvh * G + (g < G ? g : 0)) * hd;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const bool in = ks < hd16 && g < G;
        qb[ks][0] = in ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + tq * 2) : 0u;
        qb[ks][1] = in ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + tq * 2) : 0u;
      }
    }
    float o[HD / 16][4];
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    // Page `it` of the block belongs to warp it % warps and stage it % stages (a multiple of them: a stage is always
    // read by the same warp, which therefore sees every phase of the stage's barrier).
    for (int it = it0 + ((warp - it0) % DEC_WARPS + DEC_WARPS) % DEC_WARPS; it < it0 + n; it += DEC_WARPS) {
      const int s = it % stages;
      const bool ok = tc::mbar_wait(&sh->full[s], (it / stages) & 1, abort_flag);
      const uint32_t kbase = ring_addr + (uint32_t)s * 2 * page_bytes;
      if (ok)
        decode_page<HD>(o, m, l, qb, kbase, kbase + page_bytes, ring + (size_t)s * 2 * page_bytes + page_bytes,
                        (sg.page_lo + off + it - it0) * page_size, sg.pos, sg.first, page_size, hd16, nsub, sub_bytes,
                        cap, score_scale, lane);
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->empty[s]);
    }
    // ---- this warp's totals; the warps are merged in shared memory, in warp order --------------------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 4);
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 8);
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 16);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int head = 2 * tq + h;
      if (head < G) {
        float* dst = merge + ((size_t)warp * G + head) * stride_f;
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
    consumer_sync_w<DEC_WARPS>();
    const bool whole = begins && ends;
    float* partial = plan.partials + (((size_t)blockIdx.x * 2 + (begins ? 1 : 0)) * G) * pstride;
    for (int j = 0; j < G; ++j) {
      float M = -INFINITY;
#pragma unroll
      for (int wv = 0; wv < DEC_WARPS; ++wv) M = fmaxf(M, merge[((size_t)wv * G + j) * stride_f + hd]);
      float L = 0.f;
      float w[DEC_WARPS];
#pragma unroll
      for (int wv = 0; wv < DEC_WARPS; ++wv) {
        const float mg = merge[((size_t)wv * G + j) * stride_f + hd];
        w[wv] = mg == -INFINITY ? 0.f : __expf(mg - M);
        L += merge[((size_t)wv * G + j) * stride_f + hd + 1] * w[wv];
      }
      for (int d = threadIdx.x; d < hd; d += DEC_THREADS) {
        float ov = 0.f;
#pragma unroll
        for (int wv = 0; wv < DEC_WARPS; ++wv) ov += merge[((size_t)wv * G + j) * stride_f + d] * w[wv];
        if (whole) out[((size_t)t * nh + kvh * G + j) * hd + d] = __float2bfloat16_rn(L > 0.f ? ov / L : 0.f);
        else partial[(size_t)j * pstride + d] = ov;
      }
      if (!whole && threadIdx.x == 0) {
        partial[(size_t)j * pstride + hd] = M;
        partial[(size_t)j * pstride + hd + 1] = L;
      }
    }
    if (!whole) {
      // ---- the pair is shared: the block that leaves its part last adds the parts up, in block order --------
      const int b_first = (int)(pair_begin / W), b_last = (int)((pair_begin + sg.pages - 1) / W);
      consumer_sync_w<DEC_WARPS>();                               // every thread's share of the partial result is written
      if (threadIdx.x == 0) {
        __threadfence();                             // and visible to the other blocks before this block is counted
        int* counter = plan.arrive + (size_t)t * nkv + kvh;
        const int before = atomicAdd(counter, 1);
        const int last = before == b_last - b_first;
        if (last) *counter = 0;                      // for the next launch
        __threadfence();
        sh->last_one = last;
      }
      consumer_sync_w<DEC_WARPS>();
      if (sh->last_one) {
        // Four output elements per thread, and of up to eight parts at a time the maxima, the sums and the
        // elements all in flight together: one trip to L2 for a pair that two to eight blocks share (a chain
        // of dependent loads per element and part took a block that merges 17 parts 20 us).
        const int parts = b_last - b_first + 1;
        const int quads = hd >> 2;
        for (int e = threadIdx.x; e < G * quads; e += DEC_THREADS) {
          const int j = e / quads, d = (e - j * quads) * 4;
          float M = -INFINITY, L = 0.f;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int i0 = 0; i0 < parts; i0 += 8) {
            float2 ml[8];
            float4 v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int bk = b_first + i0 + k;
              ml[k] = make_float2(-INFINITY, 0.f);
              v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (i0 + k < parts) {
                const float* row = plan.partials + (((size_t)bk * 2 + (bk == b_first ? 1 : 0)) * G + j) * pstride;
                ml[k] = __ldcg(reinterpret_cast<const float2*>(row + hd));
                v[k] = __ldcg(reinterpret_cast<const float4*>(row + d));
              }
            }
            float top = M;
#pragma unroll
            for (int k = 0; k < 8; ++k) top = fmaxf(top, ml[k].x);
            const float keep = M == -INFINITY ? 0.f : __expf(M - top);
            L *= keep;
            acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float wk = ml[k].x == -INFINITY ? 0.f : __expf(ml[k].x - top);
              L += ml[k].y * wk;
              acc.x += v[k].x * wk; acc.y += v[k].y * wk; acc.z += v[k].z * wk; acc.w += v[k].w * wk;
            }
            M = top;
          }
          const float inv = L > 0.f ? 1.f / L : 0.f;
          uint2 packed;
          packed.x = pack2(acc.x * inv, acc.y * inv);
          packed.y = pack2(acc.z * inv, acc.w * inv);
          *reinterpret_cast<uint2*>(out + ((size_t)t * nh + kvh * G + j) * hd + d) = packed;
        }
      }
    }
    consumer_sync_w<DEC_WARPS>();                                 // the merge area and last_one are used again by the next pair
    it0 += n;
    if (++kvh == nkv) {
      kvh = 0;
      if (++t < T && remaining > 0) pos_t = positions[t];
    }
  }
  if (threadIdx.x == 0 && sh->abort_flag) atomicExch(status, 4);
}

// One block plans a launch: W = units per block (at least `min_units`), and for every block the pair and
// the unit where it begins (see StreamPlan).
constexpr int PLAN_THREADS = 256;
constexpr int PLAN_ROWS = 4;          // tokens per thread: launches of up to 1024 tokens

__global__ void __launch_bounds__(PLAN_THREADS)
decode_stream_plan_kernel(const int* __restrict__ positions, const int* __restrict__ token_seq, int T, int window,
                          int page_size, int nkv, int blocks, int min_units, int pair_cost, int4* __restrict__ starts,
                          int* __restrict__ header) {
  __shared__ int warp_sum[PLAN_THREADS / 32];
  __shared__ int first_unit[PLAN_THREADS * PLAN_ROWS + 1];     // of every token's first pair; [T] = units in all
  __shared__ int pair_units[PLAN_THREADS * PLAN_ROWS];         // of one pair of the token
  pdl_wait_release();
  const int r0 = threadIdx.x * PLAN_ROWS;
  int units[PLAN_ROWS], mine = 0;
#pragma unroll
  for (int i = 0; i < PLAN_ROWS; ++i) {
    units[i] = r0 + i < T ? pair_cost + stream_segment(positions[r0 + i], window, page_size).pages : 0;
    mine += units[i] * nkv;
  }
  // inclusive scan of the threads' unit counts
  int incl = mine;
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, o);
    if ((int)(threadIdx.x & 31) >= o) incl += up;
  }
  if ((threadIdx.x & 31) == 31) warp_sum[threadIdx.x >> 5] = incl;
  __syncthreads();
  int before = incl - mine, total = 0;
  for (int w = 0; w < PLAN_THREADS / 32; ++w) {
    if (w < (int)(threadIdx.x >> 5)) before += warp_sum[w];
    total += warp_sum[w];
  }
#pragma unroll
  for (int i = 0; i < PLAN_ROWS; ++i) {
    if (r0 + i < T) {
      first_unit[r0 + i] = before;
      pair_units[r0 + i] = units[i];
      before += units[i] * nkv;
    }
  }
  if (threadIdx.x == 0) first_unit[T] = total;
  __syncthreads();
  const int W = max(min_units, (total + blocks - 1) / blocks);
  // A thread per block: the token in whose units the block begins, by bisection.  (A thread per token, writing
  // the starts of all blocks that begin inside it, left a launch of 12 tokens to three threads: 9.5 us.)
  for (int b = threadIdx.x; b < blocks; b += PLAN_THREADS) {
    const long long at = (long long)b * W;
    if (at >= total) {
      starts[2 * b] = make_int4(0, 0, 0, 0);
      continue;
    }
    int lo = 0, hi = T - 1;                 // the last token with first_unit <= at
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (first_unit[mid] <= at) lo = mid;
      else hi = mid - 1;
    }
    const int inside = (int)at - first_unit[lo], u = pair_units[lo];
    starts[2 * b] = make_int4(lo, inside / u, inside % u, min(W, total - (int)at));
    starts[2 * b + 1] = make_int4(W, positions[lo], token_seq[lo], pair_cost);
  }
  if (threadIdx.x == 0) {
    header[0] = W;
    header[1] = total;
  }
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

// Three stages of a page of keys and values (one for each of three consumer warps) have to fit a block's
// shared memory: pages of up to 64 tokens at head size 256, 128 at 128, 256 at 64.
GLINT_API int glint_attention_decode_supported(int nh, int nkv, int hd, int page_size) {
  if (!(nkv > 0 && nh % nkv == 0 && hd % 16 == 0 && hd >= 16 && hd <= 256 && page_size % 16 == 0 &&
        page_size >= 16 && page_size <= 256))
    return 0;
  const long long page_bytes = (long long)((hd + 63) / 64) * page_size * SUB_BYTES_PER_ROW;
  const int G = nh / nkv, HP = G < DEC_HEADS ? G : DEC_HEADS;
  const long long fixed = 3ll * HP * (hd + 2) * 4 + (long long)G * (hd + 2) * 4 + 2048;
  return 3 * 2 * page_bytes + fixed <= 227 * 1024 ? 1 : 0;
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
  int warps = decode_consumer_warps(T);
  if (warps > 3 && warps * 2 * page_bytes + (long long)warps * HP * (hd + 2) * 4 + (long long)G * (hd + 2) * 4 + 2048 >
                       227 * 1024)
    warps = 3;                      // large pages: a stage for each of four warps does not fit
  const long long fixed = (long long)warps * HP * (hd + 2) * 4 + (splits > 1 ? (long long)G * (hd + 2) * 4 : 0) +
                          sizeof(DecodeShared) + 1024 + 64;
  // a multiple of the consumer warps (see the kernel), as many as let two blocks share an SM
  int stages = (int)((110 * 1024 - fixed) / (2 * page_bytes)) / warps * warps;
  if (stages > DEC_MAX_STAGES) stages = DEC_MAX_STAGES;
  if (stages < warps) stages = warps;
  const long long smem = stages * 2 * page_bytes + fixed;
  if (smem > 227 * 1024) return GLINT_ERR_UNSUPPORTED_SIZE;
  dim3 grid(T, nkv, splits);
  const __nv_bfloat16* qq = (const __nv_bfloat16*)q;
  __nv_bfloat16* oo = (__nv_bfloat16*)out;
#define LAUNCH_W(HD, W)                                                                                           \
  {                                                                                                               \
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem);                                                              \
    if (e != cudaSuccess) return (int)e;                                                                          \
    if (splits > 8) {                                                                                             \
      e = cudaFuncSetAttribute(attention_decode_kernel<HD, W>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);  \
      if (e != cudaSuccess) return (int)e;                                                                        \
    }                                                                                                             \
    e = launch_kernel_cluster(attention_decode_kernel<HD, W>, grid, dim3(W * 32 + 32), (size_t)smem, stream, splits, \
                              map_k, map_v, qq, positions, token_seq, block_table, max_pages, oo, nh, nkv, hd,      \
                              page_size, num_pages, multiplier, cap, window, splits, stages, whole_page, status);   \
    if (e != cudaSuccess) return (int)e;                                                                          \
  }
#define LAUNCH(HD)                 \
  {                                \
    if (warps == 4) LAUNCH_W(HD, 4) \
    else LAUNCH_W(HD, 3)           \
  }
  if (hd <= 64) LAUNCH(64)
  else if (hd <= 128) LAUNCH(128)
  else LAUNCH(256)
#undef LAUNCH
#undef LAUNCH_W
  return (int)cudaGetLastError();
}

// ---- the stream variant ----------------------------------------------------------------------------------
GLINT_API int glint_attention_decode_stream_supported(int nh, int nkv, int hd, int page_size) {
  return (glint_attention_decode_supported(nh, nkv, hd, page_size) && nh / nkv <= DEC_HEADS) ? 1 : 0;
}

// Floats of workspace a launch of `blocks` blocks needs.
GLINT_API long long glint_attention_decode_stream_workspace(int blocks, int nh, int nkv, int hd) {
  return (long long)blocks * 2 * (nh / nkv) * (hd + 4);
}

// Plans a launch of T single tokens (at most 1024) over `blocks` blocks: starts [blocks][2] int4, header [2]
// (units per block, units in all; for tests and measurements).  `pair_cost` < 0: what a pair costs a block
// beside its pages, in pages of this size (about 5 us of a block's stream).
// One plan serves every layer of a step with the same window, page size and number of kv heads.
GLINT_API int glint_attention_decode_stream_plan(const int* positions, const int* token_seq, int T, int window,
                                                 int page_size, int hd, int nkv, int blocks, int min_pages,
                                                 int pair_cost, void* starts, int* header, cudaStream_t stream) {
  if (T <= 0) return GLINT_OK;
  if (T > PLAN_THREADS * PLAN_ROWS || page_size <= 0 || nkv <= 0 || blocks < 1 || hd <= 0)
    return GLINT_ERR_UNSUPPORTED_SIZE;
  if (pair_cost < 0) {
    const long long page_bytes = 2ll * ((hd + 63) / 64) * page_size * SUB_BYTES_PER_ROW;   // keys and values
    pair_cost = (int)((160 * 1024 + page_bytes / 2) / page_bytes);
    if (pair_cost < 1) pair_cost = 1;
  }
  cudaError_t e = launch_kernel(decode_stream_plan_kernel, dim3(1), dim3(PLAN_THREADS), 0, stream, positions, token_seq, T,
                                window, page_size, nkv, blocks, min_pages < 1 ? 1 : min_pages, pair_cost, (int4*)starts,
                                header);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// `partials`: glint_attention_decode_stream_workspace floats; `arrive`: [T][nkv] counters that are zero before
// the first launch (every launch leaves them zero).  `early`: see the kernel; 0 is always right.  The plan must have been made for the same positions,
// window, page size, kv heads and number of blocks.
GLINT_API int glint_attention_decode_stream(const void* q, const void* k_pool, const void* v_pool,
                                            const int* positions, const int* token_seq, const int* block_table,
                                            int max_pages, void* out, int T, int nh, int nkv, int hd, int page_size,
                                            int num_pages, float multiplier, float cap, int window, int blocks,
                                            const void* starts, float* partials, int* arrive, int early,
                                            int* status, cudaStream_t stream) {
  if (T <= 0) return GLINT_OK;
  if (!starts || !partials || !arrive || blocks < 1 || ((uintptr_t)partials & 15)) return GLINT_ERR_BAD_ARG;
  if (!glint_attention_decode_stream_supported(nh, nkv, hd, page_size)) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)k_pool | (uintptr_t)v_pool) & 15 || ((uintptr_t)q & 3)) return GLINT_ERR_UNSUPPORTED_SIZE;
  CUtensorMap map_k, map_v;
  const long long rows = (long long)num_pages * nkv * page_size;
  const int whole_page = (hd % 64 == 0 && page_size <= 256) ? 1 : 0;
  int rc = pool_map(&map_k, k_pool, rows, hd, page_size, whole_page);
  if (rc != GLINT_OK) return rc;
  rc = pool_map(&map_v, v_pool, rows, hd, page_size, whole_page);
  if (rc != GLINT_OK) return rc;
  const int G = nh / nkv;
  const long long page_bytes = (long long)((hd + 63) / 64) * page_size * SUB_BYTES_PER_ROW;
  int warps = decode_consumer_warps(T);
  if (warps > 3 && warps * 2 * page_bytes + (long long)warps * G * (hd + 2) * 4 + 2048 > 227 * 1024) warps = 3;
  const long long fixed = (long long)warps * G * (hd + 2) * 4 + sizeof(StreamShared) + 1024 + 64;
  int stages = (int)((110 * 1024 - fixed) / (2 * page_bytes)) / warps * warps;
  if (stages > DEC_MAX_STAGES) stages = DEC_MAX_STAGES;
  if (stages < warps) stages = warps;
  const long long smem = stages * 2 * page_bytes + fixed;
  if (smem > 227 * 1024) return GLINT_ERR_UNSUPPORTED_SIZE;
  StreamPlan plan = {(const int4*)starts, partials, arrive};
  const __nv_bfloat16* qq = (const __nv_bfloat16*)q;
  __nv_bfloat16* oo = (__nv_bfloat16*)out;
#define LAUNCH_W(HD, W)                                                                                                 \
  {                                                                                                                     \
    cudaError_t e = cudaFuncSetAttribute(attention_decode_stream_kernel<HD, W>,                                         \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                       \
    if (e != cudaSuccess) return (int)e;                                                                                \
    e = launch_kernel(attention_decode_stream_kernel<HD, W>, dim3(blocks), dim3(W * 32 + 32), (size_t)smem, stream,      \
                      map_k, map_v, qq, positions, token_seq, block_table, max_pages, oo, T, nh, nkv, hd, page_size,     \
                      num_pages, multiplier, cap, window, stages, whole_page, early ? 1 : 0, plan, status);             \
    if (e != cudaSuccess) return (int)e;                                                                                \
  }
#define LAUNCH(HD)                 \
  {                                \
    if (warps == 4) LAUNCH_W(HD, 4) \
    else LAUNCH_W(HD, 3)           \
  }
  if (hd <= 64) LAUNCH(64)
  else if (hd <= 128) LAUNCH(128)
  else LAUNCH(256)
#undef LAUNCH
#undef LAUNCH_W
  return (int)cudaGetLastError();
}

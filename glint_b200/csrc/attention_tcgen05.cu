// Flash attention for prompt portions over the paged cache on the 5th-generation tensor cores.
//
// One block per (query tile, request, kv head), longest tiles first; one block per SM.  A block owns 128
// query rows: rows are (token, query head of the group) pairs, so the heads that share a kv head
// share every key/value tile.  Keys come in tiles of 64 whose boundaries are multiples of 64 in
// absolute position.
//   warp 0     TMA: the query tile once (one 4-D box per 64 columns), then key and value tiles
//              page by page into two-deep rings (one elected thread issues every box)
//   warp 1     tcgen05.mma: S = Q K^T into tensor memory (two buffers), then O += P V with P read from
//              tensor memory as the A operand and V as the MN-major B operand
//   warps 2-9  softmax: two threads share one row of S (tcgen05.ld), scale, soft-cap and mask it
//              by absolute position, keeps the running max and sum in 32-bit, writes P as bfloat16
//              pairs into tensor memory (tcgen05.st, two buffers), and rescales its row of O in
//              tensor memory only when the running max grew by more than 8 (the result is the same:
//              the sum carries the same stale max)
// Formulas: src/tensor/flash.rs:65-123 (online softmax), :76-87 (multiplier, cap * tanh(x / cap)),
// src/transformer/forward.rs:933-942 (window per absolute position).  The soft cap uses
// tanh.approx and the exponentials ex2.approx; sums and maxima are float32.
#include "common.cuh"
#include "tcgen05.cuh"

namespace glint {

constexpr int FA_M = 128;             // query rows per block
constexpr int FA_N = 64;              // keys per tile
constexpr int FA_THREADS = 320;      // TMA warp, MMA warp, 8 softmax warps
constexpr int FA_Q_SUB = FA_M * 128;  // bytes of a 64-column slice of the query tile
constexpr int FA_KV_SUB = FA_N * 128; // bytes of a 64-column slice of a key or value tile
constexpr float FA_RESCALE = 8.0f;

struct FaParams {
  const int* cu_seqlens;
  const int* seq_start;
  const int* block_table;
  int max_pages;
  __nv_bfloat16* out;
  int nh, nkv, hd, page_size, num_pages;
  float multiplier, cap;
  int window;
  int q_tiles, n_seqs;
  int whole;       // keys in boxes of 8 rows x head_dim, values in boxes of a page x head_dim (see the producer)
  int* status;
};

struct FaShared {
  uint64_t q_full, p_ready, o_full;
  uint64_t p_free[2];            // one per P buffer: the product that read it has completed
  uint64_t s_full[2];
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  float row_max[2][2][FA_M];     // [tile parity][column half][row]
  float row_sum[2][FA_M];
};

__global__ void __launch_bounds__(FA_THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const FaParams p) {
  extern __shared__ uint8_t fa_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_raw) + 1023) & ~(uintptr_t)1023);
  const int hd = p.hd, hd16 = hd >> 4, nsub = (hd + 63) >> 6;
  const int G = p.nh / p.nkv;
  const int tok_per_tile = FA_M / G;
  uint8_t* sq = smem;
  uint8_t* sk = sq + (size_t)nsub * FA_Q_SUB;            // [2][nsub][64 keys x 128 B]
  uint8_t* sv = sk + (size_t)2 * nsub * FA_KV_SUB;
  FaShared* sh = reinterpret_cast<FaShared*>(sv + (size_t)2 * nsub * FA_KV_SUB);

  // blockIdx.x counts (query tile from the last, request, kv head): the blocks with the most key tiles
  // start first whatever their head (with heads in the slow grid dimensions the long tiles of the
  // last heads started last: 4096 tokens 122 -> 91 us)
  const int per_tile = p.n_seqs * p.nkv;
  const int tile = p.q_tiles - 1 - (int)blockIdx.x / per_tile;
  const int seq = ((int)blockIdx.x % per_tile) / p.nkv, kvh = (int)blockIdx.x % p.nkv;
  const int t_begin = p.cu_seqlens[seq];
  const int q_len = p.cu_seqlens[seq + 1] - t_begin;
  const int tok0 = tile * tok_per_tile;
  if (tok0 >= q_len) return;
  const int n_tok = min(tok_per_tile, q_len - tok0);
  const int n_rows = n_tok * G;
  const int pos0 = p.seq_start[seq] + tok0;
  const int pos_last = pos0 + n_tok - 1;
  const int kv_first = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int kv_begin = kv_first & ~(FA_N - 1);
  const int n_tiles = (pos_last - kv_begin) / FA_N + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tc::mbar_init(&sh->q_full, 1);
    tc::mbar_init(&sh->p_ready, 256);
    tc::mbar_init(&sh->p_free[0], 1);
    tc::mbar_init(&sh->p_free[1], 1);
    tc::mbar_init(&sh->o_full, 1);
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&sh->s_full[b], 1);
      tc::mbar_init(&sh->k_full[b], 1);
      tc::mbar_init(&sh->k_empty[b], 1);
      tc::mbar_init(&sh->v_full[b], 1);
      tc::mbar_init(&sh->v_empty[b], 1);
    }
    sh->abort_flag = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(&map_q);
    tc::tma_prefetch_desc(&map_k);
    tc::tma_prefetch_desc(&map_v);
  }
  if (warp == 1) tc::tmem_alloc(&sh->tmem_base, 512);
  tc::fence_before_thread_sync();
  __syncthreads();
  tc::fence_after_thread_sync();
  const uint32_t tmem_s = sh->tmem_base;          // two score tiles: columns [0, 64) and [64, 128)
  const uint32_t tmem_o = tmem_s + 2 * FA_N;
  // P as bfloat16 pairs, two buffers of 32 columns behind O (head sizes up to 256: 128 + 256 + 64 <= 512)
  const uint32_t tmem_p = tmem_o + 256;
  volatile int* abort_flag = &sh->abort_flag;

  if (warp == 0) {
    // ---- producer ---------------------------------------------------------------------------------
    // The whole warp walks the tiles: lane pi looks up the page pi of the next tile (its table entry
    // is requested one tile ahead and looked at only when it is used), the page numbers go round by
    // shuffle, and one elected thread issues the copies.  Inside elect.sync the compiler keeps
    // addresses and coordinates in uniform registers, which the TMA instructions take directly; a
    // table load inside that region would be waited for on the spot.
    if (tc::elect_one()) {
      tc::mbar_expect_tx(&sh->q_full, (uint32_t)nsub * tok_per_tile * G * 128);
      for (int sub = 0; sub < nsub; ++sub)
        tc::tma_load_4d(sq + (size_t)sub * FA_Q_SUB, &map_q, &sh->q_full, sub * 64, 0, kvh, t_begin + tok0);
    }
    __syncwarp();
    const int ppt = FA_N / p.page_size;                        // pages per tile: 4, 2 or 1
    const int* table = p.block_table + (size_t)seq * p.max_pages;
    const int page_lo = kv_first / p.page_size, page_hi = pos_last / p.page_size;
    const int first_page = kv_begin / p.page_size;
    // pages outside [page_lo, page_hi] are masked by the softmax; they are filled from page 0
    auto fetch = [&](int j) -> int {
      const int page_idx = first_page + j * ppt + lane;
      return lane < ppt ? table[min(max(page_idx, page_lo), page_hi)] : 0;
    };
    int next = fetch(0);
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1;
      int mine = next;
      const int page_idx = first_page + j * ppt + lane;
      if (lane >= ppt || page_idx < page_lo || page_idx > page_hi) {
        mine = 0;
      } else if (mine < 0 || mine >= p.num_pages) {
        atomicExch(p.status, 3);
        mine = 0;
      }
      if (j + 1 < n_tiles) next = fetch(j + 1);
      int pages[4];
#pragma unroll
      for (int pi = 0; pi < 4; ++pi) pages[pi] = __shfl_sync(0xffffffffu, mine, pi);
      for (int which = 0; which < 2 && ok; ++which) {          // keys first: they are needed first
        uint64_t* full = which ? &sh->v_full[b] : &sh->k_full[b];
        if (j >= 2) ok = tc::mbar_wait(which ? &sh->v_empty[b] : &sh->k_empty[b], ((j >> 1) - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (tc::elect_one()) {
          tc::mbar_expect_tx(full, (uint32_t)nsub * FA_KV_SUB);
          const CUtensorMap* map = which ? &map_v : &map_k;
          uint8_t* ring = (which ? sv : sk) + (size_t)b * nsub * FA_KV_SUB;
          if (p.whole && which) {
            // values: one box per page, [slice][row of the page][64 columns]
#pragma unroll
            for (int pi = 0; pi < 4; ++pi)
              if (pi < ppt)
                tc::tma_load_3d(ring + (size_t)pi * nsub * p.page_size * 128, map, full, 0,
                                (pages[pi] * p.nkv + kvh) * p.page_size, 0);
          } else if (p.whole) {
            // keys: one box per 8 rows, [slice][8 rows][64 columns]; the groups of 8 rows of the tile are
            // then nsub KB apart, which the operand descriptor takes as its stride
#pragma unroll
            for (int a = 0; a < FA_N / 8; ++a) {
              const int key = a * 8;
              const int pg = p.page_size == 16 ? pages[a >> 1] : p.page_size == 32 ? pages[a >> 2] : pages[0];
              tc::tma_load_3d(ring + (size_t)a * nsub * 1024, map, full, 0,
                              (pg * p.nkv + kvh) * p.page_size + (key & (p.page_size - 1)), 0);
            }
          } else {
#pragma unroll
            for (int pi = 0; pi < 4; ++pi) {
              if (pi < ppt) {
                const int row = (pages[pi] * p.nkv + kvh) * p.page_size;
                uint8_t* dst = ring + (size_t)pi * p.page_size * 128;
                for (int sub = 0; sub < nsub; ++sub) tc::tma_load_2d(dst + (size_t)sub * FA_KV_SUB, map, full, sub * 64, row);
              }
            }
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -------------------------------------------------------------------------------
    // elect.sync rather than "lane 0": descriptors then live in uniform registers and one MMA costs
    // the issuing thread about 45 cycles instead of about 105.
    if (tc::elect_one()) {
      const uint32_t idesc_s = tc::idesc_bf16_f32(FA_M, FA_N);
      const uint32_t idesc_o = tc::idesc_bf16_f32_b_mn(FA_M, hd);
      const uint32_t q_addr = tc::smem_u32(sq), k_addr = tc::smem_u32(sk), v_addr = tc::smem_u32(sv);
      // Order of issue: S(0), S(1), then for every tile j: O += P(j) V(j), S(j+2).  While the softmax
      // warps work on S(j+1) the tensor pipe runs P(j) V(j) and S(j+2).  This one thread issues 20
      // MMAs per tile, so its instruction count is what matters: every descriptor is a constant base
      // plus a small offset (the address field counts 16 bytes).
      const uint64_t qd0 = tc::smem_desc_k_sw128(q_addr);
      // Two layouts of a key or value tile (see the producer).  Separate boxes per 64-column slice:
      // [slice][64 keys][128 B].  Whole boxes: keys [group of 8][slice][8 rows][128 B], values
      // [page][slice][rows of the page][128 B].
      const uint32_t k_slice = p.whole ? 1024u : (uint32_t)FA_KV_SUB;          // bytes between slices of keys
      const uint32_t k_sbo = p.whole ? (uint32_t)nsub * 1024u : 1024u;         // bytes between groups of 8 keys
      const uint32_t v_lbo = p.whole ? (uint32_t)p.page_size * 128u : (uint32_t)FA_KV_SUB;
      const uint32_t v_page = (uint32_t)nsub * p.page_size * 128u;             // whole boxes: bytes of a page
      uint64_t kd0[2], vd0[2];
      for (int b = 0; b < 2; ++b) {
        kd0[b] = tc::smem_desc_k_sw128_sbo(k_addr + b * nsub * FA_KV_SUB, k_sbo);
        vd0[b] = tc::smem_desc_mn_sw128(v_addr + b * nsub * FA_KV_SUB, v_lbo, 1024);
      }
      uint32_t v_step[FA_N / 16];                                              // start of keys 16 kk, in 16 bytes
#pragma unroll
      for (int kk = 0; kk < FA_N / 16; ++kk)
        v_step[kk] = p.whole ? (((kk * 16) / p.page_size) * v_page + ((kk * 16) % p.page_size) * 128u) >> 4
                             : (uint32_t)(kk * 2048) >> 4;
      auto issue_s = [&](int j) -> bool {
        const int b = j & 1;
        if (!tc::mbar_wait(&sh->k_full[b], (j >> 1) & 1, abort_flag)) return false;
        tc::fence_after_thread_sync();
        const uint32_t d = tmem_s + b * FA_N;
        const uint64_t kd = b ? kd0[1] : kd0[0];
#pragma unroll
        for (int ks = 0; ks < 16; ++ks) {
          if (ks < hd16) {
            const uint32_t oq = ((ks >> 2) * FA_Q_SUB + (ks & 3) * 32) >> 4;     // compile-time constants
            const uint32_t ok_ = ((ks >> 2) * k_slice + (ks & 3) * 32) >> 4;
            tc::mma_bf16_ss(d, qd0 + oq, kd + ok_, idesc_s, ks > 0 ? 1u : 0u);
          }
        }
        tc::mma_commit(&sh->s_full[b]);
        tc::mma_commit(&sh->k_empty[b]);
        return true;
      };
      bool ok = tc::mbar_wait(&sh->q_full, 0, abort_flag);
      if (ok) ok = issue_s(0);
      if (ok && n_tiles > 1) ok = issue_s(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int b = j & 1;
        ok = tc::mbar_wait(&sh->p_ready, j & 1, abort_flag);
        if (ok) ok = tc::mbar_wait(&sh->v_full[b], (j >> 1) & 1, abort_flag);
        if (!ok) break;
        tc::fence_after_thread_sync();
        const uint64_t vd = b ? vd0[1] : vd0[0];
#pragma unroll
        for (int kk = 0; kk < FA_N / 16; ++kk)
          tc::mma_bf16_ts(tmem_o, tmem_p + (uint32_t)(j & 1) * 32 + 8 * kk, vd + v_step[kk], idesc_o,
                          (j > 0 || kk > 0) ? 1u : 0u);
        tc::mma_commit(&sh->v_empty[b]);
        tc::mma_commit(&sh->p_free[j & 1]);      // this P buffer, and O, may be touched again
        if (j + 2 < n_tiles) ok = issue_s(j + 2);
      }
      tc::mma_commit(&sh->o_full);
    }
    __syncwarp();
  } else {
    // ---- softmax, correction and epilogue: two threads per row of the tile ------------------------------
    // Warps 2..5 take columns [0, 32) of the score tile, warps 6..9 columns [32, 64); a warp reaches
    // the 32 lanes of tensor memory of its quarter (warp index mod 4).  Two warps per scheduler hide
    // each other's latencies; the row maximum is exchanged through shared memory.
    constexpr int HALF = FA_N / 2;
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const bool rv = r < n_rows;
    const int qpos = pos0 + (rv ? r / G : 0);
    const int lo = p.window > 0 ? qpos - p.window + 1 : 0;
    const uint32_t lane_base = ((uint32_t)(quarter * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    const float in_scale = p.cap > 0.f ? p.multiplier / p.cap : p.multiplier;
    const float out_scale = p.cap > 0.f ? p.cap * LOG2E : LOG2E;   // scores are kept in log2 units
    const int o_lo = half ? ((hd16 + 1) >> 1) * 16 : 0;            // this thread's columns of O
    const int o_hi = half ? hd : ((hd16 + 1) >> 1) * 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = tc::mbar_wait(&sh->s_full[j & 1], (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc::fence_after_thread_sync();
      uint32_t raw[HALF];
#pragma unroll
      for (int c0 = 0; c0 < HALF; c0 += 16)
        tc::tmem_ld_16(tmem_s + (j & 1) * FA_N + lane_base + half * HALF + c0, raw + c0);
      tc::tmem_ld_wait();
      const int key0 = kv_begin + j * FA_N + half * HALF;
      float x[HALF];
      float mt4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      // most tiles lie wholly inside every row's range: those skip the per-key comparisons
      const bool inside = rv && key0 >= lo && key0 + HALF - 1 <= qpos;
      if (__all_sync(0xffffffffu, inside)) {
        if (p.cap > 0.f) {
#pragma unroll
          for (int c = 0; c < HALF; ++c) {
            x[c] = tc::tanh_approx(__uint_as_float(raw[c]) * in_scale) * out_scale;
            mt4[c & 3] = fmaxf(mt4[c & 3], x[c]);
          }
        } else {
#pragma unroll
          for (int c = 0; c < HALF; ++c) {
            x[c] = __uint_as_float(raw[c]) * (in_scale * out_scale);
            mt4[c & 3] = fmaxf(mt4[c & 3], x[c]);
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < HALF; ++c) {
          const int key = key0 + c;
          const bool valid = rv && key <= qpos && key >= lo;
          float v = __uint_as_float(raw[c]) * in_scale;
          if (p.cap > 0.f) v = tc::tanh_approx(v);
          v = valid ? v * out_scale : -INFINITY;
          x[c] = v;
          mt4[c & 3] = fmaxf(mt4[c & 3], v);
        }
      }
      // the row's maximum over both halves
      sh->row_max[j & 1][half][r] = fmaxf(fmaxf(mt4[0], mt4[1]), fmaxf(mt4[2], mt4[3]));
      asm volatile("bar.sync 2, 256;" ::: "memory");
      const float mt = fmaxf(sh->row_max[j & 1][0][r], sh->row_max[j & 1][1][r]);
      // rescale only when the running max grew by more than 8 (in natural units)
      const bool grow = mt > m_used + FA_RESCALE * LOG2E;
      float corr = 1.f;
      if (grow) {
        corr = m_used == -INFINITY ? 0.f : tc::exp2_approx(m_used - mt);
        l *= corr;
        m_used = mt;
      }
      // P(j) goes into the buffer that the product of tile j-2 read: that one must be complete (it
      // long is).  O is rescaled only after the product of tile j-1.
      if (j > 1) {
        ok = tc::mbar_wait(&sh->p_free[j & 1], ((j - 2) >> 1) & 1, abort_flag);
        if (!ok) break;
      }
      const bool rescale = j > 0 && __any_sync(0xffffffffu, grow);
      if (rescale) {
        ok = tc::mbar_wait(&sh->p_free[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag);
        if (!ok) break;
      }
      tc::fence_after_thread_sync();
      if (rescale) {
        for (int c0 = o_lo; c0 < o_hi; c0 += 16) {
          uint32_t o[16];
          tc::tmem_ld_16(tmem_o + lane_base + c0, o);
          tc::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
          tc::tmem_st_16(tmem_o + lane_base + c0, o);
        }
        tc::tmem_st_wait();
      }
      const float base = m_used == -INFINITY ? 0.f : m_used;
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[HALF / 2];               // this thread's 32 keys of its row, two to a column
#pragma unroll
      for (int c = 0; c < HALF; c += 2) {
        const float p0 = tc::exp2_approx(x[c] - base), p1 = tc::exp2_approx(x[c + 1] - base);
        l4[c & 3] += p0;
        l4[(c + 1) & 3] += p1;
        const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
        packed[c >> 1] = *reinterpret_cast<const uint32_t*>(&h);
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      tc::tmem_st_16(tmem_p + (uint32_t)(j & 1) * 32 + lane_base + half * (HALF / 2), packed);
      tc::tmem_st_wait();
      tc::fence_before_thread_sync();
      tc::mbar_arrive(&sh->p_ready);
    }
    // ---- epilogue: O / l as bfloat16; the row's sum is the two halves' sums ----------------------------
    sh->row_sum[half][r] = l;
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (ok) ok = tc::mbar_wait(&sh->o_full, 0, abort_flag);
    if (ok) {
      tc::fence_after_thread_sync();
      const float total = sh->row_sum[0][r] + sh->row_sum[1][r];
      const float inv = total > 0.f ? 1.0f / total : 0.f;
      __nv_bfloat16* orow = p.out + ((size_t)(t_begin + tok0 + (rv ? r / G : 0)) * p.nh + kvh * G + (rv ? r % G : 0)) * hd;
      for (int c0 = o_lo; c0 < o_hi; c0 += 16) {
        uint32_t o[16];
        tc::tmem_ld_16(tmem_o + lane_base + c0, o);
        tc::tmem_ld_wait();
        if (rv) {
          uint4 lo4, hi4;
          __nv_bfloat162 h[8];
#pragma unroll
          for (int i = 0; i < 8; ++i)
            h[i] = __floats2bfloat162_rn(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
          lo4 = make_uint4(*reinterpret_cast<uint32_t*>(&h[0]), *reinterpret_cast<uint32_t*>(&h[1]),
                           *reinterpret_cast<uint32_t*>(&h[2]), *reinterpret_cast<uint32_t*>(&h[3]));
          hi4 = make_uint4(*reinterpret_cast<uint32_t*>(&h[4]), *reinterpret_cast<uint32_t*>(&h[5]),
                           *reinterpret_cast<uint32_t*>(&h[6]), *reinterpret_cast<uint32_t*>(&h[7]));
          *reinterpret_cast<uint4*>(orow + c0) = lo4;
          *reinterpret_cast<uint4*>(orow + c0 + 8) = hi4;
        }
      }
    }
  }
  tc::fence_before_thread_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_thread_sync();
    tc::tmem_dealloc(sh->tmem_base, 512);
  }
  if (threadIdx.x == 0 && sh->abort_flag) atomicExch(p.status, 4);
}

// ---- host side ---------------------------------------------------------------------------------

typedef CUresult (*FaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static FaEncodeFn fa_encode_fn() {
  static FaEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<FaEncodeFn>(ptr);
  }
  return fn;
}

static int fa_map(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                  const cuuint32_t* box) {
  FaEncodeFn fn = fa_encode_fn();
  if (!fn) return GLINT_ERR_BAD_ARG;
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? GLINT_OK : GLINT_ERR_BAD_ARG;
}

}  // namespace glint

using namespace glint;

// head_dim a multiple of 16 up to 256; at most 128 query heads per kv head; pages of 16, 32 or 64.
GLINT_API int glint_attention_tcgen05_supported(int nh, int nkv, int hd, int page_size) {
  return (nkv > 0 && nh % nkv == 0 && nh / nkv <= FA_M && hd % 16 == 0 && hd >= 16 && hd <= 256 &&
          (page_size == 16 || page_size == 32 || page_size == 64)) ? 1 : 0;
}

// q, out: [T, nh * hd] bf16; pools [pages][nkv][page_size][hd] bf16.
GLINT_API int glint_attention_tcgen05(const void* q, const void* k_pool, const void* v_pool, const int* cu_seqlens,
                                      const int* seq_start, const int* block_table, int max_pages, void* out,
                                      int T, int n_seqs, int max_q_len, int nh, int nkv, int hd, int page_size,
                                      int num_pages, float multiplier, float cap, int window, int* status,
                                      cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0 || T <= 0) return GLINT_OK;
  if (!glint_attention_tcgen05_supported(nh, nkv, hd, page_size)) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) return GLINT_ERR_UNSUPPORTED_SIZE;
  const int G = nh / nkv;
  const int tok_per_tile = FA_M / G;
  CUtensorMap map_q, map_k, map_v;
  {
    cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)G, (cuuint64_t)nkv, (cuuint64_t)T};
    cuuint64_t strides[3] = {(cuuint64_t)hd * 2, (cuuint64_t)G * hd * 2, (cuuint64_t)nh * hd * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)G, 1, (cuuint32_t)tok_per_tile};
    const int rc = fa_map(&map_q, q, 4, dims, strides, box);
    if (rc != GLINT_OK) return rc;
  }
  // With head_dim a multiple of 64 the 64-column slices are a third dimension of the pools and one
  // box brings all slices of its rows: 12 copies per tile of 64 keys instead of 32 with pages of 16
  // (the copy unit spends about 65 cycles on a box whatever its size).
  const int whole = hd % 64 == 0 ? 1 : 0;
  if (whole) {
    cuuint64_t dims[3] = {64, (cuuint64_t)num_pages * nkv * page_size, (cuuint64_t)(hd / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)hd * 2, 128};
    cuuint32_t box_k[3] = {64, 8, (cuuint32_t)(hd / 64)};
    cuuint32_t box_v[3] = {64, (cuuint32_t)page_size, (cuuint32_t)(hd / 64)};
    int rc = fa_map(&map_k, k_pool, 3, dims, strides, box_k);
    if (rc != GLINT_OK) return rc;
    rc = fa_map(&map_v, v_pool, 3, dims, strides, box_v);
    if (rc != GLINT_OK) return rc;
  } else {
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)num_pages * nkv * page_size};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    int rc = fa_map(&map_k, k_pool, 2, dims, strides, box);
    if (rc != GLINT_OK) return rc;
    rc = fa_map(&map_v, v_pool, 2, dims, strides, box);
    if (rc != GLINT_OK) return rc;
  }
  FaParams p;
  p.cu_seqlens = cu_seqlens; p.seq_start = seq_start; p.block_table = block_table; p.max_pages = max_pages;
  p.out = (__nv_bfloat16*)out; p.nh = nh; p.nkv = nkv; p.hd = hd; p.page_size = page_size; p.num_pages = num_pages;
  p.multiplier = multiplier; p.cap = cap; p.window = window; p.whole = whole; p.status = status;
  const int nsub = (hd + 63) / 64;
  const int smem = nsub * FA_Q_SUB + 4 * nsub * FA_KV_SUB + (int)sizeof(FaShared) + 1024 + 64;
  if (smem > 227 * 1024) return GLINT_ERR_UNSUPPORTED_SIZE;
  p.q_tiles = (max_q_len + tok_per_tile - 1) / tok_per_tile;
  p.n_seqs = n_seqs;
  const long long blocks = (long long)p.q_tiles * n_seqs * nkv;
  if (blocks > 0x7fffffffLL) return GLINT_ERR_UNSUPPORTED_SIZE;
  dim3 grid((unsigned)blocks, 1, 1);
  cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  attention_tcgen05_kernel<<<grid, FA_THREADS, smem, stream>>>(map_q, map_k, map_v, p);
  return (int)cudaGetLastError();
}

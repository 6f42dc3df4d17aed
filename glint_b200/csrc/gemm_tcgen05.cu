// out[tokens, features] = X[tokens, K] * W[features, K]^T in bfloat16 on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in tensor memory, operands staged by TMA).
//
// The product is computed transposed: the weight tile is the 128-row M operand and the tokens
// are the N operand (16..256 wide), so one kernel serves a decode step with a handful of
// tokens and a prefill with thousands, and the weight matrix is always streamed in full
// 128-row tiles at HBM speed.  (The reference's batched matvec keeps the same [rows, batch]
// orientation, src/tensor/quantized.rs:278-337.)  Each accumulator lane is one output
// feature, each column one token; a lane's K-loop order is fixed by K and the split factor
// alone, never by which tokens share the launch.
//
// Roles in a block: warp 0 issues TMA loads into a ring of shared-memory stages, warp 1 allocates
// tensor memory and issues the MMAs, the other warps read the accumulator back and write the
// result: four of them (192 threads) for token tiles narrower than 64 columns, eight (320
// threads, two per quarter of the accumulator lanes on alternate groups of 16 columns) from 64
// columns on.  When a launch has too few tiles to fill the GPU the K range is split over
// blockIdx.z and partial tiles go to a workspace.  If every block of the launch is on an SM at
// once, all blocks of a tile wait for one another at the tile's counter (a spin with a limit,
// after which the status word is set) and each adds up a share of the tile's columns;
// otherwise the block that arrives last adds up all of them.  Both add the splits in order, so
// the result is deterministic.  Epilogues: soft cap (output head); with two weight tiles per
// stage (gate rows and up rows of the same features) act(gate) * up written as bfloat16; two
// plain tiles side by side for products with more 128-feature tiles than SMs; and, for the
// q/k/v product, rotary encoding with the cache write.
#include <stdlib.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

namespace glint {

constexpr int GEMM_BM = 128;      // weight rows (output features) per tile
constexpr int GEMM_BK = 64;       // K elements per stage: 128 bytes, one swizzle atom
constexpr int GEMM_THREADS = 192;        // TMA warp, MMA warp, four epilogue warps
constexpr int GEMM_THREADS_WIDE = 320;   // eight epilogue warps: two per quarter of the accumulator lanes, on alternate 16-column groups
constexpr int GEMM_SPREAD_DEPARTED = 4096;   // second half of the counters: blocks that have finished reading
constexpr int GEMM_MAX_STAGES = 8;
constexpr int A_STAGE_BYTES = GEMM_BM * GEMM_BK * 2;

// The q/k/v product of a prompt portion with the rotary encoding and the cache write as its epilogue:
// the dual kernel's two weight tiles are rows j and j + hd/2 of one head, so that a thread holds
// both members of a rotation pair (hd a multiple of 256).
struct RopeEpilogue {
  int on;
  const float2* trig;        // [tokens][hd / 2] (cos, sin) of every token's angles
  const int* positions;      // [tokens]
  const int* token_seq;      // [tokens] row of the block table
  const int* block_table;    // [requests][max_pages]
  int max_pages;
  void* k_pool;              // [pages][nkv][page_size][hd] bf16; null: only q is computed
  void* v_pool;
  int nh, nkv, hd, page_size, num_pages;
  int bn;                    // largest token tile (host side)
};

struct GemmParams {
  RopeEpilogue rope;
  int M, N, K;          // tokens, output features, reduction length
  int BN;               // tokens per tile
  int m_tiles;          // token tiles (the fast index of blockIdx.x)
  int wide;             // dual kernel without gating: the second tile is the next 128 features (dual_offset 128)
  int spread;           // split-K: every block of a tile adds up a share of its columns (the grid fits the SMs at once)
  int tma_store;        // the epilogue stages the tile in shared memory and stores it with one bulk copy
  int stages;
  int splits, kb_per_split, total_kb;
  int dual_offset;      // row offset of the second weight tile (dual kernels)
  int act;              // activation of the dual epilogue
  float cap;            // soft cap of the plain epilogue (<= 0: none)
  int out_bf16;
  void* out;
  float* workspace;
  int* counters;
  int* status;
};

struct GemmShared {
  uint64_t full[GEMM_MAX_STAGES];
  uint64_t empty[GEMM_MAX_STAGES];
  uint64_t tmem_full;
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
  int epilogue_ok;
};

// tanh GELU with the hardware tanh (relative error about 2^-11, below the bfloat16 rounding of the
// result): 0.5 x (1 + tanh(0.7978846 (x + 0.044715 x^3)))   (src/tensor/ops.rs:169-178)
__device__ __forceinline__ float gelu_tanh_fast(float v) {
  return 0.5f * v * (1.0f + tc::tanh_approx(0.7978846f * (v + 0.044715f * v * v * v)));
}


// cap * tanh(v / cap) as cap * (1 - 2 / (exp(2 v / cap) + 1)) with the hardware exponential and
// division: a few instructions, so that the epilogue loops can be unrolled without outgrowing the
// instruction cache (the library tanhf is a long sequence); relative error about 1e-6, far inside
// the bfloat16 operands' own rounding.  The 32-bit engine does not use this kernel.
__device__ __forceinline__ float softcap_fast(float v, float cap, float two_over_cap) {
  return cap * (1.0f - __fdividef(2.0f, __expf(v * two_over_cap) + 1.0f));
}

// Writes 16 token columns of one feature per lane as bfloat16 pairs: neighbouring lanes (features
// f, f+1) swap halves so that an even lane stores (f, f+1) of token j and the odd lane (f-1, f) of
// token j+1, four bytes each (two-byte stores are several times slower).  N must be even.
__device__ __forceinline__ void store_bf16_pairs(__nv_bfloat16* out, size_t N, int f, bool f_pair_ok, int c0,
                                                 int n, const float* v, int lane) {
  const bool odd = lane & 1;
#pragma unroll
  for (int j = 0; j < 16; j += 2) {
    const float send = odd ? v[j] : v[j + 1];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
    const int tok = j + (odd ? 1 : 0);
    if (f_pair_ok && tok < n) {
      const __nv_bfloat162 pair = odd ? __floats2bfloat162_rn(recv, v[j + 1]) : __floats2bfloat162_rn(v[j], recv);
      *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(c0 + tok) * N + (f & ~1)) = pair;
    }
  }
}

// barrier of the epilogue warps alone
__device__ __forceinline__ void epi_sync(int threads) { asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory"); }

template <bool DUAL>
__device__ __forceinline__ void store_result(const GemmParams& p, int f, int t, float a, float b) {
  if (f >= p.N || t >= p.M) return;
  float y;
  if (DUAL) {
    const float g = p.act == 0 ? gelu_tanh(a) : a * (1.0f / (1.0f + expf(-a)));
    y = g * b;
  } else {
    y = p.cap > 0.f ? softcap_fast(a, p.cap, 2.0f / p.cap) : a;
  }
  if (p.out_bf16)
    reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)t * p.N + f] = __float2bfloat16_rn(y);
  else
    reinterpret_cast<float*>(p.out)[(size_t)t * p.N + f] = y;
}

template <bool DUAL>
__global__ void __launch_bounds__(GEMM_THREADS_WIDE, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_out, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int b_stage_bytes = p.BN * GEMM_BK * 2;
  const int stage_bytes = A_STAGE_BYTES * (DUAL ? 2 : 1) + b_stage_bytes;
  GemmShared* sh = reinterpret_cast<GemmShared*>(smem + (size_t)p.stages * stage_bytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // blockIdx.x walks the token tiles of one feature tile first: the blocks that run at the same
  // time then share their weight tiles, which come from HBM once and from L2 for the other token
  // tiles (feature tiles first re-read the weights once per token tile: 346 MB instead of 94 MB for
  // the gate/up product of a 2048-token portion).
  const int m_tile = (int)blockIdx.x % p.m_tiles, n_tile = (int)blockIdx.x / p.m_tiles;
  const int rope_subs = (DUAL && p.rope.on) ? p.rope.hd / (2 * GEMM_BM) : 1;   // 128-pair groups per head
  const int n0 = (DUAL && p.rope.on) ? (n_tile / rope_subs) * p.rope.hd + (n_tile % rope_subs) * GEMM_BM
                                     : n_tile * (p.wide ? 2 * GEMM_BM : GEMM_BM);
  const int m0 = m_tile * p.BN;
  const int split = blockIdx.z;
  const int kb_begin = split * p.kb_per_split;
  const int kb_end = min(p.total_kb, kb_begin + p.kb_per_split);
  const int n_kb = kb_end - kb_begin;
  const uint32_t tmem_cols_used = p.BN * (DUAL ? 2 : 1);
  uint32_t tmem_cols = 32;
  while (tmem_cols < tmem_cols_used) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      tc::mbar_init(&sh->full[s], 1);
      tc::mbar_init(&sh->empty[s], 1);
    }
    tc::mbar_init(&sh->tmem_full, 1);
    sh->abort_flag = 0;
    sh->is_last = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(&map_w);
    tc::tma_prefetch_desc(&map_x);
  }
  if (warp == 1) tc::tmem_alloc(&sh->tmem_base, tmem_cols);
  tc::fence_before_thread_sync();
  __syncthreads();
  tc::fence_after_thread_sync();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;

  if (warp == 0) {
    // ---- producer: TMA loads of the weight tile(s) and the token tile --------------------------
    // The issuing thread is chosen with elect.sync, not as "lane 0": the compiler then keeps
    // addresses and descriptors in uniform registers, which the TMA and MMA instructions take
    // directly (measured: about 45 instead of 105 cycles per MMA issued).
    if (tc::elect_one()) {
      // The weights are written by no kernel: the first ring of weight tiles is requested before
      // waiting for the kernel that produces the tokens, and so streams in under its tail.
      const int pre = min(n_kb, p.stages);
      for (int i = 0; i < pre; ++i) {
        uint8_t* stage = smem + (size_t)i * stage_bytes;
        tc::mbar_expect_tx(&sh->full[i], stage_bytes);
        const int k = (kb_begin + i) * GEMM_BK;
        tc::tma_load_2d(stage, &map_w, &sh->full[i], k, n0);
        if (DUAL) tc::tma_load_2d(stage + A_STAGE_BYTES, &map_w, &sh->full[i], k, n0 + p.dual_offset);
      }
      pdl_wait_release();
      for (int i = 0; i < pre; ++i)
        tc::tma_load_2d(smem + (size_t)i * stage_bytes + A_STAGE_BYTES * (DUAL ? 2 : 1), &map_x, &sh->full[i],
                        (kb_begin + i) * GEMM_BK, m0);
      int s = 0;                 // pre == stages whenever this loop runs
      uint32_t parity = 0;       // the first refill of a stage waits for its first release
      int k = (kb_begin + pre) * GEMM_BK;
      uint8_t* stage = smem;
      for (int i = pre; i < n_kb; ++i, k += GEMM_BK) {
        if (!tc::mbar_wait(&sh->empty[s], parity, abort_flag)) break;
        tc::mbar_expect_tx(&sh->full[s], stage_bytes);
        tc::tma_load_2d(stage, &map_w, &sh->full[s], k, n0);
        if (DUAL) tc::tma_load_2d(stage + A_STAGE_BYTES, &map_w, &sh->full[s], k, n0 + p.dual_offset);
        tc::tma_load_2d(stage + A_STAGE_BYTES * (DUAL ? 2 : 1), &map_x, &sh->full[s], k, m0);
        if (++s == p.stages) {
          s = 0;
          parity ^= 1;
          stage = smem;
        } else {
          stage += stage_bytes;
        }
      }
    } else {
      pdl_wait_release();
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----------------------------------------------------------------------------
    pdl_wait_release();
    if (tc::elect_one()) {
      // One thread issues everything, so its instruction count per K block is what bounds a
      // launch with few tokens: stage index and phase are counters (no division), and the
      // descriptors are built once and advanced by addition (the address field counts 16 bytes).
      const uint32_t idesc = tc::idesc_bf16_f32(GEMM_BM, p.BN);
      const uint64_t a0 = tc::smem_desc_k_sw128(tc::smem_u32(smem));
      const uint64_t b0 = tc::smem_desc_k_sw128(tc::smem_u32(smem) + A_STAGE_BYTES * (DUAL ? 2 : 1));
      const uint64_t stage_step = (uint64_t)(stage_bytes >> 4);
      int s = 0;
      uint32_t phase = 0;
      uint64_t da = a0, db = b0;
      for (int i = 0; i < n_kb; ++i) {
        if (!tc::mbar_wait(&sh->full[s], phase, abort_flag)) break;
        tc::fence_after_thread_sync();
#pragma unroll
        for (int k = 0; k < GEMM_BK / 16; ++k) {
          const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
          tc::mma_bf16_ss(tmem_base, da + 2 * k, db + 2 * k, idesc, acc);
          if (DUAL) tc::mma_bf16_ss(tmem_base + p.BN, da + (A_STAGE_BYTES >> 4) + 2 * k, db + 2 * k, idesc, acc);
        }
        tc::mma_commit(&sh->empty[s]);   // the stage is free once these MMAs have read it
        if (++s == p.stages) {
          s = 0;
          phase ^= 1;
          da = a0;
          db = b0;
        } else {
          da += stage_step;
          db += stage_step;
        }
      }
      tc::mma_commit(&sh->tmem_full);    // the accumulator is complete
    }
  } else {
    // ---- epilogue: each warp owns the 32 accumulator lanes of its quarter; with eight warps two share
    // a quarter and take alternate groups of 16 columns (one warp per scheduler leaves the tensor
    // memory loads, the activation and the stores of a wide tile waiting on each other) -------------
    pdl_wait_release();
    const int q = warp & 3;
    const int ep_threads = (int)blockDim.x - 64;
    const int eg = (warp - 2) >> 2, c_first = eg * 16, c_step = ep_threads >> 3;   // 16 or 32 columns
    const int f = n0 + q * 32 + lane;              // this thread's output feature
    tc::mbar_wait(&sh->tmem_full, 0, abort_flag);
    epi_sync(ep_threads);
    if (threadIdx.x == 64) sh->epilogue_ok = !*abort_flag;
    epi_sync(ep_threads);
    const bool ok = sh->epilogue_ok != 0;   // one thread decides, so all take the same branch
    tc::fence_after_thread_sync();
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const int tile_id = (int)blockIdx.x;
    const int halves = DUAL ? 2 : 1;
    if (DUAL && ok && p.rope.on) {
      // q and k heads: (lo, hi) -> (lo cos - hi sin, lo sin + hi cos) with the token's angles from the
      // table; v heads pass.  The tile is staged as [token][lo 128 | hi 128] bfloat16 and then copied
      // row by row, 16 bytes per lane, to q_out or to each token's place in its page.
      const RopeEpilogue& r = p.rope;
      const int half = r.hd >> 1;
      const int head = n_tile / rope_subs, sub = n_tile % rope_subs;
      const bool rotate = head < r.nh + r.nkv;
      const int fl = q * 32 + lane;
      const int jt = sub * GEMM_BM + fl;                 // this thread's pair within the head
      const int t_end = min(p.BN, p.M - m0);
      __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem);
      for (int c0 = c_first; c0 < t_end; c0 += c_step) {
        uint32_t a[16], b[16];
        tc::tmem_ld_16(lane_addr + c0, a);
        tc::tmem_ld_16(lane_addr + p.BN + c0, b);
        float2 cs[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int t = min(m0 + c0 + j, p.M - 1);
          cs[j] = rotate ? __ldg(r.trig + (size_t)t * half + jt) : make_float2(1.f, 0.f);
        }
        tc::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float lo = __uint_as_float(a[j]), hi = __uint_as_float(b[j]);
          __nv_bfloat16* row = stage + (size_t)(c0 + j) * (2 * GEMM_BM);
          row[fl] = __float2bfloat16_rn(rotate ? lo * cs[j].x - hi * cs[j].y : lo);
          row[GEMM_BM + fl] = __float2bfloat16_rn(rotate ? lo * cs[j].y + hi * cs[j].x : hi);
        }
      }
      epi_sync(ep_threads);
      const int wi = warp - 2, n_w = ep_threads >> 5;
      __nv_bfloat16* dst_base;
      if (head < r.nh) dst_base = reinterpret_cast<__nv_bfloat16*>(p.out);
      else if (head < r.nh + r.nkv) dst_base = reinterpret_cast<__nv_bfloat16*>(r.k_pool);
      else dst_base = reinterpret_cast<__nv_bfloat16*>(r.v_pool);
      const int kvh = head < r.nh ? 0 : (head - r.nh) % r.nkv;
      // a lane's 16 bytes: lanes 0-15 the lo half, lanes 16-31 the hi half of the staged row
      const int seg = (lane < 16 ? 0 : half) + sub * GEMM_BM + (lane & 15) * 8;
      for (int base = 0; base < t_end; base += 32 * n_w) {
        const int tl = base + lane * n_w + wi;           // this lane looks up one token's destination row
        long long dst = -1;
        if (tl < t_end) {
          const int t = m0 + tl;
          if (head < r.nh) {
            dst = ((long long)t * r.nh + head) * r.hd;
          } else {
            const int pos = r.positions[t];
            const int page = r.block_table[(size_t)r.token_seq[t] * r.max_pages + pos / r.page_size];
            if (page < 0 || page >= r.num_pages) atomicExch(p.status, 2);
            else dst = (((long long)page * r.nkv + kvh) * r.page_size + pos % r.page_size) * r.hd;
          }
        }
        for (int l = 0; l < 32; ++l) {
          const int tl2 = base + l * n_w + wi;
          if (tl2 >= t_end) break;
          const long long d = __shfl_sync(0xffffffffu, dst, l);
          if (d >= 0) {
            const uint4 v = *reinterpret_cast<const uint4*>(stage + (size_t)tl2 * (2 * GEMM_BM) + lane * 8);
            *reinterpret_cast<uint4*>(dst_base + d + seg) = v;
          }
        }
      }
    } else if (ok && p.splits == 1 && p.tma_store) {
      // Wide token tiles: the tile is staged in the stage ring (free now: every MMA has completed) as
      // [token][128 features], 32 consecutive features per warp store, and leaves with one bulk tensor
      // store, which clips it at the edges of the output.  256 shared-memory stores per thread instead
      // of 256 global ones.
      const int t_end = min(p.BN, p.M - m0);
      const bool capped = p.cap > 0.f;
      const float two_over_cap = capped ? 2.0f / p.cap : 0.f;
      const int fl = q * 32 + lane;
      for (int c0 = c_first; c0 < t_end; c0 += c_step) {
        uint32_t a[16], b[16];
        tc::tmem_ld_16(lane_addr + c0, a);
        if (DUAL) tc::tmem_ld_16(lane_addr + p.BN + c0, b);
        tc::tmem_ld_wait();
        float v[16];
        if (DUAL) {
          if (p.act == 0) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = gelu_tanh_fast(__uint_as_float(a[j])) * __uint_as_float(b[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float g = __uint_as_float(a[j]);
              v[j] = g * (1.0f / (1.0f + __expf(-g))) * __uint_as_float(b[j]);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(a[j]);
          if (capped) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = softcap_fast(v[j], p.cap, two_over_cap);
          }
        }
        if (p.out_bf16) {
          __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(smem) + (size_t)c0 * GEMM_BM + fl;
#pragma unroll
          for (int j = 0; j < 16; ++j) st[(size_t)j * GEMM_BM] = __float2bfloat16_rn(v[j]);
        } else {
          float* st = reinterpret_cast<float*>(smem) + (size_t)c0 * GEMM_BM + fl;
#pragma unroll
          for (int j = 0; j < 16; ++j) st[(size_t)j * GEMM_BM] = v[j];
        }
      }
      tc::fence_proxy_async();                     // the bulk copy reads shared memory through the async proxy
      epi_sync(ep_threads);
      if (threadIdx.x == 64) tc::tma_store_2d_and_wait_read(smem, &map_out, n0, m0);
    } else if (ok && p.splits == 1) {
      // One row pointer per thread, advanced by a whole output row per token; the epilogue kind is
      // chosen once, outside the loops, so that each loop body is a load, a little math and a store.
      const bool f_ok = f < p.N;
      const int t_end = min(p.BN, p.M - m0);                  // columns of this tile that are tokens
      // bfloat16 outputs go out as pairs of features (N even; the last feature of an odd N has no
      // partner and takes the scalar store)
      const bool pairs = (p.N & 1) == 0;
      const bool f_pair_ok = (f | 1) < p.N;
      if (DUAL && p.wide) {
        // two plain tiles of 128 features side by side: a block of 256 features x 256 tokens takes in
        // 64 KB per 8 MMAs where two blocks of 128 features take 96 KB, and one SM's intake from L2 is
        // what bounds a 128 x 256 tile
        const int f2 = f + GEMM_BM;
        const bool f2_ok = f2 < p.N, f2_pair_ok = (f2 | 1) < p.N;
        const bool capped = p.cap > 0.f;
        const float two_over_cap = capped ? 2.0f / p.cap : 0.f;
        for (int c0 = c_first; c0 < t_end; c0 += c_step) {
          uint32_t a[16], b[16];
          tc::tmem_ld_16(lane_addr + c0, a);
          tc::tmem_ld_16(lane_addr + p.BN + c0, b);
          tc::tmem_ld_wait();
          const int n = min(16, t_end - c0);
          float va[16], vb[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            va[j] = __uint_as_float(a[j]);
            vb[j] = __uint_as_float(b[j]);
            if (capped) {
              va[j] = softcap_fast(va[j], p.cap, two_over_cap);
              vb[j] = softcap_fast(vb[j], p.cap, two_over_cap);
            }
          }
          if (p.out_bf16) {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m0 * p.N;
            if (pairs) {
              store_bf16_pairs(o, p.N, f, f_pair_ok, c0, n, va, lane);
              store_bf16_pairs(o, p.N, f2, f2_pair_ok, c0, n, vb, lane);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (j < n && f_ok) o[(size_t)(c0 + j) * p.N + f] = __float2bfloat16_rn(va[j]);
                if (j < n && f2_ok) o[(size_t)(c0 + j) * p.N + f2] = __float2bfloat16_rn(vb[j]);
              }
            }
          } else {
            float* o = reinterpret_cast<float*>(p.out) + (size_t)m0 * p.N;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (j < n && f_ok) o[(size_t)(c0 + j) * p.N + f] = va[j];
              if (j < n && f2_ok) o[(size_t)(c0 + j) * p.N + f2] = vb[j];
            }
          }
        }
      } else if (DUAL) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m0 * p.N;
        for (int c0 = c_first; c0 < t_end; c0 += c_step) {
          uint32_t a[16], b[16];
          tc::tmem_ld_16(lane_addr + c0, a);
          tc::tmem_ld_16(lane_addr + p.BN + c0, b);
          tc::tmem_ld_wait();
          const int n = min(16, t_end - c0);
          float v[16];
          if (p.act == 0) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = gelu_tanh_fast(__uint_as_float(a[j])) * __uint_as_float(b[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float g = __uint_as_float(a[j]);
              v[j] = g * (1.0f / (1.0f + __expf(-g))) * __uint_as_float(b[j]);
            }
          }
          if (pairs) {
            store_bf16_pairs(o, p.N, f, f_pair_ok, c0, n, v, lane);
          } else if (f_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (j < n) o[(size_t)(c0 + j) * p.N + f] = __float2bfloat16_rn(v[j]);
          }
        }
      } else if (p.out_bf16) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m0 * p.N;
        const bool capped = p.cap > 0.f;
        for (int c0 = c_first; c0 < t_end; c0 += c_step) {
          uint32_t a[16];
          tc::tmem_ld_16(lane_addr + c0, a);
          tc::tmem_ld_wait();
          const int n = min(16, t_end - c0);
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(a[j]);
          if (capped) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = softcap_fast(v[j], p.cap, 2.0f / p.cap);
          }
          if (pairs) {
            store_bf16_pairs(o, p.N, f, f_pair_ok, c0, n, v, lane);
          } else if (f_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (j < n) o[(size_t)(c0 + j) * p.N + f] = __float2bfloat16_rn(v[j]);
          }
        }
      } else {
        float* o = reinterpret_cast<float*>(p.out) + (size_t)m0 * p.N + f;
        const bool capped = p.cap > 0.f;
        const float two_over_cap = capped ? 2.0f / p.cap : 0.f;
        for (int c0 = c_first; c0 < t_end; c0 += c_step) {
          uint32_t a[16];
          tc::tmem_ld_16(lane_addr + c0, a);
          tc::tmem_ld_wait();
          const int n = min(16, t_end - c0);
          if (f_ok) {
            if (capped) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (j < n) o[(size_t)(c0 + j) * p.N] = softcap_fast(__uint_as_float(a[j]), p.cap, two_over_cap);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (j < n) o[(size_t)(c0 + j) * p.N] = __uint_as_float(a[j]);
            }
          }
        }
      }
    } else if (ok) {
      // partial sums of this split: workspace[tile][split][half][column][row]
      float* mine = p.workspace + ((size_t)(tile_id * p.splits + split) * halves) * p.BN * GEMM_BM;
      for (int c0 = c_first; c0 < p.BN * halves; c0 += c_step) {
        uint32_t a[16];
        tc::tmem_ld_16(lane_addr + c0, a);
        tc::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) mine[(size_t)(c0 + j) * GEMM_BM + q * 32 + lane] = __uint_as_float(a[j]);
      }
      epi_sync(ep_threads);
      if (p.spread) {
        // Every block of the tile waits until all of them have written (they are all on an SM at the
        // same time: the host takes this path only for grids of at most one block per SM) and adds up
        // its share of the columns: one block alone would read all partial tiles through one SM.
        int* arrived = &p.counters[tile_id];
        int* departed = &p.counters[GEMM_SPREAD_DEPARTED + tile_id];
        if (threadIdx.x == 64) {
          __threadfence();
          atomicAdd(arrived, 1);
          int seen = 0;
          for (uint32_t i = 0; i < tc::WAIT_LIMIT && seen < p.splits; ++i) seen = atomicAdd(arrived, 0);
          if (seen < p.splits) *abort_flag = 1;
          sh->is_last = seen >= p.splits;
          __threadfence();
        }
        epi_sync(ep_threads);
        if (sh->is_last) {
          const float* base = p.workspace + ((size_t)tile_id * p.splits * halves) * p.BN * GEMM_BM;
          const size_t split_stride = (size_t)halves * p.BN * GEMM_BM;
          const int per = (p.BN + p.splits - 1) / p.splits;
          const int c_begin = split * per, c_end = min(p.BN, c_begin + per);
          for (int c0 = c_begin + eg * 4; c0 < c_end; c0 += c_step >> 2) {      // splits are added in order, four in flight
            float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
            for (int s0 = 0; s0 < p.splits; s0 += 4) {
              float va[4][4], vb[DUAL ? 4 : 1][4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const bool in = s0 + u < p.splits;
                const float* src = base + (size_t)(in ? s0 + u : s0) * split_stride + (size_t)c0 * GEMM_BM + q * 32 + lane;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const bool inj = in && c0 + j < c_end;
                  va[u][j] = inj ? __ldcg(src + (size_t)j * GEMM_BM) : 0.f;
                  if (DUAL) vb[u][j] = inj ? __ldcg(src + (size_t)(p.BN + j) * GEMM_BM) : 0.f;
                }
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  a[j] += va[u][j];
                  if (DUAL) b[j] += vb[u][j];
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (c0 + j < c_end) store_result<DUAL>(p, f, m0 + c0 + j, a[j], b[j]);
          }
          epi_sync(ep_threads);
          if (threadIdx.x == 64 && atomicAdd(departed, 1) == p.splits - 1) {   // everybody has read: ready for the next launch
            *arrived = 0;
            *departed = 0;
          }
        }
        sh->is_last = 0;
      }
      if (!p.spread && threadIdx.x == 64) {
        __threadfence();                 // cumulative: orders the whole block's partial sums before the count
        const int prev = atomicAdd(&p.counters[tile_id], 1);
        sh->is_last = (prev == p.splits - 1);
      }
      epi_sync(ep_threads);
      if (sh->is_last) {
        __threadfence();
        const float* base = p.workspace + ((size_t)tile_id * p.splits * halves) * p.BN * GEMM_BM;
        const size_t split_stride = (size_t)halves * p.BN * GEMM_BM;
        // 16 columns at a time; the loads of four splits are in flight together; splits are added in order
        for (int c0 = c_first; c0 < p.BN; c0 += c_step) {
          float a[16], b[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) a[j] = b[j] = 0.f;
          for (int s0 = 0; s0 < p.splits; s0 += 4) {
            float va[4][16], vb[DUAL ? 4 : 1][16];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const bool in = s0 + u < p.splits;
              const float* src = base + (size_t)(in ? s0 + u : s0) * split_stride + (size_t)c0 * GEMM_BM + q * 32 + lane;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                va[u][j] = in ? __ldcg(src + (size_t)j * GEMM_BM) : 0.f;
                if (DUAL) vb[u][j] = in ? __ldcg(src + (size_t)(p.BN + j) * GEMM_BM) : 0.f;
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                a[j] += va[u][j];
                if (DUAL) b[j] += vb[u][j];
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) store_result<DUAL>(p, f, m0 + c0 + j, a[j], b[j]);
        }
        if (threadIdx.x == 64) p.counters[tile_id] = 0;   // ready for the next launch on this stream
      }
    }
  }
  tc::fence_before_thread_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_thread_sync();
    tc::tmem_dealloc(tmem_base, tmem_cols);
  }
  if (threadIdx.x == 0 && sh->abort_flag) atomicExch(p.status, 4);
}

// ---- host side ---------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// An encoded tensor map is a pure function of the address, the shape and the box: launches look theirs
// up instead of encoding three per product (weights never move, and the allocator hands activations the
// same addresses step after step).
struct MapKey {
  const void* base;
  long long rows, cols;
  int box_rows, box_cols, kind;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows && box_cols == o.box_cols &&
           kind == o.kind;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= (size_t)k.rows * 0xC2B2AE3D27D4EB4Full + (size_t)k.cols * 0x165667B19E3779F9ull;
    h ^= ((size_t)k.box_rows << 40) ^ ((size_t)k.box_cols << 20) ^ (size_t)k.kind;
    return h;
  }
};

// kind 0: bf16 with the 128-byte swizzle (operands); 1: bf16, 2: float32 without swizzle (outputs)
static int cached_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows, int box_cols,
                      int kind) {
  static std::mutex lock;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, rows, cols, box_rows, box_cols, kind};
  {
    std::lock_guard<std::mutex> g(lock);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *map = it->second;
      return GLINT_OK;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return GLINT_ERR_BAD_ARG;
  const int es = kind == 2 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * es};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, kind == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  kind == 0 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return GLINT_ERR_BAD_ARG;
  std::lock_guard<std::mutex> g(lock);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *map);
  return GLINT_OK;
}

// A [rows, K] bf16 row-major matrix viewed as tiles of box_rows x 64 with the 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
  return cached_map(map, base, rows, K, box_rows, GEMM_BK, 0);
}

}  // namespace glint

using namespace glint;

// Sizes this kernel takes: K a multiple of 8 (rows must start on 16-byte boundaries for TMA) and
// 16-byte aligned bases.  Everything else (any M, N, K tail) is handled by zero-filled tiles.
GLINT_API int glint_gemm_tcgen05_supported(long long M, long long N, long long K) {
  return (M > 0 && N > 0 && K > 0 && K % 8 == 0) ? 1 : 0;
}

// room for the partial tiles of one block per SM at the widest tile: 148 x 2 x 256 x 128 floats and some
GLINT_API long long glint_gemm_workspace_bytes() { return 48ll << 20; }
GLINT_API int glint_gemm_counter_count() { return 8192; }

// The launch behind both entry points; ``rope`` selects the rotary epilogue of the dual kernel.
static int gemm_launch(const void* x, const void* w, void* out, int out_bf16, int M, int N, int K,
                       long long w_rows, float cap, int dual, int dual_offset, int act, float* workspace,
                       int* counters, int* status, int force_splits, const RopeEpilogue* rope, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return GLINT_OK;
  if (!glint_gemm_tcgen05_supported(M, N, K)) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return GLINT_ERR_UNSUPPORTED_SIZE;
  GemmParams p;
  if (rope) p.rope = *rope;
  else p.rope = RopeEpilogue{};
  p.M = M; p.N = N; p.K = K;
  const int bn_max = rope ? rope->bn : 256;
  const int m_tiles_256 = (M + bn_max - 1) / bn_max;
  int bn = ((M + m_tiles_256 - 1) / m_tiles_256 + 15) / 16 * 16;
  if (dual && bn > 256) bn = 256;
  int m_tiles = (M + bn - 1) / bn;
  int n_tiles = rope ? N / (2 * GEMM_BM) : (N + GEMM_BM - 1) / GEMM_BM;
  // A plain product whose 128-feature tiles would need more than one wave, and whose 256-feature
  // tiles still fill three quarters of the SMs, runs as the dual kernel with two plain tiles.
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  const int n_tiles_wide = (N + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
  p.wide = 0;
  if (!dual && !rope && force_splits <= 1 && bn == 256 && (long long)n_tiles * m_tiles > sms &&
      (long long)n_tiles_wide * m_tiles * 4 >= 3LL * sms) {
    p.wide = 1;
    dual = 1;
    dual_offset = GEMM_BM;
    n_tiles = n_tiles_wide;
  }
  // More tiles than half the SMs (fewer get a split of K below): the launch lasts as many waves as the tiles
  // need, the last one mostly empty when the count falls just behind a multiple of the SMs (4096 tokens x 3584 features in tiles of 256 x 256:
  // 224 tiles, two waves for the work of one and a half).  Token tiles a little narrower that fill the last
  // wave cost less, and so do narrower tiles that still fit one wave (2048 tokens x 16 pairs of q/k/v tiles: 128
  // tiles of 256 tokens, or 144 of 240).  A K block of a tile takes the longer of its tensor time (0.75 us for 256 features x 256
  // tokens) and its operands' way into shared memory (0.54 us for 256 + 256 rows of 128 bytes), as measured in
  // the prefill products, and a tile costs about 3 us and 8 ns per token beside its K loop (its start and its
  // epilogue, which do not overlap the next tile's loop); waves x that is made smallest, down to tiles of 128
  // tokens.
  if ((force_splits == 0 || rope) && 2ll * n_tiles * m_tiles > sms) {
    const int features = dual ? 2 * GEMM_BM : GEMM_BM;
    const int k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
    auto waves_cost = [&](int tokens, int mt) {
      const float tensor = 0.75f * features * tokens / 65536.f, intake = 0.54f * (features + tokens) / 512.f;
      return (float)(((long long)n_tiles * mt + sms - 1) / sms) * (fmaxf(tensor, intake) * k_blocks + 3.0f + 0.008f * tokens);
    };
    float best = waves_cost(bn, m_tiles);
    for (int mt = m_tiles + 1; mt <= (M + 127) / 128; ++mt) {
      const int bn_c = ((M + mt - 1) / mt + 15) / 16 * 16;
      if (bn_c < 128) break;
      const int mt_c = (M + bn_c - 1) / bn_c;
      const float cost = waves_cost(bn_c, mt_c);
      if (cost < 0.97f * best) {          // a clear gain only: the tiles of 256 tokens are the ones measured most
        best = cost;
        bn = bn_c;
        m_tiles = mt_c;
      }
    }
  }
  p.BN = bn;
  const int stage_bytes = A_STAGE_BYTES * (dual ? 2 : 1) + bn * GEMM_BK * 2;
  int stages = (227 * 1024 - 1024 - (int)sizeof(GemmShared) - 256) / stage_bytes;
  if (stages > GEMM_MAX_STAGES) stages = GEMM_MAX_STAGES;
  if (stages < 2) return GLINT_ERR_UNSUPPORTED_SIZE;
  p.stages = stages;
  p.total_kb = (K + GEMM_BK - 1) / GEMM_BK;
  const int tiles = m_tiles * n_tiles;
  int splits = 1;
  if (force_splits > 0) {
    splits = force_splits;
  } else if (2 * tiles <= sms) {
    // At most half a wave of tiles: a split of K puts the other SMs to work.  Estimated time (microseconds, fitted to measurements): the
    // K blocks a block streams at ~0.3 each, plus for a split launch the reduction through the
    // workspace, which grows with the splits and the width of the token tile.
    const int width = bn * (dual ? 2 : 1);
    float best = 1e30f;
    for (int cand = 1; cand <= 32 && tiles * cand <= sms && cand <= p.total_kb; ++cand) {
      const int per = (p.total_kb + cand - 1) / cand;
      // spread over the tile's blocks, the reduction costs the wait for the slowest block and one tile's worth of reads
      const float reduce = 6.0f + 0.04f * width;
      const float kb_us = fmaxf(0.2f, 0.0015f * width);       // a K block: instruction-bound for narrow tiles, tensor-bound for wide ones
      const float est = kb_us * per + (cand > 1 ? reduce : 0.f);
      if (est < best) {
        best = est;
        splits = cand;
      }
    }
  }
  if (splits > p.total_kb) splits = p.total_kb;
  p.kb_per_split = (p.total_kb + splits - 1) / splits;
  splits = (p.total_kb + p.kb_per_split - 1) / p.kb_per_split;
  const long long ws_need = (long long)tiles * splits * (dual ? 2 : 1) * bn * GEMM_BM * 4;
  if (splits > 1 && (ws_need > glint_gemm_workspace_bytes() || tiles > glint_gemm_counter_count() ||
                     !workspace || !counters)) {      // cannot happen while tiles x splits fit the SMs (see the workspace's size)
    splits = 1;
    p.kb_per_split = p.total_kb;
  }
  p.splits = splits;
  p.spread = (splits > 1 && (long long)tiles * splits <= sms && tiles <= GEMM_SPREAD_DEPARTED) ? 1 : 0;
  p.dual_offset = dual_offset;
  p.act = act;
  p.cap = cap;
  p.out_bf16 = out_bf16;
  p.out = out;
  p.workspace = workspace;
  p.counters = counters;
  p.status = status;

  CUtensorMap map_w, map_x;
  int rc = make_map(&map_w, w, w_rows, K, GEMM_BM);
  if (rc != GLINT_OK) return rc;
  rc = make_map(&map_x, x, M, K, bn);
  if (rc != GLINT_OK) return rc;
  const int smem_bytes = stages * stage_bytes + (int)sizeof(GemmShared) + 1024;
  p.m_tiles = m_tiles;
  // the staged epilogue: bfloat16 output (two-byte global stores are slow; for float32 the direct
  // stores measured faster), token tiles of 64 and more, no split, output rows on 16-byte boundaries
  CUtensorMap map_out = map_x;
  const int es = out_bf16 ? 2 : 4;
  p.tma_store = 0;
  if (!p.wide && !rope && out_bf16 && splits == 1 && bn >= 64 && ((long long)N * es) % 16 == 0 && ((uintptr_t)out & 15) == 0 &&
      (long long)bn * GEMM_BM * es <= (long long)stages * stage_bytes) {
    if (cached_map(&map_out, out, M, N, bn, GEMM_BM, out_bf16 ? 1 : 2) == GLINT_OK) p.tma_store = 1;
  }
  const int threads = bn * (dual ? 2 : 1) >= 64 ? GEMM_THREADS_WIDE : GEMM_THREADS;
  dim3 grid(n_tiles * m_tiles, 1, splits);
  cudaError_t e;
  // the shared-memory limit of each kernel is raised once, to the most a launch may ask for
  static int limit_set[2] = {-1, -1};      // the device it was raised on
  const int smem_limit = 227 * 1024;
  int device_now = 0;
  cudaGetDevice(&device_now);
  if (limit_set[dual ? 1 : 0] != device_now) {
    e = dual ? cudaFuncSetAttribute(gemm_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_limit)
             : cudaFuncSetAttribute(gemm_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_limit);
    if (e != cudaSuccess) return (int)e;
    limit_set[dual ? 1 : 0] = device_now;
  }
  if (dual)
    e = launch_kernel(gemm_tcgen05_kernel<true>, grid, dim3(threads), smem_bytes, stream, map_w, map_x, map_out, p);
  else
    e = launch_kernel(gemm_tcgen05_kernel<false>, grid, dim3(threads), smem_bytes, stream, map_w, map_x, map_out, p);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

// x: [M, K] bf16; w: [N (or 2N rows when dual), K] bf16; out: [M, N] float32 or bf16.
// dual != 0: out = act(x w[0:N]^T) * (x w[dual_offset : dual_offset+N]^T), written as bf16.
// workspace: glint_gemm_workspace_bytes() bytes; counters: glint_gemm_counter_count() zeroed ints.
GLINT_API int glint_gemm_tcgen05(const void* x, const void* w, void* out, int out_bf16, int M, int N, int K,
                                 long long w_rows, float cap, int dual, int dual_offset, int act,
                                 float* workspace, int* counters, int* status, int force_splits,
                                 cudaStream_t stream) {
  return gemm_launch(x, w, out, out_bf16, M, N, K, w_rows, cap, dual, dual_offset, act, workspace, counters, status,
                     force_splits, nullptr, stream);
}

// Head sizes the rotary epilogue takes: a thread of the dual kernel holds features j and j + 128 g.
// The grid is heads x token tiles with no split of K, so it also wants enough tokens to fill half of the
// SMs with tiles of 256 or of 128 tokens (``min_blocks`` 0: any number of tokens).
static int rope_token_tile(long long M, int head_tiles, int min_blocks) {
  for (int bn = 256; bn >= 128; bn >>= 1)
    if (head_tiles * ((M + bn - 1) / bn) >= min_blocks) return bn;
  return 0;
}

GLINT_API int glint_gemm_tcgen05_rope_supported(long long M, long long K, int hd, int heads, int min_blocks) {
  if (!(M > 0 && K > 0 && K % 8 == 0 && hd >= 256 && hd % 256 == 0 && heads > 0)) return 0;
  return rope_token_tile(M, heads * (hd / 256), min_blocks) ? 1 : 0;
}

// q, k, v = x w^T for w: [(nh + 2 nkv) hd, K] with the rotation by the angles of ``trig`` ([M][hd/2]
// (cos, sin)) and the cache write in the epilogue: q to q_out [M, nh hd] bf16, k and v into the pages
// named by block_table at each token's position (k_pool null: only q is computed).
GLINT_API int glint_gemm_tcgen05_rope(const void* x, const void* w, int M, int K, const float* trig,
                                      const int* positions, const int* token_seq, const int* block_table,
                                      int max_pages, void* q_out, void* k_pool, void* v_pool, int nh, int nkv,
                                      int hd, int page_size, int num_pages, int min_blocks, int* status,
                                      cudaStream_t stream) {
  if (M <= 0) return GLINT_OK;
  if (nh <= 0 || nkv <= 0 || page_size <= 0 || !glint_gemm_tcgen05_rope_supported(M, K, hd, nh, 0)) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (!trig || !status || !q_out || (k_pool && !v_pool)) return GLINT_ERR_BAD_ARG;
  if (((uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)trig) & 15) return GLINT_ERR_UNSUPPORTED_SIZE;
  RopeEpilogue r;
  r.on = 1;
  r.trig = reinterpret_cast<const float2*>(trig);
  r.positions = positions; r.token_seq = token_seq; r.block_table = block_table; r.max_pages = max_pages;
  r.k_pool = k_pool; r.v_pool = v_pool;
  r.nh = nh; r.nkv = nkv; r.hd = hd; r.page_size = page_size; r.num_pages = num_pages;
  const long long rows = (long long)(nh + 2 * nkv) * hd;
  const int heads = k_pool ? nh + 2 * nkv : nh;
  r.bn = rope_token_tile(M, heads * (hd / 256), min_blocks);
  if (r.bn == 0) r.bn = 128;
  return gemm_launch(x, w, q_out, 1, M, heads * hd, K, rows, 0.f, 1, hd / 2, 0, nullptr, nullptr, status, 1, &r, stream);
}

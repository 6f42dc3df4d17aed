// Weight-streaming product for a handful of tokens: out[M, N] = x[M, K] @ w[N, K]^T, M <= 16.
//
// With so few tokens a projection is a stream of its weights and nothing else, and what a launch
// costs besides the stream decides its time: the tiled tensor-memory kernel pays for barriers,
// tensor-memory allocation, a copy pipeline and a split-K pass through a workspace (8 to 10 us for
// a product whose weights stream in 2 us).  This kernel has none of that.  A block owns 16 output
// features; its warps split K among themselves in steps of 64 and every lane loads its operands
// straight from global memory into the registers of m16n8k16 fragments:
//
//   lane (g = lane / 4, tq = lane % 4) reads 16 bytes of weight rows g and g + 8 and of token g at
//   k = step * 64 + chunk * 32 + 8 * tq.  The four bfloat16 pairs it holds feed two MMAs: pairs 0, 1
//   stand at the fragment's k = 2 tq and 2 tq + 8 in the first, pairs 2, 3 in the second.  The
//   contraction index is permuted the same way in both operands, so the sum is the same, and each
//   weight row is read in whole 128-byte lines.
//
// The first weights are requested before the wait for the kernel that produces x, partial sums of
// the warps are added in shared memory in a fixed order (the result does not depend on timing), and
// the epilogue applies the soft cap or the gated activation.  Arithmetic: bfloat16 products, float32
// sums.  The reference's counterpart is its batched matvec, src/tensor/quantized.rs:278-337.
#include "common.cuh"

namespace glint {

constexpr int SK_MAX_WARPS = 16;
constexpr int SK_ROWS = 16;       // output features per block
constexpr int SK_STEP = 64;       // k per step and warp

__device__ __forceinline__ void mma_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// weights are read once: keep them out of L1
__device__ __forceinline__ uint4 load_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

struct SkinnyParams {
  const __nv_bfloat16* w;
  const __nv_bfloat16* x;
  void* out;
  int out_bf16;
  int M, N, K;
  float cap;
  int dual_offset;      // gated: row of w where the second (up) half begins
  int activation;       // gated: 0 gelu_tanh, 1 silu
  // rotary mode: w is [q heads | k heads | v heads] x head_dim rows; q is rotated into q_out, k is
  // rotated and v copied into the cache row of each token's position
  const int* positions;
  const int* token_slot;
  const int* block_table;
  int max_pages;
  const float* inv_freq;
  float factor;
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_pool;
  __nv_bfloat16* v_pool;
  int nh, nkv, hd, page_size, num_pages;
  int* status;
};

constexpr int SK_PLAIN = 0, SK_GATED = 1, SK_ROPE = 2;

// NT: token tiles of 8; U: steps in flight per warp.  MODE: plain (soft cap in the epilogue), gated
// (two weight rows per feature and act(gate) * up in the epilogue) or rotary (see SkinnyParams:
// a block owns 8 rotation pairs (j, j + head_dim / 2) of one q or k head, or 16 dims of a v head,
// so that the epilogue holds both halves of every pair it turns; src/tensor/ops.rs:212-245).
template <int NT, int MODE, int U>
__global__ void __launch_bounds__(SK_MAX_WARPS * 32) gemm_skinny_kernel(const SkinnyParams p) {
  constexpr bool GATED = MODE == SK_GATED;
  constexpr int SETS = GATED ? 2 : 1;
  __shared__ float red[SK_MAX_WARPS][SETS][SK_ROWS][8 * NT + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_warps = blockDim.x >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int row0 = blockIdx.x * SK_ROWS;
  const int K = p.K;
  const int n_steps = K / SK_STEP;
  // rows beyond N are clamped for the loads and masked at the store
  int ra = min(row0 + g, p.N - 1), rb = min(row0 + g + 8, p.N - 1);
  int rope_head = 0, rope_sub = 0;
  if (MODE == SK_ROPE) {
    const int per_head = p.hd >> 4;
    rope_head = blockIdx.x / per_head;
    rope_sub = blockIdx.x - rope_head * per_head;
    if (rope_head < p.nh + p.nkv) {                  // q or k: dims 8 sub + g and that + head_dim / 2
      ra = rope_head * p.hd + rope_sub * 8 + g;
      rb = ra + (p.hd >> 1);
    } else {                                         // v: 16 consecutive dims
      ra = rope_head * p.hd + rope_sub * 16 + g;
      rb = ra + 8;
    }
  }
  const __nv_bfloat16* wrow[SETS][2];
  wrow[0][0] = p.w + (size_t)ra * K + 8 * tq;
  wrow[0][1] = p.w + (size_t)rb * K + 8 * tq;
  if (GATED) {
    wrow[SETS - 1][0] = p.w + (size_t)(ra + p.dual_offset) * K + 8 * tq;
    wrow[SETS - 1][1] = p.w + (size_t)(rb + p.dual_offset) * K + 8 * tq;
  }
  const __nv_bfloat16* xrow[NT];
  bool xvalid[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int tok = nt * 8 + g;
    xvalid[nt] = tok < p.M;
    xrow[nt] = p.x + (size_t)(xvalid[nt] ? tok : 0) * K + 8 * tq;
  }
  float acc[SETS][NT][4];
#pragma unroll
  for (int s = 0; s < SETS; ++s)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[s][nt][i] = 0.f;

  bool waited = false;
  for (int s0 = warp; s0 < n_steps; s0 += n_warps * U) {
    uint4 wv[U][2][SETS][2];       // [step][chunk][set][row g / g + 8]
    uint4 xv[U][2][NT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = s0 + u * n_warps;
      if (s < n_steps) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int set = 0; set < SETS; ++set)
#pragma unroll
            for (int h = 0; h < 2; ++h) wv[u][c][set][h] = load_stream(wrow[set][h] + s * SK_STEP + c * 32);
      }
    }
    if (!waited) {       // x comes from the kernel before this one; the weights above did not have to wait
      pdl_wait_release();
      waited = true;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = s0 + u * n_warps;
      if (s < n_steps) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
            xv[u][c][nt] = xvalid[nt] ? *reinterpret_cast<const uint4*>(xrow[nt] + s * SK_STEP + c * 32)
                                      : make_uint4(0u, 0u, 0u, 0u);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = s0 + u * n_warps;
      if (s < n_steps) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int set = 0; set < SETS; ++set) {
            const uint4 a = wv[u][c][set][0], b = wv[u][c][set][1];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const uint4 x = xv[u][c][nt];
              mma_16816(acc[set][nt], a.x, b.x, a.y, b.y, x.x, x.y);
              mma_16816(acc[set][nt], a.z, b.z, a.w, b.w, x.z, x.w);
            }
          }
      }
    }
  }
  if (!waited) pdl_wait_release();

  // ---- the warps' partial sums, added in warp order ---------------------------------------------------
#pragma unroll
  for (int set = 0; set < SETS; ++set)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      red[warp][set][g][nt * 8 + 2 * tq] = acc[set][nt][0];
      red[warp][set][g][nt * 8 + 2 * tq + 1] = acc[set][nt][1];
      red[warp][set][g + 8][nt * 8 + 2 * tq] = acc[set][nt][2];
      red[warp][set][g + 8][nt * 8 + 2 * tq + 1] = acc[set][nt][3];
    }
  __syncthreads();
  if (MODE == SK_ROPE) {
    // thread (pair j, token): both halves of the pair, turned by the token's position
    if (threadIdx.x < 64 * NT) {
      const int j = threadIdx.x & 7, tok = threadIdx.x >> 3;
      if (tok < p.M) {
        float v0 = 0.f, v1 = 0.f;
        for (int w = 0; w < n_warps; ++w) {
          v0 += red[w][0][j][tok];
          v1 += red[w][0][j + 8][tok];
        }
        const int pos = p.positions[tok];
        const bool rotated = rope_head < p.nh + p.nkv;
        int d0, d1;
        if (rotated) {
          d0 = rope_sub * 8 + j;
          d1 = d0 + (p.hd >> 1);
          float sn, cs;
          sincosf(((float)pos / p.factor) * p.inv_freq[d0], &sn, &cs);
          const float a = v0 * cs - v1 * sn, b = v0 * sn + v1 * cs;
          v0 = a;
          v1 = b;
        } else {
          d0 = rope_sub * 16 + j;
          d1 = d0 + 8;
        }
        __nv_bfloat16* dst = nullptr;
        if (rope_head < p.nh) {
          dst = p.q_out + ((size_t)tok * p.nh + rope_head) * p.hd;
        } else if (p.k_pool) {
          const int page = p.block_table[(size_t)p.token_slot[tok] * p.max_pages + pos / p.page_size];
          if (page < 0 || page >= p.num_pages) {
            atomicExch(p.status, 2);
          } else {
            const bool is_k = rope_head < p.nh + p.nkv;
            const int kvh = rope_head - p.nh - (is_k ? 0 : p.nkv);
            dst = (is_k ? p.k_pool : p.v_pool) + (((size_t)page * p.nkv + kvh) * p.page_size + pos % p.page_size) * p.hd;
          }
        }
        if (dst) {
          dst[d0] = __float2bfloat16_rn(v0);
          dst[d1] = __float2bfloat16_rn(v1);
        }
      }
    }
    return;
  }
  // consecutive threads take consecutive features of one token: whole segments of the output row
  for (int e = threadIdx.x; e < SK_ROWS * 8 * NT; e += blockDim.x) {
    const int r = e % SK_ROWS, tok = e / SK_ROWS;
    const int f = row0 + r;
    if (tok >= p.M || f >= p.N) continue;
    float v = 0.f;
    for (int w = 0; w < n_warps; ++w) v += red[w][0][r][tok];
    if (GATED) {
      float up = 0.f;
      for (int w = 0; w < n_warps; ++w) up += red[w][SETS - 1][r][tok];
      v = (p.activation == 0 ? gelu_tanh(v) : v / (1.0f + __expf(-v))) * up;
    } else if (p.cap > 0.f) {
      v = softcap(v, p.cap);
    }
    const size_t o = (size_t)tok * p.N + f;
    if (p.out_bf16) reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(p.out)[o] = v;
  }
}

}  // namespace glint

using namespace glint;

// Every pass of a warp over its steps costs one memory latency.  When the blocks fill the SMs at
// most once, a block has 12 or 16 warps, whichever makes the passes fewest and leaves the fewest
// step slots empty: more bytes in flight per SM.  With more blocks than that, small blocks (8
// warps) pack the SMs better.
static int skinny_warps(int U, int n_steps, int n_blocks) {
  int device = 0, sms = 148;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  int warps = 8;
  if (n_blocks <= sms) {
    int best_passes = 1 << 30, best_waste = 1 << 30;
    for (int w = 12; w <= SK_MAX_WARPS; w += 4) {
      const int passes = (n_steps + w * U - 1) / (w * U), waste = passes * w * U - n_steps;
      if (passes < best_passes || (passes == best_passes && waste < best_waste)) {
        warps = w; best_passes = passes; best_waste = waste;
      }
    }
  }
  return warps;
}


// Up to 16 tokens, K a multiple of 64, 16-byte aligned operands.
GLINT_API int glint_gemm_skinny_supported(int M, int N, int K) {
  return (M >= 1 && M <= 16 && N >= 1 && K >= SK_STEP && K % SK_STEP == 0) ? 1 : 0;
}

// x [M, K], w [w_rows, K] bfloat16; out [M, N] float32 or bfloat16.  gated: feature f is
// act(x . w[f]) * (x . w[dual_offset + f]), out is [M, N] with N the gated width.
GLINT_API int glint_gemm_skinny(const void* x, const void* w, void* out, int out_bf16, int M, int N, int K, float cap,
                                int gated, int dual_offset, int activation, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return GLINT_OK;
  if (!glint_gemm_skinny_supported(M, N, K)) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (gated && (activation < 0 || activation > 1)) return GLINT_ERR_BAD_ARG;
  SkinnyParams p;
  p.w = (const __nv_bfloat16*)w; p.x = (const __nv_bfloat16*)x; p.out = out; p.out_bf16 = out_bf16;
  p.M = M; p.N = N; p.K = K; p.cap = cap; p.dual_offset = dual_offset; p.activation = activation;
  const int warps = skinny_warps(M <= 8 ? (gated ? 2 : 4) : (gated ? 1 : 2), K / SK_STEP, (N + SK_ROWS - 1) / SK_ROWS);
  const dim3 grid((N + SK_ROWS - 1) / SK_ROWS), block(warps * 32);
  cudaError_t e;
  if (M <= 8) {
    if (gated) e = launch_kernel(gemm_skinny_kernel<1, SK_GATED, 2>, grid, block, 0, stream, p);
    else e = launch_kernel(gemm_skinny_kernel<1, SK_PLAIN, 4>, grid, block, 0, stream, p);
  } else {
    if (gated) e = launch_kernel(gemm_skinny_kernel<2, SK_GATED, 1>, grid, block, 0, stream, p);
    else e = launch_kernel(gemm_skinny_kernel<2, SK_PLAIN, 2>, grid, block, 0, stream, p);
  }
  return (int)e;
}

// The q, k, v product of up to 16 tokens with the rotary encoding and the cache write in its
// epilogue: x [M, K]; w [(nh + 2 nkv) * hd, K]; q_out [M, nh * hd]; pools [pages][nkv][page_size][hd]
// (null: q only).  The whole head is rotated (pairs (j, j + hd / 2)); hd a multiple of 16.
GLINT_API int glint_gemm_skinny_rope_supported(int M, int K, int hd) {
  return (M >= 1 && M <= 16 && K >= SK_STEP && K % SK_STEP == 0 && hd >= 16 && hd % 16 == 0) ? 1 : 0;
}

GLINT_API int glint_gemm_skinny_rope(const void* x, const void* w, int M, int K, const int* positions,
                                     const int* token_slot, const int* block_table, int max_pages,
                                     const float* inv_freq, float factor, void* q_out, void* k_pool, void* v_pool,
                                     int nh, int nkv, int hd, int page_size, int num_pages, int* status,
                                     cudaStream_t stream) {
  if (M <= 0) return GLINT_OK;
  if (!glint_gemm_skinny_rope_supported(M, K, hd) || nh <= 0 || nkv < 0 || page_size <= 0 || factor == 0.f)
    return GLINT_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return GLINT_ERR_UNSUPPORTED_SIZE;
  SkinnyParams p = {};
  p.w = (const __nv_bfloat16*)w; p.x = (const __nv_bfloat16*)x; p.M = M; p.K = K;
  const int heads = k_pool ? nh + 2 * nkv : nh;       // without a cache to write, k and v are not computed
  p.N = heads * hd;
  p.positions = positions; p.token_slot = token_slot; p.block_table = block_table; p.max_pages = max_pages;
  p.inv_freq = inv_freq; p.factor = factor; p.q_out = (__nv_bfloat16*)q_out; p.k_pool = (__nv_bfloat16*)k_pool;
  p.v_pool = (__nv_bfloat16*)v_pool; p.nh = nh; p.nkv = nkv; p.hd = hd; p.page_size = page_size;
  p.num_pages = num_pages; p.status = status;
  const int n_blocks = heads * (hd / 16);
  if (M > 8) {
    const int warps = skinny_warps(2, K / SK_STEP, n_blocks);
    return (int)launch_kernel(gemm_skinny_kernel<2, SK_ROPE, 2>, dim3(n_blocks), dim3(warps * 32), 0, stream, p);
  }
  const int warps = skinny_warps(4, K / SK_STEP, n_blocks);
  return (int)launch_kernel(gemm_skinny_kernel<1, SK_ROPE, 4>, dim3(n_blocks), dim3(warps * 32), 0, stream, p);
}

// Attention of prompt portions over the paged cache: flash attention in bfloat16 with
// mma.sync tensor-core tiles and 32-bit online softmax.
//
// grid = (query tiles, requests of the step, kv heads).  A block of 4 warps owns 64 query rows:
// rows are (token, query head of the group) pairs, so the heads that share a kv head share each
// key/value tile.  Keys come in tiles of 64 whose boundaries are multiples of 64 in absolute
// position; a tile is gathered page by page with 16-byte cp.async copies.  Scores, soft cap,
// masks (causal and sliding window by absolute position), running max/sum and the output
// accumulator are float32; probabilities are rounded to bfloat16 for the second product.
// Formulas: src/tensor/flash.rs:65-123 (online softmax), :76-87 (multiplier, cap),
// src/transformer/forward.rs:933-942 (window per absolute position).
#include "common.cuh"

namespace glint {

constexpr int PF_ROWS = 64;      // query rows per block
constexpr int PF_KEYS = 64;      // keys per tile
constexpr int PF_THREADS = 128;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, bool valid) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* smem_ptr) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* smem_ptr) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// HD: capacity of a shared-memory row (head_dim <= HD, head_dim a multiple of 16).
template <int HD>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ cu_seqlens,
                         const int* __restrict__ seq_start, const int* __restrict__ block_table, int max_pages,
                         __nv_bfloat16* __restrict__ out, int nh, int nkv, int hd, int page_size, int num_pages,
                         float multiplier, float cap, int window, int* __restrict__ status) {
  constexpr int LD = HD + 8;   // padded row: ldmatrix rows land in different banks
  extern __shared__ __align__(16) uint8_t pf_smem[];
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(pf_smem);
  __nv_bfloat16* sk = sq + PF_ROWS * LD;
  __nv_bfloat16* sv = sk + PF_KEYS * LD;

  const int seq = blockIdx.y, kvh = blockIdx.z;
  const int G = nh / nkv;
  const int tok_per_tile = PF_ROWS / G;
  const int t_begin = cu_seqlens[seq];
  const int q_len = cu_seqlens[seq + 1] - t_begin;
  const int tok0 = blockIdx.x * tok_per_tile;
  if (tok0 >= q_len) return;
  const int n_tok = min(tok_per_tile, q_len - tok0);
  const int n_rows = n_tok * G;
  const int pos0 = seq_start[seq] + tok0;          // position of the tile's first token
  const int pos_last = pos0 + n_tok - 1;
  const int* table = block_table + (size_t)seq * max_pages;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pieces = hd >> 3, hd16 = hd >> 4;

  // zero the padding columns once (dims >= head_dim take part in the products as zeros)
  if (hd < HD) {
    const int extra = (HD - hd) >> 3;
    for (int idx = tid; idx < 3 * PF_ROWS * extra; idx += PF_THREADS) {
      const int r = idx / extra, c = pieces + idx % extra;
      *reinterpret_cast<uint4*>(sq + (size_t)r * LD + c * 8) = make_uint4(0, 0, 0, 0);
    }
  }
  // the query tile: row r = (token r / G, head kvh * G + r % G)
  for (int idx = tid; idx < PF_ROWS * pieces; idx += PF_THREADS) {
    const int r = idx / pieces, c = idx % pieces;
    const bool valid = r < n_rows;
    const __nv_bfloat16* src =
        q + ((size_t)(t_begin + tok0 + (valid ? r / G : 0)) * nh + kvh * G + (valid ? r % G : 0)) * hd + c * 8;
    cp_async16(sq + (size_t)r * LD + c * 8, src, valid);
  }
  cp_async_commit();

  const int g = lane >> 2, tq = lane & 3;
  const int row0 = warp * 16 + g, row1 = row0 + 8;
  const int qpos0 = pos0 + row0 / G, qpos1 = pos0 + row1 / G;      // meaningful for valid rows only
  const bool rv0 = row0 < n_rows, rv1 = row1 < n_rows;
  const int lo0 = window > 0 ? qpos0 - window + 1 : 0, lo1 = window > 0 ? qpos1 - window + 1 : 0;

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  const int kv_first = window > 0 ? max(0, pos0 - window + 1) : 0;
  for (int kv0 = kv_first & ~(PF_KEYS - 1); kv0 <= pos_last; kv0 += PF_KEYS) {
    __syncthreads();   // everyone is done with the previous tile
    for (int idx = tid; idx < PF_KEYS * pieces; idx += PF_THREADS) {
      const int r = idx / pieces, c = idx % pieces;
      const int key = kv0 + r;
      bool valid = key >= kv_first && key <= pos_last;
      int page = 0;
      if (valid) {
        page = table[key / page_size];
        if (page < 0 || page >= num_pages) {
          atomicExch(status, 3);
          valid = false;
          page = 0;
        }
      }
      const size_t off = (((size_t)page * nkv + kvh) * page_size + (valid ? key % page_size : 0)) * hd + c * 8;
      cp_async16(sk + (size_t)r * LD + c * 8, k_pool + off, valid);
      cp_async16(sv + (size_t)r * LD + c * 8, v_pool + off, valid);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // ---- S = Q K^T : 16 rows x 64 keys per warp ---------------------------------------------------
    float s[PF_KEYS / 8][4];
#pragma unroll
    for (int i = 0; i < PF_KEYS / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      if (ks < hd16) {
        uint32_t a[4];
        ldmatrix_x4(a, sq + (size_t)(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int nb2 = 0; nb2 < PF_KEYS / 16; ++nb2) {
          uint32_t b[4];
          ldmatrix_x4(b, sk + (size_t)(nb2 * 16 + (lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * nb2], a, b[0], b[1]);
          mma_bf16(s[2 * nb2 + 1], a, b[2], b[3]);
        }
      }
    }
    // ---- scale, cap, mask, online softmax -----------------------------------------------------------
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < PF_KEYS / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kv0 + nb * 8 + tq * 2 + (e & 1);
        const bool upper = e < 2;
        const bool ok = upper ? (rv0 && key <= qpos0 && key >= lo0) : (rv1 && key <= qpos1 && key >= lo1);
        const float v = ok ? softcap(s[nb][e] * multiplier, cap) : -INFINITY;
        s[nb][e] = v;
        if (upper) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
    const float corr0 = __expf(m0 - base0), corr1 = __expf(m1 - base1);
    m0 = mn0;
    m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int nb = 0; nb < PF_KEYS / 8; ++nb) {
      s[nb][0] = __expf(s[nb][0] - base0);
      s[nb][1] = __expf(s[nb][1] - base0);
      s[nb][2] = __expf(s[nb][2] - base1);
      s[nb][3] = __expf(s[nb][3] - base1);
      sum0 += s[nb][0] + s[nb][1];
      sum1 += s[nb][2] + s[nb][3];
    }
    l0 = l0 * corr0 + sum0;   // per-thread partial sums; the four lanes of a row are added at the end
    l1 = l1 * corr1 + sum1;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      o[i][0] *= corr0;
      o[i][1] *= corr0;
      o[i][2] *= corr1;
      o[i][3] *= corr1;
    }
    // ---- O += P V ---------------------------------------------------------------------------------
#pragma unroll
    for (int kk = 0; kk < PF_KEYS / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int db = 0; db < HD / 16; ++db) {
        if (db < hd16) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, sv + (size_t)(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + db * 16 + (lane >> 4) * 8);
          mma_bf16(o[2 * db], a, b[0], b[1]);
          mma_bf16(o[2 * db + 1], a, b[2], b[3]);
        }
      }
    }
  }
  // ---- normalize and write -----------------------------------------------------------------------
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.0f / l0 : 0.f, inv1 = l1 > 0.f ? 1.0f / l1 : 0.f;
  __nv_bfloat16* orow0 = out + ((size_t)(t_begin + tok0 + (rv0 ? row0 / G : 0)) * nh + kvh * G + (rv0 ? row0 % G : 0)) * hd;
  __nv_bfloat16* orow1 = out + ((size_t)(t_begin + tok0 + (rv1 ? row1 / G : 0)) * nh + kvh * G + (rv1 ? row1 % G : 0)) * hd;
#pragma unroll
  for (int nb = 0; nb < HD / 8; ++nb) {
    const int d = nb * 8 + tq * 2;
    if (d < hd) {
      if (rv0) *reinterpret_cast<uint32_t*>(orow0 + d) = pack_bf16(o[nb][0] * inv0, o[nb][1] * inv0);
      if (rv1) *reinterpret_cast<uint32_t*>(orow1 + d) = pack_bf16(o[nb][2] * inv1, o[nb][3] * inv1);
    }
  }
}

}  // namespace glint

using namespace glint;

// head_dim a multiple of 16 up to 256; heads per kv head at most 64.
GLINT_API int glint_attention_prefill_supported(int nh, int nkv, int hd) {
  return (nkv > 0 && nh % nkv == 0 && nh / nkv <= PF_ROWS && hd % 16 == 0 && hd >= 16 && hd <= 256) ? 1 : 0;
}

GLINT_API int glint_attention_prefill(const void* q, const void* k_pool, const void* v_pool, const int* cu_seqlens,
                                      const int* seq_start, const int* block_table, int max_pages, void* out,
                                      int n_seqs, int max_q_len, int nh, int nkv, int hd, int page_size,
                                      int num_pages, float multiplier, float cap, int window, int* status,
                                      cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return GLINT_OK;
  if (!glint_attention_prefill_supported(nh, nkv, hd)) return GLINT_ERR_UNSUPPORTED_SIZE;
  if (page_size <= 0) return GLINT_ERR_BAD_ARG;
  const int tok_per_tile = PF_ROWS / (nh / nkv);
  dim3 grid((max_q_len + tok_per_tile - 1) / tok_per_tile, n_seqs, nkv);
  if (grid.y > 65535 || grid.z > 65535) return GLINT_ERR_UNSUPPORTED_SIZE;
  const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)k_pool,
                      *vv = (const __nv_bfloat16*)v_pool;
#define LAUNCH(HD)                                                                                              \
  {                                                                                                             \
    const int smem = 3 * PF_ROWS * (HD + 8) * 2;                                                                \
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         smem);                                                                 \
    if (e != cudaSuccess) return (int)e;                                                                        \
    attention_prefill_kernel<HD><<<grid, PF_THREADS, smem, stream>>>(qq, kk, vv, cu_seqlens, seq_start, block_table, \
                                                                    max_pages, (__nv_bfloat16*)out, nh, nkv, hd, \
                                                                    page_size, num_pages, multiplier, cap, window, \
                                                                    status);                                    \
  }
  if (hd <= 64) LAUNCH(64)
  else if (hd <= 128) LAUNCH(128)
  else LAUNCH(256)
#undef LAUNCH
  return (int)cudaGetLastError();
}

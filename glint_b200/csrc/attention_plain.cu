// Attention over the paged cache, plain form: one warp per (token, query head).
//
// The warp walks the keys of its request from the window start to the token's own position
// in order, one key at a time, with an online softmax; so the result for a token depends
// only on the cache contents and its position, never on how the batch was cut.  Formulas:
// score = (q . k) * multiplier, then cap * tanh(score / cap) (src/tensor/flash.rs:76-87);
// online softmax and weighted sum of values (src/tensor/flash.rs:65-123); keys from
// max(0, pos - window + 1) to pos (src/transformer/forward.rs:574-582); query head h reads
// kv head h / (heads / kv_heads) (src/transformer/forward.rs:255).
// This is the attention of the 32-bit path and the yardstick of the tensor-core kernels.
#include "common.cuh"

namespace glint {

constexpr int MAX_DIMS_PER_LANE = 16;  // head_dim <= 512

template <typename S>
__global__ void __launch_bounds__(128)
attention_plain_kernel(const S* __restrict__ q, const S* __restrict__ k_pool,
                       const S* __restrict__ v_pool, const int* __restrict__ positions,
                       const int* __restrict__ token_slot, const int* __restrict__ block_table,
                       int max_pages, S* __restrict__ out, int T, int nh, int nkv, int hd,
                       int page_size, int num_pages, float multiplier, float cap, int window,
                       int* __restrict__ status) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T * nh) return;
  const int t = warp / nh, h = warp % nh;
  const int g = h / (nh / nkv);
  const int pos = positions[t];
  const int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* table = block_table + (size_t)token_slot[t] * max_pages;
  const int per_lane = (hd + 31) / 32;

  float qv[MAX_DIMS_PER_LANE], acc[MAX_DIMS_PER_LANE];
  const S* qrow = q + ((size_t)t * nh + h) * hd;
#pragma unroll
  for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    qv[i] = (i < per_lane && d < hd) ? to_float(qrow[d]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int p = start; p <= pos; ++p) {
    const int page = table[p / page_size];
    if (page < 0 || page >= num_pages) {  // a key the block table does not hold: report, skip
      if (lane == 0) atomicExch(status, 3);
      continue;
    }
    const size_t base = (((size_t)page * nkv + g) * page_size + (p % page_size)) * hd;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (i < per_lane && d < hd) dot = fmaf(qv[i], to_float(k_pool[base + d]), dot);
    }
    dot = warp_sum(dot);
    const float s = softcap(dot * multiplier, cap);
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);
    const float e = expf(s - m_new);
    l = l * corr + e;
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (i < per_lane && d < hd) acc[i] = acc[i] * corr + e * to_float(v_pool[base + d]);
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  S* orow = out + ((size_t)t * nh + h) * hd;
#pragma unroll
  for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (i < per_lane && d < hd) orow[d] = from_float<S>(acc[i] * inv);
  }
}

}  // namespace glint

using namespace glint;

// window <= 0: attend from position 0.  cap <= 0: no soft cap.
GLINT_API int glint_attention_plain(const void* q, const void* k_pool, const void* v_pool, int dtype,
                                    const int* positions, const int* token_slot,
                                    const int* block_table, int max_pages, void* out, int T, int nh,
                                    int nkv, int hd, int page_size, int num_pages, float multiplier,
                                    float cap, int window, int* status, cudaStream_t stream) {
  if (T <= 0) return GLINT_OK;
  if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0) return GLINT_ERR_BAD_ARG;
  if (hd <= 0 || hd > 32 * MAX_DIMS_PER_LANE) return GLINT_ERR_UNSUPPORTED_SIZE;
  const long long warps = (long long)T * nh;
  const unsigned blocks = (unsigned)((warps + 3) / 4);
  if (dtype == GLINT_DTYPE_F32)
    attention_plain_kernel<float><<<blocks, 128, 0, stream>>>(
        (const float*)q, (const float*)k_pool, (const float*)v_pool, positions, token_slot, block_table,
        max_pages, (float*)out, T, nh, nkv, hd, page_size, num_pages, multiplier, cap, window, status);
  else if (dtype == GLINT_DTYPE_BF16)
    attention_plain_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, positions,
        token_slot, block_table, max_pages, (__nv_bfloat16*)out, T, nh, nkv, hd, page_size, num_pages,
        multiplier, cap, window, status);
  else
    return GLINT_ERR_BAD_ARG;
  return (int)cudaGetLastError();
}

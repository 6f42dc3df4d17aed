// Embedding, norms, position encoding with cache write, gated activation, soft cap.
//
// Plain one-block-per-row kernels, templated on the storage type (float or bf16); all
// arithmetic, and the residual stream itself, is 32-bit float.  Reference formulas:
// embedding * sqrt(hidden) src/transformer/forward.rs:73-83; (1+w) RMSNorm
// src/tensor/ops.rs:134-152; RoPE src/tensor/ops.rs:212-245 (applied here in the
// rotate-half pairing (j, j+rot/2) on un-permuted rows, which the reference proves equal to
// its adjacent-pair form on permuted rows, src/transformer/weights.rs:473-530, :626-671);
// tanh GELU src/tensor/ops.rs:169-178; soft cap src/tensor/ops.rs:98-103.
#include "common.cuh"

namespace glint {

// ---------------------------------------------------------------------------------------------
// x[t, :] = table[ids[t], :] * scale
// ---------------------------------------------------------------------------------------------
template <typename S>
__global__ void embed_scale_kernel(const S* __restrict__ table, const int* __restrict__ ids,
                                   float* __restrict__ x, int H, float scale, int vocab,
                                   int* __restrict__ status) {
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < 0 || id >= vocab) {  // never read outside the table; report and write zeros
    if (threadIdx.x == 0) atomicExch(status, 1);
    for (int i = threadIdx.x; i < H; i += blockDim.x) x[(size_t)t * H + i] = 0.f;
    return;
  }
  const S* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) x[(size_t)t * H + i] = to_float(row[i]) * scale;
}

// ---------------------------------------------------------------------------------------------
// out[r, :] = x[src(r), :] * rsqrt(mean(x^2) + eps) * (offset + w)
// ---------------------------------------------------------------------------------------------
template <typename S>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ row_index,
                               const float* __restrict__ w, S* __restrict__ out, int H, float eps,
                               float offset) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(row_index ? row_index[r] : r) * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = xr[i];
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rs = 1.0f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(size_t)r * H + i] = from_float<S>(xr[i] * rs * (offset + w[i]));
}

// ---------------------------------------------------------------------------------------------
// x[r, :] += norm_a(y[r, :])            (norm_a is the identity when w_a is null)
// out[r, :] = norm_b(x[r, :])           (skipped when out is null)
// ---------------------------------------------------------------------------------------------
template <typename S>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ y,
                                   const float* __restrict__ w_a, float eps_a, float offset_a,
                                   S* __restrict__ out, const float* __restrict__ w_b, float eps_b,
                                   float offset_b, int H) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  float* xr = x + (size_t)r * H;
  const float* yr = y + (size_t)r * H;
  float rs_a = 1.f;
  if (w_a) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = yr[i];
      ss += v * v;
    }
    ss = block_sum(ss, scratch);
    rs_a = 1.0f / sqrtf(ss / (float)H + eps_a);
  }
  float ss_x = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float add = w_a ? yr[i] * rs_a * (offset_a + w_a[i]) : yr[i];
    const float v = xr[i] + add;
    xr[i] = v;
    ss_x += v * v;
  }
  if (!out) return;
  ss_x = block_sum(ss_x, scratch);
  const float rs_b = 1.0f / sqrtf(ss_x / (float)H + eps_b);
  // each thread re-reads only the elements it wrote itself
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(size_t)r * H + i] = from_float<S>(w_b ? xr[i] * rs_b * (offset_b + w_b[i]) : xr[i]);
}

// ---------------------------------------------------------------------------------------------
// Rotary encoding of q and k, and the write of k and v into the request's pages.
//
// qkv: [T, (nh + 2 nkv) * hd] float (q heads, then k heads, then v heads).
// q_out: [T, nh * hd].  Pools: [page][nkv][page_size][hd].  block_table: [slots, max_pages].
// Pair (j, j + rot/2) of a head rotates by (pos / factor) * inv_freq[j]; dims >= rot copy.
// ---------------------------------------------------------------------------------------------
template <typename S>
__global__ void rope_kv_write_kernel(const float* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ token_slot,
                                     const int* __restrict__ block_table, int max_pages,
                                     const float* __restrict__ inv_freq, float factor, int rot,
                                     S* __restrict__ q_out, S* __restrict__ k_pool,
                                     S* __restrict__ v_pool, int nh, int nkv, int hd, int page_size,
                                     int num_pages, int* __restrict__ status) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const float ps = (float)pos / factor;
  const int half = rot >> 1;
  const float* row = qkv + (size_t)t * (nh + 2 * nkv) * hd;
  long long page_base = -1;
  if (k_pool) {
    const int slot = token_slot[t];
    const int page = block_table[(size_t)slot * max_pages + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicExch(status, 2);
    } else {
      page_base = ((long long)page * nkv) * page_size * hd + (long long)(pos % page_size) * hd;
    }
  }
  // rotated heads: q (nh) and k (nkv); work items are (head, j) with j < hd/2 ... handled per pair
  const int pairs_per_head = hd >> 1;  // includes un-rotated dims, taken two at a time
  const int n_rot_heads = nh + nkv;
  for (int w = threadIdx.x; w < n_rot_heads * pairs_per_head; w += blockDim.x) {
    const int head = w / pairs_per_head;
    const int j = w % pairs_per_head;
    const float* src = row + (size_t)head * hd;
    float a, b;
    int ia, ib;
    if (j < half) {
      ia = j;
      ib = j + half;
      float s, c;
      sincosf(ps * inv_freq[j], &s, &c);
      const float x0 = src[ia], x1 = src[ib];
      a = x0 * c - x1 * s;
      b = x0 * s + x1 * c;
    } else {  // dims past the rotary part, copied: (rot + 2(j-half), +1)
      ia = rot + 2 * (j - half);
      ib = ia + 1;
      a = src[ia];
      b = src[ib];
    }
    if (head < nh) {
      S* dst = q_out + (size_t)t * nh * hd + (size_t)head * hd;
      dst[ia] = from_float<S>(a);
      dst[ib] = from_float<S>(b);
    } else if (page_base >= 0) {
      S* dst = k_pool + page_base + (long long)(head - nh) * page_size * hd;
      dst[ia] = from_float<S>(a);
      dst[ib] = from_float<S>(b);
    }
  }
  if (page_base >= 0) {
    const float* vsrc = row + (size_t)(nh + nkv) * hd;
    for (int w = threadIdx.x; w < nkv * hd; w += blockDim.x) {
      const int head = w / hd, d = w % hd;
      v_pool[page_base + (long long)head * page_size * hd + d] = from_float<S>(vsrc[w]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// out[t, i] = act(gu[t, i]) * gu[t, I + i]
// ---------------------------------------------------------------------------------------------
template <typename S>
__global__ void gated_act_kernel(const float* __restrict__ gu, S* __restrict__ out, long long total,
                                 int I, int act) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / I;
  const int i = (int)(idx % I);
  const float g = gu[t * 2 * I + i];
  const float u = gu[t * 2 * I + I + i];
  const float a = act == 0 ? gelu_tanh(g) : g * (1.0f / (1.0f + expf(-g)));
  out[idx] = from_float<S>(a * u);
}

__global__ void softcap_kernel(float* __restrict__ x, long long n, float cap) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < n) x[idx] = softcap(x[idx], cap);
}

}  // namespace glint

using namespace glint;

#define DISPATCH(dtype, ...)                                 \
  if ((dtype) == GLINT_DTYPE_F32) {                          \
    typedef float S;                                         \
    __VA_ARGS__;                                             \
  } else if ((dtype) == GLINT_DTYPE_BF16) {                  \
    typedef __nv_bfloat16 S;                                 \
    __VA_ARGS__;                                             \
  } else {                                                   \
    return GLINT_ERR_BAD_ARG;                                \
  }

GLINT_API int glint_embed_scale(const void* table, int dtype, const int* ids, float* x, int T, int H,
                                float scale, int vocab, int* status, cudaStream_t stream) {
  if (T <= 0) return GLINT_OK;
  DISPATCH(dtype, embed_scale_kernel<S><<<T, 256, 0, stream>>>((const S*)table, ids, x, H, scale, vocab, status));
  return (int)cudaGetLastError();
}

GLINT_API int glint_rmsnorm(const float* x, const int* row_index, const float* w, void* out, int dtype,
                            int rows, int H, float eps, float offset, cudaStream_t stream) {
  if (rows <= 0) return GLINT_OK;
  const int threads = H >= 1024 ? 256 : 128;
  DISPATCH(dtype, rmsnorm_kernel<S><<<rows, threads, 0, stream>>>(x, row_index, w, (S*)out, H, eps, offset));
  return (int)cudaGetLastError();
}

GLINT_API int glint_add_rmsnorm(float* x, const float* y, const float* w_a, float eps_a, float offset_a,
                                void* out, int dtype, const float* w_b, float eps_b, float offset_b,
                                int rows, int H, cudaStream_t stream) {
  if (rows <= 0) return GLINT_OK;
  const int threads = H >= 1024 ? 256 : 128;
  DISPATCH(dtype, add_rmsnorm_kernel<S><<<rows, threads, 0, stream>>>(x, y, w_a, eps_a, offset_a, (S*)out, w_b,
                                                                    eps_b, offset_b, H));
  return (int)cudaGetLastError();
}

GLINT_API int glint_rope_kv_write(const float* qkv, const int* positions, const int* token_slot,
                                  const int* block_table, int max_pages, const float* inv_freq,
                                  float factor, int rot, void* q_out, void* k_pool, void* v_pool,
                                  int dtype, int T, int nh, int nkv, int hd, int page_size,
                                  int num_pages, int* status, cudaStream_t stream) {
  if (T <= 0) return GLINT_OK;
  if (hd % 2 || rot % 2 || rot > hd || rot < 0 || factor <= 0.f) return GLINT_ERR_BAD_ARG;
  DISPATCH(dtype, rope_kv_write_kernel<S><<<T, 256, 0, stream>>>(
                      qkv, positions, token_slot, block_table, max_pages, inv_freq, factor, rot, (S*)q_out,
                      (S*)k_pool, (S*)v_pool, nh, nkv, hd, page_size, num_pages, status));
  return (int)cudaGetLastError();
}

GLINT_API int glint_gated_act(const float* gu, void* out, int dtype, int T, int I, int act,
                              cudaStream_t stream) {
  const long long total = (long long)T * I;
  if (total <= 0) return GLINT_OK;
  if (act != 0 && act != 1) return GLINT_ERR_BAD_ARG;
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  DISPATCH(dtype, gated_act_kernel<S><<<(unsigned)blocks, threads, 0, stream>>>(gu, (S*)out, total, I, act));
  return (int)cudaGetLastError();
}

GLINT_API int glint_softcap(float* x, long long n, float cap, cudaStream_t stream) {
  if (n <= 0 || !(cap > 0.f)) return GLINT_OK;
  const int threads = 256;
  softcap_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, stream>>>(x, n, cap);
  return (int)cudaGetLastError();
}

GLINT_API const char* glint_error_string(int code) {
  switch (code) {
    case GLINT_OK: return "ok";
    case GLINT_ERR_BAD_ARG: return "bad argument";
    case GLINT_ERR_UNSUPPORTED_SIZE: return "size not supported by this kernel";
    case GLINT_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
  }
}

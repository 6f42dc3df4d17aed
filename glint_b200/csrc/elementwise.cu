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
// Fast forms of the row kernels for widths that are a multiple of 4: a row is loaded once into
// registers as float4 (all loads in flight together), reduced, and written; nothing is re-read.
// ---------------------------------------------------------------------------------------------
constexpr int ROW_THREADS = 256;   // the most; a launch takes 256, 192 or 128, see row_threads()

template <typename S>
__device__ __forceinline__ void store4(S* dst, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<const uint32_t*>(&lo);
  v.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = v;
}

template <typename S, int ITERS>
__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_fast_kernel(const float* __restrict__ x, const int* __restrict__ row_index, const float* __restrict__ w,
                    S* __restrict__ out, int H, float eps, float offset) {
  __shared__ float scratch[33];
  pdl_wait_release();
  const int r = blockIdx.x;
  const int H4 = H >> 2;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(row_index ? row_index[r] : r) * H);
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4 xv[ITERS], wv[ITERS];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    xv[it] = i < H4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    wv[it] = i < H4 ? w4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it)
    ss += xv[it].x * xv[it].x + xv[it].y * xv[it].y + xv[it].z * xv[it].z + xv[it].w * xv[it].w;
  ss = block_sum(ss, scratch);
  const float rs = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (i < H4)
      store4<S>(out + (size_t)r * H + 4 * i, xv[it].x * rs * (offset + wv[it].x), xv[it].y * rs * (offset + wv[it].y),
                xv[it].z * rs * (offset + wv[it].z), xv[it].w * rs * (offset + wv[it].w));
  }
}

template <typename S, int ITERS>
__global__ void __launch_bounds__(ROW_THREADS)
add_rmsnorm_fast_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w_a,
                        float eps_a, float offset_a, S* __restrict__ out, const float* __restrict__ w_b,
                        float eps_b, float offset_b, int H) {
  __shared__ float scratch[33];
  pdl_wait_release();
  const int r = blockIdx.x;
  const int H4 = H >> 2;
  float4* xr = reinterpret_cast<float4*>(x + (size_t)r * H);
  const float4* yr = reinterpret_cast<const float4*>(y + (size_t)r * H);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 xv[ITERS], yv[ITERS], wa[ITERS], wb[ITERS];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    const bool in = i < H4;
    xv[it] = in ? xr[i] : zero;
    yv[it] = in ? yr[i] : zero;
    wa[it] = (in && w_a) ? reinterpret_cast<const float4*>(w_a)[i] : zero;
    wb[it] = (in && w_b && out) ? reinterpret_cast<const float4*>(w_b)[i] : zero;
  }
  float rs_a = 1.f;
  if (w_a) {
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
      ss += yv[it].x * yv[it].x + yv[it].y * yv[it].y + yv[it].z * yv[it].z + yv[it].w * yv[it].w;
    ss = block_sum(ss, scratch);
    rs_a = 1.0f / sqrtf(ss / (float)H + eps_a);
  }
  float ss_x = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (w_a) {
      xv[it].x += yv[it].x * rs_a * (offset_a + wa[it].x);
      xv[it].y += yv[it].y * rs_a * (offset_a + wa[it].y);
      xv[it].z += yv[it].z * rs_a * (offset_a + wa[it].z);
      xv[it].w += yv[it].w * rs_a * (offset_a + wa[it].w);
    } else {
      xv[it].x += yv[it].x;
      xv[it].y += yv[it].y;
      xv[it].z += yv[it].z;
      xv[it].w += yv[it].w;
    }
    if (i < H4) xr[i] = xv[it];
    ss_x += xv[it].x * xv[it].x + xv[it].y * xv[it].y + xv[it].z * xv[it].z + xv[it].w * xv[it].w;
  }
  if (!out) return;
  ss_x = block_sum(ss_x, scratch);
  const float rs_b = w_b ? 1.0f / sqrtf(ss_x / (float)H + eps_b) : 1.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * blockDim.x;
    if (i >= H4) continue;
    if (w_b)
      store4<S>(out + (size_t)r * H + 4 * i, xv[it].x * rs_b * (offset_b + wb[it].x),
                xv[it].y * rs_b * (offset_b + wb[it].y), xv[it].z * rs_b * (offset_b + wb[it].z),
                xv[it].w * rs_b * (offset_b + wb[it].w));
    else
      store4<S>(out + (size_t)r * H + 4 * i, xv[it].x, xv[it].y, xv[it].z, xv[it].w);
  }
}

// (cos, sin) of every token's rotation angles, [token][hd / 2]: the same expression as in the
// kernels that compute them in place, once per step for the epilogue of the q/k/v product.
__global__ void __launch_bounds__(128)
rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, float factor,
                  float2* __restrict__ out, int half) {
  pdl_wait_release();
  const int t = blockIdx.x;
  const float ps = (float)positions[t] / factor;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float s, c;
    sincosf(ps * inv_freq[j], &s, &c);
    out[(size_t)t * half + j] = make_float2(c, s);
  }
}

// Rotary encoding, fast form: the sines and cosines of the token's position are computed once
// per block into shared memory, then every head reads them.  Same arithmetic as the plain form.
template <typename S>
__global__ void __launch_bounds__(256)
rope_kv_write_fast_kernel(const float* __restrict__ qkv, const int* __restrict__ positions,
                          const int* __restrict__ token_slot, const int* __restrict__ block_table, int max_pages,
                          const float* __restrict__ inv_freq, float factor, S* __restrict__ q_out,
                          S* __restrict__ k_pool, S* __restrict__ v_pool, int nh, int nkv, int hd, int page_size,
                          int num_pages, int* __restrict__ status) {
  extern __shared__ float trig[];   // cos[half], sin[half]
  pdl_wait_release();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = hd >> 1;
  const float ps = (float)pos / factor;
  const float* row = qkv + (size_t)t * (nh + 2 * nkv) * hd;
  const int half4 = half >> 2;   // items: four adjacent j of one head (hd is a multiple of 8 here)
  const int n_items = (nh + nkv) * half4;
  // The first items' operands are requested before the sines and cosines are computed (accurate
  // sincosf of a large angle is a long sequence): the memory latency passes meanwhile.  An item is
  // read as two float4 and written as two groups of four values (two-byte stores are slow).
  constexpr int HELD = 2;
  float4 lo[HELD], hi[HELD];
#pragma unroll
  for (int u = 0; u < HELD; ++u) {
    const int w = threadIdx.x + u * blockDim.x;
    if (w < n_items) {
      const float* src = row + (size_t)(w / half4) * hd + (w % half4) * 4;
      lo[u] = *reinterpret_cast<const float4*>(src);
      hi[u] = *reinterpret_cast<const float4*>(src + half);
    }
  }
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float s, c;
    sincosf(ps * inv_freq[j], &s, &c);
    trig[j] = c;
    trig[half + j] = s;
  }
  long long page_base = -1;
  if (k_pool) {
    const int page = block_table[(size_t)token_slot[t] * max_pages + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicExch(status, 2);
    } else {
      page_base = ((long long)page * nkv) * page_size * hd + (long long)(pos % page_size) * hd;
    }
  }
  __syncthreads();
  auto rotate = [&](int w, float4 l, float4 h) {
    const int head = w / half4, j = (w % half4) * 4;
    const float4 c = *reinterpret_cast<const float4*>(trig + j), sn = *reinterpret_cast<const float4*>(trig + half + j);
    S* dst = nullptr;
    if (head < nh) dst = q_out + (size_t)t * nh * hd + (size_t)head * hd;
    else if (page_base >= 0) dst = k_pool + page_base + (long long)(head - nh) * page_size * hd;
    if (dst) {
      store4<S>(dst + j, l.x * c.x - h.x * sn.x, l.y * c.y - h.y * sn.y, l.z * c.z - h.z * sn.z, l.w * c.w - h.w * sn.w);
      store4<S>(dst + j + half, l.x * sn.x + h.x * c.x, l.y * sn.y + h.y * c.y, l.z * sn.z + h.z * c.z,
                l.w * sn.w + h.w * c.w);
    }
  };
#pragma unroll
  for (int u = 0; u < HELD; ++u) {
    const int w = threadIdx.x + u * blockDim.x;
    if (w < n_items) rotate(w, lo[u], hi[u]);
  }
  for (int w = threadIdx.x + HELD * blockDim.x; w < n_items; w += blockDim.x) {
    const float* src = row + (size_t)(w / half4) * hd + (w % half4) * 4;
    rotate(w, *reinterpret_cast<const float4*>(src), *reinterpret_cast<const float4*>(src + half));
  }
  if (page_base >= 0) {
    const float* vsrc = row + (size_t)(nh + nkv) * hd;
    for (int w = threadIdx.x; w < (nkv * hd) >> 2; w += blockDim.x) {
      const int head = (w * 4) / hd, d = (w * 4) % hd;
      const float4 v = *reinterpret_cast<const float4*>(vsrc + (size_t)w * 4);
      store4<S>(v_pool + page_base + (long long)head * page_size * hd + d, v.x, v.y, v.z, v.w);
    }
  }
}

// x[t, :] = table[ids[t], :] * scale, 8 elements at a time (bfloat16 table, width a multiple of 8)
__global__ void embed_scale_fast_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids,
                                        float* __restrict__ x, int H, float scale, int vocab,
                                        int* __restrict__ status) {
  pdl_wait_release();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) atomicExch(status, 1);
  const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)(bad ? 0 : id) * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) {
    const uint4 raw = row[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float4 a, b;
    const float2 p0 = __bfloat1622float2(h[0]), p1 = __bfloat1622float2(h[1]);
    const float2 p2 = __bfloat1622float2(h[2]), p3 = __bfloat1622float2(h[3]);
    const float m = bad ? 0.f : scale;
    a = make_float4(p0.x * m, p0.y * m, p1.x * m, p1.y * m);
    b = make_float4(p2.x * m, p2.y * m, p3.x * m, p3.y * m);
    float4* dst = reinterpret_cast<float4*>(x + (size_t)t * H + 8 * i);
    dst[0] = a;
    dst[1] = b;
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

// ids[dst_rows[i]] = src[src_idx[i]]: tokens sampled by the previous step, which never left the device
__global__ void place_tokens_kernel(int* __restrict__ ids, const int* __restrict__ dst_rows,
                                    const int* __restrict__ src, const int* __restrict__ src_idx, int n) {
  pdl_wait_release();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) ids[dst_rows[i]] = src[src_idx[i]];
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

// Number of float4 loads per thread the fast row kernels need, or 0 when the row does not
// qualify (width not a multiple of 4, too wide, or a pointer not 16-byte aligned).
// Threads of a row block: of 256, 192 and 128 the count that leaves the fewest idle lanes in the
// last pass over the row (a width of 2304 is three passes of 192 float4 exactly, against 2.25 of 256).
static int row_threads(int H) {
  const int H4 = H / 4;
  int best = ROW_THREADS, best_waste = 1 << 30;
  for (int t = ROW_THREADS; t >= 128; t -= 64) {
    const int iters = (H4 + t - 1) / t;
    const int waste = iters * t - H4;
    if (iters <= 8 && waste < best_waste) {
      best = t;
      best_waste = waste;
    }
  }
  return best;
}

static int fast_iters(int H, const void* a, const void* b, const void* c, const void* d) {
  if (H % 4 || H <= 0) return 0;
  if ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)c) | ((uintptr_t)d)) & 15) return 0;
  const int threads = row_threads(H);
  const int iters = (H / 4 + threads - 1) / threads;
  return iters <= 8 ? iters : 0;
}

GLINT_API int glint_embed_scale(const void* table, int dtype, const int* ids, float* x, int T, int H,
                                float scale, int vocab, int* status, cudaStream_t stream) {
  if (T <= 0) return GLINT_OK;
  if (dtype == GLINT_DTYPE_BF16 && H % 8 == 0 && ((uintptr_t)table & 15) == 0 && ((uintptr_t)x & 15) == 0) {
    return (int)launch_kernel(embed_scale_fast_kernel, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16*)table, ids, x, H, scale, vocab, status);
  }
  DISPATCH(dtype, embed_scale_kernel<S><<<T, 256, 0, stream>>>((const S*)table, ids, x, H, scale, vocab, status));
  return (int)cudaGetLastError();
}

GLINT_API int glint_rmsnorm(const float* x, const int* row_index, const float* w, void* out, int dtype,
                            int rows, int H, float eps, float offset, cudaStream_t stream) {
  if (rows <= 0) return GLINT_OK;
  const int iters = fast_iters(H, x, w, out, nullptr);
  int rc = 0;
#define RMS_FAST(N) DISPATCH(dtype, rc = (int)launch_kernel(rmsnorm_fast_kernel<S, N>, dim3(rows), dim3(row_threads(H)), 0, stream, x, row_index, w, (S*)out, H, eps, offset))
  if (iters == 1) { RMS_FAST(1); }
  else if (iters == 2) { RMS_FAST(2); }
  else if (iters > 0 && iters <= 4) { RMS_FAST(4); }
  else if (iters > 0 && iters <= 8) { RMS_FAST(8); }
  else {
    const int threads = H >= 1024 ? 256 : 128;
    DISPATCH(dtype, rmsnorm_kernel<S><<<rows, threads, 0, stream>>>(x, row_index, w, (S*)out, H, eps, offset));
  }
#undef RMS_FAST
  return rc ? rc : (int)cudaGetLastError();
}

GLINT_API int glint_add_rmsnorm(float* x, const float* y, const float* w_a, float eps_a, float offset_a,
                                void* out, int dtype, const float* w_b, float eps_b, float offset_b,
                                int rows, int H, cudaStream_t stream) {
  if (rows <= 0) return GLINT_OK;
  int iters = fast_iters(H, x, y, out, w_a);
  if (w_b && ((uintptr_t)w_b & 15)) iters = 0;
  int rc = 0;
#define ADD_FAST(N) DISPATCH(dtype, rc = (int)launch_kernel(add_rmsnorm_fast_kernel<S, N>, dim3(rows), dim3(row_threads(H)), 0, stream, x, y, w_a, eps_a, offset_a, (S*)out, w_b, eps_b, offset_b, H))
  if (iters == 1) { ADD_FAST(1); }
  else if (iters == 2) { ADD_FAST(2); }
  else if (iters <= 4 && iters > 0) { ADD_FAST(4); }
  else if (iters <= 8 && iters > 0) { ADD_FAST(8); }
  else {
    const int threads = H >= 1024 ? 256 : 128;
    DISPATCH(dtype, add_rmsnorm_kernel<S><<<rows, threads, 0, stream>>>(x, y, w_a, eps_a, offset_a, (S*)out, w_b,
                                                                      eps_b, offset_b, H));
  }
#undef ADD_FAST
  return rc ? rc : (int)cudaGetLastError();
}

GLINT_API int glint_rope_table(const int* positions, const float* inv_freq, float factor, float* out, int T,
                               int half, cudaStream_t stream) {
  if (T <= 0 || half <= 0) return GLINT_OK;
  if (factor <= 0.f) return GLINT_ERR_BAD_ARG;
  const int rc = (int)launch_kernel(rope_table_kernel, dim3(T), dim3(half < 128 ? 64 : 128), 0, stream, positions,
                                    inv_freq, factor, reinterpret_cast<float2*>(out), half);
  return rc ? rc : (int)cudaGetLastError();
}

GLINT_API int glint_rope_kv_write(const float* qkv, const int* positions, const int* token_slot,
                                  const int* block_table, int max_pages, const float* inv_freq,
                                  float factor, int rot, void* q_out, void* k_pool, void* v_pool,
                                  int dtype, int T, int nh, int nkv, int hd, int page_size,
                                  int num_pages, int* status, cudaStream_t stream) {
  if (T <= 0) return GLINT_OK;
  if (hd % 2 || rot % 2 || rot > hd || rot < 0 || factor <= 0.f) return GLINT_ERR_BAD_ARG;
  if (rot == hd && hd % 8 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)q_out & 15) == 0 &&
      ((uintptr_t)k_pool & 15) == 0 && ((uintptr_t)v_pool & 15) == 0) {
    int rc = 0;
    DISPATCH(dtype, rc = (int)launch_kernel(rope_kv_write_fast_kernel<S>, dim3(T), dim3(256), hd * sizeof(float), stream,
                                            qkv, positions, token_slot, block_table, max_pages, inv_freq, factor,
                                            (S*)q_out, (S*)k_pool, (S*)v_pool, nh, nkv, hd, page_size, num_pages,
                                            status));
    return rc ? rc : (int)cudaGetLastError();
  }
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

GLINT_API int glint_place_tokens(int* ids, const int* dst_rows, const int* src, const int* src_idx, int n,
                                 cudaStream_t stream) {
  if (n <= 0) return GLINT_OK;
  place_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(ids, dst_rows, src, src_idx, n);
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

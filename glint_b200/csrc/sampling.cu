// Token choice on the device: argmax, and the reference's sampling pipeline
// penalty -> temperature -> top-k -> min-p -> softmax -> top-p -> draw
// (src/sampling/sampler.rs:179-235; stages :254-388).  One block per logits row.
//
// Differences from the reference's sequential code, all confined to exact ties or to sums
// that land within rounding of a threshold: top-k and top-p keep every element equal to the
// threshold value (the reference's unstable partial sort keeps an arbitrary subset), and sums
// are block reductions rather than index-order running sums.  The draw walks the cumulative
// distribution in index order as the reference does (:377-388).
#include "common.cuh"

namespace glint {

constexpr int SAMPLE_THREADS = 1024;

struct ArgBest {
  float v;
  int i;
};

// Later index wins among equal values: the reference's max_by keeps the last maximum
// (src/sampling/sampler.rs:245-252).
__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
  if (b.v > a.v || (b.v == a.v && b.i > a.i)) return b;
  return a;
}

__device__ __forceinline__ ArgBest block_argmax(ArgBest best, ArgBest* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest other;
    other.v = __shfl_xor_sync(0xffffffffu, best.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, best.i, o);
    best = better(best, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = best;
  __syncthreads();
  if (warp == 0) {
    const int nwarps = (blockDim.x + 31) >> 5;
    ArgBest b = lane < nwarps ? scratch[lane] : ArgBest{-INFINITY, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgBest other;
      other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
      other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
      b = better(b, other);
    }
    if (lane == 0) scratch[32] = b;
  }
  __syncthreads();
  return scratch[32];
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, long long row_stride, int V, int* __restrict__ out) {
  __shared__ ArgBest scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const float* row = logits + (size_t)blockIdx.x * row_stride;
  ArgBest best{-INFINITY, -1};
  if ((V & 3) == 0 && ((uintptr_t)row & 15) == 0) {
    // four float4 loads in flight per thread; indices still visited in increasing order per thread
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int V4 = V >> 2;
    for (int i0 = threadIdx.x; i0 < V4; i0 += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        v[u] = i < V4 ? row4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < V4) {
          best = better(best, ArgBest{v[u].x, 4 * i});
          best = better(best, ArgBest{v[u].y, 4 * i + 1});
          best = better(best, ArgBest{v[u].z, 4 * i + 2});
          best = better(best, ArgBest{v[u].w, 4 * i + 3});
        }
      }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) best = better(best, ArgBest{row[i], i});
  }
  best = block_argmax(best, scratch);
  if (threadIdx.x == 0) out[blockIdx.x] = best.i < 0 ? 0 : best.i;
}

__device__ __forceinline__ unsigned ordered_key(float v);

// The same over a wide row with several blocks: block (row, chunk) finds the best of its chunk,
// the chunks meet in one 64-bit atomic maximum per row (value key above, index below, so that among
// equal values the later index wins as in `better`), and the block that arrives last at the row's
// counter writes the index and leaves key and counter zero for the next launch.  `keys` and
// `counters` hold one zeroed entry per row.
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_wide_kernel(const float* __restrict__ logits, long long row_stride, int V, int chunk,
                   unsigned long long* __restrict__ keys, int* __restrict__ counters, int* __restrict__ out) {
  __shared__ ArgBest scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  const int begin = blockIdx.y * chunk, end = min(V, begin + chunk);     // chunk is a multiple of 4
  ArgBest best{-INFINITY, -1};
  if (((uintptr_t)(row + begin) & 15) == 0) {
    const int n4 = (end - begin) >> 2;
    const float4* row4 = reinterpret_cast<const float4*>(row + begin);
    for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        v[u] = i < n4 ? row4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < n4) {
          best = better(best, ArgBest{v[u].x, begin + 4 * i});
          best = better(best, ArgBest{v[u].y, begin + 4 * i + 1});
          best = better(best, ArgBest{v[u].z, begin + 4 * i + 2});
          best = better(best, ArgBest{v[u].w, begin + 4 * i + 3});
        }
      }
    }
    for (int i = begin + (n4 << 2) + threadIdx.x; i < end; i += blockDim.x) best = better(best, ArgBest{row[i], i});
  } else {
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) best = better(best, ArgBest{row[i], i});
  }
  best = block_argmax(best, scratch);
  if (threadIdx.x == 0) {
    if (best.i >= 0)   // -0 and +0 are equal to `better`: give them one key
      atomicMax(&keys[r], ((unsigned long long)ordered_key(best.v + 0.0f) << 32) | (unsigned)best.i);
    __threadfence();
    if (atomicAdd(&counters[r], 1) == (int)gridDim.y - 1) {
      __threadfence();
      const unsigned long long k = atomicExch(&keys[r], 0ull);
      out[r] = k ? (int)(unsigned)(k & 0xffffffffull) : 0;
      counters[r] = 0;
    }
  }
}

// work[r, :] = logits[r, :]; then every (token, count) pair of row r divides a positive logit by
// the penalty `count` times, or multiplies a non-positive one (src/sampling/sampler.rs:262-273
// loops over every past occurrence).
__global__ void penalty_kernel(const float* __restrict__ logits, long long row_stride, int V,
                               float* __restrict__ work, const int* __restrict__ pen_offsets,
                               const int* __restrict__ pen_tokens, const int* __restrict__ pen_counts,
                               const float* __restrict__ penalty) {
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  float* w = work + (size_t)r * V;
  for (int i = threadIdx.x; i < V; i += blockDim.x) w[i] = row[i];
  __syncthreads();
  const float pen = penalty[r];
  for (int e = pen_offsets[r] + threadIdx.x; e < pen_offsets[r + 1]; e += blockDim.x) {
    const int tok = pen_tokens[e];
    if (tok < 0 || tok >= V) continue;
    float v = w[tok];
    for (int c = 0; c < pen_counts[e]; ++c) v = v > 0.f ? v / pen : v * pen;
    w[tok] = v;
  }
}

__device__ __forceinline__ unsigned ordered_key(float v) {
  const unsigned u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Finds the key K such that the total weight of elements with key > K is < target and with
// key >= K is >= target, elements taken from the largest key down.  With weight 1 this is the
// target-th largest element; with weight p_i it is the top-p cutoff.
template <bool BY_PROB>
__device__ unsigned radix_threshold(const float* __restrict__ vals, int V, float target,
                                    float* hist /*256*/, unsigned* sh_prefix, float* sh_target) {
  unsigned prefix = 0, mask = 0;
  float remaining = target;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0.f;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = vals[i];
      const unsigned key = ordered_key(v);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], BY_PROB ? v : 1.0f);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float cum = 0.f;
      int bin = 255;
      for (; bin > 0; --bin) {
        if (cum + hist[bin] >= remaining) break;
        cum += hist[bin];
      }
      *sh_prefix = prefix | ((unsigned)bin << shift);
      *sh_target = remaining - cum;
    }
    __syncthreads();
    prefix = *sh_prefix;
    remaining = *sh_target;
    mask |= 255u << shift;
    __syncthreads();
  }
  return prefix;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ src, long long src_stride, float* __restrict__ work, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ uniform, int* __restrict__ out) {
  __shared__ float red[33];
  __shared__ float hist[256];
  __shared__ unsigned sh_prefix;
  __shared__ float sh_target;
  __shared__ float chunk_sum[SAMPLE_THREADS];
  __shared__ int sh_pick;
  const int r = blockIdx.x;
  const float* in = src + (size_t)r * src_stride;
  float* x = work + (size_t)r * V;
  const float temp = temperature[r];
  const float inv_temp = 1.0f / temp;

  // temperature (skipped at exactly 1, as the reference does) and the row maximum
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = temp != 1.0f ? in[i] * inv_temp : in[i];
    x[i] = v;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : -INFINITY;
    t = warp_max(t);
    if (threadIdx.x == 0) red[32] = t;
  }
  __syncthreads();
  mx = red[32];
  __syncthreads();

  const int k = top_k[r];
  if (k > 0 && k < V) {
    const unsigned thr = radix_threshold<false>(x, V, (float)k, hist, &sh_prefix, &sh_target);
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (ordered_key(x[i]) < thr) x[i] = -INFINITY;
    __syncthreads();
  }
  const float mp = min_p[r];
  if (mp > 0.f) {
    const float thr = mx + logf(mp);
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (x[i] < thr) x[i] = -INFINITY;
    __syncthreads();
  }
  // softmax
  float sum = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float e = expf(x[i] - mx);
    x[i] = e;
    sum += e;
  }
  sum = block_sum(sum, red);
  if (!(sum > 0.f)) {  // every logit was -inf: uniform (src/sampling/sampler.rs:331-333)
    for (int i = threadIdx.x; i < V; i += blockDim.x) x[i] = 1.0f / (float)V;
  } else {
    const float inv = 1.0f / sum;
    for (int i = threadIdx.x; i < V; i += blockDim.x) x[i] = x[i] / sum;
    (void)inv;
  }
  __syncthreads();
  const float tp = top_p[r];
  if (tp < 1.0f) {
    const unsigned thr = radix_threshold<true>(x, V, tp, hist, &sh_prefix, &sh_target);
    float kept = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      if (ordered_key(x[i]) < thr) x[i] = 0.f;
      kept += x[i];
    }
    kept = block_sum(kept, red);
    if (kept > 0.f)
      for (int i = threadIdx.x; i < V; i += blockDim.x) x[i] = x[i] / kept;
    __syncthreads();
  }
  // draw: first index whose running sum exceeds u, else the last index
  const float u = uniform[r];
  const int per = (V + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * per, hi = min(V, lo + per);
  float part = 0.f;
  for (int i = lo; i < hi; ++i) part += x[i];
  chunk_sum[threadIdx.x] = part;
  if (threadIdx.x == 0) sh_pick = V - 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float cum = 0.f;
    int owner = -1;
    for (int c = 0; c < (int)blockDim.x; ++c) {
      if (u < cum + chunk_sum[c]) {
        owner = c;
        break;
      }
      cum += chunk_sum[c];
    }
    if (owner >= 0) {
      const int l2 = owner * per, h2 = min(V, l2 + per);
      int pick = -1;
      for (int i = l2; i < h2; ++i) {
        cum += x[i];
        if (u < cum) {
          pick = i;
          break;
        }
      }
      // rounding between the chunk sum and the element walk: fall to the chunk's last kept index
      if (pick < 0) {
        for (int i = h2 - 1; i >= l2; --i)
          if (x[i] > 0.f) {
            pick = i;
            break;
          }
      }
      if (pick >= 0) sh_pick = pick;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = sh_pick;
}

}  // namespace glint

using namespace glint;

GLINT_API int glint_argmax(const float* logits, long long row_stride, int rows, int V, int* out,
                           cudaStream_t stream) {
  if (rows <= 0) return GLINT_OK;
  if (V <= 0) return GLINT_ERR_BAD_ARG;
  const cudaError_t e = launch_kernel(argmax_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, row_stride,
                                      V, out);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Rows of 64 K entries and more are shared by several blocks; `keys` (64-bit) and `counters` hold one
// zeroed entry per row and are left zeroed.  Without them, or for narrow rows, one block per row.
GLINT_API int glint_argmax_wide(const float* logits, long long row_stride, int rows, int V, int* out,
                                unsigned long long* keys, int* counters, cudaStream_t stream) {
  if (rows <= 0) return GLINT_OK;
  if (V <= 0) return GLINT_ERR_BAD_ARG;
  int chunks = V / 16384;
  if (chunks > 32) chunks = 32;
  if (!keys || !counters || chunks < 2 || rows > 65535) return glint_argmax(logits, row_stride, rows, V, out, stream);
  const int chunk = (((V + chunks - 1) / chunks) + 3) & ~3;
  chunks = (V + chunk - 1) / chunk;
  const cudaError_t e = launch_kernel(argmax_wide_kernel, dim3(rows, chunks), dim3(SAMPLE_THREADS), 0, stream, logits,
                                      row_stride, V, chunk, keys, counters, out);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

GLINT_API int glint_apply_penalty(const float* logits, long long row_stride, int rows, int V, float* work,
                                  const int* pen_offsets, const int* pen_tokens, const int* pen_counts,
                                  const float* penalty, cudaStream_t stream) {
  if (rows <= 0) return GLINT_OK;
  penalty_kernel<<<rows, 256, 0, stream>>>(logits, row_stride, V, work, pen_offsets, pen_tokens, pen_counts,
                                           penalty);
  return (int)cudaGetLastError();
}

// `work` is scratch of rows * V floats; `src` may be `work` itself (after glint_apply_penalty).
GLINT_API int glint_sample(const float* src, long long src_stride, float* work, int rows, int V,
                           const float* temperature, const int* top_k, const float* top_p,
                           const float* min_p, const float* uniform, int* out, cudaStream_t stream) {
  if (rows <= 0) return GLINT_OK;
  if (V <= 0) return GLINT_ERR_BAD_ARG;
  sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(src, src_stride, work, V, temperature, top_k, top_p,
                                                     min_p, uniform, out);
  return (int)cudaGetLastError();
}

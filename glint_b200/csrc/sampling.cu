// Token choice on the device: argmax, and the reference's sampling pipeline
// penalty -> temperature -> top-k -> min-p -> softmax -> top-p -> draw
// (src/sampling/sampler.rs:179-235; stages :254-388).  One block per logits row.
//
// Differences from the reference's sequential code, all confined to exact ties or to sums
// that land within rounding of a threshold: top-k and top-p keep every element equal to the
// threshold value (the reference's unstable partial sort keeps an arbitrary subset), and sums
// are block reductions rather than index-order running sums.  The draw walks the cumulative
// distribution in index order as the reference does (:377-388).  The histograms of probabilities
// behind top-p are added up with floating-point atomics, whose order is not fixed: a row whose top-p
// boundary lies within rounding of a bin's edge may, from run to run, keep one token more or less.
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
  pdl_wait_release();
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
constexpr int ARGMAX_WIDE_THREADS = 256;   // eight blocks to an SM: the launch of 64 rows is one wave

__global__ void __launch_bounds__(ARGMAX_WIDE_THREADS)
argmax_wide_kernel(const float* __restrict__ logits, long long row_stride, int V, int chunk,
                   unsigned long long* __restrict__ keys, int* __restrict__ counters, int* __restrict__ out) {
  __shared__ ArgBest scratch[33];
  pdl_wait_release();
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


// ---- wide rows: a thread-block cluster per row ------------------------------------------------------
//
// One block takes 250 elements per thread over a 256 K vocabulary and walks them a dozen times through
// global memory, with shared-memory atomics that mostly hit the same few histogram bins: milliseconds
// per step.  Here the SW_CLUSTER blocks of a cluster hold a row in their shared memory, an eighth each,
// and meet at cluster barriers: extrema, sums and histograms are exchanged through distributed shared
// memory and combined in block order by every block alike, so all of them reach the same decisions.
//
// A threshold (the k-th largest value, or the value at which the probabilities from the largest down
// reach top-p) is found in two levels.  Level 0 spreads the row over 256 bins that are monotone in the
// value: equal steps between the row's minimum and maximum for top-k, eight bins per octave below the
// largest probability for top-p; this finds the bin with the threshold, and few elements share a bin
// where it matters.  Then the radix selection over the 32 key bits runs among that bin's elements
// alone.  The repeat penalty is applied to the block's part of the row as it is loaded.

constexpr int SW_CLUSTER = 8;
constexpr int SW_WARPS = SAMPLE_THREADS / 32;
constexpr int SW_CAND = 1024;    // candidates of a cluster that are ranked directly

struct WideShared {
  float hist[2][256];       // this block's histogram of the current pass; the whole cluster reads it
  float slots[8];           // this block's share of a cluster-wide extremum or sum
  float total[256];         // the cluster's histogram
  float red[33];
  float warp_tot[SW_WARPS];
  float target;             // result of find_bin
  int bin;
  int cand_n;               // this block's elements in the bin with the threshold ...
  unsigned thr, thr_min;    // ... and the key found among all blocks' candidates
  float cand[SW_CAND];      // (the whole cluster reads cand_n and cand)
};

__device__ __forceinline__ uint32_t shared_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <bool MAX>
__device__ __forceinline__ float block_extremum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = MAX ? fmaxf(v, other) : fminf(v, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < SW_WARPS ? scratch[lane] : (MAX ? -INFINITY : INFINITY);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, t, o);
      t = MAX ? fmaxf(t, other) : fminf(t, other);
    }
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Every block publishes `v` (the same in all of its threads) in a slot; after a cluster barrier all
// get the blocks' values combined in block order.  KIND 0: sum, 1: maximum, 2: minimum.  One slot
// serves one exchange.
__device__ __forceinline__ void cluster_publish(WideShared* sh, int slot, float v) {
  if (threadIdx.x == 0) sh->slots[slot] = v;
}

template <int KIND>
__device__ __forceinline__ float cluster_gather(WideShared* sh, int slot, int blocks) {
  const uint32_t a = shared_addr(&sh->slots[slot]);
  float r = KIND == 0 ? 0.f : (KIND == 1 ? -INFINITY : INFINITY);
  for (int c = 0; c < blocks; ++c) {
    const float o = cluster_load(cluster_map(a, c));
    r = KIND == 0 ? r + o : (KIND == 1 ? fmaxf(r, o) : fminf(r, o));
  }
  return r;
}

template <int KIND>
__device__ __forceinline__ float cluster_combine(WideShared* sh, int slot, float v, int blocks) {
  cluster_publish(sh, slot, v);
  cluster_sync();
  return cluster_gather<KIND>(sh, slot, blocks);
}

// The block's histogram (per-warp copies in `whist` are added up first) goes to hist[buf]; after the
// barrier every block adds all blocks' histograms in block order into sh->total.
__device__ __forceinline__ void cluster_histogram(WideShared* sh, const float* whist, int buf, int blocks) {
  __syncthreads();
  if (threadIdx.x < 256) {
    float s = 0.f;
    for (int w = 0; w < SW_WARPS; ++w) s += whist[w * 256 + threadIdx.x];
    sh->hist[buf][threadIdx.x] = s;
  }
  cluster_sync();
  if (threadIdx.x < 256) {
    const uint32_t a = shared_addr(&sh->hist[buf][threadIdx.x]);
    float s = 0.f;
    for (int c = 0; c < blocks; ++c) s += cluster_load(cluster_map(a, c));
    sh->total[threadIdx.x] = s;
  }
  __syncthreads();
}

__device__ __forceinline__ void clear_histograms(float* whist) {
  for (int i = threadIdx.x; i < SW_WARPS * 256; i += blockDim.x) whist[i] = 0.f;
  __syncthreads();
}

// Walks the cluster's histogram from bin 0 up (DESC false) or from bin 255 down and stops at the first bin
// at which the running sum reaches `target`, or at the last bin of the walk: sh->bin is that bin and
// sh->target what is still wanted inside it.  Warp 0 does it, eight bins per lane (one thread walking
// 256 bins costs more than the rest of a pass).
template <bool DESC>
__device__ __forceinline__ void find_bin(WideShared* sh, float target) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float v[8], local = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = lane * 8 + j;
      v[j] = sh->total[DESC ? 255 - i : i];
      local += v[j];
    }
    float incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const float before = incl - local;
    const unsigned hit = __ballot_sync(0xffffffffu, before + local >= target);
    const int owner = hit ? __ffs(hit) - 1 : 31;
    if (lane == owner) {
      float cum = before;
      int j = 0;
      for (; j < 7; ++j) {
        if (cum + v[j] >= target) break;
        cum += v[j];
      }
      const int i = lane * 8 + j;
      sh->bin = DESC ? 255 - i : i;
      sh->target = target - cum;
    }
  }
  __syncthreads();
}

// The key K with: weight of the elements above K < target <= weight of the elements at or above K
// (weight 1, or the element itself for BY_PROB).  `top` is the row's maximum, `scale` 255.99 / (maximum
// - minimum) for level 0 of top-k (unused for BY_PROB).
template <bool BY_PROB>
__device__ unsigned wide_threshold(const float* data, int n, float target, float top, float scale, WideShared* sh,
                                   float* whist, int blocks, int& buf) {
  const int warp = threadIdx.x >> 5;
  const unsigned top_key = ordered_key(top);
  auto level0 = [&](float v) -> int {
    if (BY_PROB) {
      const unsigned d = (top_key - ordered_key(v)) >> 20;      // 8 bins per octave below the largest
      return d < 255u ? (int)d : 255;
    }
    return (int)fminf((top - v) * scale, 255.f);                // -inf lands in the last bin
  };
  // level 0: bin 0 holds the largest values
  clear_histograms(whist);
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const float v = data[e];
    if (BY_PROB && v == 0.f) continue;      // dropped by an earlier stage: no weight, and all in one bin
    atomicAdd(&whist[warp * 256 + level0(v)], BY_PROB ? v : 1.0f);
  }
  cluster_histogram(sh, whist, buf, blocks);
  buf ^= 1;
  find_bin<false>(sh, target);
  const int the_bin = sh->bin;
  float remaining = sh->target;
  // Few elements in that bin (the usual case): every block lists its own, in element order, all read
  // all lists and rank the candidates against each other: one barrier instead of four.
  {
    int mine = 0;
    for (int e = threadIdx.x; e < n; e += blockDim.x) mine += level0(data[e]) == the_bin ? 1 : 0;
    int incl = mine;
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    __syncthreads();
    if (lane == 31) sh->warp_tot[warp] = (float)incl;        // counts below 2^24 are exact
    __syncthreads();
    int at = incl - mine, local_total = 0;
    for (int w = 0; w < SW_WARPS; ++w) {
      const int t = (int)sh->warp_tot[w];
      if (w < warp) at += t;
      local_total += t;
    }
    if (local_total <= SW_CAND)
      for (int e = threadIdx.x; e < n; e += blockDim.x) {
        const float v = data[e];
        if (level0(v) == the_bin) sh->cand[at++] = v;
      }
    if (threadIdx.x == 0) {
      sh->cand_n = local_total;
      sh->thr = 0u;
      sh->thr_min = 0xffffffffu;
    }
    cluster_sync();
    int total = 0, first[SW_CLUSTER];
#pragma unroll
    for (int c = 0; c < SW_CLUSTER; ++c) {
      first[c] = total;
      if (c < blocks) {
        int n_c;
        asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(n_c) : "r"(cluster_map(shared_addr(&sh->cand_n), c)) : "memory");
        total += n_c;
      }
    }
    if (total <= SW_CAND) {                                   // the same answer in every block
      float* all = whist;
      for (int i = threadIdx.x; i < total; i += blockDim.x) {
        int c = 0, first_c = 0;
#pragma unroll
        for (int b = 1; b < SW_CLUSTER; ++b)
          if (b < blocks && i >= first[b]) {
            c = b;
            first_c = first[b];
          }
        all[i] = cluster_load(cluster_map(shared_addr(&sh->cand[i - first_c]), c));
      }
      __syncthreads();
      if ((int)threadIdx.x < total) {
        const unsigned key = ordered_key(all[threadIdx.x]);
        float above = 0.f, equal = 0.f;
        bool lowest = true;
        for (int j = 0; j < total; ++j) {
          const float v = all[j];
          const unsigned kj = ordered_key(v);
          const float w = BY_PROB ? v : 1.0f;
          if (kj > key) above += w;
          else if (kj == key) equal += w;
          else lowest = false;
        }
        if (above < remaining && above + equal >= remaining) atomicMax(&sh->thr, key);
        if (lowest) sh->thr_min = key;                        // equal keys write the same value
      }
      __syncthreads();
      // the target lies past the last candidate (sums that fall short by rounding): the lowest of them;
      // an empty bin: everything is kept
      unsigned thr = sh->thr;
      if (thr == 0u && total > 0) thr = sh->thr_min;
      __syncthreads();
      return thr;
    }
  }
  // the radix selection among the elements of that bin
  unsigned prefix = 0, mask = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    clear_histograms(whist);
    for (int e = threadIdx.x; e < n; e += blockDim.x) {
      const float v = data[e];
      const unsigned key = ordered_key(v);
      if ((key & mask) == prefix && level0(v) == the_bin)
        atomicAdd(&whist[warp * 256 + ((key >> shift) & 255u)], BY_PROB ? v : 1.0f);
    }
    cluster_histogram(sh, whist, buf, blocks);
    buf ^= 1;
    find_bin<true>(sh, remaining);
    prefix |= (unsigned)sh->bin << shift;
    remaining = sh->target;
    mask |= 255u << shift;
  }
  return prefix;
}

__global__ void __launch_bounds__(SAMPLE_THREADS, 1)
sample_wide_kernel(const float* __restrict__ src, long long src_stride, int V, int chunk,
                   const float* __restrict__ temperature, const int* __restrict__ top_k,
                   const float* __restrict__ top_p, const float* __restrict__ min_p,
                   const float* __restrict__ uniform, const int* __restrict__ pen_offsets,
                   const int* __restrict__ pen_tokens, const int* __restrict__ pen_counts,
                   const float* __restrict__ penalty, int* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t wide_raw[];
  WideShared* sh = reinterpret_cast<WideShared*>(wide_raw);
  float* whist = reinterpret_cast<float*>(wide_raw + ((sizeof(WideShared) + 15) & ~(size_t)15));
  float* data = whist + SW_WARPS * 256;
  const int r = blockIdx.x, rank = blockIdx.z, blocks = gridDim.z;
  const int begin = rank * chunk;
  const int n = max(0, min(V, begin + chunk) - begin);
  const float* in = src + (size_t)r * src_stride + begin;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int buf = 0;

  if ((((uintptr_t)in | (uintptr_t)data) & 15) == 0) {
    const int n4 = n >> 2;
    const float4* in4 = reinterpret_cast<const float4*>(in);
    float4* data4 = reinterpret_cast<float4*>(data);
    for (int e0 = threadIdx.x; e0 < n4; e0 += 4 * blockDim.x) {       // four loads in flight per thread
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = e0 + u * blockDim.x;
        if (e < n4) v[u] = in4[e];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = e0 + u * blockDim.x;
        if (e < n4) data4[e] = v[u];
      }
    }
    for (int e = (n4 << 2) + threadIdx.x; e < n; e += blockDim.x) data[e] = in[e];
  } else {
    for (int e = threadIdx.x; e < n; e += blockDim.x) data[e] = in[e];
  }
  __syncthreads();
  if (pen_offsets) {
    // every past token once, with its count (src/sampling/sampler.rs:262-273 loops over every occurrence)
    const float pen = penalty[r];
    for (int i = pen_offsets[r] + threadIdx.x; i < pen_offsets[r + 1]; i += blockDim.x) {
      const int tok = pen_tokens[i] - begin;
      if (tok < 0 || tok >= n) continue;
      float v = data[tok];
      for (int c = 0; c < pen_counts[i]; ++c) v = v > 0.f ? v / pen : v * pen;
      data[tok] = v;
    }
    __syncthreads();
  }
  // temperature (skipped at exactly 1, as the reference does), maximum and smallest finite value
  const float temp = temperature[r];
  const float inv_temp = 1.0f / temp;
  float mx = -INFINITY, mn = INFINITY;
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const float v = temp != 1.0f ? data[e] * inv_temp : data[e];
    data[e] = v;
    mx = fmaxf(mx, v);
    if (v > -INFINITY) mn = fminf(mn, v);
  }
  cluster_publish(sh, 0, block_extremum<true>(mx, sh->red));
  cluster_publish(sh, 1, block_extremum<false>(mn, sh->red));
  cluster_sync();
  mx = cluster_gather<1>(sh, 0, blocks);
  mn = cluster_gather<2>(sh, 1, blocks);

  const int k = top_k[r];
  if (k > 0 && k < V) {
    const float span = mx - mn;
    const float scale = span > 0.f && span < INFINITY ? 255.99f / span : 0.f;
    const unsigned thr = wide_threshold<false>(data, n, (float)k, mx, scale, sh, whist, blocks, buf);
    for (int e = threadIdx.x; e < n; e += blockDim.x)
      if (ordered_key(data[e]) < thr) data[e] = -INFINITY;
  }
  const float mp = min_p[r];
  if (mp > 0.f) {
    const float thr = mx + logf(mp);
    for (int e = threadIdx.x; e < n; e += blockDim.x)
      if (data[e] < thr) data[e] = -INFINITY;
  }
  // softmax
  float sum = 0.f;
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const float ex = expf(data[e] - mx);
    data[e] = ex;
    sum += ex;
  }
  sum = cluster_combine<0>(sh, 2, block_sum(sum, sh->red), blocks);
  if (!(sum > 0.f)) {  // every logit was -inf: uniform (src/sampling/sampler.rs:331-333)
    for (int e = threadIdx.x; e < n; e += blockDim.x) data[e] = 1.0f / (float)V;
  } else {
    for (int e = threadIdx.x; e < n; e += blockDim.x) data[e] = data[e] / sum;
  }
  __syncthreads();
  const float tp = top_p[r];
  if (tp < 1.0f) {
    const float pmax = sum > 0.f ? 1.0f / sum : 1.0f / (float)V;     // exp(0) / sum: the largest probability
    const unsigned thr = wide_threshold<true>(data, n, tp, pmax, 0.f, sh, whist, blocks, buf);
    float kept = 0.f;
    for (int e = threadIdx.x; e < n; e += blockDim.x) {
      if (ordered_key(data[e]) < thr) data[e] = 0.f;
      kept += data[e];
    }
    kept = cluster_combine<0>(sh, 3, block_sum(kept, sh->red), blocks);
    if (kept > 0.f)
      for (int e = threadIdx.x; e < n; e += blockDim.x) data[e] = data[e] / kept;
    __syncthreads();
  }
  // draw: the first index whose running sum exceeds u, else the last index.  A warp owns a run of
  // consecutive elements, a block its part of the row: sums per warp, per block, then the walk.
  const float u = uniform[r];
  const int wper = ((n + SW_WARPS - 1) / SW_WARPS + 31) & ~31;
  const int lo = min(n, warp * wper), hi = min(n, lo + wper);
  float part = 0.f;
  for (int e = lo + lane; e < hi; e += 32) part += data[e];
  part = warp_sum(part);
  __syncthreads();
  if (lane == 0) sh->warp_tot[warp] = part;
  __syncthreads();
  float mine = 0.f;
  for (int w = 0; w < SW_WARPS; ++w) mine += sh->warp_tot[w];
  if (threadIdx.x == 0) sh->slots[4] = mine;
  cluster_sync();
  float before = 0.f;
  int owner = -1;
  {
    const uint32_t a = shared_addr(&sh->slots[4]);
    float cum = 0.f;
    for (int c = 0; c < blocks; ++c) {
      const float s = cluster_load(cluster_map(a, c));
      if (owner < 0 && u < cum + s) {
        owner = c;
        before = cum;
      }
      cum += s;
    }
  }
  if (owner < 0) {
    if (rank == blocks - 1 && threadIdx.x == 0) out[r] = V - 1;
  } else if (owner == rank) {
    float cum = before;
    int owner_warp = -1;
    for (int w = 0; w < SW_WARPS; ++w) {
      if (u < cum + sh->warp_tot[w]) {
        owner_warp = w;
        break;
      }
      cum += sh->warp_tot[w];
    }
    // rounding between the block's sum and its warps' sums: the last warp that kept anything
    if (owner_warp < 0) {
      cum = before;
      for (int w = 0; w < SW_WARPS; ++w) {
        if (sh->warp_tot[w] > 0.f) owner_warp = w;
      }
      for (int w = 0; w < owner_warp; ++w) cum += sh->warp_tot[w];
    }
    if (warp == owner_warp) {
      int pick = -1, last_kept = -1;
      for (int e0 = lo; e0 < hi && pick < 0; e0 += 32) {
        const int e = e0 + lane;
        const float v = e < hi ? data[e] : 0.f;
        float incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, u < cum + incl && e < hi);
        const unsigned has = __ballot_sync(0xffffffffu, v > 0.f);
        if (has) last_kept = e0 + 31 - __clz(has);
        if (hit) pick = e0 + __ffs(hit) - 1;
        cum += __shfl_sync(0xffffffffu, incl, 31);
      }
      // rounding between the warp's sum and the walk: its last kept element
      if (pick < 0) pick = last_kept;
      if (lane == 0) out[r] = pick >= 0 ? begin + pick : V - 1;
    }
  }
  cluster_sync();   // nobody leaves while its shared memory may still be read
}

// ---------------------------------------------------------------------------------------------
// The per-request record of the sampler, one row of SAMPLER_RECORD 32-bit words per request slot:
//   0 temperature  1 top-p  2 min-p  3 repeat penalty (floats)   4 top-k   5 1 if the request is not greedy
//   6, 7 the low and high word of its xorshift64 generator's state
//   8 the position of its newest token + 1   9 how many tokens have been chosen for it
// Words 0 to 7 are written by the host when the request takes the slot; this kernel keeps 6 to 9 up to
// date on the device.  For each row of a step that is about to be sampled it copies the row's options into
// per-row arrays (the layout the sampling kernels read) and, for a row that is not greedy, advances the
// generator (s ^= s << 13; s ^= s >> 7; s ^= s << 17; uniform from the upper 24 bits:
// src/sampling/sampler.rs:35-70) and hands the draw over.  The reference keeps position and generator
// with the session (src/session/mod.rs:86, src/sampling/sampler.rs:35-37).
// row_opts: [7][stride] floats: temperature, uniform, top-p, min-p, penalty, not-greedy, top-k (int bits).
// ---------------------------------------------------------------------------------------------
constexpr int SAMPLER_RECORD = 10;

__global__ void sample_prepare_kernel(int* __restrict__ records, const int* __restrict__ row_slots,
                                      const int* __restrict__ positions, const int* __restrict__ logit_rows,
                                      int rows, int num_slots, float* __restrict__ row_opts, int stride) {
  pdl_wait_release();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int slot = row_slots[r];
  if (slot < 0 || slot >= num_slots) return;
  int* rec = records + (size_t)slot * SAMPLER_RECORD;
  const bool draws = rec[5] != 0;
  float uniform = 0.f;
  if (draws) {
    unsigned long long x = (unsigned long long)(unsigned)rec[6] | ((unsigned long long)(unsigned)rec[7] << 32);
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    rec[6] = (int)(unsigned)(x & 0xffffffffull);
    rec[7] = (int)(unsigned)(x >> 32);
    uniform = (float)(x >> 40) / 16777216.0f;
  }
  rec[8] = positions[logit_rows[r]] + 1;
  rec[9] += 1;
  row_opts[0 * stride + r] = draws ? __int_as_float(rec[0]) : 1.0f;
  row_opts[1 * stride + r] = uniform;
  row_opts[2 * stride + r] = __int_as_float(rec[1]);
  row_opts[3 * stride + r] = __int_as_float(rec[2]);
  row_opts[4 * stride + r] = __int_as_float(rec[3]);
  row_opts[5 * stride + r] = draws ? 1.0f : 0.0f;
  reinterpret_cast<int*>(row_opts)[6 * stride + r] = rec[4];
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

// Rows of 32 K entries and more are shared by several blocks; `keys` (64-bit) and `counters` hold one
// zeroed entry per row and are left zeroed.  Without them, or for narrow rows, one block per row.
GLINT_API int glint_argmax_wide(const float* logits, long long row_stride, int rows, int V, int* out,
                                unsigned long long* keys, int* counters, cudaStream_t stream) {
  if (rows <= 0) return GLINT_OK;
  if (V <= 0) return GLINT_ERR_BAD_ARG;
  if (!keys || !counters || V < 32768 || rows > 65535) return glint_argmax(logits, row_stride, rows, V, out, stream);
  // About four blocks of 256 threads for every SM, a chunk of at least 4096 entries each (one round of four
  // 16-byte loads per thread): blocks of 1024 threads with 17,000 entries each, three waves of them for 64 rows,
  // spent their time on their own start, reduction and atomics (64 rows of 256,000: 33 us for 65 MB).
  static int sms = 0;
  if (sms <= 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 128;
  }
  int chunks = (4 * sms + rows - 1) / rows;
  if (chunks > V / 4096) chunks = V / 4096;
  if (chunks > 64) chunks = 64;
  if (chunks < 2) chunks = 2;
  const int chunk = (((V + chunks - 1) / chunks) + 3) & ~3;
  chunks = (V + chunk - 1) / chunk;
  const cudaError_t e = launch_kernel(argmax_wide_kernel, dim3(rows, chunks), dim3(ARGMAX_WIDE_THREADS), 0, stream, logits,
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

// Rows this wide go to the cluster kernel: a row has to fit the cluster's shared memory.
static bool sample_wide_takes(int V) { return V >= 16384 && V <= SW_CLUSTER * 44000; }

// The whole pipeline for `rows` rows: penalty (pen_offsets null: none) -> temperature -> top-k -> min-p ->
// softmax -> top-p -> draw.  `work` is scratch of rows * V floats (used for narrow rows only).
// pen_offsets [rows + 1] delimits each row's (token, count) pairs; a token occurs once per row.
GLINT_API int glint_sample_rows(const float* logits, long long row_stride, float* work, int rows, int V,
                                const float* temperature, const int* top_k, const float* top_p, const float* min_p,
                                const float* uniform, const int* pen_offsets, const int* pen_tokens,
                                const int* pen_counts, const float* penalty, int* out, cudaStream_t stream) {
  if (rows <= 0) return GLINT_OK;
  if (V <= 0) return GLINT_ERR_BAD_ARG;
  if (pen_offsets && (!pen_tokens || !pen_counts || !penalty)) return GLINT_ERR_BAD_ARG;
  if (sample_wide_takes(V) && rows <= 65535) {
    const int chunk = (V + SW_CLUSTER - 1) / SW_CLUSTER;
    const size_t smem = ((sizeof(WideShared) + 15) & ~(size_t)15) + (size_t)(SW_WARPS * 256 + chunk) * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(sample_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = launch_kernel_cluster(sample_wide_kernel, dim3(rows, 1, SW_CLUSTER), dim3(SAMPLE_THREADS), smem, stream,
                              SW_CLUSTER, logits, row_stride, V, chunk, temperature, top_k, top_p, min_p, uniform,
                              pen_offsets, pen_tokens, pen_counts, penalty, out);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
  }
  const float* src = logits;
  long long stride = row_stride;
  if (pen_offsets) {
    penalty_kernel<<<rows, 256, 0, stream>>>(logits, row_stride, V, work, pen_offsets, pen_tokens, pen_counts, penalty);
    src = work;
    stride = V;
  }
  sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(src, stride, work, V, temperature, top_k, top_p, min_p, uniform,
                                                     out);
  return (int)cudaGetLastError();
}

GLINT_API int glint_sampler_record_words() { return SAMPLER_RECORD; }

// Before the rows of a step are sampled: options from the slots' records into per-row arrays, the
// generators of the rows that draw advanced by one, position and count brought up to date.
GLINT_API int glint_sample_prepare(int* records, const int* row_slots, const int* positions, const int* logit_rows,
                                   int rows, int num_slots, float* row_opts, int stride, cudaStream_t stream) {
  if (rows <= 0) return GLINT_OK;
  if (!records || !row_slots || !positions || !logit_rows || !row_opts || stride < rows) return GLINT_ERR_BAD_ARG;
  const cudaError_t e = launch_kernel(sample_prepare_kernel, dim3((rows + 127) / 128), dim3(128), 0, stream, records,
                                      row_slots, positions, logit_rows, rows, num_slots, row_opts, stride);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

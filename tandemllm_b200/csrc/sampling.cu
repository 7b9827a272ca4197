// Token choice on the device: argmax, and temperature / min_p / top-k / top-p sampling by the Gumbel-max
// trick with noise keyed by (seed, sequence position, token id).
//
// Order of the filters (engine/sample.py:172-199 of the reference): logits / temperature, then min_p
// (keep z >= max + log(min_p)), then top-k (keep the k largest), then top-p (sorted descending, keep a
// token while the mass ranked before it does not exceed top_p; the first is always kept), then a draw
// from the softmax of what is left. temperature 0 is the argmax whatever the filters say (sample.py:134-141).
// A draw is argmax(z + G) with G Gumbel noise (sample.py:311-322); the noise depends on the request's
// seed, the position and the token only, so a seeded request repeats whatever else is in the batch.
//
// Every filter is a threshold on z, found without sorting: the k-th largest value and the top-p cut are
// located by a 32-step search over the bits of an order-preserving integer image of the floats, each step
// one counting (or mass-summing) pass over the row. Ties at a threshold are all kept.
#include "common.cuh"

namespace tl {

__device__ __forceinline__ unsigned ordered_key(float x) {
  const unsigned u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
  return x ^ (x >> 31);
}

// uniform in (0, 1) with 23 bits, for (request key, token): (n + 0.5) / 2^23 is exact in 32-bit for every n < 2^23,
// so neither 0 nor 1 can come out
__device__ __forceinline__ float keyed_uniform(unsigned long long key, unsigned token) {
  const unsigned long long r = splitmix64(key ^ ((unsigned long long)(token + 1u) * 0xD1342543DE82EF95ULL));
  return ((float)(unsigned)(r >> 41) + 0.5f) * (1.f / 8388608.f);
}

struct Best {
  float v;
  int i;
};

__device__ __forceinline__ Best better(Best a, Best b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__device__ __forceinline__ Best block_best(Best x, Best* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  if (warp == 0) {
    Best t;
    t.v = -INFINITY;
    t.i = 0x7fffffff;
    if (lane < nwarps) t = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best y;
      y.v = __shfl_xor_sync(0xffffffffu, t.v, o);
      y.i = __shfl_xor_sync(0xffffffffu, t.i, o);
      t = better(t, y);
    }
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// This thread's best of a row it strides over: 16-byte loads, eight in flight, when the row allows
__device__ __forceinline__ Best row_best(const float* __restrict__ row, int V) {
  Best b;
  b.v = -INFINITY;
  b.i = 0x7fffffff;
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int n4 = V >> 2, stride = blockDim.x;
    constexpr int GROUP = 8;                     // loads issued together, then compared in index order
    for (int i0 = threadIdx.x; i0 < n4; i0 += GROUP * stride) {
      float4 x[GROUP];
#pragma unroll
      for (int g = 0; g < GROUP; ++g) {
        const int i = i0 + g * stride;
        x[g] = i < n4 ? row4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int g = 0; g < GROUP; ++g) {
        const int i = i0 + g * stride;
        const float v[4] = {x[g].x, x[g].y, x[g].z, x[g].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          Best c;
          c.v = v[j];
          c.i = 4 * i + j;
          if (i < n4 && c.v == c.v) b = better(b, c);
        }
      }
    }
  } else {
#pragma unroll 4
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      Best c;
      c.v = row[i];
      c.i = i;
      if (c.v == c.v) b = better(b, c);
    }
  }
  return b;
}

// one block per row; the lowest index wins a tie; NaN is never the maximum
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, long long ld, int V,
                                                      int* __restrict__ out) {
  __shared__ Best scratch[33];
  const float* row = logits + (long long)blockIdx.x * ld;
  Best b = row_best(row, V);
  b = block_best(b, scratch);
  if (threadIdx.x == 0) out[blockIdx.x] = b.i == 0x7fffffff ? 0 : b.i;
}

__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, long long ld, int V,
                                                      const float* __restrict__ temperature,
                                                      const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                      const float* __restrict__ min_p,
                                                      const unsigned long long* __restrict__ seed,
                                                      const int* __restrict__ position, int* __restrict__ out) {
  __shared__ Best best_scratch[33];
  __shared__ float red[33];
  const int n = blockIdx.x;
  const float* row = logits + (long long)n * ld;
  const float T = temperature[n];
  Best b;
  b.v = -INFINITY;
  b.i = 0x7fffffff;
  if (!(T > 0.f)) {
    b = row_best(row, V);
    b = block_best(b, best_scratch);
    if (threadIdx.x == 0) out[n] = b.i == 0x7fffffff ? 0 : b.i;
    return;
  }
  const float inv_t = 1.f / T;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float z = row[i] * inv_t;
    if (z == z) mx = fmaxf(mx, z);
  }
  mx = block_max(mx, red);
  float thr = -INFINITY;
  const float mp = min_p[n];
  if (mp > 0.f) thr = mx + logf(mp);
  const int k = top_k[n];
  if (k > 0 && k < V) {
    unsigned t = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = t | (1u << bit);
      int cnt = 0;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float z = row[i] * inv_t;
        cnt += (z == z) && ordered_key(z) >= cand;
      }
      const float total = block_sum((float)cnt, red);   // exact: V is far below 2^24
      if (total >= (float)k) t = cand;
    }
    // t is the key of the k-th largest value
    const unsigned u = (t & 0x80000000u) ? (t & 0x7fffffffu) : ~t;
    thr = fmaxf(thr, __uint_as_float(u));
  }
  const float p = top_p[n];
  if (p < 1.f) {
    float mass = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float z = row[i] * inv_t;
      if (z == z && z >= thr) mass += expf(z - mx);
    }
    const float Z = block_sum(mass, red);
    const float want = p * Z;
    const unsigned kthr = thr == -INFINITY ? 0u : ordered_key(thr);
    unsigned t = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = t | (1u << bit);
      const unsigned lo = cand > kthr ? cand : kthr;
      float h = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float z = row[i] * inv_t;
        if (z == z && ordered_key(z) >= lo) h += expf(z - mx);
      }
      h = block_sum(h, red);
      if (h > want) t = cand;     // the mass at or above cand still exceeds top_p: the cut is at or above cand
    }
    const unsigned u = (t & 0x80000000u) ? (t & 0x7fffffffu) : ~t;
    thr = fmaxf(thr, __uint_as_float(u));
  }
  const unsigned long long key =
      splitmix64(seed[n] * 0x9E3779B97F4A7C15ULL + (unsigned long long)(long long)position[n] + 1ULL);
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float z = row[i] * inv_t;
    if (!(z == z) || z < thr) continue;
    const float u = keyed_uniform(key, (unsigned)i);
    Best c;
    c.v = z - logf(-logf(u));
    c.i = i;
    b = better(b, c);
  }
  b = block_best(b, best_scratch);
  if (threadIdx.x == 0) out[n] = b.i == 0x7fffffff ? 0 : b.i;
}

// Penalties and added logits (engine/penalty.py of the reference), in place on the rows that ask for them, before the
// choice. A row first takes its `logit_bias` entries (penalty.py:189-204: added before everything else); then, where
// the row's request has seen a token (its count row: prompt and generated tokens, penalty.py:206-232), the logit is
// multiplied by the repetition penalty if negative and divided by it if not, loses the presence penalty once and the
// frequency penalty times the count (penalty.py:320-331). slot < 0: a row without penalties (it may still have a bias).
__global__ void penalize_kernel(float* __restrict__ logits, long long ld, int V, const int* __restrict__ counts,
                                long long counts_ld, int slots, const int* __restrict__ slot,
                                const float* __restrict__ repetition,
                                const float* __restrict__ presence, const float* __restrict__ frequency,
                                const int* __restrict__ bias_begin, const int* __restrict__ bias_token,
                                const float* __restrict__ bias_value) {
  const int r = blockIdx.x;
  float* row = logits + (long long)r * ld;
  if (bias_begin != nullptr) {
    const int b1 = bias_begin[r + 1];
    for (int i = bias_begin[r] + threadIdx.x; i < b1; i += blockDim.x) {
      const int t = bias_token[i];
      if (t >= 0 && t < V) row[t] += bias_value[i];      // a request's bias names a token once
    }
    __syncthreads();
  }
  const int s = slot[r];
  if (s < 0 || s >= slots) return;
  const int* seen = counts + (long long)s * counts_ld;
  const float rp = repetition[r], pr = presence[r], fq = frequency[r];
  for (int v = threadIdx.x; v < V; v += blockDim.x) {
    const int n = seen[v];
    if (n <= 0) continue;
    float x = row[v];
    if (rp != 1.f) x = x < 0.f ? x * rp : x / rp;
    if (pr != 0.f) x -= pr;
    if (fq != 0.f) x -= fq * (float)n;
    row[v] = x;
  }
}

// counts[slot, token] += 1 for every (slot, token) given; `slot` null: all go to `one_slot` (a request's history at
// its start). Tokens repeat within a history, so the additions are atomic; a negative slot or token is passed over.
__global__ void count_tokens_kernel(int* __restrict__ counts, long long ld, int slots, int V,
                                    const int* __restrict__ slot,
                                    int one_slot, const int* __restrict__ token, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int s = slot != nullptr ? slot[i] : one_slot, t = token[i];
  if (s < 0 || s >= slots || t < 0 || t >= V) return;
  atomicAdd(counts + (long long)s * ld + t, 1);
}

}  // namespace tl

using namespace tl;

extern "C" int tl_argmax(const float* logits, long long ld, int rows, int V, int* out, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(V > 0 && ld >= V, "argmax: vocabulary %d, row stride %lld", V, ld);
  argmax_kernel<<<rows, V >= 4096 ? 1024 : 256, 0, stream>>>(logits, ld, V, out);
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_sample(const float* logits, long long ld, int rows, int V, const float* temperature, const int* top_k,
                         const float* top_p, const float* min_p, const unsigned long long* seed, const int* position,
                         int* out, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(V > 0 && V < (1 << 24) && ld >= V, "sample: vocabulary %d, row stride %lld", V, ld);
  sample_kernel<<<rows, V >= 4096 ? 1024 : 256, 0, stream>>>(logits, ld, V, temperature, top_k, top_p, min_p, seed,
                                                             position, out);
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_penalize(float* logits, long long ld, int rows, int V, const int* counts, long long counts_ld,
                           int slots, const int* slot, const float* repetition, const float* presence,
                           const float* frequency, const int* bias_begin, const int* bias_token,
                           const float* bias_value, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(V > 0 && ld >= V, "penalize: vocabulary %d, row stride %lld", V, ld);
  TL_REQUIRE(slots == 0 || (counts != nullptr && counts_ld >= V), "penalize: %d count rows with stride %lld", slots,
             counts_ld);
  TL_REQUIRE((bias_begin == nullptr) == (bias_token == nullptr) && (bias_begin == nullptr) == (bias_value == nullptr),
             "penalize: the bias needs its offsets, tokens and values together (%d)", 0);
  penalize_kernel<<<rows, V >= 4096 ? 1024 : 256, 0, stream>>>(logits, ld, V, counts, counts_ld, slots, slot,
                                                               repetition, presence, frequency, bias_begin, bias_token,
                                                               bias_value);
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_count_tokens(int* counts, long long ld, int slots, int V, const int* slot, int one_slot,
                               const int* token, int n, cudaStream_t stream) {
  if (n == 0) return 0;
  TL_REQUIRE(V > 0 && ld >= V && slots > 0, "count tokens: vocabulary %d, row stride %lld", V, ld);
  TL_REQUIRE(slot != nullptr || (one_slot >= 0 && one_slot < slots), "count tokens: slot %d of %d", one_slot, slots);
  count_tokens_kernel<<<(n + 255) / 256, 256, 0, stream>>>(counts, ld, slots, V, slot, one_slot, token, n);
  TL_LAUNCH_CHECK();
  return 0;
}

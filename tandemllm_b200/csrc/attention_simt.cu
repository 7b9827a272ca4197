// Attention over the paged cache on the CUDA cores (every head size in steps of 16 up to 256, any
// number of heads and groups, 32-bit or bfloat16 storage with 32-bit arithmetic), and the kernel in
// front of it: per-head RMS norm of q and k, rotary position encoding, and the write of k and v
// into their pages.
//
//   q = rms_D(q_proj(n)) , k = rms_D(k_proj(n)) , v = v_proj(n)            engine/models/lfm2_moe/ref.py:158-160
//   x' = x cos + rotate_half(x) sin, angle = position * theta^(-2i/D)       ref.py:84, 111-120, 162-165
//   s = q k^T * scale over the visible keys, softmax in 32-bit, o = a v     ref.py:166-178
//   query head h reads KV head h / (Hq / Hk)                                 ref.py:173-174
//
// Cache layout per site: K and V are [pages, kv heads, page_size, head_dim]; the token at position p of a
// request lives in page table[request][p / page_size] at offset p % page_size. A row sees the keys at
// positions max(0, pos - window + 1) .. pos of its own request (window 0: all of them); the step's own
// keys are written before attention runs, so prompt portions, single decoded tokens and any mix of
// them are the same case. Keys are visited in chunks of 32 aligned to absolute positions with an
// online softmax, so the order of additions for a row depends on its position only.
#include "common.cuh"

namespace tl {

constexpr int MAX_HEAD_DIM = 256;

// grid (rows, groups of heads), 128 threads: a block takes `heads_per_block` consecutive heads of one fused qkv row (all of
// them when they fit QK_GROUP_FLOATS), brings them into shared memory with 16-byte loads that are all in flight at once,
// and its warps then take a head each in turn. The row's rotation angles are computed once a block.
constexpr int QK_GROUP_FLOATS = 8192;

// DS: the head size when it is 64 or 128 and the whole head is rotated (a lane then owns DS / 64 pairs (f, f + DS / 2), its
// weights and its angles for all heads, and the loops unroll), else 0 (any size, any rotary part).
template <typename T, int DS>
__global__ void __launch_bounds__(128) qk_prepare_kernel(
    const T* __restrict__ qkv, long long ld_qkv, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
    float eps, const float* __restrict__ inv_freq, int rotary_dim, const int* __restrict__ positions,
    const int* __restrict__ req_of_row, const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
    T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache, T* __restrict__ k_out,
    T* __restrict__ v_out, int Hq, int Hk, int D, int heads_per_block, int* __restrict__ status) {
  __shared__ __align__(16) float vec[QK_GROUP_FLOATS];
  __shared__ float s_sin[MAX_HEAD_DIM / 2], s_cos[MAX_HEAD_DIM / 2];
  chain_next();
  chain_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x;
  const int head0 = blockIdx.y * heads_per_block;
  const int n_heads = min(heads_per_block, Hq + 2 * Hk - head0);
  const int pos = positions[r];
  // sincosf of a large argument is a hundred instructions, and the angles are the same for all heads of the row
  if (inv_freq && (int)threadIdx.x < rotary_dim / 2)
    sincosf((float)pos * inv_freq[threadIdx.x], &s_sin[threadIdx.x], &s_cos[threadIdx.x]);
  const T* src = qkv + (long long)r * ld_qkv + (long long)head0 * D;
  const int n = n_heads * D;
  constexpr int V = 16 / (int)sizeof(T);
  if (((uintptr_t)src % 16) == 0 && n % V == 0) {
    for (int i = threadIdx.x; i < n / V; i += 128) {
      const uint4 raw = reinterpret_cast<const uint4*>(src)[i];
      const T* e = reinterpret_cast<const T*>(&raw);
      float f[V];
#pragma unroll
      for (int j = 0; j < V; ++j) f[j] = to_f32(e[j]);
#pragma unroll
      for (int j = 0; j < V; j += 4)
        *reinterpret_cast<float4*>(vec + i * V + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += 128) vec[i] = to_f32(src[i]);
  }
  __syncthreads();
  // where this row's key and value go
  long long kv_at = -1;
  if (k_cache) {
    const int b = req_of_row[r];
    const int page = table_page(block_table + (long long)b * max_pages, pos / page_size, max_pages, num_pages);
    if (page >= 0) kv_at = ((long long)page * Hk) * page_size + pos % page_size;
  }
  if constexpr (DS > 0) {
    constexpr int PAIRS = DS / 64, HALF = DS / 2;
    float wq[2 * PAIRS], wk[2 * PAIRS], sn[PAIRS], cs[PAIRS];
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      const int f = lane + 32 * p;
      wq[2 * p] = q_weight ? q_weight[f] : 1.f;
      wq[2 * p + 1] = q_weight ? q_weight[f + HALF] : 1.f;
      wk[2 * p] = k_weight ? k_weight[f] : 1.f;
      wk[2 * p + 1] = k_weight ? k_weight[f + HALF] : 1.f;
      sn[p] = inv_freq ? s_sin[f] : 0.f;
      cs[p] = inv_freq ? s_cos[f] : 1.f;
    }
    for (int h = warp; h < n_heads; h += 4) {
      const int head = head0 + h;
      const float* x = vec + h * DS;
      float a[PAIRS], b2[PAIRS], ss = 0.f;
      // (the sum of squares in the order of the general form: elements lane, lane + 32, ...)
#pragma unroll
      for (int p = 0; p < PAIRS; ++p) a[p] = x[lane + 32 * p];
#pragma unroll
      for (int p = 0; p < PAIRS; ++p) b2[p] = x[lane + 32 * p + HALF];
#pragma unroll
      for (int p = 0; p < PAIRS; ++p) ss += a[p] * a[p];
#pragma unroll
      for (int p = 0; p < PAIRS; ++p) ss += b2[p] * b2[p];
      ss = warp_sum(ss);
      const bool is_q = head < Hq, is_k = !is_q && head < Hq + Hk;
      const int kvh = is_q ? 0 : (is_k ? head - Hq : head - Hq - Hk);
      T* dst;
      if (is_q) {
        dst = q_out + ((long long)r * Hq + head) * DS;
      } else if (k_cache) {
        if (kv_at < 0) {
          if (lane == 0) atomicExch(status, 2);
          continue;
        }
        dst = (is_k ? k_cache : v_cache) + (kv_at + (long long)kvh * page_size) * DS;
      } else {
        dst = (is_k ? k_out : v_out) + ((long long)r * Hk + kvh) * DS;
      }
      if (is_q || is_k) {
        const float inv = (is_q ? q_weight : k_weight) ? rsqrtf(ss / (float)DS + eps) : 1.f;
#pragma unroll
        for (int p = 0; p < PAIRS; ++p) {
          const int f = lane + 32 * p;
          const float u = a[p] * inv * (is_q ? wq[2 * p] : wk[2 * p]), v = b2[p] * inv * (is_q ? wq[2 * p + 1] : wk[2 * p + 1]);
          dst[f] = from_f32<T>(u * cs[p] - v * sn[p]);
          dst[f + HALF] = from_f32<T>(v * cs[p] + u * sn[p]);
        }
      } else {
#pragma unroll
        for (int p = 0; p < PAIRS; ++p) {
          dst[lane + 32 * p] = from_f32<T>(a[p]);
          dst[lane + 32 * p + HALF] = from_f32<T>(b2[p]);
        }
      }
    }
    return;
  }
  for (int h = warp; h < n_heads; h += 4) {
    const int head = head0 + h;
    const float* x = vec + h * D;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const bool is_q = head < Hq, is_k = !is_q && head < Hq + Hk;
    const int kvh = is_q ? 0 : (is_k ? head - Hq : head - Hq - Hk);
    T* dst;
    if (is_q) {
      dst = q_out + ((long long)r * Hq + head) * D;
    } else if (k_cache) {
      if (kv_at < 0) {   // no page behind this position (or an entry outside the pool): record it and drop the write
        if (lane == 0) atomicExch(status, 2);
        continue;
      }
      dst = (is_k ? k_cache : v_cache) + (kv_at + (long long)kvh * page_size) * D;
    } else {
      dst = (is_k ? k_out : v_out) + ((long long)r * Hk + kvh) * D;
    }
    if (is_q || is_k) {
      const float* w = is_q ? q_weight : k_weight;
      const float inv = w ? rsqrtf(ss / (float)D + eps) : 1.f;
      const int half = inv_freq ? rotary_dim / 2 : 0;
      for (int f = lane; f < half; f += 32) {          // a lane rotates the pair (f, f + half)
        const float a = x[f] * inv * (w ? w[f] : 1.f), b2 = x[f + half] * inv * (w ? w[f + half] : 1.f);
        const float sn = s_sin[f], c = s_cos[f];
        dst[f] = from_f32<T>(a * c - b2 * sn);
        dst[f + half] = from_f32<T>(b2 * c + a * sn);
      }
      for (int i = 2 * half + lane; i < D; i += 32) dst[i] = from_f32<T>(x[i] * inv * (w ? w[i] : 1.f));
    } else {
      for (int i = lane; i < D; i += 32) dst[i] = from_f32<T>(x[i]);
    }
  }
}

// Writes k and v rows [R, Hk, D] into their pages (for position encodings applied outside the fused kernel).
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ k, const T* __restrict__ v, const int* __restrict__ positions,
                                const int* __restrict__ req_of_row, const int* __restrict__ block_table, int max_pages,
                                int page_size, int num_pages, T* __restrict__ k_cache, T* __restrict__ v_cache, int Hk, int D,
                                int* __restrict__ status) {
  const int r = blockIdx.x, kvh = blockIdx.y;
  const int pos = positions[r], b = req_of_row[r];
  const int page = table_page(block_table + (long long)b * max_pages, pos / page_size, max_pages, num_pages);
  if (page < 0) {
    if (threadIdx.x == 0) atomicExch(status, 2);
    return;
  }
  const long long at = (((long long)page * Hk + kvh) * page_size + pos % page_size) * D;
  const long long from = ((long long)r * Hk + kvh) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    k_cache[at + i] = k[from + i];
    v_cache[at + i] = v[from + i];
  }
}

// grid (rows, ceil(Hq / 4)), 128 threads: one warp per (row, query head).
template <typename T>
__global__ void __launch_bounds__(128) paged_attention_simt_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int* __restrict__ block_table, int max_pages, int page_size, int num_pages, const int* __restrict__ req_of_row,
    const int* __restrict__ positions, float scale, int window, T* __restrict__ out, int Hq, int Hk, int D,
    int* __restrict__ status) {
  __shared__ float qs[4][MAX_HEAD_DIM];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * 4 + warp, r = blockIdx.x;
  if (h >= Hq) return;
  const int kvh = h / (Hq / Hk);
  const int b = req_of_row[r], pos = positions[r];
  const int* table = block_table + (long long)b * max_pages;
  const T* qrow = q + ((long long)r * Hq + h) * D;
  float* qv = qs[warp];
  for (int i = lane; i < D; i += 32) qv[i] = to_f32(qrow[i]) * scale;
  __syncwarp();

  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  constexpr int NACC = MAX_HEAD_DIM / 32;
  float acc[NACC];
#pragma unroll
  for (int t = 0; t < NACC; ++t) acc[t] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int base = (lo / 32) * 32; base <= pos; base += 32) {
    const int kp = base + lane;
    const bool valid = kp >= lo && kp <= pos;
    long long off = -1;
    float s = -INFINITY;
    if (valid) {
      const int page = table_page(table, kp / page_size, max_pages, num_pages);
      if (page < 0) {
        atomicExch(status, 3);      // a visible key without a page: recorded, the key is skipped
      } else {
        off = (((long long)page * Hk + kvh) * page_size + kp % page_size) * D;
        const T* kr = k_cache + off;
        float d = 0.f;
        for (int i = 0; i < D; ++i) d = fmaf(qv[i], to_f32(kr[i]), d);
        s = d;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float p = off >= 0 ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int t = 0; t < NACC; ++t) acc[t] *= alpha;
    const int n_here = min(32, pos - base + 1);
    for (int j = 0; j < n_here; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long oj = __shfl_sync(0xffffffffu, off, j);
      if (oj < 0) continue;
      const T* vr = v_cache + oj;
#pragma unroll
      for (int t = 0; t < NACC; ++t) {
        const int i = lane + 32 * t;
        if (i < D) acc[t] = fmaf(pj, to_f32(vr[i]), acc[t]);
      }
    }
    m = m_new;
  }
  T* o = out + ((long long)r * Hq + h) * D;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int t = 0; t < NACC; ++t) {
    const int i = lane + 32 * t;
    if (i < D) o[i] = from_f32<T>(acc[t] * inv);
  }
}

}  // namespace tl

using namespace tl;

static int check_heads(const char* what, int Hq, int Hk, int D) {
  TL_REQUIRE(Hq > 0 && Hk > 0 && Hq % Hk == 0, "%s: %d query heads over %d KV heads", what, Hq, Hk);
  TL_REQUIRE(D >= 16 && D <= MAX_HEAD_DIM && D % 16 == 0,
             "%s: head size %d; multiples of 16 from 16 to %d are implemented", what, D, MAX_HEAD_DIM);
  return 0;
}

extern "C" int tl_qk_prepare(const void* qkv, long long ld_qkv, const float* q_weight, const float* k_weight, float eps,
                             const float* inv_freq, int rotary_dim, const int* positions, const int* req_of_row,
                             const int* block_table, int max_pages, int page_size, int num_pages, void* q_out, void* k_cache,
                             void* v_cache, void* k_out, void* v_out, int rows, int Hq, int Hk, int D, int dtype,
                             int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (int e = check_heads("qk_prepare", Hq, Hk, D)) return e;
  TL_REQUIRE(!inv_freq || (rotary_dim > 0 && rotary_dim <= D && rotary_dim % 2 == 0),
             "qk_prepare: rotary size %d for head size %d", rotary_dim, D);
  TL_REQUIRE((k_cache && v_cache && page_size > 0 && max_pages > 0) || (k_out && v_out),
             "qk_prepare: neither cache pages nor plain outputs for k and v");
  // a decode step's few rows: a few heads a block, so that a row's heads run side by side and not twelve after one another a warp
  int heads_per_block = max(1, min(Hq + 2 * Hk, QK_GROUP_FLOATS / D));
  if (rows <= 64 && heads_per_block > 8) heads_per_block = 8;
  dim3 grid(rows, ceil_div(Hq + 2 * Hk, heads_per_block));
  TL_REQUIRE(grid.y <= 65535, "qk_prepare: %d heads exceed the grid limit", Hq + 2 * Hk);
  // the unrolled form: the whole head is rotated (or nothing is) and a lane's pairs are (f, f + D / 2)
  const int ds = (!inv_freq || rotary_dim == D) && (D == 64 || D == 128) ? D : 0;
  cudaError_t e;
#define TL_QK(T_, DS_)                                                                                                     \
  e = launch_chained(qk_prepare_kernel<T_, DS_>, grid, dim3(128), 0, stream, (const T_*)qkv, ld_qkv, q_weight, k_weight, eps, \
                     inv_freq, rotary_dim, positions, req_of_row, block_table, max_pages, page_size, num_pages, (T_*)q_out,  \
                     (T_*)k_cache, (T_*)v_cache, (T_*)k_out, (T_*)v_out, Hq, Hk, D, heads_per_block, status)
  if (dtype == TL_FP32) {
    if (ds == 64) TL_QK(float, 64);
    else if (ds == 128) TL_QK(float, 128);
    else TL_QK(float, 0);
  } else {
    if (ds == 64) TL_QK(bf16, 64);
    else if (ds == 128) TL_QK(bf16, 128);
    else TL_QK(bf16, 0);
  }
#undef TL_QK
  return (int)e;
}

extern "C" int tl_kv_store(const void* k, const void* v, const int* positions, const int* req_of_row,
                           const int* block_table, int max_pages, int page_size, int num_pages, void* k_cache, void* v_cache,
                           int rows, int Hk, int D, int dtype, int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (int e = check_heads("kv_store", Hk, Hk, D)) return e;
  dim3 grid(rows, Hk);
  TL_REQUIRE(Hk <= 65535, "kv_store: %d KV heads exceed the grid limit", Hk);
  if (dtype == TL_FP32)
    kv_store_kernel<float><<<grid, 64, 0, stream>>>((const float*)k, (const float*)v, positions, req_of_row, block_table,
                                                    max_pages, page_size, num_pages, (float*)k_cache, (float*)v_cache, Hk, D,
                                                    status);
  else
    kv_store_kernel<bf16><<<grid, 64, 0, stream>>>((const bf16*)k, (const bf16*)v, positions, req_of_row, block_table,
                                                   max_pages, page_size, num_pages, (bf16*)k_cache, (bf16*)v_cache, Hk, D,
                                                   status);
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_paged_attention_simt(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                       int max_pages, int page_size, int num_pages, const int* req_of_row,
                                       const int* positions, float scale, int window, void* out, int rows, int Hq, int Hk,
                                       int D, int dtype, int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (int e = check_heads("paged_attention", Hq, Hk, D)) return e;
  TL_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "paged_attention: page size %d, table width %d, window %d",
             page_size, max_pages, window);
  dim3 grid(rows, ceil_div(Hq, 4));
  if (dtype == TL_FP32)
    paged_attention_simt_kernel<float><<<grid, 128, 0, stream>>>(
        (const float*)q, (const float*)k_cache, (const float*)v_cache, block_table, max_pages, page_size, num_pages,
        req_of_row, positions, scale, window, (float*)out, Hq, Hk, D, status);
  else
    paged_attention_simt_kernel<bf16><<<grid, 128, 0, stream>>>(
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_pages, page_size, num_pages,
        req_of_row, positions, scale, window, (bf16*)out, Hq, Hk, D, status);
  TL_LAUNCH_CHECK();
  return 0;
}

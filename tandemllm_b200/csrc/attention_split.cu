// Attention over the paged cache split along the keys (flash-decoding): one CTA per (row, KV head, span of 256
// key positions) computes, for the group's query heads together, the scores of its span, a partial softmax
// (running maximum, sum, weighted values, all 32-bit), and a second kernel joins the spans of a row in ascending
// order. Keys and values are read once per group with 16-byte loads, so a decode step reads the cache at memory
// speed; the reference splits its decode attention the same way (engine/models/lfm2_moe/kernels.py:181-262,
// 512-key spans joined in order). Spans are aligned to absolute positions, so how a row's sum is split depends
// on its position only, never on the batch.
//
//   s = q k^T * scale over positions max(0, pos - window + 1) .. pos; softmax in 32-bit; o = a v
//   query head h reads KV head h / (Hq / Hk)                      (engine/models/lfm2_moe/ref.py:166-178)
//
// Scratch: partial values [rows, Hq, spans, D] and (max, sum) [rows, Hq, spans, 2] in 32-bit, given by the caller.
#include "common.cuh"

namespace tl {

constexpr int SPAN = 256;        // key positions per CTA
constexpr int MAX_GROUP = 8;     // query heads per KV head handled in one pass
constexpr int MAX_D = 256;

template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
};
template <> struct Vec<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const bf16* p, float* v) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// grid (rows, Hk, spans), 128 threads
template <typename T>
__global__ void __launch_bounds__(128) attention_span_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int* __restrict__ block_table, int max_pages, int page_size, const int* __restrict__ req_of_row,
    const int* __restrict__ positions, float scale, int window, float* __restrict__ part_o, float* __restrict__ part_ml,
    T* __restrict__ out, int Hq, int Hk, int D, int n_spans, int* __restrict__ status) {
  constexpr int VEC = Vec<T>::N;
  extern __shared__ float smem[];
  const int r = blockIdx.x, g = blockIdx.y, span = blockIdx.z;
  const int tid = threadIdx.x;
  const int pos = positions[r];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int k_begin = max(lo, span * SPAN), k_end = min(pos + 1, (span + 1) * SPAN);
  if (k_begin >= k_end) return;
  const int n_keys = k_end - k_begin;
  const int G = Hq / Hk;
  const int* table = block_table + (long long)req_of_row[r] * max_pages;
  const int nch = D / VEC;                        // 16-byte chunks per key row
  const int nkl = 128 / nch;                      // key lanes of the value phase
  float* qs = smem;                               // [MAX_GROUP][D]
  float* sc = qs + MAX_GROUP * D;                 // [MAX_GROUP][SPAN]
  long long* offs = (long long*)(sc + MAX_GROUP * SPAN);   // [SPAN] element offset of each key row, -1: no page
  float* red = (float*)(offs + SPAN);             // [128 * VEC * MAX_GROUP] value-phase partials; also reductions

  for (int i = tid; i < n_keys; i += 128) {
    const int kp = k_begin + i;
    const int page = table[kp / page_size];
    if (page < 0) {
      atomicExch(status, 3);
      offs[i] = -1;
    } else {
      offs[i] = (((long long)page * Hk + g) * page_size + kp % page_size) * D;
    }
  }
  const bool single = (lo / SPAN) == (pos / SPAN);     // the row has one span: write the result directly

  for (int h0 = 0; h0 < G; h0 += MAX_GROUP) {
    const int gc = min(MAX_GROUP, G - h0);            // heads in this pass
    const int head0 = g * G + h0;
    __syncthreads();
    for (int i = tid; i < gc * D; i += 128)
      qs[i] = to_f32(q[((long long)r * Hq + head0 + i / D) * D + i % D]) * scale;
    __syncthreads();
    // ---- scores: one thread per key ----
    float mx[MAX_GROUP];
#pragma unroll
    for (int j = 0; j < MAX_GROUP; ++j) mx[j] = -INFINITY;
    for (int i = tid; i < n_keys; i += 128) {
      float dot[MAX_GROUP];
#pragma unroll
      for (int j = 0; j < MAX_GROUP; ++j) dot[j] = 0.f;
      const long long off = offs[i];
      if (off >= 0) {
        const T* kr = k_cache + off;
        for (int c = 0; c < nch; ++c) {
          float kv[VEC];
          Vec<T>::load(kr + c * VEC, kv);
#pragma unroll
          for (int j = 0; j < MAX_GROUP; ++j) {
            if (j < gc) {
              const float* qj = qs + j * D + c * VEC;
#pragma unroll
              for (int e = 0; e < VEC; ++e) dot[j] = fmaf(qj[e], kv[e], dot[j]);
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < MAX_GROUP; ++j) {
        if (j < gc) {
          const float s = off >= 0 ? dot[j] : -INFINITY;
          sc[j * SPAN + i] = s;
          mx[j] = fmaxf(mx[j], s);
        }
      }
    }
    // ---- per-head maximum over the span ----
#pragma unroll
    for (int j = 0; j < MAX_GROUP; ++j) mx[j] = warp_max(mx[j]);
    __syncthreads();
    if ((tid & 31) == 0)
#pragma unroll
      for (int j = 0; j < MAX_GROUP; ++j) red[(tid >> 5) * MAX_GROUP + j] = mx[j];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < MAX_GROUP; ++j)
      mx[j] = fmaxf(fmaxf(red[j], red[MAX_GROUP + j]), fmaxf(red[2 * MAX_GROUP + j], red[3 * MAX_GROUP + j]));
    __syncthreads();
    // ---- exponentials and their sums ----
    float sum[MAX_GROUP];
#pragma unroll
    for (int j = 0; j < MAX_GROUP; ++j) sum[j] = 0.f;
    for (int i = tid; i < n_keys; i += 128) {
#pragma unroll
      for (int j = 0; j < MAX_GROUP; ++j) {
        if (j < gc) {
          const float s = sc[j * SPAN + i];
          const float p = (s == -INFINITY) ? 0.f : expf(s - mx[j]);
          sc[j * SPAN + i] = p;
          sum[j] += p;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < MAX_GROUP; ++j) sum[j] = warp_sum(sum[j]);
    if ((tid & 31) == 0)
#pragma unroll
      for (int j = 0; j < MAX_GROUP; ++j) red[(tid >> 5) * MAX_GROUP + j] = sum[j];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < MAX_GROUP; ++j)
      sum[j] = (red[j] + red[MAX_GROUP + j]) + (red[2 * MAX_GROUP + j] + red[3 * MAX_GROUP + j]);
    __syncthreads();
    // ---- values: thread (key lane kl, chunk c) adds p * v over keys kl, kl + nkl, ... ----
    const int c = tid % nch, kl = tid / nch;
    float acc[MAX_GROUP][VEC];
#pragma unroll
    for (int j = 0; j < MAX_GROUP; ++j)
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[j][e] = 0.f;
    if (kl < nkl) {
      for (int i = kl; i < n_keys; i += nkl) {
        const long long off = offs[i];
        if (off < 0) continue;
        float vv[VEC];
        Vec<T>::load(v_cache + off + c * VEC, vv);
#pragma unroll
        for (int j = 0; j < MAX_GROUP; ++j) {
          if (j < gc) {
            const float p = sc[j * SPAN + i];
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[j][e] = fmaf(p, vv[e], acc[j][e]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < MAX_GROUP; ++j)
        if (j < gc)
#pragma unroll
          for (int e = 0; e < VEC; ++e) red[((long long)kl * MAX_GROUP + j) * D + c * VEC + e] = acc[j][e];
    }
    __syncthreads();
    // ---- join the key lanes in order and store ----
    for (int i = tid; i < gc * D; i += 128) {
      const int j = i / D, d = i % D;
      float o = 0.f;
      for (int l = 0; l < nkl; ++l) o += red[((long long)l * MAX_GROUP + j) * D + d];
      const int head = head0 + j;
      if (single) {
        out[((long long)r * Hq + head) * D + d] = from_f32<T>(sum[j] > 0.f ? o / sum[j] : 0.f);
      } else {
        part_o[(((long long)r * Hq + head) * n_spans + span) * D + d] = o;
      }
    }
    if (!single && tid < gc) {
      const long long at = (((long long)r * Hq + head0 + tid) * n_spans + span) * 2;
      // the loop above left mx[], sum[] identical in every thread
      float m_t = 0.f, s_t = 0.f;
#pragma unroll
      for (int j = 0; j < MAX_GROUP; ++j)
        if (j == tid) {
          m_t = mx[j];
          s_t = sum[j];
        }
      part_ml[at] = m_t;
      part_ml[at + 1] = s_t;
    }
  }
}

// grid (rows, Hq): joins the spans of a row in ascending order
template <typename T>
__global__ void attention_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      const int* __restrict__ positions, int window, T* __restrict__ out, int Hq, int D,
                                      int n_spans) {
  const int r = blockIdx.x, h = blockIdx.y;
  const int pos = positions[r];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int s0 = lo / SPAN, s1 = pos / SPAN;
  if (s0 == s1) return;                                 // written directly by the span kernel
  const long long base = ((long long)r * Hq + h) * n_spans;
  float m = -INFINITY;
  for (int s = s0; s <= s1; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
  float denom = 0.f;
  for (int s = s0; s <= s1; ++s) denom += expf(part_ml[(base + s) * 2] - m) * part_ml[(base + s) * 2 + 1];
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int s = s0; s <= s1; ++s) o += expf(part_ml[(base + s) * 2] - m) * part_o[(base + s) * D + d];
    out[((long long)r * Hq + h) * D + d] = from_f32<T>(o * inv);
  }
}

template <typename T>
static size_t span_smem(int D) {
  return (size_t)(MAX_GROUP * D + MAX_GROUP * SPAN) * sizeof(float) + SPAN * sizeof(long long) +
         (size_t)128 * Vec<T>::N * MAX_GROUP * sizeof(float);
}

}  // namespace tl

using namespace tl;

extern "C" int tl_attention_spans(int max_context) { return max_context <= 0 ? 1 : ceil_div(max_context, SPAN); }

// Floats of scratch for `rows` rows: partial values then (max, sum) pairs.
extern "C" long long tl_attention_scratch_floats(int rows, int Hq, int D, int n_spans) {
  return (long long)rows * Hq * n_spans * (D + 2);
}

extern "C" int tl_paged_attention_split(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                        int max_pages, int page_size, const int* req_of_row, const int* positions,
                                        float scale, int window, void* out, float* scratch, int rows, int Hq, int Hk, int D,
                                        int n_spans, int dtype, int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(Hq > 0 && Hk > 0 && Hq % Hk == 0, "paged_attention: %d query heads over %d KV heads", Hq, Hk);
  TL_REQUIRE(D >= 16 && D <= MAX_D && D % 16 == 0, "paged_attention: head size %d; multiples of 16 from 16 to %d are implemented",
             D, MAX_D);
  TL_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0 && n_spans > 0,
             "paged_attention: page size %d, table width %d, window %d, spans %d", page_size, max_pages, window, n_spans);
  TL_REQUIRE(Hk <= 65535 && n_spans <= 65535, "paged_attention: %d KV heads or %d spans exceed the grid limit", Hk, n_spans);
  TL_REQUIRE(scratch != nullptr, "paged_attention: no scratch memory given");
  float* part_o = scratch;
  float* part_ml = scratch + (long long)rows * Hq * n_spans * D;
  dim3 grid(rows, Hk, n_spans), join(rows, Hq);
  if (dtype == TL_FP32) {
    const size_t smem = span_smem<float>(D);
    static bool set = false;
    if (!set) {
      cudaFuncSetAttribute(attention_span_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)span_smem<float>(MAX_D));
      set = true;
    }
    attention_span_kernel<float><<<grid, 128, smem, stream>>>(
        (const float*)q, (const float*)k_cache, (const float*)v_cache, block_table, max_pages, page_size, req_of_row,
        positions, scale, window, part_o, part_ml, (float*)out, Hq, Hk, D, n_spans, status);
    TL_LAUNCH_CHECK();
    if (n_spans > 1)
      attention_join_kernel<float><<<join, D <= 64 ? 64 : 128, 0, stream>>>(part_o, part_ml, positions, window, (float*)out,
                                                                          Hq, D, n_spans);
  } else {
    const size_t smem = span_smem<bf16>(D);
    static bool set = false;
    if (!set) {
      cudaFuncSetAttribute(attention_span_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)span_smem<bf16>(MAX_D));
      set = true;
    }
    attention_span_kernel<bf16><<<grid, 128, smem, stream>>>(
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_pages, page_size, req_of_row,
        positions, scale, window, part_o, part_ml, (bf16*)out, Hq, Hk, D, n_spans, status);
    TL_LAUNCH_CHECK();
    if (n_spans > 1)
      attention_join_kernel<bf16><<<join, D <= 64 ? 64 : 128, 0, stream>>>(part_o, part_ml, positions, window, (bf16*)out, Hq,
                                                                         D, n_spans);
  }
  TL_LAUNCH_CHECK();
  return 0;
}

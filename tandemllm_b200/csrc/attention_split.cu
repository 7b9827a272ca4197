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
// GM (a template parameter, 4 or 8): query heads of a KV head handled in one pass; larger groups take more passes
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
template <typename T, int GM>
__global__ void __launch_bounds__(128) attention_span_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int* __restrict__ block_table, int max_pages, int page_size, int num_pages, const int* __restrict__ req_of_row,
    const int* __restrict__ positions, float scale, int window, float* __restrict__ part_o, float* __restrict__ part_ml,
    T* __restrict__ out, int Hq, int Hk, int D, int n_spans, int* __restrict__ status) {
  constexpr int VEC = Vec<T>::N;
  extern __shared__ float smem[];
  const int r = blockIdx.x, g = blockIdx.y, span = blockIdx.z;
  const int tid = threadIdx.x;
  const int pos = positions[r];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  // A row whose position lies past the spans the caller sized its scratch for: its far keys have no CTA and no place in
  // the scratch. Recorded like a visible key without a page (the join stops at the last span there is).
  if (span == n_spans - 1 && tid == 0 && pos / SPAN >= n_spans && status != nullptr) atomicExch(status, 3);
  const int k_begin = max(lo, span * SPAN), k_end = min(pos + 1, (span + 1) * SPAN);
  if (k_begin >= k_end) return;
  const int n_keys = k_end - k_begin;
  const int G = Hq / Hk;
  const int* table = block_table + (long long)req_of_row[r] * max_pages;
  const int nch = D / VEC;                        // 16-byte chunks per key row
  const int nkl = 128 / nch;                      // key lanes of the value phase
  float* qs = smem;                               // [GM][D]
  float* sc = qs + GM * D;                 // [GM][SPAN]
  long long* offs = (long long*)(sc + GM * SPAN);   // [SPAN] element offset of each key row, -1: no page
  float* red = (float*)(offs + SPAN);             // [128 * VEC * GM] value-phase partials; also reductions

  for (int i = tid; i < n_keys; i += 128) {
    const int kp = k_begin + i;
    const int page = table_page(table, kp / page_size, max_pages, num_pages);
    if (page < 0) {
      atomicExch(status, 3);
      offs[i] = -1;
    } else {
      offs[i] = (((long long)page * Hk + g) * page_size + kp % page_size) * D;
    }
  }
  const bool single = (lo / SPAN) == (pos / SPAN);     // the row has one span: write the result directly

  for (int h0 = 0; h0 < G; h0 += GM) {
    const int gc = min(GM, G - h0);            // heads in this pass
    const int head0 = g * G + h0;
    __syncthreads();
    for (int i = tid; i < gc * D; i += 128)
      qs[i] = to_f32(q[((long long)r * Hq + head0 + i / D) * D + i % D]) * scale;
    __syncthreads();
    float mx[GM];
#pragma unroll
    for (int j = 0; j < GM; ++j) mx[j] = -INFINITY;
    const bool pow2 = (nch & (nch - 1)) == 0 && nch <= 32;
    if (pow2) {
      // ---- scores, coalesced: thread (key lane, chunk) multiplies its 16 bytes of each key row by the matching
      // part of q; the chunks of a key sit in neighbouring lanes and are added by shuffles in a fixed order ----
      const int c = tid % nch, kl = tid / nch;
      float qreg[GM][VEC];
#pragma unroll
      for (int j = 0; j < GM; ++j)
#pragma unroll
        for (int e = 0; e < VEC; ++e) qreg[j][e] = j < gc ? qs[j * D + c * VEC + e] : 0.f;
      const int rounds = (n_keys + nkl - 1) / nkl;          // every lane runs every round: the shuffles are warp-wide
      for (int t = 0; t < rounds; t += 2) {
        long long off[2];
        float kv[2][VEC];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int i = (t + u) * nkl + kl;
          off[u] = (t + u < rounds && i < n_keys) ? offs[i] : -1;
          if (off[u] >= 0) Vec<T>::load(k_cache + off[u] + c * VEC, kv[u]);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (t + u >= rounds) break;
          const int i = (t + u) * nkl + kl;
          float dot[GM];
#pragma unroll
          for (int j = 0; j < GM; ++j) {
            dot[j] = 0.f;
            if (off[u] >= 0)
#pragma unroll
              for (int e = 0; e < VEC; ++e) dot[j] = fmaf(qreg[j][e], kv[u][e], dot[j]);
          }
          for (int w = nch >> 1; w > 0; w >>= 1)
#pragma unroll
            for (int j = 0; j < GM; ++j)
              if (j < gc) dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], w);
          if (c == 0 && i < n_keys) {
#pragma unroll
            for (int j = 0; j < GM; ++j) {
              if (j < gc) {
                const float s = off[u] >= 0 ? dot[j] : -INFINITY;
                sc[j * SPAN + i] = s;
                mx[j] = fmaxf(mx[j], s);
              }
            }
          }
        }
      }
    } else
    // ---- scores: one thread per key ----
    for (int i = tid; i < n_keys; i += 128) {
      float dot[GM];
#pragma unroll
      for (int j = 0; j < GM; ++j) dot[j] = 0.f;
      const long long off = offs[i];
      if (off >= 0) {
        const T* kr = k_cache + off;
        for (int c = 0; c < nch; ++c) {
          float kv[VEC];
          Vec<T>::load(kr + c * VEC, kv);
#pragma unroll
          for (int j = 0; j < GM; ++j) {
            if (j < gc) {
              const float* qj = qs + j * D + c * VEC;
#pragma unroll
              for (int e = 0; e < VEC; ++e) dot[j] = fmaf(qj[e], kv[e], dot[j]);
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < GM; ++j) {
        if (j < gc) {
          const float s = off >= 0 ? dot[j] : -INFINITY;
          sc[j * SPAN + i] = s;
          mx[j] = fmaxf(mx[j], s);
        }
      }
    }
    // ---- per-head maximum over the span ----
#pragma unroll
    for (int j = 0; j < GM; ++j) mx[j] = warp_max(mx[j]);
    __syncthreads();
    if ((tid & 31) == 0)
#pragma unroll
      for (int j = 0; j < GM; ++j) red[(tid >> 5) * GM + j] = mx[j];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < GM; ++j)
      mx[j] = fmaxf(fmaxf(red[j], red[GM + j]), fmaxf(red[2 * GM + j], red[3 * GM + j]));
    __syncthreads();
    // ---- exponentials and their sums ----
    float sum[GM];
#pragma unroll
    for (int j = 0; j < GM; ++j) sum[j] = 0.f;
    for (int i = tid; i < n_keys; i += 128) {
#pragma unroll
      for (int j = 0; j < GM; ++j) {
        if (j < gc) {
          const float s = sc[j * SPAN + i];
          const float p = (s == -INFINITY) ? 0.f : expf(s - mx[j]);
          sc[j * SPAN + i] = p;
          sum[j] += p;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < GM; ++j) sum[j] = warp_sum(sum[j]);
    if ((tid & 31) == 0)
#pragma unroll
      for (int j = 0; j < GM; ++j) red[(tid >> 5) * GM + j] = sum[j];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < GM; ++j)
      sum[j] = (red[j] + red[GM + j]) + (red[2 * GM + j] + red[3 * GM + j]);
    __syncthreads();
    // ---- values: thread (key lane kl, chunk c) adds p * v over keys kl, kl + nkl, ... ----
    const int c = tid % nch, kl = tid / nch;
    float acc[GM][VEC];
#pragma unroll
    for (int j = 0; j < GM; ++j)
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[j][e] = 0.f;
    if (kl < nkl) {
      for (int i0 = kl; i0 < n_keys; i0 += 4 * nkl) {
        long long off[4];
        float vv[4][VEC];
#pragma unroll
        for (int u = 0; u < 4; ++u) {           // four loads in flight before any is used
          const int i = i0 + u * nkl;
          off[u] = i < n_keys ? offs[i] : -1;
          if (off[u] >= 0) Vec<T>::load(v_cache + off[u] + c * VEC, vv[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (off[u] < 0) continue;
          const int i = i0 + u * nkl;
#pragma unroll
          for (int j = 0; j < GM; ++j) {
            if (j < gc) {
              const float p = sc[j * SPAN + i];
#pragma unroll
              for (int e = 0; e < VEC; ++e) acc[j][e] = fmaf(p, vv[u][e], acc[j][e]);
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < GM; ++j)
        if (j < gc)
#pragma unroll
          for (int e = 0; e < VEC; ++e) red[((long long)kl * GM + j) * D + c * VEC + e] = acc[j][e];
    }
    __syncthreads();
    // ---- join the key lanes in order and store ----
    for (int i = tid; i < gc * D; i += 128) {
      const int j = i / D, d = i % D;
      float o = 0.f;
      for (int l = 0; l < nkl; ++l) o += red[((long long)l * GM + j) * D + d];
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
      for (int j = 0; j < GM; ++j)
        if (j == tid) {
          m_t = mx[j];
          s_t = sum[j];
        }
      part_ml[at] = m_t;
      part_ml[at + 1] = s_t;
    }
  }
}

// grid (rows, Hq), JOIN_Q x DT threads: joins the spans of a row. A decode step at a long context has dozens of spans a
// row and this kernel is a link in the step's chain, so it is laid out for few trips to memory: every warp finds the
// largest of the spans' maxima with a span a lane (one trip for up to 32 spans), thread (q, d) adds the spans s with
// s % JOIN_Q == q for dimension d in ascending order, eight loads in flight, and the JOIN_Q partial sums are added in
// the order of q. The order depends on the row's position and window alone, never on what else the step holds.
constexpr int JOIN_Q = 4;
template <typename T>
__global__ void attention_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      const int* __restrict__ positions, int window, T* __restrict__ out, int Hq, int D,
                                      int n_spans, int span_keys) {
  __shared__ float s_o[JOIN_Q][MAX_D];
  __shared__ float s_sum[JOIN_Q];
  chain_next();
  chain_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int pos = positions[r];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int s0 = lo / span_keys, s1 = min(pos / span_keys, n_spans - 1);      // never past the scratch's last span
  if (s0 >= s1) return;                                 // one span: written directly by the span kernel
  const long long base = ((long long)r * Hq + h) * n_spans;
  const float2* ml2 = reinterpret_cast<const float2*>(part_ml);      // (max, sum) pairs
  const int lane = threadIdx.x & 31;
  const int DT = blockDim.x / JOIN_Q, q = threadIdx.x / DT, dd = threadIdx.x - q * DT;
  float m = -INFINITY;
  for (int s = s0 + lane; s <= s1; s += 32) m = fmaxf(m, ml2[base + s].x);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  constexpr int GROUP = 8;
  const int first = s0 + ((q - s0 % JOIN_Q) + JOIN_Q) % JOIN_Q;      // the first span >= s0 with s % JOIN_Q == q
  for (int d0 = 0; d0 < D; d0 += DT) {
    const int d = d0 + dd;
    float o = 0.f, sum = 0.f;
    if (d < D) {
      for (int g0 = first; g0 <= s1; g0 += GROUP * JOIN_Q) {
        float2 w[GROUP];
        float x[GROUP];
#pragma unroll
        for (int i = 0; i < GROUP; ++i) {
          const int sp = g0 + i * JOIN_Q;
          const bool in = sp <= s1;
          w[i] = in ? ml2[base + sp] : make_float2(-INFINITY, 0.f);
          x[i] = in ? part_o[(base + sp) * D + d] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < GROUP; ++i) {
          const float f = w[i].x == -INFINITY ? 0.f : expf(w[i].x - m);
          sum += f * w[i].y;
          o += f * x[i];
        }
      }
      s_o[q][d] = o;
    }
    if (dd == 0 && d0 == 0) s_sum[q] = sum;
    __syncthreads();
    if (q == 0 && d < D) {
      float denom = 0.f, total = 0.f;
#pragma unroll
      for (int i = 0; i < JOIN_Q; ++i) {
        denom += s_sum[i];
        total += s_o[i][d];
      }
      out[((long long)r * Hq + h) * D + d] = from_f32<T>(denom > 0.f ? total / denom : 0.f);
    }
    __syncthreads();
  }
}

template <typename T, int GM>
static size_t span_smem(int D) {
  return (size_t)(GM * D + GM * SPAN) * sizeof(float) + SPAN * sizeof(long long) +
         (size_t)128 * Vec<T>::N * GM * sizeof(float);
}

template <typename T, int GM>
static int launch_spans(const void* q, const void* k_cache, const void* v_cache, const int* block_table, int max_pages,
                        int page_size, int num_pages, const int* req_of_row, const int* positions, float scale, int window, void* out,
                        float* part_o, float* part_ml, int rows, int Hq, int Hk, int D, int n_spans, int* status,
                        cudaStream_t stream) {
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(attention_span_kernel<T, GM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)span_smem<T, GM>(MAX_D));
    if (e != cudaSuccess) return (int)e;
    set = true;
  }
  dim3 grid(rows, Hk, n_spans);
  attention_span_kernel<T, GM><<<grid, 128, span_smem<T, GM>(D), stream>>>(
      (const T*)q, (const T*)k_cache, (const T*)v_cache, block_table, max_pages, page_size, num_pages, req_of_row, positions,
      scale, window, part_o, part_ml, (T*)out, Hq, Hk, D, n_spans, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (n_spans > 1) {
    dim3 join(rows, Hq);
    attention_join_kernel<T><<<join, JOIN_Q * (D <= 64 ? 64 : 128), 0, stream>>>(part_o, part_ml, positions, window, (T*)out, Hq, D,
                                                                    n_spans, SPAN);
    e = cudaGetLastError();
  }
  return (int)e;
}

}  // namespace tl

using namespace tl;

extern "C" int tl_attention_spans(int max_context) { return max_context <= 0 ? 1 : ceil_div(max_context, SPAN); }

// Floats of scratch for `rows` rows: partial values then (max, sum) pairs.
extern "C" long long tl_attention_scratch_floats(int rows, int Hq, int D, int n_spans) {
  return (long long)rows * Hq * n_spans * (D + 2);
}

extern "C" int tl_paged_attention_split(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                        int max_pages, int page_size, int num_pages, const int* req_of_row, const int* positions,
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
  const bool small = Hq / Hk <= 4;
#define TL_SPANS(T, GM) launch_spans<T, GM>(q, k_cache, v_cache, block_table, max_pages, page_size, num_pages, req_of_row, \
                                            positions, scale, window, out, part_o, part_ml, rows, Hq, Hk, D, n_spans, status, stream)
  if (dtype == TL_FP32) return small ? TL_SPANS(float, 4) : TL_SPANS(float, 8);
  return small ? TL_SPANS(bf16, 4) : TL_SPANS(bf16, 8);
#undef TL_SPANS
}

// Joins the spans that another kernel left in `scratch` (same layout as above) into `out`, in ascending order.
// `span_keys`: the key positions a span covers (the kernel that wrote the spans chose it).
extern "C" int tl_attention_join(const float* scratch, const int* positions, int window, void* out, int rows, int Hq, int D,
                                 int n_spans, int span_keys, int dtype, cudaStream_t stream) {
  if (rows == 0 || n_spans <= 1) return 0;
  TL_REQUIRE(scratch != nullptr && Hq > 0 && Hq <= 65535 && D > 0 && span_keys > 0,
             "attention join: %d heads of size %d, spans of %d keys", Hq, D, span_keys);
  const float* part_o = scratch;
  const float* part_ml = scratch + (long long)rows * Hq * n_spans * D;
  dim3 join(rows, Hq);
  cudaError_t e;
  if (dtype == TL_FP32)
    e = launch_chained(attention_join_kernel<float>, join, dim3(JOIN_Q * (D <= 64 ? 64 : 128)), 0, stream, part_o, part_ml, positions,
                       window, (float*)out, Hq, D, n_spans, span_keys);
  else
    e = launch_chained(attention_join_kernel<bf16>, join, dim3(JOIN_Q * (D <= 64 ? 64 : 128)), 0, stream, part_o, part_ml, positions,
                       window, (bf16*)out, Hq, D, n_spans, span_keys);
  return (int)e;
}

// ------------------------------------------------------------------------------------------------------------------
// The split kernel with its scratch inside the library, for callers that cannot allocate device memory.
// attention_noalloc.h says who they are, what the array costs and the rules that come with sharing it.
#include <mutex>

#include "attention_noalloc.h"

// The scratch itself: device memory that exists on every GPU the library is loaded on, until the process ends.
// In host code this name is only a handle for cudaGetSymbolAddress; kernels must be given the address it returns.
static __device__ __align__(256) float tl_static_scratch[TL_STATIC_SCRATCH_FLOATS];

static const int TL_MAX_DEVICES = 64;
static float* tl_static_scratch_address[TL_MAX_DEVICES];     // per device, looked up at the first call there
static std::mutex tl_static_scratch_mutex;

extern "C" int tl_paged_attention_split_static(const void* q, const void* k_cache, const void* v_cache,
                                               const int* block_table, int max_pages, int page_size, int num_pages,
                                               const int* req_of_row, const int* positions, float scale, int window,
                                               void* out, int rows, int Hq, int Hk, int D, int n_spans, int dtype,
                                               int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && Hq > 0 && D > 0 && n_spans > 0, "paged_attention (static scratch): rows %d, heads %d, head size %d, spans %d",
             rows, Hq, D, n_spans);
  const long long need = tl_attention_scratch_floats(rows, Hq, D, n_spans);
  TL_REQUIRE(need <= (long long)TL_STATIC_SCRATCH_FLOATS,
             "paged_attention (static scratch): %d rows x %d heads x %d spans x (%d + 2) = %lld floats of scratch, the "
             "library's fixed array holds %d; bring your own scratch to tl_paged_attention_split for sizes like this",
             rows, Hq, n_spans, D, need, (int)TL_STATIC_SCRATCH_FLOATS);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  TL_REQUIRE(device >= 0 && device < TL_MAX_DEVICES, "paged_attention (static scratch): device index %d", device);
  float* scratch;
  {
    // set-up, once per device, with that device current: the array's address on this device
    std::lock_guard<std::mutex> guard(tl_static_scratch_mutex);
    if (tl_static_scratch_address[device] == nullptr) {
      float* address = nullptr;
      e = cudaGetSymbolAddress((void**)&address, tl_static_scratch);
      if (e != cudaSuccess) return (int)e;
      tl_static_scratch_address[device] = address;
    }
    scratch = tl_static_scratch_address[device];
  }
  // from here on it is the ordinary entry point, which launches the two kernels and allocates nothing
  return tl_paged_attention_split(q, k_cache, v_cache, block_table, max_pages, page_size, num_pages, req_of_row, positions, scale,
                                  window, out, scratch, rows, Hq, Hk, D, n_spans, dtype, status, stream);
}

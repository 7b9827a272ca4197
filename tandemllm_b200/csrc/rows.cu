// Row-wise kernels: embedding gather, residual add fused with RMS norm (and, for the rows of an expert layer, with
// the router), SwiGLU gating, and the last error message of the library.
//
// The residual stream is 32-bit in both precisions; norms compute mean(x^2), rsqrt and the scale in
// 32-bit and round once to the compute type. Formulas: engine/models/lfm2_moe/ref.py:105-109 (norm),
// :230 (embedding), :180-183 (SwiGLU), :185-197 (router) of the reference, which fuses the add and the norm too
// (`add_rms`, engine/models/lfm2_moe/kernels.py:90-107).
#include "route.cuh"

extern "C" const char* tl_last_error() { return tl_error_text; }

extern "C" const char* tl_cuda_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

namespace tl {

// residual[r, :] = float(table[token[r], :])
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                  float* __restrict__ residual, int hidden, int vocab, int* __restrict__ status) {
  chain_next();
  chain_wait();
  const int r = blockIdx.x;
  int tok = tokens[r];
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0) atomicExch(status, 1);   // recorded, and the row reads token 0 instead of faulting
    tok = 0;
  }
  const T* src = table + (size_t)tok * hidden;
  float* dst = residual + (size_t)r * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_f32(src[c]);
}

// What is added to the residual before the norm. The previous branch's output comes in one of three forms, so
// that the kernel which would only have summed it can be left out:
//   delta, parts = 1          a plain 32-bit tensor [rows, hidden]
//   delta, parts = S          S partial sums [S, rows, hidden] of a product split along k, added in order 0..S-1
//   expert_rows               the rows a routed expert layer computed, [pairs, hidden] in expert-sorted order:
//                             row r adds sum_j wts[r, j] * expert_rows[pos_of_pair[r k + j]] over its slots in
//                             ascending expert id (engine/models/lfm2_moe/ref.py:207-214)
struct NormParams {
  float* residual;
  const float* delta;
  int parts;
  long long part_stride;
  const float* expert_rows;
  int expert_parts;          // the expert rows come as this many partial sums (1: whole), expert_part_stride floats apart
  long long expert_part_stride;
  const int* pos_of_pair;
  const int* ids;
  const float* wts;
  int top_k;
  const float* weight;
  float eps;
  void* normed;
  float* normed32;
  const int* gather;
  int hidden;
  // the router of the layer that reads the normed rows (optional)
  const float* router_w;     // [E, hidden] 32-bit
  const float* router_bias;  // [E] or nullptr
  int E, route_k, normalize;
  float floor_, scale;
  int* route_ids;            // [rows, route_k]
  float* route_wts;
  int rows_per_block, out_rows;
  unsigned zero;             // 0 (see router_logits_one_row)
  int split;                 // CTAs a row (a cluster; one row a block with a router): each takes every split-th expert
};

// With a router and many rows, a block norms this many rows before it multiplies them by the router's weights,
// so that the weights are read once per block and not once per row.
constexpr int ROUTER_SPLIT = 8;            // CTAs a row (a cluster) for a decode step's router
constexpr int ROUTER_SPLIT_ROWS = 16;      // rows of a step up to which the router's rows are split
constexpr int MAX_ROWS_PER_BLOCK = 8;
constexpr int PLAIN_ROWS_PER_BLOCK = 4;   // without a router

// logits[rr, e] = rows[rr] . router_w[e] for the block's n_rows <= ROWS rows (in shared memory). Sixteen-byte loads,
// eight of them in flight a lane, when the width allows.
template <int ROWS>
__device__ __forceinline__ void router_logits(const NormParams& p, const float* rows, float* logits, int n_rows, int lane,
                                              int warp, int nwarps) {
  const int hidden = p.hidden;
  if (ROWS > 1 && (hidden & 3) == 0) {
    // two experts a pass: a piece of a row read from shared memory serves both (these reads are what the loop waits for)
    const int h4 = hidden >> 2;
    for (int e = warp; e < p.E; e += 2 * nwarps) {
      const int e2 = e + nwarps;
      const bool two = e2 < p.E;
      const float4* wa = reinterpret_cast<const float4*>(p.router_w + (size_t)e * hidden);
      const float4* wb = reinterpret_cast<const float4*>(p.router_w + (size_t)(two ? e2 : e) * hidden);
      float acc_a[ROWS], acc_b[ROWS];
#pragma unroll
      for (int rr = 0; rr < ROWS; ++rr) acc_a[rr] = acc_b[rr] = 0.f;
#pragma unroll 2
      for (int c = lane; c < h4; c += 32) {
        const float4 va = __ldg(wa + c), vb = __ldg(wb + c);
#pragma unroll
        for (int rr = 0; rr < ROWS; ++rr)
          if (rr < n_rows) {
            const float4 x = reinterpret_cast<const float4*>(rows + (size_t)rr * hidden)[c];
            acc_a[rr] = fmaf(x.w, va.w, fmaf(x.z, va.z, fmaf(x.y, va.y, fmaf(x.x, va.x, acc_a[rr]))));
            acc_b[rr] = fmaf(x.w, vb.w, fmaf(x.z, vb.z, fmaf(x.y, vb.y, fmaf(x.x, vb.x, acc_b[rr]))));
          }
      }
#pragma unroll
      for (int rr = 0; rr < ROWS; ++rr) {
        if (rr < n_rows) {
          const float a = warp_sum(acc_a[rr]), b = warp_sum(acc_b[rr]);
          if (lane == 0) {
            logits[rr * p.E + e] = a;
            if (two) logits[rr * p.E + e2] = b;
          }
        }
      }
    }
    return;
  }
  for (int e = warp; e < p.E; e += nwarps) {
    const float* w = p.router_w + (size_t)e * hidden;
    float acc[ROWS];
#pragma unroll
    for (int rr = 0; rr < ROWS; ++rr) acc[rr] = 0.f;
    if ((hidden & 3) == 0) {
      const int h4 = hidden >> 2;
      const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll 8
      for (int c = lane; c < h4; c += 32) {
        const float4 wv = __ldg(w4 + c);
#pragma unroll
        for (int rr = 0; rr < ROWS; ++rr)
          if (rr < n_rows) {
            const float4 x = reinterpret_cast<const float4*>(rows + (size_t)rr * hidden)[c];
            acc[rr] = fmaf(x.w, wv.w, fmaf(x.z, wv.z, fmaf(x.y, wv.y, fmaf(x.x, wv.x, acc[rr]))));
          }
      }
    } else {
#pragma unroll 4
      for (int c = lane; c < hidden; c += 32) {
        const float wv = __ldg(w + c);
#pragma unroll
        for (int rr = 0; rr < ROWS; ++rr)
          if (rr < n_rows) acc[rr] = fmaf(rows[(size_t)rr * hidden + c], wv, acc[rr]);
      }
    }
#pragma unroll
    for (int rr = 0; rr < ROWS; ++rr) {
      if (rr < n_rows) {
        const float v = warp_sum(acc[rr]);
        if (lane == 0) logits[rr * p.E + e] = v;
      }
    }
  }
}

// The same for a block's single row (a decode step), written so that a lane's sixteen 16-byte loads of an expert's
// weights are all on their way before the first product needs one: the first product is made to depend on every
// load (`zero` is 0, which only the host knows), or the compiler would set each product right behind its own load and
// the warp, which issues in order, would wait there with the other loads unsent. The sum is built in the same order
// as above.
__device__ __forceinline__ void router_logits_one_row(const NormParams& p, const float* row, float* logits, int lane,
                                                      int warp, int nwarps, int rank) {
  constexpr int CH = 16;
  const int hidden = p.hidden, h4 = hidden >> 2;
  const float4* row4 = reinterpret_cast<const float4*>(row);
  // With `split` CTAs a row (a cluster), this one takes experts rank, rank + split, ..., a warp an expert as ever, and
  // hands each logit to the cluster's first CTA, which makes the choice.
  uint32_t first_cta_logits = 0;
  if (p.split > 1)
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(first_cta_logits) : "r"((uint32_t)__cvta_generic_to_shared(logits)), "r"(0));
  for (int j = warp; j * p.split + rank < p.E; j += nwarps) {
    const int e = j * p.split + rank;
    const float4* w4 = reinterpret_cast<const float4*>(p.router_w + (size_t)e * hidden);
    float acc = 0.f;
    for (int c0 = lane; c0 < h4; c0 += 32 * CH) {
      float4 wv[CH];
      unsigned all = 0u;
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int c = c0 + 32 * i;
        wv[i] = c < h4 ? __ldg(w4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        all ^= __float_as_uint(wv[i].w);
      }
      wv[0].x = __uint_as_float(__float_as_uint(wv[0].x) ^ (all & p.zero));
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int c = c0 + 32 * i;
        if (c < h4) {
          const float4 x = row4[c];
          acc = fmaf(x.w, wv[i].w, fmaf(x.z, wv[i].z, fmaf(x.y, wv[i].y, fmaf(x.x, wv[i].x, acc))));
        }
      }
    }
    const float v = warp_sum(acc);
    if (lane == 0) {
      if (p.split > 1) asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(first_cta_logits + 4u * (uint32_t)e), "f"(v) : "memory");
      else logits[e] = v;
    }
  }
}

// A block takes rows_per_block consecutive output rows at once, blockDim / rows_per_block threads (whole warps) a row:
// one row for a decode step, several for a prompt, so that every thread has a few 16-byte loads of each input in
// flight and the router's weights are read once a block.
//   gather == nullptr: row r:  residual[r] += added[r];  normed[r] = w * residual[r] * rsqrt(mean + eps)
//   gather != nullptr: output row i reads row gather[i] and leaves the residual as it is (the final norm of the
//                      wanted rows only)
// normed32 (optional) receives the normalised row unrounded. With a router, the row's logits are computed from
// the unrounded row in 32-bit, and the choice and weights are written as well.
// ROUTE_PER: 0 without a router (a small kernel, three blocks an SM), else the experts a lane of the choosing warp holds.
// ONE_ROW: the launch gives every block one row (a decode step: few blocks, which may take all the registers they like).
template <typename T, int ROUTE_PER, bool ONE_ROW>
__global__ void __launch_bounds__(512, ONE_ROW ? 1 : (ROUTE_PER <= 4 ? 2 : 1)) add_rmsnorm_kernel(NormParams p) {
  // rows_per_block rows of `hidden` floats, 33 for the reduction, then rows_per_block x E logits
  extern __shared__ __align__(16) float rows_buf[];
  float* scratch = rows_buf + (size_t)p.rows_per_block * p.hidden;
  float* logits = scratch + 33;
  __shared__ int s_src[MAX_ROWS_PER_BLOCK][MAX_TOP_K];
  __shared__ float s_w[MAX_ROWS_PER_BLOCK][MAX_TOP_K];
  chain_next();
  chain_wait();
  const int hidden = p.hidden;
  // One row a block: the thread's piece of the norm's weight does not depend on the row and is asked for first, or its
  // round trip would come after the row's sum of squares, at the end of the kernel's chain.
  float4 norm_w = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool has_norm_w = ONE_ROW && (hidden & 3) == 0 && (int)threadIdx.x < (hidden >> 2);
  if (has_norm_w) norm_w = reinterpret_cast<const float4*>(p.weight)[threadIdx.x];
  // (a router's one-row form may run `split` CTAs a row: all of them put the row together, the first one stores it)
  const int split = (ONE_ROW && ROUTE_PER > 0) ? p.split : 1;
  const int rank = split > 1 ? (int)(blockIdx.x % split) : 0;
  const int first_row = (int)(blockIdx.x / split) * p.rows_per_block;
  if constexpr (ONE_ROW && ROUTE_PER > 0) {
    // The router's weights that this CTA's warps will read are asked into L2 now (they are cold every step: a step
    // streams gigabytes through L2), so that their trip to DRAM runs under the row's chain. No registers are held.
    const int lane_ = threadIdx.x & 31, warp_ = threadIdx.x >> 5, nwarps_ = blockDim.x >> 5;
    for (int j = warp_; j * split + rank < p.E; j += nwarps_) {
      const char* w = reinterpret_cast<const char*>(p.router_w + (size_t)(j * split + rank) * hidden);
      for (int b = lane_ * 128; b < hidden * 4; b += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(w + b));
    }
  }
  const int n_rows = min(p.rows_per_block, p.out_rows - first_row);
  const int G = blockDim.x / p.rows_per_block;           // threads a row
  const int rr = threadIdx.x / G, t = threadIdx.x - rr * G;
  const bool live = rr < n_rows;
  const int out_r = first_row + (live ? rr : 0);
  float* row = rows_buf + (size_t)rr * hidden;
  const int r = p.gather ? p.gather[out_r] : out_r;
  if (p.expert_rows) {
    if (live && t < 32) {
      // the row's slots in ascending expert id (the slot index breaks ties): lane j ranks slot j among the others
      const int k = p.top_k, j = t;
      const bool mine = j < k;
      const int e = mine ? p.ids[(long long)r * k + j] : 0x7fffffff;
      const int src = mine ? p.pos_of_pair[(long long)r * k + j] : 0;
      const float w = mine ? p.wts[(long long)r * k + j] : 0.f;
      int rank = 0;
      for (int i = 0; i < k; ++i) {
        const int ei = __shfl_sync(0xffffffffu, e, i);
        rank += (ei < e) || (ei == e && i < j);
      }
      if (mine) {
        s_src[rr][rank] = src;
        s_w[rr][rank] = w;
      }
    }
    __syncthreads();
  }
  float* res = p.residual + (size_t)r * hidden;
  const bool adds = p.delta || p.expert_rows;
  const bool vec = (hidden & 3) == 0;           // rows are then 16-byte aligned: four elements a step
  float ss = 0.f;
  // A row that gets a plain tensor added (or nothing) and whose thread holds at most IN_REGS 16-byte pieces of it: all
  // of the thread's loads are sent before the first is used, and the pieces stay in registers until they are normed.
  constexpr int IN_REGS = 4;
  const bool in_regs = vec && !p.expert_rows && (hidden >> 2) <= G * IN_REGS;
  float4 xr[IN_REGS];
  if (in_regs) {
    const int h4 = hidden >> 2;
    const float4* res4 = reinterpret_cast<const float4*>(res);
    const float4* d4 = p.delta ? reinterpret_cast<const float4*>(p.delta + (size_t)r * hidden) : nullptr;
    float4 dr[IN_REGS];
#pragma unroll
    for (int i = 0; i < IN_REGS; ++i) {
      const int c = t + i * G;
      const bool ok = live && c < h4;
      xr[i] = ok ? res4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
      dr[i] = ok && d4 ? d4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // a product left in partial sums: the further parts, added in order, a round of the thread's loads a part
    for (int s = 1; s < p.parts; ++s) {
      const float4* ds4 = reinterpret_cast<const float4*>(p.delta + (long long)s * p.part_stride + (size_t)r * hidden);
      float4 more[IN_REGS];
#pragma unroll
      for (int i = 0; i < IN_REGS; ++i) {
        const int c = t + i * G;
        more[i] = live && c < h4 ? ds4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int i = 0; i < IN_REGS; ++i) {
        dr[i].x += more[i].x; dr[i].y += more[i].y; dr[i].z += more[i].z; dr[i].w += more[i].w;
      }
    }
#pragma unroll
    for (int i = 0; i < IN_REGS; ++i) {
      xr[i].x += dr[i].x; xr[i].y += dr[i].y; xr[i].z += dr[i].z; xr[i].w += dr[i].w;
      ss += xr[i].x * xr[i].x + xr[i].y * xr[i].y + xr[i].z * xr[i].z + xr[i].w * xr[i].w;
    }
  } else if (live) {
    if (vec) {
      const int h4 = hidden >> 2;
      const float4* res4 = reinterpret_cast<const float4*>(res);
      for (int c = t; c < h4; c += G) {
        float4 x = res4[c];
        if (p.delta) {
          float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int s = 0; s < p.parts; ++s) {
            const float4 v = reinterpret_cast<const float4*>(p.delta + (long long)s * p.part_stride + (size_t)r * hidden)[c];
            d.x += v.x; d.y += v.y; d.z += v.z; d.w += v.w;
          }
          x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w;
        }
        if (p.expert_rows) {
          // four expert rows at a time, all loaded (with the further parts of a split down product) before the first
          // is used; added in ascending expert id as ever
          float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
          constexpr int STEP = 4;
          for (int j0 = 0; j0 < p.top_k; j0 += STEP) {
            float4 v[STEP];
#pragma unroll
            for (int i = 0; i < STEP; ++i)
              v[i] = j0 + i < p.top_k ? reinterpret_cast<const float4*>(p.expert_rows + (long long)s_src[rr][j0 + i] * hidden)[c]
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 1; s < p.expert_parts; ++s) {       // a down projection split along k: its partial sums, in order
              float4 more[STEP];
#pragma unroll
              for (int i = 0; i < STEP; ++i)
                more[i] = j0 + i < p.top_k
                              ? reinterpret_cast<const float4*>(p.expert_rows + (long long)s * p.expert_part_stride +
                                                                (long long)s_src[rr][j0 + i] * hidden)[c]
                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
              for (int i = 0; i < STEP; ++i) {
                v[i].x += more[i].x; v[i].y += more[i].y; v[i].z += more[i].z; v[i].w += more[i].w;
              }
            }
#pragma unroll
            for (int i = 0; i < STEP; ++i)
              if (j0 + i < p.top_k) {
                const float w = s_w[rr][j0 + i];
                d.x = fmaf(w, v[i].x, d.x); d.y = fmaf(w, v[i].y, d.y); d.z = fmaf(w, v[i].z, d.z); d.w = fmaf(w, v[i].w, d.w);
              }
          }
          x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w;
        }
        reinterpret_cast<float4*>(row)[c] = x;
        ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
      }
    } else {
      for (int c = t; c < hidden; c += G) {
        float x = res[c];
        if (p.delta) {
          float d = 0.f;
          for (int s = 0; s < p.parts; ++s) d += p.delta[(long long)s * p.part_stride + (size_t)r * hidden + c];
          x += d;
        }
        if (p.expert_rows) {
          float d = 0.f;
          for (int j = 0; j < p.top_k; ++j) {
            float v = p.expert_rows[(long long)s_src[rr][j] * hidden + c];
            for (int s = 1; s < p.expert_parts; ++s)
              v += p.expert_rows[(long long)s * p.expert_part_stride + (long long)s_src[rr][j] * hidden + c];
            d = fmaf(s_w[rr][j], v, d);
          }
          x += d;
        }
        row[c] = x;
        ss += x * x;
      }
    }
  }
  // a row's sum of squares: its warps' sums, added in warp order
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = ss;
  __syncthreads();
  ss = 0.f;
  for (int wi = rr * (G >> 5); wi < (rr + 1) * (G >> 5); ++wi) ss += scratch[wi];
  const float inv = rsqrtf(ss / (float)hidden + p.eps);
  T* out = (T*)p.normed + (size_t)out_r * hidden;
  float* out32 = p.normed32 ? p.normed32 + (size_t)out_r * hidden : nullptr;
  if (live) {
    if (vec) {
      const int h4 = hidden >> 2;
      auto finish = [&](int c, const float4 x) {
        if (!p.gather && adds && rank == 0) reinterpret_cast<float4*>(res)[c] = x;
        const float4 w = (has_norm_w && c == (int)threadIdx.x) ? norm_w : reinterpret_cast<const float4*>(p.weight)[c];
        const float4 y = make_float4(w.x * (x.x * inv), w.y * (x.y * inv), w.z * (x.z * inv), w.w * (x.w * inv));
        if (rank == 0) {
          if constexpr (sizeof(T) == 2) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(out)[c] = packed;
          } else {
            reinterpret_cast<float4*>(out)[c] = y;
          }
          if (out32) reinterpret_cast<float4*>(out32)[c] = y;
        }
        if (ROUTE_PER > 0) reinterpret_cast<float4*>(row)[c] = y;      // the router reads the normed rows from here
      };
      if (in_regs) {
#pragma unroll
        for (int i = 0; i < IN_REGS; ++i)
          if (t + i * G < h4) finish(t + i * G, xr[i]);
      } else {
        for (int c = t; c < h4; c += G) finish(c, reinterpret_cast<const float4*>(row)[c]);
      }
    } else {
      for (int c = t; c < hidden; c += G) {
        const float x = row[c];
        const float y = p.weight[c] * (x * inv);
        if (rank == 0) {
          if (!p.gather && adds) res[c] = x;
          out[c] = from_f32<T>(y);
          if (out32) out32[c] = y;
        }
        row[c] = y;
      }
    }
  }
  if constexpr (ROUTE_PER > 0) {
    __syncthreads();
    // logits[row, e] = row . router_w[e]: each warp takes experts warp, warp + nwarps, ...; lanes stride over the
    // columns; an expert's weights are read once for all rows of the block. A row's sum is built in the same order
    // whether the block holds one row or several.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (ONE_ROW && (p.hidden & 3) == 0) router_logits_one_row(p, rows_buf, logits, lane, warp, nwarps, rank);
    else if (n_rows == 1) router_logits<1>(p, rows_buf, logits, 1, lane, warp, nwarps);
    else router_logits<MAX_ROWS_PER_BLOCK>(p, rows_buf, logits, n_rows, lane, warp, nwarps);
    if (split > 1) {
      // every CTA of the row has sent its logits to the first one
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
      if (rank != 0) return;
    }
    __syncthreads();
    for (int rr = warp; rr < n_rows; rr += nwarps)
      warp_route_sized<ROUTE_PER>(logits + rr * p.E, p.router_bias, p.E, p.route_k, p.normalize, p.floor_, p.scale,
                                  p.route_ids + (size_t)(first_row + rr) * p.route_k,
                                  p.route_wts + (size_t)(first_row + rr) * p.route_k);
  }
}

// out[r, i] = act(gate_up[r, i]) * gate_up[r, inter + i]
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long rows, int inter, int act) {
  chain_next();
  chain_wait();
  const long long n = rows * inter;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / inter;
    const int c = (int)(i - r * inter);
    const float g = to_f32(gate_up[r * 2 * inter + c]);
    const float u = to_f32(gate_up[r * 2 * inter + inter + c]);
    out[i] = from_f32<T>(gated(g, u, act));
  }
}

}  // namespace tl

using namespace tl;

extern "C" int tl_embed_rows(const void* table, const int* tokens, float* residual, int rows, int hidden, int vocab,
                             int dtype, int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && hidden > 0 && vocab > 0, "embed_rows: rows %d hidden %d vocab %d", rows, hidden, vocab);
  const int threads = hidden >= 1024 ? 256 : 128;
  cudaError_t e;
  if (dtype == TL_FP32)
    e = launch_chained(embed_rows_kernel<float>, dim3(rows), dim3(threads), 0, stream, (const float*)table, tokens, residual,
                       hidden, vocab, status);
  else
    e = launch_chained(embed_rows_kernel<bf16>, dim3(rows), dim3(threads), 0, stream, (const bf16*)table, tokens, residual,
                       hidden, vocab, status);
  return (int)e;
}

extern "C" void tl_set_chained_launches(int enabled) { chained_launches() = enabled; }

// See NormParams for the forms of what is added. Null pointers switch a form or the router off.
// An ordinary launch in clusters of `cluster` CTAs along x.
template <typename... KernelArgs, typename... Args>
static cudaError_t launch_clustered(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    int cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KernelArgs>(args)...);
}

extern "C" int tl_add_rmsnorm(float* residual, const float* delta, int parts, long long part_stride,
                              const float* expert_rows, int expert_parts, long long expert_part_stride,
                              const int* pos_of_pair, const int* ids, const float* wts, int top_k,
                              const float* weight, void* normed, float* normed32, const int* gather, int out_rows,
                              int hidden, float eps, int dtype, const float* router_w, const float* router_bias, int E,
                              int route_k, int normalize, float floor_, float scale, int* route_ids, float* route_wts,
                              cudaStream_t stream) {
  if (out_rows == 0) return 0;
  TL_REQUIRE(out_rows > 0 && hidden > 0, "add_rmsnorm: rows %d hidden %d", out_rows, hidden);
  TL_REQUIRE(!delta || parts >= 1, "add_rmsnorm: %d parts", parts);
  TL_REQUIRE(!expert_rows || (top_k > 0 && top_k <= MAX_TOP_K && pos_of_pair && ids && wts),
             "add_rmsnorm: expert rows with top-%d", top_k);
  if (router_w) {
    TL_REQUIRE(E > 0 && E <= MAX_EXPERTS, "router: %d experts; up to %d are implemented", E, MAX_EXPERTS);
    TL_REQUIRE(route_k > 0 && route_k <= E && route_k <= MAX_TOP_K && route_ids && route_wts,
               "router: top-%d of %d experts; up to top-%d is implemented", route_k, E, MAX_TOP_K);
    TL_REQUIRE(normalize >= 0 && (normalize >> 1) <= TL_SCORE_LAST, "router: scoring function %d is not one of 0..%d",
               normalize >> 1, TL_SCORE_LAST);
  }
  // prompts: several rows a block (eight beside a router, whose weights are then read once for eight rows)
  // (a few hundred rows: fewer rows a block, so that there are about as many blocks as SMs: at 128 rows eight rows a
  // block were 16 blocks, 22 us a norm where one row a block takes 7)
  const int most = router_w ? MAX_ROWS_PER_BLOCK : PLAIN_ROWS_PER_BLOCK;
  int rows_per_block = 1;
  while (rows_per_block < most && out_rows > 160 * rows_per_block) rows_per_block *= 2;
  while (rows_per_block > 1 && (size_t)rows_per_block * (hidden + E) * sizeof(float) > 96 * 1024) rows_per_block /= 2;
  const size_t smem = ((size_t)rows_per_block * hidden + 33 + (router_w ? (size_t)rows_per_block * E : 0)) * sizeof(float);
  TL_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: hidden size %d needs %zu bytes of shared memory, the limit is 204800",
             hidden, smem);
  NormParams p = {};
  p.residual = residual; p.delta = delta; p.parts = parts; p.part_stride = part_stride; p.expert_rows = expert_rows;
p.expert_parts = expert_parts < 1 ? 1 : expert_parts; p.expert_part_stride = expert_part_stride;
  p.pos_of_pair = pos_of_pair; p.ids = ids; p.wts = wts; p.top_k = top_k; p.weight = weight; p.eps = eps;
  p.normed = normed; p.normed32 = normed32; p.gather = gather; p.hidden = hidden; p.router_w = router_w;
  p.router_bias = router_bias; p.E = E; p.route_k = route_k; p.normalize = normalize; p.floor_ = floor_; p.scale = scale;
  p.route_ids = route_ids; p.route_wts = route_wts;
  p.rows_per_block = rows_per_block; p.out_rows = out_rows; p.zero = 0u;
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (threads < 32 * rows_per_block) threads = 32 * rows_per_block;       // whole warps a row
  // A decode step's router: one block a row would pull all of the router's weights through one SM (256 KB for 32
  // experts of 2048: a third of the kernel's time). A cluster of CTAs a row shares them out; every CTA of the cluster
  // puts the row together for itself, which a step of many rows no longer pays (measured: 2.415 -> 2.374 ms a step at
  // batch 8, 773 -> 797 tok/s at batch 1, but 13.2 k -> 12.5 k tok/s at batch 64). Above 16 rows the cluster shrinks so
  // that all CTAs still run at once, one an SM (37 rows x 4, 74 rows x 2: 8119 -> 8246 tok/s at batch 32, 13.2 k -> 13.5 k
  // at batch 64).
  p.split = 1;
  if (rows_per_block == 1 && router_w && E >= 16 && (hidden & 3) == 0)
    p.split = out_rows <= ROUTER_SPLIT_ROWS ? ROUTER_SPLIT : (out_rows <= 37 ? 4 : (out_rows <= 74 ? 2 : 1));
  const dim3 grid(ceil_div(out_rows, rows_per_block) * p.split);
  const int per = !router_w ? 0 : (E <= 32 ? 1 : (E <= 128 ? 4 : MAX_EXPERTS / 32));
#define TL_NORM1(T_, PER_, ONE_)                                                                                          \
  do {                                                                                                                    \
    if (smem > 48 * 1024)                                                                                                 \
      cudaFuncSetAttribute(add_rmsnorm_kernel<T_, PER_, ONE_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
    if (p.split > 1) return (int)launch_clustered(add_rmsnorm_kernel<T_, PER_, ONE_>, grid, dim3(threads), smem, stream, p.split, p); \
    return (int)launch_chained(add_rmsnorm_kernel<T_, PER_, ONE_>, grid, dim3(threads), smem, stream, p);                 \
  } while (0)
#define TL_NORM(T_, PER_)                          \
  do {                                             \
    if (rows_per_block == 1) TL_NORM1(T_, PER_, true); \
    TL_NORM1(T_, PER_, false);                     \
  } while (0)
  if (dtype == TL_FP32) {
    if (per == 0) TL_NORM(float, 0);
    if (per == 1) TL_NORM(float, 1);
    if (per == 4) TL_NORM(float, 4);
    TL_NORM(float, MAX_EXPERTS / 32);
  }
  if (per == 0) TL_NORM(bf16, 0);
  if (per == 1) TL_NORM(bf16, 1);
  if (per == 4) TL_NORM(bf16, 4);
  TL_NORM(bf16, MAX_EXPERTS / 32);
#undef TL_NORM
#undef TL_NORM1
}

// out [rows, inter] = act(gate_up[:, :inter]) * gate_up[:, inter:], act one of TL_ACT_SILU .. TL_ACT_IDENTITY
extern "C" int tl_gated_mul(const void* gate_up, void* out, int rows, int inter, int act, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && inter > 0, "gated_mul: rows %d width %d", rows, inter);
  TL_REQUIRE(act >= TL_ACT_SILU && act <= TL_ACT_LAST, "gated_mul: gate activation %d is not one of 1..%d", act, TL_ACT_LAST);
  const long long n = (long long)rows * inter;
  const long long most = (long long)sm_count() * 16;
  const int blocks = (int)(ceil_div64(n, 256) < most ? ceil_div64(n, 256) : most);
  cudaError_t e;
  if (dtype == TL_FP32)
    e = launch_chained(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, (float*)out,
                       (long long)rows, inter, act);
  else
    e = launch_chained(silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gate_up, (bf16*)out,
                       (long long)rows, inter, act);
  return (int)e;
}

// Routing of the sigmoid top-k experts: the choice, the expert-sorted plan of (row, slot) pairs with its
// row-tile map, and the weighted combine. Everything stays on the device: no count comes back to the host.
//
//   s = sigmoid(logits); choice by s + expert_bias (bias for the choice only); w = s[chosen]
//   w = w / (sum w + floor) when normalised; w *= scale            engine/models/lfm2_moe/ref.py:185-197
//   ties go to the lower expert id                                  engine/models/lfm2_moe/kernels.py:265-287
//   out[r] = sum over the row's experts in ascending expert id of w * expert(x[r])    ref.py:207-214
//
// The plan is a stable counting sort: pairs keep their row order inside an expert, so the order of every
// sum is fixed by the inputs alone (the only atomics count integers). Two forms build the same plan: for any
// number of pairs, a kernel that counts each chunk of 256 pairs per expert and one that places them; and one
// kernel for up to 4096 pairs (a decode step) that also copies the token rows into expert-sorted order for the
// tensor-core kernels.
#include "route.cuh"

namespace tl {

// one warp per row
__global__ void __launch_bounds__(128) router_topk_kernel(const float* __restrict__ logits, long long ld,
                                                          const float* __restrict__ bias, int rows, int E, int k,
                                                          int normalize, float floor_, float scale,
                                                          int* __restrict__ ids, float* __restrict__ wts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (warp >= rows) return;
  warp_route(logits + (long long)warp * ld, bias, E, k, normalize, floor_, scale, ids + (long long)warp * k,
             wts + (long long)warp * k);
}

constexpr int PLAN_CHUNK = 256;      // pairs a block of the two-kernel plan takes
constexpr int PLAN_WARPS = PLAN_CHUNK / 32;
constexpr int SELF_COUNT_PAIRS = 16384;   // up to here the placing kernel needs no histogram kernel in front

// grid ceil(P / PLAN_CHUNK): block b counts its chunk's pairs per expert into block_hist[b, :]
__global__ void __launch_bounds__(PLAN_CHUNK) moe_hist_kernel(const int* __restrict__ ids, int P, int E,
                                                              int* __restrict__ block_hist) {
  __shared__ int hist[MAX_EXPERTS];
  chain_next();
  chain_wait();
  for (int e = threadIdx.x; e < E; e += PLAN_CHUNK) hist[e] = 0;
  __syncthreads();
  const int p = blockIdx.x * PLAN_CHUNK + threadIdx.x;
  if (p < P) {
    const int e = ids[p];
    if ((unsigned)e < (unsigned)E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += PLAN_CHUNK) block_hist[(long long)blockIdx.x * E + e] = hist[e];
}

// grid ceil(P / PLAN_CHUNK): block b places its chunk's pairs: a pair of expert e lands behind all pairs of lower
// experts, behind the pairs of e in earlier chunks, behind those of e in earlier warps of its own chunk and behind the
// earlier lanes of its own warp, so the sorted list keeps pair order within an expert. Block 0 also writes counts,
// offsets and the row tiles.
__global__ void __launch_bounds__(PLAN_CHUNK) moe_place_kernel(const int* __restrict__ ids, int P, int E, int tile_m,
                                                               const int* __restrict__ block_hist, int* __restrict__ counts,
                                                               int* __restrict__ offsets, int* __restrict__ sorted_pairs,
                                                               int* __restrict__ pos_of_pair, int* __restrict__ tile_group,
                                                               int* __restrict__ tile_row0, int* __restrict__ tile_rows,
                                                               int* __restrict__ n_tiles) {
  __shared__ int total[MAX_EXPERTS];                  // pairs of each expert in all chunks
  __shared__ int base[MAX_EXPERTS];                   // where this chunk's first pair of each expert lands
  __shared__ int in_warp[PLAN_WARPS][MAX_EXPERTS];    // pairs of each expert in each warp of this chunk, then the sums before each warp
  chain_next();
  chain_wait();
  const int b = blockIdx.x, nb = gridDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int w = 0; w < PLAN_WARPS; ++w)
    for (int e = tid; e < E; e += PLAN_CHUNK) in_warp[w][e] = 0;
  if (block_hist) {
    for (int e = tid; e < E; e += PLAN_CHUNK) {
      int all = 0, before = 0;
      for (int i = 0; i < nb; ++i) {
        const int v = block_hist[(long long)i * E + e];
        all += v;
        if (i < b) before += v;
      }
      total[e] = all;
      base[e] = before;
    }
  } else {
    // No histograms from a kernel in front (a moderate number of pairs): the block counts all pairs itself, those of the
    // chunks before its own into base, the others into total.
    for (int e = tid; e < E; e += PLAN_CHUNK) total[e] = base[e] = 0;
    __syncthreads();
    const int mine = b * PLAN_CHUNK;
    constexpr int BATCH = 16;                       // loads of a thread that are sent before the first is counted
    for (int i0 = 0; i0 < P; i0 += BATCH * PLAN_CHUNK) {
      int v[BATCH];
#pragma unroll
      for (int j = 0; j < BATCH; ++j) {
        const int i = i0 + j * PLAN_CHUNK + tid;
        v[j] = i < P ? ids[i] : -1;
      }
#pragma unroll
      for (int j = 0; j < BATCH; ++j)
        if ((unsigned)v[j] < (unsigned)E) atomicAdd(i0 + j * PLAN_CHUNK < mine ? &base[v[j]] : &total[v[j]], 1);
    }
    __syncthreads();
    for (int e = tid; e < E; e += PLAN_CHUNK) total[e] += base[e];
  }
  __syncthreads();
  const int p = b * PLAN_CHUNK + tid;
  int e = p < P ? ids[p] : -1;
  if ((unsigned)e >= (unsigned)E) e = -1;
  const bool hit = e >= 0;
  const unsigned hits = __ballot_sync(0xffffffffu, hit);
  unsigned same = 0;
  if (hit) {
    same = __match_any_sync(hits, e);
    if (lane == __ffs(same) - 1) in_warp[warp][e] = __popc(same);
  }
  __syncthreads();
  for (int x = tid; x < E; x += PLAN_CHUNK) {
    int lower = 0;
    for (int i = 0; i < x; ++i) lower += total[i];
    base[x] += lower;
    int run = 0;                                     // pairs of x in this chunk's earlier warps
    for (int w = 0; w < PLAN_WARPS; ++w) {
      const int c = in_warp[w][x];
      in_warp[w][x] = run;
      run += c;
    }
    if (b == 0) {
      counts[x] = total[x];
      offsets[x] = lower;
      if (x == E - 1) offsets[E] = lower + total[x];
      // the expert's row tiles come behind those of the experts before it
      int tiles = 0;
      for (int i = 0; i < x; ++i) tiles += (total[i] + tile_m - 1) / tile_m;
      const int cnt = total[x];
      for (int t = 0; t * tile_m < cnt; ++t, ++tiles) {
        tile_group[tiles] = x;
        tile_row0[tiles] = lower + t * tile_m;
        tile_rows[tiles] = min(tile_m, cnt - t * tile_m);
      }
      if (x == E - 1) *n_tiles = tiles;
    }
  }
  __syncthreads();
  if (hit) {
    const int at = base[e] + in_warp[warp][e] + __popc(same & ((1u << lane) - 1u));
    sorted_pairs[at] = p;
    pos_of_pair[p] = at;
  }
}

// The one-kernel form below does work that grows with the square of the pairs (every block reads all ids): measured, it
// costs 8 us at 256 pairs, 24 us at 2048 and 41 us at 4096, where the chunked form and a kernel that copies the rows take
// 17 us together at 8192. It is the form of decode steps and short portions.
constexpr int SMALL_PLAN_PAIRS = 1024;

// grid P (one block per pair), 128 threads: block p finds where pair p lands in the expert-sorted order (pairs of
// lower experts first, then earlier pairs of its own expert), records it, and copies the pair's token row there.
// Block 0 also writes the counts, offsets and row tiles.
__global__ void __launch_bounds__(128) moe_plan_small_kernel(const int* __restrict__ ids, int P, int E, int tile_m, int top_k,
                                                             int* __restrict__ counts, int* __restrict__ offsets,
                                                             int* __restrict__ sorted_pairs, int* __restrict__ pos_of_pair,
                                                             int* __restrict__ tile_group, int* __restrict__ tile_row0,
                                                             int* __restrict__ tile_rows, int* __restrict__ n_tiles,
                                                             const bf16* __restrict__ x, long long ldx,
                                                             bf16* __restrict__ x_sorted, int width) {
  __shared__ int s_ids[SMALL_PLAN_PAIRS];
  __shared__ float scratch[33];
  __shared__ int s_counts[MAX_EXPERTS];
  chain_next();
  chain_wait();
  const int p = blockIdx.x, tid = threadIdx.x;
  for (int i = tid; i < P; i += 128) s_ids[i] = ids[i];
  __syncthreads();
  const int e = s_ids[p];
  int n = 0;
  for (int i = tid; i < P; i += 128) n += (s_ids[i] < e) || (s_ids[i] == e && i < p);
  const int at = (int)(block_sum((float)n, scratch) + 0.5f);
  if (tid == 0) {
    sorted_pairs[at] = p;
    pos_of_pair[p] = at;
  }
  if (x) {
    const uint4* src = (const uint4*)(x + (long long)(p / top_k) * ldx);
    uint4* dst = (uint4*)(x_sorted + (long long)at * width);
    for (int c = tid; c < width / 8; c += 128) dst[c] = src[c];
  }
  if (p != 0) return;
  for (int ex = tid; ex < E; ex += 128) {
    int cnt = 0;
    for (int i = 0; i < P; ++i) cnt += s_ids[i] == ex;
    s_counts[ex] = cnt;
    counts[ex] = cnt;
  }
  __syncthreads();
  // a thread an expert: its pairs and row tiles come behind those of the experts before it
  for (int ex = tid; ex < E; ex += 128) {
    int off = 0, tiles = 0;
    for (int i = 0; i < ex; ++i) {
      off += s_counts[i];
      tiles += (s_counts[i] + tile_m - 1) / tile_m;
    }
    offsets[ex] = off;
    const int cnt = s_counts[ex];
    for (int t = 0; t * tile_m < cnt; ++t, ++tiles) {
      tile_group[tiles] = ex;
      tile_row0[tiles] = off + t * tile_m;
      tile_rows[tiles] = min(tile_m, cnt - t * tile_m);
    }
    if (ex == E - 1) {
      offsets[E] = off + cnt;
      *n_tiles = tiles;
    }
  }
}

// The same plan for at most WARP_PLAN_PAIRS pairs (a decode step of a few rows) by one warp, a pair or two a lane: no
// shared memory and no barrier, because this kernel is a link in the chain of a step whose kernels each take a few
// microseconds. A lane finds its pairs' places by looking at every lane's experts; then the experts are taken 32 at a
// time, an expert a lane, counted the same way and summed up over the lanes for the offsets and the tiles.
constexpr int WARP_PLAN_PAIRS = 64;
__global__ void __launch_bounds__(32) moe_plan_warp_kernel(const int* __restrict__ ids, int P, int E, int tile_m,
                                                           int* __restrict__ counts, int* __restrict__ offsets,
                                                           int* __restrict__ sorted_pairs, int* __restrict__ pos_of_pair,
                                                           int* __restrict__ tile_group, int* __restrict__ tile_row0,
                                                           int* __restrict__ tile_rows, int* __restrict__ n_tiles) {
  chain_next();
  chain_wait();
  const int lane = threadIdx.x;
  constexpr int PER = WARP_PLAN_PAIRS / 32;             // pair lane + 32 q is this lane's q-th
  int e[PER], at[PER];
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    e[q] = lane + 32 * q < P ? ids[lane + 32 * q] : 0x7fffffff;
    at[q] = 0;
  }
#pragma unroll
  for (int qj = 0; qj < PER; ++qj) {
    const int n = min(32, P - 32 * qj);
    for (int j = 0; j < n; ++j) {
      const int ej = __shfl_sync(0xffffffffu, e[qj], j), pj = j + 32 * qj;
#pragma unroll
      for (int q = 0; q < PER; ++q) at[q] += (ej < e[q]) || (ej == e[q] && pj < lane + 32 * q);
    }
  }
#pragma unroll
  for (int q = 0; q < PER; ++q)
    if (lane + 32 * q < P) {
      sorted_pairs[at[q]] = lane + 32 * q;
      pos_of_pair[lane + 32 * q] = at[q];
    }
  int off_before = 0, tiles_before = 0;                 // over the experts of the groups of 32 already done
  for (int e0 = 0; e0 < E; e0 += 32) {
    const int ex = e0 + lane;
    int cnt = 0;
#pragma unroll
    for (int qj = 0; qj < PER; ++qj) {
      const int n = min(32, P - 32 * qj);
      for (int j = 0; j < n; ++j) cnt += __shfl_sync(0xffffffffu, e[qj], j) == ex;
    }
    const int tl = (cnt + tile_m - 1) / tile_m;
    int off = cnt, tiles = tl;                          // inclusive sums over the lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, off, o), b = __shfl_up_sync(0xffffffffu, tiles, o);
      if (lane >= o) {
        off += a;
        tiles += b;
      }
    }
    const int off_all = __shfl_sync(0xffffffffu, off, 31), tiles_all = __shfl_sync(0xffffffffu, tiles, 31);
    off += off_before - cnt;                            // exclusive, over all experts before this one
    tiles += tiles_before - tl;
    if (ex < E) {
      counts[ex] = cnt;
      offsets[ex] = off;
      for (int t = 0; t < tl; ++t) {
        tile_group[tiles + t] = ex;
        tile_row0[tiles + t] = off + t * tile_m;
        tile_rows[tiles + t] = min(tile_m, cnt - t * tile_m);
      }
    }
    off_before += off_all;
    tiles_before += tiles_all;
  }
  if (lane == 0) {
    offsets[E] = off_before;
    *n_tiles = tiles_before;
  }
}

// one block per row: out[r, :] = sum over the row's slots in ascending expert id of wts * y[pos_of_pair]  (32-bit)
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos_of_pair,
                                                          const int* __restrict__ ids, const float* __restrict__ wts,
                                                          float* __restrict__ out, int hidden, int k) {
  __shared__ int s_src[MAX_TOP_K];
  __shared__ float s_w[MAX_TOP_K];
  const int r = blockIdx.x;
  if (threadIdx.x == 0) {
    int order[MAX_TOP_K];
    for (int j = 0; j < k; ++j) {       // insertion sort of the slots by expert id (slot index breaks ties)
      int i = j;
      const int e = ids[(long long)r * k + j];
      while (i > 0 && ids[(long long)r * k + order[i - 1]] > e) {
        order[i] = order[i - 1];
        --i;
      }
      order[i] = j;
    }
    for (int j = 0; j < k; ++j) {
      s_src[j] = pos_of_pair[(long long)r * k + order[j]];
      s_w[j] = wts[(long long)r * k + order[j]];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < k; ++j) acc = fmaf(s_w[j], y[(long long)s_src[j] * hidden + c], acc);
    out[(long long)r * hidden + c] = acc;
  }
}

}  // namespace tl

using namespace tl;

extern "C" int tl_router_topk(const float* logits, long long ld, const float* bias, int rows, int E, int k,
                              int normalize, float floor_, float scale, int* ids, float* wts, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(E > 0 && E <= MAX_EXPERTS, "router: %d experts; up to %d are implemented", E, MAX_EXPERTS);
  TL_REQUIRE(k > 0 && k <= E && k <= MAX_TOP_K, "router: top-%d of %d experts; up to top-%d is implemented", k, E,
             MAX_TOP_K);
  TL_REQUIRE(ld >= E, "router: row stride %lld for %d experts", ld, E);
  TL_REQUIRE(normalize >= 0 && (normalize >> 1) <= TL_SCORE_LAST, "router: scoring function %d is not one of 0..%d",
             normalize >> 1, TL_SCORE_LAST);
  router_topk_kernel<<<ceil_div(rows, 4), 128, 0, stream>>>(logits, ld, bias, rows, E, k, normalize, floor_, scale, ids,
                                                            wts);
  TL_LAUNCH_CHECK();
  return 0;
}

// Upper bound on the row tiles of any plan over `pairs` pairs and E experts with tiles of tile_m rows.
extern "C" int tl_moe_max_tiles(int pairs, int E, int tile_m) {
  const int by_rows = ceil_div(pairs, tile_m) + E;
  return by_rows < pairs ? by_rows : (pairs > 0 ? pairs : 1);
}

// Builds the plan of `pairs` (row, slot) pairs. With `x` (bfloat16 rows [pairs / top_k, width], stride ldx) it also
// writes x_sorted[i] = x[sorted_pairs[i] / top_k]. Returns the number of kernels it launched through *launched.
// 1 when tl_moe_plan runs its one-kernel form for these sizes, the form that also copies the token rows it is given
extern "C" int tl_moe_plan_copies_rows(int pairs, int E) { return pairs > 0 && pairs <= SMALL_PLAN_PAIRS && E <= MAX_EXPERTS; }

extern "C" int tl_moe_plan(const int* ids, int pairs, int E, int tile_m, int top_k, int* counts, int* offsets,
                           int* sorted_pairs, int* pos_of_pair, int* tile_group, int* tile_row0, int* tile_rows,
                           int* n_tiles, int* block_hist, const void* x, long long ldx, void* x_sorted, int width,
                           int* launched, cudaStream_t stream) {
  TL_REQUIRE(E > 0 && E <= 65535 && tile_m > 0 && top_k > 0, "moe plan: %d experts, tile of %d rows, top-%d", E, tile_m, top_k);
  TL_REQUIRE(pairs >= 0 && pairs < (1 << 24), "moe plan: %d pairs; fewer than 2^24 are implemented", pairs);
  TL_REQUIRE(!x || (width % 8 == 0 && ldx % 8 == 0 && x_sorted), "moe plan: row copy of width %d, stride %lld", width, ldx);
  if (launched) *launched = 0;
  if (pairs == 0) return 0;
  if (pairs <= WARP_PLAN_PAIRS && !x && E <= MAX_EXPERTS) {
    cudaError_t e = launch_chained(moe_plan_warp_kernel, dim3(1), dim3(32), 0, stream, ids, pairs, E, tile_m, counts, offsets,
                                   sorted_pairs, pos_of_pair, tile_group, tile_row0, tile_rows, n_tiles);
    if (e != cudaSuccess) return (int)e;
    if (launched) *launched = 1;
    return 0;
  }
  if (pairs <= SMALL_PLAN_PAIRS && E <= MAX_EXPERTS) {
    cudaError_t e = launch_chained(moe_plan_small_kernel, dim3(pairs), dim3(128), 0, stream, ids, pairs, E, tile_m, top_k,
                                   counts, offsets, sorted_pairs, pos_of_pair, tile_group, tile_row0, tile_rows, n_tiles,
                                   (const bf16*)x, ldx, (bf16*)x_sorted, width);
    if (e != cudaSuccess) return (int)e;
    if (launched) *launched = 1;
    return 0;
  }
  TL_REQUIRE(E <= MAX_EXPERTS && block_hist, "moe plan: %d experts; up to %d are implemented", E, MAX_EXPERTS);
  const int chunks = ceil_div(pairs, PLAN_CHUNK);
  // up to SELF_COUNT_PAIRS every placing block counts all pairs itself (64 passes of its 256 threads at most): one kernel
  const bool self_count = pairs <= SELF_COUNT_PAIRS;
  cudaError_t e = cudaSuccess;
  if (!self_count)
    e = launch_chained(moe_hist_kernel, dim3(chunks), dim3(PLAN_CHUNK), 0, stream, ids, pairs, E, block_hist);
  if (e != cudaSuccess) return (int)e;
  e = launch_chained(moe_place_kernel, dim3(chunks), dim3(PLAN_CHUNK), 0, stream, ids, pairs, E, tile_m,
                     self_count ? (const int*)nullptr : (const int*)block_hist, counts, offsets, sorted_pairs, pos_of_pair,
                     tile_group, tile_row0, tile_rows, n_tiles);
  if (e != cudaSuccess) return (int)e;
  if (launched) *launched = self_count ? 1 : 2;
  return 0;
}

extern "C" int tl_moe_combine(const float* y, const int* pos_of_pair, const int* ids, const float* wts, float* out,
                              int rows, int hidden, int k, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(k > 0 && k <= MAX_TOP_K && hidden > 0, "moe combine: top-%d, hidden %d", k, hidden);
  moe_combine_kernel<<<rows, 256, 0, stream>>>(y, pos_of_pair, ids, wts, out, hidden, k);
  TL_LAUNCH_CHECK();
  return 0;
}

// bfloat16 products of a few token rows with a weight matrix of moderate size, for decode steps:
//
//   C[m, n] = sum_k X[m, k] * W[n, k] (+ bias[n])       m < 32 tokens; X, W row-major with k contiguous
//
// At these sizes (a mixer's projections: some MB of weights, a handful of tokens) a product's time is the length
// of its chain of dependent steps, not its bytes, so this kernel has the shortest chain there is: no shared-memory
// staging, no barriers, no tensor memory. A CTA of eight warps owns 16 weight rows. Every lane loads 16 bytes of
// two of those rows and 16 bytes of one token row straight from global memory into the registers that
// mma.sync m16n8k16 wants (the weights as the A operand, the tokens as B), many loads in flight, and the eight
// warps split k between them, chunk by chunk of 32. Because a dot product does not care about the order of k,
// the 8 consecutive elements a lane holds feed two MMAs whose k slots are mapped to those elements the same way
// for both operands. The warps' 32-bit partial tiles are added in warp order through shared memory, so the result
// does not depend on timing. (The reference sends every product through one `lin`,
// engine/models/lfm2_moe/ref.py:99-103; this is the decode-step form of it.)
#include "common.cuh"

namespace tl {

constexpr int SKINNY_WARPS = 8;
constexpr int SKINNY_MAX_TOKENS = 32;

__device__ __forceinline__ void mma_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16 bytes through the read-only path, zeros when not valid. Volatile, so that the compiler keeps a round's loads in
// front of its MMAs, all in flight together, instead of moving each load next to its use to save registers.
__device__ __forceinline__ uint4 load16(const bf16* p, bool valid) {
  uint4 v;
  asm volatile(
      "{\n\t.reg .pred ok;\n\t"
      "setp.ne.b32 ok, %5, 0;\n\t"
      "mov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;\n\t"
      "@ok ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];\n\t}"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p), "r"((int)valid));
  return v;
}

// NT: token tiles of 8 (M <= 8 NT). UNROLL chunks of 32 k-elements are in flight a warp: with eight, a k of 2048
// is one round of loads, all issued before the first is used.
template <int NT, typename TOut>
__global__ void __launch_bounds__(SKINNY_WARPS * 32) gemm_skinny_mma_kernel(
    const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ w, long long ldw, const float* __restrict__ bias,
    TOut* __restrict__ out, long long ldc, int M, int N, int K, uint32_t zero) {
  constexpr int UNROLL = NT == 1 ? 8 : (NT == 2 ? 4 : 2);
  __shared__ float part[SKINNY_WARPS][NT][16][8 + 1];
  chain_next();
  chain_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int r_lo = n0 + g, r_hi = n0 + g + 8;                     // this lane's two weight rows
  const bool v_lo = r_lo < N, v_hi = r_hi < N;
  const bf16* w_lo = w + (long long)(v_lo ? r_lo : 0) * ldw + t * 8;
  const bf16* w_hi = w + (long long)(v_hi ? r_hi : 0) * ldw + t * 8;
  const bf16* x_row[NT];
  bool x_ok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int m = j * 8 + g;                                      // this lane's token of tile j
    x_ok[j] = m < M;
    x_row[j] = x + (long long)(x_ok[j] ? m : 0) * ldx + t * 8;
  }
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  const int chunks = (K + 31) / 32;
  // chunk c belongs to warp c % 8; a lane's 8 elements of a chunk start at k = 32 c + 8 t
  for (int c0 = warp; c0 < chunks; c0 += SKINNY_WARPS * UNROLL) {
    uint4 a_lo[UNROLL], a_hi[UNROLL], b[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int c = c0 + u * SKINNY_WARPS;
      const int k = c * 32 + t * 8;
      const bool in = c < chunks && k < K;                        // K is a multiple of 8: 8 elements are in or out
      a_lo[u] = load16(w_lo + c * 32, in && v_lo);
      a_hi[u] = load16(w_hi + c * 32, in && v_hi);
#pragma unroll
      for (int j = 0; j < NT; ++j) b[u][j] = load16(x_row[j] + c * 32, in && x_ok[j]);
    }
    // The round's first MMA is made to wait for the round's last loads: otherwise the compiler moves every MMA up
    // to just behind its own loads, and the warp, which issues in order, stalls there with most loads not yet sent.
    // (`zero` is 0, which only the host knows: the compiler can neither drop the term nor the dependence it carries)
    a_lo[0].x ^= (a_lo[UNROLL - 1].w ^ a_hi[UNROLL - 1].w ^ b[UNROLL - 1][NT - 1].w) & zero;
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        mma_16816(acc[j], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, b[u][j].x, b[u][j].y);
        mma_16816(acc[j], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, b[u][j].z, b[u][j].w);
      }
    }
  }
  // acc[j]: (row g, tokens 8 j + 2 t, + 1), (row g + 8, the same tokens)
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    part[warp][j][g][2 * t] = acc[j][0];
    part[warp][j][g][2 * t + 1] = acc[j][1];
    part[warp][j][g + 8][2 * t] = acc[j][2];
    part[warp][j][g + 8][2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  // 16 rows x 8 NT tokens: a thread takes one row of one token, consecutive threads consecutive rows
  for (int i = threadIdx.x; i < 16 * 8 * NT; i += SKINNY_WARPS * 32) {
    const int row = i & 15, m = i >> 4;
    const int n = n0 + row;
    if (m >= M || n >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int s = 0; s < SKINNY_WARPS; ++s) v += part[s][m >> 3][row][m & 7];
    if (bias) v += bias[n];
    out[(long long)m * ldc + n] = from_f32<TOut>(v);
  }
}


// The same for the routed experts of a small step (a dozen rows): grid (ceil(N / 16), plan tiles), a CTA takes
// 16 outputs of one tile's expert for the tile's token rows (at most 8: the plan is built with tiles of 8). With SWIGLU
// it multiplies by the expert's gate rows and up rows of those outputs and stores silu(gate) * up. Token rows are
// fetched through `row_index` (position i of the plan stands for row row_index[i] / row_div of x) or, without it, lie
// in the plan's order. Tiles past *n_tiles exit at once. Without a plan (`pair_group`: the group of each of n_pairs <= 256
// pairs, tile_* null) out row p is pair p, x row p / row_div, and the CTAs find each group's pairs themselves: up to 32 pairs,
// tile j is the j-th group to appear; more, tile p is pair p and the CTA of a group's first pair takes the group. A few experts' weights are all such a step reads: many small
// CTAs that start at once stream them faster than the few 128-row CTAs of the tcgen05 product.
// the position of the n-th (from 0) set bit of m, which has more than n bits set
__device__ __forceinline__ int nth_set_bit(uint32_t m, int n) {
  for (int i = 0; i < n; ++i) m &= m - 1;
  return __ffs(m) - 1;
}

template <bool SWIGLU, typename TOut>
__global__ void __launch_bounds__(SKINNY_WARPS * 32) gemm_skinny_grouped_kernel(
    const bf16* __restrict__ x, long long ldx, const int* __restrict__ row_index, int row_div, const bf16* __restrict__ w,
    long long ldw, long long rows_per_group, TOut* __restrict__ out, long long ldc, int N, int K,
    const int* __restrict__ tile_group, const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
    const int* __restrict__ n_tiles, const int* __restrict__ pair_group, int n_pairs, int n_groups,
    int* __restrict__ status, int act, uint32_t zero) {
  constexpr int W_TILES = SWIGLU ? 2 : 1;
  constexpr int UNROLL = SWIGLU ? 4 : 8;
  __shared__ float part[SKINNY_WARPS][W_TILES][16][8 + 1];
  __shared__ uint32_t s_match[SKINNY_WARPS];
  __shared__ int s_pair[8];
  chain_next();
  chain_wait();
  const int tile = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  int rows, group, pos_known = -1;
  if (pair_group && n_pairs <= 32) {
    // No plan, and the pairs fit a warp: tile j is the j-th group in the order in which the groups first appear among
    // the pairs, so the CTAs that have work are the first of the grid and start together, and those behind them leave.
    // Every warp works this out for itself from the same 32 ids: no shared memory, no barrier in front of the loads.
    const int mine = lane < n_pairs ? pair_group[lane] : -1;
    const bool ok = mine >= 0 && mine < n_groups;
    const uint32_t same = __match_any_sync(0xffffffffu, ok ? mine : -1);      // (pairs without a group match each other only)
    const uint32_t firsts = __ballot_sync(0xffffffffu, ok && lane == __ffs(same) - 1);
    if (tile >= __popc(firsts)) return;
    const int leader = nth_set_bit(firsts, tile);
    group = __shfl_sync(0xffffffffu, mine, leader);
    const uint32_t members = __shfl_sync(0xffffffffu, same, leader);
    rows = __popc(members);
    pos_known = nth_set_bit(members, g < rows ? g : 0);
    if (threadIdx.x < 8) s_pair[threadIdx.x] = nth_set_bit(members, (int)threadIdx.x < rows ? (int)threadIdx.x : 0);
  } else if (pair_group) {
    // No plan: tile p stands for pair p. The CTA of the first pair of a group takes all of the group's pairs (they are
    // at most as many as the step has rows), the CTAs of the group's later pairs have nothing to do.
    group = pair_group[tile];
    const int mine = (int)threadIdx.x < n_pairs ? pair_group[threadIdx.x] : -1;
    const uint32_t match = __ballot_sync(0xffffffffu, mine == group);
    if (lane == 0) s_match[warp] = match;
    __syncthreads();
    if (group < 0 || group >= n_groups) return;
    int before = 0, total = 0;                         // matching pairs before this thread's, and in all
    bool earlier = false;                              // a matching pair before pair `tile`
#pragma unroll
    for (int w2 = 0; w2 < SKINNY_WARPS; ++w2) {
      const uint32_t m = s_match[w2];
      total += __popc(m);
      if (w2 < warp) before += __popc(m);
      const int first = w2 * 32;
      if (first < tile) earlier |= (m & (tile - first >= 32 ? 0xffffffffu : (1u << (tile - first)) - 1u)) != 0u;
    }
    if (earlier) return;
    before += __popc(match & ((1u << lane) - 1u));
    if (mine == group && before < 8) s_pair[before] = threadIdx.x;
    rows = total;
    __syncthreads();
  } else {
    // (every thread reads the tile's three words itself: no barrier stands between them and the loads that follow)
    if (tile >= *n_tiles) return;
    rows = tile_rows[tile];
    group = tile_group[tile];
    const int row0 = tile_row0[tile];
    pos_known = row0 + (g < rows ? g : 0);
    if (threadIdx.x < 8) s_pair[threadIdx.x] = row0 + threadIdx.x;
  }
  if (rows > 8) {                                      // taller tiles than this kernel takes
    if (threadIdx.x == 0) atomicExch(status, 5);
    rows = 8;
  }
  const long long w_base = (long long)group * rows_per_group;
  const int n0 = blockIdx.x * 16;
  const bool v_lo = n0 + g < N, v_hi = n0 + g + 8 < N;
  const bf16* w_lo[W_TILES];
  const bf16* w_hi[W_TILES];
#pragma unroll
  for (int j = 0; j < W_TILES; ++j) {
    const long long first = w_base + (long long)j * N + n0;               // gate rows, then (SWIGLU) the up rows
    w_lo[j] = w + (first + (v_lo ? g : 0)) * ldw + t * 8;
    w_hi[j] = w + (first + (v_hi ? g + 8 : 0)) * ldw + t * 8;
  }
  const bool x_ok = g < rows;
  const int pos = pos_known >= 0 ? pos_known : s_pair[x_ok ? g : 0];
  const bf16* x_row = x + (long long)(row_index ? row_index[pos] / row_div : pos / row_div) * ldx + t * 8;
  float acc[W_TILES][4];
#pragma unroll
  for (int j = 0; j < W_TILES; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  const int chunks = (K + 31) / 32;
  for (int c0 = warp; c0 < chunks; c0 += SKINNY_WARPS * UNROLL) {
    uint4 a_lo[UNROLL][W_TILES], a_hi[UNROLL][W_TILES], b[UNROLL];
    uint32_t all = 0u;
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int c = c0 + u * SKINNY_WARPS;
      const bool in = c < chunks && c * 32 + t * 8 < K;
#pragma unroll
      for (int j = 0; j < W_TILES; ++j) {
        a_lo[u][j] = load16(w_lo[j] + c * 32, in && v_lo);
        a_hi[u][j] = load16(w_hi[j] + c * 32, in && v_hi);
        all ^= a_lo[u][j].w ^ a_hi[u][j].w;
      }
      b[u] = load16(x_row + c * 32, in && x_ok);
      all ^= b[u].w;
    }
    a_lo[0][0].x ^= all & zero;                 // the round's first MMA waits for all of the round's loads (zero is 0)
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
      for (int j = 0; j < W_TILES; ++j) {
        mma_16816(acc[j], a_lo[u][j].x, a_hi[u][j].x, a_lo[u][j].y, a_hi[u][j].y, b[u].x, b[u].y);
        mma_16816(acc[j], a_lo[u][j].z, a_hi[u][j].z, a_lo[u][j].w, a_hi[u][j].w, b[u].z, b[u].w);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < W_TILES; ++j) {
    part[warp][j][g][2 * t] = acc[j][0];
    part[warp][j][g][2 * t + 1] = acc[j][1];
    part[warp][j][g + 8][2 * t] = acc[j][2];
    part[warp][j][g + 8][2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 16 * 8; i += SKINNY_WARPS * 32) {
    const int row = i & 15, m = i >> 4;
    if (m >= rows || n0 + row >= N) continue;
    float v[W_TILES];
#pragma unroll
    for (int j = 0; j < W_TILES; ++j) {
      v[j] = 0.f;
#pragma unroll
      for (int s = 0; s < SKINNY_WARPS; ++s) v[j] += part[s][j][row][m];
    }
    const float r = SWIGLU ? gated(v[0], v[W_TILES - 1], act) : v[0];
    out[(long long)s_pair[m] * ldc + n0 + row] = from_f32<TOut>(r);
  }
}

// The in-projection of a short-convolution mixer and the convolution behind it, for a decode step of at most 8 rows
// (one row a request): w [3 hidden, K] holds the B, C and x rows of every channel. A CTA owns 8 channels: their B and C
// rows are the two halves of one MMA tile, their x rows the lower half of a second. Its epilogue rounds the three sums
// to bfloat16 as the projection alone would, convolves bx = B x with the request's state, writes y = C conv and shifts
// the state: the same bits as the projection kernel above followed by short_conv_decode_kernel (conv.cu), one launch
// less a layer.
constexpr int CONV_MAX_TAPS = 16;
__global__ void __launch_bounds__(SKINNY_WARPS * 32) gemm_skinny_conv_kernel(
    const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ w, long long ldw, const float* __restrict__ proj_bias,
    const float* __restrict__ taps, const float* __restrict__ conv_bias, float* __restrict__ state,
    const int* __restrict__ state_slot, const int* __restrict__ req_of_row, const int* __restrict__ positions,
    bf16* __restrict__ y, int M, int hidden, int K, int n_taps, int write_state, uint32_t zero) {
  constexpr int UNROLL = 4;
  __shared__ float part[SKINNY_WARPS][2][16][8 + 1];
  chain_next();
  chain_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int c0 = blockIdx.x * 8;
  const bool ch_ok = c0 + g < hidden;
  const long long ch = ch_ok ? c0 + g : 0;
  const bf16* w_b = w + ch * ldw + t * 8;
  const bf16* w_c = w + (hidden + ch) * ldw + t * 8;
  const bf16* w_x = w + (2LL * hidden + ch) * ldw + t * 8;
  const bool x_ok = g < M;
  const bf16* x_row = x + (long long)(x_ok ? g : 0) * ldx + t * 8;
  float acc[2][4];
#pragma unroll
  for (int j = 0; j < 2; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  // What the epilogue needs beside the sums does not depend on them: the row's position and state slot, then the state
  // and the taps of its channel. They are asked for behind the first round of weight loads (up to PRE_TAPS taps), so
  // that their round trips run under the product and not after it, at the end of the kernel's chain.
  constexpr int PRE_TAPS = 4;
  const int e_ep = threadIdx.x & 7, m_ep = threadIdx.x >> 3, c_ep = c0 + e_ep;
  const bool ep = threadIdx.x < 64 && m_ep < M && c_ep < hidden;
  const bool pre = n_taps <= PRE_TAPS;
  int pre_pos = 0, pre_slot = 0;
  float pre_old[PRE_TAPS - 1], pre_tap[PRE_TAPS], pre_cb = 0.f;
#pragma unroll
  for (int i = 0; i < PRE_TAPS - 1; ++i) pre_old[i] = 0.f;
#pragma unroll
  for (int i = 0; i < PRE_TAPS; ++i) pre_tap[i] = 0.f;
  const int chunks = (K + 31) / 32;
  for (int k0 = warp; k0 < chunks; k0 += SKINNY_WARPS * UNROLL) {
    uint4 a_b[UNROLL], a_c[UNROLL], a_x[UNROLL], b[UNROLL];
    uint32_t all = 0u;
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int c = k0 + u * SKINNY_WARPS;
      const bool in = c < chunks && c * 32 + t * 8 < K;
      a_b[u] = load16(w_b + c * 32, in && ch_ok);
      a_c[u] = load16(w_c + c * 32, in && ch_ok);
      a_x[u] = load16(w_x + c * 32, in && ch_ok);
      b[u] = load16(x_row + c * 32, in && x_ok);
      all ^= a_b[u].w ^ a_c[u].w ^ a_x[u].w ^ b[u].w;
    }
    if (k0 == warp && ep && pre) {              // behind the first round's loads
      pre_pos = positions[m_ep];
      pre_slot = state_slot[req_of_row[m_ep]];
#pragma unroll
      for (int j = 0; j < PRE_TAPS; ++j)
        if (j < n_taps) pre_tap[j] = taps[(long long)c_ep * n_taps + j];
      if (conv_bias) pre_cb = conv_bias[c_ep];
    }
    a_b[0].x ^= all & zero;                     // the round's first MMA waits for all of the round's loads (zero is 0)
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      mma_16816(acc[0], a_b[u].x, a_c[u].x, a_b[u].y, a_c[u].y, b[u].x, b[u].y);
      mma_16816(acc[0], a_b[u].z, a_c[u].z, a_b[u].w, a_c[u].w, b[u].z, b[u].w);
      mma_16816(acc[1], a_x[u].x, 0u, a_x[u].y, 0u, b[u].x, b[u].y);
      mma_16816(acc[1], a_x[u].z, 0u, a_x[u].w, 0u, b[u].z, b[u].w);
    }
    if (k0 == warp && ep && pre) {              // the slot is here by now: the channel's state
      const float* st0 = state + ((long long)pre_slot * (n_taps - 1)) * hidden + c_ep;
#pragma unroll
      for (int i = 0; i < PRE_TAPS - 1; ++i)
        if (i < n_taps - 1) pre_old[i] = st0[(long long)i * hidden];
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    part[warp][j][g][2 * t] = acc[j][0];
    part[warp][j][g][2 * t + 1] = acc[j][1];
    part[warp][j][g + 8][2 * t] = acc[j][2];
    part[warp][j][g + 8][2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  if (threadIdx.x >= 64) return;
  const int e = threadIdx.x & 7, m = threadIdx.x >> 3;        // channel c0 + e of row m
  const int c = c0 + e;
  if (m >= M || c >= hidden) return;
  float in[3];                                                 // B, C, x as the projection alone would have stored them
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    float v = 0.f;
#pragma unroll
    for (int s = 0; s < SKINNY_WARPS; ++s) v += part[s][j >> 1][e + (j & 1) * 8][m];
    if (proj_bias) v += proj_bias[(long long)j * hidden + c];
    in[j] = to_f32(from_f32<bf16>(v));
  }
  // from here on: short_conv_decode_kernel, line by line
  const float bx = in[0] * in[2];
  const int S = n_taps - 1;
  const int pos = pre ? pre_pos : positions[m];
  float* st = state + ((long long)(pre ? pre_slot : state_slot[req_of_row[m]]) * S) * hidden;
  float old[CONV_MAX_TAPS];
  float sum;
  if (pre) {
#pragma unroll
    for (int s = 0; s < PRE_TAPS - 1; ++s) old[s] = pre_old[s];
    sum = conv_bias ? pre_cb : 0.f;
#pragma unroll
    for (int j = 0; j < PRE_TAPS; ++j) {
      const int back = n_taps - 1 - j;
      if (j >= n_taps || pos - back < 0) continue;       // before the sequence's first token: zero
      float v = bx;
#pragma unroll
      for (int s = 0; s < PRE_TAPS - 1; ++s)
        if (back != 0 && s == S - back) v = pre_old[s];
      sum = fmaf(pre_tap[j], v, sum);
    }
  } else {
#pragma unroll 1
    for (int s = 0; s < S; ++s) old[s] = st[(long long)s * hidden + c];
    sum = conv_bias ? conv_bias[c] : 0.f;
#pragma unroll 1
    for (int j = 0; j < n_taps; ++j) {
      const int back = n_taps - 1 - j;
      if (pos - back < 0) continue;                // before the sequence's first token: zero
      const float v = back == 0 ? bx : old[S - back];
      sum = fmaf(taps[(long long)c * n_taps + j], v, sum);
    }
  }
  y[(long long)m * hidden + c] = from_f32<bf16>(in[1] * sum);
  if (write_state) {
#pragma unroll 1
    for (int s = 0; s + 1 < S; ++s) st[(long long)s * hidden + c] = (pos - (S - (s + 1)) >= 0) ? old[s + 1] : 0.f;
    st[(long long)(S - 1) * hidden + c] = bx;
  }
}

}  // namespace tl

using namespace tl;

extern "C" int tl_gemm_skinny_supported(int M, int N, int K, long long ldx, long long ldw) {
  return M >= 1 && M <= SKINNY_MAX_TOKENS && N >= 1 && K >= 8 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0;
}

// x [M, K] bfloat16 (row stride ldx), w [N, K] bfloat16 (row stride ldw), bias [N] 32-bit or null,
// out [M, N] (row stride ldc) in bfloat16 (out_dtype TL_BF16) or 32-bit. Pointers 16-byte aligned.
extern "C" int tl_gemm_skinny_mma(const void* x, long long ldx, const void* w, long long ldw, const float* bias, void* out,
                                  long long ldc, int M, int N, int K, int out_dtype, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  TL_REQUIRE(tl_gemm_skinny_supported(M, N, K, ldx, ldw), "skinny product: %d tokens x (%d x %d), strides %lld and %lld", M, N,
             K, ldx, ldw);
  TL_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0, "skinny product: operands must be 16-byte aligned (%d)", 0);
  const dim3 grid(ceil_div(N, 16)), block(SKINNY_WARPS * 32);
  const int nt = ceil_div(M, 8);
#define TL_SKINNY(NT_)                                                                                                  \
  do {                                                                                                                  \
    if (out_dtype == TL_FP32)                                                                                           \
      return (int)launch_chained(gemm_skinny_mma_kernel<NT_, float>, grid, block, 0, stream, (const bf16*)x, ldx,       \
                                 (const bf16*)w, ldw, bias, (float*)out, ldc, M, N, K, 0u);                                 \
    return (int)launch_chained(gemm_skinny_mma_kernel<NT_, bf16>, grid, block, 0, stream, (const bf16*)x, ldx,          \
                               (const bf16*)w, ldw, bias, (bf16*)out, ldc, M, N, K, 0u);                                    \
  } while (0)
  if (nt == 1) TL_SKINNY(1);
  if (nt == 2) TL_SKINNY(2);
  if (nt == 3) TL_SKINNY(3);
  TL_SKINNY(4);
#undef TL_SKINNY
}

// The routed experts of a very small step. x [*, K] bfloat16; w [groups * rows_per_group, K] bfloat16 with, per group, N
// rows (or, with swiglu, which is then the gate's activation TL_ACT_*, N gate rows then N up rows); the plan's tiles hold at most 8 rows; out [pairs, N] in the plan's
// order, bfloat16 or 32-bit. row_index (or null) and row_div as in the kernel's comment.
extern "C" int tl_gemm_skinny_grouped(const void* x, long long ldx, const int* row_index, int row_div, const void* w,
                                      long long ldw, long long rows_per_group, void* out, long long ldc, int N, int K,
                                      int swiglu, int out_dtype, const int* tile_group, const int* tile_row0,
                                      const int* tile_rows, const int* n_tiles, int max_tiles, const int* pair_group,
                                      int n_pairs, int n_groups, int* status, cudaStream_t stream) {
  if (pair_group) max_tiles = n_pairs;
  if (max_tiles == 0 || N == 0) return 0;
  TL_REQUIRE(N >= 1 && K >= 8 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && row_div >= 1 && max_tiles <= 65535,
             "skinny grouped product: %d outputs, k %d, strides %lld and %lld", N, K, ldx, ldw);
  TL_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 &&
                 (pair_group ? (n_pairs <= SKINNY_WARPS * 32 && n_groups >= 1 && !row_index)
                             : (tile_group && tile_row0 && tile_rows && n_tiles)),
             "skinny grouped product: operands must be 16-byte aligned and the plan complete, or at most %d pairs given",
             SKINNY_WARPS * 32);
  TL_REQUIRE(swiglu >= 0 && swiglu <= TL_ACT_LAST, "skinny grouped product: gate activation %d is not one of 0..%d", swiglu,
             TL_ACT_LAST);
  const dim3 grid(ceil_div(N, 16), max_tiles), block(SKINNY_WARPS * 32);
#define TL_GROUPED(SW_, T_)                                                                                              \
  return (int)launch_chained(gemm_skinny_grouped_kernel<SW_, T_>, grid, block, 0, stream, (const bf16*)x, ldx, row_index,  \
                             row_div, (const bf16*)w, ldw, rows_per_group, (T_*)out, ldc, N, K, tile_group, tile_row0,    \
                             tile_rows, n_tiles, pair_group, n_pairs, n_groups, status, swiglu, 0u)
  if (swiglu) {
    if (out_dtype == TL_FP32) TL_GROUPED(true, float);
    TL_GROUPED(true, bf16);
  }
  if (out_dtype == TL_FP32) TL_GROUPED(false, float);
  TL_GROUPED(false, bf16);
#undef TL_GROUPED
}

// in-projection + short convolution of a decode step of at most 8 rows (one row a request): x [M, K] bfloat16,
// w [3 hidden, K] bfloat16 (B rows, C rows, x rows), proj_bias [3 hidden] or null, taps [hidden, n_taps] 32-bit,
// conv_bias [hidden] or null, state [slots, n_taps - 1, hidden] 32-bit, y [M, hidden] bfloat16.
extern "C" int tl_gemm_skinny_conv(const void* x, long long ldx, const void* w, long long ldw, const float* proj_bias,
                                   const float* taps, const float* conv_bias, float* state, const int* state_slot,
                                   const int* req_of_row, const int* positions, void* y, int M, int hidden, int K,
                                   int n_taps, int write_state, cudaStream_t stream) {
  if (M == 0) return 0;
  TL_REQUIRE(M >= 1 && M <= 8 && hidden >= 1 && K >= 8 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0,
             "skinny in-projection + conv: %d rows, %d channels, k %d, strides %lld and %lld", M, hidden, K, ldx, ldw);
  TL_REQUIRE(n_taps >= 2 && n_taps <= CONV_MAX_TAPS && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0,
             "skinny in-projection + conv: %d taps (2..%d), operands 16-byte aligned", n_taps, CONV_MAX_TAPS);
  const dim3 grid(ceil_div(hidden, 8)), block(SKINNY_WARPS * 32);
  return (int)launch_chained(gemm_skinny_conv_kernel, grid, block, 0, stream, (const bf16*)x, ldx, (const bf16*)w, ldw,
                             proj_bias, taps, conv_bias, state, state_slot, req_of_row, positions, (bf16*)y, M, hidden, K,
                             n_taps, write_state, 0u);
}

// Matrix products on the CUDA cores with 32-bit accumulation: the true 32-bit path of every projection
// (no tensor-core and no reduced-precision mode is involved), and a plain fallback for bfloat16 inputs.
//
//   C[m, n] = sum_k A[m, k] * W[n, k] (+ bias[n])            both operands row-major with k contiguous
//
// Each output element is accumulated over k = 0..K-1 in ascending order by one thread, so a row's result
// does not depend on how many other rows the call has (the reference's row invariance,
// engine/models/lfm2_moe/kernels.py:290-306). The same kernel runs the experts: a tile map built on the
// device (moe_route.cu) names, per row tile, the expert whose weights it multiplies by and the rows of
// the expert-sorted pair list it covers; with `swiglu` the epilogue is silu(gate) * up over the two
// halves of the expert's fused [2 I, H] matrix (engine/models/lfm2_moe/ref.py:199-205).
#include "common.cuh"

namespace tl {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

struct GemmParams {
  const void* A;
  const void* W;
  const float* bias;
  void* C;
  long long lda, ldw, ldc, w_group_stride;
  int M, N, K;
  // grouped (nullptr tile_group: plain)
  const int* tile_group;   // [max_tiles] expert of the tile
  const int* tile_row0;    // [max_tiles] first row of the tile in the sorted list
  const int* tile_rows;    // [max_tiles] rows of the tile
  const int* n_tiles;      // [1]
  const int* a_gather;     // [M] or nullptr: A row of sorted row i is a_gather[i] / a_div
  int a_div;
  int swiglu;              // a gate activation TL_ACT_* (1: SiLU): W holds 2 N rows per group; C = act(A W[0:N]^T) * (A W[N:2N]^T)
};

template <typename TIn, typename TOut, bool SWIGLU>
__global__ void __launch_bounds__(256) gemm_tiled_kernel(GemmParams p) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[SWIGLU ? 2 : 1][BK][BN + 4];

  int row0 = blockIdx.y * BM, rows = BM;
  const TIn* W = (const TIn*)p.W;
  if (p.tile_group) {
    const int t = blockIdx.y;
    if (t >= *p.n_tiles) return;
    row0 = p.tile_row0[t];
    rows = p.tile_rows[t];
    W += (long long)p.tile_group[t] * p.w_group_stride;
  } else {
    rows = min(BM, p.M - row0);
  }
  const int col0 = blockIdx.x * BN;
  const TIn* A = (const TIn*)p.A;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;          // thread's 4 columns start at tx*4, 4 rows at ty*4
  const int lr = tid >> 2, lk = (tid & 3) * 4;     // loader: row lr of the tile, k offset lk..lk+3

  // the A row this loader thread reads (-1: out of the tile)
  long long a_row = -1;
  if (lr < rows) {
    const int i = row0 + lr;
    a_row = p.a_gather ? (long long)(p.a_gather[i] / p.a_div) : (long long)i;
  }
  const int w_row = col0 + lr;                      // weight row (output column) this loader thread reads

  float acc[TM][TN];
  float acc2[SWIGLU ? TM : 1][SWIGLU ? TN : 1];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      acc[i][j] = 0.f;
      if constexpr (SWIGLU) acc2[i][j] = 0.f;
    }

  for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      float a = 0.f, w = 0.f, w2 = 0.f;
      if (k < p.K) {
        if (a_row >= 0) a = to_f32(A[a_row * p.lda + k]);
        if (w_row < p.N) {
          w = to_f32(W[(long long)w_row * p.ldw + k]);
          if constexpr (SWIGLU) w2 = to_f32(W[(long long)(w_row + p.N) * p.ldw + k]);
        }
      }
      As[lk + j][lr] = a;
      Ws[0][lk + j][lr] = w;
      if constexpr (SWIGLU) Ws[1][lk + j][lr] = w2;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN], b2[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        b[j] = Ws[0][kk][tx * TN + j];
        if constexpr (SWIGLU) b2[j] = Ws[1][kk][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if constexpr (SWIGLU) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }

  TOut* C = (TOut*)p.C;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int lr_out = ty * TM + i;
    if (lr_out >= rows) continue;
    const long long r = row0 + lr_out;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = col0 + tx * TN + j;
      if (n >= p.N) continue;
      float v = acc[i][j];
      if constexpr (SWIGLU) {
        v = gated(v, acc2[i][j], p.swiglu);
      } else {
        if (p.bias) v += p.bias[n];
      }
      C[r * p.ldc + n] = from_f32<TOut>(v);
    }
  }
}

// Few rows (M <= 8): one warp per output column, lanes stride over k. Weight rows are read once, coalesced.
template <typename TIn, typename TOut, int MAXM>
__global__ void __launch_bounds__(256) gemm_skinny_kernel(GemmParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= p.N) return;
  const TIn* A = (const TIn*)p.A;
  const TIn* w = (const TIn*)p.W + (long long)warp * p.ldw;
  float acc[MAXM];
#pragma unroll
  for (int m = 0; m < MAXM; ++m) acc[m] = 0.f;
  for (int k = lane; k < p.K; k += 32) {
    const float wv = to_f32(w[k]);
#pragma unroll
    for (int m = 0; m < MAXM; ++m)
      if (m < p.M) acc[m] = fmaf(to_f32(A[(long long)m * p.lda + k]), wv, acc[m]);
  }
  TOut* C = (TOut*)p.C;
#pragma unroll
  for (int m = 0; m < MAXM; ++m) {
    if (m >= p.M) break;
    float v = warp_sum(acc[m]);
    if (lane == 0) {
      if (p.bias) v += p.bias[warp];
      C[(long long)m * p.ldc + warp] = from_f32<TOut>(v);
    }
  }
}

// Few rows and few output columns (a router's E x H product): one CTA per output column, its 256 threads stride
// over k and their sums are joined in a fixed order (lanes by shuffles, then the 8 warps in order).
template <typename TIn, typename TOut, int MAXM>
__global__ void __launch_bounds__(256) gemm_skinny_narrow_kernel(GemmParams p) {
  __shared__ float part[8][MAXM];
  const int n = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const TIn* A = (const TIn*)p.A;
  const TIn* w = (const TIn*)p.W + (long long)n * p.ldw;
  float acc[MAXM];
#pragma unroll
  for (int m = 0; m < MAXM; ++m) acc[m] = 0.f;
  for (int k = tid; k < p.K; k += 256) {
    const float wv = to_f32(w[k]);
#pragma unroll
    for (int m = 0; m < MAXM; ++m)
      if (m < p.M) acc[m] = fmaf(to_f32(A[(long long)m * p.lda + k]), wv, acc[m]);
  }
#pragma unroll
  for (int m = 0; m < MAXM; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0) part[warp][m] = v;
  }
  __syncthreads();
  if (tid < p.M) {
    float v = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; ++wi) v += part[wi][tid];
    if (p.bias) v += p.bias[n];
    ((TOut*)p.C)[(long long)tid * p.ldc + n] = from_f32<TOut>(v);
  }
}

// Many rows and few output columns (a router over a prompt portion): a CTA takes 16 rows and all of up to 64
// columns, so that the grid has M / 16 CTAs instead of one column of 64-row tiles. k is walked in order.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) gemm_tall_narrow_kernel(GemmParams p) {
  constexpr int RM = 16, RN = 64, RK = 32;
  __shared__ float As[RK][RM + 1];
  __shared__ float Ws[RK][RN + 1];
  const int tid = threadIdx.x;
  const int row0 = blockIdx.x * RM;
  const int r = tid >> 4, cg = (tid & 15) * 4;
  const TIn* A = (const TIn*)p.A;
  const TIn* W = (const TIn*)p.W;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < p.K; k0 += RK) {
    for (int i = tid; i < RM * RK; i += 256) {
      const int rr = i / RK, kk = i % RK;
      As[kk][rr] = (row0 + rr < p.M && k0 + kk < p.K) ? to_f32(A[(long long)(row0 + rr) * p.lda + k0 + kk]) : 0.f;
    }
    for (int i = tid; i < RN * RK; i += 256) {
      const int nn = i / RK, kk = i % RK;
      Ws[kk][nn] = (nn < p.N && k0 + kk < p.K) ? to_f32(W[(long long)nn * p.ldw + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < RK; ++kk) {
      const float a = As[kk][r];
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] = fmaf(a, Ws[kk][cg + j], acc[j]);
    }
    __syncthreads();
  }
  if (row0 + r < p.M) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = cg + j;
      if (n < p.N) ((TOut*)p.C)[(long long)(row0 + r) * p.ldc + n] = from_f32<TOut>(acc[j] + (p.bias ? p.bias[n] : 0.f));
    }
  }
}

template <typename TIn, typename TOut>
static int launch(const GemmParams& p, int max_tiles, cudaStream_t stream) {
  if (!p.tile_group && !p.swiglu && p.N <= 64 && p.M > 64) {
    gemm_tall_narrow_kernel<TIn, TOut><<<ceil_div(p.M, 16), 256, 0, stream>>>(p);
    return 0;
  }
  if (!p.tile_group && !p.swiglu && p.M <= 8) {
    if (p.N <= 512 && p.K >= 512) {
      gemm_skinny_narrow_kernel<TIn, TOut, 8><<<p.N, 256, 0, stream>>>(p);
      return 0;
    }
    const int blocks = ceil_div(p.N, 8);
    gemm_skinny_kernel<TIn, TOut, 8><<<blocks, 256, 0, stream>>>(p);
    return 0;
  }
  dim3 grid(ceil_div(p.N, BN), p.tile_group ? max_tiles : ceil_div(p.M, BM));
  if (p.swiglu)
    gemm_tiled_kernel<TIn, TOut, true><<<grid, 256, 0, stream>>>(p);
  else
    gemm_tiled_kernel<TIn, TOut, false><<<grid, 256, 0, stream>>>(p);
  return 0;
}

}  // namespace tl

using namespace tl;

// in_dtype / out_dtype: TL_FP32 or TL_BF16 (an fp32 input with a bf16 output is refused).
extern "C" int tl_gemm_simt(const void* A, long long lda, const void* W, long long ldw, const float* bias, void* C,
                            long long ldc, int M, int N, int K, int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  TL_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: M %d N %d K %d", M, N, K);
  TL_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm: strides lda %lld ldw %lld ldc %lld for M %d N %d K %d", lda, ldw,
             ldc, M, N, K);
  TL_REQUIRE(ceil_div(M, BM) <= 65535, "gemm: %d rows exceed the grid limit of %d", M, 65535 * BM);
  GemmParams p = {};
  p.A = A; p.W = W; p.bias = bias; p.C = C; p.lda = lda; p.ldw = ldw; p.ldc = ldc;
  p.M = M; p.N = N; p.K = K; p.a_div = 1;
  if (in_dtype == TL_FP32 && out_dtype == TL_FP32) launch<float, float>(p, 0, stream);
  else if (in_dtype == TL_BF16 && out_dtype == TL_BF16) launch<bf16, bf16>(p, 0, stream);
  else if (in_dtype == TL_BF16 && out_dtype == TL_FP32) launch<bf16, float>(p, 0, stream);
  else TL_REQUIRE(false, "gemm: input dtype %d with output dtype %d is not implemented", in_dtype, out_dtype);
  TL_LAUNCH_CHECK();
  return 0;
}

// Grouped product over the expert-sorted pair list. Sorted row i multiplies A row (a_gather ? a_gather[i] / a_div : i)
// by the weights of its tile's expert and writes C row i.
extern "C" int tl_gemm_simt_grouped(const void* A, long long lda, const int* a_gather, int a_div, const void* W,
                                    long long ldw, long long w_group_stride, void* C, long long ldc, int n_sorted_rows,
                                    int N, int K, const int* tile_group, const int* tile_row0, const int* tile_rows,
                                    const int* n_tiles, int max_tiles, int swiglu, int in_dtype, int out_dtype,
                                    cudaStream_t stream) {
  if (n_sorted_rows == 0 || N == 0) return 0;
  TL_REQUIRE(n_sorted_rows > 0 && N > 0 && K > 0 && max_tiles > 0, "grouped gemm: rows %d N %d K %d tiles %d",
             n_sorted_rows, N, K, max_tiles);
  TL_REQUIRE(max_tiles <= 65535, "grouped gemm: %d row tiles exceed the grid limit", max_tiles);
  TL_REQUIRE(a_div >= 1, "grouped gemm: a_div %d", a_div);
  GemmParams p = {};
  p.A = A; p.W = W; p.bias = nullptr; p.C = C; p.lda = lda; p.ldw = ldw; p.ldc = ldc;
  p.w_group_stride = w_group_stride; p.M = n_sorted_rows; p.N = N; p.K = K;
  p.tile_group = tile_group; p.tile_row0 = tile_row0; p.tile_rows = tile_rows; p.n_tiles = n_tiles;
  p.a_gather = a_gather; p.a_div = a_div; p.swiglu = swiglu;
  if (in_dtype == TL_FP32 && out_dtype == TL_FP32) launch<float, float>(p, max_tiles, stream);
  else if (in_dtype == TL_BF16 && out_dtype == TL_BF16) launch<bf16, bf16>(p, max_tiles, stream);
  else if (in_dtype == TL_BF16 && out_dtype == TL_FP32) launch<bf16, float>(p, max_tiles, stream);
  else TL_REQUIRE(false, "grouped gemm: input dtype %d with output dtype %d is not implemented", in_dtype, out_dtype);
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_gemm_simt_tile_rows() { return BM; }

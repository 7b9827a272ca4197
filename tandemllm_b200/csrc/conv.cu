// The double-gated causal depthwise short convolution over a mixed batch, and its per-request state.
//
//   bcx = in_proj(n)  [R, 3H]:  B = bcx[:, :H], C = bcx[:, H:2H], x = bcx[:, 2H:]
//   bx  = B * x;  conv_t = sum_j taps[:, j] * win_t[j]  (+ bias),  win_t = the K inputs ending at row t, oldest first
//   y   = C * conv                                         (engine/models/lfm2_moe/ref.py:134-151)
//   state after the step = the last K-1 inputs bx of the sequence  (ref.py:253)
//
// A request's rows in this step are consecutive. An input that lies before the step's first row comes
// from the request's state slot (the K-1 inputs before the step, oldest first, 32-bit); an input before
// position 0 of the sequence is zero whatever the slot holds. bx is formed in 32-bit from the stored
// bcx in both cases, so a row's result does not depend on where the prompt was cut.
// The state is rewritten by a second kernel after every row has read it. A step of single rows (decoding) runs one
// kernel that does both.
#include "common.cuh"

namespace tl {

constexpr int MAX_TAPS = 16;

// V consecutive elements as 32-bit values, with 16-byte accesses for V = 8
template <typename T, int V> __device__ __forceinline__ void load_run(const T* __restrict__ p, float* out) {
  if constexpr (V == 8 && sizeof(T) == 2) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  } else if constexpr (V == 8) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = to_f32(p[i]);
  }
}

template <typename T, int V> __device__ __forceinline__ void store_run(T* __restrict__ p, const float* v) {
  if constexpr (V == 8 && sizeof(T) == 2) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  } else if constexpr (V == 8) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) p[i] = from_f32<T>(v[i]);
  }
}

// One thread: one row and V consecutive channels (V = 8 when the width is a multiple of 8, else 1).
template <typename T, int V>
__global__ void short_conv_kernel(const T* __restrict__ bcx, const float* __restrict__ taps,
                                  const float* __restrict__ bias, const float* __restrict__ state,
                                  const int* __restrict__ state_slot, const int* __restrict__ req_of_row,
                                  const int* __restrict__ row_start, const int* __restrict__ positions,
                                  T* __restrict__ y, int hidden, int K) {
  chain_next();
  chain_wait();
  const int r = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  if (c >= hidden) return;
  const int b = req_of_row[r];
  const int first = row_start[b];          // first row of this request in the step
  const int pos = positions[r];            // absolute position of row r
  const long long ld = 3LL * hidden;
  const float* st = state + ((long long)state_slot[b] * (K - 1)) * hidden;
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = bias ? bias[c + i] : 0.f;
  // tap j multiplies the input K-1-j rows back; tap K-1 the row itself
  for (int j = 0; j < K; ++j) {
    const int back = K - 1 - j;
    if (pos - back < 0) continue;            // before the sequence's first token: zero
    const int rr = r - back;
    float v[V];
    if (rr >= first) {
      const T* row = bcx + (long long)rr * ld;
      float bv[V], xv[V];
      load_run<T, V>(row + c, bv);
      load_run<T, V>(row + 2 * hidden + c, xv);
#pragma unroll
      for (int i = 0; i < V; ++i) v[i] = bv[i] * xv[i];
    } else {
      // (first - rr) rows before the step's first row: state index K-1 - (first - rr)
      load_run<float, V>(st + (long long)(K - 1 - (first - rr)) * hidden + c, v);
    }
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = fmaf(taps[(long long)(c + i) * K + j], v[i], acc[i]);
  }
  float cv[V];
  load_run<T, V>(bcx + (long long)r * ld + hidden + c, cv);
#pragma unroll
  for (int i = 0; i < V; ++i) cv[i] *= acc[i];
  store_run<T, V>(y + (long long)r * hidden + c, cv);
}

// The same for a prompt's many rows: a thread walks CONV_RUN consecutive rows for its 8 channels with the last KT - 1
// inputs bx in registers, so every B, C and x is read once, and the loads of four rows are sent before the first is
// used. Rows of a run that belong to several requests (a run across a request's edge) go the way of the kernel above,
// row by row. Same results: a tap whose input lies before the sequence's first token multiplies a zero here and is
// left out there.
constexpr int CONV_RUN = 8;
template <typename T, int KT>
__global__ void __launch_bounds__(128) short_conv_run_kernel(const T* __restrict__ bcx, const float* __restrict__ taps,
                                                             const float* __restrict__ bias, const float* __restrict__ state,
                                                             const int* __restrict__ state_slot,
                                                             const int* __restrict__ req_of_row,
                                                             const int* __restrict__ row_start,
                                                             const int* __restrict__ positions, T* __restrict__ y, int rows,
                                                             int hidden) {
  constexpr int V = 8, S = KT - 1;
  chain_next();
  chain_wait();
  const int r0 = blockIdx.x * CONV_RUN;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  if (c >= hidden) return;
  const int n = min(CONV_RUN, rows - r0);
  const long long ld = 3LL * hidden;
  float tp[KT][V], bs[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    bs[i] = bias ? bias[c + i] : 0.f;
#pragma unroll
    for (int j = 0; j < KT; ++j) tp[j][i] = taps[(long long)(c + i) * KT + j];
  }
  const int b = req_of_row[r0];
  if (req_of_row[r0 + n - 1] != b) {
    // several requests in the run: every row looks its inputs up by itself
    for (int r = r0; r < r0 + n; ++r) {
      const int rb = req_of_row[r], first = row_start[rb], pos = positions[r];
      const float* st = state + ((long long)state_slot[rb] * S) * hidden;
      float acc[V];
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = bs[i];
#pragma unroll
      for (int j = 0; j < KT; ++j) {
        const int back = KT - 1 - j;
        if (pos - back < 0) continue;
        const int rr = r - back;
        float v[V];
        if (rr >= first) {
          float bv[V], xv[V];
          load_run<T, V>(bcx + (long long)rr * ld + c, bv);
          load_run<T, V>(bcx + (long long)rr * ld + 2 * hidden + c, xv);
#pragma unroll
          for (int i = 0; i < V; ++i) v[i] = bv[i] * xv[i];
        } else {
          load_run<float, V>(st + (long long)(KT - 1 - (first - rr)) * hidden + c, v);
        }
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = fmaf(tp[j][i], v[i], acc[i]);
      }
      float cv[V];
      load_run<T, V>(bcx + (long long)r * ld + hidden + c, cv);
#pragma unroll
      for (int i = 0; i < V; ++i) cv[i] *= acc[i];
      store_run<T, V>(y + (long long)r * hidden + c, cv);
    }
    return;
  }
  // one request: the window starts with the S inputs before row r0 (earlier rows of the step, the state, or zeros)
  const int first = row_start[b], pos0 = positions[r0];
  const float* st = state + ((long long)state_slot[b] * S) * hidden;
  float win[S][V];                                  // win[s]: the input S - s rows back
#pragma unroll
  for (int s2 = 0; s2 < S; ++s2) {
    const int back = S - s2, rr = r0 - back;
#pragma unroll
    for (int i = 0; i < V; ++i) win[s2][i] = 0.f;
    if (pos0 - back >= 0) {
      if (rr >= first) {
        float bv[V], xv[V];
        load_run<T, V>(bcx + (long long)rr * ld + c, bv);
        load_run<T, V>(bcx + (long long)rr * ld + 2 * hidden + c, xv);
#pragma unroll
        for (int i = 0; i < V; ++i) win[s2][i] = bv[i] * xv[i];
      } else {
        load_run<float, V>(st + (long long)(KT - 1 - (first - rr)) * hidden + c, win[s2]);
      }
    }
  }
  constexpr int AHEAD = 4;
  for (int q0 = 0; q0 < n; q0 += AHEAD) {
    float bv[AHEAD][V], cv[AHEAD][V], xv[AHEAD][V];
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
      const int r = min(r0 + q0 + a, r0 + n - 1);     // (past the run's end: the last row again, not stored)
      const T* row = bcx + (long long)r * ld + c;
      load_run<T, V>(row, bv[a]);
      load_run<T, V>(row + hidden, cv[a]);
      load_run<T, V>(row + 2 * hidden, xv[a]);
    }
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
      if (q0 + a >= n) break;
      float bx[V], acc[V];
#pragma unroll
      for (int i = 0; i < V; ++i) {
        bx[i] = bv[a][i] * xv[a][i];
        acc[i] = bs[i];
      }
#pragma unroll
      for (int j = 0; j < S; ++j)
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = fmaf(tp[j][i], win[j][i], acc[i]);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        acc[i] = fmaf(tp[S][i], bx[i], acc[i]);
        cv[a][i] *= acc[i];
      }
      store_run<T, V>(y + (long long)(r0 + q0 + a) * hidden + c, cv[a]);
#pragma unroll
      for (int j = 0; j + 1 < S; ++j)
#pragma unroll
        for (int i = 0; i < V; ++i) win[j][i] = win[j + 1][i];
#pragma unroll
      for (int i = 0; i < V; ++i) win[S - 1][i] = bx[i];
    }
  }
}

// new state = last K-1 of [old state ; this step's bx rows], per request and channel; one thread does both
// the reads and the writes of its channel, so no other thread's input is overwritten early.
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ bcx, float* __restrict__ state,
                                        const int* __restrict__ state_slot, const int* __restrict__ row_start,
                                        const int* __restrict__ positions, int hidden, int K) {
  chain_next();
  chain_wait();
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= hidden) return;
  const int first = row_start[b], n = row_start[b + 1] - first;
  if (n <= 0) return;
  const int S = K - 1;
  const long long ld = 3LL * hidden;
  float* st = state + ((long long)state_slot[b] * S) * hidden;
  const int start_pos = positions[first];
  float keep[MAX_TAPS];
#pragma unroll 1
  for (int s = 0; s < S; ++s) {
    // entry s of the new state is element n - S + s of the step's rows (negative: old state entry s + n)
    const int i = n - S + s;
    float v;
    if (i >= 0) {
      const T* row = bcx + (long long)(first + i) * ld;
      v = to_f32(row[c]) * to_f32(row[2 * hidden + c]);
    } else {
      // old entry s + n sits S - (s + n) inputs before the step: before position 0 it is zero
      v = (start_pos - (S - (s + n)) >= 0) ? st[(long long)(s + n) * hidden + c] : 0.f;
    }
    keep[s] = v;
  }
#pragma unroll 1
  for (int s = 0; s < S; ++s) st[(long long)s * hidden + c] = keep[s];
}

// A step in which every request has one row (decoding): the convolution and the state's shift in one kernel, one
// thread a (request, channel). The projection's output may come as `parts` 32-bit partial sums [parts, rows, 3H]
// (a product split along k): they are added in order and rounded to T first, as the separate reduction would have.
// Results equal those of the two kernels above bit for bit.
template <typename T>
__global__ void short_conv_decode_kernel(const T* __restrict__ bcx, const float* __restrict__ partial, int parts,
                                         long long part_stride, const float* __restrict__ taps,
                                         const float* __restrict__ bias, float* __restrict__ state,
                                         const int* __restrict__ state_slot, const int* __restrict__ req_of_row,
                                         const int* __restrict__ positions, T* __restrict__ y, int hidden, int K,
                                         int write_state) {
  chain_next();
  chain_wait();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= hidden) return;
  const int b = req_of_row[r];
  const int pos = positions[r];
  const long long ld = 3LL * hidden;
  float in[3];                                   // B, C, x of this row and channel
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const long long at = (long long)r * ld + (long long)j * hidden + c;
    if (partial) {
      float acc = 0.f;
      for (int s = 0; s < parts; ++s) acc += partial[(long long)s * part_stride + at];
      in[j] = to_f32(from_f32<T>(acc));
    } else {
      in[j] = to_f32(bcx[at]);
    }
  }
  const float bx = in[0] * in[2];
  const int S = K - 1;
  float* st = state + ((long long)state_slot[b] * S) * hidden;
  float old[MAX_TAPS];
#pragma unroll 1
  for (int s = 0; s < S; ++s) old[s] = st[(long long)s * hidden + c];
  float acc = bias ? bias[c] : 0.f;
#pragma unroll 1
  for (int j = 0; j < K; ++j) {
    const int back = K - 1 - j;
    if (pos - back < 0) continue;                // before the sequence's first token: zero
    const float v = back == 0 ? bx : old[S - back];
    acc = fmaf(taps[(long long)c * K + j], v, acc);
  }
  y[(long long)r * hidden + c] = from_f32<T>(in[1] * acc);
  if (write_state) {
#pragma unroll 1
    for (int s = 0; s + 1 < S; ++s)              // old entry s + 1 sits S - (s + 1) inputs before this row
      st[(long long)s * hidden + c] = (pos - (S - (s + 1)) >= 0) ? old[s + 1] : 0.f;
    st[(long long)(S - 1) * hidden + c] = bx;
  }
}

}  // namespace tl

using namespace tl;

extern "C" int tl_short_conv(const void* bcx, const float* taps, const float* bias, const float* state,
                             const int* state_slot, const int* req_of_row, const int* row_start, const int* positions,
                             void* y, int rows, int hidden, int K, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && hidden > 0, "short_conv: rows %d hidden %d", rows, hidden);
  TL_REQUIRE(K >= 2 && K <= MAX_TAPS, "short_conv: %d taps; 2..%d are implemented", K, MAX_TAPS);
  // 16-byte accesses when every row, of the projection, the state and the output, starts on a 16-byte boundary
  const bool wide = hidden % 8 == 0 && ((uintptr_t)bcx % 16) == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)state % 16) == 0;
  dim3 grid(rows, ceil_div(hidden, 128 * (wide ? 8 : 1)));
  TL_REQUIRE(grid.y <= 65535, "short_conv: hidden size %d exceeds the grid limit", hidden);
  // many rows, 16-byte accesses, 2 to 4 taps: the form that walks runs of rows
  if (wide && rows >= 4 * CONV_RUN && K <= 4) {
    dim3 run_grid(ceil_div(rows, CONV_RUN), grid.y);
#define TL_RUN(T_, K_)                                                                                                     \
  return (int)launch_chained(short_conv_run_kernel<T_, K_>, run_grid, dim3(128), 0, stream, (const T_*)bcx, taps, bias,   \
                             state, state_slot, req_of_row, row_start, positions, (T_*)y, rows, hidden)
    if (dtype == TL_FP32) {
      if (K == 2) TL_RUN(float, 2);
      if (K == 3) TL_RUN(float, 3);
      TL_RUN(float, 4);
    }
    if (K == 2) TL_RUN(bf16, 2);
    if (K == 3) TL_RUN(bf16, 3);
    TL_RUN(bf16, 4);
#undef TL_RUN
  }
#define TL_CONV(T_, V_)                                                                                                   \
  return (int)launch_chained(short_conv_kernel<T_, V_>, grid, dim3(128), 0, stream, (const T_*)bcx, taps, bias, state,    \
                             state_slot, req_of_row, row_start, positions, (T_*)y, hidden, K)
  if (dtype == TL_FP32) {
    if (wide) TL_CONV(float, 8);
    TL_CONV(float, 1);
  }
  if (wide) TL_CONV(bf16, 8);
  TL_CONV(bf16, 1);
#undef TL_CONV
}

extern "C" int tl_short_conv_state(const void* bcx, float* state, const int* state_slot, const int* row_start,
                                   const int* positions, int requests, int hidden, int K, int dtype,
                                   cudaStream_t stream) {
  if (requests == 0) return 0;
  TL_REQUIRE(requests > 0 && hidden > 0, "short_conv_state: requests %d hidden %d", requests, hidden);
  TL_REQUIRE(K >= 2 && K <= MAX_TAPS, "short_conv_state: %d taps; 2..%d are implemented", K, MAX_TAPS);
  dim3 grid(requests, ceil_div(hidden, 256));
  cudaError_t e;
  if (dtype == TL_FP32)
    e = launch_chained(short_conv_state_kernel<float>, grid, dim3(256), 0, stream, (const float*)bcx, state, state_slot,
                       row_start, positions, hidden, K);
  else
    e = launch_chained(short_conv_state_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)bcx, state, state_slot,
                       row_start, positions, hidden, K);
  return (int)e;
}

// One row a request. `partial` (or null) holds the projection's output as `parts` partial sums, `part_stride` floats
// apart; else `bcx` holds it.
extern "C" int tl_short_conv_decode(const void* bcx, const float* partial, int parts, long long part_stride,
                                    const float* taps, const float* bias, float* state, const int* state_slot,
                                    const int* req_of_row, const int* positions, void* y, int rows, int hidden, int K,
                                    int dtype, int write_state, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && hidden > 0 && (bcx || (partial && parts >= 1)), "short_conv_decode: rows %d hidden %d", rows, hidden);
  TL_REQUIRE(K >= 2 && K <= MAX_TAPS, "short_conv_decode: %d taps; 2..%d are implemented", K, MAX_TAPS);
  dim3 grid(rows, ceil_div(hidden, 128));
  TL_REQUIRE(grid.y <= 65535, "short_conv_decode: hidden size %d exceeds the grid limit", hidden);
  cudaError_t e;
  if (dtype == TL_FP32)
    e = launch_chained(short_conv_decode_kernel<float>, grid, dim3(128), 0, stream, (const float*)bcx, partial, parts,
                       part_stride, taps, bias, state, state_slot, req_of_row, positions, (float*)y, hidden, K, write_state);
  else
    e = launch_chained(short_conv_decode_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)bcx, partial, parts,
                       part_stride, taps, bias, state, state_slot, req_of_row, positions, (bf16*)y, hidden, K, write_state);
  return (int)e;
}

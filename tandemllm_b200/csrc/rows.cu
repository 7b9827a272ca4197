// Row-wise kernels: embedding gather, residual add fused with RMS norm, SwiGLU gating, and the last
// error message of the library.
//
// The residual stream is 32-bit in both precisions; norms compute mean(x^2), rsqrt and the scale in
// 32-bit and round once to the compute type. Formulas: engine/models/lfm2_moe/ref.py:105-109 (norm),
// :230 (embedding), :180-183 (SwiGLU) of the reference.
#include "common.cuh"

extern "C" const char* tl_last_error() { return tl_error_text; }

extern "C" const char* tl_cuda_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

namespace tl {

// residual[r, :] = float(table[token[r], :])
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                  float* __restrict__ residual, int hidden, int vocab, int* __restrict__ status) {
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

// One block per output row. The branch output `delta` is 32-bit in both precisions.
//   gather == nullptr: row r:  residual[r] += delta[r] (when delta);  normed[r] = w * residual[r] * rsqrt(mean + eps)
//   gather != nullptr: output row i reads row gather[i]: x = residual[g] + delta[g]; normed[i] = norm(x);
//                      the residual is left as it is (used for the final norm at the wanted rows only)
// normed32 (optional) receives the same normalised row unrounded, for consumers that compute in 32-bit (the router).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const float* __restrict__ delta,
                                   const float* __restrict__ weight, T* __restrict__ normed,
                                   float* __restrict__ normed32, const int* __restrict__ gather, int hidden, float eps) {
  extern __shared__ float row[];       // hidden floats, then 33 for the reduction
  float* scratch = row + hidden;
  const int out_r = blockIdx.x;
  const int r = gather ? gather[out_r] : out_r;
  float* res = residual + (size_t)r * hidden;
  const float* del = delta ? delta + (size_t)r * hidden : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float x = res[c];
    if (del) x += del[c];
    row[c] = x;
    ss += x * x;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  T* out = normed + (size_t)out_r * hidden;
  float* out32 = normed32 ? normed32 + (size_t)out_r * hidden : nullptr;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float x = row[c];
    if (!gather && del) res[c] = x;
    const float y = weight[c] * (x * inv);
    out[c] = from_f32<T>(y);
    if (out32) out32[c] = y;
  }
}

// out[r, i] = silu(gate_up[r, i]) * gate_up[r, inter + i]
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long rows, int inter) {
  const long long n = rows * inter;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / inter;
    const int c = (int)(i - r * inter);
    const float g = to_f32(gate_up[r * 2 * inter + c]);
    const float u = to_f32(gate_up[r * 2 * inter + inter + c]);
    out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
  }
}

}  // namespace tl

using namespace tl;

extern "C" int tl_embed_rows(const void* table, const int* tokens, float* residual, int rows, int hidden, int vocab,
                             int dtype, int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && hidden > 0 && vocab > 0, "embed_rows: rows %d hidden %d vocab %d", rows, hidden, vocab);
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == TL_FP32)
    embed_rows_kernel<float><<<rows, threads, 0, stream>>>((const float*)table, tokens, residual, hidden, vocab, status);
  else
    embed_rows_kernel<bf16><<<rows, threads, 0, stream>>>((const bf16*)table, tokens, residual, hidden, vocab, status);
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_add_rmsnorm(float* residual, const float* delta, const float* weight, void* normed, float* normed32,
                              const int* gather, int out_rows, int hidden, float eps, int dtype, cudaStream_t stream) {
  if (out_rows == 0) return 0;
  TL_REQUIRE(out_rows > 0 && hidden > 0, "add_rmsnorm: rows %d hidden %d", out_rows, hidden);
  const size_t smem = (size_t)(hidden + 33) * sizeof(float);
  TL_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: hidden size %d needs %zu bytes of shared memory, the limit is 204800",
             hidden, smem);
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (dtype == TL_FP32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    add_rmsnorm_kernel<float><<<out_rows, threads, smem, stream>>>(residual, delta, weight, (float*)normed, normed32,
                                                                  gather, hidden, eps);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    add_rmsnorm_kernel<bf16><<<out_rows, threads, smem, stream>>>(residual, delta, weight, (bf16*)normed, normed32,
                                                                 gather, hidden, eps);
  }
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_silu_mul(const void* gate_up, void* out, int rows, int inter, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && inter > 0, "silu_mul: rows %d width %d", rows, inter);
  const long long n = (long long)rows * inter;
  const int blocks = (int)(ceil_div64(n, 256) < 148 * 16 ? ceil_div64(n, 256) : 148 * 16);
  if (dtype == TL_FP32)
    silu_mul_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, rows, inter);
  else
    silu_mul_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)gate_up, (bf16*)out, rows, inter);
  TL_LAUNCH_CHECK();
  return 0;
}

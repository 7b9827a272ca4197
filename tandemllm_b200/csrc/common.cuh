// Shared device helpers of the sm_100a kernels: element types, warp and block reductions, argument checks.
//
// Every exported launcher is `extern "C" int tl_<name>(..., cudaStream_t stream)`: it validates its
// arguments, launches on `stream`, and returns 0, a cudaError_t from the launch, or TL_BAD_ARGUMENT
// after storing a message that tl_last_error() returns. Nothing here allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TL_BAD_ARGUMENT 100001
#define TL_FP32 0
#define TL_BF16 1

#include <stdarg.h>
#include <stdio.h>

// The last refusal's message of the calling thread. Each library exports a function that returns it.
inline thread_local char tl_error_text[512] = "";

inline void tl_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error_text, sizeof(tl_error_text), fmt, ap);
  va_end(ap);
}

#define TL_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      tl_set_error(__VA_ARGS__);         \
      return TL_BAD_ARGUMENT;            \
    }                                    \
  } while (0)

#define TL_LAUNCH_CHECK()                      \
  do {                                         \
    cudaError_t e__ = cudaGetLastError();      \
    if (e__ != cudaSuccess) return (int)e__;   \
  } while (0)

namespace tl {

typedef __nv_bfloat16 bf16;

// Programmatic dependent launch, so that the many short kernels of a decode step overlap their launch and
// set-up with the tail of the kernel before them (the reference does the same with `griddepcontrol` in its
// row kernels, engine/models/lfm2_moe/kernels.py:79-84). A chained kernel
//   * calls chain_next() first: the kernel after it may be launched and run up to its own chain_wait();
//   * calls chain_wait() before it reads or writes any global memory: it returns once every kernel before it
//     in the stream has finished and its writes are visible.
// What a kernel does before chain_wait() must not touch global memory that other kernels write.
// Both calls do nothing in a kernel that was launched the ordinary way.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_next() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Entry `index` of a request's block table, or -1 when there is none: the index lies past the table, the entry is
// negative (a page given back or never taken) or it names no page of the pool (`num_pages`; 0: the pool's size is
// not known and only the sign is checked). Kernels record what they skip in the status word instead of faulting.
__device__ __forceinline__ int table_page(const int* __restrict__ table, int index, int max_pages, int num_pages) {
  if (index < 0 || index >= max_pages) return -1;
  const int page = table[index];
  return (page < 0 || (num_pages > 0 && page >= num_pages)) ? -1 : page;
}

// Off unless switched on (tl_set_chained_launches): measured on a B200, decode steps replayed from CUDA graphs gained
// nothing from chaining (3.50 ms against 3.51 ms a step at batch 8, and batch 1 lost 7 %), because a graph replay
// already hides launch latency; the kernels' own run times are what a step consists of.
inline int& chained_launches() {
  static int enabled = 0;
  return enabled;
}

// Launches `kernel` so that it may start before the previous kernel of `stream` has finished (see above); the
// kernel must call chain_wait(). With chaining switched off it is an ordinary launch.
template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained_launches() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KernelArgs>(args)...);
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block; every thread gets the result. `scratch` holds at least 33 floats of shared memory.
// The order of additions depends only on blockDim, never on the data or the grid.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Gated feed-forwards: out = act(gate) * up. The activation travels as an integer (the launchers' `act` / `swiglu`
// argument: 0 means a plain product without gating, 1 the SiLU of the LFM2 experts). All in 32-bit.
#define TL_ACT_NONE 0
#define TL_ACT_SILU 1
#define TL_ACT_GELU 2        // the exact form: x * 0.5 * (1 + erf(x / sqrt(2)))
#define TL_ACT_RELU2 3       // max(x, 0)^2
#define TL_ACT_IDENTITY 4    // gate * up
#define TL_ACT_LAST 4

__device__ __forceinline__ float gate_activation(float g, int act) {
  switch (act) {
    case TL_ACT_GELU: return 0.5f * g * (1.f + erff(g * 0.70710678118654752f));
    case TL_ACT_RELU2: { const float r = fmaxf(g, 0.f); return r * r; }
    case TL_ACT_IDENTITY: return g;
    default: return g / (1.f + expf(-g));
  }
}
__device__ __forceinline__ float gated(float g, float u, int act) { return gate_activation(g, act) * u; }

// The current device's number of SMs (asked once a device; 148 on a B200), for grids sized to the GPU.
inline int sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (counts[dev] == 0) {
    int n = 0;
    counts[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
  }
  return counts[dev];
}

__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ long long ceil_div64(long long a, long long b) { return (a + b - 1) / b; }

}  // namespace tl

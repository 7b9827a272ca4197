// What the kernels that move tiles with TMA share: mbarrier and bulk-tensor-copy wrappers for the device, and the host's
// cache of tensor maps. A tensor map here always describes a 2D bfloat16 tensor [rows, cols] whose boxes are 64 columns
// (128 bytes, one swizzle atom) wide and land in shared memory with the 128-byte swizzle: 16-byte piece c of row r of a
// box lies at r * 128 + ((c ^ (r & 7)) << 4) from a base that is 1024-byte aligned.
#pragma once
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace tl {

constexpr int TMA_BOX_COLS = 64;
// Polls of an mbarrier before a wait gives up (every wait in these kernels is bounded: a wait that runs out records status
// 11 and its kernel drains its copies, frees its tensor memory and returns). One copy a source file; tc_gemm.cu exports a
// setter so that a test can make a wait run out in milliseconds instead of seconds.
static __constant__ uint32_t wait_limit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Waits for the phase with the given parity to complete; false when the bound ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  const uint32_t limit = wait_limit;
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// One box from (column x, row y) of the map's tensor; x times 2 bytes must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// ------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows, cols, ld;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.ptr;
    h ^= (size_t)k.rows * 0x9E3779B97F4A7C15ULL + (size_t)k.cols * 0xBF58476D1CE4E5B9ULL + (size_t)k.ld * 31 + k.box_rows;
    return h;
  }
};

// A 2D bf16 tensor [rows, cols] with row stride ld (elements), box [box_rows, 64 columns], 128-byte swizzle. Maps are
// kept by (pointer, shape, box): the same weights and caches come back every step.
inline int tensor_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  EncodeTiledFn fn = encode_fn();
  TL_REQUIRE(fn != nullptr, "tensor map: the driver does not export cuTensorMapEncodeTiled (%d)", 0);
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TMA_BOX_COLS, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TL_REQUIRE(r == CUDA_SUCCESS, "tensor map: cuTensorMapEncodeTiled failed with %d (rows %lld cols %lld ld %lld box %d)",
             (int)r, rows, cols, ld, box_rows);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

}  // namespace tl

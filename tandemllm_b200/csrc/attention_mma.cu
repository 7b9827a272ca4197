// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, 32-bit accumulation), for
// prompt portions and for decoding, head sizes 64 and 128.
//
//   s = q k^T * scale over positions max(0, pos - window + 1) .. pos; softmax in 32-bit; o = a v
//   query head h reads KV head h / (Hq / Hk)                      (engine/models/lfm2_moe/ref.py:166-178)
//
// One CTA of four warps takes a tile of query rows of one request and one KV head. The G query heads of that KV
// head are packed into the tile's 64 M rows (M row m = query row m / G, head m % G), so keys and values are read
// once for the whole group: a tile holds 64 / G query rows, and a decode step's single row still fills G rows.
// Keys and values come page by page through cp.async into swizzled shared memory, two stages deep; scores and
// the running maximum, sum and output stay in registers (the online softmax of flash attention).
//   split = 0   the CTA walks all visible keys of its tile and writes the output (prompt portions)
//   split = S   grid.z spans of S key positions (a multiple of 64), aligned to absolute positions; a row whose keys
//               lie in one span is written directly, else the span's (max, sum, weighted values) go to scratch and
//               the join kernel of attention_split.cu adds the spans in order (decoding at long contexts). The
//               caller picks S so that the grid fills the GPU: short spans for one request, long ones for many.
// The tile table (request, first row, rows) comes from the host with the step's other integers.
#include "common.cuh"

namespace tl {

constexpr int KT = 64;            // keys per tile; a span's length is a multiple of it

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;          // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold D bf16: chunks are XOR-swizzled by the
// row so that the eight rows an ldmatrix reads fall into different banks.
template <int D> __device__ __forceinline__ int swz(int row, int chunk) { return row * (D * 2) + ((chunk ^ (row & 7)) << 4); }

template <int D>
__global__ void __launch_bounds__(128) attention_mma_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    const int* __restrict__ block_table, int max_pages, int page_size, const int* __restrict__ tiles,
    const int* __restrict__ positions, float scale, int window, bf16* __restrict__ out, float* __restrict__ part_o,
    float* __restrict__ part_ml, int n_spans, int split, int Hq, int Hk, int* __restrict__ status) {
  constexpr int CH = D / 8;                 // 16-byte chunks per row
  constexpr int TILE_BYTES = 64 * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sq = smem;                        // [64][D]
  uint8_t* sk = sq + TILE_BYTES;             // [2][64][D]
  uint8_t* sv = sk + 2 * TILE_BYTES;         // [2][64][D]

  chain_next();
  chain_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t = blockIdx.x, g = blockIdx.y, span = blockIdx.z;
  const int b = tiles[3 * t], row0 = tiles[3 * t + 1], nq = tiles[3 * t + 2];
  const int G = Hq / Hk;
  const int pos0 = positions[row0];
  const int* table = block_table + (long long)b * max_pages;
  // keys any row of the tile may see
  int k_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  int k_hi = pos0 + nq - 1;
  const int span_keys = split > 0 ? split : 1;     // `split` carries the span's length in key positions (0: no split)
  if (split) {
    k_lo = max(k_lo, span * span_keys);
    k_hi = min(k_hi, (span + 1) * span_keys - 1);
  }
  if (k_lo > k_hi) return;
  const int kt_first = k_lo / KT, kt_last = k_hi / KT;

  // ---- Q tile: M row m = (query row m / G, head m % G); rows past the tile's queries are zero ----
  for (int i = tid; i < 64 * CH; i += 128) {
    const int m = i / CH, c = i % CH;
    const int qi = m / G, hj = m % G;
    const bool valid = qi < nq;
    const bf16* src = q + ((long long)(row0 + (valid ? qi : 0)) * Hq + g * G + hj) * D + c * 8;
    cp_async16(sq + swz<D>(m, c), src, valid);
  }
  auto load_kv = [&](int kt, int stage) {
    for (int i = tid; i < 64 * CH; i += 128) {
      const int key = i / CH, c = i % CH;
      const int kp = kt * KT + key;
      bool valid = kp >= k_lo && kp <= k_hi;
      long long off = 0;
      if (valid) {
        const int page = table[kp / page_size];
        if (page < 0) {
          atomicExch(status, 3);
          valid = false;
        } else {
          off = (((long long)page * Hk + g) * page_size + kp % page_size) * D + c * 8;
        }
      }
      cp_async16(sk + stage * TILE_BYTES + swz<D>(key, c), k_cache + off, valid);
      cp_async16(sv + stage * TILE_BYTES + swz<D>(key, c), v_cache + off, valid);
    }
  };
  load_kv(kt_first, 0);
  cp_async_commit();

  // this thread's two M rows and their query positions
  const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const int q_lo = r_lo / G, q_hi = r_hi / G;
  const bool v_lo = q_lo < nq, v_hi = q_hi < nq;
  const int p_lo = pos0 + q_lo, p_hi = pos0 + q_hi;
  const int w_lo = window > 0 ? max(0, p_lo - window + 1) : 0, w_hi = window > 0 ? max(0, p_hi - window + 1) : 0;

  const bool active = warp * 16 < nq * G;
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  uint32_t qf[D / 16][4];

  for (int kt = kt_first; kt <= kt_last; ++kt) {
    const int stage = (kt - kt_first) & 1;
    if (kt < kt_last) load_kv(kt + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (!active) {                // a warp whose 16 M rows lie past the tile's queries only helps with the loads
      __syncthreads();
      continue;
    }
    if (kt == kt_first) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const int row = warp * 16 + (lane & 15), c = kk * 2 + (lane >> 4);
        ldmatrix_x4(smem_addr(sq + swz<D>(row, c)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
      }
    }
    const uint8_t* ks = sk + stage * TILE_BYTES;
    const uint8_t* vs = sv + stage * TILE_BYTES;
    // ---- scores of this warp's 16 rows against 64 keys ----
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int n = 0; n < 8; n += 2) {
        uint32_t b0, b1, b2, b3;
        const int row = (n + (lane >> 4)) * 8 + (lane & 7), c = kk * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(smem_addr(ks + swz<D>(row, c)), b0, b1, b2, b3);
        mma_bf16(s[n], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
        mma_bf16(s[n + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
      }
    }
    // ---- mask, running maximum ----
    const int key0 = kt * KT + (lane & 3) * 2;
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int kp = key0 + n * 8 + e;
        const bool in = kp >= k_lo && kp <= k_hi;
        s[n][e] = (in && v_lo && kp <= p_lo && kp >= w_lo) ? s[n][e] * scale : -INFINITY;
        s[n][2 + e] = (in && v_hi && kp <= p_hi && kp >= w_hi) ? s[n][2 + e] * scale : -INFINITY;
        mx_lo = fmaxf(mx_lo, s[n][e]);
        mx_hi = fmaxf(mx_hi, s[n][2 + e]);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float n_lo = fmaxf(m_lo, mx_lo), n_hi = fmaxf(m_hi, mx_hi);
    const float a_lo = n_lo == -INFINITY ? 1.f : expf(m_lo - n_lo), a_hi = n_hi == -INFINITY ? 1.f : expf(m_hi - n_hi);
    m_lo = n_lo;
    m_hi = n_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t pf[4][4];                        // P as A fragments: k-step j covers keys 16 j .. 16 j + 15
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float p0 = s[n][0] == -INFINITY ? 0.f : expf(s[n][0] - n_lo);
      const float p1 = s[n][1] == -INFINITY ? 0.f : expf(s[n][1] - n_lo);
      const float p2 = s[n][2] == -INFINITY ? 0.f : expf(s[n][2] - n_hi);
      const float p3 = s[n][3] == -INFINITY ? 0.f : expf(s[n][3] - n_hi);
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l_lo = l_lo * a_lo + sum_lo;
    l_hi = l_hi * a_hi + sum_hi;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      o[n][0] *= a_lo;
      o[n][1] *= a_lo;
      o[n][2] *= a_hi;
      o[n][3] *= a_hi;
    }
    // ---- o += P V ----
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int n = 0; n < D / 8; n += 2) {
        uint32_t b0, b1, b2, b3;
        const int row = j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = n + (lane >> 4);
        ldmatrix_x4_trans(smem_addr(vs + swz<D>(row, c)), b0, b1, b2, b3);
        mma_bf16(o[n], pf[j][0], pf[j][1], pf[j][2], pf[j][3], b0, b1);
        mma_bf16(o[n + 1], pf[j][0], pf[j][1], pf[j][2], pf[j][3], b2, b3);
      }
    }
    __syncthreads();            // the stage read here is the one the next iteration's prefetch overwrites
  }
  cp_async_wait<0>();
  // the row sums live in the four lanes of a quad
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const bool valid = half ? v_hi : v_lo;
    if (!valid) continue;
    const int r = half ? r_hi : r_lo;
    const int qi = r / G, head = g * G + r % G;
    const long long row = row0 + qi;
    const float l = half ? l_hi : l_lo, mrow = half ? m_hi : m_lo;
    const int pos = pos0 + qi;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const bool direct = !split || (lo / span_keys == pos / span_keys);
    if (direct) {
      if (split && span != pos / span_keys) continue;      // only the CTA of the row's own span holds its keys
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = out + (row * Hq + head) * D + (lane & 3) * 2;
#pragma unroll
      for (int n = 0; n < D / 8; ++n)
        *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
    } else {
      // a span that holds none of the row's keys writes nothing: the join kernel reads only the spans of lo .. pos
      if (span < lo / span_keys || span > pos / span_keys) continue;
      float* dst = part_o + ((row * Hq + head) * n_spans + span) * D + (lane & 3) * 2;
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        dst[n * 8] = o[n][half * 2];
        dst[n * 8 + 1] = o[n][half * 2 + 1];
      }
      if ((lane & 3) == 0) {
        float* ml = part_ml + ((row * Hq + head) * n_spans + span) * 2;
        ml[0] = mrow;
        ml[1] = l;
      }
    }
  }
}

template <int D>
static int launch_mma(const void* q, const void* k_cache, const void* v_cache, const int* block_table, int max_pages,
                      int page_size, const int* tiles, int n_tiles, const int* positions, float scale, int window,
                      void* out, float* part_o, float* part_ml, int n_spans, int split, int Hq, int Hk, int* status,
                      cudaStream_t stream) {
  constexpr int SMEM = 5 * 64 * D * 2;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    set = true;
  }
  dim3 grid(n_tiles, Hk, split ? n_spans : 1);
  return (int)launch_chained(attention_mma_kernel<D>, grid, dim3(128), SMEM, stream, (const bf16*)q, (const bf16*)k_cache,
                             (const bf16*)v_cache, block_table, max_pages, page_size, tiles, positions, scale, window,
                             (bf16*)out, part_o, part_ml, n_spans, split, Hq, Hk, status);
}

}  // namespace tl

using namespace tl;

// Query rows of one request that fit a tile: 64 M rows hold 64 / G query rows of the G heads of a KV head.
extern "C" int tl_attention_mma_tile_rows(int Hq, int Hk) {
  const int G = Hk > 0 ? Hq / Hk : 0;
  return (G >= 1 && G <= 64) ? 64 / G : 0;
}

extern "C" int tl_attention_mma_supported(int Hq, int Hk, int D) {
  return (D == 64 || D == 128) && Hk > 0 && Hq % Hk == 0 && Hq / Hk <= 64;
}

// tiles: int32 [n_tiles, 3] = (request index, first row, query rows <= tile_rows), rows of a tile consecutive in position.
// With split, scratch holds rows * Hq * n_spans * (D + 2) floats and the caller runs the join afterwards
// (tl_attention_join) when n_spans > 1.
extern "C" int tl_paged_attention_mma(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                      int max_pages, int page_size, const int* tiles, int n_tiles, const int* positions,
                                      float scale, int window, void* out, float* scratch, int rows, int Hq, int Hk, int D,
                                      int n_spans, int split, int* status, cudaStream_t stream) {
  if (rows == 0 || n_tiles == 0) return 0;
  TL_REQUIRE(tl_attention_mma_supported(Hq, Hk, D), "attention (tensor cores): %d heads over %d KV heads of size %d", Hq, Hk, D);
  TL_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "attention: page size %d, table width %d, window %d", page_size,
             max_pages, window);
  TL_REQUIRE(!split || (scratch && n_spans >= 1 && n_spans <= 65535 && split % KT == 0),
             "attention: split over %d spans of %d keys (a multiple of %d) needs scratch", n_spans, split, KT);
  TL_REQUIRE(Hk <= 65535, "attention: %d KV heads exceed the grid limit", Hk);
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (long long)rows * Hq * n_spans * D : nullptr;
  int e = D == 64 ? launch_mma<64>(q, k_cache, v_cache, block_table, max_pages, page_size, tiles, n_tiles, positions, scale,
                                   window, out, part_o, part_ml, n_spans, split, Hq, Hk, status, stream)
                  : launch_mma<128>(q, k_cache, v_cache, block_table, max_pages, page_size, tiles, n_tiles, positions, scale,
                                    window, out, part_o, part_ml, n_spans, split, Hq, Hk, status, stream);
  return e;
}

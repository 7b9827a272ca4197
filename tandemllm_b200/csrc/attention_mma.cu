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
//
// TMA (page sizes that divide 64 or are multiples of it; both forms of the kernel): a fifth warp is the producer. For every key tile
// its lanes look the tile's pages up and each sends one bulk tensor copy (a page's rows of one KV head, 64 columns, with
// the 128-byte swizzle the ldmatrix reads expect) onto the stage's `full` mbarrier; the four consumer warps wait on
// it, compute, and arrive on the stage's `empty` mbarrier. No thread of a consumer warp computes an address or issues
// a copy, and the CTA never stops at a block-wide barrier inside the loop. Every mbarrier wait is bounded (status 11).
#include "tma.cuh"

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

// The same for a key or value tile. Tiles that TMA wrote consist of D / 64 halves of 64 columns, each [64 keys][128
// bytes] with the 128-byte swizzle (for a head size of 64 that is the layout above).
template <int D, bool TMA> __device__ __forceinline__ int kv_off(int row, int chunk) {
  if constexpr (TMA) return (chunk >> 3) * (KT * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
  return swz<D>(row, chunk);
}

// KEYSPLIT: every tile of the launch has at most 16 M rows in use (decoding: one query row of up to 16 heads). The
// four warps then share those rows and split each 64-key tile among themselves, 16 keys a warp, each with its own
// running (max, sum, output); they are merged in warp order through shared memory at the end. Otherwise each warp
// owns 16 of the tile's 64 M rows and walks all keys. STAGES is the depth of the cp.async ring of key/value tiles.
struct KvMaps {
  CUtensorMap k, v;       // the key and value caches as [pages * KV heads * page size, D], boxes of box_rows x 64 columns
};

template <int D, bool KEYSPLIT, int STAGES, bool TMA>
__global__ void __launch_bounds__(TMA ? 160 : 128, D == 64 ? (TMA ? 3 : 4) : 2) attention_mma_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    const int* __restrict__ block_table, int max_pages, int page_size, int page_shift, int num_pages,
    const int* __restrict__ tiles,
    const int* __restrict__ positions, float scale, int window, bf16* __restrict__ out, float* __restrict__ part_o,
    float* __restrict__ part_ml, int n_spans, int split, int Hq, int Hk, int* __restrict__ status,
    const __grid_constant__ KvMaps maps, int box_rows) {
  constexpr int CH = D / 8;                 // 16-byte chunks per row
  constexpr int TILE_BYTES = 64 * D * 2;
  constexpr int QROWS = KEYSPLIT ? 16 : 64;
  constexpr int NS = KEYSPLIT ? 2 : 8;      // 8-key score tiles a warp computes per key tile
  extern __shared__ __align__(128) uint8_t smem_raw[];
  // TMA's swizzle is a function of the shared-memory address: its tiles start on 1024-byte boundaries
  uint8_t* smem = TMA ? (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023) : smem_raw;
  uint8_t* sq = smem;                            // [QROWS][D]
  uint8_t* sk = sq + QROWS * D * 2;              // [STAGES][64][D]
  uint8_t* sv = sk + STAGES * TILE_BYTES;        // [STAGES][64][D]
  uint64_t* full = reinterpret_cast<uint64_t*>(sv + STAGES * TILE_BYTES);      // TMA: [STAGES], then empty [STAGES]
  uint64_t* empty = full + STAGES;

  chain_next();
  chain_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t = blockIdx.x, g = blockIdx.y, span = blockIdx.z;
  const int b = tiles[3 * t], row0 = tiles[3 * t + 1], nq = tiles[3 * t + 2];
  const int G = Hq / Hk;
  if (KEYSPLIT && nq * G > 16) {                 // the caller promised small tiles
    if (tid == 0) atomicExch(status, 4);
    return;
  }
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

  if constexpr (TMA) {
    if (tid == 0) {
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(&full[s], 1);           // the producer's arrival, with the bytes of the stage's copies
        mbar_init(&empty[s], 4);          // one arrival a consumer warp
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
  }
  // ---- Q tile: M row m = (query row m / G, head m % G); rows past the tile's queries are zero ----
  for (int i = tid; i < QROWS * CH && tid < 128; i += 128) {
    const int m = i / CH, c = i % CH;
    const int qi = m / G, hj = m % G;
    const bool valid = qi < nq;
    const bf16* src = q + ((long long)(row0 + (valid ? qi : 0)) * Hq + g * G + hj) * D + c * 8;
    cp_async16(sq + swz<D>(m, c), src, valid);
  }
  // Two threads copy one key's row: one page lookup a thread and tile, and each pair of threads fills whole 32-byte
  // sectors with every copy.
  const int my_key = tid >> 1;
  auto load_kv = [&](int kt, int stage) {
    const int kp = kt * KT + my_key;
    bool valid = kp >= k_lo && kp <= k_hi;
    long long off = 0;
    if (valid) {
      const int pg = page_shift >= 0 ? kp >> page_shift : kp / page_size;
      const int page = table_page(table, pg, max_pages, num_pages);
      if (page < 0) {
        atomicExch(status, 3);
        valid = false;
      } else {
        off = (((long long)page * Hk + g) * page_size + (kp - pg * page_size)) * D;
      }
    }
    uint8_t* dk = sk + stage * TILE_BYTES;
    uint8_t* dv = sv + stage * TILE_BYTES;
#pragma unroll
    for (int j = 0; j < CH / 2; ++j) {
      const int c = (tid & 1) + 2 * j;
      cp_async16(dk + swz<D>(my_key, c), k_cache + off + c * 8, valid);
      cp_async16(dv + swz<D>(my_key, c), v_cache + off + c * 8, valid);
    }
  };
  if constexpr (!TMA) {
#pragma unroll
    for (int s0 = 0; s0 < STAGES - 1; ++s0) {
      if (kt_first + s0 <= kt_last) load_kv(kt_first + s0, s0);
      cp_async_commit();
    }
  } else {
    cp_async_commit();
    if (warp == 4) {
      // ---- the producer warp: lane i sends box i of every tile (a page's rows, 64 columns, of the keys or the values) ----
      constexpr int HALVES = D / 64;
      const int n_boxes = (KT / box_rows) * HALVES * 2;
      const uint32_t box_bytes = (uint32_t)box_rows * 128u;
      const int which = lane & 1, half = (lane >> 1) % HALVES, pi = lane / (2 * HALVES);
      bool ok = true;
      int issued = 0;
      for (int kt = kt_first; kt <= kt_last; ++kt) {
        const int it = kt - kt_first, stage = it % STAGES;
        if (it >= STAGES && !mbar_wait(&empty[stage], ((it / STAGES) - 1) & 1)) {
          ok = false;
          break;
        }
        bool need = false;
        int y = 0;
        uint8_t* dst = (which ? sv : sk) + stage * TILE_BYTES + half * (KT * 128) + pi * box_rows * 128;
        if (lane < n_boxes) {
          const int key0 = kt * KT + pi * box_rows;                    // the box's first key position
          need = key0 + box_rows - 1 >= k_lo && key0 <= k_hi;         // (a page no row of the tile sees may be gone)
          if (need) {
            const int pg = page_shift >= 0 ? key0 >> page_shift : key0 / page_size;
            const int page = table_page(table, pg, max_pages, num_pages);
            if (page < 0) {
              atomicExch(status, 3);
              need = false;
            } else {
              y = (page * Hk + g) * page_size + (key0 - pg * page_size);
            }
          }
          // values that are not fetched are multiplied by weights of zero: they must be numbers
          if (!need && which) {
            for (uint32_t j = 0; j < box_bytes; j += 16) *reinterpret_cast<uint4*>(dst + j) = make_uint4(0u, 0u, 0u, 0u);
            // these bytes are written by TMA (the async proxy) when the stage comes round again
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          }
        }
        const uint32_t n_need = __popc(__ballot_sync(0xffffffffu, need));
        __syncwarp();       // every lane's zeros are written before lane 0's arrival, which may complete the phase by itself
        if (lane == 0) mbar_expect_tx(&full[stage], n_need * box_bytes);
        __syncwarp();
        if (need) tma_load_2d(dst, which ? &maps.v : &maps.k, &full[stage], half * 64, y);
        issued = it + 1;
      }
      if (!ok) {
        // a consumer gave up: what was sent must still land before the CTA's shared memory is given back
        if (lane == 0) atomicExch(status, 11);
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(&full[i % STAGES], (i / STAGES) & 1);
      }
    } else {
      cp_async_wait<0>();
      asm volatile("bar.sync 1, 128;" ::: "memory");       // the four consumer warps: the Q tile is complete
    }
  }
  const bool consumer = !TMA || warp < 4;

  // this thread's two M rows and their query positions
  const int wrow = KEYSPLIT ? 0 : warp * 16;
  const int r_lo = wrow + (lane >> 2), r_hi = r_lo + 8;
  const int q_lo = r_lo / G, q_hi = r_hi / G;
  const bool v_lo = q_lo < nq, v_hi = q_hi < nq;
  const int p_lo = pos0 + q_lo, p_hi = pos0 + q_hi;
  const int w_lo = window > 0 ? max(0, p_lo - window + 1) : 0, w_hi = window > 0 ? max(0, p_hi - window + 1) : 0;
  const int n_base = KEYSPLIT ? warp * 2 : 0;      // first 8-key score tile of this warp
  const float scale2 = scale * 1.4426950408889634f;   // scores are kept in units of log 2: exponentials are exp2

  const bool active = wrow < nq * G;
  // the warp's 16 M rows: whether all of them are query rows, the earliest position among them and the latest start
  // of a window (what decides, for the whole warp, whether a key tile needs masking)
  const bool rows_all_valid = (wrow + 15) / G < nq;
  const int first_pos = pos0 + wrow / G;
  const int last_w_lo = window > 0 ? max(0, pos0 + (wrow + 15) / G - window + 1) : 0;
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  uint32_t qf[D / 16][4];

  for (int kt = kt_first; consumer && kt <= kt_last; ++kt) {
    const int it = kt - kt_first;
    const int stage = it % STAGES;
    if constexpr (TMA) {
      if (!mbar_wait(&full[stage], (it / STAGES) & 1)) {      // the tile's copies have landed
        if (lane == 0) atomicExch(status, 11);
        break;
      }
    } else {
      cp_async_wait<STAGES - 2>();      // this thread's copies of tile kt have landed
      __syncthreads();                  // everybody's have, and everybody is done with the tile before
      if (kt + STAGES - 1 <= kt_last) load_kv(kt + STAGES - 1, (it + STAGES - 1) % STAGES);
      cp_async_commit();
    }
    if (!active) {                    // a warp whose 16 M rows lie past the tile's queries only helps with the loads
      if constexpr (TMA) {
        if (lane == 0) mbar_arrive(&empty[stage]);
      }
      continue;
    }
    if (kt == kt_first) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const int row = wrow + (lane & 15), c = kk * 2 + (lane >> 4);
        ldmatrix_x4(smem_addr(sq + swz<D>(row, c)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
      }
    }
    const uint8_t* ks = sk + stage * TILE_BYTES;
    const uint8_t* vs = sv + stage * TILE_BYTES;
    // ---- scores of this warp's 16 rows against its keys of the tile ----
    float s[NS][4];
#pragma unroll
    for (int n = 0; n < NS; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int n = 0; n < NS; n += 2) {
        uint32_t b0, b1, b2, b3;
        const int row = (n_base + n + (lane >> 4)) * 8 + (lane & 7), c = kk * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(smem_addr(ks + kv_off<D, TMA>(row, c)), b0, b1, b2, b3);
        mma_bf16(s[n], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
        mma_bf16(s[n + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
      }
    }
    // ---- mask, running maximum ----
    const int key0 = kt * KT + n_base * 8 + (lane & 3) * 2;
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
    // Most key tiles of a prompt lie wholly before every row of the warp and inside every row's window: nothing to mask.
    const bool open = !KEYSPLIT && rows_all_valid && kt * KT >= k_lo && kt * KT + KT - 1 <= min(k_hi, first_pos) && kt * KT >= last_w_lo;
    if (open) {
#pragma unroll
      for (int n = 0; n < NS; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e] *= scale2;
        mx_lo = fmaxf(mx_lo, fmaxf(s[n][0], s[n][1]));
        mx_hi = fmaxf(mx_hi, fmaxf(s[n][2], s[n][3]));
      }
    } else {
#pragma unroll
      for (int n = 0; n < NS; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kp = key0 + n * 8 + e;
          const bool in = kp >= k_lo && kp <= k_hi;
          s[n][e] = (in && v_lo && kp <= p_lo && kp >= w_lo) ? s[n][e] * scale2 : -INFINITY;
          s[n][2 + e] = (in && v_hi && kp <= p_hi && kp >= w_hi) ? s[n][2 + e] * scale2 : -INFINITY;
          mx_lo = fmaxf(mx_lo, s[n][e]);
          mx_hi = fmaxf(mx_hi, s[n][2 + e]);
        }
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float n_lo = fmaxf(m_lo, mx_lo), n_hi = fmaxf(m_hi, mx_hi);
    // a row that has seen no key yet keeps 0 as its reference, so that exp2(-inf - reference) is 0, not NaN
    const float c_lo = n_lo == -INFINITY ? 0.f : n_lo, c_hi = n_hi == -INFINITY ? 0.f : n_hi;
    const float a_lo = exp2f(m_lo - c_lo), a_hi = exp2f(m_hi - c_hi);      // 0 where the row had no key before
    m_lo = n_lo;
    m_hi = n_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t pf[NS / 2][4];                   // P as A fragments: k-step j covers 16 of the warp's keys
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      const float p0 = exp2f(s[n][0] - c_lo), p1 = exp2f(s[n][1] - c_lo);
      const float p2 = exp2f(s[n][2] - c_hi), p3 = exp2f(s[n][3] - c_hi);
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l_lo = l_lo * a_lo + sum_lo;
    l_hi = l_hi * a_hi + sum_hi;
    if (__any_sync(0xffffffffu, a_lo != 1.f || a_hi != 1.f)) {      // most tiles leave the maxima as they are
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        o[n][0] *= a_lo;
        o[n][1] *= a_lo;
        o[n][2] *= a_hi;
        o[n][3] *= a_hi;
      }
    }
    // ---- o += P V ----
#pragma unroll
    for (int j = 0; j < NS / 2; ++j) {
#pragma unroll
      for (int n = 0; n < D / 8; n += 2) {
        uint32_t b0, b1, b2, b3;
        const int row = (n_base / 2 + j) * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = n + (lane >> 4);
        ldmatrix_x4_trans(smem_addr(vs + kv_off<D, TMA>(row, c)), b0, b1, b2, b3);
        mma_bf16(o[n], pf[j][0], pf[j][1], pf[j][2], pf[j][3], b0, b1);
        mma_bf16(o[n + 1], pf[j][0], pf[j][1], pf[j][2], pf[j][3], b2, b3);
      }
    }
    if constexpr (TMA) {
      __syncwarp();                                  // every lane has read the stage
      if (lane == 0) mbar_arrive(&empty[stage]);
    }
  }
  cp_async_wait<0>();
  // the row sums live in the four lanes of a quad
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  // One finished pair of columns of a row goes to the output, or, when the row's keys lie in several spans, to scratch.
  auto emit = [&](int r, int col, float o0, float o1, float mrow, float l, bool first) {
    const int qi = r / G, head = g * G + r % G;
    const long long row = row0 + qi;
    const int pos = pos0 + qi;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const bool direct = !split || (lo / span_keys == pos / span_keys);
    if (direct) {
      if (split && span != pos / span_keys) return;        // only the CTA of the row's own span holds its keys
      const float inv = l > 0.f ? 1.f / l : 0.f;
      *reinterpret_cast<uint32_t*>(out + (row * Hq + head) * D + col) = pack_bf16(o0 * inv, o1 * inv);
    } else {
      // a span that holds none of the row's keys writes nothing: the join kernel reads only the spans of lo .. pos
      if (span < lo / span_keys || span > pos / span_keys) return;
      float* dst = part_o + ((row * Hq + head) * n_spans + span) * D + col;
      dst[0] = o0;
      dst[1] = o1;
      if (first) {
        float* ml = part_ml + ((row * Hq + head) * n_spans + span) * 2;
        ml[0] = mrow * 0.6931471805599453f;             // the join kernel works in natural units
        ml[1] = l;
      }
    }
  };

  if constexpr (!KEYSPLIT) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (!consumer || !(half ? v_hi : v_lo)) continue;
      const int r = half ? r_hi : r_lo;
      const float l = half ? l_hi : l_lo, mrow = half ? m_hi : m_lo;
#pragma unroll
      for (int n = 0; n < D / 8; ++n)
        emit(r, n * 8 + (lane & 3) * 2, o[n][half * 2], o[n][half * 2 + 1], mrow, l, n == 0 && (lane & 3) == 0);
    }
  } else {
    // ---- merge the four warps' shares of the keys, in warp order ----
    float* mo = reinterpret_cast<float*>(sk);              // [4][16][D]
    float* mml = mo + 4 * 16 * D;                          // [4][16][2]
    __syncthreads();                                       // every warp is done with the key/value stages
#pragma unroll
    for (int half = 0; half < 2 && consumer; ++half) {
      const int r = (lane >> 2) + half * 8;
      float* dst = mo + (warp * 16 + r) * D + (lane & 3) * 2;
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        dst[n * 8] = o[n][half * 2];
        dst[n * 8 + 1] = o[n][half * 2 + 1];
      }
      if ((lane & 3) == 0) {
        mml[(warp * 16 + r) * 2] = half ? m_hi : m_lo;
        mml[(warp * 16 + r) * 2 + 1] = half ? l_hi : l_lo;
      }
    }
    __syncthreads();
    for (int i = tid; i < 16 * (D / 2) && consumer; i += 128) {
      const int r = i / (D / 2), col = (i % (D / 2)) * 2;
      if (r >= nq * G) continue;
      float mrow = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mrow = fmaxf(mrow, mml[(w * 16 + r) * 2]);
      float l = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = mml[(w * 16 + r) * 2];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - mrow);
        l += f * mml[(w * 16 + r) * 2 + 1];
        o0 += f * mo[(w * 16 + r) * D + col];
        o1 += f * mo[(w * 16 + r) * D + col + 1];
      }
      emit(r, col, o0, o1, mrow, l, col == 0);
    }
  }
}

template <int D, bool KEYSPLIT, int STAGES, bool TMA>
static int launch_mma(const void* q, const void* k_cache, const void* v_cache, const int* block_table, int max_pages,
                      int page_size, int num_pages, const int* tiles, int n_tiles, const int* positions, float scale, int window,
                      void* out, float* part_o, float* part_ml, int n_spans, int split, int Hq, int Hk, int* status,
                      cudaStream_t stream) {
  // with TMA: room to start the tiles on a 1024-byte boundary, and the stages' mbarriers behind them
  constexpr int SMEM = ((KEYSPLIT ? 16 : 64) + 2 * STAGES * 64) * D * 2 + (TMA ? 1024 + 2 * STAGES * 8 : 0);
  static_assert(!KEYSPLIT || 4 * 16 * (D + 2) * 4 <= 2 * STAGES * 64 * D * 2, "the merge buffer reuses the stages");
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<D, KEYSPLIT, STAGES, TMA>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    set = true;
  }
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size;) ++page_shift;
  KvMaps maps;
  memset(&maps, 0, sizeof(maps));
  const int box_rows = page_size < KT ? page_size : KT;
  if (TMA) {
    const long long cache_rows = (long long)num_pages * Hk * page_size;
    int e = tensor_map(k_cache, cache_rows, D, D, box_rows, &maps.k);
    if (e == 0) e = tensor_map(v_cache, cache_rows, D, D, box_rows, &maps.v);
    if (e != 0) return e;
  }
  dim3 grid(n_tiles, Hk, split ? n_spans : 1);
  return (int)launch_chained(attention_mma_kernel<D, KEYSPLIT, STAGES, TMA>, grid, dim3(TMA ? 160 : 128), SMEM, stream,
                             (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_pages, page_size,
                             page_shift, num_pages, tiles, positions, scale, window, (bf16*)out, part_o, part_ml, n_spans, split,
                             Hq, Hk, status, maps, box_rows);
}

static int& decode_with_tma() {
  static int on = 1;
  return on;
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
// max_tile_rows: the most query rows any tile holds; when they and their heads fit 16 M rows (decoding), the kernel
// form that splits the keys among the warps runs. With split, scratch holds rows * Hq * n_spans * (D + 2) floats and
// the caller runs the join afterwards (tl_attention_join) when n_spans > 1.
extern "C" int tl_paged_attention_mma(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                      int max_pages, int page_size, int num_pages, const int* tiles, int n_tiles, int max_tile_rows,
                                      const int* positions, float scale, int window, void* out, float* scratch, int rows,
                                      int Hq, int Hk, int D, int n_spans, int split, int* status, cudaStream_t stream) {
  if (rows == 0 || n_tiles == 0) return 0;
  TL_REQUIRE(tl_attention_mma_supported(Hq, Hk, D), "attention (tensor cores): %d heads over %d KV heads of size %d", Hq, Hk, D);
  TL_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "attention: page size %d, table width %d, window %d", page_size,
             max_pages, window);
  TL_REQUIRE(!split || (scratch && n_spans >= 1 && n_spans <= 65535 && split % KT == 0),
             "attention: split over %d spans of %d keys (a multiple of %d) needs scratch", n_spans, split, KT);
  TL_REQUIRE(Hk <= 65535, "attention: %d KV heads exceed the grid limit", Hk);
  TL_REQUIRE(max_tile_rows >= 1 && max_tile_rows <= tl_attention_mma_tile_rows(Hq, Hk),
             "attention: tiles of %d query rows, at most %d fit", max_tile_rows, tl_attention_mma_tile_rows(Hq, Hk));
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (long long)rows * Hq * n_spans * D : nullptr;
  const bool keysplit = max_tile_rows * (Hq / Hk) <= 16;
  // the producer warp's copies are whole pages (or 64-row pieces of one) that tile the 64 keys of a stage, every box on
  // a 1024-byte boundary of shared memory; the caches start on 16-byte boundaries and hold at most 2^31 rows
  const bool tma = decode_with_tma() && ((page_size % 8 == 0 && KT % page_size == 0) || page_size % KT == 0) &&
                   ((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0 &&
                   (long long)num_pages * Hk * page_size < (1LL << 31);
#define TL_MMA(D_, KS_, ST_, TMA_)                                                                                          \
  launch_mma<D_, KS_, ST_, TMA_>(q, k_cache, v_cache, block_table, max_pages, page_size, num_pages, tiles, n_tiles, positions, \
                                 scale, window, out, part_o, part_ml, n_spans, split, Hq, Hk, status, stream)
  if (D == 64)
    return keysplit ? (tma ? TL_MMA(64, true, 4, true) : TL_MMA(64, true, 4, false))
                    : (tma ? TL_MMA(64, false, 3, true) : TL_MMA(64, false, 2, false));
  return keysplit ? (tma ? TL_MMA(128, true, 3, true) : TL_MMA(128, true, 3, false))
                  : (tma ? TL_MMA(128, false, 2, true) : TL_MMA(128, false, 2, false));
#undef TL_MMA
}

// 0: keys and values are fetched with cp.async from every thread instead of a producer warp's TMA copies
extern "C" void tl_attention_mma_use_tma(int on) { decode_with_tma() = on; }

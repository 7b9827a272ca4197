// bfloat16 attention of prompt portions over the paged cache on the fifth-generation tensor cores: scores and values
// are tcgen05.mma products with their accumulators in tensor memory, keys and values arrive by TMA. Head size 64.
//
//   s = q k^T * scale over positions max(0, pos - window + 1) .. pos; softmax in 32-bit; o = a v
//   query head h reads KV head h / (Hq / Hk)                      (engine/models/lfm2_moe/ref.py:166-178)
//
// The reference's prompt attention is the library's flash kernel (engine/models/lfm2_moe/engine.py:65-88); this is the
// same online softmax laid out for sm_100a. One CTA takes a tile of query rows of one request and one KV head: the G
// query heads of that KV head are packed into the tile's 128 M rows (M row m = query row m / G, head m % G), so a tile
// holds 128 / G query rows and keys and values are read once for the whole group. Per tile of 128 keys:
//
//   warp 0      the producer: its lanes look the tile's pages up in the block table and each sends one bulk tensor copy
//               (a page's rows of the KV head, 64 columns, 128-byte swizzle) into a ring of three 16 KB slots that holds
//               keys and values in turn (K0 V0 K1 V1 ...); a slot is reused when the product that read it has completed
//   warp 1      one thread issues S = Q K^T (M 128, N 128, k = the head size; Q and K K-major) into tensor-memory columns
//               0..127 and commits; it issues the next tile's S as soon as the softmax warps hold this tile's S in their
//               registers, so that product runs under their exponentials; once they have written P it issues O += P V
//               (M 128, N = head size, k = 128 keys; P K-major from shared memory, V as it lies in the cache: N-major,
//               "MN-major" in the descriptor) into columns 128.., and commits
//   warps 2..5  the softmax: thread i owns M row i (tensor-memory lane i). It reads its row of S with tcgen05.ld (all
//               128 columns in flight, one wait), gives S back, takes the maximum, forms p = exp2(s * scale * log2 e -
//               max), sums it in 32-bit, rounds it to bfloat16 and stores it to shared memory in the layout the MMA reads
//               (128-byte swizzle). When a row's maximum rose, its O row in tensor memory is rescaled first (tcgen05.ld,
//               multiply, tcgen05.st). At the end the same threads read O, divide by the row sums and store.
//
// S and O together take 192 of a CTA's 256 tensor-memory columns and the CTA 98 KB of shared memory, so two CTAs share an
// SM: one's softmax runs beside the other's products. With `split` the keys are cut into spans exactly as in
// attention_mma.cu (partial results to scratch, joined in order by tl_attention_join). Every mbarrier wait is bounded
// (status 11: the kernel waits for the copies it started, frees its tensor memory and returns). No copy is a multicast.
#include "tma.cuh"

namespace tl {

constexpr int TC_KT = 128;        // keys per tile
constexpr int TC_M = 128;         // M rows per tile
constexpr float TC_SLACK = 8.f;   // in units of log 2: how far a row's maximum may rise above its reference before O is rescaled
constexpr int TC_THREADS = 192;

// K-major operand tile with 128-byte rows and 128-byte swizzle (Q, K and P): 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t tc_desc_k_major(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                 // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset: between 8-row groups
  d |= (uint64_t)1 << 46;                 // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
  return d;
}

// N-major operand (V: [keys][64 values], a key's 64 values contiguous, 128-byte swizzle over groups of 8 keys): the
// stride byte offset steps over 8 keys (1024 bytes), the leading byte offset over 64 values (another 64-column half).
__device__ __forceinline__ uint64_t tc_desc_mn_major(uint32_t smem_addr, uint32_t half_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((half_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// f32 accumulate, bf16 operands, A K-major, M = 128, N = n; B K-major or N-major.
__host__ __device__ constexpr uint32_t tc_idesc(int n, bool b_n_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_n_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(TC_M >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 32 consecutive columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
      "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The same without the wait: several loads may be in flight before one tc_ld_wait().
__device__ __forceinline__ void tc_ld32_async(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
      "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
      "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// A from tensor memory (P: lane = M row, a column holds two consecutive bfloat16 of the row), B from shared memory.
__device__ __forceinline__ void tc_mma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ float tc_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t tc_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct TcKvMaps {
  CUtensorMap k, v;       // the key and value caches as [pages * KV heads * page size, D], boxes of box_rows x 64 columns
};

// P_TMEM: P goes back to tensor memory (columns 192..255) and is the MMA's A operand from there, which leaves shared
// memory for a ring of RING key/value slots; else P goes through 32 KB of shared memory.
template <int D, bool P_TMEM, int RING>
__global__ void __launch_bounds__(TC_THREADS, 2) attention_tc_kernel(
    const bf16* __restrict__ q, const int* __restrict__ block_table, int max_pages, int page_size, int page_shift,
    int num_pages, const int* __restrict__ tiles, int n_tiles, const int* __restrict__ positions, float scale, int window,
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int n_spans, int split, int Hq, int Hk,
    int* __restrict__ status, const __grid_constant__ TcKvMaps maps, int box_rows) {
  static_assert(D == 64, "the tensor-core prompt attention is built for a head size of 64");
  constexpr int SLOT_BYTES = TC_KT * 128;          // 16 KB: 128 keys x 64 columns
  constexpr int Q_BYTES = TC_M * D * 2;            // 16 KB
  constexpr int P_BYTES = P_TMEM ? 0 : TC_M * TC_KT * 2;        // 32 KB: two halves of 64 keys, each [128 rows][128 bytes]
  constexpr uint32_t TMEM_COLS = 256;
  constexpr uint32_t O_COL = 128, P_COL = 192;
  constexpr int TC_RING = RING;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sq = smem;
  uint8_t* sp = sq + Q_BYTES;
  uint8_t* ring = sp + P_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + TC_RING * SLOT_BYTES);      // [TC_RING]
  uint64_t* empty = full + TC_RING;                                               // [TC_RING]
  uint64_t* s_ready = empty + TC_RING;
  uint64_t* p_ready = s_ready + 1;
  uint64_t* o_done = p_ready + 1;
  uint64_t* s_free = o_done + 1;
  uint64_t* o_ready = s_free + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_ready + 1);
  volatile uint32_t* aborted = tmem_slot + 1;

  chain_next();
  chain_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t = n_tiles - 1 - (int)blockIdx.x;        // a request's last tiles see the most keys: they start first
  const int g = blockIdx.y, span = blockIdx.z;
  const int b = tiles[3 * t], row0 = tiles[3 * t + 1], nq = tiles[3 * t + 2];
  const int G = Hq / Hk;
  if (nq * G > TC_M) {                                 // the caller promised tiles that fit
    if (tid == 0) atomicExch(status, 4);
    return;
  }
  const int pos0 = positions[row0];
  const int* table = block_table + (long long)b * max_pages;
  int k_lo = window > 0 ? max(0, pos0 - window + 1) : 0;       // keys any row of the tile may see
  int k_hi = pos0 + nq - 1;
  const int span_keys = split > 0 ? split : 1;
  if (split) {
    k_lo = max(k_lo, span * span_keys);
    k_hi = min(k_hi, (span + 1) * span_keys - 1);
  }
  if (k_lo > k_hi) return;
  const int kt_first = k_lo / TC_KT, kt_last = k_hi / TC_KT;
  const int n_kt = kt_last - kt_first + 1;

  if (tid == 0) {
    for (int s = 0; s < TC_RING; ++s) {
      mbar_init(&full[s], 1);         // the producer's arrival, with the bytes of the slot's copies
      mbar_init(&empty[s], 1);        // the commit of the product that read the slot
    }
    mbar_init(s_ready, 1);
    mbar_init(p_ready, 4);            // one arrival a softmax warp
    mbar_init(o_done, 1);
    mbar_init(s_free, 4);             // one arrival a softmax warp: S is in their registers
    mbar_init(o_ready, 1);            // the commit behind a tile's O += P V
    *aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  // ---- Q tile: M row m = (query row m / G, head m % G), 128 bytes a row, 128-byte swizzle; rows past the tile are zero ----
  for (int i = tid; i < TC_M * 8; i += TC_THREADS) {
    const int m = i >> 3, c = i & 7;
    const int qi = m / G, hj = m - qi * G;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (qi < nq) v = *reinterpret_cast<const uint4*>(q + ((long long)(row0 + qi) * Hq + g * G + hj) * D + c * 8);
    *reinterpret_cast<uint4*>(sq + m * 128 + ((c ^ (m & 7)) << 4)) = v;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the MMA reads Q through the async proxy
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- producer: item i of the ring is the keys (even i) or the values (odd i) of key tile kt_first + i / 2 ----
    const int boxes = TC_KT / box_rows;                 // boxes of an item: whole pages, or 128-row pieces of one
    const uint32_t box_bytes = (uint32_t)box_rows * 128u;
    bool ok = true;
    int issued = 0;
    for (int i = 0; i < 2 * n_kt; ++i) {
      const int slot = i % TC_RING, kt = kt_first + (i >> 1), is_v = i & 1;
      if (i >= TC_RING && !mbar_wait(&empty[slot], ((i / TC_RING) - 1) & 1)) {
        ok = false;
        break;
      }
      if (*aborted) {
        ok = false;
        break;
      }
      uint32_t n_need = 0;
      for (int b0 = 0; b0 < boxes; b0 += 32) {
        const int bi = b0 + lane;
        bool need = false;
        int y = 0;
        uint8_t* dst = ring + slot * SLOT_BYTES + bi * box_rows * 128;
        if (bi < boxes) {
          const int key0 = kt * TC_KT + bi * box_rows;
          need = key0 + box_rows - 1 >= k_lo && key0 <= k_hi;          // (a page no row of the tile sees may be gone)
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
          if (!need && is_v) {
            for (uint32_t j = 0; j < box_bytes; j += 16) *reinterpret_cast<uint4*>(dst + j) = make_uint4(0u, 0u, 0u, 0u);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          }
        }
        const uint32_t mask = __ballot_sync(0xffffffffu, need);
        n_need += __popc(mask);
        if (b0 + 32 >= boxes) {                          // the last round: the slot's byte count is known
          __syncwarp();
          if (lane == 0) mbar_expect_tx(&full[slot], n_need * box_bytes);
          __syncwarp();
        }
        // with more than 32 boxes an item the earlier rounds' copies would run ahead of the count: such page sizes are
        // refused by the launcher (a box is at least 8 rows, so an item has at most 16)
        if (need) tma_load_2d(dst, is_v ? &maps.v : &maps.k, &full[slot], 0, y);
      }
      issued = i + 1;
    }
    if (!ok) {
      if (lane == 0) {
        *aborted = 1;
        atomicExch(status, 11);
      }
      // what was sent must still land before the CTA's shared memory is given back
      for (int i = max(0, issued - TC_RING); i < issued; ++i) mbar_wait(&full[i % TC_RING], (i / TC_RING) & 1);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      constexpr uint32_t idesc_s = tc_idesc(TC_KT, false);
      constexpr uint32_t idesc_o = tc_idesc(D, true);
      const uint32_t q_addr = smem_u32(sq), p_addr = smem_u32(sp);
      bool ok = true;
      auto scores = [&](int j) -> bool {         // S = Q K^T of key tile j into columns 0..127
        const int ik = 2 * j, slot_k = ik % TC_RING;
        if (!mbar_wait(&full[slot_k], (ik / TC_RING) & 1)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k_addr = smem_u32(ring + slot_k * SLOT_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          tc_mma(tmem_base, tc_desc_k_major(q_addr + kk * 32), tc_desc_k_major(k_addr + kk * 32), idesc_s, kk > 0 ? 1u : 0u);
        tc_commit(&empty[slot_k]);                       // the keys' slot is free once the scores are done
        tc_commit(s_ready);
        return true;
      };
      ok = scores(0);
      for (int j = 0; j < n_kt && ok; ++j) {
        // the next tile's scores as soon as this tile's S has been read out: they run under the softmax
        if (j + 1 < n_kt) {
          if (!mbar_wait(s_free, j & 1)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (!scores(j + 1)) { ok = false; break; }
        }
        const int iv = 2 * j + 1, slot_v = iv % TC_RING;
        if (!mbar_wait(p_ready, j & 1)) { ok = false; break; }       // P is in shared memory, O is rescaled
        if (!mbar_wait(&full[slot_v], (iv / TC_RING) & 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_addr = smem_u32(ring + slot_v * SLOT_BYTES);
#pragma unroll
        for (int kk = 0; kk < TC_KT / 16; ++kk) {
          // 16 keys: P's columns 16 kk .. (half kk / 4, 32 bytes a step inside the 128-byte row), V's rows 16 kk ..
          if constexpr (P_TMEM) {
            tc_mma_a_tmem(tmem_base + O_COL, tmem_base + P_COL + kk * 8, tc_desc_mn_major(v_addr + kk * 2048, SLOT_BYTES),
                          idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
          } else {
            const uint32_t pa = p_addr + (kk >> 2) * (TC_M * 128) + (kk & 3) * 32;
            tc_mma(tmem_base + O_COL, tc_desc_k_major(pa), tc_desc_mn_major(v_addr + kk * 2048, SLOT_BYTES), idesc_o,
                   (j > 0 || kk > 0) ? 1u : 0u);
          }
        }
        tc_commit(&empty[slot_v]);
        tc_commit(o_ready);
        if (j == n_kt - 1) tc_commit(o_done);
      }
      if (!ok) {
        *aborted = 1;
        atomicExch(status, 11);
      }
    }
  } else {
    // ---- softmax and epilogue: this thread owns M row m = tensor-memory lane m ----
    const int quad = warp & 3;
    const int m = quad * 32 + lane;
    const int qi = m / G, hj = m - qi * G;
    const bool v_row = qi < nq;
    const int p_row = pos0 + qi;
    const int w_row = window > 0 ? max(0, p_row - window + 1) : 0;
    const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float scale2 = scale * 1.4426950408889634f;       // scores in units of log 2: exponentials are exp2
    // what decides, for the whole warp, whether a key tile needs masking: its 32 M rows' validity, the earliest position
    // among them and the latest start of a window
    const int m_first = quad * 32, m_last = quad * 32 + 31;
    const bool rows_all_valid = m_last / G < nq;
    const int first_pos = pos0 + m_first / G;
    const int last_w_lo = window > 0 ? max(0, pos0 + m_last / G - window + 1) : 0;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kt; ++j) {
      const int kt = kt_first + j;
      // (the warp decides together: the tensor-memory loads below are warp-wide)
      if (!__all_sync(0xffffffffu, mbar_wait(s_ready, j & 1)) || __any_sync(0xffffffffu, *aborted != 0)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int key_base = kt * TC_KT;
      const bool open = rows_all_valid && key_base >= k_lo && key_base + TC_KT - 1 <= min(k_hi, first_pos) && key_base >= last_w_lo;
      // ---- the row of S into registers (four loads in flight, one wait), and S is free for the next tile's scores ----
      uint32_t r[TC_KT];
#pragma unroll
      for (int c = 0; c < TC_KT / 32; ++c) tc_ld32_async(t_row + c * 32, r + c * 32);
      tc_ld_wait();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      // ---- the row's maximum ----
      if (!open) {
#pragma unroll
        for (int e = 0; e < TC_KT; ++e) {
          const int kp = key_base + e;
          const bool in = v_row && kp >= k_lo && kp <= k_hi && kp <= p_row && kp >= w_row;
          r[e] = in ? r[e] : 0xff800000u;                 // -inf: exp2 of it is 0
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains: a single one is 128 dependent steps
#pragma unroll
      for (int e = 0; e < TC_KT; e += 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) mx4[i] = fmaxf(mx4[i], __uint_as_float(r[e + i]));
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx = mx == -INFINITY ? mx : mx * scale2;
      float m_new = fmaxf(m_run, mx);
      // A maximum that rose by little keeps the old reference: p then reaches 2^TC_SLACK at most, which bfloat16 and the
      // 32-bit sums hold as well as values below 1, and neither O nor the sum needs rescaling for this tile.
      if (m_run != -INFINITY && m_new - m_run <= TC_SLACK) m_new = m_run;
      // a row that has seen no key yet keeps 0 as its reference, so that exp2(-inf - reference) is 0, not NaN
      const float ref = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = tc_exp2(m_run - ref);             // 0 where the row had no key before
      m_run = m_new;
      l_run *= alpha;
      // ---- rescale O where a maximum rose, once the products into O up to the last tile's are complete ----
      if (j > 0) {
        if (!__all_sync(0xffffffffu, mbar_wait(o_ready, (j - 1) & 1))) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tc_ld32(t_row + O_COL + c * 32, o);
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tc_st32(t_row + O_COL + c * 32, o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      // ---- p = exp2(s - max), summed in 32-bit, rounded to bfloat16 into shared memory: 32 keys = four 16-byte pieces
      // of this row, piece index 4 c + i, in half (4 c + i) / 8 ----
      float sum = 0.f, sum_b = 0.f;
#pragma unroll
      for (int c = 0; c < TC_KT / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float p0 = tc_exp2(fmaf(__uint_as_float(r[c * 32 + 2 * e]), scale2, -ref));
          const float p1 = tc_exp2(fmaf(__uint_as_float(r[c * 32 + 2 * e + 1]), scale2, -ref));
          sum += p0;
          sum_b += p1;
          pk[e] = tc_pack(p0, p1);
        }
        if constexpr (P_TMEM) {
          tc_st16(t_row + P_COL + c * 16, pk);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int piece = c * 4 + i;
            uint8_t* dst = sp + (piece >> 3) * (TC_M * 128) + m * 128 + (((piece & 7) ^ (m & 7)) << 4);
            *reinterpret_cast<uint4*>(dst) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
          }
        }
      }
      if constexpr (P_TMEM) asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      l_run += sum + sum_b;
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");     // this thread's tensor-memory reads and writes
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");         // its P row, for the MMA's async reads
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    // ---- the output: O / l ----
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(o_done, 0)) && !__any_sync(0xffffffffu, *aborted != 0);
    if (!ok) {
      if (lane == 0) {
        *aborted = 1;
        atomicExch(status, 11);
      }
    } else {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int head = g * G + hj;
      const long long row = row0 + qi;
      const int lo = window > 0 ? max(0, p_row - window + 1) : 0;
      const bool direct = !split || (lo / span_keys == p_row / span_keys);
      // a row past the tile's queries stores nothing; with a split, only the spans that hold keys of the row do
      const bool mine = v_row && (direct ? (!split || span == p_row / span_keys)
                                         : (span >= lo / span_keys && span <= p_row / span_keys));
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tc_ld32(t_row + O_COL + c * 32, r);          // every lane of the warp takes part in the load
        if (mine && direct) {
          uint4* dst = reinterpret_cast<uint4*>(out + (row * Hq + head) * D + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            dst[i] = make_uint4(tc_pack(__uint_as_float(r[8 * i]) * inv, __uint_as_float(r[8 * i + 1]) * inv),
                                tc_pack(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv),
                                tc_pack(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv),
                                tc_pack(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv));
        } else if (mine) {
          float4* dst = reinterpret_cast<float4*>(part_o + ((row * Hq + head) * n_spans + span) * D + c * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                                 __uint_as_float(r[4 * i + 3]));
        }
      }
      if (mine && !direct) {
        float* ml = part_ml + ((row * Hq + head) * n_spans + span) * 2;
        ml[0] = m_run * 0.6931471805599453f;              // the join kernel works in natural units
        ml[1] = l_run;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

static int& p_in_tensor_memory() {
  static int on = 1;
  return on;
}

}  // namespace tl

using namespace tl;

// Query rows of one request that fit a tile of the tcgen05 kernel: 128 M rows hold 128 / G query rows of G heads.
extern "C" int tl_attention_tc_tile_rows(int Hq, int Hk) {
  const int G = Hk > 0 ? Hq / Hk : 0;
  return (G >= 1 && G <= TC_M) ? TC_M / G : 0;
}

// Head size 64; pages that tile the 128 keys of a key tile in boxes TMA can send (8 to 128 rows that divide 128, or
// multiples of 128 rows).
extern "C" int tl_attention_tc_supported(int Hq, int Hk, int D, int page_size) {
  if (D != 64 || Hk <= 0 || Hq % Hk != 0 || Hq / Hk > TC_M) return 0;
  return (page_size >= 8 && page_size % 8 == 0 && TC_KT % page_size == 0) || (page_size > 0 && page_size % TC_KT == 0);
}

// Same arguments as tl_paged_attention_mma; tiles hold at most tl_attention_tc_tile_rows query rows. With split, scratch
// holds rows * Hq * n_spans * (D + 2) floats and the caller runs tl_attention_join afterwards when n_spans > 1.
extern "C" int tl_paged_attention_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                     int max_pages, int page_size, int num_pages, const int* tiles, int n_tiles,
                                     int max_tile_rows, const int* positions, float scale, int window, void* out,
                                     float* scratch, int rows, int Hq, int Hk, int D, int n_spans, int split, int* status,
                                     cudaStream_t stream) {
  if (rows == 0 || n_tiles == 0) return 0;
  TL_REQUIRE(tl_attention_tc_supported(Hq, Hk, D, page_size),
             "attention (tcgen05): %d heads over %d KV heads of size %d with pages of %d tokens", Hq, Hk, D, page_size);
  TL_REQUIRE(max_pages > 0 && window >= 0 && num_pages > 0 && scale > 0.f,
             "attention (tcgen05): table width %d, window %d, %d pages, a positive scale", max_pages, window, num_pages);
  TL_REQUIRE(!split || (scratch && n_spans >= 1 && n_spans <= 65535 && split % TC_KT == 0),
             "attention (tcgen05): split over %d spans of %d keys (a multiple of %d) needs scratch", n_spans, split, TC_KT);
  TL_REQUIRE(Hk <= 65535, "attention (tcgen05): %d KV heads exceed the grid limit", Hk);
  TL_REQUIRE(max_tile_rows >= 1 && max_tile_rows <= tl_attention_tc_tile_rows(Hq, Hk),
             "attention (tcgen05): tiles of %d query rows, at most %d fit", max_tile_rows, tl_attention_tc_tile_rows(Hq, Hk));
  TL_REQUIRE(((uintptr_t)q % 16) == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)k_cache % 16) == 0 &&
                 ((uintptr_t)v_cache % 16) == 0 && (!scratch || ((uintptr_t)scratch % 16) == 0),
             "attention (tcgen05): operands must be 16-byte aligned (%d)", 0);
  TL_REQUIRE((long long)num_pages * Hk * page_size < (1LL << 31), "attention (tcgen05): a cache of %d pages is too large", num_pages);
  const bool p_tmem = p_in_tensor_memory() != 0;
  constexpr int RING_S = 3, RING_T = 5;
  constexpr int SMEM_S = TC_M * 64 * 2 + TC_M * TC_KT * 2 + RING_S * TC_KT * 128 + 256 + 1024;
  constexpr int SMEM_T = TC_M * 64 * 2 + RING_T * TC_KT * 128 + 256 + 1024;
  const int SMEM = p_tmem ? SMEM_T : SMEM_S;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel<64, false, RING_S>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_S);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_tc_kernel<64, true, RING_T>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_T);
    if (e != cudaSuccess) return (int)e;
    set = true;
  }
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size;) ++page_shift;
  TcKvMaps maps;
  memset(&maps, 0, sizeof(maps));
  const int box_rows = page_size < TC_KT ? page_size : TC_KT;
  const long long cache_rows = (long long)num_pages * Hk * page_size;
  int e = tensor_map(k_cache, cache_rows, D, D, box_rows, &maps.k);
  if (e == 0) e = tensor_map(v_cache, cache_rows, D, D, box_rows, &maps.v);
  if (e != 0) return e;
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (long long)rows * Hq * n_spans * D : nullptr;
  dim3 grid(n_tiles, Hk, split ? n_spans : 1);
  if (p_tmem)
    return (int)launch_chained(attention_tc_kernel<64, true, RING_T>, grid, dim3(TC_THREADS), SMEM, stream, (const bf16*)q,
                               block_table, max_pages, page_size, page_shift, num_pages, tiles, n_tiles, positions, scale, window,
                               (bf16*)out, part_o, part_ml, n_spans, split, Hq, Hk, status, maps, box_rows);
  return (int)launch_chained(attention_tc_kernel<64, false, RING_S>, grid, dim3(TC_THREADS), SMEM, stream, (const bf16*)q,
                             block_table, max_pages, page_size, page_shift, num_pages, tiles, n_tiles, positions, scale, window,
                             (bf16*)out, part_o, part_ml, n_spans, split, Hq, Hk, status, maps, box_rows);
}

// 1 (the default): P is the MMA's operand from tensor memory; 0: P goes through shared memory (kept for comparison).
extern "C" void tl_attention_tc_p_in_tensor_memory(int on) { p_in_tensor_memory() = on; }

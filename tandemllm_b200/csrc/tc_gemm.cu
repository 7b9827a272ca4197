// bfloat16 matrix products on the 5th-generation tensor cores (tcgen05) for sm_100a:
//
//   C[m, n] = sum_k X[m, k] * W[n, k] (+ bias[n])     X: rows (tokens), W: weight rows, both row-major, k contiguous
//
// One CTA computes one output tile. Operand tiles of 64 k-elements (128 bytes a row) are brought into shared
// memory by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast: every CTA fetches its own tiles) through
// a ring of stages guarded by mbarriers; one elected thread issues tcgen05.mma (kind::f16, bf16 inputs, f32
// accumulation) from shared-memory descriptors into an accumulator in tensor memory; tcgen05.commit releases the
// stage and, after the last k-block, signals the epilogue warps, which read the accumulator with tcgen05.ld,
// apply the bias or silu(gate) * up, and store.
//
// Two orientations share the code. The MMA's M side is always a tile of 128 rows:
//   SWAP    M side = 128 weight rows, N side = BN token rows (16..256). For decode: few tokens, weights streamed
//           once at full TMA rate; thread t of the epilogue owns weight row t, so a store of one token is 32
//           consecutive outputs per warp.
//   !SWAP   M side = 128 token rows, N side = BN weight rows. For prompts: each thread owns a token row and
//           stores BN consecutive outputs.
// SWIGLU: the weight matrix holds gate rows [0, N) and up rows [N, 2N) (per group); the CTA accumulates both for
// the same columns in two accumulators and stores silu(gate) * up.
// Grouped (experts): a tile map built on the device names, per token tile, the group (expert) whose weights it
// multiplies by and the rows of the expert-sorted list it covers; tiles past *n_tiles exit at once.
// Split-K (SWAP, plain): grid.z CTAs each take a range of k-blocks and write 32-bit partial sums to a workspace
// [splits, M, N]; `splitk_reduce` adds them in a fixed order, so results do not depend on timing.
//
// Every wait on an mbarrier is bounded: when a bound is hit the CTA records status 11, stops issuing work, waits
// (bounded again) for the copies it already started, frees its tensor memory and returns.
#include "tma.cuh"

namespace tl {

constexpr int TILE_M = 128;         // rows of the MMA's M side
constexpr int TILE_K = TMA_BOX_COLS;   // k-elements per stage: 128 bytes, one swizzle atom
constexpr int UMMA_K = 16;

struct TcParams {
  void* C;
  const float* bias;
  float* partial;             // split-K workspace or nullptr
  long long ldc;
  int M, N, K;                // tokens, outputs (per group), reduction length
  int k_blocks_per_split;
  long long rows_per_group;   // weight rows per group in the weight tensor (grouped), else 0
  const int* tile_group;
  const int* tile_row0;
  const int* tile_rows;
  const int* n_tiles;
  const int* row_index;       // grouped, swapped: token row of sorted position i is row_index[i] / row_div of X (or nullptr:
  int row_div;                // X is already in sorted order)
  int act;                    // the gate's activation of a gated product (TL_ACT_*), 0 for a plain one
  int skip_kb;                // -1; a test sets the k-block whose copies the producer leaves out, so that a wait runs out
  int* status;
};

inline int& skip_kb_for_test() {
  static int kb = -1;
  return kb;
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and 128-byte swizzle: 8-row groups are
// 1024 bytes apart (stride byte offset), version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                 // leading byte offset (unused for swizzled K-major), in 16-byte units
  d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
  d |= (uint64_t)1 << 46;                 // descriptor version
  d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
  return d;
}

// Instruction descriptor: f32 accumulate, bf16 A and B, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

template <typename TOut> __device__ __forceinline__ void store_out(TOut* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int BN, bool SWAP, bool SWIGLU>
struct Smem {
  static constexpr int A_BYTES = TILE_M * TILE_K * 2;                  // the M-side tile
  static constexpr int B_BYTES = BN * TILE_K * 2;                      // the N-side tile
  // with SWIGLU the weight side is loaded twice (gate rows and up rows)
  static constexpr int W_TILES = SWIGLU ? 2 : 1;
  static constexpr int STAGE_BYTES = SWAP ? (W_TILES * A_BYTES + B_BYTES) : (A_BYTES + W_TILES * B_BYTES);
  // Every form keeps to about half of an SM's shared memory (the swapped gate/up product, with two weight tiles a
  // stage, a little more for a third stage), so that two CTAs share an SM: one's epilogue runs under the other's main loop, and with chained launches the next product's CTA sits
  // beside the running one with its first weight tiles already on the way. Two CTAs an SM also put a decode step's
  // expert tiles (a few hundred CTAs) into one wave.
  // The swapped plain product keeps to a third: its CTAs stream little each (a decode step's down projections are a
  // few hundred CTAs of half a MB), and three an SM put them into one wave.
  static constexpr int BUDGET = SWAP ? (SWIGLU ? 110 * 1024 : 74 * 1024) : 100 * 1024;
  static constexpr int FIT = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = FIT > 8 ? 8 : (FIT < 2 ? 2 : FIT);
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
  static constexpr int TMEM_COLS_RAW = BN * W_TILES;
  static constexpr int TMEM_COLS = TMEM_COLS_RAW <= 32 ? 32 : TMEM_COLS_RAW <= 64 ? 64 : TMEM_COLS_RAW <= 128 ? 128
                                   : TMEM_COLS_RAW <= 256 ? 256 : 512;
};

template <int BN, bool SWAP, bool SWIGLU, typename TOut>
__global__ void __launch_bounds__(192) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmW,
                                                      const __grid_constant__ CUtensorMap tmX, TcParams p) {
  using S = Smem<BN, SWAP, SWIGLU>;
  // Chained launches: the weights are written by no kernel, so a product without a tile map sets itself up and
  // requests its first weight tiles before it waits for the kernels in front of it; only the token rows, and
  // everything a grouped product reads through the tile map, have to wait.
  chain_next();
  if (p.tile_group) chain_wait();
  // ---- which tile ----
  int tok0, tok_rows;
  long long w_base = 0;                 // first weight row of this tile's group in the weight tensor
  const int tok_tile = SWAP ? BN : TILE_M;
  if (p.tile_group) {
    const int t = blockIdx.y;
    if (t >= *p.n_tiles) return;
    tok0 = p.tile_row0[t];
    tok_rows = p.tile_rows[t];
    w_base = (long long)p.tile_group[t] * p.rows_per_group;
  } else {
    tok0 = blockIdx.y * tok_tile;
    tok_rows = min(tok_tile, p.M - tok0);
  }
  const int n0 = blockIdx.x * (SWAP ? TILE_M : BN);        // first output column (weight row within the group)
  const int total_kb = (p.K + TILE_K - 1) / TILE_K;
  const int kb_begin = blockIdx.z * p.k_blocks_per_split;
  const int kb_end = min(total_kb, kb_begin + p.k_blocks_per_split);
  const int num_kb = kb_end - kb_begin;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + S::STAGES * S::STAGE_BYTES);
  uint64_t* empty = full + S::STAGES;
  uint64_t* acc_ready = empty + S::STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_ready + 1);
  volatile uint32_t* aborted = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_ready, 1);
    *aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)S::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // A side = M side (128 rows), B side = N side (BN rows). With SWAP the weights are the A side.
  const CUtensorMap* mapA = SWAP ? &tmW : &tmX;
  const CUtensorMap* mapB = SWAP ? &tmX : &tmW;
  const int rowA = SWAP ? (int)(w_base + n0) : tok0;
  const int rowB = SWAP ? tok0 : (int)(w_base + n0);
  const int rowW2 = (int)(w_base + p.N + n0);               // the up rows (SWIGLU)

  if (warp == 0 && lane == 0) {
    // ---- producer ----
    int issued = 0;
    // With a row index the token rows are fetched one by one from where they lie (a decode step's tiles hold a row
    // or two each); the tile's other rows keep whatever the stage held, and only feed output columns nobody stores.
    const bool gathers = SWAP && p.row_index != nullptr;
    const uint32_t stage_tx = gathers ? (uint32_t)(S::W_TILES * S::A_BYTES + tok_rows * TILE_K * 2) : (uint32_t)S::STAGE_BYTES;
    auto load_weights = [&](int i) {
      const int s = i % S::STAGES;
      uint8_t* st = tiles + s * S::STAGE_BYTES;
      mbar_expect_tx(&full[s], stage_tx);
      const int kx = (kb_begin + i) * TILE_K;
      if (SWAP) {
        tma_load_2d(st, mapA, &full[s], kx, rowA);
        if (SWIGLU) tma_load_2d(st + S::A_BYTES, mapA, &full[s], kx, rowW2);
      } else {
        tma_load_2d(st + S::A_BYTES, mapB, &full[s], kx, rowB);
        if (SWIGLU) tma_load_2d(st + S::A_BYTES + S::B_BYTES, mapB, &full[s], kx, rowW2);
      }
    };
    auto load_tokens = [&](int i) {
      const int s = i % S::STAGES;
      uint8_t* st = tiles + s * S::STAGE_BYTES;
      const int kx = (kb_begin + i) * TILE_K;
      if (gathers) {
        uint8_t* dst = st + S::W_TILES * S::A_BYTES;
        for (int t = 0; t < tok_rows; ++t)
          tma_load_2d(dst + t * (TILE_K * 2), mapB, &full[s], kx, p.row_index[tok0 + t] / p.row_div);
      } else if (SWAP) {
        tma_load_2d(st + S::W_TILES * S::A_BYTES, mapB, &full[s], kx, rowB);
      } else {
        tma_load_2d(st, mapA, &full[s], kx, rowA);
      }
    };
    const int ahead = p.tile_group ? 0 : min(num_kb, S::STAGES);      // the ring's first fill: weights first
    for (int i = 0; i < ahead; ++i)
      if (i != p.skip_kb) load_weights(i);
    if (!p.tile_group) chain_wait();
    for (int i = 0; i < ahead; ++i)
      if (i != p.skip_kb) load_tokens(i);
    issued = ahead;
    for (int i = ahead; i < num_kb; ++i) {
      const int s = i % S::STAGES;
      if (i >= S::STAGES && !mbar_wait(&empty[s], ((i / S::STAGES) - 1) & 1)) {
        *aborted = 1;
        atomicExch(p.status, 11);
        break;
      }
      if (*aborted) break;
      if (i != p.skip_kb) {
        load_weights(i);
        load_tokens(i);
      }
      issued = i + 1;
    }
    if (p.skip_kb >= 0) {       // a test's run: the consumers' wait for the left-out k-block has to run out before the drain
      for (uint32_t spin = 0; spin < wait_limit && !*aborted; ++spin) __nanosleep(256);
    }
    if (*aborted) {
      // copies already started must land before the CTA's shared memory goes away
      for (int i = max(0, issued - S::STAGES); i < issued; ++i)
        if (i != p.skip_kb) mbar_wait(&full[i % S::STAGES], (i / S::STAGES) & 1);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    constexpr uint32_t idesc = umma_idesc(BN);
    for (int i = 0; i < num_kb; ++i) {
      const int s = i % S::STAGES;
      if (!mbar_wait(&full[s], (i / S::STAGES) & 1)) {
        *aborted = 1;
        atomicExch(p.status, 11);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t st = smem_u32(tiles + s * S::STAGE_BYTES);
      const uint32_t a0 = st;
      const uint32_t b0 = st + (SWAP ? S::W_TILES * S::A_BYTES : S::A_BYTES);
#pragma unroll
      for (int k = 0; k < TILE_K / UMMA_K; ++k) {
        const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
        const uint32_t koff = k * UMMA_K * 2;
        umma(tmem_base, umma_desc(a0 + koff), umma_desc(b0 + koff), idesc, acc);
        if (SWIGLU) {
          if (SWAP) umma(tmem_base + BN, umma_desc(a0 + S::A_BYTES + koff), umma_desc(b0 + koff), idesc, acc);
          else umma(tmem_base + BN, umma_desc(a0 + koff), umma_desc(b0 + S::B_BYTES + koff), idesc, acc);
        }
      }
      umma_commit(&empty[s]);
    }
    umma_commit(acc_ready);
  } else if (warp >= 2) {
    // ---- epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. + 31 ----
    const int quad = warp & 3;
    const int m_row = quad * 32 + lane;                  // row of the M side this thread owns
    bool ok = num_kb > 0 ? mbar_wait(acc_ready, 0) : true;
    if (num_kb <= 0) chain_wait();      // an empty k range writes zeros, and nothing else has ordered them behind the kernels in front
    if (!ok) {
      *aborted = 1;
      atomicExch(p.status, 11);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && !*aborted) {
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
      TOut* C = (TOut*)p.C;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16], u[16];
        if (num_kb > 0) {
          tmem_ld16(taddr + c0, v);
          if (SWIGLU) tmem_ld16(taddr + BN + c0, u);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = u[j] = 0.f;
        }
        if (SWAP) {
          // this thread: output column n0 + m_row; registers: tokens tok0 + c0 + j
          const int n = n0 + m_row;
          if (n < p.N) {
            const float b = (p.bias && blockIdx.z == 0) ? p.bias[n] : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = c0 + j;
              if (t < tok_rows) {
                const float r = SWIGLU ? gated(v[j], u[j], p.act) : v[j] + b;
                if (p.partial) p.partial[((long long)blockIdx.z * p.M + tok0 + t) * p.N + n] = r;
                else store_out<TOut>(C + (long long)(tok0 + t) * p.ldc + n, r);
              }
            }
          }
        } else {
          // this thread: token tok0 + m_row; registers: output columns n0 + c0 + j
          if (m_row < tok_rows) {
            TOut* row = C + (long long)(tok0 + m_row) * p.ldc;
            float r[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int n = n0 + c0 + j;
              r[j] = SWIGLU ? gated(v[j], u[j], p.act) : v[j] + ((p.bias && n < p.N) ? p.bias[n] : 0.f);
            }
            // 16 consecutive outputs of one row: 16-byte stores when they are all there and aligned
            const bool whole = n0 + c0 + 16 <= p.N && (((uintptr_t)(row + n0 + c0)) & 15) == 0;
            if (whole) {
              if constexpr (sizeof(TOut) == 2) {
                uint4 lo, hi;
                __nv_bfloat162 t;
#define TL_PACK(dst, a, b) t = __floats2bfloat162_rn(a, b); dst = *reinterpret_cast<uint32_t*>(&t)
                TL_PACK(lo.x, r[0], r[1]); TL_PACK(lo.y, r[2], r[3]); TL_PACK(lo.z, r[4], r[5]); TL_PACK(lo.w, r[6], r[7]);
                TL_PACK(hi.x, r[8], r[9]); TL_PACK(hi.y, r[10], r[11]); TL_PACK(hi.z, r[12], r[13]); TL_PACK(hi.w, r[14], r[15]);
#undef TL_PACK
                uint4* dst = reinterpret_cast<uint4*>(row + n0 + c0);
                dst[0] = lo;
                dst[1] = hi;
              } else {
                float4* dst = reinterpret_cast<float4*>(row + n0 + c0);
#pragma unroll
                for (int j = 0; j < 4; ++j) dst[j] = make_float4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (n0 + c0 + j < p.N) store_out<TOut>(row + n0 + c0 + j, r[j]);
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The prompt-sized product as a persistent kernel: one CTA an SM walks over output tiles of 128 token rows by 256
// weight rows (SWIGLU: 128 gate rows and the 128 up rows of the same outputs, stacked into one 256-row operand, so
// one MMA of N = 256 fills gate in accumulator columns 0..127 and up in 128..255). Three roles run side by side:
//   warp 0      one thread keeps the ring of four 48 KB stages full, across tile borders
//   warp 1      one thread issues the MMAs of a tile into one of two 256-column accumulators in tensor memory
//   warps 2..5  read the finished accumulator (tcgen05.ld), apply bias or silu(gate) * up and store, while the MMAs
//               of the next tile fill the other accumulator
// A 128 x 256 tile reads 48 KB of operands per 2 M multiply-adds, half of what 128 x 128 tiles read, which is what
// the path from L2 can feed. Every wait is bounded as in the kernel above.
struct PersistentSmem {
  static constexpr int A_BYTES = TILE_M * TILE_K * 2;          // 128 token rows
  static constexpr int B_BYTES = 256 * TILE_K * 2;             // 256 weight rows
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 4;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

template <bool SWIGLU, typename TOut>
__global__ void __launch_bounds__(192) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmW,
                                                                 const __grid_constant__ CUtensorMap tmX, TcParams p) {
  using S = PersistentSmem;
  constexpr int OUT_N = SWIGLU ? 128 : 256;            // output columns of a tile
  chain_next();
  chain_wait();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + S::STAGES * S::STAGE_BYTES);
  uint64_t* empty = full + S::STAGES;
  uint64_t* acc_full = empty + S::STAGES;              // [2] the accumulator holds a finished tile
  uint64_t* acc_empty = acc_full + 2;                  // [2] the epilogue has read it
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile uint32_t* aborted = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);                     // one arrival an epilogue warp
    }
    *aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_n = (p.N + OUT_N - 1) / OUT_N;
  const int tiles_m = p.tile_group ? *p.n_tiles : (p.M + TILE_M - 1) / TILE_M;
  const int work = tiles_m * tiles_n;
  const int num_kb = (p.K + TILE_K - 1) / TILE_K;

  // work item w: token tile w / tiles_n, weight tile w % tiles_n (neighbouring CTAs share token rows)
  auto tile_of = [&](int w, int& tok0, int& tok_rows, long long& w_base, int& n0) {
    const int tm = w / tiles_n;
    n0 = (w - tm * tiles_n) * OUT_N;
    if (p.tile_group) {
      tok0 = p.tile_row0[tm];
      tok_rows = p.tile_rows[tm];
      w_base = (long long)p.tile_group[tm] * p.rows_per_group;
    } else {
      tok0 = tm * TILE_M;
      tok_rows = min(TILE_M, p.M - tok0);
      w_base = 0;
    }
  };

  if (warp == 0 && lane == 0) {
    // ---- producer ----
    int it = 0, issued = 0;                            // k-blocks requested so far, over all tiles
    for (int w = blockIdx.x; w < work && !*aborted; w += gridDim.x) {
      int tok0, tok_rows, n0;
      long long w_base;
      tile_of(w, tok0, tok_rows, w_base, n0);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % S::STAGES;
        if (it >= S::STAGES && !mbar_wait(&empty[s], ((it / S::STAGES) - 1) & 1)) {
          *aborted = 1;
          atomicExch(p.status, 11);
        }
        if (*aborted) break;
        uint8_t* st = tiles + s * S::STAGE_BYTES;
        mbar_expect_tx(&full[s], S::STAGE_BYTES);
        const int kx = kb * TILE_K;
        tma_load_2d(st, &tmX, &full[s], kx, tok0);
        if (SWIGLU) {
          tma_load_2d(st + S::A_BYTES, &tmW, &full[s], kx, (int)(w_base + n0));
          tma_load_2d(st + S::A_BYTES + S::B_BYTES / 2, &tmW, &full[s], kx, (int)(w_base + p.N + n0));
        } else {
          tma_load_2d(st + S::A_BYTES, &tmW, &full[s], kx, (int)(w_base + n0));
          tma_load_2d(st + S::A_BYTES + S::B_BYTES / 2, &tmW, &full[s], kx, (int)(w_base + n0 + 128));
        }
        issued = it + 1;
      }
    }
    if (*aborted) {
      // copies already started must land before the CTA's shared memory goes away
      for (int i = max(0, issued - S::STAGES); i < issued; ++i) mbar_wait(&full[i % S::STAGES], (i / S::STAGES) & 1);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    constexpr uint32_t idesc = umma_idesc(256);
    int it = 0, n = 0;                                 // k-blocks and tiles so far
    for (int w = blockIdx.x; w < work && !*aborted; w += gridDim.x, ++n) {
      const int buf = n & 1;
      if (n >= 2 && !mbar_wait(&acc_empty[buf], ((n >> 1) - 1) & 1)) {
        *aborted = 1;
        atomicExch(p.status, 11);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = tmem_base + buf * 256;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % S::STAGES;
        if (!mbar_wait(&full[s], (it / S::STAGES) & 1)) {
          *aborted = 1;
          atomicExch(p.status, 11);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a0 = smem_u32(tiles + s * S::STAGE_BYTES), b0 = a0 + S::A_BYTES;
#pragma unroll
        for (int k = 0; k < TILE_K / UMMA_K; ++k)
          umma(acc, umma_desc(a0 + k * UMMA_K * 2), umma_desc(b0 + k * UMMA_K * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty[s]);
      }
      if (*aborted) break;
      umma_commit(&acc_full[buf]);
    }
  } else if (warp >= 2) {
    // ---- epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. + 31, one token row a thread ----
    const int quad = warp & 3;
    const int m_row = quad * 32 + lane;
    TOut* C = (TOut*)p.C;
    int n = 0;
    for (int w = blockIdx.x; w < work && !*aborted; w += gridDim.x, ++n) {
      int tok0, tok_rows, n0;
      long long w_base;
      tile_of(w, tok0, tok_rows, w_base, n0);
      const int buf = n & 1;
      if (num_kb > 0 && !mbar_wait(&acc_full[buf], (n >> 1) & 1)) {
        *aborted = 1;
        atomicExch(p.status, 11);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * 256;
      TOut* row = C + (long long)(tok0 + m_row) * p.ldc;
#pragma unroll 1
      for (int c0 = 0; c0 < OUT_N; c0 += 16) {
        float v[16], u[16];
        if (num_kb > 0) {
          tmem_ld16(taddr + c0, v);
          if (SWIGLU) tmem_ld16(taddr + 128 + c0, u);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = u[j] = 0.f;
        }
        if (m_row < tok_rows && n0 + c0 < p.N) {
          float r[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int col = n0 + c0 + j;
            r[j] = SWIGLU ? gated(v[j], u[j], p.act) : v[j] + ((p.bias && col < p.N) ? p.bias[col] : 0.f);
          }
          const bool whole = n0 + c0 + 16 <= p.N && (((uintptr_t)(row + n0 + c0)) & 15) == 0;
          if (whole) {
            if constexpr (sizeof(TOut) == 2) {
              uint4 lo, hi;
              __nv_bfloat162 t;
#define TL_PACK(dst, a, b) t = __floats2bfloat162_rn(a, b); dst = *reinterpret_cast<uint32_t*>(&t)
              TL_PACK(lo.x, r[0], r[1]); TL_PACK(lo.y, r[2], r[3]); TL_PACK(lo.z, r[4], r[5]); TL_PACK(lo.w, r[6], r[7]);
              TL_PACK(hi.x, r[8], r[9]); TL_PACK(hi.y, r[10], r[11]); TL_PACK(hi.z, r[12], r[13]); TL_PACK(hi.w, r[14], r[15]);
#undef TL_PACK
              uint4* dst = reinterpret_cast<uint4*>(row + n0 + c0);
              dst[0] = lo;
              dst[1] = hi;
            } else {
              float4* dst = reinterpret_cast<float4*>(row + n0 + c0);
#pragma unroll
              for (int j = 0; j < 4; ++j) dst[j] = make_float4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (n0 + c0 + j < p.N) store_out<TOut>(row + n0 + c0 + j, r[j]);
          }
        }
      }
      // the accumulator may be overwritten once all four warps have read it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u));
  }
}

// out[m, n] = sum over splits (in order) of partial[s, m, n] (+ nothing: the bias went into split 0)
template <typename TOut>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, TOut* __restrict__ out, long long ldc, int M, int N,
                                     int splits) {
  chain_next();
  chain_wait();
  const long long total = (long long)M * N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[(long long)s * total + i];
    const long long m = i / N;
    store_out<TOut>(out + m * ldc + (i - m * N), acc);
  }
}

// rows[i, :] = x[index[i] / div, :]   (the expert-sorted copy of the token rows)
// A warp a row, eight rows a block; a lane's (up to eight) 16-byte pieces of a pass are all loaded before the first is stored.
__global__ void __launch_bounds__(256) gather_rows_kernel(const bf16* __restrict__ x, long long ldx,
                                                          const int* __restrict__ index, int div, bf16* __restrict__ out,
                                                          int width, int rows) {
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (i >= rows) return;
  const uint4* src = (const uint4*)(x + (long long)(index[i] / div) * ldx);
  uint4* dst = (uint4*)(out + (long long)i * width);
  const int n = width / 8;
  for (int c0 = lane; c0 < n; c0 += 8 * 32) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + 32 * j < n) v[j] = src[c0 + 32 * j];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + 32 * j < n) dst[c0 + 32 * j] = v[j];
  }
}

// ------------------------------------------------------------------------------------------ host side
template <int BN, bool SWAP, bool SWIGLU, typename TOut>
static int launch_one(const CUtensorMap& tmW, const CUtensorMap& tmX, const TcParams& p, dim3 grid, cudaStream_t stream) {
  using S = Smem<BN, SWAP, SWIGLU>;
  auto kernel = gemm_tc_kernel<BN, SWAP, SWIGLU, TOut>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)launch_chained(kernel, grid, dim3(192), S::TOTAL, stream, tmW, tmX, p);
}

template <bool SWIGLU, typename TOut>
static int launch_persistent(const CUtensorMap& tmW, const CUtensorMap& tmX, const TcParams& p, dim3 grid, cudaStream_t stream) {
  auto kernel = gemm_tc_persistent_kernel<SWIGLU, TOut>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PersistentSmem::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)launch_chained(kernel, grid, dim3(192), PersistentSmem::TOTAL, stream, tmW, tmX, p);
}

template <bool SWAP, bool SWIGLU, typename TOut>
static int launch_bn(int bn, const CUtensorMap& tmW, const CUtensorMap& tmX, const TcParams& p, dim3 grid, cudaStream_t s) {
  switch (bn) {
    case 16: return launch_one<16, SWAP, SWIGLU, TOut>(tmW, tmX, p, grid, s);
    case 32: return launch_one<32, SWAP, SWIGLU, TOut>(tmW, tmX, p, grid, s);
    case 64: return launch_one<64, SWAP, SWIGLU, TOut>(tmW, tmX, p, grid, s);
    case 128: return launch_one<128, SWAP, SWIGLU, TOut>(tmW, tmX, p, grid, s);
    case 256: return launch_one<256, SWAP, SWIGLU, TOut>(tmW, tmX, p, grid, s);
  }
  tl_set_error("tensor-core gemm: tile of %d rows on the N side; 16, 32, 64, 128 and 256 are built", bn);
  return TL_BAD_ARGUMENT;
}

}  // namespace tl

using namespace tl;

extern "C" const char* tl_tc_last_error() { return tl_error_text; }

// The token-tile height the grouped kernel wants for a given orientation (the MoE plan is built with it).
extern "C" int tl_tc_token_tile(int swap, int bn) { return swap ? bn : TILE_M; }

// bn = 256 without swap selects the persistent kernel (tiles of 128 token rows by 256 weight rows, or by 128 gate and
// 128 up rows with swiglu).

// X [M, K] (row stride ldx), W [groups * rows_per_group, K] (row stride ldw). Plain: groups = 1, tile_group = nullptr.
// swiglu: W holds 2 N rows per group (gate then up) and C = silu(gate) * up. out_dtype: TL_BF16 or TL_FP32.
// splits > 1 (swap, not swiglu): `partial` must hold splits * M * N floats; a grouped product leaves the sums to the caller.
// row_index (swap, grouped; or null): the tile map's rows are positions of this list, and position i stands for row
// row_index[i] / row_div of X; without it X itself is in the tile map's order.
extern "C" int tl_gemm_tc(const void* X, long long ldx, long long x_rows, const void* W, long long ldw, long long w_rows,
                          long long rows_per_group, const float* bias, void* C, long long ldc, int M, int N, int K, int swap,
                          int bn, int swiglu, int out_dtype, const int* tile_group, const int* tile_row0,
                          const int* tile_rows, const int* n_tiles, int max_tiles, const int* row_index, int row_div,
                          int splits, float* partial, int reduce, int* status, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  TL_REQUIRE(M > 0 && N > 0 && K > 0, "tensor-core gemm: M %d N %d K %d", M, N, K);
  TL_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0,
             "tensor-core gemm: K %d and the row strides %lld, %lld must be multiples of 8 elements (16 bytes) for TMA", K,
             ldx, ldw);
  TL_REQUIRE(((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0, "tensor-core gemm: operands must be 16-byte aligned");
  TL_REQUIRE(out_dtype == TL_BF16 || out_dtype == TL_FP32, "tensor-core gemm: output dtype %d", out_dtype);
  TL_REQUIRE(splits >= 1 && (splits == 1 || (swap && !swiglu && partial && (!tile_group || !reduce))),
             "tensor-core gemm: split-K needs the swapped plain kernel and a workspace (grouped: the caller adds the sums)");
  TL_REQUIRE(!bias || !swiglu, "tensor-core gemm: a bias with the gated epilogue is not implemented");
  TL_REQUIRE(swiglu >= 0 && swiglu <= TL_ACT_LAST, "tensor-core gemm: gate activation %d is not one of 0..%d", swiglu, TL_ACT_LAST);
  TL_REQUIRE(!row_index || (swap && tile_group && row_div >= 1),
             "tensor-core gemm: a row index needs the swapped grouped kernel (divisor %d)", row_div);
  CUtensorMap tmW, tmX;
  const bool persistent = !swap && bn == 256;          // the prompt-sized kernel: its weight tiles come as two boxes of 128 rows
  const int w_box = (swap || persistent) ? TILE_M : bn, x_box = row_index ? 1 : (swap ? bn : TILE_M);
  if (int e = tensor_map(W, w_rows, K, ldw, w_box, &tmW)) return e;
  if (int e = tensor_map(X, x_rows, K, ldx, x_box, &tmX)) return e;
  const int total_kb = ceil_div(K, TILE_K);
  TcParams p = {};
  p.C = C; p.bias = bias; p.partial = splits > 1 ? partial : nullptr; p.ldc = ldc; p.M = M; p.N = N; p.K = K;
  p.k_blocks_per_split = ceil_div(total_kb, splits);
  p.rows_per_group = rows_per_group;
  p.tile_group = tile_group; p.tile_row0 = tile_row0; p.tile_rows = tile_rows; p.n_tiles = n_tiles; p.status = status;
  p.row_index = row_index; p.row_div = row_index ? row_div : 1;
  p.act = swiglu;
  p.skip_kb = skip_kb_for_test();
  const int tok_tile = swap ? bn : TILE_M, n_tile = swap ? TILE_M : bn;
  // one CTA layer a split, also where rounding leaves the last splits without k-blocks: they write zeros
  dim3 grid(ceil_div(N, n_tile), tile_group ? max_tiles : ceil_div(M, tok_tile), splits);
  TL_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "tensor-core gemm: grid %u x %u x %u exceeds the limits", grid.x, grid.y, grid.z);
  int e;
  if (persistent) {
    const int out_n = swiglu ? 128 : 256;
    const long long work = (long long)ceil_div(N, out_n) * (tile_group ? max_tiles : ceil_div(M, TILE_M));
    const int sms = sm_count();
    const dim3 pgrid((unsigned)(work < sms ? work : sms));
    if (swiglu) e = out_dtype == TL_BF16 ? launch_persistent<true, bf16>(tmW, tmX, p, pgrid, stream)
                                         : launch_persistent<true, float>(tmW, tmX, p, pgrid, stream);
    else e = out_dtype == TL_BF16 ? launch_persistent<false, bf16>(tmW, tmX, p, pgrid, stream)
                                  : launch_persistent<false, float>(tmW, tmX, p, pgrid, stream);
    return e;
  }
  if (swap) {
    if (swiglu) e = out_dtype == TL_BF16 ? launch_bn<true, true, bf16>(bn, tmW, tmX, p, grid, stream)
                                         : launch_bn<true, true, float>(bn, tmW, tmX, p, grid, stream);
    else e = out_dtype == TL_BF16 ? launch_bn<true, false, bf16>(bn, tmW, tmX, p, grid, stream)
                                  : launch_bn<true, false, float>(bn, tmW, tmX, p, grid, stream);
  } else {
    if (swiglu) e = out_dtype == TL_BF16 ? launch_bn<false, true, bf16>(bn, tmW, tmX, p, grid, stream)
                                         : launch_bn<false, true, float>(bn, tmW, tmX, p, grid, stream);
    else e = out_dtype == TL_BF16 ? launch_bn<false, false, bf16>(bn, tmW, tmX, p, grid, stream)
                                  : launch_bn<false, false, float>(bn, tmW, tmX, p, grid, stream);
  }
  if (e) return e;
  if (splits > 1 && reduce) {     // without `reduce` the caller adds the partial sums itself (fused into its next kernel)
    const long long total = (long long)M * N;
    const int blocks = (int)(ceil_div64(total, 256) < 1184 ? ceil_div64(total, 256) : 1184);
    cudaError_t r;
    if (out_dtype == TL_BF16)
      r = launch_chained(splitk_reduce_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const float*)partial, (bf16*)C, ldc,
                         M, N, (int)grid.z);
    else
      r = launch_chained(splitk_reduce_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)partial, (float*)C,
                         ldc, M, N, (int)grid.z);
    if (r != cudaSuccess) return (int)r;
  }
  return 0;
}

extern "C" void tl_tc_set_chained_launches(int enabled) { chained_launches() = enabled; }

// For tests of the bounded waits: the polls after which an mbarrier wait of this file's kernels gives up (0 puts the
// default back), and the k-block whose copies the plain (not persistent) kernel's producer leaves out (-1: none). With a
// k-block left out the MMA issuer's wait for it runs out: the kernel records status 11, stores nothing, frees its tensor
// memory and returns; nothing waits without a bound, so the next launch finds the GPU as it was.
extern "C" int tl_tc_set_wait_limit(unsigned int polls) {
  const uint32_t v = polls ? polls : (1u << 22);
  return (int)cudaMemcpyToSymbol(wait_limit, &v, sizeof(v));
}
extern "C" void tl_tc_test_skip_k_block(int kb) { skip_kb_for_test() = kb; }

extern "C" int tl_gather_rows(const void* x, long long ldx, const int* index, int div, void* out, int rows, int width,
                              cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(width % 8 == 0 && ldx % 8 == 0 && div >= 1, "gather_rows: width %d, stride %lld, div %d", width, ldx, div);
  gather_rows_kernel<<<ceil_div(rows, 8), 256, 0, stream>>>((const bf16*)x, ldx, index, div, (bf16*)out, width, rows);
  TL_LAUNCH_CHECK();
  return 0;
}

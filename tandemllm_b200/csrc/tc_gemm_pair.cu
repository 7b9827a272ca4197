// Prompt-sized bfloat16 products on pairs of SMs (tcgen05 with cta_group::2) for sm_100a:
//
//   C[m, n] = sum_k X[m, k] * W[n, k] (+ bias[n])      or, gated:  C[m, n] = act(X . Wgate[n]) * (X . Wup[n])
//
// A cluster of two CTAs works on one output tile: 256 outputs (weight rows) by up to 256 token rows. The weights are the MMA's M side: each CTA brings its own 128 weight rows (gated: its 128 gate rows and the
// 128 up rows of the same outputs) and gets their accumulator rows in its own tensor memory. The token rows are the N
// side, which the pair shares: each CTA brings half of them, and one tcgen05.mma issued by the pair's first CTA reads
// both halves, so a token row crosses from L2 into shared memory once per 256 outputs instead of once per 128. That
// path, not the tensor pipe, is what bounds the one-CTA kernel at these sizes.
//
// The N side of an MMA is a run-time number (a multiple of 16 up to 256): a tile of the routed experts' products that
// holds 40 rows costs an MMA of N = 48 and not a padded 128-row one, and its token rows come as a box of 64 rows a CTA
// and not of 128 (three box heights are kept: 16, 64 and 128), so ragged expert sizes cost about what they hold.
//
// Roles in each CTA, as in the one-CTA persistent kernel (tc_gemm.cu): warp 0, one thread, keeps a ring of stages full
// by TMA (plain loads, each CTA its own; their bytes are counted on the first CTA's barrier); warp 1 of the first CTA,
// one thread, issues the MMAs into one of two accumulators and releases stages and accumulators in both CTAs with
// tcgen05.commit; warps 2..9 read a finished accumulator (one output a thread, 16 tokens a load), apply the bias or
// the gate, turn the block through shared memory and store 16 outputs of a token at a time. The plain product has two
// accumulators of 256 columns, so that the next tile's MMAs run under a tile's epilogue; the gated product's gate and
// up accumulators fill all 512 columns, and its MMAs wait for the epilogue while the ring goes on filling: what the
// pair saves on the way from L2 (48 KB a CTA for 2 x 128 x 256 x 64 multiply-adds, against 40 KB for half of them
// with tiles of 128 token rows) is worth more than the overlap. The kernel is persistent: as many clusters as fit the
// GPU walk over the tiles.
//
// Every wait on an mbarrier is bounded: when a bound is hit the CTA records status 11 and tells its peer, both stop
// issuing work, the first CTA waits (bounded again) for the copies in flight, the pair meets at the cluster barrier,
// frees its tensor memory and returns.
#include "tma.cuh"

namespace tl {

namespace pair {

constexpr int ROWS = 128;               // weight rows a CTA, and the height of one TMA box of weights
constexpr int TILE_K = TMA_BOX_COLS;    // k-elements a stage: 128 bytes, one swizzle atom
constexpr int UMMA_K = 16;

struct Params {
  void* C;
  const float* bias;
  long long ldc;
  int M, N, K;                // tokens, outputs (per group), reduction length
  long long rows_per_group;   // weight rows per group in the weight tensor (grouped), else 0
  const int* tile_group;
  const int* tile_row0;
  const int* tile_rows;
  const int* n_tiles;
  int plan_rows;              // the height of the tile map's tiles, at most TOKENS
  int act;                    // the gate's activation (TL_ACT_*), 0 for a plain product
  int skip_kb;                // -1; a test sets the k-block (counted over a cluster's tiles) whose copies both producers leave out
  int splits;                 // plain, ungrouped: work items a tile, each a run of k-blocks with a 32-bit partial result of its own
  int kb_per_split;           // k-blocks a run (every run holds at least one)
  long long part_stride;      // elements from one run's [M, ldc] result to the next one's
  int* status;
};

inline int& skip_kb_for_test() {
  static int kb = -1;
  return kb;
}

// PER_SM: CTAs an SM. One: the forms described above. Two: half the shared memory and half the tensor memory each (the
// gated product then takes tiles of 128 token rows, gate and up accumulators of 128 columns; one accumulator set, so the
// other CTA of the SM is what runs under an epilogue). Twice the pairs are resident, which is what a product bound by
// its weights wants: its work items all cost the same (what their weight tiles take to load), and when the last round
// leaves an SM with one CTA instead of two, that CTA loads at the SM's full rate. Measured on the experts' two products
// of 128 to 512 tokens (32 experts, 16 to 64 rows each): 170 to 176 us -> 158 to 164 us; from 128 rows an expert on the
// form with one CTA an SM and its deeper ring is faster again.
template <bool GATED, int PER_SM>
struct Smem {
  static constexpr int TOKENS = (GATED && PER_SM == 2) ? 128 : 256;  // token rows a tile at most
  static constexpr int W_TILES = GATED ? 2 : 1;
  static constexpr int ACC_BUFS = (GATED || PER_SM == 2) ? 1 : 2;  // accumulators (sets of them) in tensor memory
  static constexpr int TMEM_COLS = PER_SM == 2 ? 256 : 512;
  static constexpr int UP_COL = TOKENS;                            // the gated product's second accumulator
  // Epilogue warps: one a quarter of the accumulator's lanes, or, where the MMAs wait for the epilogue, two that take
  // every other block of 16 tokens (measured: the plain product is a little slower with eight)
  static constexpr int EPI_WARPS = GATED ? 8 : 4;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int A_BYTES = ROWS * TILE_K * 2;                // one box of weights
  static constexpr int B_BYTES = (TOKENS / 2) * TILE_K * 2;        // this CTA's half of the token rows, at most
  static constexpr int STAGE_BYTES = W_TILES * A_BYTES + B_BYTES;
  static constexpr int STAGES = PER_SM == 2 ? (GATED ? 2 : 3) : (GATED ? 4 : 6);
  static constexpr int TURN_BYTES = EPI_WARPS * 16 * 32 * 4;       // the epilogue warps' blocks
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ + TURN_BYTES;
  static_assert(PER_SM * TOTAL <= 227 * 1024, "the CTAs of an SM share its shared memory");
};

// K-major tile with 128-byte rows and the 128-byte swizzle: 8-row groups 1024 bytes apart, descriptor version 1.
__device__ __forceinline__ uint64_t desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// f32 accumulate, bf16 A and B, both K-major, M = 256 over the pair, N = n
__device__ __forceinline__ uint32_t idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

__device__ __forceinline__ void mma2(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t id, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(id), "r"(accumulate)
      : "memory");
}

// arrives, once the MMAs issued so far are done, on the barrier at this address in both CTAs of the pair
__device__ __forceinline__ void commit_both(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// the address, in the cluster's shared window, of `p` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t in_cta(const void* p, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
  return a;
}

__device__ __forceinline__ void arrive_at(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void store_at(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// One box from (column x, row y) into this CTA's shared memory; its bytes are counted on the barrier at `bar_addr`,
// which lies in the pair's first CTA. No multicast: the box goes to this CTA alone.
__device__ __forceinline__ void load_2d(void* dst, const CUtensorMap* map, uint32_t bar_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_addr), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void ld16(uint32_t taddr, float* v) {
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

template <typename TOut> __device__ __forceinline__ void put(TOut* p, float v);
template <> __device__ __forceinline__ void put<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void put<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <bool GATED, int PER_SM, typename TOut>
__global__ void __launch_bounds__(Smem<GATED, PER_SM>::THREADS, PER_SM) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmW,
                                                           const __grid_constant__ CUtensorMap tmX16,
                                                           const __grid_constant__ CUtensorMap tmX64,
                                                           const __grid_constant__ CUtensorMap tmX128, Params p) {
  using S = Smem<GATED, PER_SM>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + S::STAGES * S::STAGE_BYTES);   // used in the first CTA: both CTAs' bytes
  uint64_t* empty = full + S::STAGES;                                  // in each CTA: the MMAs have read the stage
  uint64_t* acc_full = empty + S::STAGES;                              // [2] in each CTA: a tile's accumulator is done
  uint64_t* acc_empty = acc_full + 2;                                  // [2] used in the first CTA: both epilogues read it
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile uint32_t* aborted = tmem_slot + 1;
  float* turns = (float*)(tiles + S::STAGES * S::STAGE_BYTES + 256);   // [warps][16 tokens][32 outputs]: see the epilogue

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool first = rank == 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 2 * S::EPI_WARPS);         // one arrival an epilogue warp of either CTA
    }
    *aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // the same warp of both CTAs: the pair's tensor memory is given out, and later freed, together
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)S::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();                                      // the peer's barriers are initialised before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t peer_aborted = in_cta((const void*)aborted, rank ^ 1u);

  auto give_up = [&]() {
    *aborted = 1;
    store_at(peer_aborted, 1u);
    atomicExch(p.status, 11);
  };

  const int tiles_n = (p.N + 2 * ROWS - 1) / (2 * ROWS);
  const int tiles_m = p.tile_group ? *p.n_tiles : (p.M + S::TOKENS - 1) / S::TOKENS;
  const int work = tiles_m * tiles_n * p.splits;
  const int all_kb = (p.K + TILE_K - 1) / TILE_K;
  const int cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;

  // work item w: token tile w / tiles_n, weight tile w % tiles_n (neighbouring clusters share token rows); with runs of
  // k-blocks, run w / (tiles_m tiles_n) of that tile
  auto tile_of = [&](int w, int& tok0, int& tok_rows, long long& w_base, int& n0, int& kb0, int& num_kb) {
    const int run = w / (tiles_m * tiles_n);
    w -= run * tiles_m * tiles_n;
    kb0 = run * p.kb_per_split;
    num_kb = p.splits > 1 ? min(p.kb_per_split, all_kb - kb0) : all_kb;
    const int tm = w / tiles_n;
    n0 = (w - tm * tiles_n) * 2 * ROWS;
    if (p.tile_group) {
      tok0 = p.tile_row0[tm];
      tok_rows = min(p.tile_rows[tm], S::TOKENS);
      w_base = (long long)p.tile_group[tm] * p.rows_per_group;
    } else {
      tok0 = tm * S::TOKENS;
      tok_rows = min(S::TOKENS, p.M - tok0);
      w_base = 0;
    }
  };

  if (warp == 0 && lane == 0) {
    // ---- producer (each CTA for its own shared memory) ----
    int it = 0, issued = 0;
    for (int w = cluster; w < work && !*aborted; w += clusters) {
      int tok0, tok_rows, n0, kb0, num_kb;
      long long w_base;
      tile_of(w, tok0, tok_rows, w_base, n0, kb0, num_kb);
      if (tok_rows <= 0) continue;
      const int n_mma = (tok_rows + 15) & ~15;
      const int half = n_mma >> 1;
      const int my_tok = tok0 + (int)rank * half;                    // this CTA's half of the N side
      const int my_row = (int)(w_base + n0) + (int)rank * ROWS;      // this CTA's 128 outputs
      // the smallest box that holds the half; rows of it behind the half are read and never used
      const int box = half <= 16 ? 16 : (half <= 64 ? 64 : 128);      // (a half is at most TOKENS / 2 rows)
      const CUtensorMap* tmX = box == 16 ? &tmX16 : (box == 64 ? &tmX64 : &tmX128);
      const uint32_t cta_bytes = (uint32_t)(S::W_TILES * S::A_BYTES + box * TILE_K * 2);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % S::STAGES;
        if (it >= S::STAGES && !mbar_wait(&empty[s], ((it / S::STAGES) - 1) & 1)) give_up();
        if (*aborted) break;
        if (it != p.skip_kb) {
          uint8_t* st = tiles + s * S::STAGE_BYTES;
          const uint32_t bar = in_cta(&full[s], 0);
          if (first) mbar_expect_tx(&full[s], 2 * cta_bytes);
          const int kx = (kb0 + kb) * TILE_K;
          load_2d(st, &tmW, bar, kx, my_row);
          if (GATED) load_2d(st + S::A_BYTES, &tmW, bar, kx, my_row + p.N);
          load_2d(st + S::W_TILES * S::A_BYTES, tmX, bar, kx, my_tok);
        }
        issued = it + 1;
      }
    }
    if (*aborted && first) {
      // copies already started (the peer's are counted here too) must land before the shared memory goes away
      for (int i = max(0, issued - S::STAGES); i < issued; ++i)
        if (i != p.skip_kb) mbar_wait(&full[i % S::STAGES], (i / S::STAGES) & 1);
    }
  } else if (warp == 1 && lane == 0 && first) {
    // ---- MMA issuer (the first CTA for the pair) ----
    int it = 0, n = 0;
    for (int w = cluster; w < work && !*aborted; w += clusters) {
      int tok0, tok_rows, n0, kb0, num_kb;
      long long w_base;
      tile_of(w, tok0, tok_rows, w_base, n0, kb0, num_kb);
      if (tok_rows <= 0) continue;
      const int n_mma = (tok_rows + 15) & ~15;
      const uint32_t id = idesc(n_mma);
      const int buf = n % S::ACC_BUFS, round = n / S::ACC_BUFS;
      if (round >= 1 && !mbar_wait(&acc_empty[buf], (round - 1) & 1)) {
        give_up();
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = tmem_base + buf * 256;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % S::STAGES;
        if (!mbar_wait(&full[s], (it / S::STAGES) & 1)) {
          give_up();
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a0 = smem_u32(tiles + s * S::STAGE_BYTES), b0 = a0 + S::W_TILES * S::A_BYTES;
#pragma unroll
        for (int k = 0; k < TILE_K / UMMA_K; ++k) {
          const uint32_t more = (kb > 0 || k > 0) ? 1u : 0u, koff = k * UMMA_K * 2;
          mma2(acc, desc(a0 + koff), desc(b0 + koff), id, more);
          if (GATED) mma2(acc + S::UP_COL, desc(a0 + S::A_BYTES + koff), desc(b0 + koff), id, more);
        }
        commit_both(&empty[s]);
      }
      if (*aborted) break;
      commit_both(&acc_full[buf]);
      ++n;
    }
  } else if (warp >= 2) {
    // ---- epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. + 31, one output a thread; the two warps of a
    // quarter take every other block of 16 tokens ----
    const int quad = warp & 3, turn_of = (warp - 2) >> 2;
    const int m_row = quad * 32 + lane;
    float* turn = turns + (warp - 2) * (16 * 32);
    TOut* C = (TOut*)p.C;
    int n = 0;
    if (p.tile_group && p.plan_rows > S::TOKENS && threadIdx.x == 64) atomicExch(p.status, 5);   // taller tiles than the kernel takes
    for (int w = cluster; w < work && !*aborted; w += clusters) {
      int tok0, tok_rows, n0, kb0, num_kb;
      long long w_base;
      tile_of(w, tok0, tok_rows, w_base, n0, kb0, num_kb);
      if (tok_rows <= 0) continue;
      const int n_mma = (tok_rows + 15) & ~15;
      const int buf = n % S::ACC_BUFS, round = n / S::ACC_BUFS;
      if (num_kb > 0 && !mbar_wait(&acc_full[buf], round & 1)) {
        give_up();
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * 256;
      const int col = n0 + (int)rank * ROWS + m_row;                 // this thread's output
      const float b = (!GATED && p.bias && col < p.N && kb0 == 0) ? p.bias[col] : 0.f;
      const int j_tok = lane >> 1, c_half = (lane & 1) * 16;        // after the turn: token c0 + j_tok, 16 outputs
      const int out0 = n0 + (int)rank * ROWS + quad * 32 + c_half;
#pragma unroll 1
      for (int c0 = 16 * turn_of; c0 < n_mma; c0 += 16 * (S::EPI_WARPS / 4)) {
        float v[16], u[16];
        if (num_kb > 0) {
          ld16(taddr + c0, v);
          if (GATED) ld16(taddr + S::UP_COL + c0, u);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = u[j] = 0.f;
        }
        // The thread holds 16 tokens of one output; a store wants 16 outputs of one token. The warp turns its block of
        // 16 tokens by 32 outputs through shared memory: row j (a token) is 32 words, rotated by 4 j words so that
        // neither the writes (a row a time, a word a lane) nor the 16-byte reads meet in a bank.
        if (GATED) {
          // The gated product's MMAs wait for this loop, so it is written for speed: the choice of the activation
          // stands outside the 16 independent evaluations, and SiLU, the usual one, takes the fast exponential and
          // division (the result is rounded to bfloat16, far coarser than their error).
          if (p.act == TL_ACT_SILU) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __fdividef(v[j], 1.f + __expf(-v[j])) * u[j];
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = gated(v[j], u[j], p.act);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] += b;
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 16; ++j) turn[j * 32 + ((lane + 4 * j) & 31)] = v[j];
        __syncwarp();
        float r[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 q = *reinterpret_cast<const float4*>(turn + j_tok * 32 + ((c_half + 4 * i + 4 * j_tok) & 31));
          r[4 * i] = q.x; r[4 * i + 1] = q.y; r[4 * i + 2] = q.z; r[4 * i + 3] = q.w;
        }
        const int t = c0 + j_tok;
        if (t < tok_rows && out0 < p.N) {
          TOut* dst = C + (kb0 / p.kb_per_split) * p.part_stride + (long long)(tok0 + t) * p.ldc + out0;
          if (out0 + 16 <= p.N && (((uintptr_t)dst) & 15) == 0) {
            if constexpr (sizeof(TOut) == 2) {
              uint4 lo, hi;
              __nv_bfloat162 h2;
#define TL_PACK(dst_, a_, b_) h2 = __floats2bfloat162_rn(a_, b_); dst_ = *reinterpret_cast<uint32_t*>(&h2)
              TL_PACK(lo.x, r[0], r[1]); TL_PACK(lo.y, r[2], r[3]); TL_PACK(lo.z, r[4], r[5]); TL_PACK(lo.w, r[6], r[7]);
              TL_PACK(hi.x, r[8], r[9]); TL_PACK(hi.y, r[10], r[11]); TL_PACK(hi.z, r[12], r[13]); TL_PACK(hi.w, r[14], r[15]);
#undef TL_PACK
              reinterpret_cast<uint4*>(dst)[0] = lo;
              reinterpret_cast<uint4*>(dst)[1] = hi;
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                reinterpret_cast<float4*>(dst)[i] = make_float4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (out0 + i < p.N) put<TOut>(dst + i, r[i]);
          }
        }
      }
      // the accumulator may be overwritten once the epilogue warps of both CTAs have read it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) arrive_at(in_cta(&acc_empty[buf], 0));
      ++n;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();                                      // neither CTA leaves while the other may still signal it or read its tiles
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS));
  }
}

// How many pairs of this kernel the GPU holds at a time (asked once a kernel); negative: a CUDA error code, negated.
template <bool GATED, int PER_SM, typename TOut>
static int resident_pairs() {
  using S = Smem<GATED, PER_SM>;
  static int clusters = 0;
  if (clusters != 0) return clusters;
  auto kernel = gemm_tc_pair_kernel<GATED, PER_SM, TOut>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
  if (e != cudaSuccess) return -(int)e;
  // all of the SM's configurable memory as shared memory: two CTAs an SM need it
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return -(int)e;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(2 * PER_SM * (sm_count() / 2));
  cfg.blockDim = dim3(S::THREADS);
  cfg.dynamicSmemBytes = S::TOTAL;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
  if (e != cudaSuccess) return -(int)e;
  clusters = n;
  // Two CTAs an SM: the query answers as if a pair had the two SMs to itself (74), yet two pairs do share them
  // (ncu: 296 CTAs are one wave, 20 warps active an SM). No pair waits for another in this kernel, so a grid of twice
  // the pairs is safe either way: on a GPU that held only one CTA an SM the others would simply start later.
  if (PER_SM == 2 && n >= 1) clusters = 2 * (sm_count() / 2);
  return clusters;
}

template <bool GATED, int PER_SM, typename TOut>
static int launch(const CUtensorMap& tmW, const CUtensorMap* tmX, const Params& p, long long work, cudaStream_t stream) {
  using S = Smem<GATED, PER_SM>;
  const int clusters = resident_pairs<GATED, PER_SM, TOut>();
  if (clusters < 0) return -clusters;
  TL_REQUIRE(clusters >= 1, "pair product: no cluster of two CTAs with %d bytes of shared memory fits this GPU", S::TOTAL);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3((unsigned)(2 * (work < clusters ? work : clusters)));
  cfg.blockDim = dim3(S::THREADS);
  cfg.dynamicSmemBytes = S::TOTAL;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<GATED, PER_SM, TOut>, tmW, tmX[0], tmX[1], tmX[2], p);
}

}  // namespace pair
}  // namespace tl

using namespace tl;

// The token rows a tile of the pair kernel holds at most (a routing plan for it is built with tiles of this height).
extern "C" int tl_tc_pair_token_tile(int per_sm) {
  return per_sm == 2 ? pair::Smem<true, 2>::TOKENS : pair::Smem<true, 1>::TOKENS;      // what the gated product takes
}

extern "C" int tl_tc_pair_resident(int gated, int per_sm) {
  if (per_sm == 2) return gated ? pair::resident_pairs<true, 2, bf16>() : pair::resident_pairs<false, 2, bf16>();
  return gated ? pair::resident_pairs<true, 1, bf16>() : pair::resident_pairs<false, 1, bf16>();
}

// X [M, K] (row stride ldx, x_rows rows in the tensor), W [groups * rows_per_group, K] (row stride ldw). Plain: groups = 1,
// tile_group = nullptr. gated (an activation code TL_ACT_*, or 0): W holds 2 N rows per group (gate then up) and
// C = act(gate) * up. out_dtype: TL_BF16 or TL_FP32. Grouped: the tile map's tiles hold at most tl_tc_pair_token_tile()
// rows (plan_rows: the height the map was built with). per_sm: 1 or 2 CTAs an SM (see Smem). splits > 1 (plain, ungrouped,
// 32-bit output): the reduction is cut into `splits` runs of k-blocks, each a work item of its own, and C receives the
// runs' partial results one behind the other, [splits, M, ldc], for the caller to add in order (a product with fewer
// tiles than the GPU has pairs of SMs: a pair streams a tile's operands at the rate of its two SMs whatever else is idle).
extern "C" int tl_gemm_tc_pair(const void* X, long long ldx, long long x_rows, const void* W, long long ldw, long long w_rows,
                               long long rows_per_group, const float* bias, void* C, long long ldc, int M, int N, int K,
                               int gated, int out_dtype, const int* tile_group, const int* tile_row0, const int* tile_rows,
                               const int* n_tiles, int max_tiles, int plan_rows, int per_sm, int splits, int* status,
                               cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  TL_REQUIRE(M > 0 && N > 0 && K > 0, "pair product: M %d N %d K %d", M, N, K);
  TL_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0,
             "pair product: K %d and the row strides %lld, %lld must be multiples of 8 elements (16 bytes) for TMA", K, ldx, ldw);
  TL_REQUIRE(((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0, "pair product: operands must be 16-byte aligned (%d)", 0);
  TL_REQUIRE(out_dtype == TL_BF16 || out_dtype == TL_FP32, "pair product: output dtype %d", out_dtype);
  TL_REQUIRE(!bias || !gated, "pair product: a bias with the gated epilogue is not implemented (%d)", gated);
  TL_REQUIRE(gated >= 0 && gated <= TL_ACT_LAST, "pair product: gate activation %d is not one of 0..%d", gated, TL_ACT_LAST);
  TL_REQUIRE(!tile_group || (tile_row0 && tile_rows && n_tiles && max_tiles > 0 && plan_rows > 0),
             "pair product: incomplete tile map (tiles of %d rows)", plan_rows);
  TL_REQUIRE(per_sm == 1 || per_sm == 2, "pair product: %d CTAs an SM; 1 or 2", per_sm);
  const int all_kb = ceil_div(K, pair::TILE_K);
  TL_REQUIRE(splits >= 1 && splits <= all_kb, "pair product: %d runs of k-blocks; the reduction has %d k-blocks", splits, all_kb);
  const int kb_per_split = ceil_div(all_kb, splits);
  TL_REQUIRE(splits == 1 || (!gated && !tile_group && out_dtype == TL_FP32 && (long long)(splits - 1) * kb_per_split < all_kb),
             "pair product: runs of k-blocks need the plain, ungrouped product with 32-bit output, and none may be empty (%d runs)",
             splits);
  const int tokens = (gated && per_sm == 2) ? 128 : 256;
  TL_REQUIRE(!tile_group || plan_rows <= tokens, "pair product: a tile map with tiles of %d rows; at most %d", plan_rows, tokens);
  CUtensorMap tmW, tmX[3];
  if (int e = tensor_map(W, w_rows, K, ldw, pair::ROWS, &tmW)) return e;
  if (int e = tensor_map(X, x_rows, K, ldx, 16, &tmX[0])) return e;
  if (int e = tensor_map(X, x_rows, K, ldx, 64, &tmX[1])) return e;
  if (int e = tensor_map(X, x_rows, K, ldx, 128, &tmX[2])) return e;
  pair::Params p = {};
  p.C = C; p.bias = bias; p.ldc = ldc; p.M = M; p.N = N; p.K = K;
  p.rows_per_group = rows_per_group;
  p.tile_group = tile_group; p.tile_row0 = tile_row0; p.tile_rows = tile_rows; p.n_tiles = n_tiles;
  p.plan_rows = plan_rows;
  p.act = gated; p.status = status;
  p.skip_kb = pair::skip_kb_for_test();
  p.splits = splits; p.kb_per_split = kb_per_split; p.part_stride = splits > 1 ? (long long)M * ldc : 0;
  const long long work = (long long)ceil_div(N, 2 * pair::ROWS) * (tile_group ? max_tiles : ceil_div(M, tokens)) * splits;
#define TL_PAIR(G_, P_) \
  (out_dtype == TL_BF16 ? pair::launch<G_, P_, bf16>(tmW, tmX, p, work, stream) : pair::launch<G_, P_, float>(tmW, tmX, p, work, stream))
  if (per_sm == 2) return gated ? TL_PAIR(true, 2) : TL_PAIR(false, 2);
  return gated ? TL_PAIR(true, 1) : TL_PAIR(false, 1);
#undef TL_PAIR
}

// For tests of the bounded waits, as in tc_gemm.cu: the polls after which an mbarrier wait of this file's kernel gives up
// (0 puts the default back), and the k-block whose copies the producers of both CTAs leave out (-1: none). The MMA
// issuer's wait for it then runs out: the pair records status 11, each CTA tells the other, every role stops at its
// next wait, the pair meets at the cluster barrier, frees its tensor memory and returns.
extern "C" int tl_tc_pair_set_wait_limit(unsigned int polls) {
  const uint32_t v = polls ? polls : (1u << 22);
  return (int)cudaMemcpyToSymbol(wait_limit, &v, sizeof(v));
}
extern "C" void tl_tc_pair_test_skip_k_block(int kb) { pair::skip_kb_for_test() = kb; }

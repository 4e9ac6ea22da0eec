// bfloat16 matrix product of the linear layers for steps of many tokens, on pairs of multiprocessors:
//   out[T, N] = x[T, K] . w[N, K]^T            (float32 accumulation, one rounding at the store)
//
// Two CTAs of a thread-block cluster work on one 256 x 256 tile (256 tokens by 256 weight rows) with
// tcgen05.mma.cta_group::2: each CTA brings 128 token rows (its half of the M side) and 128 weight
// rows (its half of the N side) of every 64-element k-block through TMA into its own shared memory,
// one thread of the pair's first CTA issues the product for both, and each CTA ends up with its 128
// tokens by all 256 weight rows in its own tensor memory.  Against two independent CTAs this halves
// the operand bytes every CTA reads from shared memory per product, which is what bounds a single
// CTA's 128 x 256 tile.
//
// The tokens are the accumulator's lanes, so a thread of the epilogue owns a token's row of the tile:
// it writes 16 bytes at a time along a row of the result, and what a layer does to a row is the thread's
// own business: the scale that a norm before the product left open, a bias, SiLU(gate) * up (the first CTA
// brings 128 gate rows, the second the 128 up rows that belong to them, and every thread finds both in its
// lane), and the norm that follows (the product is added to the float32 residual, the result is the new
// residual times the norm's weight, and the sums of squares of every 32 columns go to a table that the
// next product turns into the row's scale).  A tile leaves through shared memory (128-byte swizzle, so that
// 32 rows written at once do not meet in a bank) and TMA stores.
//
// The kernel is persistent and deals the work out evenly whatever the shape: the (tile, k-block) units
// of the whole product, tile after tile (token tile fastest, so that the pairs running at one time share
// weight rows and activations in L2), are cut into as many equal runs as there are pairs.  A run begins
// and ends in the middle of a tile, so a tile's k-range may be shared by two or more pairs.  The pair
// that holds a tile's first k-blocks owns the tile: the others (for which that segment is the first
// thing they do) leave their float32 partial tiles in global scratch and count themselves in; the owner,
// which reaches the tile at the end of its run, adds them to its accumulator in run order and stores.
// Nothing waits for work that has not started, and the sum does not depend on timing.  Without this,
// 192 tiles on 74 pairs take three rounds for 2.6 rounds of work.  Roles per CTA:
// warp 0 copies (TMA; the copies of both CTAs complete on the first CTA's barrier; the weights of the
// first stages leave before griddepcontrol.wait, the tokens' after it), warp 1 of the
// first CTA issues products and commits to the barriers of both, warps 2..5 read the accumulator
// (two buffers of 256 tensor-memory columns, so a tile's epilogue overlaps the next tile's products)
// and store.  No copy here is a multicast: each CTA fetches its own halves.
//
// Every mbarrier wait is bounded by time; the two cluster barriers (after set-up, before exit) are
// reached by every thread on every path.
//
// The reference calls a library product here (rapid_llm/kernels/ops/gemm/linear.py:17-40) and runs the
// activation and the norms as kernels of their own (rapid_llm/kernels/ops/activation/swiglu.py:91-121,
// rapid_llm/kernels/ops/layernorm/skip_rmsnorm.py:41-48).
#include <cuda.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace rl {

using bf16 = __nv_bfloat16;

constexpr int kPairRows = 128;            // tokens per CTA = lanes of its accumulator; also its weight rows of a tile
constexpr int kPairCols = 2 * kPairRows;  // columns of the accumulator: the weight rows of the pair's tile
constexpr int kPairTokens = 2 * kPairRows;  // tokens of the pair's tile
constexpr int kPairTileK = 64;
constexpr int kPairThreads = 192;
constexpr int kPairMaxTiles = 4096;       // tiles of one product (two counters each)
constexpr int kPairStageBytes = 2 * kPairRows * kPairTileK * 2;     // 128 token rows and 128 weight rows of a k-block
constexpr int kPairSubTileBytes = kPairRows * 128;                  // 128 tokens by 64 columns of the result, swizzled
constexpr int kPairStagingBytes = (kPairCols / 64) * kPairSubTileBytes;
constexpr int kPairStages = 4;
constexpr size_t kPairSmemBytes = static_cast<size_t>(kPairStages) * kPairStageBytes + kPairStagingBytes + 1024;
constexpr int kPairTmemColumns = 2 * kPairCols;                     // two accumulators
constexpr uint32_t kPairIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kPairCols >> 3) << 17) |
                                (static_cast<uint32_t>(kPairTokens >> 4) << 24);
constexpr size_t kPairPartialFloats = static_cast<size_t>(kPairCols) * kPairRows;     // one CTA's partial tile
static_assert(kPairSmemBytes <= 227 * 1024 && kPairTmemColumns == 512, "a CTA's shared and tensor memory");

struct PairArgs {
  int* fault;
  int T, N, K;             // N: columns of the result (SwiGLU: the intermediate size; w has 2 N rows, the gate's first)
  int n_tiles, t_tiles, k_blocks;
  int out_cols;            // columns of the result per tile: 256, SwiGLU 128
  int pdl;
  const float* bias;       // [N] (SwiGLU: [2 N]) or null
  // a norm that came before and left its scale open: row t is multiplied by rsqrt(sum(sumsq_in[t, :]) * inv + eps)
  const float* sumsq_in;
  int sumsq_count;
  float norm_eps, inv_norm_size;
  // a norm that follows: residual[T, N] += result; out = bf16(residual * norm_weight); sumsq_out[t, slot of 32 columns]
  float* residual;
  const float* norm_weight;
  float* sumsq_out;
  int sumsq_out_count;
  float* scratch;      // [pairs][2][256][128]: the partial tile of a pair's first segment, per CTA
  unsigned* counters;  // [tiles][2]: partial tiles stored so far, per CTA rank; zero between launches
};

// What one pair does, in order.  Whole rounds of tiles are dealt round-robin (the pairs running at one time then
// work on neighbouring tiles and share their operands in L2).  The tiles left over, fewer than there are pairs,
// come first and are not dealt whole: their (tile, k-block) units are cut into equal runs, one per pair, so a
// pair's run begins and ends inside a tile.
struct PairRun {
  long long u, end;          // this pair's run of the left-over tiles' units
  int next_whole, tiles, pairs, k_blocks;
  __device__ __forceinline__ static int leftover(int tiles, int pairs) { return tiles % pairs; }
  // pairs that share the left-over tiles: a run is at least eight k-blocks
  __device__ __forceinline__ static int sharers(int tiles, int pairs, int k_blocks) {
    const long long units = static_cast<long long>(leftover(tiles, pairs)) * k_blocks;
    const long long most = units / 8;
    return most < 1 ? 1 : (most < pairs ? static_cast<int>(most) : pairs);
  }
  __device__ __forceinline__ static long long run_begin(int tiles, int pairs, int k_blocks, int pair) {
    const long long units = static_cast<long long>(leftover(tiles, pairs)) * k_blocks;
    const int share = sharers(tiles, pairs, k_blocks);
    return pair >= share ? units : units * pair / share;
  }
  __device__ __forceinline__ PairRun(const PairArgs& args, int pair, int pairs_) {
    tiles = args.n_tiles * args.t_tiles;
    pairs = pairs_;
    k_blocks = args.k_blocks;
    u = run_begin(tiles, pairs, k_blocks, pair);
    end = run_begin(tiles, pairs, k_blocks, pair + 1);
    next_whole = leftover(tiles, pairs) + pair;
  }
  __device__ __forceinline__ bool next(int& tile, int& kb0, int& len) {
    if (u < end) {
      tile = static_cast<int>(u / k_blocks);
      kb0 = static_cast<int>(u - static_cast<long long>(tile) * k_blocks);
      const long long left = end - u;
      len = k_blocks - kb0 < left ? k_blocks - kb0 : static_cast<int>(left);
      u += len;
      return true;
    }
    if (next_whole < tiles) {
      tile = next_whole;
      kb0 = 0;
      len = k_blocks;
      next_whole += pairs;
      return true;
    }
    return false;
  }
};

// ---- the cta_group::2 forms of the tensor-core instructions ----
__device__ __forceinline__ void tmem_alloc_pair(uint32_t result_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives, once every product issued so far has finished, on the barrier at this offset in each CTA of `mask`.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}
// A tile into this CTA's shared memory whose bytes are counted on a barrier of the pair's first CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_address) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}

__device__ __forceinline__ unsigned pair_load_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float pair_silu_mul(float gate, float up) { return __fdividef(gate, 1.0f + __expf(-gate)) * up; }

template <bool kSwiglu>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                      const __grid_constant__ CUtensorMap map_out, const PairArgs args) {
  constexpr int kOutCols = kSwiglu ? kPairCols / 2 : kPairCols;     // columns of the result a tile gives
  extern __shared__ unsigned char pair_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kPairStages], empty_bar[kPairStages], acc_full_bar[2], acc_empty_bar[2], drain_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int aborted_flag;
  volatile int* aborted = &aborted_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();                 // 0: the CTA that issues the products
  const bool leader = rank == 0;
  const int pair = static_cast<int>(blockIdx.x) >> 1, pairs = static_cast<int>(gridDim.x) >> 1;
  const uint32_t smem_base = (smem_addr(pair_smem_raw) + 1023u) & ~1023u;
  auto stage_a = [&](int s) { return smem_base + s * kPairStageBytes; };                                  // tokens
  auto stage_b = [&](int s) { return smem_base + s * kPairStageBytes + kPairRows * kPairTileK * 2; };     // weight rows
  const uint32_t staging = smem_base + kPairStages * kPairStageBytes;
  // the weight rows this CTA brings of weight tile n_tile: its half of the tile, or with SwiGLU the gate rows
  // (first CTA) or the up rows that belong to them (second CTA)
  auto weight_row = [&](int n_tile) {
    return kSwiglu ? (leader ? 0 : args.N) + n_tile * kOutCols : n_tile * kPairCols + static_cast<int>(rank) * kPairRows;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(smem_addr(&full_bar[s]), 1);      // the first CTA's: its own expect_tx arrival; both CTAs' bytes
      mbar_init(smem_addr(&empty_bar[s]), 1);     // each CTA's own: the commit of the products that read the stage
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_addr(&acc_full_bar[b]), 1);  // each CTA's own: the commit of a tile's last product
      mbar_init(smem_addr(&acc_empty_bar[b]), 8); // the first CTA's: four epilogue warps of each CTA
    }
    mbar_init(smem_addr(&drain_bar), 1);
    aborted_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x == 64) {
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
    prefetch_tensormap(&map_out);
  }
  if (warp == 1) {                                // the same warp in both CTAs, together
    tmem_alloc_pair(smem_addr(&tmem_base_slot), kPairTmemColumns);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                                 // the partner's barriers exist before anything is signalled to them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  if (args.pdl && threadIdx.x == 0) pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------------------------ copies (both CTAs)
    if (lane == 0) {
      // the weights of the first stages may leave while the kernel before still runs: nothing in the stream writes them
      int early = 0;
      {
        PairRun ahead(args, pair, pairs);
        int tile, kb0, len;
        while (early < kPairStages && ahead.next(tile, kb0, len)) {
          const int w_row = weight_row(tile / args.t_tiles);
          for (int kb = kb0; kb < kb0 + len && early < kPairStages; ++kb, ++early) {
            const uint32_t leader_bar = peer_smem(smem_addr(&full_bar[early]), 0);
            if (leader) mbar_expect_tx(smem_addr(&full_bar[early]), 2 * kPairStageBytes);
            tma_load_2d_pair(stage_b(early), &map_w, leader_bar, kb * kPairTileK, w_row);
          }
        }
      }
      if (args.pdl) pdl_wait();
      int stage = 0;
      uint32_t phase = 0;
      long long filled = 0;
      bool ok = true;
      PairRun run(args, pair, pairs);
      int tile, kb0, len;
      while (ok && run.next(tile, kb0, len)) {
        const int n_tile = tile / args.t_tiles, t_tile = tile - n_tile * args.t_tiles;
        const int w_row = weight_row(n_tile);
        const int x_row = t_tile * kPairTokens + static_cast<int>(rank) * kPairRows;
        for (int kb = kb0; kb < kb0 + len && ok; ++kb) {
          const uint32_t leader_bar = peer_smem(smem_addr(&full_bar[stage]), 0);
          if (filled >= early) {
            ok = mbar_wait(smem_addr(&empty_bar[stage]), phase ^ 1u, aborted, args.fault, 1 << 8);
            if (!ok) break;
            if (leader) mbar_expect_tx(smem_addr(&full_bar[stage]), 2 * kPairStageBytes);
            tma_load_2d_pair(stage_b(stage), &map_w, leader_bar, kb * kPairTileK, w_row);
          }
          tma_load_2d_pair(stage_a(stage), &map_x, leader_bar, kb * kPairTileK, x_row);
          ++filled;
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
      if ((!ok || *aborted) && (filled > 0 || early > 0)) {
        // Copies still in flight must land before this CTA's shared memory is given up, and their completion
        // is counted in the first CTA only: give them a hundred microseconds, far more than a copy takes.
        const unsigned long long begin = global_ns();
        while (global_ns() - begin < 100000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ products (the first CTA only)
    if (leader && lane == 0) {
      int stage = 0, buf = 0;
      uint32_t phase = 0, acc_phase[2] = {0, 0};
      bool ok = true;
      PairRun run(args, pair, pairs);
      int tile, kb0, len;
      while (ok && run.next(tile, kb0, len)) {
        ok = mbar_wait(smem_addr(&acc_empty_bar[buf]), acc_phase[buf] ^ 1u, aborted, args.fault, 1 << 9);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kPairCols;
        for (int kb = 0; kb < len; ++kb) {
          ok = mbar_wait(smem_addr(&full_bar[stage]), phase, aborted, args.fault, 1 << 10);
          if (!ok) break;
          tc_fence_after();
          const uint64_t a_desc = operand_desc(stage_a(stage));
          const uint64_t b_desc = operand_desc(stage_b(stage));
#pragma unroll
          for (int k = 0; k < kPairTileK / 16; ++k)
            umma_bf16_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, kPairIdesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(smem_addr(&empty_bar[stage]), 3);     // the stage is free in both CTAs
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_pair(smem_addr(&acc_full_bar[buf]), 3);
        acc_phase[buf] ^= 1u;
        buf ^= 1;
      }
      umma_commit_pair(smem_addr(&drain_bar), 1);
      mbar_wait(smem_addr(&drain_bar), 0, aborted, args.fault);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs): a thread owns a token
    const int quarter = warp & 3;
    const int row_local = quarter * 32 + lane;
    int buf = 0;
    uint32_t acc_phase[2] = {0, 0};
    bool ok = true;
    bool store_in_flight = false;        // a tile of the result is leaving the staging buffer (thread 64 issued it)
    if (args.pdl) pdl_wait();
    PairRun run(args, pair, pairs);
    int tile, kb0, len;
    // where this thread's 16-byte pieces of a 64-column part of its row go: piece p to place p ^ (row & 7)
    const uint32_t staging_row = staging + row_local * 128;
    const uint32_t swizzle = static_cast<uint32_t>(row_local & 7);
    while (ok && run.next(tile, kb0, len)) {
      const int n_tile = tile / args.t_tiles, t_tile = tile - n_tile * args.t_tiles;
      const int n_base = n_tile * kOutCols;
      const int token0 = t_tile * kPairTokens + static_cast<int>(rank) * kPairRows;     // this CTA's first token of the tile
      const int token = token0 + row_local;
      const bool live = token < args.T;
      if (!kSwiglu && args.residual != nullptr && kb0 == 0 && live) {
        // this thread's kilobyte of the residual, asked into L2 while the tile's products run: eight neighbouring
        // lines at once (one row of the memory's pages) instead of one every few microseconds
        const float* mine = args.residual + static_cast<size_t>(token) * args.N + n_base;
#pragma unroll
        for (int line = 0; line < kOutCols / 32; ++line)
          if (n_base + line * 32 < args.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(mine + line * 32));
      }
      ok = named_barrier_and(1, 128, mbar_wait(smem_addr(&acc_full_bar[buf]), acc_phase[buf], aborted, args.fault, 1 << 11));
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + buf * kPairCols + (static_cast<uint32_t>(quarter * 32) << 16);
      unsigned* counter = args.counters + 2 * tile + rank;
      if (kb0 > 0) {
        // not the tile's first k-blocks: the partial tile goes to this pair's place in scratch, [column][token]
        float* mine = args.scratch + (static_cast<size_t>(pair) * 2 + rank) * kPairPartialFloats + row_local;
#pragma unroll 1
        for (int c = 0; c < kPairCols; c += 64) {
          uint32_t raw[2][32];
          tmem_load32(acc + c, raw[0]);
          tmem_load32(acc + c + 32, raw[1]);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 64; ++j) __stcg(mine + static_cast<size_t>(c + j) * kPairRows, __uint_as_float(raw[j >> 5][j & 31]));
        }
        __threadfence();
        named_barrier(1, 128);
        if (threadIdx.x == 64) atomicAdd(counter, 1u);
      } else {
        // the tile's first k-blocks: this pair stores the tile, after adding what the pairs behind it left
        int others = 0;
        if (len < args.k_blocks) {
          const long long tile_end = static_cast<long long>(tile + 1) * args.k_blocks;
          const int share = PairRun::sharers(run.tiles, pairs, args.k_blocks);
          while (pair + 1 + others < share && PairRun::run_begin(run.tiles, pairs, args.k_blocks, pair + 1 + others) < tile_end) ++others;
          bool complete = true;
          if (threadIdx.x == 64) {
            const unsigned long long begin = global_ns();
            while (pair_load_acquire(counter) < static_cast<unsigned>(others)) {
              if (*aborted || global_ns() - begin > kWaitLimitNs) {
                if (!*aborted) atomicOr(args.fault, kFaultWaitLimit | (1 << 12));
                *aborted = 1;
                complete = false;
                break;
              }
              __nanosleep(64);
            }
            if (complete) *counter = 0u;          // nobody else touches it again in this launch
          }
          ok = named_barrier_and(1, 128, complete);
          if (!ok) break;
        }
        if (store_in_flight) {
          // the tile stored before has left the staging buffer (its products took far longer than that)
          if (threadIdx.x == 64) tma_store_wait_read();
          named_barrier(1, 128);
          store_in_flight = false;
        }
        // the scale that the norm before this product left open
        float scale = 1.0f;
        if (args.sumsq_in != nullptr && live) {
          const float4* row = reinterpret_cast<const float4*>(args.sumsq_in + static_cast<size_t>(token) * args.sumsq_count);
          // eight loads in flight at a time; the order of the additions is fixed
          float sum = 0.0f;
          const int groups = args.sumsq_count / 4;
          for (int p0 = 0; p0 < groups; p0 += 8) {
            float4 four[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) four[i] = p0 + i < groups ? __ldcg(row + p0 + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < 8; ++i) sum += (four[i].x + four[i].y) + (four[i].z + four[i].w);
          }
          scale = rsqrtf(sum * args.inv_norm_size + args.norm_eps);
        }
        const float* theirs = args.scratch + (static_cast<size_t>(pair + 1) * 2 + rank) * kPairPartialFloats + row_local;
#pragma unroll 1
        for (int c = 0; c < kOutCols; c += 32) {
          if (n_base + c >= args.N) break;                   // the same for every thread
          // 32 columns of the result: the accumulator's, plus what the pairs behind left, in run order
          uint32_t raw[32], raw_up[kSwiglu ? 32 : 1];
          tmem_load32(acc + c, raw);
          if (kSwiglu) tmem_load32(acc + kOutCols + c, *reinterpret_cast<uint32_t(*)[32]>(raw_up));
          float v[32], u[kSwiglu ? 32 : 1];
          if (others > 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.0f;
            if (kSwiglu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) u[j] = 0.0f;
            }
            for (int q = 0; q < others; ++q) {
              const float* part = theirs + static_cast<size_t>(q) * 2 * kPairPartialFloats + static_cast<size_t>(c) * kPairRows;
              float got[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) got[j] = __ldcg(part + static_cast<size_t>(j) * kPairRows);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += got[j];
              if (kSwiglu) {
                const float* part_up = part + static_cast<size_t>(kOutCols) * kPairRows;
#pragma unroll
                for (int j = 0; j < 32; ++j) got[j] = __ldcg(part_up + static_cast<size_t>(j) * kPairRows);
#pragma unroll
                for (int j = 0; j < 32; ++j) u[j] += got[j];
              }
            }
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += __uint_as_float(raw[j]);
            if (kSwiglu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) u[j] += __uint_as_float(raw_up[j]);
            }
          } else {
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
            if (kSwiglu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) u[j] = __uint_as_float(raw_up[j]);
            }
          }
          // the row's scale, the bias, the activation
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = n_base + c + j;
            const bool inside = n < args.N;
            float value = v[j] * scale + (args.bias != nullptr && inside ? __ldg(args.bias + n) : 0.0f);
            if (kSwiglu) {
              const float up = u[j] * scale + (args.bias != nullptr && inside ? __ldg(args.bias + args.N + n) : 0.0f);
              value = pair_silu_mul(value, up);
            }
            v[j] = value;
          }
          if (!kSwiglu && args.residual != nullptr) {
            // the following norm rides: the residual takes the sum, the output the sum times the norm's weight, and
            // the squares of these 32 columns are the row's slot of the table
            float squares = 0.0f;
            if (live) {
              float4* rows = reinterpret_cast<float4*>(args.residual + static_cast<size_t>(token) * args.N + n_base + c);
              const float4* weights = reinterpret_cast<const float4*>(args.norm_weight + n_base + c);
              // all of the row's 128 bytes are asked for before any of them is used or written back
              float4 old[8];
#pragma unroll
              for (int q = 0; q < 8; ++q)             // N is a multiple of 8: a group of four is inside or outside
                old[q] = n_base + c + 4 * q < args.N ? __ldcg(rows + q) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                if (n_base + c + 4 * q < args.N) {
                  float4 sum = old[q];
                  const float4 weight = __ldg(weights + q);
                  sum.x += v[4 * q]; sum.y += v[4 * q + 1]; sum.z += v[4 * q + 2]; sum.w += v[4 * q + 3];
                  __stcg(rows + q, sum);
                  squares += (sum.x * sum.x + sum.y * sum.y) + (sum.z * sum.z + sum.w * sum.w);
                  v[4 * q] = sum.x * weight.x; v[4 * q + 1] = sum.y * weight.y;
                  v[4 * q + 2] = sum.z * weight.z; v[4 * q + 3] = sum.w * weight.w;
                }
              }
              args.sumsq_out[static_cast<size_t>(token) * args.sumsq_out_count + (n_base + c) / 32] = squares;
            }
          }
          // into the staging buffer: 64 bytes of this thread's row, four pieces of 16
          const uint32_t sub = staging_row + static_cast<uint32_t>(c >> 6) * kPairSubTileBytes;
          const uint32_t first_piece = static_cast<uint32_t>((c & 63) >> 3);
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            uint32_t packed[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const __nv_bfloat162 two = __floats2bfloat162_rn(v[8 * p + 2 * h], v[8 * p + 2 * h + 1]);
              packed[h] = *reinterpret_cast<const uint32_t*>(&two);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(sub + (((first_piece + p) ^ swizzle) << 4)),
                         "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3])
                         : "memory");
          }
        }
        // the tile with the last column clears the row's slots past it: their sum is the row's sum of squares
        if (!kSwiglu && args.residual != nullptr && live && n_base < args.N && n_base + kOutCols >= args.N)
          for (int slot = (args.N + 31) / 32; slot < args.sumsq_out_count; ++slot)
            args.sumsq_out[static_cast<size_t>(token) * args.sumsq_out_count + slot] = 0.0f;
        // the tile is whole in the staging buffer: copies of 64 columns take it out (what lies past the matrix's
        // edges is not written)
        fence_async_smem();
        named_barrier(1, 128);
        if (threadIdx.x == 64 && token0 < args.T) {
          for (int part = 0; part < kOutCols / 64; ++part)
            if (n_base + part * 64 < args.N)
              tma_store_2d(&map_out, staging + part * kPairSubTileBytes, n_base + part * 64, token0);
          tma_store_commit();
        }
        store_in_flight = true;
      }
      // the accumulator may be overwritten: every epilogue warp of both CTAs tells the first CTA
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(peer_smem(smem_addr(&acc_empty_bar[buf]), 0));
      acc_phase[buf] ^= 1u;
      buf ^= 1;
    }
    if (threadIdx.x == 64 && store_in_flight) tma_store_wait_read();   // shared memory is given up below
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();           // the partner may read this CTA's shared memory and signal its barriers until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kPairTmemColumns);
  }
}

static bool g_pair_configured[2] = {false, false};   // [swiglu]; file-local on purpose

template <bool kSwiglu>
static int launch_pair(const void* x, const void* w, void* out, PairArgs args, int pairs, cudaStream_t stream) {
  CUtensorMap map_w, map_x, map_out;
  int status = make_map(&map_w, w, static_cast<long long>(args.N) * (kSwiglu ? 2 : 1), args.K, kPairRows);
  if (status != 0) return status;
  status = make_map(&map_x, x, args.T, args.K, kPairRows);
  if (status != 0) return status;
  status = make_map(&map_out, out, args.T, args.N, kPairRows);      // boxes of 128 tokens by 64 columns, swizzled
  if (status != 0) return status;
  auto kernel = gemm_bf16_pair_kernel<kSwiglu>;
  bool& configured = g_pair_configured[kSwiglu ? 1 : 0];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kPairSmemBytes));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2 * pairs);
  config.blockDim = dim3(kPairThreads);
  config.dynamicSmemBytes = kPairSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = 2;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  int count = 1;
  if (args.pdl) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  return static_cast<int>(cudaLaunchKernelEx(&config, kernel, map_x, map_w, map_out, args));
}

static int pair_count() {
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 2)
    sms = 148;
  return sms / 2;
}

}  // namespace rl

extern "C" {

// float32 words of scratch and unsigned words of counters (zeroed once by the caller) the product needs
long long rl_gemm_bf16_pair_scratch_floats() { return static_cast<long long>(rl::pair_count()) * 2 * rl::kPairPartialFloats; }
int rl_gemm_bf16_pair_counter_words() { return 2 * rl::kPairMaxTiles; }

// x: [tokens, k], w: [n_out, k] (swiglu: [2 n_out, k], the gate rows first), out: [tokens, n_out]; bfloat16,
// contiguous, 16-byte aligned, k and n_out multiples of 8.  Made for steps of hundreds to thousands of tokens.
// bias: float32 [n_out] (swiglu: [2 n_out]) or null.  sumsq_in [tokens, sumsq_count] with norm_eps and norm_size: the
// scale a norm before the product left open.  residual [tokens, n_out], norm_weight [n_out] and
// sumsq_out [tokens, sumsq_out_count] (a slot per 32 columns; not with swiglu): the norm that follows.
int rl_gemm_bf16_pair(const void* x, const void* w, void* out, int tokens, int n_out, int k, int swiglu, int pdl,
                      float* residual, const float* norm_weight, float* sumsq_out, int sumsq_out_count,
                      const float* sumsq_in, int sumsq_count, float norm_eps, int norm_size, const float* bias,
                      float* scratch, unsigned* counters, int* fault, cudaStream_t stream) {
  if (tokens == 0 || n_out == 0) return 0;
  if (tokens < 0 || n_out < 0 || n_out % 8 != 0 || k <= 0 || k % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (reinterpret_cast<uintptr_t>(residual) & 15) || (reinterpret_cast<uintptr_t>(norm_weight) & 15) ||
      (reinterpret_cast<uintptr_t>(sumsq_in) & 15) || scratch == nullptr || counters == nullptr ||
      ((residual != nullptr) != (norm_weight != nullptr)) || ((residual != nullptr) != (sumsq_out != nullptr)) ||
      (residual != nullptr && (swiglu || sumsq_out_count < (n_out + 31) / 32)) ||
      (sumsq_in != nullptr && (sumsq_count <= 0 || sumsq_count % 4 != 0 || norm_size <= 0)))
    return static_cast<int>(cudaErrorInvalidValue);
  rl::PairArgs args;
  args.fault = fault;
  args.T = tokens; args.N = n_out; args.K = k;
  args.out_cols = swiglu ? rl::kPairCols / 2 : rl::kPairCols;
  args.n_tiles = (n_out + args.out_cols - 1) / args.out_cols;
  args.t_tiles = (tokens + rl::kPairTokens - 1) / rl::kPairTokens;
  args.k_blocks = (k + rl::kPairTileK - 1) / rl::kPairTileK;
  args.pdl = pdl;
  args.bias = bias;
  args.sumsq_in = sumsq_in; args.sumsq_count = sumsq_count; args.norm_eps = norm_eps;
  args.inv_norm_size = norm_size > 0 ? 1.0f / static_cast<float>(norm_size) : 0.0f;
  args.residual = residual; args.norm_weight = norm_weight; args.sumsq_out = sumsq_out; args.sumsq_out_count = sumsq_out_count;
  args.scratch = scratch;
  args.counters = counters;
  const long long tiles = static_cast<long long>(args.n_tiles) * args.t_tiles;
  if (tiles > rl::kPairMaxTiles) return static_cast<int>(cudaErrorInvalidValue);
  long long pairs = rl::pair_count();
  // a product of few tiles is shared by as many pairs as get eight k-blocks each
  const long long units = tiles * args.k_blocks;
  if (tiles < pairs) pairs = units / 8 > tiles ? (units / 8 < pairs ? units / 8 : pairs) : tiles;
  if (swiglu) return rl::launch_pair<true>(x, w, out, args, static_cast<int>(pairs), stream);
  return rl::launch_pair<false>(x, w, out, args, static_cast<int>(pairs), stream);
}

}  // extern "C"

// bfloat16 matrix product of the linear layers for steps of many tokens, on pairs of multiprocessors:
//   out[T, N] = x[T, K] . w[N, K]^T            (float32 accumulation, one rounding at the store)
//
// Two CTAs of a thread-block cluster work on one 256 x 256 tile (256 weight rows by 256 tokens) with
// tcgen05.mma.cta_group::2: each CTA brings 128 weight rows (its half of the M side) and 128 token
// rows (its half of the N side) of every 64-element k-block through TMA into its own shared memory,
// one thread of the pair's first CTA issues the product for both, and each CTA ends up with its 128
// weight rows by all 256 tokens in its own tensor memory.  Against two independent CTAs this halves
// the operand bytes every CTA reads from shared memory per product, which is what bounds a single
// CTA's 128 x 256 tile.
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
// warp 0 copies (TMA; the copies of both CTAs complete on the first CTA's barrier), warp 1 of the
// first CTA issues products and commits to the barriers of both, warps 2..5 read the accumulator
// (two buffers of 256 tensor-memory columns, so a tile's epilogue overlaps the next tile's products)
// and store.  No copy here is a multicast: each CTA fetches its own halves.
//
// Every mbarrier wait is bounded by time; the two cluster barriers (after set-up, before exit) are
// reached by every thread on every path.
//
// The reference calls a library product here (rapid_llm/kernels/ops/gemm/linear.py:17-40).
#include <cuda.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace rl {

using bf16 = __nv_bfloat16;

constexpr int kPairRows = 128;            // weight rows per CTA = lanes of its accumulator
constexpr int kPairTileK = 64;
constexpr int kPairThreads = 192;
constexpr int kPairMaxTiles = 4096;       // tiles of one product (two counters each)

// TN: tokens per tile = N of the product (each CTA loads half of them)
template <int TN>
struct PairShape {
  static constexpr int kStageBytes = kPairRows * kPairTileK * 2 + (TN / 2) * kPairTileK * 2;
  static constexpr int kStagingBytes = TN * kPairRows * 2;    // a CTA's tile of the result, [token][weight row], on its way out
  static constexpr int kStages = (192 * 1024 - kStagingBytes) / kStageBytes > 8 ? 8 : (192 * 1024 - kStagingBytes) / kStageBytes;
  static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + kStagingBytes + 1024;
  static constexpr int kTmemColumns = 2 * TN;        // two accumulators
  static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(TN >> 3) << 17) |
                                     (static_cast<uint32_t>((2 * kPairRows) >> 4) << 24);
  static constexpr size_t kPartialFloats = static_cast<size_t>(TN) * kPairRows;     // one CTA's partial tile
  static_assert(TN == 128 || TN == 256, "token tile");
};

struct PairArgs {
  bf16* out;           // [T, N]
  int* fault;
  int T, N, K;
  int n_tiles, t_tiles, k_blocks;
  int pdl;
  int out_by_tma;      // tiles of the result leave through map_out (N a multiple of 8, out 16-byte aligned)
  const float* bias;   // [N] or null
  float* scratch;      // [pairs][2][TN][128]: the partial tile of a pair's first segment, per CTA
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

template <int TN>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      const __grid_constant__ CUtensorMap map_out, const PairArgs args) {
  using Shape = PairShape<TN>;
  constexpr int kPairStages = Shape::kStages, kPairStageBytes = Shape::kStageBytes, kPairTokens = TN;
  constexpr int kPairTmemColumns = Shape::kTmemColumns;
  constexpr uint32_t kPairIdesc = Shape::kIdesc;
  extern __shared__ unsigned char pair_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], acc_full_bar[2], acc_empty_bar[2], drain_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int aborted_flag;
  volatile int* aborted = &aborted_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();                 // 0: the CTA that issues the products
  const bool leader = rank == 0;
  const int pair = static_cast<int>(blockIdx.x) >> 1, pairs = static_cast<int>(gridDim.x) >> 1;
  const uint32_t smem_base = (smem_addr(pair_smem_raw) + 1023u) & ~1023u;
  auto stage_a = [&](int s) { return smem_base + s * kPairStageBytes; };
  auto stage_b = [&](int s) { return smem_base + s * kPairStageBytes + kPairRows * kPairTileK * 2; };
  const uint32_t staging = smem_base + kPairStages * kPairStageBytes;

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
    if (args.out_by_tma) prefetch_tensormap(&map_out);
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
      if (args.pdl) pdl_wait();
      int stage = 0;
      uint32_t phase = 0;
      long long filled = 0;
      bool ok = true;
      PairRun run(args, pair, pairs);
      int tile, kb0, len;
      while (ok && run.next(tile, kb0, len)) {
        const int n_tile = tile / args.t_tiles, t_tile = tile - n_tile * args.t_tiles;
        const int w_row = n_tile * 2 * kPairRows + static_cast<int>(rank) * kPairRows;
        const int x_row = t_tile * kPairTokens + static_cast<int>(rank) * (kPairTokens / 2);
        for (int kb = kb0; kb < kb0 + len && ok; ++kb) {
          ok = mbar_wait(smem_addr(&empty_bar[stage]), phase ^ 1u, aborted, args.fault, 1 << 8);
          if (!ok) break;
          const uint32_t leader_bar = peer_smem(smem_addr(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(smem_addr(&full_bar[stage]), 2 * kPairStageBytes);
          tma_load_2d_pair(stage_a(stage), &map_w, leader_bar, kb * kPairTileK, w_row);
          tma_load_2d_pair(stage_b(stage), &map_x, leader_bar, kb * kPairTileK, x_row);
          ++filled;
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
      if ((!ok || *aborted) && filled > 0) {
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
        const uint32_t d_tmem = tmem_base + buf * kPairTokens;
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
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quarter = warp & 3;
    const int row_local = quarter * 32 + lane;
    int buf = 0;
    uint32_t acc_phase[2] = {0, 0};
    bool ok = true;
    bool store_in_flight = false;        // a tile of the result is leaving the staging buffer (thread 64 issued it)
    if (args.pdl) pdl_wait();
    PairRun run(args, pair, pairs);
    int tile, kb0, len;
    while (ok && run.next(tile, kb0, len)) {
      const int n_tile = tile / args.t_tiles, t_tile = tile - n_tile * args.t_tiles;
      const int n = n_tile * 2 * kPairRows + static_cast<int>(rank) * kPairRows + row_local;
      const int t0 = t_tile * kPairTokens;
      ok = named_barrier_and(1, 128, mbar_wait(smem_addr(&acc_full_bar[buf]), acc_phase[buf], aborted, args.fault, 1 << 11));
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + buf * kPairTokens + (static_cast<uint32_t>(quarter * 32) << 16);
      unsigned* counter = args.counters + 2 * tile + rank;
      if (kb0 > 0) {
        // not the tile's first k-blocks: the partial tile goes to this pair's place in scratch, [token][row]
        float* mine = args.scratch + (static_cast<size_t>(pair) * 2 + rank) * Shape::kPartialFloats + row_local;
#pragma unroll 1
        for (int c = 0; c < kPairTokens; c += 64) {
          if (t0 + c >= args.T) break;
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
        const float bias = args.bias != nullptr && n < args.N ? args.bias[n] : 0.0f;
        if (store_in_flight) {
          // the tile stored before has left the staging buffer (its products took far longer than that)
          if (threadIdx.x == 64) tma_store_wait_read();
          named_barrier(1, 128);
          store_in_flight = false;
        }
        const float* theirs = args.scratch + (static_cast<size_t>(pair + 1) * 2 + rank) * Shape::kPartialFloats + row_local;
#pragma unroll 1
        for (int c0 = 0; c0 < kPairTokens; c0 += 64) {
          if (t0 + c0 >= args.T) break;
          // the others' parts of 64 tokens at a time: many loads in flight, added in run order
          float sum[64];
#pragma unroll
          for (int j = 0; j < 64; ++j) sum[j] = 0.0f;
          for (int q = 0; q < others; ++q) {
            const float* part = theirs + static_cast<size_t>(q) * 2 * Shape::kPartialFloats + static_cast<size_t>(c0) * kPairRows;
            float got[64];
#pragma unroll
            for (int j = 0; j < 64; ++j) got[j] = __ldcg(part + static_cast<size_t>(j) * kPairRows);
#pragma unroll
            for (int j = 0; j < 64; ++j) sum[j] += got[j];
          }
          // 64 columns of the accumulator per wait: a load of tensor memory takes a fraction of a microsecond
          // to come back, and sixteen of them in a row were most of a tile's way out
          uint32_t raw[2][32];
          tmem_load32(acc + c0, raw[0]);
          tmem_load32(acc + c0 + 32, raw[1]);
          tmem_wait_ld();
          if (args.out_by_tma) {
            // [token][weight row]: a warp writes 32 neighbouring values of one token per instruction
#pragma unroll
            for (int j = 0; j < 64; ++j) {
              const __nv_bfloat16 value = __float2bfloat16_rn(__uint_as_float(raw[j >> 5][j & 31]) + sum[j] + bias);
              asm volatile("st.shared.b16 [%0], %1;" ::"r"(staging + ((c0 + j) * kPairRows + row_local) * 2),
                           "h"(*reinterpret_cast<const unsigned short*>(&value))
                           : "memory");
            }
          } else if (n < args.N) {
#pragma unroll
            for (int j = 0; j < 64; ++j)
              if (t0 + c0 + j < args.T)
                args.out[static_cast<size_t>(t0 + c0 + j) * args.N + n] =
                    __float2bfloat16_rn(__uint_as_float(raw[j >> 5][j & 31]) + sum[j] + bias);
          }
        }
      }
      if (kb0 == 0 && args.out_by_tma) {
        // the tile is whole in the staging buffer: one copy takes it out (what lies past the matrix's edge is not written)
        fence_async_smem();
        named_barrier(1, 128);
        if (threadIdx.x == 64) {
          tma_store_2d(&map_out, staging, n_tile * 2 * kPairRows + static_cast<int>(rank) * kPairRows, t0);
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

static bool g_pair_configured[2] = {false, false};

template <int TN>
static int launch_pair(const void* x, const void* w, PairArgs args, int pairs, cudaStream_t stream) {
  using Shape = PairShape<TN>;
  CUtensorMap map_w, map_x;
  int status = make_map(&map_w, w, args.N, args.K, kPairRows);
  if (status != 0) return status;
  status = make_map(&map_x, x, args.T, args.K, TN / 2);
  if (status != 0) return status;
  CUtensorMap map_out = map_x;
  args.out_by_tma = 0;
  if (args.N % 8 == 0 && (reinterpret_cast<uintptr_t>(args.out) & 15) == 0) {
    status = make_map_plain(&map_out, args.out, args.T, args.N, TN, kPairRows);
    if (status != 0) return status;
    args.out_by_tma = 1;
  }
  auto kernel = gemm_bf16_pair_kernel<TN>;
  bool& configured = g_pair_configured[TN == 256 ? 1 : 0];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Shape::kSmemBytes));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2 * pairs);
  config.blockDim = dim3(kPairThreads);
  config.dynamicSmemBytes = Shape::kSmemBytes;
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
  return static_cast<int>(cudaLaunchKernelEx(&config, kernel, map_w, map_x, map_out, args));
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
long long rl_gemm_bf16_pair_scratch_floats() { return static_cast<long long>(rl::pair_count()) * 2 * rl::PairShape<256>::kPartialFloats; }
int rl_gemm_bf16_pair_counter_words() { return 2 * rl::kPairMaxTiles; }

// x: [tokens, k], w: [n_out, k], out: [tokens, n_out]; bfloat16, contiguous, 16-byte aligned, k a multiple of 8;
// bias: float32 [n_out] or null.  Made for steps of hundreds to thousands of tokens.
int rl_gemm_bf16_pair(const void* x, const void* w, void* out, int tokens, int n_out, int k, int pdl, const float* bias,
                      float* scratch, unsigned* counters, int* fault, cudaStream_t stream) {
  if (tokens == 0 || n_out == 0) return 0;
  if (tokens < 0 || n_out < 0 || k <= 0 || k % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(w) & 15) || scratch == nullptr || counters == nullptr)
    return static_cast<int>(cudaErrorInvalidValue);
  const int token_tile = tokens <= 128 ? 128 : 256;
  rl::PairArgs args;
  args.out = static_cast<rl::bf16*>(out);
  args.fault = fault;
  args.T = tokens; args.N = n_out; args.K = k;
  args.n_tiles = (n_out + 2 * rl::kPairRows - 1) / (2 * rl::kPairRows);
  args.t_tiles = (tokens + token_tile - 1) / token_tile;
  args.k_blocks = (k + rl::kPairTileK - 1) / rl::kPairTileK;
  args.pdl = pdl;
  args.bias = bias;
  args.scratch = scratch;
  args.counters = counters;
  const long long tiles = static_cast<long long>(args.n_tiles) * args.t_tiles;
  if (tiles > rl::kPairMaxTiles) return static_cast<int>(cudaErrorInvalidValue);
  long long pairs = rl::pair_count();
  // a product of few tiles is shared by as many pairs as get eight k-blocks each
  const long long units = tiles * args.k_blocks;
  if (tiles < pairs) pairs = units / 8 > tiles ? (units / 8 < pairs ? units / 8 : pairs) : tiles;
  if (token_tile == 128) return rl::launch_pair<128>(x, w, args, static_cast<int>(pairs), stream);
  return rl::launch_pair<256>(x, w, args, static_cast<int>(pairs), stream);
}

}  // extern "C"

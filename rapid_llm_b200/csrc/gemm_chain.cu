// A chain of bfloat16 products of a small step as ONE persistent kernel:
//
//   phase 0:  out0 = x0 . w0^T          phase 1:  out1 = out0' . w1^T   ...   (up to four)
//
// where each phase is a product of gemm_bf16.cu's kind (plain, fused SwiGLU over a [2N, K] weight,
// or with the residual add and the following norm's weight in the epilogue, a preceding norm's open
// scale applied to the rows, an optional bias) and reads what the phase before it wrote.  In a decode
// step the products of a layer run back to back (output projection, gate/up, down, the next layer's
// q/k/v) and each has only a few microseconds of weights to stream.  As separate kernels each pays
// its own start, drain and reduction while the memory system idles; here one CTA per multiprocessor
// stays resident for the whole chain and the weight stream never stops:
//
//   * warp 0 copies weight tiles (TMA) into a ring that takes nearly all of shared memory.  Weights
//     depend on nothing, so this warp runs ahead across phase boundaries as far as the ring
//     allows: while the CTAs finish a phase and meet at its barrier, the next phase's first
//     ~190 KB per multiprocessor are already arriving.
//   * warp 2 copies the activation tiles into the same stages; it is the one that waits at a phase
//     boundary until every CTA has stored that phase's results.
//   * warp 1 issues tcgen05.mma (weight rows as M = 128, tokens as N = 16..64) into one of two
//     tensor-memory accumulators; warps 3..6 read them back.
//
// Work of a phase is cut into chunks (tile of 128 weight rows, segment of the inner range) dealt
// round-robin over the CTAs, continuing where the phase before stopped, so every CTA streams about
// the same number of bytes whatever the shapes.  A tile's segments meet in global scratch: each
// CTA stores its float32 partial tile and counts itself in; when a tile's count is full, each of its
// CTAs sums a share of the tile's elements over all segments in segment order (never in order of
// arrival: the result does not depend on timing), applies the epilogue and stores.  A phase ends at
// a barrier over all CTAs (an arrival counter in global memory).
//
// Waiting on other CTAs means all of them must be resident: the grid is one CTA per multiprocessor
// and a CTA takes more than half a multiprocessor's shared memory.  Dependents of a programmatic
// launch are released only when the last phase starts.  Every wait is bounded by time; one that runs
// out sets the fault word and a flag in the counters that makes all others give up at once.
//
// The counters are zero when the kernel starts and are zeroed again by the CTA that leaves last.
//
// Measured on the four products of a Qwen3-8B layer at 8 tokens (cold caches, one launch): 104 us against
// 59 us of streaming; a phase's end (partial tiles parked and counted, the others' awaited, sums, stores, the
// barrier, the next activation tiles) costs about 8 us, of which the ring hides 4.  A variant that gave each
// tile to a cluster of two CTAs (halves of the inner range, summed through distributed shared memory) ended a
// phase in 5 us, but left the narrow products (32 tiles) to 64 of 148 multiprocessors, each of which drew only
// about 35 GB/s from memory: 129 us.  Kernels chained by programmatic dependent launch take 76 us for the same
// products inside a decode step, which is why the engine does not use this kernel by default.
//
// The reference runs these products as separate library calls (rapid_llm/kernels/ops/gemm/linear.py:17-40,
// rapid_llm/modules/mlp.py:52-68, rapid_llm/models/base.py:231-266).
#include <cuda.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace rl {

using bf16 = __nv_bfloat16;

constexpr int kChainTileN = 128;        // weight rows per tile = M of one tcgen05.mma
constexpr int kChainTileK = 64;         // bf16 elements in one 128-byte swizzle row
constexpr int kChainUmmaK = 16;
constexpr int kChainThreads = 224;      // warp 0 weights, warp 1 products, warp 2 activations, warps 3..6 epilogue
constexpr int kChainMaxPhases = 4;
constexpr int kChainMaxStages = 12;
constexpr int kChainMaxTiles = 1536;    // tiles of one phase (a tile counter each)
constexpr int kChainMaxSplit = 16;
constexpr int kChainRingBytes = 200 * 1024;
// counters: [0] arrivals at phase barriers, [1] CTAs that left, [2] somebody gave up, [4 + p * kChainMaxTiles + tile]
constexpr int kChainCounterBarrier = 0, kChainCounterExit = 1, kChainCounterAbort = 2, kChainCounterTiles = 4;
constexpr int kChainCounters = kChainCounterTiles + kChainMaxPhases * kChainMaxTiles;

struct ChainPhase {
  bf16* out;                 // [T, N]
  int N, K;                  // output columns (SwiGLU: of the activation), inner size
  int swiglu;                // the weight is [2 N, K], gate rows first
  int n_tiles, k_blocks;
  int split;                 // segments of the inner range = CTAs that share a tile
  int first_cta;             // chunk c runs on CTA (first_cta + c) mod grid
  float* residual;           // with norm_weight and sumsq_out: see gemm_bf16.cu
  const float* norm_weight;
  float* sumsq_out;
  const float* sumsq_in;
  int sumsq_count;
  float norm_eps, inv_norm_size;
  const float* bias;
};

struct ChainArgs {
  int T, phases, pdl;
  int* fault;
  float* scratch;
  unsigned* counters;
  // Optional time stamps (%globaltimer, ns) for looking into a launch: [CTA][phase][kChainTraceEvents]; null = none.
  unsigned long long* trace;
  ChainPhase phase[kChainMaxPhases];
};

// events of a CTA in a phase: 0 the phase's start barrier passed (epilogue), 1 first accumulator complete,
// 2 last partial tile stored and counted, 3 the tiles of this CTA are complete, 4 results stored (arrival at
// the phase's end barrier), 5 the weight warp issued the phase's last copy, 6 the activation warp passed the
// phase's start barrier, 7 the issuing thread committed the phase's last product
constexpr int kChainTraceEvents = 8;
__device__ __forceinline__ void chain_stamp(const ChainArgs& args, int cta, int p, int event) {
  if (args.trace != nullptr)
    args.trace[(static_cast<size_t>(cta) * kChainMaxPhases + p) * kChainTraceEvents + event] = global_ns();
}

struct ChainMaps {
  CUtensorMap w[kChainMaxPhases];
  CUtensorMap x[kChainMaxPhases];
};

template <int BN>
struct ChainShape {
  static constexpr int kWeightBytes = kChainTileN * kChainTileK * 2;
  static constexpr int kTokenBytes = BN * kChainTileK * 2;
  static constexpr int kStageBytes = kWeightBytes + kTokenBytes;
  static constexpr int kFit = kChainRingBytes / kStageBytes;
  static constexpr int kStages = kFit > kChainMaxStages ? kChainMaxStages : kFit;
  static constexpr int kAccColumns = 2 * BN;                 // gate and up halves
  static constexpr int kTmemColumns = 2 * kAccColumns < 32 ? 32 : 2 * kAccColumns;
  static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + 1024;
  static_assert(BN == 16 || BN == 32 || BN == 64, "token tile");
  static_assert(kStageBytes % 1024 == 0, "stages keep the alignment of the 128-byte swizzle");
  static_assert(kSmemBytes > 114 * 1024, "one CTA per multiprocessor");
};

__device__ __forceinline__ unsigned load_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Waits until `*counter >= target`; gives up after kWaitLimitNs, or at once when some CTA already
// has.  Returns false then, with the fault recorded.
__device__ __forceinline__ bool wait_counter(const unsigned* counter, unsigned target, unsigned* counters,
                                             volatile int* aborted, int* fault) {
  if (load_acquire(counter) >= target) return true;
  const unsigned long long begin = global_ns();
  for (uint32_t spin = 0;; ++spin) {
    if (load_acquire(counter) >= target) return true;
    if ((spin & 15u) == 15u) {
      if (*aborted || load_acquire(counters + kChainCounterAbort) != 0u) break;
      if (global_ns() - begin > kWaitLimitNs) {
        atomicOr(fault, kFaultWaitLimit | (1 << 12));
        break;
      }
      __nanosleep(64);
    }
  }
  *aborted = 1;
  atomicExch(counters + kChainCounterAbort, 1u);
  return false;
}

// The k-blocks of segment `seg` of `split`: as even as the division allows, the longer ones first.
__device__ __forceinline__ void segment_range(int k_blocks, int split, int seg, int& begin, int& count) {
  const int base = k_blocks / split, rem = k_blocks - base * split;
  begin = seg * base + min(seg, rem);
  count = base + (seg < rem ? 1 : 0);
}

__device__ __forceinline__ float chain_silu_mul(float gate, float up) {
  return __fdividef(gate, 1.0f + __expf(-gate)) * up;
}

// One element of a phase's result, for the 32 lanes of a warp at once: lanes hold consecutive weight
// rows `n` of token `t` (the same for the warp); `group` is the tile's quarter the rows lie in.
__device__ __forceinline__ void chain_emit(const ChainPhase& ph, int t, int n, int n_tile, int group, int lane,
                                           float gate, float up, float scale) {
  const bool live = n < ph.N;
  if (ph.bias != nullptr && live) {
    gate = gate * scale + ph.bias[n];
    up = ph.swiglu ? up * scale + ph.bias[ph.N + n] : 0.0f;
  } else {
    gate *= scale;
    up *= scale;
  }
  const size_t at = static_cast<size_t>(t) * ph.N + n;
  if (ph.residual != nullptr) {
    float sum = 0.0f;
    if (live) {
      sum = __ldcg(ph.residual + at) + gate;
      ph.residual[at] = sum;
      ph.out[at] = __float2bfloat16_rn(sum * ph.norm_weight[n]);
    }
    const float sq = warp_sum(sum * sum);
    if (lane == 0) ph.sumsq_out[static_cast<size_t>(t) * (4 * ph.n_tiles) + 4 * n_tile + group] = sq;
  } else if (live) {
    ph.out[at] = __float2bfloat16_rn(ph.swiglu ? chain_silu_mul(gate, up) : gate);
  }
}

// Walks the weight tiles a CTA streams, in order: phase by phase, chunk by chunk, k-block by k-block, the
// gate rows' tile before the up rows'.  Two of these run in the weight warp: one names the next copy into
// shared memory, one runs ahead of it and names the next tile to ask into L2.
struct WeightCursor {
  int p, c, kb, kb_end, half, halves, tile;
  bool valid;
  __device__ __forceinline__ void enter_chunk(const ChainArgs& args) {
    const ChainPhase& ph = args.phase[p];
    tile = c / ph.split;
    int begin, count;
    segment_range(ph.k_blocks, ph.split, c - tile * ph.split, begin, count);
    kb = begin;
    kb_end = begin + count;
    half = 0;
  }
  // the first chunk this CTA has in phase `from` or a later one
  __device__ __forceinline__ void seek_phase(const ChainArgs& args, int from, int cta, int grid) {
    for (p = from; p < args.phases; ++p) {
      const ChainPhase& ph = args.phase[p];
      int first = (cta - ph.first_cta) % grid;
      if (first < 0) first += grid;
      if (first < ph.n_tiles * ph.split) {
        c = first;
        halves = ph.swiglu ? 2 : 1;
        enter_chunk(args);
        valid = true;
        return;
      }
    }
    valid = false;
  }
  __device__ __forceinline__ void next(const ChainArgs& args, int cta, int grid) {
    if (++half < halves) return;
    half = 0;
    if (++kb < kb_end) return;
    c += grid;
    if (c < args.phase[p].n_tiles * args.phase[p].split) {
      enter_chunk(args);
      return;
    }
    seek_phase(args, p + 1, cta, grid);
  }
};

__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}

// Weight tiles asked into L2 beyond the ring while the ring is full.  Measured on the 8B layer's four products
// at 8 tokens: 16 tiles ahead made the chain slower (120 us against 104 us), as every other form of asking
// ahead into L2 did in these kernels, so it is off.
constexpr int kChainL2Ahead = 0;

template <int BN>
__global__ void __launch_bounds__(kChainThreads)
gemm_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainArgs args) {
  using Shape = ChainShape<BN>;
  constexpr int kStages = Shape::kStages;
  constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                              (static_cast<uint32_t>(kChainTileN >> 4) << 24);
  extern __shared__ unsigned char chain_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kChainMaxStages], empty_bar[kChainMaxStages], acc_full_bar[2],
      acc_empty_bar[2], drain_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int aborted_flag, last_flag;
  __shared__ float row_scale[BN];
  volatile int* aborted = &aborted_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = static_cast<int>(blockIdx.x), grid = static_cast<int>(gridDim.x);
  const uint32_t smem_base = (smem_addr(chain_smem_raw) + 1023u) & ~1023u;
  auto stage_a = [&](int s) { return smem_base + s * Shape::kStageBytes; };
  auto stage_b = [&](int s) { return smem_base + s * Shape::kStageBytes + Shape::kWeightBytes; };
  // this CTA's first chunk of a phase; its chunks are that one and every grid-th after it
  auto first_chunk = [&](const ChainPhase& ph) {
    int c = (cta - ph.first_cta) % grid;
    return c < 0 ? c + grid : c;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_addr(&full_bar[s]), 2);       // the weight copy and the activation copy each arrive
      mbar_init(smem_addr(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_addr(&acc_full_bar[b]), 1);
      mbar_init(smem_addr(&acc_empty_bar[b]), 4);
    }
    mbar_init(smem_addr(&drain_bar), 1);
    aborted_flag = 0;
    last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x == 96) {
    for (int p = 0; p < args.phases; ++p) {
      prefetch_tensormap(&maps.w[p]);
      prefetch_tensormap(&maps.x[p]);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_addr(&tmem_base_slot), Shape::kTmemColumns);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ weights (TMA), never waits for a phase
    if (lane == 0) {
      const uint64_t weights_once = l2_evict_first_policy();
      int stage = 0;
      uint32_t phase = 0;
      long long filled = 0;
      bool ok = true;
      WeightCursor load, ahead;
      load.seek_phase(args, 0, cta, grid);
      ahead = load;
      int lead = 0;                       // tiles by which `ahead` leads `load`
      int stamped = 0;
      while (load.valid) {
        const uint32_t empty = smem_addr(&empty_bar[stage]);
        // While the ring is full (the products wait for a phase's barrier), keep the memory system busy:
        // ask the tiles that will be copied next into L2, a bounded distance ahead.
        while (!mbar_test(empty, phase ^ 1u)) {
          if (lead < kChainL2Ahead && ahead.valid) {
            const ChainPhase& ph = args.phase[ahead.p];
            tma_prefetch_2d(&maps.w[ahead.p], ahead.kb * kChainTileK, ahead.half * ph.N + ahead.tile * kChainTileN);
            ahead.next(args, cta, grid);
            ++lead;
          } else {
            ok = mbar_wait(empty, phase ^ 1u, aborted, args.fault, 1 << 8);
            break;
          }
        }
        if (!ok) break;
        const ChainPhase& ph = args.phase[load.p];
        const uint32_t bar = smem_addr(&full_bar[stage]);
        mbar_expect_tx(bar, Shape::kWeightBytes);
        tma_load_2d_hint(stage_a(stage), &maps.w[load.p], bar, load.kb * kChainTileK, load.half * ph.N + load.tile * kChainTileN,
                         weights_once);
        ++filled;
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
        const int was = load.p;
        load.next(args, cta, grid);
        if (lead > 0) --lead; else ahead = load;
        if (!load.valid || load.p != was) {
          for (; stamped <= was; ++stamped) chain_stamp(args, cta, stamped, 5);
        }
      }
      if (!ok || *aborted) {
        // copies in flight must land before the CTA may exit; a stage whose activation copy never came is
        // completed by hand so that the wait below can end
        for (int s = 0; s < kStages; ++s) {
          const long long fills = (filled - s + kStages - 1) / kStages;
          if (fills > 0) {
            mbar_arrive(smem_addr(&full_bar[s]));
            mbar_wait(smem_addr(&full_bar[s]), static_cast<uint32_t>((fills - 1) & 1), aborted, args.fault);
          }
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ activations (TMA), waits at phase boundaries
    if (lane == 0) {
      if (args.pdl) pdl_wait();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int p = 0; p < args.phases && ok; ++p) {
        const ChainPhase& ph = args.phase[p];
        const int chunks = ph.n_tiles * ph.split, halves = ph.swiglu ? 2 : 1;
        const int mine = first_chunk(ph);
        if (p > 0 && mine < chunks) {
          ok = wait_counter(args.counters + kChainCounterBarrier, static_cast<unsigned>(grid) * p, args.counters, aborted,
                            args.fault);
          if (!ok) break;
          fence_proxy_async_all();     // what other CTAs stored with ordinary writes is now read by the copy engine
        }
        chain_stamp(args, cta, p, 6);
        for (int c = mine; c < chunks && ok; c += grid) {
          const int tile = c / ph.split, seg = c - tile * ph.split;
          int kb_begin, kb_count;
          segment_range(ph.k_blocks, ph.split, seg, kb_begin, kb_count);
          for (int kb = kb_begin; kb < kb_begin + kb_count && ok; ++kb) {
            for (int half = 0; half < halves; ++half) {
              ok = mbar_wait(smem_addr(&empty_bar[stage]), phase ^ 1u, aborted, args.fault, 1 << 9);
              if (!ok) break;
              const uint32_t bar = smem_addr(&full_bar[stage]);
              if (half == 0) {
                mbar_expect_tx(bar, Shape::kTokenBytes);
                tma_load_2d(stage_b(stage), &maps.x[p], bar, kb * kChainTileK, 0);
              } else {
                mbar_arrive(bar);        // the up rows multiply the tokens of the gate rows' stage
              }
              if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tensor-core issuer
    if (lane == 0) {
      int stage = 0, buf = 0;
      uint32_t phase = 0, acc_phase[2] = {0, 0};
      bool ok = true;
      for (int p = 0; p < args.phases && ok; ++p) {
        const ChainPhase& ph = args.phase[p];
        const int chunks = ph.n_tiles * ph.split;
        for (int c = first_chunk(ph); c < chunks && ok; c += grid) {
          const int tile = c / ph.split, seg = c - tile * ph.split;
          int kb_begin, kb_count;
          segment_range(ph.k_blocks, ph.split, seg, kb_begin, kb_count);
          ok = mbar_wait(smem_addr(&acc_empty_bar[buf]), acc_phase[buf] ^ 1u, aborted, args.fault, 1 << 10);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * Shape::kAccColumns;
          for (int kb = 0; kb < kb_count; ++kb) {
            ok = mbar_wait(smem_addr(&full_bar[stage]), phase, aborted, args.fault, 1 << 11);
            if (!ok) break;
            tc_fence_after();
            const uint64_t b_desc = operand_desc(stage_b(stage));
            const uint64_t a_desc = operand_desc(stage_a(stage));
#pragma unroll
            for (int k = 0; k < kChainTileK / kChainUmmaK; ++k)
              umma_bf16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
            const int gate_stage = stage;
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
            if (ph.swiglu) {
              ok = mbar_wait(smem_addr(&full_bar[stage]), phase, aborted, args.fault, 1 << 11);
              if (!ok) break;
              tc_fence_after();
              const uint64_t up_desc = operand_desc(stage_a(stage));
#pragma unroll
              for (int k = 0; k < kChainTileK / kChainUmmaK; ++k)
                umma_bf16(d_tmem + BN, up_desc + 2 * k, b_desc + 2 * k, kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
              umma_commit(smem_addr(&empty_bar[gate_stage]));     // both are free once all of these retire
              umma_commit(smem_addr(&empty_bar[stage]));
              if (++stage == kStages) { stage = 0; phase ^= 1u; }
            } else {
              umma_commit(smem_addr(&empty_bar[gate_stage]));
            }
          }
          if (!ok) break;
          umma_commit(smem_addr(&acc_full_bar[buf]));
          acc_phase[buf] ^= 1u;
          buf ^= 1;
        }
        chain_stamp(args, cta, p, 7);
      }
      umma_commit(smem_addr(&drain_bar));
      mbar_wait(smem_addr(&drain_bar), 0, aborted, args.fault);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 3..6)
    const int quarter = warp & 3;                       // the 32 tensor-memory lanes this warp may read
    const int et = static_cast<int>(threadIdx.x) - 96;  // 0..127
    const int ew = warp - 3;                            // 0..3
    const int row_local = quarter * 32 + lane;
    int buf = 0;
    uint32_t acc_phase[2] = {0, 0};
    bool ok = true;
    if (args.pdl) pdl_wait();
    for (int p = 0; p < args.phases && ok; ++p) {
      const ChainPhase& ph = args.phase[p];
      const int chunks = ph.n_tiles * ph.split, halves = ph.swiglu ? 2 : 1;
      const int mine = first_chunk(ph);
      if (p > 0) {
        // Every CTA waits here, with or without work in this phase: a CTA that arrived at this phase's
        // barrier before the last phase's was complete would make the count mean nothing.
        bool passed = true;
        if (et == 0)
          passed = wait_counter(args.counters + kChainCounterBarrier, static_cast<unsigned>(grid) * p, args.counters,
                                aborted, args.fault);
        ok = named_barrier_and(1, 128, passed);
        if (!ok) break;
        if (p == args.phases - 1 && args.pdl && et == 0) pdl_trigger();
      }
      if (et == 0) chain_stamp(args, cta, p, 0);
      bool first_chunk_seen = false;
      if (mine < chunks) {
        const bool scaled = ph.sumsq_in != nullptr;
        if (scaled) {
          // 128 / BN neighbouring threads add up a token's row of the table, always in the same order
          constexpr int kPerToken = 128 / BN;
          const int token = et / kPerToken, sub = et % kPerToken;
          float sum = 0.0f;
          if (token < args.T) {
            const float4* row = reinterpret_cast<const float4*>(ph.sumsq_in + static_cast<size_t>(token) * ph.sumsq_count);
            for (int q = sub; q < ph.sumsq_count / 4; q += kPerToken) {
              const float4 four = __ldcg(row + q);
              sum += (four.x + four.y) + (four.z + four.w);
            }
          }
#pragma unroll
          for (int offset = kPerToken / 2; offset >= 1; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
          if (sub == 0) row_scale[token] = token < args.T ? rsqrtf(sum * ph.inv_norm_size + ph.norm_eps) : 1.0f;
          named_barrier(1, 128);
        }

        // pass 1: this CTA's chunks leave tensor memory, as results (an unsplit tile) or as partial tiles
        for (int c = mine; c < chunks && ok; c += grid) {
          const int tile = c / ph.split;
          ok = named_barrier_and(1, 128, mbar_wait(smem_addr(&acc_full_bar[buf]), acc_phase[buf], aborted, args.fault, 1 << 13));
          if (!ok) break;
          tc_fence_after();
          if (et == 0 && !first_chunk_seen) chain_stamp(args, cta, p, 1);
          first_chunk_seen = true;
          const uint32_t acc = tmem_base + buf * Shape::kAccColumns + (static_cast<uint32_t>(quarter * 32) << 16);
          if (ph.split == 1) {
            const int n = tile * kChainTileN + row_local;
#pragma unroll 1
            for (int col = 0; col < BN && col < args.T; col += 16) {
              float v[16], u[16];
              tmem_load16(acc + col, v);
              if (ph.swiglu) tmem_load16(acc + BN + col, u);
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int t = col + j;                  // the same for the whole warp
                if (t < args.T)
                  chain_emit(ph, t, n, tile, quarter, lane, v[j], ph.swiglu ? u[j] : 0.0f, scaled ? row_scale[t] : 1.0f);
              }
            }
          } else {
            float* mine_out = args.scratch + (static_cast<size_t>(c) * halves * BN) * kChainTileN + row_local;
#pragma unroll 1
            for (int col = 0; col < halves * BN; col += 16) {
              if ((col % BN) >= args.T) continue;       // columns of tokens that do not exist
              float v[16];
              tmem_load16(acc + col, v);
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if ((col % BN) + j < args.T) __stcg(mine_out + static_cast<size_t>(col + j) * kChainTileN, v[j]);
            }
            __threadfence();
            named_barrier(1, 128);
            if (et == 0) atomicAdd(args.counters + kChainCounterTiles + p * kChainMaxTiles + tile, 1u);
          }
          // the accumulator buffer may be overwritten from here on
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_addr(&acc_empty_bar[buf]));
          acc_phase[buf] ^= 1u;
          buf ^= 1;
        }

        if (et == 0) chain_stamp(args, cta, p, 2);
        // pass 2: every CTA of a split tile sums its share of the tile over all segments, in segment order
        if (ph.split > 1 && ok) {
          for (int c = mine; c < chunks; c += grid) {
            const int tile = c / ph.split, seg = c - tile * ph.split;
            bool complete = true;
            if (et == 0)
              complete = wait_counter(args.counters + kChainCounterTiles + p * kChainMaxTiles + tile,
                                      static_cast<unsigned>(ph.split), args.counters, aborted, args.fault);
            ok = named_barrier_and(1, 128, complete);
            if (!ok) break;
            if (et == 0) chain_stamp(args, cta, p, 3);
            const float* parts = args.scratch + (static_cast<size_t>(tile) * ph.split * halves * BN) * kChainTileN;
            const size_t seg_stride = static_cast<size_t>(halves) * BN * kChainTileN;
            // units of 32 rows of one token: unit u = 4 * token + quarter; this CTA takes every split-th,
            // its four warps take turns
            for (int u = seg + ph.split * ew; u < 4 * args.T; u += 4 * ph.split) {
              const int group = u & 3, t = u >> 2;
              const int row = group * 32 + lane;
              const float* at = parts + static_cast<size_t>(t) * kChainTileN + row;
              float gate_part[kChainMaxSplit], up_part[kChainMaxSplit];
#pragma unroll
              for (int q = 0; q < kChainMaxSplit; ++q) {
                gate_part[q] = q < ph.split ? __ldcg(at + q * seg_stride) : 0.0f;
                up_part[q] = ph.swiglu && q < ph.split ? __ldcg(at + q * seg_stride + static_cast<size_t>(BN) * kChainTileN) : 0.0f;
              }
              float gate = 0.0f, up = 0.0f;
#pragma unroll
              for (int q = 0; q < kChainMaxSplit; ++q) {
                if (q < ph.split) {
                  gate += gate_part[q];
                  up += up_part[q];
                }
              }
              chain_emit(ph, t, tile * kChainTileN + row, tile, group, lane, gate, up, scaled ? row_scale[t] : 1.0f);
            }
          }
        }
      }
      if (!ok) break;
      // the phase's results of this CTA are stored: count it in at the phase's barrier
      fence_proxy_async_all();
      __threadfence();
      named_barrier(1, 128);
      if (et == 0) {
        atomicAdd(args.counters + kChainCounterBarrier, 1u);
        chain_stamp(args, cta, p, 4);
      }
    }
    if (args.phases == 1 && args.pdl && et == 0) pdl_trigger();
    if (!ok && et == 0) atomicExch(args.counters + kChainCounterAbort, 1u);   // the others need not wait their full time
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Shape::kTmemColumns);
  }
  // the CTA that leaves last puts the counters back to zero for the next launch
  if (threadIdx.x == 0) {
    __threadfence();
    last_flag = atomicAdd(args.counters + kChainCounterExit, 1u) == static_cast<unsigned>(grid) - 1u ? 1 : 0;
  }
  __syncthreads();
  if (last_flag) {
    __threadfence();
    for (int p = 0; p < args.phases; ++p)
      for (int tile = threadIdx.x; tile < args.phase[p].n_tiles; tile += kChainThreads)
        args.counters[kChainCounterTiles + p * kChainMaxTiles + tile] = 0u;
    if (threadIdx.x == 0) {
      args.counters[kChainCounterBarrier] = 0u;
      args.counters[kChainCounterExit] = 0u;
    }
  }
}

// ----------------------------------------------------------------------------- host
static int chain_sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  return sms;
}

// Segments per tile: about two chunks per CTA and phase (so that a CTA's second chunk multiplies while its first
// leaves tensor memory, and the round-robin deal evens out), at least four k-blocks each.
static int chain_split(int n_tiles, int k_blocks, int grid) {
  int split = (2 * grid + n_tiles / 2) / n_tiles;
  if (split > kChainMaxSplit) split = kChainMaxSplit;
  if (split > k_blocks / 4) split = k_blocks / 4;
  return split < 1 ? 1 : split;
}

static int chain_token_tile(int tokens) { return tokens <= 16 ? 16 : tokens <= 32 ? 32 : 64; }

static bool g_chain_configured[3] = {};

template <int BN>
static int launch_chain(const ChainMaps& maps, const ChainArgs& args, int grid, cudaStream_t stream) {
  using Shape = ChainShape<BN>;
  auto kernel = gemm_chain_kernel<BN>;
  bool& configured = g_chain_configured[BN / 32];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(Shape::kSmemBytes));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kChainThreads);
  config.dynamicSmemBytes = Shape::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = args.pdl ? 1 : 0;
  return static_cast<int>(cudaLaunchKernelEx(&config, kernel, maps, args));
}

}  // namespace rl

extern "C" {

// One phase of a chain as the caller describes it; the fields are those of rl_gemm_bf16_norm.
struct RlChainPhase {
  const void* x;            // [tokens, k]; for phases after the first, what an earlier phase wrote
  const void* w;            // [n_out, k], SwiGLU [2 n_out, k]
  void* out;                // [tokens, n_out]
  int n_out, k, swiglu;
  float* residual;
  const float* norm_weight;
  float* sumsq_out;
  const float* sumsq_in;
  int sumsq_count;
  float norm_eps;
  int norm_size;
  const float* bias;
};

int rl_gemm_chain_max_phases() { return rl::kChainMaxPhases; }
int rl_gemm_chain_max_tokens() { return 64; }
// unsigned words of the counters a chain needs (zeroed once by the caller, kept zero by the kernel)
int rl_gemm_chain_counter_words() { return rl::kChainCounters; }

// float32 words of scratch the chain needs for its partial tiles
long long rl_gemm_chain_scratch_floats(const RlChainPhase* phases, int count, int tokens) {
  const int grid = rl::chain_sm_count(), bn = rl::chain_token_tile(tokens);
  long long most = 0;
  for (int p = 0; p < count; ++p) {
    const int n_tiles = (phases[p].n_out + rl::kChainTileN - 1) / rl::kChainTileN;
    const int k_blocks = (phases[p].k + rl::kChainTileK - 1) / rl::kChainTileK;
    const int split = rl::chain_split(n_tiles, k_blocks, grid);
    const long long need = split == 1 ? 0 : static_cast<long long>(n_tiles) * split * (phases[p].swiglu ? 2 : 1) * bn * rl::kChainTileN;
    if (need > most) most = need;
  }
  return most;
}

// Runs `count` products back to back as one persistent kernel (see the top of this file).  All operands
// bfloat16, contiguous, 16-byte aligned, inner sizes multiples of 8; at most 64 tokens; `scratch` holds at
// least rl_gemm_chain_scratch_floats() floats; `counters` holds rl_gemm_chain_counter_words() zeros; `trace`
// (null, or rl_gemm_chain_trace_words() 64-bit words per multiprocessor) receives time stamps.
int rl_gemm_chain_trace_words() { return rl::kChainMaxPhases * rl::kChainTraceEvents; }   // 64-bit words per CTA

int rl_gemm_chain(const RlChainPhase* phases, int count, int tokens, float* scratch, long long scratch_floats,
                  unsigned* counters, unsigned long long* trace, int pdl, int* fault, cudaStream_t stream) {
  if (count <= 0 || tokens == 0) return 0;
  if (count > rl::kChainMaxPhases || tokens < 0 || tokens > 64 || counters == nullptr)
    return static_cast<int>(cudaErrorInvalidValue);
  if (rl_gemm_chain_scratch_floats(phases, count, tokens) > scratch_floats) return static_cast<int>(cudaErrorInvalidValue);
  const int grid = rl::chain_sm_count(), bn = rl::chain_token_tile(tokens);
  rl::ChainMaps maps;
  rl::ChainArgs args;
  args.T = tokens;
  args.phases = count;
  args.pdl = pdl;
  args.fault = fault;
  args.scratch = scratch;
  args.counters = counters;
  args.trace = trace;
  int next_cta = 0;
  for (int p = 0; p < count; ++p) {
    const RlChainPhase& in = phases[p];
    if (in.n_out <= 0 || in.k <= 0 || in.k % 8 != 0 || (reinterpret_cast<uintptr_t>(in.x) & 15) ||
        (reinterpret_cast<uintptr_t>(in.w) & 15))
      return static_cast<int>(cudaErrorInvalidValue);
    const bool norm_follows = in.residual != nullptr || in.norm_weight != nullptr || in.sumsq_out != nullptr;
    if (norm_follows && (in.residual == nullptr || in.norm_weight == nullptr || in.sumsq_out == nullptr || in.swiglu != 0))
      return static_cast<int>(cudaErrorInvalidValue);
    if (in.sumsq_in != nullptr && (in.sumsq_count <= 0 || in.sumsq_count % 4 != 0 || in.norm_size <= 0 ||
                                   (reinterpret_cast<uintptr_t>(in.sumsq_in) & 15)))
      return static_cast<int>(cudaErrorInvalidValue);
    rl::ChainPhase& ph = args.phase[p];
    ph.out = static_cast<rl::bf16*>(in.out);
    ph.N = in.n_out;
    ph.K = in.k;
    ph.swiglu = in.swiglu != 0 ? 1 : 0;
    ph.n_tiles = (in.n_out + rl::kChainTileN - 1) / rl::kChainTileN;
    ph.k_blocks = (in.k + rl::kChainTileK - 1) / rl::kChainTileK;
    if (ph.n_tiles > rl::kChainMaxTiles) return static_cast<int>(cudaErrorInvalidValue);
    ph.split = rl::chain_split(ph.n_tiles, ph.k_blocks, grid);
    ph.first_cta = next_cta;
    next_cta = (next_cta + ph.n_tiles * ph.split) % grid;
    ph.residual = in.residual;
    ph.norm_weight = in.norm_weight;
    ph.sumsq_out = in.sumsq_out;
    ph.sumsq_in = in.sumsq_in;
    ph.sumsq_count = in.sumsq_count;
    ph.norm_eps = in.norm_eps;
    ph.inv_norm_size = in.norm_size > 0 ? 1.0f / static_cast<float>(in.norm_size) : 0.0f;
    ph.bias = in.bias;
    int status = rl::make_map(&maps.w[p], in.w, static_cast<long long>(in.n_out) * (in.swiglu ? 2 : 1), in.k, rl::kChainTileN);
    if (status != 0) return status;
    status = rl::make_map(&maps.x[p], in.x, tokens, in.k, bn);
    if (status != 0) return status;
  }
  for (int p = count; p < rl::kChainMaxPhases; ++p) {
    args.phase[p] = args.phase[0];
    maps.w[p] = maps.w[0];
    maps.x[p] = maps.x[0];
  }
  if (bn == 16) return rl::launch_chain<16>(maps, args, grid, stream);
  if (bn == 32) return rl::launch_chain<32>(maps, args, grid, stream);
  return rl::launch_chain<64>(maps, args, grid, stream);
}

}  // extern "C"

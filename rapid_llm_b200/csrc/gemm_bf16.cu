// bfloat16 matrix product of the linear layers on the sm_100a tensor cores:
//   out[T, N] = x[T, K] . w[N, K]^T                      (plain)
//   out[T, I] = silu(x . w[0:I]^T) * (x . w[I:2I]^T)     (fused SwiGLU over a [2I, K] weight)
// float32 accumulation in tensor memory, one rounding at the store.
//
// The weight is the M side of the instruction: one tcgen05.mma covers 128 weight rows by
// BN tokens (BN = 16 .. 256), so a decode step of a few tokens still fills the 128 lanes of
// the tensor core and the kernel is a pure stream of the weight matrix.  Operands reach
// shared memory through TMA in 128-byte-swizzled tiles of 64 k-elements (rows beyond T or N
// and columns beyond K read as zeros), a ring of stages decouples the copy engine from the
// tensor core, and the accumulator of a tile sits in one of two tensor-memory buffers so its
// epilogue overlaps the next tile's products.  Roles: warp 0 issues TMA, warp 1 issues
// tcgen05.mma (one elected thread each), warps 2..5 read the accumulators back
// (tcgen05.ld), apply the epilogue and store.
//
// Few tokens mean few tiles (N / 128), too few to keep 148 SMs streaming.  The k-range of a
// tile is then split over the CTAs of a thread-block cluster: each accumulates its slice in
// tensor memory, parks the float32 partial tile in its own shared memory, and after a
// cluster barrier every CTA sums a share of the tile's token columns over all ranks through
// distributed shared memory (16 bytes, four weight rows of a column, per load), in rank order
// (so the sum does not depend on timing), and stores it.  No global scratch, no atomics.  With many tokens the k-range is not split and a
// CTA walks several tiles, the epilogue of one overlapping the products of the next.
//
// A norm between two products can ride on them instead of being a kernel of its own (steps of up
// to 64 tokens).  The product before it adds its float32 result to the residual row, stores the
// sum back, writes the sum times the norm's weight as the next product's input and leaves the
// sums of squares per token and 32 output columns in a small table; the product after it adds
// the table's row up (in a fixed order) and multiplies its own result by rsqrt(mean + eps): a
// row's scale commutes with the product.  The residual add, the squares and the scale are float32
// (formula: rapid_llm/kernels/ops/layernorm/skip_rmsnorm.py:41-48).
//
// Launched with programmatic stream serialization, the kernel starts while its predecessor
// in the stream drains: barriers, tensor memory and the first weight tiles (which no kernel
// writes) are set up and in flight before griddepcontrol.wait lets it read the activations.
//
// The reference calls a library product here (rapid_llm/kernels/ops/gemm/linear.py:17-40)
// and a separate SwiGLU kernel (rapid_llm/kernels/ops/activation/swiglu.py:91-121).
#include <cuda.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace rl {

using bf16 = __nv_bfloat16;

constexpr int kTileN = 128;           // weight rows per tile = M of one tcgen05.mma
constexpr int kTileK = 64;            // bf16 elements in one 128-byte swizzle row
constexpr int kUmmaK = 16;            // k-elements of one tcgen05.mma of kind::f16
constexpr int kGemmThreads = 192;

struct GemmArgs {
  bf16* out;               // [T, N]
  int* fault;
  int T, N, K;
  int up_offset;           // first "up" row of the weight (SwiGLU), else unused
  int n_tiles, t_tiles, k_blocks;
  int tile_rows;           // weight rows a tile brings (kTileN, or fewer so that the tiles of an unsplit SwiGLU product fill the GPU evenly)
  int k_split;             // CTAs (= cluster size) that share one tile's k-range
  int pdl;                 // launched with programmatic stream serialization
  // a norm that follows this product (plain products of one token tile only; all three or none):
  // residual[T, N] += result; out = bf16(residual * norm_weight[n]); sumsq_out[t, 4 * n_tiles] gets the
  // squares of the new residual summed over each tile's four groups of 32 columns
  float* residual;
  const float* norm_weight;
  float* sumsq_out;
  // a norm that came before it and left its scale open (one token tile only): the result of row t is
  // multiplied by rsqrt(sum(sumsq_in[t, 0:sumsq_count]) * inv_norm_size + norm_eps)
  const float* sumsq_in;
  int sumsq_count;
  float norm_eps, inv_norm_size;
  // added to every row of the result (after the open scale, before the SiLU or the residual add);
  // [N], for SwiGLU [2 N] with the gate's part first; may be null
  const float* bias;
};

__device__ __forceinline__ float silu_mul(float gate, float up) {
  return __fdividef(gate, 1.0f + __expf(-gate)) * up;   // the result is rounded to bfloat16
}

// One element of a product that a norm follows: the residual takes the sum, the output the sum times
// the norm's weight; returns the sum's square for the row's mean.
__device__ __forceinline__ float store_for_norm(const GemmArgs& args, size_t at, float norm_w, float sum) {
  args.residual[at] = sum;
  args.out[at] = __float2bfloat16_rn(sum * norm_w);
  return sum * sum;
}

template <bool kSwiglu, int BN>
struct GemmShape {
  static constexpr int kHalves = kSwiglu ? 2 : 1;
  static constexpr int kStageBytes = kHalves * kTileN * kTileK * 2 + BN * kTileK * 2;
  // Small token tiles stream weights.  Their ring stays within 74 KB, so that three CTAs fit an
  // SM: while two CTAs of one product stream, a CTA of the next one sets itself up and fetches
  // its first weight tiles beside them (measured: better than a deeper ring with two per SM, and
  // than a shallower one with four).  The SwiGLU tiles are twice as large and keep 110 KB, two
  // per SM.  Large token tiles get the whole SM.
  static constexpr bool kShareSm = BN <= 64 && 3 * kStageBytes <= 110 * 1024;
  static constexpr int kBudget = kShareSm ? (kSwiglu ? 110 : 74) * 1024 : 200 * 1024;
  static constexpr int kStagesFit = kBudget / kStageBytes;
  static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
  static constexpr int kAccColumns = kHalves * BN;          // per accumulator buffer
  static constexpr int kTmemColumns = 2 * kAccColumns < 32 ? 32 : 2 * kAccColumns;
  static constexpr int kPartialBytes = kHalves * BN * kTileN * 4;
  static constexpr bool kCanSplit = BN <= 64 && kPartialBytes <= kStages * kStageBytes;
  static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + 1024;
  static_assert(kTmemColumns <= 512 && (kTmemColumns & (kTmemColumns - 1)) == 0, "tensor memory");
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "token tile");
  static_assert(kStages >= 2, "pipeline depth");
};

// grid = (k_split, tile CTAs); with k_split > 1 the x dimension is one cluster and every CTA
// has exactly one tile; otherwise a CTA walks the tiles blockIdx.y, blockIdx.y + gridDim.y, ...
template <bool kSwiglu, int BN>
__global__ void __launch_bounds__(kGemmThreads)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const GemmArgs args) {
  using Shape = GemmShape<kSwiglu, BN>;
  constexpr int kStages = Shape::kStages, kHalves = Shape::kHalves;
  constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) |
                              (static_cast<uint32_t>(BN >> 3) << 17) |
                              (static_cast<uint32_t>(kTileN >> 4) << 24);
  extern __shared__ unsigned char gemm_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], acc_full_bar[2], acc_empty_bar[2], drain_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int aborted_flag;
  __shared__ float row_scale[BN <= 64 ? BN : 1];      // the scale an earlier norm left open, per token
  volatile int* aborted = &aborted_flag;

  if (args.pdl && threadIdx.x == 0) pdl_trigger();   // the successor may set itself up beside this kernel
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_addr(gemm_smem_raw) + 1023u) & ~1023u;
  auto stage_a = [&](int s, int half) { return smem_base + s * Shape::kStageBytes + half * kTileN * kTileK * 2; };
  auto stage_b = [&](int s) { return smem_base + s * Shape::kStageBytes + kHalves * kTileN * kTileK * 2; };

  // this CTA's slice of the k-blocks and its tiles
  const int rank = blockIdx.x;
  const int k_base = args.k_blocks / args.k_split, k_rem = args.k_blocks - k_base * args.k_split;
  const int kb_begin = rank * k_base + min(rank, k_rem);
  const int kb_count = k_base + (rank < k_rem ? 1 : 0);
  const int tiles = args.n_tiles * args.t_tiles;
  const int my_tiles = (tiles - static_cast<int>(blockIdx.y) + static_cast<int>(gridDim.y) - 1) /
                       static_cast<int>(gridDim.y);
  const long long total_iters = static_cast<long long>(my_tiles) * kb_count;
  auto tile_of = [&](int index) { return static_cast<int>(blockIdx.y) + index * static_cast<int>(gridDim.y); };

  // (tile index, k-block) of an iteration advance by counting: a division per copy would cost
  // this one thread more than the copy itself
  const uint64_t weights_once = l2_evict_first_policy();
  struct Cursor { int index, kb; };
  auto advance = [&](Cursor& c) { if (++c.kb == kb_count) { c.kb = 0; ++c.index; } };
  auto load_a = [&](const Cursor& c, int stage) {
    const int n_tile = tile_of(c.index) / args.t_tiles;
    const int k = (kb_begin + c.kb) * kTileK;
    const uint32_t bar = smem_addr(&full_bar[stage]);
    // a tile of fewer than kTileN weight rows fills the first rows of its place; the product still reads all
    // kTileN, and the accumulator's lanes past the tile's rows are never looked at
    mbar_expect_tx(bar, kHalves * args.tile_rows * kTileK * 2 + BN * kTileK * 2);
    tma_load_2d_hint(stage_a(stage, 0), &map_w, bar, k, n_tile * args.tile_rows, weights_once);
    if (kSwiglu) tma_load_2d_hint(stage_a(stage, 1), &map_w, bar, k, args.up_offset + n_tile * args.tile_rows, weights_once);
  };
  auto load_b = [&](const Cursor& c, int stage) {
    const int t_tile = tile_of(c.index) % args.t_tiles;
    tma_load_2d(stage_b(stage), &map_x, smem_addr(&full_bar[stage]), (kb_begin + c.kb) * kTileK, t_tile * BN);
  };
  const int prefetch = static_cast<int>(min(static_cast<long long>(kStages), total_iters));
  Cursor cursor = {0, 0};

  if (threadIdx.x == 64) {                    // an epilogue warp: idle until the first tile is done
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_addr(&full_bar[s]), 1);
      mbar_init(smem_addr(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_addr(&acc_full_bar[b]), 1);
      mbar_init(smem_addr(&acc_empty_bar[b]), 4);
    }
    mbar_init(smem_addr(&drain_bar), 1);
    aborted_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // The first weight tiles leave at once, before the rest of the CTA is set up and before the
    // kernel upstream has finished: nothing in the stream writes weights.
    for (int it = 0; it < prefetch; ++it) { load_a(cursor, it); advance(cursor); }
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // the weights of the first stages are on their way (set-up above); the activations only
      // once the kernel upstream has finished
      if (args.pdl) pdl_wait();
      Cursor second = {0, 0};
      for (int it = 0; it < prefetch; ++it) { load_b(second, it); advance(second); }
      int stage = prefetch % kStages;
      uint32_t phase = prefetch == kStages ? 1u : 0u;
      bool ok = true;
      long long filled = prefetch;                     // iterations whose copies were issued
      for (long long it = prefetch; it < total_iters; ++it) {
        ok = mbar_wait(smem_addr(&empty_bar[stage]), phase ^ 1u, aborted, args.fault);
        if (!ok) break;
        load_a(cursor, stage);
        load_b(cursor, stage);
        advance(cursor);
        ++filled;
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
      if (!ok || *aborted) {
        // copies still in flight must land before the CTA may exit: wait (bounded, like every
        // wait here) for the last fill of every stage
        for (int s = 0; s < kStages; ++s) {
          const long long fills = (filled - s + kStages - 1) / kStages;   // fills of stage s so far
          if (fills > 0)
            mbar_wait(smem_addr(&full_bar[s]), static_cast<uint32_t>((fills - 1) & 1), aborted, args.fault);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tensor-core issuer
    if (lane == 0) {
      int stage = 0, buf = 0;
      uint32_t phase = 0, acc_phase[2] = {0, 0};
      bool ok = kb_count > 0;
      for (int index = 0; index < my_tiles && ok; ++index) {
        ok = mbar_wait(smem_addr(&acc_empty_bar[buf]), acc_phase[buf] ^ 1u, aborted, args.fault);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * Shape::kAccColumns;
        for (int kb = 0; kb < kb_count; ++kb) {
          ok = mbar_wait(smem_addr(&full_bar[stage]), phase, aborted, args.fault);
          if (!ok) break;
          tc_fence_after();
          const uint64_t b_desc = operand_desc(stage_b(stage));
#pragma unroll
          for (int half = 0; half < kHalves; ++half) {
            const uint64_t a_desc = operand_desc(stage_a(stage, half));
#pragma unroll
            for (int k = 0; k < kTileK / kUmmaK; ++k) {
              // 32 bytes further along the swizzled row = +2 in the descriptor's address field
              umma_bf16(d_tmem + half * BN, a_desc + 2 * k, b_desc + 2 * k, kIdesc,
                        (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit(smem_addr(&empty_bar[stage]));   // the stage is free once these products retire
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(smem_addr(&acc_full_bar[buf]));
        acc_phase[buf] ^= 1u;
        buf ^= 1;
      }
      // nothing of this CTA may still be running on the tensor core when its memory is freed
      umma_commit(smem_addr(&drain_bar));
      mbar_wait(smem_addr(&drain_bar), 0, aborted, args.fault);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;                       // the 32 tensor-memory lanes this warp may read
    const int n_local = quarter * 32 + lane;
    int buf = 0;
    uint32_t acc_phase[2] = {0, 0};
    bool ok = kb_count > 0;
    if (args.pdl) pdl_wait();                           // the output buffer may still be read upstream
    if constexpr (BN <= 64) {
      if (args.sumsq_in != nullptr) {
        // 128 / BN neighbouring threads add up a token's row of the table (always in the same order)
        // while the first products run
        constexpr int kPerToken = 128 / BN;
        const int token = (static_cast<int>(threadIdx.x) - 64) / kPerToken;
        const int sub = (static_cast<int>(threadIdx.x) - 64) % kPerToken;
        float sum = 0.0f;
        if (token < args.T) {
          const float4* row = reinterpret_cast<const float4*>(args.sumsq_in + static_cast<size_t>(token) * args.sumsq_count);
#pragma unroll 8
          for (int p = sub; p < args.sumsq_count / 4; p += kPerToken) {
            const float4 four = row[p];
            sum += (four.x + four.y) + (four.z + four.w);
          }
        }
#pragma unroll
        for (int offset = kPerToken / 2; offset >= 1; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
        if (sub == 0) row_scale[token] = token < args.T ? rsqrtf(sum * args.inv_norm_size + args.norm_eps) : 1.0f;
        named_barrier(1, 128);
      }
    }
    const bool scaled = BN <= 64 && args.sumsq_in != nullptr;
    for (int index = 0; index < my_tiles && ok; ++index) {
      const int tile = tile_of(index);
      const int n_tile = tile / args.t_tiles, t_tile = tile - n_tile * args.t_tiles;
      // (a tile of fewer rows than lanes: only unsplit SwiGLU products, whose lanes past the tile's rows look like
      // columns past the matrix's edge)
      const int n = n_local < args.tile_rows ? n_tile * args.tile_rows + n_local : args.N;
      const int t0 = t_tile * BN;
      ok = mbar_wait(smem_addr(&acc_full_bar[buf]), acc_phase[buf], aborted, args.fault);
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + buf * Shape::kAccColumns + (static_cast<uint32_t>(quarter * 32) << 16);
      const float bias_gate = args.bias != nullptr && n < args.N ? args.bias[n] : 0.0f;
      const float bias_up = kSwiglu && args.bias != nullptr && n < args.N ? args.bias[args.up_offset + n] : 0.0f;
      if (args.k_split == 1) {
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          if (t0 + c >= args.T) break;
          float v[16];
          tmem_load16(acc + c, v);
          if (scaled) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] *= row_scale[c + j];
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] += bias_gate;
          if (kSwiglu) {
            float u[16];
            tmem_load16(acc + BN + c, u);
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = silu_mul(v[j], (scaled ? u[j] * row_scale[c + j] : u[j]) + bias_up);
          }
          if (!kSwiglu && args.residual != nullptr) {
            const float norm_w = n < args.N ? args.norm_weight[n] : 0.0f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = t0 + c + j;                 // the same for the whole warp
              if (t < args.T) {
                const size_t at = static_cast<size_t>(t) * args.N + n;
                const float sq = warp_sum(n < args.N ? store_for_norm(args, at, norm_w, args.residual[at] + v[j]) : 0.0f);
                if (lane == 0) args.sumsq_out[static_cast<size_t>(t) * (4 * args.n_tiles) + 4 * n_tile + quarter] = sq;
              }
            }
          } else if (n < args.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (t0 + c + j < args.T)
                args.out[static_cast<size_t>(t0 + c + j) * args.N + n] = __float2bfloat16_rn(v[j]);
          }
        }
      } else if (Shape::kCanSplit) {
        // park the partial tile in this CTA's shared memory: [halves * BN columns][128 rows]
        float* mine = reinterpret_cast<float*>(gemm_smem_raw + (smem_base - smem_addr(gemm_smem_raw))) + n_local;
#pragma unroll 1
        for (int c = 0; c < kHalves * BN; c += 16) {
          float v[16];
          tmem_load16(acc + c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) mine[(c + j) * kTileN] = v[j];
        }
      }
      // the accumulator buffer may be overwritten from here on
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&acc_empty_bar[buf]));
      acc_phase[buf] ^= 1u;
      buf ^= 1;
    }
  }

  if (args.k_split > 1) {
    // sum the partial tiles of the cluster's CTAs: rank r takes the token columns r, r + k_split, ...; each of
    // its four epilogue warps takes every fourth of those, a lane four neighbouring weight rows of the column.
    // What bounds this step is the number of requests between the CTAs' shared memories, not their latency
    // (a 64-token tile summed with 4-byte loads took 3.3 us, eight columns a rank): a lane fetches its four
    // rows of a rank's partial tile in one 16-byte load, a warp 512 consecutive bytes.
    __syncwarp();
    cluster_sync();
    if (warp >= 2 && Shape::kCanSplit && !*aborted) {
      const int tile = static_cast<int>(blockIdx.y);
      const int n_tile = tile / args.t_tiles, t_tile = tile - n_tile * args.t_tiles;
      const int rows0 = 4 * lane;                                // this lane's rows of the tile
      const int n = n_tile * kTileN + rows0, t0 = t_tile * BN;
      // where the other ranks keep these rows of a column of the partial tile
      uint32_t peer[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) peer[q] = q < args.k_split ? peer_smem(smem_base + rows0 * 4, q) : 0u;
      const bool scaled = BN <= 64 && args.sumsq_in != nullptr;
      const bool norm_follows = !kSwiglu && args.residual != nullptr;
      float norm_w[4], bias_gate[4], bias_up[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const bool live = n + r < args.N;
        norm_w[r] = norm_follows && live ? args.norm_weight[n + r] : 0.0f;
        bias_gate[r] = args.bias != nullptr && live ? args.bias[n + r] : 0.0f;
        bias_up[r] = kSwiglu && args.bias != nullptr && live ? args.bias[args.up_offset + n + r] : 0.0f;
      }
      // output rows are 16-byte-aligned groups of four only if the row length allows it
      const bool wide_rows = (args.N & 3) == 0;
      for (int j = rank + (warp - 2) * args.k_split; j < BN && t0 + j < args.T; j += 4 * args.k_split) {
        // all loads first, the sums (in rank order) after
        float4 gate_part[8], up_part[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          gate_part[q] = q < args.k_split ? load_peer_f32x4(peer[q] + j * kTileN * 4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          up_part[q] = kSwiglu && q < args.k_split ? load_peer_f32x4(peer[q] + (BN + j) * kTileN * 4)
                                                    : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        float gate[4] = {0.0f, 0.0f, 0.0f, 0.0f}, up[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (q < args.k_split) {
            gate[0] += gate_part[q].x; gate[1] += gate_part[q].y; gate[2] += gate_part[q].z; gate[3] += gate_part[q].w;
            up[0] += up_part[q].x; up[1] += up_part[q].y; up[2] += up_part[q].z; up[3] += up_part[q].w;
          }
        }
        const float scale = scaled ? row_scale[j] : 1.0f;
        const size_t at = static_cast<size_t>(t0 + j) * args.N + n;
        float result[4], squares = 0.0f;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float g = gate[r] * scale + bias_gate[r], u = up[r] * scale + bias_up[r];
          result[r] = kSwiglu ? silu_mul(g, u) : g;
        }
        if (norm_follows) {
          float before[4] = {0.0f, 0.0f, 0.0f, 0.0f};
          if (wide_rows && n + 3 < args.N) {
            const float4 old = *reinterpret_cast<const float4*>(args.residual + at);
            before[0] = old.x; before[1] = old.y; before[2] = old.z; before[3] = old.w;
          } else {
#pragma unroll
            for (int r = 0; r < 4; ++r)
              if (n + r < args.N) before[r] = args.residual[at + r];
          }
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            before[r] += result[r];                                // the new residual
            result[r] = before[r] * norm_w[r];
            if (n + r < args.N) squares += before[r] * before[r];
          }
          if (wide_rows && n + 3 < args.N) {
            *reinterpret_cast<float4*>(args.residual + at) = make_float4(before[0], before[1], before[2], before[3]);
          } else {
#pragma unroll
            for (int r = 0; r < 4; ++r)
              if (n + r < args.N) args.residual[at + r] = before[r];
          }
          // the whole tile's squares of this token in the first of the tile's four places, zeros in the others
          const float sq = warp_sum(squares);
          if (lane < 4) args.sumsq_out[static_cast<size_t>(t0 + j) * (4 * args.n_tiles) + 4 * n_tile + lane] = lane == 0 ? sq : 0.0f;
        }
        if (wide_rows && n + 3 < args.N) {
          const __nv_bfloat162 lo = __floats2bfloat162_rn(result[0], result[1]), hi = __floats2bfloat162_rn(result[2], result[3]);
          uint2 packed;
          packed.x = *reinterpret_cast<const uint32_t*>(&lo);
          packed.y = *reinterpret_cast<const uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(args.out + at) = packed;
        } else {
#pragma unroll
          for (int r = 0; r < 4; ++r)
            if (n + r < args.N) args.out[at + r] = __float2bfloat16_rn(result[r]);
        }
      }
    }
    __syncwarp();
    cluster_sync();   // nobody leaves while its shared memory may still be read
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Shape::kTmemColumns);
  }
}

// ----------------------------------------------------------------------------- host
static int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  return sms;
}

static bool g_gemm_configured[2][9] = {};   // [swiglu][BN / 32]; file-local on purpose

template <bool kSwiglu, int BN>
static int launch_gemm(const CUtensorMap& map_w, const CUtensorMap& map_x, GemmArgs args, int forced_split,
                       cudaStream_t stream) {
  using Shape = GemmShape<kSwiglu, BN>;
  auto kernel = gemm_bf16_kernel<kSwiglu, BN>;
  bool& configured = g_gemm_configured[kSwiglu ? 1 : 0][BN / 32];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(Shape::kSmemBytes));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  // how many CTAs the GPU holds at once, and how finely to split k so that they all stream
  // (three CTAs of the plain products' small tiles fit an SM and splitting for three pays there; measured)
  const int resident = sm_count() * (Shape::kShareSm ? (!kSwiglu ? 3 : 2) : 1);
  const int tiles = args.n_tiles * args.t_tiles;
  int split = 1;
  if (Shape::kCanSplit) {
    if (forced_split > 0) {
      split = forced_split;
    } else {
      // the largest power of two (clusters of other sizes schedule poorly) that still lets
      // every CTA be resident at once; 8 is the portable cluster limit
      while (split < 8 && 2 * split * tiles <= resident) split *= 2;
    }
    if (split > args.k_blocks / 2) split = args.k_blocks / 2;   // at least two k-blocks per CTA
    if (split < 1) split = 1;
  }
  args.k_split = split;
  cudaLaunchConfig_t config = {};
  // a product that is not split walks its tiles with as many CTAs as fit: three per SM for the small rings
  const int walkers = Shape::kShareSm && !kSwiglu ? 3 * sm_count() : resident;
  config.gridDim = dim3(split, split > 1 ? tiles : (tiles < walkers ? tiles : walkers));
  config.blockDim = dim3(kGemmThreads);
  config.dynamicSmemBytes = Shape::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  int count = 0;
  if (split > 1) {
    attributes[count].id = cudaLaunchAttributeClusterDimension;
    attributes[count].val.clusterDim.x = split;
    attributes[count].val.clusterDim.y = 1;
    attributes[count].val.clusterDim.z = 1;
    ++count;
  }
  if (args.pdl) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  return static_cast<int>(cudaLaunchKernelEx(&config, kernel, map_w, map_x, args));
}

static int token_tile(int tokens, bool swiglu) {
  if (tokens <= 16) return 16;
  if (tokens <= 32) return 32;
  if (tokens <= 64) return 64;
  if (tokens <= 128 || swiglu) return 128;
  return 256;
}

}  // namespace rl

extern "C" {

// x: [tokens, k], w: [n_out, k] (swiglu: [2 * n_out, k], gate rows first), out: [tokens, n_out];
// all bfloat16, contiguous, 16-byte aligned, k a multiple of 8.  `pdl` launches with
// programmatic stream serialization (the previous kernel of the stream must then be one that
// tolerates an early successor; every kernel of this library does).  `k_split` forces the
// number of CTAs per tile (0 = choose).
//
// A norm that follows (`residual`, `norm_weight`, `sumsq_out`: all or none; float32; plain products of
// at most 64 tokens): residual[tokens, n_out] += result, out = residual * norm_weight, and
// sumsq_out[tokens, rl_gemm_bf16_sumsq_count(n_out)] receives partial sums of the new residual's squares.
// A norm that came before (`sumsq_in[tokens, sumsq_count]`, at most 64 tokens): row t of the result is
// multiplied by rsqrt(sum(sumsq_in[t]) / norm_size + norm_eps).
// `bias` (float32 [n_out], SwiGLU [2 n_out]; may be null) is added to every row after that scale.
int rl_gemm_bf16_norm(const void* x, const void* w, void* out, int tokens, int n_out, int k, int swiglu, int pdl,
                      int k_split, float* residual, const float* norm_weight, float* sumsq_out,
                      const float* sumsq_in, int sumsq_count, float norm_eps, int norm_size, const float* bias,
                      int* fault, cudaStream_t stream) {
  if (tokens == 0 || n_out == 0) return 0;
  if (tokens < 0 || n_out < 0 || k <= 0 || k % 8 != 0 || k_split < 0 || k_split > 8 ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return static_cast<int>(cudaErrorInvalidValue);
  const bool norm_follows = residual != nullptr || norm_weight != nullptr || sumsq_out != nullptr;
  if (norm_follows && (residual == nullptr || norm_weight == nullptr || sumsq_out == nullptr || swiglu != 0 || tokens > 64))
    return static_cast<int>(cudaErrorInvalidValue);
  if (sumsq_in != nullptr && (tokens > 64 || sumsq_count <= 0 || sumsq_count % 4 != 0 || norm_size <= 0 ||
                              (reinterpret_cast<uintptr_t>(sumsq_in) & 15)))
    return static_cast<int>(cudaErrorInvalidValue);
  const int bn = rl::token_tile(tokens, swiglu != 0);
  const int t_tiles = (tokens + bn - 1) / bn;
  // An unsplit SwiGLU product of token tiles that take a multiprocessor each (33 tokens and more) walks its weight
  // tiles in rounds of one tile per multiprocessor.  Tiles of 128 rows leave the last round part empty (96 tiles
  // of a 12,288-row product on 148 multiprocessors); tiles of fewer rows, as many as fill the rounds evenly (88:
  // 140 tiles), shorten every CTA's stream instead.
  int tile_rows = rl::kTileN;
  if (swiglu != 0 && bn >= 64 && k_split <= 1) {
    const long long sms = rl::sm_count();
    const long long tiles = static_cast<long long>((n_out + rl::kTileN - 1) / rl::kTileN) * t_tiles;
    const long long rounds = (tiles + sms - 1) / sms;
    const long long per_token_tile = rounds * sms / t_tiles;                    // weight tiles that fill the rounds
    if (per_token_tile > 0) {
      const long long rows = ((n_out + per_token_tile - 1) / per_token_tile + 7) / 8 * 8;
      if (rows >= 32 && rows < rl::kTileN) tile_rows = static_cast<int>(rows);
    }
    if (tile_rows != rl::kTileN) k_split = 1;       // such tiles are never shared by a cluster
  }
  CUtensorMap map_w, map_x;
  int status = rl::make_map(&map_w, w, static_cast<long long>(n_out) * (swiglu ? 2 : 1), k, tile_rows);
  if (status != 0) return status;
  status = rl::make_map(&map_x, x, tokens, k, bn);
  if (status != 0) return status;
  rl::GemmArgs args;
  args.out = static_cast<rl::bf16*>(out);
  args.fault = fault;
  args.T = tokens; args.N = n_out; args.K = k;
  args.up_offset = n_out;
  args.tile_rows = tile_rows;
  args.n_tiles = (n_out + tile_rows - 1) / tile_rows;
  args.t_tiles = t_tiles;
  args.k_blocks = (k + rl::kTileK - 1) / rl::kTileK;
  args.k_split = 1;
  args.pdl = pdl;
  args.residual = residual;
  args.norm_weight = norm_weight;
  args.sumsq_out = sumsq_out;
  args.sumsq_in = sumsq_in;
  args.sumsq_count = sumsq_count;
  args.norm_eps = norm_eps;
  args.inv_norm_size = norm_size > 0 ? 1.0f / static_cast<float>(norm_size) : 0.0f;
  args.bias = bias;
#define RL_GEMM_CASE(SW, BNV) \
  if ((swiglu != 0) == SW && bn == BNV) return rl::launch_gemm<SW, BNV>(map_w, map_x, args, k_split, stream);
  RL_GEMM_CASE(false, 16) RL_GEMM_CASE(false, 32) RL_GEMM_CASE(false, 64) RL_GEMM_CASE(false, 128)
  RL_GEMM_CASE(false, 256) RL_GEMM_CASE(true, 16) RL_GEMM_CASE(true, 32) RL_GEMM_CASE(true, 64)
  RL_GEMM_CASE(true, 128)
#undef RL_GEMM_CASE
  return static_cast<int>(cudaErrorInvalidValue);
}

int rl_gemm_bf16(const void* x, const void* w, void* out, int tokens, int n_out, int k, int swiglu, int pdl,
                 int k_split, int* fault, cudaStream_t stream) {
  return rl_gemm_bf16_norm(x, w, out, tokens, n_out, k, swiglu, pdl, k_split, nullptr, nullptr, nullptr, nullptr, 0,
                           0.0f, 0, nullptr, fault, stream);
}

// columns of the table of partial sums of squares that a product of `n_out` output columns writes per token
int rl_gemm_bf16_sumsq_count(int n_out) { return 4 * ((n_out + rl::kTileN - 1) / rl::kTileN); }

}  // extern "C"

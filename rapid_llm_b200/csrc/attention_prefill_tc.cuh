// Prompt-portion (chunk) attention on the 5th-generation tensor cores.
//
// One CTA serves one work item: 256 packed query rows of one request (row p = token p / group,
// head p % group of one key/value head) against the request's cached keys, those of the
// portion itself included.  The rows form two tiles of 128; both use every key/value tile that
// TMA brings in (page by page, 128 keys a block, 128-byte swizzle), and while the softmax
// threads of one tile work, the tensor core works for the other:
//
//     S[row, key]  = Q[row, :] . K[key, :]      tcgen05.mma  M = 128, N = 128 keys, K = D
//     O[row, d]   += P[row, key] . V[key, d]    A = P from tensor memory, B = V as it lies in the
//                                               cache (MN-major), M = 128, N = D, K = 128 keys
//
// S and O live in tensor memory (2 x (128 + 128) columns).  A softmax thread owns one row —
// one lane of S and O — so the row maximum and sum need no exchange between threads: it reads
// its 128 scores into registers once (the softmax warpgroups take the registers the first
// warpgroup gives up), masks them (only blocks that touch the causal diagonal or the window's
// edge need it), exponentiates in base 2 and writes P as bfloat16 over the columns S occupied,
// where the next product reads it.  O is rescaled lazily: the reference
// point of the exponentials moves only when the row maximum has grown by more than 2^8, so most
// blocks leave the accumulator untouched; the final division by the row sum makes the result
// the same.  Scores, maxima, sums and the accumulator are float32; P is rounded to bfloat16
// before P.V, as in attention_mma.cu and the reference's tensor-core kernels.
//
// Needs head size 128, pages of 8, 16, 32, 64 or a multiple of 128 tokens and an unsplit key
// range; everything else takes the mma.sync tiles.
#pragma once

#include "tc_common.cuh"

namespace rl {
namespace RL_ATTENTION_NS {

constexpr int kPfD = 128;
constexpr int kPfKeys = 128;                    // keys per block
constexpr int kPfTileRows = 128;                // rows of one query tile
constexpr int kPfTiles = 2;                     // query tiles per CTA
constexpr int kPfRows = kPfTiles * kPfTileRows; // packed rows per work item
constexpr int kPfStages = 2;                    // key tiles and value tiles in flight, each
constexpr int kPfFirstSoftmaxWarp = 4;          // warp 0: TMA of keys, warp 1: TMA of values, warp 2: MMA, warp 3: idle
constexpr int kPfFewRegisters = 80;             // per thread of warps 0..3 once the kernel is set up
constexpr int kPfManyRegisters = 208;           // per softmax thread: a row of 128 scores stays in registers
constexpr int kPfThreads = kPfFirstSoftmaxWarp * 32 + kPfTiles * 128;
// The kernel starts with the registers its launch bounds allow every thread; what the softmax
// warpgroups take must have been given up by the first, or they would wait for ever.
constexpr int kPfLaunchRegisters = 65536 / kPfThreads / 8 * 8;
static_assert(kPfFirstSoftmaxWarp == 4 && kPfFewRegisters % 8 == 0 && kPfManyRegisters % 8 == 0 &&
              128 * kPfFewRegisters + kPfTiles * 128 * kPfManyRegisters <= kPfThreads * kPfLaunchRegisters,
              "register budgets of the warpgroups");
constexpr int kPfHalfBytes = 128 * 128;         // 128 rows of one 64-wide half
constexpr int kPfTileBytes = 2 * kPfHalfBytes;  // Q tile, K tile or V tile
constexpr int kPfSmemBytes = (kPfTiles + 2 * kPfStages) * kPfTileBytes + 1024;
constexpr int kPfStagedPages = 1024;
constexpr float kPfRescaleStep = 8.0f;          // the reference maximum follows only jumps of 2^8
constexpr uint32_t kPfIdescScore = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kPfIdescValue = kPfIdescScore | (1u << 16);     // B (the values) is MN-major

// Two float32 values in one 64-bit register and the instructions that work on both at once (sm_100): the
// softmax threads are bound by what a warp can issue, and these halve the scale-and-shift and the sums.
__device__ __forceinline__ unsigned long long pf_pack2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void pf_unpack2(unsigned long long v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long pf_fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long pf_add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float pf_max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

struct PrefillTcArgs {
  const bf16* q;
  bf16* out;
  const int* items;
  const int* cu_seqlens;
  const int* entry_start;
  const int* entry_slot;
  const int* block_table;
  int hq, hkv, page_size, num_pages, max_pages, slots, window;
  float scale_log2;
  int* fault;
};

__global__ void __launch_bounds__(kPfThreads, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_cache, const PrefillTcArgs args) {
  extern __shared__ unsigned char pf_smem_raw[];
  __shared__ __align__(8) uint64_t full_k[kPfStages], full_v[kPfStages], empty_k[kPfStages], empty_v[kPfStages];
  __shared__ __align__(8) uint64_t score_ready[kPfTiles], p_ready[kPfTiles], value_done[kPfTiles];
  __shared__ __align__(8) uint64_t q_ready, drained;
  __shared__ uint32_t tmem_slot;
  __shared__ int aborted_flag;
  __shared__ int staged_pages[kPfStagedPages];
  volatile int* aborted = &aborted_flag;

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t base = (smem_addr(pf_smem_raw) + 1023u) & ~1023u;
  auto q_tile = [&](int tile) { return base + tile * kPfTileBytes; };
  auto k_tile = [&](int s) { return base + (kPfTiles + s) * kPfTileBytes; };
  auto v_tile = [&](int s) { return base + (kPfTiles + kPfStages + s) * kPfTileBytes; };

  // ---- the item ------------------------------------------------------------------------
  // the kv head is the fast grid dimension: CTAs start in the order of the item list (longest
  // first) over all heads, so the last wave holds the shortest items
  const int* item = args.items + static_cast<size_t>(blockIdx.y) * 4;
  const int entry = item[0], row0 = item[1];
  const int kv_head = blockIdx.x;
  const int group = args.hq / args.hkv;
  const int tok_begin = args.cu_seqlens[entry];
  const int n_rows_entry = (args.cu_seqlens[entry + 1] - tok_begin) * group;
  const int n_rows = min(kPfRows, n_rows_entry - row0);
  const int start = args.entry_start[entry];
  const int slot = args.entry_slot[entry];
  const int last_row = row0 + n_rows - 1;
  const int min_pos = start + row0 / group, max_pos = start + last_row / group;
  const bool bad = slot < 0 || slot >= args.slots || start < 0 || n_rows <= 0 ||
                   max_pos >= args.max_pages * args.page_size;
  if (bad && tid == 0)
    atomicOr(args.fault, (slot < 0 || slot >= args.slots) ? kFaultSlot : kFaultPosition);
  const int hi = bad ? 0 : max_pos + 1;
  const int lo = args.window > 0 ? max(0, min_pos - args.window + 1) : 0;
  const int k_begin = lo & ~(kPfKeys - 1);
  const int n_blocks = hi > k_begin ? (hi - k_begin + kPfKeys - 1) / kPfKeys : 0;
  // blocks each tile needs: up to its last row's position
  int tile_blocks[kPfTiles];
#pragma unroll
  for (int tile = 0; tile < kPfTiles; ++tile) {
    const int rows_here = min(kPfTileRows, n_rows - tile * kPfTileRows);
    const int tile_last = row0 + tile * kPfTileRows + rows_here - 1;
    tile_blocks[tile] = rows_here > 0 && !bad ? (start + tile_last / group + 1 - k_begin + kPfKeys - 1) / kPfKeys : 0;
  }
  const int* table = args.block_table + static_cast<size_t>(bad ? 0 : slot) * args.max_pages;

  // ---- set-up --------------------------------------------------------------------------
  if (tid == 0) {
    for (int s = 0; s < kPfStages; ++s) {
      mbar_init(smem_addr(&full_k[s]), 1);
      mbar_init(smem_addr(&full_v[s]), 1);
      mbar_init(smem_addr(&empty_k[s]), 1);
      mbar_init(smem_addr(&empty_v[s]), 1);
    }
    for (int tile = 0; tile < kPfTiles; ++tile) {
      mbar_init(smem_addr(&score_ready[tile]), 1);
      mbar_init(smem_addr(&p_ready[tile]), 4);
      mbar_init(smem_addr(&value_done[tile]), 1);
    }
    mbar_init(smem_addr(&q_ready), 4 * kPfTiles);
    mbar_init(smem_addr(&drained), 1);
    aborted_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    tmem_alloc(smem_addr(&tmem_slot), 512);
    tmem_relinquish();
  }
  const int first_page = k_begin / args.page_size;
  const int page_count = n_blocks > 0 ? (hi - 1) / args.page_size - first_page + 1 : 0;
  const bool staged = page_count <= kPfStagedPages;
  if (staged) {
    for (int i = tid; i < page_count; i += kPfThreads) {
      int page = table[first_page + i];
      if (page < 0 || page >= args.num_pages) {
        atomicOr(args.fault, kFaultPageId);
        page = 0;
      }
      staged_pages[i] = page;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  auto tmem_score = [&](int tile) { return tmem_base + tile * 256; };        // 128 columns; P over its first 64
  auto tmem_out = [&](int tile) { return tmem_base + tile * 256 + 128; };    // 128 columns

  // the first warpgroup gives registers up (one instruction for all four warps), the softmax
  // warpgroups take them
  if (warp < kPfFirstSoftmaxWarp) {
    register_budget_down<kPfFewRegisters>();
    if (warp < 2) {
      // -------------------------------------------------------------------- TMA producers
      const int is_value = warp;
      uint64_t* fulls = is_value ? full_v : full_k;
      uint64_t* empties = is_value ? empty_v : empty_k;
      const int box_rows = min(args.page_size, kPfKeys);
      const int boxes = kPfKeys / box_rows;
      bool waited = false, ok = true;
      int issued = 0;
      for (int b = 0; b < n_blocks && ok; ++b) {
        const int stage = b % kPfStages;
        const int kb = k_begin + b * kPfKeys;
        if (b >= kPfStages) {
          int got = 1;
          if (lane == 0)
            got = mbar_wait(smem_addr(&empties[stage]), ((b / kPfStages) - 1) & 1, aborted, args.fault, is_value ? 1 << 9 : 1 << 8) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, got, 0) != 0;
          if (!ok) break;
        }
        // keys from `start` on are written by this step's earlier kernels
        if (!waited && kb + kPfKeys > start) {
          pdl_wait();
          waited = true;
        }
        if (lane == 0) mbar_expect_tx(smem_addr(&fulls[stage]), kPfTileBytes);
        __syncwarp();
        for (int i = lane; i < boxes * 2; i += 32) {
          const int x = i >> 1, half = i & 1;
          const int j = kb + x * box_rows;                   // first key of the box
          int page = 0, in_page = 0;                         // past the range: any readable page, masked later
          if (j < hi) {
            const int page_index = j / args.page_size;
            in_page = j - page_index * args.page_size;
            if (staged) {
              page = staged_pages[page_index - first_page];
            } else {
              page = table[page_index];
              if (page < 0 || page >= args.num_pages) {
                atomicOr(args.fault, kFaultPageId);
                page = 0;
              }
            }
          }
          const int row = ((page * 2 + is_value) * args.hkv + kv_head) * args.page_size + in_page;
          const uint32_t dst = (is_value ? v_tile(stage) : k_tile(stage)) + half * kPfHalfBytes + x * box_rows * 128;
          tma_load_2d(dst, &map_cache, smem_addr(&fulls[stage]), half * 64, row);
        }
        ++issued;
      }
      if (!waited) pdl_wait();
      if (lane == 0 && n_blocks > 0 && (!ok || *aborted)) {
        for (int s = 0; s < kPfStages; ++s) {
          const int fills = (issued - s + kPfStages - 1) / kPfStages;
          if (fills > 0) mbar_wait(smem_addr(&fulls[s]), (fills - 1) & 1, aborted, args.fault);
        }
      }
    } else if (warp == 2) {
      // -------------------------------------------------------------------- tensor-core issuer
      // Per block: the scores of both tiles as soon as the keys are there; then, tile by tile, the
      // values product once the tile's P is written, followed at once by the tile's next scores,
      // so that its softmax threads have work while the other tile's values are multiplied.
      // Products run in the order they are issued: the scores of block j + 1 overwrite the
      // columns that held P of block j only after the values product that read them.
      if (lane == 0) {
        bool ok = n_blocks > 0;
        if (ok) ok = mbar_wait(smem_addr(&q_ready), 0, aborted, args.fault, 1 << 10);
        auto issue_scores = [&](int tile, int b) {
          const int stage = b % kPfStages;
          const uint64_t q_desc = operand_desc(q_tile(tile)), keys_desc = operand_desc(k_tile(stage));
  #pragma unroll
          for (int k = 0; k < kPfD / 16; ++k) {
            const uint32_t half = (k >> 2), within = (k & 3) * 2;
            umma_bf16(tmem_score(tile), q_desc + half * (kPfHalfBytes >> 4) + within,
                      keys_desc + half * (kPfHalfBytes >> 4) + within, kPfIdescScore, k > 0 ? 1u : 0u);
          }
          umma_commit(smem_addr(&score_ready[tile]));
        };
        // the last tile that uses block b releases its key tile
        auto release_keys = [&](int b) { umma_commit(smem_addr(&empty_k[b % kPfStages])); };
        if (ok) {
          ok = mbar_wait(smem_addr(&full_k[0]), 0, aborted, args.fault, 1 << 11);
          if (ok) {
            tc_fence_after();
            for (int tile = 0; tile < kPfTiles; ++tile)
              if (tile_blocks[tile] > 0) issue_scores(tile, 0);
            release_keys(0);
          }
        }
        for (int b = 0; b < n_blocks && ok; ++b) {
          const int stage = b % kPfStages;
          bool keys_next = false;
          for (int tile = 0; tile < kPfTiles && ok; ++tile) {
            if (b >= tile_blocks[tile]) continue;
            ok = mbar_wait(smem_addr(&p_ready[tile]), b & 1, aborted, args.fault, 1 << (12 + tile));
            if (!ok) break;
            ok = mbar_wait(smem_addr(&full_v[stage]), (b / kPfStages) & 1, aborted, args.fault, 1 << 14);
            if (!ok) break;
            tc_fence_after();
            const uint64_t values_desc = operand_desc_mn(v_tile(stage), kPfHalfBytes);
  #pragma unroll
            for (int k = 0; k < kPfKeys / 16; ++k)
              umma_bf16_ts(tmem_out(tile), tmem_score(tile) + k * 8, values_desc + k * (2048 >> 4), kPfIdescValue,
                           (b > 0 || k > 0) ? 1u : 0u);
            umma_commit(smem_addr(&value_done[tile]));
            if (b + 1 < tile_blocks[tile]) {
              if (!keys_next) {
                ok = mbar_wait(smem_addr(&full_k[(b + 1) % kPfStages]), ((b + 1) / kPfStages) & 1, aborted, args.fault, 1 << 15);
                if (!ok) break;
                tc_fence_after();
                keys_next = true;
              }
              issue_scores(tile, b + 1);
            }
          }
          if (!ok) break;
          umma_commit(smem_addr(&empty_v[stage]));
          if (keys_next) release_keys(b + 1);
        }
        umma_commit(smem_addr(&drained));
        mbar_wait(smem_addr(&drained), 0, aborted, args.fault, 1 << 16);
      }
    }
  } else {
    // -------------------------------------------------------------------- softmax and output
    register_budget_up<kPfManyRegisters>();
    const int tile = (warp - kPfFirstSoftmaxWarp) >> 2;
    const int quarter = warp & 3;                      // tensor-memory lanes this warp may touch
    const int r = quarter * 32 + lane;                 // row of the tile = lane of S and O
    const uint32_t lane_bits = static_cast<uint32_t>(quarter * 32) << 16;
    const int p = row0 + tile * kPfTileRows + r;       // packed row of the request
    const bool valid = p < row0 + n_rows && !bad;
    const int token = p / group;
    const int pos = valid ? start + token : -1;        // -1: a row that sees no key
    const int lo_pos = args.window > 0 ? max(0, pos - args.window + 1) : 0;
    pdl_wait();                                        // queries come from the kernel before
    {
      // The warp's 32 rows of Q, 256 bytes each, into the K-major operand [row][64] x 2 halves, swizzled: an
      // instruction fetches two whole rows (a lane 16 bytes, past L1, which the lists and page ids keep), and all
      // of a lane's fetches fly together.
      const int shift = (group & (group - 1)) == 0 ? 31 - __clz(group) : -1;
      uint4 fetched[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int rr = quarter * 32 + 2 * i + (lane >> 4);
        const int pp = row0 + tile * kPfTileRows + rr;
        const int tt = shift >= 0 ? pp >> shift : pp / group;
        fetched[i] = make_uint4(0, 0, 0, 0);
        if (pp < row0 + n_rows && !bad)
          fetched[i] = __ldcg(reinterpret_cast<const uint4*>(
              args.q + (static_cast<size_t>(tok_begin + tt) * args.hq + kv_head * group + (pp - tt * group)) * kPfD + (lane & 15) * 8));
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int rr = quarter * 32 + 2 * i + (lane >> 4), c = lane & 15;
        const uint32_t dst = q_tile(tile) + (c >> 3) * kPfHalfBytes + rr * 128 + (((c & 7) ^ (rr & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(fetched[i].x), "r"(fetched[i].y), "r"(fetched[i].z), "r"(fetched[i].w) : "memory");
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&q_ready));
    }

    const int my_blocks = tile_blocks[tile];
    float ref_max = -INFINITY;                         // exponentials are taken against ref_max
    unsigned long long row_sum2 = pf_pack2(0.0f, 0.0f);   // the row's sum as two halves (even and odd keys)
    bool ok = true;
    for (int b = 0; b < my_blocks && ok; ++b) {
      const int kb = k_begin + b * kPfKeys;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_addr(&score_ready[tile]), b & 1, aborted, args.fault, 1 << (17 + tile)));
      if (!ok) break;
      tc_fence_after();
      const bool masked = kb + kPfKeys - 1 > pos || kb < lo_pos;
      // the row's 128 scores come into registers once; keys the row may not see become -inf,
      // whose exponential is zero
      uint32_t score[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_load32(tmem_score(tile) + lane_bits + c * 32, score[c]);
      tmem_wait_ld();
      if (masked) {
#pragma unroll
        for (int i = 0; i < kPfKeys; ++i) {
          const int key = kb + i;
          if (!(key <= pos && key >= lo_pos)) score[i >> 5][i & 31] = 0xff800000u;
        }
      }
      // eight running maxima, two new scores a comparison: one chain of dependent comparisons would cost their
      // latencies in a row
      float lane_max[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) lane_max[i] = __uint_as_float(score[0][i]);
#pragma unroll
      for (int i = 8; i + 16 <= kPfKeys; i += 16) {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          lane_max[c] = pf_max3(lane_max[c], __uint_as_float(score[(i + c) >> 5][(i + c) & 31]),
                                __uint_as_float(score[(i + c + 8) >> 5][(i + c + 8) & 31]));
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) lane_max[c] = fmaxf(lane_max[c], __uint_as_float(score[3][24 + c]));
      float block_max = fmaxf(fmaxf(fmaxf(lane_max[0], lane_max[1]), fmaxf(lane_max[2], lane_max[3])),
                              fmaxf(fmaxf(lane_max[4], lane_max[5]), fmaxf(lane_max[6], lane_max[7])));
      block_max *= args.scale_log2;                    // the scale is positive
      // The values product of the block before has added to O by now: products run in order, this
      // block's scores were issued after it, and the barrier that announced them counts everything
      // the issuing thread had issued before.  So O may be rescaled here without a further wait.
      // tensor-memory accesses are warp-wide: if any row of the warp moves its reference point,
      // the whole warp rewrites its rows of O, the others with a factor of one
      const bool moves = block_max > ref_max + kPfRescaleStep || (ref_max == -INFINITY && block_max > -INFINITY);
      float alpha = 1.0f;
      if (moves) {
        alpha = ref_max == -INFINITY ? 0.0f : fast_exp2(ref_max - block_max);
        ref_max = block_max;
        float even, odd;
        pf_unpack2(row_sum2, even, odd);
        row_sum2 = pf_pack2(even * alpha, odd * alpha);
      }
      if (b > 0 && __any_sync(0xffffffffu, moves)) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t raw[32];
          tmem_load32(tmem_out(tile) + lane_bits + c * 32, raw);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
          tmem_store32(tmem_out(tile) + lane_bits + c * 32, raw);
        }
      }
      const float shift = ref_max == -INFINITY ? 0.0f : ref_max;
      // P = 2^(s * scale - ref_max) as bfloat16, two per column, over S's columns; scale-and-shift and the sum
      // work on two keys an instruction
      const unsigned long long scale2 = pf_pack2(args.scale_log2, args.scale_log2), shift2 = pf_pack2(-shift, -shift);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x0, x1;
          pf_unpack2(pf_fma2(pf_pack2(__uint_as_float(score[c][2 * i]), __uint_as_float(score[c][2 * i + 1])), scale2, shift2), x0, x1);
          const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
          row_sum2 = pf_add2(row_sum2, pf_pack2(e0, e1));
          const __nv_bfloat162 pair = __floats2bfloat162_rn(e0, e1);
          packed[i] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        tmem_store16(tmem_score(tile) + lane_bits + c * 16, packed);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&p_ready[tile]));
    }
    // the output: O / sum, one row of 128 per thread (every lane reads its row of tensor memory,
    // the rows that exist are stored)
    if (ok && my_blocks > 0) ok = mbar_wait(smem_addr(&value_done[tile]), (my_blocks - 1) & 1, aborted, args.fault, 1 << (21 + tile));
    const bool all_ok = __all_sync(0xffffffffu, ok);
    bf16* dst = args.out + (static_cast<size_t>(tok_begin + token) * args.hq + kv_head * group + (p - token * group)) * kPfD;
    if (all_ok && my_blocks > 0) {
      tc_fence_after();
      float even, odd;
      pf_unpack2(row_sum2, even, odd);
      const float row_sum = even + odd;
      const float inv = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        tmem_load32(tmem_out(tile) + lane_bits + c * 32, raw);
        tmem_wait_ld();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 value;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&value);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              h[e] = __floats2bfloat162_rn(__uint_as_float(raw[i * 8 + 2 * e]) * inv, __uint_as_float(raw[i * 8 + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = value;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace RL_ATTENTION_NS
}  // namespace rl

// Decode attention on the 5th-generation tensor cores: few query rows against many cached keys.
//
// One CTA serves one work item: the (up to 16) packed query rows of one request — its new
// token's heads of one key/value head group — against one part of the request's key range.
// A decode step is a pure stream of the cache, so the kernel is built to keep that stream
// running and to spend almost no instructions per key:
//
//   * keys and values come page by page through TMA into 128-byte-swizzled tiles of 128 keys,
//     a ring of stages ahead of the math; one thread issues them.  The block table was
//     uploaded before the step, and pages below the request's first new position were written
//     by earlier steps, so these copies start before the kernel waits for its predecessor.
//   * the products run transposed, so that the 128 keys of a block fill the 128 rows of the
//     instruction and the query rows are its narrow side:
//         S^T[key, row] = K[key, :] . Q[row, :]        (tcgen05.mma, M = 128, N = 16, K = D)
//         O^T[d, row]  += V[key, d] . P^T[key, row]    (M = D, N = 16, K = 128 keys; V is read
//                                                        as it lies in the cache, "MN-major")
//     with accumulators in tensor memory.
//   * 128 softmax threads own one key each (one lane of S^T): they scale, mask, take the block
//     maximum of every row over lanes and warps, exponentiate in base 2, write P^T as the next
//     product's operand and keep the running sum; the same threads own one output dimension
//     each (one lane of O^T) and accumulate O in registers, rescaled by the change of the
//     running maximum.  Per key this is a few instructions per thread.  Two such teams take the
//     even and the odd blocks, each with a softmax state of its own, merged at the end: the
//     softmax is a chain of dependent instructions, and two chains fill the SM where one leaves
//     it idle.
//   * when the key range of a request is split over several CTAs and the step holds nothing but
//     decode tiles, those CTAs form a thread-block cluster and merge their partial results
//     through distributed shared memory, in rank order: no scratch in global memory and no
//     second kernel.
//
// Semantics are those of attention_mma.cu (scores, running maximum and sum and the output
// accumulator in float32; P rounded to bfloat16 before P.V).  Needs head size 128 and pages of
// 8, 16, 32, 64 or a multiple of 128 tokens; everything else takes the mma.sync kernel.
#pragma once

#include "tc_common.cuh"

namespace rl {
namespace RL_ATTENTION_NS {

constexpr int kTcD = 128;
constexpr int kTcKeys = 128;                    // keys per block = M of the score product
constexpr int kTcRows = 16;                     // packed query rows per item = N of both products
constexpr int kTcMaxStages = 3;                 // tiles of keys (and of values) in flight ahead of the math, per CTA
constexpr int kTcTeams = 2;
constexpr int kTcProducerWarps = 4;             // warps 0, 1: TMA of keys, warps 2, 3: TMA of values
constexpr int kTcIssuerWarp = kTcProducerWarps;  // then one warp that issues the products
constexpr int kTcFirstSoftmaxWarp = kTcIssuerWarp + 1;
constexpr int kTcThreads = kTcFirstSoftmaxWarp * 32 + kTcTeams * 128;   // then four softmax warps per team
constexpr int kTcTmemColumns = 128;             // per team: two score and two value buffers of 16 columns
constexpr int kTcStagedPages = 512;
constexpr int kTcHalfBytes = kTcKeys * 128;     // one 64-wide half of a 128-key tile
constexpr int kTcTileBytes = 2 * kTcHalfBytes;  // K or V of one block
constexpr int kTcStageBytes = 2 * kTcTileBytes;
constexpr int kTcOperandBytes = 2 * kTcRows * 128;   // Q or P^T: 16 rows, two 64-wide halves
// Shared memory of a CTA with rings of `stages` key tiles and `stages` value tiles.  Three stages take a whole
// multiprocessor: one CTA streams by itself.  With one stage two CTAs fit a multiprocessor, and while one of
// them sets itself up for its item (page ids, queries, first tiles: a quarter of a short item's time) the other
// streams; a step with more items than multiprocessors runs faster that way.
constexpr int tc_smem_bytes(int stages) { return stages * kTcStageBytes + (1 + 2 * kTcTeams) * kTcOperandBytes + 1024; }
constexpr uint32_t kTcIdescScore = (1u << 4) | (1u << 7) | (1u << 10) | ((kTcRows >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kTcIdescValue = kTcIdescScore | (1u << 15);     // A (the values) is MN-major

constexpr int kTcMaxClusterSplits = 16;     // key ranges of a tile merged inside one cluster (more than 8: a cluster size that must be asked for)

struct DecodeTcArgs {
  const bf16* q;
  bf16* out;
  float* part_out;
  float* part_lse;
  const int* items;
  const int* cu_seqlens;
  const int* entry_start;
  const int* entry_slot;
  const int* block_table;
  int hq, hkv, page_size, num_pages, max_pages, slots, window, splits;
  int cluster_merge;        // the CTAs of an item's splits are one cluster and merge among themselves
  float scale_log2;
  int* fault;
};

// Largest value over the warp's lanes in one instruction.
__device__ __forceinline__ float warp_max_redux(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}

// kRows: how many of the 16 columns of the products carry query rows (a power of two); the
// per-row work of the softmax threads is unrolled over exactly these.
template <int kRows, int kTcStages>
__global__ void __launch_bounds__(kTcThreads, kTcStages == 1 ? 2 : 1)
attention_decode_tc_kernel(const __grid_constant__ CUtensorMap map_cache, const DecodeTcArgs args) {
  static_assert(kRows >= 1 && kRows <= kTcRows && (kRows & (kRows - 1)) == 0, "rows: a power of two up to 16");
  static_assert(kTcStages >= 1 && kTcStages <= kTcMaxStages, "stages");
  extern __shared__ unsigned char tc_smem_raw[];
  __shared__ __align__(8) uint64_t full_k[kTcStages], full_v[kTcStages], empty_k[kTcStages], empty_v[kTcStages];
  __shared__ __align__(8) uint64_t score_ready[kTcTeams][2], p_ready[kTcTeams][2], value_ready[kTcTeams][2];
  __shared__ __align__(8) uint64_t q_ready, drained;
  __shared__ uint32_t tmem_slot;
  __shared__ int aborted_flag;
  __shared__ int staged_pages[kTcStagedPages];
  __shared__ float block_maxes[kTcTeams][2][4][kTcRows];
  __shared__ float block_sums[kTcTeams][4][kTcRows];
  __shared__ float team_max[kTcRows], split_lse[kTcRows];
  __shared__ int row_pos[kTcRows], row_lo[kTcRows];
  volatile int* aborted = &aborted_flag;

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t base = (smem_addr(tc_smem_raw) + 1023u) & ~1023u;
  auto k_tile = [&](int s) { return base + s * kTcStageBytes; };
  auto v_tile = [&](int s) { return base + s * kTcStageBytes + kTcTileBytes; };
  const uint32_t q_tile = base + kTcStages * kTcStageBytes;
  auto p_tile = [&](int team, int b) { return q_tile + (1 + team * 2 + b) * kTcOperandBytes; };

  // ---- the item ------------------------------------------------------------------------
  const int* item = args.items + (static_cast<size_t>(blockIdx.z) * gridDim.x + blockIdx.x) * 4;
  const int entry = item[0], row0 = item[1], split = item[2];
  const int kv_head = blockIdx.y;
  const int group = args.hq / args.hkv;
  const int tok_begin = args.cu_seqlens[entry];
  const int n_rows_entry = (args.cu_seqlens[entry + 1] - tok_begin) * group;
  const int n_rows = min(kRows, n_rows_entry - row0);
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
  const int lo_aligned = lo & ~(kTcKeys - 1);
  const int span = max(hi - lo_aligned, 0);
  const int per_split = ((span + args.splits - 1) / args.splits + kTcKeys - 1) / kTcKeys * kTcKeys;
  const int k_begin = lo_aligned + split * per_split;
  const int k_end = min(hi, k_begin + per_split);
  const int n_blocks = k_end > k_begin ? (k_end - k_begin + kTcKeys - 1) / kTcKeys : 0;
  const int* table = args.block_table + static_cast<size_t>(bad ? 0 : slot) * args.max_pages;

  // ---- set-up --------------------------------------------------------------------------
  if (tid == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(smem_addr(&full_k[s]), 2);          // one arrival per producer warp of the tile
      mbar_init(smem_addr(&full_v[s]), 2);
      mbar_init(smem_addr(&empty_k[s]), 1);
      mbar_init(smem_addr(&empty_v[s]), 1);
    }
    for (int team = 0; team < kTcTeams; ++team) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(smem_addr(&score_ready[team][b]), 1);
        mbar_init(smem_addr(&p_ready[team][b]), 4);
        mbar_init(smem_addr(&value_ready[team][b]), 1);
      }
    }
    mbar_init(smem_addr(&q_ready), 4);
    mbar_init(smem_addr(&drained), 1);
    aborted_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kTcIssuerWarp) {
    tmem_alloc(smem_addr(&tmem_slot), kTcTmemColumns);
    tmem_relinquish();
  }
  if (tid < kTcRows) {
    const int p = row0 + tid;
    const int pos = tid < n_rows ? start + p / group : -1;       // -1: a row that sees no key
    row_pos[tid] = pos;
    row_lo[tid] = args.window > 0 ? max(0, pos - args.window + 1) : 0;
  }
  // the page ids of this item's key range (the block table is complete before the step starts)
  const int first_page = k_begin / args.page_size;
  const int page_count = n_blocks > 0 ? (k_end - 1) / args.page_size - first_page + 1 : 0;
  const bool staged = page_count <= kTcStagedPages;
  if (staged) {
    for (int i = tid; i < page_count; i += kTcThreads) {
      int page = table[first_page + i];
      if (page < 0 || page >= args.num_pages) {
        atomicOr(args.fault, kFaultPageId);
        page = 0;                                 // the null page: readable, and masked or wrong-but-flagged
      }
      staged_pages[i] = page;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  // tensor-memory columns of team `team`, buffer `buf`: scores, then values
  auto tmem_score = [&](int team, int buf) { return tmem_base + (team * 4 + buf) * kTcRows; };
  auto tmem_value = [&](int team, int buf) { return tmem_base + (team * 4 + 2 + buf) * kTcRows; };

  if (warp < kTcProducerWarps) {
    // -------------------------------------------------------------------- TMA producers
    // Two warps bring the key tiles and two the value tiles, through a ring each: a key tile is
    // free again as soon as its scores are computed, long before the values of the same block
    // are used, so the key copies run several blocks ahead of the softmax.  One box is the part
    // of one page that lies in the block (page_size, at most 128, keys by 64 elements).  A
    // thread issues its copies one after the other, so a tile's boxes are dealt over the lanes
    // of two warps; lane 0 of each posts its share of the byte count.
    const int is_value = warp >> 1, share = warp & 1;
    uint64_t* fulls = is_value ? full_v : full_k;
    uint64_t* empties = is_value ? empty_v : empty_k;
    const int box_rows = min(args.page_size, kTcKeys);
    const int boxes = kTcKeys / box_rows;
    const uint64_t read_once = l2_evict_first_policy();   // a decode step reads every key and value once
    bool waited = false, ok = true;
    int issued = 0;
    for (int b = 0; b < n_blocks && ok; ++b) {
      const int stage = b % kTcStages;
      const int kb = k_begin + b * kTcKeys;
      if (b >= kTcStages) {
        int got = 1;
        if (lane == 0)
          got = mbar_wait(smem_addr(&empties[stage]), ((b / kTcStages) - 1) & 1, aborted, args.fault) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, got, 0) != 0;
        if (!ok) break;
      }
      // keys from `start` on are written by this step's earlier kernels
      if (!waited && kb + kTcKeys > start) {
        pdl_wait();
        waited = true;
      }
      if (lane == 0) mbar_expect_tx(smem_addr(&fulls[stage]), kTcTileBytes / 2);
      __syncwarp();
      // this warp's half of the tile's boxes: with one box per half-row of pages, the other
      // warp takes the other 64 elements
      for (int i = 2 * lane + share; i < boxes * 2; i += 64) {
        const int x = i >> 1, half = i & 1;
        const int j = kb + x * box_rows;                   // first key of the box
        int page = 0, in_page = 0;                         // past the range: any readable page, masked later
        if (j < k_end) {
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
        const uint32_t dst = (is_value ? v_tile(stage) : k_tile(stage)) + half * kTcHalfBytes + x * box_rows * 128;
        tma_load_2d_hint(dst, &map_cache, smem_addr(&fulls[stage]), half * 64, row, read_once);
      }
      ++issued;
    }
    if (!waited) pdl_wait();
    if (lane == 0 && n_blocks > 0 && (!ok || *aborted)) {
      // copies in flight must land before the CTA may exit
      for (int s = 0; s < kTcStages; ++s) {
        const int fills = (issued - s + kTcStages - 1) / kTcStages;
        if (fills > 0) mbar_wait(smem_addr(&fulls[s]), (fills - 1) & 1, aborted, args.fault);
      }
    }
  } else if (warp == kTcIssuerWarp) {
    // -------------------------------------------------------------------- tensor-core issuer
    // Block b belongs to team b % 2 as that team's block b / 2; a team has two score and two
    // value buffers.  Scores are issued as soon as their keys have arrived and their buffer is
    // free (the block four before has been through its softmax), values as soon as P^T and the
    // value tile are there: the thread looks at both in turn, so neither waits behind the other.
    if (lane == 0) {
      bool ok = n_blocks > 0;
      if (ok) ok = mbar_wait(smem_addr(&q_ready), 0, aborted, args.fault);
      const uint64_t q_desc = operand_desc(q_tile);
      int next_s = 0, next_pv = 0;
      uint32_t idle = 0;
      while (ok && next_pv < n_blocks) {
        bool progressed = false;
        if (next_s < n_blocks && next_s < next_pv + 4 &&
            mbar_test(smem_addr(&full_k[next_s % kTcStages]), (next_s / kTcStages) & 1)) {
          const int stage = next_s % kTcStages, team = next_s & 1, buf = (next_s >> 1) & 1;
          tc_fence_after();
          const uint64_t keys_desc = operand_desc(k_tile(stage));
#pragma unroll
          for (int k = 0; k < kTcD / 16; ++k) {
            // descriptors count addresses in units of 16 bytes: 32 bytes further along a row = +2
            const uint32_t half = (k >> 2), within = (k & 3) * 2;
            umma_bf16(tmem_score(team, buf), keys_desc + half * (kTcHalfBytes >> 4) + within,
                      q_desc + half * (kTcRows * 128 >> 4) + within, kTcIdescScore, k > 0 ? 1u : 0u);
          }
          umma_commit(smem_addr(&score_ready[team][buf]));
          umma_commit(smem_addr(&empty_k[stage]));
          ++next_s;
          progressed = true;
        }
        if (next_pv < next_s) {
          const int stage = next_pv % kTcStages, team = next_pv & 1, buf = (next_pv >> 1) & 1;
          if (mbar_test(smem_addr(&p_ready[team][buf]), (next_pv >> 2) & 1) &&
              mbar_test(smem_addr(&full_v[stage]), (next_pv / kTcStages) & 1)) {
            tc_fence_after();
            const uint64_t values_desc = operand_desc_mn(v_tile(stage), kTcHalfBytes);
            const uint64_t p_desc = operand_desc(p_tile(team, buf));
#pragma unroll
            for (int k = 0; k < kTcKeys / 16; ++k) {
              // 16 keys further: two groups of eight 128-byte rows in the value tile, 32 bytes in P^T
              const uint32_t half = (k >> 2), within = (k & 3) * 2;
              umma_bf16(tmem_value(team, buf), values_desc + k * (2048 >> 4),
                        p_desc + half * (kTcRows * 128 >> 4) + within, kTcIdescValue, k > 0 ? 1u : 0u);
            }
            umma_commit(smem_addr(&value_ready[team][buf]));
            umma_commit(smem_addr(&empty_v[stage]));
            ++next_pv;
            progressed = true;
          }
        }
        if (progressed) {
          idle = 0;
        } else {
          __nanosleep(32);                        // leave the issue slots to the softmax warps
          if (++idle > (kSpinLimit >> 4) || ((idle & 255u) == 0 && *aborted)) {
            if (idle > (kSpinLimit >> 4)) {
              *aborted = 1;
              atomicOr(args.fault, kFaultWaitLimit);
            }
            ok = false;
          }
        }
      }
      umma_commit(smem_addr(&drained));
      mbar_wait(smem_addr(&drained), 0, aborted, args.fault);
    }
  }

  // ---------------------------------------------------------------------- softmax and output
  const bool softmax_warp = warp >= kTcFirstSoftmaxWarp;
  const int team = softmax_warp ? (warp - kTcFirstSoftmaxWarp) >> 2 : 0;
  const int quarter = warp & 3;                      // tensor-memory lanes this warp may touch
  const int t = quarter * 32 + lane;                 // key of a block / output dimension
  const uint32_t lane_bits = static_cast<uint32_t>(quarter * 32) << 16;
  float run_max[kRows], run_sum[kRows], out_acc[kRows];
#pragma unroll
  for (int n = 0; n < kRows; ++n) {
    run_max[n] = -INFINITY;
    run_sum[n] = 0.0f;
    out_acc[n] = 0.0f;
  }
  if (softmax_warp) {
    pdl_wait();                                        // queries come from the kernel before
    if (team == 0) {
      // Q: 16 rows of 128, as the K-major operand [row][64] x 2 halves with the 128-byte swizzle
      for (int idx = t; idx < kTcRows * 16; idx += 128) {
        const int r = idx >> 4, c = idx & 15;
        uint4 value = make_uint4(0, 0, 0, 0);
        if (r < n_rows && !bad) {
          const int p = row0 + r, token = p / group;
          value = *reinterpret_cast<const uint4*>(
              args.q + (static_cast<size_t>(tok_begin + token) * args.hq + kv_head * group + (p - token * group)) * kTcD + c * 8);
        }
        const uint32_t dst = q_tile + (c >> 3) * (kTcRows * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(value.x), "r"(value.y), "r"(value.z), "r"(value.w) : "memory");
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&q_ready));
    }

    float prev_alpha[kRows];
    int pos_of[kRows], lo_of[kRows];
#pragma unroll
    for (int n = 0; n < kRows; ++n) {
      pos_of[n] = row_pos[n];
      lo_of[n] = row_lo[n];
      prev_alpha[n] = 1.0f;
    }
    auto take_values = [&](int i) {
      // O += P.V of the team's block i, which was computed against the maximum after that block
      const int buf = i & 1;
      if (!mbar_wait(smem_addr(&value_ready[team][buf]), (i >> 1) & 1, aborted, args.fault)) return;
      tc_fence_after();
      float v[kTcRows];
      tmem_load16(tmem_value(team, buf) + lane_bits, v);
#pragma unroll
      for (int n = 0; n < kRows; ++n) out_acc[n] = out_acc[n] * prev_alpha[n] + v[n];
    };
    const int my_blocks = (n_blocks - team + 1) / 2;       // blocks team, team + 2, ...
    const uint32_t p_half = t >> 6, p_chunk = (t & 63) >> 3, p_elem = t & 7;
    for (int i = 0; i < my_blocks; ++i) {
      const int buf = i & 1;
      const int key = k_begin + (2 * i + team) * kTcKeys + t;
      // a wait that ran out sets the CTA's abort flag; the team's 128 threads leave together
      // after the barrier below, which every one of them reaches
      const bool got = mbar_wait(smem_addr(&score_ready[team][buf]), (i >> 1) & 1, aborted, args.fault);
      float s[kTcRows];
      if (got) {
        tc_fence_after();
        tmem_load16(tmem_score(team, buf) + lane_bits, s);
      } else {
#pragma unroll
        for (int n = 0; n < kTcRows; ++n) s[n] = 0.0f;
      }
      const bool in_range = key < k_end;
#pragma unroll
      for (int n = 0; n < kRows; ++n) {
        const bool keep = in_range && key <= pos_of[n] && key >= lo_of[n];
        s[n] = keep ? s[n] * args.scale_log2 : -INFINITY;
        const float m = warp_max_redux(s[n]);
        if (lane == 0) block_maxes[team][buf][quarter][n] = m;
      }
      named_barrier(1 + team, 128);
      if (*aborted) break;
      float alpha[kRows], block_max[kRows];
#pragma unroll
      for (int n = 0; n < kRows; ++n)
        block_max[n] = fmaxf(fmaxf(block_maxes[team][buf][0][n], block_maxes[team][buf][1][n]),
                             fmaxf(block_maxes[team][buf][2][n], block_maxes[team][buf][3][n]));
      unsigned short bits[kRows];
#pragma unroll
      for (int n = 0; n < kRows; ++n) {
        const float new_max = fmaxf(run_max[n], block_max[n]);
        const float safe = new_max == -INFINITY ? 0.0f : new_max;
        alpha[n] = fast_exp2(run_max[n] - safe);      // 0 while nothing was seen
        run_max[n] = new_max;
        const float p = fast_exp2(s[n] - safe);
        run_sum[n] = run_sum[n] * alpha[n] + p;
        bits[n] = __bfloat16_as_ushort(__float2bfloat16_rn(p));
      }
      // P^T as the next product's K-major operand: [row][64 keys] x 2 halves, swizzled.  Rows
      // beyond kRows keep whatever they held: a column of the product only reads its own row
      // of P^T, and those columns are never looked at.
      const uint32_t mine = p_tile(team, buf) + p_half * (kTcRows * 128) + p_elem * 2;
#pragma unroll
      for (int n = 0; n < kRows; ++n)
        asm volatile("st.shared.b16 [%0], %1;" ::"r"(mine + n * 128 + ((p_chunk ^ (n & 7)) << 4)), "h"(bits[n]));
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&p_ready[team][buf]));
      // meanwhile: the values of the team's block before
      if (i > 0) take_values(i - 1);                // a failure shows in the abort flag at the next barrier
#pragma unroll
      for (int n = 0; n < kRows; ++n) prev_alpha[n] = alpha[n];
    }
    if (!*aborted && my_blocks > 0) take_values(my_blocks - 1);
    // row sums over the team's 128 threads
#pragma unroll
    for (int n = 0; n < kRows; ++n) {
      const float total = warp_sum(run_sum[n]);
      if (lane == 0) block_sums[team][quarter][n] = total;
    }
  }

  // every product has retired and every copy has landed: the stages are free to hold the merges
  tc_fence_before();
  __syncthreads();
  float* exchange = reinterpret_cast<float*>(tc_smem_raw + (base - smem_addr(tc_smem_raw)));   // [16][128]
  float* split_out = exchange + kTcRows * 128;                                                  // [16][128]
  const bool healthy = !*aborted;
  if (softmax_warp && team == 1 && healthy) {
#pragma unroll
    for (int n = 0; n < kRows; ++n) {
      exchange[n * 128 + t] = out_acc[n];
      if (t == 0) team_max[n] = run_max[n];
    }
  }
  __syncthreads();
  if (softmax_warp && team == 0 && healthy) {
#pragma unroll
    for (int n = 0; n < kRows; ++n) {
      if (n >= n_rows) continue;
      const float sum0 = block_sums[0][0][n] + block_sums[0][1][n] + block_sums[0][2][n] + block_sums[0][3][n];
      const float sum1 = block_sums[1][0][n] + block_sums[1][1][n] + block_sums[1][2][n] + block_sums[1][3][n];
      const float max1 = team_max[n];
      const float m = fmaxf(run_max[n], max1);
      const float safe = m == -INFINITY ? 0.0f : m;
      const float w0 = fast_exp2(run_max[n] - safe), w1 = fast_exp2(max1 - safe);
      const float total = sum0 * w0 + sum1 * w1;
      const float value = out_acc[n] * w0 + exchange[n * 128 + t] * w1;
      const float inv = total > 0.0f ? 1.0f / total : 0.0f;
      const float lse = total > 0.0f ? m + log2f(total) : -INFINITY;
      const float merged = value * inv;
      const int p = row0 + n, token = p / group;
      const size_t row = static_cast<size_t>(tok_begin + token) * args.hq + kv_head * group + (p - token * group);
      if (args.splits == 1) {
        args.out[row * kTcD + t] = __float2bfloat16_rn(merged);
      } else if (args.cluster_merge) {
        split_out[n * 128 + t] = merged;
        if (t == 0) split_lse[n] = lse;
      } else {
        args.part_out[(row * args.splits + split) * kTcD + t] = merged;
        if (t == 0) args.part_lse[row * args.splits + split] = lse;
      }
    }
  }

  if (args.cluster_merge && args.splits > 1) {
    // the splits of this item are the ranks of one cluster: rank r merges rows r, r + splits, ...
    __syncwarp();
    cluster_sync();
    if (softmax_warp && team == 0) {
      // where the other ranks keep their row statistics and this thread's column of their results
      uint32_t peer_lse[kTcMaxClusterSplits], peer_out[kTcMaxClusterSplits];
      const bool wide = args.splits > 8;               // clusters of more than eight CTAs: the second half of the ranks
#pragma unroll
      for (int r = 0; r < kTcMaxClusterSplits; ++r) {
        peer_lse[r] = r < args.splits ? peer_smem(smem_addr(&split_lse[0]), r) : 0u;
        peer_out[r] = r < args.splits ? peer_smem(smem_addr(&split_out[t]), r) : 0u;
      }
      for (int n = split; n < n_rows; n += args.splits) {
        // all remote loads of the row first (each takes hundreds of cycles), the arithmetic after
        float lse_of[kTcMaxClusterSplits], out_of[kTcMaxClusterSplits];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          lse_of[r] = r < args.splits ? load_peer_f32(peer_lse[r] + n * 4) : -INFINITY;
          out_of[r] = r < args.splits ? load_peer_f32(peer_out[r] + n * 128 * 4) : 0.0f;
        }
#pragma unroll
        for (int r = 8; r < kTcMaxClusterSplits; ++r) {
          lse_of[r] = -INFINITY;
          out_of[r] = 0.0f;
        }
        if (wide) {
#pragma unroll
          for (int r = 8; r < kTcMaxClusterSplits; ++r) {
            if (r < args.splits) {
              lse_of[r] = load_peer_f32(peer_lse[r] + n * 4);
              out_of[r] = load_peer_f32(peer_out[r] + n * 128 * 4);
            }
          }
        }
        float m = -INFINITY;
#pragma unroll
        for (int r = 0; r < 8; ++r) m = fmaxf(m, lse_of[r]);
        if (wide) {
#pragma unroll
          for (int r = 8; r < kTcMaxClusterSplits; ++r) m = fmaxf(m, lse_of[r]);
        }
        const float safe = m == -INFINITY ? 0.0f : m;
        float total = 0.0f, value = 0.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (r < args.splits) {
            const float w = fast_exp2(lse_of[r] - safe);
            total += w;
            value += w * out_of[r];
          }
        }
        if (wide) {
#pragma unroll
          for (int r = 8; r < kTcMaxClusterSplits; ++r) {
            if (r < args.splits) {
              const float w = fast_exp2(lse_of[r] - safe);
              total += w;
              value += w * out_of[r];
            }
          }
        }
        const int p = row0 + n, token = p / group;
        const size_t row = static_cast<size_t>(tok_begin + token) * args.hq + kv_head * group + (p - token * group);
        args.out[row * kTcD + t] = __float2bfloat16_rn(total > 0.0f ? value / total : 0.0f);
      }
    }
    __syncwarp();
    cluster_sync();   // nobody leaves while its shared memory may still be read
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kTcIssuerWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTcTmemColumns);
  }
}

}  // namespace RL_ATTENTION_NS
}  // namespace rl

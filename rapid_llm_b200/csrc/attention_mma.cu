// Paged causal attention on the bfloat16 tensor cores, for one head size per build
// (compile with -DRL_HEAD_DIM=<multiple of 16 up to 256>; the Python side builds the
// library a model's head size needs at its first use).
//
// One step's batch holds portions of prompts beside single decoded tokens.  The host cuts
// it into work items, one CTA each: (request, first packed row of a query tile, part of
// the key range).  The query heads that share a key/value head are packed into the rows
// of one tile (row p of a request = token p / group, head p % group), so keys and values
// are read once per key/value head.  Two tile shapes share one code path:
//   * chunk tiles: 64 rows, four warps of 16 rows each, every warp walks all keys;
//   * decode tiles: 16 rows (one token's head group), four warps split each block of 64
//     keys between them and merge their running softmax states in shared memory.
// Keys and values come from the cache through the request's block table with cp.async,
// three (decode) or two (chunk) blocks of 64 keys in flight.  When the key range of an item
// is split, normalised partial outputs and their log-sum-exp go to scratch memory and a
// second kernel merges them in a fixed order.
//
// Formula (rapid_llm/kernels/ops/attention/flashattention2_nopad.py:85,141-168,
// rapid_llm/kernels/ops/attention/flashdecoding.py:223-230,335-407): kv head = q head //
// group; s_j = (q . k_j) * scale for cached j <= p of the same request (and j > p - window
// when a window is set); softmax over j; o = sum_j P_j v_j.  Scores, running maximum and
// sum and the output accumulator are float32; the exponent is taken in base 2 with log2(e)
// folded into the scale; P is rounded to bfloat16 before the P.V product, as the
// reference's tensor-core kernels do (flashattention2_nopad.py:162).
#include <mutex>

#include "attention_static_scratch.h"
#include "common.cuh"

#ifndef RL_HEAD_DIM
#error "compile with -DRL_HEAD_DIM=<head size>"
#endif

// Every head size is a library of its own, and several of them are loaded side by side.  The
// head size is part of the namespace so that no symbol of one build can be taken for
// another's, and nothing here is a function-local static (those are merged across libraries).
#define RL_CONCAT2(a, b) a##b
#define RL_CONCAT(a, b) RL_CONCAT2(a, b)
#define RL_ATTENTION_NS RL_CONCAT(attention_d, RL_HEAD_DIM)

namespace rl {
namespace RL_ATTENTION_NS {

using bf16 = __nv_bfloat16;
constexpr int kD = RL_HEAD_DIM;
static_assert(kD % 16 == 0 && kD >= 16 && kD <= 256, "head size: multiples of 16 up to 256");
constexpr int kBlockN = 64;                 // keys per pipeline stage
constexpr int kStride = kD + 8;             // row stride in shared memory (elements): the 16-byte
                                            // pad keeps ldmatrix free of bank conflicts
constexpr int kChunksPerRow = kD / 8;       // 16-byte chunks in a row
constexpr int kThreads = 128;
constexpr bool kQInRegisters = kD <= 128;
constexpr int kStagedPages = 1024;          // page ids of an item's key range kept in shared memory

struct AttentionArgs {
  const bf16* q;            // [tokens, hq, D]
  const bf16* cache;        // [num_pages, 2, hkv, page_size, D]
  bf16* out;                // [tokens, hq, D]
  float* part_out;          // [tokens, hq, splits, D]   (splits > 1)
  float* part_lse;          // [tokens, hq, splits]      base-2 log-sum-exp
  const int* items;         // [n_items, 4]: entry, first packed row, split, unused
  const int* cu_seqlens;    // [entries + 1]
  const int* entry_start;   // [entries]  tokens cached before this step
  const int* entry_slot;    // [entries]
  const int* block_table;   // [slots, max_pages]
  int hq, hkv, page_size, num_pages, max_pages, slots, window, splits;
  float scale_log2;         // scale * log2(e)
  int* fault;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0 = fill the 16 bytes with zeros, read nothing
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// kWarpsM warps stacked over the tile's rows, kWarpsN warps side by side over each block's keys.
template <int kWarpsM, int kWarpsN, int kStages>
__global__ void __launch_bounds__(kThreads)
attention_mma_kernel(const AttentionArgs args) {
  static_assert(kWarpsM * kWarpsN == 4, "four warps");
  constexpr int kTileM = 16 * kWarpsM;
  constexpr int kKeysPerWarp = kBlockN / kWarpsN;
  constexpr int kScoreTiles = kKeysPerWarp / 8;     // n-tiles of 8 keys per warp and block
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_smem = reinterpret_cast<bf16*>(smem_raw);                    // [kTileM][kStride]
  bf16* k_smem = q_smem + kTileM * kStride;                            // [kStages][64][kStride]
  bf16* v_smem = k_smem + kStages * kBlockN * kStride;                 // [kStages][64][kStride]

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp % kWarpsM, wn = warp / kWarpsM;
  // the kv head is the fast grid dimension: CTAs start in the order of the item list (longest
  // first) over all heads, so the last wave holds the shortest items
  const int* item = args.items + static_cast<size_t>(blockIdx.y) * 4;
  const int entry = item[0], row0 = item[1], split = item[2];
  const int kv_head = blockIdx.x;
  const int group = args.hq / args.hkv;
  const int tok_begin = args.cu_seqlens[entry];
  const int n_rows = (args.cu_seqlens[entry + 1] - tok_begin) * group;
  const int start = args.entry_start[entry];
  const int slot = args.entry_slot[entry];

  // rows of this thread in the accumulator layout: r_a = lane / 4 and r_a + 8 of its warp
  int row_pos[2], row_lo[2], row_token[2], row_head[2];
  bool row_valid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int p = row0 + wm * 16 + (lane >> 2) + 8 * i;
    row_valid[i] = p < n_rows;
    const int token = p / group;
    row_token[i] = tok_begin + token;
    row_head[i] = kv_head * group + (p - token * group);
    row_pos[i] = row_valid[i] ? start + token : -1;
    row_lo[i] = args.window > 0 ? max(0, row_pos[i] - args.window + 1) : 0;
  }

  const int last_row = min(n_rows, row0 + kTileM) - 1;
  const int min_pos = start + row0 / group, max_pos = start + last_row / group;
  bool bad = slot < 0 || slot >= args.slots || start < 0 ||
             max_pos >= args.max_pages * args.page_size || last_row < row0;
  if (bad) {
    if (tid == 0) atomicOr(args.fault, (slot < 0 || slot >= args.slots) ? kFaultSlot : kFaultPosition);
  }
  // key range of the tile, then of this split (begin on a multiple of 64)
  const int hi = bad ? 0 : max_pos + 1;
  const int lo = args.window > 0 ? max(0, min_pos - args.window + 1) : 0;
  const int lo_aligned = lo & ~(kBlockN - 1);
  const int span = max(hi - lo_aligned, 0);
  const int per_split = ((span + args.splits - 1) / args.splits + kBlockN - 1) / kBlockN * kBlockN;
  const int k_begin = lo_aligned + split * per_split;
  const int k_end = min(hi, k_begin + per_split);
  const int n_blocks = k_end > k_begin ? (k_end - k_begin + kBlockN - 1) / kBlockN : 0;
  const int* table = args.block_table + static_cast<size_t>(bad ? 0 : slot) * args.max_pages;
  const size_t v_plane = static_cast<size_t>(args.hkv) * args.page_size * kD;

  // The page ids of this item's key range, fetched once and side by side (a lookup per
  // 16-byte copy would put a dependent global load in front of every copy).  The block table
  // is uploaded before the step's first kernel, so this may run before the wait below.
  __shared__ int staged_pages[kStagedPages];
  const int first_page = k_begin / args.page_size;
  const int page_count = n_blocks > 0 ? (k_end - 1) / args.page_size - first_page + 1 : 0;
  const bool staged = page_count <= kStagedPages;
  if (staged) {
    for (int i = tid; i < page_count; i += kThreads) {
      int page = table[first_page + i];
      if (page < 0 || page >= args.num_pages) {
        atomicOr(args.fault, kFaultPageId);
        page = -1;
      }
      staged_pages[i] = page;
    }
    __syncthreads();
  }

  // ---- loads -------------------------------------------------------------------------
  auto load_q = [&]() {
    for (int idx = tid; idx < kTileM * kChunksPerRow; idx += kThreads) {
      const int r = idx / kChunksPerRow, c = idx - r * kChunksPerRow;
      const int p = row0 + r;
      const bool valid = p < n_rows && !bad;
      const int token = p / group;
      const bf16* src = args.q;
      if (valid)
        src = args.q + (static_cast<size_t>(tok_begin + token) * args.hq + kv_head * group +
                        (p - token * group)) * kD + c * 8;
      cp_async16(smem_u32(q_smem + r * kStride + c * 8), src, valid);
    }
  };
  // Where each of this thread's 16-byte copies of a block comes from.  When a block of 64 keys
  // is a whole number of pages (or lies inside one page), the page a row belongs to and its
  // place in the page do not change from block to block, so they are worked out once.
  constexpr int kLoadIters = kBlockN * kChunksPerRow / kThreads;
  static_assert(kBlockN * kChunksPerRow % kThreads == 0, "copies divide evenly over the threads");
  const bool regular = staged && (kBlockN % args.page_size == 0 || args.page_size % kBlockN == 0);
  int copy_row[kLoadIters], copy_page[kLoadIters], copy_src[kLoadIters], copy_dst[kLoadIters];
#pragma unroll
  for (int i = 0; i < kLoadIters; ++i) {
    const int idx = tid + i * kThreads;
    const int r = idx / kChunksPerRow, c = idx - r * kChunksPerRow;
    copy_row[i] = r;
    copy_dst[i] = r * kStride + c * 8;
    const bool small_pages = args.page_size <= kBlockN;
    copy_page[i] = regular && small_pages ? r / args.page_size : 0;
    copy_src[i] = (regular && small_pages ? r % args.page_size : r) * kD + c * 8;
  }
  const size_t page_stride = static_cast<size_t>(2) * args.hkv * args.page_size * kD;
  const bf16* head_base = args.cache + static_cast<size_t>(kv_head) * args.page_size * kD;

  auto load_block = [&](int stage, int kb) {
    bf16* ks = k_smem + stage * kBlockN * kStride;
    bf16* vs = v_smem + stage * kBlockN * kStride;
    if (regular) {
      const int block_page = kb / args.page_size - first_page;
      const int block_offset = (kb % args.page_size) * kD;      // 0 unless pages are larger than a block
#pragma unroll
      for (int i = 0; i < kLoadIters; ++i) {
        bool valid = kb + copy_row[i] < k_end;
        const int page = valid ? staged_pages[block_page + copy_page[i]] : -1;
        valid = page >= 0;
        const bf16* src = valid ? head_base + page * page_stride + block_offset + copy_src[i] : args.cache;
        cp_async16(smem_u32(ks + copy_dst[i]), src, valid);
        cp_async16(smem_u32(vs + copy_dst[i]), valid ? src + v_plane : src, valid);
      }
      return;
    }
    for (int idx = tid; idx < kBlockN * kChunksPerRow; idx += kThreads) {
      const int r = idx / kChunksPerRow, c = idx - r * kChunksPerRow;
      const int j = kb + r;
      bool valid = j < k_end;
      const bf16* src = args.cache;
      if (valid) {
        const int page_index = j / args.page_size;
        int page;
        if (staged) {
          page = staged_pages[page_index - first_page];
        } else {
          page = table[page_index];
          if (page < 0 || page >= args.num_pages) {
            atomicOr(args.fault, kFaultPageId);
            page = -1;
          }
        }
        if (page < 0) {
          valid = false;
        } else {
          src = head_base + page * page_stride + static_cast<size_t>(j - page_index * args.page_size) * kD + c * 8;
        }
      }
      cp_async16(smem_u32(ks + r * kStride + c * 8), src, valid);
      cp_async16(smem_u32(vs + r * kStride + c * 8), valid ? src + v_plane : src, valid);
    }
  };

  pdl_wait();   // queries and this step's keys come from the kernels before
  load_q();
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < n_blocks) load_block(s, k_begin + s * kBlockN);
    cp_async_commit();
  }

  // ---- state -------------------------------------------------------------------------
  float o_acc[kD / 8][4];
#pragma unroll
  for (int i = 0; i < kD / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[i][e] = 0.0f;
  float run_max[2] = {-INFINITY, -INFINITY}, run_sum[2] = {0.0f, 0.0f};
  uint32_t q_frag[kQInRegisters ? kD / 16 : 1][4];
  const uint32_t q_lane_addr =
      smem_u32(q_smem + (wm * 16 + (lane & 15)) * kStride + (lane >> 4) * 8);
  const int warp_max_pos = __reduce_max_sync(0xffffffffu, max(row_pos[0], row_pos[1]));

  for (int b = 0; b < n_blocks; ++b) {
    const int next = b + kStages - 1;
    if (next < n_blocks) load_block(next % kStages, k_begin + next * kBlockN);
    cp_async_commit();
    cp_async_wait<kStages - 1>();
    __syncthreads();
    if constexpr (kQInRegisters) {
      if (b == 0) {
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) ldmatrix_x4(q_frag[ks], q_lane_addr + ks * 32);
      }
    }
    const int kb = k_begin + b * kBlockN;
    const int key0 = kb + wn * kKeysPerWarp;            // first key of this warp in the block
    if (key0 <= warp_max_pos && key0 < k_end) {
      const bf16* ks_base = k_smem + (b % kStages) * kBlockN * kStride + wn * kKeysPerWarp * kStride;
      const bf16* vs_base = v_smem + (b % kStages) * kBlockN * kStride + wn * kKeysPerWarp * kStride;
      // S = Q K^T
      float s[kScoreTiles][4];
#pragma unroll
      for (int nt = 0; nt < kScoreTiles; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
      const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) {
        uint32_t a[4];
        if constexpr (kQInRegisters) {
#pragma unroll
          for (int e = 0; e < 4; ++e) a[e] = q_frag[ks][e];
        } else {
          ldmatrix_x4(a, q_lane_addr + ks * 32);
        }
#pragma unroll
        for (int np = 0; np < kScoreTiles / 2; ++np) {
          uint32_t kf[4];
          ldmatrix_x4(kf, smem_u32(ks_base + (np * 16 + (mi >> 1) * 8 + mr) * kStride + ks * 16 +
                                   (mi & 1) * 8));
          mma_bf16(s[2 * np], a, kf[0], kf[1]);
          mma_bf16(s[2 * np + 1], a, kf[2], kf[3]);
        }
      }
      // scale, mask, running softmax
      float block_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < kScoreTiles; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const int i = e >> 1;
          const bool keep = j <= row_pos[i] && j >= row_lo[i] && j < k_end;
          const float v = keep ? s[nt][e] * args.scale_log2 : -INFINITY;
          s[nt][e] = v;
          block_max[i] = fmaxf(block_max[i], v);
        }
      }
      float correction[2], safe_max[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        block_max[i] = fmaxf(block_max[i], __shfl_xor_sync(0xffffffffu, block_max[i], 1));
        block_max[i] = fmaxf(block_max[i], __shfl_xor_sync(0xffffffffu, block_max[i], 2));
        const float new_max = fmaxf(run_max[i], block_max[i]);
        safe_max[i] = new_max == -INFINITY ? 0.0f : new_max;
        correction[i] = exp2f(run_max[i] - safe_max[i]);   // 0 while nothing was seen
        run_max[i] = new_max;
        run_sum[i] *= correction[i];
      }
#pragma unroll
      for (int nt = 0; nt < kScoreTiles; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = exp2f(s[nt][e] - safe_max[e >> 1]);
          s[nt][e] = p;
          run_sum[e >> 1] += p;
        }
      }
#pragma unroll
      for (int i = 0; i < kD / 8; ++i) {
        o_acc[i][0] *= correction[0];
        o_acc[i][1] *= correction[0];
        o_acc[i][2] *= correction[1];
        o_acc[i][3] *= correction[1];
      }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < kKeysPerWarp / 16; ++kk) {
        uint32_t p_frag[4];
        p_frag[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        p_frag[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        p_frag[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        p_frag[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < kD / 16; ++dp) {
          uint32_t vf[4];
          ldmatrix_x4_trans(vf, smem_u32(vs_base + (kk * 16 + (mi & 1) * 8 + mr) * kStride +
                                         dp * 16 + (mi >> 1) * 8));
          mma_bf16(o_acc[2 * dp], p_frag, vf[0], vf[1]);
          mma_bf16(o_acc[2 * dp + 1], p_frag, vf[2], vf[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // ---- finish --------------------------------------------------------------------------
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    run_sum[i] += __shfl_xor_sync(0xffffffffu, run_sum[i], 1);
    run_sum[i] += __shfl_xor_sync(0xffffffffu, run_sum[i], 2);
  }

  if constexpr (kWarpsN == 1) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (!row_valid[i]) continue;
      const float inv = run_sum[i] > 0.0f ? 1.0f / run_sum[i] : 0.0f;
      const size_t row = static_cast<size_t>(row_token[i]) * args.hq + row_head[i];
      if (args.splits == 1) {
        bf16* dst = args.out + row * kD + (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < kD / 8; ++nt)
          *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) =
              __floats2bfloat162_rn(o_acc[nt][2 * i] * inv, o_acc[nt][2 * i + 1] * inv);
      } else {
        float* dst = args.part_out + (row * args.splits + split) * kD + (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < kD / 8; ++nt)
          *reinterpret_cast<float2*>(dst + nt * 8) =
              make_float2(o_acc[nt][2 * i] * inv, o_acc[nt][2 * i + 1] * inv);
        if ((lane & 3) == 0)
          args.part_lse[row * args.splits + split] =
              run_sum[i] > 0.0f ? run_max[i] + log2f(run_sum[i]) : -INFINITY;
      }
    }
  } else {
    // the warps hold states over disjoint keys of the same 16 rows: merge through shared memory
    constexpr int kMergeStride = kD + 4;
    float* merge_o = reinterpret_cast<float*>(k_smem);                 // [kWarpsN][16][kMergeStride]
    float* merge_ml = merge_o + kWarpsN * 16 * kMergeStride;           // [kWarpsN][16][2]
    static_assert((kWarpsN * 16 * (kMergeStride + 2)) * 4 <= 2 * kStages * kBlockN * kStride * 2,
                  "merge buffers fit in the key/value stages");
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = (lane >> 2) + 8 * i;
      float* dst = merge_o + (wn * 16 + r) * kMergeStride + (lane & 3) * 2;
#pragma unroll
      for (int nt = 0; nt < kD / 8; ++nt)
        *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o_acc[nt][2 * i], o_acc[nt][2 * i + 1]);
      if ((lane & 3) == 0) {
        merge_ml[(wn * 16 + r) * 2] = run_max[i];
        merge_ml[(wn * 16 + r) * 2 + 1] = run_sum[i];
      }
    }
    __syncthreads();
    for (int idx = tid; idx < 16 * kD; idx += kThreads) {
      const int r = idx / kD, c = idx - r * kD;
      const int p = row0 + r;
      if (p >= n_rows) continue;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < kWarpsN; ++w) m = fmaxf(m, merge_ml[(w * 16 + r) * 2]);
      const float safe = m == -INFINITY ? 0.0f : m;
      float total = 0.0f, value = 0.0f;
#pragma unroll
      for (int w = 0; w < kWarpsN; ++w) {
        const float weight = exp2f(merge_ml[(w * 16 + r) * 2] - safe);
        total += weight * merge_ml[(w * 16 + r) * 2 + 1];
        value += weight * merge_o[(w * 16 + r) * kMergeStride + c];
      }
      const float inv = total > 0.0f ? 1.0f / total : 0.0f;
      const int token = p / group;
      const size_t row = static_cast<size_t>(tok_begin + token) * args.hq + kv_head * group +
                         (p - token * group);
      if (args.splits == 1) {
        args.out[row * kD + c] = __float2bfloat16_rn(value * inv);
      } else {
        args.part_out[(row * args.splits + split) * kD + c] = value * inv;
        if (c == 0)
          args.part_lse[row * args.splits + split] = total > 0.0f ? m + log2f(total) : -INFINITY;
      }
    }
  }
}

// out[row] = sum_s w_s part[row, s] / sum_s w_s with w_s = 2^(lse_s - max lse), splits in index
// order; one warp per (token, head) row.
__global__ void attention_merge_kernel(const float* __restrict__ part_out,
                                       const float* __restrict__ part_lse, bf16* __restrict__ out,
                                       long long rows, int splits) {
  pdl_trigger();
  pdl_wait();
  const long long row = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float* lse = part_lse + row * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, lse[s]);
  const float safe = m == -INFINITY ? 0.0f : m;
  float total = 0.0f;
  for (int s = 0; s < splits; ++s) total += exp2f(lse[s] - safe);
  const float inv = total > 0.0f ? 1.0f / total : 0.0f;
  for (int c = lane; c < kD; c += 32) {
    float value = 0.0f;
    for (int s = 0; s < splits; ++s) {
      // a part without keys is not read: nothing wrote it, and 0 * (a NaN left there) would be NaN
      if (lse[s] == -INFINITY) continue;
      value += exp2f(lse[s] - safe) * part_out[(row * splits + s) * kD + c];
    }
    out[row * kD + c] = __float2bfloat16_rn(value * inv);
  }
}

template <int kWarpsM, int kWarpsN, int kStages>
constexpr size_t attention_smem_bytes() {
  return static_cast<size_t>(16 * kWarpsM + 2 * kStages * kBlockN) * kStride * sizeof(bf16);
}

static bool g_configured[2] = {false, false};   // [chunk tiles, decode tiles]; file-local on purpose

template <int kWarpsM, int kWarpsN, int kStages>
int launch_attention(const AttentionArgs& args, int n_items, bool pdl, cudaStream_t stream) {
  auto kernel = attention_mma_kernel<kWarpsM, kWarpsN, kStages>;
  constexpr size_t smem = attention_smem_bytes<kWarpsM, kWarpsN, kStages>();
  static_assert(smem <= 227 * 1024, "shared memory of one CTA");
  bool& configured = g_configured[kWarpsN == 1 ? 0 : 1];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  return launch_kernel(kernel, dim3(args.hkv, n_items), dim3(kThreads), smem, stream, pdl, args);
}

}  // namespace RL_ATTENTION_NS
}  // namespace rl

#include "attention_decode_tc.cuh"
#include "attention_prefill_tc.cuh"

namespace rl {
namespace RL_ATTENTION_NS {

// Whether the tcgen05 decode kernel takes this geometry (everything else: the mma.sync tiles).
static bool decode_tc_supported(int page_size) {
  return kD == kTcD && page_size % 8 == 0 && (kTcKeys % page_size == 0 || page_size % kTcKeys == 0);
}

static bool g_prefill_tc_configured = false;   // file-local on purpose

// Chunk tiles of 256 packed rows on the tcgen05 kernel (unsplit key ranges only).
static int launch_prefill_tc(const AttentionArgs& a, int n_items, bool pdl, cudaStream_t stream) {
  if (!g_prefill_tc_configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kPfSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_prefill_tc_configured = true;
  }
  CUtensorMap map;
  const long long rows = static_cast<long long>(a.num_pages) * 2 * a.hkv * a.page_size;
  int status = make_map(&map, a.cache, rows, kD, a.page_size < kPfKeys ? a.page_size : kPfKeys);
  if (status != 0) return status;
  PrefillTcArgs t;
  t.q = a.q; t.out = a.out; t.items = a.items; t.cu_seqlens = a.cu_seqlens; t.entry_start = a.entry_start;
  t.entry_slot = a.entry_slot; t.block_table = a.block_table; t.hq = a.hq; t.hkv = a.hkv;
  t.page_size = a.page_size; t.num_pages = a.num_pages; t.max_pages = a.max_pages; t.slots = a.slots;
  t.window = a.window; t.scale_log2 = a.scale_log2; t.fault = a.fault;
  return launch_kernel(attention_prefill_tc_kernel, dim3(a.hkv, n_items), dim3(kPfThreads), kPfSmemBytes, stream, pdl,
                       map, t);
}

static bool g_decode_tc_configured[5][2] = {};   // per row-count and ring-depth instantiation; file-local on purpose

static int decode_tc_sm_count() {
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
    sms = 148;
  return sms;
}

template <int kRows, int kStages>
static int launch_decode_tc_stages(const CUtensorMap& map, const DecodeTcArgs& t, int n_items, bool pdl,
                                   cudaStream_t stream, bool* configured) {
  auto kernel = attention_decode_tc_kernel<kRows, kStages>;
  constexpr int kTcSmemBytes = tc_smem_bytes(kStages);
  if (!*configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    // clusters of more than 8 CTAs (up to 16 key ranges of a tile) have to be asked for
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return static_cast<int>(e);
    *configured = true;
  }
  // x: the key ranges of one tile (a cluster when they merge among themselves), y: the kv head,
  // z: the tile.  CTAs start in x, y, z order: the tiles of the item list, longest first, over
  // all heads, so that the last wave holds the shortest.
  if (t.splits < 1 || n_items % t.splits != 0 || n_items / t.splits > 65535) return static_cast<int>(cudaErrorInvalidValue);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(t.splits, t.hkv, n_items / t.splits);
  config.blockDim = dim3(kTcThreads);
  config.dynamicSmemBytes = kTcSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  int count = 0;
  if (t.cluster_merge) {
    attributes[count].id = cudaLaunchAttributeClusterDimension;
    attributes[count].val.clusterDim.x = t.splits;
    attributes[count].val.clusterDim.y = 1;
    attributes[count].val.clusterDim.z = 1;
    ++count;
  }
  if (pdl) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  return static_cast<int>(cudaLaunchKernelEx(&config, kernel, map, t));
}

// More CTAs than multiprocessors, each by itself (no cluster): two shallow CTAs per multiprocessor, so that one
// streams while the other starts.  Decided by the number of items alone: a captured decode graph replays the same
// choice at every context length.
// `rings`: 0 = decide here, 2 = deep, 3 = shallow (for measurements).
template <int kRows>
static int launch_decode_tc_rows(const CUtensorMap& map, const DecodeTcArgs& t, int n_items, bool pdl,
                                 cudaStream_t stream, bool* configured, int rings) {
  const bool shallow = rings == 3 || (rings != 2 && !t.cluster_merge &&
                                      static_cast<long long>(n_items) * t.hkv > decode_tc_sm_count());
  if (shallow) return launch_decode_tc_stages<kRows, 1>(map, t, n_items, pdl, stream, configured + 1);
  return launch_decode_tc_stages<kRows, kTcMaxStages>(map, t, n_items, pdl, stream, configured);
}

// cluster_merge: the `splits` items of a tile are consecutive in the grid and launched as one
// thread-block cluster, whose CTAs merge their partial results among themselves.  max_rows: the
// most packed rows any of the items has (0 = not known).
static int launch_decode_tc(const AttentionArgs& a, int n_items, int max_rows, bool cluster_merge, bool pdl,
                            cudaStream_t stream, int rings = 0) {
  CUtensorMap map;
  const long long rows = static_cast<long long>(a.num_pages) * 2 * a.hkv * a.page_size;
  int status = make_map(&map, a.cache, rows, kD, a.page_size < kTcKeys ? a.page_size : kTcKeys);
  if (status != 0) return status;
  DecodeTcArgs t;
  t.q = a.q; t.out = a.out; t.part_out = a.part_out; t.part_lse = a.part_lse; t.items = a.items;
  t.cu_seqlens = a.cu_seqlens; t.entry_start = a.entry_start; t.entry_slot = a.entry_slot;
  t.block_table = a.block_table; t.hq = a.hq; t.hkv = a.hkv; t.page_size = a.page_size;
  t.num_pages = a.num_pages; t.max_pages = a.max_pages; t.slots = a.slots; t.window = a.window;
  t.splits = a.splits; t.cluster_merge = cluster_merge ? 1 : 0; t.scale_log2 = a.scale_log2; t.fault = a.fault;
  if (max_rows <= 0 || max_rows > kTcRows) max_rows = kTcRows;
  if (max_rows <= 1) return launch_decode_tc_rows<1>(map, t, n_items, pdl, stream, g_decode_tc_configured[0], rings);
  if (max_rows <= 2) return launch_decode_tc_rows<2>(map, t, n_items, pdl, stream, g_decode_tc_configured[1], rings);
  if (max_rows <= 4) return launch_decode_tc_rows<4>(map, t, n_items, pdl, stream, g_decode_tc_configured[2], rings);
  if (max_rows <= 8) return launch_decode_tc_rows<8>(map, t, n_items, pdl, stream, g_decode_tc_configured[3], rings);
  return launch_decode_tc_rows<16>(map, t, n_items, pdl, stream, g_decode_tc_configured[4], rings);
}

}  // namespace RL_ATTENTION_NS
}  // namespace rl

namespace attn = rl::RL_ATTENTION_NS;

extern "C" {

int rl_attention_head_dim() { return attn::kD; }

// Rows of a chunk tile and of a decode tile: the host cuts requests into items with these.
int rl_attention_chunk_rows() { return 64; }
// ... of a chunk tile of the tcgen05 kernel, or 0 where this build (head size) has none.
int rl_attention_chunk_rows_tc() { return attn::kD == attn::kPfD ? attn::kPfRows : 0; }
int rl_attention_decode_rows() { return 16; }

// chunk_rows: packed rows per chunk item: 64 (or 0) = the mma.sync tiles, 256 = the tcgen05
// kernel (head size 128, pages it takes, splits == 1).
// decode_splits: key ranges of the decode tiles where they differ from `splits` (a step of prompt portions, which
// the tcgen05 kernel does not split, beside single tokens with long contexts); 0 = the same.
// decode_kernel: 0 = the tcgen05 kernel for decode tiles where it applies, 1 = always the
// mma.sync tiles, 2 / 3 = the tcgen05 kernel with deep rings (one CTA per multiprocessor) / shallow
// rings (two) whatever the number of items.  decode_rows: the most packed rows any decode tile has (0 = not known).
// chunk_items / decode_items: [n, 4] int32 (entry, first packed row, split, 0).  With
// splits > 1, part_out [tokens, hq, splits, D] and part_lse [tokens, hq, splits] are scratch
// and every (row, split) pair must be covered by exactly one item.
// How many clusters of `cluster_size` CTAs of the tcgen05 decode kernel (deep rings: one CTA per multiprocessor)
// the GPU runs at one time, or a negative CUDA error code.  A cluster lives inside one GPC, so the answer is not
// the number of multiprocessors over the size; the host's planner asks once per size.
int rl_attention_decode_max_clusters(int cluster_size) {
  if (attn::kD != attn::kTcD || cluster_size < 1 || cluster_size > attn::kTcMaxClusterSplits) return -static_cast<int>(cudaErrorInvalidValue);
  auto kernel = attn::attention_decode_tc_kernel<4, attn::kTcMaxStages>;
  constexpr int kBytes = attn::tc_smem_bytes(attn::kTcMaxStages);
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (e != cudaSuccess) return -static_cast<int>(e);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(cluster_size, 1, 64);
  config.blockDim = dim3(attn::kTcThreads);
  config.dynamicSmemBytes = kBytes;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = cluster_size;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  int clusters = 0;
  e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &config);
  return e == cudaSuccess ? clusters : -static_cast<int>(e);
}

int rl_attention_mma(const void* q, const void* cache, void* out, float* part_out, float* part_lse,
                     const int* chunk_items, int n_chunk_items, const int* decode_items,
                     int n_decode_items, const int* cu_seqlens, const int* entry_start,
                     const int* entry_slot, const int* block_table, int tokens, int hq, int hkv,
                     int head_dim, int page_size, int num_pages, int max_pages, int slots,
                     int window, int splits, float scale, int* fault, int pdl, int decode_kernel, int decode_rows,
                     int chunk_rows, int decode_splits, cudaStream_t stream) {
  if (tokens == 0 || (n_chunk_items == 0 && n_decode_items == 0)) return 0;
  if (head_dim != attn::kD || hkv <= 0 || hq % hkv != 0 || page_size <= 0 || window < 0 ||
      splits < 1 || (splits > 1 && (part_out == nullptr || part_lse == nullptr)) ||
      hkv > 65535 || n_chunk_items > 65535 || n_decode_items > 65535)      // grid y dimensions
    return static_cast<int>(cudaErrorInvalidValue);
  // key ranges of the decode tiles alone (0 = as `splits`): only where the chunk tiles are not split and the decode
  // kernel merges its ranges inside a cluster, so that no scratch and no merge kernel are involved
  if (decode_splits < 0 || (decode_splits > 0 && decode_splits != splits &&
                            (splits != 1 || decode_kernel == 1 || !attn::decode_tc_supported(page_size) ||
                             decode_splits > attn::kTcMaxClusterSplits || n_decode_items % decode_splits != 0)))
    return static_cast<int>(cudaErrorInvalidValue);
  attn::AttentionArgs args;
  args.q = static_cast<const attn::bf16*>(q);
  args.cache = static_cast<const attn::bf16*>(cache);
  args.out = static_cast<attn::bf16*>(out);
  args.part_out = part_out;
  args.part_lse = part_lse;
  args.cu_seqlens = cu_seqlens;
  args.entry_start = entry_start;
  args.entry_slot = entry_slot;
  args.block_table = block_table;
  args.hq = hq; args.hkv = hkv; args.page_size = page_size; args.num_pages = num_pages;
  args.max_pages = max_pages; args.slots = slots; args.window = window; args.splits = splits;
  args.scale_log2 = scale * 1.4426950408889634f;
  args.fault = fault;
  int status = 0;
  bool merged_in_cluster = false;
  if (n_chunk_items > 0) {
    args.items = chunk_items;
    if (chunk_rows == attn::kPfRows) {
      // the host cut the portions into tiles of the tcgen05 kernel: it must apply
      if (attn::kD != attn::kPfD || !attn::decode_tc_supported(page_size) || splits != 1)
        return static_cast<int>(cudaErrorInvalidValue);
      status = attn::launch_prefill_tc(args, n_chunk_items, pdl != 0, stream);
    } else if (chunk_rows == 64 || chunk_rows == 0) {
      status = attn::launch_attention<4, 1, 2>(args, n_chunk_items, pdl != 0, stream);
    } else {
      return static_cast<int>(cudaErrorInvalidValue);
    }
    if (status != 0) return status;
  }
  if (n_decode_items > 0) {
    args.items = decode_items;
    if (decode_kernel != 1 && attn::decode_tc_supported(page_size)) {
      const bool own_splits = decode_splits > 1 && decode_splits != splits;
      if (own_splits) args.splits = decode_splits;
      merged_in_cluster = own_splits || (n_chunk_items == 0 && splits > 1 && splits <= attn::kTcMaxClusterSplits &&
                                         n_decode_items % splits == 0);
      status = attn::launch_decode_tc(args, n_decode_items, decode_rows, merged_in_cluster, pdl != 0, stream,
                                      decode_kernel == 2 || decode_kernel == 3 ? decode_kernel : 0);
      args.splits = splits;
    } else
      status = attn::launch_attention<1, 4, 3>(args, n_decode_items, pdl != 0, stream);
    if (status != 0) return status;
  }
  if (splits > 1 && !merged_in_cluster) {
    const long long rows = static_cast<long long>(tokens) * hq;
    status = rl::launch_kernel(attn::attention_merge_kernel, dim3(static_cast<unsigned>((rows + 3) / 4)), dim3(128), 0,
                               stream, pdl != 0, part_out, part_lse, static_cast<attn::bf16*>(out), rows, splits);
  }
  return status;
}

}  // extern "C"

// ----------------------------------------------------------------------------------------
// Allocation-free variant (declared and explained in attention_static_scratch.h; the
// reference has nothing like it).  The scratch of the split key ranges lives in the library
// image instead of in memory the caller allocates.
namespace rl {
namespace RL_ATTENTION_NS {

constexpr long long kStaticScratchFloats = 1ll << 20;   // 4 MiB per GPU that loads this library
constexpr int kStaticScratchMaxDevices = 64;

// Device memory.  In host code this name is only a handle for cudaGetSymbolAddress: it is
// not a device address and must never be handed to a kernel as one.
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

static std::mutex g_static_scratch_mutex;
static float* g_static_scratch_address[kStaticScratchMaxDevices] = {};   // per device, looked up once

// The array's address on the current device; the first call on a device asks the runtime.
static int static_scratch_address(float** address) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (device < 0 || device >= kStaticScratchMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
  std::lock_guard<std::mutex> guard(g_static_scratch_mutex);
  if (g_static_scratch_address[device] == nullptr) {
    void* found = nullptr;
    e = cudaGetSymbolAddress(&found, g_static_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (found == nullptr) return static_cast<int>(cudaErrorInvalidSymbol);
    g_static_scratch_address[device] = static_cast<float*>(found);
  }
  *address = g_static_scratch_address[device];
  return 0;
}

// lse[i] = -inf: the merge does not read the part of a (row, split) slot that no work item of this
// call writes, so what an earlier call left there (finite or not) cannot reach the output.
__global__ void static_scratch_reset_kernel(float* __restrict__ lse, long long count) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) lse[i] = -INFINITY;
}

}  // namespace RL_ATTENTION_NS
}  // namespace rl

extern "C" {

long long rl_attention_static_scratch_bytes(void) {
  return attn::kStaticScratchFloats * static_cast<long long>(sizeof(float));
}

const char* rl_attention_static_scratch_strerror(int code) {
  if (code == 0) return "success";
  if (code == RL_ATTENTION_STATIC_SCRATCH_TOO_LARGE)
    return "tokens * hq * splits * (head_dim + 1) floats exceed the library's built-in scratch array "
           "(rl_attention_static_scratch_bytes); use fewer splits or tokens per call, or rl_attention_mma "
           "with buffers of your own";
  return cudaGetErrorString(static_cast<cudaError_t>(code));
}

int rl_attention_mma_static_scratch(const void* q, const void* cache, void* out, const int* chunk_items,
                                    int n_chunk_items, const int* decode_items, int n_decode_items,
                                    const int* cu_seqlens, const int* entry_start, const int* entry_slot,
                                    const int* block_table, int tokens, int hq, int hkv, int head_dim,
                                    int page_size, int num_pages, int max_pages, int slots, int window,
                                    int splits, float scale, int* fault, cudaStream_t stream) {
  if (tokens == 0 || (n_chunk_items == 0 && n_decode_items == 0)) return 0;
  if (tokens < 0 || hq <= 0 || splits < 1 || head_dim != attn::kD)
    return static_cast<int>(cudaErrorInvalidValue);
  float* part_out = nullptr;
  float* part_lse = nullptr;
  if (splits > 1) {
    const long long rows = static_cast<long long>(tokens) * hq * splits;
    if (rows > attn::kStaticScratchFloats / (attn::kD + 1)) return RL_ATTENTION_STATIC_SCRATCH_TOO_LARGE;
    float* scratch = nullptr;
    const int status = attn::static_scratch_address(&scratch);
    if (status != 0) return status;
    part_out = scratch;                        // [rows, D]
    part_lse = scratch + rows * attn::kD;      // [rows]
    attn::static_scratch_reset_kernel<<<static_cast<unsigned>((rows + 255) / 256), 256, 0, stream>>>(part_lse, rows);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return rl_attention_mma(q, cache, out, part_out, part_lse, chunk_items, n_chunk_items, decode_items,
                          n_decode_items, cu_seqlens, entry_start, entry_slot, block_table, tokens, hq, hkv,
                          head_dim, page_size, num_pages, max_pages, slots, window, splits, scale, fault, 0, 1, 0, 64, 0, stream);
}

}  // extern "C"

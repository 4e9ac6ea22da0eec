// Paged causal attention for any head size (steps of 16 up to 256), any number of heads
// and groups, any page size, with an optional window; one warp per (token, query head).
//
// This is the kernel of the float32 path and the fallback of the bfloat16 path for head
// sizes the tensor-core kernels are not instantiated for.  Every token of the step is a
// query row of its own: a portion of a prompt and a single decoded token differ only in
// how many rows a request contributes.  Keys and values are read from the cache through
// the request's block table, so the rows of this step must have been written before.
//
// Formula (rapid_llm/kernels/ops/attention/flashattention2_nopad.py:85,141-168 and
// rapid_llm/kernels/ops/attention/flashdecoding.py:223-230): kv head = q head // group;
// s_j = (q . k_j) * scale over the cached positions j <= p of the same request (and
// j > p - window when a window is set: the query's own position counts, as in
// rapid_llm/engine/kv_cache_spec.py:204,221-224); softmax over j; o = sum_j P_j v_j.
// Scores, running maximum and sum, and the output accumulator are float32.
#include "common.cuh"

namespace rl {

constexpr int kGenericWarps = 4;
constexpr int kGenericMaxD = 256;

template <typename T>
__global__ void attention_generic_kernel(
    const T* __restrict__ q,            // [tokens, hq, d]
    const T* __restrict__ cache,        // [num_pages, 2, hkv, page_size, d]
    T* __restrict__ out,                // [tokens, hq, d]
    const int* __restrict__ positions,  // [tokens]
    const int* __restrict__ token_slot, // [tokens]
    const int* __restrict__ block_table,  // [slots, max_pages]
    int tokens, int hq, int hkv, int d, int page_size, int num_pages, int max_pages, int slots,
    int window, float scale, int* __restrict__ fault) {
  __shared__ float q_staged[kGenericWarps][kGenericMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * kGenericWarps + warp;
  if (item >= static_cast<long long>(tokens) * hq) return;
  const int t = static_cast<int>(item / hq);
  const int head = static_cast<int>(item - static_cast<long long>(t) * hq);
  const int kv_head = head / (hq / hkv);
  const int pos = positions[t];
  const int slot = token_slot[t];
  T* o = out + (static_cast<size_t>(t) * hq + head) * d;
  if (slot < 0 || slot >= slots || pos < 0 || pos >= max_pages * page_size) {
    if (lane == 0) atomicOr(fault, slot < 0 || slot >= slots ? kFaultSlot : kFaultPosition);
    for (int i = lane; i < d; i += 32) o[i] = from_float<T>(0.0f);
    return;
  }
  const int* table = block_table + static_cast<size_t>(slot) * max_pages;

  float* qs = q_staged[warp];
  const T* qr = q + (static_cast<size_t>(t) * hq + head) * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_float(qr[i]) * scale;
  __syncwarp();

  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const size_t head_stride = static_cast<size_t>(page_size) * d;
  const size_t v_offset = static_cast<size_t>(hkv) * head_stride;  // K plane -> V plane

  float running_max = -INFINITY, running_sum = 0.0f;
  float acc[kGenericMaxD / 32];
#pragma unroll
  for (int i = 0; i < kGenericMaxD / 32; ++i) acc[i] = 0.0f;

  for (int base = first; base <= pos; base += 32) {
    const int j = base + lane;
    const bool valid = j <= pos;
    long long k_row = -1;  // element offset of key row j in the cache
    float score = -INFINITY;
    if (valid) {
      const int page = table[j / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(fault, kFaultPageId);
      } else {
        k_row = static_cast<long long>(
            ((static_cast<size_t>(page) * 2 * hkv + kv_head) * page_size + (j % page_size)) * d);
        const T* kr = cache + k_row;
        float dot = 0.0f;
        for (int i = 0; i < d; i += 8) {
          float kv[8];
          load8(kr + i, kv);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(qs[i + e], kv[e], dot);
        }
        score = dot;
      }
    }
    const float chunk_max = warp_max(score);
    const float new_max = fmaxf(running_max, chunk_max);
    if (new_max == -INFINITY) continue;  // every key of this chunk was unreadable
    const float p = (k_row >= 0) ? expf(score - new_max) : 0.0f;
    const float correction = expf(running_max - new_max);
    running_sum = running_sum * correction + warp_sum(p);
    running_max = new_max;
#pragma unroll
    for (int i = 0; i < kGenericMaxD / 32; ++i) acc[i] *= correction;
    const int count = min(32, pos - base + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long row = __shfl_sync(0xffffffffu, k_row, jj);
      if (row < 0) continue;
      const T* vr = cache + row + v_offset;
#pragma unroll
      for (int i = 0; i < kGenericMaxD / 32; ++i) {
        const int col = lane + 32 * i;
        if (col < d) acc[i] = fmaf(pj, to_float(vr[col]), acc[i]);
      }
    }
  }
  const float inv_sum = running_sum > 0.0f ? 1.0f / running_sum : 0.0f;
#pragma unroll
  for (int i = 0; i < kGenericMaxD / 32; ++i) {
    const int col = lane + 32 * i;
    if (col < d) o[col] = from_float<T>(acc[i] * inv_sum);
  }
}

}  // namespace rl

extern "C" int rl_attention_generic(int dtype, const void* q, const void* cache, void* out,
                                    const int* positions, const int* token_slot,
                                    const int* block_table, int tokens, int hq, int hkv, int d,
                                    int page_size, int num_pages, int max_pages, int slots,
                                    int window, float scale, int* fault, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (d <= 0 || d % 16 != 0 || d > rl::kGenericMaxD || hkv <= 0 || hq % hkv != 0 ||
      page_size <= 0 || window < 0)
    return static_cast<int>(cudaErrorInvalidValue);
  const long long items = static_cast<long long>(tokens) * hq;
  const unsigned blocks =
      static_cast<unsigned>((items + rl::kGenericWarps - 1) / rl::kGenericWarps);
  RL_DISPATCH_DTYPE(dtype, {
    rl::attention_generic_kernel<scalar_t><<<blocks, rl::kGenericWarps * 32, 0, stream>>>(
        static_cast<const scalar_t*>(q), static_cast<const scalar_t*>(cache),
        static_cast<scalar_t*>(out), positions, token_slot, block_table, tokens, hq, hkv, d,
        page_size, num_pages, max_pages, slots, window, scale, fault);
  });
  return rl::launch_status();
}

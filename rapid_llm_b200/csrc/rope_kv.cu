// Per-head q/k RMSNorm + rotary position encoding + K/V page write, one pass over the
// output of the fused QKV product.
//
// The reference does this in three launches with two extra round trips of q and k:
// qk_rmsnorm (rapid_llm/kernels/ops/layernorm/skip_rmsnorm.py:166-194), the half-split
// rotation (rapid_llm/kernels/ops/rope/rope_emb.py:47-81; pairs (i, i + R/2), out =
// [x1*c - x2*s, x2*c + x1*s]) and the cache scatter
// (rapid_llm/kernels/ops/kvcache/update_kv_buffer.py:16-73).  Norm statistics, the
// rotation and its angles' cos/sin (a float32 table) are 32-bit here in both precisions.
//
// Cache layout of one layer: [num_pages, 2 (K, V), kv_heads, page_size, head_dim].
#include "common.cuh"

namespace rl {

constexpr int kRopeWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__global__ void qk_norm_rope_write_kernel(
    const T* __restrict__ qkv,          // [tokens, row_width]: q heads, then k heads, then v heads
    const float* __restrict__ bias,     // [(hq + 2 hkv) * d] or null
    const float* __restrict__ q_weight, // [d] or null (no q/k norm)
    const float* __restrict__ k_weight, // [d] or null
    const float* __restrict__ cos_table,  // [max_pos, rotary/2]
    const float* __restrict__ sin_table,
    const int* __restrict__ positions,  // [tokens]
    const int* __restrict__ kv_dest,    // [tokens] page * page_size + offset, or null (q only)
    T* __restrict__ q_out,              // [tokens, hq, d]
    T* __restrict__ cache,              // layer cache or null
    int tokens, int row_width, int hq, int hkv, int d, int rotary, int max_pos, int page_size,
    int num_pages, float eps, int* __restrict__ fault) {
  __shared__ float staged[kRopeWarps][kMaxHeadDim];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_per_token = kv_dest ? hq + 2 * hkv : hq;
  const long long item = static_cast<long long>(blockIdx.x) * kRopeWarps + warp;
  if (item >= static_cast<long long>(tokens) * heads_per_token) return;
  const int t = static_cast<int>(item / heads_per_token);
  const int head = static_cast<int>(item - static_cast<long long>(t) * heads_per_token);
  const T* src = qkv + static_cast<size_t>(t) * row_width + static_cast<size_t>(head) * d;
  const float* b = bias ? bias + static_cast<size_t>(head) * d : nullptr;

  // 0 = q, 1 = k, 2 = v
  const int kind = head < hq ? 0 : (head < hq + hkv ? 1 : 2);
  T* dst = nullptr;
  if (kind == 0) {
    dst = q_out + (static_cast<size_t>(t) * hq + head) * d;
  } else {
    const int kv_head = kind == 1 ? head - hq : head - hq - hkv;
    const int dest = kv_dest[t];
    const int page = dest / page_size, offset = dest - page * page_size;
    if (dest < 0 || page >= num_pages) {
      if (lane == 0) atomicOr(fault, kFaultPageId);
      return;
    }
    dst = cache +
          ((((static_cast<size_t>(page) * 2 + (kind - 1)) * hkv + kv_head) * page_size) + offset) * d;
  }

  float* mine = staged[warp];
  float sum_sq = 0.0f;
  for (int i = lane; i < d; i += 32) {
    float v = to_float(src[i]);
    if (b) v += b[i];
    mine[i] = v;
    sum_sq += v * v;
  }
  if (kind == 2) {
    __syncwarp();
    for (int i = lane; i < d; i += 32) dst[i] = from_float<T>(mine[i]);
    return;
  }
  const float* w = kind == 0 ? q_weight : k_weight;
  if (w) {
    sum_sq = warp_sum(sum_sq);
    const float inv_rms = rsqrtf(sum_sq / static_cast<float>(d) + eps);
    for (int i = lane; i < d; i += 32) mine[i] = mine[i] * inv_rms * w[i];
  }
  __syncwarp();
  int pos = positions[t];
  if (pos < 0 || pos >= max_pos) {
    if (lane == 0) atomicOr(fault, kFaultPosition);
    pos = 0;
  }
  const int half = rotary >> 1;
  const float* c = cos_table + static_cast<size_t>(pos) * half;
  const float* s = sin_table + static_cast<size_t>(pos) * half;
  for (int i = lane; i < d; i += 32) {
    float v;
    if (i < half) {
      v = mine[i] * c[i] - mine[i + half] * s[i];
    } else if (i < rotary) {
      v = mine[i] * c[i - half] + mine[i - half] * s[i - half];
    } else {
      v = mine[i];
    }
    dst[i] = from_float<T>(v);
  }
}

}  // namespace rl

extern "C" int rl_qk_norm_rope_write(int dtype, const void* qkv, int row_width, const float* bias,
                                     const float* q_weight, const float* k_weight,
                                     const float* cos_table, const float* sin_table,
                                     const int* positions, const int* kv_dest, void* q_out,
                                     void* cache, int tokens, int hq, int hkv, int d, int rotary,
                                     int max_pos, int page_size, int num_pages, float eps,
                                     int* fault, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (d > rl::kMaxHeadDim || d <= 0 || rotary < 0 || rotary > d || (rotary & 1) ||
      (kv_dest != nullptr && cache == nullptr))
    return static_cast<int>(cudaErrorInvalidValue);
  const long long items =
      static_cast<long long>(tokens) * (kv_dest ? hq + 2 * hkv : hq);
  const unsigned blocks = static_cast<unsigned>((items + rl::kRopeWarps - 1) / rl::kRopeWarps);
  RL_DISPATCH_DTYPE(dtype, {
    rl::qk_norm_rope_write_kernel<scalar_t><<<blocks, rl::kRopeWarps * 32, 0, stream>>>(
        static_cast<const scalar_t*>(qkv), bias, q_weight, k_weight, cos_table, sin_table,
        positions, kv_dest, static_cast<scalar_t*>(q_out), static_cast<scalar_t*>(cache), tokens,
        row_width, hq, hkv, d, rotary, max_pos, page_size, num_pages, eps, fault);
  });
  return rl::launch_status();
}

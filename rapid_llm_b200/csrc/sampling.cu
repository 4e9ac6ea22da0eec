// Next-token selection over [rows, vocab] logits: repetition penalty, greedy argmax,
// temperature softmax, nucleus (top-p) cut and a seeded draw, one block per row.
//
// Semantics follow rapid_llm/engine/sampler.py: the penalty divides positive and multiplies
// negative logits of tokens already generated, once per distinct token (:134-179); greedy is
// the first index of the maximum (:266-283); otherwise softmax(logits / T) in float32
// (:669-672), tokens kept while the probability mass ranked before them does not exceed
// top_p (:223-244), and one draw from the kept mass.  Two things differ by design: the
// nucleus is taken over the whole vocabulary instead of a 1024-wide pool, and the draw
// comes from a counter-based generator keyed by (seed, counter) per row, so a request's
// tokens do not depend on what else is in the batch (the reference draws from the global
// generator and has no seed).
#include "common.cuh"

namespace rl {

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c[0];
  const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c[2];
  const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k0;
  const uint32_t n1 = static_cast<uint32_t>(p1);
  const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k1;
  const uint32_t n3 = static_cast<uint32_t>(p0);
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

// Philox4x32-10 keyed by the 64-bit seed, counter = (counter, 0, 0, 0); first output word
// mapped to [0, 1) with 24 bits.
__device__ __forceinline__ float philox_uniform(unsigned long long seed, uint32_t counter) {
  uint32_t c[4] = {counter, 0u, 0u, 0u};
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return static_cast<float>(c[0] >> 8) * (1.0f / 16777216.0f);
}

struct MaxIndex {
  float value;
  int index;
};

__device__ __forceinline__ MaxIndex better(MaxIndex a, MaxIndex b) {
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}

__device__ __forceinline__ MaxIndex block_argmax(MaxIndex v, float* fscratch, int* iscratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    MaxIndex o;
    o.value = __shfl_xor_sync(0xffffffffu, v.value, offset);
    o.index = __shfl_xor_sync(0xffffffffu, v.index, offset);
    v = better(v, o);
  }
  __syncthreads();
  if (lane == 0) {
    fscratch[warp] = v.value;
    iscratch[warp] = v.index;
  }
  __syncthreads();
  MaxIndex r;
  r.value = lane < warps ? fscratch[lane] : -INFINITY;
  r.index = lane < warps ? iscratch[lane] : 0x7fffffff;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    MaxIndex o;
    o.value = __shfl_xor_sync(0xffffffffu, r.value, offset);
    o.index = __shfl_xor_sync(0xffffffffu, r.index, offset);
    r = better(r, o);
  }
  return r;
}

template <typename T>
__global__ void __launch_bounds__(1024)
sample_kernel(const T* __restrict__ logits, int vocab, long long row_stride,
              const float* __restrict__ temperature,      // [rows] or null = all greedy
              const float* __restrict__ top_p,            // [rows] or null = 1
              const float* __restrict__ penalty,          // [rows] or null = 1
              const unsigned long long* __restrict__ seeds,  // [rows] (with temperature)
              const int* __restrict__ counters,           // [rows] (with temperature)
              const int* __restrict__ seen_tokens,        // ragged generated tokens or null
              const int* __restrict__ seen_offsets,       // [rows + 1]
              int* __restrict__ out) {
  extern __shared__ unsigned seen_bits[];  // ceil(vocab / 32) words when a penalty applies
  __shared__ float fscratch[32];
  __shared__ int iscratch[32];
  __shared__ float warp_totals[32];
  pdl_trigger();
  const int row = blockIdx.x;
  const T* x = logits + static_cast<size_t>(row) * row_stride;
  pdl_wait();
  const float temp = temperature ? temperature[row] : 0.0f;
  const float pen = penalty ? penalty[row] : 1.0f;
  const int seen_begin = seen_offsets ? seen_offsets[row] : 0;
  const int seen_end = seen_offsets ? seen_offsets[row + 1] : 0;
  const bool has_pen = pen != 1.0f && seen_tokens != nullptr && seen_end > seen_begin;
  if (has_pen) {
    const int words = (vocab + 31) >> 5;
    for (int i = threadIdx.x; i < words; i += blockDim.x) seen_bits[i] = 0u;
    __syncthreads();
    for (int i = seen_begin + threadIdx.x; i < seen_end; i += blockDim.x) {
      const int id = seen_tokens[i];
      if (id >= 0 && id < vocab) atomicOr(&seen_bits[id >> 5], 1u << (id & 31));
    }
    __syncthreads();
  }
  auto value = [&](int i) -> float {
    float v = to_float(x[i]);
    if (has_pen && ((seen_bits[i >> 5] >> (i & 31)) & 1u)) v = v < 0.0f ? v * pen : v / pen;
    return v;
  };

  // Greedy pick: needed for greedy rows and as the fallback of the draw.
  MaxIndex best{-INFINITY, 0x7fffffff};
  // rows that start on a 16-byte boundary are read eight elements at a time; a thread still
  // meets its indices in rising order, so its strict comparison keeps the first maximum
  const bool vector = (reinterpret_cast<uintptr_t>(x) & (sizeof(T) == 2 ? 15 : 31)) == 0;
  const int vector_end = vector ? (vocab & ~7) : 0;
  for (int c = threadIdx.x * 8; c < vector_end; c += blockDim.x * 8) {
    float v[8];
    load8(x + c, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float e = v[j];
      if (has_pen && ((seen_bits[(c + j) >> 5] >> ((c + j) & 31)) & 1u)) e = e < 0.0f ? e * pen : e / pen;
      if (e > best.value) {
        best.value = e;
        best.index = c + j;
      }
    }
  }
  for (int i = vector_end + threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = value(i);
    if (v > best.value) {
      best.value = v;
      best.index = i;
    }
  }
  best = block_argmax(best, fscratch, iscratch);
  if (best.index < 0 || best.index >= vocab) best.index = 0;  // all -inf or NaN
  if (temp <= 0.0f) {
    if (threadIdx.x == 0) out[row] = best.index;
    return;
  }

  const float inv_t = 1.0f / temp;
  const float peak = best.value * inv_t;
  float z = 0.0f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) z += expf(value(i) * inv_t - peak);
  z = block_sum(z, fscratch);

  float threshold = 0.0f;
  const float p = top_p ? top_p[row] : 1.0f;
  if (p < 1.0f) {
    // Smallest e* with (mass of tokens whose weight exceeds e*) <= p * Z; kept = weight >= e*.
    const float budget = p * z;
    unsigned lo = 0u, hi = __float_as_uint(1.0f);
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1);
      const float cut = __uint_as_float(mid);
      float above = 0.0f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float e = expf(value(i) * inv_t - peak);
        if (e > cut) above += e;
      }
      above = block_sum(above, fscratch);
      if (above <= budget) hi = mid; else lo = mid + 1u;
    }
    threshold = __uint_as_float(lo);
  }

  // Draw by inverse CDF in index order over the kept weights.  Thread t owns a
  // contiguous range, so the prefix sums tile [0, total) exactly.
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(vocab, static_cast<int>(threadIdx.x) * chunk);
  const int end = min(vocab, begin + chunk);
  float local = 0.0f;
  for (int i = begin; i < end; ++i) {
    const float e = expf(value(i) * inv_t - peak);
    if (e >= threshold) local += e;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  float inclusive = local;
#pragma unroll
  for (int offset = 1; offset < 32; offset <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, inclusive, offset);
    if (lane >= offset) inclusive += up;
  }
  __syncthreads();
  if (lane == 31) warp_totals[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    float total = lane < warps ? warp_totals[lane] : 0.0f;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, total, offset);
      if (lane >= offset) total += up;
    }
    warp_totals[lane] = total;  // inclusive over warps
  }
  __syncthreads();
  const float warp_base = warp == 0 ? 0.0f : warp_totals[warp - 1];
  const float upto = warp_base + inclusive;                       // inclusive prefix of this thread
  float before = __shfl_up_sync(0xffffffffu, upto, 1);            // = prefix of the next thread
  if (lane == 0) before = warp_base;
  const float total = warp_totals[warps - 1];
  const float u = philox_uniform(seeds[row], static_cast<uint32_t>(counters[row]));
  const float target = u * total;
  if (threadIdx.x == 0) out[row] = best.index;
  __syncthreads();
  if (local > 0.0f && before <= target && target < upto) {
    float running = before;
    int pick = -1;
    for (int i = begin; i < end; ++i) {
      const float e = expf(value(i) * inv_t - peak);
      if (e >= threshold) {
        running += e;
        pick = i;
        if (target < running) break;
      }
    }
    if (pick >= 0) out[row] = pick;
  }
}

}  // namespace rl

// logits: [rows, vocab] of `dtype` with `row_stride` elements between rows.  Null
// `temperature` makes every row greedy.  `seen_tokens`/`seen_offsets` list, per row, the
// tokens the request has generated so far (for the repetition penalty) and may be null.
extern "C" int rl_sample(int dtype, const void* logits, int rows, int vocab, long long row_stride,
                         const float* temperature, const float* top_p, const float* penalty,
                         const unsigned long long* seeds, const int* counters,
                         const int* seen_tokens, const int* seen_offsets, int* out, int pdl,
                         cudaStream_t stream) {
  if (rows == 0) return 0;
  if (vocab <= 0 || (temperature != nullptr && (seeds == nullptr || counters == nullptr)))
    return static_cast<int>(cudaErrorInvalidValue);
  const size_t smem = (penalty && seen_tokens) ? static_cast<size_t>((vocab + 31) / 32) * 4 : 0;
  if (smem > 200 * 1024) return static_cast<int>(cudaErrorInvalidValue);
  const int threads = vocab >= 8192 ? 1024 : 256;
  RL_DISPATCH_DTYPE(dtype, {
    auto kernel = rl::sample_kernel<scalar_t>;
    if (smem > 40 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    return rl::launch_kernel(kernel, dim3(rows), dim3(threads), smem, stream, pdl != 0,
                             static_cast<const scalar_t*>(logits), vocab, row_stride, temperature, top_p,
                             penalty, seeds, counters, seen_tokens, seen_offsets, out);
  });
  return 0;
}

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

constexpr int kCuts = 15;     // thresholds tried per sweep of the nucleus search (a 16-way split)

// Sums of kCuts values over the block, every thread gets all of them; the tree is fixed.
__device__ __forceinline__ void block_sum_many(float (&v)[kCuts], float (*scratch)[kCuts]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int k = 0; k < kCuts; ++k) v[k] = warp_sum(v[k]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < kCuts; ++k) scratch[warp][k] = v[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kCuts; ++k) {
    float total = 0.0f;
    for (int w = 0; w < warps; ++w) total += scratch[w][k];
    v[k] = total;
  }
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
  __shared__ float many_scratch[32][kCuts];
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
  auto adjust = [&](float v, int i) -> float {
    if (has_pen && ((seen_bits[i >> 5] >> (i & 31)) & 1u)) v = v < 0.0f ? v * pen : v / pen;
    return v;
  };
  // Every sweep over the row: rows that start on a 16-byte boundary are read eight elements at
  // a time (thread t takes elements 8 t .. 8 t + 7, then 8 (t + threads) ..., in rising order),
  // the rest element by element.  fn(index, value) sees each element once.
  const bool vector = (reinterpret_cast<uintptr_t>(x) & (sizeof(T) == 2 ? 15 : 31)) == 0;
  const int vector_end = vector ? (vocab & ~7) : 0;
  auto sweep = [&](auto&& fn) {
    for (int c = threadIdx.x * 8; c < vector_end; c += blockDim.x * 8) {
      float v[8];
      load8(x + c, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) fn(c + j, adjust(v[j], c + j));
    }
    for (int i = vector_end + threadIdx.x; i < vocab; i += blockDim.x) fn(i, adjust(to_float(x[i]), i));
  };

  // Greedy pick: needed for greedy rows and as the fallback of the draw.  A thread meets its
  // indices in rising order, so its strict comparison keeps the first maximum.
  MaxIndex best{-INFINITY, 0x7fffffff};
  sweep([&](int i, float v) {
    if (v > best.value) {
      best.value = v;
      best.index = i;
    }
  });
  best = block_argmax(best, fscratch, iscratch);
  if (best.index < 0 || best.index >= vocab) best.index = 0;  // all -inf or NaN
  if (temp <= 0.0f) {
    if (threadIdx.x == 0) out[row] = best.index;
    return;
  }

  const float inv_t = 1.0f / temp;
  const float peak = best.value * inv_t;
  float z = 0.0f;
  sweep([&](int, float v) { z += expf(v * inv_t - peak); });
  z = block_sum(z, fscratch);

  float threshold = 0.0f;
  const float p = top_p ? top_p[row] : 1.0f;
  if (p < 1.0f) {
    // Smallest e* with (mass of tokens whose weight exceeds e*) <= p * Z; kept = weight >= e*.
    // The mass above a cut falls as the cut rises, so the search over the cut's bit pattern
    // tries kCuts cuts per sweep and keeps the sixteenth of the range that holds e*.
    const float budget = p * z;
    unsigned lo = 0u, hi = __float_as_uint(1.0f);
    while (lo < hi) {
      const unsigned width = hi - lo;
      unsigned cut_bits[kCuts];
      float cut[kCuts], above[kCuts];
#pragma unroll
      for (int k = 0; k < kCuts; ++k) {
        // distinct and rising while width >= 16; for narrow ranges some repeat, which is harmless
        cut_bits[k] = lo + static_cast<unsigned>((static_cast<unsigned long long>(width) * (k + 1)) >> 4);
        if (cut_bits[k] >= hi) cut_bits[k] = hi - 1;
        cut[k] = __uint_as_float(cut_bits[k]);
        above[k] = 0.0f;
      }
      sweep([&](int, float v) {
        const float e = expf(v * inv_t - peak);
#pragma unroll
        for (int k = 0; k < kCuts; ++k)
          if (e > cut[k]) above[k] += e;
      });
      block_sum_many(above, many_scratch);
      // the first cut that satisfies the budget bounds e* from above, the one before from below
      unsigned new_lo = cut_bits[kCuts - 1] + 1u, new_hi = hi;
#pragma unroll
      for (int k = kCuts - 1; k >= 0; --k) {
        if (above[k] <= budget) {
          new_hi = cut_bits[k];
          new_lo = k > 0 ? cut_bits[k - 1] + 1u : lo;
        }
      }
      if (new_lo > new_hi) new_lo = new_hi;
      lo = new_lo;
      hi = new_hi;
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
    const float e = expf(adjust(to_float(x[i]), i) * inv_t - peak);
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
      const float e = expf(adjust(to_float(x[i]), i) * inv_t - peak);
      if (e >= threshold) {
        running += e;
        pick = i;
        if (target < running) break;
      }
    }
    if (pick >= 0) out[row] = pick;
  }
}

// ------------------------------------------------------------------------------------------
// The same selection with a row spread over a thread-block cluster: each CTA keeps its slice of
// the row's (penalised) values in shared memory, so the row is read from global memory once,
// exponentials are taken once, and the sweeps of the nucleus search run over shared memory on
// kSampleCluster SMs instead of one.  Sums and maxima are combined over the cluster through
// distributed shared memory in rank order, so the result does not depend on timing.
constexpr int kSampleCluster = 8;
constexpr int kSampleThreads = 512;
constexpr int kSampleMaxSlice = 48 * 1024;      // floats of one CTA's slice (192 KB)

__device__ __forceinline__ void sample_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\n barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ float sample_peer_f32(const float* local, unsigned rank) {
  unsigned address = static_cast<unsigned>(__cvta_generic_to_shared(local)), remote;
  float value;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(address), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(value) : "r"(remote) : "memory");
  return value;
}

// (two CTAs a multiprocessor where the slice allows it: a cluster lives inside one GPC, only 15 clusters of 8 run at
// one time with one CTA per multiprocessor, and a batch of 64 rows then took five rounds)
template <typename T>
__global__ void __launch_bounds__(kSampleThreads, 2)
sample_cluster_kernel(const T* __restrict__ logits, int vocab, long long row_stride, int slice,
                      const float* __restrict__ temperature, const float* __restrict__ top_p,
                      const float* __restrict__ penalty, const unsigned long long* __restrict__ seeds,
                      const int* __restrict__ counters, const int* __restrict__ seen_tokens,
                      const int* __restrict__ seen_offsets, int* __restrict__ out) {
  extern __shared__ float slice_values[];          // [slice]
  __shared__ float fscratch[32];
  __shared__ int iscratch[32];
  __shared__ float many_scratch[32][kCuts];
  __shared__ float warp_totals[32];
  __shared__ float share_f[2][kCuts + 1];          // this CTA's partial sums, read by its peers
  __shared__ float gathered[kCuts + 1];            // the cluster's sums, fetched by a few threads for all
  __shared__ int share_i;
  pdl_trigger();
  const int row = blockIdx.y;
  const unsigned rank = blockIdx.x;                // cluster = the x dimension
  const T* x = logits + static_cast<size_t>(row) * row_stride;
  const int begin = min(vocab, static_cast<int>(rank) * slice), end = min(vocab, begin + slice);
  const int count = end - begin;
  pdl_wait();
  const float temp = temperature ? temperature[row] : 0.0f;
  const float pen = penalty ? penalty[row] : 1.0f;
  const int seen_begin = seen_offsets ? seen_offsets[row] : 0;
  const int seen_end = seen_offsets ? seen_offsets[row + 1] : 0;
  const bool has_pen = pen != 1.0f && seen_tokens != nullptr && seen_end > seen_begin;

  // the slice, as float; slices start on multiples of 8 elements, so an aligned row reads 16 bytes a time
  const bool vector = (reinterpret_cast<uintptr_t>(x) & (sizeof(T) == 2 ? 15 : 31)) == 0;
  const int vector_count = vector ? (count & ~7) : 0;
  for (int c = threadIdx.x * 8; c < vector_count; c += blockDim.x * 8) {
    float v[8];
    load8(x + begin + c, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) slice_values[c + j] = v[j];
  }
  for (int i = vector_count + threadIdx.x; i < count; i += blockDim.x) slice_values[i] = to_float(x[begin + i]);
  __syncthreads();
  if (has_pen) {
    // every generated token once: the first of equal ids in the list applies the penalty
    for (int i = seen_begin + threadIdx.x; i < seen_end; i += blockDim.x) {
      const int id = seen_tokens[i];
      if (id < begin || id >= end) continue;
      bool first = true;
      for (int j = seen_begin; j < i && first; ++j) first = seen_tokens[j] != id;
      if (first) {
        const float v = slice_values[id - begin];
        slice_values[id - begin] = v < 0.0f ? v * pen : v / pen;
      }
    }
    __syncthreads();
  }

  // over the cluster: partial results go to share_f / share_i, every CTA reads all ranks
  int round = 0;
  auto cluster_sum = [&](float mine) {
    const int slot = round++ & 1;
    if (threadIdx.x == 0) share_f[slot][0] = mine;
    sample_cluster_sync();
    if (threadIdx.x == 0) {                          // remote reads are slow: one thread does them for all
      float total = 0.0f;
      for (unsigned r = 0; r < kSampleCluster; ++r) total += sample_peer_f32(&share_f[slot][0], r);
      gathered[0] = total;
    }
    __syncthreads();
    const float total = gathered[0];
    __syncthreads();
    return total;
  };

  // ---- the first maximum ---------------------------------------------------------------
  MaxIndex best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    const float v = slice_values[i];
    if (v > best.value) {
      best.value = v;
      best.index = begin + i;
    }
  }
  best = block_argmax(best, fscratch, iscratch);
  {
    const int slot = round++ & 1;
    if (threadIdx.x == 0) {
      share_f[slot][0] = best.value;
      share_i = best.index;
    }
    sample_cluster_sync();
    MaxIndex all{-INFINITY, 0x7fffffff};
    for (unsigned r = 0; r < kSampleCluster; ++r) {
      MaxIndex theirs;
      theirs.value = sample_peer_f32(&share_f[slot][0], r);
      theirs.index = __float_as_int(sample_peer_f32(reinterpret_cast<const float*>(&share_i), r));
      all = better(all, theirs);
    }
    best = all;
    sample_cluster_sync();                           // share_i may be rewritten only after every read
  }
  if (best.index < 0 || best.index >= vocab) best.index = 0;
  if (temp <= 0.0f) {
    if (rank == 0 && threadIdx.x == 0) out[row] = best.index;
    return;                                          // the whole cluster takes this branch
  }

  // ---- weights, their sum, the nucleus -----------------------------------------------------
  const float inv_t = 1.0f / temp;
  const float peak = best.value * inv_t;
  float z = 0.0f;
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    const float e = expf(slice_values[i] * inv_t - peak);
    slice_values[i] = e;
    z += e;
  }
  z = cluster_sum(block_sum(z, fscratch));

  float threshold = 0.0f;
  const float p = top_p ? top_p[row] : 1.0f;
  if (p < 1.0f) {
    const float budget = p * z;
    unsigned lo = 0u, hi = __float_as_uint(1.0f);
    while (lo < hi) {
      const unsigned width = hi - lo;
      unsigned cut_bits[kCuts];
      float cut[kCuts], above[kCuts];
#pragma unroll
      for (int k = 0; k < kCuts; ++k) {
        cut_bits[k] = lo + static_cast<unsigned>((static_cast<unsigned long long>(width) * (k + 1)) >> 4);
        if (cut_bits[k] >= hi) cut_bits[k] = hi - 1;
        cut[k] = __uint_as_float(cut_bits[k]);
        above[k] = 0.0f;
      }
      for (int i = threadIdx.x; i < count; i += blockDim.x) {
        const float e = slice_values[i];
#pragma unroll
        for (int k = 0; k < kCuts; ++k)
          if (e > cut[k]) above[k] += e;
      }
      block_sum_many(above, many_scratch);
      const int slot = round++ & 1;
      if (threadIdx.x == 0) {
#pragma unroll
        for (int k = 0; k < kCuts; ++k) share_f[slot][k] = above[k];
      }
      sample_cluster_sync();
      if (threadIdx.x < kCuts) {
        float total = 0.0f;
        for (unsigned r = 0; r < kSampleCluster; ++r) total += sample_peer_f32(&share_f[slot][threadIdx.x], r);
        gathered[threadIdx.x] = total;
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < kCuts; ++k) above[k] = gathered[k];
      __syncthreads();
      unsigned new_lo = cut_bits[kCuts - 1] + 1u, new_hi = hi;
#pragma unroll
      for (int k = kCuts - 1; k >= 0; --k) {
        if (above[k] <= budget) {
          new_hi = cut_bits[k];
          new_lo = k > 0 ? cut_bits[k - 1] + 1u : lo;
        }
      }
      if (new_lo > new_hi) new_lo = new_hi;
      lo = new_lo;
      hi = new_hi;
    }
    threshold = __uint_as_float(lo);
  }

  // ---- the draw: inverse CDF in index order over the kept weights ----------------------------
  const int chunk = (count + blockDim.x - 1) / blockDim.x;
  const int my_begin = min(count, static_cast<int>(threadIdx.x) * chunk), my_end = min(count, my_begin + chunk);
  float local = 0.0f;
  for (int i = my_begin; i < my_end; ++i) {
    const float e = slice_values[i];
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
  // the CTAs' kept sums, in rank order: what lies before this CTA, and the whole
  const int slot = round++ & 1;
  if (threadIdx.x == 0) share_f[slot][0] = warp_totals[warps - 1];
  sample_cluster_sync();
  float cta_base = 0.0f, total = 0.0f;
  for (unsigned r = 0; r < kSampleCluster; ++r) {
    const float theirs = sample_peer_f32(&share_f[slot][0], r);
    if (r < rank) cta_base += theirs;
    total += theirs;
  }
  const float warp_base = cta_base + (warp == 0 ? 0.0f : warp_totals[warp - 1]);
  const float upto = warp_base + inclusive;
  float before = __shfl_up_sync(0xffffffffu, upto, 1);
  if (lane == 0) before = warp_base;
  const float u = philox_uniform(seeds[row], static_cast<uint32_t>(counters[row]));
  const float target = u * total;
  if (rank == 0 && threadIdx.x == 0) out[row] = best.index;    // stands if rounding leaves the target uncovered
  sample_cluster_sync();                                         // ... and is overwritten only after it is written
  if (local > 0.0f && before <= target && target < upto) {
    float running = before;
    int pick = -1;
    for (int i = my_begin; i < my_end; ++i) {
      const float e = slice_values[i];
      if (e >= threshold) {
        running += e;
        pick = begin + i;
        if (target < running) break;
      }
    }
    if (pick >= 0) out[row] = pick;
  }
  sample_cluster_sync();                                         // nobody leaves while its shared memory may be read
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
  if (temperature != nullptr) {
    // rows that may draw: the row spread over a cluster, its values kept in shared memory
    const int slice = ((vocab + rl::kSampleCluster - 1) / rl::kSampleCluster + 7) & ~7;
    if (slice <= rl::kSampleMaxSlice) {
      const size_t bytes = static_cast<size_t>(slice) * sizeof(float);
      cudaLaunchConfig_t config = {};
      config.gridDim = dim3(rl::kSampleCluster, rows);
      config.blockDim = dim3(rl::kSampleThreads);
      config.dynamicSmemBytes = bytes;
      config.stream = stream;
      cudaLaunchAttribute attributes[2];
      attributes[0].id = cudaLaunchAttributeClusterDimension;
      attributes[0].val.clusterDim.x = rl::kSampleCluster;
      attributes[0].val.clusterDim.y = 1;
      attributes[0].val.clusterDim.z = 1;
      attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attributes[1].val.programmaticStreamSerializationAllowed = 1;
      config.attrs = attributes;
      config.numAttrs = pdl ? 2 : 1;
      RL_DISPATCH_DTYPE(dtype, {
        auto kernel = rl::sample_cluster_kernel<scalar_t>;
        if (bytes > 40 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(bytes));
          if (e != cudaSuccess) return static_cast<int>(e);
        }
        return static_cast<int>(cudaLaunchKernelEx(&config, kernel, static_cast<const scalar_t*>(logits), vocab,
                                                   row_stride, slice, temperature, top_p, penalty, seeds, counters,
                                                   seen_tokens, seen_offsets, out));
      });
    }
  }
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

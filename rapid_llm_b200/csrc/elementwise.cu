// Embedding gather, residual-add + RMSNorm, SiLU(gate)*up.
//
// The reference runs these as a library gather (rapid_llm/modules/vocab_parallel.py:101-103),
// Triton row kernels (rapid_llm/kernels/ops/layernorm/skip_rmsnorm.py:22-85,197-240) and a
// Triton SwiGLU kernel (rapid_llm/kernels/ops/activation/swiglu.py:91-121).  Here the
// residual stream is a float32 buffer in both engine precisions: the sum x + r is formed
// and kept in 32-bit, and the norm's statistics, scaling and weight product are 32-bit
// with one rounding at the store.
//
// Rows whose length is a multiple of 8 move in 16- and 32-byte accesses; other lengths take
// the element-by-element path of the same kernel.  The order of every sum is fixed by the
// row length and the block size alone, so a row's result does not depend on the batch.
#include "common.cuh"

namespace rl {

__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// ---------------------------------------------------------------- embedding
// An id -(r + 1) stands for "the token in feedback[r]": the id the previous step sampled into
// row r of its result, which the host may not have read yet.
template <typename T>
__global__ void embedding_kernel(T* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, const int* __restrict__ feedback,
                                 int feedback_rows, int hidden, int vocab, int* __restrict__ fault) {
  pdl_trigger();
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 && feedback != nullptr && -(id + 1) < feedback_rows) id = feedback[-(id + 1)];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(fault, kFaultTokenId);
    id = 0;
  }
  const T* src = table + static_cast<size_t>(id) * hidden;
  T* dst = out + static_cast<size_t>(row) * hidden;
  constexpr int kVec = 16 / sizeof(T);
  pdl_wait();   // the output buffer may still be read by the previous step's kernels
  if (hidden % kVec == 0) {
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < hidden / kVec; i += blockDim.x) d[i] = s[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
  }
}

// ------------------------------------------------------------ add + RMSNorm
// One block per output row.  Row i of the output reads input row `row_index[i]`
// (or i when row_index is null).
//   mode 0: r = x                 (first layer: the residual stream starts here)
//   mode 1: r = x + residual
//   mode 2: r = x, residual untouched and may be null (a plain norm)
// With `write_residual` the sum is stored back to `residual` (float32).
// out = r * rsqrt(mean(r^2) + eps) * weight, all in float32, rounded once.
//
// kVector: hidden is a multiple of 8 and the block has at least hidden / 8 threads; a thread
// keeps its eight values (and the weights, fetched before the sum) in registers.
template <typename TX, typename TOut, bool kVector>
__global__ void add_rmsnorm_kernel(const TX* __restrict__ x, float* __restrict__ residual,
                                   const float* __restrict__ weight, TOut* __restrict__ out,
                                   const int* __restrict__ row_index, int hidden, float eps,
                                   int mode, int write_residual) {
  extern __shared__ float row_values[];  // [hidden] on the element-by-element path
  __shared__ float scratch[32];
  pdl_trigger();
  const int out_row = blockIdx.x;
  const int in_row = row_index ? row_index[out_row] : out_row;
  const TX* xr = x + static_cast<size_t>(in_row) * hidden;
  float* rr = residual ? residual + static_cast<size_t>(in_row) * hidden : nullptr;
  TOut* o = out + static_cast<size_t>(out_row) * hidden;

  if constexpr (kVector) {
    const int at = threadIdx.x * 8;
    const bool active = at < hidden;
    float w[8], v[8];
    if (active) load8(weight + at, w);
    pdl_wait();
    float sum_sq = 0.0f;
    if (active) {
      load8(xr + at, v);
      if (mode == 1) {
        float r[8];
        load8(rr + at, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += r[i];
      }
      if (write_residual) store8(rr + at, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) sum_sq += v[i] * v[i];
    }
    sum_sq = block_sum(sum_sq, scratch);
    const float inv_rms = rsqrtf(sum_sq / static_cast<float>(hidden) + eps);
    if (active) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * inv_rms * w[i];
      store8(o + at, v);
    }
  } else {
    pdl_wait();
    float sum_sq = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = to_float(xr[i]);
      if (mode == 1) v += rr[i];
      if (write_residual) rr[i] = v;
      row_values[i] = v;
      sum_sq += v * v;
    }
    sum_sq = block_sum(sum_sq, scratch);
    const float inv_rms = rsqrtf(sum_sq / static_cast<float>(hidden) + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      o[i] = from_float<TOut>(row_values[i] * inv_rms * weight[i]);
  }
}

// ---------------------------------------------------------------- SiLU * up
// gate_up is [rows, 2 * inter] with the gate in columns [0, inter) and up in
// [inter, 2 * inter); out[r, c] = silu(gate) * up with silu(z) = z * sigmoid(z), in float32.
// Sixteen-bit outputs keep 8 bits of mantissa: the fast exponential and division (a few units in
// the last place of float32) change no result; the 32-bit engine takes the exact ones.
template <typename T>
__device__ __forceinline__ float silu_times(float gate, float up) {
  if constexpr (sizeof(T) == 2) {
    return __fdividef(gate, 1.0f + __expf(-gate)) * up;
  } else {
    return gate / (1.0f + expf(-gate)) * up;
  }
}

template <typename T, bool kVector>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows,
                                int inter) {
  pdl_trigger();
  pdl_wait();
  constexpr int kStep = kVector ? 8 : 1;
  const size_t per_row = static_cast<size_t>(inter / kStep);
  const size_t total = static_cast<size_t>(rows) * per_row;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = idx / per_row;
    const int c = static_cast<int>(idx - r * per_row) * kStep;
    const T* gate = gate_up + r * 2 * inter + c;
    if constexpr (kVector) {
      float g[8], u[8];
      load8(gate, g);
      load8(gate + inter, u);
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = silu_times<T>(g[i], u[i]);
      store8(out + r * inter + c, g);
    } else {
      const float g = to_float(gate[0]);
      const float u = to_float(gate[inter]);
      out[r * inter + c] = from_float<T>(silu_times<T>(g, u));
    }
  }
}

// -------------------------------------------------------------- conversions
template <typename TIn>
__global__ void to_float_kernel(const TIn* __restrict__ in, float* __restrict__ out, size_t n) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < n;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x)
    out[idx] = to_float(in[idx]);
}

// ------------------------------------------------------------ block-table rows
// table[slots[i], :] = rows[i, :]: the block-table rows that changed on the host, brought over
// with the step's metadata instead of one copy per row.
__global__ void scatter_rows_kernel(int* __restrict__ table, int row_len, int table_rows,
                                    const int* __restrict__ slots, const int* __restrict__ rows,
                                    int* __restrict__ fault) {
  const int slot = slots[blockIdx.x];
  if (slot < 0 || slot >= table_rows) {
    if (threadIdx.x == 0) atomicOr(fault, kFaultSlot);
    return;
  }
  for (int c = threadIdx.x; c < row_len; c += blockDim.x)
    table[static_cast<size_t>(slot) * row_len + c] = rows[static_cast<size_t>(blockIdx.x) * row_len + c];
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace rl

extern "C" {

int rl_embedding(int dtype, void* out, const void* table, const int* ids, const int* feedback,
                 int feedback_rows, int rows, int hidden, int vocab, int* fault, int pdl, cudaStream_t stream) {
  if (rows == 0) return 0;
  RL_DISPATCH_DTYPE(dtype, {
    const int threads = hidden >= 2048 ? 256 : 128;
    return rl::launch_kernel(rl::embedding_kernel<scalar_t>, dim3(rows), dim3(threads), 0, stream, pdl != 0,
                             static_cast<scalar_t*>(out), static_cast<const scalar_t*>(table), ids, feedback,
                             feedback_rows, hidden, vocab, fault);
  });
  return 0;
}

// x and out are `dtype`; residual and weight are float32.
int rl_add_rmsnorm(int dtype, const void* x, float* residual, const float* weight, void* out,
                   const int* row_index, int rows, int hidden, float eps, int mode,
                   int write_residual, int pdl, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (mode < 0 || mode > 2 || (mode == 1 && residual == nullptr) ||
      (write_residual && residual == nullptr) || hidden <= 0)
    return static_cast<int>(cudaErrorInvalidValue);
  const bool vector = hidden % 8 == 0 && hidden <= 8 * 1024 && rl::aligned16(x) && rl::aligned16(out) &&
                      rl::aligned16(weight) && (residual == nullptr || rl::aligned16(residual));
  RL_DISPATCH_DTYPE(dtype, {
    if (vector) {
      const int threads = (hidden / 8 + 31) / 32 * 32;
      return rl::launch_kernel(rl::add_rmsnorm_kernel<scalar_t, scalar_t, true>, dim3(rows), dim3(threads), 0,
                               stream, pdl != 0, static_cast<const scalar_t*>(x), residual, weight,
                               static_cast<scalar_t*>(out), row_index, hidden, eps, mode, write_residual);
    }
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    if (smem > 200 * 1024) return static_cast<int>(cudaErrorInvalidValue);
    int threads = 128;
    while (threads < 1024 && threads * 8 < hidden) threads *= 2;
    auto kernel = rl::add_rmsnorm_kernel<scalar_t, scalar_t, false>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    return rl::launch_kernel(kernel, dim3(rows), dim3(threads), smem, stream, pdl != 0,
                             static_cast<const scalar_t*>(x), residual, weight, static_cast<scalar_t*>(out),
                             row_index, hidden, eps, mode, write_residual);
  });
  return 0;
}

int rl_silu_mul(int dtype, const void* gate_up, void* out, int rows, int inter, int pdl,
                cudaStream_t stream) {
  if (rows == 0) return 0;
  const bool vector = inter % 8 == 0 && rl::aligned16(gate_up) && rl::aligned16(out);
  const size_t total = static_cast<size_t>(rows) * (vector ? inter / 8 : inter);
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  RL_DISPATCH_DTYPE(dtype, {
    auto kernel = vector ? rl::silu_mul_kernel<scalar_t, true> : rl::silu_mul_kernel<scalar_t, false>;
    return rl::launch_kernel(kernel, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0, stream, pdl != 0,
                             static_cast<const scalar_t*>(gate_up), static_cast<scalar_t*>(out), rows, inter);
  });
  return 0;
}

int rl_scatter_rows(int* table, int row_len, int table_rows, const int* slots, const int* rows, int count,
                    int* fault, cudaStream_t stream) {
  if (count == 0 || row_len == 0) return 0;
  if (count < 0 || row_len < 0 || table_rows <= 0) return static_cast<int>(cudaErrorInvalidValue);
  rl::scatter_rows_kernel<<<count, 128, 0, stream>>>(table, row_len, table_rows, slots, rows, fault);
  return rl::launch_status();
}

int rl_to_float(int dtype, const void* in, float* out, long long n, int pdl, cudaStream_t stream) {
  if (n == 0) return 0;
  const int threads = 256;
  size_t blocks = (static_cast<size_t>(n) + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::to_float_kernel<scalar_t>, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0,
                             stream, pdl != 0, static_cast<const scalar_t*>(in), out, static_cast<size_t>(n));
  });
  return 0;
}

}  // extern "C"

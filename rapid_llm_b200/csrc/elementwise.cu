// Embedding gather, residual-add + RMSNorm, SiLU(gate)*up.
//
// The reference runs these as a library gather (rapid_llm/modules/vocab_parallel.py:101-103),
// Triton row kernels (rapid_llm/kernels/ops/layernorm/skip_rmsnorm.py:22-85,197-240) and a
// Triton SwiGLU kernel (rapid_llm/kernels/ops/activation/swiglu.py:91-121).  Here the
// residual stream is a float32 buffer in both engine precisions: the sum x + r is formed
// and kept in 32-bit, and the norm's statistics, scaling and weight product are 32-bit
// with one rounding at the store.
#include "common.cuh"

namespace rl {

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(T* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int hidden, int vocab,
                                 int* __restrict__ fault) {
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(fault, kFaultTokenId);
    id = 0;
  }
  const T* src = table + static_cast<size_t>(id) * hidden;
  T* dst = out + static_cast<size_t>(row) * hidden;
  constexpr int kVec = 16 / sizeof(T);
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
template <typename TX, typename TOut>
__global__ void add_rmsnorm_kernel(const TX* __restrict__ x, float* __restrict__ residual,
                                   const float* __restrict__ weight, TOut* __restrict__ out,
                                   const int* __restrict__ row_index, int hidden, float eps,
                                   int mode, int write_residual) {
  extern __shared__ float row_values[];  // [hidden]
  __shared__ float scratch[32];
  const int out_row = blockIdx.x;
  const int in_row = row_index ? row_index[out_row] : out_row;
  const TX* xr = x + static_cast<size_t>(in_row) * hidden;
  float* rr = residual ? residual + static_cast<size_t>(in_row) * hidden : nullptr;

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
  TOut* o = out + static_cast<size_t>(out_row) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_float<TOut>(row_values[i] * inv_rms * weight[i]);
}

// ---------------------------------------------------------------- SiLU * up
// gate_up is [rows, 2 * inter] with the gate in columns [0, inter) and up in
// [inter, 2 * inter); out[r, c] = silu(gate) * up with silu(z) = z * sigmoid(z), in float32.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows,
                                int inter) {
  const size_t total = static_cast<size_t>(rows) * inter;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = idx / inter;
    const int c = static_cast<int>(idx - r * inter);
    const float g = to_float(gate_up[r * 2 * inter + c]);
    const float u = to_float(gate_up[r * 2 * inter + inter + c]);
    const float s = g / (1.0f + expf(-g));
    out[idx] = from_float<T>(s * u);
  }
}

// -------------------------------------------------------------- conversions
template <typename TIn>
__global__ void to_float_kernel(const TIn* __restrict__ in, float* __restrict__ out, size_t n) {
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < n;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x)
    out[idx] = to_float(in[idx]);
}

}  // namespace rl

extern "C" {

int rl_embedding(int dtype, void* out, const void* table, const int* ids, int rows, int hidden,
                 int vocab, int* fault, cudaStream_t stream) {
  if (rows == 0) return 0;
  RL_DISPATCH_DTYPE(dtype, {
    const int threads = hidden >= 2048 ? 256 : 128;
    rl::embedding_kernel<scalar_t><<<rows, threads, 0, stream>>>(
        static_cast<scalar_t*>(out), static_cast<const scalar_t*>(table), ids, hidden, vocab, fault);
  });
  return rl::launch_status();
}

// x and out are `dtype`; residual and weight are float32.
int rl_add_rmsnorm(int dtype, const void* x, float* residual, const float* weight, void* out,
                   const int* row_index, int rows, int hidden, float eps, int mode,
                   int write_residual, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (mode < 0 || mode > 2 || (mode == 1 && residual == nullptr) ||
      (write_residual && residual == nullptr))
    return static_cast<int>(cudaErrorInvalidValue);
  const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
  if (smem > 200 * 1024) return static_cast<int>(cudaErrorInvalidValue);
  int threads = 128;
  while (threads < 1024 && threads * 8 < hidden) threads *= 2;
  RL_DISPATCH_DTYPE(dtype, {
    auto kernel = rl::add_rmsnorm_kernel<scalar_t, scalar_t>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    kernel<<<rows, threads, smem, stream>>>(static_cast<const scalar_t*>(x), residual, weight,
                                            static_cast<scalar_t*>(out), row_index, hidden, eps,
                                            mode, write_residual);
  });
  return rl::launch_status();
}

int rl_silu_mul(int dtype, const void* gate_up, void* out, int rows, int inter,
                cudaStream_t stream) {
  if (rows == 0) return 0;
  const size_t total = static_cast<size_t>(rows) * inter;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  RL_DISPATCH_DTYPE(dtype, {
    rl::silu_mul_kernel<scalar_t><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const scalar_t*>(gate_up), static_cast<scalar_t*>(out), rows, inter);
  });
  return rl::launch_status();
}

int rl_to_float(int dtype, const void* in, float* out, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  const int threads = 256;
  size_t blocks = (static_cast<size_t>(n) + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  RL_DISPATCH_DTYPE(dtype, {
    rl::to_float_kernel<scalar_t><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const scalar_t*>(in), out, static_cast<size_t>(n));
  });
  return rl::launch_status();
}

}  // extern "C"

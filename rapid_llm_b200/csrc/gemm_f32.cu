// True 32-bit matrix product: C[M, N] = A[M, K] * W[N, K]^T (+ bias), float32 in, float32
// fused multiply-adds, float32 out.  No tensor cores and no reduced-precision mode.
//
// Every output element is accumulated over k = 0 .. K-1 in that order by one thread, so its
// value does not depend on M, on the tile it falls in, or on what else is in the batch.
// The reference has no 32-bit path (rapid_llm/models/config.py:134-146 downgrades float32
// checkpoints); its products go through a library call (rapid_llm/kernels/ops/gemm/linear.py:17-40).
#include "common.cuh"

namespace rl {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16;

template <bool kAligned>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ w,
                const float* __restrict__ bias, float* __restrict__ c, int m, int n, int k,
                int lda, int ldc) {
  __shared__ float a_tile[kTileK][kTileM + 4];
  __shared__ float w_tile[kTileK][kTileN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * kTileM, n0 = blockIdx.x * kTileN;
  const int load_row = tid >> 2, load_k = (tid & 3) * 4;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < k; k0 += kTileK) {
    float av[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
    const int am = m0 + load_row, wn = n0 + load_row, kk = k0 + load_k;
    if (kAligned) {
      if (am < m && kk < k) {
        const float4 v = *reinterpret_cast<const float4*>(a + static_cast<size_t>(am) * lda + kk);
        av[0] = v.x; av[1] = v.y; av[2] = v.z; av[3] = v.w;
      }
      if (wn < n && kk < k) {
        const float4 v = *reinterpret_cast<const float4*>(w + static_cast<size_t>(wn) * k + kk);
        wv[0] = v.x; wv[1] = v.y; wv[2] = v.z; wv[3] = v.w;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (am < m && kk + e < k) av[e] = a[static_cast<size_t>(am) * lda + kk + e];
        if (wn < n && kk + e < k) wv[e] = w[static_cast<size_t>(wn) * k + kk + e];
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      a_tile[load_k + e][load_row] = av[e];
      w_tile[load_k + e][load_row] = wv[e];
    }
    __syncthreads();
#pragma unroll
    for (int kk2 = 0; kk2 < kTileK; ++kk2) {
      const float4 a4 = *reinterpret_cast<const float4*>(&a_tile[kk2][ty * 4]);
      const float4 w4 = *reinterpret_cast<const float4*>(&w_tile[kk2][tx * 4]);
      const float ar[4] = {a4.x, a4.y, a4.z, a4.w};
      const float wr[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + ty * 4 + i;
    if (row >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + tx * 4 + j;
      if (col < n) c[static_cast<size_t>(row) * ldc + col] = acc[i][j] + (bias ? bias[col] : 0.0f);
    }
  }
}

}  // namespace rl

// a: [m, k] with row stride lda; w: [n, k] contiguous; c: [m, n] with row stride ldc.
extern "C" int rl_gemm_f32(const float* a, const float* w, const float* bias, float* c, int m,
                           int n, int k, int lda, int ldc, cudaStream_t stream) {
  if (m == 0 || n == 0) return 0;
  if (k <= 0 || lda < k || ldc < n) return static_cast<int>(cudaErrorInvalidValue);
  const dim3 grid((n + rl::kTileN - 1) / rl::kTileN, (m + rl::kTileM - 1) / rl::kTileM);
  const bool aligned = (k % 4 == 0) && (lda % 4 == 0) &&
                       (reinterpret_cast<uintptr_t>(a) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(w) % 16 == 0);
  if (aligned)
    rl::gemm_f32_kernel<true><<<grid, 256, 0, stream>>>(a, w, bias, c, m, n, k, lda, ldc);
  else
    rl::gemm_f32_kernel<false><<<grid, 256, 0, stream>>>(a, w, bias, c, m, n, k, lda, ldc);
  return rl::launch_status();
}

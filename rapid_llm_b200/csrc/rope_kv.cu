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

struct RopeArgs {
  const void* qkv;          // [tokens, row_width]: q heads, then k heads, then v heads
  const float* bias;        // [(hq + 2 hkv) * d] or null
  const float* q_weight;    // [d] or null (no q/k norm)
  const float* k_weight;    // [d] or null
  const float* cos_table;   // [max_pos, rotary/2]
  const float* sin_table;
  const int* positions;     // [tokens]
  const int* kv_dest;       // [tokens] page * page_size + offset, or null (q only)
  void* q_out;              // [tokens, hq, d]
  void* cache;              // layer cache or null
  int tokens, row_width, hq, hkv, d, rotary, max_pos, page_size, num_pages;
  float eps;
  int* fault;
};

// One warp per (token, run of heads).  kVec > 0: the head size is 32 * kVec, the whole head
// rotates (rotary == d), and lane l holds the kVec consecutive elements from l * kVec in
// registers; its rotation partner (element + d/2) sits in lane l ^ 16.  A warp then takes
// `heads_per_warp` consecutive heads of its token and fetches the token's angles and the norm
// weights once for all of them (many heads a warp when there are many tokens, one when there
// are few and the work has to spread over the SMs).  kVec == 0: any head size up to 256 and
// any even rotary width, one head a warp, element by element through shared memory.
template <typename T, int kVec>
__global__ void qk_norm_rope_write_kernel(const RopeArgs a, const int heads_per_warp) {
  __shared__ float staged[kVec == 0 ? kRopeWarps : 1][kVec == 0 ? kMaxHeadDim : 1];
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_per_token = a.kv_dest ? a.hq + 2 * a.hkv : a.hq;
  const int warps_per_token = (heads_per_token + heads_per_warp - 1) / heads_per_warp;
  const long long index = static_cast<long long>(blockIdx.x) * kRopeWarps + warp;
  if (index >= static_cast<long long>(a.tokens) * warps_per_token) {
    pdl_wait();
    return;
  }
  const int d = a.d;
  const int t = static_cast<int>(index / warps_per_token);
  const int head_begin = static_cast<int>(index - static_cast<long long>(t) * warps_per_token) * heads_per_warp;
  const int head_end = min(heads_per_token, head_begin + heads_per_warp);
  int pos = a.positions[t];
  if (pos < 0 || pos >= a.max_pos) {
    if (lane == 0 && head_begin < a.hq + a.hkv) atomicOr(a.fault, kFaultPosition);   // only rotated heads need it
    pos = 0;
  }
  const int half = a.rotary >> 1;
  // where the token's key and value go
  int page = 0, offset = 0;
  bool bad_page = false;
  if (a.kv_dest) {
    const int dest = a.kv_dest[t];
    page = dest / a.page_size;
    offset = dest - page * a.page_size;
    bad_page = dest < 0 || page >= a.num_pages;
  }

  if constexpr (kVec > 0) {
    const int at = lane * kVec;
    const int angle = at < half ? at : at - half;      // kVec divides d / 2, so a lane never straddles
    float c[kVec], s[kVec], qw[kVec], kw[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      c[i] = a.cos_table[static_cast<size_t>(pos) * half + angle + i];
      s[i] = a.sin_table[static_cast<size_t>(pos) * half + angle + i];
      qw[i] = a.q_weight ? a.q_weight[at + i] : 1.0f;
      kw[i] = a.k_weight ? a.k_weight[at + i] : 1.0f;
    }
    pdl_wait();
    // a head's source and where it goes
    auto source_of = [&](int head) {
      return static_cast<const T*>(a.qkv) + static_cast<size_t>(t) * a.row_width + static_cast<size_t>(head) * d;
    };
    auto load_head = [&](int head, float (&v)[kVec]) {
      const T* src = source_of(head);
      if constexpr (kVec == 8) {
        load8(src + at, v);
      } else if constexpr (sizeof(T) == 2 && kVec == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(src + at);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
        v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
      } else {
#pragma unroll
        for (int i = 0; i < kVec; ++i) v[i] = to_float(src[at + i]);
      }
    };
    auto finish_head = [&](int head, float (&v)[kVec]) {
      const int kind = head < a.hq ? 0 : (head < a.hq + a.hkv ? 1 : 2);   // q, k, v
      T* dst;
      if (kind == 0) {
        dst = static_cast<T*>(a.q_out) + (static_cast<size_t>(t) * a.hq + head) * d;
      } else {
        if (bad_page) {
          if (lane == 0) atomicOr(a.fault, kFaultPageId);
          return;
        }
        const int kv_head = kind == 1 ? head - a.hq : head - a.hq - a.hkv;
        dst = static_cast<T*>(a.cache) +
              ((((static_cast<size_t>(page) * 2 + (kind - 1)) * a.hkv + kv_head) * a.page_size) + offset) * d;
      }
      float sum_sq = 0.0f;
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        if (a.bias) v[i] += a.bias[static_cast<size_t>(head) * d + at + i];
        sum_sq += v[i] * v[i];
      }
      if (kind != 2) {
        if (kind == 0 ? a.q_weight != nullptr : a.k_weight != nullptr) {
          sum_sq = warp_sum(sum_sq);
          const float inv_rms = rsqrtf(sum_sq / static_cast<float>(d) + a.eps);
#pragma unroll
          for (int i = 0; i < kVec; ++i) v[i] = v[i] * inv_rms * (kind == 0 ? qw[i] : kw[i]);
        }
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
          const float other = __shfl_xor_sync(0xffffffffu, v[i], 16);
          // first half: x1 * c - x2 * s; second half: x2 * c + x1 * s
          v[i] = lane < 16 ? v[i] * c[i] - other * s[i] : v[i] * c[i] + other * s[i];
        }
      }
      if constexpr (kVec == 8) {
        if constexpr (sizeof(T) == 2) {
          uint4 raw;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
          for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
          *reinterpret_cast<uint4*>(dst + at) = raw;
        } else {
          *reinterpret_cast<float4*>(dst + at) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(dst + at + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
      } else if constexpr (sizeof(T) == 2 && kVec == 4) {
        uint2 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
        h[0] = __floats2bfloat162_rn(v[0], v[1]);
        h[1] = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(dst + at) = raw;
      } else {
#pragma unroll
        for (int i = 0; i < kVec; ++i) dst[at + i] = from_float<T>(v[i]);
      }
    };
    // the loads of four heads fly together; their arithmetic follows
    constexpr int kHeadsInFlight = 4;
    for (int head0 = head_begin; head0 < head_end; head0 += kHeadsInFlight) {
      float v[kHeadsInFlight][kVec];
#pragma unroll
      for (int j = 0; j < kHeadsInFlight; ++j)
        if (head0 + j < head_end) load_head(head0 + j, v[j]);
#pragma unroll
      for (int j = 0; j < kHeadsInFlight; ++j)
        if (head0 + j < head_end) finish_head(head0 + j, v[j]);
    }
  } else {
    pdl_wait();
    const int head = head_begin;                       // one head a warp on this path
    const int kind = head < a.hq ? 0 : (head < a.hq + a.hkv ? 1 : 2);
    const T* src = static_cast<const T*>(a.qkv) + static_cast<size_t>(t) * a.row_width + static_cast<size_t>(head) * d;
    const float* b = a.bias ? a.bias + static_cast<size_t>(head) * d : nullptr;
    T* dst;
    if (kind == 0) {
      dst = static_cast<T*>(a.q_out) + (static_cast<size_t>(t) * a.hq + head) * d;
    } else {
      if (bad_page) {
        if (lane == 0) atomicOr(a.fault, kFaultPageId);
        return;
      }
      const int kv_head = kind == 1 ? head - a.hq : head - a.hq - a.hkv;
      dst = static_cast<T*>(a.cache) +
            ((((static_cast<size_t>(page) * 2 + (kind - 1)) * a.hkv + kv_head) * a.page_size) + offset) * d;
    }
    const float* w = kind == 0 ? a.q_weight : (kind == 1 ? a.k_weight : nullptr);
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
    if (w) {
      sum_sq = warp_sum(sum_sq);
      const float inv_rms = rsqrtf(sum_sq / static_cast<float>(d) + a.eps);
      for (int i = lane; i < d; i += 32) mine[i] = mine[i] * inv_rms * w[i];
    }
    __syncwarp();
    const float* c = a.cos_table + static_cast<size_t>(pos) * half;
    const float* s = a.sin_table + static_cast<size_t>(pos) * half;
    for (int i = lane; i < d; i += 32) {
      float v;
      if (i < half) {
        v = mine[i] * c[i] - mine[i + half] * s[i];
      } else if (i < a.rotary) {
        v = mine[i] * c[i - half] + mine[i - half] * s[i - half];
      } else {
        v = mine[i];
      }
      dst[i] = from_float<T>(v);
    }
  }
}

// Heads of 128 in bfloat16 at many tokens, the whole head rotated, no bias: half a warp per head, so
// every warp instruction works on two heads, and the loads of a warp's eight heads fly together.  A lane
// holds four consecutive elements of the head's first half and their rotation partners in the second, so
// the rotation needs no exchange between lanes and four angles a lane.  The kernel is bound by the bytes
// it keeps in flight and by instruction issue, not by arithmetic: it stays within 64 registers (eight CTAs,
// 32 warps a multiprocessor), asks for its heads before its angles (both wait on the position alone) and
// reads the norm weights where it uses them (they stay in L1).
__global__ void __launch_bounds__(kRopeWarps * 32, 8) qk_norm_rope_write_pairs_kernel(const RopeArgs a) {
  using T = __nv_bfloat16;
  constexpr int kHeadsPerWarp = 8, kD = 128, kHalf = kD / 2;
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_per_token = a.kv_dest ? a.hq + 2 * a.hkv : a.hq;
  const int warps_per_token = (heads_per_token + kHeadsPerWarp - 1) / kHeadsPerWarp;
  const long long index = static_cast<long long>(blockIdx.x) * kRopeWarps + warp;
  if (index >= static_cast<long long>(a.tokens) * warps_per_token) {
    pdl_wait();
    return;
  }
  const int t = static_cast<int>(index / warps_per_token);
  const int head_begin = static_cast<int>(index - static_cast<long long>(t) * warps_per_token) * kHeadsPerWarp;
  const int head_end = min(heads_per_token, head_begin + kHeadsPerWarp);
  int pos = a.positions[t];
  const int dest = a.kv_dest ? a.kv_dest[t] : 0;
  const int side = lane >> 4, at = (lane & 15) * 4;          // which head of the pair; first element of each half
  pdl_wait();
  const T* row = static_cast<const T*>(a.qkv) + static_cast<size_t>(t) * a.row_width;
  uint2 low[kHeadsPerWarp / 2], high[kHeadsPerWarp / 2];
#pragma unroll
  for (int pair = 0; pair < kHeadsPerWarp / 2; ++pair) {
    const int head = head_begin + 2 * pair + side;
    low[pair] = high[pair] = make_uint2(0, 0);
    if (head < head_end) {
      low[pair] = *reinterpret_cast<const uint2*>(row + static_cast<size_t>(head) * kD + at);
      high[pair] = *reinterpret_cast<const uint2*>(row + static_cast<size_t>(head) * kD + kHalf + at);
    }
  }
  if (pos < 0 || pos >= a.max_pos) {
    if (lane == 0 && head_begin < a.hq + a.hkv) atomicOr(a.fault, kFaultPosition);
    pos = 0;
  }
  float4 c = make_float4(1.0f, 1.0f, 1.0f, 1.0f), s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  if (head_begin < a.hq + a.hkv) {                             // a warp of values alone needs no angles
    c = __ldg(reinterpret_cast<const float4*>(a.cos_table + static_cast<size_t>(pos) * kHalf + at));
    s = __ldg(reinterpret_cast<const float4*>(a.sin_table + static_cast<size_t>(pos) * kHalf + at));
  }
  const int page = dest / a.page_size, offset = dest - page * a.page_size;
  const bool bad_page = a.kv_dest != nullptr && (dest < 0 || page >= a.num_pages);
#pragma unroll
  for (int pair = 0; pair < kHeadsPerWarp / 2; ++pair) {
    const int head = head_begin + 2 * pair + side;
    const int kind = head < a.hq ? 0 : (head < a.hq + a.hkv ? 1 : 2);   // q, k, v
    T* dst = nullptr;
    if (head < head_end) {
      if (kind == 0) {
        dst = static_cast<T*>(a.q_out) + (static_cast<size_t>(t) * a.hq + head) * kD + at;
      } else if (!bad_page) {
        const int kv_head = kind == 1 ? head - a.hq : head - a.hq - a.hkv;
        dst = static_cast<T*>(a.cache) +
              ((((static_cast<size_t>(page) * 2 + (kind - 1)) * a.hkv + kv_head) * a.page_size) + offset) * kD + at;
      } else if ((lane & 15) == 0) {
        atomicOr(a.fault, kFaultPageId);
      }
    }
    // the pair's two heads may be of different kinds; a warp decides together only what all its lanes share
    if (!__any_sync(0xffffffffu, kind != 2)) {                 // values: copied as they are
      if (dst != nullptr) {
        *reinterpret_cast<uint2*>(dst) = low[pair];
        *reinterpret_cast<uint2*>(dst + kHalf) = high[pair];
      }
      continue;
    }
    float x1[4], x2[4];
    {
      const __nv_bfloat162* lo = reinterpret_cast<const __nv_bfloat162*>(&low[pair]);
      const __nv_bfloat162* hi = reinterpret_cast<const __nv_bfloat162*>(&high[pair]);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float2 p = __bfloat1622float2(lo[i]), q = __bfloat1622float2(hi[i]);
        x1[2 * i] = p.x; x1[2 * i + 1] = p.y;
        x2[2 * i] = q.x; x2[2 * i + 1] = q.y;
      }
    }
    float sum_sq = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) sum_sq += x1[i] * x1[i] + x2[i] * x2[i];
#pragma unroll
    for (int step = 8; step > 0; step >>= 1) sum_sq += __shfl_xor_sync(0xffffffffu, sum_sq, step);   // within 16 lanes
    const float* weight = kind == 0 ? a.q_weight : (kind == 1 ? a.k_weight : nullptr);
    if (weight != nullptr) {
      const float inv_rms = rsqrtf(sum_sq / static_cast<float>(kD) + a.eps);
      const float4 w1 = __ldg(reinterpret_cast<const float4*>(weight + at));
      const float4 w2 = __ldg(reinterpret_cast<const float4*>(weight + kHalf + at));
      x1[0] = x1[0] * inv_rms * w1.x; x1[1] = x1[1] * inv_rms * w1.y; x1[2] = x1[2] * inv_rms * w1.z; x1[3] = x1[3] * inv_rms * w1.w;
      x2[0] = x2[0] * inv_rms * w2.x; x2[1] = x2[1] * inv_rms * w2.y; x2[2] = x2[2] * inv_rms * w2.z; x2[3] = x2[3] * inv_rms * w2.w;
    }
    if (dst == nullptr) continue;
    uint2 out1 = low[pair], out2 = high[pair];
    if (kind != 2) {
      // first half of the head: x1 * c - x2 * s; second half: x2 * c + x1 * s
      const float cs[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
      float o1[4], o2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        o1[i] = x1[i] * cs[i] - x2[i] * sn[i];
        o2[i] = x2[i] * cs[i] + x1[i] * sn[i];
      }
      __nv_bfloat162* h1 = reinterpret_cast<__nv_bfloat162*>(&out1);
      __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&out2);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        h1[i] = __floats2bfloat162_rn(o1[2 * i], o1[2 * i + 1]);
        h2[i] = __floats2bfloat162_rn(o2[2 * i], o2[2 * i + 1]);
      }
    }
    *reinterpret_cast<uint2*>(dst) = out1;
    *reinterpret_cast<uint2*>(dst + kHalf) = out2;
  }
}

}  // namespace rl

extern "C" int rl_qk_norm_rope_write(int dtype, const void* qkv, int row_width, const float* bias,
                                     const float* q_weight, const float* k_weight,
                                     const float* cos_table, const float* sin_table,
                                     const int* positions, const int* kv_dest, void* q_out,
                                     void* cache, int tokens, int hq, int hkv, int d, int rotary,
                                     int max_pos, int page_size, int num_pages, float eps,
                                     int* fault, int pdl, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (d > rl::kMaxHeadDim || d <= 0 || rotary < 0 || rotary > d || (rotary & 1) ||
      (kv_dest != nullptr && cache == nullptr))
    return static_cast<int>(cudaErrorInvalidValue);
  const int heads_per_token = kv_dest ? hq + 2 * hkv : hq;
  rl::RopeArgs a;
  a.qkv = qkv; a.bias = bias; a.q_weight = q_weight; a.k_weight = k_weight;
  a.cos_table = cos_table; a.sin_table = sin_table; a.positions = positions; a.kv_dest = kv_dest;
  a.q_out = q_out; a.cache = cache; a.tokens = tokens; a.row_width = row_width; a.hq = hq; a.hkv = hkv;
  a.d = d; a.rotary = rotary; a.max_pos = max_pos; a.page_size = page_size; a.num_pages = num_pages;
  a.eps = eps; a.fault = fault;
  // registers when the whole head rotates, a lane's elements are whole vectors and everything is aligned
  const bool aligned = ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                         reinterpret_cast<uintptr_t>(cache)) & 15) == 0 && row_width % 8 == 0;
  const int vec = (rotary == d && d % 32 == 0 && aligned) ? d / 32 : 0;
  // a warp takes several heads of a token once there are enough tokens to fill the GPU anyway
  // (the kernel for heads of 128 in bfloat16, which keeps more bytes in flight, from about 200 tokens of 48 heads
  // on: measured equal below, 15 us faster at 512 tokens and 26 us at 1,024)
  const bool pairs_kernel = d == 128 && vec == 4 && bias == nullptr && dtype == rl::kBF16;
  int heads_per_warp = 1;
  if (vec > 0 && static_cast<long long>(tokens) * heads_per_token >= (pairs_kernel ? 148ll * 64 : 148ll * 64 * 8))
    heads_per_warp = 8;
  const long long warps = static_cast<long long>(tokens) * ((heads_per_token + heads_per_warp - 1) / heads_per_warp);
  const dim3 grid(static_cast<unsigned>((warps + rl::kRopeWarps - 1) / rl::kRopeWarps)), block(rl::kRopeWarps * 32);
  const bool tables_aligned = ((reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table) |
                                reinterpret_cast<uintptr_t>(q_weight) | reinterpret_cast<uintptr_t>(k_weight)) & 15) == 0;
  if (heads_per_warp == 8 && pairs_kernel && tables_aligned)
    return rl::launch_kernel(rl::qk_norm_rope_write_pairs_kernel, grid, block, 0, stream, pdl != 0, a);
  RL_DISPATCH_DTYPE(dtype, {
    if (vec == 8) return rl::launch_kernel(rl::qk_norm_rope_write_kernel<scalar_t, 8>, grid, block, 0, stream, pdl != 0, a, heads_per_warp);
    if (vec == 4) return rl::launch_kernel(rl::qk_norm_rope_write_kernel<scalar_t, 4>, grid, block, 0, stream, pdl != 0, a, heads_per_warp);
    if (vec == 2) return rl::launch_kernel(rl::qk_norm_rope_write_kernel<scalar_t, 2>, grid, block, 0, stream, pdl != 0, a, heads_per_warp);
    if (vec == 1) return rl::launch_kernel(rl::qk_norm_rope_write_kernel<scalar_t, 1>, grid, block, 0, stream, pdl != 0, a, heads_per_warp);
    return rl::launch_kernel(rl::qk_norm_rope_write_kernel<scalar_t, 0>, grid, block, 0, stream, pdl != 0, a, heads_per_warp);
  });
  return 0;
}

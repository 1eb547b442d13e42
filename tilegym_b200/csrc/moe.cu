// The kernels around the grouped block-scaled GEMM that make up the FP8 mixture-of-experts layer
// (reference: fused_experts_impl, src/tilegym/ops/moe_interface.py:116-322, and its kernels
// src/tilegym/ops/tilecpp/moe.cuh:72-563).  The reference pads every expert's token list to a multiple of the
// tile height and lets every GEMM tile gather its rows through sorted_token_ids; here the rows are brought
// into expert order ONCE, so that both expert GEMMs run on contiguous row segments (m_indptr) with plain TMA
// loads and bulk stores, and the way back to token order is folded into the final sum over the top-k experts:
//
//   tg_moe_route          top-k ids -> per-expert segment offsets, the permutation and its inverse, and the
//                         routing weights in expert order (a counting sort on the device, no host read-back);
//   tg_moe_permute_rows   e4m3 activation rows and their 1 x 128 scales -> expert order (a row gather);
//   tg_moe_silu_mul_quant silu(gate) * up of the first GEMM's output, rounded to 16 bits like the reference's
//                         intermediate, then to e4m3 for the second GEMM (scale 1 as the reference does, or a
//                         proper 1 x 128 amax / 448 scale);
//   tg_moe_unpermute_sum  out[t] = sum over the token's top-k rows of the second GEMM's output (fp32 sum, one rounding).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdio>

#include "tg_internal.h"
#include "tg_quant_common.cuh"

namespace tg {
namespace {

// ------------------------------------------------------------------------------------------ routing
// With up to kRouteSmemExperts experts a block first counts its pairs in shared memory and then adds one number per
// expert to the global counts (a few thousand global atomics instead of one per pair, all on a handful of addresses).
constexpr int kRouteSmemExperts = 2048;
template <typename IdT>
__global__ void __launch_bounds__(256) moe_count_kernel(const IdT* __restrict__ ids, int64_t n, int num_experts,
                                                        int32_t* __restrict__ counts) {
  __shared__ int32_t local[kRouteSmemExperts];
  const bool use_smem = num_experts <= kRouteSmemExperts;
  if (use_smem) {
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) local[e] = 0;
    __syncthreads();
  }
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = static_cast<int64_t>(ids[i]);
    if (e >= 0 && e < num_experts) atomicAdd(use_smem ? local + e : counts + e, 1);
  }
  if (use_smem) {
    __syncthreads();
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x)
      if (local[e] != 0) atomicAdd(counts + e, local[e]);
  }
}

// One block: exclusive scan of the counts -> m_indptr[0 .. E]; the counts become the experts' write cursors.
__global__ void moe_scan_kernel(int32_t* __restrict__ counts, int num_experts, int32_t* __restrict__ m_indptr) {
  __shared__ int32_t carry;
  __shared__ int32_t warp_sums[32];
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < num_experts; base += blockDim.x) {
    const int e = base + threadIdx.x;
    const int32_t c = e < num_experts ? counts[e] : 0;
    int32_t incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int32_t w = lane < static_cast<int>(blockDim.x >> 5) ? warp_sums[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int32_t v = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += v;
      }
      warp_sums[lane] = w;  // inclusive sums of the warps
    }
    __syncthreads();
    const int32_t before = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - c;
    if (e < num_experts) {
      m_indptr[e] = before;
      counts[e] = before;  // cursor
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry = before + c;
    __syncthreads();
  }
  if (threadIdx.x == 0) m_indptr[num_experts] = carry;
}

// Placement: with few enough experts a block counts the pairs of its slice per expert in shared memory, reserves one
// range per expert with a single global atomic, and hands out the places inside the range from shared memory.  A
// block's slice is contiguous (the same pairs in both passes).
template <typename IdT, typename WT>
__global__ void __launch_bounds__(256) moe_place_kernel(const IdT* __restrict__ ids, const WT* __restrict__ weights,
                                                        int64_t n, int num_experts, int32_t* __restrict__ cursors,
                                                        int32_t* __restrict__ sorted_ids, int32_t* __restrict__ pos,
                                                        float* __restrict__ w_sorted) {
  __shared__ int32_t local[kRouteSmemExperts];  // per expert: count of the slice, then the next place in the block's range
  if (num_experts <= kRouteSmemExperts) {
    const int64_t per = (n + gridDim.x - 1) / gridDim.x;
    const int64_t lo = static_cast<int64_t>(blockIdx.x) * per, hi = lo + per < n ? lo + per : n;
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) local[e] = 0;
    __syncthreads();
    for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const int64_t e = static_cast<int64_t>(ids[i]);
      if (e >= 0 && e < num_experts) atomicAdd(local + e, 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
      const int32_t c = local[e];
      local[e] = c != 0 ? atomicAdd(cursors + e, c) : 0;  // first place of this block's range for expert e
    }
    __syncthreads();
    for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const int64_t e = static_cast<int64_t>(ids[i]);
      if (e >= 0 && e < num_experts) {
        const int32_t r = atomicAdd(local + e, 1);
        sorted_ids[r] = static_cast<int32_t>(i);
        pos[i] = r;
        if (w_sorted != nullptr) w_sorted[r] = weights != nullptr ? static_cast<float>(weights[i]) : 1.0f;
      } else {
        pos[i] = -1;
      }
    }
    return;
  }
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = static_cast<int64_t>(ids[i]);
    if (e >= 0 && e < num_experts) {
      const int32_t r = atomicAdd(cursors + e, 1);
      sorted_ids[r] = static_cast<int32_t>(i);
      pos[i] = r;
      if (w_sorted != nullptr) w_sorted[r] = weights != nullptr ? static_cast<float>(weights[i]) : 1.0f;
    } else {
      pos[i] = -1;  // an id outside [0, E): the (token, slot) pair takes part in nothing
    }
  }
}

// The three steps above in ONE block for decode-sized routing tables (up to 4096 pairs, up to 1024 experts): histogram
// and write cursors live in shared memory, one launch instead of a clear and three kernels (8.8 -> ~3 us).  Above that
// size one SM's scattered stores make it slower than the three-kernel form (32 against 21 us at 24576 pairs).  The
// order of the pairs inside an expert's segment depends on the arrival order of the atomics, as in the three-kernel
// form; rows are independent and the top-k sum runs in slot order, so results do not depend on it.
constexpr int kRouteSmallMaxExperts = 1024;
constexpr int64_t kRouteSmallMaxPairs = 4096;
template <typename IdT, typename WT>
__global__ void __launch_bounds__(1024) moe_route_small_kernel(const IdT* __restrict__ ids, const WT* __restrict__ weights,
                                                               int n, int num_experts, int32_t* __restrict__ m_indptr,
                                                               int32_t* __restrict__ sorted_ids, int32_t* __restrict__ pos,
                                                               float* __restrict__ w_sorted) {
  __shared__ int32_t cnt[kRouteSmallMaxExperts];
  __shared__ int32_t warp_sums[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < num_experts) cnt[threadIdx.x] = 0;
  __syncthreads();
  // up to four pairs per thread, kept in registers between the two passes
  int64_t e_of[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = threadIdx.x + k * 1024;
    e_of[k] = i < n ? static_cast<int64_t>(ids[i]) : -1;
    if (e_of[k] >= 0 && e_of[k] < num_experts) atomicAdd(cnt + e_of[k], 1);
  }
  __syncthreads();
  {  // exclusive scan over the experts (one per thread)
    const int e = threadIdx.x;
    const int32_t c = e < num_experts ? cnt[e] : 0;
    int32_t incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int32_t w = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int32_t v = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += v;
      }
      warp_sums[lane] = w;  // inclusive sums of the warps
    }
    __syncthreads();
    const int32_t before = (warp > 0 ? warp_sums[warp - 1] : 0) + incl - c;
    if (e < num_experts) {
      m_indptr[e] = before;
      cnt[e] = before;  // write cursor
    }
    if (e == num_experts - 1) m_indptr[num_experts] = before + c;
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = threadIdx.x + k * 1024;
    if (i >= n) continue;
    if (e_of[k] >= 0 && e_of[k] < num_experts) {
      const int32_t r = atomicAdd(cnt + e_of[k], 1);
      sorted_ids[r] = i;
      pos[i] = r;
      if (w_sorted != nullptr) w_sorted[r] = weights != nullptr ? static_cast<float>(weights[i]) : 1.0f;
    } else {
      pos[i] = -1;  // an id outside [0, E): the (token, slot) pair takes part in nothing
    }
  }
}

// ------------------------------------------------------------------------------------------ row gather
// dst row r = src row sorted_ids[r] / topk: `row_bytes` (a multiple of 16) of e4m3 data and `kb` scales.
__global__ void __launch_bounds__(128) moe_permute_rows_kernel(uint8_t* __restrict__ dst, float* __restrict__ dst_s,
                                                               const uint8_t* __restrict__ src,
                                                               const float* __restrict__ src_s,
                                                               const int32_t* __restrict__ sorted_ids,
                                                               const int32_t* __restrict__ m_indptr, int num_experts,
                                                               int topk, int64_t row_bytes, int64_t src_pitch, int kb,
                                                               int64_t src_s_pitch) {
  const int32_t rows = __ldg(m_indptr + num_experts);  // rows in expert order (pairs with a valid expert id)
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const int64_t t = __ldg(sorted_ids + r) / topk;
    const uint4* s4 = reinterpret_cast<const uint4*>(src + t * src_pitch);
    uint4* d4 = reinterpret_cast<uint4*>(dst + r * row_bytes);
    for (int64_t c = threadIdx.x; c < row_bytes / 16; c += blockDim.x) d4[c] = __ldg(s4 + c);
    for (int c = threadIdx.x; c < kb; c += blockDim.x) dst_s[r * kb + c] = __ldg(src_s + t * src_s_pitch + c);
  }
}

// ------------------------------------------------------------------------------------------ quantise + row scatter
// 16-bit activations straight into expert order: every token row is quantised once (1 x 128 blocks, amax / 448, 1.0
// for an all-zero block - the arithmetic of act_quant) and written to each of its top_k places pos[t * top_k + j]
// (skipped where that is -1), together with its scales.  One pass instead of act_quant + row gather.
// A thread owns 16 consecutive elements, the 8 lanes of a block sit next to each other.
template <typename T>
__global__ void __launch_bounds__(256) moe_quant_permute_kernel(uint8_t* __restrict__ y, float* __restrict__ ys,
                                                                const T* __restrict__ x,
                                                                const int32_t* __restrict__ pos, int64_t tokens, int topk,
                                                                int64_t hidden) {
  q8_allow_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t cpr = hidden / 16;  // chunks per row
  const int64_t n_chunks = tokens * cpr;
  const int64_t span = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // all lanes of a warp run the same number of iterations (the shuffles need them)
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * blockDim.x + (threadIdx.x & ~31); base < n_chunks; base += span) {
    const int64_t c = base + lane;
    const bool live = c < n_chunks;
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = 0u;
    if (live) {
      const uint4 t0 = __ldcs(reinterpret_cast<const uint4*>(x + c * 16));
      const uint4 t1 = __ldcs(reinterpret_cast<const uint4*>(x + c * 16) + 1);
      w[0] = t0.x; w[1] = t0.y; w[2] = t0.z; w[3] = t0.w;
      w[4] = t1.x; w[5] = t1.y; w[6] = t1.z; w[7] = t1.w;
    }
    uint32_t m2 = absmax_pairs<T>(w[0], w[1]);
#pragma unroll
    for (int j = 2; j < 8; j += 2) m2 = absmax_pairs<T>(m2, absmax_pairs<T>(w[j], w[j + 1]));
    const float2 mm = unpack_pair<T>(m2);
    float amax = fmaxf(mm.x, mm.y);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float scale = q8_scale_from_amax(amax, 448.f, 1.0f / 448.f);
    if (scale == 0.f) scale = 1.0f;
    const float r = __frcp_rn(scale);
    const bool fast = q8_scale_is_tame(scale);
    uint32_t out[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x0 = unpack_pair<T>(w[2 * k]), x1 = unpack_pair<T>(w[2 * k + 1]);
      if (fast) {
        const float2 q0 = q8_quot2(x0, scale, r), q1 = q8_quot2(x1, scale, r);
        out[k] = q8_cast2<kQ8E4M3>(q0.x, q0.y, -448.f, 448.f) | (q8_cast2<kQ8E4M3>(q1.x, q1.y, -448.f, 448.f) << 16);
      } else {
        out[k] = q8_pair<kQ8E4M3>(x0.x, x0.y, scale, r, false, -448.f, 448.f) |
                 (q8_pair<kQ8E4M3>(x1.x, x1.y, scale, r, false, -448.f, 448.f) << 16);
      }
    }
    if (live) {
      const int64_t t = c / cpr, col = (c - t * cpr) * 16;
      const uint4 o4 = make_uint4(out[0], out[1], out[2], out[3]);
      for (int j = 0; j < topk; ++j) {
        const int32_t dst = __ldg(pos + t * topk + j);
        if (dst < 0) continue;
        *reinterpret_cast<uint4*>(y + static_cast<int64_t>(dst) * hidden + col) = o4;
        if ((lane & 7) == 0) ys[static_cast<int64_t>(dst) * (hidden / 128) + (col >> 7)] = scale;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ silu * mul + quantise
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) {
  return __half2float(v);
}
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) {
  return __float2half_rn(v);
}
template <typename T>
__device__ __forceinline__ float round16(float v);
template <>
__device__ __forceinline__ float round16<__nv_bfloat16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
template <>
__device__ __forceinline__ float round16<__half>(float v) {
  return __half2float(__float2half_rn(v));
}

// Eight lanes per group of 128 output elements, 16 consecutive ones per lane (two 16-byte loads of gate values, two of
// up values, one 16-byte store): a warp covers four groups.  X row = [gate (I) | up (I)], or with mode bit 1 set
// 128 gate values, the 128 up values of the same outputs, the next 128 gate values, ... (what the first GEMM writes
// when its weight rows were interleaved).  mode bit 0 clear: scale 1, y = e4m3(a) (saturating); set: scale = amax / 448
// (1 for an all-zero group), y = e4m3(a / scale).
template <typename T>
__global__ void __launch_bounds__(256) moe_silu_mul_quant_kernel(uint8_t* __restrict__ y, float* __restrict__ s,
                                                                 const T* __restrict__ x,
                                                                 const int32_t* __restrict__ m_indptr, int num_experts,
                                                                 int64_t inter, int mode) {
  q8_allow_dependents();
  const int sub = threadIdx.x & 7;  // which 16 of the group's 128 outputs
  const int64_t groups_per_row = inter / 128;
  const int64_t rows = m_indptr != nullptr ? static_cast<int64_t>(__ldg(m_indptr + num_experts)) : 0;
  const int64_t n_groups = rows * groups_per_row;
  const int64_t span = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 3;
  const bool inter_l = (mode & 2) != 0;
  // all lanes of a warp run the same number of iterations (the shuffles need them): the warp's first group decides
  for (int64_t g0 = ((static_cast<int64_t>(blockIdx.x) * blockDim.x + (threadIdx.x & ~31)) >> 3); g0 < n_groups; g0 += span) {
    const int64_t g = g0 + ((threadIdx.x & 31) >> 3);
    const bool live = g < n_groups;
    const int64_t r = live ? g / groups_per_row : 0, gc = live ? g - r * groups_per_row : 0;
    const T* gate = x + r * (2 * inter) + (inter_l ? gc * 256 : gc * 128) + sub * 16;
    const T* up = gate + (inter_l ? 128 : inter);
    uint4 gv[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)}, uv[2] = {gv[0], gv[0]};
    if (live) {
      gv[0] = __ldcs(reinterpret_cast<const uint4*>(gate));
      gv[1] = __ldcs(reinterpret_cast<const uint4*>(gate) + 1);
      uv[0] = __ldcs(reinterpret_cast<const uint4*>(up));
      uv[1] = __ldcs(reinterpret_cast<const uint4*>(up) + 1);
    }
    const T* gp = reinterpret_cast<const T*>(gv);
    const T* upv = reinterpret_cast<const T*>(uv);
    float a[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float gf = to_f32<T>(gp[i]), uf = to_f32<T>(upv[i]);
      // silu(g) * u in fp32 (fast exponential and division: the result is rounded to 16 bits right away),
      // rounded once to the 16-bit type of the reference's intermediate tensor
      a[i] = round16<T>(__fdividef(gf, 1.0f + __expf(-gf)) * uf);
      amax = fmaxf(amax, fabsf(a[i]));
    }
    float scale = 1.0f;
    if (mode & 1) {
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));  // the group's 8 lanes
      scale = __fdiv_rn(amax, 448.0f);
      if (scale == 0.f) scale = 1.0f;
      if (q8_scale_is_tame(scale)) {  // 16-bit values over RN(16-bit amax / 448): the test-free quotient applies
        const float rcp = __frcp_rn(scale);
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          const float2 q = q8_quot2(make_float2(a[i], a[i + 1]), scale, rcp);
          a[i] = q.x;
          a[i + 1] = q.y;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) a[i] = __fdiv_rn(a[i], scale);
      }
    }
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      w[k] = q8_cast2<kQ8E4M3>(a[4 * k], a[4 * k + 1], -448.f, 448.f) |
             (q8_cast2<kQ8E4M3>(a[4 * k + 2], a[4 * k + 3], -448.f, 448.f) << 16);
    if (live) {
      __stcs(reinterpret_cast<uint4*>(y + r * inter + gc * 128 + sub * 16), make_uint4(w[0], w[1], w[2], w[3]));
      if (sub == 0) s[r * groups_per_row + gc] = scale;
    }
  }
}

// ------------------------------------------------------------------------------------------ back to token order
// out[t, :] = sum_j c[pos[t * topk + j], :] (fp32 sum, one rounding); eight columns per thread.
template <typename T>
__global__ void __launch_bounds__(256) moe_unpermute_sum_kernel(T* __restrict__ out, const T* __restrict__ c,
                                                                const int32_t* __restrict__ pos, int64_t tokens,
                                                                int topk, int64_t hidden) {
  const int64_t chunks = hidden / 8;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < tokens * chunks;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / chunks, ch = i - t * chunks;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < topk; ++j) {
      const int32_t r = __ldg(pos + t * topk + j);
      if (r < 0) continue;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(c + static_cast<int64_t>(r) * hidden) + ch);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += to_f32<T>(e[k]);
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int k = 0; k < 8; ++k) oe[k] = from_f32<T>(acc[k]);
    reinterpret_cast<uint4*>(out + t * hidden)[ch] = o;
  }
}

int grid_for(int64_t work_items, int per_block, int num_sms, int waves) {
  int64_t g = (work_items + per_block - 1) / per_block;
  const int64_t cap = static_cast<int64_t>(num_sms) * waves;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

struct Guard {
  int prev = -1;
  bool changed = false;
  cudaError_t err = cudaSuccess;
  explicit Guard(int dev) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != dev) {
      err = cudaSetDevice(dev);
      changed = (err == cudaSuccess);
    }
  }
  ~Guard() {
    if (changed) cudaSetDevice(prev);
  }
};

int32_t launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return TG_OK;
  char msg[200];
  snprintf(msg, sizeof(msg), "%s launch failed: %s", what, cudaGetErrorString(e));
  return api_fail(TG_ERR_LAUNCH, msg);
}

bool contiguous_2d(const TgTensorDesc* t) { return t->ndim == 2 && t->strides[1] == 1 && t->strides[0] == t->shape[1]; }

}  // namespace
}  // namespace tg

using namespace tg;

extern "C" {

TG_API int32_t tg_moe_route(const TgTensorDesc* topk_ids, const TgTensorDesc* topk_weights, int32_t num_experts,
                            uint64_t m_indptr, uint64_t sorted_ids, uint64_t pos, uint64_t w_sorted, uint64_t scratch,
                            int32_t device_id, uint64_t stream) {
  if (topk_ids == nullptr) return api_fail(TG_ERR_NULL, "topk_ids descriptor is null");
  if (topk_ids->dtype != TG_I32 && topk_ids->dtype != TG_I64) return api_fail(TG_ERR_DTYPE, "topk_ids must be int32 or int64");
  if (!contiguous_2d(topk_ids)) return api_fail(TG_ERR_ARGS, "topk_ids must be a contiguous [tokens, top_k] matrix");
  if (num_experts < 1 || num_experts > (1 << 20)) return api_fail(TG_ERR_ARGS, "num_experts out of range");
  const int64_t n = topk_ids->shape[0] * topk_ids->shape[1];
  if (n > 0x7fffffff) return api_fail(TG_ERR_ARGS, "too many (token, expert) pairs");
  if (topk_weights != nullptr) {
    if (topk_weights->dtype != TG_F32 && topk_weights->dtype != TG_BF16 && topk_weights->dtype != TG_F16)
      return api_fail(TG_ERR_DTYPE, "topk_weights must be f32, f16 or bf16");
    if (!contiguous_2d(topk_weights) || topk_weights->shape[0] != topk_ids->shape[0] ||
        topk_weights->shape[1] != topk_ids->shape[1])
      return api_fail(TG_ERR_ARGS, "topk_weights must be contiguous and shaped like topk_ids");
    if (w_sorted == 0) return api_fail(TG_ERR_NULL, "w_sorted is null");
  }
  if (m_indptr == 0 || sorted_ids == 0 || pos == 0 || scratch == 0) return api_fail(TG_ERR_NULL, "an output pointer is null");
  if ((m_indptr | sorted_ids | pos | w_sorted | scratch) & 3u) return api_fail(TG_ERR_ALIGN, "outputs must be 4-byte aligned");
  if (n > 0 && (topk_ids->ptr == 0 || (topk_weights != nullptr && topk_weights->ptr == 0)))
    return api_fail(TG_ERR_NULL, "data pointer is null");
  Guard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return api_fail(TG_ERR_DEVICE, "cannot select the CUDA device");
  }
  int num_sms = 0;
  int32_t* status = nullptr;
  int32_t rc = api_init_device(device_id, &num_sms, &status);
  if (rc != TG_OK) return rc;
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  int32_t* counts = reinterpret_cast<int32_t*>(scratch);
  if (num_experts <= kRouteSmallMaxExperts && n > 0 && n <= kRouteSmallMaxPairs) {
    int32_t* sid = reinterpret_cast<int32_t*>(sorted_ids);
    int32_t* ps = reinterpret_cast<int32_t*>(pos);
    float* ws = reinterpret_cast<float*>(w_sorted);
    int32_t* ind = reinterpret_cast<int32_t*>(m_indptr);
    const int wd = topk_weights != nullptr ? topk_weights->dtype : TG_F32;
    const void* wp = topk_weights != nullptr ? reinterpret_cast<const void*>(topk_weights->ptr) : nullptr;
    const int n32 = static_cast<int>(n);
#define TG_ROUTE_SMALL(IdT, WT)                                                                                      \
  moe_route_small_kernel<IdT, WT><<<1, 1024, 0, cs>>>(reinterpret_cast<const IdT*>(topk_ids->ptr),                    \
                                                      reinterpret_cast<const WT*>(wp), n32, num_experts, ind, sid, ps, ws)
    if (topk_ids->dtype == TG_I64) {
      if (wd == TG_BF16) TG_ROUTE_SMALL(int64_t, __nv_bfloat16);
      else if (wd == TG_F16) TG_ROUTE_SMALL(int64_t, __half);
      else TG_ROUTE_SMALL(int64_t, float);
    } else {
      if (wd == TG_BF16) TG_ROUTE_SMALL(int32_t, __nv_bfloat16);
      else if (wd == TG_F16) TG_ROUTE_SMALL(int32_t, __half);
      else TG_ROUTE_SMALL(int32_t, float);
    }
#undef TG_ROUTE_SMALL
    return launch_status("moe route");
  }
  if (cudaMemsetAsync(counts, 0, sizeof(int32_t) * static_cast<size_t>(num_experts), cs) != cudaSuccess)
    return launch_status("moe route (clear)");
  const int grid = grid_for(n, 256, num_sms, 8);
  const bool i64 = topk_ids->dtype == TG_I64;
  if (n > 0) {
    if (i64)
      moe_count_kernel<int64_t><<<grid, 256, 0, cs>>>(reinterpret_cast<const int64_t*>(topk_ids->ptr), n, num_experts, counts);
    else
      moe_count_kernel<int32_t><<<grid, 256, 0, cs>>>(reinterpret_cast<const int32_t*>(topk_ids->ptr), n, num_experts, counts);
  }
  moe_scan_kernel<<<1, 1024, 0, cs>>>(counts, num_experts, reinterpret_cast<int32_t*>(m_indptr));
  if (n > 0) {
    int32_t* sid = reinterpret_cast<int32_t*>(sorted_ids);
    int32_t* ps = reinterpret_cast<int32_t*>(pos);
    float* ws = reinterpret_cast<float*>(w_sorted);
    const int wd = topk_weights != nullptr ? topk_weights->dtype : TG_F32;
    const void* wp = topk_weights != nullptr ? reinterpret_cast<const void*>(topk_weights->ptr) : nullptr;
#define TG_PLACE(IdT, WT)                                                                                       \
  moe_place_kernel<IdT, WT><<<grid, 256, 0, cs>>>(reinterpret_cast<const IdT*>(topk_ids->ptr),                   \
                                                  reinterpret_cast<const WT*>(wp), n, num_experts, counts, sid, ps, ws)
    if (i64) {
      if (wd == TG_BF16) TG_PLACE(int64_t, __nv_bfloat16);
      else if (wd == TG_F16) TG_PLACE(int64_t, __half);
      else TG_PLACE(int64_t, float);
    } else {
      if (wd == TG_BF16) TG_PLACE(int32_t, __nv_bfloat16);
      else if (wd == TG_F16) TG_PLACE(int32_t, __half);
      else TG_PLACE(int32_t, float);
    }
#undef TG_PLACE
  }
  return launch_status("moe route");
}

TG_API int32_t tg_moe_permute_rows(const TgTensorDesc* A_sorted, const TgTensorDesc* As_sorted, const TgTensorDesc* A,
                                   const TgTensorDesc* As, uint64_t sorted_ids, uint64_t m_indptr, int32_t num_experts,
                                   int32_t topk, int32_t device_id, uint64_t stream) {
  if (A_sorted == nullptr || As_sorted == nullptr || A == nullptr || As == nullptr) return api_fail(TG_ERR_NULL, "a descriptor is null");
  if (A->dtype != TG_F8E4M3 || A_sorted->dtype != TG_F8E4M3) return api_fail(TG_ERR_DTYPE, "A and A_sorted must be float8_e4m3fn");
  if (As->dtype != TG_F32 || As_sorted->dtype != TG_F32) return api_fail(TG_ERR_DTYPE, "scales must be f32");
  if (A->ndim != 2 || As->ndim != 2 || !contiguous_2d(A_sorted) || !contiguous_2d(As_sorted))
    return api_fail(TG_ERR_ARGS, "A, As must be 2-D and the outputs contiguous 2-D");
  const int64_t T = A->shape[0], K = A->shape[1], KB = As->shape[1], R = A_sorted->shape[0];
  if (A->strides[1] != 1 || As->strides[1] != 1 || A->strides[0] < K || As->strides[0] < KB)
    return api_fail(TG_ERR_ARGS, "rows of A and As must be contiguous");
  if (K % 16 != 0 || (A->strides[0] & 15) != 0) return api_fail(TG_ERR_ALIGN, "K and the row pitch of A must be multiples of 16");
  if (As->shape[0] != T || A_sorted->shape[1] != K || As_sorted->shape[0] != R || As_sorted->shape[1] != KB)
    return api_fail(TG_ERR_ARGS, "shapes of A, As, A_sorted, As_sorted do not fit together");
  if (topk < 1 || num_experts < 1) return api_fail(TG_ERR_ARGS, "topk and num_experts must be positive");
  if (R > T * topk) return api_fail(TG_ERR_ARGS, "A_sorted has more rows than tokens x top_k");
  if (sorted_ids == 0 || m_indptr == 0) return api_fail(TG_ERR_NULL, "sorted_ids / m_indptr is null");
  if (R == 0 || T == 0) return TG_OK;
  if (A->ptr == 0 || As->ptr == 0 || A_sorted->ptr == 0 || As_sorted->ptr == 0) return api_fail(TG_ERR_NULL, "data pointer is null");
  if ((A->ptr | A_sorted->ptr) & 15u) return api_fail(TG_ERR_ALIGN, "A and A_sorted must be 16-byte aligned");
  Guard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return api_fail(TG_ERR_DEVICE, "cannot select the CUDA device");
  }
  int num_sms = 0;
  int32_t* status = nullptr;
  int32_t rc = api_init_device(device_id, &num_sms, &status);
  if (rc != TG_OK) return rc;
  const int grid = grid_for(R, 1, num_sms, 16);
  moe_permute_rows_kernel<<<grid, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<uint8_t*>(A_sorted->ptr), reinterpret_cast<float*>(As_sorted->ptr),
      reinterpret_cast<const uint8_t*>(A->ptr), reinterpret_cast<const float*>(As->ptr),
      reinterpret_cast<const int32_t*>(sorted_ids), reinterpret_cast<const int32_t*>(m_indptr), num_experts, topk, K,
      A->strides[0], static_cast<int>(KB), As->strides[0]);
  return launch_status("moe permute rows");
}

TG_API int32_t tg_moe_quant_permute_rows(const TgTensorDesc* A_sorted, const TgTensorDesc* As_sorted, const TgTensorDesc* X,
                                         uint64_t pos, int32_t topk, int32_t device_id, uint64_t stream) {
  if (A_sorted == nullptr || As_sorted == nullptr || X == nullptr) return api_fail(TG_ERR_NULL, "a descriptor is null");
  if (X->dtype != TG_BF16 && X->dtype != TG_F16) return api_fail(TG_ERR_DTYPE, "X must be bf16 or f16");
  if (A_sorted->dtype != TG_F8E4M3) return api_fail(TG_ERR_DTYPE, "A_sorted must be float8_e4m3fn");
  if (As_sorted->dtype != TG_F32) return api_fail(TG_ERR_DTYPE, "As_sorted must be f32");
  if (!contiguous_2d(A_sorted) || !contiguous_2d(As_sorted) || !contiguous_2d(X))
    return api_fail(TG_ERR_ARGS, "A_sorted, As_sorted and X must be contiguous 2-D");
  const int64_t T = X->shape[0], H = X->shape[1], R = A_sorted->shape[0];
  if (H <= 0 || H % 128 != 0) return api_fail(TG_ERR_ARGS, "the hidden size must be a positive multiple of 128");
  if (A_sorted->shape[1] != H || As_sorted->shape[0] != R || As_sorted->shape[1] != H / 128)
    return api_fail(TG_ERR_ARGS, "A_sorted must be [rows, hidden] and As_sorted [rows, hidden / 128]");
  if (topk < 1 || R > T * topk) return api_fail(TG_ERR_ARGS, "A_sorted has more rows than tokens x top_k");
  if (pos == 0) return api_fail(TG_ERR_NULL, "pos is null");
  if (pos & 3u) return api_fail(TG_ERR_ALIGN, "pos must be 4-byte aligned");
  if (T == 0 || R == 0) return TG_OK;
  if (X->ptr == 0 || A_sorted->ptr == 0 || As_sorted->ptr == 0) return api_fail(TG_ERR_NULL, "data pointer is null");
  if ((X->ptr | A_sorted->ptr) & 15u) return api_fail(TG_ERR_ALIGN, "X and A_sorted must be 16-byte aligned");
  if (As_sorted->ptr & 3u) return api_fail(TG_ERR_ALIGN, "As_sorted must be 4-byte aligned");
  Guard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return api_fail(TG_ERR_DEVICE, "cannot select the CUDA device");
  }
  int num_sms = 0;
  int32_t* status = nullptr;
  int32_t rc = api_init_device(device_id, &num_sms, &status);
  if (rc != TG_OK) return rc;
  const int grid = grid_for(T * (H / 16), 256, num_sms, 8);
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  if (X->dtype == TG_BF16)
    moe_quant_permute_kernel<__nv_bfloat16><<<grid, 256, 0, cs>>>(
        reinterpret_cast<uint8_t*>(A_sorted->ptr), reinterpret_cast<float*>(As_sorted->ptr),
        reinterpret_cast<const __nv_bfloat16*>(X->ptr), reinterpret_cast<const int32_t*>(pos), T, topk, H);
  else
    moe_quant_permute_kernel<__half><<<grid, 256, 0, cs>>>(
        reinterpret_cast<uint8_t*>(A_sorted->ptr), reinterpret_cast<float*>(As_sorted->ptr),
        reinterpret_cast<const __half*>(X->ptr), reinterpret_cast<const int32_t*>(pos), T, topk, H);
  return launch_status("moe quant_permute_rows");
}

TG_API int32_t tg_moe_silu_mul_quant(const TgTensorDesc* Y, const TgTensorDesc* S, const TgTensorDesc* X, uint64_t m_indptr,
                                     int32_t num_experts, int32_t mode, int32_t device_id, uint64_t stream) {
  if (Y == nullptr || S == nullptr || X == nullptr) return api_fail(TG_ERR_NULL, "a descriptor is null");
  if (X->dtype != TG_BF16 && X->dtype != TG_F16) return api_fail(TG_ERR_DTYPE, "X must be bf16 or f16");
  if (Y->dtype != TG_F8E4M3) return api_fail(TG_ERR_DTYPE, "Y must be float8_e4m3fn");
  if (S->dtype != TG_F32) return api_fail(TG_ERR_DTYPE, "S must be f32");
  if (!contiguous_2d(X) || !contiguous_2d(Y) || !contiguous_2d(S)) return api_fail(TG_ERR_ARGS, "X, Y and S must be contiguous 2-D");
  const int64_t R = X->shape[0], I = X->shape[1] / 2;
  if (X->shape[1] != 2 * I || I % 128 != 0 || I == 0) return api_fail(TG_ERR_ARGS, "X must be [rows, 2 * I] with I a multiple of 128");
  if (Y->shape[0] != R || Y->shape[1] != I || S->shape[0] != R || S->shape[1] != I / 128)
    return api_fail(TG_ERR_ARGS, "Y must be [rows, I] and S [rows, I / 128]");
  if (mode < 0 || mode > 3)
    return api_fail(TG_ERR_ARGS, "mode must be 0 (scale 1) or 1 (amax / 448 per 128 elements), plus 2 for interleaved gate / up blocks");
  if (m_indptr == 0) return api_fail(TG_ERR_NULL, "m_indptr is null");
  if (num_experts < 1) return api_fail(TG_ERR_ARGS, "num_experts must be positive");
  if (R == 0) return TG_OK;
  if (X->ptr == 0 || Y->ptr == 0 || S->ptr == 0) return api_fail(TG_ERR_NULL, "data pointer is null");
  if ((X->ptr & 15u) || (Y->ptr & 15u)) return api_fail(TG_ERR_ALIGN, "X and Y must be 16-byte aligned");
  Guard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return api_fail(TG_ERR_DEVICE, "cannot select the CUDA device");
  }
  int num_sms = 0;
  int32_t* status = nullptr;
  int32_t rc = api_init_device(device_id, &num_sms, &status);
  if (rc != TG_OK) return rc;
  const int grid = grid_for(R * (I / 128), 32, num_sms, 8);  // 32 groups of 128 outputs per 256-thread block
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  if (X->dtype == TG_BF16)
    moe_silu_mul_quant_kernel<__nv_bfloat16><<<grid, 256, 0, cs>>>(
        reinterpret_cast<uint8_t*>(Y->ptr), reinterpret_cast<float*>(S->ptr), reinterpret_cast<const __nv_bfloat16*>(X->ptr),
        reinterpret_cast<const int32_t*>(m_indptr), num_experts, I, mode);
  else
    moe_silu_mul_quant_kernel<__half><<<grid, 256, 0, cs>>>(
        reinterpret_cast<uint8_t*>(Y->ptr), reinterpret_cast<float*>(S->ptr), reinterpret_cast<const __half*>(X->ptr),
        reinterpret_cast<const int32_t*>(m_indptr), num_experts, I, mode);
  return launch_status("moe silu_mul_quant");
}

TG_API int32_t tg_moe_unpermute_sum(const TgTensorDesc* out, const TgTensorDesc* C, uint64_t pos, int32_t topk,
                                    int32_t device_id, uint64_t stream) {
  if (out == nullptr || C == nullptr) return api_fail(TG_ERR_NULL, "a descriptor is null");
  if ((C->dtype != TG_BF16 && C->dtype != TG_F16) || out->dtype != C->dtype)
    return api_fail(TG_ERR_DTYPE, "C and out must both be bf16 or both f16");
  if (!contiguous_2d(out) || !contiguous_2d(C)) return api_fail(TG_ERR_ARGS, "out and C must be contiguous 2-D");
  const int64_t T = out->shape[0], H = out->shape[1];
  if (C->shape[1] != H || H % 8 != 0) return api_fail(TG_ERR_ARGS, "C must have out's width, a multiple of 8");
  if (topk < 1 || C->shape[0] > T * topk) return api_fail(TG_ERR_ARGS, "C has more rows than tokens x top_k");
  if (pos == 0) return api_fail(TG_ERR_NULL, "pos is null");
  if (T == 0 || H == 0) return TG_OK;
  if (out->ptr == 0 || (C->shape[0] > 0 && C->ptr == 0)) return api_fail(TG_ERR_NULL, "data pointer is null");
  if ((out->ptr | C->ptr) & 15u) return api_fail(TG_ERR_ALIGN, "out and C must be 16-byte aligned");
  Guard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return api_fail(TG_ERR_DEVICE, "cannot select the CUDA device");
  }
  int num_sms = 0;
  int32_t* status = nullptr;
  int32_t rc = api_init_device(device_id, &num_sms, &status);
  if (rc != TG_OK) return rc;
  const int grid = grid_for(T * (H / 8), 256, num_sms, 8);
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  if (C->dtype == TG_BF16)
    moe_unpermute_sum_kernel<__nv_bfloat16><<<grid, 256, 0, cs>>>(
        reinterpret_cast<__nv_bfloat16*>(out->ptr), reinterpret_cast<const __nv_bfloat16*>(C->ptr),
        reinterpret_cast<const int32_t*>(pos), T, topk, H);
  else
    moe_unpermute_sum_kernel<__half><<<grid, 256, 0, cs>>>(reinterpret_cast<__half*>(out->ptr),
                                                           reinterpret_cast<const __half*>(C->ptr),
                                                           reinterpret_cast<const int32_t*>(pos), T, topk, H);
  return launch_status("moe unpermute_sum");
}

}  // extern "C"

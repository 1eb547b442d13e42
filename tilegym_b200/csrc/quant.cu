// e4m3 quantisers and the block dequantiser that sit either side of the FP8
// GEMMs.  All of them are single-pass streaming kernels bound by HBM
// bandwidth.  Results equal an IEEE division (div.rn) followed by the cast: an
// approximate reciprocal alone moves values across e4m3 rounding boundaries,
// so the reciprocal path of tg_quant_common.cuh redoes exactly the elements
// that sit next to a boundary with div.rn.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <type_traits>

#include "tg_internal.h"
#include "tg_quant_common.cuh"

namespace tg {

namespace {

constexpr float kE4M3Max = 448.0f;

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float from_e4m3(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Loads 4 consecutive elements as fp32 (8- or 16-byte access).
template <typename T>
__device__ __forceinline__ void load4(const T* src, float (&v)[4]) {
  if constexpr (sizeof(T) == 4) {
    float4 t = *reinterpret_cast<const float4*>(src);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    uint2 t = *reinterpret_cast<const uint2*>(src);
    const T* e = reinterpret_cast<const T*>(&t);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = to_f32<T>(e[j]);
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// act_quant (1 x 128, src/tilegym/suites/unsloth/cutile/fp8.py:77-120: amax/448, 1.0 for a zero block, IEEE
// division, cast to e4m3) is the per-token group kernel of group_quant.cu with 16 lanes per group.

// ----------------------------------------------------------- weight_dequant
// y[i,j] = x[i,j] * s[i/128, j/128]; each thread converts 16 consecutive
// columns (one 16-byte load) when N % 16 == 0, else one element.
// Follows src/tilegym/suites/unsloth/cutile/fp8.py:36-71.
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) tg_weight_dequant_kernel(T* __restrict__ y, const uint8_t* __restrict__ x,
                                                                const float* __restrict__ s, int64_t M, int64_t N,
                                                                int64_t lds, bool vec) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (vec) {
    const int64_t groups_per_row = N / 16;
    const int64_t total = M * groups_per_row;
    for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < total; g += stride) {
      const int64_t i = g / groups_per_row;
      const int64_t j = (g - i * groups_per_row) * 16;
      const float sc = __ldg(s + (i >> 7) * lds + (j >> 7));
      const uint4 raw = *reinterpret_cast<const uint4*>(x + i * N + j);
      const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
      alignas(16) T out[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) out[k] = from_f32<T>(from_e4m3(b[k]) * sc);
      uint4* dst = reinterpret_cast<uint4*>(y + i * N + j);
      const uint4* src = reinterpret_cast<const uint4*>(out);
#pragma unroll
      for (int k = 0; k < static_cast<int>(sizeof(T)); ++k) dst[k] = src[k];
    }
  } else {
    const int64_t total = M * N;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
      const int64_t i = e / N, j = e - i * N;
      y[e] = from_f32<T>(from_e4m3(x[e]) * __ldg(s + (i >> 7) * lds + (j >> 7)));
    }
  }
}

// ----------------------------------------------------------- per-tensor quant
// Pass 1: amax of |x| via an atomic max on the fp32 bit pattern (monotone for
// non-negative floats).  Pass 2: scale = amax/448 (1.0 if zero), quantise.
template <typename T>
__global__ void __launch_bounds__(256) tg_amax_kernel(const T* __restrict__ x, int64_t numel, uint32_t* amax_bits) {
  float m = 0.f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t n4 = numel / 4;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < n4; g += stride) {
    float v[4];
    load4<T>(x + g * 4, v);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
  }
  for (int64_t e = n4 * 4 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < numel; e += stride)
    m = fmaxf(m, fabsf(to_f32<T>(x[e])));
  m = warp_max(m);
  __shared__ float wm[8];
  if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? wm[threadIdx.x] : 0.f;
    t = warp_max(t);
    if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(t));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) tg_quant_pertensor_kernel(uint8_t* __restrict__ y, float* scale_out,
                                                                 const T* __restrict__ x, int64_t numel,
                                                                 const uint32_t* amax_bits) {
  float scale = __fdiv_rn(__uint_as_float(*amax_bits), kE4M3Max);
  if (scale == 0.f) scale = 1.0f;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t n4 = numel / 4;
  // x / scale through the shared reciprocal with the exactness check of tg_quant_common.cuh; the e4m3 cast
  // saturates at +-448 by itself, which is the clamp
  const bool tame = q8_scale_is_tame(scale);
  const float r = __frcp_rn(scale);
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < n4; g += 2 * stride) {
    float v[4], w[4];
    const bool second = g + stride < n4;
    load4<T>(x + g * 4, v);
    if (second) load4<T>(x + (g + stride) * 4, w);
    *reinterpret_cast<uint32_t*>(y + g * 4) =
        q8_pair<kQ8E4M3>(v[0], v[1], scale, r, tame, -kE4M3Max, kE4M3Max) |
        (q8_pair<kQ8E4M3>(v[2], v[3], scale, r, tame, -kE4M3Max, kE4M3Max) << 16);
    if (second)
      *reinterpret_cast<uint32_t*>(y + (g + stride) * 4) =
          q8_pair<kQ8E4M3>(w[0], w[1], scale, r, tame, -kE4M3Max, kE4M3Max) |
          (q8_pair<kQ8E4M3>(w[2], w[3], scale, r, tame, -kE4M3Max, kE4M3Max) << 16);
  }
  for (int64_t e = n4 * 4 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < numel; e += stride) {
    float qv = fminf(fmaxf(__fdiv_rn(to_f32<T>(x[e]), scale), -kE4M3Max), kE4M3Max);
    y[e] = to_e4m3(qv);
  }
}

// The same pass for 16-bit inputs whose size and addresses allow 16 elements per thread (two 16-byte loads, one
// 16-byte store): the tensor's scale is RN(amax / 448) of a 16-bit amax, which is the form the test-free quotient
// of tg_quant_common.cuh is verified for.
template <typename T>
__global__ void __launch_bounds__(256) tg_quant_pertensor16_kernel(uint8_t* __restrict__ y, float* scale_out,
                                                                   const T* __restrict__ x, int64_t n_chunks,
                                                                   const uint32_t* amax_bits) {
  q8_allow_dependents();
  float scale = __fdiv_rn(__uint_as_float(*amax_bits), kE4M3Max);
  if (scale == 0.f) scale = 1.0f;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
  const bool tame = q8_scale_is_tame(scale);
  const float r = __frcp_rn(scale);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  uint4 n0 = make_uint4(0u, 0u, 0u, 0u), n1 = n0;
  if (c < n_chunks) {
    n0 = __ldcs(reinterpret_cast<const uint4*>(x + c * 16));
    n1 = __ldcs(reinterpret_cast<const uint4*>(x + c * 16) + 1);
  }
  for (; c < n_chunks; c += stride) {
    const uint4 t0 = n0, t1 = n1;
    if (c + stride < n_chunks) {  // the next chunk is requested before this one is converted
      n0 = __ldcs(reinterpret_cast<const uint4*>(x + (c + stride) * 16));
      n1 = __ldcs(reinterpret_cast<const uint4*>(x + (c + stride) * 16) + 1);
    }
    const uint32_t w[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
    uint32_t out[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 x0, x1;
      if constexpr (sizeof(T) == 2 && !std::is_same<T, __half>::value) {
        x0 = make_float2(__uint_as_float(w[2 * k] << 16), __uint_as_float(w[2 * k] & 0xffff0000u));
        x1 = make_float2(__uint_as_float(w[2 * k + 1] << 16), __uint_as_float(w[2 * k + 1] & 0xffff0000u));
      } else {
        x0 = __half22float2(*reinterpret_cast<const __half2*>(&w[2 * k]));
        x1 = __half22float2(*reinterpret_cast<const __half2*>(&w[2 * k + 1]));
      }
      if (tame) {
        const float2 q0 = q8_quot2(x0, scale, r), q1 = q8_quot2(x1, scale, r);
        out[k] = q8_cast2<kQ8E4M3>(q0.x, q0.y, -kE4M3Max, kE4M3Max) | (q8_cast2<kQ8E4M3>(q1.x, q1.y, -kE4M3Max, kE4M3Max) << 16);
      } else {
        out[k] = q8_pair<kQ8E4M3>(x0.x, x0.y, scale, r, false, -kE4M3Max, kE4M3Max) |
                 (q8_pair<kQ8E4M3>(x1.x, x1.y, scale, r, false, -kE4M3Max, kE4M3Max) << 16);
      }
    }
    __stcs(reinterpret_cast<uint4*>(y + c * 16), make_uint4(out[0], out[1], out[2], out[3]));
  }
}

// Small inputs (decode-sized activations) in ONE launch instead of clear + amax + quantise: a thread-block cluster
// of up to 8 CTAs x 512 threads holds the whole tensor in registers (up to 64 elements per thread), reduces |x| to
// the block maximum, exchanges the block maxima through distributed shared memory (one cluster barrier), and
// quantises what it holds.  Same arithmetic as the two-pass form (amax / 448 by IEEE division, 1.0 for all zeros,
// test-free exact quotient), so the bytes are the same.  16-bit inputs, 16-byte aligned, size a multiple of 8.
constexpr int kFusedThreads = 512;
constexpr int kFusedVecs = 8;  // 16-byte vectors (8 elements each) a thread may hold: 32 registers of data
template <typename T>
__global__ void __launch_bounds__(kFusedThreads, 1)
    tg_quant_pertensor_fused_kernel(uint8_t* __restrict__ y, float* scale_out, const T* __restrict__ x, int64_t n_vecs) {
  __shared__ float warp_max_s[32];
  __shared__ float cta_max_s[8];  // one slot per CTA of the cluster, written by that CTA into every peer
  q8_allow_dependents();
  uint32_t n_ctas, rank;
  asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(n_ctas));
  asm volatile("mov.u32 %0, %%cluster_ctaid.x;" : "=r"(rank));
  // "this CTA runs": a peer's shared memory may only be written once that peer has started (waited for below)
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  const int64_t stride = static_cast<int64_t>(n_ctas) * kFusedThreads;
  const int64_t first = static_cast<int64_t>(rank) * kFusedThreads + threadIdx.x;
  uint4 v[kFusedVecs];
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < kFusedVecs; ++i) {
    const int64_t c = first + i * stride;
    v[i] = make_uint4(0u, 0u, 0u, 0u);
    if (c < n_vecs) v[i] = __ldg(reinterpret_cast<const uint4*>(x) + c);
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f;
      if constexpr (std::is_same<T, __half>::value) f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
      else f = make_float2(__uint_as_float(w[j] << 16), __uint_as_float(w[j] & 0xffff0000u));
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) warp_max_s[threadIdx.x >> 5] = m;
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // every CTA of the cluster has started
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = warp_max(threadIdx.x < kFusedThreads / 32 ? warp_max_s[threadIdx.x] : 0.f);
    // lane r publishes this CTA's maximum in slot `rank` of CTA r's table
    if (threadIdx.x < n_ctas) {
      uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(&cta_max_s[rank])), remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(threadIdx.x));
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(t) : "memory");
    }
  }
  // every CTA's maximum is in every table after this barrier (also orders the warp_max_s use inside the CTA)
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  float amax = 0.f;
  for (uint32_t r = 0; r < n_ctas; ++r) amax = fmaxf(amax, cta_max_s[r]);
  float scale = __fdiv_rn(amax, kE4M3Max);
  if (scale == 0.f) scale = 1.0f;
  if (rank == 0 && threadIdx.x == 0) *scale_out = scale;
  const bool tame = q8_scale_is_tame(scale);
  const float r = __frcp_rn(scale);
#pragma unroll
  for (int i = 0; i < kFusedVecs; ++i) {
    const int64_t c = first + i * stride;
    if (c >= n_vecs) break;
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
    uint32_t out[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      float2 x0, x1;
      if constexpr (std::is_same<T, __half>::value) {
        x0 = __half22float2(*reinterpret_cast<const __half2*>(&w[2 * k]));
        x1 = __half22float2(*reinterpret_cast<const __half2*>(&w[2 * k + 1]));
      } else {
        x0 = make_float2(__uint_as_float(w[2 * k] << 16), __uint_as_float(w[2 * k] & 0xffff0000u));
        x1 = make_float2(__uint_as_float(w[2 * k + 1] << 16), __uint_as_float(w[2 * k + 1] & 0xffff0000u));
      }
      if (tame) {
        const float2 q0 = q8_quot2(x0, scale, r), q1 = q8_quot2(x1, scale, r);
        out[k] = q8_cast2<kQ8E4M3>(q0.x, q0.y, -kE4M3Max, kE4M3Max) | (q8_cast2<kQ8E4M3>(q1.x, q1.y, -kE4M3Max, kE4M3Max) << 16);
      } else {
        out[k] = q8_pair<kQ8E4M3>(x0.x, x0.y, scale, r, false, -kE4M3Max, kE4M3Max) |
                 (q8_pair<kQ8E4M3>(x1.x, x1.y, scale, r, false, -kE4M3Max, kE4M3Max) << 16);
      }
    }
    *(reinterpret_cast<uint2*>(y) + c) = make_uint2(out[0], out[1]);
  }
}

template <typename T>
cudaError_t launch_quant_pertensor_fused(uint8_t* y, float* scale_out, const T* x, int64_t numel, cudaStream_t stream) {
  const int64_t n_vecs = numel / 8;
  const int64_t per_cta = static_cast<int64_t>(kFusedThreads) * kFusedVecs;
  int ctas = static_cast<int>((n_vecs + per_cta - 1) / per_cta);
  if (ctas < 1) ctas = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
  cfg.blockDim = dim3(kFusedThreads, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(ctas);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, tg_quant_pertensor_fused_kernel<T>, y, scale_out, x, n_vecs);
}

// ------------------------------------------------------- 128x128 weight quant
// One CTA per 128 x 128 block; thread t owns columns 4*(t%32) .. +3 of rows
// t/32, t/32+8, ... (16 rows), keeps them in registers across the block-wide
// amax reduction, then quantises.  Edge blocks treat missing elements as zero.
template <typename T>
__global__ void __launch_bounds__(256) tg_weight_quant_block_kernel(uint8_t* __restrict__ y, float* __restrict__ s,
                                                                    const T* __restrict__ x, int64_t N, int64_t K,
                                                                    int64_t lds, bool vec) {
  const int bi = blockIdx.y, bj = blockIdx.x;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t col = static_cast<int64_t>(bj) * 128 + lane * 4;
  float v[16][4];
  float amax = 0.f;
#pragma unroll
  for (int r = 0; r < 16; ++r) {
    const int64_t row = static_cast<int64_t>(bi) * 128 + w + 8 * r;
#pragma unroll
    for (int j = 0; j < 4; ++j) v[r][j] = 0.f;
    if (row < N) {
      if (vec && col + 4 <= K) {
        load4<T>(x + row * K + col, v[r]);
      } else {
        for (int j = 0; j < 4; ++j)
          if (col + j < K) v[r][j] = to_f32<T>(x[row * K + col + j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(v[r][j]));
  }
  amax = warp_max(amax);
  __shared__ float wm[8];
  if (lane == 0) wm[w] = amax;
  __syncthreads();
  amax = wm[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, wm[i]);
  float scale = __fdiv_rn(amax, kE4M3Max);
  if (scale == 0.f) scale = 1.0f;
  if (threadIdx.x == 0) s[static_cast<int64_t>(bi) * lds + bj] = scale;
#pragma unroll
  for (int r = 0; r < 16; ++r) {
    const int64_t row = static_cast<int64_t>(bi) * 128 + w + 8 * r;
    if (row >= N) continue;
    uint8_t qb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float qv = fminf(fmaxf(__fdiv_rn(v[r][j], scale), -kE4M3Max), kE4M3Max);
      qb[j] = to_e4m3(qv);
    }
    if (vec && col + 4 <= K) {
      *reinterpret_cast<uint32_t*>(y + row * K + col) =
          static_cast<uint32_t>(qb[0]) | (static_cast<uint32_t>(qb[1]) << 8) | (static_cast<uint32_t>(qb[2]) << 16) |
          (static_cast<uint32_t>(qb[3]) << 24);
    } else {
      for (int j = 0; j < 4; ++j)
        if (col + j < K) y[row * K + col + j] = qb[j];
    }
  }
}

int grid_for(int64_t work_items, int threads, int cap) {
  int64_t g = (work_items + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return static_cast<int>(g);
}

}  // namespace

// (launch_act_quant lives with the group quantiser in group_quant.cu: the 1 x 128 quantiser is that kernel
// with 16 lanes per group.)

cudaError_t launch_weight_dequant(void* y, int y_dtype, const uint8_t* x, const float* s, int64_t M, int64_t N,
                                  int64_t lds, cudaStream_t stream) {
  if (M == 0 || N == 0) return cudaSuccess;
  const int esz = (y_dtype == TG_F32) ? 4 : 2;
  const bool vec = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) &&
                   ((reinterpret_cast<uintptr_t>(y) & 15u) == 0) && ((N * esz) % 16 == 0);
  const int64_t items = vec ? M * (N / 16) : M * N;
  const int grid = grid_for(items, 256, 148 * 16);
  if (y_dtype == TG_BF16)
    tg_weight_dequant_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(y), x, s, M, N, lds, vec);
  else if (y_dtype == TG_F16)
    tg_weight_dequant_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<__half*>(y), x, s, M, N, lds, vec);
  else
    tg_weight_dequant_kernel<float><<<grid, 256, 0, stream>>>(static_cast<float*>(y), x, s, M, N, lds, vec);
  return cudaGetLastError();
}

cudaError_t launch_quant_pertensor(uint8_t* y, float* scale_out, const void* x, int x_dtype, int64_t numel,
                                   uint32_t* amax_scratch, int num_sms, bool allow_single_launch, cudaStream_t stream) {
  // up to 8 CTAs x 512 threads x 64 elements (262144 in all): the whole tensor fits one cluster's registers
  const bool fused = allow_single_launch && x_dtype != TG_F32 && numel > 0 && numel % 8 == 0 && numel <= 8ll * kFusedThreads * kFusedVecs * 8 &&
                     ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(y) & 7u) == 0);
  if (fused) {
    if (x_dtype == TG_BF16)
      return launch_quant_pertensor_fused(y, scale_out, static_cast<const __nv_bfloat16*>(x), numel, stream);
    return launch_quant_pertensor_fused(y, scale_out, static_cast<const __half*>(x), numel, stream);
  }
  cudaError_t e = cudaMemsetAsync(amax_scratch, 0, sizeof(uint32_t), stream);
  if (e != cudaSuccess) return e;
  const int grid = grid_for((numel + 3) / 4, 256, num_sms * 8);
  const bool wide = x_dtype != TG_F32 && numel % 16 == 0 && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) &&
                    ((reinterpret_cast<uintptr_t>(y) & 15u) == 0);
  const int grid16 = grid_for(numel / 16, 256, num_sms * 16);
  if (x_dtype == TG_BF16) {
    const auto* xx = static_cast<const __nv_bfloat16*>(x);
    tg_amax_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(xx, numel, amax_scratch);
    if (wide) tg_quant_pertensor16_kernel<__nv_bfloat16><<<grid16, 256, 0, stream>>>(y, scale_out, xx, numel / 16, amax_scratch);
    else tg_quant_pertensor_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(y, scale_out, xx, numel, amax_scratch);
  } else if (x_dtype == TG_F16) {
    const auto* xx = static_cast<const __half*>(x);
    tg_amax_kernel<__half><<<grid, 256, 0, stream>>>(xx, numel, amax_scratch);
    if (wide) tg_quant_pertensor16_kernel<__half><<<grid16, 256, 0, stream>>>(y, scale_out, xx, numel / 16, amax_scratch);
    else tg_quant_pertensor_kernel<__half><<<grid, 256, 0, stream>>>(y, scale_out, xx, numel, amax_scratch);
  } else {
    const auto* xx = static_cast<const float*>(x);
    tg_amax_kernel<float><<<grid, 256, 0, stream>>>(xx, numel, amax_scratch);
    tg_quant_pertensor_kernel<float><<<grid, 256, 0, stream>>>(y, scale_out, xx, numel, amax_scratch);
  }
  return cudaGetLastError();
}

cudaError_t launch_weight_quant_block(uint8_t* y, float* s, const void* x, int x_dtype, int64_t N, int64_t K,
                                      int64_t lds, cudaStream_t stream) {
  if (N == 0 || K == 0) return cudaSuccess;
  dim3 grid(static_cast<unsigned>((K + 127) / 128), static_cast<unsigned>((N + 127) / 128));
  const bool vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) &&
                   ((reinterpret_cast<uintptr_t>(y) & 3u) == 0);
  if (x_dtype == TG_BF16)
    tg_weight_quant_block_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(y, s, static_cast<const __nv_bfloat16*>(x), N, K, lds, vec);
  else if (x_dtype == TG_F16)
    tg_weight_quant_block_kernel<__half><<<grid, 256, 0, stream>>>(y, s, static_cast<const __half*>(x), N, K, lds, vec);
  else
    tg_weight_quant_block_kernel<float><<<grid, 256, 0, stream>>>(y, s, static_cast<const float*>(x), N, K, lds, vec);
  return cudaGetLastError();
}

}  // namespace tg

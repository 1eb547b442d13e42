// Pieces shared by the three FP8 GEMM kernels: tile geometry, the L2-friendly
// tile order, the status word, and the vectorised epilogue store.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tg_internal.h"
#include "tg_ptx.cuh"

namespace tg {

constexpr int kBM = 128;  // rows of A per tile = TMEM lanes
constexpr int kBK = 128;  // e4m3 elements per k-block = one 128-byte swizzle row = the quantisation block
constexpr int kUmmaK = 32;  // K of one kind::f8f6f4 instruction

// First expired wait wins; the host reads the word through tg_device_status().
__device__ __forceinline__ void report_timeout(int32_t* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// Linear tile id -> (tile_m, tile_n).  Tiles are walked in groups of kGroupM
// tile-rows, column by column inside a group, so that the CTAs running at the
// same moment share a few A row-panels and a band of B panels in L2 (the same
// raster the reference kernels use, src/tilegym/suites/unsloth/cutile/fp8.py:230-240).
constexpr int kGroupM = 8;
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = kGroupM * tiles_n;
  const int g = t / per_group;
  const int first_m = g * kGroupM;
  const int gsize = min(tiles_m - first_m, kGroupM);
  const int r = t - g * per_group;
  tm = first_m + r % gsize;
  tn = r / gsize;
}

__device__ __forceinline__ float load_bias(const void* bias, int dtype, int64_t col) {
  if (dtype == TG_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[col]);
  if (dtype == TG_F16) return __half2float(reinterpret_cast<const __half*>(bias)[col]);
  return reinterpret_cast<const float*>(bias)[col];
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Stores 8 consecutive fp32 values v[0..8) of one output row at columns
// col .. col+7 (clipped to N), converting to the output dtype; adds
// beta * C_old when beta != 0.  `vec_ok` says rows of C start 16-byte aligned.
__device__ __forceinline__ void store8(const GemmParams& p, int64_t row, int col, float (&v)[8], bool vec_ok) {
  const int n_valid = p.N - col;
  if (n_valid <= 0) return;
  const bool full = n_valid >= 8;
  if (p.out_dtype == TG_BF16) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col;
    if (full && vec_ok) {
      if (p.beta != 0.f) {
        uint4 old = *reinterpret_cast<const uint4*>(dst);
        const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(o2[j]);
          v[2 * j] = fmaf(p.beta, f.x, v[2 * j]);
          v[2 * j + 1] = fmaf(p.beta, f.y, v[2 * j + 1]);
        }
      }
      uint4 out;
      out.x = pack_bf16x2(v[0], v[1]);
      out.y = pack_bf16x2(v[2], v[3]);
      out.z = pack_bf16x2(v[4], v[5]);
      out.w = pack_bf16x2(v[6], v[7]);
      *reinterpret_cast<uint4*>(dst) = out;
    } else {
      for (int j = 0; j < 8 && j < n_valid; ++j) {
        float x = v[j];
        if (p.beta != 0.f) x = fmaf(p.beta, __bfloat162float(dst[j]), x);
        dst[j] = __float2bfloat16_rn(x);
      }
    }
  } else if (p.out_dtype == TG_F16) {
    __half* dst = reinterpret_cast<__half*>(p.C) + row * p.ldc + col;
    if (full && vec_ok) {
      if (p.beta != 0.f) {
        uint4 old = *reinterpret_cast<const uint4*>(dst);
        const __half2* o2 = reinterpret_cast<const __half2*>(&old);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __half22float2(o2[j]);
          v[2 * j] = fmaf(p.beta, f.x, v[2 * j]);
          v[2 * j + 1] = fmaf(p.beta, f.y, v[2 * j + 1]);
        }
      }
      uint4 out;
      out.x = pack_f16x2(v[0], v[1]);
      out.y = pack_f16x2(v[2], v[3]);
      out.z = pack_f16x2(v[4], v[5]);
      out.w = pack_f16x2(v[6], v[7]);
      *reinterpret_cast<uint4*>(dst) = out;
    } else {
      for (int j = 0; j < 8 && j < n_valid; ++j) {
        float x = v[j];
        if (p.beta != 0.f) x = fmaf(p.beta, __half2float(dst[j]), x);
        dst[j] = __float2half_rn(x);
      }
    }
  } else {
    float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col;
    if (full && vec_ok) {
      if (p.beta != 0.f) {
        float4 o0 = *reinterpret_cast<const float4*>(dst);
        float4 o1 = *reinterpret_cast<const float4*>(dst + 4);
        v[0] = fmaf(p.beta, o0.x, v[0]);
        v[1] = fmaf(p.beta, o0.y, v[1]);
        v[2] = fmaf(p.beta, o0.z, v[2]);
        v[3] = fmaf(p.beta, o0.w, v[3]);
        v[4] = fmaf(p.beta, o1.x, v[4]);
        v[5] = fmaf(p.beta, o1.y, v[5]);
        v[6] = fmaf(p.beta, o1.z, v[6]);
        v[7] = fmaf(p.beta, o1.w, v[7]);
      }
      *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      for (int j = 0; j < 8 && j < n_valid; ++j) {
        float x = v[j];
        if (p.beta != 0.f) x = fmaf(p.beta, dst[j], x);
        dst[j] = x;
      }
    }
  }
}

// Whether every row of C starts on a 16-byte boundary (so 8-element groups at
// column offsets that are multiples of 8 can use 16-byte accesses).
__device__ __forceinline__ bool c_rows_aligned(const GemmParams& p) {
  const int esz = (p.out_dtype == TG_F32) ? 4 : 2;
  return ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0) && (((p.ldc * esz) & 15) == 0);
}

// acc[j] += bias[bias_off + col0 + j] for the kCols columns col0 .. of one output row (columns >= N skipped).
// Every lane of a warp reads the same addresses, so the loads are broadcasts.
template <int kCols>
__device__ __forceinline__ void add_bias_cols(const GemmParams& p, float* acc, int col0, int64_t bias_off) {
  if (p.bias == nullptr) return;
  if (p.bias_dtype == TG_F32) {
    const float* b = reinterpret_cast<const float*>(p.bias) + bias_off + col0;
#pragma unroll
    for (int j = 0; j < kCols; ++j)
      if (col0 + j < p.N) acc[j] += __ldg(b + j);
  } else if (p.bias_dtype == TG_BF16) {
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + bias_off + col0;
#pragma unroll
    for (int j = 0; j < kCols; ++j)
      if (col0 + j < p.N) acc[j] += __bfloat162float(b[j]);
  } else {
    const __half* b = reinterpret_cast<const __half*>(p.bias) + bias_off + col0;
#pragma unroll
    for (int j = 0; j < kCols; ++j)
      if (col0 + j < p.N) acc[j] += __half2float(b[j]);
  }
}

// Final per-tensor epilogue of 32 accumulator columns of one row:
// out = acc * scale + bias[bias_off + col] (+ beta * C_old).  bias_off is the element offset of the row of a
// [groups, N] bias that applies (0 for a plain [N] bias).
__device__ __forceinline__ void epilogue_store32(const GemmParams& p, int64_t row, int col0, const float* acc,
                                                 float scale, bool vec_ok, int64_t bias_off = 0) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float v[8];
    const int col = col0 + 8 * g;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = acc[8 * g + j] * scale;
    if (p.bias != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (col + j < p.N) v[j] += load_bias(p.bias, p.bias_dtype, bias_off + col + j);
    }
    store8(p, row, col, v, vec_ok);
  }
}

// Bulk-store epilogue of one warp for two-byte outputs: the warp's 32 rows x 64 columns (v[0..64) of this
// lane's row) are converted, written to the warp's 4 KB staging buffer in the 128-byte-swizzle layout and
// sent with one bulk tensor store, which clips rows >= M and columns >= N.  `stage` must be 1024-byte
// aligned; the previous store out of it is waited for (its shared-memory reads only) before it is refilled.
__device__ __forceinline__ void stage_and_store64(const CUtensorMap* tmC, uint8_t* stage, int lane, const float* v,
                                                  int out_dtype, int col, int row0, int M, int N) {
  uint4 o[8];
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    if (out_dtype == TG_BF16) {
      o[g] = make_uint4(pack_bf16x2(v[8 * g], v[8 * g + 1]), pack_bf16x2(v[8 * g + 2], v[8 * g + 3]),
                        pack_bf16x2(v[8 * g + 4], v[8 * g + 5]), pack_bf16x2(v[8 * g + 6], v[8 * g + 7]));
    } else {
      o[g] = make_uint4(pack_f16x2(v[8 * g], v[8 * g + 1]), pack_f16x2(v[8 * g + 2], v[8 * g + 3]),
                        pack_f16x2(v[8 * g + 4], v[8 * g + 5]), pack_f16x2(v[8 * g + 6], v[8 * g + 7]));
    }
  }
  if (lane == 0) tma_store_wait_read<0>();
  __syncwarp();
  uint8_t* dst_row = stage + lane * 128;
#pragma unroll
  for (int g = 0; g < 8; ++g) *reinterpret_cast<uint4*>(dst_row + ((g ^ (lane & 7)) << 4)) = o[g];
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0 && col < N && row0 < M) {
    tma_store_2d(tmC, smem_u32(stage), col, row0);
    tma_store_commit();
  }
}

// ---- promotion helpers of the block-scaled kernels (acc += scale * partial on CUDA cores)
__device__ __forceinline__ void fma16x2(float2* acc, const uint32_t (&r)[32], float2 sc2) {
#pragma unroll
  for (int j = 0; j < 16; ++j)
    acc[j] = __ffma2_rn(make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), sc2, acc[j]);
}

// Activation scales of one row for k-blocks kb .. kb+3 (0 where out of range or the row is not in the problem).
__device__ __forceinline__ void load_as4(const float* as_row, int kb, int num_kb, bool in, bool vec, float (&a)[4]) {
  if (in && vec && kb + 4 <= num_kb) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(as_row + kb));
    a[0] = v.x;
    a[1] = v.y;
    a[2] = v.z;
    a[3] = v.w;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = (in && kb + i < num_kb) ? __ldg(as_row + kb + i) : 0.f;
  }
}

// Split-K arrival: after a warp has written its partial results and fenced,
// lane 0 bumps the counter of its (tile, slice); the warp that brings it to
// `splits` is the last one, resets the counter for the next call and reduces.
// No warp ever waits on another: the last arriver simply finds all partials.
__device__ __forceinline__ bool splitk_arrive_is_last(uint32_t* counter, int splits) {
  __threadfence();
  __syncwarp();
  uint32_t old = 0;
  if ((threadIdx.x & 31) == 0) {
    old = atomicAdd(counter, 1u);
    if (old == static_cast<uint32_t>(splits - 1)) atomicExch(counter, 0u);
  }
  old = __shfl_sync(0xffffffffu, old, 0);
  const bool last = (old == static_cast<uint32_t>(splits - 1));
  if (last) __threadfence();
  return last;
}

}  // namespace tg

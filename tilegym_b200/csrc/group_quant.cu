// Per-token group quantiser to 8 bits (e4m3, e5m2 or int8): the activation-side producer in front of an
// FP8 GEMM when the group is not the fixed 1 x 128 block of tg_act_quant.  One streaming pass, HBM-bound
// (bf16 in: 3 bytes per element): every thread owns 8 consecutive elements (one 16-byte load for bf16 / f16),
// the group_size / 8 lanes of a group reduce |x| with shuffles, and one lane writes the scale through the
// caller's strides, which covers the row-major, column-major and padded column-major scale layouts alike.
// Arithmetic follows tests/suites/flashinfer/test_per_token_group_quant_8bit.py:41-68 (the torch reference
// of src/tilegym/suites/flashinfer/cutile/per_token_group_quant_8bit.py:152-272): amax clamped from below by
// eps, scale = amax / dtype_max with IEEE division, optional rounding of the scale up to a power of two
// (UE8M0), q = clamp(x / scale, min, max), cast with round-to-nearest-even (fp8) or truncation (int8).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdio>

#include "tg_internal.h"

namespace tg {
namespace {

enum DstKind : int { kE4M3 = 0, kE5M2 = 1, kInt8 = 2 };

template <typename T>
__device__ __forceinline__ void load8(const T* src, float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(src));
    const float4 b = __ldcs(reinterpret_cast<const float4*>(src) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 t = __ldcs(reinterpret_cast<const uint4*>(src));
    const T* e = reinterpret_cast<const T*>(&t);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if constexpr (sizeof(T) == 2 && std::is_same<T, __half>::value) v[j] = __half2float(e[j]);
      else v[j] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(e)[j]);
    }
  }
}

template <int KIND>
__device__ __forceinline__ uint32_t to_8bit(float v) {
  if constexpr (KIND == kE4M3) return static_cast<uint32_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
  else if constexpr (KIND == kE5M2) return static_cast<uint32_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2));
  else return static_cast<uint32_t>(__float2int_rz(v)) & 0xffu;
}

// Smallest power of two >= max(|s|, 1e-10): ceil(log2) read off the exponent and mantissa bits, so the
// result does not depend on a log2 implementation.
__device__ __forceinline__ float round_up_pow2(float s) {
  s = fmaxf(fabsf(s), 1e-10f);
  const uint32_t b = __float_as_uint(s);
  const uint32_t exp_bits = (b & 0x7f800000u) + ((b & 0x007fffffu) ? 0x00800000u : 0u);
  return __uint_as_float(exp_bits);
}

// `tpg` = threads per group = group_size / 8 (1, 2, 4, 8, 16 or 32); groups never straddle a warp.
template <typename T, int KIND>
__global__ void __launch_bounds__(256)
    tg_per_token_group_quant_kernel(uint8_t* __restrict__ y, float* __restrict__ s, const T* __restrict__ x,
                                    int64_t n_chunks, int tpg, int64_t groups_per_row, int64_t s_row_stride,
                                    int64_t s_group_stride, float eps, float qmin, float qmax, int ue8m0) {
  const int lane = threadIdx.x & 31;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // all lanes of a warp run the same number of iterations (the shuffles need them)
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * blockDim.x + (threadIdx.x & ~31); base < n_chunks;
       base += stride) {
    const int64_t c = base + lane;
    const bool live = c < n_chunks;
    float v[8];
    if (live) {
      load8<T>(x + c * 8, v);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    for (int o = tpg >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    amax = fmaxf(amax, eps);
    float scale = __fdiv_rn(amax, qmax);
    if (ue8m0) scale = round_up_pow2(scale);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= to_8bit<KIND>(fminf(fmaxf(__fdiv_rn(v[j], scale), qmin), qmax)) << (8 * j);
      hi |= to_8bit<KIND>(fminf(fmaxf(__fdiv_rn(v[4 + j], scale), qmin), qmax)) << (8 * j);
    }
    if (live) {
      __stcs(reinterpret_cast<uint2*>(y + c * 8), make_uint2(lo, hi));
      if ((lane & (tpg - 1)) == 0) {
        const int64_t g = c / tpg;
        const int64_t row = g / groups_per_row;
        s[row * s_row_stride + (g - row * groups_per_row) * s_group_stride] = scale;
      }
    }
  }
}

template <typename T>
cudaError_t launch_kind(int kind, uint8_t* y, float* s, const T* x, int64_t n_chunks, int tpg, int64_t gpr,
                        int64_t srs, int64_t sgs, float eps, float qmin, float qmax, int ue8m0, int num_sms,
                        cudaStream_t stream) {
  const int threads = 256;
  int64_t blocks = (n_chunks + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(num_sms) * 16;  // 8 resident CTAs per SM, two rounds
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const dim3 grid(static_cast<unsigned>(blocks));
  if (kind == kE4M3)
    tg_per_token_group_quant_kernel<T, kE4M3><<<grid, threads, 0, stream>>>(y, s, x, n_chunks, tpg, gpr, srs, sgs, eps, qmin, qmax, ue8m0);
  else if (kind == kE5M2)
    tg_per_token_group_quant_kernel<T, kE5M2><<<grid, threads, 0, stream>>>(y, s, x, n_chunks, tpg, gpr, srs, sgs, eps, qmin, qmax, ue8m0);
  else
    tg_per_token_group_quant_kernel<T, kInt8><<<grid, threads, 0, stream>>>(y, s, x, n_chunks, tpg, gpr, srs, sgs, eps, qmin, qmax, ue8m0);
  return cudaGetLastError();
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

}  // namespace
}  // namespace tg

using namespace tg;

extern "C" TG_API int32_t tg_per_token_group_quant(const TgTensorDesc* Y, const TgTensorDesc* S,
                                                   const TgTensorDesc* X, int32_t group_size, float eps,
                                                   int32_t scale_ue8m0, int32_t device_id, uint64_t stream) {
  char msg[256];
  if (X == nullptr || Y == nullptr || S == nullptr) return api_fail(TG_ERR_NULL, "a descriptor is null");
  if (X->dtype != TG_BF16 && X->dtype != TG_F16 && X->dtype != TG_F32)
    return api_fail(TG_ERR_DTYPE, "X must be bf16, f16 or f32");
  int kind;
  float qmin, qmax;
  if (Y->dtype == TG_F8E4M3) { kind = kE4M3; qmin = -448.f; qmax = 448.f; }
  else if (Y->dtype == TG_F8E5M2) { kind = kE5M2; qmin = -57344.f; qmax = 57344.f; }
  else if (Y->dtype == TG_I8) { kind = kInt8; qmin = -128.f; qmax = 127.f; }
  else return api_fail(TG_ERR_DTYPE, "Y must be float8_e4m3fn (7), float8_e5m2 (5) or int8 (8)");
  if (S->dtype != TG_F32) return api_fail(TG_ERR_DTYPE, "S must be f32");
  if (X->ndim != 2 || Y->ndim != 2 || S->ndim != 2) return api_fail(TG_ERR_ARGS, "X, Y and S must be 2-D (flatten the leading dimensions)");
  const int64_t T = X->shape[0], H = X->shape[1];
  if (T < 0 || H <= 0) return api_fail(TG_ERR_ARGS, "X has a bad shape");
  if (group_size != 8 && group_size != 16 && group_size != 32 && group_size != 64 && group_size != 128 &&
      group_size != 256) {
    snprintf(msg, sizeof(msg), "group_size %d is not one of 8, 16, 32, 64, 128, 256", group_size);
    return api_fail(TG_ERR_ARGS, msg);
  }
  if (H % group_size != 0) {
    snprintf(msg, sizeof(msg), "the last dimension of X (%lld) must be divisible by group_size (%d)", (long long)H, group_size);
    return api_fail(TG_ERR_ARGS, msg);
  }
  const int64_t G = H / group_size;
  if (Y->shape[0] != T || Y->shape[1] != H) return api_fail(TG_ERR_ARGS, "Y must have the shape of X");
  if (X->strides[1] != 1 || X->strides[0] != H || Y->strides[1] != 1 || Y->strides[0] != H)
    return api_fail(TG_ERR_ARGS, "X and Y must be contiguous");
  if (S->shape[0] != T || S->shape[1] != G) return api_fail(TG_ERR_ARGS, "S must be [rows of X, H / group_size] (any strides)");
  if (S->strides[0] < 0 || S->strides[1] < 0) return api_fail(TG_ERR_ARGS, "S strides must not be negative");
  if (!(eps >= 0.f)) return api_fail(TG_ERR_ARGS, "eps must be >= 0");
  if (T == 0) return TG_OK;
  if (X->ptr == 0 || Y->ptr == 0 || S->ptr == 0) return api_fail(TG_ERR_NULL, "a data pointer is null");
  if ((X->ptr & 15u) || (Y->ptr & 7u) || (S->ptr & 3u))
    return api_fail(TG_ERR_ALIGN, "X needs 16-byte, Y 8-byte and S 4-byte alignment");
  if (device_id < 0 || device_id >= 64) return api_fail(TG_ERR_DEVICE, "device id out of range");

  Guard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return api_fail(TG_ERR_DEVICE, "cannot select the CUDA device");
  }
  int num_sms = 0;
  int32_t* status = nullptr;
  int32_t rc;
  if ((rc = api_init_device(device_id, &num_sms, &status)) != TG_OK) return rc;
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  const int64_t n_chunks = T * H / 8;
  const int tpg = group_size / 8;
  uint8_t* y = reinterpret_cast<uint8_t*>(Y->ptr);
  float* s = reinterpret_cast<float*>(S->ptr);
  cudaError_t e;
  if (X->dtype == TG_BF16)
    e = launch_kind<__nv_bfloat16>(kind, y, s, reinterpret_cast<const __nv_bfloat16*>(X->ptr), n_chunks, tpg, G,
                                   S->strides[0], S->strides[1], eps, qmin, qmax, scale_ue8m0, num_sms, cs);
  else if (X->dtype == TG_F16)
    e = launch_kind<__half>(kind, y, s, reinterpret_cast<const __half*>(X->ptr), n_chunks, tpg, G, S->strides[0],
                            S->strides[1], eps, qmin, qmax, scale_ue8m0, num_sms, cs);
  else
    e = launch_kind<float>(kind, y, s, reinterpret_cast<const float*>(X->ptr), n_chunks, tpg, G, S->strides[0],
                           S->strides[1], eps, qmin, qmax, scale_ue8m0, num_sms, cs);
  if (e != cudaSuccess) {
    snprintf(msg, sizeof(msg), "group quantiser launch failed: %s", cudaGetErrorString(e));
    return api_fail(TG_ERR_LAUNCH, msg);
  }
  return TG_OK;
}

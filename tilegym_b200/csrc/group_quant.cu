// Per-token group quantiser to 8 bits (e4m3, e5m2 or int8): the activation-side producer in front of an
// FP8 GEMM when the group is not the fixed 1 x 128 block of tg_act_quant.  One streaming pass, HBM-bound
// (bf16 in: 3 bytes per element): every thread owns 16 consecutive elements (two 16-byte loads for bf16 / f16),
// the group_size / 16 lanes of a group reduce |x| with shuffles, and one lane writes the scale through the
// caller's strides, which covers the row-major, column-major and padded column-major scale layouts alike.
// Arithmetic follows tests/suites/flashinfer/test_per_token_group_quant_8bit.py:41-68 (the torch reference
// of src/tilegym/suites/flashinfer/cutile/per_token_group_quant_8bit.py:152-272): amax clamped from below by
// eps, scale = amax / dtype_max with IEEE division, optional rounding of the scale up to a power of two
// (UE8M0), q = clamp(x / scale, min, max), cast with round-to-nearest-even (fp8) or truncation (int8).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdio>

#include <type_traits>

#include "tg_internal.h"
#include "tg_quant_common.cuh"

namespace tg {
namespace {

// EPT consecutive elements (8 or 16) as fp32; streaming loads (the input is read once).
template <typename T, int EPT>
__device__ __forceinline__ void load_elems(const T* src, float (&v)[EPT]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < EPT / 4; ++i) {
      const float4 a = __ldcs(reinterpret_cast<const float4*>(src) + i);
      v[4 * i] = a.x; v[4 * i + 1] = a.y; v[4 * i + 2] = a.z; v[4 * i + 3] = a.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < EPT / 8; ++i) {
      const uint4 t = __ldcs(reinterpret_cast<const uint4*>(src) + i);
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if constexpr (std::is_same<T, __half>::value) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
          v[8 * i + 2 * j] = f.x;
          v[8 * i + 2 * j + 1] = f.y;
        } else {  // bf16 -> fp32 is a 16-bit shift
          v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
          v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
      }
    }
  }
}

// Where group g's scale goes: row g / groups_per_row, column g % groups_per_row, through the caller's strides.
// 64-bit division costs a few hundred instructions, so the common sizes take a 32-bit one.
__device__ __forceinline__ int64_t scale_index(int64_t g, int64_t groups_per_row, int64_t row_stride,
                                               int64_t group_stride) {
  if (groups_per_row == 1) return g * row_stride;
  if (g <= 0xffffffffll && groups_per_row <= 0xffffffffll) {
    const uint32_t g32 = static_cast<uint32_t>(g), gpr = static_cast<uint32_t>(groups_per_row);
    const uint32_t row = g32 / gpr;
    return static_cast<int64_t>(row) * row_stride + static_cast<int64_t>(g32 - row * gpr) * group_stride;
  }
  const int64_t row = g / groups_per_row;
  return row * row_stride + (g - row * groups_per_row) * group_stride;
}

// A thread owns a chunk of EPT consecutive elements; the `tpg` = group_size / EPT lanes (a power of two, at
// most 32) that share a group sit next to each other in a warp.  `zero_to_one` selects the 1 x 128 activation
// quantiser's rule (scale 1.0 for an all-zero group, no eps).  16-bit inputs stay packed for the |x| maximum and
// take the test-free quotient of tg_quant_common.cuh (its precondition - a scale that is RN(amax / qmax) of a
// 16-bit amax, or a power of two - fails only where eps replaces the maximum; those groups and fp32 inputs go
// through the guarded reciprocal).  `dense_scales`: S is contiguous row-major, so group g's scale is s[g].
template <typename T, int KIND, int EPT>
__global__ void __launch_bounds__(256)
    tg_per_token_group_quant_kernel(uint8_t* __restrict__ y, float* __restrict__ s, const T* __restrict__ x,
                                    int64_t n_chunks, int tpg, int64_t groups_per_row, int64_t s_row_stride,
                                    int64_t s_group_stride, float eps, float qmin, float qmax, float qmax_rcp,
                                    int ue8m0, int zero_to_one, int dense_scales) {
  q8_allow_dependents();
  const int lane = threadIdx.x & 31;
  const int tpg_shift = 31 - __clz(tpg);
  const int64_t span = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // all lanes of a warp run the same number of iterations (the shuffles need them)
  // 16-bit inputs: the next iteration's chunk is requested before this one is worked on, which keeps a second
  // set of loads in flight per thread through the shuffle / convert / store part
  [[maybe_unused]] uint32_t w_next[EPT / 2];
  [[maybe_unused]] auto fetch = [&](int64_t chunk, uint32_t (&dst)[EPT / 2]) {
#pragma unroll
    for (int j = 0; j < EPT / 2; ++j) dst[j] = 0u;
    if (chunk < n_chunks) {
#pragma unroll
      for (int i = 0; i < EPT / 8; ++i) {
        const uint4 t = __ldcs(reinterpret_cast<const uint4*>(x + chunk * EPT) + i);
        dst[4 * i] = t.x; dst[4 * i + 1] = t.y; dst[4 * i + 2] = t.z; dst[4 * i + 3] = t.w;
      }
    }
  };
  const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x + (threadIdx.x & ~31);
  if constexpr (sizeof(T) == 2) fetch(first + lane, w_next);
  for (int64_t base = first; base < n_chunks; base += span) {
    const int64_t c = base + lane;
    const bool live = c < n_chunks;
    uint32_t out[EPT / 4];
    float scale;
    if constexpr (sizeof(T) == 2) {
      uint32_t w[EPT / 2];
#pragma unroll
      for (int j = 0; j < EPT / 2; ++j) w[j] = w_next[j];
      if (base + span < n_chunks) fetch(c + span, w_next);
      uint32_t m2 = absmax_pairs<T>(w[0], w[1]);
#pragma unroll
      for (int j = 2; j < EPT / 2; j += 2) m2 = absmax_pairs<T>(m2, absmax_pairs<T>(w[j], w[j + 1]));
      const float2 mm = unpack_pair<T>(m2);
      float amax = fmaxf(mm.x, mm.y);
      for (int o = tpg >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      bool exact_form = true;  // is the scale RN(16-bit amax / qmax) or a power of two?
      if (zero_to_one) {
        scale = q8_scale_from_amax(amax, qmax, qmax_rcp);
        if (scale == 0.f) scale = 1.0f;
      } else {
        exact_form = ue8m0 || amax >= eps;
        scale = amax >= eps ? q8_scale_from_amax(amax, qmax, qmax_rcp) : __fdiv_rn(eps, qmax);
        if (ue8m0) scale = round_up_pow2(scale);
      }
      const float r = __frcp_rn(scale);
      if (q8_scale_is_tame(scale) && exact_form) {
#pragma unroll
        for (int k = 0; k < EPT / 4; ++k) {
          const float2 q0 = q8_quot2(unpack_pair<T>(w[2 * k]), scale, r);
          const float2 q1 = q8_quot2(unpack_pair<T>(w[2 * k + 1]), scale, r);
          out[k] = q8_cast2<KIND>(q0.x, q0.y, qmin, qmax) | (q8_cast2<KIND>(q1.x, q1.y, qmin, qmax) << 16);
        }
      } else {
#pragma unroll
        for (int k = 0; k < EPT / 4; ++k) {
          const float2 x0 = unpack_pair<T>(w[2 * k]), x1 = unpack_pair<T>(w[2 * k + 1]);
          out[k] = q8_pair<KIND>(x0.x, x0.y, scale, r, false, qmin, qmax) |
                   (q8_pair<KIND>(x1.x, x1.y, scale, r, false, qmin, qmax) << 16);
        }
      }
    } else {
      float v[EPT];
#pragma unroll
      for (int j = 0; j < EPT; ++j) v[j] = 0.f;
      if (live) load_elems<T, EPT>(x + c * EPT, v);
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < EPT; ++j) amax = fmaxf(amax, fabsf(v[j]));
      for (int o = tpg >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (zero_to_one) {
        scale = __fdiv_rn(amax, qmax);
        if (scale == 0.f) scale = 1.0f;
      } else {
        scale = __fdiv_rn(fmaxf(amax, eps), qmax);
        if (ue8m0) scale = round_up_pow2(scale);
      }
      const bool tame = q8_scale_is_tame(scale);
      const float r = __frcp_rn(scale);
#pragma unroll
      for (int k = 0; k < EPT / 4; ++k)
        out[k] = q8_pair<KIND>(v[4 * k], v[4 * k + 1], scale, r, tame, qmin, qmax) |
                 (q8_pair<KIND>(v[4 * k + 2], v[4 * k + 3], scale, r, tame, qmin, qmax) << 16);
    }
    if (live) {
      if constexpr (EPT >= 16) {
#pragma unroll
        for (int i = 0; i < EPT / 16; ++i)
          __stcs(reinterpret_cast<uint4*>(y + c * EPT) + i, make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]));
      } else {
        __stcs(reinterpret_cast<uint2*>(y + c * EPT), make_uint2(out[0], out[1]));
      }
      if ((lane & (tpg - 1)) == 0) {
        const int64_t g = c >> tpg_shift;
        s[dense_scales ? g : scale_index(g, groups_per_row, s_row_stride, s_group_stride)] = scale;
      }
    }
  }
}

template <typename T, int EPT>
cudaError_t launch_kind(int kind, uint8_t* y, float* s, const T* x, int64_t n_chunks, int tpg, int64_t gpr,
                        int64_t srs, int64_t sgs, float eps, float qmin, float qmax, int ue8m0, int zero_to_one,
                        int num_sms, cudaStream_t stream) {
  const float qmax_rcp = 1.0f / qmax;  // IEEE division on the host: RN(1 / qmax)
  const int dense = (sgs == 1 && srs == gpr) || (gpr == 1 && srs == 1);
  const int threads = 256;
  int64_t blocks = (n_chunks + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(num_sms) * 16;  // 8 resident CTAs per SM, two rounds
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const dim3 grid(static_cast<unsigned>(blocks));
  if (kind == kQ8E4M3)
    tg_per_token_group_quant_kernel<T, kQ8E4M3, EPT><<<grid, threads, 0, stream>>>(y, s, x, n_chunks, tpg, gpr, srs, sgs, eps, qmin, qmax, qmax_rcp, ue8m0, zero_to_one, dense);
  else if (kind == kQ8E5M2)
    tg_per_token_group_quant_kernel<T, kQ8E5M2, EPT><<<grid, threads, 0, stream>>>(y, s, x, n_chunks, tpg, gpr, srs, sgs, eps, qmin, qmax, qmax_rcp, ue8m0, zero_to_one, dense);
  else
    tg_per_token_group_quant_kernel<T, kQ8Int8, EPT><<<grid, threads, 0, stream>>>(y, s, x, n_chunks, tpg, gpr, srs, sgs, eps, qmin, qmax, qmax_rcp, ue8m0, zero_to_one, dense);
  return cudaGetLastError();
}

// group_size 8 runs 8 elements per thread, 16-bit inputs with groups >= 32 run 32, everything else 16.
cudaError_t launch_any(int x_dtype, int kind, uint8_t* y, float* s, const void* x, int64_t numel, int group_size,
                       int64_t gpr, int64_t srs, int64_t sgs, float eps, float qmin, float qmax, int ue8m0,
                       int zero_to_one, int num_sms, cudaStream_t stream) {
#define TG_GQ_LAUNCH(T, EPT)                                                                                       \
  launch_kind<T, EPT>(kind, y, s, static_cast<const T*>(x), numel / EPT, group_size / EPT, gpr, srs, sgs, eps, qmin, \
                      qmax, ue8m0, zero_to_one, num_sms, stream)
  if (group_size == 8) {
    if (x_dtype == TG_BF16) return TG_GQ_LAUNCH(__nv_bfloat16, 8);
    if (x_dtype == TG_F16) return TG_GQ_LAUNCH(__half, 8);
    return TG_GQ_LAUNCH(float, 8);
  }
  // 16-bit inputs with groups of 32 or more: 32 elements per thread halve the share of the per-thread work that
  // does not scale with the elements (shuffles, scale, reciprocal, addresses)
  if (group_size >= 32 && x_dtype == TG_BF16) return TG_GQ_LAUNCH(__nv_bfloat16, 32);
  if (group_size >= 32 && x_dtype == TG_F16) return TG_GQ_LAUNCH(__half, 32);
  if (x_dtype == TG_BF16) return TG_GQ_LAUNCH(__nv_bfloat16, 16);
  if (x_dtype == TG_F16) return TG_GQ_LAUNCH(__half, 16);
  return TG_GQ_LAUNCH(float, 16);
#undef TG_GQ_LAUNCH
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

namespace tg {
// The 1 x 128 activation quantiser is the same kernel with its own zero rule (scale 1.0, no eps) and one
// scale per 128-element block, stored densely.
cudaError_t launch_act_quant(void* y, float* s, const void* x, int x_dtype, int64_t n_blocks, cudaStream_t stream) {
  int dev = 0, num_sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  return launch_any(x_dtype, kQ8E4M3, static_cast<uint8_t*>(y), s, x, n_blocks * 128, 128, 1, 1, 0, 0.f, -448.f,
                    448.f, 0, 1, num_sms, stream);
}
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
  if (Y->dtype == TG_F8E4M3) { kind = kQ8E4M3; qmin = -448.f; qmax = 448.f; }
  else if (Y->dtype == TG_F8E5M2) { kind = kQ8E5M2; qmin = -57344.f; qmax = 57344.f; }
  else if (Y->dtype == TG_I8) { kind = kQ8Int8; qmin = -128.f; qmax = 127.f; }
  else return api_fail(TG_ERR_DTYPE, "Y must be float8_e4m3fn (7), float8_e5m2 (5) or int8 (8)");
  if (S->dtype != TG_F32) return api_fail(TG_ERR_DTYPE, "S must be f32");
  if (X->ndim != 2 || Y->ndim != 2 || S->ndim != 2) return api_fail(TG_ERR_ARGS, "X, Y and S must be 2-D (flatten the leading dimensions)");
  const int64_t T = X->shape[0], H = X->shape[1];
  if (T < 0 || H <= 0) return api_fail(TG_ERR_ARGS, "X has a bad shape");
  if (group_size != 8 && group_size != 16 && group_size != 32 && group_size != 64 && group_size != 128 &&
      group_size != 256 && group_size != 512) {
    snprintf(msg, sizeof(msg), "group_size %d is not one of 8, 16, 32, 64, 128, 256, 512", group_size);
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
  if ((X->ptr & 15u) || (Y->ptr & 15u) || (S->ptr & 3u))
    return api_fail(TG_ERR_ALIGN, "X and Y need 16-byte, S 4-byte alignment");
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
  uint8_t* y = reinterpret_cast<uint8_t*>(Y->ptr);
  float* s = reinterpret_cast<float*>(S->ptr);
  const cudaError_t e = launch_any(X->dtype, kind, y, s, reinterpret_cast<const void*>(X->ptr), T * H, group_size, G,
                                   S->strides[0], S->strides[1], eps, qmin, qmax, scale_ue8m0, 0, num_sms, cs);
  if (e != cudaSuccess) {
    snprintf(msg, sizeof(msg), "group quantiser launch failed: %s", cudaGetErrorString(e));
    return api_fail(TG_ERR_LAUNCH, msg);
  }
  return TG_OK;
}

// tg_selftest_wait_timeout: runs the kernels' bounded-wait abort path once, on purpose and safely.
// One CTA with the role layout of the GEMM kernels (warp 0 "producer", warp 1 "MMA" and TMEM owner, warps 2-5
// "epilogue") allocates TMEM, then every role waits - with the same mbar_wait / abort flag / report_timeout
// code the GEMM kernels use - on an mbarrier that nothing ever arrives on.  The producer's wait expires after
// `limit_us`, raises the CTA's abort flag and records its code in the device status word; the other roles see
// the flag and leave; the CTA meets at its teardown barrier, frees its TMEM and returns normally.  Nothing
// faults, traps or spins without bound: the host then reads TG_ERR_TIMEOUT from tg_device_status() and the
// context stays usable.  The reference has no counterpart (its kernels contain no device-side waits of their own).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tg_gemm_common.cuh"
#include "tg_quant_common.cuh"

namespace tg {
namespace {

constexpr int kSelfTestSite = 99;

__global__ void __launch_bounds__(192, 1) tg_selftest_wait_kernel(int32_t* status, uint32_t limit_us) {
  __shared__ __align__(8) uint64_t bar_never;
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_words[2];
  volatile uint32_t* abort_flag = abort_words;
  const int warp = threadIdx.x >> 5;
  const uint32_t bar = smem_u32(&bar_never);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    init_abort_flag(abort_flag, limit_us);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  // every role waits for a phase that never completes; exactly one wait (the first to look at the clock
  // after the limit) raises the flag, the rest return because they see it
  const bool done = __all_sync(0xffffffffu, mbar_wait(bar, 0u, abort_flag));
  if (!done) {
    const int role = warp == 0 ? kRoleProducer : (warp == 1 ? kRoleMma : kRoleEpilogue);
    if ((threadIdx.x & 31) == 0) report_timeout(status, role * 1000 + kSelfTestSite);
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
}

// tg_selftest_quant16: the quantisers' test-free quotient (q8_quot2) and scale (q8_scale_from_amax) against
// div.rn for EVERY case a 16-bit input can produce.  Block b takes the group maximum whose bit pattern is
// b + 1 (all positive finite values of the type, subnormals included); its threads walk every |x| <= amax, both
// signs, +-0 and NaN, under the scale amax / qmax and under that scale rounded up to a power of two, and count
// the pairs whose bytes differ from cast(div.rn(x, s)).  counts[0] mismatching pairs, [1] pairs compared,
// [2] scales that differ from div.rn(amax, qmax), [3] maxima skipped because their scale is outside the range
// in which the kernels use the fast path at all.
template <typename T, int KIND>
__global__ void __launch_bounds__(256) tg_selftest_quant16_kernel(unsigned long long* counts, float qmin, float qmax,
                                                                  float qmax_rcp) {
  const uint32_t amax_bits = blockIdx.x + 1u;
  auto as_f32 = [](uint32_t bits16) -> float {
    if constexpr (std::is_same<T, __half>::value) {
      const __half_raw h{static_cast<unsigned short>(bits16)};
      return __half2float(__half(h));
    } else {
      return __uint_as_float(bits16 << 16);
    }
  };
  const float amax = as_f32(amax_bits);
  const float s_ref = __fdiv_rn(amax, qmax);
  const float s_fast = q8_scale_from_amax(amax, qmax, qmax_rcp);
  unsigned long long bad = 0, seen = 0;
  if (threadIdx.x == 0) {
    if (__float_as_uint(s_ref) != __float_as_uint(s_fast)) atomicAdd(counts + 2, 1ull);
    if (!q8_scale_is_tame(s_ref)) atomicAdd(counts + 3, 1ull);
  }
  if (q8_scale_is_tame(s_ref)) {
#pragma unroll 1
    for (int form = 0; form < 2; ++form) {
      const float s = form == 0 ? s_ref : round_up_pow2(s_ref);
      const float r = __frcp_rn(s);
      for (uint32_t xb = threadIdx.x; xb <= amax_bits + 1u; xb += blockDim.x) {
        // xb == amax_bits + 1 stands for NaN (quiet, both signs)
        const float v = xb <= amax_bits ? as_f32(xb) : __uint_as_float(0x7fc00000u);
        const float2 x = make_float2(v, __uint_as_float(__float_as_uint(v) | 0x80000000u));
        const float2 q = q8_quot2(x, s, r);
        const uint32_t fast = q8_cast2<KIND>(q.x, q.y, qmin, qmax);
        const uint32_t ref = q8_cast2<KIND>(__fdiv_rn(x.x, s), __fdiv_rn(x.y, s), qmin, qmax);
        bad += (fast != ref);
        ++seen;
      }
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    bad += __shfl_xor_sync(0xffffffffu, bad, o);
    seen += __shfl_xor_sync(0xffffffffu, seen, o);
  }
  if ((threadIdx.x & 31) == 0) {
    if (bad) atomicAdd(counts, bad);
    atomicAdd(counts + 1, seen);
  }
}

template <typename T>
cudaError_t launch_quant16(int kind, unsigned long long* counts, unsigned blocks, cudaStream_t stream) {
  if (kind == kQ8E4M3)
    tg_selftest_quant16_kernel<T, kQ8E4M3><<<blocks, 256, 0, stream>>>(counts, -448.f, 448.f, 1.0f / 448.f);
  else if (kind == kQ8E5M2)
    tg_selftest_quant16_kernel<T, kQ8E5M2><<<blocks, 256, 0, stream>>>(counts, -57344.f, 57344.f, 1.0f / 57344.f);
  else
    tg_selftest_quant16_kernel<T, kQ8Int8><<<blocks, 256, 0, stream>>>(counts, -128.f, 127.f, 1.0f / 127.f);
  return cudaGetLastError();
}

}  // namespace
}  // namespace tg

using namespace tg;

extern "C" TG_API int32_t tg_selftest_quant16(int32_t x_dtype, int32_t y_dtype, uint64_t counts, int32_t device_id,
                                              uint64_t stream) {
  if (x_dtype != TG_BF16 && x_dtype != TG_F16) return api_fail(TG_ERR_DTYPE, "x_dtype must be bf16 or f16");
  int kind;
  if (y_dtype == TG_F8E4M3) kind = kQ8E4M3;
  else if (y_dtype == TG_F8E5M2) kind = kQ8E5M2;
  else if (y_dtype == TG_I8) kind = kQ8Int8;
  else return api_fail(TG_ERR_DTYPE, "y_dtype must be float8_e4m3fn, float8_e5m2 or int8");
  if (counts == 0 || (counts & 7u)) return api_fail(TG_ERR_NULL, "counts must point to four 64-bit words on the device");
  if (device_id < 0 || device_id >= 64) return api_fail(TG_ERR_DEVICE, "device id out of range");
  int prev = -1;
  if (cudaGetDevice(&prev) != cudaSuccess || (prev != device_id && cudaSetDevice(device_id) != cudaSuccess)) {
    cudaGetLastError();
    return api_fail(TG_ERR_DEVICE, "cannot select the CUDA device");
  }
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  unsigned long long* c = reinterpret_cast<unsigned long long*>(counts);
  cudaError_t e = cudaMemsetAsync(c, 0, 4 * sizeof(unsigned long long), cs);
  // positive finite bit patterns: 0x0001..0x7f7f (bf16), 0x0001..0x7bff (f16)
  if (e == cudaSuccess)
    e = x_dtype == TG_BF16 ? launch_quant16<__nv_bfloat16>(kind, c, 0x7f7fu, cs) : launch_quant16<__half>(kind, c, 0x7bffu, cs);
  if (prev != device_id) cudaSetDevice(prev);
  if (e != cudaSuccess) return api_fail(TG_ERR_LAUNCH, cudaGetErrorString(e));
  return TG_OK;
}

extern "C" TG_API int32_t tg_selftest_wait_timeout(uint32_t limit_us, int32_t device_id, uint64_t stream) {
  if (limit_us == 0 || limit_us > 1000000u)
    return api_fail(TG_ERR_ARGS, "limit_us must be between 1 and 1000000 (the self-test is meant to give up quickly)");
  if (device_id < 0 || device_id >= 64) return api_fail(TG_ERR_DEVICE, "device id out of range");
  int prev = -1;
  if (cudaGetDevice(&prev) != cudaSuccess || (prev != device_id && cudaSetDevice(device_id) != cudaSuccess)) {
    cudaGetLastError();
    return api_fail(TG_ERR_DEVICE, "cannot select the CUDA device");
  }
  int num_sms = 0;
  int32_t* status = nullptr;
  int32_t rc = api_init_device(device_id, &num_sms, &status);
  if (rc == TG_OK) {
    tg_selftest_wait_kernel<<<1, 192, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status, limit_us);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) rc = api_fail(TG_ERR_LAUNCH, cudaGetErrorString(e));
  }
  if (prev != device_id) cudaSetDevice(prev);
  return rc;
}

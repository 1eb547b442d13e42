// tg_selftest_wait_timeout: runs the kernels' bounded-wait abort path once, on purpose and safely.
// One CTA with the role layout of the GEMM kernels (warp 0 "producer", warp 1 "MMA" and TMEM owner, warps 2-5
// "epilogue") allocates TMEM, then every role waits - with the same mbar_wait / abort flag / report_timeout
// code the GEMM kernels use - on an mbarrier that nothing ever arrives on.  The producer's wait expires after
// `limit_us`, raises the CTA's abort flag and records its code in the device status word; the other roles see
// the flag and leave; the CTA meets at its teardown barrier, frees its TMEM and returns normally.  Nothing
// faults, traps or spins without bound: the host then reads TG_ERR_TIMEOUT from tg_device_status() and the
// context stays usable.  The reference has no counterpart (its kernels contain no device-side waits of their own).
#include "tg_gemm_common.cuh"

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

}  // namespace
}  // namespace tg

using namespace tg;

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

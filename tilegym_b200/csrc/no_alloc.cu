// tg_fp8_gemm_pertensor_smallm_static: the small-M (M <= 64) split-K GEMM for
// callers that cannot allocate device memory.
//
// Who needs it: a serving process whose memory pool already owns the whole
// GPU (a cudaMalloc for the regular 48 MiB workspace would fail there, or
// would take memory behind the pool's back), and latency-critical decode
// loops that must never reach the allocator, because cudaMalloc / cudaFree
// synchronise the device and stall every stream.  The regular entry point
// asks such callers for a workspace pointer; this one brings its own.
//
// The split-K scratch (arrival counters + fp32 partial sums) lives in a
// file-scope __device__ array below, so the library holds kStaticScratchBytes
// of device memory on every GPU that loads it, until the process exits.
// Consequences a caller must know:
//   * sizes are capped (M <= 64, N <= kMaxN); anything larger is rejected;
//   * all calls on a device share the one array: calls that overlap on the
//     GPU (different streams, no ordering between them) race on it;
//   * the array keeps whatever the previous call left, so each call first
//     clears the counters it is about to use (a stream-ordered memset);
//   * the first call on a device resolves the array's device address and sets
//     the kernel's shared-memory attribute; make that first call before any
//     stream capture begins.
// No cudaMalloc, cudaFree or other allocating routine is called on any path.
#include <cstdio>

#include "tg_internal.h"

namespace tg {
namespace {

constexpr int kMaxCounters = 4096;                              // four per 128-row weight tile
constexpr uint64_t kStaticCounterBytes = kMaxCounters * 4ull;   // 16 KiB
constexpr uint64_t kStaticPartialBytes = 8ull << 20;            // 8 MiB of fp32 partial sums
constexpr uint64_t kStaticScratchBytes = kStaticCounterBytes + kStaticPartialBytes;
constexpr int64_t kMaxM = 64;
constexpr int64_t kMaxN = (kMaxCounters / 4) * 128ll;           // 131072 weight rows

// In host code this name is only a handle for the runtime, not an address a
// kernel can use: the device address is looked up per device below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

unsigned char* g_scratch_addr[64] = {};

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

extern "C" TG_API int32_t tg_fp8_gemm_pertensor_smallm_static(const TgTensorDesc* C, const TgTensorDesc* A,
                                                              const TgTensorDesc* B, uint64_t scale_a,
                                                              uint64_t scale_b, float alpha,
                                                              const TgTensorDesc* bias, float beta,
                                                              int32_t device_id, uint64_t stream) {
  int32_t rc;
  char msg[256];
  if ((rc = api_check_operand(A, "A")) != TG_OK) return rc;
  if ((rc = api_check_operand(B, "B")) != TG_OK) return rc;
  const int64_t M = A->shape[0], K = A->shape[1], N = B->shape[0];
  if (B->shape[1] != K) return api_fail(TG_ERR_ARGS, "A and B disagree on K");
  if ((rc = api_check_output(C, M, N)) != TG_OK) return rc;
  if (M > kMaxM) {
    snprintf(msg, sizeof(msg), "M = %lld exceeds the %lld rows this no-allocation entry point supports; "
             "use tg_fp8_gemm_pertensor with a workspace", (long long)M, (long long)kMaxM);
    return api_fail(TG_ERR_ARGS, msg);
  }
  if (N > kMaxN) {
    snprintf(msg, sizeof(msg), "N = %lld exceeds the %lld weight rows the static scratch has counters for",
             (long long)N, (long long)kMaxN);
    return api_fail(TG_ERR_ARGS, msg);
  }
  if (bias != nullptr) {
    if (bias->dtype != TG_F32 && bias->dtype != TG_BF16 && bias->dtype != TG_F16)
      return api_fail(TG_ERR_DTYPE, "bias must be f32, f16 or bf16");
    if (bias->ndim != 1 || bias->shape[0] != N || bias->strides[0] != 1)
      return api_fail(TG_ERR_ARGS, "bias must be a contiguous vector of N elements");
    if (bias->ptr == 0 && N > 0) return api_fail(TG_ERR_NULL, "bias data pointer is null");
  }
  if ((scale_a & 3u) || (scale_b & 3u)) return api_fail(TG_ERR_ALIGN, "scale pointers must be 4-byte aligned");
  if (M == 0 || N == 0) return TG_OK;
  if (device_id < 0 || device_id >= 64) return api_fail(TG_ERR_DEVICE, "device id out of range");

  Guard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return api_fail(TG_ERR_DEVICE, "cannot select the CUDA device");
  }
  int num_sms = 0;
  int32_t* status = nullptr;
  if ((rc = api_init_device(device_id, &num_sms, &status)) != TG_OK) return rc;
  // Set-up, once per device, with that device current: the device address of the scratch array.
  if (g_scratch_addr[device_id] == nullptr) {
    unsigned char* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return api_fail(TG_ERR_DEVICE, "cannot resolve the static scratch array on this device");
    }
    g_scratch_addr[device_id] = ptr;
  }
  unsigned char* scratch = g_scratch_addr[device_id];
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);

  GemmParams p = {};
  p.M = static_cast<int32_t>(M);
  p.N = static_cast<int32_t>(N);
  p.K = static_cast<int32_t>(K);
  p.num_kb = static_cast<int32_t>((K + 127) / 128);
  p.tiles_m = 1;
  p.tile_rows = 128;
  p.tiles_n = static_cast<int32_t>((N + 127) / 128);
  p.C = reinterpret_cast<void*>(C->ptr);
  p.ldc = C->strides[0];
  p.out_dtype = C->dtype;
  p.scale_a = reinterpret_cast<const float*>(scale_a);
  p.scale_b = reinterpret_cast<const float*>(scale_b);
  p.alpha = alpha;
  p.beta = beta;
  p.bias = bias ? reinterpret_cast<const void*>(bias->ptr) : nullptr;
  p.bias_dtype = bias ? bias->dtype : TG_F32;
  p.status = status;
  p.ws_counters = reinterpret_cast<uint32_t*>(scratch);
  p.ws_partial = reinterpret_cast<float*>(scratch + kStaticCounterBytes);

  // K splits: about two CTAs per SM, at least two k-blocks each, partial sums within the static array.
  const int mp = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  int splits = 1;
  if (p.tiles_n * 2 <= 2 * num_sms && p.num_kb >= 4) {
    splits = (2 * num_sms) / p.tiles_n;
    if (splits > p.num_kb / 2) splits = p.num_kb / 2;
    while (splits > 1 && static_cast<uint64_t>(p.tiles_n) * splits * mp * 128ull * 4ull > kStaticPartialBytes) --splits;
    if (splits < 1) splits = 1;
  }
  p.kb_per_split = (p.num_kb + splits - 1) / splits;
  p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;

  if (p.splits > 1) {
    // the array keeps the previous call's contents: the counters this call uses must start at zero
    cudaError_t e = cudaMemsetAsync(p.ws_counters, 0, static_cast<size_t>(p.tiles_n) * 4 * sizeof(uint32_t), cs);
    if (e != cudaSuccess) return api_fail(TG_ERR_LAUNCH, "clearing the static counters failed");
  }
  CUtensorMap tmW, tmX;
  if ((rc = api_make_map(&tmW, B->ptr, N, K, B->strides[0], 128)) != TG_OK) return rc;
  if ((rc = api_make_map(&tmX, A->ptr, M, K, A->strides[0], mp)) != TG_OK) return rc;
  cudaError_t e = launch_gemm_smallm(tmW, tmX, p, mp, cs);
  if (e != cudaSuccess) return api_fail(TG_ERR_LAUNCH, cudaGetErrorString(e));
  return TG_OK;
}

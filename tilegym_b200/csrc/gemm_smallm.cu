// Small-M (decode, M <= 64) per-tensor-scaled FP8 GEMM for sm_100a.
// The problem is a weight-streaming one (N*K bytes of e4m3 against a few
// rows of activations), bound by HBM bandwidth, so the kernel is built
// around bytes in flight rather than tensor-pipe occupancy:
//   * swap-AB: 128 weight rows ride the MMA's M axis (TMEM lanes), the M
//     activation rows (padded to MP = 16/32/64 by TMA zero fill) are the MMA's
//     N, so no tensor-core work is wasted on padding rows of a 128-row tile;
//   * split-K: the grid is (weight-row tiles) x (K splits), about two CTAs per
//     SM, each streaming its slab through a deep TMA ring;
//   * partial sums go to an fp32 workspace; the warp that arrives last for a
//     (tile, lane-quadrant) adds them in split order and runs the epilogue, so
//     nobody waits and the result does not depend on arrival order.
// Same contract as the large-M kernel: C = alpha*sa*sb * A.B^T + bias + beta*C.
#include "tg_gemm_common.cuh"

namespace tg {

namespace {

constexpr int kThreads = 192;  // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue

template <int MP>
struct SmCfg {
  static constexpr int kWBytes = kBM * kBK;  // 128 weight rows x 128 B
  static constexpr int kXBytes = MP * kBK;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kStages = (MP == 16) ? 6 : (MP == 32 ? 5 : 4);
  static constexpr int kTmemCols = MP < 32 ? 32 : MP;
  static constexpr int kCtrlBytes = 128;
  static constexpr int kSmemBytes = kStages * kStageBytes + kCtrlBytes + 1024;
  static_assert((2 * kStages + 1) * 8 + 8 <= kCtrlBytes, "control block");
};

__device__ __forceinline__ void smallm_store(const GemmParams& p, int m, int64_t n, float v) {
  const int64_t off = static_cast<int64_t>(m) * p.ldc + n;
  if (p.out_dtype == TG_BF16) {
    __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
    if (p.beta != 0.f) v = fmaf(p.beta, __bfloat162float(*c), v);
    *c = __float2bfloat16_rn(v);
  } else if (p.out_dtype == TG_F16) {
    __half* c = reinterpret_cast<__half*>(p.C) + off;
    if (p.beta != 0.f) v = fmaf(p.beta, __half2float(*c), v);
    *c = __float2half_rn(v);
  } else {
    float* c = reinterpret_cast<float*>(p.C) + off;
    if (p.beta != 0.f) v = fmaf(p.beta, *c, v);
    *c = v;
  }
}

template <int MP>
__global__ void __launch_bounds__(kThreads, 2)
    tg_fp8_gemm_smallm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                              const GemmParams p) {
  using Cfg = SmCfg<MP>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t w_base = base;
  const uint32_t x_base = base + S * Cfg::kWBytes;
  uint8_t* ctrl = smem + S * Cfg::kStageBytes;
  const uint32_t bar_full = smem_u32(ctrl);
  const uint32_t bar_empty = bar_full + 8 * S;
  const uint32_t bar_tfull = bar_empty + 8 * S;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + (2 * S + 1) * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    mbar_init(bar_tfull, 1);
    *abort_flag = 0u;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // one work unit per CTA: weight-row tile tn, K split sp
  const int u = blockIdx.x;
  const int tn = u / p.splits, sp = u - tn * p.splits;
  const int kb0 = sp * p.kb_per_split;
  const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmW);
      prefetch_tmap(&tmX);
      const uint64_t pol_w = policy_evict_first();  // weights are read once
      const uint64_t pol_x = policy_evict_last();   // activations are re-read by every CTA
      int s = 0;
      uint32_t ph = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag)) {
          report_timeout(p.status, kRoleProducer * 1000 + 21);
          break;
        }
        mbar_arrive_expect_tx(bar_full + 8 * s, Cfg::kStageBytes);
        tma_load_2d_hint(w_base + s * Cfg::kWBytes, &tmW, bar_full + 8 * s, kb * kBK, tn * kBM, pol_w);
        tma_load_2d_hint(x_base + s * Cfg::kXBytes, &tmX, bar_full + 8 * s, kb * kBK, 0, pol_x);
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_e4m3_f32(kBM, MP);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(bar_full + 8 * s, ph, abort_flag)) {
          report_timeout(p.status, kRoleMma * 1000 + 21);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t wdesc = make_kmajor_sw128_desc(w_base + s * Cfg::kWBytes);
        const uint64_t xdesc = make_kmajor_sw128_desc(x_base + s * Cfg::kXBytes);
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          mma_f8f6f4(tmem_base, wdesc + 2u * k, xdesc + 2u * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        tc_commit(bar_empty + 8 * s);
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      }
      if (ok) tc_commit(bar_tfull);
    }
  } else {
    const int q = warp & 3;
    const int n_local = q * 32 + lane;
    const int64_t n = static_cast<int64_t>(tn) * kBM + n_local;
    const bool n_ok = n < p.N;
    float scale = p.alpha;
    if (p.scale_a != nullptr) scale *= __ldg(p.scale_a);
    if (p.scale_b != nullptr) scale *= __ldg(p.scale_b);
    const float bias = (p.bias != nullptr && n_ok) ? load_bias(p.bias, p.bias_dtype, static_cast<int>(n)) : 0.f;
    const int mv = p.M < MP ? p.M : MP;

    bool w = mbar_wait(bar_tfull, 0u, abort_flag);
    w = __all_sync(0xffffffffu, w);
    if (!w) {
      report_timeout(p.status, kRoleEpilogue * 1000 + 21);
    } else {
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      float acc[MP];
      if constexpr (MP == 16) {
        uint32_t r[16];
        tmem_ld_32x16(t_addr, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = __uint_as_float(r[j]);
      } else {
#pragma unroll
        for (int c = 0; c < MP / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c * 32 + j] = __uint_as_float(r[j]);
        }
      }
      if (p.splits == 1) {
        if (n_ok) {
#pragma unroll
          for (int m = 0; m < MP; ++m)
            if (m < mv) smallm_store(p, m, n, fmaf(acc[m], scale, bias));
        }
      } else {
        float* part = p.ws_partial + static_cast<int64_t>(u) * (MP * kBM) + n_local;
#pragma unroll
        for (int m = 0; m < MP; ++m)
          if (m < mv) part[m * kBM] = acc[m];
        if (splitk_arrive_is_last(p.ws_counters + tn * 4 + q, p.splits)) {
          const float* tile_part = p.ws_partial + static_cast<int64_t>(tn) * p.splits * (MP * kBM) + n_local;
#pragma unroll
          for (int m = 0; m < MP; ++m) acc[m] = 0.f;
#pragma unroll 1
          for (int s2 = 0; s2 < p.splits; ++s2) {  // fixed order: bit-stable result
            const float* src = tile_part + static_cast<int64_t>(s2) * (MP * kBM);
#pragma unroll
            for (int m = 0; m < MP; ++m)  // MP independent loads in flight
              if (m < mv) acc[m] += __ldcg(src + m * kBM);
          }
          if (n_ok) {
#pragma unroll
            for (int m = 0; m < MP; ++m)
              if (m < mv) smallm_store(p, m, n, fmaf(acc[m], scale, bias));
          }
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int MP>
cudaError_t launch_mp(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, cudaStream_t stream) {
  using Cfg = SmCfg<MP>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tg_fp8_gemm_smallm_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int grid = p.tiles_n * p.splits;
  tg_fp8_gemm_smallm_kernel<MP><<<grid, kThreads, Cfg::kSmemBytes, stream>>>(tmW, tmX, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemm_smallm(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int mp,
                               cudaStream_t stream) {
  switch (mp) {
    case 16:
      return launch_mp<16>(tmW, tmX, p, stream);
    case 32:
      return launch_mp<32>(tmW, tmX, p, stream);
    case 64:
      return launch_mp<64>(tmW, tmX, p, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace tg

// Per-tensor-scaled FP8 GEMM for sm_100a:
//   C[M,N] = alpha*sa*sb * (A[M,K] . B[N,K]^T) + bias + beta*C
// Persistent, warp-specialised: one TMA producer warp feeds a multi-stage ring
// of 128-byte-swizzled K-major tiles, one MMA warp issues tcgen05.mma
// kind::f8f6f4 (128 x BN x 32 per instruction) into one of two TMEM
// accumulator buffers, four epilogue warps drain the other buffer
// (tcgen05.ld), scale, add bias and store, so the epilogue of tile i overlaps
// the main loop of tile i+1.  Replaces the kernel at
// src/tilegym/suites/flashinfer/cutile/gemm/gemm_alpha_beta.py:19-180 for e4m3 inputs.
#include "tg_gemm_common.cuh"

namespace tg {

namespace {

constexpr int kThreads = 192;  // warp 0 TMA, warp 1 MMA + TMEM owner, warps 2..5 epilogue

template <int BN>
struct PtCfg {
  static constexpr int kABytes = kBM * kBK;
  static constexpr int kBBytes = BN * kBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * BN;  // two accumulator buffers
  static constexpr int kCtrlBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kCtrlBytes + 1024;
  static_assert(kTmemCols >= 32 && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns");
  static_assert((2 * kStages + 4) * 8 + 12 <= kCtrlBytes, "control block");
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
    tg_fp8_gemm_pertensor_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                 const GemmParams p) {
  using Cfg = PtCfg<BN>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t a_base = base;
  const uint32_t b_base = base + S * Cfg::kABytes;
  uint8_t* ctrl = smem + S * Cfg::kStageBytes;
  const uint32_t bar_full = smem_u32(ctrl);         // S barriers
  const uint32_t bar_empty = bar_full + 8 * S;      // S barriers
  const uint32_t bar_tfull = bar_empty + 8 * S;     // 2 barriers
  const uint32_t bar_tempty = bar_tfull + 16;       // 2 barriers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + (2 * S + 4) * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  griddep_launch_dependents();  // the next kernel's CTAs may take the place of ours as we finish

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_tfull + 8 * i, 1);
      mbar_init(bar_tempty + 8 * i, 4);
    }
    init_abort_flag(abort_flag, p.wait_limit_us);
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
  // Programmatic dependent launch: the set-up above may have run while the previous kernel on the stream was
  // finishing; nothing below may touch global memory before that kernel has completed.
  griddep_wait();

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_units = num_tiles * p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    {
      const bool elected = elect_one();  // warp-uniform loops, one lane issues the copies
      if (elected) {
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
      }
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        const int t = u / p.splits, sp = u - t * p.splits;
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag))) {
            report_timeout(p.status, kRoleProducer * 1000 + 1);
            ok = false;
            break;
          }
          if (elected) {
            mbar_arrive_expect_tx(bar_full + 8 * s, Cfg::kStageBytes);
            tma_load_2d(a_base + s * Cfg::kABytes, &tmA, bar_full + 8 * s, kb * kBK, tm * kBM);
            tma_load_2d(b_base + s * Cfg::kBBytes, &tmB, bar_full + 8 * s, kb * kBK, tn * BN);
          }
          __syncwarp();
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    {
      const bool elected = elect_one();  // warp-uniform loops, one lane issues the tensor-core work
      const uint32_t idesc = make_idesc_e4m3_f32(kBM, BN) | ((p.flags & 32) ? kIdescFormat1 : 0u);  // e4m3 / e5m2
      int s = 0;
      uint32_t ph = 0;
      int buf = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        const int t = u / p.splits, sp = u - t * p.splits;
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
        if (!__all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * buf, aph ^ 1u, abort_flag))) {
          report_timeout(p.status, kRoleMma * 1000 + 1);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * s, ph, abort_flag))) {
            report_timeout(p.status, kRoleMma * 1000 + 2);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = make_kmajor_sw128_desc(a_base + s * Cfg::kABytes);
          const uint64_t bdesc = make_kmajor_sw128_desc(b_base + s * Cfg::kBBytes);
          if (elected) {
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              mma_f8f6f4(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            }
            tc_commit(bar_empty + 8 * s);  // frees the smem stage once these MMAs have read it
          }
          __syncwarp();
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        if (elected) tc_commit(bar_tfull + 8 * buf);  // accumulator complete
        __syncwarp();
        buf ^= 1;
        if (buf == 0) aph ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    float scale = p.alpha;
    if (p.scale_a != nullptr) scale *= __ldg(p.scale_a);
    if (p.scale_b != nullptr) scale *= __ldg(p.scale_b);
    const bool vec_ok = c_rows_aligned(p);
    int buf = 0;
    uint32_t aph = 0;
    for (int u = blockIdx.x; u < num_units; u += gridDim.x) {
      const int t = u / p.splits, sp = u - t * p.splits;
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      if (!mbar_wait(bar_tfull + 8 * buf, aph, abort_flag)) {
        report_timeout(p.status, kRoleEpilogue * 1000 + 1);
        break;
      }
      tc_fence_after();
      const int row_in_tile = q * 32 + lane;
      const int64_t row = static_cast<int64_t>(tm) * kBM + row_in_tile;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * BN);
      // partial tile of (tile, split): per 32-column chunk and lane quadrant 8 float4 per thread, lane-contiguous,
      // so that every store and load instruction of a warp covers 512 consecutive bytes
      float4* part = nullptr;
      if (p.splits > 1)
        part = reinterpret_cast<float4*>(p.ws_partial) + (static_cast<int64_t>(t) * p.splits + sp) * (kBM * BN / 4) +
               q * 256 + lane;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        if (c == BN / 32 - 1) {
          // the accumulator buffer is in registers: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
        }
        const float* acc = reinterpret_cast<const float*>(r);
        if (p.splits == 1) {
          if (row < p.M) epilogue_store32(p, row, tn * BN + c * 32, acc, scale, vec_ok);
        } else {
          float4* dst = part + c * 1024;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            __stcg(dst + j * 32, make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]));
        }
      }
      if (p.splits > 1) {
        if (splitk_arrive_is_last(p.ws_counters + t * 4 + q, p.splits)) {
          const float4* tile_part = reinterpret_cast<const float4*>(p.ws_partial) +
                                    static_cast<int64_t>(t) * p.splits * (kBM * BN / 4) + q * 256 + lane;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            float acc[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = 0.f;
            // fixed order (bit-stable result); two splits' loads are in flight together
            int s2 = 0;
#pragma unroll 1
            for (; s2 + 1 < p.splits; s2 += 2) {
              const float4* src = tile_part + static_cast<int64_t>(s2) * (kBM * BN / 4) + c * 1024;
              float4 v0[8], v1[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v0[j] = __ldcg(src + j * 32);
#pragma unroll
              for (int j = 0; j < 8; ++j) v1[j] = __ldcg(src + (kBM * BN / 4) + j * 32);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                acc[4 * j] = (acc[4 * j] + v0[j].x) + v1[j].x;
                acc[4 * j + 1] = (acc[4 * j + 1] + v0[j].y) + v1[j].y;
                acc[4 * j + 2] = (acc[4 * j + 2] + v0[j].z) + v1[j].z;
                acc[4 * j + 3] = (acc[4 * j + 3] + v0[j].w) + v1[j].w;
              }
            }
            if (s2 < p.splits) {
              const float4* src = tile_part + static_cast<int64_t>(s2) * (kBM * BN / 4) + c * 1024;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = __ldcg(src + j * 32);
                acc[4 * j] += v.x;
                acc[4 * j + 1] += v.y;
                acc[4 * j + 2] += v.z;
                acc[4 * j + 3] += v.w;
              }
            }
            if (row < p.M) epilogue_store32(p, row, tn * BN + c * 32, acc, scale, vec_ok);
          }
        }
      }
      buf ^= 1;
      if (buf == 0) aph ^= 1u;
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN>
cudaError_t launch_bn(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int num_sms,
                      cudaStream_t stream) {
  using Cfg = PtCfg<BN>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tg_fp8_gemm_pertensor_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int units = p.tiles_m * p.tiles_n * p.splits;
  const int grid = units < num_sms ? units : num_sms;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (p.flags & 2) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, tg_fp8_gemm_pertensor_kernel<BN>, tmA, tmB, p);
}

}  // namespace

cudaError_t launch_gemm_pertensor(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int bn,
                                  int num_sms, cudaStream_t stream) {
  switch (bn) {
    case 256:
      return launch_bn<256>(tmA, tmB, p, num_sms, stream);
    case 128:
      return launch_bn<128>(tmA, tmB, p, num_sms, stream);
    case 64:
      return launch_bn<64>(tmA, tmB, p, num_sms, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace tg

// Block-scaled W8A8 FP8 GEMM for sm_100a (1x128 activation scales, 128x128 weight scales):
//   C[m,n] = sum_kb As[m,kb] * Bs[n/128,kb] * (A[m, kb*128 .. +128) . B[n, kb*128 .. +128)) + bias[n] + beta*C[m,n]
// The fp32 scales are arbitrary (amax/448), so they cannot ride inside the MMA
// (hardware block scaling takes power-of-two scales); instead every 128-deep
// k-block is accumulated by the tensor core into its own TMEM buffer and
// promoted on CUDA cores: eight epilogue warps read the partial product with
// tcgen05.ld and FMA it, times As*Bs, into fp32 register accumulators, while
// the MMA warp is already filling the next of four TMEM buffers.  The tile is
// 128 x 128 = the quantisation block, so one weight scale covers a k-block.
// Two-byte outputs leave through per-warp swizzled staging buffers and bulk tensor stores.
// Replaces the kernel at src/tilegym/suites/unsloth/cutile/fp8.py:243-334.
#include "tg_gemm_common.cuh"

namespace tg {

namespace {

// Debug aid (compile with -DTG_TRACE): CTA 0 stamps %globaltimer at the steps of its first 256 k-blocks into
// the partial-sum area of the workspace, 40 MiB in, as [k-block][8] uint64 (0-2 MMA thread, 3-5 first promotion warp).
#ifdef TG_TRACE
#define TG_BS_STAMP(i, slot)                                                                            \
  do {                                                                                                  \
    if (blockIdx.x == 0 && (i) < 256 && p.ws_partial != nullptr)                                        \
      (reinterpret_cast<unsigned long long*>(p.ws_partial) + (5u << 20))[(i) * 8 + (slot)] = globaltimer_ns();        \
  } while (0)
// second table, 41 MiB in: per CTA, the times of its first unit's steps after the k-loop (first promotion warp)
#define TG_BS_STAMP2(slot)                                                                                        \
  do {                                                                                                            \
    if (threadIdx.x == 64 && p.ws_partial != nullptr && !stamped2)                                                \
      (reinterpret_cast<unsigned long long*>(p.ws_partial) + (5u << 20) + (1u << 17))[blockIdx.x * 8 + (slot)] =   \
          globaltimer_ns();                                                                                       \
  } while (0)
#else
#define TG_BS_STAMP(i, slot) \
  do {                       \
  } while (0)
#define TG_BS_STAMP2(slot) \
  do {                     \
  } while (0)
#endif

constexpr int kBN = 128;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;  // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
constexpr int kStages = 6;
constexpr int kAccBufs = 4;
constexpr int kABytes = kBM * kBK;
constexpr int kBBytes = kBN * kBK;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = kAccBufs * kBN;  // 512
constexpr int kCtrlBytes = 256;
constexpr int kOutBufBytes = 32 * 128;  // per promotion warp: 32 rows x 64 two-byte columns, 128-byte swizzle
constexpr int kOutStageBytes = kEpiWarps * kOutBufBytes;
constexpr int kSmemBytes = kStages * kStageBytes + kOutStageBytes + kCtrlBytes + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory per CTA");
static_assert((2 * kStages + 2 * kAccBufs) * 8 + 12 <= kCtrlBytes, "control block");

__global__ void __launch_bounds__(kThreads, 1)
    tg_fp8_gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                   const __grid_constant__ CUtensorMap tmC, const GemmParams p, int tma_out) {
  constexpr int S = kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t a_base = base;
  const uint32_t b_base = base + S * kABytes;
  uint8_t* out_stage = smem + S * kStageBytes;  // 1024-byte aligned
  uint8_t* ctrl = out_stage + kOutStageBytes;
  const uint32_t bar_full = smem_u32(ctrl);
  const uint32_t bar_empty = bar_full + 8 * S;
  const uint32_t bar_tfull = bar_empty + 8 * S;
  const uint32_t bar_tempty = bar_tfull + 8 * kAccBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + (2 * S + 2 * kAccBufs) * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  griddep_launch_dependents();  // the next kernel's CTAs may take the place of ours as we finish

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    for (int i = 0; i < kAccBufs; ++i) {
      mbar_init(bar_tfull + 8 * i, 1);
      mbar_init(bar_tempty + 8 * i, kEpiWarps);
    }
    init_abort_flag(abort_flag, p.wait_limit_us);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
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
            report_timeout(p.status, kRoleProducer * 1000 + 11);
            ok = false;
            break;
          }
          if (elected) {
            mbar_arrive_expect_tx(bar_full + 8 * s, kStageBytes);
            tma_load_2d(a_base + s * kABytes, &tmA, bar_full + 8 * s, kb * kBK, tm * kBM);
            tma_load_2d(b_base + s * kBBytes, &tmB, bar_full + 8 * s, kb * kBK, tn * kBN);
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
    {
      // all 32 lanes walk the loops (uniform control flow); one elected lane issues the tensor-core work
      const bool elected = elect_one();
      constexpr uint32_t idesc = make_idesc_e4m3_f32(kBM, kBN);
      int s = 0;
      uint32_t ph = 0;
      int buf = 0;
      uint32_t aph = 0;
      bool ok = true;
      [[maybe_unused]] int it = 0;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        const int t = u / p.splits, sp = u - t * p.splits;
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          if (!mbar_wait(bar_tempty + 8 * buf, aph ^ 1u, abort_flag)) {
            report_timeout(p.status, kRoleMma * 1000 + 11);
            ok = false;
            break;
          }
          if (elected) TG_BS_STAMP(it, 0);
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag)) {
            report_timeout(p.status, kRoleMma * 1000 + 12);
            ok = false;
            break;
          }
          if (elected) TG_BS_STAMP(it, 1);
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * kBN);
          const uint64_t adesc = make_kmajor_sw128_desc(a_base + s * kABytes);
          const uint64_t bdesc = make_kmajor_sw128_desc(b_base + s * kBBytes);
          if (elected) {
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              mma_f8f6f4(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, k > 0 ? 1u : 0u);
            }
            tc_commit(bar_empty + 8 * s);
            tc_commit(bar_tfull + 8 * buf);  // this k-block's partial product is complete
            TG_BS_STAMP(it, 2);
          }
          __syncwarp();
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
          if (++buf == kAccBufs) {
            buf = 0;
            aph ^= 1u;
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------- promotion + store
    const int e = warp - 2;
    const int q = warp & 3;   // TMEM lane quadrant
    const int half = e >> 2;  // which 64 of the tile's 128 columns
    const bool vec_ok = c_rows_aligned(p);
    uint8_t* my_stage = out_stage + e * kOutBufBytes;
    int buf = 0;
    uint32_t aph = 0;
    bool ok = true;
    [[maybe_unused]] int eit = 0;
    [[maybe_unused]] bool stamped2 = false;
    TG_BS_STAMP2(0);
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
      const int t = u / p.splits, sp = u - t * p.splits;
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int kb0 = sp * p.kb_per_split;
      const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
      const int row_in_tile = q * 32 + lane;
      const int64_t row = static_cast<int64_t>(tm) * kBM + row_in_tile;
      const bool row_ok = row < p.M;
      const float* as_row = p.As + (row_ok ? row : 0) * p.ldas;
      const float* bs_row = p.Bs + static_cast<int64_t>(tn) * p.ldbs;
      float acc[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc[j] = 0.f;
      float sc_next = (kb0 < kb1 && row_ok) ? __ldg(as_row + kb0) * __ldg(bs_row + kb0) : 0.f;
#pragma unroll 1
      for (int kb = kb0; kb < kb1; ++kb, ++eit) {
        const float sc = sc_next;
        if (kb + 1 < kb1 && row_ok) sc_next = __ldg(as_row + kb + 1) * __ldg(bs_row + kb + 1);
        bool w = mbar_wait(bar_tfull + 8 * buf, aph, abort_flag);
        w = __all_sync(0xffffffffu, w);
        if (!w) {
          report_timeout(p.status, kRoleEpilogue * 1000 + 11);
          ok = false;
          break;
        }
        tc_fence_after();
        if (threadIdx.x == 64) TG_BS_STAMP(eit, 3);
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                static_cast<uint32_t>(buf * kBN + half * 64);
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(t_addr, r0);
        tmem_ld_32x32(t_addr + 32, r1);
        tmem_ld_wait();
        if (threadIdx.x == 64) TG_BS_STAMP(eit, 4);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = fmaf(__uint_as_float(r0[j]), sc, acc[j]);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[32 + j] = fmaf(__uint_as_float(r1[j]), sc, acc[32 + j]);
        if (threadIdx.x == 64) TG_BS_STAMP(eit, 5);
        if (++buf == kAccBufs) {
          buf = 0;
          aph ^= 1u;
        }
      }
      if (!ok) break;
      TG_BS_STAMP2(1);
      const int col0 = tn * kBN + half * 64;
      const int row0 = tm * kBM + q * 32;
      if (p.splits == 1) {
        if (tma_out) {
          add_bias_cols<64>(p, acc, col0, 0);
          stage_and_store64(&tmC, my_stage, lane, acc, p.out_dtype, col0, row0, p.M, p.N);
        } else if (row_ok) {
          epilogue_store32(p, row, col0, acc, 1.0f, vec_ok);  // adds the bias and beta * C itself
          epilogue_store32(p, row, col0 + 32, acc + 32, 1.0f, vec_ok);
        }
      } else {
        // partial tile of (tile, split): per warp 16 float4 per thread, lane-contiguous, so that every store
        // and load instruction of a warp covers 512 consecutive bytes
        float4* part = reinterpret_cast<float4*>(p.ws_partial) +
                       ((static_cast<int64_t>(t) * p.splits + sp) * kEpiWarps + e) * (16 * 32) + lane;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          __stcg(part + j * 32, make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]));
        TG_BS_STAMP2(2);
        const bool last_arriver = splitk_arrive_is_last(p.ws_counters + t * kEpiWarps + e, p.splits);
        TG_BS_STAMP2(3);
        if (last_arriver) {
#pragma unroll
          for (int j = 0; j < 64; ++j) acc[j] = 0.f;
          const float4* tile_part = reinterpret_cast<const float4*>(p.ws_partial) +
                                    (static_cast<int64_t>(t) * p.splits * kEpiWarps + e) * (16 * 32) + lane;
          for (int s2 = 0; s2 < p.splits; ++s2) {  // fixed order: bit-stable result
            const float4* src = tile_part + static_cast<int64_t>(s2) * (kEpiWarps * 16 * 32);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float4 v = __ldcg(src + j * 32);
              acc[4 * j] += v.x;
              acc[4 * j + 1] += v.y;
              acc[4 * j + 2] += v.z;
              acc[4 * j + 3] += v.w;
            }
          }
          TG_BS_STAMP2(4);
          if (tma_out) {
            add_bias_cols<64>(p, acc, col0, 0);
            stage_and_store64(&tmC, my_stage, lane, acc, p.out_dtype, col0, row0, p.M, p.N);
          } else if (row_ok) {
            epilogue_store32(p, row, col0, acc, 1.0f, vec_ok);
            epilogue_store32(p, row, col0 + 32, acc + 32, 1.0f, vec_ok);
          }
          TG_BS_STAMP2(5);
        }
      }
#ifdef TG_TRACE
      stamped2 = true;
#endif
    }
    if (tma_out && lane == 0) tma_store_wait_all<0>();  // this warp's bulk stores have completed
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

cudaError_t launch_gemm_blockscaled(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap* tmC,
                                    const GemmParams& p, int num_sms, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tg_fp8_gemm_blockscaled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int units = p.tiles_m * p.tiles_n * p.splits;
  const int grid = units < num_sms ? units : num_sms;
  // tmC == nullptr selects the register -> global store epilogue (fp32 output or unaligned rows)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (p.flags & 2) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, tg_fp8_gemm_blockscaled_kernel, tmA, tmB, tmC != nullptr ? *tmC : tmA, p, tmC != nullptr ? 1 : 0);
}

}  // namespace tg

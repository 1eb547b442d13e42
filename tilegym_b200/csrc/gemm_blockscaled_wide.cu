// Block-scaled W8A8 FP8 GEMM for sm_100a, wide-tile version for problems that fill the GPU (no split-K):
//   C[m,n] = sum_kb As[m,kb] * Bs[n/128,kb] * (A[m, kb-block] . B[n, kb-block])
// A 128 x 128 tile moves 64 KB through shared memory per 128-deep k-block (32 KB written by TMA, 32 KB read
// by the tensor core) for 256 clocks of math, and the shared-memory pipe (about 110 B/clk/SM) caps the tensor
// pipe near 50 %.  Here the tile is 128 x 256: 96 KB per 512 clocks of math.  Each k-block is accumulated into
// one of two 256-column TMEM buffers and promoted on CUDA cores, acc += (As[m,kb] * Bs[nb,kb]) * partial
// (exact for arbitrary fp32 scales), by eight warps that each own 32 rows x 128 columns: 128 fp32
// accumulators per thread.  That needs more than the 168 registers a 384-thread CTA gets per thread, so the
// producer / MMA warpgroup hands registers to the two promotion warpgroups with setmaxnreg.
// Roles: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2-3 idle, warps 4-11 promotion + store.
#include "tg_gemm_common.cuh"

namespace tg {

namespace {

constexpr int kBN = 256;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 128 + 32 * kEpiWarps;  // 384
constexpr int kStages = 4;
constexpr int kAccBufs = 2;
constexpr int kABytes = kBM * kBK;  // 16 KB
constexpr int kBBytes = kBN * kBK;  // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = kAccBufs * kBN;  // 512
constexpr int kCtrlBytes = 256;
constexpr int kSmemBytes = kStages * kStageBytes + kCtrlBytes + 1024;
static_assert((2 * kStages + 2 * kAccBufs) * 8 + 8 <= kCtrlBytes, "control block");
static_assert(kSmemBytes <= 227 * 1024, "shared memory per CTA");

// 384 threads x 168 registers fill the register file; 128 threads give up 128 each, 256 threads take 64 each.
constexpr int kRegsLight = 40;
constexpr int kRegsHeavy = 224;
static_assert(128 * (168 - kRegsLight) >= 256 * (kRegsHeavy - 168), "register budget");

__device__ __forceinline__ void fma16x2(float2* acc, const uint32_t (&r)[32], float2 sc2) {
#pragma unroll
  for (int j = 0; j < 16; ++j)
    acc[j] = __ffma2_rn(make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), sc2, acc[j]);
}

__global__ void __launch_bounds__(kThreads, 1)
    tg_fp8_gemm_blockscaled_wide_kernel(const __grid_constant__ CUtensorMap tmA,
                                        const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  constexpr int S = kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t a_base = base;
  const uint32_t b_base = base + S * kABytes;
  uint8_t* ctrl = smem + S * kStageBytes;
  const uint32_t bar_full = smem_u32(ctrl);
  const uint32_t bar_empty = bar_full + 8 * S;
  const uint32_t bar_tfull = bar_empty + 8 * S;
  const uint32_t bar_tempty = bar_tfull + 8 * kAccBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + (2 * S + 2 * kAccBufs) * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    for (int i = 0; i < kAccBufs; ++i) {
      mbar_init(bar_tfull + 8 * i, 1);
      mbar_init(bar_tempty + 8 * i, kEpiWarps);
    }
    *abort_flag = 0u;
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

  const int num_tiles = p.tiles_m * p.tiles_n;  // 128 x 256 tiles

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLight));
    if (warp == 0) {
      const bool elected = elect_one();  // warp-uniform loops, one lane issues the copies
      if (elected) {
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
      }
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag))) {
            report_timeout(p.status, kRoleProducer * 1000 + 51);
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
    } else if (warp == 1) {
      // all 32 lanes walk the loops (uniform control flow); one elected lane issues the tensor-core work
      const bool elected = elect_one();
      constexpr uint32_t idesc = make_idesc_e4m3_f32(kBM, kBN);
      int s = 0;
      uint32_t ph = 0;
      int buf = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(bar_tempty + 8 * buf, aph ^ 1u, abort_flag)) {
            report_timeout(p.status, kRoleMma * 1000 + 51);
            ok = false;
            break;
          }
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag)) {
            report_timeout(p.status, kRoleMma * 1000 + 52);
            ok = false;
            break;
          }
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
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsHeavy));
    // ---------------------------------------------------- promotion + store
    const int e = warp - 4;
    const int q = warp & 3;   // TMEM lane quadrant
    const int half = e >> 2;  // which 128 of the tile's 256 columns = which quantisation block
    const bool vec_ok = c_rows_aligned(p);
    int buf = 0;
    uint32_t aph = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int row_in_tile = q * 32 + lane;
      const int64_t row = static_cast<int64_t>(tm) * kBM + row_in_tile;
      const int nb = tn * 2 + half;
      const bool in = row < p.M && nb * 128 < p.N;
      const float* as_row = p.As + (in ? row : 0) * p.ldas;
      const float* bs_row = p.Bs + static_cast<int64_t>(in ? nb : 0) * p.ldbs;
      float2 acc2[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc2[j] = make_float2(0.f, 0.f);
      float sc_next = in ? __ldg(as_row) * __ldg(bs_row) : 0.f;
#pragma unroll 1
      for (int kb = 0; kb < p.num_kb; ++kb) {
        const float2 sc2 = make_float2(sc_next, sc_next);
        if (kb + 1 < p.num_kb && in) sc_next = __ldg(as_row + kb + 1) * __ldg(bs_row + kb + 1);
        bool w = mbar_wait(bar_tfull + 8 * buf, aph, abort_flag);
        w = __all_sync(0xffffffffu, w);
        if (!w) {
          report_timeout(p.status, kRoleEpilogue * 1000 + 51);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                static_cast<uint32_t>(buf * kBN + half * 128);
        // two 32-column reads in flight while the previous two are multiplied in
        uint32_t ra[32], rb[32];
        tmem_ld_32x32(t_addr, ra);
        tmem_ld_32x32(t_addr + 32, rb);
        tmem_ld_wait();
        fma16x2(acc2, ra, sc2);
        tmem_ld_32x32(t_addr + 64, ra);
        fma16x2(acc2 + 16, rb, sc2);
        tmem_ld_32x32(t_addr + 96, rb);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);  // the buffer is in registers: hand it back
        fma16x2(acc2 + 32, ra, sc2);
        fma16x2(acc2 + 48, rb, sc2);
        if (++buf == kAccBufs) {
          buf = 0;
          aph ^= 1u;
        }
      }
      if (!ok) break;
      if (row < p.M) {
        const int col0 = tn * kBN + half * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float acc[32];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            acc[2 * j] = acc2[c * 16 + j].x;
            acc[2 * j + 1] = acc2[c * 16 + j].y;
          }
          epilogue_store32(p, row, col0 + c * 32, acc, 1.0f, vec_ok);
        }
      }
    }
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

cudaError_t launch_gemm_blockscaled_wide(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                                         int num_sms, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tg_fp8_gemm_blockscaled_wide_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < num_sms ? tiles : num_sms;
  tg_fp8_gemm_blockscaled_wide_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tmA, tmB, p);
  return cudaGetLastError();
}

}  // namespace tg

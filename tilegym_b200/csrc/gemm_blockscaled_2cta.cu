// Block-scaled W8A8 FP8 GEMM for sm_100a, CTA-pair version (tcgen05 cta_group::2), for M, N >= 256:
//   C[m,n] = sum_kb As[m,kb] * Bs[n/128,kb] * (A[m, kb-block] . B[n, kb-block])
// The single-CTA kernel's 128 x 128 tile moves 32 KB from L2 per 128-deep k-block for 256 tensor-core
// clocks, which the L2 -> SM path cannot sustain; here two CTAs share a 256 x 192 tile (each loads its
// own 128 rows of A and 96 rows of B: 28 KB per 384 clocks per SM, no multicast).  Each k-block is
// accumulated into one of two 192-column TMEM buffers per CTA and promoted on CUDA cores by twelve
// warps per CTA (three per TMEM lane quadrant, 64 columns each) with packed fp32x2 FMAs:
// acc += (As[m,kb] * Bs[nb,kb]) * partial, exact for arbitrary fp32 scales.
// Roles per CTA: warp 0 TMA producer, warp 1 MMA issuer (leader CTA only) and TMEM owner,
// warps 2..13 promotion + store.  Experimental (opt-in, TILEGYM_B200_BS_PAIR=1): two TMEM buffers cannot hide the
// cross-CTA release chain, so it runs slower than the single-CTA 128 x 256 kernel that is the default.
#include "tg_gemm_common.cuh"

namespace tg {

namespace {

// Tile 256 x 192: twelve promotion warps (three per TMEM lane quadrant, 64 columns each) keep the
// 128 x 192 fp32 accumulators of a CTA in registers at <= 128 registers per thread (14 warps are
// allocated as 16); a 256-wide tile would need 16 + 2 warps, which are allocated as 20 and leave only
// 96 registers per thread.
constexpr int kEpiWarps = 12;
constexpr int kThreads = 64 + 32 * kEpiWarps;  // 448
constexpr int kBN = 192;                       // tile width; each warp's 64 columns lie inside one 128-column block
constexpr int kBNHalf = kBN / 2;               // B rows each CTA loads
constexpr int kColsPerWarp = kBN / (kEpiWarps / 4);  // 64
constexpr int kStages = 7;
constexpr int kAccBufs = 2;
constexpr int kABytes = kBM * kBK;
constexpr int kBBytes = kBNHalf * kBK;
constexpr int kStageBytes = kABytes + kBBytes;  // 28 KB
constexpr int kTmemCols = 512;                  // 2 x 192 columns used; allocations are powers of two
static_assert(kAccBufs * kBN <= kTmemCols && kBBytes % 1024 == 0, "TMEM columns / swizzle-atom alignment");
constexpr int kCtrlBytes = 256;
constexpr int kSmemBytes = kStages * kStageBytes + kCtrlBytes + 1024;
static_assert((2 * kStages + 2 * kAccBufs) * 8 + 8 <= kCtrlBytes, "control block");
static_assert(kColsPerWarp == 64, "four 16-column tcgen05.ld per warp and k-block");

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  // default semantics (release at CTA scope): the tcgen05 fences order the TMEM accesses, and a
  // cluster-scope release here costs about a microsecond per arrival
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_f8f6f4_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

__device__ __forceinline__ void pair_tile_coords(int t, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gsize = min(tiles_m - first_m, group_m);
  const int r = t - g * per_group;
  tm = first_m + r % gsize;
  tn = r / gsize;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    tg_fp8_gemm_blockscaled_2cta_kernel(const __grid_constant__ CUtensorMap tmA,
                                        const __grid_constant__ CUtensorMap tmB, const GemmParams p, int group_m) {
  constexpr int S = kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t a_base = base;
  const uint32_t b_base = base + S * kABytes;
  uint8_t* ctrl = smem + S * kStageBytes;
  const uint32_t bar_full = smem_u32(ctrl);                 // S; the leader's are used
  const uint32_t bar_empty = bar_full + 8 * S;              // S; one set per CTA
  const uint32_t bar_tfull = bar_empty + 8 * S;             // kAccBufs; one set per CTA
  const uint32_t bar_tempty = bar_tfull + 8 * kAccBufs;     // kAccBufs; the leader's are used
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + (2 * S + 2 * kAccBufs) * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = (rank == 0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);   // the leader producer's arrive.expect_tx
      mbar_init(bar_empty + 8 * i, 1);  // one arrive by this CTA's promotion warp 0 per k-block
    }
    for (int i = 0; i < kAccBufs; ++i) {
      mbar_init(bar_tfull + 8 * i, 1);                // one commit by the leader's MMA thread
      mbar_init(bar_tempty + 8 * i, 2 * kEpiWarps);   // the promotion warps of both CTAs
    }
    *abort_flag = 0u;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;  // 256 x 192 pair tiles
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    {
      const bool elected = elect_one();  // warp-uniform loops, one lane issues the copies
      if (elected) {
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
      }
      const uint32_t leader_full = map_to_cta(bar_full, 0);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        int tm, tn;
        pair_tile_coords(t, p.tiles_m, p.tiles_n, group_m, tm, tn);
        const int a_row = tm * 256 + static_cast<int>(rank) * kBM;
        const int b_row = tn * kBN + static_cast<int>(rank) * kBNHalf;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag))) {
            report_timeout(p.status, kRoleProducer * 1000 + 41);
            ok = false;
            break;
          }
          if (elected) {
            if (leader) mbar_arrive_expect_tx(bar_full + 8 * s, 2 * kStageBytes);
            tma_load_2d_pair(a_base + s * kABytes, &tmA, leader_full + 8 * s, kb * kBK, a_row);
            tma_load_2d_pair(b_base + s * kBBytes, &tmB, leader_full + 8 * s, kb * kBK, b_row);
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
    if (leader) {
      const bool elected = elect_one();  // warp-uniform loops, one lane issues the tensor-core work
      constexpr uint32_t idesc = make_idesc_e4m3_f32(256, kBN);
      const uint32_t peer_tfull = map_to_cta(bar_tfull, 1);
      int s = 0;
      uint32_t ph = 0;
      int buf = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * buf, aph ^ 1u, abort_flag))) {
            report_timeout(p.status, kRoleMma * 1000 + 41);
            ok = false;
            break;
          }
          if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * s, ph, abort_flag))) {
            report_timeout(p.status, kRoleMma * 1000 + 42);
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
              mma_f8f6f4_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, k > 0 ? 1u : 0u);
            }
            // one k-block's partial product per buffer; the promotion warps free the smem stage when they see it
            tc_commit_pair(bar_tfull + 8 * buf);
            tc_commit_pair(peer_tfull + 8 * buf);
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
    // ---------------------------------------------------- promotion + store (both CTAs)
    const int e = warp - 2;
    const int q = warp & 3;   // TMEM lane quadrant
    const int part = e >> 2;  // which 64 of the tile's 256 columns
    const bool vec_ok = c_rows_aligned(p);
    const uint32_t leader_tempty = map_to_cta(bar_tempty, 0);
    int buf = 0;
    uint32_t aph = 0;
    int es = 0;  // smem stage of the k-block being promoted (same sequence as the MMA warp's)
    bool ok = true;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
      int tm, tn;
      pair_tile_coords(t, p.tiles_m, p.tiles_n, group_m, tm, tn);
      const int row_in_cta = q * 32 + lane;
      const int64_t row = static_cast<int64_t>(tm) * 256 + static_cast<int>(rank) * kBM + row_in_cta;
      const bool row_ok = row < p.M;
      const int col0 = tn * kBN + part * kColsPerWarp;
      const int nb = col0 >> 7;  // quantisation block of this warp's columns
      const bool nb_ok = nb * 128 < p.N;
      const float* as_row = p.As + (row_ok ? row : 0) * p.ldas;
      const float* bs_row = p.Bs + static_cast<int64_t>(nb_ok ? nb : 0) * p.ldbs;
      float2 acc2[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) acc2[j] = make_float2(0.f, 0.f);
      // scales are fetched a group of k-blocks ahead of their use
      constexpr int kAhead = 4;
      float sc_cur[kAhead], a_nxt[kAhead], b_nxt[kAhead];
#pragma unroll
      for (int i = 0; i < kAhead; ++i) {
        const bool in = row_ok && nb_ok && (i < p.num_kb);
        a_nxt[i] = in ? __ldg(as_row + i) : 0.f;
        b_nxt[i] = in ? __ldg(bs_row + i) : 0.f;
      }
#pragma unroll 1
      for (int kbg = 0; kbg < p.num_kb && ok; kbg += kAhead) {
#pragma unroll
        for (int i = 0; i < kAhead; ++i) {
          sc_cur[i] = a_nxt[i] * b_nxt[i];  // loaded one group ago
          const bool in = row_ok && nb_ok && (kbg + kAhead + i < p.num_kb);
          a_nxt[i] = in ? __ldg(as_row + kbg + kAhead + i) : 0.f;
          b_nxt[i] = in ? __ldg(bs_row + kbg + kAhead + i) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < kAhead; ++i) {
          if (kbg + i >= p.num_kb || !ok) break;
          const float2 sc2 = make_float2(sc_cur[i], sc_cur[i]);
          // one lane per warp polls the barrier, the vote hands the result to the other lanes
          bool w = (lane == 0) ? mbar_wait(bar_tfull + 8 * buf, aph, abort_flag) : true;
          w = __all_sync(0xffffffffu, w);
          if (!w) {
            report_timeout(p.status, kRoleEpilogue * 1000 + 41);
            ok = false;
            break;
          }
          tc_fence_after();
          // the k-block's MMAs are complete, so they have read this CTA's shared-memory stage: free it
          if (e == 0 && lane == 0) mbar_arrive(bar_empty + 8 * es);
          if (++es == S) es = 0;
          const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                  static_cast<uint32_t>(buf * kBN + part * kColsPerWarp);
#pragma unroll
          for (int c = 0; c < kColsPerWarp / 16; ++c) {
            uint32_t r[16];
            tmem_ld_32x16(t_addr + c * 16, r);
            tmem_ld_wait();
            if (c == kColsPerWarp / 16 - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(leader_tempty + 8 * buf);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
              acc2[c * 8 + j] = __ffma2_rn(make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), sc2,
                                           acc2[c * 8 + j]);
          }
          if (++buf == kAccBufs) {
            buf = 0;
            aph ^= 1u;
          }
        }
      }
      if (!ok) break;
      if (row_ok) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float acc[32];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            acc[2 * j] = acc2[h * 16 + j].x;
            acc[2 * j + 1] = acc2[h * 16 + j].y;
          }
          epilogue_store32(p, row, col0 + h * 32, acc, 1.0f, vec_ok);
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace

cudaError_t launch_gemm_blockscaled_2cta(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                                         int group_m, int num_sms, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tg_fp8_gemm_blockscaled_2cta_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  tg_fp8_gemm_blockscaled_2cta_kernel<<<2 * pairs, kThreads, kSmemBytes, stream>>>(tmA, tmB, p, group_m);
  return cudaGetLastError();
}

}  // namespace tg

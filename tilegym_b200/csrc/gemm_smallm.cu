// Small-M (decode, M <= 64) per-tensor-scaled FP8 GEMM for sm_100a.
// The problem is a weight-streaming one (N*K bytes of e4m3 against a few rows
// of activations), bound by HBM bandwidth, so the kernel is built around bytes
// in flight and a short tail rather than tensor-pipe occupancy:
//   * swap-AB: up to 128 weight rows ride the MMA's M axis (TMEM lanes), the M
//     activation rows (padded to MP = 16/32/64 by TMA zero fill) are the MMA's N;
//   * the grid is (weight-row tiles) x (K splits), about two CTAs per SM; the
//     host picks the rows per tile (a multiple of 16, at most 128) so that the
//     CTAs spread evenly over the SMs;
//   * the first ring of TMA loads is issued before the CTA's set-up barrier;
//   * split-K, cluster variant: the CTAs that share a weight tile form one
//     thread-block cluster and reduce through distributed shared memory.
//     M <= 32: every CTA pushes its fp32 partial rows into the inbox of the
//     CTA that owns them (row m belongs to rank m % splits), one cluster
//     barrier later each owner adds its rows in split order.  M > 32: every
//     CTA writes its partial tile to its own shared memory (over the idle
//     operand stages) and sends each peer the block of rows that peer owns
//     with ONE bulk copy (bytes counted on the owner's mbarrier); owners
//     acknowledge to the senders and add 4 columns per thread.  No global
//     scratch or atomics either way;
//   * split-K, workspace variant: partial tiles go to a global fp32 workspace
//     and the last-arriving warp per (tile, quadrant) reduces them.
// Same contract as the large-M kernel: C = alpha*sa*sb * A.B^T + bias + beta*C.
#include "tg_gemm_common.cuh"
#include "tg_cluster_reduce.cuh"

namespace tg {

namespace {

constexpr int kThreads = 192;  // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue

// Debug aid (compile with -DTG_TRACE): per-CTA %globaltimer stamps of the kernel's phases, written to the
// partial-sum area of the workspace (unused by the cluster variant) as [cta][16] uint64.
#ifdef TG_TRACE
#define TG_STAMP(slot)                                                                                   \
  do {                                                                                                   \
    if (p.ws_partial != nullptr)                                                                         \
      reinterpret_cast<unsigned long long*>(p.ws_partial)[blockIdx.x * 16 + (slot)] = globaltimer_ns(); \
  } while (0)
#else
#define TG_STAMP(slot) \
  do {                 \
  } while (0)
#endif

template <int MP>
struct SmCfg {
  static constexpr int kWBytes = kBM * kBK;  // room for 128 weight rows x 128 B per stage
  static constexpr int kXBytes = MP * kBK;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kStages = (MP == 16) ? 5 : (MP == 32 ? 4 : 3);
  static constexpr int kTmemCols = MP < 32 ? 32 : MP;
  // cluster reduction inbox: splits * ceil(M / splits) <= MP + 7 partial rows of 128 floats
  static constexpr int kInboxRows = MP + 8;
  static constexpr int kInboxBytes = kInboxRows * kBM * 4;
  static constexpr int kCtrlBytes = 128;
  static constexpr int kSmemBytes = kStages * kStageBytes + kInboxBytes + kCtrlBytes + 1024;
  static_assert((2 * kStages + 3) * 8 + 12 <= kCtrlBytes, "control block");
  static_assert(MP * kBM * 4 <= kStages * kStageBytes, "the partial tile lies over the idle stages");
  static_assert(2 * kSmemBytes <= 227 * 1024, "two CTAs per SM");
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

// With four epilogue warps per CTA nothing hides a branch: the per-element dispatch of smallm_store costs about a
// hundred cycles per stored value.  The helpers below decide output type and beta once per thread and leave
// straight-line convert + store sequences.
template <typename T>
__device__ __forceinline__ T smallm_cast(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 smallm_cast<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half smallm_cast<__half>(float v) {
  return __float2half_rn(v);
}
template <>
__device__ __forceinline__ float smallm_cast<float>(float v) {
  return v;
}

// Column n of the output (one value per activation row m < mv) from this thread's accumulators.
template <int MP, typename T>
__device__ __forceinline__ void smallm_store_column_as(T* c, int64_t ldc, const float (&acc)[MP], int mv, float scale,
                                                       float bias) {
#pragma unroll
  for (int m = 0; m < MP; ++m)
    if (m < mv) c[m * ldc] = smallm_cast<T>(fmaf(acc[m], scale, bias));
}

template <int MP>
__device__ __forceinline__ void smallm_store_column(const GemmParams& p, int64_t n, const float (&acc)[MP], int mv,
                                                    float scale, float bias) {
  if (p.beta != 0.f) {
#pragma unroll
    for (int m = 0; m < MP; ++m)
      if (m < mv) smallm_store(p, m, n, fmaf(acc[m], scale, bias));
  } else if (p.out_dtype == TG_BF16) {
    smallm_store_column_as<MP>(reinterpret_cast<__nv_bfloat16*>(p.C) + n, p.ldc, acc, mv, scale, bias);
  } else if (p.out_dtype == TG_F16) {
    smallm_store_column_as<MP>(reinterpret_cast<__half*>(p.C) + n, p.ldc, acc, mv, scale, bias);
  } else {
    smallm_store_column_as<MP>(reinterpret_cast<float*>(p.C) + n, p.ldc, acc, mv, scale, bias);
  }
}

// The whole [mv, 128] output tile of a CTA that owns its tile alone (no K split): the four epilogue warps
// transpose it through shared memory (`tile`, MP rows of 128 elements) and store 16 bytes per lane, so that a
// warp writes whole 128-byte lines of the row-major output instead of 64-byte pieces of 32 different rows.
// Needs 16-byte aligned output rows; `cols` (a multiple of 16 / sizeof(T)) columns of the tile exist.
template <int MP, typename T>
__device__ __forceinline__ void smallm_store_tile_as(T* c_tile, int64_t ldc, T* tile, const float (&acc)[MP],
                                                     bool have_acc, int n_local, int mv, int cols, float scale,
                                                     float bias) {
  if (have_acc) {
#pragma unroll
    for (int m = 0; m < MP; ++m) tile[m * kBM + n_local] = smallm_cast<T>(fmaf(acc[m], scale, bias));
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
  constexpr int kVec = 16 / static_cast<int>(sizeof(T));
  constexpr int kChunks = kBM / kVec;          // 16-byte chunks per row
  constexpr int kRowsPerPass = 128 / kChunks;  // rows the 128 threads cover at once
  const int chunk = n_local % kChunks, r0 = n_local / kChunks;
  if (have_acc && chunk * kVec < cols) {
#pragma unroll
    for (int i = 0; i < (MP + kRowsPerPass - 1) / kRowsPerPass; ++i) {
      const int m = r0 + i * kRowsPerPass;
      if (m < mv)
        *reinterpret_cast<uint4*>(c_tile + m * ldc + chunk * kVec) =
            *reinterpret_cast<const uint4*>(tile + m * kBM + chunk * kVec);
    }
  }
}

// Cluster reduction, owner side: rows rank, rank + splits, ... of the output, each the sum in split order of the
// partial rows the peers pushed into `inbox` (slot [split][j], 128 floats per row).  The loads of one row are
// issued together.
template <typename T>
__device__ __forceinline__ void smallm_reduce_rows_as(T* c, int64_t ldc, const float* inbox_col, int rank, int splits,
                                                      int rpr, int mv, float scale, float bias) {
  for (int j = 0; j * splits + rank < mv; ++j) {
    const float* src = inbox_col + j * kBM;
    float v[8];
#pragma unroll
    for (int s2 = 0; s2 < 8; ++s2) v[s2] = (s2 < splits) ? src[s2 * rpr * kBM] : 0.f;
    float sum = v[0];
#pragma unroll
    for (int s2 = 1; s2 < 8; ++s2)
      if (s2 < splits) sum += v[s2];  // split order: bit-stable
    c[static_cast<int64_t>(j * splits + rank) * ldc] = smallm_cast<T>(fmaf(sum, scale, bias));
  }
}

__device__ __forceinline__ uint32_t sm_cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t sm_map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void sm_st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
__device__ __forceinline__ void sm_cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void sm_cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void sm_cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int MP, bool CLUSTER>
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
  float* inbox = reinterpret_cast<float*>(smem + S * Cfg::kStageBytes);
  uint8_t* ctrl = smem + S * Cfg::kStageBytes + Cfg::kInboxBytes;
  const uint32_t bar_full = smem_u32(ctrl);
  const uint32_t bar_empty = bar_full + 8 * S;
  const uint32_t bar_tfull = bar_empty + 8 * S;
  const uint32_t bar_inbox = bar_tfull + 8;  // bytes of the peers' partial rows (cluster reduction)
  const uint32_t bar_done = bar_inbox + 8;   // acknowledgements of the owners this CTA sent rows to
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + (2 * S + 3) * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  griddep_launch_dependents();  // the next kernel's CTAs may take the place of ours as we finish
  if (threadIdx.x == 0) TG_STAMP(0);

  // one work unit per CTA: weight-row tile tn (p.tile_rows rows), K split sp
  const int u = blockIdx.x;
  const int tn = u / p.splits, sp = u - tn * p.splits;
  const int kb0 = sp * p.kb_per_split;
  const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
  const uint32_t stage_tx = static_cast<uint32_t>(p.tile_rows * kBK + Cfg::kXBytes);
  const int row0 = tn * p.tile_rows;
  uint64_t pol_w = 0, pol_x = 0;
  int pre = 0;  // k-blocks whose loads were issued before the set-up barrier

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    mbar_init(bar_tfull, 1);
    mbar_init(bar_inbox, 1);
    init_abort_flag(abort_flag, p.wait_limit_us);
    fence_mbar_init();
    if constexpr (CLUSTER) {
      // cluster reduction: every peer sends this CTA the block of output rows it owns (rows_owned x 128 floats)
      const int mv0 = p.M < MP ? p.M : MP;
      const int rpr0 = (mv0 + p.splits - 1) / p.splits;
      const int rows_owned = max(0, min(rpr0, mv0 - sp * rpr0));
      if (p.splits > 1 && rows_owned > 0)
        mbar_arrive_expect_tx(bar_inbox, static_cast<uint32_t>((p.splits - 1) * rows_owned * kBM * 4));
      // owners are the ranks 0 .. ceil(mv / rpr) - 1; this CTA sends to all of them but itself
      const int owners = (mv0 + rpr0 - 1) / rpr0;
      mbar_init(bar_done, static_cast<uint32_t>(max(1, owners - (rows_owned > 0 ? 1 : 0))));
      fence_mbar_init();
    }
    // The ring is empty and only this thread touches the full barriers until the barrier below:
    // start the weight stream right away, TMEM allocation and the other warps catch up meanwhile.
    pol_w = policy_evict_first();  // weights are read once
    pol_x = policy_evict_last();   // activations are re-read by every CTA
    pre = min(S, kb1 - kb0);
    // Programmatic dependent launch: this grid may have been started while the previous kernel on the
    // stream was still finishing.  Weights declared static are streamed right away; everything the
    // previous kernel may have produced (the activations) is touched only after griddep_wait().
    const bool early_w = (p.flags & 1) != 0;
    if (!early_w) griddep_wait();
    for (int i = 0; i < pre; ++i) {
      mbar_arrive_expect_tx(bar_full + 8 * i, stage_tx);
      tma_load_2d_hint(w_base + i * Cfg::kWBytes, &tmW, bar_full + 8 * i, (kb0 + i) * kBK, row0, pol_w);
    }
    if (early_w) griddep_wait();
    for (int i = 0; i < pre; ++i)
      tma_load_2d_hint(x_base + i * Cfg::kXBytes, &tmX, bar_full + 8 * i, (kb0 + i) * kBK, 0, pol_x);
    TG_STAMP(2);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  if constexpr (CLUSTER) {
    __syncwarp();
    // "this CTA runs and its inbox / done barriers are initialised" (thread 0's fence.mbarrier_init above publishes
    // them cluster-wide; a release here would add a device-scope fence, about a microsecond): matched by the wait
    // before the copies
    sm_cluster_arrive_relaxed();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  griddep_wait();  // every thread: no global read or write below may overtake the previous kernel
  if (threadIdx.x == 0) TG_STAMP(1);

  if (warp == 0) {
    pre = __shfl_sync(0xffffffffu, pre, 0);      // thread 0 issued the first ring
    pol_w = __shfl_sync(0xffffffffu, pol_w, 0);
    pol_x = __shfl_sync(0xffffffffu, pol_x, 0);
    {
      const bool elected = elect_one();  // warp-uniform loops, one lane issues the copies
      int s = pre % S;
      uint32_t ph = (pre == S) ? 1u : 0u;
      for (int kb = kb0 + pre; kb < kb1; ++kb) {
        if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag))) {
          report_timeout(p.status, kRoleProducer * 1000 + 21);
          break;
        }
        if (elected) {
          mbar_arrive_expect_tx(bar_full + 8 * s, stage_tx);
          tma_load_2d_hint(w_base + s * Cfg::kWBytes, &tmW, bar_full + 8 * s, kb * kBK, row0, pol_w);
          tma_load_2d_hint(x_base + s * Cfg::kXBytes, &tmX, bar_full + 8 * s, kb * kBK, 0, pol_x);
        }
        __syncwarp();
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    {
      const bool elected = elect_one();  // warp-uniform loops, one lane issues the tensor-core work
      const uint32_t idesc = make_idesc_e4m3_f32(kBM, MP) | ((p.flags & 32) ? kIdescFormat1 : 0u);  // e4m3 / e5m2
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * s, ph, abort_flag))) {
          report_timeout(p.status, kRoleMma * 1000 + 21);
          ok = false;
          break;
        }
        tc_fence_after();
        if (kb == kb0 && elected) TG_STAMP(3);
        const uint64_t wdesc = make_kmajor_sw128_desc(w_base + s * Cfg::kWBytes);
        const uint64_t xdesc = make_kmajor_sw128_desc(x_base + s * Cfg::kXBytes);
        if (elected) {
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // the MMA always spans 128 lanes; lanes >= tile_rows see stale shared memory and are never stored
            mma_f8f6f4(tmem_base, wdesc + 2u * k, xdesc + 2u * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(bar_empty + 8 * s);
        }
        __syncwarp();
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      }
      if (ok && elected) tc_commit(bar_tfull);
      if (elected) TG_STAMP(4);
      __syncwarp();
    }
  }

  // ---------------------------------------------------------------- epilogue
  const int q = warp & 3;
  const int n_local = q * 32 + lane;
  const int64_t n = static_cast<int64_t>(row0) + n_local;
  const bool n_ok = (warp >= 2) && n_local < p.tile_rows && n < p.N;
  const int mv = p.M < MP ? p.M : MP;
  float scale = p.alpha, bias = 0.f;
  float acc[MP];
  bool have_acc = false;
  if (warp >= 2) {
    if (p.scale_a != nullptr) scale *= __ldg(p.scale_a);
    if (p.scale_b != nullptr) scale *= __ldg(p.scale_b);
    if (p.bias != nullptr && n_ok) bias = load_bias(p.bias, p.bias_dtype, static_cast<int>(n));
    bool w = mbar_wait(bar_tfull, 0u, abort_flag);
    w = __all_sync(0xffffffffu, w);
    if (!w) {
      report_timeout(p.status, kRoleEpilogue * 1000 + 21);
    } else {
      tc_fence_after();
      if (threadIdx.x == 64) TG_STAMP(5);
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
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
      have_acc = true;
    }
  }

  if (p.splits == 1) {
    bool done = false;
    if constexpr (!CLUSTER) {
      const int vec = (p.out_dtype == TG_F32) ? 4 : 8;
      if (p.beta == 0.f && c_rows_aligned(p) && p.N % vec == 0) {  // the same answer in every thread
        done = true;
        if (warp >= 2) {
          const int left = static_cast<int>(p.N - row0);
          const int cols = left < p.tile_rows ? left : p.tile_rows;
          if (p.out_dtype == TG_BF16)
            smallm_store_tile_as<MP>(reinterpret_cast<__nv_bfloat16*>(p.C) + row0, p.ldc,
                                     reinterpret_cast<__nv_bfloat16*>(inbox), acc, have_acc, n_local, mv, cols, scale, bias);
          else if (p.out_dtype == TG_F16)
            smallm_store_tile_as<MP>(reinterpret_cast<__half*>(p.C) + row0, p.ldc, reinterpret_cast<__half*>(inbox), acc,
                                     have_acc, n_local, mv, cols, scale, bias);
          else
            smallm_store_tile_as<MP>(reinterpret_cast<float*>(p.C) + row0, p.ldc, inbox, acc, have_acc, n_local, mv, cols,
                                     scale, bias);
        }
      }
    }
    if (!done && have_acc && n_ok) smallm_store_column<MP>(p, n, acc, mv, scale, bias);
  } else if constexpr (CLUSTER) {
    if constexpr (MP < 64) {
      // Few rows: every CTA pushes its partial rows element by element into the owners' inboxes and one cluster
      // barrier publishes them (measured: 0.4-0.9 us faster than the bulk-copy scheme below for M <= 16, slower
      // by 0.4-1.1 us at M = 64, where 64 remote stores per thread queue up).
      // Output row m is finished by the CTA of rank m % splits; partial row m of split sp goes to slot
      // [sp][m / splits] of that CTA's inbox.  rows_per_rank = ceil(mv / splits).
      const int rpr = (mv + p.splits - 1) / p.splits;
      __syncwarp();
      sm_cluster_wait();  // every CTA of the cluster has started: its shared memory may be written
      if (have_acc && n_local < p.tile_rows) {
        const uint32_t inbox_addr = smem_u32(inbox) + static_cast<uint32_t>((sp * rpr) * kBM + n_local) * 4u;
        uint32_t r = 0, row_addr = inbox_addr;  // m = j * splits + r; row_addr = slot [sp][j] in the owner's inbox
#pragma unroll
        for (int m = 0; m < MP; ++m) {
          if (m < mv) {
            sm_st_cluster_f32(sm_map_to_cta(row_addr, r), acc[m]);
            if (++r == static_cast<uint32_t>(p.splits)) {
              r = 0;
              row_addr += kBM * 4u;
            }
          }
        }
      }
      if (threadIdx.x == 64) TG_STAMP(6);
      __syncwarp();
      sm_cluster_arrive();  // release: this CTA's pushes are done
      sm_cluster_wait();    // acquire: every peer's pushes into this CTA's inbox are visible
      if (threadIdx.x == 64) TG_STAMP(7);
      if (n_ok) {
        const int rank = static_cast<int>(sm_cluster_ctarank());
        const float* col = inbox + n_local;
        if (p.beta != 0.f) {
          for (int j = 0; j * p.splits + rank < mv; ++j) {
            const float* src = col + j * kBM;
            float sum = src[0];
            for (int s2 = 1; s2 < p.splits; ++s2) sum += src[s2 * rpr * kBM];  // split order: bit-stable
            smallm_store(p, j * p.splits + rank, n, fmaf(sum, scale, bias));
          }
        } else if (p.out_dtype == TG_BF16) {
          smallm_reduce_rows_as(reinterpret_cast<__nv_bfloat16*>(p.C) + n, p.ldc, col, rank, p.splits, rpr, mv, scale, bias);
        } else if (p.out_dtype == TG_F16) {
          smallm_reduce_rows_as(reinterpret_cast<__half*>(p.C) + n, p.ldc, col, rank, p.splits, rpr, mv, scale, bias);
        } else {
          smallm_reduce_rows_as(reinterpret_cast<float*>(p.C) + n, p.ldc, col, rank, p.splits, rpr, mv, scale, bias);
        }
      }
      if (threadIdx.x == 64) TG_STAMP(8);
      // no peer touches this CTA's shared memory after the barrier above: it may exit on its own
    } else {
      // Rank r of the cluster (= its K split) finishes the output rows [r * rpr, (r + 1) * rpr), rpr = ceil(mv / splits).
      const int rpr = (mv + p.splits - 1) / p.splits;
      const int my_r0 = sp * rpr;
      const int my_rows = max(0, min(rpr, mv - my_r0));
      float* tile = reinterpret_cast<float*>(smem);  // this CTA's partial tile [mv][128], over its idle stages
      bool clean = true;  // warps 0 and 1 have nothing to wait for here
      __syncwarp();
      sm_cluster_wait();  // every CTA of the cluster has started and armed its inbox barrier
      if (warp >= 2) {
        if (have_acc) {  // all MMAs have completed: nothing reads or fills the stages any more
#pragma unroll
          for (int m = 0; m < MP; ++m)
            if (m < mv) tile[m * kBM + n_local] = acc[m];
        }
        fence_proxy_async_smem();                       // the bulk copies below read what was just written
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps: the tile is complete
        // bias and geometry of the owner's part, fetched while the copies fly
        const int t = threadIdx.x - 64;
        const int c4 = (t & 31) * 4;
        const int left = static_cast<int>(p.N - row0);
        const int n_valid = (left < p.tile_rows ? left : p.tile_rows) - c4;
        float b4[4] = {0.f, 0.f, 0.f, 0.f};
        if (p.bias != nullptr && my_rows > 0) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (i < n_valid) b4[i] = load_bias(p.bias, p.bias_dtype, static_cast<int64_t>(row0) + c4 + i);
        }
        if (warp == 2 && have_acc && lane >= 1 && lane < p.splits) {  // lane i serves the peer i ranks further on
          const int r = (sp + lane) % p.splits;
          const int rows = max(0, min(rpr, mv - r * rpr));
          if (rows > 0)
            cl_bulk_copy_to_peer(cl_map_to_cta(smem_u32(inbox + sp * rpr * kBM), static_cast<uint32_t>(r)),
                                 smem_u32(tile + r * rpr * kBM), static_cast<uint32_t>(rows * kBM * 4),
                                 cl_map_to_cta(bar_inbox, static_cast<uint32_t>(r)));
        }
        if (threadIdx.x == 64) TG_STAMP(6);
        bool got = true;
        if (my_rows > 0) {
          got = mbar_wait(bar_inbox, 0u, abort_flag);  // the other splits' versions of this CTA's rows have landed
          got = __all_sync(0xffffffffu, got);
          if (!got) report_timeout(p.status, kRoleEpilogue * 1000 + 22);
          // every sender's tile has been read: tell the senders right away, before this CTA's own adds and stores
          if (got && warp == 2 && lane >= 1 && lane < p.splits)
            cl_mbar_arrive_remote(cl_map_to_cta(bar_done, static_cast<uint32_t>((sp + lane) % p.splits)));
        }
        if (threadIdx.x == 64) TG_STAMP(7);
        if (got && have_acc && n_valid > 0) {
          // thread -> four columns of every fourth owned row: a warp writes one 256-byte (bf16) piece of a row
          const int esz = (p.out_dtype == TG_F32) ? 4 : 2;
          const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0) && (((p.ldc * esz) & 15) == 0);
          for (int j = t >> 5; j < my_rows; j += 4) {
            const float4 sum = cl_sum_splits(tile + (my_r0 + j) * kBM + c4, inbox + j * kBM + c4, rpr, p.splits, sp);
            const float v[4] = {fmaf(sum.x, scale, b4[0]), fmaf(sum.y, scale, b4[1]), fmaf(sum.z, scale, b4[2]),
                                fmaf(sum.w, scale, b4[3])};
            if (p.beta != 0.f) {
              for (int i = 0; i < 4 && i < n_valid; ++i) smallm_store(p, my_r0 + j, static_cast<int64_t>(row0) + c4 + i, v[i]);
            } else {
              cl_store4(p, my_r0 + j, static_cast<int64_t>(row0) + c4, v, n_valid, vec_ok);
            }
          }
        }
        if (threadIdx.x == 64) TG_STAMP(8);
        // This CTA's tile must stay until every owner it sent rows to has them: wait for their acknowledgements.
        const int owners = (mv + rpr - 1) / rpr;
        if (have_acc && owners - (my_rows > 0 ? 1 : 0) > 0) {
          bool acked = mbar_wait(bar_done, 0u, abort_flag);
          acked = __all_sync(0xffffffffu, acked);
          if (!acked) report_timeout(p.status, kRoleEpilogue * 1000 + 23);
          got = got && acked;
        }
        clean = got && have_acc;
      }
      // Normal case: every copy into this CTA has landed and every copy out of it has been acknowledged, no peer
      // touches its shared memory again, and it leaves on its own.  If a wait above gave up, peers may still be
      // sending: such a CTA stays until all threads of the cluster have either left or arrived here as well
      // (barrier.cluster.wait counts non-exited threads only).
      clean = __syncthreads_and(clean ? 1 : 0) != 0;
      if (!clean) {
        sm_cluster_arrive();
        sm_cluster_wait();
      }
    }
  } else {
    if (have_acc) {
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
        if (n_ok) smallm_store_column<MP>(p, n, acc, mv, scale, bias);
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
  if (threadIdx.x == 0) TG_STAMP(9);
}

template <int MP, bool CLUSTER>
cudaError_t configure_once() {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tg_fp8_gemm_smallm_kernel<MP, CLUSTER>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SmCfg<MP>::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  return cudaSuccess;
}

template <int MP>
cudaError_t launch_mp_cluster(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p,
                              cudaStream_t stream) {
  cudaError_t e = configure_once<MP, true>();
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.tiles_n * p.splits), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = SmCfg<MP>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(p.splits);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch: this grid may start while the previous kernel's last CTAs finish
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (p.flags & 2) ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, tg_fp8_gemm_smallm_kernel<MP, true>, tmW, tmX, p);
}

template <int MP>
cudaError_t launch_mp(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, cudaStream_t stream) {
  cudaError_t e = configure_once<MP, false>();
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.tiles_n * p.splits), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = SmCfg<MP>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (p.flags & 2) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, tg_fp8_gemm_smallm_kernel<MP, false>, tmW, tmX, p);
}

}  // namespace

cudaError_t launch_gemm_smallm_cluster(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int mp,
                                       cudaStream_t stream) {
  if (p.splits < 1 || p.splits > 8) return cudaErrorInvalidValue;  // portable cluster size
  if (p.tile_rows < 16 || p.tile_rows > 128) return cudaErrorInvalidValue;
  switch (mp) {
    case 16:
      return launch_mp_cluster<16>(tmW, tmX, p, stream);
    case 32:
      return launch_mp_cluster<32>(tmW, tmX, p, stream);
    case 64:
      return launch_mp_cluster<64>(tmW, tmX, p, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

cudaError_t launch_gemm_smallm(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int mp,
                               cudaStream_t stream) {
  if (p.tile_rows < 16 || p.tile_rows > 128) return cudaErrorInvalidValue;
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

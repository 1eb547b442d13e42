// Block-scaled W8A8 FP8 GEMM for sm_100a, small-M version (M <= 128):
//   C[m,n] = sum_kb As[m,kb] * Bs[n/128,kb] * (A[m, kb-block] . B[n, kb-block]) + bias[n]
// With few activation rows the problem is a weight-streaming one (N*K bytes of e4m3), bound by HBM, and the
// 128-row tiles of the large-M kernels leave most SMs without work.  This kernel is built like the per-tensor
// small-M kernel:
//   * swap-AB: 128 weight rows (exactly one 128 x 128 quantisation block per k-block) ride the MMA's M axis
//     (TMEM lanes), the activation rows (padded to MP = 32 / 64 / 128 by TMA zero fill) are the MMA's N;
//   * the grid is (weight-row tiles) x (K splits), one CTA per SM, all resident at once when the problem
//     allows; the first ring of TMA loads is issued before the CTA's set-up barrier;
//   * every 128-deep k-block is accumulated into one of two TMEM buffers and promoted on CUDA cores by four
//     warps: thread = weight row, acc[m] += (As[m,kb] * Bs[nb,kb]) * partial[m].  The products As * Bs of the
//     CTA's k-range are staged once in shared memory as [k-block][m] and read as broadcasts;
//   * the K splits of a tile form a thread-block cluster and reduce through distributed shared memory: after its
//     main loop every CTA writes its fp32 partial tile to its own shared memory and sends each peer the block
//     of rows that peer owns with ONE bulk copy (cp.async.bulk shared::cta -> shared::cluster, completion counted
//     in bytes on the owner's mbarrier); each owner acknowledges to the senders (a remote mbarrier arrive, so a
//     sender leaves as soon as its rows are taken), adds its rows in split order (bit-stable) and stores whole
//     256-byte row pieces.  No global scratch, no per-element remote stores;
//   * a tile that is not split is transposed through shared memory and stored as whole 16-byte pieces of rows.
// Roles: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2-5 promotion + store.
// Replaces, for small M, the kernel at src/tilegym/suites/unsloth/cutile/fp8.py:243-334.
#include "tg_gemm_common.cuh"
#include "tg_cluster_reduce.cuh"

namespace tg {

namespace {

// Debug aid (compile with -DTG_TRACE): every CTA stamps %globaltimer at the steps of its work into the
// partial-sum area of the workspace, 40 MiB in, as [CTA][64] uint64: 0 start, 1 set-up done, 2 scale table ready,
// 8+i / 16+i / 24+i / 32+i for k-block i < 8: MMAs issued / partial product seen / buffer released / multiplied in,
// 40 main loop done, 41 cluster ready, 42 pushed, 43 all pushes in, 44 stored.
#ifdef TG_TRACE
#define TG_BSM_STAMP(slot)                                                                                      \
  do {                                                                                                          \
    if (p.ws_partial != nullptr && blockIdx.x < 512)                                                            \
      (reinterpret_cast<unsigned long long*>(p.ws_partial) + (5u << 20))[blockIdx.x * 64 + (slot)] = globaltimer_ns(); \
  } while (0)
#else
#define TG_BSM_STAMP(slot) \
  do {                     \
  } while (0)
#endif

constexpr int kThreads = 192;
constexpr int kMaxKbPerCta = 32;  // k-blocks one CTA may own (rows of the staged scale table)

// TWO: sized for two CTAs per SM (MP <= 64: one short work unit per CTA, so one CTA's start-up and reduction run
// beside the other's weight stream; half the stages each keep the bytes in flight per SM the same).
template <int MP, bool TWO = false>
struct BsmCfg {
  static constexpr int kWBytes = kBM * kBK;  // 128 weight rows x 128 B per stage
  static constexpr int kXBytes = MP * kBK;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kStages = TWO ? 4 : ((MP == 128) ? 6 : 8);
  static constexpr int kTmemCols = 2 * MP;  // two partial-product buffers
  // After the main loop the operand stages are idle and hold (a) this CTA's fp32 partial tile [MP][128] (the
  // unsplit path: the transposition tile of the output) and (b) the cluster reduction inbox: the partial rows
  // this CTA owns, one block per split, splits * ceil(M / splits) <= MP + 7 rows of 128 floats.  A cluster
  // barrier separates every CTA's main loop from the first bulk copy into an inbox.
  static constexpr int kTileBytes = MP * kBM * 4;
  static constexpr int kInboxRows = MP + 8;
  static constexpr int kInboxBytes = kTileBytes + kInboxRows * kBM * 4;
  static constexpr int kScaleBytes = kMaxKbPerCta * MP * 4;  // As * Bs of the CTA's k-range, [k-block][m]
  static constexpr int kCtrlBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kScaleBytes + kCtrlBytes + 1024;
  static_assert(kInboxBytes <= kStages * kStageBytes, "tile and inbox lie over the stages");
  static_assert((2 * kStages + 6) * 8 + 12 <= kCtrlBytes, "control block");
  static_assert(kSmemBytes * (TWO ? 2 : 1) <= 227 * 1024, "shared memory per SM");
  static_assert(kTmemCols * (TWO ? 2 : 1) <= 512, "TMEM columns per SM");
};

template <typename T>
__device__ __forceinline__ T bsm_cast(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 bsm_cast<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half bsm_cast<__half>(float v) {
  return __float2half_rn(v);
}
template <>
__device__ __forceinline__ float bsm_cast<float>(float v) {
  return v;
}

// Unsplit tile: the four promotion warps write their columns into `tile` ([MP][128] elements of T), then every
// thread stores 16-byte pieces of rows, so that a warp writes whole lines of the row-major output.
template <int MP, typename T>
__device__ __forceinline__ void bsm_store_tile(T* c_tile, int64_t ldc, T* tile, const float (&acc)[MP], bool have_acc,
                                               int n_local, int mv, int cols, float bias) {
  if (have_acc) {
#pragma unroll
    for (int m = 0; m < MP; ++m) tile[m * kBM + n_local] = bsm_cast<T>(acc[m] + bias);
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");  // the four promotion warps
  constexpr int kVec = 16 / static_cast<int>(sizeof(T));
  constexpr int kChunks = kBM / kVec;          // 16-byte chunks per row
  constexpr int kRowsPerPass = 128 / kChunks;  // rows the 128 threads cover at once
  const int chunk = n_local % kChunks, r0 = n_local / kChunks;
  if (have_acc && chunk * kVec < cols) {
#pragma unroll 4
    for (int i = 0; i < (MP + kRowsPerPass - 1) / kRowsPerPass; ++i) {
      const int m = r0 + i * kRowsPerPass;
      if (m < mv)
        *reinterpret_cast<uint4*>(c_tile + m * ldc + chunk * kVec) =
            *reinterpret_cast<const uint4*>(tile + m * kBM + chunk * kVec);
    }
  }
}

// One output column (weight row n) from this thread's accumulators, any alignment.
template <int MP, typename T>
__device__ __forceinline__ void bsm_store_column(T* c, int64_t ldc, const float (&acc)[MP], int mv, float bias) {
#pragma unroll
  for (int m = 0; m < MP; ++m)
    if (m < mv) c[m * ldc] = bsm_cast<T>(acc[m] + bias);
}

// Grouped form (GROUPED, never split): the mixture-of-experts GEMM when every expert has few rows.  Rows
// [m_indptr[g], m_indptr[g + 1]) of X use weight g (W viewed as [groups * N, K]); the MP-row tiles of all groups are
// numbered densely, one CTA per (row tile, 128 weight rows), the grid sized by the host's bound on the tile count;
// a CTA beyond the real count leaves at once.  Rows of the X tile past the end of its group belong to other groups:
// their scales are staged as 0 and they are never stored.
struct BsmGroupTile {
  int group;
  int row0;   // first row of X, As and C
  int rows;   // valid rows of the tile (<= MP)
  int valid;
};

template <int MP>
__device__ __forceinline__ BsmGroupTile bsm_locate_group_tile(int j, const GemmParams& p, int lane) {
  BsmGroupTile r = {0, 0, 0, 0};
  if (p.m_indptr == nullptr) {  // one group holding all M rows: the dense problem on this kernel's launch shape
    if (j * MP < p.M) {
      r.row0 = j * MP;
      r.rows = min(MP, p.M - r.row0);
      r.valid = 1;
    }
    return r;
  }
  int before = 0;  // tiles of the groups already scanned
  for (int g0 = 0; g0 < p.num_groups; g0 += 32) {
    const int g = g0 + lane;
    // clamped to [0, M]: whatever the offsets hold, no row outside X / C is ever touched
    const int beg = g < p.num_groups ? min(max(__ldg(p.m_indptr + g), 0), p.M) : 0;
    const int end = g < p.num_groups ? min(max(__ldg(p.m_indptr + g + 1), 0), p.M) : 0;
    const int tiles = end > beg ? (end - beg + MP - 1) / MP : 0;
    int incl = tiles;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    const int excl = before + incl - tiles;
    const bool mine = tiles > 0 && j >= excl && j < excl + tiles;
    const unsigned hit = __ballot_sync(0xffffffffu, mine);
    if (hit != 0u) {
      const int src = __ffs(hit) - 1;
      const int gbeg = __shfl_sync(0xffffffffu, beg, src), gend = __shfl_sync(0xffffffffu, end, src);
      const int gexcl = __shfl_sync(0xffffffffu, excl, src);
      r.group = g0 + src;
      r.row0 = gbeg + (j - gexcl) * MP;
      r.rows = min(MP, gend - r.row0);
      r.valid = 1;
      return r;
    }
    before += __shfl_sync(0xffffffffu, incl, 31);
  }
  return r;
}

// Up to 64 activation rows the kernel is sized for two CTAs per SM (see BsmCfg): twice as many K splits stay
// resident, and one CTA's start-up and reduction run beside the other's weight stream.
__host__ __device__ constexpr bool bsm_two_per_sm(int mp) { return mp <= 64; }

template <int MP, bool CLUSTER, bool GROUPED = false>
__global__ void __launch_bounds__(kThreads, bsm_two_per_sm(MP) ? 2 : 1)
    tg_fp8_gemm_blockscaled_smallm_kernel(const __grid_constant__ CUtensorMap tmW,
                                          const __grid_constant__ CUtensorMap tmX, const GemmParams p) {
  static_assert(!(GROUPED && CLUSTER), "the grouped form is never split");
  using Cfg = BsmCfg<MP, bsm_two_per_sm(MP)>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t w_base = base;
  const uint32_t x_base = base + S * Cfg::kWBytes;
  float* inbox = reinterpret_cast<float*>(smem);  // over the stages, used after the main loop only
  float* sc_tab = reinterpret_cast<float*>(smem + S * Cfg::kStageBytes);  // [kb][MP]
  uint8_t* ctrl = smem + S * Cfg::kStageBytes + Cfg::kScaleBytes;
  const uint32_t bar_full = smem_u32(ctrl);
  const uint32_t bar_empty = bar_full + 8 * S;
  const uint32_t bar_tfull = bar_empty + 8 * S;   // 2
  const uint32_t bar_tempty = bar_tfull + 16;     // 2
  const uint32_t bar_inbox = bar_tempty + 16;     // 1: bytes of the peers' partial rows (cluster reduction)
  const uint32_t bar_done = bar_inbox + 8;        // 1: acknowledgements of the owners this CTA sent rows to
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + (2 * S + 6) * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  griddep_launch_dependents();  // the next kernel's CTAs may take the place of ours as we finish
  if (threadIdx.x == 0) TG_BSM_STAMP(0);

  // one work unit per CTA: weight-row tile tn (128 rows = one row of Bs), K split sp
  const int u = blockIdx.x;
  int tn, sp;
  int x_row0 = 0;              // first activation row of the tile (grouped form)
  int mv_tile = p.M < MP ? p.M : MP;  // valid activation rows
  int64_t w_row0;              // first weight row in the [groups * N, K] view
  int64_t bs_row;              // row of Bs
  int64_t bias_off = 0;        // grouped form: offset of the group's bias row
  if constexpr (GROUPED) {
    // m_indptr comes from the kernel in front (the routing): nothing of this CTA may run ahead of it
    griddep_wait();
    __shared__ BsmGroupTile gt_s;
    tn = u % p.tiles_n;
    sp = 0;
    if (warp == 0) {
      const BsmGroupTile gt = bsm_locate_group_tile<MP>(u / p.tiles_n, p, lane);
      if (lane == 0) gt_s = gt;
    }
    __syncthreads();
    const BsmGroupTile gt = gt_s;
    if (!gt.valid) return;  // beyond the last tile: the whole CTA leaves before it owns anything
    x_row0 = gt.row0;
    mv_tile = gt.rows;
    w_row0 = static_cast<int64_t>(gt.group) * p.N + static_cast<int64_t>(tn) * kBM;
    bs_row = static_cast<int64_t>(gt.group) * p.tiles_n + tn;
    bias_off = static_cast<int64_t>(gt.group) * p.N;
  } else {
    tn = u / p.splits;
    sp = u - tn * p.splits;
    w_row0 = static_cast<int64_t>(tn) * kBM;
    bs_row = tn;
  }
  const int kb0 = sp * p.kb_per_split;
  const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
  const int row0 = tn * kBM;  // first output column of the tile (within the group)
  uint64_t pol_w = 0, pol_x = 0;
  int pre = 0;  // k-blocks whose loads were issued before the set-up barrier

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_tfull + 8 * i, 1);
      mbar_init(bar_tempty + 8 * i, 4);  // the four promotion warps
    }
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
    // The ring is empty and only this thread touches the full barriers until the barrier below: start the
    // weight stream right away, TMEM allocation and the other warps catch up meanwhile.
    pol_w = policy_evict_first();  // weights are read once
    pol_x = policy_evict_last();   // activations are re-read by every CTA
    pre = min(S, kb1 - kb0);
    // Programmatic dependent launch: weights declared static (flags bit 0) are streamed before the wait for the
    // previous kernel on the stream; everything it may have produced (the activations) only after it.
    const bool early_w = (p.flags & 1) != 0;
    if (!early_w) griddep_wait();
    for (int i = 0; i < pre; ++i) {
      mbar_arrive_expect_tx(bar_full + 8 * i, Cfg::kStageBytes);
      tma_load_2d_hint(w_base + i * Cfg::kWBytes, &tmW, bar_full + 8 * i, (kb0 + i) * kBK, static_cast<int>(w_row0), pol_w);
    }
    if (early_w) griddep_wait();
    for (int i = 0; i < pre; ++i)
      tma_load_2d_hint(x_base + i * Cfg::kXBytes, &tmX, bar_full + 8 * i, (kb0 + i) * kBK, x_row0, pol_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  griddep_wait();  // every thread: no global read or write below may overtake the previous kernel
  if (threadIdx.x == 0) TG_BSM_STAMP(1);

  const int mv = mv_tile;
  const int q = warp & 3;
  const int n_local = q * 32 + lane;
  const int64_t n = static_cast<int64_t>(row0) + n_local;
  const bool n_ok = (warp >= 2) && n < p.N;
  float acc[MP];
  bool have_acc = false;

  if (warp == 0) {
    pre = __shfl_sync(0xffffffffu, pre, 0);  // thread 0 issued the first ring
    pol_w = __shfl_sync(0xffffffffu, pol_w, 0);
    pol_x = __shfl_sync(0xffffffffu, pol_x, 0);
    const bool elected = elect_one();  // warp-uniform loops, one lane issues the copies
    int s = pre % S;
    uint32_t ph = (pre == S) ? 1u : 0u;
    for (int kb = kb0 + pre; kb < kb1; ++kb) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag))) {
        report_timeout(p.status, kRoleProducer * 1000 + 71);
        break;
      }
      if (elected) {
        mbar_arrive_expect_tx(bar_full + 8 * s, Cfg::kStageBytes);
        tma_load_2d_hint(w_base + s * Cfg::kWBytes, &tmW, bar_full + 8 * s, kb * kBK, static_cast<int>(w_row0), pol_w);
        tma_load_2d_hint(x_base + s * Cfg::kXBytes, &tmX, bar_full + 8 * s, kb * kBK, x_row0, pol_x);
      }
      __syncwarp();
      if (++s == S) {
        s = 0;
        ph ^= 1u;
      }
    }
  } else if (warp == 1) {
    const bool elected = elect_one();  // warp-uniform loops, one lane issues the tensor-core work
    constexpr uint32_t idesc = make_idesc_e4m3_f32(kBM, MP);
    int s = 0;
    uint32_t ph = 0;
    int buf = 0;
    uint32_t aph = 0;
    for (int kb = kb0; kb < kb1; ++kb) {
      if (!__all_sync(0xffffffffu, mbar_wait<false>(bar_tempty + 8 * buf, aph ^ 1u, abort_flag))) {
        report_timeout(p.status, kRoleMma * 1000 + 71);
        break;
      }
      if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * s, ph, abort_flag))) {
        report_timeout(p.status, kRoleMma * 1000 + 72);
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * MP);
      const uint64_t wdesc = make_kmajor_sw128_desc(w_base + s * Cfg::kWBytes);
      const uint64_t xdesc = make_kmajor_sw128_desc(x_base + s * Cfg::kXBytes);
      if (elected) {
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k)
          mma_f8f6f4(d_tmem, wdesc + 2u * k, xdesc + 2u * k, idesc, k > 0 ? 1u : 0u);
        tc_commit(bar_empty + 8 * s);
        tc_commit(bar_tfull + 8 * buf);  // this k-block's partial product is complete
        if (kb - kb0 < 8) TG_BSM_STAMP(8 + kb - kb0);
      }
      __syncwarp();
      if (++s == S) {
        s = 0;
        ph ^= 1u;
      }
      buf ^= 1;
      if (buf == 0) aph ^= 1u;
    }
  } else {
    // ------------------------------------------------------------ promotion (warps 2-5)
    // stage sc_tab[j][m] = As[m, kb0 + j] * Bs[tn, kb0 + j] (0 for rows >= M): thread t fills row m = t
    {
      const int t = threadIdx.x - 64;
      const int nkb = kb1 - kb0;
      const float* bs_ptr = p.Bs + bs_row * p.ldbs + kb0;
      for (int m = t; m < MP; m += 128) {
        const float* as_row = p.As + static_cast<int64_t>(m < mv ? x_row0 + m : 0) * p.ldas + kb0;
#pragma unroll 8
        for (int j = 0; j < nkb; ++j)  // independent loads: several are in flight at once
          sc_tab[j * MP + m] = (m < mv) ? __ldg(as_row + j) * __ldg(bs_ptr + j) : 0.f;
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four promotion warps: the table is complete
    if (threadIdx.x == 64) TG_BSM_STAMP(2);
#pragma unroll
    for (int m = 0; m < MP; ++m) acc[m] = 0.f;
    int buf = 0;
    uint32_t aph = 0;
    bool ok = true;
    float2* acc2 = reinterpret_cast<float2*>(acc);
#pragma unroll 1
    for (int kb = kb0; kb < kb1; ++kb) {
      bool w = mbar_wait<false>(bar_tfull + 8 * buf, aph, abort_flag);  // latency-critical hand-over: plain polling
      w = __all_sync(0xffffffffu, w);
      if (!w) {
        report_timeout(p.status, kRoleEpilogue * 1000 + 71);
        ok = false;
        break;
      }
      tc_fence_after();
      if (threadIdx.x == 64 && kb - kb0 < 8) TG_BSM_STAMP(16 + kb - kb0);
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * MP);
      const float4* sc4 = reinterpret_cast<const float4*>(sc_tab + (kb - kb0) * MP);
      // acc[c0 .. c0 + 32) += r * scale; the scales are read as broadcasts (every lane the same address)
      auto fma32 = [&](const uint32_t (&r)[32], int c0) {
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 s4 = sc4[(c0 >> 2) + g];
          acc2[(c0 >> 1) + 2 * g] = __ffma2_rn(make_float2(__uint_as_float(r[4 * g]), __uint_as_float(r[4 * g + 1])),
                                               make_float2(s4.x, s4.y), acc2[(c0 >> 1) + 2 * g]);
          acc2[(c0 >> 1) + 2 * g + 1] = __ffma2_rn(make_float2(__uint_as_float(r[4 * g + 2]), __uint_as_float(r[4 * g + 3])),
                                                   make_float2(s4.z, s4.w), acc2[(c0 >> 1) + 2 * g + 1]);
        }
      };
      auto release = [&]() {  // the buffer is in registers: hand it back to the MMA warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
        if (threadIdx.x == 64 && kb - kb0 < 8) TG_BSM_STAMP(24 + kb - kb0);
      };
      if constexpr (MP == 32) {
        uint32_t ra[32];
        tmem_ld_32x32(t_addr, ra);
        tmem_ld_wait();
        release();
        fma32(ra, 0);
      } else {
        uint32_t ra[32], rb[32];
        tmem_ld_32x32(t_addr, ra);
        tmem_ld_32x32(t_addr + 32, rb);
        tmem_ld_wait();
        if constexpr (MP == 64) {
          release();
          fma32(ra, 0);
          fma32(rb, 32);
        } else {  // two 32-column reads in flight while the previous two are multiplied in
          fma32(ra, 0);
          tmem_ld_32x32(t_addr + 64, ra);
          fma32(rb, 32);
          tmem_ld_32x32(t_addr + 96, rb);
          tmem_ld_wait();
          release();
          fma32(ra, 64);
          fma32(rb, 96);
        }
      }
      if (threadIdx.x == 64 && kb - kb0 < 8) TG_BSM_STAMP(32 + kb - kb0);
      buf ^= 1;
      if (buf == 0) aph ^= 1u;
    }
    if (threadIdx.x == 64) TG_BSM_STAMP(40);
    have_acc = ok;
  }

  // ---------------------------------------------------------------- reduction and store
  float bias = 0.f;
  if (n_ok && p.bias != nullptr) bias = load_bias(p.bias, p.bias_dtype, bias_off + n);
  if (p.splits == 1) {
    if (warp >= 2) {
      if constexpr (GROUPED) {
        if (have_acc && p.row_scale != nullptr) {  // e.g. the routing weight of a mixture-of-experts row
#pragma unroll
          for (int m = 0; m < MP; ++m) acc[m] *= (m < mv) ? __ldg(p.row_scale + x_row0 + m) : 0.f;  // broadcast loads
        }
      }
      const int vec = (p.out_dtype == TG_F32) ? 4 : 8;
      const int left = static_cast<int>(p.N - row0);
      const int cols = left < kBM ? left : kBM;
      const int64_t c_off = static_cast<int64_t>(x_row0) * p.ldc;  // first row of the tile's rows in C (0 unless grouped)
      if (c_rows_aligned(p) && p.N % vec == 0) {  // the same answer in every thread
        if (p.out_dtype == TG_BF16)
          bsm_store_tile<MP>(reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + row0, p.ldc,
                             reinterpret_cast<__nv_bfloat16*>(inbox), acc, have_acc, n_local, mv, cols, bias);
        else if (p.out_dtype == TG_F16)
          bsm_store_tile<MP>(reinterpret_cast<__half*>(p.C) + c_off + row0, p.ldc, reinterpret_cast<__half*>(inbox), acc,
                             have_acc, n_local, mv, cols, bias);
        else
          bsm_store_tile<MP>(reinterpret_cast<float*>(p.C) + c_off + row0, p.ldc, inbox, acc, have_acc, n_local, mv, cols,
                             bias);
      } else if (have_acc && n_ok) {
        if (p.out_dtype == TG_BF16)
          bsm_store_column<MP>(reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + n, p.ldc, acc, mv, bias);
        else if (p.out_dtype == TG_F16)
          bsm_store_column<MP>(reinterpret_cast<__half*>(p.C) + c_off + n, p.ldc, acc, mv, bias);
        else
          bsm_store_column<MP>(reinterpret_cast<float*>(p.C) + c_off + n, p.ldc, acc, mv, bias);
      }
    }
  } else if constexpr (CLUSTER) {
    // Rank r of the cluster (= its K split) finishes the output rows [r * rpr, (r + 1) * rpr), rpr = ceil(mv / splits).
    const int rpr = (mv + p.splits - 1) / p.splits;
    const int my_r0 = sp * rpr;
    const int my_rows = max(0, min(rpr, mv - my_r0));
    float* tile = inbox;              // this CTA's partial tile, [MP][128] fp32
    float* inb = inbox + MP * kBM;    // [split][rpr][128]: the rows this CTA owns, as the other splits computed them
    bool clean = true;                // warps 0 and 1 have nothing to wait for here
    // Every CTA of the cluster has finished its main loop (its promotion warps have seen the last k-block's
    // MMAs complete, so nothing reads or fills its stages any more): tiles and inboxes, which lie over the
    // stages, may be written.
    __syncwarp();
    cl_arrive();
    cl_wait();
    if (threadIdx.x == 64) TG_BSM_STAMP(41);
    if (warp >= 2) {
      if (have_acc) {
#pragma unroll
        for (int m = 0; m < MP; ++m)
          if (m < mv) tile[m * kBM + n_local] = acc[m];
      }
      fence_proxy_async_smem();                       // the bulk copies below read what was just written
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four promotion warps: the tile is complete
      // geometry and bias of the owner's part, fetched while the copies fly
      const int t = threadIdx.x - 64;
      const int c4 = (t & 31) * 4;
      const int left = static_cast<int>(p.N - row0);
      const int n_valid = (left < kBM ? left : kBM) - c4;
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
          cl_bulk_copy_to_peer(cl_map_to_cta(smem_u32(inb + sp * rpr * kBM), static_cast<uint32_t>(r)),
                               smem_u32(tile + r * rpr * kBM), static_cast<uint32_t>(rows * kBM * 4),
                               cl_map_to_cta(bar_inbox, static_cast<uint32_t>(r)));
      }
      if (threadIdx.x == 64) TG_BSM_STAMP(42);
      bool got = true;
      if (my_rows > 0) {
        got = mbar_wait(bar_inbox, 0u, abort_flag);  // the other splits' versions of this CTA's rows have landed
        got = __all_sync(0xffffffffu, got);
        if (!got) report_timeout(p.status, kRoleEpilogue * 1000 + 72);
        // every sender's tile has been read: tell the senders right away, before this CTA's own adds and stores
        if (got && warp == 2 && lane >= 1 && lane < p.splits)
          cl_mbar_arrive_remote(cl_map_to_cta(bar_done, static_cast<uint32_t>((sp + lane) % p.splits)));
      }
      if (threadIdx.x == 64) TG_BSM_STAMP(43);
      if (got && have_acc && n_valid > 0) {
        // thread -> four columns of every fourth owned row: a warp writes one 256-byte (bf16) piece of a row
        const int esz = (p.out_dtype == TG_F32) ? 4 : 2;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0) && (((p.ldc * esz) & 15) == 0);
        for (int j = t >> 5; j < my_rows; j += 4) {
          const float4 sum = cl_sum_splits(tile + (my_r0 + j) * kBM + c4, inb + j * kBM + c4, rpr, p.splits, sp);
          const float v[4] = {sum.x + b4[0], sum.y + b4[1], sum.z + b4[2], sum.w + b4[3]};
          cl_store4(p, my_r0 + j, static_cast<int64_t>(row0) + c4, v, n_valid, vec_ok);
        }
      }
      // This CTA's tile must stay until every owner it sent rows to has them: wait for their acknowledgements.
      const int owners = (mv + rpr - 1) / rpr;
      if (have_acc && owners - (my_rows > 0 ? 1 : 0) > 0) {
        bool acked = mbar_wait(bar_done, 0u, abort_flag);
        acked = __all_sync(0xffffffffu, acked);
        if (!acked) report_timeout(p.status, kRoleEpilogue * 1000 + 73);
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
      cl_arrive();
      cl_wait();
    }
  }

  if (threadIdx.x == 64) TG_BSM_STAMP(44);
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int MP>
cudaError_t launch_bsm(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, cudaStream_t stream) {
  static bool configured[64][2] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const bool cluster = p.splits > 1;
  if (dev >= 0 && dev < 64 && !configured[dev][cluster ? 1 : 0]) {
    cudaError_t e = cluster ? cudaFuncSetAttribute(tg_fp8_gemm_blockscaled_smallm_kernel<MP, true>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, BsmCfg<MP, bsm_two_per_sm(MP)>::kSmemBytes)
                            : cudaFuncSetAttribute(tg_fp8_gemm_blockscaled_smallm_kernel<MP, false>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, BsmCfg<MP, bsm_two_per_sm(MP)>::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev][cluster ? 1 : 0] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.tiles_n * p.splits), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = BsmCfg<MP, bsm_two_per_sm(MP)>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (cluster) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = static_cast<unsigned>(p.splits);
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (p.flags & 2) {  // programmatic dependent launch: this grid may start while the previous kernel's last CTAs finish
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (cluster) return cudaLaunchKernelEx(&cfg, tg_fp8_gemm_blockscaled_smallm_kernel<MP, true>, tmW, tmX, p);
  return cudaLaunchKernelEx(&cfg, tg_fp8_gemm_blockscaled_smallm_kernel<MP, false>, tmW, tmX, p);
}

}  // namespace

int blockscaled_smallm_max_kb_per_cta() { return kMaxKbPerCta; }

namespace {
template <int MP>
int max_clusters(int splits) {
  cudaFuncSetAttribute(tg_fp8_gemm_blockscaled_smallm_kernel<MP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       BsmCfg<MP, bsm_two_per_sm(MP)>::kSmemBytes);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(splits * 64), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = BsmCfg<MP, bsm_two_per_sm(MP)>::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(splits);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, tg_fp8_gemm_blockscaled_smallm_kernel<MP, true>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}
}  // namespace

// How many clusters of `splits` CTAs of the small-M kernel (activation rows padded to mp) the current device
// holds at once (cluster placement is per GPC, so this is not num_sms / splits); cached per device.
int blockscaled_smallm_resident_clusters(int mp, int splits, int num_sms) {
  if (splits <= 1) return bsm_two_per_sm(mp) ? 2 * num_sms : num_sms;
  if (splits > 8) return 0;
  static int cache[64][3][9] = {};  // 0 = not asked yet, -1 = none
  int dev = 0;
  cudaGetDevice(&dev);
  const int mi = mp == 32 ? 0 : (mp == 64 ? 1 : 2);
  if (dev < 0 || dev >= 64) return 0;
  int& c = cache[dev][mi][splits];
  if (c == 0) {
    int n = mp == 32 ? max_clusters<32>(splits) : (mp == 64 ? max_clusters<64>(splits) : max_clusters<128>(splits));
    // The occupancy query reports the same counts for the two-per-SM instantiations as for the one-per-SM one (74 /
    // 45 / 33 / 26 / 22 / 15 / 15 clusters of 2 ... 8 on a B200), but two of their CTAs do share an SM: 40 clusters of
    // 6 (240 CTAs) run as one wave - 15.1 us on N = 5120, K = 12288 against 18.0 us for 40 clusters of 3 - while 40
    // clusters of 7 do not.  Residency only decides speed (clusters are independent), so the count is doubled.
    if (bsm_two_per_sm(mp)) n *= 2;
    c = n > 0 ? n : -1;
  }
  return c > 0 ? c : 0;
}

template <int MP>
cudaError_t launch_bsm_grouped(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int units,
                               cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tg_fp8_gemm_blockscaled_smallm_kernel<MP, false, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, BsmCfg<MP, bsm_two_per_sm(MP)>::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(units), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = BsmCfg<MP, bsm_two_per_sm(MP)>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (p.flags & 2) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, tg_fp8_gemm_blockscaled_smallm_kernel<MP, false, true>, tmW, tmX, p);
}

// Grouped form: p.tiles_n = ceil(N / 128) per group, p.mtile_bound >= the number of mp-row tiles of all groups,
// p.splits == 1, p.num_kb <= the k-blocks one CTA may own; tmW maps the weights as [groups * N, K].  With
// p.m_indptr == nullptr all M rows form one group: the dense problem as many short CTAs, two per SM, for shapes with
// at least as many weight tiles as SMs and a short K, where the cluster split-K form cannot keep all CTAs resident.
cudaError_t launch_gemm_blockscaled_smallm_grouped(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p,
                                                   int mp, cudaStream_t stream) {
  if (p.splits != 1 || p.num_kb > kMaxKbPerCta || p.kb_per_split != p.num_kb) return cudaErrorInvalidValue;
  const int64_t units = static_cast<int64_t>(p.mtile_bound) * p.tiles_n;
  if (units < 1 || units > 0x7fffffff) return cudaErrorInvalidValue;
  if (mp == 32) return launch_bsm_grouped<32>(tmW, tmX, p, static_cast<int>(units), stream);
  if (mp == 64) return launch_bsm_grouped<64>(tmW, tmX, p, static_cast<int>(units), stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_gemm_blockscaled_smallm(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int mp,
                                           cudaStream_t stream) {
  if (p.splits < 1 || p.splits > 8) return cudaErrorInvalidValue;  // portable cluster size
  if (p.kb_per_split > kMaxKbPerCta) return cudaErrorInvalidValue;
  switch (mp) {
    case 32:
      return launch_bsm<32>(tmW, tmX, p, stream);
    case 64:
      return launch_bsm<64>(tmW, tmX, p, stream);
    case 128:
      return launch_bsm<128>(tmW, tmX, p, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace tg

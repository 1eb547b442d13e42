// Block-scaled W8A8 FP8 GEMM for sm_100a, wide-tile version for problems that fill the GPU (no split-K):
//   C[m,n] = sum_kb As[m,kb] * Bs[n/128,kb] * (A[m, kb-block] . B[n, kb-block]) + bias[n] + beta * C[m,n]
// A 128 x 128 tile moves 64 KB through shared memory per 128-deep k-block (32 KB written by TMA, 32 KB read
// by the tensor core) for 256 clocks of math, and the shared-memory pipe (about 110 B/clk/SM) caps the tensor
// pipe near 50 %.  Here the tile is 128 x 256: 96 KB per 512 clocks of math.  Each k-block is accumulated into
// one of two 256-column TMEM buffers and promoted on CUDA cores, acc += (As[m,kb] * Bs[nb,kb]) * partial
// (exact for arbitrary fp32 scales), by eight warps that each own 32 rows x 128 columns: 128 fp32
// accumulators per thread.  That needs more than the 168 registers a 384-thread CTA gets per thread, so the
// producer / MMA warpgroup hands registers to the two promotion warpgroups with setmaxnreg.
// Two-byte outputs leave through per-warp swizzled staging buffers and bulk tensor stores.
// The same kernel runs the grouped (ragged, MoE-style) problem of
// src/tilegym/suites/flashinfer/cutile/gemm/ragged_block_scaled_bmm.py:497-616: rows [m_indptr[g], m_indptr[g+1])
// of A use weight g; only the tile look-up differs (locate_tile).
// Roles: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2-3 idle, warps 4-11 promotion + store.
#include <cuda_fp8.h>

#include <type_traits>

#include "tg_gemm_common.cuh"
#include "tg_quant_common.cuh"

namespace tg {

namespace {

// Debug aid (compile with -DTG_TRACE): CTA 0 stamps %globaltimer at the steps of its first 256 k-blocks into
// the partial-sum area of the workspace, 40 MiB in, as [k-block][8] uint64 (0-2 MMA warp, 3-6 first promotion warp).
#ifdef TG_TRACE
#define TG_BSW_STAMP(i, slot)                                                                      \
  do {                                                                                             \
    if (blockIdx.x == 0 && (i) < 256 && p.ws_partial != nullptr)                                   \
      (reinterpret_cast<unsigned long long*>(p.ws_partial) + (5u << 20))[(i) * 8 + (slot)] = globaltimer_ns();   \
  } while (0)
#else
#define TG_BSW_STAMP(i, slot) \
  do {                        \
  } while (0)
#endif

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
constexpr int kOutBufBytes = 32 * 128;  // per promotion warp: 32 rows x 64 two-byte columns, 128-byte swizzle
constexpr int kOutStageBytes = kEpiWarps * kOutBufBytes;
constexpr int kAmaxBytes = kEpiWarps * 32 * 4;  // one float per promotion thread (SiLU * mul epilogue)
constexpr int kSmemBytes = kStages * kStageBytes + kOutStageBytes + kAmaxBytes + kCtrlBytes + 1024;
static_assert((2 * kStages + 2 * kAccBufs + 16) * 8 + 12 <= kCtrlBytes, "control block");
static_assert(kSmemBytes <= 227 * 1024, "shared memory per CTA");

// 384 threads x 168 registers fill the register file; 128 threads give up 128 each, 256 threads take 64 each.
constexpr int kRegsLight = 40;
constexpr int kRegsHeavy = 224;
constexpr int kRegsHeavyGrouped = 232;
static_assert(128 * (168 - kRegsLight) >= 256 * (kRegsHeavyGrouped - 168) && kRegsHeavyGrouped >= kRegsHeavy,
              "register budget");

// Where a tile sits.  Plain GEMM: 128-row tile tm, 256-column tile tn.  Grouped GEMM: the 128-row tiles of all
// groups are numbered consecutively (group g owns ceil(rows_g / 128) of them; a tile never spans two groups),
// its rows stop at the end of its group, and its weights / weight scales are those of the group.
struct TileRef {
  int row0;     // first row of A, As and C
  int row_end;  // rows >= row_end are not part of the tile's problem (not stored)
  int col0;     // first column of C
  int b_row0;   // first row in the 2-D view of B ([G * N, K] when grouped)
  int bs_row0;  // row of Bs of the tile's first 128 columns
  bool valid;
};

// All 32 lanes of the calling warp must be active (the grouped look-up scans m_indptr with shuffles); the
// result is the same in every lane.
// Number of 128-row tiles of all groups together (all 32 lanes active; same result in every lane).
__device__ __forceinline__ int count_group_mtiles(const GemmParams& p, int lane) {
  int sum = 0;
  for (int g = lane; g < p.num_groups; g += 32) {
    const int beg = min(max(__ldg(p.m_indptr + g), 0), p.M);
    const int end = min(max(__ldg(p.m_indptr + g + 1), 0), p.M);
    sum += end > beg ? (end - beg + 127) >> 7 : 0;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  return min(sum, p.mtile_bound);
}

// `mtiles`: count_group_mtiles() when grouped (tile ids run densely over [0, mtiles * tiles_n)), unused otherwise.
template <bool kGrouped>
__device__ __forceinline__ TileRef locate_tile(int t, int mtiles, const GemmParams& p, int lane) {
  TileRef r;
  if constexpr (!kGrouped) {
    int tm, tn;
    tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
    r.row0 = tm * kBM;
    r.row_end = p.M;
    r.col0 = tn * kBN;
    r.b_row0 = tn * kBN;
    r.bs_row0 = tn * 2;
    r.valid = true;
    return r;
  } else {
    // flags bit 6 clear: m-tiles vary fastest, so the CTAs running together share a few weight panels through L2;
    // set: the column tiles of one m-tile vary fastest, so a small group's rows and weights are used in one window
    const bool n_fastest = (p.flags & 64) != 0;
    const int tn = n_fastest ? t % p.tiles_n : t / mtiles;
    const int j = n_fastest ? t / p.tiles_n : t - tn * mtiles;
    const int nb_per_group = (p.N + 127) >> 7;
    r.valid = false;
    r.row0 = r.row_end = r.b_row0 = r.bs_row0 = 0;
    r.col0 = tn * kBN;
    int before = 0;  // m-tiles of the groups already scanned
    for (int g0 = 0; g0 < p.num_groups; g0 += 32) {
      const int g = g0 + lane;
      // clamped to [0, M]: whatever the offsets hold, no row outside A / C is ever touched
      const int beg = g < p.num_groups ? min(max(__ldg(p.m_indptr + g), 0), p.M) : 0;
      const int end = g < p.num_groups ? min(max(__ldg(p.m_indptr + g + 1), 0), p.M) : 0;
      const int tiles = end > beg ? (end - beg + 127) >> 7 : 0;
      int incl = tiles;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      const int total = __shfl_sync(0xffffffffu, incl, 31);
      if (j < before + total) {
        const int first = before + incl - tiles;  // this lane's group owns m-tiles [first, first + tiles)
        const unsigned owner = __ballot_sync(0xffffffffu, j >= first && j < first + tiles);
        const int src = __ffs(owner) - 1;
        const int mt = j - __shfl_sync(0xffffffffu, first, src);
        const int grp = g0 + src;
        r.row0 = __shfl_sync(0xffffffffu, beg, src) + mt * kBM;
        r.row_end = __shfl_sync(0xffffffffu, end, src);
        r.b_row0 = grp * p.N + tn * kBN;
        r.bs_row0 = grp * nb_per_group + tn * 2;
        r.valid = true;
        return r;
      }
      before += total;
    }
    return r;
  }
}

// kSwiglu (grouped only): the weights' rows alternate 128 gate rows and 128 up rows, so the tile's two column halves
// are gate and up of the same 128 outputs; the epilogue rounds both to the 16-bit type the reference's
// intermediate has, forms silu(gate) * up, rounds again, quantises to e4m3 (scale 1, or amax / 448 over the 128
// outputs a thread holds for its row) and stores e4m3 rows and scales: the first GEMM of a mixture-of-experts
// layer with src/tilegym/ops/moe_interface.py:262-279 in its epilogue.
template <bool kGrouped, bool kSwiglu = false>
__global__ void __launch_bounds__(kThreads, 1)
    tg_fp8_gemm_blockscaled_wide_kernel(const __grid_constant__ CUtensorMap tmA,
                                        const __grid_constant__ CUtensorMap tmB,
                                        const __grid_constant__ CUtensorMap tmC, const GemmParams p, int tma_out) {
  constexpr int S = kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t a_base = base;
  const uint32_t b_base = base + S * kABytes;
  uint8_t* out_stage = smem + S * kStageBytes;  // 1024-byte aligned
  float* xamax = reinterpret_cast<float*>(out_stage + kOutStageBytes);
  uint8_t* ctrl = out_stage + kOutStageBytes + kAmaxBytes;
  const uint32_t bar_full = smem_u32(ctrl);
  const uint32_t bar_empty = bar_full + 8 * S;
  const uint32_t bar_tfull = bar_empty + 8 * S;
  const uint32_t bar_tempty = bar_tfull + 8 * kAccBufs;
  // gate / up exchange of the SiLU * mul epilogue: per promotion warp one barrier "your partner's values are in
  // its buffer" and one "your partner's row maxima are in place (and it has drained your buffer)"
  const uint32_t bar_xdata = bar_tempty + 8 * kAccBufs;
  const uint32_t bar_xamax = bar_xdata + 8 * kEpiWarps;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + (2 * S + 2 * kAccBufs + 16) * 8);
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
    for (int i = 0; i < kEpiWarps; ++i) {
      mbar_init(bar_xdata + 8 * i, 1);
      mbar_init(bar_xamax + 8 * i, 1);
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

  // 128 x 256 tiles; grouped: every warp counts the groups' 128-row tiles itself (warp 0..11 all need it)
  const int mtiles = kGrouped ? count_group_mtiles(p, lane) : 0;
  const int num_tiles = kGrouped ? mtiles * p.tiles_n : p.tiles_m * p.tiles_n;

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
        const TileRef tile = locate_tile<kGrouped>(t, mtiles, p, lane);
        if (!tile.valid) continue;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag))) {
            report_timeout(p.status, kRoleProducer * 1000 + 51);
            ok = false;
            break;
          }
          if (elected) {
            mbar_arrive_expect_tx(bar_full + 8 * s, kStageBytes);
            tma_load_2d(a_base + s * kABytes, &tmA, bar_full + 8 * s, kb * kBK, tile.row0);
            tma_load_2d(b_base + s * kBBytes, &tmB, bar_full + 8 * s, kb * kBK, tile.b_row0);
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
      [[maybe_unused]] int it = 0;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (kGrouped && !locate_tile<kGrouped>(t, mtiles, p, lane).valid) continue;
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          if (!mbar_wait(bar_tempty + 8 * buf, aph ^ 1u, abort_flag)) {
            report_timeout(p.status, kRoleMma * 1000 + 51);
            ok = false;
            break;
          }
          if (elected) TG_BSW_STAMP(it, 0);
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag)) {
            report_timeout(p.status, kRoleMma * 1000 + 52);
            ok = false;
            break;
          }
          if (elected) TG_BSW_STAMP(it, 1);
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
            TG_BSW_STAMP(it, 2);
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
    // (the register allocator fits the grouped variant without spills at 232 and the plain one at 224)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kGrouped ? kRegsHeavyGrouped : kRegsHeavy));
    // ---------------------------------------------------- promotion + store
    const int e = warp - 4;
    const int q = warp & 3;   // TMEM lane quadrant
    const int half = e >> 2;  // which 128 of the tile's 256 columns = which quantisation block
    // rows of As that start 16-byte aligned are read four k-blocks at a time: a warp's 32 rows cost 32
    // L1 transactions per load, and L1 shares its data path with the tensor core's operand reads
    const bool as_vec = ((reinterpret_cast<uintptr_t>(p.As) & 15u) == 0) && ((p.ldas & 3) == 0);
    int buf = 0;
    uint32_t aph = 0;
    bool ok = true;
    [[maybe_unused]] int eit = 0;
    [[maybe_unused]] uint32_t xph = 0;  // phase of the gate / up exchange barriers
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const TileRef tile = locate_tile<kGrouped>(t, mtiles, p, lane);
      if (!tile.valid) continue;
      const int row_in_tile = q * 32 + lane;
      const int64_t row = static_cast<int64_t>(tile.row0) + row_in_tile;
      const int col0 = tile.col0 + half * 128;
      const bool in = row < tile.row_end && col0 < p.N;
      const float* as_row = p.As + (in ? row : 0) * p.ldas;
      const float* bs_row = p.Bs + static_cast<int64_t>(in ? tile.bs_row0 + half : 0) * p.ldbs;
      float2 acc2[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc2[j] = make_float2(0.f, 0.f);
#pragma unroll 1
      for (int kbg = 0; kbg < p.num_kb && ok; kbg += 4) {
        float a_cur[4];
        load_as4(as_row, kbg, p.num_kb, in, as_vec, a_cur);
#pragma unroll 1
        for (int i = 0; i < 4; ++i) {  // not unrolled: four copies of the body spill
          const int kb = kbg + i;
          if (kb >= p.num_kb) break;
          const float sc = in ? a_cur[0] * __ldg(bs_row + kb) : 0.f;  // the Bs load is warp-uniform
          a_cur[0] = a_cur[1];  // rotate instead of indexing: the array stays in registers
          a_cur[1] = a_cur[2];
          a_cur[2] = a_cur[3];
          const float2 sc2 = make_float2(sc, sc);
          bool w = mbar_wait(bar_tfull + 8 * buf, aph, abort_flag);
          w = __all_sync(0xffffffffu, w);
          if (!w) {
            report_timeout(p.status, kRoleEpilogue * 1000 + 51);
            ok = false;
            break;
          }
          tc_fence_after();
          if (threadIdx.x == 128) TG_BSW_STAMP(eit, 3);
          const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                  static_cast<uint32_t>(buf * kBN + half * 128);
          // two 32-column reads in flight while the previous two are multiplied in
          uint32_t ra[32], rb[32];
          tmem_ld_32x32(t_addr, ra);
          tmem_ld_32x32(t_addr + 32, rb);
          tmem_ld_wait();
          if (threadIdx.x == 128) TG_BSW_STAMP(eit, 4);
          fma16x2(acc2, ra, sc2);
          tmem_ld_32x32(t_addr + 64, ra);
          fma16x2(acc2 + 16, rb, sc2);
          tmem_ld_32x32(t_addr + 96, rb);
          tmem_ld_wait();
          if (threadIdx.x == 128) TG_BSW_STAMP(eit, 5);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);  // the buffer is in registers: hand it back
          fma16x2(acc2 + 32, ra, sc2);
          fma16x2(acc2 + 48, rb, sc2);
          if (threadIdx.x == 128) TG_BSW_STAMP(eit, 6);
          ++eit;
          if (++buf == kAccBufs) {
            buf = 0;
            aph ^= 1u;
          }
        }
      }
      if (!ok) break;
      if constexpr (kSwiglu) {
        // The tile's two column halves are gate and up of the same 128 outputs, held by two warps (same rows).
        // Each warp finishes 64 of them: the gate warp (half 0) outputs 0..63, the up warp (half 1) outputs 64..127.
        // It hands the partner the 64 values that one needs (rounded to 16 bits, as the reference's intermediate
        // tensor is) through its own staging buffer, forms silu(gate) * up for its columns, exchanges the row
        // maximum (block quantisation) and stores its half of the row's 128-byte line.  Two bounded mbarriers per
        // warp and tile: "partner's values are in" and "partner's maximum is in, and it has drained my buffer".
        const bool bf = p.out_dtype == TG_BF16;
        uint8_t* my_row = out_stage + e * kOutBufBytes + lane * 128;  // 128-byte rows, 16-byte pieces swizzled
        const uint8_t* peer_row = out_stage + (e ^ 4) * kOutBufBytes + lane * 128;
        float* acc = reinterpret_cast<float*>(acc2);
        // (send0 / keep0 are compile-time so that the accumulators stay in registers)
        auto finish = [&](auto kSend0, auto kKeep0) -> bool {
          constexpr int send0 = decltype(kSend0)::value;  // first column of what the partner needs
          constexpr int keep0 = decltype(kKeep0)::value;  // first column of what this warp finishes
          constexpr bool is_gate = keep0 == 0;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float* v = acc + send0 + g * 8;
          const uint4 o = bf ? make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                          pack_bf16x2(v[6], v[7]))
                             : make_uint4(pack_f16x2(v[0], v[1]), pack_f16x2(v[2], v[3]), pack_f16x2(v[4], v[5]),
                                          pack_f16x2(v[6], v[7]));
          *reinterpret_cast<uint4*>(my_row + ((g ^ (lane & 7)) << 4)) = o;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_xdata + 8 * (e ^ 4));  // release: the rows are in shared memory
        if (!__all_sync(0xffffffffu, mbar_wait(bar_xdata + 8 * e, xph, abort_flag))) {
          report_timeout(p.status, kRoleEpilogue * 1000 + 52);
          return false;
        }
        float amax = 0.f;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint4 u4 = *reinterpret_cast<const uint4*>(peer_row + ((g ^ (lane & 7)) << 4));
          const uint32_t uw[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float* a = acc + keep0 + g * 8 + 2 * j;
            float t0, t1, m0, m1;  // the partner's values and this warp's own, both rounded to 16 bits
            if (bf) {
              t0 = __uint_as_float(uw[j] << 16);
              t1 = __uint_as_float(uw[j] & 0xffff0000u);
              m0 = __bfloat162float(__float2bfloat16_rn(a[0]));
              m1 = __bfloat162float(__float2bfloat16_rn(a[1]));
            } else {
              const float2 tf = __half22float2(*reinterpret_cast<const __half2*>(&uw[j]));
              t0 = tf.x;
              t1 = tf.y;
              m0 = __half2float(__float2half_rn(a[0]));
              m1 = __half2float(__float2half_rn(a[1]));
            }
            const float g0 = is_gate ? m0 : t0, g1 = is_gate ? m1 : t1;
            const float u0 = is_gate ? t0 : m0, u1 = is_gate ? t1 : m1;
            const float y0 = __fdividef(g0, 1.0f + __expf(-g0)) * u0;
            const float y1 = __fdividef(g1, 1.0f + __expf(-g1)) * u1;
            a[0] = bf ? __bfloat162float(__float2bfloat16_rn(y0)) : __half2float(__float2half_rn(y0));
            a[1] = bf ? __bfloat162float(__float2bfloat16_rn(y1)) : __half2float(__float2half_rn(y1));
            amax = fmaxf(amax, fmaxf(fabsf(a[0]), fabsf(a[1])));
          }
        }
        xamax[e * 32 + lane] = amax;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_xamax + 8 * (e ^ 4));  // release: maximum stored, partner's buffer drained
        if (!__all_sync(0xffffffffu, mbar_wait(bar_xamax + 8 * e, xph, abort_flag))) {
          report_timeout(p.status, kRoleEpilogue * 1000 + 53);
          return false;
        }
        xph ^= 1u;
        if (row < tile.row_end) {
          // quantise this warp's 64 outputs of the row and store its half of the 128-byte line
          float scale = 1.0f;
          if (p.quant_mode == 1) {
            amax = fmaxf(amax, xamax[(e ^ 4) * 32 + lane]);
            scale = __fdiv_rn(amax, 448.0f);
            if (scale == 0.f) scale = 1.0f;
          }
          // the outputs are 16-bit values and the scale is RN(16-bit amax / 448): the test-free quotient applies
          const bool fast = p.quant_mode == 1 && q8_scale_is_tame(scale);
          const float rcp = __frcp_rn(scale);
          const int out_col = (tile.col0 >> 1) + keep0;  // 128 outputs per 256-column tile
          uint8_t* dst = reinterpret_cast<uint8_t*>(p.C) + row * p.ldc + out_col;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float v[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) v[i] = acc[keep0 + g * 16 + j * 4 + i];
              if (fast) {
                const float2 q0 = q8_quot2(make_float2(v[0], v[1]), scale, rcp);
                const float2 q1 = q8_quot2(make_float2(v[2], v[3]), scale, rcp);
                v[0] = q0.x; v[1] = q0.y; v[2] = q1.x; v[3] = q1.y;
              } else if (p.quant_mode == 1) {
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = __fdiv_rn(v[i], scale);
              }
              const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0], v[1]), __NV_SATFINITE, __NV_E4M3);
              const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2], v[3]), __NV_SATFINITE, __NV_E4M3);
              w[j] = lo | (hi << 16);
            }
            *reinterpret_cast<uint4*>(dst + g * 16) = make_uint4(w[0], w[1], w[2], w[3]);
          }
          if (is_gate) p.y_scale[row * (p.N >> 8) + (tile.col0 >> 8)] = scale;
        }
          return true;
        };
        ok = half == 0 ? finish(std::integral_constant<int, 64>{}, std::integral_constant<int, 0>{})
                       : finish(std::integral_constant<int, 0>{}, std::integral_constant<int, 64>{});
        if (!ok) break;
        continue;
      }
      const int row0 = tile.row0 + q * 32;
      if (kGrouped && p.row_scale != nullptr) {  // e.g. the routing weight of a mixture-of-experts row
        const float w = row < tile.row_end ? __ldg(p.row_scale + row) : 0.f;
        const float2 w2 = make_float2(w, w);
#pragma unroll
        for (int j = 0; j < 64; ++j) acc2[j] = __fmul2_rn(acc2[j], w2);
      }
      // bias row of a [groups, N] bias: the tile's weight rows start at b_row0 = group * N + col0 in the [G * N, K] view
      const int64_t bias_off = kGrouped ? static_cast<int64_t>(tile.b_row0 - tile.col0) : 0;
      // a bulk store clips at the ends of C only: in a grouped problem a 32-row slice that runs past the end
      // of its group would overwrite the next group's rows, so such slices take the row-masked stores below
      if (tma_out && (!kGrouped || row0 + 32 <= tile.row_end)) {
        // two-byte outputs with 16-byte aligned rows: 64 columns at a time go through this warp's swizzled
        // staging buffer and leave as one bulk tensor store, which clips rows >= M and columns >= N
        uint8_t* my_stage = out_stage + e * kOutBufBytes;
        uint8_t* dst_row = my_stage + lane * 128;
        add_bias_cols<128>(p, reinterpret_cast<float*>(acc2), col0, bias_off);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint4 o[8];
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float2 v0 = acc2[h * 32 + g * 4], v1 = acc2[h * 32 + g * 4 + 1];
            const float2 v2 = acc2[h * 32 + g * 4 + 2], v3 = acc2[h * 32 + g * 4 + 3];
            if (p.out_dtype == TG_BF16) {
              o[g] = make_uint4(pack_bf16x2(v0.x, v0.y), pack_bf16x2(v1.x, v1.y), pack_bf16x2(v2.x, v2.y),
                                pack_bf16x2(v3.x, v3.y));
            } else {
              o[g] = make_uint4(pack_f16x2(v0.x, v0.y), pack_f16x2(v1.x, v1.y), pack_f16x2(v2.x, v2.y),
                                pack_f16x2(v3.x, v3.y));
            }
          }
          if (lane == 0) tma_store_wait_read<0>();  // the previous store has drained the staging buffer
          __syncwarp();
#pragma unroll
          for (int g = 0; g < 8; ++g) *reinterpret_cast<uint4*>(dst_row + ((g ^ (lane & 7)) << 4)) = o[g];
          fence_proxy_async_smem();
          __syncwarp();
          const int col = col0 + h * 64;
          if (lane == 0 && col < p.N && row0 < p.M) {
            tma_store_2d(&tmC, smem_u32(my_stage), col, row0);
            tma_store_commit();
          }
        }
      } else if (row < tile.row_end) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float acc[32];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            acc[2 * j] = acc2[c * 16 + j].x;
            acc[2 * j + 1] = acc2[c * 16 + j].y;
          }
          epilogue_store32(p, row, col0 + c * 32, acc, 1.0f, c_rows_aligned(p), bias_off);
        }
      }
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

namespace {
template <bool kGrouped>
cudaError_t launch_wide(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap* tmC, const GemmParams& p,
                        int tiles, int num_sms, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tg_fp8_gemm_blockscaled_wide_kernel<kGrouped>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int grid = tiles < num_sms ? tiles : num_sms;
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
  return cudaLaunchKernelEx(&cfg, tg_fp8_gemm_blockscaled_wide_kernel<kGrouped>, tmA, tmB, tmC != nullptr ? *tmC : tmA, p, tmC != nullptr ? 1 : 0);
}
}  // namespace

cudaError_t launch_gemm_blockscaled_wide(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap* tmC,
                                         const GemmParams& p, int num_sms, cudaStream_t stream) {
  return launch_wide<false>(tmA, tmB, tmC, p, p.tiles_m * p.tiles_n, num_sms, stream);
}

cudaError_t launch_gemm_blockscaled_grouped_swiglu(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                                                   int num_sms, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tg_fp8_gemm_blockscaled_wide_kernel<true, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int tiles = p.mtile_bound * p.tiles_n;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles < num_sms ? tiles : num_sms), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (p.flags & 2) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, tg_fp8_gemm_blockscaled_wide_kernel<true, true>, tmA, tmB, tmA, p, 0);
}

// Grouped problem: p.M = total rows, p.m_indptr / num_groups / mtile_bound set, tmB maps B as [G * N, K].
cudaError_t launch_gemm_blockscaled_grouped(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap* tmC,
                                            const GemmParams& p, int num_sms, cudaStream_t stream) {
  return launch_wide<true>(tmA, tmB, tmC, p, p.mtile_bound * p.tiles_n, num_sms, stream);
}

}  // namespace tg

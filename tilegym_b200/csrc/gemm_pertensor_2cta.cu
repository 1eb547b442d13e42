// Per-tensor-scaled FP8 GEMM for sm_100a, CTA-pair version (tcgen05 cta_group::2):
//   C[M,N] = alpha*sa*sb * (A[M,K] . B[N,K]^T) + bias + beta*C
// Two CTAs of a cluster (two SMs) work on one 256 x 256 output tile.  Each CTA
// TMA-loads only its own half of the operands (128 rows of A, 128 rows of B) and
// keeps its own 128 x 256 half of the accumulator in its TMEM; the leader CTA
// issues tcgen05.mma with M = 256, which reads A and B from both CTAs' shared
// memory.  Compared with one CTA per 128 x 256 tile this halves the B bytes
// each SM pulls from L2 per flop (32 KB instead of 48 KB per 128-deep k-block),
// which is what bounds the single-CTA kernel.  No multicast copy is used: each
// CTA fetches exactly the bytes it owns.
// Roles per CTA: warp 0 TMA producer, warp 1 MMA issuer (leader only) and TMEM
// owner, warps 2..5 epilogue.  Two TMEM accumulator buffers overlap the
// epilogue of tile i with the main loop of tile i+1.
#include <cstring>

#include "tg_gemm_common.cuh"
#include "tg_pair.cuh"

namespace tg {

namespace {

constexpr int kThreads = 192;
constexpr int kBN = 256;              // tile width (both CTAs)
constexpr int kBNHalf = 128;          // B rows each CTA loads
constexpr int kStages = 6;
constexpr int kABytes = kBM * kBK;    // 16 KB
constexpr int kBBytes = kBNHalf * kBK;  // 16 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 2 * kBN;    // 512: two accumulator buffers
constexpr int kCtrlBytes = 256;
// Output staging for the TMA-store epilogue: per epilogue warp two buffers of 32 rows x 128 bytes
// (64 two-byte outputs per row, 128-byte swizzled).
constexpr int kOutBufBytes = 32 * 128;
constexpr int kOutStageBytes = 4 * 2 * kOutBufBytes;  // 32 KB
constexpr int kSmemBytes = kStages * kStageBytes + kOutStageBytes + kCtrlBytes + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
static_assert((2 * kStages + 4) * 8 + 12 <= kCtrlBytes, "control block");

// Tensor maps of the output: entry 0 is this GPU's C; further entries are the same slab inside peer GPUs'
// buffers (fused all-gather).  Plain (non-multicast) TMA stores are issued once per destination.
struct OutMaps {
  CUtensorMap m[8];
};

// Work list of one launch.  Units 0 .. full_tiles-1 are whole 256 x 256 tiles; the remaining tiles (those
// that would form a mostly idle last wave) are cut into `tail_div` column slices of 256 / tail_div columns,
// one unit each, so that the last wave spreads over more CTA pairs and finishes in a fraction of a tile time.
struct PairPlan {
  int group_m;
  int full_tiles;
  int tail_div;   // 1, 2 or 4
  int num_units;  // full_tiles + (tiles - full_tiles) * tail_div
};

__device__ __forceinline__ void decode_unit(int u, const GemmParams& p, const PairPlan& plan, int& tm, int& tn,
                                            int& col_off, int& bn) {
  int t = u;
  col_off = 0;
  bn = kBN;
  if (u >= plan.full_tiles) {
    const int v = u - plan.full_tiles;
    t = plan.full_tiles + v / plan.tail_div;
    bn = kBN / plan.tail_div;
    col_off = (v % plan.tail_div) * bn;
  }
  pair_tile_coords(t, p.tiles_m, p.tiles_n, plan.group_m, tm, tn);
}

// kDense16: bf16 / f16 operands (kind::f16) instead of e4m3 (kind::f8f6f4); a compile-time switch, because the
// MMA warp's issue loop is sensitive to any extra control flow.
template <bool kDense16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    tg_fp8_gemm_pertensor_2cta_kernel(const __grid_constant__ CUtensorMap tmA,
                                      const __grid_constant__ CUtensorMap tmB,
                                      const __grid_constant__ CUtensorMap tmBt,
                                      const __grid_constant__ OutMaps omaps, const int num_out,
                                      const GemmParams p, const PairPlan plan) {
  constexpr int S = kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t a_base = base;
  const uint32_t b_base = base + S * kABytes;
  uint8_t* out_stage = smem + S * kStageBytes;
  uint8_t* ctrl = out_stage + kOutStageBytes;
  const uint32_t bar_full = smem_u32(ctrl);      // S barriers; only the leader's are used
  const uint32_t bar_empty = bar_full + 8 * S;   // S barriers, one set per CTA
  const uint32_t bar_tfull = bar_empty + 8 * S;  // 2 barriers, one set per CTA
  const uint32_t bar_tempty = bar_tfull + 16;    // 2 barriers; only the leader's are used
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + (2 * S + 4) * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  griddep_launch_dependents();  // the next kernel's CTAs may take the place of ours as we finish
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = (rank == 0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);   // one arrive.expect_tx by the leader's producer
      mbar_init(bar_empty + 8 * i, 1);  // one commit by the leader's MMA thread
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_tfull + 8 * i, 1);   // one commit by the leader's MMA thread
      mbar_init(bar_tempty + 8 * i, 8);  // four epilogue warps of each CTA
    }
    init_abort_flag(abort_flag, p.wait_limit_us);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: the set-up above may have run while the previous kernel on the stream was
  // finishing; nothing below may touch global memory before that kernel has completed.
  griddep_wait();

  const int num_units = plan.num_units;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    // All 32 lanes walk the loops (warp-uniform control flow, so addresses and descriptors stay in
    // uniform registers); one elected lane issues the TMA copies.
    const bool elected = elect_one();
    {
      if (elected) {
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
      }
      const uint32_t leader_full = map_to_cta(bar_full, 0);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int u = pair_id; u < num_units && ok; u += num_pairs) {
        int tm, tn, col_off, bn;
        decode_unit(u, p, plan, tm, tn, col_off, bn);
        const int a_row = tm * 256 + static_cast<int>(rank) * kBM;
        const int b_row = tn * kBN + col_off + static_cast<int>(rank) * (bn >> 1);
        const CUtensorMap* mapB = (bn == kBN) ? &tmB : &tmBt;  // the slice map boxes bn / 2 rows
        const uint32_t pair_tx = 2u * static_cast<uint32_t>(kABytes + (bn >> 1) * kBK);
        // a k-block is one 128-byte swizzle row: 128 e4m3 or 64 bf16 / f16 elements (flags bits 3, 4)
        constexpr int kb_elems = kDense16 ? kBK / 2 : kBK;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag))) {
            report_timeout(p.status, kRoleProducer * 1000 + 31);
            ok = false;
            break;
          }
          if (elected) {
            if (leader) mbar_arrive_expect_tx(bar_full + 8 * s, pair_tx);  // both CTAs' bytes
            tma_load_2d_pair(a_base + s * kABytes, &tmA, leader_full + 8 * s, kb * kb_elems, a_row);
            tma_load_2d_pair(b_base + s * kBBytes, mapB, leader_full + 8 * s, kb * kb_elems, b_row);
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
    // ---------------------------------------------------------- MMA issuer (leader CTA only)
    // The whole warp walks the loops (warp-uniform control flow: the descriptors stay in uniform registers,
    // which takes the per-instruction issue cost off the critical path); one elected lane issues the MMAs.
    if (leader) {
      const bool elected = elect_one();
      const uint32_t peer_empty = map_to_cta(bar_empty, 1);
      const uint32_t peer_tfull = map_to_cta(bar_tfull, 1);
      int s = 0;
      uint32_t ph = 0;
      int buf = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int u = pair_id; u < num_units && ok; u += num_pairs) {
        const int bn = (u < plan.full_tiles) ? kBN : kBN / plan.tail_div;
        // A / B format fields in bits [7,10) and [10,13): 8-bit operands 0 = e4m3, 1 = e5m2 (flags bit 5);
        // 16-bit operands 0 = f16, 1 = bf16 (flags bit 3)
        const uint32_t fmt16 = (p.flags & (kDense16 ? 8 : 32)) ? kIdescFormat1 : 0u;
        constexpr bool dense16 = kDense16;
        const uint32_t idesc = make_idesc_e4m3_f32(256, bn) | fmt16;
        if (!__all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * buf, aph ^ 1u, abort_flag))) {
          report_timeout(p.status, kRoleMma * 1000 + 31);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * kBN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * s, ph, abort_flag))) {
            report_timeout(p.status, kRoleMma * 1000 + 32);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = make_kmajor_sw128_desc(a_base + s * kABytes);
          const uint64_t bdesc = make_kmajor_sw128_desc(b_base + s * kBBytes);
          if (elected) {
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {  // four 32-byte K steps either way
              if (dense16)
                mma_f16_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
              else
                mma_f8f6f4_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit_pair(bar_empty + 8 * s);   // this CTA's stage is free again ...
            tc_commit_pair(peer_empty + 8 * s);  // ... and so is the peer's
          }
          __syncwarp();
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        if (elected) {
          tc_commit_pair(bar_tfull + 8 * buf);
          tc_commit_pair(peer_tfull + 8 * buf);
        }
        __syncwarp();
        buf ^= 1;
        if (buf == 0) aph ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    float scale = p.alpha;
    if (p.scale_a != nullptr) scale *= __ldg(p.scale_a);
    if (p.scale_b != nullptr) scale *= __ldg(p.scale_b);
    const bool vec_ok = c_rows_aligned(p);
    const uint32_t leader_tempty = map_to_cta(bar_tempty, 0);
    uint8_t* my_stage = out_stage + (warp - 2) * (2 * kOutBufBytes);
    int sb = 0;
    int buf = 0;
    uint32_t aph = 0;
    for (int u = pair_id; u < num_units; u += num_pairs) {
      int tm, tn, col_off, bn;
      decode_unit(u, p, plan, tm, tn, col_off, bn);
      const int chunks = bn >> 5;
      bool w = mbar_wait(bar_tfull + 8 * buf, aph, abort_flag);
      w = __all_sync(0xffffffffu, w);
      if (!w) {
        report_timeout(p.status, kRoleEpilogue * 1000 + 31);
        break;
      }
      tc_fence_after();
      const int64_t row = static_cast<int64_t>(tm) * 256 + static_cast<int>(rank) * kBM + q * 32 + lane;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(buf * kBN);
      if (num_out > 0) {
        // TMA-store epilogue (two-byte outputs, beta == 0): 64 columns at a time go through a swizzled
        // shared-memory buffer and leave as one bulk tensor store per destination; rows and columns past
        // M / N are clipped by the tensor map.
        const int row0 = tm * 256 + static_cast<int>(rank) * kBM + q * 32;
        if (p.flags & 4) {
          // SwiGLU epilogue: the weight rows alternate 32 gate rows / 32 up rows, so every 64 accumulator
          // columns are (gate, up) for 32 output columns: out = silu(gate) * up.  Two such chunks fill one
          // 64-column box of the [M, N/2] output.
#pragma unroll 1
          for (int c = 0; c < (bn >> 6); ++c) {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(t_addr + c * 64, r0);
            tmem_ld_32x32(t_addr + c * 64 + 32, r1);
            tmem_ld_wait();
            if (c == (bn >> 6) - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(leader_tempty + 8 * buf);
            }
            if ((c & 1) == 0) {
              if (lane == 0) tma_store_wait_read<1>();  // the store that last read this buffer has drained it
              __syncwarp();
            }
            const int in_col = tn * kBN + col_off + c * 64;  // first gate column of this chunk
            uint8_t* dst_row = my_stage + sb * kOutBufBytes + lane * 128;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float gate = __uint_as_float(r0[8 * g + j]) * scale;
                float up = __uint_as_float(r1[8 * g + j]) * scale;
                if (p.bias != nullptr) {
                  if (in_col + 8 * g + j < p.N) gate += load_bias(p.bias, p.bias_dtype, in_col + 8 * g + j);
                  if (in_col + 32 + 8 * g + j < p.N) up += load_bias(p.bias, p.bias_dtype, in_col + 32 + 8 * g + j);
                }
                v[j] = __fdividef(gate, 1.0f + __expf(-gate)) * up;
              }
              uint4 o;
              if (p.out_dtype == TG_BF16) {
                o.x = pack_bf16x2(v[0], v[1]);
                o.y = pack_bf16x2(v[2], v[3]);
                o.z = pack_bf16x2(v[4], v[5]);
                o.w = pack_bf16x2(v[6], v[7]);
              } else {
                o.x = pack_f16x2(v[0], v[1]);
                o.y = pack_f16x2(v[2], v[3]);
                o.z = pack_f16x2(v[4], v[5]);
                o.w = pack_f16x2(v[6], v[7]);
              }
              const int chunk16 = (c & 1) * 4 + g;  // 16-byte chunk of the 128-byte staging row
              *reinterpret_cast<uint4*>(dst_row + ((chunk16 ^ (lane & 7)) << 4)) = o;  // 128-byte swizzle
            }
            if (c & 1) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                const uint32_t src = smem_u32(my_stage + sb * kOutBufBytes);
                const int out_col = (tn * kBN + col_off + (c - 1) * 64) >> 1;
                for (int d = 0; d < num_out; ++d) tma_store_2d(&omaps.m[d], src, out_col, row0);
                tma_store_commit();
              }
              sb ^= 1;
            }
          }
          buf ^= 1;
          if (buf == 0) aph ^= 1u;
          continue;
        }
#pragma unroll 1
        for (int c = 0; c < (bn >> 6); ++c) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_addr + c * 64, r0);
          tmem_ld_32x32(t_addr + c * 64 + 32, r1);
          tmem_ld_wait();
          if (c == (bn >> 6) - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_tempty + 8 * buf);
          }
          if (lane == 0) tma_store_wait_read<1>();  // the store that last read this buffer has drained it
          __syncwarp();
          const int col = tn * kBN + col_off + c * 64;
          uint8_t* dst_row = my_stage + sb * kOutBufBytes + lane * 128;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              v[j] = __uint_as_float(g < 4 ? r0[8 * g + j] : r1[8 * (g - 4) + j]) * scale;
            if (p.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (col + 8 * g + j < p.N) v[j] += load_bias(p.bias, p.bias_dtype, col + 8 * g + j);
            }
            uint4 o;
            if (p.out_dtype == TG_BF16) {
              o.x = pack_bf16x2(v[0], v[1]);
              o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]);
              o.w = pack_bf16x2(v[6], v[7]);
            } else {
              o.x = pack_f16x2(v[0], v[1]);
              o.y = pack_f16x2(v[2], v[3]);
              o.z = pack_f16x2(v[4], v[5]);
              o.w = pack_f16x2(v[6], v[7]);
            }
            *reinterpret_cast<uint4*>(dst_row + ((g ^ (lane & 7)) << 4)) = o;  // 128-byte swizzle
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const uint32_t src = smem_u32(my_stage + sb * kOutBufBytes);
            for (int d = 0; d < num_out; ++d) tma_store_2d(&omaps.m[d], src, col, row0);
            tma_store_commit();
          }
          sb ^= 1;
        }
        buf ^= 1;
        if (buf == 0) aph ^= 1u;
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < chunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        if (c == chunks - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(leader_tempty + 8 * buf);
        }
        if (row < p.M)
          epilogue_store32(p, row, tn * kBN + col_off + c * 32, reinterpret_cast<const float*>(r), scale, vec_ok);
      }
      buf ^= 1;
      if (buf == 0) aph ^= 1u;
    }
    if (num_out > 0 && lane == 0) tma_store_wait_all<0>();  // all bulk stores of this warp have completed
  }

  // ---------------------------------------------------------------- teardown
  // Neither CTA may leave while the other can still read its shared memory
  // (pair MMAs) or signal its barriers, so both meet at a cluster barrier first.
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

// How many column slices the tiles of the last, partly filled wave are cut into (1 = not at all).
int pertensor_2cta_tail_div(int tiles, int num_sms) {
  const int pairs = num_sms / 2;
  if (pairs < 1) return 1;
  const int rem = tiles % pairs;
  if (rem == 0) return 1;
  if (rem * 4 <= pairs) return 4;
  if (rem * 2 <= pairs) return 2;
  return 1;
}

cudaError_t launch_gemm_pertensor_2cta(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmBt,
                                       const CUtensorMap* out_maps, int num_out, const GemmParams& p, int group_m,
                                       int tail_div, int num_sms, cudaStream_t stream) {
  if (num_out < 0 || num_out > 8) return cudaErrorInvalidValue;
  OutMaps omaps;
  memset(&omaps, 0, sizeof(omaps));
  for (int i = 0; i < num_out; ++i) omaps.m[i] = out_maps[i];
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tg_fp8_gemm_pertensor_2cta_kernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tg_fp8_gemm_pertensor_2cta_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  int pairs = num_sms / 2;
  PairPlan plan;
  plan.group_m = group_m;
  plan.tail_div = (tail_div == 2 || tail_div == 4) ? tail_div : 1;
  plan.full_tiles = (plan.tail_div == 1) ? tiles : tiles - tiles % pairs;
  plan.num_units = plan.full_tiles + (tiles - plan.full_tiles) * plan.tail_div;
  if (plan.num_units < pairs) pairs = plan.num_units;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);  // the pair is the kernel's compile-time cluster
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (p.flags & 2) ? 1 : 0;
  if (p.flags & 24)  // bf16 / f16 operands
    return cudaLaunchKernelEx(&cfg, tg_fp8_gemm_pertensor_2cta_kernel<true>, tmA, tmB, tmBt, omaps, num_out, p, plan);
  return cudaLaunchKernelEx(&cfg, tg_fp8_gemm_pertensor_2cta_kernel<false>, tmA, tmB, tmBt, omaps, num_out, p, plan);
}

}  // namespace tg

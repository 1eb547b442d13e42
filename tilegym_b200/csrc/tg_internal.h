// Internal declarations shared by the kernel translation units and the C ABI.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tilegym_b200.h"

namespace tg {

// Codes written to the device status word by a wait that gave up
// (status = role * 1000 + site), reported through tg_device_status().
enum WaitRole : int { kRoleProducer = 1, kRoleMma = 2, kRoleEpilogue = 3 };

struct GemmParams {
  // problem
  int32_t M, N, K;
  int32_t num_kb;            // ceil(K / 128)
  int32_t tiles_m, tiles_n;  // output tiles
  int32_t tile_rows;         // small-M kernel: weight rows per tile (<= 128)
  // output
  void* C;
  int64_t ldc;        // elements
  int32_t out_dtype;  // TG_F32 / TG_F16 / TG_BF16
  // per-tensor epilogue
  const float* scale_a;  // device scalar or nullptr
  const float* scale_b;
  float alpha, beta;
  const void* bias;  // nullptr, f32 or bf16 [N]
  int32_t bias_dtype;
  // block-scaled epilogue
  const float* As;  // [M, ldas]
  const float* Bs;  // [ceil(N/128), ldbs]
  int64_t ldas, ldbs;
  // split-K (small-M and thin problems)
  int32_t splits;         // K splits (1 = none)
  int32_t kb_per_split;   // k-blocks per split
  float* ws_partial;      // [splits, tiles..., 128*BN] fp32 partial tiles
  uint32_t* ws_counters;  // one per output tile, zero on entry and on exit
  // grouped (ragged) block-scaled GEMM: rows [m_indptr[g], m_indptr[g+1]) of A / C use weight g of B [G, N, K]
  const int32_t* m_indptr;  // device, num_groups + 1 entries
  int32_t num_groups;
  int32_t mtile_bound;  // ceil(M / 128) + num_groups >= the number of 128-row tiles of all groups
  const float* row_scale;  // grouped GEMM: nullptr, or one factor per row of C applied before bias and rounding
  // grouped GEMM with the SiLU * mul + quantise epilogue (first GEMM of a mixture-of-experts layer): C is the e4m3
  // output [M, N / 2] (ldc in bytes = elements), out_dtype the 16-bit type the reference rounds to on the way,
  // y_scale its [M, N / 256] scales, quant_mode 0 (scale 1) or 1 (amax / 448 per 128 outputs)
  float* y_scale;
  int32_t quant_mode;
  // diagnostics
  int32_t* status;         // device status word
  uint32_t wait_limit_us;  // bound of every device-side wait in microseconds (0 = the 2 s default)
  // bit 0 (small-M kernel): the weight operand is not written by the kernel that precedes this one on the
  // stream, so its TMA loads may be issued before the programmatic-dependent-launch wait;
  // bit 1: launched with programmatic stream serialization; bit 2: SwiGLU epilogue; bits 3 / 4: bf16 / f16
  // operands (dense kernel); bit 5: e5m2 instead of e4m3 operands (per-tensor kernels); bit 6: grouped kernel,
  // column tiles vary fastest in the tile order
  int32_t flags;
};

// Launchers (each sets its kernel's shared-memory attribute once per device).
cudaError_t launch_gemm_pertensor(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int bn,
                                  int num_sms, cudaStream_t stream);
// CTA-pair (cta_group::2) kernel: 256 x 256 tiles; tmA and tmB both box 128 rows; p.tiles_* count 256-wide tiles.
// The tiles of the last, partly filled wave are cut into `tail_div` column slices (1, 2 or 4, from
// pertensor_2cta_tail_div); tmBt boxes 128 / tail_div rows of B for them.
int pertensor_2cta_tail_div(int tiles, int num_sms);
// out_maps[0 .. num_out): tensor maps (two-byte elements, box 64 x 32, 128-byte swizzle) of the output slab
// in this GPU's buffer and, for the fused all-gather, in the peers' buffers; num_out == 0 selects the
// register -> global store epilogue (needed for fp32 output, beta != 0 or unaligned rows).
cudaError_t launch_gemm_pertensor_2cta(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmBt,
                                       const CUtensorMap* out_maps, int num_out, const GemmParams& p, int group_m,
                                       int tail_div, int num_sms, cudaStream_t stream);
// tmC as for the wide-tile kernel below (nullptr: register -> global stores).
cudaError_t launch_gemm_blockscaled(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap* tmC,
                                    const GemmParams& p, int num_sms, cudaStream_t stream);
// Wide-tile block-scaled kernel: 128 x 256 tiles (tmB boxes 256 rows, p.tiles_n counts 256-wide tiles), no split-K.
// tmC: tensor map of the output (two-byte elements, box 64 x 32, 128-byte swizzle) for the bulk-store epilogue,
// or nullptr for register -> global stores (fp32 output, unaligned rows).
cudaError_t launch_gemm_blockscaled_wide(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap* tmC,
                                         const GemmParams& p, int num_sms, cudaStream_t stream);
// Grouped (ragged) problem on the same kernel: p.M = total rows, p.m_indptr / num_groups / mtile_bound set,
// tmB maps B [G, N, K] as [G * N, K] with 256-row boxes.
cudaError_t launch_gemm_blockscaled_grouped(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap* tmC,
                                            const GemmParams& p, int num_sms, cudaStream_t stream);
// The same with the SiLU * mul + quantise epilogue: the weights' rows alternate 128 gate rows and 128 up rows, so
// every 128 x 256 tile holds gate and up of 128 outputs; p.C / p.y_scale / p.quant_mode describe the e4m3 output.
cudaError_t launch_gemm_blockscaled_grouped_swiglu(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                                                   int num_sms, cudaStream_t stream);
// Swap-AB block-scaled kernel for M <= 128: tmW boxes 128 weight rows, tmX boxes `mp` (32 / 64 / 128) activation
// rows; p.tiles_n counts 128-row weight tiles, the p.splits (1..8) K splits of a tile form a cluster, and every
// split owns at most blockscaled_smallm_max_kb_per_cta() k-blocks.  No beta.
int blockscaled_smallm_max_kb_per_cta();
// clusters of `splits` CTAs of that kernel the current device holds at once (num_sms for splits == 1)
int blockscaled_smallm_resident_clusters(int mp, int splits, int num_sms);
cudaError_t launch_gemm_blockscaled_smallm(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int mp,
                                           cudaStream_t stream);
// Grouped (mixture-of-experts, few rows per group) form of the same kernel; mp 32 or 64.
cudaError_t launch_gemm_blockscaled_smallm_grouped(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p,
                                                   int mp, cudaStream_t stream);
// Swap-AB split-K kernel for M <= 64: tmW boxes 128 weight rows, tmX boxes `mp` activation rows.
cudaError_t launch_gemm_smallm(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int mp,
                               cudaStream_t stream);

// Same kernel with the K splits of a tile launched as one thread-block cluster (1 <= splits <= 8) and the
// partial sums reduced through distributed shared memory: needs no workspace.
cudaError_t launch_gemm_smallm_cluster(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int mp,
                                       cudaStream_t stream);

// Helpers of the main entry-point file, for entry points defined elsewhere.
int32_t api_fail(int32_t rc, const char* msg);
int32_t api_check_operand(const TgTensorDesc* t, const char* name);
int32_t api_check_output(const TgTensorDesc* C, int64_t M, int64_t N);
int32_t api_make_map(CUtensorMap* map, uint64_t ptr, int64_t rows, int64_t K, int64_t pitch, int box_rows);
int32_t api_init_device(int dev, int* num_sms, int32_t** status);  // call with `dev` current
uint32_t api_wait_limit_us();  // tg_set_wait_limit_us() value (0 = default), for GemmParams::wait_limit_us

cudaError_t launch_act_quant(void* y, float* s, const void* x, int x_dtype, int64_t n_blocks, cudaStream_t stream);
cudaError_t launch_weight_dequant(void* y, int y_dtype, const uint8_t* x, const float* s, int64_t M, int64_t N,
                                  int64_t lds, cudaStream_t stream);
cudaError_t launch_quant_pertensor(uint8_t* y, float* scale_out, const void* x, int x_dtype, int64_t numel,
                                   uint32_t* amax_scratch, int num_sms, bool allow_single_launch, cudaStream_t stream);
cudaError_t launch_weight_quant_block(uint8_t* y, float* s, const void* x, int x_dtype, int64_t N, int64_t K,
                                      int64_t lds, cudaStream_t stream);

}  // namespace tg

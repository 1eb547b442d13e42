/*
 * tilegym_b200 - C ABI of the B200 (sm_100a) FP8 scaled-GEMM library.
 *
 * Conventions (they mirror the FFI TileGym already uses for its compiled
 * cuTile-rs kernels, src/tilegym/ops/cutile_rs/ffi_util.rs:26-35,102-122 and
 * src/tilegym/ops/cutile_rs/matmul_kernel/ffi.rs:29-53):
 *   - one extern "C" symbol per operator, returning an int32 status code;
 *   - tensors cross the boundary as `const TgTensorDesc*` (device pointer,
 *     rank, shape, strides in ELEMENTS, dtype code); the callee borrows the
 *     memory and never frees it; the caller keeps descriptors alive for the
 *     duration of the call only;
 *   - the last two arguments are the CUDA device ordinal and the raw
 *     cudaStream_t as an integer; every call enqueues work on that stream and
 *     returns without synchronising;
 *   - no locks are taken on the call path: call from the thread that drives
 *     the stream.  Per-device state is created on the first call on a device.
 *
 * Status codes: 0 ok, -2 unsupported dtype, -3 launch failed, -4 device
 * initialisation failed, -5 null pointer, -6 invalid arguments, -7 a bounded
 * device-side wait expired, -8 a pointer or row pitch is not 16-byte aligned.
 * (-1 is reserved, as in the reference FFI, for "auto".)
 */
#ifndef TILEGYM_B200_H_
#define TILEGYM_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define TG_API __attribute__((visibility("default")))
#else
#define TG_API
#endif

#define TG_OK 0
#define TG_ERR_DTYPE (-2)
#define TG_ERR_LAUNCH (-3)
#define TG_ERR_DEVICE (-4)
#define TG_ERR_NULL (-5)
#define TG_ERR_ARGS (-6)
#define TG_ERR_TIMEOUT (-7)
#define TG_ERR_ALIGN (-8)

/* dtype codes of src/tilegym/ops/cutile_rs/ffi_util.rs:26-35 */
#define TG_F32 0
#define TG_F16 1
#define TG_BF16 2
#define TG_I32 3
#define TG_I64 4
#define TG_F8E5M2 5
#define TG_U8 6
#define TG_F8E4M3 7
#define TG_I8 8 /* not in the reference table (its cuTile-rs FFI has no int8 operator); used by the group quantiser */

typedef struct TgTensorDesc {
  uint64_t ptr;       /* device address */
  int32_t ndim;       /* 1..5 */
  int64_t shape[5];
  int64_t strides[5]; /* in elements */
  int32_t dtype;      /* TG_* code */
} TgTensorDesc;

/* Per-tensor-scaled FP8 GEMM with a fused epilogue:
 *     C[M,N] = alpha * sa * sb * (A[M,K] . B[N,K]^T) + bias[N] + beta * C[M,N]
 * A, B: both e4m3 or both e5m2, row-major, contiguous rows (K % 16 == 0, 16-byte aligned base).
 * C: bf16 / f16 / f32, row-major, written in place (read first only if beta != 0).
 * scale_a, scale_b: device pointers to one fp32 each, or 0 for 1.0.
 * bias: f32 or bf16 vector of N elements, or NULL.
 * workspace: device scratch of at least tg_fp8_gemm_workspace_bytes() bytes;
 *   only the small-M (M <= 64) split-K path uses it; it must be zero before
 *   the first call and is left zero by every call, and may be shared by calls
 *   that are ordered on one stream, not by calls that overlap on the GPU.
 * Replaces tilegym.suites.flashinfer.ops.gemm_alpha_beta for e4m3 inputs
 * (src/tilegym/suites/flashinfer/ops.py:25-55, kernel
 * src/tilegym/suites/flashinfer/cutile/gemm/gemm_alpha_beta.py:19-180) and
 * the matmul a Linear patch calls (src/tilegym/ops/ops.py:715-741).
 */
TG_API int32_t tg_fp8_gemm_pertensor(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B,
                              uint64_t scale_a, uint64_t scale_b, float alpha, const TgTensorDesc* bias,
                              float beta, uint64_t workspace, uint64_t workspace_bytes, uint32_t flags,
                              int32_t device_id, uint64_t stream);

/* flags of tg_fp8_gemm_pertensor.
 * TG_GEMM_STATIC_B: B (the weights) is not written by the kernel that precedes this call on the stream - true
 * for the parameters of a Linear layer.  Small-M (M <= 64) launches then start streaming B while that kernel's
 * last thread blocks are still finishing (programmatic dependent launch); A, the scales, the bias and C are
 * still touched only after it has completed.  Worth 0.7-1.7 us on a 5-20 us decode GEMM. */
#define TG_GEMM_STATIC_B 1u

/* Block-scaled W8A8 GEMM (1 x block_k activation scales, block_n x block_k
 * weight scales; only 128 x 128 is implemented, anything else is -6):
 *     C[m,n] = sum_kb  As[m,kb] * Bs[n/128,kb] * (A[m,kb-block] . B[n,kb-block]) + bias[n] + beta * C[m,n]
 * A: (M,K) e4m3; B: (N,K) e4m3; As: (M, ceil(K/128)) f32; Bs: (ceil(N/128),
 * ceil(K/128)) f32; C: (M,N) f32 / f16 / bf16, written in place (read first only
 * if beta != 0).  bias: f32 / f16 / bf16 vector of N elements, or NULL; it is added
 * in fp32 before the one rounding to C's dtype.  Rows past M, N and columns
 * past K read as zero.  workspace as above (used when K is split).
 * Replaces tilegym.suites.unsloth.ops.w8a8_block_fp8_matmul
 * (src/tilegym/suites/unsloth/ops.py:240-265; host wrapper and kernel
 * src/tilegym/suites/unsloth/cutile/fp8.py:388-446 and :243-334), which has
 * neither bias nor beta (pass NULL and 0).
 */
TG_API int32_t tg_fp8_gemm_blockscaled(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B,
                                const TgTensorDesc* As, const TgTensorDesc* Bs, int32_t block_n,
                                int32_t block_k, const TgTensorDesc* bias, float beta, uint64_t workspace,
                                uint64_t workspace_bytes, int32_t device_id, uint64_t stream);

/* Per-tensor-scaled FP8 GEMM of a fused gate/up projection with the SwiGLU activation in its epilogue:
 *     C[m, j] = silu(g) * u,   g = alpha*sa*sb*(A . B[row_g(j)]^T) + bias[row_g(j)],  u likewise with row_u(j)
 * B: (N, K) e4m3, N = 2 * I a multiple of 128, whose rows alternate 32 gate rows and 32 up rows:
 * row_g(j) = 64 * (j / 32) + j % 32, row_u(j) = row_g(j) + 32 (bias, if given, in the same order).
 * C: (M, I) bf16 / f16 with 16-byte aligned rows.  The [M, 2I] intermediate never reaches memory.
 * The reference computes this as two steps, matmul then silu_and_mul
 * (src/tilegym/ops/fused_mlp.py:85-107, PartiallyFusedSwiGLUMLP.forward); it has no fused counterpart.
 */
TG_API int32_t tg_fp8_gemm_pertensor_swiglu(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B,
                                            uint64_t scale_a, uint64_t scale_b, float alpha,
                                            const TgTensorDesc* bias, int32_t device_id, uint64_t stream);

/* Dense bf16 / f16 GEMM (no quantisation), fp32 accumulation on the same CTA-pair tcgen05 kernel (kind::f16):
 *     C[M,N] = alpha * (A[M,K] . B[N,K]^T) + bias[N] + beta * C[M,N]
 * A, B: both bf16 or both f16, row-major, contiguous rows, 16-byte aligned base and row pitch (K % 8 == 0);
 * C: bf16 / f16 / f32.  The unquantised path of tilegym.ops.matmul (src/tilegym/ops/ops.py:715-741,
 * src/tilegym/ops/cutile/matmul.py:421-455) with B given K-major ([N, K], i.e. trans_b).
 */
TG_API int32_t tg_gemm_dense16(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B, float alpha,
                               const TgTensorDesc* bias, float beta, int32_t device_id, uint64_t stream);

/* Grouped (ragged, MoE-style) block-scaled GEMM: rows [m_indptr[g], m_indptr[g+1]) of A and C belong to group g
 * and use weight B[g]:
 *     C[m,n] = sum_kb  As[m,kb] * Bs[g, n/128, kb] * (A[m,kb-block] . B[g, n, kb-block])      for m in group g
 * A: (M,K) e4m3, all groups' rows stacked; B: (G,N,K) e4m3 contiguous; As: (M, ceil(K/128)) f32;
 * Bs: (G, ceil(N/128), ceil(K/128)) f32 contiguous; C: (M,N) f32 / f16 / bf16.
 * m_indptr: DEVICE pointer to G+1 int32 offsets, non-decreasing, never read on the host (so the call can be
 * captured in a CUDA graph whose routing changes between replays); groups may be empty and need no alignment;
 * rows outside every group are left untouched; offsets are clamped to [0, M] on the device.
 * bias: NULL or a contiguous (G, N) f32 / f16 / bf16 matrix, row g added to the rows of group g; beta as above.
 * row_scale: 0, or a DEVICE pointer to M fp32 factors: row m of the product is multiplied by row_scale[m] in
 * fp32 before bias, beta * C and the rounding (the routing weight of a mixture-of-experts row,
 * src/tilegym/ops/tilecpp/moe.cuh:193-200).
 * Replaces tilegym.suites.flashinfer.ops.ragged_block_scaled_bmm for e4m3 inputs in the NT layout
 * (src/tilegym/suites/flashinfer/ops.py:126-158, kernel
 * src/tilegym/suites/flashinfer/cutile/gemm/ragged_block_scaled_bmm.py:497-616).
 */
TG_API int32_t tg_fp8_gemm_blockscaled_grouped(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B,
                                               const TgTensorDesc* As, const TgTensorDesc* Bs, uint64_t m_indptr,
                                               int32_t block_n, int32_t block_k, const TgTensorDesc* bias,
                                               float beta, uint64_t row_scale, int32_t device_id, uint64_t stream);

/* ---- Mixture-of-experts layer around the grouped GEMM (reference: fused_experts_impl,
 * src/tilegym/ops/moe_interface.py:116-322; kernels src/tilegym/ops/tilecpp/moe.cuh:72-563).  The reference pads
 * each expert's token list to the tile height and gathers rows inside every GEMM tile through sorted_token_ids
 * (moe_align_block_size, moe_interface.py:30-81); here rows are brought into expert order once, both expert
 * GEMMs run on contiguous segments through tg_fp8_gemm_blockscaled_grouped, and the way back to token order is
 * part of the final sum over the top-k experts.  Nothing is read back to the host. ---- */

/* Routing: counting sort of the (token, slot) pairs by expert.  topk_ids: (T, top_k) int32 / int64, contiguous;
 * topk_weights: same shape, f32 / f16 / bf16, or NULL.  Outputs (device pointers): m_indptr[E + 1] int32 segment
 * offsets in expert order; sorted_ids[T * top_k] int32, flat pair index t * top_k + slot of every sorted row;
 * pos[T * top_k] int32, its inverse (-1 for a pair whose expert id is outside [0, E)); w_sorted[T * top_k] f32,
 * the routing weight of every sorted row (may be 0 when topk_weights is NULL); scratch: E int32.  The order of
 * the rows inside an expert's segment is not specified (rows are computed independently of their position). */
TG_API int32_t tg_moe_route(const TgTensorDesc* topk_ids, const TgTensorDesc* topk_weights, int32_t num_experts,
                            uint64_t m_indptr, uint64_t sorted_ids, uint64_t pos, uint64_t w_sorted, uint64_t scratch,
                            int32_t device_id, uint64_t stream);

/* Row gather into expert order: A_sorted[r] = A[sorted_ids[r] / top_k], As_sorted likewise, for the
 * m_indptr[E] routed rows.  A: (T, K) e4m3, As: (T, ceil(K/128)) f32; A_sorted: (R, K), As_sorted: (R, ceil(K/128)),
 * R <= T * top_k, contiguous.  (The reference gathers per GEMM tile: ct::load_masked through offs_token / TOP_K,
 * moe.cuh:150-165.) */
TG_API int32_t tg_moe_permute_rows(const TgTensorDesc* A_sorted, const TgTensorDesc* As_sorted, const TgTensorDesc* A,
                                   const TgTensorDesc* As, uint64_t sorted_ids, uint64_t m_indptr, int32_t num_experts,
                                   int32_t topk, int32_t device_id, uint64_t stream);

/* The first expert GEMM with the step after it in its epilogue: grouped block-scaled GEMM as above whose weights'
 * rows alternate 128 gate rows and 128 up rows (B: (G, 2 I, K), Bs rows likewise; arrange once at load time), so
 * that every 128 x 256 tile holds gate and up of 128 outputs.  Per row: both rounded to round_dtype (bf16 / f16, the
 * type of the reference's intermediate), silu(gate) * up, rounded again, then e4m3 with quant_mode 0 (scale 1) or 1
 * (amax / 448 over each 128 outputs).  Y: (M, I) e4m3; Ys: (M, I / 128) f32.  The [M, 2 I] intermediate never
 * reaches memory.  Replaces invoke_fused_moe_kernel + silu_and_mul + the cast of
 * src/tilegym/ops/moe_interface.py:247-279 (kernel src/tilegym/ops/tilecpp/moe.cuh:249-405). */
TG_API int32_t tg_fp8_gemm_blockscaled_grouped_swiglu(const TgTensorDesc* Y, const TgTensorDesc* Ys, const TgTensorDesc* A,
                                                      const TgTensorDesc* B, const TgTensorDesc* As, const TgTensorDesc* Bs,
                                                      uint64_t m_indptr, int32_t round_dtype, int32_t quant_mode,
                                                      int32_t device_id, uint64_t stream);

/* tg_act_quant and tg_moe_permute_rows in one pass, for 16-bit activations: every row of X (T, H) bf16 / f16 is
 * quantised per 1 x 128 block (amax / 448, 1.0 for an all-zero block; the bytes and scales tg_act_quant produces) and
 * written, with its scales, to each of its top_k rows pos[t * top_k + j] of A_sorted (R, H) e4m3 / As_sorted
 * (R, H / 128) f32 (entries of -1 are skipped).  pos as tg_moe_route produces it.  No reference counterpart (the
 * reference gathers rows inside its GEMM tiles). */
TG_API int32_t tg_moe_quant_permute_rows(const TgTensorDesc* A_sorted, const TgTensorDesc* As_sorted, const TgTensorDesc* X,
                                         uint64_t pos, int32_t topk, int32_t device_id, uint64_t stream);

/* Between the two expert GEMMs: a = silu(X[:, :I]) * X[:, I:] in fp32, rounded to X's 16-bit type (the reference's
 * intermediate tensor, moe_interface.py:262-267), then quantised to e4m3 for the second GEMM.  mode 0: scale 1 and
 * a saturating cast, the reference's a2_scale of ones (moe_interface.py:269-279); mode 1: one scale amax / 448 per
 * 128 elements (1 for an all-zero group), IEEE division.  Adding 2 to mode says that X's columns are interleaved in
 * blocks of 128 (gate, up, gate, up, ...: what the first GEMM writes when its weight rows were rearranged for the fused
 * epilogue).  X: (R, 2 I) bf16 / f16, I % 128 == 0; Y: (R, I) e4m3; S: (R, I / 128) f32; only the first m_indptr[E]
 * rows are processed. */
TG_API int32_t tg_moe_silu_mul_quant(const TgTensorDesc* Y, const TgTensorDesc* S, const TgTensorDesc* X, uint64_t m_indptr,
                                     int32_t num_experts, int32_t mode, int32_t device_id, uint64_t stream);

/* Back to token order: out[t, :] = sum over slot j of C[pos[t * top_k + j], :] (pairs with pos < 0 skipped), summed
 * in fp32 and rounded once - the reference's torch.sum over the top-k axis (moe_interface.py:309-321) with the
 * un-permutation folded in.  C: (R, H) bf16 / f16 in expert order, out: (T, H), H % 8 == 0. */
TG_API int32_t tg_moe_unpermute_sum(const TgTensorDesc* out, const TgTensorDesc* C, uint64_t pos, int32_t topk,
                                    int32_t device_id, uint64_t stream);

/* Column-parallel GEMM fused with the all-gather of its output (multi-GPU, one
 * process per GPU).  This rank computes its slab C[M, n] = alpha*sa*sb*(A . B_shard^T)
 * + bias and the kernel's epilogue stores every finished tile into C AND into the
 * same slab of each peer GPU's output buffer over NVLink (plain, non-multicast bulk
 * tensor stores to peer-mapped memory), so no separate collective pass runs.
 * C: [M, n] bf16 / f16 view (row stride = full output width) of this rank's slab in
 * its own buffer; peer_ptrs[i]: address of the same [M, n] view inside peer i's
 * buffer (peer-mapped, e.g. CUDA IPC or a symmetric-memory allocation), num_peers
 * <= 7.  Needs M, n >= 256 and 16-byte aligned rows.  The caller orders the ranks
 * (a barrier after the call) before any rank reads the gathered result.
 * The reference is single-GPU; there is no counterpart. */
TG_API int32_t tg_fp8_gemm_pertensor_allgather(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B,
                                               uint64_t scale_a, uint64_t scale_b, float alpha,
                                               const TgTensorDesc* bias, const uint64_t* peer_ptrs,
                                               int32_t num_peers, int32_t device_id, uint64_t stream);

/* Column-parallel GEMM followed by an NCCL all-gather of the output slabs (multi-GPU, one process per GPU): this
 * rank computes its slab C_all[rank] = alpha*sa*sb*(A . B_shard^T) + bias_shard and ncclAllGather fills the other
 * ranks' slabs, in place, on the same stream.  C_all: contiguous (world, M, n) f32 / f16 / bf16; logical element
 * C[m, g*n + j] is C_all[g, m, j].  comm: the caller's ncclComm_t (as an integer); the library resolves
 * ncclAllGather at run time from the NCCL the process has loaded, so it has no link-time dependency on NCCL.
 * workspace as for tg_fp8_gemm_pertensor.  The reference is single-GPU; there is no counterpart.  (The fused
 * entry above overlaps the transfer with the GEMM; this one is the plain library collective.) */
TG_API int32_t tg_shard_gemm_allgather(const TgTensorDesc* C_all, const TgTensorDesc* A, const TgTensorDesc* B_shard,
                                       uint64_t scale_a, uint64_t scale_b, float alpha, const TgTensorDesc* bias_shard,
                                       int32_t rank, int32_t world, uint64_t comm, uint64_t workspace,
                                       uint64_t workspace_bytes, int32_t device_id, uint64_t stream);

/* The small-M (M <= 64) path of tg_fp8_gemm_pertensor for callers that cannot
 * allocate device memory - a server whose pool already owns the GPU, or a
 * decode loop that must never reach cudaMalloc / cudaFree because they
 * synchronise the device.  It has no counterpart in the reference.
 * Same arithmetic and arguments as tg_fp8_gemm_pertensor minus the workspace:
 * the split-K scratch is a fixed 8 MiB + 16 KiB __device__ array inside the
 * library (held on every GPU that loads the library until the process
 * exits).  Limits: M <= 64 and N <= 131072, otherwise -6 with a message.
 * All calls on a device share that array: calls that overlap on the GPU race;
 * calls ordered on one stream are fine (each call clears the counters it
 * uses).  The first call on a device resolves the array's address and
 * configures the kernel; make it before any stream capture.  Calls no
 * cudaMalloc, cudaFree or other allocating routine. */
TG_API int32_t tg_fp8_gemm_pertensor_smallm_static(const TgTensorDesc* C, const TgTensorDesc* A,
                                                   const TgTensorDesc* B, uint64_t scale_a, uint64_t scale_b,
                                                   float alpha, const TgTensorDesc* bias, float beta,
                                                   int32_t device_id, uint64_t stream);

/* Bytes of scratch the two GEMM entry points may need for a problem size. */
TG_API uint64_t tg_fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);

/* 1 x block activation quantiser: s = amax/448 per `block` contiguous
 * elements (1.0 for an all-zero block), y = e4m3(x / s) with IEEE division.
 * X: (..., K) bf16 / f16 / f32 contiguous, K % block == 0; Y same shape e4m3;
 * S: (..., K/block) f32.  Only block == 128 is implemented.
 * Replaces tilegym.suites.unsloth.ops.act_quant (src/tilegym/suites/unsloth/ops.py:223-237,
 * kernel src/tilegym/suites/unsloth/cutile/fp8.py:77-120).
 */
TG_API int32_t tg_act_quant(const TgTensorDesc* Y, const TgTensorDesc* S, const TgTensorDesc* X, int32_t block,
                     int32_t device_id, uint64_t stream);

/* Per-token group quantiser to 8 bits: per `group_size` contiguous elements of a row, amax = max(|x|, eps),
 * s = amax / dtype_max (IEEE division; rounded up to a power of two when scale_ue8m0 != 0),
 * y = clamp(x / s, dtype_min, dtype_max) cast to Y's dtype (e4m3 / e5m2: round to nearest even; int8: truncate).
 * X: (T, H) bf16 / f16 / f32 contiguous, H % group_size == 0, group_size in {8,16,32,64,128,256,512};
 * Y: (T, H) contiguous, dtype TG_F8E4M3, TG_F8E5M2 or TG_I8; S: (T, H/group_size) f32 with ANY strides -
 * row-major, column-major ((1, T)) and the padded column-major layout ((1, ceil4(T))) are all the same call.
 * Replaces tilegym.suites.flashinfer.ops.per_token_group_quant_8bit (src/tilegym/suites/flashinfer/ops.py:238-267,
 * kernels src/tilegym/suites/flashinfer/cutile/per_token_group_quant_8bit.py:25-150).
 */
TG_API int32_t tg_per_token_group_quant(const TgTensorDesc* Y, const TgTensorDesc* S, const TgTensorDesc* X,
                                        int32_t group_size, float eps, int32_t scale_ue8m0, int32_t device_id,
                                        uint64_t stream);

/* block x block weight dequantiser: y[i,j] = x[i,j] * s[i/block, j/block].
 * X: (M,N) e4m3; S: (ceil(M/block), ceil(N/block)) f32; Y: (M,N) bf16/f16/f32.
 * Replaces tilegym.suites.unsloth.ops.weight_dequant (src/tilegym/suites/unsloth/ops.py:199-220,
 * kernel src/tilegym/suites/unsloth/cutile/fp8.py:36-71).
 */
TG_API int32_t tg_weight_dequant(const TgTensorDesc* Y, const TgTensorDesc* X, const TgTensorDesc* S, int32_t block,
                          int32_t device_id, uint64_t stream);

/* Per-tensor quantiser: scale = amax(|x|)/448 (1.0 if all zero), y =
 * e4m3(clamp(x/scale, +-448)).  X: any shape, contiguous, bf16/f16/f32.
 * scale_out: device pointer to one fp32.  amax_scratch: device pointer to one
 * uint32 of scratch (cleared by the call itself with a stream-ordered memset).
 * The reference has no such kernel; it is the quantiser the per-tensor
 * benchmark configurations describe, placed in front of tg_fp8_gemm_pertensor
 * the way act_quant sits in front of the block-scaled GEMM.
 */
TG_API int32_t tg_quant_pertensor(const TgTensorDesc* Y, uint64_t scale_out, const TgTensorDesc* X,
                           uint64_t amax_scratch, int32_t device_id, uint64_t stream);

/* 128 x 128 weight quantiser (producer of Bs): s = amax/448 per block (1.0
 * for an all-zero block), y = e4m3(clamp(x/s, +-448)).  X: (N,K)
 * bf16/f16/f32; Y: (N,K) e4m3; S: (ceil(N/128), ceil(K/128)) f32.
 * Inverse of tg_weight_dequant; the reference has no GPU kernel for it.
 */
TG_API int32_t tg_weight_quant_block(const TgTensorDesc* Y, const TgTensorDesc* S, const TgTensorDesc* X,
                              int32_t block, int32_t device_id, uint64_t stream);

/* Process-wide form of TG_GEMM_STATIC_B, for callers that cannot pass the flag per call: a promise that the B
 * operand (weights) of small-M GEMMs (M <= 64) is
 * never written by the kernel that precedes the GEMM on its stream.  The small-M
 * kernel is launched with programmatic dependent launch; with this promise it
 * starts streaming weights while the previous kernel's last CTAs are still
 * finishing (activations, scales, bias and C are touched only after the
 * previous kernel has completed either way).  Returns the previous setting.
 * No reference counterpart. */
TG_API int32_t tg_set_static_weights(int32_t on);

/* Re-reads the TILEGYM_B200_* tuning / debug variables from the environment.  They are otherwise read once,
 * by the first call that needs one (a launch does not scan the environment).  No reference counterpart. */
TG_API void tg_reload_env(void);

/* Bound of every wait inside the kernels (on an mbarrier: a TMA copy landing, the tensor core finishing, a
 * buffer being released), in microseconds; 0 restores the default of 2 s.  A wait that runs out makes its
 * kernel record a code, leave its loops, free its TMEM and return; tg_device_status() then reports
 * TG_ERR_TIMEOUT.  After such a report the output of that launch is undefined and the split-K arrival
 * counters at the start of the workspace it used may be non-zero: clear the first 64 KiB of that workspace
 * before using it again.  Returns the previous setting.  No reference counterpart (its kernels
 * contain no device-side waits of their own). */
TG_API uint32_t tg_set_wait_limit_us(uint32_t limit_us);

/* Runs the bounded-wait give-up path once, safely: one thread block with the kernels' role layout allocates
 * TMEM and waits, with the kernels' own wait code, for a barrier nothing arrives on; after limit_us
 * (1 .. 1000000) the wait gives up, the block frees its TMEM and returns normally, and tg_device_status()
 * reports TG_ERR_TIMEOUT (detail = role * 1000 + 99) once.  Nothing faults or hangs and the context stays
 * usable.  No reference counterpart. */
TG_API int32_t tg_selftest_wait_timeout(uint32_t limit_us, int32_t device_id, uint64_t stream);

/* Self-test of the quantisers' arithmetic: compares their division-free quotient and scale with IEEE division for
 * every (group maximum, element) pair a 16-bit input type (x_dtype: TG_BF16 / TG_F16) can produce, for the target
 * format y_dtype (TG_F8E4M3 / TG_F8E5M2 / TG_I8).  counts: four 64-bit words on the device, filled on the stream
 * with {pairs whose bytes differ, pairs compared, scales that differ, maxima outside the fast path's range}; the
 * first and third must be 0.  A few milliseconds.  The reference has no counterpart. */
TG_API int32_t tg_selftest_quant16(int32_t x_dtype, int32_t y_dtype, uint64_t counts, int32_t device_id,
                                   uint64_t stream);

/* Reads (and clears) the device-side status word of `device_id` after
 * synchronising the device: 0, or TG_ERR_TIMEOUT with *detail set to a code
 * naming the wait that gave up.  detail may be NULL. */
TG_API int32_t tg_device_status(int32_t device_id, int32_t* detail);

/* Message of the last failing call made by this thread ("" if none). */
TG_API const char* tg_last_error_string(void);

/* Host-only (no CUDA call): the tile width and K-split count the library would pick on a GPU with num_sms SMs.
 * kind 0: per-tensor GEMM on single-CTA tiles (64 < M < 512 where the CTA-pair kernel would not fill the GPU);
 * kind 1: block-scaled GEMM on 128 x 128 tiles.  The counterpart of the launch-shape choice in the reference's
 * wrapper (src/tilegym/suites/unsloth/cutile/fp8.py:417-420: BLOCK_SIZE_M from M, one program per tile); here
 * the choice is a cost model, waves x (k-blocks per unit + split tail), exposed for inspection and tests. */
TG_API int32_t tg_plan_splits(int32_t kind, int64_t M, int64_t N, int64_t K, int32_t num_sms, int32_t* tile_cols,
                              int32_t* splits);

/* Library version, e.g. 100 for 0.1.0. */
TG_API int32_t tg_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TILEGYM_B200_H_ */

// Split-K reduction inside a thread-block cluster, shared by the small-M kernels: the K splits of a tile form a
// cluster; after its main loop every CTA holds its fp32 partial tile [rows][128] in its own shared memory and sends
// each peer the block of rows that peer owns with ONE bulk copy (cp.async.bulk shared::cta -> shared::cluster,
// completion counted in bytes on the owner's mbarrier); each owner adds its rows in split order (bit-stable).
// A sender may leave once every owner it sent to has acknowledged (a remote arrive on the sender's "done"
// mbarrier, made as soon as that owner's inbox is complete), so nobody waits for another CTA's stores.
#pragma once
#include "tg_gemm_common.cuh"

namespace tg {

__device__ __forceinline__ uint32_t cl_map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// Bulk copy of `bytes` (a multiple of 16) from this CTA's shared memory to the shared memory of another CTA of the
// cluster; completion is counted in bytes on an mbarrier of the destination CTA.
__device__ __forceinline__ void cl_bulk_copy_to_peer(uint32_t dst_cluster_addr, uint32_t src_cta_addr, uint32_t bytes,
                                                      uint32_t mbar_cluster_addr) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   dst_cluster_addr),
               "r"(src_cta_addr), "r"(bytes), "r"(mbar_cluster_addr)
               : "memory");
}
// Arrive (release, cluster scope) on an mbarrier in the shared memory of another CTA of the cluster.
__device__ __forceinline__ void cl_mbar_arrive_remote(uint32_t mbar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(mbar_cluster_addr) : "memory");
}
__device__ __forceinline__ void cl_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cl_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Cluster reduction, owner side, one output row: the sum over the splits, in split order (bit-stable), of four
// consecutive columns; split `own` is read from this CTA's own partial tile, the others from the inbox blocks.
// All loads are issued before the first add.
__device__ __forceinline__ float4 cl_sum_splits(const float* tile_row, const float* inbox_row, int rpr, int splits,
                                                int own) {
  float4 v[8];
#pragma unroll
  for (int s2 = 0; s2 < 8; ++s2)
    v[s2] = s2 < splits ? *reinterpret_cast<const float4*>(s2 == own ? tile_row : inbox_row + s2 * rpr * kBM)
                        : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 sum = v[0];
#pragma unroll
  for (int s2 = 1; s2 < 8; ++s2) {
    if (s2 < splits) {
      sum.x += v[s2].x;
      sum.y += v[s2].y;
      sum.z += v[s2].z;
      sum.w += v[s2].w;
    }
  }
  return sum;
}

// Stores v[0..4) at columns col .. col + 3 of one output row (columns >= n_valid skipped); `vec_ok`: the four
// elements start on a boundary of their combined size.
__device__ __forceinline__ void cl_store4(const GemmParams& p, int64_t row, int64_t col, const float (&v)[4],
                                           int n_valid, bool vec_ok) {
  const int64_t off = row * p.ldc + col;
  if (p.out_dtype == TG_BF16) {
    __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
    if (vec_ok && n_valid >= 4) {
      *reinterpret_cast<uint2*>(c) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
    } else {
      for (int i = 0; i < 4 && i < n_valid; ++i) c[i] = __float2bfloat16_rn(v[i]);
    }
  } else if (p.out_dtype == TG_F16) {
    __half* c = reinterpret_cast<__half*>(p.C) + off;
    if (vec_ok && n_valid >= 4) {
      *reinterpret_cast<uint2*>(c) = make_uint2(pack_f16x2(v[0], v[1]), pack_f16x2(v[2], v[3]));
    } else {
      for (int i = 0; i < 4 && i < n_valid; ++i) c[i] = __float2half_rn(v[i]);
    }
  } else {
    float* c = reinterpret_cast<float*>(p.C) + off;
    if (vec_ok && n_valid >= 4) {
      *reinterpret_cast<float4*>(c) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      for (int i = 0; i < 4 && i < n_valid; ++i) c[i] = v[i];
    }
  }
}

}  // namespace tg

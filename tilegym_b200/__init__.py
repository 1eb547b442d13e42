"""tilegym_b200: the FP8 scaled-GEMM path of TileGym as hand-written sm_100a kernels.

Public surface (same names and signatures as the reference operators):
    w8a8_block_fp8_matmul, act_quant, weight_dequant   (tilegym.suites.unsloth.ops)
    gemm_alpha_beta                                    (tilegym.suites.flashinfer.ops)
    matmul, bmm                                        (tilegym.ops)
plus the per-tensor pieces the reference lacks (fp8_scaled_mm, fp8_block_scaled_mm, quant_per_tensor,
weight_quant_block, FP8Linear) and apply_tilegym_kernel_to_llama / _deepseek_v2.
"""

from .ops import (  # noqa: F401
    act_quant,
    bmm,
    fp8_block_scaled_mm,
    fp8_scaled_mm,
    per_token_group_quant_8bit,
    ragged_block_scaled_bmm,
    fp8_scaled_mm_no_alloc,
    fp8_scaled_mm_swiglu,
    interleave_gate_up,
    gemm_alpha_beta,
    matmul,
    quant_per_tensor,
    reset_workspaces,
    set_static_weights,
    w8a8_block_fp8_matmul,
    weight_dequant,
    weight_quant_block,
)

from .moe import FP8MoE, fused_experts_impl, fused_moe, moe_align_block_size  # noqa: E402,F401

__version__ = "0.1.0"

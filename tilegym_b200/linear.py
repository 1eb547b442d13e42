"""FP8Linear: an nn.Linear whose matmul runs on the sm_100a FP8 GEMM.

The reference's Linear glue (`_linear_cutile`, src/tilegym/transformers/olmoe/modeling_olmoe.py:50-61, and
`PartiallyFusedSwiGLUMLP.apply_matmul_internal`, src/tilegym/ops/fused_mlp.py:109-112) calls a bf16 `matmul`
on a cached transposed weight; it has no FP8 Linear.  This module keeps the same shape contract - input
(..., in_features), weight (out_features, in_features) used as is (no transposed copy), output
(..., out_features) - and quantises the weight ONCE:

  mode "per_tensor": weight -> e4m3 with one amax/448 scale; each forward quantises the activation
                     per tensor on the GPU and calls the per-tensor GEMM with the bias fused.
  mode "block":      weight -> e4m3 with 128 x 128 block scales; each forward runs act_quant (1 x 128)
                     and the block-scaled GEMM (DeepSeek-style).
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import ops

MODES = ("per_tensor", "block")


class FP8Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, mode: str = "per_tensor",
                 device=None, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        if mode not in MODES:
            raise ValueError(f"mode must be one of {MODES}")
        if mode == "block" and in_features % 128 != 0:
            raise ValueError("block mode needs in_features to be a multiple of 128 (the activation quantisation block)")
        if in_features % 16 != 0:
            raise ValueError("in_features must be a multiple of 16 (TMA row pitch)")
        self.in_features, self.out_features, self.mode = in_features, out_features, mode
        self.out_dtype = dtype
        self.register_buffer("weight_fp8", torch.zeros(out_features, in_features, dtype=torch.float8_e4m3fn, device=device))
        if mode == "per_tensor":
            self.register_buffer("weight_scale", torch.ones(1, dtype=torch.float32, device=device))
        else:
            self.register_buffer(
                "weight_scale",
                torch.ones(-(-out_features // 128), in_features // 128, dtype=torch.float32, device=device),
            )
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device), requires_grad=False)
        else:
            self.register_parameter("bias", None)

    @classmethod
    def from_linear(cls, linear: nn.Linear, mode: str = "per_tensor") -> "FP8Linear":
        """Quantises `linear.weight` (which must live on a CUDA device) with the GPU quantisers."""
        w = linear.weight.detach()
        mod = cls(linear.in_features, linear.out_features, linear.bias is not None, mode, w.device,
                  w.dtype if w.dtype in (torch.bfloat16, torch.float16, torch.float32) else torch.bfloat16)
        mod.load_weight(w, linear.bias.detach() if linear.bias is not None else None)
        return mod

    @torch.no_grad()
    def load_weight(self, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        if self.mode == "per_tensor":
            q, s = ops.quant_per_tensor(w)
        else:
            q, s = ops.weight_quant_block(w)
        self.weight_fp8.copy_(q)
        self.weight_scale.copy_(s)
        if bias is not None and self.bias is not None:
            self.bias.copy_(bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out_dtype = x.dtype if x.dtype in (torch.bfloat16, torch.float16, torch.float32) else self.out_dtype
        if self.mode == "per_tensor":
            xq, sx = ops.quant_per_tensor(x)
            # the weight is a constant of the layer: decode-sized calls may stream it before the quantiser ends
            return ops.fp8_scaled_mm(xq, self.weight_fp8, sx, self.weight_scale, self.bias, out_dtype,
                                     static_weights=True)
        xq, sx = ops.act_quant(x, 128)
        return ops.fp8_block_scaled_mm(xq, self.weight_fp8, sx, self.weight_scale, self.bias, out_dtype)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, mode={self.mode}"


class FP8SwiGLUMLP(nn.Module):
    """down_proj(silu(gate_proj(x)) * up_proj(x)) with e4m3 weights and per-tensor scales: one fused gate/up
    GEMM whose epilogue applies SwiGLU (the [tokens, 2 * intermediate] tensor of
    src/tilegym/ops/fused_mlp.py:85-107 is never written), then the down GEMM.  Built from an MLP that has
    `gate_proj`, `up_proj` and `down_proj` Linear layers (Llama, Mistral, Qwen2, ...)."""

    def __init__(self, gate_proj: nn.Linear, up_proj: nn.Linear, down_proj: nn.Linear):
        super().__init__()
        assert gate_proj.weight.shape == up_proj.weight.shape and gate_proj.out_features % 64 == 0
        assert (gate_proj.bias is None) == (up_proj.bias is None)
        with torch.no_grad():
            w = ops.interleave_gate_up(gate_proj.weight.detach(), up_proj.weight.detach())
            q, s = ops.quant_per_tensor(w)
            self.register_buffer("gate_up_fp8", q)
            self.register_buffer("gate_up_scale", s)
            if gate_proj.bias is not None:
                self.register_buffer("gate_up_bias", ops.interleave_gate_up(gate_proj.bias.detach(), up_proj.bias.detach()))
            else:
                self.gate_up_bias = None
        self.down = FP8Linear.from_linear(down_proj, "per_tensor")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out_dtype = x.dtype if x.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
        xq, sx = ops.quant_per_tensor(x)
        h = ops.fp8_scaled_mm_swiglu(xq, self.gate_up_fp8, sx, self.gate_up_scale, self.gate_up_bias, out_dtype)
        return self.down(h)


def _linear_fp8(self, attr_name: str, x: torch.Tensor) -> torch.Tensor:
    """Counterpart of the reference helper `_linear_cutile(self, attr_name, x)`
    (src/tilegym/transformers/olmoe/modeling_olmoe.py:50-61): runs the Linear stored at `attr_name` of a
    module through the FP8 path, caching the quantised module next to it on first use."""
    cache = f"_tilegym_fp8_{attr_name}"
    mod = getattr(self, cache, None)
    if mod is None:
        mod = FP8Linear.from_linear(getattr(self, attr_name))
        object.__setattr__(self, cache, mod)
    return mod(x)


def _is_swiglu_mlp(m: nn.Module) -> bool:
    """A gate_proj / up_proj / down_proj MLP with a SiLU activation (Llama, Mistral, Qwen2, ...)."""
    parts = [getattr(m, n, None) for n in ("gate_proj", "up_proj", "down_proj")]
    if not all(isinstance(x, nn.Linear) for x in parts):
        return False
    gate, up, down = parts
    act = getattr(m, "act_fn", None)
    silu = isinstance(act, nn.SiLU) or type(act).__name__ in ("SiLUActivation", "SiLU") or act is nn.functional.silu
    return (silu and gate.weight.shape == up.weight.shape and gate.out_features % 64 == 0
            and gate.in_features % 16 == 0 and down.in_features % 16 == 0
            and (gate.bias is None) == (up.bias is None))


def convert_linears(module: nn.Module, mode: str = "per_tensor", skip=("lm_head",), fuse_swiglu: bool = False) -> int:
    """Replaces every nn.Linear under `module` (weights already on a CUDA device) by an FP8Linear,
    except children whose name is in `skip`.  With `fuse_swiglu` (per-tensor mode) a gate / up / down MLP
    with a SiLU activation becomes one FP8SwiGLUMLP instead.  Returns the number of replaced Linear layers."""
    n = 0
    for name, child in list(module.named_children()):
        if fuse_swiglu and mode == "per_tensor" and _is_swiglu_mlp(child):
            setattr(module, name, FP8SwiGLUMLP(child.gate_proj, child.up_proj, child.down_proj))
            n += 3
        elif isinstance(child, nn.Linear) and name not in skip:
            ok_block = child.in_features % 128 == 0
            if child.in_features % 16 == 0 and (mode == "per_tensor" or ok_block):
                setattr(module, name, FP8Linear.from_linear(child, mode))
                n += 1
        else:
            n += convert_linears(child, mode, skip, fuse_swiglu)
    return n

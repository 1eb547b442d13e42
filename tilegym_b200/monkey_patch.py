"""Model-level entry points with the reference's signatures.

`apply_tilegym_kernel_to_<model>(rope, rms_norm, swiglu, attn, model, use_cutile)` is the signature of
src/tilegym/transformers/monkey_patch.py:24-31 (llama), :64-72 (deepseek_v2) and the other model types; this
package covers only the FP8 Linear path, so those flags are accepted for drop-in compatibility and do nothing
here (the kernels they select are outside this library), and one opt-in keyword is added: `fp8_linear`.
With `fp8_linear=True` the nn.Linear layers of the decoder are replaced by `FP8Linear`:
  * `model` given  -> its Linear modules are converted in place (weights must be on a CUDA device);
  * `model` None   -> (the reference's "call before model initialisation" form) models of that type built
                      afterwards get a hook that converts them at their first forward, when their weights
                      are loaded and on the GPU; `convert_model(model)` does the same explicitly.
`MODEL_TYPE_TO_APPLY_TILEGYM_FN` and `_apply_tilegym_kernel(model_type, **kwargs)` mirror :555-599
(kwargs not in the target's signature are dropped).
"""

from __future__ import annotations

import inspect
import logging
from typing import Callable, Dict, Optional

from torch import nn

from .linear import convert_linears

logger = logging.getLogger("tilegym_b200")

# model_type -> default FP8 mode (DeepSeek checkpoints ship 128x128 block scales)
_DEFAULT_MODE = {"deepseek_v2": "block"}
_pending: Dict[str, tuple] = {}  # model types whose models get converted on first forward


def convert_model(model: nn.Module, mode: str = "per_tensor", fuse_swiglu: bool = False) -> int:
    """Converts the Linear layers of a loaded model (on a CUDA device); keeps `lm_head` in its dtype.  With
    `fuse_swiglu` the SiLU MLPs run their gate / up projection and the activation as one kernel."""
    n = convert_linears(model, mode, fuse_swiglu=fuse_swiglu)
    logger.info("tilegym_b200: %d nn.Linear modules now run the FP8 GEMM (%s scales)", n, mode)
    return n


def _first_forward_hook(mode: str, fuse_swiglu: bool = False) -> Callable:
    def hook(module, args, kwargs):
        if not getattr(module, "_tilegym_fp8_done", False):
            object.__setattr__(module, "_tilegym_fp8_done", True)
            convert_model(module, mode, fuse_swiglu)
        return None

    return hook


def _apply(model_type: str, model, fp8_linear: bool, fp8_mode: Optional[str], fuse_swiglu: bool = False) -> None:
    if not fp8_linear:
        return
    mode = fp8_mode or _DEFAULT_MODE.get(model_type, "per_tensor")
    if model is not None:
        convert_model(model, mode, fuse_swiglu)
        return
    # Before model initialisation: convert each model of this type when it first runs (its weights are
    # loaded and placed by then).
    _pending[model_type] = (mode, fuse_swiglu)
    try:
        from transformers import PreTrainedModel
    except Exception as exc:  # transformers is only needed for the pre-initialisation form
        raise RuntimeError("fp8_linear=True without a model needs the transformers package") from exc
    if not getattr(PreTrainedModel, "_tilegym_b200_wrapped", False):
        original_post_init = PreTrainedModel.post_init

        def post_init(self, *a, **k):
            out = original_post_init(self, *a, **k)
            mt = getattr(getattr(self, "config", None), "model_type", None)
            if mt in _pending and not getattr(self, "_tilegym_fp8_hooked", False) and hasattr(self, "lm_head"):
                object.__setattr__(self, "_tilegym_fp8_hooked", True)
                self.register_forward_pre_hook(_first_forward_hook(*_pending[mt]), with_kwargs=True)
            return out

        PreTrainedModel.post_init = post_init
        PreTrainedModel._tilegym_b200_wrapped = True


def _make(model_type: str, flags=("rope", "rms_norm", "swiglu", "attn"), defaults=None, takes_model: bool = True,
          fuse_flag: Optional[str] = "swiglu"):
    """Builds apply_tilegym_kernel_to_<model_type> with the reference's keyword list for that model (`flags`, then
    `model` where the reference takes one, then `use_cutile`) plus `fp8_linear` / `fp8_mode`.  `fuse_flag` names the
    reference switch of the fused gated MLP, which selects the fused gate/up + SiLU*mul kernel when the FP8 path is on."""
    defaults = defaults or {}
    names = list(flags) + (["model"] if takes_model else []) + ["use_cutile", "fp8_linear", "fp8_mode"]
    params = []
    for n in names:
        if n == "model" or n == "fp8_mode":
            default = None
        elif n in ("use_cutile", "fp8_linear"):
            default = False
        else:
            default = defaults.get(n, True)
        params.append(inspect.Parameter(n, inspect.Parameter.POSITIONAL_OR_KEYWORD, default=default))
    signature = inspect.Signature(params)

    def apply_fn(*args, **kwargs) -> None:
        bound = signature.bind(*args, **kwargs)
        bound.apply_defaults()
        a = bound.arguments
        for flag in flags:
            if a[flag] and not (flag == fuse_flag and a["fp8_linear"]):
                logger.debug("tilegym_b200: %s=True accepted; that kernel is not part of this library", flag)
        _apply(model_type, a.get("model"), a["fp8_linear"], a["fp8_mode"],
               fuse_swiglu=bool(a[fuse_flag]) if fuse_flag else False)

    apply_fn.__signature__ = signature
    apply_fn.__name__ = f"apply_tilegym_kernel_to_{model_type}"
    apply_fn.__doc__ = (
        f"Signature of the reference's apply_tilegym_kernel_to_{model_type} plus the opt-in `fp8_linear` / "
        "`fp8_mode` keywords; only the FP8 Linear replacement is implemented here."
    )
    return apply_fn


# keyword lists of src/tilegym/transformers/monkey_patch.py:24-31 (llama), :64-72 (deepseek_v2), :118-125 (qwen2),
# :158-166 (qwen3_5), :240-246 (gpt_oss: no `model`, swiglu off by default), :293-300 (gemma3: `mlp`), :350-357
# (mistral), :393-400 (phi3), :437-444 (olmoe), :495-502 (olmo3)
apply_tilegym_kernel_to_llama = _make("llama")
apply_tilegym_kernel_to_deepseek_v2 = _make("deepseek_v2", flags=("rope", "rms_norm", "swiglu", "attn", "moe"))
apply_tilegym_kernel_to_mistral = _make("mistral")
apply_tilegym_kernel_to_qwen2 = _make("qwen2")
apply_tilegym_kernel_to_qwen3 = _make("qwen3_5", flags=("rope", "rms_norm", "swiglu", "attn", "gated_delta_rule"))
apply_tilegym_kernel_to_gpt_oss = _make("gpt_oss", defaults={"swiglu": False}, takes_model=False)
apply_tilegym_kernel_to_gemma3 = _make("gemma3", flags=("rope", "rms_norm", "mlp", "attn"), fuse_flag=None)
apply_tilegym_kernel_to_phi3 = _make("phi3")
apply_tilegym_kernel_to_olmo3 = _make("olmo3")
apply_tilegym_kernel_to_olmoe = _make("olmoe", flags=("rope", "rms_norm", "attn", "moe"), fuse_flag=None)

MODEL_TYPE_TO_APPLY_TILEGYM_FN = {
    "llama": apply_tilegym_kernel_to_llama,
    "deepseek_v2": apply_tilegym_kernel_to_deepseek_v2,
    "gpt_oss": apply_tilegym_kernel_to_gpt_oss,
    "mistral": apply_tilegym_kernel_to_mistral,
    "qwen2": apply_tilegym_kernel_to_qwen2,
    "qwen3_5": apply_tilegym_kernel_to_qwen3,
    "gemma3": apply_tilegym_kernel_to_gemma3,
    "phi3": apply_tilegym_kernel_to_phi3,
    "olmo3": apply_tilegym_kernel_to_olmo3,
    "olmoe": apply_tilegym_kernel_to_olmoe,
}


def _apply_tilegym_kernel(model_type: str, **kwargs) -> None:
    """Same contract as the reference (src/tilegym/transformers/monkey_patch.py:569-599): unknown model
    types are ignored with a log line, kwargs the target does not take are dropped."""
    if not model_type:
        logger.info("Model type was not provided. No kernels will be applied.")
        return
    if model_type not in MODEL_TYPE_TO_APPLY_TILEGYM_FN:
        logger.info("There are currently no kernels supported for model type: %s.", model_type)
        return
    fn = MODEL_TYPE_TO_APPLY_TILEGYM_FN[model_type]
    params = inspect.signature(fn).parameters
    fn(**{k: v for k, v in kwargs.items() if k in params})

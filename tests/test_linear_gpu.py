"""FP8Linear and the model-level entry point on the GPU."""

import pytest
import torch

from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

from tilegym_b200 import monkey_patch  # noqa: E402
from tilegym_b200.linear import FP8Linear, _linear_fp8  # noqa: E402


@pytest.mark.parametrize("mode", ["per_tensor", "block"])
@pytest.mark.parametrize("bias", [False, True])
def test_fp8linear_matches_oracle_chain(dev, mode, bias):
    torch.manual_seed(3)
    lin = torch.nn.Linear(512, 384, bias=bias, dtype=torch.bfloat16)
    x = torch.randn(4, 33, 512, dtype=torch.bfloat16)
    if mode == "per_tensor":
        xq, sx = R.ref_quant_per_tensor(x.view(-1, 512))
        wq, sw = R.ref_quant_per_tensor(lin.weight.detach())
        ref = R.ref_fp8_scaled_mm(xq, wq, sx, sw, lin.bias.detach() if bias else None)
    else:
        xq, sx = R.ref_act_quant(x.view(-1, 512))
        wq, sw = R.ref_weight_quant_block(lin.weight.detach())
        # the bias joins the fp32 sum before the one rounding to bf16, in the kernel's epilogue
        ref = R.ref_fp8_block_scaled_mm(xq, wq, sx, sw, lin.bias.detach() if bias else None, torch.bfloat16)
    mod = FP8Linear.from_linear(lin.to(dev), mode)
    out = mod(x.to(dev))
    assert out.shape == (4, 33, 384) and out.dtype == torch.bfloat16
    assert R.check_tolerance(out.view(-1, 384), ref)["ok"]


def test_linear_helper_caches_quantised_module(dev):
    class Holder(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = torch.nn.Linear(256, 128, bias=False, dtype=torch.bfloat16)

    h = Holder().to(dev)
    x = torch.randn(16, 256, dtype=torch.bfloat16, device=dev)
    y1 = _linear_fp8(h, "q_proj", x)
    assert isinstance(h._tilegym_fp8_q_proj, FP8Linear)
    assert torch.equal(y1, _linear_fp8(h, "q_proj", x))
    assert torch.nn.functional.cosine_similarity(y1.float().flatten(), h.q_proj(x).float().flatten(), dim=0) > 0.995


@pytest.mark.parametrize("swiglu", [True, False])
def test_apply_to_llama_converts_decoder_linears(dev, swiglu):
    transformers = pytest.importorskip("transformers")
    from tilegym_b200.linear import FP8SwiGLUMLP

    cfg = transformers.LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=320, max_position_embeddings=128)
    torch.manual_seed(0)
    model = transformers.LlamaForCausalLM(cfg).to(dev, torch.bfloat16).eval()
    ids = torch.randint(0, 320, (2, 24), device=dev)
    with torch.no_grad():
        base = model(ids).logits.float()
    monkey_patch.apply_tilegym_kernel_to_llama(model=model, fp8_linear=True, swiglu=swiglu)
    n_fp8 = sum(isinstance(m, FP8Linear) for m in model.modules())
    n_mlp = sum(isinstance(m, FP8SwiGLUMLP) for m in model.modules())
    # per layer q, k, v, o and either gate, up, down or one fused MLP (which holds the down projection)
    assert (n_fp8, n_mlp) == ((2 * 5, 2) if swiglu else (2 * 7, 0)) and isinstance(model.lm_head, torch.nn.Linear)
    with torch.no_grad():
        got = model(ids).logits.float()
    cos = torch.nn.functional.cosine_similarity(base.flatten(), got.flatten(), dim=0)
    assert cos > 0.99, float(cos)

"""Shape sweeps that accompany the headline number of bench.py.

`run_configs` (part of the default N = 1 run) covers the other benchmark
configurations in bounded form: the 1024-cube GEMM, the decode (M <= 64,
HBM-bound) GEMMs of the Llama-3.1-8B linears, the DeepSeek-V2-style
block-scaled GEMMs and the Llama-3.1-70B gate_up GEMM on one GPU.  `run`
(`--extra`) adds the grouped GEMM, the quantisers, the SwiGLU epilogue and a
whole MLP block.

Timing method for the small kernels: R launches are captured into one CUDA
graph, each reading a different copy of the weight (the copies together are
several times the 126 MB L2, so every launch streams its weight from HBM),
the graph is replayed a few times between CUDA events and the time is divided
by the number of launches.  Host launch overhead is therefore excluded and
the L2 is cold for the weights; the few-KB activations stay L2-resident as
they would in a decode loop.
"""

from __future__ import annotations

import math

import torch

LLAMA8B = [("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]
DEEPSEEK = [(24576, 1536), (5120, 12288), (3072, 5120)]
L2_BYTES = 126e6


def graph_time_us(launch, n_variants: int, replays: int = 5) -> float:
    """`launch(i)` enqueues variant i on the current stream.  Returns microseconds per launch."""
    for i in range(min(n_variants, 2)):
        launch(i)  # warm-up outside capture: module load, attributes, workspace
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n_variants):
            launch(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (replays * n_variants)


def decode_sweep(dev, hbm_peak_gbs: float):
    import tilegym_b200 as tg

    rows = []
    for name, N, K in LLAMA8B:
        copies = max(4, math.ceil(4 * L2_BYTES / (N * K)))
        w = [torch.randn(N, K, device=dev, dtype=torch.bfloat16).mul_(0.02).to(torch.float8_e4m3fn) for _ in range(copies)]
        sb = torch.full((1,), 2e-4, device=dev)
        sa = torch.full((1,), 3e-2, device=dev)
        for M in (1, 8, 16, 64):
            a = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
            outs = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(copies)]
            launch = lambda i: tg.fp8_scaled_mm(a, w[i], sa, sb, None, torch.bfloat16, out=outs[i])  # noqa: E731
            us_default = graph_time_us(launch, copies)
            # as FP8Linear calls it: the weights are constants, so consecutive GEMMs may overlap their weight
            # streaming with the previous kernel's tail (programmatic dependent launch)
            launch_static = lambda i: tg.fp8_scaled_mm(a, w[i], sa, sb, None, torch.bfloat16, out=outs[i],  # noqa: E731
                                                       static_weights=True)
            us = graph_time_us(launch_static, copies)
            nbytes = N * K + M * K + 2 * M * N + 8
            gbs = nbytes / us / 1e3
            rows.append({"shape": name, "M": M, "N": N, "K": K, "us": round(us, 2), "gbs": round(gbs, 1),
                         "frac_of_measured_hbm": round(gbs / hbm_peak_gbs, 3), "weight_copies": copies,
                         "us_without_static_weight_promise": round(us_default, 2)})
        del w
    return rows


def block_scaled_sweep(dev, fp8_peak_tflops: float, hbm_peak_gbs: float):
    import tilegym_b200 as tg

    rows = []
    for N, K in DEEPSEEK:
        for M in (128, 4096):
            copies = max(2, math.ceil(3 * L2_BYTES / (N * K))) if M == 128 else 2
            b = [torch.randn(N, K, device=dev, dtype=torch.bfloat16).mul_(0.02).to(torch.float8_e4m3fn) for _ in range(copies)]
            a = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
            As = torch.rand(M, K // 128, device=dev) + 0.5
            Bs = torch.rand(N // 128, K // 128, device=dev) + 0.5
            us = graph_time_us(lambda i: tg.w8a8_block_fp8_matmul(a, b[i], As, Bs, [128, 128], torch.bfloat16), copies,
                               replays=5 if M == 128 else 10)
            flops = 2.0 * M * N * K
            nbytes = M * K + N * K + 2 * M * N + 4 * (As.numel() + Bs.numel())
            rows.append({"M": M, "N": N, "K": K, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                         "gbs": round(nbytes / us / 1e3, 1),
                         "bound": "hbm" if M == 128 else "tensor",
                         "frac": round((nbytes / us / 1e3) / hbm_peak_gbs if M == 128 else (flops / us / 1e6) / fp8_peak_tflops, 3)})
            del b
    return rows


def quantiser_sweep(dev, hbm_peak_gbs: float):
    """The activation-side quantisers on a [8192, 14336] bf16 activation (235 MB, > L2): algorithmic bytes
    (input + 8-bit output + scales; the per-tensor quantiser reads its input twice) over CUDA-event time."""
    import tilegym_b200 as tg

    T, H = 8192, 14336
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    cases = [
        ("act_quant_1x128", lambda: tg.act_quant(x), 3 * T * H + 4 * T * H // 128),
        ("per_token_group_quant_g128", lambda: tg.per_token_group_quant_8bit(x, 128), 3 * T * H + 4 * T * H // 128),
        ("per_token_group_quant_g32_colmajor_ue8m0",
         lambda: tg.per_token_group_quant_8bit(x, 32, column_major_scales=True, scale_ue8m0=True),
         3 * T * H + 4 * T * H // 32),
        ("quant_per_tensor", lambda: tg.quant_per_tensor(x), 5 * T * H),
    ]
    rows = []
    for name, fn, nbytes in cases:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        rows.append({"op": name, "us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1),
                     "frac_of_measured_hbm": round(nbytes / us / 1e3 / hbm_peak_gbs, 3)})
    return rows


def grouped_sweep(dev, fp8_peak_tflops: float):
    """Grouped (MoE-style) block-scaled GEMM on the DeepSeek-V2 expert shape (N, K) = (3072, 5120): 4096 rows
    routed to 8 experts, evenly and raggedly; FLOPs = 2 * rows * N * K whatever the routing."""
    import tilegym_b200 as tg

    N, K, total = 3072, 5120, 4096
    rows = []
    for name, sizes in (("8 x 512", [512] * 8), ("ragged", [37, 901, 512, 3, 1200, 640, 0, 803])):
        assert sum(sizes) == total
        G = len(sizes)
        a = torch.randn(total, K, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(G, N, K, device=dev, dtype=torch.bfloat16).mul_(0.02).to(torch.float8_e4m3fn)
        As = torch.rand(total, K // 128, device=dev) + 0.5
        Bs = torch.rand(G, N // 128, K // 128, device=dev) + 0.5
        ind = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device=dev)
        us = graph_time_us(lambda i: tg.ragged_block_scaled_bmm(a, b, As, Bs, ind, max(sizes)), 4, replays=10)
        flops = 2.0 * total * N * K
        rows.append({"routing": name, "groups": G, "rows": total, "N": N, "K": K, "us": round(us, 2),
                     "tflops": round(flops / us / 1e6, 1), "frac": round(flops / us / 1e6 / fp8_peak_tflops, 3)})
    return rows


def swiglu_sweep(dev):
    """Llama-3.1-8B gate/up projection at M = 4096 with SwiGLU: the fused epilogue against the two-step path
    (the same GEMM writing [M, 2I] bf16, then silu(gate) * up as a torch elementwise pass)."""
    import tilegym_b200 as tg

    M, I, K = 4096, 14336, 4096
    a = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
    w = torch.randn(2 * I, K, device=dev, dtype=torch.bfloat16).mul_(0.02).to(torch.float8_e4m3fn)
    sa = torch.full((1,), 3e-2, device=dev)
    sb = torch.full((1,), 2e-4, device=dev)
    out = torch.empty(M, I, dtype=torch.bfloat16, device=dev)
    y = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=dev)

    def two_step():
        tg.fp8_scaled_mm(a, w, sa, sb, None, torch.bfloat16, out=y)
        torch.mul(torch.nn.functional.silu(y[:, :I]), y[:, I:], out=out)

    res = {}
    for name, fn in (("fused_us", lambda: tg.fp8_scaled_mm_swiglu(a, w, sa, sb, None, torch.bfloat16, out=out)),
                     ("gemm_then_silu_mul_us", two_step)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            fn()
        e1.record()
        torch.cuda.synchronize()
        res[name] = round(e0.elapsed_time(e1) * 1e3 / 20, 1)
    res["shape"] = f"M={M} I={I} K={K}"
    res["fused_tflops"] = round(2.0 * M * 2 * I * K / res["fused_us"] / 1e6, 1)
    return res


def mlp_block_sweep(dev):
    """One Llama-3.1-8B MLP block (hidden 4096, intermediate 14336) on 4096 tokens, bf16 in and out:
    FP8SwiGLUMLP (activation quantiser, fused gate/up + SwiGLU GEMM, quantiser, down GEMM) against the same
    block in bf16 through torch (three cuBLAS GEMMs and an elementwise pass)."""
    from tilegym_b200.linear import FP8SwiGLUMLP

    H, I, M = 4096, 14336, 4096
    torch.manual_seed(0)
    gate, up, down = (torch.nn.Linear(H, I, bias=False), torch.nn.Linear(H, I, bias=False),
                      torch.nn.Linear(I, H, bias=False))
    gate, up, down = [m.to(dev).to(torch.bfloat16) for m in (gate, up, down)]
    x = torch.randn(M, H, device=dev, dtype=torch.bfloat16)
    mlp = FP8SwiGLUMLP(gate, up, down)

    def ref():
        return down(torch.nn.functional.silu(gate(x)) * up(x))

    res = {"shape": f"tokens={M} hidden={H} intermediate={I}"}
    with torch.no_grad():
        for name, fn in (("fp8_swiglu_mlp_us", lambda: mlp(x)), ("torch_bf16_mlp_us", ref)):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            torch.cuda.synchronize()
            res[name] = round(e0.elapsed_time(e1) * 1e3 / 10, 1)
        y, r = mlp(x).float(), ref().float()
        res["rel_err_vs_bf16"] = round(float((y - r).abs().max() / r.abs().max()), 4)
    return res


def linear_decode_sweep(dev):
    """FP8Linear forward on decode-sized bf16 activations (what a converted model's Linear costs per token step):
    activation quantiser + GEMM, replayed from a CUDA graph over rotating layers so the weights come from HBM."""
    from tilegym_b200.linear import FP8Linear

    rows = []
    for name, N, K in (("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)):
        n_layers = max(2, int(4 * 126e6 / (N * K)) + 1)
        g = torch.Generator(device=dev).manual_seed(N + K)
        layers = []
        for _ in range(n_layers):
            lin = FP8Linear(K, N, bias=False, mode="per_tensor", device=dev)
            lin.load_weight(torch.randn(N, K, generator=g, device=dev, dtype=torch.bfloat16).mul_(0.02))
            layers.append(lin)
        for M in (1, 16, 64):
            x = torch.randn(M, K, generator=g, device=dev, dtype=torch.bfloat16)
            us = graph_time_us(lambda i: layers[i](x), n_layers)
            rows.append({"shape": name, "M": M, "N": N, "K": K, "us_quantise_plus_gemm": round(us, 2)})
        del layers
        torch.cuda.empty_cache()
    return rows


def cube_1024(dev, fp8_peak_tflops: float):
    """Benchmark configuration 1: one 1024 x 1024 x 1024 per-tensor GEMM (2.1 GFLOP, 4 MB: launch-bound)."""
    import tilegym_b200 as tg

    copies = 8
    a = [torch.randn(1024, 1024, device=dev).to(torch.float8_e4m3fn) for _ in range(copies)]
    b = [torch.randn(1024, 1024, device=dev).to(torch.float8_e4m3fn) for _ in range(copies)]
    out = [torch.empty(1024, 1024, dtype=torch.bfloat16, device=dev) for _ in range(copies)]
    sa = torch.full((1,), 1e-2, device=dev)
    us = graph_time_us(lambda i: tg.fp8_scaled_mm(a[i], b[i], sa, sa, None, torch.bfloat16, out=out[i]), copies, replays=20)
    tflops = 2.0 * 1024 ** 3 / us / 1e6
    return {"M": 1024, "N": 1024, "K": 1024, "us": round(us, 2), "tflops": round(tflops, 1),
            "frac_of_burst_peak": round(tflops / fp8_peak_tflops, 3),
            "note": "16 CTA-pair tiles on 148 SMs: bounded by launch and fill / drain, not by the tensor pipe"}


def llama70b_one_gpu(dev, fp8_peak_tflops: float):
    """The multi-GPU workload (M = 8192, N = 57344, K = 8192) on ONE GPU: the same-workload base of the
    strong-scaling curve."""
    import tilegym_b200 as tg

    M, N, K = 8192, 57344, 8192
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16).to(torch.float8_e4m3fn)
    b = torch.empty(N, K, device=dev, dtype=torch.float8_e4m3fn)
    for i in range(0, N, 8192):  # in slabs: the bf16 source of the whole weight would be 0.9 GB
        b[i:i + 8192] = torch.randn(min(8192, N - i), K, device=dev, dtype=torch.bfloat16).mul_(0.02).to(torch.float8_e4m3fn)
    sa = torch.full((1,), 3e-2, device=dev)
    sb = torch.full((1,), 2e-4, device=dev)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    for _ in range(2):
        tg.fp8_scaled_mm(a, b, sa, sb, None, torch.bfloat16, out=out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    e0.record()
    for _ in range(reps):
        tg.fp8_scaled_mm(a, b, sa, sb, None, torch.bfloat16, out=out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    tflops = 2.0 * M * N * K / ms / 1e9
    return {"M": M, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(tflops, 1),
            "frac_of_burst_peak": round(tflops / fp8_peak_tflops, 3)}


def moe_layer_sweep(dev, fp8_peak_tflops: float):
    """One FP8 mixture-of-experts layer with DeepSeek-V2-Lite's expert shape (hidden 2048, intermediate 1408 -> 1536
    here, a multiple of 128; 64 experts, top-6) on 4096 tokens: the whole fused_experts_impl call, with the first
    GEMM's SiLU * mul + quantise epilogue and without it (separate elementwise pass)."""
    from tilegym_b200 import moe

    T, H, I, E, topk = 4096, 2048, 1536, 64, 6
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(T, H, generator=g, device=dev, dtype=torch.bfloat16)
    w1 = torch.randn(E, 2 * I, H, generator=g, device=dev, dtype=torch.bfloat16).mul_(0.05).to(torch.float8_e4m3fn)
    w2 = torch.randn(E, H, I, generator=g, device=dev, dtype=torch.bfloat16).mul_(0.05).to(torch.float8_e4m3fn)
    w1s = torch.rand(E, 2 * I // 128, H // 128, generator=g, device=dev) + 0.5
    w2s = torch.rand(E, H // 128, I // 128, generator=g, device=dev) + 0.5
    ids = torch.randint(0, E, (T, topk), generator=g, device=dev)
    wts = torch.softmax(torch.randn(T, topk, generator=g, device=dev), dim=-1)
    w1i, w1si = moe.interleave_gate_up_blocks(w1, w1s)
    flops = 2.0 * T * topk * (2 * I * H + H * I)
    res = {"shape": f"tokens={T} hidden={H} intermediate={I} experts={E} top_k={topk}", "gflop": round(flops / 1e9, 1)}
    fused = lambda i: moe.fused_experts_impl(x, w1i, w2, wts, ids, use_fp8_w8a8=True, w1_scale=w1si, w2_scale=w2s,  # noqa: E731
                                             a2_quant="block", w1_interleaved=True, fuse_silu_epilogue=True)
    separate = lambda i: moe.fused_experts_impl(x, w1, w2, wts, ids, use_fp8_w8a8=True, w1_scale=w1s, w2_scale=w2s,  # noqa: E731
                                                a2_quant="block")
    # the layer is a dozen short launches: replayed from a CUDA graph (its routing tables never leave the device)
    res["fused_epilogue_us"] = round(graph_time_us(fused, 2, replays=10), 1)
    res["separate_silu_mul_us"] = round(graph_time_us(separate, 2, replays=10), 1)
    best = min(res["fused_epilogue_us"], res["separate_silu_mul_us"])  # the separate pass is the default path
    res["tflops"] = round(flops / best / 1e6, 1)
    res["frac_of_burst_peak"] = round(res["tflops"] / fp8_peak_tflops, 3)
    return res


def moe_decode_sweep(dev, hbm_peak_gbs: float):
    """The same mixture-of-experts layer at decode sizes: few rows per expert, so both expert GEMMs run on the grouped
    small-M kernel and the layer is a weight-streaming problem (the weights of every expert that got a token)."""
    from tilegym_b200 import moe

    H, I, E, topk = 2048, 1536, 64, 6
    g = torch.Generator(device=dev).manual_seed(0)
    w1 = torch.randn(E, 2 * I, H, generator=g, device=dev, dtype=torch.bfloat16).mul_(0.05).to(torch.float8_e4m3fn)
    w2 = torch.randn(E, H, I, generator=g, device=dev, dtype=torch.bfloat16).mul_(0.05).to(torch.float8_e4m3fn)
    w1s = torch.rand(E, 2 * I // 128, H // 128, generator=g, device=dev) + 0.5
    w2s = torch.rand(E, H // 128, I // 128, generator=g, device=dev) + 0.5
    rows = []
    for T in (1, 16, 64, 256):
        x = torch.randn(T, H, generator=g, device=dev, dtype=torch.bfloat16)
        ids = torch.randint(0, E, (T, topk), generator=g, device=dev)
        wts = torch.softmax(torch.randn(T, topk, generator=g, device=dev), dim=-1)
        touched = int(torch.unique(ids).numel())
        weight_bytes = touched * (2 * I * H + H * I)
        us = graph_time_us(lambda i: moe.fused_experts_impl(x, w1, w2, wts, ids, use_fp8_w8a8=True, w1_scale=w1s,
                                                            w2_scale=w2s, a2_quant="block"), 2, replays=10)
        rows.append({"tokens": T, "experts_touched": touched, "us": round(us, 1),
                     "weight_gbs": round(weight_bytes / us / 1e3, 1),
                     "frac_of_measured_hbm": round(weight_bytes / us / 1e3 / hbm_peak_gbs, 3)})
    return {"shape": f"hidden={H} intermediate={I} experts={E} top_k={topk}", "rows": rows}


def run_configs(dev, peaks):
    """Bounded sweeps of the benchmark configurations the headline number does not cover."""
    hbm = float(peaks["hbm_gbs"])
    fp8 = 2.0 * float(peaks["bf16_tflops"])  # kernels timed alone, in short loops: burst figure
    return {
        "method": "CUDA-graph replay over rotating weight copies (> 3x L2), time per launch (the 70B GEMM: CUDA "
                  "events around 5 launches); fractions are of the measured HBM copy bandwidth "
                  f"({hbm:.0f} GB/s) / of 2 x measured bf16 burst ({fp8:.0f} TFLOP/s)",
        "config1_cube_1024": cube_1024(dev, fp8),
        "config3_decode_per_tensor": decode_sweep(dev, hbm),
        "config3_default": "FP8Linear passes static_weights=True (its weight is a constant of the layer), so `us` / "
                           "`gbs` are what a decode loop through FP8Linear gets; a bare fp8_scaled_mm call, whose "
                           "default makes no such promise, takes `us_without_static_weight_promise`",
        "config4_block_scaled": block_scaled_sweep(dev, fp8, hbm),
        "config5_one_gpu": llama70b_one_gpu(dev, fp8),
    }


def run(dev, peaks):
    hbm = float(peaks["hbm_gbs"])
    fp8 = 2.0 * float(peaks["bf16_tflops"])  # kernels timed alone: burst figure
    return {
        "method": "CUDA-graph replay over rotating weight copies (> 3x L2), time per launch; fractions are of the "
                  "measured HBM copy bandwidth / of 2 x measured bf16 burst",
        "grouped_block_scaled": grouped_sweep(dev, fp8),
        "moe_layer": moe_layer_sweep(dev, fp8),
        "moe_layer_decode": moe_decode_sweep(dev, hbm),
        "quantisers": quantiser_sweep(dev, hbm),
        "swiglu_gate_up": swiglu_sweep(dev),
        "llama8b_mlp_block": mlp_block_sweep(dev),
        "fp8linear_decode": linear_decode_sweep(dev),
    }

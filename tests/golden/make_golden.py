"""Generate the golden fixtures in this folder from TileGym's own test references.

Run once, in a container that has the TileGym source tree:

    PYTHONPATH=<tilegym>/src:<tilegym> python tests/golden/make_golden.py <tilegym> [family ...]

(with family names, e.g. `group_quant`, only those fixture families are rewritten).

It imports the `reference` static methods of TileGym's test classes
(tests/suites/unsloth/test_fp8.py and
tests/suites/flashinfer/test_flashinfer_gemm_alpha_beta.py) and the torch reference function of
tests/suites/flashinfer/test_per_token_group_quant_8bit.py and
tests/suites/flashinfer/test_flashinfer_ragged_block_scaled_bmm.py, feeds them inputs
drawn the way those tests draw them (same seeds and distributions, on the CPU)
and stores inputs and outputs as compressed .npz files.  fp8 and bf16 tensors
are stored as their raw bit patterns (uint8 / uint16).  The tests in
tests/test_oracle.py load these files and check the CPU oracle against them;
nothing reads the TileGym tree at test time.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def main(ref_root: str, only=()) -> None:
    def want(family: str) -> bool:
        return not only or family in only

    sys.path[:0] = [os.path.join(ref_root, "src"), ref_root]
    from tests.suites.flashinfer.test_flashinfer_gemm_alpha_beta import Test_FlashInfer_Matmul_Alpha_Beta as G
    from tests.suites.unsloth.test_fp8 import Test_Unsloth_ActQuant as Q
    from tests.suites.unsloth.test_fp8 import Test_Unsloth_W8A8_FP8_Matmul as T
    from tests.suites.unsloth.test_fp8 import Test_Unsloth_WeightDequant as W

    # --- block-scaled GEMM: recipe of test_fp8.py:213-222 (seed 42) ---------
    for M, N, K in [(128, 128, 128), (256, 256, 256), (7, 200, 320), (1, 128, 256)] if want("w8a8_block") else []:
        torch.manual_seed(42)
        bn = bk = 128
        A = (torch.randn(M, K) * 0.1).to(torch.float8_e4m3fn)
        B = (torch.randn(N, K) * 0.1).to(torch.float8_e4m3fn)
        As = torch.rand(M, -(-K // bk), dtype=torch.float32) + 0.1
        Bs = torch.rand(-(-N // bn), -(-K // bk), dtype=torch.float32) + 0.1
        C = T.reference(A, B, As, Bs, [bn, bk], torch.float32)
        Cb = T.reference(A, B, As, Bs, [bn, bk], torch.bfloat16)
        np.savez_compressed(
            os.path.join(HERE, f"w8a8_block_{M}x{N}x{K}.npz"),
            A=bits(A), B=bits(B), As=bits(As), Bs=bits(Bs), C_f32=bits(C), C_bf16=bits(Cb),
        )

    # --- act_quant: recipe of test_fp8.py:120-127 (seed 42, bf16 randn) ------
    for shape in [(64, 1024), (128, 384), (4, 128)] if want("act_quant") else []:
        torch.manual_seed(42)
        x = torch.randn(*shape, dtype=torch.bfloat16)
        if shape == (4, 128):
            x[1].zero_()  # all-zero block -> scale 1.0
        y, s = Q.reference(x, block_size=128)
        np.savez_compressed(
            os.path.join(HERE, f"act_quant_{shape[0]}x{shape[1]}.npz"), x=bits(x), y=bits(y), s=bits(s)
        )

    # --- weight_dequant: recipe of test_fp8.py:62-67 (seed 42) ---------------
    for M, N in [(256, 256), (130, 200)] if want("weight_dequant") else []:
        torch.manual_seed(42)
        x = torch.randn(M, N).to(torch.float8_e4m3fn)
        s = torch.rand(-(-M // 128), -(-N // 128), dtype=torch.float32) + 0.1
        y = W.reference(x, s, 128, torch.bfloat16)
        np.savez_compressed(os.path.join(HERE, f"weight_dequant_{M}x{N}.npz"), x=bits(x), s=bits(s), y=bits(y))

    # --- gemm_alpha_beta: recipe of test_flashinfer_gemm_alpha_beta.py:24-66 (seed 0),
    # e4m3 -> bf16, at a size that fits a fixture -----------------------------
    for (m, n, k), (alpha, beta) in ([((256, 256, 256), (1.0, 0.0)), ((256, 256, 256), (1.5, 2.0))]
                                     if want("gemm_alpha_beta") else []):
        torch.manual_seed(0)
        a = torch.rand(m * k, dtype=torch.float16).to(torch.float8_e4m3fn).view(m, k)
        b = torch.rand(k * n, dtype=torch.float16).to(torch.float8_e4m3fn).view(n, k)
        c = torch.rand((m, n), dtype=torch.bfloat16)
        out = G.reference(a, b, c.clone(), False, True, alpha, beta, torch.bfloat16)
        np.savez_compressed(
            os.path.join(HERE, f"gemm_alpha_beta_{m}_{alpha}_{beta}.npz"),
            a=bits(a), b=bits(b), c=bits(c), out=bits(out), alpha=np.float32(alpha), beta=np.float32(beta),
        )
    # --- the same operator on 16-bit operands (the test's (float16 -> float16) and (bfloat16 -> bfloat16) rows,
    # test_flashinfer_gemm_alpha_beta.py:44-53), same recipe, through the same reference ------------------
    for dt, tag in ([(torch.float16, "f16"), (torch.bfloat16, "bf16")] if want("gemm_alpha_beta16") else []):
        m = n = k = 256
        alpha, beta = 1.5, 2.0
        torch.manual_seed(0)
        a = torch.rand(m * k, dtype=torch.float16).to(dt).view(m, k)
        b = torch.rand(k * n, dtype=torch.float16).to(dt).view(n, k)
        c = torch.rand((m, n), dtype=dt)
        out = G.reference(a, b, c.clone(), False, True, alpha, beta, dt)
        as16 = lambda t: t.view(torch.int16).numpy().view(np.uint16)  # noqa: E731  raw bits of either 16-bit type
        np.savez_compressed(
            os.path.join(HERE, f"gemm_alpha_beta_{tag}_{m}_{alpha}_{beta}.npz"),
            a=as16(a), b=as16(b), c=as16(c), out=as16(out), alpha=np.float32(alpha), beta=np.float32(beta),
        )
    # --- per_token_group_quant_8bit: recipe of test_per_token_group_quant_8bit.py:119-133 (seed 0, bf16
    # randn, eps 1e-10) through that file's torch reference; one all-zero group exercises the eps clamp -----
    if want("group_quant"):
        from tests.suites.flashinfer.test_per_token_group_quant_8bit import native_per_token_group_quant_8bit as P

        for T_, H, g, dst, ue in [(33, 256, 16, torch.float8_e4m3fn, False), (33, 256, 128, torch.float8_e4m3fn, True),
                                  (17, 512, 64, torch.int8, False), (17, 512, 32, torch.int8, True),
                                  (9, 256, 128, torch.float8_e5m2, False)]:
            torch.manual_seed(0)
            x = torch.randn(T_, H, dtype=torch.bfloat16)
            x[1, :g].zero_()
            q, sc = P(x, g, 1e-10, dst, ue)
            qb = q.view(torch.uint8).numpy() if dst != torch.int8 else q.numpy()
            name = {torch.float8_e4m3fn: "e4m3", torch.float8_e5m2: "e5m2", torch.int8: "int8"}[dst]
            np.savez_compressed(os.path.join(HERE, f"group_quant_{T_}x{H}_g{g}_{name}_ue{int(ue)}.npz"),
                                x=bits(x), q=qb, s=bits(sc))
    # --- ragged_block_scaled_bmm: input recipe of test_flashinfer_ragged_block_scaled_bmm.py:157-190 (values
    # spread over the e4m3 range, scales rand * 1e-2, 128-aligned segments as its cuTile path needs) on the CPU,
    # through that test class's torch reference ------------------------------------------------------------
    if want("ragged_bmm"):
        from tests.suites.flashinfer.test_flashinfer_ragged_block_scaled_bmm import (
            Test_FlashInfer_RaggedBlockScaledBMM as RB,
        )

        for Q, m, N, K, seed in [(4, 128, 256, 256, 0), (3, 256, 384, 512, 1)]:
            torch.manual_seed(seed)
            total_m = Q * m
            ind = torch.arange(Q + 1, dtype=torch.int32) * m
            a = ((torch.empty(total_m, K).normal_(mean=0.0, std=0.3) - 0.5) * 2 * 448).clamp(-448, 448)
            b = ((torch.empty(Q, N, K).normal_(mean=0.0, std=0.3) - 0.5) * 2 * 448).clamp(-448, 448)
            a, b = a.to(torch.float8_e4m3fn), b.to(torch.float8_e4m3fn)
            sa = torch.rand(total_m, -(-K // 128)) * 1e-2
            sb = torch.rand(Q, -(-N // 128), -(-K // 128)) * 1e-2
            c = RB.reference(a, b, sa, sb, ind, 128, 128, False, True, torch.bfloat16)
            np.savez_compressed(os.path.join(HERE, f"ragged_bmm_q{Q}_m{m}_{N}x{K}.npz"),
                                a=bits(a), b=bits(b), a_scale=bits(sa), b_scale=bits(sb), m_indptr=ind.numpy(),
                                c=bits(c))
    # --- mixture of experts: the operand recipe of the reference test (tests/ops/test_moe.py:112-142: normal(0, 0.5)
    # tokens, normal(0, 0.1) weights, softmax routing weights, random expert ids) at half the width of its smallest
    # shape (:70-76) so that the fixture stays small, block-quantised on the CPU; stored are the quantised
    # operands and (a) the output of the test class's own torch reference (Test_MOE.reference) on the
    # DEQUANTISED fp32 operands, (b) the two stages through tilegym.ops.moe_interface.fused_moe_torch
    # (:82-113) on the same dequantised operands -------------------------------------------------------
    if want("moe"):
        from tests.ops.test_moe import Test_MOE as MOE
        from tilegym.ops.moe_interface import fused_moe_torch

        sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
        from oracle import torch_ref as R

        T_, H, I_, E, topk = 16, 256, 128, 4, 2
        torch.manual_seed(0)
        x = torch.empty(T_, H).normal_(0, 0.5)
        w1 = torch.empty(E, 2 * I_, H).normal_(0, 0.1)
        w2 = torch.empty(E, H, I_).normal_(0, 0.1)
        ids = torch.randint(0, E, (T_, topk), dtype=torch.long)
        wts = torch.softmax(torch.randn(T_, topk), dim=-1)
        a8, a_s = R.ref_act_quant(x, 128)
        q1 = [R.ref_weight_quant_block(w1[e]) for e in range(E)]
        q2 = [R.ref_weight_quant_block(w2[e]) for e in range(E)]
        w1q, w1s = torch.stack([q for q, _ in q1]), torch.stack([s for _, s in q1])
        w2q, w2s = torch.stack([q for q, _ in q2]), torch.stack([s for _, s in q2])
        xd = a8.float() * a_s.repeat_interleave(128, dim=1)
        w1d = torch.stack([R.ref_weight_dequant(w1q[e], w1s[e], 128, torch.float32) for e in range(E)])
        w2d = torch.stack([R.ref_weight_dequant(w2q[e], w2s[e], 128, torch.float32) for e in range(E)])
        full = MOE.reference(xd, w1d, w2d, wts, ids)
        stage1 = fused_moe_torch(xd, w1d, None, wts, ids, False)        # [T, topk, 2 I]
        mid = torch.nn.functional.silu(stage1[..., :I_]) * stage1[..., I_:]
        # second stage of the pipeline: every (token, slot) row is its own "token" with one expert (top_k = 1)
        stage2 = fused_moe_torch(mid.reshape(T_ * topk, I_), w2d, None, wts.reshape(-1, 1), ids.reshape(-1, 1), True)
        np.savez_compressed(
            os.path.join(HERE, f"moe_{T_}x{H}x{I_}_e{E}_k{topk}.npz"),
            a8=bits(a8), a_s=bits(a_s), w1=bits(w1q), w1_s=bits(w1s), w2=bits(w2q), w2_s=bits(w2s),
            ids=ids.numpy(), wts=bits(wts), full_f32=bits(full), stage1_f32=bits(stage1),
            stage2_f32=bits(stage2.reshape(T_, topk, H)),
        )
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path of a TileGym checkout> [fixture family ...]")
    main(sys.argv[1], tuple(sys.argv[2:]))

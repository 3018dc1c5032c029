"""Kernel-level sweep of the training step's pieces, one JSON line per case.

    python -m heirloom_b200.kernel_bench                      # everything
    python -m heirloom_b200.kernel_bench --only gemm          # cases whose name contains "gemm"
    python -m heirloom_b200.kernel_bench --only fc1_fwd --iters 3 --warmup 1   # small run for a profiler
    python -m heirloom_b200.kernel_bench --only gemm --split-k 1   # GEMMs without the even deal of the last wave

Cases: the bf16 GEMM shapes of the GPT-124M-shaped step (forward, input gradient, weight gradient),
causal attention forward/backward (12 heads, head_dim 64 and 128; batch 16 x T 1024 and batch 4 x T 4096), layer norm and
GELU over 16384 x 768 / 16384 x 3072, fused cross-entropy over 16384 x 50304, bias column sums, the fused
AdamW over 124 M and 1.3 G parameters, and the product-key memory layer's kernels at 16384 tokens, 2 x 512 half
keys, 262,144 slots, top-k 32.  Inputs are N(0,1) from torch's generator with seed 0.
Each case reports time from CUDA events on the library's compute stream, the algorithmic work
(flop or bytes) and the fraction of the measured peak (MEASURED_PEAKS.json when present).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from heirloom_b200 import cuda  # noqa: E402

N, D, F, V, B, T, H = 16384, 768, 3072, 50304, 16, 1024, 12
K_, MN = cuda.K_MAJOR, cuda.MN_MAJOR


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timed(ctx, fn, iters, warmup):
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx.sync()
    e0.record(ctx.stream)
    for _ in range(iters):
        fn()
    e1.record(ctx.stream)
    ctx.sync()
    return e0.elapsed_time(e1) / iters


def bf16(*shape):
    return torch.randn(*shape, device="cuda").to(torch.bfloat16)


SPLIT_K = 0  # 0: the library's own work split; 1: whole tiles only; >1: that many equal splits


def gemm_case(ctx, m, n, k, al, bl, out_dtype=torch.bfloat16, epi=cuda.EPI_NONE):
    a = bf16(*((m, k) if al == K_ else (k, m)))
    b = bf16(*((n, k) if bl == K_ else (k, n)))
    out = torch.empty(m, n, dtype=out_dtype, device="cuda")
    bias = torch.zeros(n, device="cuda") if epi in (cuda.EPI_BIAS, cuda.EPI_BIAS_GELU, cuda.EPI_BIAS_RESIDUAL) else None
    aux = bf16(m, n) if epi in (cuda.EPI_BIAS_RESIDUAL, cuda.EPI_DGELU) else None
    want_aux = epi == cuda.EPI_BIAS_GELU
    fn = lambda: cuda.gemm_bf16(ctx, a, b, m, n, k, al, bl, epi, out_dtype, bias, aux, want_aux, split_k=SPLIT_K, out=out)
    return fn, 2.0 * m * n * k, "flop"


def build_cases(ctx):
    cases = {}
    g = lambda *a, **kw: (lambda: gemm_case(ctx, *a, **kw))
    cases["gemm_qkv_fwd"] = g(N, 3 * D, D, K_, K_, epi=cuda.EPI_BIAS)
    cases["gemm_out_proj_fwd"] = g(N, D, D, K_, K_, epi=cuda.EPI_BIAS_RESIDUAL)
    cases["gemm_fc1_fwd"] = g(N, F, D, K_, K_, epi=cuda.EPI_BIAS_GELU)
    cases["gemm_fc2_fwd"] = g(N, D, F, K_, K_, epi=cuda.EPI_BIAS_RESIDUAL)
    cases["gemm_lm_head_fwd"] = g(N, V, D, K_, K_, torch.float32, cuda.EPI_BIAS)
    cases["gemm_lm_head_wgrad"] = g(V, D, N, MN, MN, torch.float32)
    cases["gemm_lm_head_dgrad"] = g(N, D, V, K_, MN, torch.float32)
    cases["gemm_fc2_wgrad"] = g(D, F, N, MN, MN, torch.float32)
    cases["gemm_fc2_dgrad_dgelu"] = g(N, F, D, K_, MN, epi=cuda.EPI_DGELU)
    cases["gemm_fc1_wgrad"] = g(F, D, N, MN, MN, torch.float32)
    cases["gemm_fc1_dgrad"] = g(N, D, F, K_, MN, torch.float32)
    cases["gemm_out_proj_wgrad"] = g(D, D, N, MN, MN, torch.float32)
    cases["gemm_out_proj_dgrad"] = g(N, D, D, K_, MN)
    cases["gemm_qkv_wgrad"] = g(3 * D, D, N, MN, MN, torch.float32)
    cases["gemm_qkv_dgrad"] = g(N, D, 3 * D, K_, MN, torch.float32)
    cases["gemm_4096_768_768"] = g(4096, D, D, K_, K_)

    def attn_fwd():
        qkv = bf16(N, 3 * D)
        q, k, v = qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:]
        return (lambda: cuda.flash_attention_forward(ctx, q, k, v, B, T, H)), 2.0 * B * H * T * T * 64, "flop"

    def attn_bwd():
        qkv = bf16(N, 3 * D)
        q, k, v = qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:]
        out, lse = cuda.flash_attention_forward(ctx, q, k, v, B, T, H)
        do = bf16(N, D)
        return (lambda: cuda.flash_attention_backward(ctx, q, k, v, out, do, lse, B, T, H)), 5.0 * B * H * T * T * 64, "flop"

    def attn_long(backward):
        # the sweep's long-sequence point: batch 16 x T 4096 would be 64 Ki tokens; batch 4 keeps the token count
        # (and the qkv buffer) of the step, the work per (batch, head) is what changes
        b4, t4 = 4, 4096
        def make():
            qkv = bf16(b4 * t4, 3 * D)
            q, k, v = qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:]
            if not backward:
                return (lambda: cuda.flash_attention_forward(ctx, q, k, v, b4, t4, H)), 2.0 * b4 * H * t4 * t4 * 64, "flop"
            out, lse = cuda.flash_attention_forward(ctx, q, k, v, b4, t4, H)
            do = bf16(b4 * t4, D)
            return (lambda: cuda.flash_attention_backward(ctx, q, k, v, out, do, lse, b4, t4, H)), \
                5.0 * b4 * H * t4 * t4 * 64, "flop"
        return make

    def attn_wide(backward, b_, t_):
        # head_dim 128: the same 12 heads, 1536 channels
        hd, C = 128, 12 * 128
        def make():
            qkv = bf16(b_ * t_, 3 * C)
            q, k, v = qkv[:, :C], qkv[:, C:2 * C], qkv[:, 2 * C:]
            if not backward:
                return (lambda: cuda.flash_attention_forward(ctx, q, k, v, b_, t_, H)), 2.0 * b_ * H * t_ * t_ * hd, "flop"
            out, lse = cuda.flash_attention_forward(ctx, q, k, v, b_, t_, H)
            do = bf16(b_ * t_, C)
            return (lambda: cuda.flash_attention_backward(ctx, q, k, v, out, do, lse, b_, t_, H)), \
                5.0 * b_ * H * t_ * t_ * hd, "flop"
        return make

    def ln_wide_fwd():
        x, w, b = bf16(N, F), torch.ones(F, device="cuda"), torch.zeros(F, device="cuda")
        return (lambda: cuda.layer_norm_forward(ctx, x, w, b)), N * F * 4.0, "bytes"

    def adamw_big():
        n = 1_300_000_000
        p, g_, m, v = (torch.empty(n, device="cuda").normal_() for _ in range(4))
        v.abs_()
        hp = cuda.adamw_params(1e-3, 0.9, 0.999, 1e-8, 0.01, 1.0, 1)
        plan = cuda.AdamWPlan(ctx, [p], [g_], [m], [v])  # built once, as an optimizer does
        return (lambda: plan.step(hp)), n * 28.0, "bytes"

    def ln_fwd():
        x, w, b = bf16(N, D), torch.ones(D, device="cuda"), torch.zeros(D, device="cuda")
        return (lambda: cuda.layer_norm_forward(ctx, x, w, b)), N * D * 4.0, "bytes"

    def ln_bwd():
        x, w, b = bf16(N, D), torch.ones(D, device="cuda"), torch.zeros(D, device="cuda")
        _, mean, rstd = cuda.layer_norm_forward(ctx, x, w, b)
        dy, res = torch.randn(N, D, device="cuda"), torch.randn(N, D, device="cuda")
        return (lambda: cuda.layer_norm_backward(ctx, x, w, dy, mean, rstd, res, want_bf16=True, want_colsum=True)), \
            N * D * 16.0, "bytes"

    def gelu_fwd():
        x = bf16(N, F)
        return (lambda: cuda.gelu(ctx, x)), N * F * 4.0, "bytes"

    def ce():
        z = torch.randn(N, V, device="cuda")
        t = torch.randint(0, V, (N,), device="cuda")
        return (lambda: cuda.cross_entropy(ctx, z, t, dlogits_dtype=torch.bfloat16)), N * V * 6.0, "bytes"

    def colsum():
        x = bf16(N, V)
        return (lambda: cuda.bias_grad(ctx, x)), N * V * 2.0, "bytes"

    def adamw():
        n = 124_000_000
        p, g_, m, v = (torch.randn(n, device="cuda") for _ in range(4))
        v.abs_()
        hp = cuda.adamw_params(1e-3, 0.9, 0.999, 1e-8, 0.01, 1.0, 1)
        plan = cuda.AdamWPlan(ctx, [p], [g_], [m], [v])  # built once, as an optimizer does
        return (lambda: plan.step(hp)), n * 28.0, "bytes"

    # product-key memory layer at the memory-transformer sizes: 16384 tokens, 2 x 512 half keys of dimension 256,
    # 262,144 slots, value dimension 512, top-k 32 (beam 32)
    MT, MSIDE, MHALF, MK, MV = 16384, 512, 256, 32, 512

    def mem_inputs():
        q = torch.randn(MT, 2 * MHALF, device="cuda")
        kl = torch.randn(MSIDE, MHALF, device="cuda") / 16.0
        kr = torch.randn(MSIDE, MHALF, device="cuda") / 16.0
        ls, rs = cuda.product_key_side_scores(ctx, q, kl, kr)
        idx = cuda.product_key_topk_from_side_scores(ctx, ls, rs, MK, 32)
        return q, kl, kr, ls, rs, idx

    def mem_side():
        q, kl, kr, *_ = mem_inputs()
        return (lambda: cuda.product_key_side_scores(ctx, q, kl, kr)), 2.0 * 2 * MT * MSIDE * MHALF, "flop"

    def mem_topk():
        _, _, _, ls, rs, _ = mem_inputs()
        return (lambda: cuda.product_key_topk_from_side_scores(ctx, ls, rs, MK, 32)), 2.0 * MT * MSIDE * 4 + MT * MK * 8.0, "bytes"

    def mem_scores_fwd():
        q, kl, kr, _, _, idx = mem_inputs()
        return (lambda: cuda.memory_selected_scores_forward(ctx, idx, q, kl, kr)), MT * MK * 2.0 * MHALF * 4, "bytes"

    def mem_scores_bwd():
        q, kl, kr, _, _, idx = mem_inputs()
        g = torch.randn(MT, MK, device="cuda")
        return (lambda: cuda.memory_selected_scores_backward(ctx, idx, q, kl, kr, g)), MT * MK * 2.0 * MHALF * 4, "bytes"

    def mem_value_fwd():
        _, _, _, _, _, idx = mem_inputs()
        vals = torch.randn(MSIDE * MSIDE, MV, device="cuda") * 0.02
        w = torch.softmax(torch.randn(MT, MK, device="cuda"), dim=1)
        return (lambda: cuda.memory_weighted_value_forward(ctx, idx, w, vals)), MT * MK * MV * 4.0, "bytes"

    def mem_value_bwd():
        _, _, _, _, _, idx = mem_inputs()
        vals = torch.randn(MSIDE * MSIDE, MV, device="cuda") * 0.02
        w = torch.softmax(torch.randn(MT, MK, device="cuda"), dim=1)
        go = torch.randn(MT, MV, device="cuda")
        dv = torch.zeros_like(vals)
        dw = torch.empty_like(w)

        def run():
            cuda.check(ctx.lib.hl_memory_weighted_value_backward(ctx.handle, cuda._p(idx), cuda._p(w), cuda._p(vals), cuda._p(go),
                                                                 cuda._p(dw), cuda._p(dv), MT, MK, MSIDE * MSIDE, MV))
        return run, MT * MK * MV * 4.0 * 3, "bytes"  # value rows read, gradient rows read and written by the atomics

    cases.update(memory_side_scores=mem_side, memory_topk=mem_topk, memory_selected_scores_fwd=mem_scores_fwd,
                 memory_selected_scores_bwd=mem_scores_bwd, memory_weighted_value_fwd=mem_value_fwd,
                 memory_weighted_value_bwd=mem_value_bwd)
    cases.update(attention_fwd_t1024=attn_fwd, attention_bwd_t1024=attn_bwd, layer_norm_fwd=ln_fwd, layer_norm_bwd=ln_bwd,
                 gelu_fwd_16384x3072=gelu_fwd, cross_entropy_16384x50304=ce, bias_colsum_16384x50304=colsum,
                 adamw_124m=adamw, attention_fwd_t4096=attn_long(False), attention_bwd_t4096=attn_long(True),
                 layer_norm_fwd_16384x3072=ln_wide_fwd, adamw_1300m=adamw_big,
                 attention_fwd_t1024_hd128=attn_wide(False, B, T), attention_bwd_t1024_hd128=attn_wide(True, B, T),
                 attention_fwd_t4096_hd128=attn_wide(False, 4, 4096), attention_bwd_t4096_hd128=attn_wide(True, 4, 4096))
    return cases


def sweep(ctx, names=None, iters=20, warmup=3):
    """Runs the named cases (all when None) and yields one result dict per case."""
    hbm, tf, src = peaks()
    for name, make in build_cases(ctx).items():
        if names is not None and name not in names:
            continue
        fn, work, unit = make()
        ms = timed(ctx, fn, iters, warmup)
        if unit == "flop":
            rate, peak, runit = work / ms / 1e9, tf, "TFLOP/s"
        else:
            rate, peak, runit = work / ms / 1e6, hbm, "GB/s"
        yield {"case": name, "us": round(ms * 1e3, 2), "achieved": round(rate, 1), "unit": runit, "peak": peak,
               "frac": round(rate / peak, 4), "peak_source": src}
        del fn
        torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--split-k", type=int, default=0, help="split_k passed to the GEMM cases (1 = whole tiles only)")
    args = ap.parse_args()
    global SPLIT_K
    SPLIT_K = args.split_k
    torch.manual_seed(0)
    ctx = cuda.Context(0)
    names = [n for n in build_cases(ctx) if not args.only or args.only in n]
    for row in sweep(ctx, names, args.iters, args.warmup):
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()

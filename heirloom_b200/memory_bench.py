"""Throughput of the memory-transformer training step on one GPU, one JSON line.

    python -m heirloom_b200.memory_bench [--steps 10] [--warmup 3] [--policy full|sparse_rows]

Model: vocab 32000, d_model 512, 8 layers, 8 heads, MLP 2048, context 512, batch 32; product-key
memory feed-forward in blocks 4 and 6 (2 x 512 half keys of dimension 256 = 262,144 slots, value
dimension 512, top-k 32, one memory head, one shared table set); bf16 compute with f32 master
weights and AdamW state; Zipf(1.1) token ids from a seed; weights N(0, 0.02), half keys
N(0, 1/sqrt(256)).  `full` runs the dense coupled AdamW over every parameter including the tables
(the reference's `Full` policy); `sparse_rows` runs the row-set AdamW over the selected rows of the
three tables only (its `SparseRows` policy).  Times come from CUDA events on the library's compute
stream, per-kernel-family times from the library's event profile.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from heirloom_b200 import cuda, nn  # noqa: E402
from heirloom_b200._lib import Profile  # noqa: E402

CFG = dict(vocab=32000, d_model=512, n_layers=8, n_heads=8, d_ff=2048, context=512)
BATCH = 32
MEM = dict(memory_layers=(4, 6), slots=262144, key_dim=512, value_dim=512, top_k=32)


def flops_per_token() -> float:
    """6 x matmul weights of the dense part + causal attention; the memory lookup is reported in bytes, not flops."""
    d, f, v, layers = CFG["d_model"], CFG["d_ff"], CFG["vocab"], CFG["n_layers"]
    n_mem = len(MEM["memory_layers"])
    p_mm = layers * 4 * d * d + (layers - n_mem) * 2 * d * f + n_mem * 3 * d * d + d * v
    return 6.0 * p_mm + 6.0 * layers * CFG["context"] * d


def init_weights(model, seed: int) -> None:
    rng = np.random.default_rng(seed)
    res = 1.0 / math.sqrt(2.0 * CFG["n_layers"])
    state = {}
    for name, shape in model.parameter_shapes().items():
        if name.endswith(".bias"):
            state[name] = np.zeros(shape, np.float32)
        elif ".ln" in name or name.startswith("ln_f"):
            state[name] = np.ones(shape, np.float32)
        elif "left_keys" in name or "right_keys" in name:
            state[name] = rng.standard_normal(shape, dtype=np.float32) / np.float32(math.sqrt(shape[-1]))
        else:
            w = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
            if "out_proj" in name or "fc2" in name:
                w *= np.float32(res)
            state[name] = w
    model.load_state_dict(state)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--policy", default="full", choices=["full", "sparse_rows"])
    args = ap.parse_args()
    ctx = cuda.Context(0)
    model = nn.DecoderLm(ctx, nn.DecoderConfig(batch=BATCH, **CFG), nn.MemoryConfig(**MEM))
    init_weights(model, 0)
    model.set_optimizer(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, clip_norm=None)
    rng = np.random.default_rng(1000)
    ranks = np.arange(1, CFG["vocab"] + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** -1.1)
    cdf /= cdf[-1]
    pool = []
    for _ in range(4):
        tok = np.minimum(np.searchsorted(cdf, rng.random((BATCH, CFG["context"] + 1)), side="right"), CFG["vocab"] - 1)
        pool.append((torch.from_numpy(tok[:, :-1].copy()).cuda(), torch.from_numpy(tok[:, 1:].copy()).cuda()))

    def step(i):
        x, y = pool[i % len(pool)]
        if args.policy == "full":
            model.train_step_device(x, y)
        else:
            model.forward_backward(x, y)
            model.optimizer_step_sparse_rows()

    for i in range(args.warmup):
        step(i)
    ctx.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ctx.stream)
    for i in range(args.steps):
        step(i)
    e1.record(ctx.stream)
    ctx.sync()
    ms = e0.elapsed_time(e1) / args.steps
    loss = model.loss()
    cuda.check(ctx.lib.hl_profile_enable(ctx.handle, 1))
    prof_steps = min(args.steps, 3)
    for i in range(prof_steps):
        step(i)
    ctx.sync()
    p = Profile()
    cuda.check(ctx.lib.hl_profile_read(ctx.handle, ctypes.byref(p)))
    cuda.check(ctx.lib.hl_profile_enable(ctx.handle, 0))
    names = ["gemm", "attention_fwd", "attention_bwd", "layer_norm", "loss", "optimizer", "bias_grad", "embedding", "other"]
    tokens = BATCH * CFG["context"]
    value = tokens / (ms * 1e-3)
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    burst = json.loads(peaks_path.read_text())["bf16_tflops"] if peaks_path.exists() else 1590.0
    print(json.dumps({
        "metric": "train tokens/s (memory transformer bf16 step)", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "policy": args.policy, "loss_after": loss,
        "config": {"workload": "memory transformer: vocab 32000, d 512, 8 layers, 8 heads, MLP 2048, context 512, batch 32, "
                               "product-key memory in blocks 4 and 6 (262,144 slots, value dim 512, top-k 32)",
                   "tokens_per_step": tokens, "parameters": sum(int(np.prod(s)) for s in model.parameter_shapes().values())},
        "mfu_dense_part": {"flops_per_token": flops_per_token(), "vs_measured_burst": value * flops_per_token() / (burst * 1e12),
                           "vs_datasheet_2250_tflops": value * flops_per_token() / 2250e12},
        "kernel_breakdown_ms_per_step": {n: round(p.ms[i] / prof_steps, 4) for i, n in enumerate(names)},
        "data": "synthetic"}))
    model.close()


if __name__ == "__main__":
    main()

"""Throughput of the memory-transformer training step on one GPU, one JSON line.

    python -m heirloom_b200.memory_bench [--steps 10] [--warmup 3] [--policy full|memory_only|sparse_rows|dense_plus_sparse_values]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m heirloom_b200.memory_bench --gpus N ...          (one rank per GPU, batch 32 per GPU: weak scaling)

Model: vocab 32000, d_model 512, 8 layers, 8 heads, MLP 2048, context 512, batch 32; product-key
memory feed-forward in blocks 4 and 6 (2 x 512 half keys of dimension 256 = 262,144 slots, value
dimension 512, top-k 32, one memory head, one shared table set); bf16 compute with f32 master
weights and AdamW state; Zipf(1.1) token ids from a seed; weights N(0, 0.02), half keys
N(0, 1/sqrt(256)).  `full` runs the dense coupled AdamW over every parameter including the tables
(the reference's `Full` policy); `sparse_rows` runs the row-set AdamW over the selected rows of the
three tables only (its `SparseRows` policy); `memory_only` the dense AdamW over the tables alone;
`dense_plus_sparse_values` the dense AdamW over everything but the value table plus the row-set AdamW over
the selected value rows.  Times come from CUDA events on the library's compute
stream, per-kernel-family times from the library's event profile.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
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
        elif name.endswith("product_key_left") or name.endswith("product_key_right"):
            state[name] = rng.standard_normal(shape, dtype=np.float32) / np.float32(math.sqrt(shape[-1]))
        else:
            w = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
            if "out_proj" in name or "fc2" in name:
                w *= np.float32(res)
            state[name] = w
    model.load_state_dict(state)


def run(ctx, dist, world: int, rank: int, steps: int, warmup: int, policy: str):
    """The memory-transformer step on a context whose communicator (if any) is already set up.  Every rank calls it;
    returns the result line as a dict (the same on every rank up to the per-kernel profile, which is this rank's)."""
    args = argparse.Namespace(steps=steps, warmup=warmup, policy=policy)
    model = nn.DecoderLm(ctx, nn.DecoderConfig(batch=BATCH, **CFG), nn.MemoryConfig(**MEM))
    init_weights(model, 0)  # the same initial weights on every rank
    model.set_optimizer(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, clip_norm=None)
    rng = np.random.default_rng(1000 + rank)  # a distinct token stream per rank
    ranks = np.arange(1, CFG["vocab"] + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** -1.1)
    cdf /= cdf[-1]
    pool = []
    for _ in range(4):
        tok = np.minimum(np.searchsorted(cdf, rng.random((BATCH, CFG["context"] + 1)), side="right"), CFG["vocab"] - 1)
        pool.append((torch.from_numpy(tok[:, :-1].copy()).cuda(), torch.from_numpy(tok[:, 1:].copy()).cuda()))

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    def step(i):
        x, y = pool[i % len(pool)]
        if args.policy == "full":
            model.train_step_device(x, y)
        else:
            model.forward_backward(x, y)
            model.optimizer_step_policy(args.policy)

    for i in range(args.warmup):
        step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ctx.stream)
    for i in range(args.steps):
        step(i)
    e1.record(ctx.stream)
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    if dist is not None:  # the slowest rank sets the step time
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    loss = model.loss()
    cuda.check(ctx.lib.hl_profile_enable(ctx.handle, 1))
    prof_steps = min(args.steps, 3)
    for i in range(prof_steps):
        step(i)
    ctx.sync()
    p = Profile()
    cuda.check(ctx.lib.hl_profile_read(ctx.handle, ctypes.byref(p)))
    cuda.check(ctx.lib.hl_profile_enable(ctx.handle, 0))
    barrier()
    shapes = model.parameter_shapes()
    model.close()
    names = ["gemm", "attention_fwd", "attention_bwd", "layer_norm", "loss", "optimizer", "bias_grad", "embedding", "other"]
    tokens = BATCH * CFG["context"] * world
    value = tokens / (ms * 1e-3)
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    burst = json.loads(peaks_path.read_text())["bf16_tflops"] if peaks_path.exists() else 1590.0
    memory_kernels = p.ms[8] / prof_steps  # the lookup, scoring, gather and table-gradient kernels carry no category of their own
    return ({
        "metric": "train tokens/s (memory transformer bf16 step)", "value": value, "unit": "tokens/s", "n_gpus": world, "scaling": "weak",
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "policy": args.policy, "loss_after": loss,
        "config": {"workload": "memory transformer: vocab 32000, d 512, 8 layers, 8 heads, MLP 2048, context 512, batch 32, "
                               "product-key memory in blocks 4 and 6 (262,144 slots, value dim 512, top-k 32)",
                   "tokens_per_step": tokens, "parameters": sum(int(np.prod(s)) for s in shapes.values())},
        "mfu_dense_part": {"flops_per_token": flops_per_token(),
                           "vs_measured_burst": value * flops_per_token() / (burst * 1e12 * world),
                           "vs_datasheet_2250_tflops": value * flops_per_token() / (2250e12 * world)},
        "kernel_breakdown_ms_per_step": {n: round(p.ms[i] / prof_steps, 4) for i, n in enumerate(names)},
        "memory_kernel_share": memory_kernels / max(sum(p.ms[i] for i in range(len(names))) / prof_steps, 1e-9),
        "data": "synthetic"})


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--policy", default="full", choices=["full", "memory_only", "sparse_rows", "dense_plus_sparse_values"])
    ap.add_argument("--gpus", type=int, default=1)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    ctx = cuda.Context(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)
        ident = (ctypes.c_uint8 * 128)()
        if rank == 0:
            cuda.check(ctx.lib.hl_nccl_unique_id(ident))
        obj = [bytes(ident)]
        dist.broadcast_object_list(obj, src=0)
        ident = (ctypes.c_uint8 * 128).from_buffer_copy(obj[0])
        cuda.check(ctx.lib.hl_nccl_init(ctx.handle, rank, world, ident))
    line = run(ctx, dist, world, rank, args.steps, args.warmup, args.policy)
    if dist is not None:
        cuda.check(ctx.lib.hl_nccl_destroy(ctx.handle))
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


if __name__ == "__main__":
    main()

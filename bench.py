"""Benchmark of the training step (forward + backward + gradient exchange + AdamW).

    python bench.py --gpus N --steps K --warmup W            (N > 1 under torchrun, one rank per GPU)
    python bench.py --impl reference ...                      (the CPU restatement of the reference path)

Workload: the GPT-124M-shaped decoder of the reference's architecture (vocab 50304, d_model 768,
12 layers, 12 heads, MLP 3072, context 1024, micro-batch 16 per GPU; 163.2 M parameters because
the head is untied and every projection has a bias), bf16 compute with f32 master weights and
AdamW state, synthetic Zipf(1.1) token ids, weights N(0, 0.02) with residual projections scaled
by 1/sqrt(2L).  One JSON line on stdout from rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GPT = dict(vocab=50304, d_model=768, n_layers=12, n_heads=12, d_ff=3072, context=1024)
MICRO_BATCH = 16
METRIC = "train tokens/s (GPT-124M-shaped bf16 step)"
DATASHEET_BF16_TFLOPS = 2250.0
# dram__bytes_read.sum + dram__bytes_write.sum per GEMM launch, averaged over the launches of two training steps
# in a one-pass ncu launch list of this command (summary kept under profiles/), and the first 16 hex digits of the
# SHA-256 of the GEMM source the capture ran with: a kernel changed since then gets no traffic figure, not a stale one.
GEMM_DRAM_BYTES_PER_LAUNCH = 153.7e6
GEMM_SOURCE_AT_CAPTURE = "6a10afcb74c80bde"


def gemm_traffic():
    """(bytes per launch or None, note)."""
    import hashlib
    src = ROOT / "heirloom_b200" / "csrc" / "gemm_tcgen05.cu"
    try:
        now = hashlib.sha256(src.read_bytes()).hexdigest()[:16]
    except OSError:
        return None, "GEMM source not found beside the library: capture cannot be matched to it"
    if now != GEMM_SOURCE_AT_CAPTURE:
        return None, "gemm_tcgen05.cu changed since the ncu capture (" + GEMM_SOURCE_AT_CAPTURE + " -> " + now + "): re-capture"
    return GEMM_DRAM_BYTES_PER_LAUNCH, "ncu launch list of this command, profiles/bench_step_launch_list.md"


def flops_per_token(cfg) -> float:
    """6·P_mm + 6·L·T·d: matmul weights only, causal attention counted at T²/2."""
    d, F, L, V, T = cfg["d_model"], cfg["d_ff"], cfg["n_layers"], cfg["vocab"], cfg["context"]
    p_mm = L * (4 * d * d + 2 * d * F) + d * V
    return 6.0 * p_mm + 6.0 * L * T * d


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_batches(n, batch, context, vocab, seed):
    """Zipf(1.1) token ids by inverse-CDF sampling; targets are the next token."""
    import torch
    rng = np.random.default_rng(seed)
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** -1.1)
    cdf /= cdf[-1]
    out = []
    for _ in range(n):
        tok = np.minimum(np.searchsorted(cdf, rng.random((batch, context + 1)), side="right"), vocab - 1)
        x = torch.from_numpy(np.ascontiguousarray(tok[:, :-1]).astype(np.int64)).pin_memory()
        y = torch.from_numpy(np.ascontiguousarray(tok[:, 1:]).astype(np.int64)).pin_memory()
        out.append((x, y))
    return out


def init_weights(model, cfg, seed):
    """N(0, 0.02); out_proj and fc2 scaled by 1/sqrt(2L); biases 0; LayerNorm weight 1."""
    rng = np.random.default_rng(seed)
    res = 1.0 / math.sqrt(2.0 * cfg["n_layers"])
    state = {}
    for name, shape in model.parameter_shapes().items():
        if name.endswith(".bias"):
            state[name] = np.zeros(shape, np.float32)
        elif ".ln" in name or name.startswith("ln_f"):
            state[name] = np.ones(shape, np.float32)
        else:
            w = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
            if "out_proj" in name or "fc2" in name:
                w *= np.float32(res)
            state[name] = w
    model.load_state_dict(state)


def cpu_port_run(sample_tokens=(8, 24)):
    """Times the C++ restatement of the reference's CPU path (f64 loops, scalar backward GEMM, one
    thread: the reference's across-batch threading never engages for rank-2 operands) on a bounded
    slice of the workload: the full 12-layer model and head, forward + backward of one sequence at
    two lengths (which separates the cost per token from the per-step cost that does not depend on
    the batch), and one AdamW step over all parameters.  The tokens/s it returns is the rate of a
    full 16384-token step built from those measurements:
    tokens / (tokens x seconds-per-token + fixed seconds + seconds-per-optimizer-step)."""
    import ctypes
    from oracle import cpp_port
    from oracle import heirloom_oracle as ho
    cfg = ho.DecoderConfig(**GPT)
    lib = cpp_port.load()
    c = cpp_port._cfg(cfg)
    total = int(lib.hr_param_count(ctypes.byref(c)))
    rng = np.random.default_rng(0)
    flat = (rng.standard_normal(total, dtype=np.float32) * np.float32(0.02)).astype(np.float64)
    at = 0
    for name, shape in ho.parameter_shapes(cfg).items():  # LayerNorm weights 1, biases 0
        n = int(np.prod(shape))
        if name.endswith(".bias"):
            flat[at:at + n] = 0.0
        elif ".ln" in name or name.startswith("ln_f"):
            flat[at:at + n] = 1.0
        at += n
    grads = np.zeros(total)
    seconds = []
    for n_tok in sample_tokens:
        tok = ho.zipf_tokens(np.random.default_rng(1), cfg.vocab, (1, n_tok + 1))
        x, y = np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:])
        t0 = time.perf_counter()
        lib.hr_loss_and_grads(ctypes.byref(c), cpp_port._dp(flat), cpp_port._ip(x), cpp_port._ip(y), 1, n_tok, 0, 0,
                              cpp_port._dp(grads))
        seconds.append(time.perf_counter() - t0)
    per_token = (seconds[1] - seconds[0]) / (sample_tokens[1] - sample_tokens[0])
    fixed = max(0.0, seconds[0] - sample_tokens[0] * per_token)
    m, v = np.zeros(total), np.zeros(total)
    t0 = time.perf_counter()
    lib.hr_adamw_step(cpp_port._dp(flat), cpp_port._dp(grads), cpp_port._dp(m), cpp_port._dp(v), total, 1, 1e-3, 0.9,
                      0.999, 1e-8, 0.01, -1.0)
    t_opt = time.perf_counter() - t0
    tokens = MICRO_BATCH * GPT["context"]
    step_s = tokens * per_token + fixed + t_opt
    return dict(value=tokens / step_s, ms_per_step=step_s * 1e3, cores=1,
                sample=f"C++ f64 restatement, 1 thread: forward+backward of 1 sequence of {sample_tokens[0]} and of "
                       f"{sample_tokens[1]} tokens through the full 12-layer model and head ({seconds[0]:.1f} s, "
                       f"{seconds[1]:.1f} s: {per_token:.3f} s per token + {fixed:.1f} s per step) and one AdamW step over "
                       f"all {total} parameters ({t_opt:.1f} s), scaled to the {tokens}-token step; the two-point fit is "
                       f"linear in the tokens, so the attention term that grows with the square of the sequence length "
                       f"(about 8 % of the flops at 1024 tokens) is left out and the CPU time is understated by that much")


def cpu_blas_run(steps, warmup, sample_tokens=256):
    """A second, optimised CPU figure (not the reference's algorithm): the NumPy oracle, whose matrix
    products run on the BLAS threads of the host, on one sequence of `sample_tokens` tokens per step."""
    from oracle import heirloom_oracle as ho
    cfg = ho.DecoderConfig(**GPT)
    params = ho.init_parameters(cfg, 0)
    state = ho.AdamWState()
    rng = np.random.default_rng(1)
    sample_cfg = ho.DecoderConfig(**{**GPT, "context": sample_tokens})
    times = []
    for i in range(warmup + steps):
        tok = ho.zipf_tokens(rng, cfg.vocab, (1, sample_tokens + 1))
        t0 = time.perf_counter()
        ho.train_steps(sample_cfg, params, [(tok[:, :-1], tok[:, 1:])], state, amp_bf16=False)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    per_step = float(np.mean(times))
    return dict(value=sample_tokens / per_step, ms_per_step=per_step * 1e3, cores=os.cpu_count() or 1,
                sample=f"NumPy f64 oracle with BLAS threads, full model, 1 sequence x {sample_tokens} tokens per step, "
                       f"{steps} steps")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = cpu_port_run()
    blas = cpu_blas_run(steps=1, warmup=1)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": 1, "warmup": 0, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "GPT-124M-shaped decoder training step, CPU restatement of the reference path"},
        "cpu_baseline": {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port",
                         "sample": r["sample"]},
        "cpu_optimised": {"value": blas["value"], "unit": "tokens/s", "cores": blas["cores"], "sample": blas["sample"]},
        "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_ours(args):
    import torch
    import torch.distributed as dist

    from heirloom_b200 import cuda, nn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    ctx = cuda.Context(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)
        ident = (ctypes_u8 * 128)()
        if rank == 0:
            cuda.check(ctx.lib.hl_nccl_unique_id(ident))
        obj = [bytes(ident)]
        dist.broadcast_object_list(obj, src=0)
        ident = (ctypes_u8 * 128).from_buffer_copy(obj[0])
        cuda.check(ctx.lib.hl_nccl_init(ctx.handle, rank, world, ident))

    cfg = nn.DecoderConfig(batch=MICRO_BATCH, **GPT)
    model = nn.DecoderLm(ctx, cfg)
    init_weights(model, GPT, seed=0)  # identical initial weights on every rank
    model.set_optimizer(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, clip_norm=None)
    n_pool = 8
    pool = make_batches(n_pool, MICRO_BATCH, GPT["context"], GPT["vocab"], seed=1000 + rank)
    dev_pool = [(x.cuda(non_blocking=True), y.cuda(non_blocking=True)) for x, y in pool]
    ctx.sync()
    tokens_per_step = MICRO_BATCH * GPT["context"] * world

    def barrier():
        ctx.sync()
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident throughput ---------------------------------------------------------------
    for i in range(args.warmup):
        model.train_step_device(*dev_pool[i % n_pool])
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(ctx.stream)
    for i in range(args.steps):
        model.train_step_device(*dev_pool[i % n_pool])
    ev1.record(ctx.stream)
    barrier()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    clocks = sampler.stop() if rank == 0 else None
    launches = model.launches_last_step
    loss_after = model.loss()

    # ---- end to end through the public call: pinned host tokens in, loss out, every step ----------
    for i in range(min(args.warmup, 3)):
        model.train_step(*pool[i % n_pool])
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        model.train_step(*pool[i % n_pool])
    barrier()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)

    # ---- per-kernel timing of one more pass, for the roofline of the dominant kernel --------------
    # Every rank runs these steps (the gradient exchange needs all of them); only rank 0 times them.
    prof, comm = None, None
    prof_steps = min(args.steps, 5)
    if rank == 0:
        cuda.check(ctx.lib.hl_profile_enable(ctx.handle, 1))
    for i in range(prof_steps):
        model.train_step_device(*dev_pool[i % n_pool])
    ctx.sync()
    if rank == 0:
        from heirloom_b200._lib import Profile
        p = Profile()
        cuda.check(ctx.lib.hl_profile_read(ctx.handle, ctypes.byref(p)))
        cuda.check(ctx.lib.hl_profile_enable(ctx.handle, 0))
        names = ["gemm", "attention_fwd", "attention_bwd", "layer_norm", "loss", "optimizer", "bias_grad", "embedding",
                 "other"]
        prof = {n: {"ms_per_step": p.ms[i] / prof_steps, "work_per_step": p.work[i] / prof_steps,
                    "scopes_per_step": p.scopes[i] / prof_steps} for i, n in enumerate(names)}
        exposed_ms, waits = model.comm_exposed_ms()
        comm = {"exposed_ms_per_step": exposed_ms / prof_steps, "waits_per_step": waits / prof_steps,
                "how": "CUDA events around every wait of the compute stream for the collective stream, profiled pass"}
    barrier()

    # ---- replicas stay identical: (sum, sum of squares) of every parameter, compared across the ranks ------------
    # (the reference's drift evidence, src/bin/heirloom/runtime.rs:3403-3416)
    total, total_sq = 0.0, 0.0
    for name in model.parameter_names():
        w = model.parameter(name).astype(np.float64)
        total += float(w.sum())
        total_sq += float((w * w).sum())
    sums = [(total, total_sq)]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, (total, total_sq))
        sums = gathered
    checksum = {"sum": sums[0][0], "sum_of_squares": sums[0][1], "ranks": len(sums),
                "equal_across_ranks": all(s == sums[0] for s in sums)}
    model.close()

    # ---- the memory-transformer configuration at the same number of GPUs (its own JSON object in the line) --------
    memory_line = None
    if not args.no_memory_step:
        from heirloom_b200 import memory_bench
        memory_line = memory_bench.run(ctx, dist if world > 1 else None, world, rank, steps=min(args.steps, 10), warmup=3,
                                       policy="full")
    if world > 1:
        cuda.check(ctx.lib.hl_nccl_destroy(ctx.handle))
        dist.destroy_process_group()

    if rank != 0:
        return
    memory_step = None if memory_line is None else {"ms_per_step": memory_line["ms_per_step"], "tokens_per_s": memory_line["value"], "policy": "full",
                   "n_gpus": world, "memory_kernel_share": memory_line["memory_kernel_share"],
                   "loss_after": memory_line["loss_after"], "config": memory_line["config"]["workload"],
                   "kernel_breakdown_ms_per_step": memory_line["kernel_breakdown_ms_per_step"]}
    kernel_sweep = None
    if world == 1 and not args.no_kernel_sweep:
        # the kernel-level configuration: one figure per piece of the step (all of heirloom_b200.kernel_bench's cases
        # but the 1.3 G-parameter AdamW, which holds 21 GB)
        from heirloom_b200 import kernel_bench
        wanted = [n for n in kernel_bench.build_cases(ctx) if n != "adamw_1300m"]
        kernel_sweep = {r["case"]: {"us": r["us"], "frac": r["frac"], "unit": r["unit"]}
                        for r in kernel_bench.sweep(ctx, wanted, iters=10, warmup=2)}
    peaks = measured_peaks()
    ms_per_step = ms_total / args.steps
    value = tokens_per_step / (ms_per_step * 1e-3)
    e2e_value = tokens_per_step / (e2e_ms / args.steps * 1e-3)
    f_tok = flops_per_token(GPT)
    gemm = prof["gemm"]
    gemm_tflops = gemm["work_per_step"] / (gemm["ms_per_step"] * 1e-3) / 1e12
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        r = cpu_port_run()
        cpu = {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]}
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "GPT-124M-shaped decoder LM training step (vocab 50304, d 768, 12 layers, 12 heads, "
                               "MLP 3072, context 1024, micro-batch 16 per GPU, 163.2M parameters, untied head)",
                   "tokens_per_step": tokens_per_step, "parallelism": f"dp{world}",
                   "l2": "working set per step (>10 GB of activations and 3.3 GB of weights/state) exceeds the 126 MB L2",
                   "loss_after": loss_after},
        "mfu": {"flops_per_token": f_tok, "vs_datasheet_2250_tflops": value * f_tok / (DATASHEET_BF16_TFLOPS * 1e12 * world),
                "vs_measured_burst": value * f_tok / (peaks["bf16_tflops"] * 1e12 * world), "peaks": peaks["source"]},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 2 * 8 * MICRO_BATCH * GPT["context"],
                "d2h_bytes_per_step": 4},
        "gpu_launches": launches * args.steps,
        "roofline": {"bound": "tensor", "kernel": "gemm_bf16_tcgen05_kernel", "achieved": gemm_tflops,
                     "peak": peaks["bf16_sustained"], "unit": "TFLOP/s", "frac": gemm_tflops / peaks["bf16_sustained"],
                     "traffic": gemm_traffic()[0], "traffic_source": gemm_traffic()[1], "peak_source": peaks["source"] + " sustained bf16 (kernel timed inside a long step)",
                     "launches_per_step": gemm["scopes_per_step"], "ms_per_step": gemm["ms_per_step"]},
        "kernel_breakdown_ms_per_step": {k: round(v["ms_per_step"], 4) for k, v in prof.items()},
        "comm": comm,
        "replica_checksum": checksum,
        "memory_step": memory_step,
        "kernel_sweep": kernel_sweep,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line))


if __name__ == "__main__":
    import ctypes
    ctypes_u8 = ctypes.c_ubyte
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernel-sweep", action="store_true")
    ap.add_argument("--no-memory-step", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)

"""Host-side checks of the data-parallel path: bucket arithmetic through the C ABI, and the
sum-then-1/world contract on two gloo ranks (CPU only)."""
import ctypes
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__
    __graft_entry__.build()
    from heirloom_b200 import _lib
    handle = _lib.load()
    handle.hl_ddp_bucket_count.restype = ctypes.c_longlong
    handle.hl_ddp_bucket_count.argtypes = [ctypes.c_longlong, ctypes.c_longlong]
    handle.hl_ddp_ready_buckets.argtypes = [ctypes.c_longlong] * 4 + [ctypes.POINTER(ctypes.c_longlong)] * 2 + [ctypes.c_int]
    return handle


def ready(lib, arena, bucket, nxt, done, cap=64):
    starts, counts = (ctypes.c_longlong * cap)(), (ctypes.c_longlong * cap)()
    n = lib.hl_ddp_ready_buckets(arena, bucket, nxt, done, starts, counts, cap)
    return [(starts[i], counts[i]) for i in range(n)]


def test_bucket_count_and_ranges_cover_the_arena_once(lib):
    arena, bucket = 163_200_000, 6_553_600   # GPT-124M-shaped arena, 25 MiB of f32
    n = lib.hl_ddp_bucket_count(arena, bucket)
    assert n == -(-arena // bucket) == 25
    all_ranges = ready(lib, arena, bucket, 0, arena)
    assert len(all_ranges) == n
    assert all_ranges[0] == (0, bucket) and sum(c for _, c in all_ranges) == arena
    assert all(all_ranges[i][0] + all_ranges[i][1] == all_ranges[i + 1][0] for i in range(n - 1))
    assert all_ranges[-1][1] == arena - (n - 1) * bucket


def test_buckets_become_ready_only_when_wholly_final(lib):
    arena, bucket = 1000, 300
    assert ready(lib, arena, bucket, 0, 299) == []
    assert ready(lib, arena, bucket, 0, 300) == [(0, 300)]
    assert ready(lib, arena, bucket, 1, 650) == [(300, 300)]
    assert ready(lib, arena, bucket, 2, 999) == [(600, 300)]
    assert ready(lib, arena, bucket, 3, 999) == []               # the short tail bucket waits for the end
    assert ready(lib, arena, bucket, 2, 1000) == [(600, 300), (900, 100)]
    assert ready(lib, arena, bucket, 0, 1000, cap=2) == [(0, 300), (300, 300)]
    assert lib.hl_ddp_ready_buckets(0, 300, 0, 0, None, None, 1) == -1


WORKER = r"""
import sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from oracle import heirloom_oracle as ho
rank, world, port = int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
cfg = ho.DecoderConfig(vocab=32, d_model=16, n_layers=1, n_heads=2, d_ff=32, context=8)
params = ho.init_parameters(cfg, 0)                       # identical weights on every rank
state = ho.AdamWState(lr=1e-2, weight_decay=0.01)
rng = np.random.default_rng(100)                          # one global stream, sliced per rank
checks = []
for step in range(3):
    tok = rng.integers(0, cfg.vocab, (2 * world, cfg.context + 1))
    mine = tok[rank * 2:(rank + 1) * 2]
    loss, grads = ho.decoder_loss_and_grads(cfg, params, mine[:, :-1], mine[:, 1:])
    for name in sorted(grads):                            # all-reduce SUM, then scale by 1/world in the update
        t = torch.from_numpy(np.ascontiguousarray(grads[name]))
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        grads[name] = t.numpy()
    ho.adamw_step(params, grads, state, grad_scale=1.0 / world)
    s = sum(float(p.sum()) for p in params.values()); q = sum(float((p * p).sum()) for p in params.values())
    both = torch.tensor([s, q], dtype=torch.float64)
    gathered = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(gathered, both)
    checks.append(max(float((g - both).abs().max()) for g in gathered))
np.save(sys.argv[5] + f".rank{rank}.npy", np.concatenate([params[n].reshape(-1) for n in sorted(params)]))
print("DRIFT", max(checks))
dist.destroy_process_group()
"""


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gloo_ranks_match_one_rank_on_the_global_batch(tmp_path):
    """Sum over ranks then 1/world inside AdamW (src/nn.rs:2100-2117) equals one rank stepping on
    the concatenated batch, and every rank ends with identical parameters (the reference's
    per-step checksum evidence, runtime.rs:3403-3416)."""
    import subprocess
    from oracle import heirloom_oracle as ho
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port, prefix, world = str(_free_port()), str(tmp_path / "params"), 2
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT), str(r), str(world), port, prefix],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    for out in outs:
        drift = float([l for l in out.splitlines() if l.startswith("DRIFT")][0].split()[1])
        assert drift == 0.0
    got = [np.load(prefix + f".rank{r}.npy") for r in range(world)]
    assert np.array_equal(got[0], got[1])
    # single rank on the global batch
    cfg = ho.DecoderConfig(vocab=32, d_model=16, n_layers=1, n_heads=2, d_ff=32, context=8)
    params = ho.init_parameters(cfg, 0)
    state = ho.AdamWState(lr=1e-2, weight_decay=0.01)
    rng = np.random.default_rng(100)
    for _ in range(3):
        tok = rng.integers(0, cfg.vocab, (2 * world, cfg.context + 1))
        _, grads = ho.decoder_loss_and_grads(cfg, params, tok[:, :-1], tok[:, 1:])
        ho.adamw_step(params, grads, state)
    want = np.concatenate([params[n].reshape(-1) for n in sorted(params)])
    assert np.max(np.abs(got[0] - want)) <= 2e-6

"""Two-rank data-parallel step on two GPUs: every rank ends with the same parameters, and they
match one rank stepping on the concatenated batch.  Skipped on a single-GPU box."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu

WORKER = r"""
import ctypes, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
rank, world, port, prefix = int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], sys.argv[5]
from heirloom_b200 import cuda, nn
from oracle import heirloom_oracle as ho
torch.cuda.set_device(rank)
ctx = cuda.Context(rank)
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
ident = (ctypes.c_ubyte * 128)()
if rank == 0:
    cuda.check(ctx.lib.hl_nccl_unique_id(ident))
box = [bytes(ident)]
dist.broadcast_object_list(box, src=0)
ident = (ctypes.c_ubyte * 128).from_buffer_copy(box[0])
cuda.check(ctx.lib.hl_nccl_init(ctx.handle, rank, world, ident))
kw = dict(vocab=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, context=128)
model = nn.DecoderLm(ctx, nn.DecoderConfig(batch=2, **kw))
model.load_state_dict(ho.init_parameters(ho.DecoderConfig(**kw), 0))
model.set_optimizer(lr=1e-3, weight_decay=0.01)
rng = np.random.default_rng(7)
losses = []
for step in range(3):
    tok = ho.zipf_tokens(rng, 512, (2 * world, 129))[rank * 2:(rank + 1) * 2]
    losses.append(model.train_step(torch.tensor(tok[:, :-1].copy()).pin_memory(), torch.tensor(tok[:, 1:].copy()).pin_memory()))
flat = np.concatenate([model.parameter(n).reshape(-1) for n in model.parameter_names()])
np.save(prefix + f".rank{rank}.npy", flat)
calls = ctx.counters().nccl_calls
model.close()
cuda.check(ctx.lib.hl_nccl_destroy(ctx.handle))
dist.destroy_process_group()
print("NCCL_CALLS", calls)
"""


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_ranks_agree_and_match_the_global_batch(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from heirloom_b200 import nn
    from oracle import heirloom_oracle as ho
    from tests.gpu_util import ctx
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port, prefix, world = str(_free_port()), str(tmp_path / "p"), 2
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT), str(r), str(world), port, prefix],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("NCCL_CALLS" in o and int(o.split("NCCL_CALLS")[1].split()[0]) >= 3 for o in outs)
    got = [np.load(prefix + f".rank{r}.npy") for r in range(world)]
    assert np.array_equal(got[0], got[1])  # replicas never drift
    # one rank on the global batch of four sequences
    kw = dict(vocab=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, context=128)
    c = ctx()
    model = nn.DecoderLm(c, nn.DecoderConfig(batch=4, **kw))
    model.load_state_dict(ho.init_parameters(ho.DecoderConfig(**kw), 0))
    model.set_optimizer(lr=1e-3, weight_decay=0.01)
    rng = np.random.default_rng(7)
    for _ in range(3):
        tok = ho.zipf_tokens(rng, 512, (4, 129))
        model.train_step(torch.tensor(tok[:, :-1].copy()).pin_memory(), torch.tensor(tok[:, 1:].copy()).pin_memory())
    want = np.concatenate([model.parameter(n).reshape(-1) for n in model.parameter_names()])
    model.close()
    # same arithmetic up to summation order and bf16 rounding of per-rank partial gradients
    bad = np.abs(got[0] - want) > 2e-2 * np.maximum(np.abs(want), 3e-3)
    assert bad.mean() <= 0.01, bad.mean()

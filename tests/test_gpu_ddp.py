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


MEMORY_WORKER = r"""
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
mem = dict(memory_layers=(1,), slots=1024, key_dim=64, value_dim=128, top_k=8)
ocfg, omem = ho.DecoderConfig(**kw), ho.MemoryConfig(**mem)
model = nn.DecoderLm(ctx, nn.DecoderConfig(batch=2, precision=nn.PRECISION_F32, **kw), nn.MemoryConfig(**mem))
model.load_state_dict(ho.init_memory_parameters(ocfg, omem, 0))
model.set_optimizer(lr=1e-3, weight_decay=0.01)
tok = ho.zipf_tokens(np.random.default_rng(7), 512, (2 * world, 129))[rank * 2:(rank + 1) * 2]
x, y = torch.tensor(tok[:, :-1].copy(), device="cuda"), torch.tensor(tok[:, 1:].copy(), device="cuda")
model.forward_backward(x, y)
np.save(prefix + f".grad{rank}.npy", model.grad("shared_memory.value"))
np.save(prefix + f".gradq{rank}.npy", model.grad("block.1.feed_forward.memory.query_proj.weight"))
np.save(prefix + f".idx{rank}.npy", model.selected_indices(1))
model.optimizer_step_policy(sys.argv[6])
np.save(prefix + f".value{rank}.npy", model.parameter("shared_memory.value"))
np.save(prefix + f".query{rank}.npy", model.parameter("block.1.feed_forward.memory.query_proj.weight"))
np.save(prefix + f".left{rank}.npy", model.parameter("shared_memory.product_key_left"))
model.close()
cuda.check(ctx.lib.hl_nccl_destroy(ctx.handle))
dist.destroy_process_group()
print("DONE")
"""


@pytest.mark.parametrize("policy", ["full", "sparse_rows", "dense_plus_sparse_values", "memory_only"])
def test_memory_model_exchanges_the_union_of_selected_value_rows(tmp_path, policy):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from heirloom_b200 import nn
    from oracle import heirloom_oracle as ho
    from tests.gpu_util import ctx
    script = tmp_path / "worker.py"
    script.write_text(MEMORY_WORKER)
    port, prefix, world = str(_free_port()), str(tmp_path / "m"), 2
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT), str(r), str(world), port, prefix, policy],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    g = [np.load(prefix + f".grad{r}.npy") for r in range(world)]
    assert np.array_equal(g[0], g[1])  # both ranks hold the summed gradient
    assert np.array_equal(np.load(prefix + ".gradq0.npy"), np.load(prefix + ".gradq1.npy"))
    idx = [np.load(prefix + f".idx{r}.npy").reshape(-1) for r in range(world)]
    union = np.union1d(idx[0], idx[1])
    untouched = np.ones(g[0].shape[0], bool); untouched[union] = False
    assert not np.any(g[0][untouched]) and np.any(g[0][union])
    # the summed gradient equals the sum of each rank's own gradient: one rank, each half of the batch in turn
    kw = dict(vocab=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, context=128)
    mem = dict(memory_layers=(1,), slots=1024, key_dim=64, value_dim=128, top_k=8)
    ocfg, omem = ho.DecoderConfig(**kw), ho.MemoryConfig(**mem)
    c = ctx()
    model = nn.DecoderLm(c, nn.DecoderConfig(batch=2, precision=nn.PRECISION_F32, **kw), nn.MemoryConfig(**mem))
    params = ho.init_memory_parameters(ocfg, omem, 0)
    model.load_state_dict(params)
    tok = ho.zipf_tokens(np.random.default_rng(7), 512, (4, 129))
    want = np.zeros_like(g[0], dtype=np.float64)
    for r in range(2):
        part = tok[r * 2:(r + 1) * 2]
        model.forward_backward(torch.tensor(part[:, :-1].copy(), device="cuda"), torch.tensor(part[:, 1:].copy(), device="cuda"))
        want += model.grad("shared_memory.value").astype(np.float64)
        assert np.array_equal(model.selected_indices(1).reshape(-1), idx[r])
    model.close()
    assert np.abs(g[0] - want).max() <= 1e-6 * max(np.abs(want).max(), 1e-12) + 1e-9
    v = [np.load(prefix + f".value{r}.npy") for r in range(world)]
    assert np.array_equal(v[0], v[1]) and np.array_equal(np.load(prefix + ".left0.npy"), np.load(prefix + ".left1.npy"))
    moved = np.any(v[0] != params["shared_memory.value"].astype(np.float32), axis=1)
    if policy in ("sparse_rows", "dense_plus_sparse_values"):
        assert np.array_equal(np.flatnonzero(moved), union)  # exactly the union's rows were updated, on both ranks
    else:
        assert moved[union].all()
    q = [np.load(prefix + f".query{r}.npy") for r in range(world)]
    assert np.array_equal(q[0], q[1])
    dense_moved = np.any(q[0] != params["block.1.feed_forward.memory.query_proj.weight"].astype(np.float32))
    assert dense_moved == (policy in ("full", "dense_plus_sparse_values"))  # the table-only policies leave dense weights alone


TRAIN_STEP_WORKER = r"""
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
mem = dict(memory_layers=(1,), slots=16384, key_dim=64, value_dim=512, top_k=8)
ocfg, omem = ho.DecoderConfig(**kw), ho.MemoryConfig(**mem)
model = nn.DecoderLm(ctx, nn.DecoderConfig(batch=8, precision=nn.PRECISION_F32, **kw), nn.MemoryConfig(**mem))
model.load_state_dict(ho.init_memory_parameters(ocfg, omem, 0))
model.set_optimizer(lr=1e-3, weight_decay=0.01)  # no clip norm: the optimizer consumes the collectives group by group
rng = np.random.default_rng(11)
for step in range(3):
    tok = ho.zipf_tokens(rng, 512, (8 * world, 129))[rank * 8:(rank + 1) * 8]
    x, y = torch.tensor(tok[:, :-1].copy(), device="cuda"), torch.tensor(tok[:, 1:].copy(), device="cuda")
    model.train_step_device(x, y)  # the gradients are never read back between backward and the update
ctx.sync()
np.save(prefix + f".value{rank}.npy", model.parameter("shared_memory.value"))
np.save(prefix + f".tok{rank}.npy", model.parameter("token_embedding.weight"))
np.save(prefix + f".left{rank}.npy", model.parameter("shared_memory.product_key_left"))
model.close()
cuda.check(ctx.lib.hl_nccl_destroy(ctx.handle))
dist.destroy_process_group()
print("DONE")
"""


def test_memory_train_step_without_gradient_readback_keeps_the_value_table_in_step(tmp_path):
    """The whole training step in one call (`full` policy, no clip norm): the AdamW update of the value table has to
    wait for the row exchange that follows the last bucket.  Both ranks end with the same tables, equal to one rank
    stepping on the global batch."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from heirloom_b200 import nn
    from oracle import heirloom_oracle as ho
    from tests.gpu_util import ctx
    script = tmp_path / "worker.py"
    script.write_text(TRAIN_STEP_WORKER)
    port, prefix, world = str(_free_port()), str(tmp_path / "t"), 2
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT), str(r), str(world), port, prefix],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    for name in ("value", "tok", "left"):
        a, b = (np.load(prefix + f".{name}{r}.npy") for r in range(world))
        assert np.array_equal(a, b), name  # replicas never drift
    kw = dict(vocab=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, context=128)
    mem = dict(memory_layers=(1,), slots=16384, key_dim=64, value_dim=512, top_k=8)
    ocfg, omem = ho.DecoderConfig(**kw), ho.MemoryConfig(**mem)
    c = ctx()
    model = nn.DecoderLm(c, nn.DecoderConfig(batch=16, precision=nn.PRECISION_F32, **kw), nn.MemoryConfig(**mem))
    params = ho.init_memory_parameters(ocfg, omem, 0)
    model.load_state_dict(params)
    model.set_optimizer(lr=1e-3, weight_decay=0.01)
    rng = np.random.default_rng(11)
    for _ in range(3):
        tok = ho.zipf_tokens(rng, 512, (16, 129))
        model.train_step_device(torch.tensor(tok[:, :-1].copy(), device="cuda"), torch.tensor(tok[:, 1:].copy(), device="cuda"))
    want = model.parameter("shared_memory.value").astype(np.float64)
    model.close()
    got = np.load(prefix + ".value0.npy").astype(np.float64)
    start = params["shared_memory.value"].astype(np.float64)
    touched = np.any(np.abs(want - start) > 1e-4, axis=1)
    assert touched.sum() > 100
    # the mean over the global batch is the average of the ranks' means; only the f32 summation order differs, which
    # AdamW's normalised step amplifies where a gradient element is close to zero
    bad = np.abs(got - want) > 2e-4
    assert bad.mean() <= 1e-3, bad.mean()

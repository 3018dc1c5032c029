"""Step-level parity on the shapes the benchmark configurations name, not on reduced models.

Two kinds of check.  (1) One step of one sequence against the oracle's restatement at the full model size: vocabulary
50304 / width 768 / 12 blocks / context 1024 for the dense decoder, 262,144 memory slots with 512 x 512 half keys for
the memory transformer.  (2) The full micro-batch against a property that does not need the oracle: the loss is a mean
over tokens and no op mixes sequences, so loss and every gradient of the whole batch equal the average over its
parts.  The batch sizes differ by a power of two, so every bf16 rounding point commutes with the 1/N scaling and only
the f32 summation order is left.  The whole-batch run is the one that reaches the paths that exist only at that size:
the panel tile order of the large GEMMs, k blocks dealt out over the CTAs, split-K weight gradients, the row-ordered
value backward.
"""
import numpy as np
import pytest
import torch

from oracle import heirloom_oracle as ho
from tests.gpu_util import ctx

pytestmark = pytest.mark.gpu

GPT = dict(vocab=50304, d_model=768, n_layers=12, n_heads=12, d_ff=3072, context=1024)
MEMORY_LM = dict(vocab=32000, d_model=512, n_layers=8, n_heads=8, d_ff=2048, context=512)
MEMORY = dict(memory_layers=(4, 6), slots=262144, key_dim=512, value_dim=512, top_k=32)


def _grad_report(model, names, want, skip=("attention.k_proj.bias",)):
    worst = {}
    for name in names:
        if any(name.endswith(s) for s in skip):
            continue
        g, w = model.grad(name).astype(np.float64), np.asarray(want[name], np.float64)
        scale = np.abs(w).max() + 1e-30
        worst[name] = (np.abs(g - w).max() / scale, np.abs(g - w).mean() / scale)
    return worst


def test_gpt_shape_one_sequence_matches_the_amp_oracle():
    from heirloom_b200 import nn
    c = ctx()
    ocfg = ho.DecoderConfig(**GPT)
    params = ho.init_parameters(ocfg, 0)
    model = nn.DecoderLm(c, nn.DecoderConfig(batch=1, **GPT))
    model.load_state_dict(params)
    tok = ho.zipf_tokens(np.random.default_rng(3), ocfg.vocab, (1, GPT["context"] + 1))
    x, y = tok[:, :-1].copy(), tok[:, 1:].copy()
    model.forward_backward(torch.tensor(x, device="cuda"), torch.tensor(y, device="cuda"))
    loss = model.loss()
    oloss, ograds = ho.decoder_loss_and_grads(ocfg, params, x, y, amp_bf16=True)
    assert abs(loss - oloss) <= 2e-3 * abs(oloss), (loss, oloss)
    worst = _grad_report(model, ho.parameter_names(ocfg), ograds)
    model.close()
    print("gpt-shape gradient deviation (max, mean of |g-w|/max|w|):",
          max(v[0] for v in worst.values()), max(v[1] for v in worst.values()))
    bad = {n: v for n, v in worst.items() if v[0] > 0.06 or v[1] > 0.01}
    assert not bad, bad


def test_gpt_shape_full_batch_equals_the_average_of_its_sequences():
    from heirloom_b200 import nn
    c = ctx()
    ocfg = ho.DecoderConfig(**GPT)
    params = ho.init_parameters(ocfg, 1)
    B = 16
    tok = ho.zipf_tokens(np.random.default_rng(5), ocfg.vocab, (B, GPT["context"] + 1))
    x, y = torch.tensor(tok[:, :-1].copy(), device="cuda"), torch.tensor(tok[:, 1:].copy(), device="cuda")
    names = [n for n in ho.parameter_names(ocfg) if not n.endswith("attention.k_proj.bias")]
    # a sample of the tensors that come out of every kind of kernel, at both ends and the middle of the stack
    probe = [n for n in names if n.startswith(("lm_head", "ln_f", "token_embedding", "position_embedding", "block.0.",
                                               "block.6.", "block.11."))]
    whole = nn.DecoderLm(c, nn.DecoderConfig(batch=B, **GPT))
    whole.load_state_dict(params)
    whole.forward_backward(x, y)
    loss_whole = whole.loss()
    got = {n: whole.grad(n).astype(np.float64) for n in probe}
    whole.close()
    part = nn.DecoderLm(c, nn.DecoderConfig(batch=2, **GPT))
    part.load_state_dict(params)
    mean = {n: np.zeros_like(got[n]) for n in probe}
    losses = []
    for b in range(0, B, 2):
        part.forward_backward(x[b:b + 2].contiguous(), y[b:b + 2].contiguous())
        losses.append(part.loss())
        for n in probe:
            mean[n] += part.grad(n).astype(np.float64) / (B // 2)
    part.close()
    assert abs(loss_whole - np.mean(losses)) <= 2e-6 * abs(loss_whole), (loss_whole, np.mean(losses))
    worst = 0.0
    for n in probe:
        scale = np.abs(mean[n]).max() + 1e-30
        dev = np.abs(got[n] - mean[n]).max() / scale
        worst = max(worst, dev)
        # f32 sums in another order (the attention backward adds its dQ tiles in arrival order), which moves a few bf16
        # roundings downstream by one step; measured worst 1.5e-3
        assert dev <= 4e-3, (n, dev)
    print("gpt-shape whole batch vs parts, worst |g-mean|/max|mean|:", worst)


def test_memory_shape_one_sequence_matches_the_oracle_with_identical_routing():
    from heirloom_b200 import nn
    c = ctx()
    ocfg, omem = ho.DecoderConfig(**MEMORY_LM), ho.MemoryConfig(**MEMORY)
    params = ho.init_memory_parameters(ocfg, omem, 0)
    model = nn.DecoderLm(c, nn.DecoderConfig(batch=1, precision=nn.PRECISION_F32, **MEMORY_LM), nn.MemoryConfig(**MEMORY))
    model.load_state_dict(params)
    tok = ho.zipf_tokens(np.random.default_rng(7), ocfg.vocab, (1, MEMORY_LM["context"] + 1))
    x, y = tok[:, :-1].copy(), tok[:, 1:].copy()
    model.forward_backward(torch.tensor(x, device="cuda"), torch.tensor(y, device="cuda"))
    oloss, ograds, oidx = ho.memory_decoder_loss_and_grads(ocfg, omem, params, x, y, return_indices=True)
    assert abs(model.loss() - oloss) <= 1e-6 * abs(oloss), (model.loss(), oloss)
    for layer in MEMORY["memory_layers"]:
        assert np.array_equal(model.selected_indices(layer), oidx[layer]), layer   # both blocks share one table set
    worst = _grad_report(model, ho.memory_parameter_names(ocfg, omem), ograds)
    model.close()
    print("memory-shape f32 gradient deviation, worst |g-w|/max|w|:", max(v[0] for v in worst.values()))
    bad = {n: v for n, v in worst.items() if v[0] > 5e-6}
    assert not bad, bad


def test_memory_shape_full_batch_equals_the_average_of_its_parts():
    from heirloom_b200 import nn
    c = ctx()
    ocfg, omem = ho.DecoderConfig(**MEMORY_LM), ho.MemoryConfig(**MEMORY)
    params = ho.init_memory_parameters(ocfg, omem, 2)
    B, part_b = 32, 8
    tok = ho.zipf_tokens(np.random.default_rng(9), ocfg.vocab, (B, MEMORY_LM["context"] + 1))
    x, y = torch.tensor(tok[:, :-1].copy(), device="cuda"), torch.tensor(tok[:, 1:].copy(), device="cuda")
    names = [n for n in ho.memory_parameter_names(ocfg, omem) if not n.endswith("attention.k_proj.bias")]
    probe = [n for n in names if n.startswith(("shared_memory", "lm_head.bias", "ln_f", "position_embedding", "block.4.",
                                               "block.6.", "block.7.", "block.0.ln1"))]
    whole = nn.DecoderLm(c, nn.DecoderConfig(batch=B, **MEMORY_LM), nn.MemoryConfig(**MEMORY))
    whole.load_state_dict(params)
    whole.forward_backward(x, y)
    loss_whole = whole.loss()
    got = {n: whole.grad(n).astype(np.float64) for n in probe}
    idx_whole = {l: whole.selected_indices(l).reshape(B, -1) for l in MEMORY["memory_layers"]}
    whole.close()
    part = nn.DecoderLm(c, nn.DecoderConfig(batch=part_b, **MEMORY_LM), nn.MemoryConfig(**MEMORY))
    part.load_state_dict(params)
    mean = {n: np.zeros_like(got[n]) for n in probe}
    losses = []
    for b in range(0, B, part_b):
        part.forward_backward(x[b:b + part_b].contiguous(), y[b:b + part_b].contiguous())
        losses.append(part.loss())
        for l in MEMORY["memory_layers"]:  # routing is per token: the same slots whatever the batch around it
            assert np.array_equal(part.selected_indices(l).reshape(part_b, -1), idx_whole[l][b:b + part_b]), (l, b)
        for n in probe:
            mean[n] += part.grad(n).astype(np.float64) / (B // part_b)
    part.close()
    assert abs(loss_whole - np.mean(losses)) <= 2e-6 * abs(loss_whole), (loss_whole, np.mean(losses))
    worst = 0.0
    for n in probe:
        scale = np.abs(mean[n]).max() + 1e-30
        dev = np.abs(got[n] - mean[n]).max() / scale
        worst = max(worst, dev)
        assert dev <= 4e-3, (n, dev)  # measured worst 1.8e-3
    print("memory-shape whole batch vs parts, worst |g-mean|/max|mean|:", worst)

"""The C++ CPU restatement against the NumPy oracle (independent code, same ops) and against the
committed loss trace.  Both are test infrastructure; neither is on any product path."""
import json
import time
from pathlib import Path

import numpy as np
import pytest

from oracle import cpp_port
from oracle import heirloom_oracle as ho
from tests.golden.make_tiny_trace import BATCH, CONFIG, TOKEN_SEED, WEIGHT_SEED


def _small():
    cfg = ho.DecoderConfig(vocab=48, d_model=32, n_layers=2, n_heads=4, d_ff=64, context=12)
    params = ho.init_parameters(cfg, 5)
    # non-trivial biases and norm weights so that every gradient path carries signal
    rng = np.random.default_rng(6)
    for n in params:
        if n.endswith(".bias"):
            params[n] = ho.f32_round(rng.standard_normal(params[n].shape) * 0.05)
        elif ".ln" in n or n.startswith("ln_f"):
            params[n] = ho.f32_round(1.0 + rng.standard_normal(params[n].shape) * 0.05)
    tok = rng.integers(0, cfg.vocab, (3, cfg.context + 1))
    return cfg, params, tok


@pytest.mark.parametrize("amp,grad_f32", [(False, False), (False, True), (True, False)])
def test_loss_and_every_gradient_match_the_numpy_oracle(amp, grad_f32):
    cfg, params, tok = _small()
    want_loss, want = ho.decoder_loss_and_grads(cfg, params, tok[:, :-1], tok[:, 1:], amp_bf16=amp, grad_f32=grad_f32)
    got_loss, got = cpp_port.loss_and_grads(cfg, params, tok[:, :-1], tok[:, 1:], amp_bf16=amp, grad_f32=grad_f32)
    assert got_loss == pytest.approx(want_loss, rel=1e-7)
    # f64 mode: only summation order differs.  With f32/bf16 rounding inside the backward a sum that lands on a
    # rounding boundary can flip one unit in the last place of the rounded type, so those modes get that slack.
    rel = 1e-9 if not (amp or grad_f32) else (2e-2 if amp else 1e-5)
    for name in ho.parameter_names(cfg):
        if name.endswith("k_proj.bias"):
            # mathematically zero (softmax is shift-invariant along a query row): both sides hold rounding noise only
            assert np.abs(got[name]).max() < 1e-6 and np.abs(want[name]).max() < 1e-6
            continue
        scale = max(np.abs(want[name]).max(), 1e-30)
        err = np.abs(got[name] - want[name]).max() / scale
        assert err <= rel, (name, err)


def test_three_training_steps_follow_the_committed_trace():
    trace = json.loads((Path(__file__).parent / "golden" / "tiny_decoder_trace.json").read_text())
    cfg = ho.DecoderConfig(**CONFIG)
    params = ho.init_parameters(cfg, WEIGHT_SEED)
    rng = np.random.default_rng(TOKEN_SEED)
    batches = np.stack([rng.integers(0, CONFIG["vocab"], (BATCH, CONFIG["context"] + 1)) for _ in range(3)])
    t0 = time.perf_counter()
    losses, _ = cpp_port.train_steps(cfg, params, batches)
    elapsed = time.perf_counter() - t0
    assert np.allclose(losses, trace["losses"][:3], rtol=1e-7, atol=0), (losses, trace["losses"][:3])
    assert elapsed < 120


def test_adamw_step_matches_the_numpy_oracle_including_clipping():
    rng = np.random.default_rng(9)
    p = ho.f32_round(rng.standard_normal(257))
    g = rng.standard_normal(257) * 3.0
    state = ho.AdamWState(lr=0.05, weight_decay=0.01, clip_norm=1.0)
    params = {"w": p.copy()}
    flat, m, v = p.copy(), np.zeros(257), np.zeros(257)
    lib = cpp_port.load()
    for step in (1, 2, 3):
        ho.adamw_step(params, {"w": g}, state)
        lib.hr_adamw_step(cpp_port._dp(flat), cpp_port._dp(g), cpp_port._dp(m), cpp_port._dp(v), 257, step, 0.05, 0.9,
                          0.999, 1e-8, 0.01, 1.0)
        assert np.array_equal(flat, params["w"]), step

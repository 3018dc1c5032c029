"""The committed tiny-decoder loss trace is what the oracle produces (first steps re-run here)."""
import json
from pathlib import Path

import numpy as np

from oracle import heirloom_oracle as ho
from tests.golden.make_tiny_trace import BATCH, CONFIG, WEIGHT_SEED, batches


def test_first_steps_of_the_committed_trace_reproduce():
    trace = json.loads((Path(__file__).parent / "golden" / "tiny_decoder_trace.json").read_text())
    cfg = ho.DecoderConfig(**CONFIG)
    params = ho.init_parameters(cfg, WEIGHT_SEED)
    state = ho.AdamWState(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
    losses = ho.train_steps(cfg, params, batches(4), state)
    assert np.allclose(losses, trace["losses"][:4], rtol=1e-7, atol=0)
    assert len(trace["losses"]) == 200 and trace["batch"] == BATCH
    # uniform random bytes: the loss stays near ln(256)
    assert abs(trace["losses"][-1] - np.log(256)) < 0.05


def test_amp_and_f32_oracle_modes_agree_within_bf16_tolerance():
    cfg = ho.DecoderConfig(vocab=64, d_model=32, n_layers=1, n_heads=2, d_ff=64, context=16)
    params = ho.init_parameters(cfg, 2)
    rng = np.random.default_rng(3)
    tok = rng.integers(0, 64, (2, 17))
    l32, g32 = ho.decoder_loss_and_grads(cfg, params, tok[:, :-1], tok[:, 1:])
    l16, g16 = ho.decoder_loss_and_grads(cfg, params, tok[:, :-1], tok[:, 1:], amp_bf16=True)
    assert abs(l32 - l16) <= 1e-2 * l32
    for n in ("lm_head.weight", "block.0.feed_forward.dense.fc1.weight"):
        assert np.abs(g32[n] - g16[n]).max() <= 0.1 * np.abs(g32[n]).max()


def test_first_steps_of_the_committed_amp_trace_reproduce():
    from tests.golden import make_amp_trace as mt
    trace = json.loads((Path(__file__).parent / "golden" / "amp_decoder_trace.json").read_text())
    assert trace["config"] == mt.CONFIG and trace["steps"] == mt.STEPS == len(trace["losses"]) and trace["batch"] == mt.BATCH
    cfg = ho.DecoderConfig(**mt.CONFIG)
    params = ho.init_parameters(cfg, mt.WEIGHT_SEED)
    state = ho.AdamWState(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
    losses = ho.train_steps(cfg, params, mt.batches(3), state, amp_bf16=True)
    assert np.allclose(losses, trace["losses"][:3], rtol=1e-6, atol=0)
    # Zipf(1.1) streams: the loss falls by well over a nat within the 200 steps, so the trace discriminates
    assert trace["losses"][0] > 6.0 and trace["losses"][-1] < 4.6

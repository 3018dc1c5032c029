"""Generates `amp_decoder_trace.json`: the oracle's 200-step loss trace of a reduced decoder on the amp-bf16 route
(vocab 512, d_model 128, 2 layers, 2 heads of 64, MLP 256, context 128, batch 4; Zipf(1.1) token streams, a fresh
batch every step, so the loss falls from ln 512 towards the entropy of the stream; weights N(0, 0.02) with scaled
residual projections; AdamW lr 1e-3, betas (0.9, 0.999), eps 1e-8, wd 0.01, no clipping).

The trace is what the reference's AMP route computes under the oracle's restatement: bf16 operands with f32
accumulation in every Linear and in attention, every round-trip point of src/memory_transformer.rs:1153-1172 and
:1636-1662 rounded to bf16, f32 gradients, f64 AdamW moments.  Takes about a minute on CPU.

Usage: python tests/golden/make_amp_trace.py
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import heirloom_oracle as ho  # noqa: E402

CONFIG = dict(vocab=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, context=128)
BATCH, STEPS, WEIGHT_SEED, TOKEN_SEED = 4, 200, 2, 3


def batches(steps):
    rng = np.random.default_rng(TOKEN_SEED)
    for _ in range(steps):
        tok = ho.zipf_tokens(rng, CONFIG["vocab"], (BATCH, CONFIG["context"] + 1))
        yield tok[:, :-1].copy(), tok[:, 1:].copy()


def main():
    cfg = ho.DecoderConfig(**CONFIG)
    params = ho.init_parameters(cfg, WEIGHT_SEED)
    state = ho.AdamWState(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
    losses = ho.train_steps(cfg, params, batches(STEPS), state, amp_bf16=True)
    out = {"config": CONFIG, "batch": BATCH, "steps": STEPS, "weight_seed": WEIGHT_SEED, "token_seed": TOKEN_SEED,
           "route": "amp_bf16", "losses": losses}
    dest = Path(__file__).with_name("amp_decoder_trace.json")
    dest.write_text(json.dumps(out, indent=1) + "\n")
    print("wrote", dest, losses[0], losses[-1])


if __name__ == "__main__":
    main()

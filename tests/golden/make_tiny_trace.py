"""Generates `tiny_decoder_trace.json`: the oracle's 200-step loss trace for the tiny byte-level
decoder (vocab 256, d_model 128, 4 layers, 4 heads, MLP 512, context 64, batch 16; tokens uniform
over [0, 256); weights N(0, 0.02); AdamW lr 1e-3, betas (0.9, 0.999), eps 1e-8, wd 0.01).

The trace is what the reference's CPU path computes under the oracle's restatement (f64 compute,
f32-rounded op outputs, f64 gradients and AdamW moments).  Takes about a minute on CPU.

Usage: python tests/golden/make_tiny_trace.py
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import heirloom_oracle as ho  # noqa: E402

CONFIG = dict(vocab=256, d_model=128, n_layers=4, n_heads=4, d_ff=512, context=64)
BATCH, STEPS, WEIGHT_SEED, TOKEN_SEED = 16, 200, 0, 1


def batches(steps):
    rng = np.random.default_rng(TOKEN_SEED)
    for _ in range(steps):
        tok = rng.integers(0, CONFIG["vocab"], (BATCH, CONFIG["context"] + 1))
        yield tok[:, :-1].copy(), tok[:, 1:].copy()


def main():
    cfg = ho.DecoderConfig(**CONFIG)
    params = ho.init_parameters(cfg, WEIGHT_SEED)
    state = ho.AdamWState(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
    losses = ho.train_steps(cfg, params, batches(STEPS), state)
    checksum = {n: [float(p.sum()), float((p * p).sum())] for n, p in params.items() if n in
                ("token_embedding.weight", "block.0.attention.q_proj.weight", "block.3.feed_forward.dense.fc2.weight",
                 "lm_head.weight", "ln_f.weight")}
    out = {"config": CONFIG, "batch": BATCH, "steps": STEPS, "weight_seed": WEIGHT_SEED, "token_seed": TOKEN_SEED,
           "losses": losses, "final_parameter_sum_and_sumsq": checksum}
    dest = Path(__file__).with_name("tiny_decoder_trace.json")
    dest.write_text(json.dumps(out, indent=1) + "\n")
    print("wrote", dest, losses[0], losses[-1])


if __name__ == "__main__":
    main()

"""Evaluation and generation around the device model, with the reference's sampling controls.

`HeirloomRng` is the reference's SplitMix64 stream (src/rng.rs:29-45); `sample_token` and its filters
follow src/nn.rs:1595-1751 statement by statement (repetition, frequency and presence penalties,
temperature, top-k, top-p, greedy at temperature 0); `evaluate_token_loss` walks the token stream in
windows of `context` tokens like src/memory_transformer.rs:1813-1912; `generate` is
src/memory_transformer.rs:1730-1769.  The model work (full-window forward, loss) runs on the GPU
through `hl_decoder_eval_loss` / `hl_decoder_next_token_logits`; sampling is host arithmetic over one
row of logits, as in the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ._lib import HeirloomError

_MASK = (1 << 64) - 1


class HeirloomRng:
    def __init__(self, seed: int):
        self.state = seed & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return z ^ (z >> 31)

    def uniform_f32(self) -> float:
        return float(np.float32(self.next_u64() >> 40) / np.float32(1 << 24))


@dataclass
class GenerationOptions:
    max_new_tokens: int
    eos_id: int
    temperature: float = 0.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0

    @staticmethod
    def greedy(max_new_tokens: int, eos_id: int) -> "GenerationOptions":
        return GenerationOptions(max_new_tokens, eos_id)

    def validate(self) -> None:
        if self.temperature < 0.0:
            raise HeirloomError(f"temperature must be non-negative, got {self.temperature}")
        if self.top_k is not None and self.top_k == 0:
            raise HeirloomError("top_k must be greater than zero when set")
        if self.top_p is not None and not (0.0 < self.top_p <= 1.0):
            raise HeirloomError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.repetition_penalty < 1.0:
            raise HeirloomError(f"repetition_penalty must be at least 1.0, got {self.repetition_penalty}")
        if self.frequency_penalty < 0.0 or self.presence_penalty < 0.0:
            raise HeirloomError("frequency_penalty and presence_penalty must be non-negative, got "
                                f"{self.frequency_penalty}/{self.presence_penalty}")


@dataclass
class GeneratedTokenStep:
    token_id: int
    probability: float
    log_probability: float


@dataclass
class GenerationOutput:
    tokens: List[int]
    new_token_count: int
    finish_reason: str  # "max_new_tokens" or "eos"
    rng_state: int
    steps: List[GeneratedTokenStep] = field(default_factory=list)


@dataclass
class LmEvalMetrics:
    batches: int
    examples: int
    tokens: int
    loss: float
    perplexity: float


def softmax_logits(logits: np.ndarray) -> np.ndarray:
    finite = np.isfinite(logits)
    if not finite.any():
        p = np.zeros(len(logits))
        if len(logits):
            p[0] = 1.0
        return p
    mx = logits[finite].max()
    p = np.where(finite, np.exp(np.where(finite, logits, mx) - mx), 0.0)
    s = 0.0
    for v in p:  # the reference accumulates in index order
        s += v
    return p if s == 0.0 else p / s


def argmax_filtered(values: np.ndarray) -> int:
    """Last maximal index under a total order, as `max_by(total_cmp)` returns it."""
    if len(values) == 0:
        return 0
    best = 0
    for i in range(1, len(values)):
        if not (values[i] < values[best]):  # later ties win
            best = i
    return best


def _apply_repetition_controls(logits: np.ndarray, context: Sequence[int], o: GenerationOptions) -> None:
    counts = {}
    for t in context:
        if t < len(logits):
            counts[t] = counts.get(t, 0) + 1
    for t, count in counts.items():
        if o.repetition_penalty > 1.0:
            logits[t] = logits[t] / o.repetition_penalty if logits[t] > 0.0 else logits[t] * o.repetition_penalty
        logits[t] -= o.frequency_penalty * count
        logits[t] -= o.presence_penalty


def _descending_stable(values: np.ndarray) -> np.ndarray:
    return np.argsort(-values, kind="stable")  # stable sort by descending value, like sort_by(total_cmp)


def sampling_filter(logits: np.ndarray, o: GenerationOptions) -> np.ndarray:
    keep = np.ones(len(logits), bool)
    if o.top_k is not None:
        keep[:] = False
        keep[_descending_stable(logits)[:min(o.top_k, len(logits))]] = True
    if o.top_p is not None and o.top_p < 1.0:
        probs = softmax_logits(np.where(keep, logits, -np.inf))
        keep[:] = False
        cumulative = 0.0
        for t in _descending_stable(probs):
            if probs[t] == 0.0:
                continue
            keep[t] = True
            cumulative += probs[t]
            if cumulative >= o.top_p:
                break
    if keep.any():
        return keep
    fallback = np.zeros(len(logits), bool)
    fallback[argmax_filtered(logits)] = True
    return fallback


def sample_token(logits: Sequence[float], context: Sequence[int], o: GenerationOptions,
                 rng: HeirloomRng) -> Tuple[int, float, float]:
    adjusted = np.asarray(logits, np.float64).copy()
    _apply_repetition_controls(adjusted, context, o)
    if o.temperature > 0.0:
        adjusted /= o.temperature
    keep = sampling_filter(adjusted, o)
    adjusted[~keep] = -np.inf
    probs = softmax_logits(adjusted)
    tiny = np.finfo(np.float64).tiny
    if o.temperature == 0.0:
        t = argmax_filtered(adjusted)
        return t, float(probs[t]), math.log(max(float(probs[t]), tiny))
    draw = rng.uniform_f32()
    cumulative = 0.0
    for t, p in enumerate(probs):
        cumulative += p
        if draw <= cumulative:
            return t, float(p), math.log(max(float(p), tiny))
    t = argmax_filtered(adjusted)
    return t, float(probs[t]), math.log(max(float(probs[t]), tiny))


def next_token_logits(model, tokens: Sequence[int]) -> np.ndarray:
    """Logits of the token after `tokens`, from the last `context` of them."""
    if len(tokens) == 0:
        raise HeirloomError("next_token_logits requires at least one token")
    window = np.asarray(tokens[-model.cfg.context:], np.int64)
    out = model.next_token_logits_device(torch.from_numpy(window).cuda())
    if not np.isfinite(out).all():
        raise HeirloomError("non-finite generation logits")
    return out.astype(np.float64)


def generate(model, prefix: Sequence[int], options: GenerationOptions, rng: HeirloomRng) -> GenerationOutput:
    options.validate()
    if len(prefix) == 0:
        raise HeirloomError("generation prefix must contain at least one token")
    tokens = list(int(t) for t in prefix)
    steps: List[GeneratedTokenStep] = []
    reason = "max_new_tokens"
    for _ in range(options.max_new_tokens):
        token, p, logp = sample_token(next_token_logits(model, tokens), tokens, options, rng)
        tokens.append(token)
        steps.append(GeneratedTokenStep(token, p, logp))
        if token == options.eos_id:
            reason = "eos"
            break
    return GenerationOutput(tokens, len(steps), reason, rng.state, steps)


def generate_greedy(model, prefix: Sequence[int], max_new_tokens: int, eos_id: int) -> List[int]:
    return generate(model, prefix, GenerationOptions.greedy(max_new_tokens, eos_id), HeirloomRng(0)).tokens


def evaluate_token_loss(model, tokens: Sequence[int], batch_size: int, max_batches: Optional[int] = None) -> LmEvalMetrics:
    block = model.cfg.context
    if batch_size == 0:
        raise HeirloomError("eval batch_size must be greater than zero")
    if batch_size > model.cfg.batch:
        raise HeirloomError(f"eval batch_size {batch_size} exceeds the batch the model was created for ({model.cfg.batch})")
    if max_batches is not None and max_batches == 0:
        raise HeirloomError("max_batches must be greater than zero when set")
    if len(tokens) <= block:
        raise HeirloomError(f"eval needs more than block_size tokens, got {len(tokens)} tokens and block_size {block}")
    stream = np.asarray(tokens, np.int64)
    offset = batches = examples = predicted = 0
    loss_sum = 0.0
    while offset + block < len(stream):
        if max_batches is not None and batches >= max_batches:
            break
        rows_in, rows_tg = [], []
        while len(rows_in) < batch_size and offset + block < len(stream):
            rows_in.append(stream[offset:offset + block])
            rows_tg.append(stream[offset + 1:offset + block + 1])
            offset += block
        if not rows_in:
            break
        loss = model.eval_loss_device(torch.from_numpy(np.stack(rows_in)).cuda(), torch.from_numpy(np.stack(rows_tg)).cuda())
        if not math.isfinite(loss):
            raise HeirloomError(f"non-finite eval loss: {loss}")
        weight = len(rows_in) * block
        loss_sum += loss * weight
        predicted += weight
        examples += len(rows_in)
        batches += 1
    if predicted == 0:
        raise HeirloomError("eval produced zero predicted tokens")
    loss = loss_sum / predicted
    return LmEvalMetrics(batches, examples, predicted, loss, math.exp(loss))

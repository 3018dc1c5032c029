"""CPU restatement of Heirloom's training-step arithmetic (TEST INFRASTRUCTURE ONLY).

This module is the parity oracle: a NumPy float64 restatement of the reference's CPU
path for the transformer training step.  It is never imported by the product package;
only tests, the smoke check and the benchmark's CPU-baseline leg may use it.

Numeric rules restated from the reference (paths are relative to the reference tree):

* every CPU op reads its inputs as f64, computes in f64 and rounds its *output* to f32
  (`src/tensor.rs:577-590`, `:5179-5191`);
* gradients stay f64 through the whole backward and reach AdamW as f64; AdamW moments are
  f64 and the parameter is rounded to f32 after the update (`src/nn.rs:2433-2465`);
* cross-entropy is the mean over all rows (`src/tensor.rs:4816-4882`);
* ties in every arg-sort go to the lower index (`src/tensor.rs:641-702`).

Pinning: `tests/test_oracle_golden.py` checks these functions against the reference's own
golden vectors (`tests/fixtures/pytorch_parity.json`, tolerance 2e-5 as in
`tests/pytorch_fixture_parity.rs:111-126`) and the known-answer tests in
`tests/memory_transformer.rs`.  No golden vector exists in the reference for a whole
training step; step-level parity rests on this restatement alone.

The forward matmul of the reference goes through the third-party crate `matrixmultiply`
0.3.10 (`Cargo.lock:531-532`, call site `heirloom-kernels/src/lib.rs:78-95`), which is not
vendored.  Its f64 summation order differs from BLAS/NumPy by a few ulp(f64), invisible
after the f32 output rounding except at exact rounding boundaries.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

F32 = np.float32
F64 = np.float64


# --------------------------------------------------------------------------------------
# dtype helpers
# --------------------------------------------------------------------------------------
def f32_round(x) -> np.ndarray:
    """f64 -> f32 -> f64: the rounding every CPU op applies to its output
    (`src/tensor.rs:5179-5191`)."""
    return np.asarray(x, dtype=F64).astype(F32).astype(F64)


def f32_to_bf16_bits(x) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit pattern (`src/storage.rs:440-445`:
    bias `0x7fff + lsb`, NaN quieted)."""
    bits = np.asarray(x, dtype=F32).view(np.uint32).astype(np.uint64)
    lsb = (bits >> 16) & 1
    rounded = ((bits + 0x7FFF + lsb) >> 16).astype(np.uint16)
    is_nan = np.isnan(np.asarray(x, dtype=F32))
    if np.any(is_nan):
        quiet = ((bits >> 16) | 0x0040).astype(np.uint16)
        rounded = np.where(is_nan, quiet, rounded)
    return rounded


def bf16_bits_to_f32(bits) -> np.ndarray:
    """bf16 bit pattern -> f32 (`src/storage.rs:447-449`)."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(F32)


def bf16_round(x) -> np.ndarray:
    """f32 -> bf16 -> f32 round trip, returned as f64 (`src/nn.rs:250-261`)."""
    return bf16_bits_to_f32(f32_to_bf16_bits(np.asarray(x, dtype=F64).astype(F32))).astype(F64)


# --------------------------------------------------------------------------------------
# forward ops (f64 compute, f32-rounded outputs) and their f64 backward formulas
# --------------------------------------------------------------------------------------
def add(a, b):
    """Broadcast add (`src/dispatch.rs:542-569`)."""
    return f32_round(np.asarray(a, F64) + np.asarray(b, F64))


def unbroadcast(grad: np.ndarray, shape: Sequence[int]) -> np.ndarray:
    """Sum a broadcast gradient back to `shape` (`src/tensor/autograd.rs:1960-2010`)."""
    g = np.asarray(grad, F64)
    while g.ndim > len(shape):
        g = g.sum(axis=0)
    for axis, dim in enumerate(shape):
        if dim == 1 and g.shape[axis] != 1:
            g = g.sum(axis=axis, keepdims=True)
    return g


def matmul(a, b):
    """`Tensor::matmul` on CPU (`src/tensor.rs:2809-2842`, kernel `src/dispatch.rs:571-677`)."""
    return f32_round(np.matmul(np.asarray(a, F64), np.asarray(b, F64)))


def matmul_backward(a, b, grad_out):
    """dA = dY·Bᵀ, dB = Aᵀ·dY in f64 (`src/tensor/autograd.rs:2012-2104`)."""
    a = np.asarray(a, F64)
    b = np.asarray(b, F64)
    g = np.asarray(grad_out, F64)
    ga = np.matmul(g, np.swapaxes(b, -1, -2))
    gb = np.matmul(np.swapaxes(a, -1, -2), g)
    return unbroadcast(ga, a.shape), unbroadcast(gb, b.shape)


def relu(x):
    return f32_round(np.maximum(np.asarray(x, F64), 0.0))


def relu_backward(x, grad_out):
    return np.where(np.asarray(x, F64) > 0.0, np.asarray(grad_out, F64), 0.0)


_GELU_C = math.sqrt(2.0 / math.pi)


def gelu_value(x: np.ndarray) -> np.ndarray:
    """tanh-approximate GELU in f64 (`src/tensor.rs:5152-5154`)."""
    x = np.asarray(x, F64)
    return 0.5 * x * (1.0 + np.tanh(_GELU_C * (x + 0.044715 * x * x * x)))


def gelu(x):
    """`Tensor::gelu` (`src/tensor.rs:3118-3145`)."""
    return f32_round(gelu_value(x))


def gelu_backward(x, grad_out):
    """Analytic derivative (`src/tensor/autograd.rs:2144-2156`, `:2891-2897`)."""
    x = np.asarray(x, F64)
    inner = _GELU_C * (x + 0.044715 * x * x * x)
    t = np.tanh(inner)
    sech2 = 1.0 - t * t
    d_inner = _GELU_C * (1.0 + 3.0 * 0.044715 * x * x)
    return np.asarray(grad_out, F64) * (0.5 * (1.0 + t) + 0.5 * x * sech2 * d_inner)


def layer_norm(x, weight, bias, eps: float = 1e-5):
    """`Tensor::layer_norm_last_dim`: biased variance, rstd = 1/sqrt(var+eps)
    (`src/tensor.rs:3175-3256`)."""
    x = np.asarray(x, F64)
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    return f32_round((x - mean) * rstd * np.asarray(weight, F64) + np.asarray(bias, F64))


def layer_norm_backward(x, weight, grad_out, eps: float = 1e-5):
    """dx, dγ, dβ (`src/tensor/autograd.rs:2158-2232`)."""
    x = np.asarray(x, F64)
    w = np.asarray(weight, F64)
    g = np.asarray(grad_out, F64)
    feat = x.shape[-1]
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    xhat = (x - mean) * rstd
    dxhat = g * w
    s1 = dxhat.sum(axis=-1, keepdims=True)
    s2 = (dxhat * xhat).sum(axis=-1, keepdims=True)
    dx = rstd * (feat * dxhat - s1 - xhat * s2) / feat
    dw = (g * xhat).reshape(-1, feat).sum(axis=0)
    db = g.reshape(-1, feat).sum(axis=0)
    return dx, dw, db


def embedding(weight, indices):
    """`out[n,:] = W[idx[n],:]` (`src/tensor.rs:3337-3395`)."""
    return f32_round(np.asarray(weight, F64)[np.asarray(indices, np.int64)])


def embedding_backward(weight_shape, indices, grad_out):
    """Scatter-add; repeated indices accumulate (`src/tensor/autograd.rs:2234-2261`)."""
    gw = np.zeros(weight_shape, F64)
    idx = np.asarray(indices, np.int64).reshape(-1)
    np.add.at(gw, idx, np.asarray(grad_out, F64).reshape(idx.shape[0], -1))
    return gw


def softmax_data(x, axis: int = -1):
    """max-subtracted softmax in f64 (`src/tensor/autograd.rs:2858-2889`)."""
    x = np.asarray(x, F64)
    m = x.max(axis=axis, keepdims=True)
    e = np.exp(x - m)
    return e / e.sum(axis=axis, keepdims=True)


def softmax(x, axis: int = -1):
    """`Tensor::softmax_dim` (`src/tensor.rs:4521-4602`)."""
    return f32_round(softmax_data(x, axis))


def softmax_backward(probs, grad_out, axis: int = -1):
    """`dx = p·(g − Σ g·p)` (`src/tensor/autograd.rs:2512-2543`)."""
    p = np.asarray(probs, F64)
    g = np.asarray(grad_out, F64)
    return p * (g - (g * p).sum(axis=axis, keepdims=True))


def cross_entropy(logits, targets):
    """Mean over rows of `−z[y] + max + ln Σ exp(z − max)` (`src/tensor.rs:4816-4882`)."""
    z = np.asarray(logits, F64)
    t = np.asarray(targets, np.int64)
    m = z.max(axis=1)
    lse = m + np.log(np.exp(z - m[:, None]).sum(axis=1))
    total = (-z[np.arange(z.shape[0]), t] + lse).sum()
    return f32_round(total / z.shape[0])


def cross_entropy_backward(logits, targets, grad_out=1.0):
    """`dz = (softmax − onehot)·g/N` (`src/tensor/autograd.rs:2591-2621`)."""
    z = np.asarray(logits, F64)
    t = np.asarray(targets, np.int64)
    p = softmax_data(z, axis=1)
    p[np.arange(z.shape[0]), t] -= 1.0
    return p * (float(grad_out) / z.shape[0])


def causal_attention(q, k, v, n_heads: int, return_probs: bool = False, round_probs_bf16: bool = False):
    """`Tensor::causal_self_attention`: q,k,v `[B,T,C]` with heads interleaved along C
    (`index = b·T·C + t·C + h·hd + j`), scale 1/sqrt(hd), causal softmax, output `[B,T,C]`
    (`src/tensor.rs:3980-4098`, indexers `:5156-5177`).

    `round_probs_bf16` restates the tensor-core AMP route, where P is fed to the PV
    product as a bf16 operand (`src/tensor.rs:4100-4402`)."""
    q = np.asarray(q, F64)
    B, T, C = q.shape
    hd = C // n_heads
    qh = q.reshape(B, T, n_heads, hd).transpose(0, 2, 1, 3)
    kh = np.asarray(k, F64).reshape(B, T, n_heads, hd).transpose(0, 2, 1, 3)
    vh = np.asarray(v, F64).reshape(B, T, n_heads, hd).transpose(0, 2, 1, 3)
    s = np.matmul(qh, kh.transpose(0, 1, 3, 2)) * (1.0 / math.sqrt(hd))
    mask = np.tril(np.ones((T, T), bool))
    s = np.where(mask, s, -np.inf)
    p = softmax_data(s, axis=-1)
    p_used = bf16_round(p) if round_probs_bf16 else p
    o = np.matmul(p_used, vh).transpose(0, 2, 1, 3).reshape(B, T, C)
    out = f32_round(o)
    if return_probs:
        return out, p
    return out


def causal_attention_backward(q, k, v, n_heads: int, grad_out, probs=None, bf16_operands: bool = False):
    """dQ, dK, dV from saved P (`src/tensor/autograd.rs:2623-2712`).

    With `bf16_operands` the backward products use bf16-rounded dO and P/dS operands as the
    reference's tensor-core route does (`src/tensor/autograd.rs:1626-1914`)."""
    q = np.asarray(q, F64)
    B, T, C = q.shape
    hd = C // n_heads
    scale = 1.0 / math.sqrt(hd)
    split = lambda x: np.asarray(x, F64).reshape(B, T, n_heads, hd).transpose(0, 2, 1, 3)
    merge = lambda x: x.transpose(0, 2, 1, 3).reshape(B, T, C)
    qh, kh, vh, go = split(q), split(k), split(v), split(grad_out)
    if probs is None:
        s = np.matmul(qh, kh.transpose(0, 1, 3, 2)) * scale
        s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
        probs = softmax_data(s, axis=-1)
    p = probs
    if bf16_operands:
        go = bf16_round(go)
        p_op = bf16_round(p)
    else:
        p_op = p
    dv = np.matmul(p_op.transpose(0, 1, 3, 2), go)
    dp = np.matmul(go, vh.transpose(0, 1, 3, 2))
    ds = p * (dp - (dp * p).sum(axis=-1, keepdims=True)) * scale
    ds_op = bf16_round(ds) if bf16_operands else ds
    dq = np.matmul(ds_op, kh)
    dk = np.matmul(ds_op.transpose(0, 1, 3, 2), qh)
    return merge(dq), merge(dk), merge(dv)


# --------------------------------------------------------------------------------------
# memory-layer ops
# --------------------------------------------------------------------------------------
def topk_indices_dim1(scores, k: int) -> np.ndarray:
    """Per-row top-k of stored f32 scores: descending score, ties to the lower index
    (`src/tensor.rs:641-702`)."""
    s = np.asarray(scores, F32)
    rows, cols = s.shape
    out = np.empty((rows, k), np.int64)
    for r in range(rows):
        # stable sort on the negated score keeps the lower index first among equals
        order = np.argsort(-s[r].astype(F64), kind="stable")
        out[r] = order[:k]
    return out


def sequential_dot_f32(q_row: np.ndarray, k_row: np.ndarray) -> np.float32:
    """`acc = acc + (q[j]*k[j])` with separately rounded f32 multiply and add
    (`src/memory_transformer.rs:2029-2034`)."""
    acc = F32(0.0)
    for j in range(q_row.shape[0]):
        acc = F32(acc + F32(q_row[j] * k_row[j]))
    return acc


def side_scores_f32(query_half: np.ndarray, half_keys: np.ndarray) -> np.ndarray:
    """All side scores `[tokens, side]` with the sequential f32 dot, vectorised over
    (token, key) but sequential over the contraction index."""
    q = np.asarray(query_half, F32)
    k = np.asarray(half_keys, F32)
    acc = np.zeros((q.shape[0], k.shape[0]), F32)
    for j in range(q.shape[1]):
        prod = (q[:, j : j + 1] * k[:, j][None, :]).astype(F32)
        acc = (acc + prod).astype(F32)
    return acc


def product_key_beam(side: int, top_k: int) -> int:
    """beam = min(side, max(top_k, ceil(sqrt(top_k)))) (`src/memory_transformer.rs:2014-2016`)."""
    return min(side, max(top_k, int(math.ceil(math.sqrt(top_k)))))


def product_key_indices_from_side_scores(left: np.ndarray, right: np.ndarray, top_k: int, beam: int) -> np.ndarray:
    """Top-`beam` per side (desc score, asc index), beam² f32 sums, then top-k by
    (desc sum, asc slot) (`src/memory_transformer.rs:847-924`, `:2004-2043`; expected-index
    helper `tests/memory_transformer.rs:73-176`)."""
    left = np.asarray(left, F32)
    right = np.asarray(right, F32)
    tokens, side = left.shape
    out = np.empty((tokens, top_k), np.int64)
    for t in range(tokens):
        lo = np.argsort(-left[t].astype(F64), kind="stable")[:beam]
        ro = np.argsort(-right[t].astype(F64), kind="stable")[:beam]
        sums = (left[t, lo][:, None] + right[t, ro][None, :]).astype(F32)
        slots = lo[:, None] * side + ro[None, :]
        flat_scores = sums.reshape(-1).astype(F64)
        flat_slots = slots.reshape(-1)
        order = np.lexsort((flat_slots, -flat_scores))
        out[t] = flat_slots[order[:top_k]]
    return out


def product_key_split_rows(rows, side: int) -> Tuple[np.ndarray, np.ndarray]:
    """`row / side`, `row % side` (`src/tensor.rs:1654-1719`)."""
    r = np.asarray(rows, np.int64)
    return r // side, r % side


def product_key_selected_scores(indices, query, left_keys, right_keys):
    """`score = q_L·K_L[slot/side] + q_R·K_R[slot%side]` (`src/tensor.rs:3593-3769`)."""
    idx = np.asarray(indices, np.int64)
    q = np.asarray(query, F64)
    kl = np.asarray(left_keys, F64)
    kr = np.asarray(right_keys, F64)
    side, half = kl.shape
    li, ri = idx // side, idx % side
    s = np.einsum("td,tkd->tk", q[:, :half], kl[li]) + np.einsum("td,tkd->tk", q[:, half:], kr[ri])
    return f32_round(s)


def product_key_selected_scores_backward(indices, query, left_keys, right_keys, grad_scores):
    """dq, dK_L, dK_R (`src/tensor/autograd.rs:2386-2494`)."""
    idx = np.asarray(indices, np.int64)
    q = np.asarray(query, F64)
    kl = np.asarray(left_keys, F64)
    kr = np.asarray(right_keys, F64)
    g = np.asarray(grad_scores, F64)
    side, half = kl.shape
    li, ri = idx // side, idx % side
    dq = np.concatenate(
        [np.einsum("tk,tkd->td", g, kl[li]), np.einsum("tk,tkd->td", g, kr[ri])], axis=1
    )
    dkl = np.zeros_like(kl)
    dkr = np.zeros_like(kr)
    np.add.at(dkl, li.reshape(-1), (g[:, :, None] * q[:, None, :half]).reshape(-1, half))
    np.add.at(dkr, ri.reshape(-1), (g[:, :, None] * q[:, None, half:]).reshape(-1, half))
    return dq, dkl, dkr


def memory_selected_scores(indices, query, keys):
    """Exact-lookup twin: `score[t,k] = q[t]·K[idx[t,k]]` (`src/tensor.rs:3465-3548`)."""
    idx = np.asarray(indices, np.int64)
    return f32_round(np.einsum("td,tkd->tk", np.asarray(query, F64), np.asarray(keys, F64)[idx]))


def memory_selected_scores_backward(indices, query, keys, grad_scores):
    """dq and dK with repeats accumulating (`src/tensor/autograd.rs:2325-2384`)."""
    idx = np.asarray(indices, np.int64)
    q = np.asarray(query, F64)
    k = np.asarray(keys, F64)
    g = np.asarray(grad_scores, F64)
    dq = np.einsum("tk,tkd->td", g, k[idx])
    dk = np.zeros_like(k)
    np.add.at(dk, idx.reshape(-1), (g[:, :, None] * q[:, None, :]).reshape(-1, q.shape[1]))
    return dq, dk


def memory_weighted_value(indices, weights, values):
    """`out[t,:] = Σ_k w[t,k]·V[idx[t,k],:]` (`src/tensor.rs:3771-3900`)."""
    idx = np.asarray(indices, np.int64)
    return f32_round(np.einsum("tk,tkd->td", np.asarray(weights, F64), np.asarray(values, F64)[idx]))


def memory_weighted_value_backward(indices, weights, values, grad_out):
    """dw = dot(dout, V row); dV scatter-add (`src/tensor/autograd.rs:2263-2323`)."""
    idx = np.asarray(indices, np.int64)
    w = np.asarray(weights, F64)
    v = np.asarray(values, F64)
    g = np.asarray(grad_out, F64)
    dw = np.einsum("td,tkd->tk", g, v[idx])
    dv = np.zeros_like(v)
    np.add.at(dv, idx.reshape(-1), (w[:, :, None] * g[:, None, :]).reshape(-1, v.shape[1]))
    return dw, dv


# --------------------------------------------------------------------------------------
# AdamW (coupled decay)
# --------------------------------------------------------------------------------------
@dataclass
class AdamWState:
    """`AdamWState` (`src/nn.rs:1927-1937`)."""

    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.01
    clip_norm: Optional[float] = None
    step: int = 0
    m: Dict[str, np.ndarray] = field(default_factory=dict)
    v: Dict[str, np.ndarray] = field(default_factory=dict)


def clip_scale(grads: Sequence[np.ndarray], clip_norm: Optional[float]) -> float:
    """`max_norm/(‖g‖+1e-12)` if the global norm exceeds `max_norm` else 1
    (`src/nn.rs:2589-2665`)."""
    if clip_norm is None:
        return 1.0
    sum_sq = float(sum((np.asarray(g, F64) ** 2).sum() for g in grads))
    norm = math.sqrt(sum_sq)
    return clip_norm / (norm + 1e-12) if norm > clip_norm else 1.0


def adamw_step(params: Dict[str, np.ndarray], grads: Dict[str, np.ndarray], state: AdamWState,
               grad_scale: float = 1.0) -> None:
    """One coupled-decay AdamW step in f64 with f32-rounded parameters
    (`src/nn.rs:2156-2220`, body `:2433-2465`).  Parameters without a gradient are skipped.
    `grad_scale` restates the data-parallel `1/world` factor applied to summed gradients
    before the step (`src/nn.rs:2100-2117`)."""
    present = [grads[n] * grad_scale for n in params if n in grads and grads[n] is not None]
    clip = clip_scale(present, state.clip_norm)
    state.step += 1
    bias1 = 1.0 - state.beta1 ** state.step
    bias2 = 1.0 - state.beta2 ** state.step
    for name, p in params.items():
        g = grads.get(name)
        if g is None:
            continue
        g = np.asarray(g, F64) * grad_scale
        if name not in state.m:
            state.m[name] = np.zeros_like(p, dtype=F64)
            state.v[name] = np.zeros_like(p, dtype=F64)
        decayed = g * clip + state.weight_decay * p
        state.m[name] = state.beta1 * state.m[name] + (1.0 - state.beta1) * decayed
        state.v[name] = state.beta2 * state.v[name] + (1.0 - state.beta2) * decayed * decayed
        m_hat = state.m[name] / bias1
        v_hat = state.v[name] / bias2
        params[name] = f32_round(p - state.lr * m_hat / (np.sqrt(v_hat) + state.eps))


def adamw_step_f32_kernel_order(p, g, m, v, lr, beta1, beta2, eps, wd, clip, bias1, bias2):
    """The reference's CUDA kernel arithmetic in f32 with its exact operation order and no
    fused multiply-add (`heirloom-kernels/src/ptx/kernels.ptx:441-467`).  Returns p', m', v'."""
    p = np.asarray(p, F32); g = np.asarray(g, F32); m = np.asarray(m, F32); v = np.asarray(v, F32)
    lr, beta1, beta2, eps, wd, clip, bias1, bias2 = (F32(x) for x in (lr, beta1, beta2, eps, wd, clip, bias1, bias2))
    one = F32(1.0)
    gd = (g * clip).astype(F32) + (p * wd).astype(F32)
    gd = gd.astype(F32)
    m2 = ((beta1 * m).astype(F32) + ((one - beta1) * gd).astype(F32)).astype(F32)
    v2 = ((beta2 * v).astype(F32) + ((one - beta2) * (gd * gd).astype(F32)).astype(F32)).astype(F32)
    mh = (m2 / bias1).astype(F32)
    vh = (v2 / bias2).astype(F32)
    upd = (mh / (np.sqrt(vh).astype(F32) + eps).astype(F32)).astype(F32)
    p2 = (p - (lr * upd).astype(F32)).astype(F32)
    return p2, m2, v2


def active_sparse_rows(selected_rows, rows: int, row_mask=None) -> np.ndarray:
    """The *set* of selected rows in first-occurrence order, optionally filtered by a bool
    row mask (`src/nn.rs:2899-2939`)."""
    seen = set()
    out = []
    for r in np.asarray(selected_rows, np.int64).reshape(-1).tolist():
        if r < 0 or r >= rows:
            raise ValueError(f"selected row {r} out of range for {rows} rows")
        if r in seen:
            continue
        seen.add(r)
        if row_mask is not None and not bool(row_mask[r]):
            continue
        out.append(r)
    return np.asarray(out, np.int64)


def adamw_sparse_rows_step(param: np.ndarray, grad: np.ndarray, m: np.ndarray, v: np.ndarray,
                           selected_rows, state: AdamWState, row_mask=None, clip: float = 1.0,
                           bump_step: bool = True) -> np.ndarray:
    """AdamW restricted to the set of selected rows; duplicates update once and every call
    increments the step counter (`src/nn.rs:2256-2323`, CPU body `:2507-2540`)."""
    if bump_step:
        state.step += 1
    bias1 = 1.0 - state.beta1 ** state.step
    bias2 = 1.0 - state.beta2 ** state.step
    rows = active_sparse_rows(selected_rows, param.shape[0], row_mask)
    p = np.asarray(param, F64).copy()
    for r in rows:
        decayed = grad[r] * clip + state.weight_decay * p[r]
        m[r] = state.beta1 * m[r] + (1.0 - state.beta1) * decayed
        v[r] = state.beta2 * v[r] + (1.0 - state.beta2) * decayed * decayed
        p[r] = p[r] - state.lr * (m[r] / bias1) / (np.sqrt(v[r] / bias2) + state.eps)
    return f32_round(p)


def smft_mask_against(foreground_counts, background_counts, trainable_fraction: float, min_rows: int):
    """TF-IDF ranking of the rows a foreground count set touched against a background set
    (`src/memory_transformer.rs:273-327`; order `:2045-2055`): score = (fg / max(sum fg, 1)) *
    ln((max(sum bg, 1) + slots) / (bg + 1)); descending score, then descending fg, ascending bg, ascending
    row; the first max(ceil(unique * fraction), min(min_rows, unique)) rows are trainable.  Returns
    `(trainable_rows, [(row, score), ...])` with the scores in rank order."""
    fg = np.asarray(foreground_counts, np.uint64).astype(F64)
    bg = np.asarray(background_counts, np.uint64).astype(F64)
    if fg.shape != bg.shape:
        raise ValueError("SMFT foreground/background memory_slots mismatch")
    slots = max(fg.size, 1)
    touched = np.flatnonzero(fg > 0)
    tf = fg[touched] / max(fg.sum(), 1.0)
    idf = np.array([math.log((max(bg.sum(), 1.0) + slots) / (b + 1.0)) for b in bg[touched]], F64)
    score = tf * idf
    # lexsort: last key is the primary one
    order = np.lexsort((touched, bg[touched], -fg[touched], -score))
    unique = touched.size
    count = min(max(int(math.ceil(unique * trainable_fraction)), min(min_rows, unique)), unique)
    ranked = [(int(touched[i]), float(score[i])) for i in order]
    return [r for r, _ in ranked[:count]], ranked


def sparse_rows_clip_scale(updates, clip_norm: Optional[float]) -> float:
    """`clip_scale_for_sparse_row_updates` (`src/nn.rs:2667-2774`): the norm runs over the active rows of
    the listed tables only.  `updates` is a sequence of `(grad, selected_rows, row_mask)`."""
    if clip_norm is None:
        return 1.0
    sum_sq = 0.0
    for grad, selected_rows, row_mask in updates:
        rows = active_sparse_rows(selected_rows, grad.shape[0], row_mask)
        sum_sq += float((np.asarray(grad, F64)[rows] ** 2).sum())
    norm = math.sqrt(sum_sq)
    return clip_norm / (norm + 1e-12) if norm > clip_norm else 1.0


# --------------------------------------------------------------------------------------
# the dense decoder LM (MemoryTransformerLm with no memory layers) and its training step
# --------------------------------------------------------------------------------------
@dataclass
class DecoderConfig:
    vocab: int
    d_model: int
    n_layers: int
    n_heads: int
    d_ff: int
    context: int


def parameter_names(cfg: DecoderConfig) -> List[str]:
    """State-dict order (`src/memory_transformer.rs:2098-2117`; per block
    `ln1, attention.{q,k,v,out}_proj, ln2, feed_forward.dense.fc{1,2}`)."""
    names = ["token_embedding.weight", "position_embedding.weight"]
    for i in range(cfg.n_layers):
        b = f"block.{i}."
        names += [b + "ln1.weight", b + "ln1.bias"]
        for proj in ("q_proj", "k_proj", "v_proj", "out_proj"):
            names += [b + f"attention.{proj}.weight", b + f"attention.{proj}.bias"]
        names += [b + "ln2.weight", b + "ln2.bias"]
        names += [b + "feed_forward.dense.fc1.weight", b + "feed_forward.dense.fc1.bias",
                  b + "feed_forward.dense.fc2.weight", b + "feed_forward.dense.fc2.bias"]
    names += ["ln_f.weight", "ln_f.bias", "lm_head.weight", "lm_head.bias"]
    return names


def parameter_shapes(cfg: DecoderConfig) -> Dict[str, Tuple[int, ...]]:
    d, f = cfg.d_model, cfg.d_ff
    shapes: Dict[str, Tuple[int, ...]] = {
        "token_embedding.weight": (cfg.vocab, d),
        "position_embedding.weight": (cfg.context, d),
    }
    for i in range(cfg.n_layers):
        b = f"block.{i}."
        for ln in ("ln1", "ln2"):
            shapes[b + ln + ".weight"] = (d,)
            shapes[b + ln + ".bias"] = (d,)
        for proj in ("q_proj", "k_proj", "v_proj", "out_proj"):
            shapes[b + f"attention.{proj}.weight"] = (d, d)
            shapes[b + f"attention.{proj}.bias"] = (d,)
        shapes[b + "feed_forward.dense.fc1.weight"] = (f, d)
        shapes[b + "feed_forward.dense.fc1.bias"] = (f,)
        shapes[b + "feed_forward.dense.fc2.weight"] = (d, f)
        shapes[b + "feed_forward.dense.fc2.bias"] = (d,)
    shapes["ln_f.weight"] = (d,)
    shapes["ln_f.bias"] = (d,)
    shapes["lm_head.weight"] = (cfg.vocab, d)
    shapes["lm_head.bias"] = (cfg.vocab,)
    return {n: shapes[n] for n in parameter_names(cfg)}


def init_parameters(cfg: DecoderConfig, seed: int) -> Dict[str, np.ndarray]:
    """Harness-side weight generator shared by both sides of every parity test: weights
    N(0, 0.02), residual projections (`out_proj`, `fc2`) scaled by 1/sqrt(2L), biases 0,
    LayerNorm γ=1 β=0.  (Weights are inputs of the step; the reference's own initialiser,
    `src/nn.rs:303-315`, is not part of the hot path.)"""
    rng = np.random.default_rng(seed)
    params: Dict[str, np.ndarray] = {}
    res_scale = 1.0 / math.sqrt(2.0 * cfg.n_layers)
    for name, shape in parameter_shapes(cfg).items():
        if name.endswith(".bias"):
            params[name] = np.zeros(shape, F64)
        elif ".ln" in name or name.startswith("ln_f"):
            params[name] = np.ones(shape, F64)
        else:
            w = rng.standard_normal(shape) * 0.02
            if "out_proj" in name or "fc2" in name:
                w = w * res_scale
            params[name] = f32_round(w)
    return params


def zipf_tokens(rng: np.random.Generator, vocab: int, shape, s: float = 1.1) -> np.ndarray:
    """Token ids with P(rank r) ∝ r^-s over [0, vocab) by inverse-CDF sampling."""
    ranks = np.arange(1, vocab + 1, dtype=F64)
    cdf = np.cumsum(ranks ** (-s))
    cdf /= cdf[-1]
    u = rng.random(size=shape)
    return np.minimum(np.searchsorted(cdf, u, side="right"), vocab - 1).astype(np.int64)


def _linear(x, w, b, amp: bool):
    """`Linear::forward` = `x·Wᵀ + b` (`src/nn.rs:454-475`).  Under AMP both operands are
    rounded to bf16 and the f32 result gets the f32 bias (`src/nn.rs:338-450`)."""
    if amp:
        y = f32_round(np.matmul(bf16_round(x), bf16_round(w).T))
    else:
        y = f32_round(np.matmul(np.asarray(x, F64), np.asarray(w, F64).T))
    return f32_round(y + b)


def _linear_backward(x, w, gy, amp: bool):
    """dX = dY·W, dW = dYᵀ·X, db = Σ dY (`src/tensor/autograd.rs:2012-2104`); under AMP dY,
    X and W enter the products as bf16 operands (`src/tensor/autograd.rs:795-850`)."""
    gy = np.asarray(gy, F64)
    db = gy.sum(axis=0)
    if amp:
        gyo = bf16_round(gy)
        dx = np.matmul(gyo, bf16_round(w))
        dw = np.matmul(gyo.T, bf16_round(x))
        # the CUDA route stores each product as an f32 tensor
        return f32_round(dx), f32_round(dw), f32_round(db)
    return np.matmul(gy, np.asarray(w, F64)), np.matmul(gy.T, np.asarray(x, F64)), db


def decoder_loss_and_grads(cfg: DecoderConfig, params: Dict[str, np.ndarray], tokens: np.ndarray,
                           targets: np.ndarray, amp_bf16: bool = False,
                           grad_f32: bool = False) -> Tuple[float, Dict[str, np.ndarray]]:
    """Forward + backward of the N-layer pre-LN decoder with mean next-token cross-entropy.

    f32 mode follows `MemoryTransformerLm::forward`/`loss` (`src/memory_transformer.rs:2069-2081`,
    `:1604-1610`) and the block `x + attn(ln1 x)`, `r + ff(ln2 r)` (`:1176-1183`).
    AMP mode inserts the bf16 round trips of `forward_amp_bf16` (`:1636-1662`, block
    `:1153-1172`, attention `src/nn.rs:718-788`, feed-forward `:873-884`); backward passes
    gradients through those round trips unchanged (`src/tensor/autograd.rs:324-329`).

    `grad_f32` rounds every op-boundary gradient to f32, which is what a device backend that
    stores f32 gradients does; the reference CPU path keeps them f64."""
    amp = amp_bf16
    rt = bf16_round if amp else (lambda a: a)
    gr = f32_round if (grad_f32 or amp) else (lambda a: np.asarray(a, F64))
    B, T = tokens.shape
    N, d, H = B * T, cfg.d_model, cfg.n_heads
    p = params
    pos_ids = np.tile(np.arange(T, dtype=np.int64), (B, 1))
    tok = rt(embedding(p["token_embedding.weight"], tokens))
    pos = rt(embedding(p["position_embedding.weight"], pos_ids))
    x = rt(add(tok, pos)).reshape(N, d)
    saved = []
    for i in range(cfg.n_layers):
        b = f"block.{i}."
        a = rt(layer_norm(x, p[b + "ln1.weight"], p[b + "ln1.bias"]))
        q = rt(_linear(a, p[b + "attention.q_proj.weight"], p[b + "attention.q_proj.bias"], amp))
        k = rt(_linear(a, p[b + "attention.k_proj.weight"], p[b + "attention.k_proj.bias"], amp))
        v = rt(_linear(a, p[b + "attention.v_proj.weight"], p[b + "attention.v_proj.bias"], amp))
        o, probs = causal_attention(q.reshape(B, T, d), k.reshape(B, T, d), v.reshape(B, T, d), H,
                                    return_probs=True, round_probs_bf16=amp)
        o = rt(o).reshape(N, d)
        pr = rt(_linear(o, p[b + "attention.out_proj.weight"], p[b + "attention.out_proj.bias"], amp))
        r = rt(add(x, pr))
        c = rt(layer_norm(r, p[b + "ln2.weight"], p[b + "ln2.bias"]))
        h = rt(_linear(c, p[b + "feed_forward.dense.fc1.weight"], p[b + "feed_forward.dense.fc1.bias"], amp))
        g = rt(gelu(h))
        f = rt(_linear(g, p[b + "feed_forward.dense.fc2.weight"], p[b + "feed_forward.dense.fc2.bias"], amp))
        y = rt(add(r, f))
        saved.append((x, a, q, k, v, probs, o, r, c, h, g))
        x = y
    z = rt(layer_norm(x, p["ln_f.weight"], p["ln_f.bias"]))
    logits = _linear(z, p["lm_head.weight"], p["lm_head.bias"], amp)
    flat_targets = targets.reshape(N)
    loss = float(cross_entropy(logits, flat_targets))

    grads: Dict[str, np.ndarray] = {}
    dlogits = gr(cross_entropy_backward(logits, flat_targets))
    dz, grads["lm_head.weight"], grads["lm_head.bias"] = _linear_backward(z, p["lm_head.weight"], dlogits, amp)
    dx, grads["ln_f.weight"], grads["ln_f.bias"] = layer_norm_backward(x, p["ln_f.weight"], gr(dz))
    dx = gr(dx)
    for i in reversed(range(cfg.n_layers)):
        b = f"block.{i}."
        x_in, a, q, k, v, probs, o, r, c, h, g = saved[i]
        # y = r + f
        dg, grads[b + "feed_forward.dense.fc2.weight"], grads[b + "feed_forward.dense.fc2.bias"] = \
            _linear_backward(g, p[b + "feed_forward.dense.fc2.weight"], dx, amp)
        dh = gr(gelu_backward(h, gr(dg)))
        dc, grads[b + "feed_forward.dense.fc1.weight"], grads[b + "feed_forward.dense.fc1.bias"] = \
            _linear_backward(c, p[b + "feed_forward.dense.fc1.weight"], dh, amp)
        dr_ln, grads[b + "ln2.weight"], grads[b + "ln2.bias"] = layer_norm_backward(r, p[b + "ln2.weight"], gr(dc))
        dr = gr(dx + gr(dr_ln))
        # r = x + pr
        do, grads[b + "attention.out_proj.weight"], grads[b + "attention.out_proj.bias"] = \
            _linear_backward(o, p[b + "attention.out_proj.weight"], dr, amp)
        dq, dk, dv = causal_attention_backward(q.reshape(B, T, d), k.reshape(B, T, d), v.reshape(B, T, d), H,
                                               gr(do).reshape(B, T, d), probs=probs, bf16_operands=amp)
        da = np.zeros((N, d), F64)
        for name, dproj in (("q_proj", dq), ("k_proj", dk), ("v_proj", dv)):
            dai, grads[b + f"attention.{name}.weight"], grads[b + f"attention.{name}.bias"] = \
                _linear_backward(a, p[b + f"attention.{name}.weight"], gr(dproj).reshape(N, d), amp)
            da = gr(da + dai)
        dx_ln, grads[b + "ln1.weight"], grads[b + "ln1.bias"] = layer_norm_backward(x_in, p[b + "ln1.weight"], da)
        dx = gr(dr + gr(dx_ln))
    dx3 = dx.reshape(B, T, d)
    grads["token_embedding.weight"] = embedding_backward(p["token_embedding.weight"].shape, tokens, dx3)
    grads["position_embedding.weight"] = embedding_backward(p["position_embedding.weight"].shape, pos_ids, dx3)
    if grad_f32 or amp:
        grads = {n: f32_round(g_) for n, g_ in grads.items()}
    return loss, grads


def decoder_logits(cfg: DecoderConfig, params: Dict[str, np.ndarray], tokens: np.ndarray, amp_bf16: bool = False) -> np.ndarray:
    """Forward pass only: logits `[B, T, vocab]` for token windows of any length T <= context
    (`MemoryTransformerLm::forward`, `src/memory_transformer.rs:2069-2081`; the window form is what
    `next_token_logits` feeds it, `:1930-1984`)."""
    amp = amp_bf16
    rt = bf16_round if amp else (lambda a: a)
    B, T = tokens.shape
    N, d, H = B * T, cfg.d_model, cfg.n_heads
    p = params
    pos_ids = np.tile(np.arange(T, dtype=np.int64), (B, 1))
    x = rt(add(rt(embedding(p["token_embedding.weight"], tokens)), rt(embedding(p["position_embedding.weight"], pos_ids)))).reshape(N, d)
    for i in range(cfg.n_layers):
        b = f"block.{i}."
        a = rt(layer_norm(x, p[b + "ln1.weight"], p[b + "ln1.bias"]))
        q, k, v = (rt(_linear(a, p[b + f"attention.{n}.weight"], p[b + f"attention.{n}.bias"], amp)).reshape(B, T, d)
                   for n in ("q_proj", "k_proj", "v_proj"))
        o = rt(causal_attention(q, k, v, H, round_probs_bf16=amp)).reshape(N, d)
        r = rt(add(x, rt(_linear(o, p[b + "attention.out_proj.weight"], p[b + "attention.out_proj.bias"], amp))))
        c = rt(layer_norm(r, p[b + "ln2.weight"], p[b + "ln2.bias"]))
        h = rt(_linear(c, p[b + "feed_forward.dense.fc1.weight"], p[b + "feed_forward.dense.fc1.bias"], amp))
        f = rt(_linear(rt(gelu(h)), p[b + "feed_forward.dense.fc2.weight"], p[b + "feed_forward.dense.fc2.bias"], amp))
        x = rt(add(r, f))
    z = rt(layer_norm(x, p["ln_f.weight"], p["ln_f.bias"]))
    return _linear(z, p["lm_head.weight"], p["lm_head.bias"], amp).reshape(B, T, cfg.vocab)


def train_steps(cfg: DecoderConfig, params: Dict[str, np.ndarray], batches, state: AdamWState,
                amp_bf16: bool = False, grad_f32: bool = False) -> List[float]:
    """Run `zero_grad → loss → backward → AdamW.step` per batch
    (`src/bin/heirloom/commands/training.rs:125-167`); returns the per-step losses and
    updates `params`/`state` in place."""
    losses = []
    for tokens, targets in batches:
        loss, grads = decoder_loss_and_grads(cfg, params, tokens, targets, amp_bf16, grad_f32)
        adamw_step(params, grads, state)
        losses.append(loss)
    return losses


# --------------------------------------------------------------------------------------
# memory transformer: the same decoder with product-key memory feed-forward blocks
# --------------------------------------------------------------------------------------
@dataclass
class MemoryConfig:
    """`MemoryTransformerConfig` restricted to what the training step uses
    (`src/memory_transformer.rs:1217-1261`): one shared table set, one memory head, product-key
    lookup, gated value path (`memory_plus`)."""
    memory_layers: Tuple[int, ...] = ()
    slots: int = 0
    key_dim: int = 0
    value_dim: int = 0
    top_k: int = 0


def memory_parameter_names(cfg: DecoderConfig, mem: MemoryConfig) -> List[str]:
    """State-dict order with shared tables (`src/memory_transformer.rs:2098-2117`, `:632-642`,
    `:1015-1032`)."""
    names = ["token_embedding.weight", "position_embedding.weight"]
    if mem.memory_layers:
        names += ["shared_memory.product_key_left", "shared_memory.product_key_right", "shared_memory.value"]
    for i in range(cfg.n_layers):
        b = f"block.{i}."
        names += [b + "ln1.weight", b + "ln1.bias"]
        for proj in ("q_proj", "k_proj", "v_proj", "out_proj"):
            names += [b + f"attention.{proj}.weight", b + f"attention.{proj}.bias"]
        names += [b + "ln2.weight", b + "ln2.bias"]
        if i in mem.memory_layers:
            for proj in ("query_proj", "gate_proj", "out_proj"):
                names += [b + f"feed_forward.memory.{proj}.weight", b + f"feed_forward.memory.{proj}.bias"]
        else:
            names += [b + "feed_forward.dense.fc1.weight", b + "feed_forward.dense.fc1.bias",
                      b + "feed_forward.dense.fc2.weight", b + "feed_forward.dense.fc2.bias"]
    names += ["ln_f.weight", "ln_f.bias", "lm_head.weight", "lm_head.bias"]
    return names


def memory_parameter_shapes(cfg: DecoderConfig, mem: MemoryConfig) -> Dict[str, Tuple[int, ...]]:
    base = parameter_shapes(cfg)
    d = cfg.d_model
    side = int(round(math.sqrt(mem.slots))) if mem.slots else 0
    shapes: Dict[str, Tuple[int, ...]] = {}
    for name in memory_parameter_names(cfg, mem):
        if name in base:
            shapes[name] = base[name]
        elif name.endswith("product_key_left") or name.endswith("product_key_right"):
            shapes[name] = (side, mem.key_dim // 2)
        elif name.endswith("shared_memory.value"):
            shapes[name] = (mem.slots, mem.value_dim)
        elif "query_proj" in name:
            shapes[name] = (mem.key_dim, d) if name.endswith("weight") else (mem.key_dim,)
        elif "gate_proj" in name:
            shapes[name] = (mem.value_dim, d) if name.endswith("weight") else (mem.value_dim,)
        elif "memory.out_proj" in name:
            shapes[name] = (d, mem.value_dim) if name.endswith("weight") else (d,)
    return shapes


def init_memory_parameters(cfg: DecoderConfig, mem: MemoryConfig, seed: int) -> Dict[str, np.ndarray]:
    """Harness-side generator: N(0, 0.02) weights (residual projections scaled), half-key tables
    N(0, 1/sqrt(half_dim)) and value table N(0, 0.02) as in `MemoryTables::new`
    (`src/memory_transformer.rs:568-601`)."""
    rng = np.random.default_rng(seed)
    res_scale = 1.0 / math.sqrt(2.0 * cfg.n_layers)
    params: Dict[str, np.ndarray] = {}
    for name, shape in memory_parameter_shapes(cfg, mem).items():
        if name.endswith(".bias"):
            params[name] = np.zeros(shape, F64)
        elif ".ln" in name or name.startswith("ln_f"):
            params[name] = np.ones(shape, F64)
        elif "product_key" in name:
            params[name] = f32_round(rng.standard_normal(shape) / math.sqrt(shape[1]))
        else:
            w = rng.standard_normal(shape) * 0.02
            if "out_proj" in name or "fc2" in name:
                w = w * res_scale
            params[name] = f32_round(w)
    return params


def memory_feed_forward(x, p: Dict[str, np.ndarray], prefix: str, mem: MemoryConfig):
    """`MemoryFeedForward::forward_named` (`src/memory_transformer.rs:742-781`): every internal op is an
    f32 tensor op, also under AMP (`:787-789`).  Returns the output and what backward needs."""
    side = int(round(math.sqrt(mem.slots)))
    half = mem.key_dim // 2
    kl, kr, val = p["shared_memory.product_key_left"], p["shared_memory.product_key_right"], p["shared_memory.value"]
    q = _linear(x, p[prefix + "query_proj.weight"], p[prefix + "query_proj.bias"], False)
    ls = side_scores_f32(q[:, :half], kl)
    rs = side_scores_f32(q[:, half:], kr)
    idx = product_key_indices_from_side_scores(ls, rs, mem.top_k, product_key_beam(side, mem.top_k))
    scores = product_key_selected_scores(idx, q, kl, kr)
    w = softmax(scores, 1)
    weighted = memory_weighted_value(idx, w, val)
    gpre = _linear(x, p[prefix + "gate_proj.weight"], p[prefix + "gate_proj.bias"], False)
    gate = gelu(gpre)
    mv = f32_round(weighted * gate)
    out = _linear(mv, p[prefix + "out_proj.weight"], p[prefix + "out_proj.bias"], False)
    return out, (x, q, idx, w, weighted, gpre, gate, mv)


def memory_feed_forward_backward(saved, p, prefix: str, mem: MemoryConfig, gout, grads, gr):
    """Gradients of the memory feed-forward; indices are not differentiable
    (`src/tensor/autograd.rs:2263-2494`).  Table gradients are added into `grads`."""
    x, q, idx, w, weighted, gpre, gate, mv = saved
    kl, kr, val = p["shared_memory.product_key_left"], p["shared_memory.product_key_right"], p["shared_memory.value"]
    dmv, grads[prefix + "out_proj.weight"], grads[prefix + "out_proj.bias"] = \
        _linear_backward(mv, p[prefix + "out_proj.weight"], gout, False)
    dmv = gr(dmv)
    dweighted = gr(dmv * gate)
    dgate = gr(dmv * weighted)
    dgpre = gr(gelu_backward(gpre, dgate))
    dx_gate, grads[prefix + "gate_proj.weight"], grads[prefix + "gate_proj.bias"] = \
        _linear_backward(x, p[prefix + "gate_proj.weight"], dgpre, False)
    dw, dval = memory_weighted_value_backward(idx, w, val, dweighted)
    dscores = gr(softmax_backward(w, gr(dw), 1))
    dq, dkl, dkr = product_key_selected_scores_backward(idx, q, kl, kr, dscores)
    dx_q, grads[prefix + "query_proj.weight"], grads[prefix + "query_proj.bias"] = \
        _linear_backward(x, p[prefix + "query_proj.weight"], gr(dq), False)
    for name, g in (("shared_memory.value", dval), ("shared_memory.product_key_left", dkl),
                    ("shared_memory.product_key_right", dkr)):
        grads[name] = g if name not in grads else gr(grads[name] + g)
    # gradient accumulation on the shared input follows the order the graph is walked: gate path
    # first, then the query path (`src/tensor.rs:1721-1846`)
    return gr(gr(dx_gate) + gr(dx_q))


def memory_decoder_loss_and_grads(cfg: DecoderConfig, mem: MemoryConfig, params, tokens, targets,
                                  amp_bf16: bool = False, grad_f32: bool = False, return_indices: bool = False,
                                  return_queries: bool = False):
    """The decoder of `decoder_loss_and_grads` with memory feed-forward blocks at `mem.memory_layers`
    (`MemoryTransformerBlock`, `src/memory_transformer.rs:1092-1183`)."""
    amp = amp_bf16
    rt = bf16_round if amp else (lambda a: a)
    gr = f32_round if (grad_f32 or amp) else (lambda a: np.asarray(a, F64))
    B, T = tokens.shape
    N, d, H = B * T, cfg.d_model, cfg.n_heads
    p = params
    pos_ids = np.tile(np.arange(T, dtype=np.int64), (B, 1))
    tok = rt(embedding(p["token_embedding.weight"], tokens))
    pos = rt(embedding(p["position_embedding.weight"], pos_ids))
    x = rt(add(tok, pos)).reshape(N, d)
    saved = []
    all_indices = {}
    all_queries = {}
    for i in range(cfg.n_layers):
        b = f"block.{i}."
        a = rt(layer_norm(x, p[b + "ln1.weight"], p[b + "ln1.bias"]))
        q = rt(_linear(a, p[b + "attention.q_proj.weight"], p[b + "attention.q_proj.bias"], amp))
        k = rt(_linear(a, p[b + "attention.k_proj.weight"], p[b + "attention.k_proj.bias"], amp))
        v = rt(_linear(a, p[b + "attention.v_proj.weight"], p[b + "attention.v_proj.bias"], amp))
        o, probs = causal_attention(q.reshape(B, T, d), k.reshape(B, T, d), v.reshape(B, T, d), H,
                                    return_probs=True, round_probs_bf16=amp)
        o = rt(o).reshape(N, d)
        pr = rt(_linear(o, p[b + "attention.out_proj.weight"], p[b + "attention.out_proj.bias"], amp))
        r = rt(add(x, pr))
        c = rt(layer_norm(r, p[b + "ln2.weight"], p[b + "ln2.bias"]))
        if i in mem.memory_layers:
            f_raw, ff_saved = memory_feed_forward(c, p, b + "feed_forward.memory.", mem)
            all_indices[i] = ff_saved[2]
            all_queries[i] = ff_saved[1]
            f = rt(f_raw)
            saved.append((x, a, q, k, v, probs, o, r, c, None, None, ff_saved))
        else:
            h = rt(_linear(c, p[b + "feed_forward.dense.fc1.weight"], p[b + "feed_forward.dense.fc1.bias"], amp))
            g = rt(gelu(h))
            f = rt(_linear(g, p[b + "feed_forward.dense.fc2.weight"], p[b + "feed_forward.dense.fc2.bias"], amp))
            saved.append((x, a, q, k, v, probs, o, r, c, h, g, None))
        x = rt(add(r, f))
    z = rt(layer_norm(x, p["ln_f.weight"], p["ln_f.bias"]))
    logits = _linear(z, p["lm_head.weight"], p["lm_head.bias"], amp)
    flat_targets = targets.reshape(N)
    loss = float(cross_entropy(logits, flat_targets))

    grads: Dict[str, np.ndarray] = {}
    dlogits = gr(cross_entropy_backward(logits, flat_targets))
    dz, grads["lm_head.weight"], grads["lm_head.bias"] = _linear_backward(z, p["lm_head.weight"], dlogits, amp)
    dx, grads["ln_f.weight"], grads["ln_f.bias"] = layer_norm_backward(x, p["ln_f.weight"], gr(dz))
    dx = gr(dx)
    for i in reversed(range(cfg.n_layers)):
        b = f"block.{i}."
        x_in, a, q, k, v, probs, o, r, c, h, g, ff_saved = saved[i]
        if ff_saved is not None:
            dc = memory_feed_forward_backward(ff_saved, p, b + "feed_forward.memory.", mem, dx, grads, gr)
        else:
            dg, grads[b + "feed_forward.dense.fc2.weight"], grads[b + "feed_forward.dense.fc2.bias"] = \
                _linear_backward(g, p[b + "feed_forward.dense.fc2.weight"], dx, amp)
            dh = gr(gelu_backward(h, gr(dg)))
            dc, grads[b + "feed_forward.dense.fc1.weight"], grads[b + "feed_forward.dense.fc1.bias"] = \
                _linear_backward(c, p[b + "feed_forward.dense.fc1.weight"], dh, amp)
        dr_ln, grads[b + "ln2.weight"], grads[b + "ln2.bias"] = layer_norm_backward(r, p[b + "ln2.weight"], gr(dc))
        dr = gr(dx + gr(dr_ln))
        do, grads[b + "attention.out_proj.weight"], grads[b + "attention.out_proj.bias"] = \
            _linear_backward(o, p[b + "attention.out_proj.weight"], dr, amp)
        dq, dk, dv = causal_attention_backward(q.reshape(B, T, d), k.reshape(B, T, d), v.reshape(B, T, d), H,
                                               gr(do).reshape(B, T, d), probs=probs, bf16_operands=amp)
        da = np.zeros((N, d), F64)
        for name, dproj in (("q_proj", dq), ("k_proj", dk), ("v_proj", dv)):
            dai, grads[b + f"attention.{name}.weight"], grads[b + f"attention.{name}.bias"] = \
                _linear_backward(a, p[b + f"attention.{name}.weight"], gr(dproj).reshape(N, d), amp)
            da = gr(da + dai)
        dx_ln, grads[b + "ln1.weight"], grads[b + "ln1.bias"] = layer_norm_backward(x_in, p[b + "ln1.weight"], da)
        dx = gr(dr + gr(dx_ln))
    dx3 = dx.reshape(B, T, d)
    grads["token_embedding.weight"] = embedding_backward(p["token_embedding.weight"].shape, tokens, dx3)
    grads["position_embedding.weight"] = embedding_backward(p["position_embedding.weight"].shape, pos_ids, dx3)
    if grad_f32 or amp:
        grads = {n: f32_round(g_) for n, g_ in grads.items()}
    if return_queries:
        return loss, grads, all_indices, all_queries
    if return_indices:
        return loss, grads, all_indices
    return loss, grads

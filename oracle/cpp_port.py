"""ctypes binding of the C++ CPU restatement (`oracle/heirloom_ref.cpp`).

Test infrastructure, like everything in this package: only the tests, the smoke check and the
benchmark's CPU legs may import it.  The library is built by `make -C oracle` (the package's
build step runs it); `load()` builds it on demand when it is missing."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import heirloom_oracle as ho

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "lib" / "libheirloom_ref.so"
_lib = None


class _Config(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("vocab", "d_model", "n_layers", "n_heads", "d_ff", "context")]


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        subprocess.run(["make", "-s", "-C", str(_HERE)], check=True)
    lib = ctypes.CDLL(str(_LIB_PATH))
    dp, ip = ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int64)
    lib.hr_param_count.restype = ctypes.c_longlong
    lib.hr_param_count.argtypes = [ctypes.POINTER(_Config)]
    lib.hr_loss_and_grads.restype = ctypes.c_double
    lib.hr_loss_and_grads.argtypes = [ctypes.POINTER(_Config), dp, ip, ip, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_int, dp]
    lib.hr_adamw_step.restype = None
    lib.hr_adamw_step.argtypes = [dp, dp, dp, dp, ctypes.c_longlong, ctypes.c_int] + [ctypes.c_double] * 6
    lib.hr_train_steps.restype = None
    lib.hr_train_steps.argtypes = [ctypes.POINTER(_Config), dp, dp, dp, ip, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                   ctypes.c_int] + [ctypes.c_double] * 6 + [ctypes.c_int, ctypes.c_int, dp]
    _lib = lib
    return lib


def _cfg(cfg: ho.DecoderConfig) -> _Config:
    return _Config(cfg.vocab, cfg.d_model, cfg.n_layers, cfg.n_heads, cfg.d_ff, cfg.context)


def _dp(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_double))


def _ip(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_int64))


def flatten(cfg: ho.DecoderConfig, params: Dict[str, np.ndarray]) -> np.ndarray:
    """Parameters as one f64 vector in state-dict order."""
    return np.concatenate([np.asarray(params[n], np.float64).reshape(-1) for n in ho.parameter_names(cfg)])


def unflatten(cfg: ho.DecoderConfig, flat: np.ndarray) -> Dict[str, np.ndarray]:
    out, at = {}, 0
    for name, shape in ho.parameter_shapes(cfg).items():
        n = int(np.prod(shape))
        out[name] = flat[at:at + n].reshape(shape).copy()
        at += n
    return out


def loss_and_grads(cfg: ho.DecoderConfig, params: Dict[str, np.ndarray], tokens: np.ndarray, targets: np.ndarray,
                   amp_bf16: bool = False, grad_f32: bool = False) -> Tuple[float, Dict[str, np.ndarray]]:
    lib = load()
    c = _cfg(cfg)
    flat = flatten(cfg, params)
    assert flat.size == lib.hr_param_count(ctypes.byref(c))
    tok = np.ascontiguousarray(tokens, np.int64)
    tgt = np.ascontiguousarray(targets, np.int64)
    grads = np.zeros_like(flat)
    B, T = tok.shape
    loss = lib.hr_loss_and_grads(ctypes.byref(c), _dp(flat), _ip(tok), _ip(tgt), B, T, int(amp_bf16), int(grad_f32),
                                 _dp(grads))
    return float(loss), unflatten(cfg, grads)


def train_steps(cfg: ho.DecoderConfig, params: Dict[str, np.ndarray], token_batches: np.ndarray, lr=1e-3, beta1=0.9,
                beta2=0.999, eps=1e-8, weight_decay=0.01, clip_norm: Optional[float] = None, amp_bf16=False,
                grad_f32=False) -> Tuple[List[float], Dict[str, np.ndarray]]:
    """`token_batches` is `[steps, B, T+1]`; returns the per-step losses and the final parameters."""
    lib = load()
    c = _cfg(cfg)
    flat = flatten(cfg, params)
    m, v = np.zeros_like(flat), np.zeros_like(flat)
    batches = np.ascontiguousarray(token_batches, np.int64)
    steps, B, t1 = batches.shape
    losses = np.zeros(steps, np.float64)
    lib.hr_train_steps(ctypes.byref(c), _dp(flat), _dp(m), _dp(v), _ip(batches), steps, B, t1 - 1, 0, lr, beta1, beta2,
                       eps, weight_decay, -1.0 if clip_norm is None else float(clip_norm), int(amp_bf16),
                       int(grad_f32), _dp(losses))
    return losses.tolist(), unflatten(cfg, flat)

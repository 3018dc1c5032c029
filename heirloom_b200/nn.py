"""Host-side mirror of the reference's model/optimizer surface for the training-step path.

`DecoderLm` stands where the reference has `MemoryTransformerLm` with no memory layers plus
its `AdamW` (src/memory_transformer.rs:1217-1261, src/nn.rs:1941-2220): named parameters in
state-dict order, `loss`/`backward`/`step`, and a one-call `train_step`.  All arithmetic runs in
`libheirloom_b200.so`; this file only moves bytes and names.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, byref, c_char_p, c_float, c_int, c_longlong, c_size_t, c_void_p
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ._lib import HeirloomError, check
from .cuda import Context

PRECISION_F32, PRECISION_AMP_BF16 = 0, 1


class _DecoderConfig(Structure):
    _fields_ = [(n, c_int) for n in ("vocab", "d_model", "n_layers", "n_heads", "d_ff", "context", "batch", "precision")]


class _MemoryConfig(Structure):
    _fields_ = [("n_memory_layers", c_int), ("memory_layers", c_int * 16), ("slots", c_int), ("key_dim", c_int),
                ("value_dim", c_int), ("top_k", c_int), ("memory_heads", c_int)]


class _AdamWConfig(Structure):
    _fields_ = [(n, c_float) for n in ("lr", "beta1", "beta2", "eps", "weight_decay", "clip_norm")]


@dataclass
class DecoderConfig:
    vocab: int
    d_model: int
    n_layers: int
    n_heads: int
    d_ff: int
    context: int
    batch: int
    precision: int = PRECISION_AMP_BF16


@dataclass
class MemoryConfig:
    """Product-key memory feed-forward blocks with one shared table set
    (`MemoryTransformerConfig`, src/memory_transformer.rs:1217-1261)."""
    memory_layers: Tuple[int, ...]
    slots: int
    key_dim: int
    value_dim: int
    top_k: int
    memory_heads: int = 1


class DecoderLm:
    """N-layer pre-LayerNorm decoder LM living on one GPU (`hl_decoder`); with `memory` the
    listed blocks use the product-key memory feed-forward."""

    def __init__(self, ctx: Context, cfg: DecoderConfig, memory: Optional[MemoryConfig] = None):
        self.ctx, self.cfg, self.memory = ctx, cfg, memory
        self._lib = ctx.lib
        self._lib.hl_decoder_launches_last_step.restype = ctypes.c_ulonglong
        self._lib.hl_decoder_optimizer_steps.restype = c_longlong
        self._lib.hl_decoder_destroy.restype = None
        c = _DecoderConfig(cfg.vocab, cfg.d_model, cfg.n_layers, cfg.n_heads, cfg.d_ff, cfg.context, cfg.batch,
                           cfg.precision)
        h = c_void_p()
        if memory is None:
            check(self._lib.hl_decoder_create(ctx.handle, byref(c), byref(h)))
        else:
            layers = (c_int * 16)(*memory.memory_layers)
            mc = _MemoryConfig(len(memory.memory_layers), layers, memory.slots, memory.key_dim, memory.value_dim,
                               memory.top_k, memory.memory_heads)
            check(self._lib.hl_memory_decoder_create(ctx.handle, byref(c), byref(mc), byref(h)))
        self.handle = h
        self._index: Dict[str, Tuple[int, Tuple[int, ...]]] = {}
        for i in range(self._lib.hl_decoder_param_count(self.handle)):
            name = ctypes.create_string_buffer(160)
            numel, rank = c_longlong(), c_int()
            shape = (c_longlong * 2)()
            check(self._lib.hl_decoder_param_info(self.handle, c_int(i), name, c_size_t(160), byref(numel), byref(rank),
                                                  shape))
            self._index[name.value.decode()] = (i, tuple(int(shape[j]) for j in range(rank.value)))
        self._pinned = None

    def close(self) -> None:
        if self.handle:
            self._lib.hl_decoder_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- parameters (Module::named_parameters, src/nn.rs:16-29) -----------------------------------
    def parameter_names(self) -> List[str]:
        return list(self._index)

    def parameter_shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: s for n, (_, s) in self._index.items()}

    def _slot(self, name: str):
        if name not in self._index:
            raise HeirloomError(f"no parameter named {name}")
        return self._index[name]

    def load_state_dict(self, state: Dict[str, np.ndarray]) -> None:
        """Loads by name and shape like `load_state_dict` (src/nn.rs:2997-3038)."""
        for name, (idx, shape) in self._index.items():
            if name not in state:
                raise HeirloomError(f"state dict is missing {name}")
            arr = np.ascontiguousarray(state[name], dtype=np.float32)
            if tuple(arr.shape) != shape:
                raise HeirloomError(f"shape mismatch for {name}: expected {shape}, got {tuple(arr.shape)}")
            check(self._lib.hl_decoder_set_param(self.handle, c_int(idx), arr.ctypes.data_as(c_void_p),
                                                 c_longlong(arr.size)))

    def _fetch(self, fn, name: str) -> np.ndarray:
        idx, shape = self._slot(name)
        out = np.empty(shape, np.float32)
        check(fn(self.handle, c_int(idx), out.ctypes.data_as(c_void_p), c_longlong(out.size)))
        return out

    def parameter(self, name: str) -> np.ndarray:
        return self._fetch(self._lib.hl_decoder_get_param, name)

    def grad(self, name: str) -> np.ndarray:
        return self._fetch(self._lib.hl_decoder_get_grad, name)

    def moments(self, name: str) -> Tuple[np.ndarray, np.ndarray]:
        idx, shape = self._slot(name)
        m, v = np.empty(shape, np.float32), np.empty(shape, np.float32)
        check(self._lib.hl_decoder_get_moments(self.handle, c_int(idx), m.ctypes.data_as(c_void_p),
                                               v.ctypes.data_as(c_void_p), c_longlong(m.size)))
        return m, v

    def set_moments(self, name: str, m: np.ndarray, v: np.ndarray) -> None:
        """`AdamW::load_state` for one parameter (src/nn.rs:2059-2080); needs `set_optimizer` first."""
        idx, shape = self._slot(name)
        m = np.ascontiguousarray(m, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        if tuple(m.shape) != shape or tuple(v.shape) != shape:
            raise HeirloomError(f"AdamW state shape mismatch for {name}: expected {shape}")
        check(self._lib.hl_decoder_set_moments(self.handle, c_int(idx), m.ctypes.data_as(c_void_p),
                                               v.ctypes.data_as(c_void_p), c_longlong(m.size)))

    def set_optimizer_steps(self, steps: int) -> None:
        check(self._lib.hl_decoder_set_optimizer_steps(self.handle, c_longlong(int(steps))))

    def state_dict(self) -> Dict[str, np.ndarray]:
        return {n: self.parameter(n) for n in self._index}

    # ---- optimizer (AdamW, src/nn.rs:1941-2220) ----------------------------------------------------
    def set_optimizer(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, clip_norm=None) -> None:
        cfg = _AdamWConfig(lr, beta1, beta2, eps, weight_decay, clip_norm if clip_norm else 0.0)
        check(self._lib.hl_decoder_set_optimizer(self.handle, byref(cfg)))

    @property
    def optimizer_steps(self) -> int:
        return int(self._lib.hl_decoder_optimizer_steps(self.handle))

    # ---- the step ----------------------------------------------------------------------------------
    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor) -> None:
        """tokens/targets: int64 CUDA tensors `[batch, context]`."""
        check(self._lib.hl_decoder_forward_backward(self.handle, c_void_p(tokens.data_ptr()),
                                                    c_void_p(targets.data_ptr())))

    def optimizer_step(self) -> None:
        check(self._lib.hl_decoder_optimizer_step(self.handle))

    def optimizer_step_sparse_rows(self) -> None:
        """The reference's `SparseRows` policy (runtime.rs:2424-2435): row-set AdamW on the two
        half-key tables and the value table over the rows the memory blocks chose in the last
        forward, no dense update in this call."""
        check(self._lib.hl_decoder_optimizer_step_sparse_rows(self.handle))

    POLICIES = {"full": 0, "memory_only": 1, "sparse_rows": 2, "frozen": 3, "dense_plus_sparse_values": 4}

    def optimizer_step_policy(self, policy: str) -> None:
        """The optimizer step under a memory update policy: the reference's `full`, `memory_only`, `sparse_rows`,
        `frozen` (`MemoryUpdatePolicy`, src/memory_transformer.rs:26-32; runtime.rs:2416-2452), or
        `dense_plus_sparse_values` (dense AdamW on everything but the value table, row-set AdamW on the value rows
        the step selected)."""
        if policy not in self.POLICIES:
            raise HeirloomError(f"unknown memory update policy {policy!r}; expected one of {sorted(self.POLICIES)}")
        check(self._lib.hl_decoder_optimizer_step_policy(self.handle, c_int(self.POLICIES[policy])))

    def eval_loss_device(self, tokens: torch.Tensor, targets: torch.Tensor) -> float:
        """Forward-only mean cross-entropy over int64 CUDA tensors `[sequences, context]`, sequences <= batch."""
        if tokens.dim() != 2 or tokens.shape[1] != self.cfg.context or tokens.shape != targets.shape:
            raise HeirloomError(f"expected token input [sequences, {self.cfg.context}], got {tuple(tokens.shape)}")
        out = c_float()
        check(self._lib.hl_decoder_eval_loss(self.handle, c_void_p(tokens.contiguous().data_ptr()),
                                             c_void_p(targets.contiguous().data_ptr()), c_int(tokens.shape[0]), byref(out)))
        return float(out.value)

    def next_token_logits_device(self, window: torch.Tensor) -> np.ndarray:
        """Logits after a window of 1..context tokens (int64 CUDA vector), as f32 `[vocab]`."""
        out = np.empty(self.cfg.vocab, np.float32)
        check(self._lib.hl_decoder_next_token_logits(self.handle, c_void_p(window.contiguous().data_ptr()),
                                                     c_int(window.numel()), out.ctypes.data_as(c_void_p)))
        return out

    def train_step_device(self, tokens: torch.Tensor, targets: torch.Tensor) -> None:
        check(self._lib.hl_decoder_train_step_device(self.handle, c_void_p(tokens.data_ptr()),
                                                     c_void_p(targets.data_ptr())))

    def train_step(self, tokens_host: torch.Tensor, targets_host: torch.Tensor) -> float:
        """The call a user makes: host int64 `[batch, context]` tensors (pinned for speed) in,
        loss out."""
        loss = c_float()
        check(self._lib.hl_decoder_train_step(self.handle, c_void_p(tokens_host.data_ptr()),
                                              c_void_p(targets_host.data_ptr()), byref(loss)))
        return float(loss.value)

    def loss(self) -> float:
        out = c_float()
        check(self._lib.hl_decoder_loss(self.handle, byref(out)))
        return float(out.value)

    def selected_indices(self, layer: int) -> np.ndarray:
        """Memory slots chosen by block `layer` in the last forward: int64 `[batch*context, top_k]`
        (`MemoryFeedForward::last_selected_indices`, src/memory_transformer.rs:734-736)."""
        n = self.cfg.batch * self.cfg.context
        out = np.empty((n, self.memory.top_k), np.int64)
        check(self._lib.hl_decoder_selected_indices(self.handle, c_int(layer), out.ctypes.data_as(c_void_p),
                                                    c_longlong(out.size)))
        return out

    def memory_access_counts(self):
        """Row-access counts of the last forward pass over every memory block, counted on the device
        (`MemoryTransformerLm::memory_access_counts`, src/memory_transformer.rs:1561-1583)."""
        from .smft import MemoryAccessCounts
        if self.memory is None:
            raise HeirloomError("memory_access_counts: the model has no memory layers")
        counts = torch.zeros(self.memory.slots, dtype=torch.int64, device="cuda")
        check(self._lib.hl_decoder_memory_access_counts(self.handle, c_void_p(counts.data_ptr())))
        self.ctx.sync()
        return MemoryAccessCounts.from_row_counts(self.memory.slots, counts.cpu().numpy().view(np.uint64))

    def smft_access_report(self, top_rows: int):
        """`smft_access_report` (src/memory_transformer.rs:1585-1591)."""
        from .smft import SmftAccessReport
        counts = self.memory_access_counts()
        return SmftAccessReport(counts, counts.top_rows(top_rows))

    def smft_row_mask_against(self, background, trainable_fraction: float, min_rows: int):
        """`smft_row_mask_against` (src/memory_transformer.rs:1593-1601)."""
        return self.memory_access_counts().smft_mask_against(background, trainable_fraction, min_rows)

    def set_smft_mask(self, mask) -> None:
        """Restricts the sparse-rows step to the mask's trainable value rows and to the half-key rows of its
        conservative projection (`memory_sparse_adamw_updates_with_mask`, src/memory_transformer.rs:1426-1468).
        `None` lifts the restriction."""
        if mask is None:
            check(self._lib.hl_decoder_set_smft_masks(self.handle, None, None, None))
            return
        if self.memory is None or mask.memory_slots != self.memory.slots:
            slots = self.memory.slots if self.memory else 0
            raise HeirloomError(f"SMFT mask memory_slots {mask.memory_slots} does not match model memory_slots {slots}")
        projection = mask.product_key_projection()
        value, left, right = mask.to_mask(), projection.left_mask(), projection.right_mask()
        check(self._lib.hl_decoder_set_smft_masks(self.handle, value.ctypes.data_as(c_void_p), left.ctypes.data_as(c_void_p),
                                                  right.ctypes.data_as(c_void_p)))

    def comm_exposed_ms(self):
        """(milliseconds, waits): how long the compute stream sat idle waiting for gradient collectives since the
        last call; measured only while the context's per-kernel timing is on."""
        ms, waits = c_float(), c_int()
        check(self._lib.hl_decoder_comm_exposed_ms(self.handle, byref(ms), byref(waits)))
        return float(ms.value), int(waits.value)

    @property
    def launches_last_step(self) -> int:
        return int(self._lib.hl_decoder_launches_last_step(self.handle))

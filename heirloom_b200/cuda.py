"""Host-side wrappers over the C ABI, one function per device op.

The names follow the safe wrappers of the reference's kernel crate
(`heirloom_kernels::cuda::*`, heirloom-kernels/src/cuda.rs:1001-6847): value-style functions that
validate, launch and return the result buffer.  Device memory is held in torch tensors (torch
is the allocator here, nothing more); every computation goes through `libheirloom_b200.so`.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_float, c_int, c_longlong, c_size_t, c_void_p
from typing import Optional

import torch

from . import _lib
from ._lib import AdamWParams, AdamWTensor, Counters, DeviceInfo, GemmDesc, HeirloomError, MatrixLayout, check

F32, BF16, F64, I64, U8 = 0, 1, 2, 3, 4
ADD, SUB, MUL, DIV = 0, 1, 2, 3
K_MAJOR, MN_MAJOR = 0, 1
EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL, EPI_DGELU = 0, 1, 2, 3, 4

_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float64: F64, torch.int64: I64, torch.uint8: U8}


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _dt(t: torch.Tensor) -> int:
    return _DT[t.dtype]


_OPEN_STREAMS = set()  # raw handles of the compute streams of the contexts that are open


class Context:
    """One compute stream + one collective stream on one device (`hl_ctx`)."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        self.device = device
        h = c_void_p()
        check(self.lib.hl_ctx_create(c_int(device), byref(h)))
        self.handle = h
        self.torch_device = torch.device("cuda", device)
        self.stream = torch.cuda.ExternalStream(self.lib.hl_ctx_stream(self.handle), device=self.torch_device)
        # torch allocations, copies and fills issued by this thread now share the compute stream,
        # so buffers handed to the library are always ordered with the kernels that use them.
        self._previous_stream = torch.cuda.current_stream(self.torch_device)
        torch.cuda.set_stream(self.stream)
        _OPEN_STREAMS.add(self.stream.cuda_stream)

    def close(self) -> None:
        if self.handle:
            # torch must not be left pointing at a stream that is about to be destroyed: hand it back the stream
            # that was current before this context (if that one still exists), else the device's default stream
            _OPEN_STREAMS.discard(self.stream.cuda_stream)
            if torch.cuda.current_stream(self.torch_device).cuda_stream == self.stream.cuda_stream:
                previous = self._previous_stream
                default = torch.cuda.default_stream(self.torch_device)
                alive = previous.cuda_stream in _OPEN_STREAMS or previous.cuda_stream == default.cuda_stream
                torch.cuda.set_stream(previous if alive else default)
            self.lib.hl_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self) -> None:
        check(self.lib.hl_ctx_sync(self.handle))

    def device_info(self) -> DeviceInfo:
        info = DeviceInfo()
        check(self.lib.hl_device_info(self.handle, byref(info)))
        return info

    def counters(self) -> Counters:
        c = Counters()
        check(self.lib.hl_counters_get(self.handle, byref(c)))
        return c

    def set_test_hooks(self, wait_limit_ns: int = 0, gemm_skip_kblock: int = -1) -> None:
        """`hl_ctx_set_test_hooks`: shorten the bound of the GEMM's pipeline waits and/or make its producer leave
        out one k block, so that the failure path (status word, clean return) can be exercised."""
        check(self.lib.hl_ctx_set_test_hooks(self.handle, ctypes.c_ulonglong(wait_limit_ns), c_int(gemm_skip_kblock)))

    def reset_counters(self) -> None:
        check(self.lib.hl_counters_reset(self.handle))

    def empty(self, shape, dtype=torch.float32) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype, device=self.torch_device)

    def zeros(self, shape, dtype=torch.float32) -> torch.Tensor:
        return torch.zeros(shape, dtype=dtype, device=self.torch_device)


# ---- plain SGD, index ranges, index concatenation ---------------------------------------------------
def sgd_update_f32(ctx: Context, param: torch.Tensor, grad: torch.Tensor, lr: float) -> None:
    """`hl_sgd_update_f32`: param -= lr * grad in place."""
    check(ctx.lib.hl_sgd_update_f32(ctx.handle, _p(param), _p(grad), c_float(lr), c_size_t(param.numel())))


def arange_i64(ctx: Context, n: int) -> torch.Tensor:
    out = torch.empty(n, dtype=torch.int64, device=ctx.torch_device)
    check(ctx.lib.hl_arange_i64(ctx.handle, _p(out), c_size_t(n)))
    return out


def concat_i64(ctx: Context, inputs) -> torch.Tensor:
    """`hl_concat_i64`: the int64 device vectors one after the other."""
    if not inputs:
        ptrs, lens = (c_void_p * 1)(), (c_size_t * 1)()
        check(ctx.lib.hl_concat_i64(ctx.handle, ptrs, lens, c_int(0), None, c_size_t(0)))
    total = sum(int(t.numel()) for t in inputs)
    out = torch.empty(total, dtype=torch.int64, device=ctx.torch_device)
    ptrs = (c_void_p * len(inputs))(*[t.data_ptr() if t.numel() else None for t in inputs])
    lens = (c_size_t * len(inputs))(*[int(t.numel()) for t in inputs])
    check(ctx.lib.hl_concat_i64(ctx.handle, ptrs, lens, c_int(len(inputs)), _p(out), c_size_t(total)))
    return out


# ---- elementwise ------------------------------------------------------------------------------
def binary_f32(ctx: Context, op: int, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(a)
    check(ctx.lib.hl_binary_f32(ctx.handle, c_int(op), _p(a), _p(b), _p(out), c_size_t(a.numel())))
    return out


def scale_f32(ctx: Context, a: torch.Tensor, s: float) -> torch.Tensor:
    out = torch.empty_like(a)
    check(ctx.lib.hl_scale_f32(ctx.handle, _p(a), c_float(s), _p(out), c_size_t(a.numel())))
    return out


def fill_f32(ctx: Context, out: torch.Tensor, value: float) -> None:
    check(ctx.lib.hl_fill_f32(ctx.handle, _p(out), c_float(value), c_size_t(out.numel())))


def relu_f32(ctx: Context, x: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    check(ctx.lib.hl_relu_f32(ctx.handle, _p(x), _p(out), c_size_t(x.numel())))
    return out


def relu_backward_f32(ctx: Context, x: torch.Tensor, grad_out: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    check(ctx.lib.hl_relu_backward_f32(ctx.handle, _p(x), _p(grad_out), _p(out), c_size_t(x.numel())))
    return out


def cast(ctx: Context, src: torch.Tensor, dst_dtype: torch.dtype) -> torch.Tensor:
    dst = torch.empty(src.shape, dtype=dst_dtype, device=src.device)
    check(ctx.lib.hl_cast(ctx.handle, _p(src), c_int(_dt(src)), _p(dst), c_int(_DT[dst_dtype]), c_size_t(src.numel())))
    return dst


def gelu(ctx: Context, x: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    check(ctx.lib.hl_gelu(ctx.handle, _p(x), _p(out), c_int(_dt(x)), c_size_t(x.numel())))
    return out


def gelu_backward(ctx: Context, x: torch.Tensor, grad_out: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    check(ctx.lib.hl_gelu_backward(ctx.handle, _p(x), _p(grad_out), _p(out), c_int(_dt(x)), c_size_t(x.numel())))
    return out


def bias_add_f32(ctx: Context, x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    rows, cols = x.numel() // bias.numel(), bias.numel()
    check(ctx.lib.hl_bias_add_f32(ctx.handle, _p(x), _p(bias), _p(out), c_int(rows), c_int(cols)))
    return out


def bias_grad(ctx: Context, grad_out: torch.Tensor) -> torch.Tensor:
    rows, cols = grad_out.shape
    out = torch.empty(cols, dtype=torch.float32, device=grad_out.device)
    check(ctx.lib.hl_bias_grad(ctx.handle, _p(grad_out), c_int(_dt(grad_out)), _p(out), c_int(rows), c_int(cols)))
    return out


def _reduce(ctx: Context, fn, x: torch.Tensor) -> torch.Tensor:
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    check(fn(ctx.handle, _p(x), c_size_t(x.numel()), _p(out)))
    return out


def sum_f32(ctx, x):
    return _reduce(ctx, ctx.lib.hl_sum_f32, x)


def mean_f32(ctx, x):
    return _reduce(ctx, ctx.lib.hl_mean_f32, x)


def sum_squares_f32(ctx, x):
    return _reduce(ctx, ctx.lib.hl_sum_squares_f32, x)


# ---- layer norm / embedding / loss ---------------------------------------------------------------
def layer_norm_forward(ctx: Context, x, gamma, beta, eps: float = 1e-5, out_dtype=None):
    rows, feat = x.numel() // x.shape[-1], x.shape[-1]
    y = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    check(ctx.lib.hl_layer_norm_forward(ctx.handle, _p(x), c_int(_dt(x)), _p(gamma), _p(beta), _p(y), c_int(_dt(y)),
                                        _p(mean), _p(rstd), c_int(rows), c_int(feat), c_float(eps)))
    return y, mean, rstd


def layer_norm_backward(ctx: Context, x, gamma, dy, mean=None, rstd=None, residual_grad=None, want_bf16=False,
                        want_colsum=False):
    rows, feat = x.numel() // x.shape[-1], x.shape[-1]
    dx = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    dxb = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if want_bf16 else None
    dg = torch.empty(feat, dtype=torch.float32, device=x.device)
    db = torch.empty(feat, dtype=torch.float32, device=x.device)
    cs = torch.empty(feat, dtype=torch.float32, device=x.device) if want_colsum else None
    check(ctx.lib.hl_layer_norm_backward(ctx.handle, _p(x), c_int(_dt(x)), _p(gamma), _p(dy), _p(mean), _p(rstd),
                                         _p(residual_grad), _p(dx), _p(dxb), _p(dg), _p(db), _p(cs), c_int(rows),
                                         c_int(feat)))
    out = (dx, dxb, dg, db) if want_bf16 else (dx, dg, db)
    return out + (cs,) if want_colsum else out


def embedding_forward(ctx: Context, table, idx, pos_table=None, out_dtype=torch.float32):
    n, dim = idx.numel(), table.shape[1]
    period = idx.shape[-1] if pos_table is not None else 0
    out = torch.empty(tuple(idx.shape) + (dim,), dtype=out_dtype, device=table.device)
    check(ctx.lib.hl_embedding_forward(ctx.handle, _p(table), c_int(table.shape[0]), _p(idx), _p(pos_table),
                                       c_int(period), _p(out), c_int(_DT[out_dtype]), c_int(n), c_int(dim)))
    return out


def embedding_backward(ctx: Context, grad_out, idx, table_rows: int, pos_rows: int = 0):
    n, dim = idx.numel(), grad_out.shape[-1]
    gt = torch.zeros(table_rows, dim, dtype=torch.float32, device=grad_out.device)
    gp = torch.zeros(pos_rows, dim, dtype=torch.float32, device=grad_out.device) if pos_rows else None
    check(ctx.lib.hl_embedding_backward(ctx.handle, _p(grad_out), _p(idx), _p(gt), c_int(table_rows), _p(gp),
                                        c_int(pos_rows), c_int(n), c_int(dim)))
    return (gt, gp) if pos_rows else gt


def cross_entropy(ctx: Context, logits, targets, grad_scale: float = 1.0, dlogits_dtype=torch.float32,
                  want_grad: bool = True):
    rows, classes = logits.shape
    loss = torch.empty(1, dtype=torch.float32, device=logits.device)
    d = torch.empty(rows, classes, dtype=dlogits_dtype, device=logits.device) if want_grad else None
    check(ctx.lib.hl_cross_entropy(ctx.handle, _p(logits), c_longlong(logits.stride(0)), _p(targets), c_int(rows),
                                   c_int(classes), c_float(grad_scale), _p(loss), c_void_p(0), _p(d),
                                   c_int(_DT[dlogits_dtype]), c_longlong(classes)))
    return loss, d


# ---- optimizer -------------------------------------------------------------------------------------
def adamw_params(lr, beta1, beta2, eps, weight_decay, clip_scale, step) -> AdamWParams:
    """Bias corrections are computed on the host in f64 and narrowed to f32, as
    `AdamW::step_mut` does (src/nn.rs:2196-2198)."""
    return AdamWParams(lr, beta1, beta2, eps, weight_decay, clip_scale, 1.0 - beta1 ** step, 1.0 - beta2 ** step)


def adamw_update_f32(ctx: Context, param, grad, m, v, hp: AdamWParams) -> None:
    check(ctx.lib.hl_adamw_f32(ctx.handle, _p(param), _p(grad), _p(m), _p(v), c_size_t(param.numel()), byref(hp)))


def adamw_update_multi(ctx: Context, params, grads, ms, vs, hp: AdamWParams, shadows=None) -> None:
    arr = (AdamWTensor * len(params))()
    for i, (p, g, m, v) in enumerate(zip(params, grads, ms, vs)):
        arr[i] = AdamWTensor(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                             shadows[i].data_ptr() if shadows is not None else 0, p.numel())
    check(ctx.lib.hl_adamw_multi(ctx.handle, arr, c_int(len(params)), byref(hp)))


class AdamWPlan:
    """The tensor table of `adamw_update_multi`, built once and stepped every iteration (`hl_adamw_plan_*`)."""

    def __init__(self, ctx: Context, params, grads, ms, vs, shadows=None):
        self.ctx = ctx
        self._keep = (params, grads, ms, vs, shadows)  # the plan holds raw pointers
        arr = (AdamWTensor * len(params))()
        for i, (p, g, m, v) in enumerate(zip(params, grads, ms, vs)):
            arr[i] = AdamWTensor(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                                 shadows[i].data_ptr() if shadows is not None else 0, p.numel())
        h = c_void_p()
        check(ctx.lib.hl_adamw_plan_create(ctx.handle, arr, c_int(len(params)), byref(h)))
        self.handle = h

    def step(self, hp: AdamWParams) -> None:
        check(self.ctx.lib.hl_adamw_plan_step(self.ctx.handle, self.handle, byref(hp)))

    def close(self) -> None:
        if self.handle:
            self.ctx.sync()
            self.ctx.lib.hl_adamw_plan_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- matmul ------------------------------------------------------------------------------------------
def _layout(t: torch.Tensor) -> MatrixLayout:
    return MatrixLayout(t.shape[0], t.shape[1], t.stride(0), t.stride(1), 0)


def matmul_f32_strided(ctx: Context, a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
                       accumulate: bool = False) -> torch.Tensor:
    """Rank-2 f32 matmul over arbitrary strided views (e.g. `weight.t()`), f64 accumulation."""
    if out is None:
        out = torch.empty(a.shape[0], b.shape[1], dtype=torch.float32, device=a.device)
    la, lb, lo = _layout(a), _layout(b), _layout(out)
    check(ctx.lib.hl_matmul_f32_strided(ctx.handle, _p(a), byref(la), _p(b), byref(lb), _p(out), byref(lo),
                                        c_int(1 if accumulate else 0)))
    return out


SPLIT_HI_MID_LO, SPLIT_HI_HI_LO, SPLIT_HI_LO, SPLIT_STACK_ROWS = 0, 1, 2, 4


def gemm_bf16(ctx: Context, a: torch.Tensor, b: torch.Tensor, m: int, n: int, k: int, a_layout=K_MAJOR,
              b_layout=K_MAJOR, epilogue=EPI_NONE, out_dtype=torch.bfloat16, bias=None, aux_in=None,
              want_aux_out=False, split_k=0, out=None, a_k_period=0, b_k_period=0):
    """C[m,n] = A·B with per-operand storage order; see `hl_gemm_bf16` in the C header."""
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    aux_out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device) if want_aux_out else None
    desc = GemmDesc(m, n, k, a_layout, b_layout, a.stride(0), b.stride(0), out.stride(0), epilogue, _DT[out.dtype],
                    split_k, aux_in.stride(0) if aux_in is not None else 0, n if want_aux_out else 0, a_k_period, b_k_period)
    check(ctx.lib.hl_gemm_bf16(ctx.handle, byref(desc), _p(a), _p(b), _p(out), _p(bias), _p(aux_in), _p(aux_out)))
    return (out, aux_out) if want_aux_out else out


def gemm_bf16_plan(ctx: Context, m: int, n: int, k: int, epilogue=EPI_NONE, out_dtype=torch.float32, split_k=0):
    """`hl_gemm_bf16_plan`: (splits, dealt tiles, scratch bytes) of the work split for this shape."""
    desc = GemmDesc(m, n, k, K_MAJOR, K_MAJOR, k, k, n, epilogue, _DT[out_dtype], split_k, 0, 0)
    splits, dealt, need = c_int(), c_int(), c_size_t()
    check(ctx.lib.hl_gemm_bf16_plan(ctx.handle, byref(desc), byref(splits), byref(dealt), byref(need)))
    return splits.value, dealt.value, need.value


def gemm_bf16_static_scratch(ctx: Context, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, m: int, n: int,
                             k: int, a_layout=K_MAJOR, b_layout=K_MAJOR, split_k=0) -> torch.Tensor:
    """`hl_gemm_bf16_static_scratch`: the split-K GEMM with its partial sums in the library's fixed
    32 MiB array, for callers that must not reach the CUDA allocator.  `out` is supplied by the
    caller (this wrapper allocates nothing either)."""
    desc = GemmDesc(m, n, k, a_layout, b_layout, a.stride(0), b.stride(0), out.stride(0), EPI_NONE, _DT[out.dtype],
                    split_k, 0, 0)
    check(ctx.lib.hl_gemm_bf16_static_scratch(ctx.handle, byref(desc), _p(a), _p(b), _p(out), _p(None), _p(None),
                                              _p(None)))
    return out


# ---- attention, f32 route ----------------------------------------------------------------------------
def causal_attention_f32_forward(ctx: Context, q, k, v, n_heads: int):
    B, T, C = q.shape
    out = torch.empty_like(q)
    probs = torch.empty(B, n_heads, T, T, dtype=torch.float32, device=q.device)
    check(ctx.lib.hl_causal_attention_f32_forward(ctx.handle, _p(q), _p(k), _p(v), _p(out), _p(probs), c_int(B),
                                                  c_int(T), c_int(C), c_int(n_heads)))
    return out, probs


def causal_attention_f32_backward(ctx: Context, q, k, v, probs, grad_out, n_heads: int):
    B, T, C = q.shape
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    check(ctx.lib.hl_causal_attention_f32_backward(ctx.handle, _p(q), _p(k), _p(v), _p(probs), _p(grad_out), _p(dq),
                                                   _p(dk), _p(dv), c_int(B), c_int(T), c_int(C), c_int(n_heads)))
    return dq, dk, dv


# ---- attention, bf16 flash route ----------------------------------------------------------------------
def flash_attention_forward(ctx: Context, q, k, v, batch: int, time: int, n_heads: int):
    """q, k, v: bf16 `[batch*time, C]` views (possibly column slices of one fused buffer with the
    same row stride).  Returns (out bf16 `[batch*time, C]`, lse f32 `[batch, heads, time]`)."""
    C = q.shape[1]
    out = torch.empty(batch * time, C, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(batch, n_heads, time, dtype=torch.float32, device=q.device)
    check(ctx.lib.hl_flash_attention_forward(ctx.handle, _p(q), _p(k), _p(v), c_longlong(q.stride(0)), _p(out),
                                             c_longlong(out.stride(0)), _p(lse), c_int(batch), c_int(time),
                                             c_int(n_heads), c_int(C // n_heads)))
    return out, lse


def flash_attention_backward(ctx: Context, q, k, v, out, dout, lse, batch: int, time: int, n_heads: int):
    """Returns one fused bf16 gradient buffer `[batch*time, 3C]` holding dq | dk | dv."""
    C = q.shape[1]
    dqkv = torch.empty(batch * time, 3 * C, dtype=torch.bfloat16, device=q.device)
    dq, dk, dv = dqkv[:, :C], dqkv[:, C:2 * C], dqkv[:, 2 * C:]
    check(ctx.lib.hl_flash_attention_backward(
        ctx.handle, _p(q), _p(k), _p(v), c_longlong(q.stride(0)), _p(out), c_longlong(out.stride(0)), _p(dout),
        c_longlong(dout.stride(0)), _p(lse), _p(dq), _p(dk), _p(dv), c_longlong(dqkv.stride(0)), c_int(batch),
        c_int(time), c_int(n_heads), c_int(C // n_heads)))
    return dqkv


# ---- product-key memory layer -------------------------------------------------------------------------
def topk_rows(ctx: Context, scores: torch.Tensor, k: int) -> torch.Tensor:
    rows, cols = scores.shape
    out = torch.empty(rows, k, dtype=torch.int64, device=scores.device)
    check(ctx.lib.hl_topk_rows_f32(ctx.handle, _p(scores), _p(out), c_int(rows), c_int(cols), c_int(k)))
    return out


def product_key_side_scores(ctx: Context, query, left_keys, right_keys):
    tokens, key_dim = query.shape
    side = left_keys.shape[0]
    ls = torch.empty(tokens, side, dtype=torch.float32, device=query.device)
    rs = torch.empty(tokens, side, dtype=torch.float32, device=query.device)
    check(ctx.lib.hl_product_key_side_scores_f32(ctx.handle, _p(query), c_longlong(query.stride(0)), _p(left_keys),
                                                 _p(right_keys), _p(ls), _p(rs), c_int(tokens), c_int(side),
                                                 c_int(key_dim)))
    return ls, rs


def product_key_topk_from_side_scores(ctx: Context, left_scores, right_scores, top_k: int, beam: int):
    tokens, side = left_scores.shape
    out = torch.empty(tokens, top_k, dtype=torch.int64, device=left_scores.device)
    check(ctx.lib.hl_product_key_topk_from_side_scores(ctx.handle, _p(left_scores), _p(right_scores), _p(out),
                                                       c_int(tokens), c_int(side), c_int(top_k), c_int(beam)))
    return out


def product_key_split_rows(ctx: Context, rows: torch.Tensor, side: int):
    left, right = torch.empty_like(rows), torch.empty_like(rows)
    check(ctx.lib.hl_product_key_split_rows(ctx.handle, _p(rows), _p(left), _p(right), c_longlong(rows.numel()),
                                            c_int(side)))
    return left, right


def memory_selected_scores_forward(ctx: Context, indices, query, left_or_keys, right_keys=None):
    tokens, top_k = indices.shape
    key_dim = query.shape[1]
    side = left_or_keys.shape[0] if right_keys is not None else 0
    slots = side * side if side else left_or_keys.shape[0]
    out = torch.empty(tokens, top_k, dtype=torch.float32, device=query.device)
    check(ctx.lib.hl_memory_selected_scores_forward(ctx.handle, _p(indices), _p(query), c_longlong(query.stride(0)),
                                                    _p(left_or_keys), _p(right_keys), _p(out), c_int(tokens),
                                                    c_int(top_k), c_int(side), c_int(key_dim), c_int(slots)))
    return out


def memory_selected_scores_backward(ctx: Context, indices, query, left_or_keys, right_keys, grad_scores):
    tokens, top_k = indices.shape
    key_dim = query.shape[1]
    side = left_or_keys.shape[0] if right_keys is not None else 0
    slots = side * side if side else left_or_keys.shape[0]
    dq = torch.empty_like(query)
    dl = torch.zeros_like(left_or_keys)
    dr = torch.zeros_like(right_keys) if right_keys is not None else None
    check(ctx.lib.hl_memory_selected_scores_backward(
        ctx.handle, _p(indices), _p(query), c_longlong(query.stride(0)), _p(left_or_keys), _p(right_keys),
        _p(grad_scores), _p(dq), c_longlong(dq.stride(0)), _p(dl), _p(dr), c_int(tokens), c_int(top_k), c_int(side),
        c_int(key_dim), c_int(slots)))
    return dq, dl, dr


def softmax_rows(ctx: Context, x):
    y = torch.empty_like(x)
    check(ctx.lib.hl_softmax_rows_f32(ctx.handle, _p(x), _p(y), c_int(x.shape[0]), c_int(x.shape[1])))
    return y


def softmax_rows_backward(ctx: Context, y, grad_y):
    gx = torch.empty_like(y)
    check(ctx.lib.hl_softmax_rows_backward_f32(ctx.handle, _p(y), _p(grad_y), _p(gx), c_int(y.shape[0]),
                                               c_int(y.shape[1])))
    return gx


def memory_weighted_value_forward(ctx: Context, indices, weights, values):
    tokens, top_k = indices.shape
    rows, dim = values.shape
    out = torch.empty(tokens, dim, dtype=torch.float32, device=values.device)
    check(ctx.lib.hl_memory_weighted_value_forward(ctx.handle, _p(indices), _p(weights), _p(values), _p(out),
                                                   c_int(tokens), c_int(top_k), c_int(rows), c_int(dim)))
    return out


def memory_weighted_value_backward(ctx: Context, indices, weights, values, grad_out):
    tokens, top_k = indices.shape
    rows, dim = values.shape
    dw = torch.empty_like(weights)
    dv = torch.zeros_like(values)
    check(ctx.lib.hl_memory_weighted_value_backward(ctx.handle, _p(indices), _p(weights), _p(values), _p(grad_out),
                                                    _p(dw), _p(dv), c_int(tokens), c_int(top_k), c_int(rows),
                                                    c_int(dim)))
    return dw, dv


def sparse_adamw_rows(ctx: Context, param, grad, m, v, selected_rows, hp: AdamWParams, row_mask=None,
                      zero_grad_rows: bool = False) -> None:
    rows, row_dim = param.shape
    flags = torch.zeros(rows, dtype=torch.uint8, device=param.device)
    check(ctx.lib.hl_sparse_adamw_rows_f32(ctx.handle, _p(param), _p(grad), _p(m), _p(v), _p(selected_rows),
                                           c_longlong(selected_rows.numel()), _p(row_mask), _p(flags), c_int(rows),
                                           c_int(row_dim), byref(hp), c_int(1 if zero_grad_rows else 0)))


# ---- row masks and packed rows (sparse data-parallel exchange) ----------------------------------------
def mark_rows(ctx: Context, selected_rows: torch.Tensor, rows: int, row_mask=None) -> torch.Tensor:
    """Byte mask with a 1 for every selected row (that the optional mask lets through)."""
    flags = torch.zeros(rows, dtype=torch.uint8, device=selected_rows.device)
    check(ctx.lib.hl_mark_rows_u8(ctx.handle, _p(selected_rows), c_longlong(selected_rows.numel()), _p(row_mask), _p(flags),
                                  c_int(rows)))
    return flags


def mask_to_indices(ctx: Context, mask: torch.Tensor) -> torch.Tensor:
    """Ascending row numbers of the non-zero bytes of `mask` (int64)."""
    rows = mask.numel()
    out = torch.empty(rows, dtype=torch.int64, device=mask.device)
    count = torch.zeros(1, dtype=torch.int32, device=mask.device)
    check(ctx.lib.hl_mask_to_indices_u8(ctx.handle, _p(mask), c_int(rows), _p(out), _p(count)))
    ctx.sync()
    return out[:int(count.item())]


def gather_rows(ctx: Context, src: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    out = torch.empty(indices.numel(), src.shape[1], dtype=torch.float32, device=src.device)
    check(ctx.lib.hl_gather_rows_f32(ctx.handle, _p(src), _p(indices), c_int(indices.numel()), c_int(src.shape[1]), _p(out)))
    return out


def scatter_rows(ctx: Context, packed: torch.Tensor, indices: torch.Tensor, dst: torch.Tensor) -> None:
    check(ctx.lib.hl_scatter_rows_f32(ctx.handle, _p(packed), _p(indices), c_int(indices.numel()), c_int(dst.shape[1]), _p(dst)))


def sparse_rows_sum_squares(ctx: Context, grad: torch.Tensor, selected_rows: torch.Tensor, row_mask=None) -> float:
    rows, row_dim = grad.shape
    flags = torch.zeros(rows, dtype=torch.uint8, device=grad.device)
    total = torch.zeros(1, dtype=torch.float64, device=grad.device)
    check(ctx.lib.hl_sparse_rows_sum_squares_f32(ctx.handle, _p(grad), _p(selected_rows), c_longlong(selected_rows.numel()),
                                                 _p(row_mask), _p(flags), c_int(rows), c_int(row_dim), _p(total)))
    ctx.sync()
    return float(total.item())


def memory_access_count_rows(ctx: Context, selected_rows: torch.Tensor, slots: int, counts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-access histogram of int64 `selected_rows` (`memory_access_count_rows_i64_u64`,
    heirloom-kernels/src/cuda.rs:2052-2088).  Counts are 64-bit; torch has no unsigned 64-bit arithmetic, so
    they live in an int64 tensor (same bits below 2^63).  Pass `counts` to keep adding to a histogram."""
    if slots <= 0:
        raise HeirloomError("memory_access_count_rows_i64_u64 requires non-zero memory_slots")
    if counts is None:
        counts = torch.zeros(slots, dtype=torch.int64, device=selected_rows.device)
    flat = selected_rows.reshape(-1).contiguous()
    check(ctx.lib.hl_memory_access_count_rows_i64_u64(ctx.handle, _p(flat), c_longlong(flat.numel()), c_int(slots), _p(counts)))
    ctx.sync()  # surfaces a bad-index status as an error, like the reference's status check
    return counts

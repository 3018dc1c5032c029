"""Generates `include/heirloom_b200.rs` from `include/heirloom_b200.h`: the Rust side of the boundary.

The reference binds its GPU backend inside the `heirloom-kernels` crate (`heirloom-kernels/src/cuda.rs`; the root
crate is `#![forbid(unsafe_code)]`).  The generated file is what a maintainer would drop there as `src/b200.rs`:

* every struct of the header as `#[repr(C)]`, every constant, every entry point in one `extern "C"` block
  (mechanical, from the header's prototypes), and
* safe wrappers that keep the names, argument meaning and `CudaResult` error type of today's
  `heirloom_kernels::cuda::*` functions for the ops on the training-step path (written out below in `SAFE_WRAPPERS`).

This image has no Rust toolchain, so the output is checked here only for completeness against the header
(`tests/test_abi.py`); it has not been compiled.

Usage: python include/make_rust_shim.py            # rewrites include/heirloom_b200.rs
"""
from __future__ import annotations

import re
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
HEADER = HERE / "heirloom_b200.h"
OUT = HERE / "heirloom_b200.rs"

SCALARS = {
    "int": "i32", "unsigned": "u32", "unsigned int": "u32", "long long": "i64", "unsigned long long": "u64",
    "size_t": "usize", "float": "f32", "double": "f64", "uint64_t": "u64", "int64_t": "i64", "uint32_t": "u32",
    "int32_t": "i32", "uint8_t": "u8", "unsigned char": "u8", "char": "c_char", "void": "c_void",
}


def strip_comments(text: str) -> str:
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


def rust_name(c_name: str) -> str:
    """hl_gemm_desc / hl_counters_t -> HlGemmDesc / HlCounters."""
    base = c_name[:-2] if c_name.endswith("_t") else c_name
    return "".join(p.capitalize() for p in base.split("_"))


def map_type(c_type: str, known: set) -> str:
    t = " ".join(c_type.replace("*", " * ").split())
    # peel pointers from the right: "const int64_t * const *" -> ["const int64_t", "const"]
    parts = [p.strip() for p in t.split("*")]
    base, ptr_quals = parts[0], parts[1:]
    const_base = False
    words = [w for w in base.split() if w not in ("struct",)]
    if "const" in words:
        const_base = True
        words = [w for w in words if w != "const"]
    name = " ".join(words)
    if name in SCALARS:
        rust = SCALARS[name]
    elif name in known:
        rust = rust_name(name)
    else:
        raise ValueError(f"unknown C type {c_type!r}")
    # the first '*' binds to the base type's constness, later ones to the qualifier written before them
    consts = [const_base] + ["const" in q.split() for q in ptr_quals[:-1]]
    for is_const in consts[: len(ptr_quals)]:
        rust = ("*const " if is_const else "*mut ") + rust
    return rust


def parse(header: str):
    text = strip_comments(header)
    defines = [(m.group(1), m.group(2)) for m in re.finditer(r"#define\s+(HL_[A-Z0-9_]+)\s+\(?(-?\d+)\)?", text)]
    enums = []
    for m in re.finditer(r"enum\s*\{([^}]*)\}\s*;", text):
        value = -1
        for item in m.group(1).split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                name, v = (s.strip() for s in item.split("="))
                value = int(v)
            else:
                name, value = item, value + 1
            enums.append((name, value))
    consts = dict(defines + [(n, str(v)) for n, v in enums])
    opaque = re.findall(r"typedef\s+struct\s+(\w+)\s+\1\s*;", text)
    structs = []
    for m in re.finditer(r"typedef\s+struct\s*\{([^}]*)\}\s*(\w+)\s*;", text):
        fields = []
        for decl in m.group(1).split(";"):
            decl = " ".join(decl.split())
            if not decl:
                continue
            # "int m, n, k" / "double ms[HL_PROF_CATEGORIES]" / "const float* params"
            first, *rest = [d.strip() for d in decl.split(",")]
            mm = re.match(r"(.*?)(\w+)(\[[^\]]*\])?$", first)
            ctype = mm.group(1).strip()
            names = [(mm.group(2), mm.group(3))]
            for r in rest:
                stars = r.count("*")
                r2 = r.replace("*", "").strip()
                m2 = re.match(r"(\w+)(\[[^\]]*\])?$", r2)
                names.append(("*" * stars + m2.group(1), m2.group(2)))
            for n, arr in names:
                ct = ctype + "*" * n.count("*")
                fields.append((n.replace("*", ""), ct, arr[1:-1] if arr else None))
        structs.append((m.group(2), fields))
    body = re.sub(r"typedef\s+struct\s*\{[^}]*\}\s*\w+\s*;", " ", text)
    body = re.sub(r"enum\s*\{[^}]*\}\s*;", " ", body)
    funcs = []
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(hl_\w+)\s*\(([^)]*)\)\s*;", body):
        ret, name, args = " ".join(m.group(1).split()), m.group(2), " ".join(m.group(3).split())
        if ret.startswith("typedef"):
            continue
        params = []
        if args and args != "void":
            for i, a in enumerate(args.split(",")):
                a = a.strip()
                arr = re.search(r"\[[^\]]*\]$", a)
                if arr:
                    a = a[: arr.start()].strip()
                mm = re.match(r"(.*?)(\w+)$", a)
                ctype, pname = mm.group(1).strip(), mm.group(2)
                if not ctype:  # unnamed parameter
                    ctype, pname = a, f"arg{i}"
                if arr:
                    ctype += "*"
                params.append((pname, ctype))
        funcs.append((name, ret, params))
    return consts, defines, enums, opaque, structs, funcs


SAFE_WRAPPERS = r'''
// ---------------------------------------------------------------------------------------------------------------
// Safe layer: the names and meaning of today's `heirloom_kernels::cuda::*` wrappers (file:line in the Heirloom tree).
// `CudaBuffer`, `CudaResult`, `CudaError` are the crate's own types (cuda.rs:259-280, :652-656); a buffer here is a
// reference-counted `hl_buffer` plus the element bookkeeping the crate already keeps.
// ---------------------------------------------------------------------------------------------------------------
use std::cell::RefCell;
use std::collections::HashMap;
use std::rc::Rc;

thread_local! {
    // one context per (thread, device), as the reference caches one stream per context per thread (cuda.rs:7653-7681)
    static CONTEXTS: RefCell<HashMap<i32, *mut HlCtx>> = RefCell::new(HashMap::new());
}

fn check(rc: i32) -> CudaResult<()> {
    if rc == HL_OK {
        return Ok(());
    }
    let msg = unsafe { std::ffi::CStr::from_ptr(hl_last_error()) }.to_string_lossy().into_owned();
    Err(CudaError::new(msg))
}

fn ctx_for(device_ordinal: i32) -> CudaResult<*mut HlCtx> {
    CONTEXTS.with(|map| {
        if let Some(ctx) = map.borrow().get(&device_ordinal) {
            return Ok(*ctx);
        }
        let mut ctx: *mut HlCtx = std::ptr::null_mut();
        check(unsafe { hl_ctx_create(device_ordinal, &mut ctx) })?;
        map.borrow_mut().insert(device_ordinal, ctx);
        Ok(ctx)
    })
}

struct Allocation {
    handle: *mut HlBuffer,
    device_ordinal: i32,
}
impl Drop for Allocation {
    fn drop(&mut self) {
        // the library frees in stream order, like the pending-release list of cuda.rs:7870-7922
        unsafe { hl_buffer_release(self.handle) };
    }
}

#[derive(Clone)]
pub struct CudaBuffer {
    inner: Rc<Allocation>,
    len: usize,
    element_size: usize,
}

impl CudaBuffer {
    pub fn uninit_bytes(device_ordinal: i32, len: usize, element_size: usize) -> CudaResult<Self> {
        let bytes = len.checked_mul(element_size).ok_or_else(|| CudaError::new("CUDA buffer byte length overflow"))?;
        let ctx = ctx_for(device_ordinal)?;
        let mut handle: *mut HlBuffer = std::ptr::null_mut();
        check(unsafe { hl_buffer_alloc(ctx, bytes.max(1), &mut handle) })?;
        Ok(Self { inner: Rc::new(Allocation { handle, device_ordinal }), len, element_size })
    }
    fn from_slice<T: Copy>(device_ordinal: i32, values: &[T]) -> CudaResult<Self> {
        let out = Self::uninit_bytes(device_ordinal, values.len(), std::mem::size_of::<T>())?;
        check(unsafe {
            hl_memcpy_h2d(ctx_for(device_ordinal)?, out.ptr(), values.as_ptr() as *const c_void, out.byte_len())
        })?;
        Ok(out)
    }
    fn to_vec<T: Copy + Default>(&self) -> CudaResult<Vec<T>> {
        let mut host = vec![T::default(); self.len];
        // waits for the compute stream first, as the reference's device-to-host copies do (cuda.rs:836)
        check(unsafe {
            hl_memcpy_d2h(ctx_for(self.device_ordinal())?, host.as_mut_ptr() as *mut c_void, self.ptr(), self.byte_len())
        })?;
        Ok(host)
    }
    pub fn from_f32(device_ordinal: i32, values: &[f32]) -> CudaResult<Self> { Self::from_slice(device_ordinal, values) }
    pub fn from_i64(device_ordinal: i32, values: &[i64]) -> CudaResult<Self> { Self::from_slice(device_ordinal, values) }
    pub fn from_u16(device_ordinal: i32, values: &[u16]) -> CudaResult<Self> { Self::from_slice(device_ordinal, values) }
    pub fn from_u8(device_ordinal: i32, values: &[u8]) -> CudaResult<Self> { Self::from_slice(device_ordinal, values) }
    pub fn to_f32(&self) -> CudaResult<Vec<f32>> { self.to_vec() }
    pub fn to_i64(&self) -> CudaResult<Vec<i64>> { self.to_vec() }
    pub fn to_u16(&self) -> CudaResult<Vec<u16>> { self.to_vec() }
    pub fn len(&self) -> usize { self.len }
    pub fn is_empty(&self) -> bool { self.len == 0 }
    pub fn element_size(&self) -> usize { self.element_size }
    pub fn byte_len(&self) -> usize { self.len * self.element_size }
    pub fn device_ordinal(&self) -> i32 { self.inner.device_ordinal }
    fn ptr(&self) -> *mut c_void { unsafe { hl_buffer_ptr(self.inner.handle) } }
}

fn ensure(buffer: &CudaBuffer, element_size: usize, label: &str) -> CudaResult<()> {
    if buffer.element_size() != element_size {
        return Err(CudaError::new(format!("{label} expects {element_size}-byte elements, got {}", buffer.element_size())));
    }
    Ok(())
}

fn dim(value: usize, label: &str) -> CudaResult<i32> {
    i32::try_from(value).map_err(|_| CudaError::new(format!("{label} exceeds the launch limit")))
}

/// cuda.rs add/sub/mul/div_f32_buffers (kernels.ptx:6-141)
fn binary(op: i32, lhs: &CudaBuffer, rhs: &CudaBuffer, label: &str) -> CudaResult<CudaBuffer> {
    ensure(lhs, 4, label)?;
    ensure(rhs, 4, label)?;
    if lhs.len() != rhs.len() || lhs.device_ordinal() != rhs.device_ordinal() {
        return Err(CudaError::new(format!("{label} expects equal lengths on one device")));
    }
    let out = CudaBuffer::uninit_bytes(lhs.device_ordinal(), lhs.len(), 4)?;
    check(unsafe {
        hl_binary_f32(ctx_for(lhs.device_ordinal())?, op, lhs.ptr() as *const f32, rhs.ptr() as *const f32,
                      out.ptr() as *mut f32, lhs.len())
    })?;
    Ok(out)
}
pub fn add_f32_buffers(lhs: &CudaBuffer, rhs: &CudaBuffer) -> CudaResult<CudaBuffer> { binary(HL_ADD, lhs, rhs, "add_f32_buffers") }
pub fn sub_f32_buffers(lhs: &CudaBuffer, rhs: &CudaBuffer) -> CudaResult<CudaBuffer> { binary(HL_SUB, lhs, rhs, "sub_f32_buffers") }
pub fn mul_f32_buffers(lhs: &CudaBuffer, rhs: &CudaBuffer) -> CudaResult<CudaBuffer> { binary(HL_MUL, lhs, rhs, "mul_f32_buffers") }
pub fn div_f32_buffers(lhs: &CudaBuffer, rhs: &CudaBuffer) -> CudaResult<CudaBuffer> { binary(HL_DIV, lhs, rhs, "div_f32_buffers") }

/// cuda.rs gelu_f32_buffer / gelu_backward_f32_buffers (kernels.ptx:4786-4907)
pub fn gelu_f32_buffer(input: &CudaBuffer) -> CudaResult<CudaBuffer> {
    ensure(input, 4, "gelu_f32_buffer")?;
    let out = CudaBuffer::uninit_bytes(input.device_ordinal(), input.len(), 4)?;
    check(unsafe { hl_gelu(ctx_for(input.device_ordinal())?, input.ptr(), out.ptr(), HL_F32, input.len()) })?;
    Ok(out)
}
pub fn gelu_backward_f32_buffers(input: &CudaBuffer, grad_out: &CudaBuffer) -> CudaResult<CudaBuffer> {
    ensure(input, 4, "gelu_backward_f32_buffers")?;
    let out = CudaBuffer::uninit_bytes(input.device_ordinal(), input.len(), 4)?;
    check(unsafe {
        hl_gelu_backward(ctx_for(input.device_ordinal())?, input.ptr(), grad_out.ptr(), out.ptr(), HL_F32, input.len())
    })?;
    Ok(out)
}

/// cuda.rs f32_to_bf16_bits_buffer / bf16_bits_to_f32_buffer (kernels.ptx:174-237; storage.rs:440-449)
pub fn f32_to_bf16_bits_buffer(input: &CudaBuffer) -> CudaResult<CudaBuffer> {
    ensure(input, 4, "f32_to_bf16_bits_buffer")?;
    let out = CudaBuffer::uninit_bytes(input.device_ordinal(), input.len(), 2)?;
    check(unsafe { hl_cast(ctx_for(input.device_ordinal())?, input.ptr(), HL_F32, out.ptr(), HL_BF16, input.len()) })?;
    Ok(out)
}
pub fn bf16_bits_to_f32_buffer(input: &CudaBuffer) -> CudaResult<CudaBuffer> {
    ensure(input, 2, "bf16_bits_to_f32_buffer")?;
    let out = CudaBuffer::uninit_bytes(input.device_ordinal(), input.len(), 4)?;
    check(unsafe { hl_cast(ctx_for(input.device_ordinal())?, input.ptr(), HL_BF16, out.ptr(), HL_F32, input.len()) })?;
    Ok(out)
}

/// cuda.rs layer_norm_forward_f32_buffers (kernels.ptx:3260-3384)
pub fn layer_norm_forward_f32_buffers(x: &CudaBuffer, gamma: &CudaBuffer, beta: &CudaBuffer, rows: usize,
                                      features: usize, eps: f32) -> CudaResult<CudaBuffer> {
    ensure(x, 4, "layer_norm_forward_f32_buffers")?;
    let out = CudaBuffer::uninit_bytes(x.device_ordinal(), rows * features, 4)?;
    check(unsafe {
        hl_layer_norm_forward(ctx_for(x.device_ordinal())?, x.ptr(), HL_F32, gamma.ptr() as *const f32,
                              beta.ptr() as *const f32, out.ptr(), HL_F32, std::ptr::null_mut(), std::ptr::null_mut(),
                              dim(rows, "layer norm rows")?, dim(features, "layer norm features")?, eps)
    })?;
    Ok(out)
}

/// cuda.rs embedding_f32_i64_buffers (kernels.ptx:1660-1713); rows that are out of range are reported by the next sync
pub fn embedding_f32_i64_buffers(weight: &CudaBuffer, indices: &CudaBuffer, vocab: usize, dim_: usize) -> CudaResult<CudaBuffer> {
    ensure(weight, 4, "embedding_f32_i64_buffers weight")?;
    ensure(indices, 8, "embedding_f32_i64_buffers indices")?;
    let out = CudaBuffer::uninit_bytes(weight.device_ordinal(), indices.len() * dim_, 4)?;
    let ctx = ctx_for(weight.device_ordinal())?;
    check(unsafe {
        hl_embedding_forward(ctx, weight.ptr() as *const f32, dim(vocab, "vocab")?, indices.ptr() as *const i64,
                             std::ptr::null(), 0, out.ptr(), HL_F32, dim(indices.len(), "tokens")?, dim(dim_, "dim")?)
    })?;
    check(unsafe { hl_ctx_sync(ctx) })?; // the reference reads its status word after the launch (cuda.rs:7184-7193)
    Ok(out)
}

/// cuda.rs matmul_bf16_tensor_core_rhs_transposed_f32_buffers (cuda.rs:4215-4386): C[m,n] = A[m,k] · B[n,k]ᵀ,
/// bf16 operands, f32 result; pad / crop / transpose kernels are gone, ragged edges are handled by the tile loads
pub fn matmul_bf16_tensor_core_rhs_transposed_f32_buffers(lhs_bf16: &CudaBuffer, rhs_bf16: &CudaBuffer, m: usize,
                                                          n: usize, k: usize) -> CudaResult<CudaBuffer> {
    ensure(lhs_bf16, 2, "matmul_bf16_tensor_core lhs")?;
    ensure(rhs_bf16, 2, "matmul_bf16_tensor_core rhs")?;
    let out = CudaBuffer::uninit_bytes(lhs_bf16.device_ordinal(), m * n, 4)?;
    let desc = HlGemmDesc { m: dim(m, "m")?, n: dim(n, "n")?, k: dim(k, "k")?, a_layout: HL_K_MAJOR, b_layout: HL_K_MAJOR,
                            lda: k as i64, ldb: k as i64, ldc: n as i64, epilogue: HL_EPI_NONE, out_dtype: HL_F32,
                            split_k: 0, ld_aux_in: 0, ld_aux_out: 0, a_k_period: 0, b_k_period: 0 };
    check(unsafe {
        hl_gemm_bf16(ctx_for(lhs_bf16.device_ordinal())?, &desc, lhs_bf16.ptr(), rhs_bf16.ptr(), out.ptr(),
                     std::ptr::null(), std::ptr::null(), std::ptr::null_mut())
    })?;
    Ok(out)
}

/// cuda.rs causal_attention_bf16_flash_tensor_core_forward_f32_buffers (cuda.rs:5283-5420): returns (output, lse)
pub fn causal_attention_bf16_flash_forward_buffers(q: &CudaBuffer, k: &CudaBuffer, v: &CudaBuffer,
                                                   dims: CausalAttentionDims) -> CudaResult<(CudaBuffer, CudaBuffer)> {
    let channels = dims.channels;  // heads interleaved along the channel dimension (src/tensor.rs:5156-5177)
    let head_dim = channels / dims.n_heads;
    let out = CudaBuffer::uninit_bytes(q.device_ordinal(), dims.batch * dims.time * channels, 2)?;
    let lse = CudaBuffer::uninit_bytes(q.device_ordinal(), dims.batch * dims.n_heads * dims.time, 4)?;
    check(unsafe {
        hl_flash_attention_forward(ctx_for(q.device_ordinal())?, q.ptr(), k.ptr(), v.ptr(), channels as i64, out.ptr(),
                                   channels as i64, lse.ptr() as *mut f32, dim(dims.batch, "batch")?,
                                   dim(dims.time, "time")?, dim(dims.n_heads, "heads")?, dim(head_dim, "head_dim")?)
    })?;
    Ok((out, lse))
}

/// cuda.rs sgd_update_f32_buffer (cuda.rs:6280-6303)
pub fn sgd_update_f32_buffer(param: &CudaBuffer, grad: &CudaBuffer, lr: f32) -> CudaResult<()> {
    ensure(param, 4, "sgd_update_f32_buffer param")?;
    ensure(grad, 4, "sgd_update_f32_buffer grad")?;
    check(unsafe {
        hl_sgd_update_f32(ctx_for(param.device_ordinal())?, param.ptr() as *mut f32, grad.ptr() as *const f32, lr, param.len())
    })
}

/// cuda.rs adamw_update_f32_buffers (cuda.rs:6305-6334; kernels.ptx:390-468): same operation order as the reference kernel
pub fn adamw_update_f32_buffers(param: &CudaBuffer, grad: &CudaBuffer, m: &CudaBuffer, v: &CudaBuffer,
                                params: AdamWParams) -> CudaResult<()> {
    let hp = HlAdamwParams { lr: params.lr, beta1: params.beta1, beta2: params.beta2, eps: params.eps,
                             weight_decay: params.weight_decay, clip_scale: params.clip_scale,
                             bias_correction1: params.bias_correction1, bias_correction2: params.bias_correction2 };
    check(unsafe {
        hl_adamw_f32(ctx_for(param.device_ordinal())?, param.ptr() as *mut f32, grad.ptr() as *const f32,
                     m.ptr() as *mut f32, v.ptr() as *mut f32, param.len(), &hp)
    })
}

/// cuda.rs i64_arange_buffer (cuda.rs:2090-2103)
pub fn i64_arange_buffer(device_ordinal: i32, len: usize) -> CudaResult<CudaBuffer> {
    let out = CudaBuffer::uninit_bytes(device_ordinal, len, 8)?;
    check(unsafe { hl_arange_i64(ctx_for(device_ordinal)?, out.ptr() as *mut i64, len) })?;
    Ok(out)
}

/// cuda.rs concat_i64_buffers (cuda.rs:6437-6490)
pub fn concat_i64_buffers(inputs: &[CudaBuffer]) -> CudaResult<CudaBuffer> {
    let first = inputs.first().ok_or_else(|| CudaError::new("concat_i64_buffers requires at least one input buffer"))?;
    let total: usize = inputs.iter().map(|b| b.len()).sum();
    let out = CudaBuffer::uninit_bytes(first.device_ordinal(), total, 8)?;
    let ptrs: Vec<*const i64> = inputs.iter().map(|b| b.ptr() as *const i64).collect();
    let lens: Vec<usize> = inputs.iter().map(|b| b.len()).collect();
    check(unsafe {
        hl_concat_i64(ctx_for(first.device_ordinal())?, ptrs.as_ptr(), lens.as_ptr(), dim(inputs.len(), "inputs")?,
                      out.ptr() as *mut i64, total)
    })?;
    Ok(out)
}

/// cuda.rs memory_product_key_topk_from_side_scores (kernels.ptx product-key family): i64 slots [tokens, top_k]
pub fn product_key_topk_from_side_scores_buffers(left: &CudaBuffer, right: &CudaBuffer, tokens: usize, side: usize,
                                                 top_k: usize, beam: usize) -> CudaResult<CudaBuffer> {
    let out = CudaBuffer::uninit_bytes(left.device_ordinal(), tokens * top_k, 8)?;
    check(unsafe {
        hl_product_key_topk_from_side_scores(ctx_for(left.device_ordinal())?, left.ptr() as *const f32,
                                             right.ptr() as *const f32, out.ptr() as *mut i64, dim(tokens, "tokens")?,
                                             dim(side, "side")?, dim(top_k, "top_k")?, dim(beam, "beam")?)
    })?;
    Ok(out)
}

/// NcclCommunicator::all_reduce_sum_in_place_f32 (cuda.rs:8049-8233) on the context's collective stream
pub fn nccl_all_reduce_sum_in_place_f32(buffer: &CudaBuffer) -> CudaResult<()> {
    ensure(buffer, 4, "all_reduce_sum_in_place_f32")?;
    check(unsafe { hl_nccl_allreduce_f32(ctx_for(buffer.device_ordinal())?, buffer.ptr() as *mut f32, buffer.len()) })
}

/// The loop body of `train-lm` (src/bin/heirloom/commands/training.rs:125-167) as one call: host token ids in, loss out.
pub struct B200Decoder {
    handle: *mut HlDecoder,
}
impl B200Decoder {
    pub fn new(device_ordinal: i32, config: HlDecoderConfig) -> CudaResult<Self> {
        let mut handle: *mut HlDecoder = std::ptr::null_mut();
        check(unsafe { hl_decoder_create(ctx_for(device_ordinal)?, &config, &mut handle) })?;
        Ok(Self { handle })
    }
    pub fn set_parameter(&mut self, state_dict_index: usize, values: &[f32]) -> CudaResult<()> {
        check(unsafe { hl_decoder_set_param(self.handle, dim(state_dict_index, "index")?, values.as_ptr(), values.len() as i64) })
    }
    pub fn set_optimizer(&mut self, config: HlAdamwConfig) -> CudaResult<()> {
        check(unsafe { hl_decoder_set_optimizer(self.handle, &config) })
    }
    pub fn train_step(&mut self, tokens: &[i64], targets: &[i64]) -> CudaResult<f32> {
        let mut loss = 0f32;
        check(unsafe { hl_decoder_train_step(self.handle, tokens.as_ptr(), targets.as_ptr(), &mut loss) })?;
        Ok(loss)
    }
}
impl Drop for B200Decoder {
    fn drop(&mut self) {
        unsafe { hl_decoder_destroy(self.handle) };
    }
}
'''


def generate() -> str:
    consts, defines, enums, opaque, structs, funcs = parse(HEADER.read_text())
    known = set(opaque) | {n for n, _ in structs}
    out = []
    out.append("// Generated by include/make_rust_shim.py from include/heirloom_b200.h; do not edit by hand.")
    out.append("// Rust side of the C ABI of libheirloom_b200.so, for heirloom-kernels (the only crate of the reference that")
    out.append("// contains unsafe code).  Not compiled in this repository: the image it is built in has no Rust toolchain.")
    out.append("#![allow(non_camel_case_types, dead_code)]")
    out.append("use std::os::raw::{c_char, c_void};")
    out.append("use super::cuda::{AdamWParams, CausalAttentionDims, CudaError, CudaResult};")
    out.append("")
    for name, value in defines + [(n, str(v)) for n, v in enums]:
        out.append(f"pub const {name}: i32 = {value};")
    out.append("")
    for name in opaque:
        out.append(f"pub enum {rust_name(name)} {{}}")
    out.append("")
    for name, fields in structs:
        out.append("#[repr(C)]")
        out.append("#[derive(Clone, Copy)]")
        out.append(f"pub struct {rust_name(name)} {{")
        for fname, ctype, arr in fields:
            rt = map_type(ctype, known)
            if arr is not None:
                n = consts.get(arr, arr)
                rt = f"[{rt}; {n}]"
            out.append(f"    pub {fname}: {rt},")
        out.append("}")
        out.append("")
    out.append('#[link(name = "heirloom_b200")]')
    out.append('extern "C" {')
    for name, ret, params in funcs:
        args = ", ".join(f"{'type_' if p == 'type' else p}: {map_type(t, known)}" for p, t in params)
        r = "" if ret == "void" else f" -> {map_type(ret, known)}"
        out.append(f"    pub fn {name}({args}){r};")
    out.append("}")
    out.append(SAFE_WRAPPERS)
    return "\n".join(out) + "\n"


def entry_points() -> list:
    return [f[0] for f in parse(HEADER.read_text())[5]]


if __name__ == "__main__":
    OUT.write_text(generate())
    print(f"wrote {OUT} ({len(entry_points())} entry points)")
    sys.exit(0)

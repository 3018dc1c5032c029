"""Checkpoints in the reference's on-disk layout, written from and loaded into the device model.

Layout (src/checkpoint.rs:124-254, src/nn.rs:2968-3050, src/npy.rs:9-120):

    <dir>/model/state.tsv                 one `name<TAB>file` line per parameter, state-dict order
    <dir>/model/NNNN_<sanitised name>.npy  NumPy v1.0 files, little-endian f32, C order
    <dir>/metadata.json                   model_family, config, dataset state, step
    <dir>/optimizer.json                  AdamW hyper-parameters, step, per-parameter m and v as f64 lists
    <dir>/tokenizer.json                  copied through when the caller supplies one (tokenizers are out of scope here)

`optimizer.json` keeps the reference schema (moments as JSON arrays of f64), which is practical for
small models only: at 163 M parameters it is several GB of text.  `moments_sidecar=True` writes
`optimizer_m.npy` / `optimizer_v.npy` (flat f32, state-dict order) beside a schema-complete
`optimizer.json` whose `m`/`v` lists are empty; only this module reads the sidecar.
"""
from __future__ import annotations

import json
import shutil
import struct
from pathlib import Path
from typing import Dict, Optional, Tuple

import numpy as np

from ._lib import HeirloomError
from .cuda import Context
from .nn import DecoderConfig, DecoderLm, MemoryConfig

_MAGIC = b"\x93NUMPY"


def sanitize_state_name(name: str) -> str:
    """ASCII letters, digits, `_` and `-` stay; everything else becomes `_` (src/nn.rs:3040-3050)."""
    return "".join(ch if (ch.isascii() and ch.isalnum()) or ch in "_-" else "_" for ch in name)


def _shape_tuple(shape) -> str:
    if len(shape) == 0:
        return "()"
    if len(shape) == 1:
        return f"({shape[0]},)"
    return "(" + ", ".join(str(int(s)) for s in shape) + ")"


def write_npy(path: Path, array: np.ndarray) -> None:
    """NumPy v1.0 file with the reference's header text and 16-byte padding (src/npy.rs:9-70)."""
    array = np.asarray(array, order="C")  # keeps rank-0 arrays rank 0
    descr = {np.dtype(np.float32): "<f4", np.dtype(np.float64): "<f8", np.dtype(np.int64): "<i8"}.get(array.dtype)
    if descr is None:
        raise HeirloomError(f"write_npy does not support dtype {array.dtype}")
    header = f"{{'descr': '{descr}', 'fortran_order': False, 'shape': {_shape_tuple(array.shape)}, }}"
    preamble = len(_MAGIC) + 2 + 2
    header += " " * ((16 - ((preamble + len(header) + 1) % 16)) % 16) + "\n"
    if len(header) > 0xFFFF:
        raise HeirloomError(f"npy v1 header too large: {len(header)} bytes")
    with open(path, "wb") as f:
        f.write(_MAGIC + bytes([1, 0]) + struct.pack("<H", len(header)) + header.encode("latin1"))
        f.write(array.astype(array.dtype.newbyteorder("<"), copy=False).tobytes())


def read_npy(path: Path) -> np.ndarray:
    """Reads what `write_npy` (or the reference) wrote; validates magic, version and layout."""
    raw = Path(path).read_bytes()
    if raw[:6] != _MAGIC:
        raise HeirloomError(f"{path} is not an npy file")
    if raw[6] != 1:
        raise HeirloomError(f"{path}: unsupported npy version {raw[6]}.{raw[7]}")
    (hlen,) = struct.unpack("<H", raw[8:10])
    header = raw[10:10 + hlen].decode("latin1")
    if "'fortran_order': False" not in header:
        raise HeirloomError(f"{path}: only C-order arrays are supported")
    descr = header.split("'descr': '")[1].split("'")[0]
    shape_text = header.split("'shape': (")[1].split(")")[0]
    shape = tuple(int(p) for p in shape_text.replace(" ", "").split(",") if p)
    dtype = {"<f4": np.float32, "<f8": np.float64, "<i8": np.int64}.get(descr)
    if dtype is None:
        raise HeirloomError(f"{path}: unsupported dtype {descr}")
    count = int(np.prod(shape)) if shape else 1
    data = np.frombuffer(raw, dtype=dtype, count=count, offset=10 + hlen)
    return data.reshape(shape).copy()


def save_state_dict(model: DecoderLm, directory: Path) -> None:
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    lines = []
    for index, name in enumerate(model.parameter_names()):
        filename = f"{index:04d}_{sanitize_state_name(name)}.npy"
        write_npy(directory / filename, model.parameter(name))
        lines.append(f"{name}\t{filename}\n")
    (directory / "state.tsv").write_text("".join(lines))


def load_state_dict(model: DecoderLm, directory: Path) -> None:
    """Validates names and shapes both ways like the reference loader (src/nn.rs:2997-3038)."""
    directory = Path(directory)
    files: Dict[str, str] = {}
    for number, line in enumerate((directory / "state.tsv").read_text().splitlines(), 1):
        if not line.strip():
            continue
        if "\t" not in line:
            raise HeirloomError(f"invalid state manifest line {number}: expected name<TAB>filename")
        name, filename = line.split("\t", 1)
        files[name] = filename
    state = {}
    for name in model.parameter_names():
        if name not in files:
            raise HeirloomError(f"missing state_dict parameter {name!r}")
        state[name] = read_npy(directory / files[name])
    for name in files:
        if name not in state:
            raise HeirloomError(f"state_dict contains unexpected parameter {name!r}")
    model.load_state_dict(state)


def _metadata(model: DecoderLm, step: int, dataset_rng_state: int, dataset_batches_seen: int,
              dataset_manifest_path: Optional[str]) -> dict:
    cfg, mem = model.cfg, model.memory
    memory_config = {
        "vocab_size": cfg.vocab, "block_size": cfg.context, "n_layers": cfg.n_layers, "d_model": cfg.d_model,
        "n_heads": cfg.n_heads, "ff_hidden": cfg.d_ff,
        "memory_layer_indices": list(mem.memory_layers) if mem else [],
        "memory_slots": mem.slots if mem else 1, "memory_key_dim": mem.key_dim if mem else cfg.d_model,
        "memory_value_dim": mem.value_dim if mem else cfg.d_model, "memory_top_k": mem.top_k if mem else 1,
        "memory_heads": mem.memory_heads if mem else 1, "memory_lookup": "product_key" if mem else "exact",
        "shared_memory": True, "memory_plus": True, "memory_update_policy": "full", "smft_mode": "disabled",
    }
    return {"model_family": "memory_transformer", "memory_config": memory_config, "dataset_rng_state": int(dataset_rng_state),
            "dataset_batches_seen": int(dataset_batches_seen), "dataset_manifest_path": dataset_manifest_path,
            "step": int(step)}


def save_checkpoint(directory, model: DecoderLm, optimizer: dict, dataset_rng_state: int = 0, dataset_batches_seen: int = 0,
                    dataset_manifest_path: Optional[str] = None, tokenizer_json: Optional[Path] = None,
                    moments_sidecar: bool = False) -> None:
    """`save_memory_lm_checkpoint_with_dataset_state` (src/checkpoint.rs:152-201) for the device model.
    `optimizer` holds the hyper-parameters given to `set_optimizer` (lr, beta1, beta2, eps, weight_decay,
    clip_norm); step and moments are read from the device."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    save_state_dict(model, directory / "model")
    if tokenizer_json is not None:
        shutil.copyfile(tokenizer_json, directory / "tokenizer.json")
    step = model.optimizer_steps
    (directory / "metadata.json").write_text(json.dumps(
        _metadata(model, step, dataset_rng_state, dataset_batches_seen, dataset_manifest_path), indent=2))
    state = {"step": step, "lr": float(optimizer.get("lr", 1e-3)), "beta1": float(optimizer.get("beta1", 0.9)),
             "beta2": float(optimizer.get("beta2", 0.999)), "eps": float(optimizer.get("eps", 1e-8)),
             "weight_decay": float(optimizer.get("weight_decay", 0.01)), "clip_norm": optimizer.get("clip_norm"),
             "m": [], "v": []}
    names = model.parameter_names()
    if moments_sidecar:
        ms, vs = zip(*(model.moments(n) for n in names))
        write_npy(directory / "optimizer_m.npy", np.concatenate([a.reshape(-1) for a in ms]))
        write_npy(directory / "optimizer_v.npy", np.concatenate([a.reshape(-1) for a in vs]))
    else:
        for n in names:  # f32 moments widened to f64, as AdamW::try_state does (src/nn.rs:2035-2057)
            m, v = model.moments(n)
            state["m"].append(m.reshape(-1).astype(np.float64).tolist())
            state["v"].append(v.reshape(-1).astype(np.float64).tolist())
    (directory / "optimizer.json").write_text(json.dumps(state))


def load_checkpoint(directory, ctx: Context, batch: int, precision: Optional[int] = None) -> Tuple[DecoderLm, dict]:
    """`load_memory_lm_checkpoint_on_device` (src/checkpoint.rs:228-254): validates the family, rebuilds the
    model from the recorded configuration, loads parameters, optimizer hyper-parameters, step and moments.
    Returns the model and the metadata."""
    directory = Path(directory)
    meta = json.loads((directory / "metadata.json").read_text())
    family = meta.get("model_family", "tiny_transformer")
    if family != "memory_transformer":
        raise HeirloomError(f"checkpoint model_family is {family!r}, but loader expected 'memory_transformer'")
    mc = meta["memory_config"]
    kwargs = dict(vocab=mc["vocab_size"], d_model=mc["d_model"], n_layers=mc["n_layers"], n_heads=mc["n_heads"],
                  d_ff=mc["ff_hidden"], context=mc["block_size"], batch=batch)
    if precision is not None:
        kwargs["precision"] = precision
    memory = None
    if mc["memory_layer_indices"]:
        memory = MemoryConfig(tuple(mc["memory_layer_indices"]), mc["memory_slots"], mc["memory_key_dim"],
                              mc["memory_value_dim"], mc["memory_top_k"], mc["memory_heads"])
    model = DecoderLm(ctx, DecoderConfig(**kwargs), memory)
    load_state_dict(model, directory / "model")
    opt = json.loads((directory / "optimizer.json").read_text())
    model.set_optimizer(lr=opt["lr"], beta1=opt["beta1"], beta2=opt["beta2"], eps=opt["eps"],
                        weight_decay=opt["weight_decay"], clip_norm=opt.get("clip_norm"))
    names = model.parameter_names()
    shapes = model.parameter_shapes()
    if opt["m"] or opt["v"]:
        if len(opt["m"]) != len(names) or len(opt["v"]) != len(names):
            raise HeirloomError("AdamW state parameter count mismatch")
        for i, n in enumerate(names):
            size = int(np.prod(shapes[n]))
            if len(opt["m"][i]) != size or len(opt["v"][i]) != size:
                raise HeirloomError(f"AdamW state shape mismatch for parameter {i}")
            model.set_moments(n, np.asarray(opt["m"][i], np.float32).reshape(shapes[n]),
                              np.asarray(opt["v"][i], np.float32).reshape(shapes[n]))
    elif (directory / "optimizer_m.npy").exists():
        flat_m, flat_v = read_npy(directory / "optimizer_m.npy"), read_npy(directory / "optimizer_v.npy")
        total = sum(int(np.prod(shapes[n])) for n in names)
        if flat_m.size != total or flat_v.size != total:
            raise HeirloomError("AdamW moment sidecar does not match the model's parameter count")
        at = 0
        for n in names:
            size = int(np.prod(shapes[n]))
            model.set_moments(n, flat_m[at:at + size].reshape(shapes[n]), flat_v[at:at + size].reshape(shapes[n]))
            at += size
    elif opt["step"] != 0:
        raise HeirloomError("checkpoint has optimizer steps but no moments")
    model.set_optimizer_steps(int(opt["step"]))
    return model, meta

"""Training-batch path either side of the step: binary token shards in the reference's format, the
deterministic data-parallel batch schedule, and a device prefetcher.

* Token shards (src/data.rs:156-250, :1805-1900, :1925-1990): `<name>.tokens.bin` holds token ids as
  little-endian u16 (all ids <= 65535) or u32; `<name>.tokens.json` holds format
  "heirloom.token_shard", version 1, payload path, dtype, token count, the FNV-1a-64 hash of the ids
  widened to little-endian u64, payload byte count and the FNV-1a-64 hash of the payload bytes.
* `deterministic_sharded_batch` (src/data.rs:362-423): sample `s` of rank `r` at step `t` starts at
  `mix_u64(seed ^ (t*world*B + r*B + s)) % (len - block - 1)`, so every rank draws different windows
  and a run can be replayed from (seed, step) alone.
* `DevicePrefetcher`: stages batch k+1 into pinned memory and copies it to the GPU on its own
  stream while step k runs.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np

from ._lib import HeirloomError

TOKEN_SHARD_FORMAT = "heirloom.token_shard"
TOKEN_SHARD_VERSION = 1
_MASK = (1 << 64) - 1


def mix_u64(value: int) -> int:
    """SplitMix64 finaliser of `value + golden ratio` (src/data.rs:764-769)."""
    value = (value + 0x9E3779B97F4A7C15) & _MASK
    value = ((value ^ (value >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    value = ((value ^ (value >> 27)) * 0x94D049BB133111EB) & _MASK
    return value ^ (value >> 31)


def stable_hash_bytes(data: bytes) -> str:
    """FNV-1a, 64 bit, as 16 hex digits (src/tokenizer.rs:968-975)."""
    import ctypes

    from ._lib import load
    lib = load()
    lib.hl_fnv1a64.restype = ctypes.c_ulonglong
    lib.hl_fnv1a64.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_ulonglong]
    return f"{lib.hl_fnv1a64(bytes(data), len(data), 0xCBF29CE484222325):016x}"


def stable_hash_tokens(tokens: Sequence[int]) -> str:
    """Hash of the ids widened to little-endian u64 (src/data.rs:1979-1985)."""
    return stable_hash_bytes(np.asarray(tokens, dtype="<u8").tobytes())


@dataclass
class TokenShardMetadata:
    format: str
    version: int
    payload_path: str
    dtype: str  # "u16" or "u32"
    token_count: int
    token_hash: str
    payload_bytes: int
    payload_hash: str

    def validate(self) -> None:
        if self.format != TOKEN_SHARD_FORMAT:
            raise HeirloomError(f"unsupported token shard format {self.format}, expected {TOKEN_SHARD_FORMAT}")
        if self.version != TOKEN_SHARD_VERSION:
            raise HeirloomError(f"unsupported token shard version {self.version}, expected {TOKEN_SHARD_VERSION}")
        if self.dtype not in ("u16", "u32"):
            raise HeirloomError(f"unsupported token shard dtype {self.dtype}")
        expected = self.token_count * (2 if self.dtype == "u16" else 4)
        if self.payload_bytes != expected:
            raise HeirloomError(f"token shard payload byte mismatch: metadata={self.payload_bytes} expected={expected}")


def write_token_shard(payload_path, metadata_path, tokens: Sequence[int]) -> TokenShardMetadata:
    payload_path, metadata_path = Path(payload_path), Path(metadata_path)
    payload_path.parent.mkdir(parents=True, exist_ok=True)
    metadata_path.parent.mkdir(parents=True, exist_ok=True)
    ids = np.asarray(tokens, dtype=np.int64)
    if ids.size and ids.min() < 0:
        raise HeirloomError("token ids must be non-negative")
    top = int(ids.max()) if ids.size else 0
    if top > 0xFFFFFFFF:
        raise HeirloomError(f"token id {top} exceeds u32 token shard limit")
    dtype = "u16" if top <= 0xFFFF else "u32"
    payload = ids.astype("<u2" if dtype == "u16" else "<u4").tobytes()
    payload_path.write_bytes(payload)
    try:
        relative = str(payload_path.resolve().relative_to(metadata_path.parent.resolve()))
    except ValueError:
        relative = str(payload_path.resolve())
    meta = TokenShardMetadata(TOKEN_SHARD_FORMAT, TOKEN_SHARD_VERSION, relative, dtype, int(ids.size), stable_hash_tokens(ids),
                              len(payload), stable_hash_bytes(payload))
    metadata_path.write_text(json.dumps(meta.__dict__, indent=2))
    return meta


def load_token_shard_metadata(metadata_path) -> TokenShardMetadata:
    meta = TokenShardMetadata(**json.loads(Path(metadata_path).read_text()))
    meta.validate()
    return meta


def read_token_shard(metadata_path, verify_hashes: bool = True) -> np.ndarray:
    """Token ids of one shard as int64; byte count, payload hash and token hash are checked."""
    metadata_path = Path(metadata_path)
    meta = load_token_shard_metadata(metadata_path)
    payload_path = Path(meta.payload_path)
    if not payload_path.is_absolute():
        payload_path = metadata_path.parent / payload_path
    payload = payload_path.read_bytes()
    if len(payload) != meta.payload_bytes:
        raise HeirloomError(f"token shard payload byte mismatch: metadata={meta.payload_bytes} actual={len(payload)}")
    if verify_hashes and stable_hash_bytes(payload) != meta.payload_hash:
        raise HeirloomError(f"token shard payload hash mismatch for {payload_path}")
    ids = np.frombuffer(payload, dtype="<u2" if meta.dtype == "u16" else "<u4").astype(np.int64)
    if ids.size != meta.token_count or (verify_hashes and stable_hash_tokens(ids) != meta.token_hash):
        raise HeirloomError(f"token shard token count/hash mismatch for {payload_path}")
    return ids


def write_token_shard_set(shards_dir, split: str, tokens: Sequence[int], shard_tokens: Optional[int] = None) -> List[dict]:
    """`<split>-NNNNNN.tokens.bin/.json` files of at most `shard_tokens` ids each (src/data.rs:1746-1772);
    returns the manifest entries (split, metadata_path, tokens, token_hash)."""
    ids = np.asarray(tokens, dtype=np.int64)
    if ids.size == 0:
        raise HeirloomError(f"{split} split has no tokens to shard")
    chunk = max(1, shard_tokens or ids.size)
    shards_dir = Path(shards_dir)
    entries = []
    for index, start in enumerate(range(0, ids.size, chunk)):
        meta_path = shards_dir / f"{split}-{index:06d}.tokens.json"
        meta = write_token_shard(shards_dir / f"{split}-{index:06d}.tokens.bin", meta_path, ids[start:start + chunk])
        entries.append({"split": split, "metadata_path": str(meta_path), "tokens": meta.token_count, "token_hash": meta.token_hash})
    return entries


def read_token_shard_set(entries: Sequence[dict]) -> np.ndarray:
    """Concatenation of the shards of one split, each checked against its manifest entry."""
    parts = []
    for e in entries:
        ids = read_token_shard(e["metadata_path"])
        if ids.size != e["tokens"] or stable_hash_tokens(ids) != e["token_hash"]:
            raise HeirloomError(f"{e['split']} token file mismatch: expected len/hash={e['tokens']}/{e['token_hash']}, got "
                                f"{ids.size}/{stable_hash_tokens(ids)}")
        parts.append(ids)
    return np.concatenate(parts)


def deterministic_sharded_batch(tokens: np.ndarray, block_size: int, batch_size: int, seed: int, global_step: int, rank: int,
                                world_size: int) -> Tuple[np.ndarray, np.ndarray]:
    """Inputs and next-token targets `[batch_size, block_size]` (int64) of one rank at one step."""
    if block_size == 0:
        raise HeirloomError("block_size must be greater than zero")
    if batch_size == 0:
        raise HeirloomError("batch_size must be greater than zero")
    if world_size == 0:
        raise HeirloomError("world_size must be greater than zero")
    if rank >= world_size:
        raise HeirloomError(f"rank must be less than world_size, got rank={rank} world_size={world_size}")
    if len(tokens) <= block_size:
        raise HeirloomError(f"dataset needs more than block_size tokens, got {len(tokens)} tokens and block_size {block_size}")
    span = len(tokens) - block_size - 1
    starts = np.empty(batch_size, np.int64)
    for sample in range(batch_size):
        logical = (global_step * world_size * batch_size + rank * batch_size + sample) & _MASK
        starts[sample] = 0 if span == 0 else mix_u64((seed ^ logical) & _MASK) % span
    window = starts[:, None] + np.arange(block_size + 1)[None, :]
    rows = np.asarray(tokens, np.int64)[window]
    return np.ascontiguousarray(rows[:, :-1]), np.ascontiguousarray(rows[:, 1:])


class DevicePrefetcher:
    """Serves device batches one step ahead: while the caller trains on batch k, batch k+1 is built by
    `make_batch(k+1)`, staged in pinned memory and copied on a separate stream.  `next()` makes the
    given consumer stream wait for the copy and returns `(tokens, targets)` CUDA tensors."""

    def __init__(self, make_batch: Callable[[int], Tuple[np.ndarray, np.ndarray]], first_step: int = 0):
        import torch
        self._torch = torch
        self._make = make_batch
        self._stream = torch.cuda.Stream()
        self._step = first_step
        self._slots = [None, None]
        self._pending = None
        self._stage(self._step)

    def _stage(self, step: int) -> None:
        torch = self._torch
        x, y = self._make(step)
        slot = step & 1
        if self._slots[slot] is None or self._slots[slot][0].shape != x.shape:
            self._slots[slot] = (torch.empty(x.shape, dtype=torch.int64).pin_memory(), torch.empty(y.shape, dtype=torch.int64).pin_memory(),
                                 torch.empty(x.shape, dtype=torch.int64, device="cuda"), torch.empty(y.shape, dtype=torch.int64, device="cuda"))
        hx, hy, dx, dy = self._slots[slot]
        hx.copy_(torch.from_numpy(x))
        hy.copy_(torch.from_numpy(y))
        with torch.cuda.stream(self._stream):
            dx.copy_(hx, non_blocking=True)
            dy.copy_(hy, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self._stream)
        self._pending = (dx, dy, done)

    def next(self, consumer_stream=None):
        torch = self._torch
        dx, dy, done = self._pending
        (consumer_stream or torch.cuda.current_stream()).wait_event(done)
        self._step += 1
        self._stage(self._step)  # the other slot: the tensors just handed out stay untouched for one step
        return dx, dy

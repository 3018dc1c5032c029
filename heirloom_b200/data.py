"""Training-batch path either side of the step: binary token shards in the reference's format, the
deterministic data-parallel batch schedule, and a device prefetcher.

* Token shards (src/data.rs:156-250, :1805-1900, :1925-1990): `<name>.tokens.bin` holds token ids as
  little-endian u16 (all ids <= 65535) or u32; `<name>.tokens.json` holds format
  "heirloom.token_shard", version 1, payload path, dtype, token count, the FNV-1a-64 hash of the ids
  widened to little-endian u64, payload byte count and the FNV-1a-64 hash of the payload bytes.
* `deterministic_sharded_batch` (src/data.rs:362-423): sample `s` of rank `r` at step `t` starts at
  `mix_u64(seed ^ (t*world*B + r*B + s)) % (len - block - 1)`, so every rank draws different windows
  and a run can be replayed from (seed, step) alone.
* `PreparedTokenData` / `StreamingTokenDataset` (src/data.rs:36-100, :425-760, :771-1000): the version-2 manifest of a
  binary-sharded dataset and batches read from its shard files by ranged reads, with the reference's three schedules
  (random windows from the SplitMix64 stream, the deterministic data-parallel schedule, consecutive windows).
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


# ---- prepared-dataset manifest and the streaming loader (src/data.rs:36-100, :425-760, :771-1000) -----------------
DATASET_MANIFEST_FORMAT = "heirloom.token_dataset"
DATASET_STORAGE_JSON, DATASET_STORAGE_BINARY_SHARDS = "json", "binary_shards"


@dataclass
class TokenDatasetState:
    """Where a token stream stands: the sampler's SplitMix64 state and the batches served (`TokenDatasetState`,
    src/data.rs:25-36); `from_seed` starts a run, a saved state resumes one exactly."""
    rng_state: int
    batches_seen: int = 0

    @staticmethod
    def from_seed(seed: int) -> "TokenDatasetState":
        return TokenDatasetState(seed & _MASK, 0)


@dataclass
class StreamingTokenLoaderStats:
    batches: int = 0
    samples: int = 0
    tokens: int = 0
    read_calls: int = 0
    bytes_read: int = 0


class PreparedTokenData:
    """A prepared dataset on disk: `manifest.json` plus what it points to (`PreparedTokenData`, src/data.rs:235-240,
    :866-1000).  Version 2 with storage "binary_shards" lists `train_shards` / `valid_shards`; paths in the manifest
    are relative to its directory."""

    def __init__(self, manifest_path, manifest: dict):
        self.manifest_path = Path(manifest_path)
        self.root = self.manifest_path.parent
        self.manifest = manifest

    @staticmethod
    def load(path) -> "PreparedTokenData":
        path = Path(path)
        try:
            manifest = json.loads(path.read_text())
        except OSError as err:
            raise HeirloomError(f"failed to read {path}: {err}")
        except ValueError as err:
            raise HeirloomError(f"failed to parse {path}: {err}")
        manifest.setdefault("storage", DATASET_STORAGE_JSON)
        for key in ("train_shards", "valid_shards", "sources"):
            manifest.setdefault(key, [])
        data = PreparedTokenData(path, manifest)
        data.validate()
        return data

    def validate(self) -> None:
        m = self.manifest
        if m.get("format") != DATASET_MANIFEST_FORMAT:
            raise HeirloomError(f"unsupported dataset manifest format {m.get('format')}, expected {DATASET_MANIFEST_FORMAT}")
        if m.get("version") not in (1, 2):
            raise HeirloomError(f"unsupported dataset manifest version {m.get('version')}, expected 1 or 2")
        fraction = m.get("split", {}).get("valid_fraction", 0.1)
        if not (0.0 <= fraction < 1.0):
            raise HeirloomError(f"valid_fraction must be in [0, 1), got {fraction}")
        if m.get("train_tokens", 0) == 0 or m.get("valid_tokens", 0) == 0:
            raise HeirloomError("prepared dataset must have non-empty train and valid splits, got "
                                f"train={m.get('train_tokens', 0)} valid={m.get('valid_tokens', 0)}")
        if m["version"] == 1:
            if m["storage"] != DATASET_STORAGE_JSON:
                raise HeirloomError(f'dataset manifest v1 storage must be "{DATASET_STORAGE_JSON}", got "{m["storage"]}"')
            return
        if m["storage"] != DATASET_STORAGE_BINARY_SHARDS:
            raise HeirloomError(f'dataset manifest v2 storage must be "{DATASET_STORAGE_BINARY_SHARDS}", got "{m["storage"]}"')
        if not m["sources"]:
            raise HeirloomError("dataset manifest v2 requires at least one source")
        if not m["train_shards"] or not m["valid_shards"]:
            raise HeirloomError("dataset manifest v2 requires non-empty train_shards and valid_shards")
        train = sum(s["tokens"] for s in m["train_shards"])
        valid = sum(s["tokens"] for s in m["valid_shards"])
        if train != m["train_tokens"] or valid != m["valid_tokens"]:
            raise HeirloomError("dataset manifest v2 shard token counts do not match split totals: "
                                f"train_shards={train} train_total={m['train_tokens']} valid_shards={valid} "
                                f"valid_total={m['valid_tokens']}")

    def is_binary_sharded(self) -> bool:
        return self.manifest["version"] == 2 and self.manifest["storage"] == DATASET_STORAGE_BINARY_SHARDS

    def resolve(self, path: str) -> Path:
        p = Path(path)
        return p if p.is_absolute() else self.root / p

    def shards(self, split: str) -> List[dict]:
        if split not in ("train", "valid"):
            raise HeirloomError(f"unknown split {split!r}, expected 'train' or 'valid'")
        return self.manifest[f"{split}_shards"]

    def materialize(self, split: str) -> np.ndarray:
        """Every token of a split in memory, each shard checked against its manifest entry (`materialize_shards`)."""
        if not self.is_binary_sharded():
            raise HeirloomError("only binary-sharded datasets are read here")
        entries = [{**e, "metadata_path": str(self.resolve(e["metadata_path"]))} for e in self.shards(split)]
        return read_token_shard_set(entries)

    def streaming_dataset(self, split: str, block_size: int, state: TokenDatasetState) -> "StreamingTokenDataset":
        return StreamingTokenDataset.open(self, split, block_size, state)


def write_prepared_manifest(out_dir, train_tokens: Sequence[int], valid_tokens: Sequence[int], shard_tokens: int,
                            source_id: str = "synthetic", tokenizer_path: str = "tokenizer.json",
                            valid_fraction: float = 0.1) -> Path:
    """A version-2 binary-sharded dataset directory (`prepare_lm_data_binary_shards`, src/data.rs:1609-1772, without
    the tokenizer run: the ids are given): `shards/<split>-NNNNNN.tokens.bin/.json` and `manifest.json` with relative
    paths.  Returns the manifest path."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    train = np.asarray(train_tokens, np.int64)
    valid = np.asarray(valid_tokens, np.int64)
    entries = {}
    for split, ids in (("train", train), ("valid", valid)):
        rows = write_token_shard_set(out_dir / "shards", split, ids, shard_tokens)
        entries[split] = [{**r, "metadata_path": str(Path(r["metadata_path"]).relative_to(out_dir))} for r in rows]
    manifest = {
        "format": DATASET_MANIFEST_FORMAT, "version": 2, "storage": DATASET_STORAGE_BINARY_SHARDS,
        "source_path": source_id, "source_bytes": 0, "source_hash": "", "tokenizer_path": tokenizer_path,
        "tokenizer_hash": "", "train_tokens_path": "", "valid_tokens_path": "", "train_tokens": int(train.size),
        "valid_tokens": int(valid.size), "train_hash": stable_hash_tokens(train), "valid_hash": stable_hash_tokens(valid),
        "split": {"kind": "contiguous_tail_valid", "valid_fraction": valid_fraction},
        "sources": [{"source_id": source_id, "path": source_id, "bytes": 0, "hash": "", "tokens": int(train.size + valid.size)}],
        "train_shards": entries["train"], "valid_shards": entries["valid"],
    }
    path = out_dir / "manifest.json"
    path.write_text(json.dumps(manifest, indent=2))
    return path


class _OpenTokenShard:
    """One shard kept open for ranged reads (`OpenTokenShard`, src/data.rs:711-762): the payload's size and hash are
    checked once at open, then every read seeks to `start * width` and takes `len * width` bytes."""

    def __init__(self, metadata_path: Path, start_token: int):
        self.metadata = load_token_shard_metadata(metadata_path)
        payload = Path(self.metadata.payload_path)
        if not payload.is_absolute():
            payload = Path(metadata_path).parent / payload
        try:
            actual = payload.stat().st_size
        except OSError as err:
            raise HeirloomError(f"failed to stat {payload}: {err}")
        if actual != self.metadata.payload_bytes:
            raise HeirloomError(f"token shard payload byte mismatch: metadata={self.metadata.payload_bytes} actual={actual}")
        digest = stable_hash_file(payload)
        if digest != self.metadata.payload_hash:
            raise HeirloomError(f"token shard payload hash mismatch: metadata={self.metadata.payload_hash} actual={digest}")
        self.start_token = start_token
        self.width = 2 if self.metadata.dtype == "u16" else 4
        self.file = open(payload, "rb")

    def read_range(self, start: int, count: int) -> np.ndarray:
        if start + count > self.metadata.token_count:
            raise HeirloomError(f"token shard read out of range: start={start} len={count} token_count={self.metadata.token_count}")
        self.file.seek(start * self.width)
        raw = self.file.read(count * self.width)
        if len(raw) != count * self.width:
            raise HeirloomError("failed to read token shard: short read")
        return np.frombuffer(raw, dtype="<u2" if self.width == 2 else "<u4").astype(np.int64)

    def close(self) -> None:
        self.file.close()


def stable_hash_file(path, chunk_bytes: int = 1 << 20) -> str:
    """FNV-1a-64 of a file, streamed in chunks (`stable_hash_file`, src/data.rs:1987-2005)."""
    import ctypes

    from ._lib import load
    lib = load()
    lib.hl_fnv1a64.restype = ctypes.c_ulonglong
    lib.hl_fnv1a64.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_ulonglong]
    state = 0xCBF29CE484222325
    with open(path, "rb") as f:
        while True:
            chunk = f.read(chunk_bytes)
            if not chunk:
                break
            state = lib.hl_fnv1a64(chunk, len(chunk), state)
    return f"{state:016x}"


class StreamingTokenDataset:
    """Batches straight from the shard files, one ranged read per window and shard it touches, nothing but the window
    in memory (`StreamingTokenDataset`, src/data.rs:450-716).  The three batch schedules of the reference: random
    windows from the SplitMix64 stream (`next_batch`), the replayable data-parallel schedule
    (`deterministic_sharded_batch`) and consecutive windows for evaluation (`sequential_batch_at`)."""

    def __init__(self, shards: List[_OpenTokenShard], total_tokens: int, block_size: int, state: TokenDatasetState):
        self._shards = shards
        self._starts = np.array([s.start_token for s in shards], np.int64)
        self.total_tokens = total_tokens
        self.block_size = block_size
        self._rng_state = state.rng_state & _MASK
        self._batches_seen = state.batches_seen
        self.stats = StreamingTokenLoaderStats()

    @staticmethod
    def open(prepared: PreparedTokenData, split: str, block_size: int, state: TokenDatasetState) -> "StreamingTokenDataset":
        m = prepared.manifest
        if not prepared.is_binary_sharded():
            raise HeirloomError(f'streaming token dataset requires manifest v2 with storage="{DATASET_STORAGE_BINARY_SHARDS}", '
                                f'got version={m["version"]} storage="{m["storage"]}"')
        if block_size == 0:
            raise HeirloomError("block_size must be greater than zero")
        shards, total = [], 0
        for entry in prepared.shards(split):
            path = prepared.resolve(entry["metadata_path"])
            shard = _OpenTokenShard(path, total)
            if shard.metadata.token_count != entry["tokens"] or shard.metadata.token_hash != entry["token_hash"]:
                raise HeirloomError(f"{split} shard metadata mismatch for {path}: manifest len/hash={entry['tokens']}/"
                                    f"{entry['token_hash']}, shard len/hash={shard.metadata.token_count}/{shard.metadata.token_hash}")
            total += shard.metadata.token_count
            shards.append(shard)
        if total <= block_size:
            raise HeirloomError(f"streaming dataset needs more than block_size tokens, got {total} tokens and block_size {block_size}")
        return StreamingTokenDataset(shards, total, block_size, state)

    def __len__(self) -> int:
        return self.total_tokens

    def state(self) -> TokenDatasetState:
        return TokenDatasetState(self._rng_state, self._batches_seen)

    def loader_stats(self) -> StreamingTokenLoaderStats:
        return self.stats

    def close(self) -> None:
        for s in self._shards:
            s.close()

    def _next_u64(self) -> int:
        self._rng_state = (self._rng_state + 0x9E3779B97F4A7C15) & _MASK
        z = self._rng_state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return z ^ (z >> 31)

    def _read_tokens(self, start: int, count: int) -> np.ndarray:
        if start + count > self.total_tokens:
            raise HeirloomError(f"streaming token read out of range: start={start} len={count} total={self.total_tokens}")
        parts, cursor, remaining = [], start, count
        while remaining > 0:
            index = int(np.searchsorted(self._starts, cursor, side="right")) - 1
            shard = self._shards[index]
            offset = cursor - shard.start_token
            take = min(remaining, shard.metadata.token_count - offset)
            parts.append(shard.read_range(offset, take))
            self.stats.read_calls += 1
            self.stats.bytes_read += take * shard.width
            cursor += take
            remaining -= take
        return parts[0] if len(parts) == 1 else np.concatenate(parts)

    def _windows(self, starts) -> Tuple[np.ndarray, np.ndarray]:
        rows = np.stack([self._read_tokens(int(s), self.block_size + 1) for s in starts])
        return np.ascontiguousarray(rows[:, :-1]), np.ascontiguousarray(rows[:, 1:])

    def _count(self, samples: int) -> None:
        self.stats.batches += 1
        self.stats.samples += samples
        self.stats.tokens += samples * self.block_size

    def next_batch(self, batch_size: int) -> Tuple[np.ndarray, np.ndarray]:
        if batch_size == 0:
            raise HeirloomError("batch_size must be greater than zero")
        span = self.total_tokens - self.block_size - 1
        starts = [0 if span == 0 else self._next_u64() % span for _ in range(batch_size)]
        out = self._windows(starts)
        self._batches_seen += 1
        self._count(batch_size)
        return out

    def deterministic_sharded_batch(self, batch_size: int, seed: int, global_step: int, rank: int,
                                    world_size: int) -> Tuple[np.ndarray, np.ndarray]:
        if batch_size == 0:
            raise HeirloomError("batch_size must be greater than zero")
        if world_size == 0:
            raise HeirloomError("world_size must be greater than zero")
        if rank >= world_size:
            raise HeirloomError(f"rank must be less than world_size, got rank={rank} world_size={world_size}")
        span = self.total_tokens - self.block_size - 1
        starts = []
        for sample in range(batch_size):
            logical = (global_step * world_size * batch_size + rank * batch_size + sample) & _MASK
            starts.append(0 if span == 0 else mix_u64((seed ^ logical) & _MASK) % span)
        out = self._windows(starts)
        self._count(batch_size)
        return out

    def sequential_batch_at(self, token_offset: int, batch_size: int):
        """Up to `batch_size` consecutive windows from `token_offset`; None when no whole window is left.  Returns
        (inputs, targets, windows served)."""
        if batch_size == 0:
            raise HeirloomError("batch_size must be greater than zero")
        starts, offset = [], token_offset
        while len(starts) < batch_size and offset + self.block_size < self.total_tokens:
            starts.append(offset)
            offset += self.block_size
        if not starts:
            return None
        x, y = self._windows(starts)
        self._count(len(starts))
        return x, y, len(starts)


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

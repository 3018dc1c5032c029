"""Token shards, the deterministic data-parallel batch schedule and the device prefetcher
(reference: src/data.rs:156-250, :362-423, :764-769, :1746-1990; src/tokenizer.rs:968-975)."""
import json

import numpy as np
import pytest

from heirloom_b200 import data as hd


def test_hashes_and_mixer_known_answers():
    assert hd.stable_hash_bytes(b"") == "cbf29ce484222325"  # FNV-1a offset basis
    assert hd.stable_hash_bytes(b"a") == "af63dc4c8601ec8c"  # published FNV-1a-64 test vector
    assert hd.stable_hash_bytes(b"foobar") == "85944171f73967e8"
    assert hd.stable_hash_tokens([1]) == hd.stable_hash_bytes(bytes([1, 0, 0, 0, 0, 0, 0, 0]))
    assert hd.mix_u64(0) == 0xE220A8397B1DCDAF  # first SplitMix64 output from state 0
    assert hd.mix_u64(0x9E3779B97F4A7C15) == 0x6E789E6AA1B965F4  # second output = mixer of the advanced state


def test_shards_round_trip_and_reject_tampering(tmp_path):
    rng = np.random.default_rng(0)
    small = rng.integers(0, 50304, 1000)
    wide = np.concatenate([small, [70000]])
    m16 = hd.write_token_shard(tmp_path / "a.tokens.bin", tmp_path / "a.tokens.json", small)
    m32 = hd.write_token_shard(tmp_path / "b.tokens.bin", tmp_path / "b.tokens.json", wide)
    assert (m16.dtype, m16.payload_bytes) == ("u16", 2000) and (m32.dtype, m32.payload_bytes) == ("u32", 4004)
    assert m16.payload_path == "a.tokens.bin" and m16.format == "heirloom.token_shard" and m16.version == 1
    assert (tmp_path / "a.tokens.bin").read_bytes()[:2] == int(small[0]).to_bytes(2, "little")
    assert np.array_equal(hd.read_token_shard(tmp_path / "a.tokens.json"), small)
    assert np.array_equal(hd.read_token_shard(tmp_path / "b.tokens.json"), wide)
    entries = hd.write_token_shard_set(tmp_path / "shards", "train", small, shard_tokens=300)
    assert [e["tokens"] for e in entries] == [300, 300, 300, 100]
    assert (tmp_path / "shards" / "train-000003.tokens.json").exists()
    assert np.array_equal(hd.read_token_shard_set(entries), small)
    # tampering: payload edited, metadata count edited, unknown format
    raw = bytearray((tmp_path / "a.tokens.bin").read_bytes())
    raw[10] ^= 1
    (tmp_path / "a.tokens.bin").write_bytes(bytes(raw))
    with pytest.raises(Exception, match="payload hash mismatch"):
        hd.read_token_shard(tmp_path / "a.tokens.json")
    meta = json.loads((tmp_path / "b.tokens.json").read_text())
    (tmp_path / "b.tokens.json").write_text(json.dumps({**meta, "token_count": 5}))
    with pytest.raises(Exception, match="payload byte mismatch"):
        hd.read_token_shard(tmp_path / "b.tokens.json")
    (tmp_path / "b.tokens.json").write_text(json.dumps({**meta, "format": "other"}))
    with pytest.raises(Exception, match="unsupported token shard format"):
        hd.read_token_shard(tmp_path / "b.tokens.json")
    with pytest.raises(Exception, match="has no tokens"):
        hd.write_token_shard_set(tmp_path / "e", "valid", [])


def test_batches_are_a_pure_function_of_seed_step_rank_and_disjoint_across_ranks():
    tokens = np.arange(10_000)
    x, y = hd.deterministic_sharded_batch(tokens, 16, 4, seed=9, global_step=3, rank=1, world_size=2)
    assert x.shape == (4, 16) and np.array_equal(y, x + 1)  # next-token targets
    span = len(tokens) - 16 - 1
    for sample in range(4):
        logical = 3 * 2 * 4 + 1 * 4 + sample
        assert x[sample, 0] == hd.mix_u64(9 ^ logical) % span
    again, _ = hd.deterministic_sharded_batch(tokens, 16, 4, 9, 3, 1, 2)
    assert np.array_equal(x, again)
    other, _ = hd.deterministic_sharded_batch(tokens, 16, 4, 9, 3, 0, 2)
    assert not np.array_equal(x, other)
    # the two ranks of a 2-rank run consume the same logical samples as one rank with a batch of 8
    whole, _ = hd.deterministic_sharded_batch(tokens, 16, 8, 9, 3, 0, 1)
    assert np.array_equal(np.concatenate([other, x]), whole)
    for kwargs, text in ((dict(block_size=0), "block_size must be greater than zero"), (dict(batch_size=0), "batch_size must be greater"),
                         (dict(world_size=0), "world_size must be greater"), (dict(rank=2), "rank must be less than world_size")):
        args = dict(tokens=tokens, block_size=16, batch_size=4, seed=9, global_step=0, rank=0, world_size=2)
        args.update(kwargs)
        with pytest.raises(Exception, match=text):
            hd.deterministic_sharded_batch(**args)
    with pytest.raises(Exception, match="more than block_size tokens"):
        hd.deterministic_sharded_batch(tokens[:16], 16, 1, 0, 0, 0, 1)
    one, _ = hd.deterministic_sharded_batch(tokens[:18], 16, 2, 5, 7, 0, 1)  # span 1: every window starts at 0
    assert one[:, 0].tolist() == [0, 0]


@pytest.mark.gpu
def test_prefetcher_hands_out_the_scheduled_batches_in_order():
    import torch
    tokens = np.random.default_rng(1).integers(0, 512, 5000)
    make = lambda step: hd.deterministic_sharded_batch(tokens, 32, 4, 11, step, 0, 1)
    pre = hd.DevicePrefetcher(make, first_step=5)
    for step in range(5, 11):
        x, y = pre.next()
        torch.cuda.synchronize()
        wx, wy = make(step)
        assert np.array_equal(x.cpu().numpy(), wx) and np.array_equal(y.cpu().numpy(), wy), step


def _dataset(tmp_path, n_train=5000, n_valid=700, shard_tokens=1111):
    rng = np.random.default_rng(5)
    train, valid = rng.integers(0, 50304, n_train), rng.integers(0, 50304, n_valid)
    manifest = hd.write_prepared_manifest(tmp_path / "prepared", train, valid, shard_tokens)
    return hd.PreparedTokenData.load(manifest), train, valid


def test_streaming_dataset_equals_the_in_memory_schedule(tmp_path):
    """Batches read by ranged reads from the shard files equal `deterministic_sharded_batch` over the concatenated
    split (the reference has the two side by side, src/data.rs:362-423 and :570-616); windows cross shard borders."""
    prepared, train, valid = _dataset(tmp_path)
    assert prepared.is_binary_sharded() and len(prepared.shards("train")) == 5
    assert np.array_equal(prepared.materialize("train"), train) and np.array_equal(prepared.materialize("valid"), valid)
    ds = prepared.streaming_dataset("train", 64, hd.TokenDatasetState.from_seed(9))
    assert len(ds) == 5000 and ds.block_size == 64
    for step in range(6):
        for rank in range(2):
            x, y = ds.deterministic_sharded_batch(4, seed=77, global_step=step, rank=rank, world_size=2)
            wx, wy = hd.deterministic_sharded_batch(train, 64, 4, 77, step, rank, 2)
            assert np.array_equal(x, wx) and np.array_equal(y, wy)
    stats = ds.loader_stats()
    assert (stats.batches, stats.samples, stats.tokens) == (12, 48, 48 * 64)
    # a window inside one shard is one read, one that crosses a border two: between 48 and 96 reads of 65 ids (u16)
    assert 48 <= stats.read_calls <= 96 and stats.bytes_read == 48 * 65 * 2
    ds.close()


def test_streaming_random_batches_follow_the_splitmix_stream_and_resume(tmp_path):
    prepared, train, _ = _dataset(tmp_path)
    ds = prepared.streaming_dataset("train", 32, hd.TokenDatasetState.from_seed(3))
    span = len(train) - 32 - 1
    state = 3
    for _ in range(3):
        x, y = ds.next_batch(5)
        for row in range(5):
            state = (state + 0x9E3779B97F4A7C15) & ((1 << 64) - 1)
            start = hd.mix_u64(state - 0x9E3779B97F4A7C15 & ((1 << 64) - 1)) % span  # next_u64 = mixer of the old state
            assert np.array_equal(x[row], train[start:start + 32]) and np.array_equal(y[row], train[start + 1:start + 33])
    saved = ds.state()
    assert saved.batches_seen == 3 and saved.rng_state == state
    x1, _ = ds.next_batch(2)
    resumed = prepared.streaming_dataset("train", 32, saved)
    x2, _ = resumed.next_batch(2)
    assert np.array_equal(x1, x2)   # exact resume from (rng state, batches seen)


def test_streaming_sequential_windows_cover_the_split_once(tmp_path):
    prepared, _, valid = _dataset(tmp_path)
    ds = prepared.streaming_dataset("valid", 100, hd.TokenDatasetState.from_seed(0))
    offset, seen = 0, []
    while True:
        got = ds.sequential_batch_at(offset, 4)
        if got is None:
            break
        x, y, n = got
        assert x.shape == (n, 100)
        for row in range(n):
            assert np.array_equal(x[row], valid[offset:offset + 100]) and np.array_equal(y[row], valid[offset + 1:offset + 101])
            offset += 100
        seen.append(n)
    assert seen == [4, 2]   # 700 tokens: six whole windows have a next token, the seventh does not


def test_streaming_dataset_rejects_what_the_reference_rejects(tmp_path):
    prepared, _, _ = _dataset(tmp_path)
    with pytest.raises(Exception, match="block_size must be greater than zero"):
        prepared.streaming_dataset("train", 0, hd.TokenDatasetState.from_seed(0))
    with pytest.raises(Exception, match="needs more than block_size tokens"):
        prepared.streaming_dataset("valid", 700, hd.TokenDatasetState.from_seed(0))
    ds = prepared.streaming_dataset("train", 16, hd.TokenDatasetState.from_seed(0))
    with pytest.raises(Exception, match="rank must be less than world_size"):
        ds.deterministic_sharded_batch(2, 1, 0, rank=2, world_size=2)
    # a manifest entry that no longer matches its shard
    manifest = json.loads(prepared.manifest_path.read_text())
    manifest["train_shards"][1]["token_hash"] = "0" * 16
    prepared.manifest_path.write_text(json.dumps(manifest))
    with pytest.raises(Exception, match="shard metadata mismatch"):
        hd.PreparedTokenData.load(prepared.manifest_path).streaming_dataset("train", 16, hd.TokenDatasetState.from_seed(0))
    # version 1 manifests are not streamable
    manifest["version"], manifest["storage"] = 1, "json"
    prepared.manifest_path.write_text(json.dumps(manifest))
    with pytest.raises(Exception, match="requires manifest v2"):
        hd.PreparedTokenData.load(prepared.manifest_path).streaming_dataset("train", 16, hd.TokenDatasetState.from_seed(0))
    # a payload edited after the manifest was written is caught when the shard is opened
    manifest["version"], manifest["storage"] = 2, "binary_shards"
    manifest["train_shards"][1]["token_hash"] = json.loads(
        (prepared.root / manifest["train_shards"][1]["metadata_path"]).read_text())["token_hash"]
    prepared.manifest_path.write_text(json.dumps(manifest))
    payload = prepared.root / "shards" / "train-000000.tokens.bin"
    raw = bytearray(payload.read_bytes())
    raw[0] ^= 1
    payload.write_bytes(bytes(raw))
    with pytest.raises(Exception, match="payload hash mismatch"):
        hd.PreparedTokenData.load(prepared.manifest_path).streaming_dataset("train", 16, hd.TokenDatasetState.from_seed(0))

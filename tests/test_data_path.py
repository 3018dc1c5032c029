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

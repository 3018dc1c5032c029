"""Checkpoint layout of the reference (state.tsv + npy + metadata.json + optimizer.json) and exact resume."""
import json

import numpy as np
import pytest

from heirloom_b200 import checkpoint as ck
from oracle import heirloom_oracle as ho


def test_npy_files_have_the_reference_header_and_numpy_reads_them(tmp_path):
    a = np.arange(6, dtype=np.float32).reshape(2, 3) * 0.5
    ck.write_npy(tmp_path / "a.npy", a)
    raw = (tmp_path / "a.npy").read_bytes()
    assert raw[:8] == b"\x93NUMPY\x01\x00"
    hlen = int.from_bytes(raw[8:10], "little")
    header = raw[10:10 + hlen].decode()
    assert header.startswith("{'descr': '<f4', 'fortran_order': False, 'shape': (2, 3), }") and header.endswith("\n")
    assert (10 + hlen) % 16 == 0
    assert np.array_equal(np.load(tmp_path / "a.npy"), a)
    assert np.array_equal(ck.read_npy(tmp_path / "a.npy"), a)
    for arr in (np.float32(3.5).reshape(()), np.arange(5, dtype=np.int64), np.ones((1, 1, 4), np.float64)):
        ck.write_npy(tmp_path / "b.npy", arr)
        assert np.array_equal(np.load(tmp_path / "b.npy"), arr) and np.array_equal(ck.read_npy(tmp_path / "b.npy"), arr)
    np.save(tmp_path / "c.npy", a)  # a file written by NumPy itself (64-byte padding) is read as well
    assert np.array_equal(ck.read_npy(tmp_path / "c.npy"), a)
    (tmp_path / "bad.npy").write_bytes(b"not an npy file")
    with pytest.raises(Exception, match="not an npy file"):
        ck.read_npy(tmp_path / "bad.npy")


def test_state_names_are_sanitised_like_the_reference():
    assert ck.sanitize_state_name("block.0.attention.q_proj.weight") == "block_0_attention_q_proj_weight"
    assert ck.sanitize_state_name("a-b_c/d e") == "a-b_c_d_e"


@pytest.mark.gpu
def test_resume_from_a_checkpoint_is_exact(tmp_path):
    import torch

    from heirloom_b200 import nn
    from tests.gpu_util import ctx
    c = ctx()
    kw = dict(vocab=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, context=128)
    opt = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, clip_norm=None)
    model = nn.DecoderLm(c, nn.DecoderConfig(batch=2, **kw))
    model.load_state_dict(ho.init_parameters(ho.DecoderConfig(**kw), 3))
    model.set_optimizer(**opt)
    rng = np.random.default_rng(8)
    batches = [ho.zipf_tokens(rng, 512, (2, 129)) for _ in range(5)]

    def step(m, tok):
        return m.train_step(torch.tensor(tok[:, :-1].copy()).pin_memory(), torch.tensor(tok[:, 1:].copy()).pin_memory())

    for tok in batches[:3]:
        step(model, tok)
    for sidecar in (False, True):
        d = tmp_path / ("side" if sidecar else "json")
        ck.save_checkpoint(d, model, opt, dataset_rng_state=77, dataset_batches_seen=3, moments_sidecar=sidecar)
    want = [step(model, tok) for tok in batches[3:]]
    want_param = model.parameter("block.1.feed_forward.dense.fc2.weight")
    model.close()

    # layout
    d = tmp_path / "json"
    lines = (d / "model" / "state.tsv").read_text().splitlines()
    assert lines[0] == "token_embedding.weight\t0000_token_embedding_weight.npy"
    assert len(lines) == len(ho.parameter_names(ho.DecoderConfig(**kw)))
    meta = json.loads((d / "metadata.json").read_text())
    assert meta["model_family"] == "memory_transformer" and meta["step"] == 3 and meta["dataset_rng_state"] == 77
    assert meta["memory_config"]["vocab_size"] == 512 and meta["memory_config"]["memory_layer_indices"] == []
    ostate = json.loads((d / "optimizer.json").read_text())
    assert ostate["step"] == 3 and len(ostate["m"]) == len(lines) and ostate["clip_norm"] is None
    assert set(ostate) == {"step", "lr", "beta1", "beta2", "eps", "weight_decay", "clip_norm", "m", "v"}

    for name in ("json", "side"):
        resumed, meta2 = ck.load_checkpoint(tmp_path / name, c, batch=2)
        assert resumed.optimizer_steps == 3 and meta2["dataset_batches_seen"] == 3
        got = [step(resumed, tok) for tok in batches[3:]]
        assert got == want, (name, got, want)  # bit-exact losses
        assert np.array_equal(resumed.parameter("block.1.feed_forward.dense.fc2.weight"), want_param)
        resumed.close()

    # a manifest that names an unknown parameter, or lacks one, is refused
    bad = tmp_path / "json" / "model" / "state.tsv"
    text = bad.read_text()
    bad.write_text(text + "extra.weight\t0000_token_embedding_weight.npy\n")
    with pytest.raises(Exception, match="unexpected parameter"):
        ck.load_checkpoint(tmp_path / "json", c, batch=2)
    bad.write_text("".join(text.splitlines(keepends=True)[1:]))
    with pytest.raises(Exception, match="missing state_dict parameter"):
        ck.load_checkpoint(tmp_path / "json", c, batch=2)

"""The C++ tensor interface above the C ABI (`heirloom_b200/host`): catalog, custom ops, views, autograd
driver and modules.  The scenarios live in `host/host_tests.cpp` and follow the reference's own tests;
the decoder case is checked here against the oracle."""
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest

from heirloom_b200 import build as hb
from oracle import heirloom_oracle as ho


def _driver() -> Path:
    hb.build_host()
    return hb.HOST_TESTS


def _run(*args) -> subprocess.CompletedProcess:
    return subprocess.run([str(_driver()), *map(str, args)], capture_output=True, text=True, timeout=600)


def test_catalog_custom_op_rules_views_and_gpu_only_routing_without_a_gpu():
    res = _run("cpu")
    assert res.returncode == 0, res.stdout + res.stderr
    assert "cpu: 0 failure(s)" in res.stdout


@pytest.mark.gpu
def test_device_ops_autograd_driver_and_adamw_closed_forms():
    res = _run("gpu")
    assert res.returncode == 0, res.stdout + res.stderr
    assert "gpu: 0 failure(s)" in res.stdout


@pytest.mark.gpu
def test_one_training_step_built_from_the_modules_matches_the_oracle(tmp_path):
    cfg = ho.DecoderConfig(vocab=48, d_model=32, n_layers=2, n_heads=4, d_ff=64, context=12)
    B, T = 3, 12
    params = ho.init_parameters(cfg, 5)
    rng = np.random.default_rng(6)
    for n in params:  # non-trivial biases and norm weights
        if n.endswith(".bias"):
            params[n] = ho.f32_round(rng.standard_normal(params[n].shape) * 0.05)
        elif ".ln" in n or n.startswith("ln_f"):
            params[n] = ho.f32_round(1.0 + rng.standard_normal(params[n].shape) * 0.05)
    tok = rng.integers(0, cfg.vocab, (B, T + 1))
    src, dst = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(src, "wb") as f:
        f.write(struct.pack("<8q", cfg.vocab, cfg.d_model, cfg.n_layers, cfg.n_heads, cfg.d_ff, cfg.context, B, T))
        for n in ho.parameter_names(cfg):
            f.write(np.asarray(params[n], np.float32).tobytes())
        f.write(np.ascontiguousarray(tok[:, :-1], np.int64).tobytes())
        f.write(np.ascontiguousarray(tok[:, 1:], np.int64).tobytes())
    res = _run("decoder", src, dst)
    assert res.returncode == 0, res.stdout + res.stderr
    raw = np.fromfile(dst, np.float32)
    want_loss, want_grads = ho.decoder_loss_and_grads(cfg, params, tok[:, :-1], tok[:, 1:], grad_f32=True)
    assert raw[0] == pytest.approx(want_loss, rel=1e-5)
    at = 1
    got_grads = {}
    for n, shape in ho.parameter_shapes(cfg).items():
        k = int(np.prod(shape))
        got_grads[n] = raw[at:at + k].astype(np.float64).reshape(shape)
        at += k
    for n in ho.parameter_names(cfg):
        if n.endswith("k_proj.bias"):  # mathematically zero: rounding noise on both sides
            assert np.abs(got_grads[n]).max() < 1e-6
            continue
        scale = max(np.abs(want_grads[n]).max(), 1e-12)
        assert np.abs(got_grads[n] - want_grads[n]).max() <= 2e-5 * scale + 1e-9, n
    state = ho.AdamWState()
    stepped = {n: p.copy() for n, p in params.items()}
    ho.adamw_step(stepped, want_grads, state)
    for n, shape in ho.parameter_shapes(cfg).items():
        k = int(np.prod(shape))
        got = raw[at:at + k].astype(np.float64).reshape(shape)
        at += k
        if n.endswith("k_proj.bias"):
            continue
        assert np.abs(got - stepped[n]).max() <= 2e-5, n
    assert at == raw.size

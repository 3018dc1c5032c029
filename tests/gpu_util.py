"""Helpers shared by the GPU parity tests."""
import numpy as np
import pytest
import torch

_CTX = None


def ctx():
    """One library context per test process (the C ABI's hl_ctx)."""
    global _CTX
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    if _CTX is None:
        from heirloom_b200 import cuda
        _CTX = cuda.Context(0)
    return _CTX


def dev(x, dtype=torch.float32):
    return torch.tensor(np.asarray(x), dtype=dtype, device="cuda")


def host(t):
    ctx().sync()
    return t.detach().to(torch.float64).cpu().numpy() if t.dtype.is_floating_point else t.cpu().numpy()


def assert_close(name, got, want, atol=0.0, rtol=0.0):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    err = np.abs(got - want)
    bound = atol + rtol * np.abs(want)
    if not np.all(err <= bound):
        i = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(f"{name}: max violation at {i}: got {got[i]!r} want {want[i]!r} (err {err[i]:.3e})")

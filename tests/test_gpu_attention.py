"""Parity of the tcgen05 flash attention against the oracle's attention on bf16-valued inputs."""
import numpy as np
import pytest
import torch

from oracle import heirloom_oracle as ho
from tests.gpu_util import assert_close, ctx, dev, host

pytestmark = pytest.mark.gpu


def reference_lse(q, k, n_heads):
    B, T, C = q.shape
    hd = C // n_heads
    qh = q.reshape(B, T, n_heads, hd).transpose(0, 2, 1, 3)
    kh = k.reshape(B, T, n_heads, hd).transpose(0, 2, 1, 3)
    s = np.matmul(qh, kh.transpose(0, 1, 3, 2)) / np.sqrt(hd)
    s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
    m = s.max(-1)
    return m + np.log(np.exp(s - m[..., None]).sum(-1))


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("B,T,H", [(1, 128, 1), (2, 256, 3), (1, 200, 2), (2, 1024, 2), (1, 72, 4), (1, 4096, 1), (1, 2100, 2)])
def test_flash_forward_matches_oracle(B, T, H, hd):
    from heirloom_b200 import cuda
    c = ctx()
    C = hd * H
    rng = np.random.default_rng(B * 1000 + T + H)
    qkv = ho.bf16_round(rng.standard_normal((B * T, 3 * C)) * 1.2)
    fused = dev(qkv, torch.bfloat16)
    q, k, v = fused[:, :C], fused[:, C:2 * C], fused[:, 2 * C:]
    out, lse = cuda.flash_attention_forward(c, q, k, v, B, T, H)
    assert out.shape == (B * T, C)
    qn, kn, vn = (qkv[:, i * C:(i + 1) * C].reshape(B, T, C) for i in range(3))
    want = ho.causal_attention(qn, kn, vn, H, round_probs_bf16=True)
    # P is rounded to bf16 before the PV product (as the reference's tensor-core route does) and
    # the row maximum it is rounded against may differ by tile order: allow 2 bf16 ulps + 1e-2.
    assert_close("flash out", host(out).reshape(B, T, C), want, atol=1e-2, rtol=2 ** -6)
    assert_close("lse", host(lse), reference_lse(qn, kn, H), atol=1e-4, rtol=1e-5)


def test_flash_forward_rejects_unsupported_shapes():
    from heirloom_b200 import cuda
    from heirloom_b200._lib import HeirloomError
    c = ctx()
    x = c.zeros((128, 96), torch.bfloat16)
    with pytest.raises(HeirloomError, match="head_dim must be 64 or 128"):
        cuda.flash_attention_forward(c, x, x, x, 1, 128, 3)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("B,T,H", [(1, 128, 1), (2, 256, 2), (1, 200, 2), (1, 1024, 2), (2, 72, 3), (1, 4096, 1), (1, 2100, 2)])
def test_flash_backward_matches_oracle(B, T, H, hd):
    from heirloom_b200 import cuda
    c = ctx()
    C = hd * H
    rng = np.random.default_rng(B * 77 + T + H)
    qkv = ho.bf16_round(rng.standard_normal((B * T, 3 * C)))
    go = ho.bf16_round(rng.standard_normal((B * T, C)))
    fused = dev(qkv, torch.bfloat16)
    q, k, v = fused[:, :C], fused[:, C:2 * C], fused[:, 2 * C:]
    out, lse = cuda.flash_attention_forward(c, q, k, v, B, T, H)
    dqkv = cuda.flash_attention_backward(c, q, k, v, out, dev(go, torch.bfloat16), lse, B, T, H)
    got = host(dqkv)
    qn, kn, vn = (qkv[:, i * C:(i + 1) * C].reshape(B, T, C) for i in range(3))
    want = ho.causal_attention_backward(qn, kn, vn, H, go.reshape(B, T, C), bf16_operands=True)
    for i, name in enumerate(("dq", "dk", "dv")):
        w = want[i].reshape(B * T, C)
        g = got[:, i * C:(i + 1) * C]
        scale = np.abs(w).max()
        # bf16 operands on both sides; rounding of P/dS happens against slightly different f32
        # values, so compare at a few bf16 ulps of the tensor's scale
        assert_close("flash " + name, g, w, atol=scale * 2 ** -6, rtol=2 ** -5)
        assert np.abs(g - w).mean() <= scale * 2 ** -9

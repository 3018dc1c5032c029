"""Parity of the tcgen05 GEMM against f64 products of the same bf16-rounded operands."""
import numpy as np
import pytest
import torch

from oracle import heirloom_oracle as ho
from tests.gpu_util import assert_close, ctx, dev, host

pytestmark = pytest.mark.gpu


def operands(rng, m, n, k, a_mn, b_mn):
    a = ho.bf16_round(rng.standard_normal((m, k)))
    b = ho.bf16_round(rng.standard_normal((k, n)))
    a_store = a.T.copy() if a_mn else a          # [k][m] or [m][k]
    b_store = b.copy() if b_mn else b.T.copy()   # [k][n] or [n][k]
    return a, b, dev(a_store, torch.bfloat16), dev(b_store, torch.bfloat16)


SHAPES = [(128, 256, 64), (256, 512, 320), (384, 768, 768), (100, 72, 40), (1000, 264, 1032), (130, 8, 16)]


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_all_operand_majors(m, n, k, a_mn, b_mn):
    from heirloom_b200 import cuda
    if (a_mn and m % 8) or (b_mn and n % 8) or (not a_mn and k % 8) or (not b_mn and k % 8):
        pytest.skip("leading dimension must be a multiple of 8")
    c = ctx()
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a, b, da, db = operands(rng, m, n, k, a_mn, b_mn)
    out = cuda.gemm_bf16(c, da, db, m, n, k, cuda.MN_MAJOR if a_mn else cuda.K_MAJOR,
                         cuda.MN_MAJOR if b_mn else cuda.K_MAJOR, out_dtype=torch.float32)
    want = a @ b
    assert_close("gemm f32 out", host(out), want, atol=1e-3 * np.sqrt(k / 64), rtol=1e-5)
    outb = cuda.gemm_bf16(c, da, db, m, n, k, cuda.MN_MAJOR if a_mn else cuda.K_MAJOR,
                          cuda.MN_MAJOR if b_mn else cuda.K_MAJOR, out_dtype=torch.bfloat16)
    assert_close("gemm bf16 out", host(outb), want, atol=1e-2, rtol=2 ** -7)
    assert c.counters().gemm_tcgen05_launches >= 2


def test_gemm_epilogues_match_the_amp_rounding_points():
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(11)
    m, n, k = 300, 520, 200
    a, b, da, db = operands(rng, m, n, k, False, False)
    bias = rng.standard_normal(n).astype(np.float32)
    acc = a @ b
    # bias
    out = cuda.gemm_bf16(c, da, db, m, n, k, epilogue=cuda.EPI_BIAS, bias=dev(bias), out_dtype=torch.float32)
    assert_close("bias", host(out), acc + bias, atol=2e-3, rtol=1e-5)
    # bias + gelu: h = bf16(acc+bias), g = bf16(gelu(h))
    h, g = cuda.gemm_bf16(c, da, db, m, n, k, epilogue=cuda.EPI_BIAS_GELU, bias=dev(bias), want_aux_out=True)
    hh = host(h)
    assert_close("h", hh, acc + bias, atol=1e-2, rtol=2 ** -7)
    # the epilogue uses the hardware tanh (relative error ~2^-11) before rounding to bf16
    assert_close("g", host(g), ho.bf16_round(ho.gelu_value(hh)), atol=2e-3, rtol=2 ** -7)
    # bias + residual: bf16(res + bf16(acc + bias))
    res = ho.bf16_round(rng.standard_normal((m, n)))
    out = cuda.gemm_bf16(c, da, db, m, n, k, epilogue=cuda.EPI_BIAS_RESIDUAL, bias=dev(bias),
                         aux_in=dev(res, torch.bfloat16))
    want = ho.bf16_round(res + ho.bf16_round(acc + bias))
    assert_close("residual", host(out), want, atol=2e-2, rtol=2 ** -6)
    # dgelu: acc * gelu'(h)
    hin = ho.bf16_round(rng.standard_normal((m, n)))
    out = cuda.gemm_bf16(c, da, db, m, n, k, epilogue=cuda.EPI_DGELU, aux_in=dev(hin, torch.bfloat16),
                         out_dtype=torch.float32)
    assert_close("dgelu", host(out), acc * ho.gelu_backward(hin, np.ones_like(hin)), atol=2e-2, rtol=2e-3)


def test_gemm_split_k_is_deterministic_and_matches():
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(12)
    m, n, k = 256, 264, 4096   # wgrad-like: small output, long contraction, both operands MN-major
    a, b, da, db = operands(rng, m, n, k, True, True)
    want = a @ b
    outs = [host(cuda.gemm_bf16(c, da, db, m, n, k, cuda.MN_MAJOR, cuda.MN_MAJOR, out_dtype=torch.float32,
                                split_k=s)) for s in (1, 4, 4, 0)]
    for o in outs:
        assert_close("split-k", o, want, atol=1e-2, rtol=1e-5)
    assert np.array_equal(outs[1], outs[2])


def test_gemm_rejects_bad_arguments_before_launch():
    from heirloom_b200 import cuda
    from heirloom_b200._lib import HeirloomError
    c = ctx()
    a = c.zeros((16, 12), torch.bfloat16)
    with pytest.raises(HeirloomError, match="multiples of 8"):
        cuda.gemm_bf16(c, a, a, 16, 16, 12)
    with pytest.raises(HeirloomError, match="positive"):
        cuda.gemm_bf16(c, a, a, 0, 16, 8)

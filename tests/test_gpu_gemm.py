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


def split_bf16(ctx_, x, mode):
    """`hl_split_bf16_f32` on an f32 matrix; returns the bf16 pieces laid side by side."""
    from heirloom_b200 import cuda
    rows, cols = x.shape
    pieces = 2 if mode == cuda.SPLIT_HI_LO else 3
    out = torch.empty(rows, pieces * cols, dtype=torch.bfloat16, device="cuda")
    cuda.check(ctx_.lib.hl_split_bf16_f32(ctx_.handle, cuda._p(x), cuda._p(out), cuda.c_longlong(rows), cuda.c_int(cols),
                                          cuda.c_int(mode)))
    return out


def test_split_pieces_rebuild_the_f32_value_exactly():
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(31)
    x = (rng.standard_normal((50, 72)) * np.exp(rng.uniform(-6, 6, (50, 72)))).astype(np.float32)
    x[0, :4] = [0.0, -0.0, 1.0, -3.5]
    p = host(split_bf16(c, dev(x), cuda.SPLIT_HI_MID_LO))
    assert np.array_equal(p[:, :72], ho.bf16_round(x))
    assert np.array_equal((p[:, :72] + p[:, 72:144] + p[:, 144:]).astype(np.float32), x)
    q = host(split_bf16(c, dev(x), cuda.SPLIT_HI_HI_LO))
    assert np.array_equal(q[:, :72], p[:, :72]) and np.array_equal(q[:, 72:144], p[:, :72]) and np.array_equal(q[:, 144:], p[:, 72:144])
    r = host(split_bf16(c, dev(x), cuda.SPLIT_HI_LO))
    assert np.array_equal(r[:, :72], p[:, :72]) and np.array_equal(r[:, 72:], p[:, 72:144])


@pytest.mark.parametrize("m,n,k", [(300, 264, 128), (1024, 512, 512)])
def test_gemm_with_a_repeated_operand_reaches_f32_accuracy(m, n, k):
    """x [m,k] bf16-exact against an f32 weight [n,k]: one accumulation over the weight's three bf16 pieces, the input
    read three times (a_k_period), equals the f64 product of the f32 operands to f32 rounding."""
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(m + n + k)
    x = ho.bf16_round(rng.standard_normal((m, k)))
    w = rng.standard_normal((n, k)).astype(np.float32)
    w3 = split_bf16(c, dev(w), cuda.SPLIT_HI_MID_LO)
    out = cuda.gemm_bf16(c, dev(x, torch.bfloat16), w3, m, n, 3 * k, out_dtype=torch.float32, a_k_period=k)
    want = x @ w.astype(np.float64).T
    scale = np.abs(want).max()
    assert np.abs(host(out) - want).max() <= 2e-6 * scale   # plain bf16 operands would be off by ~4e-3 of scale
    # both operands f32: hi*hi + lo*hi + hi*lo, the dropped lo*lo term is 2^-16 relative
    a = rng.standard_normal((m, k)).astype(np.float32)
    a2 = split_bf16(c, dev(a), cuda.SPLIT_HI_LO)
    wb = split_bf16(c, dev(w), cuda.SPLIT_HI_HI_LO)
    out = cuda.gemm_bf16(c, a2, wb, m, n, 3 * k, out_dtype=torch.float32, a_k_period=2 * k)
    want = a.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(host(out) - want).max() <= 6e-5 * np.abs(want).max()


def split_bf16_rows(ctx_, x, mode):
    """The pieces one below the other: `[pieces*rows, cols]`."""
    from heirloom_b200 import cuda
    rows, cols = x.shape
    pieces = 2 if mode == cuda.SPLIT_HI_LO else 3
    out = torch.empty(pieces * rows, cols, dtype=torch.bfloat16, device="cuda")
    cuda.check(ctx_.lib.hl_split_bf16_f32(ctx_.handle, cuda._p(x), cuda._p(out), cuda.c_longlong(rows), cuda.c_int(cols),
                                          cuda.c_int(mode | cuda.SPLIT_STACK_ROWS)))
    return out


def test_weight_gradient_shaped_products_of_f32_operands_reach_f32_accuracy():
    """dW[p,q] = sum_t dy[t,p] x[t,q]: both operands stored row-per-token, contracted down their rows.  The pieces lie
    one below the other; x bf16-exact is read three times (b_k_period), or both operands f32 with dy's two pieces read
    as hi, lo, hi (a_k_period) against x's hi, hi, lo."""
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(77)
    t, p, q = 1024, 256, 384
    dy = (rng.standard_normal((t, p)) * np.exp(rng.uniform(-3, 3, (t, 1)))).astype(np.float32)
    xb = ho.bf16_round(rng.standard_normal((t, q)))
    dy3 = split_bf16_rows(c, dev(dy), cuda.SPLIT_HI_MID_LO)
    assert np.array_equal(host(dy3)[:t], ho.bf16_round(dy))
    assert np.array_equal((host(dy3)[:t] + host(dy3)[t:2 * t] + host(dy3)[2 * t:]).astype(np.float32), dy)
    out = cuda.gemm_bf16(c, dy3, dev(xb, torch.bfloat16), p, q, 3 * t, a_layout=cuda.MN_MAJOR, b_layout=cuda.MN_MAJOR,
                         out_dtype=torch.float32, b_k_period=t)
    want = dy.astype(np.float64).T @ xb
    assert np.abs(host(out) - want).max() <= 2e-6 * np.abs(want).max()
    x = rng.standard_normal((t, q)).astype(np.float32)
    dy2 = split_bf16_rows(c, dev(dy), cuda.SPLIT_HI_LO)
    x3 = split_bf16_rows(c, dev(x), cuda.SPLIT_HI_HI_LO)
    out = cuda.gemm_bf16(c, dy2, x3, p, q, 3 * t, a_layout=cuda.MN_MAJOR, b_layout=cuda.MN_MAJOR,
                         out_dtype=torch.float32, a_k_period=2 * t)
    want = dy.astype(np.float64).T @ x.astype(np.float64)
    assert np.abs(host(out) - want).max() <= 6e-5 * np.abs(want).max()
    # the split-K route (k blocks dealt over CTAs) wraps the same way
    out2 = cuda.gemm_bf16(c, dy2, x3, p, q, 3 * t, a_layout=cuda.MN_MAJOR, b_layout=cuda.MN_MAJOR,
                          out_dtype=torch.float32, a_k_period=2 * t, split_k=4)
    assert np.abs(host(out2) - want).max() <= 6e-5 * np.abs(want).max()


def test_an_expired_pipeline_wait_ends_the_kernel_with_a_status_and_leaves_the_context_usable():
    """Failure detection without a fault: the producer is told to leave one k block of the first tile out, so the MMA
    issuer's wait for that stage can never be satisfied; with the bound set to 200 microseconds the wait gives up, every
    role leaves its loop, the kernel frees its tensor memory and returns, and the next sync reports the status word.
    Nothing traps and nothing spins: the next GEMM on the same context is correct."""
    from heirloom_b200 import cuda
    from heirloom_b200._lib import HeirloomError
    c = ctx()
    rng = np.random.default_rng(51)
    m, n, k = 128, 256, 256
    a, b, da, db = operands(rng, m, n, k, False, False)
    c.sync()
    c.set_test_hooks(wait_limit_ns=200_000, gemm_skip_kblock=1)
    try:
        cuda.gemm_bf16(c, da, db, m, n, k, out_dtype=torch.float32)
        with pytest.raises(HeirloomError, match="bounded pipeline wait expired"):
            c.sync()
    finally:
        c.set_test_hooks(0, -1)
    c.sync()  # the status was reported once and cleared
    out = cuda.gemm_bf16(c, da, db, m, n, k, out_dtype=torch.float32)
    assert_close("gemm after an expired wait", host(out), a @ b, atol=2e-3, rtol=1e-5)


def test_tiles_handed_out_by_a_counter_give_the_same_bits_as_round_robin(monkeypatch):
    """HEIRLOOM_GEMM_DYNAMIC (read at every call; on by default only beside a communicator) changes which CTA computes
    which tile, never a tile's arithmetic: outputs are bit-identical, launch after launch (the counter is never reset,
    the host tracks its value), for whole tiles, equal splits and a bf16 epilogue."""
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(91)
    monkeypatch.setenv("HEIRLOOM_GEMM_PAIRS", "0")
    cases = [(4096, 2048, 320, 0, torch.float32), (1000, 520, 1032, 4, torch.float32), (2304, 1024, 128, 1, torch.bfloat16)]
    for m, n, k, split, dt in cases:
        a = dev(ho.bf16_round(rng.standard_normal((m, k))), torch.bfloat16)
        b = dev(ho.bf16_round(rng.standard_normal((n, k))), torch.bfloat16)
        monkeypatch.setenv("HEIRLOOM_GEMM_DYNAMIC", "0")
        want = cuda.gemm_bf16(c, a, b, m, n, k, out_dtype=dt, split_k=split).clone()
        monkeypatch.setenv("HEIRLOOM_GEMM_DYNAMIC", "1")
        for _ in range(3):
            got = cuda.gemm_bf16(c, a, b, m, n, k, out_dtype=dt, split_k=split)
            assert torch.equal(got, want), (m, n, k, split)
    c.sync()


PAIR_SCRIPT = r"""
import numpy as np, torch
from oracle import heirloom_oracle as ho
from tests.gpu_util import ctx, dev, host
from heirloom_b200 import cuda
c = ctx()
rng = np.random.default_rng(5)
for (m, n, k, a_mn, b_mn) in [(256, 256, 64, False, False), (1000, 264, 1032, False, False), (384, 768, 768, True, True),
                              (2048, 512, 320, False, True), (640, 1024, 192, True, False)]:
    a = ho.bf16_round(rng.standard_normal((m, k))); b = ho.bf16_round(rng.standard_normal((k, n)))
    a_store = a.T.copy() if a_mn else a
    b_store = b.copy() if b_mn else b.T.copy()
    out = cuda.gemm_bf16(c, dev(a_store, torch.bfloat16), dev(b_store, torch.bfloat16), m, n, k,
                         cuda.MN_MAJOR if a_mn else cuda.K_MAJOR, cuda.MN_MAJOR if b_mn else cuda.K_MAJOR,
                         out_dtype=torch.float32, split_k=1)  # whole tiles: the only work split that runs on pairs
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(host(out) - want).max() <= 2e-6 * np.abs(want).max() * np.sqrt(k), (m, n, k)
# bias + residual epilogue into bf16, ragged rows
m, n, k = 1500, 768, 768
a = ho.bf16_round(rng.standard_normal((m, k))); w = ho.bf16_round(rng.standard_normal((n, k)) * 0.05)
bias = rng.standard_normal(n).astype(np.float32); res = ho.bf16_round(rng.standard_normal((m, n)))
out = cuda.gemm_bf16(c, dev(a, torch.bfloat16), dev(w, torch.bfloat16), m, n, k, epilogue=cuda.EPI_BIAS_RESIDUAL,
                     bias=dev(bias), aux_in=dev(res, torch.bfloat16))
want = ho.bf16_round(res + ho.bf16_round(a.astype(np.float64) @ w.T.astype(np.float64) + bias))
assert np.abs(host(out) - want).max() <= 2.0 ** -7 * np.abs(want).max()
# a weight-gradient shape: few tiles, the contraction in four equal splits summed by the second kernel
m, n, k = 512, 768, 4096
a = ho.bf16_round(rng.standard_normal((k, m))); b = ho.bf16_round(rng.standard_normal((k, n)))
out = cuda.gemm_bf16(c, dev(a, torch.bfloat16), dev(b, torch.bfloat16), m, n, k, cuda.MN_MAJOR, cuda.MN_MAJOR,
                     out_dtype=torch.float32, split_k=4)
want = a.T.astype(np.float64) @ b.astype(np.float64)
assert np.abs(host(out) - want).max() <= 2e-6 * np.abs(want).max() * np.sqrt(k)
c.sync()
n_pair, n_all = c.counters().gemm_pair_launches, c.counters().gemm_tcgen05_launches
assert n_pair == n_all == 7, (n_pair, n_all)
print("pairs ok")
"""


def test_gemm_on_cta_pairs_matches_in_a_process_that_opts_in():
    """HEIRLOOM_GEMM_PAIRS=1 (read once per process) runs whole-tile products on clusters of two CTAs: 256-row tiles,
    one MMA issuer for both SMs, each CTA staging half of B.  Same results, all operand majors, ragged edges."""
    import os, subprocess, sys
    from pathlib import Path
    env = dict(os.environ, HEIRLOOM_GEMM_PAIRS="1")
    res = subprocess.run([sys.executable, "-c", PAIR_SCRIPT], env=env, cwd=str(Path(__file__).resolve().parents[1]),
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "pairs ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]

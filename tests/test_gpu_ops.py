"""Parity of the memory-bound device ops against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import heirloom_oracle as ho
from tests.gpu_util import assert_close, ctx, dev, host

pytestmark = pytest.mark.gpu
F32_TOL = dict(atol=1e-6, rtol=2e-6)


def test_device_is_sm100_and_counters_count():
    from heirloom_b200 import cuda
    c = ctx()
    info = c.device_info()
    assert info.sm_major == 10 and info.supports_tcgen05 == 1 and info.sm_count > 0
    c.reset_counters()
    cuda.fill_f32(c, c.empty(10), 1.0)
    assert c.counters().launches == 1


@pytest.mark.parametrize("n", [1, 7, 1024, 100003])
def test_binary_scale_relu_fill(n):
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(n)
    a = rng.standard_normal(n).astype(np.float32)
    b = (rng.standard_normal(n) + 3.0).astype(np.float32)
    da, db = dev(a), dev(b)
    for op, fn in ((cuda.ADD, np.add), (cuda.SUB, np.subtract), (cuda.MUL, np.multiply), (cuda.DIV, np.divide)):
        assert np.array_equal(host(cuda.binary_f32(c, op, da, db)), fn(a, b).astype(np.float64))
    assert np.array_equal(host(cuda.scale_f32(c, da, 0.37)), (a * np.float32(0.37)).astype(np.float64))
    assert np.array_equal(host(cuda.relu_f32(c, da)), ho.relu(a))
    assert np.array_equal(host(cuda.relu_backward_f32(c, da, db)), ho.relu_backward(a, b))
    out = c.empty(n)
    cuda.fill_f32(c, out, 2.5)
    assert np.all(host(out) == 2.5)


@pytest.mark.parametrize("n", [5, 4096, 65537])
def test_casts_are_round_to_nearest_even_bit_exact(n):
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 10 ** rng.uniform(-3, 3, n)).astype(np.float32)
    x[:3] = [1.00390625, 1.01171875, -0.0][: min(3, n)]
    bits = host(cuda.cast(c, dev(x), torch.bfloat16).view(torch.int16)).astype(np.int16).view(np.uint16)
    assert np.array_equal(bits, ho.f32_to_bf16_bits(x))
    rt = host(cuda.cast(c, dev(x), torch.float32))
    assert np.array_equal(rt, ho.bf16_round(x))
    back = host(cuda.cast(c, cuda.cast(c, dev(x), torch.bfloat16), torch.float32))
    assert np.array_equal(back, ho.bf16_round(x))


def test_gelu_forward_backward_f32_and_bf16(golden):
    from heirloom_b200 import cuda
    c = ctx()
    case = golden["ops"]["gelu_tanh_mean"]
    x = np.asarray(case["tensors"]["x"]["values"], np.float32)
    y = host(cuda.gelu(c, dev(x)))
    assert abs(y.mean() - case["expect"]["values"][0]) <= 2e-5
    g = host(cuda.gelu_backward(c, dev(x), dev(np.full(x.shape, 1.0 / x.size, np.float32))))
    assert_close("golden gelu grad", g, case["expect_grads"]["x"], atol=2e-5)
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(50001) * 3).astype(np.float32)
    go = rng.standard_normal(50001).astype(np.float32)
    assert_close("gelu", host(cuda.gelu(c, dev(x))), ho.gelu(x), **F32_TOL)
    assert_close("gelu bwd", host(cuda.gelu_backward(c, dev(x), dev(go))), ho.gelu_backward(x, go), **F32_TOL)
    xb = ho.bf16_round(x)
    yb = host(cuda.gelu(c, dev(xb, torch.bfloat16)))
    assert_close("gelu bf16", yb, ho.bf16_round(ho.gelu_value(xb)), atol=1e-6, rtol=2 ** -7)


@pytest.mark.parametrize("rows,cols", [(3, 5), (1000, 768), (4097, 130)])
def test_bias_add_and_bias_grad(rows, cols):
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(rows)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    b = rng.standard_normal(cols).astype(np.float32)
    assert np.array_equal(host(cuda.bias_add_f32(c, dev(x), dev(b))), (x + b).astype(np.float64))
    # f32 partial sums per thread, folded in f64: the reference's kernel is a serial f32 sum
    tol = dict(atol=2e-6 * np.sqrt(rows), rtol=1e-5)
    assert_close("bias grad f32", host(cuda.bias_grad(c, dev(x))), ho.f32_round(x.astype(np.float64).sum(0)), **tol)
    xb = ho.bf16_round(x)
    assert_close("bias grad bf16", host(cuda.bias_grad(c, dev(xb, torch.bfloat16))), ho.f32_round(xb.sum(0)), **tol)


@pytest.mark.parametrize("n", [1, 1000, 3000001])
def test_reductions(n):
    from heirloom_b200 import cuda
    c = ctx()
    x = np.random.default_rng(n).standard_normal(n).astype(np.float32)
    x64 = x.astype(np.float64)
    assert_close("sum", host(cuda.sum_f32(c, dev(x)))[0], np.float32(x64.sum()), **F32_TOL)
    assert_close("mean", host(cuda.mean_f32(c, dev(x)))[0], np.float32(x64.mean()), atol=1e-7, rtol=2e-6)
    assert_close("sumsq", host(cuda.sum_squares_f32(c, dev(x)))[0], np.float32((x64 * x64).sum()), **F32_TOL)


def test_layer_norm_golden_vector(golden):
    from heirloom_b200 import cuda
    c = ctx()
    case = golden["ops"]["layer_norm_square_sum"]
    t = {k: np.asarray(v["values"], np.float32).reshape(v["dims"]) for k, v in case["tensors"].items()}
    names = list(t)
    x, w, b = (t[n] for n in names)
    y, mean, rstd = cuda.layer_norm_forward(c, dev(x), dev(w), dev(b), case["eps"])
    yh = host(y)
    assert abs((yh * yh).sum() - case["expect"]["values"][0]) <= 2e-5
    dx, dg, db = cuda.layer_norm_backward(c, dev(x), dev(w), dev(2.0 * yh), mean, rstd)
    for name, got in zip(names, (dx, dg, db)):
        assert_close(name, host(got).reshape(-1), case["expect_grads"][name], atol=2e-5)


@pytest.mark.parametrize("rows,feat", [(1, 4), (33, 128), (1024, 768), (257, 1024), (5, 6)])
def test_layer_norm_f32_matches_oracle(rows, feat):
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(rows * feat)
    x = (rng.standard_normal((rows, feat)) * 2 + 0.5).astype(np.float32)
    w = rng.standard_normal(feat).astype(np.float32)
    b = rng.standard_normal(feat).astype(np.float32)
    dy = rng.standard_normal((rows, feat)).astype(np.float32)
    y, mean, rstd = cuda.layer_norm_forward(c, dev(x), dev(w), dev(b))
    assert_close("ln fwd", host(y), ho.layer_norm(x, w, b), **F32_TOL)
    if feat % 4 == 0:
        res = rng.standard_normal((rows, feat)).astype(np.float32)
        dxo, dwo, dbo = ho.layer_norm_backward(x, w, dy)
        for saved in (True, False):
            dx, dg, db = cuda.layer_norm_backward(c, dev(x), dev(w), dev(dy), mean if saved else None,
                                                  rstd if saved else None)
            assert_close("ln dx", host(dx), dxo, atol=2e-6, rtol=1e-5)
            assert_close("ln dgamma", host(dg), dwo, atol=1e-5, rtol=1e-5)
            assert_close("ln dbeta", host(db), dbo, atol=1e-5, rtol=1e-5)
        dx, dxb, _, _ = cuda.layer_norm_backward(c, dev(x), dev(w), dev(dy), mean, rstd, dev(res), want_bf16=True)
        assert_close("ln dx+res", host(dx), res + ho.f32_round(dxo), atol=3e-6, rtol=1e-5)
        assert np.array_equal(host(dxb), ho.bf16_round(host(dx)))


def test_layer_norm_bf16_route():
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(5)
    rows, feat = 513, 768
    x = ho.bf16_round(rng.standard_normal((rows, feat)) * 1.5)
    w = (1 + 0.1 * rng.standard_normal(feat)).astype(np.float32)
    b = (0.1 * rng.standard_normal(feat)).astype(np.float32)
    y, mean, rstd = cuda.layer_norm_forward(c, dev(x, torch.bfloat16), dev(w), dev(b))
    want = ho.bf16_round(ho.layer_norm(x, w, b))
    # f32 statistics instead of f64: allow one bf16 ulp on a handful of elements
    assert_close("ln bf16", host(y), want, atol=1e-6, rtol=2 ** -7)
    assert np.mean(host(y) != want) < 0.01
    dy = rng.standard_normal((rows, feat)).astype(np.float32)
    res = rng.standard_normal((rows, feat)).astype(np.float32)
    dx, dxb, dg, db, cs = cuda.layer_norm_backward(c, dev(x, torch.bfloat16), dev(w), dev(dy), mean, rstd, dev(res),
                                                   want_bf16=True, want_colsum=True)
    dxo, dwo, dbo = ho.layer_norm_backward(x, w, dy)
    assert_close("ln bf16 dx", host(dx), res + dxo, atol=1e-4, rtol=1e-4)
    assert np.array_equal(host(dxb), ho.bf16_round(host(dx)))
    assert_close("ln bf16 dgamma", host(dg), dwo, atol=1e-3, rtol=1e-4)
    assert_close("ln bf16 dbeta", host(db), dbo, atol=1e-3, rtol=1e-4)
    assert_close("ln bf16 dx colsum", host(cs), host(dx).sum(0), atol=1e-3, rtol=1e-4)
    # the slower general route (no saved statistics) agrees
    dx2, dg2, db2, cs2 = cuda.layer_norm_backward(c, dev(x, torch.bfloat16), dev(w), dev(dy), None, None, dev(res),
                                                  want_colsum=True)
    assert_close("ln bf16 dx general", host(dx2), host(dx), atol=1e-4, rtol=1e-4)
    assert_close("ln bf16 colsum general", host(cs2), host(cs), atol=1e-3, rtol=1e-4)


def test_embedding_forward_backward(golden):
    from heirloom_b200 import cuda
    c = ctx()
    ka = golden["known_answers"]["embedding_scatter_add"]
    w = np.asarray(ka["weight"], np.float32)
    idx = np.asarray(ka["indices"], np.int64)
    out = cuda.embedding_forward(c, dev(w), dev(idx, torch.int64))
    assert np.array_equal(host(out), w[idx])
    gt = cuda.embedding_backward(c, dev(np.ones((3, 2), np.float32)), dev(idx, torch.int64), 2)
    assert np.array_equal(host(gt), np.asarray(ka["grad_weight"]))

    rng = np.random.default_rng(2)
    vocab, dim, B, T = 97, 132, 4, 33
    table = rng.standard_normal((vocab, dim)).astype(np.float32)
    pos = rng.standard_normal((T, dim)).astype(np.float32)
    tok = rng.integers(0, vocab, (B, T))
    tok[:, :5] = 3  # hot row
    out = cuda.embedding_forward(c, dev(table), dev(tok, torch.int64), dev(pos))
    assert np.array_equal(host(out), ho.add(ho.embedding(table, tok), pos[None]))
    outb = cuda.embedding_forward(c, dev(table), dev(tok, torch.int64), dev(pos), out_dtype=torch.bfloat16)
    assert np.array_equal(host(outb), ho.bf16_round(ho.bf16_round(table[tok]) + ho.bf16_round(pos[None])))
    go = rng.standard_normal((B, T, dim)).astype(np.float32)
    gt, gp = cuda.embedding_backward(c, dev(go), dev(tok, torch.int64), vocab, T)
    assert_close("dtable", host(gt), ho.embedding_backward(table.shape, tok, go), atol=1e-5, rtol=1e-5)
    assert_close("dpos", host(gp), go.astype(np.float64).sum(0), **F32_TOL)


def test_embedding_bad_index_sets_status_instead_of_faulting():
    from heirloom_b200 import cuda
    from heirloom_b200._lib import HeirloomError
    c = ctx()
    table = dev(np.zeros((4, 8), np.float32))
    cuda.embedding_forward(c, table, dev(np.array([1, 9]), torch.int64))
    with pytest.raises(HeirloomError, match="out-of-range"):
        c.sync()
    c.sync()  # the status word was cleared


def test_cross_entropy_golden_and_random(golden):
    from heirloom_b200 import cuda
    c = ctx()
    case = golden["ops"]["cross_entropy"]
    z = np.asarray(case["tensors"]["logits"]["values"], np.float32).reshape(case["tensors"]["logits"]["dims"])
    loss, d = cuda.cross_entropy(c, dev(z), dev(case["targets"], torch.int64))
    assert abs(host(loss)[0] - case["expect"]["values"][0]) <= 2e-5
    assert_close("dlogits", host(d).reshape(-1), case["expect_grads"]["logits"], atol=2e-5)
    rng = np.random.default_rng(4)
    for rows, classes in ((16, 256), (77, 50304), (5, 1001)):
        z = (rng.standard_normal((rows, classes)) * 3).astype(np.float32)
        t = rng.integers(0, classes, rows)
        loss, d = cuda.cross_entropy(c, dev(z), dev(t, torch.int64))
        assert_close("loss", host(loss)[0], ho.cross_entropy(z, t), atol=1e-6, rtol=1e-6)
        assert_close("dlogits", host(d), ho.f32_round(ho.cross_entropy_backward(z, t)), atol=1e-9, rtol=1e-5)
        loss, d = cuda.cross_entropy(c, dev(z), dev(t, torch.int64), dlogits_dtype=torch.bfloat16)
        assert_close("loss f32 math", host(loss)[0], ho.cross_entropy(z, t), atol=1e-5, rtol=1e-5)
        assert_close("dlogits bf16", host(d), ho.cross_entropy_backward(z, t), atol=1e-8, rtol=2 ** -7)


def test_adamw_matches_reference_kernel_order_bit_exact_and_multi_tensor():
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(6)
    sizes = [1, 5, 4096, 70001]
    ps = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    gs = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    ms = [np.zeros(n, np.float32) for n in sizes]
    vs = [np.zeros(n, np.float32) for n in sizes]
    dp, dg, dm, dv = ([dev(a) for a in group] for group in (ps, gs, ms, vs))
    shadows = [c.empty(n, torch.bfloat16) for n in sizes]
    single = [dev(ps[3]), dev(ms[3]), dev(vs[3])]
    for step in (1, 2, 3):
        hp = cuda.adamw_params(0.05, 0.9, 0.999, 1e-8, 0.01, 0.75, step)
        cuda.adamw_update_multi(c, dp, dg, dm, dv, hp, shadows)
        cuda.adamw_update_f32(c, single[0], dg[3], single[1], single[2], hp)
        for i in range(len(sizes)):
            ps[i], ms[i], vs[i] = ho.adamw_step_f32_kernel_order(
                ps[i], gs[i], ms[i], vs[i], 0.05, 0.9, 0.999, 1e-8, 0.01, 0.75,
                np.float32(1.0 - 0.9 ** step), np.float32(1.0 - 0.999 ** step))
            assert np.array_equal(host(dp[i]), ps[i].astype(np.float64)), (step, i)
            assert np.array_equal(host(dm[i]), ms[i].astype(np.float64))
            assert np.array_equal(host(dv[i]), vs[i].astype(np.float64))
            assert np.array_equal(host(shadows[i]), ho.bf16_round(ps[i]))
        assert np.array_equal(host(single[0]), ps[3].astype(np.float64))
    # the f32 kernel agrees with the f64 CPU body at the reference's own CPU-vs-CUDA tolerance
    params = {"w": rng.standard_normal(1000)}
    params["w"] = ho.f32_round(params["w"])
    g = ho.f32_round(rng.standard_normal(1000))
    st = ho.AdamWState(lr=0.05, weight_decay=0.01)
    p0 = dev(params["w"]); m0 = c.zeros(1000); v0 = c.zeros(1000)
    ho.adamw_step(params, {"w": g}, st)
    cuda.adamw_update_f32(c, p0, dev(g), m0, v0, cuda.adamw_params(0.05, 0.9, 0.999, 1e-8, 0.01, 1.0, 1))
    assert_close("adamw vs f64", host(p0), params["w"], atol=2e-4)


def test_matmul_f32_strided_views(golden):
    from heirloom_b200 import cuda
    c = ctx()
    case = golden["ops"]["matmul_mean"]
    names = list(case["tensors"])
    a, b = (np.asarray(case["tensors"][n]["values"], np.float32).reshape(case["tensors"][n]["dims"]) for n in names)
    out = host(cuda.matmul_f32_strided(c, dev(a), dev(b)))
    assert abs(out.mean() - case["expect"]["values"][0]) <= 2e-5
    rng = np.random.default_rng(8)
    x = rng.standard_normal((70, 45)).astype(np.float32)
    w = rng.standard_normal((33, 45)).astype(np.float32)
    got = host(cuda.matmul_f32_strided(c, dev(x), dev(w).t()))  # Linear: x · Wᵀ through a transposed view
    assert np.array_equal(got, ho.matmul(x, w.T))
    g = rng.standard_normal((70, 33)).astype(np.float32)
    ga, gb = ho.matmul_backward(x, w.T, g)
    assert np.array_equal(host(cuda.matmul_f32_strided(c, dev(g), dev(w))), ho.f32_round(ga))
    assert np.array_equal(host(cuda.matmul_f32_strided(c, dev(x).t(), dev(g))), ho.f32_round(gb))


def test_attention_f32_golden_and_random(golden):
    from heirloom_b200 import cuda
    c = ctx()
    case = golden["ops"]["causal_attention_square_sum"]
    names = list(case["tensors"])
    q, k, v = (np.asarray(case["tensors"][n]["values"], np.float32).reshape(case["tensors"][n]["dims"]) for n in names)
    o, p = cuda.causal_attention_f32_forward(c, dev(q), dev(k), dev(v), case["n_heads"])
    oh = host(o)
    assert abs((oh * oh).sum() - case["expect"]["values"][0]) <= 2e-5
    grads = cuda.causal_attention_f32_backward(c, dev(q), dev(k), dev(v), p, dev(2.0 * oh), case["n_heads"])
    for n, g in zip(names, grads):
        assert_close(n, host(g).reshape(-1), case["expect_grads"][n], atol=2e-5)
    rng = np.random.default_rng(9)
    B, T, H, hd = 2, 37, 4, 32
    q, k, v, go = (rng.standard_normal((B, T, H * hd)).astype(np.float32) for _ in range(4))
    o, p = cuda.causal_attention_f32_forward(c, dev(q), dev(k), dev(v), H)
    oo, po = ho.causal_attention(q, k, v, H, return_probs=True)
    assert_close("attn out", host(o), oo, atol=1e-6, rtol=1e-5)
    assert_close("attn probs", host(p), ho.f32_round(po), atol=1e-7, rtol=1e-5)
    dq, dk, dv = cuda.causal_attention_f32_backward(c, dev(q), dev(k), dev(v), p, dev(go), H)
    for name, got, want in zip("qkv", (dq, dk, dv), ho.causal_attention_backward(q, k, v, H, go, probs=po)):
        assert_close("attn d" + name, host(got), want, atol=1e-5, rtol=1e-4)


def test_closing_a_second_context_leaves_torch_and_the_first_context_usable():
    """A context makes its compute stream torch's current stream; closing it must hand torch a live stream back."""
    from heirloom_b200 import cuda
    first = ctx()
    second = cuda.Context(0)
    x = torch.arange(8, dtype=torch.float32, device="cuda")
    flags = cuda.mark_rows(second, torch.tensor([1, 3], device="cuda"), 4)
    second.sync()
    assert flags.cpu().tolist() == [0, 1, 0, 1]
    second.close()
    y = (x * 2).sum()                     # torch keeps working
    assert float(y) == 56.0
    flags = cuda.mark_rows(first, torch.tensor([0], device="cuda"), 4)
    first.sync()
    assert flags.cpu().tolist() == [1, 0, 0, 0]
    assert torch.cuda.current_stream().cuda_stream == first.stream.cuda_stream


def test_adamw_plan_steps_like_the_multi_tensor_call():
    """A plan built once and stepped three times gives the bits of three `adamw_update_multi` calls."""
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(16)
    sizes = [3, 4096, 50001]
    make = lambda: [dev(rng.standard_normal(n).astype(np.float32)) for n in sizes]
    ps, gs = make(), make()
    ps2 = [p.clone() for p in ps]
    zeros = lambda: [c.zeros(n) for n in sizes]
    ms, vs, ms2, vs2 = zeros(), zeros(), zeros(), zeros()
    sh, sh2 = [c.empty(n, torch.bfloat16) for n in sizes], [c.empty(n, torch.bfloat16) for n in sizes]
    plan = cuda.AdamWPlan(c, ps, gs, ms, vs, sh)
    for step in (1, 2, 3):
        hp = cuda.adamw_params(0.02, 0.9, 0.999, 1e-8, 0.01, 1.0, step)
        plan.step(hp)
        cuda.adamw_update_multi(c, ps2, gs, ms2, vs2, hp, sh2)
    for a, b in zip(ps + ms + vs + sh, ps2 + ms2 + vs2 + sh2):
        assert np.array_equal(host(a), host(b))
    plan.close()


def test_sgd_update_rounds_product_and_difference_separately():
    from heirloom_b200 import cuda
    from heirloom_b200._lib import HeirloomError
    c = ctx()
    rng = np.random.default_rng(41)
    p, g = rng.standard_normal(10007).astype(np.float32), rng.standard_normal(10007).astype(np.float32)
    dp = dev(p)
    cuda.sgd_update_f32(c, dp, dev(g), 0.05)
    want = (p - (np.float32(0.05) * g).astype(np.float32)).astype(np.float32)   # mul.f32 then sub.f32 (kernels.ptx:383-384)
    assert np.array_equal(host(dp).astype(np.float32), want)
    with pytest.raises(HeirloomError, match="learning rate must be positive"):
        cuda.sgd_update_f32(c, dp, dev(g), 0.0)


def test_arange_and_concat_of_index_vectors():
    from heirloom_b200 import cuda
    from heirloom_b200._lib import HeirloomError
    c = ctx()
    a = cuda.arange_i64(c, 1025)
    assert np.array_equal(host(a), np.arange(1025))
    parts = [torch.tensor([5, -3, 2 ** 40], dtype=torch.int64, device="cuda"), torch.empty(0, dtype=torch.int64, device="cuda"), a]
    got = cuda.concat_i64(c, parts)
    assert np.array_equal(host(got), np.concatenate([host(t) for t in parts]))
    with pytest.raises(HeirloomError, match="at least one input"):
        cuda.concat_i64(c, [])

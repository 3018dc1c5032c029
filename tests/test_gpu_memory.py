"""Parity of the product-key memory kernels: the reference's known answers, exact index equality
against the oracle on identical f32 scores, and random forward/backward checks."""
import numpy as np
import pytest
import torch

from oracle import heirloom_oracle as ho
from tests.gpu_util import assert_close, ctx, dev, host

pytestmark = pytest.mark.gpu
I64 = torch.int64


def test_topk_ties_known_answer_and_random(golden):
    from heirloom_b200 import cuda
    c = ctx()
    ka = golden["known_answers"]["topk_ties"]
    got = host(cuda.topk_rows(c, dev(ka["scores"]), ka["k"]))
    assert got.tolist() == ka["indices"]
    rng = np.random.default_rng(0)
    for rows, cols, k in ((7, 5, 5), (64, 512, 32), (33, 1000, 17)):
        s = rng.integers(-20, 20, (rows, cols)).astype(np.float32) / 4  # many exact ties
        assert np.array_equal(host(cuda.topk_rows(c, dev(s), k)), ho.topk_indices_dim1(s, k))


def test_product_key_primitives_known_answers(golden):
    from heirloom_b200 import cuda
    c = ctx()
    ka = golden["known_answers"]["product_key_primitives"]
    idx = cuda.product_key_topk_from_side_scores(c, dev(ka["left_scores"]), dev(ka["right_scores"]), ka["top_k"], ka["beam"])
    assert host(idx).tolist() == [[5, 3], [6, 0]]
    left, right = cuda.product_key_split_rows(c, dev(ka["split_rows"]["rows"], I64), ka["side"])
    assert host(left).tolist() == ka["split_rows"]["left"] and host(right).tolist() == ka["split_rows"]["right"]
    q, kl, kr = dev(ka["query"]), dev(ka["left_keys"]), dev(ka["right_keys"])
    indices = dev(ka["indices"], I64)
    s = cuda.memory_selected_scores_forward(c, indices, q, kl, kr)
    assert_close("scores", host(s), ka["scores"], atol=1e-6)
    dq, dl, dr = cuda.memory_selected_scores_backward(c, indices, q, kl, kr, dev(ka["grad_scores"]))
    assert_close("dq", host(dq), ka["grad_query"], atol=1e-6)
    assert_close("dleft", host(dl), ka["grad_left"], atol=1e-6)
    assert_close("dright", host(dr), ka["grad_right"], atol=1e-6)


def test_exact_lookup_and_weighted_value_known_answers(golden):
    from heirloom_b200 import cuda
    c = ctx()
    ka = golden["known_answers"]["selected_scores"]
    indices = dev(ka["indices"], I64)
    s = cuda.memory_selected_scores_forward(c, indices, dev(ka["query"]), dev(ka["keys"]))
    assert_close("scores", host(s), ka["scores"], atol=1e-6)
    dq, dk, _ = cuda.memory_selected_scores_backward(c, indices, dev(ka["query"]), dev(ka["keys"]), None, dev(ka["grad_scores"]))
    assert_close("dq", host(dq), ka["grad_query"], atol=1e-6)
    assert_close("dkeys", host(dk), ka["grad_keys"], atol=1e-6)
    ka = golden["known_answers"]["weighted_value"]
    indices = dev(ka["indices"], I64)
    # value rows of 2 are padded to 4 columns (row_dim must be a multiple of 4)
    vals = np.zeros((3, 4), np.float32); vals[:, :2] = ka["values"]
    out = cuda.memory_weighted_value_forward(c, indices, dev(ka["weights"]), dev(vals))
    assert_close("out", host(out)[:, :2], ka["output"], atol=1e-6)
    go = np.zeros((2, 4), np.float32); go[:, :2] = 1.0
    dw, dv = cuda.memory_weighted_value_backward(c, indices, dev(ka["weights"]), dev(vals), dev(go))
    assert_close("dw", host(dw), ka["grad_weights"], atol=1e-6)
    assert_close("dv", host(dv)[:, :2], ka["grad_values"], atol=1e-6)


@pytest.mark.parametrize("tokens,side,key_dim,top_k", [(5, 8, 16, 4), (300, 64, 64, 8), (1000, 512, 512, 32)])
def test_side_scores_are_bit_exact_and_indices_equal_the_oracle(tokens, side, key_dim, top_k):
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(tokens + side)
    half = key_dim // 2
    q = rng.standard_normal((tokens, key_dim)).astype(np.float32)
    kl = (rng.standard_normal((side, half)) / np.sqrt(half)).astype(np.float32)
    kr = (rng.standard_normal((side, half)) / np.sqrt(half)).astype(np.float32)
    ls, rs = cuda.product_key_side_scores(c, dev(q), dev(kl), dev(kr))
    want_l, want_r = ho.side_scores_f32(q[:, :half], kl), ho.side_scores_f32(q[:, half:], kr)
    assert np.array_equal(host(ls).astype(np.float32).view(np.uint32), want_l.view(np.uint32))
    assert np.array_equal(host(rs).astype(np.float32).view(np.uint32), want_r.view(np.uint32))
    beam = ho.product_key_beam(side, top_k)
    idx = cuda.product_key_topk_from_side_scores(c, ls, rs, top_k, beam)
    assert np.array_equal(host(idx), ho.product_key_indices_from_side_scores(want_l, want_r, top_k, beam))
    # quantised scores: many exact ties on both sides and in the sums
    ql = np.round(want_l * 4) / 4
    qr = np.round(want_r * 4) / 4
    idx = cuda.product_key_topk_from_side_scores(c, dev(ql), dev(qr), top_k, beam)
    assert np.array_equal(host(idx), ho.product_key_indices_from_side_scores(ql, qr, top_k, beam))


@pytest.mark.parametrize("tokens,side,top_k", [(64, 2048, 32), (33, 24, 16), (40, 512, 1), (17, 100, 9)])
def test_product_key_selection_on_degenerate_scores(tokens, side, top_k):
    """All-equal scores, signed zeros, a handful of distinct values, -inf entries: the selection must still
    follow (descending score, ascending index) and (descending sum, ascending slot)."""
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(side * 7 + top_k)
    beam = ho.product_key_beam(side, top_k)
    cases = []
    zeros = np.zeros((tokens, side), np.float32)
    cases.append((zeros, zeros))
    signed = np.where(rng.random((tokens, side)) < 0.5, np.float32(0.0), np.float32(-0.0)).astype(np.float32)
    cases.append((signed, signed[::-1].copy()))
    few_l = rng.integers(-2, 3, (tokens, side)).astype(np.float32)
    few_r = rng.integers(-2, 3, (tokens, side)).astype(np.float32)
    cases.append((few_l, few_r))
    holes = rng.standard_normal((tokens, side)).astype(np.float32)
    holes[rng.random((tokens, side)) < 0.3] = -np.inf
    cases.append((holes, rng.standard_normal((tokens, side)).astype(np.float32) * 1e-3))
    wide = (rng.standard_normal((tokens, side)) * 10.0 ** rng.integers(-30, 30, (tokens, side))).astype(np.float32)
    cases.append((wide, -wide))
    for left, right in cases:
        idx = cuda.product_key_topk_from_side_scores(c, dev(left), dev(right), top_k, beam)
        assert np.array_equal(host(idx), ho.product_key_indices_from_side_scores(left, right, top_k, beam))


def test_memory_layer_forward_backward_random():
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(3)
    tokens, side, key_dim, top_k, dim = 200, 32, 64, 8, 64
    q = rng.standard_normal((tokens, key_dim)).astype(np.float32)
    kl = rng.standard_normal((side, key_dim // 2)).astype(np.float32) * 0.2
    kr = rng.standard_normal((side, key_dim // 2)).astype(np.float32) * 0.2
    vals = rng.standard_normal((side * side, dim)).astype(np.float32)
    idx = rng.integers(0, side * side, (tokens, top_k))
    idx[:, 1] = idx[:, 0]  # repeated rows inside one token
    di = dev(idx, I64)
    s = cuda.memory_selected_scores_forward(c, di, dev(q), dev(kl), dev(kr))
    so = ho.product_key_selected_scores(idx, q, kl, kr)
    assert_close("scores", host(s), so, atol=1e-6, rtol=1e-6)
    w = cuda.softmax_rows(c, s)
    wo = ho.softmax(so, 1)
    assert_close("weights", host(w), wo, atol=1e-7, rtol=1e-5)
    out = cuda.memory_weighted_value_forward(c, di, w, dev(vals))
    assert_close("weighted", host(out), ho.memory_weighted_value(idx, wo, vals), atol=1e-5, rtol=1e-5)
    go = rng.standard_normal((tokens, dim)).astype(np.float32)
    dw, dv = cuda.memory_weighted_value_backward(c, di, w, dev(vals), dev(go))
    dwo, dvo = ho.memory_weighted_value_backward(idx, wo, vals, go)
    assert_close("dw", host(dw), dwo, atol=1e-5, rtol=1e-5)
    assert_close("dv", host(dv), dvo, atol=1e-4, rtol=1e-4)
    ds = cuda.softmax_rows_backward(c, w, dw)
    dso = ho.softmax_backward(wo, dwo, 1)
    assert_close("dscores", host(ds), dso, atol=1e-5, rtol=1e-4)
    dq, dl, dr = cuda.memory_selected_scores_backward(c, di, dev(q), dev(kl), dev(kr), ds)
    dqo, dlo, dro = ho.product_key_selected_scores_backward(idx, q, kl, kr, dso)
    assert_close("dq", host(dq), dqo, atol=1e-5, rtol=1e-4)
    assert_close("dleft", host(dl), dlo, atol=1e-4, rtol=1e-4)
    assert_close("dright", host(dr), dro, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("key", ["sparse_adamw_unique_rows", "sparse_adamw_row_mask"])
def test_sparse_adamw_known_answers(golden, key):
    from heirloom_b200 import cuda
    c = ctx()
    ka = golden["known_answers"][key]
    # rows of 2 padded to 4 columns so the same data also exercises vector-friendly shapes
    p = dev(ka["param"]); g = dev(ka["grad"])
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    mask = dev(np.asarray(ka["row_mask"], np.uint8), torch.uint8) if "row_mask" in ka else None
    hp = cuda.adamw_params(ka["lr"], 0.9, 0.999, 1e-8, ka["weight_decay"], 1.0, 1)
    cuda.sparse_adamw_rows(c, p, g, m, v, dev(ka["selected_rows"], I64), hp, row_mask=mask)
    assert_close(key, host(p), ka["expected"], atol=ka["tolerance"])


def test_sparse_adamw_updates_each_selected_row_once_and_only_those():
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(9)
    rows, dim = 1000, 48
    p0 = rng.standard_normal((rows, dim)).astype(np.float32)
    g0 = rng.standard_normal((rows, dim)).astype(np.float32)
    sel = rng.integers(0, rows, 3000)
    sel[:50] = 7
    p, g = dev(p0), dev(g0)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    hp = cuda.adamw_params(1e-2, 0.9, 0.999, 1e-8, 0.01, 1.0, 1)
    cuda.sparse_adamw_rows(c, p, g, m, v, dev(sel, I64), hp, zero_grad_rows=True)
    want, wm, wv = ho.adamw_step_f32_kernel_order(p0, g0, np.zeros_like(p0), np.zeros_like(p0), 1e-2, 0.9, 0.999, 1e-8,
                                                  0.01, 1.0, np.float32(1 - 0.9), np.float32(1 - 0.999))
    touched = np.zeros(rows, bool); touched[sel] = True
    got = host(p)
    assert np.array_equal(got[touched], want[touched].astype(np.float64))
    assert np.array_equal(got[~touched], p0[~touched].astype(np.float64))
    assert np.all(host(g)[touched] == 0) and np.array_equal(host(g)[~touched], g0[~touched].astype(np.float64))
    assert np.all(host(m)[~touched] == 0)


def test_bad_memory_index_sets_status():
    from heirloom_b200 import cuda
    from heirloom_b200._lib import HeirloomError
    c = ctx()
    vals = dev(np.zeros((4, 8), np.float32))
    cuda.memory_weighted_value_forward(c, dev([[0, 9]], I64), dev([[0.5, 0.5]]), vals)
    with pytest.raises(HeirloomError, match="out-of-range"):
        c.sync()


def test_row_masks_compaction_and_packed_rows():
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(31)
    rows, dim = 5000, 24
    selected = rng.integers(0, rows, 700)
    selected[:50] = selected[50:100]  # duplicates
    mask_in = (rng.random(rows) < 0.7).astype(np.uint8)
    sel = torch.tensor(selected, device="cuda")
    flags = cuda.mark_rows(c, sel, rows)
    want = np.zeros(rows, np.uint8); want[selected] = 1
    assert np.array_equal(host(flags), want)
    flags_m = cuda.mark_rows(c, sel, rows, row_mask=torch.tensor(mask_in, device="cuda"))
    assert np.array_equal(host(flags_m), want & mask_in)
    idx = cuda.mask_to_indices(c, flags)
    assert np.array_equal(host(idx), np.flatnonzero(want))  # ascending, each row once
    assert cuda.mask_to_indices(c, torch.zeros(rows, dtype=torch.uint8, device="cuda")).numel() == 0
    table = rng.standard_normal((rows, dim)).astype(np.float32)
    t = torch.tensor(table, device="cuda")
    packed = cuda.gather_rows(c, t, idx)
    assert np.array_equal(host(packed), table[np.flatnonzero(want)])
    dst = torch.zeros(rows, dim, device="cuda")
    cuda.scatter_rows(c, packed * 2.0, idx, dst)
    c.sync()
    expect = np.zeros_like(table); expect[np.flatnonzero(want)] = 2.0 * table[np.flatnonzero(want)]
    assert np.array_equal(host(dst), expect)
    # clip norm over the active rows only: a set, filtered by the mask
    got = cuda.sparse_rows_sum_squares(c, t, sel, row_mask=torch.tensor(mask_in, device="cuda"))
    active = np.flatnonzero(want & mask_in)
    assert got == pytest.approx(float((table[active].astype(np.float64) ** 2).sum()), rel=1e-12)


@pytest.mark.parametrize("tokens,top_k,rows,dim", [(4096, 16, 1024, 256), (2048, 32, 300, 512), (4100, 8, 70000, 64),
                                                   (1030, 32, 4096, 640)])
def test_weighted_value_backward_in_row_order_matches_a_host_sum(tokens, top_k, rows, dim):
    """Event counts from 32768 up take the row-ordered path (sort by row, one set of atomics per run): many events per
    row, rows nobody selected, chunk boundaries inside a run, a row count that is not a power of two."""
    from heirloom_b200 import cuda
    c = ctx()
    rng = np.random.default_rng(tokens + rows)
    idx = (rng.zipf(1.3, (tokens, top_k)) % rows).astype(np.int64)
    idx[0, :] = rows - 1                      # the last row, a whole token's worth
    w = rng.standard_normal((tokens, top_k)).astype(np.float32)
    vals = rng.standard_normal((rows, dim)).astype(np.float32)
    go = rng.standard_normal((tokens, dim)).astype(np.float32)
    dw, dv = cuda.memory_weighted_value_backward(c, dev(idx, I64), dev(w), dev(vals), dev(go))
    want_dw = np.einsum("td,tkd->tk", go.astype(np.float64), vals[idx].astype(np.float64))
    want_dv = np.zeros((rows, dim), np.float64)
    np.add.at(want_dv, idx.reshape(-1), (w[..., None].astype(np.float64) * go[:, None, :]).reshape(-1, dim))
    assert_close("dw", host(dw), want_dw, atol=1e-5, rtol=1e-6)
    scale = np.abs(want_dv).max()
    assert np.abs(host(dv) - want_dv).max() <= 2e-6 * scale * np.sqrt(tokens * top_k / max(np.unique(idx).size, 1)) + 1e-5
    untouched = np.ones(rows, bool); untouched[np.unique(idx)] = False
    assert not np.any(host(dv)[untouched])


def test_row_ordered_value_backward_reports_a_bad_index_and_zeroes_its_weight_gradient():
    """An index past the table in the row-ordered path: the event is left out of the row sums, its weight gradient is
    written as zero (not left as stale scratch), and the next sync reports the status word; nothing faults."""
    from heirloom_b200 import cuda
    from heirloom_b200._lib import HeirloomError
    c = ctx()
    rng = np.random.default_rng(77)
    tokens, top_k, rows, dim = 2048, 32, 500, 64
    idx = rng.integers(0, rows, (tokens, top_k)).astype(np.int64)
    idx[5, 3], idx[100, 0] = rows, -1
    w = rng.standard_normal((tokens, top_k)).astype(np.float32)
    vals = rng.standard_normal((rows, dim)).astype(np.float32)
    go = rng.standard_normal((tokens, dim)).astype(np.float32)
    c.sync()
    dw, dv = cuda.memory_weighted_value_backward(c, dev(idx, I64), dev(w), dev(vals), dev(go))
    with pytest.raises(HeirloomError, match="out-of-range index"):
        c.sync()
    c.sync()
    got = dw.cpu().numpy()
    assert got[5, 3] == 0.0 and got[100, 0] == 0.0
    good = np.ones_like(idx, bool); good[5, 3] = good[100, 0] = False
    want_dw = np.einsum("td,tkd->tk", go.astype(np.float64), vals[np.clip(idx, 0, rows - 1)].astype(np.float64))
    assert np.allclose(got[good], want_dw[good], rtol=1e-5, atol=1e-5)

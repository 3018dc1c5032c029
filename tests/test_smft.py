"""SMFT bookkeeping: access counts, TF-IDF row masks, the product-key projection, masked sparse-row AdamW.
CPU tests replay the reference's own scenarios (tests/memory_transformer.rs:327-368, :387-437, :451-500,
:1356-1374); GPU tests count on the device and run the masked step of the memory transformer."""
import math

import numpy as np
import pytest

from heirloom_b200._lib import HeirloomError
from heirloom_b200.smft import MemoryAccessCounts, SmftRowMask, sort_smft_scores, SmftRowScore
from oracle import heirloom_oracle as ho


def test_access_counts_rank_foreground_rows_against_background():
    fg = MemoryAccessCounts.from_rows(6, [1, 1, 2, 4, 4, 4])
    bg = MemoryAccessCounts.from_rows(6, [1, 2, 2, 2, 3, 4])
    assert fg.total_events == 6 and fg.unique_rows == 3
    assert fg.row_counts.tolist() == [0, 2, 1, 0, 3, 0]
    fg.validate()
    same = MemoryAccessCounts.from_row_counts(6, [0, 2, 1, 0, 3, 0])
    assert same.total_events == fg.total_events and same.unique_rows == fg.unique_rows
    assert same.row_counts.tolist() == fg.row_counts.tolist()
    merged = MemoryAccessCounts.empty(6)
    merged.merge_in(fg)
    merged.merge_in(bg)
    assert merged.total_events == 12 and merged.row_counts.tolist() == [0, 3, 4, 1, 4, 0]
    broken = MemoryAccessCounts(6, fg.total_events + 1, fg.unique_rows, fg.row_counts.copy())
    with pytest.raises(HeirloomError, match="total_events"):
        broken.validate()
    mask = fg.smft_mask_against(bg, 0.5, 1)
    assert mask.trainable_rows == [4, 1]
    assert mask.frozen_rows == 4
    assert (mask.scores[0].row, mask.scores[0].foreground_count, mask.scores[0].background_count) == (4, 3, 1)
    assert mask.scores[0].score > mask.scores[1].score
    with pytest.raises(HeirloomError, match="memory_slots mismatch"):
        fg.smft_mask_against(MemoryAccessCounts.empty(7), 0.5, 1)
    with pytest.raises(HeirloomError, match="out of range"):
        MemoryAccessCounts.from_rows(6, [6])
    with pytest.raises(HeirloomError, match="trainable_fraction"):
        fg.smft_mask_against(bg, 1.5, 1)


def test_mask_scores_match_the_oracle_on_random_counts():
    rng = np.random.default_rng(5)
    for slots, events in ((16, 40), (256, 3000), (1024, 500)):
        fg_rows = rng.zipf(1.3, events) % slots
        bg_rows = rng.integers(0, slots, events * 2)
        fg, bg = MemoryAccessCounts.from_rows(slots, fg_rows), MemoryAccessCounts.from_rows(slots, bg_rows)
        for fraction, min_rows in ((0.0, 0), (0.0, 3), (0.25, 1), (1.0, 0)):
            mask = fg.smft_mask_against(bg, fraction, min_rows)
            want_rows, want_scores = ho.smft_mask_against(fg.row_counts, bg.row_counts, fraction, min_rows)
            assert mask.trainable_rows == want_rows
            assert [s.row for s in mask.scores] == [r for r, _ in want_scores]
            assert np.allclose([s.score for s in mask.scores], [v for _, v in want_scores], rtol=1e-15, atol=0)
            assert mask.frozen_rows == slots - len(want_rows)
            mask.validate()


def test_score_order_breaks_ties_like_the_reference():
    rows = [SmftRowScore(5, 2, 1, 0.5), SmftRowScore(3, 2, 0, 0.5), SmftRowScore(1, 3, 9, 0.5), SmftRowScore(0, 2, 0, 0.5),
            SmftRowScore(7, 1, 0, 0.75)]
    sort_smft_scores(rows)
    assert [r.row for r in rows] == [7, 1, 0, 3, 5]


def test_row_mask_materialises_and_validates():
    mask = SmftRowMask(4, [1, 3], 2, 0.5)
    assert mask.to_mask().tolist() == [0, 1, 0, 1]
    with pytest.raises(HeirloomError, match="out of range"):
        SmftRowMask(4, [4], 2, 0.5).to_mask()
    with pytest.raises(HeirloomError, match="appears more than once"):
        SmftRowMask(4, [1, 1], 2, 0.5).to_mask()
    with pytest.raises(HeirloomError, match="does not match"):
        SmftRowMask(4, [1, 3], 99, 0.5).to_mask()


def test_product_key_projection_is_conservative():
    projection = SmftRowMask(4, [0, 1], 2, 0.5).product_key_projection()
    assert projection.side == 2
    assert projection.left_trainable_rows == [0] and projection.right_trainable_rows == []
    assert projection.left_mask().tolist() == [1, 0] and projection.right_mask().tolist() == [0, 0]
    full = SmftRowMask(9, list(range(9)), 0, 1.0).product_key_projection()
    assert full.left_trainable_rows == [0, 1, 2] and full.right_trainable_rows == [0, 1, 2]
    column = SmftRowMask(9, [1, 4, 7], 6, 0.3).product_key_projection()
    assert column.left_trainable_rows == [] and column.right_trainable_rows == [1]
    with pytest.raises(HeirloomError, match="square memory_slots"):
        SmftRowMask(12, [0], 11, 0.5).product_key_projection()


def test_oracle_masked_sparse_adamw_known_answer():
    # the reference's cpu_sparse_adamw_rows_respects_smft_row_mask
    p = np.array([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    g = np.array([[1.0, -2.0], [3.0, -4.0], [0.5, -0.25]])
    state = ho.AdamWState(lr=0.1, weight_decay=0.0)
    got = ho.adamw_sparse_rows_step(p, g, np.zeros_like(p), np.zeros_like(p), [2, 0, 1, 2], state,
                                    row_mask=[False, True, True])
    assert np.allclose(got.reshape(-1), [1.0, 2.0, 2.9, 4.1, 4.9, 6.1], atol=1e-4)


# ------------------------------------------------------------------------------------------------ GPU
gpu = pytest.mark.gpu


@gpu
def test_device_access_counts_equal_a_host_histogram():
    import torch
    from heirloom_b200 import cuda
    from tests.gpu_util import ctx
    c = ctx()
    rng = np.random.default_rng(9)
    for slots, n in ((12, 24), (4096, 100_000), (262_144, 1_048_576)):
        rows = (rng.zipf(1.2, n) % slots).astype(np.int64)
        counts = cuda.memory_access_count_rows(c, torch.tensor(rows, device="cuda"), slots)
        want = np.bincount(rows, minlength=slots)
        assert np.array_equal(counts.cpu().numpy(), want)
        again = cuda.memory_access_count_rows(c, torch.tensor(rows[: n // 2], device="cuda"), slots, counts)
        assert np.array_equal(again.cpu().numpy(), want + np.bincount(rows[: n // 2], minlength=slots))
    with pytest.raises(HeirloomError):
        cuda.memory_access_count_rows(c, torch.tensor([0, 12], device="cuda"), 12)
    with pytest.raises(HeirloomError, match="non-zero memory_slots"):
        cuda.memory_access_count_rows(c, torch.tensor([0], device="cuda"), 0)


@gpu
def test_masked_sparse_adamw_rows_known_answer():
    # the reference's cuda_sparse_adamw_rows_respects_smft_row_mask (tests/memory_transformer.rs:1325-1353)
    import torch
    from heirloom_b200 import cuda
    from tests.gpu_util import ctx
    c = ctx()
    p = torch.tensor([[1.0, 2.0, 0, 0], [3.0, 4.0, 0, 0], [5.0, 6.0, 0, 0]], device="cuda")
    g = torch.tensor([[1.0, -2.0, 0, 0], [3.0, -4.0, 0, 0], [0.5, -0.25, 0, 0]], device="cuda")
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    rows = torch.tensor([2, 0, 1, 2], device="cuda")
    mask = torch.tensor([0, 1, 1], dtype=torch.uint8, device="cuda")
    hp = cuda.adamw_params(0.1, 0.9, 0.999, 1e-8, 0.0, 1.0, 1)
    cuda.sparse_adamw_rows(c, p, g, m, v, rows, hp, row_mask=mask)
    assert np.allclose(p.cpu().numpy()[:, :2].reshape(-1), [1.0, 2.0, 2.9, 4.1, 4.9, 6.1], atol=1e-4)


@gpu
def test_model_counts_report_and_masked_sparse_step():
    import torch
    from heirloom_b200 import nn
    from tests.test_gpu_memory_decoder import MEM, build
    model, ocfg, omem, params = build(nn.PRECISION_F32, 2, seed=3)
    model.set_optimizer(lr=1e-2, weight_decay=0.01)
    rng = np.random.default_rng(13)
    tok = ho.zipf_tokens(rng, ocfg.vocab, (2, 129))
    x, y = tok[:, :-1].copy(), tok[:, 1:].copy()
    model.forward_backward(torch.tensor(x, device="cuda"), torch.tensor(y, device="cuda"))
    _, ograds, oidx = ho.memory_decoder_loss_and_grads(ocfg, omem, params, x, y, return_indices=True)
    selected = np.concatenate([oidx[l].reshape(-1) for l in MEM["memory_layers"]])
    slots = MEM["slots"]
    side = int(math.isqrt(slots))

    counts = model.memory_access_counts()
    assert counts.total_events == selected.size
    assert np.array_equal(counts.row_counts, np.bincount(selected, minlength=slots).astype(np.uint64))
    report = model.smft_access_report(4)
    assert 0 < len(report.top_rows) <= 4 and report.top_rows[0].foreground_count == counts.row_counts.max()

    background = MemoryAccessCounts.from_rows(slots, rng.integers(0, slots, 4000))
    mask = model.smft_row_mask_against(background, 0.5, 1)
    want_rows, _ = ho.smft_mask_against(counts.row_counts, background.row_counts, 0.5, 1)
    assert mask.trainable_rows == want_rows and 0 < len(want_rows) < counts.unique_rows
    # make one whole left row and one whole right column trainable, so that the projection is not empty
    li, ri = int(selected[0] // side), int(selected[0] % side)
    rows = sorted(set(mask.trainable_rows) | {li * side + r for r in range(side)} | {l * side + ri for l in range(side)})
    mask = SmftRowMask(slots, rows, slots - len(rows), 0.5)
    projection = mask.product_key_projection()
    assert li in projection.left_trainable_rows and ri in projection.right_trainable_rows
    model.set_smft_mask(mask)
    model.optimizer_step_sparse_rows()

    state = ho.AdamWState(lr=1e-2, weight_decay=0.01)
    tables = (("shared_memory.product_key_left", selected // side, projection.left_mask()),
              ("shared_memory.product_key_right", selected % side, projection.right_mask()),
              ("shared_memory.value", selected, mask.to_mask()))
    for name, sel, row_mask in tables:
        state.step = 0
        p = params[name]
        want = ho.adamw_sparse_rows_step(p, ograds[name], np.zeros_like(p), np.zeros_like(p), sel, state,
                                         row_mask=row_mask.astype(bool))
        got = model.parameter(name).astype(np.float64)
        active = np.zeros(p.shape[0], bool); active[sel] = True
        active &= row_mask.astype(bool)
        assert active.any()
        assert np.array_equal(got[~active], p[~active])            # masked-out and unselected rows keep their bits
        assert np.abs(got[active] - want[active]).max() <= 2e-4
        assert np.abs(got[active] - p[active]).max() > 1e-3
    # lifting the mask gives the unmasked policy back
    model.set_smft_mask(None)
    model.forward_backward(torch.tensor(x, device="cuda"), torch.tensor(y, device="cuda"))
    before = model.parameter("shared_memory.value").copy()
    model.optimizer_step_sparse_rows()
    moved = np.abs(model.parameter("shared_memory.value") - before).max(axis=1) > 0
    assert moved.sum() == np.unique(model_selected(model, MEM)).size
    with pytest.raises(HeirloomError, match="does not match model memory_slots"):
        model.set_smft_mask(SmftRowMask(slots * 4, [0], slots * 4 - 1, 0.5))
    model.close()


def model_selected(model, mem):
    return np.concatenate([model.selected_indices(l).reshape(-1) for l in mem["memory_layers"]])

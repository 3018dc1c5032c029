"""Step-level parity of the memory transformer (product-key memory feed-forward blocks)."""
import numpy as np
import pytest
import torch

from oracle import heirloom_oracle as ho
from tests.gpu_util import ctx

pytestmark = pytest.mark.gpu

KW = dict(vocab=512, d_model=128, n_layers=3, n_heads=2, d_ff=256, context=128)
MEM = dict(memory_layers=(1, 2), slots=1024, key_dim=64, value_dim=64, top_k=8)


def build(precision, batch, seed=0):
    from heirloom_b200 import nn
    c = ctx()
    model = nn.DecoderLm(c, nn.DecoderConfig(batch=batch, precision=precision, **KW), nn.MemoryConfig(**MEM))
    ocfg, omem = ho.DecoderConfig(**KW), ho.MemoryConfig(**MEM)
    params = ho.init_memory_parameters(ocfg, omem, seed)
    model.load_state_dict(params)
    return model, ocfg, omem, params


def test_parameter_names_and_shapes_follow_the_reference_state_dict():
    from heirloom_b200 import nn
    model, ocfg, omem, _ = build(nn.PRECISION_F32, 1)
    assert model.parameter_names() == ho.memory_parameter_names(ocfg, omem)
    assert model.parameter_shapes() == ho.memory_parameter_shapes(ocfg, omem)
    model.close()


def test_f32_route_matches_the_oracle_with_identical_indices():
    from heirloom_b200 import nn
    model, ocfg, omem, params = build(nn.PRECISION_F32, 2)
    rng = np.random.default_rng(11)
    tok = ho.zipf_tokens(rng, ocfg.vocab, (2, 129))
    x, y = tok[:, :-1].copy(), tok[:, 1:].copy()
    model.forward_backward(torch.tensor(x, device="cuda"), torch.tensor(y, device="cuda"))
    oloss, ograds, oidx = ho.memory_decoder_loss_and_grads(ocfg, omem, params, x, y, return_indices=True)
    assert abs(model.loss() - oloss) <= 1e-6 * abs(oloss)
    for layer in MEM["memory_layers"]:
        assert np.array_equal(model.selected_indices(layer), oidx[layer]), layer   # bit-exact top-k routing
    for name in ho.memory_parameter_names(ocfg, omem):
        if name.endswith("attention.k_proj.bias"):
            continue
        g, w = model.grad(name).astype(np.float64), ograds[name]
        scale = np.abs(w).max() + 1e-30
        assert np.abs(g - w).max() <= 5e-6 * scale + 1e-10, (name, np.abs(g - w).max(), scale)
    model.close()


def _slot_scores(q, kl, kr, slots, side):
    """Full product-key score of each slot in `slots` [tokens, k] for the queries q [tokens, key_dim] (f64)."""
    half = q.shape[1] // 2
    left, right = slots // side, slots % side
    return np.einsum("tkd,td->tk", kl[left], q[:, :half]) + np.einsum("tkd,td->tk", kr[right], q[:, half:])


def test_amp_route_tracks_the_oracle_and_routes_almost_identically():
    from heirloom_b200 import nn
    model, ocfg, omem, params = build(nn.PRECISION_AMP_BF16, 2, seed=1)
    model.set_optimizer(lr=1e-3, weight_decay=0.01)
    state = ho.AdamWState(lr=1e-3, weight_decay=0.01)
    rng = np.random.default_rng(12)
    side = int(np.sqrt(MEM["slots"]))
    agree, gaps = [], []
    for step in range(5):
        tok = ho.zipf_tokens(rng, ocfg.vocab, (2, 129))
        x, y = tok[:, :-1].copy(), tok[:, 1:].copy()
        loss = model.train_step(torch.tensor(x).pin_memory(), torch.tensor(y).pin_memory())
        oloss, ograds, oidx, oq = ho.memory_decoder_loss_and_grads(ocfg, omem, params, x, y, amp_bf16=True, return_indices=True,
                                                                   return_queries=True)
        assert abs(loss - oloss) <= 1e-2 * abs(oloss), (step, loss, oloss)
        for layer in MEM["memory_layers"]:
            got = model.selected_indices(layer)
            agree.append(np.mean([len(set(a) & set(b)) / len(a) for a, b in zip(got, oidx[layer])]))
            # every slot that differs must be a near-tie under the oracle's own queries: its score lies within the
            # bf16 noise of the block input (the layer norm output both sides round to bf16) below the oracle's k-th
            q = oq[layer].astype(np.float64)
            kl, kr = params["shared_memory.product_key_left"], params["shared_memory.product_key_right"]
            s_ref, s_got = _slot_scores(q, kl, kr, oidx[layer], side), _slot_scores(q, kl, kr, got, side)
            spread = s_ref.max(axis=1) - s_ref.min(axis=1) + 1e-30
            gaps.append(float(np.max((s_ref.min(axis=1) - s_got.min(axis=1)) / spread)))
        ho.adamw_step(params, ograds, state)
    print("amp memory routing agreement per (step, block):", [round(a, 4) for a in agree])
    print("amp memory worst score gap of a differing slot, relative to the selected scores' spread:", max(gaps))
    # the three projections run at f32 accuracy forward and backward (bf16 pieces of their f32 operands in one f32
    # accumulation), as the reference keeps them in f32; what is left are slots whose scores tie within the bf16
    # rounding of the block input (the layer norm output, which the attention before it reaches through bf16 products
    # summed in another order)
    assert min(agree) >= 0.97, agree
    assert max(gaps) <= 0.08, gaps
    floor = 5 * 1e-3
    report, measured = {}, {}
    for name in ho.memory_parameter_names(ocfg, omem):
        if name.endswith("attention.k_proj.bias"):
            continue
        got, want = model.parameter(name).astype(np.float64), params[name]
        bad = np.abs(got - want) > 2e-2 * np.maximum(np.abs(want), floor)
        # Small vectors that start at zero (biases) move by about lr per step whatever the gradient's
        # size, so a handful of sign flips already is several per cent of their elements.
        # The shared tables are where the last routing differences show: a slot chosen on one side only gives its
        # value row and half-key rows a gradient there and plain decay here, and AdamW turns any gradient into a step
        # of about lr; with 1 % of the slots differing, 0.2 % of the table elements end outside the gate.
        # The memory projections' gradients are 1e-5 of the dense ones at this initialisation (the looked-up values are
        # small) and every token with one differing slot moves them by several per cent of their scale: measured 8-19 %
        # of the tensor scale at the worst element, 1-2 % on average, with the projections themselves f32-accurate.
        cls = ("tables" if name.startswith("shared_memory") else "memory projections" if "memory" in name
               else "large" if got.size >= 1024 else "small")
        measured[cls] = max(measured.get(cls, 0.0), float(bad.mean()))
        limit = {"tables": 0.03, "memory projections": 0.25, "large": 0.01, "small": 0.07}[cls]
        if bad.mean() > limit:
            report[name] = float(bad.mean())
    print("amp memory model, worst fraction of elements outside 2e-2 after 5 steps, by class:", measured)
    assert not report, report
    model.close()


def test_memory_configuration_errors_read_like_the_reference():
    from heirloom_b200 import nn
    from heirloom_b200._lib import HeirloomError
    c = ctx()
    cfg = nn.DecoderConfig(batch=1, precision=nn.PRECISION_F32, **KW)
    with pytest.raises(HeirloomError, match="supports one memory head"):
        nn.DecoderLm(c, cfg, nn.MemoryConfig(**{**MEM, "memory_heads": 4}))
    with pytest.raises(HeirloomError, match="square memory_slots"):
        nn.DecoderLm(c, cfg, nn.MemoryConfig(**{**MEM, "slots": 1000}))


def test_sparse_rows_policy_updates_only_the_selected_table_rows():
    from heirloom_b200 import nn
    model, ocfg, omem, params = build(nn.PRECISION_F32, 2, seed=3)
    model.set_optimizer(lr=1e-2, weight_decay=0.01)
    rng = np.random.default_rng(13)
    tok = ho.zipf_tokens(rng, ocfg.vocab, (2, 129))
    x, y = tok[:, :-1].copy(), tok[:, 1:].copy()
    model.forward_backward(torch.tensor(x, device="cuda"), torch.tensor(y, device="cuda"))
    _, ograds, oidx = ho.memory_decoder_loss_and_grads(ocfg, omem, params, x, y, return_indices=True)
    model.optimizer_step_sparse_rows()
    assert model.optimizer_steps == 1
    selected = np.concatenate([oidx[l].reshape(-1) for l in MEM["memory_layers"]])
    side = int(np.sqrt(MEM["slots"]))
    state = ho.AdamWState(lr=1e-2, weight_decay=0.01)
    for name, rows in (("shared_memory.product_key_left", selected // side), ("shared_memory.product_key_right", selected % side),
                       ("shared_memory.value", selected)):
        state.step = 0
        p = params[name]
        want = ho.adamw_sparse_rows_step(p, ograds[name], np.zeros_like(p), np.zeros_like(p), rows, state)
        got = model.parameter(name).astype(np.float64)
        touched = np.zeros(p.shape[0], bool); touched[rows] = True
        assert np.array_equal(got[~touched], p[~touched])                 # untouched rows keep their bits
        assert np.abs(got[touched] - want[touched]).max() <= 2e-4         # CPU-vs-CUDA AdamW tolerance of the reference
        assert np.abs(got[touched] - p[touched]).max() > 1e-3             # and they did move
    for name in ("lm_head.weight", "block.1.feed_forward.memory.query_proj.weight", "token_embedding.weight"):
        assert np.array_equal(model.parameter(name).astype(np.float64), params[name])   # no dense update in this policy
    model.close()


def test_sparse_rows_policy_clips_by_the_norm_of_the_active_rows_only():
    from heirloom_b200 import nn
    model, ocfg, omem, params = build(nn.PRECISION_F32, 2, seed=3)
    rng = np.random.default_rng(13)
    tok = ho.zipf_tokens(rng, ocfg.vocab, (2, 129))
    x, y = tok[:, :-1].copy(), tok[:, 1:].copy()
    _, ograds, oidx = ho.memory_decoder_loss_and_grads(ocfg, omem, params, x, y, return_indices=True)
    selected = np.concatenate([oidx[l].reshape(-1) for l in MEM["memory_layers"]])
    side = int(np.sqrt(MEM["slots"]))
    tables = (("shared_memory.product_key_left", selected // side), ("shared_memory.product_key_right", selected % side),
              ("shared_memory.value", selected))
    full = ho.sparse_rows_clip_scale([(ograds[n], r, None) for n, r in tables], 1e9)
    assert full == 1.0
    norm = np.sqrt(sum(float((ograds[n][np.unique(r)] ** 2).sum()) for n, r in tables))
    clip_norm = 0.25 * norm  # well below the norm of the active rows, so the step is scaled by about 1/4
    scale = ho.sparse_rows_clip_scale([(ograds[n], r, None) for n, r in tables], clip_norm)
    assert scale == pytest.approx(0.25, rel=1e-6)
    model.set_optimizer(lr=1e-2, weight_decay=0.01, clip_norm=clip_norm)
    model.forward_backward(torch.tensor(x, device="cuda"), torch.tensor(y, device="cuda"))
    model.optimizer_step_sparse_rows()
    state = ho.AdamWState(lr=1e-2, weight_decay=0.01)
    for name, rows in tables:
        state.step = 0
        p = params[name]
        want = ho.adamw_sparse_rows_step(p, ograds[name], np.zeros_like(p), np.zeros_like(p), rows, state, clip=scale)
        unclipped = ho.adamw_sparse_rows_step(p, ograds[name], np.zeros_like(p), np.zeros_like(p), rows,
                                              ho.AdamWState(lr=1e-2, weight_decay=0.01))
        got = model.parameter(name).astype(np.float64)
        touched = np.zeros(p.shape[0], bool); touched[rows] = True
        assert np.array_equal(got[~touched], p[~touched])
        assert np.abs(got[touched] - want[touched]).max() <= 2e-4
    # the first Adam step is sign-like, so clipping shows in the moments rather than in the parameters
    m_got, _ = model.moments("shared_memory.value")
    rows = np.unique(selected)
    want_m = 0.1 * (ograds["shared_memory.value"][rows] * scale + 0.01 * params["shared_memory.value"][rows])
    assert np.abs(m_got[rows] - want_m).max() <= 1e-6 + 1e-3 * np.abs(want_m).max()
    model.close()


def test_memory_only_policy_updates_the_tables_and_nothing_else():
    """`MemoryOnly`: dense AdamW over the three tables, the clip norm taken over them alone
    (AdamW::step_parameter_indices_mut, src/nn.rs:2222-2254)."""
    from heirloom_b200 import nn
    model, ocfg, omem, params = build(nn.PRECISION_F32, 2, seed=3)
    rng = np.random.default_rng(13)
    tok = ho.zipf_tokens(rng, ocfg.vocab, (2, 129))
    x, y = tok[:, :-1].copy(), tok[:, 1:].copy()
    _, ograds, _ = ho.memory_decoder_loss_and_grads(ocfg, omem, params, x, y, return_indices=True)
    names = ("shared_memory.product_key_left", "shared_memory.product_key_right", "shared_memory.value")
    norm = np.sqrt(sum(float((ograds[n].astype(np.float64) ** 2).sum()) for n in names))
    clip_norm = 0.5 * norm
    scale = clip_norm / (norm + 1e-12)
    model.set_optimizer(lr=1e-2, weight_decay=0.01, clip_norm=clip_norm)
    model.forward_backward(torch.tensor(x, device="cuda"), torch.tensor(y, device="cuda"))
    model.optimizer_step_policy("memory_only")
    assert model.optimizer_steps == 1
    for name in names:
        p = params[name]
        state = ho.AdamWState(lr=1e-2, weight_decay=0.01)
        every_row = np.arange(p.shape[0])
        want = ho.adamw_sparse_rows_step(p, ograds[name], np.zeros_like(p), np.zeros_like(p), every_row, state, clip=scale)
        got = model.parameter(name).astype(np.float64)
        assert np.abs(got - want).max() <= 2e-4
        assert np.abs(got - p).max() > 1e-3
    for name in ("lm_head.weight", "block.1.feed_forward.memory.query_proj.weight", "token_embedding.weight", "ln_f.weight"):
        assert np.array_equal(model.parameter(name).astype(np.float64), params[name])
    model.optimizer_step_policy("frozen")
    assert model.optimizer_steps == 1
    from heirloom_b200._lib import HeirloomError
    with pytest.raises(HeirloomError, match="unknown memory update policy"):
        model.optimizer_step_policy("everything")
    model.close()


def test_dense_plus_sparse_values_policy():
    """Dense AdamW on all parameters but the value table, row-set AdamW on the selected value rows, one step count
    and one clip factor over the dense gradients plus the active value rows."""
    from heirloom_b200 import nn
    model, ocfg, omem, params = build(nn.PRECISION_F32, 2, seed=3)
    rng = np.random.default_rng(13)
    tok = ho.zipf_tokens(rng, ocfg.vocab, (2, 129))
    x, y = tok[:, :-1].copy(), tok[:, 1:].copy()
    _, ograds, oidx = ho.memory_decoder_loss_and_grads(ocfg, omem, params, x, y, return_indices=True)
    selected = np.unique(np.concatenate([oidx[l].reshape(-1) for l in MEM["memory_layers"]]))
    sum_sq = sum(float((g.astype(np.float64) ** 2).sum()) for n, g in ograds.items() if n != "shared_memory.value")
    sum_sq += float((ograds["shared_memory.value"][selected].astype(np.float64) ** 2).sum())
    norm = np.sqrt(sum_sq)
    clip_norm = 0.5 * norm
    scale = clip_norm / (norm + 1e-12)
    model.set_optimizer(lr=1e-2, weight_decay=0.01, clip_norm=clip_norm)
    model.forward_backward(torch.tensor(x, device="cuda"), torch.tensor(y, device="cuda"))
    model.optimizer_step_policy("dense_plus_sparse_values")
    assert model.optimizer_steps == 1
    for name, p in params.items():
        state = ho.AdamWState(lr=1e-2, weight_decay=0.01)
        rows = selected if name == "shared_memory.value" else np.arange(p.shape[0])
        p2 = p.reshape(p.shape[0], -1)
        g2 = ograds[name].reshape(p2.shape)
        want = ho.adamw_sparse_rows_step(p2, g2, np.zeros_like(p2), np.zeros_like(p2), rows, state, clip=scale)
        got = model.parameter(name).astype(np.float64).reshape(p2.shape)
        active = np.zeros(p2.shape[0], bool); active[rows] = True
        assert np.array_equal(got[~active], p2[~active]), name
        assert np.abs(got[active] - want[active]).max() <= 2e-4, name
    model.close()

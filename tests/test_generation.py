"""Sampling controls, the RNG stream, evaluation and generation (reference: src/nn.rs:1595-1751,
src/rng.rs:29-45, src/memory_transformer.rs:1730-1984, tests/transformer_runtime.rs:1530-1575)."""
import math

import numpy as np
import pytest

from heirloom_b200 import generation as gen
from oracle import heirloom_oracle as ho


def test_rng_stream_is_splitmix64_and_uniforms_have_24_bits():
    rng = gen.HeirloomRng(0)
    # SplitMix64 from state 0: published first outputs of the generator
    assert [rng.next_u64() for _ in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    a, b = gen.HeirloomRng(123), gen.HeirloomRng(123)
    ua = [a.uniform_f32() for _ in range(8)]
    assert ua == [b.uniform_f32() for _ in range(8)] and all(0.0 <= u < 1.0 for u in ua)
    assert all(u * (1 << 24) == int(u * (1 << 24)) for u in ua)
    assert a.state == b.state and a.state != 123


def test_greedy_and_filters_follow_the_reference_rules():
    o = gen.GenerationOptions.greedy(4, 2)
    logits = [0.1, 2.0, 2.0, -1.0]
    t, p, lp = gen.sample_token(logits, [], o, gen.HeirloomRng(0))
    assert t == 2  # max_by keeps the last of equal maxima
    assert p == pytest.approx(math.exp(2.0) / (2 * math.exp(2.0) + math.exp(0.1) + math.exp(-1.0))) and lp == pytest.approx(math.log(p))
    # top_k = 1 at temperature 1 is greedy whatever the draw (tests/transformer_runtime.rs:1546-1562)
    o1 = gen.GenerationOptions(4, 2, temperature=1.0, top_k=1, top_p=1.0)
    assert gen.sample_token([0.1, 2.5, 2.0, -1.0], [], o1, gen.HeirloomRng(123))[0] == 1
    # top_p keeps the smallest prefix of the ranked distribution that reaches the mass
    keep = gen.sampling_filter(np.log(np.array([0.5, 0.3, 0.15, 0.05])), gen.GenerationOptions(1, 0, temperature=1.0, top_p=0.75))
    assert keep.tolist() == [True, True, False, False]
    keep = gen.sampling_filter(np.array([1.0, 3.0, 2.0, 0.0]), gen.GenerationOptions(1, 0, temperature=1.0, top_k=2))
    assert keep.tolist() == [False, True, True, False]
    # repetition controls: positive logits divided, negative multiplied, then frequency and presence
    o2 = gen.GenerationOptions(1, 0, repetition_penalty=2.0, frequency_penalty=0.5, presence_penalty=0.25)
    adj = np.array([2.0, -2.0, 1.0])
    gen._apply_repetition_controls(adj, [0, 0, 1, 7], o2)
    assert adj.tolist() == [2.0 / 2 - 0.5 * 2 - 0.25, -2.0 * 2 - 0.5 - 0.25, 1.0]
    # all-filtered input falls back to one-hot on index 0
    assert gen.softmax_logits(np.array([-np.inf, -np.inf])).tolist() == [1.0, 0.0]
    # sampling walks the cumulative distribution with one 24-bit uniform draw
    rng = gen.HeirloomRng(5)
    draw = gen.HeirloomRng(5).uniform_f32()
    probs = np.array([0.2, 0.5, 0.3])
    want = int(np.searchsorted(np.cumsum(probs), draw, side="left"))
    assert gen.sample_token(np.log(probs), [], gen.GenerationOptions(1, 9, temperature=1.0), rng)[0] == want


def test_option_validation_messages():
    for kwargs, text in ((dict(temperature=-1.0), "temperature must be non-negative"), (dict(top_k=0), "top_k must be greater than zero"),
                         (dict(top_p=0.0), "top_p must be in"), (dict(repetition_penalty=0.5), "at least 1.0"),
                         (dict(presence_penalty=-0.1), "must be non-negative")):
        with pytest.raises(Exception, match=text):
            gen.GenerationOptions(1, 0, **kwargs).validate()


@pytest.mark.gpu
def test_logits_eval_and_generation_on_the_device_match_the_oracle():
    import torch

    from heirloom_b200 import nn
    from tests.gpu_util import ctx
    c = ctx()
    kw = dict(vocab=64, d_model=64, n_layers=2, n_heads=1, d_ff=128, context=16)
    ocfg = ho.DecoderConfig(**kw)
    params = ho.init_parameters(ocfg, 4)
    rng = np.random.default_rng(2)
    for n in params:  # larger weights so that the argmax chain is not a string of near ties
        if n.endswith(".weight") and params[n].ndim == 2:
            params[n] = ho.f32_round(params[n] * 8.0)
    stream = rng.integers(0, 64, 16 * 5 + 3)
    for precision, tol in ((nn.PRECISION_F32, 2e-5), (nn.PRECISION_AMP_BF16, 3e-2)):
        amp = precision == nn.PRECISION_AMP_BF16
        model = nn.DecoderLm(c, nn.DecoderConfig(batch=3, precision=precision, **kw))
        model.load_state_dict(params)
        # windows shorter than, equal to and longer than the context
        for length in (1, 5, 16, 23):
            toks = stream[:length]
            got = gen.next_token_logits(model, toks)
            want = ho.decoder_logits(ocfg, params, toks[-16:][None, :], amp_bf16=amp)[0, -1]
            assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max()), (precision, length)
        # evaluation: two full batches of 3 windows would need 6 windows; the stream holds 5, so the second batch has 2 rows
        m = gen.evaluate_token_loss(model, stream, 3)
        assert (m.batches, m.examples, m.tokens) == (2, 5, 80)
        rows = np.stack([stream[i * 16:(i + 1) * 16] for i in range(5)])
        tgts = np.stack([stream[i * 16 + 1:(i + 1) * 16 + 1] for i in range(5)])
        logits = ho.decoder_logits(ocfg, params, rows, amp_bf16=amp).reshape(80, 64)
        want_loss = float(ho.cross_entropy(logits, tgts.reshape(80)))
        assert m.loss == pytest.approx(want_loss, rel=1e-5 if not amp else 5e-3) and m.perplexity == pytest.approx(math.exp(m.loss))
        assert gen.evaluate_token_loss(model, stream, 2, max_batches=1).examples == 2
        with pytest.raises(Exception, match="more than block_size tokens"):
            gen.evaluate_token_loss(model, stream[:16], 2)
        if not amp:
            # greedy generation follows the oracle's argmax chain
            want_tokens = list(stream[:4])
            for _ in range(6):
                lg = ho.decoder_logits(ocfg, params, np.asarray(want_tokens[-16:])[None, :])[0, -1]
                want_tokens.append(gen.argmax_filtered(lg))
            got_tokens = gen.generate_greedy(model, stream[:4], 6, eos_id=10**9)
            assert got_tokens == [int(t) for t in want_tokens]
            out = gen.generate(model, stream[:4], gen.GenerationOptions(6, 10**9, temperature=1.0, top_k=1, top_p=1.0), gen.HeirloomRng(123))
            assert out.tokens == got_tokens and out.new_token_count == 6 and out.finish_reason == "max_new_tokens"
            assert all(s.probability > 0.0 for s in out.steps) and out.rng_state != 123
            eos = got_tokens[5]
            assert gen.generate(model, stream[:4], gen.GenerationOptions.greedy(6, eos), gen.HeirloomRng(0)).finish_reason == "eos"
        model.close()

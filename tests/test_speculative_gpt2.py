"""GPT-2 layer-split speculation (Sources/RealModelInference/RealModelInferenceEngine.swift:4989-5201, switch :2048-2064):
whatever the first-k-layers draft proposes, the emitted stream is the full model's greedy stream."""
import json
import os

import pytest

from espresso_b200.speculative import (
    GPT2_EOS_TOKEN,
    build_layer_split_pair,
    generate_layer_split_speculative,
    resolved_speculative_draft_layer_count,
)


def _cfg(n_layer=3):
    from espresso_b200.model_config import tiny_gpt2

    return tiny_gpt2(vocab=512, max_seq=64, n_layer=n_layer)


def test_draft_layer_count_follows_the_reference_switch():
    from espresso_b200.model_config import tiny_llama

    cfg = _cfg(4)
    on = {"ESPRESSO_ENABLE_GPT2_SPECULATIVE": "1"}
    assert resolved_speculative_draft_layer_count(cfg, 0.0, {}) is None                      # off by default
    assert resolved_speculative_draft_layer_count(cfg, 0.0, on) == 1                         # default: one layer
    assert resolved_speculative_draft_layer_count(cfg, 0.7, on) is None                      # greedy only
    assert resolved_speculative_draft_layer_count(tiny_llama(), 0.0, on) is None             # GPT-2 only
    assert resolved_speculative_draft_layer_count(_cfg(1), 0.0, on) is None                  # needs a layer to verify with
    many = dict(on, ESPRESSO_GPT2_SPECULATIVE_DRAFT_LAYERS="9")
    assert resolved_speculative_draft_layer_count(cfg, 0.0, many) == 3                       # clamped to nLayer - 1
    assert resolved_speculative_draft_layer_count(cfg, 0.0, dict(on, ESPRESSO_GPT2_SPECULATIVE_DRAFT_LAYERS="0")) == 1
    assert resolved_speculative_draft_layer_count(cfg, 0.0, dict(on, ESPRESSO_GPT2_SPECULATIVE_DRAFT_LAYERS="two")) == 1
    assert resolved_speculative_draft_layer_count(cfg, 0.0, {"ESPRESSO_ENABLE_GPT2_SPECULATIVE": "true"}) is None


class OracleDecoder:
    """The oracle's runtime under the call names of the engine object."""

    def __init__(self, oracle, model):
        self._o = oracle
        self.rt = oracle.Runtime(model)
        self._cps = []

    def reset(self):
        self.rt.reset()

    def advance(self, token):
        assert self.rt.advance(token) == 0

    def select_greedy_token(self):
        return self.rt.select_greedy()

    def capture_checkpoint(self):
        self._cps.append(self.rt.checkpoint())
        return len(self._cps) - 1

    def rollback(self, cp):
        self.rt.rollback(self._cps[cp])

    def close(self):
        for cp in self._cps:
            self.rt.free_checkpoint(cp)
        self._cps = []


def _oracle_model(oracle, weight_dir, n_layer=None):
    with open(os.path.join(weight_dir, "metadata.json")) as f:
        meta = json.load(f)
    if n_layer is not None:
        meta = dict(meta, nLayer=n_layer)
    m = oracle.Model(meta)
    assert oracle.lib().esp_oracle_model_load_dir(m.handle, os.fsencode(weight_dir)) == 0
    return m


@pytest.mark.parametrize("draft_layers", [1, 2, 3])
def test_loop_emits_the_full_models_greedy_stream_on_the_oracle(oracle_lib, tmp_models, draft_layers):
    from espresso_b200.synthetic import synthetic_prompt

    cfg = _cfg(3)
    d = tmp_models(cfg)
    prompt = synthetic_prompt(cfg.vocab, 8)
    full = _oracle_model(oracle_lib, d)
    greedy = [int(t) for t in oracle_lib.Runtime(full).generate(prompt, 40)]
    assert len(greedy) == 40
    # draft_layers == nLayer: the draft is the model itself, every proposal must be accepted
    draft = OracleDecoder(oracle_lib, _oracle_model(oracle_lib, d, draft_layers))
    verifier = OracleDecoder(oracle_lib, full)
    steps = []
    res = generate_layer_split_speculative(draft, verifier, prompt, 40, cfg.maxSeq, on_step=lambda tok, toks, ms: steps.append((tok, len(toks))))
    assert res.tokens == greedy
    assert [s[0] for s in steps] == greedy and [s[1] for s in steps] == list(range(1, 41))
    assert len(res.tokenLatenciesMs) == 40 and not res.stoppedOnEOS
    assert res.passes >= 20 and res.acceptedSecond <= res.acceptedFirst <= res.passes
    if draft_layers == 3:
        assert res.passes == 20 and res.acceptedFirst == 20 and res.acceptedSecond == 20
    draft.close()
    verifier.close()


def test_loop_limits_and_stop_rule_on_the_oracle(oracle_lib, tmp_models):
    from espresso_b200.synthetic import synthetic_prompt

    cfg = _cfg(3)
    d = tmp_models(cfg)
    prompt = synthetic_prompt(cfg.vocab, 8)
    full = _oracle_model(oracle_lib, d)
    greedy = [int(t) for t in oracle_lib.Runtime(full).generate(prompt, 56)]
    draft = OracleDecoder(oracle_lib, _oracle_model(oracle_lib, d, 1))
    verifier = OracleDecoder(oracle_lib, full)
    # the context limit: 8 prompt tokens leave room for 56 more, however many are asked for
    res = generate_layer_split_speculative(draft, verifier, prompt, 500, cfg.maxSeq)
    assert res.tokens == greedy and len(res.tokens) == cfg.maxSeq - len(prompt)
    # an odd budget ends inside a pass
    assert generate_layer_split_speculative(draft, verifier, prompt, 7, cfg.maxSeq).tokens == greedy[:7]
    assert generate_layer_split_speculative(draft, verifier, prompt, 0, cfg.maxSeq).tokens == []
    # the stop token is not emitted, at either position of a pass
    for k in (4, 5):
        stop = greedy[k]
        first = greedy.index(stop)
        res = generate_layer_split_speculative(draft, verifier, prompt, 56, cfg.maxSeq, eos_token=stop)
        assert res.tokens == greedy[:first] and res.stoppedOnEOS
    with pytest.raises(ValueError):
        generate_layer_split_speculative(draft, verifier, [], 4, cfg.maxSeq)
    with pytest.raises(ValueError):
        generate_layer_split_speculative(draft, verifier, list(range(cfg.maxSeq)), 4, cfg.maxSeq)
    assert GPT2_EOS_TOKEN == 50256
    draft.close()
    verifier.close()


@pytest.mark.gpu
def test_layer_split_pair_on_the_device_emits_the_greedy_stream(oracle_lib, tmp_models):
    from espresso_b200 import runtime
    from espresso_b200.synthetic import synthetic_prompt
    from helpers import compare_greedy_stream

    cfg = _cfg(3)
    d = tmp_models(cfg)
    prompt = synthetic_prompt(cfg.vocab, 8)
    plain = runtime.DecodeEngine.build(d)
    greedy = [int(t) for t in plain.generate(prompt, 40).tokens]
    plain.close()
    for k in (1, 2):
        draft, verifier = build_layer_split_pair(runtime, d, k)
        assert draft.config.nLayer == k and verifier.config.nLayer == 3
        res = generate_layer_split_speculative(draft, verifier, prompt, 40, cfg.maxSeq)
        assert res.tokens == greedy
        assert res.passes >= 20
        draft.close()
        verifier.close()
    compare_greedy_stream(oracle_lib.Runtime(_oracle_model(oracle_lib, d)), prompt, greedy)
    with pytest.raises(ValueError):
        build_layer_split_pair(runtime, d, 3)

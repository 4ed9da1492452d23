"""Exact two-token generation as one device-driven launch (``csrc/spec_kernel.cuh``): the draft's proposal, the target's
two-position verify pass and the commit rule of Sources/Espresso/GenerationHarness.swift:1281-1344 all run inside one
cooperative kernel when draft and target share their widths.  Whatever the draft proposes, the emitted stream must be
the target's own greedy stream; limits and the end-of-sequence rule are those of the host-driven loop
(Sources/RealModelInference/RealModelInferenceEngine.swift:6014-6190)."""
import dataclasses

import numpy as np
import pytest

from helpers import compare_greedy_stream

pytestmark = pytest.mark.gpu

NO_MEGAKERNEL = 4


@pytest.fixture(scope="module")
def rt():
    from espresso_b200 import runtime

    runtime.load_library()
    return runtime


@pytest.fixture(scope="module")
def c2_models(tmp_models):
    from espresso_b200.model_config import llama_6l, llama_draft_1l

    cfg, dcfg = llama_6l(), llama_draft_1l()
    return cfg, tmp_models(cfg), tmp_models(dcfg, seed=1235)


def test_two_token_kernel_emits_the_greedy_stream_with_any_draft(rt, oracle_lib, c2_models):
    from espresso_b200.synthetic import synthetic_prompt

    cfg, d, dd = c2_models
    prompt = synthetic_prompt(cfg.vocab, 16)
    eng = rt.DecodeEngine.build(d)
    greedy = eng.generate(prompt, 96).tokens
    for draft_dir, identical in ((dd, False), (d, True)):
        draft = rt.DecodeEngine.build(draft_dir)
        res = eng.generate_two_token(draft, prompt, 96)
        assert list(res.tokens) == list(greedy)
        assert eng.timings()["kernel_launches"] == 1  # one launch for the whole loop
        if identical:
            # the draft is the target: every proposal is accepted, two tokens per pass (the last pass may commit one)
            assert res.committedExactTokensPerPass > 1.9 and res.acceptedFutureTokensPerPass > 0.9
            assert res.speculativePasses <= 49
        else:
            assert 1.0 <= res.committedExactTokensPerPass <= 2.0
        # the engine is left where the host-driven loop leaves it: everything but the newest token is visible
        assert eng.visible_token_count() in (len(prompt) + len(res.tokens) - 1, len(prompt) + len(res.tokens))
        draft.close()
    compare_greedy_stream(oracle_lib.Runtime(oracle_lib.Model.from_dir(d)), prompt, greedy)
    eng.close()


def test_two_token_kernel_equals_the_host_driven_loop(rt, c2_models):
    """Same tokens and the same pass statistics as the loop that calls draft step, verify2 and commit from the host
    (an engine without the persistent kernel takes that loop)."""
    from espresso_b200.synthetic import synthetic_prompt

    cfg, d, dd = c2_models
    prompt = synthetic_prompt(cfg.vocab, 16, stream=3)
    fused_t, fused_d = rt.DecodeEngine.build(d), rt.DecodeEngine.build(dd)
    host_t, host_d = rt.DecodeEngine.build(d, flags=NO_MEGAKERNEL), rt.DecodeEngine.build(dd, flags=NO_MEGAKERNEL)
    for n in (1, 2, 3, 8, 41):
        a = fused_t.generate_two_token(fused_d, prompt, n)
        b = host_t.generate_two_token(host_d, prompt, n)
        assert len(a.tokens) == n and list(a.tokens) == list(b.tokens), n
    for e in (fused_t, fused_d, host_t, host_d):
        e.close()


def test_two_token_kernel_stops_on_eos_and_at_the_context_limit(rt, tmp_models, c2_models):
    from espresso_b200.synthetic import synthetic_prompt

    cfg, d, dd = c2_models
    prompt = synthetic_prompt(cfg.vocab, 16, stream=5)
    plain = rt.DecodeEngine.build(d)
    greedy = list(plain.generate(prompt, 40).tokens)
    plain.close()
    # the token emitted at step 9 (its first occurrence) becomes the end-of-sequence token: emitted, then stop
    stop_at = 9
    eos = int(greedy[stop_at])
    first = greedy.index(eos)
    ecfg = dataclasses.replace(cfg, eosToken=eos)
    eng, draft, twin = rt.DecodeEngine.build(d, config=ecfg), rt.DecodeEngine.build(dd), rt.DecodeEngine.build(d)
    for dr in (draft, twin):  # a poor draft, then a copy of the target (accepted pairs: the stop may fall on either token)
        res = eng.generate_two_token(dr, prompt, 40)
        assert list(res.tokens) == greedy[: first + 1] and res.stoppedOnEOS
    for e in (eng, draft, twin):
        e.close()
    # context limit: prompt of max_seq - 5 tokens leaves room for 5 more
    long_prompt = synthetic_prompt(cfg.vocab, cfg.maxSeq - 5, stream=7)
    eng, draft, twin = rt.DecodeEngine.build(d), rt.DecodeEngine.build(dd), rt.DecodeEngine.build(d)
    want = list(eng.generate(long_prompt, 64).tokens)
    for dr in (draft, twin):
        res = eng.generate_two_token(dr, long_prompt, 64)
        assert list(res.tokens) == want and len(want) == 5
    for e in (eng, draft, twin):
        e.close()

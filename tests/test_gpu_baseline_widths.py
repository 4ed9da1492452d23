"""GPU parity at the widths, vocabularies, storage types and batch sizes of the five benchmark configurations.

The configurations' models are cut to two layers (the CPU oracle then finishes in seconds) but keep their real
d_model / heads / hidden / vocab / dtype / batch, so every kernel runs with the launch shapes of the benchmark.
Every case drives the CUDA library through its C ABI and compares with the CPU oracle on the same seeded weights;
with many sequences the device decodes all of them and the oracle checks a few (first, last and some in between).
Also here: the GPT-2 stop rule (token 50256 ends generation without being appended) and a device wait that runs out.
"""
import dataclasses

import numpy as np
import pytest

from helpers import BF16_ABS_TOL, assert_logits_close, compare_greedy_stream, dense_pair, quantised_pair, upload_all

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    from espresso_b200 import runtime

    runtime.load_library()
    return runtime


def _check_sequences(oracle_lib, model, prompts, streams, which, max_near=2):
    for s in which:
        near = compare_greedy_stream(oracle_lib.Runtime(model), prompts[s], streams[s])
        assert len(near) <= max_near, f"sequence {s}: near ties at {near}"


def test_c2_two_token_at_real_widths(rt, oracle_lib, tmp_models):
    """The d768 6-layer target with the 1-layer draft of the same shape: 128 tokens, stream equal to the target's greedy one."""
    from espresso_b200.model_config import llama_6l, llama_draft_1l
    from espresso_b200.synthetic import synthetic_prompt

    cfg, dcfg = llama_6l(), llama_draft_1l()
    d, dd = tmp_models(cfg), tmp_models(dcfg, seed=1235)
    prompt = synthetic_prompt(cfg.vocab, 16)
    eng, draft = rt.DecodeEngine.build(d), rt.DecodeEngine.build(dd)
    res = eng.generate_two_token(draft, prompt, 128)
    assert len(res.tokens) == 128 and res.speculativePasses > 0
    near = compare_greedy_stream(oracle_lib.Runtime(oracle_lib.Model.from_dir(d)), prompt, res.tokens)
    assert len(near) <= 2
    draft.close()
    eng.close()


def test_c3_gpt2_256_sequences_context_past_256(rt, oracle_lib):
    """GPT-2 widths (d768, h3072, vocab 50257, context 1024), 256 sequences, 64-token prompts, 200 steps: the batched
    tensor-core path at its benchmark batch, positions crossing the 256-token attention split."""
    from espresso_b200.model_config import gpt2_117m
    from espresso_b200.synthetic import synthetic_prompt

    cfg = dataclasses.replace(gpt2_117m(), nLayer=2, name="gpt2-2l")
    eng, model = dense_pair(rt, oracle_lib, cfg, "f16", 256)
    prompts = np.stack([synthetic_prompt(cfg.vocab, 64, stream=s) for s in range(256)])
    streams, _ = eng.generate_batch(prompts, 200)
    assert min(len(t) for t in streams) >= 1 and max(len(t) for t in streams) == 200  # 50256 may end a sequence early
    _check_sequences(oracle_lib, model, prompts, streams, (0, 101, 255))
    eng.close()


@pytest.mark.parametrize("kind", ["q8_0", "q4_0"])
def test_c4_quantised_1b_widths_batch_1_and_16(rt, oracle_lib, kind):
    """Llama d2048, GQA 32/4, hidden 5632, vocab 32000 with GGUF blocks for the matrices and the LM head: one sequence
    (persistent kernel) and sixteen (batched path), both against the oracle on the dequantised values."""
    from espresso_b200.model_config import llama_1b
    from espresso_b200.synthetic import synthetic_prompt

    cfg = dataclasses.replace(llama_1b(max_seq=256), nLayer=2, name="llama-1b-2l")
    model, uploads = quantised_pair(oracle_lib, cfg, kind)
    prompts = np.stack([synthetic_prompt(cfg.vocab, 24, stream=s) for s in range(16)])
    eng = rt.DecodeEngine.empty(cfg, max_batch=16)
    upload_all(eng, uploads)
    one = eng.generate(prompts[0], 24)
    near = compare_greedy_stream(oracle_lib.Runtime(model), prompts[0], one.tokens)
    assert len(near) <= 2
    eng.prefill(prompts[0])
    ora = oracle_lib.Runtime(model)
    assert ora.prefill(prompts[0]) == 0
    assert_logits_close(eng.logits(), ora.logits(), f"{kind} batch 1 after the prompt")
    streams, _ = eng.generate_batch(prompts, 24)
    _check_sequences(oracle_lib, model, prompts, streams, (0, 7, 15))
    eng.close()


def test_c5_llama3_8b_widths_bf16_64_sequences(rt, oracle_lib):
    """Llama-3-8B widths (d4096, GQA 32/8, head_dim 128, hidden 14336, vocab 128256, theta 5e5) in bf16 with 64 sequences:
    the batched path's bf16 branches (operand rows, attention, epilogues, LM head) as an engine."""
    from espresso_b200.model_config import llama3_8b
    from espresso_b200.synthetic import synthetic_prompt

    cfg = dataclasses.replace(llama3_8b(max_seq=128), nLayer=2, name="llama3-8b-2l")
    eng, model = dense_pair(rt, oracle_lib, cfg, "bf16", 64)
    prompts = np.stack([synthetic_prompt(cfg.vocab, 12, stream=s) for s in range(64)])
    streams, _ = eng.generate_batch(prompts, 6)
    assert all(len(t) == 6 for t in streams)
    _check_sequences(oracle_lib, model, prompts, streams, (0, 63))
    # logits of one sequence after its prompt: the prompt runs through the tensor-core path with bf16 activations
    eng.reset()
    eng.prefill(prompts[5])
    ora = oracle_lib.Runtime(model)
    assert ora.prefill(prompts[5]) == 0
    assert_logits_close(eng.logits(), ora.logits(), "bf16 8B widths after the prompt", abs_tol=BF16_ABS_TOL)
    eng.close()


def test_gpt2_stops_on_50256_without_appending_it(rt, oracle_lib, tmp_path):
    """Sources/RealModelInference/RealModelInferenceEngine.swift:4918-4922: token 50256 ends generation and is not part
    of the output.  The LM-head row of 50256 is planted along the final hidden state of a chosen step, so its logit is
    the largest there (at the latest)."""
    import shutil

    from espresso_b200.model_config import tiny_gpt2
    from espresso_b200.synthetic import synthetic_prompt, write_synthetic_model
    from espresso_b200.weight_blob import read_blob, write_blob

    cfg = tiny_gpt2(vocab=50257, max_seq=64, n_layer=2)
    d = write_synthetic_model(cfg, str(tmp_path / "gpt2"))
    prompt = synthetic_prompt(cfg.vocab, 7)
    ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
    free = ora.generate(prompt, 40)
    assert len(free) == 40 and 50256 not in free  # the unplanted model does not hit the token by chance
    # final normalised hidden states n_t of the first ten emission steps, by least squares from the logits (logits = W n)
    head = read_blob(d + "/lm_head.bin").astype(np.float64).reshape(cfg.vocab, cfg.dModel)
    solve = np.linalg.solve(head.T @ head, head.T)
    assert ora.prefill(prompt) == 0
    states, tops = [], []
    for t in free[:10]:
        logits = ora.logits().astype(np.float64)
        states.append(solve @ logits)
        tops.append(logits.max())
        assert ora.advance(int(t)) == 0
    # the planted row is orthogonal to the states of steps 0..8 and beats every logit of step 9: the stream keeps its
    # first nine tokens and stops there
    q, _ = np.linalg.qr(np.stack(states[:9], axis=1))
    u = states[9] - q @ (q.T @ states[9])
    planted = head.copy()
    planted[50256] = u * ((tops[9] + 0.5) / float(u @ states[9]))
    d2 = str(tmp_path / "gpt2_planted")
    shutil.copytree(d, d2)
    write_blob(d2 + "/lm_head.bin", planted.astype(np.float16))
    ref = oracle_lib.Runtime(oracle_lib.Model.from_dir(d2)).generate(prompt, 40)
    assert list(ref) == list(free[:9])  # the oracle stops at step 9 and drops the token
    eng = rt.DecodeEngine.build(d2)
    out = eng.generate(prompt, 40)
    assert list(out.tokens) == list(ref) and out.stoppedOnEOS
    # the same rule in a batch: a sequence that stops leaves the others running
    other = synthetic_prompt(cfg.vocab, 7, stream=3)
    eng2 = rt.DecodeEngine.build(d2, max_batch=2)
    streams, _ = eng2.generate_batch(np.stack([prompt, other]), 40)
    assert list(streams[0]) == list(ref)
    assert list(streams[1]) == list(oracle_lib.Runtime(oracle_lib.Model.from_dir(d2)).generate(other, 40))
    eng2.close()
    eng.close()


def test_device_wait_that_runs_out_reports_a_timeout(rt, oracle_lib, tmp_models):
    """Every wait inside the persistent decode kernel is bounded.  With a limit of a few polls the first exchange between
    CTAs cannot complete in time: the kernel gives up everywhere, finishes, and the call returns ESP_CUDA_ERR_TIMEOUT
    (nothing faults or hangs).  With the default limit restored the same engine decodes correctly again."""
    from espresso_b200.model_config import tiny_llama
    from espresso_b200.synthetic import synthetic_prompt

    cfg = tiny_llama(vocab=512, max_seq=64, n_layer=2)
    d = tmp_models(cfg)
    prompt = synthetic_prompt(cfg.vocab, 9)
    eng = rt.DecodeEngine.build(d)
    good = eng.generate(prompt, 20).tokens
    eng.set_wait_limit(2)
    with pytest.raises(rt.RealModelInferenceError) as err:
        eng.generate(prompt, 20)
    assert err.value.status == 5 and "gave up waiting" in err.value.message  # ESP_CUDA_ERR_TIMEOUT
    eng.set_wait_limit(0)
    eng.reset()
    again = eng.generate(prompt, 20).tokens
    assert list(again) == list(good)
    compare_greedy_stream(oracle_lib.Runtime(oracle_lib.Model.from_dir(d)), prompt, again)
    eng.close()


def test_per_token_latencies_and_step_callback(rt, oracle_lib, tmp_models):
    """GenerationResult.tokenLatenciesMs and the inline onStep callback (Engine.swift:17-55, 6393-6405): the device-driven
    loops report one latency per token, and the token-by-token form calls back once per token with the same stream."""
    from espresso_b200.model_config import tiny_llama
    from espresso_b200.synthetic import synthetic_prompt

    cfg = tiny_llama(vocab=512, max_seq=64, n_layer=2)
    d = tmp_models(cfg)
    prompt = synthetic_prompt(cfg.vocab, 6)
    ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
    for flags in (0, rt.FLAG_NO_MEGAKERNEL):
        eng = rt.DecodeEngine.build(d, flags=flags)
        res = eng.generate(prompt, 18)
        lat = res.tokenLatenciesMs
        assert lat is not None and lat.size == 18 and np.all(lat > 0) and lat.sum() < 1e3
        seen = []
        stepped = eng.generate(prompt, 18, on_step=lambda tok, idx, ms: seen.append((tok, idx, ms)))
        assert [t for t, _, _ in seen] == list(stepped.tokens) and [i for _, i, _ in seen] == list(range(18))
        assert all(ms > 0 for _, _, ms in seen) and stepped.tokenLatenciesMs.size == 18
        compare_greedy_stream(ora, prompt, stepped.tokens)
        compare_greedy_stream(ora, prompt, res.tokens)
        eng.close()

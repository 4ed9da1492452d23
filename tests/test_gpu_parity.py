"""GPU parity tests: every case drives the CUDA library through its C ABI (ctypes) and compares with the
CPU oracle on the same seeded inputs.  Integer/byte results must be bit-exact; logits must agree within
max-abs 2e-2 and relative 1e-2 (fp16 KV cache and a different summation order are the only differences);
greedy streams must be identical wherever the oracle's top-2 logit gap exceeds that tolerance."""
import dataclasses
import os

import numpy as np
import pytest

from helpers import ABS_TOL, assert_logits_close, compare_greedy_stream, dense_pair, quantised_pair, upload_all

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def rt():
    from espresso_b200 import runtime

    runtime.load_library()
    return runtime


def test_dequantize_bit_exact(rt, oracle_lib):
    g = np.load(os.path.join(GOLD, "gguf_blocks.npz"))
    for kind in ("q8_0", "q4_0"):
        got = rt.dequantize(kind, g[kind + "_blocks"], g["x"].size)
        assert np.array_equal(got.view(np.uint32), g[kind + "_dequant"].view(np.uint32))
    rng = np.random.default_rng(9)
    x = (rng.standard_normal(32 * 5000) * 0.02).astype(np.float32)
    for kind in ("q8_0", "q4_0"):
        blocks = oracle_lib.quantize(kind, x)
        got = rt.dequantize(kind, blocks, x.size)
        assert np.array_equal(got.view(np.uint32), oracle_lib.dequantize(kind, blocks, x.size).view(np.uint32))
    assert rt.dequantize("q8_0", np.zeros(0, np.uint8), 0).size == 0  # empty input


@pytest.mark.parametrize("kind", ["f16", "bf16", "q8_0", "q4_0"])
@pytest.mark.parametrize("shape", [(96, 128), (1000, 768), (257, 2048), (64, 5632), (4807, 2048)])  # the last one: many CTAs, a ragged tail
def test_gemv_kernel_matches_oracle(rt, oracle_lib, kind, shape):
    rows, cols = shape
    rng = np.random.default_rng(rows * 31 + cols)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    if kind == "f16":
        stored = w.astype(np.float16)
        ref_w = stored.astype(np.float32)
    elif kind == "bf16":
        bits = (w.view(np.uint32) >> 16).astype(np.uint16)
        stored = bits
        ref_w = (bits.astype(np.uint32) << 16).view(np.float32)
    else:
        stored = oracle_lib.quantize(kind, w)
        ref_w = oracle_lib.dequantize(kind, stored, w.size).reshape(rows, cols)
    y, ms = rt.gemv_bench(kind, stored, rows, cols, x, warmup=1, iterations=2)
    ref = oracle_lib.gemv(ref_w, x)
    if kind in ("f16", "bf16"):
        np.testing.assert_allclose(y, ref, atol=2e-4, rtol=1e-4)  # fp32 activations and accumulation
    else:
        # quantised types multiply in packed fp16 (activations rounded to fp16, per-block fp16 partial sums);
        # the weights themselves are exact, so the error is pure rounding noise relative to the result's scale
        assert np.abs(y - ref).max() <= 4e-3 * np.abs(ref).max()
        assert np.linalg.norm(y - ref) <= 2e-3 * np.linalg.norm(ref)
    assert ms > 0


@pytest.mark.parametrize("kind,shape", [("f16", (128, 64, 16)), ("f16", (300, 768, 5)), ("f16", (2304, 768, 256)), ("bf16", (1000, 128, 33)),
                                        ("f16", (4096, 2048, 64)), ("bf16", (515, 4096, 130))])
def test_tensor_core_gemm_matches_fp32_reference(rt, kind, shape):
    """tcgen05/TMEM GEMM: exact 16-bit operands, fp32 accumulation; ragged M (TMA zero fill) and ragged batch."""
    import torch

    M, K, N = shape
    rng = np.random.default_rng(M * 7 + K + N)
    w = (rng.standard_normal((M, K)) * 0.05).astype(np.float32)
    x = rng.standard_normal((N, K)).astype(np.float32)
    if kind == "f16":
        stored = w.astype(np.float16)
        wr, xr = stored.astype(np.float32), x.astype(np.float16).astype(np.float32)
    else:
        tw = torch.from_numpy(w).to(torch.bfloat16)
        stored = tw.view(torch.int16).numpy().view(np.uint16)
        wr, xr = tw.float().numpy(), torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    y, ms = rt.gemm_tc_bench(kind, stored, M, K, x, warmup=1, iterations=2)
    ref = xr.astype(np.float64) @ wr.astype(np.float64).T
    np.testing.assert_allclose(y, ref, atol=2e-4, rtol=2e-4)
    assert ms > 0
    with pytest.raises(rt.RealModelInferenceError):
        rt.gemm_tc_bench(kind, stored, M, K, np.zeros((257, K), np.float32))  # batch beyond one accumulator tile


def _stepwise_logit_parity(rt, oracle_lib, weight_dir, prompt, extra_steps=6):
    eng = rt.DecodeEngine.build(weight_dir)
    ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(weight_dir))
    eng.reset()
    ora.reset()
    for i, t in enumerate(prompt):
        eng.advance(int(t))
        assert ora.advance(int(t)) == 0
        assert_logits_close(eng.logits(), ora.logits(), f"prompt position {i}")
    tok = eng.select_greedy_token()
    for i in range(extra_steps):
        assert_logits_close(eng.logits(), ora.logits(), f"decode step {i}")
        nxt = eng.decode_step(tok)
        assert ora.advance(tok) == 0
        tok = nxt
    assert eng.visible_token_count() == ora.visible == len(prompt) + extra_steps
    eng.close()


@pytest.mark.parametrize("gqa", [True, False])
def test_llama_tiny_logits_match_oracle(rt, oracle_lib, tmp_models, gqa):
    from espresso_b200.model_config import tiny_llama
    from espresso_b200.synthetic import synthetic_prompt

    cfg = tiny_llama(vocab=512, max_seq=64, n_layer=2, gqa=gqa)
    _stepwise_logit_parity(rt, oracle_lib, tmp_models(cfg), synthetic_prompt(cfg.vocab, 9))


def test_gpt2_tiny_logits_match_oracle(rt, oracle_lib, tmp_models):
    from espresso_b200.model_config import tiny_gpt2
    from espresso_b200.synthetic import synthetic_prompt

    cfg = tiny_gpt2(vocab=512, max_seq=64, n_layer=2)
    _stepwise_logit_parity(rt, oracle_lib, tmp_models(cfg, 777), synthetic_prompt(cfg.vocab, 9, seed=777))


def test_logits_match_huggingface_golden(rt, tmp_models):
    from espresso_b200.model_config import tiny_gpt2, tiny_llama

    g = np.load(os.path.join(GOLD, "hf_llama_tiny.npz"))
    for tag, gqa in (("gqa", True), ("mha", False)):
        cfg = tiny_llama(vocab=512, max_seq=64, n_layer=2, gqa=gqa)
        eng = rt.DecodeEngine.build(tmp_models(cfg, int(g[tag + "_seed"])))
        eng.reset()
        for i, t in enumerate(g[tag + "_prompt"]):
            eng.advance(int(t))
            assert_logits_close(eng.logits(), g[tag + "_logits"][i], f"hf llama {tag} pos {i}")
        eng.close()
    g = np.load(os.path.join(GOLD, "hf_gpt2_tiny.npz"))
    cfg = tiny_gpt2(vocab=512, max_seq=64, n_layer=2)
    eng = rt.DecodeEngine.build(tmp_models(cfg, int(g["seed"])))
    eng.reset()
    for i, t in enumerate(g["prompt"]):
        eng.advance(int(t))
        assert_logits_close(eng.logits(), g["logits"][i], f"hf gpt2 pos {i}")
    eng.close()


def test_stage_dumps_match_oracle(rt, oracle_lib, tmp_models):
    # bisect-by-stage hooks, as the reference's test_debug* helpers do (Engine.swift:419-484)
    from espresso_b200.model_config import tiny_llama

    cfg = tiny_llama(vocab=512, max_seq=64, n_layer=2, gqa=True)
    d = tmp_models(cfg)
    eng = rt.DecodeEngine.build(d)
    ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
    for layer in (0, 1):
        eng.reset(); ora.reset()
        eng.set_debug_layer(layer)
        ora.set_capture_layer(layer)
        for t in (3, 77, 301, 12):
            eng.advance(t)
            assert ora.advance(t) == 0
        for stage, tol in ((0, 2e-4), (1, 2e-3), (2, 2e-3), (3, 2e-3), (4, 2e-3), (5, 2e-3), (6, 3e-3)):
            np.testing.assert_allclose(eng.debug_dump(stage), ora.captured(stage), atol=tol, rtol=1e-2,
                                       err_msg=f"layer {layer} stage {stage}")
    eng.set_debug_layer(-1)
    eng.close()


def test_prefill_equals_token_by_token(rt, tmp_models):
    from espresso_b200.model_config import tiny_llama
    from espresso_b200.synthetic import synthetic_prompt

    cfg = tiny_llama(vocab=512, max_seq=64, n_layer=2)
    eng = rt.DecodeEngine.build(tmp_models(cfg))
    prompt = synthetic_prompt(cfg.vocab, 21)
    eng.prefill(prompt)
    a = eng.logits()
    eng.reset()
    for t in prompt:
        eng.advance(int(t))
    b = eng.logits()
    # the chunked prefill runs on the tensor cores with 16-bit activation rows, the single steps on the GEMV path
    assert_logits_close(a, b, "chunked prefill vs token by token")
    assert eng.visible_token_count() == 21
    eng.close()


def test_float32_sidecars_win_over_the_fp16_blobs(rt, oracle_lib, tmp_models, tmp_path):
    """loadWeightTablePreferringFloat32Sidecar (Sources/RealModelInference/RealModelInferenceEngine.swift:7830-7879):
    "<name>.float32.bin" beside "<name>.bin" is what gets loaded.  The sidecars here hold values that differ from the
    blobs (gains that fp16 cannot represent, a negated matrix), so ignoring them would show in the logits."""
    import shutil

    from espresso_b200.model_config import tiny_llama
    from espresso_b200.synthetic import synthetic_prompt
    from espresso_b200.weight_blob import read_blob

    cfg = tiny_llama(vocab=512, max_seq=64, n_layer=2)
    d = str(tmp_path / "sidecars")
    shutil.copytree(tmp_models(cfg), d)
    rng = np.random.default_rng(5)
    gains = (1.0 + 0.05 * rng.standard_normal(cfg.dModel)).astype(np.float32)
    assert not np.array_equal(gains, gains.astype(np.float16).astype(np.float32))
    gains.tofile(os.path.join(d, "layers/0/rms_att.float32.bin"))
    (3.0 + 0.05 * rng.standard_normal(cfg.dModel)).astype(np.float32).tofile(os.path.join(d, "rms_final.float32.bin"))
    wq = read_blob(os.path.join(d, "layers/1/wq.bin")).astype(np.float32)
    (-wq).tofile(os.path.join(d, "layers/1/wq.float32.bin"))
    prompt = synthetic_prompt(cfg.vocab, 9)
    eng = rt.DecodeEngine.build(d)
    eng.prefill(prompt)
    ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
    assert ora.prefill(prompt) == 0
    assert_logits_close(eng.logits(), ora.logits(), "directory with float32 sidecars")
    plain = oracle_lib.Runtime(oracle_lib.Model.from_dir(tmp_models(cfg)))
    assert plain.prefill(prompt) == 0
    assert np.abs(plain.logits() - ora.logits()).max() > 5 * ABS_TOL  # the sidecars do change the model (final gains x3)
    eng.close()
    # a sidecar of the wrong size is an error, not a fallback to the blob
    np.zeros(7, np.float32).tofile(os.path.join(d, "layers/0/rms_ffn.float32.bin"))
    with pytest.raises(rt.RealModelInferenceError) as ei:
        rt.DecodeEngine.build(d)
    assert ei.value.status == rt.ERR_INVALID_WEIGHTS and "invalidWeightCount" in ei.value.message


@pytest.mark.parametrize("head_dim,n_head,n_kv", [(32, 8, 2), (64, 4, 4), (128, 4, 2)])
def test_per_head_qk_norm_matches_oracle(rt, oracle_lib, tmp_path, head_dim, n_head, n_kv):
    """Qwen3-style directories carry layers/N/q_norm.bin and k_norm.bin: RMSNorm over each head of q and k before RoPE
    (applyPerHeadRMSNormInPlace, Sources/RealModelInference/RealModelInferenceEngine.swift:6648-6672).  One sequence
    runs on the row-wise kernels, twelve on the tensor-core path; both against the oracle."""
    from espresso_b200.model_config import MultiModelConfig
    from espresso_b200.synthetic import synthetic_prompt, write_synthetic_model
    from espresso_b200.weight_blob import write_blob

    cfg = MultiModelConfig(f"qk-norm-hd{head_dim}", 2, n_head, n_kv, 256, head_dim, 512, 640, 96, 1e-6, 1000000.0, None, "llama")
    d = write_synthetic_model(cfg, str(tmp_path / "m"))
    rng = np.random.default_rng(head_dim)
    for l in range(cfg.nLayer):
        for leaf in ("q_norm", "k_norm"):
            write_blob(os.path.join(d, f"layers/{l}/{leaf}.bin"), (1.0 + 0.2 * rng.standard_normal(head_dim)).astype(np.float16))
    model = oracle_lib.Model.from_dir(d)
    eng = rt.DecodeEngine.build(d, max_batch=12)
    prompts = np.stack([synthetic_prompt(cfg.vocab, 11, stream=s) for s in range(12)])
    eng.prefill(prompts[0])
    ora = oracle_lib.Runtime(model)
    assert ora.prefill(prompts[0]) == 0
    assert_logits_close(eng.logits(), ora.logits(), "q/k norm, one sequence")
    res = eng.generate(prompts[0], 20)
    assert eng.timings()["kernel_launches"] > 1  # not the persistent kernel, which has no per-head norm
    compare_greedy_stream(oracle_lib.Runtime(model), prompts[0], res.tokens)
    streams, _ = eng.generate_batch(prompts, 16)
    for s_ in (0, 7, 11):
        compare_greedy_stream(oracle_lib.Runtime(model), prompts[s_], streams[s_])
    eng.close()
    # one of the two vectors alone is an error (Engine.swift:6589-6596)
    os.remove(os.path.join(d, "layers/1/k_norm.bin"))
    with pytest.raises(rt.RealModelInferenceError) as ei:
        rt.DecodeEngine.build(d)
    assert "Mismatched llama Q/K norm weights" in ei.value.message


def test_long_prefill_in_wide_passes_equals_token_by_token(rt, oracle_lib):
    """A 600-token prompt (one full 512-row pass and a ragged one, tiled attention across ten cache tiles) on a
    head_dim-128 GQA model: same logits as feeding the tokens one by one, and as the oracle."""
    from espresso_b200.model_config import MultiModelConfig
    from espresso_b200.synthetic import synthetic_prompt

    cfg = MultiModelConfig("gqa-hd128", 2, 4, 2, 512, 128, 1024, 640, 768, 1e-5, 500000.0, None, "llama")

    eng, model = dense_pair(rt, oracle_lib, cfg)
    prompt = synthetic_prompt(cfg.vocab, 600)
    eng.prefill(prompt)
    a = eng.logits()
    assert eng.visible_token_count() == 600
    ora = oracle_lib.Runtime(model)
    assert ora.prefill(prompt) == 0
    assert_logits_close(a, ora.logits(), "600-token prefill vs oracle")
    eng.reset()
    for t in prompt:
        eng.advance(int(t))
    assert_logits_close(a, eng.logits(), "600-token prefill vs token by token")
    eng.close()


def test_prefill_batch_packs_positions_and_equals_per_sequence_prefill(rt, oracle_lib):
    """prefill_batch feeds several positions of every sequence per pass (row = sequence x position); the state it leaves
    (KV cache, last hidden state per sequence) must be the one a per-sequence prefill leaves."""
    from espresso_b200.model_config import MultiModelConfig
    from espresso_b200.synthetic import synthetic_prompt

    cfg = MultiModelConfig("gqa-hd64-batch", 2, 8, 4, 512, 64, 1024, 640, 128, 1e-5, 10000.0, None, "llama")
    n_seq, n_prompt = 12, 45  # 256 // 12 = 21 positions per pass: passes of 21, 21 and 3 positions
    eng, model = dense_pair(rt, oracle_lib, cfg, max_batch=n_seq)
    prompts = np.stack([synthetic_prompt(cfg.vocab, n_prompt, stream=s) for s in range(n_seq)])
    eng.prefill_batch(prompts)
    for s in (0, 5, 11):
        ora = oracle_lib.Runtime(model)
        assert ora.prefill(prompts[s]) == 0
        assert_logits_close(eng.logits(s), ora.logits(), f"sequence {s} after the packed prefill")
    # and decoding continues from that state
    streams, _ = eng.generate_batch(prompts, 12)
    for s in (0, 11):
        compare_greedy_stream(oracle_lib.Runtime(model), prompts[s], streams[s])
    eng.close()


def test_generate_matches_oracle_greedy_6_layer_model(rt, oracle_lib, tmp_models):
    """The reference's own benchmark shape: 6 layers, d768, 12 heads, vocab 32000, 16-token prompt, 128 steps."""
    from espresso_b200.model_config import llama_6l
    from espresso_b200.synthetic import synthetic_prompt

    cfg = llama_6l()
    d = tmp_models(cfg)
    prompt = synthetic_prompt(cfg.vocab, 16)
    eng = rt.DecodeEngine.build(d)
    res = eng.generate(prompt, 128)
    assert len(res.tokens) == 128 and res.tokensPerSecond > 0
    ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
    near = compare_greedy_stream(ora, prompt, res.tokens)
    assert len(near) <= 2, f"too many near-tie positions: {near}"
    # the device-driven loop and the step-by-step API give the same stream
    eng.prefill(prompt)
    tok = eng.select_greedy_token()
    stream = [tok]
    for _ in range(31):
        tok = eng.decode_step(tok)
        stream.append(tok)
    # (summation orders differ between the two paths, so the comparison is again through the oracle)
    assert len(compare_greedy_stream(ora, prompt, stream)) <= 2
    assert_logits_close(eng.logits(), _oracle_logits_after(ora, prompt, stream[:-1]), "after 31 steps")
    eng.close()


def test_persistent_kernel_matches_per_stage_kernels(rt, oracle_lib, tmp_models):
    """The one-launch decode loop and the per-stage kernels are two routes to the same stream."""
    from espresso_b200.model_config import llama_6l, tiny_llama
    from espresso_b200.synthetic import synthetic_prompt

    for cfg, n in ((tiny_llama(vocab=512, max_seq=64, n_layer=2, gqa=True), 40), (tiny_llama(vocab=512, max_seq=64, n_layer=3, gqa=False), 40),
                   (llama_6l(), 64)):
        d = tmp_models(cfg)
        prompt = synthetic_prompt(cfg.vocab, 11)
        ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
        streams, near = [], []
        for flags in (0, rt.FLAG_NO_MEGAKERNEL):
            eng = rt.DecodeEngine.build(d, flags=flags)
            eng.prefill(prompt)
            toks, ms = eng.decode(n)
            assert len(toks[0]) == n and ms > 0
            if flags == 0:
                assert eng.timings()["kernel_launches"] == 1  # the whole loop was one persistent launch
            else:
                assert eng.timings()["kernel_launches"] > n
            near.append(compare_greedy_stream(ora, prompt, toks[0]))
            # the state left behind continues correctly through the step API
            assert eng.visible_token_count() == len(prompt) + n - 1
            assert_logits_close(eng.logits(), _oracle_logits_after(ora, prompt, toks[0][:-1]), f"{cfg.name} flags {flags}")
            nxt = eng.decode_step(int(toks[0][-1]))
            lg = eng.logits()
            assert lg[nxt] >= lg.max() - 1e-3  # the step's token is the arg-max of the logits the engine reports
            streams.append(toks[0])
            eng.close()
        # Both routes follow the oracle's arg-max except at its near ties, so they are identical up to the first position
        # where either met one (after that the two sequences are different inputs).
        first = min(near[0] + near[1] + [n])
        assert np.array_equal(streams[0][:first], streams[1][:first]), f"{cfg.name}: streams differ before the first near tie at {first}"


def _oracle_logits_after(ora, prompt, fed):
    assert ora.prefill(prompt) == 0
    for t in fed:
        assert ora.advance(int(t)) == 0
    return ora.logits()


def test_generation_limits_and_eos(rt, oracle_lib, tmp_models, tmp_path):
    import shutil
    from espresso_b200.model_config import MultiModelConfig, tiny_gpt2, tiny_llama

    cfg = tiny_llama(vocab=64, max_seq=24, n_layer=1)
    d = tmp_models(cfg)
    eng = rt.DecodeEngine.build(d)
    ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
    prompt = [3, 4, 5]
    res = eng.generate(prompt, 100)
    assert len(res.tokens) == 21  # clamped to maxSeq - prompt (Engine.swift:1425-1426)
    compare_greedy_stream(ora, prompt, res.tokens)
    assert len(eng.generate(prompt, 0).tokens) == 0
    with pytest.raises(rt.RealModelInferenceError):
        eng.generate(list(range(24)), 4)  # prompt must be shorter than the context
    with pytest.raises(rt.RealModelInferenceError):
        eng.generate([], 4)
    eng.close()
    # Llama EOS: the EOS token is emitted, then generation stops (Engine.swift:6385-6388)
    first = int(res.tokens[0])
    third = int(res.tokens[2])
    for case, (eos, expect) in enumerate(((first, 1), (third, None))):
        d2 = str(tmp_path / f"eos_case{case}")
        shutil.copytree(d, d2)
        dataclasses.replace(cfg, eosToken=eos).save(d2)
        e2 = rt.DecodeEngine.build(d2)
        out = e2.generate(prompt, 100)
        ref = oracle_lib.Runtime(oracle_lib.Model.from_dir(d2)).generate(prompt, 100)
        assert list(out.tokens) == list(ref)
        assert out.tokens[-1] == eos and out.stoppedOnEOS
        if expect:
            assert len(out.tokens) == expect
        e2.close()


def test_batched_decode_equals_independent_sequences(rt, oracle_lib, tmp_models):
    from espresso_b200.model_config import tiny_gpt2, tiny_llama
    from espresso_b200.synthetic import synthetic_prompt

    cases = ((tiny_llama(vocab=512, max_seq=64, n_layer=2), 1234), (tiny_gpt2(vocab=512, max_seq=64, n_layer=2), 777))
    for cfg, seed in cases:
        d = tmp_models(cfg, seed)
        model = oracle_lib.Model.from_dir(d)
        for n_seq in (5, 12):  # 5 rows: row-batched GEMV stages; 12 rows: tensor-core GEMM path
            prompts = np.stack([synthetic_prompt(cfg.vocab, 7, seed=seed, stream=s) for s in range(n_seq)])
            eng = rt.DecodeEngine.build(d, max_batch=n_seq)
            toks, res = eng.generate_batch(prompts, 12)
            for s in range(n_seq):
                assert len(toks[s]) == 12
                compare_greedy_stream(oracle_lib.Runtime(model), prompts[s], toks[s])
            # step API: logits of every sequence against the oracle
            eng.prefill_batch(prompts)
            nxt = eng.decode_step_batch(prompts[:, 0])
            for s in range(n_seq):
                ora = oracle_lib.Runtime(model)
                ora.prefill(list(prompts[s]) + [int(prompts[s, 0])])
                assert_logits_close(eng.logits(s), ora.logits(), f"{cfg.name} n_seq {n_seq} seq {s}")
                lg = eng.logits(s)
                assert lg[int(nxt[s])] >= lg.max() - 2e-3
            eng.close()


def test_verify2_checkpoint_and_two_token_generation(rt, oracle_lib, tmp_models):
    from espresso_b200.model_config import tiny_llama
    from espresso_b200.synthetic import synthetic_prompt

    cfg = tiny_llama(vocab=96, max_seq=48, n_layer=2)
    dcfg = tiny_llama(vocab=96, max_seq=48, n_layer=1)
    d, dd = tmp_models(cfg), tmp_models(dcfg, 1235)
    eng = rt.DecodeEngine.build(d)
    prompt = synthetic_prompt(cfg.vocab, 6)
    greedy = eng.generate(prompt, 24).tokens
    # verify2 = two sequential exact steps when the proposal is right; one when it is wrong
    eng.prefill(prompt)
    cur = eng.select_greedy_token()
    assert cur == greedy[0]
    nxt, fut = eng.verify2(cur, int(greedy[1]))
    assert (nxt, fut) == (greedy[1], greedy[2])
    eng.commit(2)
    assert eng.visible_token_count() == len(prompt) + 2 and eng.select_greedy_token() == greedy[2]
    wrong = (int(greedy[3]) + 1) % cfg.vocab
    nxt, _ = eng.verify2(int(greedy[2]), wrong)
    assert nxt == greedy[3]
    eng.commit(1)
    assert eng.select_greedy_token() == greedy[3]
    # checkpoint / rollback (Engine.swift:647-661)
    cp = eng.capture_checkpoint()
    before = eng.logits()
    eng.advance(7); eng.advance(9)
    eng.rollback(cp)
    assert eng.visible_token_count() == len(prompt) + 3
    np.testing.assert_array_equal(eng.logits(), before)
    assert eng.decode_step(int(greedy[3])) == greedy[4]
    # two-token generation emits the plain greedy stream, with any draft
    for draft_dir, expect_all in ((dd, False), (d, True)):
        draft = rt.DecodeEngine.build(draft_dir)
        res = eng.generate_two_token(draft, prompt, 24)
        assert list(res.tokens) == list(greedy)
        assert res.speculativePasses > 0
        if expect_all:
            assert res.acceptedFutureTokensPerPass > 0.8  # an identical draft is (almost) always accepted
        draft.close()
    ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
    compare_greedy_stream(ora, prompt, greedy)
    eng.close()


@pytest.mark.parametrize("kind", ["q8_0", "q4_0"])
def test_quantised_llama_matches_oracle_on_dequantised_weights(rt, oracle_lib, kind):
    from espresso_b200.model_config import MultiModelConfig
    from espresso_b200.synthetic import synthetic_prompt

    cfg = MultiModelConfig("tiny-gqa-q", 2, 8, 2, 256, 32, 512, 640, 96, 1e-5, 10000.0, None, "llama")
    model, uploads = quantised_pair(oracle_lib, cfg, kind)
    eng = rt.DecodeEngine.empty(cfg)
    upload_all(eng, uploads)
    ora = oracle_lib.Runtime(model)
    prompt = synthetic_prompt(cfg.vocab, 10)
    eng.prefill(prompt)
    assert ora.prefill(prompt) == 0
    assert_logits_close(eng.logits(), ora.logits(), kind)
    res = eng.generate(prompt, 40)
    compare_greedy_stream(ora, prompt, res.tokens)
    eng.close()


@pytest.mark.parametrize("kind", ["q8_0", "q4_0"])
def test_quantised_batch_uses_fp16_expansion_and_matches_oracle(rt, oracle_lib, kind):
    """12 sequences of a quantised model decode on the tensor cores against the fp16 expansion of the blocks."""
    from espresso_b200.model_config import MultiModelConfig
    from espresso_b200.synthetic import synthetic_prompt

    cfg = MultiModelConfig("tiny-gqa-qb", 2, 8, 2, 256, 32, 512, 640, 96, 1e-5, 10000.0, None, "llama")
    model, uploads = quantised_pair(oracle_lib, cfg, kind)
    n_seq = 12
    prompts = np.stack([synthetic_prompt(cfg.vocab, 9, seed=5, stream=s) for s in range(n_seq)])
    eng = rt.DecodeEngine.empty(cfg, max_batch=n_seq)
    upload_all(eng, uploads)
    toks, _ = eng.generate_batch(prompts, 16)
    for s in range(n_seq):
        compare_greedy_stream(oracle_lib.Runtime(model), prompts[s], toks[s])
    eng.prefill_batch(prompts)
    eng.decode_step_batch(prompts[:, 0])
    for s in (0, 7, 11):
        ora = oracle_lib.Runtime(model)
        ora.prefill(list(prompts[s]) + [int(prompts[s, 0])])
        assert_logits_close(eng.logits(s), ora.logits(), f"{kind} seq {s}")
    eng.close()


@pytest.mark.parametrize("n_head,n_kv,head_dim", [(16, 4, 64), (16, 16, 64), (12, 4, 128), (20, 20, 32), (10, 5, 64)])
def test_many_row_attention_kernels_in_a_prefill_chunk(rt, oracle_lib, tmp_models, n_head, n_kv, head_dim):
    """A 64-row prefill chunk with rows x heads >= 4 x SMs runs the many-row attention (multi-head and grouped-query
    shapes, head_dim 32 / 64 / 128): two warps per (row, head) when n_head is a multiple of 4, one warp otherwise."""
    from espresso_b200.model_config import MultiModelConfig
    from espresso_b200.synthetic import synthetic_prompt

    d = n_head * head_dim
    cfg = MultiModelConfig(f"att-{n_head}-{n_kv}-{head_dim}", 1, n_head, n_kv, d, head_dim, 2 * d if d <= 640 else d, 320, 160, 1e-5, 10000.0, None, "llama")
    if 64 * n_head < 4 * 148:
        pytest.skip("too few (row, head) pairs for the many-row kernels")
    wd = tmp_models(cfg)
    eng = rt.DecodeEngine.build(wd)
    ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(wd))
    prompt = synthetic_prompt(cfg.vocab, 100)  # chunks of 64 and 36 rows: the second one sees 64..99 cached positions
    eng.prefill(prompt)
    assert ora.prefill(prompt) == 0
    assert_logits_close(eng.logits(), ora.logits(), cfg.name)
    compare_greedy_stream(ora, prompt, eng.generate(prompt, 8).tokens)
    eng.close()


def test_token_emission_times_of_the_persistent_loop(rt, tmp_models):
    from espresso_b200.model_config import tiny_llama
    from espresso_b200.synthetic import synthetic_prompt

    cfg = tiny_llama(vocab=128, max_seq=64, n_layer=2)
    eng = rt.DecodeEngine.build(tmp_models(cfg))
    eng.prefill(synthetic_prompt(cfg.vocab, 5))
    toks, _ = eng.decode(20)
    t = eng.token_times_ns().astype(np.int64)
    assert t.size == 20 and np.all(np.diff(t) > 0)  # one stamp per token, strictly increasing
    assert np.diff(t).max() < 5_000_000  # a token of this model takes microseconds, not milliseconds
    ref = rt.DecodeEngine.build(tmp_models(cfg), flags=rt.FLAG_NO_MEGAKERNEL)
    ref.prefill(synthetic_prompt(cfg.vocab, 5))
    ref.decode(4)
    assert ref.token_times_ns().size == 0  # the per-stage kernels record no such stamps
    ref.close()
    eng.close()


@pytest.mark.parametrize("kind", ["f16", "q8_0"])
def test_persistent_kernel_streams_wide_stages_in_chunks(rt, oracle_lib, tmp_models, kind):
    """d_model 2048 / hidden 5632: every stage slice of the persistent kernel exceeds a ring slot and arrives in chunks
    (q/k/v pairs, Wo rows, gate/up pairs, down rows); the quantised variant packs the fp16 expansion of the blocks."""
    from espresso_b200.model_config import MultiModelConfig
    from espresso_b200.synthetic import synthetic_prompt

    cfg = MultiModelConfig("wide-gqa", 2, 32, 4, 2048, 64, 5632, 768, 64, 1e-5, 10000.0, None, "llama")
    prompt = synthetic_prompt(cfg.vocab, 12)
    if kind == "f16":
        d = tmp_models(cfg)
        eng = rt.DecodeEngine.build(d)
        ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
    else:
        model, uploads = quantised_pair(oracle_lib, cfg, kind)
        eng = rt.DecodeEngine.empty(cfg)
        upload_all(eng, uploads)
        ora = oracle_lib.Runtime(model)
    res = eng.generate(prompt, 24)
    assert eng.timings()["kernel_launches"] == 1  # the whole greedy loop was one persistent launch
    compare_greedy_stream(ora, prompt, res.tokens)
    # same tokens from the per-stage kernels
    flags = rt.FLAG_NO_MEGAKERNEL
    if kind == "f16":
        ref = rt.DecodeEngine.build(tmp_models(cfg), flags=flags)
    else:
        ref = rt.DecodeEngine.empty(cfg, flags=flags)
        upload_all(ref, uploads)
    compare_greedy_stream(ora, prompt, ref.generate(prompt, 24).tokens)
    ref.close()
    eng.close()


def test_long_context_split_kv_attention(rt, oracle_lib, tmp_models):
    """Positions beyond one attention split (256) exercise the split-KV merge."""
    from espresso_b200.model_config import MultiModelConfig
    from espresso_b200.synthetic import synthetic_prompt

    cfg = MultiModelConfig("tiny-long", 1, 4, 2, 128, 32, 256, 256, 640, 1e-5, 10000.0, None, "llama")
    d = tmp_models(cfg)
    eng = rt.DecodeEngine.build(d)
    ora = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
    prompt = synthetic_prompt(cfg.vocab, 600)
    eng.prefill(prompt)
    assert ora.prefill(prompt) == 0
    assert_logits_close(eng.logits(), ora.logits(), "600-token context")
    eng.close()


def test_error_codes_and_test_hooks(rt, tmp_models):
    from espresso_b200.model_config import tiny_llama

    cfg = tiny_llama(vocab=64, max_seq=8, n_layer=1)
    before = rt.live_engine_count()
    eng = rt.DecodeEngine.build(tmp_models(cfg))
    assert rt.live_engine_count() == before + 1
    eng.prefill([1, 2])
    with pytest.raises(rt.RealModelInferenceError) as ei:
        eng.advance(64)  # token outside vocab (Engine.swift:687-689)
    assert ei.value.status == rt.ERR_OUT_OF_RANGE
    for t in range(6):
        eng.advance(t)
    with pytest.raises(rt.RealModelInferenceError) as ei:
        eng.advance(0)  # context full (Engine.swift:673-677)
    assert ei.value.status == rt.ERR_OUT_OF_RANGE
    with pytest.raises(rt.RealModelInferenceError):
        eng.prefill([])
    # forced failure hook (ane_interop_set_force_eval_failure, ane_interop.h:37-41)
    rt.set_force_failure(True)
    try:
        with pytest.raises(rt.RealModelInferenceError) as ei:
            eng.prefill([1])
        assert ei.value.status == rt.ERR_FORCED_FAILURE
    finally:
        rt.set_force_failure(False)
    eng.prefill([1])
    eng.close()
    assert rt.live_engine_count() == before
    # missing directory / missing tensor / wrong size
    with pytest.raises(rt.RealModelInferenceError) as ei:
        rt.DecodeEngine.build("/nonexistent/dir", config=cfg)
    assert ei.value.status == rt.ERR_IO
    e2 = rt.DecodeEngine.empty(cfg)
    with pytest.raises(rt.RealModelInferenceError) as ei:
        e2.load_tensor("rms_final", "f16", np.ones(3, np.float16))
    assert ei.value.status == rt.ERR_INVALID_WEIGHTS
    with pytest.raises(rt.RealModelInferenceError) as ei:
        e2.finalize()
    assert ei.value.status == rt.ERR_INVALID_WEIGHTS
    with pytest.raises(rt.RealModelInferenceError) as ei:
        e2.prefill([1])
    assert ei.value.status == rt.ERR_STATE
    e2.close()

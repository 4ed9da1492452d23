"""Known-answer tests that pin the CPU oracle.

Each case restates a test of the reference's own suite (cited by file:line inside the Espresso
project) or checks the oracle against golden vectors produced by independent implementations
(HuggingFace through the reference's Python bridge; the ``gguf`` package).
"""
import math
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def softmax_ctx(logits_by_head, values):
    out = []
    for logits in logits_by_head:
        m = max(logits)
        w = [math.exp(x - m) for x in logits]
        s = sum(w)
        out.extend(sum(wi / s * v[t] for t, wi in enumerate(w)) for v in values)
    return out


def test_rope_half_split_kat(oracle_lib):
    # Tests/CPUOpsTests/RoPEDecodeStepTests.swift:5-43
    q = oracle_lib.rope_half_split([1, 2, 3, 4], 1, 4, 1)
    k = oracle_lib.rope_half_split([5, 6, 7, 8], 1, 4, 1)
    c0, s0, c1, s1 = math.cos(1.0), math.sin(1.0), math.cos(0.01), math.sin(0.01)
    np.testing.assert_allclose(q, [1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 1 * s0 + 3 * c0, 2 * s1 + 4 * c1], atol=1e-5)
    np.testing.assert_allclose(k, [5 * c0 - 7 * s0, 6 * c1 - 8 * s1, 5 * s0 + 7 * c0, 6 * s1 + 8 * c1], atol=1e-5)


def test_rope_position_zero_is_identity_and_theta_matters(oracle_lib):
    # RoPEDecodeStepTests.swift:46-170
    v = np.array([(i % 7) * 0.1 - 0.3 for i in range(32)], np.float32)
    np.testing.assert_allclose(oracle_lib.rope_half_split(v, 4, 8, 0), v, atol=1e-6)
    ones = np.ones(8, np.float32)
    assert np.abs(oracle_lib.rope_half_split(ones, 2, 4, 5) - ones).max() > 1e-6
    a = oracle_lib.rope_half_split(ones, 2, 4, 10, 10000.0)
    b = oracle_lib.rope_half_split(ones, 2, 4, 10, 500000.0)
    assert np.abs(a - b).max() > 1e-6


def test_rmsnorm_known_values(oracle_lib):
    # Tests/CPUOpsTests/CPUOpsTests.swift:169-208 (eps 1e-5, unit weights), per token
    for x in ([1, 3, 5, 7], [2, 4, 6, 8]):
        x = np.array(x, np.float32)
        rr = 1.0 / math.sqrt(float((x * x).sum()) / 4 + 1e-5)
        np.testing.assert_allclose(oracle_lib.rmsnorm(x, np.ones(4), 1e-5), x * rr, atol=1e-5)


def test_per_head_rmsnorm_manual_reference(oracle_lib):
    # Tests/CPUOpsTests/RMSNormPerHeadDecodeTests.swift:5-52
    vals = [1.0, -2.0, 0.5, 1.5, 2.0, 0.0, -1.0, 3.0]
    w = [1.0, 0.5, 1.5, 2.0]
    got = oracle_lib.per_head_rmsnorm(vals, w, 2, 4, 1e-6)
    exp = []
    for h in range(2):
        hv = vals[h * 4:(h + 1) * 4]
        inv = 1.0 / math.sqrt(sum(v * v for v in hv) / 4 + 1e-6)
        exp += [v * inv * wi for v, wi in zip(hv, w)]
    np.testing.assert_allclose(got, exp, atol=1e-6)


def test_silu_tanh_form(oracle_lib):
    # Tests/RealModelInferenceTests/RealModelInferenceTests.swift:223-229
    for s in (-8, -1.25, 0, 0.75, 6):
        assert abs(oracle_lib.silu(s) - 0.5 * s * (1 + math.tanh(0.5 * s))) < 1e-6
        if s != 0:
            assert abs(oracle_lib.silu(s) - s / (1 + math.exp(-s))) < 1e-5  # Sources/CPUOps/SiLU.swift:6-8


def test_gelu_tanh_approximation(oracle_lib):
    for s in (-3.0, -0.5, 0.0, 0.3, 2.5):
        exp = 0.5 * s * (1 + math.tanh(0.7978846 * (s + 0.044715 * s ** 3)))
        assert abs(oracle_lib.gelu(s) - exp) < 1e-6


def test_layernorm_matches_numpy(oracle_lib):
    rng = np.random.default_rng(3)
    x, g, b = rng.standard_normal(96), rng.standard_normal(96), rng.standard_normal(96)
    exp = (x - x.mean()) / np.sqrt(x.var() + 1e-5) * g + b
    np.testing.assert_allclose(oracle_lib.layernorm(x, g, b, 1e-5), exp, atol=2e-5)


def test_decode_context_grouped_contiguous(oracle_lib):
    # Tests/EspressoTests/HybridDecodeForwardPassTests.swift:97-131
    ctx = oracle_lib.decode_context([1, 2, 3, 4], [1, 2, 0, 1], [10, 20, 30, 40], 2, 1, 2, 2, 2)
    s = 1 / math.sqrt(2.0)
    exp = softmax_ctx([[1 * s, 4 * s], [3 * s, 10 * s]], [[10, 20], [30, 40]])
    np.testing.assert_allclose(ctx, exp, atol=1e-5)


def test_decode_context_gqa_mapping_is_grouped(oracle_lib):
    # HybridDecodeForwardPassTests.swift:133-211: with 4 heads / 2 kv heads, heads 0,1 -> kv 0; 2,3 -> kv 1
    q = [1, 0, 0, 1, 0, 1, 1, 0]
    k = [1, 0, 0, 1, 0, 1, 1, 0]
    v = [10, 20, 30, 40, 50, 60, 70, 80]
    ctx = oracle_lib.decode_context(q, k, v, 4, 2, 2, 2, 2)
    s = 1 / math.sqrt(2.0)

    def head(qh, kvh):
        kk = [[k[(kvh * 2 + d) * 2 + t] for d in range(2)] for t in range(2)]
        logits = [sum(qh[d] * kk[t][d] for d in range(2)) * s for t in range(2)]
        return softmax_ctx([logits], [[v[(kvh * 2 + d) * 2 + t] for t in range(2)] for d in range(2)])

    exp = head(q[0:2], 0) + head(q[2:4], 0) + head(q[4:6], 1) + head(q[6:8], 1)
    np.testing.assert_allclose(ctx, exp, atol=1e-5)


def test_decode_context_suffix_window(oracle_lib):
    # HybridDecodeForwardPassTests.swift:213-238
    ctx = oracle_lib.decode_context([1], [0, 1, 2, 3], [10, 20, 30, 40], 1, 1, 1, 2, 4, token_base=2)
    np.testing.assert_allclose(ctx, softmax_ctx([[2.0, 3.0]], [[30, 40]]), atol=1e-5)


def test_decode_context_respects_visible_count(oracle_lib):
    # Tests/RealModelInferenceTests/RealModelInferenceTests.swift:835-870
    causal = oracle_lib.decode_context([1, 0], [1, 100, 0, 0], [5, 99, 7, 123], 1, 1, 2, 1, 2)
    full = oracle_lib.decode_context([1, 0], [1, 100, 0, 0], [5, 99, 7, 123], 1, 1, 2, 2, 2)
    assert causal[0] == 5 and causal[1] == 7
    assert abs(full[0] - 99) < 0.01 and abs(full[1] - 123) < 0.01


def test_argmax_first_max_tie_rule(oracle_lib):
    # Sources/ANEInterop/neon_convert.c:61-83; Tests/ANEInteropTests/ANEInteropTests.swift:199
    assert oracle_lib.argmax_first([1, 5, 5, 2]) == 1
    assert oracle_lib.argmax_first([-3, -3, -3]) == 0
    assert oracle_lib.argmax_first([0, 1, 2, 9]) == 3


def test_partitioned_argmax_equals_naive(oracle_lib):
    # Tests/EspressoTests/PartitionedArgmaxTests.swift:8-115, FP16TiledClassifierTests.swift:8-108
    rng = np.random.default_rng(11)
    for vocab, dim, block in ((1000, 64, 128), (4097, 32, 4000), (50, 16, 7)):
        w = rng.standard_normal((vocab, dim)).astype(np.float32)
        w[vocab // 3] *= 4  # a dominant row lets the pruning rule actually skip blocks
        x = rng.standard_normal(dim).astype(np.float32)
        naive = int(np.argmax(oracle_lib.gemv(w, x)))
        assert oracle_lib.partitioned_argmax(w, x, block) == naive
    w = np.zeros((9, 4), np.float32)
    w[2] = w[7] = 1.0
    assert oracle_lib.partitioned_argmax(w, np.ones(4), 4) == 2  # equal maxima: first index wins


def test_blobfile_header_and_roundtrip(oracle_lib, tmp_path):
    # Tests/ANETypesTests/ANETypesTests.swift:117-258, Tests/ModelSupportTests/BlobWeightLoaderTests.swift:6-41
    from espresso_b200 import weight_blob as wb

    vals = np.array([1.0, -2.5, 0.125, 65504.0], np.float16)
    p = str(tmp_path / "t.bin")
    assert oracle_lib.blob_write(p, vals.view(np.uint16)) == 0
    raw = open(p, "rb").read()
    assert len(raw) == 128 + 8 and raw[0] == 1 and raw[4] == 2 and raw[64:68] == b"\xEF\xBE\xAD\xDE" and raw[68] == 1
    assert int.from_bytes(raw[72:76], "little") == 8 and int.from_bytes(raw[80:84], "little") == 128
    assert raw[:128] == wb.make_header(8)
    n, back = oracle_lib.blob_read(p)
    assert n == 4 and np.array_equal(back, vals.astype(np.float32))
    np.testing.assert_array_equal(wb.read_blob(p), back)
    # package writer == oracle writer
    p2 = str(tmp_path / "u.bin")
    wb.write_blob(p2, vals)
    assert open(p2, "rb").read() == raw
    # error cases: truncated header, bad magic, bad offset, truncated payload
    open(p, "wb").write(raw[:100])
    assert oracle_lib.blob_read(p)[0] == -2
    with pytest.raises(wb.BlobWeightLoaderError):
        wb.read_blob(p)
    bad = bytearray(raw); bad[64] = 0
    open(p, "wb").write(bad)
    assert oracle_lib.blob_read(p)[0] == -3
    bad = bytearray(raw); bad[80] = 64
    open(p, "wb").write(bad)
    assert oracle_lib.blob_read(p)[0] == -4
    open(p, "wb").write(raw[:-2])
    assert oracle_lib.blob_read(p)[0] == -5


def test_fp16_conversion_matches_numpy(oracle_lib):
    rng = np.random.default_rng(5)
    vals = np.concatenate([rng.standard_normal(2000) * 10 ** rng.uniform(-9, 5, 2000), [0.0, -0.0, 65504, 65520, 1e-8, 6.1e-5]]).astype(np.float32)
    L = oracle_lib.lib()
    for v in vals:
        assert L.esp_oracle_float_to_half(float(v)) == int(np.float16(v).view(np.uint16)), v
    for bits in rng.integers(0, 0x7C00, 500):
        assert L.esp_oracle_half_to_float(int(bits)) == float(np.uint16(bits).view(np.float16))


def test_float32_sidecar_is_preferred(oracle_lib, tmp_models, tmp_path):
    # Tests/RealModelInferenceTests/RealModelInferenceTests.swift:318-389
    import shutil
    from espresso_b200.model_config import tiny_llama

    cfg = tiny_llama(vocab=64, max_seq=16, n_layer=1)
    d = str(tmp_path / "m")
    shutil.copytree(tmp_models(cfg), d)
    base = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
    base.prefill([1, 2, 3])
    g = np.full(cfg.dModel, 2.0, "<f4")
    g.tofile(os.path.join(d, "rms_final.float32.bin"))
    side = oracle_lib.Runtime(oracle_lib.Model.from_dir(d))
    side.prefill([1, 2, 3])
    np.testing.assert_allclose(side.logits(), 2.0 * base.logits(), rtol=1e-6, atol=1e-7)


def test_two_token_plan(oracle_lib):
    # Sources/Espresso/GenerationHarness.swift:149-181; Tests/EspressoTests/GenerationHarnessTests.swift:482-620
    assert oracle_lib.two_token_plan(5, 9, 9, 11, 4) == ([5, 9], 11)
    assert oracle_lib.two_token_plan(5, 8, 9, 11, 4) == ([5], 9)
    assert oracle_lib.two_token_plan(5, 9, 9, 11, 1) == ([5], 9)


def test_quantisers_match_gguf_golden(oracle_lib):
    from espresso_b200 import gguf_quant as gq

    g = np.load(os.path.join(GOLD, "gguf_blocks.npz"))
    x = g["x"]
    for kind in ("q8_0", "q4_0"):
        blocks = g[kind + "_blocks"]
        assert np.array_equal(oracle_lib.quantize(kind, x), blocks)
        assert np.array_equal(gq.quantize(kind, x), blocks)
        deq = g[kind + "_dequant"]
        assert np.array_equal(oracle_lib.dequantize(kind, blocks, x.size).view(np.uint32), deq.view(np.uint32))
        assert np.array_equal(gq.dequantize(kind, blocks).view(np.uint32), deq.view(np.uint32))


def test_llama_oracle_matches_hf_golden(oracle_lib, tmp_models):
    from espresso_b200.model_config import tiny_llama

    g = np.load(os.path.join(GOLD, "hf_llama_tiny.npz"))
    for tag, gqa in (("gqa", True), ("mha", False)):
        cfg = tiny_llama(vocab=512, max_seq=64, n_layer=2, gqa=gqa)
        r = oracle_lib.Runtime(oracle_lib.Model.from_dir(tmp_models(cfg, int(g[tag + "_seed"]))))
        r.reset()
        for i, t in enumerate(g[tag + "_prompt"]):
            assert r.advance(int(t)) == 0
            np.testing.assert_allclose(r.logits(), g[tag + "_logits"][i], atol=5e-6)


def test_gpt2_oracle_matches_hf_golden(oracle_lib, tmp_models):
    from espresso_b200.model_config import tiny_gpt2

    g = np.load(os.path.join(GOLD, "hf_gpt2_tiny.npz"))
    cfg = tiny_gpt2(vocab=512, max_seq=64, n_layer=2)
    r = oracle_lib.Runtime(oracle_lib.Model.from_dir(tmp_models(cfg, int(g["seed"]))))
    r.reset()
    for i, t in enumerate(g["prompt"]):
        assert r.advance(int(t)) == 0
        np.testing.assert_allclose(r.logits(), g["logits"][i], atol=5e-6)


def test_runtime_guards_and_generation_limits(oracle_lib, tmp_models):
    # position/token guards RealModelInferenceEngine.swift:673-689; limits :1419-1426; EOS rule :6385-6388
    import dataclasses
    from espresso_b200.model_config import tiny_llama

    cfg = tiny_llama(vocab=64, max_seq=8, n_layer=1)
    m = oracle_lib.Model.from_dir(tmp_models(cfg))
    r = oracle_lib.Runtime(m)
    assert r.prefill([]) != 0
    assert r.prefill([1, 2]) == 0 and r.visible == 2
    assert r.advance(64) == -2  # token outside vocab
    for t in range(6):
        assert r.advance(t) == 0
    assert r.advance(0) == -1  # context full
    toks = r.generate([3, 4, 5], 100)
    assert len(toks) == 5  # clamped to maxSeq - prompt
    with pytest.raises(RuntimeError):
        r.generate(list(range(8)), 4)  # prompt must be shorter than maxSeq
    # EOS: the token is appended, then generation stops
    first = int(toks[0])
    meta = dataclasses.replace(cfg, eosToken=first).to_metadata()
    m2 = oracle_lib.Model(meta)
    from espresso_b200.synthetic import synthetic_tensors
    for name, v in synthetic_tensors(cfg):
        m2.set_tensor(name, v.astype(np.float32))
    assert list(oracle_lib.Runtime(m2).generate([3, 4, 5], 100)) == [first]


def test_checkpoint_rollback_and_two_token_equals_greedy(oracle_lib, tmp_models):
    # RealModelInferenceEngine.swift:647-661 and :6014-6190: the two-token loop emits the plain greedy stream
    from espresso_b200.model_config import tiny_llama

    cfg = tiny_llama(vocab=96, max_seq=48, n_layer=2)
    draft_cfg = tiny_llama(vocab=96, max_seq=48, n_layer=1)
    full = oracle_lib.Runtime(oracle_lib.Model.from_dir(tmp_models(cfg)))
    draft = oracle_lib.Runtime(oracle_lib.Model.from_dir(tmp_models(draft_cfg, 1235)))
    prompt = [5, 17, 3, 80]
    greedy = full.generate(prompt, 20)
    full.prefill(prompt)
    cp = full.checkpoint()
    before = full.logits()
    full.advance(7); full.advance(9)
    full.rollback(cp)
    full.free_checkpoint(cp)
    assert full.visible == 4 and np.array_equal(full.logits(), before)
    toks, stats = oracle_lib.generate_two_token(full, draft, prompt, 20)
    assert np.array_equal(toks, greedy)
    assert stats["passes"] > 0 and stats["committed"] == len(toks) - 1
    # a draft identical to the target accepts every proposal
    twin = oracle_lib.Runtime(oracle_lib.Model.from_dir(tmp_models(cfg)))
    toks2, stats2 = oracle_lib.generate_two_token(full, twin, prompt, 21)
    assert np.array_equal(toks2[:20], greedy) and stats2["accepted"] == stats2["committed"]

"""GGUF front end: the library's own parser against the `gguf` package's reader, error kinds, and (on a GPU) an engine
built straight from a file against the oracle on the values the file decodes to."""
import os

import numpy as np
import pytest

gguf = pytest.importorskip("gguf")

from gguf_fixture import write_gguf  # noqa: E402
from helpers import assert_logits_close, compare_greedy_stream  # noqa: E402


@pytest.fixture(scope="module")
def rt():
    from espresso_b200 import runtime

    runtime.load_library()
    return runtime


def tiny_cfg(arch="llama", **kw):
    from espresso_b200.model_config import MultiModelConfig

    if arch == "gpt2":
        return MultiModelConfig("tiny-gpt2-gguf", 2, 4, 4, 128, 32, 512, 320, 64, 1e-5, 10000.0, None, "gpt2")
    return MultiModelConfig("tiny-llama-gguf", 2, 8, 2, 256, 32, 512, 384, 96, 1e-5, kw.get("theta", 50000.0), kw.get("eos"), "llama")


@pytest.mark.parametrize("arch_name,kind,tied", [("llama", "q8_0", False), ("qwen2", "q4_0", True), ("gpt2", "f16", False)])
def test_inspect_and_directory_match_the_gguf_package(rt, tmp_path, arch_name, kind, tied):
    cfg = tiny_cfg("gpt2" if arch_name == "gpt2" else "llama", eos=7)
    path = str(tmp_path / "m.gguf")
    write_gguf(path, cfg, kind, arch_name=arch_name, tied=tied)
    got, name, n_tensors, is_tied = rt.gguf_inspect(path)
    assert name == arch_name and is_tied == tied
    for f in ("nLayer", "nHead", "nKVHead", "dModel", "headDim", "hiddenDim", "vocab", "maxSeq", "architecture", "eosToken"):
        assert getattr(got, f) == getattr(cfg, f), f
    assert abs(got.normEps - cfg.normEps) < 1e-12 and abs(got.ropeTheta - (cfg.ropeTheta if cfg.architecture == "llama" else 10000.0)) < 1e-3
    reader = gguf.GGUFReader(path)
    assert n_tensors == len(reader.tensors)
    mine = {t["name"]: t for t in rt.gguf_tensors(path)}
    for t in reader.tensors:
        m = mine[t.name]
        assert m["type"] == int(t.tensor_type) and m["nbytes"] == int(t.n_bytes)
        assert m["dims"][: len(t.shape)] == [int(d) for d in t.shape]
        assert m["offset"] == int(t.data_offset) - int(reader.data_offset)
    # name mapping (Sources/ModelSupport/LayerWeightPaths.swift:22-77)
    if arch_name == "gpt2":
        assert mine["blk.1.attn_qkv.weight"]["slot"] == "layers/1/wqkv" and mine["blk.0.ffn_up.weight"]["slot"] == "layers/0/w1"
        assert mine["position_embd.weight"]["slot"] == "embeddings/position" and mine["output_norm.bias"]["slot"] == "final_norm_beta"
    else:
        assert mine["blk.1.attn_v.weight"]["slot"] == "layers/1/wv" and mine["blk.0.ffn_gate.weight"]["slot"] == "layers/0/w1"
        assert mine["blk.0.ffn_up.weight"]["slot"] == "layers/0/w3" and mine["output_norm.weight"]["slot"] == "rms_final"
        assert ("output.weight" in mine) == (not tied)


def test_gguf_error_kinds(rt, tmp_path):
    cfg = tiny_cfg()
    good = str(tmp_path / "good.gguf")
    write_gguf(good, cfg, "q8_0")
    raw = open(good, "rb").read()
    cases = {"bad_magic": b"GGUX" + raw[4:], "bad_version": raw[:4] + (9).to_bytes(4, "little") + raw[8:], "truncated": raw[:200],
             "cut_data": raw[: len(raw) - 4096]}
    for name, blob in cases.items():
        p = str(tmp_path / f"{name}.gguf")
        open(p, "wb").write(blob)
        with pytest.raises(rt.RealModelInferenceError) as ei:
            rt.gguf_inspect(p)
        assert ei.value.status == rt.ERR_INVALID_WEIGHTS, name
    # crafted tensor directory entries: an offset near 2^64 (offset + size wraps around) and dimensions whose product
    # overflows 64 bits must be refused, not turned into a wild host pointer
    name = b"token_embd.weight"
    at = raw.index(name) + len(name)
    n_dims = int.from_bytes(raw[at:at + 4], "little")
    dims_at, off_at = at + 4, at + 4 + 8 * n_dims + 4
    wild = bytearray(raw)
    wild[off_at:off_at + 8] = (2**64 - 32).to_bytes(8, "little")
    huge = bytearray(raw)
    for k in range(n_dims):
        huge[dims_at + 8 * k:dims_at + 8 * k + 8] = (2**40 + 32 * 1024).to_bytes(8, "little")
    for label, blob in (("wrapping_offset", wild), ("overflowing_dims", huge)):
        p = str(tmp_path / f"{label}.gguf")
        open(p, "wb").write(bytes(blob))
        with pytest.raises(rt.RealModelInferenceError) as ei:
            rt.gguf_inspect(p)
        assert ei.value.status == rt.ERR_INVALID_WEIGHTS, label
    with pytest.raises(rt.RealModelInferenceError) as ei:
        rt.gguf_inspect(str(tmp_path / "absent.gguf"))
    assert ei.value.status == rt.ERR_IO
    unsupported = str(tmp_path / "arch.gguf")
    write_gguf(unsupported, cfg, "f16", arch_name="falcon")
    with pytest.raises(rt.RealModelInferenceError) as ei:
        rt.gguf_inspect(unsupported)  # unsupportedArchitecture, GGUFModelLoader.swift:303-305
    assert "unsupported GGUF architecture" in str(ei.value)


@pytest.mark.gpu
@pytest.mark.parametrize("arch_name,kind,tied,quant_emb", [("llama", "q8_0", False, False), ("llama", "q4_0", True, True),
                                                          ("qwen2", "q8_0", True, False), ("gpt2", "f16", False, False)])
def test_engine_from_gguf_matches_oracle(rt, oracle_lib, tmp_path, arch_name, kind, tied, quant_emb):
    from espresso_b200.synthetic import synthetic_prompt

    cfg = tiny_cfg("gpt2" if arch_name == "gpt2" else "llama")
    model = oracle_lib.Model(cfg.to_metadata())
    path = str(tmp_path / "m.gguf")
    write_gguf(path, cfg, kind, oracle_model=model, arch_name=arch_name, tied=tied, quantise_embedding=quant_emb)
    eng = rt.DecodeEngine.from_gguf(path)
    ora = oracle_lib.Runtime(model)
    prompt = synthetic_prompt(cfg.vocab, 6)  # short: the single-row kernels read the quantised blocks
    eng.prefill(prompt)
    assert ora.prefill(prompt) == 0
    assert_logits_close(eng.logits(), ora.logits(), f"{arch_name} {kind}")
    compare_greedy_stream(ora, prompt, eng.generate(prompt, 24).tokens)
    eng.close()

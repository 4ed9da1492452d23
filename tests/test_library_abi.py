"""CPU-side checks of the boundary: the shared library loads, exports every symbol the public header
declares, and fails cleanly (status code + message, no crash) when no GPU is present."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "espresso_cuda.h")).read()
    return sorted(set(re.findall(r"ESP_CUDA_API\s+[\w\s\*]+?\b(esp_cuda_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from espresso_b200 import build, runtime

    build.build()
    lib = runtime.load_library()
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/espresso_cuda.h but not exported"
        assert n in runtime.SIGNATURES, f"{n} has no ctypes signature in espresso_b200/runtime.py"
    assert set(runtime.SIGNATURES) == set(names)


def test_calls_fail_cleanly_without_engine_or_gpu():
    import torch
    from espresso_b200 import runtime
    from espresso_b200.model_config import tiny_llama

    lib = runtime.load_library()
    assert lib.esp_cuda_version().startswith(b"espresso-cuda")
    assert lib.esp_cuda_reset(None) == runtime.ERR_INVALID_ARGUMENT
    assert b"null engine" in lib.esp_cuda_last_error_string()
    out = C.c_void_p()
    assert lib.esp_cuda_create(None, None, C.byref(out)) == runtime.ERR_INVALID_ARGUMENT
    if not torch.cuda.is_available():
        with pytest.raises(runtime.RealModelInferenceError) as ei:
            runtime.DecodeEngine.empty(tiny_llama())
        assert ei.value.status == runtime.ERR_CUDA  # no CPU fallback: the call fails loudly
    bad = runtime.make_c_config(tiny_llama())
    bad.n_kv_head = 3
    assert lib.esp_cuda_create(C.byref(bad), None, C.byref(out)) == runtime.ERR_INVALID_ARGUMENT


def test_metadata_roundtrip_and_validation(tmp_path):
    from espresso_b200.model_config import MultiModelConfig, llama_6l

    cfg = llama_6l()
    cfg.save(str(tmp_path))
    assert MultiModelConfig.load(str(tmp_path)) == cfg
    meta = cfg.to_metadata()
    del meta["ropeTheta"]
    assert MultiModelConfig.from_metadata(meta).ropeTheta == 10000.0  # ESPModelConfigIO.swift:53
    meta["architecture"] = "mamba"
    with pytest.raises(ValueError):
        MultiModelConfig.from_metadata(meta)
    # algorithmic bytes of the 6-layer benchmark shape
    assert cfg.weight_bytes_per_step() == 134108160
    assert cfg.kv_bytes_per_visible_token() == 18432

"""Seeded synthetic models and prompts.

Real checkpoints are not available offline, so every configuration is exercised with weights drawn
i.i.d. from N(0, 0.02) in fp32 (numpy Philox, one stream per tensor keyed by the seed and the tensor
name), rounded once to fp16 (or bf16) and written in the reference's weight-directory layout so that
the CUDA library and the CPU oracle read identical bits.  Norm gains are 1, LayerNorm betas 0, GPT-2
linear biases N(0, 0.02), and the GPT-2 LM head is a copy of the token embedding (tied by value).
Default seed 1234 is the reference CLI's default (Sources/EspressoGenerate/CLI.swift:40).
"""
from __future__ import annotations

import hashlib
import os

import numpy as np

from .model_config import MultiModelConfig
from .weight_blob import tensor_shapes, write_blob

DEFAULT_SEED = 1234
WEIGHT_STD = 0.02


def _rng(seed: int, name: str) -> np.random.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    key = int.from_bytes(digest[:16], "little")
    return np.random.Generator(np.random.Philox(key=key))


def synthetic_tensor(cfg: MultiModelConfig, name: str, shape: tuple[int, ...], seed: int = DEFAULT_SEED) -> np.ndarray:
    """fp32 values of one tensor before rounding to the storage type."""
    leaf = name.rsplit("/", 1)[-1]
    if leaf in ("rms_att", "rms_ffn", "rms_final", "ln_1_gamma", "ln_2_gamma", "final_norm_gamma"):
        return np.ones(shape, np.float32)
    if leaf in ("ln_1_beta", "ln_2_beta", "final_norm_beta"):
        return np.zeros(shape, np.float32)
    if leaf == "lm_head" and cfg.architecture == "gpt2":
        return synthetic_tensor(cfg, "embeddings/token", shape, seed)
    return (_rng(seed, name).standard_normal(shape, dtype=np.float32) * np.float32(WEIGHT_STD)).astype(np.float32)


def synthetic_tensors(cfg: MultiModelConfig, seed: int = DEFAULT_SEED):
    """Yield ``(name, fp16 array)`` for every tensor of the model."""
    for name, shape in tensor_shapes(cfg).items():
        yield name, synthetic_tensor(cfg, name, shape, seed).astype(np.float16)


def write_synthetic_model(cfg: MultiModelConfig, weight_dir: str, seed: int = DEFAULT_SEED) -> str:
    """Write ``metadata.json`` and one BLOBFILE per tensor; returns ``weight_dir``."""
    cfg.validate()
    cfg.save(weight_dir)
    for name, values in synthetic_tensors(cfg, seed):
        write_blob(os.path.join(weight_dir, name + ".bin"), values)
    return weight_dir


def synthetic_prompt(vocab: int, length: int, seed: int = DEFAULT_SEED, stream: int = 0) -> np.ndarray:
    """Token ids uniform in [0, vocab)."""
    return _rng(seed, f"prompt:{stream}").integers(0, vocab, size=length, dtype=np.uint32)

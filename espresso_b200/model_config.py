"""Model shape description and ``metadata.json`` I/O.

Mirrors ``MultiModelConfig`` (Sources/ModelSupport/MultiModelConfig.swift:3-55) and the
``metadata.json`` schema of ``ESPModelConfigIO`` (Sources/ESPCompiler/ESPModelConfigIO.swift:12-59):
keys ``name,nLayer,nHead,nKVHead,dModel,headDim,hiddenDim,vocab,maxSeq,normEps,ropeTheta?,eosToken?,
architecture``; ``ropeTheta`` defaults to 10000 when absent.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Optional


@dataclasses.dataclass(frozen=True)
class MultiModelConfig:
    name: str
    nLayer: int
    nHead: int
    nKVHead: int
    dModel: int
    headDim: int
    hiddenDim: int
    vocab: int
    maxSeq: int
    normEps: float
    ropeTheta: float = 10000.0
    eosToken: Optional[int] = None
    architecture: str = "llama"  # "llama" | "gpt2"

    @property
    def attentionDim(self) -> int:
        return self.nHead * self.headDim

    @property
    def kvDim(self) -> int:
        return self.nKVHead * self.headDim

    def validate(self) -> None:
        """Same rules as ``validateConfig`` (RealModelInferenceEngine.swift:7615-7634)."""
        for key in ("nLayer", "nHead", "nKVHead", "dModel", "headDim", "hiddenDim", "vocab", "maxSeq"):
            if getattr(self, key) <= 0:
                raise ValueError(f"invalid config: {key} must be > 0")
        if self.nHead % self.nKVHead != 0:
            raise ValueError("invalid config: nHead must be a multiple of nKVHead")
        if self.architecture not in ("llama", "gpt2"):
            raise ValueError(f"Unsupported metadata architecture: {self.architecture}")

    def to_metadata(self) -> dict:
        meta = {
            "name": self.name, "nLayer": self.nLayer, "nHead": self.nHead, "nKVHead": self.nKVHead,
            "dModel": self.dModel, "headDim": self.headDim, "hiddenDim": self.hiddenDim, "vocab": self.vocab,
            "maxSeq": self.maxSeq, "normEps": self.normEps, "ropeTheta": self.ropeTheta,
            "architecture": self.architecture,
        }
        if self.eosToken is not None:
            meta["eosToken"] = self.eosToken
        return meta

    @classmethod
    def from_metadata(cls, meta: dict) -> "MultiModelConfig":
        arch = str(meta["architecture"]).lower()
        if arch not in ("llama", "gpt2"):
            raise ValueError(f"Unsupported metadata architecture: {meta['architecture']}")
        cfg = cls(
            name=meta["name"], nLayer=int(meta["nLayer"]), nHead=int(meta["nHead"]), nKVHead=int(meta["nKVHead"]),
            dModel=int(meta["dModel"]), headDim=int(meta["headDim"]), hiddenDim=int(meta["hiddenDim"]),
            vocab=int(meta["vocab"]), maxSeq=int(meta["maxSeq"]), normEps=float(meta["normEps"]),
            ropeTheta=float(meta.get("ropeTheta") or 10000.0),
            eosToken=None if meta.get("eosToken") is None else int(meta["eosToken"]), architecture=arch,
        )
        cfg.validate()
        return cfg

    @classmethod
    def load(cls, weight_dir: str) -> "MultiModelConfig":
        with open(os.path.join(weight_dir, "metadata.json")) as f:
            return cls.from_metadata(json.load(f))

    def save(self, weight_dir: str) -> None:
        os.makedirs(weight_dir, exist_ok=True)
        with open(os.path.join(weight_dir, "metadata.json"), "w") as f:
            json.dump(self.to_metadata(), f, indent=2, sort_keys=True)

    # ---- algorithmic bytes per decode step, used for the HBM roofline ----
    def weight_bytes_per_step(self, bytes_per_weight: float = 2.0, head_bytes_per_weight: Optional[float] = None,
                              small_bytes: float = 2.0) -> float:
        """Bytes of weights one decode step must stream: every layer matrix, the LM head, norms
        (+ biases) and one embedding row (+ one position row for GPT-2), each read once."""
        d, q, kv, h, V, L = self.dModel, self.attentionDim, self.kvDim, self.hiddenDim, self.vocab, self.nLayer
        if head_bytes_per_weight is None:
            head_bytes_per_weight = bytes_per_weight
        if self.architecture == "gpt2":
            mats = q * d + 2 * kv * d + d * q + 2 * h * d
            small = 4 * d + q + 2 * kv + d + h + d  # two LayerNorms (gamma,beta) + biases
            top = 2 * d + 2 * d  # final gamma/beta + token row + position row
        else:
            mats = q * d + 2 * kv * d + d * q + 3 * h * d
            small = 2 * d
            top = d + d  # final norm + token row
        return L * (mats * bytes_per_weight + small * small_bytes) + V * d * head_bytes_per_weight + top * small_bytes

    def kv_bytes_per_visible_token(self, kv_elem_bytes: int = 2) -> int:
        return 2 * self.nLayer * self.kvDim * kv_elem_bytes


def llama_6l(max_seq: int = 256) -> MultiModelConfig:
    """The reference's own 6-layer benchmark shape (Sources/ANETypes/ModelConfig.swift:1-27)."""
    return MultiModelConfig("llama-6l-d768", 6, 12, 12, 768, 64, 2048, 32000, max_seq, 1e-5, 10000.0, None, "llama")


def llama_draft_1l(max_seq: int = 256) -> MultiModelConfig:
    return MultiModelConfig("llama-1l-d768-draft", 1, 12, 12, 768, 64, 2048, 32000, max_seq, 1e-5, 10000.0, None, "llama")


def gpt2_117m(max_seq: int = 1024) -> MultiModelConfig:
    return MultiModelConfig("gpt2-117m", 12, 12, 12, 768, 64, 3072, 50257, max_seq, 1e-5, 10000.0, None, "gpt2")


def llama_1b(max_seq: int = 2048) -> MultiModelConfig:
    return MultiModelConfig("llama-1.1b", 22, 32, 4, 2048, 64, 5632, 32000, max_seq, 1e-5, 10000.0, None, "llama")


def llama3_8b(max_seq: int = 1024) -> MultiModelConfig:
    return MultiModelConfig("llama3-8b", 32, 32, 8, 4096, 128, 14336, 128256, max_seq, 1e-5, 500000.0, None, "llama")


def tiny_llama(vocab: int = 512, max_seq: int = 64, n_layer: int = 2, gqa: bool = True) -> MultiModelConfig:
    return MultiModelConfig("tiny-llama", n_layer, 4, 2 if gqa else 4, 128, 32, 256, vocab, max_seq, 1e-5, 10000.0, None, "llama")


def tiny_gpt2(vocab: int = 512, max_seq: int = 64, n_layer: int = 2) -> MultiModelConfig:
    return MultiModelConfig("tiny-gpt2", n_layer, 4, 4, 128, 32, 512, vocab, max_seq, 1e-5, 10000.0, None, "gpt2")

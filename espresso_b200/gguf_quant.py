"""GGUF Q8_0 / Q4_0 block formats (numpy).

The reference delegates GGUF parsing and dequantisation to its external Edgerunner package
(Sources/EspressoGGUF/GGUFModelLoader.swift:341-369); the formats below are the public GGUF block
layouts:

* Q8_0: 34-byte block = fp16 scale ``d`` + 32 x int8 ``q``; value ``d * q``.
* Q4_0: 18-byte block = fp16 ``d`` + 16 bytes; byte ``j`` holds element ``j`` in its low nibble and
  element ``j + 16`` in its high nibble; value ``d * (nibble - 8)``.

Quantisers follow the published reference quantisers (Q8_0: ``d = amax / 127``, ``q = round(x / d)``;
Q4_0: ``d = m / -8`` with ``m`` the element of largest magnitude, ``q = min(15, trunc(x / d + 8.5))``).
They are used to build synthetic quantised models; dequantised values are bit-exact ``fp32(d) * q``.
"""
from __future__ import annotations

import numpy as np

QK = 32
BLOCK_BYTES = {"q8_0": 34, "q4_0": 18}
GGML_TYPE = {"f32": 0, "f16": 1, "q4_0": 2, "q8_0": 8, "bf16": 30}


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, QK)
    amax = np.abs(x).max(axis=1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0)).astype(np.float32)
    scaled = x * inv[:, None]
    # round half away from zero, as C roundf
    q = np.where(scaled >= 0, np.floor(scaled + np.float32(0.5)), np.ceil(scaled - np.float32(0.5))).astype(np.int8)
    out = np.empty((x.shape[0], 34), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def dequantize_q8_0(blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 34)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)
    q = b[:, 2:].view(np.int8).astype(np.float32)
    return (d * q).reshape(-1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, QK)
    idx = np.abs(x).argmax(axis=1)  # first element of largest magnitude
    m = x[np.arange(x.shape[0]), idx]
    d = (m / np.float32(-8.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0)).astype(np.float32)
    scaled = x * inv[:, None] + np.float32(8.5)
    q = np.minimum(scaled.astype(np.int8), 15).astype(np.uint8)  # trunc toward zero, values lie in [0.5, 16.5]
    out = np.empty((x.shape[0], 18), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def dequantize_q4_0(blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 18)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)
    lo = (b[:, 2:] & 0x0F).astype(np.int32) - 8
    hi = (b[:, 2:] >> 4).astype(np.int32) - 8
    q = np.concatenate([lo, hi], axis=1).astype(np.float32)
    return (d * q).reshape(-1)


def quantize(kind: str, x: np.ndarray) -> np.ndarray:
    return {"q8_0": quantize_q8_0, "q4_0": quantize_q4_0}[kind](x)


def dequantize(kind: str, blocks: np.ndarray) -> np.ndarray:
    return {"q8_0": dequantize_q8_0, "q4_0": dequantize_q4_0}[kind](blocks)

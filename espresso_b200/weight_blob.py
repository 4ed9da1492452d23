"""BLOBFILE weight files and weight-directory layout.

Byte-compatible with ``WeightBlob.writeHeader`` (Sources/ANETypes/WeightBlob.swift:6-18) and
``BlobWeightLoader.load`` (Sources/ModelSupport/BlobWeightLoader.swift:25-92): a 128-byte header
(byte 0 = 1, byte 4 = 2, bytes 64..67 = EF BE AD DE, byte 68 = 1, little-endian u32 payload size at
72, little-endian u32 data offset = 128 at 80) followed by a little-endian fp16 payload.  Matrices
are row-major ``[out, in]``.  Directory layout: ``LayerWeightPaths.forLayer``
(Sources/ModelSupport/LayerWeightPaths.swift:22-77) and the top-level names of
RealModelInferenceEngine.swift:2066-2154.
"""
from __future__ import annotations

import os
import struct

import numpy as np

from .model_config import MultiModelConfig

HEADER_BYTES = 128
MAGIC = 0xDEADBEEF


class BlobWeightLoaderError(ValueError):
    """Same failure kinds as the reference's ``BlobWeightLoaderError``."""

    def __init__(self, kind: str, detail: str = ""):
        super().__init__(f"{kind}{': ' + detail if detail else ''}")
        self.kind = kind


def make_header(payload_bytes: int) -> bytes:
    if not 0 <= payload_bytes <= 0xFFFFFFFF:
        raise ValueError("BLOBFILE payload must fit in a u32")
    h = bytearray(HEADER_BYTES)
    h[0] = 1
    h[4] = 2
    h[64:68] = b"\xEF\xBE\xAD\xDE"
    h[68] = 1
    struct.pack_into("<I", h, 72, payload_bytes)
    struct.pack_into("<I", h, 80, HEADER_BYTES)
    return bytes(h)


def write_blob(path: str, fp16_values: np.ndarray) -> None:
    """Write fp16 values (any shape, row-major) as a BLOBFILE."""
    a = np.ascontiguousarray(fp16_values)
    if a.dtype != np.float16:
        a = a.astype(np.float16)
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "wb") as f:
        f.write(make_header(a.nbytes))
        f.write(a.astype("<f2", copy=False).tobytes())


def parse_header(data: bytes) -> tuple[int, int]:
    if len(data) < HEADER_BYTES:
        raise BlobWeightLoaderError("truncatedHeader", str(len(data)))
    magic, = struct.unpack_from("<I", data, 64)
    size, = struct.unpack_from("<I", data, 72)
    off, = struct.unpack_from("<I", data, 80)
    if magic != MAGIC:
        raise BlobWeightLoaderError("invalidMagic", hex(magic))
    if off != HEADER_BYTES:
        raise BlobWeightLoaderError("invalidDataOffset", str(off))
    return size, off


def read_blob_fp16(path: str) -> np.ndarray:
    """Return the payload as a flat fp16 array."""
    with open(path, "rb") as f:
        size, off = parse_header(f.read(HEADER_BYTES))
        if size % 2:
            raise BlobWeightLoaderError("invalidPayloadSize", str(size))
        f.seek(off)
        payload = f.read(size)
    if len(payload) != size:
        raise BlobWeightLoaderError("truncatedPayload", f"expected {size}, got {len(payload)}")
    return np.frombuffer(payload, dtype="<f2").astype(np.float16, copy=False)


def read_blob(path: str) -> np.ndarray:
    """Return the payload widened to fp32, as ``BlobWeightLoader.load`` does."""
    return read_blob_fp16(path).astype(np.float32)


def tensor_shapes(cfg: MultiModelConfig) -> dict[str, tuple[int, ...]]:
    """Every tensor of a weight directory (name = relative path without ``.bin``) with its shape."""
    d, q, kv, h, V = cfg.dModel, cfg.attentionDim, cfg.kvDim, cfg.hiddenDim, cfg.vocab
    out: dict[str, tuple[int, ...]] = {"embeddings/token": (V, d)}
    if cfg.architecture == "gpt2":
        out["embeddings/position"] = (cfg.maxSeq, d)
        out["final_norm_gamma"] = (d,)
        out["final_norm_beta"] = (d,)
    else:
        out["rms_final"] = (d,)
    out["lm_head"] = (V, d)
    for l in range(cfg.nLayer):
        p = f"layers/{l}/"
        if cfg.architecture == "gpt2":
            out.update({
                p + "ln_1_gamma": (d,), p + "ln_1_beta": (d,), p + "wq": (q, d), p + "wk": (kv, d), p + "wv": (kv, d),
                p + "wo": (d, q), p + "bq": (q,), p + "bk": (kv,), p + "bv": (kv,), p + "bo": (d,),
                p + "ln_2_gamma": (d,), p + "ln_2_beta": (d,), p + "w1": (h, d), p + "b1": (h,), p + "w2": (d, h),
                p + "b2": (d,),
            })
        else:
            out.update({
                p + "rms_att": (d,), p + "wq": (q, d), p + "wk": (kv, d), p + "wv": (kv, d), p + "wo": (d, q),
                p + "rms_ffn": (d,), p + "w1": (h, d), p + "w2": (d, h), p + "w3": (h, d),
            })
    return out


def is_matrix(name: str) -> bool:
    leaf = name.rsplit("/", 1)[-1]
    return leaf in ("wq", "wk", "wv", "wo", "w1", "w2", "w3", "lm_head")

"""Synthetic weights generated on the GPU for models too large to write to disk quickly.

Used by the benchmark for the 1.1B / 8B shapes: tensors are drawn N(0, 0.02) with torch on the device,
rounded once to fp16/bf16 (or quantised to GGUF Q8_0/Q4_0 blocks with the same rules as
``espresso_b200.gguf_quant``) and handed to ``esp_cuda_load_tensor`` as device pointers.  torch is plumbing
here (a device RNG and a few elementwise ops at set-up time); nothing on the decode path uses it.
"""
from __future__ import annotations

import hashlib

import torch

from .model_config import MultiModelConfig
from .weight_blob import is_matrix, tensor_shapes


def _seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:7], "little")


def quantize_q8_0_torch(x: torch.Tensor) -> torch.Tensor:
    """x: fp32 [n] with n % 32 == 0 -> uint8 [n/32*34] GGUF Q8_0 blocks."""
    xb = x.float().reshape(-1, 32)
    d = xb.abs().amax(dim=1) / 127.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    s = xb * inv[:, None]
    q = torch.where(s >= 0, torch.floor(s + 0.5), torch.ceil(s - 0.5)).to(torch.int8)
    out = torch.empty((xb.shape[0], 34), dtype=torch.uint8, device=x.device)
    out[:, 0:2] = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(torch.uint8)
    return out.reshape(-1)


def quantize_q4_0_torch(x: torch.Tensor) -> torch.Tensor:
    """x: fp32 [n] with n % 32 == 0 -> uint8 [n/32*18] GGUF Q4_0 blocks."""
    xb = x.float().reshape(-1, 32)
    idx = xb.abs().argmax(dim=1, keepdim=True)
    m = xb.gather(1, idx).squeeze(1)
    d = m / -8.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = torch.clamp((xb * inv[:, None] + 8.5).to(torch.int32), max=15).to(torch.uint8)
    out = torch.empty((xb.shape[0], 18), dtype=torch.uint8, device=x.device)
    out[:, 0:2] = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def upload_synthetic(engine, cfg: MultiModelConfig, kind: str = "f16", seed: int = 1234, quantise_head: bool = True,
                     device: int = 0, tp_rank: int = 0, tp_size: int = 1) -> None:
    """Generate every tensor on ``cuda:device`` and upload it; ``kind``: f16 | bf16 | q8_0 | q4_0 for the matrices.

    With ``tp_size > 1`` every rank draws the full tensor from the same seed and uploads only its Megatron shard,
    so the group holds exactly the model a single GPU would hold."""
    from .sharding import tp_shard
    dev = torch.device("cuda", device)
    dense = torch.bfloat16 if kind == "bf16" else torch.float16
    dense_kind = "bf16" if kind == "bf16" else "f16"
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit("/", 1)[-1]
        if leaf in ("rms_att", "rms_ffn", "rms_final", "ln_1_gamma", "ln_2_gamma", "final_norm_gamma"):
            t = torch.ones(shape, dtype=torch.float32, device=dev)
        elif leaf in ("ln_1_beta", "ln_2_beta", "final_norm_beta"):
            t = torch.zeros(shape, dtype=torch.float32, device=dev)
        else:
            src = "embeddings/token" if (leaf == "lm_head" and cfg.architecture == "gpt2") else name
            g = torch.Generator(device=dev)
            g.manual_seed(_seed(seed, src))
            t = torch.randn(shape, dtype=torch.float32, device=dev, generator=g) * 0.02
        t = tp_shard(name, t, tp_rank, tp_size).contiguous()
        if is_matrix(name) and kind in ("q8_0", "q4_0") and (leaf != "lm_head" or quantise_head):
            master = t.to(torch.float16).float().reshape(-1)
            blocks = quantize_q8_0_torch(master) if kind == "q8_0" else quantize_q4_0_torch(master)
            torch.cuda.synchronize(dev)
            engine.load_tensor(name, kind, (blocks.data_ptr(), blocks.numel()))
        else:
            v = t.to(dense).contiguous()
            torch.cuda.synchronize(dev)
            engine.load_tensor(name, dense_kind, (v.data_ptr(), v.numel() * 2))
        del t
    engine.finalize()

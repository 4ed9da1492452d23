"""Writes small GGUF model files with the `gguf` package's own writer (test infrastructure).

The tensors come from the same synthetic generator as every other test; names, metadata keys and the per-head row
interleave of Wq / Wk follow what llama.cpp's converter writes, so the file is what the GGUF front end meets in the
field.
"""
from __future__ import annotations

import numpy as np

from espresso_b200 import gguf_quant
from espresso_b200.synthetic import synthetic_tensors
from espresso_b200.weight_blob import is_matrix

LLAMA_NAMES = {"embeddings/token": "token_embd.weight", "rms_final": "output_norm.weight", "lm_head": "output.weight",
               "rms_att": "attn_norm.weight", "rms_ffn": "ffn_norm.weight", "wq": "attn_q.weight", "wk": "attn_k.weight",
               "wv": "attn_v.weight", "wo": "attn_output.weight", "w1": "ffn_gate.weight", "w3": "ffn_up.weight", "w2": "ffn_down.weight"}
GPT2_NAMES = {"embeddings/token": "token_embd.weight", "embeddings/position": "position_embd.weight",
              "final_norm_gamma": "output_norm.weight", "final_norm_beta": "output_norm.bias", "lm_head": "output.weight",
              "ln_1_gamma": "attn_norm.weight", "ln_1_beta": "attn_norm.bias", "ln_2_gamma": "ffn_norm.weight", "ln_2_beta": "ffn_norm.bias",
              "wo": "attn_output.weight", "bo": "attn_output.bias", "w1": "ffn_up.weight", "b1": "ffn_up.bias", "w2": "ffn_down.weight",
              "b2": "ffn_down.bias"}


def interleave_rows(w: np.ndarray, n_head: int) -> np.ndarray:
    """llama.cpp's converter: row (half h, pair i) of every head moves to row 2 i + h."""
    rows = w.shape[0]
    return w.reshape(n_head, 2, rows // n_head // 2, *w.shape[1:]).swapaxes(1, 2).reshape(w.shape)


def gguf_name(cfg, name: str) -> str:
    table = GPT2_NAMES if cfg.architecture == "gpt2" else LLAMA_NAMES
    if name.startswith("layers/"):
        _, layer, leaf = name.split("/")
        return f"blk.{layer}.{table[leaf]}"
    return table[name]


def write_gguf(path: str, cfg, kind: str, oracle_model=None, arch_name: str | None = None, tied: bool = False, seed: int = 1234,
               quantise_embedding: bool = False) -> None:
    """Writes ``cfg``'s synthetic tensors as a GGUF file; matrices in ``kind`` ("f16", "f32", "q8_0", "q4_0").

    When ``oracle_model`` is given it receives the values the file decodes to (dequantised blocks), in the reference's
    own layout, so that the oracle and the engine built from the file see the same model."""
    import gguf

    arch = arch_name or cfg.architecture
    w = gguf.GGUFWriter(path, arch)
    w.add_uint32(f"{arch}.block_count", cfg.nLayer)
    w.add_uint32(f"{arch}.context_length", cfg.maxSeq)
    w.add_uint32(f"{arch}.embedding_length", cfg.dModel)
    w.add_uint32(f"{arch}.feed_forward_length", cfg.hiddenDim)
    w.add_uint32(f"{arch}.attention.head_count", cfg.nHead)
    w.add_uint32(f"{arch}.attention.head_count_kv", cfg.nKVHead)
    if cfg.headDim * cfg.nHead != cfg.dModel:
        w.add_uint32(f"{arch}.attention.key_length", cfg.headDim)
    if cfg.architecture == "gpt2":
        w.add_float32(f"{arch}.attention.layer_norm_epsilon", cfg.normEps)
    else:
        w.add_float32(f"{arch}.attention.layer_norm_rms_epsilon", cfg.normEps)
        w.add_float32(f"{arch}.rope.freq_base", cfg.ropeTheta)
    w.add_array("tokenizer.ggml.tokens", [f"<{i}>" for i in range(cfg.vocab)])
    if cfg.eosToken is not None:
        w.add_uint32("tokenizer.ggml.eos_token_id", cfg.eosToken)
    interleaved = arch in ("llama", "llama2", "llama3", "mistral")
    fused = {}  # GPT-2: layer -> {"wq": ..., ...}
    quant_types = {"q8_0": gguf.GGMLQuantizationType.Q8_0, "q4_0": gguf.GGMLQuantizationType.Q4_0}

    def add_matrix(gname: str, vals: np.ndarray, store_kind: str) -> np.ndarray:
        """Adds the matrix and returns the fp32 values it decodes to."""
        if store_kind in quant_types:
            blocks = gguf_quant.quantize(store_kind, vals.astype(np.float32))
            per_row = vals.shape[1] // 32 * (34 if store_kind == "q8_0" else 18)
            w.add_tensor(gname, blocks.reshape(vals.shape[0], per_row), raw_dtype=quant_types[store_kind])
            return gguf_quant.dequantize(store_kind, blocks).reshape(vals.shape)
        if store_kind == "f32":
            w.add_tensor(gname, np.ascontiguousarray(vals, dtype=np.float32))
            return vals.astype(np.float32)
        h = np.ascontiguousarray(vals, dtype=np.float16)
        w.add_tensor(gname, h)
        return h.astype(np.float32)

    for name, vals in synthetic_tensors(cfg, seed):
        leaf = name.rsplit("/", 1)[-1]
        if name == "lm_head" and tied:
            continue
        decoded = None
        if cfg.architecture == "gpt2" and leaf in ("wq", "wk", "wv", "bq", "bk", "bv"):
            fused.setdefault(name.split("/")[1], {})[leaf] = vals
            decoded = vals.astype(np.float16).astype(np.float32) if leaf.startswith("w") else vals.astype(np.float32)
        elif is_matrix(name):
            stored = vals
            if interleaved and leaf in ("wq", "wk"):
                stored = interleave_rows(vals, cfg.nHead if leaf == "wq" else cfg.nKVHead)
            dec = add_matrix(gguf_name(cfg, name), stored, kind)
            if interleaved and leaf in ("wq", "wk"):  # back to the reference's row order for the oracle
                heads = cfg.nHead if leaf == "wq" else cfg.nKVHead
                dec = dec.reshape(heads, dec.shape[0] // heads // 2, 2, -1).swapaxes(1, 2).reshape(dec.shape)
            decoded = dec
        elif name.startswith("embeddings/"):
            decoded = add_matrix(gguf_name(cfg, name), vals, kind if (quantise_embedding and name == "embeddings/token") else "f16")
            # the engine keeps embedding tables in fp16
            decoded = decoded.astype(np.float16).astype(np.float32)
        else:
            w.add_tensor(gguf_name(cfg, name), np.ascontiguousarray(vals, dtype=np.float32))
            decoded = vals.astype(np.float32)
        if oracle_model is not None:
            oracle_model.set_tensor(name, decoded)
            if name == "embeddings/token" and tied:
                head = decoded
                if quantise_embedding and kind in quant_types:  # the tied head multiplies by the blocks themselves
                    head = gguf_quant.dequantize(kind, gguf_quant.quantize(kind, vals.astype(np.float32))).reshape(vals.shape)
                oracle_model.set_tensor("lm_head", head)
    for layer, parts in fused.items():  # GPT-2 files hold one fused projection per layer
        w.add_tensor(f"blk.{layer}.attn_qkv.weight", np.concatenate([parts["wq"], parts["wk"], parts["wv"]]).astype(np.float16))
        w.add_tensor(f"blk.{layer}.attn_qkv.bias", np.concatenate([parts["bq"], parts["bk"], parts["bv"]]).astype(np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()

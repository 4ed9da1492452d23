"""Generate ``hf_gpt2_tiny.npz``: logits of HuggingFace ``GPT2LMHeadModel`` on a seeded tiny model.

The synthetic weights of this repository are loaded into an HF GPT-2 (``gelu_new`` = the tanh
approximation), the reference's own exporter ``scripts/convert_weights_gpt2.py:save_gpt2_artifacts``
writes them back out as a weight directory, and that directory must be byte-identical to the one
written by ``espresso_b200.synthetic`` (this pins the directory layout and the Conv1D transposes).
The HF logits are the golden values; the tests regenerate the weights from the seed.

    python tests/golden/make_hf_gpt2_golden.py <path to the reference checkout>
"""
import filecmp
import os
import shutil
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from espresso_b200.model_config import tiny_gpt2  # noqa: E402
from espresso_b200.synthetic import synthetic_prompt, synthetic_tensors, write_synthetic_model  # noqa: E402
from espresso_b200.weight_blob import tensor_shapes  # noqa: E402


def main(reference_root: str) -> None:
    sys.path.insert(0, os.path.join(reference_root, "scripts"))
    import torch
    from pathlib import Path
    from transformers import GPT2Config, GPT2LMHeadModel
    from convert_weights_gpt2 import save_gpt2_artifacts

    seed = 777
    cfg = tiny_gpt2(vocab=512, max_seq=64, n_layer=2)
    t = {name: torch.from_numpy(v.astype(np.float32)) for name, v in synthetic_tensors(cfg, seed)}
    hf = GPT2LMHeadModel(GPT2Config(
        vocab_size=cfg.vocab, n_positions=cfg.maxSeq, n_embd=cfg.dModel, n_layer=cfg.nLayer, n_head=cfg.nHead,
        n_inner=cfg.hiddenDim, activation_function="gelu_new", layer_norm_epsilon=cfg.normEps,
        resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0, tie_word_embeddings=False))
    sd = {
        "transformer.wte.weight": t["embeddings/token"], "transformer.wpe.weight": t["embeddings/position"],
        "transformer.ln_f.weight": t["final_norm_gamma"], "transformer.ln_f.bias": t["final_norm_beta"],
        "lm_head.weight": t["lm_head"],
    }
    for l in range(cfg.nLayer):
        p, q = f"layers/{l}/", f"transformer.h.{l}."
        sd[q + "ln_1.weight"] = t[p + "ln_1_gamma"]
        sd[q + "ln_1.bias"] = t[p + "ln_1_beta"]
        sd[q + "attn.c_attn.weight"] = torch.cat([t[p + "wq"].T, t[p + "wk"].T, t[p + "wv"].T], dim=1).contiguous()
        sd[q + "attn.c_attn.bias"] = torch.cat([t[p + "bq"], t[p + "bk"], t[p + "bv"]])
        sd[q + "attn.c_proj.weight"] = t[p + "wo"].T.contiguous()
        sd[q + "attn.c_proj.bias"] = t[p + "bo"]
        sd[q + "ln_2.weight"] = t[p + "ln_2_gamma"]
        sd[q + "ln_2.bias"] = t[p + "ln_2_beta"]
        sd[q + "mlp.c_fc.weight"] = t[p + "w1"].T.contiguous()
        sd[q + "mlp.c_fc.bias"] = t[p + "b1"]
        sd[q + "mlp.c_proj.weight"] = t[p + "w2"].T.contiguous()
        sd[q + "mlp.c_proj.bias"] = t[p + "b2"]
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not unexpected and all(".attn.bias" in m or ".masked_bias" in m for m in missing), (missing, unexpected)
    hf.eval()

    mine = tempfile.mkdtemp(prefix="esp_gpt2_mine_")
    theirs = tempfile.mkdtemp(prefix="esp_gpt2_ref_")
    try:
        write_synthetic_model(cfg, mine, seed=seed)
        save_gpt2_artifacts(hf, Path(theirs), metadata_name=cfg.name)
        for name in tensor_shapes(cfg):
            assert filecmp.cmp(os.path.join(mine, name + ".bin"), os.path.join(theirs, name + ".bin"), shallow=False), name
    finally:
        shutil.rmtree(mine, ignore_errors=True)
        shutil.rmtree(theirs, ignore_errors=True)

    prompt = synthetic_prompt(cfg.vocab, 12, seed=seed)
    with torch.no_grad():
        logits = hf(torch.from_numpy(prompt.astype(np.int64))[None]).logits[0].numpy()
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "hf_gpt2_tiny.npz"),
                        seed=np.int64(seed), prompt=prompt, logits=logits.astype(np.float32))
    print("weight directories byte-identical; logits", logits.shape)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: " + sys.argv[0] + " <path to the reference checkout>")
    main(sys.argv[1])

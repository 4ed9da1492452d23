"""Generate ``hf_llama_tiny.npz``: logits of HuggingFace ``LlamaForCausalLM`` on a seeded tiny model.

Run once in a container that holds the reference checkout; the reference's own Python bridge
(``scripts/espresso_llama_weights.py``) turns the BLOBFILE weight directory into the HF model, so the
fixture pins the oracle (and the weight-directory layout) against an implementation that is
independent of this repository.  The fixture stores only the model seed/shape, the prompt and the
logits; the tests regenerate the identical weights from the seed.

    python tests/golden/make_hf_llama_golden.py <path to the reference checkout>
"""
import os
import shutil
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from espresso_b200.model_config import tiny_llama  # noqa: E402
from espresso_b200.synthetic import synthetic_prompt, write_synthetic_model  # noqa: E402


def main(reference_root: str) -> None:
    sys.path.insert(0, os.path.join(reference_root, "scripts"))
    import torch
    from espresso_llama_weights import load_espresso_llama_for_causal_lm
    from pathlib import Path

    out = {}
    for tag, gqa, seed in (("gqa", True, 1234), ("mha", False, 4321)):
        cfg = tiny_llama(vocab=512, max_seq=64, n_layer=2, gqa=gqa)
        tmp = tempfile.mkdtemp(prefix="esp_golden_")
        try:
            write_synthetic_model(cfg, tmp, seed=seed)
            shutil.copy(os.path.join(tmp, "rms_final.bin"), os.path.join(tmp, "final_norm.bin"))
            _, model = load_espresso_llama_for_causal_lm(Path(tmp), torch_dtype=torch.float32)
            prompt = synthetic_prompt(cfg.vocab, 12, seed=seed)
            with torch.no_grad():
                logits = model(torch.from_numpy(prompt.astype(np.int64))[None]).logits[0].numpy()
            out[f"{tag}_seed"] = np.int64(seed)
            out[f"{tag}_prompt"] = prompt
            out[f"{tag}_logits"] = logits.astype(np.float32)
        finally:
            shutil.rmtree(tmp, ignore_errors=True)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "hf_llama_tiny.npz"), **out)
    print({k: getattr(v, "shape", v) for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: " + sys.argv[0] + " <path to the reference checkout>")
    main(sys.argv[1])

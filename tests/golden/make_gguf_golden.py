"""Generate ``gguf_blocks.npz``: Q8_0 / Q4_0 blocks and their dequantised values from the ``gguf``
Python package (an implementation independent of this repository) on a seeded input.

    python tests/golden/make_gguf_golden.py
"""
import os

import numpy as np
from gguf import GGMLQuantizationType as T
from gguf import quants


def main() -> None:
    rng = np.random.default_rng(20240607)
    x = (rng.standard_normal(32 * 256).astype(np.float32) * np.float32(0.02))
    x[:32] = 0.0                       # all-zero block (d = 0)
    x[32:64] = np.float32(0.5)         # constant block
    x[64:96] *= np.float32(1000.0)     # large magnitudes
    x[96] = np.float32(-1.0)           # the extreme element is negative (Q4_0 sign rule)
    out = {"x": x}
    for kind, t in (("q8_0", T.Q8_0), ("q4_0", T.Q4_0)):
        blocks = quants.quantize(x.reshape(-1, 256), t)
        out[kind + "_blocks"] = blocks.reshape(-1)
        out[kind + "_dequant"] = quants.dequantize(blocks, t).reshape(-1).astype(np.float32)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "gguf_blocks.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()

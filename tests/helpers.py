"""Shared helpers of the GPU parity tests."""
import numpy as np

from espresso_b200 import gguf_quant
from espresso_b200.synthetic import synthetic_tensors
from espresso_b200.weight_blob import is_matrix

ABS_TOL = 2e-2   # max-abs logit tolerance (fp16 KV cache, different summation order)
REL_TOL = 1e-2   # relative tolerance
# bf16 activations on the tensor-core path carry 8 mantissa bits against fp16's 11: rounding per product is 8x
# coarser, so the max-abs bound of a bf16 model is 4x the fp16 one (the relative bound stays)
BF16_ABS_TOL = 8e-2


def assert_logits_close(got, ref, what="", abs_tol=ABS_TOL):
    got = np.asarray(got, np.float32)
    ref = np.asarray(ref, np.float32)
    err = np.abs(got - ref)
    assert err.max() <= abs_tol, f"{what}: max-abs {err.max():.3e} > {abs_tol}"
    rel = np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-12)
    assert rel <= REL_TOL, f"{what}: relative error {rel:.3e} > {REL_TOL}"


def compare_greedy_stream(oracle_runtime, prompt, gpu_tokens, tol=ABS_TOL):
    """Teacher-forced comparison of a greedy stream with the oracle.

    The oracle is fed the GPU's tokens.  At every step the GPU token must be the oracle's argmax unless the
    oracle's top-2 logit gap is within ``tol`` (then the GPU token's oracle logit must be within ``tol`` of the
    maximum).  Returns the list of positions where the two argmaxes differed inside the tolerance.
    """
    assert oracle_runtime.prefill(prompt) == 0
    near_ties = []
    for i, tok in enumerate(gpu_tokens):
        logits = oracle_runtime.logits()
        best = int(np.argmax(logits))
        if int(tok) != best:
            gap = float(logits[best] - logits[int(tok)])
            assert gap <= tol, f"step {i}: GPU token {tok} vs oracle {best}, oracle logit gap {gap:.4f} > {tol}"
            near_ties.append(i)
        if i + 1 < len(gpu_tokens):
            assert oracle_runtime.advance(int(tok)) == 0
    return near_ties


def quantised_pair(oracle_lib, cfg, kind, seed=1234, quantise_head=True):
    """Returns (oracle model holding the dequantised fp32 values, list of (name, kind, array) uploads)."""
    model = oracle_lib.Model(cfg.to_metadata())
    uploads = []
    for name, vals in synthetic_tensors(cfg, seed):
        leaf = name.rsplit("/", 1)[-1]
        if is_matrix(name) and (leaf != "lm_head" or quantise_head):
            blocks = gguf_quant.quantize(kind, vals.astype(np.float32))
            model.set_tensor(name, gguf_quant.dequantize(kind, blocks))
            uploads.append((name, kind, blocks))
        else:
            model.set_tensor(name, vals.astype(np.float32))
            uploads.append((name, "f16", vals))
    return model, uploads


def upload_all(engine, uploads):
    for name, kind, arr in uploads:
        engine.load_tensor(name, kind, arr)
    engine.finalize()


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, returned as the 16 stored bits."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def dense_pair(rt, oracle_lib, cfg, kind="f16", max_batch=1, seed=1234):
    """Engine and oracle model holding the same seeded weights in a 16-bit storage type (f16 or bf16)."""
    from espresso_b200.synthetic import synthetic_tensor
    from espresso_b200.weight_blob import is_matrix, tensor_shapes

    eng = rt.DecodeEngine.empty(cfg, max_batch=max_batch)
    model = oracle_lib.Model(cfg.to_metadata())
    for name, shape in tensor_shapes(cfg).items():
        vals = synthetic_tensor(cfg, name, shape, seed)
        wide = is_matrix(name) or name.startswith("embeddings/")
        if kind == "bf16" and wide:
            bits = to_bf16_bits(vals)
            eng.load_tensor(name, "bf16", bits)
            model.set_tensor(name, (bits.astype(np.uint32) << np.uint32(16)).view(np.float32).reshape(shape))
        else:
            h = vals.astype(np.float16)
            eng.load_tensor(name, "f16", h)
            model.set_tensor(name, h.astype(np.float32))
        del vals
    eng.finalize()
    return eng, model

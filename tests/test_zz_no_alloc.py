"""The allocation-free LM-head entry point (collected last on purpose: a run that stops at the first failure
has then already run every other test).

``esp_cuda_lm_head_argmax_static`` is for hosts that cannot call the CUDA allocator while they run (a fixed
device-memory budget, someone else's arena, a loop that must not stall the device); its working memory is an
array built into the library.  The test drives it through the C ABI with caller-owned device buffers (held in
torch tensors here) and checks the tokens against the logits of the existing ``esp_cuda_gemv_bench`` entry
point, which allocates its own buffers, on two calls in a row that share the built-in array."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _reference_tokens(rt, lm_head, hidden, gain, eps):
    toks, margins = [], []
    for h in hidden:
        x = h.astype(np.float32)
        if gain is not None:
            x = x * np.float32(1.0 / np.sqrt(np.float32((x * x).sum()) / np.float32(x.size) + np.float32(eps))) * gain
        logits, _ = rt.gemv_bench("f16", lm_head, lm_head.shape[0], lm_head.shape[1], x, warmup=0, iterations=1)
        order = np.argsort(-logits, kind="stable")
        toks.append(int(np.argmax(logits)))
        margins.append(float(logits[order[0]] - logits[order[1]]))
    return toks, margins


def test_static_lm_head_matches_allocating_entry_point_on_two_calls():
    import torch
    from espresso_b200 import runtime as rt

    rt.load_library()
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(2024)
    vocab, d = 5003, 768  # odd vocab: the last work item holds a single row
    lm_head = (rng.standard_normal((vocab, d)) * 0.02).astype(np.float16)
    gain = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    d_w = torch.from_numpy(lm_head).to(dev)
    d_gain = torch.from_numpy(gain).to(dev)
    d_tok = torch.zeros(rt.STATIC_HEAD_MAX_ROWS, dtype=torch.int32, device=dev)
    # two calls in a row with different row counts and inputs; the second must not see the first's leftovers
    for call, (rows, use_gain) in enumerate(((7, True), (3, False))):
        hidden = rng.standard_normal((rows, d)).astype(np.float32)
        d_h = torch.from_numpy(hidden).to(dev)
        d_tok.fill_(-1)
        torch.cuda.synchronize()
        rt.lm_head_argmax_static(d_w.data_ptr(), vocab, d, d_h.data_ptr(), rows, d_gain.data_ptr() if use_gain else None, 1e-5,
                                 d_tok.data_ptr(), stream=0, device=0)
        torch.cuda.synchronize()
        got = d_tok.cpu().numpy()[:rows].astype(np.int64)
        ref, margins = _reference_tokens(rt, lm_head, hidden, gain if use_gain else None, 1e-5)
        for r in range(rows):
            # identical tokens wherever the top-2 gap exceeds the rounding tolerance of the two summation orders
            assert got[r] == ref[r] or margins[r] <= 2e-4, f"call {call} row {r}: {got[r]} vs {ref[r]} (margin {margins[r]:.2e})"
        assert (d_tok.cpu().numpy()[rows:] == -1).all()  # nothing beyond `rows` is written


def test_static_lm_head_rejects_sizes_beyond_its_fixed_array():
    import torch
    from espresso_b200 import runtime as rt

    dev = torch.device("cuda", 0)
    w = torch.zeros((16, 64), dtype=torch.float16, device=dev)
    h = torch.zeros((rt.STATIC_HEAD_MAX_ROWS + 1, 64), dtype=torch.float32, device=dev)
    t = torch.zeros(rt.STATIC_HEAD_MAX_ROWS + 1, dtype=torch.int32, device=dev)
    with pytest.raises(rt.RealModelInferenceError) as ei:
        rt.lm_head_argmax_static(w.data_ptr(), 16, 64, h.data_ptr(), rt.STATIC_HEAD_MAX_ROWS + 1, None, 1e-5, t.data_ptr())
    assert ei.value.status == rt.ERR_INVALID_ARGUMENT and "fixed array" in ei.value.message
    with pytest.raises(rt.RealModelInferenceError):
        rt.lm_head_argmax_static(w.data_ptr(), 16, 8200, h.data_ptr(), 1, None, 1e-5, t.data_ptr())

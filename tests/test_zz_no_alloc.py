"""The allocation-free LM-head entry point (collected last on purpose: a run that stops at the first failure
has then already run every other test).

``esp_cuda_lm_head_argmax_static`` is for hosts that cannot call the CUDA allocator while they run (a fixed
device-memory budget, someone else's arena, a loop that must not stall the device); its working memory is an
array built into the library.  The test drives it through the C ABI with caller-owned device buffers (held in
torch tensors here) and checks the tokens against the logits of the existing ``esp_cuda_gemv_bench`` entry
point, which allocates its own buffers, and against a numpy fp32 product, on two calls in a row that share the
built-in array."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _reference_tokens(rt, lm_head, hidden, gain, eps):
    """Tokens and top-2 margins from the allocating entry point, and tokens from a numpy fp32 product."""
    toks, margins, np_toks = [], [], []
    w32 = lm_head.astype(np.float32)
    for h in hidden:
        x = h.astype(np.float32)
        if gain is not None:
            x = x * np.float32(1.0 / np.sqrt(np.float32((x * x).sum()) / np.float32(x.size) + np.float32(eps))) * gain
        logits, _ = rt.gemv_bench("f16", lm_head, lm_head.shape[0], lm_head.shape[1], x, warmup=0, iterations=1)
        order = np.argsort(-logits, kind="stable")
        toks.append(int(np.argmax(logits)))
        margins.append(float(logits[order[0]] - logits[order[1]]))
        host = w32 @ x
        assert np.abs(host - logits).max() <= 1e-3  # the allocating entry point itself agrees with the host product
        np_toks.append(int(np.argmax(host)))
    return toks, margins, np_toks


def test_static_lm_head_matches_allocating_entry_point_on_two_calls():
    import torch
    from espresso_b200 import runtime as rt

    rt.load_library()
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(2024)
    _two_calls(rt, torch, dev, rng, vocab=5003, d=768, calls=((7, True), (3, False)))  # odd vocab: the last work item holds a single row


def test_static_lm_head_at_its_row_limit_and_with_a_ragged_width():
    """Every slot of the built-in array (rows = the maximum) and a d_model that is not a multiple of the 256-element
    slices of the dot products."""
    import torch
    from espresso_b200 import runtime as rt

    rt.load_library()
    _two_calls(rt, torch, torch.device("cuda", 0), np.random.default_rng(7), vocab=1201, d=72, calls=((rt.STATIC_HEAD_MAX_ROWS, True), (5, False)))


def _two_calls(rt, torch, dev, rng, vocab, d, calls):
    lm_head = (rng.standard_normal((vocab, d)) * 0.02).astype(np.float16)
    gain = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    d_w = torch.from_numpy(lm_head).to(dev)
    d_gain = torch.from_numpy(gain).to(dev)
    d_tok = torch.zeros(rt.STATIC_HEAD_MAX_ROWS + 4, dtype=torch.int32, device=dev)
    # two calls in a row with different row counts and inputs; the second must not see the first's leftovers
    for call, (rows, use_gain) in enumerate(calls):
        hidden = rng.standard_normal((rows, d)).astype(np.float32)
        d_h = torch.from_numpy(hidden).to(dev)
        d_tok.fill_(-1)
        torch.cuda.synchronize()
        rt.lm_head_argmax_static(d_w.data_ptr(), vocab, d, d_h.data_ptr(), rows, d_gain.data_ptr() if use_gain else None, 1e-5,
                                 d_tok.data_ptr(), stream=0, device=0)
        torch.cuda.synchronize()
        got = d_tok.cpu().numpy()[:rows].astype(np.int64)
        ref, margins, host = _reference_tokens(rt, lm_head, hidden, gain if use_gain else None, 1e-5)
        for r in range(rows):
            # identical tokens wherever the top-2 gap exceeds the rounding tolerance of the two summation orders
            assert got[r] == ref[r] or margins[r] <= 2e-4, f"call {call} row {r}: {got[r]} vs {ref[r]} (margin {margins[r]:.2e})"
            assert got[r] == host[r] or margins[r] <= 2e-4, f"call {call} row {r}: {got[r]} vs numpy {host[r]}"
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
    # a matrix view that does not start on a 16-byte boundary is refused on the host instead of faulting on the device
    with pytest.raises(rt.RealModelInferenceError) as ea:
        rt.lm_head_argmax_static(w.data_ptr() + 2, 15, 64, h.data_ptr(), 1, None, 1e-5, t.data_ptr())
    assert ea.value.status == rt.ERR_INVALID_ARGUMENT and "aligned" in ea.value.message

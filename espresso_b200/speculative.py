"""GPT-2 layer-split speculation: a draft made of the model's first k layers proposes, the full model decides.

Mirrors ``generateIncrementalHybridSpeculative`` (Sources/RealModelInference/RealModelInferenceEngine.swift:4989-5201)
and the switch that enables it (``resolvedSpeculativeDraftLayerCount``, :2048-2064).  The loop is host-side control over
two decoder objects that expose the reference runtime's calls (``reset``, ``advance``, ``select_greedy_token``,
``capture_checkpoint``, ``rollback``); every emitted token is the verifier's own greedy token, so the stream equals plain
greedy decoding of the full model whatever the draft proposes.  In the reference the verifier consumes the draft's final
hidden state and runs only the remaining layers; here the verifier is a complete engine of the model, the draft a second
engine built from the same weight directory with ``nLayer = k`` — the tokens are the same, the draft's work is not
shared.
"""
from __future__ import annotations

import dataclasses
import os
import time
from typing import Callable, Mapping, Optional, Sequence

GPT2_EOS_TOKEN = 50256  # RealModelInferenceEngine.gpt2EOSToken


def resolved_speculative_draft_layer_count(config, temperature: float, environment: Optional[Mapping[str, str]] = None) -> Optional[int]:
    """Number of draft layers, or None when the speculative loop does not apply: GPT-2 only, greedy only, at least two
    layers, and ``ESPRESSO_ENABLE_GPT2_SPECULATIVE=1``; ``ESPRESSO_GPT2_SPECULATIVE_DRAFT_LAYERS`` (default 1) is clamped
    to [1, nLayer - 1]; a value that is not an integer falls back to the default."""
    env = os.environ if environment is None else environment
    if config.architecture != "gpt2" or temperature != 0 or config.nLayer <= 1 or env.get("ESPRESSO_ENABLE_GPT2_SPECULATIVE") != "1":
        return None
    requested = 1
    raw = env.get("ESPRESSO_GPT2_SPECULATIVE_DRAFT_LAYERS")
    if raw is not None:
        try:
            requested = int(raw)
        except ValueError:
            requested = 1
    return min(max(requested, 1), config.nLayer - 1)


@dataclasses.dataclass
class SpeculativeResult:
    tokens: list
    tokenLatenciesMs: list
    firstTokenLatencyMs: float
    tokensPerSecond: float
    passes: int            # iterations of the propose / verify loop
    acceptedFirst: int     # passes whose first proposal was the verifier's token
    acceptedSecond: int    # passes whose second proposal was the verifier's token too
    stoppedOnEOS: bool


def generate_layer_split_speculative(draft, verifier, prompt_tokens: Sequence[int], max_tokens: int, max_seq: int,
                                     eos_token: int = GPT2_EOS_TOKEN,
                                     on_step: Optional[Callable[[int, list, float], None]] = None) -> SpeculativeResult:
    """Runs the propose / verify loop.  ``draft`` and ``verifier`` are fresh or used decoders (they are reset here).

    One pass: the draft proposes a token, consumes it and proposes a second one.  The verifier's token for the first
    position is emitted; if it differs from the proposal the draft returns to its checkpoint and both consume the
    verifier's token.  Otherwise the verifier consumes it, its token for the second position is emitted and both consume
    that.  The end-of-sequence token ends the loop without being emitted (the GPT-2 rule); generation also ends at
    ``max_tokens`` emitted tokens or when the context holds ``max_seq`` tokens."""
    prompt = [int(t) for t in prompt_tokens]
    if not prompt:
        raise ValueError("Prompt tokens must not be empty")
    if max_tokens < 0:
        raise ValueError("maxTokens must be >= 0")
    if len(prompt) >= max_seq:
        raise ValueError("Prompt token count exceeds model context")
    effective = min(max_tokens, max_seq - len(prompt))
    draft.reset()
    verifier.reset()
    for tok in prompt:
        draft.advance(tok)
        verifier.advance(tok)
    out: list = []
    latencies: list = []
    n_all = len(prompt)
    t_start = time.perf_counter()
    t_prev = t_start
    first_latency = 0.0
    passes = accepted_first = accepted_second = 0
    stopped = False

    def emit(token: int) -> None:
        nonlocal t_prev, first_latency, n_all
        now = time.perf_counter()
        out.append(token)
        n_all += 1
        latencies.append((now - t_prev) * 1e3)
        if len(out) == 1:
            first_latency = (now - t_start) * 1e3
        t_prev = now
        if on_step is not None:
            on_step(token, list(out), (now - t_start) * 1e3)

    while len(out) < effective:
        passes += 1
        checkpoint = draft.capture_checkpoint()
        proposed0 = draft.select_greedy_token()
        draft.advance(proposed0)
        proposed1 = draft.select_greedy_token()
        exact0 = verifier.select_greedy_token()
        if exact0 == eos_token:
            stopped = True
            break
        if exact0 != proposed0:
            draft.rollback(checkpoint)
            draft.advance(exact0)
            verifier.advance(exact0)
            emit(exact0)
            if len(out) >= effective or n_all >= max_seq:
                break
            continue
        accepted_first += 1
        verifier.advance(exact0)
        emit(exact0)
        if len(out) >= effective or n_all >= max_seq:
            break
        exact1 = verifier.select_greedy_token()
        if exact1 == eos_token:
            stopped = True
            break
        if exact1 == proposed1:
            accepted_second += 1
        draft.advance(exact1)
        verifier.advance(exact1)
        emit(exact1)
        if n_all >= max_seq:
            break
    elapsed = max(time.perf_counter() - t_start, 1e-9)
    return SpeculativeResult(out, latencies, first_latency, len(out) / elapsed if out else 0.0, passes, accepted_first,
                             accepted_second, stopped)


def build_layer_split_pair(runtime, weight_dir: str, draft_layers: int, device: int = 0, flags: int = 0):
    """(draft, verifier) engines of one GPT-2 weight directory: the verifier is the whole model, the draft its first
    ``draft_layers`` layers with the same embeddings, final norm and output head."""
    from .model_config import MultiModelConfig
    import json

    with open(os.path.join(weight_dir, "metadata.json")) as f:
        cfg = MultiModelConfig.from_metadata(json.load(f))
    if not 1 <= draft_layers < cfg.nLayer:
        raise ValueError("draft_layers must be in [1, nLayer - 1]")
    verifier = runtime.DecodeEngine.build(weight_dir, max_batch=1, device=device, flags=flags)
    draft = runtime.DecodeEngine.build(weight_dir, config=dataclasses.replace(cfg, nLayer=draft_layers), max_batch=1, device=device, flags=flags)
    return draft, verifier

"""ctypes binding of ``libespresso_cuda.so`` and a host-side mirror of the reference's engine API.

``DecodeEngine`` keeps the token-id surface of ``RealModelInferenceEngine``
(Sources/RealModelInference/RealModelInferenceEngine.swift: ``build`` :1377, ``generate`` :1405,
``generate*ForTesting`` :1681-1876) and of its decoder object ``CPUExactLlamaRuntime`` (:548-850):
``reset / prefill / advance / select_greedy_token / capture_checkpoint / rollback``.  Every method is one
call through the C ABI declared in ``include/espresso_cuda.h``; there is no CPU fallback, and importing
this module fails if the CUDA library has not been built.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import os
from typing import Optional, Sequence

import numpy as np

from .model_config import MultiModelConfig

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libespresso_cuda.so")

OK = 0
ERR_INVALID_ARGUMENT, ERR_OUT_OF_RANGE, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT = 1, 2, 3, 4, 5
ERR_OUT_OF_MEMORY, ERR_IO, ERR_INVALID_WEIGHTS, ERR_FORCED_FAILURE, ERR_STATE = 6, 7, 8, 9, 10

F32, F16, Q4_0, Q8_0, BF16 = 0, 1, 2, 8, 30
TENSOR_TYPES = {"f32": F32, "f16": F16, "q4_0": Q4_0, "q8_0": Q8_0, "bf16": BF16}

FLAG_KEEP_LOGITS = 1
FLAG_NO_GRAPH = 2
FLAG_NO_MEGAKERNEL = 4
FLAG_NO_TC_SHADOW = 8


class RealModelInferenceError(RuntimeError):
    """Mirrors ``RealModelInferenceError`` (Engine.swift:85-115); ``status`` is the C status code."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[esp_cuda status {status}] {message}")
        self.status = status
        self.message = message


class EspCudaConfig(C.Structure):
    _fields_ = [
        ("architecture", C.c_int32), ("n_layer", C.c_int32), ("n_head", C.c_int32), ("n_kv_head", C.c_int32),
        ("d_model", C.c_int32), ("head_dim", C.c_int32), ("hidden_dim", C.c_int32), ("vocab", C.c_int32),
        ("max_seq", C.c_int32), ("norm_eps", C.c_float), ("rope_theta", C.c_float), ("eos_token", C.c_int32),
        ("max_batch", C.c_int32), ("device", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32),
        ("flags", C.c_int32),
    ]


class EspCudaGenerationResult(C.Structure):
    _fields_ = [
        ("generated_tokens", C.c_int32), ("prompt_tokens", C.c_int32), ("tokens_per_second", C.c_double),
        ("prefill_ms", C.c_double), ("first_token_latency_ms", C.c_double), ("total_decode_ms", C.c_double),
        ("committed_exact_tokens_per_pass", C.c_double), ("accepted_future_tokens_per_pass", C.c_double),
        ("speculative_passes", C.c_int32), ("stopped_on_eos", C.c_int32),
    ]


class EspCudaTimings(C.Structure):
    _fields_ = [("qkv_ms", C.c_float), ("attention_ms", C.c_float), ("ffn_ms", C.c_float), ("head_ms", C.c_float),
                ("total_ms", C.c_float), ("kernel_launches", C.c_int32)]


# Every symbol that include/espresso_cuda.h declares: name -> (restype, argtypes)
_vp, _u32p, _i32p, _f32p = C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_int32), C.POINTER(C.c_float)
SIGNATURES = {
    "esp_cuda_create": (C.c_int32, [C.POINTER(EspCudaConfig), C.c_char_p, C.POINTER(_vp)]),
    "esp_cuda_create_from_directory": (C.c_int32, [C.c_char_p, C.c_int32, C.c_int32, C.c_uint32, C.POINTER(_vp)]),
    "esp_cuda_gguf_inspect": (C.c_int32, [C.c_char_p, C.POINTER(EspCudaConfig), C.c_char_p, C.c_int32, _i32p, _i32p]),
    "esp_cuda_gguf_tensor_info": (C.c_int32, [C.c_char_p, C.c_int32, C.c_char_p, C.c_int32, C.c_char_p, C.c_int32, _i32p,
                                              C.POINTER(C.c_int64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "esp_cuda_create_from_gguf": (C.c_int32, [C.c_char_p, C.c_int32, C.c_int32, C.c_uint32, C.POINTER(_vp)]),
    "esp_cuda_load_tensor": (C.c_int32, [_vp, C.c_char_p, C.c_int32, _vp, C.c_uint64]),
    "esp_cuda_tp_unique_id": (C.c_int32, [C.POINTER(C.c_uint8), C.c_int32]),
    "esp_cuda_tp_init": (C.c_int32, [_vp, C.POINTER(C.c_uint8), C.c_int32]),
    "esp_cuda_finalize": (C.c_int32, [_vp]),
    "esp_cuda_destroy": (C.c_int32, [_vp]),
    "esp_cuda_get_config": (C.c_int32, [_vp, C.POINTER(EspCudaConfig)]),
    "esp_cuda_reset": (C.c_int32, [_vp]),
    "esp_cuda_prefill": (C.c_int32, [_vp, _u32p, C.c_int32]),
    "esp_cuda_advance": (C.c_int32, [_vp, C.c_uint32]),
    "esp_cuda_select_greedy": (C.c_int32, [_vp, _u32p]),
    "esp_cuda_decode_step": (C.c_int32, [_vp, C.c_uint32, _u32p]),
    "esp_cuda_visible_token_count": (C.c_int32, [_vp, C.c_int32, _i32p]),
    "esp_cuda_get_logits": (C.c_int32, [_vp, C.c_int32, _f32p, C.c_int32]),
    "esp_cuda_checkpoint": (C.c_int32, [_vp, _i32p]),
    "esp_cuda_rollback": (C.c_int32, [_vp, C.c_int32]),
    "esp_cuda_verify2": (C.c_int32, [_vp, C.c_uint32, C.c_uint32, _u32p, _u32p]),
    "esp_cuda_commit": (C.c_int32, [_vp, C.c_int32]),
    "esp_cuda_prefill_batch": (C.c_int32, [_vp, _u32p, C.c_int32, C.c_int32]),
    "esp_cuda_decode_step_batch": (C.c_int32, [_vp, _u32p, C.c_int32, _u32p]),
    "esp_cuda_decode": (C.c_int32, [_vp, C.c_int32, C.c_int32, _u32p, _i32p, _f32p]),
    "esp_cuda_generate": (C.c_int32, [_vp, _u32p, C.c_int32, C.c_int32, _u32p, _i32p, C.POINTER(EspCudaGenerationResult)]),
    "esp_cuda_generate_batch": (C.c_int32, [_vp, _u32p, C.c_int32, C.c_int32, C.c_int32, _u32p, _i32p, C.POINTER(EspCudaGenerationResult)]),
    "esp_cuda_generate_two_token": (C.c_int32, [_vp, _vp, _u32p, C.c_int32, C.c_int32, _u32p, _i32p, C.POINTER(EspCudaGenerationResult)]),
    "esp_cuda_get_timings": (C.c_int32, [_vp, C.POINTER(EspCudaTimings)]),
    "esp_cuda_stage_trace": (C.c_int32, [_vp, C.c_int32, C.POINTER(C.c_int64), C.c_int32, _i32p]),
    "esp_cuda_token_times": (C.c_int32, [_vp, C.POINTER(C.c_uint64), C.c_int32, _i32p]),
    "esp_cuda_set_debug_layer": (C.c_int32, [_vp, C.c_int32]),
    "esp_cuda_debug_dump": (C.c_int32, [_vp, C.c_int32, _f32p, C.c_int32]),
    "esp_cuda_last_error_string": (C.c_char_p, []),
    "esp_cuda_set_force_failure": (None, [C.c_int32]),
    "esp_cuda_set_wait_limit": (C.c_int32, [_vp, C.c_uint32]),
    "esp_cuda_generate_steps": (C.c_int32, [_vp, _u32p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, _u32p, _i32p, C.POINTER(EspCudaGenerationResult)]),
    "esp_cuda_token_latencies": (C.c_int32, [_vp, _f32p, C.c_int32, _i32p]),
    "esp_cuda_tp_sum_stats": (C.c_int32, [_vp, C.POINTER(C.c_uint64)]),
    "esp_cuda_live_engine_count": (C.c_int32, []),
    "esp_cuda_version": (C.c_char_p, []),
    "esp_cuda_dequantize": (C.c_int32, [C.c_int32, _vp, C.c_int64, _f32p, C.c_int32]),
    "esp_cuda_lm_head_argmax_static": (C.c_int32, [_vp, C.c_int32, C.c_int32, _vp, C.c_int32, _vp, C.c_float, _vp, _vp, C.c_int32]),
    "esp_cuda_gemm_tc_bench": (C.c_int32, [C.c_int32, _vp, C.c_int32, C.c_int32, _f32p, C.c_int32, _f32p, C.c_int32, C.c_int32, _f32p, C.c_int32]),
    "esp_cuda_gemv_bench": (C.c_int32, [C.c_int32, _vp, C.c_int32, C.c_int32, _f32p, _f32p, C.c_int32, C.c_int32, C.c_int32, _f32p, C.c_int32]),
}

_lib: Optional[C.CDLL] = None


def load_library() -> C.CDLL:
    """Load the CUDA library; raises if it is missing (there is no other implementation to fall back to)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m espresso_b200.build` (needs nvcc)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _check(status: int) -> None:
    if status != OK:
        msg = load_library().esp_cuda_last_error_string()
        raise RealModelInferenceError(status, msg.decode() if msg else "")


def _u32(a) -> tuple[np.ndarray, C.POINTER(C.c_uint32)]:
    arr = np.ascontiguousarray(a, dtype=np.uint32)
    return arr, arr.ctypes.data_as(_u32p)


@dataclasses.dataclass
class GenerationResult:
    """Numeric fields of the reference's ``GenerationResult`` (Engine.swift:17-55)."""
    tokens: np.ndarray
    promptTokens: np.ndarray
    tokensPerSecond: float
    prefillMs: float
    firstTokenLatencyMs: float
    totalDecodeMs: float
    committedExactTokensPerPass: Optional[float] = None
    acceptedFutureTokensPerPass: Optional[float] = None
    speculativePasses: int = 0
    stoppedOnEOS: bool = False
    tokenLatenciesMs: Optional[np.ndarray] = None


def make_c_config(cfg: MultiModelConfig, max_batch: int = 1, device: int = 0, flags: int = 0, tp_rank: int = 0,
                  tp_size: int = 1) -> EspCudaConfig:
    return EspCudaConfig(
        1 if cfg.architecture == "gpt2" else 0, cfg.nLayer, cfg.nHead, cfg.nKVHead, cfg.dModel, cfg.headDim,
        cfg.hiddenDim, cfg.vocab, cfg.maxSeq, cfg.normEps, cfg.ropeTheta, -1 if cfg.eosToken is None else cfg.eosToken,
        max_batch, device, tp_rank, tp_size, flags)


class DecodeEngine:
    """One model replica on one GPU."""

    def __init__(self, handle: int, config: MultiModelConfig, max_batch: int):
        self._h = C.c_void_p(handle)
        self.config = config
        self.max_batch = max_batch
        self._lib = load_library()

    # ---- construction (RealModelInferenceEngine.build, Engine.swift:1377) ----
    @classmethod
    def build(cls, weight_dir: str, config: Optional[MultiModelConfig] = None, max_batch: int = 1, device: int = 0,
              flags: int = 0) -> "DecodeEngine":
        lib = load_library()
        out = C.c_void_p()
        if config is None:
            config = MultiModelConfig.load(weight_dir)
        cc = make_c_config(config, max_batch, device, flags)
        _check(lib.esp_cuda_create(C.byref(cc), os.fsencode(weight_dir), C.byref(out)))
        return cls(out.value, config, max_batch)

    @classmethod
    def from_gguf(cls, path: str, max_batch: int = 1, device: int = 0, flags: int = 0) -> "DecodeEngine":
        """An engine built straight from a ``.gguf`` file (GGUFModelLoader.prepare + engine construction)."""
        config, _, _, _ = gguf_inspect(path)
        out = C.c_void_p()
        _check(load_library().esp_cuda_create_from_gguf(os.fsencode(path), max_batch, device, flags, C.byref(out)))
        return cls(out.value, config, max_batch)

    @classmethod
    def empty(cls, config: MultiModelConfig, max_batch: int = 1, device: int = 0, flags: int = 0, tp_rank: int = 0,
              tp_size: int = 1) -> "DecodeEngine":
        """An engine whose tensors are uploaded with :meth:`load_tensor` and sealed with :meth:`finalize`.

        With ``tp_size > 1`` this is one rank of a tensor-parallel group: upload the rank's Megatron shard
        (see :func:`espresso_b200.sharding.tp_shard`) and call :meth:`tp_init` before :meth:`finalize`."""
        lib = load_library()
        config.validate()
        out = C.c_void_p()
        cc = make_c_config(config, max_batch, device, flags, tp_rank, tp_size)
        _check(lib.esp_cuda_create(C.byref(cc), None, C.byref(out)))
        return cls(out.value, config, max_batch)

    def load_tensor(self, name: str, kind: str, data) -> None:
        """``data``: a numpy array (host) or an ``(address, nbytes)`` pair naming device memory."""
        if isinstance(data, tuple):
            ptr, nbytes = data
        else:
            arr = np.ascontiguousarray(data)
            self._keep = arr
            ptr, nbytes = arr.ctypes.data, arr.nbytes
        _check(self._lib.esp_cuda_load_tensor(self._h, name.encode(), TENSOR_TYPES[kind], C.c_void_p(ptr), nbytes))

    def tp_init(self, unique_id: bytes) -> None:
        """Join the NCCL communicator of the tensor-parallel group (collective: every rank calls it)."""
        buf = (C.c_uint8 * len(unique_id)).from_buffer_copy(unique_id)
        _check(self._lib.esp_cuda_tp_init(self._h, buf, len(unique_id)))

    def finalize(self) -> None:
        _check(self._lib.esp_cuda_finalize(self._h))

    def close(self) -> None:
        if self._h:
            self._lib.esp_cuda_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- decoder object (CPUExactLlamaRuntime) ----
    def reset(self) -> None:
        _check(self._lib.esp_cuda_reset(self._h))

    def prefill(self, prompt_tokens: Sequence[int]) -> None:
        arr, p = _u32(prompt_tokens)
        _check(self._lib.esp_cuda_prefill(self._h, p, arr.size))

    def advance(self, token: int) -> None:
        _check(self._lib.esp_cuda_advance(self._h, int(token)))

    def select_greedy_token(self) -> int:
        out = C.c_uint32()
        _check(self._lib.esp_cuda_select_greedy(self._h, C.byref(out)))
        return int(out.value)

    def decode_step(self, token: int) -> int:
        out = C.c_uint32()
        _check(self._lib.esp_cuda_decode_step(self._h, int(token), C.byref(out)))
        return int(out.value)

    def visible_token_count(self, seq: int = 0) -> int:
        out = C.c_int32()
        _check(self._lib.esp_cuda_visible_token_count(self._h, seq, C.byref(out)))
        return int(out.value)

    def logits(self, seq: int = 0) -> np.ndarray:
        out = np.empty(self.config.vocab, np.float32)
        _check(self._lib.esp_cuda_get_logits(self._h, seq, out.ctypes.data_as(_f32p), out.size))
        return out

    def capture_checkpoint(self) -> int:
        out = C.c_int32()
        _check(self._lib.esp_cuda_checkpoint(self._h, C.byref(out)))
        return int(out.value)

    def rollback(self, checkpoint: int) -> None:
        _check(self._lib.esp_cuda_rollback(self._h, checkpoint))

    def verify2(self, current: int, proposed_future: int) -> tuple[int, int]:
        a, b = C.c_uint32(), C.c_uint32()
        _check(self._lib.esp_cuda_verify2(self._h, int(current), int(proposed_future), C.byref(a), C.byref(b)))
        return int(a.value), int(b.value)

    def commit(self, steps: int) -> None:
        _check(self._lib.esp_cuda_commit(self._h, steps))

    # ---- batched decoder ----
    def prefill_batch(self, tokens) -> None:
        arr, p = _u32(tokens)
        assert arr.ndim == 2
        _check(self._lib.esp_cuda_prefill_batch(self._h, p, arr.shape[0], arr.shape[1]))

    def decode_step_batch(self, tokens) -> np.ndarray:
        arr, p = _u32(tokens)
        out = np.empty(arr.size, np.uint32)
        _check(self._lib.esp_cuda_decode_step_batch(self._h, p, arr.size, out.ctypes.data_as(_u32p)))
        return out

    def decode(self, count: int, n_seq: int = 1) -> tuple[list[np.ndarray], float]:
        """Device-driven greedy decode from the current state; returns (tokens per sequence, device ms)."""
        out = np.zeros((n_seq, max(count, 1)), np.uint32)
        n = np.zeros(n_seq, np.int32)
        ms = C.c_float()
        _check(self._lib.esp_cuda_decode(self._h, n_seq, count, out.ctypes.data_as(_u32p), n.ctypes.data_as(_i32p), C.byref(ms)))
        return [out[s, : n[s]].copy() for s in range(n_seq)], float(ms.value)

    # ---- generation (generate*ForTesting: token ids in, token ids out) ----
    def _result(self, res: EspCudaGenerationResult, tokens, prompt, two_token=False) -> GenerationResult:
        return GenerationResult(
            tokens=tokens, promptTokens=np.asarray(prompt, dtype=np.uint32), tokensPerSecond=res.tokens_per_second,
            prefillMs=res.prefill_ms, firstTokenLatencyMs=res.first_token_latency_ms, totalDecodeMs=res.total_decode_ms,
            committedExactTokensPerPass=res.committed_exact_tokens_per_pass if two_token else None,
            acceptedFutureTokensPerPass=res.accepted_future_tokens_per_pass if two_token else None,
            speculativePasses=res.speculative_passes, stoppedOnEOS=bool(res.stopped_on_eos),
            tokenLatenciesMs=None if two_token else self.token_latencies_ms())

    def token_latencies_ms(self) -> np.ndarray:
        """``GenerationResult.tokenLatenciesMs`` of the most recent generation of sequence 0 (see ``esp_cuda_token_latencies``)."""
        out = np.zeros(self.config.maxSeq + 1, np.float32)
        n = C.c_int32()
        _check(self._lib.esp_cuda_token_latencies(self._h, out.ctypes.data_as(_f32p), out.size, C.byref(n)))
        return out[: n.value].copy()

    def generate(self, prompt_tokens: Sequence[int], max_tokens: int = 128, on_step=None) -> GenerationResult:
        """Greedy generation.  With ``on_step(token, index, latency_ms)`` the loop runs token by token and calls it inline
        after every token (the reference's ``onStep``, Engine.swift:6393-6405); without it the loop is device-driven."""
        arr, p = _u32(prompt_tokens)
        out = np.zeros(max(max_tokens, 1), np.uint32)
        n = C.c_int32()
        res = EspCudaGenerationResult()
        if on_step is None:
            _check(self._lib.esp_cuda_generate(self._h, p, arr.size, max_tokens, out.ctypes.data_as(_u32p), C.byref(n), C.byref(res)))
        else:
            cb_type = C.CFUNCTYPE(None, C.c_void_p, C.c_uint32, C.c_int32, C.c_double)
            cb = cb_type(lambda _user, token, index, latency: on_step(int(token), int(index), float(latency)))
            _check(self._lib.esp_cuda_generate_steps(self._h, p, arr.size, max_tokens, C.cast(cb, C.c_void_p), None,
                                                     out.ctypes.data_as(_u32p), C.byref(n), C.byref(res)))
        return self._result(res, out[: n.value].copy(), arr)

    def generate_text(self, tokenizer, prompt: str, max_tokens: int = 128) -> tuple[str, GenerationResult]:
        """``generate(prompt:maxTokens:)`` on text (RealModelInferenceEngine.swift:1405-1460): the prompt is encoded
        with ``tokenizer`` (see :mod:`espresso_b200.tokenizers`), an empty encoding is ``invalidPrompt`` as in the
        reference (:5405-5408), and the generated ids are decoded back."""
        ids = tokenizer.encode(prompt)
        if not ids:
            raise RealModelInferenceError(ERR_INVALID_ARGUMENT, "Prompt produced no tokens")
        res = self.generate(ids, max_tokens)
        return tokenizer.decode([int(t) for t in res.tokens]), res

    def generate_batch(self, prompts, max_tokens: int = 128) -> tuple[list[np.ndarray], GenerationResult]:
        arr, p = _u32(prompts)
        assert arr.ndim == 2
        n_seq = arr.shape[0]
        out = np.zeros((n_seq, max(max_tokens, 1)), np.uint32)
        n = np.zeros(n_seq, np.int32)
        res = EspCudaGenerationResult()
        _check(self._lib.esp_cuda_generate_batch(self._h, p, n_seq, arr.shape[1], max_tokens, out.ctypes.data_as(_u32p),
                                                 n.ctypes.data_as(_i32p), C.byref(res)))
        toks = [out[s, : n[s]].copy() for s in range(n_seq)]
        return toks, self._result(res, np.concatenate(toks) if toks else out[:0], arr)

    def generate_two_token(self, draft: "DecodeEngine", prompt_tokens: Sequence[int], max_tokens: int = 128) -> GenerationResult:
        arr, p = _u32(prompt_tokens)
        out = np.zeros(max(max_tokens, 1), np.uint32)
        n = C.c_int32()
        res = EspCudaGenerationResult()
        _check(self._lib.esp_cuda_generate_two_token(self._h, draft._h, p, arr.size, max_tokens, out.ctypes.data_as(_u32p),
                                                     C.byref(n), C.byref(res)))
        return self._result(res, out[: n.value].copy(), arr, two_token=True)

    # ---- diagnostics ----
    def timings(self) -> dict:
        t = EspCudaTimings()
        _check(self._lib.esp_cuda_get_timings(self._h, C.byref(t)))
        return {k: getattr(t, k) for k, _ in EspCudaTimings._fields_}

    def tp_sum_stats(self) -> dict:
        """Peer-memory all-reduces of this rank since the previous call: count, mean device microseconds, mean wait for the peers."""
        out = (C.c_uint64 * 3)()
        _check(self._lib.esp_cuda_tp_sum_stats(self._h, out))
        n = int(out[0])
        return {"count": n, "mean_us": out[1] / n / 1e3 if n else 0.0, "mean_wait_us": out[2] / n / 1e3 if n else 0.0}

    def stage_trace(self, next_cta: int = 0) -> np.ndarray:
        """SM clock stamps of the persistent kernel's last token (see ``esp_cuda_stage_trace``)."""
        out = np.zeros(max(1024, 10 * self.config.nLayer + 8), np.int64)
        n = C.c_int32()
        _check(self._lib.esp_cuda_stage_trace(self._h, next_cta, out.ctypes.data_as(C.POINTER(C.c_int64)), out.size, C.byref(n)))
        return out[: n.value].copy()

    def token_times_ns(self) -> np.ndarray:
        """GPU timer value (ns) at which each token of the last persistent decode loop became known (empty otherwise)."""
        out = np.zeros(self.config.maxSeq + 1, np.uint64)
        n = C.c_int32()
        _check(self._lib.esp_cuda_token_times(self._h, out.ctypes.data_as(C.POINTER(C.c_uint64)), out.size, C.byref(n)))
        return out[: n.value].copy()

    def set_wait_limit(self, spins: int) -> None:
        """Test hook: every device-side wait of the persistent decode kernel polls at most ``spins`` times (0 = default)."""
        _check(self._lib.esp_cuda_set_wait_limit(self._h, spins))

    def set_debug_layer(self, layer: int) -> None:
        _check(self._lib.esp_cuda_set_debug_layer(self._h, layer))

    def debug_dump(self, stage: int) -> np.ndarray:
        c = self.config
        sizes = [c.attentionDim, c.kvDim, c.kvDim, c.attentionDim, c.dModel, c.hiddenDim, c.dModel]
        out = np.empty(sizes[stage], np.float32)
        _check(self._lib.esp_cuda_debug_dump(self._h, stage, out.ctypes.data_as(_f32p), out.size))
        return out


def tp_unique_id() -> bytes:
    """A fresh NCCL unique id (rank 0 creates it and shares the bytes with the other ranks)."""
    buf = (C.c_uint8 * 128)()
    _check(load_library().esp_cuda_tp_unique_id(buf, 128))
    return bytes(buf)


def set_force_failure(enabled: bool) -> None:
    load_library().esp_cuda_set_force_failure(int(enabled))


def live_engine_count() -> int:
    return load_library().esp_cuda_live_engine_count()


def dequantize(kind: str, blocks: np.ndarray, n_elements: int, device: int = 0) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.empty(n_elements, np.float32)
    _check(load_library().esp_cuda_dequantize(TENSOR_TYPES[kind], C.c_void_p(blocks.ctypes.data), n_elements,
                                              out.ctypes.data_as(_f32p), device))
    return out


STATIC_HEAD_MAX_ROWS = 64


def lm_head_argmax_static(lm_head_ptr: int, vocab: int, d_model: int, hidden_ptr: int, rows: int, gain_ptr: Optional[int],
                          eps: float, tokens_ptr: int, stream: int = 0, device: int = 0) -> None:
    """Allocation-free final norm + LM head + argmax; every ``*_ptr`` is a device address owned by the caller."""
    _check(load_library().esp_cuda_lm_head_argmax_static(
        C.c_void_p(lm_head_ptr), vocab, d_model, C.c_void_p(hidden_ptr), rows, C.c_void_p(gain_ptr) if gain_ptr else None,
        eps, C.c_void_p(tokens_ptr), C.c_void_p(stream) if stream else None, device))


def gguf_inspect(path: str) -> tuple[MultiModelConfig, str, int, bool]:
    """``(model shape, GGUF architecture name, tensor count, LM head tied to the embedding)`` of a ``.gguf`` file."""
    cc = EspCudaConfig()
    name = C.create_string_buffer(64)
    n, tied = C.c_int32(), C.c_int32()
    _check(load_library().esp_cuda_gguf_inspect(os.fsencode(path), C.byref(cc), name, 64, C.byref(n), C.byref(tied)))
    arch = "gpt2" if cc.architecture == 1 else "llama"
    cfg = MultiModelConfig(name.value.decode(), cc.n_layer, cc.n_head, cc.n_kv_head, cc.d_model, cc.head_dim, cc.hidden_dim, cc.vocab,
                           cc.max_seq, cc.norm_eps, cc.rope_theta, None if cc.eos_token < 0 else cc.eos_token, arch)
    return cfg, name.value.decode(), int(n.value), bool(tied.value)


def gguf_tensors(path: str) -> list[dict]:
    """The tensor directory of a ``.gguf`` file: name, mapped weight-directory path, GGML type, dims, offset, bytes."""
    _, _, n, _ = gguf_inspect(path)
    out = []
    for i in range(n):
        name, slot = C.create_string_buffer(256), C.create_string_buffer(256)
        t, dims, off, nb = C.c_int32(), (C.c_int64 * 4)(), C.c_uint64(), C.c_uint64()
        _check(load_library().esp_cuda_gguf_tensor_info(os.fsencode(path), i, name, 256, slot, 256, C.byref(t), dims, C.byref(off), C.byref(nb)))
        out.append({"name": name.value.decode(), "slot": slot.value.decode(), "type": int(t.value), "dims": [int(d) for d in dims],
                    "offset": int(off.value), "nbytes": int(nb.value)})
    return out


def gemm_tc_bench(kind: str, weights: np.ndarray, rows: int, cols: int, x: np.ndarray, warmup: int = 3, iterations: int = 20,
                  device: int = 0) -> tuple[np.ndarray, float]:
    """Tensor-core ``Y = X . W^T`` for a batch ``x`` of shape ``[n, cols]``; returns ``(Y [n, rows], mean kernel ms)``."""
    w = np.ascontiguousarray(weights)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n = x.shape[0]
    y = np.empty((n, rows), np.float32)
    ms = C.c_float()
    _check(load_library().esp_cuda_gemm_tc_bench(TENSOR_TYPES[kind], C.c_void_p(w.ctypes.data), rows, cols, x.ctypes.data_as(_f32p), n,
                                                 y.ctypes.data_as(_f32p), warmup, iterations, C.byref(ms), device))
    return y, float(ms.value)


def gemv_bench(kind: str, weights: np.ndarray, rows: int, cols: int, x: np.ndarray, warmup: int = 3, iterations: int = 20,
               copies: int = 1, device: int = 0) -> tuple[np.ndarray, float]:
    """Runs ``y = W.x`` on the device; returns ``(y, mean kernel milliseconds)``."""
    w = np.ascontiguousarray(weights)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(rows, np.float32)
    ms = C.c_float()
    _check(load_library().esp_cuda_gemv_bench(TENSOR_TYPES[kind], C.c_void_p(w.ctypes.data), rows, cols, x.ctypes.data_as(_f32p),
                                              y.ctypes.data_as(_f32p), warmup, iterations, copies, C.byref(ms), device))
    return y, float(ms.value)

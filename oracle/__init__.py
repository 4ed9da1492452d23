"""ctypes binding of the CPU oracle (``espresso_oracle.c``).

TEST INFRASTRUCTURE ONLY.  The oracle restates the reference's CPU decode path and is what the
CUDA library is checked against.  Only the test-suite, the smoke check and the benchmark's CPU
baseline may import this package; nothing under ``espresso_b200/`` does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libespresso_oracle.so")

ARCH_LLAMA = 0
ARCH_GPT2 = 1


def build(force: bool = False) -> str:
    """Compile the oracle shared library with the committed Makefile."""
    src = os.path.join(_HERE, "espresso_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


class Config(C.Structure):
    _fields_ = [
        ("architecture", C.c_int32),
        ("n_layer", C.c_int32),
        ("n_head", C.c_int32),
        ("n_kv_head", C.c_int32),
        ("d_model", C.c_int32),
        ("head_dim", C.c_int32),
        ("hidden_dim", C.c_int32),
        ("vocab", C.c_int32),
        ("max_seq", C.c_int32),
        ("norm_eps", C.c_float),
        ("rope_theta", C.c_float),
        ("eos_token", C.c_int32),
    ]


class TwoTokenStats(C.Structure):
    _fields_ = [("passes", C.c_int), ("committed_exact_tokens", C.c_int), ("accepted_future_tokens", C.c_int)]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        build()
    L = C.CDLL(_LIB_PATH)
    f32p = C.POINTER(C.c_float)
    u32p = C.POINTER(C.c_uint32)
    u8p = C.POINTER(C.c_uint8)
    vp = C.c_void_p

    def sig(name, res, *args):
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = list(args)

    sig("esp_oracle_half_to_float", C.c_float, C.c_uint16)
    sig("esp_oracle_float_to_half", C.c_uint16, C.c_float)
    sig("esp_oracle_gemv", None, f32p, C.c_int, C.c_int, f32p, f32p)
    sig("esp_oracle_rmsnorm", None, f32p, f32p, C.c_int, C.c_float, f32p)
    sig("esp_oracle_layernorm", None, f32p, f32p, f32p, C.c_int, C.c_float, f32p)
    sig("esp_oracle_per_head_rmsnorm", None, f32p, f32p, C.c_int, C.c_int, C.c_float)
    sig("esp_oracle_rope_half_split", None, f32p, C.c_int, C.c_int, C.c_int, C.c_float)
    sig("esp_oracle_decode_context", None, f32p, f32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p)
    sig("esp_oracle_silu", C.c_float, C.c_float)
    sig("esp_oracle_gelu", C.c_float, C.c_float)
    sig("esp_oracle_argmax_first", C.c_int, f32p, C.c_int)
    sig("esp_oracle_partitioned_argmax", C.c_int, f32p, f32p, C.c_int, C.c_int, C.c_int)
    sig("esp_oracle_quantize_q8_0", None, f32p, C.c_int64, u8p)
    sig("esp_oracle_dequantize_q8_0", None, u8p, C.c_int64, f32p)
    sig("esp_oracle_quantize_q4_0", None, f32p, C.c_int64, u8p)
    sig("esp_oracle_dequantize_q4_0", None, u8p, C.c_int64, f32p)
    sig("esp_oracle_blob_write", C.c_int, C.c_char_p, C.POINTER(C.c_uint16), C.c_uint32)
    sig("esp_oracle_blob_read", C.c_int64, C.c_char_p, f32p, C.c_int64)
    sig("esp_oracle_validate_config", C.c_int, C.POINTER(Config))
    sig("esp_oracle_model_create", vp, C.POINTER(Config))
    sig("esp_oracle_model_destroy", None, vp)
    sig("esp_oracle_model_set_tensor", C.c_int, vp, C.c_char_p, f32p, C.c_int64)
    sig("esp_oracle_model_load_dir", C.c_int, vp, C.c_char_p)
    sig("esp_oracle_runtime_create", vp, vp, C.c_int)
    sig("esp_oracle_runtime_destroy", None, vp)
    sig("esp_oracle_runtime_reset", None, vp)
    sig("esp_oracle_runtime_advance", C.c_int, vp, C.c_uint32)
    sig("esp_oracle_runtime_prefill", C.c_int, vp, u32p, C.c_int)
    sig("esp_oracle_runtime_logits", None, vp, f32p)
    sig("esp_oracle_runtime_select_greedy", C.c_uint32, vp)
    sig("esp_oracle_runtime_visible", C.c_int, vp)
    sig("esp_oracle_runtime_last_hidden", f32p, vp)
    sig("esp_oracle_runtime_k_cache", f32p, vp, C.c_int)
    sig("esp_oracle_runtime_v_cache", f32p, vp, C.c_int)
    sig("esp_oracle_runtime_set_capture_layer", None, vp, C.c_int)
    sig("esp_oracle_runtime_captured", f32p, vp, C.c_int)
    sig("esp_oracle_runtime_checkpoint", vp, vp)
    sig("esp_oracle_runtime_rollback", None, vp, vp)
    sig("esp_oracle_checkpoint_destroy", None, vp)
    sig("esp_oracle_generate", C.c_int, vp, u32p, C.c_int, C.c_int, u32p)
    sig("esp_oracle_generate_two_token", C.c_int, vp, vp, u32p, C.c_int, C.c_int, u32p, C.POINTER(TwoTokenStats))
    sig("esp_oracle_two_token_plan", C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, u32p, u32p)
    sig("esp_oracle_num_threads", C.c_int)
    sig("esp_oracle_set_num_threads", None, C.c_int)
    _lib = L
    return L


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _u32(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint32))


def make_config(meta: dict) -> Config:
    """Build the oracle config from a ``metadata.json`` dictionary (ESPModelConfigIO key names)."""
    arch = meta["architecture"].lower()
    eos = meta.get("eosToken")
    return Config(
        ARCH_GPT2 if arch == "gpt2" else ARCH_LLAMA,
        meta["nLayer"], meta["nHead"], meta["nKVHead"], meta["dModel"], meta["headDim"], meta["hiddenDim"],
        meta["vocab"], meta["maxSeq"], float(meta["normEps"]), float(meta.get("ropeTheta") or 10000.0),
        -1 if eos is None else int(eos),
    )


# ---- thin functional wrappers used by the known-answer tests -------------------------------------

def gemv(w, x):
    w, wp = _f32(w)
    x, xp = _f32(x)
    y = np.empty(w.shape[0], np.float32)
    lib().esp_oracle_gemv(wp, w.shape[0], w.shape[1], xp, y.ctypes.data_as(C.POINTER(C.c_float)))
    return y


def rmsnorm(x, w, eps):
    x, xp = _f32(x)
    w, wp = _f32(w)
    y = np.empty_like(x)
    lib().esp_oracle_rmsnorm(xp, wp, x.size, eps, y.ctypes.data_as(C.POINTER(C.c_float)))
    return y


def layernorm(x, g, b, eps):
    x, xp = _f32(x)
    g, gp = _f32(g)
    b, bp = _f32(b)
    y = np.empty_like(x)
    lib().esp_oracle_layernorm(xp, gp, bp, x.size, eps, y.ctypes.data_as(C.POINTER(C.c_float)))
    return y


def per_head_rmsnorm(v, w, heads, head_dim, eps):
    v, vp = _f32(np.array(v, dtype=np.float32, copy=True))
    w, wp = _f32(w)
    lib().esp_oracle_per_head_rmsnorm(vp, wp, heads, head_dim, eps)
    return v


def rope_half_split(v, heads, head_dim, position, theta=10000.0):
    v, vp = _f32(np.array(v, dtype=np.float32, copy=True))
    lib().esp_oracle_rope_half_split(vp, heads, head_dim, position, theta)
    return v


def decode_context(q, k_cache, v_cache, heads, kv_heads, head_dim, visible, cache_stride, token_base=0):
    q, qp = _f32(q)
    k, kp = _f32(k_cache)
    v, vp = _f32(v_cache)
    ctx = np.empty(heads * head_dim, np.float32)
    lib().esp_oracle_decode_context(qp, kp, vp, heads, kv_heads, head_dim, visible, token_base, cache_stride,
                                    ctx.ctypes.data_as(C.POINTER(C.c_float)))
    return ctx


def silu(x):
    return lib().esp_oracle_silu(float(x))


def gelu(x):
    return lib().esp_oracle_gelu(float(x))


def argmax_first(v):
    v, vp = _f32(v)
    return lib().esp_oracle_argmax_first(vp, v.size)


def partitioned_argmax(classifier, x, block_size=4000):
    w, wp = _f32(classifier)
    x, xp = _f32(x)
    return lib().esp_oracle_partitioned_argmax(wp, xp, w.shape[0], w.shape[1], block_size)


def quantize(kind: str, x):
    x, xp = _f32(x)
    n = x.size
    assert n % 32 == 0
    per = 34 if kind == "q8_0" else 18
    out = np.empty(n // 32 * per, np.uint8)
    fn = lib().esp_oracle_quantize_q8_0 if kind == "q8_0" else lib().esp_oracle_quantize_q4_0
    fn(xp, n, out.ctypes.data_as(C.POINTER(C.c_uint8)))
    return out


def dequantize(kind: str, blocks, n):
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.empty(n, np.float32)
    fn = lib().esp_oracle_dequantize_q8_0 if kind == "q8_0" else lib().esp_oracle_dequantize_q4_0
    fn(blocks.ctypes.data_as(C.POINTER(C.c_uint8)), n, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def blob_write(path, fp16_bits):
    a = np.ascontiguousarray(fp16_bits, dtype=np.uint16)
    return lib().esp_oracle_blob_write(os.fsencode(path), a.ctypes.data_as(C.POINTER(C.c_uint16)), a.size)


def blob_read(path):
    n = lib().esp_oracle_blob_read(os.fsencode(path), None, 0)
    if n < 0:
        return int(n), None
    out = np.empty(n, np.float32)
    n2 = lib().esp_oracle_blob_read(os.fsencode(path), out.ctypes.data_as(C.POINTER(C.c_float)), n)
    return int(n2), out


class Model:
    """Weights of one model held as fp32 (the oracle's precision model)."""

    def __init__(self, meta: dict):
        self.meta = dict(meta)
        self.cfg = make_config(meta)
        self.handle = lib().esp_oracle_model_create(C.byref(self.cfg))
        if not self.handle:
            raise ValueError("invalid model config")

    @classmethod
    def from_dir(cls, weight_dir: str):
        import json

        with open(os.path.join(weight_dir, "metadata.json")) as f:
            meta = json.load(f)
        m = cls(meta)
        rc = lib().esp_oracle_model_load_dir(m.handle, os.fsencode(weight_dir))
        if rc != 0:
            raise RuntimeError(f"oracle failed to load {weight_dir}: {rc}")
        return m

    def set_tensor(self, name: str, values):
        a, p = _f32(values)
        rc = lib().esp_oracle_model_set_tensor(self.handle, name.encode(), p, a.size)
        if rc != 0:
            raise ValueError(f"set_tensor({name}) failed: {rc}")

    def __del__(self):
        if getattr(self, "handle", None):
            lib().esp_oracle_model_destroy(self.handle)
            self.handle = None


class Runtime:
    """Stateful single-sequence decoder mirroring the reference's CPU-exact runtime."""

    def __init__(self, model: Model, round_fp16: bool = False):
        self.model = model
        self.handle = lib().esp_oracle_runtime_create(model.handle, int(round_fp16))
        if not self.handle:
            raise RuntimeError("model is missing tensors")

    def reset(self):
        lib().esp_oracle_runtime_reset(self.handle)

    def advance(self, token: int) -> int:
        return lib().esp_oracle_runtime_advance(self.handle, int(token))

    def prefill(self, tokens) -> int:
        t, p = _u32(tokens)
        return lib().esp_oracle_runtime_prefill(self.handle, p, t.size)

    def logits(self):
        out = np.empty(self.model.cfg.vocab, np.float32)
        lib().esp_oracle_runtime_logits(self.handle, out.ctypes.data_as(C.POINTER(C.c_float)))
        return out

    def select_greedy(self) -> int:
        return int(lib().esp_oracle_runtime_select_greedy(self.handle))

    @property
    def visible(self) -> int:
        return lib().esp_oracle_runtime_visible(self.handle)

    def last_hidden(self):
        p = lib().esp_oracle_runtime_last_hidden(self.handle)
        return np.ctypeslib.as_array(p, (self.model.cfg.d_model,)).copy()

    def kv_cache(self, layer: int):
        c = self.model.cfg
        shape = (c.n_kv_head * c.head_dim, c.max_seq)
        k = np.ctypeslib.as_array(lib().esp_oracle_runtime_k_cache(self.handle, layer), shape).copy()
        v = np.ctypeslib.as_array(lib().esp_oracle_runtime_v_cache(self.handle, layer), shape).copy()
        return k, v

    def set_capture_layer(self, layer: int):
        lib().esp_oracle_runtime_set_capture_layer(self.handle, layer)

    def captured(self, stage: int):
        c = self.model.cfg
        sizes = [c.n_head * c.head_dim, c.n_kv_head * c.head_dim, c.n_kv_head * c.head_dim, c.n_head * c.head_dim,
                 c.d_model, c.hidden_dim, c.d_model]
        p = lib().esp_oracle_runtime_captured(self.handle, stage)
        return np.ctypeslib.as_array(p, (sizes[stage],)).copy()

    def checkpoint(self):
        return lib().esp_oracle_runtime_checkpoint(self.handle)

    def rollback(self, cp):
        lib().esp_oracle_runtime_rollback(self.handle, cp)

    def free_checkpoint(self, cp):
        lib().esp_oracle_checkpoint_destroy(cp)

    def generate(self, prompt, max_tokens: int):
        t, p = _u32(prompt)
        out = np.zeros(max(max_tokens, 1), np.uint32)
        n = lib().esp_oracle_generate(self.handle, p, t.size, max_tokens, out.ctypes.data_as(C.POINTER(C.c_uint32)))
        if n < 0:
            raise RuntimeError(f"oracle generate failed: {n}")
        return out[:n].copy()

    def __del__(self):
        if getattr(self, "handle", None):
            lib().esp_oracle_runtime_destroy(self.handle)
            self.handle = None


def generate_two_token(full: Runtime, draft: Runtime, prompt, max_tokens: int):
    t, p = _u32(prompt)
    out = np.zeros(max(max_tokens, 1), np.uint32)
    st = TwoTokenStats()
    n = lib().esp_oracle_generate_two_token(full.handle, draft.handle, p, t.size, max_tokens,
                                            out.ctypes.data_as(C.POINTER(C.c_uint32)), C.byref(st))
    if n < 0:
        raise RuntimeError(f"oracle two-token generate failed: {n}")
    return out[:n].copy(), {"passes": st.passes, "committed": st.committed_exact_tokens, "accepted": st.accepted_future_tokens}


def two_token_plan(current, proposed_future, exact_next, exact_future, remaining):
    committed = (C.c_uint32 * 2)()
    nxt = C.c_uint32()
    n = lib().esp_oracle_two_token_plan(current, proposed_future, exact_next, exact_future, remaining, committed, C.byref(nxt))
    return list(committed[:n]), int(nxt.value)

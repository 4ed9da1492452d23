"""Benchmark of the decode hot path.

A "step" is one pass of the hot path over one batch of synthetic input: a greedy decode of
``decode_tokens`` tokens for every sequence of the workload, continuing from a prefilled prompt.
``value`` is decode tokens/s with everything resident in HBM (device-timed with CUDA events);
``e2e`` is the same metric through the public generate call with host buffers (prompt upload, prefill,
decode, token download all inside the timed region).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1] [--impl ours|reference]
    python bench.py --kernel gemv|gemm --rows R --cols C --type f16|bf16|q8_0|q4_0 [--batch N]   # one stand-alone kernel

The second form times a single kernel on a matrix of the given shape and prints one JSON line (mean kernel
milliseconds, GB/s over the algorithmic bytes, TFLOP/s for the GEMM); it launches nothing but that kernel (plus, for
a K-sliced GEMM, the clearing of its output), which makes it the command the profiler summaries capture.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from espresso_b200 import model_config as mc  # noqa: E402
from espresso_b200.synthetic import synthetic_prompt, write_synthetic_model  # noqa: E402

WORKLOADS = {
    # cfg factory, prompt tokens, decode tokens, sequences per GPU (total for sharded jobs), weight storage
    "c1": dict(cfg=mc.llama_6l, prompt=16, decode=128, n_seq=1, kind="f16", bpw=2.0,
               label="llama 6L d768 12h vocab32000 ctx256 fp16, batch 1, 16-token prompt, 128 greedy steps"),
    "c2": dict(cfg=mc.llama_6l, draft=mc.llama_draft_1l, prompt=16, decode=128, n_seq=1, kind="f16", bpw=2.0,
               label="llama 6L d768 target + 1-layer draft, exact two-token verify, batch 1, 16-token prompt, 128 tokens"),
    "c3": dict(cfg=mc.gpt2_117m, prompt=64, decode=256, n_seq=256, sharded=True, kind="f16", bpw=2.0,
               label="gpt2-117M shape 12L d768 vocab50257 ctx1024 fp16, 256 independent sequences sharded over the GPUs, 64-token prompts, 256 greedy steps"),
    # profiling aid: the c3 shape truncated to 4 layers and 512 positions (1.6 GB of KV cache), decode at context ~450
    "c3long": dict(cfg=lambda: dataclasses.replace(mc.gpt2_117m(max_seq=512), nLayer=4, name="gpt2-117m-4l"), prompt=448, decode=16, n_seq=256,
                   sharded=True, kind="f16", bpw=2.0,
                   label="gpt2-117M widths, 4 layers, ctx512, 256 sequences, 448-token prompts, 16 greedy steps (attention at long context)"),
    "c5": dict(cfg=mc.llama3_8b, prompt=512, decode=256, n_seq=64, kind="bf16", bpw=2.0, device_weights=True, tp=True,
               label="llama-3-8B shape 32L d4096 GQA 32/8 hd128 vocab128256 ctx1024 bf16, 64 sequences, 512-token prompts, 256 greedy steps, tensor parallel over the GPUs (sum after Wo and W2 over peer memory)"),
    "c4q8": dict(cfg=mc.llama_1b, prompt=128, decode=256, n_seq=1, kind="q8_0", bpw=34.0 / 32, device_weights=True,
                 label="llama 1.1B shape 22L d2048 GQA 32/4 ctx2048, GGUF Q8_0 matrices + LM head, batch 1, 128-token prompt, 256 steps"),
    "c4q4": dict(cfg=mc.llama_1b, prompt=128, decode=256, n_seq=1, kind="q4_0", bpw=18.0 / 32, device_weights=True,
                 label="llama 1.1B shape 22L d2048 GQA 32/4 ctx2048, GGUF Q4_0 matrices + LM head, batch 1, 128-token prompt, 256 steps"),
    "c4q8b16": dict(cfg=mc.llama_1b, prompt=128, decode=256, n_seq=16, kind="q8_0", bpw=34.0 / 32, device_weights=True,
                    label="llama 1.1B shape Q8_0, batch 16, 128-token prompts, 256 steps"),
    "c4q4b16": dict(cfg=mc.llama_1b, prompt=128, decode=256, n_seq=16, kind="q4_0", bpw=18.0 / 32, device_weights=True,
                    label="llama 1.1B shape Q4_0, batch 16, 128-token prompts, 256 steps"),
}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v for v in vis.split(",") if v.strip()]
        if local_rank < len(ids) and ids[local_rank].strip().isdigit():
            return int(ids[local_rank])
    return local_rank


def algorithmic_bytes_per_token(cfg, prompt: int, decode: int, n_seq: int, bytes_per_weight: float) -> float:
    """bytes(t) = W / n_seq + KVr * visible + KVw, averaged over the forward steps of one run."""
    w = cfg.weight_bytes_per_step(bytes_per_weight)
    kv = cfg.kv_bytes_per_visible_token()
    visible = [prompt + i + 1 for i in range(1, decode)]  # each forward step attends to this many positions
    mean_vis = sum(visible) / max(len(visible), 1)
    return w / n_seq + kv * mean_vis + kv


def truncated(cfg, n_layer):
    import dataclasses
    return dataclasses.replace(cfg, nLayer=n_layer, name=f"{cfg.name}-{n_layer}l")


def time_oracle_decode(weight_dir: str, prompt, decode: int, steps: int, warmup: int) -> list[float]:
    """Seconds per decode run (prefill untimed) of the CPU restatement of the reference's path."""
    import oracle

    rt = oracle.Runtime(oracle.Model.from_dir(weight_dir))
    times = []
    for i in range(warmup + steps):
        assert rt.prefill(prompt) == 0
        t0 = time.perf_counter()
        tok = rt.select_greedy()
        for _ in range(decode - 1):
            assert rt.advance(tok) == 0
            tok = rt.select_greedy()
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    return times


def run_cpu_oracle(workload: dict, steps: int, warmup: int, threads: int | None = None) -> dict:
    """Times the CPU restatement of the reference's decode path on the host cores.

    Small models run the whole workload.  For the larger shapes one sequence is decoded for a few tokens on
    1- and 2-layer truncations of the model and the per-token time is extrapolated linearly in the layer count
    (per-layer cost = t(2 layers) - t(1 layer); the remainder is embedding + head); the sample says so.
    """
    import oracle

    lib = oracle.lib()
    # all host cores, also under torchrun (which exports OMP_NUM_THREADS=1 to its workers)
    lib.esp_oracle_set_num_threads(threads or len(os.sched_getaffinity(0)))
    cores = lib.esp_oracle_num_threads()
    cfg = workload["cfg"]()
    decode = workload["decode"]
    prompt = synthetic_prompt(cfg.vocab, workload["prompt"])
    small = cfg.nLayer * cfg.dModel * cfg.hiddenDim < 6 * 768 * 2048 * 1.5 and not workload.get("sharded")
    tmp = tempfile.mkdtemp(prefix="esp_cpu_")
    try:
        if small and "draft" not in workload:
            write_synthetic_model(cfg, tmp)
            times = time_oracle_decode(tmp, prompt, decode, steps, warmup)
            total = sum(times)
            return {"value": decode * len(times) / total, "ms_per_step": 1e3 * total / len(times), "cores": cores,
                    "sample": f"full workload per step: {workload['prompt']}-token prompt (untimed prefill) + {decode} greedy decode steps, {len(times)} steps"}
        if "draft" in workload:
            # the reference's two-token loop on the CPU: target and draft advance token by token (Engine.swift:6014-6190)
            write_synthetic_model(cfg, tmp)
            dtmp = tempfile.mkdtemp(prefix="esp_cpu_draft_")
            write_synthetic_model(workload["draft"](), dtmp, seed=1235)
            full = oracle.Runtime(oracle.Model.from_dir(tmp))
            draft = oracle.Runtime(oracle.Model.from_dir(dtmp))
            times = []
            for i in range(warmup + steps):
                t0 = time.perf_counter()
                toks, st = oracle.generate_two_token(full, draft, prompt, decode)
                if i >= warmup:
                    times.append(time.perf_counter() - t0)
            shutil.rmtree(dtmp, ignore_errors=True)
            total = sum(times)
            return {"value": decode * len(times) / total, "ms_per_step": 1e3 * total / len(times), "cores": cores,
                    "sample": f"full two-token loop incl. token-by-token prefill of target and draft, {decode} tokens, {len(times)} steps"}
        few = 8
        per = {}
        for nl in (1, 2):
            d = os.path.join(tmp, f"l{nl}")
            write_synthetic_model(truncated(cfg, nl), d)
            per[nl] = min(time_oracle_decode(d, prompt[:16], few, 1, 1)) / few
            shutil.rmtree(d, ignore_errors=True)
        layer = max(per[2] - per[1], 1e-9)
        tok_s = 1.0 / (per[1] - layer + cfg.nLayer * layer)
        return {"value": tok_s, "ms_per_step": 1e3 * decode / tok_s, "cores": cores,
                "sample": f"one sequence, {few} decode steps at context ~16 on 1- and 2-layer truncations of the fp32 model, "
                          f"per-token time extrapolated linearly to {cfg.nLayer} layers; sequences are decoded one at a time on the CPU"}
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def gemv_table(runtime, device: int, peak: float) -> dict:
    """Kernel-level y = W.x bandwidth for every weight storage type (matrix copies rotate so that reads miss L2)."""
    import numpy as np
    from espresso_b200 import gguf_quant

    out = {}
    rng = np.random.default_rng(7)
    rows, cols = 32768, 4096  # an LM-head sized matrix: 268 MB fp16, 143 MB Q8_0, 75 MB Q4_0
    w = (rng.standard_normal((rows, cols)).astype(np.float32) * np.float32(0.02))
    x = rng.standard_normal(cols).astype(np.float32)
    for kind, bpw in (("f16", 2.0), ("bf16", 2.0), ("q8_0", 34 / 32), ("q4_0", 18 / 32)):
        if kind == "f16":
            stored = w.astype(np.float16)
        elif kind == "bf16":
            stored = (w.view(np.uint32) >> 16).astype(np.uint16)
        else:
            stored = gguf_quant.quantize(kind, w)
        nbytes = rows * cols * bpw
        copies = max(2, int(400e6 // nbytes) + 1)
        _, ms = runtime.gemv_bench(kind, stored, rows, cols, x, warmup=5, iterations=40, copies=copies, device=device)
        gbs = (nbytes + cols * 4 + rows * 4) / (ms / 1e3) / 1e9
        out[kind] = {"rows": rows, "cols": cols, "ms": ms, "GBps": gbs, "frac_of_hbm_peak": gbs / peak}
    return out


def stage_trace_us(eng, cfg, prompt, n_decode: int, sm_mhz: float) -> dict:
    """Per-layer averages (microseconds) of the persistent kernel's stage stamps for the last decoded token; empty when
    the engine decodes with the per-stage kernels."""
    import numpy as np

    names = ["x_wait_norm", "qkv_rows", "qkv_wait", "attention", "wo_partial", "xmid_wait_norm", "gate_up", "act_wait", "down"]
    eng.prefill(prompt)
    eng.decode(n_decode)
    eng.stage_trace(100)  # selects the CTA whose stamps the next loop records
    eng.prefill(prompt)
    eng.decode(n_decode)
    t = eng.stage_trace(100).astype(np.float64) / sm_mhz
    L = cfg.nLayer
    if t.size < 10 * L + 4 or not t.any():
        return {}
    per = np.zeros(9)
    for layer in range(L):
        per += np.diff(t[10 * layer:10 * layer + 10])
    head = np.diff(t[10 * L:10 * L + 4])
    out = {n: round(float(v) / L, 2) for n, v in zip(names, per)}
    out.update({"layer_total": round(float(t[10 * L] - t[0]) / L, 2), "head_x_wait": round(float(head[0]), 2), "head_rows": round(float(head[1]), 2),
                "head_token_wait": round(float(head[2]), 2),
                "cta": 100, "note": "per-layer means over the last token, SM clock stamps of one CTA; *_wait = polling for another CTA's words"})
    return out


def cpu_model() -> str:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def gemm_table(runtime, device: int, peak: float) -> dict:
    """Kernel-level Y = X.W^T on the tensor cores (the batched path's product) on an LM-head sized fp16 matrix."""
    import numpy as np

    out = {}
    rng = np.random.default_rng(11)
    rows, cols = 32768, 4096  # 268 MB of weights: every launch streams them from HBM
    w = (rng.standard_normal((rows, cols)).astype(np.float32) * np.float32(0.02)).astype(np.float16)
    for n in (16, 64, 256):
        x = rng.standard_normal((n, cols)).astype(np.float32)
        _, ms = runtime.gemm_tc_bench("f16", w, rows, cols, x, warmup=5, iterations=40, device=device)
        nbytes = rows * cols * 2 + n * cols * 2 + n * rows * 4  # weights + 16-bit operand rows + fp32 result
        out[f"n{n}"] = {"rows": rows, "cols": cols, "batch": n, "ms": ms, "GBps": nbytes / (ms / 1e3) / 1e9,
                        "frac_of_hbm_peak": nbytes / (ms / 1e3) / 1e9 / peak, "TFLOPs": 2.0 * rows * cols * n / (ms / 1e3) / 1e12}
    return out


def run_kernel_probe(args) -> None:
    """Times one stand-alone kernel of the library on a seeded matrix (see the module docstring)."""
    from espresso_b200 import gguf_quant, runtime

    bpw = {"f16": 2.0, "bf16": 2.0, "q8_0": 34 / 32, "q4_0": 18 / 32}[args.type]
    rng = np.random.default_rng(3)
    w = rng.standard_normal((args.rows, args.cols)).astype(np.float32) * np.float32(0.02)
    stored = w.astype(np.float16) if args.type == "f16" else (w.view(np.uint32) >> 16).astype(np.uint16) if args.type == "bf16" else gguf_quant.quantize(args.type, w)
    wbytes = args.rows * args.cols * bpw
    if args.kernel == "gemm":
        x = rng.standard_normal((args.batch, args.cols)).astype(np.float32)
        _, ms = runtime.gemm_tc_bench(args.type, stored, args.rows, args.cols, x, args.warmup, args.iterations, 0)
        nbytes = wbytes + args.batch * args.cols * 2 + args.batch * args.rows * 4
        flops = 2.0 * args.rows * args.cols * args.batch
    else:
        x = rng.standard_normal(args.cols).astype(np.float32)
        copies = max(2, int(400e6 // wbytes) + 1)  # rotate copies so that reads miss L2
        _, ms = runtime.gemv_bench(args.type, stored, args.rows, args.cols, x, args.warmup, args.iterations, copies, 0)
        nbytes = wbytes + args.cols * 4 + args.rows * 4
        flops = 2.0 * args.rows * args.cols
    print(json.dumps({"kernel": args.kernel, "type": args.type, "rows": args.rows, "cols": args.cols,
                      "batch": args.batch if args.kernel == "gemm" else 1, "ms": ms, "algorithmic_bytes": nbytes,
                      "GBps": nbytes / (ms / 1e3) / 1e9, "TFLOPs": flops / (ms / 1e3) / 1e12}))


def config_of(wl: dict, world: int) -> dict:
    """The `config` object of a bench line: identical for both arms (ours and --impl reference)."""
    if world > 1:
        par = ("tensor parallel over the GPUs, partial sums after Wo and W2 added over NVLink peer memory, arg-max over NCCL" if wl.get("tp") else
               "sequences sharded across GPUs, no collective" if wl.get("sharded") else
               "replicas only (one independent job per GPU)")
    else:
        par = "single GPU"
    return {"workload": wl["label"], "parallelism": par,
            "l2": "no flush: every decode step streams more weight + KV bytes than the 126 MB L2 holds"}


def measure(args, wl: dict, rank: int, local_rank: int, world: int, steps: int, warmup: int, full: bool) -> dict:
    """Times one workload on this job's GPUs (every rank calls it).  Returns the numbers of a bench line; with `full`
    also the end-to-end figure through the public generate call and, for the persistent kernel, its stage trace."""
    import torch
    import torch.distributed as dist

    from espresso_b200 import runtime
    from espresso_b200.sharding import shard_range

    cfg = wl["cfg"]()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    tmp = tempfile.mkdtemp(prefix=f"esp_bench_r{rank}_")
    eng = draft = None
    try:
        n_prompt, n_decode = wl["prompt"], wl["decode"]
        tp = bool(wl.get("tp")) and world > 1
        if wl.get("tp"):
            n_seq, first_stream, scaling = wl["n_seq"], 0, "strong"  # every rank drives the same sequences
        elif wl.get("sharded"):
            b, e = shard_range(wl["n_seq"], rank, world)
            n_seq, first_stream, scaling = e - b, b, "strong"
        else:
            n_seq, first_stream, scaling = wl["n_seq"], rank * wl["n_seq"], "weak"
        prompts = np.stack([synthetic_prompt(cfg.vocab, n_prompt, stream=first_stream + s) for s in range(n_seq)])
        flags = runtime.FLAG_NO_MEGAKERNEL if args.per_stage else 0
        if wl.get("device_weights"):
            from espresso_b200.synthetic_device import upload_synthetic

            eng = runtime.DecodeEngine.empty(cfg, max_batch=n_seq, device=local_rank, flags=flags, tp_rank=rank if tp else 0,
                                             tp_size=world if tp else 1)
            if tp:
                ids = [runtime.tp_unique_id() if rank == 0 else None]
                dist.broadcast_object_list(ids, src=0)
                eng.tp_init(ids[0])
            upload_synthetic(eng, cfg, wl["kind"], device=local_rank, tp_rank=rank if tp else 0, tp_size=world if tp else 1)
        else:
            write_synthetic_model(cfg, tmp)
            eng = runtime.DecodeEngine.build(tmp, max_batch=n_seq, device=local_rank, flags=flags)
        if "draft" in wl:
            dtmp = os.path.join(tmp, "draft")
            write_synthetic_model(wl["draft"](), dtmp, seed=1235)
            draft = runtime.DecodeEngine.build(dtmp, device=local_rank, flags=flags)

        prefill_s = []  # wall time of every prompt pass (the call returns after the device has finished)

        def prefill():
            t0 = time.perf_counter()
            if n_seq == 1:
                eng.prefill(prompts[0])
            else:
                eng.prefill_batch(prompts)
            torch.cuda.synchronize()
            prefill_s.append(time.perf_counter() - t0)

        sampler = ClockSampler(physical_gpu_index(local_rank))
        step_ms, launches, extra = [], 0, {}
        if draft is None:
            # ---- device-resident throughput: K timed steps, each a device-driven decode of n_decode tokens ----
            prefill()
            cp = eng.capture_checkpoint() if n_seq == 1 else None
            for _ in range(warmup):
                if cp is not None:
                    eng.rollback(cp)
                else:
                    prefill()
                eng.decode(n_decode, n_seq)
            barrier()
            sampler.start()
            for _ in range(steps):
                if cp is not None:
                    eng.rollback(cp)  # positions return to the end of the prompt; KV slots are simply overwritten
                else:
                    prefill()
                if tp:
                    eng.tp_sum_stats()  # (clears the counters: what follows covers the decode steps only)
                toks, ms = eng.decode(n_decode, n_seq)
                assert all(len(t) == n_decode for t in toks) or cfg.architecture == "gpt2"
                step_ms.append(ms)
                launches += eng.timings()["kernel_launches"]
                if tp:
                    extra["tp_sum"] = eng.tp_sum_stats()
            barrier()
        else:
            # ---- two-token speculative loop (one device-driven launch when draft and target share their widths, else
            # host-driven passes), timed on the host from the end of prefill ----
            for _ in range(warmup):
                eng.generate_two_token(draft, prompts[0], n_decode)
            barrier()
            sampler.start()
            acc, com = [], []
            for _ in range(steps):
                res = eng.generate_two_token(draft, prompts[0], n_decode)
                assert len(res.tokens) == n_decode
                step_ms.append(res.totalDecodeMs)
                acc.append(res.acceptedFutureTokensPerPass)
                com.append(res.committedExactTokensPerPass)
                per_call = eng.timings()["kernel_launches"]
                fused = per_call == 1  # a host-driven verify pass is dozens of launches
                launches += 1 if fused else res.speculativePasses * (per_call + draft.timings()["kernel_launches"])
            barrier()
            extra["two_token"] = {"accepted_future_tokens_per_pass": statistics.mean(acc), "committed_exact_tokens_per_pass": statistics.mean(com),
                                  "loop": "one launch of k_spec_mega (draft, two-position verify and commit rule on the device)" if fused else "host-driven passes",
                                  "note": "draft and target are independent random models, so proposals are almost never accepted"}
        clocks = sampler.stop()
        total_ms = sum(step_ms)

        # ---- end to end through the public generate call with host buffers ----
        e2e_total = None
        if full:
            e2e_times = []
            for i in range(warmup + steps):
                t0 = time.perf_counter()
                if draft is not None:
                    res = eng.generate_two_token(draft, prompts[0], n_decode)
                elif n_seq == 1:
                    res = eng.generate(prompts[0], n_decode)
                else:
                    _, res = eng.generate_batch(prompts, n_decode)
                torch.cuda.synchronize()
                if i >= warmup:
                    e2e_times.append(time.perf_counter() - t0)
            e2e_total = sum(e2e_times)

        tokens_local = n_seq * n_decode * steps
        if wl.get("tp") and world > 1 and rank != 0:
            tokens_local = 0  # the ranks of a tensor-parallel group decode the same sequences together
        if world > 1:
            t = torch.tensor([total_ms, e2e_total or 0.0], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total_ms, e2e_max = float(t[0]), float(t[1])
            e2e_total = e2e_max if e2e_total is not None else None
            lt = torch.tensor([launches, tokens_local], dtype=torch.int64, device="cuda")
            dist.all_reduce(lt)
            launches, tokens_all = int(lt[0]), int(lt[1])
        else:
            tokens_all = tokens_local
        value = tokens_all / (total_ms / 1e3)

        # ---- roofline of the dominant kernel, timed live with CUDA events ----
        peak, peak_kind = read_peaks()
        bpw = wl["bpw"]
        head_bytes = cfg.vocab * cfg.dModel * bpw + cfg.dModel * 2
        bytes_tok = algorithmic_bytes_per_token(cfg, n_prompt, n_decode, n_seq, bpw)
        persistent = draft is None and n_seq == 1 and launches == steps * world
        if persistent:
            # one launch of the persistent kernel = one whole step (n_decode heads, n_decode - 1 forward passes)
            launch_bytes = head_bytes + (n_decode - 1) * bytes_tok
            launch_s = statistics.mean(step_ms) / 1e3
            roofline = {"bound": "hbm", "kernel": "k_decode_mega (whole greedy loop: all layers + LM head, one launch per step)",
                        "achieved": launch_bytes / launch_s / 1e9, "peak": peak, "unit": "GB/s",
                        "frac": launch_bytes / launch_s / 1e9 / peak,
                        # DRAM bytes of one launch: measured with ncu on a 4-token launch of this kernel as a multiple of its
                        # algorithmic bytes; traffic grows in proportion to the tokens of a launch
                        "traffic": MEGA_TRAFFIC_RATIO[args.workload] * launch_bytes if args.workload in MEGA_TRAFFIC_RATIO else None,
                        "peak_kind": peak_kind,
                        "bytes_per_launch": launch_bytes, "bytes_per_token": bytes_tok}
        else:
            head_ms = []
            if full and n_seq == 1 and draft is None and not wl.get("device_weights"):
                prof = runtime.DecodeEngine.build(tmp, max_batch=n_seq, device=local_rank, flags=runtime.FLAG_NO_GRAPH)
                prof.prefill(prompts[0])
                tok = prof.select_greedy_token()
                for i in range(40):
                    tok = prof.decode_step(tok)
                    if i >= 8:
                        head_ms.append(prof.timings()["head_ms"])
                prof.close()
            head_t = statistics.mean(head_ms) if head_ms else None
            per_gpu_tok_s = value / world
            if tp:
                # a tensor-parallel rank streams its shard of the weights for all the sequences, and its KV heads
                step_bytes = (cfg.weight_bytes_per_step(bpw) / world + (bytes_tok - cfg.weight_bytes_per_step(bpw) / n_seq) * n_seq / world)
                whole = {"bytes_per_step_per_gpu": step_bytes, "achieved": step_bytes / (total_ms / steps / n_decode / 1e3) / 1e9}
                whole["frac"] = whole["achieved"] / peak
            else:
                whole = {"bytes_per_token": bytes_tok, "achieved": per_gpu_tok_s * bytes_tok / 1e9, "frac": per_gpu_tok_s * bytes_tok / 1e9 / peak}
            roofline = {"bound": "hbm", "kernel": "k_lm_head (final norm + LM head + argmax)" if head_t else "whole decode step (all per-stage kernels of one token)",
                        "achieved": (head_bytes / (head_t / 1e3) / 1e9) if head_t else whole["achieved"], "peak": peak, "unit": "GB/s",
                        "frac": ((head_bytes / (head_t / 1e3) / 1e9) if head_t else whole["achieved"]) / peak, "traffic": None,
                        "peak_kind": peak_kind, "whole_step": whole}
        roofline["frac_of_nominal_8000_GBps"] = roofline["achieved"] / 8000.0  # beside the fraction of the measured copy peak

        out = {"value": value, "ms_per_step": total_ms / steps, "ms_per_token": total_ms / steps / n_decode, "scaling": scaling,
               "launches": launches, "clocks": clocks, "roofline": roofline, "extra": extra, "n_seq_per_gpu": n_seq,
               "e2e_value": tokens_all / e2e_total if e2e_total else None,
               "h2d": int(n_seq * n_prompt * 4), "d2h": int(n_seq * n_decode * 4), "steps": steps, "warmup": warmup}
        if n_seq > 1 and len(prefill_s) > warmup:
            # prompt processing: rows of a pass = positions x sequences on the tensor-core path; FLOPs = 2 per weight of the
            # layer matrices per token + the causal attention products (the LM head is not run on prompt tokens)
            t = statistics.mean(prefill_s[-steps:])
            toks = n_seq * n_prompt
            layer_w = cfg.nLayer * (cfg.dModel * (cfg.attentionDim + 2 * cfg.kvDim) + cfg.attentionDim * cfg.dModel
                                    + (3 if cfg.architecture == "llama" else 2) * cfg.dModel * cfg.hiddenDim)
            att = cfg.nLayer * 4 * cfg.attentionDim * (n_prompt + 1) / 2
            tflops = toks * (2 * layer_w / (world if tp else 1) + att / (world if tp else 1)) / t / 1e12
            peaks = {}
            if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
                with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                    peaks = json.load(f)
            sustained = float(peaks.get("bf16_tflops_sustained", 1400.0))
            out["prefill"] = {"tokens_per_s": toks / t, "ms": t * 1e3, "TFLOPs_per_gpu": tflops, "frac_of_bf16_sustained": tflops / sustained,
                              "peak_kind": "measured" if peaks else "fallback", "prompt_tokens": toks,
                              "note": "prefill_batch(): host wall clock around the call incl. prompt upload; passes of up to 512 rows"}
        if full and rank == 0 and draft is None and n_seq == 1:
            st = stage_trace_us(eng, cfg, prompts[0], n_decode, clocks.get("sm_mhz") or 1965.0)
            if st:
                out["stage_trace_us"] = st
            tt = eng.token_times_ns()  # of the loop stage_trace_us just ran
            if tt.size > 2:
                gaps = np.diff(tt.astype(np.int64)) / 1e6
                out["ms_per_token_gaps"] = {"median": float(np.median(gaps)), "p95": float(np.percentile(gaps, 95)), "tokens": int(tt.size),
                                            "note": "GPU-timer gaps between consecutive tokens inside one decode loop"}
        return out
    finally:
        if world > 1:
            dist.barrier()  # members of a tensor-parallel group tear their communicator down together
        if eng is not None:
            eng.close()
        if draft is not None:
            draft.close()
        shutil.rmtree(tmp, ignore_errors=True)


def tp_matches_single_gpu(rank: int, local_rank: int, world: int) -> bool | None:
    """A small model decoded tensor parallel over this job's GPUs and, on rank 0, by a single-GPU engine of this library:
    the greedy streams must be identical wherever the single-GPU logits leave no near tie (the comparison with the CPU
    restatement of the reference is the test suite's job)."""
    import torch.distributed as dist

    from espresso_b200 import runtime
    from espresso_b200.model_config import MultiModelConfig
    from espresso_b200.sharding import tp_shard
    from espresso_b200.synthetic import synthetic_tensors

    if world < 2:
        return None
    # eight KV heads of 64 channels and 512 hidden units: every shard of a group of 2, 4 or 8 ranks keeps the 64-element
    # alignment the tensor-core path needs
    cfg = MultiModelConfig("tp-check", 2, 8, 8, 256, 64, 512, 1024, 64, 1e-5, 10000.0, None, "llama")
    if cfg.nKVHead % world:
        return None
    n_seq, n_prompt, n_decode = 6, 9, 14
    prompts = np.stack([synthetic_prompt(cfg.vocab, n_prompt, stream=s) for s in range(n_seq)])
    ids = [runtime.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    eng = runtime.DecodeEngine.empty(cfg, max_batch=n_seq, device=local_rank, tp_rank=rank, tp_size=world)
    eng.tp_init(ids[0])
    for name, vals in synthetic_tensors(cfg):
        eng.load_tensor(name, "f16", np.ascontiguousarray(tp_shard(name, vals, rank, world)))
    eng.finalize()
    toks, _ = eng.generate_batch(prompts, n_decode)
    ok = None
    if rank == 0:
        ref = runtime.DecodeEngine.empty(cfg, max_batch=n_seq, device=local_rank)
        for name, vals in synthetic_tensors(cfg):
            ref.load_tensor(name, "f16", np.ascontiguousarray(vals))
        ref.finalize()
        ok = True
        for s in range(n_seq):
            # teacher-forced: the single-GPU engine is fed the tensor-parallel stream
            ref.reset()
            ref.prefill(prompts[s])
            for i, t in enumerate(toks[s]):
                lg = ref.logits()
                if int(t) != int(np.argmax(lg)) and float(lg.max() - lg[int(t)]) > 2e-2:
                    ok = False
                if i + 1 < len(toks[s]):
                    ref.advance(int(t))
        ref.close()
    dist.barrier()
    eng.close()
    dist.barrier()
    return ok


# DRAM bytes of a launch of the persistent kernel as a multiple of its algorithmic bytes (ncu, dram__bytes_read.sum +
# dram__bytes_write.sum of a 4-token launch).  Below 1 at c1: the part of the LM head that the kernel prefetches into
# L2 with an evict-last policy survives from one token to the next.
MEGA_TRAFFIC_RATIO = {"c1": 0.808, "c4q8": 0.972}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c1", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-steps", type=int, default=3)
    ap.add_argument("--decode-tokens", type=int, default=0, help="override the workload's decode length (profiling of small cases)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gemv-table", action="store_true")
    ap.add_argument("--no-sharded", action="store_true", help="skip the sequence-sharded (c3) and tensor-parallel (c5) figures that accompany the default workload")
    ap.add_argument("--per-stage", action="store_true", help="use the per-stage kernels even where the persistent kernel applies")
    ap.add_argument("--kernel", choices=["gemv", "gemm"], help="time one stand-alone kernel instead of a workload")
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=64, help="--kernel gemm: activation rows (1..256)")
    ap.add_argument("--type", default="f16", choices=["f16", "bf16", "q8_0", "q4_0"])
    ap.add_argument("--iterations", type=int, default=40)
    args = ap.parse_args()
    if args.kernel:
        run_kernel_probe(args)
        return
    if args.impl == "ours":
        args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    wl = dict(WORKLOADS[args.workload])
    if args.decode_tokens > 0:
        wl["decode"] = args.decode_tokens
    metric, unit = "decode tokens/s (whole job)", "tokens/s"

    if args.impl == "reference":
        # The reference's own CPU implementation of the path, restated (the Swift/Accelerate original does not
        # build on Linux); rank 0 alone runs it on all host cores, the other ranks leave at once.
        if rank != 0:
            return
        r = run_cpu_oracle(wl, max(args.steps, 1), args.warmup)
        line = {
            "impl": "reference", "metric": metric, "value": r["value"], "unit": unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_of(wl, max(args.gpus, 1)),
            "cpu_baseline": {"value": r["value"], "unit": unit, "cores": r["cores"], "cpu_model": cpu_model(), "kind": "port", "sample": r["sample"]},
            "e2e": {"value": r["value"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement of the reference's path on the host cores, fp32 weights larger than the host caches",
        }
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist

    from espresso_b200 import runtime

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode path has no CPU implementation")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    r = measure(args, wl, rank, local_rank, world, args.steps, args.warmup, full=True)
    line = {
        "metric": metric, "value": r["value"], "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": r["ms_per_step"], "ms_per_token": r["ms_per_token"], "higher_is_better": True,
        "scaling": r["scaling"], "vs_baseline": None, "dtype": f"{wl['kind']} weights, f16 KV, f32 accumulate", "data": "synthetic",
        "config": config_of(wl, world),
        "e2e": {"value": r["e2e_value"], "unit": unit, "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"],
                "note": "generate(): prompt upload + prefill + decode + token download, wall clock"},
        "gpu_launches": r["launches"], "clocks": r["clocks"], "roofline": r["roofline"],
    }
    line.update(r["extra"])
    for k in ("stage_trace_us", "ms_per_token_gaps", "prefill"):
        if k in r:
            line[k] = r[k]

    # ---- the two configurations that partition work across GPUs, measured on the same GPUs in the same run ----
    if args.workload == "c1" and not args.no_sharded and args.decode_tokens == 0:
        for key, name, k_steps in (("sharded_c3", "c3", 2), ("tp_c5", "c5", 1)):
            w2 = dict(WORKLOADS[name])
            if name == "c5" and (w2["cfg"]().nKVHead % world or world > w2["cfg"]().nKVHead):
                continue
            m = measure(args, w2, rank, local_rank, world, k_steps, 1, full=False)
            entry = {"workload": w2["label"], "tokens_per_s": m["value"], "ms_per_step": m["ms_per_step"], "ms_per_token_step": m["ms_per_token"],
                     "sequences_per_gpu": m["n_seq_per_gpu"], "steps": k_steps, "warmup": 1, "gpu_launches": m["launches"],
                     "roofline_whole_step_frac": m["roofline"].get("whole_step", {}).get("frac"), "clocks": m["clocks"],
                     "parallelism": config_of(w2, world)["parallelism"]}
            if "prefill" in m:
                entry["prefill"] = m["prefill"]
            if name == "c5":
                L = w2["cfg"]().nLayer
                entry["all_reduce"] = {"path": "peer memory (k_tp_sum_peers)" if world > 1 and not os.environ.get("ESP_CUDA_TP_NCCL_ONLY") else ("NCCL" if world > 1 else "none (one GPU)"),
                                       "per_decode_step": 2 * L if world > 1 else 0, "bytes_each": w2["n_seq"] * w2["cfg"]().dModel * 4}
                if "tp_sum" in m["extra"]:  # rank 0's kernel k_tp_sum_peers during the decode steps: arrival -> last sum, and the wait for the peers in it
                    entry["all_reduce"].update(mean_us=m["extra"]["tp_sum"]["mean_us"], mean_wait_for_peers_us=m["extra"]["tp_sum"]["mean_wait_us"])
                entry["matches_single_gpu_engine"] = tp_matches_single_gpu(rank, local_rank, world)
            line[key] = entry

    # kernel-level tables and the CPU baseline belong to the single-GPU line: under torchrun no rank may sit in a
    # collective while rank 0 works on the host
    if world == 1 and not args.no_gemv_table:
        peak, _ = read_peaks()
        line["gemv"] = gemv_table(runtime, local_rank, peak)
        line["gemm_tc"] = gemm_table(runtime, local_rank, peak)
    if world == 1 and not args.no_cpu_baseline:
        c = run_cpu_oracle(wl, args.cpu_steps, 1)
        line["cpu_baseline"] = {"value": c["value"], "unit": unit, "cores": c["cores"], "cpu_model": cpu_model(), "kind": "port", "sample": c["sample"]}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

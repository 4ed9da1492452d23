"""Benchmark of the decode hot path.

A "step" is one pass of the hot path over one batch of synthetic input: a greedy decode of
``decode_tokens`` tokens for every sequence of the workload, continuing from a prefilled prompt.
``value`` is decode tokens/s with everything resident in HBM (device-timed with CUDA events);
``e2e`` is the same metric through the public generate call with host buffers (prompt upload, prefill,
decode, token download all inside the timed region).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1] [--impl ours|reference]
"""
from __future__ import annotations

import argparse
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
    # name: (config factory, prompt tokens, decode tokens, sequences per GPU, weight storage)
    "c1": dict(cfg=mc.llama_6l, prompt=16, decode=128, n_seq=1, kind="f16",
               label="llama 6L d768 12h vocab32000 ctx256 fp16, batch 1, 16-token prompt, 128 greedy steps"),
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


def run_cpu_oracle(workload: dict, weight_dir: str, steps: int, warmup: int, threads: int | None = None) -> dict:
    """Times the CPU restatement of the reference's decode path on the host cores."""
    import oracle

    lib = oracle.lib()
    if threads:
        lib.esp_oracle_set_num_threads(threads)
    cores = lib.esp_oracle_num_threads()
    cfg = workload["cfg"]()
    model = oracle.Model.from_dir(weight_dir)
    rt = oracle.Runtime(model)
    prompt = synthetic_prompt(cfg.vocab, workload["prompt"])
    decode = workload["decode"]
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
    total = sum(times)
    return {"value": decode * len(times) / total, "ms_per_step": 1e3 * total / len(times), "cores": cores,
            "sample": f"full workload per step: {workload['prompt']}-token prompt (untimed prefill) + {decode} greedy decode steps, {len(times)} steps"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c1", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    wl = WORKLOADS[args.workload]
    cfg = wl["cfg"]()
    metric, unit = "decode tokens/s (whole job)", "tokens/s"

    tmp = tempfile.mkdtemp(prefix=f"esp_bench_r{rank}_")
    try:
        if args.impl == "reference":
            # The reference's own CPU implementation of the path, restated (the Swift/Accelerate original does not
            # build on Linux); rank 0 alone runs it.
            if rank != 0:
                return
            write_synthetic_model(cfg, tmp)
            r = run_cpu_oracle(wl, tmp, max(args.steps, 1), args.warmup)
            line = {
                "impl": "reference", "metric": metric, "value": r["value"], "unit": unit, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": wl["label"], "l2": "weights (268 MB fp32) exceed the host caches"},
                "cpu_baseline": {"value": r["value"], "unit": unit, "cores": r["cores"], "kind": "port", "sample": r["sample"]},
                "e2e": {"value": r["value"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        write_synthetic_model(cfg, tmp)
        n_seq, n_prompt, n_decode = wl["n_seq"], wl["prompt"], wl["decode"]
        prompts = np.stack([synthetic_prompt(cfg.vocab, n_prompt, stream=rank * n_seq + s) for s in range(n_seq)])
        eng = runtime.DecodeEngine.build(tmp, max_batch=n_seq, device=local_rank)

        def prefill():
            if n_seq == 1:
                eng.prefill(prompts[0])
            else:
                eng.prefill_batch(prompts)

        # ---- device-resident throughput: K timed steps, each a device-driven decode of n_decode tokens ----
        prefill()
        cp = eng.capture_checkpoint() if n_seq == 1 else None
        for _ in range(args.warmup):
            if cp is not None:
                eng.rollback(cp)
            else:
                prefill()
            eng.decode(n_decode, n_seq)
        sampler = ClockSampler(physical_gpu_index(local_rank))
        barrier()
        sampler.start()
        step_ms, launches = [], 0
        for _ in range(args.steps):
            if cp is not None:
                eng.rollback(cp)  # positions return to the end of the prompt; KV slots are simply overwritten
            else:
                prefill()
            toks, ms = eng.decode(n_decode, n_seq)
            assert all(len(t) == n_decode for t in toks)
            step_ms.append(ms)
            launches += eng.timings()["kernel_launches"]
        barrier()
        clocks = sampler.stop()
        total_ms = sum(step_ms)

        # ---- end to end through the public generate call with host buffers ----
        e2e_times = []
        for i in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            if n_seq == 1:
                res = eng.generate(prompts[0], n_decode)
                assert len(res.tokens) == n_decode
            else:
                toks, res = eng.generate_batch(prompts, n_decode)
            torch.cuda.synchronize()
            if i >= args.warmup:
                e2e_times.append(time.perf_counter() - t0)
        e2e_total = sum(e2e_times)

        if world > 1:
            t = torch.tensor([total_ms, e2e_total], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total_ms, e2e_total = float(t[0]), float(t[1])
            lt = torch.tensor([launches], dtype=torch.int64, device="cuda")
            dist.all_reduce(lt)
            launches = int(lt[0])
        tokens_all = world * n_seq * n_decode * args.steps
        value = tokens_all / (total_ms / 1e3)
        e2e_value = tokens_all / e2e_total

        # ---- roofline of the dominant kernel, timed live with CUDA events ----
        peak, peak_kind = read_peaks()
        head_bytes = cfg.vocab * cfg.dModel * 2 + cfg.dModel * 2
        bytes_tok = algorithmic_bytes_per_token(cfg, n_prompt, n_decode, n_seq, 2.0)
        persistent = n_seq == 1 and launches == args.steps
        if persistent:
            # one launch of the persistent kernel = one whole step (n_decode heads, n_decode - 1 forward passes)
            launch_bytes = head_bytes + (n_decode - 1) * bytes_tok
            launch_s = statistics.mean(step_ms) / 1e3
            roofline = {"bound": "hbm", "kernel": "k_decode_mega (whole greedy loop: all layers + LM head, one launch per step)",
                        "achieved": launch_bytes / launch_s / 1e9, "peak": peak, "unit": "GB/s",
                        "frac": launch_bytes / launch_s / 1e9 / peak, "traffic": None, "peak_kind": peak_kind,
                        "bytes_per_launch": launch_bytes, "bytes_per_token": bytes_tok}
        else:
            prof = runtime.DecodeEngine.build(tmp, max_batch=n_seq, device=local_rank, flags=runtime.FLAG_NO_GRAPH)
            head_ms = []
            if n_seq == 1:
                prof.prefill(prompts[0])
                tok = prof.select_greedy_token()
                for i in range(40):
                    tok = prof.decode_step(tok)
                    if i >= 8:
                        head_ms.append(prof.timings()["head_ms"])
            prof.close()
            head_t = statistics.mean(head_ms) if head_ms else None
            roofline = {"bound": "hbm", "kernel": "k_lm_head (final norm + LM head + argmax)",
                        "achieved": (head_bytes / (head_t / 1e3) / 1e9) if head_t else None, "peak": peak, "unit": "GB/s",
                        "frac": (head_bytes / (head_t / 1e3) / 1e9 / peak) if head_t else None, "traffic": None, "peak_kind": peak_kind,
                        "whole_step": {"bytes_per_token": bytes_tok, "achieved": value / world * bytes_tok / 1e9,
                                       "frac": value / world * bytes_tok / 1e9 / peak}}

        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps, "ms_per_token": total_ms / args.steps / n_decode, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 weights and KV, f32 accumulate", "data": "synthetic",
            "config": {"workload": wl["label"], "parallelism": "replicas only (one independent sequence per GPU)" if world > 1 else "single GPU",
                       "l2": "no flush: every decode step streams 134 MB of weights + KV, more than the 126 MB L2"},
            "e2e": {"value": e2e_value, "unit": unit,
                    "h2d_bytes_per_step": int(n_seq * n_prompt * 4), "d2h_bytes_per_step": int(n_seq * n_decode * 4),
                    "note": "generate(): prompt upload + prefill + decode + token download, wall clock"},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
        }
        if rank == 0 and not args.no_cpu_baseline:
            r = run_cpu_oracle(wl, tmp, args.cpu_steps, 1)
            line["cpu_baseline"] = {"value": r["value"], "unit": unit, "cores": r["cores"], "kind": "port", "sample": r["sample"]}
        eng.close()
        if rank == 0:
            print(json.dumps(line))
        if world > 1:
            dist.destroy_process_group()
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    main()

"""Worker of the tensor-parallel GPU test: launched by torchrun with one rank per GPU (see test_gpu_tp.py)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from espresso_b200 import runtime  # noqa: E402
from espresso_b200.model_config import MultiModelConfig  # noqa: E402
from espresso_b200.sharding import tp_shard  # noqa: E402
from espresso_b200.synthetic import synthetic_prompt, synthetic_tensors  # noqa: E402
from espresso_b200.weight_blob import is_matrix  # noqa: E402


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    case = os.environ.get("ESP_TP_CASE", "small")
    if case == "wide_bf16":
        # bf16 storage, head_dim 128 with grouped queries, theta 5e5 and widths at which the Wo / W2 shards are cut along K
        # (partial sums of several CTAs per output tile) before they cross to the peers
        cfg = MultiModelConfig("tp-llama-wide", 2, 8, 4, 1024, 128, 4096, 4096, 96, 1e-5, 500000.0, None, "llama")
        n_seq, n_prompt, n_decode = 16, 12, 10
    else:
        cfg = MultiModelConfig("tp-llama", 2, 8, 4, 256, 32, 512, 1024, 64, 1e-5, 10000.0, None, "llama")
        n_seq, n_prompt, n_decode = 6, 9, 14
    bf16 = case == "wide_bf16"

    def stored(vals, wide):
        """(array to upload, type name, the fp32 values the storage decodes to)"""
        if bf16 and wide:
            u = np.ascontiguousarray(vals, np.float32).view(np.uint32)
            bits = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
            return bits, "bf16", (bits.astype(np.uint32) << np.uint32(16)).view(np.float32).reshape(vals.shape)
        h = vals.astype(np.float16)
        return h, "f16", h.astype(np.float32)

    prompts = np.stack([synthetic_prompt(cfg.vocab, n_prompt, stream=s) for s in range(n_seq)])
    ids = [runtime.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    eng = runtime.DecodeEngine.empty(cfg, max_batch=n_seq, device=rank, tp_rank=rank, tp_size=world)
    eng.tp_init(ids[0])
    for name, vals in synthetic_tensors(cfg):
        arr, kind, _ = stored(vals, is_matrix(name) or name.startswith("embeddings/"))
        eng.load_tensor(name, kind, np.ascontiguousarray(tp_shard(name, arr, rank, world)))
    eng.finalize()
    toks, res = eng.generate_batch(prompts, n_decode)
    single = eng.generate(prompts[0], n_decode).tokens  # rows = 1 also runs tensor parallel
    if rank == 0:
        import oracle
        from helpers import ABS_TOL, BF16_ABS_TOL, compare_greedy_stream

        tol = BF16_ABS_TOL if bf16 else ABS_TOL

        model = oracle.Model(cfg.to_metadata())
        for name, vals in synthetic_tensors(cfg):
            model.set_tensor(name, stored(vals, is_matrix(name) or name.startswith("embeddings/"))[2])
        for s in range(n_seq):
            assert len(toks[s]) == n_decode
            compare_greedy_stream(oracle.Runtime(model), prompts[s], toks[s], tol=tol)
        compare_greedy_stream(oracle.Runtime(model), prompts[0], single, tol=tol)
        print(f"tensor parallel x{world} ok ({case}): {n_seq} streams match the oracle")
    dist.barrier()  # the ranks leave together: a communicator is torn down by all of its members
    eng.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

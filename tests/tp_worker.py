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


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    cfg = MultiModelConfig("tp-llama", 2, 8, 4, 256, 32, 512, 1024, 64, 1e-5, 10000.0, None, "llama")
    n_seq, n_prompt, n_decode = 6, 9, 14
    prompts = np.stack([synthetic_prompt(cfg.vocab, n_prompt, stream=s) for s in range(n_seq)])
    ids = [runtime.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    eng = runtime.DecodeEngine.empty(cfg, max_batch=n_seq, device=rank, tp_rank=rank, tp_size=world)
    eng.tp_init(ids[0])
    for name, vals in synthetic_tensors(cfg):
        eng.load_tensor(name, "f16", np.ascontiguousarray(tp_shard(name, vals, rank, world)))
    eng.finalize()
    toks, res = eng.generate_batch(prompts, n_decode)
    single = eng.generate(prompts[0], n_decode).tokens  # rows = 1 also runs tensor parallel
    if rank == 0:
        import oracle
        from helpers import compare_greedy_stream

        model = oracle.Model(cfg.to_metadata())
        for name, vals in synthetic_tensors(cfg):
            model.set_tensor(name, vals.astype(np.float32))
        for s in range(n_seq):
            assert len(toks[s]) == n_decode
            compare_greedy_stream(oracle.Runtime(model), prompts[s], toks[s])
        compare_greedy_stream(oracle.Runtime(model), prompts[0], single)
        print(f"tensor parallel x{world} ok: {n_seq} streams match the oracle")
    dist.barrier()  # the ranks leave together: a communicator is torn down by all of its members
    eng.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

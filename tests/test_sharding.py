"""Host-side logic of the multi-GPU path: sequence sharding and result gathering (gloo, world size 2)."""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_partitions_exactly():
    from espresso_b200.sharding import shard_range

    for n in (0, 1, 7, 8, 256, 257):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def test_quantisers_torch_match_numpy():
    import torch
    from espresso_b200 import gguf_quant as gq
    from espresso_b200.synthetic_device import quantize_q4_0_torch, quantize_q8_0_torch

    g = np.load(os.path.join(ROOT, "tests", "golden", "gguf_blocks.npz"))
    x = torch.from_numpy(g["x"])
    assert np.array_equal(quantize_q8_0_torch(x).numpy(), g["q8_0_blocks"])
    assert np.array_equal(quantize_q4_0_torch(x).numpy(), g["q4_0_blocks"])
    rng = np.random.default_rng(1)
    y = (rng.standard_normal(32 * 999) * 0.02).astype(np.float32)
    assert np.array_equal(quantize_q8_0_torch(torch.from_numpy(y)).numpy(), gq.quantize_q8_0(y))
    assert np.array_equal(quantize_q4_0_torch(torch.from_numpy(y)).numpy(), gq.quantize_q4_0(y))


WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    import torch.distributed as dist
    sys.path.insert(0, os.environ["ESP_ROOT"])
    from espresso_b200.sharding import gather_token_streams, shard_range
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    n_total = 5
    b, e = shard_range(n_total, rank, world)
    # every sequence s "generates" the stream [s, s+1, ..., s+s] (ragged lengths, including an empty one)
    local = [np.arange(s, s + s, dtype=np.uint32) for s in range(b, e)]
    out = gather_token_streams(local, n_total, rank, world, max_tokens=8)
    if rank == 0:
        assert len(out) == n_total
        for s, t in enumerate(out):
            assert list(t) == list(range(s, s + s)), (s, t)
        print("gather ok")
    dist.destroy_process_group()
""")


def test_gather_token_streams_world_size_2(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, ESP_ROOT=ROOT)
    res = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
         "--master-port", str(port), str(script)],
        capture_output=True, text=True, env=env, timeout=240)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "gather ok" in res.stdout

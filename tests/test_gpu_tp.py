"""Tensor-parallel decode on 2 GPUs (skipped where fewer are visible): token streams of the TP group against the oracle."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_tp_shard_shapes():
    from espresso_b200.sharding import tp_shard

    w = np.arange(8 * 6).reshape(8, 6)
    assert np.array_equal(tp_shard("layers/0/wq", w, 1, 2), w[4:])
    assert np.array_equal(tp_shard("layers/0/wo", w, 1, 2), w[:, 3:])
    assert np.array_equal(tp_shard("layers/0/rms_att", w[0], 1, 2), w[0])
    assert np.array_equal(tp_shard("embeddings/token", w, 1, 2), w)
    assert np.array_equal(tp_shard("lm_head", w, 0, 4), w[:2])
    with pytest.raises(ValueError):
        tp_shard("layers/0/w1", w, 0, 3)
    # the shards of a row-split matrix and of the column-split matrix that follows it reproduce the full product
    rng = np.random.default_rng(0)
    w1, w2, x = rng.standard_normal((8, 5)), rng.standard_normal((5, 8)), rng.standard_normal(5)
    full = w2 @ (w1 @ x)
    parts = sum(tp_shard("w2", w2, r, 4) @ (tp_shard("w1", w1, r, 4) @ x) for r in range(4))
    np.testing.assert_allclose(parts, full, atol=1e-12)


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["small", "wide_bf16"])
def test_tensor_parallel_two_gpus_matches_oracle(case):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", ESP_TP_CASE=case)
    res = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
         "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py")],
        capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert f"tensor parallel x2 ok ({case})" in res.stdout

"""Two and more ranks of the column-parallel configuration, one process per GPU
(skipped on a box with a single GPU).  The ranks are child processes started
with torch.distributed.run on 127.0.0.1; NVLS is off and the collectives are
plain NCCL rings, as this pool asks of tests that start and stop ranks."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _run_ranks(n, what, tmp_path):
    out = tmp_path / f"{what}_{n}.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(29400 + n),
           str(ROOT / "tests" / "multi_rank_worker.py"), what, str(out)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return json.loads(out.read_text())


@pytest.mark.parametrize("n", [2, 4, 8])
def test_column_parallel_linear_equals_unsplit(built_lib, tmp_path, n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    r = _run_ranks(n, "linear", tmp_path)
    assert r["acc_equal"] and r["chain_equal"] and r["scale_equal"] and r["status"] == 0


@pytest.mark.parametrize("n", [2, 4])
def test_decoder_ranks_agree_with_one_gpu(built_lib, tmp_path, n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    r = _run_ranks(n, "decoder", tmp_path)
    assert r["prefill_close"] > 0.99 and r["decode_close"] > 0.99 and r["status"] == 0

"""Tensor parallelism on real GPUs: one process per GPU under torchrun (NCCL). Skipped with fewer than
two GPUs; the host-side rules (ordered sum, candidate merge, sharding) are covered on CPU with gloo in
test_distributed_cpu.py."""

import os
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("world,exchange", [(2, "peer"), (2, "nccl"), (4, "peer"), (8, "peer")])
def test_window_rows_equal_serial_steps_under_tp(lib, world, exchange):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1", TP_EXCHANGE=exchange)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29400 + world + (20 if exchange == "nccl" else 0)), str(ROOT / "tests" / "tp_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = re.search(r"TP_RESULT world=(\d+) window_equals_serial=(\d) head_ok=(\d) cos_vs_one_gpu=([0-9.]+) fused_equals_gathered=(\d)", out.stdout)
    assert m, out.stdout[-2000:]
    print(m.group(0))                                  # kept in the test log (pytest -s / -rA)
    assert int(m.group(1)) == world
    assert m.group(2) == "1", "window rows differ from the same ranks' serial decode"
    assert m.group(3) == "1", "vocabulary-split draw differs from the whole-vocabulary draw"
    assert float(m.group(4)) > 0.999          # the reference's cross-world bound (tests/cuda/test_flashnext_tp.py:218-227)
    assert m.group(5) == "1", "the exchange fused into matmul + norm differs from all-gather + ordered sum"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_block_has_the_bits_of_one_gpu(lib, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29460 + world), str(ROOT / "tests" / "ep_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = re.search(r"EP_RESULT world=(\d+) equals_one_gpu=(\d) one_row_(\d+)_exchanges_ok=(\d)", out.stdout)
    assert m and int(m.group(1)) == world, out.stdout[-2000:]
    print(m.group(0))
    assert m.group(2) == "1", "the expert-parallel block differs from the one-GPU block"
    assert m.group(4) == "1", "one row over many exchanges: a stall, or bits that differ from the one-GPU block"

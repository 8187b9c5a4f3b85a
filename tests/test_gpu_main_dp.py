"""The data-parallel entry point's --tiny smoke run (the reference's own integration check,
multi_gpu/scripts/main_dp.py:55-61,117-124): weights finite and changed, step counts right."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _run(cmd):
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT, env=env)
    assert res.returncode == 0, (res.stdout[-1500:], res.stderr[-3000:])
    return res.stdout


def test_tiny_single_gpu(tmp_path):
    out = _run([sys.executable, "-m", "slideformer_b200.main_dp", "--tiny", "--steps", "3", "--batch-size", "2",
                "--save-model", str(tmp_path / "m")])
    assert "rank=0 tiny_weight_checks=passed" in out and "rank=0 completed=3" in out
    assert (tmp_path / "m" / "config.json").exists()


def test_tiny_single_gpu_with_schedule_and_clipping():
    """Warm-up + cosine schedule and delayed global-norm clipping driven by the statistics the
    update kernels gather."""
    out = _run([sys.executable, "-m", "slideformer_b200.main_dp", "--tiny", "--steps", "4", "--batch-size", "2",
                "--warmup-steps", "2", "--total-steps", "10", "--clip-norm", "0.05"])
    assert "rank=0 completed=4" in out
    norms = [float(line.split("grad_norm=")[1].split()[0]) for line in out.splitlines() if "grad_norm=" in line]
    clips = [float(line.split("next_clip=")[1].split()[0]) for line in out.splitlines() if "next_clip=" in line]
    assert len(norms) == 4 and all(n > 0 for n in norms)
    assert all(abs(c - min(1.0, 0.05 / n)) < 1e-3 for n, c in zip(norms, clips))


@pytest.mark.parametrize("extra", [[], ["--tied"], ["--double-buffer", "--chunk-numel", "4096"], ["--clip-norm", "0.05"]])
def test_tiny_two_gpus(extra):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                "--master-addr", "127.0.0.1", "--master-port", "29571", "-m", "slideformer_b200.main_dp", "--tiny",
                "--steps", "3", "--batch-size", "2", *extra])
    for r in (0, 1):
        assert f"rank={r} tiny_weight_checks=passed" in out and f"rank={r} completed=3" in out

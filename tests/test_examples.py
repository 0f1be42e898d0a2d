"""The example scripts run end to end on CPU (their own exit code is the verdict: both
check that the loss went down and that a checkpoint round trip preserved the state)."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(cmd, timeout=600):
    env = dict(os.environ, OMP_NUM_THREADS="2", PYTHONWARNINGS="ignore")
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    return out.stdout


def test_mnist_example_cpu():
    out = _run([sys.executable, "examples/train_mnist.py", "--device", "cpu", "--epochs", "1", "--gradient-release"])
    assert "accuracy" in out.lower()


@pytest.mark.parametrize("extra", [[], ["--gradient-release", "--compress-state-dict"]])
def test_fsdp2_example_two_gloo_ranks(extra):
    out = _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                "--master-addr", "127.0.0.1", "--master-port", "29613", "examples/train_fsdp2.py",
                "--device", "cpu", "--steps", "12", *extra])
    assert "checkpoint round trip" in out

"""The sharded layers on real GPUs: needs at least two. One torchrun rank per GPU runs tests/dist_gpu_check.py."""
import os, pathlib, subprocess, sys
import pytest

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parent.parent


def gpus():
  import torch
  return torch.cuda.device_count()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_layers_on_gpus(world):
  if gpus() < world: pytest.skip(f"needs {world} GPUs")
  env = dict(os.environ, MASTER_ADDR="127.0.0.1")
  run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", "29541", str(ROOT / "tests" / "dist_gpu_check.py")], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
  assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-3000:]
  assert run.stdout.count(": ok") == world
